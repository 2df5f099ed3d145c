"""Seeded synthetic inputs with the shapes of the benchmark configurations: ``_splithead`` dim tables
(the on-disk format the cache reads, cache_utils_fourier.py:433-455 of the reference) and rotary-embedded
Gaussian K/V."""
import json

import numpy as np
import torch


def make_splithead_tables(num_layers, num_kv_heads, head_dim, n_compressed, seed, upper_weight=3.0):
    """Per layer and KV head, ``n_compressed`` of the ``head_dim`` dims are drawn without replacement; a dim
    in the upper half of the head is ``upper_weight`` times as likely as one in the lower half.  K and V
    sets are drawn independently.  Returns the dict that ``json.dump`` turns into a ``_splithead`` file."""
    rng = np.random.default_rng(seed)
    w = np.ones(head_dim)
    w[head_dim // 2:] = upper_weight
    w = w / w.sum()
    out = {}
    for layer in range(num_layers):
        ent = {}
        for t in ("k", "v"):
            c_list, n_list, c_h, n_h = [], [], [], []
            for h in range(num_kv_heads):
                sel = rng.choice(head_dim, size=n_compressed, replace=False, p=w) if n_compressed else []
                mask = np.zeros(head_dim, bool)
                mask[np.asarray(sel, dtype=np.int64)] = True
                c_list += [int(h * head_dim + i) for i in np.nonzero(mask)[0]]
                n_list += [int(h * head_dim + i) for i in np.nonzero(~mask)[0]]
                c_h.append(len(c_list)); n_h.append(len(n_list))
            ent[f"{t}c_list"], ent[f"{t}n_list"] = c_list, n_list
            ent[f"{t}c_h_list"], ent[f"{t}n_h_list"] = c_h, n_h
        out[f"Layer_{layer}"] = ent
    return out


def write_tables(tables, path):
    with open(path, "w") as f:
        json.dump(tables, f)
    return path


def rope_kv(B, Hkv, L, D, dtype, device, generator, theta=500000.0, start=0):
    """K, V ~ N(0,1) of shape (B, Hkv, L, D) in (B, L, Hkv, D) memory order; K carries a plain rotary
    embedding (half-split convention) at positions start..start+L-1."""
    k = torch.randn((B, L, Hkv, D), device=device, dtype=torch.float32, generator=generator)
    v = torch.randn((B, L, Hkv, D), device=device, dtype=torch.float32, generator=generator)
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=device, dtype=torch.float32) / D))
    ang = torch.arange(start, start + L, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    cos = torch.cat([ang.cos(), ang.cos()], -1)[None, :, None, :]
    sin = torch.cat([ang.sin(), ang.sin()], -1)[None, :, None, :]
    rot = torch.cat([-k[..., D // 2:], k[..., : D // 2]], -1)
    k = k * cos + rot * sin
    return k.to(dtype).transpose(1, 2), v.to(dtype).transpose(1, 2)
