"""GPU tests of the callers and the sharded forms of the cache, each against the CPU oracle:

* ``LlamaSdpaAttention.forward`` (the reference's dispatcher, modeling_llama_fourier.py:565-667): prefill
  branch, Fourier decode branch and the never-compressed branch, in a two-layer random Llama;
* ``DynamicCache(kv_head_range=...)``: the shards' outputs, concatenated, equal the unsharded cache's;
* ``DynamicCache(seq_shard=...)``: the product's own collectives (all_reduce of the coefficient partials at
  prefill, all_gather + log-sum-exp merge at decode) in a one-rank group on one GPU and, when two GPUs are
  visible, as two real ranks over NCCL.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from oracle import fourier_oracle as fo
from tests.gpu_util import dev, host, make_config, oracle_cache, update_arg, write_tables
from tests.helpers import attn_tol, case_inputs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


# ------------------------------------------------------------------------------------------------
# LlamaSdpaAttention.forward
# ------------------------------------------------------------------------------------------------
def _to_oracle(t):
    """(B, H, L, D) device tensor -> numpy float32 (values already on the model-dtype grid)."""
    return t.detach().float().cpu().numpy()


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("P", [200, 40])
def test_llama_attention_forward_matches_oracle(dtype, P):
    """A two-layer random Llama (hidden 256, 8 query / 2 KV heads, D = 32).  P = 200 exceeds S + M + W = 42,
    so the prompt is compressed and decode takes the Fourier branch; P = 40 is never compressed and decode
    stays on dense attention over ``k_local`` (modeling_llama_fourier.py:623-633).  The attention output that
    reaches ``o_proj`` is compared with the oracle's, and the module's result with that output pushed through
    the same ``o_proj`` in float32."""
    from fourierattention_b200 import DynamicCache
    from fourierattention_b200.modeling_llama_fourier import LlamaConfig, LlamaModel, apply_rotary_pos_emb
    tdt = torch.float16 if dtype == "fp16" else torch.bfloat16
    B, hidden, Hq, Hkv, D, S, W, M, steps = 2, 256, 8, 2, 32, 2, 24, 16, 3
    torch.manual_seed(11)
    cfg = LlamaConfig(vocab_size=97, hidden_size=hidden, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=Hq, num_key_value_heads=Hkv, max_position_embeddings=4096)
    model = LlamaModel(cfg)
    for p_ in model.parameters():
        if p_.dim() > 1:
            p_.data.normal_(0.0, 0.08)
    model = model.to("cuda", tdt).eval()
    tables = fo.make_splithead_tables(2, Hkv, D, 20, seed=12)
    path = write_tables(tables)
    g = dict(S=S, W=W, M=M, mpe=4096, Hkv=Hkv, steps=steps)
    try:
        cache = DynamicCache(make_config(g, path))
    finally:
        os.unlink(path)
    oc = fo.OracleCache([fo.DimTables(tables[f"Layer_{i}"]) for i in range(2)], S, W, M, steps, 4096, dtype)

    captured = {}

    def grab(layer):
        def pre(mod, args):
            captured[layer] = args[0].detach().float()
        return pre
    hooks = [model.layers[i].self_attn.o_proj.register_forward_pre_hook(grab(i)) for i in range(2)]
    projected = {}
    hooks += [model.layers[i].self_attn.o_proj.register_forward_hook(
        lambda m, a, o, i=i: projected.__setitem__(i, o.detach().float())) for i in range(2)]
    ids = torch.randint(0, 97, (B, P + steps), device="cuda")
    compressed = P > S + M + W

    def qkv(layer, hs, pos):
        """q, k, v after the rotary embedding, recomputed with the module's own weights."""
        at = model.layers[layer].self_attn
        b, n, _ = hs.shape
        q = at.q_proj(hs).view(b, n, Hq, D).transpose(1, 2)
        k = at.k_proj(hs).view(b, n, Hkv, D).transpose(1, 2)
        v = at.v_proj(hs).view(b, n, Hkv, D).transpose(1, 2)
        cos, sin = model.rotary_emb(v, pos)
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        return q, k, v

    def dense_ref(q, k_all, v_all):
        """float64 causal attention, query rows bottom-right aligned; inputs rounded to float16 as the
        prefill branch does (modeling_llama_fourier.py:633)."""
        qh = q.half().double().cpu().numpy(); kh = k_all.half().double().cpu().numpy(); vh = v_all.half().double().cpu().numpy()
        b, _, n, _ = qh.shape
        L = kh.shape[2]
        out = np.zeros((b, n, Hq, D))
        for h in range(Hq):
            s = np.einsum("bqd,bkd->bqk", qh[:, h], kh[:, h // (Hq // Hkv)]) / np.sqrt(D)
            mask = np.tril(np.ones((n, L), bool), k=L - n)
            s = np.where(mask[None], s, -np.inf)
            p = np.exp(s - s.max(-1, keepdims=True))
            p /= p.sum(-1, keepdims=True)
            out[:, :, h] = np.einsum("bqk,bkd->bqd", p, vh[:, h // (Hq // Hkv)])
        return out.reshape(b, n, Hq * D)

    with torch.no_grad():
        # ---- prefill: hidden states entering each layer are taken from the model itself ---------------
        layer_in = {}
        hk = [model.layers[i].register_forward_pre_hook(lambda m, a, i=i: layer_in.__setitem__(i, a[0].detach()))
              for i in range(2)]
        out = model(ids[:, :P], past_key_values=cache)
        assert tuple(out.shape) == (B, P, hidden)
        pos = torch.arange(P, device="cuda")[None].expand(B, -1)
        dense_k, dense_v = {}, {}
        for i in range(2):
            hs = model.layers[i].input_layernorm(layer_in[i])
            q, k, v = qkv(i, hs, pos)
            oc.update(_to_oracle(k), _to_oracle(v), i)
            dense_k[i], dense_v[i] = k, v
            ref = dense_ref(q, k, v)
            got = captured[i].cpu().numpy()
            # the module hands o_proj the attention output rounded to the model dtype
            grid = 2.0 ** (-11 if dtype == "fp16" else -8)
            err = np.abs(got - ref) - grid * np.abs(ref)
            assert err.max() <= 2e-3, ("prefill attention", i, err.max())
        # ---- decode --------------------------------------------------------------------------------------
        for s in range(steps):
            out = model(ids[:, P + s:P + s + 1], past_key_values=cache)
            assert tuple(out.shape) == (B, 1, hidden)
            pos = torch.full((B, 1), P + s, device="cuda")
            for i in range(2):
                hs = model.layers[i].input_layernorm(layer_in[i])
                q, k, v = qkv(i, hs, pos)
                kd, vd = oc.update(_to_oracle(k), _to_oracle(v), i)
                got = captured[i].cpu().numpy()                       # (B, 1, Hq*D), already cast to the model dtype
                if compressed:
                    assert kd["k_init"] is not None
                    for nm in ("k_scale", "v_scale", "k_layer_average", "v_layer_average", "kd_layer_average",
                               "vd_layer_average"):
                        getattr(oc, nm)[i] = host(getattr(cache, nm)[i])
                    ref = oc.attend(_to_oracle(q)[:, :, 0].reshape(B, -1), i, Hq, Hkv, faithful=False)
                    ref = ref[:, :, 0].reshape(B, 1, Hq * D)
                else:
                    assert kd["k_init"] is None
                    dense_k[i] = torch.cat([dense_k[i], k], 2)
                    dense_v[i] = torch.cat([dense_v[i], v], 2)
                    ref = dense_ref(q, dense_k[i], dense_v[i])
                # the module rounds the attention output to the model dtype before o_proj
                grid = 2.0 ** (-11 if dtype == "fp16" else -8)
                err = np.abs(got - ref) - grid * np.abs(ref)
                assert err.max() <= attn_tol(dtype), ("decode attention", s, i, err.max())
                # the module's own output: o_proj of what it was handed, checked in float32
                w = model.layers[i].self_attn.o_proj.weight.float()
                want = captured[i] @ w.t()
                assert float((projected[i] - want).abs().max()) <= 2.0 ** -7 * max(1.0, float(want.abs().max()))
        for h in hooks + hk:
            h.remove()
    assert cache.get_seq_length(0) == P + steps
    if compressed:
        assert cache.key_cache[0]["k_uncompressed"].shape[1] == P - S - W + steps


def test_attention_module_output_is_o_proj_of_attention():
    """One ``LlamaSdpaAttention`` on its own: the returned tensor equals ``o_proj`` applied (in float32) to
    the oracle's attention output, on the Fourier decode branch."""
    from fourierattention_b200 import DynamicCache
    from fourierattention_b200.modeling_llama_fourier import LlamaConfig, LlamaSdpaAttention, apply_rotary_pos_emb
    B, hidden, Hq, Hkv, D, S, W, M, P = 2, 128, 4, 2, 32, 2, 10, 8, 90
    torch.manual_seed(3)
    cfg = LlamaConfig(hidden_size=hidden, num_attention_heads=Hq, num_key_value_heads=Hkv, num_hidden_layers=1)
    at = LlamaSdpaAttention(cfg, layer_idx=0)
    for p_ in at.parameters():
        p_.data.normal_(0.0, 0.1)
    at = at.to("cuda", torch.float16).eval()
    tables = fo.make_splithead_tables(1, Hkv, D, 20, seed=5)
    path = write_tables(tables)
    try:
        cache = DynamicCache(make_config(dict(S=S, W=W, M=M, mpe=4096, Hkv=Hkv, steps=2), path))
    finally:
        os.unlink(path)
    oc = fo.OracleCache([fo.DimTables(tables["Layer_0"])], S, W, M, 2, 4096, "fp16")
    hs = (torch.randn(B, P + 1, hidden, device="cuda") * 0.5).half()

    def qkv(x, pos):
        b, n, _ = x.shape
        q = at.q_proj(x).view(b, n, Hq, D).transpose(1, 2)
        k = at.k_proj(x).view(b, n, Hkv, D).transpose(1, 2)
        v = at.v_proj(x).view(b, n, Hkv, D).transpose(1, 2)
        cos, sin = at.rotary_emb(v, pos)
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        return q, k, v
    with torch.no_grad():
        pos = torch.arange(P, device="cuda")[None].expand(B, -1)
        o, none, pk = at(hs[:, :P], position_ids=pos, past_key_value=cache)
        assert none is None and pk is cache and tuple(o.shape) == (B, P, hidden)
        q, k, v = qkv(hs[:, :P], pos)
        oc.update(_to_oracle(k), _to_oracle(v), 0)
        pos1 = torch.full((B, 1), P, device="cuda")
        o, _, _ = at(hs[:, P:P + 1], position_ids=pos1, past_key_value=cache)
        q, k, v = qkv(hs[:, P:P + 1], pos1)
        oc.update(_to_oracle(k), _to_oracle(v), 0)
        for nm in ("k_scale", "v_scale", "k_layer_average", "v_layer_average", "kd_layer_average", "vd_layer_average"):
            getattr(oc, nm)[0] = host(getattr(cache, nm)[0])
        ref = oc.attend(_to_oracle(q)[:, :, 0].reshape(B, -1), 0, Hq, Hkv, faithful=False)[:, :, 0].reshape(B, 1, Hq * D)
        want = torch.from_numpy(ref).cuda().float() @ at.o_proj.weight.float().t()
        scale = float(want.abs().max())
        assert float((o.float() - want).abs().max()) <= 4e-3 * max(1.0, scale)
        with pytest.raises(NotImplementedError):
            at(hs[:, P:P + 1], position_ids=pos1, past_key_value=cache, output_attentions=True)


# ------------------------------------------------------------------------------------------------
# head sharding through the cache class
# ------------------------------------------------------------------------------------------------
def test_cache_head_shards_equal_unsharded():
    from fourierattention_b200 import DynamicCache
    g = dict(B=2, Hq=16, Hkv=4, D=64, S=4, W=40, M=32, P=1500, steps=3, mpe=1 << 20, dtype="bf16", ncomp=40,
             ragged=False, seed=611)
    tables, k, v, qs = case_inputs(g)
    dt, P, D, R = g["dtype"], g["P"], g["D"], g["Hq"] // g["Hkv"]
    path = write_tables(tables)
    try:
        full = DynamicCache(make_config(g, path))
        shards = [DynamicCache(make_config(g, path), kv_head_range=r) for r in ((0, 1), (1, 4))]
    finally:
        os.unlink(path)
    oc = oracle_cache(g, tables)
    full.update(update_arg(k[:, :, :P], dt), update_arg(v[:, :, :P], dt), 0)
    oc.update(k[:, :, :P], v[:, :, :P], 0)
    for c, (h0, h1) in zip(shards, ((0, 1), (1, 4))):
        c.update(update_arg(k[:, h0:h1, :P], dt), update_arg(v[:, h0:h1, :P], dt), 0)
    for nm in ("k_scale", "v_scale", "k_layer_average", "v_layer_average", "kd_layer_average", "vd_layer_average"):
        getattr(oc, nm)[0] = host(getattr(full, nm)[0])
    for s in range(g["steps"]):
        sl = slice(P + s, P + s + 1)
        full.update(update_arg(k[:, :, sl], dt), update_arg(v[:, :, sl], dt), 0)
        oc.update(k[:, :, sl], v[:, :, sl], 0)
        want = host(full.fourier_attention(dev(qs[s], dt), 0, g["Hq"]))
        ideal = oc.attend(qs[s], 0, g["Hq"], g["Hkv"], faithful=False)
        assert np.abs(want - ideal).max() <= 1.5e-4
        parts = []
        for c, (h0, h1) in zip(shards, ((0, 1), (1, 4))):
            c.update(update_arg(k[:, h0:h1, sl], dt), update_arg(v[:, h0:h1, sl], dt), 0)
            ql = qs[s].reshape(g["B"], g["Hq"], D)[:, h0 * R:h1 * R].reshape(g["B"], -1)
            parts.append(host(c.fourier_attention(dev(ql, dt), 0, (h1 - h0) * R)))
        got = np.concatenate(parts, axis=1)
        # a shard's chunk plan differs from the unsharded one (fewer heads per launch), so the two results
        # agree to rounding, not bit for bit; both are held to the oracle
        assert np.abs(got - ideal).max() <= 1.5e-4
        assert np.abs(got - want).max() <= 2e-4
    for c, (h0, h1) in zip(shards, ((0, 1), (1, 4))):
        tb = oc.tables[0]
        ck = slice(tb.kc_h[h0], tb.kc_h[h1])
        assert np.array_equal(host(c.key_cache[0]["k_local"]), host(full.key_cache[0]["k_local"])[:, :, h0 * D:h1 * D])
        assert np.abs(host(c.key_cache[0]["k_compressed"]) - host(full.key_cache[0]["k_compressed"])[:, :, ck]).max() <= 1e-3


# ------------------------------------------------------------------------------------------------
# sequence split through the cache class
# ------------------------------------------------------------------------------------------------
SEQ_G = dict(B=2, Hq=8, Hkv=2, D=64, S=4, W=24, M=32, P=1300, steps=3, mpe=1 << 20, dtype="bf16", ncomp=40,
             ragged=False, seed=612)


def _seq_rank(rank, world, port, backend, out, g=SEQ_G):
    """One rank of the sequence split: builds DynamicCache(seq_shard=(rank, world)), runs prefill and the
    decode steps, and (rank 0) compares the merged result with the oracle."""
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from fourierattention_b200 import DynamicCache
    torch.cuda.set_device(rank % torch.cuda.device_count())
    if world > 1 or backend:
        dist.init_process_group(backend or "nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        tables, k, v, qs = case_inputs(g)
        dt, P = g["dtype"], g["P"]
        path = write_tables(tables)
        try:
            cache = DynamicCache(make_config(g, path), seq_shard=(rank, world))
        finally:
            os.unlink(path)
        oc = oracle_cache(g, tables)
        cache.update(update_arg(k[:, :, :P], dt), update_arg(v[:, :, :P], dt), 0)
        oc.update(k[:, :, :P], v[:, :, :P], 0)
        err_coef = float(np.abs(host(cache.key_cache[0]["k_compressed"]) - oc.key_cache[0]["k_compressed"]).max())
        for nm in ("k_scale", "v_scale", "k_layer_average", "v_layer_average", "kd_layer_average", "vd_layer_average"):
            getattr(oc, nm)[0] = host(getattr(cache, nm)[0])
        worst = 0.0
        for s in range(g["steps"]):
            sl = slice(P + s, P + s + 1)
            cache.update(update_arg(k[:, :, sl], dt), update_arg(v[:, :, sl], dt), 0)
            oc.update(k[:, :, sl], v[:, :, sl], 0)
            o = host(cache.fourier_attention(dev(qs[s], dt), 0, g["Hq"]))
            ideal = oc.attend(qs[s], 0, g["Hq"], g["Hkv"], faithful=False)
            worst = max(worst, float(np.abs(o - ideal).max()))
        err_coef = max(err_coef, float(np.abs(host(cache.key_cache[0]["k_compressed"]) - oc.key_cache[0]["k_compressed"]).max()))
        out[f"attn{rank}"] = worst
        out[f"coef{rank}"] = err_coef
    finally:
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()


def test_cache_sequence_split_one_rank_group():
    """world = 1: every collective of the split path runs (on a one-rank NCCL group) and the result is the
    unsharded one."""
    out = {}
    _seq_rank(0, 1, _free_port(), "nccl", out)
    assert out["attn0"] <= 1.5e-4 and out["coef0"] <= 2e-3, out


@pytest.mark.parametrize("world", [2])
def test_cache_sequence_split_real_ranks(world):
    """Two processes, one GPU each, NCCL: prefill all_reduce of the coefficient partials, per-step all_gather
    of the partial outputs and the log-sum-exp merge, compared with the oracle on every rank."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_seq_rank, args=(r, world, port, "nccl", out)) for r in range(world)]
    for p_ in procs:
        p_.start()
    for p_ in procs:
        p_.join(300)
        assert p_.exitcode == 0
    res = dict(out)
    assert all(res[f"attn{r}"] <= 1.5e-4 and res[f"coef{r}"] <= 2e-3 for r in range(world)), res


def test_sequence_split_rank_without_rows_still_joins(monkeypatch):
    """A rank whose slice of the span is empty (more ranks than rows) contributes an empty partial instead
    of failing before the collective: 9 middle rows over 8 ranks leave ranks 5-7 without rows.  One such
    rank is run here alone (the prefill all_reduce is replaced by a no-op: its coefficients are not what is
    checked) up to the point where it would enter the all_gather."""
    import torch.distributed as dist
    monkeypatch.setattr(dist, "all_reduce", lambda t, group=None: None)
    from fourierattention_b200.cache_utils_fourier import span_slice
    slices = [span_slice(9, r, 8) for r in range(8)]
    assert slices[4] == (8, 9) and slices[5] == (9, 9) and slices[7] == (9, 9)
    from fourierattention_b200 import DynamicCache
    g = dict(B=1, Hq=4, Hkv=2, D=16, S=2, W=7, M=8, P=18, steps=1, mpe=4096, dtype="fp16", ncomp=12, ragged=False, seed=613)
    tables, k, v, qs = case_inputs(g)
    dt, P = g["dtype"], g["P"]
    path = write_tables(tables)
    try:
        cache = DynamicCache(make_config(g, path), seq_shard=(6, 8))
    finally:
        os.unlink(path)
    cache.update(update_arg(k[:, :, :P], dt), update_arg(v[:, :, :P], dt), 0)
    cache.update(update_arg(k[:, :, P:P + 1], dt), update_arg(v[:, :, P:P + 1], dt), 0)
    o, m, l = cache.partial_attention(dev(qs[0], dt), 0, g["Hq"])
    assert float(l.abs().max()) == 0.0 and bool(torch.isfinite(o).all())
