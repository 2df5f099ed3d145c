"""Two-rank checks of the sharding logic on CPU (gloo): the product's table sharding / span slicing feed the
CPU oracle on each rank, results travel through torch.distributed collectives exactly as the GPU path sends
them, and the reassembled answer must equal the single-rank answer."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _state():
    from oracle import fourier_oracle as fo
    from tests.helpers import case_inputs
    g = dict(B=2, Hq=8, Hkv=4, D=16, S=3, W=9, M=8, P=90, steps=1, mpe=4096, dtype="fp16", ncomp=10, ragged=True, seed=77)
    tables, k, v, qs = case_inputs(g)
    oc = fo.OracleCache([fo.DimTables(tables["Layer_0"])], g["S"], g["W"], g["M"], 4, g["mpe"], g["dtype"])
    oc.update(k[:, :, :g["P"]], v[:, :, :g["P"]], 0)
    oc.update(k[:, :, g["P"]:g["P"] + 1], v[:, :, g["P"]:g["P"] + 1], 0)
    return g, tables, oc, qs[0]


def _attend(fo, g, oc, tb, q, kc, vc, stats, Hq, Hkv, faithful=False):
    return fo.fourier_attn(q, np.concatenate([kc["k_init"], kc["k_local"]], 1),
                           np.concatenate([vc["v_init"], vc["v_local"]], 1), kc["k_compressed"], vc["v_compressed"],
                           kc["k_uncompressed"], vc["v_uncompressed"], *stats, tb.kc, tb.kn, tb.vc, tb.vn, Hq, Hkv,
                           oc.T, g["dtype"], faithful=faithful)


def _head_shard_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    from oracle import fourier_oracle as fo
    from fourierattention_b200.cache_utils_fourier import shard_tables
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    g, tables, oc, q = _state()
    D, R = g["D"], g["Hq"] // g["Hkv"]
    hk = g["Hkv"] // world
    h0, h1 = rank * hk, (rank + 1) * hk
    tb_full = oc.tables[0]
    tb = fo.DimTables(shard_tables(tables["Layer_0"], h0, h1))
    sl = slice(h0 * D, h1 * D)
    ck, cv = slice(tb_full.kc_h[h0], tb_full.kc_h[h1]), slice(tb_full.vc_h[h0], tb_full.vc_h[h1])
    nk, nv = slice(tb_full.kn_h[h0], tb_full.kn_h[h1]), slice(tb_full.vn_h[h0], tb_full.vn_h[h1])
    kc, vc = oc.key_cache[0], oc.value_cache[0]
    kcl = {"k_init": kc["k_init"][:, :, sl], "k_local": kc["k_local"][:, :, sl],
           "k_compressed": kc["k_compressed"][:, :, ck], "k_uncompressed": kc["k_uncompressed"][:, :, nk]}
    vcl = {"v_init": vc["v_init"][:, :, sl], "v_local": vc["v_local"][:, :, sl],
           "v_compressed": vc["v_compressed"][:, :, cv], "v_uncompressed": vc["v_uncompressed"][:, :, nv]}
    stats = (oc.k_layer_average[0][:, ck], oc.kd_layer_average[0][:, ck], oc.k_scale[0][:, ck],
             oc.v_layer_average[0][:, cv], oc.vd_layer_average[0][:, cv], oc.v_scale[0][:, cv])
    ql = q.reshape(g["B"], g["Hq"], D)[:, h0 * R:h1 * R].reshape(g["B"], -1)
    mine = _attend(fo, g, oc, tb, ql, kcl, vcl, stats, hk * R, hk)                  # (B, hk*R, 1, D)
    parts = [torch.empty_like(torch.from_numpy(mine)) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(mine)))            # no collective on the data path
    if rank == 0:                                                                   # itself; this only collects
        full = torch.cat(parts, dim=1).numpy()
        stats_f = (oc.k_layer_average[0], oc.kd_layer_average[0], oc.k_scale[0], oc.v_layer_average[0],
                   oc.vd_layer_average[0], oc.v_scale[0])
        want = _attend(fo, g, oc, tb_full, q, kc, vc, stats_f, g["Hq"], g["Hkv"])
        out["err"] = float(np.abs(full - want).max())
    dist.barrier()
    dist.destroy_process_group()


def _seq_split_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    from oracle import fourier_oracle as fo
    from fourierattention_b200.cache_utils_fourier import span_slice
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    g, tables, oc, q = _state()
    tb = oc.tables[0]
    kc, vc = oc.key_cache[0], oc.value_cache[0]
    n_mid = kc["k_uncompressed"].shape[1]
    lo, hi = span_slice(n_mid, rank, world)
    D, Hq, Hkv, B = g["D"], g["Hq"], g["Hkv"], g["B"]
    R = Hq // Hkv
    N = kc["k_compressed"].shape[1] // 2
    sm = 1.0 / np.sqrt(D)
    qh = q.reshape(B, Hq, D).astype(np.float64)
    fc, fs = fo._basis_exact(np.arange(lo, hi), N, oc.T)                            # phases at the slice's span positions
    o = np.zeros((B * Hq, D)); m = np.zeros(B * Hq); l = np.zeros(B * Hq)
    for b in range(B):
        for h in range(Hq):
            gk = h // R
            xk = (np.concatenate([fc, fs], 1) @ kc["k_compressed"][b].astype(np.float64)) / N
            xk = (xk - oc.kd_layer_average[0][b]) * oc.k_scale[0][b] + oc.k_layer_average[0][b]
            xv = (np.concatenate([fc, fs], 1) @ vc["v_compressed"][b].astype(np.float64)) / N
            xv = (xv - oc.vd_layer_average[0][b]) * oc.v_scale[0][b] + oc.v_layer_average[0][b]
            km = np.zeros((hi - lo, Hkv * D)); vm = np.zeros((hi - lo, Hkv * D))
            km[:, tb.kc] = xk; km[:, tb.kn] = kc["k_uncompressed"][b, lo:hi]
            vm[:, tb.vc] = xv; vm[:, tb.vn] = vc["v_uncompressed"][b, lo:hi]
            ks, vs = km[:, gk * D:(gk + 1) * D], vm[:, gk * D:(gk + 1) * D]
            if rank == 0:                                                           # sinks + window live on rank 0
                il_k = np.concatenate([kc["k_init"][b], kc["k_local"][b]])[:, gk * D:(gk + 1) * D]
                il_v = np.concatenate([vc["v_init"][b], vc["v_local"][b]])[:, gk * D:(gk + 1) * D]
                ks, vs = np.concatenate([il_k, ks]), np.concatenate([il_v, vs])
            s = (ks @ qh[b, h]) * sm * np.log2(np.e)
            mm = s.max()
            p = np.exp2(s - mm)
            i = b * Hq + h
            m[i], l[i], o[i] = mm, p.sum(), (p @ vs) / p.sum()
    pack = torch.from_numpy(np.concatenate([o, m[:, None], l[:, None]], 1))          # Hq*(D+2) numbers per sequence
    parts = [torch.empty_like(pack) for _ in range(world)]
    dist.all_gather(parts, pack)
    allp = torch.stack(parts).numpy()
    merged = fo.merge_partials(allp[:, :, D].T, allp[:, :, D + 1].T,
                               (allp[:, :, :D] * allp[:, :, D + 1:D + 2]).transpose(1, 0, 2))
    stats_f = (oc.k_layer_average[0], oc.kd_layer_average[0], oc.k_scale[0], oc.v_layer_average[0],
               oc.vd_layer_average[0], oc.v_scale[0])
    want = _attend(fo, g, oc, tb, q, kc, vc, stats_f, Hq, Hkv).reshape(B * Hq, D)
    out[f"err{rank}"] = float(np.abs(merged - want).max())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("worker", [_head_shard_worker, _seq_split_worker])
def test_two_ranks(worker):
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=worker, args=(r, world, port, out)) for r in range(world)]
    for p_ in procs:
        p_.start()
    for p_ in procs:
        p_.join(180)
        assert p_.exitcode == 0
    assert out and all(v < 1e-10 for v in out.values()), dict(out)


def test_shard_tables_partition():
    from fourierattention_b200.cache_utils_fourier import shard_tables, span_slice
    from oracle import fourier_oracle as fo
    t = fo.make_splithead_tables(1, 8, 16, 10, 5, ragged=True)["Layer_0"]
    seen = {k: [] for k in ("kc", "kn", "vc", "vn")}
    for h0, h1 in ((0, 3), (3, 4), (4, 8)):
        s = shard_tables(t, h0, h1)
        for k in seen:
            assert len(s[f"{k}_h_list"]) == h1 - h0 and (not s[f"{k}_h_list"] or s[f"{k}_h_list"][-1] == len(s[f"{k}_list"]))
            assert all(0 <= i < (h1 - h0) * 16 for i in s[f"{k}_list"])
            seen[k] += [i + h0 * 16 for i in s[f"{k}_list"]]
    for k in seen:
        assert seen[k] == t[f"{k}_list"]
    cuts = [span_slice(1001, r, 4) for r in range(4)]
    assert cuts[0][0] == 0 and cuts[-1][1] == 1001 and all(cuts[i][1] == cuts[i + 1][0] for i in range(3))
