"""GPU parity at the shapes the benchmark configurations run, through ``DynamicCache`` (prefill, steady-state
``update`` and ``fourier_attention``) and against the CPU oracle -- not against another GPU entry point.

Covered: the Llama-3.1-8B / 32k layer exactly as the benchmark runs it (several sequences per launch, the
two periods ``T_c = T - 1``, the warp-specialised pass with the accumulator in tensor memory), the single-layer fp16 configuration with its 64
decode steps, the Llama-3.2-3B layer (24 query heads, 80 of 128 dims compressed) and one long single
sequence (131072 tokens, M = 1024).

The float64 rebuild of a 32k span costs a few seconds per sequence on the host, so the oracle follows two
sequences of the batch and the "ideal" result uses the oracle's reassociated float64 form (which the CPU
suite proves equal to its rebuild-then-attend form).
"""
import os

import numpy as np
import pytest
import torch

from oracle import fourier_oracle as fo
from tests.gpu_util import dev, host, update_arg, write_tables
from tests.helpers import attn_err_excess, attn_tol

pytestmark = pytest.mark.gpu

STAT_NAMES = ("k_scale", "v_scale", "k_layer_average", "v_layer_average", "kd_layer_average", "vd_layer_average")


def _config(g, path):
    import types
    return types.SimpleNamespace(numinittokens=g["S"], maxlocallen=g["W"], maxmidstates=g["M"],
                                 non_critical_dims_path=path, max_position_embeddings=g["mpe"],
                                 num_key_value_heads=g["Hkv"], max_new_tokens=g["new_tokens"], model_type="llama")


def _ideal(oc, q, Hq, Hkv):
    """float64 attention on the oracle's state, reassociated form (cheap at long spans)."""
    kc, vc, tb = oc.key_cache[0], oc.value_cache[0], oc.tables[0]
    return fo.fourier_attn_reassociated(
        q, np.concatenate([kc["k_init"], kc["k_local"]], 1), np.concatenate([vc["v_init"], vc["v_local"]], 1),
        kc["k_compressed"], vc["v_compressed"], kc["k_uncompressed"], vc["v_uncompressed"],
        oc.k_layer_average[0], oc.kd_layer_average[0], oc.k_scale[0], oc.v_layer_average[0], oc.vd_layer_average[0],
        oc.v_scale[0], tb.kc, tb.kc_h, tb.kn, tb.kn_h, tb.vc, tb.vc_h, tb.vn, tb.vn_h, Hq, Hkv, oc.T)


def _run(g, follow, steps, check_steps, faithful_steps, want_path, ideal_tol=1.5e-4, coef_rel=0.0):
    """Prefill + ``steps`` decode steps on the GPU cache (all B sequences) and on the oracle (the sequences
    listed in ``follow``); outputs compared at ``check_steps``."""
    from fourierattention_b200 import DynamicCache, ops
    dt = g["dtype"]
    tables = fo.make_splithead_tables(1, g["Hkv"], g["D"], g["ncomp"], g["seed"])
    k, v = fo.synth_kv(g["seed"], g["B"], g["Hkv"], g["P"] + steps, g["D"], dt)
    rng = np.random.default_rng(g["seed"] + 1000)
    qs = fo.rnd(rng.standard_normal((steps, g["B"], g["Hq"] * g["D"])).astype(np.float32), dt)
    path = write_tables(tables)
    try:
        cache = DynamicCache(_config(g, path))
    finally:
        os.unlink(path)
    oc = fo.OracleCache([fo.DimTables(tables["Layer_0"])], g["S"], g["W"], g["M"], g["new_tokens"], g["mpe"], dt)
    P = g["P"]
    cache.update(update_arg(k[:, :, :P], dt), update_arg(v[:, :, :P], dt), 0)
    oc.update(k[follow][:, :, :P], v[follow][:, :, :P], 0)
    assert cache.attention_period == oc.T
    if "T" in g:
        assert oc.T == g["T"] and fo.compress_period(oc.T) == g.get("T_c", g["T"])
    kc, vc = cache.key_cache[0], cache.value_cache[0]
    okc, ovc = oc.key_cache[0], oc.value_cache[0]
    # cache layout bit exact, coefficients within the contract
    assert np.array_equal(host(kc["k_uncompressed"][follow]), okc["k_uncompressed"])
    assert np.array_equal(host(vc["v_uncompressed"][follow]), ovc["v_uncompressed"])
    assert np.array_equal(host(kc["k_local"][follow]), okc["k_local"])
    assert np.array_equal(host(kc["k_init"][follow]), okc["k_init"])
    tol = attn_tol(dt)
    for mine, ref in ((kc["k_compressed"], okc["k_compressed"]), (vc["v_compressed"], ovc["v_compressed"])):
        err = np.abs(host(mine[follow]) - ref).max()
        assert err <= max(tol, coef_rel * np.abs(ref).max()), ("prefill coefficients", err)
    # the statistics are compared on their own grids, then the oracle continues with the cache's values so
    # that a one-ulp flip of a float16 statistic cannot mask (or fake) an error of the attention kernel
    for nm in STAT_NAMES:
        mine, ref = host(getattr(cache, nm)[0][follow]), np.asarray(getattr(oc, nm)[0], np.float32)
        rel = 2.0 ** -7 if (dt == "bf16" and nm in ("k_layer_average", "v_layer_average")) else 2.0 ** -9
        assert np.all(np.abs(mine - ref) <= rel * np.maximum(np.abs(ref), 2.0 ** -14) + 1e-6), nm
        getattr(oc, nm)[0] = mine
    for s in range(steps):
        cache.update(update_arg(k[:, :, P + s:P + s + 1], dt), update_arg(v[:, :, P + s:P + s + 1], dt), 0)
        oc.update(k[follow][:, :, P + s:P + s + 1], v[follow][:, :, P + s:P + s + 1], 0)
        o = cache.fourier_attention(dev(qs[s], dt), 0, g["Hq"])
        assert ops.last_decode_path in want_path, ops.last_decode_path
        assert tuple(o.shape) == (g["B"], g["Hq"], 1, g["D"]) and o.dtype == torch.float32
        assert bool(torch.isfinite(o).all())
        if s in check_steps:
            mine = host(o[follow])
            ideal = _ideal(oc, qs[s][follow], g["Hq"], g["Hkv"])
            err = np.abs(mine - ideal).max()
            assert err <= ideal_tol * max(1.0, np.abs(ideal).max()), (s, err)
            if s in faithful_steps:
                ref = oc.attend(qs[s][follow], 0, g["Hq"], g["Hkv"], faithful=True)
                assert attn_err_excess(mine, ref, dt) <= 0, (s, np.abs(mine - ref).max())
    kc, vc = cache.key_cache[0], cache.value_cache[0]
    okc, ovc = oc.key_cache[0], oc.value_cache[0]
    assert cache.curr_tokennum[0] == oc.curr_tokennum[0]
    assert np.array_equal(host(kc["k_local"][follow]), okc["k_local"])
    assert np.array_equal(host(vc["v_local"][follow]), ovc["v_local"])
    assert np.array_equal(host(kc["k_uncompressed"][follow][:, -steps:]), okc["k_uncompressed"][:, -steps:])
    assert np.array_equal(host(vc["v_uncompressed"][follow][:, -steps:]), ovc["v_uncompressed"][:, -steps:])
    for mine, ref in ((kc["k_compressed"], okc["k_compressed"]), (vc["v_compressed"], ovc["v_compressed"])):
        err = np.abs(host(mine[follow]) - ref).max()
        assert err <= max(tol, coef_rel * np.abs(ref).max()), ("final coefficients", err)
    return cache


def test_llama31_8b_32k_layer_as_benchmarked():
    """32 query / 8 KV heads, D = 128, bf16, 32768-token prompts, M = 512, max_new_tokens = 256 so that
    T = 31996 and the projection period is T - 1; four sequences per launch, three decode steps."""
    g = dict(B=4, Hq=32, Hkv=8, D=128, S=4, W=1024, M=512, P=32768, new_tokens=256, mpe=1 << 30, dtype="bf16",
             ncomp=96, seed=4201, T=31996, T_c=31995)
    _run(g, follow=[0, 3], steps=3, check_steps={0, 1, 2}, faithful_steps={2}, want_path=(3,))


def test_single_layer_8k_fp16_64_steps():
    """The single-layer configuration: fp16, context 8192, W = 1024, M = 256, 64 decode steps; outputs are
    checked every 8th step and the final state after all 64."""
    g = dict(B=1, Hq=32, Hkv=8, D=128, S=4, W=1024, M=256, P=8192, new_tokens=64, mpe=131072, dtype="fp16",
             ncomp=96, seed=4202, T=7228)
    _run(g, follow=[0], steps=64, check_steps=set(range(7, 64, 8)) | {0}, faithful_steps={0, 63}, want_path=(1, 2, 3))


def test_llama32_3b_16k_layer():
    """24 query / 8 KV heads, 80 of 128 dims compressed (384 verbatim columns per row), W = 512, M = 256."""
    g = dict(B=4, Hq=24, Hkv=8, D=128, S=4, W=512, M=256, P=16384, new_tokens=256, mpe=1 << 30, dtype="bf16",
             ncomp=80, seed=4203)
    _run(g, follow=[1, 2], steps=3, check_steps={0, 2}, faithful_steps={2}, want_path=(2,))


def test_long_single_sequence_131k():
    """One 131072-token sequence, W = 2048, M = 1024 (N = 512 frequencies)."""
    g = dict(B=1, Hq=32, Hkv=8, D=128, S=4, W=2048, M=1024, P=131072, new_tokens=16, mpe=1 << 30, dtype="bf16",
             ncomp=96, seed=4204)
    # |C| reaches ~1e3 at this span, so the absolute 2e-3 contract sits at the float32 rounding floor of the
    # coefficients themselves; the allowance grows with their size here (4e-6 relative to the largest one)
    _run(g, follow=[0], steps=2, check_steps={0, 1}, faithful_steps=set(), want_path=(2,), coef_rel=4e-6)


def test_llama31_8b_32k_kv_head_shards_as_benchmarked():
    """The shards the 4- and 8-GPU benchmark lines run: 2 of 8 and 1 of 8 KV heads of the Llama-3.1-8B / 32k layer
    (``kv_head_range``), eight sequences, so that four sequences share a CTA of the warp-specialised pass and the
    sinks+window rows go through tiles of 32 and 64 rows.  Each shard is compared with the same heads of the
    unsharded cache, which the test above holds to the oracle; the chunk plans differ, so the results agree to
    rounding."""
    from fourierattention_b200 import DynamicCache, ops
    g = dict(B=8, Hq=32, Hkv=8, D=128, S=4, W=1024, M=512, P=32768, new_tokens=256, mpe=1 << 30, dtype="bf16",
             ncomp=96, seed=4205)
    dt, P, D, R, steps = g["dtype"], g["P"], g["D"], g["Hq"] // g["Hkv"], 2
    tables = fo.make_splithead_tables(1, g["Hkv"], D, g["ncomp"], g["seed"])
    k, v = fo.synth_kv(g["seed"], g["B"], g["Hkv"], P + steps, D, dt)
    rng = np.random.default_rng(g["seed"] + 1000)
    qs = fo.rnd(rng.standard_normal((steps, g["B"], g["Hq"] * D)).astype(np.float32), dt)
    ranges = ((2, 4), (7, 8))
    path = write_tables(tables)
    try:
        full = DynamicCache(_config(g, path))
        shards = [DynamicCache(_config(g, path), kv_head_range=r) for r in ranges]
    finally:
        os.unlink(path)
    full.update(update_arg(k[:, :, :P], dt), update_arg(v[:, :, :P], dt), 0)
    for c, (h0, h1) in zip(shards, ranges):
        c.update(update_arg(k[:, h0:h1, :P], dt), update_arg(v[:, h0:h1, :P], dt), 0)
    for s in range(steps):
        sl = slice(P + s, P + s + 1)
        full.update(update_arg(k[:, :, sl], dt), update_arg(v[:, :, sl], dt), 0)
        want = host(full.fourier_attention(dev(qs[s], dt), 0, g["Hq"]))
        assert ops.last_decode_path == 3
        for c, (h0, h1) in zip(shards, ranges):
            c.update(update_arg(k[:, h0:h1, sl], dt), update_arg(v[:, h0:h1, sl], dt), 0)
            ql = qs[s].reshape(g["B"], g["Hq"], D)[:, h0 * R:h1 * R].reshape(g["B"], -1)
            got = host(c.fourier_attention(dev(ql, dt), 0, (h1 - h0) * R))
            assert ops.last_decode_path == 3, ops.last_decode_path
            ref = want[:, h0 * R:h1 * R]
            assert np.isfinite(got).all()
            assert np.abs(got - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max()), (s, (h0, h1), np.abs(got - ref).max())
