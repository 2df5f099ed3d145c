"""GPU parity of the cache + decode attention against the golden fixtures (outputs of the reference's
own code) and against the CPU oracle, through the drop-in Python API and the C ABI underneath."""
import os

import numpy as np
import pytest
import torch

from oracle import fourier_oracle as fo
from tests.gpu_util import dev, host, make_config, oracle_cache, update_arg, write_tables
from tests.helpers import GOLDEN_CASES, attn_err_excess, attn_tol, case_inputs, load_golden

pytestmark = pytest.mark.gpu


def _ulp_close(mine, ref, rel):
    return np.all(np.abs(mine - ref) <= rel * np.maximum(np.abs(ref), 2.0 ** -14) + 1e-7)


@pytest.mark.parametrize("name", [c for c in GOLDEN_CASES if c != "short_fp16"])
def test_golden_case(name):
    from fourierattention_b200 import DynamicCache
    z, g = load_golden(name)
    tables, k, v, qs = case_inputs(g)
    path = write_tables(tables)
    try:
        cache = DynamicCache(make_config(g, path))
    finally:
        os.unlink(path)
    P, dt = g["P"], g["dtype"]
    kd, vd = cache.update(update_arg(k[:, :, :P], dt), update_arg(v[:, :, :P], dt), 0)
    assert kd["k_init"] is None and kd["k_compressed"] is None and kd["k_uncompressed"] is None
    assert tuple(kd["k_local"].shape) == (g["B"], P, g["Hkv"] * g["D"])
    assert cache.maxtokens == int(z["maxtokens"])
    assert cache.curr_tokennum[0] == int(z["curr_tokennum_prefill"])
    kc, vc = cache.key_cache[0], cache.value_cache[0]
    # cache layout: bit exact
    assert np.array_equal(host(kc["k_uncompressed"]), z["pre_k_uncompressed"])
    assert np.array_equal(host(vc["v_uncompressed"]), z["pre_v_uncompressed"])
    assert kc["k_compressed"].dtype == torch.float32
    tol = attn_tol(dt)
    for mine, ref in ((kc["k_compressed"], z["pre_k_compressed"]), (vc["v_compressed"], z["pre_v_compressed"])):
        assert tuple(mine.shape) == ref.shape
        assert np.abs(host(mine) - ref).max() <= tol
    for nm in ("k_scale", "v_scale", "k_layer_average", "v_layer_average", "kd_layer_average", "vd_layer_average"):
        t = getattr(cache, nm)[0]
        assert str(t.dtype) == str(z[nm + "_dtype"]), nm
        rel = 2.0 ** -7 if (dt == "bf16" and nm in ("k_layer_average", "v_layer_average")) else 2.0 ** -10
        assert _ulp_close(host(t), z[nm], rel), nm
    # decode with the reference's statistics so that a one-ulp flip there cannot mask (or fake) an
    # error of the attention kernel; the statistics themselves were compared just above
    cache.set_layer_statistics(0, tuple(dev(np.asarray(z[nm], np.float32)) for nm in (
        "k_layer_average", "kd_layer_average", "k_scale", "v_layer_average", "vd_layer_average", "v_scale")))
    for s in range(g["steps"]):
        kd, vd = cache.update(update_arg(k[:, :, P + s:P + s + 1], dt), update_arg(v[:, :, P + s:P + s + 1], dt), 0)
        assert kd["k_init"] is not None
        assert cache.get_seq_length(0) == int(z[f"seq_len_{s}"])
        o = cache.fourier_attention(dev(qs[s], dt), 0, g["Hq"])
        ref = z[f"attn_{s}"]
        assert tuple(o.shape) == ref.shape and o.dtype == torch.float32
        assert attn_err_excess(host(o), ref, dt) <= 0, (s, np.abs(host(o) - ref).max())
    kc, vc = cache.key_cache[0], cache.value_cache[0]
    assert cache.curr_tokennum[0] == int(z["curr_tokennum_final"])
    assert np.array_equal(host(kc["k_local"]), z["fin_k_local"])
    assert np.array_equal(host(vc["v_local"]), z["fin_v_local"])
    assert np.array_equal(host(kc["k_init"]), z["fin_k_init"])
    assert np.array_equal(host(kc["k_uncompressed"][:, -g["steps"]:]), z["fin_k_uncompressed_tail"])
    assert np.array_equal(host(vc["v_uncompressed"][:, -g["steps"]:]), z["fin_v_uncompressed_tail"])
    for mine, ref in ((kc["k_compressed"], z["fin_k_compressed"]), (vc["v_compressed"], z["fin_v_compressed"])):
        assert np.abs(host(mine) - ref).max() <= tol


def test_short_prompt_is_never_compressed():
    from fourierattention_b200 import DynamicCache
    z, g = load_golden("short_fp16")
    tables, k, v, qs = case_inputs(g)
    path = write_tables(tables)
    try:
        cache = DynamicCache(make_config(g, path))
    finally:
        os.unlink(path)
    P, dt = g["P"], g["dtype"]
    cache.update(update_arg(k[:, :, :P], dt), update_arg(v[:, :, :P], dt), 0)
    for s in range(g["steps"]):
        kd, vd = cache.update(update_arg(k[:, :, P + s:P + s + 1], dt), update_arg(v[:, :, P + s:P + s + 1], dt), 0)
        assert kd["k_init"] is None and kd["k_compressed"] is None and kd["k_uncompressed"] is None
        assert kd["k_local"].shape[1] == int(z[f"local_len_{s}"])
        assert cache.get_seq_length(0) == int(z[f"seq_len_{s}"])
        want = np.ascontiguousarray(k[:, :, :P + s + 1].transpose(0, 2, 1, 3)).reshape(g["B"], P + s + 1, -1)
        assert np.array_equal(host(kd["k_local"]), want)


def test_window_wraps_many_steps():
    """More decode steps than the window is long: the sliding view is copied back to the front of its
    buffer several times; state and outputs must keep matching the oracle."""
    from fourierattention_b200 import DynamicCache
    g = dict(B=2, Hq=4, Hkv=2, D=16, S=3, W=5, M=8, P=60, steps=17, mpe=4096, dtype="fp16", ncomp=10, ragged=False, seed=31)
    tables, k, v, qs = case_inputs(g)
    path = write_tables(tables)
    try:
        cache = DynamicCache(make_config(g, path))
    finally:
        os.unlink(path)
    oc = oracle_cache(g, tables)
    P, dt = g["P"], g["dtype"]
    cache.update(update_arg(k[:, :, :P], dt), update_arg(v[:, :, :P], dt), 0)
    oc.update(k[:, :, :P], v[:, :, :P], 0)
    for nm in ("k_scale", "v_scale", "k_layer_average", "v_layer_average", "kd_layer_average", "vd_layer_average"):
        getattr(oc, nm)[0] = host(getattr(cache, nm)[0])
    for s in range(g["steps"]):
        kd, vd = cache.update(update_arg(k[:, :, P + s:P + s + 1], dt), update_arg(v[:, :, P + s:P + s + 1], dt), 0)
        okd, ovd = oc.update(k[:, :, P + s:P + s + 1], v[:, :, P + s:P + s + 1], 0)
        assert np.array_equal(host(kd["k_local"]), okd["k_local"])
        assert np.array_equal(host(vd["v_local"]), ovd["v_local"])
        assert np.array_equal(host(kd["k_uncompressed"]), okd["k_uncompressed"])
        assert np.abs(host(kd["k_compressed"]) - okd["k_compressed"]).max() <= attn_tol(dt)
        o = cache.fourier_attention(dev(qs[s], dt), 0, g["Hq"])
        ref = oc.attend(qs[s], 0, g["Hq"], g["Hkv"], faithful=False)
        assert np.abs(host(o) - ref).max() <= 1e-4, s


def test_reference_module_names():
    import fourierattention_b200 as pkg
    pkg.install_aliases(overwrite=True)
    import lxr_cache_utils_fourier as cu
    from lxr_fourier_triton_valid4_v2 import MultiDimHiPPO2, mat_avg_std_triton, mat_fourier_avg_std_triton  # noqa
    from modeling_llama_fourier import LLAMA_ATTENTION_CLASSES, LlamaForCausalLM, LlamaSdpaAttention  # noqa
    assert cu.DynamicCache is pkg.DynamicCache


def test_kernel_module_api_matches_oracle():
    """The reference's kernel-module entry points, called with its own argument conventions."""
    from fourierattention_b200 import fourier_triton_valid4_v2 as km
    rng = np.random.default_rng(5)
    B, K, M, N, T = 2, 77, 21, 6, 93
    a = fo.rnd(rng.standard_normal((B, K, M)).astype(np.float32), "fp16")
    ad = dev(a, "fp16")
    c = km.mat_fourier_triton(ad, N, T, K_start=5)
    ref = fo.fourier_project(a, N, T, 5)
    assert c.dtype == torch.float32 and tuple(c.shape) == (B, 2 * N, M)
    assert np.abs(host(c) - ref).max() < 2e-4
    avg, dv = km.mat_avg_std_triton(ad)
    ravg, rdev = fo.col_stats(a, "fp16")
    assert avg.dtype == torch.float16 and _ulp_close(host(avg), ravg, 2.0 ** -10) and _ulp_close(host(dv), rdev, 2.0 ** -10)
    iavg, idev = km.mat_fourier_avg_std_triton(c, K, T)
    ri, rd = fo.recon_stats(ref, K, T)
    assert iavg.dtype == torch.float16 and _ulp_close(host(iavg), ri, 2.0 ** -9) and _ulp_close(host(idev), rd, 2.0 ** -9)
    inv = km.mat_fourier_inv_torch(c, K, T)
    rinv = fo.fourier_reconstruct(ref, K, T, faithful=False)
    assert tuple(inv.shape) == (B, K, M) and np.abs(host(inv) - rinv).max() < 1e-3
    flat = c[0].t().contiguous()
    inv2 = km.mat_fourier_inv_triton(flat, K, T)
    assert np.abs(host(inv2) - rinv[0].T).max() < 1e-3
    hip = km.MultiDimHiPPO2(N=M * 2 * N, input_dim=M, dt=1 / T)
    c0 = hip(ad, 0)
    assert np.abs(host(c0) - fo.prefill_compress(a, N, fo.compress_period(T))).max() < 2e-4
    row = fo.rnd(rng.standard_normal((B, 1, M)).astype(np.float32), "fp16")
    c1 = hip(c0, 80, slice_input=dev(row, "fp16"))
    want = fo.evict_update(host(c0), row, 80, fo.compress_period(T), "km57")
    assert np.abs(host(c1) - want).max() < 1e-5
    with pytest.raises(AssertionError):
        km.mat_fourier_triton(ad.transpose(1, 2), N, T)
