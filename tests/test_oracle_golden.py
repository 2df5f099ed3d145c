"""Pins the CPU oracle to outputs of the reference's own code (tests/golden/*.npz)."""
import numpy as np
import pytest

from oracle import fourier_oracle as fo
from tests.helpers import GOLDEN_CASES, attn_err_excess, case_inputs, input_digest, load_golden


def _run_oracle(g, tables, k, v):
    cache = fo.OracleCache([fo.DimTables(tables["Layer_0"])], g["S"], g["W"], g["M"], g["steps"],
                           g["mpe"], g["dtype"])
    P = g["P"]
    kd, vd = cache.update(k[:, :, :P], v[:, :, :P], 0)
    return cache, kd, vd


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_inputs_reproduce(name):
    z, g = load_golden(name)
    _, k, v, qs = case_inputs(g)
    assert np.array_equal(input_digest(k, v, qs), z["input_sha256"])


@pytest.mark.parametrize("name", [c for c in GOLDEN_CASES if c != "short_fp16"])
def test_prefill_state(name):
    z, g = load_golden(name)
    tables, k, v, qs = case_inputs(g)
    cache, kd, vd = _run_oracle(g, tables, k, v)
    assert kd["k_init"] is None and kd["k_compressed"] is None and kd["k_uncompressed"] is None
    assert kd["k_local"].shape[1] == g["P"]
    assert cache.maxtokens == int(z["maxtokens"])
    assert cache.curr_tokennum[0] == int(z["curr_tokennum_prefill"])
    kc, vc = cache.key_cache[0], cache.value_cache[0]
    # verbatim parts: bit exact
    assert np.array_equal(kc["k_uncompressed"], z["pre_k_uncompressed"])
    assert np.array_equal(vc["v_uncompressed"], z["pre_v_uncompressed"])
    # coefficients: the reference computes them with a complex64 FFT
    for mine, ref in ((kc["k_compressed"], z["pre_k_compressed"]), (vc["v_compressed"], z["pre_v_compressed"])):
        assert mine.shape == ref.shape and mine.dtype == np.float32
        assert np.abs(mine - ref).max() <= 2e-6 * max(1.0, np.abs(ref).max()) + 1e-5
    # statistics (fp16 / model dtype grids): allow one unit in the last place
    for nm, mine in (("k_layer_average", cache.k_layer_average[0]), ("kd_layer_average", cache.kd_layer_average[0]),
                     ("v_layer_average", cache.v_layer_average[0]), ("vd_layer_average", cache.vd_layer_average[0]),
                     ("k_scale", cache.k_scale[0]), ("v_scale", cache.v_scale[0])):
        ref = z[nm]
        ulp = 2.0 ** -7 if (g["dtype"] == "bf16" and nm in ("k_layer_average", "v_layer_average")) else 2.0 ** -10
        assert np.all(np.abs(mine - ref) <= ulp * np.maximum(np.abs(ref), 2.0 ** -14) + 1e-7), nm


@pytest.mark.parametrize("name", [c for c in GOLDEN_CASES if c != "short_fp16"])
def test_decode_steps(name):
    z, g = load_golden(name)
    tables, k, v, qs = case_inputs(g)
    cache, _, _ = _run_oracle(g, tables, k, v)
    # take the reference's statistics so that one-ulp flips in them do not leak into the
    # attention comparison (they are checked separately above)
    for nm in ("k_scale", "v_scale", "k_layer_average", "v_layer_average", "kd_layer_average", "vd_layer_average"):
        getattr(cache, nm)[0] = z[nm]
    P = g["P"]
    for s in range(g["steps"]):
        kd, vd = cache.update(k[:, :, P + s:P + s + 1], v[:, :, P + s:P + s + 1], 0)
        assert cache.get_seq_length(0) == int(z[f"seq_len_{s}"])
        assert kd["k_init"] is not None
        o = cache.attend(qs[s], 0, g["Hq"], g["Hkv"], faithful=True)
        ref = z[f"attn_{s}"]
        assert o.shape == ref.shape
        assert np.abs(o - ref).max() <= 2.0 ** -10 * max(1.0, np.abs(ref).max()), (s, np.abs(o - ref).max())
        # the un-rounded float64 evaluation stays inside the build's tolerance as well
        o64 = cache.attend(qs[s], 0, g["Hq"], g["Hkv"], faithful=False)
        assert attn_err_excess(o64, ref, g["dtype"]) <= 0, (s, np.abs(o64 - ref).max())
    kc, vc = cache.key_cache[0], cache.value_cache[0]
    assert cache.curr_tokennum[0] == int(z["curr_tokennum_final"])
    assert np.array_equal(kc["k_local"], z["fin_k_local"])
    assert np.array_equal(vc["v_local"], z["fin_v_local"])
    assert np.array_equal(kc["k_init"], z["fin_k_init"])
    assert np.array_equal(kc["k_uncompressed"][:, -g["steps"]:], z["fin_k_uncompressed_tail"])
    assert np.array_equal(vc["v_uncompressed"][:, -g["steps"]:], z["fin_v_uncompressed_tail"])
    for mine, ref in ((kc["k_compressed"], z["fin_k_compressed"]), (vc["v_compressed"], z["fin_v_compressed"])):
        assert np.abs(mine - ref).max() <= 3e-6 * max(1.0, np.abs(ref).max()) + 2e-5


def test_short_prompt_never_compresses():
    z, g = load_golden("short_fp16")
    tables, k, v, qs = case_inputs(g)
    cache, kd, vd = _run_oracle(g, tables, k, v)
    P = g["P"]
    for s in range(g["steps"]):
        kd, vd = cache.update(k[:, :, P + s:P + s + 1], v[:, :, P + s:P + s + 1], 0)
        assert kd["k_init"] is None and kd["k_compressed"] is None
        assert kd["k_local"].shape[1] == int(z[f"local_len_{s}"])
        assert cache.get_seq_length(0) == int(z[f"seq_len_{s}"])


def test_periods():
    assert fo.compress_period(93) == 92
    assert fo.compress_period(31996) == 31995      # Llama-3.1-8B, 32k prompt + 256 new tokens
    assert fo.compress_period(7228) == 7228
    assert fo.attention_period(8256, 4, 1024) == 7228


@pytest.mark.parametrize("name", ["toy_fp16_ragged", "small_bf16_tc", "mid_bf16_ragged"])
def test_reassociated_equals_rebuild(name):
    """Moving the spectral contraction onto the query side is exact algebra (float64)."""
    z, g = load_golden(name)
    tables, k, v, qs = case_inputs(g)
    cache, _, _ = _run_oracle(g, tables, k, v)
    P = g["P"]
    kd, vd = cache.update(k[:, :, P:P + 1], v[:, :, P:P + 1], 0)
    tb = cache.tables[0]
    k_il = np.concatenate([kd["k_init"], kd["k_local"]], 1)
    v_il = np.concatenate([vd["v_init"], vd["v_local"]], 1)
    args = (qs[0], k_il, v_il, kd["k_compressed"], vd["v_compressed"], kd["k_uncompressed"], vd["v_uncompressed"],
            cache.k_layer_average[0], cache.kd_layer_average[0], cache.k_scale[0],
            cache.v_layer_average[0], cache.vd_layer_average[0], cache.v_scale[0])
    a = fo.fourier_attn(*args, tb.kc, tb.kn, tb.vc, tb.vn, g["Hq"], g["Hkv"], cache.T, g["dtype"], faithful=False)
    b = fo.fourier_attn_reassociated(*args, tb.kc, tb.kc_h, tb.kn, tb.kn_h, tb.vc, tb.vc_h, tb.vn, tb.vn_h,
                                     g["Hq"], g["Hkv"], cache.T)
    assert np.abs(a - b).max() < 1e-11


def test_fft_identity():
    """First N bins of a length-T DFT equal the dense cosine / sine projection (float64)."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((1, 37, 5))
    T, N = 48, 6
    ref = np.fft.fft(np.concatenate([x, np.zeros((1, T - 37, 5))], 1), axis=1)[:, :N]
    c = fo.fourier_project(x, N, T)
    assert np.abs(c[:, :N] - ref.real).max() < 1e-5 and np.abs(c[:, N:] + ref.imag).max() < 1e-5


def test_merge_partials():
    rng = np.random.default_rng(1)
    s = rng.standard_normal((3, 40)) * 3
    v = rng.standard_normal((3, 40, 4))
    p = np.exp2(s - s.max(-1, keepdims=True))
    full = (p[..., None] * v).sum(1) / p.sum(-1, keepdims=True)
    ms, ls, os_ = [], [], []
    for lo, hi in ((0, 7), (7, 29), (29, 40)):
        m = s[:, lo:hi].max(-1)
        pp = np.exp2(s[:, lo:hi] - m[:, None])
        ms.append(m); ls.append(pp.sum(-1)); os_.append((pp[..., None] * v[:, lo:hi]).sum(1))
    got = fo.merge_partials(np.stack(ms, -1), np.stack(ls, -1), np.stack(os_, -2))
    assert np.abs(got - full).max() < 1e-12
