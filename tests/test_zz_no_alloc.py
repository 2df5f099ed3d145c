"""fa_decode_attn_static: decode attention for hosts that cannot allocate device memory.

Some hosts of this library give every byte of HBM to their own allocator when they start (inference servers
with paged KV memory do) or call it from places where a cudaMalloc is off limits, so they cannot supply
the scratch buffer ``fa_decode_attn`` wants.  ``fa_decode_attn_static`` uses a fixed 24 MiB buffer inside
the library instead.  These checks call it through the C ABI, twice in a row on different problems (the
buffer keeps the previous call's contents and must not care), and compare with the ordinary entry point.
The file name sorts last on purpose, so a run that stops at the first failure has already run the rest.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.gpu_util import decode_inputs_from_oracle, dev, host
from tests.test_gpu_kernels import DECODE_CASES, FAST_CASES, _state

pytestmark = pytest.mark.gpu


def _both(name):
    import fourierattention_b200.ops as ops
    g = DECODE_CASES[name] if name in DECODE_CASES else FAST_CASES[name]
    oc, q = _state(g)
    inp = decode_inputs_from_oracle(oc, g["dtype"])
    kw = dict(num_head_q=g["Hq"], num_head_kv=g["Hkv"], T=oc.T, return_lse=True, **inp)
    want = ops.decode_attn(dev(q, g["dtype"]), **kw)
    got = ops.decode_attn(dev(q, g["dtype"]), static_scratch=True, **kw)
    path = ops.last_decode_path
    torch.cuda.synchronize()
    ideal = oc.attend(q, 0, g["Hq"], g["Hkv"], faithful=False)[:, :, 0]
    return want, got, path, ideal


def test_static_scratch_matches_on_two_calls_in_a_row():
    """The comparison is with the ordinary entry point, which the other test files hold to the oracle on
    these same cases; the float64 oracle result is checked here as well, loosely, so that this file also
    stands on its own."""
    for name in ("wide", "gqa3_bf16", "wide"):
        want, got, path, ideal = _both(name)
        assert path == 0
        for w, g_ in zip(want, got):
            assert np.abs(host(w) - host(g_)).max() <= 2e-6, name
        assert np.abs(host(got[0]) - ideal).max() <= 3e-5 * max(1.0, np.abs(ideal).max())


def test_static_scratch_on_the_tensor_core_passes_with_changing_plans():
    """The shared buffer keeps whatever the previous call left in it, and consecutive calls here have
    different chunk counts, batch sizes and sequences per CTA (a warp-specialised plan with the accumulator in
    tensor memory, an exact-kernel plan, such a plan that packs four sequences per CTA with a batch of five, a
    64-token super-tile plan, a warp-specialised plan with six-head column tiles and the accumulator in
    registers): every word a call reads must have been written by that same call."""
    seen = set()
    for name in ("fast_32heads_fp16", "wide", "fast_packed_4seq", "fast_gqa3_half_tiles", "fast_packed_2seq",
                 "gqa3_bf16", "fast_llama8b_layer", "fast_gqa3_six_head_tiles", "fast_packed_4seq"):
        want, got, path, ideal = _both(name)
        seen.add(path)
        for w, g_ in zip(want, got):
            assert np.abs(host(w) - host(g_)).max() <= 2e-6, name
        assert np.abs(host(got[0]) - ideal).max() <= 1.5e-4 * max(1.0, np.abs(ideal).max()), name
    assert seen == {0, 1, 2, 3}, seen


def test_static_scratch_allocates_nothing_and_rejects_oversize():
    import fourierattention_b200.ops as ops
    from fourierattention_b200 import _lib
    g = DECODE_CASES["tiny"]
    oc, q = _state(g)
    inp = decode_inputs_from_oracle(oc, g["dtype"])
    qd = dev(q, g["dtype"])
    out = torch.empty((g["B"], g["Hq"], g["D"]), dtype=torch.float32, device="cuda")
    ops.decode_attn(qd, num_head_q=g["Hq"], num_head_kv=g["Hkv"], T=oc.T, out=out, static_scratch=True, **inp)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free0, _ = torch.cuda.mem_get_info()
    ops.decode_attn(qd, num_head_q=g["Hq"], num_head_kv=g["Hkv"], T=oc.T, out=out, static_scratch=True, **inp)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == before and free1 == free0
    # a plan far beyond the built-in buffer is refused before anything is launched
    a = _lib.DecodeArgs()
    for k, v in dict(B=1, Hq=32, Hkv=8, D=128, n_sink=4, n_win=2048, n_mid=500000, N=512, T=524288, Mc_k=768,
                     Mn_k=256, Mc_v=768, Mn_v=256, dtype=1, sm_scale=-1.0, k_mn_sk=256, v_mn_sk=256).items():
        setattr(a, k, v)
    assert _lib.lib.fa_decode_scratch_bytes(C.byref(a)) > _lib.FA_DECODE_STATIC_SCRATCH_BYTES
    assert _lib.lib.fa_decode_attn_static(C.byref(a), None) == -5
    assert b"built-in buffer" in _lib.lib.fa_last_error_string()
