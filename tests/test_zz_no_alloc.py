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
from tests.test_gpu_kernels import DECODE_CASES, _state

pytestmark = pytest.mark.gpu


def _both(name):
    import fourierattention_b200.ops as ops
    g = DECODE_CASES[name]
    oc, q = _state(g)
    inp = decode_inputs_from_oracle(oc, g["dtype"])
    kw = dict(num_head_q=g["Hq"], num_head_kv=g["Hkv"], T=oc.T, return_lse=True, **inp)
    want = ops.decode_attn(dev(q, g["dtype"]), **kw)
    got = ops.decode_attn(dev(q, g["dtype"]), static_scratch=True, **kw)
    torch.cuda.synchronize()
    return want, got


def test_static_scratch_matches_on_two_calls_in_a_row():
    for name in ("wide", "gqa3_bf16", "wide"):
        want, got = _both(name)
        for w, g_ in zip(want, got):
            assert np.abs(host(w) - host(g_)).max() <= 2e-6, name


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
