"""CPU checks of the C ABI: the library loads, exports every declared symbol, the ctypes mirror of the
argument block matches the C layout, and argument validation / planning work without a GPU."""
import ctypes as C
import os
import re
import subprocess
import sys
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fourier_b200.h")


@pytest.fixture(scope="module")
def L():
    sys.path.insert(0, ROOT)
    import __graft_entry__
    __graft_entry__._load_builder().build()
    from fourierattention_b200 import _lib
    return _lib


def test_every_declared_symbol_is_exported(L):
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b(fa_[a-z0-9_]+)\s*\(", text))
    assert declared and declared == set(L.EXPORTS)
    for name in declared:
        assert hasattr(L.lib, name), name
    assert L.lib.fa_version() >= 100


@pytest.mark.parametrize("ctype,pytype", [("fa_decode_args_t", "DecodeArgs"), ("fa_layer_desc_t", "LayerDesc")])
def test_argument_block_layout_matches_c(L, ctype, pytype):
    mirror = getattr(L, pytype)
    fields = [f[0] for f in mirror._fields_]
    prog = '#include <stdio.h>\n#include <stddef.h>\n#include "fourier_b200.h"\nint main(){printf("%zu\\n", sizeof(' + ctype + '));\n'
    for f in fields:
        prog += f'printf("%zu\\n", offsetof({ctype}, {f}));\n'
    prog += "return 0;}\n"
    with tempfile.TemporaryDirectory() as d:
        src, exe = os.path.join(d, "t.c"), os.path.join(d, "t")
        open(src, "w").write(prog)
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), src, "-o", exe])
        vals = [int(x) for x in subprocess.check_output([exe]).split()]
    assert vals[0] == C.sizeof(mirror)
    for f, off in zip(fields, vals[1:]):
        assert getattr(mirror, f).offset == off, f


def _args(L, **kw):
    a = L.DecodeArgs()
    d = dict(B=8, Hq=32, Hkv=8, D=128, n_sink=4, n_win=1024, n_mid=31740, N=256, T=31996, Mc_k=768, Mn_k=256,
             Mc_v=768, Mn_v=256, dtype=1, sm_scale=-1.0, k_mn_sk=256, v_mn_sk=256)
    d.update(kw)
    for k, v in d.items():
        setattr(a, k, v)
    return a


@pytest.mark.parametrize("kw", [
    dict(),                                                                      # Llama-3.1-8B, 32k, M=512
    dict(B=1, n_mid=7164, N=128, T=7228, dtype=0),                               # single layer, 8k, M=256
    dict(B=32, Hq=24, n_win=512, n_mid=15868, N=128, T=16124, Mc_k=640, Mn_k=384, Mc_v=640, Mn_v=384,
         k_mn_sk=384, v_mn_sk=384),                                              # Llama-3.2-3B, 16k
    dict(B=1, n_win=2048, n_mid=524288 - 2052, N=512, T=524288),                 # long context, M=1024
    dict(B=8, Hq=4, Hkv=1, Mc_k=96, Mn_k=32, Mc_v=96, Mn_v=32, k_mn_sk=32, v_mn_sk=32),   # one KV head per GPU
])
def test_benchmark_shapes_have_a_plan(L, kw):
    a = _args(L, **kw)
    n = L.lib.fa_decode_scratch_bytes(C.byref(a))
    assert n > 0, L.lib.fa_last_error_string()
    assert n < (2 << 30)


def test_validation_without_a_gpu(L):
    a = _args(L, Hq=30)
    assert L.lib.fa_decode_scratch_bytes(C.byref(a)) == 0
    assert b"multiple of Hkv" in L.lib.fa_last_error_string()
    assert L.lib.fa_decode_attn(C.byref(_args(L, dtype=7)), None) == -3
    assert L.lib.fa_decode_attn(C.byref(_args(L, D=12)), None) == -4
    assert L.lib.fa_decode_attn(C.byref(_args(L, N=4096)), None) == -5
    assert L.lib.fa_decode_attn(C.byref(_args(L)), None) == -1            # null tensors
    assert L.lib.fa_decode_attn(None, None) == -1
    assert L.lib.fa_colstats(None, 0, 1, 1, 1, 1, None, 1, None, None, None) == -1
    assert L.lib.fa_colstats(None, 5, 1, 1, 1, 1, None, 1, None, None, None) == -3
    assert L.lib.fa_compress(None, 0, 1, 0, 1, 1, 1, None, 1, 1, 1, 0, None, 0, None, 0, None) == -2
    assert L.lib.fa_merge(None, None, None, 0, 1, 1, None, None) == -2
    with pytest.raises(ValueError):
        L.check(-2, "x")
    with pytest.raises(RuntimeError):
        L.check(-6, "x")


def test_scratch_size_queries(L):
    assert L.lib.fa_compress_scratch_bytes(1, 1, 128, 768, 1024) == 0
    assert L.lib.fa_compress_scratch_bytes(1, 31740, 256, 768, 1024) > 0
    assert L.lib.fa_recon_stats_scratch_bytes(8, 31740, 768) > 0


def test_layer_handle_validation_without_a_gpu(L):
    """fa_layer_create checks sizes and pointers on the host; the handle plans without touching a device."""
    h = C.c_void_p()
    d = L.LayerDesc()
    assert L.lib.fa_layer_create(C.byref(d), C.byref(h)) == -2
    assert L.lib.fa_layer_create(None, C.byref(h)) == -1
    for k, v in dict(B=8, Hkv=8, D=128, S=4, W=1024, N=256, T=31996, T_c=31995, angle_mode=1, dtype=1, Mc_k=768,
                     Mn_k=256, Mc_v=768, Mn_v=256, with_il=1, kbuf=4096, vbuf=8192, buf_sb=2052 * 1024, buf_rows=2052,
                     k_unc=4096, v_unc=4096, k_unc_sb=32004 * 256, v_unc_sb=32004 * 256, k_unc_sk=256, v_unc_sk=256,
                     unc_rows=32004).items():
        setattr(d, k, v)
    assert L.lib.fa_layer_create(C.byref(d), C.byref(h)) == 0 and h.value
    n0 = L.lib.fa_layer_scratch_bytes(h, 32, 31740)
    assert n0 > 0
    # the plan, and with it the scratch need, stays put while n_mid grows inside one 128-token super-tile
    assert all(L.lib.fa_layer_scratch_bytes(h, 32, n) == n0 for n in range(31617, 31745))
    assert L.lib.fa_layer_update(h, 1024, 31740, 31741, 1, None, None, 0, 0, None) == -2      # window offset out of range
    assert L.lib.fa_layer_update(h, 0, 32004, 31741, 1, None, None, 0, 0, None) == -5         # stores are full
    L.lib.fa_layer_destroy(h)
