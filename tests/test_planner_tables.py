"""Which decode pass the planner picks for the dim tables the reference ships (CPU only: ``fa_decode_path``
reads sizes and the host copies of the per-head offset tables, nothing runs on a device).

The fixture holds the cumulative per-head counts of every ``_splithead`` table under the reference's
``compressed_dims_file/`` (written by ``tests/golden/make_shipped_offsets.py``).  The warp-specialised
tensor-core pass takes a layer when every column tile of 8 (or 6) query heads finds at most 128 verbatim K and
128 verbatim V columns; layers that keep more dims verbatim than that (the last eight layers of the shipped
tables keep 50 %) fall back to the general kernels.  The counts below are what the planner delivers today;
the test keeps them from shrinking unnoticed.
"""
import ctypes as C
import json
import os

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def L():
    from fourierattention_b200 import _lib
    return _lib


def _paths(L, layers, Hq, M, ctx):
    out = []
    for e in layers:
        knh, vnh = [0] + e["kn_h_list"], [0] + e["vn_h_list"]
        a = L.DecodeArgs()
        Mn_k, Mn_v = knh[-1], vnh[-1]
        for k, v in dict(B=1, Hq=Hq, Hkv=8, D=128, n_sink=4, n_win=1020, n_mid=ctx - 1024, N=M // 2, T=ctx + 256 - 1024,
                         Mc_k=1024 - Mn_k, Mn_k=Mn_k, Mc_v=1024 - Mn_v, Mn_v=Mn_v, dtype=1, sm_scale=-1.0,
                         k_mn_sk=(Mn_k + 7) // 8 * 8, v_mn_sk=(Mn_v + 7) // 8 * 8).items():
            setattr(a, k, v)
        kh, vh = (C.c_int32 * 9)(*knh), (C.c_int32 * 9)(*vnh)
        a.kn_h_host, a.vn_h_host = C.cast(kh, C.c_void_p), C.cast(vh, C.c_void_p)
        out.append(L.lib.fa_decode_path(C.byref(a)))
    return out


def test_shipped_tables_reach_the_tensor_core_passes(L):
    with open(os.path.join(HERE, "golden", "shipped_table_offsets.json")) as f:
        tables = json.load(f)
    assert len(tables) == 8
    fast_layers = total = wide_layers = 0
    for name, layers in tables.items():
        Hq = 32 if "8b" in name else 24
        p512 = _paths(L, layers, Hq, 512, 32768)
        assert all(p in (0, 1, 2, 3) for p in p512)
        fast_layers += sum(p in (1, 2, 3) for p in p512)
        total += len(p512)
        # M = 1024 needs a context long enough that the top frequency turns at most 1.5 times per 128-token
        # super-tile (T >= 43605); at 64k most layers the M = 512 plan takes are taken again (the single, larger
        # node-basis buffer leaves less shared memory for wide verbatim rows)
        p1024 = _paths(L, layers, Hq, 1024, 65536)
        assert all(a in (2, 3) for a, b in zip(p512, p1024) if b == 2), name
        wide_layers += sum(p == 2 for p in p1024)
    # 22 of 32 layers of the Llama-3.1-8B table and 15 to 20 of 28 of each Llama-3.2-3B table take the
    # warp-specialised pass, a few more the phase-by-phase pass
    assert fast_layers >= 170 and total == 228 and wide_layers >= 100, (fast_layers, total, wide_layers)
    p8b = _paths(L, tables["llama3.1-8b-fourier/compressed_dims_32k_1024states_splithead.json"], 32, 512, 32768)
    assert sum(p in (2, 3) for p in p8b) >= 22
    # ... those whose column tiles of 8 heads find at most 64 verbatim K and V columns with the spectral accumulator
    # in tensor memory (4 layers of this table; a uniform 96-of-128 split, as the benchmark uses, always does)
    assert sum(p == 3 for p in p8b) >= 4, p8b
