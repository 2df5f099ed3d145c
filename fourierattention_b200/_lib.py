"""ctypes binding of ``libfourier_b200.so`` (the C ABI of ``include/fourier_b200.h``).

There is no fallback: if the library has not been built, importing this module raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libfourier_b200.so")

FA_DTYPE_F16, FA_DTYPE_BF16 = 0, 1
FA_ANGLE_EXACT, FA_ANGLE_KM57 = 0, 1
FA_DECODE_STATIC_SCRATCH_BYTES = 24 << 20

STATUS_NAMES = {0: "FA_OK", -1: "FA_ERR_NULL", -2: "FA_ERR_SHAPE", -3: "FA_ERR_DTYPE", -4: "FA_ERR_ALIGN",
                -5: "FA_ERR_CAPACITY", -6: "FA_ERR_CUDA", -7: "FA_ERR_UNSUPPORTED"}

# every symbol include/fourier_b200.h declares
EXPORTS = ["fa_version", "fa_last_error_string", "fa_gather_cols", "fa_colstats", "fa_compress_scratch_bytes",
           "fa_compress", "fa_evict_update", "fa_recon_stats_scratch_bytes", "fa_recon_stats", "fa_fourier_inverse",
           "fa_cache_step", "fa_evict_step", "fa_decode_scratch_bytes", "fa_decode_path", "fa_decode_attn", "fa_decode_attn_static", "fa_merge",
           "fa_layer_create", "fa_layer_destroy", "fa_layer_rebind_stores", "fa_layer_update", "fa_layer_scratch_bytes",
           "fa_layer_attend", "fa_layer_decode_path"]

i32, i64, vp, f32, sz = C.c_int32, C.c_int64, C.c_void_p, C.c_float, C.c_size_t


class DecodeArgs(C.Structure):
    """Mirror of ``fa_decode_args_t``."""
    _fields_ = [
        ("B", i32), ("Hq", i32), ("Hkv", i32), ("D", i32),
        ("n_sink", i32), ("n_win", i32), ("n_mid", i32), ("mid_l0", i32), ("N", i32), ("T", i32),
        ("Mc_k", i32), ("Mn_k", i32), ("Mc_v", i32), ("Mn_v", i32),
        ("dtype", i32), ("sm_scale", f32),
        ("q", vp), ("q_sb", i64),
        ("k_sink", vp), ("v_sink", vp), ("sink_sb", i64),
        ("k_win", vp), ("v_win", vp), ("win_sb", i64),
        ("k_mn", vp), ("v_mn", vp), ("k_mn_sb", i64), ("v_mn_sb", i64), ("k_mn_sk", i64), ("v_mn_sk", i64),
        ("k_coef", vp), ("v_coef", vp),
        ("avg_k_u", vp), ("avg_k_d", vp), ("scale_k", vp),
        ("avg_v_u", vp), ("avg_v_d", vp), ("scale_v", vp),
        ("kc_list", vp), ("kc_h", vp), ("kn_list", vp), ("kn_h", vp),
        ("vc_list", vp), ("vc_h", vp), ("vn_list", vp), ("vn_h", vp),
        ("out", vp), ("m_out", vp), ("l_out", vp),
        ("scratch", vp), ("scratch_bytes", sz),
        ("phase_events_host", vp),
        ("kn_h_host", vp), ("vn_h_host", vp),
    ]


class LayerDesc(C.Structure):
    """Mirror of ``fa_layer_desc_t``."""
    _fields_ = [
        ("B", i32), ("Hkv", i32), ("D", i32), ("S", i32), ("W", i32), ("N", i32), ("T", i32), ("T_c", i32),
        ("angle_mode", i32), ("dtype", i32), ("mid_l0", i32),
        ("Mc_k", i32), ("Mn_k", i32), ("Mc_v", i32), ("Mn_v", i32),
        ("with_il", i32),
        ("kbuf", vp), ("vbuf", vp), ("buf_sb", i64), ("buf_rows", i32),
        ("k_unc", vp), ("v_unc", vp), ("k_unc_sb", i64), ("v_unc_sb", i64), ("k_unc_sk", i64), ("v_unc_sk", i64),
        ("unc_rows", i32),
        ("k_coef", vp), ("v_coef", vp),
        ("avg_k_u", vp), ("avg_k_d", vp), ("scale_k", vp), ("avg_v_u", vp), ("avg_v_d", vp), ("scale_v", vp),
        ("kc_list", vp), ("kc_h", vp), ("kn_list", vp), ("kn_h", vp),
        ("vc_list", vp), ("vc_h", vp), ("vn_list", vp), ("vn_h", vp),
        ("kn_h_host", vp), ("vn_h_host", vp),
    ]


def _load():
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python fourierattention_b200/build.py` "
            "(nvcc, sm_100a).  This package has no fallback path.")
    lib = C.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(lib, name):
            raise RuntimeError(f"{LIB_PATH} does not export {name}: it is stale, rebuild it with "
                               "`python fourierattention_b200/build.py`")
    lib.fa_version.restype = C.c_int
    lib.fa_last_error_string.restype = C.c_char_p
    lib.fa_gather_cols.argtypes = [vp, C.c_int, C.c_int, C.c_int, i64, i64, vp, C.c_int, vp, i64, i64, vp]
    lib.fa_colstats.argtypes = [vp, C.c_int, C.c_int, C.c_int, i64, i64, vp, C.c_int, vp, vp, vp]
    lib.fa_compress_scratch_bytes.argtypes = [C.c_int] * 5
    lib.fa_compress_scratch_bytes.restype = sz
    lib.fa_compress.argtypes = [vp, C.c_int, C.c_int, C.c_int, i64, i64, C.c_int, vp, C.c_int, C.c_int, C.c_int, i64, vp,
                                C.c_int, vp, sz, vp]
    lib.fa_evict_update.argtypes = [vp, vp, i64, vp, C.c_int, vp, vp, i64, vp, C.c_int, C.c_int, C.c_int, C.c_int,
                                    i64, C.c_int, C.c_int, vp]
    lib.fa_recon_stats_scratch_bytes.argtypes = [C.c_int] * 3
    lib.fa_recon_stats_scratch_bytes.restype = sz
    lib.fa_recon_stats.argtypes = [vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp, vp, sz, vp]
    lib.fa_fourier_inverse.argtypes = [vp, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp]
    lib.fa_cache_step.argtypes = [vp, vp, i64, vp, C.c_int, vp, C.c_int, vp, i64, vp, i64, vp, vp, i64, i64, vp, vp,
                                  i64, C.c_int, C.c_int, C.c_int, C.c_int, vp]
    lib.fa_evict_step.argtypes = [vp, vp, i64, vp, C.c_int, vp, vp, i64, vp, C.c_int, C.c_int, i64, C.c_int, C.c_int,
                                  vp, vp, i64, vp, C.c_int, vp, C.c_int, vp, i64, vp, i64, vp, vp, i64, i64, vp, vp,
                                  i64, C.c_int, C.c_int, C.c_int, C.c_int, vp]
    lib.fa_decode_scratch_bytes.argtypes = [C.POINTER(DecodeArgs)]
    lib.fa_decode_scratch_bytes.restype = sz
    lib.fa_decode_path.argtypes = [C.POINTER(DecodeArgs)]
    lib.fa_decode_attn.argtypes = [C.POINTER(DecodeArgs), vp]
    lib.fa_decode_attn_static.argtypes = [C.POINTER(DecodeArgs), vp]
    lib.fa_merge.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_int, vp, vp]
    lib.fa_layer_create.argtypes = [C.POINTER(LayerDesc), C.POINTER(vp)]
    lib.fa_layer_destroy.argtypes = [vp]
    lib.fa_layer_destroy.restype = None
    lib.fa_layer_rebind_stores.argtypes = [vp, vp, vp, i64, i64, i64, i64, i32]
    lib.fa_layer_update.argtypes = [vp, i32, i32, i64, i32, vp, vp, i64, i64, vp]
    lib.fa_layer_scratch_bytes.argtypes = [vp, i32, i32]
    lib.fa_layer_scratch_bytes.restype = sz
    lib.fa_layer_attend.argtypes = [vp, i32, i32, i32, vp, i64, f32, vp, vp, vp, vp, sz, vp, vp]
    lib.fa_layer_decode_path.argtypes = [vp]
    for name in EXPORTS:
        f = getattr(lib, name)
        if f.restype is C.c_int and name != "fa_version":
            pass
    return lib


lib = _load()


def check(rc, what):
    """Turn a negative status into the Python exception the reference would raise."""
    if rc == 0:
        return
    msg = lib.fa_last_error_string().decode("utf-8", "replace")
    name = STATUS_NAMES.get(rc, str(rc))
    if rc in (-2, -3, -4, -7):
        raise ValueError(f"{what}: {name}: {msg}")
    raise RuntimeError(f"{what}: {name}: {msg}")
