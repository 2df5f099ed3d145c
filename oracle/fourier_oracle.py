"""CPU oracle for the Fourier-compressed KV-cache hot path.  TEST INFRASTRUCTURE ONLY.

This module is a numpy restatement of the reference algorithm (FourierAttention's
``fourier_attn_triton`` package).  It exists to check the CUDA kernels; it is never
imported by the shipped package.  Only the test-suite, the smoke check and the CPU
baseline leg of the benchmark may call it.

Parity status: PINNED.  ``tests/golden/*.npz`` hold outputs of the reference's own
Python code executed on CPU (generator: ``tests/golden/make_golden.py``);
``tests/test_oracle_golden.py`` checks every function below against them.

Reference files are cited as ``KM`` = fourier_attn_triton/fourier_triton_valid4_v2.py,
``CU`` = fourier_attn_triton/cache_utils_fourier.py, ``ML`` =
fourier_attn_triton/modeling_llama_fourier.py.

Conventions
-----------
* Tensors are numpy arrays.  A "model dtype" tensor (fp16 or bf16) is carried as a
  float32 array whose values are exactly representable in that dtype; ``rnd`` rounds
  (nearest-even) onto the grid.  ``dtype`` arguments are the strings "fp16"/"bf16".
* Coefficients are float32, shape (B, 2N, Mc): rows 0..N-1 cosine, N..2N-1 sine
  (KM:68-78, KM:865).
"""
from __future__ import annotations

import json
import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

# --------------------------------------------------------------------------------------
# dtype helpers
# --------------------------------------------------------------------------------------

def to_bf16(x: np.ndarray) -> np.ndarray:
    """Round float32 values to the bfloat16 grid (nearest-even); result stays float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    nan = np.isnan(x)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    r = (u + np.uint32(0x7FFF) + lsb) & np.uint32(0xFFFF0000)
    out = r.view(np.float32).copy()
    out[nan] = np.nan
    return out


def rnd(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round onto the value grid of ``dtype`` ("fp16", "bf16", "fp32"); returns float32."""
    if dtype == "fp16":
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        return to_bf16(np.asarray(x, dtype=np.float32))
    if dtype == "fp32":
        return np.asarray(x, dtype=np.float32)
    raise ValueError(f"unknown dtype {dtype!r}")


# --------------------------------------------------------------------------------------
# periods (CU:547, KM:856, KM:859)
# --------------------------------------------------------------------------------------

def attention_period(maxtokens: int, numinittokens: int, maxlocallen: int) -> int:
    """T handed to the attention kernel and the reconstruction statistics (ML:660, CU:566)."""
    return int(maxtokens) - int(numinittokens) - int(maxlocallen)


def compress_period(T: int) -> int:
    """Period used by the forward projection.

    The cache builds the compressor with ``dt = 1/T`` (CU:547) and the compressor uses
    ``int(1/dt)`` (KM:856, KM:859).  In IEEE double this is T-1 for some T.
    """
    return int(1.0 / (1.0 / float(T)))


# --------------------------------------------------------------------------------------
# forward projection  (KM:57-62 decode form, KM:857-865 prefill form)
# --------------------------------------------------------------------------------------

def _basis_exact(pos: np.ndarray, N: int, T: int) -> Tuple[np.ndarray, np.ndarray]:
    """cos/sin(2*pi*pos*n/T) with the phase reduced modulo T in integers (float64 out)."""
    n = np.arange(N, dtype=np.int64)
    ph = (pos.astype(np.int64)[:, None] * n[None, :]) % int(T)
    ang = (2.0 * np.pi / float(T)) * ph.astype(np.float64)
    return np.cos(ang), np.sin(ang)


def _basis_km57(pos: np.ndarray, N: int, T: int) -> Tuple[np.ndarray, np.ndarray]:
    """The angle exactly as the reference's projection kernel rounds it (KM:57).

    angle = fl32(fl32(fl32(c * pos) * n) / T), c = fl32(2 * 3.14159265359); cos/sin of the
    float32 angle.
    """
    c = np.float32(2.0 * 3.14159265359)
    p = pos.astype(np.float32)
    n = np.arange(N, dtype=np.float32)
    a = (c * p).astype(np.float32)
    a = (a[:, None] * n[None, :]).astype(np.float32)
    a = (a / np.float32(T)).astype(np.float32)
    return np.cos(a).astype(np.float64), np.sin(a).astype(np.float64)


def fourier_project(x: np.ndarray, N: int, T_c: int, k_start: int = 0,
                    angle: str = "exact") -> np.ndarray:
    """C[b,n,m] = sum_k x[b,k,m] cos(2 pi (k+k_start) n / T_c); rows N.. hold the sine sums.

    ``x`` (B, K, Mc) -> float32 (B, 2N, Mc).  Accumulates in float64.
    ``angle="exact"`` is the mathematical definition (and what the prefill FFT, KM:858-865,
    delivers up to float32 rounding); ``angle="km57"`` reproduces the float32 angle of the
    decode-time kernel (KM:57).
    """
    x = np.asarray(x)
    B, K, Mc = x.shape
    pos = np.arange(K, dtype=np.int64) + int(k_start)
    fc, fs = (_basis_exact if angle == "exact" else _basis_km57)(pos, N, T_c)
    out = np.empty((B, 2 * N, Mc), dtype=np.float32)
    xd = x.astype(np.float64)
    for b in range(B):
        out[b, :N] = (fc.T @ xd[b]).astype(np.float32)
        out[b, N:] = (fs.T @ xd[b]).astype(np.float32)
    return out


def prefill_compress(x: np.ndarray, N: int, T_c: int) -> np.ndarray:
    """Prefill compression: first N bins of a length-T_c DFT (KM:858-865).

    ``torch.fft.fft(x, n=T_c)`` zero-pads a shorter span and *truncates* a longer one, so
    rows beyond T_c are dropped here as well.
    """
    x = np.asarray(x)
    if x.shape[1] > T_c:
        x = x[:, :T_c]
    return fourier_project(x, N, T_c, 0, "exact")


def evict_update(coef: np.ndarray, row: np.ndarray, phase: int, T_c: int,
                 angle: str = "km57") -> np.ndarray:
    """Decode-time rank-1 update  C + project(row, k_start=phase)  (KM:855-856, CU:733)."""
    N = coef.shape[1] // 2
    inc = fourier_project(row, N, T_c, phase, angle)
    return (coef.astype(np.float32) + inc).astype(np.float32)


# --------------------------------------------------------------------------------------
# reconstruction (KM:782-791) and statistics (KM:417-420, KM:461, KM:256-265, KM:319-326)
# --------------------------------------------------------------------------------------

def fourier_reconstruct(coef: np.ndarray, K: int, T: int, faithful: bool = True) -> np.ndarray:
    """x_hat[b,l,m] = (1/N) sum_n [C[b,n,m] cos(2 pi l n/T) + C[b,N+n,m] sin(2 pi l n/T)].

    ``faithful`` follows KM:784-791: float32 angle ``(l*n)*2*pi/T`` and a float32 contraction.
    Otherwise exact integer phases and float64.
    """
    coef = np.asarray(coef)
    B, N2, Mc = coef.shape
    N = N2 // 2
    if faithful:
        l = np.arange(K, dtype=np.float32)
        n = np.arange(N, dtype=np.float32)
        a = (l[:, None] * n[None, :]).astype(np.float32)
        a = (a * np.float32(2)).astype(np.float32)
        a = (a * np.float32(np.pi)).astype(np.float32)
        a = (a / np.float32(T)).astype(np.float32)
        basis = np.concatenate([np.cos(a), np.sin(a)], axis=-1).astype(np.float32)  # (K, 2N)
        out = np.empty((B, K, Mc), dtype=np.float32)
        c32 = coef.astype(np.float32)
        for b in range(B):
            out[b] = (basis @ c32[b]) / np.float32(N)
        return out
    fc, fs = _basis_exact(np.arange(K), N, T)
    basis = np.concatenate([fc, fs], axis=-1)
    out = np.empty((B, K, Mc), dtype=np.float64)
    cd = coef.astype(np.float64)
    for b in range(B):
        out[b] = (basis @ cd[b]) / float(N)
    return out


def col_stats(a: np.ndarray, dtype: str) -> Tuple[np.ndarray, np.ndarray]:
    """Column mean and max one-sided deviation over axis 1, cast to the input dtype.

    Follows KM:417-420 (float32 accumulation) and the cast at KM:461.
    """
    a32 = np.asarray(a, dtype=np.float32)
    K = a32.shape[1]
    avg = (a32.astype(np.float64).sum(axis=1) / K).astype(np.float32)
    dev = np.maximum(a32.max(axis=1) - avg, avg - a32.min(axis=1)).astype(np.float32)
    return rnd(avg, dtype), rnd(dev, dtype)


def recon_stats(coef: np.ndarray, K: int, T: int) -> Tuple[np.ndarray, np.ndarray]:
    """Mean / max-deviation of the reconstructed span, returned as float16 (KM:319-326).

    The reference kernel forms the angle as fl32(fl32(fl32(2 pi / T) * k) * n) (KM:256); the
    difference to exact phases is far below the float16 output grid, so exact phases are used.
    """
    xh = fourier_reconstruct(coef, K, T, faithful=False)
    avg = xh.sum(axis=1) / K
    dev = np.maximum(xh.max(axis=1) - avg, avg - xh.min(axis=1))
    return rnd(avg, "fp16"), rnd(dev, "fp16")


def renorm_scale(u_dev: np.ndarray, i_dev: np.ndarray, dtype: str) -> np.ndarray:
    """scale = u_dev / i_dev (CU:567).  u_dev has the model dtype, i_dev is float16, so the
    quotient is float16 for fp16 models and float32 for bf16 models (type promotion)."""
    q = (np.asarray(u_dev, np.float32) / np.asarray(i_dev, np.float32)).astype(np.float32)
    return rnd(q, "fp16") if dtype == "fp16" else q


# --------------------------------------------------------------------------------------
# dense attention (stand-in for flash_attn_func with one query row; ML:633, KM:835)
# --------------------------------------------------------------------------------------

def dense_decode_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, Hq: int, Hkv: int,
                           sm_scale: float, wide: bool = False) -> np.ndarray:
    """softmax(q k^T * sm_scale) v for one query token with grouped KV heads.

    q (B, Hq*D), k/v (B, L, Hkv*D).  A single query with bottom-right causal alignment sees
    every key, so no mask.  Returns (B, Hq, D) in float32 (float64 if ``wide``).
    """
    ft = np.float64 if wide else np.float32
    B, L, F = k.shape
    D = F // Hkv
    R = Hq // Hkv
    qh = q.reshape(B, Hkv, R, D).astype(ft)
    kh = k.reshape(B, L, Hkv, D).astype(ft)
    vh = v.reshape(B, L, Hkv, D).astype(ft)
    out = np.empty((B, Hkv, R, D), dtype=ft)
    for b in range(B):
        for g in range(Hkv):
            s = (qh[b, g] @ kh[b, :, g].T) * ft(sm_scale)          # (R, L)
            s = s - s.max(axis=1, keepdims=True)
            p = np.exp(s)
            p = p / p.sum(axis=1, keepdims=True)
            out[b, g] = p @ vh[b, :, g]
    return out.reshape(B, Hq, D)


# --------------------------------------------------------------------------------------
# the reference PyTorch attention path (KM:794-837)
# --------------------------------------------------------------------------------------

def fourier_attn(q, k_il, v_il, k_mc, v_mc, k_mn, v_mn,
                 avg_k_u, avg_k_d, scale_k, avg_v_u, avg_v_d, scale_v,
                 kc_list, kn_list, vc_list, vn_list,
                 num_head_q: int, num_head_kv: int, T: int, dtype: str,
                 sm_scale: Optional[float] = None, faithful: bool = True) -> np.ndarray:
    """Rebuild-then-attend decode attention.

    ``faithful=True`` follows the reference line by line, including its roundings: float32
    reconstruction, renormalisation, cast of the rebuilt values to the model dtype when they
    are scattered into the dense tensor (KM:817-822), cast of q/k/v to float16 (KM:835),
    float16 output.  ``faithful=False`` evaluates the same mathematics in float64 with no
    intermediate rounding.  Returns (B, Hq, 1, D).
    """
    q = np.asarray(q, np.float32)
    B = q.shape[0]
    F = k_il.shape[2]
    D = q.shape[-1] // num_head_q
    n_mid = k_mn.shape[1]
    if sm_scale is None or sm_scale == -1:
        sm_scale = 1.0 / math.sqrt(D)
    kc_list = np.asarray(kc_list); kn_list = np.asarray(kn_list)
    vc_list = np.asarray(vc_list); vn_list = np.asarray(vn_list)
    ft = np.float32 if faithful else np.float64

    def rebuild(coef, avg_d, scale, avg_u, c_list, n_list, verbatim):
        md = fourier_reconstruct(coef, n_mid, T, faithful=faithful).astype(ft)
        md = (md - np.asarray(avg_d, ft)[:, None, :]) * np.asarray(scale, ft)[:, None, :] \
            + np.asarray(avg_u, ft)[:, None, :]
        full = np.zeros((B, n_mid, F), dtype=ft)
        full[..., c_list] = rnd(md, dtype) if faithful else md
        full[..., n_list] = np.asarray(verbatim, ft)
        return full

    k_m = rebuild(k_mc, avg_k_d, scale_k, avg_k_u, kc_list, kn_list, k_mn)
    v_m = rebuild(v_mc, avg_v_d, scale_v, avg_v_u, vc_list, vn_list, v_mn)
    k_all = np.concatenate([np.asarray(k_il, ft), k_m], axis=1)
    v_all = np.concatenate([np.asarray(v_il, ft), v_m], axis=1)
    if faithful:
        qq = rnd(q.reshape(B, -1), "fp16")
        k_all = rnd(k_all, "fp16")
        v_all = rnd(v_all, "fp16")
        o = dense_decode_attention(qq, k_all, v_all, num_head_q, num_head_kv, sm_scale)
        o = rnd(o, "fp16")
    else:
        o = dense_decode_attention(q.reshape(B, -1).astype(ft), k_all, v_all,
                                   num_head_q, num_head_kv, sm_scale, wide=True)
    return o.reshape(B, num_head_q, 1, D)


def fourier_attn_reassociated(q, k_il, v_il, k_mc, v_mc, k_mn, v_mn,
                              avg_k_u, avg_k_d, scale_k, avg_v_u, avg_v_d, scale_v,
                              kc_list, kc_h, kn_list, kn_h, vc_list, vc_h, vn_list, vn_h,
                              num_head_q: int, num_head_kv: int, T: int,
                              sm_scale: Optional[float] = None) -> np.ndarray:
    """The same attention with the spectral contraction moved onto the query side (float64).

    Scores of the compressed dims become ``(1/N) F w + const`` with ``w = C_k^T (scale_k*q_c)``,
    and the compressed-V output becomes ``scale_v*((1/N) C_v^T (F^T p) - avg_vd*P) + avg_vu*P``.
    This is the algebra the CUDA decode kernel evaluates; the test-suite checks that it equals
    ``fourier_attn(..., faithful=False)`` to float64 rounding.
    ``*_h`` are cumulative per-head offsets with a leading 0 (length Hkv+1).
    """
    f8 = np.float64
    q = np.asarray(q, f8)
    B = q.shape[0]
    D = q.shape[-1] // num_head_q
    R = num_head_q // num_head_kv
    n_mid = k_mn.shape[1]
    N = k_mc.shape[1] // 2
    if sm_scale is None or sm_scale == -1:
        sm_scale = 1.0 / math.sqrt(D)
    qh = q.reshape(B, num_head_q, D)
    fc, fs = _basis_exact(np.arange(n_mid), N, T)
    out = np.zeros((B, num_head_q, D), f8)
    kc_list = np.asarray(kc_list); kn_list = np.asarray(kn_list)
    vc_list = np.asarray(vc_list); vn_list = np.asarray(vn_list)
    for b in range(B):
        for h in range(num_head_q):
            g = h // R
            kc = slice(int(kc_h[g]), int(kc_h[g + 1])); kn = slice(int(kn_h[g]), int(kn_h[g + 1]))
            vc = slice(int(vc_h[g]), int(vc_h[g + 1])); vn = slice(int(vn_h[g]), int(vn_h[g + 1]))
            q_c = qh[b, h, kc_list[kc] - g * D]
            q_n = qh[b, h, kn_list[kn] - g * D]
            sk = np.asarray(scale_k, f8)[b, kc]
            w_cos = np.asarray(k_mc, f8)[b, :N, kc] @ (sk * q_c)
            w_sin = np.asarray(k_mc, f8)[b, N:, kc] @ (sk * q_c)
            const = np.dot(q_c, np.asarray(avg_k_u, f8)[b, kc] - np.asarray(avg_k_d, f8)[b, kc] * sk)
            s_mid = (fc @ w_cos + fs @ w_sin) / N + const + np.asarray(k_mn, f8)[b, :, kn] @ q_n
            s_il = np.asarray(k_il, f8)[b, :, g * D:(g + 1) * D] @ qh[b, h]
            s = np.concatenate([s_il, s_mid]) * sm_scale
            p = np.exp(s - s.max())
            n_il = s_il.shape[0]
            p_il, p_mid = p[:n_il], p[n_il:]
            o = p_il @ np.asarray(v_il, f8)[b, :, g * D:(g + 1) * D]
            P = p_mid.sum()
            g_cos = fc.T @ p_mid
            g_sin = fs.T @ p_mid
            sv = np.asarray(scale_v, f8)[b, vc]
            oc = sv * ((g_cos @ np.asarray(v_mc, f8)[b, :N, vc] + g_sin @ np.asarray(v_mc, f8)[b, N:, vc]) / N
                       - np.asarray(avg_v_d, f8)[b, vc] * P) + np.asarray(avg_v_u, f8)[b, vc] * P
            o[vc_list[vc] - g * D] += oc
            o[vn_list[vn] - g * D] += p_mid @ np.asarray(v_mn, f8)[b, :, vn]
            out[b, h] = o / p.sum()
    return out.reshape(B, num_head_q, 1, D)


def merge_partials(m: np.ndarray, l: np.ndarray, o: np.ndarray) -> np.ndarray:
    """Log-sum-exp merge of split-KV partials (KM:756-776), base 2.

    m, l: (..., P) running maxima (log2 domain) and denominators; o: (..., P, D) un-normalised
    numerators.  Parts with l <= 0 are ignored (KM:756)."""
    m = np.where(l > 0, m, -1e6)
    ms = m.max(axis=-1, keepdims=True)
    a = np.exp2(m - ms)
    return (o * a[..., None]).sum(axis=-2) / (l * a).sum(axis=-1, keepdims=True)


# --------------------------------------------------------------------------------------
# compressed-dims tables (CU:411-455)
# --------------------------------------------------------------------------------------

class DimTables:
    """Per-layer index sets of the ``_splithead`` JSON format (CU:433-455).

    ``kc``/``vc``: flat dims whose middle span is compressed (sorted), ``kn``/``vn``: the dims
    kept verbatim; ``*_h`` cumulative per-head counts with a leading zero (CU:449-452)."""

    def __init__(self, layer: Dict[str, Sequence[int]]):
        self.kc = np.asarray(layer["kc_list"], dtype=np.int64)
        self.kn = np.asarray(layer["kn_list"], dtype=np.int64)
        self.vc = np.asarray(layer["vc_list"], dtype=np.int64)
        self.vn = np.asarray(layer["vn_list"], dtype=np.int64)
        self.kc_h = np.asarray([0] + list(layer["kc_h_list"]), dtype=np.int64)
        self.kn_h = np.asarray([0] + list(layer["kn_h_list"]), dtype=np.int64)
        self.vc_h = np.asarray([0] + list(layer["vc_h_list"]), dtype=np.int64)
        self.vn_h = np.asarray([0] + list(layer["vn_h_list"]), dtype=np.int64)


def load_tables(path: str) -> List[DimTables]:
    with open(path, "r") as f:
        d = json.load(f)
    out = []
    for i in range(len(d)):
        key = f"Layer_{i}"
        if key not in d:
            raise ValueError(f"Layer index {i} not found in non-critical dimensions JSON file.")
        out.append(DimTables(d[key]))
    return out


def make_splithead_tables(num_layers: int, num_kv_heads: int, head_dim: int,
                          n_compressed: int, seed: int, upper_weight: float = 3.0,
                          ragged: bool = False) -> Dict[str, Dict[str, List[int]]]:
    """Seeded synthetic ``_splithead`` tables.

    Per layer and KV head, ``n_compressed`` of the ``head_dim`` dims are drawn without
    replacement; a dim in the upper half of the head is ``upper_weight`` times as likely as one
    in the lower half.  K and V sets are drawn independently.  With ``ragged`` the per-head
    count itself is drawn uniformly from 0..head_dim (first head 0, second head head_dim, so
    both extremes occur)."""
    rng = np.random.default_rng(seed)
    w = np.ones(head_dim)
    w[head_dim // 2:] = upper_weight
    w = w / w.sum()
    out: Dict[str, Dict[str, List[int]]] = {}
    for layer in range(num_layers):
        ent: Dict[str, List[int]] = {}
        for t in ("k", "v"):
            c_list: List[int] = []; n_list: List[int] = []; c_h: List[int] = []; n_h: List[int] = []
            for h in range(num_kv_heads):
                if ragged:
                    cnt = int(rng.integers(0, head_dim + 1))
                    if h == 0:
                        cnt = 0
                    elif h == 1:
                        cnt = head_dim
                else:
                    cnt = n_compressed
                sel = np.sort(rng.choice(head_dim, size=cnt, replace=False, p=w)) if cnt else np.zeros(0, np.int64)
                mask = np.zeros(head_dim, bool); mask[sel] = True
                c_list += [int(h * head_dim + i) for i in np.nonzero(mask)[0]]
                n_list += [int(h * head_dim + i) for i in np.nonzero(~mask)[0]]
                c_h.append(len(c_list)); n_h.append(len(n_list))
            ent[f"{t}c_list"] = c_list; ent[f"{t}n_list"] = n_list
            ent[f"{t}c_h_list"] = c_h; ent[f"{t}n_h_list"] = n_h
        out[f"Layer_{layer}"] = ent
    return out


# --------------------------------------------------------------------------------------
# the cache state machine (CU:389-464, CU:494-750)
# --------------------------------------------------------------------------------------

class OracleCache:
    """Restatement of ``DynamicCache.update`` (CU:494-750) on numpy arrays.

    Observable behaviour replicated: sink / middle / window split of a long prompt
    (CU:556-561), compression + statistics (CU:562-569), ``maxtokens`` clamp (CU:542), the
    two periods, the decode phase that is incremented before use (CU:732-733), statistics
    frozen at prefill, and the branch test that reads the batch size where the window length
    was meant (CU:680): after a compressed prefill the eviction branch is taken whenever
    ``S + 2N + n_mid + B + 1 > maxlen + 1``; otherwise the new token is appended to the window.
    """

    def __init__(self, tables: List[DimTables], numinittokens: int, maxlocallen: int,
                 maxmidstates: int, max_new_tokens: int, max_position_embeddings: int,
                 dtype: str, update_angle: str = "km57"):
        self.tables = tables
        self.S = int(numinittokens); self.W = int(maxlocallen); self.M = int(maxmidstates)
        self.maxlen = self.S + self.W + self.M                       # CU:398
        self.maxnewtokens = int(max_new_tokens)
        self.maxtokens = int(max_position_embeddings)                # CU:400
        self.dtype = dtype
        self.update_angle = update_angle
        L = len(tables)
        self.curr_tokennum = [0] * L
        self.key_cache: List[dict] = []
        self.value_cache: List[dict] = []
        self.k_scale: List = []; self.v_scale: List = []
        self.k_layer_average: List = []; self.v_layer_average: List = []
        self.kd_layer_average: List = []; self.vd_layer_average: List = []
        self._seen_tokens = 0

    @property
    def T(self) -> int:
        return attention_period(self.maxtokens, self.S, self.W)

    def _compress_side(self, x_mid, c_list, n_list):
        N = self.M // 2                                               # KM:854
        T = self.T
        unc = x_mid[:, :, n_list]
        toc = x_mid[:, :, c_list]
        coef = prefill_compress(toc, N, compress_period(T))           # CU:562
        u_avg, u_dev = col_stats(toc, self.dtype)                     # CU:564
        i_avg, i_dev = recon_stats(coef, toc.shape[1], T)             # CU:565-566
        return unc, coef, renorm_scale(u_dev, i_dev, self.dtype), u_avg, i_avg

    def update(self, key_states: np.ndarray, value_states: np.ndarray, layer_idx: int):
        """key/value_states: (B, Hkv, q, D) values on the model-dtype grid.  Returns the two
        dicts of CU:613 / CU:686 / CU:748."""
        B, H, q_len, D = key_states.shape
        if layer_idx == 0:
            self._seen_tokens += q_len
        k = np.ascontiguousarray(key_states.transpose(0, 2, 1, 3)).reshape(B, q_len, H * D)
        v = np.ascontiguousarray(value_states.transpose(0, 2, 1, 3)).reshape(B, q_len, H * D)
        tb = self.tables[layer_idx]
        none_k = {"k_init": None, "k_compressed": None, "k_uncompressed": None}
        none_v = {"v_init": None, "v_compressed": None, "v_uncompressed": None}
        if len(self.key_cache) <= layer_idx:
            if layer_idx == 0:
                self.prefilllen = q_len
                self.maxtokens = min(q_len + self.maxnewtokens, self.maxtokens)   # CU:542
            if len(self.key_cache) < layer_idx:
                # skipped layers: the reference's back-fill branch (CU:616-674) indexes statistic
                # lists that were never extended, so it cannot run; not restated.
                raise NotImplementedError("layers must be updated in order")
            if q_len > self.maxlen:                                               # CU:555
                S, W = self.S, self.W
                k_unc, k_coef, k_sc, k_ua, k_ia = self._compress_side(k[:, S:-W], tb.kc, tb.kn)
                v_unc, v_coef, v_sc, v_ua, v_ia = self._compress_side(v[:, S:-W], tb.vc, tb.vn)
                self.k_scale.append(k_sc); self.k_layer_average.append(k_ua); self.kd_layer_average.append(k_ia)
                self.v_scale.append(v_sc); self.v_layer_average.append(v_ua); self.vd_layer_average.append(v_ia)
                self.curr_tokennum[layer_idx] += q_len - S - W                     # CU:593
                self.key_cache.append({"k_init": k[:, :S], "k_compressed": k_coef,
                                       "k_uncompressed": k_unc, "k_local": k[:, -W:]})
                self.value_cache.append({"v_init": v[:, :S], "v_compressed": v_coef,
                                         "v_uncompressed": v_unc, "v_local": v[:, -W:]})
            else:                                                                  # CU:598-611
                self.key_cache.append({"k_init": np.zeros((B, 0, H * D), np.float32),
                                       "k_compressed": np.zeros((B, 0, len(tb.kc)), np.float32),
                                       "k_uncompressed": np.zeros((B, 0, len(tb.kn)), np.float32),
                                       "k_local": k})
                self.value_cache.append({"v_init": np.zeros((B, 0, H * D), np.float32),
                                         "v_compressed": np.zeros((B, 0, len(tb.vc)), np.float32),
                                         "v_uncompressed": np.zeros((B, 0, len(tb.vn)), np.float32),
                                         "v_local": v})
            return dict(none_k, k_local=k), dict(none_v, v_local=v)

        kc, vc = self.key_cache[layer_idx], self.value_cache[layer_idx]
        # CU:680 -- note k_local.size(0) is the batch size
        q_tot = kc["k_init"].shape[1] + kc["k_compressed"].shape[1] + kc["k_uncompressed"].shape[1] + B + 1
        if q_tot <= self.maxlen:                                                   # CU:681-686
            kc["k_local"] = np.concatenate([kc["k_local"], k], axis=1)
            vc["v_local"] = np.concatenate([vc["v_local"], v], axis=1)
            return dict(none_k, k_local=kc["k_local"]), dict(none_v, v_local=vc["v_local"])
        if q_tot == self.maxlen + 1:
            raise NotImplementedError("first-time compression during decode (CU:688-729) needs "
                                      "batch == maxlen and is not exercised")
        # steady state (CU:731-748)
        self.curr_tokennum[layer_idx] += 1
        ph = self.curr_tokennum[layer_idx]
        T_c = compress_period(self.T)
        old_k = kc["k_local"][:, 0:1]; old_v = vc["v_local"][:, 0:1]
        kc["k_compressed"] = evict_update(kc["k_compressed"], old_k[:, :, tb.kc], ph, T_c, self.update_angle)
        kc["k_uncompressed"] = np.concatenate([kc["k_uncompressed"], old_k[:, :, tb.kn]], axis=1)
        kc["k_local"] = np.concatenate([kc["k_local"], k], axis=1)[:, 1:]
        vc["v_compressed"] = evict_update(vc["v_compressed"], old_v[:, :, tb.vc], ph, T_c, self.update_angle)
        vc["v_uncompressed"] = np.concatenate([vc["v_uncompressed"], old_v[:, :, tb.vn]], axis=1)
        vc["v_local"] = np.concatenate([vc["v_local"], v], axis=1)[:, 1:]
        return dict(kc), dict(vc)

    def get_seq_length(self, layer_idx: int = 0) -> int:                          # CU:752-761
        if len(self.key_cache) <= layer_idx or not self.key_cache[layer_idx]:
            return 0
        c = self.key_cache[layer_idx]
        return c["k_init"].shape[1] + c["k_uncompressed"].shape[1] + c["k_local"].shape[1]

    def attend(self, q: np.ndarray, layer_idx: int, num_head_q: int, num_head_kv: int,
               faithful: bool = True) -> np.ndarray:
        """The Fourier branch of the attention forward (ML:641-660) on the cached state.
        q: (B, Hq*D).  Returns (B, Hq, 1, D)."""
        kc, vc = self.key_cache[layer_idx], self.value_cache[layer_idx]
        tb = self.tables[layer_idx]
        k_il = np.concatenate([kc["k_init"], kc["k_local"]], axis=1)
        v_il = np.concatenate([vc["v_init"], vc["v_local"]], axis=1)
        return fourier_attn(q, k_il, v_il, kc["k_compressed"], vc["v_compressed"],
                            kc["k_uncompressed"], vc["v_uncompressed"],
                            self.k_layer_average[layer_idx], self.kd_layer_average[layer_idx],
                            self.k_scale[layer_idx], self.v_layer_average[layer_idx],
                            self.vd_layer_average[layer_idx], self.v_scale[layer_idx],
                            tb.kc, tb.kn, tb.vc, tb.vn, num_head_q, num_head_kv, self.T,
                            self.dtype, faithful=faithful)


# --------------------------------------------------------------------------------------
# seeded synthetic inputs (shapes of the benchmark configurations)
# --------------------------------------------------------------------------------------

def rope_rotate(x: np.ndarray, positions: np.ndarray, theta: float = 500000.0) -> np.ndarray:
    """Plain rotary embedding, half-split convention (ML:213-244).  x: (B, H, L, D)."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (np.arange(0, D, 2, dtype=np.float64) / D))
    ang = positions.astype(np.float64)[:, None] * inv[None, :]
    cos = np.concatenate([np.cos(ang), np.cos(ang)], -1)
    sin = np.concatenate([np.sin(ang), np.sin(ang)], -1)
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    rot = np.concatenate([-x2, x1], -1)
    return x * cos + rot * sin


def synth_kv(seed: int, B: int, Hkv: int, L: int, D: int, dtype: str, rope: bool = True,
             start: int = 0) -> Tuple[np.ndarray, np.ndarray]:
    """K, V ~ N(0,1), (B, Hkv, L, D), K rotated at positions start..start+L-1, on the dtype grid."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((B, Hkv, L, D))
    v = rng.standard_normal((B, Hkv, L, D))
    if rope:
        k = rope_rotate(k, np.arange(start, start + L))
    return rnd(k.astype(np.float32), dtype), rnd(v.astype(np.float32), dtype)
