"""Drop-in for the reference kernel module ``fourier_attn_triton/fourier_triton_valid4_v2.py``.

Same public names and signatures (reference lines in each docstring); the device work is done by
the sm_100a kernels of ``libfourier_b200.so``.  CUDA tensors only.
"""
import numpy as np
import torch
import torch.nn as nn

from . import ops

__all__ = ["mat_fourier_triton", "mat_fourier_inv_triton", "mat_fourier_avg_std_triton", "mat_avg_std_triton",
           "triton_fourier_attn", "torch_fourier_attn", "mat_fourier_inv_torch", "MultiDimHiPPO2"]

_table_cache = {}


def mat_fourier_triton(a, N, T, K_start=0):
    """(B, K, M) fp16/bf16 -> (B, 2N, M) float32 cosine / sine sums with phase offset ``K_start`` and
    period ``T`` (reference: mat_fourier_triton, fourier_triton_valid4_v2.py:81-102)."""
    assert a.is_contiguous(), "Matrix A must be contiguous"
    return ops.compress(a, None, int(N), int(T), int(K_start))


def mat_fourier_inv_triton(c, K, T):
    """(M, 2N) float32 -> (M, K) float32 inverse (reference: fourier_triton_valid4_v2.py:170-183)."""
    assert c.is_contiguous(), "Matrix C must be contiguous"
    return ops.fourier_inverse(c.float(), int(K), int(T))


def mat_fourier_avg_std_triton(c, K, T):
    """Mean and maximum one-sided deviation of the span rebuilt from coefficients ``c`` (B, 2N, M),
    both float16 (reference: fourier_triton_valid4_v2.py:285-326)."""
    assert c.is_contiguous(), "Matrix C must be contiguous"
    avg, dev = ops.recon_stats(c, int(K), int(T))
    return avg.to(torch.float16), dev.to(torch.float16)


def mat_avg_std_triton(a):
    """Column mean and maximum one-sided deviation over dim 1 of a (B, K, M) tensor, in ``a.dtype``
    (reference: fourier_triton_valid4_v2.py:433-461)."""
    assert a.is_cuda and a.is_contiguous(), "Input tensor must be a contiguous CUDA tensor"
    assert a.dim() == 3, "Input tensor must be 3-dimensional"
    avg, dev = ops.colstats(a, None)
    return avg.to(a.dtype), dev.to(a.dtype)


def _tables_for(lists, device):
    key = tuple((t.data_ptr(), t.numel(), t._version) for t in lists) + (str(device),)
    tb = _table_cache.get(key)
    if tb is None:
        if len(_table_cache) > 512:
            _table_cache.clear()
        tb = ops.DecodeTables(*lists, device=device)
        _table_cache[key] = (tb, lists)          # keep the sources alive so data_ptr stays unique
        return tb
    return tb[0]


def triton_fourier_attn(q, k_il, v_il, k_mc, v_mc, k_mn, v_mn,
                        avg_k_u, avg_k_d, scale_k, avg_v_u, avg_v_d, scale_v,
                        kc_list, kc_h_list, kn_list, kn_h_list,
                        vc_list, vc_h_list, vn_list, vn_h_list,
                        num_head_q, num_head_kv, seq_len_m, T, sm_scale=-1):
    """Decode attention over [sinks; window] rows ``k_il/v_il`` (B, S+W, F), spectral coefficients
    ``k_mc/v_mc`` (B, 2N, Mc) and verbatim middle-span dims ``k_mn/v_mn`` (B, n_mid, Mn).
    Returns (B, Hq, 1, D) float32 (reference: triton_fourier_attn, fourier_triton_valid4_v2.py:684-779)."""
    batch_size, seq_len_q, feature_dim = q.shape
    assert seq_len_q == 1, f"{q.shape = }"
    head_dim = feature_dim // num_head_q
    tb = _tables_for((kc_list, kc_h_list, kn_list, kn_h_list, vc_list, vc_h_list, vn_list, vn_h_list), q.device)
    f32 = lambda t: t.to(torch.float32).contiguous()
    seq_len_m = int(seq_len_m)
    out = ops.decode_attn(
        q.contiguous(), None, None, k_il.contiguous(), v_il.contiguous(),
        k_mn[:, :seq_len_m] if seq_len_m else None, v_mn[:, :seq_len_m] if seq_len_m else None,
        f32(k_mc), f32(v_mc), f32(avg_k_u), f32(avg_k_d), f32(scale_k), f32(avg_v_u), f32(avg_v_d), f32(scale_v),
        tb, num_head_q, num_head_kv, T, sm_scale)
    return out.view(batch_size, num_head_q, 1, head_dim)


def torch_fourier_attn(*args, **kwargs):
    """Same arguments as :func:`triton_fourier_attn`; returns float16 like the reference's PyTorch path
    (fourier_triton_valid4_v2.py:794-837).  Here both names run the same CUDA kernels."""
    return triton_fourier_attn(*args, **kwargs).to(torch.float16)


def mat_fourier_inv_torch(c, K, T):
    """(B, 2N, Mc) -> (B, K, Mc) reconstruction (reference: fourier_triton_valid4_v2.py:782-791)."""
    B, N2, Mc = c.shape
    flat = c.float().permute(0, 2, 1).reshape(B * Mc, N2).contiguous()
    return ops.fourier_inverse(flat, int(K), int(T)).view(B, Mc, int(K)).permute(0, 2, 1)


class MultiDimHiPPO2(nn.Module):
    """Compressor object of the cache (reference: fourier_triton_valid4_v2.py:840-867).

    ``forward(base_input, token_num)`` projects a (B, K, M) span onto ``N // input_dim // 2`` cosines and
    sines of period ``int(1/dt)``; ``forward(coef, token_num, slice_input=row)`` returns ``coef`` plus the
    projection of one more row at phase ``token_num``."""

    def __init__(self, N, input_dim, method='legt', dt=1.0, T=1.0, discretization='bilinear', scale=False, c=0.0):
        super().__init__()
        self.method = method
        self.N = N
        self.input_dim = input_dim
        self.dt = dt
        self.T = T
        self.c = c
        self.base_N = N // input_dim

    def forward(self, base_input, token_num, slice_input=None, fast=False):
        base_N = self.N // self.input_dim // 2
        period = int(1 / self.dt)
        if slice_input is not None:
            out = base_input.clone()
            row = slice_input.reshape(slice_input.shape[0], -1)
            ops.evict_update(out, row, None, None, None, None, int(token_num), period, ops.ANGLE_KM57)
            return out
        x = base_input
        if x.shape[1] > period:       # torch.fft.fft(x, n=period) truncates a longer span
            x = x[:, :period]
        return ops.compress(x, None, base_N, period, 0)
