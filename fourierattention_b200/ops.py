"""Tensor-level wrappers of the C ABI: pointer/stride marshalling only, no arithmetic.

Every function runs the sm_100a kernels on the current CUDA stream of the tensors' device.
PyTorch is used for device memory and streams.
"""
import ctypes as C

import torch

from . import _lib
from ._lib import DecodeArgs, check, lib

_DT = {torch.float16: _lib.FA_DTYPE_F16, torch.bfloat16: _lib.FA_DTYPE_BF16}
ANGLE_EXACT, ANGLE_KM57 = _lib.FA_ANGLE_EXACT, _lib.FA_ANGLE_KM57

_scratch = {}
launch_count = 0          # kernels-launching C-ABI calls made so far (for benchmark accounting)
last_decode_path = None   # fa_decode_path() of the most recent decode_attn call (0 exact, 1 tensor-core pass, 2 warp-specialised, 3 warp-specialised with the accumulator in tensor memory)


def _dt(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}: the cache stores float16 or bfloat16") from None


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("fourierattention_b200 kernels need CUDA tensors (there is no CPU path)")


def _stream(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def scratch(device, nbytes):
    """A grow-only byte buffer per (device, stream); kernels on one stream are ordered, so one
    buffer per stream is enough."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def _rows3(x):
    """(B, K, C) view parameters of a tensor whose last dim is contiguous."""
    if x.dim() != 3 or x.stride(2) != 1:
        raise ValueError("expected a (B, K, C) tensor with a contiguous last dimension")
    return x.shape[0], x.shape[1], x.stride(0), x.stride(1)


def gather_cols(x, idx32, out):
    _need_cuda(x, idx32, out)
    B, K, sb, sk = _rows3(x)
    with torch.cuda.device(x.device):
        check(lib.fa_gather_cols(_p(x), _dt(x), B, K, sb, sk, _p(idx32), idx32.numel(), _p(out), out.stride(0),
                                 out.stride(1), _stream(x)), "fa_gather_cols")
    _count(1)
    return out


def colstats(x, idx32=None):
    _need_cuda(x, idx32)
    B, K, sb, sk = _rows3(x)
    Mc = idx32.numel() if idx32 is not None else x.shape[2]
    avg = torch.empty((B, Mc), dtype=torch.float32, device=x.device)
    dev = torch.empty_like(avg)
    with torch.cuda.device(x.device):
        check(lib.fa_colstats(_p(x), _dt(x), B, K, sb, sk, _p(idx32), Mc, _p(avg), _p(dev), _stream(x)), "fa_colstats")
    _count(1)
    return avg, dev


def compress(x, idx32, N, T_c, k_start=0, coef=None, accumulate=False):
    _need_cuda(x, idx32, coef)
    B, K, sb, sk = _rows3(x)
    Mc = idx32.numel() if idx32 is not None else x.shape[2]
    if coef is None:
        coef = torch.empty((B, 2 * N, Mc), dtype=torch.float32, device=x.device)
        accumulate = False
    elif coef.shape != (B, 2 * N, Mc) or coef.dtype != torch.float32 or not coef.is_contiguous():
        raise ValueError("coef must be a contiguous float32 (B, 2N, Mc) tensor")
    with torch.cuda.device(x.device):
        nbytes = lib.fa_compress_scratch_bytes(B, K, N, Mc, x.shape[2])
        sc = scratch(x.device, nbytes) if nbytes else None
        check(lib.fa_compress(_p(x), _dt(x), B, K, sb, sk, x.shape[2], _p(idx32), Mc, N, int(T_c), int(k_start), _p(coef),
                              int(bool(accumulate)), _p(sc), nbytes, _stream(x)), "fa_compress")
    _count(2 if nbytes else 1)
    return coef


def evict_update(k_coef, k_row, k_idx32, v_coef, v_row, v_idx32, phase, T_c, angle_mode=ANGLE_KM57):
    """In place: coef += basis(phase) (x) row[idx] for K and V.  ``*_row``: (B, F) with contiguous rows."""
    _need_cuda(k_coef, k_row, v_coef, v_row)
    ref = k_coef if k_coef is not None else v_coef
    B, N2 = ref.shape[0], ref.shape[1]
    row = k_row if k_row is not None else v_row
    with torch.cuda.device(ref.device):
        check(lib.fa_evict_update(_p(k_coef), _p(k_row), k_row.stride(0) if k_row is not None else 0, _p(k_idx32),
                                  k_coef.shape[2] if k_coef is not None else 0,
                                  _p(v_coef), _p(v_row), v_row.stride(0) if v_row is not None else 0, _p(v_idx32),
                                  v_coef.shape[2] if v_coef is not None else 0,
                                  _dt(row), B, N2 // 2, int(phase), int(T_c), int(angle_mode), _stream(ref)),
              "fa_evict_update")
    _count(1)


def recon_stats(coef, K, T):
    _need_cuda(coef)
    if coef.dim() != 3 or coef.dtype != torch.float32 or not coef.is_contiguous():
        raise ValueError("coef must be a contiguous float32 (B, 2N, Mc) tensor")
    B, N2, Mc = coef.shape
    avg = torch.empty((B, Mc), dtype=torch.float32, device=coef.device)
    dev = torch.empty_like(avg)
    with torch.cuda.device(coef.device):
        nbytes = lib.fa_recon_stats_scratch_bytes(B, int(K), Mc)
        sc = scratch(coef.device, nbytes)
        check(lib.fa_recon_stats(_p(coef), B, N2 // 2, Mc, int(K), int(T), _p(avg), _p(dev), _p(sc), nbytes,
                                 _stream(coef)), "fa_recon_stats")
    _count(2)
    return avg, dev


def fourier_inverse(c, K, T):
    _need_cuda(c)
    if c.dim() != 2 or c.dtype != torch.float32 or not c.is_contiguous():
        raise ValueError("c must be a contiguous float32 (M, 2N) tensor")
    M, N2 = c.shape
    out = torch.empty((M, int(K)), dtype=torch.float32, device=c.device)
    with torch.cuda.device(c.device):
        check(lib.fa_fourier_inverse(_p(c), M, N2 // 2, int(K), int(T), _p(out), _stream(c)), "fa_fourier_inverse")
    _count(1)
    return out


def cache_step(k_evict, v_evict, kn32, vn32, k_unc_row, v_unc_row, k_new, v_new, k_dst, v_dst):
    """``*_evict``/``*_dst``: (B, F) row views; ``*_unc_row``: (B, Mn) row views of the verbatim stores;
    ``*_new``: (B, Hkv, 1, D) or (B, Hkv, D) with a contiguous last dim."""
    _need_cuda(k_evict, k_new, k_dst)
    B, F = k_evict.shape
    if k_new.dim() == 4:
        k_new, v_new = k_new[:, :, 0], v_new[:, :, 0]
    Hkv, D = k_new.shape[1], k_new.shape[2]
    if k_new.stride(2) != 1 or v_new.stride() != k_new.stride() or v_evict.stride() != k_evict.stride() \
            or v_dst.stride() != k_dst.stride():
        raise ValueError("fa_cache_step: K and V must share strides and have a contiguous last dimension")
    with torch.cuda.device(k_evict.device):
        check(lib.fa_cache_step(_p(k_evict), _p(v_evict), k_evict.stride(0), _p(kn32), kn32.numel(), _p(vn32),
                                vn32.numel(), _p(k_unc_row), k_unc_row.stride(0), _p(v_unc_row), v_unc_row.stride(0),
                                _p(k_new), _p(v_new), k_new.stride(0), k_new.stride(1), _p(k_dst), _p(v_dst),
                                k_dst.stride(0), _dt(k_evict), B, Hkv, D, _stream(k_evict)), "fa_cache_step")
    _count(1)


def evict_step(k_coef, k_idx32, v_coef, v_idx32, phase, T_c, angle_mode,
               k_evict, v_evict, kn32, vn32, k_unc_row, v_unc_row, k_new, v_new, k_dst, v_dst):
    """``evict_update`` of the evicted row followed by ``cache_step``, as one launch."""
    _need_cuda(k_evict, k_new, k_dst)
    B, F = k_evict.shape
    if k_new.dim() == 4:
        k_new, v_new = k_new[:, :, 0], v_new[:, :, 0]
    Hkv, D = k_new.shape[1], k_new.shape[2]
    if k_new.stride(2) != 1 or v_new.stride() != k_new.stride() or v_evict.stride() != k_evict.stride() \
            or v_dst.stride() != k_dst.stride():
        raise ValueError("fa_evict_step: K and V must share strides and have a contiguous last dimension")
    ref = k_coef if k_coef is not None else v_coef
    N = ref.shape[1] // 2 if ref is not None else 1
    with torch.cuda.device(k_evict.device):
        check(lib.fa_evict_step(_p(k_coef), _p(k_evict) if k_coef is not None else None, k_evict.stride(0),
                                _p(k_idx32), k_coef.shape[2] if k_coef is not None else 0,
                                _p(v_coef), _p(v_evict) if v_coef is not None else None, v_evict.stride(0),
                                _p(v_idx32), v_coef.shape[2] if v_coef is not None else 0,
                                N, int(phase), int(T_c), int(angle_mode),
                                _p(k_evict), _p(v_evict), k_evict.stride(0), _p(kn32), kn32.numel(), _p(vn32),
                                vn32.numel(), _p(k_unc_row), k_unc_row.stride(0), _p(v_unc_row), v_unc_row.stride(0),
                                _p(k_new), _p(v_new), k_new.stride(0), k_new.stride(1), _p(k_dst), _p(v_dst),
                                k_dst.stride(0), _dt(k_evict), B, Hkv, D, _stream(k_evict)), "fa_evict_step")
    _count(1)


class DecodeTables:
    """int32 device copies of the eight index vectors the attention kernel reads."""

    def __init__(self, kc_list, kc_h, kn_list, kn_h, vc_list, vc_h, vn_list, vn_h, device):
        def cv(t):
            return torch.as_tensor(t).to(device=device, dtype=torch.int32).contiguous()
        self.kc_list, self.kc_h, self.kn_list, self.kn_h = cv(kc_list), cv(kc_h), cv(kn_list), cv(kn_h)
        self.vc_list, self.vc_h, self.vn_list, self.vn_h = cv(vc_list), cv(vc_h), cv(vn_list), cv(vn_h)
        # host copies of the two verbatim offset tables: the planner reads them to choose the kernel
        kh, vh = self.kn_h.cpu().tolist(), self.vn_h.cpu().tolist()
        self.kn_h_host = (C.c_int32 * len(kh))(*kh)
        self.vn_h_host = (C.c_int32 * len(vh))(*vh)


def decode_attn(q, k_sink, v_sink, k_win, v_win, k_mn, v_mn, k_coef, v_coef,
                avg_k_u, avg_k_d, scale_k, avg_v_u, avg_v_d, scale_v, tables,
                num_head_q, num_head_kv, T, sm_scale=-1.0, mid_l0=0, out=None, return_lse=False, phase_events=None,
                static_scratch=False):
    """Fused decode attention.  q: (B, Hq*D) (or (B,1,Hq*D)); sinks/window: (B, n, F) or None;
    k_mn/v_mn: (B, n_mid, Mn) row-strided views; coefficients (B, 2N, Mc) float32; statistics
    (B, Mc) float32.  Returns (B, Hq, D) float32 (plus (m, l) if ``return_lse``).
    ``static_scratch=True`` goes through ``fa_decode_attn_static``: no scratch tensor is taken from
    PyTorch's allocator, the kernels use the fixed buffer inside the library (see fourier_b200.h)."""
    _need_cuda(q)
    if q.dim() == 3:
        q = q[:, 0]
    B = q.shape[0]
    D = q.shape[1] // num_head_q
    F = num_head_kv * D
    dev = q.device
    a = DecodeArgs()
    a.B, a.Hq, a.Hkv, a.D = B, num_head_q, num_head_kv, D
    a.n_sink = k_sink.shape[1] if k_sink is not None else 0
    a.n_win = k_win.shape[1] if k_win is not None else 0
    a.n_mid = k_mn.shape[1] if k_mn is not None else 0
    a.mid_l0 = int(mid_l0)
    a.N = k_coef.shape[1] // 2 if k_coef is not None else 0
    a.T = int(T)
    a.Mc_k = k_coef.shape[2] if k_coef is not None else 0
    a.Mc_v = v_coef.shape[2] if v_coef is not None else 0
    a.Mn_k, a.Mn_v = F - a.Mc_k, F - a.Mc_v
    a.dtype = _dt(q)
    a.sm_scale = float(sm_scale) if sm_scale is not None else -1.0
    if q.stride(1) != 1:
        raise ValueError("q must have a contiguous last dimension")
    a.q, a.q_sb = q.data_ptr(), q.stride(0)

    def rows(t, name):
        if t is None:
            return 0, 0
        if t.stride(2) != 1 or t.stride(1) != F or t.dtype != q.dtype:
            raise ValueError(f"{name}: expected dtype {q.dtype} and dense (B, n, {F}) rows")
        return t.data_ptr(), t.stride(0)
    a.k_sink, a.sink_sb = rows(k_sink, "k_sink")
    a.v_sink, sb2 = rows(v_sink, "v_sink")
    a.k_win, a.win_sb = rows(k_win, "k_win")
    a.v_win, wb2 = rows(v_win, "v_win")
    if (k_sink is not None and sb2 != a.sink_sb) or (k_win is not None and wb2 != a.win_sb):
        raise ValueError("K and V segments must share their batch stride")
    if a.n_mid > 0:
        for t, nm in ((k_mn, "k_mn"), (v_mn, "v_mn")):
            if (t.shape[2] > 0 and t.stride(2) != 1) or t.dtype != q.dtype:
                raise ValueError(f"{nm}: expected dtype {q.dtype} with a contiguous last dimension")
        for t in (k_coef, v_coef, avg_k_u, avg_k_d, scale_k, avg_v_u, avg_v_d, scale_v):
            if t.dtype != torch.float32 or not t.is_contiguous():
                raise ValueError("coefficients and statistics must be contiguous float32")
        a.k_mn, a.k_mn_sb, a.k_mn_sk = k_mn.data_ptr(), k_mn.stride(0), max(k_mn.stride(1), a.Mn_k)
        a.v_mn, a.v_mn_sb, a.v_mn_sk = v_mn.data_ptr(), v_mn.stride(0), max(v_mn.stride(1), a.Mn_v)
        a.k_coef, a.v_coef = k_coef.data_ptr(), v_coef.data_ptr()
        a.avg_k_u, a.avg_k_d, a.scale_k = avg_k_u.data_ptr(), avg_k_d.data_ptr(), scale_k.data_ptr()
        a.avg_v_u, a.avg_v_d, a.scale_v = avg_v_u.data_ptr(), avg_v_d.data_ptr(), scale_v.data_ptr()
        tb = tables
        a.kc_list, a.kc_h, a.kn_list, a.kn_h = (tb.kc_list.data_ptr(), tb.kc_h.data_ptr(), tb.kn_list.data_ptr(),
                                                tb.kn_h.data_ptr())
        a.vc_list, a.vc_h, a.vn_list, a.vn_h = (tb.vc_list.data_ptr(), tb.vc_h.data_ptr(), tb.vn_list.data_ptr(),
                                                tb.vn_h.data_ptr())
        a.kn_h_host = C.cast(tb.kn_h_host, C.c_void_p)
        a.vn_h_host = C.cast(tb.vn_h_host, C.c_void_p)
    if out is None:
        out = torch.empty((B, num_head_q, D), dtype=torch.float32, device=dev)
    a.out = out.data_ptr()
    m = l = None
    if return_lse:
        m = torch.empty((B, num_head_q), dtype=torch.float32, device=dev)
        l = torch.empty_like(m)
        a.m_out, a.l_out = m.data_ptr(), l.data_ptr()
    if phase_events is not None:       # five torch.cuda.Event(enable_timing=True), see fourier_b200.h
        ev = (C.c_void_p * 5)(*[(e.cuda_event if e is not None else None) for e in phase_events])
        a.phase_events_host = C.cast(ev, C.c_void_p)
    global last_decode_path
    last_decode_path = lib.fa_decode_path(C.byref(a))
    if static_scratch:
        with torch.cuda.device(dev):
            check(lib.fa_decode_attn_static(C.byref(a), _stream(q)), "fa_decode_attn_static")
        _count(3 if a.n_mid > 0 else 2)
        return (out, m, l) if return_lse else out
    with torch.cuda.device(dev):
        nbytes = lib.fa_decode_scratch_bytes(C.byref(a))
        if nbytes == 0:
            check(lib.fa_decode_attn(C.byref(a), _stream(q)), "fa_decode_attn")   # reports the plan error
            raise RuntimeError("fa_decode_attn: empty scratch plan")
        sc = scratch(dev, nbytes)
        a.scratch, a.scratch_bytes = sc.data_ptr(), sc.numel()
        check(lib.fa_decode_attn(C.byref(a), _stream(q)), "fa_decode_attn")
    _count(3 if a.n_mid > 0 else 2)
    return (out, m, l) if return_lse else out


class LayerCalls:
    """The two per-step calls of one cached layer behind a library-side handle (``fa_layer_*``): buffers,
    tables, statistics, planner switches and tensor maps are bound once when the layer is created, a decode
    step passes the window offset, the span length and the new tensors only."""

    def __init__(self, kbuf, vbuf, k_unc, v_unc, k_coef, v_coef, stats32, tables, S, W, num_head_kv, T, mid_l0,
                 T_c, angle_mode, with_il=True):
        self.dev = kbuf.device
        self.B, rows, self.F = kbuf.shape
        self.S, self.W, self.Hkv = int(S), int(W), int(num_head_kv)
        self.D = self.F // self.Hkv
        self.tables, self.stats32 = tables, stats32           # keep the tensors alive
        self.k_coef, self.v_coef = k_coef, v_coef
        self.kbuf, self.vbuf = kbuf, vbuf
        if vbuf.stride(0) != kbuf.stride(0) or kbuf.stride(1) != self.F or kbuf.stride(2) != 1 \
                or vbuf.stride(1) != self.F or vbuf.stride(2) != 1:
            raise ValueError("K and V window buffers must be dense (B, rows, F) with equal strides")
        for t in stats32:
            if t.dtype != torch.float32 or not t.is_contiguous():
                raise ValueError("statistics must be contiguous float32")
        self.with_il = with_il
        tb = tables
        d = self.desc = _lib.LayerDesc()
        d.B, d.Hkv, d.D, d.S, d.W = self.B, self.Hkv, self.D, self.S, self.W
        have = k_coef if k_coef is not None else v_coef
        d.N = have.shape[1] // 2 if have is not None else 1
        d.T, d.T_c, d.angle_mode, d.dtype, d.mid_l0 = int(T), int(T_c), int(angle_mode), _dt(kbuf), int(mid_l0)
        d.Mc_k, d.Mc_v = tb.kc_list.numel(), tb.vc_list.numel()
        d.Mn_k, d.Mn_v = tb.kn_list.numel(), tb.vn_list.numel()
        d.with_il = 1 if with_il else 0
        d.kbuf, d.vbuf, d.buf_sb, d.buf_rows = kbuf.data_ptr(), vbuf.data_ptr(), kbuf.stride(0), rows
        d.k_coef = k_coef.data_ptr() if k_coef is not None else None
        d.v_coef = v_coef.data_ptr() if v_coef is not None else None
        (d.avg_k_u, d.avg_k_d, d.scale_k, d.avg_v_u, d.avg_v_d, d.scale_v) = [t.data_ptr() for t in stats32]
        d.kc_list, d.kc_h, d.kn_list, d.kn_h = (tb.kc_list.data_ptr(), tb.kc_h.data_ptr(), tb.kn_list.data_ptr(),
                                                tb.kn_h.data_ptr())
        d.vc_list, d.vc_h, d.vn_list, d.vn_h = (tb.vc_list.data_ptr(), tb.vc_h.data_ptr(), tb.vn_list.data_ptr(),
                                                tb.vn_h.data_ptr())
        d.kn_h_host = C.cast(tb.kn_h_host, C.c_void_p)
        d.vn_h_host = C.cast(tb.vn_h_host, C.c_void_p)
        self._set_stores(k_unc, v_unc)
        h = C.c_void_p()
        with torch.cuda.device(self.dev):
            check(lib.fa_layer_create(C.byref(d), C.byref(h)), "fa_layer_create")
        self._h = h
        self._scratch_key = None
        self._scratch_bytes = 0

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            lib.fa_layer_destroy(h)
            self._h = None

    def _set_stores(self, k_unc, v_unc):
        self.k_unc, self.v_unc = k_unc, v_unc
        d = self.desc
        d.k_unc, d.v_unc = k_unc.data_ptr(), v_unc.data_ptr()
        d.k_unc_sb, d.v_unc_sb = k_unc.stride(0), v_unc.stride(0)
        d.k_unc_sk, d.v_unc_sk = max(k_unc.stride(1), d.Mn_k), max(v_unc.stride(1), d.Mn_v)
        d.unc_rows = k_unc.shape[1]

    def set_statistics(self, stats32):
        """Replace the six float32 statistics tensors (avg_k_u, avg_k_d, scale_k, avg_v_u, avg_v_d, scale_v);
        the handle is made anew around the same buffers."""
        for t in stats32:
            if t.dtype != torch.float32 or not t.is_contiguous():
                raise ValueError("statistics must be contiguous float32")
        self.stats32 = stats32
        d = self.desc
        (d.avg_k_u, d.avg_k_d, d.scale_k, d.avg_v_u, d.avg_v_d, d.scale_v) = [t.data_ptr() for t in stats32]
        lib.fa_layer_destroy(self._h)
        h = C.c_void_p()
        with torch.cuda.device(self.dev):
            check(lib.fa_layer_create(C.byref(d), C.byref(h)), "fa_layer_create")
        self._h = h
        self._scratch_key = None

    def rebind(self, k_unc, v_unc):
        """(Re)attach the verbatim stores (they are reallocated when they grow)."""
        self._set_stores(k_unc, v_unc)
        d = self.desc
        check(lib.fa_layer_rebind_stores(self._h, d.k_unc, d.v_unc, d.k_unc_sb, d.v_unc_sb, d.k_unc_sk, d.v_unc_sk,
                                         d.unc_rows), "fa_layer_rebind_stores")
        self._scratch_key = None

    def step(self, off, n_mid, phase, k_new, v_new, appends=True):
        """One steady-state cache step: the window row at offset ``off`` is evicted (its compressed dims go into
        the coefficients at ``phase``, its verbatim dims to row ``n_mid`` of the stores) and the new token is
        written behind the window."""
        if k_new.dim() == 4:
            k_new, v_new = k_new[:, :, 0], v_new[:, :, 0]
        if k_new.stride(2) != 1 or v_new.stride() != k_new.stride():
            raise ValueError("fa_layer_update: K and V must share strides and have a contiguous last dimension")
        if torch.cuda.current_device() != self.dev.index:
            torch.cuda.set_device(self.dev)
        rc = lib.fa_layer_update(self._h, off, n_mid, int(phase), 1 if appends else 0, k_new.data_ptr(),
                                 v_new.data_ptr(), k_new.stride(0), k_new.stride(1),
                                 torch.cuda.current_stream(self.dev).cuda_stream)
        if rc:
            check(rc, "fa_layer_update")
        _count(1)

    def attend(self, q, off, n_mid, num_head_q, sm_scale=-1.0, phase_events=None, return_lse=False):
        """Decode attention of one query token per sequence; ``q``: (B, Hq*D).  Returns (B, Hq, D) float32
        (plus the softmax statistics (m, l) with ``return_lse``)."""
        global last_decode_path
        if q.stride(1) != 1 or q.dtype != self.kbuf.dtype:
            raise ValueError("q must have the cache dtype and a contiguous last dimension")
        out = torch.empty((self.B, num_head_q, self.D), dtype=torch.float32, device=self.dev)
        m = l = None
        if return_lse:
            m = torch.empty((self.B, num_head_q), dtype=torch.float32, device=self.dev)
            l = torch.empty_like(m)
        if n_mid == 0 and not self.with_il:
            # this rank holds no key at all (a span slice with no rows): an empty partial result that the
            # log-sum-exp merge ignores (l = 0), so that the rank still takes part in the exchange
            out.zero_()
            if return_lse:
                m.fill_(-1.0e30)
                l.zero_()
            return (out, m, l) if return_lse else out
        if torch.cuda.current_device() != self.dev.index:
            torch.cuda.set_device(self.dev)
        stream = torch.cuda.current_stream(self.dev).cuda_stream
        # the plan (and with it the scratch need) is constant while n_mid stays inside one 128-token super-tile
        key = (num_head_q, (n_mid + 127) >> 7)
        if key != self._scratch_key:
            nbytes = lib.fa_layer_scratch_bytes(self._h, num_head_q, n_mid)
            if nbytes == 0:
                check(lib.fa_layer_attend(self._h, off, n_mid, num_head_q, q.data_ptr(), q.stride(0), -1.0,
                                          out.data_ptr(), None, None, None, 0, None, stream), "fa_layer_attend")
                raise RuntimeError("fa_layer_attend: empty scratch plan")
            self._scratch_bytes = 2 * int(nbytes)
            self._scratch_key = key
            last_decode_path = lib.fa_layer_decode_path(self._h)
        sc = scratch(self.dev, self._scratch_bytes)
        ev = None
        if phase_events is not None:
            ev = (C.c_void_p * 5)(*[(e.cuda_event if e is not None else None) for e in phase_events])
        rc = lib.fa_layer_attend(self._h, off, n_mid, num_head_q, q.data_ptr(), q.stride(0),
                                 float(sm_scale) if sm_scale is not None else -1.0, out.data_ptr(),
                                 m.data_ptr() if m is not None else None, l.data_ptr() if l is not None else None,
                                 sc.data_ptr(), sc.numel(), ev, stream)
        if rc:
            check(rc, "fa_layer_attend")
        _count(3 if n_mid > 0 else 2)
        return (out, m, l) if return_lse else out


def merge(o, m, l):
    """o: (P, rows, D) normalised partial outputs, m/l: (P, rows).  Returns (rows, D)."""
    _need_cuda(o, m, l)
    P, rows, D = o.shape
    o, m, l = o.contiguous(), m.contiguous(), l.contiguous()
    out = torch.empty((rows, D), dtype=torch.float32, device=o.device)
    with torch.cuda.device(o.device):
        check(lib.fa_merge(_p(o), _p(m), _p(l), P, rows, D, _p(out), _stream(o)), "fa_merge")
    _count(1)
    return out


def _count(n):
    global launch_count
    launch_count += n
