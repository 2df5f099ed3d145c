"""Drop-in for the Fourier KV cache of ``fourier_attn_triton/cache_utils_fourier.py``.

``DynamicCache(extra_config)`` keeps the reference's constructor, attributes, ``update`` contract and
returned dict layout (cache_utils_fourier.py:363-761), but the state lives in pre-allocated device
buffers that the sm_100a kernels update in place:

* sinks and the local window share one linear buffer ``(B, S + 2W, F)``; the window is a sliding view
  that is copied back to the front every W steps (amortised one row per step);
* the verbatim dims of the middle span live in a ``(B, capacity, Mn_pad)`` buffer that grows by one row
  per step (row pitch padded to 16 bytes so rows stream with 128-bit loads);
* the spectral coefficients ``(B, 2N, Mc)`` float32 are updated in place by a rank-1 kernel.

Tensors handed out by ``update`` are views of these buffers and stay valid until the next ``update`` of
the same layer.
"""
import json
from typing import Any, Dict, List, Optional, Tuple

import torch

from . import ops

__all__ = ["Cache", "DynamicCache", "StaticCache", "compress_period", "shard_tables", "span_slice"]


def compress_period(T: int) -> int:
    """Period of the forward projection.  The reference builds its compressor with ``dt = 1/T``
    (cache_utils_fourier.py:547) and the compressor uses ``int(1/dt)``
    (fourier_triton_valid4_v2.py:856, 859); in IEEE double that is ``T - 1`` for some ``T``."""
    return int(1.0 / (1.0 / float(T)))


class Cache(torch.nn.Module):
    """Minimal base class (the reference's ``Cache`` is the stock HuggingFace one)."""

    def __init__(self):
        super().__init__()

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        raise NotImplementedError

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        raise NotImplementedError

    def get_max_cache_shape(self) -> Optional[int]:
        return None


class StaticCache(Cache):
    """Name kept importable for modeling code; the stock HuggingFace static cache is not part of the
    Fourier path."""

    def __init__(self, *args, **kwargs):
        raise NotImplementedError("StaticCache is not provided by fourierattention_b200")


def _round8(x):
    return (x + 7) // 8 * 8


def shard_tables(ent, h0, h1):
    """Restrict one layer's ``_splithead`` entry to KV heads h0..h1-1 and rebase the flat dims, so that a
    rank owning those heads can run the path on its slice alone (every quantity on the path is per KV
    head: cache_utils_fourier.py:444-452 keeps cumulative per-head offsets for exactly this lookup)."""
    n_heads = len(ent["kc_h_list"])
    F = len(ent["kc_list"]) + len(ent["kn_list"])
    D = F // n_heads
    out = {}
    for t in ("kc", "kn", "vc", "vn"):
        cum = [0] + list(ent[f"{t}_h_list"])
        lst = ent[f"{t}_list"][cum[h0]:cum[h1]]
        out[f"{t}_list"] = [int(i) - h0 * D for i in lst]
        out[f"{t}_h_list"] = [cum[h] - cum[h0] for h in range(h0 + 1, h1 + 1)]
    return out


def span_slice(n_rows, rank, world):
    """Rows [lo, hi) of a middle span of ``n_rows`` rows that rank ``rank`` of ``world`` keeps when the span
    is split by sequence (equal contiguous slices, the last one may be shorter)."""
    per = (n_rows + world - 1) // world
    return min(n_rows, rank * per), min(n_rows, (rank + 1) * per)


class _LayerState:
    __slots__ = ("compressed", "kbuf", "vbuf", "off", "k_unc", "v_unc", "n_mid", "k_coef", "v_coef",
                 "stats32", "local_len", "mid_l0", "calls")


class DynamicCache(Cache):
    """Fourier-compressed KV cache (reference: DynamicCache, cache_utils_fourier.py:363-761).

    ``extra_config`` is duck-typed with the attributes the reference reads
    (cache_utils_fourier.py:394-403): ``max_new_tokens, maxlocallen, maxmidstates, numinittokens,
    num_key_value_heads, max_position_embeddings, non_critical_dims_path``.

    Extra keyword arguments (not in the reference):
      ``device``          where tables and state live (default: current CUDA device);
      ``kv_head_range``   ``(h0, h1)``: this rank owns KV heads h0..h1-1 (head sharding, no communication);
      ``seq_shard``       ``(rank, world)``: this rank keeps an equal contiguous slice of the middle span
                          (sequence split; partial results are merged with a log-sum-exp reduction);
      ``process_group``   ``torch.distributed`` group used by the sequence split;
      ``update_angle``    ``ops.ANGLE_KM57`` (default, the reference's float32 angle in decode-time
                          updates) or ``ops.ANGLE_EXACT``.
    """

    def __init__(self, extra_config, num_hidden_layers: Optional[int] = None, device=None,
                 kv_head_range: Optional[Tuple[int, int]] = None, seq_shard: Optional[Tuple[int, int]] = None,
                 process_group=None, update_angle: int = ops.ANGLE_KM57) -> None:
        super().__init__()
        self._seen_tokens = 0
        self.key_cache: List[Dict[str, torch.Tensor]] = []
        self.value_cache: List[Dict[str, torch.Tensor]] = []
        self.maxnewtokens = extra_config.max_new_tokens
        self.maxlocallen = extra_config.maxlocallen
        self.maxmidstates = extra_config.maxmidstates
        self.numinittokens = extra_config.numinittokens
        self.maxlen = self.maxlocallen + self.maxmidstates + self.numinittokens
        self.heads = extra_config.num_key_value_heads
        self.maxtokens = extra_config.max_position_embeddings
        self.curr_tokennum: List[int] = []
        if device is None:
            if not torch.cuda.is_available():
                raise RuntimeError("fourierattention_b200.DynamicCache needs a CUDA device (there is no CPU path)")
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = torch.device(device)
        self.kv_head_range = kv_head_range
        self.seq_shard = seq_shard
        self.process_group = process_group
        self.update_angle = update_angle

        with open(extra_config.non_critical_dims_path, "r") as f:
            non_critical_dims = json.load(f)

        self.k_scale, self.v_scale = [], []
        self.k_layer_average, self.v_layer_average = [], []
        self.kd_layer_average, self.vd_layer_average = [], []
        self.k_non_critical_dims, self.k_non_critical_head_dims = [], []
        self.k_critical_dims, self.k_critical_head_dims = [], []
        self.v_non_critical_dims, self.v_non_critical_head_dims = [], []
        self.v_critical_dims, self.v_critical_head_dims = [], []
        self._tables: List[ops.DecodeTables] = []
        self._state: List[_LayerState] = []

        for layer_idx in range(len(non_critical_dims)):
            self.curr_tokennum.append(0)
            layer_key = f"Layer_{layer_idx}"
            if layer_key not in non_critical_dims:
                raise ValueError(f"Layer index {layer_idx} not found in non-critical dimensions JSON file.")
            ent = self._shard_tables(non_critical_dims[layer_key])
            i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=self.device)
            self.k_non_critical_dims.append(i64(ent["kc_list"]))
            self.k_critical_dims.append(i64(ent["kn_list"]))
            self.v_non_critical_dims.append(i64(ent["vc_list"]))
            self.v_critical_dims.append(i64(ent["vn_list"]))
            self.k_non_critical_head_dims.append(i64([0] + ent["kc_h_list"]))
            self.k_critical_head_dims.append(i64([0] + ent["kn_h_list"]))
            self.v_non_critical_head_dims.append(i64([0] + ent["vc_h_list"]))
            self.v_critical_head_dims.append(i64([0] + ent["vn_h_list"]))
            self._tables.append(ops.DecodeTables(ent["kc_list"], [0] + ent["kc_h_list"], ent["kn_list"],
                                                 [0] + ent["kn_h_list"], ent["vc_list"], [0] + ent["vc_h_list"],
                                                 ent["vn_list"], [0] + ent["vn_h_list"], device=self.device))

    # ------------------------------------------------------------------------------------------
    def _shard_tables(self, ent):
        if self.kv_head_range is None:
            return ent
        return shard_tables(ent, *self.kv_head_range)

    def __len__(self):
        return len(self.key_cache)

    def __getitem__(self, layer_idx):
        return None

    def __iter__(self):
        return iter(())

    @property
    def attention_period(self) -> int:
        """T of the reconstruction (modeling_llama_fourier.py:660)."""
        return self.maxtokens - self.numinittokens - self.maxlocallen

    # ------------------------------------------------------------------------------------------
    def _compress_side(self, x, lo, hi, c32, n32, unc_buf, dtype):
        """Build coefficients, statistics and the verbatim store of one of K / V from prompt rows
        ``x[:, lo:hi]`` (cache_utils_fourier.py:560-569)."""
        B = x.shape[0]
        N = self.maxmidstates // 2
        T = self.attention_period
        T_c = compress_period(T)
        mid = x[:, lo:hi]
        K_all = mid.shape[1]
        Mc = c32.numel()
        # this rank's slice of the span (everything unless the span is split by sequence)
        r0, r1 = self._span_slice(K_all)
        if n32.numel() and r1 > r0:
            ops.gather_cols(mid[:, r0:r1], n32, unc_buf)
        # rows beyond T_c are dropped by the reference's length-T_c FFT
        k_used = min(K_all, T_c)
        if Mc == 0:
            coef = torch.zeros((B, 2 * N, 0), dtype=torch.float32, device=x.device)
            z = torch.zeros((B, 0), dtype=torch.float32, device=x.device)
            return coef, z.to(dtype), z.to(torch.float16), z.to(torch.float16), z.to(dtype)
        if self.seq_shard is None:
            coef = ops.compress(mid[:, :k_used], c32, N, T_c, 0)
        else:
            import torch.distributed as dist
            coef = torch.zeros((B, 2 * N, Mc), dtype=torch.float32, device=x.device)
            s0, s1 = min(r0, k_used), min(r1, k_used)
            if s1 > s0:
                ops.compress(mid[:, s0:s1], c32, N, T_c, s0, coef=coef, accumulate=False)
            dist.all_reduce(coef, group=self.process_group)
        u_avg, u_dev = ops.colstats(mid, c32)
        i_avg, i_dev = ops.recon_stats(coef, K_all, T)
        u_avg, u_dev = u_avg.to(dtype), u_dev.to(dtype)                   # fourier_triton_valid4_v2.py:461
        i_avg, i_dev = i_avg.to(torch.float16), i_dev.to(torch.float16)   # fourier_triton_valid4_v2.py:326
        return coef, u_avg, i_avg, i_dev, u_dev

    def _span_slice(self, n_rows):
        if self.seq_shard is None:
            return 0, n_rows
        return span_slice(n_rows, *self.seq_shard)

    def _prefill_layer(self, key_states, value_states, layer_idx):
        B, P, F = key_states.shape
        S, W, M = self.numinittokens, self.maxlocallen, self.maxmidstates
        dtype, dev = key_states.dtype, key_states.device
        tb = self._tables[layer_idx]
        st = _LayerState()
        st.compressed = True
        st.off = 0
        n_mid = P - S - W
        r0, r1 = self._span_slice(n_mid)
        st.mid_l0 = r0
        last_rank = self.seq_shard is None or self.seq_shard[0] == self.seq_shard[1] - 1
        cap = (r1 - r0) + (self.maxnewtokens + 8 if last_rank else 0)
        Mn_k, Mn_v = tb.kn_list.numel(), tb.vn_list.numel()
        # zero-filled: the kernels fetch whole tiles, and rows a tile covers beyond the live ones (masked with
        # probability 0) must hold finite values
        st.kbuf = torch.zeros((B, S + 2 * W, F), dtype=dtype, device=dev)
        st.vbuf = torch.zeros((B, S + 2 * W, F), dtype=dtype, device=dev)
        st.kbuf[:, :S].copy_(key_states[:, :S]); st.kbuf[:, S:S + W].copy_(key_states[:, P - W:])
        st.vbuf[:, :S].copy_(value_states[:, :S]); st.vbuf[:, S:S + W].copy_(value_states[:, P - W:])
        st.k_unc = torch.zeros((B, max(cap, 1), max(_round8(Mn_k), 8)), dtype=dtype, device=dev)
        st.v_unc = torch.zeros((B, max(cap, 1), max(_round8(Mn_v), 8)), dtype=dtype, device=dev)
        st.n_mid = r1 - r0
        k_coef, k_ua, k_ia, k_idev, k_udev = self._compress_side(key_states, S, P - W, tb.kc_list, tb.kn_list,
                                                                  st.k_unc[:, :st.n_mid, :Mn_k], dtype)
        v_coef, v_ua, v_ia, v_idev, v_udev = self._compress_side(value_states, S, P - W, tb.vc_list, tb.vn_list,
                                                                  st.v_unc[:, :st.n_mid, :Mn_v], dtype)
        st.k_coef, st.v_coef = k_coef, v_coef
        k_scale, v_scale = k_udev / k_idev, v_udev / v_idev             # cache_utils_fourier.py:567, 589
        if len(self.k_scale) == layer_idx:
            self.k_scale.append(k_scale); self.k_layer_average.append(k_ua); self.kd_layer_average.append(k_ia)
            self.v_scale.append(v_scale); self.v_layer_average.append(v_ua); self.vd_layer_average.append(v_ia)
        else:
            raise NotImplementedError("layers must be cached in order")
        st.stats32 = tuple(t.to(torch.float32).contiguous() for t in (k_ua, k_ia, k_scale, v_ua, v_ia, v_scale))
        owner = self.seq_shard is None or self.seq_shard[0] == 0      # the rank that attends sinks + window
        st.calls = ops.LayerCalls(st.kbuf, st.vbuf, st.k_unc, st.v_unc,
                                  k_coef if tb.kc_list.numel() else None, v_coef if tb.vc_list.numel() else None,
                                  st.stats32, tb, S, W, self.heads, self.attention_period, st.mid_l0,
                                  compress_period(self.attention_period), self.update_angle, with_il=owner)
        self.curr_tokennum[layer_idx] += n_mid                          # cache_utils_fourier.py:593
        return st

    def _views(self, st, layer_idx):
        S, W = self.numinittokens, self.maxlocallen
        tb = self._tables[layer_idx]
        Mn_k, Mn_v = tb.kn_list.numel(), tb.vn_list.numel()
        lo = S + st.off
        kd = {"k_init": st.kbuf[:, :S], "k_compressed": st.k_coef,
              "k_uncompressed": st.k_unc[:, :st.n_mid, :Mn_k], "k_local": st.kbuf[:, lo:lo + W]}
        vd = {"v_init": st.vbuf[:, :S], "v_compressed": st.v_coef,
              "v_uncompressed": st.v_unc[:, :st.n_mid, :Mn_v], "v_local": st.vbuf[:, lo:lo + W]}
        return kd, vd

    # ------------------------------------------------------------------------------------------
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[Dict[str, Any]] = None):
        """Add ``key_states``/``value_states`` ``(B, Hkv, q, D)`` of layer ``layer_idx``; returns the two dicts
        of the reference (cache_utils_fourier.py:494-750): only ``*_local`` is set while nothing is
        compressed (prefill, short prompts), all four entries in steady-state decode."""
        if not key_states.is_cuda:
            raise RuntimeError("fourierattention_b200.DynamicCache.update needs CUDA tensors")
        if layer_idx == 0:
            self._seen_tokens += key_states.shape[-2]
        self.heads = key_states.shape[1]
        self.head_dim = key_states.shape[-1]
        bsz, q_len = key_states.shape[0], key_states.shape[-2]
        F = self.heads * self.head_dim
        none_k = {"k_init": None, "k_compressed": None, "k_uncompressed": None}
        none_v = {"v_init": None, "v_compressed": None, "v_uncompressed": None}

        if len(self.key_cache) <= layer_idx:                      # first call for this layer
            if len(self.key_cache) < layer_idx:
                raise NotImplementedError("layers must be cached in order")
            ks = key_states.permute(0, 2, 1, 3).reshape(bsz, q_len, F)
            vs = value_states.permute(0, 2, 1, 3).reshape(bsz, q_len, F)
            if layer_idx == 0:
                self.prefilllen = q_len
                self.maxtokens = min(self.prefilllen + self.maxnewtokens, self.maxtokens)
            if q_len > self.maxlen:
                st = self._prefill_layer(ks, vs, layer_idx)
            else:                                                # never compressed (cache_utils_fourier.py:598-611)
                st = _LayerState()
                st.compressed = False
                cap = q_len + self.maxnewtokens + 8
                st.kbuf = torch.empty((bsz, cap, F), dtype=ks.dtype, device=ks.device)
                st.vbuf = torch.empty((bsz, cap, F), dtype=ks.dtype, device=ks.device)
                st.kbuf[:, :q_len].copy_(ks); st.vbuf[:, :q_len].copy_(vs)
                st.local_len = q_len
                st.n_mid = 0
            self._state.append(st)
            if st.compressed:
                kd, vd = self._views(st, layer_idx)
            else:
                tb = self._tables[layer_idx]
                e = lambda n: torch.empty((bsz, 0, n), dtype=ks.dtype, device=ks.device)
                kd = {"k_init": e(F), "k_compressed": e(tb.kc_list.numel()), "k_uncompressed": e(tb.kn_list.numel()),
                      "k_local": st.kbuf[:, :q_len]}
                vd = {"v_init": e(F), "v_compressed": e(tb.vc_list.numel()), "v_uncompressed": e(tb.vn_list.numel()),
                      "v_local": st.vbuf[:, :q_len]}
            self.key_cache.append(kd); self.value_cache.append(vd)
            return dict(none_k, k_local=ks), dict(none_v, v_local=vs)

        st = self._state[layer_idx]
        if not st.compressed:                                    # cache_utils_fourier.py:681-686
            if q_len != 1:
                raise ValueError("decode updates carry one token")
            n = st.local_len
            if n + 1 > st.kbuf.shape[1]:
                grow = lambda b: torch.cat([b, torch.empty_like(b)], dim=1)
                st.kbuf, st.vbuf = grow(st.kbuf), grow(st.vbuf)
            st.kbuf[:, n].copy_(key_states[:, :, 0].reshape(bsz, F))
            st.vbuf[:, n].copy_(value_states[:, :, 0].reshape(bsz, F))
            st.local_len = n + 1
            self.key_cache[layer_idx]["k_local"] = st.kbuf[:, :n + 1]
            self.value_cache[layer_idx]["v_local"] = st.vbuf[:, :n + 1]
            return dict(none_k, k_local=st.kbuf[:, :n + 1]), dict(none_v, v_local=st.vbuf[:, :n + 1])

        if q_len != 1:
            raise ValueError("decode updates carry one token")
        # The reference's branch test reads the batch size where the window length was meant
        # (cache_utils_fourier.py:680): with q_len = S + M + n_mid + B + 1 it appends to the window while
        # q_len <= maxlen (n_mid + B + 1 <= W), re-compresses when q_len == maxlen + 1 (n_mid + B == W) and
        # evicts otherwise.  Every practical configuration has n_mid + B > W and evicts.  At the boundary
        # n_mid + B == W the reference's re-compression appends a second cache entry for the layer and its
        # state is unusable afterwards; this cache evicts there too (the behaviour on either side of it),
        # and only the window-growth case below it is refused.
        n_mid_total = self.curr_tokennum[layer_idx]
        if n_mid_total + bsz + 1 <= self.maxlocallen:
            raise NotImplementedError("window growth after a compressed prefill (cache_utils_fourier.py:681-729) "
                                      "is not supported: it needs n_mid + batch + 1 <= maxlocallen")
        S, W = self.numinittokens, self.maxlocallen
        self.curr_tokennum[layer_idx] += 1                        # incremented before use (cache_utils_fourier.py:732)
        phase = self.curr_tokennum[layer_idx]
        appends = self.seq_shard is None or self.seq_shard[0] == self.seq_shard[1] - 1   # else another rank stores the row
        if appends and st.n_mid + 1 > st.k_unc.shape[1]:
            grow = lambda b: torch.cat([b, torch.zeros_like(b)], dim=1)
            st.k_unc, st.v_unc = grow(st.k_unc), grow(st.v_unc)
            st.calls.rebind(st.k_unc, st.v_unc)
        # eviction into the coefficients, verbatim append and window slide in one launch
        st.calls.step(st.off, st.n_mid if appends else 0, phase, key_states, value_states, appends)
        if appends:
            st.n_mid += 1
        st.off += 1
        if st.off == W:                                          # slide the window back to the front
            st.kbuf[:, S:S + W].copy_(st.kbuf[:, S + W:S + 2 * W])
            st.vbuf[:, S:S + W].copy_(st.vbuf[:, S + W:S + 2 * W])
            st.off = 0
        kd, vd = self._views(st, layer_idx)
        self.key_cache[layer_idx] = kd
        self.value_cache[layer_idx] = vd
        return dict(kd), dict(vd)

    # ------------------------------------------------------------------------------------------
    def fourier_attention(self, query, layer_idx: int, num_head_q: int, sm_scale: float = -1.0, phase_events=None):
        """Decode attention of one new token against the cached state of ``layer_idx``:
        the Fourier branch of the reference forward (modeling_llama_fourier.py:641-660) without the
        ``torch.cat`` of sinks and window.  ``query``: (B, 1, Hq*D) or (B, Hq*D).  Returns (B, Hq, 1, D)
        float32.  With a sequence split the partial results of all ranks are merged here."""
        st = self._state[layer_idx]
        if not st.compressed:
            raise RuntimeError("layer is not compressed; use dense attention on k_local / v_local")
        q = query if query.dim() == 2 else query[:, 0]
        B = q.shape[0]
        D = q.shape[1] // num_head_q
        if self.seq_shard is None:
            out = st.calls.attend(q, st.off, st.n_mid, num_head_q, sm_scale, phase_events)
            return out.view(B, num_head_q, 1, D)
        import torch.distributed as dist
        out, m, l = self.partial_attention(q, layer_idx, num_head_q, sm_scale)
        world = self.seq_shard[1]
        rows = B * num_head_q
        pack = torch.cat([out.view(rows, D), m.view(rows, 1), l.view(rows, 1)], dim=1)
        gathered = torch.empty((world,) + pack.shape, dtype=pack.dtype, device=pack.device)
        dist.all_gather_into_tensor(gathered, pack, group=self.process_group)
        merged = ops.merge(gathered[:, :, :D], gathered[:, :, D], gathered[:, :, D + 1])
        return merged.view(B, num_head_q, 1, D)

    def set_layer_statistics(self, layer_idx: int, stats32):
        """Make the attention kernels of ``layer_idx`` use these float32 statistics ``(k_layer_average,
        kd_layer_average, k_scale, v_layer_average, vd_layer_average, v_scale)``, each ``(B, Mc)`` (for
        instance statistics restored from a saved cache); the public per-layer lists are not touched."""
        st = self._state[layer_idx]
        st.stats32 = tuple(t.to(torch.float32).contiguous() for t in stats32)
        st.calls.set_statistics(st.stats32)

    def partial_attention(self, query, layer_idx: int, num_head_q: int, sm_scale: float = -1.0):
        """This rank's share of the attention under a sequence split: the output normalised over the keys the
        rank holds, ``(B, Hq, D)``, with the softmax statistics ``(m, l)``, each ``(B, Hq)`` (maximum score in
        the log2 domain, denominator relative to it), that the log-sum-exp merge needs
        (fourier_triton_valid4_v2.py:756-776).  A rank without any key returns ``l = 0``."""
        st = self._state[layer_idx]
        q = query if query.dim() == 2 else query[:, 0]
        return st.calls.attend(q, st.off, st.n_mid, num_head_q, sm_scale, return_lse=True)

    # ------------------------------------------------------------------------------------------
    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        """Cached sequence length (reference: cache_utils_fourier.py:752-761)."""
        if len(self.key_cache) <= layer_idx or len(self.key_cache[layer_idx]) == 0:
            return 0
        c = self.key_cache[layer_idx]
        return c["k_init"].shape[-2] + c["k_uncompressed"].shape[-2] + c["k_local"].shape[-2]

    def get_max_cache_shape(self) -> Optional[int]:
        return None
