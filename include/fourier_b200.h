/*
 * fourier_b200.h -- C ABI of the sm_100a kernels behind the Fourier-compressed KV cache.
 *
 * The reference (FourierAttention, fourier_attn_triton/) has no native interface: its device
 * code is Triton launched from Python.  Each entry point below therefore names the reference
 * Python function whose device work it replaces; "KM" is
 * fourier_attn_triton/fourier_triton_valid4_v2.py, "CU" is
 * fourier_attn_triton/cache_utils_fourier.py, "ML" is
 * fourier_attn_triton/modeling_llama_fourier.py.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host;
 *   - element strides are in ELEMENTS, not bytes;
 *   - "model dtype" tensors are fp16 or bf16 (fa_dtype_t); coefficients and statistics are fp32;
 *   - index tables are int32;
 *   - every call is asynchronous on `stream`, allocates nothing, never synchronises, and returns
 *     FA_OK or a negative fa_status_t; fa_last_error_string() describes the last failure of the
 *     calling thread;
 *   - coefficient layout (KM:68-78, KM:865): (B, 2N, Mc) fp32, rows 0..N-1 cosine sums, rows
 *     N..2N-1 sine sums.
 */
#ifndef FOURIER_B200_H
#define FOURIER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { FA_DTYPE_F16 = 0, FA_DTYPE_BF16 = 1 } fa_dtype_t;

typedef enum {
  FA_OK = 0,
  FA_ERR_NULL = -1,        /* a required pointer is null                       */
  FA_ERR_SHAPE = -2,       /* a size is non-positive or inconsistent            */
  FA_ERR_DTYPE = -3,       /* unknown fa_dtype_t                                */
  FA_ERR_ALIGN = -4,       /* a pointer or stride breaks a stated alignment     */
  FA_ERR_CAPACITY = -5,    /* the problem exceeds a stated maximum              */
  FA_ERR_CUDA = -6,        /* a CUDA runtime call failed                        */
  FA_ERR_UNSUPPORTED = -7  /* valid but not implemented for this configuration  */
} fa_status_t;

/* How the decode-time projection forms its angle.
 * FA_ANGLE_EXACT: 2*pi*((pos*n) mod T)/T with the phase reduced in integers.
 * FA_ANGLE_KM57 : fl32(fl32(fl32(c*pos)*n)/T), c = fl32(2*3.14159265359) -- the float32 roundings
 *                 of the reference projection kernel (KM:57), for parity of the rank-1 updates. */
typedef enum { FA_ANGLE_EXACT = 0, FA_ANGLE_KM57 = 1 } fa_angle_t;

typedef void* fa_stream_t; /* a cudaStream_t */

int fa_version(void);
const char* fa_last_error_string(void);

/* out[b,k,i] = x[b,k,idx[i]], i < n_idx, k < K.
 * Replaces the advanced-index gathers `k_mid[:, :, list]` of CU:560-561 / CU:578-579 and the
 * per-step `k_local[:, 0:1, list]` of CU:735 / CU:741. */
int fa_gather_cols(const void* x, int dtype, int B, int K, int64_t x_sb, int64_t x_sk,
                   const int32_t* idx, int n_idx, void* out, int64_t o_sb, int64_t o_sk,
                   fa_stream_t stream);

/* Column mean and one-sided maximum deviation over k < K of x[b,k,idx[m]] (idx may be null:
 * identity).  avg/dev: (B, Mc) fp32; the caller casts to the model dtype as KM:461 does.
 * Replaces mat_avg_std_triton (KM:433-461, kernel KM:332-430). */
int fa_colstats(const void* x, int dtype, int B, int K, int64_t x_sb, int64_t x_sk,
                const int32_t* idx, int Mc, float* avg, float* dev, fa_stream_t stream);

/* Forward projection of K rows onto N cosines + N sines of period T_c with phase offset k_start:
 *   coef[b,n,m]   (+)= sum_k x[b,k,idx[m]] cos(2 pi (k+k_start) n / T_c)
 *   coef[b,N+n,m] (+)= sum_k x[b,k,idx[m]] sin(2 pi (k+k_start) n / T_c)
 * x has x_cols valid columns per row (idx values < x_cols); idx may be null (identity, Mc == x_cols).
 * accumulate != 0 adds to coef.  scratch: device buffer of at least fa_compress_scratch_bytes(...) bytes,
 * 16-byte aligned (split-K partials, reduced in a fixed order).
 * Spans of 256 rows or more whose rows are 16-byte aligned (x 16-byte aligned, strides multiples of 8) run
 * on the tcgen05 tensor cores with TMA-staged tiles; the rest runs on CUDA cores.
 * Replaces the prefill FFT of MultiDimHiPPO2.forward (KM:857-865) and the general-K
 * mat_fourier_triton (KM:81-102, kernel KM:21-78). */
size_t fa_compress_scratch_bytes(int B, int K, int N, int Mc, int x_cols);
int fa_compress(const void* x, int dtype, int B, int K, int64_t x_sb, int64_t x_sk, int x_cols,
                const int32_t* idx, int Mc, int N, int T_c, int64_t k_start, float* coef,
                int accumulate, void* scratch, size_t scratch_bytes, fa_stream_t stream);

/* Decode-time rank-1 update for K and V in one launch (either side may be skipped with a null
 * coefficient pointer):  coef[b,n,m] += cos(angle(phase,n)) * row[b, idx[m]], sine rows likewise.
 * Replaces `base_input + mat_fourier_triton(slice_input, N, T_c, K_start=phase)` with K = 1
 * (KM:855-856; call sites CU:733, CU:739). */
int fa_evict_update(float* k_coef, const void* k_row, int64_t k_row_sb, const int32_t* k_idx, int Mc_k,
                    float* v_coef, const void* v_row, int64_t v_row_sb, const int32_t* v_idx, int Mc_v,
                    int dtype, int B, int N, int64_t phase, int T_c, int angle_mode,
                    fa_stream_t stream);

/* Statistics of the reconstructed span: x^[k,m] = (1/N) sum_n [coef[n,m] cos(2 pi k n/T) +
 * coef[N+n,m] sin(2 pi k n/T)], k < K;  avg = mean_k, dev = max(max_k - avg, avg - min_k).
 * Outputs (B, Mc) fp32; the caller casts to fp16 as KM:326 does.
 * scratch: at least fa_recon_stats_scratch_bytes(...) bytes.
 * Replaces mat_fourier_avg_std_triton (KM:285-326, kernel KM:189-282). */
size_t fa_recon_stats_scratch_bytes(int B, int K, int Mc);
int fa_recon_stats(const float* coef, int B, int N, int Mc, int K, int T, float* avg, float* dev,
                   void* scratch, size_t scratch_bytes, fa_stream_t stream);

/* Stand-alone inverse: out[m,k] = (1/N) sum_n [c[m,n] cos(2 pi k n/T) + c[m,N+n] sin(2 pi k n/T)].
 * c: (M, 2N) fp32 row-major, out: (M, K) fp32.  Replaces mat_fourier_inv_triton (KM:170-183). */
int fa_fourier_inverse(const float* c, int M, int N, int K, int T, float* out, fa_stream_t stream);

/* One steady-state cache step for K and V (CU:735-737, CU:741-743): the verbatim dims of the
 * evicted window row are appended to the uncompressed store and the new token row is written
 * behind the window.
 *   *_evict : (B, F) evicted row,   stride *_evict_sb
 *   *_unc   : (B, 1, Mn) destination row (already offset to the append position), stride *_unc_sb
 *   *_new   : new token, element (b, h, d) at b*new_sb + h*new_sh + d
 *   *_dst   : (B, F) destination row in the window buffer, stride *_dst_sb */
int fa_cache_step(const void* k_evict, const void* v_evict, int64_t evict_sb,
                  const int32_t* kn_idx, int Mn_k, const int32_t* vn_idx, int Mn_v,
                  void* k_unc, int64_t k_unc_sb, void* v_unc, int64_t v_unc_sb,
                  const void* k_new, const void* v_new, int64_t new_sb, int64_t new_sh,
                  void* k_dst, void* v_dst, int64_t dst_sb,
                  int dtype, int B, int Hkv, int D, fa_stream_t stream);

/* fa_evict_update and fa_cache_step of one decode step in a single launch (same arguments, same results:
 * the two touch disjoint memory).  No separate counterpart in the reference: it is the body of the
 * steady-state branch of DynamicCache.update (CU:732-743) as one call. */
int fa_evict_step(float* k_coef, const void* k_row, int64_t k_row_sb, const int32_t* k_idx, int Mc_k,
                  float* v_coef, const void* v_row, int64_t v_row_sb, const int32_t* v_idx, int Mc_v,
                  int N, int64_t phase, int T_c, int angle_mode,
                  const void* k_evict, const void* v_evict, int64_t evict_sb,
                  const int32_t* kn_idx, int Mn_k, const int32_t* vn_idx, int Mn_v,
                  void* k_unc, int64_t k_unc_sb, void* v_unc, int64_t v_unc_sb,
                  const void* k_new, const void* v_new, int64_t new_sb, int64_t new_sh,
                  void* k_dst, void* v_dst, int64_t dst_sb,
                  int dtype, int B, int Hkv, int D, fa_stream_t stream);

/* ---- fused decode attention over the compressed cache --------------------------------------
 * Replaces triton_fourier_attn (KM:684-779: kernel KM:470-681 plus the PyTorch split-KV merge
 * KM:756-776) and, in semantics, torch_fourier_attn (KM:794-837).  One query token per sequence.
 */
typedef struct {
  /* geometry */
  int32_t B, Hq, Hkv, D;
  int32_t n_sink, n_win; /* rows of the two verbatim segments ("k_init", "k_local")          */
  int32_t n_mid;         /* rows of the middle span held here (k_uncompressed.size(1))       */
  int32_t mid_l0;        /* span position of row 0 of k_mn/v_mn (0 unless the span is split
                            by sequence across devices)                                     */
  int32_t N;             /* cosine count; coefficients have 2N rows                          */
  int32_t T;             /* reconstruction period (ML:660)                                   */
  int32_t Mc_k, Mn_k, Mc_v, Mn_v;
  int32_t dtype;         /* fa_dtype_t of q, sinks, window and verbatim stores               */
  float sm_scale;        /* softmax scale; <= 0 selects 1/sqrt(D) (KM:696)                   */
  /* tensors */
  const void* q;         /* (B, Hq*D), stride q_sb                                           */
  int64_t q_sb;
  const void *k_sink, *v_sink; /* (B, n_sink, F) strides sink_sb, F                          */
  int64_t sink_sb;
  const void *k_win, *v_win;   /* (B, n_win, F) strides win_sb, F                            */
  int64_t win_sb;
  const void *k_mn, *v_mn;     /* (B, n_mid, Mn_*) batch strides *_mn_sb, row strides *_mn_sk  */
  int64_t k_mn_sb, v_mn_sb;
  int64_t k_mn_sk, v_mn_sk;    /* >= Mn_*; rows whose start is 16-byte aligned stream fastest   */
  const float *k_coef, *v_coef; /* (B, 2N, Mc_*) contiguous                                  */
  const float *avg_k_u, *avg_k_d, *scale_k; /* (B, Mc_k) contiguous fp32                     */
  const float *avg_v_u, *avg_v_d, *scale_v; /* (B, Mc_v) contiguous fp32                     */
  /* index tables (CU:444-452): flat dims and cumulative per-head offsets with leading 0      */
  const int32_t *kc_list, *kc_h, *kn_list, *kn_h, *vc_list, *vc_h, *vn_list, *vn_h;
  /* output */
  float* out;            /* (B, Hq, D) fp32 contiguous                                        */
  /* optional softmax statistics for a cross-device merge (fa_merge): per (b, h) the maximum
   * score in the log2 domain and the denominator relative to it                               */
  float* m_out;          /* (B, Hq) or null                                                   */
  float* l_out;          /* (B, Hq) or null                                                   */
  /* scratch */
  void* scratch;
  size_t scratch_bytes;
  /* optional profiling aid: a HOST array of five cudaEvent_t recorded on `stream` before the first
   * launch and after each launch (prepare, main; the third and fourth event both follow main, the fifth follows
   * finish); null = off, and a null entry of the array skips that record   */
  void* const* phase_events_host;
  /* optional HOST copies of kn_h and vn_h (Hkv + 1 entries each); with them the planner can check the
   * per-head column ranges and pick the warp-specialised middle-span pass; null = not given          */
  const int32_t* kn_h_host;
  const int32_t* vn_h_host;
} fa_decode_args_t;

/* Bytes of scratch fa_decode_attn needs for this geometry (only the size fields are read). */
size_t fa_decode_scratch_bytes(const fa_decode_args_t* args_host);
/* Which middle-span pass fa_decode_attn will run for these arguments (sizes, strides and pointer
 * alignment are read):
 *   3 = warp-specialised tensor-core pass with the spectral accumulator in tensor memory (tcgen05): the spectral
 *       score is evaluated at 16 nodes per 128-token super-tile and interpolated; the accumulator g and the
 *       query-side weights w live in tensor memory, g is updated by tcgen05.mma.  Needs what 2 needs and N <= 256,
 *       8 query heads per column tile (Hq / Hkv one of 1, 2, 4, 8), at most 64 verbatim-K and 64 verbatim-V columns
 *       per tile after rounding to 16, at most 256 verbatim columns per row, fewer than 40 KV heads.
 *   2 = the same pass with the accumulator in registers (mma.sync).  Needs N % 8 == 0, N <= 512, Hq <= 32,
 *       head_dim % 16 == 0, 16-byte aligned verbatim rows, at most 1.5 turns of the highest frequency per super-tile
 *       (128 (N - 1) <= 1.5 T), kn_h_host / vn_h_host, and per column tile of 8 (or 6) query heads at most 128
 *       verbatim-K and 128 verbatim-V columns after rounding to 16.  Above N = 256 the heads of a sequence are
 *       served in groups of 16 by different CTAs.
 *   1 = the same mathematics phase by phase (all warps together): N <= 256, Mn_* <= 256, 64- or 128-token
 *       super-tiles, no host tables needed.
 *   0 = exact CUDA-core pass (any shape).
 *   negative = fa_status_t.
 * Environment: FA_DECODE_EXACT forces 0, FA_DECODE_NO_WS keeps 2 and 3 from being chosen, FA_DECODE_NO_TMEM
 * keeps 3 from being chosen. */
int fa_decode_path(const fa_decode_args_t* args_host);
int fa_decode_attn(const fa_decode_args_t* args_host, fa_stream_t stream);

/* The same attention for hosts that cannot allocate device memory around the call.
 *
 * This entry point has no counterpart in the reference.  It exists for callers such as inference
 * servers that hand the whole HBM heap to their own page allocator at start-up, or code running where a
 * cudaMalloc (and the device-wide synchronisation it implies) is not allowed: they have nowhere to get
 * the scratch buffer fa_decode_attn asks for.  Here the scratch is a fixed array of
 * FA_DECODE_STATIC_SCRATCH_BYTES inside the library's own device image; args->scratch and
 * args->scratch_bytes are ignored, inputs and outputs are still the caller's.
 *
 *  - The call makes no cudaMalloc / cudaFree and uses no allocating library routine.
 *  - A problem whose plan needs more scratch than the array holds is refused with FA_ERR_CAPACITY
 *    (fa_decode_scratch_bytes() tells the need); the Llama-3.1-8B / 32k / batch-8 layer call needs
 *    18.4 MiB, a single 512k-token sequence with M = 1024 needs 33.6 MiB and is refused.
 *  - Every GPU that loads the library reserves the array until the process ends.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *    device current).  Make that first call outside any stream capture.
 *  - All calls on a device share the one array and it keeps whatever the last call left there.  Nothing
 *    has to be cleared between calls: every word a call reads was written earlier in that same call.  Two
 *    calls that overlap on the GPU (different streams, or graphs replayed concurrently) race on it; keep
 *    calls of this entry point ordered on one stream per device.
 *  - The looked-up address is kept per device for the life of the process; do not use this entry point
 *    across a cudaDeviceReset of that device. */
#define FA_DECODE_STATIC_SCRATCH_BYTES (24u << 20)
int fa_decode_attn_static(const fa_decode_args_t* args_host, fa_stream_t stream);

/* ---- layer handle: the per-step calls of one cached layer with everything static bound once --------
 * Replaces, per decode step and layer, the steady-state branch of DynamicCache.update (CU:731-748) and the
 * Fourier branch of LlamaSdpaAttention.forward (ML:641-660: the two torch.cat of sinks and window and the
 * call of triton_fourier_attn, KM:684-779).  The reference rebuilds every view and re-reads every attribute
 * on each step in Python; here the buffers, tables, statistics and tensor maps of a layer are bound when the
 * handle is made and a step passes integers only.
 *
 *   kbuf / vbuf : (B, buf_rows, Hkv*D) dense rows, batch stride buf_sb; rows [0, S) are the sinks, the
 *                 window is the W rows starting at row S + win_off (0 <= win_off <= W), a new token is
 *                 written at row S + win_off + W; buf_rows >= S + 2W.  Rows the window has not reached yet
 *                 must hold finite values (zeros).
 *   k_unc/v_unc : (B, unc_rows, Mn_*) verbatim stores over their whole capacity, row strides *_unc_sk, batch
 *                 strides *_unc_sb; rows [0, n_mid) are live, the rest must hold finite values (zeros).
 *   statistics, tables: as in fa_decode_args_t.  with_il = 0 leaves sinks and window to another rank
 *                 (sequence split).  mid_l0: span position of row 0 of the stores.
 * The planner switches FA_DECODE_EXACT / FA_DECODE_NO_WS are read when the handle is created. */
typedef struct fa_layer fa_layer_t;
typedef struct {
  int32_t B, Hkv, D, S, W, N, T, T_c, angle_mode, dtype, mid_l0;
  int32_t Mc_k, Mn_k, Mc_v, Mn_v;
  int32_t with_il;
  void *kbuf, *vbuf;
  int64_t buf_sb;
  int32_t buf_rows;
  void *k_unc, *v_unc;
  int64_t k_unc_sb, v_unc_sb, k_unc_sk, v_unc_sk;
  int32_t unc_rows;
  float *k_coef, *v_coef;
  const float *avg_k_u, *avg_k_d, *scale_k, *avg_v_u, *avg_v_d, *scale_v;
  const int32_t *kc_list, *kc_h, *kn_list, *kn_h, *vc_list, *vc_h, *vn_list, *vn_h;
  const int32_t *kn_h_host, *vn_h_host; /* HOST copies of kn_h / vn_h (Hkv + 1 entries), kept by the caller */
} fa_layer_desc_t;

int fa_layer_create(const fa_layer_desc_t* desc_host, fa_layer_t** out);
void fa_layer_destroy(fa_layer_t* layer);
/* the verbatim stores were reallocated (they grew) */
int fa_layer_rebind_stores(fa_layer_t* layer, void* k_unc, void* v_unc, int64_t k_unc_sb, int64_t v_unc_sb,
                           int64_t k_unc_sk, int64_t v_unc_sk, int32_t unc_rows);
/* One steady-state cache step (= fa_evict_step on the layer's buffers): the window row at offset win_off is
 * evicted -- its compressed dims go into the coefficients at `phase`, its verbatim dims to row n_mid of the
 * stores (appends != 0) -- and the new token (element (b, h, d) at b*new_sb + h*new_sh + d) is written
 * behind the window.  Afterwards the window starts at win_off + 1 and the span holds n_mid + 1 rows. */
int fa_layer_update(fa_layer_t* layer, int32_t win_off, int32_t n_mid, int64_t phase, int32_t appends,
                    const void* k_new, const void* v_new, int64_t new_sb, int64_t new_sh, fa_stream_t stream);
/* Scratch fa_layer_attend needs for Hq query heads at span length n_mid (constant while n_mid stays inside
 * one 128-token super-tile). */
size_t fa_layer_scratch_bytes(fa_layer_t* layer, int32_t Hq, int32_t n_mid);
/* Decode attention of one query token per sequence (= fa_decode_attn on the layer's state): q (B, Hq*D) with
 * batch stride q_sb, out (B, Hq, D) fp32, m_out / l_out (B, Hq) or null. */
int fa_layer_attend(fa_layer_t* layer, int32_t win_off, int32_t n_mid, int32_t Hq, const void* q, int64_t q_sb,
                    float sm_scale, float* out, float* m_out, float* l_out, void* scratch, size_t scratch_bytes,
                    void* const* phase_events_host, fa_stream_t stream);
/* middle-span pass the last plan of this layer chose (see fa_decode_path) */
int fa_layer_decode_path(fa_layer_t* layer);

/* Log-sum-exp merge of n_parts partial results (KM:756-776), e.g. one per device of a
 * sequence split:  out = sum_i o_i l_i 2^(m_i - m*) / sum_i l_i 2^(m_i - m*),
 * with o_i the NORMALISED partial outputs (rows, D), m_i/l_i (rows).  parts are stacked:
 * o: (n_parts, rows, D), m, l: (n_parts, rows). */
int fa_merge(const float* o, const float* m, const float* l, int n_parts, int rows, int D,
             float* out, fa_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FOURIER_B200_H */
