// Cache maintenance kernels: column gathers, the per-step window/verbatim update and the
// column statistics of the span that is about to be compressed.  All are HBM-bound byte movers.
#include "common.cuh"

namespace fa {

// out[b,k,i] = x[b,k,idx[i]]; one CTA per (row block, b); threads sweep the gathered columns so
// that writes are fully coalesced and reads hit each 32-byte sector of the source row once.
__global__ void gather_cols_kernel(const uint16_t* __restrict__ x, int K, int64_t x_sb, int64_t x_sk,
                                   const int32_t* __restrict__ idx, int n_idx, uint16_t* __restrict__ out,
                                   int64_t o_sb, int64_t o_sk, int rows_per_cta) {
  const int b = blockIdx.y;
  const int k0 = blockIdx.x * rows_per_cta;
  const int k1 = min(K, k0 + rows_per_cta);
  const uint16_t* xb = x + (int64_t)b * x_sb;
  uint16_t* ob = out + (int64_t)b * o_sb;
  for (int i = threadIdx.x; i < n_idx; i += blockDim.x) {
    const int c = idx[i];
    for (int k = k0; k < k1; ++k) ob[(int64_t)k * o_sk + i] = xb[(int64_t)k * x_sk + c];
  }
}

// One launch per layer step: grid.x = B, blockDim = 256.
template <typename T>
__global__ void cache_step_kernel(const T* __restrict__ k_evict, const T* __restrict__ v_evict, int64_t evict_sb,
                                  const int32_t* __restrict__ kn_idx, int Mn_k,
                                  const int32_t* __restrict__ vn_idx, int Mn_v,
                                  T* __restrict__ k_unc, int64_t k_unc_sb, T* __restrict__ v_unc, int64_t v_unc_sb,
                                  const T* __restrict__ k_new, const T* __restrict__ v_new, int64_t new_sb,
                                  int64_t new_sh, T* __restrict__ k_dst, T* __restrict__ v_dst, int64_t dst_sb,
                                  int Hkv, int D) {
  const int b = blockIdx.x;
  // (1) verbatim dims of the evicted row.  The evicted row and the destination row of the new
  // token are different rows of the window buffer, so the two phases do not alias.
  for (int i = threadIdx.x; i < Mn_k; i += blockDim.x)
    k_unc[(int64_t)b * k_unc_sb + i] = k_evict[(int64_t)b * evict_sb + kn_idx[i]];
  for (int i = threadIdx.x; i < Mn_v; i += blockDim.x)
    v_unc[(int64_t)b * v_unc_sb + i] = v_evict[(int64_t)b * evict_sb + vn_idx[i]];
  // (2) the new token, flattened head-major (CU:529-534)
  const int F = Hkv * D;
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    const int h = f / D, d = f - h * D;
    k_dst[(int64_t)b * dst_sb + f] = k_new[(int64_t)b * new_sb + (int64_t)h * new_sh + d];
    v_dst[(int64_t)b * dst_sb + f] = v_new[(int64_t)b * new_sb + (int64_t)h * new_sh + d];
  }
}

// Column statistics.  CTA = (32-column block, b); 8 warps take interleaved rows; lane = column.
// Sums are carried in double so the result does not depend on the row partition.
template <typename T>
__global__ void colstats_kernel(const T* __restrict__ x, int K, int64_t x_sb, int64_t x_sk,
                                const int32_t* __restrict__ idx, int Mc, float* __restrict__ avg,
                                float* __restrict__ dev) {
  constexpr int NW = 32;   // warps per CTA: the walk down the rows is bound by the loads in flight, so as many as fit
  __shared__ double s_sum[NW][32];
  __shared__ float s_max[NW][32];
  __shared__ float s_min[NW][32];
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int m = blockIdx.x * 32 + lane;
  const bool live = m < Mc;
  const int c = live ? (idx ? idx[m] : m) : 0;
  const T* xb = x + (int64_t)b * x_sb + c;
  double sum = 0.0;
  float mx = -INFINITY, mn = INFINITY;
  if (live) {
    // eight rows per trip: a warp has that many loads in flight instead of one (the walk is bound by latency, not by
    // bytes)
    constexpr int U = 8;
    int k = warp;
    for (; k + NW * (U - 1) < K; k += NW * U) {
      float v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = to_f32(xb[(int64_t)(k + NW * u) * x_sk]);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        sum += (double)v[u];
        mx = fmaxf(mx, v[u]);
        mn = fminf(mn, v[u]);
      }
    }
    for (; k < K; k += NW) {
      const float v = to_f32(xb[(int64_t)k * x_sk]);
      sum += (double)v;
      mx = fmaxf(mx, v);
      mn = fminf(mn, v);
    }
  }
  s_sum[warp][lane] = sum;
  s_max[warp][lane] = mx;
  s_min[warp][lane] = mn;
  __syncthreads();
  if (warp == 0 && live) {
    for (int w = 1; w < NW; ++w) {
      sum += s_sum[w][lane];
      mx = fmaxf(mx, s_max[w][lane]);
      mn = fminf(mn, s_min[w][lane]);
    }
    const float a = (float)(sum / (double)K);
    avg[(int64_t)b * Mc + m] = a;
    dev[(int64_t)b * Mc + m] = fmaxf(mx - a, a - mn);
  }
}

}  // namespace fa

using namespace fa;

extern "C" int fa_gather_cols(const void* x, int dtype, int B, int K, int64_t x_sb, int64_t x_sk,
                              const int32_t* idx, int n_idx, void* out, int64_t o_sb, int64_t o_sk,
                              fa_stream_t stream) {
  FA_REQUIRE(dtype == FA_DTYPE_F16 || dtype == FA_DTYPE_BF16, FA_ERR_DTYPE, "fa_gather_cols: bad dtype %d", dtype);
  FA_REQUIRE(B >= 0 && K >= 0 && n_idx >= 0, FA_ERR_SHAPE, "fa_gather_cols: negative size");
  if (B == 0 || K == 0 || n_idx == 0) return FA_OK;
  FA_REQUIRE(x && idx && out, FA_ERR_NULL, "fa_gather_cols: null pointer");
  const int rows = 16;
  dim3 grid(ceil_div(K, rows), B);
  gather_cols_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)x, K, x_sb, x_sk, idx, n_idx,
                                                             (uint16_t*)out, o_sb, o_sk, rows);
  FA_CHECK_LAUNCH("fa_gather_cols");
  return FA_OK;
}

extern "C" int fa_cache_step(const void* k_evict, const void* v_evict, int64_t evict_sb, const int32_t* kn_idx,
                             int Mn_k, const int32_t* vn_idx, int Mn_v, void* k_unc, int64_t k_unc_sb, void* v_unc,
                             int64_t v_unc_sb, const void* k_new, const void* v_new, int64_t new_sb, int64_t new_sh,
                             void* k_dst, void* v_dst, int64_t dst_sb, int dtype, int B, int Hkv, int D,
                             fa_stream_t stream) {
  FA_REQUIRE(dtype == FA_DTYPE_F16 || dtype == FA_DTYPE_BF16, FA_ERR_DTYPE, "fa_cache_step: bad dtype %d", dtype);
  FA_REQUIRE(B > 0 && Hkv > 0 && D > 0 && Mn_k >= 0 && Mn_v >= 0, FA_ERR_SHAPE, "fa_cache_step: bad sizes");
  FA_REQUIRE(k_evict && v_evict && k_new && v_new && k_dst && v_dst, FA_ERR_NULL, "fa_cache_step: null pointer");
  FA_REQUIRE((Mn_k == 0 || (kn_idx && k_unc)) && (Mn_v == 0 || (vn_idx && v_unc)), FA_ERR_NULL,
             "fa_cache_step: null verbatim table or store");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FA_DTYPE_F16)
    cache_step_kernel<__half><<<B, 256, 0, st>>>((const __half*)k_evict, (const __half*)v_evict, evict_sb, kn_idx,
                                                 Mn_k, vn_idx, Mn_v, (__half*)k_unc, k_unc_sb, (__half*)v_unc,
                                                 v_unc_sb, (const __half*)k_new, (const __half*)v_new, new_sb,
                                                 new_sh, (__half*)k_dst, (__half*)v_dst, dst_sb, Hkv, D);
  else
    cache_step_kernel<__nv_bfloat16><<<B, 256, 0, st>>>(
        (const __nv_bfloat16*)k_evict, (const __nv_bfloat16*)v_evict, evict_sb, kn_idx, Mn_k, vn_idx, Mn_v,
        (__nv_bfloat16*)k_unc, k_unc_sb, (__nv_bfloat16*)v_unc, v_unc_sb, (const __nv_bfloat16*)k_new,
        (const __nv_bfloat16*)v_new, new_sb, new_sh, (__nv_bfloat16*)k_dst, (__nv_bfloat16*)v_dst, dst_sb, Hkv, D);
  FA_CHECK_LAUNCH("fa_cache_step");
  return FA_OK;
}

extern "C" int fa_colstats(const void* x, int dtype, int B, int K, int64_t x_sb, int64_t x_sk, const int32_t* idx,
                           int Mc, float* avg, float* dev, fa_stream_t stream) {
  FA_REQUIRE(dtype == FA_DTYPE_F16 || dtype == FA_DTYPE_BF16, FA_ERR_DTYPE, "fa_colstats: bad dtype %d", dtype);
  FA_REQUIRE(B > 0 && K > 0 && Mc > 0, FA_ERR_SHAPE, "fa_colstats: B, K, Mc must be positive (got %d, %d, %d)", B, K,
             Mc);
  FA_REQUIRE(x && avg && dev, FA_ERR_NULL, "fa_colstats: null pointer");
  dim3 grid(ceil_div(Mc, 32), B);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FA_DTYPE_F16)
    colstats_kernel<__half><<<grid, 1024, 0, st>>>((const __half*)x, K, x_sb, x_sk, idx, Mc, avg, dev);
  else
    colstats_kernel<__nv_bfloat16><<<grid, 1024, 0, st>>>((const __nv_bfloat16*)x, K, x_sb, x_sk, idx, Mc, avg, dev);
  FA_CHECK_LAUNCH("fa_colstats");
  return FA_OK;
}
