// Spectral kernels of the cache: forward projection (compression), decode-time rank-1 update,
// statistics of the reconstructed span, stand-alone inverse.
//
// All phases are formed as (position * frequency) mod period in integers, so the basis keeps full
// float32 accuracy at any context length.  Accumulation is float32 over bounded chunks of the
// token axis; chunk partials are reduced in a fixed order.
#include <stdlib.h>

#include "common.cuh"

namespace fa {

// =====================================================================================
// forward projection:  coef[2N x Mc] (+)= Basis^T[2N x K] * X[K x Mc]
// CTA tile: 32 frequencies (32 cosine + 32 sine rows) x 64 columns, 32 tokens per inner step.
// =====================================================================================
constexpr int CP_NT = 32, CP_MT = 64, CP_KT = 32;

struct CompressPlan {
  int n_tiles, m_tiles, nsplit, kchunk;
};

static CompressPlan compress_plan(int B, int K, int N, int Mc) {
  CompressPlan p;
  p.n_tiles = ceil_div(N, CP_NT);
  p.m_tiles = ceil_div(Mc, CP_MT);
  const int64_t tiles = (int64_t)p.n_tiles * p.m_tiles * B;
  int want = (int)ceil_div64(4 * 148, tiles);
  int maxsplit = ceil_div(K, 256);
  int ns = want < 1 ? 1 : want;
  if (ns > maxsplit) ns = maxsplit;
  if (ns > 64) ns = 64;
  if (ns < 1) ns = 1;
  int kc = ceil_div(K, ns);
  kc = ceil_div(kc, CP_KT) * CP_KT;
  p.kchunk = kc;
  p.nsplit = ceil_div(K, kc);
  return p;
}

template <typename T>
__global__ void __launch_bounds__(256)
compress_kernel(const T* __restrict__ x, int K, int64_t x_sb, int64_t x_sk, const int32_t* __restrict__ idx, int Mc,
                int N, uint32_t T_c, uint64_t k_start, float* __restrict__ dst, int64_t dst_split_stride,
                int64_t dst_b_stride, int kchunk, int n_tiles, int add) {
  __shared__ __align__(16) float xs[CP_KT][CP_MT];
  __shared__ __align__(16) float fc[CP_KT][CP_NT];
  __shared__ __align__(16) float fs[CP_KT][CP_NT];
  const int tid = threadIdx.x;
  const int tile_n = blockIdx.x % n_tiles, tile_m = blockIdx.x / n_tiles;
  const int split = blockIdx.y, b = blockIdx.z;
  const int n0 = tile_n * CP_NT, m0 = tile_m * CP_MT;
  const int kbeg = split * kchunk, kend = min(K, kbeg + kchunk);
  const int ty = tid >> 4, tx = tid & 15;
  const float inv_T = 1.0f / (float)T_c;
  const T* xb = x + (int64_t)b * x_sb;

  // gathered source column of the (up to) 8 elements this thread stages per step
  int colsrc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = tid + 256 * i;
    const int mm = e % CP_MT;
    const int col = m0 + mm;
    colsrc[i] = (col < Mc) ? (idx ? idx[col] : col) : -1;
  }

  // two-level accumulation: running sums are folded into the totals every 512 tokens, which keeps
  // each float32 chain short however long the span is
  float ac[2][4], as[2][4], tc[2][4], ts[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) ac[i][j] = as[i][j] = tc[i][j] = ts[i][j] = 0.f;

  int fold = 0;
  for (int kt = kbeg; kt < kend; kt += CP_KT) {
    if (++fold == 17) {
      fold = 1;
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          tc[i][j] += ac[i][j];
          ts[i][j] += as[i][j];
          ac[i][j] = as[i][j] = 0.f;
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = tid + 256 * i;
      const int kk = e / CP_MT, mm = e % CP_MT;
      const int tok = kt + kk;
      float v = 0.f;
      if (tok < kend && colsrc[i] >= 0) v = to_f32(xb[(int64_t)tok * x_sk + colsrc[i]]);
      xs[kk][mm] = v;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + 256 * i;
      const int kk = e / CP_NT, nn = e % CP_NT;
      const uint32_t ph = phase_mod(k_start + (uint64_t)(kt + kk), (uint32_t)(n0 + nn), T_c);
      float s, c;
      sincos_phase(ph, inv_T, &s, &c);
      fc[kk][nn] = c;
      fs[kk][nn] = s;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < CP_KT; ++kk) {
      const float4 xv = *reinterpret_cast<const float4*>(&xs[kk][tx * 4]);
      const float2 c2 = *reinterpret_cast<const float2*>(&fc[kk][ty * 2]);
      const float2 s2 = *reinterpret_cast<const float2*>(&fs[kk][ty * 2]);
      const float xa[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        ac[0][j] = fmaf(c2.x, xa[j], ac[0][j]);
        ac[1][j] = fmaf(c2.y, xa[j], ac[1][j]);
        as[0][j] = fmaf(s2.x, xa[j], as[0][j]);
        as[1][j] = fmaf(s2.y, xa[j], as[1][j]);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      ac[i][j] += tc[i][j];
      as[i][j] += ts[i][j];
    }
  float* d = dst + (int64_t)split * dst_split_stride + (int64_t)b * dst_b_stride;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int n = n0 + ty * 2 + i;
    if (n >= N) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = m0 + tx * 4 + j;
      if (col >= Mc) continue;
      float* pc = d + (int64_t)n * Mc + col;
      float* ps = d + (int64_t)(N + n) * Mc + col;
      *pc = add ? *pc + ac[i][j] : ac[i][j];
      *ps = add ? *ps + as[i][j] : as[i][j];
    }
  }
}

// coef = (accumulate ? coef : 0) + sum_split partial[split], splits added in index order
__global__ void compress_reduce_kernel(const float* __restrict__ part, int nsplit, int64_t split_stride,
                                       float* __restrict__ coef, int64_t total, int accumulate) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float a = accumulate ? coef[i] : 0.f;
  for (int s = 0; s < nsplit; ++s) a += part[(int64_t)s * split_stride + i];
  coef[i] = a;
}

// =====================================================================================
// rank-1 update at decode time, K and V in one launch (blockIdx.z selects the side)
// =====================================================================================
constexpr int EV_ROWS = 4;

// the window slide / verbatim append of one decode step (what cache_step_kernel does), carried along by
// the eviction kernel's third grid slice when the two are launched together
struct StepArgs {
  const void *k_evict, *v_evict, *k_new, *v_new;
  const int32_t *kn_idx, *vn_idx;
  void *k_unc, *v_unc, *k_dst, *v_dst;
  int64_t evict_sb, k_unc_sb, v_unc_sb, new_sb, new_sh, dst_sb;
  int Mn_k, Mn_v, Hkv, D;
};

template <typename T>
__device__ void cache_step_body(const StepArgs& s, int b, int t0, int nthreads) {
  const T* k_evict = reinterpret_cast<const T*>(s.k_evict);
  const T* v_evict = reinterpret_cast<const T*>(s.v_evict);
  T* k_unc = reinterpret_cast<T*>(s.k_unc);
  T* v_unc = reinterpret_cast<T*>(s.v_unc);
  for (int i = t0; i < s.Mn_k; i += nthreads) k_unc[(int64_t)b * s.k_unc_sb + i] = k_evict[(int64_t)b * s.evict_sb + s.kn_idx[i]];
  for (int i = t0; i < s.Mn_v; i += nthreads) v_unc[(int64_t)b * s.v_unc_sb + i] = v_evict[(int64_t)b * s.evict_sb + s.vn_idx[i]];
  const T* k_new = reinterpret_cast<const T*>(s.k_new);
  const T* v_new = reinterpret_cast<const T*>(s.v_new);
  T* k_dst = reinterpret_cast<T*>(s.k_dst);
  T* v_dst = reinterpret_cast<T*>(s.v_dst);
  const int F = s.Hkv * s.D;
  for (int f = t0; f < F; f += nthreads) {
    const int h = f / s.D, d = f - h * s.D;
    k_dst[(int64_t)b * s.dst_sb + f] = k_new[(int64_t)b * s.new_sb + (int64_t)h * s.new_sh + d];
    v_dst[(int64_t)b * s.dst_sb + f] = v_new[(int64_t)b * s.new_sb + (int64_t)h * s.new_sh + d];
  }
}

template <typename T>
__global__ void evict_update_kernel(float* __restrict__ k_coef, const T* __restrict__ k_row, int64_t k_row_sb,
                                    const int32_t* __restrict__ k_idx, int Mc_k, float* __restrict__ v_coef,
                                    const T* __restrict__ v_row, int64_t v_row_sb, const int32_t* __restrict__ v_idx,
                                    int Mc_v, int N, uint64_t phase, uint32_t T_c, int angle_mode, StepArgs step) {
  const int side = blockIdx.z, b = blockIdx.y;
  if (side == 2) {   // only launched together with a cache step: the CTAs of this slice share its work
    cache_step_body<T>(step, b, blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x);
    return;
  }
  float* coef = side ? v_coef : k_coef;
  if (coef == nullptr) return;
  const T* row = (side ? v_row + (int64_t)b * v_row_sb : k_row + (int64_t)b * k_row_sb);
  const int32_t* idx = side ? v_idx : k_idx;
  const int Mc = side ? Mc_v : Mc_k;
  const int n0 = blockIdx.x * EV_ROWS;
  float c[EV_ROWS], s[EV_ROWS];
#pragma unroll
  for (int r = 0; r < EV_ROWS; ++r) {
    const int n = n0 + r;
    if (angle_mode == FA_ANGLE_KM57) {
      const float a = km57_angle((float)phase, (float)n, (float)T_c);
      c[r] = cosf(a);
      s[r] = sinf(a);
    } else {
      sincos_phase(phase_mod(phase, (uint32_t)n, T_c), 1.0f / (float)T_c, &s[r], &c[r]);
    }
  }
  float* cb = coef + (int64_t)b * 2 * N * Mc;
  if ((Mc & 3) == 0 && (reinterpret_cast<uintptr_t>(cb) & 15) == 0) {
    // four columns per thread: every load of the update is requested before the first value is used, so a CTA
    // pays one trip to memory instead of one per row (same arithmetic per element)
    for (int m = 4 * threadIdx.x; m < Mc; m += 4 * blockDim.x) {
      float xv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) xv[j] = to_f32(row[idx ? idx[m + j] : m + j]);
      float4 vc[EV_ROWS], vs[EV_ROWS];
#pragma unroll
      for (int r = 0; r < EV_ROWS; ++r) {
        const int n = n0 + r;
        if (n < N) {
          vc[r] = *reinterpret_cast<const float4*>(cb + (int64_t)n * Mc + m);
          vs[r] = *reinterpret_cast<const float4*>(cb + (int64_t)(N + n) * Mc + m);
        }
      }
#pragma unroll
      for (int r = 0; r < EV_ROWS; ++r) {
        const int n = n0 + r;
        if (n < N) {
          // one rounding per term, as `base + increment` of the reference (KM:856)
          float4 oc, os;
          oc.x = __fadd_rn(vc[r].x, __fmul_rn(c[r], xv[0]));
          oc.y = __fadd_rn(vc[r].y, __fmul_rn(c[r], xv[1]));
          oc.z = __fadd_rn(vc[r].z, __fmul_rn(c[r], xv[2]));
          oc.w = __fadd_rn(vc[r].w, __fmul_rn(c[r], xv[3]));
          os.x = __fadd_rn(vs[r].x, __fmul_rn(s[r], xv[0]));
          os.y = __fadd_rn(vs[r].y, __fmul_rn(s[r], xv[1]));
          os.z = __fadd_rn(vs[r].z, __fmul_rn(s[r], xv[2]));
          os.w = __fadd_rn(vs[r].w, __fmul_rn(s[r], xv[3]));
          *reinterpret_cast<float4*>(cb + (int64_t)n * Mc + m) = oc;
          *reinterpret_cast<float4*>(cb + (int64_t)(N + n) * Mc + m) = os;
        }
      }
    }
    return;
  }
  for (int m = threadIdx.x; m < Mc; m += blockDim.x) {
    const float xv = to_f32(row[idx ? idx[m] : m]);
#pragma unroll
    for (int r = 0; r < EV_ROWS; ++r) {
      const int n = n0 + r;
      if (n < N) {
        // one rounding per term, as `base + increment` of the reference (KM:856)
        cb[(int64_t)n * Mc + m] = __fadd_rn(cb[(int64_t)n * Mc + m], __fmul_rn(c[r], xv));
        cb[(int64_t)(N + n) * Mc + m] = __fadd_rn(cb[(int64_t)(N + n) * Mc + m], __fmul_rn(s[r], xv));
      }
    }
  }
}

// =====================================================================================
// statistics of the reconstructed span: X^[K x Mc] = (1/N) Basis[K x 2N] * coef[2N x Mc],
// reduced over rows to sum / max / min per column.  CTA tile 64 rows x 64 columns.
// =====================================================================================
constexpr int RS_KT = 64, RS_MT = 64, RS_NT = 16;

struct ReconPlan {
  int m_tiles, nchunk, kchunk;
};

static ReconPlan recon_plan(int B, int K, int Mc) {
  ReconPlan p;
  p.m_tiles = ceil_div(Mc, RS_MT);
  int want = (int)ceil_div64(4 * 148, (int64_t)p.m_tiles * B);
  int maxc = ceil_div(K, RS_KT);
  int nc = want < 1 ? 1 : want;
  if (nc > maxc) nc = maxc;
  int kc = ceil_div(K, nc);
  kc = ceil_div(kc, RS_KT) * RS_KT;
  p.kchunk = kc;
  p.nchunk = ceil_div(K, kc);
  return p;
}

__global__ void __launch_bounds__(256)
recon_stats_kernel(const float* __restrict__ coef, int N, int Mc, int K, uint32_t T, float* __restrict__ part,
                   int kchunk, int nchunk) {
  __shared__ __align__(16) float bc[RS_NT][RS_KT];
  __shared__ __align__(16) float bs[RS_NT][RS_KT];
  __shared__ __align__(16) float cc[RS_NT][RS_MT];
  __shared__ __align__(16) float cs[RS_NT][RS_MT];
  __shared__ float r_sum[16][RS_MT];
  __shared__ float r_max[16][RS_MT];
  __shared__ float r_min[16][RS_MT];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int m0 = blockIdx.x * RS_MT, chunk = blockIdx.y, b = blockIdx.z;
  const int kbeg = chunk * kchunk, kend = min(K, kbeg + kchunk);
  const float inv_T = 1.0f / (float)T, inv_N = 1.0f / (float)N;
  const float* cb = coef + (int64_t)b * 2 * N * Mc;

  float csum[4] = {0.f, 0.f, 0.f, 0.f};
  float cmax[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  float cmin[4] = {INFINITY, INFINITY, INFINITY, INFINITY};

  for (int kt = kbeg; kt < kend; kt += RS_KT) {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int nb = 0; nb < N; nb += RS_NT) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = tid + 256 * i;
        const int nn = e / RS_MT, mm = e % RS_MT;
        const int n = nb + nn, col = m0 + mm;
        const bool ok = (n < N) && (col < Mc);
        cc[nn][mm] = ok ? cb[(int64_t)n * Mc + col] : 0.f;
        cs[nn][mm] = ok ? cb[(int64_t)(N + n) * Mc + col] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = tid + 256 * i;
        const int nn = e / RS_KT, kk = e % RS_KT;
        float s, c;
        sincos_phase(phase_mod((uint64_t)(kt + kk), (uint32_t)(nb + nn), T), inv_T, &s, &c);
        bc[nn][kk] = c;
        bs[nn][kk] = s;
      }
      __syncthreads();
#pragma unroll 4
      for (int nn = 0; nn < RS_NT; ++nn) {
        const float4 b4 = *reinterpret_cast<const float4*>(&bc[nn][ty * 4]);
        const float4 s4 = *reinterpret_cast<const float4*>(&bs[nn][ty * 4]);
        const float4 c4 = *reinterpret_cast<const float4*>(&cc[nn][tx * 4]);
        const float4 d4 = *reinterpret_cast<const float4*>(&cs[nn][tx * 4]);
        const float ba[4] = {b4.x, b4.y, b4.z, b4.w}, sa[4] = {s4.x, s4.y, s4.z, s4.w};
        const float ca[4] = {c4.x, c4.y, c4.z, c4.w}, da[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ba[i], ca[j], fmaf(sa[i], da[j], acc[i][j]));
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = kt + ty * 4 + i;
      if (k < kend) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float v = acc[i][j] * inv_N;
          csum[j] += v;
          cmax[j] = fmaxf(cmax[j], v);
          cmin[j] = fminf(cmin[j], v);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    r_sum[ty][tx * 4 + j] = csum[j];
    r_max[ty][tx * 4 + j] = cmax[j];
    r_min[ty][tx * 4 + j] = cmin[j];
  }
  __syncthreads();
  if (tid < RS_MT) {
    const int col = m0 + tid;
    if (col < Mc) {
      float s = 0.f, mx = -INFINITY, mn = INFINITY;
      for (int r = 0; r < 16; ++r) {
        s += r_sum[r][tid];
        mx = fmaxf(mx, r_max[r][tid]);
        mn = fminf(mn, r_min[r][tid]);
      }
      float* p = part + ((int64_t)(b * nchunk + chunk) * 3) * Mc;
      p[col] = s;
      p[Mc + col] = mx;
      p[2 * Mc + col] = mn;
    }
  }
}

__global__ void recon_finalize_kernel(const float* __restrict__ part, int nchunk, int Mc, int K,
                                      float* __restrict__ avg, float* __restrict__ dev) {
  const int b = blockIdx.y;
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= Mc) return;
  double s = 0.0;
  float mx = -INFINITY, mn = INFINITY;
  for (int c = 0; c < nchunk; ++c) {
    const float* p = part + ((int64_t)(b * nchunk + c) * 3) * Mc;
    s += (double)p[col];
    mx = fmaxf(mx, p[Mc + col]);
    mn = fminf(mn, p[2 * Mc + col]);
  }
  const float a = (float)(s / (double)K);
  avg[(int64_t)b * Mc + col] = a;
  dev[(int64_t)b * Mc + col] = fmaxf(mx - a, a - mn);
}

#include "recon_interp.cuh"

// stand-alone inverse; one thread per output element (an API-completeness path, not a hot one)
__global__ void fourier_inverse_kernel(const float* __restrict__ c, int N, int K, uint32_t T, float* __restrict__ out) {
  const int m = blockIdx.y;
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= K) return;
  const float* cm = c + (int64_t)m * 2 * N;
  const float inv_T = 1.0f / (float)T;
  float acc = 0.f;
  for (int n = 0; n < N; ++n) {
    float s, co;
    sincos_phase(phase_mod((uint64_t)k, (uint32_t)n, T), inv_T, &s, &co);
    acc = fmaf(cm[n], co, fmaf(cm[N + n], s, acc));
  }
  out[(int64_t)m * K + k] = acc / (float)N;
}

}  // namespace fa

using namespace fa;

static size_t simt_compress_scratch_bytes(int B, int K, int N, int Mc) {
  CompressPlan p = compress_plan(B, K, N, Mc);
  if (p.nsplit <= 1) return 0;
  return (size_t)p.nsplit * B * 2 * N * Mc * sizeof(float);
}

extern "C" size_t fa_compress_scratch_bytes(int B, int K, int N, int Mc, int x_cols) {
  if (B <= 0 || K <= 0 || N <= 0 || Mc <= 0) return 0;
  // the caller cannot know which path the alignment of x will select: size for the larger one
  const size_t a = simt_compress_scratch_bytes(B, K, N, Mc);
  const size_t b = (K >= 256 && x_cols > 0) ? compress_tc_scratch_bytes(B, K, N, x_cols) : 0;
  return a > b ? a : b;
}

extern "C" int fa_compress(const void* x, int dtype, int B, int K, int64_t x_sb, int64_t x_sk, int x_cols,
                           const int32_t* idx, int Mc, int N, int T_c, int64_t k_start, float* coef, int accumulate,
                           void* scratch, size_t scratch_bytes, fa_stream_t stream) {
  FA_REQUIRE(dtype == FA_DTYPE_F16 || dtype == FA_DTYPE_BF16, FA_ERR_DTYPE, "fa_compress: bad dtype %d", dtype);
  FA_REQUIRE(B > 0 && K > 0 && N > 0 && Mc > 0 && T_c > 0 && k_start >= 0 && x_cols > 0, FA_ERR_SHAPE,
             "fa_compress: B, K, N, Mc, T_c, x_cols must be positive (got %d, %d, %d, %d, %d, %d)", B, K, N, Mc, T_c,
             x_cols);
  FA_REQUIRE(idx != nullptr || Mc == x_cols, FA_ERR_SHAPE, "fa_compress: without an index list Mc must equal x_cols");
  FA_REQUIRE(x && coef, FA_ERR_NULL, "fa_compress: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  if (compress_tc_usable(x, B, K, x_sb, x_sk, x_cols, N))
    return compress_tc_launch(x, dtype, B, K, x_sb, x_sk, x_cols, idx, Mc, N, T_c, k_start, coef, accumulate, scratch,
                              scratch_bytes, st);
  CompressPlan p = compress_plan(B, K, N, Mc);
  const size_t need = simt_compress_scratch_bytes(B, K, N, Mc);
  FA_REQUIRE(need == 0 || (scratch && scratch_bytes >= need), FA_ERR_CAPACITY,
             "fa_compress: scratch too small (%zu < %zu bytes)", scratch_bytes, need);
  const int64_t per_b = (int64_t)2 * N * Mc;
  // a single split writes (or adds to) the coefficients directly; several splits go through
  // scratch partials and a fixed-order reduction
  const bool direct = (p.nsplit == 1);
  float* dst = direct ? coef : (float*)scratch;
  const int add = (direct && accumulate) ? 1 : 0;
  dim3 grid(p.n_tiles * p.m_tiles, p.nsplit, B);
  const int64_t split_stride = (int64_t)B * per_b;
  if (dtype == FA_DTYPE_F16)
    compress_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, K, x_sb, x_sk, idx, Mc, N, (uint32_t)T_c,
                                                  (uint64_t)k_start, dst, split_stride, per_b, p.kchunk, p.n_tiles, add);
  else
    compress_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, K, x_sb, x_sk, idx, Mc, N,
                                                         (uint32_t)T_c, (uint64_t)k_start, dst, split_stride, per_b,
                                                         p.kchunk, p.n_tiles, add);
  FA_CHECK_LAUNCH("fa_compress");
  if (!direct) {
    const int64_t total = (int64_t)B * per_b;
    compress_reduce_kernel<<<(unsigned)ceil_div64(total, 256), 256, 0, st>>>((const float*)scratch, p.nsplit,
                                                                            split_stride, coef, total, accumulate);
    FA_CHECK_LAUNCH("fa_compress(reduce)");
  }
  return FA_OK;
}

extern "C" int fa_evict_update(float* k_coef, const void* k_row, int64_t k_row_sb, const int32_t* k_idx, int Mc_k,
                               float* v_coef, const void* v_row, int64_t v_row_sb, const int32_t* v_idx, int Mc_v,
                               int dtype, int B, int N, int64_t phase, int T_c, int angle_mode, fa_stream_t stream) {
  FA_REQUIRE(dtype == FA_DTYPE_F16 || dtype == FA_DTYPE_BF16, FA_ERR_DTYPE, "fa_evict_update: bad dtype %d", dtype);
  FA_REQUIRE(B > 0 && N > 0 && T_c > 0 && phase >= 0, FA_ERR_SHAPE, "fa_evict_update: bad sizes");
  FA_REQUIRE(angle_mode == FA_ANGLE_EXACT || angle_mode == FA_ANGLE_KM57, FA_ERR_SHAPE,
             "fa_evict_update: bad angle mode %d", angle_mode);
  FA_REQUIRE(!k_coef || (k_row && Mc_k > 0), FA_ERR_NULL, "fa_evict_update: K side incomplete");
  FA_REQUIRE(!v_coef || (v_row && Mc_v > 0), FA_ERR_NULL, "fa_evict_update: V side incomplete");
  if (!k_coef && !v_coef) return FA_OK;
  dim3 grid(ceil_div(N, EV_ROWS), B, 2);
  cudaStream_t st = (cudaStream_t)stream;
  const StepArgs none = {};
  if (dtype == FA_DTYPE_F16)
    evict_update_kernel<__half><<<grid, 256, 0, st>>>(k_coef, (const __half*)k_row, k_row_sb, k_idx, Mc_k, v_coef,
                                                      (const __half*)v_row, v_row_sb, v_idx, Mc_v, N,
                                                      (uint64_t)phase, (uint32_t)T_c, angle_mode, none);
  else
    evict_update_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        k_coef, (const __nv_bfloat16*)k_row, k_row_sb, k_idx, Mc_k, v_coef, (const __nv_bfloat16*)v_row, v_row_sb,
        v_idx, Mc_v, N, (uint64_t)phase, (uint32_t)T_c, angle_mode, none);
  FA_CHECK_LAUNCH("fa_evict_update");
  return FA_OK;
}

extern "C" int fa_evict_step(float* k_coef, const void* k_row, int64_t k_row_sb, const int32_t* k_idx, int Mc_k,
                             float* v_coef, const void* v_row, int64_t v_row_sb, const int32_t* v_idx, int Mc_v, int N,
                             int64_t phase, int T_c, int angle_mode, const void* k_evict, const void* v_evict,
                             int64_t evict_sb, const int32_t* kn_idx, int Mn_k, const int32_t* vn_idx, int Mn_v,
                             void* k_unc, int64_t k_unc_sb, void* v_unc, int64_t v_unc_sb, const void* k_new,
                             const void* v_new, int64_t new_sb, int64_t new_sh, void* k_dst, void* v_dst,
                             int64_t dst_sb, int dtype, int B, int Hkv, int D, fa_stream_t stream) {
  FA_REQUIRE(dtype == FA_DTYPE_F16 || dtype == FA_DTYPE_BF16, FA_ERR_DTYPE, "fa_evict_step: bad dtype %d", dtype);
  FA_REQUIRE(B > 0 && N > 0 && T_c > 0 && phase >= 0 && Hkv > 0 && D > 0 && Mn_k >= 0 && Mn_v >= 0, FA_ERR_SHAPE,
             "fa_evict_step: bad sizes");
  FA_REQUIRE(angle_mode == FA_ANGLE_EXACT || angle_mode == FA_ANGLE_KM57, FA_ERR_SHAPE,
             "fa_evict_step: bad angle mode %d", angle_mode);
  FA_REQUIRE(!k_coef || (k_row && Mc_k > 0), FA_ERR_NULL, "fa_evict_step: K side incomplete");
  FA_REQUIRE(!v_coef || (v_row && Mc_v > 0), FA_ERR_NULL, "fa_evict_step: V side incomplete");
  FA_REQUIRE(k_evict && v_evict && k_new && v_new && k_dst && v_dst, FA_ERR_NULL, "fa_evict_step: null row pointer");
  FA_REQUIRE((Mn_k == 0 || (kn_idx && k_unc)) && (Mn_v == 0 || (vn_idx && v_unc)), FA_ERR_NULL,
             "fa_evict_step: null verbatim store or index list");
  StepArgs sa;
  sa.k_evict = k_evict; sa.v_evict = v_evict; sa.k_new = k_new; sa.v_new = v_new;
  sa.kn_idx = kn_idx; sa.vn_idx = vn_idx;
  sa.k_unc = k_unc; sa.v_unc = v_unc; sa.k_dst = k_dst; sa.v_dst = v_dst;
  sa.evict_sb = evict_sb; sa.k_unc_sb = k_unc_sb; sa.v_unc_sb = v_unc_sb; sa.new_sb = new_sb; sa.new_sh = new_sh;
  sa.dst_sb = dst_sb; sa.Mn_k = Mn_k; sa.Mn_v = Mn_v; sa.Hkv = Hkv; sa.D = D;
  dim3 grid(ceil_div(N, EV_ROWS), B, 3);   // slices 0 / 1: K / V coefficients, slice 2: the cache step
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FA_DTYPE_F16)
    evict_update_kernel<__half><<<grid, 256, 0, st>>>(k_coef, (const __half*)k_row, k_row_sb, k_idx, Mc_k, v_coef,
                                                      (const __half*)v_row, v_row_sb, v_idx, Mc_v, N,
                                                      (uint64_t)phase, (uint32_t)T_c, angle_mode, sa);
  else
    evict_update_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        k_coef, (const __nv_bfloat16*)k_row, k_row_sb, k_idx, Mc_k, v_coef, (const __nv_bfloat16*)v_row, v_row_sb,
        v_idx, Mc_v, N, (uint64_t)phase, (uint32_t)T_c, angle_mode, sa);
  FA_CHECK_LAUNCH("fa_evict_step");
  return FA_OK;
}

// chunks of super-tiles per (column tile, sequence) of the interpolating kernel; depends on the sizes only,
// so that the scratch query does not need N and T
static int recon_interp_chunks(int B, int K, int Mc) {
  const int64_t tiles = (int64_t)ceil_div(Mc, RI_CT) * B;
  int want = (int)ceil_div64(2 * 148, tiles);
  const int maxc = ceil_div(K, 128);
  if (want < 1) want = 1;
  if (want > maxc) want = maxc;
  return want;
}

extern "C" size_t fa_recon_stats_scratch_bytes(int B, int K, int Mc) {
  if (B <= 0 || K <= 0 || Mc <= 0) return 0;
  ReconPlan p = recon_plan(B, K, Mc);
  const int nc = recon_interp_chunks(B, K, Mc);
  return (size_t)B * (p.nchunk > nc ? p.nchunk : nc) * 3 * Mc * sizeof(float);
}

extern "C" int fa_recon_stats(const float* coef, int B, int N, int Mc, int K, int T, float* avg, float* dev,
                              void* scratch, size_t scratch_bytes, fa_stream_t stream) {
  FA_REQUIRE(B > 0 && N > 0 && Mc > 0 && K > 0 && T > 0, FA_ERR_SHAPE,
             "fa_recon_stats: B, N, Mc, K, T must be positive (got %d, %d, %d, %d, %d)", B, N, Mc, K, T);
  FA_REQUIRE(coef && avg && dev && scratch, FA_ERR_NULL, "fa_recon_stats: null pointer");
  ReconPlan p = recon_plan(B, K, Mc);
  const size_t need = fa_recon_stats_scratch_bytes(B, K, Mc);
  FA_REQUIRE(scratch_bytes >= need, FA_ERR_CAPACITY, "fa_recon_stats: scratch too small (%zu < %zu bytes)",
             scratch_bytes, need);
  cudaStream_t st = (cudaStream_t)stream;
  // interpolating kernel: needs at most 1.5 turns of the highest frequency per 128- or 64-token super-tile
  int J = 0;
  if ((int64_t)128 * (N - 1) * 2 <= (int64_t)3 * T) J = 128;
  else if ((int64_t)64 * (N - 1) * 2 <= (int64_t)3 * T) J = 64;
  int nchunk = p.nchunk;
  if (J > 0 && N <= 256 && getenv("FA_RECON_DIRECT") == nullptr) {
    nchunk = recon_interp_chunks(B, K, Mc);
    const int nst = ceil_div(K, J);
    const int spc = ceil_div(nst, nchunk);
    nchunk = ceil_div(nst, spc);
    const int smem = ri_smem(N, J).total;
    dim3 grid(ceil_div(Mc, RI_CT), nchunk, B);
    if (J == 128) {
      cudaError_t e = cudaFuncSetAttribute(recon_stats_interp_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");
      recon_stats_interp_kernel<128><<<grid, RI_T, smem, st>>>(coef, N, Mc, K, (uint32_t)T, (float*)scratch, spc, nchunk);
    } else {
      cudaError_t e = cudaFuncSetAttribute(recon_stats_interp_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");
      recon_stats_interp_kernel<64><<<grid, RI_T, smem, st>>>(coef, N, Mc, K, (uint32_t)T, (float*)scratch, spc, nchunk);
    }
  } else {
    dim3 grid(p.m_tiles, p.nchunk, B);
    recon_stats_kernel<<<grid, 256, 0, st>>>(coef, N, Mc, K, (uint32_t)T, (float*)scratch, p.kchunk, p.nchunk);
  }
  FA_CHECK_LAUNCH("fa_recon_stats");
  dim3 g2(ceil_div(Mc, 128), B);
  recon_finalize_kernel<<<g2, 128, 0, st>>>((const float*)scratch, nchunk, Mc, K, avg, dev);
  FA_CHECK_LAUNCH("fa_recon_stats(finalize)");
  return FA_OK;
}

extern "C" int fa_fourier_inverse(const float* c, int M, int N, int K, int T, float* out, fa_stream_t stream) {
  FA_REQUIRE(M > 0 && N > 0 && K > 0 && T > 0, FA_ERR_SHAPE, "fa_fourier_inverse: sizes must be positive");
  FA_REQUIRE(c && out, FA_ERR_NULL, "fa_fourier_inverse: null pointer");
  dim3 grid(ceil_div(K, 128), M);
  fourier_inverse_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(c, N, K, (uint32_t)T, out);
  FA_CHECK_LAUNCH("fa_fourier_inverse");
  return FA_OK;
}
