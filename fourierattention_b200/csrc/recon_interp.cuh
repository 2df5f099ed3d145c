// Statistics of the reconstructed span by interpolation.  Included by compress.cu (namespace fa).
//
// The reconstruction x^[k, m] = (1/N) sum_n [C[n,m] cos(2 pi k n/T) + C[N+n,m] sin(2 pi k n/T)] is a
// trigonometric polynomial of degree N-1 in the token index k, so over a super-tile of J tokens that the
// highest frequency crosses at most 1.5 times it is reproduced to ~1e-7 by Lagrange interpolation through
// 16 fixed integer nodes (the same node sets and weights as the decode kernels use).  Per super-tile the
// kernel therefore contracts the 2N coefficients only at the 16 nodes (fp32 FMAs; the node basis is a
// fixed table rotated to the super-tile's centre, exact integer phases modulo 2T) and expands the
// 16 x 32 node values to J x 32 token values with the weight table, reducing them straight into the
// running sum / max / min of each column.  This is 8 times fewer multiply-adds than the direct product
// and no sincos per (token, frequency) pair.
#pragma once

namespace ri {
#include "interp_tables.inc"
__constant__ int r_nodes128[16] = {0, 3, 7, 14, 23, 34, 45, 57, 70, 82, 93, 104, 113, 120, 124, 127};
__constant__ int r_nodes64[16] = {0, 1, 4, 7, 12, 17, 22, 28, 35, 41, 46, 51, 56, 59, 62, 63};
}  // namespace ri

constexpr int RI_T = 512;    // threads
constexpr int RI_CT = 32;    // columns per CTA
constexpr int RI_W = RI_T / 32;

struct RiSmem {
  int coef, fn, ec, es, part, xn, interp, red, total;
};
__host__ __device__ inline RiSmem ri_smem(int N, int J) {
  RiSmem s;
  int o = 0;
  auto take = [&](int bytes) {
    int r = o;
    o += (bytes + 15) / 16 * 16;
    return r;
  };
  s.coef = take(2 * N * RI_CT * 4);        // [2N][32]
  s.fn = take(2 * N * 16 * 4);             // [2N][16 nodes]
  s.ec = take(8 * N * 4);
  s.es = take(8 * N * 4);
  s.part = take(RI_W * 16 * RI_CT * 4);    // per-warp partial node values
  s.xn = take(16 * RI_CT * 4);
  s.interp = take(J * 16 * 4);
  s.red = take(3 * RI_W * RI_CT * 4);
  s.total = o;
  return s;
}

// grid (column tiles, chunks of super-tiles, B); part[(b * nchunk + chunk) * 3 * Mc + {0, Mc, 2 Mc} + col]
template <int J>
__global__ void __launch_bounds__(RI_T, 1)
recon_stats_interp_kernel(const float* __restrict__ coef, int N, int Mc, int K, uint32_t T, float* __restrict__ part,
                          int st_per_chunk, int nchunk) {
  extern __shared__ __align__(16) unsigned char ri_raw[];
  const RiSmem L = ri_smem(N, J);
  float* cs = reinterpret_cast<float*>(ri_raw + L.coef);
  float* fn = reinterpret_cast<float*>(ri_raw + L.fn);
  float* ec = reinterpret_cast<float*>(ri_raw + L.ec);
  float* es = reinterpret_cast<float*>(ri_raw + L.es);
  float* pw = reinterpret_cast<float*>(ri_raw + L.part);
  float* xn = reinterpret_cast<float*>(ri_raw + L.xn);
  float* itp = reinterpret_cast<float*>(ri_raw + L.interp);
  float* red = reinterpret_cast<float*>(ri_raw + L.red);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int m0 = blockIdx.x * RI_CT, chunk = blockIdx.y, b = blockIdx.z;
  const uint32_t T2 = 2u * T;
  const float inv_T = 1.0f / (float)T, inv_N = 1.0f / (float)N;
  const int* nodes = (J == 128) ? ri::r_nodes128 : ri::r_nodes64;
  const float* tab = (J == 128) ? ri::g_interp128 : ri::g_interp64;
  const int nst = (K + J - 1) / J;
  const int st0 = chunk * st_per_chunk, st1 = min(nst, st0 + st_per_chunk);

  // coefficient tile, node table (nodes right of the centre), interpolation weights
  const float* cb = coef + (int64_t)b * 2 * N * Mc;
  for (int e = tid; e < 2 * N * RI_CT; e += RI_T) {
    const int n = e / RI_CT, c = e - n * RI_CT;
    cs[e] = (m0 + c < Mc) ? cb[(int64_t)n * Mc + m0 + c] : 0.f;
  }
  for (int e = tid; e < 8 * N; e += RI_T) {
    const int k = e / N, n = e - k * N;
    const uint32_t ph = phase_mod((uint64_t)(2 * nodes[8 + k] - (J - 1)), (uint32_t)n, T2);
    float s, c;
    sincospif((float)ph * inv_T, &s, &c);
    ec[e] = c;
    es[e] = s;
  }
  for (int e = tid; e < J * 16; e += RI_T) itp[e] = tab[e];

  // thread roles
  const int kq = lane >> 3, cq = lane & 7;           // node quad, column quad of the node contraction
  const int rows_per_warp = (2 * N + RI_W - 1) / RI_W;
  const int col = tid & 31, tg = tid >> 5;           // column and token group of the expansion
  constexpr int TPG = J / RI_W;                      // tokens per group
  float csum = 0.f, cmax = -INFINITY, cmin = INFINITY;
  __syncthreads();

  for (int st = st0; st < st1; ++st) {
    // ---- node basis of this super-tile: rotate the table to the tile's centre --------------------
    for (int n = tid; n < N; n += RI_T) {
      const uint64_t centre2 = 2ull * (uint64_t)st * J + (uint64_t)(J - 1);
      const uint32_t ph = phase_mod(centre2 % (uint64_t)T2, (uint32_t)n, T2);
      float rs, rc;
      sincospif((float)ph * inv_T, &rs, &rc);
      float fc[16], fs[16];
#pragma unroll
      for (int kp = 0; kp < 8; ++kp) {
        const float e_c = ec[kp * N + n], e_s = es[kp * N + n];
        const float t1 = rc * e_c, t2 = rs * e_s, t3 = rs * e_c, t4 = rc * e_s;
        fc[8 + kp] = t1 - t2;   // centre + d
        fs[8 + kp] = t3 + t4;
        fc[7 - kp] = t1 + t2;   // centre - d
        fs[7 - kp] = t3 - t4;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        *reinterpret_cast<float4*>(fn + n * 16 + 4 * q) = make_float4(fc[4 * q], fc[4 * q + 1], fc[4 * q + 2], fc[4 * q + 3]);
        *reinterpret_cast<float4*>(fn + (N + n) * 16 + 4 * q) =
            make_float4(fs[4 * q], fs[4 * q + 1], fs[4 * q + 2], fs[4 * q + 3]);
      }
    }
    __syncthreads();
    // ---- values at the nodes: X[16 x 32] = Fn^T[16 x 2N] * C[2N x 32]; a warp takes a slice of the rows ----
    {
      float acc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
      const int r0 = warp * rows_per_warp, r1 = min(2 * N, r0 + rows_per_warp);
#pragma unroll 4
      for (int r = r0; r < r1; ++r) {
        const float4 f4 = *reinterpret_cast<const float4*>(fn + r * 16 + 4 * kq);
        const float4 c4 = *reinterpret_cast<const float4*>(cs + r * RI_CT + 4 * cq);
        const float fa_[4] = {f4.x, f4.y, f4.z, f4.w}, ca[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(fa_[i], ca[j], acc[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
        *reinterpret_cast<float4*>(pw + (warp * 16 + 4 * kq + i) * RI_CT + 4 * cq) =
            make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    }
    __syncthreads();
    {
      float v = 0.f;   // 16 x 32 node values, one per thread
#pragma unroll
      for (int w = 0; w < RI_W; ++w) v += pw[w * 16 * RI_CT + tid];
      xn[tid] = v * inv_N;
    }
    __syncthreads();
    // ---- expand to the tokens of the super-tile and fold into the column statistics ----------------
    {
      float x[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) x[k] = xn[k * RI_CT + col];
      const int tok0 = st * J + tg * TPG;
#pragma unroll
      for (int j = 0; j < TPG; ++j) {
        const float* wj = itp + (tg * TPG + j) * 16;
        float v = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 w4 = *reinterpret_cast<const float4*>(wj + 4 * q);
          v = fmaf(w4.x, x[4 * q], fmaf(w4.y, x[4 * q + 1], fmaf(w4.z, x[4 * q + 2], fmaf(w4.w, x[4 * q + 3], v))));
        }
        if (tok0 + j < K) {
          csum += v;
          cmax = fmaxf(cmax, v);
          cmin = fminf(cmin, v);
        }
      }
    }
    // the next super-tile's basis overwrites fn only after every warp has passed the barrier that follows
    // its own node contraction, so no further barrier is needed here: xn and pw are rewritten behind
    // two more barriers
  }
  red[tg * RI_CT + col] = csum;
  red[(RI_W + tg) * RI_CT + col] = cmax;
  red[(2 * RI_W + tg) * RI_CT + col] = cmin;
  __syncthreads();
  if (tid < RI_CT && m0 + tid < Mc) {
    float s = 0.f, mx = -INFINITY, mn = INFINITY;
    for (int g = 0; g < RI_W; ++g) {
      s += red[g * RI_CT + tid];
      mx = fmaxf(mx, red[(RI_W + g) * RI_CT + tid]);
      mn = fminf(mn, red[(2 * RI_W + g) * RI_CT + tid]);
    }
    float* p = part + ((int64_t)(b * nchunk + chunk) * 3) * Mc;
    p[m0 + tid] = s;
    p[Mc + m0 + tid] = mx;
    p[2 * Mc + m0 + tid] = mn;
  }
}
