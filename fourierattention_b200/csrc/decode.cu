// Decode attention over the Fourier-compressed KV cache (one query token per sequence).
//
// Scores and outputs of the compressed dims are never rebuilt per token.  With
//   w[h,n] = sum_m C_k[n,m] scale_k[m] q_c[h,m]           (a mat-vec over the coefficients)
// the score of middle-span token l is (1/N) sum_n [w_cos[n] cos(2 pi l n/T) + w_sin[n] sin(..)]
// + const + q_n . k_verbatim[l], and with g[h,n] = sum_l p[l] cos/sin(2 pi l n/T) the compressed
// V dims of the output are scale_v*((1/N) C_v^T g - avg_vd*P) + avg_vu*P.  The basis of a tile of
// J consecutive tokens is a fixed J x N table times a per-frequency rotation, so the table lives in
// shared memory for the whole kernel and only w (forward) and g (backward) are rotated per tile.
//
// Three launches per call:
//   prepare  : w and const from q and C_k                      (reads C_k once)
//   main     : split-KV pass over sinks+window rows and over the middle span; per chunk partials
//              (max, denominator, verbatim-V numerator, g)      (reads every cache row once)
//   finish   : merge g over chunks and contract it with C_v (reads C_v once), merge numerators and
//              denominators, add the compressed-V part, normalise
#include <cuda.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <new>
#include <type_traits>

#include "common.cuh"

namespace fa {

constexpr int R_MAX = 8;        // query heads per KV head
constexpr int DEC_THREADS = 256;
constexpr int IT_G = 4;         // (frequency, 8-head block) items per thread in the g update
constexpr int IT_V = 4;         // verbatim-V columns per thread
constexpr int IT_IL = 2;        // 4-dim groups per thread in the sinks+window PV
constexpr float NEG_BIG = -1.0e30f;

struct DecodeParams {
  // tensor maps of the verbatim stores (tensor-core pass only): (column, row, sequence) tiles of
  // 64 x 64 elements, 128-byte swizzle, out-of-range rows and columns read as zero
  alignas(64) CUtensorMap tm_k;
  alignas(64) CUtensorMap tm_v;
  // tensor maps of the sink and window rows (tensor-core sinks+window pass): 64 columns x TRm rows
  alignas(64) CUtensorMap tm_ks;
  alignas(64) CUtensorMap tm_vs;
  alignas(64) CUtensorMap tm_kw;
  alignas(64) CUtensorMap tm_vw;
  fa_decode_args_t a;
  int R, F, n_il;
  int TRm, il_tpc;  // tensor-core sinks+window pass: rows per tile, tiles per chunk
  int sink_row0, win_row0;  // row of the sink / window tensor maps where the first sink / window row lies
  float c2;  // sm_scale * log2(e)
  // plan
  int J, kvh, HG, HGp, n_groups, TR, Hqp;
  int il_chunk_rows, n_il_chunks, mid_chunk, n_mid_chunks, NCH;
  int pitchK, pitchV, qpitch;
  int smem_main, smem_prepare;
  int force_exact;     // debugging / testing aid: never pick the tensor-core pass
  int fast, fNT, fNH;  // tensor-core middle-span pass: column tiles of 8 heads, halves per super-tile
  int wsSEQ, wsNTs;    // warp-specialised form: sequences per CTA, column tiles per sequence
  int wsGN, wsHG, wsNB;   // ... column tiles per CTA (4 or 2), head groups per sequence, node-basis buffers
  int wsSlotK, wsSlotV;   // ... columns of a ring slot (whole 64-column boxes of all sequences of the CTA)
  int wsHPT, wsKS;        // ... query heads per column tile (8, or 6 for three per KV head), 16-column steps per tile
  int w_frag;          // prepare writes w as fp16 hi + lo in MMA-fragment order (warp-specialised kernels) instead of fp32 rows
  int ws2;             // ... with the spectral accumulator in tensor memory (tcgen05 g update, 20 warps) instead of registers (16 warps)
  // scratch
  float *w, *cst, *m_part, *l_part, *o_part, *g_part;
  int* err;  // set by a kernel whose bounded wait gave up; the finish kernel then poisons the result
  float* tab;   // tensor-memory variant: node-offset rotation table and interpolation matrix as the main kernel's
                // shared-memory images (written by the prepare kernel: they depend on N and T only)
  int64_t scratch_floats;
};

__host__ __device__ inline int rup(int x, int m) { return (x + m - 1) / m * m; }

// byte offsets of the middle-span CTA's shared memory
struct MidSmem {
  int fc0, fs0, Wp, S, alpha, m_run, l_run, cst, rotc, rots, dltc, dlts, ph, dJ, qn, kofs, klen, vofs, kbuf, vbuf, total;
};
__host__ __device__ inline MidSmem mid_smem(int J, int N, int HGp, int kvh, int pitchK, int pitchV, int qpitch) {
  MidSmem s;
  int o = 0;
  auto take = [&](int bytes) {
    int r = o;
    o += rup(bytes, 16);
    return r;
  };
  s.fc0 = take(J * (N + 1) * 4);
  s.fs0 = take(J * (N + 1) * 4);
  s.Wp = take(2 * N * HGp * 4);
  s.S = take(J * HGp * 4);
  s.alpha = take(HGp * 4);
  s.m_run = take(HGp * 4);
  s.l_run = take(HGp * 4);
  s.cst = take(HGp * 4);
  s.rotc = take(N * 4);
  s.rots = take(N * 4);
  s.dltc = take(N * 4);
  s.dlts = take(N * 4);
  s.ph = take(N * 4);
  s.dJ = take(N * 4);
  s.qn = take(HGp * qpitch * 4);
  s.kofs = take((kvh + 1) * 4);
  s.klen = take((kvh + 1) * 4);
  s.vofs = take((kvh + 1) * 4);
  s.kbuf = take(2 * J * pitchK * 2);
  s.vbuf = take(2 * J * pitchV * 2);
  s.total = o;
  return s;
}

__host__ __device__ inline int il_smem_bytes(int TR, int F, int Hq, int Hqp, int D) {
  return 2 * TR * (F + 8) * 2 + Hq * D * 4 + TR * Hqp * 4 + 3 * Hqp * 4;
}

// ---------------------------------------------------------------------------------------------
// prepare: w[b,h,n] = (c2/N) sum_c C_k[b,n,c] scale_k[b,c] q[b,h,dim(c)],  cst[b,h] likewise
// grid (blocks of 256 coefficient rows, KV head, sequence); a thread owns one row of one KV head and
// walks the head's contiguous column segment with 128-bit loads, every load independent of the others
// ---------------------------------------------------------------------------------------------
// floats of the table block of the tensor-memory variant: cos / sin of the 8 node offsets for N frequencies,
// then the 128 x 16 interpolation matrix as fp16 hi and lo terms with rows of 24
__host__ __device__ inline int ws2_table_floats(int N) { return 16 * N + 2 * 128 * 24 / 2; }
__device__ void ws2_write_tables(const DecodeParams& p, int idx, int stride);   // defined with the kernel that reads them

template <typename T>
__global__ void __launch_bounds__(DEC_THREADS) decode_prepare_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const fa_decode_args_t& a = p.a;
  const int g = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int R = p.R, D = a.D, Mc = a.Mc_k, N = a.N;
  const int c0 = a.kc_h[g], c1 = a.kc_h[g + 1];
  const bool vec = (Mc & 3) == 0;                            // every row starts on a 16-byte boundary
  const int ca = vec ? (c0 & ~3) : c0;                       // first column read
  const int len = vec ? ((c1 - ca + 3) & ~3) : (c1 - ca);    // columns read; the pads get weight zero
  float* qs = reinterpret_cast<float*>(smem_raw);            // [R][len] query x scale
  const T* q = reinterpret_cast<const T*>(a.q) + (int64_t)b * a.q_sb;
  for (int e = tid; e < R * len; e += DEC_THREADS) {
    const int r = e / len, c = ca + e - r * len;
    float v = 0.f;
    if (c >= c0 && c < c1) v = to_f32(q[(g * R + r) * D + a.kc_list[c] - g * D]) * a.scale_k[(int64_t)b * Mc + c];
    qs[e] = v;
  }
  __syncthreads();
  const int row = blockIdx.x * DEC_THREADS + tid;
  if (row < 2 * N) {
    float acc[R_MAX];
#pragma unroll
    for (int r = 0; r < R_MAX; ++r) acc[r] = 0.f;
    const float* cr = a.k_coef + ((int64_t)b * 2 * N + row) * Mc + ca;
    if (vec) {
#pragma unroll 8
      for (int i = 0; i < len; i += 4) {
        const float4 cv = __ldg(reinterpret_cast<const float4*>(cr + i));
#pragma unroll
        for (int r = 0; r < R_MAX; ++r) {
          if (r < R) {
            const float4 qv = *reinterpret_cast<const float4*>(qs + r * len + i);
            acc[r] = fmaf(cv.x, qv.x, fmaf(cv.y, qv.y, fmaf(cv.z, qv.z, fmaf(cv.w, qv.w, acc[r]))));
          }
        }
      }
    } else {
#pragma unroll 4
      for (int i = 0; i < len; ++i) {
        const float cv = __ldg(cr + i);
#pragma unroll
        for (int r = 0; r < R_MAX; ++r)
          if (r < R) acc[r] = fmaf(cv, qs[r * len + i], acc[r]);
      }
    }
    const float wscale = p.c2 / (float)N;
    if (p.w_frag) {
      // fp16 hi + lo in the order the spectral warps load their m16n8k16 B fragments: per head, 16 bytes per
      // (16-row step, lane quad position tq) = {hi rows 2tq,2tq+1 | hi rows 2tq+8,+9 | lo ... | lo ...}
      const int ks = row >> 4, j = row & 15, rr = j >> 3, tq = (j & 7) >> 1, odd = j & 1;
#pragma unroll
      for (int r = 0; r < R_MAX; ++r) {
        if (r < R) {
          const float v = acc[r] * wscale;
          const __half hi = __float2half_rn(v), lo = __float2half_rn(v - __half2float(hi));
          __half* dst = reinterpret_cast<__half*>(p.w) + (((int64_t)b * a.Hq + g * R + r) * (2 * N / 16) + ks) * 32 + tq * 8;
          dst[rr * 2 + odd] = hi;
          dst[4 + rr * 2 + odd] = lo;
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < R_MAX; ++r)
        if (r < R) p.w[((int64_t)b * a.Hq + g * R + r) * 2 * N + row] = acc[r] * wscale;
    }
  }
  if (blockIdx.x == 0 && g == 0 && b == 0 && tid == 0) *p.err = 0;
  if (p.ws2)   // spread over the whole grid: at most a few entries per thread
    ws2_write_tables(p, ((b * gridDim.y + g) * gridDim.x + blockIdx.x) * DEC_THREADS + tid, gridDim.x * gridDim.y * gridDim.z * DEC_THREADS);
  if (blockIdx.x == 0 && warp < R) {
    const int h = g * R + warp;
    float acc = 0.f;
    for (int c = c0 + lane; c < c1; c += 32) {
      const int64_t o = (int64_t)b * Mc + c;
      acc = fmaf(to_f32(q[h * D + a.kc_list[c] - g * D]), a.avg_k_u[o] - a.avg_k_d[o] * a.scale_k[o], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) p.cst[(int64_t)b * a.Hq + h] = acc * p.c2;
  }
}

// barrier of the 256 threads of a CTA
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// main, part 1: sinks + window rows (dense K/V rows, all heads of the rank)
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void il_issue_tile(const DecodeParams& p, int b, const void* sink, const void* win,
                                              int row0, int row_end, T* dst, int TR, int F, int tid) {
  const fa_decode_args_t& a = p.a;
  const int pitch = F + 8;
  const int cpr = F / 8;  // 16-byte chunks per row
  const T* sb = reinterpret_cast<const T*>(sink) + (int64_t)b * a.sink_sb;
  const T* wb = reinterpret_cast<const T*>(win) + (int64_t)b * a.win_sb;
  for (int e = tid; e < TR * cpr; e += DEC_THREADS) {
    const int r = e / cpr, c = e - r * cpr;
    const int row = row0 + r;
    T* d = dst + r * pitch + c * 8;
    if (row < row_end) {
      const T* src = (row < a.n_sink) ? sb + (int64_t)row * F : wb + (int64_t)(row - a.n_sink) * F;
      cp_async16(d, src + c * 8);
    } else {
      *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

template <typename T>
__device__ void il_chunk(const DecodeParams& p, int b, int chunk, unsigned char* smem) {
  const fa_decode_args_t& a = p.a;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int F = p.F, D = a.D, Hq = a.Hq, Hkv = a.Hkv, R = p.R, TR = p.TR, Hqp = p.Hqp;
  const int pitch = F + 8;
  T* ks = reinterpret_cast<T*>(smem);
  T* vs = ks + TR * pitch;
  float* qs = reinterpret_cast<float*>(vs + TR * pitch);  // [Hq][D], pre-scaled by c2
  float* S = qs + Hq * D;                                   // [TR][Hqp]
  float* m_run = S + TR * Hqp;
  float* l_run = m_run + Hqp;
  float* alpha = l_run + Hqp;

  const int r0 = chunk * p.il_chunk_rows;
  const int r1 = min(p.n_il, r0 + p.il_chunk_rows);
  const int nt = (r1 - r0 + TR - 1) / TR;

  il_issue_tile<T>(p, b, a.k_sink, a.k_win, r0, r1, ks, TR, F, tid);
  cp_async_commit();
  il_issue_tile<T>(p, b, a.v_sink, a.v_win, r0, r1, vs, TR, F, tid);
  cp_async_commit();

  const T* q = reinterpret_cast<const T*>(a.q) + (int64_t)b * a.q_sb;
  for (int i = tid; i < Hq * D; i += DEC_THREADS) qs[i] = to_f32(q[i]) * p.c2;
  for (int h = tid; h < Hqp; h += DEC_THREADS) {
    m_run[h] = NEG_BIG;
    l_run[h] = 0.f;
    alpha[h] = 1.f;
  }

  float oacc[IT_IL][R_MAX][4];
#pragma unroll
  for (int i = 0; i < IT_IL; ++i)
#pragma unroll
    for (int r = 0; r < R_MAX; ++r)
#pragma unroll
      for (int k = 0; k < 4; ++k) oacc[i][r][k] = 0.f;

  for (int t = 0; t < nt; ++t) {
    const int row0 = r0 + t * TR;
    const int valid = min(TR, r1 - row0);
    cp_async_wait<1>();
    compute_sync();
    // ---- scores -------------------------------------------------------------------------
    for (int it = tid; it < TR * Hkv; it += DEC_THREADS) {
      const int row = it % TR, g = it / TR;
      float acc[R_MAX];
#pragma unroll
      for (int r = 0; r < R_MAX; ++r) acc[r] = 0.f;
      const T* kr = ks + row * pitch + g * D;
      for (int d0 = 0; d0 < D; d0 += 8) {
        float kf[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(kr + d0), kf);
#pragma unroll
        for (int r = 0; r < R_MAX; ++r) {
          if (r < R) {
            const float* qp = qs + (g * R + r) * D + d0;
            const float4 q0 = *reinterpret_cast<const float4*>(qp);
            const float4 q1 = *reinterpret_cast<const float4*>(qp + 4);
            acc[r] += kf[0] * q0.x + kf[1] * q0.y + kf[2] * q0.z + kf[3] * q0.w + kf[4] * q1.x + kf[5] * q1.y +
                      kf[6] * q1.z + kf[7] * q1.w;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < R_MAX; ++r)
        if (r < R) S[row * Hqp + g * R + r] = acc[r];
    }
    compute_sync();
    if (t + 1 < nt) il_issue_tile<T>(p, b, a.k_sink, a.k_win, row0 + TR, r1, ks, TR, F, tid);
    cp_async_commit();
    // ---- online softmax, one warp per head ----------------------------------------------
    for (int h = warp; h < Hq; h += DEC_THREADS / 32) {
      float mt = NEG_BIG;
      for (int row = lane; row < valid; row += 32) mt = fmaxf(mt, S[row * Hqp + h]);
      mt = warp_max(mt);
      const float m_old = m_run[h];
      const float m_new = fmaxf(m_old, mt);
      float lt = 0.f;
      for (int row = lane; row < TR; row += 32) {
        const float pv = (row < valid) ? exp2f(S[row * Hqp + h] - m_new) : 0.f;
        S[row * Hqp + h] = pv;
        lt += pv;
      }
      lt = warp_sum(lt);
      if (lane == 0) {
        const float al = exp2f(m_old - m_new);
        alpha[h] = al;
        l_run[h] = l_run[h] * al + lt;
        m_run[h] = m_new;
      }
    }
    cp_async_wait<1>();
    compute_sync();
    // ---- PV -----------------------------------------------------------------------------
#pragma unroll
    for (int i = 0; i < IT_IL; ++i) {
      const int f = (tid + i * DEC_THREADS) * 4;
      if (f < F) {
        const int g = f / D;
#pragma unroll
        for (int r = 0; r < R_MAX; ++r) {
          if (r < R) {
            const float al = alpha[g * R + r];
#pragma unroll
            for (int k = 0; k < 4; ++k) oacc[i][r][k] *= al;
          }
        }
        for (int row = 0; row < TR; ++row) {
          const uint2 raw = *reinterpret_cast<const uint2*>(vs + row * pitch + f);
          using P2 = typename Pack2<T>::type;
          const P2* pp = reinterpret_cast<const P2*>(&raw);
          const float2 v01 = Pack2<T>::cvt(pp[0]), v23 = Pack2<T>::cvt(pp[1]);
#pragma unroll
          for (int r = 0; r < R_MAX; ++r) {
            if (r < R) {
              const float pv = S[row * Hqp + g * R + r];
              oacc[i][r][0] = fmaf(pv, v01.x, oacc[i][r][0]);
              oacc[i][r][1] = fmaf(pv, v01.y, oacc[i][r][1]);
              oacc[i][r][2] = fmaf(pv, v23.x, oacc[i][r][2]);
              oacc[i][r][3] = fmaf(pv, v23.y, oacc[i][r][3]);
            }
          }
        }
      }
    }
    compute_sync();
    if (t + 1 < nt) il_issue_tile<T>(p, b, a.v_sink, a.v_win, row0 + TR, r1, vs, TR, F, tid);
    cp_async_commit();
  }
  cp_async_wait<0>();

  const int64_t slot = (int64_t)b * p.NCH + chunk;
  for (int h = tid; h < Hq; h += DEC_THREADS) {
    p.m_part[slot * Hq + h] = m_run[h];
    p.l_part[slot * Hq + h] = l_run[h];
  }
#pragma unroll
  for (int i = 0; i < IT_IL; ++i) {
    const int f = (tid + i * DEC_THREADS) * 4;
    if (f < F) {
      const int g = f / D, d = f - g * D;
#pragma unroll
      for (int r = 0; r < R_MAX; ++r) {
        if (r < R) {
          float* o = p.o_part + (slot * Hq + g * R + r) * D + d;
          *reinterpret_cast<float4*>(o) = make_float4(oacc[i][r][0], oacc[i][r][1], oacc[i][r][2], oacc[i][r][3]);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// main, part 2: the middle span (verbatim dims from memory, compressed dims from w / into g)
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void mid_issue_rows(const T* base, int64_t sk, bool fast, int a0, int n8, int seg0,
                                               int seg, int shift, int l_first, int l_end, int J, T* dst, int pitch,
                                               int tid) {
  if (fast) {
    for (int e = tid; e < J * n8; e += DEC_THREADS) {
      const int j = e / n8, c = e - j * n8;
      const int l = l_first + j;
      T* d = dst + j * pitch + c * 8;
      if (l < l_end)
        cp_async16(d, base + (int64_t)l * sk + a0 + c * 8);
      else
        *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
  } else {
    for (int e = tid; e < J * seg; e += DEC_THREADS) {
      const int j = e / seg, c = e - j * seg;
      const int l = l_first + j;
      T v = (l < l_end) ? base[(int64_t)l * sk + seg0 + c] : T(0.f);
      dst[j * pitch + shift + c] = v;
    }
  }
}

template <typename T>
__device__ void mid_chunk(const DecodeParams& p, int b, int chunk, int group, unsigned char* smem) {
  const fa_decode_args_t& a = p.a;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = a.N, D = a.D, R = p.R, J = p.J, HGp = p.HGp, Hq = a.Hq;
  const uint32_t T_ = (uint32_t)a.T;
  const float inv_T = 1.0f / (float)a.T;
  const MidSmem L = mid_smem(J, N, HGp, p.kvh, p.pitchK, p.pitchV, p.qpitch);
  float* fc0 = reinterpret_cast<float*>(smem + L.fc0);
  float* fs0 = reinterpret_cast<float*>(smem + L.fs0);
  float* Wp = reinterpret_cast<float*>(smem + L.Wp);
  float* S = reinterpret_cast<float*>(smem + L.S);
  float* alpha = reinterpret_cast<float*>(smem + L.alpha);
  float* m_run = reinterpret_cast<float*>(smem + L.m_run);
  float* l_run = reinterpret_cast<float*>(smem + L.l_run);
  float* cst = reinterpret_cast<float*>(smem + L.cst);
  float* rotc = reinterpret_cast<float*>(smem + L.rotc);
  float* rots = reinterpret_cast<float*>(smem + L.rots);
  float* dltc = reinterpret_cast<float*>(smem + L.dltc);
  float* dlts = reinterpret_cast<float*>(smem + L.dlts);
  uint32_t* ph = reinterpret_cast<uint32_t*>(smem + L.ph);
  uint32_t* dJ = reinterpret_cast<uint32_t*>(smem + L.dJ);
  float* qn = reinterpret_cast<float*>(smem + L.qn);
  int* kofs = reinterpret_cast<int*>(smem + L.kofs);
  int* klen = reinterpret_cast<int*>(smem + L.klen);
  int* vofs = reinterpret_cast<int*>(smem + L.vofs);
  T* kbuf = reinterpret_cast<T*>(smem + L.kbuf);
  T* vbuf = reinterpret_cast<T*>(smem + L.vbuf);
  const int pitchK = p.pitchK, pitchV = p.pitchV, qpitch = p.qpitch, N1 = N + 1;

  // heads of this CTA
  const int g0 = group * p.kvh;
  const int g1 = min(a.Hkv, g0 + p.kvh);
  const int ng = g1 - g0;
  const int h0 = g0 * R;
  const int nh = ng * R;

  // token range
  const int l0 = chunk * p.mid_chunk;
  const int l1 = min(a.n_mid, l0 + p.mid_chunk);
  const int nt = (l1 - l0 + J - 1) / J;

  // verbatim column spans of this head group
  const int seg0K = a.kn_h[g0], segK = a.kn_h[g1] - seg0K;
  const int seg0V = a.vn_h[g0], segV = a.vn_h[g1] - seg0V;
  const T* kbase = reinterpret_cast<const T*>(a.k_mn) + (int64_t)b * a.k_mn_sb;
  const T* vbase = reinterpret_cast<const T*>(a.v_mn) + (int64_t)b * a.v_mn_sb;
  const bool fastK = ((reinterpret_cast<uintptr_t>(kbase) & 15) == 0) && (a.k_mn_sk % 8 == 0);
  const bool fastV = ((reinterpret_cast<uintptr_t>(vbase) & 15) == 0) && (a.v_mn_sk % 8 == 0);
  const int a0K = fastK ? (seg0K & ~7) : seg0K, a0V = fastV ? (seg0V & ~7) : seg0V;
  const int shiftK = seg0K - a0K, shiftV = seg0V - a0V;
  const int n8K = (rup(seg0K + segK, 8) - a0K) / 8, n8V = (rup(seg0V + segV, 8) - a0V) / 8;

  // first tile in flight while the tables are built
  mid_issue_rows<T>(kbase, a.k_mn_sk, fastK, a0K, n8K, seg0K, segK, shiftK, l0, l1, J, kbuf, pitchK, tid);
  mid_issue_rows<T>(vbase, a.v_mn_sk, fastV, a0V, n8V, seg0V, segV, shiftV, l0, l1, J, vbuf, pitchV, tid);
  cp_async_commit();

  // ---- per-CTA tables ---------------------------------------------------------------------
  for (int e = tid; e < J * N; e += DEC_THREADS) {
    const int j = e / N, n = e - j * N;
    float s, c;
    sincos_phase(phase_mod((uint64_t)j, (uint32_t)n, T_), inv_T, &s, &c);
    fc0[j * N1 + n] = c;
    fs0[j * N1 + n] = s;
  }
  for (int n = tid; n < N; n += DEC_THREADS) {
    const uint32_t d = phase_mod((uint64_t)J, (uint32_t)n, T_);
    dJ[n] = d;
    float s, c;
    sincos_phase(d, inv_T, &s, &c);
    dltc[n] = c;
    dlts[n] = s;
    ph[n] = phase_mod((uint64_t)a.mid_l0 + (uint64_t)l0, (uint32_t)n, T_);
  }
  for (int i = tid; i <= ng; i += DEC_THREADS) {
    kofs[i] = a.kn_h[g0 + i] - seg0K + shiftK;
    vofs[i] = a.vn_h[g0 + i] - seg0V;  // relative to the span start (no shift)
    if (i < ng) klen[i] = a.kn_h[g0 + i + 1] - a.kn_h[g0 + i];
  }
  for (int hh = tid; hh < HGp; hh += DEC_THREADS) {
    alpha[hh] = 1.f;
    m_run[hh] = NEG_BIG;
    l_run[hh] = 0.f;
    cst[hh] = (hh < nh) ? p.cst[(int64_t)b * Hq + h0 + hh] : 0.f;
  }
  __syncthreads();
  {
    // rotated weights for the first tile: W'_c = w_c cos(a) + w_s sin(a), W'_s = -w_c sin(a) + w_s cos(a)
    const float* wb = p.w + ((int64_t)b * Hq + h0) * 2 * N;
    for (int e = tid; e < N * HGp; e += DEC_THREADS) {
      const int hh = e / N, n = e - hh * N;  // consecutive threads read consecutive n
      float wc = 0.f, ws = 0.f;
      if (hh < nh) {
        wc = wb[(int64_t)hh * 2 * N + n];
        ws = wb[(int64_t)hh * 2 * N + N + n];
      }
      float s, c;
      sincos_phase(ph[n], inv_T, &s, &c);
      Wp[n * HGp + hh] = wc * c + ws * s;
      Wp[(N + n) * HGp + hh] = -wc * s + ws * c;
    }
    // verbatim-K query slices, pre-scaled
    const T* q = reinterpret_cast<const T*>(a.q) + (int64_t)b * a.q_sb;
    for (int e = tid; e < nh * qpitch; e += DEC_THREADS) {
      const int hh = e / qpitch, i = e - hh * qpitch;
      const int gl = hh / R;
      float v = 0.f;
      if (i < klen[gl]) {
        const int d = a.kn_list[a.kn_h[g0 + gl] + i] - (g0 + gl) * D;
        v = to_f32(q[(h0 + hh) * D + d]) * p.c2;
      }
      qn[hh * qpitch + i] = v;
    }
  }

  // persistent accumulators
  float Gc[IT_G][8], Gs[IT_G][8];
#pragma unroll
  for (int i = 0; i < IT_G; ++i)
#pragma unroll
    for (int k = 0; k < 8; ++k) Gc[i][k] = Gs[i][k] = 0.f;
  float ov[IT_V][R_MAX];
  int vgl[IT_V];
#pragma unroll
  for (int i = 0; i < IT_V; ++i) {
#pragma unroll
    for (int r = 0; r < R_MAX; ++r) ov[i][r] = 0.f;
    const int c = tid + i * DEC_THREADS;
    int gl = 0;
    if (c < segV)
      while (gl + 1 < ng && c >= vofs[gl + 1]) ++gl;
    vgl[i] = gl;
  }
  const int n_items_g = N * (HGp / 8);
  __syncthreads();

  for (int t = 0; t < nt; ++t) {
    const int lt0 = l0 + t * J;
    const int valid = min(J, l1 - lt0);
    T* kb = kbuf + (t & 1) * J * pitchK;
    T* vb = vbuf + (t & 1) * J * pitchV;
    if (t + 1 < nt) {
      T* kb2 = kbuf + ((t + 1) & 1) * J * pitchK;
      T* vb2 = vbuf + ((t + 1) & 1) * J * pitchV;
      mid_issue_rows<T>(kbase, a.k_mn_sk, fastK, a0K, n8K, seg0K, segK, shiftK, lt0 + J, l1, J, kb2, pitchK, tid);
      mid_issue_rows<T>(vbase, a.v_mn_sk, fastV, a0V, n8V, seg0V, segV, shiftV, lt0 + J, l1, J, vb2, pitchV, tid);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    // [A] rotation of this tile for the g update; advance the integer phases
    for (int n = tid; n < N; n += DEC_THREADS) {
      float s, c;
      const uint32_t v = ph[n];
      sincos_phase(v, inv_T, &s, &c);
      rotc[n] = c;
      rots[n] = s;
      uint32_t nx = v + dJ[n];
      if (nx >= T_) nx -= T_;
      ph[n] = nx;
    }
    // [B]+[C] scores: spectral part from the base table and W', verbatim part from the K rows
    for (int it = tid; it < J * (HGp / 4); it += DEC_THREADS) {
      const int j = it % J, hq4 = it / J;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const float* fcr = fc0 + j * N1;
      const float* fsr = fs0 + j * N1;
      const float* wcol = Wp + hq4 * 4;
#pragma unroll 4
      for (int n = 0; n < N; ++n) {
        const float c = fcr[n], s = fsr[n];
        const float4 wc = *reinterpret_cast<const float4*>(wcol + n * HGp);
        const float4 ws = *reinterpret_cast<const float4*>(wcol + (N + n) * HGp);
        acc[0] = fmaf(c, wc.x, fmaf(s, ws.x, acc[0]));
        acc[1] = fmaf(c, wc.y, fmaf(s, ws.y, acc[1]));
        acc[2] = fmaf(c, wc.z, fmaf(s, ws.z, acc[2]));
        acc[3] = fmaf(c, wc.w, fmaf(s, ws.w, acc[3]));
      }
      const T* krow = kb + j * pitchK;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int hh = hq4 * 4 + k;
        float v = 0.f;
        if (hh < nh) {
          const int gl = hh / R;
          const T* kr = krow + kofs[gl];
          const float* qh = qn + hh * qpitch;
          const int len = klen[gl];
          float d = 0.f;
          for (int i = 0; i < len; ++i) d = fmaf(qh[i], to_f32(kr[i]), d);
          v = acc[k] + cst[hh] + d;
        }
        S[j * HGp + hh] = v;
      }
    }
    __syncthreads();
    // [D] online softmax, one warp per head
    for (int hh = warp; hh < nh; hh += DEC_THREADS / 32) {
      const float sv = (lane < valid) ? S[lane * HGp + hh] : NEG_BIG;
      const float mt = warp_max(sv);
      const float m_old = m_run[hh];
      const float m_new = fmaxf(m_old, mt);
      const float pv = (lane < valid) ? exp2f(sv - m_new) : 0.f;
      if (lane < J) S[lane * HGp + hh] = pv;
      const float lt = warp_sum(pv);
      if (lane == 0) {
        const float al = exp2f(m_old - m_new);
        alpha[hh] = al;
        l_run[hh] = l_run[hh] * al + lt;
        m_run[hh] = m_new;
      }
    }
    __syncthreads();
    // [E] g update: tile sums against the base table, rotated into the absolute frame
#pragma unroll
    for (int i = 0; i < IT_G; ++i) {
      const int item = tid + i * DEC_THREADS;
      if (item < n_items_g) {
        const int n = item % N, hb = item / N;
        float tc[8], ts[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) tc[k] = ts[k] = 0.f;
        for (int j = 0; j < J; ++j) {
          const float c = fc0[j * N1 + n], s = fs0[j * N1 + n];
          const float4 p0 = *reinterpret_cast<const float4*>(S + j * HGp + hb * 8);
          const float4 p1 = *reinterpret_cast<const float4*>(S + j * HGp + hb * 8 + 4);
          const float pa[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            tc[k] = fmaf(c, pa[k], tc[k]);
            ts[k] = fmaf(s, pa[k], ts[k]);
          }
        }
        const float rc = rotc[n], rs = rots[n];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float al = alpha[hb * 8 + k];
          Gc[i][k] = fmaf(Gc[i][k], al, rc * tc[k] - rs * ts[k]);
          Gs[i][k] = fmaf(Gs[i][k], al, rs * tc[k] + rc * ts[k]);
        }
      }
    }
    // [F] verbatim V numerators
#pragma unroll
    for (int i = 0; i < IT_V; ++i) {
      const int c = tid + i * DEC_THREADS;
      if (c < segV) {
        const int gl = vgl[i];
#pragma unroll
        for (int r = 0; r < R_MAX; ++r)
          if (r < R) ov[i][r] *= alpha[gl * R + r];
        const T* vc = vb + shiftV + c;
        for (int j = 0; j < J; ++j) {
          const float v = to_f32(vc[j * pitchV]);
#pragma unroll
          for (int r = 0; r < R_MAX; ++r)
            if (r < R) ov[i][r] = fmaf(S[j * HGp + gl * R + r], v, ov[i][r]);
        }
      }
    }
    // [G] rotate W' to the next tile
    if (t + 1 < nt) {
      for (int e = tid; e < N * HGp; e += DEC_THREADS) {
        const int n = e / HGp, hh = e - n * HGp;
        const float wc = Wp[n * HGp + hh], ws = Wp[(N + n) * HGp + hh];
        const float dc = dltc[n], ds = dlts[n];
        Wp[n * HGp + hh] = wc * dc + ws * ds;
        Wp[(N + n) * HGp + hh] = ws * dc - wc * ds;
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // ---- chunk partials -----------------------------------------------------------------------
  const int64_t slot = (int64_t)b * p.NCH + p.n_il_chunks + chunk;
  for (int hh = tid; hh < nh; hh += DEC_THREADS) {
    p.m_part[slot * Hq + h0 + hh] = m_run[hh];
    p.l_part[slot * Hq + h0 + hh] = l_run[hh];
  }
  float* ob = p.o_part + (slot * Hq + h0) * D;
  for (int e = tid; e < nh * D; e += DEC_THREADS) ob[e] = 0.f;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < IT_V; ++i) {
    const int c = tid + i * DEC_THREADS;
    if (c < segV) {
      const int gl = vgl[i];
      const int d = a.vn_list[seg0V + c] - (g0 + gl) * D;
#pragma unroll
      for (int r = 0; r < R_MAX; ++r)
        if (r < R) ob[(gl * R + r) * D + d] = ov[i][r];
    }
  }
  float* gb = p.g_part + (((int64_t)b * p.n_mid_chunks + chunk) * Hq + h0) * 2 * N;
#pragma unroll
  for (int i = 0; i < IT_G; ++i) {
    const int item = tid + i * DEC_THREADS;
    if (item < n_items_g) {
      const int n = item % N, hb = item / N;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int hh = hb * 8 + k;
        if (hh < nh) {
          gb[(int64_t)hh * 2 * N + n] = Gc[i][k];
          gb[(int64_t)hh * 2 * N + N + n] = Gs[i][k];
        }
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(DEC_THREADS, 1) decode_main_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int b = blockIdx.y;
  if ((int)blockIdx.x < p.n_il_chunks) {
    il_chunk<T>(p, b, blockIdx.x, smem_raw);
  } else {
    const int idx = blockIdx.x - p.n_il_chunks;
    mid_chunk<T>(p, b, idx / p.n_groups, idx % p.n_groups, smem_raw);
  }
}

#include "decode_fast.cuh"

#include "decode_il.cuh"
#include "decode_ws.cuh"
#include "decode_ws2.cuh"

// (called by the prepare kernel) entry e of the node-offset table: node 8+k lies (2 x_k - 127) / 2 tokens right of a
// super-tile's centre; the interpolation matrix is split into fp16 hi + lo
__device__ void ws2_write_tables(const DecodeParams& p, int idx, int stride) {
  const int N = p.a.N;
  const uint32_t T2 = 2u * (uint32_t)p.a.T;
  const float inv_T = 1.0f / (float)p.a.T;
  for (int e = idx; e < 8 * N; e += stride) {
    const int k = e / N, n = e - k * N;
    const uint32_t ph = phase_mod((uint64_t)(2 * c_nodes128[8 + k] - 127), (uint32_t)n, T2);
    float sn, cs;
    sincospif((float)ph * inv_T, &sn, &cs);
    p.tab[e] = cs;
    p.tab[8 * N + e] = sn;
  }
  __half* ih = reinterpret_cast<__half*>(p.tab + 16 * N);
  __half* il = ih + 128 * 24;
  for (int e = idx; e < 128 * 24; e += stride) {
    const int j = e / 24, k = e - j * 24;
    __half hi = __float2half_rn(0.f), lo = hi;
    if (k < FD) split_h(g_interp128[j * FD + k], hi, lo);
    ih[e] = hi;
    il[e] = lo;
  }
}

constexpr int FAST_THREADS = FAST_T;

template <typename T, int NT, int NH>
__global__ void __launch_bounds__(FAST_THREADS, 1) decode_main_fast_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int b = blockIdx.y;
  if ((int)blockIdx.x < p.n_il_chunks) {
    il_chunk_mma<T>(p, b, blockIdx.x, smem_raw);
  } else {
    mid_chunk_fast<T, NT, NH>(p, b, blockIdx.x - p.n_il_chunks, smem_raw);
  }
}

template <typename T, int GN, int KS>
__global__ void __launch_bounds__(WS_T, 1) decode_main_ws_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int b = blockIdx.y;
  // blockIdx.y is a group of wsSEQ sequences: first the sinks+window CTAs of each of them, then the group's
  // middle-span CTAs
  const int n_il_ctas = p.wsSEQ * p.n_il_chunks;
  if ((int)blockIdx.x < n_il_ctas) {
    const int seq = blockIdx.x / p.n_il_chunks, chunk = blockIdx.x - seq * p.n_il_chunks;
    if (b * p.wsSEQ + seq >= p.a.B) return;
    if (p.TRm == 16)   // wide rows (Hkv*D = 1024): 16-row tiles, the common case, unrolled for exactly one
      il_chunk_mma<T, 1>(p, b * p.wsSEQ + seq, chunk, smem_raw);
    else
      il_chunk_mma<T>(p, b * p.wsSEQ + seq, chunk, smem_raw);
  } else {
    const int idx = blockIdx.x - n_il_ctas;   // (chunk, head group)
    mid_chunk_ws<T, GN, KS>(p, b * p.wsSEQ, idx / p.wsHG, idx % p.wsHG, smem_raw);
  }
}

template <typename T>
__global__ void __launch_bounds__(W2_T, 1) decode_main_ws2_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int b = blockIdx.y;
  const int n_il_ctas = p.wsSEQ * p.n_il_chunks;
  if ((int)blockIdx.x < n_il_ctas) {
    // sinks + window rows: a 512-thread pass (its barriers name 512 threads); the other warps hand their
    // registers to it and leave
    if (threadIdx.x >= IL_T) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 24;\n");
      return;
    }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 112;\n");
    const int seq = blockIdx.x / p.n_il_chunks, chunk = blockIdx.x - seq * p.n_il_chunks;
    if (b * p.wsSEQ + seq >= p.a.B) return;
    // unrolled for exactly the 16-row blocks a tile of rows has (16 rows at Hkv*D = 1024, 32 at 512, 64 at 256): the
    // pass has 112 registers here, and what it spills is reloaded from L2 behind the K / V stream of the other CTAs
    if (p.TRm == 16)
      il_chunk_mma<T, 1>(p, b * p.wsSEQ + seq, chunk, smem_raw);
    else if (p.TRm == 32)
      il_chunk_mma<T, 2>(p, b * p.wsSEQ + seq, chunk, smem_raw);
    else   // (the planner keeps tiles of rows at 64 rows or fewer for this kernel)
      il_chunk_mma<T, 4>(p, b * p.wsSEQ + seq, chunk, smem_raw);
  } else {
    mid_chunk_ws2<T>(p, b * p.wsSEQ, blockIdx.x - n_il_ctas, smem_raw);
  }
}

// ---------------------------------------------------------------------------------------------
// finish, one CTA per (query head, sequence): merge weights a_i = 2^(m_i - m*) of the chunk slots,
// G*[n] = sum_chunks a_i g_i[h,n], the compressed-V dims  (1/N) sum_n G*[n] C_v[n,c]  of the head's
// column segment, the merged verbatim numerators, normalisation
// ---------------------------------------------------------------------------------------------
constexpr int FIN_THREADS = 512;

__host__ __device__ inline int finish_smem_bytes(int NCH, int N, int D) {
  return (rup(NCH, 4) + 2 * N + rup(D, 4) + 4 * FIN_THREADS) * 4;
}

__global__ void __launch_bounds__(FIN_THREADS, 2) decode_finish_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const fa_decode_args_t& a = p.a;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int D = a.D, Hq = a.Hq, R = p.R, N = a.N, Mc = a.Mc_v, NCH = p.NCH, NM = p.n_mid_chunks;
  const bool mid = a.n_mid > 0;
  float* aw = reinterpret_cast<float*>(smem_raw);   // [NCH]
  float* Gs = aw + rup(NCH, 4);                     // [2N]
  float* O = Gs + 2 * N;                            // [D]
  float* red = O + rup(D, 4);                       // [FIN_THREADS][4]
  __shared__ float s_L, s_P, s_ms;
  const int g = h / R;
  float P, L, ms_all;
  if (NCH <= 32) {
    // Few chunk slots: every warp works the merge weights out for itself (lane i <-> slot i) while the
    // loads of the partial results it is going to merge are already in flight; nothing waits on a barrier.
    const int lane = tid & 31;
    float li = 0.f, mi = NEG_BIG;
    if (lane < NCH) {
      const int64_t o = ((int64_t)b * NCH + lane) * Hq + h;
      li = p.l_part[o];
      mi = p.m_part[o];
    }
    float pv[32];   // this thread's partial results, first of g, then of the verbatim numerators
    const bool has_n = mid && tid < 2 * N, has_d = tid < D;
    const float* gp = p.g_part + ((int64_t)b * NM * Hq + h) * 2 * N + tid;
    const float* op = p.o_part + ((int64_t)b * NCH * Hq + h) * D + tid;
#pragma unroll
    for (int i = 0; i < 32; ++i) pv[i] = (has_n && i < NM) ? gp[(int64_t)i * Hq * 2 * N] : 0.f;
    const float ms = warp_max(li > 0.f ? mi : NEG_BIG);
    const float wi = li > 0.f ? exp2f(mi - ms) : 0.f;
    L = warp_sum(wi * li);
    P = warp_sum(lane >= p.n_il_chunks ? wi * li : 0.f);
    ms_all = ms;
    float gacc = 0.f, oacc = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float w_mid = __shfl_sync(0xffffffffu, wi, (p.n_il_chunks + i) & 31);
      gacc = fmaf(i < NM ? w_mid : 0.f, pv[i], gacc);
    }
    if (tid < 32 * ((D + 31) / 32)) {   // whole warps, so that the shuffles stay converged
#pragma unroll
      for (int i = 0; i < 32; ++i) pv[i] = (has_d && i < NCH) ? op[(int64_t)i * Hq * D] : 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) oacc = fmaf(__shfl_sync(0xffffffffu, wi, i), pv[i], oacc);
    }
    if (has_n) Gs[tid] = gacc;
    if (has_d) O[tid] = oacc;
    if (mid) {
      for (int n = tid + FIN_THREADS; n < 2 * N; n += FIN_THREADS) {   // 2N > 512 only
        const float* gp = p.g_part + ((int64_t)b * NM * Hq + h) * 2 * N + n;
        float acc = 0.f;
        for (int i = 0; i < NM; ++i) acc = fmaf(__shfl_sync(0xffffffffu, wi, (p.n_il_chunks + i) & 31), gp[(int64_t)i * Hq * 2 * N], acc);
        Gs[n] = acc;
      }
    }
    for (int d = tid + FIN_THREADS; d < D; d += FIN_THREADS) {           // D > 512 only
      const float* op = p.o_part + ((int64_t)b * NCH * Hq + h) * D + d;
      float acc = 0.f;
      for (int i = 0; i < NCH; ++i) acc = fmaf(__shfl_sync(0xffffffffu, wi, i), op[(int64_t)i * Hq * D], acc);
      O[d] = acc;
    }
  } else {
    if (tid < 32) {
      float ms = NEG_BIG;
      for (int i = tid; i < NCH; i += 32) {
        const int64_t o = ((int64_t)b * NCH + i) * Hq + h;
        if (p.l_part[o] > 0.f) ms = fmaxf(ms, p.m_part[o]);
      }
      ms = warp_max(ms);
      float Ls = 0.f, Ps = 0.f;
      for (int i = tid; i < NCH; i += 32) {
        const int64_t o = ((int64_t)b * NCH + i) * Hq + h;
        const float l = p.l_part[o];
        const float w = (l > 0.f) ? exp2f(p.m_part[o] - ms) : 0.f;
        aw[i] = w;
        Ls = fmaf(w, l, Ls);
        if (i >= p.n_il_chunks) Ps = fmaf(w, l, Ps);
      }
      Ls = warp_sum(Ls);
      Ps = warp_sum(Ps);
      if (tid == 0) {
        s_L = Ls;
        s_P = Ps;
        s_ms = ms;
      }
    }
    __syncthreads();
    if (mid) {
      for (int n = tid; n < 2 * N; n += FIN_THREADS) {
        const float* gp = p.g_part + ((int64_t)b * NM * Hq + h) * 2 * N + n;
        float acc = 0.f;
#pragma unroll 8
        for (int i = 0; i < NM; ++i) acc = fmaf(aw[p.n_il_chunks + i], gp[(int64_t)i * Hq * 2 * N], acc);
        Gs[n] = acc;
      }
    }
    for (int d = tid; d < D; d += FIN_THREADS) {
      const float* op = p.o_part + ((int64_t)b * NCH * Hq + h) * D + d;
      float acc = 0.f;
#pragma unroll 8
      for (int i = 0; i < NCH; ++i) acc = fmaf(aw[i], op[(int64_t)i * Hq * D], acc);
      O[d] = acc;
    }
    __syncthreads();   // s_L, s_P, s_ms are read below
    P = s_P;
    L = s_L;
    ms_all = s_ms;
  }
  __syncthreads();
  const int c0 = mid ? a.vc_h[g] : 0, c1 = mid ? a.vc_h[g + 1] : 0;
  const bool vec = (Mc & 3) == 0;   // coefficient rows start on 16-byte boundaries
  const int W = vec ? 4 : 1;
  const int ca = vec ? (c0 & ~3) : c0;
  const int nck = (c1 - ca + W - 1) / W;   // column groups of the segment
  if (nck > 0) {
    // thread = (column group, slice of the 2N rows)
    const int nsl = FIN_THREADS / nck;
    const int ck = tid % nck, sl = tid / nck;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (sl < nsl) {
      const float* cp = a.v_coef + (int64_t)b * 2 * N * Mc + ca + W * ck;
      if (vec) {
#pragma unroll 8
        for (int n = sl; n < 2 * N; n += nsl) {
          const float4 cv = __ldg(reinterpret_cast<const float4*>(cp + (int64_t)n * Mc));
          const float gv = Gs[n];
          acc.x = fmaf(gv, cv.x, acc.x);
          acc.y = fmaf(gv, cv.y, acc.y);
          acc.z = fmaf(gv, cv.z, acc.z);
          acc.w = fmaf(gv, cv.w, acc.w);
        }
      } else {
#pragma unroll 8
        for (int n = sl; n < 2 * N; n += nsl) acc.x = fmaf(Gs[n], __ldg(cp + (int64_t)n * Mc), acc.x);
      }
    }
    *reinterpret_cast<float4*>(red + 4 * tid) = acc;
    __syncthreads();
    for (int c = c0 + tid; c < c1; c += FIN_THREADS) {
      const int ck2 = (c - ca) / W, e = (c - ca) - W * ck2;
      float s = 0.f;
      for (int s2 = 0; s2 < nsl; ++s2) s += red[4 * (s2 * nck + ck2) + e];
      const int64_t o = (int64_t)b * Mc + c;
      const float oc = a.scale_v[o] * (s / (float)N - a.avg_v_d[o] * P) + a.avg_v_u[o] * P;
      O[a.vc_list[c] - g * D] += oc;   // each compressed dim belongs to exactly one column
    }
  }
  __syncthreads();
  // a kernel of this call gave up a bounded wait: make the failure visible instead of returning numbers
  const bool poisoned = mid && (*p.err != 0);
  const float inv = poisoned ? __int_as_float(0x7fc00000) : 1.0f / L;
  for (int d = tid; d < D; d += FIN_THREADS) a.out[((int64_t)b * Hq + h) * D + d] = O[d] * inv;
  if (tid == 0) {
    if (a.m_out) a.m_out[(int64_t)b * Hq + h] = ms_all;
    if (a.l_out) a.l_out[(int64_t)b * Hq + h] = L;
  }
}

// log-sum-exp merge of normalised partial results
__global__ void merge_kernel(const float* __restrict__ o, const float* __restrict__ m, const float* __restrict__ l,
                             int n_parts, int rows, int D, float* __restrict__ out) {
  const int row = blockIdx.x;
  float ms = NEG_BIG;
  for (int i = 0; i < n_parts; ++i)
    if (l[(int64_t)i * rows + row] > 0.f) ms = fmaxf(ms, m[(int64_t)i * rows + row]);
  float den = 0.f;
  for (int i = 0; i < n_parts; ++i) {
    const float li = l[(int64_t)i * rows + row];
    if (li > 0.f) den += li * exp2f(m[(int64_t)i * rows + row] - ms);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < n_parts; ++i) {
      const float li = l[(int64_t)i * rows + row];
      if (li > 0.f) acc = fmaf(li * exp2f(m[(int64_t)i * rows + row] - ms), o[((int64_t)i * rows + row) * D + d], acc);
    }
    out[(int64_t)row * D + d] = acc / den;
  }
}

// ---------------------------------------------------------------------------------------------
// host side: plan, validation, launches
// ---------------------------------------------------------------------------------------------
constexpr int SMEM_LIMIT = 200 * 1024;

// Switches of the planner.  The one-shot entry points read them from the environment on every call (FA_DECODE_EXACT,
// FA_DECODE_NO_WS, FA_DECODE_NO_TMEM); a layer handle reads them once when it is created.
struct PlanFlags {
  bool force_exact, no_ws, ws_tmem;
};
static PlanFlags env_flags() {
  PlanFlags f;
  f.force_exact = getenv("FA_DECODE_EXACT") != nullptr;
  f.no_ws = getenv("FA_DECODE_NO_WS") != nullptr;
  f.ws_tmem = getenv("FA_DECODE_NO_TMEM") == nullptr;   // spectral accumulator in tensor memory where the shape allows
  return f;
}

// scratch layout (floats, each block 16-byte aligned); depends on the plan's chunk counts only
static void bind_scratch(DecodeParams& p, void* scratch) {
  const fa_decode_args_t& a = p.a;
  int64_t o = 0;
  auto take = [&](int64_t n) {
    int64_t r = o;
    o += (n + 3) / 4 * 4;
    return r;
  };
  const int64_t B = a.B, Hq = a.Hq;
  const int64_t ow = take(B * Hq * 2 * a.N), oc = take(B * Hq), om = take(B * p.NCH * Hq), ol = take(B * p.NCH * Hq);
  const int64_t oo = take(B * p.NCH * Hq * a.D), og = take(B * p.n_mid_chunks * Hq * 2 * a.N);
  const int64_t oe = take(4);
  const int64_t ot = take(p.ws2 ? ws2_table_floats(a.N) : 0);
  p.scratch_floats = o;
  float* s = reinterpret_cast<float*>(scratch);
  p.w = s + ow; p.cst = s + oc; p.m_part = s + om; p.l_part = s + ol; p.o_part = s + oo; p.g_part = s + og;
  p.err = reinterpret_cast<int*>(s + oe);
  p.tab = s + ot;
}

static int make_plan(const fa_decode_args_t& a, DecodeParams& p, const PlanFlags& flags) {
  FA_REQUIRE(a.B > 0 && a.Hq > 0 && a.Hkv > 0 && a.D > 0, FA_ERR_SHAPE, "fa_decode_attn: B, Hq, Hkv, D must be positive");
  FA_REQUIRE(a.Hq % a.Hkv == 0, FA_ERR_SHAPE, "fa_decode_attn: Hq (%d) must be a multiple of Hkv (%d)", a.Hq, a.Hkv);
  FA_REQUIRE(a.dtype == FA_DTYPE_F16 || a.dtype == FA_DTYPE_BF16, FA_ERR_DTYPE, "fa_decode_attn: bad dtype %d", a.dtype);
  FA_REQUIRE(a.n_sink >= 0 && a.n_win >= 0 && a.n_mid >= 0 && a.n_sink + a.n_win + a.n_mid > 0, FA_ERR_SHAPE,
             "fa_decode_attn: no keys to attend");
  FA_REQUIRE(a.D % 8 == 0, FA_ERR_ALIGN, "fa_decode_attn: head_dim (%d) must be a multiple of 8", a.D);
  p.a = a;
  p.force_exact = flags.force_exact;
  p.sink_row0 = 0;
  p.win_row0 = 0;
  p.R = a.Hq / a.Hkv;
  FA_REQUIRE(p.R <= R_MAX, FA_ERR_CAPACITY, "fa_decode_attn: at most %d query heads per KV head (got %d)", R_MAX, p.R);
  p.F = a.Hkv * a.D;
  FA_REQUIRE(p.F <= 2048, FA_ERR_CAPACITY, "fa_decode_attn: Hkv*D (%d) exceeds 2048", p.F);
  p.n_il = a.n_sink + a.n_win;
  const float sc = (a.sm_scale > 0.f) ? a.sm_scale : 1.0f / sqrtf((float)a.D);
  p.c2 = sc * 1.4426950408889634f;
  p.Hqp = rup(a.Hq, 4);
  // sinks + window tiles
  int TR = 128;
  while (TR > 8 && TR * p.F > 32768) TR >>= 1;
  p.TR = TR;
  const int il_smem = il_smem_bytes(TR, p.F, a.Hq, p.Hqp, a.D);
  p.n_il_chunks = p.n_il > 0 ? ceil_div(p.n_il, 256) : 0;
  p.il_chunk_rows = p.n_il > 0 ? rup(ceil_div(p.n_il, p.n_il_chunks), TR) : TR;
  p.n_il_chunks = p.n_il > 0 ? ceil_div(p.n_il, p.il_chunk_rows) : 0;

  int mid_smem_bytes = 0, il_smem_fast = 0;
  p.J = 8; p.kvh = 1; p.HG = p.R; p.HGp = 8; p.n_groups = 1; p.pitchK = p.pitchV = 16; p.qpitch = 4;
  p.n_mid_chunks = 0; p.mid_chunk = 8;
  p.fast = 0; p.fNT = 1; p.fNH = 1; p.wsSEQ = 1; p.wsNTs = 1; p.ws2 = 0; p.w_frag = 0; p.TRm = 16; p.il_tpc = 1;
  if (a.n_mid > 0) {
    FA_REQUIRE(a.N > 0 && a.T > 0, FA_ERR_SHAPE, "fa_decode_attn: N and T must be positive");
    FA_REQUIRE(a.N <= 1024, FA_ERR_CAPACITY, "fa_decode_attn: N (%d) exceeds 1024", a.N);
    FA_REQUIRE(a.Mc_k >= 0 && a.Mn_k >= 0 && a.Mc_k + a.Mn_k == p.F && a.Mc_v >= 0 && a.Mn_v >= 0 &&
                   a.Mc_v + a.Mn_v == p.F, FA_ERR_SHAPE,
               "fa_decode_attn: compressed + verbatim dims must add up to Hkv*D for K and for V");
    FA_REQUIRE(a.k_mn_sk >= a.Mn_k && a.v_mn_sk >= a.Mn_v, FA_ERR_SHAPE, "fa_decode_attn: verbatim row stride too small");
    int J = 32;
    while (J > 8 && J * a.N > 8192) J >>= 1;
    p.J = J;
    bool ok = false;
    for (int kvh = a.Hkv; kvh >= 1; --kvh) {
      const int HG = kvh * p.R, HGp = rup(HG, 8);
      if ((int64_t)HGp * 2 * a.N > 16384) continue;           // W' and the g accumulators
      if ((int64_t)a.N * (HGp / 8) > IT_G * DEC_THREADS) continue;
      const int boundK = a.Mn_k < kvh * a.D ? a.Mn_k : kvh * a.D;
      const int boundV = a.Mn_v < kvh * a.D ? a.Mn_v : kvh * a.D;
      if (boundV > IT_V * DEC_THREADS) continue;
      const int pitchK = rup(boundK, 8) + 16, pitchV = rup(boundV, 8) + 16;
      const int qpitch = rup((a.Mn_k < a.D ? a.Mn_k : a.D) + 1, 4);
      const MidSmem L = mid_smem(J, a.N, HGp, kvh, pitchK, pitchV, qpitch);
      if (L.total > SMEM_LIMIT) continue;
      p.kvh = kvh; p.HG = HG; p.HGp = HGp; p.pitchK = pitchK; p.pitchV = pitchV; p.qpitch = qpitch;
      p.n_groups = ceil_div(a.Hkv, kvh);
      mid_smem_bytes = L.total;
      ok = true;
      break;
    }
    FA_REQUIRE(ok, FA_ERR_UNSUPPORTED, "fa_decode_attn: no head grouping fits shared memory (N=%d, R=%d, D=%d)", a.N,
               p.R, a.D);
    // tensor-core pass: usable when the spectral score turns by at most 1.5 cycles over a 128- or
    // 64-token super-tile (interpolation through 16 nodes is then exact to ~1e-7) and the shape fits
    // its register / shared-memory tiling; otherwise the exact CUDA-core pass above is used
    p.fast = 0;
    p.wsSEQ = 1;
    p.wsNTs = 1;
    p.wsGN = 4; p.wsHG = 1; p.wsNB = 2; p.wsSlotK = 64; p.wsSlotV = 64; p.wsHPT = 8; p.wsKS = 4;
    {
      const int NT = ceil_div(a.Hq, 8);
      auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
      // rows per tile of the tensor-core sinks+window pass: three ring stages have to fit
      int TRm = 128;
      while (TRm > 16 && il_mma_smem(TRm, p.F, a.Hkv, a.D, a.dtype == FA_DTYPE_BF16).total > 227 * 1024) TRm >>= 1;
      il_smem_fast = il_mma_smem(TRm, p.F, a.Hkv, a.D, a.dtype == FA_DTYPE_BF16).total;
      p.TRm = TRm;
      const bool shape_ok = a.N % 8 == 0 && a.N <= 256 && NT <= FNT_MAX && a.Mn_k <= 256 && a.Mn_v <= 256 &&
                            a.D % 16 == 0 && il_smem_fast <= 227 * 1024;
      const bool align_ok = (a.Mn_k == 0 || (al16(a.k_mn) && a.k_mn_sk % 8 == 0 && a.k_mn_sb % 8 == 0)) &&
                            (a.Mn_v == 0 || (al16(a.v_mn) && a.v_mn_sk % 8 == 0 && a.v_mn_sb % 8 == 0));
      int NH = 0;
      if ((int64_t)128 * (a.N - 1) * 2 <= (int64_t)3 * a.T) NH = 2;
      else if ((int64_t)64 * (a.N - 1) * 2 <= (int64_t)3 * a.T) NH = 1;
      if (shape_ok && align_ok && NH > 0 && !p.force_exact) {
        const FastSmem L = fast_smem(a.N, NT, NH, a.Mn_k, a.Mn_v, a.dtype == FA_DTYPE_BF16);
        if (L.total <= 227 * 1024) {
          p.fast = 1; p.fNT = NT; p.fNH = NH;
          p.n_groups = 1; p.kvh = a.Hkv; p.HG = a.Hq;
          J = FH * NH;
          p.J = J;
          mid_smem_bytes = L.total;
        }
      }
      // warp-specialised form: 128-token super-tiles, and every 8-head column tile must find its
      // verbatim columns inside WS_KS (K) and WS_MTV (V) 16-column tiles, which only the host copies
      // of the offset tables can tell.  Up to 2N = 512 coefficient rows a CTA serves four column tiles;
      // up to 2N = 1024 the heads are divided into groups of 16 (two column tiles per CTA) and a CTA
      // fetches the verbatim columns of its own KV heads only.
      // heads per column tile: 8, or the largest multiple of the GQA ratio below 8 when 8 is not one (a tile then
      // never cuts the query heads of a KV head in two)
      const int HPT = (p.R >= 8 || 8 % p.R == 0) ? 8 : (8 / p.R) * p.R;
      const int NTw = ceil_div(a.Hq, HPT);
      const bool ws_shape = a.N % 8 == 0 && a.N <= 512 && NTw <= FNT_MAX && a.D % 16 == 0 && il_smem_fast <= 227 * 1024;
      if (ws_shape && align_ok && NH == 2 && a.kn_h_host && a.vn_h_host && !flags.no_ws && !p.force_exact) {
        const int NT = NTw;
        int steps = 1;   // most 16-column steps a tile needs for its verbatim K or V columns
        for (int nt = 0; nt < NT; ++nt) {
          const int g0 = (HPT * nt) / p.R, last = (a.Hq < HPT * nt + HPT ? a.Hq : HPT * nt + HPT) - 1, g1 = last / p.R;
          const int kc0 = a.kn_h_host[g0] & ~15, kc1 = (a.kn_h_host[g1 + 1] + 15) & ~15;
          const int mtv0 = a.vn_h_host[g0] >> 4, mtvn = ((a.vn_h_host[g1 + 1] + 15) >> 4) - mtv0;
          if ((kc1 - kc0) / 16 > steps) steps = (kc1 - kc0) / 16;
          if (mtvn > steps) steps = mtvn;
        }
        const bool ok = steps <= WS_KS_MAX;
        const int KS = (steps <= 4 && HPT == 8) ? 4 : 8;   // the KS = 4 instances are compiled for 8 heads per tile
        const int GN = a.N <= 256 ? 4 : 2;            // column tiles per CTA
        const int HGn = ceil_div(NT, GN);             // head groups per sequence
        const int NB = a.N <= 256 ? 2 : 1;            // node-basis buffers
        // widest run of 64-column boxes a CTA fetches per sequence (its head group's KV heads)
        int nbK = 0, nbV = 0;
        for (int hg = 0; hg < HGn; ++hg) {
          const int hb = hg * HPT * GN, gA = hb / p.R;
          const int gB = ((a.Hq < hb + HPT * GN ? a.Hq : hb + HPT * GN) - 1) / p.R;
          const int k0 = a.kn_h_host[gA] & ~63, v0 = a.vn_h_host[gA] & ~63;
          const int bk = ceil_div(a.kn_h_host[gB + 1] - k0, 64), bv = ceil_div(a.vn_h_host[gB + 1] - v0, 64);
          if (bk > nbK) nbK = bk;
          if (bv > nbV) nbV = bv;
        }
        // sequences per CTA: as many as fill the four column tiles (and the 32 lanes that issue their boxes)
        int seq = HGn > 1 ? 1 : FNT_MAX / NT;
        if (GN != 4) seq = 1;
        if (seq > a.B) seq = a.B;
        while (seq > 1 && (seq * (nbK > nbV ? nbK : nbV) > 32 ||
                           ws_smem(a.N, seq * nbK * 64, seq * nbV * 64, NB, 8 / GN).total > 227 * 1024))
          --seq;
        const WsSmem L = ws_smem(a.N, seq * nbK * 64, seq * nbV * 64, NB, 8 / GN);
        const Ws2Smem L2 = ws2_smem(a.N, seq * nbK * 64, seq * nbV * 64);
        // the tensor-memory form where it applies: measured at the Llama-3.1-8B / 32k layer it takes 0.114 ms per launch
        // against 0.133 ms of the form that keeps the accumulator in registers
        p.ws2 = (flags.ws_tmem && GN == 4 && HPT == 8 && KS == 4 && a.Mn_k <= W2_IDX && a.Mn_v <= W2_IDX && a.Hkv < 40 &&
                 L2.total <= 227 * 1024) ? 1 : 0;
        const int need = p.ws2 ? L2.total : L.total;
        if (ok && need <= 227 * 1024 && (nbK > nbV ? nbK : nbV) <= 32) {
          p.fast = 2;
          p.w_frag = 1;
          if (p.ws2) {
            // The sinks+window pass has 112 registers inside the tensor-memory kernel, and what it spills is reloaded
            // from L2 behind the K / V stream: tiles of at most 32 rows (two 16-row blocks, no spills), 64 rows with a
            // single KV head (measured: 2 KV heads 3.45 -> 3.02 ms per step with 32-row tiles, 1 KV head 3.07 ->
            // 2.95 ms with 64-row tiles at the Llama-3.1-8B shard shapes)
            const int cap = a.Hkv == 1 ? 64 : 32;
            if (p.TRm > cap) {
              p.TRm = cap;
              il_smem_fast = il_mma_smem(cap, p.F, a.Hkv, a.D, a.dtype == FA_DTYPE_BF16).total;
            }
          }
          p.wsSEQ = seq;
          p.wsNTs = NT;
          p.wsGN = GN;
          p.wsHG = HGn;
          p.wsNB = NB;
          p.wsSlotK = seq * nbK * 64;
          p.wsSlotV = seq * nbV * 64;
          p.wsHPT = HPT;
          p.wsKS = KS;
          p.fNT = seq * NT;
          p.fNH = 2;
          p.n_groups = 1; p.kvh = a.Hkv; p.HG = a.Hq;
          J = 128;
          p.J = J;
          mid_smem_bytes = need;
        }
      }
    }
    const int sms = sm_count();
    // The split is made for the span length rounded up to whole super-tiles, so that the plan (chunk length,
    // chunk count, scratch need) stays the same while n_mid grows inside one super-tile; every chunk still
    // starts below n_mid.
    const int n_mid_r = rup(a.n_mid, J);
    const int max_chunks = n_mid_r / J;
    if (p.fast && p.n_il > 0) {
      // One wave of CTAs per launch.  Split the CTAs of a sequence between sinks+window rows and the
      // middle span so that the slowest CTA is as short as possible; costs in clock ticks as measured
      // on B200 (cost_il_row per sinks+window row, cost_mid_tok per middle-span token, plus set-up).
      // (the warp-specialised kernel serves wsSEQ sequences per middle-span CTA: count CTAs per such group)
      const int seqs = p.fast == 2 ? p.wsSEQ : 1;
      const int per_seq = sms / ceil_div(a.B, seqs) > 2 * seqs ? sms / ceil_div(a.B, seqs) : 2 * seqs;
      // a sinks+window tile costs a fixed part (barriers, waits, refill) plus its MMA / softmax work, which
      // grows with rows x KV heads (7.2 K ticks for 16 rows x 8 heads)
      // (the warp-specialised kernels run 16-row tiles through a pass unrolled for exactly one 16-row block: 5.6 K
      // ticks per tile at 8 KV heads)
      // (next to middle-span CTAs of the tensor-memory form, which leave it less of the memory system, the same pass
      // was measured at 6.4 K ticks per tile; those CTAs take 7.5 K ticks per 128-token super-tile and 40 K of set-up)
      const bool tm = p.fast == 2 && p.ws2;
      const double cost_il_tile = (p.fast == 2 && p.TRm == 16) ? 2000.0 + (tm ? 34.0 : 28.0) * p.TRm * a.Hkv : 2500.0 + 37.0 * p.TRm * a.Hkv;
      const double cost_mid_tok = p.fast == 2 ? (tm ? 60.0 : p.wsGN == 2 ? 130.0 : 100.0) : 142.0;
      const double cost_mid_fix = tm ? 40000.0 : 24000.0;
      const int n_tiles = ceil_div(a.n_sink, p.TRm) + ceil_div(a.n_win, p.TRm);
      double best = 1e30;
      int best_il = 1;
      const int hgs = p.fast == 2 ? p.wsHG : 1;   // CTAs per middle-span chunk (one per head group)
      for (int n_il = 1; n_il < per_seq && n_il <= n_tiles; ++n_il) {
        const int tpc = ceil_div(n_tiles, n_il);
        int n_mid = (per_seq - seqs * ceil_div(n_tiles, tpc)) / hgs;
        if (n_mid < 1) break;
        if (n_mid > max_chunks) n_mid = max_chunks;
        const int mid_tok = rup(ceil_div(n_mid_r, n_mid), J);
        const double t_il = 8000.0 + cost_il_tile * tpc, t_mid = cost_mid_fix + cost_mid_tok * mid_tok;
        const double t = t_il > t_mid ? t_il : t_mid;
        if (t < best) {
          best = t;
          best_il = n_il;
        }
      }
      p.il_tpc = ceil_div(n_tiles, best_il);
      p.n_il_chunks = ceil_div(n_tiles, p.il_tpc);
      p.il_chunk_rows = p.il_tpc * p.TRm;
    }
    int target = ((p.fast ? 1 : 3) * sms) / (a.B * p.n_groups) - p.n_il_chunks;
    if (p.fast == 2) target = (sms / ceil_div(a.B, p.wsSEQ) - p.wsSEQ * p.n_il_chunks) / p.wsHG;
    if (target < 1) target = 1;
    if (target > max_chunks) target = max_chunks;
    p.mid_chunk = rup(ceil_div(n_mid_r, target), J);
    p.n_mid_chunks = ceil_div(n_mid_r, p.mid_chunk);
  }
  p.NCH = p.n_il_chunks + p.n_mid_chunks;
  const int il_need = p.fast ? il_smem_fast : il_smem;   // the 512-thread kernels run the sinks+window rows as MMAs
  p.smem_main = il_need > mid_smem_bytes ? il_need : mid_smem_bytes;
  if (p.n_il == 0) p.smem_main = mid_smem_bytes;
  FA_REQUIRE(p.smem_main <= 227 * 1024, FA_ERR_CAPACITY, "fa_decode_attn: shared memory need %d exceeds 227 KB", p.smem_main);
  p.smem_prepare = p.R * (a.D + 8) * 4;   // one KV head's column segment (at most D wide) plus alignment pads
  bind_scratch(p, a.scratch);
  return FA_OK;
}

// Raises a kernel's dynamic shared-memory limit; remembers per (device, kernel) what has been granted, so the
// attribute call is made once and not on every launch.
template <typename K>
static int set_smem(K kernel, int bytes) {
  if (bytes <= 48 * 1024) return FA_OK;
  struct Entry {
    int dev;
    const void* fn;
    int bytes;
  };
  static std::mutex mu;
  static Entry seen[256];
  static int n_seen = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  const void* fn = reinterpret_cast<const void*>(kernel);
  std::lock_guard<std::mutex> lock(mu);
  Entry* hit = nullptr;
  for (int i = 0; i < n_seen; ++i)
    if (seen[i].dev == dev && seen[i].fn == fn) hit = &seen[i];
  if (hit && hit->bytes >= bytes) return FA_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");
  if (hit) hit->bytes = bytes;
  else if (n_seen < 256) seen[n_seen++] = Entry{dev, fn, bytes};
  return FA_OK;
}

template <typename T>
static int launch_decode(const DecodeParams& p, cudaStream_t st) {
  const fa_decode_args_t& a = p.a;
  int rc;
  auto mark = [&](int i) {
    if (a.phase_events_host && a.phase_events_host[i]) cudaEventRecord((cudaEvent_t)a.phase_events_host[i], st);
  };
  mark(0);
  if (a.n_mid > 0) {
    if ((rc = set_smem(decode_prepare_kernel<T>, p.smem_prepare)) != FA_OK) return rc;
    dim3 g1(ceil_div(2 * a.N, DEC_THREADS), a.Hkv, a.B);
    decode_prepare_kernel<T><<<g1, DEC_THREADS, p.smem_prepare, st>>>(p);
    FA_CHECK_LAUNCH("fa_decode_attn(prepare)");
  }
  mark(1);
  dim3 g2(p.n_il_chunks + p.n_mid_chunks * p.n_groups, a.B);
  if (p.fast == 2) {
    const dim3 gw(p.wsSEQ * p.n_il_chunks + p.n_mid_chunks * p.wsHG, ceil_div(a.B, p.wsSEQ));
    if (p.ws2) {
      if ((rc = set_smem(decode_main_ws2_kernel<T>, p.smem_main)) != FA_OK) return rc;
      decode_main_ws2_kernel<T><<<gw, W2_T, p.smem_main, st>>>(p);
    } else {
#define FA_WS_CASE(GN_, KS_)                                                                 \
  if (p.wsGN == GN_ && p.wsKS == KS_) {                                                       \
    if ((rc = set_smem(decode_main_ws_kernel<T, GN_, KS_>, p.smem_main)) != FA_OK) return rc; \
    decode_main_ws_kernel<T, GN_, KS_><<<gw, WS_T, p.smem_main, st>>>(p);                     \
  }
      FA_WS_CASE(4, 4) FA_WS_CASE(4, 8) FA_WS_CASE(2, 4) FA_WS_CASE(2, 8)
#undef FA_WS_CASE
    }
  } else if (p.fast) {
#define FA_FAST_CASE(NT_, NH_)                                                                   \
  if (p.fNT == NT_ && p.fNH == NH_) {                                                            \
    if ((rc = set_smem(decode_main_fast_kernel<T, NT_, NH_>, p.smem_main)) != FA_OK) return rc;  \
    decode_main_fast_kernel<T, NT_, NH_><<<g2, FAST_THREADS, p.smem_main, st>>>(p);               \
  }
    FA_FAST_CASE(1, 1) FA_FAST_CASE(2, 1) FA_FAST_CASE(3, 1) FA_FAST_CASE(4, 1)
    FA_FAST_CASE(1, 2) FA_FAST_CASE(2, 2) FA_FAST_CASE(3, 2) FA_FAST_CASE(4, 2)
#undef FA_FAST_CASE
  } else {
    if ((rc = set_smem(decode_main_kernel<T>, p.smem_main)) != FA_OK) return rc;
    decode_main_kernel<T><<<g2, DEC_THREADS, p.smem_main, st>>>(p);
  }
  FA_CHECK_LAUNCH("fa_decode_attn(main)");
  mark(2);
  mark(3);
  dim3 g4(a.Hq, a.B);
  const int smem_fin = finish_smem_bytes(p.NCH, a.n_mid > 0 ? a.N : 0, a.D);
  if ((rc = set_smem(decode_finish_kernel, smem_fin)) != FA_OK) return rc;
  decode_finish_kernel<<<g4, FIN_THREADS, smem_fin, st>>>(p);
  FA_CHECK_LAUNCH("fa_decode_attn(finish)");
  mark(4);
  return FA_OK;
}

// ---------------------------------------------------------------------------------------------
// Scratch for callers that must not allocate: a fixed array in device memory, owned by this
// library.  Every GPU that loads the library holds these bytes until the process exits.
// In host code the array's name is only a handle (not a device address), so the address is looked
// up once per device with cudaGetSymbolAddress and that pointer is what the kernels receive.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[FA_DECODE_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;

static int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* ptrs[MAX_DEVICES] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  FA_REQUIRE(dev >= 0 && dev < MAX_DEVICES, FA_ERR_CAPACITY, "fa_decode_attn_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);   // resolves against the current device
    if (e != cudaSuccess || p == nullptr) return cuda_fail(e, "cudaGetSymbolAddress(g_static_scratch)");
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return FA_OK;
}

}  // namespace fa

using namespace fa;

extern "C" size_t fa_decode_scratch_bytes(const fa_decode_args_t* args) {
  if (!args) return 0;
  DecodeParams p;
  fa_decode_args_t a = *args;
  a.scratch = nullptr;
  if (make_plan(a, p, env_flags()) != FA_OK) return 0;
  return (size_t)p.scratch_floats * sizeof(float);
}

extern "C" int fa_decode_path(const fa_decode_args_t* args) {
  FA_REQUIRE(args, FA_ERR_NULL, "fa_decode_path: null argument block");
  DecodeParams p;
  fa_decode_args_t a = *args;
  a.scratch = nullptr;
  int rc = make_plan(a, p, env_flags());
  if (rc != FA_OK) return rc;
  return a.n_mid > 0 ? (p.fast == 2 && p.ws2 ? 3 : p.fast) : 0;
}

// Pointer / alignment checks of a planned call (p.a holds the caller's arguments, scratch already bound).
static int validate_planned(const DecodeParams& p) {
  const fa_decode_args_t& a = p.a;
  FA_REQUIRE(a.q && a.out, FA_ERR_NULL, "fa_decode_attn: q / out is null");
  FA_REQUIRE(a.n_sink == 0 || (a.k_sink && a.v_sink), FA_ERR_NULL, "fa_decode_attn: sink rows are null");
  FA_REQUIRE(a.n_win == 0 || (a.k_win && a.v_win), FA_ERR_NULL, "fa_decode_attn: window rows are null");
  if (a.n_mid > 0) {
    FA_REQUIRE(a.Mc_k == 0 || (a.k_coef && a.avg_k_u && a.avg_k_d && a.scale_k), FA_ERR_NULL,
               "fa_decode_attn: K coefficient or statistics pointer is null");
    FA_REQUIRE(a.Mc_v == 0 || (a.v_coef && a.avg_v_u && a.avg_v_d && a.scale_v), FA_ERR_NULL,
               "fa_decode_attn: V coefficient or statistics pointer is null");
    FA_REQUIRE((a.Mn_k == 0 || a.k_mn) && (a.Mn_v == 0 || a.v_mn), FA_ERR_NULL, "fa_decode_attn: verbatim store is null");
    FA_REQUIRE(a.kc_h && a.kn_h && a.vc_h && a.vn_h && (a.Mc_k == 0 || a.kc_list) && (a.Mc_v == 0 || a.vc_list) &&
                   (a.Mn_k == 0 || a.kn_list) && (a.Mn_v == 0 || a.vn_list), FA_ERR_NULL,
               "fa_decode_attn: index table is null");
    FA_REQUIRE(a.mid_l0 >= 0, FA_ERR_SHAPE, "fa_decode_attn: mid_l0 must be non-negative");
  }
  FA_REQUIRE(a.scratch && a.scratch_bytes >= (size_t)p.scratch_floats * sizeof(float), FA_ERR_CAPACITY,
             "fa_decode_attn: scratch too small (%zu < %zu bytes)", a.scratch_bytes,
             (size_t)p.scratch_floats * sizeof(float));
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  FA_REQUIRE(al16(a.scratch) && al16(a.q), FA_ERR_ALIGN, "fa_decode_attn: q and scratch must be 16-byte aligned");
  if (a.n_sink > 0)
    FA_REQUIRE(al16(a.k_sink) && al16(a.v_sink) && a.sink_sb % 8 == 0, FA_ERR_ALIGN,
               "fa_decode_attn: sink rows must be 16-byte aligned");
  if (a.n_win > 0)
    FA_REQUIRE(al16(a.k_win) && al16(a.v_win) && a.win_sb % 8 == 0, FA_ERR_ALIGN,
               "fa_decode_attn: window rows must be 16-byte aligned");
  FA_REQUIRE(a.q_sb % 8 == 0 || a.B == 1, FA_ERR_ALIGN, "fa_decode_attn: q batch stride must be a multiple of 8");
  return FA_OK;
}

// One-shot form: tensor maps over exactly the rows of this call (rows past them read as zeros).
static int decode_planned(DecodeParams& p, cudaStream_t st) {
  const fa_decode_args_t& a = p.a;
  int rc = validate_planned(p);
  if (rc != FA_OK) return rc;
  if (p.fast) {
    if (a.n_sink > 0 &&
        ((rc = make_tensor_map_3d(&p.tm_ks, a.k_sink, a.dtype, p.F, a.n_sink, p.F, a.B, a.sink_sb, 64, p.TRm)) != FA_OK ||
         (rc = make_tensor_map_3d(&p.tm_vs, a.v_sink, a.dtype, p.F, a.n_sink, p.F, a.B, a.sink_sb, 64, p.TRm)) != FA_OK))
      return rc;
    if (a.n_win > 0 &&
        ((rc = make_tensor_map_3d(&p.tm_kw, a.k_win, a.dtype, p.F, a.n_win, p.F, a.B, a.win_sb, 64, p.TRm)) != FA_OK ||
         (rc = make_tensor_map_3d(&p.tm_vw, a.v_win, a.dtype, p.F, a.n_win, p.F, a.B, a.win_sb, 64, p.TRm)) != FA_OK))
      return rc;
    if (a.Mn_k > 0 && (rc = make_tensor_map_3d(&p.tm_k, a.k_mn, a.dtype, a.Mn_k, a.n_mid, a.k_mn_sk, a.B, a.k_mn_sb, 64, 64)) != FA_OK)
      return rc;
    if (a.Mn_v > 0 && (rc = make_tensor_map_3d(&p.tm_v, a.v_mn, a.dtype, a.Mn_v, a.n_mid, a.v_mn_sk, a.B, a.v_mn_sb, 64, 64)) != FA_OK)
      return rc;
  }
  return a.dtype == FA_DTYPE_F16 ? launch_decode<__half>(p, st) : launch_decode<__nv_bfloat16>(p, st);
}

extern "C" int fa_decode_attn(const fa_decode_args_t* args, fa_stream_t stream) {
  FA_REQUIRE(args, FA_ERR_NULL, "fa_decode_attn: null argument block");
  DecodeParams p;
  int rc = make_plan(*args, p, env_flags());
  if (rc != FA_OK) return rc;
  return decode_planned(p, (cudaStream_t)stream);
}

extern "C" int fa_merge(const float* o, const float* m, const float* l, int n_parts, int rows, int D, float* out,
                        fa_stream_t stream) {
  FA_REQUIRE(n_parts > 0 && rows > 0 && D > 0, FA_ERR_SHAPE, "fa_merge: sizes must be positive");
  FA_REQUIRE(o && m && l && out, FA_ERR_NULL, "fa_merge: null pointer");
  merge_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>(o, m, l, n_parts, rows, D, out);
  FA_CHECK_LAUNCH("fa_merge");
  return FA_OK;
}

extern "C" int fa_decode_attn_static(const fa_decode_args_t* args, fa_stream_t stream) {
  FA_REQUIRE(args, FA_ERR_NULL, "fa_decode_attn_static: null argument block");
  fa_decode_args_t a = *args;
  a.scratch = nullptr;
  a.scratch_bytes = 0;
  DecodeParams p;
  int rc = make_plan(a, p, env_flags());
  if (rc != FA_OK) return rc;
  const size_t need = (size_t)p.scratch_floats * sizeof(float);
  FA_REQUIRE(need <= (size_t)FA_DECODE_STATIC_SCRATCH_BYTES, FA_ERR_CAPACITY,
             "fa_decode_attn_static: this problem needs %zu bytes of scratch, the built-in buffer holds %zu; "
             "use fa_decode_attn with caller-provided scratch", need, (size_t)FA_DECODE_STATIC_SCRATCH_BYTES);
  void* ptr = nullptr;
  rc = static_scratch_address(&ptr);
  if (rc != FA_OK) return rc;
  p.a.scratch = ptr;
  p.a.scratch_bytes = (size_t)FA_DECODE_STATIC_SCRATCH_BYTES;
  bind_scratch(p, ptr);   // the plan made above stands; only the scratch pointers move
  return decode_planned(p, (cudaStream_t)stream);
}


// ---------------------------------------------------------------------------------------------
// Layer handle: everything of one cached layer that does not change between decode steps is bound once
// (buffers, tables, statistics, planner switches, tensor maps over the WHOLE allocations), so a decode
// step costs two short calls on the host.  The window slides inside its buffer and the middle span
// grows by a row per step; both enter as plain integers (window offset, n_mid): the window's position is
// a row coordinate of the tensor-copy requests, n_mid bounds the tokens a chunk walks.  The plan is kept
// while n_mid stays inside one super-tile and the query-head count does not change.
// ---------------------------------------------------------------------------------------------
struct fa_layer {
  fa_layer_desc_t d;
  PlanFlags flags;
  DecodeParams p;
  bool planned, maps_ready;
  int plan_lo, plan_hi, plan_Hq, plan_TRm, plan_fast;
  int last_path;
};

extern "C" int fa_layer_create(const fa_layer_desc_t* desc, fa_layer_t** out) {
  FA_REQUIRE(desc && out, FA_ERR_NULL, "fa_layer_create: null argument");
  const fa_layer_desc_t& d = *desc;
  FA_REQUIRE(d.B > 0 && d.Hkv > 0 && d.D > 0 && d.S >= 0 && d.W > 0 && d.N > 0 && d.T > 0 && d.T_c > 0, FA_ERR_SHAPE,
             "fa_layer_create: sizes must be positive");
  FA_REQUIRE(d.dtype == FA_DTYPE_F16 || d.dtype == FA_DTYPE_BF16, FA_ERR_DTYPE, "fa_layer_create: bad dtype %d", d.dtype);
  FA_REQUIRE(d.kbuf && d.vbuf && d.buf_rows >= d.S + 2 * d.W, FA_ERR_SHAPE,
             "fa_layer_create: the window buffers must hold S + 2W rows");
  FA_REQUIRE(d.unc_rows > 0 && (d.Mn_k == 0 || d.k_unc) && (d.Mn_v == 0 || d.v_unc), FA_ERR_NULL,
             "fa_layer_create: verbatim store missing");
  FA_REQUIRE(d.Mc_k + d.Mn_k == d.Hkv * d.D && d.Mc_v + d.Mn_v == d.Hkv * d.D, FA_ERR_SHAPE,
             "fa_layer_create: compressed + verbatim dims must add up to Hkv*D");
  fa_layer* L = new (std::nothrow) fa_layer();
  FA_REQUIRE(L != nullptr, FA_ERR_CAPACITY, "fa_layer_create: out of host memory");
  L->d = d;
  L->flags = env_flags();
  L->planned = false;
  L->maps_ready = false;
  L->last_path = 0;
  *out = L;
  return FA_OK;
}

extern "C" void fa_layer_destroy(fa_layer_t* layer) { delete layer; }

extern "C" int fa_layer_rebind_stores(fa_layer_t* L, void* k_unc, void* v_unc, int64_t k_unc_sb, int64_t v_unc_sb,
                                      int64_t k_unc_sk, int64_t v_unc_sk, int32_t unc_rows) {
  FA_REQUIRE(L, FA_ERR_NULL, "fa_layer_rebind_stores: null handle");
  L->d.k_unc = k_unc; L->d.v_unc = v_unc;
  L->d.k_unc_sb = k_unc_sb; L->d.v_unc_sb = v_unc_sb; L->d.k_unc_sk = k_unc_sk; L->d.v_unc_sk = v_unc_sk;
  L->d.unc_rows = unc_rows;
  L->planned = false;
  L->maps_ready = false;
  return FA_OK;
}

extern "C" int fa_layer_update(fa_layer_t* L, int32_t win_off, int32_t n_mid, int64_t phase, int32_t appends,
                               const void* k_new, const void* v_new, int64_t new_sb, int64_t new_sh,
                               fa_stream_t stream) {
  FA_REQUIRE(L, FA_ERR_NULL, "fa_layer_update: null handle");
  const fa_layer_desc_t& d = L->d;
  FA_REQUIRE(win_off >= 0 && win_off < d.W && n_mid >= 0, FA_ERR_SHAPE, "fa_layer_update: bad window offset or n_mid");
  FA_REQUIRE(!appends || n_mid < d.unc_rows, FA_ERR_CAPACITY, "fa_layer_update: the verbatim stores are full (%d rows)",
             d.unc_rows);
  const int64_t F = (int64_t)d.Hkv * d.D, es = 2;
  unsigned char* kb = reinterpret_cast<unsigned char*>(d.kbuf);
  unsigned char* vb = reinterpret_cast<unsigned char*>(d.vbuf);
  const int64_t row_b = (int64_t)(d.S + win_off) * F * es, dst_b = row_b + (int64_t)d.W * F * es;
  const int mn_k = appends ? d.Mn_k : 0, mn_v = appends ? d.Mn_v : 0;
  unsigned char* ku = reinterpret_cast<unsigned char*>(d.k_unc) + (int64_t)n_mid * d.k_unc_sk * es;
  unsigned char* vu = reinterpret_cast<unsigned char*>(d.v_unc) + (int64_t)n_mid * d.v_unc_sk * es;
  return fa_evict_step(d.Mc_k ? d.k_coef : nullptr, kb + row_b, d.buf_sb, d.kc_list, d.Mc_k,
                       d.Mc_v ? d.v_coef : nullptr, vb + row_b, d.buf_sb, d.vc_list, d.Mc_v, d.N, phase, d.T_c,
                       d.angle_mode, kb + row_b, vb + row_b, d.buf_sb, d.kn_list, mn_k, d.vn_list, mn_v, ku, d.k_unc_sb,
                       vu, d.v_unc_sb, k_new, v_new, new_sb, new_sh, kb + dst_b, vb + dst_b, d.buf_sb, d.dtype, d.B,
                       d.Hkv, d.D, stream);
}

// (re)plans for the query-head count and the super-tile n_mid lies in
static int layer_plan(fa_layer* L, int Hq, int n_mid, float sm_scale) {
  const fa_layer_desc_t& d = L->d;
  fa_decode_args_t a;
  memset(&a, 0, sizeof(a));
  a.B = d.B; a.Hq = Hq; a.Hkv = d.Hkv; a.D = d.D;
  a.n_sink = d.with_il ? d.S : 0;
  a.n_win = d.with_il ? d.W : 0;
  a.n_mid = n_mid; a.mid_l0 = d.mid_l0; a.N = d.N; a.T = d.T;
  a.Mc_k = d.Mc_k; a.Mn_k = d.Mn_k; a.Mc_v = d.Mc_v; a.Mn_v = d.Mn_v;
  a.dtype = d.dtype; a.sm_scale = sm_scale;
  a.k_sink = d.kbuf; a.v_sink = d.vbuf; a.sink_sb = d.buf_sb;
  a.k_win = d.kbuf; a.v_win = d.vbuf; a.win_sb = d.buf_sb;
  a.k_mn = d.k_unc; a.v_mn = d.v_unc; a.k_mn_sb = d.k_unc_sb; a.v_mn_sb = d.v_unc_sb;
  a.k_mn_sk = d.k_unc_sk; a.v_mn_sk = d.v_unc_sk;
  a.k_coef = d.k_coef; a.v_coef = d.v_coef;
  a.avg_k_u = d.avg_k_u; a.avg_k_d = d.avg_k_d; a.scale_k = d.scale_k;
  a.avg_v_u = d.avg_v_u; a.avg_v_d = d.avg_v_d; a.scale_v = d.scale_v;
  a.kc_list = d.kc_list; a.kc_h = d.kc_h; a.kn_list = d.kn_list; a.kn_h = d.kn_h;
  a.vc_list = d.vc_list; a.vc_h = d.vc_h; a.vn_list = d.vn_list; a.vn_h = d.vn_h;
  a.kn_h_host = d.kn_h_host; a.vn_h_host = d.vn_h_host;
  int rc = make_plan(a, L->p, L->flags);
  if (rc != FA_OK) return rc;
  DecodeParams& p = L->p;
  L->planned = true;
  L->plan_Hq = Hq;
  L->plan_hi = n_mid > 0 ? rup(n_mid, p.J) : 0;
  L->plan_lo = n_mid > 0 ? L->plan_hi - p.J : -1;
  L->last_path = n_mid > 0 ? (p.fast == 2 && p.ws2 ? 3 : p.fast) : 0;
  return FA_OK;
}

// tensor maps, one per buffer, over every row it owns: sinks at rows [0, S), the window wherever it has slid to;
// encoded once (again only if the stores are rebound or the tile height of the sinks+window pass changes)
static int layer_maps(fa_layer* L) {
  const fa_layer_desc_t& d = L->d;
  DecodeParams& p = L->p;
  if (!p.fast || (L->maps_ready && L->plan_TRm == p.TRm)) return FA_OK;
  int rc;
  if (d.with_il) {
    if ((rc = make_tensor_map_3d(&p.tm_ks, d.kbuf, d.dtype, p.F, d.buf_rows, p.F, d.B, d.buf_sb, 64, p.TRm)) != FA_OK ||
        (rc = make_tensor_map_3d(&p.tm_vs, d.vbuf, d.dtype, p.F, d.buf_rows, p.F, d.B, d.buf_sb, 64, p.TRm)) != FA_OK)
      return rc;
    p.tm_kw = p.tm_ks;
    p.tm_vw = p.tm_vs;
  }
  if (d.Mn_k > 0 && (rc = make_tensor_map_3d(&p.tm_k, d.k_unc, d.dtype, d.Mn_k, d.unc_rows, d.k_unc_sk, d.B, d.k_unc_sb, 64, 64)) != FA_OK)
    return rc;
  if (d.Mn_v > 0 && (rc = make_tensor_map_3d(&p.tm_v, d.v_unc, d.dtype, d.Mn_v, d.unc_rows, d.v_unc_sk, d.B, d.v_unc_sb, 64, 64)) != FA_OK)
    return rc;
  L->maps_ready = true;
  L->plan_TRm = p.TRm;
  return FA_OK;
}

static bool layer_plan_holds(const fa_layer* L, int Hq, int n_mid) {
  if (!L->planned || Hq != L->plan_Hq) return false;
  if (n_mid == 0) return L->plan_hi == 0;
  return n_mid > L->plan_lo && n_mid <= L->plan_hi;
}

extern "C" size_t fa_layer_scratch_bytes(fa_layer_t* L, int32_t Hq, int32_t n_mid) {
  if (!L) return 0;
  if (!layer_plan_holds(L, Hq, n_mid) && layer_plan(L, Hq, n_mid, -1.0f) != FA_OK) return 0;
  return (size_t)L->p.scratch_floats * sizeof(float);
}

extern "C" int fa_layer_decode_path(fa_layer_t* L) { return L ? L->last_path : FA_ERR_NULL; }

extern "C" int fa_layer_attend(fa_layer_t* L, int32_t win_off, int32_t n_mid, int32_t Hq, const void* q, int64_t q_sb,
                               float sm_scale, float* out, float* m_out, float* l_out, void* scratch,
                               size_t scratch_bytes, void* const* phase_events_host, fa_stream_t stream) {
  FA_REQUIRE(L, FA_ERR_NULL, "fa_layer_attend: null handle");
  const fa_layer_desc_t& d = L->d;
  FA_REQUIRE(win_off >= 0 && win_off <= d.W && n_mid >= 0 && n_mid <= d.unc_rows, FA_ERR_SHAPE,
             "fa_layer_attend: bad window offset or n_mid");
  int rc;
  if (!layer_plan_holds(L, Hq, n_mid) && (rc = layer_plan(L, Hq, n_mid, sm_scale)) != FA_OK) return rc;
  if ((rc = layer_maps(L)) != FA_OK) return rc;
  DecodeParams& p = L->p;
  fa_decode_args_t& a = p.a;
  const int64_t F = (int64_t)d.Hkv * d.D;
  a.n_mid = n_mid;
  a.q = q; a.q_sb = q_sb;
  a.sm_scale = sm_scale;
  const float sc = (sm_scale > 0.f) ? sm_scale : 1.0f / sqrtf((float)d.D);
  p.c2 = sc * 1.4426950408889634f;
  a.out = out; a.m_out = m_out; a.l_out = l_out;
  a.phase_events_host = phase_events_host;
  a.scratch = scratch; a.scratch_bytes = scratch_bytes;
  bind_scratch(p, scratch);
  if (d.with_il) {
    a.k_win = reinterpret_cast<unsigned char*>(d.kbuf) + (int64_t)(d.S + win_off) * F * 2;
    a.v_win = reinterpret_cast<unsigned char*>(d.vbuf) + (int64_t)(d.S + win_off) * F * 2;
    p.sink_row0 = 0;
    p.win_row0 = d.S + win_off;
  }
  if ((rc = validate_planned(p)) != FA_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  return d.dtype == FA_DTYPE_F16 ? launch_decode<__half>(p, st) : launch_decode<__nv_bfloat16>(p, st);
}
