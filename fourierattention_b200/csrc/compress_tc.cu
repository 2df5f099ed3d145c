// Forward projection (compression) on the 5th-generation tensor cores:
//   coef[2N x C] += Basis^T[2N x K] * X[K x C]      per sequence, C = every column of the source rows
// as tcgen05.mma (M = 128 frequency rows, N = 256 columns, K = 16 tokens per instruction) with the
// accumulator in tensor memory.  Per CTA: one 128-row block of the 2N basis rows, one 256-column block of
// X, one chunk of the token axis (split-K, partials reduced afterwards in a fixed order).
//
// Warp roles (448 threads):
//   warps 0-7  generate the basis tile of each stage straight into shared memory in the K-major
//              core-matrix layout the MMA reads (exact integer phase every 8 tokens, 3 rotations between),
//              split into 2 (fp16) or 3 (bf16) terms so that the 16-bit operand carries ~22 bits;
//   warp 8     streams X tiles with TMA (64-column x 32-token boxes, 128-byte swizzle = MN-major operand);
//   warp 9     owns tensor memory and issues the MMAs (one thread), releasing stages with tcgen05.commit;
//              it alternates between two accumulators, one per 256-token segment;
//   warps 10-13 drain the finished segment's accumulator (tcgen05.ld) and add it to the CTA's partial tile.
// Every wait is bounded; a wait that gives up sets a flag that makes the reduction write NaN.
#include <cuda.h>

#include <stdlib.h>

#include "common.cuh"

namespace fa {

constexpr int TC_KT = 32;        // tokens per stage
constexpr int TC_ST = 4;         // stages
constexpr int TC_NC = 256;       // columns per CTA (MMA N)
constexpr int TC_THREADS = 448;
constexpr int TC_SEG = 8;         // stages per accumulation segment (256 tokens): the tensor core adds into its
                                 // fp32 accumulator with truncation, so chains are kept short and the segments
                                 // are summed with round-to-nearest adds outside
constexpr int TC_B_BYTES = 4 * TC_KT * 128;   // four 64-column boxes
constexpr int TC_A_BYTES = 128 * TC_KT * 2;   // one term of the basis tile

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(void* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tc_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem(bar)) : "memory");
}
__device__ __forceinline__ void tc_mbar_expect_tx(void* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tc_smem(bar)), "r"(bytes) : "memory");
}
// bounded wait (about a second); on failure marks the CTA dead and raises the global flag, then returns
__device__ __forceinline__ void tc_mbar_wait(void* bar, uint32_t parity, volatile int* dead, int* err) {
  if (*dead) return;
  const uint32_t addr = tc_smem(bar);
  const long long t0 = clock64();
  for (;;) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return;
    if (*dead || clock64() - t0 > 2000000000LL) {
      *dead = 1;
      atomicExch(err, 1);
      return;
    }
  }
}
__device__ __forceinline__ void tc_tma_box(void* dst, const CUtensorMap* map, int x, int y, int z, void* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(
          tc_smem(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(tc_smem(bar)) : "memory");
}

// shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in 16-byte
// units, descriptor version 1, layout type (0 = no swizzle, 2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(
          d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tc_smem(bar)) : "memory");
}

template <typename T>
struct TcSplit;
template <>
struct TcSplit<__half> {
  static constexpr int NTERM = 2;
  static constexpr uint32_t FMT = 0;
  __device__ static __forceinline__ void split(float v, uint16_t* t) {
    const __half h = __float2half_rn(v);
    const __half l = __float2half_rn(v - __half2float(h));
    t[0] = __half_as_ushort(h);
    t[1] = __half_as_ushort(l);
  }
};
template <>
struct TcSplit<__nv_bfloat16> {
  static constexpr int NTERM = 3;
  static constexpr uint32_t FMT = 1;
  __device__ static __forceinline__ void split(float v, uint16_t* t) {
    const __nv_bfloat16 a = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(a);
    const __nv_bfloat16 b = __float2bfloat16_rn(r1);
    const __nv_bfloat16 c = __float2bfloat16_rn(r1 - __bfloat162float(b));
    t[0] = __bfloat16_as_ushort(a);
    t[1] = __bfloat16_as_ushort(b);
    t[2] = __bfloat16_as_ushort(c);
  }
};

struct TcParams {
  alignas(64) CUtensorMap tm_x;
  int K, C, N, n_rb, n_cb, kchunk;
  uint32_t T_c;
  uint64_t k_start;
  float* part;               // [split][B][2N][C]
  int64_t split_stride, b_stride;
  int* err;
};

__device__ __forceinline__ void tc_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

template <typename T>
__global__ void __launch_bounds__(TC_THREADS, 1) compress_tc_kernel(const __grid_constant__ TcParams p) {
  constexpr int NTERM = TcSplit<T>::NTERM;
  constexpr int STAGE = TC_B_BYTES + NTERM * TC_A_BYTES;
  extern __shared__ __align__(1024) unsigned char smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TC_ST * STAGE);   // full_b, full_a, empty [ST]; acc_full/empty [2]
  uint64_t* full_b = bars;
  uint64_t* full_a = bars + TC_ST;
  uint64_t* empty = bars + 2 * TC_ST;
  uint64_t* acc_full = bars + 3 * TC_ST;
  uint64_t* acc_empty = bars + 3 * TC_ST + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * TC_ST + 4);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rb = blockIdx.x % p.n_rb, cb = blockIdx.x / p.n_rb;
  const int split = blockIdx.y, b = blockIdx.z;
  const int kbeg = split * p.kchunk, kend = min(p.K, kbeg + p.kchunk);
  const int nkt = (kend - kbeg + TC_KT - 1) / TC_KT;

  if (tid == 0) {
    for (int s = 0; s < TC_ST; ++s) {
      tc_mbar_init(full_b + s, 1);
      tc_mbar_init(full_a + s, 256);
      tc_mbar_init(empty + s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc_mbar_init(acc_full + i, 1);
      tc_mbar_init(acc_empty + i, 128);
    }
    *dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(tmem_slot)),
                 "r"(2 * TC_NC) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp < 8) {
    // ---- basis generators (warps 0-3: tokens 0-15 of a stage, warps 4-7: tokens 16-31) ---------------------------------------------------------------------
    const int r = tid & 127;                // row of the 128-row block
    const int th = tid >> 7;                // which half of the stage's tokens
    const int R = rb * 128 + r;             // row of the 2N x C result
    const bool live = R < 2 * p.N;
    const bool is_sin = R >= p.N;
    const uint32_t n = live ? (uint32_t)(is_sin ? R - p.N : R) : 0u;
    const float inv_T = 1.0f / (float)p.T_c;
    float sd, cd;                           // rotation by one token
    sincos_phase(phase_mod(1ull, n, p.T_c), inv_T, &sd, &cd);
    for (int it = 0; it < nkt; ++it) {
      const int s = it % TC_ST;
      if (it >= TC_ST) tc_mbar_wait(empty + s, ((it / TC_ST) - 1) & 1, dead, p.err);
      unsigned char* abase = smem + s * STAGE + TC_B_BYTES + (r >> 3) * 512 + (r & 7) * 16;
      const uint64_t pos0 = p.k_start + (uint64_t)(kbeg + it * TC_KT);
#pragma unroll
      for (int g8 = 2 * th; g8 < 2 * th + 2; ++g8) {
        float sv, cv;
        sincos_phase(phase_mod(pos0 + 8 * g8, n, p.T_c), inv_T, &sv, &cv);
        uint16_t tt[3][8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          uint16_t t[3];
          TcSplit<T>::split(live ? (is_sin ? sv : cv) : 0.f, t);
#pragma unroll
          for (int e = 0; e < NTERM; ++e) tt[e][k] = t[e];
          const float c2 = cv * cd - sv * sd, s2 = sv * cd + cv * sd;
          cv = c2;
          sv = s2;
        }
#pragma unroll
        for (int e = 0; e < NTERM; ++e) {
          uint4 w;
          w.x = tt[e][0] | ((uint32_t)tt[e][1] << 16);
          w.y = tt[e][2] | ((uint32_t)tt[e][3] << 16);
          w.z = tt[e][4] | ((uint32_t)tt[e][5] << 16);
          w.w = tt[e][6] | ((uint32_t)tt[e][7] << 16);
          *reinterpret_cast<uint4*>(abase + e * TC_A_BYTES + g8 * 128) = w;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes -> MMA reads
      tc_mbar_arrive(full_a + s);
    }
  } else if (warp == 8) {
    // ---- TMA producer ----------------------------------------------------------------------------
    if (lane == 0) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&p.tm_x) : "memory");
    for (int it = 0; it < nkt; ++it) {
      const int s = it % TC_ST;
      if (it >= TC_ST) tc_mbar_wait(empty + s, ((it / TC_ST) - 1) & 1, dead, p.err);
      if (lane == 0) tc_mbar_expect_tx(full_b + s, TC_B_BYTES);
      __syncwarp();
      if (lane < 4)
        tc_tma_box(smem + s * STAGE + lane * (TC_KT * 128), &p.tm_x, cb * TC_NC + 64 * lane, kbeg + it * TC_KT, b,
                   full_b + s);
    }
  } else if (warp == 9) {
    // ---- MMA issuer ------------------------------------------------------------------------------
    // instruction descriptor: fp32 accumulate, A K-major, B MN-major, N = 256, M = 128
    const uint32_t idesc = (1u << 4) | (TcSplit<T>::FMT << 7) | (TcSplit<T>::FMT << 10) | (1u << 16) |
                           ((uint32_t)(TC_NC >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    for (int it = 0; it < nkt; ++it) {
      const int s = it % TC_ST;
      const int sg = it / TC_SEG, acc = sg & 1;
      const bool seg_first = (it % TC_SEG) == 0, seg_last = ((it % TC_SEG) == TC_SEG - 1) || (it == nkt - 1);
      if (seg_first && sg >= 2) tc_mbar_wait(acc_empty + acc, ((sg >> 1) - 1) & 1, dead, p.err);   // drained
      tc_mbar_wait(full_a + s, (it / TC_ST) & 1, dead, p.err);
      tc_mbar_wait(full_b + s, (it / TC_ST) & 1, dead, p.err);
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      if (lane == 0) {
        const uint32_t bsm = tc_smem(smem + s * STAGE), asm_ = bsm + TC_B_BYTES;
#pragma unroll
        for (int kk = 0; kk < TC_KT / 16; ++kk) {
          // B: 16 tokens = two 8-row groups of 1024 bytes; 64-column boxes 4096 bytes apart
          const uint64_t bd = tc_desc(bsm + kk * 2048, TC_KT * 128, 1024, 2);
#pragma unroll
          for (int e = 0; e < NTERM; ++e) {
            // A: core matrices of 8 rows x 8 tokens; K-adjacent ones 128 bytes apart, 8-row groups 512 bytes
            const uint64_t ad = tc_desc(asm_ + e * TC_A_BYTES + kk * 256, 128, 512, 0);
            tc_mma(tmem + acc * TC_NC, ad, bd, idesc, (!seg_first || kk > 0 || e > 0) ? 1u : 0u);
          }
        }
        tc_commit(empty + s);                      // arrives when the MMAs above have finished reading the stage
        if (seg_last) tc_commit(acc_full + acc);   // ... and when the segment's accumulator is complete
      }
      __syncwarp();
    }
  } else {
    // ---- segment drain: accumulator -> running partial tile (round-to-nearest adds) ---------------
    const int q = warp & 3;                    // tensor-memory lane quadrant this warp may read
    // rows of this warp: rb*128 + q*32 + (0..31).  A 32 x 32 block leaves tensor memory one row per lane;
    // it is turned through shared memory so that the global read-modify-write runs along the columns.
    float* tile = reinterpret_cast<float*>(smem + TC_ST * STAGE + 256) + q * (32 * 33);
    const int R0 = rb * 128 + q * 32;
    float* dst0 = p.part + (int64_t)split * p.split_stride + (int64_t)b * p.b_stride + (int64_t)R0 * p.C + cb * TC_NC;
    const int nseg = (nkt + TC_SEG - 1) / TC_SEG;
    if (nseg == 0) {
      for (int j = 0; j < 32; ++j)
        for (int i = lane; i < TC_NC; i += 32)
          if (R0 + j < 2 * p.N && cb * TC_NC + i < p.C) dst0[(int64_t)j * p.C + i] = 0.f;
    }
    for (int sg = 0; sg < nseg; ++sg) {
      const int acc = sg & 1;
      tc_mbar_wait(acc_full + acc, (sg >> 1) & 1, dead, p.err);
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
      for (int c = 0; c < TC_NC / 32; ++c) {
        const int col = cb * TC_NC + c * 32 + lane;
        const bool col_ok = col < p.C;
        // the running sums of this 32 x 32 block are requested first, so their latency overlaps the
        // tensor-memory read and the turn through shared memory
        float old[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          old[j] = (sg > 0 && col_ok && R0 + j < 2 * p.N) ? dst0[(int64_t)j * p.C + c * 32 + lane] : 0.f;
        float v[32];
        tc_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * TC_NC + c * 32), v);
        if (c == TC_NC / 32 - 1) {
          asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
          tc_mbar_arrive(acc_empty + acc);     // the accumulator may be overwritten
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) tile[lane * 33 + i] = v[i];
        __syncwarp();
        if (col_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (R0 + j < 2 * p.N) dst0[(int64_t)j * p.C + c * 32 + lane] = old[j] + tile[j * 33 + lane];
        }
        __syncwarp();
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  }
  __syncthreads();
  if (warp == 9) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * TC_NC) : "memory");
  }
}

// coef[b][r][m] = (accumulate ? coef : 0) + sum_split part[split][b][r][idx[m]]; NaN if a wait gave up
__global__ void compress_tc_reduce_kernel(const float* __restrict__ part, int nsplit, int64_t split_stride,
                                          int64_t b_stride, int C, const int32_t* __restrict__ idx, int Mc, int rows,
                                          float* __restrict__ coef, int accumulate, const int* __restrict__ err) {
  const int b = blockIdx.z, r = blockIdx.y;
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= Mc) return;
  const int col = idx ? idx[m] : m;
  float a = accumulate ? coef[((int64_t)b * rows + r) * Mc + m] : 0.f;
  for (int s = 0; s < nsplit; ++s) a += part[(int64_t)s * split_stride + (int64_t)b * b_stride + (int64_t)r * C + col];
  if (*err) a = __int_as_float(0x7fc00000);
  coef[((int64_t)b * rows + r) * Mc + m] = a;
}

}  // namespace fa

namespace fa {

struct TcPlan {
  int n_rb, n_cb, nsplit, kchunk;
};
static TcPlan tc_plan(int B, int K, int N, int C) {
  TcPlan p;
  p.n_rb = ceil_div(2 * N, 128);
  p.n_cb = ceil_div(C, TC_NC);
  const int64_t tiles = (int64_t)p.n_rb * p.n_cb * B;
  int ns = (int)ceil_div64(2 * (int64_t)sm_count(), tiles);
  const int maxs = ceil_div(K, 1024);   // chunks of at least 1024 tokens
  if (ns > maxs) ns = maxs;
  if (ns > 32) ns = 32;
  if (ns < 1) ns = 1;
  int kc = ceil_div(K, ns);
  kc = ceil_div(kc, TC_KT) * TC_KT;
  p.kchunk = kc;
  p.nsplit = ceil_div(K, kc);
  return p;
}

bool compress_tc_usable(const void* x, int B, int K, int64_t x_sb, int64_t x_sk, int x_cols, int N) {
  if (getenv("FA_COMPRESS_SIMT")) return false;
  return K >= 256 && N >= 1 && x_cols >= 8 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && x_sk % 8 == 0 &&
         (B == 1 || x_sb % 8 == 0) && x_sk >= x_cols;
}

size_t compress_tc_scratch_bytes(int B, int K, int N, int x_cols) {
  if (B <= 0 || K <= 0 || N <= 0 || x_cols <= 0) return 0;
  const TcPlan p = tc_plan(B, K, N, x_cols);
  return 16 + (size_t)p.nsplit * B * 2 * N * x_cols * sizeof(float);
}

template <typename T>
static int tc_launch_t(const TcParams& prm, const TcPlan& pl, int B, cudaStream_t st) {
  constexpr int smem = TC_ST * (TC_B_BYTES + TcSplit<T>::NTERM * TC_A_BYTES) + 256 + 4 * 32 * 33 * 4;
  cudaError_t e = cudaFuncSetAttribute(compress_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(compress_tc)");
  dim3 grid(pl.n_rb * pl.n_cb, pl.nsplit, B);
  compress_tc_kernel<T><<<grid, TC_THREADS, smem, st>>>(prm);
  FA_CHECK_LAUNCH("fa_compress(tensor-core)");
  return FA_OK;
}

int compress_tc_launch(const void* x, int dtype, int B, int K, int64_t x_sb, int64_t x_sk, int x_cols, const int32_t* idx,
                       int Mc, int N, int T_c, int64_t k_start, float* coef, int accumulate, void* scratch,
                       size_t scratch_bytes, cudaStream_t st) {
  const size_t need = compress_tc_scratch_bytes(B, K, N, x_cols);
  FA_REQUIRE(scratch && scratch_bytes >= need && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0, FA_ERR_CAPACITY,
             "fa_compress: scratch too small or misaligned (%zu < %zu bytes)", scratch_bytes, need);
  const TcPlan pl = tc_plan(B, K, N, x_cols);
  TcParams prm;
  int rc = make_tensor_map_3d(&prm.tm_x, x, dtype, x_cols, K, x_sk, B, x_sb, 64, TC_KT);
  if (rc != FA_OK) return rc;
  prm.K = K; prm.C = x_cols; prm.N = N; prm.n_rb = pl.n_rb; prm.n_cb = pl.n_cb; prm.kchunk = pl.kchunk;
  prm.T_c = (uint32_t)T_c;
  prm.k_start = (uint64_t)k_start;
  prm.err = reinterpret_cast<int*>(scratch);
  prm.part = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(scratch) + 16);
  prm.b_stride = (int64_t)2 * N * x_cols;
  prm.split_stride = prm.b_stride * B;
  cudaError_t e = cudaMemsetAsync(scratch, 0, 16, st);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync");
  rc = (dtype == FA_DTYPE_F16) ? tc_launch_t<__half>(prm, pl, B, st) : tc_launch_t<__nv_bfloat16>(prm, pl, B, st);
  if (rc != FA_OK) return rc;
  dim3 g2(ceil_div(Mc, 128), 2 * N, B);
  compress_tc_reduce_kernel<<<g2, 128, 0, st>>>(prm.part, pl.nsplit, prm.split_stride, prm.b_stride, x_cols, idx, Mc,
                                                 2 * N, coef, accumulate, prm.err);
  FA_CHECK_LAUNCH("fa_compress(reduce)");
  return FA_OK;
}

}  // namespace fa
