// Middle-span pass of the decode attention on tensor cores.  Included by decode.cu (namespace fa).
//
// Two observations make the span HBM-bound instead of arithmetic-bound:
//
// 1. Along the token axis the spectral score  s(l) = sum_n [w_cos[n] cos(2 pi l n/T) + w_sin[n] sin(..)]
//    is band-limited (highest frequency (N-1)/T cycles per token) and therefore heavily oversampled:
//    over a super-tile of J = 64*NH tokens it turns by at most ~1.5 cycles, so it is reproduced to
//    ~1e-7 by Lagrange interpolation through 16 fixed integer nodes x_k of the super-tile.  The
//    2N-long contraction is done only at the 16 nodes (a 16 x 2N x Hq GEMM) and a 64 x 16 x Hq GEMM
//    per half interpolates it to the tokens.  The PV side is the adjoint: probabilities are first
//    projected onto the nodes (16 x 64 x Hq), then one 2N x 16 x Hq GEMM adds them to g.
//    This cuts the spectral multiply-adds by J/16 and the basis table to 16 rows.
// 2. The node basis of a super-tile is the fixed table at the node offsets times a per-frequency
//    rotation by the super-tile's start, so it is rebuilt per super-tile with four multiply-adds per
//    entry from exact integer phases; w stays unrotated in registers (as MMA B fragments) and g is
//    accumulated directly in the absolute frame.
//
// All GEMMs are m16n8k16 tensor-core MMAs with fp32 accumulation.  Operands generated in the kernel
// (basis, w, interpolation weights, node scores) are fp16 hi+lo pairs where their rounding would
// reach the scores (three MMAs per product); probabilities are rounded once to 16 bits, as any
// flash-attention kernel does.  The verbatim dims are plain GEMMs of the cached rows against a
// block-diagonal query matrix (QK) and of the probabilities against the cached rows (PV), in the
// model dtype.  K/V rows stream through a 3-slot ring of 64-token half tiles that the last warp
// fills with TMA tensor-map boxes (64 columns x 64 tokens, 128-byte swizzle) completing on mbarriers.
#pragma once


constexpr int FD = 16;   // interpolation nodes per super-tile
constexpr int FH = 64;   // tokens per half tile (staging granularity)
constexpr int FNT_MAX = 4;
constexpr int FW = 16;            // warps of a middle-span CTA
constexpr int FAST_T = 32 * FW;   // its threads
constexpr int FNG = FW / 4;       // column-tile groups: warp = (16-token slice w & 3, group w >> 2)
constexpr int FNI = (FNT_MAX + FNG - 1) / FNG;   // column tiles a warp visits

__constant__ int c_nodes128[FD] = {0, 3, 7, 14, 23, 34, 45, 57, 70, 82, 93, 104, 113, 120, 124, 127};
__constant__ int c_nodes64[FD] = {0, 1, 4, 7, 12, 17, 22, 28, 35, 41, 46, 51, 56, 59, 62, 63};
// Lagrange weights L[j][k] of the two node sets (exact rational arithmetic, rounded once to float)
#include "interp_tables.inc"

// ---- tensor-core primitives ----------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2_t(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// ---- async-copy pipeline primitives ---------------------------------------------------------------
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(FAST_T) : "memory"); }
__device__ __forceinline__ void mbar_init(void* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: gives up after ~2e9 clock ticks (about a second), records the failure in *dead (shared,
// makes every later wait of the CTA return at once) and in *err (global, read by the finish kernel),
// and lets the caller carry on so that no thread is left behind at a barrier.
__device__ __forceinline__ void mbar_wait(void* bar, uint32_t parity, volatile int* dead, int* err) {
  if (*dead) return;
  const uint32_t addr = smem_u32(bar);
  const long long t0 = clock64();
  for (;;) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return;
    // back off between looks: a warp that spins at full rate takes issue slots from the warps it is waiting for
    __nanosleep(40);
    if (*dead || clock64() - t0 > 2000000000LL) {
      *dead = 1;
      atomicExch(err, 1);
      return;
    }
  }
}
// one 64 x 64 box of a verbatim store: global -> shared through the tensor-copy engine (TMA); the bytes
// landing are counted on `bar`.  x is a multiple of 64 elements, so the 16-byte start rule holds.
__device__ __forceinline__ void tma_box(void* dst, const CUtensorMap* map, int x, int y, int z, void* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(
          smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
// byte offset of the 16-byte chunk holding (row r, column 8*chunk) inside a ring slot: 64-column boxes of
// 8 KB side by side, rows of 128 bytes, chunk position XOR-swizzled with the row (128-byte swizzle)
__device__ __forceinline__ int sw_off(int r, int chunk) {
  return (chunk >> 3) * 8192 + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
}

// per-lane row/column offsets of the ldmatrix address patterns (j = lane>>3 selects the 8x8 matrix)
//  A, row-major tile  [m][k]:  row = (lane&7) + (j&1)*8,  col = (j>>1)*8
//  A, transposed tile [k][m]:  row = (lane&7) + (j>>1)*8, col = (j&1)*8      (with .trans)
//  B, tile [n][k], one n-tile: row = (lane&7),            col = (j&1)*8      (x2, lanes 0..15)
__device__ __forceinline__ int lds_a_row(int lane) { return (lane & 7) + ((lane >> 3) & 1) * 8; }
__device__ __forceinline__ int lds_a_col(int lane) { return (lane >> 4) * 8; }
__device__ __forceinline__ int lds_at_row(int lane) { return (lane & 7) + (lane >> 4) * 8; }
__device__ __forceinline__ int lds_at_col(int lane) { return ((lane >> 3) & 1) * 8; }
__device__ __forceinline__ int lds_b_row(int lane) { return lane & 7; }
__device__ __forceinline__ int lds_b_col(int lane) { return ((lane >> 3) & 1) * 8; }

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void split_h(float v, __half& hi, __half& lo) {
  hi = __float2half_rn(v);
  lo = __float2half_rn(v - __half2float(hi));
}
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- shared-memory layout ------------------------------------------------------------------
struct FastSmem {
  int fn0c, fn0s, fnt_hi, fnt_lo, interp_hi, interp_lo, rot, ph, dJ, snode32, snode_hi, snode_lo, pt_b, pt_lo, p16, pm, pm_lo, qn,
      smax, ssum, alpha, alpha_prod, m_run, l_run, cst, kcol, vnt, vhead, bars, slots, total;
  int fpitch, kpad, qpitch, spitch, slot_bytes, ppitch;
};
__host__ __device__ inline FastSmem fast_smem(int N, int NT, int NH, int Mn_k, int Mn_v, bool two_p) {
  FastSmem s;
  int o = 0;
  auto take = [&](int bytes) {
    int r = o;
    o += (bytes + 15) / 16 * 16;
    return r;
  };
  s.kpad = (2 * N + 15) / 16 * 16;
  s.fpitch = s.kpad + 8;
  const int HN = 8 * NT;
  s.fn0c = take(FD * N * 4);
  s.fn0s = take(FD * N * 4);
  s.fnt_hi = take(FD * s.fpitch * 2);
  s.fnt_lo = take(FD * s.fpitch * 2);
  s.interp_hi = take(FH * NH * 24 * 2);
  s.interp_lo = take(FH * NH * 24 * 2);
  s.rot = take(N * 8);
  s.ph = take(N * 4);
  s.dJ = take(N * 4);
  s.snode32 = take(FNG * FD * HN * 4);   // partial sums over parts of the 2N rows
  s.snode_hi = take(HN * 24 * 2);
  s.snode_lo = take(HN * 24 * 2);
  s.pt_b = take(HN * 24 * 2);
  s.pt_lo = take(HN * 24 * 2);
  s.ppitch = FH + 8;
  s.p16 = take((HN + 8) * s.ppitch * 2);
  s.pm = two_p ? take((HN + 8) * s.ppitch * 2) : s.p16;
  s.pm_lo = two_p ? take((HN + 8) * s.ppitch * 2) : s.p16;
  const int mnk16 = (Mn_k + 15) / 16 * 16, mnv16 = (Mn_v + 15) / 16 * 16;
  s.qpitch = mnk16 + 8;
  s.qn = take(HN * s.qpitch * 2);
  s.smax = take(4 * HN * 4);
  s.ssum = take(4 * HN * 4);   // running denominators, one row per 16-token slice of a half tile
  s.alpha = take(HN * 4);
  s.alpha_prod = take(HN * 4);
  s.m_run = take(2 * HN * 4);  // running maxima, ping-pong between consecutive half tiles
  s.l_run = take(HN * 4);
  s.cst = take(HN * 4);
  s.kcol = take(2 * FNT_MAX * 4);
  s.vnt = take(2 * (mnv16 / 16 + 1) * 4);
  s.vhead = take((mnv16 + 16) * 2);
  s.bars = take(8 * 8);   // full[3], empty[3] mbarriers + the CTA's give-up flag
  const int w = mnk16 > mnv16 ? mnk16 : mnv16;
  s.spitch = 0;
  const int boxes = (w + 63) / 64 > 0 ? (w + 63) / 64 : 1;
  s.slot_bytes = boxes * 8192;   // 64 rows x 64 columns x 2 bytes per box
  o = (o + 1023) / 1024 * 1024;  // the swizzle pattern repeats every 1024 bytes
  s.slots = take(3 * s.slot_bytes);
  s.total = o;
  return s;
}

// NT: 8-head column tiles of the CTA (all query heads of the rank, padded to 8*NT); NH: halves per super-tile
template <typename T, int NT, int NH>
__device__ void mid_chunk_fast(const DecodeParams& p, int b, int chunk, unsigned char* smem) {
  constexpr int HN = 8 * NT;
  constexpr int J = FH * NH;
  constexpr int KH = 32 / FNG;   // k16 steps of the node contraction per warp: one column tile, 1/FNG of 2N <= 512
  constexpr int MT = 32 / FW;    // 16-row tiles of g per warp
  constexpr int MTW = 16 / FW;   // 16-column tiles of verbatim V per warp (Mn_v <= 256)
  const fa_decode_args_t& a = p.a;
  const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const int N = a.N, D = a.D, R = p.R, Hq = a.Hq, Mn_k = a.Mn_k, Mn_v = a.Mn_v;
  const uint32_t T_ = (uint32_t)a.T;
  const float inv_T = 1.0f / (float)a.T;
  const FastSmem L = fast_smem(N, NT, NH, Mn_k, Mn_v, !std::is_same<T, __half>::value);
  float* fn0c = reinterpret_cast<float*>(smem + L.fn0c);
  float* fn0s = reinterpret_cast<float*>(smem + L.fn0s);
  __half* fnt_hi = reinterpret_cast<__half*>(smem + L.fnt_hi);
  __half* fnt_lo = reinterpret_cast<__half*>(smem + L.fnt_lo);
  __half* interp_hi = reinterpret_cast<__half*>(smem + L.interp_hi);
  __half* interp_lo = reinterpret_cast<__half*>(smem + L.interp_lo);
  float2* rot = reinterpret_cast<float2*>(smem + L.rot);
  uint32_t* ph = reinterpret_cast<uint32_t*>(smem + L.ph);
  uint32_t* dJ = reinterpret_cast<uint32_t*>(smem + L.dJ);
  float* snode32 = reinterpret_cast<float*>(smem + L.snode32);
  __half* snode_hi = reinterpret_cast<__half*>(smem + L.snode_hi);
  __half* snode_lo = reinterpret_cast<__half*>(smem + L.snode_lo);
  __half* pt_b = reinterpret_cast<__half*>(smem + L.pt_b);
  __half* pt_lo = reinterpret_cast<__half*>(smem + L.pt_lo);
  __half* p16 = reinterpret_cast<__half*>(smem + L.p16);
  T* pm = reinterpret_cast<T*>(smem + L.pm);
  T* pm_lo = reinterpret_cast<T*>(smem + L.pm_lo);
  T* qn = reinterpret_cast<T*>(smem + L.qn);
  float* smax = reinterpret_cast<float*>(smem + L.smax);
  float* ssum = reinterpret_cast<float*>(smem + L.ssum);
  float* alpha = reinterpret_cast<float*>(smem + L.alpha);
  float* alpha_prod = reinterpret_cast<float*>(smem + L.alpha_prod);
  float* m_run = reinterpret_cast<float*>(smem + L.m_run);
  float* l_run = reinterpret_cast<float*>(smem + L.l_run);
  float* cst = reinterpret_cast<float*>(smem + L.cst);
  int* kcol = reinterpret_cast<int*>(smem + L.kcol);      // [nt][2]
  int* vnt = reinterpret_cast<int*>(smem + L.vnt);        // [mt][2]
  int16_t* vhead = reinterpret_cast<int16_t*>(smem + L.vhead);
  T* slots = reinterpret_cast<T*>(smem + L.slots);
  const int fpitch = L.fpitch, kpad = L.kpad, qpitch = L.qpitch, ppitch = L.ppitch;
  const int* nodes = (NH == 2) ? c_nodes128 : c_nodes64;

  const int l0 = chunk * p.mid_chunk;
  const int l1 = min(a.n_mid, l0 + p.mid_chunk);
  const int nst = (l1 - l0 + J - 1) / J;       // super-tiles
  const int n_loads = nst * NH * 2;            // K and V half tiles, in consumption order
  // (node, frequency-pair) walk of this thread through the node-basis table
  const int halfN = N / 2;
  const int fk0 = tid / halfN, fp0 = tid % halfN, fdk = FAST_T / halfN, fdp = FAST_T % halfN;

  // ---- setup ------------------------------------------------------------------------------
  // The ring of half tiles is filled by the tensor-copy engine (TMA): lane 0 of warp 7 issues one copy
  // per 64 x 64 box and the bytes landing complete the slot's mbarrier.  A slot is refilled only after a CTA barrier that every
  // warp reaches after its last read of the slot, so no "empty" barriers are needed.
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bars);   // full[0..2]
  volatile int* dead = reinterpret_cast<volatile int*>(bars + 6);
  // zero everything that is read but never (or only partly) written later
  for (int e = tid; e < (L.smax - L.fnt_hi) / 16; e += FAST_T)
    reinterpret_cast<uint4*>(smem + L.fnt_hi)[e] = make_uint4(0u, 0u, 0u, 0u);
  if (tid == 0) {
    for (int i = 0; i < 3; ++i) mbar_init(bars + i, 1);   // completed by expect_tx + the copied bytes
    *dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // zeros before the engine's writes
  consumer_sync();
  const int nbK = (Mn_k + 63) / 64, nbV = (Mn_v + 63) / 64;   // 64-column boxes per half tile
  int issued = 0, issue_slot = 0;   // next half tile to request and its ring slot (warp 7)
  int consumed = 0;                 // half tiles this warp has finished reading
  auto issue_upto = [&](int limit) {
    if (wp != FW - 1) return;
    if (limit > n_loads) limit = n_loads;
    while (issued < limit) {
      const int i = issued;
      const int lf = l0 + (i >> 1) * FH;   // K and V half tiles alternate, 64 tokens each
      const bool is_v = (i & 1) != 0;
      const int nb = is_v ? nbV : nbK;
      if (lane == 0) mbar_expect_tx(bars + issue_slot, (uint32_t)nb * 8192u);
      __syncwarp();
      if (lane < nb) {   // one box per lane, so the copies are issued side by side
        unsigned char* dst = reinterpret_cast<unsigned char*>(slots) + issue_slot * L.slot_bytes;
        tma_box(dst + lane * 8192, is_v ? &p.tm_v : &p.tm_k, 64 * lane, lf, b, bars + issue_slot);
      }
      issue_slot = (issue_slot == 2) ? 0 : issue_slot + 1;
      ++issued;
    }
  };
  if (tid == (FW - 1) * 32) {
    if (nbK) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&p.tm_k) : "memory");
    if (nbV) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&p.tm_v) : "memory");
  }
  issue_upto(3);

  for (int e = tid; e < FD * N; e += FAST_T) {
    const int k = e / N, n = e - k * N;
    float s, c;
    sincos_phase(phase_mod((uint64_t)nodes[k], (uint32_t)n, T_), inv_T, &s, &c);
    fn0c[e] = c;
    fn0s[e] = s;
  }
  {
    const float* tab = (NH == 2) ? g_interp128 : g_interp64;
    for (int e = tid; e < J * FD; e += FAST_T) {
      const int j = e / FD, k = e - j * FD;
      __half hi, lo;
      split_h(tab[e], hi, lo);
      interp_hi[j * 24 + k] = hi;
      interp_lo[j * 24 + k] = lo;
    }
  }
  for (int n = tid; n < N; n += FAST_T) {
    dJ[n] = phase_mod((uint64_t)J, (uint32_t)n, T_);
    ph[n] = phase_mod((uint64_t)a.mid_l0 + (uint64_t)l0, (uint32_t)n, T_);
  }
  {
    // block-diagonal verbatim-K query matrix, raw model-dtype values (the scale is applied to the fp32
    // sum); the zeros are already there, only the R x Mn_k entries inside the blocks are fetched
    const T* q = reinterpret_cast<const T*>(a.q) + (int64_t)b * a.q_sb;
    for (int e = tid; e < R * Mn_k; e += FAST_T) {
      const int r = e / Mn_k, col = e - r * Mn_k;
      int g = 0;
      while (g + 1 < a.Hkv && col >= a.kn_h[g + 1]) ++g;
      const int h = g * R + r;
      qn[h * qpitch + col] = q[h * D + a.kn_list[col] - g * D];
    }
  }
  for (int h = tid; h < HN; h += FAST_T) {
    alpha[h] = 1.f;
    alpha_prod[h] = 1.f;
    m_run[h] = NEG_BIG;
    m_run[HN + h] = NEG_BIG;
    l_run[h] = 0.f;
    for (int r = 0; r < 4; ++r) ssum[r * HN + h] = 0.f;
    cst[h] = (h < Hq) ? p.cst[(int64_t)b * Hq + h] : 0.f;
  }
  if (tid < NT) {
    // verbatim-K column range (multiples of 16) that the heads of column tile `tid` touch
    const int h_first = 8 * tid, h_last = min(Hq, 8 * tid + 8) - 1;
    int c0 = 0, c1 = 0;
    if (h_first < Hq) {
      c0 = a.kn_h[h_first / R] & ~15;
      c1 = (a.kn_h[h_last / R + 1] + 15) & ~15;
    }
    kcol[2 * tid] = c0;
    kcol[2 * tid + 1] = c1;
  }
  for (int c = tid; c < Mn_v; c += FAST_T) {
    int g = 0;
    while (g + 1 < a.Hkv && c >= a.vn_h[g + 1]) ++g;
    vhead[c] = (int16_t)g;
  }
  consumer_sync();
  for (int mt = tid; mt * 16 < Mn_v; mt += FAST_T) {
    const int g_first = vhead[16 * mt], g_last = vhead[min(Mn_v, 16 * mt + 16) - 1];
    vnt[2 * mt] = (R * g_first) / 8;
    vnt[2 * mt + 1] = (R * (g_last + 1) - 1) / 8;
  }

  // w as persistent B fragments (hi / lo halves): k = frequency row, n = head.  Warp w holds column tile
  // w & 3 for part w >> 2 of the 2N rows.
  const int nt1 = wp & 3, khalf = wp >> 2;
  const int ktot = kpad / 16;            // k16 steps of the node contraction == 16-row tiles of g
  const int kh_steps = (ktot + FNG - 1) / FNG;   // steps per part
  uint32_t bhi[KH][2], blo[KH][2];
  {
    const float* wb = p.w + (int64_t)b * Hq * 2 * N;
    const int h = 8 * nt1 + gq;
#pragma unroll
    for (int i = 0; i < KH; ++i) {
      const int k0 = 16 * (khalf * kh_steps + i);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int k = k0 + 2 * tq + 8 * r;
        float v0 = 0.f, v1 = 0.f;
        if (nt1 < NT && i < kh_steps && h < Hq && k < 2 * N) {   // 2N is even, so k+1 is in range as well
          v0 = wb[(int64_t)h * 2 * N + k];
          v1 = wb[(int64_t)h * 2 * N + k + 1];
        }
        __half h0, l0_, h1, l1_;
        split_h(v0, h0, l0_);
        split_h(v1, h1, l1_);
        __half2 hh = __halves2half2(h0, h1), ll = __halves2half2(l0_, l1_);
        bhi[i][r] = *reinterpret_cast<uint32_t*>(&hh);
        blo[i][r] = *reinterpret_cast<uint32_t*>(&ll);
      }
    }
  }
  // persistent accumulators
  float Gacc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) Gacc[i][nt][e] = 0.f;
  float Oacc[MTW][NT][4];
#pragma unroll
  for (int i = 0; i < MTW; ++i)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) Oacc[i][nt][e] = 0.f;
  const int mt4 = wp & 3, ntp = wp >> 2;   // 16-token slice of a half tile, column-tile group
  consumer_sync();

  int mbuf = 0;            // which copy of m_run holds the current maxima
  int use_slot = 0;        // ring slot of the next half tile to consume
  uint32_t use_round = 0;  // how many times the ring has wrapped
  for (int st = 0; st < nst; ++st) {
    const int st_tok0 = l0 + st * J;
    // ---- A: node basis of this super-tile ----------------------------------------------------
    for (int n = tid; n < N; n += FAST_T) {
      float s, c;
      const uint32_t v = ph[n];
      sincos_phase(v, inv_T, &s, &c);
      rot[n] = make_float2(c, s);
      uint32_t nx = v + dJ[n];
      if (nx >= T_) nx -= T_;
      ph[n] = nx;
    }
    consumer_sync();
    for (int k = fk0, np = fp0; k < FD;) {
      const int n = 2 * np;
      const float2 c0 = *reinterpret_cast<const float2*>(fn0c + k * N + n);
      const float2 s0 = *reinterpret_cast<const float2*>(fn0s + k * N + n);
      const float2 ra = rot[n], rb = rot[n + 1];
      const float ca = c0.x * ra.x - s0.x * ra.y, sa = s0.x * ra.x + c0.x * ra.y;
      const float cb = c0.y * rb.x - s0.y * rb.y, sb = s0.y * rb.x + c0.y * rb.y;
      const __half2 ch = __floats2half2_rn(ca, cb), sh = __floats2half2_rn(sa, sb);
      const float2 chf = __half22float2(ch), shf = __half22float2(sh);
      const __half2 cl = __floats2half2_rn(ca - chf.x, cb - chf.y), sl = __floats2half2_rn(sa - shf.x, sb - shf.y);
      *reinterpret_cast<__half2*>(fnt_hi + k * fpitch + n) = ch;
      *reinterpret_cast<__half2*>(fnt_lo + k * fpitch + n) = cl;
      *reinterpret_cast<__half2*>(fnt_hi + k * fpitch + N + n) = sh;
      *reinterpret_cast<__half2*>(fnt_lo + k * fpitch + N + n) = sl;
      np += fdp;
      k += fdk;
      if (np >= halfN) {
        np -= halfN;
        ++k;
      }
    }
    consumer_sync();
    // ---- B: scores at the nodes,  s_node[16 x HN] = Fn_t[16 x 2N] * w[2N x HN] ------------------
    // warp = (column tile, half of the 2N rows); four accumulators keep the MMA chains short
    if (nt1 < NT) {
      float acc[4][4];
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[c][e] = 0.f;
#pragma unroll
      for (int i = 0; i < KH; ++i) {
        const int ks = khalf * kh_steps + i;
        if (i < kh_steps && ks < ktot) {
          uint32_t ah[4], al[4];
          const int off = lds_a_row(lane) * fpitch + 16 * ks + lds_a_col(lane);
          ldsm_x4(ah, fnt_hi + off);
          ldsm_x4(al, fnt_lo + off);
          mma16816<__half>(acc[i & 3], ah, bhi[i]);
          mma16816<__half>(acc[i & 3], al, bhi[i]);
          mma16816<__half>(acc[i & 3], ah, blo[i]);
        }
      }
      float* red = snode32 + khalf * (FD * HN);
      const int col = 8 * nt1 + 2 * tq;
      red[gq * HN + col] = (acc[0][0] + acc[1][0]) + (acc[2][0] + acc[3][0]);
      red[gq * HN + col + 1] = (acc[0][1] + acc[1][1]) + (acc[2][1] + acc[3][1]);
      red[(gq + 8) * HN + col] = (acc[0][2] + acc[1][2]) + (acc[2][2] + acc[3][2]);
      red[(gq + 8) * HN + col + 1] = (acc[0][3] + acc[1][3]) + (acc[2][3] + acc[3][3]);
    }
    consumer_sync();
    for (int e = tid; e < FD * HN; e += FAST_T) {
      const int k = e / HN, h = e - k * HN;
      __half hi, lo;
      float sv = 0.f;
#pragma unroll
      for (int part = 0; part < FNG; ++part) sv += snode32[part * FD * HN + e];
      split_h(sv, hi, lo);
      snode_hi[h * 24 + k] = hi;
      snode_lo[h * 24 + k] = lo;
    }
    consumer_sync();

    float pt_acc[4] = {0.f, 0.f, 0.f, 0.f};   // probabilities projected on the nodes (warps < NT)
#pragma unroll 1
    for (int half = 0; half < NH; ++half) {
      const int tok0 = st_tok0 + half * FH;    // first token of this half
      // ---- C: interpolate the node scores to this warp's 16 tokens ---------------------------
      float sc[FNI][4];
#pragma unroll
      for (int i = 0; i < FNI; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[i][e] = 0.f;
      {
        uint32_t ah[4], al[4];
        const int off = (half * FH + 16 * mt4 + lds_a_row(lane)) * 24 + lds_a_col(lane);
        ldsm_x4(ah, interp_hi + off);
        ldsm_x4(al, interp_lo + off);
#pragma unroll
        for (int i = 0; i < FNI; ++i) {
          const int nt = ntp + FNG * i;
          if (nt < NT) {
            uint32_t bh[2], bl[2];
            const int boff = (8 * nt + lds_b_row(lane)) * 24 + lds_b_col(lane);
            ldsm_x2(bh, snode_hi + boff);
            ldsm_x2(bl, snode_lo + boff);
            mma16816<__half>(sc[i], ah, bh);
            mma16816<__half>(sc[i], al, bh);
            mma16816<__half>(sc[i], ah, bl);
          }
        }
      }
      // ---- D: verbatim-dim scores from the K rows ----------------------------------------------
      mbar_wait(bars + use_slot, use_round & 1, dead, p.err);
      {
        const unsigned char* ks_ = reinterpret_cast<const unsigned char*>(slots) + use_slot * L.slot_bytes;
#pragma unroll
        for (int i = 0; i < FNI; ++i) {
          const int nt = ntp + FNG * i;
          if (nt < NT) {
            float vb[4] = {0.f, 0.f, 0.f, 0.f};
            const int c_end = kcol[2 * nt + 1];
            for (int c = kcol[2 * nt]; c < c_end; c += 16) {
              uint32_t af[4], bf[2];
              ldsm_x4(af, ks_ + sw_off(16 * mt4 + lds_a_row(lane), (c + lds_a_col(lane)) >> 3));
              ldsm_x2(bf, qn + (8 * nt + lds_b_row(lane)) * qpitch + c + lds_b_col(lane));
              mma16816<T>(vb, af, bf);
            }
            const int col = 8 * nt + 2 * tq;
            const float k0 = cst[col], k1 = cst[col + 1];
            sc[i][0] = sc[i][0] + p.c2 * vb[0] + k0;
            sc[i][1] = sc[i][1] + p.c2 * vb[1] + k1;
            sc[i][2] = sc[i][2] + p.c2 * vb[2] + k0;
            sc[i][3] = sc[i][3] + p.c2 * vb[3] + k1;
          }
        }
      }
      ++consumed;   // done with the K half tile
      if (++use_slot == 3) {
        use_slot = 0;
        ++use_round;
      }
      // ---- E: online softmax over the 64 tokens of this half -----------------------------------
      const bool ok0 = (tok0 + 16 * mt4 + gq) < l1, ok1 = (tok0 + 16 * mt4 + gq + 8) < l1;
#pragma unroll
      for (int i = 0; i < FNI; ++i) {
        const int nt = ntp + FNG * i;
        if (nt < NT) {
          float v0 = fmaxf(ok0 ? sc[i][0] : NEG_BIG, ok1 ? sc[i][2] : NEG_BIG);
          float v1 = fmaxf(ok0 ? sc[i][1] : NEG_BIG, ok1 ? sc[i][3] : NEG_BIG);
#pragma unroll
          for (int o = 4; o < 32; o <<= 1) {
            v0 = fmaxf(v0, __shfl_xor_sync(0xffffffffu, v0, o));
            v1 = fmaxf(v1, __shfl_xor_sync(0xffffffffu, v1, o));
          }
          if (gq == 0) {
            smax[mt4 * HN + 8 * nt + 2 * tq] = v0;
            smax[mt4 * HN + 8 * nt + 2 * tq + 1] = v1;
          }
        }
      }
      consumer_sync();
      issue_upto(consumed + 3);   // every warp is past its reads of the half tiles consumed so far
#pragma unroll
      for (int i = 0; i < FNI; ++i) {
        const int nt = ntp + FNG * i;
        if (nt < NT) {
          const int col = 8 * nt + 2 * tq;
          const float mo0 = m_run[mbuf * HN + col], mo1 = m_run[mbuf * HN + col + 1];
          float mn0 = mo0, mn1 = mo1;
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            mn0 = fmaxf(mn0, smax[r * HN + col]);
            mn1 = fmaxf(mn1, smax[r * HN + col + 1]);
          }
          const float p0 = ok0 ? exp2f(sc[i][0] - mn0) : 0.f, p1 = ok0 ? exp2f(sc[i][1] - mn1) : 0.f;
          const float p2 = ok1 ? exp2f(sc[i][2] - mn0) : 0.f, p3 = ok1 ? exp2f(sc[i][3] - mn1) : 0.f;
          // probabilities as B operands [head][token]; rounded once, sums use the rounded values
          const int j0 = 16 * mt4 + gq;
          const __half h0 = __float2half_rn(p0), h1 = __float2half_rn(p1), h2 = __float2half_rn(p2),
                       h3 = __float2half_rn(p3);
          p16[col * ppitch + j0] = h0;
          p16[(col + 1) * ppitch + j0] = h1;
          p16[col * ppitch + j0 + 8] = h2;
          p16[(col + 1) * ppitch + j0 + 8] = h3;
          if (!std::is_same<T, __half>::value) {
            // an fp16 value splits exactly into two bf16 values, so the verbatim-V GEMM (model dtype)
            // sees the same probabilities as the spectral side and the denominator
            const float f[4] = {__half2float(h0), __half2float(h1), __half2float(h2), __half2float(h3)};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const T hi = from_f32<T>(f[e]);
              const T lo = from_f32<T>(f[e] - to_f32(hi));
              const int o = (col + (e & 1)) * ppitch + j0 + 8 * (e >> 1);
              pm[o] = hi;
              pm_lo[o] = lo;
            }
          }
          const float q0 = __half2float(h0), q1 = __half2float(h1), q2 = __half2float(h2), q3 = __half2float(h3);
          float s0 = q0 + q2, s1 = q1 + q3;
#pragma unroll
          for (int o = 4; o < 32; o <<= 1) {
            s0 += __shfl_xor_sync(0xffffffffu, s0, o);
            s1 += __shfl_xor_sync(0xffffffffu, s1, o);
          }
          if (gq == 0) {
            // one lane owns (16-token slice, column): its denominator is rescaled and extended here,
            // the four slices are added when the chunk is finished
            const float al0 = exp2f(mo0 - mn0), al1 = exp2f(mo1 - mn1);
            ssum[mt4 * HN + col] = ssum[mt4 * HN + col] * al0 + s0;
            ssum[mt4 * HN + col + 1] = ssum[mt4 * HN + col + 1] * al1 + s1;
            if (mt4 == 0) {
              alpha[col] = al0;
              alpha[col + 1] = al1;
              alpha_prod[col] *= al0;
              alpha_prod[col + 1] *= al1;
              m_run[(mbuf ^ 1) * HN + col] = mn0;
              m_run[(mbuf ^ 1) * HN + col + 1] = mn1;
            }
          }
        }
      }
      mbuf ^= 1;
      consumer_sync();
      // ---- F: project the probabilities onto the nodes (warps 0..NT-1, one column tile each) -----
      if (wp < NT) {
        const int col = 8 * wp + 2 * tq;
        const float a0 = alpha[col], a1 = alpha[col + 1];
        pt_acc[0] *= a0; pt_acc[1] *= a1; pt_acc[2] *= a0; pt_acc[3] *= a1;
#pragma unroll
        for (int ks = 0; ks < FH / 16; ++ks) {
          uint32_t af[4], al[4], bf[2];
          const int ioff = (half * FH + 16 * ks + lds_at_row(lane)) * 24 + lds_at_col(lane);
          ldsm_x4_t(af, interp_hi + ioff);
          ldsm_x4_t(al, interp_lo + ioff);
          ldsm_x2(bf, p16 + (8 * wp + lds_b_row(lane)) * ppitch + 16 * ks + lds_b_col(lane));
          mma16816<__half>(pt_acc, af, bf);
          mma16816<__half>(pt_acc, al, bf);
        }
      }
      // ---- G: verbatim-V numerators from the V rows ----------------------------------------------
      mbar_wait(bars + use_slot, use_round & 1, dead, p.err);
      {
        const unsigned char* vs_ = reinterpret_cast<const unsigned char*>(slots) + use_slot * L.slot_bytes;
#pragma unroll
        for (int i = 0; i < MTW; ++i) {
          const int mt = wp + FW * i;
          if (16 * mt < Mn_v) {
            const int nlo = vnt[2 * mt], nhi = vnt[2 * mt + 1];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              if (nt >= nlo && nt <= nhi) {
                const float a0 = alpha[8 * nt + 2 * tq], a1 = alpha[8 * nt + 2 * tq + 1];
                Oacc[i][nt][0] *= a0; Oacc[i][nt][1] *= a1; Oacc[i][nt][2] *= a0; Oacc[i][nt][3] *= a1;
              }
            }
#pragma unroll
            for (int ks = 0; ks < FH / 16; ++ks) {
              uint32_t af[4];
              ldsm_x4_t(af, vs_ + sw_off(16 * ks + lds_at_row(lane), (16 * mt + lds_at_col(lane)) >> 3));
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                if (nt >= nlo && nt <= nhi) {
                  uint32_t bf[2];
                  const int poff = (8 * nt + lds_b_row(lane)) * ppitch + 16 * ks + lds_b_col(lane);
                  ldsm_x2(bf, pm + poff);
                  mma16816<T>(Oacc[i][nt], af, bf);
                  if (!std::is_same<T, __half>::value) {
                    ldsm_x2(bf, pm_lo + poff);
                    mma16816<T>(Oacc[i][nt], af, bf);
                  }
                }
              }
            }
          }
        }
      }
      ++consumed;   // done with the V half tile
      if (++use_slot == 3) {
        use_slot = 0;
        ++use_round;
      }
    }
    // ---- H: add the node-projected probabilities to g,  g[2N x HN] += Fn_t^T[2N x 16] * pt[16 x HN] ----
    if (wp < NT) {
      const int col = 8 * wp + 2 * tq;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        __half hi, lo;
        split_h(pt_acc[e], hi, lo);
        const int o = (col + (e & 1)) * 24 + gq + 8 * (e >> 1);
        pt_b[o] = hi;
        pt_lo[o] = lo;
      }
    }
    consumer_sync();
    issue_upto(consumed + 3);
    {
      uint32_t bf[NT][2], bl[NT][2];
      float ap[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        ldsm_x2(bf[nt], pt_b + (8 * nt + lds_b_row(lane)) * 24 + lds_b_col(lane));
        ldsm_x2(bl[nt], pt_lo + (8 * nt + lds_b_row(lane)) * 24 + lds_b_col(lane));
        ap[nt][0] = alpha_prod[8 * nt + 2 * tq];
        ap[nt][1] = alpha_prod[8 * nt + 2 * tq + 1];
      }
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const int mt = wp + FW * i;
        if (mt < ktot) {
          uint32_t ah[4], al[4];
          const int off = lds_at_row(lane) * fpitch + 16 * mt + lds_at_col(lane);
          ldsm_x4_t(ah, fnt_hi + off);
          ldsm_x4_t(al, fnt_lo + off);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            Gacc[i][nt][0] *= ap[nt][0]; Gacc[i][nt][1] *= ap[nt][1];
            Gacc[i][nt][2] *= ap[nt][0]; Gacc[i][nt][3] *= ap[nt][1];
            mma16816<__half>(Gacc[i][nt], ah, bf[nt]);
            mma16816<__half>(Gacc[i][nt], al, bf[nt]);
            mma16816<__half>(Gacc[i][nt], ah, bl[nt]);
          }
        }
      }
    }
    consumer_sync();
    for (int h = tid; h < HN; h += FAST_T) alpha_prod[h] = 1.f;
  }
  consumer_sync();

  // ---- chunk partials ---------------------------------------------------------------------------
  const int64_t slot = (int64_t)b * p.NCH + p.n_il_chunks + chunk;
  for (int h = tid; h < Hq; h += FAST_T) {
    p.m_part[slot * Hq + h] = m_run[mbuf * HN + h];
    p.l_part[slot * Hq + h] = (ssum[h] + ssum[HN + h]) + (ssum[2 * HN + h] + ssum[3 * HN + h]);
  }
  float* ob = p.o_part + slot * Hq * D;
  for (int e = tid; e < Hq * D; e += FAST_T) ob[e] = 0.f;
  consumer_sync();
#pragma unroll
  for (int i = 0; i < MTW; ++i) {
    const int mt = wp + FW * i;
    if (16 * mt < Mn_v) {
      const int nlo = vnt[2 * mt], nhi = vnt[2 * mt + 1];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        if (nt >= nlo && nt <= nhi) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = 16 * mt + gq + 8 * (e >> 1);
            const int h = 8 * nt + 2 * tq + (e & 1);
            if (c < Mn_v && h < Hq) {
              const int g = vhead[c];
              if (h / R == g) ob[h * D + a.vn_list[c] - g * D] = Oacc[i][nt][e];
            }
          }
        }
      }
    }
  }
  float* gb = p.g_part + (((int64_t)b * p.n_mid_chunks + chunk) * Hq) * 2 * N;
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    const int mt = wp + FW * i;
    if (mt < ktot) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = 16 * mt + gq + 8 * (e >> 1);
          const int h = 8 * nt + 2 * tq + (e & 1);
          if (n < 2 * N && h < Hq) gb[(int64_t)h * 2 * N + n] = Gacc[i][nt][e];
        }
      }
    }
  }
}

