// Warp-specialised middle-span pass with the spectral accumulator in tensor memory.  Included by decode.cu
// after decode_ws.cuh (same namespace; same ldmatrix / mma.sync / mbarrier / TMA helpers and the same
// mathematics as decode_fast.cuh: node interpolation of the band-limited spectral score).
//
// 20 warps per CTA (5 warp groups; registers are handed out per group of four warps):
//
//   spectral warps (0..7)    node basis of super-tile j (rotation of a fixed table to the super-tile's centre),
//                            written in the core-matrix layout that both ldmatrix and the tcgen05 descriptors
//                            read, and the node scores s_node = Fn_j * w as mma.sync GEMMs (w stays in
//                            registers); they run up to two super-tiles ahead
//   score warps (8..15)      warp = (8-head column tile nt, 64-token half): verbatim-K scores, interpolation of
//                            the node scores, softmax, projection of the probabilities onto the nodes,
//                            verbatim-V numerators.  The two warps of a column tile exchange the tile's maximum
//                            through shared memory and a 64-thread named barrier; they never meet other tiles.
//   service warps (16..19)   everything that is a hand-off rather than arithmetic.  Warp 16 refills the ring of
//                            K / V half tiles (TMA boxes) as the score warps release the slots; warp 17 waits
//                            until both halves of every tile have delivered their projected probabilities, adds
//                            them up, writes them as the B operand and issues the g update on the tensor cores.
//                            All four own one lane quadrant of tensor memory each: together they rescale a
//                            tile's accumulators when its running maximum moves, and at the end they stage g in
//                            shared memory for the bulk copies that write it out.
//
// The spectral accumulator g[2N x 32 head columns] of the four column tiles lives in tensor memory (4 blocks of
// 128 rows x 32 columns): after the halves have been added up, warp 17 issues
//     g += Fn_j^T[2N x 16 nodes] * pt[16 nodes x 32 head columns]
// as tcgen05.mma (M = 128, N = 32, K = 16; basis and pt as fp16 hi + lo pairs, three products per row block)
// and commits it to the mbarrier that hands the basis buffer back to the spectral warps.  No score
// warp waits for that GEMM or touches tensor memory, and the accumulator costs no registers.
//
// Accumulators in tensor memory cannot be rescaled for free, so the running maximum is lazy: it moves only when
// a super-tile's maximum exceeds it by more than 2^6.  The score warps then rescale what they hold in registers
// and publish the factors with their projected probabilities; warp 17 sees factors other than 1, asks the other
// service warps in (a sequence number in shared memory that they poll), each multiplies its lane quadrant of the
// tile's accumulators once the updates issued so far have landed, and only then is the next update issued.
// Probabilities are at most 2^6 and stay inside fp16; all sums use the same reference maximum, which is what
// the chunk reports.
#pragma once

constexpr int W2_T = 640;                 // threads: 8 spectral + 8 score + 4 service warps
// registers per thread after setmaxnreg: 256 x 72 (spectral) + 256 x 136 (score) + 128 x 56 (service)
// <= 640 x 96, the registers the CTA holds at launch (the pool setmaxnreg moves them within)
constexpr int W2_SREG = 72, W2_QREG = 136, W2_VREG = 56;
constexpr int W2_MTV = 4;                 // 16-column tiles of verbatim V a score warp owns
constexpr int W2_KS = 4;                  // 16-column steps of verbatim K a score warp contracts
constexpr float W2_LAZY = 6.0f;           // log2 headroom before the running maximum moves
constexpr int W2_TMEM_COLS = 256;         // g: 4 row blocks x 32 columns (4 column tiles x 8 heads); w fragments: 128 columns
constexpr int W2_TMEM_W = 128;            // first column of the w fragments
constexpr int W2_IDX = 256;               // verbatim columns per store at most (4 column tiles x 64), KV heads at most 39

struct Ws2Smem {
  int ec, es, fnt, interp_hi, interp_lo, snode32, snode, pw, ptb, ptp, mx, alpha, lx, idx, bars, slots, total;
  int fterm, kpad, slot_bytes;
};
__host__ __device__ inline Ws2Smem ws2_smem(int N, int Mn_k, int Mn_v) {
  Ws2Smem s;
  int o = 0;
  auto take = [&](int bytes) {
    int r = o;
    o += (bytes + 15) / 16 * 16;
    return r;
  };
  s.kpad = (2 * N + 15) / 16 * 16;
  s.fterm = (s.kpad + 127) / 128 * 128 * 32;   // one term (hi or lo) of one buffer: [row][16 nodes], whole 128-row blocks
  s.ec = take(8 * N * 4);
  s.es = take(8 * N * 4);
  s.fnt = take(2 * 2 * s.fterm);              // [buffer][hi, lo]
  s.interp_hi = take(128 * 24 * 2);
  s.interp_lo = take(128 * 24 * 2);
  s.snode32 = take(2 * FD * 32 * 4);          // partial node scores of the two halves of the 2N rows
  s.snode = take(2 * 2 * 32 * 24 * 2);        // [buffer][hi, lo][head][16 nodes, pitch 24]
  s.pw = take(8 * 64 * 8 * 2);                // per score warp: probabilities [64 tokens][8 heads]
  s.ptb = take(2 * 1024);                     // [hi, lo]: B operand [32 head columns][16 nodes] as core matrices
  s.ptp = take(2 * 4 * 2 * FD * 8 * 4);       // [buffer][tile][half][node][head]: projections of the halves
  s.mx = take(2 * 4 * 2 * 8 * 4);             // [super-tile parity][tile][half][head]
  s.alpha = take(2 * 4 * 8 * 4);              // [buffer][tile][head]: factor the running maximum's move asks for
  s.lx = take(4 * 2 * 8 * 4);
  s.idx = take(2 * (W2_IDX + 40) * 4);         // verbatim column lists of K and V and the KV heads' segment bounds
  s.bars = take(24 * 8);
  const int mnk16 = (Mn_k + 15) / 16 * 16, mnv16 = (Mn_v + 15) / 16 * 16;
  const int w = mnk16 > mnv16 ? mnk16 : mnv16;
  const int boxes = (w + 63) / 64 > 0 ? (w + 63) / 64 : 1;
  s.slot_bytes = boxes * 8192;
  o = (o + 1023) / 1024 * 1024;
  s.slots = take(3 * s.slot_bytes);
  s.total = o;
  return s;
}

__device__ __forceinline__ void w2_spec_sync() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }
__device__ __forceinline__ void w2_tile_sync(int nt) { asm volatile("bar.sync %0, 64;\n" ::"r"(2 + nt) : "memory"); }

// shared-memory matrix descriptor of an operand without swizzle: 8 x 8 core matrices of 128 contiguous bytes,
// K-adjacent ones `lbo` bytes apart, 8-row groups `sbo` bytes apart (descriptor version 1)
__device__ __forceinline__ uint64_t w2_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
__device__ __forceinline__ void w2_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(
          d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void w2_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void w2_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
// 16 consecutive columns of this warp's lane quadrant, one lane per thread; completion is awaited separately
__device__ __forceinline__ void w2_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void w2_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void w2_st4(uint32_t taddr, uint4 v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(taddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void w2_st8(uint32_t taddr, const float (&v)[8]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// one non-blocking look at an mbarrier phase by a whole warp (lane 0 looks, everybody gets the answer)
__device__ __forceinline__ bool mbar_test(void* bar, uint32_t parity) {
  uint32_t ok = 0;
  if ((threadIdx.x & 31) == 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  __syncwarp();
  return ok != 0;
}

// byte offset of (row f, node k) inside one term of the node basis: core matrices of 8 rows x 8 nodes
__device__ __forceinline__ int w2_foff(int f, int k) { return (f >> 3) * 256 + (k >> 3) * 128 + (f & 7) * 16 + (k & 7) * 2; }

template <typename T>
__device__ void mid_chunk_ws2(const DecodeParams& p, int b0, int chunk, unsigned char* smem) {
  constexpr int J = 128, HN = 32;   // tokens per super-tile, head columns per CTA
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  const fa_decode_args_t& a = p.a;
  const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const int N = a.N, D = a.D, R = p.R, Hq = a.Hq, Mn_k = a.Mn_k, Mn_v = a.Mn_v;
  const int NTs = p.wsNTs;
  const int nseq = min(p.wsSEQ, a.B - b0);
  const int NT = nseq * NTs;
  const uint32_t T2 = 2u * (uint32_t)a.T;
  const float inv_T = 1.0f / (float)a.T;
  const Ws2Smem L = ws2_smem(N, p.wsSEQ * ((Mn_k + 63) / 64) * 64, p.wsSEQ * ((Mn_v + 63) / 64) * 64);
  float* ec = reinterpret_cast<float*>(smem + L.ec);
  float* es = reinterpret_cast<float*>(smem + L.es);
  unsigned char* fnt = smem + L.fnt;
  __half* interp_hi = reinterpret_cast<__half*>(smem + L.interp_hi);
  __half* interp_lo = reinterpret_cast<__half*>(smem + L.interp_lo);
  float* snode32 = reinterpret_cast<float*>(smem + L.snode32);
  __half* snode = reinterpret_cast<__half*>(smem + L.snode);
  unsigned char* ptb = smem + L.ptb;
  float* ptp = reinterpret_cast<float*>(smem + L.ptp);
  float* mx = reinterpret_cast<float*>(smem + L.mx);
  float* alpha_s = reinterpret_cast<float*>(smem + L.alpha);
  float* lx = reinterpret_cast<float*>(smem + L.lx);
  int* kn_s = reinterpret_cast<int*>(smem + L.idx);   // copies of kn_list, kn_h, vn_list, vn_h: the score warps index
  int* knh_s = kn_s + W2_IDX;                          // them at both ends of the chunk, when anything fetched from
  int* vn_s = knh_s + 40;                              // global memory queues behind the K / V stream
  int* vnh_s = vn_s + W2_IDX;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* full_slot = bars;         // [3] a K or V half tile has landed
  uint64_t* empty_slot = bars + 3;    // [3] the score warps of its half are done with it
  uint64_t* full_sp = bars + 6;       // [2] node basis + node scores of a super-tile are written
  uint64_t* empty_sp = bars + 8;      // [2] ... and the g update has read the basis
  uint64_t* pt_full = bars + 10;      // [2] both halves of every tile have delivered their projected probabilities
  uint64_t* g_done = bars + 12;       // [1] the g update of a super-tile has completed
  uint64_t* resc_done = bars + 13;    // [1] the four service warps have rescaled their lane quadrants
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* dead = reinterpret_cast<volatile int*>(bars + 15);
  volatile int* resc_seq = reinterpret_cast<volatile int*>(bars + 16);   // rescale requests issued so far
  volatile int* resc_st = reinterpret_cast<volatile int*>(bars + 17);    // super-tile of the latest request
  volatile int* svc_exit = reinterpret_cast<volatile int*>(bars + 18);   // every g update has been issued
  uint64_t* tab_bar = bars + 19;      // [1] the tables have landed
  unsigned char* slots = smem + L.slots;
  const int kpad = L.kpad, ktot = kpad / 16, fterm = L.fterm;
  const int nblk = (kpad + 127) / 128;   // 128-row blocks of g

  const int l0 = chunk * p.mid_chunk;
  const int l1 = min(a.n_mid, l0 + p.mid_chunk);
  const int nst = (l1 - l0 + J - 1) / J;
  // Half tiles per super-tile, in ring order: K half 0, K half 1, V half 1, V half 0.  A warp reads only the
  // tiles of its half, i.e. every other phase of a ring slot's barrier, and a parity wait cannot tell "my tile
  // has landed" from "the tile before the one before mine has not landed yet".  In this order the tile that held
  // the slot before (three places back) was either read by the same warp or by the warp's tile mate before a
  // pair barrier the warp has passed since, so it has landed whenever a warp starts to wait.
  const int n_tiles = 4 * nst;
  const int nbK = (Mn_k + 63) / 64, nbV = (Mn_v + 63) / 64;
  auto slot_of = [&](int bb) { return (int64_t)bb * p.NCH + p.n_il_chunks + chunk; };

  // called by a whole warp: request half tile i into ring slot i % 3
  auto issue_tile = [&](int i) {
    if (i >= n_tiles) return;
    const int s = i % 3, r = i & 3;
    const int lf = l0 + (i >> 2) * J + ((r == 1 || r == 2) ? FH : 0);
    const bool is_v = r >= 2;
    const int nb = is_v ? nbV : nbK;
    if (lane == 0) mbar_expect_tx(full_slot + s, (uint32_t)(nseq * nb) * 8192u);
    __syncwarp();
    if (lane < nseq * nb) {   // the boxes of sequence 0, then those of sequence 1, ...
      const int sq = lane / nb, bx = lane - sq * nb;
      tma_box(slots + s * L.slot_bytes + lane * 8192, is_v ? &p.tm_v : &p.tm_k, 64 * bx, lf, b0 + sq, full_slot + s);
    }
  };

  // ---- set-up (all warps) ---------------------------------------------------------------------
  // the index lists first: their latency (global memory) passes while the rest of the set-up runs
  const int kn_v = tid < Mn_k ? a.kn_list[tid] : 0, vn_v = tid < Mn_v ? a.vn_list[tid] : 0;
  const int knh_v = tid <= a.Hkv ? a.kn_h[tid] : 0, vnh_v = tid <= a.Hkv ? a.vn_h[tid] : 0;
  if (tid == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(full_slot + i, 1);
      mbar_init(empty_slot + i, NT);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(full_sp + i, 8);
      mbar_init(empty_sp + i, 1);
      mbar_init(pt_full + i, 2 * NT);
    }
    mbar_init(g_done, 1);
    mbar_init(resc_done, 4);
    mbar_init(tab_bar, 1);
    *dead = 0;
    *resc_seq = 0;
    *resc_st = 0;
    *svc_exit = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    // node-offset rotation table (ec and es lie back to back, 8N floats each) and interpolation matrix (hi and lo
    // terms back to back, 128 x 24 halves each): shared-memory images prepared once per launch, fetched by two
    // bulk copies while the set-up goes on
    const uint32_t b_e = 64u * (uint32_t)N, b_i = 2u * 128u * 24u * 2u;
    mbar_expect_tx(tab_bar, b_e + b_i);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_u32(ec)),
                 "l"(p.tab), "r"(b_e), "r"(smem_u32(tab_bar)) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                     smem_u32(interp_hi)), "l"(p.tab + 16 * N), "r"(b_i), "r"(smem_u32(tab_bar)) : "memory");
  }
  if (wp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                 "r"(W2_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  for (int e = tid; e < 2 * FD * 32; e += W2_T) snode32[e] = 0.f;
  // rows past 2N of the node basis' last 128-row block stay zero, and so do the B operand's columns of absent tiles
  for (int t = 0; t < 4; ++t)
    for (int e = 2 * N * 32 / 16 + tid; e < fterm / 16; e += W2_T) reinterpret_cast<uint4*>(fnt + t * fterm)[e] = make_uint4(0u, 0u, 0u, 0u);
  for (int e = tid; e < (2 * 1024) / 16; e += W2_T) reinterpret_cast<uint4*>(ptb)[e] = make_uint4(0u, 0u, 0u, 0u);
  if (tid < Mn_k) kn_s[tid] = kn_v;
  if (tid < Mn_v) vn_s[tid] = vn_v;
  if (tid <= a.Hkv) {
    knh_s[tid] = knh_v;
    vnh_s[tid] = vnh_v;
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  if (wp == 16) {
    if (lane == 0) {
      if (nbK) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&p.tm_k) : "memory");
      if (nbV) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&p.tm_v) : "memory");
    }
    for (int i = 0; i < 3; ++i) issue_tile(i);
  }

  if (wp < 8) {
    // =========================== spectral warps ================================================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(W2_SREG));
    const int nt1 = wp & 3, khalf = wp >> 2;
    // w as B fragments (hi / lo): k = coefficient row, n = head; this warp contracts column tile nt1 over part
    // `khalf` of the 2N rows.  The prepare kernel has written them in fragment order, 16 bytes per step and lane.
    // They live in tensor memory (this warp's lane quadrant, 4 columns per step) and are read back for every
    // super-tile: 64 registers per thread would not survive the basis phase, and anything fetched from L2 while the
    // K / V stream saturates the memory system takes microseconds.
    constexpr int KH = 16;
    const int kh_steps = (ktot + 1) / 2;
    const uint32_t tw = tmem + (uint32_t)(W2_TMEM_W + khalf * 4 * KH) + ((uint32_t)(nt1 * 32) << 16);
    {
      const int wh = 8 * (nt1 % NTs) + gq;
      const uint4* wf = reinterpret_cast<const uint4*>(p.w) + ((int64_t)(b0 + nt1 / NTs) * Hq + wh) * (2 * N / 16) * 4 + tq;
#pragma unroll
      for (int i = 0; i < KH; ++i) {
        const int ks = khalf * kh_steps + i;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (nt1 < NT && i < kh_steps && wh < Hq && ks < ktot) v = __ldg(wf + ks * 4);
        w2_st4(tw + 4 * i, v);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
    }
    // this thread builds the cosine row n and the sine row N + n of the node basis; phase (modulo 2T) of its
    // frequency at the centre of the first super-tile
    const int n = tid;
    uint32_t ph2 = 0, d2 = 0;
    if (n < N) {
      const uint64_t centre2 = 2ull * ((uint64_t)a.mid_l0 + (uint64_t)l0) + (uint64_t)(J - 1);
      ph2 = phase_mod(centre2 % (uint64_t)T2, (uint32_t)n, T2);
      d2 = phase_mod((uint64_t)(2 * J), (uint32_t)n, T2);
    }
    // this chunk's verbatim-V partial starts from zero (only the verbatim dims are written at the end)
    for (int sq = 0; sq < nseq; ++sq) {
      float* ob = p.o_part + slot_of(b0 + sq) * Hq * D;
      for (int e = tid; e < Hq * D; e += 256) ob[e] = 0.f;
    }
    mbar_wait(tab_bar, 0, dead, p.err);
    for (int j = 0; j < nst; ++j) {
      const int buf = j & 1;
      unsigned char* fh = fnt + (buf * 2 + 0) * fterm;
      unsigned char* fl = fnt + (buf * 2 + 1) * fterm;
      if (j >= 2) mbar_wait(empty_sp + buf, ((j >> 1) - 1) & 1, dead, p.err);
      // ---- node basis: rotate the table to this super-tile's centre ------------------------------
      if (n < N) {
        float rs, rc;
        sincospif((float)ph2 * inv_T, &rs, &rc);
        ph2 += d2;
        if (ph2 >= T2) ph2 -= T2;
        // values of the 16 nodes: node 8 + kp = centre + d_kp, node 7 - kp = centre - d_kp; the lower and the upper
        // eight in turn (few live registers), each as four packed pairs of neighbouring nodes, hi and lo terms
        const int oc = w2_foff(n, 0), os = w2_foff(N + n, 0);
#pragma unroll
        for (int up = 0; up < 2; ++up) {
          float cv[8], sv[8];
#pragma unroll
          for (int kp = 0; kp < 8; ++kp) {
            const float e_c = ec[kp * N + n], e_s = es[kp * N + n];
            const float t1 = rc * e_c, t2 = rs * e_s, t3 = rs * e_c, t4 = rc * e_s;
            if (up) {
              cv[kp] = t1 - t2;
              sv[kp] = t3 + t4;
            } else {
              cv[7 - kp] = t1 + t2;
              sv[7 - kp] = t3 - t4;
            }
          }
          uint32_t ch[4], cl[4], sh[4], sl[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __half2 c2 = __floats2half2_rn(cv[2 * i], cv[2 * i + 1]), s2 = __floats2half2_rn(sv[2 * i], sv[2 * i + 1]);
            const float2 cf = __half22float2(c2), sf = __half22float2(s2);
            const __half2 c2l = __floats2half2_rn(cv[2 * i] - cf.x, cv[2 * i + 1] - cf.y);
            const __half2 s2l = __floats2half2_rn(sv[2 * i] - sf.x, sv[2 * i + 1] - sf.y);
            ch[i] = *reinterpret_cast<const uint32_t*>(&c2);
            cl[i] = *reinterpret_cast<const uint32_t*>(&c2l);
            sh[i] = *reinterpret_cast<const uint32_t*>(&s2);
            sl[i] = *reinterpret_cast<const uint32_t*>(&s2l);
          }
          *reinterpret_cast<uint4*>(fh + oc + 128 * up) = make_uint4(ch[0], ch[1], ch[2], ch[3]);
          *reinterpret_cast<uint4*>(fl + oc + 128 * up) = make_uint4(cl[0], cl[1], cl[2], cl[3]);
          *reinterpret_cast<uint4*>(fh + os + 128 * up) = make_uint4(sh[0], sh[1], sh[2], sh[3]);
          *reinterpret_cast<uint4*>(fl + os + 128 * up) = make_uint4(sl[0], sl[1], sl[2], sl[3]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes -> tcgen05.mma reads
      w2_spec_sync();
      // ---- scores at the nodes: s_node[16 x HN] = Fn[16 x 2N] * w[2N x HN] -----------------------
      if (nt1 < NT) {
        // consecutive MMAs never share an accumulator: a dependent MMA would wait out the latency of the one before
        float acc[6][4];
#pragma unroll
        for (int c = 0; c < 6; ++c)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[c][e] = 0.f;
        // four steps' fragments per read of tensor memory; the next four are on their way while these are used
        uint32_t wv[2][16];
        w2_ld16_nowait(tw, wv[0]);
        w2_wait_ld();
#pragma unroll
        for (int c = 0; c < KH / 4; ++c) {
          if (c + 1 < KH / 4) w2_ld16_nowait(tw + 16 * (c + 1), wv[(c + 1) & 1]);
#pragma unroll
          for (int ii = 0; ii < 4; ++ii) {
            const int i = 4 * c + ii, ks = khalf * kh_steps + i;
            const uint32_t bhi[2] = {wv[c & 1][4 * ii], wv[c & 1][4 * ii + 1]};
            const uint32_t blo[2] = {wv[c & 1][4 * ii + 2], wv[c & 1][4 * ii + 3]};
            if (i < kh_steps && ks < ktot) {
              uint32_t ah[4], al[4];
              ldsm_x4_t(ah, fh + ks * 512 + lane * 16);
              ldsm_x4_t(al, fl + ks * 512 + lane * 16);
              mma16816<__half>(acc[3 * (i & 1)], ah, bhi);
              mma16816<__half>(acc[3 * (i & 1) + 1], al, bhi);
              mma16816<__half>(acc[3 * (i & 1) + 2], ah, blo);
            }
          }
          if (c + 1 < KH / 4) w2_wait_ld();
        }
        float* red = snode32 + khalf * (FD * HN);
        const int col = 8 * nt1 + 2 * tq;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          red[(gq + 8 * (e >> 1)) * HN + col + (e & 1)] = ((acc[0][e] + acc[3][e]) + (acc[1][e] + acc[4][e])) + (acc[2][e] + acc[5][e]);
      }
      w2_spec_sync();
      {
        __half* sh_ = snode + (buf * 2 + 0) * 32 * 24;
        __half* sl_ = snode + (buf * 2 + 1) * 32 * 24;
        for (int e = tid; e < FD * HN; e += 256) {
          const int k = e / HN, h = e - k * HN;
          __half hi, lo;
          split_h(snode32[e] + snode32[FD * HN + e], hi, lo);
          sh_[h * 24 + k] = hi;
          sl_[h * 24 + k] = lo;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(full_sp + buf);
    }
    __syncthreads();
    if (wp == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(W2_TMEM_COLS) : "memory");
    }
    return;
  }

  if (wp >= 16) {
    // ============================= service warps ====================================================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(W2_VREG));
    const int sv = wp - 16;   // role, and (16 being a multiple of 4) the tensor-memory lane quadrant of this warp
    // Rescale this warp's lane quadrant of every tile whose running maximum moved at super-tile st (st > 0): the
    // factors lie in alpha_s; the updates issued so far must have landed first.
    auto rescale_quadrant = [&](int st) {
      const int buf = st & 1;
      mbar_wait(g_done, (uint32_t)(st - 1) & 1u, dead, p.err);
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      for (int tile = 0; tile < NT; ++tile) {
        float av[8];
        bool any = false;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          av[c] = alpha_s[(buf * 4 + tile) * 8 + c];
          any = any || av[c] != 1.f;
        }
        if (!any) continue;   // (the same for every lane)
        for (int mb = 0; mb < nblk; ++mb) {
          float v[8];
          const uint32_t ta = tmem + (uint32_t)(mb * 32 + tile * 8) + ((uint32_t)(sv * 32) << 16);
          w2_ld8(ta, v);
#pragma unroll
          for (int c = 0; c < 8; ++c) v[c] *= av[c];
          w2_st8(ta, v);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(resc_done);
    };
    int resc_seen = 0;
    if (sv == 1) {
      // ---- combine + issue: one pass per super-tile ---------------------------------------------------------
      // instruction descriptor of the g update: fp32 accumulator, fp16 A and B, both K-major, N = 32, M = 128
      const uint32_t idesc = (1u << 4) | ((uint32_t)(32 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      for (int st = 0; st < nst; ++st) {
        const int buf = st & 1;
        mbar_wait(pt_full + buf, (uint32_t)(st >> 1) & 1u, dead, p.err);
        if (*dead) break;
        if (st > 0) {
          const float al = lane < 8 * NT ? alpha_s[buf * 32 + lane] : 1.f;
          if (__any_sync(0xffffffffu, al != 1.f)) {
            if (lane == 0) {
              *resc_st = st;
              __threadfence_block();
              *resc_seq = resc_seen + 1;
            }
            __syncwarp();
            rescale_quadrant(st);
            mbar_wait(resc_done, (uint32_t)resc_seen & 1u, dead, p.err);
            ++resc_seen;
          }
          // the previous update has finished reading the B operands
          mbar_wait(g_done, (uint32_t)(st - 1) & 1u, dead, p.err);
        }
        // lane -> (tile, 16 of the tile's 128 (node, head) entries): node = 2 * (lane & 7) + {0, 1}, heads 0..7
        {
          const int tile = lane >> 3, n0 = 2 * (lane & 7);
          if (tile < NT) {
            const float* src = ptp + ((buf * 4 + tile) * 2) * (FD * 8) + n0 * 8;
            unsigned char* bh_ = ptb + tile * 256;   // the tile's 8 head columns: one 8-row group of the operand
            unsigned char* bl_ = ptb + 1024 + tile * 256;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              // heads 4c .. 4c+3 of the two nodes
              const float4 a0 = *reinterpret_cast<const float4*>(src + 4 * c);
              const float4 a1 = *reinterpret_cast<const float4*>(src + FD * 8 + 4 * c);
              const float4 b0_ = *reinterpret_cast<const float4*>(src + 8 + 4 * c);
              const float4 b1_ = *reinterpret_cast<const float4*>(src + FD * 8 + 8 + 4 * c);
              const float va[4] = {a0.x + a1.x, a0.y + a1.y, a0.z + a1.z, a0.w + a1.w};
              const float vb[4] = {b0_.x + b1_.x, b0_.y + b1_.y, b0_.z + b1_.z, b0_.w + b1_.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                // operand element (row h, K index node): core matrix (node >> 3), row h, position node & 7; this
                // lane's two nodes are neighbours
                const int h = 4 * c + i;
                __half h0, l0_, h1, l1_;
                split_h(va[i], h0, l0_);
                split_h(vb[i], h1, l1_);
                const int off = (n0 >> 3) * 128 + h * 16 + (n0 & 7) * 2;
                *reinterpret_cast<__half2*>(bh_ + off) = __halves2half2(h0, h1);
                *reinterpret_cast<__half2*>(bl_ + off) = __halves2half2(l0_, l1_);
              }
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t fh = smem_u32(fnt + (buf * 2 + 0) * fterm), fl = smem_u32(fnt + (buf * 2 + 1) * fterm);
          const uint64_t bdh = w2_desc(smem_u32(ptb), 128, 256), bdl = w2_desc(smem_u32(ptb + 1024), 128, 256);
          for (int mb = 0; mb < nblk; ++mb) {   // all four column tiles at once: 128 rows x 32 head columns
            const uint64_t adh = w2_desc(fh + mb * 4096, 128, 256), adl = w2_desc(fl + mb * 4096, 128, 256);
            const uint32_t d = tmem + (uint32_t)(mb * 32);
            w2_mma(d, adl, bdh, idesc, st > 0 ? 1u : 0u);
            w2_mma(d, adh, bdl, idesc, 1u);
            w2_mma(d, adh, bdh, idesc, 1u);
          }
          w2_commit(empty_sp + buf);   // the basis buffer may be rebuilt once these have been read
          w2_commit(g_done);           // ... and the accumulators are up to date
        }
        __syncwarp();
      }
      if (lane == 0) {
        __threadfence_block();
        *svc_exit = 1;
      }
      __syncwarp();
    } else {
      // ---- warp 16 refills the ring; warps 16, 18 and 19 answer rescale requests until warp 17 is through -------
      int t_next = sv == 0 ? 3 : n_tiles;
      long long t_last = clock64();
      while (!*dead) {
        bool progress = false;
        if (t_next < n_tiles) {
          const int i = t_next - 3;   // the half tile whose slot is reused
          if (mbar_test(empty_slot + i % 3, (uint32_t)(i / 3) & 1u)) {
            issue_tile(t_next);
            ++t_next;
            progress = true;
          }
        }
        int rs = 0, ex = 0;
        if (lane == 0) {
          rs = *resc_seq;
          ex = *svc_exit;
        }
        rs = __shfl_sync(0xffffffffu, rs, 0);
        ex = __shfl_sync(0xffffffffu, ex, 0);
        if (rs != resc_seen) {
          __threadfence_block();
          rescale_quadrant(*resc_st);
          ++resc_seen;
          progress = true;
        } else if (ex && t_next >= n_tiles) {
          break;   // (warp 17 raises the exit flag only after its last request has been answered)
        }
        if (progress) {
          t_last = clock64();
        } else {
          __nanosleep(sv == 0 ? 60 : 400);
          if (clock64() - t_last > 2000000000LL) {   // about a second without any event: give up
            *dead = 1;
            atomicExch(p.err, 1);
          }
        }
      }
    }
    // ---- g of every tile -> g_part[h][row] ----------------------------------------------------------------------
    // Each service warp moves its lane quadrant of every row block into shared memory (the node-basis buffers: the
    // last update has read them), head-major like g_part; one bulk copy per tile then takes it to global memory.
    // (Plain stores from registers, 128 per warp, queue behind the K / V stream of the other CTAs for microseconds.)
    if (nst > 0) mbar_wait(g_done, (uint32_t)(nst - 1) & 1u, dead, p.err);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    float* g_s = reinterpret_cast<float*>(fnt);   // [tile][8 heads][2N]
    for (int tile = 0; tile < NT; ++tile) {
      for (int mb = 0; mb < nblk; ++mb) {
        float v[8];
        w2_ld8(tmem + (uint32_t)(mb * 32 + tile * 8) + ((uint32_t)(sv * 32) << 16), v);
        const int row = 128 * mb + 32 * sv + lane;
        if (row < 2 * N) {
#pragma unroll
          for (int c = 0; c < 8; ++c) g_s[(tile * 8 + c) * 2 * N + row] = nst > 0 ? v[c] : 0.f;
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes -> bulk copy reads
    asm volatile("bar.sync 6, 128;\n" ::: "memory");
    if (sv == 0 && lane == 0) {
      for (int tile = 0; tile < NT; ++tile) {
        const int sq = tile / NTs, ntl = tile - sq * NTs;
        const int heads = min(8, Hq - 8 * ntl);
        float* gb = p.g_part + ((((int64_t)(b0 + sq) * p.n_mid_chunks + chunk) * Hq) + 8 * ntl) * 2 * N;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(gb), "r"(smem_u32(g_s + tile * 8 * 2 * N)),
                     "r"((uint32_t)(heads * 2 * N * 4)) : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
      asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");   // shared memory must outlive the reads
    }
    __syncthreads();
    return;
  }

  // ============================= score warps ======================================================
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(W2_QREG));
  const int qw = wp - 8, nt = qw & 3, half = qw >> 2;
  const bool act = nt < NT;
  if (!act) {   // no column tile for this warp
    __syncthreads();
    return;
  }
  const int sq = nt / NTs, ntl = nt - sq * NTs;   // sequence of this column tile, tile within the sequence
  const int bb = b0 + sq;
  __half* pw16 = reinterpret_cast<__half*>(smem + L.pw) + qw * 64 * 8;   // this warp's probabilities [64 tokens][8 heads]
  T* pwT = reinterpret_cast<T*>(pw16);
  // column ranges of this warp's heads in the verbatim stores
  int kc0, kc1, mtv0, mtvn;
  {
    const int g0 = (8 * ntl) / R, g1 = (min(Hq, 8 * ntl + 8) - 1) / R;
    kc0 = knh_s[g0] & ~15;
    kc1 = (knh_s[g1 + 1] + 15) & ~15;
    mtv0 = vnh_s[g0] >> 4;
    mtvn = ((vnh_s[g1 + 1] + 15) >> 4) - mtv0;
  }
  const int nks = (kc1 - kc0) >> 4;   // 16-column steps of the verbatim-K contraction
  // the heads' verbatim-K query entries as MMA B fragments (raw model-dtype values; the softmax scale is
  // applied to the fp32 sums)
  uint32_t bq[W2_KS][2];
  {
    const T* q = reinterpret_cast<const T*>(a.q) + (int64_t)bb * a.q_sb;
    const int h = 8 * ntl + gq;
    const int g = h / R;
    int c_lo = 0, c_hi = 0;
    if (h < Hq) {
      c_lo = knh_s[g];
      c_hi = knh_s[g + 1];
    }
#pragma unroll
    for (int ks = 0; ks < W2_KS; ++ks) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int col = kc0 + 16 * ks + 2 * tq + 8 * r;
        T v0 = from_f32<T>(0.f), v1 = from_f32<T>(0.f);
        if (col >= c_lo && col < c_hi) v0 = q[h * D + kn_s[col] - g * D];
        if (col + 1 >= c_lo && col + 1 < c_hi) v1 = q[h * D + kn_s[col + 1] - g * D];
        bq[ks][r] = pack_pair<T>(v0, v1);
      }
    }
  }
  const int hl0 = 8 * ntl + 2 * tq;   // the heads of sequence bb this thread's two columns stand for
  const float cst0 = (hl0 < Hq) ? p.cst[(int64_t)bb * Hq + hl0] : 0.f;
  const float cst1 = (hl0 + 1 < Hq) ? p.cst[(int64_t)bb * Hq + hl0 + 1] : 0.f;
  const int cbK = sq * nbK * 64, cbV = sq * nbV * 64;   // first column of this sequence's boxes inside a ring slot
  float m_run0 = NEG_BIG, m_run1 = NEG_BIG, lsum0 = 0.f, lsum1 = 0.f;
  float Oacc[W2_MTV][4];
#pragma unroll
  for (int i = 0; i < W2_MTV; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) Oacc[i][e] = 0.f;

  mbar_wait(tab_bar, 0, dead, p.err);
  for (int st = 0; st < nst; ++st) {
    const int buf = st & 1;
    const int tok0 = l0 + st * J + half * FH;   // first token of this warp's half
    float sc[4][4];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[mt][e] = 0.f;
    const int iK = 4 * st + half, sK = iK % 3;
    const uint32_t parK = (uint32_t)(iK / 3) & 1u;
    // Every run of MMAs below visits four different accumulators in turn: a dependent MMA issued right after
    // its predecessor would wait out that one's whole latency.
    // ---- verbatim-dim scores from the K rows (needs only the K tile, so it comes first) -----------
    mbar_wait(full_slot + sK, parK, dead, p.err);
    {
      const unsigned char* ks_ = slots + sK * L.slot_bytes;
#pragma unroll
      for (int ks = 0; ks < W2_KS; ++ks) {
        if (ks < nks) {
#pragma unroll
          for (int mt = 0; mt < 4; ++mt) {
            uint32_t af[4];
            ldsm_x4(af, ks_ + sw_off(16 * mt + lds_a_row(lane), (cbK + kc0 + 16 * ks + lds_a_col(lane)) >> 3));
            mma16816<T>(sc[mt], af, bq[ks]);
          }
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      sc[mt][0] = p.c2 * sc[mt][0] + cst0;
      sc[mt][1] = p.c2 * sc[mt][1] + cst1;
      sc[mt][2] = p.c2 * sc[mt][2] + cst0;
      sc[mt][3] = p.c2 * sc[mt][3] + cst1;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_slot + sK);
    mbar_wait(full_sp + buf, (st >> 1) & 1, dead, p.err);
    {
      // ---- add the node scores interpolated to this warp's 64 tokens ---------------------------------
      uint32_t bh[2], bl[2];
      const int boff = (8 * nt + lds_b_row(lane)) * 24 + lds_b_col(lane);
      ldsm_x2(bh, snode + (buf * 2 + 0) * 32 * 24 + boff);
      ldsm_x2(bl, snode + (buf * 2 + 1) * 32 * 24 + boff);
      const int ioff = (half * FH + lds_a_row(lane)) * 24 + lds_a_col(lane);
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t al[4];
        ldsm_x4(al, interp_lo + ioff + 16 * mt * 24);
        mma16816<__half>(sc[mt], al, bh);
      }
      uint32_t ah[4][4];
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        ldsm_x4(ah[mt], interp_hi + ioff + 16 * mt * 24);
        mma16816<__half>(sc[mt], ah[mt], bl);
      }
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) mma16816<__half>(sc[mt], ah[mt], bh);
    }
    // ---- softmax over the 128 tokens of the super-tile (both halves agree on the maximum) ----------
    float mx0 = NEG_BIG, mx1 = NEG_BIG;
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      const bool ok0 = (tok0 + 16 * mt + gq) < l1, ok1 = (tok0 + 16 * mt + gq + 8) < l1;
      mx0 = fmaxf(mx0, fmaxf(ok0 ? sc[mt][0] : NEG_BIG, ok1 ? sc[mt][2] : NEG_BIG));
      mx1 = fmaxf(mx1, fmaxf(ok0 ? sc[mt][1] : NEG_BIG, ok1 ? sc[mt][3] : NEG_BIG));
    }
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    // (two copies by super-tile parity: a warp may be a whole super-tile ahead of its tile mate, which has not read yet)
    if (gq == 0) {
      mx[((buf * 4 + nt) * 2 + half) * 8 + 2 * tq] = mx0;
      mx[((buf * 4 + nt) * 2 + half) * 8 + 2 * tq + 1] = mx1;
    }
    w2_tile_sync(nt);
    mx0 = fmaxf(mx0, mx[((buf * 4 + nt) * 2 + (half ^ 1)) * 8 + 2 * tq]);
    mx1 = fmaxf(mx1, mx[((buf * 4 + nt) * 2 + (half ^ 1)) * 8 + 2 * tq + 1]);
    // lazy running maximum: it moves only when this super-tile exceeds it by more than 2^W2_LAZY
    float al0 = 1.f, al1 = 1.f;
    if (mx0 > m_run0 + W2_LAZY) {
      al0 = exp2f(m_run0 - mx0);
      m_run0 = mx0;
    }
    if (mx1 > m_run1 + W2_LAZY) {
      al1 = exp2f(m_run1 - mx1);
      m_run1 = mx1;
    }
    // the factors travel with the projected probabilities: the service warps rescale the accumulators in tensor memory
    if (half == 0 && gq == 0) {
      alpha_s[(buf * 4 + nt) * 8 + 2 * tq] = al0;
      alpha_s[(buf * 4 + nt) * 8 + 2 * tq + 1] = al1;
    }
    if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
      lsum0 *= al0;
      lsum1 *= al1;
#pragma unroll
      for (int i = 0; i < W2_MTV; ++i) {
        Oacc[i][0] *= al0;
        Oacc[i][1] *= al1;
        Oacc[i][2] *= al0;
        Oacc[i][3] *= al1;
      }
    }
    __half2 ph[4][2];   // probabilities rounded to fp16: (head 2tq, 2tq+1) of token rows gq and gq+8 per 16-token tile
    {
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        const bool ok0 = (tok0 + 16 * mt + gq) < l1, ok1 = (tok0 + 16 * mt + gq + 8) < l1;
        ph[mt][0] = __floats2half2_rn(ok0 ? exp2f(sc[mt][0] - m_run0) : 0.f, ok0 ? exp2f(sc[mt][1] - m_run1) : 0.f);
        ph[mt][1] = __floats2half2_rn(ok1 ? exp2f(sc[mt][2] - m_run0) : 0.f, ok1 ? exp2f(sc[mt][3] - m_run1) : 0.f);
        // token-major [token][8 heads]: a thread's two heads are one 32-bit store, the B operands come back
        // through ldmatrix.trans; the sums use the rounded values
        const int j0 = 16 * mt + gq;
        *reinterpret_cast<__half2*>(pw16 + j0 * 8 + 2 * tq) = ph[mt][0];
        *reinterpret_cast<__half2*>(pw16 + (j0 + 8) * 8 + 2 * tq) = ph[mt][1];
        const float2 f0 = __half22float2(ph[mt][0]), f1 = __half22float2(ph[mt][1]);
        s0 += f0.x + f1.x;
        s1 += f0.y + f1.y;
      }
      lsum0 += s0;   // this thread's rows only; lanes and halves are added at the end
      lsum1 += s1;
    }
    __syncwarp();
    // ---- project the probabilities onto the nodes: pt[16 x 8] = Interp^T[16 x 64] * P[64 x 8] ------
    uint32_t bp[4][2];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) ldsm_x2_t(bp[ks], pw16 + (16 * ks + (lane & 15)) * 8);
    {
      float pt4[4][4];
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) pt4[c][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t af[4], al_[4];
        const int ioff = (half * FH + 16 * ks + lds_at_row(lane)) * 24 + lds_at_col(lane);
        ldsm_x4_t(af, interp_hi + ioff);
        ldsm_x4_t(al_, interp_lo + ioff);
        mma16816<__half>(pt4[2 * (ks & 1)], af, bp[ks]);
        mma16816<__half>(pt4[2 * (ks & 1) + 1], al_, bp[ks]);
      }
      // this half's share goes to the service warp, which adds the two up and issues the g update
      float* dst = ptp + (((buf * 4 + nt) * 2 + half) * FD) * 8;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        dst[(gq + 8 * (e >> 1)) * 8 + 2 * tq + (e & 1)] = (pt4[0][e] + pt4[2][e]) + (pt4[1][e] + pt4[3][e]);
      __syncwarp();
      if (lane == 0) mbar_arrive(pt_full + buf);
    }
    // ---- verbatim-V numerators -------------------------------------------------------------------
    uint32_t bp_lo[4][2];
    if constexpr (kBf16) {
      // an fp16 value splits exactly into two bf16 values, so the verbatim-V GEMM (model dtype) sees the same
      // probabilities as the spectral side and the denominator
      using T2 = __nv_bfloat162;
      float2 res[4][2];   // what the bf16 rounding leaves over
      __syncwarp();
#pragma unroll
      for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float2 f = __half22float2(ph[mt][r]);
          const T2 hi = __floats2bfloat162_rn(f.x, f.y);
          const float2 hf = __bfloat1622float2(hi);
          res[mt][r] = make_float2(f.x - hf.x, f.y - hf.y);
          *reinterpret_cast<T2*>(pwT + (16 * mt + gq + 8 * r) * 8 + 2 * tq) = hi;
        }
      __syncwarp();
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) ldsm_x2_t(bp[ks], pwT + (16 * ks + (lane & 15)) * 8);
      __syncwarp();
#pragma unroll
      for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int r = 0; r < 2; ++r)
          *reinterpret_cast<T2*>(pwT + (16 * mt + gq + 8 * r) * 8 + 2 * tq) = __floats2bfloat162_rn(res[mt][r].x, res[mt][r].y);
      __syncwarp();
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) ldsm_x2_t(bp_lo[ks], pwT + (16 * ks + (lane & 15)) * 8);
    }
    const int iV = 4 * st + 3 - half, sV = iV % 3;
    const uint32_t parV = (uint32_t)(iV / 3) & 1u;
    mbar_wait(full_slot + sV, parV, dead, p.err);
    {
      const unsigned char* vs_ = slots + sV * L.slot_bytes;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t af[W2_MTV][4];
#pragma unroll
        for (int i = 0; i < W2_MTV; ++i)
          if (i < mtvn)
            ldsm_x4_t(af[i], vs_ + sw_off(16 * ks + lds_at_row(lane), (cbV + 16 * (mtv0 + i) + lds_at_col(lane)) >> 3));
#pragma unroll
        for (int i = 0; i < W2_MTV; ++i)
          if (i < mtvn) mma16816<T>(Oacc[i], af[i], bp[ks]);
        if (kBf16) {
#pragma unroll
          for (int i = 0; i < W2_MTV; ++i)
            if (i < mtvn) mma16816<T>(Oacc[i], af[i], bp_lo[ks]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_slot + sV);
  }

  // ---- chunk partials ---------------------------------------------------------------------------
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    lsum0 += __shfl_xor_sync(0xffffffffu, lsum0, o);
    lsum1 += __shfl_xor_sync(0xffffffffu, lsum1, o);
  }
  if (half == 1 && gq == 0) {
    lx[nt * 8 + 2 * tq] = lsum0;
    lx[nt * 8 + 2 * tq + 1] = lsum1;
  }
  __syncthreads();   // the spectral warps have zeroed this chunk's verbatim-V partial; all ring traffic is over
  {
    // the verbatim-V numerators of the second half -> shared memory (the ring slots are free now), the first half
    // adds them and writes the chunk's partial
    float* red = reinterpret_cast<float*>(slots) + nt * (W2_MTV * 4 * 32);
    if (half == 1) {
#pragma unroll
      for (int i = 0; i < W2_MTV; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[(i * 4 + e) * 32 + lane] = Oacc[i][e];
    }
    w2_tile_sync(nt);
    if (half == 0) {
      const int64_t slot_id = slot_of(bb);
      if (gq == 0) {
        if (hl0 < Hq) {
          p.m_part[slot_id * Hq + hl0] = m_run0;
          p.l_part[slot_id * Hq + hl0] = lsum0 + lx[nt * 8 + 2 * tq];
        }
        if (hl0 + 1 < Hq) {
          p.m_part[slot_id * Hq + hl0 + 1] = m_run1;
          p.l_part[slot_id * Hq + hl0 + 1] = lsum1 + lx[nt * 8 + 2 * tq + 1];
        }
      }
      float* ob = p.o_part + slot_id * Hq * D;
#pragma unroll
      for (int i = 0; i < W2_MTV; ++i) {
        if (i < mtvn) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float v = Oacc[i][e] + red[(i * 4 + e) * 32 + lane];
            const int c = 16 * (mtv0 + i) + gq + 8 * (e >> 1);
            const int h = hl0 + (e & 1);
            if (c < Mn_v && h < Hq) {
              const int g = h / R;
              if (c >= vnh_s[g] && c < vnh_s[g + 1]) ob[h * D + vn_s[c] - g * D] = v;
            }
          }
        }
      }
    }
  }
}
