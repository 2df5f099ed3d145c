// Warp-specialised form of the tensor-core middle-span pass.  Included by decode.cu after
// decode_fast.cuh (same namespace, same MMA / TMA primitives, same mathematics).
//
// decode_fast.cuh runs the phases of a super-tile one after another on all warps, so every phase
// exposes its own latency.  Here the 16 warps of a CTA split into two groups that work on different
// super-tiles at the same time:
//
//   spectral warps (0..7)   node basis of super-tile j (rotation of a fixed table) and the node
//                           scores  s_node = Fn_t * w  (w stays in registers as MMA fragments);
//                           they run up to two super-tiles ahead of the score warps
//   score warps (8..15)     warp = (8-head column tile nt, 64-token half): interpolation of the node
//                           scores, verbatim-K scores, softmax, projection of the probabilities onto
//                           the nodes, verbatim-V numerators; then all eight add the projected
//                           probabilities to g (each owns 16-row tiles of the 2N rows)
//
// Hand-offs are mbarriers with bounded waits (node scores + basis: full/empty per buffer; K/V half
// tiles: full/empty per ring slot); the two halves of a column tile agree on the running maximum
// through a 64-thread named barrier, and the score warps meet once per super-tile before the g update.
// The score warps refill the ring themselves: one warp of a half (column tile 0 for K tiles, tile 1 for V
// tiles) waits until the other warps of that half have released the slot and issues the TMA boxes of the
// tile three places ahead.
// Registers move with the work: the spectral warps give up registers (setmaxnreg) that the score
// warps, which hold the g and verbatim-V accumulators, take over.
//
// When a sequence has 16 or fewer query heads a CTA takes the column tiles of two or four sequences of the
// batch (their K/V boxes side by side in a ring slot): the node basis and the interpolation weights are the
// same for all of them, so narrow head counts do not leave score warps idle.
//
// Up to 2N = 512 coefficient rows a CTA serves four column tiles (32 heads) and keeps two node-basis buffers, so
// the spectral warps run ahead.  For 512 < 2N <= 1024 (template parameter GN = 2) the heads of a sequence are
// divided into groups of 16 that go to different CTAs: a CTA then serves two column tiles, fetches only the
// verbatim columns of its own KV heads, splits the 2N rows four ways among the spectral warps, gives every score
// warp eight 16-row tiles of g, and keeps a single node-basis buffer (the accumulators and the w fragments cost
// the same registers in both forms).
//
// The node set is symmetric about the centre of the super-tile, so the basis table holds the eight
// nodes right of the centre only and the rotation is taken at the centre (a half-integer position:
// phases are kept modulo 2T).
#pragma once

constexpr int WS_KS_MAX = 8;   // most 16-column steps of verbatim K (and 16-column tiles of verbatim V) a score warp
                               // handles (template parameter KS: 4 or 8)
constexpr int WS_T = 512;
constexpr int WS_SREG = 56, WS_QREG = 200;   // registers per thread of the two groups (sum = 2 x 128): the
// score warps must not spill (with 222 KB of shared memory the L1 that would catch spills is tiny), the spectral
// warps have time to spare


struct WsSmem {
  int ec, es, fnt, interp_hi, interp_lo, snode32, snode, pw, ptx, ptp, alpha, mx, lx, bars, slots, total;
  int fpitch, kpad, slot_bytes;
};
__host__ __device__ inline WsSmem ws_smem(int N, int Mn_k, int Mn_v, int NB = 2, int KP = 2) {
  WsSmem s;
  int o = 0;
  auto take = [&](int bytes) {
    int r = o;
    o += (bytes + 15) / 16 * 16;
    return r;
  };
  s.kpad = (2 * N + 15) / 16 * 16;
  s.fpitch = s.kpad + 8;
  s.ec = take(8 * N * 4);
  s.es = take(8 * N * 4);
  s.fnt = take(NB * 2 * FD * s.fpitch * 2);   // [buffer][hi, lo][node][fpitch]
  s.interp_hi = take(128 * 24 * 2);
  s.interp_lo = take(128 * 24 * 2);
  s.snode32 = take(KP * FD * 32 * 4);         // partial node scores of the KP parts of the 2N rows
  s.snode = take(2 * 2 * 32 * 24 * 2);        // [buffer][hi, lo][head][24]
  s.pw = take(8 * 64 * 8 * 2);                // per score warp: probabilities [64 tokens][8 heads]
  s.ptx = take(2 * 2 * 32 * 24 * 2);          // [buffer][hi, lo][head][24]  probabilities on the nodes
  s.ptp = take(4 * FD * 8 * 4);               // second half's contribution to them, per column tile
  s.alpha = take(2 * 32 * 4);
  s.mx = take(4 * 2 * 8 * 4);
  s.lx = take(4 * 8 * 4);
  s.bars = take(16 * 8);
  const int mnk16 = (Mn_k + 15) / 16 * 16, mnv16 = (Mn_v + 15) / 16 * 16;
  const int w = mnk16 > mnv16 ? mnk16 : mnv16;
  const int boxes = (w + 63) / 64 > 0 ? (w + 63) / 64 : 1;
  s.slot_bytes = boxes * 8192;
  o = (o + 1023) / 1024 * 1024;
  s.slots = take(3 * s.slot_bytes);
  s.total = o;
  return s;
}

__device__ __forceinline__ void ws_group_sync(int id) { asm volatile("bar.sync %0, 256;\n" ::"r"(id) : "memory"); }
__device__ __forceinline__ void ws_pair_sync(int id) { asm volatile("bar.sync %0, 64;\n" ::"r"(id) : "memory"); }

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(T a, T b) {
  const uint16_t lo = *reinterpret_cast<uint16_t*>(&a), hi = *reinterpret_cast<uint16_t*>(&b);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

template <typename T, int GN, int KS>
__device__ void mid_chunk_ws(const DecodeParams& p, int b0, int chunk, int hg, unsigned char* smem) {
  constexpr int MTV = KS;       // 16-column tiles of verbatim V a score warp owns
  constexpr int J = 128, HN = 32;
  constexpr int GI = 16 / GN;   // 16-row tiles of g per score warp
  constexpr int KP = 8 / GN;    // parts of the 2N rows among the spectral warps of a column tile
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  const fa_decode_args_t& a = p.a;
  const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const int N = a.N, D = a.D, R = p.R, Hq = a.Hq, Mn_k = a.Mn_k, Mn_v = a.Mn_v;
  // A CTA serves `nseq` sequences at once when a sequence has few heads: column tile nt belongs to sequence
  // b0 + nt / NTs and is that sequence's tile nt % NTs; the node basis is the same for all of them.
  const int NB = p.wsNB;                 // node-basis buffers
  // A column tile holds HPT heads (8, or the largest multiple of the GQA ratio below 8 so that a tile never cuts
  // a KV head's query heads in two: 6 for three query heads per KV head); columns HPT..7 of a tile are padding.
  // (the KS = 4 instances are compiled for HPT = 8, so that the common shapes pay nothing for the general case)
  const int HPT = KS == 4 ? 8 : p.wsHPT;
  const int hb = hg * HPT * GN;          // first head of this CTA's head group (0 unless the heads are split)
  const int NTs = p.wsHG > 1 ? min(GN, (Hq - hb + HPT - 1) / HPT) : p.wsNTs;
  const int nseq = min(p.wsSEQ, a.B - b0);
  const int NT = nseq * NTs;
  const uint32_t T2 = 2u * (uint32_t)a.T;
  const float inv_T = 1.0f / (float)a.T;
  // a ring slot holds the 64-column boxes of all wsSEQ sequences side by side
  const WsSmem L = ws_smem(N, p.wsSlotK, p.wsSlotV, NB, KP);
  float* ec = reinterpret_cast<float*>(smem + L.ec);
  float* es = reinterpret_cast<float*>(smem + L.es);
  __half* fnt = reinterpret_cast<__half*>(smem + L.fnt);
  __half* interp_hi = reinterpret_cast<__half*>(smem + L.interp_hi);
  __half* interp_lo = reinterpret_cast<__half*>(smem + L.interp_lo);
  float* snode32 = reinterpret_cast<float*>(smem + L.snode32);
  __half* snode = reinterpret_cast<__half*>(smem + L.snode);
  __half* ptx = reinterpret_cast<__half*>(smem + L.ptx);
  float* ptp = reinterpret_cast<float*>(smem + L.ptp);
  float* alpha = reinterpret_cast<float*>(smem + L.alpha);
  float* mx = reinterpret_cast<float*>(smem + L.mx);
  float* lx = reinterpret_cast<float*>(smem + L.lx);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* full_slot = bars;         // [3] a K or V half tile has landed
  uint64_t* empty_slot = bars + 3;    // [3] the score warps of its half are done with it
  uint64_t* full_sp = bars + 6;       // [2] node basis + node scores of a super-tile are written
  uint64_t* empty_sp = bars + 8;      // [2] ... and no longer needed
  volatile int* dead = reinterpret_cast<volatile int*>(bars + 10);
  unsigned char* slots = smem + L.slots;
  const int fpitch = L.fpitch, kpad = L.kpad;
  const int ktot = kpad / 16;

  const int l0 = chunk * p.mid_chunk;
  const int l1 = min(a.n_mid, l0 + p.mid_chunk);
  const int nst = (l1 - l0 + J - 1) / J;
  const int n_tiles = 4 * nst;   // per super-tile: K half 0, K half 1, V half 0, V half 1
  // verbatim columns of this CTA's KV heads (all of them unless the heads are split): whole 64-column boxes
  const int gA = hb / R, gB = (min(Hq, hb + HPT * GN) - 1) / R;
  const int colK0 = a.kn_h[gA] & ~63, colV0 = a.vn_h[gA] & ~63;
  const int nbK = (a.kn_h[gB + 1] - colK0 + 63) / 64, nbV = (a.vn_h[gB + 1] - colV0 + 63) / 64;
  auto slot_of = [&](int bb) { return (int64_t)bb * p.NCH + p.n_il_chunks + chunk; };

  // called by a whole warp: request half tile i into ring slot i % 3
  auto issue_tile = [&](int i) {
    if (i >= n_tiles) return;
    const int s = i % 3, r = i & 3;
    const int lf = l0 + (i >> 2) * J + (r & 1) * FH;
    const bool is_v = r >= 2;
    const int nb = is_v ? nbV : nbK;
    if (lane == 0) mbar_expect_tx(full_slot + s, (uint32_t)(nseq * nb) * 8192u);
    __syncwarp();
    if (lane < nseq * nb) {   // the boxes of sequence 0, then those of sequence 1, ...
      const int sq = lane / nb, bx = lane - sq * nb;
      tma_box(slots + s * L.slot_bytes + lane * 8192, is_v ? &p.tm_v : &p.tm_k, (is_v ? colV0 : colK0) + 64 * bx, lf,
              b0 + sq, full_slot + s);
    }
  };

  // ---- set-up (all warps) ---------------------------------------------------------------------
  if (tid == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(full_slot + i, 1);
      mbar_init(empty_slot + i, NT);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(full_sp + i, 8);
      mbar_init(empty_sp + i, 8);
    }
    *dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  for (int e = tid; e < KP * FD * 32; e += WS_T) snode32[e] = 0.f;
  __syncthreads();
  if (wp == 8) {
    if (lane == 0) {
      if (nbK) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&p.tm_k) : "memory");
      if (nbV) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&p.tm_v) : "memory");
    }
    for (int i = 0; i < 3; ++i) issue_tile(i);
  }
  for (int e = tid; e < 8 * N; e += WS_T) {
    const int k = e / N, n = e - k * N;
    // node 8+k lies (2 x_k - 127) / 2 tokens right of the centre
    const uint32_t ph = phase_mod((uint64_t)(2 * c_nodes128[8 + k] - (J - 1)), (uint32_t)n, T2);
    float s, c;
    sincospif((float)ph * inv_T, &s, &c);
    ec[e] = c;
    es[e] = s;
  }
  for (int e = tid; e < J * FD; e += WS_T) {
    const int j = e / FD, k = e - j * FD;
    __half hi, lo;
    split_h(g_interp128[e], hi, lo);
    interp_hi[j * 24 + k] = hi;
    interp_lo[j * 24 + k] = lo;
  }
  __syncthreads();

  if (wp < 8) {
    // =========================== spectral warps ================================================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(WS_SREG));
    const int nt1 = wp % GN, khalf = wp / GN;   // column tile and part of the 2N rows of this warp
    // this chunk's verbatim-V partial starts from zero (the score warps add into it at the end)
    {
      const int nh = p.wsHG > 1 ? min(Hq - hb, HPT * GN) : Hq;   // heads this CTA writes
      for (int sq = 0; sq < nseq; ++sq) {
        float* ob = p.o_part + (slot_of(b0 + sq) * Hq + hb) * D;
        for (int e = tid; e < nh * D; e += 256) ob[e] = 0.f;
      }
    }
    // w as persistent B fragments (hi / lo): k = coefficient row, n = head; this warp holds column tile nt1 for part
    // `khalf` of the 2N rows.  The prepare kernel has written them in fragment order: one 16-byte load per step.
    constexpr int KH = 16;
    const int kh_steps = (ktot + KP - 1) / KP;
    uint32_t bhi[KH][2], blo[KH][2];
    {
      const int h = gq < HPT ? hb + HPT * (nt1 % NTs) + gq : Hq   /* padding columns: no head */;
      const uint4* wf = reinterpret_cast<const uint4*>(p.w) + ((int64_t)(b0 + nt1 / NTs) * Hq + h) * (2 * N / 16) * 4 + tq;
#pragma unroll
      for (int i = 0; i < KH; ++i) {
        const int ks = khalf * kh_steps + i;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (nt1 < NT && i < kh_steps && h < Hq && ks < ktot) v = __ldg(wf + ks * 4);
        bhi[i][0] = v.x;
        bhi[i][1] = v.y;
        blo[i][0] = v.z;
        blo[i][1] = v.w;
      }
    }
    // phases (modulo 2T) of this thread's two frequencies at the centre of the first super-tile
    // (a thread serves the frequency pairs np0, np0 + 128: the second one exists for N > 256 only)
    constexpr int NIT = GN == 4 ? 1 : 2;
    const int np0 = tid & 127, kk = tid >> 7;
    uint32_t ph2[NIT][2], d2[NIT][2];
#pragma unroll
    for (int it = 0; it < NIT; ++it)
#pragma unroll
      for (int f = 0; f < 2; ++f) {
        const uint32_t n = (uint32_t)(2 * (np0 + 128 * it) + f);
        const uint64_t centre2 = 2ull * ((uint64_t)a.mid_l0 + (uint64_t)l0) + (uint64_t)(J - 1);
        ph2[it][f] = phase_mod(centre2 % (uint64_t)T2, n, T2);
        d2[it][f] = phase_mod((uint64_t)(2 * J), n, T2);
      }
    for (int j = 0; j < nst; ++j) {
      const int buf = j & 1, fb = j % NB;
      __half* fh = fnt + (fb * 2 + 0) * FD * fpitch;
      __half* fl = fnt + (fb * 2 + 1) * FD * fpitch;
      if (j >= NB) mbar_wait(empty_sp + fb, ((j / NB) - 1) & 1, dead, p.err);
      // ---- node basis: rotate the table to this super-tile's centre ------------------------------
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        const int np = np0 + 128 * it;
        if (2 * np >= N) break;
        float rc[2], rs[2];
#pragma unroll
        for (int f = 0; f < 2; ++f) {
          sincospif((float)ph2[it][f] * inv_T, &rs[f], &rc[f]);
          ph2[it][f] += d2[it][f];
          if (ph2[it][f] >= T2) ph2[it][f] -= T2;
        }
        auto put = [&](int k, float c0, float c1, float s0, float s1) {
          const __half2 ch = __floats2half2_rn(c0, c1), sh = __floats2half2_rn(s0, s1);
          const float2 chf = __half22float2(ch), shf = __half22float2(sh);
          const __half2 cl = __floats2half2_rn(c0 - chf.x, c1 - chf.y), sl = __floats2half2_rn(s0 - shf.x, s1 - shf.y);
          *reinterpret_cast<__half2*>(fh + k * fpitch + 2 * np) = ch;
          *reinterpret_cast<__half2*>(fl + k * fpitch + 2 * np) = cl;
          *reinterpret_cast<__half2*>(fh + k * fpitch + N + 2 * np) = sh;
          *reinterpret_cast<__half2*>(fl + k * fpitch + N + 2 * np) = sl;
        };
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int kp = kk * 4 + i;
          const float2 e_c = *reinterpret_cast<const float2*>(ec + kp * N + 2 * np);
          const float2 e_s = *reinterpret_cast<const float2*>(es + kp * N + 2 * np);
          const float t1a = rc[0] * e_c.x, t2a = rs[0] * e_s.x, t3a = rs[0] * e_c.x, t4a = rc[0] * e_s.x;
          const float t1b = rc[1] * e_c.y, t2b = rs[1] * e_s.y, t3b = rs[1] * e_c.y, t4b = rc[1] * e_s.y;
          put(8 + kp, t1a - t2a, t1b - t2b, t3a + t4a, t3b + t4b);   // centre + d
          put(7 - kp, t1a + t2a, t1b + t2b, t3a - t4a, t3b - t4b);   // centre - d
        }
      }
      ws_group_sync(1);
      // ---- scores at the nodes: s_node[16 x HN] = Fn_t[16 x 2N] * w[2N x HN] -----------------------
      if (nt1 < NT) {
        // consecutive MMAs never share an accumulator: a dependent MMA would wait out the whole latency
        // of the one before it
        float acc[6][4];
#pragma unroll
        for (int c = 0; c < 6; ++c)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[c][e] = 0.f;
#pragma unroll
        for (int i = 0; i < KH; ++i) {
          const int ks = khalf * kh_steps + i;
          if (i < kh_steps && ks < ktot) {
            uint32_t ah[4], al[4];
            const int off = lds_a_row(lane) * fpitch + 16 * ks + lds_a_col(lane);
            ldsm_x4(ah, fh + off);
            ldsm_x4(al, fl + off);
            mma16816<__half>(acc[3 * (i & 1)], ah, bhi[i]);
            mma16816<__half>(acc[3 * (i & 1) + 1], al, bhi[i]);
            mma16816<__half>(acc[3 * (i & 1) + 2], ah, blo[i]);
          }
        }
        float* red = snode32 + khalf * (FD * HN);   // this part's partial sums
        const int col = 8 * nt1 + 2 * tq;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float v = ((acc[0][e] + acc[3][e]) + (acc[1][e] + acc[4][e])) + (acc[2][e] + acc[5][e]);
          red[(gq + 8 * (e >> 1)) * HN + col + (e & 1)] = v;
        }
      }
      ws_group_sync(1);
      {
        __half* sh_ = snode + (buf * 2 + 0) * 32 * 24;
        __half* sl_ = snode + (buf * 2 + 1) * 32 * 24;
        for (int e = tid; e < FD * HN; e += 256) {
          const int k = e / HN, h = e - k * HN;
          __half hi, lo;
          float v = snode32[e];
#pragma unroll
          for (int kp = 1; kp < KP; ++kp) v += snode32[kp * FD * HN + e];
          split_h(v, hi, lo);
          sh_[h * 24 + k] = hi;
          sl_[h * 24 + k] = lo;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(full_sp + fb);
    }
    __syncthreads();
    return;
  }

  // ============================= score warps ======================================================
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(WS_QREG));
  const int qw = wp - 8, nt = qw & 3, half = qw >> 2;
  const bool act = nt < NT;
  const int sq = act ? nt / NTs : 0, ntl = nt - sq * NTs;   // sequence of this column tile, tile within the sequence
  const int bb = b0 + sq;
  const int v_issuer = NT > 1 ? 1 : 0;   // column tile whose warp refills V slots (tile 0's warp refills K slots)
  __half* pw16 = reinterpret_cast<__half*>(smem + L.pw) + qw * 64 * 8;   // this warp's probabilities [64 tokens][8 heads]
  T* pwT = reinterpret_cast<T*>(pw16);
  // column ranges of this warp's heads in the verbatim stores
  int kc0 = 0, kc1 = 0, mtv0 = 0, mtvn = 0;
  if (act) {
    const int g0 = (hb + HPT * ntl) / R, g1 = (min(Hq, hb + HPT * ntl + HPT) - 1) / R;
    kc0 = a.kn_h[g0] & ~15;
    kc1 = (a.kn_h[g1 + 1] + 15) & ~15;
    mtv0 = a.vn_h[g0] >> 4;
    mtvn = ((a.vn_h[g1 + 1] + 15) >> 4) - mtv0;
  }
  const int nks = (kc1 - kc0) >> 4;   // 16-column steps of the verbatim-K contraction
  // the heads' verbatim-K query entries as MMA B fragments (raw model-dtype values; the softmax
  // scale is applied to the fp32 sums)
  uint32_t bq[KS][2];
  {
    const T* q = reinterpret_cast<const T*>(a.q) + (int64_t)bb * a.q_sb;
    const int h = gq < HPT ? hb + HPT * ntl + gq : Hq;   // padding columns: no head
    const int g = h / R;
    int c_lo = 0, c_hi = 0;
    if (act && h < Hq) {
      c_lo = a.kn_h[g];
      c_hi = a.kn_h[g + 1];
    }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int col = kc0 + 16 * ks + 2 * tq + 8 * r;
        T v0 = from_f32<T>(0.f), v1 = from_f32<T>(0.f);
        if (col >= c_lo && col < c_hi) v0 = q[h * D + a.kn_list[col] - g * D];
        if (col + 1 >= c_lo && col + 1 < c_hi) v1 = q[h * D + a.kn_list[col + 1] - g * D];
        bq[ks][r] = pack_pair<T>(v0, v1);
      }
    }
  }
  const int hc0 = 8 * nt + 2 * tq;    // this thread's two columns among the CTA's 32
  const int hl0 = hb + HPT * ntl + 2 * tq;   // ... and the heads of sequence bb they stand for
  const bool hv0 = act && 2 * tq < HPT && hl0 < Hq, hv1 = act && 2 * tq + 1 < HPT && hl0 + 1 < Hq;   // real heads?
  const float cst0 = hv0 ? p.cst[(int64_t)bb * Hq + hl0] : 0.f;
  const float cst1 = hv1 ? p.cst[(int64_t)bb * Hq + hl0 + 1] : 0.f;
  // first column of this sequence's boxes inside a K / V ring slot
  const int cbK = sq * nbK * 64 - colK0, cbV = sq * nbV * 64 - colV0;   // absolute column -> column inside a ring slot
  float m_run0 = NEG_BIG, m_run1 = NEG_BIG, lsum0 = 0.f, lsum1 = 0.f;
  float Gacc[GI][GN][4];
#pragma unroll
  for (int i = 0; i < GI; ++i)
#pragma unroll
    for (int n = 0; n < GN; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) Gacc[i][n][e] = 0.f;
  float Oacc[MTV][4];
#pragma unroll
  for (int i = 0; i < MTV; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) Oacc[i][e] = 0.f;

  for (int st = 0; st < nst; ++st) {
    const int buf = st & 1, fb = st % NB;
    const int tok0 = l0 + st * J + half * FH;   // first token of this warp's half
    const __half* fh = fnt + (fb * 2 + 0) * FD * fpitch;
    const __half* fl = fnt + (fb * 2 + 1) * FD * fpitch;
    float sc[4][4];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[mt][e] = 0.f;
    const int iK = 4 * st + half, sK = iK % 3;
    const uint32_t parK = (uint32_t)(iK / 3) & 1u;
    // Every run of MMAs below visits four different accumulators in turn: a dependent MMA issued right
    // after its predecessor would wait out that one's whole latency.
    if (act) {
      // ---- verbatim-dim scores from the K rows (needs only the K tile, so it comes first) -----------
      mbar_wait(full_slot + sK, parK, dead, p.err);
      const unsigned char* ks_ = slots + sK * L.slot_bytes;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        if (ks < nks) {
#pragma unroll
          for (int mt = 0; mt < 4; ++mt) {
            uint32_t af[4];
            ldsm_x4(af, ks_ + sw_off(16 * mt + lds_a_row(lane), (cbK + kc0 + 16 * ks + lds_a_col(lane)) >> 3));
            mma16816<T>(sc[mt], af, bq[ks]);
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
    }
    if (nt == 0) {   // refill the slot once every warp of this half has released it
      mbar_wait(empty_slot + sK, parK, dead, p.err);
      issue_tile(iK + 3);
    }
    mbar_wait(full_sp + fb, (st / NB) & 1, dead, p.err);
    if (act) {
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
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t ah[4];
        ldsm_x4(ah, interp_hi + ioff + 16 * mt * 24);
        mma16816<__half>(sc[mt], ah, bl);
      }
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t ah[4];
        ldsm_x4(ah, interp_hi + ioff + 16 * mt * 24);
        mma16816<__half>(sc[mt], ah, bh);
      }
    }
    // ---- softmax over the 128 tokens of the super-tile (both halves agree on the maximum) ----------
    float al0 = 1.f, al1 = 1.f;
    __half2 ph[4][2];   // probabilities rounded to fp16: (head 2tq, 2tq+1) of token rows gq and gq+8 per 16-token tile
    float pt_acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int iV = 4 * st + 2 + half, sV = iV % 3;
    const uint32_t parV = (uint32_t)(iV / 3) & 1u;
    if (act) {
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
      if (gq == 0) {
        mx[(nt * 2 + half) * 8 + 2 * tq] = mx0;
        mx[(nt * 2 + half) * 8 + 2 * tq + 1] = mx1;
      }
      ws_pair_sync(2 + nt);
      const float mn0 = fmaxf(m_run0, fmaxf(mx0, mx[(nt * 2 + (half ^ 1)) * 8 + 2 * tq]));
      const float mn1 = fmaxf(m_run1, fmaxf(mx1, mx[(nt * 2 + (half ^ 1)) * 8 + 2 * tq + 1]));
      al0 = exp2f(m_run0 - mn0);
      al1 = exp2f(m_run1 - mn1);
      m_run0 = mn0;
      m_run1 = mn1;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        const bool ok0 = (tok0 + 16 * mt + gq) < l1, ok1 = (tok0 + 16 * mt + gq + 8) < l1;
        ph[mt][0] = __floats2half2_rn(ok0 ? exp2f(sc[mt][0] - mn0) : 0.f, ok0 ? exp2f(sc[mt][1] - mn1) : 0.f);
        ph[mt][1] = __floats2half2_rn(ok1 ? exp2f(sc[mt][2] - mn0) : 0.f, ok1 ? exp2f(sc[mt][3] - mn1) : 0.f);
        // token-major [token][8 heads]: a thread's two heads are one 32-bit store, the B operands come back
        // through ldmatrix.trans; the sums use the rounded values
        const int j0 = 16 * mt + gq;
        *reinterpret_cast<__half2*>(pw16 + j0 * 8 + 2 * tq) = ph[mt][0];
        *reinterpret_cast<__half2*>(pw16 + (j0 + 8) * 8 + 2 * tq) = ph[mt][1];
        const float2 f0 = __half22float2(ph[mt][0]), f1 = __half22float2(ph[mt][1]);
        s0 += f0.x + f1.x;
        s1 += f0.y + f1.y;
      }
      lsum0 = lsum0 * al0 + s0;   // this thread's rows only; the lanes are added at the end
      lsum1 = lsum1 * al1 + s1;
      __syncwarp();
      // ---- project the probabilities onto the nodes: pt[16 x 8] = Interp^T[16 x 64] * P[64 x 8] ------
      uint32_t bp[4][2];
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) ldsm_x2_t(bp[ks], pw16 + (16 * ks + (lane & 15)) * 8);
      {
        float pt2[3][4];
#pragma unroll
        for (int c = 0; c < 3; ++c)
#pragma unroll
          for (int e = 0; e < 4; ++e) pt2[c][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          uint32_t af[4], al_[4];
          const int ioff = (half * FH + 16 * ks + lds_at_row(lane)) * 24 + lds_at_col(lane);
          ldsm_x4_t(af, interp_hi + ioff);
          ldsm_x4_t(al_, interp_lo + ioff);
          if (ks & 1) {
            mma16816<__half>(pt2[0], af, bp[ks]);
            mma16816<__half>(pt2[1], al_, bp[ks]);
          } else {
            mma16816<__half>(pt_acc, af, bp[ks]);
            mma16816<__half>(pt2[2], al_, bp[ks]);
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) pt_acc[e] = (pt_acc[e] + pt2[0][e]) + (pt2[1][e] + pt2[2][e]);
      }
      // ---- verbatim-V numerators -------------------------------------------------------------------
      uint32_t bp_lo[4][2];
      if constexpr (kBf16) {
        // an fp16 value splits exactly into two bf16 values, so the verbatim-V GEMM (model dtype)
        // sees the same probabilities as the spectral side and the denominator
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
            *reinterpret_cast<T2*>(pwT + (16 * mt + gq + 8 * r) * 8 + 2 * tq) =
                __floats2bfloat162_rn(res[mt][r].x, res[mt][r].y);
        __syncwarp();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) ldsm_x2_t(bp_lo[ks], pwT + (16 * ks + (lane & 15)) * 8);
      }
      mbar_wait(full_slot + sV, parV, dead, p.err);
      const unsigned char* vs_ = slots + sV * L.slot_bytes;
#pragma unroll
      for (int i = 0; i < MTV; ++i) {
        Oacc[i][0] *= al0;
        Oacc[i][1] *= al1;
        Oacc[i][2] *= al0;
        Oacc[i][3] *= al1;
      }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
        for (int i0 = 0; i0 < MTV; i0 += 4) {   // four V tiles at a time: their fragments are in flight together
          uint32_t af[4][4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (i0 + i < mtvn)
              ldsm_x4_t(af[i], vs_ + sw_off(16 * ks + lds_at_row(lane), (cbV + 16 * (mtv0 + i0 + i) + lds_at_col(lane)) >> 3));
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (i0 + i < mtvn) mma16816<T>(Oacc[i0 + i], af[i], bp[ks]);
          if (kBf16) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (i0 + i < mtvn) mma16816<T>(Oacc[i0 + i], af[i], bp_lo[ks]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_slot + sV);
    }
    if (nt == v_issuer) {
      mbar_wait(empty_slot + sV, parV, dead, p.err);
      issue_tile(iV + 3);
    }
    // ---- hand the node-projected probabilities of the column tile to every score warp -------------
    if (act) {
      if (half == 1) {
#pragma unroll
        for (int e = 0; e < 4; ++e) ptp[nt * FD * 8 + (gq + 8 * (e >> 1)) * 8 + 2 * tq + (e & 1)] = pt_acc[e];
      }
      ws_pair_sync(2 + nt);
      if (half == 0) {
        __half* ph_ = ptx + (buf * 2 + 0) * 32 * 24;
        __half* pl_ = ptx + (buf * 2 + 1) * 32 * 24;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float v = pt_acc[e] + ptp[nt * FD * 8 + (gq + 8 * (e >> 1)) * 8 + 2 * tq + (e & 1)];
          __half hi, lo;
          split_h(v, hi, lo);
          const int o = (hc0 + (e & 1)) * 24 + gq + 8 * (e >> 1);
          ph_[o] = hi;
          pl_[o] = lo;
        }
        if (gq == 0) {
          alpha[buf * 32 + hc0] = al0;
          alpha[buf * 32 + hc0 + 1] = al1;
        }
      }
    }
    ws_group_sync(7);
    // ---- g[2N x HN] += Fn_t^T[2N x 16] * pt[16 x HN]  (this warp's 16-row tiles) -------------------
    {
      uint32_t bf[GN][2], bl[GN][2];
      float ap[GN][2];
#pragma unroll
      for (int n = 0; n < GN; ++n) {
        if (n < NT) {
          const int o = (8 * n + lds_b_row(lane)) * 24 + lds_b_col(lane);
          ldsm_x2(bf[n], ptx + (buf * 2 + 0) * 32 * 24 + o);
          ldsm_x2(bl[n], ptx + (buf * 2 + 1) * 32 * 24 + o);
          ap[n][0] = alpha[buf * 32 + 8 * n + 2 * tq];
          ap[n][1] = alpha[buf * 32 + 8 * n + 2 * tq + 1];
        }
      }
#pragma unroll
      for (int i = 0; i < GI; ++i) {
        const int mt = qw + 8 * i;
        if (mt < ktot) {
          uint32_t ah[4], al_[4];
          const int off = lds_at_row(lane) * fpitch + 16 * mt + lds_at_col(lane);
          ldsm_x4_t(ah, fh + off);
          ldsm_x4_t(al_, fl + off);
#pragma unroll
          for (int n = 0; n < GN; ++n) {
            if (n < NT) {
              Gacc[i][n][0] *= ap[n][0];
              Gacc[i][n][1] *= ap[n][1];
              Gacc[i][n][2] *= ap[n][0];
              Gacc[i][n][3] *= ap[n][1];
            }
          }
#pragma unroll
          for (int n = 0; n < GN; ++n)
            if (n < NT) mma16816<__half>(Gacc[i][n], al_, bf[n]);
#pragma unroll
          for (int n = 0; n < GN; ++n)
            if (n < NT) mma16816<__half>(Gacc[i][n], ah, bl[n]);
#pragma unroll
          for (int n = 0; n < GN; ++n)
            if (n < NT) mma16816<__half>(Gacc[i][n], ah, bf[n]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_sp + fb);
  }

  // ---- chunk partials ---------------------------------------------------------------------------
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    lsum0 += __shfl_xor_sync(0xffffffffu, lsum0, o);
    lsum1 += __shfl_xor_sync(0xffffffffu, lsum1, o);
  }
  if (act && half == 1 && gq == 0) {
    lx[nt * 8 + 2 * tq] = lsum0;
    lx[nt * 8 + 2 * tq + 1] = lsum1;
  }
  __syncthreads();   // the spectral warps have zeroed this chunk's verbatim-V partial
  if (act && half == 0 && gq == 0) {
    const int64_t slot_id = slot_of(bb);
    if (hv0) {
      p.m_part[slot_id * Hq + hl0] = m_run0;
      p.l_part[slot_id * Hq + hl0] = lsum0 + lx[nt * 8 + 2 * tq];
    }
    if (hv1) {
      p.m_part[slot_id * Hq + hl0 + 1] = m_run1;
      p.l_part[slot_id * Hq + hl0 + 1] = lsum1 + lx[nt * 8 + 2 * tq + 1];
    }
  }
  if (act) {
    // both halves add their numerators (two addends onto zero: the order does not change the sum)
    float* ob = p.o_part + slot_of(bb) * Hq * D;
#pragma unroll
    for (int i = 0; i < MTV; ++i) {
      if (i < mtvn) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c = 16 * (mtv0 + i) + gq + 8 * (e >> 1);
          const int h = hl0 + (e & 1);
          if (c < Mn_v && ((e & 1) ? hv1 : hv0)) {
            const int g = h / R;
            if (c >= a.vn_h[g] && c < a.vn_h[g + 1]) atomicAdd(ob + h * D + a.vn_list[c] - g * D, Oacc[i][e]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < GI; ++i) {
    const int mt = qw + 8 * i;
    if (mt < ktot) {
#pragma unroll
      for (int n = 0; n < GN; ++n) {
        if (n < NT) {
          const int sqn = n / NTs, ntn = n - sqn * NTs;   // sequence and tile-within-sequence of column tile n
          float* gb = p.g_part + (((int64_t)(b0 + sqn) * p.n_mid_chunks + chunk) * Hq) * 2 * N;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = 16 * mt + gq + 8 * (e >> 1);
            const int h = hb + HPT * ntn + 2 * tq + (e & 1);
            if (row < 2 * N && 2 * tq + (e & 1) < HPT && h < Hq) gb[(int64_t)h * 2 * N + row] = Gacc[i][n][e];
          }
        }
      }
    }
  }
}

