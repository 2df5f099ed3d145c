// Sinks + window rows on tensor cores, for the 512-thread main kernels.  Included by decode.cu after
// decode_fast.cuh (same namespace, same ldmatrix / mma / mbarrier / TMA helpers).
//
// The rows are walked in tiles of TR rows: first the tiles of the sink rows, then the tiles of the
// window rows (a tile never mixes the two tensors; its missing rows read as zeros and are masked).
// Per tile and KV head g the scores are one GEMM S[TR x 8] = K_g[TR x D] * Q_g[D x 8] (the R query
// heads of g padded to 8 columns, raw model-dtype values; the softmax scale is applied to the fp32
// sums) and the numerators one GEMM O_g^T[D x 8] += V_g^T[D x TR] * P_g[TR x 8], both as m16n8k16
// MMAs.  One warp owns all rows of a tile for one KV head, so the online softmax never leaves the
// warp; the probabilities are rounded once to fp16 and, for bf16 caches, split exactly into two bf16
// values, as in the middle-span pass.  K and V tiles arrive as TMA boxes (64 columns x TR rows,
// 128-byte swizzle) in a three-stage ring, each stage completing on its own mbarrier (bounded waits).
#pragma once

constexpr int IL_T = 512;      // threads of the CTA
constexpr int IL_W = IL_T / 32;
constexpr int IL_U = 8;        // (KV head, 16-dim tile) units of the numerators per warp: Hkv * D / 16 <= 16 * IL_U
constexpr int IL_STAGES = 3;
constexpr int IL_MT = 8;       // 16-row tiles per tile of rows (TR <= 128)

struct IlSmem {
  int ring, qb, pm, pl, m_run, l_run, alpha, bars, total;
  int qpitch, ppitch, HP, box_bytes, nbF, stage_bytes;
};
__host__ __device__ inline IlSmem il_mma_smem(int TR, int F, int Hkv, int D, bool two_p) {
  IlSmem s;
  int o = 0;
  auto take = [&](int bytes) {
    int r = o;
    o += (bytes + 15) / 16 * 16;
    return r;
  };
  s.qpitch = D + 8;
  s.ppitch = TR + 8;
  s.HP = Hkv * 8;
  s.box_bytes = 128 * TR;                       // 64 columns x TR rows of 16-bit values
  s.nbF = (F + 63) / 64;
  s.stage_bytes = 2 * s.nbF * s.box_bytes;      // K boxes, then V boxes
  s.ring = take(IL_STAGES * s.stage_bytes);     // first: keeps the 1024-byte alignment of the swizzle
  s.qb = take(s.HP * s.qpitch * 2);
  s.pm = take(s.HP * s.ppitch * 2);
  s.pl = two_p ? take(s.HP * s.ppitch * 2) : s.pm;
  s.m_run = take(s.HP * 4);
  s.l_run = take(s.HP * 4);
  s.alpha = take(s.HP * 4);
  s.bars = take(8 * 8);
  s.total = o;
  return s;
}

// barrier of the pass's 512 threads (a CTA may carry more warps than the pass uses)
__device__ __forceinline__ void il_sync() { asm volatile("bar.sync 1, 512;\n" ::: "memory"); }

// byte offset of the 16-byte chunk (row r, columns 8*chunk ..) inside one tensor's part of a stage
__device__ __forceinline__ int il_sw(int r, int chunk, int box_bytes) {
  return (chunk >> 3) * box_bytes + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
}


// scores + softmax of one KV head over all rows of a tile, by one warp (defined below); MT = 16-row tiles the
// code is unrolled for (a tile of rows has at most 16 * MT rows)
template <typename T, int MT>
__device__ __forceinline__ void il_scores_softmax(const unsigned char* ks, const T* qb, T* pm, T* pl, float* m_run,
                                                  float* l_run, float* alpha, int g, int D, int mtiles, int valid,
                                                  int qpitch, int ppitch, int box_bytes, float c2, int lane);

template <typename T, int MT = IL_MT>
__device__ void il_chunk_mma(const DecodeParams& p, int b, int chunk, unsigned char* smem) {
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  const fa_decode_args_t& a = p.a;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const int F = p.F, D = a.D, Hq = a.Hq, Hkv = a.Hkv, R = p.R, TR = p.TRm;
  const IlSmem L = il_mma_smem(TR, F, Hkv, D, kBf16);
  const int qpitch = L.qpitch, ppitch = L.ppitch, HP = L.HP, box_bytes = L.box_bytes;
  unsigned char* ring = smem + L.ring;
  T* qb = reinterpret_cast<T*>(smem + L.qb);
  T* pm = reinterpret_cast<T*>(smem + L.pm);
  T* pl = reinterpret_cast<T*>(smem + L.pl);
  float* m_run = reinterpret_cast<float*>(smem + L.m_run);
  float* l_run = reinterpret_cast<float*>(smem + L.l_run);
  float* alpha = reinterpret_cast<float*>(smem + L.alpha);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);   // [IL_STAGES]
  volatile int* dead = reinterpret_cast<volatile int*>(full + IL_STAGES);

  // this chunk's tiles in the list [sink tiles | window tiles]
  const int n_st = (a.n_sink + TR - 1) / TR;
  const int n_all = n_st + (a.n_win + TR - 1) / TR;
  const int t0 = chunk * p.il_tpc;
  const int nt = min(n_all, t0 + p.il_tpc) - t0;

  if (tid == 0) {
    for (int i = 0; i < IL_STAGES; ++i) mbar_init(full + i, 1);
    *dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  il_sync();
  // called by a whole warp: request tile t (chunk-relative) into its ring stage
  auto issue = [&](int t) {
    if (t >= nt) return;
    const int s = t % IL_STAGES;
    const int gt = t0 + t;
    const bool sink = gt < n_st;
    const int row = (sink ? p.sink_row0 + gt * TR : p.win_row0 + (gt - n_st) * TR);
    const CUtensorMap* mk = sink ? &p.tm_ks : &p.tm_kw;
    const CUtensorMap* mv = sink ? &p.tm_vs : &p.tm_vw;
    if (lane == 0) mbar_expect_tx(full + s, (uint32_t)L.stage_bytes);
    __syncwarp();
    unsigned char* dst = ring + s * L.stage_bytes;
    for (int i = lane; i < 2 * L.nbF; i += 32) {
      const bool is_v = i >= L.nbF;
      const int bx = is_v ? i - L.nbF : i;
      tma_box(dst + i * box_bytes, is_v ? mv : mk, 64 * bx, row, b, full + s);
    }
  };
  if (warp == IL_W - 1) {
    issue(0);
    issue(1);
  }

  // query rows of KV head g at rows 8g .. 8g+R-1, zero rows above; probabilities start as zeros
  const T* q = reinterpret_cast<const T*>(a.q) + (int64_t)b * a.q_sb;
  for (int e = tid; e < HP * D; e += IL_T) {
    const int hp = e / D, d = e - hp * D;
    const int g = hp >> 3, r = hp & 7;
    qb[hp * qpitch + d] = (r < R) ? q[(g * R + r) * D + d] : from_f32<T>(0.f);
  }
  for (int e = tid; e < HP * ppitch; e += IL_T) {
    pm[e] = from_f32<T>(0.f);
    if (kBf16) pl[e] = from_f32<T>(0.f);
  }
  for (int h = tid; h < HP; h += IL_T) {
    m_run[h] = NEG_BIG;
    l_run[h] = 0.f;
    alpha[h] = 1.f;
  }
  const int mtiles = TR / 16;            // 16-row tiles of a tile of rows
  const int dtiles = D / 16;             // 16-dim tiles of a head
  const int n_units = Hkv * dtiles;      // numerator units (KV head, dim tile)
  int ug[IL_U], umt[IL_U];               // this warp's numerator units
  float Oacc[IL_U][4];
#pragma unroll
  for (int i = 0; i < IL_U; ++i) {
    const int u = warp + IL_W * i;
    ug[i] = u < n_units ? u / dtiles : -1;
    umt[i] = u < n_units ? u - ug[i] * dtiles : 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) Oacc[i][e] = 0.f;
  }

  for (int t = 0; t < nt; ++t) {
    const int s = t % IL_STAGES;
    const int gt = t0 + t;
    const bool sink = gt < n_st;
    const int row0 = (sink ? gt : gt - n_st) * TR;
    const int valid = min(TR, (sink ? a.n_sink : a.n_win) - row0);
    mbar_wait(full + s, (uint32_t)(t / IL_STAGES) & 1u, dead, p.err);
    il_sync();   // everyone is done with tile t-1: its stage, the probabilities and alpha are free
    if (warp == IL_W - 1) issue(t + 2);
    const unsigned char* ks = ring + s * L.stage_bytes;
    const unsigned char* vs = ks + L.nbF * box_bytes;
    for (int g = warp; g < Hkv; g += IL_W)
      il_scores_softmax<T, MT>(ks, qb, pm, pl, m_run, l_run, alpha, g, D, mtiles, valid, qpitch, ppitch, box_bytes,
                               p.c2, lane);
    il_sync();
    // ---- numerators: unit = (KV head, 16-dim tile) --------------------------------------------------
#pragma unroll
    for (int i = 0; i < IL_U; ++i) {
      if (ug[i] >= 0) {
        const int g = ug[i], mt = umt[i];
        const float a0 = alpha[8 * g + 2 * tq], a1 = alpha[8 * g + 2 * tq + 1];
        Oacc[i][0] *= a0;
        Oacc[i][1] *= a1;
        Oacc[i][2] *= a0;
        Oacc[i][3] *= a1;
        for (int k = 0; k < mtiles; ++k) {
          uint32_t af[4], bf[2];
          ldsm_x4_t(af, vs + il_sw(16 * k + lds_at_row(lane), (g * D + 16 * mt + lds_at_col(lane)) >> 3, box_bytes));
          ldsm_x2(bf, pm + (8 * g + lds_b_row(lane)) * ppitch + 16 * k + lds_b_col(lane));
          mma16816<T>(Oacc[i], af, bf);
          if (kBf16) {
            ldsm_x2(bf, pl + (8 * g + lds_b_row(lane)) * ppitch + 16 * k + lds_b_col(lane));
            mma16816<T>(Oacc[i], af, bf);
          }
        }
      }
    }
  }
  il_sync();

  const int64_t slot = (int64_t)b * p.NCH + chunk;
  for (int h = tid; h < Hq; h += IL_T) {
    const int hp = (h / R) * 8 + (h % R);
    p.m_part[slot * Hq + h] = m_run[hp];
    p.l_part[slot * Hq + h] = l_run[hp];
  }
#pragma unroll
  for (int i = 0; i < IL_U; ++i) {
    if (ug[i] >= 0) {
      const int g = ug[i], mt = umt[i];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = 2 * tq + (e & 1), d = 16 * mt + gq + 8 * (e >> 1);
        if (r < R) p.o_part[(slot * Hq + g * R + r) * D + d] = Oacc[i][e];
      }
    }
  }
}

template <typename T, int MT>
__device__ __forceinline__ void il_scores_softmax(const unsigned char* ks, const T* qb, T* pm, T* pl, float* m_run,
                                                  float* l_run, float* alpha, int g, int D, int mtiles, int valid,
                                                  int qpitch, int ppitch, int box_bytes, float c2, int lane) {
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  const int gq = lane >> 2, tq = lane & 3;
  const int dtiles = D / 16;
  float sc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    if (mt < mtiles) {
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      for (int k = 0; k < dtiles; k += 2) {   // two 16-dim steps at a time, two accumulators
        uint32_t af0[4], af1[4], bf0[2], bf1[2];
        const int c0 = g * D + 16 * k + lds_a_col(lane);
        const bool two = k + 1 < dtiles;
        ldsm_x4(af0, ks + il_sw(16 * mt + lds_a_row(lane), c0 >> 3, box_bytes));
        ldsm_x2(bf0, qb + (8 * g + lds_b_row(lane)) * qpitch + 16 * k + lds_b_col(lane));
        if (two) {
          ldsm_x4(af1, ks + il_sw(16 * mt + lds_a_row(lane), (c0 + 16) >> 3, box_bytes));
          ldsm_x2(bf1, qb + (8 * g + lds_b_row(lane)) * qpitch + 16 * k + 16 + lds_b_col(lane));
        }
        mma16816<T>(acc[0], af0, bf0);
        if (two) mma16816<T>(acc[1], af1, bf1);
      }
      const bool ok0 = 16 * mt + gq < valid, ok1 = 16 * mt + gq + 8 < valid;
      sc[mt][0] = ok0 ? (acc[0][0] + acc[1][0]) * c2 : NEG_BIG;
      sc[mt][1] = ok0 ? (acc[0][1] + acc[1][1]) * c2 : NEG_BIG;
      sc[mt][2] = ok1 ? (acc[0][2] + acc[1][2]) * c2 : NEG_BIG;
      sc[mt][3] = ok1 ? (acc[0][3] + acc[1][3]) * c2 : NEG_BIG;
    }
  }
  float mx0 = NEG_BIG, mx1 = NEG_BIG;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    if (mt < mtiles) {
      mx0 = fmaxf(mx0, fmaxf(sc[mt][0], sc[mt][2]));
      mx1 = fmaxf(mx1, fmaxf(sc[mt][1], sc[mt][3]));
    }
  }
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
  }
  const int hp0 = 8 * g + 2 * tq;
  const float mo0 = m_run[hp0], mo1 = m_run[hp0 + 1];
  const float mn0 = fmaxf(mo0, mx0), mn1 = fmaxf(mo1, mx1);
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    if (mt < mtiles) {
      const bool ok0 = 16 * mt + gq < valid, ok1 = 16 * mt + gq + 8 < valid;
      const float f0 = ok0 ? __half2float(__float2half_rn(exp2f(sc[mt][0] - mn0))) : 0.f;
      const float f1 = ok0 ? __half2float(__float2half_rn(exp2f(sc[mt][1] - mn1))) : 0.f;
      const float f2 = ok1 ? __half2float(__float2half_rn(exp2f(sc[mt][2] - mn0))) : 0.f;
      const float f3 = ok1 ? __half2float(__float2half_rn(exp2f(sc[mt][3] - mn1))) : 0.f;
      s0 += f0 + f2;   // the denominator uses the rounded values, like the numerators
      s1 += f1 + f3;
      const int j0 = 16 * mt + gq;
      T* r0p = pm + hp0 * ppitch + j0;
      T* r1p = r0p + ppitch;
      const T h0 = from_f32<T>(f0), h1 = from_f32<T>(f1), h2 = from_f32<T>(f2), h3 = from_f32<T>(f3);
      r0p[0] = h0;
      r1p[0] = h1;
      r0p[8] = h2;
      r1p[8] = h3;
      if (kBf16) {
        T* q0p = pl + hp0 * ppitch + j0;
        T* q1p = q0p + ppitch;
        q0p[0] = from_f32<T>(f0 - to_f32(h0));
        q1p[0] = from_f32<T>(f1 - to_f32(h1));
        q0p[8] = from_f32<T>(f2 - to_f32(h2));
        q1p[8] = from_f32<T>(f3 - to_f32(h3));
      }
    }
  }
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    s0 += __shfl_xor_sync(0xffffffffu, s0, o);
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
  }
  __syncwarp();
  if (gq == 0) {
    const float al0 = exp2f(mo0 - mn0), al1 = exp2f(mo1 - mn1);
    alpha[hp0] = al0;
    alpha[hp0 + 1] = al1;
    l_run[hp0] = l_run[hp0] * al0 + s0;
    l_run[hp0 + 1] = l_run[hp0 + 1] * al1 + s1;
    m_run[hp0] = mn0;
    m_run[hp0 + 1] = mn1;
  }
}
