// Channel-wise gate (one log decay per token, head and key channel): the `prepare` kernel.
//
// With a per-channel decay the ratio exp(G_i,d - G_s,d) sits inside the contraction over d, so
// M[i,s] = beta_i sum_d k[i,d] k[s,d] exp(G_i,d - G_s,d) and A[i,s] are not plain Gram products
// (reference: gdn2_chunkwise_cw.py:155-157,168-169).  Splitting the ratio as exp(G_i - G_ref) *
// exp(G_ref - G_s) is only safe when both exponents are <= 0, i.e. when s <= ref <= i.  The 64-token
// chunk is therefore cut into four blocks of 16 rows:
//   * row block I against earlier blocks (s < 16 I): reference row a_I = 16 I.  Left operand rows
//     x[i] exp(G_i - G_{a_I}) (one tile serves all I: blocks are disjoint row ranges), right operand
//     rows k[s] exp(G_{a_I} - G_s) for s < 16 I (three row ranges packed into one tile).  Three
//     tcgen05 products with N = 16, 32, 48.
//   * the four diagonal 16 x 16 blocks: exact per-pair exponentials on the CUDA cores, while the
//     products run.
// Everything after M and A (inverse, WY factors, state map) is the scalar-gate kernel's, with
// per-channel decays in the operand scalings.
#include "gdn_common.cuh"
#include "host_util.h"

namespace lg {

constexpr int kMsC = 68;
constexpr int kPrepCwThreads = 256;
constexpr int kDg = 17;                               // row stride (floats) of the diagonal-block buffers
constexpr int kGateSegs = kPrepCwThreads / 128;       // row segments of the cumulative sum (thread = segment x channel)
constexpr int kGateRows = kC / kGateSegs;

template <int V, bool DELTA>
__global__ void __launch_bounds__(kPrepCwThreads)
prepare_cw_kernel(const Problem p, const __grid_constant__ CUtensorMap mq,
                  const __grid_constant__ CUtensorMap mk, const __grid_constant__ CUtensorMap mv) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = align1024(smem_raw);
  unsigned char* KQ = sm;                      // 32 KB: rows 0-63 k, 64-127 q (fp16); later M (fp32), then [w | u]
  unsigned char* LA = KQ + 32768;              // 32 KB: rows 0-63 k exp(G_i - G_a), rows 64-127 q exp(G_i - G_a)
  unsigned char* KR = LA + 32768;              // 32 KB: rows [0,16) [16,48) [48,96): k exp(G_{a_I} - G_s), I = 1, 2, 3
  float* Gt = reinterpret_cast<float*>(KR + 32768);   // 32 KB: cumulative log decay [64][128]
  unsigned char* BGK = reinterpret_cast<unsigned char*>(Gt) + 32768;   // 16 KB
  unsigned char* BV = BGK + 16384;             // V*128
  unsigned char* KD = BV + V * 128;            // 16 KB
  unsigned char* TA = KD + 16384;              // 16 KB
  float* fs = reinterpret_cast<float*>(TA + 16384);
  // diagonal blocks of A and of M, [64][16] with rows kDg floats apart: an odd stride keeps both the epilogue's
  // reads (thread r reads row r) and the diagonal phase's stores off each other's banks
  float* Adg = fs;
  float* Mdg = fs + 64 * kDg;
  float* betas = fs + 128 * kDg;     // [64]
  CtaShared* cs = reinterpret_cast<CtaShared*>(fs + 128 * kDg + 64);
  float* Msm = reinterpret_cast<float*>(KQ);
  unsigned char* WU = KQ;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int bh = p.bh0 + blockIdx.x / p.cn, c = p.c0 + blockIdx.x % p.cn, z = bh * p.NT + c, b = bh / p.H, h = bh % p.H;
  CtaCtl ctl{p.status, &cs->abort_flag};
  uint64_t* bar_load = &cs->bar[0];
  uint64_t* bar_mma = &cs->bar[1];
  // Everything that has to come from global memory is requested first - the tensor-map loads of k, q, v by
  // the thread that has just initialised their barrier, the gate values and beta by every thread - so that
  // the one memory latency of the chunk overlaps the tensor-memory allocation and the first barrier.
  if (tid == 0) {
    cs->abort_flag = 0;
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    fence_mbar_init();
    fence_proxy_async();
    mbar_expect_tx(bar_load, 32768u + V * 128u);
    for (int a = 0; a < 2; ++a) {
      tma_load_4d(KQ + a * 16384, &mk, bar_load, a * 64, h, c * kC, b);
      tma_load_4d(KQ + a * 16384 + 8192, &mq, bar_load, a * 64, h, c * kC, b);
    }
    for (int a = 0; a < V / 64; ++a) tma_load_4d(BV + a * 8192, &mv, bar_load, a * 64, h, c * kC, b);
  }
  const size_t tok0 = (static_cast<size_t>(b) * p.L + c * kC) * p.H + h;
  const int seg = tid >> 7;
  float x[kGateRows];
#pragma unroll
  for (int i = 0; i < kGateRows; ++i)
    x[i] = p.g[(tok0 + static_cast<size_t>(seg * kGateRows + i) * p.H) * kK + (tid & 127)];
  // full op (per-channel erase gate b, write gate w): the gates enter the operand tiles element by
  // element and the per-row beta is one
  const bool full = p.bch != nullptr;
  float beta_r = 1.f;
  if (DELTA && tid < 64 && !full) beta_r = p.beta[tok0 + static_cast<size_t>(tid) * p.H];
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, 256);
    tmem_relinquish();
  }
  if (DELTA && tid < 64) betas[tid] = beta_r;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;
  {
    // cumulative decay: thread (segment of rows, channel) sums its rows, the segment totals are exchanged
    // through shared memory (Adg is free until the diagonal blocks), every thread adds the totals of the
    // segments before its own and writes its entries once, in log2 units
    const int d = tid & 127;
#pragma unroll
    for (int i = 1; i < kGateRows; ++i) x[i] += x[i - 1];
    Adg[seg * kK + d] = x[kGateRows - 1];
    __syncthreads();
    float base = 0.f;
    for (int s2 = 0; s2 < seg; ++s2) base += Adg[s2 * kK + d];
#pragma unroll
    for (int i = 0; i < kGateRows; ++i) Gt[gidx(seg * kGateRows + i, d)] = (base + x[i]) * kLog2e;
    if (seg == kGateSegs - 1)
      reinterpret_cast<float*>(p.saved + p.lay.ad)[static_cast<size_t>(z) * kK + d] = __expf(base + x[kGateRows - 1]);
    fence_proxy_async();
  }
  __syncthreads();

  if (tid == 0) {   // the gate tile becomes a record: later kernels load it instead of rebuilding it
    bulk_s2g(p.saved + p.lay.gt + static_cast<size_t>(z) * (kC * kK * 4), Gt, 32768);
    bulk_commit();
  }
  // ---- operand tiles
  mbar_wait_warp(bar_load, 0, ctl, 501);
  for (int idx = tid; idx < 64 * 16; idx += kPrepCwThreads) {
    const int r = idx >> 4, ch = idx & 15, d0 = ch * 8;
    const int blk = r >> 4;
    float kx[8], qx[8], y[8], gr[8], ga[8], gl[8];
    unpack8_in(tile_ld_chunk(KQ, r, ch, 128), kx, p.qk16);
    unpack8_in(tile_ld_chunk(KQ, 64 + r, ch, 128), qx, p.qk16);
    tile_st_chunk(KQ, r, ch, 128, pack8_f16(kx));
    tile_st_chunk(KQ, 64 + r, ch, 128, pack8_f16(qx));
    gt8(Gt, r, d0, gr);
    gt8(Gt, blk * 16, d0, ga);
    gt8(Gt, 63, d0, gl);
    float ea[8], bb[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) ea[e] = exp2f(gr[e] - ga[e]);
    if (DELTA && full) {
      ld8(p.bch + (tok0 + static_cast<size_t>(r) * p.H) * kK + d0, bb);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = kx[e] * bb[e] * ea[e];     // left factor of M is b k
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = kx[e] * ea[e];
    }
    tile_st_chunk(LA, r, ch, 128, pack8_f16(y));
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = qx[e] * ea[e];
    tile_st_chunk(LA, 64 + r, ch, 128, pack8_f16(y));
    // scale * gamma * q for the output kernel and the adjoint scan's input kernel, staged in the [T; A] tile
    // (not written before the first epilogue) and stored as a record
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = qx[e] * (p.scale * exp2f(gr[e]));
    tile_st_chunk(TA, r, ch, 64, pack8_f16(y));
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = kx[e] * exp2f(gl[e] - gr[e]);
    tile_st_chunk(KD, r, ch, 64, pack8_f16(y));
    if (DELTA) {
      if (!full) {
        const float be = betas[r];
#pragma unroll
        for (int e = 0; e < 8; ++e) bb[e] = be;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = kx[e] * bb[e] * exp2f(gr[e]);
      tile_st_chunk(BGK, r, ch, 64, pack8_f16(y));
    }
    for (int I = blk + 1; I < 4; ++I) {     // row r is a source row for every later row block I
      const int off = (I == 1) ? 0 : (I == 2 ? 16 : 48);
      gt8(Gt, I * 16, d0, ga);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = kx[e] * exp2f(ga[e] - gr[e]);
      tile_st_chunk(KR, off + r, ch, 128, pack8_f16(y));
    }
  }
  for (int idx = tid; idx < 64 * (V / 8); idx += kPrepCwThreads) {
    const int r = idx / (V / 8), ch = idx % (V / 8);
    float x[8];
    unpack8_bf16(tile_ld_chunk(BV, r, ch, 64), x);
    if (DELTA && full) {
      float wv[8];
      ld8(p.wch + (tok0 + static_cast<size_t>(r) * p.H) * V + ch * 8, wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] *= wv[i];
    } else {
      const float be = DELTA ? betas[r] : 1.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] *= be;
    }
    tile_st_chunk(BV, r, ch, 64, pack8_f16(x));
  }
  sync_for_issue();

  // ---- off-diagonal blocks on the tensor cores: columns [0,16) I=1, [16,48) I=2, [48,96) I=3
  uint32_t ph = 0;
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, tmem + 0, Tile{smem_u32(LA), 128, false}, Tile{smem_u32(KR), 128, false}, 16, 128, 0u);
    issue_product_led(leader, tmem + 16, Tile{smem_u32(LA), 128, false}, Tile{smem_u32(KR) + 16 * 128, 128, false}, 32, 128, 0u);
    issue_product_led(leader, tmem + 48, Tile{smem_u32(LA), 128, false}, Tile{smem_u32(KR) + 48 * 128, 128, false}, 48, 128, 0u);
    umma_commit_led(leader, bar_mma);
    if (tid == 0) {
      bulk_s2g(p.saved + p.lay.qg + static_cast<size_t>(z) * 16384, TA, 16384);
      bulk_commit();
    }
  }
  __syncwarp();
  // ---- diagonal blocks, exact: pairs (i, s) of one 16-row block, s <= i, one exp2 per pair and channel.
  // Thread (block, row pair j, piece c): rows 16 blk + j and 16 blk + 15 - j - together 17 pairs, the same
  // count for every thread - over channels [8 c, 8 c + 8) and [64 + 8 c, 64 + 8 c + 8): the eight pieces of a
  // row read eight neighbouring 16-byte chunks of a tile row (and two whole lines of the gate tile), which
  // keeps the shared-memory pipe - the limit of this phase - free of replays.  The row operands stay in registers while
  // the source rows stream by; the eight pieces of a pair sit in neighbouring lanes and are added by a
  // butterfly (fixed order: deterministic).
  {
    static_assert(kPrepCwThreads == 256, "8 row pairs (one per warp) x 4 blocks x 8 pieces");
    // (a warp holds one row pair j of all four blocks: which source row comes next, and when the thread moves
    // on to its second row, is then the same for every lane)
    const int c = tid & 7, blk = (tid >> 3) & 3, j = tid >> 5;
    float qi[16], ki[16], gi[16];
    auto load_row = [&](int i) {
      unpack8_f16(tile_ld_chunk(KQ, 64 + i, c, 128), qi);
      unpack8_f16(tile_ld_chunk(KQ, 64 + i, c + 8, 128), qi + 8);
      unpack8_f16(tile_ld_chunk(KQ, i, c, 128), ki);
      unpack8_f16(tile_ld_chunk(KQ, i, c + 8, 128), ki + 8);
      gt8(Gt, i, 8 * c, gi);
      gt8(Gt, i, 64 + 8 * c, gi + 8);
      if (DELTA && full) {
        float bi[16];
        const float* bp = p.bch + (tok0 + static_cast<size_t>(i) * p.H) * kK + 8 * c;
        ld8(bp, bi);
        ld8(bp + 64, bi + 8);
#pragma unroll
        for (int e = 0; e < 16; ++e) ki[e] *= bi[e];
      }
    };
    int i = blk * 16 + j;
    load_row(i);
    // (unrolled: the loads of a pair overlap the arithmetic of the pair before it; the partial sums of all 17
    // pairs stay in registers and are added across the eight pieces at the end, 34 independent butterflies
    // instead of one after every pair)
    float pa[17], pm[17];
#pragma unroll
    for (int t = 0; t < 17; ++t) {
      if (t == j + 1) {               // the first row's pairs are done: on to the mirrored row
        i = blk * 16 + 15 - j;
        load_row(i);
      }
      const int ss = (t > j) ? t - j - 1 : t;
      const int s = blk * 16 + ss;
      float ks[16], gs[16];
      unpack8_f16(tile_ld_chunk(KQ, s, c, 128), ks);
      unpack8_f16(tile_ld_chunk(KQ, s, c + 8, 128), ks + 8);
      gt8(Gt, s, 8 * c, gs);
      gt8(Gt, s, 64 + 8 * c, gs + 8);
      float aa0 = 0.f, aa1 = 0.f, mm0 = 0.f, mm1 = 0.f;
#pragma unroll
      for (int e = 0; e < 16; e += 2) {
        const float k0 = ks[e] * exp2f(gi[e] - gs[e]);
        const float k1 = ks[e + 1] * exp2f(gi[e + 1] - gs[e + 1]);
        aa0 = fmaf(qi[e], k0, aa0);
        aa1 = fmaf(qi[e + 1], k1, aa1);
        mm0 = fmaf(ki[e], k0, mm0);
        mm1 = fmaf(ki[e + 1], k1, mm1);
      }
      pa[t] = aa0 + aa1;
      pm[t] = mm0 + mm1;
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
#pragma unroll
      for (int t = 0; t < 17; ++t) {
        pa[t] += __shfl_xor_sync(0xffffffffu, pa[t], o);
        pm[t] += __shfl_xor_sync(0xffffffffu, pm[t], o);
      }
    }
    if (c == 0) {
#pragma unroll
      for (int t = 0; t < 17; ++t) {
        const int row = (t > j) ? blk * 16 + 15 - j : blk * 16 + j;
        const int ss = (t > j) ? t - j - 1 : t;
        const int ii = row - blk * 16;
        Adg[row * kDg + ss] = p.scale * pa[t];
        Mdg[row * kDg + ss] = (DELTA && ss < ii) ? betas[row] * pm[t] : 0.f;
      }
    }
  }
  if (tid == 0) bulk_wait_read();      // the query record has left the [T; A] tile, which the epilogue now fills
  __syncthreads();
  wait_products(bar_mma, ph, ctl, 502);
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  {
    // thread t & 127 owns accumulator lane t & 127 (row r of M for lanes 0-63, of A for lanes 64-127); the two
    // warps that reach a lane quadrant split the row's 64 columns in halves
    const int t = tid & 127, half = tid >> 7;
    float d[96];
    tmem_ld32(tmem + lane_base, d);
    tmem_ld32(tmem + lane_base + 32, d + 32);
    tmem_ld32(tmem + lane_base + 64, d + 64);
    tmem_ld_wait();
    const int r = t & 63, I = r >> 4;
    float row[32];                       // this half's off-diagonal values: columns [32 half, 32 half + 32)
#pragma unroll
    for (int s = 0; s < 32; ++s) row[s] = 0.f;
    if (half == 0) {
      if (I == 1) {
#pragma unroll
        for (int s = 0; s < 16; ++s) row[s] = d[s];
      } else if (I == 2) {
#pragma unroll
        for (int s = 0; s < 32; ++s) row[s] = d[16 + s];
      } else if (I == 3) {
#pragma unroll
        for (int s = 0; s < 32; ++s) row[s] = d[48 + s];
      }
    } else if (I == 3) {
#pragma unroll
      for (int s = 0; s < 16; ++s) row[s] = d[80 + s];
    }
    if (t < 64) {
      if (DELTA) {
        const float be = betas[r];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int s = half * 32 + j;
          float m = row[j] * be;                               // off-diagonal blocks (zero beyond 16 I)
          if ((s >> 4) == I) m = (s < r) ? Mdg[r * kDg + (s & 15)] : 0.f;
          Msm[r * kMsC + s] = m;
        }
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int s8 = half * 4 + q;
        float a[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int s = s8 * 8 + e;
          float x = row[q * 8 + e] * p.scale;
          if ((s >> 4) == I) x = (s <= r) ? Adg[r * kDg + (s & 15)] : 0.f;
          a[e] = x;
        }
        tile_st_chunk(TA, 64 + r, s8, 128, pack8_f16(a));
      }
    }
  }
  tc_fence_before();
  __syncthreads();

  // ---- T = (I + M)^-1 (fp32, CUDA cores)
  if (DELTA) {
    unit_lower_inverse64_blocked<kMsC>(Msm, Msm + 64 * kMsC, TA, tid);
  } else if (tid < 64) {
    {
#pragma unroll
      for (int i = 0; i < 64; ++i)
        *reinterpret_cast<__half*>(TA + sw128_off(i, tid, 128)) = __float2half_rn((i == tid) ? 1.f : 0.f);
    }
  }
  sync_for_issue();

  if (DELTA) {
    if (warp == 0) {
      tc_fence_after();
      const uint32_t leader = elect_leader();
      issue_product_led(leader, tmem, Tile{smem_u32(TA), 128, false}, Tile{smem_u32(BGK), 64, true}, 128 + V, 64, 0u);
      umma_commit_led(leader, bar_mma);
      if (tid == 0) bulk_s2g(p.saved + p.lay.ta + static_cast<size_t>(z) * p.lay.sz_ta, TA, 16384);
      if (tid == 0) bulk_commit();
    }
    wait_products(bar_mma, ph, ctl, 503);
    if ((tid & 127) < 64) {     // rows 0-63: lane quadrants 0 and 1; the four warps of a quadrant split the columns
#pragma unroll 1
      for (int jb = tid >> 7; jb < (128 + V) / 32; jb += kPrepCwThreads / 128) {
        float d[32];
        tmem_ld32(tmem + lane_base + jb * 32, d);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) tile_st_chunk(WU, tid & 127, jb * 4 + i, 64, pack8_f16(d + 8 * i));
      }
    }
    sync_for_issue();
  } else if (tid == 0) {
    bulk_s2g(p.saved + p.lay.ta + static_cast<size_t>(z) * p.lay.sz_ta, TA, 16384);
    bulk_commit();
  }

  constexpr int N3 = DELTA ? 128 + V : V;
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, tmem, Tile{smem_u32(KD), 64, true}, Tile{smem_u32(DELTA ? WU : BV), 64, true}, N3, 64, 0u);
    umma_commit_led(leader, bar_mma);
    if (DELTA) {
      if (tid == 0) bulk_s2g(p.saved + p.lay.w + static_cast<size_t>(z) * p.lay.sz_w, WU, 16384);
      if (tid == 0) bulk_s2g(p.saved + p.lay.u + static_cast<size_t>(z) * p.lay.sz_u, WU + 16384, V * 128);
    } else {
      if (tid == 0) bulk_s2g(p.saved + p.lay.u + static_cast<size_t>(z) * p.lay.sz_u, BV, V * 128);
    }
    if (tid == 0) bulk_commit();
  }
  wait_products(bar_mma, ph, ctl, 504);
  {
    // P and R are staged as their record images in the two ratio-scaled operand tiles (dead now) and
    // leave by bulk stores; the two thread halves split the columns.
    unsigned char* SP = LA;
    unsigned char* SR = KR;
    const int tq = tid & 127;
    // warp w reads the lanes of quadrant w & 3; the four warps of a quadrant split the 32-column blocks
#pragma unroll 1
    for (int jb = tid >> 7; jb < N3 / 32; jb += kPrepCwThreads / 128) {
      float d[32];
      tmem_ld32(tmem + lane_base + jb * 32, d);
      tmem_ld_wait();
      if (DELTA && jb < 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) tile_st_chunk(SP, tq, jb * 4 + i, 128, pack8_f16(d + 8 * i));
      } else {
        const int c8 = (jb - (DELTA ? 4 : 0)) * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (DELTA) *reinterpret_cast<uint4*>(SR + rrec_off(tq, c8 + i)) = pack8_f16(d + 8 * i);
          else tile_st_chunk(SR, tq, c8 + i, 128, pack8_f16(d + 8 * i));     // no delta term: plain tile image
        }
      }
    }
    fence_proxy_async();
    __syncthreads();
    if (tid == 0) {
      if (DELTA) bulk_s2g(p.saved + p.lay.p + static_cast<size_t>(z) * p.lay.sz_p, SP, 32768);
      bulk_s2g(p.saved + p.lay.r + static_cast<size_t>(z) * p.lay.sz_r, SR, V * 256);
      bulk_commit();
    }
  }
  if (tid == 0) bulk_wait_read();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

template <int V, bool DELTA>
static int launch_prepare_cw_t(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk,
                               const CUtensorMap& mv, cudaStream_t st) {
  const int smem = 32768 * 4 + 16384 + V * 128 + 16384 + 16384 + (128 * kDg + 64) * 4 +
                   static_cast<int>(sizeof(CtaShared)) + 1024;
  auto kern = prepare_cw_kernel<V, DELTA>;
  static SmemAttr attr;
  if (attr.set(kern, smem)) return kErrLaunch;
  kern<<<p.nbh * p.cn, kPrepCwThreads, smem, st>>>(p, mq, mk, mv);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

int launch_prepare_cw(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                      cudaStream_t st) {
  if (p.V == 64) return p.delta ? launch_prepare_cw_t<64, true>(p, mq, mk, mv, st) : launch_prepare_cw_t<64, false>(p, mq, mk, mv, st);
  return p.delta ? launch_prepare_cw_t<128, true>(p, mq, mk, mv, st) : launch_prepare_cw_t<128, false>(p, mq, mk, mv, st);
}

}  // namespace lg
