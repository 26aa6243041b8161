// Chunk-parallel forward kernels: `prepare` (UT / WY transform and the per-chunk state map) and
// `output` (v_new and o from the chunk-entry states).  One CTA per chunk: 256 threads in `prepare`,
// 128 in `output`.
//
// All tensor-core products are tcgen05 with M = 128, fp16 operands in SW128 shared-memory tiles and
// fp32 accumulators in TMEM; two 64-row operands that share the other operand are stacked into one
// 128-row tile so that a single product serves both (rows 0-63 of the accumulator belong to the
// first, rows 64-127 to the second).
#include "gdn_common.cuh"
#include "host_util.h"

namespace lg {

constexpr int kMs = 68;  // row stride (floats) of the fp32 copy of M used by the inverse

// ---------------------------------------------------------------------------------------------
// prepare: per chunk
//   G = cumsum(g), ratio[i,s] = exp(G_i - G_s) (s <= i)
//   [KK; QK] = [k; q] k^T                                    (product 1)
//   M = strict_lower(beta_i ratio KK), A = tril(scale ratio QK), T = (I + M)^-1  (fp32, CUDA cores)
//   [w | u] = T [beta gamma k | beta v]                      (product 2)
//   [P | R] = kd^T [w | u],  kd = k exp(G_last - G_i)        (product 3)
// Reference: gdn2_chunkwise.py:130-158 of the reference project; P and R fold its state update
// h' = exp(G_last) h + kd^T (u - w h) into h' = exp(G_last) h - P h + R.
// ---------------------------------------------------------------------------------------------
template <int V, bool DELTA>
__global__ void __launch_bounds__(256)
prepare_kernel(const Problem p, const __grid_constant__ CUtensorMap mq,
               const __grid_constant__ CUtensorMap mk, const __grid_constant__ CUtensorMap mv) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = DELTA ? align1024(smem_raw) : align1024_generic(smem_raw);   // measured per variant
  unsigned char* KQ = sm;                      // 32 KB: rows 0-63 k, rows 64-127 q; later M (fp32), then [w | u]
  unsigned char* BGK = sm + 32768;             // 16 KB: beta gamma k   (64 x 128)
  unsigned char* BV = BGK + 16384;             // beta v (64 x V), directly behind BGK: one N = 128 + V operand
  unsigned char* KD = BV + V * 128;            // 16 KB: kd            (64 x 128)
  unsigned char* TA = KD + 16384;              // 16 KB: [T; A]        (128 x 64)
  float* fs = reinterpret_cast<float*>(TA + 16384);
  float* Gs = fs;            // [64] cumulative log decay
  float* betas = fs + 64;    // [64]
  float* decs = fs + 128;    // [64] exp(G_last - G_i)
  float* bgs = fs + 192;     // [64] beta_i exp(G_i)
  float* tmp = fs + 256;     // [2]
  CtaShared* cs = reinterpret_cast<CtaShared*>(fs + 264);
  float* Msm = reinterpret_cast<float*>(KQ);           // [64][kMs]
  float* Tsm = Msm + 64 * kMs;                          // scratch of the inverse (kInvScratchFloats)
  unsigned char* WU = KQ;

  // Threads 0-127 and 128-255 reach the same TMEM lanes (lane quadrant = warp & 3): the two halves take
  // the same rows and split the columns of every epilogue.
  const int tid = threadIdx.x, warp = tid >> 5, tq = tid & 127, half = tid >> 7;
  const int bh = p.bh0 + blockIdx.x / p.cn, c = p.c0 + blockIdx.x % p.cn, z = bh * p.NT + c, b = bh / p.H, h = bh % p.H;
  CtaCtl ctl{p.status, &cs->abort_flag};
  uint64_t* bar_load = &cs->bar[0];
  uint64_t* bar_mma = &cs->bar[1];

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
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, 256);
    tmem_relinquish();
  }
  float gval = 0.f, bval = 1.f;
  if (tid < 64) {
    const size_t tok = (static_cast<size_t>(b) * p.L + c * kC + tid) * p.H + h;
    if (p.gate == LETHE_GATE_SCALAR) gval = p.g[tok];
    if (DELTA) bval = p.beta[tok];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;


  // ---- gate: cumulative log decay of the chunk
  const float G = chunk_cumsum(gval, tid, tmp);
  if (tid < 64) {
    Gs[tid] = G;
    betas[tid] = bval;
  }
  __syncthreads();
  const float Glast = Gs[63];
  if (tid < 64) {
    decs[tid] = __expf(Glast - G);
    bgs[tid] = bval * __expf(G);
  }
  if (tid < kK) reinterpret_cast<float*>(p.saved + p.lay.ad)[static_cast<size_t>(z) * kK + tid] = __expf(Glast);
  __syncthreads();

  // ---- operands: k, q -> fp16 in place; kd, beta gamma k, beta v
  mbar_wait_warp(bar_load, 0, ctl, 201);
  for (int idx = tid; idx < 64 * 16; idx += 256) {
    const int r = idx >> 4, ch = idx & 15;
    float x[8], y[8];
    unpack8_in(tile_ld_chunk(KQ, r, ch, 128), x, p.qk16);
    tile_st_chunk(KQ, r, ch, 128, pack8_f16(x));
    const float de = decs[r];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = x[i] * de;
    tile_st_chunk(KD, r, ch, 64, pack8_f16(y));
    if (DELTA) {
      const float bg = bgs[r];
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = x[i] * bg;
      tile_st_chunk(BGK, r, ch, 64, pack8_f16(y));
    }
    unpack8_in(tile_ld_chunk(KQ, 64 + r, ch, 128), x, p.qk16);
    tile_st_chunk(KQ, 64 + r, ch, 128, pack8_f16(x));
  }
  for (int idx = tid; idx < 64 * (V / 8); idx += 256) {
    const int r = idx / (V / 8), ch = idx % (V / 8);
    float x[8];
    unpack8_bf16(tile_ld_chunk(BV, r, ch, 64), x);
    const float be = DELTA ? betas[r] : 1.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] *= be;
    tile_st_chunk(BV, r, ch, 64, pack8_f16(x));
  }
  fence_proxy_async();
  __syncthreads();

  // ---- product 1: [KK; QK] = [k; q] k^T
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, tmem, Tile{smem_u32(KQ), 128, false}, Tile{smem_u32(KQ), 128, false}, 64, 128, 0u);
    umma_commit_led(leader, bar_mma);
  }
  __syncwarp();
  mbar_wait_warp(bar_mma, 0, ctl, 202);
  tc_fence_after();
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  {
    // each half takes 32 of the 64 columns; rows 0-31 (lane quadrant 0 of either operand half) have
    // nothing right of column 31, so the triangle is cut per warp
    const bool live = (half == 0) || ((warp & 1) != 0);
    float d[32];
    if (live) {
      tmem_ld32(tmem + lane_base + half * 32, d);
      tmem_ld_wait();
    }
    if (tq < 64) {
      if (DELTA) {
        const int r = tq;
        const float Gr = Gs[r], be = betas[r];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int s = half * 32 + j;
          float m = 0.f;
          if (live) m = (s < r) ? be * __expf(Gr - Gs[s]) * d[j] : 0.f;
          Msm[r * kMs + s] = m;
        }
      }
    } else {
      const int r = tq - 64;
      const float Gr = Gs[r];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int s8 = half * 4 + q;
        float a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = 0.f;
        if (live) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int s = s8 * 8 + i;
            a[i] = (s <= r) ? p.scale * __expf(Gr - Gs[s]) * d[q * 8 + i] : 0.f;
          }
        }
        tile_st_chunk(TA, 64 + r, s8, 128, pack8_f16(a));
      }
    }
  }
  tc_fence_before();
  __syncthreads();

  // ---- T = (I + M)^-1 (fp32, CUDA cores)
  if (DELTA) {
    unit_lower_inverse64_blocked<kMs>(Msm, Tsm, TA, tid);
  } else if (tid < 64) {
    {
#pragma unroll
      for (int i = 0; i < 64; ++i)
        *reinterpret_cast<__half*>(TA + sw128_off(i, tid, 128)) = __float2half_rn((i == tid) ? 1.f : 0.f);
    }
  }
  fence_proxy_async();
  __syncthreads();

  uint32_t ph = 1;
  if (DELTA) {
    // ---- product 2: [w | u] = T [beta gamma k | beta v]
    if (warp == 0) {
      tc_fence_after();
      const uint32_t leader = elect_leader();
      issue_product_led(leader, tmem, Tile{smem_u32(TA), 128, false}, Tile{smem_u32(BGK), 64, true}, 128 + V, 64, 0u);
      umma_commit_led(leader, bar_mma);
      if (tid == 0) bulk_s2g(p.saved + p.lay.ta + static_cast<size_t>(z) * p.lay.sz_ta, TA, 16384);
      if (tid == 0) bulk_commit();
    }
    __syncwarp();
    mbar_wait_warp(bar_mma, ph, ctl, 203);
    ph ^= 1;
    tc_fence_after();
    if (tq < 64) {
      constexpr int kHalf2 = (128 + V) / 64;
#pragma unroll
      for (int jb = half * kHalf2; jb < (half + 1) * kHalf2; ++jb) {
        float d[32];
        tmem_ld32(tmem + lane_base + jb * 32, d);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) tile_st_chunk(WU, tq, jb * 4 + i, 64, pack8_f16(d + 8 * i));
      }
    }
    tc_fence_before();
    fence_proxy_async();
    __syncthreads();
  } else if (tid == 0) {
    bulk_s2g(p.saved + p.lay.ta + static_cast<size_t>(z) * p.lay.sz_ta, TA, 16384);
    bulk_commit();
  }

  // ---- product 3: [P | R] = kd^T [w | u]   (no delta: R = kd^T v)
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
  __syncwarp();
  mbar_wait_warp(bar_mma, ph, ctl, 204);
  tc_fence_after();
  // P and R are staged as their record images in tiles nothing reads any more and leave by bulk
  // stores: P behind BGK (beta gamma k, beta v, kd are dead), R where k and q were once the stores
  // of [w | u] have finished reading it.
  if (tid == 0) bulk_wait_read();
  __syncthreads();
  {
    unsigned char* SP = BGK;
    unsigned char* SR = KQ;
    constexpr int kHalf3 = N3 / 64;
#pragma unroll 1
    for (int jb = half * kHalf3; jb < (half + 1) * kHalf3; ++jb) {
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

// ---------------------------------------------------------------------------------------------
// output: per chunk, given the state h entering it
//   [w h ; (scale gamma q) h] = [w; qg] h                    (product 1)
//   v_new = u - w h
//   o = qg h + A v_new                                       (product 2 accumulates onto rows 64-127)
// Reference: gdn2_chunkwise.py:146-153.
// ---------------------------------------------------------------------------------------------
template <int V, bool DELTA, bool CW>
__global__ void __launch_bounds__(128)
output_kernel(const Problem p, const __grid_constant__ CUtensorMap mq) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = CW ? align1024(smem_raw) : align1024_generic(smem_raw);   // measured per variant
  unsigned char* WQ = sm;                       // 32 KB: rows 0-63 w, rows 64-127 scale gamma q
  unsigned char* HT = sm + 32768;               // state image 128 x V
  unsigned char* TAt = HT + V * 256;            // 16 KB [T; A]
  unsigned char* VN = TAt + 16384;              // v_new 64 x V
  float* fs = reinterpret_cast<float*>(VN + V * 128);
  float* Gs = fs;
  float* tmp = fs + 64;
  CtaShared* cs = reinterpret_cast<CtaShared*>(fs + 72);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int bh = p.bh0 + blockIdx.x / p.cn, c = p.c0 + blockIdx.x % p.cn, z = bh * p.NT + c, b = bh / p.H, h = bh % p.H;
  CtaCtl ctl{p.status, &cs->abort_flag};
  const unsigned char* Ug = p.saved + p.lay.u + static_cast<size_t>(z) * p.lay.sz_u;
  uint64_t* bar_load = &cs->bar[0];
  uint64_t* bar_mma = &cs->bar[1];
  uint64_t* bar_ht = &cs->bar[2];       // the state image, loaded once the scan before this kernel is complete

  if (tid == 0) {
    cs->abort_flag = 0;
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    mbar_init(bar_ht, 1);
    fence_mbar_init();
    fence_proxy_async();
    mbar_expect_tx(bar_load, 16384u + (DELTA ? 16384u : V * 128u) + 16384u);
    for (int a = 0; a < 2; ++a) {
      // the query operand: q from the user tensor (scaled below), or - channel-wise gate - the record of
      // scale * gamma * q that the prepare kernel left (two 64-row atoms of 8 KB)
      if (CW) bulk_g2s(WQ + a * 16384 + 8192, p.saved + p.lay.qg + static_cast<size_t>(z) * 16384 + a * 8192, 8192, bar_load);
      else tma_load_4d(WQ + a * 16384 + 8192, &mq, bar_load, a * 64, h, c * kC, b);
      if (DELTA)
        bulk_g2s(WQ + a * 16384, p.saved + p.lay.w + static_cast<size_t>(z) * p.lay.sz_w + a * 8192, 8192, bar_load);
    }
    if (!DELTA) bulk_g2s(VN, Ug, V * 128, bar_load);   // v_new = u = v
    bulk_g2s(TAt, p.saved + p.lay.ta + static_cast<size_t>(z) * p.lay.sz_ta, 16384, bar_load);
    // (the state image, written by the scan just before this kernel, is loaded after griddep_wait)
  }
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, V);
    tmem_relinquish();
  }
  float gval = 0.f;
  if (tid < 64 && p.gate == LETHE_GATE_SCALAR)
    gval = p.g[(static_cast<size_t>(b) * p.L + c * kC + tid) * p.H + h];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;

  // u row of this thread (threads 0-63), kept packed
  uint4 upk[V / 8];
  if (DELTA && tid < 64) {
#pragma unroll
    for (int ch = 0; ch < V / 8; ++ch) upk[ch] = *reinterpret_cast<const uint4*>(Ug + sw128_chunk(tid, ch, 64));
  }
  const float G = chunk_cumsum(gval, tid, tmp);
  if (tid < 64) Gs[tid] = G;
  __syncthreads();

  // the loads above fetch inputs and records older than the scan; once the scan is complete (at once,
  // except for the CTAs that started early) its state image is fetched too
  griddep_wait();
  griddep_launch();
  if (tid == 0) {
    mbar_expect_tx(bar_ht, V * 256u);
    bulk_g2s(HT, p.saved + p.lay.hc + static_cast<size_t>(z + bh) * p.lay.sz_hc, V * 256, bar_ht);
  }
  mbar_wait_warp(bar_load, 0, ctl, 211);
  for (int idx = tid; idx < 64 * 16; idx += 128) {
    const int r = idx >> 4, ch = idx & 15;
    if (!CW) {
      float x[8];
      unpack8_in(tile_ld_chunk(WQ, 64 + r, ch, 128), x, p.qk16);
      const float sg = p.scale * __expf(Gs[r]);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] *= sg;
      tile_st_chunk(WQ, 64 + r, ch, 128, pack8_f16(x));
    }
    if (!DELTA) tile_st_chunk(WQ, r, ch, 128, make_uint4(0, 0, 0, 0));
  }
  fence_proxy_async();
  __syncthreads();
  mbar_wait_warp(bar_ht, 0, ctl, 214);

  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, tmem, Tile{smem_u32(WQ), 128, false}, Tile{smem_u32(HT), 128, true}, V, 128, 0u);
    umma_commit_led(leader, bar_mma);
  }
  __syncwarp();
  mbar_wait_warp(bar_mma, 0, ctl, 212);
  tc_fence_after();
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  if (DELTA) {
    if (tid < 64) {
#pragma unroll
      for (int jb = 0; jb < V / 32; ++jb) {
        float d[32];
        tmem_ld32(tmem + lane_base + jb * 32, d);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float u8[8];
          unpack8_f16(upk[jb * 4 + i], u8);
#pragma unroll
          for (int e = 0; e < 8; ++e) u8[e] -= d[8 * i + e];
          tile_st_chunk(VN, tid, jb * 4 + i, 64, pack8_f16(u8));
        }
      }
    }
  }
  // Every thread must be past its wait on the first product before the second one is committed: a
  // thread still polling the barrier's first phase when the second phase completes would wait for
  // a third completion that never comes.
  tc_fence_before();
  fence_proxy_async();
  __syncthreads();

  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, tmem, Tile{smem_u32(TAt), 128, false}, Tile{smem_u32(VN), 64, true}, V, 64, 1u);
    umma_commit_led(leader, bar_mma);
    if (tid == 0) bulk_s2g(p.saved + p.lay.vn + static_cast<size_t>(z) * p.lay.sz_vn, VN, V * 128);
    if (tid == 0) bulk_commit();
  }
  __syncwarp();
  mbar_wait_warp(bar_mma, 1, ctl, 213);
  tc_fence_after();
  if (tid >= 64) {
    const int r = tid - 64;
    __nv_bfloat16* og = p.o + ((static_cast<size_t>(b) * p.L + c * kC + r) * p.H + h) * V;
#pragma unroll
    for (int jb = 0; jb < V / 32; ++jb) {
      float d[32];
      tmem_ld32(tmem + lane_base + jb * 32, d);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(og + jb * 32 + 8 * i) = pack8_bf16(d + 8 * i);
    }
  }
  if (tid == 0) bulk_wait_read();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, V);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <int V, bool DELTA>
static int launch_prepare_t(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk,
                            const CUtensorMap& mv, cudaStream_t st) {
  const int smem = 32768 + 16384 + V * 128 + 16384 + 16384 + 264 * 4 + static_cast<int>(sizeof(CtaShared)) + 1024;
  auto kern = prepare_kernel<V, DELTA>;
  static SmemAttr attr;
  if (attr.set(kern, smem)) return kErrLaunch;
  kern<<<p.nbh * p.cn, 256, smem, st>>>(p, mq, mk, mv);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
template <int V, bool DELTA, bool CW>
static int launch_output_t(const Problem& p, const CUtensorMap& mq, cudaStream_t st) {
  const int smem = 32768 + V * 256 + 16384 + V * 128 + 128 * 4 + 1024;
  auto kern = output_kernel<V, DELTA, CW>;
  static SmemAttr attr;
  if (attr.set(kern, smem)) return kErrLaunch;
  if (launch_dependent(kern, dim3(p.nbh * p.cn), dim3(128), smem, st, p, mq) != cudaSuccess) return kErrLaunch;
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

int launch_prepare(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                   cudaStream_t st) {
  if (p.V == 64) return p.delta ? launch_prepare_t<64, true>(p, mq, mk, mv, st) : launch_prepare_t<64, false>(p, mq, mk, mv, st);
  return p.delta ? launch_prepare_t<128, true>(p, mq, mk, mv, st) : launch_prepare_t<128, false>(p, mq, mk, mv, st);
}
int launch_output(const Problem& p, const CUtensorMap& mq, cudaStream_t st) {
  if (p.gate == LETHE_GATE_CHANNEL) {
    if (p.V == 64) return p.delta ? launch_output_t<64, true, true>(p, mq, st) : launch_output_t<64, false, true>(p, mq, st);
    return p.delta ? launch_output_t<128, true, true>(p, mq, st) : launch_output_t<128, false, true>(p, mq, st);
  }
  if (p.V == 64) return p.delta ? launch_output_t<64, true, false>(p, mq, st) : launch_output_t<64, false, false>(p, mq, st);
  return p.delta ? launch_output_t<128, true, false>(p, mq, st) : launch_output_t<128, false, false>(p, mq, st);
}

}  // namespace lg
