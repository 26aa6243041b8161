// Chunk-parallel backward kernels.  One CTA per chunk (128 threads in `bwd_pre`, 256 in Stage B),
// tcgen05 products with M = 128 and stacked 64-row operands as in the forward kernels.
//
//   bwd_pre    : Rb = (scale gamma q)^T do - w^T (A^T do)          input of the adjoint state scan
//   bwd_stageb : dv2, dq, the Stage-B part of dk and of the gate gradient, dw
//   (the WY / triangular-inverse VJP, which closes dv, dbeta, dk and dg, lives in gdn_bwd_wy.cu)
//
// Reference (file:line in the reference project): reverse scan K#1 gdn2_assemble.py:71-99, closed
// Stage B gdn2_assemble.py:521-585 (scalar-gate form: gate broadcast over channels, dg summed),
// K#2 gdn2_assemble.py:102-147.
//
// Scalar-gate identities used to avoid per-channel work (i, s index tokens of the chunk):
//   sum_d q~[i,d] dq_intra[i,d] = sum_s dA[i,s] A[i,s]            (row sums of E = dA . A)
//   sum_d k[s,d] dk_intra[s,d]  = <v_new[s,:], (A^T do)[s,:]>     (column sums of E)
//   sum_d dde[s,d]              = <v_new[s,:], (kd dh)[s,:]>
// The gate gradient is a reverse cumulative sum in which large terms cancel (every -dde_i of a row
// against the +sum_i dde_i of the chunk's last row, row sums of E against its column sums); each
// such pair is therefore formed from the same fp32 numbers, as the reference's closed form does.
#include "gdn_common.cuh"
#include "host_util.h"

namespace lg {

// ---------------------------------------------------------------------------------------------
template <int V, bool DELTA, bool CW>
__global__ void __launch_bounds__(128)
bwd_pre_kernel(const Problem p, const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mdo) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = CW ? align1024(smem_raw) : align1024_generic(smem_raw);   // measured per variant
  unsigned char* QG = sm;                    // 16 KB: scale gamma q (64 x 128)
  unsigned char* Wt = QG + 16384;            // 16 KB: w
  unsigned char* DO = Wt + 16384;            // do (64 x V)
  unsigned char* TAt = DO + V * 128;         // 16 KB: [T | A]
  unsigned char* DVL = TAt + 16384;          // A^T do (64 x V)
  float* fs = reinterpret_cast<float*>(DVL + V * 128);
  float* Gs = fs;
  float* tmp = fs + 64;
  CtaShared* cs = reinterpret_cast<CtaShared*>(fs + 72);

  const int tid = threadIdx.x, warp = tid >> 5;
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
    mbar_expect_tx(bar_load, 16384u + V * 128u + (DELTA ? 32768u : 0u));
    // scale * gamma * q: built below from q, or - channel-wise gate - read as the record the forward's prepare kernel left
    if (CW) bulk_g2s(QG, p.saved + p.lay.qg + static_cast<size_t>(z) * 16384, 16384, bar_load);
    else for (int a = 0; a < 2; ++a) tma_load_4d(QG + a * 8192, &mq, bar_load, a * 64, h, c * kC, b);
    for (int a = 0; a < V / 64; ++a) tma_load_4d(DO + a * 8192, &mdo, bar_load, a * 64, h, c * kC, b);
    if (DELTA) {
      bulk_g2s(Wt, p.saved + p.lay.w + static_cast<size_t>(z) * p.lay.sz_w, 16384, bar_load);
      bulk_g2s(TAt, p.saved + p.lay.ta + static_cast<size_t>(z) * p.lay.sz_ta, 16384, bar_load);
    }
  }
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, 2 * V);     // two accumulators of V columns: three CTAs fit an SM at d_v = 64
    tmem_relinquish();
  }
  float gval = 0.f;
  if (tid < 64 && p.gate == LETHE_GATE_SCALAR) gval = p.g[(static_cast<size_t>(b) * p.L + c * kC + tid) * p.H + h];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;
  const float G = chunk_cumsum(gval, tid, tmp);
  if (tid < 64) Gs[tid] = G;
  __syncthreads();
  mbar_wait_warp(bar_load, 0, ctl, 401);
  if (!CW) {
    for (int idx = tid; idx < 64 * 16; idx += 128) {
      const int r = idx >> 4, ch = idx & 15;
      float x[8];
      unpack8_in(tile_ld_chunk(QG, r, ch, 64), x, p.qk16);
      const float sg = p.scale * __expf(Gs[r]);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] *= sg;
      tile_st_chunk(QG, r, ch, 64, pack8_f16(x));
    }
  }
  for (int idx = tid; idx < 64 * (V / 8); idx += 128) {
    const int r = idx / (V / 8), ch = idx % (V / 8);
    float x[8];
    unpack8_bf16(tile_ld_chunk(DO, r, ch, 64), x);
    tile_st_chunk(DO, r, ch, 64, pack8_f16(x));
  }
  sync_for_issue();
  uint32_t ph = 0;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  if (DELTA) {
    // rows 64-127: A^T do
    if (warp == 0) {
      tc_fence_after();
      const uint32_t leader = elect_leader();
      issue_product_led(leader, tmem, Tile{smem_u32(TAt), 64, true}, Tile{smem_u32(DO), 64, true}, V, 64, 0u);
      issue_product_led(leader, tmem + V, Tile{smem_u32(QG), 64, true}, Tile{smem_u32(DO), 64, true}, V, 64, 0u);
      umma_commit_led(leader, bar_mma);
    }
    wait_products(bar_mma, ph, ctl, 402);
    if (tid >= 64) {
#pragma unroll
      for (int jb = 0; jb < V / 32; ++jb) {
        float d[32];
        tmem_ld32(tmem + lane_base + jb * 32, d);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) tile_st_chunk(DVL, tid - 64, jb * 4 + i, 64, pack8_f16(d + 8 * i));
      }
    }
    sync_for_issue();
    if (warp == 0) {
      tc_fence_after();
      const uint32_t leader = elect_leader();
      issue_product_led(leader, tmem + V, Tile{smem_u32(Wt), 64, true}, Tile{smem_u32(DVL), 64, true}, V, 64, 1u, true);
      umma_commit_led(leader, bar_mma);
    }
  } else if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, tmem + V, Tile{smem_u32(QG), 64, true}, Tile{smem_u32(DO), 64, true}, V, 64, 0u);
    umma_commit_led(leader, bar_mma);
  }
  wait_products(bar_mma, ph, ctl, 403);
  {
    unsigned char* SR = QG;   // q and w are dead: Rb is staged there as its record image
#pragma unroll
    for (int jb = 0; jb < V / 32; ++jb) {
      float d[32];
      tmem_ld32(tmem + V + lane_base + jb * 32, d);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (DELTA) *reinterpret_cast<uint4*>(SR + rrec_off(tid, jb * 4 + i)) = pack8_f16(d + 8 * i);
        else tile_st_chunk(SR, tid, jb * 4 + i, 128, pack8_f16(d + 8 * i));     // no delta term: plain tile image
      }
    }
    fence_proxy_async();
    __syncthreads();
    if (tid == 0) {
      bulk_s2g(p.scratch + p.lay.rb + static_cast<size_t>(z) * p.lay.sz_rb, SR, V * 256);
      bulk_commit();
      bulk_wait_read();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 2 * V);
}

// ---------------------------------------------------------------------------------------------
// Stage B in three product groups, so that 256 TMEM columns and 107 KB of shared memory suffice at
// d_v = 64 and two CTAs share an SM (the loads and the stores of one chunk overlap the other's work):
//   group 1 : k dh (lanes 64-127), A^T do (lanes 64-127), dA = do v_new^T (lanes 0-63)
//   group 2a: [do; dv2] h^T (dq_inter | -dw), dAr k (dq_intra)
//   group 2b: dAr^T q, v_new dh^T  ->  Stage-B dk = dAr^T q + dec_end (v_new dh^T)
// The decay to the chunk end is applied in the epilogues in fp32 (kd = k dec_end and dec_end v_new are
// never formed as operands).  Operands that have to land in lanes 64-127 are 64-row tiles read through a
// 128-row view that starts 64 rows early; rows 0-63 of such a view are the neighbouring tile, and what
// they produce (lanes 0-63 of that accumulator) is never read.
// ---------------------------------------------------------------------------------------------
template <int V, bool DELTA>
__global__ void __launch_bounds__(256)
bwd_stageb_kernel(const Problem p, const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                  const __grid_constant__ CUtensorMap mdo, const __grid_constant__ CUtensorMap mdq,
                  const __grid_constant__ CUtensorMap mdk) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = align1024(smem_raw);
  unsigned char* QT = sm;                       // 16 KB: q (64 x 128)
  unsigned char* KT = QT + 16384;               // 16 KB: k (64 x 128), directly behind q (early view reads q)
  unsigned char* DD = KT + 16384;               // V*256: rows 0-63 do, rows 64-127 dv2
  unsigned char* DS = DD + V * 256;             // 8 KB: scale * dA * ratio (64 x 64)
  unsigned char* AT = DS + 8192;                // 8 KB: A (64 x 64), directly behind DS (early view reads DS)
  unsigned char* VN = AT + 8192;                // V*128: v_new (64 x V); 128-row views run on into Ht
  unsigned char* Ht = VN + V * 128;             // V*256: h entering the chunk
  unsigned char* DHt = Ht + V * 256;            // V*256: dh
  float* fs = reinterpret_cast<float*>(DHt + V * 256);
  float* Gs = fs;            // [64]
  float* t3p = fs + 64;      // [2][64] per column half: column sum of E plus dde row sum
  float* ddep = fs + 192;    // [2][64] per column half: dde row sums
  float* t2p = fs + 320;     // [2][64] per column half: row sums of dA o A
  float* t1p = fs + 448;     // [2][64] per column half: <dq_inter, q>
  float* decs = fs + 576;    // [64] exp(G_last - G_i)
  float* tmp = fs + 640;     // [16]
  CtaShared* cs = reinterpret_cast<CtaShared*>(fs + 656);

  // Threads 0-127 and 128-255 reach the same TMEM lanes (lane quadrant = warp & 3): the two halves
  // take the same rows and split the columns of every epilogue.
  const int tid = threadIdx.x, warp = tid >> 5, tq = tid & 127, half = tid >> 7;
  const int bh = p.bh0 + blockIdx.x / p.cn, c = p.c0 + blockIdx.x % p.cn, z = bh * p.NT + c, b = bh / p.H, h = bh % p.H;
  CtaCtl ctl{p.status, &cs->abort_flag};
  uint64_t* bar_load = &cs->bar[0];
  uint64_t* bar_mma = &cs->bar[1];
  uint64_t* bar_dh = &cs->bar[2];       // dh, loaded once the adjoint scan before this kernel is complete
  constexpr uint32_t kCols = (V == 64) ? 256u : 512u;
  if (tid == 0) {
    cs->abort_flag = 0;
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 2);     // two issuing warps commit every product group
    mbar_init(bar_dh, 1);
    fence_mbar_init();
    fence_proxy_async();
    mbar_expect_tx(bar_load, 16384u + 16384u + V * 128u + 8192u + V * 128u + V * 256u);
    for (int a = 0; a < 2; ++a) {
      tma_load_4d(KT + a * 8192, &mk, bar_load, a * 64, h, c * kC, b);
      tma_load_4d(QT + a * 8192, &mq, bar_load, a * 64, h, c * kC, b);
    }
    for (int a = 0; a < V / 64; ++a) {
      tma_load_4d(DD + a * 16384, &mdo, bar_load, a * 64, h, c * kC, b);
      bulk_g2s(VN + a * 8192, p.saved + p.lay.vn + static_cast<size_t>(z) * p.lay.sz_vn + a * 8192, 8192, bar_load);
    }
    // the [T; A] record is 128 rows of one 64-column atom: its second half is the image of A
    bulk_g2s(AT, p.saved + p.lay.ta + static_cast<size_t>(z) * p.lay.sz_ta + 8192, 8192, bar_load);
    bulk_g2s(Ht, p.saved + p.lay.hc + static_cast<size_t>(z + bh) * p.lay.sz_hc, V * 256, bar_load);
    // (dh, written by the adjoint scan just before this kernel, is loaded after griddep_wait)
  }
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, kCols);
    tmem_relinquish();
  }
  const size_t tok0 = (static_cast<size_t>(b) * p.L + c * kC) * p.H + h;   // token index of row 0 (stride H)
  float gval = 0.f;
  if (tid < 64 && p.gate == LETHE_GATE_SCALAR) gval = p.g[tok0 + static_cast<size_t>(tid) * p.H];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;
  // group 1: k dh, A^T do, dA;  group 2a: [do; dv2] h^T, dAr k;  group 2b: dAr^T q, v_new dh^T
  const uint32_t g1D = tmem, g1A = tmem + V, g1C = tmem + 2 * V;
  const uint32_t cB = tmem, cA2 = tmem + 128, cD1 = tmem, cD2 = tmem + 128;

  const float G = chunk_cumsum(gval, tid, tmp);
  if (tid < 64) Gs[tid] = G;
  __syncthreads();
  const float Glast = Gs[63];
  if (tid < 64) decs[tid] = __expf(Glast - G);

  // the loads above fetch inputs and records older than the adjoint scan; once it is complete (at once,
  // except for the CTAs that started early) its dh image is fetched too
  griddep_wait();
  griddep_launch();
  if (tid == 0) {
    mbar_expect_tx(bar_dh, V * 256u);
    bulk_g2s(DHt, p.scratch + p.lay.dh + static_cast<size_t>(z) * p.lay.sz_dh, V * 256, bar_dh);
  }
  mbar_wait_warp(bar_load, 0, ctl, 411);
  for (int idx = tid; idx < 64 * 16; idx += 256) {
    const int r = idx >> 4, ch = idx & 15;
    float x[8];
    unpack8_in(tile_ld_chunk(KT, r, ch, 64), x, p.qk16);
    tile_st_chunk(KT, r, ch, 64, pack8_f16(x));
    unpack8_in(tile_ld_chunk(QT, r, ch, 64), x, p.qk16);
    tile_st_chunk(QT, r, ch, 64, pack8_f16(x));
  }
  for (int idx = tid; idx < 64 * (V / 8); idx += 256) {
    const int r = idx / (V / 8), ch = idx % (V / 8);
    float x[8];
    unpack8_bf16(tile_ld_chunk(DD, r, ch, 128), x);
    tile_st_chunk(DD, r, ch, 128, pack8_f16(x));
  }
  sync_for_issue();
  mbar_wait_warp(bar_dh, 0, ctl, 415);

  uint32_t ph = 0;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  // ---- group 1 (two warps issue, half of the group's products each)
  if (warp == 0 || warp == 4) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    if (warp == 0) {
      issue_product_led(leader, g1D, Tile{smem_u32(KT) - 8192, 64, false}, Tile{smem_u32(DHt), 128, true}, V, 128, 0u);
    } else {
      issue_product_led(leader, g1A, Tile{smem_u32(AT) - 8192, 64, true}, Tile{smem_u32(DD), 128, true}, V, 64, 0u);
      issue_product_led(leader, g1C, Tile{smem_u32(DD), 128, false}, Tile{smem_u32(VN), 64, false}, 64, V, 0u);
    }
    umma_commit_led(leader, bar_mma);
  }
  // in the shadow of the products: exp(G_last) <dh, h>; the two tile images share the swizzle, so the
  // product is elementwise (the tiles are only read)
  float dhh = 0.f;
  for (int idx = tid; idx < kK * V / 8; idx += 256) {
    float x[8], y[8];
    unpack8_f16(*reinterpret_cast<const uint4*>(DHt + idx * 16), x);
    unpack8_f16(*reinterpret_cast<const uint4*>(Ht + idx * 16), y);
#pragma unroll
    for (int i = 0; i < 8; ++i) dhh += x[i] * y[i];
  }
  dhh = cta_sum256(dhh, tid, tmp + 2) * __expf(Glast);
  wait_products(bar_mma, ph, ctl, 412);
  if (tq >= 64) {
    const int r = tq - 64;
    const float de = decs[r];
    float t3 = 0.f, dde = 0.f;
    __nv_bfloat16* dv_g = p.dv + (tok0 + static_cast<size_t>(r) * p.H) * V;
#pragma unroll
    for (int jj = 0; jj < V / 64; ++jj) {
      const int jb = half * (V / 64) + jj;
      float d[32], d1[32];
      tmem_ld32(g1A + lane_base + jb * 32, d);
      tmem_ld32(g1D + lane_base + jb * 32, d1);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float vn[8];
        unpack8_f16(tile_ld_chunk(VN, r, jb * 4 + i, 64), vn);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float kd_dh = de * d1[8 * i + e];            // (k dec_end) dh
          t3 += vn[e] * d[8 * i + e];
          dde += vn[e] * kd_dh;
          d[8 * i + e] += kd_dh;
        }
        const uint4 pk = pack8_f16(d + 8 * i);
        tile_st_chunk(DD, 64 + r, jb * 4 + i, 128, pk);
        if (!DELTA) *reinterpret_cast<uint4*>(dv_g + jb * 32 + 8 * i) = pack8_bf16(d + 8 * i);
      }
    }
    t3p[half * 64 + r] = t3 + dde;
    ddep[half * 64 + r] = dde;
  } else {
    const int r = tq;
    float d[32];
    tmem_ld32(g1C + lane_base + half * 32, d);
    tmem_ld_wait();
    const float Gr = Gs[r];
    float t2 = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int s8 = half * 4 + q;
      float a[8], y[8];
      unpack8_f16(tile_ld_chunk(AT, r, s8, 64), a);          // A[r, s] (already holds scale * ratio)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int s = s8 * 8 + i;
        const float da = (s <= r) ? d[q * 8 + i] : 0.f;
        t2 += da * a[i];
        y[i] = (s <= r) ? p.scale * __expf(Gr - Gs[s]) * da : 0.f;
      }
      tile_st_chunk(DS, r, s8, 64, pack8_f16(y));
    }
    t2p[half * 64 + r] = t2;
  }
  sync_for_issue();

  // ---- group 2a: cB = [do; dv2] h^T;  cA2 = dAr k (lanes 0-63: dq_intra)
  if (warp == 0 || warp == 4) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    if (warp == 0) {
      issue_product_led(leader, cB, Tile{smem_u32(DD), 128, false}, Tile{smem_u32(Ht), 128, false}, 128, V, 0u);
    } else {
      issue_product_led(leader, cA2, Tile{smem_u32(DS), 64, false}, Tile{smem_u32(KT), 64, true}, 128, 64, 0u);
    }
    umma_commit_led(leader, bar_mma);
    if (DELTA && tid == 0) {   // dv2 record: rows 64-127 of each DD atom are one atom of the 64-row image
      unsigned char* dv2_g = p.scratch + p.lay.dv2 + static_cast<size_t>(z) * p.lay.sz_dv2;
      for (int a = 0; a < V / 64; ++a) bulk_s2g(dv2_g + a * 8192, DD + a * 16384 + 8192, 8192);
      bulk_commit();
    }
  }
  wait_products(bar_mma, ph, ctl, 413);
  // The operand tiles of this group are dead now: dq and dw are staged in them as the images their
  // consumers read and leave by tensor-map / bulk stores.
  if (tid == 0) bulk_wait_read();
  __syncthreads();
  unsigned char* SQ = KT;            // dq, bf16 64 x 128 (two atoms)
  unsigned char* SW = DD;            // dw, fp16 64 x 128
  if (tq < 64) {
    const int r = tq;
    const float sg = p.scale * __expf(Gs[r]);
    float t1 = 0.f;
#pragma unroll 1
    for (int jb = 2 * half; jb < 2 * half + 2; ++jb) {
      float dqg[32], dqi[32];
      tmem_ld32(cB + lane_base + jb * 32, dqg);
      tmem_ld32(cA2 + lane_base + jb * 32, dqi);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float qv[8], o8[8];
        unpack8_f16(tile_ld_chunk(QT, r, jb * 4 + i, 64), qv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float a = sg * dqg[8 * i + e];
          t1 += a * qv[e];
          o8[e] = a + dqi[8 * i + e];
        }
        tile_st_chunk(SQ, r, jb * 4 + i, 64, pack8_out(o8, p.qk16));
      }
    }
    t1p[half * 64 + r] = t1;
  } else if (DELTA) {
    const int r = tq - 64;
#pragma unroll 1
    for (int jb = 2 * half; jb < 2 * half + 2; ++jb) {
      float d[32];
      tmem_ld32(cB + lane_base + jb * 32, d);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) d[e] = -d[e];
#pragma unroll
      for (int i = 0; i < 4; ++i) tile_st_chunk(SW, r, jb * 4 + i, 64, pack8_f16(d + 8 * i));
    }
  }
  sync_for_issue();

  // ---- group 2b: cD1 = dAr^T q;  cD2 = v_new dh^T  (lanes 0-63)
  if (warp == 0 || warp == 4) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    if (warp == 0) {
      issue_product_led(leader, cD1, Tile{smem_u32(DS), 64, true}, Tile{smem_u32(QT), 64, true}, 128, 64, 0u);
    } else {
      issue_product_led(leader, cD2, Tile{smem_u32(VN), 64, false}, Tile{smem_u32(DHt), 128, false}, 128, V, 0u);
    }
    umma_commit_led(leader, bar_mma);
    if (tid == 0) {
      for (int a = 0; a < 2; ++a) tma_store_4d(&mdq, SQ + a * 8192, a * 64, h, c * kC, b);
      if (DELTA) bulk_s2g(p.scratch + p.lay.dw + static_cast<size_t>(z) * p.lay.sz_dw, SW, 16384);
      bulk_commit();
    }
  }
  wait_products(bar_mma, ph, ctl, 414);
  __syncthreads();                   // every thread is past the products: h / dh become the dk staging tile
  unsigned char* SK = Ht;            // delta: fp32 dk partial, 32 KB (runs on into dh); else dk bf16
  if (tq < 64) {
    const int r = tq;
    const float de = decs[r];
    // fp32 dk partial for the WY kernel: four 32-column blocks of [row][eight 16-byte pieces], piece c
    // of row r stored at c ^ (r & 7), so that the record can be read back from shared memory row-wise
    float* dkb_s = reinterpret_cast<float*>(SK) + r * 32;
#pragma unroll 1
    for (int jb = 2 * half; jb < 2 * half + 2; ++jb) {
      float dkv[32], dkd[32];
      tmem_ld32(cD1 + lane_base + jb * 32, dkv);
      tmem_ld32(cD2 + lane_base + jb * 32, dkd);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) dkv[e] += de * dkd[e];
      if (DELTA) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<float4*>(dkb_s + jb * 2048 + 4 * (i ^ (r & 7))) =
              make_float4(dkv[4 * i], dkv[4 * i + 1], dkv[4 * i + 2], dkv[4 * i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) tile_st_chunk(SK, r, jb * 4 + i, 64, pack8_out(dkv + 8 * i, p.qk16));
      }
    }
  }
  fence_proxy_async();
  __syncthreads();
  if (tid == 0) {
    if (DELTA) {
      bulk_s2g(p.scratch + p.lay.dkb + static_cast<size_t>(z) * p.lay.sz_dkb, SK, 32768);
    } else {
      for (int a = 0; a < 2; ++a) tma_store_4d(&mdk, SK + a * 8192, a * 64, h, c * kC, b);
    }
    bulk_commit();
  }
  // ---- Stage-B gate gradient of the chunk (before the reverse cumulative sum)
  float dG = 0.f;
  {
    float sdde = (tid < 64) ? ddep[tid] + ddep[64 + tid] : 0.f;   // sum over the chunk's rows, fixed tree
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sdde += __shfl_xor_sync(0xffffffffu, sdde, o);
    if (tid == 0 || tid == 32) tmp[12 + (tid >> 5)] = sdde;
  }
  __syncthreads();
  if (tid < 64) {
    dG = (t1p[tid] + t1p[64 + tid]) + (t2p[tid] + t2p[64 + tid]) - (t3p[tid] + t3p[64 + tid]);
    if (tid == 63) dG += dhh + (tmp[12] + tmp[13]);
    if (DELTA) reinterpret_cast<float*>(p.scratch + p.lay.dgb + static_cast<size_t>(z) * p.lay.sz_dgb)[tid] = dG;
  }
  if (!DELTA) {
    const float acc = chunk_rev_cumsum(dG, tid, tmp);
    if (tid < 64 && p.gate == LETHE_GATE_SCALAR) p.dg[tok0 + static_cast<size_t>(tid) * p.H] = acc;
  }
  if (tid == 0) bulk_wait_read();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kCols);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <int V, bool DELTA, bool CW>
static int launch_pre_t(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mdo, cudaStream_t st) {
  const int smem = 16384 * 3 + V * 256 + 128 * 4 + 1024;
  static SmemAttr attr;
  if (attr.set(bwd_pre_kernel<V, DELTA, CW>, smem)) return kErrLaunch;
  bwd_pre_kernel<V, DELTA, CW><<<p.nbh * p.cn, 128, smem, st>>>(p, mq, mdo);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
template <int V, bool DELTA>
static int launch_stageb_t(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mdo,
                           const OutMaps& mo, cudaStream_t st) {
  const int smem = 16384 + 16384 + V * 256 + 8192 + 8192 + V * 128 + V * 256 * 2 + 656 * 4 +
                   static_cast<int>(sizeof(CtaShared)) + 1024;
  static SmemAttr attr;
  if (attr.set(bwd_stageb_kernel<V, DELTA>, smem)) return kErrLaunch;
  if (launch_dependent(bwd_stageb_kernel<V, DELTA>, dim3(p.nbh * p.cn), dim3(256), smem, st, p, mq, mk, mdo,
                       mo.dq, mo.dk) != cudaSuccess) return kErrLaunch;
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
int launch_bwd_pre(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mdo, cudaStream_t st) {
  if (p.gate == LETHE_GATE_CHANNEL) {
    if (p.V == 64) return p.delta ? launch_pre_t<64, true, true>(p, mq, mdo, st) : launch_pre_t<64, false, true>(p, mq, mdo, st);
    return p.delta ? launch_pre_t<128, true, true>(p, mq, mdo, st) : launch_pre_t<128, false, true>(p, mq, mdo, st);
  }
  if (p.V == 64) return p.delta ? launch_pre_t<64, true, false>(p, mq, mdo, st) : launch_pre_t<64, false, false>(p, mq, mdo, st);
  return p.delta ? launch_pre_t<128, true, false>(p, mq, mdo, st) : launch_pre_t<128, false, false>(p, mq, mdo, st);
}

int launch_bwd_wy(const Problem& p, const CUtensorMap& mk, const CUtensorMap& mv, const OutMaps& mo, cudaStream_t st);

// mask bit 4: Stage B, bit 8: WY VJP (delta variants only)
int launch_bwd_main(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                    const CUtensorMap& mdo, const OutMaps& mo, cudaStream_t st, uint32_t mask) {
  int e = kOk;
  if (mask & 4u) {
    if (p.V == 64) e = p.delta ? launch_stageb_t<64, true>(p, mq, mk, mdo, mo, st) : launch_stageb_t<64, false>(p, mq, mk, mdo, mo, st);
    else e = p.delta ? launch_stageb_t<128, true>(p, mq, mk, mdo, mo, st) : launch_stageb_t<128, false>(p, mq, mk, mdo, mo, st);
  }
  if (e || !p.delta || !(mask & 8u)) return e;
  return launch_bwd_wy(p, mk, mv, mo, st);
}

}  // namespace lg
