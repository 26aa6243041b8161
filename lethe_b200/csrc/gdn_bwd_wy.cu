// WY / triangular-inverse VJP for the scalar gate (reference K#2: gdn2_assemble.py:102-147), laid out
// so that two CTAs fit on one SM at d_v = 64 (256 TMEM columns, < 100 KB of shared memory).
//
// With T = (I + strict_lower(M))^-1, du = dv2, dw from Stage B:
//   dT  = du (beta v)^T + dw (beta gamma k)^T = [du v^T + dw (gamma k)^T] . beta_s      (column scale)
//   dM  = strict_lower(-T^T dT T^T),  dkk = dM . beta_i . ratio
//   dk  = (dkk + dkk^T) k + beta gamma . (T^T dw) + Stage-B part
//       = sym k + T'^T dw + DKB,     T'[l,i] = T[l,i] beta_i gamma_i     (one accumulator)
//   p_i = <(T^T dw)[i,:], k[i,:]> = sum_l T[l,i] (k dw^T)[i,l]           (no d x d_k read-back)
//   dv = beta . (T^T du),  dbeta = <T^T du, v> + gamma p + sum_s dM ratio KK,
//   dG = rowsum(e) - colsum(e) + beta p gamma,  e = dkk . KK,  dg = reverse cumsum (+ Stage-B part)
//
// Accumulators (TMEM columns): R0 [0,128) = [KK | k dw^T] (rows 0-63), later the dk accumulator;
// R1 [128,192) = dT, then X = dT T^T, then dM; R2 [192, 192+V) = T^T du.
#include "gdn_common.cuh"
#include "host_util.h"

namespace lg {

template <int V>
__global__ void __launch_bounds__(256)
bwd_wy2_kernel(const Problem p, const __grid_constant__ CUtensorMap mk, const __grid_constant__ CUtensorMap mv,
               const __grid_constant__ CUtensorMap mdk, const __grid_constant__ CUtensorMap mdv) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = align1024(smem_raw);
  unsigned char* T1 = sm;                       // 32 KB: rows 0-63 k, rows 64-127 dw
  unsigned char* GK = T1 + 32768;               // 16 KB: gamma k (64 x 128); later the fp32 transpose buffer
  unsigned char* TAt = GK + 16384;              // 16 KB: [T | A]
  unsigned char* TP = TAt + 16384;              // 8 KB: T'   (its second atom is W8: junk rows)
  unsigned char* W8 = TP + 8192;                // 8 KB: dT, then X, then dkk + dkk^T (over-reads run into DV2t)
  unsigned char* DV2t = W8 + 8192;              // du (64 x V)
  unsigned char* VT = DV2t + V * 128;           // v (64 x V) (+ 8 KB behind it for over-reads)
  float* fs = reinterpret_cast<float*>(VT + V * 128 + 8192);
  float* Gs = fs;          // [64]
  float* betas = fs + 64;  // [64]
  float* tmp = fs + 192;   // [8]
  float* bgs = fs + 200;   // [64] beta_i exp(G_i)
  float* prt = fs + 264;   // [2][5][64] per column half: pk, dbeta_m, rowsum_e, colsum_e, rv
  CtaShared* cs = reinterpret_cast<CtaShared*>(fs + 904);
  float* DK = reinterpret_cast<float*>(GK);    // fp32 [64][64], column XOR swizzle

  // Threads 0-127 and 128-255 reach the same TMEM lanes (lane quadrant = warp & 3): the two halves take
  // the same rows and split the columns of every epilogue; per-row sums are combined through `prt`.
  const int tid = threadIdx.x, warp = tid >> 5, tq = tid & 127, half = tid >> 7;
  const int bh = p.bh0 + blockIdx.x / p.cn, c = p.c0 + blockIdx.x % p.cn, z = bh * p.NT + c, b = bh / p.H, h = bh % p.H;
  CtaCtl ctl{p.status, &cs->abort_flag};
  uint64_t* bar_load = &cs->bar[0];
  uint64_t* bar_mma = &cs->bar[1];
  uint64_t* bar_dkb = &cs->bar[2];
  uint64_t* bar_g1 = &cs->bar[3];     // first product group: two issuing warps
  uint64_t* bar_post = &cs->bar[4];   // dw and du, loaded once Stage B before this kernel is complete
  constexpr uint32_t kCols = (V == 64) ? 256u : 512u;
  if (tid == 0) {
    cs->abort_flag = 0;
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    mbar_init(bar_dkb, 1);
    mbar_init(bar_g1, 2);
    mbar_init(bar_post, 1);
    fence_mbar_init();
    fence_proxy_async();
    mbar_expect_tx(bar_load, 16384u + V * 128u + 16384u);
    for (int a = 0; a < 2; ++a) tma_load_4d(T1 + a * 16384, &mk, bar_load, a * 64, h, c * kC, b);
    for (int a = 0; a < V / 64; ++a) tma_load_4d(VT + a * 8192, &mv, bar_load, a * 64, h, c * kC, b);
    bulk_g2s(TAt, p.saved + p.lay.ta + static_cast<size_t>(z) * p.lay.sz_ta, 16384, bar_load);
    // (dw, du and the Stage-B parts of dk and dG, written just before this kernel, come after griddep_wait)
  }
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, kCols);
    tmem_relinquish();
  }
  const size_t tok0 = (static_cast<size_t>(b) * p.L + c * kC) * p.H + h;
  float gval = 0.f, bval = 0.f, dgb = 0.f;
  if (tid < 64) {
    if (p.gate == LETHE_GATE_SCALAR) gval = p.g[tok0 + static_cast<size_t>(tid) * p.H];
    bval = p.beta[tok0 + static_cast<size_t>(tid) * p.H];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;
  const uint32_t R0 = tmem, R1 = tmem + 128, R2 = tmem + 192;
  const float G = chunk_cumsum(gval, tid, tmp);
  if (tid < 64) {
    Gs[tid] = G;
    betas[tid] = bval;
    bgs[tid] = bval * __expf(G);
  }
  __syncthreads();
  // the loads above fetch inputs and records older than Stage B; once Stage B is complete (at once, except
  // for the CTAs that started early) what it wrote is fetched too
  griddep_wait();
  griddep_launch();
  if (tid == 0) {
    mbar_expect_tx(bar_post, 16384u + V * 128u);
    for (int a = 0; a < 2; ++a)
      bulk_g2s(T1 + a * 16384 + 8192, p.scratch + p.lay.dw + static_cast<size_t>(z) * p.lay.sz_dw + a * 8192, 8192,
               bar_post);
    bulk_g2s(DV2t, p.scratch + p.lay.dv2 + static_cast<size_t>(z) * p.lay.sz_dv2, V * 128, bar_post);
  }
  if (tid < 64) dgb = reinterpret_cast<const float*>(p.scratch + p.lay.dgb + static_cast<size_t>(z) * p.lay.sz_dgb)[tid];
  mbar_wait_warp(bar_load, 0, ctl, 421);
  for (int idx = tid; idx < 64 * 16; idx += 256) {
    const int r = idx >> 4, ch = idx & 15;
    float x[8], y[8];
    unpack8_in(tile_ld_chunk(T1, r, ch, 128), x, p.qk16);
    tile_st_chunk(T1, r, ch, 128, pack8_f16(x));
    const float ga = __expf(Gs[r]);
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = x[i] * ga;
    tile_st_chunk(GK, r, ch, 64, pack8_f16(y));
    if (ch < 8) {   // T'[l, i] = T[l, i] beta_i gamma_i  (row l = r, columns 8 ch .. 8 ch + 7)
      float t[8];
      unpack8_f16(tile_ld_chunk(TAt, r, ch, 128), t);
#pragma unroll
      for (int i = 0; i < 8; ++i) t[i] *= bgs[ch * 8 + i];
      tile_st_chunk(TP, r, ch, 64, pack8_f16(t));
    }
  }
  for (int idx = tid; idx < 64 * (V / 8); idx += 256) {
    const int r = idx / (V / 8), ch = idx % (V / 8);
    float x[8];
    unpack8_bf16(tile_ld_chunk(VT, r, ch, 64), x);
    tile_st_chunk(VT, r, ch, 64, pack8_f16(x));
  }
  sync_for_issue();
  mbar_wait_warp(bar_post, 0, ctl, 427);

  uint32_t ph = 0;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  // ---- group 1: [KK | k dw^T], dT / beta_s, T^T du
  // (24 products: two warps issue half each, issuing is what the group costs)
  if (warp == 0 || warp == 4) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    if (warp == 0) {
      issue_product_led(leader, R0, Tile{smem_u32(T1), 128, false}, Tile{smem_u32(T1), 128, false}, 128, 128, 0u);
      issue_product_led(leader, R2, Tile{smem_u32(TAt), 64, true}, Tile{smem_u32(DV2t), 64, true}, V, 64, 0u);
    } else {
      issue_product_led(leader, R1, Tile{smem_u32(DV2t), 64, false}, Tile{smem_u32(VT), 64, false}, 64, V, 0u);
      issue_product_led(leader, R1, Tile{smem_u32(T1) + 8192, 128, false}, Tile{smem_u32(GK), 64, false}, 64, 128, 1u);
    }
    umma_commit_led(leader, bar_g1);
  }
  {
    uint32_t ph1 = 0;
    wait_products(bar_g1, ph1, ctl, 422);
  }
  const int c0 = half * 32;           // this half's 32 columns of every 64-column accumulator
  const bool live = (half == 0) || ((warp & 1) != 0);   // rows 0-31 have nothing right of column 31 in a triangle
  float pk = 0.f;
  if (tq < 64) {
    float d[32];
    tmem_ld32(R1 + lane_base + c0, d);
    tmem_ld_wait();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = d[q * 8 + i] * betas[c0 + q * 8 + i];
      tile_st_chunk(W8, tq, half * 4 + q, 64, pack8_f16(y));
    }
    // p_i = sum_l T[l, i] (k dw^T)[i, l]
    tmem_ld32(R0 + 64 + lane_base + c0, d);
    tmem_ld_wait();
#pragma unroll
    for (int l = 0; l < 32; ++l)
      pk += d[l] * __half2float(*reinterpret_cast<const __half*>(TAt + sw128_off(c0 + l, tq, 128)));
    prt[(half * 5 + 0) * 64 + tq] = pk;
  }
  sync_for_issue();
  // ---- group 2: X = dT T^T
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, R1, Tile{smem_u32(W8), 64, false}, Tile{smem_u32(TAt), 128, false}, 64, 64, 0u);
    umma_commit_led(leader, bar_mma);
  }
  wait_products(bar_mma, ph, ctl, 423);
  if (tq < 64) {
    float d[32];
    tmem_ld32(R1 + lane_base + c0, d);
    tmem_ld_wait();
#pragma unroll
    for (int q = 0; q < 4; ++q) tile_st_chunk(W8, tq, half * 4 + q, 64, pack8_f16(d + 8 * q));
  }
  sync_for_issue();
  // ---- group 3: dM = -T^T X
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, R1, Tile{smem_u32(TAt), 64, true}, Tile{smem_u32(W8), 64, true}, 64, 64, 0u, true);
    umma_commit_led(leader, bar_mma);
  }
  wait_products(bar_mma, ph, ctl, 424);
  float kk[32];
  if (tq < 64) {
    const int r = tq;
    float rowsum_e = 0.f, dbeta_m = 0.f;
    float dm[32];
    if (live) {
      tmem_ld32(R1 + lane_base + c0, dm);
      tmem_ld32(R0 + lane_base + c0, kk);
      tmem_ld_wait();
    }
    const float Gr = Gs[r], bval_r = betas[r];
    // the gate values of this thread's 32 columns go to registers first: a shared-memory load the
    // compiler cannot tell apart from the stores below would wait for the store before it in every
    // iteration and serialise the loop at the load latency
    float gcol[32];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 g4 = *reinterpret_cast<const float4*>(Gs + c0 + 4 * q);
      gcol[4 * q] = g4.x; gcol[4 * q + 1] = g4.y; gcol[4 * q + 2] = g4.z; gcol[4 * q + 3] = g4.w;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int s = c0 + j;
      float dkk = 0.f;
      if (live) {
        const float x = (s < r) ? dm[j] * __expf(Gr - gcol[j]) : 0.f;      // dM * ratio, strictly lower
        dbeta_m += x * kk[j];
        dkk = x * bval_r;
        rowsum_e += dkk * kk[j];
      }
      DK[r * 64 + (s ^ (r & 31))] = dkk;
    }
    prt[(half * 5 + 1) * 64 + r] = dbeta_m;
    prt[(half * 5 + 2) * 64 + r] = rowsum_e;
  }
  __syncthreads();
  if (tq < 64) {
    const int r = tq;
    float colsum_e = 0.f;
    // column sums need KK[s, r] = KK[r, s] for s > r: rows 32-63 of the lower half's columns are not
    // loaded above (cut), so take them from the symmetric entry only where this thread holds it
    if (!live) {
      tmem_ld32(R0 + lane_base + c0, kk);
      tmem_ld_wait();
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int s = c0 + q * 8 + i;
        const float up = DK[s * 64 + (r ^ (s & 31))];          // dkk[s, r], non-zero for s > r
        y[i] = DK[r * 64 + (s ^ (r & 31))] + up;
        colsum_e += up * kk[q * 8 + i];                        // KK is symmetric
      }
      tile_st_chunk(W8, r, half * 4 + q, 64, pack8_f16(y));
    }
    prt[(half * 5 + 3) * 64 + r] = colsum_e;
  }
  sync_for_issue();
  // ---- group 4: dk accumulator = (dkk + dkk^T) k + T'^T dw
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, R0, Tile{smem_u32(W8), 64, false}, Tile{smem_u32(T1), 128, true}, 128, 64, 0u);
    issue_product_led(leader, R0, Tile{smem_u32(TP), 64, true}, Tile{smem_u32(T1) + 8192, 128, true}, 128, 64, 1u);
    umma_commit_led(leader, bar_mma);
    // Stage B's fp32 dk partial lands in the two tiles nothing reads any more (GK / DK and [T | A])
    if (tid == 0) {
      mbar_expect_tx(bar_dkb, 32768u);
      bulk_g2s(GK, p.scratch + p.lay.dkb + static_cast<size_t>(z) * p.lay.sz_dkb, 32768u, bar_dkb);
    }
  }
  wait_products(bar_mma, ph, ctl, 425);
  // [k; dw] is dead once the last products are done: dk and dv are staged there as bf16 tiles and
  // leave by tensor-map stores
  unsigned char* SKo = T1;            // dk: 64 x 128, two atoms
  unsigned char* SV = T1 + 16384;     // dv: 64 x V
  if (tq < 64) {
    const int r = tq;
    const float bval_r = betas[r];
    float rv = 0.f;
#pragma unroll
    for (int jj = 0; jj < V / 64; ++jj) {
      const int jb = half * (V / 64) + jj;
      float d[32];
      tmem_ld32(R2 + lane_base + jb * 32, d);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float vv[8], o8[8];
        unpack8_f16(tile_ld_chunk(VT, r, jb * 4 + i, 64), vv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          rv += d[8 * i + e] * vv[e];
          o8[e] = bval_r * d[8 * i + e];
        }
        tile_st_chunk(SV, r, jb * 4 + i, 64, pack8_bf16(o8));
      }
    }
    prt[(half * 5 + 4) * 64 + r] = rv;
    const float* dkb_s = reinterpret_cast<const float*>(GK) + r * 32;
    mbar_wait_warp(bar_dkb, 0, ctl, 426);
#pragma unroll 1
    for (int jb = 2 * half; jb < 2 * half + 2; ++jb) {
      float sk[32];
      tmem_ld32(R0 + lane_base + jb * 32, sk);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 b0 = *reinterpret_cast<const float4*>(dkb_s + jb * 2048 + 4 * ((2 * i) ^ (r & 7)));
        const float4 b1 = *reinterpret_cast<const float4*>(dkb_s + jb * 2048 + 4 * ((2 * i + 1) ^ (r & 7)));
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        float o8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o8[e] = bb[e] + sk[8 * i + e];
        tile_st_chunk(SKo, r, jb * 4 + i, 64, pack8_out(o8, p.qk16));
      }
    }
  }
  fence_proxy_async();
  __syncthreads();
  if (tid == 0) {
    for (int a = 0; a < 2; ++a) tma_store_4d(&mdk, SKo + a * 8192, a * 64, h, c * kC, b);
    for (int a = 0; a < V / 64; ++a) tma_store_4d(&mdv, SV + a * 8192, a * 64, h, c * kC, b);
    bulk_commit();
  }
  float dgv = 0.f;
  if (tid < 64) {
    const int r = tid;
    const float gam = __expf(Gs[r]);
    const float pks = prt[0 * 64 + r] + prt[5 * 64 + r];
    const float dbm = prt[1 * 64 + r] + prt[6 * 64 + r];
    const float rse = prt[2 * 64 + r] + prt[7 * 64 + r];
    const float cse = prt[3 * 64 + r] + prt[8 * 64 + r];
    const float rvs = prt[4 * 64 + r] + prt[9 * 64 + r];
    if (p.dbeta_w) {
      p.dbeta_w[tok0 + static_cast<size_t>(r) * p.H] = rvs;
      p.dbeta[tok0 + static_cast<size_t>(r) * p.H] = gam * pks + dbm;
    } else {
      p.dbeta[tok0 + static_cast<size_t>(r) * p.H] = rvs + gam * pks + dbm;
    }
    dgv = dgb + rse - cse + bval * pks * gam;
  }
  {
    const float acc = chunk_rev_cumsum(dgv, tid, tmp);
    if (tid < 64 && p.gate == LETHE_GATE_SCALAR) p.dg[tok0 + static_cast<size_t>(tid) * p.H] = acc;
  }
  if (tid == 0) bulk_wait_read();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kCols);
}

template <int V>
static int launch_wy2_t(const Problem& p, const CUtensorMap& mk, const CUtensorMap& mv, const OutMaps& mo,
                        cudaStream_t st) {
  const int smem = 32768 + 16384 + 16384 + 8192 + 8192 + V * 256 + 8192 + 904 * 4 + static_cast<int>(sizeof(CtaShared)) + 1024;
  static SmemAttr attr;
  if (attr.set(bwd_wy2_kernel<V>, smem)) return kErrLaunch;
  if (launch_dependent(bwd_wy2_kernel<V>, dim3(p.nbh * p.cn), dim3(256), smem, st, p, mk, mv, mo.dk, mo.dv) !=
      cudaSuccess) return kErrLaunch;
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

int launch_bwd_wy(const Problem& p, const CUtensorMap& mk, const CUtensorMap& mv, const OutMaps& mo, cudaStream_t st) {
  return p.V == 64 ? launch_wy2_t<64>(p, mk, mv, mo, st) : launch_wy2_t<128>(p, mk, mv, mo, st);
}

}  // namespace lg
