// Channel-wise gate: chunk-parallel backward kernels (after the adjoint state scan).
//
//   bwd_cw_sb1  : dv2, dA, dw and the parts of dq, dk and of the gate gradient that are plain
//                 products followed by per-element decays
//   bwd_cw_wy1  : WY / triangular-inverse VJP up to dM; dv, the value part of dbeta, d(beta gamma k)
//   bwd_cw_pair : the decay-coupled pair sums
//                     out1[i,d] = sum_{s<=i} C[i,s] k[s,d] exp(G_i,d - G_s,d)
//                     out2[s,d] = sum_{i>=s} C[i,s] x[i,d] exp(G_i,d - G_s,d)
//                 with (C, x) = (scale dA, q) for Stage B and (dM, beta k) for the WY VJP, and the
//                 final assembly of dq / dk / dbeta / dg.
//
// Reference: closed channel-wise Stage B gdn2_assemble.py:521-585, channel-wise K#2
// gdn2_assemble.py:407-473 (its two decay einsums are `out1` / `out2` here), the SIMT kernel
// gdn2_sb_einsum.py:44-76 that the reference uses for them.
//
// The pair sums use the 16-row block scheme of the forward (gdn_cw_fwd.cu): blocks strictly below
// the diagonal go through tcgen05 with both decay factors <= 1 (reference row 16 I for out1, last
// row of the source block for out2), the four diagonal blocks are summed exactly on the CUDA cores.
#include "gdn_common.cuh"
#include "host_util.h"

namespace lg {

// fp32 [64][128] records passed between the backward kernels (dq / dk / dG parts): element (i, d) of
// a record lives at ridx(i, d) - the 16-byte pieces of a row are XOR-ed with the low row bits, so that
// a shared-memory image of the record takes row-wise 16-byte stores and column-wise reads without
// bank conflicts, and global accesses by 128 threads along d stay coalesced.
__device__ __forceinline__ int ridx(int i, int d) { return i * kK + (d ^ ((i & 7) << 2)); }

// Four neighbouring channels [4 c4, 4 c4 + 4) of row `row` of an exchange tile (layout exi): they share one
// aligned 16-byte piece, in which channel e sits at position e ^ (row & 3).
__device__ __forceinline__ void ex_perm4(float* a, int row) {
  if (row & 1) {
    float t = a[0]; a[0] = a[1]; a[1] = t;
    t = a[2]; a[2] = a[3]; a[3] = t;
  }
  if (row & 2) {
    float t = a[0]; a[0] = a[2]; a[2] = t;
    t = a[1]; a[1] = a[3]; a[3] = t;
  }
}
__device__ __forceinline__ void ex_ld4(const float* T, int row, int c4, float* out) {
  const float4 v = *reinterpret_cast<const float4*>(T + row * kK + 4 * (c4 ^ ((row & 31) >> 2)));
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  ex_perm4(out, row);
}
__device__ __forceinline__ void ex_st4(float* T, int row, int c4, const float* in) {
  float a[4] = {in[0], in[1], in[2], in[3]};
  ex_perm4(a, row);
  *reinterpret_cast<float4*>(T + row * kK + 4 * (c4 ^ ((row & 31) >> 2))) = make_float4(a[0], a[1], a[2], a[3]);
}
__device__ __forceinline__ void unpack4_f16(const uint2& u, float* v) {
  const __half2* h = reinterpret_cast<const __half2*>(&u);
  const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
// four 16-bit results (bf16, or fp16 when the call runs with fp16 q, k) as one 8-byte store
__device__ __forceinline__ void store_out16x4(__nv_bfloat16* dst, const float* x, int f16) {
  uint2 u;
  if (f16) {
    __half2* h = reinterpret_cast<__half2*>(&u);
    h[0] = __floats2half2_rn(x[0], x[1]);
    h[1] = __floats2half2_rn(x[2], x[3]);
  } else {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
    h[0] = __floats2bfloat162_rn(x[0], x[1]);
    h[1] = __floats2bfloat162_rn(x[2], x[3]);
  }
  *reinterpret_cast<uint2*>(dst) = u;
}


// ---------------------------------------------------------------------------------------------
// Stage B, part 1.  Accumulators: cA [0,128) dv2; cB [128,256) [do; dv2] h^T; cC [256,320) dA;
// cD [320,448) v_new dh^T.
// ---------------------------------------------------------------------------------------------
template <int V, bool DELTA>
__global__ void __launch_bounds__(256)
bwd_cw_sb1_kernel(const Problem p, const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                  const __grid_constant__ CUtensorMap mdo) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = align1024(smem_raw);
  unsigned char* X1 = sm;                       // 32 KB: rows 0-63 k, rows 64-127 kd
  unsigned char* QT = X1 + 32768;               // 16 KB: q
  unsigned char* DD = QT + 16384;               // V*256: rows 0-63 do, rows 64-127 dv2
  unsigned char* TAt = DD + V * 256;            // 16 KB
  unsigned char* VNt = TAt + 16384;             // V*128: v_new (64 rows); over-reads run into Ht
  unsigned char* Ht = VNt + V * 128;            // V*256
  unsigned char* DHt = Ht + V * 256;            // V*256
  float* Gt = reinterpret_cast<float*>(DHt + V * 256);    // 32 KB
  float* fs = Gt + 64 * kK;
  float* hh = fs;                // [128] exp(G_last) <dh, h> per channel
  CtaShared* cs = reinterpret_cast<CtaShared*>(fs + 128);
  float* DDE = reinterpret_cast<float*>(Ht);   // [64][128] fp32 exchange tile, after the products are done

  const int tid = threadIdx.x, warp = tid >> 5;
  const int bh = p.bh0 + blockIdx.x / p.cn, c = p.c0 + blockIdx.x % p.cn, z = bh * p.NT + c, b = bh / p.H, h = bh % p.H;
  CtaCtl ctl{p.status, &cs->abort_flag};
  uint64_t* bar_load = &cs->bar[0];
  uint64_t* bar_mma = &cs->bar[1];
  uint64_t* bar_dh = &cs->bar[2];       // dh, loaded once the adjoint scan before this kernel is complete
  if (tid == 0) {
    cs->abort_flag = 0;
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    mbar_init(bar_dh, 1);
    fence_mbar_init();
    fence_proxy_async();
    // every load that does not depend on the kernel just before this one is requested at once
    mbar_expect_tx(bar_load, 16384u + 16384u + V * 128u + 16384u + V * 128u + V * 256u + 32768u);
    bulk_g2s(Gt, p.saved + p.lay.gt + static_cast<size_t>(z) * (kC * kK * 4), 32768, bar_load);
    for (int a = 0; a < 2; ++a) {
      tma_load_4d(X1 + a * 16384, &mk, bar_load, a * 64, h, c * kC, b);
      tma_load_4d(QT + a * 8192, &mq, bar_load, a * 64, h, c * kC, b);
    }
    for (int a = 0; a < V / 64; ++a) tma_load_4d(DD + a * 16384, &mdo, bar_load, a * 64, h, c * kC, b);
    bulk_g2s(VNt, p.saved + p.lay.vn + static_cast<size_t>(z) * p.lay.sz_vn, V * 128, bar_load);
    bulk_g2s(TAt, p.saved + p.lay.ta + static_cast<size_t>(z) * p.lay.sz_ta, 16384, bar_load);
    bulk_g2s(Ht, p.saved + p.lay.hc + static_cast<size_t>(z + bh) * p.lay.sz_hc, V * 256, bar_load);
    // (dh, written by the adjoint scan just before this kernel, is loaded after griddep_wait)
  }
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, 512);
    tmem_relinquish();
  }
  const size_t tok0 = (static_cast<size_t>(b) * p.L + c * kC) * p.H + h;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;
  const uint32_t cA = tmem, cB = tmem + 128, cC = tmem + 256, cD = tmem + 320;
  __syncthreads();
  // the loads above fetch inputs and records older than the adjoint scan; once it is complete (at once,
  // except for the CTAs that started early) its dh image is fetched too
  griddep_wait();
  griddep_launch();
  if (tid == 0) {
    mbar_expect_tx(bar_dh, V * 256u);
    bulk_g2s(DHt, p.scratch + p.lay.dh + static_cast<size_t>(z) * p.lay.sz_dh, V * 256, bar_dh);
  }
  mbar_wait_warp(bar_load, 0, ctl, 601);
  for (int idx = tid; idx < 64 * 16; idx += 256) {
    const int r = idx >> 4, ch = idx & 15;
    float x[8], y[8];
    unpack8_in(tile_ld_chunk(X1, r, ch, 128), x, p.qk16);
    tile_st_chunk(X1, r, ch, 128, pack8_f16(x));
    float gl8[8], gr8[8];
    gt8(Gt, 63, ch * 8, gl8);
    gt8(Gt, r, ch * 8, gr8);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = x[e] * exp2f(gl8[e] - gr8[e]);
    tile_st_chunk(X1, 64 + r, ch, 128, pack8_f16(y));
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
  mbar_wait_warp(bar_dh, 0, ctl, 604);

  uint32_t ph = 0;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, cA, Tile{smem_u32(X1), 128, false}, Tile{smem_u32(DHt), 128, true}, V, 128, 0u);
    issue_product_led(leader, cA, Tile{smem_u32(TAt), 64, true}, Tile{smem_u32(DD), 128, true}, V, 64, 1u);
    issue_product_led(leader, cC, Tile{smem_u32(DD), 128, false}, Tile{smem_u32(VNt), 64, false}, 64, V, 0u);
    umma_commit_led(leader, bar_mma);
  }
  // in the shadow of the products (both images are only read)
  if (tid < 128) {  // exp(G_last,d) sum_v dh[d,v] h[d,v]: thread d owns row d of both images
    float acc = 0.f;
#pragma unroll
    for (int ch = 0; ch < V / 8; ++ch) {
      float x[8], y[8];
      unpack8_f16(tile_ld_chunk(DHt, tid, ch, 128), x);
      unpack8_f16(tile_ld_chunk(Ht, tid, ch, 128), y);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += x[e] * y[e];
    }
    hh[tid] = acc * exp2f(Gt[gidx(63, tid)]);
  }
  wait_products(bar_mma, ph, ctl, 602);
  if (tid >= 64 && tid < 128) {
    const int r = tid - 64;
    unsigned char* dv2_g = p.scratch + p.lay.dv2 + static_cast<size_t>(z) * p.lay.sz_dv2;
    __nv_bfloat16* dv_g = p.dv + (tok0 + static_cast<size_t>(r) * p.H) * V;
#pragma unroll
    for (int jb = 0; jb < V / 32; ++jb) {
      float d[32];
      tmem_ld32(cA + lane_base + jb * 32, d);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 pk = pack8_f16(d + 8 * i);
        tile_st_chunk(DD, 64 + r, jb * 4 + i, 128, pk);
        if (DELTA) *reinterpret_cast<uint4*>(dv2_g + sw128_chunk(r, jb * 4 + i, 64)) = pk;
        else *reinterpret_cast<uint4*>(dv_g + jb * 32 + 8 * i) = pack8_bf16(d + 8 * i);
      }
    }
  } else if (tid < 64) {
    const int r = tid;
    float d[64];
    tmem_ld32(cC + lane_base, d);
    tmem_ld32(cC + lane_base + 32, d + 32);
    tmem_ld_wait();
    unsigned char* da_g = p.scratch + p.lay.da + static_cast<size_t>(z) * 8192;
#pragma unroll
    for (int s8 = 0; s8 < 8; ++s8) {
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = (s8 * 8 + i <= r) ? p.scale * d[s8 * 8 + i] : 0.f;
      *reinterpret_cast<uint4*>(da_g + sw128_chunk(r, s8, 64)) = pack8_f16(y);
    }
  }
  sync_for_issue();
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, cB, Tile{smem_u32(DD), 128, false}, Tile{smem_u32(Ht), 128, false}, 128, V, 0u);
    issue_product_led(leader, cD, Tile{smem_u32(VNt), 64, false}, Tile{smem_u32(DHt), 128, false}, 128, V, 0u);
    umma_commit_led(leader, bar_mma);
  }
  wait_products(bar_mma, ph, ctl, 603);
  __syncthreads();          // every thread is past the products: Ht / DHt may be overwritten (DDE)
  float* dqp_g = reinterpret_cast<float*>(p.scratch + p.lay.dqp + static_cast<size_t>(z) * (kC * kK * 4));
  float* dkb_g = reinterpret_cast<float*>(p.scratch + p.lay.dkb + static_cast<size_t>(z) * p.lay.sz_dkb);
  float* dgb_g = reinterpret_cast<float*>(p.scratch + p.lay.dgb + static_cast<size_t>(z) * p.lay.sz_dgb);
  // With d_v = 128 three dead operand tiles hold the three records as images that leave by bulk
  // stores; with d_v = 64 there is no room and the rows go to global memory directly.
  constexpr bool kStage = (V == 128);
  float* dqp_w = kStage ? reinterpret_cast<float*>(DD) : dqp_g;
  float* dkb_w = kStage ? reinterpret_cast<float*>(TAt) : dkb_g;     // [T | A] and v_new, contiguous
  float* dgb_w = kStage ? reinterpret_cast<float*>(DHt) : dgb_g;
  const int tq = tid & 127, jb0 = 2 * (tid >> 7);   // threads 128-255 take the upper 64 columns
  if (tq < 64) {
    const int r = tq;
#pragma unroll 1
    for (int jb = jb0; jb < jb0 + 2; ++jb) {
      float dqg[32], dkd[32];
      tmem_ld32(cB + lane_base + jb * 32, dqg);
      tmem_ld32(cD + lane_base + jb * 32, dkd);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float qv[8], kv[8];
        unpack8_f16(tile_ld_chunk(QT, r, jb * 4 + i, 64), qv);
        unpack8_f16(tile_ld_chunk(X1, r, jb * 4 + i, 128), kv);
        float o1[8], o2[8], o3[8], g8[8], gl8[8];
        gt8(Gt, r, jb * 32 + i * 8, g8);
        gt8(Gt, 63, jb * 32 + i * 8, gl8);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int d = jb * 32 + i * 8 + e;
          const float g = g8[e];
          const float sg = p.scale * exp2f(g);
          const float de = exp2f(gl8[e] - g);
          o1[e] = sg * dqg[8 * i + e];                       // part of dq
          o2[e] = dkd[8 * i + e] * de;                       // part of dk
          const float dde = o2[e] * kv[e];
          DDE[exi(r, d)] = dde;
          o3[e] = o1[e] * qv[e] - dde;                       // part of dG
        }
        const int c0 = jb * 32 + i * 8;
        *reinterpret_cast<float4*>(dqp_w + ridx(r, c0)) = make_float4(o1[0], o1[1], o1[2], o1[3]);
        *reinterpret_cast<float4*>(dqp_w + ridx(r, c0 + 4)) = make_float4(o1[4], o1[5], o1[6], o1[7]);
        *reinterpret_cast<float4*>(dkb_w + ridx(r, c0)) = make_float4(o2[0], o2[1], o2[2], o2[3]);
        *reinterpret_cast<float4*>(dkb_w + ridx(r, c0 + 4)) = make_float4(o2[4], o2[5], o2[6], o2[7]);
        *reinterpret_cast<float4*>(dgb_w + ridx(r, c0)) = make_float4(o3[0], o3[1], o3[2], o3[3]);
        *reinterpret_cast<float4*>(dgb_w + ridx(r, c0 + 4)) = make_float4(o3[4], o3[5], o3[6], o3[7]);
      }
    }
  } else if (DELTA) {
    const int r = tq - 64;
    unsigned char* dw_g = p.scratch + p.lay.dw + static_cast<size_t>(z) * p.lay.sz_dw;
#pragma unroll 1
    for (int jb = jb0; jb < jb0 + 2; ++jb) {
      float d[32];
      tmem_ld32(cB + lane_base + jb * 32, d);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) d[e] = -d[e];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        *reinterpret_cast<uint4*>(dw_g + sw128_chunk(r, jb * 4 + i, 64)) = pack8_f16(d + 8 * i);
    }
  }
  __syncthreads();
  if (tid < 128) {  // last row of the chunk: exp(G_last) <dh, h> + sum_i dde[i, d]   (thread d, column d)
    float acc = hh[tid];
    for (int i = 0; i < 64; ++i) acc += DDE[exi(i, tid)];
    dgb_w[ridx(63, tid)] += acc;
  }
  if (kStage) {
    fence_proxy_async();
    __syncthreads();
    if (tid == 0) {
      bulk_s2g(dqp_g, dqp_w, 32768);
      bulk_s2g(dkb_g, dkb_w, 32768);
      bulk_s2g(dgb_g, dgb_w, 32768);
      bulk_commit();
      bulk_wait_read();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------
// WY VJP, part 1.  Accumulators: c1 [64,128) dT; c2 [128,192) X; c3 [192,256) dM;
// c4 [256, 256+V+128) [dbv | d(beta gamma k)].
// ---------------------------------------------------------------------------------------------
constexpr int kWy1Threads = 256;

template <int V>
__global__ void __launch_bounds__(kWy1Threads)
bwd_cw_wy1_kernel(const Problem p, const __grid_constant__ CUtensorMap mk, const __grid_constant__ CUtensorMap mv) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = align1024(smem_raw);
  unsigned char* KB = sm;                       // 32 KB: rows 0-63 k, rows 64-127 beta gamma k
  unsigned char* VT = KB + 32768;               // v
  unsigned char* BVt = VT + V * 128;            // beta v
  unsigned char* TAt = BVt + V * 128;           // 16 KB
  unsigned char* DV2t = TAt + 16384;            // dv2
  unsigned char* DWt = DV2t + V * 128;          // 16 KB dw
  unsigned char* DTt = DWt + 16384;             // 8 KB dT
  unsigned char* XT = DTt + 8192;               // 8 KB X (+ 8 KB padding behind it)
  float* Gt = reinterpret_cast<float*>(XT + 16384);
  float* fs = Gt + 64 * kK;
  float* betas = fs;
  float* part = fs + 64;                        // [2][64]: the second column half's share of the two row sums
  CtaShared* cs = reinterpret_cast<CtaShared*>(fs + 64 + 128);

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
    // every load that does not depend on the kernel just before this one is requested at once
    mbar_expect_tx(bar_load, 16384u + V * 128u + 16384u + V * 128u + 16384u + 32768u);
    bulk_g2s(Gt, p.saved + p.lay.gt + static_cast<size_t>(z) * (kC * kK * 4), 32768, bar_load);
    for (int a = 0; a < 2; ++a) tma_load_4d(KB + a * 16384, &mk, bar_load, a * 64, h, c * kC, b);
    for (int a = 0; a < V / 64; ++a) tma_load_4d(VT + a * 8192, &mv, bar_load, a * 64, h, c * kC, b);
    bulk_g2s(TAt, p.saved + p.lay.ta + static_cast<size_t>(z) * p.lay.sz_ta, 16384, bar_load);
    bulk_g2s(DV2t, p.scratch + p.lay.dv2 + static_cast<size_t>(z) * p.lay.sz_dv2, V * 128, bar_load);
    bulk_g2s(DWt, p.scratch + p.lay.dw + static_cast<size_t>(z) * p.lay.sz_dw, 16384, bar_load);
  }
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, 512);
    tmem_relinquish();
  }
  const size_t tok0 = (static_cast<size_t>(b) * p.L + c * kC) * p.H + h;
  // full op (per-channel erase gate b, write gate w): the gates enter element by element, beta is one
  const bool full = p.bch != nullptr;
  if (tid < 64) betas[tid] = full ? 1.f : p.beta[tok0 + static_cast<size_t>(tid) * p.H];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;
  const uint32_t c1 = tmem + 64, c2 = tmem + 128, c3 = tmem + 192, c4 = tmem + 256;
  __syncthreads();
  mbar_wait_warp(bar_load, 0, ctl, 611);
  for (int idx = tid; idx < 64 * 16; idx += kWy1Threads) {
    const int r = idx >> 4, ch = idx & 15;
    float x[8], y[8];
    unpack8_in(tile_ld_chunk(KB, r, ch, 128), x, p.qk16);
    tile_st_chunk(KB, r, ch, 128, pack8_f16(x));
    float bb[8];
    if (full) {
      ld8(p.bch + (tok0 + static_cast<size_t>(r) * p.H) * kK + ch * 8, bb);
    } else {
      const float be = betas[r];
#pragma unroll
      for (int e = 0; e < 8; ++e) bb[e] = be;
    }
    float gg[8];
    gt8(Gt, r, ch * 8, gg);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = x[e] * bb[e] * exp2f(gg[e]);
    tile_st_chunk(KB, 64 + r, ch, 128, pack8_f16(y));
  }
  for (int idx = tid; idx < 64 * (V / 8); idx += kWy1Threads) {
    const int r = idx / (V / 8), ch = idx % (V / 8);
    float x[8];
    unpack8_bf16(tile_ld_chunk(VT, r, ch, 64), x);
    tile_st_chunk(VT, r, ch, 64, pack8_f16(x));
    if (full) {
      float wv[8];
      ld8(p.wch + (tok0 + static_cast<size_t>(r) * p.H) * V + ch * 8, wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] *= wv[i];
    } else {
      const float be = betas[r];
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] *= be;
    }
    tile_st_chunk(BVt, r, ch, 64, pack8_f16(x));
  }
  sync_for_issue();
  uint32_t ph = 0;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, c1, Tile{smem_u32(DV2t), 64, false}, Tile{smem_u32(BVt), 64, false}, 64, V, 0u);
    issue_product_led(leader, c1, Tile{smem_u32(DWt), 64, false}, Tile{smem_u32(KB) + 8192, 128, false}, 64, 128, 1u);
    issue_product_led(leader, c4, Tile{smem_u32(TAt), 64, true}, Tile{smem_u32(DV2t), 64, true}, V + 128, 64, 0u);
    umma_commit_led(leader, bar_mma);
  }
  wait_products(bar_mma, ph, ctl, 612);
  // The accumulators have 64 rows (lanes 0-63): warps 0, 1, 4, 5 reach them, warp w and w + 4 the same
  // lanes, and split the columns of every epilogue between them.
  const bool owner = (warp & 3) < 2;
  const int r = (warp & 3) * 32 + (tid & 31), half = warp >> 2;
  if (owner) {
    float d[32];
    tmem_ld32(c1 + lane_base + half * 32, d);
    tmem_ld_wait();
#pragma unroll
    for (int s8 = 0; s8 < 4; ++s8) tile_st_chunk(DTt, r, half * 4 + s8, 64, pack8_f16(d + 8 * s8));
  }
  sync_for_issue();
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, c2, Tile{smem_u32(DTt), 64, false}, Tile{smem_u32(TAt), 128, false}, 64, 64, 0u);
    umma_commit_led(leader, bar_mma);
  }
  wait_products(bar_mma, ph, ctl, 613);
  if (owner) {
    float d[32];
    tmem_ld32(c2 + lane_base + half * 32, d);
    tmem_ld_wait();
#pragma unroll
    for (int s8 = 0; s8 < 4; ++s8) tile_st_chunk(XT, r, half * 4 + s8, 64, pack8_f16(d + 8 * s8));
  }
  sync_for_issue();
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    issue_product_led(leader, c3, Tile{smem_u32(TAt), 64, true}, Tile{smem_u32(XT), 64, true}, 64, 64, 0u, true);
    umma_commit_led(leader, bar_mma);
  }
  wait_products(bar_mma, ph, ctl, 614);
  // Everything read so far is older than the kernel before this one (the Stage-B pair kernel), which
  // still reads the dq-part record that is overwritten below: wait for it before writing anything.
  griddep_wait();
  griddep_launch();
  // Results are staged in tiles that are dead by now and leave as bulk copies: dM in the dT tile, the fp32
  // record of d(beta gamma k) in the 32 KB that start at the [T; A] tile and run over the dv2 tile (and, at
  // d_v = 64, half of the dw tile); its global layout is its shared-memory image.
  float* DQs = reinterpret_cast<float*>(TAt);
  float rv = 0.f, pq = 0.f;
  if (owner) {
    {  // dM, strictly lower
      float dm[32];
      tmem_ld32(c3 + lane_base + half * 32, dm);
      tmem_ld_wait();
#pragma unroll
      for (int s8 = 0; s8 < 4; ++s8) {
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = (half * 32 + s8 * 8 + i < r) ? dm[s8 * 8 + i] : 0.f;
        tile_st_chunk(DTt, r, half * 4 + s8, 64, pack8_f16(y));
      }
    }
    // dv = beta dbv; value part of dbeta
    __nv_bfloat16* dv_g = p.dv + (tok0 + static_cast<size_t>(r) * p.H) * V;
#pragma unroll
    for (int jj = 0; jj < V / 64; ++jj) {
      const int jb = half * (V / 64) + jj;
      float d[32];
      tmem_ld32(c4 + lane_base + jb * 32, d);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float vv[8], o8[8];
        unpack8_f16(tile_ld_chunk(VT, r, jb * 4 + i, 64), vv);
        if (full) {   // dv = w dbv, dw = dbv v, element by element
          float wv[8], dwv[8];
          const size_t at = (tok0 + static_cast<size_t>(r) * p.H) * V + jb * 32 + 8 * i;
          ld8(p.wch + at, wv);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            dwv[e] = d[8 * i + e] * vv[e];
            o8[e] = wv[e] * d[8 * i + e];
          }
          st8(p.dwch + at, dwv);
        } else {
          const float bval = betas[r];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            rv += d[8 * i + e] * vv[e];
            o8[e] = bval * d[8 * i + e];
          }
        }
        *reinterpret_cast<uint4*>(dv_g + jb * 32 + 8 * i) = pack8_bf16(o8);
      }
    }
    // d(beta gamma k) = T^T dw: fp32 -> record; its direct part of the erase-gate gradient,
    // sum_d d(beta gamma k) gamma k, is closed here
#pragma unroll 1
    for (int jj = 0; jj < 2; ++jj) {
      const int jb = half * 2 + jj;
      float d[32];
      tmem_ld32(c4 + V + lane_base + jb * 32, d);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float kv[8], gg[8];
        unpack8_f16(tile_ld_chunk(KB, r, jb * 4 + i, 128), kv);
        gt8(Gt, r, jb * 32 + i * 8, gg);
#pragma unroll
        for (int e = 0; e < 8; ++e) pq += d[8 * i + e] * kv[e] * exp2f(gg[e]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
        *reinterpret_cast<float4*>(DQs + ridx(r, jb * 32 + 4 * i)) = make_float4(d[4 * i], d[4 * i + 1], d[4 * i + 2], d[4 * i + 3]);
    }
    if (half == 1) {
      part[r] = rv;
      part[64 + r] = pq;
    }
  }
  fence_proxy_async();
  __syncthreads();
  if (tid == 0) {
    bulk_s2g(p.scratch + p.lay.dm + static_cast<size_t>(z) * 8192, DTt, 8192);
    bulk_s2g(p.scratch + p.lay.dqp + static_cast<size_t>(z) * (kC * kK * 4), DQs, kC * kK * 4);
    bulk_commit();
  }
  if (owner && half == 0 && !full) {
    rv += part[r];
    pq += part[64 + r];
    if (p.dbeta_w) {
      p.dbeta_w[tok0 + static_cast<size_t>(r) * p.H] = rv;
      p.dbeta[tok0 + static_cast<size_t>(r) * p.H] = pq;
    } else {
      p.dbeta[tok0 + static_cast<size_t>(r) * p.H] = rv + pq;
    }
  }
  if (tid == 0) bulk_wait_read();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------
// Decay-coupled pair sums and final assembly.  MODE 0: Stage B (C = scale dA, x = q);
// MODE 1: WY VJP (C = dM, x = beta k).  FINAL_G: this kernel closes the gate gradient (reverse
// cumulative sum per channel); otherwise it leaves its contribution in the DGB record.
// Accumulators: out1 rows 0-63 of [0,128); out2 rows 64-127 of [128,256).
// ---------------------------------------------------------------------------------------------
// 512 threads for the same reason as the forward's prepare kernel: one CTA per SM (197 KB of tiles) whose
// CUDA-core phases are bound by instruction latency.
constexpr int kPairThreads = 512;

template <int MODE, bool FINAL_G>
__global__ void __launch_bounds__(kPairThreads)
bwd_cw_pair_kernel(const Problem p, const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = align1024(smem_raw);
  unsigned char* KX = sm;                       // 32 KB: rows 0-63 k, rows 64-127 x
  unsigned char* KR = KX + 32768;               // 32 KB: k exp(G_{16 I} - G_s), rows [0,16) [16,48) [48,96)
  unsigned char* XE = KR + 32768;               // 32 KB: x exp(G_i - G_{16 J + 15}), rows [0,48) [48,80) [80,96)
  unsigned char* CS = XE + 32768;               // 8 KB: C as loaded; doubles as the junk atom in front of MB_0
  unsigned char* MB = CS + 8192;                // 3 x 8 KB: C restricted to column block J and rows >= 16 (J + 1)
  unsigned char* MA = MB + 3 * 8192;            // 3 x 8 KB: C restricted to row block I and columns < 16 I
  float* Gt = reinterpret_cast<float*>(MA + 4 * 8192);   // (one spare 8 KB tile behind MA_3 for over-reads)
  float* fs = Gt + 64 * kK;
  float* Cd = fs;                // [64][16] diagonal blocks of C
  float* betas = fs + 1024;      // [64]
  float* red = fs + 1088;        // [4][64] partial row sums for dbeta
  CtaShared* cs = reinterpret_cast<CtaShared*>(fs + 1344);
  float* EX1 = reinterpret_cast<float*>(KR);    // exchange tiles, once the products are done
  float* EX2 = reinterpret_cast<float*>(XE);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int bh = p.bh0 + blockIdx.x / p.cn, c = p.c0 + blockIdx.x % p.cn, z = bh * p.NT + c, b = bh / p.H, h = bh % p.H;
  CtaCtl ctl{p.status, &cs->abort_flag};
  uint64_t* bar_load = &cs->bar[0];
  uint64_t* bar_mma = &cs->bar[1];
  uint64_t* bar_c = &cs->bar[2];        // C (dA or dM), written by the kernel just before this one
  uint64_t* bar_rec = &cs->bar[3];      // the fp32 records of phase B, fetched into dead operand tiles
  float* RQ = reinterpret_cast<float*>(CS);               // 32 KB: the dq part (Stage B) / d(beta gamma k) part (WY VJP)
  float* RK = reinterpret_cast<float*>(CS + 32768);       // 32 KB: the dk part
  if (tid == 0) {
    cs->abort_flag = 0;
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    mbar_init(bar_c, 1);
    mbar_init(bar_rec, 1);
    fence_mbar_init();
    fence_proxy_async();
    // every load that does not depend on the kernel just before this one is requested at once
    mbar_expect_tx(bar_load, 32768u + 32768u);
    bulk_g2s(Gt, p.saved + p.lay.gt + static_cast<size_t>(z) * (kC * kK * 4), 32768, bar_load);
    for (int a = 0; a < 2; ++a) {
      tma_load_4d(KX + a * 16384, &mk, bar_load, a * 64, h, c * kC, b);
      tma_load_4d(KX + a * 16384 + 8192, MODE == 0 ? &mq : &mk, bar_load, a * 64, h, c * kC, b);
    }
  }
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, 256);
    tmem_relinquish();
  }
  const size_t tok0 = (static_cast<size_t>(b) * p.L + c * kC) * p.H + h;
  const bool full = (MODE == 1) && p.bch != nullptr;    // per-channel erase gate: x = b k element by element
  if (tid < 64) betas[tid] = (MODE == 1 && !full) ? p.beta[tok0 + static_cast<size_t>(tid) * p.H] : 1.f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;
  __syncthreads();
  // the loads above fetch inputs and the gate record; C and the fp32 records come from the kernels just
  // before this one
  griddep_wait();
  griddep_launch();
  if (tid == 0) {
    mbar_expect_tx(bar_c, 8192u);
    bulk_g2s(CS, p.scratch + (MODE == 0 ? p.lay.da : p.lay.dm) + static_cast<size_t>(z) * 8192, 8192, bar_c);
  }
  mbar_wait_warp(bar_load, 0, ctl, 621);
  // ---- decayed operand rows
  for (int idx = tid; idx < 64 * 16; idx += kPairThreads) {
    const int r = idx >> 4, ch = idx & 15, d0 = ch * 8, blk = r >> 4;
    float kx[8], xx[8], y[8], gr[8];
    unpack8_in(tile_ld_chunk(KX, r, ch, 128), kx, p.qk16);
    unpack8_in(tile_ld_chunk(KX, 64 + r, ch, 128), xx, p.qk16);
    const float be = betas[r];
    if (full) {
      float bb[8];
      ld8(p.bch + (tok0 + static_cast<size_t>(r) * p.H) * kK + d0, bb);
#pragma unroll
      for (int e = 0; e < 8; ++e) xx[e] *= bb[e];
    }
    gt8(Gt, r, d0, gr);
#pragma unroll
    for (int e = 0; e < 8; ++e) xx[e] *= be;
    tile_st_chunk(KX, r, ch, 128, pack8_f16(kx));
    tile_st_chunk(KX, 64 + r, ch, 128, pack8_f16(xx));
    for (int I = blk + 1; I < 4; ++I) {
      const int off = (I == 1) ? 0 : (I == 2 ? 16 : 48);
      float ga[8];
      gt8(Gt, I * 16, d0, ga);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = kx[e] * exp2f(ga[e] - gr[e]);
      tile_st_chunk(KR, off + r, ch, 128, pack8_f16(y));
    }
    for (int J = 0; J < blk; ++J) {
      const int off = (J == 0) ? 0 : (J == 1 ? 48 : 80);
      float ga[8];
      gt8(Gt, J * 16 + 15, d0, ga);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = xx[e] * exp2f(gr[e] - ga[e]);
      tile_st_chunk(XE, off + (r - 16 * (J + 1)), ch, 128, pack8_f16(y));
    }
  }
  mbar_wait_warp(bar_c, 0, ctl, 623);
  // ---- masked copies of C and its diagonal blocks
  for (int idx = tid; idx < 64 * 8; idx += kPairThreads) {
    const int r = idx >> 3, s8 = idx & 7, blk = r >> 4, cb = s8 >> 1;
    const uint4 cv = tile_ld_chunk(CS, r, s8, 64);
    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int I = 1; I < 4; ++I) tile_st_chunk(MA + (I - 1) * 8192, r, s8, 64, (I == blk && cb < I) ? cv : zero);
#pragma unroll
    for (int J = 0; J < 3; ++J) tile_st_chunk(MB + J * 8192, r, s8, 64, (cb == J && blk > J) ? cv : zero);
    if (cb == blk) {
      float cf[8];
      unpack8_f16(cv, cf);
#pragma unroll
      for (int e = 0; e < 8; ++e) Cd[r * 16 + (s8 & 1) * 8 + e] = cf[e];
    }
  }
  sync_for_issue();
  uint32_t ph = 0;
  if (warp == 0) {
    tc_fence_after();
    const uint32_t leader = elect_leader();
    for (int I = 1; I < 4; ++I) {
      const int off = (I == 1) ? 0 : (I == 2 ? 16 : 48);
      issue_product_led(leader, tmem, Tile{smem_u32(MA + (I - 1) * 8192), 64, false},
                    Tile{smem_u32(KR) + off * 128, 128, true}, 128, 16 * I, I > 1 ? 1u : 0u);
    }
    for (int J = 0; J < 3; ++J) {
      const int off = (J == 0) ? 0 : (J == 1 ? 48 : 80);
      const int r0 = 16 * (J + 1);
      issue_product_led(leader, tmem + 128, Tile{smem_u32(MB + J * 8192) - 8192 + r0 * 128, 64, true},
                    Tile{smem_u32(XE) + off * 128, 128, true}, 128, 64 - r0, J > 0 ? 1u : 0u);
    }
    umma_commit_led(leader, bar_mma);
  }
  wait_products(bar_mma, ph, ctl, 622);
  __syncthreads();          // products done for every thread: KR / XE become the exchange tiles
  // The masked copies of C (CS, MB, MA: 64 KB in a row) are dead too: two of the three fp32 records phase B
  // combines are fetched into them now, by bulk copies that run under the diagonal blocks and phase A,
  // instead of being read element by element from global memory when phase B needs them.
  if (tid == 0) {
    mbar_expect_tx(bar_rec, 65536u);
    bulk_g2s(RQ, p.scratch + p.lay.dqp + static_cast<size_t>(z) * (kC * kK * 4), 32768u, bar_rec);
    bulk_g2s(RK, p.scratch + p.lay.dkb + static_cast<size_t>(z) * p.lay.sz_dkb, 32768u, bar_rec);
  }
  // ---- diagonal blocks, exact; thread (block, channel d) owns channel d of one 16-row block
  {
    const int d = tid & 127;
    {
      const int blk = tid >> 7;
      float g[16], kk[16], xv[16], a1[16], a2[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int r = blk * 16 + j;
        g[j] = Gt[gidx(r, d)];
        kk[j] = __half2float(*reinterpret_cast<const __half*>(KX + sw128_off(r, d, 128)));
        xv[j] = __half2float(*reinterpret_cast<const __half*>(KX + sw128_off(64 + r, d, 128)));
        a1[j] = 0.f;
        a2[j] = 0.f;
      }
      // ratio(i, s) = exp2(g_i - g_s) for the 136 pairs s <= i of the block with 54 exponentials instead of
      // 136 (the special-function unit is what bounds this phase).  The 16 rows are cut into four groups of
      // four; with a_G the first and l_G the last row of group G:
      //   s == i                              1
      //   s < i in the same group             exp2(g_i - g_s)                                       (24)
      //   i in group A, s in an earlier B     exp2(g_i - g_aA) * exp2(g_aA - g_lB) * exp2(g_lB - g_s)   (12 + 6 + 12)
      // Every factor is a decay between two rows that lie between s and i, so each is <= 1 and >= the
      // ratio itself: nothing can overflow, and nothing underflows before the ratio does.
      float eu[16], fd[16], br[6];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        eu[j] = (j & 3) ? exp2f(g[j] - g[j & ~3]) : 1.f;
        fd[j] = ((j & 3) != 3) ? exp2f(g[j | 3] - g[j]) : 1.f;
      }
#pragma unroll
      for (int A = 1; A < 4; ++A)
#pragma unroll
        for (int B = 0; B < A; ++B) br[A * (A - 1) / 2 + B] = exp2f(g[4 * A] - g[4 * B + 3]);
#pragma unroll
      for (int ii = 0; ii < 16; ++ii) {
#pragma unroll
        for (int ss = 0; ss <= ii; ++ss) {
          const int A = ii >> 2, B = ss >> 2;
          float r;
          if (ss == ii) r = 1.f;
          else if (A == B) r = exp2f(g[ii] - g[ss]);
          else r = (eu[ii] * br[A * (A - 1) / 2 + B]) * fd[ss];
          const float cv = Cd[(blk * 16 + ii) * 16 + ss];
          const float e = cv * r;
          a1[ii] += e * kk[ss];
          a2[ss] += e * xv[ii];
        }
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        EX1[exi(blk * 16 + j, d)] = a1[j];
        EX2[exi(blk * 16 + j, d)] = a2[j];
      }
    }
  }
  __syncthreads();
  // ---- phase A: row owners fold the tensor-core part (with its decay) into the exchange tiles.
  // Thread t & 127 owns accumulator lane t & 127; the four warps that reach a lane quadrant (w, w + 4, w + 8,
  // w + 12) take one 32-column block each.
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  {
    const int t = tid & 127, jb0 = tid >> 7;      // the four warps of a lane quadrant take one 32-column block each
    if (t < 64) {
      const int i = t, a = (i >> 4) * 16;      // out1 row i: decay from the block's reference row
      float rsum = 0.f;
#pragma unroll 1
      for (int jb = jb0; jb < jb0 + 1; ++jb) {
        float acc[32];
        tmem_ld32(tmem + lane_base + jb * 32, acc);
        tmem_ld_wait();
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {
          float kv[8], gi8[8], ga8[8];
          if (MODE == 1) unpack8_f16(tile_ld_chunk(KX, i, jb * 4 + q8, 128), kv);
          gt8(Gt, i, jb * 32 + q8 * 8, gi8);
          gt8(Gt, a, jb * 32 + q8 * 8, ga8);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int d = jb * 32 + q8 * 8 + e;
            const float o1 = acc[8 * q8 + e] * exp2f(gi8[e] - ga8[e]) + EX1[exi(i, d)];
            EX1[exi(i, d)] = o1;
            if (MODE == 1) rsum += o1 * kv[e];
          }
        }
      }
      if (MODE == 1) red[(tid >> 7) * 64 + i] = rsum;
    } else {
      const int s = t - 64, el = (s >> 4) * 16 + 15;   // out2 row s: decay to the last row of its block
#pragma unroll 1
      for (int jb = jb0; jb < jb0 + 1; ++jb) {
        float acc[32];
        tmem_ld32(tmem + 128 + lane_base + jb * 32, acc);
        tmem_ld_wait();
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {
          float ge8[8], gs8[8];
          gt8(Gt, el, jb * 32 + q8 * 8, ge8);
          gt8(Gt, s, jb * 32 + q8 * 8, gs8);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int d = jb * 32 + q8 * 8 + e;
            EX2[exi(s, d)] = acc[8 * q8 + e] * exp2f(ge8[e] - gs8[e]) + EX2[exi(s, d)];
          }
        }
      }
    }
  }
  __syncthreads();
  if (MODE == 1 && !full && tid < 64)      // sum_d d(bk)_m k
    p.dbeta[tok0 + static_cast<size_t>(tid) * p.H] += (red[tid] + red[64 + tid]) + (red[128 + tid] + red[192 + tid]);
  // ---- phase B: every (row, group of four channels) combines the two sums with the fp32 records: the dq / dk
  // parts from their shared-memory copies, the gate-gradient part from global memory.  A warp covers one row
  // (32 groups), a thread four rows 16 apart; every access is a 16-byte (8-byte for the fp16 tiles and the
  // 16-bit outputs) piece, coalesced along the channels.
  mbar_wait_warp(bar_rec, 0, ctl, 624);
  {
    float* __restrict__ dkb_g = reinterpret_cast<float*>(p.scratch + p.lay.dkb + static_cast<size_t>(z) * p.lay.sz_dkb);
    float* __restrict__ dgb_g = reinterpret_cast<float*>(p.scratch + p.lay.dgb + static_cast<size_t>(z) * p.lay.sz_dgb);
    constexpr bool kFinalK = (MODE == 1) || FINAL_G;     // without the delta term Stage B closes dk
    constexpr int kItems = 64 * 32 / kPairThreads;
    float4 dgb4[kItems];
#pragma unroll
    for (int u = 0; u < kItems; ++u) {
      const int item = tid + u * kPairThreads;
      dgb4[u] = *reinterpret_cast<const float4*>(dgb_g + ridx(item >> 5, (item & 31) * 4));
    }
#pragma unroll
    for (int u = 0; u < kItems; ++u) {
      const int item = tid + u * kPairThreads, i = item >> 5, c4 = item & 31, d0 = c4 * 4;
      const float4 part4 = *reinterpret_cast<const float4*>(RQ + ridx(i, d0));
      const float4 dkb4 = *reinterpret_cast<const float4*>(RK + ridx(i, d0));
      const float part[4] = {part4.x, part4.y, part4.z, part4.w}, dkb[4] = {dkb4.x, dkb4.y, dkb4.z, dkb4.w};
      const float dgb[4] = {dgb4[u].x, dgb4[u].y, dgb4[u].z, dgb4[u].w};
      float o1[4], o2[4], kv[4], xv[4];
      ex_ld4(EX1, i, c4, o1);
      ex_ld4(EX2, i, c4, o2);
      unpack4_f16(*reinterpret_cast<const uint2*>(KX + sw128_chunk(i, c4 >> 1, 128) + (c4 & 1) * 8), kv);
      unpack4_f16(*reinterpret_cast<const uint2*>(KX + sw128_chunk(64 + i, c4 >> 1, 128) + (c4 & 1) * 8), xv);
      const size_t tok = (tok0 + static_cast<size_t>(i) * p.H) * kK + d0;
      float dk[4], dG[4];
      if (MODE == 0) {
        float dq[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          dq[e] = part[e] + o1[e];
          dk[e] = dkb[e] + o2[e];
          dG[e] = dgb[e] + xv[e] * o1[e] - kv[e] * o2[e];          // q~ . dq_intra - k . dk_intra (the scale sits in C)
        }
        store_out16x4(p.dq + tok, dq, p.qk16);
      } else {
        const float4 g4 = gt4(Gt, i, d0);
        const float gg[4] = {g4.x, g4.y, g4.z, g4.w};
        float bb[4];
        if (full) {
          const float4 b4 = *reinterpret_cast<const float4*>(p.bch + tok);
          bb[0] = b4.x; bb[1] = b4.y; bb[2] = b4.z; bb[3] = b4.w;
        } else {
          bb[0] = bb[1] = bb[2] = bb[3] = betas[i];
        }
        float dbkk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float eg = exp2f(gg[e]);
          const float dbk = part[e] * eg + o1[e];                  // d(beta k), or d(b k) of the full op
          dk[e] = dkb[e] + dbk * bb[e] + o2[e];
          dbkk[e] = dbk * kv[e];
          dG[e] = dgb[e] + part[e] * xv[e] * eg + xv[e] * o1[e] - kv[e] * o2[e];   // dq_wy (b gamma k) + (b k) dbk_m - k dk_m
        }
        if (full) *reinterpret_cast<float4*>(p.dbch + tok) = make_float4(dbkk[0], dbkk[1], dbkk[2], dbkk[3]);
      }
      if (kFinalK) store_out16x4(p.dk + tok, dk, p.qk16);
      else *reinterpret_cast<float4*>(dkb_g + ridx(i, d0)) = make_float4(dk[0], dk[1], dk[2], dk[3]);
      if (FINAL_G) ex_st4(EX1, i, c4, dG);                         // closed below by the reverse cumulative sum
      else *reinterpret_cast<float4*>(dgb_g + ridx(i, d0)) = make_float4(dG[0], dG[1], dG[2], dG[3]);
    }
  }
  if (FINAL_G) {
    // dg[i, d] = sum_{j >= i} dG[j, d]: thread (row group, channel) forms the suffix sums of its 16 rows, the
    // group totals are exchanged through shared memory (Cd is dead since the diagonal blocks) and the totals
    // of the groups below are added
    __syncthreads();
    const int d = tid & 127, grp = tid >> 7;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = EX1[exi(grp * 16 + j, d)];
#pragma unroll
    for (int j = 14; j >= 0; --j) v[j] += v[j + 1];
    Cd[grp * kK + d] = v[0];
    __syncthreads();
    float below = 0.f;
    for (int g2 = 3; g2 > grp; --g2) below += Cd[g2 * kK + d];
#pragma unroll
    for (int j = 0; j < 16; ++j) p.dg[(tok0 + static_cast<size_t>(grp * 16 + j) * p.H) * kK + d] = v[j] + below;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------
template <int V, bool DELTA>
static int launch_sb1_t(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mdo,
                        cudaStream_t st) {
  const int smem = 32768 + 16384 + V * 256 + 16384 + V * 128 + V * 512 + 32768 + 128 * 4 +
                   static_cast<int>(sizeof(CtaShared)) + 1024;
  static SmemAttr attr;
  if (attr.set(bwd_cw_sb1_kernel<V, DELTA>, smem)) return kErrLaunch;
  if (launch_dependent(bwd_cw_sb1_kernel<V, DELTA>, dim3(p.nbh * p.cn), dim3(256), smem, st, p, mq, mk, mdo) !=
      cudaSuccess) return kErrLaunch;
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
template <int V>
static int launch_wy1_t(const Problem& p, const CUtensorMap& mk, const CUtensorMap& mv, cudaStream_t st) {
  const int smem = 32768 + V * 128 * 3 + 16384 * 2 + 8192 + 16384 + 32768 + (64 + 128) * 4 +
                   static_cast<int>(sizeof(CtaShared)) + 1024;
  static SmemAttr attr;
  if (attr.set(bwd_cw_wy1_kernel<V>, smem)) return kErrLaunch;
  if (launch_dependent(bwd_cw_wy1_kernel<V>, dim3(p.nbh * p.cn), dim3(kWy1Threads), smem, st, p, mk, mv) != cudaSuccess)
    return kErrLaunch;
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
template <int MODE, bool FINAL_G>
static int launch_pair_t(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk, cudaStream_t st) {
  const int smem = 32768 * 3 + 8192 * 8 + 32768 + 1344 * 4 + static_cast<int>(sizeof(CtaShared)) + 1024;
  static SmemAttr attr;
  if (attr.set(bwd_cw_pair_kernel<MODE, FINAL_G>, smem)) return kErrLaunch;
  if (launch_dependent(bwd_cw_pair_kernel<MODE, FINAL_G>, dim3(p.nbh * p.cn), dim3(kPairThreads), smem, st, p, mq, mk) !=
      cudaSuccess) return kErrLaunch;
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// mask bit 4: Stage B (two kernels), bit 8: WY VJP (two kernels, delta variants only)
int launch_bwd_main_cw(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                       const CUtensorMap& mdo, cudaStream_t st, uint32_t mask) {
  int e = kOk;
  if (mask & 4u) {
    if (p.V == 64) e = p.delta ? launch_sb1_t<64, true>(p, mq, mk, mdo, st) : launch_sb1_t<64, false>(p, mq, mk, mdo, st);
    else e = p.delta ? launch_sb1_t<128, true>(p, mq, mk, mdo, st) : launch_sb1_t<128, false>(p, mq, mk, mdo, st);
    if (e) return e;
    e = p.delta ? launch_pair_t<0, false>(p, mq, mk, st) : launch_pair_t<0, true>(p, mq, mk, st);
    if (e) return e;
  }
  if (!p.delta || !(mask & 8u)) return e;
  e = p.V == 64 ? launch_wy1_t<64>(p, mk, mv, st) : launch_wy1_t<128>(p, mk, mv, st);
  if (e) return e;
  return launch_pair_t<1, true>(p, mq, mk, st);
}

}  // namespace lg
