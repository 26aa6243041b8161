// Shared definitions of the GDN kernels: problem description, workspace layout, small device helpers.
//
// Work decomposition.  A "chunk" is 64 consecutive tokens of one (batch, head) pair; chunks are
// numbered z = (b*H + h)*NT + c.  Chunk-parallel kernels run one CTA (128 or 256 threads) per chunk;
// the scan kernel runs one CTA per (b, h, 16-column slice of V) and walks the chunks in order.
//
// Per-chunk records in the workspaces ("image" = the SW128 shared-memory tile image, so that a
// record moves between global and shared memory with one contiguous bulk copy):
//   saved (forward -> backward)
//     TA    16 KB   image, 128 rows x 64: rows 0-63 T = (I + strict_lower(M))^-1, rows 64-127 A
//     W     16 KB   image, 64 x 128: WY factor w = T (beta gamma k)
//     U     64 x V  image: u = T (beta v)
//     P     32 KB   image, 128 x 128: kd^T w           (state transition, without the decay)
//     R     128 x V fp16 row-major: kd^T u            (state input)
//     Hc    128 x V image: state entering the chunk; NT + 1 records per (b, h), the last one being
//           the final state, so record index is (b*H + h)*(NT + 1) + c
//     VN    64 x V  image: v_new = u - w h
//     AD    128 fp32: exp(G_last) per key channel     (the decay of the chunk)
//     GT    channel-wise gate only: 64 x 128 fp32, the cumulative decay of the chunk in log2 units in the
//           swizzled shared-memory arrangement of gidx(), written once by prepare and bulk-loaded
//           by every later kernel instead of being recomputed
//     QG    channel-wise gate only: 16 KB image, 64 x 128: scale * gamma * q, the query operand of the output
//           kernel and of the adjoint scan's input kernel (written by prepare, which has q and the gate in
//           registers anyway, so that those two kernels need neither the 32 KB gate tile nor a conversion)
//   scratch (backward only)
//     RB    128 x V fp16 row-major: (q gamma)^T do - w^T (A^T do)
//     DH    128 x V image: adjoint of the state leaving the chunk
//     DV2   64 x V  image: adjoint of v_new
//     DW    64 x 128 image: adjoint of w
//     DKB   64 x 128 fp32: key gradient of Stage B
//     DGB   64 x 128 fp32 (channel-wise) or 64 fp32 (scalar): gate-gradient of Stage B before the cumsum
//   channel-wise gate only:
//     DA    64 x 64 image: scale * tril(do v_new^T)         DM   64 x 64 image: strict_lower(-T^T dT T^T)
//     DQP   64 x 128 fp32: the part of dq (Stage B), then of d(beta gamma k) (WY VJP), outside the
//           decay-coupled sums
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "../../include/lethe_gdn.h"
#include "tiles.cuh"

namespace lg {

constexpr int kC = 64;    // chunk length
constexpr int kK = 128;   // key dimension

struct Layout {
  // byte offsets of the record arrays inside `saved` / `scratch`, and record sizes
  size_t ta, w, u, p, r, hc, vn, ad, gt, qg, carry_f, saved_total;
  size_t rb, dh, dv2, dw, dkb, dgb, da, dm, dqp, carry_b, scratch_total;
  size_t sz_ta, sz_w, sz_u, sz_p, sz_r, sz_hc, sz_vn, sz_ad;
  size_t sz_rb, sz_dh, sz_dv2, sz_dw, sz_dkb, sz_dgb;
};

__host__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__host__ inline Layout make_layout(const LetheGdnDims& d) {
  Layout l{};
  const size_t Z = static_cast<size_t>(d.B) * d.H * (d.L / kC);
  const size_t V = d.V;
  l.sz_ta = 16384; l.sz_w = 16384; l.sz_u = kC * V * 2; l.sz_p = 32768; l.sz_r = kK * V * 2;
  l.sz_hc = kK * V * 2; l.sz_vn = kC * V * 2; l.sz_ad = kK * 4;
  size_t o = 0;
  l.ta = o; o = align_up(o + Z * l.sz_ta, 1024);
  l.w = o;  o = align_up(o + Z * l.sz_w, 1024);
  l.u = o;  o = align_up(o + Z * l.sz_u, 1024);
  l.p = o;  o = align_up(o + Z * l.sz_p, 1024);
  l.r = o;  o = align_up(o + Z * l.sz_r, 1024);
  l.hc = o; o = align_up(o + (Z + static_cast<size_t>(d.B) * d.H) * l.sz_hc, 1024);
  l.vn = o; o = align_up(o + Z * l.sz_vn, 1024);
  l.ad = o; o = align_up(o + Z * l.sz_ad, 1024);
  if (d.gate == LETHE_GATE_CHANNEL) {
    l.gt = o; o = align_up(o + Z * static_cast<size_t>(kC * kK * 4), 1024);
    l.qg = o; o = align_up(o + Z * static_cast<size_t>(16384), 1024);
  }
  // fp32 master state handed from one chunk-range call of the forward scan to the next ([B, H, K, V])
  l.carry_f = o; o = align_up(o + static_cast<size_t>(d.B) * d.H * kK * V * 4, 1024);
  l.saved_total = o;
  l.sz_rb = kK * V * 2; l.sz_dh = kK * V * 2; l.sz_dv2 = kC * V * 2; l.sz_dw = 16384;
  l.sz_dkb = kC * kK * 4; l.sz_dgb = (d.gate == LETHE_GATE_CHANNEL ? kC * kK : kC) * 4;
  o = 0;
  l.rb = o;  o = align_up(o + Z * l.sz_rb, 1024);
  l.dh = o;  o = align_up(o + Z * l.sz_dh, 1024);
  l.dv2 = o; o = align_up(o + Z * l.sz_dv2, 1024);
  l.dw = o;  o = align_up(o + Z * l.sz_dw, 1024);
  l.dkb = o; o = align_up(o + Z * l.sz_dkb, 1024);
  l.dgb = o; o = align_up(o + Z * l.sz_dgb, 1024);
  if (d.gate == LETHE_GATE_CHANNEL) {
    l.da = o;  o = align_up(o + Z * 8192, 1024);
    l.dm = o;  o = align_up(o + Z * 8192, 1024);
    l.dqp = o; o = align_up(o + Z * static_cast<size_t>(kC * kK * 4), 1024);
  }
  l.carry_b = o; o = align_up(o + static_cast<size_t>(d.B) * d.H * kK * V * 4, 1024);   // the same for the adjoint scan
  l.scratch_total = o;
  return l;
}

// Everything a kernel needs besides its tensor maps.
struct Problem {
  int B, H, L, NT, V, gate, delta;
  int bh0, nbh;      // the (batch, head) pairs this call works on: [bh0, bh0 + nbh) of the B * H pairs
  int c0, cn;        // the chunks of every pair this call works on: [c0, c0 + cn) of the NT chunks
  int qk16;          // non-zero: q, k, dq, dk hold fp16 instead of bf16
  float scale;
  const __nv_bfloat16 *q, *k, *v, *d_o;
  const float *g, *beta, *h0, *dhT;
  __nv_bfloat16 *o, *dq, *dk, *dv;
  float *hT, *dg, *dbeta, *dh0, *dbeta_w;
  // full op only (null otherwise): per-channel erase gate [B,L,H,K], write gate [B,L,H,V] and their gradients
  const float *bch, *wch;
  float *dbch, *dwch;
  unsigned char* saved;
  unsigned char* scratch;
  Layout lay;
  int* status;
};

// ---------------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------------
// Inclusive prefix sum of one value per thread over threads 0..63 (two warps); every thread of the
// CTA must call it (it contains __syncthreads).  `tmp` is a shared float[2].
__device__ __forceinline__ float chunk_cumsum(float x, int tid, float* tmp) {
  const int lane = tid & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (tid == 31) tmp[0] = x;
  __syncthreads();
  if (tid >= 32 && tid < 64) x += tmp[0];
  return x;
}

// Inclusive suffix sum over threads 0..63 (x_t + x_{t+1} + ... + x_63), same calling rules.
__device__ __forceinline__ float chunk_rev_cumsum(float x, int tid, float* tmp) {
  const int lane = tid & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float y = __shfl_down_sync(0xffffffffu, x, o);
    if (lane + o < 32) x += y;
  }
  if (tid == 32) tmp[0] = x;
  __syncthreads();
  if (tid < 32) x += tmp[0];
  return x;
}

// Channel-wise gate tile: cumulative decay of the chunk in LOG2 units (G * log2 e, so that every decay
// factor is one exp2 of a difference), 64 rows x 128 channels of fp32 in shared memory.  Element (row, col)
// lives at gidx(row, col).  A row is 32 pieces of 16 bytes (four channels).  The even pieces - the first
// halves of the 8-channel groups that match one 16-byte chunk of an fp16 operand tile - come first, then
// the odd pieces, and within every 128-byte line the pieces are XOR-ed with the low three row bits (the odd
// half with 4 more).  All three ways the kernels read the tile then run without bank replays:
//   "lane = chunk of one row" (operand builds): 16 lanes read 16 neighbouring pieces, twice (gt8);
//   "thread i reads row i" (epilogues): eight neighbouring rows land in eight different pieces of a line;
//   "thread d walks column d": 32 channels are 4 + 4 pieces in two lines, on disjoint banks.
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ int gidx(int row, int col) {
  const int p = col >> 2;
  const int piece = ((p >> 1) + ((p & 1) << 4)) ^ ((row & 7) ^ ((p & 1) << 2));
  return row * kK + (piece << 2) + (col & 3);
}
// four / eight consecutive gate values of one row (col0 a multiple of 4 / 8)
__device__ __forceinline__ float4 gt4(const float* Gt, int row, int col0) {
  return *reinterpret_cast<const float4*>(Gt + gidx(row, col0));
}
__device__ __forceinline__ void gt8(const float* Gt, int row, int col0, float* g) {
  const float4 a = gt4(Gt, row, col0), b = gt4(Gt, row, col0 + 4);
  g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
}
// fp32 exchange tiles [64][128] (not the gate tile): the column is XOR-ed with the low five row bits, so that
// both "thread d walks column d" and "thread i walks row i" with scalar accesses are free of bank conflicts
__device__ __forceinline__ int exi(int row, int col) { return row * kK + (col ^ (row & 31)); }

// Control block at the start of every kernel: barriers, TMEM slot, abort flag.
struct CtaShared {
  uint64_t bar[8];
  uint32_t tmem_slot;
  int abort_flag;
};


// Next 1024-byte boundary of the dynamic shared memory window, two ways.  `align1024` is plain
// pointer arithmetic on the shared symbol, so the compiler keeps the shared address space and emits
// shared-memory loads and stores; `align1024_generic` goes through an integer, after which every
// access is a generic one.  Same addresses, different instruction selection and scheduling: the
// channel-wise kernels run 10-15 % faster with the first, the scalar kernels 3-5 % except the prepare
// kernel without the delta term, which is 10 % faster with the second, as are the scans by 1-3 %
// (measured per kernel on a B200), so each kernel names the one it wants.
__device__ __forceinline__ unsigned char* align1024_s_(unsigned char* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  return p + ((1024u - (a & 1023u)) & 1023u);
}
__device__ __forceinline__ unsigned char* align1024_g_(unsigned char* p) {
  return reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}
// (-DLETHE_ALL_SHARED / -DLETHE_ALL_GENERIC force one flavour everywhere, to repeat the comparison)
__device__ __forceinline__ unsigned char* align1024(unsigned char* p) {
#ifdef LETHE_ALL_GENERIC
  return align1024_g_(p);
#else
  return align1024_s_(p);
#endif
}
__device__ __forceinline__ unsigned char* align1024_generic(unsigned char* p) {
#ifdef LETHE_ALL_SHARED
  return align1024_s_(p);
#else
  return align1024_g_(p);
#endif
}

// Called by all threads before one thread issues products that read tiles written by this CTA's
// threads and / or overwrite accumulators that this CTA's threads have been reading.
__device__ __forceinline__ void sync_for_issue() {
  tc_fence_before();
  fence_proxy_async();
  __syncthreads();
}

// Called by all threads after the issuing thread committed to `bar`: waits for the products.
__device__ __forceinline__ void wait_products(uint64_t* bar, uint32_t& phase, const CtaCtl& ctl, int code) {
  __syncwarp();
  mbar_wait_warp(bar, phase, ctl, code);
  phase ^= 1u;
  tc_fence_after();
}

// eight consecutive floats (16-byte aligned)
__device__ __forceinline__ void ld8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void st8(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// With the delta term the scan's input records R / Rb (128 rows x V columns, fp16) are stored as V / 16 column blocks of
// [128 rows][16 columns]: one contiguous 4 KB block per scan CTA, 32 bytes per thread.  Byte offset of
// the 8-column piece `col8` of `row` (without the delta term they are plain 128-row tile images, read by
// scan_nodelta_kernel with full-line accesses):
__device__ __forceinline__ uint32_t rrec_off(int row, int col8) {
  return static_cast<uint32_t>((col8 >> 1) * 4096 + row * 32 + (col8 & 1) * 16);
}

// T = (I + M)^-1 for a strictly lower-triangular 64 x 64 M (fp32, row stride MS floats, zeros on and
// above the diagonal), by 16 x 16 blocks on threads 0-255 of a CTA (every thread of the CTA must call: four
// CTA-wide barriers inside; threads beyond 255 only take part in the barriers).  With D_b the inverses of the four diagonal blocks of I + M and N_ba = D_b M_ba
// (b > a), I + N is unit block-lower with N^4 = 0, so
//   X = (I + N)^-1:  X_b,b-1 = -N_b,b-1;  X_20 = -N_20 + N_21 N_10;  X_31 = -N_31 + N_32 N_21;
//                    X_30 = -N_30 + N_31 N_10 - N_32 X_20
//   T_bb = D_b,  T_ba = X_ba D_a.
// Five short stages of independent 16-long dot products replace 64 dependent row steps.  Block rows
// live at a stride of 20 floats (left factors are read one row per lane, right factors as float4).
// `scratch`: 3200 floats (D, then N); X overwrites `Msm`, which is dead once N is formed.
// T leaves as fp16 in rows 0-63 of the 128-row SW128 tile `TA`, blocks above the diagonal zeroed.
constexpr int kInvBs = 20;                 // row stride of a 16 x 16 block
constexpr int kInvBlk = 16 * kInvBs;       // floats per block
constexpr int kInvScratchFloats = 10 * kInvBlk;

// acc[0..W) += sum_k left[k] * right[k][0..W), W in {2, 4, 8}; right rows RS floats apart
template <int W, int RS>
__device__ __forceinline__ void blk_mac(float* acc, const float* left, const float* right) {
#pragma unroll 4
  for (int k = 0; k < 16; ++k) {
    const float a = left[k];
    if (W == 2) {
      const float2 r = *reinterpret_cast<const float2*>(right + k * RS);
      acc[0] = fmaf(a, r.x, acc[0]);
      acc[1] = fmaf(a, r.y, acc[1]);
    } else {
#pragma unroll
      for (int q = 0; q < W / 4; ++q) {
        const float4 r = *reinterpret_cast<const float4*>(right + k * RS + 4 * q);
        acc[4 * q] = fmaf(a, r.x, acc[4 * q]);
        acc[4 * q + 1] = fmaf(a, r.y, acc[4 * q + 1]);
        acc[4 * q + 2] = fmaf(a, r.z, acc[4 * q + 2]);
        acc[4 * q + 3] = fmaf(a, r.w, acc[4 * q + 3]);
      }
    }
  }
}

__device__ __forceinline__ int inv_pair(int b, int a) { return b * (b - 1) / 2 + a; }   // (1,0) (2,0) (2,1) (3,0) (3,1) (3,2)

template <int MS>
__device__ __forceinline__ void unit_lower_inverse64_blocked(float* Msm, float* scratch, unsigned char* TA, int tid) {
  float* Ds = scratch;                     // [4] diagonal-block inverses
  float* Ns = scratch + 4 * kInvBlk;       // [6] N_ba, pair order of inv_pair
  float* Xs = Msm;                         // [3] X_20, X_31, X_30 (from stage 3 on)
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

  const bool on = tid < 256;
  // ---- stage 1: D_b by forward substitution, one column per thread; the rest clear T above the diagonal
  if (!on) {
  } else if (tid < 64) {
    const int b = tid >> 4, j = tid & 15;
    const float* Mb = Msm + (16 * b) * MS + 16 * b;
    float col[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) col[r] = (r == j) ? 1.f : 0.f;
#pragma unroll
    for (int r = 1; r < 16; ++r) {
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int q = 0; q < (r + 3) / 4; ++q) {
        const float4 m = *reinterpret_cast<const float4*>(Mb + r * MS + 4 * q);
        a0 += m.x * col[4 * q];
        if (4 * q + 1 < r) a1 += m.y * col[4 * q + 1];
        if (4 * q + 2 < r) a0 += m.z * col[4 * q + 2];
        if (4 * q + 3 < r) a1 += m.w * col[4 * q + 3];
      }
      col[r] -= a0 + a1;
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) Ds[b * kInvBlk + r * kInvBs + j] = col[r];
  } else {
    const int u = tid - 64, pu = u >> 5, r = (u >> 1) & 15, ch = u & 1;
    // blocks (b, a) with a > b: (0,1) (0,2) (0,3) (1,2) (1,3) (2,3)
    const int b = pu < 3 ? 0 : (pu < 5 ? 1 : 2);
    const int a = pu < 3 ? pu + 1 : (pu < 5 ? pu - 1 : 3);
    tile_st_chunk(TA, 16 * b + r, 2 * a + ch, 128, zero4);
  }
  __syncthreads();

  // ---- stage 2: N_ba = D_b M_ba (one warp per block, a lane = one row x 8 columns); T_bb = D_b
  if (!on) {
  } else if (tid < 192) {
    const int p = tid >> 5, lane = tid & 31, i = lane >> 1, j0 = 8 * (lane & 1);
    const int b = p < 1 ? 1 : (p < 3 ? 2 : 3), a = p - b * (b - 1) / 2;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    blk_mac<8, MS>(acc, Ds + b * kInvBlk + i * kInvBs, Msm + (16 * b) * MS + 16 * a + j0);
    float* out = Ns + p * kInvBlk + i * kInvBs + j0;
    *reinterpret_cast<float4*>(out) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(out + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  } else {
    const int u = tid - 192;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int idx = 2 * u + e, b = idx >> 5, r = (idx >> 1) & 15, ch = idx & 1;
      tile_st_chunk(TA, 16 * b + r, 2 * b + ch, 128, pack8_f16(Ds + b * kInvBlk + r * kInvBs + 8 * ch));
    }
  }
  __syncthreads();

  // ---- stage 3: X_20, X_31 (a thread = one row x 4 columns); T_b,b-1 = -N_b,b-1 D_b-1
  if (tid < 128) {
    const int x = tid >> 6, i = (tid >> 2) & 15, j0 = 4 * (tid & 3);
    // x = 0: N_21 N_10 - N_20;  x = 1: N_32 N_21 - N_31
    const float* left = Ns + (x == 0 ? inv_pair(2, 1) : inv_pair(3, 2)) * kInvBlk + i * kInvBs;
    const float* right = Ns + (x == 0 ? inv_pair(1, 0) : inv_pair(2, 1)) * kInvBlk + j0;
    const float* sub = Ns + (x == 0 ? inv_pair(2, 0) : inv_pair(3, 1)) * kInvBlk + i * kInvBs + j0;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    blk_mac<4, kInvBs>(acc, left, right);
    const float4 n = *reinterpret_cast<const float4*>(sub);
    *reinterpret_cast<float4*>(Xs + x * kInvBlk + i * kInvBs + j0) =
        make_float4(acc[0] - n.x, acc[1] - n.y, acc[2] - n.z, acc[3] - n.w);
  } else if (tid < 224) {
    const int u = tid - 128, b = (u >> 5) + 1, i = (u >> 1) & 15, jh = u & 1;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    blk_mac<8, kInvBs>(acc, Ns + inv_pair(b, b - 1) * kInvBlk + i * kInvBs, Ds + (b - 1) * kInvBlk + 8 * jh);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = -acc[e];
    tile_st_chunk(TA, 16 * b + i, 2 * (b - 1) + jh, 128, pack8_f16(acc));
  }
  __syncthreads();

  // ---- stage 4: X_30 (a thread = one row x 2 columns); T_20 = X_20 D_0, T_31 = X_31 D_1
  if (tid < 128) {
    const int i = tid >> 3, j0 = 2 * (tid & 7);
    float acc[2] = {0.f, 0.f}, acc2[2] = {0.f, 0.f};
    blk_mac<2, kInvBs>(acc, Ns + inv_pair(3, 1) * kInvBlk + i * kInvBs, Ns + inv_pair(1, 0) * kInvBlk + j0);
    blk_mac<2, kInvBs>(acc2, Ns + inv_pair(3, 2) * kInvBlk + i * kInvBs, Xs + j0);
    const float2 n = *reinterpret_cast<const float2*>(Ns + inv_pair(3, 0) * kInvBlk + i * kInvBs + j0);
    *reinterpret_cast<float2*>(Xs + 2 * kInvBlk + i * kInvBs + j0) =
        make_float2((acc[0] - acc2[0]) - n.x, (acc[1] - acc2[1]) - n.y);
  } else if (tid < 192) {
    const int u = tid - 128, x = u >> 5, i = (u >> 1) & 15, jh = u & 1;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    blk_mac<8, kInvBs>(acc, Xs + x * kInvBlk + i * kInvBs, Ds + x * kInvBlk + 8 * jh);
    tile_st_chunk(TA, 16 * (x + 2) + i, 2 * x + jh, 128, pack8_f16(acc));
  }
  __syncthreads();

  // ---- stage 5: T_30 = X_30 D_0, one element per thread (a lone warp with eight columns per lane
  // takes more than twice as long)
  if (on) {
    const int i = tid >> 4, j = tid & 15;
    const float* left = Xs + 2 * kInvBlk + i * kInvBs;
    const float* right = Ds + j;
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int k = 0; k < 16; k += 2) {
      a0 = fmaf(left[k], right[k * kInvBs], a0);
      a1 = fmaf(left[k + 1], right[(k + 1) * kInvBs], a1);
    }
    *reinterpret_cast<__half*>(TA + sw128_off(48 + i, j, 128)) = __float2half_rn(a0 + a1);
  }
}

// Deterministic sum over the 128 threads of a CTA (fixed tree).  `red` is a shared float[4].
__device__ __forceinline__ float cta_sum128(float x, int tid, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = x;
  __syncthreads();
  return (red[0] + red[1]) + (red[2] + red[3]);
}

// The same over 256 threads.  `red` is a shared float[8].
__device__ __forceinline__ float cta_sum256(float x, int tid, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = x;
  __syncthreads();
  return ((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]));
}

}  // namespace lg
