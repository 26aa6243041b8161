// Shared definitions of the GDN kernels: problem description, workspace layout, small device helpers.
//
// Work decomposition.  A "chunk" is 64 consecutive tokens of one (batch, head) pair; chunks are
// numbered z = (b*H + h)*NT + c.  Chunk-parallel kernels run one CTA of 128 threads per chunk;
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
//     GT    channel-wise gate only: 64 x 128 fp32, the cumulative log decay of the chunk in the
//           swizzled shared-memory arrangement of gidx(), written once by prepare and bulk-loaded
//           by every later kernel instead of being recomputed
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

// Development aid: with -DLETHE_PHASE_TIMING one CTA of every instrumented kernel records clock64()
// at its phase boundaries and prints the differences when it ends (never enabled in a normal build).
#ifdef LETHE_PHASE_TIMING
#include <stdio.h>
static __device__ long long g_ph_t[32];
static __device__ const char* g_ph_name[32];
#define LETHE_PHASE_INIT()                                                                         \
  int ph_i_ = 0;                                                                                   \
  const bool ph_on_ = (blockIdx.x == 200 && blockIdx.y == 0 && threadIdx.x == 0);                  \
  LETHE_PHASE("start")
#define LETHE_PHASE(name)                                                                          \
  do {                                                                                             \
    if (ph_on_ && ph_i_ < 32) {                                                                    \
      g_ph_t[ph_i_] = clock64();                                                                   \
      g_ph_name[ph_i_] = name;                                                                     \
      ++ph_i_;                                                                                     \
    }                                                                                              \
  } while (0)
#define LETHE_PHASE_DUMP()                                                                         \
  do {                                                                                             \
    if (ph_on_) {                                                                                  \
      g_ph_t[ph_i_] = clock64();                                                                   \
      printf("PHASE %s:", __func__);                                                               \
      for (int i_ = 1; i_ <= ph_i_; ++i_)                                                          \
        printf(" %s %lld", i_ < ph_i_ ? g_ph_name[i_] : "end", g_ph_t[i_] - g_ph_t[i_ - 1]);       \
      printf(" | total %lld\n", g_ph_t[ph_i_] - g_ph_t[0]);                                        \
    }                                                                                              \
  } while (0)
#else
#define LETHE_PHASE_INIT()
#define LETHE_PHASE(name)
#define LETHE_PHASE_DUMP()
#endif

namespace lg {

constexpr int kC = 64;    // chunk length
constexpr int kK = 128;   // key dimension

struct Layout {
  // byte offsets of the record arrays inside `saved` / `scratch`, and record sizes
  size_t ta, w, u, p, r, hc, vn, ad, gt, saved_total;
  size_t rb, dh, dv2, dw, dkb, dgb, da, dm, dqp, scratch_total;
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
  }
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
  l.scratch_total = o;
  return l;
}

// Everything a kernel needs besides its tensor maps.
struct Problem {
  int B, H, L, NT, V, gate, delta;
  int bh0, nbh;      // the (batch, head) pairs this call works on: [bh0, bh0 + nbh) of the B * H pairs
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

// Channel-wise gate tile: cumulative log decay of the chunk, 64 rows x 128 channels of fp32 in
// shared memory.  Element (row, col) lives at gidx(row, col): the column is XOR-ed with the low row
// bits so that both "thread d walks column d" and "thread i walks row i" are free of bank conflicts.
__device__ __forceinline__ int gidx(int row, int col) { return row * kK + (col ^ (row & 31)); }

// Thread d owns channel d.  `tok0` is the token index of the chunk's first row for this head (tokens
// of a head are H apart).  All 64 loads are issued before the first add so that they overlap.
__device__ __forceinline__ void gate_tile_cw(const float* g, size_t tok0, int H, int tid, float* Gt) {
  float x[kC];
#pragma unroll
  for (int i = 0; i < kC; ++i) x[i] = g[(tok0 + static_cast<size_t>(i) * H) * kK + tid];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < kC; ++i) {
    acc += x[i];
    Gt[gidx(i, tid)] = acc;
  }
}

// Control block at the start of every kernel: barriers, TMEM slot, abort flag.
struct CtaShared {
  uint64_t bar[8];
  uint32_t tmem_slot;
  int abort_flag;
};


__device__ __forceinline__ unsigned char* align1024(unsigned char* p) {
  return reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
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
// above the diagonal), by forward substitution: thread j (0..63) owns column j and works through four
// blocks of 16 rows.  A block first collects what the finished blocks above it contribute (sixteen
// independent sums, T read back from `Tsm`, [48][64] fp32), then resolves its own 16 rows in registers.
// T is written as fp16 into rows 0-63 of the 128-row SW128 tile `TA`.  No synchronisation inside: a
// thread reads back only what it wrote itself.
template <int MS>
__device__ __forceinline__ void unit_lower_inverse64(const float* Msm, float* Tsm, unsigned char* TA, int j) {
  const int jb = j >> 4;
#pragma unroll 1
  for (int blk = 0; blk < 4; ++blk) {
    float col[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) col[r] = (blk * 16 + r == j) ? 1.f : 0.f;
    if (blk >= jb) {
      const float* Mb = Msm + blk * 16 * MS;
      for (int s = jb * 16; s < blk * 16; s += 8) {
        float t[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = Tsm[(s + i) * 64 + j];
#pragma unroll
        for (int r = 0; r < 16; ++r) {
          const float4 m0 = *reinterpret_cast<const float4*>(Mb + r * MS + s);
          const float4 m1 = *reinterpret_cast<const float4*>(Mb + r * MS + s + 4);
          col[r] -= ((m0.x * t[0] + m0.y * t[1]) + (m0.z * t[2] + m0.w * t[3])) +
                    ((m1.x * t[4] + m1.y * t[5]) + (m1.z * t[6] + m1.w * t[7]));
        }
      }
#pragma unroll
      for (int r = 1; r < 16; ++r) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int q = 0; q < (r + 3) / 4; ++q) {
          const float4 m = *reinterpret_cast<const float4*>(Mb + r * MS + blk * 16 + 4 * q);
          a0 += m.x * col[4 * q];
          if (4 * q + 1 < r) a1 += m.y * col[4 * q + 1];
          if (4 * q + 2 < r) a0 += m.z * col[4 * q + 2];
          if (4 * q + 3 < r) a1 += m.w * col[4 * q + 3];
        }
        col[r] -= a0 + a1;
      }
      if (blk < 3) {
#pragma unroll
        for (int r = 0; r < 16; ++r) Tsm[(blk * 16 + r) * 64 + j] = col[r];
      }
    }
#pragma unroll
    for (int r = 0; r < 16; ++r)
      *reinterpret_cast<__half*>(TA + sw128_off(blk * 16 + r, j, 128)) = __float2half_rn(col[r]);
  }
}

// The same inverse on 128 threads (four warps): warp w owns columns 16 w .. 16 w + 15, lanes l and
// l + 16 share column 16 w + (l & 15).  Of a block's sixteen sums over the finished rows each lane of
// the pair takes eight; the upper lane hands its eight to the lower one, which resolves the block's
// rows and writes them out.  Every lane of the four warps must call (warp-level exchange inside).
template <int MS>
__device__ __forceinline__ void unit_lower_inverse64_pairs(const float* Msm, float* Tsm, unsigned char* TA, int t) {
  const int w = t >> 5, lane = t & 31, hh = lane >> 4, j = 16 * w + (lane & 15);
#pragma unroll 1
  for (int blk = 0; blk < 4; ++blk) {
    if (blk < w) {   // rows above the column's own block are zero (uniform per warp)
      if (hh == 0) {
#pragma unroll
        for (int r = 0; r < 16; ++r) *reinterpret_cast<__half*>(TA + sw128_off(blk * 16 + r, j, 128)) = __float2half_rn(0.f);
      }
      continue;
    }
    const float* Mb = Msm + blk * 16 * MS;
    float part[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) part[r] = 0.f;
    const float* Mh = Mb + hh * 8 * MS;
    for (int s = w * 16; s < blk * 16; s += 8) {
      float tv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) tv[i] = Tsm[(s + i) * 64 + j];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float4 m0 = *reinterpret_cast<const float4*>(Mh + r * MS + s);
        const float4 m1 = *reinterpret_cast<const float4*>(Mh + r * MS + s + 4);
        part[r] += ((m0.x * tv[0] + m0.y * tv[1]) + (m0.z * tv[2] + m0.w * tv[3])) +
                   ((m1.x * tv[4] + m1.y * tv[5]) + (m1.z * tv[6] + m1.w * tv[7]));
      }
    }
    float col[16];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const float up = __shfl_down_sync(0xffffffffu, part[r], 16);   // rows 8-15 from the upper lane
      col[r] = ((blk * 16 + r == j) ? 1.f : 0.f) - part[r];
      col[8 + r] = ((blk * 16 + 8 + r == j) ? 1.f : 0.f) - up;
    }
    if (hh == 0) {
#pragma unroll
      for (int r = 1; r < 16; ++r) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int q = 0; q < (r + 3) / 4; ++q) {
          const float4 m = *reinterpret_cast<const float4*>(Mb + r * MS + blk * 16 + 4 * q);
          a0 += m.x * col[4 * q];
          if (4 * q + 1 < r) a1 += m.y * col[4 * q + 1];
          if (4 * q + 2 < r) a0 += m.z * col[4 * q + 2];
          if (4 * q + 3 < r) a1 += m.w * col[4 * q + 3];
        }
        col[r] -= a0 + a1;
      }
      if (blk < 3) {
#pragma unroll
        for (int r = 0; r < 16; ++r) Tsm[(blk * 16 + r) * 64 + j] = col[r];
      }
#pragma unroll
      for (int r = 0; r < 16; ++r)
        *reinterpret_cast<__half*>(TA + sw128_off(blk * 16 + r, j, 128)) = __float2half_rn(col[r]);
    }
    __syncwarp();   // the upper lanes read the rows just written
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
