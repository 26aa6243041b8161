// Operand tiles and product issue helpers built on umma.cuh.
#pragma once
#include "umma.cuh"

namespace lg {

// An operand tile in shared memory: SW128 image whose atoms hold `rows` rows of 64 elements.
//   mn == false: the product contracts along the tile's columns; the tile's rows are the M (or N)
//                index.  `saddr` may point at any row that is a multiple of 8.
//   mn == true : the product contracts along the tile's rows; the tile's columns are the M (or N)
//                index.  `saddr` may point at any atom (multiple of 64 columns).
struct Tile {
  uint32_t saddr;
  uint32_t rows;
  bool mn;
};

__device__ __forceinline__ uint64_t tile_desc(const Tile& t, int kstep) {
  if (!t.mn) {
    const uint32_t a = t.saddr + static_cast<uint32_t>(kstep >> 2) * t.rows * 128u +
                       static_cast<uint32_t>(kstep & 3) * 32u;
    return make_desc(a, 16u, 1024u);
  }
  const uint32_t a = t.saddr + static_cast<uint32_t>(kstep) * 2048u;
  return make_desc(a, t.rows * 128u, 1024u);
}

// D[128 x N] (+)= A * B over a contraction of length kc (multiple of 16).  One thread calls this.
// `acc` != 0 keeps what D already holds.
__device__ __forceinline__ void issue_product(uint32_t tmem_d, const Tile& A, const Tile& B, int N, int kc,
                                              uint32_t acc, bool a_neg = false) {
  const uint32_t idesc = make_idesc(128, static_cast<uint32_t>(N), A.mn, B.mn, a_neg);
  for (int j = 0; j < kc / 16; ++j) {
    umma(tmem_d, tile_desc(A, j), tile_desc(B, j), idesc, (j > 0) ? 1u : acc);
  }
}

// The same, called by every lane of a converged warp with identical arguments; the lane whose
// `leader` (from elect_leader) is non-zero issues.  With the whole warp on the path the descriptors
// are uniform values, which is markedly cheaper per product than issuing from a one-thread branch.
__device__ __forceinline__ void issue_product_led(uint32_t leader, uint32_t tmem_d, const Tile& A, const Tile& B,
                                                  int N, int kc, uint32_t acc, bool a_neg = false) {
  const uint32_t idesc = make_idesc(128, static_cast<uint32_t>(N), A.mn, B.mn, a_neg);
  for (int j = 0; j < kc / 16; ++j) {
    umma_led(leader, tmem_d, tile_desc(A, j), tile_desc(B, j), idesc, (j > 0) ? 1u : acc);
  }
}

// ---------------------------------------------------------------------------------------------
// register <-> tile helpers (16-bit elements, 8 per 16-byte chunk)
// ---------------------------------------------------------------------------------------------
// Two floats to one fp16 pair (lo in the low half), round to nearest, SATURATING: a magnitude beyond
// the fp16 range becomes +-65504 instead of infinity, so that an out-of-range activation or gradient
// degrades a result instead of turning it (and, through 0 * inf, its neighbours) into NaN.  NaN stays NaN.
__device__ __forceinline__ uint32_t f16x2_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint4 pack8_f16(const float* v) {
  uint4 u;
  u.x = f16x2_sat(v[0], v[1]);
  u.y = f16x2_sat(v[2], v[3]);
  u.z = f16x2_sat(v[4], v[5]);
  u.w = f16x2_sat(v[6], v[7]);
  return u;
}
__device__ __forceinline__ void unpack8_f16(const uint4& u, float* v) {
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void unpack8_bf16(const uint4& u, float* v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ uint4 pack8_bf16(const float* v) {
  uint4 u;
  __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]);
  __nv_bfloat162 h1 = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]);
  __nv_bfloat162 h3 = __floats2bfloat162_rn(v[6], v[7]);
  u.x = *reinterpret_cast<uint32_t*>(&h0);
  u.y = *reinterpret_cast<uint32_t*>(&h1);
  u.z = *reinterpret_cast<uint32_t*>(&h2);
  u.w = *reinterpret_cast<uint32_t*>(&h3);
  return u;
}

// q and k arrive, and dq and dk leave, as bf16 or - when the caller says so (LetheGdnArgs::qk_f16) - as
// fp16, the type of the tensor-core operands (a caller that normalises q, k in fp32 then rounds once).
__device__ __forceinline__ void unpack8_in(const uint4& u, float* v, int f16) {
  if (f16) unpack8_f16(u, v);
  else unpack8_bf16(u, v);
}
__device__ __forceinline__ uint4 pack8_out(const float* v, int f16) { return f16 ? pack8_f16(v) : pack8_bf16(v); }
__device__ __forceinline__ void store_out16(__nv_bfloat16* dst, float x, int f16) {
  if (f16) *reinterpret_cast<__half*>(dst) = __float2half_rn(x);
  else *dst = __float2bfloat16_rn(x);
}

// chunk access on a tile given as a generic pointer to its first byte
__device__ __forceinline__ uint4 tile_ld_chunk(const unsigned char* tile, int r, int ch, int rows) {
  return *reinterpret_cast<const uint4*>(tile + sw128_chunk(r, ch, rows));
}
__device__ __forceinline__ void tile_st_chunk(unsigned char* tile, int r, int ch, int rows, const uint4& u) {
  *reinterpret_cast<uint4*>(tile + sw128_chunk(r, ch, rows)) = u;
}

}  // namespace lg
