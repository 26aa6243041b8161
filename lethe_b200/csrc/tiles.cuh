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
__device__ __forceinline__ uint4 pack8_f16(const float* v) {
  __half2 h0 = __floats2half2_rn(v[0], v[1]);
  __half2 h1 = __floats2half2_rn(v[2], v[3]);
  __half2 h2 = __floats2half2_rn(v[4], v[5]);
  __half2 h3 = __floats2half2_rn(v[6], v[7]);
  uint4 u;
  u.x = *reinterpret_cast<uint32_t*>(&h0);
  u.y = *reinterpret_cast<uint32_t*>(&h1);
  u.z = *reinterpret_cast<uint32_t*>(&h2);
  u.w = *reinterpret_cast<uint32_t*>(&h3);
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

// chunk access on a tile given as a generic pointer to its first byte
__device__ __forceinline__ uint4 tile_ld_chunk(const unsigned char* tile, int r, int ch, int rows) {
  return *reinterpret_cast<const uint4*>(tile + sw128_chunk(r, ch, rows));
}
__device__ __forceinline__ void tile_st_chunk(unsigned char* tile, int r, int ch, int rows, const uint4& u) {
  *reinterpret_cast<uint4*>(tile + sw128_chunk(r, ch, rows)) = u;
}

}  // namespace lg
