// L2 normalisation of q and k on the input side of the path and its VJP on the output side
// (reference gdn_backward.py:9-10: y = x * rsqrt(sum x^2 + eps), eps inside the root; the reference
// differentiates it by autograd, gdn2_assemble.py:300-312):
//
//   forward    y  = x r,                       r = rsqrt(sum_d x_d^2 + eps)
//   backward   dx = r (dy - y (y . dy))        (exact, eps included: d r / d x = -r^3 x)
//
// One launch covers q and k.  A row of D channels is held by D / 8 neighbouring lanes, 8 channels
// (one 16-byte piece of bf16) each; the row sum is a butterfly over those lanes.  HBM-bound: the
// forward moves 2 D + 2 D bytes per row and tensor (4 D + 2 D for fp32 inputs), the backward
// reads x and dy and writes dx.  The normalised rows leave as bf16 or as fp16 (the operand type of
// the GDN kernels: one rounding instead of two), and their gradients come back in the same type.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../../include/lethe_gdn.h"
#include "host_util.h"

namespace lg {

template <bool F32>
__device__ __forceinline__ void load8(const void* base, size_t idx, float* x) {
  if (F32) {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
    const float4 a = p[0], b = p[1];
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + idx);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      x[2 * j] = f.x;
      x[2 * j + 1] = f.y;
    }
  }
}

template <bool F32>
__device__ __forceinline__ void store8(void* base, size_t idx, const float* x) {
  if (F32) {
    float4* p = reinterpret_cast<float4*>(static_cast<float*>(base) + idx);
    p[0] = make_float4(x[0], x[1], x[2], x[3]);
    p[1] = make_float4(x[4], x[5], x[6], x[7]);
  } else {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(base) + idx) = u;
  }
}

// 16-bit rows: bf16 or fp16, chosen at run time
__device__ __forceinline__ void load8_16(const void* base, size_t idx, float* x, int f16) {
  const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + idx);
  if (f16) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      x[2 * j] = f.x;
      x[2 * j + 1] = f.y;
    }
  } else {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      x[2 * j] = f.x;
      x[2 * j + 1] = f.y;
    }
  }
}
__device__ __forceinline__ void store8_16(void* base, size_t idx, const float* x, int f16) {
  uint4 u;
  if (f16) {
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(x[2 * j], x[2 * j + 1]);
  } else {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
  }
  *reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + idx) = u;
}

template <int LANES>
__device__ __forceinline__ float row_sum(float s) {
#pragma unroll
  for (int m = LANES / 2; m >= 1; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
  return s;
}

struct L2Problem {
  const void* x[2];     // q, k
  const void* dy[2];    // backward: gradients of the normalised rows (bf16 or fp16)
  void* out[2];         // forward: normalised rows (bf16 or fp16); backward: dx in the type of x
  long long rows;
  float eps;
  int norm_f16;         // the normalised rows and their gradients are fp16
};

// grid.y selects the tensor; LANES = D / 8 lanes per row.  A thread works on kPieces 16-byte pieces, 256
// pieces apart, and requests all of them before it uses the first: with one piece per thread an SM has
// 32 KB of loads in flight, too little to cover the latency of HBM (the forward reached 0.44 of the copy
// bandwidth that way).
constexpr int kPieces = 4;

template <int LANES, bool F32, bool BACKWARD>
__global__ void __launch_bounds__(256)
l2norm_qk_kernel(const L2Problem p) {
  const int t = blockIdx.y;
  const long long first = static_cast<long long>(blockIdx.x) * (256 * kPieces) + threadIdx.x;
  // a warp never straddles the end of the tensor inside a row: rows * LANES pieces are padded to whole
  // CTAs by the row test only, so every lane of a live row takes part in the butterfly
  bool live[kPieces];
  size_t idx[kPieces];
  float x[kPieces][8], dy[BACKWARD ? kPieces : 1][8];
#pragma unroll
  for (int u = 0; u < kPieces; ++u) {
    const long long piece = first + u * 256;
    live[u] = piece / LANES < p.rows;
    idx[u] = static_cast<size_t>(live[u] ? piece : 0) * 8;
  }
#pragma unroll
  for (int u = 0; u < kPieces; ++u) load8<F32>(p.x[t], idx[u], x[u]);
  if (BACKWARD) {
#pragma unroll
    for (int u = 0; u < kPieces; ++u) load8_16(p.dy[t], idx[u], dy[u], p.norm_f16);
  }
#pragma unroll
  for (int u = 0; u < kPieces; ++u) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(x[u][j], x[u][j], ss);
    const float r = rsqrtf(row_sum<LANES>(ss) + p.eps);
    if (!BACKWARD) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[u][j] *= r;
      if (live[u]) store8_16(p.out[t], idx[u], x[u], p.norm_f16);
    } else {
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) dot = fmaf(x[u][j], dy[u][j], dot);
      const float c = row_sum<LANES>(dot) * r * r;       // dx = r dy - x r^3 (x . dy)
#pragma unroll
      for (int j = 0; j < 8; ++j) x[u][j] = r * (dy[u][j] - x[u][j] * c);
      if (live[u]) store8<F32>(p.out[t], idx[u], x[u]);
    }
  }
}

template <bool BACKWARD>
int launch_l2norm(const L2Problem& p, int D, bool f32, cudaStream_t st) {
  const int lanes = D / 8;
  const long long pieces = p.rows * lanes;
  const int per_cta = 256 * kPieces;
  const dim3 grid(static_cast<unsigned>((pieces + per_cta - 1) / per_cta), 2);
  if (lanes == 16) {
    if (f32) l2norm_qk_kernel<16, true, BACKWARD><<<grid, 256, 0, st>>>(p);
    else l2norm_qk_kernel<16, false, BACKWARD><<<grid, 256, 0, st>>>(p);
  } else {
    if (f32) l2norm_qk_kernel<8, true, BACKWARD><<<grid, 256, 0, st>>>(p);
    else l2norm_qk_kernel<8, false, BACKWARD><<<grid, 256, 0, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

inline bool aligned16(const void* a) { return (reinterpret_cast<uintptr_t>(a) & 15) == 0; }

}  // namespace lg

extern "C" int lethe_gdn_l2norm_qk(const void* q, const void* k, void* qn, void* kn, int64_t rows, int32_t D,
                                   int32_t flags, float eps, void* stream) {
  using namespace lg;
  if (!q || !k || !qn || !kn) return kErrNull;
  if (rows <= 0 || (D != 64 && D != 128)) return kErrDims;
  if (!aligned16(q) || !aligned16(k) || !aligned16(qn) || !aligned16(kn)) return kErrAlign;
  DeviceGuard guard(q);
  if (!guard.ok) return kErrDevice;
  L2Problem p{{q, k}, {nullptr, nullptr}, {qn, kn}, rows, eps, (flags & LETHE_L2_NORM_F16) ? 1 : 0};
  return launch_l2norm<false>(p, D, (flags & LETHE_L2_IN_F32) != 0, static_cast<cudaStream_t>(stream));
}

extern "C" int lethe_gdn_l2norm_qk_vjp(const void* q, const void* k, const void* dqn, const void* dkn, void* dq,
                                       void* dk, int64_t rows, int32_t D, int32_t flags, float eps,
                                       void* stream) {
  using namespace lg;
  if (!q || !k || !dqn || !dkn || !dq || !dk) return kErrNull;
  if (rows <= 0 || (D != 64 && D != 128)) return kErrDims;
  if (!aligned16(q) || !aligned16(k) || !aligned16(dqn) || !aligned16(dkn) || !aligned16(dq) || !aligned16(dk))
    return kErrAlign;
  DeviceGuard guard(q);
  if (!guard.ok) return kErrDevice;
  L2Problem p{{q, k}, {dqn, dkn}, {dq, dk}, rows, eps, (flags & LETHE_L2_NORM_F16) ? 1 : 0};
  return launch_l2norm<true>(p, D, (flags & LETHE_L2_IN_F32) != 0, static_cast<cudaStream_t>(stream));
}
