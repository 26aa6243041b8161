// Token-serial form of the path for generation: one recurrence step per (batch, head) pair with the
// state kept in HBM between calls,
//
//   S <- S * exp(g);   v_new = beta (v - k^T S);   S <- S + k v_new^T;   o = (scale q)^T S
//
// (reference gdn_backward.py:45-53, one iteration of its token loop; beta == null drops the delta term).
// The step is bound by reading and writing the fp32 state once: K x V x 4 bytes each way per pair.
// One CTA of 4 V threads per pair: four threads share column c of S (32 rows each) and keep their
// entries in registers between the two passes over the column (first k^T S, then the update and q^T S), so the state crosses HBM
// exactly once in each direction and every load of a warp is one contiguous row segment.  No tensor
// cores: 4 flops per state byte.
#include <cuda_bf16.h>

#include "../../include/lethe_gdn.h"
#include "host_util.h"

namespace lg {

constexpr int kDK = 128;

struct DecodeProblem {
  int BH, H, V, gate, delta;
  float scale;
  const __nv_bfloat16 *q, *k, *v;
  const float *g, *beta;
  float* state;
  __nv_bfloat16* o;
};

// kSplit threads share a column of S (kDK / kSplit rows each).
constexpr int kSplit = 4;

template <int V>
__global__ void __launch_bounds__(kSplit * V, 1024 / (kSplit * V))
decode_step_kernel(const DecodeProblem p) {
  __shared__ float ks[kDK], qs[kDK], as[kDK], part[kSplit][V];
  const int bh = blockIdx.x, c = threadIdx.x % V, part_id = threadIdx.x / V;   // rows [kRows part_id, + kRows)
  for (int d = threadIdx.x; d < kDK; d += kSplit * V) {
    ks[d] = __bfloat162float(p.k[static_cast<size_t>(bh) * kDK + d]);
    qs[d] = p.scale * __bfloat162float(p.q[static_cast<size_t>(bh) * kDK + d]);
    float a = 1.f;
    if (p.gate == LETHE_GATE_SCALAR) a = __expf(p.g[bh]);
    else if (p.gate == LETHE_GATE_CHANNEL) a = __expf(p.g[static_cast<size_t>(bh) * kDK + d]);
    as[d] = a;
  }
  constexpr int kRows = kDK / kSplit;
  float* S = p.state + (static_cast<size_t>(bh) * kDK + part_id * kRows) * V + c;
  float col[kRows];
#pragma unroll
  for (int d = 0; d < kRows; ++d) col[d] = S[static_cast<size_t>(d) * V];   // all loads in flight at once
  __syncthreads();
  const float* kh = ks + part_id * kRows;
  const float* qh = qs + part_id * kRows;
  const float* ah = as + part_id * kRows;
  float ksum = 0.f;
#pragma unroll
  for (int d = 0; d < kRows; ++d) {
    col[d] *= ah[d];
    ksum += kh[d] * col[d];
  }
  part[part_id][c] = ksum;
  __syncthreads();
  ksum = 0.f;
#pragma unroll
  for (int s = 0; s < kSplit; ++s) ksum += part[s][c];
  float vn = __bfloat162float(p.v[static_cast<size_t>(bh) * V + c]);
  if (p.delta) vn = p.beta[bh] * (vn - ksum);
  float o = 0.f;
#pragma unroll
  for (int d = 0; d < kRows; ++d) {
    col[d] += kh[d] * vn;
    o += qh[d] * col[d];
    S[static_cast<size_t>(d) * V] = col[d];
  }
  __syncthreads();
  part[part_id][c] = o;
  __syncthreads();
  if (part_id == 0) {
    float os = 0.f;
#pragma unroll
    for (int s = 0; s < kSplit; ++s) os += part[s][c];
    p.o[static_cast<size_t>(bh) * V + c] = __float2bfloat16_rn(os);
  }
}

}  // namespace lg

extern "C" int lethe_gdn_decode_step(const LetheGdnDecodeArgs* a, void* stream) {
  using namespace lg;
  if (!a || !a->q || !a->k || !a->v || !a->state || !a->o) return kErrNull;
  if (a->B <= 0 || a->H <= 0 || a->K != kDK || (a->V != 64 && a->V != 128)) return kErrDims;
  if (a->gate != LETHE_GATE_NONE && a->gate != LETHE_GATE_SCALAR && a->gate != LETHE_GATE_CHANNEL) return kErrFlags;
  if (a->gate != LETHE_GATE_NONE && !a->g) return kErrNull;
  if (a->delta && !a->beta) return kErrNull;
  DeviceGuard guard(a->state);
  if (!guard.ok) return kErrDevice;
  DecodeProblem p;
  p.BH = a->B * a->H;
  p.H = a->H;
  p.V = a->V;
  p.gate = a->gate;
  p.delta = a->delta;
  p.scale = a->scale;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.v = static_cast<const __nv_bfloat16*>(a->v);
  p.g = a->g;
  p.beta = a->beta;
  p.state = a->state;
  p.o = static_cast<__nv_bfloat16*>(a->o);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->V == 64) decode_step_kernel<64><<<p.BH, kSplit * 64, 0, st>>>(p);
  else decode_step_kernel<128><<<p.BH, kSplit * 128, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
