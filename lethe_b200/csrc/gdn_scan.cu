// The serial part of the path: the chunk-to-chunk state recurrence, forward and adjoint.
//
//   forward :  x_{c+1} = a_c * x_c - P_c   x_c + R_c      c = 0 .. NT-1     (x_0 = h0)
//   adjoint :  x_{c-1} = a_c * x_c - P_c^T x_c + Rb_c     c = NT-1 .. 0     (x_NT = dhT)
//
// a_c is the chunk's decay per key channel, P_c = kd^T w (128 x 128) and R_c / Rb_c (128 x V) come
// from the chunk-parallel kernels.  The recurrence is independent per column of x, so the grid is
// (V / 16) x (B*H): every CTA owns 16 columns, keeps them as fp32 in registers (thread d = key
// channel d) and does ONE tcgen05 product per chunk, with P streamed through a ring of shared-memory
// stages by bulk copies that run ahead of the recurrence.  The state seen by chunk c is written out
// as a shared-memory tile image for the chunk-parallel kernels.
// Reference: the forward recurrence gdn2_chunkwise.py:155-158 and the reverse scan K#1
// gdn2_assemble.py:71-99 of the reference project, after substituting v_new / dv2.
#include "gdn_common.cuh"
#include "host_util.h"

namespace lg {

constexpr int kStages = 3;
constexpr int kVs = 16;  // columns of the state per CTA

template <bool ADJOINT>
__global__ void __launch_bounds__(128)
scan_kernel(const Problem p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                       ~static_cast<uintptr_t>(1023));
  unsigned char* Pst = sm;                          // kStages x 32 KB
  unsigned char* XB = sm + kStages * 32768;         // 4 KB: x as a (16 x 128) operand, 2 atoms of 2 KB
  CtaShared* cs = reinterpret_cast<CtaShared*>(XB + 4096);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int v0 = blockIdx.x * kVs, bh = blockIdx.y;
  const int V = p.V, NT = p.NT;
  const bool has_p = p.delta != 0;
  CtaCtl ctl{p.status, &cs->abort_flag};
  uint64_t* bar_mma = &cs->bar[kStages];

  if (tid == 0) {
    cs->abort_flag = 0;
    for (int s = 0; s < kStages; ++s) mbar_init(&cs->bar[s], 1);
    mbar_init(bar_mma, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;

  const unsigned char* Pg = p.saved + p.lay.p;
  const __half* Rg = reinterpret_cast<const __half*>(ADJOINT ? p.scratch + p.lay.rb : p.saved + p.lay.r);
  const float* ADg = reinterpret_cast<const float*>(p.saved + p.lay.ad);
  unsigned char* Xg = ADJOINT ? p.scratch + p.lay.dh : p.saved + p.lay.hc;
  const size_t szx = p.lay.sz_hc;
  auto chunk_of = [&](int it) { return ADJOINT ? NT - 1 - it : it; };

  if (has_p && tid == 0) {
    for (int s = 0; s < kStages && s < NT; ++s) {
      mbar_expect_tx(&cs->bar[s], 32768u);
      bulk_g2s(Pst + s * 32768, Pg + (static_cast<size_t>(bh) * NT + chunk_of(s)) * 32768, 32768u, &cs->bar[s]);
    }
  }

  float x[kVs];
  {
    const float* x0 = ADJOINT ? p.dhT : p.h0;
#pragma unroll
    for (int j = 0; j < kVs; ++j)
      x[j] = x0 ? x0[(static_cast<size_t>(bh) * kK + tid) * V + v0 + j] : 0.f;
  }
  uint4 rnext[2];
  {
    const __half* r = Rg + ((static_cast<size_t>(bh) * NT + chunk_of(0)) * kK + tid) * V + v0;
    rnext[0] = *reinterpret_cast<const uint4*>(r);
    rnext[1] = *reinterpret_cast<const uint4*>(r + 8);
  }

  float a_next = ADg[(static_cast<size_t>(bh) * NT + chunk_of(0)) * kK + tid];
  for (int it = 0; it < NT; ++it) {
    const int c = chunk_of(it);
    const size_t z = static_cast<size_t>(bh) * NT + c;
    const int st = it % kStages;
    const uint32_t st_par = static_cast<uint32_t>((it / kStages) & 1);
    const float a = a_next;
    const uint4 r0 = rnext[0], r1 = rnext[1];
    if (it + 1 < NT) {   // next chunk's decay and input: a whole step of latency cover
      const size_t zn = static_cast<size_t>(bh) * NT + chunk_of(it + 1);
      const __half* r = Rg + (zn * kK + tid) * V + v0;
      rnext[0] = *reinterpret_cast<const uint4*>(r);
      rnext[1] = *reinterpret_cast<const uint4*>(r + 8);
      a_next = ADg[zn * kK + tid];
    }
    if (has_p) {
      // critical path: the state as a tensor-core operand, then the product
#pragma unroll
      for (int n = 0; n < kVs; ++n)
        *reinterpret_cast<__half*>(XB + sw128_off(n, tid, kVs)) = __float2half_rn(x[n]);
      fence_proxy_async();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        mbar_wait(&cs->bar[st], st_par, ctl, 301);
        tc_fence_after();
        issue_product(tmem, Tile{smem_u32(Pst + st * 32768), 128, ADJOINT}, Tile{smem_u32(XB), kVs, false},
                      kVs, 128, 0u);
        umma_commit(bar_mma);
      }
      __syncwarp();
    }
    // off the critical path (overlaps the product): the state record
    {
      unsigned char* rec = Xg + (ADJOINT ? z : z + bh) * szx;
      *reinterpret_cast<uint4*>(rec + sw128_chunk(tid, v0 / 8, 128)) = pack8_f16(x);
      *reinterpret_cast<uint4*>(rec + sw128_chunk(tid, v0 / 8 + 1, 128)) = pack8_f16(x + 8);
    }
    float rr[kVs];
    unpack8_f16(r0, rr);
    unpack8_f16(r1, rr + 8);
    if (has_p) {
      mbar_wait_warp(bar_mma, static_cast<uint32_t>(it & 1), ctl, 302);
      tc_fence_after();
      float acc[kVs];
      tmem_ld16(tmem + lane_base, acc);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < kVs; ++j) x[j] = a * x[j] + rr[j] - acc[j];
      if (tid == 0 && it + kStages < NT) {
        mbar_expect_tx(&cs->bar[st], 32768u);
        bulk_g2s(Pst + st * 32768, Pg + (static_cast<size_t>(bh) * NT + chunk_of(it + kStages)) * 32768, 32768u,
                 &cs->bar[st]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < kVs; ++j) x[j] = a * x[j] + rr[j];
    }
  }
  if (!ADJOINT) {   // the final state as one more record (the adjoint of the gate needs it)
    unsigned char* rec = Xg + (static_cast<size_t>(bh) * (NT + 1) + NT) * szx;
    *reinterpret_cast<uint4*>(rec + sw128_chunk(tid, v0 / 8, 128)) = pack8_f16(x);
    *reinterpret_cast<uint4*>(rec + sw128_chunk(tid, v0 / 8 + 1, 128)) = pack8_f16(x + 8);
  }
  float* xT = ADJOINT ? p.dh0 : p.hT;
  if (xT) {
#pragma unroll
    for (int j = 0; j < kVs; j += 4)
      *reinterpret_cast<float4*>(xT + (static_cast<size_t>(bh) * kK + tid) * V + v0 + j) =
          make_float4(x[j], x[j + 1], x[j + 2], x[j + 3]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 32);
}

int launch_scan(const Problem& p, bool adjoint, cudaStream_t st) {
  const int smem = kStages * 32768 + 4096 + static_cast<int>(sizeof(CtaShared)) + 1024;
  dim3 grid(p.V / kVs, p.B * p.H);
  if (adjoint) {
    if (cudaFuncSetAttribute(scan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return kErrLaunch;
    scan_kernel<true><<<grid, 128, smem, st>>>(p);
  } else {
    if (cudaFuncSetAttribute(scan_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return kErrLaunch;
    scan_kernel<false><<<grid, 128, smem, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

}  // namespace lg
