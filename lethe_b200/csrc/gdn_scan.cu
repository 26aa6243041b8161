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
constexpr int kVs = 16;        // columns of the state per CTA
constexpr int kMmaWarps = 2;   // warps that issue the step's products (each its own accumulator)
// warps 0-3 hold the state (thread d = key channel d), warp 4 streams P, warps 5.. issue products
constexpr int kScanThreads = (5 + kMmaWarps) * 32;
constexpr int kStepBarrier = 128 + kMmaWarps * 32;
constexpr int kTmemCols = kMmaWarps * 16 < 32 ? 32 : kMmaWarps * 16;

// Step barrier of the delta path: the state-holding warps arrive once the operand is written (and go
// on to work that does not depend on the product), the issuing warps wait for them.
__device__ __forceinline__ void step_arrive() { asm volatile("bar.arrive 1, %0;" ::"n"(kStepBarrier) : "memory"); }
__device__ __forceinline__ void step_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kStepBarrier) : "memory"); }

template <bool ADJOINT>
__global__ void __launch_bounds__(kScanThreads)
scan_kernel(const Problem p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = align1024_generic(smem_raw);
  unsigned char* Pst = sm;                          // kStages x 32 KB
  // 4 KB: x as the B operand, contracted along its rows (row k = key channel k, 16 columns = 32 bytes):
  // atoms of 8 rows x 32 bytes with the 32-byte swizzle, so that thread k stores its row as two 16-byte pieces
  unsigned char* XB = sm + kStages * 32768;
  CtaShared* cs = reinterpret_cast<CtaShared*>(XB + 4096);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int v0 = blockIdx.x * kVs, bh = blockIdx.y + p.bh0;
  // This launch walks the chunks [c0, c0 + cn) of every pair (all NT of them in an ordinary call), forward in
  // chunk order, the adjoint in reverse.  A launch that does not start at the sequence's first (adjoint: last)
  // chunk takes its fp32 state from the carry buffer the launch before it left, and one that does not end at
  // the other end leaves its state there: a scan cut into chunk ranges is bit-identical to one launch.
  const int V = p.V, NT = p.NT, n = p.cn;
  const bool seg_first = ADJOINT ? (p.c0 + p.cn == NT) : (p.c0 == 0);
  const bool seg_last = ADJOINT ? (p.c0 == 0) : (p.c0 + p.cn == NT);
  CtaCtl ctl{p.status, &cs->abort_flag};
  uint64_t* bar_full = &cs->bar[0];                 // [kStages] P stage loaded
  uint64_t* bar_free = &cs->bar[kStages];           // [kStages] the products reading the stage are done
  uint64_t* bar_mma = &cs->bar[2 * kStages];        // the step's products are done

  if (tid == 0) {
    cs->abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_free[s], kMmaWarps);
    }
    mbar_init(bar_mma, kMmaWarps);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&cs->tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = cs->tmem_slot;
  auto chunk_of = [&](int it) { return ADJOINT ? p.c0 + n - 1 - it : p.c0 + it; };
  // The kernel before this one wrote R (forward) or Rb (adjoint); P comes from the same kernel in the
  // forward and from the forward call in the adjoint, whose producer may start at once.
  if (!(ADJOINT && warp == 4)) {
    griddep_wait();
    griddep_launch();
  }

  if (warp == 4) {
    // ---- producer: keeps the ring of P stages full
    if (tid == 128) {
      const unsigned char* Pg = p.saved + p.lay.p;
      for (int it = 0; it < n; ++it) {
        const int st = it % kStages;
        if (it >= kStages) mbar_wait(&bar_free[st], static_cast<uint32_t>(((it / kStages) - 1) & 1), ctl, 303);
        mbar_expect_tx(&bar_full[st], 32768u);
        bulk_g2s(Pst + st * 32768, Pg + (static_cast<size_t>(bh) * NT + chunk_of(it)) * 32768, 32768u, &bar_full[st]);
      }
    }
  } else if (warp > 4) {
    // ---- product issue: warp m takes contraction steps [m * 8 / kMmaWarps, ...) into accumulator m.
    // All lanes stay on the path (uniform descriptors); the elected lane issues.
    const int m = warp - 5;
    constexpr int kPer = 8 / kMmaWarps;
    const uint32_t leader = elect_leader();
    // A = the P stage (contracted along its columns forward, along its rows for the adjoint),
    // B = the state operand; one 16-element contraction step moves each by a fixed amount
    const uint64_t b_desc0 = make_desc_sw32(smem_u32(XB), 16u, 256u);
    const uint32_t idesc = make_idesc(128, kVs, ADJOINT, true);
    const uint32_t acc = tmem + static_cast<uint32_t>(m * kVs);
    for (int it = 0; it < n; ++it) {
      const int st = it % kStages;
      mbar_wait_warp(&bar_full[st], static_cast<uint32_t>((it / kStages) & 1), ctl, 301);
      step_sync();
      tc_fence_after();
      const uint32_t pa = smem_u32(Pst + st * 32768);
      const uint64_t a_desc0 = ADJOINT ? make_desc(pa, 16384u, 1024u) : make_desc(pa, 16u, 1024u);
#pragma unroll
      for (int jj = 0; jj < kPer; ++jj) {
        const int j = m * kPer + jj;
        // byte offsets of contraction step j, in the descriptors' 16-byte units
        const uint32_t aoff = ADJOINT ? static_cast<uint32_t>(j * 2048) >> 4
                                      : static_cast<uint32_t>((j >> 2) * 16384 + (j & 3) * 32) >> 4;
        const uint32_t boff = static_cast<uint32_t>(j * 512) >> 4;     // 16 rows of 32 bytes per step
        umma_led(leader, acc, a_desc0 + aoff, b_desc0 + boff, idesc, jj > 0 ? 1u : 0u);
      }
      umma_commit_led(leader, bar_mma);
      umma_commit_led(leader, &bar_free[st]);
    }
  } else {
    // ---- the state: thread d holds row d of x (16 columns) in fp32
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const __half* Rg = reinterpret_cast<const __half*>(ADJOINT ? p.scratch + p.lay.rb : p.saved + p.lay.r);
    const float* ADg = reinterpret_cast<const float*>(p.saved + p.lay.ad);
    unsigned char* Xg = ADJOINT ? p.scratch + p.lay.dh : p.saved + p.lay.hc;
    const size_t szx = p.lay.sz_hc;
    // R / Rb records are [V / 16 column blocks][128 rows][16 columns]: this CTA's block, this thread's row
    const size_t rofs = (static_cast<size_t>(blockIdx.x) * kK + tid) * kVs;

    float* carry = reinterpret_cast<float*>(ADJOINT ? p.scratch + p.lay.carry_b : p.saved + p.lay.carry_f);
    float x[kVs];
    {
      const float* x0 = seg_first ? (ADJOINT ? p.dhT : p.h0) : carry;
#pragma unroll
      for (int j = 0; j < kVs; ++j) x[j] = x0 ? x0[(static_cast<size_t>(bh) * kK + tid) * V + v0 + j] : 0.f;
    }
    uint4 rnext[2];
    {
      const __half* r = Rg + (static_cast<size_t>(bh) * NT + chunk_of(0)) * kK * V + rofs;
      rnext[0] = *reinterpret_cast<const uint4*>(r);
      rnext[1] = *reinterpret_cast<const uint4*>(r + 8);
    }
    float a_next = ADg[(static_cast<size_t>(bh) * NT + chunk_of(0)) * kK + tid];

    for (int it = 0; it < n; ++it) {
      const size_t z = static_cast<size_t>(bh) * NT + chunk_of(it);
      // critical path: the state as a tensor-core operand
      {
        const int sw = (tid >> 2) & 1;     // 32-byte swizzle: the two 16-byte pieces of rows 4-7 of an atom swap
        *reinterpret_cast<uint4*>(XB + tid * 32 + (sw << 4)) = pack8_f16(x);
        *reinterpret_cast<uint4*>(XB + tid * 32 + ((sw ^ 1) << 4)) = pack8_f16(x + 8);
      }
      fence_proxy_async();
      tc_fence_before();
      step_arrive();
      // in the shadow of the product: this chunk's input and decay, the next chunk's loads, the record
      const float a = a_next;
      float rr[kVs];
      unpack8_f16(rnext[0], rr);
      unpack8_f16(rnext[1], rr + 8);
#pragma unroll
      for (int j = 0; j < kVs; ++j) rr[j] = fmaf(a, x[j], rr[j]);
      if (it + 1 < n) {
        const size_t zn = static_cast<size_t>(bh) * NT + chunk_of(it + 1);
        const __half* r = Rg + zn * kK * V + rofs;
        rnext[0] = *reinterpret_cast<const uint4*>(r);
        rnext[1] = *reinterpret_cast<const uint4*>(r + 8);
        a_next = ADg[zn * kK + tid];
      }
      {
        unsigned char* rec = Xg + (ADJOINT ? z : z + bh) * szx;
        *reinterpret_cast<uint4*>(rec + sw128_chunk(tid, v0 / 8, 128)) = pack8_f16(x);
        *reinterpret_cast<uint4*>(rec + sw128_chunk(tid, v0 / 8 + 1, 128)) = pack8_f16(x + 8);
      }
      mbar_wait_warp(bar_mma, static_cast<uint32_t>(it & 1), ctl, 302);
      tc_fence_after();
      float acc[kMmaWarps * kVs];
      if (kMmaWarps == 1) tmem_ld16(tmem + lane_base, acc);
      if (kMmaWarps >= 2) tmem_ld32(tmem + lane_base, acc);
      if (kMmaWarps == 4) tmem_ld32(tmem + lane_base + 32, acc + 32);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < kVs; ++j) {
        float s = acc[j];
        if (kMmaWarps >= 2) s += acc[kVs + j];
        if (kMmaWarps == 4) s += acc[2 * kVs + j] + acc[3 * kVs + j];
        x[j] = rr[j] - s;
      }
    }
    if (!ADJOINT && seg_last) {   // the final state as one more record
      unsigned char* rec = Xg + (static_cast<size_t>(bh) * (NT + 1) + NT) * szx;
      *reinterpret_cast<uint4*>(rec + sw128_chunk(tid, v0 / 8, 128)) = pack8_f16(x);
      *reinterpret_cast<uint4*>(rec + sw128_chunk(tid, v0 / 8 + 1, 128)) = pack8_f16(x + 8);
    }
    float* xT = seg_last ? (ADJOINT ? p.dh0 : p.hT) : carry;
    if (xT) {
#pragma unroll
      for (int j = 0; j < kVs; j += 4)
        *reinterpret_cast<float4*>(xT + (static_cast<size_t>(bh) * kK + tid) * V + v0 + j) =
            make_float4(x[j], x[j + 1], x[j + 2], x[j + 3]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// Without the delta term the recurrence is x <- a x + R per element: no product, nothing serial but the
// chunk order, and the kernel is bound by reading R and writing the state records once.  Every thread
// owns one 16-byte piece (8 columns) of one row of the state; a warp covers four whole 128-byte rows
// of a record atom, so every access is a full line.  R / Rb and the state records are 128-row tile images.
// Grid: (V / 64 atoms x 4 row blocks, pairs) x 256 threads.
// ---------------------------------------------------------------------------------------------
template <bool ADJOINT>
__global__ void __launch_bounds__(256)
scan_nodelta_kernel(const Problem p) {
  const int tid = threadIdx.x;
  const int atom = blockIdx.x >> 2, d = (blockIdx.x & 3) * 32 + (tid >> 3), c8 = tid & 7;
  const int bh = blockIdx.y + p.bh0, V = p.V, NT = p.NT, n = p.cn;
  const bool seg_first = ADJOINT ? (p.c0 + p.cn == NT) : (p.c0 == 0);        // chunk ranges as in scan_kernel
  const bool seg_last = ADJOINT ? (p.c0 == 0) : (p.c0 + p.cn == NT);
  float* carry = reinterpret_cast<float*>(ADJOINT ? p.scratch + p.lay.carry_b : p.saved + p.lay.carry_f);
  const int col0 = atom * 64 + c8 * 8;
  griddep_wait();
  griddep_launch();
  const unsigned char* Rg = ADJOINT ? p.scratch + p.lay.rb : p.saved + p.lay.r;
  const float* ADg = reinterpret_cast<const float*>(p.saved + p.lay.ad);
  unsigned char* Xg = ADJOINT ? p.scratch + p.lay.dh : p.saved + p.lay.hc;
  const size_t szx = p.lay.sz_hc;
  const uint32_t off = sw128_chunk(d, atom * 8 + c8, 128);     // this thread's piece inside any 128-row image
  auto chunk_of = [&](int it) { return ADJOINT ? p.c0 + n - 1 - it : p.c0 + it; };

  float x[8];
  {
    const float* x0 = seg_first ? (ADJOINT ? p.dhT : p.h0) : carry;
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = x0 ? x0[(static_cast<size_t>(bh) * kK + d) * V + col0 + j] : 0.f;
  }
  constexpr int kBatch = 8;
  for (int it0 = 0; it0 < n; it0 += kBatch) {
    uint4 rb[kBatch];
    float ab[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (it0 + j < n) {
        const size_t zj = static_cast<size_t>(bh) * NT + chunk_of(it0 + j);
        rb[j] = *reinterpret_cast<const uint4*>(Rg + zj * p.lay.sz_r + off);
        ab[j] = ADg[zj * kK + d];
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (it0 + j < n) {
        const size_t zj = static_cast<size_t>(bh) * NT + chunk_of(it0 + j);
        *reinterpret_cast<uint4*>(Xg + (ADJOINT ? zj : zj + bh) * szx + off) = pack8_f16(x);
        float rr[8];
        unpack8_f16(rb[j], rr);
#pragma unroll
        for (int n = 0; n < 8; ++n) x[n] = fmaf(ab[j], x[n], rr[n]);
      }
    }
  }
  if (!ADJOINT && seg_last)   // the final state as one more record
    *reinterpret_cast<uint4*>(Xg + (static_cast<size_t>(bh) * (NT + 1) + NT) * szx + off) = pack8_f16(x);
  float* xT = seg_last ? (ADJOINT ? p.dh0 : p.hT) : carry;
  if (xT) {
    float* dst = xT + (static_cast<size_t>(bh) * kK + d) * V + col0;
    *reinterpret_cast<float4*>(dst) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(x[4], x[5], x[6], x[7]);
  }
}

int launch_scan(const Problem& p, bool adjoint, cudaStream_t st) {
  if (!p.delta) {
    const dim3 g((p.V / 64) * 4, p.nbh);
    const cudaError_t e = adjoint ? launch_dependent(scan_nodelta_kernel<true>, g, dim3(256), 0, st, p)
                                  : launch_dependent(scan_nodelta_kernel<false>, g, dim3(256), 0, st, p);
    return e == cudaSuccess ? kOk : kErrLaunch;
  }
  const int smem = kStages * 32768 + 4096 + static_cast<int>(sizeof(CtaShared)) + 1024;
  dim3 grid(p.V / kVs, p.nbh);
  if (adjoint) {
    static SmemAttr attr;
    if (attr.set(scan_kernel<true>, smem)) return kErrLaunch;
    if (launch_dependent(scan_kernel<true>, grid, dim3(kScanThreads), smem, st, p) != cudaSuccess) return kErrLaunch;
  } else {
    static SmemAttr attr;
    if (attr.set(scan_kernel<false>, smem)) return kErrLaunch;
    if (launch_dependent(scan_kernel<false>, grid, dim3(kScanThreads), smem, st, p) != cudaSuccess) return kErrLaunch;
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

}  // namespace lg
