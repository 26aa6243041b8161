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
constexpr int kMmaWarps = 2;   // warps that issue the step's products (each its own accumulator)
// Columns of the state per CTA (template parameter kVs of the kernel): 16, or 32 when the 16-column CTAs of a
// launch could not all be resident at once.  With 32 columns the scan needs half the CTAs and reads P half as
// often, but a step takes about a fifth longer (measured: 39 against 33 us for 32 chunks), so the narrow form
// is kept wherever it fits in one wave.
// warps 0-3 hold the state (thread d = key channel d), warp 4 streams P, warps 5.. issue products
constexpr int kScanThreads = (5 + kMmaWarps) * 32;
constexpr int kStepBarrier = 128 + kMmaWarps * 32;

// Step barrier of the delta path: the state-holding warps arrive once the operand is written (and go
// on to work that does not depend on the product), the issuing warps wait for them.
__device__ __forceinline__ void step_arrive() { asm volatile("bar.arrive 1, %0;" ::"n"(kStepBarrier) : "memory"); }
__device__ __forceinline__ void step_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kStepBarrier) : "memory"); }

template <bool ADJOINT, int kVs>
__global__ void __launch_bounds__(kScanThreads, 2)
scan_kernel(const Problem p) {
  constexpr int kTmemCols = kMmaWarps * kVs;        // 32 or 64
  constexpr int kXB = 128 * kVs * 2;                 // bytes of the state operand tile
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = align1024_generic(smem_raw);
  unsigned char* Pst = sm;                          // kStages x 32 KB
  // x as the B operand, contracted along its rows (row k = key channel k, kVs columns = 32 or 64 bytes):
  // atoms of 8 rows x 32 (64) bytes with the 32-byte (64-byte) swizzle, so that thread k stores its row as
  // two (four) 16-byte pieces
  unsigned char* XB = sm + kStages * 32768;
  CtaShared* cs = reinterpret_cast<CtaShared*>(XB + kXB);

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
    const uint64_t b_desc0 = kVs == 16 ? make_desc_sw32(smem_u32(XB), 16u, 256u) : make_desc_sw64(smem_u32(XB), 16u, 512u);
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
        const uint32_t boff = static_cast<uint32_t>(j * 32 * kVs) >> 4;     // 16 rows of 2 kVs bytes per step
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
    const size_t rofs = (static_cast<size_t>(blockIdx.x) * (kVs / 16) * kK + tid) * 16;

    float* carry = reinterpret_cast<float*>(ADJOINT ? p.scratch + p.lay.carry_b : p.saved + p.lay.carry_f);
    float x[kVs];
    {
      const float* x0 = seg_first ? (ADJOINT ? p.dhT : p.h0) : carry;
#pragma unroll
      for (int j = 0; j < kVs; ++j) x[j] = x0 ? x0[(static_cast<size_t>(bh) * kK + tid) * V + v0 + j] : 0.f;
    }
    constexpr int kPieces = kVs / 8;             // 16-byte pieces of this thread's row
    uint4 rnext[kPieces];
    auto load_r = [&](int chunk) {
      // the record is cut into blocks of 16 columns: piece q lies in block q / 2 of this CTA's blocks
      const __half* r = Rg + (static_cast<size_t>(bh) * NT + chunk) * kK * V + rofs;
#pragma unroll
      for (int q = 0; q < kPieces; ++q)
        rnext[q] = *reinterpret_cast<const uint4*>(r + (q >> 1) * (kK * 16) + (q & 1) * 8);
    };
    load_r(chunk_of(0));
    float a_next = ADg[(static_cast<size_t>(bh) * NT + chunk_of(0)) * kK + tid];

    for (int it = 0; it < n; ++it) {
      const size_t z = static_cast<size_t>(bh) * NT + chunk_of(it);
      // critical path: the state as a tensor-core operand
      {
        // 32-byte swizzle: the two pieces of rows 4-7 of an atom swap; 64-byte swizzle: piece q of row r sits
        // at q ^ ((r >> 1) & 3)
        const int sw = kVs == 16 ? (tid >> 2) & 1 : (tid >> 1) & 3;
#pragma unroll
        for (int q = 0; q < kPieces; ++q)
          *reinterpret_cast<uint4*>(XB + tid * (2 * kVs) + ((q ^ sw) << 4)) = pack8_f16(x + 8 * q);
      }
      fence_proxy_async();
      tc_fence_before();
      step_arrive();
      // in the shadow of the product: this chunk's input and decay, the next chunk's loads, the record
      const float a = a_next;
      float rr[kVs];
#pragma unroll
      for (int q = 0; q < kPieces; ++q) unpack8_f16(rnext[q], rr + 8 * q);
#pragma unroll
      for (int j = 0; j < kVs; ++j) rr[j] = fmaf(a, x[j], rr[j]);
      if (it + 1 < n) {
        const int cn = chunk_of(it + 1);
        load_r(cn);
        a_next = ADg[(static_cast<size_t>(bh) * NT + cn) * kK + tid];
      }
      {
        unsigned char* rec = Xg + (ADJOINT ? z : z + bh) * szx;
#pragma unroll
        for (int q = 0; q < kPieces; ++q)
          *reinterpret_cast<uint4*>(rec + sw128_chunk(tid, v0 / 8 + q, 128)) = pack8_f16(x + 8 * q);
      }
      mbar_wait_warp(bar_mma, static_cast<uint32_t>(it & 1), ctl, 302);
      tc_fence_after();
      static_assert(kMmaWarps == 2, "two accumulators of kVs columns, one per half of the contraction");
      if (kVs == 16) {
        float acc[32];
        tmem_ld32(tmem + lane_base, acc);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) x[j] = rr[j] - (acc[j] + acc[16 + j]);
      } else {
        float a0[32], a1[32];
        tmem_ld32(tmem + lane_base, a0);
        tmem_ld32(tmem + lane_base + 32, a1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = rr[j] - (a0[j] + a1[j]);
      }
    }
    if (!ADJOINT && seg_last) {   // the final state as one more record
      unsigned char* rec = Xg + (static_cast<size_t>(bh) * (NT + 1) + NT) * szx;
#pragma unroll
      for (int q = 0; q < kPieces; ++q)
        *reinterpret_cast<uint4*>(rec + sw128_chunk(tid, v0 / 8 + q, 128)) = pack8_f16(x + 8 * q);
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

template <int kVs>
static int launch_scan_t(const Problem& p, bool adjoint, cudaStream_t st) {
  const int smem = kStages * 32768 + 128 * kVs * 2 + static_cast<int>(sizeof(CtaShared)) + 1024;
  dim3 grid(p.V / kVs, p.nbh);
  if (adjoint) {
    static SmemAttr attr;
    if (attr.set(scan_kernel<true, kVs>, smem)) return kErrLaunch;
    if (launch_dependent(scan_kernel<true, kVs>, grid, dim3(kScanThreads), smem, st, p) != cudaSuccess) return kErrLaunch;
  } else {
    static SmemAttr attr;
    if (attr.set(scan_kernel<false, kVs>, smem)) return kErrLaunch;
    if (launch_dependent(scan_kernel<false, kVs>, grid, dim3(kScanThreads), smem, st, p) != cudaSuccess) return kErrLaunch;
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

int launch_scan(const Problem& p, bool adjoint, cudaStream_t st) {
  if (!p.delta) {
    const dim3 g((p.V / 64) * 4, p.nbh);
    const cudaError_t e = adjoint ? launch_dependent(scan_nodelta_kernel<true>, g, dim3(256), 0, st, p)
                                  : launch_dependent(scan_nodelta_kernel<false>, g, dim3(256), 0, st, p);
    return e == cudaSuccess ? kOk : kErrLaunch;
  }
  // 32 columns per CTA when the CTAs of the 16-column form could not all be resident at once (two per SM):
  // the recurrence is serial, so a second wave of CTAs doubles the time of the scan
  const int sms = sm_count();
  if (sms <= 0) return kErrDevice;
  const bool wide = (p.V / 16) * p.nbh > 2 * sms;
  return wide ? launch_scan_t<32>(p, adjoint, st) : launch_scan_t<16>(p, adjoint, st);
}

}  // namespace lg
