// Self-test of the tcgen05 / TMA toolkit: one CTA computes D[128 x N] = (+/-) A * B (optionally
// twice, accumulating) with every combination of operand orientation and fill method the GDN
// kernels rely on.  The Python test compares D with a plain matrix product.
//
// A second kernel, `starved_wait_kernel`, exercises the bounded wait: it arms an mbarrier for bytes
// that nobody sends and waits on it with a short limit.  The wait has to give up, leave its site code
// in the status word, let the CTA's later waits fall through, free the tensor memory and return.
// Nothing faults and nothing hangs: the kernel ends by itself after `limit_cycles`.
#include <string.h>

#include "host_util.h"
#include "lethe_probe.h"
#include "tiles.cuh"

namespace lg {

struct ProbeParams {
  const __half* A;   // a_mn=0: [128 x kc] row-major;  a_mn=1: [kc x 128] row-major
  const __half* B;   // b_mn=0: [N x kc] row-major;    b_mn=1: [kc x N] row-major
  float* D;          // [128 x N]
  int* status;
  int a_mn, b_mn, N, kc, fill, a_neg, twice;
  // fill: 0 = threads write the swizzled tiles, 1 = TMA tensor-map loads,
  //       2 = bulk copy of tiles that the host has already swizzled (A and B point at images)
};

__global__ void __launch_bounds__(128, 1)
probe_kernel(const ProbeParams p, const __grid_constant__ CUtensorMap mapA,
             const __grid_constant__ CUtensorMap mapB) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char* tA = smem;             // up to 32 KB
  unsigned char* tB = smem + 32768;     // up to 64 KB
  __shared__ uint64_t bar_load, bar_mma;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  CtaCtl ctl{p.status, &abort_flag};

  const int a_rows = p.a_mn ? p.kc : 128;               // rows per atom of tile A
  const int a_cols = p.a_mn ? 128 : p.kc;
  const int b_rows = p.b_mn ? p.kc : p.N;
  const int b_cols = p.b_mn ? p.N : p.kc;
  const int a_atoms = (a_cols + 63) / 64, b_atoms = (b_cols + 63) / 64;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (p.fill == 0) {
    for (int i = tid; i < a_rows * a_cols; i += 128) {
      const int r = i / a_cols, c = i % a_cols;
      *reinterpret_cast<__half*>(tA + sw128_off(r, c, a_rows)) = p.A[i];
    }
    for (int i = tid; i < b_rows * b_cols; i += 128) {
      const int r = i / b_cols, c = i % b_cols;
      *reinterpret_cast<__half*>(tB + sw128_off(r, c, b_rows)) = p.B[i];
    }
    fence_proxy_async();
  } else if (tid == 0) {
    const uint32_t bytes = static_cast<uint32_t>(a_atoms * a_rows * 128 + b_atoms * b_rows * 128);
    mbar_expect_tx(&bar_load, bytes);
    if (p.fill == 1) {
      for (int a = 0; a < a_atoms; ++a) tma_load_2d(tA + a * a_rows * 128, &mapA, &bar_load, a * 64, 0);
      for (int a = 0; a < b_atoms; ++a) tma_load_2d(tB + a * b_rows * 128, &mapB, &bar_load, a * 64, 0);
    } else {
      bulk_g2s(tA, p.A, static_cast<uint32_t>(a_atoms * a_rows * 128), &bar_load);
      bulk_g2s(tB, p.B, static_cast<uint32_t>(b_atoms * b_rows * 128), &bar_load);
    }
  }
  if (p.fill != 0) mbar_wait_warp(&bar_load, 0, ctl, 101);
  __syncthreads();

  if (tid == 0) {
    tc_fence_after();
    Tile A{smem_u32(tA), static_cast<uint32_t>(a_rows), p.a_mn != 0};
    Tile B{smem_u32(tB), static_cast<uint32_t>(b_rows), p.b_mn != 0};
    issue_product(tmem, A, B, p.N, p.kc, 0u, p.a_neg != 0);
    if (p.twice) issue_product(tmem, A, B, p.N, p.kc, 1u, p.a_neg != 0);
    umma_commit(&bar_mma);
  }
  __syncwarp();
  mbar_wait_warp(&bar_mma, 0, ctl, 102);
  tc_fence_after();

  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  for (int c0 = 0; c0 < p.N; c0 += 16) {
    float v[16];
    tmem_ld16(tmem + lane_base + static_cast<uint32_t>(c0), v);
    tmem_ld_wait();
    for (int j = 0; j < 16 && c0 + j < p.N; ++j) p.D[tid * p.N + c0 + j] = v[j];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// One CTA: TMEM allocated, a barrier armed for 64 bytes that never arrive, every thread waits.
__global__ void __launch_bounds__(128, 1)
starved_wait_kernel(int* status, long long limit_cycles, int* trace) {
  __shared__ uint64_t bar_a, bar_b;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  CtaCtl ctl{status, &abort_flag, limit_cycles};
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_a, 1);
    mbar_init(&bar_b, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (tid == 0) mbar_expect_tx(&bar_a, 64u);          // armed, and no copy is ever issued
  const long long t0 = clock64();
  mbar_wait_warp(&bar_a, 0, ctl, 101);                // runs out after limit_cycles
  const long long t1 = clock64();
  mbar_wait_warp(&bar_b, 0, ctl, 102);                // must return at once: the abort flag is up
  const long long t2 = clock64();
  if (tid == 0) {
    trace[0] = abort_flag;
    trace[1] = static_cast<int>((t1 - t0) >> 10);     // kilo-cycles spent in the first wait
    trace[2] = static_cast<int>((t2 - t1) >> 10);     // ... in the second
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 64);
}

}  // namespace lg

extern "C" int lethe_probe_starved_wait(int* status, long long limit_cycles, int* trace, void* stream) {
  using namespace lg;
  if (!status || !trace) return kErrNull;
  if (limit_cycles < 1000 || limit_cycles > 200000000LL) return kErrDims;    // at most a tenth of a second
  starved_wait_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_cycles, trace);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// Test entry point; not part of the GDN interface.
extern "C" int lethe_probe_umma(const void* A, const void* B, float* D, int* status, int a_mn, int b_mn,
                                int N, int kc, int fill, int a_neg, int twice, void* stream) {
  using namespace lg;
  if (!A || !B || !D || !status) return kErrNull;
  if (N < 16 || N > 256 || (N % 16) || kc < 16 || kc > 128 || (kc % 16)) return kErrDims;
  ProbeParams p{static_cast<const __half*>(A), static_cast<const __half*>(B), D, status,
                a_mn, b_mn, N, kc, fill, a_neg, twice};
  CUtensorMap mapA, mapB;
  memset(&mapA, 0, sizeof(mapA));
  memset(&mapB, 0, sizeof(mapB));
  if (fill == 1) {
    const int a_rows = a_mn ? kc : 128, a_cols = a_mn ? 128 : kc;
    const int b_rows = b_mn ? kc : N, b_cols = b_mn ? N : kc;
    if ((a_cols % 64) || (b_cols % 64)) return kErrDims;
    uint64_t da[2] = {static_cast<uint64_t>(a_cols), static_cast<uint64_t>(a_rows)};
    uint64_t sa[1] = {static_cast<uint64_t>(a_cols) * 2};
    uint32_t ba[2] = {64, static_cast<uint32_t>(a_rows)};
    uint64_t db[2] = {static_cast<uint64_t>(b_cols), static_cast<uint64_t>(b_rows)};
    uint64_t sb[1] = {static_cast<uint64_t>(b_cols) * 2};
    uint32_t bb[2] = {64, static_cast<uint32_t>(b_rows)};
    int e = make_tmap_16bit(&mapA, A, 2, da, sa, ba);
    if (e) return e;
    e = make_tmap_16bit(&mapB, B, 2, db, sb, bb);
    if (e) return e;
  }
  const int smem = 32768 + 65536 + 1024;
  static SmemAttr attr;
  if (attr.set(probe_kernel, smem)) return kErrLaunch;
  probe_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(p, mapA, mapB);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
