// Thin PTX wrappers for the Blackwell (sm_100a) asynchronous units used by the GDN kernels:
// mbarriers, bulk / tensor copies (TMA), tensor memory (TMEM) and tcgen05 matrix products.
//
// Conventions
//  * Every wait is bounded.  A wait that runs out records a code in the kernel's status word in
//    global memory, raises a CTA-wide abort flag in shared memory and returns; every later wait of
//    the CTA returns at once, so the kernel always runs to its end, frees its TMEM and exits.  The
//    host reads the status word after the stream has been synchronised.
//  * All products use cta_group::1 with M = 128: accumulator row r lives in TMEM lane r and
//    accumulator column n in TMEM column n (32-bit), so thread t of a 128-thread group owns row t.
//  * Operand tiles in shared memory use the 128-byte swizzle ("SW128"): a tile is a sequence of
//    atoms of 64 sixteen-bit elements (128 B) per row; inside an atom row r lives at r*128 B and its
//    16-byte chunk c is stored at chunk (c ^ (r & 7)).  Tiles are 1024-byte aligned.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace lg {

// ---------------------------------------------------------------------------------------------
// status / abort
// ---------------------------------------------------------------------------------------------
constexpr long long kWaitLimitCycles = 2000000000LL;  // about one second at 1.9 GHz

struct CtaCtl {
  int* status;              // global status word (0 = ok)
  volatile int* abort_flag; // shared-memory flag, set when any wait of this CTA gave up
  long long limit = kWaitLimitCycles;   // cycles a wait may spin before it gives up
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait on phase `parity`.  `code` identifies the wait site in the status word.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, const CtaCtl& ctl, int code) {
  if (*ctl.abort_flag) return;
  if (mbar_try(bar, parity)) return;
  const long long t0 = clock64();
  while (!mbar_try(bar, parity)) {
    if (*ctl.abort_flag) return;
    if (clock64() - t0 > ctl.limit) {
      atomicCAS(ctl.status, 0, code);
      *ctl.abort_flag = 1;
      return;
    }
  }
}

// Same, for a wait that every lane of the calling warp executes: the warp leaves it converged, which
// the .sync.aligned tcgen05 instructions that usually follow require.
__device__ __forceinline__ void mbar_wait_warp(uint64_t* bar, uint32_t parity, const CtaCtl& ctl, int code) {
  mbar_wait(bar, parity, ctl, code);
  __syncwarp();
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with the attribute may start while the kernel
// before it in the stream is still running; `griddep_wait` blocks until that kernel has completed and
// its writes are visible (a no-op for a plain launch), `griddep_launch` lets the next kernel of the
// stream start its own prologue.  Every kernel here triggers only after its own wait, so when a
// kernel starts, everything older than its immediate predecessor is complete: before the wait it
// may read anything except what the immediate predecessor writes.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// proxy fences
// ---------------------------------------------------------------------------------------------
// Make this thread's earlier shared-memory writes visible to the asynchronous proxy (TMA, tcgen05).
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA: tensor-map tiled loads, and plain bulk copies of contiguous bytes
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5, %6}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// Contiguous global -> shared copy (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// Contiguous shared -> global copy.
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(smem_u32(src)), "r"(bytes)
               : "memory");
}
// Tensor-map tiled store of one box from shared memory (joins this thread's bulk group).
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* src, int c0, int c1, int c2,
                                             int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// All of this thread's bulk stores have finished reading shared memory and writing global memory.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// ... have finished reading shared memory: the source may be overwritten, or the CTA may exit (the
// global writes complete on their own and are visible when the kernel ends).
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// TMEM allocation (one warp, all 32 lanes, executes these)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05 ordering
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle.  Offsets in bytes.
//   contraction along the tile's columns ("K-major"): sbo = distance between 8-row groups
//     (1024 for a dense atom), lbo unused (encoded as 16 B).
//   contraction along the tile's rows ("MN-major"): lbo = distance between 64-column atoms,
//     sbo = distance between 8-row groups.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;  // descriptor version of this architecture
  d |= 2ull << 61;  // 128-byte swizzle
  return d;
}

// The same for tiles in the 32-byte swizzle (atoms of 8 rows x 32 bytes; 16-byte piece c of row r stored
// at c ^ ((r >> 2) & 1)), used for a 16-column operand that is contracted along its rows.
__device__ __forceinline__ uint64_t make_desc_sw32(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;  // descriptor version of this architecture
  d |= 6ull << 61;  // 32-byte swizzle
  return d;
}

// ... and in the 64-byte swizzle (atoms of 8 rows x 64 bytes; piece c of row r stored at c ^ ((r >> 1) & 3)),
// for a 32-column operand contracted along its rows.
__device__ __forceinline__ uint64_t make_desc_sw64(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;  // descriptor version of this architecture
  d |= 4ull << 61;  // 64-byte swizzle
  return d;
}

enum : uint32_t { kFmtF16 = 0, kFmtBF16 = 1 };

// Instruction descriptor for kind::f16, fp32 accumulate.  a_mn / b_mn: operand is contracted along
// its tile rows (MN-major) instead of its columns.  a_neg: use -A.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t M, uint32_t N, bool a_mn, bool b_mn,
                                                  bool a_neg = false, uint32_t a_fmt = kFmtF16,
                                                  uint32_t b_fmt = kFmtF16) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((a_neg ? 1u : 0u) << 13) |
         ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// One tcgen05 product D[128 x N] (+)= A * B with a 16-element contraction step.  One thread issues.
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                     uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Warp-converged forms: every lane of the warp executes the call with identical arguments and the
// lane with `leader` != 0 (from elect_leader) issues.  Keeping the whole warp on the path lets the
// descriptors live in uniform registers instead of being moved there per instruction.
__device__ __forceinline__ uint32_t elect_leader() {
  uint32_t leader;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(leader));
  return leader;
}
__device__ __forceinline__ void umma_led(uint32_t leader, uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}
__device__ __forceinline__ void umma_commit_led(uint32_t leader, uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar)),
      "r"(leader)
      : "memory");
}
// Arrive on `bar` once every product issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// TMEM -> registers.  taddr = base + (lane << 16) + column; the lane field must be the first lane
// of the calling warp's quadrant (32 * (warp & 3)).  Thread l of the warp receives lane base + l.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, "
      "[%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// SW128 tile addressing (16-bit elements)
// ---------------------------------------------------------------------------------------------
// Byte offset of element (r, c) in a tile whose atoms hold `rows` rows each.
__host__ __device__ __forceinline__ uint32_t sw128_off(int r, int c, int rows) {
  const int atom = c >> 6, cc = c & 63;
  return static_cast<uint32_t>(atom * rows * 128 + r * 128 + ((((cc >> 3) ^ (r & 7)) & 7) << 4) +
                               ((cc & 7) << 1));
}
// Byte offset of the 16-byte chunk holding columns [8*ch, 8*ch+8) of row r.
__host__ __device__ __forceinline__ uint32_t sw128_chunk(int r, int ch, int rows) {
  const int atom = ch >> 3, c8 = ch & 7;
  return static_cast<uint32_t>(atom * rows * 128 + r * 128 + (((c8 ^ (r & 7)) & 7) << 4));
}

}  // namespace lg
