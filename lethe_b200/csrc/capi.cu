// C-ABI entry points: argument checks, tensor maps, kernel sequence.  See include/lethe_gdn.h.
#include <string.h>

#include <mutex>

#include "gdn_common.cuh"
#include "host_util.h"

namespace lg {
int launch_prepare(const Problem&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);
int launch_prepare_cw(const Problem&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);
int launch_output(const Problem&, const CUtensorMap&, cudaStream_t);
int launch_scan(const Problem&, bool adjoint, cudaStream_t);
int launch_bwd_pre(const Problem&, const CUtensorMap& mq, const CUtensorMap& mdo, cudaStream_t);
int launch_bwd_main(const Problem&, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                    const CUtensorMap& mdo, const OutMaps& mo, cudaStream_t, uint32_t mask);
int launch_bwd_main_cw(const Problem&, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                       const CUtensorMap& mdo, cudaStream_t, uint32_t mask);

static bool dims_ok(const LetheGdnDims& d) {
  if (d.B <= 0 || d.H <= 0 || d.L <= 0) return false;
  if (d.K != kK || (d.V != 64 && d.V != 128)) return false;
  if (d.L % kC) return false;
  if (d.gate < LETHE_GATE_NONE || d.gate > LETHE_GATE_CHANNEL) return false;
  if (d.delta < 0 || d.delta > 2) return false;
  if (d.delta == 2 && d.gate != LETHE_GATE_CHANNEL) return false;
  return true;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Tensor map of a token-major [B, L, H, D] 16-bit tensor; one box = 64 tokens x 64 channels of one head.
static int token_map(CUtensorMap* m, const void* ptr, const LetheGdnDims& d, int D) {
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(d.H), static_cast<uint64_t>(d.L),
                      static_cast<uint64_t>(d.B)};
  uint64_t str[3] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(d.H) * D * 2,
                     static_cast<uint64_t>(d.L) * d.H * D * 2};
  uint32_t box[4] = {64, 1, 64, 1};
  return make_tmap_16bit(m, ptr, 4, dims, str, box);
}

static int fill_problem(const LetheGdnArgs* a, Problem* p, bool backward) {
  if (!a) return kErrNull;
  const LetheGdnDims& d = a->dims;
  if (!dims_ok(d)) return kErrDims;
  if (!a->q || !a->k || !a->v || !a->saved || !a->status) return kErrNull;
  if (d.gate != LETHE_GATE_NONE && !a->g) return kErrNull;
  if (d.delta == 1 && !a->beta) return kErrNull;
  if (d.delta == 2 && (!a->b_gate || !a->w_gate)) return kErrNull;
  if (!backward && !a->o) return kErrNull;
  if (backward) {
    if (!a->d_o || !a->dq || !a->dk || !a->dv || !a->scratch) return kErrNull;
    if (d.gate != LETHE_GATE_NONE && !a->dg) return kErrNull;
    if (d.delta == 1 && !a->dbeta) return kErrNull;
    if (d.delta == 2 && (!a->db_gate || !a->dw_gate)) return kErrNull;
  }
  const void* ptrs[] = {a->q, a->k, a->v, a->o, a->d_o, a->dq, a->dk, a->dv, a->h0, a->hT, a->dhT, a->dh0,
                        a->saved, a->scratch, a->b_gate, a->w_gate, a->db_gate, a->dw_gate};
  for (const void* x : ptrs)
    if (x && !aligned16(x)) return kErrAlign;
  Layout lay = make_layout(d);
  if (a->saved_bytes < lay.saved_total) return kErrWorkspace;
  if (backward && a->scratch_bytes < lay.scratch_total) return kErrWorkspace;
  if (!aligned16(a->saved) || (reinterpret_cast<uintptr_t>(a->saved) & 1023u)) return kErrAlign;
  if (backward && (reinterpret_cast<uintptr_t>(a->scratch) & 1023u)) return kErrAlign;
  p->B = d.B; p->H = d.H; p->L = d.L; p->NT = d.L / kC; p->V = d.V; p->gate = d.gate; p->delta = d.delta ? 1 : 0;
  if (a->bh_count == 0) {
    if (a->bh_begin != 0) return kErrDims;
    p->bh0 = 0;
    p->nbh = d.B * d.H;
  } else {
    if (static_cast<uint64_t>(a->bh_begin) + a->bh_count > static_cast<uint64_t>(d.B) * d.H) return kErrDims;
    p->bh0 = static_cast<int>(a->bh_begin);
    p->nbh = static_cast<int>(a->bh_count);
  }
  if (a->c_count == 0) {
    if (a->c_begin != 0) return kErrDims;
    p->c0 = 0;
    p->cn = p->NT;
  } else {
    if (static_cast<uint64_t>(a->c_begin) + a->c_count > static_cast<uint64_t>(p->NT)) return kErrDims;
    p->c0 = static_cast<int>(a->c_begin);
    p->cn = static_cast<int>(a->c_count);
  }
  p->scale = a->scale;
  p->qk16 = a->qk_f16 ? 1 : 0;
  p->q = static_cast<const __nv_bfloat16*>(a->q);
  p->k = static_cast<const __nv_bfloat16*>(a->k);
  p->v = static_cast<const __nv_bfloat16*>(a->v);
  p->d_o = static_cast<const __nv_bfloat16*>(a->d_o);
  p->g = a->g; p->beta = a->beta; p->h0 = a->h0; p->dhT = a->dhT;
  p->o = static_cast<__nv_bfloat16*>(a->o);
  p->dq = static_cast<__nv_bfloat16*>(a->dq);
  p->dk = static_cast<__nv_bfloat16*>(a->dk);
  p->dv = static_cast<__nv_bfloat16*>(a->dv);
  p->hT = a->hT; p->dg = a->dg; p->dbeta = a->dbeta; p->dh0 = a->dh0; p->dbeta_w = a->dbeta_write;
  if (d.delta == 2) {
    p->bch = a->b_gate; p->wch = a->w_gate; p->dbch = a->db_gate; p->dwch = a->dw_gate;
    p->beta = nullptr; p->dbeta = nullptr; p->dbeta_w = nullptr;
  }
  p->saved = static_cast<unsigned char*>(a->saved);
  p->scratch = static_cast<unsigned char*>(a->scratch);
  p->lay = lay;
  p->status = a->status;
  return kOk;
}

}  // namespace lg

using namespace lg;

extern "C" size_t lethe_gdn_saved_bytes(const LetheGdnDims* d) {
  if (!d || !dims_ok(*d)) return 0;
  return make_layout(*d).saved_total;
}
extern "C" size_t lethe_gdn_scratch_bytes(const LetheGdnDims* d) {
  if (!d || !dims_ok(*d)) return 0;
  return make_layout(*d).scratch_total;
}

extern "C" int lethe_gdn_forward(const LetheGdnArgs* a, void* stream) {
  Problem p;
  memset(&p, 0, sizeof(p));
  int e = fill_problem(a, &p, false);
  if (e) return e;
  DeviceGuard guard(a->q);
  if (!guard.ok) return kErrDevice;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap mq, mk, mv;
  if ((e = token_map(&mq, a->q, a->dims, kK))) return e;
  if ((e = token_map(&mk, a->k, a->dims, kK))) return e;
  if ((e = token_map(&mv, a->v, a->dims, a->dims.V))) return e;
  const uint32_t m = a->kernel_mask ? a->kernel_mask : 7u;
  if ((m & 1u) && (e = (p.gate == LETHE_GATE_CHANNEL ? launch_prepare_cw(p, mq, mk, mv, st)
                                                     : launch_prepare(p, mq, mk, mv, st)))) return e;
  if ((m & 2u) && (e = launch_scan(p, false, st))) return e;
  if ((m & 4u) && (e = launch_output(p, mq, st))) return e;
  return kOk;
}

extern "C" int lethe_gdn_backward(const LetheGdnArgs* a, void* stream) {
  Problem p;
  memset(&p, 0, sizeof(p));
  int e = fill_problem(a, &p, true);
  if (e) return e;
  DeviceGuard guard(a->q);
  if (!guard.ok) return kErrDevice;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap mq, mk, mv, mdo;
  if ((e = token_map(&mq, a->q, a->dims, kK))) return e;
  if ((e = token_map(&mk, a->k, a->dims, kK))) return e;
  if ((e = token_map(&mv, a->v, a->dims, a->dims.V))) return e;
  if ((e = token_map(&mdo, a->d_o, a->dims, a->dims.V))) return e;
  const uint32_t m = a->kernel_mask ? a->kernel_mask : 15u;
  if ((m & 1u) && (e = launch_bwd_pre(p, mq, mdo, st))) return e;
  if ((m & 2u) && (e = launch_scan(p, true, st))) return e;
  if (m & 12u) {
    if (p.gate == LETHE_GATE_CHANNEL) {
      if ((e = launch_bwd_main_cw(p, mq, mk, mv, mdo, st, m))) return e;
    } else {
      OutMaps mo;
      if ((e = token_map(&mo.dq, a->dq, a->dims, kK))) return e;
      if ((e = token_map(&mo.dk, a->dk, a->dims, kK))) return e;
      if ((e = token_map(&mo.dv, a->dv, a->dims, a->dims.V))) return e;
      if ((e = launch_bwd_main(p, mq, mk, mv, mdo, mo, st, m))) return e;
    }
  }
  return kOk;
}

// ---------------------------------------------------------------------------------------------
// Forward for callers that cannot allocate device memory.
//
// Some hosts of this library have no allocator to offer: a plug-in that is handed tensors by a
// runtime whose memory pool it may not touch, an inference server that has pinned its whole memory
// budget at start-up, a caller inside a region where cudaMalloc is forbidden.  They cannot supply
// the `saved` workspace the forward kernels pass their per-chunk records through.  For them the
// workspace lives in the array below, which is part of the library image: every GPU that loads the
// library holds these 16 MiB (+1 KiB for alignment) until the process exits.
//
// The array is shared by every call on a device and keeps whatever the last call wrote.  Nothing
// in it has to start at zero: each forward kernel writes every record of a chunk before a later
// kernel of the same call reads it, and no record of an earlier call is read.  Two calls whose
// kernels overlap on the GPU (different streams, or different threads on different streams) would
// race on it; callers serialise them on one stream.
//
// In host code the array's name is only a handle; the device address comes from
// cudaGetSymbolAddress.  Every GPU has its own copy of the array, so the address is looked up per
// device, by the first call whose tensors live on that device, with that device made current for
// the lookup: the device is the one that owns `q`, not whatever device the calling thread happens
// to have selected (a worker thread of a multi-GPU process usually has device 0 selected).  That
// first call may also make the driver load the library's code onto the GPU, which is the moment
// the 16 MiB are reserved there; it should therefore happen before any stream capture begins.
// ---------------------------------------------------------------------------------------------
constexpr size_t kStaticSavedBytes = size_t(16) << 20;
constexpr int kMaxDevices = 64;
static __device__ __align__(256) unsigned char g_static_saved[kStaticSavedBytes + 1024];
static unsigned char* g_static_saved_ptr[kMaxDevices] = {};
static std::mutex g_static_saved_mu;

// Device that owns a device pointer, or -1.
static int device_of(const void* ptr) {
  cudaPointerAttributes at;
  if (!ptr || cudaPointerGetAttributes(&at, ptr) != cudaSuccess || at.type != cudaMemoryTypeDevice) {
    cudaGetLastError();      // a host pointer leaves a sticky-looking error behind on some drivers
    return -1;
  }
  return at.device;
}

// Address of the built-in workspace on device `dev`, which must be the calling thread's current device.
static int static_saved_address(int dev, unsigned char** out) {
  if (dev < 0 || dev >= kMaxDevices) return kErrDevice;
  std::lock_guard<std::mutex> lock(g_static_saved_mu);
  if (!g_static_saved_ptr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_saved) != cudaSuccess || !ptr) return kErrSymbol;
    const int owner = device_of(ptr);
    if (owner >= 0 && owner != dev) return kErrSymbol;     // never hand a kernel another GPU's copy
    const uintptr_t a = (reinterpret_cast<uintptr_t>(ptr) + 1023) & ~static_cast<uintptr_t>(1023);
    g_static_saved_ptr[dev] = reinterpret_cast<unsigned char*>(a);   // the records want 1 KiB alignment
  }
  *out = g_static_saved_ptr[dev];
  return kOk;
}

extern "C" size_t lethe_gdn_forward_static_capacity(void) { return kStaticSavedBytes; }

extern "C" int lethe_gdn_forward_static(const LetheGdnArgs* a, void* stream) {
  if (!a) return kErrNull;
  if (!dims_ok(a->dims)) return kErrDims;
  if (!a->q) return kErrNull;
  if (make_layout(a->dims).saved_total > kStaticSavedBytes) return kErrTooLarge;
  const int dev = device_of(a->q);
  if (dev < 0) return kErrDevice;
  DeviceGuard guard(a->q);            // the lookup below and the launches run with q's device current
  if (!guard.ok || guard.dev != dev) return kErrDevice;
  unsigned char* ws = nullptr;
  const int e = static_saved_address(dev, &ws);
  if (e) return e;
  LetheGdnArgs b = *a;
  b.saved = ws;
  b.saved_bytes = kStaticSavedBytes;
  b.kernel_mask = 0;
  return lethe_gdn_forward(&b, stream);
}

extern "C" const char* lethe_gdn_strerror(int code) {
  switch (code) {
    case kOk: return "ok";
    case kErrNull: return "a required pointer is null";
    case kErrDims: return "unsupported sizes (need K = 128, V in {64, 128}, L a multiple of 64)";
    case kErrAlign: return "a pointer is not aligned (16 bytes for tensors, 1024 for workspaces)";
    case kErrWorkspace: return "workspace too small";
    case kErrDriver: return "tensor-map encoding failed (driver entry point missing or bad tensor geometry)";
    case kErrLaunch: return "kernel launch failed";
    case kErrFlags: return "unsupported gate / delta combination";
    case kErrDevice: return "the device that owns q could not be made current, or a buffer is not device memory of that GPU";
    case kErrSymbol: return "the address of the library's built-in workspace could not be looked up on this GPU";
    case kErrTooLarge: return "problem needs more workspace than the library's built-in 16 MiB (use lethe_gdn_forward)";
    default: break;
  }
  if (code >= 100) return "device-side wait timed out (status word holds the wait site)";
  return "unknown error";
}
