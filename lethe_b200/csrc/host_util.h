// Host-side helpers shared by the C-ABI entry points: error codes and TMA tensor-map encoding.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

namespace lg {

enum : int {
  kOk = 0,
  kErrNull = 1,        // a required pointer is null
  kErrDims = 2,        // unsupported sizes
  kErrAlign = 3,       // pointer or stride not 16-byte aligned
  kErrWorkspace = 4,   // workspace too small
  kErrDriver = 5,      // tensor-map encoding or driver entry point failed
  kErrLaunch = 6,      // kernel launch failed
  kErrFlags = 7,       // unsupported flag combination
  kErrTooLarge = 8,    // problem larger than a fixed-capacity entry point accepts
  kErrDevice = 9,      // the device that owns the tensors could not be made current, or a buffer lives elsewhere
  kErrSymbol = 10,     // the address of the library's built-in workspace could not be looked up
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// Looked up once per process; safe to call from several threads at once.
inline EncodeTiledFn encode_tiled_fn() {
  static std::once_flag once;
  static EncodeTiledFn fn = nullptr;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

// Tensor map over 16-bit elements with the 128-byte swizzle.  dims / box are innermost first,
// strides (bytes) belong to dims 1..rank-1.  Out-of-range elements read as zero.
inline int make_tmap_16bit(CUtensorMap* map, const void* ptr, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return kErrDriver;
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, static_cast<cuuint32_t>(rank),
                  const_cast<void*>(ptr), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kErrDriver;
}

// Tensor maps of the token-major gradient outputs that leave by tensor-map stores.
struct OutMaps {
  CUtensorMap dq, dk, dv;
};

// Makes the device that owns `ptr` current on the calling thread for the duration of a call and
// binds its primary context.  A host framework may call from a worker thread that has never touched
// CUDA (PyTorch's autograd thread when nothing else ran on it yet): without this the driver-level
// tensor-map encoding fails with "invalid context".
struct DeviceGuard {
  int prev = -1, dev = -1;
  bool ok = false;
  explicit DeviceGuard(const void* ptr) {
    cudaPointerAttributes at;
    if (cudaGetDevice(&prev) != cudaSuccess) return;
    dev = prev;
    if (ptr && cudaPointerGetAttributes(&at, ptr) == cudaSuccess && at.type == cudaMemoryTypeDevice) dev = at.device;
    ok = cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceGuard() {
    if (ok && prev >= 0 && prev != dev) cudaSetDevice(prev);
  }
};

// Number of SMs of the current device (looked up once per device ordinal).
inline int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return 0;
  if (dev < 64) {
    const int c = cached[dev].load(std::memory_order_acquire);
    if (c > 0) return c;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 0;
  if (dev < 64) cached[dev].store(n, std::memory_order_release);
  return n;
}

// Opt-in to more than 48 KB of dynamic shared memory, done once per kernel and device instead of on
// every launch.  One object per kernel instantiation (a function-local static of its launcher).
struct SmemAttr {
  std::atomic<uint64_t> done{0};     // bit d: the attribute is set on device ordinal d
  template <typename Kern>
  int set(Kern kern, int smem) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return kErrLaunch;
    if (dev < 64 && (done.load(std::memory_order_acquire) >> dev) & 1u) return kOk;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kErrLaunch;
    if (dev < 64) done.fetch_or(uint64_t(1) << dev, std::memory_order_release);
    return kOk;
  }
};

// Launch with the programmatic-dependent-launch attribute: the kernel may begin (prologue, loads of data
// older than its predecessor's) before the previous kernel of the stream has finished; it must call
// griddep_wait() before touching what that kernel writes.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace lg
