// Peer-memory plumbing for the tensor-parallel path: one process drives one GPU, buffers that other
// GPUs write into are shared through CUDA IPC handles, and a small kernel is the barrier between the
// phases of a layer.
//
//   qlin_ipc_export / qlin_ipc_open / qlin_ipc_close
//       An allocation made by this process (any pointer inside a cudaMalloc block) becomes a 64-byte
//       handle plus the pointer's offset in its block; another process on the same node maps it and
//       gets an address its own kernels can store to (over NVLink when the GPUs are peers).
//   qlin_peer_copy2d
//       A (pitched) device-to-device copy queued on a stream; with a mapped peer address on one side the
//       copy engines move the bytes over NVLink while the SMs run other kernels.
//   qlin_peer_barrier
//       Every rank stores the next epoch number into its slot of every peer's flag array
//       (st.release.sys) and waits until all of its own slots show that epoch (ld.acquire.sys).
//       Plain peer stores written by earlier kernels of the stream are visible to the peers' later
//       kernels once the barrier has passed.  The wait is bounded by wall-clock time (timeout_ns of the
//       argument block, 10 s when that is 0): when a peer never arrives the kernel records
//       QLIN_ERR_TIMEOUT in `status` and returns; the context stays usable.
#include <cstring>

#include <cuda.h>

#include "qlin_internal.h"

namespace qlin {

constexpr unsigned long long kBarrierTimeoutNs = 10000000000ull;  // default, 10 s: peers may still be loading libraries on their first step

__device__ __forceinline__ unsigned long long peer_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct BarrierParams {
  uint32_t* local_flags;   // [world]: slot r is written by rank r
  uint32_t* peer_flags[8]; // the flag array of every rank (own entry = local_flags)
  uint32_t* epoch;         // local counter, one per barrier object
  int32_t* status;
  int32_t rank, world;
  unsigned long long timeout_ns;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const BarrierParams p) {
  const int lane = threadIdx.x;
  uint32_t e = 0;
  if (lane == 0) {
    e = *p.epoch + 1u;
    *p.epoch = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  if (lane < p.world) {
    uint32_t* dst = p.peer_flags[lane] + p.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(e) : "memory");
    const uint32_t* src = p.local_flags + lane;
    const unsigned long long t0 = peer_now_ns();
    bool seen = false;
    while (!seen) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
      seen = static_cast<int32_t>(v - e) >= 0;
      if (!seen && peer_now_ns() - t0 > p.timeout_ns) {
        if (p.status != nullptr) atomicExch(p.status, static_cast<int32_t>(QLIN_ERR_TIMEOUT));
        break;
      }
    }
  }
  __syncwarp();
}

}  // namespace qlin

using namespace qlin;

extern "C" int qlin_ipc_export(const void* dev_ptr, void* handle_out, int64_t* offset_out) {
  if (dev_ptr == nullptr || handle_out == nullptr || offset_out == nullptr) return fail(QLIN_ERR_NULL, "qlin_ipc_export: NULL argument");
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, dev_ptr);
  if (e != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
    cudaGetLastError();
    return fail(QLIN_ERR_DEVICE, "qlin_ipc_export: not a device pointer");
  }
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QLIN_ERR_DEVICE, "qlin_ipc_export: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  // The handle names the whole allocation; find the pointer's offset in it by mapping nothing: the
  // driver reports the base of the range the pointer lies in.
  void* base = nullptr;
  size_t size = 0;
  typedef CUresult (*GetRange)(CUdeviceptr*, size_t*, CUdeviceptr);
  static GetRange get_range = nullptr;
  if (get_range == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || fn == nullptr) {
      cudaGetLastError();
      return fail(QLIN_ERR_DEVICE, "qlin_ipc_export: cuMemGetAddressRange is not available");
    }
    get_range = reinterpret_cast<GetRange>(fn);
  }
  CUdeviceptr b = 0;
  if (get_range(&b, &size, reinterpret_cast<CUdeviceptr>(dev_ptr)) != CUDA_SUCCESS)
    return fail(QLIN_ERR_DEVICE, "qlin_ipc_export: cuMemGetAddressRange failed");
  base = reinterpret_cast<void*>(b);
  memcpy(handle_out, &h, sizeof(h));
  *offset_out = static_cast<int64_t>(reinterpret_cast<const uint8_t*>(dev_ptr) - reinterpret_cast<const uint8_t*>(base));
  return QLIN_OK;
}

extern "C" int qlin_ipc_open(const void* handle, int64_t offset, void** base_out, void** ptr_out) {
  if (handle == nullptr || base_out == nullptr || ptr_out == nullptr) return fail(QLIN_ERR_NULL, "qlin_ipc_open: NULL argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* base = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QLIN_ERR_DEVICE, "qlin_ipc_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  }
  *base_out = base;
  *ptr_out = static_cast<uint8_t*>(base) + offset;
  return QLIN_OK;
}

extern "C" int qlin_ipc_close(void* base) {
  if (base == nullptr) return QLIN_OK;
  cudaError_t e = cudaIpcCloseMemHandle(base);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QLIN_ERR_DEVICE, "qlin_ipc_close: %s", cudaGetErrorString(e));
  }
  return QLIN_OK;
}

extern "C" int qlin_peer_copy2d(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width, int64_t height,
                                void* stream) {
  if (dst == nullptr || src == nullptr) return fail(QLIN_ERR_NULL, "qlin_peer_copy2d: NULL pointer");
  if (width < 0 || height < 0 || (height > 1 && (dpitch < width || spitch < width))) return fail(QLIN_ERR_BAD_SHAPE, "qlin_peer_copy2d: bad extent or pitch");
  if (width == 0 || height == 0) return QLIN_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = height == 1 ? cudaMemcpyAsync(dst, src, static_cast<size_t>(width), cudaMemcpyDeviceToDevice, s)
                              : cudaMemcpy2DAsync(dst, static_cast<size_t>(dpitch), src, static_cast<size_t>(spitch),
                                                  static_cast<size_t>(width), static_cast<size_t>(height), cudaMemcpyDeviceToDevice, s);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QLIN_ERR_LAUNCH, "qlin_peer_copy2d: %s", cudaGetErrorString(e));
  }
  return QLIN_OK;
}

extern "C" int qlin_peer_barrier(const qlin_peer_barrier_args* a, void* stream) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_peer_barrier: args is NULL");
  if (a->world < 1 || a->world > 8 || a->rank < 0 || a->rank >= a->world) return fail(QLIN_ERR_BAD_SHAPE, "qlin_peer_barrier: bad rank / world");
  if (a->local_flags == nullptr || a->epoch == nullptr) return fail(QLIN_ERR_NULL, "qlin_peer_barrier: local_flags or epoch is NULL");
  BarrierParams p;
  p.local_flags = a->local_flags;
  p.epoch = a->epoch;
  p.status = a->status;
  p.rank = a->rank;
  p.world = a->world;
  if (a->timeout_ns < 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_peer_barrier: negative timeout_ns");
  p.timeout_ns = a->timeout_ns > 0 ? static_cast<unsigned long long>(a->timeout_ns) : kBarrierTimeoutNs;
  for (int i = 0; i < 8; ++i) {
    p.peer_flags[i] = i < a->world ? a->peer_flags[i] : nullptr;
    if (i < a->world && p.peer_flags[i] == nullptr) return fail(QLIN_ERR_NULL, "qlin_peer_barrier: peer_flags[%d] is NULL", i);
  }
  peer_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  QLIN_CHECK_LAUNCH("qlin_peer_barrier");
  return QLIN_OK;
}
