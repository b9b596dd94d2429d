// Row-oriented building blocks of the HBM-bound quantise kernels: 16-element vector loads and
// stores for fp32 / fp16 / bf16 rows, dtype rounding helpers, and a block-wide reduction that
// needs one barrier per row.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace qlin {

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float rnd(float v) { return v; }
};
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float rnd(float v) { return __half2float(__float2half_rn(v)); }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// Rounds to T when `native` is set: the value a torch op on a T tensor would have produced.
template <typename T>
__device__ __forceinline__ float rnd_if(float v, bool native) {
  return native ? Elem<T>::rnd(v) : v;
}

// ---- 16 consecutive elements <-> 16 floats --------------------------------------------------
__device__ __forceinline__ void load16(const float* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 t = reinterpret_cast<const float4*>(p)[i];
    v[4 * i] = t.x;
    v[4 * i + 1] = t.y;
    v[4 * i + 2] = t.z;
    v[4 * i + 3] = t.w;
  }
}
__device__ __forceinline__ void load16(const __half* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint4 t = reinterpret_cast<const uint4*>(p)[i];
    const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      v[8 * i + 2 * j] = f.x;
      v[8 * i + 2 * j + 1] = f.y;
    }
  }
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint4 t = reinterpret_cast<const uint4*>(p)[i];
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
      v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
  }
}
__device__ __forceinline__ void store16(float* p, const float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}
__device__ __forceinline__ void store16(__half* p, const float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 t;
    __half2* h = reinterpret_cast<__half2*>(&t);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
    reinterpret_cast<uint4*>(p)[i] = t;
  }
}
__device__ __forceinline__ void store16(__nv_bfloat16* p, const float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 t;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
    reinterpret_cast<uint4*>(p)[i] = t;
  }
}
__device__ __forceinline__ float load1(const float* p) { return *p; }
__device__ __forceinline__ float load1(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void store1(float* p, float v) { *p = v; }
__device__ __forceinline__ void store1(__half* p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// ---- block reductions -------------------------------------------------------------------------
struct OpMax {
  static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
};
struct OpSum {
  static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};

template <typename Op>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Reduces `v` over the block in a fixed order and returns the result to every thread.  `slot`
// points at 32 floats of shared memory; callers alternate between two slots from one call to the
// next so that a single __syncthreads() per call is enough.
template <typename Op>
__device__ __forceinline__ float block_reduce(float v, float* slot, float identity) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_reduce<Op>(v);
  if (lane == 0) slot[warp] = v;
  __syncthreads();
  float r = lane < nwarps ? slot[lane] : identity;
  return warp_reduce<Op>(r);
}

}  // namespace qlin
