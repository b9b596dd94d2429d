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
// Round to the 16-bit type and widen back.  The scalar conversion instructions issue on the quarter-rate conversion
// pipe, which was what bounded the 16-bit fake-quant kernels (88 % busy in the PACT+ forward); the packed forms (two
// floats -> one register) and the widening by a shift / a packed add issue on the full-rate pipes and round identically
// for every input, NaN and infinities included.
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float rnd(float v) { return __half22float2(__floats2half2_rn(v, 0.0f)).x; }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float rnd(float v) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v, 0.0f);
    return __uint_as_float(*reinterpret_cast<const uint32_t*>(&h) << 16);
  }
};

// Rounds to T when `native` is set: the value a torch op on a T tensor would have produced.
template <typename T>
__device__ __forceinline__ float rnd_if(float v, bool native) {
  return native ? Elem<T>::rnd(v) : v;
}

// ---- rounding on the FMA / ALU pipes ---------------------------------------------------------------
// The conversion instructions (float -> bf16, rint, float -> int) issue on the quarter-rate
// conversion pipe and bound the quantise kernels.  These produce the same results with additions:
// adding and subtracting 1.5 * 2^k makes the hardware's round-to-nearest-even act at 2^(k-23).
template <typename T>
__device__ __forceinline__ float fast_rnd(float v) {
  return Elem<T>::rnd(v);
}
// bf16 keeps 8 significant bits: for |v| in [2^e, 2^(e+1)) round at 2^(e-7), i.e. k = e + 16.
// Valid for normal v up to 2^110 (callers bound their values far below that).
template <>
__device__ __forceinline__ float fast_rnd<__nv_bfloat16>(float v) {
  const float m = __uint_as_float((__float_as_uint(v) & 0x7F800000u) + 0x08400000u);
  return __fsub_rn(__fadd_rn(v, m), m);
}
// rintf for |v| < 2^22 with two additions, sign of zero kept (rintf(-0.3) is -0.0).  Inputs beyond that range give an
// unspecified finite value: for callers that clamp first or discard such lanes.
__device__ __forceinline__ float rint_small(float v) {
  return copysignf(__fsub_rn(__fadd_rn(v, 12582912.0f), 12582912.0f), v);
}
// rint for |v| < 2^22, and the integer itself from the low bits of the biased sum.
__device__ __forceinline__ float fast_rint(float v, int& as_int) {
  const float t = __fadd_rn(v, 12582912.0f);
  as_int = __float_as_int(t) - 0x4B400000;
  return __fsub_rn(t, 12582912.0f);
}

// ---- exact division through a precomputed reciprocal ---------------------------------------------
// RN(x / s) from r = RN(1 / s) with three fused operations (Markstein): q = RN(x r), the exact
// remainder rem = x - s q (one FMA), q' = RN(q + rem r).  q' is the correctly rounded quotient when
// r is the correctly rounded reciprocal and s's significand is not all ones; callers pass r = NaN
// for such s.  Results outside a comfortable normal range (where the remainder could be subnormal),
// NaN and infinities take the ordinary IEEE division.
__device__ __forceinline__ float div_exact(float x, float s, float r) {
  const float q = __fmul_rn(x, r);
  const float rem = __fmaf_rn(-s, q, x);
  const float q2 = __fmaf_rn(rem, r, q);
  if (x == 0.0f && r == r) return q;  // keeps the sign of a zero quotient (r is NaN where the caller asked for the IEEE division)
  const float a = fabsf(q2);
  if (!(a > 1e-15f && a < 1e15f)) return __fdiv_rn(x, s);
  return q2;
}
// r for div_exact: RN(1 / s), or NaN when the shortcut is not proven for this s.
__device__ __forceinline__ float rcp_for_div(float s) {
  const uint32_t bits = __float_as_uint(s);
  const float a = fabsf(s);
  if ((bits & 0x7FFFFFu) == 0x7FFFFFu || !(a > 1e-15f && a < 1e15f)) return __int_as_float(0x7fc00000);
  return __frcp_rn(s);
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
// block_reduce that also ORs a per-thread flag over the block through the same barrier.
template <typename Op>
__device__ __forceinline__ float block_reduce_flag(float v, float* slot, float identity, bool flag, bool& any_flag) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_reduce<Op>(v);
  if (lane == 0) slot[warp] = v;
  any_flag = __syncthreads_or(flag ? 1 : 0) != 0;
  float r = lane < nwarps ? slot[lane] : identity;
  return warp_reduce<Op>(r);
}

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
