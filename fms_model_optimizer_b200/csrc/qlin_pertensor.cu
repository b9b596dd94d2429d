// qlin_tensor_fq: per-tensor fake quantisers (one clip value / one scale for the whole tensor).
//
// Three launches on the caller's stream, no host round trip:
//   1. statistics  : every block reduces its grid-stride share of the tensor to (sum |x|, sum x*x,
//                    max |x|) and writes the three partials to the workspace;
//   2. finish      : one block adds the partials in index order (so the result does not depend on
//                    scheduling) and forms the clip value / scale in the tensor dtype;
//   3. apply       : elementwise quantise-dequantise with the value read from device memory.
// With QLIN_W_GIVEN only the third kernel runs.  The tensor is read twice (the second time mostly
// from L2 for weights of a few tens of MB) and written once.
//
// Arithmetic follows the reference's eager expressions operation by operation, each result rounded
// to the tensor dtype.
#include <type_traits>

#include <cuda_fp8.h>

#include "qlin_internal.h"
#include "qlin_rows.cuh"

namespace qlin {

constexpr int kPtThreads = 256;
constexpr int kPtMaxBlocks = 148 * 8;

struct PtParams {
  const void* x;
  void* out;
  float* clip_io;
  float* ws;
  int64_t numel;
  int32_t num_bits, mode, kind, align_zero, dequantize, nblocks;
  float c0, c1;
};

template <typename XT>
__global__ void __launch_bounds__(kPtThreads) pt_stats_kernel(const PtParams p) {
  __shared__ float red[3][32];
  const XT* x = reinterpret_cast<const XT*>(p.x);
  const bool vec = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  const int64_t nvec = vec ? (p.numel >> 4) : 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  float sa = 0.0f, sq = 0.0f, am = 0.0f;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float v[16];
    load16(x + i * 16, v);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float a = fabsf(v[j]);
      sa += a;
      sq += Elem<XT>::rnd(__fmul_rn(v[j], v[j]));  // x.mul(x) is rounded to the dtype before the mean
      am = fmaxf(am, a);
    }
  }
  for (int64_t i = nvec * 16 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.numel; i += stride) {
    const float v = load1(x + i), a = fabsf(v);
    sa += a;
    sq += Elem<XT>::rnd(__fmul_rn(v, v));
    am = fmaxf(am, a);
  }
  sa = block_reduce<OpSum>(sa, red[0], 0.0f);
  sq = block_reduce<OpSum>(sq, red[1], 0.0f);
  am = block_reduce<OpMax>(am, red[2], 0.0f);
  if (threadIdx.x == 0) {
    p.ws[3 * blockIdx.x] = sa;
    p.ws[3 * blockIdx.x + 1] = sq;
    p.ws[3 * blockIdx.x + 2] = am;
  }
}

template <typename XT>
__global__ void __launch_bounds__(kPtThreads) pt_finish_kernel(const PtParams p) {
  __shared__ float red[3][32];
  float sa = 0.0f, sq = 0.0f, am = 0.0f;
  for (int i = threadIdx.x; i < p.nblocks; i += blockDim.x) {
    sa += p.ws[3 * i];
    sq += p.ws[3 * i + 1];
    am = fmaxf(am, p.ws[3 * i + 2]);
  }
  sa = block_reduce<OpSum>(sa, red[0], 0.0f);
  sq = block_reduce<OpSum>(sq, red[1], 0.0f);
  am = block_reduce<OpMax>(am, red[2], 0.0f);
  if (threadIdx.x != 0) return;
  float clip = am;
  if (p.mode == QLIN_W_SAWB) {
    // sawb_params_code, per tensor: clip = c1 * mean|x| + c0 * sqrt(mean x^2); a non-positive
    // result falls back to max|x|.
    const float n = static_cast<float>(p.numel);
    const float mu = Elem<XT>::rnd(__fdiv_rn(sa, n));
    const float sd = Elem<XT>::rnd(__fsqrt_rn(Elem<XT>::rnd(__fdiv_rn(sq, n))));
    clip = Elem<XT>::rnd(__fadd_rn(Elem<XT>::rnd(__fmul_rn(p.c1, mu)), Elem<XT>::rnd(__fmul_rn(p.c0, sd))));
    if (clip <= 0.0f) clip = am;
  }
  p.clip_io[0] = clip;
}

__device__ __forceinline__ uint8_t pt_to_e4m3(float v) {  // torch's cast: NaN above 464
  if (!(fabsf(v) <= 464.0f)) return static_cast<uint8_t>(0x7F | (signbit(v) ? 0x80 : 0));
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float pt_from_e4m3(uint8_t c) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(c), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

struct PtScalars {
  float cv, inv_cv, levels, half_levels, f8_scale;
  float rlevels, rf8_scale;  // reciprocals for div_exact (NaN: take the IEEE division)
};

template <typename XT>
__device__ __forceinline__ PtScalars pt_scalars(const PtParams& p) {
  PtScalars s;
  s.cv = Elem<XT>::rnd(p.clip_io[0]);
  s.inv_cv = Elem<XT>::rnd(__fdiv_rn(1.0f, s.cv));
  s.levels = static_cast<float>((1 << p.num_bits) - (p.align_zero ? 2 : 1));
  s.half_levels = Elem<XT>::rnd(s.levels * 0.5f);
  // max_to_scale: 448 / clamp(max, 1e-12) evaluated as reciprocal * 448; capped at the fp16 maximum
  const float eps = Elem<XT>::rnd(1e-12f);
  float sc = Elem<XT>::rnd(__fmul_rn(Elem<XT>::rnd(__fdiv_rn(1.0f, fmaxf(s.cv, eps))), 448.0f));
  if (std::is_same<XT, __half>::value) sc = fminf(sc, 65504.0f);
  s.f8_scale = sc;
  s.rlevels = rcp_for_div(s.levels);
  s.rf8_scale = rcp_for_div(sc);
  return s;
}

template <typename XT>
__device__ __forceinline__ float pt_one(const PtParams& p, const PtScalars& s, float x) {
  if (p.kind == QLIN_PT_INT_SYM) {
    // SAWBPlusZeroSTE / QmaxSTE: x.mul(1/cv).clamp(-1,1).mul(0.5).add(0.5) -> round(levels * t)
    //   -> / levels -> (2 t - 1) * cv    (or round(...) - levels/2 without dequantisation)
    float t = Elem<XT>::rnd(__fmul_rn(x, s.inv_cv));
    t = fminf(fmaxf(t, -1.0f), 1.0f);
    t = Elem<XT>::rnd(__fmul_rn(t, 0.5f));
    t = Elem<XT>::rnd(__fadd_rn(t, 0.5f));
    const float q = rint_small(Elem<XT>::rnd(__fmul_rn(s.levels, t)));  // 0 <= levels * t <= 65535
    if (!p.dequantize) return Elem<XT>::rnd(__fsub_rn(q, s.half_levels));
    float d = Elem<XT>::rnd(div_exact(q, s.levels, s.rlevels));
    d = Elem<XT>::rnd(__fmul_rn(2.0f, d));
    d = Elem<XT>::rnd(__fsub_rn(d, 1.0f));
    return Elem<XT>::rnd(__fmul_rn(d, s.cv));
  }
  // to_fp8_scaled (QLIN_PT_F8_SCALED) / to_fp8_saturated (QLIN_PT_F8_SAT), e4m3, emulation
  float t = x;
  if (p.kind == QLIN_PT_F8_SCALED) t = Elem<XT>::rnd(__fmul_rn(x, s.f8_scale));
  const bool is_nan = t != t;  // torch.clamp keeps NaN, fminf / fmaxf would drop it
  t = fminf(fmaxf(t, -448.0f), 448.0f);
  if (is_nan) t = __int_as_float(0x7FC00000);
  float f = pt_from_e4m3(pt_to_e4m3(t));
  if (p.kind == QLIN_PT_F8_SCALED) f = Elem<XT>::rnd(div_exact(f, s.f8_scale, s.rf8_scale));
  return f;
}

template <typename XT>
__global__ void __launch_bounds__(kPtThreads) pt_apply_kernel(const PtParams p) {
  const PtScalars s = pt_scalars<XT>(p);
  const XT* x = reinterpret_cast<const XT*>(p.x);
  XT* out = reinterpret_cast<XT*>(p.out);
  const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  const int64_t nvec = vec ? (p.numel >> 4) : 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float v[16];
    load16(x + i * 16, v);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = pt_one<XT>(p, s, v[j]);
    store16(out + i * 16, v);
  }
  for (int64_t i = nvec * 16 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.numel; i += stride)
    store1(out + i, pt_one<XT>(p, s, load1(x + i)));
}

static int pt_grid(int64_t numel) {
  const int64_t per_block = static_cast<int64_t>(kPtThreads) * 16;
  int64_t blocks = (numel + per_block - 1) / per_block;
  if (blocks > kPtMaxBlocks) blocks = kPtMaxBlocks;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

template <typename XT>
static int launch_pt(PtParams p, cudaStream_t stream) {
  const int grid = pt_grid(p.numel);
  p.nblocks = grid;
  if (p.mode != QLIN_W_GIVEN) {
    pt_stats_kernel<XT><<<grid, kPtThreads, 0, stream>>>(p);
    pt_finish_kernel<XT><<<1, kPtThreads, 0, stream>>>(p);
  }
  if (p.out != nullptr) pt_apply_kernel<XT><<<grid, kPtThreads, 0, stream>>>(p);
  QLIN_CHECK_LAUNCH("qlin_tensor_fq");
  return QLIN_OK;
}

}  // namespace qlin

using namespace qlin;

extern "C" int64_t qlin_tensor_fq_workspace_bytes(int64_t numel) {
  (void)numel;
  return static_cast<int64_t>(kPtMaxBlocks) * 3 * sizeof(float);
}

extern "C" int qlin_tensor_fq(const qlin_tensor_fq_args* a, void* stream) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_tensor_fq: args is NULL");
  if (a->x == nullptr || a->clip_io == nullptr) return fail(QLIN_ERR_NULL, "qlin_tensor_fq: x or clip_io is NULL");
  if (a->numel < 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_tensor_fq: negative numel");
  if (a->mode < QLIN_W_SAWB || a->mode > QLIN_W_GIVEN) return fail(QLIN_ERR_UNSUPPORTED, "qlin_tensor_fq: unknown mode");
  if (a->kind < QLIN_PT_INT_SYM || a->kind > QLIN_PT_F8_SAT) return fail(QLIN_ERR_UNSUPPORTED, "qlin_tensor_fq: unknown kind");
  if (a->mode != QLIN_W_GIVEN && a->workspace == nullptr) return fail(QLIN_ERR_NULL, "qlin_tensor_fq: workspace is NULL");
  if (a->mode == QLIN_W_GIVEN && a->out == nullptr) return fail(QLIN_ERR_NULL, "qlin_tensor_fq: no output requested");
  if (a->kind == QLIN_PT_INT_SYM && (a->num_bits < 2 || a->num_bits > 16))
    return fail(QLIN_ERR_UNSUPPORTED, "qlin_tensor_fq: num_bits must be in [2, 16]");
  if (a->numel == 0) return QLIN_OK;
  PtParams p;
  p.x = a->x;
  p.out = a->out;
  p.clip_io = a->clip_io;
  p.ws = a->workspace;
  p.numel = a->numel;
  p.num_bits = a->num_bits;
  p.mode = a->mode;
  p.kind = a->kind;
  p.align_zero = a->align_zero != 0;
  p.dequantize = a->dequantize != 0;
  p.nblocks = 0;
  p.c0 = a->c0;
  p.c1 = a->c1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (a->dtype) {
    case QLIN_DT_F32:
      return launch_pt<float>(p, s);
    case QLIN_DT_F16:
      return launch_pt<__half>(p, s);
    case QLIN_DT_BF16:
      return launch_pt<__nv_bfloat16>(p, s);
    default:
      return fail(QLIN_ERR_BAD_DTYPE, "qlin_tensor_fq: dtype must be F32, F16 or BF16");
  }
}
