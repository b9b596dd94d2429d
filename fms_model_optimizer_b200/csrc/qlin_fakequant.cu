// qlin_pact2_fwd / qlin_pact2_bwd: PACT+ two-sided fake quantisation for QAT activations.
//
// Elementwise, HBM-bound: fwd reads x and writes y (2*s bytes per element); bwd reads x and
// grad_out and writes grad_x (3*s bytes per element) and reduces the two clip-value gradients.
// The reduction is two-stage and ordered: every block writes its pair of partial sums to the
// workspace, a one-block kernel adds them in index order, so results repeat bit for bit from run
// to run.  The quantiser parameters are derived on the device from the clip values, exactly in
// the order the reference derives them, so no host synchronisation is needed.
#include "qlin_internal.h"
#include "qlin_rows.cuh"

namespace qlin {

constexpr int kFqThreads = 256;

struct PactParams {
  const void* x;
  const void* g;
  void* out;
  const float* cv;
  const float* cvn;
  float* grad_clip;
  float* ws;
  int64_t numel;
  int32_t num_bits, align_zero, variant;
};

struct PactScalars {
  float cv, cvn, step, zp, n;
  float rstep, rn;  // reciprocals for div_exact (NaN where the shortcut is not proven: those take the IEEE division)
  int variant;
};

template <typename XT>
__device__ __forceinline__ PactScalars pact_scalars(const PactParams& p) {
  PactScalars s;
  s.variant = p.variant;
  s.cv = Elem<XT>::rnd(*p.cv);
  // `n_levels / tensor` and `1.0 / scale` have a Python scalar on the left: torch evaluates them as
  // reciprocal(tensor) * scalar, each step rounded to the tensor dtype.
  if (p.variant == QLIN_PACT_TWO_SIDED) {
    s.cvn = Elem<XT>::rnd(*p.cvn);
    s.n = static_cast<float>((1 << p.num_bits) - 1);
    const float inv = Elem<XT>::rnd(__fdiv_rn(1.0f, Elem<XT>::rnd(__fsub_rn(s.cv, s.cvn))));
    const float scale = Elem<XT>::rnd(__fmul_rn(inv, s.n));
    s.step = Elem<XT>::rnd(__fdiv_rn(1.0f, scale));
    s.zp = Elem<XT>::rnd(__fmul_rn(s.cvn, scale));
    if (p.align_zero) s.zp = rintf(s.zp);
  } else if (p.variant == QLIN_PACT_ONE_SIDED) {
    s.cvn = 0.0f;
    s.zp = 0.0f;
    s.n = static_cast<float>((1 << p.num_bits) - 1);
    const float scale = Elem<XT>::rnd(__fmul_rn(Elem<XT>::rnd(__fdiv_rn(1.0f, s.cv)), s.n));
    s.step = Elem<XT>::rnd(__fdiv_rn(1.0f, scale));
  } else {  // symmetric: levels 2^b - 2 when the zero point is integral
    s.cvn = -s.cv;
    s.zp = 0.0f;
    s.n = static_cast<float>((1 << p.num_bits) - (p.align_zero ? 2 : 1));
    const float two_cv = Elem<XT>::rnd(__fmul_rn(2.0f, s.cv));
    const float scale = Elem<XT>::rnd(__fmul_rn(Elem<XT>::rnd(__fdiv_rn(1.0f, two_cv)), s.n));
    s.step = Elem<XT>::rnd(__fdiv_rn(1.0f, scale));
  }
  s.rstep = rcp_for_div(s.step);
  s.rn = rcp_for_div(s.n);
  return s;
}

template <typename XT>
__device__ __forceinline__ float pact_fwd_one(const PactScalars& s, float x) {
  if (s.variant == QLIN_PACT_TWO_SIDED) {
    float y = fminf(x, s.cv);
    y = fmaxf(y, s.cvn);
    float t = Elem<XT>::rnd(div_exact(y, s.step, s.rstep));
    t = Elem<XT>::rnd(__fsub_rn(t, s.zp));
    const float q = rint_small(t);  // |t| <= 2^16: y is clamped to the clip range
    return Elem<XT>::rnd(__fmul_rn(Elem<XT>::rnd(__fadd_rn(q, s.zp)), s.step));
  }
  if (s.variant == QLIN_PACT_ONE_SIDED) {
    // PACTplusSTE.forward: round(clamp(x, 0, cv) / step) * step
    const float y = fminf(fmaxf(x, 0.0f), s.cv);
    return Elem<XT>::rnd(__fmul_rn(rint_small(Elem<XT>::rnd(div_exact(y, s.step, s.rstep))), s.step));
  }
  // PACTplusSymSTE_rev1.forward: round((clamp(x, -cv, cv) + cv) / step) * step - cv
  float y = x > s.cv ? s.cv : x;
  y = y < -s.cv ? -s.cv : y;
  const float q = rint_small(Elem<XT>::rnd(div_exact(Elem<XT>::rnd(__fadd_rn(y, s.cv)), s.step, s.rstep)));
  return Elem<XT>::rnd(__fsub_rn(Elem<XT>::rnd(__fmul_rn(q, s.step)), s.cv));
}

template <typename XT>
__device__ __forceinline__ float pact_bwd_one(const PactScalars& s, float x, float g, float& ga, float& gan) {
  if (s.variant == QLIN_PACT_TWO_SIDED) {
    // lanes outside the clip range never use delz, so rint_small's range (|z| < 2^22) covers every lane that matters
    const float z = Elem<XT>::rnd(div_exact(Elem<XT>::rnd(__fsub_rn(x, s.cvn)), s.step, s.rstep));
    const float delz = Elem<XT>::rnd(div_exact(Elem<XT>::rnd(__fsub_rn(z, rint_small(z))), s.n, s.rn));
    const float inner = Elem<XT>::rnd(__fmul_rn(-g, delz));
    const bool hi = x >= s.cv, lo = x <= s.cvn;
    ga += hi ? g : (lo ? 0.0f : inner);
    gan += lo ? g : (hi ? 0.0f : -inner);
    return (hi || lo) ? 0.0f : g;
  }
  if (s.variant == QLIN_PACT_ONE_SIDED) {
    // PACTplusSTE.backward: z = x / step; delz = (z - round(z)) / n
    const float z = Elem<XT>::rnd(div_exact(x, s.step, s.rstep));
    const float delz = Elem<XT>::rnd(div_exact(Elem<XT>::rnd(__fsub_rn(z, rint_small(z))), s.n, s.rn));
    const float inner = Elem<XT>::rnd(__fmul_rn(-g, delz));
    const bool hi = x >= s.cv, lo = x <= 0.0f;
    ga += hi ? g : (lo ? 0.0f : inner);
    return (hi || lo) ? 0.0f : g;
  }
  // PACTplusSymSTE_rev1.backward: z = (x + cv) / step; delz = 2 (round(z) - z) / n; +-1 outside
  const float z = Elem<XT>::rnd(div_exact(Elem<XT>::rnd(__fadd_rn(x, s.cv)), s.step, s.rstep));
  const float d0 = Elem<XT>::rnd(__fsub_rn(rint_small(z), z));
  const float delz = Elem<XT>::rnd(div_exact(Elem<XT>::rnd(__fmul_rn(2.0f, d0)), s.n, s.rn));
  const bool hi = x >= s.cv, lo = x <= -s.cv;
  const float w = hi ? 1.0f : (lo ? -1.0f : delz);
  ga += Elem<XT>::rnd(__fmul_rn(w, g));
  return (hi || lo) ? 0.0f : g;
}

template <typename XT>
__global__ void __launch_bounds__(kFqThreads) pact2_fwd_kernel(const PactParams p) {
  const PactScalars s = pact_scalars<XT>(p);
  const XT* x = reinterpret_cast<const XT*>(p.x);
  XT* out = reinterpret_cast<XT*>(p.out);
  const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  const int64_t nvec = vec ? (p.numel >> 4) : 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float v[16];
    load16(x + i * 16, v);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = pact_fwd_one<XT>(s, v[j]);
    store16(out + i * 16, v);
  }
  for (int64_t i = nvec * 16 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.numel; i += stride)
    store1(out + i, pact_fwd_one<XT>(s, load1(x + i)));
}

template <typename XT>
__global__ void __launch_bounds__(kFqThreads) pact2_bwd_kernel(const PactParams p) {
  __shared__ float red[2][32];
  const PactScalars s = pact_scalars<XT>(p);
  const XT* x = reinterpret_cast<const XT*>(p.x);
  const XT* g = reinterpret_cast<const XT*>(p.g);
  XT* out = reinterpret_cast<XT*>(p.out);
  const bool vec =
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  const int64_t nvec = vec ? (p.numel >> 4) : 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  float ga = 0.0f, gan = 0.0f;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float v[16], gv[16];
    load16(x + i * 16, v);
    load16(g + i * 16, gv);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = pact_bwd_one<XT>(s, v[j], gv[j], ga, gan);
    store16(out + i * 16, v);
  }
  for (int64_t i = nvec * 16 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.numel; i += stride)
    store1(out + i, pact_bwd_one<XT>(s, load1(x + i), load1(g + i), ga, gan));
  ga = block_reduce<OpSum>(ga, red[0], 0.0f);
  gan = block_reduce<OpSum>(gan, red[1], 0.0f);
  if (threadIdx.x == 0) {
    p.ws[2 * blockIdx.x] = ga;
    p.ws[2 * blockIdx.x + 1] = gan;
  }
}

// Adds the per-block partial sums in index order.
__global__ void __launch_bounds__(kFqThreads) pact2_bwd_finish_kernel(const float* ws, int nblocks, float* grad_clip) {
  __shared__ float red[2][32];
  float ga = 0.0f, gan = 0.0f;
  for (int i = threadIdx.x; i < nblocks; i += blockDim.x) {
    ga += ws[2 * i];
    gan += ws[2 * i + 1];
  }
  ga = block_reduce<OpSum>(ga, red[0], 0.0f);
  gan = block_reduce<OpSum>(gan, red[1], 0.0f);
  if (threadIdx.x == 0) {
    grad_clip[0] = ga;
    grad_clip[1] = gan;
  }
}

// Fixed upper bound on the grid of the elementwise kernels; qlin_pact2_bwd_noalloc sizes its built-in scratch by it.
constexpr int kFqMaxBlocks = 148 * 8;

// Grid of the elementwise kernels: a function of numel and of the device's SM count only, so the reduction order is
// fixed on a given GPU model (eight blocks per SM, never more than kFqMaxBlocks).
static int fq_grid(int64_t numel) {
  const int64_t per_block = static_cast<int64_t>(kFqThreads) * 16;
  int64_t blocks = (numel + per_block - 1) / per_block;
  int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (cap < 1 || cap > kFqMaxBlocks) cap = kFqMaxBlocks;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

// Argument checks shared by every PACT+ entry point.  `needs_workspace` is false for the entry point that brings its
// own scratch memory.
static int check_pact(const qlin_pact2_args* a, bool bwd, const char* name, bool needs_workspace = true) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "%s: args is NULL", name);
  if (a->x == nullptr || a->out == nullptr || a->clip_val == nullptr ||
      (a->variant == QLIN_PACT_TWO_SIDED && a->clip_valn == nullptr))
    return fail(QLIN_ERR_NULL, "%s: x, out, clip_val or clip_valn is NULL", name);
  if (a->variant < QLIN_PACT_TWO_SIDED || a->variant > QLIN_PACT_SYMMETRIC)
    return fail(QLIN_ERR_UNSUPPORTED, "%s: unknown variant %d", name, a->variant);
  if (bwd && (a->grad_out == nullptr || a->grad_clip == nullptr || (needs_workspace && a->workspace == nullptr)))
    return fail(QLIN_ERR_NULL, "%s: grad_out, grad_clip or workspace is NULL", name);
  if (a->numel < 0) return fail(QLIN_ERR_BAD_SHAPE, "%s: negative numel", name);
  if (a->num_bits < 2 || a->num_bits > 16) return fail(QLIN_ERR_UNSUPPORTED, "%s: num_bits must be in [2, 16]", name);
  if (a->dtype != QLIN_DT_F32 && a->dtype != QLIN_DT_F16 && a->dtype != QLIN_DT_BF16)
    return fail(QLIN_ERR_BAD_DTYPE, "%s: dtype must be F32, F16 or BF16", name);
  return QLIN_OK;
}

static PactParams to_params(const qlin_pact2_args* a) {
  PactParams p;
  p.x = a->x;
  p.g = a->grad_out;
  p.out = a->out;
  p.cv = a->clip_val;
  p.cvn = a->clip_valn;
  p.grad_clip = a->grad_clip;
  p.ws = static_cast<float*>(a->workspace);
  p.numel = a->numel;
  p.num_bits = a->num_bits;
  p.align_zero = a->align_zero != 0;
  p.variant = a->variant;
  return p;
}

}  // namespace qlin

using namespace qlin;

extern "C" size_t qlin_pact2_bwd_workspace_bytes(int64_t numel) {
  return static_cast<size_t>(fq_grid(numel < 0 ? 0 : numel)) * 2 * sizeof(float);
}

extern "C" int qlin_pact2_fwd(const qlin_pact2_args* a, void* stream) {
  int rc = check_pact(a, false, "qlin_pact2_fwd");
  if (rc != QLIN_OK) return rc;
  if (a->numel == 0) return QLIN_OK;
  const PactParams p = to_params(a);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = fq_grid(a->numel);
  switch (a->dtype) {
    case QLIN_DT_F32:
      pact2_fwd_kernel<float><<<grid, kFqThreads, 0, s>>>(p);
      break;
    case QLIN_DT_F16:
      pact2_fwd_kernel<__half><<<grid, kFqThreads, 0, s>>>(p);
      break;
    default:
      pact2_fwd_kernel<__nv_bfloat16><<<grid, kFqThreads, 0, s>>>(p);
      break;
  }
  QLIN_CHECK_LAUNCH("qlin_pact2_fwd");
  return QLIN_OK;
}

extern "C" int qlin_pact2_bwd(const qlin_pact2_args* a, void* stream) {
  int rc = check_pact(a, true, "qlin_pact2_bwd");
  if (rc != QLIN_OK) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const PactParams p = to_params(a);
  const int grid = fq_grid(a->numel);
  if (a->numel > 0) {
    switch (a->dtype) {
      case QLIN_DT_F32:
        pact2_bwd_kernel<float><<<grid, kFqThreads, 0, s>>>(p);
        break;
      case QLIN_DT_F16:
        pact2_bwd_kernel<__half><<<grid, kFqThreads, 0, s>>>(p);
        break;
      default:
        pact2_bwd_kernel<__nv_bfloat16><<<grid, kFqThreads, 0, s>>>(p);
        break;
    }
    QLIN_CHECK_LAUNCH("qlin_pact2_bwd");
  }
  pact2_bwd_finish_kernel<<<1, kFqThreads, 0, s>>>(p.ws, a->numel > 0 ? grid : 0, p.grad_clip);
  QLIN_CHECK_LAUNCH("qlin_pact2_bwd(finish)");
  return QLIN_OK;
}

// ------------------------------------------------------------------------------------------------
// qlin_pact2_bwd_noalloc: the PACT+ backward for callers that have no device memory to lend.
//
// qlin_pact2_bwd needs a small workspace for the per-block partial sums of the two clip-value
// gradients, and the caller has to get it from somewhere.  Some callers cannot: a host runtime whose
// device pool is carved up once at start-up and sealed, an autograd hook that is handed nothing but
// its input and output buffers, a step loop that must not call cudaMalloc because it may fail under
// a fixed memory budget or stall the device in the middle of a step.  For them the same two kernels
// run with the partial sums in a fixed array that is part of the library image: every GPU that loads
// the library holds these kNoAllocScratchFloats * 4 bytes until the process exits.
//
// In host code the array's name is only a handle; the device address is looked up once per device
// with cudaGetSymbolAddress, while that device is current, and that pointer is what the kernels
// receive.  The look-up happens in the first call on each device, so make that first call outside
// any stream capture.  Nothing in the array has to start at zero: each call writes every slot that
// its second kernel reads.  All calls on a device share the array, so two calls whose kernels can
// overlap on the GPU (different streams without an ordering between them) race on it.
// ------------------------------------------------------------------------------------------------
namespace qlin {

constexpr int kNoAllocMaxBlocks = kFqMaxBlocks;            // the grid cap of the elementwise kernels
constexpr int kNoAllocScratchFloats = 2 * kNoAllocMaxBlocks;  // 9472 bytes
constexpr int64_t kNoAllocMaxNumel = int64_t(1) << 31;     // elements per call

static __device__ __align__(256) float g_pact2_noalloc_scratch[kNoAllocScratchFloats];

// Device address of the scratch array on the current device, looked up once per device.
static int noalloc_scratch_ptr(float** out) {
  static float* cached[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(QLIN_ERR_DEVICE, "qlin_pact2_bwd_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(QLIN_ERR_DEVICE, "qlin_pact2_bwd_noalloc: device ordinal %d out of range", dev);
  if (cached[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_pact2_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(QLIN_ERR_DEVICE, "qlin_pact2_bwd_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return QLIN_OK;
}

}  // namespace qlin

extern "C" int64_t qlin_pact2_bwd_noalloc_max_numel(void) { return qlin::kNoAllocMaxNumel; }

extern "C" int qlin_pact2_bwd_noalloc(const qlin_pact2_args* a, void* stream) {
  const char* name = "qlin_pact2_bwd_noalloc";
  int rc = check_pact(a, true, name, /*needs_workspace=*/false);
  if (rc != QLIN_OK) return rc;
  if (a->numel > kNoAllocMaxNumel)
    return fail(QLIN_ERR_TOO_LARGE, "%s: numel %lld exceeds the built-in scratch limit of %lld elements per call", name,
                static_cast<long long>(a->numel), static_cast<long long>(kNoAllocMaxNumel));
  const int grid = fq_grid(a->numel);
  if (grid > kNoAllocMaxBlocks) return fail(QLIN_ERR_TOO_LARGE, "%s: grid %d exceeds the built-in scratch", name, grid);
  float* scratch = nullptr;
  rc = noalloc_scratch_ptr(&scratch);
  if (rc != QLIN_OK) return rc;
  PactParams p = to_params(a);
  p.ws = scratch;  // the looked-up device address, never the host-side symbol
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->numel > 0) {
    switch (a->dtype) {
      case QLIN_DT_F32:
        pact2_bwd_kernel<float><<<grid, kFqThreads, 0, s>>>(p);
        break;
      case QLIN_DT_F16:
        pact2_bwd_kernel<__half><<<grid, kFqThreads, 0, s>>>(p);
        break;
      default:
        pact2_bwd_kernel<__nv_bfloat16><<<grid, kFqThreads, 0, s>>>(p);
        break;
    }
    QLIN_CHECK_LAUNCH("qlin_pact2_bwd_noalloc");
  }
  pact2_bwd_finish_kernel<<<1, kFqThreads, 0, s>>>(scratch, a->numel > 0 ? grid : 0, p.grad_clip);
  QLIN_CHECK_LAUNCH("qlin_pact2_bwd_noalloc(finish)");
  return QLIN_OK;
}
