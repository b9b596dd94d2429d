// qlin_col_absmax: per-input-channel absolute maximum of an activation tensor, kept as a running maximum over
// calibration batches.  This is the statistic SmoothQuant calibration collects for every Linear input
// (activation_stats, fms_mo/quant/ptq.py:2586-2596: tensor.view(-1, hidden).abs().max(dim=0), then torch.max with the
// value kept so far) and the only device work of that pass; the reference copies every batch's result to the host, here
// the running vector stays on the device.
//
// HBM-bound: one read of x (rows x cols), cols * 4 bytes written.  A block owns a tile of 16 * TPB columns and a
// slice of the rows; every thread walks its 16 columns down the slice with 16-byte (2-byte dtypes) or 64-byte (fp32)
// loads, and the slices are combined with atomicMax on the bit patterns (non-negative floats order like unsigned
// integers), so the result does not depend on scheduling.  NaNs are propagated as torch.max does: a NaN in a column
// makes the column's result NaN.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "qlin_internal.h"
#include "qlin_rows.cuh"

namespace qlin {

constexpr int kCalThreads = 128;

struct ColAbsmaxParams {
  const void* x;
  float* amax_io;
  int64_t ldx;
  int32_t rows, cols, rows_per_block;
};

// Largest of a and b as torch.max sees them: NaN wins.
__device__ __forceinline__ float max_nan(float a, float b) { return (a != a || b != b) ? __int_as_float(0x7fc00000) : fmaxf(a, b); }

__device__ __forceinline__ void col_publish(float* dst, float v) {
  // |v| >= 0: the unsigned order of the bit patterns is the numeric order; a NaN pattern (0x7fc00000) is above every
  // finite pattern and below none, so it survives the maximum
  atomicMax(reinterpret_cast<unsigned int*>(dst), __float_as_uint(v));
}

template <typename XT>
__global__ void __launch_bounds__(kCalThreads) col_absmax_vec_kernel(const ColAbsmaxParams p) {
  const int chunk = blockIdx.x * kCalThreads + threadIdx.x;  // 16 columns each
  if (chunk * 16 >= p.cols) return;
  const int r0 = blockIdx.y * p.rows_per_block;
  const int r1 = min(p.rows, r0 + p.rows_per_block);
  const XT* x = reinterpret_cast<const XT*>(p.x) + static_cast<int64_t>(chunk) * 16;
  float m[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) m[i] = 0.0f;
  int r = r0;
  for (; r + 1 < r1; r += 2) {  // two rows in flight
    float a[16], b[16];
    load16(x + static_cast<int64_t>(r) * p.ldx, a);
    load16(x + static_cast<int64_t>(r + 1) * p.ldx, b);
#pragma unroll
    for (int i = 0; i < 16; ++i) m[i] = max_nan(m[i], max_nan(fabsf(a[i]), fabsf(b[i])));
  }
  if (r < r1) {
    float a[16];
    load16(x + static_cast<int64_t>(r) * p.ldx, a);
#pragma unroll
    for (int i = 0; i < 16; ++i) m[i] = max_nan(m[i], fabsf(a[i]));
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) col_publish(p.amax_io + chunk * 16 + i, m[i]);
}

// Any alignment, any column count: one thread per column.
template <typename XT>
__global__ void __launch_bounds__(kCalThreads) col_absmax_scalar_kernel(const ColAbsmaxParams p) {
  const int c = blockIdx.x * kCalThreads + threadIdx.x;
  if (c >= p.cols) return;
  const int r0 = blockIdx.y * p.rows_per_block;
  const int r1 = min(p.rows, r0 + p.rows_per_block);
  const XT* x = reinterpret_cast<const XT*>(p.x) + c;
  float m = 0.0f;
  for (int r = r0; r < r1; ++r) m = max_nan(m, fabsf(load1(x + static_cast<int64_t>(r) * p.ldx)));
  col_publish(p.amax_io + c, m);
}

template <typename XT>
static int launch_col_absmax(ColAbsmaxParams p, cudaStream_t s) {
  const int es = static_cast<int>(sizeof(XT));
  const bool vec = p.cols % 16 == 0 && aligned16(p.x) && (p.ldx * es) % 16 == 0;
  const int col_blocks = vec ? (p.cols / 16 + kCalThreads - 1) / kCalThreads : (p.cols + kCalThreads - 1) / kCalThreads;
  // enough row slices to fill the GPU about four times over, at least 32 rows each
  int slices = (sm_count() * 16 + col_blocks - 1) / col_blocks;
  const int max_slices = (p.rows + 31) / 32;
  if (slices > max_slices) slices = max_slices;
  if (slices < 1) slices = 1;
  if (slices > 65535) slices = 65535;
  p.rows_per_block = (p.rows + slices - 1) / slices;
  slices = (p.rows + p.rows_per_block - 1) / p.rows_per_block;
  const dim3 grid(static_cast<unsigned>(col_blocks), static_cast<unsigned>(slices), 1);
  if (vec) {
    col_absmax_vec_kernel<XT><<<grid, kCalThreads, 0, s>>>(p);
  } else {
    col_absmax_scalar_kernel<XT><<<grid, kCalThreads, 0, s>>>(p);
  }
  QLIN_CHECK_LAUNCH("qlin_col_absmax");
  return QLIN_OK;
}

}  // namespace qlin

using namespace qlin;

extern "C" int qlin_col_absmax(const qlin_col_absmax_args* a, void* stream) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_col_absmax: args is NULL");
  if (a->rows < 0 || a->cols < 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_col_absmax: negative dimension");
  if ((a->x == nullptr && a->rows > 0 && a->cols > 0) || (a->amax_io == nullptr && a->cols > 0))
    return fail(QLIN_ERR_NULL, "qlin_col_absmax: x or amax_io is NULL");
  if (a->ldx < a->cols) return fail(QLIN_ERR_BAD_SHAPE, "qlin_col_absmax: ldx smaller than the row length");
  if (a->dtype != QLIN_DT_F32 && a->dtype != QLIN_DT_F16 && a->dtype != QLIN_DT_BF16)
    return fail(QLIN_ERR_BAD_DTYPE, "qlin_col_absmax: dtype must be F32, F16 or BF16");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->cols == 0) return QLIN_OK;
  if (!a->accumulate) {
    cudaError_t e = cudaMemsetAsync(a->amax_io, 0, static_cast<size_t>(a->cols) * sizeof(float), s);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(QLIN_ERR_LAUNCH, "qlin_col_absmax: cudaMemsetAsync: %s", cudaGetErrorString(e));
    }
  }
  if (a->rows == 0) return QLIN_OK;
  ColAbsmaxParams p;
  p.x = a->x;
  p.amax_io = a->amax_io;
  p.ldx = a->ldx;
  p.rows = a->rows;
  p.cols = a->cols;
  p.rows_per_block = a->rows;
  switch (a->dtype) {
    case QLIN_DT_F32:
      return launch_col_absmax<float>(p, s);
    case QLIN_DT_F16:
      return launch_col_absmax<__half>(p, s);
    default:
      return launch_col_absmax<__nv_bfloat16>(p, s);
  }
}
