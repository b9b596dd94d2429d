// qlin_shard_reduce: the reduce-scatter half of a row-parallel Linear, done by the NVLink switch.
//
// Every GPU of the node has written its partial output [tokens, hidden] (bf16) into its own copy of a buffer that
// all of them have bound to one multicast object.  The owner of a block of tokens reads that block through the
// multicast mapping with multimem.ld_reduce: each 16-byte load returns the sum over all GPUs' copies (accumulated in
// fp32 in the switch, rounded to bf16 once).  This kernel streams such a block, optionally adds a local tensor (the
// residual stream) in fp32, and writes the bf16 result to local memory:
//     out[r, c] = bf16( float(add[r, c]) + float(sum over GPUs of part[r, c]) )
// It is bound by the links, not by the SMs: a few CTAs with many loads in flight each (eight 16-byte loads per thread
// before the first use) are enough, and `max_ctas` keeps it off the SMs that a GEMM of another stream is using.
#include <cuda_bf16.h>

#include "qlin_internal.h"

namespace qlin {

constexpr int kMcThreads = 512;
constexpr int kMcUnroll = 8;

struct ShardReduceParams {
  const uint4* src_mc;  // multicast mapping, first element of the block
  const uint4* add;     // optional local addend
  uint4* out;
  int64_t ld_src, ld_add, ld_out;  // in 16-byte vectors
  int32_t rows, vec_per_row;
};

__device__ __forceinline__ uint4 mc_ld_reduce(const uint4* p) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ uint32_t mc_add_pair(uint32_t a, uint32_t b) {
  const float lo = __uint_as_float(a << 16) + __uint_as_float(b << 16);
  const float hi = __uint_as_float(a & 0xFFFF0000u) + __uint_as_float(b & 0xFFFF0000u);
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(kMcThreads) shard_reduce_kernel(const ShardReduceParams p) {
  const int64_t total = static_cast<int64_t>(p.rows) * p.vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kMcThreads;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * kMcThreads + threadIdx.x; base < total; base += stride * kMcUnroll) {
    uint4 v[kMcUnroll], a[kMcUnroll];
    int64_t r[kMcUnroll];
    int c[kMcUnroll];
#pragma unroll
    for (int u = 0; u < kMcUnroll; ++u) {
      const int64_t i = base + u * stride;
      r[u] = i / p.vec_per_row;
      c[u] = static_cast<int>(i - r[u] * p.vec_per_row);
      if (i < total) v[u] = mc_ld_reduce(p.src_mc + r[u] * p.ld_src + c[u]);
    }
    if (p.add != nullptr) {
#pragma unroll
      for (int u = 0; u < kMcUnroll; ++u)
        if (base + u * stride < total) a[u] = p.add[r[u] * p.ld_add + c[u]];
    }
#pragma unroll
    for (int u = 0; u < kMcUnroll; ++u) {
      if (base + u * stride >= total) continue;
      uint4 o = v[u];
      if (p.add != nullptr) {
        o.x = mc_add_pair(a[u].x, v[u].x);
        o.y = mc_add_pair(a[u].y, v[u].y);
        o.z = mc_add_pair(a[u].z, v[u].z);
        o.w = mc_add_pair(a[u].w, v[u].w);
      }
      p.out[r[u] * p.ld_out + c[u]] = o;
    }
  }
}

}  // namespace qlin

using namespace qlin;

extern "C" int qlin_shard_reduce(const qlin_shard_reduce_args* a, void* stream) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_shard_reduce: args is NULL");
  if (a->rows < 0 || a->cols < 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_shard_reduce: negative dimension");
  if (a->rows == 0 || a->cols == 0) return QLIN_OK;
  if (a->src_multicast == nullptr || a->out == nullptr) return fail(QLIN_ERR_NULL, "qlin_shard_reduce: src_multicast or out is NULL");
  if (a->cols % 8 != 0 || a->ld_src % 8 != 0 || a->ld_out % 8 != 0 || (a->add != nullptr && a->ld_add % 8 != 0))
    return fail(QLIN_ERR_BAD_SHAPE, "qlin_shard_reduce: cols and leading dimensions must be multiples of 8 elements");
  if (!aligned16(a->src_multicast) || !aligned16(a->out) || !aligned16(a->add))
    return fail(QLIN_ERR_BAD_ALIGN, "qlin_shard_reduce: pointers must be 16-byte aligned");
  if (a->ld_src < a->cols || a->ld_out < a->cols || (a->add != nullptr && a->ld_add < a->cols))
    return fail(QLIN_ERR_BAD_SHAPE, "qlin_shard_reduce: leading dimension smaller than the row length");
  ShardReduceParams p;
  p.src_mc = static_cast<const uint4*>(a->src_multicast);
  p.add = static_cast<const uint4*>(a->add);
  p.out = static_cast<uint4*>(a->out);
  p.ld_src = a->ld_src / 8;
  p.ld_add = a->ld_add / 8;
  p.ld_out = a->ld_out / 8;
  p.rows = a->rows;
  p.vec_per_row = a->cols / 8;
  const int64_t total = static_cast<int64_t>(p.rows) * p.vec_per_row;
  int64_t grid = (total + static_cast<int64_t>(kMcThreads) * kMcUnroll - 1) / (static_cast<int64_t>(kMcThreads) * kMcUnroll);
  const int64_t cap = a->max_ctas > 0 ? a->max_ctas : static_cast<int64_t>(sm_count()) * 2;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  shard_reduce_kernel<<<static_cast<int>(grid), kMcThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  QLIN_CHECK_LAUNCH("qlin_shard_reduce");
  return QLIN_OK;
}
