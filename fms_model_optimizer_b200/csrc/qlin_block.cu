// qlin_block_quant and qlin_rope: the per-token work that surrounds the W8A8 Linears of a decoder
// block, fused so that every activation tensor is read once.
//
// qlin_block_quant builds the bf16 input row of up to three Linears that share it and quantises it
// per token for each of them (each Linear has its own SmoothQuant scale), in one pass:
//   prologue NORM  : t = x (+ r);  optionally store t;  h = bf16(t * rsqrt(mean t^2 + eps) * w)
//   prologue SILU  : h = bf16(bf16(silu(x)) * r)
//   prologue PLAIN : h = x
//   for each output o: v = bf16(h / smooth_o); s = bf16(max(amax |v|, 1e-5) / 127) (or given);
//                      codes_o = int8(rint(bf16(v / s)))   -- qa_dynamic_max_qfunc of the reference
// A block owns a row at a time; each thread keeps its 16-element slice of h in registers across the
// outputs, so the traffic per row is one read of the inputs plus the writes of the codes.
//
// The quantise step is the bf16 single-multiply path of qlin_quant.cu: with bf16 values and
// bf16-valued smoothing / row scales, bf16(a * RN_f32(1 / b)) equals the reference's
// bf16(RN_f32(a / b)) (a quotient of two 8-bit significands is never within 2^-18 of a bf16
// rounding boundary).  Callers must pass correctly rounded reciprocals of bf16-valued scales.
#include <cstdlib>

#include <cuda_bf16.h>

#include "qlin_internal.h"
#include "qlin_rows.cuh"

namespace qlin {

struct BlockQuantParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* r;
  __nv_bfloat16* x_out;
  __nv_bfloat16* h_out;
  const __nv_bfloat16* norm_w;
  const float* mul[3];
  uint8_t* codes[3];
  float* scale_out[3];
  const float* scale_in;
  int64_t scale_in_stride;
  int32_t scale_in_parts;
  int64_t ldx, ldr, ldxo, ldh, ldq[3];
  int64_t r_part_stride;
  int32_t r_parts;
  int32_t rows, cols, nout, prologue, mode, levels;
  float norm_eps, dyn_eps;
  // replicated outputs
  uint8_t* dst_base[8];
  int64_t codes_off[3], scale_off[3];
  int32_t ndst, dst_row0;
  int32_t max_ctas;
  int32_t r_multimem, dst_multimem;
};

__device__ __forceinline__ uint32_t bq_pack(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// Packed pair arithmetic: two bf16 values of one word as float2, multiplied by two fp32 factors with one packed
// instruction and rounded back to a bf16 pair with one packed conversion (the same roundings as the scalar forms).
__device__ __forceinline__ float2 bq_unpack(uint32_t w) { return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u)); }
__device__ __forceinline__ uint32_t bq_mul_pack(uint32_t w, float2 f) {
  const __nv_bfloat162 h = __float22bfloat162_rn(__fmul2_rn(bq_unpack(w), f));
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float bq_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bq_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
// SiLU rounded to bf16; the fast exponential and division are exact to well below half a bf16 place
__device__ __forceinline__ float bq_silu(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

__device__ __forceinline__ void bq_load8(const __nv_bfloat16* p, uint32_t (&w)[8]) {
  const uint4 a = reinterpret_cast<const uint4*>(p)[0], b = reinterpret_cast<const uint4*>(p)[1];
  w[0] = a.x, w[1] = a.y, w[2] = a.z, w[3] = a.w, w[4] = b.x, w[5] = b.y, w[6] = b.z, w[7] = b.w;
}
__device__ __forceinline__ void bq_store8(__nv_bfloat16* p, const uint32_t (&w)[8]) {
  reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
  reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// NVLink-switch forms for buffers that every GPU of the node has bound to one multicast object: a load that returns the
// sum of all GPUs' copies (bf16 pairs, accumulated in fp32 by the switch, rounded once), and a store that lands in
// every GPU's copy.  The address is the multicast mapping of the buffer, not a peer pointer.
__device__ __forceinline__ void bq_load8_reduce(const __nv_bfloat16* mc, uint32_t (&w)[8]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
               : "l"(mc)
               : "memory");
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
               : "l"(mc + 8)
               : "memory");
}
__device__ __forceinline__ void bq_store16_all(uint8_t* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ void bq_store_f32_all(float* mc, float v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(v) : "memory");
}

template <int TPB>
__global__ void __launch_bounds__(TPB) block_quant_kernel(const BlockQuantParams p, int mul_in_smem) {
  // The reciprocal SmoothQuant vectors are the same for every row: with `mul_in_smem` the block copies them into shared
  // memory once, quarter-transposed ([output][quarter][slice] of four floats) so that the four 16-byte reads of a
  // thread's slice are conflict free, instead of re-reading them through L1 for every row and output.
  extern __shared__ __align__(16) float mul_s[];
  __shared__ float red[2][32];
  const int nchunks = p.cols >> 4;
  const int ch = threadIdx.x;
  const bool active = ch < nchunks;
  if (mul_in_smem) {
    for (int o = 0; o < p.nout; ++o) {
      if (p.mul[o] == nullptr) continue;
      for (int i = threadIdx.x; i < nchunks * 4; i += TPB) {
        const int c = i >> 2, q = i & 3;
        reinterpret_cast<float4*>(mul_s)[(o * 4 + q) * nchunks + c] = reinterpret_cast<const float4*>(p.mul[o])[i];
      }
    }
    __syncthreads();
  }
  const float eps = Elem<__nv_bfloat16>::rnd(p.dyn_eps);
  const float inv_cols = 1.0f / static_cast<float>(p.cols);
  int flip = 0;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
    uint32_t h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) h[j] = 0u;
    if (p.prologue == QLIN_BLOCK_NORM) {
      float ssq = 0.0f;
      if (active) {
        bq_load8(p.x + static_cast<int64_t>(row) * p.ldx + ch * 16, h);
        if (p.r != nullptr) {
          uint32_t a[8];
          const __nv_bfloat16* rp = p.r + static_cast<int64_t>(row) * p.ldr + ch * 16;
          if (p.r_multimem) {
            bq_load8_reduce(rp, a);  // the switch adds the row-parallel shards' partial outputs
          } else {
            bq_load8(rp, a);
          }
          if (p.r_parts > 1 && !p.r_multimem) {  // sum of the shards' partial outputs: fp32 in index order, one rounding
            float acc[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[2 * j] = bq_lo(a[j]), acc[2 * j + 1] = bq_hi(a[j]);
            for (int s = 1; s < p.r_parts; ++s) {
              bq_load8(rp + s * p.r_part_stride, a);
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[2 * j] += bq_lo(a[j]), acc[2 * j + 1] += bq_hi(a[j]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] = bq_pack(acc[2 * j], acc[2 * j + 1]);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) h[j] = bq_pack(__fadd_rn(bq_lo(h[j]), bq_lo(a[j])), __fadd_rn(bq_hi(h[j]), bq_hi(a[j])));
          if (p.x_out != nullptr) bq_store8(p.x_out + static_cast<int64_t>(row) * p.ldxo + ch * 16, h);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ssq += bq_lo(h[j]) * bq_lo(h[j]) + bq_hi(h[j]) * bq_hi(h[j]);
      }
      ssq = block_reduce<OpSum>(ssq, red[flip], 0.0f);
      flip ^= 1;
      const float rstd = rsqrtf(ssq * inv_cols + p.norm_eps);
      if (active) {
        uint32_t w[8];
        bq_load8(p.norm_w + ch * 16, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = bq_pack(bq_lo(h[j]) * rstd * bq_lo(w[j]), bq_hi(h[j]) * rstd * bq_hi(w[j]));
      }
    } else if (active) {
      bq_load8(p.x + static_cast<int64_t>(row) * p.ldx + ch * 16, h);
      if (p.prologue == QLIN_BLOCK_SILU_MUL) {
        uint32_t u[8];
        bq_load8(p.r + static_cast<int64_t>(row) * p.ldr + ch * 16, u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t sl = bq_pack(bq_silu(bq_lo(h[j])), bq_silu(bq_hi(h[j])));
          h[j] = bq_pack(__fmul_rn(bq_lo(sl), bq_lo(u[j])), __fmul_rn(bq_hi(sl), bq_hi(u[j])));
        }
      }
    }
    if (active && p.h_out != nullptr) bq_store8(p.h_out + static_cast<int64_t>(row) * p.ldh + ch * 16, h);

    for (int o = 0; o < p.nout; ++o) {
      uint32_t v[8];
      __nv_bfloat162 amax2 = __floats2bfloat162_rn(0.0f, 0.0f);
      if (active) {
        if (p.mul[o] != nullptr) {
          float m[16];
          if (mul_in_smem) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 f = reinterpret_cast<const float4*>(mul_s)[(o * 4 + q) * nchunks + ch];
              m[4 * q] = f.x, m[4 * q + 1] = f.y, m[4 * q + 2] = f.z, m[4 * q + 3] = f.w;
            }
          } else {
            load16(p.mul[o] + ch * 16, m);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = bq_mul_pack(h[j], make_float2(m[2 * j], m[2 * j + 1]));
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = h[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) amax2 = __hmax2(amax2, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&v[j])));
      }
      float s;
      if (p.mode == QLIN_BLOCK_GIVEN_SCALE) {
        s = p.scale_in[row];
        // the shards of a row-parallel Linear each reported the scale of their slice: the row's scale is the largest
        for (int k = 1; k < p.scale_in_parts; ++k) s = fmaxf(s, p.scale_in[k * p.scale_in_stride + row]);
        if (threadIdx.x == 0 && p.scale_out[o] != nullptr) p.scale_out[o][row] = s;
      } else {
        float amax = fmaxf(__low2float(amax2), __high2float(amax2));
        amax = block_reduce<OpMax>(amax, red[flip], 0.0f);
        flip ^= 1;
        s = Elem<__nv_bfloat16>::rnd(__fdiv_rn(fmaxf(amax, eps), static_cast<float>(p.levels)));
        if (p.dst_multimem) {
          if (threadIdx.x == 0) {
            bq_store_f32_all(reinterpret_cast<float*>(p.dst_base[0] + p.scale_off[o]) + p.dst_row0 + row, s);
            if (p.ndst > 1) reinterpret_cast<float*>(p.dst_base[1] + p.scale_off[o])[p.dst_row0 + row] = s;
          }
        } else if (p.ndst > 0) {
          if (static_cast<int>(threadIdx.x) < p.ndst)
            reinterpret_cast<float*>(p.dst_base[threadIdx.x] + p.scale_off[o])[p.dst_row0 + row] = s;
        } else if (threadIdx.x == 0 && p.scale_out[o] != nullptr) {
          p.scale_out[o][row] = s;
        }
      }
      if (p.mode == QLIN_BLOCK_SCALE_ONLY || !active) continue;
      const float rs = __frcp_rn(s);
      const float2 rs2 = make_float2(rs, rs);
      const float2 magic = make_float2(12582912.0f, 12582912.0f);  // 1.5 * 2^23: the sum's low mantissa byte is rint's code
      uint32_t out[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const float2 qa = __fadd2_rn(bq_unpack(bq_mul_pack(v[2 * g], rs2)), magic);
        const float2 qb = __fadd2_rn(bq_unpack(bq_mul_pack(v[2 * g + 1], rs2)), magic);
        out[g] = __byte_perm(__byte_perm(__float_as_uint(qa.x), __float_as_uint(qa.y), 0x0040),
                             __byte_perm(__float_as_uint(qb.x), __float_as_uint(qb.y), 0x0040), 0x5410);
      }
      const uint4 packed = make_uint4(out[0], out[1], out[2], out[3]);
      if (p.dst_multimem) {
        const int64_t off = p.codes_off[o] + static_cast<int64_t>(p.dst_row0 + row) * p.ldq[o] + ch * 16;
        bq_store16_all(p.dst_base[0] + off, packed);
        // this GPU's own copy also gets a plain store: its own later kernels must not depend on the round trip of the
        // multicast store through the switch (the copy that arrives that way carries the same bytes)
        if (p.ndst > 1) *reinterpret_cast<uint4*>(p.dst_base[1] + off) = packed;
      } else if (p.ndst > 0) {
        const int64_t off = p.codes_off[o] + static_cast<int64_t>(p.dst_row0 + row) * p.ldq[o] + ch * 16;
        for (int d = 0; d < p.ndst; ++d) *reinterpret_cast<uint4*>(p.dst_base[d] + off) = packed;
      } else {
        *reinterpret_cast<uint4*>(p.codes[o] + static_cast<int64_t>(row) * p.ldq[o] + ch * 16) = packed;
      }
    }
  }
}

// Rotary embedding in place on [tokens, heads, head_dim] bf16: position = token % seq_len;
// out[..., i] = x[i] cos[i] - x[i + d/2] sin[i], out[..., i + d/2] = x[i + d/2] cos[i] + x[i] sin[i],
// computed in fp32 and rounded once.  One thread rotates 8 pairs.
struct RopeParams {
  __nv_bfloat16* x;
  const float* cos;
  const float* sin;
  int64_t ld_token;
  int32_t tokens, heads, head_dim, seq_len;
};

__global__ void __launch_bounds__(256) rope_kernel(const RopeParams p) {
  const int half = p.head_dim >> 1;
  const int groups = half >> 3;  // 8 pairs per thread
  const int64_t total = static_cast<int64_t>(p.tokens) * p.heads * groups;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i % groups);
    const int64_t th = i / groups;
    const int head = static_cast<int>(th % p.heads);
    const int64_t token = th / p.heads;
    const int pos = static_cast<int>(token % p.seq_len);
    __nv_bfloat16* base = p.x + token * p.ld_token + static_cast<int64_t>(head) * p.head_dim + g * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(base), b = *reinterpret_cast<const uint4*>(base + half);
    const float4 c0 = *reinterpret_cast<const float4*>(p.cos + static_cast<int64_t>(pos) * half + g * 8);
    const float4 c1 = *reinterpret_cast<const float4*>(p.cos + static_cast<int64_t>(pos) * half + g * 8 + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(p.sin + static_cast<int64_t>(pos) * half + g * 8);
    const float4 s1 = *reinterpret_cast<const float4*>(p.sin + static_cast<int64_t>(pos) * half + g * 8 + 4);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint32_t ao[4], bo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float x0 = bq_lo(aw[j]), x1 = bq_hi(aw[j]), y0 = bq_lo(bw[j]), y1 = bq_hi(bw[j]);
      ao[j] = bq_pack(x0 * cs[2 * j] - y0 * sn[2 * j], x1 * cs[2 * j + 1] - y1 * sn[2 * j + 1]);
      bo[j] = bq_pack(y0 * cs[2 * j] + x0 * sn[2 * j], y1 * cs[2 * j + 1] + x1 * sn[2 * j + 1]);
    }
    *reinterpret_cast<uint4*>(base) = make_uint4(ao[0], ao[1], ao[2], ao[3]);
    *reinterpret_cast<uint4*>(base + half) = make_uint4(bo[0], bo[1], bo[2], bo[3]);
  }
}

template <int TPB>
static int launch_block_quant_tpb(const BlockQuantParams& p, cudaStream_t s) {
  static bool configured[64] = {};
  constexpr int kSmemMax = TPB >= 1024 ? 98304 : 49152;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(block_quant_kernel<TPB>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax) != cudaSuccess)
      return fail(QLIN_ERR_LAUNCH, "cudaFuncSetAttribute failed for qlin_block_quant");
    configured[dev] = true;
  }
  // resident blocks per SM by registers (64 per thread): 1024 threads
  const int per_sm = TPB >= 1024 ? 2 : (TPB >= 512 ? 2 : 2 * (1024 / TPB));
  int grid = sm_count() * per_sm;
  if (grid > p.rows) grid = p.rows;
  if (p.max_ctas > 0) {  // the cap counts blocks of 256 threads
    int cap = TPB >= 256 ? p.max_ctas : p.max_ctas * (256 / TPB);
    if (cap < 1) cap = 1;
    if (grid > cap) grid = cap;
  }
  const int smem = p.nout * p.cols * 4;
  const bool in_smem = smem > 0 && smem <= kSmemMax && p.rows >= 4 * grid;
  block_quant_kernel<TPB><<<grid, TPB, in_smem ? smem : 0, s>>>(p, in_smem ? 1 : 0);
  QLIN_CHECK_LAUNCH("qlin_block_quant");
  return QLIN_OK;
}

static int launch_block_quant(const BlockQuantParams& p, int nchunks, cudaStream_t s) {
  if (nchunks <= 32) return launch_block_quant_tpb<32>(p, s);
  if (nchunks <= 64) return launch_block_quant_tpb<64>(p, s);
  if (nchunks <= 128) return launch_block_quant_tpb<128>(p, s);
  if (nchunks <= 256) return launch_block_quant_tpb<256>(p, s);
  if (nchunks <= 512) return launch_block_quant_tpb<512>(p, s);
  return launch_block_quant_tpb<1024>(p, s);
}

}  // namespace qlin

using namespace qlin;

extern "C" int qlin_block_quant(const qlin_block_quant_args* a, void* stream) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_block_quant: args is NULL");
  if (a->x == nullptr) return fail(QLIN_ERR_NULL, "qlin_block_quant: x is NULL");
  if (a->rows < 0 || a->cols < 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_block_quant: negative dimension");
  if (a->rows == 0 || a->cols == 0) return QLIN_OK;
  if (a->cols % 16 != 0 || a->cols > 16384) return fail(QLIN_ERR_BAD_SHAPE, "qlin_block_quant: cols must be a multiple of 16, at most 16384");
  if (a->prologue < QLIN_BLOCK_PLAIN || a->prologue > QLIN_BLOCK_SILU_MUL) return fail(QLIN_ERR_UNSUPPORTED, "qlin_block_quant: unknown prologue");
  if (a->mode < QLIN_BLOCK_DYN || a->mode > QLIN_BLOCK_SCALE_ONLY) return fail(QLIN_ERR_UNSUPPORTED, "qlin_block_quant: unknown mode");
  if (a->nout < 0 || a->nout > 3) return fail(QLIN_ERR_BAD_SHAPE, "qlin_block_quant: between 0 and 3 outputs");
  if (a->prologue == QLIN_BLOCK_NORM && a->norm_w == nullptr) return fail(QLIN_ERR_NULL, "qlin_block_quant: norm_w is NULL");
  if (a->prologue == QLIN_BLOCK_SILU_MUL && a->r == nullptr) return fail(QLIN_ERR_NULL, "qlin_block_quant: the second factor is NULL");
  if (a->mode == QLIN_BLOCK_GIVEN_SCALE && (a->scale_in == nullptr || a->nout != 1))
    return fail(QLIN_ERR_NULL, "qlin_block_quant: GIVEN_SCALE takes scale_in and exactly one output");
  if (a->qmax_levels < 1 || a->qmax_levels > 127) return fail(QLIN_ERR_UNSUPPORTED, "qlin_block_quant: qmax_levels must be in [1, 127]");
  BlockQuantParams p;
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.r = static_cast<const __nv_bfloat16*>(a->r);
  p.x_out = static_cast<__nv_bfloat16*>(a->x_out);
  p.h_out = static_cast<__nv_bfloat16*>(a->h_out);
  p.norm_w = static_cast<const __nv_bfloat16*>(a->norm_w);
  bool ok = aligned16(p.x) && aligned16(p.r) && aligned16(p.x_out) && aligned16(p.h_out) && aligned16(p.norm_w) && a->ldx % 8 == 0 &&
            a->ldr % 8 == 0 && a->ldxo % 8 == 0 && a->ldh % 8 == 0;
  for (int o = 0; o < 3; ++o) {
    const bool used = o < a->nout;
    p.mul[o] = used ? a->smooth_rcp[o] : nullptr;
    p.codes[o] = used ? static_cast<uint8_t*>(a->codes[o]) : nullptr;
    p.scale_out[o] = used ? a->scale_out[o] : nullptr;
    p.ldq[o] = a->ldq[o];
    p.codes_off[o] = a->codes_off[o];
    p.scale_off[o] = a->scale_off[o];
    if (used && a->ndst > 0) {
      ok = ok && aligned16(p.mul[o]) && a->ldq[o] % 16 == 0 && a->codes_off[o] % 16 == 0 && a->scale_off[o] % 4 == 0;
    } else if (used) {
      if (a->mode != QLIN_BLOCK_SCALE_ONLY && p.codes[o] == nullptr) return fail(QLIN_ERR_NULL, "qlin_block_quant: codes[%d] is NULL", o);
      if (a->mode == QLIN_BLOCK_SCALE_ONLY && p.scale_out[o] == nullptr) return fail(QLIN_ERR_NULL, "qlin_block_quant: scale_out[%d] is NULL", o);
      ok = ok && aligned16(p.codes[o]) && aligned16(p.mul[o]) && (p.codes[o] == nullptr || a->ldq[o] % 16 == 0);
    }
  }
  if (a->ndst < 0 || a->ndst > 8) return fail(QLIN_ERR_BAD_SHAPE, "qlin_block_quant: at most 8 destinations");
  if (a->ndst > 0 && a->mode == QLIN_BLOCK_GIVEN_SCALE)
    return fail(QLIN_ERR_UNSUPPORTED, "qlin_block_quant: replicated outputs take the dynamic or the scale-only mode");
  if (a->scale_in_parts < 0 || a->scale_in_parts > 8) return fail(QLIN_ERR_BAD_SHAPE, "qlin_block_quant: scale_in_parts must be in [0, 8]");
  for (int d = 0; d < 8; ++d) {
    p.dst_base[d] = d < a->ndst ? static_cast<uint8_t*>(a->dst_base[d]) : nullptr;
    if (d < a->ndst && (p.dst_base[d] == nullptr || !aligned16(p.dst_base[d]))) return fail(QLIN_ERR_NULL, "qlin_block_quant: dst_base[%d] is NULL or unaligned", d);
  }
  p.ndst = a->ndst;
  p.dst_row0 = a->dst_row0;
  p.max_ctas = a->max_ctas;
  p.r_multimem = a->r_multimem != 0;
  p.dst_multimem = a->dst_multimem != 0;
  if (p.dst_multimem && a->ndst != 1 && a->ndst != 2)
    return fail(QLIN_ERR_BAD_SHAPE, "qlin_block_quant: dst_multimem takes the multicast address and, optionally, this GPU's own buffer");
  if (p.r_multimem && (a->prologue != QLIN_BLOCK_NORM || a->r == nullptr))
    return fail(QLIN_ERR_UNSUPPORTED, "qlin_block_quant: r_multimem is the addend of the NORM prologue");
  if (a->r_parts < 0 || a->r_parts > 8 || (a->r_parts > 1 && a->r_part_stride % 8 != 0))
    return fail(QLIN_ERR_BAD_SHAPE, "qlin_block_quant: r_parts must be in [0, 8] with a part stride that is a multiple of 8 elements");
  p.r_parts = a->r_parts;
  p.r_part_stride = a->r_part_stride;
  if (!ok) return fail(QLIN_ERR_BAD_ALIGN, "qlin_block_quant: pointers must be 16-byte aligned and leading dimensions multiples of 16 bytes");
  p.scale_in = a->scale_in;
  p.scale_in_parts = a->scale_in_parts;
  p.scale_in_stride = a->scale_in_stride;
  p.ldx = a->ldx;
  p.ldr = a->ldr;
  p.ldxo = a->ldxo;
  p.ldh = a->ldh;
  p.rows = a->rows;
  p.cols = a->cols;
  p.nout = a->nout;
  p.prologue = a->prologue;
  p.mode = a->mode;
  p.levels = a->qmax_levels;
  p.norm_eps = a->norm_eps;
  p.dyn_eps = a->dyn_eps;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nchunks = p.cols / 16;
  // One block per row at a time, one 16-element slice per thread: the block size is the smallest power of two that
  // covers the row (a shard's rows can be a few hundred elements long; idle lanes still cost issue slots).
  return launch_block_quant(p, nchunks, s);
}


extern "C" int qlin_rope(const qlin_rope_args* a, void* stream) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_rope: args is NULL");
  if (a->x == nullptr || a->cos == nullptr || a->sin == nullptr) return fail(QLIN_ERR_NULL, "qlin_rope: x, cos or sin is NULL");
  if (a->tokens < 0 || a->heads < 0 || a->seq_len < 1) return fail(QLIN_ERR_BAD_SHAPE, "qlin_rope: bad dimensions");
  if (a->head_dim < 16 || a->head_dim % 16 != 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_rope: head_dim must be a multiple of 16");
  if (a->tokens == 0 || a->heads == 0) return QLIN_OK;
  if (!aligned16(a->x) || !aligned16(a->cos) || !aligned16(a->sin) || a->ld_token % 8 != 0)
    return fail(QLIN_ERR_BAD_ALIGN, "qlin_rope: pointers must be 16-byte aligned and the token pitch a multiple of 8 elements");
  RopeParams p;
  p.x = static_cast<__nv_bfloat16*>(a->x);
  p.cos = a->cos;
  p.sin = a->sin;
  p.ld_token = a->ld_token;
  p.tokens = a->tokens;
  p.heads = a->heads;
  p.head_dim = a->head_dim;
  p.seq_len = a->seq_len;
  const int64_t total = static_cast<int64_t>(p.tokens) * p.heads * (p.head_dim / 16);
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  rope_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  QLIN_CHECK_LAUNCH("qlin_rope");
  return QLIN_OK;
}
