// qlin_act_quant and qlin_weight_fq_perch: single-pass, row-per-block quantise kernels.
//
// A block owns one row at a time (grid-stride over rows).  Each thread keeps its 16-element slices
// of the row in registers between the statistics pass (absmax, or mean|w| and mean w^2) and the
// quantise pass, so a row is read from HBM once and written once:
//   activation quantise : read s*cols (+4*cols smooth), write cols codes + 4 bytes scale
//   weight fake-quantise: read s*cols, write s*cols (and / or cols codes) + 4 bytes clip
// Rows longer than the register budget fall back to re-reading the row (from L2) in the second
// pass; rows whose length or alignment rules out 16-byte vectors take a scalar path with the same
// arithmetic.
//
// Arithmetic follows the reference's eager tensor expressions operation by operation: every
// division, multiplication and addition is a separately rounded fp32 operation, optionally rounded
// again to the tensor dtype ("native chain") where the reference computes in bf16 / fp16.
#include <type_traits>

#include <cuda_fp8.h>

#include "qlin_internal.h"
#include "qlin_ptx.cuh"
#include "qlin_rows.cuh"

namespace qlin {

struct QuantParams {
  const void* x;
  const float* smooth;
  const float* smooth_rcp;
  const float* scale_in;
  uint8_t* codes;
  float* scale_out;
  void* dq_out;
  int32_t* status;
  int64_t ldx, ldq, lddq;
  int32_t rows, cols;
  int32_t smooth_exact;  // smoothing scales are exactly representable in the dtype of x
  int32_t mode, native, native_smooth, smooth_mul, clamp_codes, levels, dl8_flush, scale_in_stride;
  float scale0, zp0, lo, hi, shift, add2, dyn_eps;
  int32_t f8_e5m2;
};

template <typename XT>
__device__ __forceinline__ float smooth_apply(const QuantParams& p, float x, float sm, float rsm) {
  const float v = p.smooth_mul ? __fmul_rn(x, sm) : div_exact(x, sm, rsm);
  return rnd_if<XT>(v, p.native_smooth);
}

// Row scale from the row's absmax.
template <typename XT>
__device__ __forceinline__ float dyn_scale(const QuantParams& p, float amax) {
  const float eps = rnd_if<XT>(p.dyn_eps, p.native);
  if (p.mode == QLIN_Q_F8_FAKE_SCALED) {
    // max_to_scale: 448 / clamp(amax, eps) is reciprocal * 448 (scalar numerator), then the fp16 cap
    const float r = rnd_if<XT>(__fdiv_rn(1.0f, fmaxf(amax, eps)), p.native);
    float sc = rnd_if<XT>(__fmul_rn(r, 448.0f), p.native);
    if (std::is_same<XT, __half>::value && p.native) sc = fminf(sc, 65504.0f);
    return sc;
  }
  if (p.mode == QLIN_Q_F8_DYN) {
    const float a = rnd_if<XT>(__fdiv_rn(amax, 448.0f), p.native);
    return fmaxf(a, eps);
  }
  const float a = fmaxf(amax, eps);
  return rnd_if<XT>(__fdiv_rn(a, static_cast<float>(p.levels)), p.native);
}

// torch's float -> float8_e4m3fn conversion: round to nearest even, NaN above 464.
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  if (!(fabsf(v) <= 464.0f)) return static_cast<uint8_t>(0x7F | (signbit(v) ? 0x80 : 0));
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
// torch's float -> float8_e5m2 conversion: round to nearest even, infinity from 61440 upwards.
__device__ __forceinline__ uint8_t to_e5m2(float v) {
  if (v != v) return 0x7F;
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_NOSAT, __NV_E5M2));
}
__device__ __forceinline__ float from_e5m2(uint8_t c) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(c), __NV_E5M2);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
__device__ __forceinline__ float from_e4m3(uint8_t c) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(c), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// One element: value after smoothing -> code byte, and the fake-quantised value for dq_out.
template <typename XT>
__device__ __forceinline__ uint8_t quant_one(const QuantParams& p, float v, float s, float rs, float& dq) {
  const bool nat = p.native;
  switch (p.mode) {
    case QLIN_Q_I8_DYN:
    case QLIN_Q_I8_GIVEN_SCALE: {
      const float r = rintf(rnd_if<XT>(div_exact(v, s, rs), nat));
      dq = rnd_if<XT>(__fmul_rn(r, s), nat);
      float c = r;
      if (p.mode == QLIN_Q_I8_GIVEN_SCALE) c = rnd_if<XT>(__fadd_rn(c, p.zp0), nat);
      int q = static_cast<int>(c);
      if (p.clamp_codes) q = max(-p.levels, min(p.levels, q));
      return static_cast<uint8_t>(q & 0xFF);
    }
    case QLIN_Q_I8_STATIC: {
      float t = rnd_if<XT>(div_exact(v, s, rs), nat);
      t = rnd_if<XT>(__fadd_rn(t, p.zp0), nat);
      t = rnd_if<XT>(__fsub_rn(t, p.shift), nat);
      t = rnd_if<XT>(__fadd_rn(t, p.add2), nat);
      const float r = fminf(fmaxf(rintf(t), -128.0f), 127.0f);
      dq = r;
      return static_cast<uint8_t>(static_cast<int>(r) & 0xFF);
    }
    case QLIN_Q_I8_STATIC_CLAMP_FIRST: {
      float t = fminf(fmaxf(v, p.lo), p.hi);
      t = rnd_if<XT>(div_exact(t, s, rs), nat);
      t = rnd_if<XT>(__fsub_rn(t, p.zp0), nat);
      const float r = rnd_if<XT>(__fsub_rn(rintf(t), p.shift), nat);
      dq = r;
      return static_cast<uint8_t>(static_cast<int>(r) & 0xFF);
    }
    case QLIN_Q_I8_STATIC_ROUND_FIRST: {  // clamp(rint(v / s + zp), lo, hi) - shift
      float t = rnd_if<XT>(div_exact(v, s, rs), nat);
      t = rnd_if<XT>(__fadd_rn(t, p.zp0), nat);
      const float r = fminf(fmaxf(rintf(t), p.lo), p.hi) - p.shift;
      dq = r;
      return static_cast<uint8_t>(static_cast<int>(r) & 0xFF);
    }
    case QLIN_Q_I8_AFFINE_RCP: {  // torch.quantize_per_tensor: clamp(nearbyint(v * (1 / s)) + zp, -128, 127)
      const float r = fminf(fmaxf(nearbyintf(__fmul_rn(v, __fdiv_rn(1.0f, s))) + p.zp0, -128.0f), 127.0f);
      dq = r;
      return static_cast<uint8_t>(static_cast<int>(r) & 0xFF);
    }
    case QLIN_Q_F8_TENSOR: {  // one scale for the whole tensor, e4m3 or e5m2 codes
      const float t = rnd_if<XT>(div_exact(v, s, rs), nat);
      uint8_t c = p.f8_e5m2 ? to_e5m2(t) : to_e4m3(t);
      float f = p.f8_e5m2 ? from_e5m2(c) : from_e4m3(c);
      if (p.dl8_flush && fabsf(f) < 0.0087890625f) {
        c = 0;
        f = 0.0f;
      }
      dq = f;
      return c;
    }
    case QLIN_Q_F8_FAKE_SCALED: {  // s multiplies: x * s, saturate, cast to e4m3 and back, / s
      float t = rnd_if<XT>(__fmul_rn(v, s), nat);
      const bool is_nan = t != t;  // torch.clamp keeps NaN, fminf / fmaxf would drop it
      t = fminf(fmaxf(t, -448.0f), 448.0f);
      if (is_nan) t = __int_as_float(0x7FC00000);
      const uint8_t c = to_e4m3(t);
      dq = rnd_if<XT>(__fdiv_rn(from_e4m3(c), s), nat);
      return c;
    }
    default: {  // QLIN_Q_F8_DYN
      const float t = rnd_if<XT>(div_exact(v, s, rs), nat);
      uint8_t c = to_e4m3(t);
      float f = from_e4m3(c);
      if (p.dl8_flush && fabsf(f) < 0.0087890625f) {
        c = 0;
        f = 0.0f;
      }
      dq = f;
      return c;
    }
  }
}

__device__ __forceinline__ bool is_dynamic(int mode) {
  return mode == QLIN_Q_I8_DYN || mode == QLIN_Q_F8_DYN || mode == QLIN_Q_F8_FAKE_SCALED;
}

template <typename XT>
__device__ __forceinline__ float row_scale_of(const QuantParams& p, int row, float amax) {
  if (is_dynamic(p.mode)) return dyn_scale<XT>(p, amax);
  if (p.mode == QLIN_Q_I8_GIVEN_SCALE) return p.scale_in[static_cast<int64_t>(row) * p.scale_in_stride];
  if (p.mode == QLIN_Q_F8_TENSOR) {
    const float a = rnd_if<XT>(__fdiv_rn(p.scale_in[0], p.scale0), p.native);
    return fmaxf(a, rnd_if<XT>(p.dyn_eps, p.native));
  }
  return p.scale0;
}

// Vector path: cols % 16 == 0 and every row start 16-byte aligned.  MAXC = register-resident
// 16-element slices per thread; MAXC == 0 re-reads the row in the second pass.
template <typename XT, int MAXC>
__global__ void __launch_bounds__(1024) act_quant_vec_kernel(const QuantParams p) {
  __shared__ float red[2][32];
  const int nchunks = p.cols >> 4;
  const bool has_smooth = p.smooth != nullptr;
  constexpr int NREG = MAXC > 0 ? MAXC : 1;
  int iter = 0;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x, ++iter) {
    const XT* xr = reinterpret_cast<const XT*>(p.x) + static_cast<int64_t>(row) * p.ldx;
    float v[NREG][16];
    float amax = 0.0f;
    if (MAXC > 0) {
#pragma unroll
      for (int c = 0; c < NREG; ++c) {
        const int ch = threadIdx.x + c * blockDim.x;
        if (ch < nchunks) {
          load16(xr + ch * 16, v[c]);
          if (has_smooth) {
            float sm[16], rsm[16];
            load16(p.smooth + ch * 16, sm);
            if (!p.smooth_mul) load16(p.smooth_rcp + ch * 16, rsm);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[c][i] = smooth_apply<XT>(p, v[c][i], sm[i], rsm[i]);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[c][i]));
        }
      }
    } else if (is_dynamic(p.mode)) {
      for (int ch = threadIdx.x; ch < nchunks; ch += blockDim.x) {
        load16(xr + ch * 16, v[0]);
        if (has_smooth) {
          float sm[16], rsm[16];
          load16(p.smooth + ch * 16, sm);
          if (!p.smooth_mul) load16(p.smooth_rcp + ch * 16, rsm);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[0][i] = smooth_apply<XT>(p, v[0][i], sm[i], rsm[i]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[0][i]));
      }
    }
    if (is_dynamic(p.mode)) amax = block_reduce<OpMax>(amax, red[iter & 1], 0.0f);
    const float s = row_scale_of<XT>(p, row, amax);
    const float rs = rcp_for_div(s);
    if (threadIdx.x == 0 && p.scale_out != nullptr) p.scale_out[row] = s;

    auto emit = [&](int ch, const float (&val)[16]) {
      float dq[16];
      uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t c = quant_one<XT>(p, val[i], s, rs, dq[i]);
        w[i >> 2] |= c << (8 * (i & 3));
      }
      if (p.codes != nullptr)
        *reinterpret_cast<uint4*>(p.codes + static_cast<int64_t>(row) * p.ldq + ch * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      if (p.dq_out != nullptr) store16(reinterpret_cast<XT*>(p.dq_out) + static_cast<int64_t>(row) * p.lddq + ch * 16, dq);
    };
    if (MAXC > 0) {
#pragma unroll
      for (int c = 0; c < NREG; ++c) {
        const int ch = threadIdx.x + c * blockDim.x;
        if (ch < nchunks) emit(ch, v[c]);
      }
    } else {
      for (int ch = threadIdx.x; ch < nchunks; ch += blockDim.x) {
        load16(xr + ch * 16, v[0]);
        if (has_smooth) {
          float sm[16], rsm[16];
          load16(p.smooth + ch * 16, sm);
          if (!p.smooth_mul) load16(p.smooth_rcp + ch * 16, rsm);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[0][i] = smooth_apply<XT>(p, v[0][i], sm[i], rsm[i]);
        }
        emit(ch, v[0]);
      }
    }
  }
}


// ------------------------------------------------------------------------------------------------
// Specialised fast path of the dynamic quantisers (the per-token int8 / e4m3 quantise of the deploy
// Linears).  Two things make it HBM-bound instead of issue-bound:
//   * mode, rounding chain and outputs are template parameters, so the per-element instruction
//     stream is only: widen, three fused operations per exact division, round to the tensor dtype,
//     |.| / max; then three fused operations, round, rint, convert, pack;
//   * rows stream into a ring of shared-memory slots with 1-D bulk copies (cp.async.bulk, completion
//     counted on an mbarrier per slot) several rows ahead of the one being quantised.  A thread
//     copies its 16-element slices from the slot into registers, and the barrier of the block-wide
//     reduction doubles as the "slot is free" signal: right after it thread 0 refills the slot.
// Exactness of the divisions: x / s is formed from r = RN(1/s) as q = x r, rem = fma(-s, q, x),
// q' = fma(rem, r, q), which is the correctly rounded quotient unless s has an all-ones
// significand or an intermediate leaves the normal range.  Columns whose reciprocal the caller
// marked NaN, rows whose scale is such a value and rows whose absmax reaches 1e15 are recomputed
// with the ordinary IEEE division; quotients below the normal range only ever produce the code 0.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float fast_div(float x, float s, float r) {
  const float q = __fmul_rn(x, r);
  return __fmaf_rn(__fmaf_rn(-s, q, x), r, q);
}

template <typename XT, int MODE, bool NATIVE, bool DQ, int MAXC, int TPB>
__global__ void __launch_bounds__(TPB) act_quant_fast_kernel(const QuantParams p, int stages, int row_bytes) {
  // Blocks of at most 256 threads have the register budget to keep their slice of the smoothing
  // vector (and its reciprocal) in registers for all rows; larger blocks re-read it through L1.
  constexpr bool SMREG = TPB <= 256 && MAXC == 1;
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ uint64_t full[8];
  __shared__ float red[2][32];
  __shared__ int abort_flag;
  constexpr bool F8 = MODE == QLIN_Q_F8_DYN;
  constexpr bool DYN = MODE != QLIN_Q_I8_GIVEN_SCALE;
  const int nchunks = p.cols >> 4;
  const bool has_smooth = p.smooth != nullptr;
  const bool smooth_div = has_smooth && !p.smooth_mul;
  const int my_rows = (p.rows - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const uint8_t* xbase = reinterpret_cast<const uint8_t*>(p.x);
  const int64_t pitch = p.ldx * static_cast<int64_t>(sizeof(XT));

  auto issue = [&](int i) {  // thread 0 only
    const int slot = i % stages;
    const int64_t row = static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(i) * gridDim.x;
    mbar_arrive_expect_tx(&full[slot], static_cast<uint32_t>(row_bytes));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(ring + static_cast<size_t>(slot) * row_bytes)),
                 "l"(reinterpret_cast<uint64_t>(xbase + row * pitch)), "r"(row_bytes), "r"(smem_u32(&full[slot]))
                 : "memory");
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int pre = my_rows < stages ? my_rows : stages;
    for (int i = 0; i < pre; ++i) issue(i);
  }
  // A thread owns the same column slices in every row: decide once whether any of its columns
  // needs the ordinary division.
  bool slow_cols = false;
  float sm_reg[16], rsm_reg[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) sm_reg[j] = rsm_reg[j] = 1.0f;
  if (has_smooth) {
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunks) {
        float rsm[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) rsm[j] = 1.0f;
        if (smooth_div) load16(p.smooth_rcp + ch * 16, rsm);
#pragma unroll
        for (int j = 0; j < 16; ++j) slow_cols = slow_cols || (rsm[j] != rsm[j]);
        if (SMREG) {
          load16(p.smooth + ch * 16, sm_reg);
#pragma unroll
          for (int j = 0; j < 16; ++j) rsm_reg[j] = rsm[j];
        }
      }
    }
  }
  const float eps = NATIVE ? Elem<XT>::rnd(p.dyn_eps) : p.dyn_eps;

  for (int i = 0; i < my_rows; ++i) {
    const int slot = i % stages;
    const int row = static_cast<int>(blockIdx.x) + i * static_cast<int>(gridDim.x);
    const bool ok = mbar_wait(&full[slot], static_cast<uint32_t>((i / stages) & 1), &abort_flag);
    const XT* xr = reinterpret_cast<const XT*>(ring + static_cast<size_t>(slot) * row_bytes);
    float v[MAXC][16];
    float amax = 0.0f;
    auto smooth_chunk = [&](int c, int ch, bool exact) {
      load16(xr + ch * 16, v[c]);
      if (has_smooth) {
        float sm[16], rsm[16];
        if (SMREG) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            sm[j] = sm_reg[j];
            rsm[j] = rsm_reg[j];
          }
        } else {
          load16(p.smooth + ch * 16, sm);
          if (smooth_div) load16(p.smooth_rcp + ch * 16, rsm);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float t;
          if (!smooth_div) {
            t = __fmul_rn(v[c][j], sm[j]);
          } else if (exact) {
            t = __fdiv_rn(v[c][j], sm[j]);
          } else {
            t = fast_div(v[c][j], sm[j], rsm[j]);
            if (F8) t = copysignf(t, __fmul_rn(v[c][j], sm[j]));
          }
          v[c][j] = NATIVE ? fast_rnd<XT>(t) : t;
        }
      }
    };
    if (ok) {
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        const int ch = threadIdx.x + c * blockDim.x;
        if (ch < nchunks) {
          if (slow_cols) {
            smooth_chunk(c, ch, true);
          } else {
            smooth_chunk(c, ch, false);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[c][j]));
        }
      }
    }
    bool any_bad;
    amax = block_reduce_flag<OpMax>(amax, red[i & 1], 0.0f, !ok, any_bad);
    if (any_bad) {
      if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, static_cast<int32_t>(QLIN_ERR_TIMEOUT));
      break;
    }
    if (smooth_div && !(amax < 1e15f)) {
      // some quotient may have left the range in which the fused division is exact: redo the row
      float a2 = 0.0f;
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        const int ch = threadIdx.x + c * blockDim.x;
        if (ch < nchunks) {
          smooth_chunk(c, ch, true);
#pragma unroll
          for (int j = 0; j < 16; ++j) a2 = fmaxf(a2, fabsf(v[c][j]));
        }
      }
      amax = block_reduce<OpMax>(a2, red[i & 1], 0.0f);
      __syncthreads();
    }
    if (threadIdx.x == 0 && i + stages < my_rows) issue(i + stages);

    float s;
    if (MODE == QLIN_Q_F8_DYN) {
      const float a = __fdiv_rn(amax, 448.0f);
      s = fmaxf(NATIVE ? Elem<XT>::rnd(a) : a, eps);
    } else if (MODE == QLIN_Q_I8_DYN) {
      const float a = __fdiv_rn(fmaxf(amax, eps), static_cast<float>(p.levels));
      s = NATIVE ? Elem<XT>::rnd(a) : a;
    } else {
      s = p.scale_in[static_cast<int64_t>(row) * p.scale_in_stride];
    }
    if (threadIdx.x == 0 && p.scale_out != nullptr) p.scale_out[row] = s;
    const float rs = rcp_for_div(s);
    const bool slow_row = rs != rs;

    auto emit_chunk = [&](int c, int ch, bool exact) {
      uint32_t w[4];
      float dq[16];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t b[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int j = 4 * g + k;
          float t = exact ? __fdiv_rn(v[c][j], s) : fast_div(v[c][j], s, rs);
          if (F8 && !exact) t = copysignf(t, v[c][j]);
          if (NATIVE) t = fast_rnd<XT>(t);
          if (F8) {
            uint8_t code = to_e4m3(t);
            if (p.dl8_flush && fabsf(from_e4m3(code)) < 0.0087890625f) code = 0;
            b[k] = code;
          } else {
            // dynamic scales keep |t| <= ~128, far inside the range of the additive rint
            int q;
            const float r = DYN ? fast_rint(t, q) : rintf(t);
            if (DQ) {
              const float d = __fmul_rn(r, s);
              dq[j] = NATIVE ? fast_rnd<XT>(d) : d;
            }
            if (!DYN) {
              float cf = __fadd_rn(r, p.zp0);
              if (NATIVE) cf = Elem<XT>::rnd(cf);
              q = static_cast<int>(cf);
            }
            if (p.clamp_codes) q = max(-p.levels, min(p.levels, q));
            b[k] = static_cast<uint32_t>(q);
          }
        }
        w[g] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
      }
      if (p.codes != nullptr)
        *reinterpret_cast<uint4*>(p.codes + static_cast<int64_t>(row) * p.ldq + ch * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      if (DQ) store16(reinterpret_cast<XT*>(p.dq_out) + static_cast<int64_t>(row) * p.lddq + ch * 16, dq);
    };
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunks) {
        if (slow_row) {
          emit_chunk(c, ch, true);
        } else {
          emit_chunk(c, ch, false);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// bf16 rows, bf16 rounding chain, bf16-valued smoothing scales: the deploy Linear of a bf16 model.
//
// Here the reference computes RN_bf16(RN_f32(x / s)) with x and s both bf16 values, and the same
// again for the division by the (bf16) row scale.  Two facts collapse that to one multiplication:
//   * a quotient of two 8-bit significands is never a bf16 rounding midpoint (an odd 9-bit value
//     times any significand needs at least 9 bits) and stays at least 2^-18 (relative) away from
//     one, so rounding it to fp32 first cannot change the bf16 result;
//   * x * RN_f32(1 / s) is within 2^-23 (relative) of x / s, far inside that margin.
// So RN_bf16(x * r) is bit-identical to the reference's value.  Values stay packed as bf16 pairs in
// registers; conversions are done two at a time.  Same ring pipeline as above.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int MODE, int MAXC, int TPB>
__global__ void __launch_bounds__(TPB) act_quant_bf16_kernel(const QuantParams p, int stages, int row_bytes) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ uint64_t full[8];
  __shared__ float red[2][32];
  __shared__ int abort_flag;
  constexpr bool DYN = MODE == QLIN_Q_I8_DYN;
  constexpr bool SMREG = TPB <= 256 && MAXC == 1;
  const int nchunks = p.cols >> 4;
  const bool has_smooth = p.smooth != nullptr;
  const float* mulvec = p.smooth_mul ? p.smooth : p.smooth_rcp;  // what every element is multiplied by
  const int my_rows = (p.rows - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const uint8_t* xbase = reinterpret_cast<const uint8_t*>(p.x);
  const int64_t pitch = p.ldx * 2;

  auto issue = [&](int i) {  // thread 0 only
    const int slot = i % stages;
    const int64_t row = static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(i) * gridDim.x;
    mbar_arrive_expect_tx(&full[slot], static_cast<uint32_t>(row_bytes));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(ring + static_cast<size_t>(slot) * row_bytes)),
                 "l"(reinterpret_cast<uint64_t>(xbase + row * pitch)), "r"(row_bytes), "r"(smem_u32(&full[slot]))
                 : "memory");
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int pre = my_rows < stages ? my_rows : stages;
    for (int i = 0; i < pre; ++i) issue(i);
  }
  float mreg[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) mreg[j] = 1.0f;
  if (SMREG && has_smooth && static_cast<int>(threadIdx.x) < nchunks) load16(mulvec + threadIdx.x * 16, mreg);
  const float eps = Elem<__nv_bfloat16>::rnd(p.dyn_eps);

  for (int i = 0; i < my_rows; ++i) {
    const int slot = i % stages;
    const int row = static_cast<int>(blockIdx.x) + i * static_cast<int>(gridDim.x);
    const bool ok = mbar_wait(&full[slot], static_cast<uint32_t>((i / stages) & 1), &abort_flag);
    const uint4* xr = reinterpret_cast<const uint4*>(ring + static_cast<size_t>(slot) * row_bytes);
    uint32_t vp[MAXC][8];
    __nv_bfloat162 amax2 = __floats2bfloat162_rn(0.0f, 0.0f);
    if (ok) {
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        const int ch = threadIdx.x + c * blockDim.x;
        if (ch < nchunks) {
          const uint4 a = xr[ch * 2], b = xr[ch * 2 + 1];
          const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
          if (has_smooth) {
            float m[16];
            if (SMREG) {
#pragma unroll
              for (int j = 0; j < 16; ++j) m[j] = mreg[j];
            } else {
              load16(mulvec + ch * 16, m);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float lo = __fmul_rn(__uint_as_float(w[j] << 16), m[2 * j]);
              const float hi = __fmul_rn(__uint_as_float(w[j] & 0xFFFF0000u), m[2 * j + 1]);
              vp[c][j] = pack_bf16x2(lo, hi);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) vp[c][j] = w[j];
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            amax2 = __hmax2(amax2, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&vp[c][j])));
        }
      }
    }
    float amax = fmaxf(__low2float(amax2), __high2float(amax2));
    bool any_bad;
    amax = block_reduce_flag<OpMax>(amax, red[i & 1], 0.0f, !ok, any_bad);
    if (any_bad) {
      if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, static_cast<int32_t>(QLIN_ERR_TIMEOUT));
      break;
    }
    if (threadIdx.x == 0 && i + stages < my_rows) issue(i + stages);
    float s;
    if (DYN) {
      s = Elem<__nv_bfloat16>::rnd(__fdiv_rn(fmaxf(amax, eps), static_cast<float>(p.levels)));
    } else {
      s = p.scale_in[static_cast<int64_t>(row) * p.scale_in_stride];
    }
    if (threadIdx.x == 0 && p.scale_out != nullptr) p.scale_out[row] = s;
    const float rs = __frcp_rn(s);
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunks) {
        uint32_t out[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          int q[4];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t w = vp[c][2 * g + h];
            const uint32_t t2 = pack_bf16x2(__fmul_rn(__uint_as_float(w << 16), rs), __fmul_rn(__uint_as_float(w & 0xFFFF0000u), rs));
            float r0, r1;
            if (DYN) {
              r0 = fast_rint(__uint_as_float(t2 << 16), q[2 * h]);
              r1 = fast_rint(__uint_as_float(t2 & 0xFFFF0000u), q[2 * h + 1]);
            } else {
              r0 = rintf(__uint_as_float(t2 << 16));
              r1 = rintf(__uint_as_float(t2 & 0xFFFF0000u));
              q[2 * h] = static_cast<int>(Elem<__nv_bfloat16>::rnd(__fadd_rn(r0, p.zp0)));
              q[2 * h + 1] = static_cast<int>(Elem<__nv_bfloat16>::rnd(__fadd_rn(r1, p.zp0)));
            }
            (void)r0;
            (void)r1;
          }
          if (p.clamp_codes) {
#pragma unroll
            for (int k = 0; k < 4; ++k) q[k] = max(-p.levels, min(p.levels, q[k]));
          }
          out[g] = __byte_perm(__byte_perm(q[0], q[1], 0x0040), __byte_perm(q[2], q[3], 0x0040), 0x5410);
        }
        *reinterpret_cast<uint4*>(p.codes + static_cast<int64_t>(row) * p.ldq + ch * 16) = make_uint4(out[0], out[1], out[2], out[3]);
      }
    }
  }
}

template <int MODE, int MAXC, int TPB>
static int launch_bf16(const QuantParams& p, int threads, cudaStream_t stream) {
  const int row_bytes = p.cols * 2;
  int stages = 32768 / row_bytes;
  stages = stages < 2 ? 2 : (stages > 8 ? 8 : stages);
  const int smem = stages * row_bytes;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(act_quant_bf16_kernel<MODE, MAXC, TPB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 98304);
    if (e != cudaSuccess) return fail(QLIN_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  int per_sm_threads = 2048 / threads;
  int per_sm_smem = (220 * 1024) / (smem + 1024);
  int per_sm = per_sm_threads < per_sm_smem ? per_sm_threads : per_sm_smem;
  if (per_sm < 1) per_sm = 1;
  int grid = sm_count() * per_sm;
  if (grid > p.rows) grid = p.rows;
  act_quant_bf16_kernel<MODE, MAXC, TPB><<<grid, threads, smem, stream>>>(p, stages, row_bytes);
  QLIN_CHECK_LAUNCH("qlin_act_quant");
  return QLIN_OK;
}

template <int MODE>
static int launch_bf16_c(const QuantParams& p, int threads, int nchunks, cudaStream_t stream) {
  if (nchunks <= threads && threads <= 256) return launch_bf16<MODE, 1, 256>(p, threads, stream);
  return nchunks <= threads ? launch_bf16<MODE, 1, 1024>(p, threads, stream) : launch_bf16<MODE, 2, 1024>(p, threads, stream);
}

template <typename XT, int MODE, bool NATIVE, bool DQ, int MAXC, int TPB>
static int launch_fast(const QuantParams& p, int threads, cudaStream_t stream) {
  const int row_bytes = p.cols * static_cast<int>(sizeof(XT));
  int stages = 32768 / row_bytes;
  stages = stages < 2 ? 2 : (stages > 8 ? 8 : stages);
  const int smem = stages * row_bytes;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(act_quant_fast_kernel<XT, MODE, NATIVE, DQ, MAXC, TPB>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 98304);
    if (e != cudaSuccess) return fail(QLIN_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  int per_sm_threads = 2048 / threads;
  int per_sm_smem = (220 * 1024) / (smem + 1024);
  int per_sm = per_sm_threads < per_sm_smem ? per_sm_threads : per_sm_smem;
  if (per_sm < 1) per_sm = 1;
  int grid = sm_count() * per_sm;
  if (grid > p.rows) grid = p.rows;
  act_quant_fast_kernel<XT, MODE, NATIVE, DQ, MAXC, TPB><<<grid, threads, smem, stream>>>(p, stages, row_bytes);
  QLIN_CHECK_LAUNCH("qlin_act_quant");
  return QLIN_OK;
}

template <typename XT, int MODE, bool NATIVE, bool DQ>
static int launch_fast_c(const QuantParams& p, int threads, int nchunks, cudaStream_t stream) {
  if (nchunks <= threads && threads <= 256) return launch_fast<XT, MODE, NATIVE, DQ, 1, 256>(p, threads, stream);
  return nchunks <= threads ? launch_fast<XT, MODE, NATIVE, DQ, 1, 1024>(p, threads, stream)
                            : launch_fast<XT, MODE, NATIVE, DQ, 2, 1024>(p, threads, stream);
}

// Dispatches to a specialised kernel when the call is one of the hot configurations; returns 1 when
// it is not (the caller then takes the general kernels).
template <typename XT>
static int try_fast(const QuantParams& p, int threads, int nchunks, cudaStream_t stream) {
  constexpr bool kIsF32 = sizeof(XT) == 4;
  // the two rounding switches move together on this path; fp32 rows have nothing to round
  const bool native = !kIsF32 && p.native;
  if (!kIsF32 && (p.native != p.native_smooth) && p.smooth != nullptr) return 1;
  const bool dq = p.dq_out != nullptr;
  if (std::is_same<XT, __nv_bfloat16>::value && native && !dq && p.codes != nullptr && (p.smooth == nullptr || p.smooth_exact)) {
    if (p.mode == QLIN_Q_I8_DYN) return launch_bf16_c<QLIN_Q_I8_DYN>(p, threads, nchunks, stream);
    if (p.mode == QLIN_Q_I8_GIVEN_SCALE) return launch_bf16_c<QLIN_Q_I8_GIVEN_SCALE>(p, threads, nchunks, stream);
  }
  if (p.mode == QLIN_Q_I8_DYN) {
    if (kIsF32 || !native)
      return dq ? launch_fast_c<XT, QLIN_Q_I8_DYN, false, true>(p, threads, nchunks, stream)
                : launch_fast_c<XT, QLIN_Q_I8_DYN, false, false>(p, threads, nchunks, stream);
    return dq ? launch_fast_c<XT, QLIN_Q_I8_DYN, !kIsF32, true>(p, threads, nchunks, stream)
              : launch_fast_c<XT, QLIN_Q_I8_DYN, !kIsF32, false>(p, threads, nchunks, stream);
  }
  if (dq) return 1;
  if (p.mode == QLIN_Q_F8_DYN) {
    if (kIsF32 || !native) return launch_fast_c<XT, QLIN_Q_F8_DYN, false, false>(p, threads, nchunks, stream);
    return launch_fast_c<XT, QLIN_Q_F8_DYN, !kIsF32, false>(p, threads, nchunks, stream);
  }
  if (p.mode == QLIN_Q_I8_GIVEN_SCALE) {
    if (kIsF32 || !native) return launch_fast_c<XT, QLIN_Q_I8_GIVEN_SCALE, false, false>(p, threads, nchunks, stream);
    return launch_fast_c<XT, QLIN_Q_I8_GIVEN_SCALE, !kIsF32, false>(p, threads, nchunks, stream);
  }
  return 1;
}

// Scalar path for any shape / alignment.
template <typename XT>
__global__ void __launch_bounds__(256) act_quant_scalar_kernel(const QuantParams p) {
  __shared__ float red[2][32];
  const bool has_smooth = p.smooth != nullptr;
  int iter = 0;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x, ++iter) {
    const XT* xr = reinterpret_cast<const XT*>(p.x) + static_cast<int64_t>(row) * p.ldx;
    float amax = 0.0f;
    if (is_dynamic(p.mode)) {
      for (int c = threadIdx.x; c < p.cols; c += blockDim.x) {
        float v = load1(xr + c);
        if (has_smooth) v = smooth_apply<XT>(p, v, p.smooth[c], p.smooth_mul ? 0.0f : p.smooth_rcp[c]);
        amax = fmaxf(amax, fabsf(v));
      }
      amax = block_reduce<OpMax>(amax, red[iter & 1], 0.0f);
    }
    const float s = row_scale_of<XT>(p, row, amax);
    const float rs = rcp_for_div(s);
    if (threadIdx.x == 0 && p.scale_out != nullptr) p.scale_out[row] = s;
    for (int c = threadIdx.x; c < p.cols; c += blockDim.x) {
      float v = load1(xr + c);
      if (has_smooth) v = smooth_apply<XT>(p, v, p.smooth[c], p.smooth_mul ? 0.0f : p.smooth_rcp[c]);
      float dq;
      const uint8_t code = quant_one<XT>(p, v, s, rs, dq);
      if (p.codes != nullptr) p.codes[static_cast<int64_t>(row) * p.ldq + c] = code;
      if (p.dq_out != nullptr) store1(reinterpret_cast<XT*>(p.dq_out) + static_cast<int64_t>(row) * p.lddq + c, dq);
    }
  }
}

template <typename XT>
static int launch_act_quant(const QuantParams& p, cudaStream_t stream) {
  const int es = static_cast<int>(sizeof(XT));
  bool vec = (p.cols % 16 == 0) && aligned16(p.x) && ((p.ldx * es) % 16 == 0);
  if (p.smooth != nullptr) vec = vec && aligned16(p.smooth) && (p.smooth_mul || aligned16(p.smooth_rcp));
  if (p.codes != nullptr) vec = vec && aligned16(p.codes) && (p.ldq % 16 == 0);
  if (p.dq_out != nullptr) vec = vec && aligned16(p.dq_out) && ((p.lddq * es) % 16 == 0);
  const int max_blocks = sm_count() * 16;
  if (!vec) {
    const int grid = p.rows < max_blocks ? p.rows : max_blocks;
    act_quant_scalar_kernel<XT><<<grid, 256, 0, stream>>>(p);
    QLIN_CHECK_LAUNCH("qlin_act_quant");
    return QLIN_OK;
  }
  const int nchunks = p.cols / 16;
  int threads = ((nchunks + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  const int blocks_per_sm = 2048 / threads;
  int grid = sm_count() * (blocks_per_sm > 0 ? blocks_per_sm : 1);
  if (grid > p.rows) grid = p.rows;
  const int row_bytes = p.cols * es;
  if (row_bytes <= 49152 && nchunks <= 2 * threads) {
    const int rc = try_fast<XT>(p, threads, nchunks, stream);
    if (rc <= 0) return rc;
  }
  if (nchunks <= threads) {
    act_quant_vec_kernel<XT, 1><<<grid, threads, 0, stream>>>(p);
  } else if (nchunks <= 2 * threads) {
    act_quant_vec_kernel<XT, 2><<<grid, threads, 0, stream>>>(p);
  } else {
    act_quant_vec_kernel<XT, 0><<<grid, threads, 0, stream>>>(p);
  }
  QLIN_CHECK_LAUNCH("qlin_act_quant");
  return QLIN_OK;
}

// ------------------------------------------------------------------------------------------------
// Per-output-channel weight fake quantisation (SAWB+ / max), statistics and quantise in one pass.
// ------------------------------------------------------------------------------------------------
struct WfqParams {
  const void* w;
  const float* smooth;
  void* dq_out;
  int8_t* codes;
  float* clip_io;
  int64_t ldw, ldo, ldq;
  int32_t rows, cols, num_bits, mode, native_mul, clip_dtype;
  float c0, c1;
};

template <typename XT>
__device__ __forceinline__ float wfq_clip(const WfqParams& p, float sum_abs, float sum_sq, float amax, int row) {
  if (p.mode == QLIN_W_GIVEN) return p.clip_io[row];
  if (p.mode == QLIN_W_MAX) return amax;
  // clip = c1 * mean|w| + c0 * sqrt(mean w^2), every step rounded to the weight dtype.
  const float n = static_cast<float>(p.cols);
  const float mu = Elem<XT>::rnd(__fdiv_rn(sum_abs, n));
  const float sd = Elem<XT>::rnd(__fsqrt_rn(Elem<XT>::rnd(__fdiv_rn(sum_sq, n))));
  const float a = Elem<XT>::rnd(__fmul_rn(p.c1, mu));
  const float b = Elem<XT>::rnd(__fmul_rn(p.c0, sd));
  return Elem<XT>::rnd(__fadd_rn(a, b));
}

// scale = clip * 2 / nspace, each step rounded to the dtype of the clip tensor (the weight dtype unless
// the caller names another one).
template <typename XT>
__device__ __forceinline__ float wfq_scale(const WfqParams& p, float clip, float nspace) {
  switch (p.clip_dtype) {
    case QLIN_DT_F32:
      return __fdiv_rn(__fmul_rn(clip, 2.0f), nspace);
    case QLIN_DT_F16:
      return Elem<__half>::rnd(__fdiv_rn(Elem<__half>::rnd(__fmul_rn(clip, 2.0f)), nspace));
    case QLIN_DT_BF16:
      return Elem<__nv_bfloat16>::rnd(__fdiv_rn(Elem<__nv_bfloat16>::rnd(__fmul_rn(clip, 2.0f)), nspace));
    default:
      return Elem<XT>::rnd(__fdiv_rn(Elem<XT>::rnd(__fmul_rn(clip, 2.0f)), nspace));
  }
}

// torch.fake_quantize_per_channel_affine with zero_point 0:
//   q = clamp(nearbyint(w * (1 / scale)), -L, L);  out = q * scale.
__device__ __forceinline__ float wfq_one(float w, float inv_scale, float scale, float lim, int& q) {
  // nearbyintf with two additions (the rounding instruction issues on the quarter-rate pipe); the clamp to +-2^21 first
  // keeps the sum inside the range where that is exact and cannot change a result that is clamped to +-lim afterwards
  float r = rint_small(fminf(fmaxf(__fmul_rn(w, inv_scale), -2097152.0f), 2097152.0f));
  r = fminf(fmaxf(r, -lim), lim);
  q = static_cast<int>(r);
  return __fmul_rn(r, scale);
}

template <typename XT, int MAXC>
__global__ void __launch_bounds__(1024) wfq_vec_kernel(const WfqParams p) {
  __shared__ float red[2][3][32];
  const int nchunks = p.cols >> 4;
  const bool has_smooth = p.smooth != nullptr;
  constexpr int NREG = MAXC > 0 ? MAXC : 1;
  const float lim = static_cast<float>((1 << (p.num_bits - 1)) - 1);
  const float nspace = static_cast<float>((1 << p.num_bits) - 2);
  int iter = 0;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x, ++iter) {
    const XT* wr = reinterpret_cast<const XT*>(p.w) + static_cast<int64_t>(row) * p.ldw;
    float v[NREG][16];
    float sa = 0.0f, sq = 0.0f, am = 0.0f;
    auto fetch = [&](int ch, float (&dst)[16]) {
      load16(wr + ch * 16, dst);
      if (has_smooth) {
        float sm[16];
        load16(p.smooth + ch * 16, sm);
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = rnd_if<XT>(__fmul_rn(dst[i], sm[i]), p.native_mul);
      }
    };
    auto stats = [&](const float (&val)[16]) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float a = fabsf(val[i]);
        sa += a;
        sq += Elem<XT>::rnd(__fmul_rn(val[i], val[i]));
        am = fmaxf(am, a);
      }
    };
    if (MAXC > 0) {
#pragma unroll
      for (int c = 0; c < NREG; ++c) {
        const int ch = threadIdx.x + c * blockDim.x;
        if (ch < nchunks) {
          fetch(ch, v[c]);
          stats(v[c]);
        }
      }
    } else if (p.mode != QLIN_W_GIVEN) {
      for (int ch = threadIdx.x; ch < nchunks; ch += blockDim.x) {
        fetch(ch, v[0]);
        stats(v[0]);
      }
    }
    if (p.mode == QLIN_W_SAWB) {
      sa = block_reduce<OpSum>(sa, red[iter & 1][0], 0.0f);
      // the second reduction may reuse the barrier of the first: distinct slot
      sq = block_reduce<OpSum>(sq, red[iter & 1][1], 0.0f);
    } else if (p.mode == QLIN_W_MAX) {
      am = block_reduce<OpMax>(am, red[iter & 1][2], 0.0f);
    }
    const float clip = wfq_clip<XT>(p, sa, sq, am, row);
    if (threadIdx.x == 0 && p.mode != QLIN_W_GIVEN) p.clip_io[row] = clip;
    // scale = clip * 2 / nspace in the weight dtype, then widened
    const float scale = wfq_scale<XT>(p, clip, nspace);
    const float inv_scale = __fdiv_rn(1.0f, scale);
    auto emit = [&](int ch, const float (&val)[16]) {
      float dq[16];
      uint32_t wds[4] = {0, 0, 0, 0};
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        int q;
        dq[i] = wfq_one(val[i], inv_scale, scale, lim, q);
        wds[i >> 2] |= static_cast<uint32_t>(q & 0xFF) << (8 * (i & 3));
      }
      if (p.codes != nullptr)
        *reinterpret_cast<uint4*>(p.codes + static_cast<int64_t>(row) * p.ldq + ch * 16) =
            make_uint4(wds[0], wds[1], wds[2], wds[3]);
      if (p.dq_out != nullptr) store16(reinterpret_cast<XT*>(p.dq_out) + static_cast<int64_t>(row) * p.ldo + ch * 16, dq);
    };
    if (MAXC > 0) {
#pragma unroll
      for (int c = 0; c < NREG; ++c) {
        const int ch = threadIdx.x + c * blockDim.x;
        if (ch < nchunks) emit(ch, v[c]);
      }
    } else {
      for (int ch = threadIdx.x; ch < nchunks; ch += blockDim.x) {
        fetch(ch, v[0]);
        emit(ch, v[0]);
      }
    }
  }
}

template <typename XT>
__global__ void __launch_bounds__(256) wfq_scalar_kernel(const WfqParams p) {
  __shared__ float red[2][3][32];
  const bool has_smooth = p.smooth != nullptr;
  const float lim = static_cast<float>((1 << (p.num_bits - 1)) - 1);
  const float nspace = static_cast<float>((1 << p.num_bits) - 2);
  int iter = 0;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x, ++iter) {
    const XT* wr = reinterpret_cast<const XT*>(p.w) + static_cast<int64_t>(row) * p.ldw;
    float sa = 0.0f, sq = 0.0f, am = 0.0f;
    if (p.mode != QLIN_W_GIVEN) {
      for (int c = threadIdx.x; c < p.cols; c += blockDim.x) {
        float v = load1(wr + c);
        if (has_smooth) v = rnd_if<XT>(__fmul_rn(v, p.smooth[c]), p.native_mul);
        const float a = fabsf(v);
        sa += a;
        sq += Elem<XT>::rnd(__fmul_rn(v, v));
        am = fmaxf(am, a);
      }
      if (p.mode == QLIN_W_SAWB) {
        sa = block_reduce<OpSum>(sa, red[iter & 1][0], 0.0f);
        sq = block_reduce<OpSum>(sq, red[iter & 1][1], 0.0f);
      } else {
        am = block_reduce<OpMax>(am, red[iter & 1][2], 0.0f);
      }
    }
    const float clip = wfq_clip<XT>(p, sa, sq, am, row);
    if (threadIdx.x == 0 && p.mode != QLIN_W_GIVEN) p.clip_io[row] = clip;
    const float scale = wfq_scale<XT>(p, clip, nspace);
    const float inv_scale = __fdiv_rn(1.0f, scale);
    for (int c = threadIdx.x; c < p.cols; c += blockDim.x) {
      float v = load1(wr + c);
      if (has_smooth) v = rnd_if<XT>(__fmul_rn(v, p.smooth[c]), p.native_mul);
      int q;
      const float dq = wfq_one(v, inv_scale, scale, lim, q);
      if (p.codes != nullptr) p.codes[static_cast<int64_t>(row) * p.ldq + c] = static_cast<int8_t>(q);
      if (p.dq_out != nullptr) store1(reinterpret_cast<XT*>(p.dq_out) + static_cast<int64_t>(row) * p.ldo + c, dq);
    }
  }
}

template <typename XT>
static int launch_wfq(const WfqParams& p, cudaStream_t stream) {
  const int es = static_cast<int>(sizeof(XT));
  bool vec = (p.cols % 16 == 0) && aligned16(p.w) && ((p.ldw * es) % 16 == 0);
  if (p.smooth != nullptr) vec = vec && aligned16(p.smooth);
  if (p.codes != nullptr) vec = vec && aligned16(p.codes) && (p.ldq % 16 == 0);
  if (p.dq_out != nullptr) vec = vec && aligned16(p.dq_out) && ((p.ldo * es) % 16 == 0);
  const int max_blocks = sm_count() * 16;
  if (!vec) {
    const int grid = p.rows < max_blocks ? p.rows : max_blocks;
    wfq_scalar_kernel<XT><<<grid, 256, 0, stream>>>(p);
    QLIN_CHECK_LAUNCH("qlin_weight_fq_perch");
    return QLIN_OK;
  }
  const int nchunks = p.cols / 16;
  int threads = ((nchunks + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  const int blocks_per_sm = 2048 / threads;
  int grid = sm_count() * (blocks_per_sm > 0 ? blocks_per_sm : 1);
  if (grid > p.rows) grid = p.rows;
  if (nchunks <= threads) {
    wfq_vec_kernel<XT, 1><<<grid, threads, 0, stream>>>(p);
  } else if (nchunks <= 2 * threads) {
    wfq_vec_kernel<XT, 2><<<grid, threads, 0, stream>>>(p);
  } else {
    wfq_vec_kernel<XT, 0><<<grid, threads, 0, stream>>>(p);
  }
  QLIN_CHECK_LAUNCH("qlin_weight_fq_perch");
  return QLIN_OK;
}

}  // namespace qlin

using namespace qlin;

extern "C" int qlin_act_quant(const qlin_quant_args* a, void* stream) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_act_quant: args is NULL");
  if (a->x == nullptr) return fail(QLIN_ERR_NULL, "qlin_act_quant: x is NULL");
  if (a->codes == nullptr && a->dq_out == nullptr && a->scale_out == nullptr)
    return fail(QLIN_ERR_NULL, "qlin_act_quant: no output requested");
  if (a->rows < 0 || a->cols < 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_act_quant: negative dimension");
  if (a->rows == 0 || a->cols == 0) return QLIN_OK;
  if (a->ldx < a->cols || (a->codes != nullptr && a->ldq < a->cols) || (a->dq_out != nullptr && a->lddq < a->cols))
    return fail(QLIN_ERR_BAD_SHAPE, "qlin_act_quant: leading dimension smaller than the row length");
  if (a->mode < QLIN_Q_I8_DYN || a->mode > QLIN_Q_F8_TENSOR)
    return fail(QLIN_ERR_UNSUPPORTED, "qlin_act_quant: unknown mode %d", a->mode);
  if (a->smooth != nullptr && !a->smooth_mul && a->smooth_rcp == nullptr)
    return fail(QLIN_ERR_NULL, "qlin_act_quant: smooth_rcp is required when rows are divided by smooth");
  if (a->mode == QLIN_Q_F8_TENSOR && (a->scale_in == nullptr || !(a->scale0 > 0.0f)))
    return fail(QLIN_ERR_NULL, "qlin_act_quant: QLIN_Q_F8_TENSOR needs the tensor absmax in scale_in and a positive scale0");
  if (a->mode == QLIN_Q_I8_GIVEN_SCALE && a->scale_in == nullptr)
    return fail(QLIN_ERR_NULL, "qlin_act_quant: scale_in is required by QLIN_Q_I8_GIVEN_SCALE");
  if ((a->mode == QLIN_Q_I8_DYN || a->mode == QLIN_Q_I8_GIVEN_SCALE) && (a->qmax_levels < 1 || a->qmax_levels > 127))
    return fail(QLIN_ERR_UNSUPPORTED, "qlin_act_quant: qmax_levels must be in [1, 127]");
  QuantParams p;
  p.x = a->x;
  p.smooth = a->smooth;
  p.smooth_rcp = a->smooth_rcp;
  p.scale_in = a->scale_in;
  p.codes = static_cast<uint8_t*>(a->codes);
  p.scale_out = a->scale_out;
  p.dq_out = a->dq_out;
  p.status = a->status;
  p.ldx = a->ldx;
  p.ldq = a->ldq;
  p.lddq = a->lddq;
  p.rows = a->rows;
  p.cols = a->cols;
  p.mode = a->mode;
  p.native = (a->native_chain & 2) != 0;
  p.native_smooth = (a->native_chain & 1) != 0;
  p.smooth_exact = (a->native_chain & 4) != 0;
  p.smooth_mul = a->smooth_mul != 0;
  p.clamp_codes = a->clamp_codes != 0;
  p.levels = a->qmax_levels;
  p.dl8_flush = a->dl8_flush != 0;
  p.scale_in_stride = a->scale_in_stride != 0 ? 1 : 0;
  p.scale0 = a->scale0;
  p.zp0 = a->zp0;
  p.lo = a->lo;
  p.hi = a->hi;
  p.shift = a->shift;
  p.add2 = a->add2;
  p.dyn_eps = a->dyn_eps;
  p.f8_e5m2 = a->f8_format == 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (a->x_dtype) {
    case QLIN_DT_F32:
      return launch_act_quant<float>(p, s);
    case QLIN_DT_F16:
      return launch_act_quant<__half>(p, s);
    case QLIN_DT_BF16:
      return launch_act_quant<__nv_bfloat16>(p, s);
    default:
      return fail(QLIN_ERR_BAD_DTYPE, "qlin_act_quant: x_dtype must be F32, F16 or BF16");
  }
}

extern "C" int qlin_weight_fq_perch(const qlin_wfq_args* a, void* stream) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_weight_fq_perch: args is NULL");
  if (a->w == nullptr || a->clip_io == nullptr) return fail(QLIN_ERR_NULL, "qlin_weight_fq_perch: w or clip_io is NULL");
  if (a->dq_out == nullptr && a->codes == nullptr) return fail(QLIN_ERR_NULL, "qlin_weight_fq_perch: no output requested");
  if (a->rows < 0 || a->cols < 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_weight_fq_perch: negative dimension");
  if (a->rows == 0 || a->cols == 0) return QLIN_OK;
  if (a->num_bits != 2 && a->num_bits != 4 && a->num_bits != 8)
    return fail(QLIN_ERR_UNSUPPORTED, "qlin_weight_fq_perch: num_bits must be 2, 4 or 8");
  if (a->mode < QLIN_W_SAWB || a->mode > QLIN_W_GIVEN) return fail(QLIN_ERR_UNSUPPORTED, "qlin_weight_fq_perch: unknown mode");
  if (a->ldw < a->cols || (a->dq_out != nullptr && a->ldo < a->cols) || (a->codes != nullptr && a->ldq < a->cols))
    return fail(QLIN_ERR_BAD_SHAPE, "qlin_weight_fq_perch: leading dimension smaller than the row length");
  WfqParams p;
  p.w = a->w;
  p.smooth = a->smooth;
  p.dq_out = a->dq_out;
  p.codes = static_cast<int8_t*>(a->codes);
  p.clip_io = a->clip_io;
  p.ldw = a->ldw;
  p.ldo = a->ldo;
  p.ldq = a->ldq;
  p.rows = a->rows;
  p.cols = a->cols;
  p.num_bits = a->num_bits;
  p.mode = a->mode;
  p.native_mul = a->native_mul != 0;
  p.clip_dtype = a->clip_dtype;
  p.c0 = a->c0;
  p.c1 = a->c1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (a->dtype) {
    case QLIN_DT_F32:
      return launch_wfq<float>(p, s);
    case QLIN_DT_F16:
      return launch_wfq<__half>(p, s);
    case QLIN_DT_BF16:
      return launch_wfq<__nv_bfloat16>(p, s);
    default:
      return fail(QLIN_ERR_BAD_DTYPE, "qlin_weight_fq_perch: dtype must be F32, F16 or BF16");
  }
}
