/*
 * qlin_b200.h -- C ABI of libqlin_b200.so: the quantized-Linear hot path of
 * fms-model-optimizer, written for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless a comment says otherwise.
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream.
 *   - The library never allocates, frees or keeps device memory; the caller owns all
 *     inputs, outputs and workspaces.  Calls are asynchronous on `stream`.
 *   - Return value: 0 (QLIN_OK) or a negative qlin_status.  The text of the last error
 *     on the calling host thread is available from qlin_last_error_string().
 *   - Kernels never trap.  A kernel that gives up a bounded wait writes a negative
 *     qlin_status to `*status` (when the caller passed one) and returns.
 *
 * Each entry point names the fms-model-optimizer interface it stands in for
 * (paths relative to that project's root).
 */
#ifndef QLIN_B200_H
#define QLIN_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QLIN_VERSION 100

typedef enum qlin_status {
  QLIN_OK = 0,
  QLIN_ERR_BAD_SHAPE = -1,
  QLIN_ERR_BAD_ALIGN = -2,
  QLIN_ERR_BAD_DTYPE = -3,
  QLIN_ERR_UNSUPPORTED = -4,
  QLIN_ERR_LAUNCH = -5,
  QLIN_ERR_TIMEOUT = -6,
  QLIN_ERR_NULL = -7,
  QLIN_ERR_DEVICE = -8,
  QLIN_ERR_TOO_LARGE = -9
} qlin_status;

typedef enum qlin_dtype {
  QLIN_DT_NONE = 0,
  QLIN_DT_I8 = 1,
  QLIN_DT_U8 = 2,
  QLIN_DT_I32 = 3,
  QLIN_DT_F32 = 4,
  QLIN_DT_F16 = 5,
  QLIN_DT_BF16 = 6,
  QLIN_DT_F8E4M3 = 7,
  QLIN_DT_F8E5M2 = 8
} qlin_dtype;

/* ------------------------------------------------------------------------------------------------
 * Library / device queries
 * ---------------------------------------------------------------------------------------------- */
int qlin_version(void);
const char* qlin_last_error_string(void);
/* 1 when `device` has compute capability 10.x (tcgen05 + TMA), 0 otherwise, <0 on error. */
int qlin_device_supported(int device);

/* ------------------------------------------------------------------------------------------------
 * qlin_gemm -- 8-bit tensor-core GEMM  D[M,N] = epilogue( C + sum_chunks f(A_chunk . B_chunk^T) )
 *
 * Replaces: tl_matmul_chunk_truncate / imatmul_kernel / matmul_kernel(_DABC)
 *           (fms_mo/custom_ext_kernels/triton_kernels.py:468, :212, :97, :306),
 *           cutlass_mm.run (fms_mo/custom_ext_kernels/cutlass_i8i32gemm.cpp:34,
 *           cutlass_i8i32gemm.cu:67-120), cublas_gemm::gemm_nt_i8i32
 *           (fms_mo/custom_ext_kernels/ext_kernel_cublas.cpp:103-195, :295) and the dequantise
 *           chain of QLinearINT8Deploy.iaddmm_int (fms_mo/modules/linear.py:1115-1188),
 *           fms_mo::iaddmm / q_iaddmm_dq (fms_mo/custom_ext_kernels/utils.py:729-790) and
 *           LinearFuncFPxFwdBwd.forward (fms_mo/modules/linear.py:1958-1973).
 *
 * Operands: A is [M,K], B is [N,K], both with K contiguous ("NT"; B is the `.t()` view the
 * reference passes as its [k,n] operand).  kind = QLIN_DT_I8 (int32 accumulation) or
 * QLIN_DT_F8E4M3 / QLIN_DT_F8E5M2 (fp32 accumulation; e5m2 operands are what the backward of the FP8 Linear
 * multiplies, fms_mo/modules/linear.py:2003-2046).  a, b must be 16-byte aligned, lda/ldb multiples of 16.
 *
 * Chunked accumulation (K1/K2 semantics): K is cut into chunks of `chunk_k` elements (a multiple
 * of 32; <=0 means one chunk).  Per chunk p = A_c . B_c^T; integer kinds: clamp p to
 * max_acc_bits (if < 32), then p = ((p + (1 << (t-1))) >> t) << t with t = trun_bits;
 * float kinds: bits(p) = (bits(p) + (1 << (t-1))) & ~((1 << t) - 1), then the optional DL16
 * clamp/flush.  trunc_then_acc != 0 applies f to each chunk product and adds it to the
 * running sum; == 0 applies f to (running sum + product).  The K tail is zero-filled.
 *
 * Epilogue, per element with acc the final accumulator (converted to fp32 for the scaled
 * modes), rs = row_scale[m * row_scale_stride] (1 if NULL), cs likewise:
 *   QLIN_EPI_RAW        d = acc                             (out_dtype I32 for I8, F32 for F8)
 *   QLIN_EPI_SCALE_PROD s = round(round(rs * cs, prod_round), scale_round); y = acc * s; y = y + bias[n];
 *                       y = round(y, acc_round); d = cast(y, out_dtype)
 *   QLIN_EPI_SCALE_SEQ  y = (acc * rs) * cs; y = round(y, mid_round); y = y + bias[n];
 *                       y = round(y, acc_round); d = cast(y, out_dtype)
 * round(.., QLIN_DT_NONE/F32) is the identity; F16 / BF16 round to nearest even and widen back.
 * Every multiply and add is a separately rounded fp32 operation (no FMA contraction), which is
 * what the reference's eager tensor expressions compute.
 * ---------------------------------------------------------------------------------------------- */
typedef enum qlin_epilogue {
  QLIN_EPI_RAW = 0,
  QLIN_EPI_SCALE_PROD = 1,
  QLIN_EPI_SCALE_SEQ = 2
} qlin_epilogue;

typedef struct qlin_gemm_args {
  const void* a;
  const void* b;
  const void* c;          /* optional [M,N] initial accumulator (int32 / fp32); may alias d */
  void* d;
  const float* row_scale; /* optional */
  const float* col_scale; /* optional */
  const float* bias;      /* optional [N] */
  int32_t* status;        /* optional device status word, written only on failure */
  int64_t lda, ldb, ldc, ldd; /* leading dimensions in elements */
  int32_t M, N, K;
  int32_t kind;             /* qlin_dtype of A and B */
  int32_t chunk_k;
  int32_t trun_bits;
  int32_t max_acc_bits;     /* 32 = no clamp (integer kinds only) */
  int32_t trunc_then_acc;
  int32_t clamp_dl16;       /* float kinds only */
  int32_t epilogue;         /* qlin_epilogue */
  int32_t row_scale_stride; /* 0 = one scalar, 1 = per row */
  int32_t col_scale_stride; /* 0 = one scalar, 1 = per column */
  int32_t prod_round;       /* qlin_dtype: dtype the reference forms input_scale * w_scale in */
  int32_t scale_round;      /* qlin_dtype */
  int32_t mid_round;        /* qlin_dtype */
  int32_t acc_round;        /* qlin_dtype */
  int32_t out_dtype;        /* qlin_dtype */
  /* Row-block scatter of the output (the reduce-scatter half of a row-parallel Linear, done by the epilogue's own
     stores): when scatter_rows > 0, output row m goes to scatter_d[m / scatter_rows] at row
     scatter_row0 + m % scatter_rows (leading dimension ldd, d unused).  The bases may be buffers of other GPUs
     mapped into this process; scatter_rows must be a multiple of 128.  No counterpart in the reference. */
  void* scatter_d[8];
  int32_t scatter_rows;
  int32_t scatter_row0;
  int32_t max_ctas;         /* 0: one persistent CTA per SM; > 0: at most this many CTAs (each needs a whole SM),
                               leaving SMs free for a kernel that runs concurrently on another stream, e.g. a
                               collective.  Results do not depend on it. */
} qlin_gemm_args;

int qlin_gemm(const qlin_gemm_args* args, void* stream);

/* qlin_gemm_batched -- the same problem `batch` times over operands that lie `stride_a`, `stride_b` (elements of
 * the operand type) and `stride_d` (elements of the output type) apart: D[i] = epilogue(A[i] . B[i]^T).  The batched
 * int8 product behind QBmmINT8Deploy (fms_mo/modules/bmm.py:719-752), where the reference itself "has not implemented
 * any batched CUTLASS matmul" and simulates with torch.matmul on fp16 copies of the codes.  Scales, bias and the
 * status word are shared by all problems; `c` must be NULL; row-block scatter is not provided.  Dense stacks of
 * unchunked problems (stride_a = M * lda, stride_b = N * ldb, stride_d a multiple of 16 bytes) run as ONE launch whose
 * tiles walk over all problems; anything else as one launch per problem on `stream`, in order. */
int qlin_gemm_batched(const qlin_gemm_args* args, int32_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, void* stream);

/* ------------------------------------------------------------------------------------------------
 * qlin_act_quant -- row-wise (per-token / per-channel) dynamic 8-bit quantisation in one pass.
 *
 * Replaces: `x / smoothq_scale` + QLinearINT8Deploy.qa_dynamic_max_qfunc
 *           (fms_mo/modules/linear.py:1331-1334, :1085-1100), QMaxDynamic.forward / PerTokenMax
 *           (fms_mo/quant/quantizers.py:3531-3534, :3479-3501), the static quantisers
 *           qa_raw_qfunc / qa_fmo_mo_qfunc (fms_mo/modules/linear.py:1061-1083), fms_mo::q_per_t_sym
 *           (fms_mo/custom_ext_kernels/utils.py:792-802), the FP8 scaling of
 *           LinearFuncFPxFwdBwd.forward (fms_mo/modules/linear.py:1935-1953) and the weight
 *           quantisation of QLinearINT8Deploy.from_fms_mo (fms_mo/modules/linear.py:859-871).
 *
 * x is [rows, cols] with cols contiguous; `smooth` (optional, [cols] fp32) divides
 * (smooth_mul == 0) or multiplies (smooth_mul != 0) every row first.
 *   QLIN_Q_I8_DYN     amax per row; scale = max(amax, 1e-5) / qmax_levels; code = rint(v / scale)
 *                     cast to int8 with two's-complement wrap (the reference does not clamp) or
 *                     clamped to +-qmax_levels when clamp_codes != 0.
 *   QLIN_Q_I8_STATIC  code = clamp(rint(((v / scale0 + zp0) - shift) + add2), -128, 127)
 *                     (qa_raw_qfunc: zp0 = input_zp, shift = 128, add2 = useSymAct)
 *   QLIN_Q_I8_STATIC_CLAMP_FIRST
 *                     code = rint(clamp(v, lo, hi) / scale0 - zp0) - shift, wrapped to int8
 *                     (qa_fmo_mo_qfunc: scale0 = quant_stepsize, zp0 = quant_zero_point)
 *   QLIN_Q_F8_DYN     scale = max(amax / 448, 1e-5); code = e4m3(v / scale), optional DL8 flush
 *   QLIN_Q_I8_GIVEN_SCALE
 *                     scale = scale_in[row * scale_in_stride]; code = rint(v / scale) + zp0,
 *                     wrapped to int8 or clamped to +-qmax_levels
 *   QLIN_Q_I8_STATIC_ROUND_FIRST
 *                     code = clamp(rint(v / scale0 + zp0), lo, hi) - shift
 *                     (QLinearCublasI8I32NT.forward, fms_mo/modules/linear.py:1505-1512: uint8 codes
 *                     shifted by 128, or symmetric codes clamped to +-127)
 *   QLIN_Q_I8_AFFINE_RCP
 *                     code = clamp(nearbyint(v * (1 / scale0)) + zp0, -128, 127), fp32 rows:
 *                     torch.quantize_per_tensor(...).int_repr() (fms_mo::q_per_t_sym,
 *                     fms_mo/custom_ext_kernels/utils.py:792-794)
 *   QLIN_Q_F8_TENSOR  one scale for the whole tensor from its absmax: scale = max(scale_in[0] / scale0, dyn_eps);
 *                     code = fp8(v / scale) in e4m3 (f8_format 0) or e5m2 (f8_format 1), optional DL8 flush; the per-tensor
 *                     branch of LinearFuncFPxFwdBwd (fms_mo/modules/linear.py:1939-1953 with scale0 = 448, dyn_eps = 1e-5;
 *                     :2003-2017 with scale0 = 57344, dyn_eps = 0, e5m2).  scale_out receives the scale in every row.
 *   QLIN_Q_F8_FAKE_SCALED
 *                     to_fp8_scaled_perToken / _perCh (fms_mo/quant/quantizers.py:5336-5420), e4m3:
 *                     scale = 448 / max(amax, dyn_eps) (a multiplier, capped at 65504 on fp16 rows);
 *                     code = e4m3(clamp(v * scale, +-448)); dq_out = e4m3 value / scale;
 *                     scale_out receives the multiplier
 * native_chain is a bit mask: bit 0 rounds the smoothed value to the dtype of x, bit 1 rounds every
 * later intermediate to the dtype of x (what the reference computes when the tensors involved are
 * bf16 / fp16); 0 evaluates the same formulas in fp32 on the widened inputs.  Bit 2 is a promise by the
 * caller that every smooth[c] is exactly representable in the dtype of x (the reference casts its
 * SmoothQuant scale to that dtype); with bits 0-2 set on bf16 rows the kernel uses a shorter, still
 * bit-identical instruction sequence.
 * Outputs: codes [rows, cols] (1 byte each), scale_out [rows] fp32 (optional),
 * dq_out (optional, dtype of x): the fake-quantised value code * scale, QMaxDynamic's output.
 * ---------------------------------------------------------------------------------------------- */
typedef enum qlin_quant_mode {
  QLIN_Q_I8_DYN = 0,
  QLIN_Q_I8_STATIC = 1,
  QLIN_Q_I8_STATIC_CLAMP_FIRST = 2,
  QLIN_Q_F8_DYN = 3,
  QLIN_Q_I8_GIVEN_SCALE = 4,
  QLIN_Q_F8_FAKE_SCALED = 5,
  QLIN_Q_I8_STATIC_ROUND_FIRST = 6,
  QLIN_Q_I8_AFFINE_RCP = 7,
  QLIN_Q_F8_TENSOR = 8
} qlin_quant_mode;

typedef struct qlin_quant_args {
  const void* x;
  const float* smooth;    /* optional [cols] */
  const float* smooth_rcp;/* [cols], required when smooth divides: the correctly rounded fp32 reciprocal of
                             smooth[c], or NaN to make column c take the plain IEEE division.  The kernel
                             derives the exact quotient x / smooth[c] from it with three fused operations. */
  const float* scale_in;  /* QLIN_Q_I8_GIVEN_SCALE: [rows] */
  void* codes;            /* optional [rows, cols] int8 / e4m3 */
  float* scale_out;       /* optional [rows] */
  void* dq_out;           /* optional [rows, cols], dtype of x */
  int32_t* status;
  int64_t ldx, ldq, lddq; /* leading dimensions in elements */
  int32_t rows, cols;
  int32_t x_dtype;        /* F32 / F16 / BF16 */
  int32_t mode;           /* qlin_quant_mode */
  int32_t native_chain;
  int32_t smooth_mul;
  int32_t clamp_codes;
  int32_t qmax_levels;    /* 127 for int8 */
  int32_t dl8_flush;      /* QLIN_Q_F8_DYN: flush |code| < 0.0087890625 to 0 */
  int32_t scale_in_stride;/* QLIN_Q_I8_GIVEN_SCALE: 0 = one scalar, 1 = per row */
  float scale0, zp0, lo, hi, shift, add2; /* static modes */
  float dyn_eps;          /* dynamic modes: lower clamp of the row absmax; the deploy modules use 1e-5,
                             QLinearINT8Train uses 0 (fms_mo/modules/linear.py:2167-2171) */
  int32_t f8_format;      /* QLIN_Q_F8_TENSOR: 0 = e4m3, 1 = e5m2 */
} qlin_quant_args;

int qlin_act_quant(const qlin_quant_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * qlin_pact2_fwd / qlin_pact2_bwd -- PACT+ two-sided fake quantisation (QAT activations).
 *
 * Replaces: PACT2.forward -> PACTplus2STE.forward / .backward
 *           (fms_mo/quant/quantizers.py:1465-1476, :1949-2102).
 * fwd:  y = clamp(x, cvn, cv); q = rint(y / step - zp); out = (q + zp) * step
 *       with n = 2^bits - 1, scale = n / (cv - cvn), step = 1 / scale, zp = cvn * scale,
 *       zp = rint(zp) when align_zero.  cv / cvn are read from device memory ([1] fp32).
 * bwd:  z = (x - cvn) / step; delz = (z - rint(z)) / n;
 *       grad_x = g where cvn < x < cv else 0;
 *       grad_cv  = sum( x >= cv ? g : (x <= cvn ? 0 : -g * delz) );
 *       grad_cvn = sum( x <= cvn ? g : (x >= cv ? 0 :  g * delz) ).
 *       The two sums are reduced in a fixed order (run-to-run deterministic) through a
 *       caller-provided workspace of qlin_pact2_bwd_workspace_bytes(numel) bytes.
 * ---------------------------------------------------------------------------------------------- */
/* variant: which member of the PACT+ family.
 *   QLIN_PACT_TWO_SIDED  PACT2 / PACTplus2STE (above).
 *   QLIN_PACT_ONE_SIDED  PACT / PACTplusSTE (fms_mo/quant/quantizers.py:1016-1070): clamp to [0, cv],
 *                        step = cv / (2^b - 1); grad_clip[0] only.
 *   QLIN_PACT_SYMMETRIC  PACTplusSym / PACTplusSymSTE_rev1 (:1073-1154): clamp to [-cv, cv], levels
 *                        2^b - 2 when align_zero (the reference's intg_zp) else 2^b - 1, out-of-range
 *                        input gradients zeroed; grad_clip[0] only. */
typedef enum qlin_pact_variant { QLIN_PACT_TWO_SIDED = 0, QLIN_PACT_ONE_SIDED = 1, QLIN_PACT_SYMMETRIC = 2 } qlin_pact_variant;

typedef struct qlin_pact2_args {
  const void* x;
  const void* grad_out;   /* bwd only */
  void* out;              /* fwd: y ; bwd: grad_x */
  const float* clip_val;  /* [1] */
  const float* clip_valn; /* [1] */
  float* grad_clip;       /* bwd: [2] = {grad_cv, grad_cvn} */
  void* workspace;        /* bwd */
  int64_t numel;
  int32_t dtype;          /* F32 / F16 / BF16 (x, out, grad_out) */
  int32_t num_bits;
  int32_t align_zero;
  int32_t variant;        /* qlin_pact_variant */
} qlin_pact2_args;

int qlin_pact2_fwd(const qlin_pact2_args* args, void* stream);
int qlin_pact2_bwd(const qlin_pact2_args* args, void* stream);
size_t qlin_pact2_bwd_workspace_bytes(int64_t numel);

/* qlin_pact2_bwd_noalloc -- qlin_pact2_bwd without a caller-provided workspace.
 *
 * No counterpart in fms-model-optimizer: this entry point exists only for hosts of this library.
 * It is for callers that cannot hand over scratch memory -- a runtime whose device pool is sealed
 * after start-up, a hook that receives only its input and output buffers, a step loop that must not
 * call cudaMalloc because it can fail under a fixed budget or stall the device.  `workspace` in the
 * argument block is ignored; the partial sums of the two clip gradients go to a 9472-byte array that
 * is part of the library image and stays resident on every GPU that loads the library.  The call
 * allocates and frees nothing.  Results are identical to qlin_pact2_bwd.
 *   - numel above qlin_pact2_bwd_noalloc_max_numel() (2^31 elements) is rejected with
 *     QLIN_ERR_TOO_LARGE.
 *   - The first call on each device looks up the array's device address; make that call while the
 *     device is current and before any stream capture.
 *   - All calls on a device share the array: calls that may overlap on the GPU race on it.  Nothing
 *     needs clearing between calls (each call writes every slot it later reads). */
int qlin_pact2_bwd_noalloc(const qlin_pact2_args* args, void* stream);
int64_t qlin_pact2_bwd_noalloc_max_numel(void);

/* ------------------------------------------------------------------------------------------------
 * qlin_weight_fq_perch -- per-output-channel symmetric weight fake quantisation with the
 * clip value computed in the same pass.
 *
 * Replaces: SAWB.forward -> SAWBPlusZeroPerChSTE.forward + sawb_params_code(perCh=True)
 *           (fms_mo/quant/quantizers.py:434-446, :503-567, :633-655) and
 *           Qmax.forward -> QmaxPerChSTE.forward (fms_mo/quant/quantizers.py:3048-3141, :3190-3220).
 * w is [rows, cols] (one row per output channel), optionally multiplied by smooth[cols] first.
 *   QLIN_W_SAWB  clip = c1 * mean|w| + c0 * sqrt(mean w^2)   (c0, c1 given by the caller)
 *   QLIN_W_MAX   clip = max|w|
 *   QLIN_W_GIVEN clip read from clip_io
 * scale = clip * 2 / (2^bits - 2); q = clamp(nearbyint(w / scale), -(2^(bits-1) - 1), +..);
 * out = q * scale (dq_out, dtype of w) and / or q as int8 (codes).  clip_io [rows] fp32 is
 * written for SAWB / MAX and read for GIVEN.
 * ---------------------------------------------------------------------------------------------- */
typedef enum qlin_wq_mode { QLIN_W_SAWB = 0, QLIN_W_MAX = 1, QLIN_W_GIVEN = 2 } qlin_wq_mode;

typedef struct qlin_wfq_args {
  const void* w;
  const float* smooth;  /* optional [cols] */
  void* dq_out;         /* optional [rows, cols] */
  void* codes;          /* optional [rows, cols] int8 */
  float* clip_io;       /* [rows] */
  int64_t ldw, ldo, ldq;
  int32_t rows, cols;
  int32_t dtype;        /* F32 / F16 / BF16 */
  int32_t num_bits;
  int32_t mode;         /* qlin_wq_mode */
  int32_t native_mul;   /* round w * smooth to dtype before use (reference multiplies in the weight dtype) */
  int32_t clip_dtype;   /* 0: scale = clip * 2 / (2^bits - 2) is formed in the weight dtype; F32 / F16 / BF16: in that
                           dtype (QLIN_W_GIVEN with a clip_val buffer whose dtype differs from the weights') */
  float c0, c1;
} qlin_wfq_args;

int qlin_weight_fq_perch(const qlin_wfq_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * qlin_tensor_fq -- per-tensor fake quantisers: one clip value (or one FP8 scale) for all elements.
 *
 * Replaces: SAWB.forward -> SAWBPlusZeroSTE.forward + sawb_params_code(perCh=False)
 *           (fms_mo/quant/quantizers.py:434-446, :455-500, :657-671), the recipe default "sawb+";
 *           Qmax.forward -> QmaxSTE.forward (fms_mo/quant/quantizers.py:3048-3141, :3159-3187);
 *           to_fp8_scaled / to_fp8_saturated (fms_mo/quant/quantizers.py:5316-5372), e4m3, emulate.
 * mode (qlin_wq_mode): QLIN_W_SAWB  clip = c1 * mean|x| + c0 * sqrt(mean x^2), max|x| if that is <= 0
 *                      QLIN_W_MAX   clip = max|x|
 *                      QLIN_W_GIVEN clip read from clip_io[0]
 * clip_io[0] is written for SAWB / MAX (out may then be NULL to get the statistic alone).
 * kind: QLIN_PT_INT_SYM    t = clamp(x * (1/clip), -1, 1) * 0.5 + 0.5; q = rint(levels * t) with
 *                          levels = 2^bits - 2 (align_zero) or 2^bits - 1;
 *                          out = (2 * (q / levels) - 1) * clip, or q - levels / 2 when dequantize == 0
 *       QLIN_PT_F8_SCALED  s = 448 / max(clip, 1e-12); out = e4m3(clamp(x * s, +-448)) / s
 *       QLIN_PT_F8_SAT     out = e4m3(clamp(x, +-448))   (mode must be QLIN_W_GIVEN; clip unused)
 * workspace: qlin_tensor_fq_workspace_bytes(numel) bytes of device memory (not needed for GIVEN).
 * ---------------------------------------------------------------------------------------------- */
typedef enum qlin_pt_kind { QLIN_PT_INT_SYM = 0, QLIN_PT_F8_SCALED = 1, QLIN_PT_F8_SAT = 2 } qlin_pt_kind;

typedef struct qlin_tensor_fq_args {
  const void* x;
  void* out;         /* optional for SAWB / MAX */
  float* clip_io;    /* [1] */
  float* workspace;
  int64_t numel;
  int32_t dtype;     /* F32 / F16 / BF16 */
  int32_t num_bits;
  int32_t mode;      /* qlin_wq_mode */
  int32_t kind;      /* qlin_pt_kind */
  int32_t align_zero;
  int32_t dequantize;
  float c0, c1;
} qlin_tensor_fq_args;

int qlin_tensor_fq(const qlin_tensor_fq_args* args, void* stream);
int64_t qlin_tensor_fq_workspace_bytes(int64_t numel);

/* ------------------------------------------------------------------------------------------------
 * qlin_block_quant -- builds the bf16 input row of up to three W8A8 Linears that share it and
 * quantises it per token for each of them, reading the activations once.
 *
 * The quantise step replaces QLinearINT8Deploy.qa_dynamic_max_qfunc after the SmoothQuant division
 * (fms_mo/modules/linear.py:1085-1100, :1322-1324) for bf16 activations, bit for bit.  The prologues
 * have no counterpart in the reference: a model runs them as separate PyTorch kernels around its
 * Linears (RMSNorm, residual add, SiLU * up); they are fused here because at prefill sizes those
 * kernels move more bytes than the quantiser itself.
 *   QLIN_BLOCK_PLAIN     h = x
 *   QLIN_BLOCK_NORM      t = x (+ r, stored to x_out when given); h = bf16(t * rsqrt(mean t^2 + norm_eps) * norm_w)
 *   QLIN_BLOCK_SILU_MUL  h = bf16(bf16(x / (1 + exp(-x))) * r)
 * For output o < nout: v = bf16(h * smooth_rcp[o]) (h when smooth_rcp[o] is NULL),
 *   QLIN_BLOCK_DYN          s = bf16(max(amax|v|, dyn_eps) / qmax_levels) -> scale_out[o]; codes[o] = int8(rint(bf16(v / s)))
 *   QLIN_BLOCK_GIVEN_SCALE  s = scale_in[row] (one output): the second pass of a row-parallel shard,
 *                           after the scales of all shards were reduced with MAX
 *   QLIN_BLOCK_SCALE_ONLY   only scale_out[o] is written (or, with ndst > 0, stored to every destination): the first pass
 *                           of a row-parallel shard
 * smooth_rcp[o][c] must be the correctly rounded fp32 reciprocal of a bf16-valued SmoothQuant scale
 * (the reference casts that scale to the activation dtype).  All tensors bf16, 16-byte aligned rows,
 * cols a multiple of 16 and at most 16384.  h_out (optional) receives h.
 * ---------------------------------------------------------------------------------------------- */
typedef enum qlin_block_prologue { QLIN_BLOCK_PLAIN = 0, QLIN_BLOCK_NORM = 1, QLIN_BLOCK_SILU_MUL = 2 } qlin_block_prologue;
typedef enum qlin_block_mode { QLIN_BLOCK_DYN = 0, QLIN_BLOCK_GIVEN_SCALE = 1, QLIN_BLOCK_SCALE_ONLY = 2 } qlin_block_mode;

typedef struct qlin_block_quant_args {
  const void* x;        /* [rows, cols] bf16 */
  const void* r;        /* NORM: optional addend; SILU_MUL: the second factor */
  int32_t r_parts;      /* NORM: number of addends (0 or 1: just r); part i starts r_part_stride elements after part i-1.
                           The parts are summed in fp32 in index order and rounded to bf16 once, then added to x:
                           the reduction of a row-parallel Linear whose shards wrote their partial outputs side by side */
  int64_t r_part_stride;
  void* x_out;          /* NORM with r: x + r (may alias x) */
  void* h_out;          /* optional: the row the Linears see */
  const void* norm_w;   /* NORM: [cols] bf16 */
  const float* smooth_rcp[3];
  void* codes[3];       /* [rows, cols] int8 */
  float* scale_out[3];  /* [rows] */
  const float* scale_in;/* GIVEN_SCALE: [rows] */
  int64_t scale_in_stride; /* GIVEN_SCALE with scale_in_parts > 1: elements between the parts */
  int32_t scale_in_parts;  /* GIVEN_SCALE: 0 or 1 = scale_in as is; n > 1 = the row's scale is the maximum of n arrays
                              (the scales the shards of a row-parallel Linear stored side by side) */
  /* Replicated outputs (the all-gather half of sequence parallelism, done by the kernel's own stores): when ndst > 0
     codes[o] and scale_out[o] are ignored; for every d < ndst the codes of output o go to
     (int8*)dst_base[d] + codes_off[o] at row dst_row0 + row (leading dimension ldq[o]) and the scales to
     (float*)((char*)dst_base[d] + scale_off[o]) + dst_row0 + row.  Offsets in bytes; bases may be other GPUs' buffers. */
  void* dst_base[8];
  int64_t codes_off[3];
  int64_t scale_off[3];
  int32_t ndst;
  int32_t dst_row0;
  int64_t ldx, ldr, ldxo, ldh, ldq[3];
  int32_t rows, cols, nout;
  int32_t prologue;     /* qlin_block_prologue */
  int32_t mode;         /* qlin_block_mode */
  int32_t qmax_levels;
  float norm_eps, dyn_eps;
  int32_t max_ctas;     /* 0: fill the GPU; > 0: at most this many blocks, leaving SMs to kernels of other streams (a launch
                           whose replicated outputs are bound by the links anyway) */
  /* NVLink-switch forms, for buffers that all GPUs of the node have bound to one multicast object (the addresses are
     then the multicast mapping, not a peer pointer).
     r_multimem != 0:   NORM only; r is read with multimem.ld_reduce: every 16-byte load returns the sum over all GPUs'
                        copies of the buffer (bf16, accumulated in fp32 by the switch, rounded once): the reduction of a
                        row-parallel Linear whose shards each wrote their partial output into their own copy.
                        r_parts is ignored.
     dst_multimem != 0: dst_base[0] is the multicast address: codes and scales are written with multimem.st, one store
                        that lands in every GPU's copy.  ndst is 1, or 2 with dst_base[1] = this GPU's own buffer, which
                        then also gets a plain store, so that later kernels of this GPU need not wait for the store's
                        round trip through the switch. */
  int32_t r_multimem;
  int32_t dst_multimem;
} qlin_block_quant_args;

int qlin_block_quant(const qlin_block_quant_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * qlin_col_absmax -- per-column (input-channel) absolute maximum of x [rows, cols], kept as a running maximum.
 *
 * Replaces: activation_stats of the SmoothQuant calibration pass (fms_mo/quant/ptq.py:2586-2596):
 *           tensor.view(-1, hidden).abs().max(dim=0) followed by torch.max with the value kept so far; called from the
 *           forward hooks get_act_scales installs on every Linear (fms_mo/quant/ptq.py:2609-2657).  The result feeds
 *           QLinear.set_act_scale / the smoothq_act_scale buffer (fms_mo/modules/linear.py:345-368).
 * amax_io [cols] fp32: with accumulate == 0 it is overwritten with max_r |x[r, c]|; with accumulate != 0 it receives
 * max(amax_io[c], max_r |x[r, c]|) (its content must then be non-negative or NaN).  A NaN anywhere in a column makes that
 * column's result NaN, as torch.max does.  The result is exact (a maximum does not depend on the order it is taken in).
 * ---------------------------------------------------------------------------------------------- */
typedef struct qlin_col_absmax_args {
  const void* x;
  float* amax_io;
  int64_t ldx;       /* elements between rows */
  int32_t rows, cols;
  int32_t dtype;     /* F32 / F16 / BF16 */
  int32_t accumulate;
} qlin_col_absmax_args;

int qlin_col_absmax(const qlin_col_absmax_args* args, void* stream);

/* qlin_rope -- rotary position embedding in place on x [tokens, heads, head_dim] bf16 (token pitch
 * ld_token elements), position = token % seq_len, cos / sin [seq_len, head_dim / 2] fp32, halves
 * rotated as (x[i], x[i + head_dim / 2]).  No counterpart in the reference (model plumbing between
 * the q/k Linears and attention). */
typedef struct qlin_rope_args {
  void* x;
  const float* cos;
  const float* sin;
  int64_t ld_token;
  int32_t tokens, heads, head_dim, seq_len;
} qlin_rope_args;

int qlin_rope(const qlin_rope_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Peer-memory plumbing of the tensor-parallel path (one process per GPU).  No counterpart in the
 * reference, which leaves sharding to the serving stack around it.
 *   qlin_ipc_export   handle_out receives 64 bytes naming the allocation dev_ptr lies in, offset_out the
 *                     pointer's offset in that allocation; send both to the peer processes.
 *   qlin_ipc_open     maps a peer's allocation into this process (peer access is enabled on first use);
 *                     base_out is what qlin_ipc_close takes, ptr_out = base + offset.
 *   qlin_peer_barrier launches a one-warp kernel: rank stores the next epoch into slot `rank` of every
 *                     peer's flag array and waits (at most timeout_ns, then QLIN_ERR_TIMEOUT in *status) until all
 *                     `world` slots of its own array carry it.  Stores made to peer memory by earlier work of
 *                     the stream are visible to the peers' work after their barrier.  `epoch` is a device
 *                     counter owned by this barrier object; flag arrays and epoch start zeroed.
 * ---------------------------------------------------------------------------------------------- */
int qlin_ipc_export(const void* dev_ptr, void* handle_out, int64_t* offset_out);
int qlin_ipc_open(const void* handle, int64_t offset, void** base_out, void** ptr_out);
int qlin_ipc_close(void* base);
/* Queues a device-to-device copy of `height` rows of `width` bytes (pitches in bytes) on `stream`; either side may be
 * a mapped peer address.  The copy engines carry it, so it overlaps kernels of other streams without taking SMs. */
int qlin_peer_copy2d(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width, int64_t height, void* stream);

/* qlin_shard_reduce -- the reduce-scatter half of a row-parallel Linear through the NVLink switch: every GPU holds its
 * partial output in its own copy of a buffer bound to one multicast object; the owner of a block of rows reads the block
 * through the multicast mapping (multimem.ld_reduce: the sum over all copies, accumulated in fp32, rounded to bf16 once),
 * adds an optional local bf16 tensor in fp32 and writes bf16:  out = bf16(add + sum over GPUs of part).  All bf16,
 * 16-byte aligned, cols and leading dimensions multiples of 8 elements; out may alias add.  max_ctas > 0 caps the grid
 * (the kernel is bound by the links; a dozen CTAs carry it).  No counterpart in the reference. */
typedef struct qlin_shard_reduce_args {
  const void* src_multicast; /* multicast address of the first element of this GPU's block */
  const void* add;           /* optional [rows, cols] local */
  void* out;                 /* [rows, cols] local */
  int64_t ld_src, ld_add, ld_out;
  int32_t rows, cols;
  int32_t max_ctas;
} qlin_shard_reduce_args;

int qlin_shard_reduce(const qlin_shard_reduce_args* args, void* stream);

typedef struct qlin_peer_barrier_args {
  uint32_t* local_flags;
  uint32_t* peer_flags[8];
  uint32_t* epoch;
  int32_t* status;
  int32_t rank, world;
  int64_t timeout_ns;      /* longest wait in nanoseconds; 0 = the default of 10 s */
} qlin_peer_barrier_args;

int qlin_peer_barrier(const qlin_peer_barrier_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QLIN_B200_H */
