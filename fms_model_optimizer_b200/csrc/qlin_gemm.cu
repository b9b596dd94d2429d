// qlin_gemm: persistent, warp-specialised tcgen05 GEMM for 8-bit operands on sm_100a.
//
//   D[M,N] = epilogue( C + sum over K-chunks of f( A[M,Kc] . B[N,Kc]^T ) )
//
// Both operands are K-major ("NT"), which is the layout the reference hands to its Triton / CUTLASS
// kernels (activations [m,k]; weight [n,k] passed as its .t() view).
//
// Per CTA (one per SM, 320 or 576 threads):
//   warp E      TMA producer (E = number of epilogue warps: 8 unchunked, 16 chunked): 128-byte-swizzled [128 x 128B] A tile and [BN x 128B] B tile per stage
//   warp E+1    MMA issuer: tcgen05.mma.cta_group::1 (M=128, N=BN, K=32 bytes per instruction),
//               accumulators in tensor memory; owns the TMEM allocation
//   warps 0..E-1 epilogue: tcgen05.ld of the accumulator, chunk rounding / running sum, dequantise,
//               global stores.  Warp w reads TMEM lanes 32*(w%4).. and column half w/4.
// Unchunked: BN=256, two 256-column accumulators so the epilogue of tile i overlaps the mainloop of
// tile i+1.  Chunked: BN=128, four 128-column accumulators; every K-chunk is a fresh accumulation
// that the epilogue warps drain, round and add to a running sum held in registers.
//
// Three kernels share this file: the CTA-pair kernel (cta_group::2, unchunked problems of at least 256 rows), the
// single-CTA kernel described above (chunked problems and the shapes in between), and the few-row kernel (at most
// 128 rows: weight rows as the MMA's M dimension, K split over a thread-block cluster).  Environment switches for
// A/B measurements: QLIN_GEMM_PAIR=0, QLIN_GEMM_SKINNY=0, QLIN_GEMM_LOWBYTE=0 select the kernel or mode each replaces.
//
// All mbarrier waits are bounded; a wait that runs out raises an abort flag, the CTA drains its
// copies and MMAs, frees TMEM, writes QLIN_ERR_TIMEOUT to the status word and returns.
#include <cstdlib>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "qlin_internal.h"
#include "qlin_ptx.cuh"

namespace qlin {

constexpr int kBM = 128;          // rows of A per tile = MMA M
constexpr int kBK = 128;          // bytes of K per pipeline stage = one swizzle row
constexpr int kGroupM = 16;       // m-blocks per raster group
constexpr int kTmemCols = 512;
constexpr int kStageOutBytes = 4096;  // per epilogue warp: 32 rows x 128 bytes of output

struct Aux {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tfull[4];
  uint64_t tempty[4];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
  float cs[256];
  float bias[256];
};

template <bool CHUNKED>
struct Cfg {
  static constexpr int BN = CHUNKED ? 128 : 256;
  static constexpr int NBUF = CHUNKED ? 4 : 2;
  static constexpr int STAGES = CHUNKED ? 5 : 4;
  // Epilogue warps: w % 4 selects the 32 TMEM lanes a warp may read, w / 4 its column slice.  The
  // chunked kernel drains an accumulator per K-chunk, a chain of short dependent steps, and hides
  // that latency with twice as many, narrower warps.
  static constexpr int EPI_WARPS = CHUNKED ? 16 : 8;
  static constexpr int PRODUCER_WARP = EPI_WARPS;
  static constexpr int MMA_WARP = EPI_WARPS + 1;
  static constexpr int THREADS = (EPI_WARPS + 2) * 32;
  static constexpr int A_BYTES = kBM * kBK;
  static constexpr int B_BYTES = BN * kBK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int COLS_PER_WARP = BN / (EPI_WARPS / 4);  // 128 (unchunked) or 32 (chunked) columns
  static constexpr int OUT_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int AUX_OFFSET = OUT_OFFSET + EPI_WARPS * kStageOutBytes;
  static constexpr int SMEM_BYTES = AUX_OFFSET + static_cast<int>(sizeof(Aux));
};
static_assert(Cfg<false>::SMEM_BYTES <= 232448 && Cfg<true>::SMEM_BYTES <= 232448, "shared memory budget");

struct GemmParams {
  const void* c;
  void* d;
  const float* rs;
  const float* cs;
  const float* bias;
  int32_t* status;
  int64_t ldc, ldd;
  int32_t M, N;
  int32_t kbytes;      // K in bytes
  int32_t chunk_k32;   // 32-byte MMA steps per accumulation chunk
  int32_t trun_bits, max_acc_bits, trunc_then_acc, clamp_dl16;
  int32_t epilogue, rs_stride, cs_stride, prod_round, scale_round, mid_round, acc_round, out_dtype;
  int32_t num_m, num_n, max_ctas;
  int32_t scatter_rows, scatter_row0;
  uint8_t* scatter_d[8];
  int32_t f8_ab_format;  // float kinds: operand format of the instruction descriptor, 0 = e4m3, 1 = e5m2
  int32_t batch;             // batched launch: problems stacked along the rows of A, B and along D (see qlin_gemm_batched)
  int64_t batch_stride_d;    // elements of the output type between the problems' outputs
  int32_t low_byte_mode;  // chunked int8, 8 truncated bits: the total on the tensor core, the chunks' low bytes on the ALU
  int32_t sk_mt, sk_split, sk_stages;  // few-row kernel: padded row count, K splits (= cluster size), pipeline stages
};

__device__ __forceinline__ float round_to(float y, int dt) {
  if (dt == QLIN_DT_F16) return __half2float(__float2half_rn(y));
  if (dt == QLIN_DT_BF16) return __bfloat162float(__float2bfloat16_rn(y));
  return y;
}

// The per-chunk rounding of the reference kernels.
template <bool F8>
__device__ __forceinline__ uint32_t chunk_round(uint32_t p, bool clamp, int32_t lo, int32_t hi, uint32_t rb,
                                                uint32_t mask, bool dl16) {
  if (!F8) {
    if (clamp) {
      int32_t v = static_cast<int32_t>(p);
      v = v > hi ? hi : v;
      v = v < lo ? lo : v;
      p = static_cast<uint32_t>(v);
    }
    return (p + rb) & mask;
  } else {
    p = (p + rb) & mask;
    if (dl16) {
      float x = __uint_as_float(p);
      const float dl16_max = 8581545984.0f;
      const float dl16_min = 4.665707820095122e-10f;
      if (x >= dl16_max) x = __int_as_float(0x7f800000);
      if (x <= -dl16_max) x = __int_as_float(0xff800000);
      if (fabsf(x) < dl16_min) x = 0.0f;
      p = __float_as_uint(x);
    }
    return p;
  }
}

template <bool F8>
__device__ __forceinline__ uint32_t acc_add(uint32_t a, uint32_t b) {
  if (F8) return __float_as_uint(__fadd_rn(__uint_as_float(a), __uint_as_float(b)));
  return a + b;
}

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& mb, int& nb) {
  const int per_group = kGroupM * num_n;
  const int g = t / per_group;
  const int first_m = g * kGroupM;
  const int gsz = min(num_m - first_m, kGroupM);
  const int r = t - g * per_group;
  mb = first_m + r % gsz;
  nb = r / gsz;
}

// Accumulator -> output value (fp32, already rounded the way the epilogue mode asks).
template <bool F8>
__device__ __forceinline__ float dequant_one(const GemmParams& p, uint32_t v, float rs, float cs, float bias,
                                             bool prod, bool has_bias) {
  const float a = F8 ? __uint_as_float(v) : __int2float_rn(static_cast<int32_t>(v));
  float t;
  if (prod) {
    const float s = round_to(round_to(__fmul_rn(rs, cs), p.prod_round), p.scale_round);
    t = __fmul_rn(a, s);
  } else {
    t = round_to(__fmul_rn(__fmul_rn(a, rs), cs), p.mid_round);
  }
  if (has_bias) t = __fadd_rn(t, bias);
  return round_to(t, p.acc_round);
}

__device__ __forceinline__ uint32_t pack16(const GemmParams& p, float lo, float hi) {
  if (p.out_dtype == QLIN_DT_BF16) {
    return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) |
           (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
  }
  return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(lo))) |
         (static_cast<uint32_t>(__half_as_ushort(__float2half_rn(hi))) << 16);
}

// Byte address of output row `row`, column 0 (`elt` bytes per element).  With row-block scatter the block of
// scatter_rows rows that contains `row` lives in its own buffer (possibly another GPU's).
__device__ __forceinline__ uint8_t* out_row(const GemmParams& p, int row, int elt) {
  if (p.scatter_rows > 0) {
    const int owner = row / p.scatter_rows;
    return p.scatter_d[owner] + static_cast<int64_t>(row - owner * p.scatter_rows + p.scatter_row0) * p.ldd * elt;
  }
  return reinterpret_cast<uint8_t*>(p.d) + static_cast<int64_t>(row) * p.ldd * elt;
}

// Direct (uncoalesced, bounds-checked) store of NC consecutive columns of one row held by this
// thread: the path for ragged right edges and for outputs that rule out 16-byte vectors.
template <bool F8, int NC>
__device__ __forceinline__ void store_row_direct(const GemmParams& p, const uint32_t (&v)[NC], int row, int col0,
                                                 const float* s_cs, const float* s_bias, int s_off, float rs) {
  if (row >= p.M) return;
  const int ncol = min(NC, p.N - col0);
  if (ncol <= 0) return;
  const bool prod = p.epilogue == QLIN_EPI_SCALE_PROD;
  const bool has_bias = p.bias != nullptr;
  const int elt = (p.epilogue == QLIN_EPI_RAW || p.out_dtype == QLIN_DT_F32) ? 4 : 2;
  uint8_t* base = out_row(p, row, elt) + static_cast<int64_t>(col0) * elt;
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    if (j < ncol) {
      if (p.epilogue == QLIN_EPI_RAW) {
        reinterpret_cast<uint32_t*>(base)[j] = v[j];
      } else {
        const float y = dequant_one<F8>(p, v[j], rs, s_cs[s_off + j], s_bias[s_off + j], prod, has_bias);
        if (p.out_dtype == QLIN_DT_F32) {
          reinterpret_cast<float*>(base)[j] = y;
        } else {
          reinterpret_cast<uint16_t*>(base)[j] = static_cast<uint16_t>(pack16(p, y, 0.0f) & 0xFFFFu);
        }
      }
    }
  }
}

// Coalesced store through this warp's 32 x 128-byte staging tile.  `w` holds this thread's row as
// 32 packed 32-bit words (128 bytes).  The tile is written with a 16-byte-chunk XOR swizzle so both
// the row-per-lane writes and the row-contiguous reads are bank-conflict free; every global store
// instruction then covers four full 128-byte lines.
__device__ __forceinline__ void store_tile_coalesced(uint8_t* stage, const uint32_t (&w)[32], uint8_t* gbase,
                                                     int64_t row_pitch_bytes, int rows_valid, int lane) {
  const uint32_t sbase = smem_u32(stage);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t addr = sbase + lane * 128 + ((c ^ (lane & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * c]), "r"(w[4 * c + 1]),
                 "r"(w[4 * c + 2]), "r"(w[4 * c + 3])
                 : "memory");
  }
  __syncwarp();
  const int c = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3);
    uint32_t x0, x1, x2, x3;
    const uint32_t addr = sbase + r * 128 + ((c ^ (r & 7)) << 4);
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(addr) : "memory");
    if (r < rows_valid) *reinterpret_cast<uint4*>(gbase + r * row_pitch_bytes + c * 16) = make_uint4(x0, x1, x2, x3);
  }
  __syncwarp();
}

// Loads NC columns of the optional initial accumulator C for one row (zeros when absent / outside).
template <int NC>
__device__ __forceinline__ void load_c_row(const GemmParams& p, uint32_t (&v)[NC], int row, int col0) {
#pragma unroll
  for (int j = 0; j < NC; ++j) v[j] = 0u;
  if (p.c == nullptr || row >= p.M) return;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(p.c) + static_cast<int64_t>(row) * p.ldc + col0;
#pragma unroll
  for (int j = 0; j < NC; ++j)
    if (col0 + j < p.N) v[j] = src[j];
}

// Emits 64 accumulator columns [col0, col0+64) of this thread's row.  `vec_ok` says the output
// allows 16-byte row-contiguous stores.
template <bool F8>
__device__ __forceinline__ void emit64(const GemmParams& p, const uint32_t (&v)[64], int row0, int lane, int col0,
                                       const float* s_cs, const float* s_bias, int s_off, float rs, bool vec_ok,
                                       uint8_t* stage) {
  const int row = row0 + lane;
  const bool prod = p.epilogue == QLIN_EPI_SCALE_PROD;
  const bool has_bias = p.bias != nullptr;
  const int rows_valid = p.M - row0;
  if (!vec_ok || col0 + 64 > p.N) {
    store_row_direct<F8, 64>(p, v, row, col0, s_cs, s_bias, s_off, rs);
    return;
  }
  if (p.epilogue != QLIN_EPI_RAW && p.out_dtype != QLIN_DT_F32) {
    // 2-byte outputs: 64 columns = one 128-byte staging row
    uint32_t w[32];
    if (prod && p.scale_round == QLIN_DT_F16 && p.acc_round == QLIN_DT_F16 && p.out_dtype == QLIN_DT_BF16 &&
        (p.prod_round == QLIN_DT_BF16 || p.prod_round == QLIN_DT_NONE || p.prod_round == QLIN_DT_F32)) {
      // The deploy Linear's chain, two columns per instruction: s = fp16(bf16?(rs * cs)); y = fp16(acc * s (+ bias));
      // the same roundings as dequant_one, done with packed fp32 arithmetic and packed conversions.
      const bool prod_bf16 = p.prod_round == QLIN_DT_BF16;
      const float2 rs2 = make_float2(rs, rs);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float2 c2 = *reinterpret_cast<const float2*>(s_cs + s_off + 2 * j);
        float2 sc = __fmul2_rn(rs2, c2);
        if (prod_bf16) {
          const __nv_bfloat162 b2 = __float22bfloat162_rn(sc);
          const uint32_t bw = *reinterpret_cast<const uint32_t*>(&b2);
          sc = make_float2(__uint_as_float(bw << 16), __uint_as_float(bw & 0xFFFF0000u));
        }
        sc = __half22float2(__float22half2_rn(sc));
        float2 a2;
        if (F8) {
          a2 = make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
        } else {
          a2 = make_float2(__int2float_rn(static_cast<int32_t>(v[2 * j])), __int2float_rn(static_cast<int32_t>(v[2 * j + 1])));
        }
        float2 t = __fmul2_rn(a2, sc);
        if (has_bias) t = __fadd2_rn(t, *reinterpret_cast<const float2*>(s_bias + s_off + 2 * j));
        t = __half22float2(__float22half2_rn(t));
        const __nv_bfloat162 o2 = __float22bfloat162_rn(t);
        w[j] = *reinterpret_cast<const uint32_t*>(&o2);
      }
    } else if (!prod && p.out_dtype == QLIN_DT_BF16 && (p.mid_round == QLIN_DT_BF16 || p.mid_round == QLIN_DT_NONE) &&
               (p.acc_round == QLIN_DT_BF16 || p.acc_round == QLIN_DT_NONE)) {
      // (acc * rs) * cs, optional bf16 rounding, + bias, bf16: the chain of the FP8 Linear and of the fused ops, two columns
      // per instruction; the final packed conversion is the last rounding
      const bool mid_bf16 = p.mid_round == QLIN_DT_BF16;
      const float2 rs2 = make_float2(rs, rs);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float2 a2;
        if (F8) {
          a2 = make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
        } else {
          a2 = make_float2(__int2float_rn(static_cast<int32_t>(v[2 * j])), __int2float_rn(static_cast<int32_t>(v[2 * j + 1])));
        }
        float2 t = __fmul2_rn(__fmul2_rn(a2, rs2), *reinterpret_cast<const float2*>(s_cs + s_off + 2 * j));
        if (has_bias) {
          if (mid_bf16) {
            const __nv_bfloat162 b2 = __float22bfloat162_rn(t);
            const uint32_t bw = *reinterpret_cast<const uint32_t*>(&b2);
            t = make_float2(__uint_as_float(bw << 16), __uint_as_float(bw & 0xFFFF0000u));
          }
          t = __fadd2_rn(t, *reinterpret_cast<const float2*>(s_bias + s_off + 2 * j));
        }
        const __nv_bfloat162 o2 = __float22bfloat162_rn(t);
        w[j] = *reinterpret_cast<const uint32_t*>(&o2);
      }
    } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float y0 = dequant_one<F8>(p, v[2 * j], rs, s_cs[s_off + 2 * j], s_bias[s_off + 2 * j], prod, has_bias);
      const float y1 =
          dequant_one<F8>(p, v[2 * j + 1], rs, s_cs[s_off + 2 * j + 1], s_bias[s_off + 2 * j + 1], prod, has_bias);
      w[j] = pack16(p, y0, y1);
    }
    }
    uint8_t* g = out_row(p, row0, 2) + static_cast<int64_t>(col0) * 2;
    store_tile_coalesced(stage, w, g, p.ldd * 2, rows_valid, lane);
  } else {
    // 4-byte outputs: two staging passes of 32 columns
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t w[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int k = h * 32 + j;
        w[j] = p.epilogue == QLIN_EPI_RAW
                   ? v[k]
                   : __float_as_uint(dequant_one<F8>(p, v[k], rs, s_cs[s_off + k], s_bias[s_off + k], prod, has_bias));
      }
      uint8_t* g = out_row(p, row0, 4) + static_cast<int64_t>(col0 + h * 32) * 4;
      store_tile_coalesced(stage, w, g, p.ldd * 4, rows_valid, lane);
    }
  }
}

// Emits 32 accumulator columns of this thread's row (the chunked kernel's final store): 4-byte
// outputs go through the coalescing tile, 2-byte outputs (64 bytes per row) are stored directly.
template <bool F8>
__device__ __forceinline__ void emit32(const GemmParams& p, const uint32_t (&v)[32], int row0, int lane, int col0,
                                       const float* s_cs, const float* s_bias, int s_off, float rs, bool vec_ok,
                                       uint8_t* stage) {
  const bool four_byte = p.epilogue == QLIN_EPI_RAW || p.out_dtype == QLIN_DT_F32;
  if (!vec_ok || col0 + 32 > p.N || !four_byte) {
    store_row_direct<F8, 32>(p, v, row0 + lane, col0, s_cs, s_bias, s_off, rs);
    return;
  }
  const bool prod = p.epilogue == QLIN_EPI_SCALE_PROD;
  const bool has_bias = p.bias != nullptr;
  uint32_t w[32];
#pragma unroll
  for (int j = 0; j < 32; ++j)
    w[j] = p.epilogue == QLIN_EPI_RAW
               ? v[j]
               : __float_as_uint(dequant_one<F8>(p, v[j], rs, s_cs[s_off + j], s_bias[s_off + j], prod, has_bias));
  uint8_t* g = out_row(p, row0, 4) + static_cast<int64_t>(col0) * 4;
  store_tile_coalesced(stage, w, g, p.ldd * 4, p.M - row0, lane);
}

// BATCHED: p.batch problems of the same shape whose operands are stacked along the rows (A is [batch * M, K], B is
// [batch * N, K]); a tile of problem b starts at row b * M of A and row b * N of B, its rows and columns beyond the
// problem's M and N belong to the next problem (or lie outside and read as zeros) and are dropped by the epilogue's
// bounds checks, and its output goes to D + b * batch_stride_d.
template <bool F8, bool CHUNKED, bool BATCHED = false>
__global__ void __launch_bounds__(Cfg<CHUNKED>::THREADS, 1)
qlin_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  using C = Cfg<CHUNKED>;
  extern __shared__ __align__(1024) uint8_t smem[];
  Aux* aux = reinterpret_cast<Aux*>(smem + C::AUX_OFFSET);
  volatile int* abort_flag = &aux->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // The 128-byte swizzle atoms need a 1024-byte aligned base; dynamic shared memory starts at the
  // base of the CTA's window, so this only guards against a toolchain that would place it elsewhere.
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, static_cast<int32_t>(QLIN_ERR_BAD_ALIGN));
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&aux->full[s], 1);
      mbar_init(&aux->empty[s], 1);
    }
    for (int b = 0; b < C::NBUF; ++b) {
      mbar_init(&aux->tfull[b], 1);
      mbar_init(&aux->tempty[b], C::EPI_WARPS);
    }
    mbar_init(&aux->drain, 1);
    aux->abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == C::MMA_WARP) {
    tmem_alloc(&aux->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  if (warp == C::PRODUCER_WARP && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = aux->tmem_base;

  const int per_batch = p.num_m * p.num_n;
  const int num_tiles = BATCHED ? per_batch * p.batch : per_batch;
  const int num_kb = (p.kbytes + kBK - 1) / kBK;
  const int total_k32 = (p.kbytes + 31) / 32;
  bool timed_out = false;

  if (warp == C::PRODUCER_WARP) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the loop converged; one elected lane issues.  The next stage's
    // barrier is polled (non-blocking) before the current stage is issued, which takes the
    // barrier round trip off the loop's critical path.
    uint32_t s = 0, ph = 0, issued = 0;
    bool ok = true;
    bool ready = false;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int mb, nb;
      const int bi = BATCHED ? t / per_batch : 0;
      tile_coords(t - bi * per_batch, p.num_m, p.num_n, mb, nb);
      const int ya = mb * kBM + bi * p.M, yb = nb * C::BN + bi * p.N;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!ready) {
          ok = warp_mbar_wait(&aux->empty[s], ph ^ 1u, abort_flag);
          if (!ok) break;
        }
        const uint32_t ns = (s + 1 == C::STAGES) ? 0u : s + 1;
        const uint32_t nph = (ns == 0u) ? (ph ^ 1u) : ph;
        const uint32_t peek = warp_mbar_test_begin(&aux->empty[ns], nph ^ 1u);
        uint8_t* sa = smem + s * C::STAGE_BYTES;
        tma_issue_stage(&aux->full[s], C::STAGE_BYTES, sa, &tmap_a, ya, sa + C::A_BYTES, &tmap_b, yb, kb * kBK);
        ++issued;
        ready = warp_mbar_test_end(peek);
        s = ns;
        ph = nph;
      }
    }
    if (!ok) {
      if (lane == 0) {
        timed_out = !*abort_flag;
        *abort_flag = 1;
      }
      // Let the copies already issued land before the CTA gives its shared memory back.
      for (uint32_t st = 0; st < static_cast<uint32_t>(C::STAGES); ++st) {
        if (issued <= st) continue;
        const uint32_t last = ((issued - 1 - st) / C::STAGES);  // index of the last fill of stage st
        mbar_wait_drain(&aux->full[st], last & 1u);
      }
    }
    __syncwarp();
  } else if (warp == C::MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    // One instruction stream feeds the tensor pipe, so this loop is latency-critical: no
    // divisions, positions carried as counters, a whole 128-byte K block issued by one fused
    // statement, and the next stage's barrier polled before the current block is issued.
    const uint32_t idesc = F8 ? make_idesc(1u, static_cast<uint32_t>(p.f8_ab_format), kBM, C::BN) : make_idesc(2u, 1u, kBM, C::BN);
    const uint64_t adesc0 = make_smem_desc_sw128(smem_u32(smem));
    const uint64_t bdesc0 = make_smem_desc_sw128(smem_u32(smem) + C::A_BYTES);
    uint32_t s = 0, ph = 0;          // smem stage and its phase
    uint32_t buf = 0, bph = 0;       // TMEM accumulator buffer to use next and its phase
    bool ok = true;
    bool ready = false;
    bool tready = false;  // next accumulator buffer known to be drained
    // chunks that tile a 128-byte K block exactly (32, 64 or 128 elements, K a multiple of 128)
    const bool chunk_fast = CHUNKED && (p.chunk_k32 == 1 || p.chunk_k32 == 2 || p.chunk_k32 == 4) && (total_k32 % 4 == 0);
    // low-byte mode: the last accumulator holds the tile's untruncated total, the others rotate over the chunks
    const bool low_mode = CHUNKED && !F8 && p.low_byte_mode != 0;
    const uint32_t nbuf = low_mode ? C::NBUF - 1 : C::NBUF;
    const uint32_t d_total = tmem_base + (C::NBUF - 1) * C::BN;
    uint32_t tot_ph = 0;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      uint32_t accumulate = 0, cur = 0;
      if (low_mode) {
        // the epilogue warps must have read the previous tile's total before it is overwritten
        ok = warp_mbar_wait(&aux->tempty[C::NBUF - 1], tot_ph ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        tot_ph ^= 1u;
      }
      int chunk_pos = 0;
      int k32_left = total_k32;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        if (!ready) {
          ok = warp_mbar_wait(&aux->full[s], ph, abort_flag);
          if (!ok) break;
        }
        tc_fence_after();
        const uint32_t ns = (s + 1 == C::STAGES) ? 0u : s + 1;
        const uint32_t nph = (ns == 0u) ? (ph ^ 1u) : ph;
        const uint32_t peek = warp_mbar_test_begin(&aux->full[ns], nph);
        const uint64_t adesc = adesc0 + static_cast<uint64_t>(s * (C::STAGE_BYTES >> 4));
        const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(s * (C::STAGE_BYTES >> 4));
        if (!CHUNKED && k32_left >= 4) {
          if (kb == 0) {
            ok = warp_mbar_wait(&aux->tempty[buf], bph ^ 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
            cur = buf;
            if (++buf == C::NBUF) {
              buf = 0;
              bph ^= 1u;
            }
          }
          tc_mma4_release<F8 ? 1 : 0>(tmem_base + cur * C::BN, adesc, bdesc, idesc, accumulate, &aux->empty[s]);
          accumulate = 1;
          k32_left -= 4;
          if (k32_left == 0) tc_commit_elect(&aux->tfull[cur]);
        } else if (CHUNKED && chunk_fast && k32_left >= 4) {
          // whole chunks inside this 128-byte K block: one fused statement per chunk, the next
          // accumulator's "empty" barrier polled before the current chunk is issued
          const int cpk = 4 / p.chunk_k32;
          for (int c = 0; c < cpk && ok; ++c) {
            if (!tready) {
              ok = warp_mbar_wait(&aux->tempty[buf], bph ^ 1u, abort_flag);
              if (!ok) break;
            }
            tc_fence_after();
            const uint32_t nb = (buf + 1 == nbuf) ? 0u : buf + 1;
            const uint32_t nbph = (nb == 0u) ? (bph ^ 1u) : bph;
            const uint32_t tpeek = warp_mbar_test_begin(&aux->tempty[nb], nbph ^ 1u);
            const uint64_t off = static_cast<uint64_t>(c * p.chunk_k32 * 2);
            const uint32_t d = tmem_base + buf * C::BN;
            if constexpr (CHUNKED && !F8) {
              if (low_mode) {
                const uint32_t acc_total = (kb == 0 && c == 0) ? 0u : 1u;
                if (p.chunk_k32 == 1) {
                  tc_mma_chunk_and_total_i8<1>(d, d_total, adesc + off, bdesc + off, idesc, acc_total, &aux->tfull[buf]);
                } else if (p.chunk_k32 == 2) {
                  tc_mma_chunk_and_total_i8<2>(d, d_total, adesc + off, bdesc + off, idesc, acc_total, &aux->tfull[buf]);
                } else {
                  tc_mma_chunk_and_total_i8<4>(d, d_total, adesc + off, bdesc + off, idesc, acc_total, &aux->tfull[buf]);
                }
                tready = warp_mbar_test_end(tpeek);
                buf = nb;
                bph = nbph;
                continue;
              }
            }
            if (p.chunk_k32 == 1) {
              tc_mma_chunk<F8 ? 1 : 0, 1>(d, adesc + off, bdesc + off, idesc, &aux->tfull[buf]);
            } else if (p.chunk_k32 == 2) {
              tc_mma_chunk<F8 ? 1 : 0, 2>(d, adesc + off, bdesc + off, idesc, &aux->tfull[buf]);
            } else {
              tc_mma_chunk<F8 ? 1 : 0, 4>(d, adesc + off, bdesc + off, idesc, &aux->tfull[buf]);
            }
            tready = warp_mbar_test_end(tpeek);
            buf = nb;
            bph = nbph;
          }
          k32_left -= 4;
          if (ok) tc_commit_elect(&aux->empty[s]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (k32_left > 0 && ok) {
              if (chunk_pos == 0 && (CHUNKED || accumulate == 0)) {
                ok = warp_mbar_wait(&aux->tempty[buf], bph ^ 1u, abort_flag);
                if (ok) {
                  tc_fence_after();
                  cur = buf;
                  accumulate = 0;
                  if (++buf == C::NBUF) {
                    buf = 0;
                    bph ^= 1u;
                  }
                }
              }
              if (ok) {
                ++chunk_pos;
                --k32_left;
                const bool last_of_chunk = chunk_pos == p.chunk_k32 || k32_left == 0;
                tc_mma1<F8 ? 1 : 0>(tmem_base + cur * C::BN, adesc + static_cast<uint64_t>(j * 2),
                                    bdesc + static_cast<uint64_t>(j * 2), idesc, accumulate);
                if (last_of_chunk) tc_commit_elect(&aux->tfull[cur]);
                accumulate = 1;
                if (last_of_chunk) chunk_pos = 0;
              }
            }
          }
          if (ok) tc_commit_elect(&aux->empty[s]);
        }
        ready = warp_mbar_test_end(peek);
        s = ns;
        ph = nph;
      }
    }
    if (!ok && lane == 0) {
      timed_out = !*abort_flag;
      *abort_flag = 1;
    }
    // Nothing may still be reading shared memory or writing TMEM when the CTA retires.
    tc_commit_elect(&aux->drain);
    mbar_wait_drain(&aux->drain, 0);
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;
    const int half = warp >> 2;  // column slice of this warp
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* stage = smem + C::OUT_OFFSET + warp * kStageOutBytes;
    const int elt = (p.out_dtype == QLIN_DT_F16 || p.out_dtype == QLIN_DT_BF16) ? 2 : 4;
    const bool vec_ok = (p.scatter_rows > 0 || (reinterpret_cast<uintptr_t>(p.d) & 15u) == 0) && ((p.ldd * elt) % 16 == 0);
    const bool clamp = !F8 && p.max_acc_bits < 32;
    const int32_t lo = clamp ? -(1 << (p.max_acc_bits - 1)) : 0;
    const int32_t hi = clamp ? (1 << (p.max_acc_bits - 1)) - 1 : 0;
    const uint32_t rb = p.trun_bits > 0 ? (1u << (p.trun_bits - 1)) : 0u;
    const uint32_t mask = p.trun_bits > 0 ? ~((1u << p.trun_bits) - 1u) : 0xFFFFFFFFu;
    const bool dl16 = F8 && p.clamp_dl16;
    const bool scaled = p.epilogue != QLIN_EPI_RAW;
    uint32_t ebuf = 0, ebph = 0;
    bool eready = false;
    bool ok = true;
    const bool elow = CHUNKED && !F8 && p.low_byte_mode != 0;
    const uint32_t enbuf = elow ? C::NBUF - 1 : C::NBUF;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int mb, nb;
      const int bi = BATCHED ? t / per_batch : 0;
      tile_coords(t - bi * per_batch, p.num_m, p.num_n, mb, nb);
      GemmParams pb;
      const GemmParams* pp = &p;
      if constexpr (BATCHED) {
        pb = p;
        pb.d = static_cast<uint8_t*>(p.d) + static_cast<int64_t>(bi) * p.batch_stride_d * elt;
        pp = &pb;
      }
      const GemmParams& pe = *pp;
      const int row0 = mb * kBM + q * 32;
      const int row = row0 + lane;
      const int col_w = nb * C::BN + half * C::COLS_PER_WARP;
      float rs = 1.0f;
      if (scaled) {
        // Stage this tile's column scales and bias once; all lanes then read them as broadcasts.
        asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_WARPS * 32) : "memory");
        for (int i = threadIdx.x; i < C::BN; i += C::EPI_WARPS * 32) {
          const int n = nb * C::BN + i;
          aux->cs[i] = (p.cs != nullptr && n < p.N) ? p.cs[static_cast<int64_t>(n) * p.cs_stride] : 1.0f;
          aux->bias[i] = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.0f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_WARPS * 32) : "memory");
        if (p.rs != nullptr && row < p.M) rs = p.rs[static_cast<int64_t>(row) * p.rs_stride];
      }
      if constexpr (!CHUNKED) {
        const uint32_t buf = ebuf, bph = ebph;
        if (++ebuf == C::NBUF) {
          ebuf = 0;
          ebph ^= 1u;
        }
        if (!warp_mbar_wait(&aux->tfull[buf], bph, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll 1
        for (int j = 0; j < C::COLS_PER_WARP; j += 64) {
          uint32_t v[64];
          tmem_ld64(tmem_base + lane_base + buf * C::BN + half * C::COLS_PER_WARP + j, v);
          if (p.c != nullptr) {
            uint32_t cv[64];
            load_c_row<64>(p, cv, row, col_w + j);
#pragma unroll
            for (int i = 0; i < 64; ++i) v[i] = acc_add<F8>(cv[i], v[i]);
          }
          emit64<F8>(pe, v, row0, lane, col_w + j, aux->cs, aux->bias, half * C::COLS_PER_WARP + j, rs, vec_ok, stage);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&aux->tempty[buf]);
      } else {
        uint32_t run[C::COLS_PER_WARP];
        load_c_row<C::COLS_PER_WARP>(p, run, row, col_w);
        int k32_left = total_k32;
#pragma unroll 1
        while (k32_left > 0) {
          k32_left -= p.chunk_k32;
          const uint32_t buf = ebuf, bph = ebph;
          if (++ebuf == enbuf) {
            ebuf = 0;
            ebph ^= 1u;
          }
          if (!eready && !warp_mbar_wait(&aux->tfull[buf], bph, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (elow) {
            // ((p + 128) >> 8) << 8 = p - sext8(low byte of p): the sum of the chunks is the untruncated total (kept by
            // the tensor core in its own accumulator) minus the sum of the sign-extended low bytes.  Only the low bits
            // of the chunk's accumulator are read (two columns per register), one dp4a per element picks its byte.
            uint32_t v16[C::COLS_PER_WARP / 2];
            tmem_ld32_low16(tmem_base + lane_base + buf * C::BN + half * C::COLS_PER_WARP, v16);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&aux->tempty[buf]);
            const uint32_t epeek = warp_mbar_test_begin(&aux->tfull[ebuf], ebph);
#pragma unroll
            for (int i = 0; i < C::COLS_PER_WARP / 2; ++i) {
              run[2 * i] = static_cast<uint32_t>(__dp4a(static_cast<int>(v16[i]), 0x000000FF, static_cast<int>(run[2 * i])));
              run[2 * i + 1] = static_cast<uint32_t>(__dp4a(static_cast<int>(v16[i]), 0x00FF0000, static_cast<int>(run[2 * i + 1])));
            }
            eready = warp_mbar_test_end(epeek);
            continue;
          }
          uint32_t v[C::COLS_PER_WARP];
          tmem_ld32(tmem_base + lane_base + buf * C::BN + half * C::COLS_PER_WARP, v);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&aux->tempty[buf]);
          // poll the next chunk's barrier now; the answer is consumed after this chunk's arithmetic
          const uint32_t epeek = warp_mbar_test_begin(&aux->tfull[ebuf], ebph);
          if (p.trunc_then_acc && !clamp && !dl16) {
            // the common case, kept free of per-element predicates: run += (p + rb) & mask
#pragma unroll
            for (int i = 0; i < C::COLS_PER_WARP; ++i) run[i] = acc_add<F8>(run[i], (v[i] + rb) & mask);
          } else if (p.trunc_then_acc) {
#pragma unroll
            for (int i = 0; i < C::COLS_PER_WARP; ++i)
              run[i] = acc_add<F8>(run[i], chunk_round<F8>(v[i], clamp, lo, hi, rb, mask, dl16));
          } else {
#pragma unroll
            for (int i = 0; i < C::COLS_PER_WARP; ++i)
              run[i] = chunk_round<F8>(acc_add<F8>(run[i], v[i]), clamp, lo, hi, rb, mask, dl16);
          }
          eready = warp_mbar_test_end(epeek);
        }
        if (!ok) break;
        if (elow) {
          // the last chunk's commit covers every MMA of the tile: the total is complete
          uint32_t tot[C::COLS_PER_WARP];
          tmem_ld32(tmem_base + lane_base + (C::NBUF - 1) * C::BN + half * C::COLS_PER_WARP, tot);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&aux->tempty[C::NBUF - 1]);
#pragma unroll
          for (int i = 0; i < C::COLS_PER_WARP; ++i) run[i] += tot[i];
        }
        if (!ok) break;
        emit32<F8>(p, run, row0, lane, col_w, aux->cs, aux->bias, half * C::COLS_PER_WARP, rs, vec_ok, stage);
      }
    }
    if (!ok && lane == 0) {
      timed_out = !*abort_flag;
      *abort_flag = 1;
    }
  }

  if (timed_out && p.status != nullptr) atomicExch(p.status, static_cast<int32_t>(QLIN_ERR_TIMEOUT));
  tc_fence_before();
  __syncthreads();
  if (warp == C::MMA_WARP) {
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant of the unchunked kernel (cta_group::2).  A cluster of two CTAs computes a
// 256 x 256 tile: CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and of the B tile
// into its own shared memory (32 KB per stage instead of 48 KB for the same MMA work per SM, so six
// stages fit and the L2 -> SM traffic per operation drops by a third), the even CTA issues the MMAs
// for both, and each CTA drains its own 128 accumulator rows.  Barriers:
//   full[s]   leader's copy: 1 arrival (the leader's expect_tx) + the bytes of both CTAs' loads
//   empty[s]  every CTA's own copy, arrived on by the leader's commit (two-CTA mask)
//   tfull[b]  every CTA's own copy, arrived on by the leader's commit (two-CTA mask)
//   tempty[b] leader's copy: one arrival per epilogue warp of both CTAs
// ------------------------------------------------------------------------------------------------
struct PairCfg {
  static constexpr int BN = 256;
  static constexpr int NBUF = 2;
  static constexpr int STAGES = 6;
  static constexpr int EPI_WARPS = 8;
  static constexpr int PRODUCER_WARP = EPI_WARPS;
  static constexpr int MMA_WARP = EPI_WARPS + 1;
  static constexpr int THREADS = (EPI_WARPS + 2) * 32;
  static constexpr int A_BYTES = kBM * kBK;        // this CTA's 128 rows of A
  static constexpr int B_BYTES = (BN / 2) * kBK;   // this CTA's 128 rows of B
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int COLS_PER_WARP = BN / (EPI_WARPS / 4);
  static constexpr int OUT_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int AUX_OFFSET = OUT_OFFSET + EPI_WARPS * kStageOutBytes;
  static constexpr int SMEM_BYTES = AUX_OFFSET + static_cast<int>(sizeof(Aux));
};
static_assert(PairCfg::SMEM_BYTES <= 232448, "shared memory budget");
constexpr int kGroupM2 = 8;  // 256-row blocks per raster group

__device__ __forceinline__ void tile_coords2(int t, int num_m, int num_n, int& mb, int& nb) {
  const int per_group = kGroupM2 * num_n;
  const int g = t / per_group;
  const int first_m = g * kGroupM2;
  const int gsz = min(num_m - first_m, kGroupM2);
  const int r = t - g * per_group;
  mb = first_m + r % gsz;
  nb = r / gsz;
}

template <bool F8>
__global__ void __launch_bounds__(PairCfg::THREADS, 1)
qlin_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  using C = PairCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  Aux* aux = reinterpret_cast<Aux*>(smem + C::AUX_OFFSET);
  volatile int* abort_flag = &aux->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const bool aligned = (smem_u32(smem) & 1023u) == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&aux->full[s], 1);
      mbar_init(&aux->empty[s], 1);
    }
    for (int b = 0; b < C::NBUF; ++b) {
      mbar_init(&aux->tfull[b], 1);
      mbar_init(&aux->tempty[b], 2 * C::EPI_WARPS);
    }
    mbar_init(&aux->drain, 1);
    aux->abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == C::MMA_WARP) {
    tmem_alloc_pair(&aux->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  if (warp == C::PRODUCER_WARP && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive_wait();  // both CTAs' barriers exist before either touches the other's
  tc_fence_after();
  const uint32_t tmem_base = aux->tmem_base;

  const int num_m2 = (p.M + 2 * kBM - 1) / (2 * kBM);
  const int num_tiles = num_m2 * p.num_n;
  const int num_kb = (p.kbytes + kBK - 1) / kBK;
  const int total_k32 = (p.kbytes + 31) / 32;
  bool timed_out = false;

  if (!aligned) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, static_cast<int32_t>(QLIN_ERR_BAD_ALIGN));
  } else if (warp == C::PRODUCER_WARP) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    uint32_t s = 0, ph = 0;
    bool ok = true, ready = false;
    for (int t = pair; t < num_tiles && ok; t += num_pairs) {
      int mb, nb;
      tile_coords2(t, num_m2, p.num_n, mb, nb);
      const int ya = mb * 2 * kBM + static_cast<int>(rank) * kBM;
      const int yb = nb * C::BN + static_cast<int>(rank) * (C::BN / 2);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!ready) {
          ok = warp_mbar_wait(&aux->empty[s], ph ^ 1u, abort_flag);
          if (!ok) break;
        }
        const uint32_t ns = (s + 1 == C::STAGES) ? 0u : s + 1;
        const uint32_t nph = (ns == 0u) ? (ph ^ 1u) : ph;
        const uint32_t peek = warp_mbar_test_begin(&aux->empty[ns], nph ^ 1u);
        uint8_t* sa = smem + s * C::STAGE_BYTES;
        tma_issue_stage_pair(map_to_cta(&aux->full[s], 0), leader, 2 * C::STAGE_BYTES, sa, &tmap_a, ya, sa + C::A_BYTES, &tmap_b, yb,
                             kb * kBK);
        ready = warp_mbar_test_end(peek);
        s = ns;
        ph = nph;
      }
    }
    if (!ok && lane == 0) {
      timed_out = !*abort_flag;
      *abort_flag = 1;
    }
    __syncwarp();
  } else if (warp == C::MMA_WARP) {
    if (leader) {
      // ---------------------------------------------------------------- MMA issuer (leader only)
      const uint32_t idesc = F8 ? make_idesc(1u, static_cast<uint32_t>(p.f8_ab_format), 2 * kBM, C::BN) : make_idesc(2u, 1u, 2 * kBM, C::BN);
      const uint64_t adesc0 = make_smem_desc_sw128(smem_u32(smem));
      const uint64_t bdesc0 = make_smem_desc_sw128(smem_u32(smem) + C::A_BYTES);
      uint32_t s = 0, ph = 0, buf = 0, bph = 0;
      bool ok = true, ready = false;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        uint32_t accumulate = 0, cur = 0;
        int k32_left = total_k32;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          if (!ready) {
            ok = warp_mbar_wait(&aux->full[s], ph, abort_flag);
            if (!ok) break;
          }
          tc_fence_after();
          const uint32_t ns = (s + 1 == C::STAGES) ? 0u : s + 1;
          const uint32_t nph = (ns == 0u) ? (ph ^ 1u) : ph;
          const uint32_t peek = warp_mbar_test_begin(&aux->full[ns], nph);
          const uint64_t adesc = adesc0 + static_cast<uint64_t>(s * (C::STAGE_BYTES >> 4));
          const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(s * (C::STAGE_BYTES >> 4));
          if (kb == 0) {
            ok = warp_mbar_wait(&aux->tempty[buf], bph ^ 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
            cur = buf;
            if (++buf == C::NBUF) {
              buf = 0;
              bph ^= 1u;
            }
          }
          if (k32_left >= 4) {
            tc_mma4_release_pair<F8 ? 1 : 0>(tmem_base + cur * C::BN, adesc, bdesc, idesc, accumulate, &aux->empty[s]);
            accumulate = 1;
            k32_left -= 4;
          } else {
            for (int j = 0; j < k32_left; ++j) {
              tc_mma1_pair<F8 ? 1 : 0>(tmem_base + cur * C::BN, adesc + static_cast<uint64_t>(j * 2), bdesc + static_cast<uint64_t>(j * 2),
                                       idesc, accumulate);
              accumulate = 1;
            }
            k32_left = 0;
            tc_commit_pair_elect(&aux->empty[s]);
          }
          if (k32_left == 0) tc_commit_pair_elect(&aux->tfull[cur]);
          ready = warp_mbar_test_end(peek);
          s = ns;
          ph = nph;
        }
      }
      if (!ok && lane == 0) {
        timed_out = !*abort_flag;
        *abort_flag = 1;
      }
      // Nothing of the pair may still be reading shared memory or writing TMEM when the CTAs retire.
      tc_commit_pair_elect(&aux->drain);
      mbar_wait_drain(&aux->drain, 0);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps (both CTAs)
    const int q = warp & 3;
    const int half = warp >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* stage = smem + C::OUT_OFFSET + warp * kStageOutBytes;
    const int elt = (p.out_dtype == QLIN_DT_F16 || p.out_dtype == QLIN_DT_BF16) ? 2 : 4;
    const bool vec_ok = (p.scatter_rows > 0 || (reinterpret_cast<uintptr_t>(p.d) & 15u) == 0) && ((p.ldd * elt) % 16 == 0);
    const bool scaled = p.epilogue != QLIN_EPI_RAW;
    uint32_t ebuf = 0, ebph = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs) {
      int mb, nb;
      tile_coords2(t, num_m2, p.num_n, mb, nb);
      const int row0 = mb * 2 * kBM + static_cast<int>(rank) * kBM + q * 32;
      const int row = row0 + lane;
      const int col_w = nb * C::BN + half * C::COLS_PER_WARP;
      float rs = 1.0f;
      if (scaled) {
        asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_WARPS * 32) : "memory");
        for (int i = threadIdx.x; i < C::BN; i += C::EPI_WARPS * 32) {
          const int n = nb * C::BN + i;
          aux->cs[i] = (p.cs != nullptr && n < p.N) ? p.cs[static_cast<int64_t>(n) * p.cs_stride] : 1.0f;
          aux->bias[i] = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.0f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_WARPS * 32) : "memory");
        if (p.rs != nullptr && row < p.M) rs = p.rs[static_cast<int64_t>(row) * p.rs_stride];
      }
      const uint32_t buf = ebuf, bph = ebph;
      if (++ebuf == C::NBUF) {
        ebuf = 0;
        ebph ^= 1u;
      }
      if (!warp_mbar_wait(&aux->tfull[buf], bph, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll 1
      for (int j = 0; j < C::COLS_PER_WARP; j += 64) {
        uint32_t v[64];
        tmem_ld64(tmem_base + lane_base + buf * C::BN + half * C::COLS_PER_WARP + j, v);
        if (p.c != nullptr) {
          uint32_t cv[64];
          load_c_row<64>(p, cv, row, col_w + j);
#pragma unroll
          for (int i = 0; i < 64; ++i) v[i] = acc_add<F8>(cv[i], v[i]);
        }
        emit64<F8>(p, v, row0, lane, col_w + j, aux->cs, aux->bias, half * C::COLS_PER_WARP + j, rs, vec_ok, stage);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&aux->tempty[buf], 0));
    }
    if (!ok && lane == 0) {
      timed_out = !*abort_flag;
      *abort_flag = 1;
    }
  }

  if (timed_out && p.status != nullptr) atomicExch(p.status, static_cast<int32_t>(QLIN_ERR_TIMEOUT));
  if (*abort_flag) {
    // a wait gave up: copies of this CTA may still be in flight; give them time to land before the
    // shared memory is handed back
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(256);
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive_wait();
  if (warp == C::MMA_WARP) {
    __syncwarp();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// Few-row kernel (M <= 128, unchunked): the decode-time shapes, where the weight matrix is read once
// and everything else is small.  The operands swap roles: 128 rows of the WEIGHT are the MMA's M
// dimension and the M activation rows, padded to a multiple of 32, are its N dimension, so a K block
// costs 128 x MT x 128 multiply-adds of tensor time instead of the 128 x 256 x 128 a weight-as-B tile
// costs whatever M is, and the kernel runs at the rate the weights stream in.  One CTA per
// (128 output channels, K split); the CTAs of one channel block form a cluster, park their partial
// accumulators in their own shared memory, and after a cluster barrier CTA r sums rows r, r+S, ...
// over the splits in split order through distributed shared memory (a fixed order: the result does not
// depend on scheduling), dequantises and stores them.  Accumulator lane = output channel, so the
// stores of one row are contiguous across the warp.
//   warps 0-3  epilogue (TMEM lanes 32 w ..), warp 4 TMA producer, warp 5 MMA issuer / TMEM owner
// ------------------------------------------------------------------------------------------------
constexpr int kSkEpiWarps = 8;  // warp w reads TMEM lanes 32 (w % 4) .., half w / 4 of the 32-row groups
constexpr int kSkProducerWarp = kSkEpiWarps;
constexpr int kSkMmaWarp = kSkEpiWarps + 1;
constexpr int kSkThreads = (kSkEpiWarps + 2) * 32;
constexpr int kSkWBytes = kBM * kBK;  // 128 weight rows x 128 bytes of K per stage
constexpr int kSkTmemCols = 128;

template <bool F8>
__device__ __forceinline__ void skinny_emit(const GemmParams& p, uint32_t v, int m, int n, float rs, float cs, float bias,
                                            bool prod, bool has_bias) {
  if (p.c != nullptr) v = acc_add<F8>(reinterpret_cast<const uint32_t*>(p.c)[static_cast<int64_t>(m) * p.ldc + n], v);
  if (p.epilogue == QLIN_EPI_RAW) {
    reinterpret_cast<uint32_t*>(p.d)[static_cast<int64_t>(m) * p.ldd + n] = v;
    return;
  }
  const float y = dequant_one<F8>(p, v, rs, cs, bias, prod, has_bias);
  if (p.out_dtype == QLIN_DT_F32) {
    reinterpret_cast<float*>(p.d)[static_cast<int64_t>(m) * p.ldd + n] = y;
  } else {
    reinterpret_cast<uint16_t*>(p.d)[static_cast<int64_t>(m) * p.ldd + n] = static_cast<uint16_t>(pack16(p, y, 0.0f) & 0xFFFFu);
  }
}

// Sum of one accumulator element over the NS splits, in split order; the loads are issued together.
template <bool F8, int NS>
__device__ __forceinline__ uint32_t skinny_sum_splits(const uint32_t* src) {
  uint32_t t[NS];
#pragma unroll
  for (int q = 0; q < NS; ++q) t[q] = ld_cluster_u32(map_to_cta(src, static_cast<uint32_t>(q)));
  uint32_t acc = t[0];
#pragma unroll
  for (int q = 1; q < NS; ++q) acc = acc_add<F8>(acc, t[q]);
  return acc;
}

template <bool F8>
__global__ void __launch_bounds__(kSkThreads, 1)
qlin_gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int MT = p.sk_mt, S = p.sk_split, STG = p.sk_stages;
  const int stage_bytes = kSkWBytes + MT * kBK;
  Aux* aux = reinterpret_cast<Aux*>(smem + STG * stage_bytes);
  volatile int* abort_flag = &aux->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile = blockIdx.x / S;
  const int sp = S > 1 ? static_cast<int>(cluster_cta_rank()) : 0;
  const int num_kb = (p.kbytes + kBK - 1) / kBK;
  const int kb0 = static_cast<int>(static_cast<int64_t>(sp) * num_kb / S);
  const int kb1 = static_cast<int>(static_cast<int64_t>(sp + 1) * num_kb / S);
  const bool scaled = p.epilogue != QLIN_EPI_RAW;
  const bool prod = p.epilogue == QLIN_EPI_SCALE_PROD;
  const bool has_bias = p.bias != nullptr;

  // Every thread of every CTA of the cluster reaches the two cluster barriers below, whatever happens before them.
  const bool bad = (smem_u32(smem) & 1023u) != 0;
  if (bad && threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, static_cast<int32_t>(QLIN_ERR_BAD_ALIGN));

  if (threadIdx.x == 0) {
    for (int s = 0; s < STG; ++s) {
      mbar_init(&aux->full[s], 1);
      mbar_init(&aux->empty[s], 1);
    }
    mbar_init(&aux->tfull[0], 1);
    mbar_init(&aux->drain, 1);
    aux->abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == kSkMmaWarp) {
    tmem_alloc(&aux->tmem_base, kSkTmemCols);
    tmem_relinquish();
  }
  if (warp == kSkProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  // the row scales of the (at most 128) activation rows, read by every epilogue thread
  float* s_rs = aux->cs;
  if (threadIdx.x < MT) s_rs[threadIdx.x] = (scaled && p.rs != nullptr && static_cast<int>(threadIdx.x) < p.M) ? p.rs[static_cast<int64_t>(threadIdx.x) * p.rs_stride] : 1.0f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = aux->tmem_base;
  bool timed_out = false;
  uint32_t* part = reinterpret_cast<uint32_t*>(smem);  // [MT][128] partial accumulators, over the drained pipeline stages

  if (bad) {
    // nothing: fall through to the barriers
  } else if (warp == kSkProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    uint32_t s = 0, ph = 0, issued = 0;
    bool ok = true;
    for (int kb = kb0; kb < kb1; ++kb) {
      ok = warp_mbar_wait(&aux->empty[s], ph ^ 1u, abort_flag);
      if (!ok) break;
      uint8_t* sa = smem + s * stage_bytes;
      tma_issue_stage(&aux->full[s], static_cast<uint32_t>(stage_bytes), sa, &tmap_w, tile * kBM, sa + kSkWBytes, &tmap_x, 0, kb * kBK);
      ++issued;
      if (++s == static_cast<uint32_t>(STG)) {
        s = 0;
        ph ^= 1u;
      }
    }
    if (!ok) {
      if (lane == 0) {
        timed_out = !*abort_flag;
        *abort_flag = 1;
      }
      for (uint32_t st = 0; st < static_cast<uint32_t>(STG); ++st) {
        if (issued <= st) continue;
        const uint32_t last = (issued - 1 - st) / static_cast<uint32_t>(STG);
        mbar_wait_drain(&aux->full[st], last & 1u);
      }
    }
    __syncwarp();
  } else if (warp == kSkMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = F8 ? make_idesc(1u, static_cast<uint32_t>(p.f8_ab_format), kBM, static_cast<uint32_t>(MT))
                              : make_idesc(2u, 1u, kBM, static_cast<uint32_t>(MT));
    const uint64_t wdesc0 = make_smem_desc_sw128(smem_u32(smem));
    const uint64_t xdesc0 = make_smem_desc_sw128(smem_u32(smem) + kSkWBytes);
    uint32_t s = 0, ph = 0, accumulate = 0;
    bool ok = true;
    for (int kb = kb0; kb < kb1; ++kb) {
      ok = warp_mbar_wait(&aux->full[s], ph, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint64_t off = static_cast<uint64_t>(s * (stage_bytes >> 4));
      tc_mma4_release<F8 ? 1 : 0>(tmem_base, wdesc0 + off, xdesc0 + off, idesc, accumulate, &aux->empty[s]);
      accumulate = 1;
      if (++s == static_cast<uint32_t>(STG)) {
        s = 0;
        ph ^= 1u;
      }
    }
    if (ok) tc_commit_elect(&aux->tfull[0]);
    if (!ok && lane == 0) {
      timed_out = !*abort_flag;
      *abort_flag = 1;
    }
    tc_commit_elect(&aux->drain);
    mbar_wait_drain(&aux->drain, 0);
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps, first half
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    const int n = tile * kBM + n_local;
    if (warp_mbar_wait(&aux->tfull[0], 0, abort_flag)) {
      tc_fence_after();
      const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
      float cs = 1.0f, bias = 0.0f;
      if (S == 1 && n < p.N && scaled) {
        if (p.cs != nullptr) cs = p.cs[static_cast<int64_t>(n) * p.cs_stride];
        if (has_bias) bias = p.bias[n];
      }
#pragma unroll 1
      for (int c = (warp >> 2) * 32; c < MT; c += 64) {
        if (c >= p.M) break;
        uint32_t v[32];
        tmem_ld32(tmem_base + lane_base + c, v);
        if (S == 1) {
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c + j < p.M) skinny_emit<F8>(p, v[j], c + j, n, s_rs[c + j], cs, bias, prod, has_bias);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c + j < p.M) part[(c + j) * kBM + n_local] = v[j];
        }
      }
      tc_fence_before();
    } else if (lane == 0) {
      timed_out = !*abort_flag;
      *abort_flag = 1;
    }
    __syncwarp();
  }

  if (S > 1) {
    __syncwarp();
    cluster_arrive_wait();  // every split's partial tile is in its CTA's shared memory
    if (!bad && warp < kSkEpiWarps) {
      const int n_local = threadIdx.x & (kBM - 1);
      const int n = tile * kBM + n_local;
      if (n < p.N) {
        float cs = 1.0f, bias = 0.0f;
        if (scaled) {
          if (p.cs != nullptr) cs = p.cs[static_cast<int64_t>(n) * p.cs_stride];
          if (has_bias) bias = p.bias[n];
        }
        // this CTA's rows are sp, sp + S, ...; the two halves of the epilogue warps take every other one of them
        // two rows per iteration: both rows' loads are in flight before the first sum is needed
        auto sum_row = [&](int m) -> uint32_t {
          const uint32_t* src = part + m * kBM + n_local;
          if (S == 2) return skinny_sum_splits<F8, 2>(src);
          if (S == 4) return skinny_sum_splits<F8, 4>(src);
          return skinny_sum_splits<F8, 8>(src);
        };
        for (int m = sp + S * static_cast<int>(threadIdx.x >> 7); m < p.M; m += 4 * S) {
          const int m2 = m + 2 * S;
          const uint32_t acc = sum_row(m);
          const uint32_t acc2 = m2 < p.M ? sum_row(m2) : 0u;
          skinny_emit<F8>(p, acc, m, n, s_rs[m], cs, bias, prod, has_bias);
          if (m2 < p.M) skinny_emit<F8>(p, acc2, m2, n, s_rs[m2], cs, bias, prod, has_bias);
        }
      }
    }
    __syncwarp();
    cluster_arrive_wait();  // nobody leaves while a neighbour still reads its shared memory
  }

  if (timed_out && p.status != nullptr) atomicExch(p.status, static_cast<int32_t>(QLIN_ERR_TIMEOUT));
  tc_fence_before();
  __syncthreads();
  if (warp == kSkMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem_base, kSkTmemCols);
  }
}

// ---------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  }
  return fn;
}

// [rows, kbytes] byte matrix with `ld_bytes` between rows, read in boxes of [box_rows x 128 bytes].
static int make_operand_map(CUtensorMap* tm, const void* base, int64_t rows, int64_t kbytes, int64_t ld_bytes,
                            int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return fail(QLIN_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(kbytes), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QLIN_ERR_BAD_ALIGN, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return QLIN_OK;
}

template <bool F8, bool CHUNKED, bool BATCHED = false>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  using C = Cfg<CHUNKED>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return fail(QLIN_ERR_DEVICE, "device ordinal %d out of range", dev);
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(qlin_gemm_kernel<F8, CHUNKED, BATCHED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) return fail(QLIN_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  const int64_t tiles = static_cast<int64_t>(p.num_m) * p.num_n * (BATCHED ? p.batch : 1);
  int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  if (p.max_ctas > 0 && grid > p.max_ctas) grid = p.max_ctas;
  qlin_gemm_kernel<F8, CHUNKED, BATCHED><<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(ta, tb, p);
  QLIN_CHECK_LAUNCH("qlin_gemm");
  return QLIN_OK;
}

// Largest number of two-CTA clusters of the pair kernel that can be resident at once (cached per device).
template <bool F8>
static int pair_max_clusters() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 0;
  if (cached[dev] != 0) return cached[dev] > 0 ? cached[dev] : 0;
  cached[dev] = -1;
  if (cudaFuncSetAttribute(qlin_gemm_pair_kernel<F8>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::SMEM_BYTES) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sm_count() & ~1), 1, 1);
  cfg.blockDim = dim3(PairCfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = PairCfg::SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, qlin_gemm_pair_kernel<F8>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cached[dev] = n > 0 ? n : -1;
  return n > 0 ? n : 0;
}

template <bool F8>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  int clusters = pair_max_clusters<F8>();
  if (clusters <= 0) return 1;  // not available: the caller takes the single-CTA kernel
  const int tiles = ((p.M + 2 * kBM - 1) / (2 * kBM)) * p.num_n;
  if (clusters > tiles) clusters = tiles;
  if (p.max_ctas > 0 && clusters > p.max_ctas / 2) clusters = p.max_ctas / 2 > 0 ? p.max_ctas / 2 : 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters), 1, 1);
  cfg.blockDim = dim3(PairCfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = PairCfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, qlin_gemm_pair_kernel<F8>, ta, tb, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QLIN_ERR_LAUNCH, "qlin_gemm (CTA-pair kernel): %s", cudaGetErrorString(e));
  }
  return QLIN_OK;
}

// The CTA-pair kernel is used for unchunked problems of at least 256 rows unless QLIN_GEMM_PAIR=0.
static bool pair_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("QLIN_GEMM_PAIR");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

static bool low_byte_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("QLIN_GEMM_LOWBYTE");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// The few-row kernel is used for unchunked problems of at most 128 rows unless QLIN_GEMM_SKINNY=0.
static bool skinny_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("QLIN_GEMM_SKINNY");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <bool F8>
static int launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, GemmParams p, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return fail(QLIN_ERR_DEVICE, "device ordinal %d out of range", dev);
  const int smem_max = 232448;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(qlin_gemm_skinny_kernel<F8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
    if (e != cudaSuccess) return fail(QLIN_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  const int stage_bytes = kSkWBytes + p.sk_mt * kBK;
  int stages = (smem_max - static_cast<int>(sizeof(Aux))) / stage_bytes;
  p.sk_stages = stages > 8 ? 8 : stages;
  const int tiles = (p.N + kBM - 1) / kBM;
  // K splits: the largest power of two that keeps one CTA per SM and at least four K blocks per split
  const int num_kb = (p.kbytes + kBK - 1) / kBK;
  int split = 1;
  while (split < 8 && tiles * split * 2 <= sm_count() && num_kb / (split * 2) >= 4) split *= 2;
  p.sk_split = split;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * split), 1, 1);
  cfg.blockDim = dim3(kSkThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(p.sk_stages) * stage_bytes + sizeof(Aux);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(split);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, qlin_gemm_skinny_kernel<F8>, tw, tx, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QLIN_ERR_LAUNCH, "qlin_gemm (few-row kernel): %s", cudaGetErrorString(e));
  }
  return QLIN_OK;
}

static bool is_round_dtype(int dt) {
  return dt == QLIN_DT_NONE || dt == QLIN_DT_F32 || dt == QLIN_DT_F16 || dt == QLIN_DT_BF16;
}

}  // namespace qlin

using namespace qlin;

// batch > 1: the problems' operands are stacked along the rows (dense), one launch of the batched single-CTA kernel.
static int gemm_impl(const qlin_gemm_args* a, void* stream, int32_t batch, int64_t stride_d) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_gemm: args is NULL");
  if (a->a == nullptr || a->b == nullptr || (a->d == nullptr && a->scatter_rows <= 0))
    return fail(QLIN_ERR_NULL, "qlin_gemm: a, b or d is NULL");
  if (a->scatter_rows < 0 || (a->scatter_rows > 0 && a->scatter_rows % 128 != 0))
    return fail(QLIN_ERR_BAD_SHAPE, "qlin_gemm: scatter_rows must be a multiple of 128");
  if (a->scatter_rows > 0) {
    const int64_t owners = (static_cast<int64_t>(a->M) + a->scatter_rows - 1) / a->scatter_rows;
    if (owners > 8) return fail(QLIN_ERR_BAD_SHAPE, "qlin_gemm: more than 8 scatter destinations");
    for (int i = 0; i < owners; ++i) {
      if (a->scatter_d[i] == nullptr) return fail(QLIN_ERR_NULL, "qlin_gemm: scatter_d[%d] is NULL", i);
      if (!aligned16(a->scatter_d[i])) return fail(QLIN_ERR_BAD_ALIGN, "qlin_gemm: scatter_d[%d] is not 16-byte aligned", i);
    }
    if (a->c != nullptr) return fail(QLIN_ERR_UNSUPPORTED, "qlin_gemm: scatter with an accumulator input is not provided");
  }
  if (a->M < 0 || a->N < 0 || a->K < 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_gemm: negative dimension");
  if (a->kind != QLIN_DT_I8 && a->kind != QLIN_DT_F8E4M3 && a->kind != QLIN_DT_F8E5M2)
    return fail(QLIN_ERR_BAD_DTYPE, "qlin_gemm: kind must be QLIN_DT_I8, QLIN_DT_F8E4M3 or QLIN_DT_F8E5M2");
  const bool f8 = a->kind != QLIN_DT_I8;
  if (a->M == 0 || a->N == 0) return QLIN_OK;
  if (a->K == 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_gemm: K must be positive");
  if (a->lda < a->K || a->ldb < a->K || a->ldd < a->N || (a->c != nullptr && a->ldc < a->N))
    return fail(QLIN_ERR_BAD_SHAPE, "qlin_gemm: leading dimension smaller than the row length");
  if (!aligned16(a->a) || !aligned16(a->b) || a->lda % 16 != 0 || a->ldb % 16 != 0)
    return fail(QLIN_ERR_BAD_ALIGN, "qlin_gemm: a and b must be 16-byte aligned with lda, ldb multiples of 16");
  if (a->epilogue == QLIN_EPI_RAW) {
    if (a->out_dtype != (f8 ? QLIN_DT_F32 : QLIN_DT_I32))
      return fail(QLIN_ERR_BAD_DTYPE, "qlin_gemm: raw output is int32 for int8 operands and fp32 for fp8 operands");
  } else if (a->epilogue == QLIN_EPI_SCALE_PROD || a->epilogue == QLIN_EPI_SCALE_SEQ) {
    if (a->out_dtype != QLIN_DT_F32 && a->out_dtype != QLIN_DT_F16 && a->out_dtype != QLIN_DT_BF16)
      return fail(QLIN_ERR_BAD_DTYPE, "qlin_gemm: scaled output must be fp32, fp16 or bf16");
    if (!is_round_dtype(a->prod_round) || !is_round_dtype(a->scale_round) || !is_round_dtype(a->mid_round) || !is_round_dtype(a->acc_round))
      return fail(QLIN_ERR_BAD_DTYPE, "qlin_gemm: rounding dtypes must be NONE, F32, F16 or BF16");
    if ((a->row_scale_stride != 0 && a->row_scale_stride != 1) || (a->col_scale_stride != 0 && a->col_scale_stride != 1))
      return fail(QLIN_ERR_BAD_SHAPE, "qlin_gemm: scale strides must be 0 or 1");
  } else {
    return fail(QLIN_ERR_UNSUPPORTED, "qlin_gemm: unknown epilogue %d", a->epilogue);
  }
  if (a->trun_bits < 0 || a->trun_bits > (f8 ? 22 : 31))
    return fail(QLIN_ERR_UNSUPPORTED, "qlin_gemm: trun_bits out of range");
  if (!f8 && (a->max_acc_bits < 2 || a->max_acc_bits > 32))
    return fail(QLIN_ERR_UNSUPPORTED, "qlin_gemm: max_acc_bits must be in [2, 32]");
  if (a->chunk_k > 0 && a->chunk_k % 32 != 0)
    return fail(QLIN_ERR_UNSUPPORTED, "qlin_gemm: chunk_k must be a multiple of 32");

  const bool needs_chunks = (a->trun_bits > 0) || (!f8 && a->max_acc_bits < 32) || (f8 && a->clamp_dl16);
  const bool chunked = needs_chunks;  // without a per-chunk function the chunking is not observable for ints
  const int total_k32 = (a->K + 31) / 32;
  int chunk_k32 = total_k32;
  if (chunked && a->chunk_k > 0 && a->chunk_k < a->K) chunk_k32 = a->chunk_k / 32;

  GemmParams p;
  p.c = a->c;
  p.d = a->d;
  p.rs = a->row_scale;
  p.cs = a->col_scale;
  p.bias = a->bias;
  p.status = a->status;
  p.ldc = a->ldc;
  p.ldd = a->ldd;
  p.M = a->M;
  p.N = a->N;
  p.kbytes = a->K;
  p.chunk_k32 = chunk_k32;
  p.trun_bits = a->trun_bits;
  p.max_acc_bits = f8 ? 32 : a->max_acc_bits;
  p.trunc_then_acc = a->trunc_then_acc;
  p.clamp_dl16 = a->clamp_dl16;
  p.epilogue = a->epilogue;
  p.rs_stride = a->row_scale_stride;
  p.cs_stride = a->col_scale_stride;
  p.prod_round = a->prod_round;
  p.scale_round = a->scale_round;
  p.mid_round = a->mid_round;
  p.acc_round = a->acc_round;
  p.out_dtype = a->out_dtype;
  p.max_ctas = a->max_ctas;
  p.scatter_rows = a->scatter_rows;
  p.scatter_row0 = a->scatter_row0;
  p.f8_ab_format = a->kind == QLIN_DT_F8E5M2 ? 1 : 0;
  for (int i = 0; i < 8; ++i) p.scatter_d[i] = static_cast<uint8_t*>(a->scatter_d[i]);
  const int bn = chunked ? Cfg<true>::BN : Cfg<false>::BN;
  p.num_m = (a->M + kBM - 1) / kBM;
  p.num_n = (a->N + bn - 1) / bn;

  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  p.sk_mt = p.sk_split = p.sk_stages = 0;
  p.batch = batch;
  p.batch_stride_d = stride_d;
  // int8 chunks with the low byte rounded away, summed after rounding, no clamp, chunks of 32 / 64 / 128 that tile K:
  // sum of ((p + 128) >> 8 << 8) = sum of p - sum of sext8(p), the first sum kept by the tensor core (QLIN_GEMM_LOWBYTE=0: off)
  p.low_byte_mode = (chunked && !f8 && a->trun_bits == 8 && a->trunc_then_acc && a->max_acc_bits >= 32 &&
                     (chunk_k32 == 1 || chunk_k32 == 2 || chunk_k32 == 4) && total_k32 % 4 == 0 && low_byte_enabled())
                        ? 1
                        : 0;
  if (batch > 1) {
    if (chunked || a->c != nullptr || a->scatter_rows != 0) return fail(QLIN_ERR_UNSUPPORTED, "qlin_gemm_batched: one launch takes unchunked problems without accumulator input or scatter");
    if (static_cast<int64_t>(batch) * a->M > 0x7fffffff || static_cast<int64_t>(batch) * a->N > 0x7fffffff)
      return fail(QLIN_ERR_BAD_SHAPE, "qlin_gemm_batched: batch * rows exceeds the coordinate range");
    CUtensorMap ta, tb;
    int rc = make_operand_map(&ta, a->a, static_cast<int64_t>(batch) * a->M, a->K, a->lda, kBM);
    if (rc != QLIN_OK) return rc;
    rc = make_operand_map(&tb, a->b, static_cast<int64_t>(batch) * a->N, a->K, a->ldb, bn);
    if (rc != QLIN_OK) return rc;
    return f8 ? launch<true, false, true>(ta, tb, p, s) : launch<false, false, true>(ta, tb, p, s);
  }
  if (!chunked && a->M <= kBM && a->scatter_rows == 0 && a->max_ctas <= 0 && skinny_enabled()) {
    // weight rows as the MMA's M dimension, the few activation rows (padded to 32) as its N dimension
    p.sk_mt = (a->M + 31) / 32 * 32;
    CUtensorMap tw, tx;
    int rc = make_operand_map(&tw, a->b, a->N, a->K, a->ldb, kBM);
    if (rc != QLIN_OK) return rc;
    rc = make_operand_map(&tx, a->a, a->M, a->K, a->lda, p.sk_mt);
    if (rc != QLIN_OK) return rc;
    rc = f8 ? launch_skinny<true>(tw, tx, p, s) : launch_skinny<false>(tw, tx, p, s);
    // a device that cannot place the cluster (fewer SMs per GPC than the split needs): the wide tile below does the job
    if (rc != QLIN_ERR_LAUNCH) return rc;
    p.sk_mt = p.sk_split = p.sk_stages = 0;
  }

  CUtensorMap ta, tb;
  int rc = make_operand_map(&ta, a->a, a->M, a->K, a->lda, kBM);
  if (rc != QLIN_OK) return rc;
  rc = make_operand_map(&tb, a->b, a->N, a->K, a->ldb, bn);
  if (rc != QLIN_OK) return rc;

  if (!chunked && a->M >= 2 * kBM && pair_enabled()) {
    CUtensorMap tb_half;  // each CTA of a pair loads 128 of the tile's 256 B rows
    rc = make_operand_map(&tb_half, a->b, a->N, a->K, a->ldb, PairCfg::BN / 2);
    if (rc != QLIN_OK) return rc;
    rc = f8 ? launch_pair<true>(ta, tb_half, p, s) : launch_pair<false>(ta, tb_half, p, s);
    if (rc <= 0) return rc;
  }
  if (f8) return chunked ? launch<true, true>(ta, tb, p, s) : launch<true, false>(ta, tb, p, s);
  return chunked ? launch<false, true>(ta, tb, p, s) : launch<false, false>(ta, tb, p, s);
}

extern "C" int qlin_gemm(const qlin_gemm_args* a, void* stream) { return gemm_impl(a, stream, 1, 0); }

extern "C" int qlin_gemm_batched(const qlin_gemm_args* a, int32_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, void* stream) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_gemm_batched: args is NULL");
  if (batch < 0 || stride_a < 0 || stride_b < 0 || stride_d < 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_gemm_batched: negative batch or stride");
  if (a->c != nullptr || a->scatter_rows != 0) return fail(QLIN_ERR_UNSUPPORTED, "qlin_gemm_batched: no accumulator input and no row-block scatter");
  if (batch > 1 && (stride_a % 16 != 0 || stride_b % 16 != 0)) return fail(QLIN_ERR_BAD_ALIGN, "qlin_gemm_batched: operand strides must be multiples of 16 bytes");
  if (batch == 0) return QLIN_OK;
  const int64_t out_elt = (a->epilogue == QLIN_EPI_RAW || a->out_dtype == QLIN_DT_F32) ? 4 : 2;
  const bool needs_chunks = (a->trun_bits > 0) || (a->kind == QLIN_DT_I8 && a->max_acc_bits < 32) || (a->kind != QLIN_DT_I8 && a->clamp_dl16);
  // dense stacks of unchunked problems: one launch whose tiles walk over all problems
  if (batch > 1 && !needs_chunks && stride_a == static_cast<int64_t>(a->M) * a->lda && stride_b == static_cast<int64_t>(a->N) * a->ldb &&
      (stride_d * out_elt) % 16 == 0 && a->M > 0 && a->N > 0)
    return gemm_impl(a, stream, batch, stride_d);
  qlin_gemm_args one = *a;
  for (int32_t i = 0; i < batch; ++i) {
    one.a = static_cast<const uint8_t*>(a->a) + i * stride_a;
    one.b = static_cast<const uint8_t*>(a->b) + i * stride_b;
    one.d = static_cast<uint8_t*>(a->d) + i * stride_d * out_elt;
    const int rc = gemm_impl(&one, stream, 1, 0);
    if (rc != QLIN_OK) return rc;
  }
  return QLIN_OK;
}
