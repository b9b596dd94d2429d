// qlin_gemm: persistent, warp-specialised tcgen05 GEMM for 8-bit operands on sm_100a.
//
//   D[M,N] = epilogue( C + sum over K-chunks of f( A[M,Kc] . B[N,Kc]^T ) )
//
// Both operands are K-major ("NT"), which is the layout the reference hands to its Triton / CUTLASS
// kernels (activations [m,k]; weight [n,k] passed as its .t() view).
//
// Per CTA (one per SM, 320 threads):
//   warp 8      TMA producer: 128-byte-swizzled [128 x 128B] A tile and [BN x 128B] B tile per stage
//   warp 9      MMA issuer: tcgen05.mma.cta_group::1 (M=128, N=BN, K=32 bytes per instruction),
//               accumulators in tensor memory; owns the TMEM allocation
//   warps 0-7   epilogue: tcgen05.ld of the accumulator, chunk rounding / running sum, dequantise,
//               global stores.  Warp w reads TMEM lanes 32*(w%4).. and column half w/4.
// Unchunked: BN=256, two 256-column accumulators so the epilogue of tile i overlaps the mainloop of
// tile i+1.  Chunked: BN=128, four 128-column accumulators; every K-chunk is a fresh accumulation
// that the epilogue warps drain, round and add to a running sum held in registers.
//
// All mbarrier waits are bounded; a wait that runs out raises an abort flag, the CTA drains its
// copies and MMAs, frees TMEM, writes QLIN_ERR_TIMEOUT to the status word and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "qlin_internal.h"
#include "qlin_ptx.cuh"

namespace qlin {

constexpr int kBM = 128;          // rows of A per tile = MMA M
constexpr int kBK = 128;          // bytes of K per pipeline stage = one swizzle row
constexpr int kEpiWarps = 8;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kThreads = 320;
constexpr int kGroupM = 16;       // m-blocks per raster group
constexpr int kTmemCols = 512;

template <bool CHUNKED>
struct Cfg {
  static constexpr int BN = CHUNKED ? 128 : 256;
  static constexpr int NBUF = CHUNKED ? 4 : 2;
  static constexpr int STAGES = CHUNKED ? 6 : 4;
  static constexpr int A_BYTES = kBM * kBK;
  static constexpr int B_BYTES = BN * kBK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int COLS_PER_WARP = BN / 2;  // each epilogue warp: 32 rows x BN/2 columns
  static constexpr int AUX_BYTES = 4096;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + AUX_BYTES + 1024;
};

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
  int32_t epilogue, rs_stride, cs_stride, scale_round, mid_round, acc_round, out_dtype;
  int32_t num_m, num_n;
};

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
static_assert(sizeof(Aux) <= 4096, "aux block too large");

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

// Converts, scales and stores NC consecutive columns of one output row held by this thread.
template <bool F8, int NC>
__device__ __forceinline__ void store_row(const GemmParams& p, const uint32_t (&v)[NC], int row, int col0,
                                          const float* s_cs, const float* s_bias, int s_off, float rs,
                                          bool vec_ok) {
  if (row >= p.M) return;
  const int ncol = min(NC, p.N - col0);
  if (ncol <= 0) return;
  if (p.epilogue == QLIN_EPI_RAW) {
    uint32_t* out = reinterpret_cast<uint32_t*>(p.d) + static_cast<int64_t>(row) * p.ldd + col0;
    if (vec_ok && ncol == NC) {
#pragma unroll
      for (int j = 0; j < NC; j += 4) {
        *reinterpret_cast<uint4*>(out + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < NC; ++j)
        if (j < ncol) out[j] = v[j];
    }
    return;
  }
  float y[NC];
  const bool prod = p.epilogue == QLIN_EPI_SCALE_PROD;
  const bool has_bias = p.bias != nullptr;
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    const float a = F8 ? __uint_as_float(v[j]) : __int2float_rn(static_cast<int32_t>(v[j]));
    const float cs = s_cs[s_off + j];
    float t;
    if (prod) {
      float s = round_to(__fmul_rn(rs, cs), p.scale_round);
      t = __fmul_rn(a, s);
    } else {
      t = round_to(__fmul_rn(__fmul_rn(a, rs), cs), p.mid_round);
    }
    if (has_bias) t = __fadd_rn(t, s_bias[s_off + j]);
    y[j] = round_to(t, p.acc_round);
  }
  if (p.out_dtype == QLIN_DT_F32) {
    float* out = reinterpret_cast<float*>(p.d) + static_cast<int64_t>(row) * p.ldd + col0;
    if (vec_ok && ncol == NC) {
#pragma unroll
      for (int j = 0; j < NC; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(y[j], y[j + 1], y[j + 2], y[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < NC; ++j)
        if (j < ncol) out[j] = y[j];
    }
  } else {
    uint16_t h[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      if (p.out_dtype == QLIN_DT_BF16) {
        h[j] = __bfloat16_as_ushort(__float2bfloat16_rn(y[j]));
      } else {
        h[j] = __half_as_ushort(__float2half_rn(y[j]));
      }
    }
    uint16_t* out = reinterpret_cast<uint16_t*>(p.d) + static_cast<int64_t>(row) * p.ldd + col0;
    if (vec_ok && ncol == NC) {
#pragma unroll
      for (int j = 0; j < NC; j += 8) {
        uint4 w;
        w.x = h[j] | (static_cast<uint32_t>(h[j + 1]) << 16);
        w.y = h[j + 2] | (static_cast<uint32_t>(h[j + 3]) << 16);
        w.z = h[j + 4] | (static_cast<uint32_t>(h[j + 5]) << 16);
        w.w = h[j + 6] | (static_cast<uint32_t>(h[j + 7]) << 16);
        *reinterpret_cast<uint4*>(out + j) = w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < NC; ++j)
        if (j < ncol) out[j] = h[j];
    }
  }
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

template <bool F8, bool CHUNKED>
__global__ void __launch_bounds__(kThreads, 1)
qlin_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  using C = Cfg<CHUNKED>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Aux* aux = reinterpret_cast<Aux*>(smem + C::STAGES * C::STAGE_BYTES);
  volatile int* abort_flag = &aux->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&aux->full[s], 1);
      mbar_init(&aux->empty[s], 1);
    }
    for (int b = 0; b < C::NBUF; ++b) {
      mbar_init(&aux->tfull[b], 1);
      mbar_init(&aux->tempty[b], kEpiWarps);
    }
    mbar_init(&aux->drain, 1);
    aux->abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&aux->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = aux->tmem_base;

  const int num_tiles = p.num_m * p.num_n;
  const int num_kb = (p.kbytes + kBK - 1) / kBK;
  const int total_k32 = (p.kbytes + 31) / 32;
  bool timed_out = false;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the loop (so it stays converged for the final barrier); lane 0 issues.
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int mb, nb;
      tile_coords(t, p.num_m, p.num_n, mb, nb);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const uint32_t s = it % C::STAGES;
        const uint32_t ph = (it / C::STAGES) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(&aux->empty[s], ph ^ 1u, abort_flag));
        if (!ok) break;
        if (lane == 0) {
          uint8_t* sa = smem + s * C::STAGE_BYTES;
          uint8_t* sb = sa + C::A_BYTES;
          mbar_arrive_expect_tx(&aux->full[s], C::STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &aux->full[s], kb * kBK, mb * kBM);
          tma_load_2d(sb, &tmap_b, &aux->full[s], kb * kBK, nb * C::BN);
        }
        __syncwarp();
      }
    }
    if (!ok) {
      if (lane == 0) {
        timed_out = !*abort_flag;
        *abort_flag = 1;
      }
      // Let the copies already issued land before the CTA gives its shared memory back.
      const uint32_t issued = it;
      for (uint32_t s = 0; s < static_cast<uint32_t>(C::STAGES); ++s) {
        if (issued <= s) continue;
        const uint32_t last = ((issued - 1 - s) / C::STAGES);  // index of the last fill of stage s
        mbar_wait_drain(&aux->full[s], last & 1u);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = F8 ? make_idesc(1u, 0u, kBM, C::BN) : make_idesc(2u, 1u, kBM, C::BN);
    uint32_t it = 0, acc_it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      uint32_t buf = 0, accumulate = 0;
      for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
        const uint32_t s = it % C::STAGES;
        const uint32_t ph = (it / C::STAGES) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(&aux->full[s], ph, abort_flag));
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * C::STAGE_BYTES);
        const uint64_t adesc = make_smem_desc_sw128(sa);
        const uint64_t bdesc = make_smem_desc_sw128(sa + C::A_BYTES);
        const int nsteps = min(4, total_k32 - kb * 4);
        for (int j = 0; j < nsteps; ++j) {
          const int kk = kb * 4 + j;
          if (kk % p.chunk_k32 == 0) {
            buf = acc_it % C::NBUF;
            const uint32_t bph = (acc_it / C::NBUF) & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(&aux->tempty[buf], bph ^ 1u, abort_flag));
            if (!ok) break;
            tc_fence_after();
            accumulate = 0;
          }
          const bool last_of_chunk = (kk + 1) % p.chunk_k32 == 0 || kk + 1 == total_k32;
          if (lane == 0) {
            tc_mma<F8 ? 1 : 0>(tmem_base + buf * C::BN, adesc + static_cast<uint64_t>(j * 2),
                               bdesc + static_cast<uint64_t>(j * 2), idesc, accumulate);
            if (last_of_chunk) tc_commit(&aux->tfull[buf]);
          }
          accumulate = 1;
          if (last_of_chunk) ++acc_it;
        }
        if (ok && lane == 0) tc_commit(&aux->empty[s]);
        __syncwarp();
      }
    }
    if (lane == 0) {
      if (!ok) {
        timed_out = !*abort_flag;
        *abort_flag = 1;
      }
      // Nothing may still be reading shared memory or writing TMEM when the CTA retires.
      tc_commit(&aux->drain);
      mbar_wait_drain(&aux->drain, 0);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;
    const int half = warp >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int elt = (p.out_dtype == QLIN_DT_F16 || p.out_dtype == QLIN_DT_BF16) ? 2 : 4;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.d) & 15u) == 0) && ((p.ldd * elt) % 16 == 0);
    const bool clamp = !F8 && p.max_acc_bits < 32;
    const int32_t lo = clamp ? -(1 << (p.max_acc_bits - 1)) : 0;
    const int32_t hi = clamp ? (1 << (p.max_acc_bits - 1)) - 1 : 0;
    const uint32_t rb = p.trun_bits > 0 ? (1u << (p.trun_bits - 1)) : 0u;
    const uint32_t mask = p.trun_bits > 0 ? ~((1u << p.trun_bits) - 1u) : 0xFFFFFFFFu;
    const bool dl16 = F8 && p.clamp_dl16;
    const bool scaled = p.epilogue != QLIN_EPI_RAW;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int mb, nb;
      tile_coords(t, p.num_m, p.num_n, mb, nb);
      const int row = mb * kBM + q * 32 + lane;
      const int col_w = nb * C::BN + half * C::COLS_PER_WARP;
      float rs = 1.0f;
      if (scaled) {
        // Stage this tile's column scales and bias once; all lanes then read them as broadcasts.
        asm volatile("bar.sync 1, 256;" ::: "memory");
        for (int i = threadIdx.x; i < C::BN; i += kEpiWarps * 32) {
          const int n = nb * C::BN + i;
          aux->cs[i] = (p.cs != nullptr && n < p.N) ? p.cs[static_cast<int64_t>(n) * p.cs_stride] : 1.0f;
          aux->bias[i] = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.0f;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (p.rs != nullptr && row < p.M) rs = p.rs[static_cast<int64_t>(row) * p.rs_stride];
      }
      if constexpr (!CHUNKED) {
        const uint32_t buf = acc_it % C::NBUF;
        const uint32_t bph = (acc_it / C::NBUF) & 1u;
        ++acc_it;
        if (!mbar_wait(&aux->tfull[buf], bph, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll 1
        for (int j = 0; j < C::COLS_PER_WARP; j += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_base + lane_base + buf * C::BN + half * C::COLS_PER_WARP + j, v);
          if (p.c != nullptr) {
            uint32_t cv[32];
            load_c_row<32>(p, cv, row, col_w + j);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = acc_add<F8>(cv[i], v[i]);
          }
          store_row<F8, 32>(p, v, row, col_w + j, aux->cs, aux->bias, half * C::COLS_PER_WARP + j, rs, vec_ok);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&aux->tempty[buf]);
      } else {
        uint32_t run[C::COLS_PER_WARP];
        load_c_row<C::COLS_PER_WARP>(p, run, row, col_w);
        const int num_chunks = (total_k32 + p.chunk_k32 - 1) / p.chunk_k32;
#pragma unroll 1
        for (int ch = 0; ch < num_chunks; ++ch) {
          const uint32_t buf = acc_it % C::NBUF;
          const uint32_t bph = (acc_it / C::NBUF) & 1u;
          ++acc_it;
          if (!mbar_wait(&aux->tfull[buf], bph, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          uint32_t v[C::COLS_PER_WARP];
          tmem_ld64(tmem_base + lane_base + buf * C::BN + half * C::COLS_PER_WARP, v);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&aux->tempty[buf]);
          if (p.trunc_then_acc) {
#pragma unroll
            for (int i = 0; i < C::COLS_PER_WARP; ++i)
              run[i] = acc_add<F8>(run[i], chunk_round<F8>(v[i], clamp, lo, hi, rb, mask, dl16));
          } else {
#pragma unroll
            for (int i = 0; i < C::COLS_PER_WARP; ++i)
              run[i] = chunk_round<F8>(acc_add<F8>(run[i], v[i]), clamp, lo, hi, rb, mask, dl16);
          }
        }
        if (!ok) break;
        store_row<F8, C::COLS_PER_WARP>(p, run, row, col_w, aux->cs, aux->bias, half * C::COLS_PER_WARP, rs,
                                        vec_ok);
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
  if (warp == kMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
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

template <bool F8, bool CHUNKED>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  using C = Cfg<CHUNKED>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return fail(QLIN_ERR_DEVICE, "device ordinal %d out of range", dev);
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(qlin_gemm_kernel<F8, CHUNKED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) return fail(QLIN_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  const int tiles = p.num_m * p.num_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  qlin_gemm_kernel<F8, CHUNKED><<<grid, kThreads, C::SMEM_BYTES, stream>>>(ta, tb, p);
  QLIN_CHECK_LAUNCH("qlin_gemm");
  return QLIN_OK;
}

static bool is_round_dtype(int dt) {
  return dt == QLIN_DT_NONE || dt == QLIN_DT_F32 || dt == QLIN_DT_F16 || dt == QLIN_DT_BF16;
}

}  // namespace qlin

using namespace qlin;

extern "C" int qlin_gemm(const qlin_gemm_args* a, void* stream) {
  if (a == nullptr) return fail(QLIN_ERR_NULL, "qlin_gemm: args is NULL");
  if (a->a == nullptr || a->b == nullptr || a->d == nullptr) return fail(QLIN_ERR_NULL, "qlin_gemm: a, b or d is NULL");
  if (a->M < 0 || a->N < 0 || a->K < 0) return fail(QLIN_ERR_BAD_SHAPE, "qlin_gemm: negative dimension");
  if (a->kind != QLIN_DT_I8 && a->kind != QLIN_DT_F8E4M3)
    return fail(QLIN_ERR_BAD_DTYPE, "qlin_gemm: kind must be QLIN_DT_I8 or QLIN_DT_F8E4M3");
  const bool f8 = a->kind == QLIN_DT_F8E4M3;
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
    if (!is_round_dtype(a->scale_round) || !is_round_dtype(a->mid_round) || !is_round_dtype(a->acc_round))
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
  p.scale_round = a->scale_round;
  p.mid_round = a->mid_round;
  p.acc_round = a->acc_round;
  p.out_dtype = a->out_dtype;
  const int bn = chunked ? Cfg<true>::BN : Cfg<false>::BN;
  p.num_m = (a->M + kBM - 1) / kBM;
  p.num_n = (a->N + bn - 1) / bn;

  CUtensorMap ta, tb;
  int rc = make_operand_map(&ta, a->a, a->M, a->K, a->lda, kBM);
  if (rc != QLIN_OK) return rc;
  rc = make_operand_map(&tb, a->b, a->N, a->K, a->ldb, bn);
  if (rc != QLIN_OK) return rc;

  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (f8) return chunked ? launch<true, true>(ta, tb, p, s) : launch<true, false>(ta, tb, p, s);
  return chunked ? launch<false, true>(ta, tb, p, s) : launch<false, false>(ta, tb, p, s);
}
