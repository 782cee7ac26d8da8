// Grouped GEMM on the 5th-generation tensor cores (tcgen05) for the expert linears.
//
// Replaces the reference's host loop of one cuBLAS call per expert with stream
// synchronisations around it (cuda/parallel_linear.cuh:56-163): one persistent kernel covers
// every expert, reads the expert row offsets from device memory (no host counts), and fuses
// bias, activation, activation-derivative and dtype conversion into its epilogue.
//
// Structure of a CTA (192 threads, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer: cp.async.bulk.tensor (no multicast) into a 4-stage ring of
//               128-byte-swizzled shared-memory tiles, completion on mbarriers;
//   warp 1      one elected thread issues tcgen05.mma (128 x 256 x 16 per instruction, fp32
//               accumulators in TMEM) and tcgen05.commit; the warp owns the TMEM allocation;
//   warps 2-5   epilogue: tcgen05.ld of the accumulator (each warp its 32 TMEM lanes),
//               bias / activation / derivative, 16-byte stores.
// Two 256-column accumulators (all 512 TMEM columns) let the epilogue of tile i overlap the
// main loop of tile i+1.
//
// The weight-gradient mode reduces over token rows, so both operands are MN-major; the last
// K block of an expert is ragged, and the producer warp zeroes the rows past the segment end
// in shared memory before handing the stage to the MMA thread.
#include "grouped_gemm.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "ptx.cuh"

namespace fmoe {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;      // 16 KB
constexpr int B_BYTES = BN * BK * 2;      // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;  // one 64-wide MN-major box: 8 KB
constexpr int MAX_GROUPS = 1024;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;

constexpr int STATUS_TIMEOUT_PRODUCER = 101;
constexpr int STATUS_TIMEOUT_MMA = 102;
constexpr int STATUS_TIMEOUT_EPILOGUE = 103;

struct SharedAux {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t tail;
  uint32_t tmem_base;
  int abort;
  int total_tiles;
  int tile_prefix[MAX_GROUPS + 1];
};

constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + static_cast<int>(sizeof(SharedAux)) + 1024;

struct KernelParams {
  int num_groups;
  int m;  // wgrad only
  int n;
  int k;  // row modes
  const int* offs;
  void* out;
  void* pre_out;
  const void* bias;
  const void* aux;
  int act;
  int epi;
  int accumulate;
  int out_fp32;
  int* status;
};

struct TileCoord {
  int group;
  int m_tile;
  int n_tile;
  int row_begin;  // first row of the group
  int row_end;    // one past the last row of the group
};

template <int MODE>
__device__ __forceinline__ int tiles_of_group(const KernelParams& p, int rows) {
  const int n_tiles = (p.n + BN - 1) / BN;
  if (MODE == kWgrad) return ((p.m + BM - 1) / BM) * n_tiles;
  return ((rows + BM - 1) / BM) * n_tiles;
}

template <int MODE>
__device__ __forceinline__ TileCoord decode_tile(const KernelParams& p, const SharedAux* aux,
                                                 int tile) {
  // Binary search of the group whose tile range contains `tile`.
  int lo = 0, hi = p.num_groups;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (aux->tile_prefix[mid] <= tile) lo = mid; else hi = mid;
  }
  TileCoord c;
  c.group = lo;
  const int local = tile - aux->tile_prefix[lo];
  const int n_tiles = (p.n + BN - 1) / BN;
  c.m_tile = local / n_tiles;
  c.n_tile = local - c.m_tile * n_tiles;
  c.row_begin = p.offs[lo];
  c.row_end = p.offs[lo + 1];
  return c;
}

__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}
__device__ __forceinline__ float gelu_erf_grad(float x) {
  const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752f));
  const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  const float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}
__device__ __forceinline__ float apply_act(int act, float x) {
  switch (act) {
    case kActRelu: return x > 0.f ? x : 0.f;
    case kActGelu: return gelu_erf(x);
    case kActGeluTanh: return gelu_tanh(x);
    default: return x;
  }
}
__device__ __forceinline__ float apply_act_grad(int act, float x) {
  switch (act) {
    case kActRelu: return x > 0.f ? 1.f : 0.f;
    case kActGelu: return gelu_erf_grad(x);
    case kActGeluTanh: return gelu_tanh_grad(x);
    default: return 1.f;
  }
}

template <typename T> struct Cvt;
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ void unpack(uint32_t w, float& a, float& b) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&w);
    a = __low2float(v);
    b = __high2float(v);
  }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ void unpack(uint32_t w, float& a, float& b) {
    __half2 v = *reinterpret_cast<__half2*>(&w);
    a = __low2float(v);
    b = __high2float(v);
  }
};

// Loads 32 consecutive 16-bit values (64 bytes, 16-byte aligned) as floats.
template <typename T>
__device__ __forceinline__ void load32(const T* src, float (&v)[32]) {
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 w = __ldg(s4 + q);
    Cvt<T>::unpack(w.x, v[q * 8 + 0], v[q * 8 + 1]);
    Cvt<T>::unpack(w.y, v[q * 8 + 2], v[q * 8 + 3]);
    Cvt<T>::unpack(w.z, v[q * 8 + 4], v[q * 8 + 5]);
    Cvt<T>::unpack(w.w, v[q * 8 + 6], v[q * 8 + 7]);
  }
}

template <typename T>
__device__ __forceinline__ void store32(T* dst, const float (&v)[32]) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 w;
    w.x = Cvt<T>::pack(v[q * 8 + 0], v[q * 8 + 1]);
    w.y = Cvt<T>::pack(v[q * 8 + 2], v[q * 8 + 3]);
    w.z = Cvt<T>::pack(v[q * 8 + 4], v[q * 8 + 5]);
    w.w = Cvt<T>::pack(v[q * 8 + 6], v[q * 8 + 7]);
    d4[q] = w;
  }
}

__device__ __forceinline__ void fail(SharedAux* aux, int* status, int code) {
  aux->abort = 1;
  if (status != nullptr) atomicCAS(status, 0, code);
}

template <int MODE, typename T>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a,
                    const __grid_constant__ CUtensorMap tm_b, const KernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  SharedAux* aux = reinterpret_cast<SharedAux*>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---------------------------------------------------------------- set-up
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&aux->full[s], 1);
      ptx::mbar_init(&aux->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&aux->tmem_full[a], 1);
      ptx::mbar_init(&aux->tmem_empty[a], 128);
    }
    ptx::mbar_init(&aux->tail, 1);
    aux->abort = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tm_a);
    ptx::prefetch_tmap(&tm_b);
  }
  for (int g = threadIdx.x; g < p.num_groups; g += NUM_THREADS) {
    aux->tile_prefix[g + 1] = tiles_of_group<MODE>(p, p.offs[g + 1] - p.offs[g]);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&aux->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    aux->tile_prefix[0] = 0;
    for (int g = 0; g < p.num_groups; ++g) {
      run += aux->tile_prefix[g + 1];
      aux->tile_prefix[g + 1] = run;
    }
    aux->total_tiles = run;
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();

  const uint32_t tmem_base = aux->tmem_base;
  const int total_tiles = aux->total_tiles;
  const volatile int* abort_flag = &aux->abort;

  if (warp == 0) {
    // ============================================================== TMA producer
    int stage = 0;
    uint32_t phase = 0;
    uint32_t tail_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const TileCoord c = decode_tile<MODE>(p, aux, tile);
      const int rows = c.row_end - c.row_begin;
      const int num_kb = (MODE == kWgrad) ? (rows + BK - 1) / BK : p.k / BK;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!ptx::mbar_wait(&aux->empty[stage], phase ^ 1, abort_flag)) {
          if (lane == 0) fail(aux, p.status, STATUS_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        uint8_t* sa = smem + stage * STAGE_BYTES;
        uint8_t* sb = sa + A_BYTES;
        const int valid = (MODE == kWgrad) ? min(BK, rows - kb * BK) : BK;
        const bool ragged = (MODE == kWgrad) && valid < BK;
        uint64_t* bar = ragged ? &aux->tail : &aux->full[stage];
        if (lane == 0) {
          ptx::mbar_arrive_expect_tx(bar, STAGE_BYTES);
          if (MODE == kRowsNT) {
            ptx::tma_load_2d(sa, &tm_a, bar, kb * BK, c.row_begin + c.m_tile * BM);
            ptx::tma_load_2d(sb, &tm_b, bar, kb * BK, c.group * p.n + c.n_tile * BN);
          } else if (MODE == kRowsNN) {
            ptx::tma_load_2d(sa, &tm_a, bar, kb * BK, c.row_begin + c.m_tile * BM);
#pragma unroll
            for (int ch = 0; ch < BN / 64; ++ch) {
              ptx::tma_load_2d(sb + ch * CHUNK_BYTES, &tm_b, bar, c.n_tile * BN + ch * 64,
                               c.group * p.k + kb * BK);
            }
          } else {
            const int row0 = c.row_begin + kb * BK;
#pragma unroll
            for (int ch = 0; ch < BM / 64; ++ch) {
              ptx::tma_load_2d(sa + ch * CHUNK_BYTES, &tm_a, bar, c.m_tile * BM + ch * 64, row0);
            }
#pragma unroll
            for (int ch = 0; ch < BN / 64; ++ch) {
              ptx::tma_load_2d(sb + ch * CHUNK_BYTES, &tm_b, bar, c.n_tile * BN + ch * 64, row0);
            }
          }
        }
        if constexpr (MODE == kWgrad) if (ragged) {
          // Rows >= valid of this K block belong to the next expert (or lie past the buffer):
          // wait for the copies, zero those rows in all six boxes, publish to the async proxy.
          if (!ptx::mbar_wait(&aux->tail, tail_phase, abort_flag)) {
            if (lane == 0) fail(aux, p.status, STATUS_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          tail_phase ^= 1;
          const int zero_rows = BK - valid;
          // One row of a box is 128 bytes = 8 x uint4; a box has BK rows.
          const int items = (BM / 64 + BN / 64) * zero_rows * 8;
          for (int it = lane; it < items; it += 32) {
            const int box = it / (zero_rows * 8);
            const int rem = it - box * (zero_rows * 8);
            const int r = valid + rem / 8;
            const int q = rem & 7;
            uint4* dst = reinterpret_cast<uint4*>(sa + box * CHUNK_BYTES + r * 128 + q * 16);
            *dst = make_uint4(0, 0, 0, 0);
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&aux->full[stage]);
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ============================================================== MMA issuer
    if (lane == 0) {
      constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
      constexpr uint32_t idesc =
          ptx::make_idesc(kBf16, MODE == kWgrad, MODE != kRowsNT, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++iter) {
        const TileCoord c = decode_tile<MODE>(p, aux, tile);
        const int rows = c.row_end - c.row_begin;
        const int num_kb = (MODE == kWgrad) ? (rows + BK - 1) / BK : p.k / BK;
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!ptx::mbar_wait(&aux->tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          fail(aux, p.status, STATUS_TIMEOUT_MMA);
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&aux->full[stage], phase, abort_flag)) {
            fail(aux, p.status, STATUS_TIMEOUT_MMA);
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sa = ptx::smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k16 = 0; k16 < BK / UMMA_K; ++k16) {
            // K-major operands: 32 bytes per K step inside the 128-byte swizzle row, 8-row
            // groups 1024 bytes apart.  MN-major operands: 16 K rows (2048 bytes) per step,
            // 64-element MN chunks one box (8 KB) apart, 8-row groups 1024 bytes apart.
            const uint64_t a_desc = (MODE == kWgrad)
                ? ptx::make_smem_desc_sw128(sa + k16 * (UMMA_K * 128), CHUNK_BYTES, 1024)
                : ptx::make_smem_desc_sw128(sa + k16 * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc = (MODE == kRowsNT)
                ? ptx::make_smem_desc_sw128(sb + k16 * (UMMA_K * 2), 16, 1024)
                : ptx::make_smem_desc_sw128(sb + k16 * (UMMA_K * 128), CHUNK_BYTES, 1024);
            ptx::umma_f16(d_tmem, a_desc, b_desc, idesc, (kb | k16) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&aux->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        ptx::umma_commit(&aux->tmem_full[acc]);
      }
    }
  } else {
    // ============================================================== epilogue (warps 2..5)
    const int part = warp & 3;  // TMEM lane partition this warp may read
    const int row_in_tile = part * 32 + lane;
    int iter = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++iter) {
      const TileCoord c = decode_tile<MODE>(p, aux, tile);
      const int rows = c.row_end - c.row_begin;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!ptx::mbar_wait(&aux->tmem_full[acc], acc_phase, abort_flag)) {
        if (lane == 0) fail(aux, p.status, STATUS_TIMEOUT_EPILOGUE);
        break;
      }
      ptx::tc_fence_after_sync();

      bool row_ok;
      long out_row;  // row index into the output matrix
      if (MODE == kWgrad) {
        const int mrow = c.m_tile * BM + row_in_tile;
        row_ok = mrow < p.m;
        out_row = static_cast<long>(c.group) * p.m + mrow;
      } else {
        const int r = c.m_tile * BM + row_in_tile;
        row_ok = r < rows;
        out_row = static_cast<long>(c.row_begin) + r;
      }
      const bool have_acc = (MODE != kWgrad) || rows > 0;
      const int n0 = c.n_tile * BN;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(part * 32) << 16) + acc * BN;

#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        const int col0 = n0 + ch * 32;
        if (col0 >= p.n) break;
        float v[32];
        if (have_acc) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(t_row + ch * 32, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        if (!row_ok) continue;
        const long off = out_row * p.n + col0;
        if (MODE == kWgrad) {
          if (p.out_fp32) {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + off);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 w = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              if (p.accumulate) {
                float4 o = dst[q];
                w.x += o.x; w.y += o.y; w.z += o.z; w.w += o.w;
              }
              dst[q] = w;
            }
          } else {
            T* dst = static_cast<T*>(p.out) + off;
            if (p.accumulate) {
              float o[32];
              load32<T>(dst, o);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += o[j];
            }
            store32<T>(dst, v);
          }
        } else if (p.epi == kEpiDAct) {
          float a[32];
          load32<T>(static_cast<const T*>(p.aux) + off, a);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= apply_act_grad(p.act, a[j]);
          store32<T>(static_cast<T*>(p.out) + off, v);
        } else {
          if (p.bias != nullptr) {
            float b[32];
            load32<T>(static_cast<const T*>(p.bias) + static_cast<long>(c.group) * p.n + col0, b);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += b[j];
          }
          if (p.pre_out != nullptr) store32<T>(static_cast<T*>(p.pre_out) + off, v);
          if (p.act != kActNone) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = apply_act(p.act, v[j]);
          }
          store32<T>(static_cast<T*>(p.out) + off, v);
        }
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&aux->tmem_empty[acc]);
    }
  }

  // ---------------------------------------------------------------- tear-down
  if (*abort_flag != 0) {
    // Give copies that were already issued time to land before the CTA's shared memory goes away.
    const unsigned long long t0 = ptx::globaltimer();
    while (ptx::globaltimer() - t0 < 200000ull) __nanosleep(1000);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

// 2-D row-major tensor [outer, inner] of 16-bit elements, 128-byte swizzle.
bool make_map_2d(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
                 uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int MODE, typename T>
cudaError_t launch_typed(const CUtensorMap& ta, const CUtensorMap& tb, const KernelParams& kp,
                         int grid, cudaStream_t stream) {
  // The attribute is per device; remember which devices of this process have it.
  static std::mutex mu;
  static uint64_t configured = 0;
  auto kernel = grouped_gemm_kernel<MODE, T>;
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!(configured >> (dev & 63) & 1)) {
      cudaError_t e =
          cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      if (e != cudaSuccess) return e;
      configured |= 1ull << (dev & 63);
    }
  }
  kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, kp);
  return cudaGetLastError();
}

}  // namespace

bool grouped_gemm_supported(int mode, int m, int n, int k, int num_groups) {
  if (num_groups < 1 || num_groups > MAX_GROUPS) return false;
  if (n % 32 != 0 || n < 32) return false;
  if (mode == kWgrad) return m % 8 == 0 && m >= 8;
  return k % 64 == 0 && k >= 64;
}

cudaError_t launch_grouped_gemm(const GroupedGemmArgs& a) {
  if (!grouped_gemm_supported(a.mode, a.m, a.n, a.k, a.num_groups)) return cudaErrorInvalidValue;
  CUtensorMap ta, tb;
  bool ok = true;
  if (a.mode == kRowsNT) {
    ok = make_map_2d(&ta, a.dtype, a.a, a.k, a.rows_cap, BK, BM) &&
         make_map_2d(&tb, a.dtype, a.b, a.k, static_cast<uint64_t>(a.num_groups) * a.n, BK, BN);
  } else if (a.mode == kRowsNN) {
    ok = make_map_2d(&ta, a.dtype, a.a, a.k, a.rows_cap, BK, BM) &&
         make_map_2d(&tb, a.dtype, a.b, a.n, static_cast<uint64_t>(a.num_groups) * a.k, 64, BK);
  } else {
    ok = make_map_2d(&ta, a.dtype, a.a, a.m, a.rows_cap, 64, BK) &&
         make_map_2d(&tb, a.dtype, a.b, a.n, a.rows_cap, 64, BK);
  }
  if (!ok) return cudaErrorInvalidValue;

  KernelParams kp;
  kp.num_groups = a.num_groups;
  kp.m = a.m;
  kp.n = a.n;
  kp.k = a.k;
  kp.offs = a.offs;
  kp.out = a.out;
  kp.pre_out = a.pre_out;
  kp.bias = a.bias;
  kp.aux = a.aux;
  kp.act = a.act;
  kp.epi = a.epi;
  kp.accumulate = a.accumulate;
  kp.out_fp32 = a.out_fp32;
  kp.status = a.status;

  const int grid = a.num_sms > 0 ? a.num_sms : 148;
  const bool bf16 = a.dtype == kBF16;
  switch (a.mode) {
    case kRowsNT:
      return bf16 ? launch_typed<kRowsNT, __nv_bfloat16>(ta, tb, kp, grid, a.stream)
                  : launch_typed<kRowsNT, __half>(ta, tb, kp, grid, a.stream);
    case kRowsNN:
      return bf16 ? launch_typed<kRowsNN, __nv_bfloat16>(ta, tb, kp, grid, a.stream)
                  : launch_typed<kRowsNN, __half>(ta, tb, kp, grid, a.stream);
    default:
      return bf16 ? launch_typed<kWgrad, __nv_bfloat16>(ta, tb, kp, grid, a.stream)
                  : launch_typed<kWgrad, __half>(ta, tb, kp, grid, a.stream);
  }
}

}  // namespace fmoe
