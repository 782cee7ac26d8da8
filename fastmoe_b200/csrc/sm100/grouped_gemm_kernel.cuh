// Grouped GEMM on the 5th-generation tensor cores (tcgen05) for the expert linears.
//
// Replaces the reference's host loop of one cuBLAS call per expert with stream
// synchronisations around it (cuda/parallel_linear.cuh:56-163): one persistent kernel covers
// every expert, reads the expert row offsets from device memory (no host counts), and fuses
// bias, activation, activation-derivative and dtype conversion into its epilogue.
//
// Structure of a CTA (384 threads = 3 warpgroups, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer: cp.async.bulk.tensor (no multicast) into a 4-stage ring of
//               128-byte-swizzled shared-memory tiles, completion on mbarriers;
//   warp 1      one elected thread issues tcgen05.mma (128 x 256 x 16 per instruction, fp32
//               accumulators in TMEM) and tcgen05.commit; the warp owns the TMEM allocation;
//   warps 2-3   idle (they complete the first warpgroup);
//   warps 4-11  epilogue (two warpgroups): two warps per
//               TMEM lane quarter, taking alternate 32-column chunks
//               of the 256 accumulator columns; the tcgen05.ld of chunk i+1 and the cp.async
//               staging of the side operand (saved pre-activation) for chunk i+1 are in
//               flight while chunk i gets bias / activation / derivative and leaves as 32-byte
//               stores.  The side operand is fetched with coalesced 64-byte row segments
//               into a per-warp shared-memory patch and read back one row per lane.
// Two 256-column accumulators (all 512 TMEM columns) let the epilogue of tile i overlap the
// main loop of tile i+1.
//
// The weight-gradient mode reduces over token rows, so both operands are MN-major; the last
// K block of an expert is ragged, and the producer warp zeroes the rows past the segment end
// in shared memory before handing the stage to the MMA thread.
#pragma once
#include "grouped_gemm.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "ptx.cuh"

namespace fmoe {
namespace gg {

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
constexpr int NUM_EPI_WARPS = 8;
constexpr int FIRST_EPI_WARP = 4;
constexpr int NUM_THREADS = (FIRST_EPI_WARP + NUM_EPI_WARPS) * 32;



constexpr int CHUNKS_PER_WARP = BN / 32 / 2;  // 4 chunks of 32 columns per epilogue warp
constexpr int SIDE_PITCH = 80;                // bytes per staged row (64 data + 16 pad: no bank conflicts)
constexpr int SIDE_BYTES = 32 * SIDE_PITCH;   // one 32-row x 32-column patch per epilogue warp
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

constexpr int AUX_BYTES = (static_cast<int>(sizeof(SharedAux)) + 127) & ~127;
constexpr int BIAS_BYTES = CHUNKS_PER_WARP * 64;  // per epilogue warp: its four 32-column bias slices
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + AUX_BYTES + NUM_EPI_WARPS * (SIDE_BYTES + BIAS_BYTES) + 1024;

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
  void* psum;        // wgrad only, optional: [num_groups, m] column sums of P per group (element type T)
  const void* psrc;  // wgrad only: P itself, for the warps that form the sums with plain loads
  int* status;
  const int64_t* push_meta;
  PeerPtrs push_dst;
  PeerPtrs push_flags;
  const int* push_epoch;
  int* push_counter;
  int push_me;
  int push_world;
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

// GELU pieces in about 14 instructions.  Phi(x) = 0.5 (1 + erf(x / sqrt 2)) with erf from
// Abramowitz & Stegun 7.1.26 (absolute error below 1.5e-7):
//   erfc(z) = (a1 t + ... + a5 t^5) exp(-z^2),  t = 1 / (1 + 0.3275911 z),  z >= 0.
// With z = |x| / sqrt 2 the exponential is exp(-x^2 / 2), which is also what the Gaussian
// density in the derivative needs, so forward and derivative share one ex2 and one rcp.
struct GeluParts {
  float cdf;   // Phi(x)
  float gauss; // exp(-x^2 / 2)
};
__device__ __forceinline__ GeluParts gelu_parts(float x) {
  const float z = fabsf(x) * 0.70710678118654752f;
  float t;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.0f)));
  float poly = fmaf(0.5f * 1.061405429f, t, 0.5f * -1.453152027f);
  poly = fmaf(poly, t, 0.5f * 1.421413741f);
  poly = fmaf(poly, t, 0.5f * -0.284496736f);
  poly = fmaf(poly, t, 0.5f * 0.254829592f);
  poly *= t;
  GeluParts g;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(g.gauss) : "f"(x * (x * -0.72134752044448170f)));
  const float half_erfc = poly * g.gauss;  // 0.5 * erfc(|x| / sqrt 2)
  g.cdf = x >= 0.f ? 1.0f - half_erfc : half_erfc;
  return g;
}
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int ACT> __device__ __forceinline__ float act_fwd(float x) {
  if (ACT == kActRelu) return fmaxf(x, 0.f);
  if (ACT == kActGelu) return x * gelu_parts(x).cdf;
  if (ACT == kActGeluTanh) {
    const float u = 0.7978845608028654f * fmaf(0.044715f * x * x, x, x);
    return 0.5f * x * (1.0f + tanh_approx(u));
  }
  return x;
}
template <int ACT> __device__ __forceinline__ float act_grad(float x) {
  if (ACT == kActRelu) return x > 0.f ? 1.f : 0.f;
  if (ACT == kActGelu) {
    const GeluParts g = gelu_parts(x);
    return fmaf(x * 0.3989422804014327f, g.gauss, g.cdf);
  }
  if (ACT == kActGeluTanh) {
    const float x2 = x * x;
    const float u = 0.7978845608028654f * fmaf(0.044715f * x2, x, x);
    const float t = tanh_approx(u);
    const float du = 0.7978845608028654f * fmaf(3.0f * 0.044715f, x2, 1.0f);
    return fmaf(0.5f * x * (1.0f - t * t), du, 0.5f * (1.0f + t));
  }
  return 1.f;
}

template <typename T> struct Cvt;
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
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
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
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

// 256-bit global accesses (sm_100): one full 32-byte sector per lane and instruction.
__device__ __forceinline__ void ldg256(const void* p, uint32_t (&r)[8]) {
  asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                 "=r"(r[6]), "=r"(r[7])
               : "l"(p));
}
__device__ __forceinline__ void ld256(const void* p, uint32_t (&r)[8]) {
  asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                 "=r"(r[6]), "=r"(r[7])
               : "l"(p)
               : "memory");
}
__device__ __forceinline__ void st256(void* p, const uint32_t (&r)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// 32 consecutive 16-bit values (64 bytes, 32-byte aligned) held as 16 packed words.
struct Packed32 {
  uint32_t w[16];
};

// Stage a 32-row x 64-byte patch of a row-major 16-bit matrix into shared memory with
// coalesced 16-byte cp.async copies: per instruction 4 lanes cover one row, 8 rows per
// instruction.  Rows >= valid_rows are zero-filled without touching global memory.
__device__ __forceinline__ void stage_side(uint8_t* patch, const uint8_t* gbase, long row_pitch,
                                           int valid_rows, int lane) {
  const int seg = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = i * 8 + (lane >> 2);
    const bool ok = rr < valid_rows;
    const uint8_t* src = gbase + (ok ? rr : 0) * row_pitch + seg * 16;
    const uint32_t dst = ptx::smem_u32(patch + rr * SIDE_PITCH + seg * 16);
    const uint32_t bytes = ok ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
                 "r"(bytes)
                 : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

__device__ __forceinline__ void read_side(const uint8_t* patch, int lane, Packed32& d) {
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncwarp();
  const uint4* row = reinterpret_cast<const uint4*>(patch + lane * SIDE_PITCH);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 w = row[q];
    d.w[q * 4 + 0] = w.x;
    d.w[q * 4 + 1] = w.y;
    d.w[q * 4 + 2] = w.z;
    d.w[q * 4 + 3] = w.w;
  }
  __syncwarp();
}

template <typename T>
__device__ __forceinline__ void unpack32(const Packed32& s, float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) Cvt<T>::unpack(s.w[i], v[2 * i], v[2 * i + 1]);
}

template <typename T>
__device__ __forceinline__ void store32(T* dst, const float (&v)[32]) {
  uint32_t lo[8], hi[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    lo[i] = Cvt<T>::pack(v[2 * i], v[2 * i + 1]);
    hi[i] = Cvt<T>::pack(v[16 + 2 * i], v[16 + 2 * i + 1]);
  }
  st256(dst, lo);
  st256(reinterpret_cast<uint8_t*>(dst) + 32, hi);
}

__device__ __forceinline__ void fail(SharedAux* aux, int* status, int code) {
  aux->abort = 1;
  if (status != nullptr) atomicCAS(status, 0, code);
}

struct EpiTile {
  uint32_t t_row;
  int half;
  int lane;
  int n0;
  long out_row;
  int group;
  int warp_valid;
  bool row_ok;
  bool have_acc;
  bool use_aux;
  bool read_old;
  bool use_side;
  const uint8_t* side;
  long side_pitch;
  uint8_t* patch;
  uint8_t* out_row_base;    // first byte of this lane's output row (local, or a peer's slot row)
  bool remote_row;          // the row lives on another GPU: leave through bulk async stores
  const uint8_t* bias_sm;   // staged bias slices of this tile (null when there is no bias)
  uint64_t* empty_bar;      // accumulator-free barrier, signalled once the last tcgen05.ld landed
};

// Arithmetic and stores of one 32-column chunk held in `r` (raw accumulator bits).
template <int MODE, typename T, int ACT>
__device__ __forceinline__ void finish_chunk(const KernelParams& p, const EpiTile& et, int col0, int ch,
                                             const uint32_t (&r)[32], const Packed32& side_cur) {
  const long off = et.out_row * p.n + col0;
  if (MODE == kWgrad) {
    if (p.out_fp32) {
      float* dst = static_cast<float*>(p.out) + off;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t w[8];
        if (p.accumulate) {
          ld256(dst + q * 8, w);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            w[j] = __float_as_uint(__uint_as_float(w[j]) + (et.have_acc ? __uint_as_float(r[q * 8 + j]) : 0.f));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) w[j] = et.have_acc ? r[q * 8 + j] : 0u;
        }
        st256(dst + q * 8, w);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float a = et.have_acc ? __uint_as_float(r[q * 16 + 2 * j]) : 0.f;
          float b = et.have_acc ? __uint_as_float(r[q * 16 + 2 * j + 1]) : 0.f;
          if (et.read_old) {
            float oa, ob;
            Cvt<T>::unpack(side_cur.w[q * 8 + j], oa, ob);
            a += oa;
            b += ob;
          }
          w[j] = Cvt<T>::pack(a, b);
        }
        st256(reinterpret_cast<uint8_t*>(static_cast<T*>(p.out) + off) + q * 32, w);
      }
    }
  } else if (et.use_aux) {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float sa, sb;
        Cvt<T>::unpack(side_cur.w[q * 8 + j], sa, sb);
        const float a = __uint_as_float(r[q * 16 + 2 * j]) * act_grad<ACT>(sa);
        const float b = __uint_as_float(r[q * 16 + 2 * j + 1]) * act_grad<ACT>(sb);
        w[j] = Cvt<T>::pack(a, b);
      }
      st256(et.out_row_base + col0 * 2 + q * 32, w);
    }
  } else {
    const uint8_t* bias = et.bias_sm == nullptr ? nullptr : et.bias_sm + ch * 64;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t bw[8];
      if (bias != nullptr) {
        const uint4 b0 = *reinterpret_cast<const uint4*>(bias + q * 32);
        const uint4 b1 = *reinterpret_cast<const uint4*>(bias + q * 32 + 16);
        bw[0] = b0.x; bw[1] = b0.y; bw[2] = b0.z; bw[3] = b0.w;
        bw[4] = b1.x; bw[5] = b1.y; bw[6] = b1.z; bw[7] = b1.w;
      }
      uint32_t wp[8], wo[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float a = __uint_as_float(r[q * 16 + 2 * j]);
        float b = __uint_as_float(r[q * 16 + 2 * j + 1]);
        if (bias != nullptr) {
          float ba, bb;
          Cvt<T>::unpack(bw[j], ba, bb);
          a += ba;
          b += bb;
        }
        if (ACT != kActNone) {
          wp[j] = Cvt<T>::pack(a, b);
          a = act_fwd<ACT>(a);
          b = act_fwd<ACT>(b);
        }
        wo[j] = Cvt<T>::pack(a, b);
      }
      if (ACT != kActNone && p.pre_out != nullptr) {
        st256(reinterpret_cast<uint8_t*>(static_cast<T*>(p.pre_out) + off) + q * 32, wp);
      }
      if (et.remote_row) {
        // Rows bound for a peer are staged in this lane's 64-byte slot of the warp's patch and
        // leave as one bulk asynchronous store per chunk: NVLink sees 64-byte writes instead
        // of scattered 32-byte ones, and the warp does not wait for them.
        uint8_t* slot = et.patch + et.lane * SIDE_PITCH + q * 32;
        if (q == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        *reinterpret_cast<uint4*>(slot) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
        *reinterpret_cast<uint4*>(slot + 16) = make_uint4(wo[4], wo[5], wo[6], wo[7]);
        if (q == 1) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 64;" ::"l"(
                           et.out_row_base + col0 * 2),
                       "r"(ptx::smem_u32(et.patch + et.lane * SIDE_PITCH))
                       : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      } else {
        st256(et.out_row_base + col0 * 2 + q * 32, wo);
      }
    }
  }
}

// One output tile for one epilogue warp: its 32 rows and the four 32-column chunks
// 2 * i + half.  Two register buffers alternate: while chunk i is finished, the tcgen05.ld of
// chunk i + 1 and the staging of its side operand are in flight.
template <int MODE, typename T, int ACT>
__device__ __forceinline__ void epilogue_tile(const KernelParams& p, const EpiTile& et) {
  const int lane = et.lane;
  uint32_t ra[32], rb[32];
  bool released = false;
  const int first_col = et.n0 + et.half * 32;
  if (first_col < p.n) {
    if (et.have_acc) ptx::tmem_ld_32x32(et.t_row + et.half * 32, ra);

#pragma unroll 1
    for (int pair = 0; pair < CHUNKS_PER_WARP / 2; ++pair) {
      // ---- even chunk of the pair (held in ra)
      {
        const int cg = 2 * (2 * pair) + et.half;
        const int col0 = et.n0 + cg * 32;
        if (col0 >= p.n) break;
        if (et.have_acc) ptx::tmem_ld_wait();
        Packed32 side_cur;
        if (et.use_side) read_side(et.patch, lane, side_cur);
        if (col0 + 64 < p.n) {
          if (et.have_acc) ptx::tmem_ld_32x32(et.t_row + (cg + 2) * 32, rb);
          if (et.use_side) stage_side(et.patch, et.side + (cg + 2) * 64, et.side_pitch, et.warp_valid, lane);
        } else if (!released) {
          // nothing more to read from this accumulator: hand it back to the MMA warp now
          ptx::tc_fence_before_sync();
          ptx::mbar_arrive(et.empty_bar);
          released = true;
        }
        if (et.row_ok) finish_chunk<MODE, T, ACT>(p, et, col0, 2 * pair, ra, side_cur);
      }
      // ---- odd chunk of the pair (held in rb)
      {
        const int cg = 2 * (2 * pair + 1) + et.half;
        const int col0 = et.n0 + cg * 32;
        if (col0 >= p.n) break;
        if (et.have_acc) ptx::tmem_ld_wait();
        Packed32 side_cur;
        if (et.use_side) read_side(et.patch, lane, side_cur);
        if (pair + 1 < CHUNKS_PER_WARP / 2 && col0 + 64 < p.n) {
          if (et.have_acc) ptx::tmem_ld_32x32(et.t_row + (cg + 2) * 32, ra);
          if (et.use_side) stage_side(et.patch, et.side + (cg + 2) * 64, et.side_pitch, et.warp_valid, lane);
        } else if (!released) {
          ptx::tc_fence_before_sync();
          ptx::mbar_arrive(et.empty_bar);
          released = true;
        }
        if (et.row_ok) finish_chunk<MODE, T, ACT>(p, et, col0, 2 * pair + 1, rb, side_cur);
      }
    }
  }
  if (!released) {
    ptx::tc_fence_before_sync();
    ptx::mbar_arrive(et.empty_bar);
  }
}

template <int MODE, typename T, int ACT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a,
                    const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ KernelParams p) {
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
      ptx::mbar_init(&aux->tmem_empty[a], NUM_EPI_WARPS * 32);
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
  } else if (warp >= FIRST_EPI_WARP) {
    // ============================================================== epilogue (warps 4..11)
    const int part = warp & 3;                          // TMEM lane quarter this warp may read
    const int half = (warp - FIRST_EPI_WARP) >> 2;      // takes the 32-column chunks 2 * i + half
    uint8_t* patch = smem + STAGES * STAGE_BYTES + AUX_BYTES + (warp - FIRST_EPI_WARP) * SIDE_BYTES;
    uint8_t* bias_sm = smem + STAGES * STAGE_BYTES + AUX_BYTES + NUM_EPI_WARPS * SIDE_BYTES +
                       (warp - FIRST_EPI_WARP) * BIAS_BYTES;
    int iter = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++iter) {
      const TileCoord c = decode_tile<MODE>(p, aux, tile);
      const int rows = c.row_end - c.row_begin;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;

      // Rows of the output matrix covered by this warp: [warp_row0, warp_row0 + warp_valid).
      long warp_row0;
      int warp_valid;
      if (MODE == kWgrad) {
        const int m0 = c.m_tile * BM + part * 32;
        warp_row0 = static_cast<long>(c.group) * p.m + m0;
        warp_valid = min(32, p.m - m0);
      } else {
        const int r0 = c.m_tile * BM + part * 32;
        warp_row0 = static_cast<long>(c.row_begin) + r0;
        warp_valid = min(32, rows - r0);
      }
      const bool row_ok = lane < warp_valid;
      const long out_row = warp_row0 + lane;
      const bool have_acc = (MODE != kWgrad) || rows > 0;
      const int n0 = c.n_tile * BN;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(part * 32) << 16) + acc * BN;
      const bool use_aux = (MODE != kWgrad) && p.epi == kEpiDAct;
      const bool read_old = (MODE == kWgrad) && p.accumulate && !p.out_fp32;
      const bool use_side = (use_aux || read_old) && warp_valid > 0;
      const uint8_t* side = reinterpret_cast<const uint8_t*>(use_aux ? p.aux : p.out) +
                            (warp_row0 * p.n + n0) * 2;
      const long side_pitch = static_cast<long>(p.n) * 2;
      const int first_col = n0 + half * 32;

      if constexpr (MODE == kWgrad) {
        // The bias gradient of a grouped linear is the per-group column sum of the matrix the
        // weight gradient takes as P.  The epilogue warps have nothing to do while the main
        // loop of this tile runs, so on the tiles of the first N column block they add up the
        // tile's 128 columns of P over the group's rows with plain 16-byte loads (the rows are
        // on their way through L2 for the TMA loads of this and the neighbouring CTAs) and
        // write the sums in the operands' type: no extra launch, no atomics, no scratch.
        if (p.psum != nullptr && c.n_tile == 0) {
          const int ew = warp - FIRST_EPI_WARP;
          const int col = c.m_tile * BM + (lane & 15) * 8;
          float cs[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) cs[q] = 0.f;
          if (col < p.m) {
            const T* src = static_cast<const T*>(p.psrc) + col;
            int r = c.row_begin + ew * 2 + (lane >> 4);
            constexpr int kUnroll = 8;
            for (; r + 16 * (kUnroll - 1) < c.row_end; r += 16 * kUnroll) {
              uint4 v[kUnroll];
#pragma unroll
              for (int i = 0; i < kUnroll; ++i) {
                v[i] = __ldg(reinterpret_cast<const uint4*>(src + static_cast<long>(r + 16 * i) * p.m));
              }
#pragma unroll
              for (int i = 0; i < kUnroll; ++i) {
                float a, b;
                Cvt<T>::unpack(v[i].x, a, b); cs[0] += a; cs[1] += b;
                Cvt<T>::unpack(v[i].y, a, b); cs[2] += a; cs[3] += b;
                Cvt<T>::unpack(v[i].z, a, b); cs[4] += a; cs[5] += b;
                Cvt<T>::unpack(v[i].w, a, b); cs[6] += a; cs[7] += b;
              }
            }
            for (; r < c.row_end; r += 16) {
              const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + static_cast<long>(r) * p.m));
              float a, b;
              Cvt<T>::unpack(v.x, a, b); cs[0] += a; cs[1] += b;
              Cvt<T>::unpack(v.y, a, b); cs[2] += a; cs[3] += b;
              Cvt<T>::unpack(v.z, a, b); cs[4] += a; cs[5] += b;
              Cvt<T>::unpack(v.w, a, b); cs[6] += a; cs[7] += b;
            }
          }
          float* mine_f = reinterpret_cast<float*>(patch);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            cs[q] += __shfl_xor_sync(0xffffffffu, cs[q], 16);
            if (lane < 16) mine_f[lane * 8 + q] = cs[q];
          }
          asm volatile("bar.sync 2, %0;" ::"n"(NUM_EPI_WARPS * 32) : "memory");
          const int tid = static_cast<int>(threadIdx.x) - FIRST_EPI_WARP * 32;
          if (tid < BM && c.m_tile * BM + tid < p.m) {
            const uint8_t* first = smem + STAGES * STAGE_BYTES + AUX_BYTES;
            float total = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < NUM_EPI_WARPS; ++w8) {
              total += reinterpret_cast<const float*>(first + w8 * SIDE_BYTES)[tid];
            }
            T* dst = static_cast<T*>(p.psum) + static_cast<long>(c.group) * p.m + c.m_tile * BM + tid;
            if (p.accumulate) total += Cvt<T>::to_f(*dst);
            *dst = Cvt<T>::from_f(total);
          }
          asm volatile("bar.sync 2, %0;" ::"n"(NUM_EPI_WARPS * 32) : "memory");
        }
      }
      // The side operand (saved pre-activation, or the old gradient when accumulating) does
      // not depend on the accumulator: fetch its first chunk before waiting for the MMAs.
      if (use_side && first_col < p.n) {
        stage_side(patch, side + half * 64, side_pitch, warp_valid, lane);
      }
      // Bias slices of this warp's four chunks go to shared memory once per tile.
      const bool use_bias = (MODE != kWgrad) && !use_aux && p.bias != nullptr;
      if (use_bias) {
        __syncwarp();
        if (lane < CHUNKS_PER_WARP * 4) {
          const int q = lane >> 2, seg = lane & 3;
          const int col = n0 + (2 * q + half) * 32;
          if (col < p.n) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>(p.bias) +
                                 (static_cast<long>(c.group) * p.n + col) * 2 + seg * 16;
            *reinterpret_cast<uint4*>(bias_sm + q * 64 + seg * 16) =
                __ldg(reinterpret_cast<const uint4*>(src));
          }
        }
        __syncwarp();
      }
      // Pull the side operand of the next tile of this CTA towards L2 while this tile is
      // being finished: each lane asks for two of the four 128-byte lines of its row.
      if (use_aux && tile + static_cast<int>(gridDim.x) < total_tiles) {
        const TileCoord nx = decode_tile<MODE>(p, aux, tile + gridDim.x);
        const int r0 = nx.m_tile * BM + part * 32 + lane;
        if (r0 < nx.row_end - nx.row_begin) {
          const uint8_t* row = reinterpret_cast<const uint8_t*>(p.aux) +
                               ((static_cast<long>(nx.row_begin) + r0) * p.n + nx.n_tile * BN) * 2;
#pragma unroll
          for (int l = 0; l < 2; ++l) {
            const int line = half * 2 + l;
            if (nx.n_tile * BN + line * 64 < p.n) {
              asm volatile("prefetch.global.L2 [%0];" ::"l"(row + line * 128));
            }
          }
        }
      }

      if (!ptx::mbar_wait(&aux->tmem_full[acc], acc_phase, abort_flag)) {
        if (lane == 0) fail(aux, p.status, STATUS_TIMEOUT_EPILOGUE);
        break;
      }
      ptx::tc_fence_after_sync();

      EpiTile et;
      et.t_row = t_row;
      et.half = half;
      et.lane = lane;
      et.n0 = n0;
      et.out_row = out_row;
      et.group = c.group;
      et.warp_valid = warp_valid;
      et.row_ok = row_ok;
      et.have_acc = have_acc;
      et.use_aux = use_aux;
      et.read_old = read_old;
      et.use_side = use_side;
      et.side = side;
      et.side_pitch = side_pitch;
      et.patch = patch;
      if (MODE != kWgrad && p.push_meta != nullptr) {
        // Fused combine: this lane's output row lives in the source rank's return buffer.
        et.out_row_base = nullptr;
        et.remote_row = false;
        if (row_ok) {
          const int64_t m = p.push_meta[out_row];
          const int src = static_cast<int>(m >> 32);
          const long slot = static_cast<long>(m & 0xffffffffll);
          et.out_row_base = static_cast<uint8_t*>(p.push_dst.p[src]) + slot * p.n * 2;
          et.remote_row = src != p.push_me;
        }
      } else {
        et.out_row_base = static_cast<uint8_t*>(p.out) + out_row * p.n * 2;
        et.remote_row = false;
      }
      et.bias_sm = use_bias ? bias_sm : nullptr;
      et.empty_bar = &aux->tmem_empty[acc];
      epilogue_tile<MODE, T, ACT>(p, et);
    }
    if (MODE != kWgrad && p.push_meta != nullptr) {
      // All rows of this CTA are on their way: wait for the bulk stores, order everything
      // before the completion count; the last CTA of the grid publishes the epoch on every
      // peer's return channel.
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async;" ::: "memory");
      __threadfence_system();
      asm volatile("bar.sync 1, %0;" ::"n"(NUM_EPI_WARPS * 32) : "memory");
      if (threadIdx.x == FIRST_EPI_WARP * 32) {
        const int prev = atomicAdd(p.push_counter, 1);
        if (prev == static_cast<int>(gridDim.x) - 1) {
          *p.push_counter = 0;
          __threadfence_system();
          const int epoch = *p.push_epoch;
          for (int peer = 0; peer < p.push_world; ++peer) {
            int* flag = static_cast<int*>(p.push_flags.p[peer]) + kChanReturn * kMaxPeers + p.push_me;
            asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
          }
        }
      }
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


// ------------------------------------------------------------------------------- launch
template <int MODE, typename T, int ACT>
cudaError_t launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const KernelParams& kp,
                       int grid, cudaStream_t stream) {
  // The shared-memory attribute is per device; remember which devices of this process have it.
  static std::mutex mu;
  static uint64_t configured = 0;
  auto kernel = grouped_gemm_kernel<MODE, T, ACT>;
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

template <int MODE, typename T>
cudaError_t launch_act(const CUtensorMap& ta, const CUtensorMap& tb, const KernelParams& kp,
                       int grid, cudaStream_t stream) {
  switch (kp.act) {
    case kActRelu: return launch_one<MODE, T, kActRelu>(ta, tb, kp, grid, stream);
    case kActGelu: return launch_one<MODE, T, kActGelu>(ta, tb, kp, grid, stream);
    case kActGeluTanh: return launch_one<MODE, T, kActGeluTanh>(ta, tb, kp, grid, stream);
    default: return launch_one<MODE, T, kActNone>(ta, tb, kp, grid, stream);
  }
}

// One translation unit per element type instantiates this.
template <typename T>
cudaError_t launch_for_type(int mode, const CUtensorMap& ta, const CUtensorMap& tb,
                            const KernelParams& kp, int grid, cudaStream_t stream) {
  switch (mode) {
    case kRowsNT: return launch_act<kRowsNT, T>(ta, tb, kp, grid, stream);
    case kRowsNN: return launch_act<kRowsNN, T>(ta, tb, kp, grid, stream);
    default: return launch_one<kWgrad, T, kActNone>(ta, tb, kp, grid, stream);
  }
}

cudaError_t launch_bf16(int mode, const CUtensorMap& ta, const CUtensorMap& tb,
                        const KernelParams& kp, int grid, cudaStream_t stream);
cudaError_t launch_f16(int mode, const CUtensorMap& ta, const CUtensorMap& tb,
                       const KernelParams& kp, int grid, cudaStream_t stream);

}  // namespace gg
}  // namespace fmoe
