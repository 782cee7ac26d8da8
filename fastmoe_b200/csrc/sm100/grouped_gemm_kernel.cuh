// Grouped GEMM on the 5th-generation tensor cores (tcgen05) for the expert linears.
//
// Replaces the reference's host loop of one cuBLAS call per expert with stream
// synchronisations around it (cuda/parallel_linear.cuh:56-163): one persistent kernel covers
// every expert, reads the expert row offsets from device memory (no host counts), and fuses
// bias, activation, activation-derivative and dtype conversion into its epilogue.
//
// Structure of a CTA (384 threads = 3 warpgroups, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer: plain cp.async.bulk.tensor loads into a 4-stage ring of
//               128-byte-swizzled shared-memory tiles, completion on mbarriers;
//   warp 1      one elected thread issues tcgen05.mma (128 x 256 x 16 per instruction, fp32
//               accumulators in TMEM) and tcgen05.commit; the warp owns the TMEM allocation;
//   warps 2-3   idle, or row senders of the fused dispatch (see below);
//   warps 4-11  epilogue (two warpgroups): two warps per TMEM lane quarter.  Row modes: each
//               warp owns 32 rows x 128 columns of the tile; the tcgen05.ld of chunk i+1 and
//               the load of its saved pre-activation are in flight while chunk i gets bias /
//               activation / derivative and is written into the lane's row of a swizzled
//               per-warp shared-memory patch; after every second chunk the warp stores whole
//               128-byte lines of the 32 rows (8 lanes per row), locally or into a peer's
//               return buffer over NVLink.  The pre-activation is kept in a tile-blocked
//               layout that both its producer and its consumer access with fully coalesced
//               16-byte accesses straight from registers.  Weight-gradient mode: alternate
//               32-column chunks, 32-byte stores.
// Two 256-column accumulators (all 512 TMEM columns) let the epilogue of tile i overlap the
// main loop of tile i+1.
//
// Optional roles of a row-mode launch (expert parallelism):
//   * sender warps (warps 2 and 3 of every CTA): they copy this rank's token rows through
//     registers into the owning peers' receive buffers and publish per-(row block, source)
//     arrival flags;
//   * gated producer: the TMA warp waits (bounded) for the arrival flags of a tile's row
//     block before loading it, so GEMM tiles start as their rows land.
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
constexpr int MAX_GROUPS = 256;
constexpr int NUM_EPI_WARPS = 8;
constexpr int FIRST_EPI_WARP = 4;
constexpr int NUM_THREADS = (FIRST_EPI_WARP + NUM_EPI_WARPS) * 32;



constexpr int CHUNKS_PER_WARP = BN / 32 / 2;  // 4 chunks of 32 columns per epilogue warp
constexpr int SIDE_PITCH = 80;                // bytes per staged row (64 data + 16 pad: no bank conflicts)
constexpr int SIDE_BYTES = 32 * SIDE_PITCH;   // weight-gradient mode: one 32-row x 32-column patch per epilogue warp
constexpr int PATCH_PITCH = 128;              // row modes: one 128-byte line (two 32-column chunks) of a row, 16-byte pieces XOR-swizzled by row
constexpr int PATCH_BYTES = 32 * PATCH_PITCH; // 32 rows per epilogue warp
// Tile-blocked layout of the saved pre-activation: per output tile 8 warps x 4 chunks x 2 KB,
// each 2 KB being 4 pieces x 32 lanes x 16 bytes in exactly the order the epilogue threads
// produce (first GEMM) and consume (activation derivative of the input-gradient GEMM) them.
constexpr int PRE_TILE_BYTES = BM * BN * 2;
constexpr int PRE_CHUNK_BYTES = 32 * 64;
constexpr int TMEM_COLS = 512;

// Sender warps (warps 2 and 3 of every CTA): a unit of work is SEND_UNIT_ROWS consecutive
// destination rows of one 128-row block.  Small units put the first arrival flags up early (the
// tiles of the first wave all wait for them); SEND_ROWS_IN_FLIGHT rows are loaded before any is
// stored, which is what bounds a warp's bytes in flight.
constexpr int SEND_UNIT_ROWS = 8;
constexpr int SEND_ROWS_IN_FLIGHT = 4;
constexpr int SEND_UNITS_PER_ITEM = BM / SEND_UNIT_ROWS;
constexpr int FIRST_SEND_WARP = 2;
constexpr int BLK_ORDER_SHIFT = 20;   // (group << 20) | block, as written by the count exchange
constexpr int TRACE_SLOTS = 10;  // time stamps and counters per CTA when tracing is on
constexpr int NUM_SEND_WARPS = 2;
constexpr int NUM_WARPS = FIRST_EPI_WARP + NUM_EPI_WARPS;

constexpr int STATUS_TIMEOUT_PRODUCER = 101;
constexpr int STATUS_TIMEOUT_MMA = 102;
constexpr int STATUS_TIMEOUT_EPILOGUE = 103;
constexpr int STATUS_TIMEOUT_SENDER = 104;
constexpr int STATUS_BAD_PUSH_META = 105;    // a row's (source, slot) word was out of range: row skipped

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
template <int MODE> struct Layout {
  static constexpr int kStages = STAGES;
  static constexpr int kPatch = (MODE == kWgrad) ? SIDE_BYTES : PATCH_BYTES;
  static constexpr int kAuxOff = kStages * STAGE_BYTES;
  static constexpr int kEpiOff = kAuxOff + AUX_BYTES;
  static constexpr int kBytes = kEpiOff + NUM_EPI_WARPS * kPatch + 1024;
};
static_assert(Layout<kRowsNT>::kBytes <= 232448 && Layout<kWgrad>::kBytes <= 232448, "shared memory");
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
  long push_slots;
  SendArgs send;
  GateArgs gate;
  unsigned long long* trace;
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
  TileCoord c;
  const int n_tiles = (p.n + BN - 1) / BN;
  if (MODE != kWgrad && p.gate.blk_order != nullptr) {
    // Row blocks in the order given by the caller (arrival order under expert parallelism).
    const int i = tile / n_tiles;
    const int packed = __ldg(p.gate.blk_order + i);
    c.group = min(packed >> BLK_ORDER_SHIFT, p.num_groups - 1);
    c.m_tile = packed & ((1 << BLK_ORDER_SHIFT) - 1);
    c.n_tile = tile - i * n_tiles;
    c.row_begin = p.offs[c.group];
    c.row_end = p.offs[c.group + 1];
    return c;
  }
  // Binary search of the group whose tile range contains `tile`.
  int lo = 0, hi = p.num_groups;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (aux->tile_prefix[mid] <= tile) lo = mid; else hi = mid;
  }
  c.group = lo;
  const int local = tile - aux->tile_prefix[lo];
  c.m_tile = local / n_tiles;
  c.n_tile = local - c.m_tile * n_tiles;
  c.row_begin = p.offs[lo];
  c.row_end = p.offs[lo + 1];
  return c;
}

// Where a tile's block of the tile-blocked pre-activation lives: groups in order, whatever
// order the tiles are walked in.
__device__ __forceinline__ long pre_tile_index(const KernelParams& p, const SharedAux* aux,
                                               const TileCoord& c) {
  const int n_tiles = (p.n + BN - 1) / BN;
  return static_cast<long>(aux->tile_prefix[c.group]) + c.m_tile * n_tiles + c.n_tile;
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
template <int PITCH = SIDE_PITCH>
__device__ __forceinline__ void stage_side(uint8_t* patch, const uint8_t* gbase, long row_pitch,
                                           int valid_rows, int lane) {
  const int seg = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = i * 8 + (lane >> 2);
    const bool ok = rr < valid_rows;
    const uint8_t* src = gbase + (ok ? rr : 0) * row_pitch + seg * 16;
    const uint32_t dst = ptx::smem_u32(patch + rr * PITCH + seg * 16);
    const uint32_t bytes = ok ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
                 "r"(bytes)
                 : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

template <int PITCH = SIDE_PITCH>
__device__ __forceinline__ void read_side(const uint8_t* patch, int lane, Packed32& d) {
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncwarp();
  const uint4* row = reinterpret_cast<const uint4*>(patch + lane * PITCH);
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
  if (status != nullptr) record_failure(status, code);
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


// ------------------------------------------------------------------------------------------
// Row modes: outputs leave through a shared-memory patch as whole 128-byte lines.
// ------------------------------------------------------------------------------------------
struct RowTile {
  uint32_t t_row;          // TMEM address: this warp's lane quarter, first column of its span
  int lane;
  int col_first;           // first output column of this warp's 128-column span
  int n_chunks;            // valid 32-column chunks of the span (0..4)
  bool row_ok;
  bool use_aux;            // multiply by the activation derivative of the saved pre-activation
  uint8_t* patch;          // this warp's 32 rows x 128 bytes
  uint8_t* out_row;        // column 0 of this lane's output row (local or a peer's); null = no store
  uint8_t* pre_tile;       // this warp's 4 x 2 KB of the tile-blocked pre-activation (out or in), or null
  const uint8_t* bias;     // bias of the span's first column (global memory), or null
  uint64_t* empty_bar;
};

// 16-byte piece `c` (0..7) of patch row `row`; pieces are XOR-swizzled so that 32 lanes writing
// the same piece of 32 different rows, and 8 lanes reading the 8 pieces of one row, are both
// free of bank conflicts.
__device__ __forceinline__ uint8_t* patch_piece(uint8_t* patch, int row, int c) {
  return patch + row * PATCH_PITCH + ((c ^ (row & 7)) << 4);
}

__device__ __forceinline__ void load_pre_chunk(const uint8_t* pre_tile, int i, int lane, Packed32& d) {
  const uint8_t* base = pre_tile + i * PRE_CHUNK_BYTES + lane * 16;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(base + q * 512));
    d.w[q * 4 + 0] = w.x;
    d.w[q * 4 + 1] = w.y;
    d.w[q * 4 + 2] = w.z;
    d.w[q * 4 + 3] = w.w;
  }
}

// Bias / activation (or activation derivative) of one 32-column chunk.  The output values go
// into the lane's own row of the patch (half (i & 1) of the line); the pre-activation, when
// wanted, goes straight to its tile-blocked buffer with fully coalesced 16-byte stores.
template <typename T, int ACT>
__device__ __forceinline__ void rows_chunk(const RowTile& rt, int i, bool with_pre,
                                           const uint32_t (&r)[32], const Packed32& side_cur) {
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    uint32_t wo[8];
    if (rt.use_aux) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float sa, sb;
        Cvt<T>::unpack(side_cur.w[q * 8 + j], sa, sb);
        const float a = __uint_as_float(r[q * 16 + 2 * j]) * act_grad<ACT>(sa);
        const float b = __uint_as_float(r[q * 16 + 2 * j + 1]) * act_grad<ACT>(sb);
        wo[j] = Cvt<T>::pack(a, b);
      }
    } else {
      uint32_t bw[8];
      if (rt.bias != nullptr) {
        const uint4 b0 = __ldg(reinterpret_cast<const uint4*>(rt.bias + i * 64 + q * 32));
        const uint4 b1 = __ldg(reinterpret_cast<const uint4*>(rt.bias + i * 64 + q * 32 + 16));
        bw[0] = b0.x; bw[1] = b0.y; bw[2] = b0.z; bw[3] = b0.w;
        bw[4] = b1.x; bw[5] = b1.y; bw[6] = b1.z; bw[7] = b1.w;
      }
      uint32_t wp[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float a = __uint_as_float(r[q * 16 + 2 * j]);
        float b = __uint_as_float(r[q * 16 + 2 * j + 1]);
        if (rt.bias != nullptr) {
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
      if (ACT != kActNone && with_pre) {
        uint8_t* pd = rt.pre_tile + i * PRE_CHUNK_BYTES + rt.lane * 16 + q * 1024;
        *reinterpret_cast<uint4*>(pd) = make_uint4(wp[0], wp[1], wp[2], wp[3]);
        *reinterpret_cast<uint4*>(pd + 512) = make_uint4(wp[4], wp[5], wp[6], wp[7]);
      }
    }
    if (rt.row_ok) {
      const int c = (i & 1) * 4 + q * 2;
      *reinterpret_cast<uint4*>(patch_piece(rt.patch, rt.lane, c)) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
      *reinterpret_cast<uint4*>(patch_piece(rt.patch, rt.lane, c + 1)) = make_uint4(wo[4], wo[5], wo[6], wo[7]);
    }
  }
}

// After an odd chunk (or the last one): the line of every valid row goes to its destination,
// 8 lanes per row with 16-byte accesses, four rows per instruction — whole 128-byte lines,
// local or over NVLink.
__device__ __forceinline__ void rows_send(const RowTile& rt, int i) {
  const bool last = i + 1 == rt.n_chunks;
  if (!(last || (i & 1))) return;
  const int bytes = ((i & 1) + 1) * 64;
  const long dst_off = static_cast<long>(rt.col_first + (i & ~1) * 32) * 2;
  const int sub = rt.lane & 7;
  const unsigned long long mine =
      rt.row_ok ? reinterpret_cast<unsigned long long>(rt.out_row) : 0ull;
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int row = 4 * it + (rt.lane >> 3);
    const unsigned long long dst = __shfl_sync(0xffffffffu, mine, row);
    if (dst != 0ull && sub * 16 < bytes) {
      const uint4 v = *reinterpret_cast<const uint4*>(patch_piece(rt.patch, row, sub));
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(dst) + dst_off + sub * 16) = v;
    }
  }
  __syncwarp();  // the next pair of chunks overwrites the patch
}

// One output tile for one epilogue warp in the row modes: 32 rows x up to four contiguous
// 32-column chunks.  Two register buffers alternate: while chunk i is finished, the tcgen05.ld
// of chunk i + 1 and the load of its saved pre-activation are in flight.
template <typename T, int ACT>
__device__ __forceinline__ void epilogue_tile_rows(const RowTile& rt, Packed32& side_first) {
  const int lane = rt.lane;
  const bool with_pre = (ACT != kActNone) && !rt.use_aux && rt.pre_tile != nullptr;
  uint32_t ra[32], rb[32];
  Packed32 sb;
  bool released = false;
  if (rt.n_chunks > 0) {
    ptx::tmem_ld_32x32(rt.t_row, ra);
#pragma unroll 1
    for (int pair = 0; pair < CHUNKS_PER_WARP / 2; ++pair) {
      {
        const int i = 2 * pair;
        if (i >= rt.n_chunks) break;
        ptx::tmem_ld_wait();
        if (i + 1 < rt.n_chunks) {
          ptx::tmem_ld_32x32(rt.t_row + (i + 1) * 32, rb);
          if (rt.use_aux) load_pre_chunk(rt.pre_tile, i + 1, lane, sb);
        } else if (!released) {
          ptx::tc_fence_before_sync();
          ptx::mbar_arrive(rt.empty_bar);
          released = true;
        }
        rows_chunk<T, ACT>(rt, i, with_pre, ra, side_first);
        rows_send(rt, i);
      }
      {
        const int i = 2 * pair + 1;
        if (i >= rt.n_chunks) break;
        ptx::tmem_ld_wait();
        if (i + 1 < rt.n_chunks) {
          ptx::tmem_ld_32x32(rt.t_row + (i + 1) * 32, ra);
          if (rt.use_aux) load_pre_chunk(rt.pre_tile, i + 1, lane, side_first);
        } else if (!released) {
          ptx::tc_fence_before_sync();
          ptx::mbar_arrive(rt.empty_bar);
          released = true;
        }
        rows_chunk<T, ACT>(rt, i, with_pre, rb, sb);
        rows_send(rt, i);
      }
    }
  }
  if (!released) {
    ptx::tc_fence_before_sync();
    ptx::mbar_arrive(rt.empty_bar);
  }
}


// ------------------------------------------------------------------------------------------
// Sender warps: the dispatch direction of the exchange inside a GEMM launch.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_sys_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_i32(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys_i32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One item of sender work: the part of one 128-row block of a peer's expert segment that this
// rank's rows fill.  Rows are relative to the first row of the expert's segment on the owner.
struct SendItem {
  int peer;
  int blk;      // block index inside the peer's flag array
  int r_lo;     // rows [r_lo, r_hi) of the segment
  int r_hi;
  int rel0;     // segment row of this rank's first row for the expert
  long seg;     // first row of the segment in the peer's receive buffer
  int src0;     // index into `pos` of this rank's first slot of the expert
};

// Send order: peer distance j outer (j = 0 is this rank itself), local expert e inner — first
// everything that stays on this GPU, then the rows of the next rank, and so on; receivers walk
// their tiles in the matching order.  The count-exchange kernel builds `item_prefix` in the
// same order.
__device__ __forceinline__ int send_order_expert(const SendArgs& s, int q) {
  const int j = q / s.n_expert;
  const int e = q - j * s.n_expert;
  int peer = s.me + j;
  if (peer >= s.world) peer -= s.world;
  return peer * s.n_expert + e;
}

__device__ __forceinline__ SendItem send_decode(const SendArgs& s, int tot, int item) {
  int lo = 0, hi = tot;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(s.item_prefix + mid) <= item) lo = mid; else hi = mid;
  }
  const int g = send_order_expert(s, lo);
  SendItem it;
  it.peer = g / s.n_expert;
  const int seg = __ldg(s.seg_base + g);
  const int cnt = __ldg(s.my_offs + g + 1) - __ldg(s.my_offs + g);
  const int rel0 = __ldg(s.dst_base + g) - seg;
  int r_end = rel0 + cnt;
  if (r_end > s.capacity - seg) r_end = s.capacity - seg;
  const int b = rel0 / BM + (item - __ldg(s.item_prefix + lo));
  it.blk = __ldg(s.blk_base + g) + b;
  it.r_lo = max(rel0, b * BM);
  it.r_hi = min(r_end, (b + 1) * BM);
  it.rel0 = rel0;
  it.seg = seg;
  it.src0 = __ldg(s.my_offs + g);
  return it;
}

// The per-expert tables of the send order, one entry per lane (used when world * n_expert <= 32):
// decoding an item then costs one ballot and a few shuffles instead of a chain of dependent
// loads in front of every unit.
struct SendLaneTable {
  int prefix;   // first item of send-order entry `lane`
  int seg;      // first row of the expert's segment in the owner's receive buffer
  int off0;     // index into `pos` of this rank's first slot of the expert
  int cnt;      // this rank's rows for the expert
  int rel0;     // segment row of this rank's first row
  int blkb;     // first flag block of the segment on the owner
  int peer;
};

__device__ __forceinline__ SendLaneTable send_lane_table(const SendArgs& s, int tot, int lane) {
  SendLaneTable t;
  t.prefix = 0x7fffffff;
  t.seg = t.off0 = t.cnt = t.rel0 = t.blkb = t.peer = 0;
  if (lane < tot) {
    const int g = send_order_expert(s, lane);
    t.prefix = __ldg(s.item_prefix + lane);
    t.seg = __ldg(s.seg_base + g);
    t.off0 = __ldg(s.my_offs + g);
    t.cnt = __ldg(s.my_offs + g + 1) - t.off0;
    t.rel0 = __ldg(s.dst_base + g) - t.seg;
    t.blkb = __ldg(s.blk_base + g);
    t.peer = g / s.n_expert;
  }
  return t;
}

__device__ __forceinline__ SendItem send_decode_lanes(const SendArgs& s, const SendLaneTable& t, int item) {
  // entries are in send order and their first items never decrease: the entry of `item` is the
  // last one whose first item is <= item
  const int lo = __popc(__ballot_sync(0xffffffffu, t.prefix <= item)) - 1;
  const int first = __shfl_sync(0xffffffffu, t.prefix, lo);
  const int seg = __shfl_sync(0xffffffffu, t.seg, lo);
  const int cnt = __shfl_sync(0xffffffffu, t.cnt, lo);
  const int rel0 = __shfl_sync(0xffffffffu, t.rel0, lo);
  SendItem it;
  it.peer = __shfl_sync(0xffffffffu, t.peer, lo);
  int r_end = rel0 + cnt;
  if (r_end > s.capacity - seg) r_end = s.capacity - seg;
  const int b = rel0 / BM + (item - first);
  it.blk = __shfl_sync(0xffffffffu, t.blkb, lo) + b;
  it.r_lo = max(rel0, b * BM);
  it.r_hi = min(r_end, (b + 1) * BM);
  it.rel0 = rel0;
  it.seg = seg;
  it.src0 = __shfl_sync(0xffffffffu, t.off0, lo);
  return it;
}

// One sender warp.  Units are dealt round-robin over all sender warps of the grid; the units of
// an item are therefore in flight on different warps at once and the item's flag goes up
// early.  A row travels global -> registers -> (peer) global, 16 bytes per lane and access,
// SEND_ROWS_IN_FLIGHT rows at a time; nothing here waits for anything.
template <typename T>
__device__ __forceinline__ void sender_warp(const KernelParams& p, int sender_id, int n_senders,
                                            int lane, unsigned long long* stamps) {
  const SendArgs& s = p.send;
  constexpr int R = SEND_ROWS_IN_FLIGHT;
  // `stamps` (tracing, one warp per CTA): when the warp's first unit had its slot ids, had issued
  // its stores, had passed the fence, had counted / signalled
  int stamp_at = (stamps != nullptr && lane == 0) ? 0 : 4;
  auto stamp = [&]() {
    if (stamp_at < 4) stamps[stamp_at++] = ptx::globaltimer();
  };
  const int tot = s.world * s.n_expert;
  const int total_items = __ldg(s.item_prefix + tot);
  const int total_units = total_items * SEND_UNITS_PER_ITEM;
  const int epoch = *s.epoch;
  const int nv = s.d >> 3;                    // 16-byte pieces per row
  const bool scaled = s.scale != nullptr;
  const bool lanes_hold_tables = tot <= 32;
  SendLaneTable table;
  if (lanes_hold_tables) table = send_lane_table(s, tot, lane);
  for (int u = sender_id; u < total_units; u += n_senders) {
    const int item = u / SEND_UNITS_PER_ITEM;
    const SendItem it = lanes_hold_tables ? send_decode_lanes(s, table, item) : send_decode(s, tot, item);
    const int r0 = it.r_lo + (u - item * SEND_UNITS_PER_ITEM) * SEND_UNIT_ROWS;
    const int r1 = min(r0 + SEND_UNIT_ROWS, it.r_hi);
    if (r0 >= r1) continue;
    // the first lanes fetch the slot ids (and scales) of the unit's rows with one load
    int slot_of = -1;
    float scale_of = 1.f;
    T* dst_rows = static_cast<T*>(s.rows.p[it.peer]);
    int64_t* dst_meta = static_cast<int64_t*>(s.meta.p[it.peer]);
    if (r0 + lane < r1) {
      slot_of = __ldg(s.pos + it.src0 + (r0 + lane - it.rel0));
      if (scaled) scale_of = Cvt<T>::to_f(static_cast<const T*>(s.scale)[slot_of]);
      if (dst_meta != nullptr) {
        dst_meta[it.seg + r0 + lane] = (static_cast<int64_t>(s.me) << 32) | static_cast<int64_t>(slot_of);
      }
    }
    if (stamp_at == 0) stamp();
    for (int r = r0; r < r1; r += R) {
      const uint4* in[R];
      uint4* out[R];
      float sc[R];
      bool on[R];
#pragma unroll
      for (int t = 0; t < R; ++t) {
        on[t] = r + t < r1;
        const int from = on[t] ? r + t - r0 : r - r0;
        const int sl = __shfl_sync(0xffffffffu, slot_of, from);
        sc[t] = __shfl_sync(0xffffffffu, scale_of, from);
        in[t] = reinterpret_cast<const uint4*>(static_cast<const T*>(s.x) + static_cast<long>(sl / s.k) * s.d);
        out[t] = reinterpret_cast<uint4*>(dst_rows + (it.seg + r + t) * s.d);
      }
      for (int i0 = lane; i0 < nv; i0 += 128) {
        uint4 v[R][4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (i0 + q * 32 < nv) {
#pragma unroll
            for (int t = 0; t < R; ++t) {
              if (on[t]) v[t][q] = __ldg(in[t] + i0 + q * 32);
            }
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (i0 + q * 32 < nv) {
#pragma unroll
            for (int t = 0; t < R; ++t) {
              if (!on[t]) continue;
              if (scaled) {
                uint32_t* w = reinterpret_cast<uint32_t*>(&v[t][q]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float a, b;
                  Cvt<T>::unpack(w[j], a, b);
                  w[j] = Cvt<T>::pack(a * sc[t], b * sc[t]);
                }
              }
              out[t][i0 + q * 32] = v[t][q];
            }
          }
        }
      }
    }
    // Every lane orders its own stores, lane 0 then counts the unit's rows; the warp that
    // completes the item clears the counter and raises the flag on the owner.  Rows that stay
    // on this GPU need device scope only (writer and reader are both here); a system-scope
    // fence costs far more and is kept for rows that went to a peer.
    const bool local = it.peer == s.me;
    if (stamp_at == 1) stamp();
    if (local) __threadfence(); else __threadfence_system();
    __syncwarp();
    if (stamp_at == 2) stamp();
    if (lane == 0) {
      const int n = r1 - r0;
      const int old = atomicAdd(s.item_count + item, n);
      if (old + n == it.r_hi - it.r_lo) {
        s.item_count[item] = 0;
        int* flag = static_cast<int*>(s.flags.p[it.peer]) + static_cast<long>(it.blk) * kMaxPeers + s.me;
        if (local) st_release_gpu_i32(flag, epoch); else st_release_sys_i32(flag, epoch);
      }
      if (stamp_at == 3) stamp();
    }
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
  using L = Layout<MODE>;
  constexpr int kStages = L::kStages;

  const int cta = static_cast<int>(blockIdx.x);
  const int num_ctas = static_cast<int>(gridDim.x);
  SharedAux* aux = reinterpret_cast<SharedAux*>(smem + L::kAuxOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---------------------------------------------------------------- set-up
  if (threadIdx.x == 0) {
    if (p.trace != nullptr) p.trace[cta * TRACE_SLOTS + 0] = ptx::globaltimer();
    for (int s = 0; s < kStages; ++s) {
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
  // When tiles wait for rows from peers, the roles behind the producer must outlast the
  // longest wait the producer may legitimately sit in.
  const unsigned long long wait_limit =
      ptx::kWaitLimitNs + ((MODE != kWgrad && p.gate.flags != nullptr) ? p.gate.timeout_ns : 0ull);

  if (warp == 0) {
    // ============================================================== TMA producer
    int stage = 0;
    uint32_t phase = 0;
    uint32_t tail_phase = 0;
    bool ok = true;
    // Arrival gating (row modes under expert parallelism): lane j looks after the j-th source
    // of a tile's row block.  The flag of the NEXT tile is read one tile ahead, so that in the
    // steady state the value is already in a register when the tile starts.
    const bool gated = (MODE != kWgrad) && p.gate.flags != nullptr;
    const int gate_epoch = gated ? *p.gate.epoch : 0;
    const int n_tiles_n = (p.n + BN - 1) / BN;
    auto gate_flag = [&](int tile) -> const int* {
      if (!gated || tile >= total_tiles || lane >= p.gate.world) return nullptr;
      const TileCoord c = decode_tile<MODE>(p, aux, tile);
      const int r0 = c.row_begin + c.m_tile * BM;
      const int r1 = min(r0 + BM, c.row_end);
      const int* so = p.gate.seg_off + c.group * (p.gate.world + 1) + lane;
      // a source without rows for this expert sends nothing and raises no flag: never wait
      // for it, also when its (empty) range lies strictly inside the block
      if (!(so[0] < so[1] && so[0] < r1 && so[1] > r0)) return nullptr;
      int src = p.gate.me - lane;
      if (src < 0) src += p.gate.world;
      const int blk = aux->tile_prefix[c.group] / n_tiles_n + c.m_tile;
      return p.gate.flags + static_cast<long>(blk) * kMaxPeers + src;
    };
    const int* flag_next = gate_flag(cta);
    int seen_next = flag_next != nullptr ? ld_acquire_sys_i32(flag_next) : gate_epoch;
    for (int tile = cta; tile < total_tiles && ok; tile += num_ctas) {
      const TileCoord c = decode_tile<MODE>(p, aux, tile);
      const int rows = c.row_end - c.row_begin;
      const int num_kb = (MODE == kWgrad) ? (rows + BK - 1) / BK : p.k / BK;
      if constexpr (MODE != kWgrad) {
        if (gated) {
          const int* flag = flag_next;
          int seen = seen_next;
          flag_next = gate_flag(tile + num_ctas);
          seen_next = flag_next != nullptr ? ld_acquire_sys_i32(flag_next) : gate_epoch;
          bool here = true;
          const unsigned long long wait_from = p.trace != nullptr ? ptx::globaltimer() : 0ull;
          if (flag != nullptr && seen - gate_epoch < 0) {
            const unsigned long long t0 = ptx::globaltimer();
            unsigned spins = 0;
            while (true) {
              if (ld_acquire_sys_i32(flag) - gate_epoch >= 0) break;
              if ((++spins & 0x3f) == 0) {
                // a failure already recorded on this GPU (by any kernel) ends the wait at once:
                // one lost peer must not cost a full time-out in every tile that follows
                const bool failed_before =
                    p.status != nullptr && status_is_failure(*reinterpret_cast<const volatile int*>(p.status));
                if (*abort_flag != 0 || failed_before || ptx::globaltimer() - t0 > p.gate.timeout_ns) {
                  here = false;
                  break;
                }
              }
              __nanosleep(100);
            }
          }
          if (!__all_sync(0xffffffffu, here)) {
            if (lane == 0) fail(aux, p.status, STATUS_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          // the rows were written by other GPUs and are now read through the async proxy
          ptx::fence_proxy_async_all();
          if (p.trace != nullptr && lane == 0) {
            const unsigned long long now = ptx::globaltimer();
            if (tile == cta) p.trace[cta * TRACE_SLOTS + 1] = now;
            // time the producer spent waiting for rows, all tiles, and how many tiles waited
            p.trace[cta * TRACE_SLOTS + 8] += now - wait_from;
            if (now - wait_from > 1000ull) p.trace[cta * TRACE_SLOTS + 9] += 1ull;
          }
        }
      }
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
        if (++stage == kStages) { stage = 0; phase ^= 1; }
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
      for (int tile = cta; tile < total_tiles && ok; tile += num_ctas, ++iter) {
        const TileCoord c = decode_tile<MODE>(p, aux, tile);
        const int rows = c.row_end - c.row_begin;
        const int num_kb = (MODE == kWgrad) ? (rows + BK - 1) / BK : p.k / BK;
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!ptx::mbar_wait(&aux->tmem_empty[acc], acc_phase ^ 1, abort_flag, wait_limit)) {
          fail(aux, p.status, STATUS_TIMEOUT_MMA);
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&aux->full[stage], phase, abort_flag, wait_limit)) {
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
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        ptx::umma_commit(&aux->tmem_full[acc]);
      }
    }
  } else if (warp < FIRST_EPI_WARP) {
    // ============================================================== sender warps (2, 3)
    if constexpr (MODE != kWgrad) {
      if (p.send.enabled) {
        sender_warp<T>(p, cta * NUM_SEND_WARPS + (warp - FIRST_SEND_WARP), num_ctas * NUM_SEND_WARPS, lane,
                       (p.trace != nullptr && warp == FIRST_SEND_WARP) ? p.trace + cta * TRACE_SLOTS + 4 : nullptr);
        if (p.trace != nullptr && lane == 0 && warp == FIRST_SEND_WARP) {
          p.trace[cta * TRACE_SLOTS + 2] = ptx::globaltimer();
        }
      }
    }
  } else {
    // ============================================================== epilogue (warps 4..11)
    const int part = warp & 3;                          // TMEM lane quarter this warp may read
    const int half = (warp - FIRST_EPI_WARP) >> 2;      // which half of the accumulator columns
    uint8_t* patch = smem + L::kEpiOff + (warp - FIRST_EPI_WARP) * L::kPatch;
    int iter = 0;
    for (int tile = cta; tile < total_tiles; tile += num_ctas, ++iter) {
      const TileCoord c = decode_tile<MODE>(p, aux, tile);
      const int rows = c.row_end - c.row_begin;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      const int n0 = c.n_tile * BN;

      if constexpr (MODE == kWgrad) {
        // Rows of the output matrix covered by this warp: [warp_row0, warp_row0 + warp_valid).
        const int m0 = c.m_tile * BM + part * 32;
        const long warp_row0 = static_cast<long>(c.group) * p.m + m0;
        const int warp_valid = min(32, p.m - m0);
        const bool row_ok = lane < warp_valid;
        const long out_row = warp_row0 + lane;
        const bool have_acc = rows > 0;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(part * 32) << 16) + acc * BN;
        const bool read_old = p.accumulate && !p.out_fp32;
        const bool use_side = read_old && warp_valid > 0;
        const uint8_t* side = reinterpret_cast<const uint8_t*>(p.out) + (warp_row0 * p.n + n0) * 2;
        const long side_pitch = static_cast<long>(p.n) * 2;
        const int first_col = n0 + half * 32;
        {
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
            const uint8_t* first = smem + L::kEpiOff;
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
        // The old gradient (when accumulating in 16 bits) does not depend on the accumulator:
        // fetch its first chunk before waiting for the MMAs.
        if (use_side && first_col < p.n) {
          stage_side(patch, side + half * 64, side_pitch, warp_valid, lane);
        }
        if (!ptx::mbar_wait(&aux->tmem_full[acc], acc_phase, abort_flag, wait_limit)) {
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
        et.use_aux = false;
        et.read_old = read_old;
        et.use_side = use_side;
        et.side = side;
        et.side_pitch = side_pitch;
        et.patch = patch;
        et.out_row_base = nullptr;
        et.remote_row = false;
        et.bias_sm = nullptr;
        et.empty_bar = &aux->tmem_empty[acc];
        epilogue_tile<MODE, T, ACT>(p, et);
      } else {
        // This warp: rows [r0, r0 + 32) of the tile, columns [col_first, col_first + 128).
        const int r0 = c.m_tile * BM + part * 32;
        const long warp_row0 = static_cast<long>(c.row_begin) + r0;
        const int warp_valid = max(0, min(32, rows - r0));
        const bool row_ok = lane < warp_valid;
        const long out_row = warp_row0 + lane;
        const int col_first = n0 + half * (BN / 2);
        const int n_chunks = max(0, min(CHUNKS_PER_WARP, (p.n - col_first) / 32));
        const bool use_aux = p.epi == kEpiDAct;
        const int ew = warp - FIRST_EPI_WARP;

        RowTile rt;
        rt.lane = lane;
        rt.col_first = col_first;
        rt.n_chunks = n_chunks;
        rt.row_ok = row_ok;
        rt.use_aux = use_aux;
        rt.patch = patch;
        rt.out_row = nullptr;
        rt.pre_tile = nullptr;
        // The saved pre-activation is tile-blocked: this warp's four chunks of this tile.
        if (use_aux) {
          rt.pre_tile = const_cast<uint8_t*>(static_cast<const uint8_t*>(p.aux)) +
                        pre_tile_index(p, aux, c) * PRE_TILE_BYTES + ew * (CHUNKS_PER_WARP * PRE_CHUNK_BYTES);
        } else if (p.pre_out != nullptr) {
          rt.pre_tile = static_cast<uint8_t*>(p.pre_out) + pre_tile_index(p, aux, c) * PRE_TILE_BYTES +
                        ew * (CHUNKS_PER_WARP * PRE_CHUNK_BYTES);
        }
        // It does not depend on the accumulator: fetch the first chunk before waiting for the
        // MMAs, and pull the next tile's chunks of this warp (8 KB, two lines per lane) to L2.
        Packed32 side_first;
        if (use_aux && n_chunks > 0) {
          load_pre_chunk(rt.pre_tile, 0, lane, side_first);
          if (tile + num_ctas < total_tiles) {
            const TileCoord cn = decode_tile<MODE>(p, aux, tile + num_ctas);
            const uint8_t* nx = static_cast<const uint8_t*>(p.aux) + pre_tile_index(p, aux, cn) * PRE_TILE_BYTES +
                                ew * (CHUNKS_PER_WARP * PRE_CHUNK_BYTES) + lane * 256;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(nx));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + 128));
          }
        }
        if (p.push_meta != nullptr) {
          // Fused combine: this lane's output row lives in the source rank's return buffer.
          if (row_ok) {
            const int64_t m = p.push_meta[out_row];
            const int src = static_cast<int>(m >> 32);
            const long slot = static_cast<long>(m & 0xffffffffll);
            if (src >= 0 && src < p.push_world && slot < p.push_slots) {
              rt.out_row = static_cast<uint8_t*>(p.push_dst.p[src]) + slot * p.n * 2;
            } else if (p.status != nullptr) {
              record_failure(p.status, STATUS_BAD_PUSH_META);
            }
          }
        } else {
          rt.out_row = static_cast<uint8_t*>(p.out) + out_row * p.n * 2;
        }
        rt.bias = (!use_aux && p.bias != nullptr)
                      ? static_cast<const uint8_t*>(p.bias) + (static_cast<long>(c.group) * p.n + col_first) * 2
                      : nullptr;
        rt.empty_bar = &aux->tmem_empty[acc];
        rt.t_row = tmem_base + (static_cast<uint32_t>(part * 32) << 16) + acc * BN + half * (BN / 2);

        if (!ptx::mbar_wait(&aux->tmem_full[acc], acc_phase, abort_flag, wait_limit)) {
          if (lane == 0) fail(aux, p.status, STATUS_TIMEOUT_EPILOGUE);
          break;
        }
        ptx::tc_fence_after_sync();
        epilogue_tile_rows<T, ACT>(rt, side_first);
      }
    }
    if constexpr (MODE != kWgrad) {
      if (p.push_meta != nullptr) {
        // All rows of this CTA are on their way: order them before the completion count; the
        // last CTA of the grid publishes the epoch on every peer's return channel.  A CTA that
        // gave up still counts, so that the counter is zero again for the next launch.
        __threadfence_system();
        asm volatile("bar.sync 1, %0;" ::"n"(NUM_EPI_WARPS * 32) : "memory");
        if (threadIdx.x == FIRST_EPI_WARP * 32) {
          const int prev = atomicAdd(p.push_counter, 1);
          if (prev == num_ctas - 1) {
            *p.push_counter = 0;
            __threadfence_system();
            const int epoch = *p.push_epoch;
            for (int peer = 0; peer < p.push_world; ++peer) {
              int* flag = static_cast<int*>(p.push_flags.p[peer]) + kChanReturn * kMaxPeers + p.push_me;
              st_release_sys_i32(flag, epoch);
            }
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
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[cta * TRACE_SLOTS + 3] = ptx::globaltimer();
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
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           Layout<MODE>::kBytes);
      if (e != cudaSuccess) return e;
      configured |= 1ull << (dev & 63);
    }
  }
  kernel<<<grid, NUM_THREADS, Layout<MODE>::kBytes, stream>>>(ta, tb, kp);
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
