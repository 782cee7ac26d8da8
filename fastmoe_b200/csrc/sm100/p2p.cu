// Peer-to-peer exchange kernels: see p2p.cuh for the contract of each launcher.
//
// Memory model.  Data rows are written into a peer's memory with ordinary 16-byte stores;
// a producer then executes a system-scope fence and a release store of the exchange epoch
// into the consumer's flag word; the consumer polls that word with acquire loads.  Epochs
// only grow, live in device memory and are advanced by the kernels themselves, so the same
// launch sequence can be replayed from a CUDA graph.  A wait gives up after
// `timeout_ns`, records kStatusPeerTimeout and lets the kernel finish.
#include "p2p.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace fmoe {
namespace {

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int* flag_of(void* signal_base, int channel, int src) {
  return static_cast<int*>(signal_base) + channel * kMaxPeers + src;
}

// Polls my flag of `src` on `channel` until it reaches `target`.  False on time-out or when
// the status word already reports a failure (so that one failure does not cost a full
// time-out in every later wait of the step).
__device__ __forceinline__ bool wait_flag(const ExchangeCtx& c, int channel, int src, int target) {
  const int* f = flag_of(c.flags.p[c.me], channel, src);
  if (ld_acquire_sys(f) - target >= 0) return true;
  const unsigned long long t0 = now_ns();
  unsigned spins = 0;
  while (true) {
    if (ld_acquire_sys(f) - target >= 0) return true;
    if ((++spins & 0xff) == 0) {
      if (status_is_failure(*reinterpret_cast<volatile int*>(c.status))) return false;
      if (now_ns() - t0 > c.timeout_ns) {
        record_failure(c.status, kStatusPeerTimeout);
        return false;
      }
    }
    __nanosleep(64);
  }
}

// All threads of the block call this; threads 0..world-1 each wait for one peer.
__device__ __forceinline__ void block_wait_all(const ExchangeCtx& c, int channel, int target) {
  if (static_cast<int>(threadIdx.x) < c.world) wait_flag(c, channel, threadIdx.x, target);
  __syncthreads();
}

// Called by one thread after the whole grid's stores are ordered before it.
__device__ __forceinline__ void signal_all(const ExchangeCtx& c, int channel, int value) {
  __threadfence_system();
  for (int p = 0; p < c.world; ++p) st_release_sys(flag_of(c.flags.p[p], channel, c.me), value);
}

// Kernel parameters that are indexed with a runtime value (peer pointer tables, the exchange
// context) are declared __grid_constant__: without it the compiler copies the whole table to
// each thread's local memory before indexing it, which cost the row-push kernel 39 MB of
// local stores (20 us of a 21 us kernel) for 16 MB of payload.

// Grid-wide "I am the last CTA" test on a counter in local memory (reset for the next use).
__device__ __forceinline__ bool last_block(int* counter) {
  __shared__ int is_last;
  // Every thread orders its own stores at system scope before the barrier; thread 0 then
  // counts the block.  (One fence by thread 0 behind the barrier would be enough by the
  // memory model's cumulativity, and was not measurably faster.)
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(counter, 1);
    is_last = (prev == static_cast<int>(gridDim.x) - 1);
    if (is_last) *counter = 0;
  }
  __syncthreads();
  return is_last != 0;
}

// ------------------------------------------------------------------------------ counts
// Receive layout on every rank p: local expert outer; inside an expert segment the rows of
// source rank w sit at position (p - w) mod world — the rank's own rows first, then those of
// rank p - 1, p - 2, ...  A sender serves its peers in the order me, me + 1, me + 2, ... (peer
// distance outer, expert inner), and `blk_order` lists the receiver's 128-row blocks in the
// matching order — by the source position of a block's last row, then expert, then row — so
// that a GEMM which walks its tiles through that table reads rows in the order they arrive:
// first everything that never left the GPU, then what the nearest source sent, and so on.
__device__ __forceinline__ int source_position(int owner, int src, int world) {
  int j = owner - src;
  return j < 0 ? j + world : j;
}

__global__ void __launch_bounds__(1024, 1)
count_exchange_kernel(const __grid_constant__ ExchangeCtx c, const int* __restrict__ lec, const __grid_constant__ PeerPtrs cnt, int n_expert,
                      int capacity_rows, int* __restrict__ dst_base, int* __restrict__ seg_base,
                      int* __restrict__ blk_base, int* __restrict__ expert_offs,
                      int* __restrict__ seg_off, int* __restrict__ total_rows,
                      int* __restrict__ item_prefix, int* __restrict__ blk_order) {
  extern __shared__ int sh[];  // [world * width] matrix, [tot] column sums, [tot] items per pair,
                               // [tot] first block and [tot + 1] block prefix per (position, expert)
  const int tot = n_expert * c.world;
  const int width = tot + 1;   // a rank's row: its counts, then its receive capacity
  const int epoch = c.epoch[0] + 1;
  // 1. my row into every peer's matrix
  for (int g = threadIdx.x; g < width; g += blockDim.x) {
    const int v = g < tot ? lec[g] : capacity_rows;
    for (int p = 0; p < c.world; ++p) static_cast<int*>(cnt.p[p])[c.me * width + g] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < c.world) {
    st_release_sys(flag_of(c.flags.p[threadIdx.x], kChanCounts, c.me), epoch);
  }
  // 2. everybody's rows
  block_wait_all(c, kChanCounts, epoch);
  const volatile int* mine = static_cast<const volatile int*>(cnt.p[c.me]);
  int* mat = sh;
  int* col = sh + c.world * width;
  for (int i = threadIdx.x; i < c.world * width; i += blockDim.x) mat[i] = mine[i];
  __syncthreads();
  for (int g = threadIdx.x; g < tot; g += blockDim.x) {
    int s = 0;
    for (int w = 0; w < c.world; ++w) s += mat[w * width + g];
    col[g] = s;
  }
  __syncthreads();
  // 3. offsets of every global expert on its owner, and of my rows inside them
  for (int g = threadIdx.x; g < tot; g += blockDim.x) {
    const int p = g / n_expert;
    const int e = g - p * n_expert;
    int seg = 0, blk = 0;
    for (int e2 = 0; e2 < e; ++e2) {
      const int n = col[p * n_expert + e2];
      seg += n;
      blk += (n + kRowBlock - 1) / kRowBlock;
    }
    const int my_pos = source_position(p, c.me, c.world);
    int before = 0;
    for (int j = 0; j < my_pos; ++j) {
      int w = p - j;
      if (w < 0) w += c.world;
      before += mat[w * width + g];
    }
    seg_base[g] = seg;
    blk_base[g] = blk;
    dst_base[g] = seg + before;
    // row blocks my rows touch on the owner (clamped to its capacity), stored at the pair's
    // place in send order; turned into a prefix below
    int items = 0;
    const int cnt_mine = mat[c.me * width + g];
    int r_end = before + cnt_mine;
    if (r_end > capacity_rows - seg) r_end = capacity_rows - seg;
    if (cnt_mine > 0 && r_end > before) items = (r_end - 1) / kRowBlock - before / kRowBlock + 1;
    int j = p - c.me;
    if (j < 0) j += c.world;
    col[tot + j * n_expert + e] = items;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    item_prefix[0] = 0;
    for (int q = 0; q < tot; ++q) {
      run += col[tot + q];
      item_prefix[q + 1] = run;
    }
  }
  // 4. my own segments: expert offsets and, per expert, where each source's rows begin
  for (int e = threadIdx.x; e < n_expert; e += blockDim.x) {
    int seg = 0;
    for (int e2 = 0; e2 < e; ++e2) seg += col[c.me * n_expert + e2];
    expert_offs[e] = seg < capacity_rows ? seg : capacity_rows;
    int run = seg;
    for (int j = 0; j <= c.world; ++j) {
      seg_off[e * (c.world + 1) + j] = run < capacity_rows ? run : capacity_rows;
      if (j < c.world) {
        int w = c.me - j;
        if (w < 0) w += c.world;
        run += mat[w * width + c.me * n_expert + e];
      }
    }
    if (e == n_expert - 1) {
      const int end = run < capacity_rows ? run : capacity_rows;
      expert_offs[n_expert] = end;
      total_rows[0] = end;
    }
  }
  // 5. my row blocks in the order their rows arrive.  Blocks of expert e whose last row comes
  // from position j are consecutive: with f(t) = number of blocks whose last row is below t,
  // they are [f(s_j), f(s_j+1)), s_j being where position j starts inside the segment.
  __syncthreads();
  int* ord_lo = col + 2 * tot;
  int* ord_prefix = col + 3 * tot;
  for (int q = threadIdx.x; q < tot; q += blockDim.x) {
    const int j = q / n_expert;
    const int e = q - j * n_expert;
    const int* so = seg_off + e * (c.world + 1);
    const int n_e = so[c.world] - so[0];
    const int n_blk = (n_e + kRowBlock - 1) / kRowBlock;
    const int s_lo = so[j] - so[0];
    const int s_hi = so[j + 1] - so[0];
    const int f_lo = s_lo >= n_e ? n_blk : s_lo / kRowBlock;
    const int f_hi = s_hi >= n_e ? n_blk : s_hi / kRowBlock;
    ord_lo[q] = f_lo;
    ord_prefix[q + 1] = f_hi - f_lo;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    ord_prefix[0] = 0;
    for (int q = 0; q < tot; ++q) {
      run += ord_prefix[q + 1];
      ord_prefix[q + 1] = run;
    }
  }
  __syncthreads();
  for (int q = threadIdx.x; q < tot; q += blockDim.x) {
    const int e = q % n_expert;
    const int n = ord_prefix[q + 1] - ord_prefix[q];
    for (int t = 0; t < n; ++t) blk_order[ord_prefix[q] + t] = (e << kBlkOrderShift) | (ord_lo[q] + t);
  }
  // Overflow anywhere is visible to everybody (same matrix): report it on every rank.  So is a
  // peer that sized its receive buffer differently: senders clamp against THEIR capacity, so
  // a smaller buffer elsewhere would be overrun.
  if (static_cast<int>(threadIdx.x) < c.world) {
    const int p = threadIdx.x;
    int t = 0;
    for (int e = 0; e < n_expert; ++e) t += col[p * n_expert + e];
    if (t > capacity_rows) atomicCAS(c.status, 0, kStatusRecvOverflow);
    if (mat[p * width + tot] != capacity_rows) record_failure(c.status, kStatusCapacityMismatch);
  }
  if (threadIdx.x == 0) c.epoch[0] = epoch;
}

__global__ void begin_epoch_kernel(const __grid_constant__ ExchangeCtx c, int word) {
  if (threadIdx.x == 0 && blockIdx.x == 0) c.epoch[word] = c.epoch[word] + 1;
}

// ------------------------------------------------------------------------------ row helpers
template <typename T> struct V2;
template <> struct V2<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ float2 to_f2(type v) { return __bfloat1622float2(v); }
  static __device__ __forceinline__ type from_f2(float a, float b) { return __floats2bfloat162_rn(a, b); }
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16(v); }
};
template <> struct V2<__half> {
  using type = __half2;
  static __device__ __forceinline__ float2 to_f2(type v) { return __half22float2(v); }
  static __device__ __forceinline__ type from_f2(float a, float b) { return __floats2half2_rn(a, b); }
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half(v); }
};

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
  using P = typename V2<T>::type;
  const P* p = reinterpret_cast<const P*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 v = V2<T>::to_f2(p[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  using P = typename V2<T>::type;
  uint4 w;
  P* p = reinterpret_cast<P*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = V2<T>::from_f2(f[2 * i], f[2 * i + 1]);
  return w;
}

// Capacity grants in one exchange.  Every rank writes its per-expert request counts and its
// own per-expert capacities into every peer's matrix; with the full matrix on every rank the
// rank-ordered grants (`grant[w][g] = min(request[w][g], what ranks < w left of cap[g])`) are
// computed locally by everybody, so the second all-to-all of the reference
// (fmoe/gates/utils.py:19-24: grants travel back to the requesters) is not needed.
// Matrix row of rank w: [tot request counts | n_expert capacities]; two matrices alternate
// with the epoch so that a fast rank cannot overwrite a matrix a slow rank still reads.
__global__ void __launch_bounds__(1024, 1)
capacity_grant_kernel(const __grid_constant__ ExchangeCtx c, const int* __restrict__ lec, const int* __restrict__ cap,
                      const __grid_constant__ PeerPtrs cnt, int n_expert, int64_t* __restrict__ new_lec,
                      int64_t* __restrict__ new_gec) {
  extern __shared__ int sh[];
  const int tot = n_expert * c.world;
  const int width = tot + n_expert;
  const int epoch = c.epoch[0];
  const long half = static_cast<long>(epoch & 1) * c.world * width;
  for (int g = threadIdx.x; g < width; g += blockDim.x) {
    const int v = g < tot ? lec[g] : cap[g - tot];
    for (int p = 0; p < c.world; ++p) static_cast<int*>(cnt.p[p])[half + c.me * width + g] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < c.world) {
    st_release_sys(flag_of(c.flags.p[threadIdx.x], kChanCounts, c.me), epoch);
  }
  block_wait_all(c, kChanCounts, epoch);
  const volatile int* mine = static_cast<const volatile int*>(cnt.p[c.me]) + half;
  for (int i = threadIdx.x; i < c.world * width; i += blockDim.x) sh[i] = mine[i];
  __syncthreads();
  for (int g = threadIdx.x; g < tot; g += blockDim.x) {
    const int owner = g / n_expert;
    const int e = g - owner * n_expert;
    int remaining = sh[owner * width + tot + e];
    for (int w = 0; w < c.world; ++w) {
      const int want = sh[w * width + g];
      const int grant = want < remaining ? want : remaining;
      remaining -= grant;
      if (w == c.me) new_lec[g] = grant;
      if (owner == c.me) new_gec[w * n_expert + e] = grant;
    }
  }
}


// One SWIPE round's exchange and plan (cuda/balancing.cu:83-186 in the reference: two count
// exchanges, an all-reduce and an all-gather with a host sync after each).  Every rank writes
// [tokens it wants to send to each worker | capacity it has left] into every peer's table;
// with the full table each rank computes the same plan: workers accept requests in rank order
// until full, the overflow is handed to workers with room in rank order.  Outputs for this
// rank: quota[j] = tokens it may send to worker j, cap_left = its own remaining capacity.
// Two tables alternate with the epoch, as for the capacity grants.
__global__ void __launch_bounds__(256, 1)
swipe_exchange_kernel(const __grid_constant__ ExchangeCtx c, const int* __restrict__ want,
                      const int64_t* __restrict__ cap, const __grid_constant__ PeerPtrs tab,
                      int* __restrict__ quota, int64_t* __restrict__ cap_left) {
  __shared__ long sh[kMaxPeers * (kMaxPeers + 1)];
  __shared__ long left[kMaxPeers];
  __shared__ long dropped[kMaxPeers];
  const int W = c.world;
  const int width = W + 1;
  const int epoch = c.epoch[0];
  const long half = static_cast<long>(epoch & 1) * W * width;
  if (static_cast<int>(threadIdx.x) < width) {
    const long v = static_cast<int>(threadIdx.x) < W ? want[threadIdx.x] : cap[0];
    for (int p = 0; p < W; ++p) {
      static_cast<long*>(tab.p[p])[half + c.me * width + threadIdx.x] = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < W) {
    st_release_sys(flag_of(c.flags.p[threadIdx.x], kChanCounts, c.me), epoch);
  }
  block_wait_all(c, kChanCounts, epoch);
  const volatile long* mine = static_cast<const volatile long*>(tab.p[c.me]) + half;
  for (int i = threadIdx.x; i < W * width; i += blockDim.x) sh[i] = mine[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int j = 0; j < W; ++j) left[j] = sh[j * width + W];
    for (int i = 0; i < W; ++i) dropped[i] = 0;
    for (int j = 0; j < W; ++j) {
      for (int i = 0; i < W; ++i) {
        const long w = sh[i * width + j];
        const long take = w < left[j] ? w : left[j];
        sh[i * width + j] = take;          // the table now holds the accepted counts
        left[j] -= take;
        dropped[i] += w - take;
      }
    }
    int j = 0;
    for (int i = 0; i < W; ++i) {
      while (dropped[i] > 0 && j < W) {
        const long take = dropped[i] < left[j] ? dropped[i] : left[j];
        sh[i * width + j] += take;
        left[j] -= take;
        dropped[i] -= take;
        if (left[j] == 0) ++j;
      }
    }
    for (int q = 0; q < W; ++q) quota[q] = static_cast<int>(sh[c.me * width + q]);
    cap_left[0] = left[c.me];
  }
}

// ------------------------------------------------------------------------------ dispatch
// One warp per slot, persistent grid.  Stores go to the owner's staging buffer over NVLink.
template <typename T>
__global__ void __launch_bounds__(1024, 1) dispatch_push_kernel(const __grid_constant__ ExchangeCtx c, const T* __restrict__ x,
                                     const int64_t* __restrict__ idx, const int* __restrict__ rank,
                                     const int* __restrict__ dst_base, const T* __restrict__ scale,
                                     const __grid_constant__ PeerPtrs rows, const __grid_constant__ PeerPtrs meta, int n_expert, int n_slots, int k,
                                     int d, int capacity_rows) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int nv = d >> 3;
  for (int s = blockIdx.x * warps_per_block + (threadIdx.x >> 5); s < n_slots;
       s += gridDim.x * warps_per_block) {
    const long g = idx[s];
    if (g < 0) continue;
    const int p = static_cast<int>(g / n_expert);
    const long row = static_cast<long>(dst_base[g]) + rank[s];
    if (row >= capacity_rows) continue;  // overflow is reported by the count exchange
    const uint4* in = reinterpret_cast<const uint4*>(x + static_cast<long>(s / k) * d);
    uint4* out = reinterpret_cast<uint4*>(static_cast<T*>(rows.p[p]) + row * d);
    const float sc = scale == nullptr ? 1.f : V2<T>::to_f(scale[s]);
    for (int i0 = lane; i0 < nv; i0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + u * 32 < nv) v[u] = __ldg(in + i0 + u * 32);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + u * 32 < nv) {
          if (scale != nullptr) {
            float f[8];
            unpack8<T>(v[u], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] *= sc;
            v[u] = pack8<T>(f);
          }
          out[i0 + u * 32] = v[u];
        }
      }
    }
    if (lane == 0 && meta.p[p] != nullptr) {
      static_cast<int64_t*>(meta.p[p])[row] = (static_cast<int64_t>(c.me) << 32) | static_cast<int64_t>(s);
    }
  }
  if (last_block(c.epoch + 1)) {
    if (threadIdx.x == 0) signal_all(c, kChanDispatch, c.epoch[0]);
  }
}

template <typename T>
__global__ void wait_copy_kernel(const __grid_constant__ ExchangeCtx c, int channel, const T* __restrict__ stage_rows,
                                 const int64_t* __restrict__ stage_meta,
                                 const int* __restrict__ total_rows, int d, int capacity_rows,
                                 T* __restrict__ out_rows, int64_t* __restrict__ out_meta) {
  block_wait_all(c, channel, c.epoch[0]);
  int n_rows = total_rows[0];
  if (n_rows > capacity_rows) n_rows = capacity_rows;
  const long nv = static_cast<long>(n_rows) * (d >> 3);
  const uint4* in = reinterpret_cast<const uint4*>(stage_rows);
  uint4* out = reinterpret_cast<uint4*>(out_rows);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    out[i] = __ldcg(in + i);
  }
  if (out_meta != nullptr) {
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n_rows;
         i += static_cast<long>(gridDim.x) * blockDim.x) {
      out_meta[i] = __ldcg(stage_meta + i);
    }
  }
}

// One warp per received row.
template <typename T>
__global__ void __launch_bounds__(1024, 1) return_push_kernel(const __grid_constant__ ExchangeCtx c, const T* __restrict__ rows_in,
                                   const int64_t* __restrict__ meta,
                                   const int* __restrict__ total_rows, const __grid_constant__ PeerPtrs ret, int d,
                                   int capacity_rows, long ret_slots) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  int n_rows = total_rows[0];
  if (n_rows > capacity_rows) n_rows = capacity_rows;
  const int nv = d >> 3;
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < n_rows;
       r += gridDim.x * warps_per_block) {
    const int64_t m = meta[r];
    const int src = static_cast<int>(m >> 32);
    const long slot = static_cast<long>(m & 0xffffffffll);
    if (src < 0 || src >= c.world || slot >= ret_slots) continue;
    const uint4* in = reinterpret_cast<const uint4*>(rows_in + static_cast<long>(r) * d);
    uint4* out = reinterpret_cast<uint4*>(static_cast<T*>(ret.p[src]) + slot * d);
    for (int i0 = lane; i0 < nv; i0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + u * 32 < nv) v[u] = __ldg(in + i0 + u * 32);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + u * 32 < nv) out[i0 + u * 32] = v[u];
      }
    }
  }
  if (last_block(c.epoch + 2)) {
    if (threadIdx.x == 0) signal_all(c, kChanReturn, c.epoch[0]);
  }
}

// One warp per token.
template <typename T>
__global__ void wait_combine_kernel(const __grid_constant__ ExchangeCtx c, const T* __restrict__ ret,
                                    const int64_t* __restrict__ idx, const T* __restrict__ weight,
                                    const int* __restrict__ rank, const int* __restrict__ dst_base,
                                    int capacity_rows, int n_tokens, int k, int d,
                                    T* __restrict__ out, T* __restrict__ keep) {
  block_wait_all(c, kChanReturn, c.epoch[0]);
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int nv = d >> 3;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < n_tokens;
       t += gridDim.x * warps_per_block) {
    uint4* o = reinterpret_cast<uint4*>(out + static_cast<long>(t) * d);
    for (int i0 = lane; i0 < nv; i0 += 64) {
      float acc[2][8];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[u][q] = 0.f;
      }
      for (int j = 0; j < k; ++j) {
        const long s = static_cast<long>(t) * k + j;
        const long e = idx[s];
        if (e < 0) continue;
        // A slot whose row did not fit into the owner's receive buffer was never sent and
        // nothing came back for it: it counts as zero (in `keep` too).
        const bool sent = rank == nullptr || __ldg(dst_base + e) + __ldg(rank + s) < capacity_rows;
        const float w = weight != nullptr ? V2<T>::to_f(weight[s]) : 1.f;
        uint4 v[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          v[u] = make_uint4(0u, 0u, 0u, 0u);
          if (sent && i0 + u * 32 < nv) v[u] = __ldcg(reinterpret_cast<const uint4*>(ret + s * d) + i0 + u * 32);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (i0 + u * 32 < nv) {
            if (keep != nullptr) reinterpret_cast<uint4*>(keep + s * d)[i0 + u * 32] = v[u];
            float f[8];
            unpack8<T>(v[u], f);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[u][q] += w * f[q];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (i0 + u * 32 < nv) o[i0 + u * 32] = pack8<T>(acc[u]);
      }
    }
  }
}

template <typename T>
__global__ void slot_dot_kernel(const T* __restrict__ dout, const T* __restrict__ y,
                                const int64_t* __restrict__ idx, int n_slots, int k, int d,
                                T* __restrict__ dscore) {
  const int s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (s >= n_slots) return;
  float dot = 0.f;
  if (idx[s] >= 0) {
    const uint4* g = reinterpret_cast<const uint4*>(dout + static_cast<long>(s / k) * d);
    const uint4* v = reinterpret_cast<const uint4*>(y + static_cast<long>(s) * d);
    for (int i = lane; i < (d >> 3); i += 32) {
      float gf[8], yf[8];
      unpack8<T>(__ldg(g + i), gf);
      unpack8<T>(__ldg(v + i), yf);
#pragma unroll
      for (int q = 0; q < 8; ++q) dot += gf[q] * yf[q];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0) dscore[s] = V2<T>::from_f(dot);
}

// ------------------------------------------------------------------------------ all-reduce
__device__ __forceinline__ float as_float(float v) { return v; }
__device__ __forceinline__ float as_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float as_float(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half(v); }

// One-shot: after everybody published "my buffer is filled", every rank reads all peers'
// buffers in rank order (so all ranks compute bit-identical sums), scales and writes its own
// output; the kernel leaves only when every peer has finished reading this rank's buffer.
template <typename T, typename Vec, int PER>
__global__ void allreduce_kernel(const __grid_constant__ ExchangeCtx c, const __grid_constant__ PeerPtrs bufs, T* __restrict__ out, long n,
                                 float scale) {
  const int target_ready = 2 * c.epoch[kReduceEpochWord];
  if (blockIdx.x == 0 && threadIdx.x == 0) signal_all(c, kChanReduce, target_ready);
  block_wait_all(c, kChanReduce, target_ready);
  const long nvec = n / PER;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float acc[PER];
#pragma unroll
    for (int q = 0; q < PER; ++q) acc[q] = 0.f;
    for (int p = 0; p < c.world; ++p) {
      Vec v = __ldcg(reinterpret_cast<const Vec*>(bufs.p[p]) + i);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int q = 0; q < PER; ++q) acc[q] += as_float(e[q]);
    }
    Vec r;
    T* e = reinterpret_cast<T*>(&r);
#pragma unroll
    for (int q = 0; q < PER; ++q) e[q] = from_float<T>(acc[q] * scale);
    reinterpret_cast<Vec*>(out)[i] = r;
  }
  // tail elements
  for (long i = nvec * PER + blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float acc = 0.f;
    for (int p = 0; p < c.world; ++p) acc += as_float(static_cast<const T*>(bufs.p[p])[i]);
    out[i] = from_float<T>(acc * scale);
  }
  if (last_block(c.epoch + 3)) {
    if (threadIdx.x == 0) signal_all(c, kChanReduce, target_ready + 1);
    block_wait_all(c, kChanReduce, target_ready + 1);
  }
}

// Two-shot: rank r owns the r-th slice of the vectors.  It sums that slice over all peers'
// buffers (rank order, fp32), scales, and stores the result into the same slice of EVERY
// peer's buffer (nobody else reads or writes slice r); after all ranks have published "my
// slices are written", each rank copies its own, now fully reduced, buffer to `out`.  Per GPU
// (W - 1) / W of the bytes are read and as many written over NVLink, against (W - 1) times the
// bytes for the one-shot kernel, so this is the kernel for large buckets.  The buffer must
// hold the element count rounded up to a whole vector.
template <typename T, typename Vec, int PER>
__global__ void allreduce_two_shot_kernel(const __grid_constant__ ExchangeCtx c, const __grid_constant__ PeerPtrs bufs, T* __restrict__ out, long n,
                                          float scale) {
  const int target_ready = 2 * c.epoch[kReduceEpochWord];
  if (blockIdx.x == 0 && threadIdx.x == 0) signal_all(c, kChanReduce, target_ready);
  block_wait_all(c, kChanReduce, target_ready);
  const long tid = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  const long nvec = (n + PER - 1) / PER;
  const long per_rank = (nvec + c.world - 1) / c.world;
  const long lo = per_rank * c.me;
  const long hi = (lo + per_rank < nvec) ? lo + per_rank : nvec;
  for (long i = lo + tid; i < hi; i += stride) {
    float acc[PER];
#pragma unroll
    for (int q = 0; q < PER; ++q) acc[q] = 0.f;
    for (int p = 0; p < c.world; ++p) {
      Vec v = __ldcg(reinterpret_cast<const Vec*>(bufs.p[p]) + i);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int q = 0; q < PER; ++q) acc[q] += as_float(e[q]);
    }
    Vec r;
    T* e = reinterpret_cast<T*>(&r);
#pragma unroll
    for (int q = 0; q < PER; ++q) e[q] = from_float<T>(acc[q] * scale);
    for (int p = 0; p < c.world; ++p) reinterpret_cast<Vec*>(bufs.p[p])[i] = r;
  }
  if (last_block(c.epoch + 3)) {
    if (threadIdx.x == 0) signal_all(c, kChanReduce, target_ready + 1);
  }
  block_wait_all(c, kChanReduce, target_ready + 1);
  const Vec* mine = reinterpret_cast<const Vec*>(bufs.p[c.me]);
  const long nfull = n / PER;
  for (long i = tid; i < nfull; i += stride) reinterpret_cast<Vec*>(out)[i] = __ldcg(mine + i);
  for (long i = nfull * PER + tid; i < n; i += stride) {
    out[i] = *(reinterpret_cast<const volatile T*>(bufs.p[c.me]) + i);
  }
}

// NVSwitch (NVLS) variant of the two-shot all-reduce.  `mc` is the multicast address of the
// symmetric buffers: one `multimem.ld_reduce` on it returns the sum of the same 16 bytes of all
// ranks' buffers, formed inside the switch (fp32 accumulation for the 16-bit types), and one
// `multimem.st` writes a value into all of them.  Rank r reduces the r-th slice, scales it and
// broadcasts it; afterwards every rank copies its own, fully reduced buffer out.  Per GPU only
// 1 / W of the data is pulled through the switch and 1 / W pushed, against (W - 1) / W read and
// written by the peer-to-peer two-shot kernel.  Every rank gets the same bits.
template <int DT> struct MultimemOps;
template <> struct MultimemOps<0> {  // bf16
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ uint4 scale(uint4 v, float s) {
    float f[8];
    unpack8<__nv_bfloat16>(v, f);
#pragma unroll
    for (int q = 0; q < 8; ++q) f[q] *= s;
    return pack8<__nv_bfloat16>(f);
  }
};
template <> struct MultimemOps<1> {  // fp16
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ uint4 scale(uint4 v, float s) {
    float f[8];
    unpack8<__half>(v, f);
#pragma unroll
    for (int q = 0; q < 8; ++q) f[q] *= s;
    return pack8<__half>(f);
  }
};
template <> struct MultimemOps<2> {  // fp32
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ uint4 scale(uint4 v, float s) {
    v.x = __float_as_uint(__uint_as_float(v.x) * s);
    v.y = __float_as_uint(__uint_as_float(v.y) * s);
    v.z = __float_as_uint(__uint_as_float(v.z) * s);
    v.w = __float_as_uint(__uint_as_float(v.w) * s);
    return v;
  }
};

template <int DT>
__global__ void allreduce_multimem_kernel(const __grid_constant__ ExchangeCtx c, uint8_t* __restrict__ mc,
                                          const uint8_t* __restrict__ mine, uint8_t* __restrict__ out,
                                          long nbytes, float scale) {
  const int target_ready = 2 * c.epoch[kReduceEpochWord];
  if (blockIdx.x == 0 && threadIdx.x == 0) signal_all(c, kChanReduce, target_ready);
  block_wait_all(c, kChanReduce, target_ready);
  const long tid = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  const long nvec = (nbytes + 15) / 16;      // the buffers are padded to whole 16-byte pieces
  const long per_rank = (nvec + c.world - 1) / c.world;
  const long lo = per_rank * c.me;
  const long hi = (lo + per_rank < nvec) ? lo + per_rank : nvec;
  for (long i = lo + tid; i < hi; i += stride) {
    const uint4 v = MultimemOps<DT>::scale(MultimemOps<DT>::ld_reduce(mc + i * 16), scale);
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc + i * 16),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
  }
  if (last_block(c.epoch + 3)) {
    if (threadIdx.x == 0) signal_all(c, kChanReduce, target_ready + 1);
  }
  block_wait_all(c, kChanReduce, target_ready + 1);
  const long nfull = nbytes / 16;
  for (long i = tid; i < nfull; i += stride) {
    reinterpret_cast<uint4*>(out)[i] = __ldcg(reinterpret_cast<const uint4*>(mine) + i);
  }
  for (long b = nfull * 16 + tid; b < nbytes; b += stride) {
    out[b] = *(reinterpret_cast<const volatile uint8_t*>(mine) + b);
  }
}

// All-gather of equal slices: every rank stores its slice at offset `me` of every peer's
// symmetric buffer, publishes, waits for all peers and copies the assembled buffer out.
// The first handshake makes sure no peer is still reading its buffer from an earlier call.
__global__ void allgather_kernel(const __grid_constant__ ExchangeCtx c, const uint4* __restrict__ src, const __grid_constant__ PeerPtrs bufs,
                                 uint4* __restrict__ out, long nvec) {
  const int target_ready = 2 * c.epoch[kReduceEpochWord];
  if (blockIdx.x == 0 && threadIdx.x == 0) signal_all(c, kChanReduce, target_ready);
  block_wait_all(c, kChanReduce, target_ready);
  const long tid = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i = tid; i < nvec; i += stride) {
    const uint4 v = __ldg(src + i);
    for (int p = 0; p < c.world; ++p) {
      reinterpret_cast<uint4*>(bufs.p[p])[static_cast<long>(c.me) * nvec + i] = v;
    }
  }
  if (last_block(c.epoch + 3)) {
    if (threadIdx.x == 0) signal_all(c, kChanReduce, target_ready + 1);
  }
  block_wait_all(c, kChanReduce, target_ready + 1);
  const uint4* mine = reinterpret_cast<const uint4*>(bufs.p[c.me]);
  const long total = nvec * c.world;
  for (long i = tid; i < total; i += stride) out[i] = __ldcg(mine + i);
}

// Broadcast from `root`: the owner pushes its data into every peer's symmetric buffer — one
// write per peer, (W - 1) x n bytes over NVLink in total — after every peer has reported that
// its buffer may be overwritten; everybody then copies its own buffer out.  This is the
// shadow-expert parameter broadcast (cuda/fastermoe/smart_schedule.h:182, ncclBcast there).
__global__ void broadcast_kernel(const __grid_constant__ ExchangeCtx c, const uint4* __restrict__ src,
                                 const __grid_constant__ PeerPtrs bufs, uint4* __restrict__ out, long nvec,
                                 int root) {
  const int target = 2 * c.epoch[kReduceEpochWord];
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    st_release_sys(flag_of(c.flags.p[root], kChanReduce, c.me), target);
  }
  const long tid = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  if (c.me == root) {
    block_wait_all(c, kChanReduce, target);
    for (long i = tid; i < nvec; i += stride) {
      const uint4 v = __ldg(src + i);
      for (int p = 0; p < c.world; ++p) reinterpret_cast<uint4*>(bufs.p[p])[i] = v;
    }
    if (last_block(c.epoch + 5)) {
      if (threadIdx.x == 0) signal_all(c, kChanReduce, target + 1);
    }
  }
  if (threadIdx.x == 0) wait_flag(c, kChanReduce, root, target + 1);
  __syncthreads();
  const uint4* mine = reinterpret_cast<const uint4*>(bufs.p[c.me]);
  for (long i = tid; i < nvec; i += stride) out[i] = __ldcg(mine + i);
}

// Reduce to `root`: every rank has put its contribution into its own symmetric buffer; the
// owner sums all of them in rank order (fp32 accumulation) into `out`; the others only wait
// until the owner is done reading.  This is the gradient reduction of a shadowed expert
// (cuda/fastermoe/smart_schedule.cpp:41-63, ncclReduce there).
template <typename T, typename Vec, int PER>
__global__ void reduce_to_root_kernel(const __grid_constant__ ExchangeCtx c, const __grid_constant__ PeerPtrs bufs,
                                      T* __restrict__ out, long n, int root) {
  const int target = 2 * c.epoch[kReduceEpochWord];
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    st_release_sys(flag_of(c.flags.p[root], kChanReduce, c.me), target);
  }
  if (c.me == root) {
    block_wait_all(c, kChanReduce, target);
    const long nvec = n / PER;
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long>(gridDim.x) * blockDim.x) {
      float acc[PER];
#pragma unroll
      for (int q = 0; q < PER; ++q) acc[q] = 0.f;
      for (int p = 0; p < c.world; ++p) {
        Vec v = __ldcg(reinterpret_cast<const Vec*>(bufs.p[p]) + i);
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int q = 0; q < PER; ++q) acc[q] += as_float(e[q]);
      }
      Vec r;
      T* e = reinterpret_cast<T*>(&r);
#pragma unroll
      for (int q = 0; q < PER; ++q) e[q] = from_float<T>(acc[q]);
      reinterpret_cast<Vec*>(out)[i] = r;
    }
    for (long i = nvec * PER + blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long>(gridDim.x) * blockDim.x) {
      float acc = 0.f;
      for (int p = 0; p < c.world; ++p) acc += as_float(static_cast<const T*>(bufs.p[p])[i]);
      out[i] = from_float<T>(acc);
    }
    if (last_block(c.epoch + 5)) {
      if (threadIdx.x == 0) signal_all(c, kChanReduce, target + 1);
    }
  } else {
    if (threadIdx.x == 0) wait_flag(c, kChanReduce, root, target + 1);
    __syncthreads();
  }
}

// Waits until every peer has published the current epoch on `channel` (its rows have landed in
// this rank's staging buffer); the kernels behind it in the stream may then read the buffer in
// place.
__global__ void wait_arrival_kernel(const __grid_constant__ ExchangeCtx c, int channel) {
  block_wait_all(c, channel, c.epoch[0]);
}

__global__ void wait_only_kernel(const __grid_constant__ ExchangeCtx c, int channel) {
  // Waits for an epoch nobody will publish: exercises the time-out path.
  block_wait_all(c, channel, c.epoch[0] + 1000000);
}

int push_grid(int work_items, int warps_per_block) {
  int blocks = (work_items + warps_per_block - 1) / warps_per_block;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  return blocks;
}

}  // namespace

#define FMOE_P2P_16(dtype, ...)                                        \
  if ((dtype) == 0) { using T = __nv_bfloat16; __VA_ARGS__; }          \
  else { using T = __half; __VA_ARGS__; }

cudaError_t launch_count_exchange(const ExchangeCtx& ctx, const int* lec, const PeerPtrs& cnt,
                                  int n_expert, int capacity_rows, int* dst_base, int* seg_base,
                                  int* blk_base, int* expert_offs, int* seg_off, int* total_rows,
                                  int* item_prefix, int* blk_order, cudaStream_t stream) {
  const int tot = n_expert * ctx.world;
  if (n_expert >= (1 << (31 - kBlkOrderShift)) || capacity_rows / kRowBlock >= (1 << kBlkOrderShift)) {
    return cudaErrorInvalidValue;
  }
  const size_t smem = (static_cast<size_t>(ctx.world) * (tot + 1) + 4 * tot + 1) * sizeof(int);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(count_exchange_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
  }
  count_exchange_kernel<<<1, 1024, smem, stream>>>(ctx, lec, cnt, n_expert, capacity_rows, dst_base,
                                                   seg_base, blk_base, expert_offs, seg_off,
                                                   total_rows, item_prefix, blk_order);
  return cudaGetLastError();
}

cudaError_t launch_capacity_grant(const ExchangeCtx& ctx, const int* lec, const int* cap,
                                  const PeerPtrs& cnt, int n_expert, int64_t* new_lec,
                                  int64_t* new_gec, cudaStream_t stream) {
  const int width = n_expert * ctx.world + n_expert;
  const size_t smem = static_cast<size_t>(ctx.world) * width * sizeof(int);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(capacity_grant_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
  }
  capacity_grant_kernel<<<1, 1024, smem, stream>>>(ctx, lec, cap, cnt, n_expert, new_lec, new_gec);
  return cudaGetLastError();
}

cudaError_t launch_swipe_exchange(const ExchangeCtx& ctx, const int* want, const int64_t* cap,
                                  const PeerPtrs& tab, int* quota, int64_t* cap_left,
                                  cudaStream_t stream) {
  swipe_exchange_kernel<<<1, 256, 0, stream>>>(ctx, want, cap, tab, quota, cap_left);
  return cudaGetLastError();
}

cudaError_t launch_begin_epoch(const ExchangeCtx& ctx, cudaStream_t stream) {
  begin_epoch_kernel<<<1, 32, 0, stream>>>(ctx, 0);
  return cudaGetLastError();
}

cudaError_t launch_begin_reduce_epoch(const ExchangeCtx& ctx, cudaStream_t stream) {
  begin_epoch_kernel<<<1, 32, 0, stream>>>(ctx, kReduceEpochWord);
  return cudaGetLastError();
}

cudaError_t launch_dispatch_push(const ExchangeCtx& ctx, int dtype, const void* x,
                                 const int64_t* idx, const int* rank, const int* dst_base,
                                 const void* scale, const PeerPtrs& rows, const PeerPtrs& meta,
                                 int n_expert, int n_slots, int k, int d, int capacity_rows,
                                 cudaStream_t stream) {
  if (d % 8 != 0) return cudaErrorInvalidValue;
  // One block of 32 warps per SM.  Every block ends with a system-scope fence and an atomic
  // on one counter (`last_block`), and that tail, not the copy, is most of the kernel once
  // the rows are in flight: 148 blocks measured 3 us faster than 1024 blocks of 8 warps for
  // 8192 rows of 2 KB.
  const int wpb = 32;
  int grid = (n_slots + wpb - 1) / wpb;
  if (grid > 148) grid = 148;
  if (grid < 1) grid = 1;
  FMOE_P2P_16(dtype, (dispatch_push_kernel<T><<<grid, wpb * 32, 0, stream>>>(
      ctx, static_cast<const T*>(x), idx, rank, dst_base, static_cast<const T*>(scale), rows, meta,
      n_expert, n_slots, k, d, capacity_rows)));
  return cudaGetLastError();
}

cudaError_t launch_wait_copy(const ExchangeCtx& ctx, int channel, int dtype, const void* stage_rows,
                             const int64_t* stage_meta, const int* total_rows, int d,
                             int capacity_rows, void* out_rows, int64_t* out_meta,
                             cudaStream_t stream) {
  if (d % 8 != 0) return cudaErrorInvalidValue;
  FMOE_P2P_16(dtype, (wait_copy_kernel<T><<<148 * 4, 256, 0, stream>>>(
      ctx, channel, static_cast<const T*>(stage_rows), stage_meta, total_rows, d, capacity_rows,
      static_cast<T*>(out_rows), out_meta)));
  return cudaGetLastError();
}

cudaError_t launch_return_push(const ExchangeCtx& ctx, int dtype, const void* rows,
                               const int64_t* meta, const int* total_rows, const PeerPtrs& ret,
                               int d, int capacity_rows, long ret_slots, cudaStream_t stream) {
  if (d % 8 != 0) return cudaErrorInvalidValue;
  const int wpb = 32;  // one block per SM: see launch_dispatch_push
  FMOE_P2P_16(dtype, (return_push_kernel<T><<<148, wpb * 32, 0, stream>>>(
      ctx, static_cast<const T*>(rows), meta, total_rows, ret, d, capacity_rows, ret_slots)));
  return cudaGetLastError();
}

cudaError_t launch_wait_combine(const ExchangeCtx& ctx, int dtype, const void* ret,
                                const int64_t* idx, const void* weight, const int* rank,
                                const int* dst_base, int capacity_rows, int n_tokens, int k, int d,
                                void* out, void* keep, cudaStream_t stream) {
  if (d % 8 != 0) return cudaErrorInvalidValue;
  const int wpb = 8;
  FMOE_P2P_16(dtype, (wait_combine_kernel<T><<<push_grid(n_tokens, wpb), wpb * 32, 0, stream>>>(
      ctx, static_cast<const T*>(ret), idx, static_cast<const T*>(weight), rank, dst_base,
      capacity_rows, n_tokens, k, d, static_cast<T*>(out), static_cast<T*>(keep))));
  return cudaGetLastError();
}

cudaError_t launch_slot_dot(int dtype, const void* dout, const void* y, const int64_t* idx,
                            int n_slots, int k, int d, void* dscore, cudaStream_t stream) {
  if (n_slots == 0) return cudaSuccess;
  if (d % 8 != 0) return cudaErrorInvalidValue;
  const int wpb = 8;
  FMOE_P2P_16(dtype, (slot_dot_kernel<T><<<(n_slots + wpb - 1) / wpb, wpb * 32, 0, stream>>>(
      static_cast<const T*>(dout), static_cast<const T*>(y), idx, n_slots, k, d,
      static_cast<T*>(dscore))));
  return cudaGetLastError();
}

cudaError_t launch_allreduce(const ExchangeCtx& ctx, int dtype, const PeerPtrs& bufs, void* out,
                             long n, float scale, cudaStream_t stream) {
  long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (blocks < 1) blocks = 1;
  const int grid = static_cast<int>(blocks);
  if (dtype == 0) {
    allreduce_kernel<__nv_bfloat16, uint4, 8><<<grid, 256, 0, stream>>>(
        ctx, bufs, static_cast<__nv_bfloat16*>(out), n, scale);
  } else if (dtype == 1) {
    allreduce_kernel<__half, uint4, 8><<<grid, 256, 0, stream>>>(ctx, bufs, static_cast<__half*>(out),
                                                               n, scale);
  } else if (dtype == 2) {
    allreduce_kernel<float, uint4, 4><<<grid, 256, 0, stream>>>(ctx, bufs, static_cast<float*>(out),
                                                              n, scale);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_allreduce_two_shot(const ExchangeCtx& ctx, int dtype, const PeerPtrs& bufs,
                                      void* out, long n, float scale, cudaStream_t stream) {
  // Every block waits for the peers in the middle of the kernel, so the whole grid must be
  // resident at once: at most two 256-thread blocks per SM.
  long blocks = (n / 8 / ctx.world + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (blocks < 1) blocks = 1;
  const int grid = static_cast<int>(blocks);
  if (dtype == 0) {
    allreduce_two_shot_kernel<__nv_bfloat16, uint4, 8><<<grid, 256, 0, stream>>>(
        ctx, bufs, static_cast<__nv_bfloat16*>(out), n, scale);
  } else if (dtype == 1) {
    allreduce_two_shot_kernel<__half, uint4, 8><<<grid, 256, 0, stream>>>(
        ctx, bufs, static_cast<__half*>(out), n, scale);
  } else if (dtype == 2) {
    allreduce_two_shot_kernel<float, uint4, 4><<<grid, 256, 0, stream>>>(
        ctx, bufs, static_cast<float*>(out), n, scale);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_allreduce_multimem(const ExchangeCtx& ctx, int dtype, void* mc, const void* mine,
                                      void* out, long nbytes, float scale, cudaStream_t stream) {
  if (mc == nullptr || nbytes <= 0) return cudaErrorInvalidValue;
  long blocks = (nbytes / 16 / ctx.world + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;   // whole grid resident: every block waits mid-kernel
  if (blocks < 1) blocks = 1;
  const int grid = static_cast<int>(blocks);
  uint8_t* m = static_cast<uint8_t*>(mc);
  const uint8_t* l = static_cast<const uint8_t*>(mine);
  uint8_t* o = static_cast<uint8_t*>(out);
  if (dtype == 0) allreduce_multimem_kernel<0><<<grid, 256, 0, stream>>>(ctx, m, l, o, nbytes, scale);
  else if (dtype == 1) allreduce_multimem_kernel<1><<<grid, 256, 0, stream>>>(ctx, m, l, o, nbytes, scale);
  else if (dtype == 2) allreduce_multimem_kernel<2><<<grid, 256, 0, stream>>>(ctx, m, l, o, nbytes, scale);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t launch_allgather(const ExchangeCtx& ctx, const void* src, const PeerPtrs& bufs,
                             void* out, long bytes_per_rank, cudaStream_t stream) {
  if (bytes_per_rank % 16 != 0) return cudaErrorInvalidValue;
  const long nvec = bytes_per_rank / 16;
  long blocks = (nvec * ctx.world + 255) / 256;  // the copy-out is the larger loop
  if (blocks > 148 * 2) blocks = 148 * 2;        // whole grid resident: every block waits mid-kernel
  if (blocks < 1) blocks = 1;
  allgather_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      ctx, static_cast<const uint4*>(src), bufs, static_cast<uint4*>(out), nvec);
  return cudaGetLastError();
}

cudaError_t launch_broadcast(const ExchangeCtx& ctx, const void* src, const PeerPtrs& bufs, void* out,
                             long bytes, int root, cudaStream_t stream) {
  if (bytes % 16 != 0 || root < 0 || root >= ctx.world) return cudaErrorInvalidValue;
  const long nvec = bytes / 16;
  long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;  // whole grid resident: every block waits mid-kernel
  if (blocks < 1) blocks = 1;
  broadcast_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      ctx, static_cast<const uint4*>(src), bufs, static_cast<uint4*>(out), nvec, root);
  return cudaGetLastError();
}

cudaError_t launch_reduce_to_root(const ExchangeCtx& ctx, int dtype, const PeerPtrs& bufs, void* out,
                                  long n, int root, cudaStream_t stream) {
  if (root < 0 || root >= ctx.world) return cudaErrorInvalidValue;
  long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (blocks < 1) blocks = 1;
  const int grid = static_cast<int>(blocks);
  if (dtype == 0) {
    reduce_to_root_kernel<__nv_bfloat16, uint4, 8><<<grid, 256, 0, stream>>>(
        ctx, bufs, static_cast<__nv_bfloat16*>(out), n, root);
  } else if (dtype == 1) {
    reduce_to_root_kernel<__half, uint4, 8><<<grid, 256, 0, stream>>>(ctx, bufs, static_cast<__half*>(out), n, root);
  } else if (dtype == 2) {
    reduce_to_root_kernel<float, uint4, 4><<<grid, 256, 0, stream>>>(ctx, bufs, static_cast<float*>(out), n, root);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_wait_arrival(const ExchangeCtx& ctx, int channel, cudaStream_t stream) {
  wait_arrival_kernel<<<1, 32, 0, stream>>>(ctx, channel);
  return cudaGetLastError();
}

cudaError_t launch_wait_only(const ExchangeCtx& ctx, int channel, cudaStream_t stream) {
  wait_only_kernel<<<1, 32, 0, stream>>>(ctx, channel);
  return cudaGetLastError();
}

}  // namespace fmoe
