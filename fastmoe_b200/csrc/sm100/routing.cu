// Routing bookkeeping, row scatter / combine, gate top-k and balancing kernels.
//
// Replaces cuda/local_exchange.cuh (expert_count, assign_pos), cuda/balancing.cuh
// (limit_by_capacity, prune_gate_by_capacity), cuda/parallel_linear.cuh:8-53 (column_reduce)
// and the ATen index_select / index_copy_ / bmm / topk / softmax calls of the reference's layer.
// All kernels are deterministic: no result depends on the order in which atomics land.
#include "routing.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace fmoe {
namespace {

constexpr int kRouteThreads = 1024;
constexpr int kRouteSmemLimit = 200 * 1024;

__device__ __forceinline__ unsigned lanemask_lt() {
  unsigned m;
  asm volatile("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// CTA b owns the contiguous slot range [b * cta_slots, (b + 1) * cta_slots), warp w of it the
// sub-range [w * chunk, (w + 1) * chunk): pass 1 builds per-warp histograms, the CTA turns them
// into exclusive prefixes over warps, pass 2 hands every slot its rank.  Within a warp slots
// are visited in order, 32 at a time.  One CTA does everything in one launch.  For many slots
// the work is spread over several CTAs and two launches: the first (`part_out`) only writes
// every CTA's per-expert totals, the second (`part_in`) starts each CTA's prefixes at the sum
// of the totals of the CTAs before it, so ranks stay those of a single ordered scan.
__global__ void __launch_bounds__(kRouteThreads, 1)
route_kernel(const int64_t* __restrict__ idx, int n_slots, int tot, int nw, int cta_slots,
             const int* __restrict__ part_in, int* __restrict__ part_out, int* __restrict__ counts,
             int* __restrict__ rank, int* __restrict__ offs, int* __restrict__ pos) {
  extern __shared__ int hist[];  // [nw][tot], then [tot + 1] expert offsets when `pos` is wanted
  int* eoff = hist + nw * tot;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < nw * tot; i += blockDim.x) hist[i] = 0;
  __syncthreads();

  const int cta_begin = blockIdx.x * cta_slots;
  const int cta_end = min(n_slots, cta_begin + cta_slots);
  int chunk = (cta_slots + nw - 1) / nw;
  chunk = (chunk + 31) & ~31;
  const int begin = cta_begin + warp * chunk;
  const int end = min(cta_end, begin + chunk);

  if (warp < nw) {
    int* h = hist + warp * tot;
    for (int s0 = begin; s0 < end; s0 += 32) {
      const int s = s0 + lane;
      long e = (s < end) ? idx[s] : -1;
      const bool valid = e >= 0 && e < tot;
      const int key = valid ? static_cast<int>(e) : tot + lane;
      const unsigned peers = __match_any_sync(0xffffffffu, key);
      if (valid && (peers & lanemask_lt()) == 0) h[key] += __popc(peers);
      __syncwarp();
    }
  }
  __syncthreads();
  if (part_out != nullptr) {
    // first launch of the multi-CTA scheme: this CTA's totals, nothing else
    for (int e = threadIdx.x; e < tot; e += blockDim.x) {
      int run = 0;
      for (int w = 0; w < nw; ++w) run += hist[w * tot + e];
      part_out[blockIdx.x * tot + e] = run;
    }
    return;
  }
  for (int e = threadIdx.x; e < tot; e += blockDim.x) {
    int run = 0, total = 0;
    if (part_in != nullptr) {
      for (int b = 0; b < static_cast<int>(gridDim.x); ++b) {
        const int t = part_in[b * tot + e];
        if (b < static_cast<int>(blockIdx.x)) run += t;
        total += t;
      }
    }
    for (int w = 0; w < nw; ++w) {
      const int t = hist[w * tot + e];
      hist[w * tot + e] = run;
      run += t;
    }
    if (part_in == nullptr) total = run;
    if (blockIdx.x == 0) counts[e] = total;
    if (pos != nullptr || offs != nullptr) eoff[e + 1] = total;
  }
  __syncthreads();
  if (pos != nullptr || offs != nullptr) {
    // exclusive prefix of the counts: where the slots of every expert start in `pos`
    if (threadIdx.x == 0) {
      int run = 0;
      eoff[0] = 0;
      for (int e = 0; e < tot; ++e) {
        run += eoff[e + 1];
        eoff[e + 1] = run;
      }
    }
    __syncthreads();
  }
  if (warp < nw) {
    int* h = hist + warp * tot;
    for (int s0 = begin; s0 < end; s0 += 32) {
      const int s = s0 + lane;
      long e = (s < end) ? idx[s] : -1;
      const bool valid = e >= 0 && e < tot;
      const int key = valid ? static_cast<int>(e) : tot + lane;
      const unsigned peers = __match_any_sync(0xffffffffu, key);
      const int before = __popc(peers & lanemask_lt());
      int r = -1;
      if (valid) r = h[key] + before;
      __syncwarp();
      if (valid && before == 0) h[key] += __popc(peers);
      __syncwarp();
      if (s < end) rank[s] = r;
      if (pos != nullptr && valid) pos[eoff[key] + r] = s;
    }
  }
  if (offs != nullptr && blockIdx.x == 0) {
    for (int e = threadIdx.x; e <= tot; e += blockDim.x) offs[e] = eoff[e];
  }
}

__global__ void prune_kernel(const int64_t* __restrict__ idx, const int* __restrict__ rank,
                             const int* __restrict__ cap, int n_slots, int tot,
                             int64_t* __restrict__ out) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_slots) return;
  const long e = idx[s];
  out[s] = (e >= 0 && e < tot && rank[s] < cap[e]) ? e : -1;
}

__global__ void limit_kernel(const int64_t* __restrict__ ec, int* __restrict__ cap,
                             int64_t* __restrict__ eca, int n_expert, int n_worker) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_expert) return;
  long left = cap[e];
  for (int w = 0; w < n_worker; ++w) {
    const long want = ec[w * n_expert + e];
    const long room = left > 0 ? left : 0;
    eca[w * n_expert + e] = want < room ? want : room;
    left -= want;
  }
  cap[e] = static_cast<int>(left);
}

__global__ void fill_pos_kernel(const int64_t* __restrict__ idx, const int* __restrict__ rank,
                                const int* __restrict__ cum_incl, int n_slots, int tot,
                                int64_t* __restrict__ pos) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_slots) return;
  const long e = idx[s];
  if (e < 0 || e >= tot) return;
  const int base = e == 0 ? 0 : cum_incl[e - 1];
  pos[base + rank[s]] = s;
}

// SWIPE reassignment, two passes around a ranking of the moved tokens.  A token keeps its
// expert while its worker's quota lasts (slot order); `swipe_mark` writes key 0 for the others
// (and -1 for the kept ones), the routing kernel ranks them, and `swipe_assign` sends the i-th
// moved token to expert `bias` of the worker that owns the i-th unit of spare quota.
__global__ void swipe_mark_kernel(const int64_t* __restrict__ idx, const int* __restrict__ rank,
                                  const int* __restrict__ quota, int n, int n_expert, int n_worker,
                                  int64_t* __restrict__ key) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n) return;
  const long e = idx[s];
  const int w = static_cast<int>(e / n_expert);
  const bool valid = e >= 0 && w < n_worker;
  key[s] = (valid && rank[s] >= quota[w]) ? 0 : -1;
}

__global__ void swipe_assign_kernel(const int64_t* __restrict__ idx, const int64_t* __restrict__ key,
                                    const int* __restrict__ mrank, const int* __restrict__ count,
                                    const int* __restrict__ quota, int n, int n_expert, int n_worker,
                                    int bias, int64_t* __restrict__ out) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n) return;
  if (key[s] < 0) {
    out[s] = idx[s];
    return;
  }
  const int o = mrank[s];
  int run = 0, target = -1;
  for (int j = 0; j < n_worker; ++j) {
    const int kept = count[j] < quota[j] ? count[j] : quota[j];
    run += quota[j] - kept;
    if (o < run) {
      target = j;
      break;
    }
  }
  out[s] = target < 0 ? -1 : static_cast<int64_t>(target) * n_expert + bias;
}

// ------------------------------------------------------------------------------ row movement
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

// One warp per slot; d % 8 == 0.
template <typename T>
__global__ void scatter_rows_kernel(const T* __restrict__ src, const int64_t* __restrict__ idx,
                                    const int* __restrict__ rank, const int* __restrict__ base,
                                    const T* __restrict__ scale, int n_slots, int k, int d,
                                    T* __restrict__ dst, int* __restrict__ row_slot) {
  const int s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (s >= n_slots) return;
  const long e = idx[s];
  if (e < 0) return;
  const long row = static_cast<long>(base[e]) + rank[s];
  const uint4* in = reinterpret_cast<const uint4*>(src + static_cast<long>(s / k) * d);
  uint4* out = reinterpret_cast<uint4*>(dst + row * d);
  const int nv = d >> 3;
  const float sc = scale == nullptr ? 1.f : V2<T>::to_f(scale[s]);
  // Four 16-byte loads in flight per lane before the first store.
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
  if (row_slot != nullptr && lane == 0) row_slot[row] = s;
}

// One warp per token; d % 8 == 0.  At most 64 registers, so that four blocks fit on an SM and a
// batch of 4096 tokens is one wave on 148 SMs.
template <typename T>
__global__ void __launch_bounds__(256, 4) gather_combine_kernel(const T* __restrict__ rows, const int64_t* __restrict__ idx,
                                      const int* __restrict__ rank, const int* __restrict__ base,
                                      const T* __restrict__ weight, int n_tokens, int k, int d,
                                      T* __restrict__ out) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  const int nv = d >> 3;
  uint4* o = reinterpret_cast<uint4*>(out + static_cast<long>(t) * d);
  // Rows and weights of the k slots first, then four 16-byte chunks of every row in flight.
  constexpr int kMaxInline = 4;
  long rows_of[kMaxInline];
  float w_of[kMaxInline];
  const int kk = k < kMaxInline ? k : kMaxInline;
#pragma unroll
  for (int j = 0; j < kMaxInline; ++j) {
    rows_of[j] = -1;
    w_of[j] = 0.f;
    if (j < kk) {
      const int s = t * k + j;
      const long e = idx[s];
      if (e >= 0) {
        rows_of[j] = static_cast<long>(base[e]) + rank[s];
        w_of[j] = weight != nullptr ? V2<T>::to_f(weight[s]) : 1.f;
      }
    }
  }
  for (int i0 = lane; i0 < nv; i0 += 64) {
    float acc[2][8];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[u][q] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < kMaxInline; ++j) {
      if (j >= kk || rows_of[j] < 0) continue;
      const uint4* src = reinterpret_cast<const uint4*>(rows + rows_of[j] * d);
      uint4 v[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (i0 + u * 32 < nv) v[u] = __ldg(src + i0 + u * 32);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (i0 + u * 32 < nv) {
          float f[8];
          unpack8<T>(v[u], f);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[u][q] += w_of[j] * f[q];
        }
      }
    }
    for (int j = kk; j < k; ++j) {  // more than kMaxInline slots per token: plain path
      const int s = t * k + j;
      const long e = idx[s];
      if (e < 0) continue;
      const long row = static_cast<long>(base[e]) + rank[s];
      const float w = weight != nullptr ? V2<T>::to_f(weight[s]) : 1.f;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (i0 + u * 32 < nv) {
          float f[8];
          unpack8<T>(__ldg(reinterpret_cast<const uint4*>(rows + row * d) + i0 + u * 32), f);
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

// One warp per slot.
template <typename T>
__global__ void combine_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ rows,
                                   const int64_t* __restrict__ idx, const int* __restrict__ rank,
                                   const int* __restrict__ base, const T* __restrict__ weight,
                                   int n_slots, int k, int d, T* __restrict__ drows,
                                   T* __restrict__ dscore) {
  const int s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (s >= n_slots) return;
  const long e = idx[s];
  if (e < 0) {
    if (lane == 0 && dscore != nullptr) dscore[s] = V2<T>::from_f(0.f);
    return;
  }
  const long row = static_cast<long>(base[e]) + rank[s];
  const uint4* g = reinterpret_cast<const uint4*>(dout + static_cast<long>(s / k) * d);
  const uint4* y = reinterpret_cast<const uint4*>(rows + row * d);
  uint4* dy = reinterpret_cast<uint4*>(drows + row * d);
  const float w = V2<T>::to_f(weight[s]);
  const int nv = d >> 3;
  float dot = 0.f;
  for (int i = lane; i < nv; i += 32) {
    float gf[8], yf[8];
    unpack8<T>(__ldg(g + i), gf);
    unpack8<T>(__ldg(y + i), yf);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      dot += gf[q] * yf[q];
      gf[q] *= w;
    }
    dy[i] = pack8<T>(gf);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0 && dscore != nullptr) dscore[s] = V2<T>::from_f(dot);
}

// Column sums per group.  A block takes 128 rows x 256 columns; blockIdx.y enumerates the
// (group, 128-row chunk) pieces, found by scanning the offsets.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_kernel(const T* __restrict__ x, const int* __restrict__ offs, int num_groups, int n,
              long rows_cap, float* __restrict__ out) {
  __shared__ float red[8][256 + 8];
  int piece = blockIdx.x;  // pieces on x (up to 2^31 - 1 blocks), column blocks on y
  int g = 0, r0 = 0, r1 = 0;
  bool found = false;
  for (; g < num_groups; ++g) {
    const int b = offs[g], e = offs[g + 1];
    const int pieces = (e - b + 127) >> 7;
    if (piece < pieces) {
      r0 = b + piece * 128;
      r1 = min(e, r0 + 128);
      if (r1 > rows_cap) r1 = static_cast<int>(rows_cap);  // offsets past the matrix are not followed
      found = true;
      break;
    }
    piece -= pieces;
  }
  if (!found) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.y * 256 + lane * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < n) {
    for (int r = r0 + warp; r < r1; r += 8) {
      float f[8];
      unpack8<T>(__ldg(reinterpret_cast<const uint4*>(x + static_cast<long>(r) * n + col)), f);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += f[q];
    }
  }
#pragma unroll
  for (int q = 0; q < 8; ++q) red[warp][lane * 8 + q] = acc[q];
  __syncthreads();
  const int c = blockIdx.y * 256 + threadIdx.x;
  if (c < n) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
    atomicAdd(out + static_cast<long>(g) * n + c, s);
  }
}

// ------------------------------------------------------------------------------ gate
template <typename T> struct Ld;
template <> struct Ld<float> {
  static __device__ __forceinline__ float get(const float* p, long i) { return p[i]; }
  static __device__ __forceinline__ void put(float* p, long i, float v) { p[i] = v; }
};
template <> struct Ld<__nv_bfloat16> {
  static __device__ __forceinline__ float get(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }
  static __device__ __forceinline__ void put(__nv_bfloat16* p, long i, float v) { p[i] = __float2bfloat16(v); }
};
template <> struct Ld<__half> {
  static __device__ __forceinline__ float get(const __half* p, long i) { return __half2float(p[i]); }
  static __device__ __forceinline__ void put(__half* p, long i, float v) { p[i] = __float2half(v); }
};

constexpr int kMaxK = 8;

// One warp per row.  k rounds of warp arg-max; ties go to the lower expert id.
template <typename T>
__global__ void gate_topk_softmax_kernel(const T* __restrict__ logits, int n_rows, int n_experts,
                                         int k, int64_t* __restrict__ idx, T* __restrict__ prob) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const T* in = logits + static_cast<long>(row) * n_experts;
  float sel_v[kMaxK];
  int sel_i[kMaxK];
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      bool taken = false;
      for (int q = 0; q < j; ++q) taken |= (sel_i[q] == e);
      if (taken) continue;
      const float v = Ld<T>::get(in, e);
      if (v > best || (v == best && e < best_i) || best_i == 0x7fffffff) {
        best = v;
        best_i = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (oi != 0x7fffffff && (best_i == 0x7fffffff || ov > best || (ov == best && oi < best_i))) {
        best = ov;
        best_i = oi;
      }
    }
    sel_v[j] = best;
    sel_i[j] = best_i;
  }
  if (lane == 0) {
    const float mx = sel_v[0];
    float den = 0.f;
    float ex[kMaxK];
    for (int j = 0; j < k; ++j) {
      ex[j] = __expf(sel_v[j] - mx);
      den += ex[j];
    }
    for (int j = 0; j < k; ++j) {
      idx[static_cast<long>(row) * k + j] = sel_i[j];
      Ld<T>::put(prob, static_cast<long>(row) * k + j, ex[j] / den);
    }
  }
}

// dlogits[row, idx_j] = p_j * (g_j - sum_i g_i p_i), zero elsewhere.  One warp per row.
template <typename T>
__global__ void gate_topk_softmax_bwd_kernel(const T* __restrict__ dprob,
                                             const int64_t* __restrict__ idx,
                                             const T* __restrict__ prob, int n_rows, int n_experts,
                                             int k, T* __restrict__ dlogits) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  float g[kMaxK], p[kMaxK];
  int id[kMaxK];
  float dotp = 0.f;
  for (int j = 0; j < k; ++j) {
    g[j] = Ld<T>::get(dprob, static_cast<long>(row) * k + j);
    p[j] = Ld<T>::get(prob, static_cast<long>(row) * k + j);
    id[j] = static_cast<int>(idx[static_cast<long>(row) * k + j]);
    dotp += g[j] * p[j];
  }
  T* out = dlogits + static_cast<long>(row) * n_experts;
  for (int e = lane; e < n_experts; e += 32) {
    float v = 0.f;
    for (int j = 0; j < k; ++j) {
      if (id[j] == e) v = p[j] * (g[j] - dotp);
    }
    Ld<T>::put(out, e, v);
  }
}

// ------------------------------------------------------------------------------ fused gate
// logits = x W^T + b for a handful of experts (tot <= kGateMaxExperts), top-k and softmax of the
// selected logits, one warp per token: x is read once, W comes from L1/L2, nothing but the
// [B, tot] logits and the [B, k] ids / probabilities is written.
constexpr int kGateMaxExperts = 64;

template <typename T, int TOT>
__global__ void __launch_bounds__(256)
gate_linear_topk_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                        int n_rows, int d, int tot, int k, T* __restrict__ logits,
                        int64_t* __restrict__ idx, T* __restrict__ prob) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  float acc[TOT];
#pragma unroll
  for (int e = 0; e < TOT; ++e) acc[e] = 0.f;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long>(row) * d);
  const int nv = d >> 3;
#pragma unroll 4
  for (int i = lane; i < nv; i += 32) {
    float xf[8];
    unpack8<T>(__ldg(xr + i), xf);
#pragma unroll
    for (int e = 0; e < TOT; ++e) {
      if (e < tot) {
        float wf[8];
        unpack8<T>(__ldg(reinterpret_cast<const uint4*>(w + static_cast<long>(e) * d) + i), wf);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[e] = fmaf(xf[q], wf[q], acc[e]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < TOT; ++e) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
    if (e < tot && bias != nullptr) acc[e] += V2<T>::to_f(bias[e]);
    // the logits leave in the layer's dtype; selection below uses the rounded values so that
    // ids and probabilities are consistent with what autograd consumers see
    if (e < tot) acc[e] = V2<T>::to_f(V2<T>::from_f(acc[e]));
  }
  if (lane < tot) {
    float mine = 0.f;
#pragma unroll
    for (int e = 0; e < TOT; ++e) {
      if (e == lane) mine = acc[e];
    }
    logits[static_cast<long>(row) * tot + lane] = V2<T>::from_f(mine);
  }
  if (TOT > 32 && lane + 32 < tot) {
    float mine = 0.f;
#pragma unroll
    for (int e = 0; e < TOT; ++e) {
      if (e == lane + 32) mine = acc[e];
    }
    logits[static_cast<long>(row) * tot + lane + 32] = V2<T>::from_f(mine);
  }
  if (lane == 0) {
    float sel_v[kMaxK];
    int sel_i[kMaxK];
    unsigned long long taken = 0ull;
    for (int j = 0; j < k; ++j) {
      float best = -INFINITY;
      int best_i = -1;
#pragma unroll
      for (int e = 0; e < TOT; ++e) {
        if (e < tot && !((taken >> e) & 1ull) && (best_i < 0 || acc[e] > best)) {
          best = acc[e];
          best_i = e;
        }
      }
      taken |= 1ull << best_i;
      sel_v[j] = best;
      sel_i[j] = best_i;
    }
    float den = 0.f, ex[kMaxK];
    for (int j = 0; j < k; ++j) {
      ex[j] = __expf(sel_v[j] - sel_v[0]);
      den += ex[j];
    }
    for (int j = 0; j < k; ++j) {
      idx[static_cast<long>(row) * k + j] = sel_i[j];
      prob[static_cast<long>(row) * k + j] = V2<T>::from_f(ex[j] / den);
    }
  }
}

// dl[t, e] = softmax backward of the selected logits scattered to their experts, plus the
// gradient that reached the logits directly (may be null).  dx[t, :] = sum_e dl[t, e] W[e, :].
// dl is written out (fp32) for the weight-gradient kernel.  One warp per token.
template <typename T, int TOT>
__global__ void __launch_bounds__(256)
gate_bwd_dx_kernel(const T* __restrict__ dprob, const int64_t* __restrict__ idx,
                   const T* __restrict__ prob, const T* __restrict__ dlogits_in,
                   const T* __restrict__ w, int n_rows, int d, int tot, int k,
                   float* __restrict__ dl_out, T* __restrict__ dx) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  float dl[TOT];
#pragma unroll
  for (int e = 0; e < TOT; ++e) {
    dl[e] = (e < tot && dlogits_in != nullptr)
                ? V2<T>::to_f(dlogits_in[static_cast<long>(row) * tot + e]) : 0.f;
  }
  if (dprob != nullptr) {
    float g[kMaxK], pj[kMaxK];
    int id[kMaxK];
    float dotp = 0.f;
    for (int j = 0; j < k; ++j) {
      g[j] = V2<T>::to_f(dprob[static_cast<long>(row) * k + j]);
      pj[j] = V2<T>::to_f(prob[static_cast<long>(row) * k + j]);
      id[j] = static_cast<int>(idx[static_cast<long>(row) * k + j]);
      dotp += g[j] * pj[j];
    }
    for (int j = 0; j < k; ++j) {
      const float v = pj[j] * (g[j] - dotp);
#pragma unroll
      for (int e = 0; e < TOT; ++e) {
        if (e == id[j]) dl[e] += v;
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int e = 0; e < TOT; ++e) {
      if (e < tot) dl_out[static_cast<long>(row) * tot + e] = dl[e];
    }
  }
  if (dx != nullptr) {
    uint4* out = reinterpret_cast<uint4*>(dx + static_cast<long>(row) * d);
    const int nv = d >> 3;
#pragma unroll 4
    for (int i = lane; i < nv; i += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int e = 0; e < TOT; ++e) {
        if (e < tot && dl[e] != 0.f) {
          float wf[8];
          unpack8<T>(__ldg(reinterpret_cast<const uint4*>(w + static_cast<long>(e) * d) + i), wf);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] = fmaf(dl[e], wf[q], acc[q]);
        }
      }
      out[i] = pack8<T>(acc);
    }
  }
}

// dW[e, c] += sum_t dl[t, e] x[t, c] and db[e] += sum_t dl[t, e] (fp32, pre-zeroed).  A block
// takes a 64-column strip and one of `gridDim.y` token ranges; a lane owns two columns.
template <typename T, int TOT>
__global__ void __launch_bounds__(256)
gate_bwd_dw_kernel(const float* __restrict__ dl, const T* __restrict__ x, int n_rows, int d, int tot,
                   float* __restrict__ dw, float* __restrict__ db) {
  __shared__ float red[8][TOT][64 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 64 + lane * 2;
  const int per = (n_rows + gridDim.y - 1) / gridDim.y;
  const int t0 = blockIdx.y * per, t1 = min(n_rows, t0 + per);
  float a0[TOT], a1[TOT], bsum[TOT];
#pragma unroll
  for (int e = 0; e < TOT; ++e) a0[e] = a1[e] = bsum[e] = 0.f;
#pragma unroll 4
  for (int t = t0 + warp; t < t1; t += 8) {
    float x0 = 0.f, x1 = 0.f;
    if (col < d) {
      const typename V2<T>::type v = *reinterpret_cast<const typename V2<T>::type*>(x + static_cast<long>(t) * d + col);
      const float2 f = V2<T>::to_f2(v);
      x0 = f.x;
      x1 = f.y;
    }
#pragma unroll
    for (int e = 0; e < TOT; ++e) {
      if (e < tot) {
        const float g = __ldg(dl + static_cast<long>(t) * tot + e);
        a0[e] = fmaf(g, x0, a0[e]);
        a1[e] = fmaf(g, x1, a1[e]);
        bsum[e] += g;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < TOT; ++e) {
    red[warp][e][lane * 2] = a0[e];
    red[warp][e][lane * 2 + 1] = a1[e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < tot * 64; i += blockDim.x) {
    const int e = i / 64, c = i % 64;
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < 8; ++wv) s += red[wv][e][c];
    if (blockIdx.x * 64 + c < d) atomicAdd(dw + static_cast<long>(e) * d + blockIdx.x * 64 + c, s);
  }
  if (db != nullptr && blockIdx.x == 0 && lane == 0) {
#pragma unroll
    for (int e = 0; e < TOT; ++e) {
      if (e < tot) atomicAdd(db + e, bsum[e]);
    }
  }
}

// ------------------------------------------------------------------------------ SIMT GEMM
template <typename T> struct Acc { using type = float; };
template <> struct Acc<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type ldv(const T* p, long i) {
  return static_cast<typename Acc<T>::type>(p[i]);
}
template <> __device__ __forceinline__ float ldv<__nv_bfloat16>(const __nv_bfloat16* p, long i) {
  return __bfloat162float(p[i]);
}
template <> __device__ __forceinline__ float ldv<__half>(const __half* p, long i) {
  return __half2float(p[i]);
}
template <typename T> __device__ __forceinline__ void stv(T* p, long i, typename Acc<T>::type v) {
  p[i] = static_cast<T>(v);
}
template <> __device__ __forceinline__ void stv<__nv_bfloat16>(__nv_bfloat16* p, long i, float v) {
  p[i] = __float2bfloat16(v);
}
template <> __device__ __forceinline__ void stv<__half>(__half* p, long i, float v) {
  p[i] = __float2half(v);
}

__device__ __forceinline__ int group_of_row(const int* offs, int num_groups, int row) {
  int lo = 0, hi = num_groups;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (offs[mid] <= row) lo = mid; else hi = mid;
  }
  return lo;
}

// Shared-memory tiled SIMT GEMM for the reference-precision types (fp32, fp64) and for 16-bit
// shapes the tensor-core kernel does not take.  One CTA of 256 threads computes a 64 x 64 tile
// of C = A B with a K step of 16; every thread owns a 4 x 4 block of the tile and accumulates in
// fp32 (fp64 for doubles).  The three products of a grouped linear differ only in where A(i, kk)
// and B(kk, j) live:
//   mode 0 (NT)   rows of expert g:  A = a[row, kk],   B = b[g, j, kk]
//   mode 1 (NN)   rows of expert g:  A = a[row, kk],   B = b[g, kk, j]
//   mode 2 (wgrad) out[g, i, j]:     A = p[r0 + kk, i], B = q[r0 + kk, j], K = rows of expert g
// (the reference calls cublasSgemm / cublasDgemm per expert here, cuda/utils/cublas_wrapper.h:51-72).
constexpr int kSimtTile = 64;
constexpr int kSimtK = 16;

template <typename T, int MODE>
__global__ void __launch_bounds__(256)
simt_tiled_kernel(int num_groups, int m, int n, int k, const T* __restrict__ a, const T* __restrict__ b,
                  const int* __restrict__ offs, const T* __restrict__ bias, T* __restrict__ out) {
  using A = typename Acc<T>::type;
  __shared__ A As[kSimtK][kSimtTile + 4];
  __shared__ A Bs[kSimtK][kSimtTile + 4];
  int g, i0, rows_i, kk_total, row_base;
  const int j0 = blockIdx.y * kSimtTile;
  if (MODE == 2) {
    g = blockIdx.z;
    i0 = blockIdx.x * kSimtTile;
    rows_i = m;
    row_base = offs[g];
    kk_total = offs[g + 1] - row_base;
  } else {
    // blockIdx.x walks the 64-row pieces of all experts: find the expert this piece belongs to
    int piece = blockIdx.x;
    bool found = false;
    for (g = 0; g < num_groups; ++g) {
      const int cnt = offs[g + 1] - offs[g];
      const int pieces = (cnt + kSimtTile - 1) / kSimtTile;
      if (piece < pieces) {
        found = true;
        break;
      }
      piece -= pieces;
    }
    if (!found) return;
    row_base = offs[g];
    i0 = piece * kSimtTile;
    rows_i = offs[g + 1] - row_base;
    kk_total = k;
  }
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  A acc[4][4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
#pragma unroll
    for (int v = 0; v < 4; ++v) acc[u][v] = 0;
  }
  for (int kk0 = 0; kk0 < kk_total; kk0 += kSimtK) {
    // 16 x 64 elements of each operand, 4 per thread
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const int e = threadIdx.x + l * 256;
      int kk, ii;
      if (MODE == 2) { kk = e / kSimtTile; ii = e % kSimtTile; }    // A is row-major over (kk, i)
      else { ii = e / kSimtK; kk = e % kSimtK; }                    // A is row-major over (i, kk)
      A va = 0;
      if (kk0 + kk < kk_total && i0 + ii < rows_i) {
        va = MODE == 2 ? ldv<T>(a, static_cast<long>(row_base + kk0 + kk) * m + i0 + ii)
                       : ldv<T>(a, static_cast<long>(row_base + i0 + ii) * k + kk0 + kk);
      }
      As[kk][ii] = va;
      int kb, jj;
      if (MODE == 0) { jj = e / kSimtK; kb = e % kSimtK; }          // B is row-major over (j, kk)
      else { kb = e / kSimtTile; jj = e % kSimtTile; }              // B is row-major over (kk, j)
      A vb = 0;
      if (kk0 + kb < kk_total && j0 + jj < n) {
        if (MODE == 0) vb = ldv<T>(b, (static_cast<long>(g) * n + j0 + jj) * k + kk0 + kb);
        else if (MODE == 1) vb = ldv<T>(b, (static_cast<long>(g) * k + kk0 + kb) * n + j0 + jj);
        else vb = ldv<T>(b, static_cast<long>(row_base + kk0 + kb) * n + j0 + jj);
      }
      Bs[kb][jj] = vb;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSimtK; ++kk) {
      A ra[4], rb[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) ra[u] = As[kk][ty * 4 + u];
#pragma unroll
      for (int v = 0; v < 4; ++v) rb[v] = Bs[kk][tx * 4 + v];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] += ra[u] * rb[v];
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int ii = i0 + ty * 4 + u;
    if (ii >= rows_i) continue;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int jj = j0 + tx * 4 + v;
      if (jj >= n) continue;
      A val = acc[u][v];
      if (MODE != 2 && bias != nullptr) val += ldv<T>(bias, static_cast<long>(g) * n + jj);
      const long o = MODE == 2 ? (static_cast<long>(g) * m + ii) * n + jj
                               : static_cast<long>(row_base + ii) * n + jj;
      stv<T>(out, o, val);
    }
  }
}

template <typename T>
cudaError_t simt_typed(int mode, int num_groups, long rows_cap, int m, int n, int k, const void* a,
                       const void* b, const int* offs, const void* bias, void* out,
                       cudaStream_t stream) {
  const T* ap = static_cast<const T*>(a);
  const T* bp = static_cast<const T*>(b);
  const T* biasp = static_cast<const T*>(bias);
  T* op = static_cast<T*>(out);
  const unsigned nt = (n + kSimtTile - 1) / kSimtTile;
  if (mode == 2) {
    dim3 grid((m + kSimtTile - 1) / kSimtTile, nt, num_groups);
    simt_tiled_kernel<T, 2><<<grid, 256, 0, stream>>>(num_groups, m, n, k, ap, bp, offs, biasp, op);
  } else {
    if (rows_cap == 0) return cudaSuccess;
    dim3 grid(static_cast<unsigned>((rows_cap + kSimtTile - 1) / kSimtTile + num_groups), nt);
    if (mode == 0) {
      simt_tiled_kernel<T, 0><<<grid, 256, 0, stream>>>(num_groups, m, n, k, ap, bp, offs, biasp, op);
    } else {
      simt_tiled_kernel<T, 1><<<grid, 256, 0, stream>>>(num_groups, m, n, k, ap, bp, offs, biasp, op);
    }
  }
  return cudaGetLastError();
}

}  // namespace

// ------------------------------------------------------------------------------ launchers
int route_blocks(int n_slots) {
  // one CTA up to 32 K slots (a single launch, about 8 us); beyond that 16 K slots per CTA
  if (n_slots <= 32768) return 1;
  int nb = (n_slots + 16383) / 16384;
  return nb > 148 ? 148 : nb;
}

cudaError_t launch_route(const int64_t* idx, int n_slots, int tot, int* counts, int* rank,
                         int* offs, int* pos, int* part, cudaStream_t stream) {
  if (tot <= 0) return cudaErrorInvalidValue;
  int nw = (kRouteSmemLimit - 4 * (tot + 1)) / (4 * tot);
  if (nw < 1) return cudaErrorInvalidValue;
  if (nw > 32) nw = 32;
  const int nb = part != nullptr ? route_blocks(n_slots) : 1;
  int cta_slots = (n_slots + nb - 1) / nb;
  cta_slots = (cta_slots + 31) & ~31;
  if (cta_slots < 32) cta_slots = 32;
  const int by_work = (cta_slots + 31) / 32;
  if (nw > by_work) nw = by_work > 0 ? by_work : 1;
  const size_t smem = static_cast<size_t>(nw) * tot * 4 + static_cast<size_t>(tot + 1) * 4;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kRouteSmemLimit);
    if (e != cudaSuccess) return e;
  }
  if (nb > 1) {
    route_kernel<<<nb, kRouteThreads, smem, stream>>>(idx, n_slots, tot, nw, cta_slots, nullptr, part,
                                                     counts, rank, offs, pos);
    route_kernel<<<nb, kRouteThreads, smem, stream>>>(idx, n_slots, tot, nw, cta_slots, part, nullptr,
                                                     counts, rank, offs, pos);
  } else {
    route_kernel<<<1, kRouteThreads, smem, stream>>>(idx, n_slots, tot, nw, cta_slots, nullptr, nullptr,
                                                    counts, rank, offs, pos);
  }
  return cudaGetLastError();
}

cudaError_t launch_swipe_mark(const int64_t* idx, const int* rank, const int* quota, int n,
                              int n_expert, int n_worker, int64_t* key, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  swipe_mark_kernel<<<(n + 255) / 256, 256, 0, stream>>>(idx, rank, quota, n, n_expert, n_worker, key);
  return cudaGetLastError();
}

cudaError_t launch_swipe_assign(const int64_t* idx, const int64_t* key, const int* mrank,
                                const int* count, const int* quota, int n, int n_expert,
                                int n_worker, int bias, int64_t* out, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  swipe_assign_kernel<<<(n + 255) / 256, 256, 0, stream>>>(idx, key, mrank, count, quota, n, n_expert,
                                                          n_worker, bias, out);
  return cudaGetLastError();
}

cudaError_t launch_prune(const int64_t* idx, const int* rank, const int* cap, int n_slots, int tot,
                         int64_t* new_idx, cudaStream_t stream) {
  if (n_slots == 0) return cudaSuccess;
  prune_kernel<<<(n_slots + 255) / 256, 256, 0, stream>>>(idx, rank, cap, n_slots, tot, new_idx);
  return cudaGetLastError();
}

cudaError_t launch_limit_by_capacity(const int64_t* ec, int* cap, int64_t* eca, int n_expert,
                                     int n_worker, cudaStream_t stream) {
  limit_kernel<<<(n_expert + 127) / 128, 128, 0, stream>>>(ec, cap, eca, n_expert, n_worker);
  return cudaGetLastError();
}

cudaError_t launch_fill_pos(const int64_t* idx, const int* rank, const int* cum_incl, int n_slots,
                            int tot, int64_t* pos, cudaStream_t stream) {
  if (n_slots == 0) return cudaSuccess;
  fill_pos_kernel<<<(n_slots + 255) / 256, 256, 0, stream>>>(idx, rank, cum_incl, n_slots, tot, pos);
  return cudaGetLastError();
}

#define FMOE_DISPATCH_16(dtype, ...)                                  \
  if ((dtype) == 0) { using T = __nv_bfloat16; __VA_ARGS__; }         \
  else { using T = __half; __VA_ARGS__; }

cudaError_t launch_scatter_rows(int dtype, const void* src, const int64_t* idx, const int* rank,
                                const int* base, const void* scale, int n_slots, int k, int d,
                                void* dst, int* row_slot, cudaStream_t stream) {
  if (n_slots == 0) return cudaSuccess;
  if (d % 8 != 0) return cudaErrorInvalidValue;
  const int wpb = 8;
  FMOE_DISPATCH_16(dtype, (scatter_rows_kernel<T><<<(n_slots + wpb - 1) / wpb, wpb * 32, 0, stream>>>(
      static_cast<const T*>(src), idx, rank, base, static_cast<const T*>(scale), n_slots, k, d,
      static_cast<T*>(dst), row_slot)));
  return cudaGetLastError();
}

cudaError_t launch_gather_combine(int dtype, const void* rows, const int64_t* idx, const int* rank,
                                  const int* base, const void* weight, int n_tokens, int k, int d,
                                  void* out, cudaStream_t stream) {
  if (n_tokens == 0) return cudaSuccess;
  if (d % 8 != 0) return cudaErrorInvalidValue;
  const int wpb = 8;
  FMOE_DISPATCH_16(dtype, (gather_combine_kernel<T><<<(n_tokens + wpb - 1) / wpb, wpb * 32, 0, stream>>>(
      static_cast<const T*>(rows), idx, rank, base, static_cast<const T*>(weight), n_tokens, k, d,
      static_cast<T*>(out))));
  return cudaGetLastError();
}

cudaError_t launch_combine_bwd(int dtype, const void* dout, const void* rows, const int64_t* idx,
                               const int* rank, const int* base, const void* weight, int n_tokens,
                               int k, int d, void* drows, void* dscore, cudaStream_t stream) {
  const int n_slots = n_tokens * k;
  if (n_slots == 0) return cudaSuccess;
  if (d % 8 != 0) return cudaErrorInvalidValue;
  const int wpb = 8;
  FMOE_DISPATCH_16(dtype, (combine_bwd_kernel<T><<<(n_slots + wpb - 1) / wpb, wpb * 32, 0, stream>>>(
      static_cast<const T*>(dout), static_cast<const T*>(rows), idx, rank, base,
      static_cast<const T*>(weight), n_slots, k, d, static_cast<T*>(drows),
      static_cast<T*>(dscore))));
  return cudaGetLastError();
}

cudaError_t launch_colsum(int dtype, const void* x, const int* offs, int num_groups, long rows_cap,
                          int n, float* out, cudaStream_t stream) {
  if (rows_cap == 0) return cudaSuccess;
  if (n % 8 != 0) return cudaErrorInvalidValue;
  if ((n + 255) / 256 > 65535 || (rows_cap + 127) / 128 + num_groups > 2147483647L) {
    return cudaErrorInvalidValue;
  }
  dim3 grid(static_cast<unsigned>((rows_cap + 127) / 128 + num_groups), (n + 255) / 256);
  FMOE_DISPATCH_16(dtype, (colsum_kernel<T><<<grid, 256, 0, stream>>>(
      static_cast<const T*>(x), offs, num_groups, n, rows_cap, out)));
  return cudaGetLastError();
}

cudaError_t launch_gate_topk_softmax(int logit_dtype, const void* logits, int n_rows, int n_experts,
                                     int k, int64_t* idx, void* prob, cudaStream_t stream) {
  if (n_rows == 0) return cudaSuccess;
  if (k < 1 || k > kMaxK || k > n_experts) return cudaErrorInvalidValue;
  const int wpb = 8;
  const int grid = (n_rows + wpb - 1) / wpb;
  if (logit_dtype == 0) {
    gate_topk_softmax_kernel<__nv_bfloat16><<<grid, wpb * 32, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), n_rows, n_experts, k, idx,
        static_cast<__nv_bfloat16*>(prob));
  } else if (logit_dtype == 1) {
    gate_topk_softmax_kernel<__half><<<grid, wpb * 32, 0, stream>>>(
        static_cast<const __half*>(logits), n_rows, n_experts, k, idx, static_cast<__half*>(prob));
  } else {
    gate_topk_softmax_kernel<float><<<grid, wpb * 32, 0, stream>>>(
        static_cast<const float*>(logits), n_rows, n_experts, k, idx, static_cast<float*>(prob));
  }
  return cudaGetLastError();
}

cudaError_t launch_gate_topk_softmax_bwd(int logit_dtype, const void* dprob, const int64_t* idx,
                                         const void* prob, int n_rows, int n_experts, int k,
                                         void* dlogits, cudaStream_t stream) {
  if (n_rows == 0) return cudaSuccess;
  if (k < 1 || k > kMaxK) return cudaErrorInvalidValue;
  const int wpb = 8;
  const int grid = (n_rows + wpb - 1) / wpb;
  if (logit_dtype == 0) {
    gate_topk_softmax_bwd_kernel<__nv_bfloat16><<<grid, wpb * 32, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(dprob), idx, static_cast<const __nv_bfloat16*>(prob),
        n_rows, n_experts, k, static_cast<__nv_bfloat16*>(dlogits));
  } else if (logit_dtype == 1) {
    gate_topk_softmax_bwd_kernel<__half><<<grid, wpb * 32, 0, stream>>>(
        static_cast<const __half*>(dprob), idx, static_cast<const __half*>(prob), n_rows,
        n_experts, k, static_cast<__half*>(dlogits));
  } else {
    gate_topk_softmax_bwd_kernel<float><<<grid, wpb * 32, 0, stream>>>(
        static_cast<const float*>(dprob), idx, static_cast<const float*>(prob), n_rows, n_experts,
        k, static_cast<float*>(dlogits));
  }
  return cudaGetLastError();
}

#define FMOE_GATE_TOT(tot, ...)                          \
  if ((tot) <= 2) { constexpr int TOT = 2; __VA_ARGS__; }       \
  else if ((tot) <= 4) { constexpr int TOT = 4; __VA_ARGS__; }  \
  else if ((tot) <= 8) { constexpr int TOT = 8; __VA_ARGS__; }  \
  else if ((tot) <= 16) { constexpr int TOT = 16; __VA_ARGS__; } \
  else if ((tot) <= 32) { constexpr int TOT = 32; __VA_ARGS__; } \
  else { constexpr int TOT = 64; __VA_ARGS__; }

bool gate_fused_supported(int tot, int d, int k) {
  return tot >= 1 && tot <= kGateMaxExperts && d % 8 == 0 && k >= 1 && k <= kMaxK && k <= tot;
}

cudaError_t launch_gate_linear_topk(int dtype, const void* x, const void* w, const void* bias,
                                    int n_rows, int d, int tot, int k, void* logits, int64_t* idx,
                                    void* prob, cudaStream_t stream) {
  if (n_rows == 0) return cudaSuccess;
  if (!gate_fused_supported(tot, d, k)) return cudaErrorInvalidValue;
  const int grid = (n_rows + 7) / 8;
  FMOE_DISPATCH_16(dtype, FMOE_GATE_TOT(tot, (gate_linear_topk_kernel<T, TOT><<<grid, 256, 0, stream>>>(
      static_cast<const T*>(x), static_cast<const T*>(w), static_cast<const T*>(bias), n_rows, d, tot,
      k, static_cast<T*>(logits), idx, static_cast<T*>(prob)))));
  return cudaGetLastError();
}

cudaError_t launch_gate_bwd(int dtype, const void* dprob, const int64_t* idx, const void* prob,
                            const void* dlogits_in, const void* x, const void* w, int n_rows, int d,
                            int tot, int k, float* dl_scratch, void* dx, float* dw, float* db,
                            cudaStream_t stream) {
  if (n_rows == 0) return cudaSuccess;
  if (!gate_fused_supported(tot, d, k)) return cudaErrorInvalidValue;
  const int grid = (n_rows + 7) / 8;
  FMOE_DISPATCH_16(dtype, FMOE_GATE_TOT(tot, (gate_bwd_dx_kernel<T, TOT><<<grid, 256, 0, stream>>>(
      static_cast<const T*>(dprob), idx, static_cast<const T*>(prob), static_cast<const T*>(dlogits_in),
      static_cast<const T*>(w), n_rows, d, tot, k, dl_scratch, static_cast<T*>(dx)))));
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  if (dw == nullptr) return cudaSuccess;
  if (tot > 16) return cudaErrorInvalidValue;
  // Each warp walks its token range serially (one dependent load chain), so the ranges are
  // kept short: many blocks, a few tokens per warp, partial sums merged with atomics.
  int splits = n_rows / 64;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  dim3 g2((d + 63) / 64, splits);
  if (tot <= 2) {
    FMOE_DISPATCH_16(dtype, (gate_bwd_dw_kernel<T, 2><<<g2, 256, 0, stream>>>(
        dl_scratch, static_cast<const T*>(x), n_rows, d, tot, dw, db)));
  } else if (tot <= 8) {
    FMOE_DISPATCH_16(dtype, (gate_bwd_dw_kernel<T, 8><<<g2, 256, 0, stream>>>(
        dl_scratch, static_cast<const T*>(x), n_rows, d, tot, dw, db)));
  } else {
    FMOE_DISPATCH_16(dtype, (gate_bwd_dw_kernel<T, 16><<<g2, 256, 0, stream>>>(
        dl_scratch, static_cast<const T*>(x), n_rows, d, tot, dw, db)));
  }
  return cudaGetLastError();
}

cudaError_t launch_simt_grouped_gemm(int mode, int elem, int num_groups, long rows_cap, int m, int n,
                                     int k, const void* a, const void* b, const int* offs,
                                     const void* bias, void* out, cudaStream_t stream) {
  switch (elem) {
    case 0: return simt_typed<__nv_bfloat16>(mode, num_groups, rows_cap, m, n, k, a, b, offs, bias, out, stream);
    case 1: return simt_typed<__half>(mode, num_groups, rows_cap, m, n, k, a, b, offs, bias, out, stream);
    case 2: return simt_typed<float>(mode, num_groups, rows_cap, m, n, k, a, b, offs, bias, out, stream);
    case 3: return simt_typed<double>(mode, num_groups, rows_cap, m, n, k, a, b, offs, bias, out, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace fmoe
