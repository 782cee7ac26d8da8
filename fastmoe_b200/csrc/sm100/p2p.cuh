// Peer-to-peer (NVLink 5 / NVSwitch) kernels of the expert-parallel data path.
//
// They replace the reference's host-driven exchange — the NCCL all-to-all of counts
// (cuda/global_exchange.cpp:9-46) and the per-(expert, peer) ncclSend/ncclRecv loops of
// global_scatter / global_gather (cuda/global_exchange.h:11-100) — with kernels that store
// straight into the peers' symmetric buffers and publish completion through flags.  No count
// ever reaches the host, and every wait on a peer is bounded.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fmoe {

constexpr int kMaxPeers = 16;

struct PeerPtrs {
  void* p[kMaxPeers];
};

// Status codes written to the status word when something goes wrong (0 = fine).
constexpr int kStatusPeerTimeout = 201;      // a peer's flag did not arrive in time
constexpr int kStatusRecvOverflow = 202;     // more rows routed to a rank than its buffer holds
constexpr int kStatusCapacityMismatch = 203; // the ranks of a group sized their receive buffers differently

#ifdef __CUDACC__
// A receive overflow is a report, not a failure: rows beyond the buffer are dropped, everything
// else of the step is still exchanged and computed.  Every other code means that a wait gave up;
// later waits on the same GPU then end at once instead of spending a full time-out each.
__device__ __forceinline__ bool status_is_failure(int s) { return s != 0 && s != kStatusRecvOverflow; }
// First failure wins; a failure replaces an overflow report.
__device__ __forceinline__ void record_failure(int* status, int code) {
  const int old = atomicCAS(status, 0, code);
  if (old == kStatusRecvOverflow) atomicCAS(status, kStatusRecvOverflow, code);
}
#endif

// Arrival of dispatched rows is tracked per block of this many rows of the receive buffer
// (the M extent of a GEMM tile).
constexpr int kRowBlock = 128;
// An entry of the block-order table: (local expert << kBlkOrderShift) | block inside the expert.
constexpr int kBlkOrderShift = 20;

// Flag channels inside the symmetric signal buffer: int32 [kNumChannels][kMaxPeers].
constexpr int kChanCounts = 0;
constexpr int kChanDispatch = 1;
constexpr int kChanReturn = 2;
constexpr int kChanReduce = 3;
constexpr int kNumChannels = 4;

// Word of the local epoch array that counts the reductions (all-reduce, all-gather): separate
// from the exchange epoch [0], so a gradient reduction on a side stream may run beside a layer.
constexpr int kReduceEpochWord = 6;

struct ExchangeCtx {
  PeerPtrs flags;        // each peer's signal buffer
  int* epoch;            // local int32[8]: [0] exchange epoch, [1]-[4] CTA completion counters
                         // (dispatch, return, reduce, GEMM push), [6] reduction epoch
  int me;
  int world;
  int* status;           // local status word
  unsigned long long timeout_ns;
};

// Starts a new exchange epoch and (forward only) exchanges the routing counts:
//   lec[tot]            my tokens per global expert
//   cnt                 every peer's count matrix int32 [world][tot + 1] (symmetric; the last
//                       entry of a row is that rank's receive capacity)
// Outputs, all in local memory:
//   dst_base[tot]       first row of my rows inside the owner's receive buffer, per global expert
//   seg_base[tot]       first row of the expert's whole segment on its owner
//   blk_base[tot]       index of the segment's first kRowBlock-row block on its owner
//   expert_offs[E + 1]  row offsets of my local experts inside my receive buffer
//   seg_off[E][world + 1]  inside my expert e, the row where the rows of the j-th source begin
//                       (source j is rank (me - j) mod world)
//   total_rows[1]
//   item_prefix[tot + 1]  exclusive prefix of the number of kRowBlock-row blocks my rows touch
//                       on the owner, per (peer, expert) pair in send order: peer distance j
//                       outer, local expert e inner, global expert ((me + j) mod world) * E + e
//   blk_order[capacity / kRowBlock + E]  my kRowBlock-row blocks in the order their rows arrive:
//                       source position of the block's last row outer, expert, then row
cudaError_t launch_count_exchange(const ExchangeCtx& ctx, const int* lec, const PeerPtrs& cnt,
                                  int n_expert, int capacity_rows, int* dst_base, int* seg_base,
                                  int* blk_base, int* expert_offs, int* seg_off, int* total_rows,
                                  int* item_prefix, int* blk_order, cudaStream_t stream);

// Backward passes reuse the forward routing: only the epoch advances.
cudaError_t launch_begin_epoch(const ExchangeCtx& ctx, cudaStream_t stream);
// Advances the reduction epoch (all-reduce and all-gather launches follow it).
cudaError_t launch_begin_reduce_epoch(const ExchangeCtx& ctx, cudaStream_t stream);

// rows[p][dst_base[g] + rank[s]] = scale[s] * x[s / k]  on the owner p = g / n_expert of the
// slot's expert g, plus meta[p][row] = (me << 32) | s.  The last CTA publishes the flags.
cudaError_t launch_dispatch_push(const ExchangeCtx& ctx, int dtype, const void* x,
                                 const int64_t* idx, const int* rank, const int* dst_base,
                                 const void* scale, const PeerPtrs& rows, const PeerPtrs& meta,
                                 int n_expert, int n_slots, int k, int d, int capacity_rows,
                                 cudaStream_t stream);

// Waits for every peer's flag on `channel`, then copies the first total_rows rows (and their
// meta words when requested) out of the staging buffers.
cudaError_t launch_wait_copy(const ExchangeCtx& ctx, int channel, int dtype, const void* stage_rows,
                             const int64_t* stage_meta, const int* total_rows, int d,
                             int capacity_rows, void* out_rows, int64_t* out_meta,
                             cudaStream_t stream);

// ret[src][slot] = rows[r] for every received row r with meta[r] = (src << 32) | slot; rows
// whose source or slot (>= ret_slots, the rows of every return buffer) is out of range are skipped.
cudaError_t launch_return_push(const ExchangeCtx& ctx, int dtype, const void* rows,
                               const int64_t* meta, const int* total_rows, const PeerPtrs& ret,
                               int d, int capacity_rows, long ret_slots, cudaStream_t stream);

// Waits for the return flags, then out[t] = sum_j w[t, j] * ret[t * k + j] over kept slots
// (w = 1 when null) and, when `keep` is given, keep[s] = ret[s] for the backward pass.  With
// `rank` / `dst_base` / `capacity_rows` a slot whose row dst_base[idx[s]] + rank[s] lies beyond
// the owner's receive buffer (it was never sent) counts as zero.
cudaError_t launch_wait_combine(const ExchangeCtx& ctx, int dtype, const void* ret,
                                const int64_t* idx, const void* weight, const int* rank,
                                const int* dst_base, int capacity_rows, int n_tokens, int k, int d,
                                void* out, void* keep, cudaStream_t stream);

// dscore[s] = <dout[s / k], y[s]>  (0 for dropped slots)
cudaError_t launch_slot_dot(int dtype, const void* dout, const void* y, const int64_t* idx,
                            int n_slots, int k, int d, void* dscore, cudaStream_t stream);

// In-place sum over ranks of a symmetric buffer (one-shot: every rank reads all peers), with
// scaling; `n` elements of 16-bit or fp32 type (dtype: 0 bf16, 1 f16, 2 f32).
cudaError_t launch_allreduce(const ExchangeCtx& ctx, int dtype, const PeerPtrs& bufs, void* out,
                             long n, float scale, cudaStream_t stream);

// Same result for large buckets (two-shot: reduce-scatter into every peer's buffer, then a
// local copy-out).  The symmetric buffers must hold `n` rounded up to 16 bytes.
cudaError_t launch_allreduce_two_shot(const ExchangeCtx& ctx, int dtype, const PeerPtrs& bufs,
                                      void* out, long n, float scale, cudaStream_t stream);

// The same sum through NVSwitch: `mc` is the multicast address of the symmetric buffers (a
// multiple of 16 bytes long, at least `nbytes`), `mine` this rank's own buffer.  In-switch
// reduction (`multimem.ld_reduce`) of one slice per rank, result broadcast with `multimem.st`.
cudaError_t launch_allreduce_multimem(const ExchangeCtx& ctx, int dtype, void* mc, const void* mine,
                                      void* out, long nbytes, float scale, cudaStream_t stream);

// All-gather of equal slices (`bytes_per_rank` a multiple of 16) through symmetric buffers of
// at least world * bytes_per_rank bytes: out = [slice of rank 0, slice of rank 1, ...].
cudaError_t launch_allgather(const ExchangeCtx& ctx, const void* src, const PeerPtrs& bufs,
                             void* out, long bytes_per_rank, cudaStream_t stream);

// Broadcast of `bytes` (a multiple of 16) from rank `root`: the owner stores its `src` into every
// peer's symmetric buffer once; every rank copies its buffer to `out`.  `src` is read on the
// root only.  Call launch_begin_reduce_epoch right before.
cudaError_t launch_broadcast(const ExchangeCtx& ctx, const void* src, const PeerPtrs& bufs, void* out,
                             long bytes, int root, cudaStream_t stream);

// Sum over ranks of the symmetric buffers (n elements; dtype 0 bf16, 1 f16, 2 f32), formed by
// rank `root` alone into its `out`; other ranks' `out` is not written.  Call
// launch_begin_reduce_epoch right before.
cudaError_t launch_reduce_to_root(const ExchangeCtx& ctx, int dtype, const PeerPtrs& bufs, void* out,
                                  long n, int root, cudaStream_t stream);

// Rank-ordered capacity grants from one exchange of request counts and capacities.
// lec: int32 [world * n_expert] requests of this rank; cap: int32 [n_expert] capacities of this
// rank's experts; cnt: symmetric int32 buffers of 2 * world * (world + 1) * n_expert entries.
// new_lec[g]: what this rank may send to global expert g; new_gec[w * n_expert + e]: what rank
// w may send to local expert e.  Call launch_begin_epoch right before.
cudaError_t launch_capacity_grant(const ExchangeCtx& ctx, const int* lec, const int* cap,
                                  const PeerPtrs& cnt, int n_expert, int64_t* new_lec,
                                  int64_t* new_gec, cudaStream_t stream);

// Exchange and plan of one SWIPE round.  want: int32 [world] tokens this rank routes to every
// worker; cap: int64 [1] capacity this rank has left; tab: symmetric int64 buffers of
// 2 * world * (world + 1) entries.  quota: int32 [world] tokens this rank may send to every
// worker after balancing; cap_left: int64 [1].  Call launch_begin_epoch right before.
cudaError_t launch_swipe_exchange(const ExchangeCtx& ctx, const int* want, const int64_t* cap,
                                  const PeerPtrs& tab, int* quota, int64_t* cap_left,
                                  cudaStream_t stream);

// Waits (bounded) for all peers' current-epoch flags on `channel` without touching any data.
cudaError_t launch_wait_arrival(const ExchangeCtx& ctx, int channel, cudaStream_t stream);

// Test hook: waits on `channel` for flags that nothing sets, with the given limit; the
// kernel returns and leaves kStatusPeerTimeout in the status word.
cudaError_t launch_wait_only(const ExchangeCtx& ctx, int channel, cudaStream_t stream);

}  // namespace fmoe
