// Host-visible interface of the tcgen05 grouped GEMM (no torch types here, so the kernel
// translation units compile without the torch headers).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "p2p.cuh"

namespace fmoe {

enum GemmMode : int {
  // C[rows_e, N] = A[rows_e, K] * B_e[N, K]^T       (forward of a grouped linear)
  kRowsNT = 0,
  // C[rows_e, N] = A[rows_e, K] * B_e[K, N]         (input gradient: B is the weight [E, K, N])
  kRowsNN = 1,
  // C_e[M, N] = P[rows_e, M]^T * Q[rows_e, N]       (weight gradient; the reduction runs over rows)
  kWgrad = 2,
};

enum ActKind : int { kActNone = 0, kActRelu = 1, kActGelu = 2, kActGeluTanh = 3 };

enum EpiKind : int {
  kEpiBiasAct = 0,   // out = act(acc + bias); optionally pre_out = acc + bias
  kEpiDAct = 1,      // out = acc * act'(aux)          (aux = saved pre-activation)
};

enum DType : int { kBF16 = 0, kF16 = 1 };

// Row dispatch fused into a row-mode GEMM launch (optional).  Warps 2 and 3 of every CTA,
// which the GEMM roles leave idle, walk this rank's slots in destination order and copy every
// token row (optionally scaled) through registers into the owning peer's receive buffer; one
// flag word per (128-row block of the receiver, source rank) is published when all rows of the
// block have left.  The TMA producer gates every tile on the flags of its row block
// (`GateArgs`), so the transfer overlaps the math tile by tile and no SM is set aside for it.
struct SendArgs {
  int enabled = 0;
  const void* x = nullptr;        // [n_tokens, d] rows to send (row s / k serves slot s)
  const int* pos = nullptr;       // [n_slots] slot ids sorted by (global expert, rank in expert)
  const int* my_offs = nullptr;   // [tot + 1] exclusive prefix of this rank's per-expert slot counts
  const int* dst_base = nullptr;  // [tot] first destination row of my rows, per global expert
  const int* seg_base = nullptr;  // [tot] first row of the expert's whole segment on its owner
  const int* blk_base = nullptr;  // [tot] index of the expert's first 128-row block on its owner
  const int* item_prefix = nullptr;  // [tot + 1] exclusive prefix of the 128-row blocks my rows touch,
                                     // per (expert, peer) in send order
  int* item_count = nullptr;      // local, zero between launches: rows sent so far, per block in send order
  const void* scale = nullptr;    // optional [n_slots]: row s is multiplied by scale[s]
  PeerPtrs rows = {};             // every peer's receive buffer [capacity, d]
  PeerPtrs meta = {};             // every peer's int64 [capacity] (source rank << 32 | slot); entries may be null
  PeerPtrs flags = {};            // every peer's int32 [blocks][kMaxPeers] arrival flags
  const int* epoch = nullptr;     // value to publish
  int n_expert = 0;
  int world = 1;
  int me = 0;
  int k = 1;
  int d = 0;
  int capacity = 0;
};

// Arrival gating of a row-mode GEMM whose A operand is being filled by the peers' sender warps.
struct GateArgs {
  const int* flags = nullptr;     // local int32 [blocks][kMaxPeers]; null = not gated
  const int* seg_off = nullptr;   // [num_groups][world + 1] row where the rows of the j-th source begin
  // Optional: the (group, 128-row block) pairs of the problem in the order the tiles are to be
  // walked, (group << 20) | block — every pair exactly once.  Null = groups in order.
  const int* blk_order = nullptr;
  const int* epoch = nullptr;
  int world = 1;
  int me = 0;
  unsigned long long timeout_ns = 0;
};

struct GroupedGemmArgs {
  int mode = kRowsNT;
  int dtype = kBF16;
  int num_groups = 0;
  // Row modes: A is [rows_cap, k]; output [rows_cap, n].  Wgrad: P is [rows_cap, m], Q is
  // [rows_cap, n]; output [num_groups, m, n].
  long rows_cap = 0;
  int m = 0;
  int n = 0;
  int k = 0;
  const void* a = nullptr;       // A (row modes) or P (wgrad)
  const void* b = nullptr;       // weights (row modes) or Q (wgrad)
  const int* offs = nullptr;     // device, [num_groups + 1] exclusive row offsets
  void* out = nullptr;
  void* pre_out = nullptr;       // optional, row modes only
  const void* bias = nullptr;    // optional [num_groups, n]
  const void* aux = nullptr;     // kEpiDAct: [rows_cap, n]
  int act = kActNone;
  int epi = kEpiBiasAct;
  int accumulate = 0;            // wgrad: out += result
  int out_fp32 = 0;              // wgrad: output buffer is fp32
  // wgrad, optional: [num_groups, m] per-group column sums of P in the operands' element type
  // (the bias gradient of the grouped linear whose weight gradient this is); produced by the
  // epilogue warps while they wait for the main loop.  `accumulate` applies to it too.
  void* psum = nullptr;
  int* status = nullptr;         // device status word (0 = ok)
  // Row modes, optional: instead of storing row r of the result into `out`, store it into
  // row (meta[r] & 0xffffffff) of the buffer push_dst.p[meta[r] >> 32] — a peer's slot-indexed
  // return buffer — and, once the whole grid is done, publish `*push_epoch` on the return
  // channel of every peer's signal buffer.  This fuses the second expert GEMM (or the last
  // input-gradient GEMM) with the combine direction of the exchange.
  const int64_t* push_meta = nullptr;
  PeerPtrs push_dst = {};
  PeerPtrs push_flags = {};
  const int* push_epoch = nullptr;
  int* push_counter = nullptr;   // zero-initialised word in local memory (CTA completion count)
  int push_me = 0;
  int push_world = 0;
  long push_slots = 0;           // rows of every return buffer: rows whose meta names a slot beyond it are skipped
  SendArgs send;
  GateArgs gate;
  // Optional trace, ten int64 per CTA, zeroed by the caller.  %globaltimer stamps (ns): kernel
  // entry, first tile's rows available to the TMA producer, sender warp 2 done, kernel exit;
  // for the first unit of sender warp 2: slot ids loaded, stores issued, fence passed, counted.
  // Then two counters: ns the producer waited for rows over all tiles, tiles that waited > 1 us.
  unsigned long long* trace = nullptr;
  int num_sms = 148;
  cudaStream_t stream = nullptr;
};

// Returns cudaSuccess or the launch error; shape requirements: k % 64 == 0 (row modes),
// n % 32 == 0, m % 8 == 0 (wgrad), num_groups <= 256, 16-byte aligned base pointers.
cudaError_t launch_grouped_gemm(const GroupedGemmArgs& args);

bool grouped_gemm_supported(int mode, int m, int n, int k, int num_groups);

}  // namespace fmoe
