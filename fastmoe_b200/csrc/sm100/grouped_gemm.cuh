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
  int num_sms = 148;
  cudaStream_t stream = nullptr;
};

// Returns cudaSuccess or the launch error; shape requirements: k % 64 == 0 (row modes),
// n % 32 == 0, m % 8 == 0 (wgrad), num_groups <= 1024, 16-byte aligned base pointers.
cudaError_t launch_grouped_gemm(const GroupedGemmArgs& args);

bool grouped_gemm_supported(int mode, int m, int n, int k, int num_groups);

}  // namespace fmoe
