// Routing, row movement, gating and balancing kernels (SIMT; bandwidth or latency bound).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fmoe {

// counts[tot] (int32), rank[n_slots] (int32, -1 for dropped slots), optional offs[tot + 1]
// (exclusive prefix of counts) and optional pos[n_slots] (slot ids sorted by expert, then by
// rank: pos[offs[e] + rank[s]] = s; entries past offs[tot] are not written).  Deterministic:
// slots of one expert are ranked by slot id.
// `part` (optional): int32 scratch of route_blocks(n_slots) * tot entries; with it, more than
// 32 K slots are ranked by several CTAs in two launches instead of by one CTA.
int route_blocks(int n_slots);
cudaError_t launch_route(const int64_t* idx, int n_slots, int tot, int* counts, int* rank,
                         int* offs, int* pos, int* part, cudaStream_t stream);

// new_idx[s] = (idx[s] >= 0 && rank[s] < cap[idx[s]]) ? idx[s] : -1
cudaError_t launch_prune(const int64_t* idx, const int* rank, const int* cap, int n_slots, int tot,
                         int64_t* new_idx, cudaStream_t stream);

// SWIPE reassignment of one choice column (idx: global expert ids; rank: slot rank of every
// token inside its worker; count / quota: int32 [n_worker] tokens routed to / accepted by every
// worker).  `mark` writes key 0 for tokens beyond their worker's quota and -1 otherwise; after
// ranking the moved tokens (mrank), `assign` writes the balanced ids.
cudaError_t launch_swipe_mark(const int64_t* idx, const int* rank, const int* quota, int n,
                              int n_expert, int n_worker, int64_t* key, cudaStream_t stream);
cudaError_t launch_swipe_assign(const int64_t* idx, const int64_t* key, const int* mrank,
                                const int* count, const int* quota, int n, int n_expert,
                                int n_worker, int bias, int64_t* out, cudaStream_t stream);

// Rank-ordered capacity grant; ec/eca are [n_worker, n_expert] int64, cap[n_expert] int32 (in/out).
cudaError_t launch_limit_by_capacity(const int64_t* ec, int* cap, int64_t* eca, int n_expert,
                                     int n_worker, cudaStream_t stream);

// pos[base_excl[idx[s]] + rank[s]] = s   (the reference's `pos` array)
cudaError_t launch_fill_pos(const int64_t* idx, const int* rank, const int* cum_incl, int n_slots,
                            int tot, int64_t* pos, cudaStream_t stream);

// dst[base[idx[s]] + rank[s], :] = scale[s] * src[s / k, :]   (16-bit element types)
// `row_slot` (optional) receives the slot id of every written row.
cudaError_t launch_scatter_rows(int dtype, const void* src, const int64_t* idx, const int* rank,
                                const int* base, const void* scale, int n_slots, int k, int d,
                                void* dst, int* row_slot, cudaStream_t stream);

// out[t, :] = sum_j w[t, j] * rows[base[idx[t, j]] + rank[t, j], :]   (w = 1 when null)
cudaError_t launch_gather_combine(int dtype, const void* rows, const int64_t* idx, const int* rank,
                                  const int* base, const void* weight, int n_tokens, int k, int d,
                                  void* out, cudaStream_t stream);

// Backward of the weighted combine:  dscore[t, j] = <dout[t], rows[dest(t, j)]>  and
// drows[dest(t, j), :] = w[t, j] * dout[t, :].
cudaError_t launch_combine_bwd(int dtype, const void* dout, const void* rows, const int64_t* idx,
                               const int* rank, const int* base, const void* weight, int n_tokens,
                               int k, int d, void* drows, void* dscore, cudaStream_t stream);

// out[g, :] += column sums of x[offs[g] : offs[g + 1], :]  (fp32 accumulation buffer, pre-zeroed)
cudaError_t launch_colsum(int dtype, const void* x, const int* offs, int num_groups, long rows_cap,
                          int n, float* out, cudaStream_t stream);

// Top-k of each logits row (descending) with softmax over the selected values.
// logit_dtype: 0 bf16, 1 f16, 2 f32; prob has the dtype of the logits.
cudaError_t launch_gate_topk_softmax(int logit_dtype, const void* logits, int n_rows, int n_experts,
                                     int k, int64_t* idx, void* prob, cudaStream_t stream);
cudaError_t launch_gate_topk_softmax_bwd(int logit_dtype, const void* dprob, const int64_t* idx,
                                         const void* prob, int n_rows, int n_experts, int k,
                                         void* dlogits, cudaStream_t stream);

// Fused gate: logits = x W^T + b (tot <= 64 experts, 16-bit types), top-k ids (descending) and
// softmax over the selected logits; one pass over x.
bool gate_fused_supported(int tot, int d, int k);
cudaError_t launch_gate_linear_topk(int dtype, const void* x, const void* w, const void* bias,
                                    int n_rows, int d, int tot, int k, void* logits, int64_t* idx,
                                    void* prob, cudaStream_t stream);
// Backward of the fused gate.  dl_scratch: fp32 [n_rows, tot]; dx (optional) [n_rows, d];
// dw fp32 [tot, d] and db fp32 [tot] (optional) must be zero on entry (accumulated with
// atomics).  The weight gradient kernel covers tot <= 16: pass dw = nullptr above that and
// form dW = dl^T x from dl_scratch with a library GEMM.
cudaError_t launch_gate_bwd(int dtype, const void* dprob, const int64_t* idx, const void* prob,
                            const void* dlogits_in, const void* x, const void* w, int n_rows, int d,
                            int tot, int k, float* dl_scratch, void* dx, float* dw, float* db,
                            cudaStream_t stream);

// Reference-precision grouped GEMM for fp32 / fp64 and for shapes the tensor-core kernel
// does not take (elem: 0 bf16, 1 f16, 2 f32, 3 f64).  Same modes as the tcgen05 kernel.
cudaError_t launch_simt_grouped_gemm(int mode, int elem, int num_groups, long rows_cap, int m, int n,
                                     int k, const void* a, const void* b, const int* offs,
                                     const void* bias, void* out, cudaStream_t stream);

}  // namespace fmoe
