// C++ CPU implementations of the native ops: the execution path for CPU tensors once the
// extension is built, and an oracle for the sm_100a kernels that is independent of the
// PyTorch restatement in ops/torch_impl.py.
#pragma once
#include <torch/extension.h>

#include <vector>

namespace fmoe {
namespace cpu {

// (counts int32 [tot], rank int32 [n_slots]); rank = -1 for dropped slots.
std::vector<torch::Tensor> route(torch::Tensor idx, int64_t tot);

// Rank-ordered grant; `capacity` (int32 [n_expert]) is decremented by the proposals.
torch::Tensor limit_by_capacity(torch::Tensor expert_count, torch::Tensor capacity,
                                int64_t n_expert, int64_t n_worker);

// Keep the first cap[g] slots of expert g; `cap` (int32) is decremented by the requests.
torch::Tensor prune_gate_by_capacity(torch::Tensor idx, torch::Tensor cap, int64_t n_expert,
                                     int64_t n_worker);

torch::Tensor linear_forward(torch::Tensor inp, torch::Tensor expert_count, torch::Tensor weight,
                             c10::optional<torch::Tensor> bias);
std::vector<torch::Tensor> linear_backward(torch::Tensor grad_out, torch::Tensor inp,
                                           torch::Tensor expert_count, torch::Tensor weight,
                                           c10::optional<torch::Tensor> bias);

// SWIPE plan: want[i][j] tokens rank i sends to worker j, cap[j] room of worker j.
// Returns (accepted [n, n] int64, cap_left [n] int64).
std::vector<torch::Tensor> swipe_plan(torch::Tensor want, torch::Tensor cap);

// Per-step split sizes and buffer layouts of the FasterMoE group-wise exchange (see the .cpp).
std::vector<torch::Tensor> smart_schedule_plan(torch::Tensor lec, torch::Tensor gec,
                                               torch::Tensor stored, int64_t num_expert,
                                               int64_t world_size, int64_t me, int64_t group_size);

}  // namespace cpu
}  // namespace fmoe
