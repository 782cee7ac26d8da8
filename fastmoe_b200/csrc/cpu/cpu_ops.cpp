#include "cpu_ops.h"

#include <algorithm>

namespace fmoe {
namespace cpu {

std::vector<torch::Tensor> route(torch::Tensor idx, int64_t tot) {
  TORCH_CHECK(!idx.is_cuda() && idx.scalar_type() == torch::kLong, "cpu_route: int64 CPU tensor");
  auto flat = idx.contiguous().view({-1});
  const int64_t n = flat.numel();
  auto counts = torch::zeros({tot}, torch::kInt32);
  auto rank = torch::empty({n}, torch::kInt32);
  const int64_t* in = flat.data_ptr<int64_t>();
  int* c = counts.data_ptr<int>();
  int* r = rank.data_ptr<int>();
  for (int64_t s = 0; s < n; ++s) {
    const int64_t e = in[s];
    r[s] = (e >= 0 && e < tot) ? c[e]++ : -1;
  }
  return {counts, rank};
}

torch::Tensor limit_by_capacity(torch::Tensor expert_count, torch::Tensor capacity,
                                int64_t n_expert, int64_t n_worker) {
  auto ec = expert_count.contiguous();
  auto out = torch::empty_like(ec);
  const int64_t* in = ec.data_ptr<int64_t>();
  int64_t* o = out.data_ptr<int64_t>();
  int* cap = capacity.data_ptr<int>();
  for (int64_t e = 0; e < n_expert; ++e) {
    int64_t left = cap[e];
    for (int64_t w = 0; w < n_worker; ++w) {
      const int64_t want = in[w * n_expert + e];
      o[w * n_expert + e] = std::min<int64_t>(want, std::max<int64_t>(left, 0));
      left -= want;
    }
    cap[e] = static_cast<int>(left);
  }
  return out;
}

torch::Tensor prune_gate_by_capacity(torch::Tensor idx, torch::Tensor cap, int64_t n_expert,
                                     int64_t n_worker) {
  auto flat = idx.contiguous();
  auto out = torch::empty_like(flat);
  const int64_t tot = n_expert * n_worker;
  const int64_t* in = flat.data_ptr<int64_t>();
  int64_t* o = out.data_ptr<int64_t>();
  int* c = cap.data_ptr<int>();
  for (int64_t s = 0; s < flat.numel(); ++s) {
    const int64_t e = in[s];
    if (e < 0 || e >= tot) {
      o[s] = -1;
      continue;
    }
    o[s] = (c[e] > 0) ? e : -1;
    --c[e];
  }
  return out;
}

torch::Tensor linear_forward(torch::Tensor inp, torch::Tensor expert_count, torch::Tensor weight,
                             c10::optional<torch::Tensor> bias) {
  auto out = torch::empty({inp.size(0), weight.size(1)}, inp.options());
  auto cnt = expert_count.to(torch::kLong).contiguous();
  const int64_t* c = cnt.data_ptr<int64_t>();
  int64_t base = 0;
  for (int64_t e = 0; e < cnt.numel(); ++e) {
    if (c[e] > 0) {
      auto y = at::matmul(inp.narrow(0, base, c[e]), weight[e].t());
      if (bias.has_value() && bias->defined()) y = y + (*bias)[e];
      out.narrow(0, base, c[e]).copy_(y);
    }
    base += c[e];
  }
  return out;
}

std::vector<torch::Tensor> linear_backward(torch::Tensor grad_out, torch::Tensor inp,
                                           torch::Tensor expert_count, torch::Tensor weight,
                                           c10::optional<torch::Tensor> bias) {
  auto grad_in = torch::empty({inp.size(0), weight.size(2)}, grad_out.options());
  auto grad_w = torch::zeros_like(weight);
  const bool has_bias = bias.has_value() && bias->defined();
  auto grad_b = has_bias ? torch::zeros_like(*bias) : torch::Tensor();
  auto cnt = expert_count.to(torch::kLong).contiguous();
  const int64_t* c = cnt.data_ptr<int64_t>();
  int64_t base = 0;
  for (int64_t e = 0; e < cnt.numel(); ++e) {
    if (c[e] > 0) {
      auto go = grad_out.narrow(0, base, c[e]);
      grad_in.narrow(0, base, c[e]).copy_(at::matmul(go, weight[e]));
      grad_w[e].copy_(at::matmul(go.t(), inp.narrow(0, base, c[e])));
      if (has_bias) grad_b[e].copy_(go.sum(0));
    }
    base += c[e];
  }
  return {grad_in, grad_w, grad_b};
}

std::vector<torch::Tensor> swipe_plan(torch::Tensor want, torch::Tensor cap) {
  auto w = want.to(torch::kLong).contiguous();
  const int64_t n = w.size(0);
  auto accepted = torch::zeros({n, n}, torch::kLong);
  auto left = cap.to(torch::kLong).clone().contiguous();
  const int64_t* wp = w.data_ptr<int64_t>();
  int64_t* ap = accepted.data_ptr<int64_t>();
  int64_t* lp = left.data_ptr<int64_t>();
  std::vector<int64_t> dropped(n, 0);
  for (int64_t j = 0; j < n; ++j) {
    for (int64_t i = 0; i < n; ++i) {
      const int64_t take = std::min(wp[i * n + j], lp[j]);
      ap[i * n + j] = take;
      lp[j] -= take;
      dropped[i] += wp[i * n + j] - take;
    }
  }
  int64_t j = 0;
  for (int64_t i = 0; i < n; ++i) {
    while (dropped[i] > 0 && j < n) {
      const int64_t take = std::min(dropped[i], lp[j]);
      ap[i * n + j] += take;
      lp[j] -= take;
      dropped[i] -= take;
      if (lp[j] == 0) ++j;
    }
  }
  return {accepted, left};
}

// Chunk plan of the group-wise pipelined exchange (the host-side bookkeeping the reference
// does in `computePtrs` / the step loops of cuda/fastermoe/smart_schedule.h:48-80,105-261).
// Ranks form groups of `group_size`; in step s rank `me` sends to group (mine + s) and receives
// from group (mine - s).  Shadowed experts (`stored`) take no part in the exchange.
//   send_sizes, recv_sizes : [steps, world]  rows to / from every rank in that step
//   send_experts, send_offsets : global expert ids whose row segments make up the send buffer
//                                of step s, in order: send_experts[send_offsets[s] : send_offsets[s+1]]
//   recv_cursor, recv_count : [steps, group_size, num_expert]  where the rows of (source rank of
//                             the step's group, local expert) start in the received buffer and
//                             how many there are (cursor -1 for shadowed experts)
std::vector<torch::Tensor> smart_schedule_plan(torch::Tensor lec, torch::Tensor gec,
                                               torch::Tensor stored, int64_t num_expert,
                                               int64_t world_size, int64_t me, int64_t group_size) {
  auto l = lec.to(torch::kLong).contiguous().cpu();
  auto g = gec.to(torch::kLong).contiguous().cpu();
  auto st = stored.to(torch::kBool).contiguous().cpu();
  const int64_t tot = num_expert * world_size;
  TORCH_CHECK(l.numel() == tot && g.numel() == tot && st.numel() == tot, "plan: count shapes");
  TORCH_CHECK(group_size >= 1 && world_size % group_size == 0, "plan: group size");
  const int64_t steps = world_size / group_size;
  const int64_t my_group = me / group_size;
  const int64_t* lp = l.data_ptr<int64_t>();
  const int64_t* gp = g.data_ptr<int64_t>();
  const bool* sp = st.data_ptr<bool>();
  auto send_sizes = torch::zeros({steps, world_size}, torch::kLong);
  auto recv_sizes = torch::zeros({steps, world_size}, torch::kLong);
  auto recv_cursor = torch::full({steps, group_size, num_expert}, -1, torch::kLong);
  auto recv_count = torch::zeros({steps, group_size, num_expert}, torch::kLong);
  auto send_offsets = torch::zeros({steps + 1}, torch::kLong);
  std::vector<int64_t> experts;
  int64_t* ss = send_sizes.data_ptr<int64_t>();
  int64_t* rs = recv_sizes.data_ptr<int64_t>();
  int64_t* rc = recv_cursor.data_ptr<int64_t>();
  int64_t* rn = recv_count.data_ptr<int64_t>();
  int64_t* so = send_offsets.data_ptr<int64_t>();
  for (int64_t s = 0; s < steps; ++s) {
    const int64_t to_group = (my_group + s) % steps;
    const int64_t from_group = ((my_group - s) % steps + steps) % steps;
    for (int64_t p = to_group * group_size; p < (to_group + 1) * group_size; ++p) {
      for (int64_t e = 0; e < num_expert; ++e) {
        const int64_t id = p * num_expert + e;
        if (!sp[id] && lp[id] > 0) {
          experts.push_back(id);
          ss[s * world_size + p] += lp[id];
        }
      }
    }
    so[s + 1] = static_cast<int64_t>(experts.size());
    int64_t cursor = 0;
    for (int64_t i = 0; i < group_size; ++i) {
      const int64_t src = from_group * group_size + i;
      for (int64_t e = 0; e < num_expert; ++e) {
        if (sp[me * num_expert + e]) continue;
        const int64_t n = gp[src * num_expert + e];
        rs[s * world_size + src] += n;
        rc[(s * group_size + i) * num_expert + e] = cursor;
        rn[(s * group_size + i) * num_expert + e] = n;
        cursor += n;
      }
    }
  }
  auto send_experts = torch::empty({static_cast<int64_t>(experts.size())}, torch::kLong);
  std::copy(experts.begin(), experts.end(), send_experts.data_ptr<int64_t>());
  return {send_sizes, recv_sizes, send_experts, send_offsets, recv_cursor, recv_count};
}

}  // namespace cpu
}  // namespace fmoe
