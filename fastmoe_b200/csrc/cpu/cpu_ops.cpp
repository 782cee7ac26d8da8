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

}  // namespace cpu
}  // namespace fmoe
