// Python bindings of the native extension.
//
// The reference exposes 13 functions from one pybind module (cuda/fmoe_cuda.cpp:104-125).
// Their counterparts are bound here under the same names where the calling convention could
// be kept (expert_count, assign_pos, limit_by_capacity, prune_gate_by_capacity); the rest of
// the surface is the device-count-driven API the fused layer uses (route, grouped_gemm,
// scatter_rows, gather_combine, combine_bwd, colsum, gate_topk_softmax, ...).  Errors raise
// Python exceptions; nothing calls exit().
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <atomic>
#include <map>
#include <mutex>

#include "cpu/cpu_ops.h"
#include "sm100/grouped_gemm.cuh"
#include "sm100/routing.cuh"
#include "sm100/p2p.cuh"

namespace {

#define FMOE_CUDA_CHECK(expr)                                                       \
  do {                                                                              \
    cudaError_t _e = (expr);                                                        \
    TORCH_CHECK(_e == cudaSuccess, "fastmoe_b200: ", #expr, " failed: ",            \
                cudaGetErrorString(_e));                                            \
  } while (0)

// Number of kernels of this library launched by this process (benchmarks report it).
std::atomic<int64_t> g_launches{0};

}  // namespace

// Called by the exchange bindings (other translation unit) for every kernel they launch.
void fmoe_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

namespace {

cudaStream_t cur_stream() {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return at::cuda::getCurrentCUDAStream().stream();
}

int dtype16(const torch::Tensor& t) {
  if (t.scalar_type() == torch::kBFloat16) return fmoe::kBF16;
  TORCH_CHECK(t.scalar_type() == torch::kHalf, "expected a bf16 or fp16 tensor");
  return fmoe::kF16;
}

int elem_code(const torch::Tensor& t) {
  switch (t.scalar_type()) {
    case torch::kBFloat16: return 0;
    case torch::kHalf: return 1;
    case torch::kFloat: return 2;
    case torch::kDouble: return 3;
    default: TORCH_CHECK(false, "unsupported dtype for the grouped GEMM"); return -1;
  }
}

void check_cuda_contig(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

// One int32 status word per device; kernels write a non-zero code when a bounded wait ran out.
std::mutex g_status_mu;
std::map<int, torch::Tensor> g_status;

torch::Tensor status_tensor(int device) {
  std::lock_guard<std::mutex> lock(g_status_mu);
  auto it = g_status.find(device);
  if (it != g_status.end()) return it->second;
  auto t = torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
  g_status[device] = t;
  return t;
}

int num_sms(int device) {
  static std::map<int, int> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(device);
  if (it != cache.end()) return it->second;
  int n = 148;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
  cache[device] = n;
  return n;
}

// ------------------------------------------------------------------------------ routing
std::vector<torch::Tensor> route(torch::Tensor idx, int64_t tot, bool want_offs, bool want_pos = false) {
  check_cuda_contig(idx, "idx");
  TORCH_CHECK(idx.scalar_type() == torch::kLong, "idx must be int64");
  c10::cuda::CUDAGuard guard(idx.device());
  const int n_slots = static_cast<int>(idx.numel());
  auto opt = torch::dtype(torch::kInt32).device(idx.device());
  auto counts = torch::empty({tot}, opt);
  auto rank = torch::empty({n_slots}, opt);
  torch::Tensor offs;
  int* offs_ptr = nullptr;
  if (want_offs || want_pos) {
    offs = torch::empty({tot + 1}, opt);
    offs_ptr = offs.data_ptr<int>();
  }
  torch::Tensor pos;
  int* pos_ptr = nullptr;
  if (want_pos) {
    pos = torch::empty({n_slots > 0 ? n_slots : 1}, opt);
    pos_ptr = pos.data_ptr<int>();
  }
  torch::Tensor part;
  int* part_ptr = nullptr;
  const int nb = fmoe::route_blocks(n_slots);
  if (nb > 1) {
    part = torch::empty({static_cast<int64_t>(nb) * tot}, opt);
    part_ptr = part.data_ptr<int>();
    g_launches.fetch_add(1, std::memory_order_relaxed);  // the second launch of the pair
  }
  FMOE_CUDA_CHECK(fmoe::launch_route(idx.data_ptr<int64_t>(), n_slots, static_cast<int>(tot),
                                     counts.data_ptr<int>(), rank.data_ptr<int>(), offs_ptr,
                                     pos_ptr, part_ptr, cur_stream()));
  if (want_pos) return {counts, rank, offs, pos};
  if (want_offs) return {counts, rank, offs};
  return {counts, rank};
}

void expert_count(torch::Tensor idx, torch::Tensor counts_inout) {
  auto res = route(idx.contiguous().view({-1}), counts_inout.numel(), false);
  counts_inout.add_(res[0]);
}

void assign_pos(torch::Tensor cum_count, torch::Tensor idx, torch::Tensor pos) {
  check_cuda_contig(cum_count, "cum_count");
  check_cuda_contig(pos, "pos");
  auto flat = idx.contiguous().view({-1});
  const int tot = static_cast<int>(cum_count.numel());
  auto res = route(flat, tot, false);
  c10::cuda::CUDAGuard guard(idx.device());
  FMOE_CUDA_CHECK(fmoe::launch_fill_pos(flat.data_ptr<int64_t>(), res[1].data_ptr<int>(),
                                        cum_count.data_ptr<int>(), static_cast<int>(flat.numel()),
                                        tot, pos.data_ptr<int64_t>(), cur_stream()));
}

torch::Tensor limit_by_capacity(torch::Tensor ec, torch::Tensor cap, int64_t n_expert,
                                int64_t n_worker) {
  check_cuda_contig(ec, "expert_count");
  check_cuda_contig(cap, "capacity");
  TORCH_CHECK(ec.scalar_type() == torch::kLong && cap.scalar_type() == torch::kInt,
              "limit_by_capacity: expert_count int64, capacity int32");
  c10::cuda::CUDAGuard guard(ec.device());
  auto eca = torch::empty_like(ec);
  FMOE_CUDA_CHECK(fmoe::launch_limit_by_capacity(ec.data_ptr<int64_t>(), cap.data_ptr<int>(),
                                                 eca.data_ptr<int64_t>(), static_cast<int>(n_expert),
                                                 static_cast<int>(n_worker), cur_stream()));
  return eca;
}

torch::Tensor prune_gate_by_capacity(torch::Tensor idx, torch::Tensor cap, int64_t n_expert,
                                     int64_t n_worker) {
  check_cuda_contig(idx, "gate_idx");
  check_cuda_contig(cap, "expert_count");
  TORCH_CHECK(cap.scalar_type() == torch::kInt, "prune_gate_by_capacity: capacity must be int32");
  const int tot = static_cast<int>(n_expert * n_worker);
  auto flat = idx.view({-1});
  auto res = route(flat, tot, false);
  c10::cuda::CUDAGuard guard(idx.device());
  auto out = torch::empty_like(idx);
  FMOE_CUDA_CHECK(fmoe::launch_prune(flat.data_ptr<int64_t>(), res[1].data_ptr<int>(),
                                     cap.data_ptr<int>(), static_cast<int>(flat.numel()), tot,
                                     out.data_ptr<int64_t>(), cur_stream()));
  cap.sub_(res[0]);
  return out;
}

// SWIPE on the device: balanced ids of one choice column from the quota the exchange kernel
// computed.  No count reaches the host.
torch::Tensor swipe_reassign(torch::Tensor idx, torch::Tensor quota, int64_t n_expert, int64_t bias) {
  check_cuda_contig(idx, "idx");
  check_cuda_contig(quota, "quota");
  TORCH_CHECK(idx.scalar_type() == torch::kLong && quota.scalar_type() == torch::kInt,
              "swipe_reassign: int64 ids, int32 quota");
  c10::cuda::CUDAGuard guard(idx.device());
  const int n = static_cast<int>(idx.numel());
  const int n_worker = static_cast<int>(quota.numel());
  auto worker = torch::div(idx, n_expert, "floor");
  auto r1 = route(worker.contiguous(), n_worker, false);          // counts per worker, slot ranks
  auto key = torch::empty_like(idx);
  FMOE_CUDA_CHECK(fmoe::launch_swipe_mark(idx.data_ptr<int64_t>(), r1[1].data_ptr<int>(),
                                          quota.data_ptr<int>(), n, static_cast<int>(n_expert),
                                          n_worker, key.data_ptr<int64_t>(), cur_stream()));
  auto r2 = route(key, 1, false);                                  // ordinal among the moved tokens
  auto out = torch::empty_like(idx);
  FMOE_CUDA_CHECK(fmoe::launch_swipe_assign(idx.data_ptr<int64_t>(), key.data_ptr<int64_t>(),
                                            r2[1].data_ptr<int>(), r1[0].data_ptr<int>(),
                                            quota.data_ptr<int>(), n, static_cast<int>(n_expert),
                                            n_worker, static_cast<int>(bias),
                                            out.data_ptr<int64_t>(), cur_stream()));
  return out;
}

// ------------------------------------------------------------------------------ grouped GEMM
// Generic entry: see sm100/grouped_gemm.cuh for the meaning of mode / act / epi.
void grouped_gemm(int64_t mode, torch::Tensor a, torch::Tensor b, torch::Tensor offs,
                  torch::Tensor out, c10::optional<torch::Tensor> bias,
                  c10::optional<torch::Tensor> pre_out, c10::optional<torch::Tensor> aux,
                  int64_t act, int64_t epi, bool accumulate,
                  c10::optional<torch::Tensor> psum) {
  check_cuda_contig(a, "a");
  check_cuda_contig(b, "b");
  check_cuda_contig(offs, "offs");
  check_cuda_contig(out, "out");
  TORCH_CHECK(offs.scalar_type() == torch::kInt, "offs must be int32");
  c10::cuda::CUDAGuard guard(a.device());
  fmoe::GroupedGemmArgs g;
  g.mode = static_cast<int>(mode);
  g.dtype = dtype16(a);
  TORCH_CHECK(b.scalar_type() == a.scalar_type(), "operand dtypes differ");
  g.num_groups = static_cast<int>(offs.numel() - 1);
  g.rows_cap = a.size(0);
  if (mode == fmoe::kWgrad) {
    // a = P [rows, m], b = Q [rows, n], out [G, m, n]
    TORCH_CHECK(b.size(0) == a.size(0), "wgrad operands need the same number of rows");
    g.m = static_cast<int>(a.size(1));
    g.n = static_cast<int>(b.size(1));
    g.k = 0;
    TORCH_CHECK(out.numel() == static_cast<int64_t>(g.num_groups) * g.m * g.n, "wgrad out shape");
    g.out_fp32 = out.scalar_type() == torch::kFloat ? 1 : 0;
    TORCH_CHECK(g.out_fp32 || out.scalar_type() == a.scalar_type(), "wgrad out dtype");
  } else {
    g.k = static_cast<int>(a.size(1));
    if (mode == fmoe::kRowsNT) {
      TORCH_CHECK(b.dim() == 3 && b.size(2) == g.k, "weight must be [G, n, k]");
      g.n = static_cast<int>(b.size(1));
    } else {
      TORCH_CHECK(b.dim() == 3 && b.size(1) == g.k, "weight must be [G, k, n]");
      g.n = static_cast<int>(b.size(2));
    }
    TORCH_CHECK(b.size(0) == g.num_groups, "weight group count");
    TORCH_CHECK(out.size(0) == a.size(0) && out.size(1) == g.n, "out shape");
    TORCH_CHECK(out.scalar_type() == a.scalar_type(), "out dtype");
  }
  auto aligned32 = [](const torch::Tensor& t) {
    return reinterpret_cast<uintptr_t>(t.data_ptr()) % 32 == 0;
  };
  TORCH_CHECK(aligned32(a) && aligned32(b) && aligned32(out),
              "grouped_gemm: operands must be 32-byte aligned");
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.offs = offs.data_ptr<int>();
  g.out = out.data_ptr();
  if (bias.has_value() && bias->defined()) {
    check_cuda_contig(*bias, "bias");
    TORCH_CHECK(bias->scalar_type() == a.scalar_type(), "bias dtype");
    TORCH_CHECK(aligned32(*bias), "grouped_gemm: bias must be 32-byte aligned");
    g.bias = bias->data_ptr();
  }
  // The pre-activation (written as pre_out, read back as aux) is tile-blocked: one 128 x 256
  // block per output tile, (ceil(rows / 128) + groups) * ceil(n / 256) blocks at most.
  const int64_t pre_elems = mode == fmoe::kWgrad ? 0
      : ((a.size(0) + 127) / 128 + g.num_groups) * ((g.n + 255) / 256) * (128 * 256);
  if (pre_out.has_value() && pre_out->defined()) {
    check_cuda_contig(*pre_out, "pre_out");
    TORCH_CHECK(aligned32(*pre_out) && pre_out->numel() >= pre_elems &&
                    pre_out->scalar_type() == a.scalar_type(),
                "grouped_gemm: pre_out must be a 32-byte aligned tile-blocked buffer of ", pre_elems,
                " elements");
    g.pre_out = pre_out->data_ptr();
  }
  if (aux.has_value() && aux->defined()) {
    check_cuda_contig(*aux, "aux");
    TORCH_CHECK(aligned32(*aux) && aux->numel() >= pre_elems && aux->scalar_type() == a.scalar_type(),
                "grouped_gemm: aux must be a 32-byte aligned tile-blocked buffer of ", pre_elems,
                " elements");
    g.aux = aux->data_ptr();
  }
  if (psum.has_value() && psum->defined()) {
    TORCH_CHECK(mode == fmoe::kWgrad, "psum is an output of the weight-gradient mode");
    check_cuda_contig(*psum, "psum");
    TORCH_CHECK(psum->scalar_type() == a.scalar_type() &&
                    psum->numel() == static_cast<int64_t>(g.num_groups) * g.m,
                "psum must be [groups, m] in the operands' dtype");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(psum->data_ptr()) % 16 == 0, "psum must be 16-byte aligned");
    g.psum = psum->data_ptr();
  }
  g.act = static_cast<int>(act);
  g.epi = static_cast<int>(epi);
  g.accumulate = accumulate ? 1 : 0;
  g.status = status_tensor(a.device().index()).data_ptr<int>();
  g.num_sms = num_sms(a.device().index());
  g.stream = cur_stream();
  TORCH_CHECK(fmoe::grouped_gemm_supported(g.mode, g.m, g.n, g.k, g.num_groups),
              "grouped_gemm: shape not supported by the tcgen05 kernel (m=", g.m, " n=", g.n,
              " k=", g.k, " groups=", g.num_groups, ")");
  FMOE_CUDA_CHECK(fmoe::launch_grouped_gemm(g));
}

bool grouped_gemm_supported(int64_t mode, int64_t m, int64_t n, int64_t k, int64_t groups) {
  return fmoe::grouped_gemm_supported(static_cast<int>(mode), static_cast<int>(m),
                                      static_cast<int>(n), static_cast<int>(k),
                                      static_cast<int>(groups));
}

void simt_grouped_gemm(int64_t mode, torch::Tensor a, torch::Tensor b, torch::Tensor offs,
                       torch::Tensor out, c10::optional<torch::Tensor> bias) {
  check_cuda_contig(a, "a");
  check_cuda_contig(b, "b");
  check_cuda_contig(out, "out");
  c10::cuda::CUDAGuard guard(a.device());
  const int groups = static_cast<int>(offs.numel() - 1);
  int m = 0, n = 0, k = 0;
  if (mode == fmoe::kWgrad) {
    m = static_cast<int>(a.size(1));
    n = static_cast<int>(b.size(1));
  } else {
    k = static_cast<int>(a.size(1));
    n = static_cast<int>(mode == fmoe::kRowsNT ? b.size(1) : b.size(2));
  }
  const void* bias_ptr = nullptr;
  if (bias.has_value() && bias->defined()) bias_ptr = bias->data_ptr();
  FMOE_CUDA_CHECK(fmoe::launch_simt_grouped_gemm(static_cast<int>(mode), elem_code(a), groups,
                                                 a.size(0), m, n, k, a.data_ptr(), b.data_ptr(),
                                                 offs.data_ptr<int>(), bias_ptr, out.data_ptr(),
                                                 cur_stream()));
}

// ------------------------------------------------------------------------------ row movement
void scatter_rows(torch::Tensor src, torch::Tensor idx, torch::Tensor rank, torch::Tensor base,
                  c10::optional<torch::Tensor> scale, int64_t k, torch::Tensor dst,
                  c10::optional<torch::Tensor> row_slot) {
  check_cuda_contig(src, "src");
  check_cuda_contig(dst, "dst");
  c10::cuda::CUDAGuard guard(src.device());
  const void* sc = (scale.has_value() && scale->defined()) ? scale->data_ptr() : nullptr;
  int* rs = (row_slot.has_value() && row_slot->defined()) ? row_slot->data_ptr<int>() : nullptr;
  FMOE_CUDA_CHECK(fmoe::launch_scatter_rows(dtype16(src), src.data_ptr(), idx.data_ptr<int64_t>(),
                                            rank.data_ptr<int>(), base.data_ptr<int>(), sc,
                                            static_cast<int>(idx.numel()), static_cast<int>(k),
                                            static_cast<int>(src.size(1)), dst.data_ptr(), rs,
                                            cur_stream()));
}

void gather_combine(torch::Tensor rows, torch::Tensor idx, torch::Tensor rank, torch::Tensor base,
                    c10::optional<torch::Tensor> weight, int64_t k, torch::Tensor out) {
  check_cuda_contig(rows, "rows");
  check_cuda_contig(out, "out");
  c10::cuda::CUDAGuard guard(rows.device());
  const void* w = (weight.has_value() && weight->defined()) ? weight->data_ptr() : nullptr;
  FMOE_CUDA_CHECK(fmoe::launch_gather_combine(dtype16(rows), rows.data_ptr(),
                                              idx.data_ptr<int64_t>(), rank.data_ptr<int>(),
                                              base.data_ptr<int>(), w,
                                              static_cast<int>(out.size(0)), static_cast<int>(k),
                                              static_cast<int>(rows.size(1)), out.data_ptr(),
                                              cur_stream()));
}

void combine_bwd(torch::Tensor dout, torch::Tensor rows, torch::Tensor idx, torch::Tensor rank,
                 torch::Tensor base, torch::Tensor weight, int64_t k, torch::Tensor drows,
                 torch::Tensor dscore) {
  check_cuda_contig(dout, "dout");
  check_cuda_contig(rows, "rows");
  c10::cuda::CUDAGuard guard(dout.device());
  FMOE_CUDA_CHECK(fmoe::launch_combine_bwd(dtype16(dout), dout.data_ptr(), rows.data_ptr(),
                                           idx.data_ptr<int64_t>(), rank.data_ptr<int>(),
                                           base.data_ptr<int>(), weight.data_ptr(),
                                           static_cast<int>(dout.size(0)), static_cast<int>(k),
                                           static_cast<int>(dout.size(1)), drows.data_ptr(),
                                           dscore.data_ptr(), cur_stream()));
}

torch::Tensor colsum(torch::Tensor x, torch::Tensor offs) {
  check_cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int groups = static_cast<int>(offs.numel() - 1);
  auto out = torch::zeros({groups, x.size(1)}, torch::dtype(torch::kFloat).device(x.device()));
  FMOE_CUDA_CHECK(fmoe::launch_colsum(dtype16(x), x.data_ptr(), offs.data_ptr<int>(), groups,
                                      x.size(0), static_cast<int>(x.size(1)),
                                      out.data_ptr<float>(), cur_stream()));
  return out;
}

// ------------------------------------------------------------------------------ gate
int logit_code(const torch::Tensor& t) {
  if (t.scalar_type() == torch::kBFloat16) return 0;
  if (t.scalar_type() == torch::kHalf) return 1;
  TORCH_CHECK(t.scalar_type() == torch::kFloat, "gate logits must be bf16, fp16 or fp32");
  return 2;
}

std::vector<torch::Tensor> gate_topk_softmax(torch::Tensor logits, int64_t k) {
  check_cuda_contig(logits, "logits");
  c10::cuda::CUDAGuard guard(logits.device());
  const int rows = static_cast<int>(logits.size(0));
  const int ne = static_cast<int>(logits.size(1));
  auto idx = torch::empty({rows, k}, torch::dtype(torch::kLong).device(logits.device()));
  auto prob = torch::empty({rows, k}, logits.options());
  FMOE_CUDA_CHECK(fmoe::launch_gate_topk_softmax(logit_code(logits), logits.data_ptr(), rows, ne,
                                                 static_cast<int>(k), idx.data_ptr<int64_t>(),
                                                 prob.data_ptr(), cur_stream()));
  return {idx, prob};
}

torch::Tensor gate_topk_softmax_bwd(torch::Tensor dprob, torch::Tensor idx, torch::Tensor prob,
                                    int64_t n_experts) {
  check_cuda_contig(dprob, "dprob");
  c10::cuda::CUDAGuard guard(dprob.device());
  const int rows = static_cast<int>(dprob.size(0));
  const int k = static_cast<int>(dprob.size(1));
  auto dlogits = torch::empty({rows, n_experts}, dprob.options());
  FMOE_CUDA_CHECK(fmoe::launch_gate_topk_softmax_bwd(
      logit_code(dprob), dprob.data_ptr(), idx.data_ptr<int64_t>(), prob.data_ptr(), rows,
      static_cast<int>(n_experts), k, dlogits.data_ptr(), cur_stream()));
  return dlogits;
}

bool gate_fused_supported(int64_t tot, int64_t d, int64_t k) {
  return fmoe::gate_fused_supported(static_cast<int>(tot), static_cast<int>(d), static_cast<int>(k));
}

// logits [B, tot], idx [B, k] and prob [B, k] of a linear gate in one pass over x.
std::vector<torch::Tensor> gate_linear_topk(torch::Tensor x, torch::Tensor w,
                                            c10::optional<torch::Tensor> bias, int64_t k) {
  check_cuda_contig(x, "x");
  check_cuda_contig(w, "w");
  TORCH_CHECK(x.scalar_type() == w.scalar_type(), "gate input and weight dtypes differ");
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = static_cast<int>(x.size(0));
  const int d = static_cast<int>(x.size(1));
  const int tot = static_cast<int>(w.size(0));
  auto logits = torch::empty({rows, tot}, x.options());
  auto idx = torch::empty({rows, k}, torch::dtype(torch::kLong).device(x.device()));
  auto prob = torch::empty({rows, k}, x.options());
  FMOE_CUDA_CHECK(fmoe::launch_gate_linear_topk(
      dtype16(x), x.data_ptr(), w.data_ptr(), bias.has_value() ? bias->data_ptr() : nullptr, rows, d,
      tot, static_cast<int>(k), logits.data_ptr(), idx.data_ptr<int64_t>(), prob.data_ptr(),
      cur_stream()));
  return {logits, idx, prob};
}

// Returns {dx or empty, dw (layer dtype), db or empty, dl fp32 [B, tot]}.
std::vector<torch::Tensor> gate_linear_topk_bwd(c10::optional<torch::Tensor> dprob, torch::Tensor idx,
                                                torch::Tensor prob,
                                                c10::optional<torch::Tensor> dlogits,
                                                torch::Tensor x, torch::Tensor w, bool need_dx,
                                                bool need_db) {
  check_cuda_contig(x, "x");
  check_cuda_contig(w, "w");
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = static_cast<int>(x.size(0));
  const int d = static_cast<int>(x.size(1));
  const int tot = static_cast<int>(w.size(0));
  const int k = static_cast<int>(idx.size(1));
  auto f32 = torch::dtype(torch::kFloat).device(x.device());
  auto dl = torch::empty({rows, tot}, f32);
  torch::Tensor dx = need_dx ? torch::empty_like(x) : torch::Tensor();
  const bool fused_dw = tot <= 16;
  // one zero-filled buffer for dW and db so that a single fill and a single cast serve both
  torch::Tensor acc = fused_dw ? torch::zeros({static_cast<long>(tot) * d + tot}, f32) : torch::Tensor();
  FMOE_CUDA_CHECK(fmoe::launch_gate_bwd(
      dtype16(x), dprob.has_value() ? dprob->data_ptr() : nullptr, idx.data_ptr<int64_t>(),
      prob.data_ptr(), dlogits.has_value() ? dlogits->data_ptr() : nullptr, x.data_ptr(),
      w.data_ptr(), rows, d, tot, k, dl.data_ptr<float>(), need_dx ? dx.data_ptr() : nullptr,
      fused_dw ? acc.data_ptr<float>() : nullptr,
      fused_dw ? acc.data_ptr<float>() + static_cast<long>(tot) * d : nullptr, cur_stream()));
  torch::Tensor dw, db;
  if (fused_dw) {
    g_launches.fetch_add(1, std::memory_order_relaxed);  // the weight-gradient kernel
    auto cast = acc.to(x.scalar_type());
    dw = cast.narrow(0, 0, static_cast<long>(tot) * d).view({tot, d});
    if (need_db) db = cast.narrow(0, static_cast<long>(tot) * d, tot);
  } else {
    auto dl16 = dl.to(x.scalar_type());
    dw = dl16.t().matmul(x);
    if (need_db) db = dl.sum(0).to(x.scalar_type());
  }
  return {dx, dw, db, dl};
}

// ------------------------------------------------------------------------------ status
int64_t read_status(int64_t device) {
  auto t = status_tensor(static_cast<int>(device));
  return t.cpu().data_ptr<int>()[0];
}

void clear_status(int64_t device) { status_tensor(static_cast<int>(device)).zero_(); }

torch::Tensor status_word(int64_t device) { return status_tensor(static_cast<int>(device)); }

}  // namespace

void bind_p2p(pybind11::module& m);  // sm100/p2p_binding.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "fastmoe_b200 native ops (sm_100a kernels + C++ host runtime)";
  // reference-compatible names
  m.def("expert_count", &expert_count);
  m.def("assign_pos", &assign_pos);
  m.def("limit_by_capacity", &limit_by_capacity);
  m.def("prune_gate_by_capacity", &prune_gate_by_capacity);
  // device-count-driven API
  m.def("route", [](torch::Tensor idx, int64_t tot) { return route(idx, tot, false); });
  m.def("route_offs", [](torch::Tensor idx, int64_t tot) { return route(idx, tot, true); });
  // counts, rank, offs and pos (slot ids sorted by expert then rank: the send order of the
  // fused dispatch)
  m.def("route_pos", [](torch::Tensor idx, int64_t tot) { return route(idx, tot, true, true); });
  m.def("swipe_reassign", &swipe_reassign);
  m.def("grouped_gemm", &grouped_gemm, py::arg("mode"), py::arg("a"), py::arg("b"), py::arg("offs"),
        py::arg("out"), py::arg("bias") = py::none(), py::arg("pre_out") = py::none(),
        py::arg("aux") = py::none(), py::arg("act") = 0, py::arg("epi") = 0,
        py::arg("accumulate") = false, py::arg("psum") = py::none());
  m.def("grouped_gemm_supported", &grouped_gemm_supported);
  m.def("simt_grouped_gemm", &simt_grouped_gemm, py::arg("mode"), py::arg("a"), py::arg("b"),
        py::arg("offs"), py::arg("out"), py::arg("bias") = py::none());
  m.def("scatter_rows", &scatter_rows, py::arg("src"), py::arg("idx"), py::arg("rank"),
        py::arg("base"), py::arg("scale"), py::arg("k"), py::arg("dst"),
        py::arg("row_slot") = py::none());
  m.def("gather_combine", &gather_combine);
  m.def("combine_bwd", &combine_bwd);
  m.def("colsum", &colsum);
  m.def("gate_topk_softmax", &gate_topk_softmax);
  m.def("gate_topk_softmax_bwd", &gate_topk_softmax_bwd);
  m.def("gate_fused_supported", &gate_fused_supported);
  m.def("gate_linear_topk", &gate_linear_topk);
  m.def("gate_linear_topk_bwd", &gate_linear_topk_bwd);
  m.def("launch_count", []() { return g_launches.load(); });
  m.def("read_status", &read_status);
  m.def("clear_status", &clear_status);
  m.def("status_word", &status_word);
  // C++ CPU ops
  m.def("cpu_route", &fmoe::cpu::route);
  m.def("cpu_limit_by_capacity", &fmoe::cpu::limit_by_capacity);
  m.def("cpu_prune_gate_by_capacity", &fmoe::cpu::prune_gate_by_capacity);
  m.def("cpu_linear_forward", &fmoe::cpu::linear_forward);
  m.def("cpu_linear_backward", &fmoe::cpu::linear_backward);
  m.def("cpu_swipe_plan", &fmoe::cpu::swipe_plan);
  m.def("cpu_smart_schedule_plan", &fmoe::cpu::smart_schedule_plan);
  bind_p2p(m);
}
