// Bindings of the peer-to-peer kernels: an ExchangeContext object per expert-parallel group
// holds the peers' signal-buffer addresses, the device-resident epoch words and the status
// word; its methods launch the kernels of p2p.cu on the current stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <pybind11/stl.h>

#include "grouped_gemm.cuh"
#include "p2p.cuh"

void fmoe_count_launch();  // binding.cpp: the library's launch counter

namespace {

#define FMOE_P2P_CHECK(expr)                                                        \
  do {                                                                              \
    cudaError_t _e = (expr);                                                        \
    TORCH_CHECK(_e == cudaSuccess, "fastmoe_b200: ", #expr, " failed: ",            \
                cudaGetErrorString(_e));                                            \
  } while (0)

fmoe::PeerPtrs to_ptrs(const std::vector<int64_t>& v) {
  TORCH_CHECK(static_cast<int>(v.size()) <= fmoe::kMaxPeers, "at most ", fmoe::kMaxPeers, " peers");
  fmoe::PeerPtrs p;
  for (int i = 0; i < fmoe::kMaxPeers; ++i) p.p[i] = nullptr;
  for (size_t i = 0; i < v.size(); ++i) p.p[i] = reinterpret_cast<void*>(v[i]);
  return p;
}

int dtype16(const torch::Tensor& t) {
  if (t.scalar_type() == torch::kBFloat16) return 0;
  TORCH_CHECK(t.scalar_type() == torch::kHalf, "expected a bf16 or fp16 tensor");
  return 1;
}

class ExchangeContext {
 public:
  ExchangeContext(std::vector<int64_t> flag_ptrs, torch::Tensor epoch, int64_t me, int64_t world,
                  torch::Tensor status, double timeout_ms)
      : epoch_(epoch), status_(status) {
    TORCH_CHECK(epoch.is_cuda() && epoch.scalar_type() == torch::kInt && epoch.numel() >= 8,
                "epoch must be an int32 CUDA tensor with at least 8 elements");
    TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt, "status must be int32 CUDA");
    TORCH_CHECK(static_cast<int64_t>(flag_ptrs.size()) == world, "one signal buffer per rank");
    ctx_.flags = to_ptrs(flag_ptrs);
    ctx_.epoch = epoch.data_ptr<int>();
    ctx_.me = static_cast<int>(me);
    ctx_.world = static_cast<int>(world);
    ctx_.status = status.data_ptr<int>();
    set_timeout_ms(timeout_ms);
  }

  void set_timeout_ms(double ms) { ctx_.timeout_ns = static_cast<unsigned long long>(ms * 1e6); }

  // `tables` is one int32 tensor holding, back to back: dst_base[tot], seg_base[tot],
  // blk_base[tot], expert_offs[E + 1], seg_off[E * (world + 1)], total_rows[1],
  // item_prefix[tot + 1], blk_order[capacity / 128 + E].
  void count_exchange(torch::Tensor lec, std::vector<int64_t> cnt_ptrs, int64_t n_expert,
                      int64_t capacity_rows, torch::Tensor tables) {
    c10::cuda::CUDAGuard guard(lec.device());
    const int64_t tot = n_expert * ctx_.world;
    const int64_t fixed = 4 * tot + (n_expert + 1) + n_expert * (ctx_.world + 1) + 2;
    TORCH_CHECK(tables.scalar_type() == torch::kInt && tables.is_contiguous() &&
                    tables.numel() >= fixed + capacity_rows / fmoe::kRowBlock + n_expert,
                "count_exchange: table tensor too small");
    int* t = tables.data_ptr<int>();
    FMOE_P2P_CHECK(fmoe::launch_count_exchange(
        ctx_, lec.data_ptr<int>(), to_ptrs(cnt_ptrs), static_cast<int>(n_expert),
        static_cast<int>(capacity_rows), t, t + tot, t + 2 * tot, t + 3 * tot,
        t + 3 * tot + n_expert + 1, t + 3 * tot + n_expert + 1 + n_expert * (ctx_.world + 1),
        t + 3 * tot + n_expert + 2 + n_expert * (ctx_.world + 1), t + fixed, stream()));
  }

  std::vector<torch::Tensor> capacity_grant(torch::Tensor lec, torch::Tensor cap,
                                            std::vector<int64_t> cnt_ptrs, int64_t n_expert) {
    TORCH_CHECK(lec.scalar_type() == torch::kInt && cap.scalar_type() == torch::kInt,
                "capacity_grant: int32 counts and capacities");
    TORCH_CHECK(lec.numel() == n_expert * ctx_.world && cap.numel() == n_expert,
                "capacity_grant: shapes");
    c10::cuda::CUDAGuard guard(lec.device());
    auto opts = torch::dtype(torch::kLong).device(lec.device());
    auto new_lec = torch::empty({lec.numel()}, opts);
    auto new_gec = torch::empty({lec.numel()}, opts);
    FMOE_P2P_CHECK(fmoe::launch_begin_epoch(ctx_, stream()));
    FMOE_P2P_CHECK(fmoe::launch_capacity_grant(ctx_, lec.data_ptr<int>(), cap.data_ptr<int>(),
                                               to_ptrs(cnt_ptrs), static_cast<int>(n_expert),
                                               new_lec.data_ptr<int64_t>(),
                                               new_gec.data_ptr<int64_t>(), stream()));
    return {new_lec, new_gec};
  }

  std::vector<torch::Tensor> swipe_exchange(torch::Tensor want, torch::Tensor cap,
                                            std::vector<int64_t> tab_ptrs) {
    TORCH_CHECK(want.scalar_type() == torch::kInt && want.numel() == ctx_.world && want.is_cuda(),
                "swipe_exchange: int32 [world] request counts on the GPU");
    TORCH_CHECK(cap.scalar_type() == torch::kLong && cap.numel() == 1 && cap.is_cuda(),
                "swipe_exchange: int64 [1] capacity on the GPU");
    c10::cuda::CUDAGuard guard(want.device());
    auto quota = torch::empty({ctx_.world}, torch::dtype(torch::kInt).device(want.device()));
    auto left = torch::empty({1}, torch::dtype(torch::kLong).device(want.device()));
    FMOE_P2P_CHECK(fmoe::launch_begin_epoch(ctx_, stream()));
    FMOE_P2P_CHECK(fmoe::launch_swipe_exchange(ctx_, want.data_ptr<int>(), cap.data_ptr<int64_t>(),
                                               to_ptrs(tab_ptrs), quota.data_ptr<int>(),
                                               left.data_ptr<int64_t>(), stream()));
    return {quota, left};
  }

  void begin_epoch() {
    c10::cuda::CUDAGuard guard(epoch_.device());
    FMOE_P2P_CHECK(fmoe::launch_begin_epoch(ctx_, stream()));
  }

  void dispatch_push(torch::Tensor x, torch::Tensor idx, torch::Tensor rank, torch::Tensor dst_base,
                     c10::optional<torch::Tensor> scale, std::vector<int64_t> rows_ptrs,
                     std::vector<int64_t> meta_ptrs, int64_t n_expert, int64_t k,
                     int64_t capacity_rows) {
    c10::cuda::CUDAGuard guard(x.device());
    const void* sc = (scale.has_value() && scale->defined()) ? scale->data_ptr() : nullptr;
    FMOE_P2P_CHECK(fmoe::launch_dispatch_push(
        ctx_, dtype16(x), x.data_ptr(), idx.data_ptr<int64_t>(), rank.data_ptr<int>(),
        dst_base.data_ptr<int>(), sc, to_ptrs(rows_ptrs), to_ptrs(meta_ptrs),
        static_cast<int>(n_expert), static_cast<int>(idx.numel()), static_cast<int>(k),
        static_cast<int>(x.size(1)), static_cast<int>(capacity_rows), stream()));
  }

  void wait_copy(int64_t channel, torch::Tensor stage_rows, c10::optional<torch::Tensor> stage_meta,
                 torch::Tensor total_rows, torch::Tensor out_rows,
                 c10::optional<torch::Tensor> out_meta) {
    c10::cuda::CUDAGuard guard(out_rows.device());
    const bool with_meta = stage_meta.has_value() && stage_meta->defined() &&
                           out_meta.has_value() && out_meta->defined();
    FMOE_P2P_CHECK(fmoe::launch_wait_copy(
        ctx_, static_cast<int>(channel), dtype16(out_rows), stage_rows.data_ptr(),
        with_meta ? stage_meta->data_ptr<int64_t>() : nullptr, total_rows.data_ptr<int>(),
        static_cast<int>(out_rows.size(1)), static_cast<int>(out_rows.size(0)), out_rows.data_ptr(),
        with_meta ? out_meta->data_ptr<int64_t>() : nullptr, stream()));
  }

  void wait_arrival(int64_t channel) {
    c10::cuda::CUDAGuard guard(epoch_.device());
    FMOE_P2P_CHECK(fmoe::launch_wait_arrival(ctx_, static_cast<int>(channel), stream()));
  }

  void return_push(torch::Tensor rows, torch::Tensor meta, torch::Tensor total_rows,
                   std::vector<int64_t> ret_ptrs, int64_t ret_slots) {
    c10::cuda::CUDAGuard guard(rows.device());
    FMOE_P2P_CHECK(fmoe::launch_return_push(ctx_, dtype16(rows), rows.data_ptr(),
                                            meta.data_ptr<int64_t>(), total_rows.data_ptr<int>(),
                                            to_ptrs(ret_ptrs), static_cast<int>(rows.size(1)),
                                            static_cast<int>(rows.size(0)), ret_slots, stream()));
  }

  void wait_combine(torch::Tensor ret, torch::Tensor idx, c10::optional<torch::Tensor> weight,
                    int64_t k, torch::Tensor out, c10::optional<torch::Tensor> keep,
                    c10::optional<torch::Tensor> rank, c10::optional<torch::Tensor> dst_base,
                    int64_t capacity_rows) {
    c10::cuda::CUDAGuard guard(out.device());
    const void* w = (weight.has_value() && weight->defined()) ? weight->data_ptr() : nullptr;
    void* kp = (keep.has_value() && keep->defined()) ? keep->data_ptr() : nullptr;
    const int* rk = nullptr;
    const int* db = nullptr;
    if (rank.has_value() && rank->defined()) {
      TORCH_CHECK(dst_base.has_value() && dst_base->defined() && rank->scalar_type() == torch::kInt &&
                      dst_base->scalar_type() == torch::kInt && rank->numel() == idx.numel(),
                  "wait_combine: int32 slot ranks (one per slot) and destination bases");
      rk = rank->data_ptr<int>();
      db = dst_base->data_ptr<int>();
    }
    FMOE_P2P_CHECK(fmoe::launch_wait_combine(ctx_, dtype16(out), ret.data_ptr(),
                                             idx.data_ptr<int64_t>(), w, rk, db,
                                             static_cast<int>(capacity_rows),
                                             static_cast<int>(out.size(0)), static_cast<int>(k),
                                             static_cast<int>(out.size(1)), out.data_ptr(), kp,
                                             stream()));
  }

  void allreduce(std::vector<int64_t> buf_ptrs, torch::Tensor out, int64_t n, double scale,
                 bool two_shot) {
    c10::cuda::CUDAGuard guard(out.device());
    int code;
    switch (out.scalar_type()) {
      case torch::kBFloat16: code = 0; break;
      case torch::kHalf: code = 1; break;
      case torch::kFloat: code = 2; break;
      default: TORCH_CHECK(false, "allreduce: bf16, fp16 or fp32"); code = -1;
    }
    FMOE_P2P_CHECK(fmoe::launch_begin_reduce_epoch(ctx_, stream()));
    if (two_shot) {
      FMOE_P2P_CHECK(fmoe::launch_allreduce_two_shot(ctx_, code, to_ptrs(buf_ptrs), out.data_ptr(),
                                                     n, static_cast<float>(scale), stream()));
    } else {
      FMOE_P2P_CHECK(fmoe::launch_allreduce(ctx_, code, to_ptrs(buf_ptrs), out.data_ptr(), n,
                                            static_cast<float>(scale), stream()));
    }
  }

  // All-reduce through the NVSwitch multicast mapping of the symmetric buffers.
  void allreduce_multimem(int64_t mc_ptr, int64_t mine_ptr, torch::Tensor out, double scale) {
    c10::cuda::CUDAGuard guard(out.device());
    int code;
    switch (out.scalar_type()) {
      case torch::kBFloat16: code = 0; break;
      case torch::kHalf: code = 1; break;
      case torch::kFloat: code = 2; break;
      default: TORCH_CHECK(false, "allreduce_multimem: bf16, fp16 or fp32"); code = -1;
    }
    TORCH_CHECK(mc_ptr != 0 && mc_ptr % 16 == 0 && mine_ptr % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0,
                "allreduce_multimem: a multicast mapping and 16-byte aligned buffers are required");
    FMOE_P2P_CHECK(fmoe::launch_begin_reduce_epoch(ctx_, stream()));
    FMOE_P2P_CHECK(fmoe::launch_allreduce_multimem(
        ctx_, code, reinterpret_cast<void*>(mc_ptr), reinterpret_cast<const void*>(mine_ptr),
        out.data_ptr(), out.numel() * out.element_size(), static_cast<float>(scale), stream()));
  }

  // out = rank `root`'s `src` on every rank (flat bytes, a multiple of 16).
  void broadcast(torch::Tensor src, std::vector<int64_t> buf_ptrs, torch::Tensor out, int64_t root) {
    TORCH_CHECK(src.is_cuda() && src.is_contiguous() && out.is_contiguous(), "broadcast operands");
    const int64_t bytes = out.numel() * out.element_size();
    TORCH_CHECK(src.numel() * src.element_size() == bytes && bytes % 16 == 0, "broadcast sizes");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0,
                "broadcast operands must be 16-byte aligned");
    c10::cuda::CUDAGuard guard(out.device());
    FMOE_P2P_CHECK(fmoe::launch_begin_reduce_epoch(ctx_, stream()));
    FMOE_P2P_CHECK(fmoe::launch_broadcast(ctx_, src.data_ptr(), to_ptrs(buf_ptrs), out.data_ptr(),
                                          bytes, static_cast<int>(root), stream()));
  }

  // out (on `root` only) = sum over ranks of the symmetric buffers' first n elements.
  void reduce_to_root(std::vector<int64_t> buf_ptrs, torch::Tensor out, int64_t n, int64_t root) {
    c10::cuda::CUDAGuard guard(out.device());
    int code;
    switch (out.scalar_type()) {
      case torch::kBFloat16: code = 0; break;
      case torch::kHalf: code = 1; break;
      case torch::kFloat: code = 2; break;
      default: TORCH_CHECK(false, "reduce_to_root: bf16, fp16 or fp32"); code = -1;
    }
    FMOE_P2P_CHECK(fmoe::launch_begin_reduce_epoch(ctx_, stream()));
    FMOE_P2P_CHECK(fmoe::launch_reduce_to_root(ctx_, code, to_ptrs(buf_ptrs), out.data_ptr(), n,
                                               static_cast<int>(root), stream()));
  }

  // out[r * n : (r + 1) * n] = rank r's `src` (flat bytes; src.nbytes a multiple of 16).
  void allgather(torch::Tensor src, std::vector<int64_t> buf_ptrs, torch::Tensor out) {
    TORCH_CHECK(src.is_cuda() && src.is_contiguous() && out.is_contiguous(), "allgather operands");
    const int64_t bytes = src.numel() * src.element_size();
    TORCH_CHECK(out.numel() * out.element_size() == bytes * ctx_.world, "allgather out size");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0,
                "allgather operands must be 16-byte aligned");
    c10::cuda::CUDAGuard guard(out.device());
    FMOE_P2P_CHECK(fmoe::launch_begin_reduce_epoch(ctx_, stream()));
    FMOE_P2P_CHECK(fmoe::launch_allgather(ctx_, src.data_ptr(), to_ptrs(buf_ptrs), out.data_ptr(),
                                          bytes, stream()));
  }

  // Row-mode grouped GEMM with the expert-parallel roles of the tcgen05 kernel:
  //   * `send` (dict, optional): sender warps copy this rank's token rows `x` (scaled by
  //     `scale` when given) into the peers' receive buffers in the order of `pos` and publish
  //     arrival flags — the dispatch direction of the exchange inside the GEMM launch;
  //   * `gate_flags` / `seg_off` (optional): the A operand is this rank's receive buffer and
  //     every tile waits for the arrival flags of its row block; with `blk_order` the tiles are
  //     walked in the order in which their row blocks arrive;
  //   * `push_meta` / `ret_ptrs` (optional): result rows go straight into their source ranks'
  //     return buffers and the return flags are raised when the grid is done.
  void gemm_ep(int64_t mode, torch::Tensor a, torch::Tensor b, torch::Tensor offs,
               c10::optional<torch::Tensor> out, c10::optional<torch::Tensor> bias,
               c10::optional<torch::Tensor> pre_out, c10::optional<torch::Tensor> aux, int64_t act,
               int64_t epi, c10::optional<torch::Tensor> push_meta, std::vector<int64_t> ret_ptrs,
               int64_t push_slots, c10::optional<pybind11::dict> send,
               std::vector<int64_t> gate_flag_ptrs, c10::optional<torch::Tensor> seg_off,
               c10::optional<torch::Tensor> blk_order, c10::optional<torch::Tensor> trace) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(mode == fmoe::kRowsNT || mode == fmoe::kRowsNN, "gemm_ep: row modes only");
    TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && offs.scalar_type() == torch::kInt,
                "gemm_ep: contiguous operands, int32 offsets");
    auto opt_ptr = [](const c10::optional<torch::Tensor>& t) -> void* {
      return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr;
    };
    fmoe::GroupedGemmArgs g;
    g.mode = static_cast<int>(mode);
    g.dtype = dtype16(a);
    g.num_groups = static_cast<int>(offs.numel() - 1);
    g.rows_cap = a.size(0);
    g.k = static_cast<int>(a.size(1));
    g.n = static_cast<int>(mode == fmoe::kRowsNT ? b.size(1) : b.size(2));
    g.a = a.data_ptr();
    g.b = b.data_ptr();
    g.offs = offs.data_ptr<int>();
    g.out = opt_ptr(out);
    g.bias = opt_ptr(bias);
    g.pre_out = opt_ptr(pre_out);
    g.aux = opt_ptr(aux);
    g.act = static_cast<int>(act);
    g.epi = static_cast<int>(epi);
    g.status = ctx_.status;
    if (push_meta.has_value() && push_meta->defined()) {
      g.push_meta = push_meta->data_ptr<int64_t>();
      g.push_dst = to_ptrs(ret_ptrs);
      g.push_flags = ctx_.flags;
      g.push_epoch = ctx_.epoch;
      g.push_counter = ctx_.epoch + 4;
      g.push_me = ctx_.me;
      g.push_world = ctx_.world;
      g.push_slots = push_slots;
    } else {
      TORCH_CHECK(g.out != nullptr, "gemm_ep: an output tensor or a push target is required");
    }
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, a.device().index());
    g.num_sms = sms;
    if (send.has_value()) {
      const pybind11::dict& d = *send;
      auto tensor = [&](const char* key) { return d[key].cast<torch::Tensor>(); };
      auto ptrs = [&](const char* key) { return to_ptrs(d[key].cast<std::vector<int64_t>>()); };
      fmoe::SendArgs& sa = g.send;
      torch::Tensor x = tensor("x");
      TORCH_CHECK(x.is_contiguous() && x.scalar_type() == a.scalar_type() &&
                      reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0,
                  "gemm_ep: rows to send must be contiguous, 16-byte aligned, of the GEMM's dtype");
      sa.x = x.data_ptr();
      sa.d = static_cast<int>(x.size(1));
      sa.pos = tensor("pos").data_ptr<int>();
      sa.my_offs = tensor("my_offs").data_ptr<int>();
      sa.dst_base = tensor("dst_base").data_ptr<int>();
      sa.seg_base = tensor("seg_base").data_ptr<int>();
      sa.blk_base = tensor("blk_base").data_ptr<int>();
      if (d.contains("scale") && !d["scale"].is_none()) sa.scale = tensor("scale").data_ptr();
      sa.rows = ptrs("rows_ptrs");
      if (d.contains("meta_ptrs") && !d["meta_ptrs"].is_none()) {
        sa.meta = ptrs("meta_ptrs");
      } else {
        for (int i = 0; i < fmoe::kMaxPeers; ++i) sa.meta.p[i] = nullptr;
      }
      sa.flags = ptrs("flag_ptrs");
      sa.epoch = ctx_.epoch;
      sa.n_expert = d["n_expert"].cast<int>();
      sa.world = ctx_.world;
      sa.me = ctx_.me;
      sa.k = d["k"].cast<int>();
      sa.capacity = d["capacity"].cast<int>();
      sa.item_prefix = tensor("item_prefix").data_ptr<int>();
      sa.item_count = tensor("item_count").data_ptr<int>();
      sa.enabled = 1;
      TORCH_CHECK(sa.d == g.k, "gemm_ep: sent rows must have the GEMM's K extent");
    }
    if (!gate_flag_ptrs.empty()) {
      TORCH_CHECK(seg_off.has_value() && seg_off->defined() && seg_off->scalar_type() == torch::kInt,
                  "gemm_ep: gating needs the per-source segment offsets");
      g.gate.flags = reinterpret_cast<const int*>(gate_flag_ptrs[ctx_.me]);
      g.gate.seg_off = seg_off->data_ptr<int>();
      g.gate.epoch = ctx_.epoch;
      g.gate.world = ctx_.world;
      g.gate.me = ctx_.me;
      g.gate.timeout_ns = ctx_.timeout_ns;
      if (blk_order.has_value() && blk_order->defined()) {
        // tiles are walked in the arrival order of their row blocks (count_exchange's table)
        TORCH_CHECK(blk_order->scalar_type() == torch::kInt && blk_order->is_contiguous() &&
                        blk_order->numel() >= a.size(0) / fmoe::kRowBlock + g.num_groups,
                    "gemm_ep: block-order table too small for the receive buffer");
        g.gate.blk_order = blk_order->data_ptr<int>();
      }
    }
    if (trace.has_value() && trace->defined()) {
      TORCH_CHECK(trace->scalar_type() == torch::kLong && trace->is_cuda() &&
                      trace->numel() >= static_cast<int64_t>(sms) * 10,
                  "gemm_ep: trace must be a zeroed int64 CUDA tensor of 10 entries per SM");
      g.trace = reinterpret_cast<unsigned long long*>(trace->data_ptr<int64_t>());
    }
    g.stream = stream();
    TORCH_CHECK(fmoe::grouped_gemm_supported(g.mode, 0, g.n, g.k, g.num_groups),
                "gemm_ep: shape not supported by the tcgen05 kernel");
    FMOE_P2P_CHECK(fmoe::launch_grouped_gemm(g));
  }

  void wait_only(int64_t channel) {
    c10::cuda::CUDAGuard guard(epoch_.device());
    FMOE_P2P_CHECK(fmoe::launch_wait_only(ctx_, static_cast<int>(channel), stream()));
  }

 private:
  // One call per kernel launch: also feeds the library's launch counter.
  cudaStream_t stream() {
    fmoe_count_launch();
    return at::cuda::getCurrentCUDAStream().stream();
  }
  fmoe::ExchangeCtx ctx_;
  torch::Tensor epoch_;
  torch::Tensor status_;
};

void slot_dot(torch::Tensor dout, torch::Tensor y, torch::Tensor idx, int64_t k,
              torch::Tensor dscore) {
  c10::cuda::CUDAGuard guard(dout.device());
  fmoe_count_launch();
  FMOE_P2P_CHECK(fmoe::launch_slot_dot(dtype16(dout), dout.data_ptr(), y.data_ptr(),
                                       idx.data_ptr<int64_t>(), static_cast<int>(idx.numel()),
                                       static_cast<int>(k), static_cast<int>(dout.size(1)),
                                       dscore.data_ptr(),
                                       at::cuda::getCurrentCUDAStream().stream()));
}

}  // namespace

void bind_p2p(pybind11::module& m) {
  namespace py = pybind11;
  py::class_<ExchangeContext>(m, "ExchangeContext")
      .def(py::init<std::vector<int64_t>, torch::Tensor, int64_t, int64_t, torch::Tensor, double>())
      .def("set_timeout_ms", &ExchangeContext::set_timeout_ms)
      .def("count_exchange", &ExchangeContext::count_exchange)
      .def("capacity_grant", &ExchangeContext::capacity_grant)
      .def("begin_epoch", &ExchangeContext::begin_epoch)
      .def("swipe_exchange", &ExchangeContext::swipe_exchange)
      .def("dispatch_push", &ExchangeContext::dispatch_push)
      .def("wait_copy", &ExchangeContext::wait_copy)
      .def("wait_arrival", &ExchangeContext::wait_arrival)
      .def("return_push", &ExchangeContext::return_push)
      .def("wait_combine", &ExchangeContext::wait_combine, py::arg("ret"), py::arg("idx"),
           py::arg("weight"), py::arg("k"), py::arg("out"), py::arg("keep"),
           py::arg("rank") = py::none(), py::arg("dst_base") = py::none(),
           py::arg("capacity_rows") = 0)
      .def("allgather", &ExchangeContext::allgather)
      .def("allreduce_multimem", &ExchangeContext::allreduce_multimem)
      .def("broadcast", &ExchangeContext::broadcast)
      .def("reduce_to_root", &ExchangeContext::reduce_to_root)
      .def("allreduce", &ExchangeContext::allreduce, py::arg("buf_ptrs"), py::arg("out"),
           py::arg("n"), py::arg("scale"), py::arg("two_shot") = false)
      .def("gemm_ep", &ExchangeContext::gemm_ep, py::arg("mode"), py::arg("a"), py::arg("b"),
           py::arg("offs"), py::arg("out") = py::none(), py::arg("bias") = py::none(),
           py::arg("pre_out") = py::none(), py::arg("aux") = py::none(), py::arg("act") = 0,
           py::arg("epi") = 0, py::arg("push_meta") = py::none(),
           py::arg("ret_ptrs") = std::vector<int64_t>(), py::arg("push_slots") = 0,
           py::arg("send") = py::none(), py::arg("gate_flag_ptrs") = std::vector<int64_t>(),
           py::arg("seg_off") = py::none(), py::arg("blk_order") = py::none(),
           py::arg("trace") = py::none())
      .def("wait_only", &ExchangeContext::wait_only);
  m.def("slot_dot", &slot_dot);
  m.attr("P2P_CHAN_COUNTS") = fmoe::kChanCounts;
  m.attr("P2P_CHAN_DISPATCH") = fmoe::kChanDispatch;
  m.attr("P2P_CHAN_RETURN") = fmoe::kChanReturn;
  m.attr("P2P_CHAN_REDUCE") = fmoe::kChanReduce;
  m.attr("P2P_MAX_PEERS") = fmoe::kMaxPeers;
  m.attr("P2P_NUM_CHANNELS") = fmoe::kNumChannels;
  m.attr("STATUS_PEER_TIMEOUT") = fmoe::kStatusPeerTimeout;
  m.attr("STATUS_RECV_OVERFLOW") = fmoe::kStatusRecvOverflow;
}
