// Bindings of the peer-to-peer kernels: an ExchangeContext object per expert-parallel group
// holds the peers' signal-buffer addresses, the device-resident epoch words and the status
// word; its methods launch the kernels of p2p.cu on the current stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

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
    TORCH_CHECK(epoch.is_cuda() && epoch.scalar_type() == torch::kInt && epoch.numel() >= 4,
                "epoch must be an int32 CUDA tensor with at least 4 elements");
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

  void count_exchange(torch::Tensor lec, std::vector<int64_t> cnt_ptrs, int64_t n_expert,
                      int64_t capacity_rows, torch::Tensor dst_base, torch::Tensor expert_offs,
                      torch::Tensor total_rows) {
    c10::cuda::CUDAGuard guard(lec.device());
    FMOE_P2P_CHECK(fmoe::launch_count_exchange(
        ctx_, lec.data_ptr<int>(), to_ptrs(cnt_ptrs), static_cast<int>(n_expert),
        static_cast<int>(capacity_rows), dst_base.data_ptr<int>(), expert_offs.data_ptr<int>(),
        total_rows.data_ptr<int>(), stream()));
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
                   std::vector<int64_t> ret_ptrs) {
    c10::cuda::CUDAGuard guard(rows.device());
    FMOE_P2P_CHECK(fmoe::launch_return_push(ctx_, dtype16(rows), rows.data_ptr(),
                                            meta.data_ptr<int64_t>(), total_rows.data_ptr<int>(),
                                            to_ptrs(ret_ptrs), static_cast<int>(rows.size(1)),
                                            static_cast<int>(rows.size(0)), stream()));
  }

  void wait_combine(torch::Tensor ret, torch::Tensor idx, c10::optional<torch::Tensor> weight,
                    int64_t k, torch::Tensor out, c10::optional<torch::Tensor> keep) {
    c10::cuda::CUDAGuard guard(out.device());
    const void* w = (weight.has_value() && weight->defined()) ? weight->data_ptr() : nullptr;
    void* kp = (keep.has_value() && keep->defined()) ? keep->data_ptr() : nullptr;
    FMOE_P2P_CHECK(fmoe::launch_wait_combine(ctx_, dtype16(out), ret.data_ptr(),
                                             idx.data_ptr<int64_t>(), w,
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
    FMOE_P2P_CHECK(fmoe::launch_begin_epoch(ctx_, stream()));
    if (two_shot) {
      FMOE_P2P_CHECK(fmoe::launch_allreduce_two_shot(ctx_, code, to_ptrs(buf_ptrs), out.data_ptr(),
                                                     n, static_cast<float>(scale), stream()));
    } else {
      FMOE_P2P_CHECK(fmoe::launch_allreduce(ctx_, code, to_ptrs(buf_ptrs), out.data_ptr(), n,
                                            static_cast<float>(scale), stream()));
    }
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
    FMOE_P2P_CHECK(fmoe::launch_begin_epoch(ctx_, stream()));
    FMOE_P2P_CHECK(fmoe::launch_allgather(ctx_, src.data_ptr(), to_ptrs(buf_ptrs), out.data_ptr(),
                                          bytes, stream()));
  }

  // Grouped GEMM (forward mode 0 or input-gradient mode 1) whose epilogue stores each result
  // row into the slot-indexed return buffer of the row's source rank (`meta`, `ret_ptrs`) and
  // publishes the return flags when the grid is done: GEMM + combine-direction exchange in
  // one kernel.
  void gemm_push(int64_t mode, torch::Tensor a, torch::Tensor b, torch::Tensor offs,
                 c10::optional<torch::Tensor> bias, torch::Tensor meta,
                 std::vector<int64_t> ret_ptrs) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(mode == fmoe::kRowsNT || mode == fmoe::kRowsNN, "gemm_push: row modes only");
    TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && offs.scalar_type() == torch::kInt,
                "gemm_push: contiguous operands, int32 offsets");
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
    g.out = nullptr;
    if (bias.has_value() && bias->defined()) g.bias = bias->data_ptr();
    g.status = ctx_.status;
    g.push_meta = meta.data_ptr<int64_t>();
    g.push_dst = to_ptrs(ret_ptrs);
    g.push_flags = ctx_.flags;
    g.push_epoch = ctx_.epoch;
    g.push_counter = ctx_.epoch + 4;
    g.push_me = ctx_.me;
    g.push_world = ctx_.world;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, a.device().index());
    g.num_sms = sms;
    g.stream = stream();
    TORCH_CHECK(fmoe::grouped_gemm_supported(g.mode, 0, g.n, g.k, g.num_groups),
                "gemm_push: shape not supported by the tcgen05 kernel");
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
      .def("dispatch_push", &ExchangeContext::dispatch_push)
      .def("wait_copy", &ExchangeContext::wait_copy)
      .def("wait_arrival", &ExchangeContext::wait_arrival)
      .def("return_push", &ExchangeContext::return_push)
      .def("wait_combine", &ExchangeContext::wait_combine)
      .def("allgather", &ExchangeContext::allgather)
      .def("allreduce", &ExchangeContext::allreduce, py::arg("buf_ptrs"), py::arg("out"),
           py::arg("n"), py::arg("scale"), py::arg("two_shot") = false)
      .def("gemm_push", &ExchangeContext::gemm_push)
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
