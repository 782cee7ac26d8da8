// Host side of the tcgen05 grouped GEMM: tensor-map construction and dispatch.  The kernel
// lives in grouped_gemm_kernel.cuh and is instantiated per element type in
// grouped_gemm_bf16.cu / grouped_gemm_f16.cu.
#include "grouped_gemm_kernel.cuh"

namespace fmoe {
using namespace gg;
namespace {

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

// 2-D row-major tensor [outer, inner] of 16-bit elements, 128-byte swizzle.
bool make_map_2d(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
                 uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

bool grouped_gemm_supported(int mode, int m, int n, int k, int num_groups) {
  if (num_groups < 1 || num_groups > MAX_GROUPS) return false;
  if (n % 32 != 0 || n < 32) return false;
  if (mode == kWgrad) return m % 8 == 0 && m >= 8;
  return k % 64 == 0 && k >= 64;
}

cudaError_t launch_grouped_gemm(const GroupedGemmArgs& a) {
  if (!grouped_gemm_supported(a.mode, a.m, a.n, a.k, a.num_groups)) return cudaErrorInvalidValue;
  CUtensorMap ta, tb;
  bool ok = true;
  if (a.mode == kRowsNT) {
    ok = make_map_2d(&ta, a.dtype, a.a, a.k, a.rows_cap, BK, BM) &&
         make_map_2d(&tb, a.dtype, a.b, a.k, static_cast<uint64_t>(a.num_groups) * a.n, BK, BN);
  } else if (a.mode == kRowsNN) {
    ok = make_map_2d(&ta, a.dtype, a.a, a.k, a.rows_cap, BK, BM) &&
         make_map_2d(&tb, a.dtype, a.b, a.n, static_cast<uint64_t>(a.num_groups) * a.k, 64, BK);
  } else {
    ok = make_map_2d(&ta, a.dtype, a.a, a.m, a.rows_cap, 64, BK) &&
         make_map_2d(&tb, a.dtype, a.b, a.n, a.rows_cap, 64, BK);
  }
  if (!ok) return cudaErrorInvalidValue;

  KernelParams kp;
  kp.num_groups = a.num_groups;
  kp.m = a.m;
  kp.n = a.n;
  kp.k = a.k;
  kp.offs = a.offs;
  kp.out = a.out;
  kp.pre_out = a.pre_out;
  kp.bias = a.bias;
  kp.aux = a.aux;
  kp.act = a.act;
  kp.epi = a.epi;
  kp.accumulate = a.accumulate;
  kp.out_fp32 = a.out_fp32;
  kp.psum = (a.mode == kWgrad) ? a.psum : nullptr;
  kp.psrc = a.a;
  kp.status = a.status;
  kp.push_meta = a.push_meta;
  kp.push_dst = a.push_dst;
  kp.push_flags = a.push_flags;
  kp.push_epoch = a.push_epoch;
  kp.push_counter = a.push_counter;
  kp.push_me = a.push_me;
  kp.push_world = a.push_world;
  kp.push_slots = a.push_slots;
  kp.send = a.send;
  kp.gate = a.gate;
  kp.trace = a.trace;
  if (a.mode == kWgrad) {
    kp.send.enabled = 0;
    kp.gate.flags = nullptr;
  }
  if (kp.send.enabled && (kp.send.d % 8 != 0 || kp.send.item_prefix == nullptr ||
                          kp.send.item_count == nullptr)) {
    return cudaErrorInvalidValue;
  }

  const int grid = a.num_sms > 0 ? a.num_sms : 148;
  return a.dtype == kBF16 ? gg::launch_bf16(a.mode, ta, tb, kp, grid, a.stream)
                          : gg::launch_f16(a.mode, ta, tb, kp, grid, a.stream);
}

}  // namespace fmoe
