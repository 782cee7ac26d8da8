// Allocation-free variant of the bias-gradient (column sum per expert) path: the fp32
// accumulation buffer that the regular entry point obtains from torch is a file-scope device
// array here.  See noalloc_bias_grad.h for the contract.
#include "noalloc_bias_grad.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <mutex>

#include "routing.cuh"

namespace {

// The accumulation scratch.  In host code this name is only a handle for
// cudaGetSymbolAddress; the device address differs per GPU and is looked up once per device.
static __device__ __align__(256) float g_bias_scratch[FMOE_NOALLOC_MAX_ELEMS];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_mu;
thread_local const char* g_last_error = "";

__global__ void clear_kernel(float* p, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = 0.f;
}

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }

template <typename T>
__global__ void convert_kernel(const float* __restrict__ src, T* __restrict__ dst, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = from_f<T>(src[i]);
}

// Address of the scratch array on the current device; resolved on first use per device.
float* scratch_for_current_device(cudaError_t* err) {
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= kMaxDevices) {
    *err = cudaErrorInvalidDevice;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    *err = cudaGetSymbolAddress(&p, g_bias_scratch);
    if (*err != cudaSuccess) return nullptr;
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  return g_scratch_ptr[dev];
}

}  // namespace

extern "C" int fmoe_bias_grad_noalloc(const void* x, const int* offs, int num_groups, long rows_cap,
                                      int n, int dtype, void* out, cudaStream_t stream) {
  if (x == nullptr || offs == nullptr || out == nullptr || num_groups < 1 || rows_cap < 0 ||
      n < 8 || n % 8 != 0 || (dtype != 0 && dtype != 1)) {
    g_last_error = "fmoe_bias_grad_noalloc: bad argument (null pointer, n not a multiple of 8, or dtype not 0/1)";
    return -1;
  }
  // The kernels read x sixteen bytes at a time and the offsets as 32-bit words: a pointer a
  // C caller got wrong must come back as an error code, not as a device fault.
  if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(offs) % 4 != 0 ||
      reinterpret_cast<uintptr_t>(out) % 2 != 0) {
    g_last_error = "fmoe_bias_grad_noalloc: x must be 16-byte aligned, offs 4-byte, out 2-byte";
    return -1;
  }
#if CUDART_VERSION >= 12080
  {
    // A stream of another device would run the kernels against this device's scratch address.
    int cur = -1, sdev = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cudaStreamGetDevice(stream, &sdev) == cudaSuccess &&
        sdev != cur) {
      g_last_error = "fmoe_bias_grad_noalloc: the stream does not belong to the current device";
      return -1;
    }
    (void)cudaGetLastError();
  }
#endif
  const long elems = static_cast<long>(num_groups) * n;
  if (elems > FMOE_NOALLOC_MAX_ELEMS) {
    g_last_error = "fmoe_bias_grad_noalloc: num_groups * n exceeds FMOE_NOALLOC_MAX_ELEMS (65536)";
    return -2;
  }
  cudaError_t err = cudaSuccess;
  float* scratch = scratch_for_current_device(&err);
  if (scratch == nullptr) {
    g_last_error = cudaGetErrorString(err);
    return -3;
  }
  const int count = static_cast<int>(elems);
  const int blocks = (count + 255) / 256;
  // The array keeps the previous call's sums: clear the part this call accumulates into.
  clear_kernel<<<blocks, 256, 0, stream>>>(scratch, count);
  err = cudaGetLastError();
  if (err == cudaSuccess) {
    err = fmoe::launch_colsum(dtype, x, offs, num_groups, rows_cap, n, scratch, stream);
  }
  if (err == cudaSuccess) {
    if (dtype == 0) {
      convert_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(scratch, static_cast<__nv_bfloat16*>(out), count);
    } else {
      convert_kernel<__half><<<blocks, 256, 0, stream>>>(scratch, static_cast<__half*>(out), count);
    }
    err = cudaGetLastError();
  }
  if (err != cudaSuccess) {
    g_last_error = cudaGetErrorString(err);
    return -3;
  }
  g_last_error = "";
  return 0;
}

extern "C" const char* fmoe_noalloc_last_error(void) { return g_last_error; }
