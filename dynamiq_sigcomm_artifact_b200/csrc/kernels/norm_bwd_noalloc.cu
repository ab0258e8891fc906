// RMSNorm backward without any allocation: the same kernels as torch.ops.dq.norm_bwd, with the
// per-warp partial sums of dw kept in a fixed device array of this library instead of a tensor
// obtained from the allocator.  Declaration and usage rules: dq_noalloc.h.  There is no
// counterpart of this entry point in the reference implementation.
#include "dq_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "norm_kernels.cuh"

namespace {

// Scratch shared by every call on a device: [DQ_NOALLOC_MAX_PARTS][hidden] floats, fully
// rewritten by norm_bwd_rows_kernel before reduce_parts2_kernel reads it.
static __device__ __align__(256) float g_noalloc_scratch[DQ_NOALLOC_MAX_PARTS * DQ_NOALLOC_MAX_HIDDEN];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch_addr[kMaxDevices] = {nullptr};  // device address of g_noalloc_scratch, per device
thread_local int t_last_cuda_error = 0;

// In host code `g_noalloc_scratch` is only a handle for the symbol; the address a kernel can
// use has to be asked for, once per device, with that device current.
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    t_last_cuda_error = static_cast<int>(e != cudaSuccess ? e : cudaErrorInvalidDevice);
    return DQ_NOALLOC_CUDA_ERROR;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {  // a null address with a success code still is a failure to report
      t_last_cuda_error = static_cast<int>(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
      return DQ_NOALLOC_CUDA_ERROR;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return DQ_NOALLOC_OK;
}

template <typename T, int NC>
void launch_rows(const void* dy, const void* x, const float* w, const float* rstd, void* dx, float* parts, int rows,
                 int hidden, int grid, cudaStream_t stream) {
  using namespace dq::normk;
  norm_bwd_rows_kernel<T, true, NC><<<grid, kNormWarps * 32, 0, stream>>>(
      static_cast<const T*>(dy), static_cast<const T*>(x), w, nullptr, rstd, static_cast<T*>(dx), parts, nullptr, rows,
      hidden);
}

template <typename T>
void launch_rows_nc(int nchunk, const void* dy, const void* x, const float* w, const float* rstd, void* dx,
                    float* parts, int rows, int hidden, int grid, cudaStream_t stream) {
  switch (nchunk) {
    case 1: launch_rows<T, 1>(dy, x, w, rstd, dx, parts, rows, hidden, grid, stream); break;
    case 2: launch_rows<T, 2>(dy, x, w, rstd, dx, parts, rows, hidden, grid, stream); break;
    case 3: launch_rows<T, 3>(dy, x, w, rstd, dx, parts, rows, hidden, grid, stream); break;
    case 4: launch_rows<T, 4>(dy, x, w, rstd, dx, parts, rows, hidden, grid, stream); break;
    case 5:
    case 6: launch_rows<T, 6>(dy, x, w, rstd, dx, parts, rows, hidden, grid, stream); break;
    default: launch_rows<T, 8>(dy, x, w, rstd, dx, parts, rows, hidden, grid, stream); break;
  }
}

bool bad_ptr(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

}  // namespace

extern "C" int dq_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, void* dx,
                                      float* dw, int rows, int hidden, int is_bf16, void* stream_ptr) {
  using namespace dq::normk;
  if (hidden <= 0 || hidden > DQ_NOALLOC_MAX_HIDDEN || hidden % 8 != 0) return DQ_NOALLOC_BAD_HIDDEN;
  if (rows <= 0) return DQ_NOALLOC_BAD_ROWS;
  if (bad_ptr(dy) || bad_ptr(x) || bad_ptr(w) || bad_ptr(dx) || bad_ptr(dw) || rstd == nullptr)
    return DQ_NOALLOC_BAD_POINTER;
  float* parts = nullptr;
  const int rc = scratch_for_current_device(&parts);
  if (rc != DQ_NOALLOC_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  (void)cudaGetLastError();  // an error left behind by the caller's earlier launches is not this call's
  const int max_grid = DQ_NOALLOC_MAX_PARTS / kNormWarps;
  int grid = (rows + kNormWarps - 1) / kNormWarps;
  if (grid > max_grid) grid = max_grid;
  const int nparts = grid * kNormWarps;  // <= DQ_NOALLOC_MAX_PARTS rows of `hidden` floats
  const int nchunk = (hidden + 255) / 256;
  if (is_bf16) launch_rows_nc<__nv_bfloat16>(nchunk, dy, x, w, rstd, dx, parts, rows, hidden, grid, stream);
  else launch_rows_nc<float>(nchunk, dy, x, w, rstd, dx, parts, rows, hidden, grid, stream);
  dim3 rb(32, 32);
  reduce_parts2_kernel<<<(hidden + 31) / 32, rb, 0, stream>>>(parts, dw, nparts, hidden);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    t_last_cuda_error = static_cast<int>(e);
    return DQ_NOALLOC_CUDA_ERROR;
  }
  return DQ_NOALLOC_OK;
}

extern "C" const char* dq_noalloc_strerror(int code) {
  switch (code) {
    case DQ_NOALLOC_OK: return "ok";
    case DQ_NOALLOC_BAD_HIDDEN: return "hidden size must be a positive multiple of 8 and at most DQ_NOALLOC_MAX_HIDDEN (2048)";
    case DQ_NOALLOC_BAD_ROWS: return "rows must be positive";
    case DQ_NOALLOC_BAD_POINTER: return "a pointer is null or not 16-byte aligned";
    case DQ_NOALLOC_CUDA_ERROR: return "a CUDA call failed (see dq_noalloc_last_cuda_error)";
    default: return "unknown code";
  }
}

extern "C" int dq_noalloc_last_cuda_error(void) { return t_last_cuda_error; }
