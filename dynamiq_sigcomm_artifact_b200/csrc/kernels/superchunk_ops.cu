// Superchunk mean-centring and its inverse: one warp per 256-element superchunk.
//   centre:   residual = x - mean(x),  stats = (mean / W, sum((x / W)^2))     (fp32)
//   add_mean: out = residual + mean
// Counterparts of superchunk_mean_center_kernel / superchunk_add_mean_copy_kernel
// (cuda_kernels/src/srrcomp/eden_utils/csrc/cuda_hadamard.cu:1257-1369), which use one 256-thread
// CTA per superchunk with a shared-memory tree and bf16 statistics.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <torch/extension.h>

namespace dq {
namespace {

__device__ __forceinline__ float ld_as_float(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float ld_as_float(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st_from_float(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st_from_float(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) sc_center_kernel(const T* __restrict__ x, float* __restrict__ resid,
                                                        float* __restrict__ stats, long long n, long long nsc,
                                                        float inv_world) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * static_cast<long long>(blockDim.x)) >> 5;
  for (long long sc = warp; sc < nsc; sc += nwarps) {
    float v[8], s = 0.f, ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long i = sc * 256 + j * 32 + lane;
      float f = i < n ? ld_as_float(x, i) : 0.f;
      f = (fabsf(f) <= 3.402823466e38f) ? f : 0.f;
      v[j] = f;
      s += f;
      ss += (f * inv_world) * (f * inv_world);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
      ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    }
    const float mean = s * (1.0f / 256.0f);  // padded positions count as zeros, as in the reference
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long i = sc * 256 + j * 32 + lane;
      resid[i] = i < n ? v[j] - mean : 0.f;
    }
    if (lane == 0) {
      stats[2 * sc] = mean * inv_world;
      stats[2 * sc + 1] = ss;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) sc_add_mean_kernel(const float* __restrict__ resid,
                                                          const float* __restrict__ mean, T* __restrict__ out,
                                                          long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    st_from_float(out, i, resid[i] + mean[i >> 8]);
}

}  // namespace

// x: flat fp32 / bf16 -> (residual fp32 [nsc * 256], stats fp32 [nsc, 2])
std::tuple<at::Tensor, at::Tensor> superchunk_center(at::Tensor x, int64_t world) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && (x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16),
              "superchunk_center: contiguous CUDA fp32 / bf16 tensor");
  c10::cuda::CUDAGuard guard(x.device());
  const long long n = x.numel(), nsc = (n + 255) / 256;
  auto fopt = x.options().dtype(at::kFloat);
  at::Tensor resid = at::empty({nsc * 256}, fopt), stats = at::empty({nsc, 2}, fopt);
  if (n == 0) return {resid, stats};
  const int grid = static_cast<int>(std::min<long long>((nsc + 7) / 8, 148LL * 8));
  auto stream = at::cuda::getCurrentCUDAStream();
  const float inv = 1.0f / static_cast<float>(world);
  if (x.scalar_type() == at::kFloat)
    sc_center_kernel<float><<<grid, 256, 0, stream>>>(x.data_ptr<float>(), resid.data_ptr<float>(), stats.data_ptr<float>(), n, nsc, inv);
  else
    sc_center_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), resid.data_ptr<float>(), stats.data_ptr<float>(), n, nsc, inv);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {resid, stats};
}

// out[i] = residual[i] + mean[i / 256] for i < out.numel()
void superchunk_add_mean(at::Tensor resid, at::Tensor mean, at::Tensor out) {
  TORCH_CHECK(resid.is_cuda() && resid.scalar_type() == at::kFloat && resid.is_contiguous() && mean.is_cuda() &&
                  mean.scalar_type() == at::kFloat && mean.is_contiguous() && out.is_cuda() && out.is_contiguous(),
              "superchunk_add_mean: contiguous CUDA tensors, fp32 residual and mean");
  const long long n = out.numel();
  TORCH_CHECK(resid.numel() >= n && mean.numel() * 256 >= n, "superchunk_add_mean: residual / mean too short");
  if (n == 0) return;
  c10::cuda::CUDAGuard guard(out.device());
  const int grid = static_cast<int>(std::min<long long>((n + 255) / 256, 148LL * 16));
  auto stream = at::cuda::getCurrentCUDAStream();
  if (out.scalar_type() == at::kFloat)
    sc_add_mean_kernel<float><<<grid, 256, 0, stream>>>(resid.data_ptr<float>(), mean.data_ptr<float>(), out.data_ptr<float>(), n);
  else if (out.scalar_type() == at::kBFloat16)
    sc_add_mean_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(resid.data_ptr<float>(), mean.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), n);
  else
    TORCH_CHECK(false, "superchunk_add_mean: fp32 or bf16 output");
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace dq
