// Elementwise halves of the THC baseline as single kernels: clip + scale + stochastic rounding to integer bins
// (rounding offsets from the counter-based generator, so a run is reproducible from its seed), and the inverse.
// The Hadamard rotation around them is fwht_tcgen05.cu / fwht_strided.cu; the bins travel over the fused
// kernel's identity wire.
//
// Reference counterparts (chains of torch operators): testbed_evaluation/new_comm_hooks/thc_hooks.py:152-223
// (quantise), :226-270 (dequantise); simulation stack simulations_llm/new_comm_hooks/thc_hooks.py:123-339.
//
// `stats` is what one small sum all-reduce leaves on every rank: stats[r] = ||g_r|| for r < world (each rank
// contributes its own entry), stats[world] = sum over ranks of the first rotated coordinate, which THC sends
// exactly.  range = T * max_r stats[r] / sqrt(d), at least 1e-30.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../common/philox.cuh"

namespace dq {
namespace {

__device__ __forceinline__ float thc_range(const float* stats, int world, float t_over_sqrt_d) {
  float m = 0.0f;
  for (int r = 0; r < world; ++r) m = fmaxf(m, stats[r]);
  return fmaxf(__fmul_rn(t_over_sqrt_d, m), 1e-30f);
}

// bins = clamp(floor((clamp(y, -range, range) + range) / (2 range) * (levels - 1) + u), 0, levels - 1),
// u = (byte + 0.5) / 256 with byte i from Philox-4x32-7 counter (i / 16, 0, stream, step): thread handles 16 values
__global__ void __launch_bounds__(256) thc_quantize_kernel(float* __restrict__ y, const float* __restrict__ stats, int world,
                                                           float t_over_sqrt_d, int levels, long long d, uint32_t stream,
                                                           uint32_t step, uint32_t seed_lo, uint32_t seed_hi) {
  const float range = thc_range(stats, world, t_over_sqrt_d);
  const float two_range = __fmul_rn(2.0f, range), top = static_cast<float>(levels - 1);
  for (long long call = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; call * 16 < d;
       call += static_cast<long long>(gridDim.x) * blockDim.x) {
    const U4 r = philox4x32<7>(static_cast<uint32_t>(call), 0u, stream, step, seed_lo, seed_hi);
    const uint32_t words[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const long long i = call * 16 + k;
      if (i >= d) break;
      const float u = __fmul_rn(__fadd_rn(static_cast<float>((words[k >> 2] >> (8 * (k & 3))) & 0xFFu), 0.5f), 1.0f / 256.0f);
      const float c = fminf(fmaxf(y[i], -range), range);
      const float t = __fmul_rn(__fdiv_rn(__fadd_rn(c, range), two_range), top);
      y[i] = fminf(fmaxf(floorf(__fadd_rn(t, u)), 0.0f), top);
    }
  }
}

// mean = (total / (levels - 1) * (2 range) - world * range) / world; mean[0] = stats[world] / world
__global__ void __launch_bounds__(256) thc_dequantize_kernel(float* __restrict__ total, const float* __restrict__ stats,
                                                             int world, float t_over_sqrt_d, int levels, long long d) {
  const float range = thc_range(stats, world, t_over_sqrt_d);
  const float two_range = __fmul_rn(2.0f, range), top = static_cast<float>(levels - 1);
  const float w = static_cast<float>(world), shift = __fmul_rn(w, range);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < d;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = __fdiv_rn(__fsub_rn(__fmul_rn(__fdiv_rn(total[i], top), two_range), shift), w);
    total[i] = i == 0 ? __fdiv_rn(stats[world], w) : v;
  }
}

void check_thc(const at::Tensor& y, const at::Tensor& stats, int64_t world, int64_t levels) {
  TORCH_CHECK(y.is_cuda() && y.scalar_type() == at::kFloat && y.is_contiguous() && y.dim() == 1, "thc: flat fp32 CUDA tensor");
  TORCH_CHECK(stats.is_cuda() && stats.scalar_type() == at::kFloat && stats.is_contiguous() && stats.numel() >= world + 1,
              "thc: stats needs world + 1 fp32 entries on the device");
  TORCH_CHECK(world >= 1 && world <= 4096 && levels >= 2, "thc: bad world / levels");
}

}  // namespace

void thc_quantize_(at::Tensor y, at::Tensor stats, int64_t world, double t_over_sqrt_d, int64_t levels, int64_t stream,
                   int64_t step, int64_t seed) {
  check_thc(y, stats, world, levels);
  c10::cuda::CUDAGuard guard(y.device());
  const long long d = y.numel();
  if (d == 0) return;
  const int grid = static_cast<int>(std::min<long long>((d / 16 + 255) / 256 + 1, 148 * 8));
  const uint64_t s = static_cast<uint64_t>(seed);
  thc_quantize_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      y.data_ptr<float>(), stats.data_ptr<float>(), static_cast<int>(world), static_cast<float>(t_over_sqrt_d),
      static_cast<int>(levels), d, static_cast<uint32_t>(stream), static_cast<uint32_t>(step),
      static_cast<uint32_t>(s & 0xFFFFFFFFull), static_cast<uint32_t>(s >> 32));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void thc_dequantize_(at::Tensor total, at::Tensor stats, int64_t world, double t_over_sqrt_d, int64_t levels) {
  check_thc(total, stats, world, levels);
  c10::cuda::CUDAGuard guard(total.device());
  const long long d = total.numel();
  if (d == 0) return;
  const int grid = static_cast<int>(std::min<long long>((d + 255) / 256, 148 * 8));
  thc_dequantize_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      total.data_ptr<float>(), stats.data_ptr<float>(), static_cast<int>(world), static_cast<float>(t_over_sqrt_d),
      static_cast<int>(levels), d);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace dq
