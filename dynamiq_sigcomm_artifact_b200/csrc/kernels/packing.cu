// Bit-plane packing of quantisation bins (EDEN's wire layout): plane b of 32 consecutive bins
// becomes one 32-bit word built with a warp ballot; planes are stored one after another.
// Counterpart of BinsToBitsKernel / BitsToBinsKernel
// (cuda_kernels/src/srrcomp/eden_utils/csrc/cuda_packing.cu:11-29,76-95).  Here a warp keeps its
// 32 bins in registers and emits all planes, so every bin is read once and every word written once.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

namespace dq {
namespace {

__global__ void __launch_bounds__(256) bins_to_bits_kernel(const uint8_t* __restrict__ bins,
                                                           uint32_t* __restrict__ words, long long n,
                                                           long long nwords, int nbits) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * static_cast<long long>(blockDim.x)) >> 5;
  for (long long wd = warp; wd < nwords; wd += nwarps) {
    const long long i = wd * 32 + lane;
    const uint32_t v = i < n ? bins[i] : 0u;
    for (int b = 0; b < nbits; ++b) {
      const uint32_t word = __ballot_sync(0xFFFFFFFFu, (v >> b) & 1u);
      if (lane == 0) words[static_cast<long long>(b) * nwords + wd] = word;
    }
  }
}

__global__ void __launch_bounds__(256) bits_to_bins_kernel(const uint32_t* __restrict__ words,
                                                           uint8_t* __restrict__ bins, long long n, long long nwords,
                                                           int nbits) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const long long wd = i >> 5;
  const int bit = static_cast<int>(i & 31);
  uint32_t v = 0;
  for (int b = 0; b < nbits; ++b) v |= ((words[static_cast<long long>(b) * nwords + wd] >> bit) & 1u) << b;
  bins[i] = static_cast<uint8_t>(v);
}

}  // namespace

// bins: uint8 [n], values < 2^nbits -> int32 [nbits, ceil(n / 32)]
at::Tensor bins_to_bits(at::Tensor bins, int64_t nbits) {
  TORCH_CHECK(bins.is_cuda() && bins.is_contiguous() && bins.scalar_type() == at::kByte, "bins: contiguous CUDA uint8");
  TORCH_CHECK(nbits >= 1 && nbits <= 8, "nbits must be in 1..8");
  c10::cuda::CUDAGuard guard(bins.device());
  const long long n = bins.numel(), nwords = (n + 31) / 32;
  at::Tensor out = at::empty({nbits, nwords}, bins.options().dtype(at::kInt));
  if (n == 0) return out;
  const int grid = static_cast<int>(std::min<long long>((nwords * 32 + 255) / 256, 148LL * 16));
  bins_to_bits_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      bins.data_ptr<uint8_t>(), reinterpret_cast<uint32_t*>(out.data_ptr<int>()), n, nwords, static_cast<int>(nbits));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

at::Tensor bits_to_bins(at::Tensor words, int64_t nbits, int64_t n) {
  TORCH_CHECK(words.is_cuda() && words.is_contiguous() && words.scalar_type() == at::kInt && words.dim() == 2 &&
                  words.size(0) == nbits && words.size(1) == (n + 31) / 32,
              "words: contiguous CUDA int32 [nbits, ceil(n / 32)]");
  c10::cuda::CUDAGuard guard(words.device());
  at::Tensor out = at::empty({n}, words.options().dtype(at::kByte));
  if (n == 0) return out;
  bits_to_bins_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const uint32_t*>(words.data_ptr<int>()), out.data_ptr<uint8_t>(), n, (n + 31) / 32,
      static_cast<int>(nbits));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

}  // namespace dq
