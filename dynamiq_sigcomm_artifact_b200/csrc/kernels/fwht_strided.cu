// Upper butterfly levels of a Walsh-Hadamard transform longer than 1024.
//
// H_{2^k} = H_{2^(k-10)} (x) H_1024 in Sylvester order: the tcgen05 kernel (fwht_tcgen05.cu) transforms every
// contiguous 1024-block (levels 0..9); this kernel applies levels [first, first + n) - element pairs 2^level
// apart - in one pass over the array, up to five levels (radix 32) at a time held in registers.  With
// first >= 10 consecutive threads touch consecutive addresses, so each pass streams the array once at
// memory speed.  Used by THC's whole-partition rotation (reference: testbed_evaluation/new_comm_hooks/
// thc_hooks.py:124-149, which calls the SIMT Hadamard of cuda_kernels/.../cuda_hadamard.cu:58-251 on
// partitions of up to 2^23 elements).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

namespace dq {
namespace {

template <int LOGR>
__global__ void __launch_bounds__(256) fwht_levels_kernel(float* __restrict__ x, long long n, int first, float scale) {
  constexpr int R = 1 << LOGR;
  const long long stride = 1ll << first;
  const long long nthreads = n >> LOGR;
  for (long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; t < nthreads;
       t += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long inner = t & (stride - 1), outer = t >> first;
    float* base = x + ((outer << (first + LOGR)) + inner);
    float v[R];
#pragma unroll
    for (int j = 0; j < R; ++j) v[j] = base[j * stride];
#pragma unroll
    for (int h = 1; h < R; h <<= 1) {
#pragma unroll
      for (int j = 0; j < R; ++j) {
        if ((j & h) == 0) {
          const float a = v[j], b = v[j | h];
          v[j] = a + b;
          v[j | h] = a - b;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < R; ++j) base[j * stride] = v[j] * scale;
  }
}

}  // namespace

// in place: butterfly levels [first, first + nlevels) of a flat fp32 tensor whose length is a power of two;
// `scale` multiplies the result (1 for an unnormalised transform)
void fwht_levels_(at::Tensor x, int64_t first, int64_t nlevels, double scale) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous(), "fwht_levels_: contiguous CUDA fp32 tensor");
  const long long n = x.numel();
  TORCH_CHECK(n > 0 && (n & (n - 1)) == 0, "fwht_levels_: length must be a power of two, got ", n);
  TORCH_CHECK(nlevels >= 1 && nlevels <= 5 && first >= 0 && (1ll << (first + nlevels)) <= n,
              "fwht_levels_: levels [", first, ", ", first + nlevels, ") outside a transform of length ", n);
  c10::cuda::CUDAGuard guard(x.device());
  const long long nthreads = n >> nlevels;
  const int grid = static_cast<int>(std::min<long long>((nthreads + 255) / 256, 148LL * 16));
  auto stream = at::cuda::getCurrentCUDAStream();
  float* p = x.data_ptr<float>();
  const float s = static_cast<float>(scale);
  const int f = static_cast<int>(first);
  switch (nlevels) {
    case 1: fwht_levels_kernel<1><<<grid, 256, 0, stream>>>(p, n, f, s); break;
    case 2: fwht_levels_kernel<2><<<grid, 256, 0, stream>>>(p, n, f, s); break;
    case 3: fwht_levels_kernel<3><<<grid, 256, 0, stream>>>(p, n, f, s); break;
    case 4: fwht_levels_kernel<4><<<grid, 256, 0, stream>>>(p, n, f, s); break;
    default: fwht_levels_kernel<5><<<grid, 256, 0, stream>>>(p, n, f, s); break;
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace dq
