// Column sums of a row-major [rows, cols] bf16 / fp32 matrix in fp32: the bias gradient of a linear layer.
//
// The library reduction spends ~21 us on an [8192, 768] bf16 matrix that the previous kernel has just left
// in L2; this two-stage form (per-CTA partial sums over a slab of rows, then a deterministic sum of the
// partials) reads every element once with 8-byte loads and finishes in a few microseconds.  The reference
// leaves bias gradients to autograd (Hugging Face nn.Linear, testbed_evaluation/train_llm_causal.py:490-497).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <torch/extension.h>

namespace dq {
namespace {

constexpr int kTileCols = 128;  // one warp row: 32 lanes x 4 columns
constexpr int kWarps = 8;

__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  v[0] = __low2float(a), v[1] = __high2float(a), v[2] = __low2float(b), v[3] = __high2float(b);
}
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 raw = *reinterpret_cast<const float4*>(p);
  v[0] = raw.x, v[1] = raw.y, v[2] = raw.z, v[3] = raw.w;
}

// grid (col tiles, row splits); partial[split, cols]
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) colsum_partial_kernel(const T* __restrict__ x, float* __restrict__ partial,
                                                                    long long rows, int cols, int rows_per_split) {
  __shared__ float sm[kWarps][kTileCols];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * kTileCols + lane * 4;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_split;
  const long long r1 = min(rows, r0 + rows_per_split);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (c0 + 3 < cols) {  // cols is a multiple of 4: a lane's four columns are all inside or all outside
    for (long long r = r0 + warp; r < r1; r += kWarps) {
      float v[4];
      load4(x + r * cols + c0, v);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] += v[k];
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) sm[warp][lane * 4 + k] = acc[k];
  __syncthreads();
  if (threadIdx.x < kTileCols) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) s += sm[w][threadIdx.x];
    const int c = blockIdx.x * kTileCols + threadIdx.x;
    if (c < cols) partial[static_cast<long long>(blockIdx.y) * cols + c] = s;
  }
}

__global__ void __launch_bounds__(256) colsum_final_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                           int cols, int splits) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int i = 0; i < splits; ++i) s += partial[static_cast<long long>(i) * cols + c];
  out[c] = s;
}

}  // namespace

// x [rows, cols] (bf16 / fp32, contiguous); out: fp32 [cols], written in place when given
at::Tensor colsum(at::Tensor x, c10::optional<at::Tensor> out) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2, "colsum: contiguous 2-D CUDA tensor");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat, "colsum: bf16 or fp32 input");
  c10::cuda::CUDAGuard guard(x.device());
  const long long rows = x.size(0);
  const int cols = static_cast<int>(x.size(1));
  at::Tensor result = out.has_value() ? *out : at::empty({cols}, x.options().dtype(at::kFloat));
  TORCH_CHECK(result.is_cuda() && result.scalar_type() == at::kFloat && result.is_contiguous() && result.numel() == cols,
              "colsum: out must be a contiguous CUDA fp32 tensor of `cols` elements");
  if (cols == 0) return result;
  if (rows == 0) return result.zero_();
  const int tiles = (cols + kTileCols - 1) / kTileCols;
  // enough CTAs to fill the GPU a few times over, at least 32 rows each
  int splits = static_cast<int>(std::max<long long>(1, std::min<long long>(rows / 32, (148LL * 4 + tiles - 1) / tiles)));
  const int rows_per_split = static_cast<int>((rows + splits - 1) / splits);
  splits = static_cast<int>((rows + rows_per_split - 1) / rows_per_split);
  TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "colsum: input must be 16-byte aligned");
  at::Tensor partial = at::empty({splits, cols}, result.options());
  auto stream = at::cuda::getCurrentCUDAStream();
  dim3 grid(tiles, splits);
  if (x.scalar_type() == at::kBFloat16) {
    TORCH_CHECK(cols % 4 == 0, "colsum: bf16 input needs a column count that is a multiple of 4");
    colsum_partial_kernel<__nv_bfloat16><<<grid, kWarps * 32, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), partial.data_ptr<float>(), rows, cols, rows_per_split);
  } else {
    TORCH_CHECK(cols % 4 == 0, "colsum: fp32 input needs a column count that is a multiple of 4");
    colsum_partial_kernel<float><<<grid, kWarps * 32, 0, stream>>>(x.data_ptr<float>(), partial.data_ptr<float>(), rows, cols,
                                                                  rows_per_split);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  colsum_final_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(partial.data_ptr<float>(), result.data_ptr<float>(), cols, splits);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return result;
}

}  // namespace dq

// ---- deterministic row scatter-add: grad[ids[k], :] += scale * rows[k, :] ------------------------------------
// `order` sorts the ids (stable); CTA k works only if position k starts a run of equal ids and then adds the
// run's rows in sorted order, so every output row has one writer and a fixed summation order: ranks that hold
// the same (ids, rows) produce the same bits.  Used for the embedding-lookup part of a tied embedding's
// gradient, which is exchanged as token rows instead of a dense vocabulary-sized matrix.
namespace dq {
namespace {

__global__ void __launch_bounds__(256) scatter_add_rows_kernel(float* __restrict__ grad, const long long* __restrict__ ids,
                                                               const long long* __restrict__ order,
                                                               const __nv_bfloat16* __restrict__ rows, long long n, int d,
                                                               long long nrows_out, float scale) {
  const long long k = blockIdx.x;
  const long long id = ids[order[k]];
  if (k > 0 && ids[order[k - 1]] == id) return;  // not the start of a run
  if (id < 0 || id >= nrows_out) return;          // never write outside the matrix
  for (int c = threadIdx.x * 4; c < d; c += 256 * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (long long j = k; j < n && ids[order[j]] == id; ++j) {
      float v[4];
      load4(rows + order[j] * d + c, v);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] += v[i];
    }
    float4* dst = reinterpret_cast<float4*>(grad + id * d + c);
    float4 g = *dst;
    g.x += scale * acc[0], g.y += scale * acc[1], g.z += scale * acc[2], g.w += scale * acc[3];
    *dst = g;
  }
}

}  // namespace

// grad [V, d] fp32 (in place), ids [n] int64, rows [n, d] bf16
void scatter_add_rows(at::Tensor grad, at::Tensor ids, at::Tensor rows, double scale) {
  TORCH_CHECK(grad.is_cuda() && grad.scalar_type() == at::kFloat && grad.is_contiguous() && grad.dim() == 2,
              "scatter_add_rows: grad must be a contiguous CUDA fp32 matrix");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && ids.dim() == 1,
              "scatter_add_rows: ids must be a contiguous CUDA int64 vector");
  TORCH_CHECK(rows.is_cuda() && rows.scalar_type() == at::kBFloat16 && rows.is_contiguous() && rows.dim() == 2 &&
                  rows.size(0) == ids.size(0) && rows.size(1) == grad.size(1),
              "scatter_add_rows: rows must be a contiguous CUDA bf16 [n, d] matrix");
  const long long n = ids.numel();
  const int d = static_cast<int>(grad.size(1));
  TORCH_CHECK(d % 4 == 0, "scatter_add_rows: row length must be a multiple of 4");
  if (n == 0) return;
  c10::cuda::CUDAGuard guard(grad.device());
  at::Tensor order = at::argsort(ids, /*stable=*/true, /*dim=*/0, /*descending=*/false);
  scatter_add_rows_kernel<<<static_cast<unsigned>(n), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      grad.data_ptr<float>(), reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()),
      reinterpret_cast<const long long*>(order.data_ptr<int64_t>()),
      reinterpret_cast<const __nv_bfloat16*>(rows.data_ptr()), n, d, grad.size(0), static_cast<float>(scale));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace dq
