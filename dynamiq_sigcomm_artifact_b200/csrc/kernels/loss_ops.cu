// Fused softmax cross-entropy over (padded) vocabulary logits, forward and backward.
//
// The reference gets its loss from the Hugging Face model's forward
// (testbed_evaluation/train_llm_causal.py:367-369), i.e. an fp32 up-cast of the logits,
// log_softmax, nll_loss and their separate backward kernels.  Here one CTA owns one row:
// the forward reads the bf16/fp32 logits once (online max / sum-exp) and emits the row's
// log-sum-exp and loss; the backward overwrites the logits in place with
// (softmax - onehot) * grad / n_valid.  Columns >= `vocab` are padding (the logits matrix is
// padded so that the projection GEMM has aligned leading dimensions): they are ignored by the
// forward and receive a zero gradient.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <torch/extension.h>

namespace dq {
namespace {

constexpr int kCeThreads = 512;
constexpr unsigned kFull = 0xFFFFFFFFu;

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&o)[8]);
template <>
__device__ __forceinline__ void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = __uint_as_float(w[i] << 16);
    o[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
template <>
__device__ __forceinline__ void ld8<float>(const float* p, float (&o)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x, o[1] = a.y, o[2] = a.z, o[3] = a.w, o[4] = b.x, o[5] = b.y, o[6] = b.z, o[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&o)[8]);
template <>
__device__ __forceinline__ void st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&o)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ void st8<float>(float* p, const float (&o)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(o[4], o[5], o[6], o[7]);
}
__device__ __forceinline__ float elem_to_float(float x) { return x; }
__device__ __forceinline__ float elem_to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

// combine two (max, sum-exp) pairs
__device__ __forceinline__ void merge(float& m, float& s, float m2, float s2) {
  const float mn = fmaxf(m, m2);
  if (mn == -INFINITY) {  // both sides empty (threads past the end of a short row)
    s = 0.f;
    return;
  }
  s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
  m = mn;
}

template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_fwd_kernel(const T* __restrict__ logits,
                                                            const long long* __restrict__ labels,
                                                            float* __restrict__ lse, float* __restrict__ loss_rows,
                                                            int vocab, long long stride, long long ignore_index) {
  const long long row = blockIdx.x;
  const T* x = logits + row * stride;
  const long long label = labels[row];
  if (label == ignore_index) {  // CTA-uniform
    if (threadIdx.x == 0) lse[row] = 0.f, loss_rows[row] = 0.f;
    return;
  }
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x * 8; c < vocab; c += kCeThreads * 8) {
    float v[8];
    ld8<T>(x + c, v);
    float lm = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (c + i >= vocab) v[i] = -INFINITY;
      lm = fmaxf(lm, v[i]);
    }
    const float mn = fmaxf(m, lm);
    float acc = s * __expf(m - mn);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += __expf(v[i] - mn);
    m = mn, s = acc;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(kFull, m, o), s2 = __shfl_xor_sync(kFull, s, o);
    merge(m, s, m2, s2);
  }
  __shared__ float sm[kCeThreads / 32], ss[kCeThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sm[warp] = m, ss[warp] = s;
  __syncthreads();
  if (warp == 0) {
    m = lane < kCeThreads / 32 ? sm[lane] : -INFINITY;
    s = lane < kCeThreads / 32 ? ss[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(kFull, m, o), s2 = __shfl_xor_sync(kFull, s, o);
      merge(m, s, m2, s2);
    }
    if (lane == 0) {
      const float l = m + logf(s);
      lse[row] = l;
      loss_rows[row] = l - elem_to_float(x[label]);
    }
  }
}

// logits <- (softmax(logits) - onehot(label)) * gout / n_valid, in place; padding and ignored rows <- 0
template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_bwd_kernel(T* __restrict__ logits,
                                                            const long long* __restrict__ labels,
                                                            const float* __restrict__ lse,
                                                            const float* __restrict__ gout,
                                                            const float* __restrict__ n_valid, int vocab,
                                                            long long stride, long long ignore_index) {
  const long long row = blockIdx.x;
  T* x = logits + row * stride;
  const long long label = labels[row];
  const bool ignored = label == ignore_index;
  const float scale = ignored ? 0.f : gout[0] / fmaxf(n_valid[0], 1.f);
  const float l = lse[row];
  for (int c = threadIdx.x * 8; c < stride; c += kCeThreads * 8) {
    float v[8];
    if (ignored) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    } else {
      ld8<T>(x + c, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int col = c + i;
        const float p = col < vocab ? __expf(v[i] - l) : 0.f;
        v[i] = (p - (col == label ? 1.f : 0.f)) * scale;
      }
    }
    st8<T>(x + c, v);
  }
}

}  // namespace

// logits [N, stride] (row-major, stride % 8 == 0), labels [N] int64.  Returns (lse [N], loss_rows [N]).
std::tuple<at::Tensor, at::Tensor> ce_fwd(at::Tensor logits, at::Tensor labels, int64_t vocab, int64_t ignore_index) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous(), "ce: logits must be contiguous [N, Vp]");
  TORCH_CHECK(logits.scalar_type() == at::kBFloat16 || logits.scalar_type() == at::kFloat, "ce: bf16 or fp32 logits");
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == at::kLong && labels.is_contiguous() &&
                  labels.numel() == logits.size(0), "ce: labels must be int64 [N]");
  const int64_t N = logits.size(0), stride = logits.size(1);
  TORCH_CHECK(stride % 8 == 0 && vocab <= stride && vocab > 0, "ce: padded width must be a multiple of 8 and >= vocab");
  c10::cuda::CUDAGuard guard(logits.device());
  auto fopt = logits.options().dtype(at::kFloat);
  at::Tensor lse = at::empty({N}, fopt), rows = at::empty({N}, fopt);
  if (N == 0) return {lse, rows};
  auto stream = at::cuda::getCurrentCUDAStream();
  if (logits.scalar_type() == at::kBFloat16)
    ce_fwd_kernel<__nv_bfloat16><<<static_cast<unsigned>(N), kCeThreads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits.data_ptr()), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
        lse.data_ptr<float>(), rows.data_ptr<float>(), static_cast<int>(vocab), stride, ignore_index);
  else
    ce_fwd_kernel<float><<<static_cast<unsigned>(N), kCeThreads, 0, stream>>>(
        logits.data_ptr<float>(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), lse.data_ptr<float>(),
        rows.data_ptr<float>(), static_cast<int>(vocab), stride, ignore_index);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {lse, rows};
}

// Overwrites `logits` with its gradient and returns it.  gout, n_valid: one-element fp32 CUDA tensors.
at::Tensor ce_bwd(at::Tensor logits, at::Tensor labels, at::Tensor lse, at::Tensor gout, at::Tensor n_valid,
                  int64_t vocab, int64_t ignore_index) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous(), "ce: logits must be contiguous [N, Vp]");
  TORCH_CHECK(gout.is_cuda() && gout.scalar_type() == at::kFloat && gout.numel() == 1 && n_valid.is_cuda() &&
                  n_valid.scalar_type() == at::kFloat && n_valid.numel() == 1, "ce: gout / n_valid must be fp32 scalars on the device");
  const int64_t N = logits.size(0), stride = logits.size(1);
  if (N == 0) return logits;
  c10::cuda::CUDAGuard guard(logits.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  if (logits.scalar_type() == at::kBFloat16)
    ce_bwd_kernel<__nv_bfloat16><<<static_cast<unsigned>(N), kCeThreads, 0, stream>>>(
        reinterpret_cast<__nv_bfloat16*>(logits.data_ptr()), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
        lse.data_ptr<float>(), gout.data_ptr<float>(), n_valid.data_ptr<float>(), static_cast<int>(vocab), stride, ignore_index);
  else
    ce_bwd_kernel<float><<<static_cast<unsigned>(N), kCeThreads, 0, stream>>>(
        logits.data_ptr<float>(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), lse.data_ptr<float>(),
        gout.data_ptr<float>(), n_valid.data_ptr<float>(), static_cast<int>(vocab), stride, ignore_index);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return logits;
}

}  // namespace dq
