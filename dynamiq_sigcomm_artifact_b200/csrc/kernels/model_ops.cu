// Model-side hot ops as hand-written sm_100a kernels: LayerNorm, RMSNorm, rotary embedding
// and a multi-tensor fused AdamW.  The reference takes these from Hugging Face modules and
// torch.optim.AdamW (testbed_evaluation/train_llm_causal.py:490-497,614); here each is one
// memory-bound pass with 16-byte accesses, fp32 statistics, and a deterministic two-stage
// reduction for the weight gradients (no atomics on values).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <type_traits>
#include <torch/extension.h>

#include "norm_kernels.cuh"

namespace dq {

namespace {

using namespace normk;

// One warp per row.  RMS = true: y = x * rstd * w;  false: y = (x - mean) * rstd * w + b.
template <typename T, bool RMS>
__global__ void __launch_bounds__(kNormWarps * 32) norm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                                    const float* __restrict__ b, T* __restrict__ y,
                                                                    float* __restrict__ mean, float* __restrict__ rstd,
                                                                    int rows, int H, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int row = blockIdx.x * kNormWarps + warp; row < rows; row += gridDim.x * kNormWarps) {
    const T* xr = x + static_cast<size_t>(row) * H;
    float s = 0.f, ss = 0.f;
    for (int c = lane * 8; c < H; c += 256) {
      float v[8];
      Vec8<T>::load(xr + c, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += v[i], ss += v[i] * v[i];
    }
    s = warp_sum(s), ss = warp_sum(ss);
    const float mu = RMS ? 0.f : s / H;
    const float var = RMS ? ss / H : fmaxf(ss / H - mu * mu, 0.f);
    const float rs = rsqrtf(var + eps);
    if (lane == 0) {
      if (!RMS) mean[row] = mu;
      rstd[row] = rs;
    }
    T* yr = y + static_cast<size_t>(row) * H;
    for (int c = lane * 8; c < H; c += 256) {
      float v[8], g[8], o[8];
      Vec8<T>::load(xr + c, v);
      Vec8<float>::load(w + c, g);
      if (RMS) {
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = v[i] * rs * g[i];
      } else {
        float bb[8];
        Vec8<float>::load(b + c, bb);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (v[i] - mu) * rs * g[i] + bb[i];
      }
      Vec8<T>::store(yr + c, o);
    }
  }
}

// dx for one row per warp, plus per-CTA partial sums of dw (and db) over the CTA's rows.
template <typename T, bool RMS>
__global__ void __launch_bounds__(kNormWarps * 32) norm_bwd_kernel(
    const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ mean,
    const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw_part, float* __restrict__ db_part,
    int rows, int H) {
  extern __shared__ float sm[];  // [2][H] accumulated by the CTA's warps in turn
  float* sdw = sm;
  float* sdb = sm + H;
  for (int c = threadIdx.x; c < (RMS ? H : 2 * H); c += blockDim.x) sm[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rows_per_cta = (rows + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * rows_per_cta, r1 = min(r0 + rows_per_cta, rows);
  for (int base = r0; base < r1; base += kNormWarps) {
    const int row = base + warp;
    const bool active = row < r1;
    float mu = 0.f, rs = 0.f, s1 = 0.f, s2 = 0.f;
    if (active) {
      mu = RMS ? 0.f : mean[row];
      rs = rstd[row];
      const T* xr = x + static_cast<size_t>(row) * H;
      const T* dr = dy + static_cast<size_t>(row) * H;
      for (int c = lane * 8; c < H; c += 256) {
        float v[8], d[8], g[8];
        Vec8<T>::load(xr + c, v);
        Vec8<T>::load(dr + c, d);
        Vec8<float>::load(w + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xhat = (v[i] - mu) * rs, gdy = g[i] * d[i];
          s1 += gdy;
          s2 += gdy * xhat;
        }
      }
      s1 = warp_sum(s1), s2 = warp_sum(s2);
    }
    const float m1 = RMS ? 0.f : s1 / H, m2 = s2 / H;
    // warps take turns adding their row into the CTA's partial sums (deterministic order)
    for (int turn = 0; turn < kNormWarps; ++turn) {
      if (turn == warp && active) {
        const T* xr = x + static_cast<size_t>(row) * H;
        const T* dr = dy + static_cast<size_t>(row) * H;
        T* dxr = dx + static_cast<size_t>(row) * H;
        for (int c = lane * 8; c < H; c += 256) {
          float v[8], d[8], g[8], o[8];
          Vec8<T>::load(xr + c, v);
          Vec8<T>::load(dr + c, d);
          Vec8<float>::load(w + c, g);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float xhat = (v[i] - mu) * rs;
            o[i] = rs * (g[i] * d[i] - m1 - xhat * m2);
            sdw[c + i] += d[i] * xhat;
            if (!RMS) sdb[c + i] += d[i];
          }
          Vec8<T>::store(dxr + c, o);
        }
      }
      __syncthreads();
    }
  }
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    dw_part[static_cast<size_t>(blockIdx.x) * H + c] = sdw[c];
    if (!RMS) db_part[static_cast<size_t>(blockIdx.x) * H + c] = sdb[c];
  }
}


__global__ void reduce_parts_kernel(const float* __restrict__ part, float* __restrict__ out, int nparts, int H) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += part[static_cast<size_t>(p) * H + c];
  out[c] = s;
}

// x: [B, S, nH, D] (contiguous); cos/sin: [S, D/2] fp32.  Rotate-half convention:
// o[:D/2] = x1 cos - x2 sin, o[D/2:] = x2 cos + x1 sin; the backward pass is the same with -sin.
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            T* __restrict__ y, long long total_pairs8, int S, int nH, int D, float sin_sign) {
  const int half = D / 2, groups = half / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total_pairs8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i % groups);
    const long long head = i / groups;  // (b * S + s) * nH + h
    const int s = static_cast<int>((head / nH) % S);
    const T* xp = x + head * D + g * 8;
    float a[8], b[8], c[8], d[8], o1[8], o2[8];
    Vec8<T>::load(xp, a);
    Vec8<T>::load(xp + half, b);
    Vec8<float>::load(cs + static_cast<size_t>(s) * half + g * 8, c);
    Vec8<float>::load(sn + static_cast<size_t>(s) * half + g * 8, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sk = d[k] * sin_sign;
      o1[k] = a[k] * c[k] - b[k] * sk;
      o2[k] = b[k] * c[k] + a[k] * sk;
    }
    T* yp = y + head * D + g * 8;
    Vec8<T>::store(yp, o1);
    Vec8<T>::store(yp + half, o2);
  }
}

// Multi-tensor AdamW (decoupled weight decay), fp32 state.  table[t] = {param, grad, m, v, shadow}
// device addresses (shadow = 0 or a bf16 copy of the parameter that the kernel keeps in step, so that
// no separate cast pass runs before the next forward), numel[t], and chunk_start[t] = first chunk of
// tensor t (chunk = 4096 elements).
constexpr int kAdamChunk = 4096;
constexpr int kAdamCols = 5;
template <typename P, typename G>
__global__ void __launch_bounds__(256) adamw_kernel(const long long* __restrict__ table,
                                                    const long long* __restrict__ numel,
                                                    const int* __restrict__ chunk_start, int ntensors, float lr,
                                                    float beta1, float beta2, float eps, float wd, float bc1,
                                                    float bc2, float grad_scale) {
  const int chunk = blockIdx.x;
  int lo = 0, hi = ntensors - 1;
  while (lo < hi) {  // last tensor whose first chunk is <= chunk
    const int mid = (lo + hi + 1) >> 1;
    if (chunk_start[mid] <= chunk) lo = mid;
    else hi = mid - 1;
  }
  const int t = lo;
  P* p = reinterpret_cast<P*>(table[kAdamCols * t]);
  const G* g = reinterpret_cast<const G*>(table[kAdamCols * t + 1]);
  float* m = reinterpret_cast<float*>(table[kAdamCols * t + 2]);
  float* v = reinterpret_cast<float*>(table[kAdamCols * t + 3]);
  __nv_bfloat16* shadow = reinterpret_cast<__nv_bfloat16*>(table[kAdamCols * t + 4]);
  const long long n = numel[t];
  const long long base = static_cast<long long>(chunk - chunk_start[t]) * kAdamChunk;
  const float step_size = lr / bc1, inv_bc2_sqrt = rsqrtf(bc2);
  auto update = [&](float gi, float& pi, float& mi, float& vi) {
    gi *= grad_scale;
    mi = beta1 * mi + (1.f - beta1) * gi;
    vi = beta2 * vi + (1.f - beta2) * gi * gi;
    pi -= lr * wd * pi;
    pi -= step_size * mi / (sqrtf(vi) * inv_bc2_sqrt + eps);
  };
  if constexpr (std::is_same<P, float>::value && std::is_same<G, float>::value) {
    // fp32 fast path: 16-byte streaming accesses (every array is touched exactly once per step, so none of it
    // should displace the GEMM operands of the backward pass that runs beside this kernel), all loads of a
    // thread's four groups in flight before the arithmetic
    const bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                           reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15u) == 0 &&
                         (reinterpret_cast<uintptr_t>(shadow) & 7u) == 0;
    if (aligned && base + kAdamChunk <= n) {
      constexpr int kGroups = kAdamChunk / 4 / 256;  // float4 groups per thread
      float4 p4[kGroups], g4[kGroups], m4[kGroups], v4[kGroups];
#pragma unroll
      for (int j = 0; j < kGroups; ++j) {
        const long long i = base + 4ll * (threadIdx.x + 256 * j);
        g4[j] = __ldcs(reinterpret_cast<const float4*>(g + i));
        p4[j] = __ldcs(reinterpret_cast<const float4*>(p + i));
        m4[j] = __ldcs(reinterpret_cast<const float4*>(m + i));
        v4[j] = __ldcs(reinterpret_cast<const float4*>(v + i));
      }
#pragma unroll
      for (int j = 0; j < kGroups; ++j) {
        const long long i = base + 4ll * (threadIdx.x + 256 * j);
        update(g4[j].x, p4[j].x, m4[j].x, v4[j].x);
        update(g4[j].y, p4[j].y, m4[j].y, v4[j].y);
        update(g4[j].z, p4[j].z, m4[j].z, v4[j].z);
        update(g4[j].w, p4[j].w, m4[j].w, v4[j].w);
        __stcs(reinterpret_cast<float4*>(m + i), m4[j]);
        __stcs(reinterpret_cast<float4*>(v + i), v4[j]);
        __stcs(reinterpret_cast<float4*>(p + i), p4[j]);
        if (shadow != nullptr) {
          const __nv_bfloat162 lo = __floats2bfloat162_rn(p4[j].x, p4[j].y), hi = __floats2bfloat162_rn(p4[j].z, p4[j].w);
          uint2 packed;
          packed.x = *reinterpret_cast<const unsigned int*>(&lo);
          packed.y = *reinterpret_cast<const unsigned int*>(&hi);
          *reinterpret_cast<uint2*>(shadow + i) = packed;
        }
      }
      return;
    }
  }
#pragma unroll 4
  for (int k = threadIdx.x; k < kAdamChunk; k += 256) {
    const long long i = base + k;
    if (i >= n) break;
    float pi = to_f(p[i]), mi = m[i], vi = v[i];
    update(to_f(g[i]), pi, mi, vi);
    m[i] = mi;
    v[i] = vi;
    p[i] = from_f<P>(pi);
    if (shadow != nullptr) shadow[i] = __float2bfloat16_rn(pi);
  }
}

// SwiGLU: in [rows, 2 I] = (gate | up), out [rows, I] = silu(gate) * up; eight elements per thread.
template <typename T>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const T* __restrict__ in, T* __restrict__ out, long long rows,
                                                         int inner) {
  const int groups = inner / 8;
  const long long total = rows * groups;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / groups;
    const int c = static_cast<int>(i % groups) * 8;
    float g[8], u[8], o[8];
    Vec8<T>::load(in + r * 2 * inner + c, g);
    Vec8<T>::load(in + r * 2 * inner + inner + c, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    Vec8<T>::store(out + r * inner + c, o);
  }
}

// din = (dy * up * d silu(gate) | dy * silu(gate))
template <typename T>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ in,
                                                         T* __restrict__ din, long long rows, int inner) {
  const int groups = inner / 8;
  const long long total = rows * groups;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / groups;
    const int c = static_cast<int>(i % groups) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    Vec8<T>::load(in + r * 2 * inner + c, g);
    Vec8<T>::load(in + r * 2 * inner + inner + c, u);
    Vec8<T>::load(dy + r * inner + c, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sg = 1.f / (1.f + __expf(-g[k]));
      du[k] = d[k] * g[k] * sg;
      dg[k] = d[k] * u[k] * sg * (1.f + g[k] * (1.f - sg));
    }
    Vec8<T>::store(din + r * 2 * inner + c, dg);
    Vec8<T>::store(din + r * 2 * inner + inner + c, du);
  }
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

void check_norm_inputs(const at::Tensor& x, const at::Tensor& w) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "norm: x must be a contiguous CUDA tensor");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat, "norm: bf16 or fp32 activations");
  TORCH_CHECK(w.scalar_type() == at::kFloat && w.is_contiguous(), "norm: fp32 weight");
  const int64_t H = x.size(-1);
  TORCH_CHECK(H % 8 == 0 && w.numel() == H, "norm: hidden size must be a multiple of 8 and match the weight");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "norm: x must be 16-byte aligned");
}

}  // namespace

// returns (y, mean, rstd); mean is empty for RMSNorm
std::tuple<at::Tensor, at::Tensor, at::Tensor> norm_fwd(at::Tensor x, at::Tensor w, c10::optional<at::Tensor> b,
                                                        double eps, bool rms) {
  check_norm_inputs(x, w);
  c10::cuda::CUDAGuard guard(x.device());
  const int H = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / H);
  at::Tensor y = at::empty_like(x);
  auto fopt = x.options().dtype(at::kFloat);
  at::Tensor mean = at::empty({rms ? 0 : rows}, fopt), rstd = at::empty({rows}, fopt);
  TORCH_CHECK(rms || (b.has_value() && b->scalar_type() == at::kFloat && b->numel() == H), "layernorm needs an fp32 bias");
  const int grid = std::max(1, std::min((rows + kNormWarps - 1) / kNormWarps, sm_count() * 8));
  auto stream = at::cuda::getCurrentCUDAStream();
  const float* bp = rms ? nullptr : b->data_ptr<float>();
#define DQ_LAUNCH(T, RMS)                                                                                           \
  norm_fwd_kernel<T, RMS><<<grid, kNormWarps * 32, 0, stream>>>(reinterpret_cast<const T*>(x.data_ptr()),          \
                                                                 w.data_ptr<float>(), bp, reinterpret_cast<T*>(y.data_ptr()), \
                                                                 rms ? nullptr : mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, H, static_cast<float>(eps))
  if (x.scalar_type() == at::kBFloat16) {
    if (rms) DQ_LAUNCH(__nv_bfloat16, true);
    else DQ_LAUNCH(__nv_bfloat16, false);
  } else {
    if (rms) DQ_LAUNCH(float, true);
    else DQ_LAUNCH(float, false);
  }
#undef DQ_LAUNCH
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, mean, rstd};
}

// returns (dx, dw, db); db is empty for RMSNorm
// `dw_out` / `db_out` (fp32 [H], optional): where the weight / bias gradient is written instead of a new tensor
std::tuple<at::Tensor, at::Tensor, at::Tensor> norm_bwd(at::Tensor dy, at::Tensor x, at::Tensor w, at::Tensor mean,
                                                        at::Tensor rstd, bool rms, c10::optional<at::Tensor> dw_out,
                                                        c10::optional<at::Tensor> db_out) {
  check_norm_inputs(x, w);
  TORCH_CHECK(dy.is_contiguous() && dy.scalar_type() == x.scalar_type() && dy.numel() == x.numel(), "norm_bwd: dy/x mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  const int H = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / H);
  at::Tensor dx = at::empty_like(x);
  auto fopt = x.options().dtype(at::kFloat);
  auto stream = at::cuda::getCurrentCUDAStream();
  auto usable = [&](const c10::optional<at::Tensor>& t) {
    if (!t.has_value()) return false;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == H,
                "norm_bwd: an output gradient must be a contiguous CUDA fp32 tensor of H elements");
    return true;
  };
  at::Tensor dw = usable(dw_out) ? *dw_out : at::empty({H}, fopt);
  at::Tensor db = rms ? at::empty({0}, fopt) : (usable(db_out) ? *db_out : at::empty({H}, fopt));
  if (H <= 2048) {
    const int grid = std::max(1, std::min((rows + kNormWarps - 1) / kNormWarps, 2 * sm_count()));
    const int nparts = grid * kNormWarps;
    at::Tensor dw_part = at::empty({nparts, H}, fopt), db_part = at::empty({rms ? 0 : nparts, H}, fopt);
    const int nchunk = (H + 255) / 256;
#define DQ_ROWS(T, RMS, NC)                                                                                        \
  norm_bwd_rows_kernel<T, RMS, NC><<<grid, kNormWarps * 32, 0, stream>>>(                                          \
      reinterpret_cast<const T*>(dy.data_ptr()), reinterpret_cast<const T*>(x.data_ptr()), w.data_ptr<float>(),    \
      rms ? nullptr : mean.data_ptr<float>(), rstd.data_ptr<float>(), reinterpret_cast<T*>(dx.data_ptr()),         \
      dw_part.data_ptr<float>(), rms ? nullptr : db_part.data_ptr<float>(), rows, H)
#define DQ_ROWS_NC(T, RMS)                                 \
  switch (nchunk) {                                        \
    case 1: DQ_ROWS(T, RMS, 1); break;                     \
    case 2: DQ_ROWS(T, RMS, 2); break;                     \
    case 3: DQ_ROWS(T, RMS, 3); break;                     \
    case 4: DQ_ROWS(T, RMS, 4); break;                     \
    case 5: case 6: DQ_ROWS(T, RMS, 6); break;             \
    default: DQ_ROWS(T, RMS, 8); break;                    \
  }
    if (x.scalar_type() == at::kBFloat16) {
      if (rms) { DQ_ROWS_NC(__nv_bfloat16, true) } else { DQ_ROWS_NC(__nv_bfloat16, false) }
    } else {
      if (rms) { DQ_ROWS_NC(float, true) } else { DQ_ROWS_NC(float, false) }
    }
#undef DQ_ROWS_NC
#undef DQ_ROWS
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    dim3 rb(32, 32);
    if (rms)
      reduce_parts2_kernel<<<(H + 31) / 32, rb, 0, stream>>>(dw_part.data_ptr<float>(), dw.data_ptr<float>(), nparts, H);
    else
      reduce_parts2_pair_kernel<<<dim3((H + 31) / 32, 2), rb, 0, stream>>>(dw_part.data_ptr<float>(), dw.data_ptr<float>(),
                                                                           db_part.data_ptr<float>(), db.data_ptr<float>(),
                                                                           nparts, H);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {dx, dw, db};
  }
  const int grid = std::max(1, std::min((rows + kNormWarps - 1) / kNormWarps, sm_count() * 2));
  at::Tensor dw_part = at::empty({grid, H}, fopt), db_part = at::empty({rms ? 0 : grid, H}, fopt);
  const size_t smem = static_cast<size_t>(rms ? 1 : 2) * H * sizeof(float);
#define DQ_LAUNCH(T, RMS)                                                                                          \
  do {                                                                                                             \
    C10_CUDA_CHECK(cudaFuncSetAttribute(norm_bwd_kernel<T, RMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))); \
    norm_bwd_kernel<T, RMS><<<grid, kNormWarps * 32, smem, stream>>>(                                              \
        reinterpret_cast<const T*>(dy.data_ptr()), reinterpret_cast<const T*>(x.data_ptr()), w.data_ptr<float>(),  \
        rms ? nullptr : mean.data_ptr<float>(), rstd.data_ptr<float>(), reinterpret_cast<T*>(dx.data_ptr()),       \
        dw_part.data_ptr<float>(), rms ? nullptr : db_part.data_ptr<float>(), rows, H);                            \
  } while (0)
  if (x.scalar_type() == at::kBFloat16) {
    if (rms) DQ_LAUNCH(__nv_bfloat16, true);
    else DQ_LAUNCH(__nv_bfloat16, false);
  } else {
    if (rms) DQ_LAUNCH(float, true);
    else DQ_LAUNCH(float, false);
  }
#undef DQ_LAUNCH
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  reduce_parts_kernel<<<(H + 255) / 256, 256, 0, stream>>>(dw_part.data_ptr<float>(), dw.data_ptr<float>(), grid, H);
  if (!rms) reduce_parts_kernel<<<(H + 255) / 256, 256, 0, stream>>>(db_part.data_ptr<float>(), db.data_ptr<float>(), grid, H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dx, dw, db};
}

at::Tensor swiglu_fwd(at::Tensor in) {
  TORCH_CHECK(in.is_cuda() && in.is_contiguous() && in.dim() >= 1 && in.size(-1) % 16 == 0,
              "swiglu: contiguous CUDA tensor whose last dimension (2 I) is a multiple of 16");
  TORCH_CHECK(in.scalar_type() == at::kBFloat16 || in.scalar_type() == at::kFloat, "swiglu: bf16 or fp32");
  c10::cuda::CUDAGuard guard(in.device());
  const int inner = static_cast<int>(in.size(-1) / 2);
  const long long rows = in.numel() / (2 * inner);
  auto shape = in.sizes().vec();
  shape.back() = inner;
  at::Tensor out = at::empty(shape, in.options());
  const long long total = rows * (inner / 8);
  const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((total + 255) / 256, sm_count() * 16LL)));
  auto stream = at::cuda::getCurrentCUDAStream();
  if (in.scalar_type() == at::kBFloat16)
    swiglu_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(in.data_ptr()), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), rows, inner);
  else
    swiglu_fwd_kernel<float><<<grid, 256, 0, stream>>>(in.data_ptr<float>(), out.data_ptr<float>(), rows, inner);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

at::Tensor swiglu_bwd(at::Tensor dy, at::Tensor in) {
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && in.is_contiguous() && dy.scalar_type() == in.scalar_type() &&
                  dy.numel() * 2 == in.numel(), "swiglu_bwd: dy [.., I] and in [.., 2 I] must be contiguous and agree");
  c10::cuda::CUDAGuard guard(in.device());
  const int inner = static_cast<int>(in.size(-1) / 2);
  const long long rows = in.numel() / (2 * inner);
  at::Tensor din = at::empty_like(in);
  const long long total = rows * (inner / 8);
  const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((total + 255) / 256, sm_count() * 16LL)));
  auto stream = at::cuda::getCurrentCUDAStream();
  if (in.scalar_type() == at::kBFloat16)
    swiglu_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(in.data_ptr()), reinterpret_cast<__nv_bfloat16*>(din.data_ptr()), rows, inner);
  else
    swiglu_bwd_kernel<float><<<grid, 256, 0, stream>>>(dy.data_ptr<float>(), in.data_ptr<float>(), din.data_ptr<float>(), rows, inner);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return din;
}

at::Tensor rope(at::Tensor x, at::Tensor cos, at::Tensor sin, bool backward) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 4, "rope: x must be contiguous [B, S, heads, D]");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat, "rope: bf16 or fp32");
  const int S = static_cast<int>(x.size(1)), nH = static_cast<int>(x.size(2)), D = static_cast<int>(x.size(3));
  TORCH_CHECK(D % 16 == 0, "rope: head dim must be a multiple of 16");
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.is_contiguous() &&
                  sin.is_contiguous() && cos.size(0) >= S && cos.size(1) == D / 2 && sin.size(0) >= S && sin.size(1) == D / 2,
              "rope: cos/sin must be fp32 [S, D/2]");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty_like(x);
  const long long total = x.numel() / D * (D / 16);
  const int threads = 256;
  const int grid = static_cast<int>(std::min<long long>((total + threads - 1) / threads, sm_count() * 16LL));
  auto stream = at::cuda::getCurrentCUDAStream();
  const float sgn = backward ? -1.f : 1.f;
  if (x.scalar_type() == at::kBFloat16)
    rope_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), cos.data_ptr<float>(), sin.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), total, S, nH, D, sgn);
  else
    rope_kernel<float><<<grid, threads, 0, stream>>>(x.data_ptr<float>(), cos.data_ptr<float>(), sin.data_ptr<float>(), y.data_ptr<float>(), total, S, nH, D, sgn);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return y;
}

// table: int64 [T, 5] device tensor of addresses (param, grad, m, v, bf16 shadow or 0); numel: int64 [T] device; chunk_start: int32 [T] device.
void adamw_step(at::Tensor table, at::Tensor numel, at::Tensor chunk_start, int64_t total_chunks, bool param_bf16,
                bool grad_bf16, double lr, double beta1, double beta2, double eps, double weight_decay, int64_t step,
                double grad_scale) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.dim() == 2 && table.size(1) == kAdamCols, "adamw: bad table");
  TORCH_CHECK(numel.is_cuda() && numel.scalar_type() == at::kLong && chunk_start.is_cuda() && chunk_start.scalar_type() == at::kInt, "adamw: bad metadata");
  if (total_chunks == 0) return;
  c10::cuda::CUDAGuard guard(table.device());
  const int T = static_cast<int>(table.size(0));
  const float bc1 = static_cast<float>(1.0 - std::pow(beta1, static_cast<double>(step)));
  const float bc2 = static_cast<float>(1.0 - std::pow(beta2, static_cast<double>(step)));
  auto stream = at::cuda::getCurrentCUDAStream();
#define DQ_LAUNCH(P, G)                                                                                              \
  adamw_kernel<P, G><<<static_cast<unsigned>(total_chunks), 256, 0, stream>>>(                                      \
      reinterpret_cast<const long long*>(table.data_ptr<int64_t>()), reinterpret_cast<const long long*>(numel.data_ptr<int64_t>()), \
      chunk_start.data_ptr<int>(), T, static_cast<float>(lr), static_cast<float>(beta1), static_cast<float>(beta2), \
      static_cast<float>(eps), static_cast<float>(weight_decay), bc1, bc2, static_cast<float>(grad_scale))
  if (param_bf16 && grad_bf16) DQ_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (param_bf16) DQ_LAUNCH(__nv_bfloat16, float);
  else if (grad_bf16) DQ_LAUNCH(float, __nv_bfloat16);
  else DQ_LAUNCH(float, float);
#undef DQ_LAUNCH
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace dq
