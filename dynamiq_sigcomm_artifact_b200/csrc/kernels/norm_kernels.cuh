// Kernel templates of the normalisation backward pass shared by the operator in model_ops.cu
// and the allocation-free C entry point in norm_bwd_noalloc.cu.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace dq {
namespace normk {

constexpr unsigned kFull = 0xFFFFFFFFu;

template <typename T>
struct Vec8;  // 8 elements = 16 bytes for bf16, 32 bytes for float (two float4)
template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&o)[8]) {
    uint4 q = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&o)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&o)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x, o[1] = a.y, o[2] = a.z, o[3] = a.w, o[4] = b.x, o[5] = b.y, o[6] = b.z, o[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&o)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(o[4], o[5], o[6], o[7]);
  }
};

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename P>
__device__ __forceinline__ P from_f(float x);
template <>
__device__ __forceinline__ float from_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}

constexpr int kNormWarps = 8;


// Fast path for H <= 2048: lane owns columns lane*8 + 256*i.  Each warp walks its rows once for
// the row statistics and once more (L1-resident) for dx, accumulating its share of dw / db in
// registers; per-warp partial sums go to dw_part[warp] and are reduced by a second kernel in a
// fixed order.
template <typename T, bool RMS, int NCHUNK>
__global__ void __launch_bounds__(kNormWarps * 32) norm_bwd_rows_kernel(
    const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ mean,
    const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw_part, float* __restrict__ db_part,
    int rows, int H) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gw = blockIdx.x * kNormWarps + warp, nw = gridDim.x * kNormWarps;
  float adw[NCHUNK][8], adb[RMS ? 1 : NCHUNK][8];
#pragma unroll
  for (int i = 0; i < NCHUNK; ++i)
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      adw[i][k] = 0.f;
      if (!RMS) adb[i][k] = 0.f;
    }
  for (int row = gw; row < rows; row += nw) {
    const T* xr = x + static_cast<size_t>(row) * H;
    const T* dr = dy + static_cast<size_t>(row) * H;
    const float mu = RMS ? 0.f : mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
      const int c = lane * 8 + 256 * i;
      if (c < H) {
        float v[8], d[8], g[8];
        Vec8<T>::load(xr + c, v);
        Vec8<T>::load(dr + c, d);
        Vec8<float>::load(w + c, g);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float gdy = g[k] * d[k];
          s1 += gdy;
          s2 += gdy * (v[k] - mu) * rs;
        }
      }
    }
    s1 = warp_sum(s1), s2 = warp_sum(s2);
    const float m1 = RMS ? 0.f : s1 / H, m2 = s2 / H;
    T* dxr = dx + static_cast<size_t>(row) * H;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
      const int c = lane * 8 + 256 * i;
      if (c < H) {
        float v[8], d[8], g[8], o[8];
        Vec8<T>::load(xr + c, v);
        Vec8<T>::load(dr + c, d);
        Vec8<float>::load(w + c, g);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float xhat = (v[k] - mu) * rs;
          o[k] = rs * (g[k] * d[k] - m1 - xhat * m2);
          adw[i][k] += d[k] * xhat;
          if (!RMS) adb[i][k] += d[k];
        }
        Vec8<T>::store(dxr + c, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NCHUNK; ++i) {
    const int c = lane * 8 + 256 * i;
    if (c < H) {
      Vec8<float>::store(dw_part + static_cast<size_t>(gw) * H + c, adw[i]);
      if (!RMS) Vec8<float>::store(db_part + static_cast<size_t>(gw) * H + c, adb[i]);
    }
  }
}

// out[c] = sum over parts; 32 row-groups per CTA (block 32 x 32) combined through shared memory in a
// fixed order, so the result does not depend on scheduling
static __global__ void __launch_bounds__(1024) reduce_parts2_kernel(const float* __restrict__ part,
                                                                    float* __restrict__ out, int nparts, int H) {
  __shared__ float sm[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x, g = threadIdx.y;
  float s = 0.f;
  if (c < H)
    for (int p = g; p < nparts; p += 32) s += part[static_cast<size_t>(p) * H + c];
  sm[g][threadIdx.x] = s;
  __syncthreads();
  if (g == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += sm[k][threadIdx.x];
    out[c] = t;
  }
}

// the same reduction for two partial-sum arrays (weight and bias gradient) in one launch: blockIdx.y picks the pair
static __global__ void __launch_bounds__(1024) reduce_parts2_pair_kernel(const float* __restrict__ part_a,
                                                                         float* __restrict__ out_a,
                                                                         const float* __restrict__ part_b,
                                                                         float* __restrict__ out_b, int nparts, int H) {
  __shared__ float sm[32][33];
  const float* part = blockIdx.y == 0 ? part_a : part_b;
  float* out = blockIdx.y == 0 ? out_a : out_b;
  const int c = blockIdx.x * 32 + threadIdx.x, g = threadIdx.y;
  float s = 0.f;
  if (c < H)
    for (int p = g; p < nparts; p += 32) s += part[static_cast<size_t>(p) * H + c];
  sm[g][threadIdx.x] = s;
  __syncthreads();
  if (g == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += sm[k][threadIdx.x];
    out[c] = t;
  }
}

}  // namespace normk
}  // namespace dq
