// Warp-level building blocks of the rotation codec: one warp owns one block of 1024 values,
// 32 per lane.  CPU oracle with the same arithmetic order: codec_ref.py.
//
// Replaces the reference's per-superchunk CTAs (one 256-thread CTA per 512 bytes, scalar
// 2-byte loads, a serial thread-0 max between two block barriers;
// cuda_kernels/src/srrcomp/eden_utils/csrc/cuda_hierarchical_mee.cu:203-270,526-604) and its
// separate Hadamard passes (csrc/cuda_hadamard.cu:66-274).
//
// Register layouts of a lane
//   load layout        reg t = 4 j + k   holds element     e = 128 j + 4 lane + k
//   coefficient layout reg k             holds coefficient e = (lane & 3) + 4 k + 128 (lane >> 2)
// The Hadamard transform runs five butterfly stages in registers, swaps the five lane bits
// with the five register bits through a swizzled 4 KiB shared-memory tile, and runs five more.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "philox.cuh"

namespace dq {

constexpr int kBlock = 1024;
constexpr unsigned kFullMask = 0xFFFFFFFFu;
constexpr int kUniformRounds = 7;  // Philox-4x32-7 for the rounding uniforms (philox.py: UNIFORM_ROUNDS)

// Five butterfly stages over the 32 registers of a lane.  Stage 0 pairs neighbouring registers;
// stages 1..4 act on register pairs (2i, 2i+1) and use the packed fp32x2 add / fma of sm_100
// (a - b is fma(b, -1, a): one rounding, same bits as a subtraction).
__device__ __forceinline__ void butterflies32(float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const float a = v[i], b = v[i + 1];
    v[i] = a + b;
    v[i + 1] = a - b;
  }
  const float2 neg1 = make_float2(-1.0f, -1.0f);
#pragma unroll
  for (int m = 1; m < 5; ++m) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      if ((i & (1 << m)) == 0) {
        const int j = i | (1 << m);
        const float2 a = make_float2(v[i], v[i + 1]), b = make_float2(v[j], v[j + 1]);
        const float2 sum = __fadd2_rn(a, b), dif = __ffma2_rn(b, neg1, a);
        v[i] = sum.x, v[i + 1] = sum.y;
        v[j] = dif.x, v[j + 1] = dif.y;
      }
    }
  }
}

// load layout -> coefficient layout through the warp's 1024-float tile
__device__ __forceinline__ void transpose_to_coeff(float (&v)[32], float* tile, int lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float4 q = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    *reinterpret_cast<float4*>(tile + j * 128 + ((lane ^ j) << 2)) = q;
  }
  __syncwarp();
  const int J = lane >> 2, K = lane & 3;
#pragma unroll
  for (int t = 0; t < 32; ++t) v[t] = tile[J * 128 + ((t ^ J) << 2) + K];
  __syncwarp();
}

// coefficient layout -> load layout
__device__ __forceinline__ void transpose_to_load(float (&v)[32], float* tile, int lane) {
  const int J = lane >> 2, K = lane & 3;
#pragma unroll
  for (int t = 0; t < 32; ++t) tile[J * 128 + ((t ^ J) << 2) + K] = v[t];
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float4 q = *reinterpret_cast<const float4*>(tile + j * 128 + ((lane ^ j) << 2));
    v[4 * j] = q.x;
    v[4 * j + 1] = q.y;
    v[4 * j + 2] = q.z;
    v[4 * j + 3] = q.w;
  }
  __syncwarp();
}

// Sign tables.  The Rademacher diagonal is applied by multiplying with +-1.0 (forward) or +-c (inverse, c =
// post_scale / 1024) read from two 1024-float tables in shared memory that a CTA builds once from the 32 sign
// words; a packed multiply replaces the per-element bit extraction and xor.  Table order: element index.
__device__ __forceinline__ void fill_sign_tables(float* sgn_fwd, float* sgn_inv, const uint32_t* sign_words, float c,
                                                 int tid, int nthreads) {
  for (int e = tid; e < 1024; e += nthreads) {
    const bool neg = (sign_words[e >> 5] >> (e & 31)) & 1u;
    sgn_fwd[e] = neg ? -1.0f : 1.0f;
    sgn_inv[e] = neg ? -c : c;
  }
}

// v (load layout) *= table (element order): eight 16-byte table reads and sixteen packed multiplies
__device__ __forceinline__ void scale_by_table(float (&v)[32], const float* table, int lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float4 q = *reinterpret_cast<const float4*>(table + j * 128 + lane * 4);
    const float2 a = __fmul2_rn(make_float2(v[4 * j], v[4 * j + 1]), make_float2(q.x, q.y));
    const float2 b = __fmul2_rn(make_float2(v[4 * j + 2], v[4 * j + 3]), make_float2(q.z, q.w));
    v[4 * j] = a.x, v[4 * j + 1] = a.y, v[4 * j + 2] = b.x, v[4 * j + 3] = b.y;
  }
}

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ void load4(const float* p, float (&o)[4]) {
    float4 q = *reinterpret_cast<const float4*>(p);
    o[0] = q.x, o[1] = q.y, o[2] = q.z, o[3] = q.w;
  }
  static __device__ __forceinline__ void store4(float* p, const float (&o)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  }
  static __device__ __forceinline__ float to_float(float x) { return x; }
  static __device__ __forceinline__ float from_float(float x) { return x; }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&o)[4]) {
    uint2 q = *reinterpret_cast<const uint2*>(p);
    o[0] = __uint_as_float(q.x << 16), o[1] = __uint_as_float(q.x & 0xFFFF0000u);
    o[2] = __uint_as_float(q.y << 16), o[3] = __uint_as_float(q.y & 0xFFFF0000u);
  }
  static __device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&o)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(o[2], o[3]);
    uint2 q;
    q.x = *reinterpret_cast<uint32_t*>(&a);
    q.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = q;
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

// 1024 elements starting at `base` in the load layout; elements >= valid read as 0.
template <typename T>
__device__ __forceinline__ void load_block(const T* base, int valid, bool vec_ok, int lane, float (&v)[32]) {
  if (valid == kBlock && vec_ok) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float o[4];
      Elem<T>::load4(base + j * 128 + lane * 4, o);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[4 * j + k] = o[k];
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        int e = j * 128 + lane * 4 + k;
        v[4 * j + k] = e < valid ? Elem<T>::to_float(base[e]) : 0.0f;
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ void store_block(T* base, int valid, bool vec_ok, int lane, const float (&v)[32]) {
  if (valid == kBlock && vec_ok) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float o[4] = {v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]};
      Elem<T>::store4(base + j * 128 + lane * 4, o);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        int e = j * 128 + lane * 4 + k;
        if (e < valid) base[e] = Elem<T>::from_float(v[4 * j + k]);
      }
    }
  }
}

// raw gradients (load layout) -> rotated coefficients (coefficient layout): y = H (s * x), unnormalised.
// Non-finite inputs are not filtered here: they reach every coefficient of the block, and the quantiser
// then transmits the whole block as zeros.
__device__ __forceinline__ void rotate_forward(float (&v)[32], const float* sgn_fwd, float* tile, int lane) {
  scale_by_table(v, sgn_fwd, lane);
  butterflies32(v);
  transpose_to_coeff(v, tile, lane);
  butterflies32(v);
}

// rotated coefficients -> gradients in the load layout: x = s * (H y) * c, c = post_scale / 1024
__device__ __forceinline__ void rotate_inverse(float (&v)[32], const float* sgn_inv, float* tile, int lane) {
  butterflies32(v);
  transpose_to_load(v, tile, lane);
  butterflies32(v);
  scale_by_table(v, sgn_inv, lane);
}

__device__ __forceinline__ float sanitize(float x) { return (fabsf(x) <= 3.402823466e38f) ? x : 0.0f; }

// Dense packing of 32 codes of B bits into B words.  `f[k]` = G + code k, where G (the bit pattern of the
// quantiser's magic number) is the same for every k and has its low bits clear.  The words are built as
// sum_k f[k] * 2^shift_k, one integer multiply-add per code, and the known contribution of G is subtracted
// once per word; a code that straddles two words adds its high part with a shift.
template <int B>
__device__ __forceinline__ void pack_codes(const uint32_t (&f)[32], uint32_t (&w)[B], uint32_t G) {
  if constexpr (B == 8) {  // byte 0 of four values per word: three byte permutes
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t lo = __byte_perm(f[4 * j], f[4 * j + 1], 0x0040u);
      const uint32_t hi = __byte_perm(f[4 * j + 2], f[4 * j + 3], 0x0040u);
      w[j] = __byte_perm(lo, hi, 0x5410u);
    }
  } else {
    uint32_t gsum[B];  // multiples of G accumulated in each word (compile-time after unrolling)
#pragma unroll
    for (int j = 0; j < B; ++j) w[j] = 0, gsum[j] = 0;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      const int off = k * B, wi = off >> 5, sh = off & 31;
      w[wi] += f[k] * (1u << sh);
      gsum[wi] += 1u << sh;
      if (sh + B > 32) {  // the code's top bits open the next word: (G + c) >> r = (G >> r) + (c >> r), r < B
        w[wi + 1] += f[k] >> (32 - sh);
        w[wi + 1] -= G >> (32 - sh);
      }
    }
#pragma unroll
    for (int j = 0; j < B; ++j) w[j] -= G * gsum[j];
  }
}

template <int B>
__device__ __forceinline__ uint32_t unpack_code(const uint32_t (&w)[B], int k) {
  const int off = k * B, wi = off >> 5, sh = off & 31;
  uint32_t x = (sh + B > 32) ? __funnelshift_r(w[wi], w[wi + 1], sh) : (w[wi] >> sh);
  return x & ((1u << B) - 1u);
}

// Largest magnitude of the block (fmaxf ignores NaN operands; the absolute values fold into the max
// instruction as operand modifiers).  A NaN among the inputs of a rotation reaches EVERY coefficient of the
// block, so a block with a NaN arrives here with all 32 x 32 values NaN and the result stays 0; an infinite
// input gives coefficients that are infinite or NaN, and the result is infinite or 0.  Both fail the
// caller's range check, which is all that is asked of them.
__device__ __forceinline__ float warp_absmax(const float (&y)[32]) {
  float m = 0.0f;
#pragma unroll
  for (int k = 0; k < 32; k += 2) m = fmaxf(m, fmaxf(fabsf(y[k]), fabsf(y[k + 1])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(kFullMask, m, o));
  return m;
}

// The packed words of a block whose every code is R (the zero level), word j of B.
template <int B>
__device__ __forceinline__ constexpr uint32_t zero_block_word(int j) {
  constexpr uint32_t R = (1u << (B - 1)) - 1u;
  uint32_t w = 0;
  for (int k = 0; k < 32; ++k) {
    const int off = k * B, wi = off >> 5, sh = off & 31;
    if (wi == j) w |= R << sh;
    if (sh + B > 32 && wi + 1 == j) w |= R >> (32 - sh);
  }
  return w;
}

// Stochastic b-bit quantisation of a block in the coefficient layout.  Returns the block scale.
//   code = floor(y * R / absmax + u) + R,   u = (byte + 0.5) / 256
// computed 256 times larger and shifted by 2^15, so that every step is one instruction on bit patterns:
//   a = 2^15 + byte + 0.5         one byte permute: the float 0x47'00'bb'80 has the byte at value 1
//   t = fma(y, 256 R / absmax, a)
//   g = t + (1.5 * 2^31 + 256 (R - 128))   rounded DOWN; one ulp = 256 there, so the low bits of g's
//                                          pattern are floor((t - 2^15) / 256) + R = the code
// No conversion, subtraction or clamp is issued.  No clamp is needed because |y| <= absmax holds exactly:
// |y * (R / absmax)| <= R (1 + 2^-24), so t - 2^15 lies strictly inside (-256 R, 256 (R + 1)).
// A block whose absmax is infinite or below 1e-30 (which includes the all-NaN block, see warp_absmax) is sent as
// zeros (scale 0, every code = R); the codes computed from its values are discarded, y itself is left as it is.
//
// Stratified ("correlated") rounding, strat_world > 1: all ranks draw the same byte per value and
// rank r uses u = (((r + shift) mod W) * 256 + byte + 0.5) / (256 W), shift = the byte of the
// lane's next value, so the W rounding errors that meet in a sum are negatively correlated.
// The 32 random bytes of a lane for one block (two Philox-4x32-7 calls); independent of the data, so a
// caller may draw them while something else (a tensor-core pass) is in flight.
__device__ __forceinline__ void draw_block_randoms(uint32_t (&rw)[8], uint32_t block_idx, uint32_t tag, uint32_t step,
                                                   uint32_t k0, uint32_t k1, int lane) {
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    U4 r = philox4x32<kUniformRounds>(block_idx, static_cast<uint32_t>(lane * 2 + q), tag, step, k0, k1);
    rw[4 * q] = r.x, rw[4 * q + 1] = r.y, rw[4 * q + 2] = r.z, rw[4 * q + 3] = r.w;
  }
}

template <int B>
__device__ __forceinline__ float quantize_block_rw(float (&y)[32], uint32_t (&w)[B], const uint32_t (&rw)[8],
                                                   int lane, int strat_rank = 0, int strat_world = 1) {
  constexpr int R = (1 << (B - 1)) - 1;
  const float m = warp_absmax(y);
  const bool ok = (m >= 1e-30f) && (m <= 3.402823466e38f);
  const float scale = ok ? __fdiv_rn(m, static_cast<float>(R)) : 0.0f;
  const float inv = ok ? __fdiv_rn(static_cast<float>(R), m) : 0.0f;
  uint32_t f[32];
  if (strat_world > 1) {
    const float2 half_off = make_float2(-8388607.5f, -8388607.5f);
    const float cw = 1.0f / (256.0f * static_cast<float>(strat_world));
    const uint32_t recip = 65536u / static_cast<uint32_t>(strat_world) + 1u;  // x / W for x < 512
    const float2 inv2 = make_float2(inv, inv), cw2 = make_float2(cw, cw);
    const float2 magic1 = make_float2(12582912.0f + R, 12582912.0f + R);  // 1.5 * 2^23 + R, one ulp = 1
#pragma unroll
    for (int k = 0; k < 32; k += 2) {
      float xs[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int kk = k + j, kn = (kk + 1) & 31;
        const uint32_t byte = (rw[kk >> 2] >> (8 * (kk & 3))) & 0xFFu;
        const uint32_t sh = ((rw[kn >> 2] >> (8 * (kn & 3))) & 0xFFu) + static_cast<uint32_t>(strat_rank);
        const uint32_t stratum = sh - static_cast<uint32_t>(strat_world) * ((sh * recip) >> 16);
        xs[j] = __uint_as_float(0x4B000000u | (stratum * 256u + byte));  // 2^23 + (stratum * 256 + byte)
      }
      const float2 u = __fmul2_rn(__fadd2_rn(make_float2(xs[0], xs[1]), half_off), cw2);
      const float2 t = __ffma2_rn(make_float2(y[k], y[k + 1]), inv2, u);
      const float2 g = __fadd2_rd(t, magic1);
      f[k] = __float_as_uint(g.x);
      f[k + 1] = __float_as_uint(g.y);
    }
  } else {
    const float2 inv256 = make_float2(inv * 256.0f, inv * 256.0f);
    const float magic_v = 3221225472.0f + 256.0f * (R - 128);  // 1.5 * 2^31 + 256 (R - 128): exact
    const float2 magic = make_float2(magic_v, magic_v);
#pragma unroll
    for (int k = 0; k < 32; k += 2) {
      const float a0 = __uint_as_float(__byte_perm(rw[k >> 2], 0x47000080u, 0x7504u | ((k & 3) << 4)));
      const float a1 = __uint_as_float(__byte_perm(rw[k >> 2], 0x47000080u, 0x7504u | (((k + 1) & 3) << 4)));
      const float2 t = __ffma2_rn(make_float2(y[k], y[k + 1]), inv256, make_float2(a0, a1));
      const float2 g = __fadd2_rd(t, magic);
      f[k] = __float_as_uint(g.x);
      f[k + 1] = __float_as_uint(g.y);
    }
  }
  pack_codes<B>(f, w, strat_world > 1 ? 0x4B400000u : 0x4F400000u);
  if (!ok) {  // warp-uniform and rare: whatever the non-finite values produced above is replaced by the zero block
#pragma unroll
    for (int j = 0; j < B; ++j) w[j] = zero_block_word<B>(j);
  }
  return scale;
}

template <int B>
__device__ __forceinline__ float quantize_block(float (&y)[32], uint32_t (&w)[B], uint32_t block_idx,
                                                uint32_t tag, uint32_t step, uint32_t k0, uint32_t k1, int lane,
                                                int strat_rank = 0, int strat_world = 1) {
  uint32_t rw[8];
  draw_block_randoms(rw, block_idx, tag, step, k0, k1, lane);
  return quantize_block_rw<B>(y, w, rw, lane, strat_rank, strat_world);
}

// float(code - R) without a conversion: 0x4B400000 | code is 1.5 * 2^23 + code
template <int B>
__device__ __forceinline__ float2 code_pair(const uint32_t (&w)[B], int k) {
  constexpr int R = (1 << (B - 1)) - 1;
  const float2 off = make_float2(-(12582912.0f + R), -(12582912.0f + R));
  const float a = __uint_as_float(0x4B400000u | unpack_code<B>(w, k));
  const float b = __uint_as_float(0x4B400000u | unpack_code<B>(w, k + 1));
  return __fadd2_rn(make_float2(a, b), off);
}

template <int B>
__device__ __forceinline__ void dequantize_block(const uint32_t (&w)[B], float scale, float (&y)[32]) {
  const float2 s2 = make_float2(scale, scale);
#pragma unroll
  for (int k = 0; k < 32; k += 2) {
    const float2 r = __fmul2_rn(code_pair<B>(w, k), s2);
    y[k] = r.x, y[k + 1] = r.y;
  }
}

// y <- fma(code - R, scale, y)
template <int B>
__device__ __forceinline__ void dequantize_add_block(const uint32_t (&w)[B], float scale, float (&y)[32]) {
  const float2 s2 = make_float2(scale, scale);
#pragma unroll
  for (int k = 0; k < 32; k += 2) {
    const float2 r = __ffma2_rn(code_pair<B>(w, k), s2, make_float2(y[k], y[k + 1]));
    y[k] = r.x, y[k + 1] = r.y;
  }
}

}  // namespace dq
