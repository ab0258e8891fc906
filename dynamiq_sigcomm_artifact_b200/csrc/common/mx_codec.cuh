// Warp-level block-float codec with the conversion instructions of sm_100a: MXFP8 (E4M3), FP6 (E3M2) and
// FP4 (E2M1) codes with one power-of-two (E8M0) scale per 32 values.
//
// A warp owns 1024 values; lane l holds the 32 consecutive values [32 l, 32 l + 32) = one scaling block.
// Encoded block: 32 lanes x 4 b code bytes (lane-major; inside a lane a little-endian stream of b-bit
// codes), then the 32 scale bytes: 128 b + 32 bytes, i.e. 8.25 / 6.25 / 4.25 bit per value - the figures
// the reference's bandwidth emulation charges for fp8 / fp6 / fp4
// (testbed_evaluation/new_comm_hooks/comm_hooks.py:239-241); its numerics come from the simulation stack
// (simulations_llm/new_comm_hooks/utils_aggregation.py:422-506).  PyTorch-op twin: codecs.BlockFloatCodec.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "rht_codec.cuh"

namespace dq {

template <int B>
struct MxGeom {
  static constexpr int kLaneBytes = 4 * B;            // 32 codes of b bits
  static constexpr int kBlockBytes = 128 * B + 32;    // 1056 / 800 / 544
};

template <int B>
__device__ __forceinline__ float mx_vmax() { return B == 8 ? 448.0f : (B == 6 ? 28.0f : 6.0f); }

// two floats -> two codes (low 16 bits: a in bits 0..7 (or 0..3 for E2M1), b above)
template <int B>
__device__ __forceinline__ uint32_t mx_cvt_pair(float a, float b) {
  uint32_t out;
  if (B == 8) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(a), "f"(b));  // first source -> upper byte
    out = r;
  } else if (B == 6) {
    uint16_t r;
    asm("cvt.rn.satfinite.e3m2x2.f32 %0, %2, %1;" : "=h"(r) : "f"(a), "f"(b));
    out = r;
  } else {
    uint16_t r;
    asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %2, %1;\n\tcvt.u16.u8 %0, t;\n\t}" : "=h"(r) : "f"(a), "f"(b));
    out = (r & 0xFu) | ((r & 0xF0u) << 4);  // spread the two nibbles into two bytes
  }
  return out;  // byte 0 = code(a), byte 1 = code(b)
}

// two codes (byte 0, byte 1) -> two floats
template <int B>
__device__ __forceinline__ float2 mx_decode_pair(uint32_t two_bytes) {
  uint32_t h2;
  if (B == 8) {
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(two_bytes)));
  } else if (B == 6) {
    asm("cvt.rn.f16x2.e3m2x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(two_bytes)));
  } else {
    const uint16_t packed = static_cast<uint16_t>((two_bytes & 0xFu) | ((two_bytes >> 4) & 0xF0u));
    asm("{\n\t.reg .b8 t;\n\tcvt.u8.u16 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(h2) : "h"(packed));
  }
  const __half2 h = *reinterpret_cast<__half2*>(&h2);
  return __half22float2(h);
}

// ceil(log2(r)) for a positive normal float, exactly: exponent, minus one... plus one unless r is a power of two
__device__ __forceinline__ int ceil_log2_exact(float r) {
  const uint32_t bits = __float_as_uint(r);
  const int e = static_cast<int>((bits >> 23) & 0xFFu) - 127;
  return (bits & 0x7FFFFFu) ? e + 1 : e;
}

// Encode the block in v into `tile` (shared memory, >= kBlockBytes): codes lane-major, then 32 scale bytes.
template <int B>
__device__ __forceinline__ void mx_encode_block(const float (&v)[32], uint8_t* tile, int lane) {
  float x[32], am = 0.f;
#pragma unroll
  for (int k = 0; k < 32; ++k) {
    x[k] = sanitize(v[k]);
    am = fmaxf(am, fabsf(x[k]));
  }
  int e = -127;
  if (am >= 1e-30f) e = max(-127, min(127, ceil_log2_exact(__fdiv_rn(am, mx_vmax<B>()))));
  const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);  // 2^-e, exact (e in -127..127 -> clamp below)
  const float invs = (e == -127) ? 1.7014118e38f : inv;                     // 2^127 for the smallest scale
  uint32_t codes[32];
#pragma unroll
  for (int k = 0; k < 32; k += 2) {
    const uint32_t two = mx_cvt_pair<B>(x[k] * invs, x[k + 1] * invs);
    codes[k] = two & 0xFFu;
    codes[k + 1] = (two >> 8) & 0xFFu;
  }
  uint32_t w[B];
  pack_codes<B>(codes, w, 0u);  // 32 clean codes of b bits -> b words, little-endian bit stream
  uint32_t* dst = reinterpret_cast<uint32_t*>(tile + lane * MxGeom<B>::kLaneBytes);
#pragma unroll
  for (int j = 0; j < B; ++j) dst[j] = w[j];
  tile[128 * B + lane] = static_cast<uint8_t>(e + 127);
}

template <int B, bool ADD>
__device__ __forceinline__ void mx_decode_block(float (&v)[32], const uint8_t* tile, int lane) {
  const uint32_t* src = reinterpret_cast<const uint32_t*>(tile + lane * MxGeom<B>::kLaneBytes);
  uint32_t w[B];
#pragma unroll
  for (int j = 0; j < B; ++j) w[j] = src[j];
  const int e = static_cast<int>(tile[128 * B + lane]) - 127;
  const float scale = (e == -127) ? 5.877471754e-39f : __uint_as_float(static_cast<uint32_t>(e + 127) << 23);  // 2^e
#pragma unroll
  for (int k = 0; k < 32; k += 2) {
    const uint32_t two = unpack_code<B>(w, k) | (unpack_code<B>(w, k + 1) << 8);
    const float2 f = mx_decode_pair<B>(two);
    const float a = f.x * scale, b = f.y * scale;
    v[k] = ADD ? __fadd_rn(v[k], a) : a;
    v[k + 1] = ADD ? __fadd_rn(v[k + 1], b) : b;
  }
}

// Identity wire: the block as 1024 bf16 (B = 16) or fp32 (B = 32) values, lane-contiguous.  The custom
// point-to-point all-reduce of uncompressed gradients (the reference's BFloat16 / Float32 "compressors"
// on its ring, utils_aggregation.py:575-686, and bf16_add_kernel, ring_allreduce_backend.cu:581-587).
template <int B>
struct CastGeom {
  static constexpr int kBlockBytes = 128 * B;  // 2048 / 4096
};

template <int B>
__device__ __forceinline__ void cast_encode_block(const float (&v)[32], uint8_t* tile, int lane) {
  if (B == 16) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(tile) + 32 * lane;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float o[4] = {sanitize(v[4 * q]), sanitize(v[4 * q + 1]), sanitize(v[4 * q + 2]), sanitize(v[4 * q + 3])};
      Elem<__nv_bfloat16>::store4(dst + 4 * q, o);
    }
  } else {
    float* dst = reinterpret_cast<float*>(tile) + 32 * lane;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float o[4] = {sanitize(v[4 * q]), sanitize(v[4 * q + 1]), sanitize(v[4 * q + 2]), sanitize(v[4 * q + 3])};
      Elem<float>::store4(dst + 4 * q, o);
    }
  }
}

template <int B, bool ADD>
__device__ __forceinline__ void cast_decode_block(float (&v)[32], const uint8_t* tile, int lane) {
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    float o[4];
    if (B == 16) Elem<__nv_bfloat16>::load4(reinterpret_cast<const __nv_bfloat16*>(tile) + 32 * lane + 4 * q, o);
    else Elem<float>::load4(reinterpret_cast<const float*>(tile) + 32 * lane + 4 * q, o);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[4 * q + k] = ADD ? __fadd_rn(v[4 * q + k], o[k]) : o[k];
  }
}

// ---- identity wire without staging ---------------------------------------------------------------------
// The message of the identity codec is the block's values in element order, so a warp can move them straight
// between global memory and registers in the coalesced load layout (element j * 128 + lane * 4 + k in
// v[4 j + k], the layout of load_block / store_block): every access is a full 512-byte (fp32) or 256-byte
// (bf16) line run per instruction, and nothing passes through shared memory.

// what the wire keeps of each value (non-finite -> 0, bf16 rounding for the 16-bit wire)
template <int B>
__device__ __forceinline__ void cast_round(float (&v)[32]) {
#pragma unroll
  for (int k = 0; k < 32; k += 2) {
    const float a = sanitize(v[k]), b = sanitize(v[k + 1]);
    if (B == 16) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
      const uint32_t q = *reinterpret_cast<const uint32_t*>(&h);
      v[k] = __uint_as_float(q << 16), v[k + 1] = __uint_as_float(q & 0xFFFF0000u);
    } else {
      v[k] = a, v[k + 1] = b;
    }
  }
}

// values already rounded by cast_round -> message
template <int B>
__device__ __forceinline__ void cast_msg_store(uint8_t* dst, const float (&v)[32], int lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float o[4] = {v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]};
    if (B == 16) Elem<__nv_bfloat16>::store4(reinterpret_cast<__nv_bfloat16*>(dst) + j * 128 + lane * 4, o);
    else Elem<float>::store4(reinterpret_cast<float*>(dst) + j * 128 + lane * 4, o);
  }
}

// message -> v (ADD: accumulate); the message was written by a peer: read past L1
template <int B, bool ADD>
__device__ __forceinline__ void cast_msg_load(float (&v)[32], const uint8_t* src, int lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float o[4];
    if (B == 16) {
      const uint2 q = __ldcg(reinterpret_cast<const uint2*>(src) + j * 32 + lane);
      o[0] = __uint_as_float(q.x << 16), o[1] = __uint_as_float(q.x & 0xFFFF0000u);
      o[2] = __uint_as_float(q.y << 16), o[3] = __uint_as_float(q.y & 0xFFFF0000u);
    } else {
      const float4 q = __ldcg(reinterpret_cast<const float4*>(src) + j * 32 + lane);
      o[0] = q.x, o[1] = q.y, o[2] = q.z, o[3] = q.w;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) v[4 * j + k] = ADD ? __fadd_rn(v[4 * j + k], o[k]) : o[k];
  }
}

template <int NBYTES>
__device__ __forceinline__ void bytes_copy_out(uint8_t* dst, const uint8_t* tile, int lane) {
  for (int i = lane; i < NBYTES / 16; i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(tile)[i];
}
template <int NBYTES>
__device__ __forceinline__ void bytes_copy_in(uint8_t* tile, const uint8_t* src, int lane) {
  for (int i = lane; i < NBYTES / 16; i += 32) reinterpret_cast<uint4*>(tile)[i] = __ldcg(reinterpret_cast<const uint4*>(src) + i);
}

template <int B>
__device__ __forceinline__ void mx_copy_out(uint8_t* dst, const uint8_t* tile, int lane) {
  constexpr int n8 = MxGeom<B>::kBlockBytes / 8;
  for (int i = lane; i < n8; i += 32)
    reinterpret_cast<unsigned long long*>(dst)[i] = reinterpret_cast<const unsigned long long*>(tile)[i];
}
template <int B>
__device__ __forceinline__ void mx_copy_in(uint8_t* tile, const uint8_t* src, int lane) {
  constexpr int n8 = MxGeom<B>::kBlockBytes / 8;
  for (int i = lane; i < n8; i += 32)
    reinterpret_cast<unsigned long long*>(tile)[i] = __ldcg(reinterpret_cast<const unsigned long long*>(src) + i);
}

}  // namespace dq
