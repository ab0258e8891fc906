// Warp-level hierarchical "scaling quantisation" codec (the reference's superchunk format).
//
// A warp owns a block of 1024 values = 4 superchunks of 256 = 16 chunks of 16.  Lane l holds the 32
// consecutive values [32 l, 32 l + 32): two whole chunks of superchunk l / 8, so chunk maxima need
// no shuffles and the superchunk maximum is a 3-step butterfly inside an 8-lane group.
//
// Wire record of a superchunk (byte for byte the reference's layout, eden_utils.cpp:33-40,
// scaling_quantization_algorithm.md:347-388): 16 x [2 b bytes of codes, little end first | 1 byte
// round-up chunk scale] + 2 bytes bf16 scale unit = 16 (2 b + 1) + 2 bytes.  A block's four records are
// contiguous (an 8-byte multiple), are assembled in the warp's shared-memory tile and move with 8-byte
// accesses.
//
// Arithmetic restates parallel/codecs.py::SuperchunkCodec operation by operation (fp32, one rounding
// per operation), which itself restates the reference kernels
// (cuda_hierarchical_mee.cu:203-343 encode, :345-505 decode, :526-696 hop); partial sums stay fp32.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "philox.cuh"
#include "rht_codec.cuh"

namespace dq {

struct ScParams {
  float lattice_max;  // R for the linear lattice, lattice(R) for the logarithmic one
  float c1, c2;       // (1 + e^2) / (2 e^2) and log2(1 + 2 e^2)
  const float* lut;   // decode levels [2^b], device memory
};

template <int B>
struct ScGeom {
  static constexpr int kChunkBytes = 2 * B + 1;
  static constexpr int kRecordBytes = 16 * kChunkBytes + 2;  // 82 / 146 / 274
  static constexpr int kBlockBytes = 4 * kRecordBytes;       // 328 / 584 / 1096: multiples of 8
};

__device__ __forceinline__ float sc_sanitize(float x) { return (fabsf(x) <= 3.402823466e38f) ? x : 0.0f; }

// lane-contiguous layout: reg k of lane l = element 32 l + k
template <typename T>
__device__ __forceinline__ void sc_load_block(const T* base, int valid, bool vec_ok, int lane, float (&v)[32]) {
  if (valid == 1024 && vec_ok) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float o[4];
      Elem<T>::load4(base + 32 * lane + 4 * q, o);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[4 * q + k] = o[k];
    }
  } else {
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      const int e = 32 * lane + k;
      v[k] = e < valid ? Elem<T>::to_float(base[e]) : 0.0f;
    }
  }
}

template <typename T>
__device__ __forceinline__ void sc_store_block(T* base, int valid, bool vec_ok, int lane, const float (&v)[32]) {
  if (valid == 1024 && vec_ok) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float o[4] = {v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]};
      Elem<T>::store4(base + 32 * lane + 4 * q, o);
    }
  } else {
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      const int e = 32 * lane + k;
      if (e < valid) base[e] = Elem<T>::from_float(v[k]);
    }
  }
}

// The same two moves for whole fp32 blocks with fully coalesced global accesses: the warp reads or writes 512
// contiguous bytes per instruction and the lane-contiguous runs are formed through a warp-private 4 KiB shared
// buffer.  16-byte chunk c (= element / 4) of the block lives at chunk c ^ ((c >> 3) & 7) of the buffer, which
// makes both the linear side (chunk j * 32 + lane) and the per-lane side (chunk lane * 8 + i) free of bank
// conflicts while every register index stays a compile-time constant.
__device__ __forceinline__ void sc_load_block_coalesced(const float* base, float* buf, int lane, float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = j * 32 + lane;
    const float4 q = *reinterpret_cast<const float4*>(base + 4 * c);
    *reinterpret_cast<float4*>(buf + 4 * (c ^ ((c >> 3) & 7))) = q;
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 q = *reinterpret_cast<const float4*>(buf + 4 * ((lane * 8 + i) ^ (lane & 7)));
    v[4 * i] = q.x, v[4 * i + 1] = q.y, v[4 * i + 2] = q.z, v[4 * i + 3] = q.w;
  }
  __syncwarp();
}

__device__ __forceinline__ void sc_store_block_coalesced(float* base, float* buf, int lane, const float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 8; ++i)
    *reinterpret_cast<float4*>(buf + 4 * ((lane * 8 + i) ^ (lane & 7))) =
        make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = j * 32 + lane;
    *reinterpret_cast<float4*>(base + 4 * c) = *reinterpret_cast<const float4*>(buf + 4 * (c ^ ((c >> 3) & 7)));
  }
  __syncwarp();
}

// Encode the block held in v into four records in `tile` (shared memory, >= kBlockBytes).
template <int B, bool MEE>
__device__ __forceinline__ void sc_encode_block(const float (&v)[32], uint8_t* tile, const ScParams& sp,
                                                uint32_t first_call, uint32_t tag, uint32_t step, uint32_t k0,
                                                uint32_t k1, int lane) {
  constexpr int R = (1 << (B - 1)) - 1;
  using G = ScGeom<B>;
  float x[32], s[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float am = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      x[16 * h + k] = sc_sanitize(v[16 * h + k]);
      am = fmaxf(am, fabsf(x[16 * h + k]));
    }
    s[h] = fmaxf(__fadd_rn(__fdiv_rn(am, sp.lattice_max), 1e-7f), 1e-30f);
  }
  float S = fmaxf(s[0], s[1]);
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) S = fmaxf(S, __shfl_xor_sync(0xFFFFFFFFu, S, o));
  const __nv_bfloat16 unit_bf = __float2bfloat16_rn(fmaxf(__fdiv_rn(S, 255.0f), 1e-30f));
  const float unit = fmaxf(__bfloat162float(unit_bf), 1e-30f);
  uint8_t* rec = tile + (lane >> 3) * G::kRecordBytes;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float q = fminf(fmaxf(ceilf(__fmul_rn(__fdiv_rn(s[h], S), 255.0f)), 1.0f), 255.0f);
    const float dec = fmaxf(__fmul_rn(q, unit), 1e-30f);
    U4 r = philox4x32<7>(first_call + 2u * static_cast<uint32_t>(lane) + h, 0u, tag, step, k0, k1);
    const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
    uint32_t code[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float y = __fdiv_rn(x[16 * h + k], dec);
      if (MEE) {
        const float mag = __fdiv_rn(log2f(__fadd_rn(__fdiv_rn(fabsf(y), sp.c1), 1.0f)), sp.c2);
        y = y > 0.f ? mag : (y < 0.f ? -mag : 0.f);
      }
      const float u = __fmul_rn(__fadd_rn(static_cast<float>((rw[k >> 2] >> (8 * (k & 3))) & 0xFFu), 0.5f), 1.0f / 256.0f);
      const float fl = floorf(y);
      float c = fl + ((__fsub_rn(y, fl) > u) ? 1.0f : 0.0f);
      c = fminf(fmaxf(c, static_cast<float>(-R)), static_cast<float>(R));
      code[k] = static_cast<uint32_t>(static_cast<int>(c) + R);
    }
    uint8_t* ch = rec + (2 * (lane & 7) + h) * G::kChunkBytes;
    constexpr int per = 8 / B;  // codes per byte, little end first
#pragma unroll
    for (int byte = 0; byte < 2 * B; ++byte) {
      uint32_t val = 0;
#pragma unroll
      for (int j = 0; j < per; ++j) val |= code[byte * per + j] << (j * B);
      ch[byte] = static_cast<uint8_t>(val);
    }
    ch[2 * B] = static_cast<uint8_t>(q);
  }
  if ((lane & 7) == 0) {
    const unsigned short bits = __bfloat16_as_ushort(unit_bf);
    rec[16 * G::kChunkBytes] = static_cast<uint8_t>(bits & 0xFF);
    rec[16 * G::kChunkBytes + 1] = static_cast<uint8_t>(bits >> 8);
  }
}

// Decode the four records in `tile`; ADD: v <- v + decoded (one rounding each), else v <- decoded.
template <int B, bool MEE, bool ADD>
__device__ __forceinline__ void sc_decode_block(float (&v)[32], const uint8_t* tile, const ScParams& sp, int lane) {
  constexpr int R = (1 << (B - 1)) - 1;
  using G = ScGeom<B>;
  const uint8_t* rec = tile + (lane >> 3) * G::kRecordBytes;
  const unsigned short ub = static_cast<unsigned short>(rec[16 * G::kChunkBytes]) |
                            (static_cast<unsigned short>(rec[16 * G::kChunkBytes + 1]) << 8);
  const float unit = fmaxf(__bfloat162float(__ushort_as_bfloat16(ub)), 1e-30f);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint8_t* ch = rec + (2 * (lane & 7) + h) * G::kChunkBytes;
    const float dec = fmaxf(__fmul_rn(static_cast<float>(ch[2 * B]), unit), 1e-30f);
    constexpr int per = 8 / B;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const uint32_t code = (static_cast<uint32_t>(ch[k / per]) >> ((k % per) * B)) & ((1u << B) - 1u);
      const float level = MEE ? sp.lut[code] : static_cast<float>(static_cast<int>(code) - R);
      const float val = __fmul_rn(level, dec);
      v[16 * h + k] = ADD ? __fadd_rn(v[16 * h + k], val) : val;
    }
  }
}

// shared-memory tile <-> global record area, 8 bytes per lane per trip
template <int B>
__device__ __forceinline__ void sc_copy_out(uint8_t* dst, const uint8_t* tile, int lane) {
  constexpr int n8 = ScGeom<B>::kBlockBytes / 8;
  for (int i = lane; i < n8; i += 32)
    reinterpret_cast<unsigned long long*>(dst)[i] = reinterpret_cast<const unsigned long long*>(tile)[i];
}
template <int B>
__device__ __forceinline__ void sc_copy_in(uint8_t* tile, const uint8_t* src, int lane) {
  constexpr int n8 = ScGeom<B>::kBlockBytes / 8;
  for (int i = lane; i < n8; i += 32)
    reinterpret_cast<unsigned long long*>(tile)[i] = __ldcg(reinterpret_cast<const unsigned long long*>(src) + i);
}

// ---- mixed widths: every superchunk of a block has its own code width (2, 4 or 8) -----------------
//
// Per block the host side supplies `wpack` (byte j = width of superchunk j) and the block's byte offset
// inside the message (a prefix sum over the blocks' record bytes; any four records add up to a multiple of
// 8 bytes because 82, 146 and 274 are all 2 mod 8).  The arithmetic per superchunk is the fixed-width
// codec's, operation for operation, with the width as a run-time value: a record written here equals the
// record the fixed-width codec of that width writes for the same block, tag and step.
//
// Constant table (fp32, device): [0..2] lattice_max, [4..6] c1, [8..10] c2 for widths 2, 4, 8 (index
// log2(width) - 1); decode levels of width 2 at [16..20), width 4 at [20..36), width 8 at [36..292).
constexpr int kScMixTableFloats = 292;

__device__ __forceinline__ int sc_rec_bytes(int b) { return 16 * (2 * b + 1) + 2; }
__device__ __forceinline__ int sc_mix_block_bytes(uint32_t wpack) {
  return sc_rec_bytes(wpack & 0xFF) + sc_rec_bytes((wpack >> 8) & 0xFF) + sc_rec_bytes((wpack >> 16) & 0xFF) +
         sc_rec_bytes((wpack >> 24) & 0xFF);
}
__device__ __forceinline__ int sc_mix_slot(int b) { return b == 2 ? 0 : (b == 4 ? 1 : 2); }
__device__ __forceinline__ int sc_mix_lut_base(int b) { return b == 2 ? 16 : (b == 4 ? 20 : 36); }

__device__ __forceinline__ int sc_mix_rec_base(uint32_t wpack, int g) {
  int base = 0;
#pragma unroll
  for (int i = 0; i < 3; ++i)
    if (i < g) base += sc_rec_bytes((wpack >> (8 * i)) & 0xFF);
  return base;
}

template <bool MEE>
__device__ __forceinline__ void sc_encode_block_mix(const float (&v)[32], uint8_t* tile, const float* table,
                                                    uint32_t wpack, uint32_t first_call, uint32_t tag, uint32_t step,
                                                    uint32_t k0, uint32_t k1, int lane) {
  const int g = lane >> 3;
  const int B = static_cast<int>((wpack >> (8 * g)) & 0xFF);
  const int R = (1 << (B - 1)) - 1;
  const int ti = sc_mix_slot(B);
  const float lattice_max = __ldg(table + ti), c1 = __ldg(table + 4 + ti), c2 = __ldg(table + 8 + ti);
  const int chunk_bytes = 2 * B + 1;
  float x[32], s[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float am = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      x[16 * h + k] = sc_sanitize(v[16 * h + k]);
      am = fmaxf(am, fabsf(x[16 * h + k]));
    }
    s[h] = fmaxf(__fadd_rn(__fdiv_rn(am, lattice_max), 1e-7f), 1e-30f);
  }
  float S = fmaxf(s[0], s[1]);
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) S = fmaxf(S, __shfl_xor_sync(0xFFFFFFFFu, S, o));
  const __nv_bfloat16 unit_bf = __float2bfloat16_rn(fmaxf(__fdiv_rn(S, 255.0f), 1e-30f));
  const float unit = fmaxf(__bfloat162float(unit_bf), 1e-30f);
  uint8_t* rec = tile + sc_mix_rec_base(wpack, g);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float q = fminf(fmaxf(ceilf(__fmul_rn(__fdiv_rn(s[h], S), 255.0f)), 1.0f), 255.0f);
    const float dec = fmaxf(__fmul_rn(q, unit), 1e-30f);
    U4 r = philox4x32<7>(first_call + 2u * static_cast<uint32_t>(lane) + h, 0u, tag, step, k0, k1);
    const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
    unsigned long long acc[2] = {0ull, 0ull};
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float y = __fdiv_rn(x[16 * h + k], dec);
      if (MEE) {
        const float mag = __fdiv_rn(log2f(__fadd_rn(__fdiv_rn(fabsf(y), c1), 1.0f)), c2);
        y = y > 0.f ? mag : (y < 0.f ? -mag : 0.f);
      }
      const float u = __fmul_rn(__fadd_rn(static_cast<float>((rw[k >> 2] >> (8 * (k & 3))) & 0xFFu), 0.5f), 1.0f / 256.0f);
      const float fl = floorf(y);
      float c = fl + ((__fsub_rn(y, fl) > u) ? 1.0f : 0.0f);
      c = fminf(fmaxf(c, static_cast<float>(-R)), static_cast<float>(R));
      acc[k >> 3] |= static_cast<unsigned long long>(static_cast<uint32_t>(static_cast<int>(c) + R)) << ((k & 7) * B);
    }
    uint8_t* ch = rec + (2 * (lane & 7) + h) * chunk_bytes;
    for (int byte = 0; byte < B; ++byte) {  // codes 0..7 fill B bytes, codes 8..15 the next B, little end first
      ch[byte] = static_cast<uint8_t>(acc[0] >> (8 * byte));
      ch[B + byte] = static_cast<uint8_t>(acc[1] >> (8 * byte));
    }
    ch[2 * B] = static_cast<uint8_t>(q);
  }
  if ((lane & 7) == 0) {
    const unsigned short bits = __bfloat16_as_ushort(unit_bf);
    rec[16 * chunk_bytes] = static_cast<uint8_t>(bits & 0xFF);
    rec[16 * chunk_bytes + 1] = static_cast<uint8_t>(bits >> 8);
  }
}

template <bool MEE, bool ADD>
__device__ __forceinline__ void sc_decode_block_mix(float (&v)[32], const uint8_t* tile, const float* table,
                                                    uint32_t wpack, int lane) {
  const int g = lane >> 3;
  const int B = static_cast<int>((wpack >> (8 * g)) & 0xFF);
  const int R = (1 << (B - 1)) - 1;
  const uint32_t mask = (1u << B) - 1u;
  const int chunk_bytes = 2 * B + 1;
  const float* lut = table + sc_mix_lut_base(B);
  const uint8_t* rec = tile + sc_mix_rec_base(wpack, g);
  const unsigned short ub = static_cast<unsigned short>(rec[16 * chunk_bytes]) |
                            (static_cast<unsigned short>(rec[16 * chunk_bytes + 1]) << 8);
  const float unit = fmaxf(__bfloat162float(__ushort_as_bfloat16(ub)), 1e-30f);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint8_t* ch = rec + (2 * (lane & 7) + h) * chunk_bytes;
    const float dec = fmaxf(__fmul_rn(static_cast<float>(ch[2 * B]), unit), 1e-30f);
    unsigned long long acc[2] = {0ull, 0ull};
    for (int byte = 0; byte < B; ++byte) {
      acc[0] |= static_cast<unsigned long long>(ch[byte]) << (8 * byte);
      acc[1] |= static_cast<unsigned long long>(ch[B + byte]) << (8 * byte);
    }
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const uint32_t code = static_cast<uint32_t>(acc[k >> 3] >> ((k & 7) * B)) & mask;
      const float level = MEE ? __ldg(lut + code) : static_cast<float>(static_cast<int>(code) - R);
      const float val = __fmul_rn(level, dec);
      v[16 * h + k] = ADD ? __fadd_rn(v[16 * h + k], val) : val;
    }
  }
}

__device__ __forceinline__ void sc_copy_out_n(uint8_t* dst, const uint8_t* tile, int n8, int lane) {
  for (int i = lane; i < n8; i += 32)
    reinterpret_cast<unsigned long long*>(dst)[i] = reinterpret_cast<const unsigned long long*>(tile)[i];
}
__device__ __forceinline__ void sc_copy_in_n(uint8_t* tile, const uint8_t* src, int n8, int lane) {
  for (int i = lane; i < n8; i += 32)
    reinterpret_cast<unsigned long long*>(tile)[i] = __ldcg(reinterpret_cast<const unsigned long long*>(src) + i);
}

}  // namespace dq
