// Philox-4x32-10 counter-based generator, identical on host and device.
// Python twin: dynamiq_sigcomm_artifact_b200/utils/philox.py (tests compare them word for word).
// Replaces the reference's pre-generated uniform pool and LCG window
// (testbed_evaluation/new_comm_hooks/utils_aggregation.py:384-420): every uniform is a pure
// function of (seed, step, bucket, stream tag, block, position).
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define DQ_HD __host__ __device__ __forceinline__
#else
#define DQ_HD inline
#endif

namespace dq {

constexpr uint32_t kPhiloxM0 = 0xD2511F53u;
constexpr uint32_t kPhiloxM1 = 0xCD9E8D57u;
constexpr uint32_t kPhiloxW0 = 0x9E3779B9u;
constexpr uint32_t kPhiloxW1 = 0xBB67AE85u;

constexpr uint32_t kTagSign = 0x5349474Eu;
constexpr uint32_t kTagEncode = 0x100u;
constexpr uint32_t kTagFinal = 0x200u;
constexpr uint32_t kTagScale = 0x300u;

struct U4 {
  uint32_t x, y, z, w;
};

DQ_HD void mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
  const uint64_t p = static_cast<uint64_t>(a) * b;  // one wide multiply on the device
  hi = static_cast<uint32_t>(p >> 32);
  lo = static_cast<uint32_t>(p);
}

template <int ROUNDS = 10>
DQ_HD U4 philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    mulhilo(kPhiloxM0, c0, hi0, lo0);
    mulhilo(kPhiloxM1, c2, hi1, lo1);
    uint32_t n0 = hi1 ^ c1 ^ k0;
    uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0;
    c1 = lo1;
    c2 = n2;
    c3 = lo0;
    k0 += kPhiloxW0;
    k1 += kPhiloxW1;
  }
  return U4{c0, c1, c2, c3};
}

// RNG stream id of an encode: the bucket index occupies the high half of counter word c2.
DQ_HD uint32_t stream_tag(uint32_t bucket, uint32_t tag) { return ((bucket & 0xFFFFu) << 16) | tag; }

// Word w (0..31) of the 1024-bit Rademacher diagonal of (step, bucket, seed).
DQ_HD uint32_t sign_word(int w, uint32_t step, uint32_t bucket, uint32_t seed_lo, uint32_t seed_hi) {
  U4 r = philox4x32(static_cast<uint32_t>(w >> 2), step, kTagSign, bucket, seed_lo, seed_hi);
  switch (w & 3) {
    case 0: return r.x;
    case 1: return r.y;
    case 2: return r.z;
    default: return r.w;
  }
}

}  // namespace dq
