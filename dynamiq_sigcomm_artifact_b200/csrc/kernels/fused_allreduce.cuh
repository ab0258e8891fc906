// Parameters of the persistent compressed all-reduce kernel (one struct per rank).
#pragma once
#include <cstdint>

namespace dq {

constexpr int kMaxWorld = 8;
constexpr int kMaxSteps = 32;
constexpr int kStepInts = 8;
constexpr uint32_t kTagStratified = 0x4000u;  // step tag flag: stratified rounding (schedules.py)

// local operand / result of a step: keep in sync with parallel/schedules.py
enum : int { kLocalRaw = 0, kLocalWs = 1 };
enum : int { kOutSend = 0, kOutStore = 1, kOutFinal = 2, kOutDecode = 3 };
enum : int {
  kCodecRht = 0, kCodecRhtTc = 1, kCodecScAee = 2, kCodecScMee = 3, kCodecMx = 4, kCodecCast = 5,
  kCodecScMixAee = 6, kCodecScMixMee = 7,  // superchunk records whose width (2 / 4 / 8) varies per superchunk
  kCodecRhtMix = 8                         // rotation codec whose code width (2..8) varies per 1024-element block
};

// error codes left in status[0]; status[1] = (step << 16) | cta, status[2] = slot
enum : uint32_t {
  kOk = 0, kErrWaitTimeout = 1, kErrBadProgram = 2, kErrCopyTimeout = 3, kErrMmaTimeout = 4,
  kErrBounds = 5  // debug mode: a slot index or a block's offset inside a slot left its region; the step is not run
};

struct ARParams {
  void* bucket;        // this rank's gradient bucket: input, scratch for partial sums, and output
  float* tail_ws;      // 1024 floats: stands in for a partial last block when it holds partial sums
  long long n;         // elements in the bucket
  int nblocks;         // ceil(n / 1024)
  int blocks_per_shard;
  int world, rank;
  int nsteps;
  uint8_t* mail[kMaxWorld];    // every rank's mailbox (peer mapped); mail[rank] is local
  uint32_t* flags[kMaxWorld];  // every rank's flag array
  unsigned long long slot_stride;  // bytes between consecutive slots of a mailbox
  unsigned long long scales_off;   // byte offset of the scales inside a slot
  uint32_t flag_base;              // first flag word of this collective's slot set
  uint32_t epoch;                  // value a flag must reach
  uint32_t seed_lo, seed_hi, step, bucket_id;
  float finish_scale;              // post_scale / 1024 applied by the inverse rotation
  unsigned long long timeout_ns;   // budget of each wait on a flag
  uint32_t* status;                // 4 words, local
  int no_transmit;                 // debug: run the maths, skip remote payload stores
  int prefetch;                    // 1: per-warp bulk-copy staging of the next raw block (4 KiB of shared memory per
                                   // warp); 0: read raw blocks directly, half the shared memory per CTA
  int tensor_rotation;             // host-side selector: 1 = tcgen05 rotation, 0 = SIMT butterflies
  int codec;                       // host-side selector: kCodecRht / kCodecScAee / kCodecScMee
  unsigned int block_bytes;        // bytes of one encoded 1024-element block inside a message
  float sc_lattice_max, sc_c1, sc_c2;  // superchunk codec constants
  const float* sc_lut;             // superchunk codec decode levels [2^bits] (device memory); mixed widths: the
                                   // constant table of sc_codec.cuh (kScMixTableFloats)
  const uint32_t* sc_plan;         // mixed widths: [nblocks + 1] message offsets of the blocks in 8-byte units (a prefix
                                   // sum), then [nblocks] packed widths (byte j = width of superchunk j of the block);
                                   // kCodecRhtMix: offsets in 128-byte units, then one width (2..8) per block
  int debug;                       // 1 (DQ_DEBUG=1 / debug=True): before a step touches a mailbox every CTA checks the
  int nslots;                      // step's slot indices against nslots, and the offset and length of every block of
  unsigned long long set_bytes;    // its range against the slot (plan-driven codecs: offsets come from device memory)
  int steps[kMaxSteps][kStepInts];
};

}  // namespace dq
