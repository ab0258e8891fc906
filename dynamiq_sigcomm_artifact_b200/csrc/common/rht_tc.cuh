// Warpgroup-level Hadamard rotation on the tensor cores for the fused collective kernel.
//
// Four warps (one warpgroup) hold four blocks, one per warp.  H_1024 = H_32 (x) H_32 is applied as
// two tcgen05.mma passes D = A . H_32 over a shared 128 x 32 TF32 operand (see
// kernels/fwht_tcgen05.cu for the algebra); accumulators live in the warpgroup's 64 TMEM
// columns and come back with tcgen05.ld, one coefficient row or column per thread.
//
// Register layouts of a lane
//   load layout (as in rht_codec.cuh)  reg t = 4 j + k holds element e = 128 j + 4 lane + k
//   coefficient layout (tensor path)   reg n holds coefficient        e = 32 n + lane
//   column layout (after the inverse)  reg m holds element            e = 32 m + lane
//
// Operands are single TF32 (10 explicit mantissa bits): the rotation then carries a relative
// error of ~2^-11 per value, three orders of magnitude below the rounding noise of an 8-bit code.
// Results are deterministic but not bit-identical to the fp32 butterflies of the SIMT path, so a
// collective must use one rotation on all ranks.
#pragma once
#include "rht_codec.cuh"
#include "tcgen05.cuh"

namespace dq {

struct TcGroup {
  uint8_t* a;           // this warpgroup's operand buffer (tc::kOperandBytes)
  uint32_t hmat;        // shared-memory address of H_32
  uint64_t* bar;        // MMA-completion barrier of the warpgroup
  uint32_t tmem_d1;     // TMEM address of D1 with this warp's lane offset; D2 is 32 columns further
  uint32_t tmem_wg;     // TMEM address of D1 without the lane offset (for the issuing thread)
  uint32_t parity;      // phase of `bar` to wait for next
  int barrier_id;       // named barrier of the warpgroup
  int wi;               // warp index inside the warpgroup
  bool leader;          // the one thread that issues the MMAs
  int* error;           // shared flag, set when a wait gave up
};

__device__ __forceinline__ void wg_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

struct NoWork {
  __device__ __forceinline__ void operator()() const {}
};

// operand in shared memory -> one pass D = A . H_32 -> 32 accumulator columns into registers.
// `while_in_flight` runs between the issue of the MMAs and the wait for their completion.
template <class F = NoWork>
__device__ __forceinline__ void tc_pass(TcGroup& g, uint32_t col_off, float (&out)[32], F&& while_in_flight = F()) {
  tc::fence_async_smem();
  tc::tc_fence_before();
  wg_sync(g.barrier_id);
  if (g.leader) {
    tc::tc_fence_after();
    tc::mma_tile_k32(g.tmem_wg + col_off, tc::smem_u32(g.a), g.hmat, false);
    tc::mma_commit(g.bar);
  }
  while_in_flight();
  if (!tc::mbar_wait(g.bar, g.parity)) atomicExch(g.error, 1);
  g.parity ^= 1u;
  tc::tc_fence_after();
  tc::tmem_load32(g.tmem_d1 + col_off, out);
}

// second operand: each block transposed, A2[(32 wi + c), k = lane] = d[c]
__device__ __forceinline__ void tc_scatter_transposed(TcGroup& g, const float (&d)[32], int lane) {
#pragma unroll
  for (int c = 0; c < 32; ++c) *reinterpret_cast<float*>(g.a + tc::operand_offset(32 * g.wi + c, lane)) = d[c];
}

// raw gradients in the load layout -> rotated coefficients in the tensor-path coefficient layout
template <class F = NoWork>
__device__ __forceinline__ void rotate_forward_tc(float (&v)[32], uint32_t sign_mask, TcGroup& g, int lane,
                                                  F&& while_in_flight = F()) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = flip(sanitize(v[4 * j + k]), (sign_mask >> (4 * j + k)) & 1u);
    const uint32_t off = tc::operand_offset(32 * g.wi + 4 * j + (lane >> 3), (lane & 7) * 4);
    *reinterpret_cast<float4*>(g.a + off) = make_float4(o[0], o[1], o[2], o[3]);
  }
  float d[32];
  tc_pass(g, 0, d, while_in_flight);
  tc_scatter_transposed(g, d, lane);
  tc_pass(g, 32, v);
}

// coefficients (tensor-path layout: reg n = W[n][lane]) -> gradients in the column layout:
// x = s * (H W H) * c.  Both operands are transposed scatters, so that the thread ends with a
// column of the result and the global stores of a warp are contiguous 128-byte lines.
//   pass 1: A1[(b, n), k = lane] = W[n][lane]      -> D1 = W H, thread (b, n) holds row n
//   pass 2: A2[(b, c), k = n]    = D1[n][c]        -> D2[(b, c)][m] = (H W H)[m][c]
__device__ __forceinline__ void rotate_inverse_tc(float (&v)[32], uint32_t col_signs, float c, TcGroup& g, int lane) {
  tc_scatter_transposed(g, v, lane);
  float d[32];
  tc_pass(g, 0, d);
  tc_scatter_transposed(g, d, lane);
  tc_pass(g, 32, v);
#pragma unroll
  for (int m = 0; m < 32; ++m) v[m] = flip(__fmul_rn(v[m], c), (col_signs >> m) & 1u);
}

// bit m of the result = sign bit of element 32 m + lane (the column layout's register m)
__device__ __forceinline__ uint32_t lane_col_signs(const uint32_t* sign_words, int lane) {
  uint32_t mask = 0;
#pragma unroll
  for (int m = 0; m < 32; ++m) mask |= ((sign_words[m] >> lane) & 1u) << m;
  return mask;
}

// 1024 elements in the column layout: register m of a lane is element 32 m + lane
template <typename T>
__device__ __forceinline__ void store_block_cols(T* base, int valid, int lane, const float (&v)[32]) {
#pragma unroll
  for (int m = 0; m < 32; ++m) {
    const int e = 32 * m + lane;
    if (e < valid) base[e] = Elem<T>::from_float(v[m]);
  }
}

}  // namespace dq
