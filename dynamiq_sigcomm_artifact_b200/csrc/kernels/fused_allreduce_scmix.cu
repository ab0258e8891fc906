// Mixed-width superchunk (AEE / MEE) instantiation of the persistent compressed all-reduce kernel: every
// 256-element superchunk carries its own code width (2, 4 or 8 bits), as the reference's threshold table and
// dynamic-bitrate controller assign them (testbed_evaluation/new_comm_hooks/comm_hooks.py:713-780, 903-1144),
// in ONE collective instead of one per width group.
#include "fused_allreduce_impl.cuh"
namespace dq {
DQ_INSTANTIATE_FUSED_ALLREDUCE_SCMIX
}  // namespace dq
