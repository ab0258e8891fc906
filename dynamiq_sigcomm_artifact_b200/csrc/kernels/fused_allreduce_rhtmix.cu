// Explicit instantiation of the persistent all-reduce kernel for the rotation codec with a code width per
// 1024-element block (no counterpart in the reference, whose widths vary per 256-element superchunk).
#include "fused_allreduce_impl.cuh"

namespace dq {
DQ_INSTANTIATE_FUSED_ALLREDUCE_RHTMIX
}  // namespace dq
