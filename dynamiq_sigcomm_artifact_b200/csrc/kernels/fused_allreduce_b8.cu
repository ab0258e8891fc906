// 8-bit instantiation of the persistent compressed all-reduce kernel.
#include "fused_allreduce_impl.cuh"
namespace dq {
DQ_INSTANTIATE_FUSED_ALLREDUCE(8)
}  // namespace dq
