// Explicit instantiations of the paged decode kernel: scale mode "mx8k_mx4v", head_dim 128.
#include "decode_launch.cuh"
namespace b200 {
B200_DEFINE_DECODE_FAMILY(128, 3)
}  // namespace b200
