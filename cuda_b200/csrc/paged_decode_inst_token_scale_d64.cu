// Explicit instantiations of the paged decode kernel: scale mode "token_scale", head_dim 64.
#include "decode_launch.cuh"
namespace b200 {
B200_DEFINE_DECODE_FAMILY(64, 1)
}  // namespace b200
