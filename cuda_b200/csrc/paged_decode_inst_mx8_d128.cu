// Explicit instantiations of the paged decode kernel: scale mode "mx8", head_dim 128.
#include "decode_launch.cuh"
namespace b200 {
B200_DEFINE_DECODE_FAMILY(128, 2)
}  // namespace b200
