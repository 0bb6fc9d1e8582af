// Explicit instantiations of the paged decode kernel: scale mode "page_scale", head_dim 64.
#include "decode_launch.cuh"
namespace b200 {
B200_DEFINE_DECODE_FAMILY(64, 0)
}  // namespace b200
