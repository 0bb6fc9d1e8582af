// Explicit instantiations of the paged decode kernel: scale mode "page_scale", head_dim 128.
#include "decode_launch.cuh"
namespace b200 {
B200_DEFINE_DECODE_FAMILY(128, 0)
}  // namespace b200
