// Explicit instantiations of the paged decode kernel: unquantised fp16 / bf16 cache, head_dim 64.
#include "decode_launch.cuh"
namespace b200 {
#define B200_KV16_FAMILY(MODE)                         \
  B200_DEFINE_DECODE_LAUNCH(64, 16, MODE, 1, false)   \
  B200_DEFINE_DECODE_LAUNCH(64, 16, MODE, 2, false)   \
  B200_DEFINE_DECODE_LAUNCH(64, 32, MODE, 1, false)   \
  B200_DEFINE_DECODE_LAUNCH(64, 32, MODE, 2, false)   \
  B200_DEFINE_DECODE_LAUNCH(64, 64, MODE, 1, false)   \
  B200_DEFINE_DECODE_LAUNCH(64, 64, MODE, 2, false)
B200_KV16_FAMILY(MODE_KV_F16)
B200_KV16_FAMILY(MODE_KV_BF16)
// contiguous K/V [batch, heads, seq, head_dim]: no pages, one row tile
B200_DEFINE_DECODE_LAUNCH(64, 16, MODE_KV_F16_TM, 1, false)
B200_DEFINE_DECODE_LAUNCH(64, 16, MODE_KV_BF16_TM, 1, false)
}  // namespace b200
