"""Stand-in for the reference's pybind module ``fused_online_softmax_cuda`` (decode path only):
``paged_attention_forward`` (``fused_softmax_binding.cpp:734-740`` in the reference project),
``fp8_paged_attention_forward`` (``:800-807``) and ``async_flash_decode`` (``:759-763``), same
positional arguments, same ``RuntimeError`` messages; extensions are keyword-only."""
from cuda_b200.ops import (async_flash_decode, fp8_paged_attention_forward,  # noqa: F401
                           paged_attention_forward)

__all__ = ["paged_attention_forward", "fp8_paged_attention_forward", "async_flash_decode"]
