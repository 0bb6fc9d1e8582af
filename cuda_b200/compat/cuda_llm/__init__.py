"""The reference's ``cuda_llm`` package name, decode path only.  The reference documents
``cuda_llm.flash_decode(q_single, k_cache, v_cache)`` (``README.md:75`` in the reference project);
``paged_attention`` and ``fp8_paged_attention`` mirror the pybind signatures of the same path.  The
functions are those of the compiled extension ``fused_online_softmax_cuda`` beside this package."""
from fused_online_softmax_cuda import async_flash_decode as flash_decode  # noqa: F401
from fused_online_softmax_cuda import fp8_paged_attention_forward as fp8_paged_attention  # noqa: F401
from fused_online_softmax_cuda import paged_attention_forward as paged_attention  # noqa: F401

__all__ = ["flash_decode", "paged_attention", "fp8_paged_attention"]
