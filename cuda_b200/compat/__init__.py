"""Directory of the modules that carry the reference's own names.

Put it on ``sys.path`` (``sys.path.insert(0, cuda_b200.compat.PATH)``) and code written against the
reference imports ``fused_online_softmax_cuda`` (a compiled PyTorch extension, built by
``cuda_b200.build.build_extension`` from ``cuda_b200/ext/fused_online_softmax_cuda.cpp``; the
reference's is ``fused_softmax_binding.cpp``) or ``cuda_llm`` (its Python package) and gets this
library's decode entry points behind the same function names, argument names and defaults.  Only the
decode-attention path exists here; every other attribute raises ``AttributeError``."""
import os

PATH = os.path.dirname(os.path.abspath(__file__))
