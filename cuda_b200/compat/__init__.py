"""Import shims under the reference's own module names.

Put this directory on ``sys.path`` (``sys.path.insert(0, cuda_b200.compat.PATH)``) and code written
against the reference imports ``fused_online_softmax_cuda`` (the pybind module of
``fused_softmax_binding.cpp`` in the reference project) or ``cuda_llm`` (its Python package) and
gets this library's decode ops behind the same function names and positional signatures.  Only
the decode-attention path exists here; every other attribute raises ``AttributeError``."""
import os

PATH = os.path.dirname(os.path.abspath(__file__))
