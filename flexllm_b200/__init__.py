"""flexllm_b200 -- B200 (sm_100a) kernels for FlexLLM's quantized Llama-3.2-1B operator path.

The product is ``libflexllm_b200.so`` (CUDA kernels behind the C ABI of ``include/flexllm_b200.h``)
plus the C++ host API in ``include/flexllm/``. This Python package is plumbing only: it loads the
library with ctypes and hands it device pointers of torch tensors. There is no CPU or PyTorch
fallback: if the library is missing or a call fails, an exception is raised.
"""
from . import _lib
from .ops import *  # noqa: F401,F403
from .ops import FlexLLMError, lib  # noqa: F401
