"""based_b200: B200 (sm_100a) kernels for the hot path of HazyResearch/based.

Linear attention with the 2nd-order Taylor feature map (prefill + recurrent decode) and
sliding-window softmax attention, behind mixer modules that keep the reference's
constructor / forward signatures and state-cache layout.

The compute path is a C-ABI CUDA library (``based_b200/_lib/libbased_b200.so``, declared in
``include/based_b200.h``).  There is no CPU or eager fallback: every op raises if the
library is missing.
"""
from .build import build_library, library_path  # noqa: F401

__all__ = ["build_library", "library_path"]
