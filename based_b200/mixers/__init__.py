"""Drop-in mixer modules (same constructor / forward signatures and state layout as
based/models/mixers/linear_attention.py, slide_attention.py and convolution.py of the reference)."""
from .linear_attention import FeatureMap, LinearAttention, TaylorExp  # noqa: F401
from .slide_attention import RotaryEmbedding, SlidingAttention  # noqa: F401
from .convolution import BaseConv, ShortConvolution  # noqa: F401
