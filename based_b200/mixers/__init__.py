"""Drop-in mixer modules (same constructor / forward signatures and state layout as
based/models/mixers/linear_attention.py and slide_attention.py of the reference)."""
from .linear_attention import FeatureMap, LinearAttention, TaylorExp  # noqa: F401
from .slide_attention import RotaryEmbedding, SlidingAttention  # noqa: F401
