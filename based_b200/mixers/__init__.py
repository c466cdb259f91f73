"""Drop-in mixer modules (same constructor / forward signatures and state layout as
based/models/mixers/linear_attention.py and slide_attention.py of the reference)."""
