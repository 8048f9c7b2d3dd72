"""Same import surface as the reference package (`layers/__init__.py:1`)."""
from .mvpa import MVPFormerGQAAttention, MVPFormerGQAFlashAttention  # noqa: F401
