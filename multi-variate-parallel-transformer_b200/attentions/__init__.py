"""Same import surface as the reference package (`attentions/__init__.py:1`)."""
from .attn import flash_mvpa as flashmvpa  # noqa: F401
from .attn import FlashMVPA, flash_mvpa, flash_mvpa_into  # noqa: F401
