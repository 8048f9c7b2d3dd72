"""B200-native Flash-MVPA: the fused multi-variate parallel attention of MVPFormer.

The directory is laid out so that putting it on ``sys.path`` shadows exactly two
reference packages, ``attentions`` and ``layers``: the reference's model code
(`models/mvpformer.py`) then imports this implementation unchanged.  Importing this
package does that path insertion and re-exports the public names.
"""
import os as _os
import sys as _sys

_here = _os.path.dirname(_os.path.abspath(__file__))
if _here not in _sys.path:
    _sys.path.insert(0, _here)

import mvpa_native as native  # noqa: E402
from attentions import FlashMVPA, flash_mvpa, flashmvpa  # noqa: E402,F401
from layers import MVPFormerGQAAttention, MVPFormerGQAFlashAttention  # noqa: E402,F401

__all__ = ["native", "flash_mvpa", "flashmvpa", "FlashMVPA", "MVPFormerGQAAttention",
           "MVPFormerGQAFlashAttention"]
