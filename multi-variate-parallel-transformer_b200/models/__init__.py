"""Model-level code around the MVPA layer, with the reference's class names (`models/__init__.py`,
`models/mvpformer.py`, `models/fftencoder.py`) and state-dict layout, without the training stack."""
from torch.nn import Module


class BrainEncoder(Module):
    """Base class name of the reference's encoders (`models/__init__.py`)."""


class BrainDecider(Module):
    """Base class name of the reference's heads (`models/__init__.py`)."""


from .fftencoder import WaveEncoder  # noqa: E402,F401
from .mvpformer import (ClassificationHMVPFormer, HMVPFormer, MVPFormerBlock, MVPFormerConfig,  # noqa: E402,F401
                        MVPFormerHead, MVPFormerModel, RMSNorm)
