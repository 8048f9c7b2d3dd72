"""`WaveEncoder` with the reference's constructor, parameter names and output
(`models/fftencoder.py:49-97`): every level of the periodic db4 wavelet transform of a segment,
concatenated, RMS-normalised, projected to the model width.

The reference runs `ptwt.wavedec` (a padded strided convolution per level, eight launches plus the
concatenation), a Triton RMSNorm and the projection.  Here one kernel (`mvpa_wave_encode`) produces the
normalised coefficient row of each segment in shared memory and writes it once, in the projection's
dtype, padded to a multiple of 32 columns so that the projection is an aligned cuBLAS GEMM on a
zero-padded copy of `proj.weight`.  The filters are derived numerically (`mvpa_ops.db4_filters`); `pywt`
is not needed.  CUDA tensors only.
"""
from __future__ import annotations

import torch

import mvpa_ops
from models import BrainEncoder


class _Weight(torch.nn.Module):
    """Holds `weight` under the name the reference's RMSNorm does (`ln.weight`)."""

    def __init__(self, n, eps):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(n))
        self.eps = eps


class WaveEncoder(BrainEncoder):
    def __init__(self, size_input: int, size_output: int, wavelet: str = "db4", gradient_checkpointing: bool = False):
        super().__init__()
        if wavelet != "db4":
            raise NotImplementedError("WaveEncoder: only the db4 wavelet of the shipped configurations is built")
        self.size_input, self.size_output = size_input, size_output
        self.gradient_checkpointing = gradient_checkpointing
        sizes, total = mvpa_ops.wave_sizes(size_input)
        self.sizes = sizes + [sizes[-1]]               # `_compute_dwt_size` (`models/fftencoder.py:69-78`)
        self.dwt_size = total
        self.ln = _Weight(self.dwt_size, 1e-5)
        self.proj = torch.nn.Linear(self.dwt_size, size_output, bias=False)
        self._padded = None                             # (version, zero-padded copy of proj.weight)

    def _proj_padded(self):
        w = self.proj.weight
        k = (self.dwt_size + 31) // 32 * 32
        tag = (w._version, w.data_ptr(), w.dtype)
        if self._padded is None or self._padded[0] != tag:
            wp = torch.zeros((w.shape[0], k), dtype=w.dtype, device=w.device)
            wp[:, :self.dwt_size] = w.detach()
            self._padded = (tag, wp)
        return self._padded[1]

    @torch.no_grad()
    def block(self, x: torch.Tensor) -> torch.Tensor:
        """Normalised coefficient rows (rows, K padded to a multiple of 32) in the projection's dtype."""
        wp = self._proj_padded()
        return mvpa_ops.wave_encode(x.contiguous(), self.ln.weight.detach().to(wp.dtype).contiguous(), self.ln.eps,
                                    pad_to=wp.shape[1])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x (rows, size_input) fp32 or bf16 -> (rows, size_output)."""
        return torch.nn.functional.linear(self.block(x), self._proj_padded())

    encode = forward
