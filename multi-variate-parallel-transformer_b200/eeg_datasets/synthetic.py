"""Seeded synthetic iEEG in the shape the reference's loader hands to the model
(`eeg_datasets/longterm.py:595-620`: (batch, segments, channels, samples), float32, 512 Hz, 5 s segments).

Per sample and channel one continuous record of `segments * samples` points: white Gaussian noise shaped
to a 1/f power spectrum (rFFT amplitudes scaled by f^-1/2, DC removed), z-scored per channel; then
`bursts` high-amplitude episodes per sample on a random 25-50 % of the channels: a 3-8 Hz sinusoid under a
Hann envelope, 2-10 s long, 5-10 standard deviations high; finally the record is cut into segments.
Runs on whatever device the generator lives on, so that a benchmark can create its input in HBM.
"""
from __future__ import annotations

import math

import torch


def synthetic_ieeg(batch: int, segments: int, channels: int, samples: int = 2560, seed: int = 0, bursts: int = 4,
                   rate_hz: float = 512.0, device="cpu", dtype=torch.float32) -> torch.Tensor:
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    n = segments * samples
    out = torch.empty((batch, segments, channels, samples), dtype=dtype, device=dev)
    f = torch.fft.rfftfreq(n, d=1.0 / rate_hz).to(dev)
    shape = torch.zeros_like(f)
    shape[1:] = f[1:].rsqrt()
    t = torch.arange(n, device=dev, dtype=torch.float32) / rate_hz
    for b in range(batch):                                   # one sample at a time keeps the peak memory low
        spec = torch.fft.rfft(torch.randn((channels, n), generator=g, device=dev), dim=-1) * shape
        rec = torch.fft.irfft(spec, n=n, dim=-1)
        rec = (rec - rec.mean(-1, keepdim=True)) / rec.std(-1, keepdim=True)
        for _ in range(bursts):
            r = torch.rand(5, generator=g, device=dev)
            frac, onset, dur = 0.25 + 0.25 * r[0], r[1], 2.0 + 8.0 * r[2]
            freq, amp = 3.0 + 5.0 * r[3], 5.0 + 5.0 * r[4]
            chans = torch.rand(channels, generator=g, device=dev) < frac
            t0 = onset * max(n / rate_hz - float(dur), 0.0)
            phase = ((t - t0) / dur).clamp(0, 1)
            env = torch.sin(math.pi * phase) ** 2 * ((t >= t0) & (t <= t0 + dur))
            rec += chans[:, None] * (amp * env * torch.sin(2 * math.pi * freq * (t - t0)))[None, :]
        out[b] = rec.view(channels, segments, samples).permute(1, 0, 2).to(dtype)
    return out
