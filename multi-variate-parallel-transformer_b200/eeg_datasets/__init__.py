"""Stand-in for the reference's data package: only the synthetic iEEG generator lives here (the SWEC
recordings the reference loads, `eeg_datasets/longterm.py`, are not redistributable and not needed by
the kernels)."""
from .synthetic import synthetic_ieeg  # noqa: F401
