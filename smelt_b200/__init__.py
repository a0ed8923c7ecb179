"""smelt_b200 — B200 (sm_100a) kernels for the Smelt decode hot path behind a C ABI.

``capi`` binds ``libsmelt_cuda.so``; ``synth`` makes seeded synthetic packages; ``package``
lays tensors out as a ``weights.bin`` image and drives the decoder through dispatch records.
"""
from . import capi, synth  # noqa: F401

__all__ = ["capi", "synth"]
