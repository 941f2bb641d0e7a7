"""faith_b200: forward linear-bound propagation operators for NVIDIA B200 (sm_100a).

Host-side mirror of the reference's operator interface over libfaith_b200.so:
  - `faith_b200.c_bound`  -- the pybind module surface of HandTunedKernels/kernel.cpp
  - `faith_b200.Bounds`   -- the `Bounds` class of Verifiers/Bounds.py with every operator on the GPU
  - `faith_b200.EncoderVerifier` -- the whole forward bound pass in one C++ driver call
  - `faith_b200.EpsilonSearch`   -- the reference's search for the certified radius (Verifier.py:106-147), batched
"""
from . import c_bound, ops  # noqa: F401
from .bounds import Bounds, BoundsLite  # noqa: F401
from .encoder import EncoderVerifier  # noqa: F401
from .search import EpsilonSearch, result_record, run_and_record, write_result  # noqa: F401
from ._lib import FaithError, load  # noqa: F401
