"""sddmm_gpu_b200 -- B200 (sm_100a) SDDMM engine: P = S o (W H^T) on a row-sorted COO.

The product is the C ABI of ``csrc/libsddmm_b200.so`` (declared in
``include/sddmm_b200.h``); ``api`` is its ctypes mirror, ``synth`` the seeded
synthetic inputs of the benchmark configurations, ``multi_gpu`` the row-block
sharding over ``torch.distributed``.
"""
from . import api, synth  # noqa: F401
from .api import Handle, Plan, SddmmError  # noqa: F401
