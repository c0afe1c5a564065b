"""CPU oracle for the SDDMM hot path -- TEST INFRASTRUCTURE, not the product.

``oracle.cpu`` wraps ``liboracle.so`` (the plain-C restatement in
``sddmm_oracle.c``); ``oracle.ref`` wraps ``_ref/libsddmm_ref.so`` (the
reference's own translation unit compiled through ``ref_bridge.cu``) and is
``None`` when that library has not been built.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package.  ``sddmm_gpu_b200`` never does.
"""
from . import pyoracle as _py

cpu = _py.load_cpu()
ref = _py.load_ref()
build = _py.build
