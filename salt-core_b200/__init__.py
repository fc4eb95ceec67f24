"""B200 (sm_100a) backend for the quantized MoE feed-forward path of SALT-core.

The product is ``libsalt_gpu_b200.so`` (C ABI in ``include/salt_gpu_b200.h``);
this package is the Python plumbing around it: a loader that fails loudly when
the library or a usable GPU is missing, ctypes mirrors of the reference operator
surface (``backend.SaltGpu``) and of the device-resident stack (``stack.MoeStack``),
and the seeded synthetic tensors of the benchmark configurations (``synth``).
"""
from . import synth  # noqa: F401
from ._lib import LIB_PATH, library_path, load_library  # noqa: F401
