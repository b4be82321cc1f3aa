"""B200-native MXFP / minifloat fake-quantisation behind the mase-triton Python API.

``import mase_triton_b200 as mase_triton`` gives the same module paths, names and
signatures as the reference for this path: ``mxfp.functional``, ``mxfp.layers``,
``mxfp.meta``, ``minifloat.functional``, ``minifloat.layers``, ``minifloat.meta``,
``manager.KernelManager`` and the ``utils`` helpers the layers use.  All numeric
work runs in hand-written sm_100a CUDA kernels behind the C ABI declared in
``include/mxq.h``; there is no CPU fallback.
"""

from . import manager, minifloat, mxfp, utils  # noqa: F401

__version__ = "0.1.0"
