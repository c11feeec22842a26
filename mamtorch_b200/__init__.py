"""B200-native Multiply-And-Max/min (MAM) layers: a drop-in for the hot path of SSIGPRO/mamtorch.

    import mamtorch_b200 as mamtorch

keeps the reference's import surface (`mamtorch/__init__.py:1-7`): `mamtorch.kernel.v1 / v4`
(plus v2 / v3, which the reference ships as source only), `mamtorch.nn.FullyConnected`,
`mamtorch.sparse`, and the deprecated `mamtorch.MAMDense`.  The operators live under the same
`torch.ops.mamtorch_kernel_v*` names and run hand-written sm_100a kernels through the C ABI in
include/mam_b200.h.  There is no CPU implementation.
"""
from . import _lib

_lib.load_ops()

from . import kernel  # noqa: E402
from . import nn  # noqa: E402
from . import sparse  # noqa: E402
from .nn.compat import MAMDense  # noqa: E402,F401

__version__ = "0.1.0"
