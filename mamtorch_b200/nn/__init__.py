"""Modules (`mamtorch/nn/__init__.py`): v1 and v4 generations, `FullyConnected` = v4, plus the
convolution modules the reference keeps only as text backups (`mamtorch/nn/backup/`)."""
from . import functional
from . import v1
from . import v4
from . import vit
from .conv import MAMConv1d, MAMConv2d
from .v4.fullyconnected import FullyConnected

__all__ = ["FullyConnected", "MAMConv1d", "MAMConv2d", "functional", "v1", "v4", "vit"]
