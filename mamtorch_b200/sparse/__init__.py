from . import kernel  # noqa: F401
from .pruned import (PrunedFullyConnected, global_magnitude_threshold, magnitude_keep_mask,  # noqa: F401
                     magnitude_threshold)
