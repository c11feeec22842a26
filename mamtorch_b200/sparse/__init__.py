from . import kernel  # noqa: F401
