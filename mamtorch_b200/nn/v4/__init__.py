from .fullyconnected import FullyConnected  # noqa: F401
