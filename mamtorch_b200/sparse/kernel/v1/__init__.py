"""Sparse side of the package (`mamtorch/sparse/kernel/v1/`).  Filled in by the CSR kernels."""
__all__: list[str] = []
