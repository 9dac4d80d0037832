"""B200-native implementation of torch-spyre's data-parallel hot path.

The package keeps the reference's import name and public surface
(torch_spyre/__init__.py of the reference) while the kernels underneath are
hand-written sm_100a CUDA reached through the C ABI of libspyre_b200.so.
"""
from .layout import SpyreTensorLayout, storage_nbytes  # noqa: F401

__all__ = ["SpyreTensorLayout", "storage_nbytes"]
