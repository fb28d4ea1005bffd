"""ferrograd_b200: a B200 (sm_100a) execution backend for ferrograd's hot path.

The product is libferrograd_b200.so (C ABI in include/ferrograd_b200.h).  This package
is its Python host side: `GpuContext` mirrors the reference's context interface, and
`mlp` drives data-parallel MLP training steps through the same entry points.
"""
from .backend import Buffer, FgError, GpuContext, Plan, Tensor  # noqa: F401
