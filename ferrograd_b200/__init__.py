"""ferrograd_b200: a B200 (sm_100a) execution backend for ferrograd's hot path.

The product is libferrograd_b200.so (C ABI in include/ferrograd_b200.h).  This package
is its Python host side: `GpuContext` mirrors the reference's context interface, `graph`
mirrors its graph API (Graph / define_ops / alloc_tensors / schedule / dispatch_*), and
`mlp` drives data-parallel MLP training steps through the same entry points.
"""
from .backend import Buffer, FgError, GpuContext, Plan, Tensor  # noqa: F401
from .graph import (BINARY_CROSS_ENTROPY, CROSS_ENTROPY, MEAN_SQUARED_ERROR, Graph, Metadata, Optim, SimpleDType,  # noqa: F401
                    f32_bits)
from . import bpat  # noqa: F401,E402
