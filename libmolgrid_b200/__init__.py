"""B200 (sm_100a) implementation of libmolgrid's gridding path behind the reference's interface.

``GridMaker``, ``GridInterpolater``, ``Transform``, ``Quaternion`` and ``float3`` mirror the
classes of the reference's ``molgrid`` Python module for this path; all arithmetic runs in
hand-written CUDA kernels reached through the C ABI of ``include/lmg_b200.h``.
"""
from .api import (GridMaker, GridInterpolater, Transform, Quaternion, float3,  # noqa: F401
                  set_random_seed)
from .torch_bindings import (Coords2Grid, Coords2GridFunction, BatchedCoords2GridFunction,  # noqa: F401
                             Grid2CoordsGradientFunction)
from . import _cabi  # noqa: F401

__all__ = ["GridMaker", "GridInterpolater", "Transform", "Quaternion", "float3", "set_random_seed",
           "Coords2Grid", "Coords2GridFunction", "BatchedCoords2GridFunction", "Grid2CoordsGradientFunction"]
