"""B200 (sm_100a) implementation of libmolgrid's gridding path behind the reference's interface.

``GridMaker``, ``GridInterpolater``, ``Transform``, ``Quaternion``, ``float3``, the ``Grid``/``MGrid``
families, ``CoordinateSet`` and ``Example`` mirror the classes of the reference's ``molgrid`` Python
module for this path (``import libmolgrid_b200 as molgrid``); all arithmetic runs in
hand-written CUDA kernels reached through the C ABI of ``include/lmg_b200.h``.
"""
from .api import (GridMaker, GridInterpolater, Transform, Quaternion, float3,  # noqa: F401
                  set_random_seed)
from .torch_bindings import (Coords2Grid, Coords2GridFunction, BatchedCoords2GridFunction,  # noqa: F401
                             Grid2CoordsGradientFunction)
from .grids import *  # noqa: F401,F403  Grid1f..Grid8dCUDA, MGrid1f..MGrid8d, set/get_gpu_enabled, ...
from .grids import __all__ as _grid_names
from .coordinates import CoordinateSet, Example, ExampleVec  # noqa: F401
from .atom_typing import (GninaIndexTyper, FileAtomMapper, FileMappedGninaTyper, NullIndexTyper,  # noqa: F401
                          default_receptor_typer, default_ligand_typer, defaultGninaReceptorTyper,
                          defaultGninaLigandTyper)
from .coord_cache import (CoordCache, DeviceBatch, ExampleDataset, ExampleProvider,  # noqa: F401
                          read_gninatypes)
from .example_order import ExampleProviderSettings, IterationScheme  # noqa: F401
from . import _cabi  # noqa: F401

__all__ = ["GridMaker", "GridInterpolater", "Transform", "Quaternion", "float3", "set_random_seed",
           "Coords2Grid", "Coords2GridFunction", "BatchedCoords2GridFunction", "Grid2CoordsGradientFunction",
           "CoordinateSet", "Example", "ExampleVec", "GninaIndexTyper", "FileAtomMapper",
           "FileMappedGninaTyper", "NullIndexTyper", "default_receptor_typer", "default_ligand_typer",
           "defaultGninaReceptorTyper", "defaultGninaLigandTyper", "CoordCache",
           "ExampleProvider", "ExampleDataset", "ExampleProviderSettings", "IterationScheme", "DeviceBatch",
           "read_gninatypes"] + list(_grid_names)
