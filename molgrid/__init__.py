"""``import molgrid``: the reference's module name for the classes of libmolgrid_b200 (GridMaker,
GridInterpolater, Transform, Quaternion, float3, Grid/MGrid families, CoordinateSet, Example,
ExampleProvider, Coords2Grid ...), so that code written against libmolgrid's Python module runs on
the CUDA path of this repository without edits."""
from libmolgrid_b200 import *  # noqa: F401,F403
from libmolgrid_b200 import __all__  # noqa: F401
