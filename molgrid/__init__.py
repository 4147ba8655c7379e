"""``import molgrid``: the reference's module name on the CUDA path of this repository.

GridMaker, GridInterpolater, Transform, Quaternion, float3, the Grid/MGrid families, CoordinateSet,
Example and ExampleVec are the classes of the compiled module (``libmolgrid_b200.molgrid_native``:
pybind11 over the C++ host layer over the C ABI), so code written against libmolgrid's Python module
reaches the kernels through C++, as it does in the reference.  What the compiled module does not
define comes from the Python layer of ``libmolgrid_b200``: atom typers, pre-typed file readers, the
example provider (which hands out the compiled Example / CoordinateSet types here), the device-side
batch assembly and the torch.autograd bindings.  Calls that use this library's extensions to the
reference interface are served by the compiled GridMaker when every argument is a CUDA tensor
(batched arrays with per-example ``transforms=`` and ``n_atoms=``, batched backward: the calls of a
training loop) and by the Python layer's GridMaker with the same settings otherwise (host arrays,
lists of Transform objects, ``DeviceBatch`` arguments).
"""
import numpy as np

import libmolgrid_b200 as _py
from libmolgrid_b200 import build as _build

_build.build_library()
_build.build_native_module()
from libmolgrid_b200 import molgrid_native as native  # noqa: E402

# the Python layer first ...
from libmolgrid_b200 import *  # noqa: F401,F403,E402
# ... then the compiled classes over it
for _name in dir(native):
    if not _name.startswith("_"):
        globals()[_name] = getattr(native, _name)
del _name

from libmolgrid_b200.coord_cache import DeviceBatch as _DeviceBatch  # noqa: E402
from libmolgrid_b200 import grids as _grids  # noqa: E402

__all__ = sorted(set(list(_py.__all__) + [n for n in dir(native) if not n.startswith("_")] + ["native"]))


def set_gpu_enabled(on):
    """Whether MGrids handed to an operator are taken by their GPU side (both layers follow)."""
    native.set_gpu_enabled(bool(on))
    _grids.set_gpu_enabled(on)


def get_gpu_enabled():
    return native.get_gpu_enabled()


def _ndim(x):
    return len(x.shape) if hasattr(x, "shape") else -1


class GridMaker(native.GridMaker):
    """The compiled GridMaker with the reference's Python-side helpers (``make_ndarray``,
    ``make_tensor``) and this library's extensions served by the Python layer."""

    def _twin(self):
        g = _py.GridMaker(self.get_resolution(), self.get_dimension(), self.get_binary(),
                          self.get_radii_type_indexed(), self._radius_scale, self._grm)
        return g

    def __init__(self, resolution=0.5, dimension=23.5, binary=False, radius_type_indexed=False,
                 radius_scale=1.0, gaussian_radius_multiple=1.0):
        native.GridMaker.__init__(self, resolution, dimension, binary, radius_type_indexed, radius_scale,
                                  gaussian_radius_multiple)
        self._radius_scale, self._grm = radius_scale, gaussian_radius_multiple

    @staticmethod
    def _extension(args, kw):
        if "transforms" in kw or "n_atoms" in kw:
            return True
        return bool(args) and isinstance(args[0], _DeviceBatch)

    @staticmethod
    def _resident_batch(args, kw):
        """A batch the compiled module takes as it is: every array a CUDA tensor, per-example
        transforms as a (B,10) float32 CUDA tensor, atom counts as an int32 CUDA tensor."""
        import torch
        if len(args) < 5 or _ndim(args[1]) != 3 or set(kw) - {"transforms", "n_atoms"}:
            return False
        if not all(type(x) is torch.Tensor and x.is_cuda for x in args):
            return False
        tr, na = kw.get("transforms"), kw.get("n_atoms")
        if tr is not None and not (type(tr) is torch.Tensor and tr.is_cuda and tr.dtype is torch.float32):
            return False
        return na is None or (type(na) is torch.Tensor and na.is_cuda and na.dtype is torch.int32)

    def forward(self, *args, **kw):
        if self._resident_batch(args, kw):
            return native.GridMaker.forward(self, *args, **kw)
        # a batch of arrays about one common centre given as a tuple is this library's shorthand
        one_centre = len(args) > 1 and _ndim(args[1]) == 3 and _ndim(args[0]) < 0
        if self._extension(args, kw) or one_centre:
            return self._twin().forward(*args, **kw)
        return native.GridMaker.forward(self, *args, **kw)

    def backward(self, *args, **kw):
        if self._resident_batch(args, kw):
            return native.GridMaker.backward(self, *args, **kw)
        batched = len(args) > 1 and _ndim(args[1]) == 3
        if self._extension(args, kw) or batched:
            return self._twin().backward(*args, **kw)
        return native.GridMaker.backward(self, *args, **kw)

    def backward_arrays(self, *args, **kw):
        return self._twin().backward_arrays(*args, **kw)

    def forward_arrays(self, *args, **kw):
        return self._twin().forward_arrays(*args, **kw)

    def backward_gradients(self, *args, **kw):
        batched = len(args) > 1 and _ndim(args[1]) == 3
        if batched or self._extension(args, kw):
            return self._twin().backward_gradients(*args, **kw)
        return native.GridMaker.backward_gradients(self, *args, **kw)

    def make_ndarray(self, center, c):
        """New numpy array holding the grid of CoordinateSet ``c`` (python/__init__.py:29-35)."""
        t = np.zeros(self.grid_dimensions(c.max_type), dtype=np.float32)
        self.forward(center, c, t)
        return t

    def make_tensor(self, center, c):
        """New torch tensor holding the grid of ``c``: on the current GPU while ``get_gpu_enabled()``,
        else on the host (python/torch_bindings.py:32-42)."""
        import torch
        dev = torch.device("cuda", torch.cuda.current_device()) if get_gpu_enabled() else "cpu"
        t = torch.zeros(self.grid_dimensions(c.max_type), dtype=torch.float32, device=dev)
        self.forward(center, c, t)
        return t


def _native_set(cs):
    """The compiled CoordinateSet with the contents of a Python-layer one."""
    if cs.size() == 0:
        out = native.CoordinateSet()
        out.max_type = cs.max_type
        return out
    coords = cs.coords.tonumpy()
    radii = cs.radii.tonumpy()
    if cs.type_vector.size() > 0:
        return native.CoordinateSet(coords, cs.type_vector.tonumpy(), radii)
    return native.CoordinateSet(coords, cs.type_index.tonumpy(), radii, cs.max_type)


class ExampleProvider(_py.ExampleProvider):
    """The example provider handing out the compiled Example / ExampleVec types."""

    def _make(self, ref):
        pex = _py.ExampleProvider._make(self, ref)
        ex = native.Example()
        for s in pex.coord_sets:
            ex.coord_sets.append(_native_set(s))
        ex.labels = [float(v) for v in pex.labels]
        ex.group = int(pex.group) if pex.group is not None else -1
        return ex

    def next_batch(self, batch_size=0):
        B = int(batch_size) or int(self.settings.default_batch_size)
        if hasattr(self._order, "check_batch_size"):
            self._order.check_batch_size(B)
        return native.ExampleVec([self.next() for _ in range(B)])


class ExampleDataset(_py.ExampleDataset):
    """Random access to the examples of the lists, as compiled Example objects."""

    _make = ExampleProvider._make
