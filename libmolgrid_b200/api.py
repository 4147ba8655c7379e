"""Python host mirror of the reference's gridding classes over the CUDA C ABI.

Same names, argument order and error behaviour as the ``molgrid`` Python module for the path:
``GridMaker`` (python/bindings.in.cpp:816-918), ``GridInterpolater`` (:920-943), ``Transform``
(:497-520), ``Quaternion`` (:478-493), ``float3`` (:455-475), ``set_random_seed`` (:400).
Arrays are torch tensors.  CUDA float32 tensors are used in place; CPU tensors and numpy arrays
are staged through device memory around the call (every result is computed on the GPU).
"""
import ctypes

import numpy as np
import torch

from . import _cabi
from . import grids as _grids
from ._cabi import check


# ------------------------------------------------------------------------------------------------
# small value types
# ------------------------------------------------------------------------------------------------
class float3(object):
    """x, y, z triple; also constructible from a 3-tuple, like the reference's float3."""

    def __init__(self, x=0.0, y=0.0, z=0.0):
        if not np.isscalar(x):
            x, y, z = x[0], x[1], x[2]
        self.x, self.y, self.z = float(np.float32(x)), float(np.float32(y)), float(np.float32(z))

    def __getitem__(self, i):
        if i in (0, 1, 2):
            return (self.x, self.y, self.z)[i]
        raise IndexError("float3")

    def __iter__(self):
        return iter((self.x, self.y, self.z))

    def __len__(self):
        return 3

    def __repr__(self):
        return "float3(%r, %r, %r)" % (self.x, self.y, self.z)


def _f3(v):
    return v if isinstance(v, float3) else float3(v)


_F = np.float32


class Quaternion(object):
    """Float quaternion with the reference's operation order (include/libmolgrid/quaternion.h)."""

    def __init__(self, a=1.0, b=0.0, c=0.0, d=0.0):
        self.a, self.b, self.c, self.d = _F(a), _F(b), _F(c), _F(d)

    def R_component_1(self): return float(self.a)
    def R_component_2(self): return float(self.b)
    def R_component_3(self): return float(self.c)
    def R_component_4(self): return float(self.d)
    def real(self): return float(self.a)

    def conj(self):
        return Quaternion(self.a, -self.b, -self.c, -self.d)

    def norm(self):
        return float(self.a * self.a + self.b * self.b + self.c * self.c + self.d * self.d)

    def inverse(self):
        n = self.a * self.a + self.b * self.b + self.c * self.c + self.d * self.d
        return Quaternion(self.a / n, -self.b / n, -self.c / n, -self.d / n)

    def __mul__(self, r):
        a, b, c, d = self.a, self.b, self.c, self.d
        return Quaternion(a * r.a - b * r.b - c * r.c - d * r.d,
                          a * r.b + b * r.a + c * r.d - d * r.c,
                          a * r.c - b * r.d + c * r.a + d * r.b,
                          a * r.d + b * r.c - c * r.b + d * r.a)

    def __truediv__(self, r):
        a, b, c, d = self.a, self.b, self.c, self.d
        den = r.a * r.a + r.b * r.b + r.c * r.c + r.d * r.d
        return Quaternion((a * r.a + b * r.b + c * r.c + d * r.d) / den,
                          (-a * r.b + b * r.a - c * r.d + d * r.c) / den,
                          (-a * r.c + b * r.d + c * r.a - d * r.b) / den,
                          (-a * r.d - b * r.c + c * r.b + d * r.a) / den)

    def __eq__(self, r):
        return (self.a, self.b, self.c, self.d) == (r.a, r.b, r.c, r.d)

    def rotate(self, x, y, z):
        n = _F(self.norm())
        cn = Quaternion(self.a / n, -self.b / n, -self.c / n, -self.d / n)
        p = self * Quaternion(0, x, y, z) * cn
        return float3(p.b, p.c, p.d)

    def transform(self, x, y, z, center, translate):
        c, t = _f3(center), _f3(translate)
        p = self.rotate(_F(x) - _F(c.x), _F(y) - _F(c.y), _F(z) - _F(c.z))
        return float3(_F(p.x) + _F(c.x) + _F(t.x), _F(p.y) + _F(c.y) + _F(t.y), _F(p.z) + _F(c.z) + _F(t.z))

    def __repr__(self):
        return "Quaternion(%r, %r, %r, %r)" % (float(self.a), float(self.b), float(self.c), float(self.d))


def set_random_seed(seed):
    """Reseed the engine that draws random Transforms (python/bindings.in.cpp:400)."""
    _cabi.lib().lmg_set_random_seed(int(seed) & 0xffffffff)


# ------------------------------------------------------------------------------------------------
# tensor plumbing
# ------------------------------------------------------------------------------------------------
def _stream_ptr(device):
    # the raw handle of torch's current stream on the device, without building a Stream object
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(device.index))


class _Arg(object):
    """A float32 array argument made resident on the GPU for the duration of one call."""

    def __init__(self, obj, device, ndim, name, output=False):
        self.host = None
        if type(obj) is torch.Tensor and obj.is_cuda and obj.dtype is torch.float32 and obj.dim() == ndim \
                and obj.device == device and obj.is_contiguous():
            self.t, self.output = obj, output      # the common case: a resident tensor, nothing to stage
            return
        obj = _grids.operand_tensor(obj)
        if isinstance(obj, np.ndarray):
            if obj.dtype != np.float32 or not obj.flags["C_CONTIGUOUS"]:
                raise ValueError("%s: numpy arrays must be C-contiguous float32" % name)
            self.host = torch.from_numpy(obj)
            t = self._stage(self.host, device, output)
        elif torch.is_tensor(obj):
            if obj.dtype != torch.float32:
                raise ValueError("%s: tensors must be float32 (double grids are not supported on the GPU path)" % name)
            if not obj.is_contiguous():
                raise ValueError("%s: tensor is not contiguous" % name)
            if obj.is_cuda:
                if obj.device != device:
                    raise ValueError("%s: tensor on %s but current device is %s" % (name, obj.device, device))
                t = obj
            else:
                self.host = obj
                t = self._stage(obj, device, output)
        else:
            raise TypeError("%s: expected a Grid, MGrid, torch tensor or numpy array" % name)
        if t.dim() != ndim:
            raise TypeError("%s: expected %d dimensions, got %d" % (name, ndim, t.dim()))
        self.t = t
        self.output = output

    @staticmethod
    def _stage(host, device, output):
        # outputs are fully overwritten by the kernels, so only inputs are copied in
        if output:
            return torch.empty(host.shape, dtype=host.dtype, device=device)
        return host.to(device, non_blocking=True)

    @property
    def ptr(self):
        return ctypes.c_void_p(self.t.data_ptr())

    def finish(self):
        if self.output and self.host is not None:
            self.host.copy_(self.t)


_have_cuda = []   # filled on the first successful check


def _current_device():
    if not _have_cuda:
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this library has no CPU path")
        _have_cuda.append(True)
    return torch.device("cuda", torch.cuda.current_device())


_workspaces = {}
_transform_ring = {}   # (device, batch) -> pinned staging buffers of GridMaker.batch_transforms


def _workspace(device, nbytes):
    """Per-device scratch buffer reused across calls (grown on demand)."""
    ws = _workspaces.get(device)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
        _workspaces[device] = ws
    return ws


MAX_WORKSPACE_BYTES = 4 << 30  # larger batches run in several passes inside the C call


class Transform(object):
    """Rotation about a centre followed by a translation (include/libmolgrid/transform.h)."""

    def __init__(self, *args, **kw):
        self.Q = Quaternion()
        self.center = float3(0, 0, 0)
        self.translate = float3(0, 0, 0)
        if args and isinstance(args[0], Quaternion):
            self.Q = args[0]
            if len(args) > 1:
                self.center = _f3(args[1])
            if len(args) > 2:
                self.translate = _f3(args[2])
        elif args or kw:
            # Transform(center, random_translate=0, random_rotation=False), src/transform.cpp:13-33
            center = _f3(args[0] if args else kw["center"])
            rt = args[1] if len(args) > 1 else kw.get("random_translate", 0.0)
            rr = args[2] if len(args) > 2 else kw.get("random_rotation", False)
            s = _cabi.TransformStruct()
            c = (ctypes.c_float * 3)(center.x, center.y, center.z)
            check(_cabi.lib().lmg_transform_random(ctypes.byref(s), c, float(rt), int(bool(rr))))
            self.Q = Quaternion(*s.q)
            self.center = center
            self.translate = float3(*s.translate)

    def get_quaternion(self): return self.Q
    def get_rotation_center(self): return self.center
    def get_translation(self): return self.translate
    def set_quaternion(self, q): self.Q = q
    def set_rotation_center(self, c): self.center = _f3(c)
    def set_translation(self, t): self.translate = _f3(t)

    def is_identity(self):
        return self.Q == Quaternion() and tuple(self.translate) == (0.0, 0.0, 0.0)

    def struct(self):
        s = _cabi.TransformStruct()
        s.q[:] = [self.Q.a, self.Q.b, self.Q.c, self.Q.d]
        s.center[:] = list(self.center)
        s.translate[:] = list(self.translate)
        return s

    def as_row(self):
        """The 10 floats of lmg_transform: q, centre, translation."""
        return [float(self.Q.a), float(self.Q.b), float(self.Q.c), float(self.Q.d)] + \
            list(self.center) + list(self.translate)

    def _apply(self, fn, inp, out, dotranslate):
        dev = _current_device()
        i = _Arg(inp, dev, 2, "in")
        o = _Arg(out, dev, 2, "out", output=True)
        # Transform::checkGrids, include/libmolgrid/transform.h:130-147
        if i.t.shape[0] != o.t.shape[0]:
            raise ValueError("Different dimensions and input and output coordinates grids.")
        if i.t.shape[1] != 3:
            raise ValueError("Input coordinates wrong dimension.")
        if o.t.shape[1] != 3:
            raise ValueError("Output coordinates are wrong dimension.")
        s = self.struct()
        check(fn(ctypes.byref(s), int(i.t.shape[0]), i.ptr, o.ptr, int(bool(dotranslate)), _stream_ptr(dev)))
        o.finish()

    def _apply_sets(self, fn, inp, out, dotranslate):
        """CoordinateSet and Example overloads (src/transform.cpp:35-55): only coordinates change;
        types and radii are copied when ``out`` is another object."""
        from .coordinates import CoordinateSet, Example
        if isinstance(inp, Example):
            if not isinstance(out, Example):
                raise TypeError("Example input needs an Example output")
            if out is not inp:
                out.coord_sets = [s.clone() for s in inp.coord_sets]
                out.labels, out.group, out.seqcont = list(inp.labels), inp.group, inp.seqcont
            for s in out.coord_sets:
                self._apply_sets(fn, s, s, dotranslate)
            return True
        if isinstance(inp, CoordinateSet):
            if not isinstance(out, CoordinateSet):
                raise TypeError("CoordinateSet input needs a CoordinateSet output")
            if out is not inp:
                c = inp.clone()
                out.coords, out.type_index, out.type_vector = c.coords, c.type_index, c.type_vector
                out.radii, out.max_type, out.src = c.radii, c.max_type, c.src
            if out.coords.size() > 0:
                g = out.coords.gpu()
                out.coords.togpu()
                self._apply(fn, g, g, dotranslate)
            return True
        return False

    def forward(self, inp, out, dotranslate=True):
        if not self._apply_sets(_cabi.lib().lmg_transform_forward, inp, out, dotranslate):
            self._apply(_cabi.lib().lmg_transform_forward, inp, out, dotranslate)

    def backward(self, inp, out, dotranslate=True):
        if not self._apply_sets(_cabi.lib().lmg_transform_backward, inp, out, dotranslate):
            self._apply(_cabi.lib().lmg_transform_backward, inp, out, dotranslate)


def _transforms_tensor(transforms, batch, device):
    """[batch][10] device tensor from a tensor/array or a list of Transform objects."""
    if transforms is None:
        return None
    if torch.is_tensor(transforms):
        t = transforms
    elif isinstance(transforms, np.ndarray):
        t = torch.from_numpy(np.ascontiguousarray(transforms, dtype=np.float32))
    else:
        t = torch.tensor([tr.as_row() for tr in transforms], dtype=torch.float32)
    if t.dtype != torch.float32 or tuple(t.shape) != (batch, 10):
        raise ValueError("transforms must be float32 of shape (batch, 10)")
    return t.contiguous().to(device)


class GridMaker(object):
    """Density / occupancy grids from atoms and the matching backward passes.

    Mirrors libmolgrid::GridMaker (include/libmolgrid/grid_maker.h) for float CUDA grids; every
    overload taking raw arrays is here, single example or batched, selected by array rank as the
    reference's overload set is (python/bindings.in.cpp:845-918).
    """

    def __init__(self, resolution=0.5, dimension=23.5, binary=False, radius_type_indexed=False,
                 radius_scale=1.0, gaussian_radius_multiple=1.0):
        self.s = _cabi.GridMakerStruct()
        check(_cabi.lib().lmg_gridmaker_init(ctypes.byref(self.s), resolution, dimension, int(bool(binary)),
                                             int(bool(radius_type_indexed)), radius_scale,
                                             gaussian_radius_multiple))

    # --- settings, include/libmolgrid/grid_maker.h:88-113.  As in the reference, the setters only
    # recompute the number of grid points, never the density coefficients.
    def _redim(self):
        self.s.dim = int(np.round(np.float32(self.s.dimension) / np.float32(self.s.resolution)) + 1)

    def get_resolution(self): return self.s.resolution
    def set_resolution(self, r): self.s.resolution = r; self._redim()
    def get_dimension(self): return self.s.dimension
    def set_dimension(self, d): self.s.dimension = d; self._redim()
    def get_binary(self): return bool(self.s.binary)
    def set_binary(self, b): self.s.binary = int(bool(b))
    def get_radii_type_indexed(self): return bool(self.s.radii_type_indexed)
    def set_radii_type_indexed(self, b): self.s.radii_type_indexed = int(bool(b))
    def get_radiusmultiple(self): return float(_F(self.s.radius_scale) * _F(self.s.final_radius_multiple))

    def spatial_grid_dimensions(self):
        return (int(self.s.dim),) * 3

    def grid_dimensions(self, ntypes):
        return (int(ntypes),) + self.spatial_grid_dimensions()

    def make_tensor(self, center, c):
        """New torch tensor holding the grid of CoordinateSet ``c`` about ``center``: on the current
        GPU while ``get_gpu_enabled()``, else on the host (python/torch_bindings.py:32-42)."""
        dims = self.grid_dimensions(c.max_type)
        t = torch.zeros(dims, dtype=torch.float32, device=_current_device() if _grids.get_gpu_enabled() else "cpu")
        self.forward(center, c, t)
        return t

    def empty_grid(self, ntypes, batch=None, device=None):
        """Zero tensor of this grid maker's shape for ``ntypes`` channels (optionally batched)."""
        shape = self.grid_dimensions(ntypes)
        if batch is not None:
            shape = (batch,) + shape
        return torch.zeros(shape, dtype=torch.float32, device=device or _current_device())

    def make_ndarray(self, center, c):
        """New numpy array holding the grid of CoordinateSet ``c`` (python/__init__.py:29-35)."""
        t = np.zeros(self.grid_dimensions(c.max_type), dtype=np.float32)
        self.forward(center, c, t)
        return t

    # --- argument handling -------------------------------------------------------------------
    def _atoms(self, center, coords, types, radii, transforms=None, n_atoms=None):
        dev = _current_device()
        coords, types, radii = (_grids.operand_tensor(x) for x in (coords, types, radii))
        batched = (coords.ndim if isinstance(coords, np.ndarray) else coords.dim()) == 3
        keep = []
        A = _cabi.AtomsStruct()
        c = _Arg(coords, dev, 3 if batched else 2, "coords")
        tnd = types.ndim if isinstance(types, np.ndarray) else types.dim()
        vec = tnd == (3 if batched else 2)
        t = _Arg(types, dev, tnd, "types")
        r = _Arg(radii, dev, 2 if batched else 1, "radii")
        keep += [c, t, r]
        B = int(c.t.shape[0]) if batched else 1
        N = int(c.t.shape[1] if batched else c.t.shape[0])
        if c.t.shape[-1] != 3:
            raise ValueError("Coordinates and radius wrong secondary dimension")
        if batched:
            # batch-size checks of include/libmolgrid/grid_maker.h:270-282
            for name, x in (("types", t.t), ("radii", r.t)):
                if x.shape[0] != B:
                    raise ValueError("Mismatched batch sizes: %d vs %d" % (x.shape[0], B))
        A.batch, A.max_atoms = B, N
        A.coords, A.radii = c.t.data_ptr(), r.t.data_ptr()
        tshape = tuple(t.t.shape[1:] if batched else t.t.shape)
        if tshape[0] != N:
            raise IndexError("type_index does not match number of atoms: %d vs %d" % (tshape[0], N))
        if vec:
            A.type_vector = t.t.data_ptr()
            A.ntypes = int(tshape[1])
        else:
            A.type_index = t.t.data_ptr()
        nr = int(r.t.shape[-1])
        if center is not None and (torch.is_tensor(center) or isinstance(center, np.ndarray)) and batched:
            ce = _Arg(center, dev, 2, "centers")
            if ce.t.shape[0] != B or ce.t.shape[1] != 3:
                raise ValueError("Mismatched batch sizes: %d vs %d" % (ce.t.shape[0], B))
            keep.append(ce)
            A.centers = ce.t.data_ptr()
        else:
            cf = _f3(center)
            A.center_host[:] = [cf.x, cf.y, cf.z]
        if isinstance(transforms, Transform):
            ts = transforms.struct()
            keep.append(ts)
            A.transform_host = ctypes.pointer(ts)
        elif transforms is not None:
            tt = _transforms_tensor(transforms, B, dev)
            keep.append(tt)
            A.transforms = tt.data_ptr()
        if n_atoms is not None:
            na = n_atoms.to(device=dev, dtype=torch.int32).contiguous()
            if na.numel() != B:
                raise ValueError("n_atoms must have one entry per example")
            keep.append(na)
            A.n_atoms = na.data_ptr()
        return dev, A, keep, batched, vec, B, N, nr

    def _check_radii(self, vec, N, T, nr, exc):
        # src/grid_maker.cpp:51,83-88 (forward, std::out_of_range) and :446-452,494-498 (backward,
        # std::invalid_argument)
        if vec and self.s.radii_type_indexed:
            if nr != T:
                raise exc("radii does not match number of types: %d vs %d" % (nr, T))
        elif nr != N:
            raise exc("radii does not match number of atoms: %d vs %d" % (nr, N))

    def _ws(self, dev, op, B, N, T, vec):
        # the size depends on the shapes and the settings: asked once per combination
        key = (op, B, N, T, vec, self.s.radii_type_indexed, self.s.binary, self.s.dim)
        sizes = self.__dict__.setdefault("_ws_sizes", {})
        need = sizes.get(key)
        if need is None:
            need = sizes[key] = _cabi.lib().lmg_workspace_bytes(ctypes.byref(self.s), op, B, N, T, int(vec))
        return _workspace(dev, min(need, MAX_WORKSPACE_BYTES))

    # --- forward -----------------------------------------------------------------------------
    def forward(self, *args, **kw):
        """The reference's forward overload set (python/bindings.in.cpp:829-868):

        * ``forward(example, grid, random_translation=0.0, random_rotation=False)``
        * ``forward(examples, grid5, random_translation=0.0, random_rotation=False)``
        * ``forward(center, coordinate_set, grid)``
        * ``forward(example, transform, grid)``
        * ``forward(center, coords, types, radii, grid)`` - index or vector types, single or batched
          (plus the ``transforms=`` / ``n_atoms=`` extensions of :meth:`forward_arrays`).
        """
        from .coordinates import CoordinateSet, Example
        from .coord_cache import DeviceBatch
        a0 = args[0] if args else kw.get("example", kw.get("examples", kw.get("examplevec")))
        if isinstance(a0, DeviceBatch):
            rest = list(args[1:])
            grid = rest[0] if rest else kw["grid"]
            rt = rest[1] if len(rest) > 1 else kw.get("random_translation", 0.0)
            rr = rest[2] if len(rest) > 2 else kw.get("random_rotation", False)
            return self.forward_arrays(a0.centers, a0.coords, a0.type_index, a0.radii, grid,
                                       transforms=self.batch_transforms(a0, rt, rr), n_atoms=a0.n_atoms)
        if isinstance(a0, Example):
            rest = list(args[1:])
            if rest and isinstance(rest[0], Transform):
                return self._forward_example(a0, rest[0], rest[1] if len(rest) > 1 else kw["grid"])
            grid = rest[0] if rest else kw["grid"]
            rt = rest[1] if len(rest) > 1 else kw.get("random_translation", 0.0)
            rr = rest[2] if len(rest) > 2 else kw.get("random_rotation", False)
            return self._forward_example(a0, Transform(self._default_center(a0), rt, rr), grid)
        if isinstance(a0, (list, tuple)) and (len(a0) == 0 or isinstance(a0[0], Example)):
            rest = list(args[1:])
            grid = rest[0] if rest else kw["grid"]
            rt = rest[1] if len(rest) > 1 else kw.get("random_translation", 0.0)
            rr = rest[2] if len(rest) > 2 else kw.get("random_rotation", False)
            return self._forward_examples(list(a0), grid, rt, rr)
        if len(args) >= 2 and isinstance(args[1], CoordinateSet):
            center, cs, grid = args[0], args[1], args[2] if len(args) > 2 else kw["grid"]
            # vector types win when the set has both (include/libmolgrid/grid_maker.h:132-153)
            if cs.has_vector_types() and cs.size() > 0:
                return self.forward_arrays(center, cs.coords, cs.type_vector, cs.radii, grid)
            return self.forward_arrays(center, cs.coords, cs.type_index, cs.radii, grid)
        return self.forward_arrays(*args, **kw)

    @staticmethod
    def batch_transforms(batch, random_translation=0.0, random_rotation=False):
        """(B,10) device array of per-example random Transforms about the batch's grid centres, drawn
        in example order like the reference's loop (include/libmolgrid/grid_maker.h:194-201).  Keep
        it to hand the same transforms to ``backward``."""
        B = len(batch)
        dev = batch.centers.device
        # B x lmg_transform, drawn on the host into one of a few pinned buffers and copied without
        # blocking; a buffer is reused only after the copy that last read it has finished
        ring = _transform_ring.setdefault((dev, B), {"next": 0, "slots": []})
        if len(ring["slots"]) < 4:
            ring["slots"].append([torch.empty((B, 10), dtype=torch.float32).pin_memory(), None])
            slot = ring["slots"][-1]
        else:
            slot = ring["slots"][ring["next"]]
            ring["next"] = (ring["next"] + 1) % 4
            if slot[1] is not None:
                slot[1].synchronize()
        rows = slot[0]
        zero = (ctypes.c_float * 3)(0, 0, 0)
        check(_cabi.lib().lmg_transform_random_batch(ctypes.c_void_p(rows.data_ptr()), B, zero,
                                                     float(random_translation), int(bool(random_rotation))))
        tr = rows.to(dev, non_blocking=True)
        slot[1] = torch.cuda.Event()
        slot[1].record(torch.cuda.current_stream(dev))
        tr[:, 4:7] = batch.centers
        return tr

    @staticmethod
    def _default_center(ex):
        """Grid centre of forward(example, grid, ...): the centre of the LAST set, taken as soon as
        any set from the back is non-empty (src/grid_maker.cpp:126-137)."""
        for s in reversed(ex.coord_sets):
            if s.size():
                return ex.coord_sets[-1].center()
        return float3(0, 0, 0)

    def _forward_example(self, ex, transform, grid):
        """forward(Example, Transform, grid), src/grid_maker.cpp:109-116: sets merged, the transform
        applied (here inside the gridding kernel), the rotation centre used as grid centre."""
        c = ex.merge_coordinates()
        T = int(_grids.operand_tensor(grid).shape[0])
        if c.max_type != T:
            raise IndexError("Incorrect number of channels in output grid: %d vs %d" % (c.max_type, T))
        types = c.type_vector if (c.has_vector_types() and c.size() > 0) else c.type_index
        return self.forward_arrays(transform.get_rotation_center(), c.coords, types, c.radii, grid,
                                   transforms=transform)

    def _forward_examples(self, examples, grid, random_translation, random_rotation):
        """forward(vector<Example>, grid5, ...), include/libmolgrid/grid_maker.h:194-201, as ONE
        batched call: examples are merged, padded to the longest and gridded together, each with its
        own random Transform drawn in example order (the reference's sequence of draws)."""
        gt = _grids.operand_tensor(grid)
        if gt.shape[0] != len(examples):
            raise ValueError("output grid dimension doesn't match examples vector size")
        if not examples:
            return
        T = int(gt.shape[1])
        merged, trs = [], []
        for ex in examples:
            c = ex.merge_coordinates()
            if c.max_type != T:
                raise IndexError("Incorrect number of channels in output grid: %d vs %d" % (c.max_type, T))
            merged.append(c)
            trs.append(Transform(self._default_center(ex), random_translation, random_rotation))
        vec = any(c.has_vector_types() and c.size() > 0 for c in merged)
        B = len(merged)
        nmax = max(1, max(c.size() for c in merged))
        dev = _current_device()
        coords = torch.zeros((B, nmax, 3), dtype=torch.float32, device=dev)
        nr = T if (vec and self.s.radii_type_indexed) else nmax
        radii = torch.zeros((B, nr), dtype=torch.float32, device=dev)
        types = torch.zeros((B, nmax, T) if vec else (B, nmax), dtype=torch.float32, device=dev)
        ns = torch.zeros(B, dtype=torch.int32)
        for b, c in enumerate(merged):
            n = c.size()
            ns[b] = n
            if n == 0:
                continue
            coords[b, :n] = c.coords._current().t
            src_t = c.type_vector if vec else c.type_index
            types[b, :n] = src_t._current().t
            r = c.radii._current().t
            radii[b, :r.shape[0]] = r
        centers = torch.tensor([list(t.get_rotation_center()) for t in trs], dtype=torch.float32, device=dev)
        return self.forward_arrays(centers, coords, types, radii, grid, transforms=trs, n_atoms=ns)

    def forward_arrays(self, center, coords, types, radii, out, transforms=None, n_atoms=None):
        """out[T,D,D,D] (or out[B,T,D,D,D] for batched inputs) from atoms.

        ``center`` is a float3/tuple, or a (B,3) array for batched input.  ``transforms`` (a
        Transform, a list of them, or a (B,10) array) is applied to the coordinates inside the
        gridding kernels - the fused form of forward(Example, Transform, grid)
        (src/grid_maker.cpp:109-116).  ``n_atoms`` marks padded batches.
        """
        dev, A, keep, batched, vec, B, N, nr = self._atoms(center, coords, types, radii, transforms, n_atoms)
        o = _Arg(out, dev, 5 if batched else 4, "out", output=True)
        oshape = tuple(o.t.shape[1:] if batched else o.t.shape)
        if batched and o.t.shape[0] != B:
            raise ValueError("Mismatched batch sizes: %d vs %d" % (o.t.shape[0], B))
        d = int(self.s.dim)
        for i in (1, 2, 3):  # check_index_args / check_vector_args, src/grid_maker.cpp:46-48,74-76
            if oshape[i] != d:
                raise IndexError("Output grid dimension incorrect: %d vs %d" % (d, oshape[i]))
        T = int(oshape[0])
        if vec and A.ntypes != T:
            raise IndexError("number of types in type_vector does not match number of output "
                             "channels: %d vs %d" % (A.ntypes, T))
        A.ntypes = T
        self._check_radii(vec, N, T, nr, IndexError)
        ws = self._ws(dev, _cabi.OP_FORWARD, B, N, T, vec)
        check(_cabi.lib().lmg_forward(ctypes.byref(self.s), ctypes.byref(A), o.ptr,
                                      ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(dev)))
        self._last_ws = ws
        o.finish()

    def check_types(self):
        """Synchronise and raise IndexError/ValueError if the last call met a type index >= the
        number of channels - the check the reference makes while looping over atoms on the host
        (src/grid_maker.cpp:172, :458-460)."""
        ws = getattr(self, "_last_ws", None)
        if ws is not None:
            check(_cabi.lib().lmg_check_status(ctypes.c_void_p(ws.data_ptr()), _stream_ptr(ws.device)))

    # --- backward ----------------------------------------------------------------------------
    def backward(self, *args, **kw):
        """The reference's backward overload set (python/bindings.in.cpp:869-896):
        ``backward(center, coordinate_set, diff, atom_gradients[, type_gradients])`` or
        ``backward(center, coords, types, radii, diff, atom_gradients[, type_gradients])``."""
        from .coordinates import CoordinateSet
        from .coord_cache import DeviceBatch
        if args and isinstance(args[0], DeviceBatch):
            # backward(batch, diff, atom_gradients, transforms=...): the arrays of a DeviceBatch
            batch, diff, ag = args[:3]
            tr = args[3] if len(args) > 3 else kw.get("transforms")
            return self.backward_arrays(batch.centers, batch.coords, batch.type_index, batch.radii, diff, ag,
                                        transforms=tr, n_atoms=batch.n_atoms)
        if len(args) >= 2 and isinstance(args[1], CoordinateSet):
            center, cs, diff, ag = args[:4]
            tg = args[4] if len(args) > 4 else kw.get("type_gradients")
            if tg is not None:
                if not cs.has_vector_types():
                    raise ValueError("Vector types missing from coordinate set")
                return self.backward_arrays(center, cs.coords, cs.type_vector, cs.radii, diff, ag, tg)
            if not cs.has_indexed_types():
                raise ValueError("Index types missing from coordinate set")
            return self.backward_arrays(center, cs.coords, cs.type_index, cs.radii, diff, ag)
        return self.backward_arrays(*args, **kw)

    def backward_arrays(self, center, coords, types, radii, diff, atom_gradients, type_gradients=None,
                        transforms=None, n_atoms=None, want_type_gradients=True):
        """Atom (and, for vector types, type) gradients from grid gradients ``diff``.
        ``want_type_gradients=False`` (vector types only) skips the type gradients, which lets the
        kernels read just the channels in which an atom carries weight."""
        dev, A, keep, batched, vec, B, N, nr = self._atoms(center, coords, types, radii, transforms, n_atoms)
        df = _Arg(diff, dev, 5 if batched else 4, "diff")
        ag = _Arg(atom_gradients, dev, 3 if batched else 2, "atom_gradients", output=True)
        dshape = tuple(df.t.shape[1:] if batched else df.t.shape)
        T = int(dshape[0])
        d = int(self.s.dim)
        if ag.t.shape[-2] != N:
            raise ValueError("Gradient dimension doesn't equal number of coordinates")
        for i in (1, 2, 3):
            if dshape[i] != d:
                raise ValueError("diff does not have correct dimension %d: %d vs %d" % (i, dshape[i], d))
        tg = None
        if vec and not want_type_gradients:
            if A.ntypes != T:
                raise ValueError("Channels in diff doesn't equal number of types")
        elif vec:
            if type_gradients is None:
                raise TypeError("vector types need type_gradients")
            tg = _Arg(type_gradients, dev, 3 if batched else 2, "type_gradients", output=True)
            if A.ntypes != T:
                raise ValueError("Channels in diff doesn't equal number of types")
            if tg.t.shape[-2] != N:
                raise ValueError("Type gradient dimension doesn't equal number of coordinates")
            if tg.t.shape[-1] != T:
                raise ValueError("Type gradient dimension has wrong number of types")
        elif type_gradients is not None:
            raise TypeError("type_gradients given with index types")
        A.ntypes = T
        self._check_radii(vec, N, T, nr, ValueError)
        ws = self._ws(dev, _cabi.OP_BACKWARD, B, N, T, vec)
        check(_cabi.lib().lmg_backward(ctypes.byref(self.s), ctypes.byref(A), df.ptr, ag.ptr,
                                       tg.ptr if tg is not None else None,
                                       ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(dev)))
        self._last_ws = ws
        ag.finish()
        if tg is not None:
            tg.finish()

    def backward_relevance(self, *args, **kw):
        """``backward_relevance(center, coordinate_set, density, diff, relevance)`` or the array form
        of :meth:`backward_relevance_arrays` (include/libmolgrid/grid_maker.h:558-618)."""
        from .coordinates import CoordinateSet
        if len(args) >= 2 and isinstance(args[1], CoordinateSet):
            center, cs, density, diff, rel = args[:5]
            if not cs.has_indexed_types():
                raise ValueError("Index types missing from coordinate set in backward relevance")
            return self.backward_relevance_arrays(center, cs.coords, cs.type_index, cs.radii, density, diff, rel)
        return self.backward_relevance_arrays(*args, **kw)

    def backward_relevance_arrays(self, center, coords, types, radii, density, diff, relevance,
                                  transforms=None, n_atoms=None):
        """Per-atom relevance; C++-only in the reference (include/libmolgrid/grid_maker.h:558-618)."""
        dev, A, keep, batched, vec, B, N, nr = self._atoms(center, coords, types, radii, transforms, n_atoms)
        if vec:
            raise TypeError("backward_relevance takes index types")
        de = _Arg(density, dev, 5 if batched else 4, "density")
        df = _Arg(diff, dev, 5 if batched else 4, "diff")
        rel = _Arg(relevance, dev, 2 if batched else 1, "relevance", output=True)
        if rel.t.shape[-1] != N:
            raise ValueError("Relevance dimension doesn't equal number of coordinates")
        if nr != N:
            raise ValueError("Radii dimension doesn't equal number of coordinates")
        if de.t.shape != df.t.shape:
            raise ValueError("density and diff differ in shape")
        T = int(df.t.shape[-4])
        A.ntypes = T
        ws = self._ws(dev, _cabi.OP_BACKWARD_RELEVANCE, B, N, T, False)
        check(_cabi.lib().lmg_backward_relevance(ctypes.byref(self.s), ctypes.byref(A), de.ptr, df.ptr,
                                                 rel.ptr, ctypes.c_void_p(ws.data_ptr()), ws.numel(),
                                                 _stream_ptr(dev)))
        self._last_ws = ws
        rel.finish()

    def backward_gradients(self, *args, **kw):
        """``backward_gradients(center, coordinate_set, diff, atom_gradients, type_gradients, diffdiff,
        atom_diffdiff, type_diffdiff)`` or the array form (python/bindings.in.cpp:897-918)."""
        from .coordinates import CoordinateSet
        if len(args) >= 2 and isinstance(args[1], CoordinateSet):
            cs = args[1]
            if not cs.has_vector_types():
                raise ValueError("Vector types missing from coordinate set")
            return self.backward_gradients_arrays(args[0], cs.coords, cs.type_vector, cs.radii, *args[2:], **kw)
        return self.backward_gradients_arrays(*args, **kw)

    def backward_gradients_arrays(self, center, coords, types, radii, diff, atom_gradients, type_gradients,
                                  diffdiff, atom_diffdiff, type_diffdiff, transforms=None, n_atoms=None):
        """Second-order pass (vector types only), src/grid_maker.cpp:529-672."""
        dev, A, keep, batched, vec, B, N, nr = self._atoms(center, coords, types, radii, transforms, n_atoms)
        if not vec:
            raise TypeError("backward_gradients takes vector types")
        df = _Arg(diff, dev, 5 if batched else 4, "diff")
        ag = _Arg(atom_gradients, dev, 3 if batched else 2, "atom_gradients")
        tg = _Arg(type_gradients, dev, 3 if batched else 2, "type_gradients")
        dd = _Arg(diffdiff, dev, 5 if batched else 4, "diffdiff", output=True)
        add = _Arg(atom_diffdiff, dev, 3 if batched else 2, "atom_diffdiff", output=True)
        tdd = _Arg(type_diffdiff, dev, 3 if batched else 2, "type_diffdiff", output=True)
        dshape = tuple(df.t.shape[1:] if batched else df.t.shape)
        T = int(dshape[0])
        d = int(self.s.dim)
        for i in (1, 2, 3):
            if dshape[i] != d:
                raise IndexError("Output grid dimension incorrect: %d vs %d" % (d, dshape[i]))
        if A.ntypes != T:
            raise IndexError("number of types in type_vector does not match number of output channels")
        self._check_radii(vec, N, T, nr, IndexError)
        if dd.t.shape != df.t.shape:
            raise ValueError("diffdiff and diff differ in shape")
        for name, x, last in (("Atom gradient", ag, 3), ("Type gradient", tg, T),
                              ("Atom gradient gradients", add, 3), ("Type gradient gradients", tdd, T)):
            if x.t.shape[-2] != N:
                raise ValueError("%s dimension doesn't equal number of coordinates" % name)
            if x.t.shape[-1] != last:
                raise ValueError("%s dimension has wrong number of types" % name)
        ws = self._ws(dev, _cabi.OP_BACKWARD_GRADIENTS, B, N, T, True)
        check(_cabi.lib().lmg_backward_gradients(
            ctypes.byref(self.s), ctypes.byref(A), df.ptr, ag.ptr, tg.ptr, dd.ptr, add.ptr, tdd.ptr,
            ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(dev)))
        self._last_ws = ws
        for x in (dd, add, tdd):
            x.finish()


class GridInterpolater(object):
    """Trilinear resample of a grid under a Transform (include/libmolgrid/grid_interpolater.h)."""

    def __init__(self, in_resolution=0.5, in_dimension=23.5, out_resolution=0.5, out_dimension=23.5):
        self.s = _cabi.InterpolaterStruct()
        check(_cabi.lib().lmg_interpolater_init(ctypes.byref(self.s), in_resolution, in_dimension,
                                                out_resolution, out_dimension))

    def get_in_resolution(self): return self.s.in_resolution
    def get_out_resolution(self): return self.s.out_resolution
    def get_in_dimension(self): return self.s.in_dimension
    def get_out_dimension(self): return self.s.out_dimension

    # The reference's setters recompute in_dim from the OLD values before storing the new one and
    # never recompute out_dim (include/libmolgrid/grid_interpolater.h:74-94); kept as is.
    def set_in_resolution(self, r):
        self.s.in_dim = int(np.round(_F(self.s.in_dimension) / _F(self.s.in_resolution)) + 1)
        self.s.in_resolution = r

    def set_in_dimension(self, d):
        self.s.in_dim = int(np.round(_F(self.s.in_dimension) / _F(self.s.in_resolution)) + 1)
        self.s.in_dimension = d

    def set_out_resolution(self, r): self.s.out_resolution = r
    def set_out_dimension(self, d): self.s.out_dimension = d

    def forward(self, *args):
        """forward(in, transform, out) or forward(in_center, in, transform, out_center, out).

        ``in``/``out`` are (K,D,D,D) grids with one Transform, or batched (B,K,D,D,D) grids with a
        list of B Transforms (and (B,3) centres in the five-argument form).
        """
        self._run(args, backward=False)

    def backward(self, *args):
        """backward(grad_out, transform, grad_in) or backward(in_center, grad_out, transform, out_center,
        grad_in): the gradient with respect to the forward pass's input from the gradient with respect
        to its output, for the same transform(s) and centres.  Not in the reference, which leaves the
        backward pass open (include/libmolgrid/grid_interpolater.h:179)."""
        self._run(args, backward=True)

    def _run(self, args, backward):
        if len(args) == 3:
            inp, transform, out = args
            in_center = out_center = None
        elif len(args) == 5:
            in_center, inp, transform, out_center, out = args
        else:
            raise TypeError("forward takes 3 or 5 arguments")
        dev = _current_device()
        inp, out = _grids.operand_tensor(inp), _grids.operand_tensor(out)
        nd = inp.ndim if isinstance(inp, np.ndarray) else inp.dim()
        batched = nd == 5
        i = _Arg(inp, dev, nd, "in")
        o = _Arg(out, dev, nd, "out", output=True)
        B = int(i.t.shape[0]) if batched else 1
        trs = list(transform) if batched else [transform]
        if len(trs) != B:
            raise ValueError("need one transform per example")
        ish = tuple(i.t.shape[1:] if batched else i.t.shape)
        osh = tuple(o.t.shape[1:] if batched else o.t.shape)
        if backward:
            ish, osh = osh, ish   # the first grid is the output's gradient, the last the input's
        # GridInterpolater::checkGrids, src/grid_interpolater.cpp:55-76
        if i.t.data_ptr() == o.t.data_ptr():
            raise ValueError("Input and output grid can not be the same in GridInterpolator.")
        if ish[0] != osh[0] or (batched and o.t.shape[0] != B):
            raise ValueError("Different channel dimensions for input and output  grids.")
        if ish[1:] != (self.s.in_dim,) * 3:
            raise ValueError("Input grid wrong dimension. Should be %d along all axes but is %d,%d,%d"
                             % ((self.s.in_dim,) + ish[1:]))
        if osh[1:] != (self.s.out_dim,) * 3:
            raise ValueError("Output grid wrong dimension. Should be %d along all axes but is %d,%d,%d"
                             % ((self.s.out_dim,) + osh[1:]))
        T = (_cabi.TransformStruct * B)(*[t.struct() for t in trs])

        def centers(c):
            arr = (ctypes.c_float * (3 * B))()
            for b in range(B):
                if c is None:
                    v = trs[b].get_rotation_center()
                elif batched:
                    v = c[b]
                else:
                    v = c
                arr[3 * b:3 * b + 3] = [float(v[0]), float(v[1]), float(v[2])]
            return arr

        ic, oc = centers(in_center), centers(out_center)
        fn = _cabi.lib().lmg_interpolate_backward if backward else _cabi.lib().lmg_interpolate
        check(fn(ctypes.byref(self.s), B, int(ish[0]), i.ptr, T, ic, oc, o.ptr, _stream_ptr(dev)))
        o.finish()
