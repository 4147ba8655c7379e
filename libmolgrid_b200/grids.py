"""Grid and MGrid: the array views and owning arrays of the reference's Python module.

``Grid{1..8}{f,d}[CUDA]`` are non-owning views (include/libmolgrid/grid.h:43-335); ``MGrid{1..8}{f,d}``
own a host buffer and a lazily created device mirror with one "data is on the GPU" flag shared by
every view of the buffer (include/libmolgrid/managed_grid.h:23-616).  Members follow
python/bindings_grids.cpp:218-279 and python/__init__.py:12-25 (``tonumpy``/``__array__``).

Storage is a torch tensor in both cases; nothing here computes - the classes exist so that code
written against the reference (``molgrid.MGrid4f(*dims)``, ``grid.cpu()``, ``coords.togpu()`` ...)
runs unchanged in front of the CUDA path.
"""
import ctypes

import numpy as np
import torch

_gpu_enabled = None  # decided at first use: on when a CUDA device is present


def set_gpu_enabled(on):
    """MGrids handed to an operator convert to their GPU view when enabled, else to their CPU view
    (python/bindings_grids.cpp:146-161).  The arithmetic runs on the GPU either way."""
    global _gpu_enabled
    _gpu_enabled = bool(on)


def get_gpu_enabled():
    global _gpu_enabled
    if _gpu_enabled is None:
        _gpu_enabled = torch.cuda.is_available()
    return _gpu_enabled


def set_gpu_device(dev):
    torch.cuda.set_device(int(dev))


def get_gpu_device():
    return torch.cuda.current_device()


class _Pointer(object):
    """What tofloatptr/todoubleptr return: an address with an element type
    (python/bindings.in.cpp:402-405)."""

    def __init__(self, addr, dtype):
        self.addr = int(addr)
        self.dtype = dtype


def tofloatptr(addr):
    return _Pointer(addr, torch.float32)


def todoubleptr(addr):
    return _Pointer(addr, torch.float64)


_NP = {torch.float32: np.float32, torch.float64: np.float64}
_CT = {torch.float32: ctypes.c_float, torch.float64: ctypes.c_double}


class _CudaMem(object):
    """Device memory at a caller-owned address, presented through __cuda_array_interface__."""

    def __init__(self, addr, shape, dtype):
        self.__cuda_array_interface__ = {
            "shape": tuple(shape), "typestr": "<f4" if dtype == torch.float32 else "<f8",
            "data": (addr, False), "version": 2, "strides": None}


def _from_pointer(p, shape, cuda):
    if p.addr == 0:
        return torch.empty(tuple(shape), dtype=p.dtype, device="cuda" if cuda else "cpu")
    if cuda:
        return torch.as_tensor(_CudaMem(p.addr, shape, p.dtype), device="cuda")
    n = int(np.prod(shape))
    buf = (_CT[p.dtype] * n).from_address(p.addr)
    return torch.from_numpy(np.ctypeslib.as_array(buf).reshape(shape))


class GridBase(object):
    """Non-owning N-dimensional view over contiguous memory; subclasses fix N, dtype and device."""
    N = 0
    dtype = torch.float32
    cuda = False

    def __init__(self, *args):
        if len(args) == 1:
            self.t = self._view_of(args[0])
        elif args and isinstance(args[0], _Pointer):
            # Grid(pointer, d0, d1, ...)
            if args[0].dtype != self.dtype or len(args) != self.N + 1:
                raise TypeError("%s(pointer, %d sizes) expected" % (type(self).__name__, self.N))
            self.t = _from_pointer(args[0], [int(d) for d in args[1:]], self.cuda)
        else:
            raise TypeError("%s takes an array-like object or a pointer and %d sizes"
                            % (type(self).__name__, self.N))

    @classmethod
    def _view_of(cls, obj):
        """The tensor behind ``obj`` if it can be seen as this grid type, else an exception with the
        reference's conversion rules (python/bindings_grids.cpp:91-194)."""
        if isinstance(obj, ManagedGridBase):
            if obj.N != cls.N or obj.dtype != cls.dtype:
                raise TypeError("MGrid of other rank or type")
            return (obj.gpu() if cls.cuda else obj.cpu()).t
        if isinstance(obj, GridBase):
            t = obj.t
        elif isinstance(obj, np.ndarray):
            if cls.cuda:
                raise TypeError("numpy arrays convert to CPU grids only")
            if not obj.flags["C_CONTIGUOUS"]:
                raise ValueError("numpy array is not C-contiguous")
            t = torch.from_numpy(obj)
        elif torch.is_tensor(obj):
            t = obj
        else:
            raise TypeError("cannot view %s as a grid" % type(obj).__name__)
        if t.dim() != cls.N or t.dtype != cls.dtype or t.is_cuda != cls.cuda:
            raise TypeError("expected a %d-dimensional %s %s array" %
                            (cls.N, "CUDA" if cls.cuda else "CPU", str(cls.dtype).replace("torch.", "")))
        if t.is_cuda and t.device.index != torch.cuda.current_device():
            raise ValueError("Tensor on different device than current: %d vs %d"
                             % (t.device.index, torch.cuda.current_device()))
        if not t.is_contiguous():
            raise ValueError("Attempt to use non-contiguous tensor as grid")
        return t

    @classmethod
    def _wrap(cls, t):
        g = cls.__new__(cls)
        g.t = t
        return g

    # --- members ---------------------------------------------------------------------------------
    def size(self):
        return int(self.t.numel())

    def dimension(self, i):
        return int(self.t.shape[i])

    def data(self):
        return int(self.t.data_ptr())

    @property
    def shape(self):
        return tuple(int(d) for d in self.t.shape)

    def type(self):
        return "float32" if self.dtype == torch.float32 else "float64"

    def __len__(self):
        return int(self.t.shape[0])

    def __getitem__(self, idx):
        if isinstance(idx, tuple):
            if len(idx) != self.N:
                raise IndexError("need %d indices" % self.N)
            return float(self.t[idx])
        if idx < 0 or idx >= self.t.shape[0]:
            raise IndexError("grid index out of range")
        if self.N == 1:
            return float(self.t[idx])
        return _grid_class(self.N - 1, self.dtype, self.cuda)._wrap(self.t[idx])

    def __setitem__(self, idx, val):
        if isinstance(idx, tuple):
            if len(idx) != self.N:
                raise IndexError("need %d indices" % self.N)
        elif self.N != 1:
            raise TypeError("assignment needs one index per dimension")
        self.t[idx] = val

    def fill_zero(self):
        self.t.zero_()

    def copyTo(self, dest):
        """Copies min(size, dest.size) elements in storage order; returns how many."""
        d = _flat_of(dest)
        s = self.t.reshape(-1)
        n = min(s.numel(), d.numel())
        d[:n].copy_(s[:n])
        return int(n)

    def copyFrom(self, src):
        s = _flat_of(src)
        d = self.t.reshape(-1)
        n = min(s.numel(), d.numel())
        d[:n].copy_(s[:n])
        return int(n)

    def copyInto(self, start, src):
        """Copies ``src`` into this grid starting at row ``start`` (grid.h copyInto)."""
        s = _flat_of(src)
        d = self.t.reshape(-1)
        off = int(start) * (self.t.numel() // self.t.shape[0] if self.t.shape[0] else 0)
        n = min(s.numel(), d.numel() - off)
        if n > 0:
            d[off:off + n].copy_(s[:n])
        return int(max(n, 0))

    def tonumpy(self):
        return self.t.detach().cpu().numpy().copy()

    def __array__(self, dtype=None, copy=None):
        a = self.tonumpy()
        return a.astype(dtype) if dtype is not None else a

    def __repr__(self):
        return "%s%s" % (type(self).__name__, self.shape)


def _flat_of(obj):
    """Flat tensor sharing memory with a Grid, MGrid (its current side), numpy array or tensor."""
    if isinstance(obj, ManagedGridBase):
        return (obj.gpu() if obj.ongpu() else obj.cpu()).t.reshape(-1)
    if isinstance(obj, GridBase):
        return obj.t.reshape(-1)
    if isinstance(obj, np.ndarray):
        if not obj.flags["C_CONTIGUOUS"]:
            raise ValueError("numpy array is not C-contiguous")
        return torch.from_numpy(obj).reshape(-1)
    if torch.is_tensor(obj):
        if not obj.is_contiguous():
            raise ValueError("Attempt to use non-contiguous tensor as grid")
        return obj.reshape(-1)
    raise TypeError("cannot view %s as a grid" % type(obj).__name__)


class _Buffer(object):
    """Host storage, optional device mirror and the flag saying which one is current."""

    def __init__(self, numel, dtype):
        self.host = torch.zeros(int(numel), dtype=dtype)  # grids are always zero initialised
        self.dev = None
        self.sent_to_gpu = False

    def togpu(self, copy=True):
        if self.dev is None:
            self.dev = torch.empty(self.host.numel(), dtype=self.host.dtype, device="cuda")
            if not copy:
                self.dev.zero_()
        if not self.sent_to_gpu:
            if copy:
                self.dev.copy_(self.host)
            self.sent_to_gpu = True

    def tocpu(self, copy=True):
        if self.sent_to_gpu:
            if copy and self.dev is not None:
                self.host.copy_(self.dev)
            self.sent_to_gpu = False


class ManagedGridBase(object):
    """Owning grid; ``cpu()``/``gpu()`` return views and move the data when the other side is current."""
    N = 0
    dtype = torch.float32

    def __init__(self, *dims):
        if len(dims) == 1 and isinstance(dims[0], ManagedGridBase):
            o = dims[0]  # copy constructor: another view of the same buffer
            if o.N != self.N or o.dtype != self.dtype:
                raise TypeError("MGrid of other rank or type")
            self.buf, self.off, self.dims = o.buf, o.off, o.dims
            return
        if len(dims) != self.N:
            raise TypeError("%s takes %d sizes" % (type(self).__name__, self.N))
        self.dims = tuple(int(d) for d in dims)
        self.off = 0
        self.buf = _Buffer(int(np.prod(self.dims)) if self.dims else 0, self.dtype)

    @classmethod
    def _view(cls, buf, off, dims):
        g = cls.__new__(cls)
        g.buf, g.off, g.dims = buf, off, tuple(dims)
        return g

    def _numel(self):
        return int(np.prod(self.dims)) if self.dims else 0

    def cpu(self):
        self.buf.tocpu()
        t = self.buf.host[self.off:self.off + self._numel()].view(self.dims)
        return _grid_class(self.N, self.dtype, False)._wrap(t)

    def gpu(self):
        self.buf.togpu()
        t = self.buf.dev[self.off:self.off + self._numel()].view(self.dims)
        return _grid_class(self.N, self.dtype, True)._wrap(t)

    def togpu(self, copy=True):
        self.buf.togpu(copy)

    def tocpu(self, copy=True):
        self.buf.tocpu(copy)

    def ongpu(self):
        return self.buf.sent_to_gpu

    def oncpu(self):
        return not self.buf.sent_to_gpu

    def _current(self):
        return self.gpu() if self.ongpu() else self.cpu()

    def clone(self):
        c = type(self)(*self.dims)
        if self.ongpu():
            c.togpu(copy=False)
        c._current().t.copy_(self._current().t)
        return c

    def resized(self, *dims):
        """A grid of the new size holding as much of this one's data as fits (managed_grid.h resized)."""
        if tuple(int(d) for d in dims) == self.dims:
            return self
        c = type(self)(*dims)
        if self.ongpu():
            c.togpu(copy=False)
        self._current().copyTo(c._current())
        return c

    # --- grid members, forwarded to the current side ----------------------------------------------
    def size(self):
        return self._numel()

    def dimension(self, i):
        return self.dims[i]

    @property
    def shape(self):
        return self.dims

    def data(self):
        return self._current().data()

    def type(self):
        return "float32" if self.dtype == torch.float32 else "float64"

    def __len__(self):
        return self.dims[0]

    def __getitem__(self, idx):
        if isinstance(idx, tuple) or self.N == 1:
            return self.cpu()[idx]  # element access reads the host side, moving data back if needed
        if idx < 0 or idx >= self.dims[0]:
            raise IndexError("grid index out of range")
        sub = self.dims[1:]
        return _mgrid_class(self.N - 1, self.dtype)._view(self.buf, self.off + idx * int(np.prod(sub)), sub)

    def __setitem__(self, idx, val):
        self.cpu()[idx] = val

    def fill_zero(self):
        self._current().fill_zero()

    def copyTo(self, dest):
        return self._current().copyTo(dest)

    def copyFrom(self, src):
        return self._current().copyFrom(src)

    def copyInto(self, start, src):
        return self._current().copyInto(start, src)

    def tonumpy(self):
        return self._current().tonumpy()

    def __array__(self, dtype=None, copy=None):
        a = self.tonumpy()
        return a.astype(dtype) if dtype is not None else a

    def __repr__(self):
        return "%s%s" % (type(self).__name__, self.dims)


_grid_classes = {}
_mgrid_classes = {}


def _grid_class(n, dtype, cuda):
    return _grid_classes[(n, dtype, cuda)]


def _mgrid_class(n, dtype):
    return _mgrid_classes[(n, dtype)]


def _define():
    names = {}
    for n in range(1, 9):
        for dtype, tag in ((torch.float32, "f"), (torch.float64, "d")):
            for cuda in (False, True):
                name = "Grid%d%s%s" % (n, tag, "CUDA" if cuda else "")
                cls = type(name, (GridBase,), {"N": n, "dtype": dtype, "cuda": cuda})
                _grid_classes[(n, dtype, cuda)] = cls
                names[name] = cls
            name = "MGrid%d%s" % (n, tag)
            cls = type(name, (ManagedGridBase,), {"N": n, "dtype": dtype})
            _mgrid_classes[(n, dtype)] = cls
            names[name] = cls
    return names


_names = _define()
globals().update(_names)
__all__ = sorted(_names) + ["set_gpu_enabled", "get_gpu_enabled", "set_gpu_device", "get_gpu_device",
                            "tofloatptr", "todoubleptr", "tonumpy"]


def tonumpy(g):
    """Numpy copy of a grid (python/__init__.py:12-17)."""
    return g.tonumpy()


def operand_tensor(obj):
    """The tensor an operator should read or write for ``obj``: Grids give their memory, MGrids their
    GPU side when GPU use is enabled (and their host side otherwise); anything else is returned
    unchanged."""
    if isinstance(obj, ManagedGridBase):
        return (obj.gpu() if get_gpu_enabled() else obj.cpu()).t
    if isinstance(obj, GridBase):
        return obj.t
    return obj
