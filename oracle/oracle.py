"""TEST INFRASTRUCTURE ONLY - CPU checkers for the gridding path.

Two interchangeable back ends with the same numpy interface:

* ``port``: ``oracle/lmg_oracle.c``, a plain-C restatement of the reference's CPU
  algorithm (``oracle/_build/liblmg_oracle.so``, built by ``make -C oracle port``).
* ``ref``: the reference's own CPU sources compiled unmodified
  (``oracle/_ref/liblmg_ref.so``, built by ``make -C oracle ref`` where the
  reference tree is present).

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``
may import this module; the product never does.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATHS = {
    "port": os.path.join(_HERE, "_build", "liblmg_oracle.so"),
    "ref": os.path.join(_HERE, "_ref", "liblmg_ref.so"),
}
_PREFIX = {"port": "lmgo_", "ref": "lmgref_"}

_f32p = ctypes.POINTER(ctypes.c_float)


def _fp(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(_f32p)


def _f32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


class OracleError(Exception):
    """code 1 = std::out_of_range, 2 = std::invalid_argument, 3 = other."""

    def __init__(self, code, msg):
        super().__init__("oracle error %d: %s" % (code, msg))
        self.code = code


def build_port():
    subprocess.check_call(["make", "-s", "-C", _HERE, "port"])


def available(kind):
    return os.path.exists(_PATHS[kind])


class CpuOracle(object):
    """GridMaker/Transform/GridInterpolater CPU results on numpy arrays."""

    def __init__(self, kind="port"):
        if kind == "port" and not available("port"):
            build_port()
        if not available(kind):
            raise RuntimeError("oracle back end %r is not built (%s)" % (kind, _PATHS[kind]))
        self.kind = kind
        self.lib = ctypes.CDLL(_PATHS[kind])
        self.p = _PREFIX[kind]
        self._fn("last_error").restype = ctypes.c_char_p

    def _fn(self, name):
        return getattr(self.lib, self.p + name)

    def _call(self, name, *args):
        rc = self._fn(name)(*args)
        if rc != 0:
            raise OracleError(rc, self._fn("last_error")().decode())

    @staticmethod
    def gm(resolution=0.5, dimension=23.5, binary=False, radii_type_indexed=False,
           radius_scale=1.0, gaussian_radius_multiple=1.0):
        return _f32([resolution, dimension, float(binary), float(radii_type_indexed),
                     radius_scale, gaussian_radius_multiple])

    @staticmethod
    def dim_of(gm):
        return int(np.round(np.float32(gm[1]) / np.float32(gm[0])) + 1)

    def consts(self, gm):
        """A, B, C, D, E, final_radius_multiple, dim, |gaussian_radius_multiple|."""
        out = np.zeros(8, np.float32)
        self._call("consts", _fp(gm), _fp(out))
        return out

    def forward_index(self, gm, center, coords, types, radii, ntypes):
        coords, types, radii = _f32(coords), _f32(types), _f32(radii)
        d = self.dim_of(gm)
        out = np.empty((ntypes, d, d, d), np.float32)
        self._call("forward_index", _fp(gm), _fp(_f32(center)), ctypes.c_uint(coords.shape[0]),
                   _fp(coords), _fp(types), _fp(radii), ctypes.c_uint(ntypes), _fp(out))
        return out

    def forward_vector(self, gm, center, coords, type_vector, radii):
        coords, type_vector, radii = _f32(coords), _f32(type_vector), _f32(radii)
        d = self.dim_of(gm)
        n, nt = type_vector.shape
        out = np.empty((nt, d, d, d), np.float32)
        self._call("forward_vector", _fp(gm), _fp(_f32(center)), ctypes.c_uint(n), ctypes.c_uint(nt),
                   _fp(coords), _fp(type_vector), _fp(radii), ctypes.c_uint(radii.shape[0]), _fp(out))
        return out

    def backward_index(self, gm, center, coords, types, radii, diff):
        coords, types, radii, diff = _f32(coords), _f32(types), _f32(radii), _f32(diff)
        n = coords.shape[0]
        ag = np.empty((n, 3), np.float32)
        self._call("backward_index", _fp(gm), _fp(_f32(center)), ctypes.c_uint(n), _fp(coords),
                   _fp(types), _fp(radii), ctypes.c_uint(diff.shape[0]), _fp(diff), _fp(ag))
        return ag

    def backward_vector(self, gm, center, coords, type_vector, radii, diff):
        coords, type_vector, radii, diff = _f32(coords), _f32(type_vector), _f32(radii), _f32(diff)
        n, nt = type_vector.shape
        ag = np.empty((n, 3), np.float32)
        tg = np.empty((n, nt), np.float32)
        self._call("backward_vector", _fp(gm), _fp(_f32(center)), ctypes.c_uint(n), ctypes.c_uint(nt),
                   _fp(coords), _fp(type_vector), _fp(radii), ctypes.c_uint(radii.shape[0]),
                   _fp(diff), _fp(ag), _fp(tg))
        return ag, tg

    def backward_gradients(self, gm, center, coords, type_vector, radii, diff, atom_gradients,
                           type_gradients):
        coords, type_vector, radii, diff = _f32(coords), _f32(type_vector), _f32(radii), _f32(diff)
        atom_gradients, type_gradients = _f32(atom_gradients), _f32(type_gradients)
        n, nt = type_vector.shape
        dd = np.empty_like(diff)
        add = np.empty((n, 3), np.float32)
        tdd = np.empty((n, nt), np.float32)
        self._call("backward_gradients", _fp(gm), _fp(_f32(center)), ctypes.c_uint(n),
                   ctypes.c_uint(nt), _fp(coords), _fp(type_vector), _fp(radii),
                   ctypes.c_uint(radii.shape[0]), _fp(diff), _fp(atom_gradients),
                   _fp(type_gradients), _fp(dd), _fp(add), _fp(tdd))
        return dd, add, tdd

    def backward_relevance(self, gm, center, coords, types, radii, density, diff):
        coords, types, radii = _f32(coords), _f32(types), _f32(radii)
        density, diff = _f32(density), _f32(diff)
        n = coords.shape[0]
        rel = np.empty((n,), np.float32)
        self._call("backward_relevance", _fp(gm), _fp(_f32(center)), ctypes.c_uint(n), _fp(coords),
                   _fp(types), _fp(radii), ctypes.c_uint(diff.shape[0]), _fp(density), _fp(diff),
                   _fp(rel))
        return rel

    @staticmethod
    def tr(q=(1, 0, 0, 0), center=(0, 0, 0), translate=(0, 0, 0)):
        return _f32(list(q) + list(center) + list(translate))

    def transform_forward(self, tr, coords, dotranslate=True):
        coords = _f32(coords)
        out = np.empty_like(coords)
        self._call("transform_forward", _fp(_f32(tr)), ctypes.c_uint(coords.shape[0]), _fp(coords),
                   _fp(out), ctypes.c_int(int(dotranslate)))
        return out

    def transform_backward(self, tr, coords, dotranslate=True):
        coords = _f32(coords)
        out = np.empty_like(coords)
        self._call("transform_backward", _fp(_f32(tr)), ctypes.c_uint(coords.shape[0]), _fp(coords),
                   _fp(out), ctypes.c_int(int(dotranslate)))
        return out

    def quaternion_ops(self, qa, qb, pt):
        """rows: a*b, a/b, a.inverse() (4 each) then a.rotate(pt) (3)."""
        out = np.zeros(15, np.float32)
        self._call("quaternion_ops", _fp(_f32(qa)), _fp(_f32(qb)), _fp(_f32(pt)), _fp(out))
        return out

    def interpolate(self, gi, in_center, grid, tr, out_center):
        gi, grid = _f32(gi), _f32(grid)
        dout = int(np.round(gi[3] / gi[2]) + 1)
        out = np.empty((grid.shape[0], dout, dout, dout), np.float32)
        self._call("interpolate", _fp(gi), _fp(_f32(in_center)), ctypes.c_uint(grid.shape[0]),
                   _fp(grid), _fp(_f32(tr)), _fp(_f32(out_center)), _fp(out))
        return out

    def random_transform(self, seed, center, random_translate, random_rotate, ndraws=1):
        """Only the ``ref`` back end has this (it replays the reference's seeded engine)."""
        out = np.zeros((ndraws, 10), np.float32)
        self._call("random_transform", ctypes.c_uint(seed), _fp(_f32(center)),
                   ctypes.c_float(random_translate), ctypes.c_int(int(random_rotate)),
                   ctypes.c_uint(ndraws), _fp(out))
        return out
