"""CoordinateSet and Example: the atom containers GridMaker and Transform accept.

Mirrors include/libmolgrid/coordinateset.h:32-133 with src/coordinateset.cpp:75-310 and
include/libmolgrid/example.h with src/example.cpp:40-228 for what the gridding path uses:
construction from arrays, index/vector typing, merging of sets with type offsets, centre, clone,
host/device affinity.  Construction from molecule files is outside this path.
"""
import ctypes

import numpy as np
import torch

from . import _cabi
from . import grids as G
from .grids import MGrid1f, MGrid2f


def _as_f32_tensor(x, ndim, name):
    """Contiguous float32 tensor view or copy of a Grid, MGrid, tensor, array or nested sequence."""
    t = G.operand_tensor(x)
    if not torch.is_tensor(t):
        a = np.asarray([tuple(v) for v in t] if name == "coords" and not isinstance(t, np.ndarray) else t,
                       dtype=np.float32)
        if name == "coords" and a.size == 0:
            a = a.reshape(0, 3)
        t = torch.from_numpy(np.ascontiguousarray(a))
    if t.dtype != torch.float32:
        t = t.to(torch.float32)
    if t.dim() != ndim:
        raise ValueError("%s must have %d dimensions" % (name, ndim))
    return t.contiguous()


def _mgrid_from(t):
    """New MGrid holding a copy of tensor ``t``, resident where ``t`` is."""
    m = (MGrid1f if t.dim() == 1 else MGrid2f)(*t.shape)
    if t.is_cuda:
        m.togpu(copy=False)
        m.gpu().t.copy_(t)
    else:
        m.cpu().t.copy_(t)
    return m


class CoordinateSet(object):
    """Coordinates, types (indices or vectors) and radii of a set of atoms."""

    def __init__(self, *args, **kw):
        self.coords = MGrid2f(0, 3)
        self.type_index = MGrid1f(0)
        self.type_vector = MGrid2f(0, 0)
        self.radii = MGrid1f(0)
        self.max_type = 0
        self.src = None
        if not args and not kw:
            return
        if isinstance(args[0], CoordinateSet):
            # merger of two sets (src/coordinateset.cpp:192-200)
            rec, lig = args[0], args[1]
            unique = args[2] if len(args) > 2 else kw.get("unique_index_types", True)
            self.mergeInto(rec, lig, unique)
            return
        c = _as_f32_tensor(args[0], 2, "coords")
        t = G.operand_tensor(args[1])
        tnd = t.dim() if torch.is_tensor(t) else np.asarray(t).ndim
        r = _as_f32_tensor(args[2], 1, "radii")
        if tnd == 1:
            if len(args) < 4 and "max_type" not in kw:
                raise TypeError("index-typed CoordinateSet needs the number of types")
            ti = _as_f32_tensor(args[1], 1, "types")
            if ti.shape[0] != c.shape[0]:
                raise ValueError("Types and coordinates are of different sizes")
            if r.shape[0] != c.shape[0]:
                raise ValueError("Radii and coordinates are of different sizes")
            self.type_index = _mgrid_from(ti)
            self.max_type = int(args[3] if len(args) > 3 else kw["max_type"])
        else:
            tv = _as_f32_tensor(args[1], 2, "types")
            if tv.shape[0] != c.shape[0]:
                raise ValueError("Types and coordinates are of different sizes")
            if r.shape[0] != c.shape[0] and r.shape[0] != tv.shape[1]:
                raise ValueError("Radius and coordinates/types are of different sizes: %d %d %d"
                                 % (c.shape[0], r.shape[0], tv.shape[1]))
            self.type_vector = _mgrid_from(tv)
            self.max_type = int(tv.shape[1])
        self.coords = _mgrid_from(c)
        self.radii = _mgrid_from(r)

    # --- queries -----------------------------------------------------------------------------------
    def has_indexed_types(self):
        return self.type_index.size() > 0 or self.coords.size() == 0

    def has_vector_types(self):
        return self.type_vector.size() > 0 or self.coords.size() == 0

    def size(self):
        return self.coords.dimension(0)

    def num_types(self):
        return self.max_type

    def set_num_types(self, maxt):
        self.max_type = int(maxt)

    def center(self):
        """Mean of the coordinates, summed in float in atom order (src/coordinateset.cpp:228-243)."""
        from .api import float3
        n = self.size()
        if n == 0:
            return float3(0, 0, 0)
        c = self.coords.cpu().t.numpy()
        acc = np.zeros(3, dtype=np.float32)
        for i in range(n):
            acc += c[i]
        acc /= np.float32(n)
        return float3(*[float(v) for v in acc])

    # --- affinity ----------------------------------------------------------------------------------
    def togpu(self, copy=True):
        for g in (self.coords, self.type_index, self.type_vector, self.radii):
            g.togpu(copy)

    def tocpu(self, copy=True):
        for g in (self.coords, self.type_index, self.type_vector, self.radii):
            g.tocpu(copy)

    def clone(self):
        c = CoordinateSet()
        c.coords, c.type_index = self.coords.clone(), self.type_index.clone()
        c.type_vector, c.radii = self.type_vector.clone(), self.radii.clone()
        c.max_type, c.src = self.max_type, self.src
        return c

    # --- conversions -------------------------------------------------------------------------------
    def make_vector_types(self, include_dummy_type=False, type_radii=()):
        """One-hot type vectors from the type indices, in place (src/coordinateset.cpp:203-226)."""
        type_radii = list(type_radii)
        n = self.type_index.size()
        if type_radii and len(type_radii) != self.max_type:
            raise ValueError("Type radii size %d does not equal max type %d" % (len(type_radii), self.max_type))
        if include_dummy_type:
            self.max_type += 1
        tv = MGrid2f(n, self.max_type)
        idx = self.type_index.cpu().t
        host = tv.cpu().t
        for i in range(n):
            t = int(idx[i])  # float to unsigned: truncation
            if 0 <= t < self.max_type:
                host[i, t] = 1.0
        self.type_vector = tv
        if type_radii:
            r = MGrid1f(self.max_type)
            r.cpu().t[:len(type_radii)] = torch.tensor(type_radii, dtype=torch.float32)
            self.radii = r

    def copyTo(self, c, t, r):
        """Copies into caller grids, truncating to their size; returns the number of atoms copied."""
        ct = G.operand_tensor(c)
        if (ct.shape[1] if hasattr(ct, "shape") else 3) != 3:
            raise ValueError("Coordinates have wrong secondary dimension in copyTo")
        ret = self.coords.copyTo(c)
        tt = G.operand_tensor(t)
        if len(tt.shape) == 1:
            self.type_index.copyTo(t)
        else:
            # a row at a time, so a narrower or wider destination truncates or pads per atom
            src = self.type_vector._current().t
            dst = tt if torch.is_tensor(tt) else torch.from_numpy(tt)
            n, w = min(src.shape[0], dst.shape[0]), min(src.shape[1] if src.dim() > 1 else 0, dst.shape[1])
            if n and w:
                dst[:n, :w].copy_(src[:n, :w])
        self.radii.copyTo(r)
        return ret // 3

    def sum_types(self, out, zerofirst=True):
        """Per-type sum of the type vectors (or counts of the rounded type indices) added into
        ``out`` (src/coordinateset.cpp:352-374).  With the output on the GPU the sums are formed by
        ``lmg_sum_types`` on the device; a host output is summed on the host, as the container's
        other host-side bookkeeping is."""
        o = G.operand_tensor(out)
        o = torch.from_numpy(o) if isinstance(o, np.ndarray) else o
        if o.shape[0] != self.num_types():
            raise ValueError("Type sum output dimension does not match number of types: %d vs %d"
                             % (o.shape[0], self.num_types()))
        vec = self.type_vector.size() > 0
        if o.is_cuda:
            if not o.is_contiguous() or o.dtype != torch.float32:
                raise ValueError("type sums: a contiguous float32 tensor is needed")
            src = (self.type_vector if vec else self.type_index)._current().t.to(o.device).contiguous()
            status = torch.empty(1, dtype=torch.int32, device=o.device)
            vp = ctypes.c_void_p
            with torch.cuda.device(o.device):
                _cabi.check(_cabi.lib().lmg_sum_types(
                    None if vec else vp(src.data_ptr()), vp(src.data_ptr()) if vec else None,
                    int(self.size()), int(o.shape[0]), vp(o.data_ptr()), int(bool(zerofirst)),
                    vp(status.data_ptr()), vp(torch.cuda.current_stream(o.device).cuda_stream)))
            if not vec and int(status.item()) != 0:
                raise IndexError("Somehow an index type is too large (internal error).")
            return
        if zerofirst:
            o.zero_()
        if self.size() == 0:
            return
        if vec:
            tv = self.type_vector._current().t.cpu().numpy()
            acc = o.numpy()
            for row in tv:           # atom by atom, as the reference's loop
                acc += row
        else:
            ti = np.round(self.type_index._current().t.cpu().numpy()).astype(np.int64)
            if (ti >= o.shape[0]).any():
                raise IndexError("Somehow an index type is too large (internal error).")
            cnt = np.bincount(ti[ti >= 0], minlength=o.shape[0]).astype(np.float32)
            o += torch.from_numpy(cnt)

    def mergeInto(self, rec, lig, unique_index_types=True):
        """This set becomes ``rec`` followed by ``lig``; with ``unique_index_types`` the second set's
        type indices are offset by the first's number of types (src/coordinateset.cpp:263-310)."""
        if rec.type_vector.dimension(1) != lig.type_vector.dimension(1):
            raise ValueError("Type vectors are incompatible sizes")
        if (rec.has_vector_types() != lig.has_vector_types()) and \
                (rec.has_indexed_types() != lig.has_indexed_types()):
            raise ValueError("Incompatible types when combining coodinate sets")
        if rec.has_indexed_types():
            self.max_type = rec.max_type + lig.max_type if unique_index_types else max(rec.max_type, lig.max_type)
        else:
            if rec.max_type != lig.max_type:
                raise ValueError("Type vectors are incompatible sizes, weirdly")
            self.max_type = rec.max_type
        ongpu = rec.coords.ongpu() or lig.coords.ongpu()
        dev = torch.device("cuda", torch.cuda.current_device()) if ongpu else torch.device("cpu")

        def cat(a, b):
            return torch.cat([a._current().t.to(dev), b._current().t.to(dev)], 0)

        ti = cat(rec.type_index, lig.type_index)
        if unique_index_types and lig.type_index.size() > 0:
            ti[rec.type_index.dimension(0):] += float(rec.max_type)
        self.coords = _mgrid_from(cat(rec.coords, lig.coords))
        self.type_index = _mgrid_from(ti)
        self.type_vector = _mgrid_from(cat(rec.type_vector, lig.type_vector))
        self.radii = _mgrid_from(cat(rec.radii, lig.radii))

    def __eq__(self, o):
        return self is o

    def __hash__(self):
        return id(self)


class Example(object):
    """Coordinate sets plus labels (include/libmolgrid/example.h); ``coord_sets`` is the list the
    reference exposes under that name (python/bindings.in.cpp:739)."""

    def __init__(self):
        self.coord_sets = []
        self.labels = []
        self.group = -1
        self.seqcont = False

    @property
    def sets(self):
        return self.coord_sets

    def num_coordinates(self):
        return sum(s.size() for s in self.coord_sets)

    def num_types(self, unique_index_type=True):
        """src/example.cpp:23-37: the sum of the sets' type counts, or their maximum."""
        if unique_index_type:
            return sum(s.num_types() for s in self.coord_sets)
        return max([s.num_types() for s in self.coord_sets] or [0])

    def has_vector_types(self, start=0):
        for s in self.coord_sets[start:]:
            if s.size() > 0 and not s.has_vector_types():
                return False
        return True

    def has_index_types(self, start=0):
        for s in self.coord_sets[start:]:
            if s.size() > 0 and not s.has_indexed_types():
                return False
        return True

    def togpu(self):
        for s in self.coord_sets:
            s.togpu()

    def tocpu(self):
        for s in self.coord_sets:
            s.tocpu()

    def merge_coordinates(self, *args, **kw):
        """merge_coordinates(start=0, unique_index_types=True) -> CoordinateSet, or
        merge_coordinates(coord, types, radius, start=0, unique_index_types=True) into caller grids
        (src/example.cpp:40-228)."""
        if args and not isinstance(args[0], (int, bool)):
            coord, types, radius = args[:3]
            start = args[3] if len(args) > 3 else kw.get("start", 0)
            unique = args[4] if len(args) > 4 else kw.get("unique_index_types", True)
            m = self._merged(start, unique, force_vector=len(G.operand_tensor(types).shape) == 2)
            if m.size() == 0 and len(G.operand_tensor(types).shape) == 2:
                return
            ct, tt, rt = (G.operand_tensor(x) for x in (coord, types, radius))
            if ct.shape[0] != m.size():
                raise ValueError("Coordinates do not have correct dimension: %d != %d" % (ct.shape[0], m.size()))
            if ct.shape[1] != 3:
                raise ValueError("Coordinates do not have correct second dimension (3): %d" % ct.shape[1])
            src_t = m.type_vector if len(tt.shape) == 2 else m.type_index
            if tuple(tt.shape) != tuple(src_t.shape):
                raise ValueError("Types do not have correct dimension: %s != %s" % (tuple(tt.shape), src_t.shape))
            if rt.shape[0] != m.radii.size():
                raise ValueError("Radii do not have correct dimension: %d != %d" % (rt.shape[0], m.radii.size()))
            m.coords.copyTo(coord)
            src_t.copyTo(types)
            m.radii.copyTo(radius)
            return
        start = args[0] if args else kw.get("start", 0)
        unique = args[1] if len(args) > 1 else kw.get("unique_index_types", True)
        has_vec, has_ind = self.has_vector_types(start), self.has_index_types(start)
        if not has_ind and not has_vec:
            raise ValueError("Inconsistent typing schemes in merge_coordinates")
        if len(self.coord_sets) <= start:
            return CoordinateSet()
        if len(self.coord_sets) == start + 1:
            return self.coord_sets[start].clone()
        # vector types win when every non-empty set has them (src/example.cpp:211-227)
        return self._merged(start, unique, force_vector=has_vec)

    def _merged(self, start, unique, force_vector):
        sets = self.coord_sets[start:]
        out = CoordinateSet()
        if not sets:
            return out
        ongpu = any(s.coords.ongpu() for s in sets if s.size())
        dev = torch.device("cuda", torch.cuda.current_device()) if ongpu else torch.device("cpu")

        def cur(g):
            return g._current().t.to(dev)

        if not force_vector:
            cs, ts, rs = [], [], []
            toffset = 0
            for s in sets:
                if s.size() == 0:
                    continue  # empties do not advance the type offset
                if not s.has_indexed_types():
                    raise RuntimeError("Coordinate sets do not have compatible index types for merge.")
                cs.append(cur(s.coords))
                ts.append(cur(s.type_index) + float(toffset))
                rs.append(cur(s.radii))
                if unique:
                    toffset += s.max_type
            if cs:
                out.coords = _mgrid_from(torch.cat(cs, 0))
                out.type_index = _mgrid_from(torch.cat(ts, 0))
                out.radii = _mgrid_from(torch.cat(rs, 0))
            out.max_type = self.num_types(unique)  # over all sets, whatever `start` is
            return out
        maxt = 0
        for i, s in enumerate(sets):
            maxt = maxt + s.max_type if unique else max(maxt, s.max_type)
            if s.size() == 0:
                continue
            if not s.has_vector_types():
                raise RuntimeError("Coordinate sets do not have compatible vector types for merge.")
            if s.max_type != s.type_vector.dimension(1):
                raise RuntimeError("Coordinate set %d does not have consistent max_type/vector type sizes"
                                   % (i + start))
        n = sum(s.size() for s in sets)
        tv = torch.zeros((n, maxt), dtype=torch.float32, device=dev)
        cs, rs = [], []
        row = offset = 0
        for s in sets:
            k = s.size()
            if k:
                w = s.type_vector.dimension(1)
                if offset + w > maxt:
                    raise RuntimeError("Incompatible vector sizes in merge_coordinates")
                tv[row:row + k, offset:offset + w] = cur(s.type_vector)
                cs.append(cur(s.coords))
            if s.radii.size():
                rs.append(cur(s.radii))
            row += k
            if unique:
                offset += s.max_type
        if cs:
            out.coords = _mgrid_from(torch.cat(cs, 0))
            out.type_vector = _mgrid_from(tv)
            out.radii = _mgrid_from(torch.cat(rs, 0)) if rs else MGrid1f(0)
        out.max_type = maxt
        return out

    def sum_types(self, out, unique_types=True):
        """Type sums of the sets side by side (``unique_types``: every set clears and fills its own
        range) or added into one shared range, which is not cleared first (src/example.cpp:355-374)."""
        o = G.operand_tensor(out)
        o = torch.from_numpy(o) if isinstance(o, np.ndarray) else o
        nt_all = self.num_types(unique_types)
        if o.shape[0] != nt_all:
            raise ValueError("Size of sum output doesn't match number of types in example: %d vs %d"
                             % (o.shape[0], nt_all))
        offset = 0
        for s in self.coord_sets:
            if unique_types:
                nt = s.num_types()
                if nt == 0:
                    continue
                s.sum_types(o[offset:offset + nt], zerofirst=True)
                offset += nt
            else:
                s.sum_types(o, zerofirst=False)


class ExampleVec(list):
    """A batch of Examples (python/bindings.in.cpp:436-450)."""

    def extract_labels(self, out):
        """out[i][j] = label j of example i (src/example.cpp:252-281)."""
        o = G.operand_tensor(out)
        if len(self) == 0:
            return
        nl = len(self[0].labels)
        if tuple(o.shape) != (len(self), nl):
            raise ValueError("Incorrect output grid shape for labels")
        vals = torch.tensor([[float(v) for v in ex.labels] for ex in self], dtype=torch.float32).reshape(len(self), nl)
        (o if torch.is_tensor(o) else torch.from_numpy(o)).copy_(vals)

    def extract_label(self, labelpos, out):
        """out[i] = label ``labelpos`` of example i (src/example.cpp:283-296)."""
        o = G.operand_tensor(out)
        if o.shape[0] != len(self):
            raise ValueError("Incorrect output grid shape for label")
        vals = torch.tensor([float(ex.labels[labelpos]) for ex in self], dtype=torch.float32)
        (o if torch.is_tensor(o) else torch.from_numpy(o)).copy_(vals)

    def sum_types(self, out, unique_types=True):
        o = G.operand_tensor(out)
        for i, ex in enumerate(self):
            ex.sum_types(o[i], unique_types)
