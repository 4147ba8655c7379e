"""Grid / MGrid / CoordinateSet / Example host classes (no GPU needed): the behaviours the
reference's own tests check (test/test_grid.py, test/test_numpy.py, test/test_coordinateset.py:69-87,
test/test_example.py:11-41), restated on arrays since molecule parsing is outside the path."""
import numpy as np
import pytest

import libmolgrid_b200 as molgrid


def test_grid_views_share_memory():
    g = molgrid.MGrid2f(10, 2)
    assert g.size() == 20
    g2 = molgrid.Grid2f(g.cpu())
    g2[5][1] = 3.0
    assert g[5, 1] == g2[5, 1] == 3.0
    g1 = g2[5]
    g1[1] = 4.0
    assert g[5, 1] == 4.0
    gclone = g.clone()
    gclone[5, 1] = 5.5
    assert g[5, 1] == 4.0
    assert gclone[5][1] == 5.5


def test_numpy_views_and_copies():
    mg3d = molgrid.MGrid3d(3, 3, 3)
    mg2f = molgrid.MGrid2f(2, 4)
    a2f = np.arange(27).astype(np.float32).reshape(3, -1)
    a3d = np.arange(27).astype(np.float64).reshape(3, 3, -1)
    g2f = molgrid.Grid2f(a2f)
    g3d = molgrid.Grid3d(a3d)
    g2f[0, 0] = 100
    g3d[0, 0, 0] = 101
    assert a2f[0, 0] == 100 and a3d[0, 0, 0] == 101
    mg2f.copyFrom(g2f)
    mg3d.copyFrom(g3d)
    assert mg2f[1, 3] == 7
    mg2f[1, 3] = 200
    assert g2f[1, 3] == 12 and a2f[1, 3] == 12
    mg2f.copyTo(g2f)
    assert g2f[0, 7] == 200 and a2f[0, 7] == 200
    # the same with arrays converted on the fly
    mg2f.copyFrom(np.arange(27).astype(np.float32).reshape(3, -1))
    assert mg2f[1, 3] == 7


def test_tonumpy_copies_and_fill_zero():
    mg = molgrid.MGrid1d(10)
    for i in range(10):
        mg[i] = i
    a1 = mg.tonumpy()
    mg[0] = 100
    a2 = molgrid.tonumpy(mg)
    assert a1.sum() == 45 and a2.sum() == 145 and a1.dtype == np.float64
    assert np.asarray(mg).sum() == 145
    g1 = molgrid.Grid1d(np.random.rand(20))
    mg3 = molgrid.MGrid3d(4, 5, 6)
    mg3.copyFrom(np.random.rand(4, 5, 6))
    mg3.fill_zero()
    g1.fill_zero()
    assert np.all(g1.tonumpy() == 0) and np.all(mg3.tonumpy() == 0)


def test_conversion_rules():
    a = np.zeros((4, 3), np.float32)
    with pytest.raises(TypeError):
        molgrid.Grid2d(a)          # wrong element type
    with pytest.raises(TypeError):
        molgrid.Grid3f(a)          # wrong rank
    with pytest.raises(TypeError):
        molgrid.Grid2fCUDA(a)      # numpy converts to CPU grids only
    with pytest.raises(ValueError):
        molgrid.Grid2f(a.T)        # not contiguous
    g = molgrid.Grid2f(a)
    assert g.shape == (4, 3) and len(g) == 4 and g.type() == "float32" and g.data() == a.ctypes.data
    with pytest.raises(IndexError):
        g[4]
    p = molgrid.Grid2f(molgrid.tofloatptr(a.ctypes.data), 4, 3)
    p[2, 1] = 9
    assert a[2, 1] == 9


def test_coordset_from_arrays_and_clone():
    coords = np.array([[1, 0, -1], [1, 3, -1], [1, 0, -1]], np.float32)
    types = np.array([3, 2, 1], np.float32)
    radii = np.array([1.5, 1.5, 1.0], np.float32)
    c = molgrid.CoordinateSet(coords, types, radii, 4)
    assert c.size() == 3 and c.num_types() == 4
    assert c.has_indexed_types() and not c.has_vector_types()
    assert tuple(c.center()) == pytest.approx((1.0, 1.0, -1.0))
    c2 = c.clone()
    c2.coords[1, 1] = 0
    assert c.coords[1, 1] == 3.0
    with pytest.raises(ValueError):
        molgrid.CoordinateSet(coords, types[:2], radii, 4)
    empty = molgrid.CoordinateSet()
    assert empty.has_indexed_types() and empty.has_vector_types() and empty.size() == 0


def test_make_vector_types_and_copyto():
    coords = np.random.rand(8, 3).astype(np.float32)
    types = np.array([0, 1, 2, 3, 10, 1, 0, 5], np.float32)
    c = molgrid.CoordinateSet(coords, types, np.ones(8, np.float32), 11)
    c.make_vector_types()
    tv = c.type_vector.tonumpy()
    assert tv.shape == (8, 11) and np.all(tv.sum(1) == 1) and tv[4, 10] == 1
    assert c.has_indexed_types() and c.has_vector_types()
    co, ty, ra = np.zeros((10, 3), np.float32), np.zeros((10, 15), np.float32), np.zeros(10, np.float32)
    assert c.copyTo(co, ty, ra) == 8
    assert ty[:, 11:].sum() == 0 and co[8:].sum() == 0 and ra[8:].sum() == 0 and ty.sum() == 8
    com, tym, ram = np.zeros((5, 3), np.float32), np.zeros((5, 8), np.float32), np.zeros(5, np.float32)
    assert c.copyTo(com, tym, ram) == 5
    assert np.array_equal(tym, tv[:5, :8])
    # dummy type and per-type radii
    c3 = molgrid.CoordinateSet(coords, np.array([0, 1, 2, 1, 0, 2, 2, 1], np.float32), np.ones(8, np.float32), 3)
    c3.make_vector_types(True, [1.0, 2.0, 3.0])
    assert c3.max_type == 4 and c3.type_vector.shape == (8, 4)
    assert np.array_equal(c3.radii.tonumpy(), [1, 2, 3, 0])
    with pytest.raises(ValueError):
        c3.make_vector_types(False, [1.0])


def test_merges():
    rng = np.random.default_rng(3)
    c = molgrid.CoordinateSet(rng.random((16, 3), np.float32), rng.integers(0, 7, 16).astype(np.float32),
                              np.ones(16, np.float32), 7)
    c2 = molgrid.CoordinateSet(rng.random((8, 3), np.float32), rng.integers(0, 11, 8).astype(np.float32),
                               np.ones(8, np.float32), 11)
    c3 = molgrid.CoordinateSet(c, c2)
    c4 = molgrid.CoordinateSet(c, c2, False)
    assert c3.max_type == 18 and c4.max_type == 11 and c3.size() == c4.size() == 24
    t = np.concatenate([c.type_index.tonumpy(), c2.type_index.tonumpy() + c.max_type])
    assert np.array_equal(t, c3.type_index.tonumpy())
    assert np.array_equal(np.concatenate([c.type_index.tonumpy(), c2.type_index.tonumpy()]), c4.type_index.tonumpy())

    c2.make_vector_types()  # must not disturb the index types
    ex = molgrid.Example()
    ex.coord_sets.append(c)
    ex.coord_sets.append(c2)
    assert ex.num_types() == 18 and ex.num_coordinates() == 24
    m = ex.merge_coordinates()
    assert m.coords.tonumpy().shape == (24, 3) and m.max_type == 18
    assert np.array_equal(t, m.type_index.tonumpy())
    m4 = ex.merge_coordinates(0, False)
    assert np.array_equal(c4.type_index.tonumpy(), m4.type_index.tonumpy()) and m4.max_type == 11
    m5 = ex.merge_coordinates(1, False)
    assert m5.coords.tonumpy().shape == (8, 3)
    # into caller arrays, with size checks
    co, ty, ra = np.zeros((24, 3), np.float32), np.zeros(24, np.float32), np.zeros(24, np.float32)
    ex.merge_coordinates(co, ty, ra)
    assert np.array_equal(ty, t) and np.array_equal(co[16:], c2.coords.tonumpy())
    with pytest.raises(ValueError):
        ex.merge_coordinates(np.zeros((23, 3), np.float32), ty, ra)

    # vector types: columns of the second set are offset by the first's number of types
    c.make_vector_types()
    mv = ex._merged(0, True, force_vector=True)
    tv = mv.type_vector.tonumpy()
    assert tv.shape == (24, 18) and np.all(tv.sum(1) == 1)
    assert np.array_equal(tv[16:, 7:], c2.type_vector.tonumpy()) and tv[16:, :7].sum() == 0


def test_examplevec_labels():
    ex, ex2 = molgrid.Example(), molgrid.Example()
    ex.labels += [0, 2.5]
    ex2.labels += [1, 3.5]
    ev = molgrid.ExampleVec([ex, ex2])
    lab = np.zeros((2, 2), np.float32)
    ev.extract_labels(lab)
    assert np.array_equal(lab, [[0, 2.5], [1, 3.5]])
    one = molgrid.MGrid1f(2)
    ev.extract_label(1, one)
    assert np.array_equal(one.tonumpy(), [2.5, 3.5])


def test_reference_module_name():
    import molgrid as mg
    from libmolgrid_b200 import molgrid_native
    # the compiled classes where the compiled module defines them ...
    assert issubclass(mg.GridMaker, molgrid_native.GridMaker) and mg.MGrid4f is molgrid_native.MGrid4f
    assert mg.CoordinateSet is molgrid_native.CoordinateSet and mg.Transform is molgrid_native.Transform
    # ... the Python layer for the rest
    assert mg.Coords2Grid is molgrid.Coords2Grid and issubclass(mg.ExampleProvider, molgrid.ExampleProvider)
    assert mg.FileMappedGninaTyper is molgrid.FileMappedGninaTyper
