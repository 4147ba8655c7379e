"""The object types of the compiled module (Grid / MGrid families, CoordinateSet, Example,
ExampleVec) and the GridMaker / Transform overloads that take them: host-side behaviour here, and on
the GPU the same results as the ctypes layer and the CPU checker."""
import numpy as np
import pytest

from tests import cases


@pytest.fixture(scope="module")
def n():
    from libmolgrid_b200 import build
    build.build_library()
    build.build_native_module()
    from libmolgrid_b200 import molgrid_native
    return molgrid_native


def test_every_grid_class_is_bound(n):
    for rank in range(1, 9):
        for suffix in ("f", "d", "fCUDA", "dCUDA"):
            assert hasattr(n, "Grid%d%s" % (rank, suffix))
        for suffix in ("f", "d"):
            assert hasattr(n, "MGrid%d%s" % (rank, suffix))
    for name in ("CoordinateSet", "Example", "ExampleVec", "CoordinateSetVec", "FloatVec"):
        assert hasattr(n, name)


def test_grid_views_of_numpy_arrays(n):
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    g = n.Grid3f(a)
    assert g.shape == (2, 3, 4) and g.size() == 24 and len(g) == 2 and g.dimension(2) == 4
    assert g[1, 2, 3] == 23.0 and g[1][2][3] == 23.0 and g[1].shape == (3, 4) and g.type() == "float32"
    g[0, 0, 0] = 5            # a view: the array changes
    assert a[0, 0, 0] == 5
    np.testing.assert_array_equal(np.array(g), a)
    np.testing.assert_array_equal(g.tonumpy(), a)
    out = np.zeros_like(a)
    assert g.copyTo(out) == 24 and (out == a).all()
    g.fill_zero()
    assert not a.any()
    assert n.Grid2d(np.zeros((2, 2))).type() == "float64"
    with pytest.raises(TypeError):
        n.Grid3f(a.astype(np.float64))       # wrong element type
    with pytest.raises(TypeError):
        n.Grid2f(a)                          # wrong rank
    with pytest.raises(ValueError):
        n.Grid2f(np.zeros((4, 4), np.float32).T[:, :2])   # not contiguous
    with pytest.raises(IndexError):
        g[2, 0, 0]
    one = n.Grid1f(np.array([1, 2, 3], np.float32))
    one[1] = 9
    assert one[1] == 9 and one[(2,)] == 3


def test_managed_grids_on_the_host(n):
    m = n.MGrid2f(3, 4)
    assert m.shape == (3, 4) and m.size() == 12 and m.oncpu() and not m.ongpu()
    assert not m.tonumpy().any()              # zero-initialised
    m[1, 2] = 7
    assert m[1, 2] == 7 and m[1][2] == 7 and m[1].shape == (4,)
    c = m.clone()
    c[0, 0] = 1
    assert m[0, 0] == 0 and c[0, 0] == 1      # a clone owns its data; a row shares it
    row = m[2]
    row[3] = 4
    assert m[2, 3] == 4
    m.copyFrom(np.ones((3, 4), np.float32))
    out = np.zeros((3, 4), np.float32)
    m.copyTo(out)
    assert out.sum() == 12
    assert n.MGrid1d(5).type() == "float64" and n.MGrid8f(1, 1, 1, 1, 1, 1, 1, 2).size() == 2
    with pytest.raises(TypeError):
        n.MGrid2f(3)


def test_coordinate_sets_and_examples_on_the_host(n):
    coords = np.array([[0, 0, 0], [1, 2, 3]], np.float32)
    cs = n.CoordinateSet(coords, np.array([0, 2], np.float32), np.array([1.5, 2], np.float32), 4)
    assert cs.size() == 2 and cs.num_types() == 4 and cs.max_type == 4 and cs.src is None
    assert cs.has_indexed_types() and not cs.has_vector_types()
    assert tuple(cs.center()) == (0.5, 1.0, 1.5)
    np.testing.assert_array_equal(cs.coords.tonumpy(), coords)
    s = np.full(4, 9, np.float32)
    cs.sum_types(s)
    np.testing.assert_array_equal(s, [1, 0, 1, 0])
    cv = n.CoordinateSet(np.zeros((2, 3), np.float32), np.array([[0.5, 0.5], [0, 1]], np.float32),
                         np.ones(2, np.float32))
    assert cv.has_vector_types() and cv.num_types() == 2
    s2 = np.ones(2, np.float32)
    cv.sum_types(s2, zerofirst=False)
    np.testing.assert_array_equal(s2, [1.5, 2.5])
    with pytest.raises(TypeError):
        n.CoordinateSet(coords, np.array([0, 2], np.float32), np.array([1.5, 2], np.float32))   # no max_type
    with pytest.raises(ValueError):
        cs.sum_types(np.zeros(3, np.float32))

    ex = n.Example()
    ex.coord_sets.append(cs)
    ex.coord_sets.append(n.CoordinateSet(np.ones((1, 3), np.float32), np.array([1], np.float32),
                                         np.ones(1, np.float32), 3))
    ex.labels = [1.0, 2.5]
    ex.labels.append(3.0)
    assert ex.num_coordinates() == 3 and ex.num_types() == 7 and ex.num_types(False) == 4
    assert list(ex.labels) == [1.0, 2.5, 3.0] and ex.group == -1
    assert ex.has_index_types() and not ex.has_vector_types()
    mc = ex.merge_coordinates()
    assert mc.size() == 3 and mc.max_type == 7
    np.testing.assert_array_equal(mc.type_index.tonumpy(), [0, 2, 5])     # second set shifted by 4
    st = np.full(7, 3, np.float32)
    ex.sum_types(st)
    np.testing.assert_array_equal(st, [1, 0, 1, 0, 0, 1, 0])
    ev = n.ExampleVec([ex, ex])
    lab = np.zeros((2, 3), np.float32)
    ev.extract_labels(lab)
    np.testing.assert_array_equal(lab, [[1, 2.5, 3], [1, 2.5, 3]])
    one = np.zeros(2, np.float32)
    ev.extract_label(1, one)
    np.testing.assert_array_equal(one, [2.5, 2.5])
    both = np.zeros((2, 7), np.float32)
    ev.sum_types(both)
    np.testing.assert_array_equal(both[1], st)
    cs.make_vector_types()
    np.testing.assert_array_equal(cs.type_vector.tonumpy(), [[1, 0, 0, 0], [0, 0, 1, 0]])
    merged = n.CoordinateSet(cs, cs, True)
    assert merged.size() == 4 and merged.max_type == 8


@pytest.mark.gpu
def test_object_overloads_on_the_gpu(n, port):
    import torch
    import libmolgrid_b200 as molgrid
    T = 5
    coords, types, radii = cases.index_case(3, 80, T, 7.0)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    gm = n.GridMaker(0.5, 11.5)
    og = port.gm(0.5, 11.5)
    dims = gm.grid_dimensions(T)
    cs = n.CoordinateSet(coords, types, radii, T)
    center = (0.1, -0.2, 0.3)
    want = port.forward_index(og, center, coords, types, radii, T)

    out = torch.full(dims, -1.0, device="cuda")
    gm.forward(center, cs, out)                                   # (center, CoordinateSet, grid)
    assert np.allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    mg = n.MGrid4f(*dims)
    gm.forward(center, cs, mg)                                    # an MGrid as the output
    assert np.allclose(mg.tonumpy(), want, rtol=1e-5, atol=1e-6) and mg.ongpu()
    host = np.zeros(dims, np.float32)
    gm.forward(center, cs, host)                                  # a host array, staged through the device
    assert np.allclose(host, want, rtol=1e-5, atol=1e-6)

    # Example overloads: explicit Transform, and the random one against the ctypes layer with the same seed
    ex = n.Example()
    ex.coord_sets.append(cs)
    q = cases.random_quaternion(np.random.default_rng(1), 1)[0]
    tr = n.Transform(n.Quaternion(*[float(v) for v in q]), (0.5, 0.0, -0.5), (1.0, -1.0, 0.25))
    moved = port.transform_forward(port.tr(q, (0.5, 0.0, -0.5), (1.0, -1.0, 0.25)), coords)
    gm.forward(ex, tr, out)
    want_t = port.forward_index(og, (0.5, 0.0, -0.5), moved, types, radii, T)
    assert np.allclose(out.cpu().numpy(), want_t, rtol=1e-5, atol=1e-6)
    pex = molgrid.Example()
    pex.coord_sets.append(molgrid.CoordinateSet(coords, types, radii, T))
    pgm = molgrid.GridMaker(0.5, 11.5)
    a, b = torch.zeros(dims, device="cuda"), torch.zeros(dims, device="cuda")
    n.set_random_seed(7)
    gm.forward(ex, a, 1.5, True)
    molgrid.set_random_seed(7)
    pgm.forward(pex, b, 1.5, True)
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-6) and float(a.sum()) > 1
    batch = torch.zeros((2,) + dims, device="cuda")
    n.set_random_seed(7)
    gm.forward(n.ExampleVec([ex, ex]), batch, random_translation=1.5, random_rotation=True)
    assert torch.allclose(batch[0], a, rtol=1e-5, atol=1e-6) and not torch.equal(batch[0], batch[1])

    # backward with a CoordinateSet; Transform on CoordinateSets
    diff = np.random.default_rng(2).normal(size=dims).astype(np.float32)
    ag = torch.zeros((80, 3), device="cuda")
    gm.backward(center, cs, d(diff), ag)
    wantg = port.backward_index(og, center, coords, types, radii, diff)
    scale = max(1.0, float(np.abs(wantg).max()))
    assert np.allclose(ag.cpu().numpy(), wantg, rtol=1e-4, atol=1e-5 * scale)
    outset = cs.clone()
    tr.forward(cs, outset)
    np.testing.assert_array_equal(outset.coords.tonumpy(), moved)
    # sums of types on the device
    s = torch.full((T,), 4.0, device="cuda")
    cs.sum_types(s)
    hs = np.zeros(T, np.float32)
    cs.sum_types(hs)
    np.testing.assert_array_equal(s.cpu().numpy(), hs)
    # Grid views of CUDA tensors
    gt = n.Grid4fCUDA(out)
    assert gt.shape == dims and gt[0, 3, 3, 3] == float(out[0, 3, 3, 3])
    with pytest.raises(TypeError):
        n.Grid4f(out)


def test_merge_prefers_vector_types_in_both_layers():
    """Sets that carry index AND vector types (after make_vector_types) merge as vector types, type
    vectors side by side and the radii concatenated (src/example.cpp:198-228), in the compiled classes
    and in the Python layer alike."""
    import libmolgrid_b200 as molgrid
    from libmolgrid_b200 import molgrid_native
    rng = np.random.default_rng(4)
    merged = []
    for mod in (molgrid, molgrid_native):
        ex = mod.Example()
        for n, T in ((5, 3), (0, 2), (4, 2)):
            c = rng.normal(size=(n, 3)).astype(np.float32)
            t = rng.integers(0, T, n).astype(np.float32)
            r = rng.uniform(1, 2, n).astype(np.float32)
            cs = mod.CoordinateSet(c, t, r, T) if n else mod.CoordinateSet()
            if n:
                cs.make_vector_types(False, [1.0 + k for k in range(T)])
            else:
                cs.max_type = T
            ex.coord_sets.append(cs)
        rng = np.random.default_rng(4)      # the same numbers for the second module
        m = ex.merge_coordinates()
        assert m.has_vector_types() and m.max_type == 7
        merged.append((m.coords.tonumpy(), m.type_vector.tonumpy(), m.radii.tonumpy()))
    for a, b in zip(*merged):
        assert np.array_equal(a, b)
    tv, radii = merged[0][1], merged[0][2]
    assert tv.shape == (9, 7) and not tv[:5, 3:].any() and not tv[5:, :5].any() and np.array_equal(tv.sum(1), np.ones(9))
    assert np.array_equal(radii, [1, 2, 3, 1, 2])          # by type: set 0's three, set 2's two
