"""GridMaker / Transform overloads that take CoordinateSet, Example, Grid and MGrid arguments, on the
GPU.  Known answers follow the reference's own tests (test/test_gridmaker.py:131-214); the rest checks
that every overload reaches the same kernels as the array form."""
import numpy as np
import pytest
import torch

import libmolgrid_b200 as molgrid

pytestmark = pytest.mark.gpu


def one_atom(radius=1.0, x=0.0):
    c = np.array([[x, 0, 0]], np.float32)
    t = np.array([0], np.float32)
    r = np.array([radius], np.float32)
    return c, t, r


def test_line_profile_through_coordinate_set_and_mgrid():
    g1 = molgrid.GridMaker(resolution=.1, dimension=6.0)
    c, t, r = one_atom()
    coords = molgrid.CoordinateSet(molgrid.Grid2f(c), molgrid.Grid1f(t), molgrid.Grid1f(r), 1)
    shape = g1.grid_dimensions(1)
    a, b, d = molgrid.MGrid4f(*shape), molgrid.MGrid4f(*shape), molgrid.MGrid4f(*shape)
    g1.forward((0, 0, 0), coords, a.cpu())   # host view: staged through the device
    g1.forward((0, 0, 0), coords, b.gpu())   # device view: written in place
    g1.forward((0, 0, 0), c, t, r, d.cpu())  # array form
    assert b.ongpu() and a.oncpu()
    np.testing.assert_array_equal(a.tonumpy(), b.tonumpy())
    np.testing.assert_array_equal(a.tonumpy(), d.tonumpy())
    g = a.tonumpy()
    assert g[0, 30, 30, 30] == pytest.approx(1)
    line = g[0, 30, 30, :]
    xvals = np.abs(np.arange(-3, 3.1, .1))
    gauss = np.exp(-2 * xvals ** 2)
    quad = 4 * np.exp(-2) * xvals ** 2 - 12 * np.exp(-2) * xvals + 9 * np.exp(-2)
    for i in range(20, 41):
        assert line[i] == pytest.approx(gauss[i])
    for i in list(range(0, 15)) + list(range(45, 61)):
        assert line[i] == pytest.approx(0)
    for i in list(range(15, 20)) + list(range(41, 45)):
        assert line[i] == pytest.approx(quad[i], abs=1e-5)
    # numpy output and make_ndarray
    out = np.zeros(shape, np.float32)
    g1.forward((0, 0, 0), coords, out)
    np.testing.assert_array_equal(out, g)
    np.testing.assert_array_equal(g1.make_ndarray((0, 0, 0), coords), g)

    g2 = molgrid.GridMaker(resolution=.1, dimension=6.0, radius_scale=0.5, gaussian_radius_multiple=3.0)
    e = molgrid.MGrid4f(*shape)
    g2.forward((0, 0, 0), coords, e)  # an MGrid passed directly converts to its GPU side
    assert e.ongpu()
    line = e.tonumpy()[0, 30, :, 30]
    gauss = np.exp(-2 * (xvals * 2.0) ** 2)
    for i in range(0, 61):
        assert line[i] == pytest.approx(gauss[i], abs=1e-5)


def test_backward_after_random_rotation():
    g1 = molgrid.GridMaker(resolution=.1, dimension=6.0)
    c, t, r = one_atom(radius=2.0, x=1.0)
    coords = molgrid.CoordinateSet(c, t, r, 1)
    shape = g1.grid_dimensions(1)
    diff = molgrid.MGrid4f(*shape)
    diff[0, 30, 30, 30] = 1.0
    hostatoms, devatoms = molgrid.MGrid2f(1, 3), molgrid.MGrid2f(1, 3)
    T = molgrid.Transform((0, 0, 0), 0, True)
    T.forward(coords, coords)
    assert np.linalg.norm(coords.coords.tonumpy()) == pytest.approx(1.0, abs=1e-5)
    g1.backward((0, 0, 0), coords, diff.cpu(), hostatoms.cpu())
    g1.backward((0, 0, 0), coords, diff.gpu(), devatoms.gpu())
    T.backward(hostatoms.cpu(), hostatoms.cpu(), False)
    T.backward(devatoms.gpu(), devatoms.gpu(), False)
    np.testing.assert_allclose(hostatoms.tonumpy(), devatoms.tonumpy(), atol=1e-6)
    np.testing.assert_allclose(hostatoms.tonumpy().flatten(), [-0.60653067, 0, 0], atol=1e-5)
    with pytest.raises(ValueError):  # type gradients asked of a set without vector types
        g1.backward((0, 0, 0), coords, diff.gpu(), devatoms.gpu(), molgrid.MGrid2f(1, 1).gpu())


def make_example(rng, n1=40, n2=15, t1=5, t2=3):
    def cs(n, nt):
        pts = rng.uniform(-4, 4, (n, 3)).astype(np.float32)
        return molgrid.CoordinateSet(pts, rng.integers(0, nt, n).astype(np.float32),
                                     rng.uniform(1.0, 2.0, n).astype(np.float32), nt)
    ex = molgrid.Example()
    ex.coord_sets.append(cs(n1, t1))
    ex.coord_sets.append(cs(n2, t2))
    return ex


def test_example_overloads_match_array_form():
    rng = np.random.default_rng(11)
    ex = make_example(rng)
    gm = molgrid.GridMaker(0.5, 11.5)
    T = ex.num_types()
    assert T == 8
    dims = gm.grid_dimensions(T)
    m = ex.merge_coordinates()
    center = ex.coord_sets[-1].center()

    # forward(example, grid): identity transform about the last set's centre
    out = torch.zeros(dims, device="cuda")
    gm.forward(ex, out)
    want = torch.zeros(dims, device="cuda")
    gm.forward(center, m.coords.tonumpy(), m.type_index.tonumpy(), m.radii.tonumpy(), want)
    assert float(want.sum()) > 10
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-6)

    # forward(example, transform, grid) == transform the coordinates first, then grid
    tr = molgrid.Transform(molgrid.Quaternion(0.5, -0.5, 0.5, 0.5), (0.3, -0.2, 0.1), (1.0, -0.5, 0.25))
    gm.forward(ex, tr, out)
    moved = molgrid.CoordinateSet(m.coords.tonumpy(), m.type_index.tonumpy(), m.radii.tonumpy(), T)
    tr.forward(moved, moved)
    gm.forward(tr.get_rotation_center(), moved, want)
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-6)

    # random transforms: the same seed gives the same grid as drawing the Transform by hand
    molgrid.set_random_seed(7)
    gm.forward(ex, out, random_translation=2.0, random_rotation=True)
    molgrid.set_random_seed(7)
    tr = molgrid.Transform(center, 2.0, True)
    gm.forward(ex, tr, want)
    # (the grid is a sum of floating-point reductions in arbitrary order: equal to rounding)
    torch.testing.assert_close(out, want, rtol=1e-6, atol=1e-7)

    with pytest.raises(IndexError):
        gm.forward(ex, torch.zeros(gm.grid_dimensions(T + 1), device="cuda"))


def test_example_vector_is_one_batched_call():
    rng = np.random.default_rng(12)
    exs = molgrid.ExampleVec([make_example(rng, n1=30 + 7 * i, n2=5 + i) for i in range(4)])
    exs[2].coord_sets[1] = molgrid.CoordinateSet()  # an empty set in the middle of the batch
    exs[2].coord_sets[1].max_type = 3
    gm = molgrid.GridMaker(0.5, 11.5)
    dims = gm.grid_dimensions(8)
    batch = torch.zeros((4,) + dims, device="cuda")
    molgrid.set_random_seed(3)
    gm.forward(exs, batch, random_translation=1.0, random_rotation=True)
    molgrid.set_random_seed(3)
    for i, ex in enumerate(exs):
        one = torch.zeros(dims, device="cuda")
        gm.forward(ex, one, 1.0, True)
        torch.testing.assert_close(batch[i], one, rtol=1e-5, atol=1e-6)
    # MGrid5f output
    mg = molgrid.MGrid5f(4, *dims)
    molgrid.set_random_seed(3)
    gm.forward(exs, mg, 1.0, True)
    np.testing.assert_allclose(mg.tonumpy(), batch.cpu().numpy(), rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        gm.forward(exs, torch.zeros((3,) + dims, device="cuda"))


def test_vector_types_win_when_a_set_has_both():
    rng = np.random.default_rng(13)
    pts = rng.uniform(-3, 3, (20, 3)).astype(np.float32)
    types = rng.integers(0, 4, 20).astype(np.float32)
    c = molgrid.CoordinateSet(pts, types, np.full(20, 1.5, np.float32), 4)
    gm = molgrid.GridMaker(0.5, 9.5)
    dims = gm.grid_dimensions(4)
    a = torch.zeros(dims, device="cuda")
    gm.forward((0, 0, 0), c, a)
    c.make_vector_types()
    c.type_vector.cpu().t.mul_(0.5)   # halve the weights: only the vector path can see this
    b = torch.zeros(dims, device="cuda")
    gm.forward((0, 0, 0), c, b)
    torch.testing.assert_close(b, 0.5 * a, rtol=1e-5, atol=1e-6)
    # backward through the set: index form and vector form
    diff = torch.randn(dims, device="cuda")
    ag_i = torch.zeros((20, 3), device="cuda")
    gm.backward((0, 0, 0), c, diff, ag_i)
    ag_v, tg = torch.zeros((20, 3), device="cuda"), torch.zeros((20, 4), device="cuda")
    gm.backward((0, 0, 0), c, diff, ag_v, tg)
    torch.testing.assert_close(ag_v, 0.5 * ag_i, rtol=1e-4, atol=1e-5)
    # relevance through the set
    rel = torch.zeros(20, device="cuda")
    gm.backward_relevance((0, 0, 0), c, a, diff, rel)
    want = torch.zeros(20, device="cuda")
    gm.backward_relevance((0, 0, 0), pts, types, np.full(20, 1.5, np.float32), a, diff, want)
    torch.testing.assert_close(rel, want, rtol=0, atol=0)


def test_gpu_disabled_keeps_results_on_the_host_side():
    gm = molgrid.GridMaker(0.5, 6.0)
    c, t, r = one_atom()
    cs = molgrid.CoordinateSet(c, t, r, 1)
    out = molgrid.MGrid4f(*gm.grid_dimensions(1))
    try:
        molgrid.set_gpu_enabled(False)
        assert not molgrid.get_gpu_enabled()
        gm.forward((0, 0, 0), cs, out)
        assert out.oncpu()
    finally:
        molgrid.set_gpu_enabled(True)
    assert out[0, 6, 6, 6] == pytest.approx(1.0)
    assert molgrid.get_gpu_device() == torch.cuda.current_device()
    dev = molgrid.Grid1fCUDA(torch.arange(4, dtype=torch.float32, device="cuda"))
    alias = molgrid.Grid1fCUDA(molgrid.tofloatptr(dev.data()), 4)
    assert alias[3] == 3.0


def test_vector_types_through_coordinate_sets():
    """test/test_gridmaker.py:217-277: index and one-hot vector types give the same grid, half
    weights half the density, and the gradients of two atoms towards a target between them are
    opposite."""
    g1 = molgrid.GridMaker(resolution=.25, dimension=6.0)
    c = np.array([[0, 0, 0], [2, 0, 0]], np.float32)
    t = np.array([0, 1], np.float32)
    vt = np.array([[1.0, 0], [0, 1.0]], np.float32)
    vt2 = np.array([[0.5, 0.0], [0.0, 0.5]], np.float32)
    r = np.array([1.0, 1.0], np.float32)
    coords = molgrid.CoordinateSet(molgrid.Grid2f(c), molgrid.Grid1f(t), molgrid.Grid1f(r), 2)
    vcoords = molgrid.CoordinateSet(molgrid.Grid2f(c), molgrid.Grid2f(vt), molgrid.Grid1f(r))
    v2coords = molgrid.CoordinateSet(molgrid.Grid2f(c), molgrid.Grid2f(vt2), molgrid.Grid1f(r))
    shape = g1.grid_dimensions(2)
    reference, vgrid, v2grid, v3grid = (molgrid.MGrid4f(*shape) for _ in range(4))
    g1.forward((0, 0, 0), coords, reference.cpu())
    g1.forward((0, 0, 0), vcoords, vgrid.gpu())
    g1.forward((0, 0, 0), v2coords, v2grid.gpu())
    g1.forward((0, 0, 0), c, vt, r, v3grid.cpu())
    g = reference.tonumpy()
    assert g.sum() > 50
    np.testing.assert_allclose(g, vgrid.tonumpy(), atol=1e-5)
    np.testing.assert_allclose(vgrid.tonumpy(), v3grid.tonumpy(), atol=1e-6)
    np.testing.assert_allclose(g, v2grid.tonumpy() * 2.0, atol=1e-5)

    tc = molgrid.Grid2f(np.array([[1, 0, 0]], np.float32))
    tv = molgrid.Grid2f(np.array([[0.5, 0.5]], np.float32))
    tr = molgrid.Grid1f(np.array([1.0], np.float32))
    tgrid = molgrid.MGrid4f(*shape)
    g1.forward((0, 0, 0), molgrid.CoordinateSet(tc, tv, tr), tgrid.cpu())
    gradc, gradt = molgrid.MGrid2f(2, 3), molgrid.MGrid2f(2, 2)
    g1.backward((0, 0, 0), vcoords, tgrid.gpu(), gradc.gpu(), gradt.gpu())
    assert gradc[0, 0] == pytest.approx(-gradc[1, 0], abs=1e-4)
    assert gradc[0, 0] > 0


def test_vector_backward_signs():
    """test/test_gridmaker.py:364-391."""
    g1 = molgrid.GridMaker(resolution=.1, dimension=6.0)
    c = np.array([[1.0, 0, 0], [-1, -1, 0]], np.float32)
    t = np.array([[0, 1.0, 0], [1.0, 0, 0]], np.float32)
    r = np.array([2.0, 2.0], np.float32)
    coords = molgrid.CoordinateSet(c, t, r)
    shape = g1.grid_dimensions(3)
    diff = molgrid.MGrid4f(*shape)
    diff[0, 30, 30, 30] = 1.0
    diff[1, 30, 30, 30] = -1.0
    atoms, types = molgrid.MGrid2f(2, 3), molgrid.MGrid2f(2, 3)
    g1.backward((0, 0, 0), coords, diff.gpu(), atoms.gpu(), types.gpu())
    assert types[0][0] > 0 and types[0][1] < 0 and types[0][2] == 0
    host_atoms, host_types = molgrid.MGrid2f(2, 3), molgrid.MGrid2f(2, 3)
    g1.backward((0, 0, 0), coords, diff.cpu(), host_atoms.cpu(), host_types.cpu())
    np.testing.assert_array_equal(atoms.tonumpy(), host_atoms.tonumpy())
    np.testing.assert_array_equal(types.tonumpy(), host_types.tonumpy())


def test_type_indexed_radii_with_dummy_type():
    """test/test_gridmaker.py:393-437: make_vector_types(True, radii) adds an empty dummy type and
    turns the radii into per-type radii."""
    g1 = molgrid.GridMaker(resolution=.25, dimension=6.0, radius_type_indexed=True)
    c = np.array([[0, 0, 0]], np.float32)
    coords = molgrid.CoordinateSet(molgrid.Grid2f(c), molgrid.Grid1f(np.array([0], np.float32)),
                                   molgrid.Grid1f(np.array([1.0], np.float32)), 2)
    coords.make_vector_types(True, [3.0, 1.0])
    shape = g1.grid_dimensions(3)
    assert g1.get_radii_type_indexed()
    data = molgrid.MGrid4f(*shape)
    g1.forward((0, 0, 0), coords, data.gpu())
    assert data.tonumpy().sum() > 2980          # a radius of 1 would give 116
    data.fill_zero()
    data[0, 20, 12, 12] = -1
    data[1, 20, 12, 12] = 1
    data[2, 20, 12, 12] = 2
    atoms, types = molgrid.MGrid2f(1, 3), molgrid.MGrid2f(1, 3)
    g1.backward((0, 0, 0), coords, data.gpu(), atoms.gpu(), types.gpu())
    assert atoms[0][0] < 0 and atoms[0][1] == 0 and atoms[0][2] == 0
    assert types[0][0] < 0 and types[0][1] == 0 and types[0][2] == 0


def test_second_derivative_along_each_axis():
    """test/test_gridmaker.py:439-487: with a truncated Gaussian (gaussian_radius_multiple = -2) the
    gradient of |d grid point / d coords|^2 is -128 d^3 e^{-4 d^2} + 32 d e^{-4 d^2} along each axis,
    and symmetric on the diagonal."""
    gmaker = molgrid.GridMaker(resolution=0.5, dimension=6.0, gaussian_radius_multiple=-2.0)
    types = torch.ones(1, 1, dtype=torch.float32, device="cuda")
    radii = torch.ones(1, dtype=torch.float32, device="cuda")
    for i in range(3):
        for x in np.arange(-0.9, 3, .3):
            coords = torch.zeros(1, 3, dtype=torch.float32, device="cuda")
            coords[0][i] = x
            coords.requires_grad = True
            outgrid = molgrid.Coords2GridFunction.apply(gmaker, (0, 0, 0), coords, types, radii)
            idx = [0, 6, 6, 6]
            idx[i + 1] = 8
            gp = outgrid[tuple(idx)]
            Lg = torch.autograd.grad(gp, coords, create_graph=True)[0]
            val = float(torch.autograd.grad(torch.sum(Lg ** 2), coords)[0][0][i])
            d = x - 1
            assert val == pytest.approx(-128 * d ** 3 * np.exp(-4 * d ** 2) + 32 * d * np.exp(-4 * d ** 2), abs=1e-4)
    coords = torch.zeros(1, 3, dtype=torch.float32, requires_grad=True, device="cuda")
    outgrid = molgrid.Coords2GridFunction.apply(gmaker, (0, 0, 0), coords, types, radii)
    f = []
    for p in (7, 8):
        Lg = torch.autograd.grad(outgrid[0][p][p][p], coords, create_graph=True)[0]
        f.append(torch.autograd.grad(torch.sum(Lg ** 2), coords, retain_graph=True)[0][0])
    for fl in f:
        assert float(fl[0]) == pytest.approx(float(fl[1]), rel=1e-5)
        assert float(fl[2]) == pytest.approx(float(fl[1]), rel=1e-5)
    assert float(f[1][0]) < float(f[0][0])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_devices():
    """test/test_gridmaker.py:105-128: a tensor on another device than the current one is refused
    with ValueError; after set_gpu_device it is accepted, and each device computes the same grid."""
    gm = molgrid.GridMaker(0.5, 6.0)
    c, t, r = one_atom()
    cs = molgrid.CoordinateSet(c, t, r, 1)
    dims = gm.grid_dimensions(1)
    out0 = torch.zeros(dims, device="cuda:0")
    out1 = torch.zeros(dims, device="cuda:1")
    assert molgrid.get_gpu_device() == 0
    gm.forward((0, 0, 0), cs, out0)
    with pytest.raises(ValueError):
        gm.forward((0, 0, 0), c, t, r, out1)
    try:
        molgrid.set_gpu_device(1)
        assert molgrid.get_gpu_device() == 1
        gm.forward((0, 0, 0), c, t, r, out1)
        with pytest.raises(ValueError):
            gm.forward((0, 0, 0), c, t, r, out0)
    finally:
        molgrid.set_gpu_device(0)
    assert torch.equal(out0.cpu(), out1.cpu()) and float(out0[0, 6, 6, 6]) == pytest.approx(1.0)
