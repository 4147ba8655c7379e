"""GPU parity of GridMaker forward/backward/relevance against the CPU oracle.

Every call goes through the C ABI (libmolgrid_b200.api is a ctypes wrapper over it).
Tolerances are the ones the path states: binary grids and channel assignment bit-exact, densities
rel 1e-5 / abs 1e-6, gradients and relevance rel 1e-4 (abs floor 1e-5 x the gradient scale).
"""
import numpy as np
import pytest
import torch

from tests import cases

pytestmark = pytest.mark.gpu

DENS = dict(rtol=1e-5, atol=1e-6)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def gm_pair(port, **kw):
    import libmolgrid_b200 as lmg
    g = lmg.GridMaker(kw.get("resolution", 0.5), kw.get("dimension", 23.5), kw.get("binary", False),
                      kw.get("radius_type_indexed", False), kw.get("radius_scale", 1.0),
                      kw.get("gaussian_radius_multiple", 1.0))
    og = port.gm(kw.get("resolution", 0.5), kw.get("dimension", 23.5), kw.get("binary", False),
                 kw.get("radius_type_indexed", False), kw.get("radius_scale", 1.0),
                 kw.get("gaussian_radius_multiple", 1.0))
    return g, og


def grad_close(a, b, what):
    scale = max(1.0, float(np.abs(b).max()))
    assert np.allclose(a, b, rtol=1e-4, atol=1e-5 * scale), \
        "%s: max abs diff %g (scale %g)" % (what, np.abs(a - b).max(), scale)


SETTINGS = [
    dict(),                                                           # the benchmark's settings
    dict(resolution=0.5, dimension=6.0),                              # 13 points: not a multiple of 4
    dict(resolution=0.25, dimension=7.75, radius_scale=0.5, gaussian_radius_multiple=3.0),
    dict(resolution=0.5, dimension=11.5, radius_scale=1.2, gaussian_radius_multiple=-2.0),
    dict(resolution=0.5, dimension=11.5, gaussian_radius_multiple=-1.5),
    dict(resolution=0.375, dimension=9.0, gaussian_radius_multiple=0.7),
]


@pytest.mark.parametrize("kw", SETTINGS)
@pytest.mark.parametrize("binary", [False, True])
def test_forward_index(port, kw, binary):
    kw = dict(kw, binary=binary)
    g, og = gm_pair(port, **kw)
    T = 28 if not kw.get("dimension") else 5
    ext = 10.0 if not kw.get("dimension") else kw["dimension"] / 2 + 1
    coords, types, radii = cases.index_case(1000, 300, T, ext)
    center = (0.1, -0.2, 0.3)
    want = port.forward_index(og, center, coords, types, radii, T)
    out = torch.full(g.grid_dimensions(T), -7.0, device="cuda")
    g.forward(center, dev(coords), dev(types), dev(radii), out)
    g.check_types()
    got = out.cpu().numpy()
    if binary:
        assert np.array_equal(got, want)
    else:
        assert np.array_equal(got != 0, want != 0) or kw.get("gaussian_radius_multiple", 1) > 0
        assert np.allclose(got, want, **DENS), np.abs(got - want).max()


def test_forward_c0_known_answers(port):
    """Line profile of one atom (test/test_gridmaker.py:131-164 of the reference)."""
    g, og = gm_pair(port, resolution=0.1, dimension=6.0)
    out = torch.zeros(g.grid_dimensions(1), device="cuda")
    g.forward((0, 0, 0), dev(np.zeros((1, 3), np.float32)), dev(np.zeros(1, np.float32)),
              dev(np.ones(1, np.float32)), out)
    o = out.cpu().numpy()[0]
    c = o.shape[0] // 2
    assert o[c, c, c] == pytest.approx(1.0, abs=1e-6)
    assert o[c + 5, c, c] == pytest.approx(0.60653066, rel=1e-5)
    assert o[c, c - 12, c] == pytest.approx(0.0487206, rel=1e-4)
    assert o[c, c, c + 15] == pytest.approx(0.0, abs=1e-6)


def test_forward_transform_fused(port):
    g, og = gm_pair(port)
    T = 28
    coords, types, radii = cases.index_case(7, 500, T, 10.0)
    rng = np.random.default_rng(3)
    q = cases.random_quaternion(rng, 1)[0]
    tr = port.tr(q, (0.5, 1.0, -0.5), rng.uniform(-2, 2, 3))
    moved = port.transform_forward(tr, coords)
    for binary in (False, True):
        g.set_binary(binary)
        og[2] = float(binary)
        want = port.forward_index(og, (0.5, 1.0, -0.5), moved, types, radii, T)
        import libmolgrid_b200 as lmg
        t = lmg.Transform(lmg.Quaternion(*q), tuple(tr[4:7]), tuple(tr[7:10]))
        out = torch.empty(g.grid_dimensions(T), device="cuda")
        g.forward((0.5, 1.0, -0.5), dev(coords), dev(types), dev(radii), out, transforms=t)
        got = out.cpu().numpy()
        if binary:
            assert np.array_equal(got, want)
        else:
            assert np.allclose(got, want, **DENS)


@pytest.mark.parametrize("binary", [False, True])
def test_forward_batched_blob(port, binary):
    """A small batch with the benchmark's atom statistics, ragged sizes, per-example transforms."""
    g, og = gm_pair(port, binary=binary)
    B, T = 3, 28
    coords, types, radii, ns, tr = cases.blob_batch(1001, B, 2000, 4000, T)
    out = torch.empty((B,) + g.grid_dimensions(T), device="cuda")
    centers = np.zeros((B, 3), np.float32)
    g.forward(dev(centers), dev(coords), dev(types), dev(radii), out, transforms=dev(tr),
              n_atoms=torch.from_numpy(ns))
    got = out.cpu().numpy()
    for b in range(B):
        n = ns[b]
        moved = port.transform_forward(tr[b], coords[b, :n])
        want = port.forward_index(og, (0, 0, 0), moved, types[b, :n], radii[b, :n], T)
        if binary:
            assert np.array_equal(got[b], want)
        else:
            assert np.allclose(got[b], want, **DENS), np.abs(got[b] - want).max()


@pytest.mark.parametrize("rti", [False, True])
@pytest.mark.parametrize("binary", [False, True])
@pytest.mark.parametrize("kw", [dict(resolution=0.5, dimension=11.5),
                                dict(resolution=0.25, dimension=7.75),
                                dict(resolution=0.5, dimension=6.0, gaussian_radius_multiple=-1.5)])
def test_forward_vector(port, kw, rti, binary):
    kw = dict(kw, binary=binary, radius_type_indexed=rti)
    g, og = gm_pair(port, **kw)
    T = 6
    coords, tv, radii = cases.vector_case(11, 200, T, kw["dimension"] / 2 + 1, rti=rti)
    want = port.forward_vector(og, (0, 0, 0), coords, tv, radii)
    out = torch.empty(g.grid_dimensions(T), device="cuda")
    g.forward((0, 0, 0), dev(coords), dev(tv), dev(radii), out)
    got = out.cpu().numpy()
    assert np.allclose(got, want, **DENS), np.abs(got - want).max()
    if binary:
        assert np.array_equal(got != 0, want != 0)


def test_vector_equals_index(port):
    """One-hot type vectors give the index-typed grid (test/test_gridmaker.py:217-240)."""
    g, og = gm_pair(port, resolution=0.5, dimension=11.5)
    T = 5
    coords, types, radii = cases.index_case(5, 100, T, 6.0, ties=False)
    tv = np.zeros((100, T), np.float32)
    tv[np.arange(100), types.astype(int)] = 1
    a = torch.empty(g.grid_dimensions(T), device="cuda")
    b = torch.empty(g.grid_dimensions(T), device="cuda")
    g.forward((0, 0, 0), dev(coords), dev(types), dev(radii), a)
    g.forward((0, 0, 0), dev(coords), dev(tv), dev(radii), b)
    assert torch.allclose(a, b, rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("kw", SETTINGS)
def test_backward_index_and_relevance(port, kw):
    g, og = gm_pair(port, **kw)
    T = 28 if not kw.get("dimension") else 5
    ext = 10.0 if not kw.get("dimension") else kw["dimension"] / 2 + 1
    coords, types, radii = cases.index_case(1002, 300, T, ext)
    rng = np.random.default_rng(5)
    diff = rng.normal(size=g.grid_dimensions(T)).astype(np.float32)
    want = port.backward_index(og, (0, 0, 0), coords, types, radii, diff)
    ag = torch.full((300, 3), 9.0, device="cuda")
    g.backward((0, 0, 0), dev(coords), dev(types), dev(radii), dev(diff), ag)
    grad_close(ag.cpu().numpy(), want, "atom gradients")

    dens = port.forward_index(og, (0, 0, 0), coords, types, radii, T)
    wantr = port.backward_relevance(og, (0, 0, 0), coords, types, radii, dens, diff)
    rel = torch.full((300,), 9.0, device="cuda")
    g.backward_relevance((0, 0, 0), dev(coords), dev(types), dev(radii), dev(dens), dev(diff), rel)
    grad_close(rel.cpu().numpy(), wantr, "relevance")


def test_backward_known_answer(port):
    """d/dx of one atom at (1,0,0), r=2, upstream 1 at the centre voxel: -0.60653
    (test/test_gridmaker.py:186-214, test/test_torch.py:128-140 of the reference)."""
    g, og = gm_pair(port, resolution=0.5, dimension=29.5 + 0.5)
    d = g.spatial_grid_dimensions()[0]
    diff = np.zeros((1, d, d, d), np.float32)
    diff[0, d // 2, d // 2, d // 2] = 1.0
    coords = np.array([[1, 0, 0]], np.float32)
    ag = torch.zeros((1, 3), device="cuda")
    g.backward((0, 0, 0), dev(coords), dev(np.zeros(1, np.float32)), dev(np.full(1, 2.0, np.float32)),
               dev(diff), ag)
    want = port.backward_index(og, (0, 0, 0), coords, [0], [2.0], diff)
    grad_close(ag.cpu().numpy(), want, "single atom")
    if d % 2 == 1:
        assert ag[0, 0].item() == pytest.approx(-0.60653066, rel=1e-4)


@pytest.mark.parametrize("dimension", [11.5, 11.0])   # 24 points, and 23: rows not 16-byte aligned
@pytest.mark.parametrize("rti", [False, True])
@pytest.mark.parametrize("binary", [False, True])
def test_backward_vector(port, rti, binary, dimension):
    kw = dict(resolution=0.5, dimension=dimension, binary=binary, radius_type_indexed=rti)
    g, og = gm_pair(port, **kw)
    T = 6
    coords, tv, radii = cases.vector_case(13, 150, T, dimension / 2 + 0.75, rti=rti)
    rng = np.random.default_rng(6)
    diff = rng.normal(size=g.grid_dimensions(T)).astype(np.float32)
    wag, wtg = port.backward_vector(og, (0, 0, 0), coords, tv, radii, diff)
    ag = torch.full((150, 3), 9.0, device="cuda")
    tg = torch.full((150, T), 9.0, device="cuda")
    g.backward((0, 0, 0), dev(coords), dev(tv), dev(radii), dev(diff), ag, tg)
    grad_close(ag.cpu().numpy(), wag, "atom gradients")
    grad_close(tg.cpu().numpy(), wtg, "type gradients")


def test_backward_batched(port):
    g, og = gm_pair(port)
    B, T = 2, 28
    coords, types, radii, ns, tr = cases.blob_batch(1002, B, 2000, 2500, T)
    rng = np.random.default_rng(8)
    diff = rng.normal(size=(B,) + g.grid_dimensions(T)).astype(np.float32)
    N = coords.shape[1]
    ag = torch.full((B, N, 3), 9.0, device="cuda")
    g.backward(dev(np.zeros((B, 3), np.float32)), dev(coords), dev(types), dev(radii), dev(diff), ag,
               transforms=dev(tr), n_atoms=torch.from_numpy(ns))
    got = ag.cpu().numpy()
    for b in range(B):
        n = ns[b]
        moved = port.transform_forward(tr[b], coords[b, :n])
        want = port.backward_index(og, (0, 0, 0), moved, types[b, :n], radii[b, :n], diff[b])
        grad_close(got[b, :n], want, "example %d" % b)
        assert np.all(got[b, n:] == 0)


def test_errors(port):
    import libmolgrid_b200 as lmg
    g = lmg.GridMaker(0.5, 5.5)
    c = torch.zeros((4, 3), device="cuda")
    t = torch.zeros(4, device="cuda")
    r = torch.ones(4, device="cuda")
    with pytest.raises(IndexError):          # wrong grid size -> std::out_of_range
        g.forward((0, 0, 0), c, t, r, torch.zeros((2, 11, 11, 11), device="cuda"))
    with pytest.raises(IndexError):          # radii length
        g.forward((0, 0, 0), c, t, torch.ones(3, device="cuda"), torch.zeros((2, 12, 12, 12), device="cuda"))
    with pytest.raises(ValueError):          # non-contiguous
        g.forward((0, 0, 0), torch.zeros((3, 4), device="cuda").t(), t, r,
                  torch.zeros((2, 12, 12, 12), device="cuda"))
    g2 = lmg.GridMaker(0.5, 5.5, False, True)
    with pytest.raises(ValueError):          # type-indexed radii with index types
        g2.forward((0, 0, 0), c, t, r, torch.zeros((2, 12, 12, 12), device="cuda"))
    # a type index beyond the channels is reported through the status word
    out = torch.zeros((2, 12, 12, 12), device="cuda")
    g.forward((0, 0, 0), c, torch.full((4,), 2.0, device="cuda"), r, out)
    with pytest.raises(IndexError):
        g.check_types()
    # negative types are skipped silently
    g.forward((0, 0, 0), c, torch.full((4,), -1.0, device="cuda"), r, out)
    g.check_types()
    assert float(out.abs().sum()) == 0.0


def test_small_workspace_runs_in_passes(port):
    """A workspace that holds one example at a time gives the same grids."""
    import libmolgrid_b200.api as api
    g, og = gm_pair(port, resolution=0.5, dimension=11.5)
    B, T, N = 5, 4, 64
    rng = np.random.default_rng(0)
    coords = rng.uniform(-6, 6, (B, N, 3)).astype(np.float32)
    types = rng.integers(0, T, (B, N)).astype(np.float32)
    radii = rng.uniform(1, 2, (B, N)).astype(np.float32)
    centers = np.zeros((B, 3), np.float32)
    a = torch.empty((B,) + g.grid_dimensions(T), device="cuda")
    g.forward(dev(centers), dev(coords), dev(types), dev(radii), a)
    old = api.MAX_WORKSPACE_BYTES
    try:
        one = api._cabi.lib().lmg_workspace_bytes(g.s, 0, 1, N, T, 0)
        api.MAX_WORKSPACE_BYTES = one + 1024
        api._workspaces.clear()
        b = torch.empty_like(a)
        g.forward(dev(centers), dev(coords), dev(types), dev(radii), b)
    finally:
        api.MAX_WORKSPACE_BYTES = old
        api._workspaces.clear()
    assert torch.equal(a != 0, b != 0)
    assert torch.allclose(a, b, rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("binary", [False, True])
def test_footprints_wider_than_the_column_buffer(port, binary):
    """Atoms whose footprint holds more columns than a warp compacts at a time (256), and whose z
    extent needs several passes of quads: radius 4 A at 0.25 A is 49 points across."""
    g, og = gm_pair(port, resolution=0.25, dimension=11.75, binary=binary)
    T = 3
    coords, types, radii = cases.index_case(21, 40, T, 6.5)
    radii[::3] = 4.0
    want = port.forward_index(og, (0, 0, 0), coords, types, radii, T)
    out = torch.empty(g.grid_dimensions(T), device="cuda")
    g.forward((0, 0, 0), dev(coords), dev(types), dev(radii), out)
    got = out.cpu().numpy()
    if binary:
        assert np.array_equal(got, want)
    else:
        assert np.allclose(got, want, **DENS), np.abs(got - want).max()
    diff = np.random.default_rng(2).normal(size=want.shape).astype(np.float32)
    ag = torch.empty((40, 3), device="cuda")
    g.backward((0, 0, 0), dev(coords), dev(types), dev(radii), dev(diff), ag)
    grad_close(ag.cpu().numpy(), port.backward_index(og, (0, 0, 0), coords, types, radii, diff), "atom gradients")
    vc, tv, vr = cases.vector_case(22, 30, T, 6.5)
    vr[::2] = 3.5
    outv = torch.empty(g.grid_dimensions(T), device="cuda")
    g.forward((0, 0, 0), dev(vc), dev(tv), dev(vr), outv)
    assert np.allclose(outv.cpu().numpy(), port.forward_vector(og, (0, 0, 0), vc, tv, vr), **DENS)


@pytest.mark.parametrize("binary", [False, True])
def test_many_atoms_in_one_channel(port, binary):
    """More atoms of one channel than a block lists at a time, all other channels empty."""
    g, og = gm_pair(port, resolution=0.5, dimension=11.5, binary=binary)
    T, N = 4, 5000
    rng = np.random.default_rng(77)
    coords = cases.sphere(rng, N, 7.5)
    types = np.full(N, 2.0, np.float32)
    types[:40] = rng.integers(0, T, 40)
    radii = rng.uniform(0.6, 1.2, N).astype(np.float32)
    want = port.forward_index(og, (0, 0, 0), coords, types, radii, T)
    out = torch.full(g.grid_dimensions(T), -1.0, device="cuda")
    g.forward((0, 0, 0), dev(coords), dev(types), dev(radii), out)
    got = out.cpu().numpy()
    if binary:
        assert np.array_equal(got, want)
    else:
        # hundreds of terms per voxel, summed in no fixed order
        assert np.allclose(got, want, rtol=2e-5, atol=1e-6), np.abs(got - want).max()
    diff = rng.normal(size=want.shape).astype(np.float32)
    ag = torch.empty((N, 3), device="cuda")
    g.backward((0, 0, 0), dev(coords), dev(types), dev(radii), dev(diff), ag)
    grad_close(ag.cpu().numpy(), port.backward_index(og, (0, 0, 0), coords, types, radii, diff), "atom gradients")


@pytest.mark.parametrize("rti", [False, True])
@pytest.mark.parametrize("kw", [dict(resolution=0.5, dimension=11.5),
                                dict(resolution=0.5, dimension=6.0),   # 13 points: rows not 16-byte aligned
                                dict(resolution=0.25, dimension=5.75, gaussian_radius_multiple=-2.0)])
def test_backward_gradients(port, kw, rti):
    """Second-order pass against the oracle; also batched with per-example transforms."""
    kw = dict(kw, radius_type_indexed=rti)
    g, og = gm_pair(port, **kw)
    T, N, B = 4, 40, 2
    rng = np.random.default_rng(17)
    coords = np.stack([cases.vector_case(30 + b, N, T, kw["dimension"] / 2 + 0.5, rti=rti)[0] for b in range(B)])
    tv = np.stack([cases.vector_case(30 + b, N, T, 5, rti=rti)[1] for b in range(B)])
    radii = np.stack([cases.vector_case(30 + b, N, T, 5, rti=rti)[2] for b in range(B)])
    shape = (B,) + g.grid_dimensions(T)
    diff = rng.normal(size=shape).astype(np.float32)
    ag = rng.normal(size=(B, N, 3)).astype(np.float32)
    tg = rng.normal(size=(B, N, T)).astype(np.float32)
    q = cases.random_quaternion(rng, B)
    tr = np.zeros((B, 10), np.float32)
    tr[:, :4] = q
    tr[:, 7:] = rng.uniform(-1, 1, (B, 3))
    dd = torch.empty(shape, device="cuda")
    add = torch.empty((B, N, 3), device="cuda")
    tdd = torch.full((B, N, T), 3.0, device="cuda")
    g.backward_gradients(dev(np.zeros((B, 3), np.float32)), dev(coords), dev(tv), dev(radii), dev(diff), dev(ag),
                         dev(tg), dd, add, tdd, transforms=dev(tr))
    for b in range(B):
        moved = port.transform_forward(tr[b], coords[b])
        wdd, wadd, wtdd = port.backward_gradients(og, (0, 0, 0), moved, tv[b], radii[b], diff[b], ag[b], tg[b])
        grad_close(dd[b].cpu().numpy(), wdd, "diffdiff")
        grad_close(add[b].cpu().numpy(), wadd, "atom_diffdiff")
    assert not tdd.any()


@pytest.mark.parametrize("rti", [False, True])
@pytest.mark.parametrize("kw", [dict(resolution=0.5, dimension=11.5), dict(resolution=0.5, dimension=11.0)])
def test_backward_vector_without_type_gradients(port, kw, rti):
    """Vector types, atom gradients only: same atom gradients as the full call, on the per-atom
    kernels (per-atom radii, rows 16-byte aligned) and on the per-(atom, channel) kernels."""
    g, og = gm_pair(port, radius_type_indexed=rti, **kw)
    T, N = 6, 50
    coords, tv, radii = cases.vector_case(5, N, T, kw["dimension"] / 2 + 1, rti=rti)
    tv[:10] = 0
    tv[np.arange(10), np.arange(10) % T] = 1.0      # some one-hot atoms
    dims = g.grid_dimensions(T)
    diff = np.random.default_rng(6).normal(size=dims).astype(np.float32)
    ag, tg = torch.zeros((N, 3), device="cuda"), torch.zeros((N, T), device="cuda")
    g.backward((0, 0, 0), dev(coords), dev(tv), dev(radii), dev(diff), ag, tg)
    only = torch.full((N, 3), 9.0, device="cuda")
    g.backward_arrays((0, 0, 0), dev(coords), dev(tv), dev(radii), dev(diff), only, want_type_gradients=False)
    wag, wtg = port.backward_vector(og, (0, 0, 0), coords, tv, radii, diff)
    grad_close(ag.cpu().numpy(), wag, "atom gradients")
    grad_close(tg.cpu().numpy(), wtg, "type gradients")
    grad_close(only.cpu().numpy(), wag, "atom gradients alone")


@pytest.mark.parametrize("binary", [False, True])
def test_backward_vector_rounds_of_channels(port, binary):
    """Per-atom radii with 28 channels: the kernel takes the channels in rounds, and a round may hold
    no weighted channel of an atom, one or two (one-hot and two-hot types) or many."""
    g, og = gm_pair(port, resolution=0.5, dimension=11.5, binary=binary)
    T, N = 28, 120
    coords, tv, radii = cases.vector_case(21, N, T, 6.5)
    rng = np.random.default_rng(3)
    tv[:40] = 0
    tv[np.arange(40), rng.integers(0, T, 40)] = 1.0                 # one-hot
    tv[40:80] = 0
    for a in range(40, 80):                                         # two channels, often in one round
        c = rng.integers(0, T - 1)
        tv[a, c], tv[a, c + 1] = 0.25, 0.75
    tv[80:90] = rng.uniform(0.1, 1.0, (10, T)).astype(np.float32)   # every channel weighted
    diff = rng.normal(size=g.grid_dimensions(T)).astype(np.float32)
    wag, wtg = port.backward_vector(og, (0, 0, 0), coords, tv, radii, diff)
    ag = torch.full((N, 3), 9.0, device="cuda")
    tg = torch.full((N, T), 9.0, device="cuda")
    g.backward((0, 0, 0), dev(coords), dev(tv), dev(radii), dev(diff), ag, tg)
    grad_close(ag.cpu().numpy(), wag, "atom gradients")
    grad_close(tg.cpu().numpy(), wtg, "type gradients")


def test_empty_and_ragged_inputs(port):
    """No atoms, no examples, examples of a ragged batch without atoms, atoms far outside the grid:
    the forward still clears its output, the backward still writes every gradient row."""
    g, og = gm_pair(port, resolution=0.5, dimension=11.5)
    T = 5
    dims = g.grid_dimensions(T)
    none = torch.zeros((0, 3), device="cuda")
    out = torch.full(dims, 7.0, device="cuda")
    g.forward((0, 0, 0), none, torch.zeros((0,), device="cuda"), torch.zeros((0,), device="cuda"), out)
    assert not out.any()
    ag = torch.full((0, 3), 7.0, device="cuda")
    g.backward((0, 0, 0), none, torch.zeros((0,), device="cuda"), torch.zeros((0,), device="cuda"),
               torch.ones(dims, device="cuda"), ag)
    # a batch of no examples
    outb = torch.empty((0,) + dims, device="cuda")
    g.forward(torch.zeros((0, 3), device="cuda"), torch.zeros((0, 4, 3), device="cuda"),
              torch.zeros((0, 4), device="cuda"), torch.zeros((0, 4), device="cuda"), outb)
    # ragged: example 1 has no atoms, example 2 only atoms far outside the grid
    coords, types, radii = cases.index_case(9, 30, T, 5.0)
    B, N = 3, 30
    cb = np.zeros((B, N, 3), np.float32); tb = np.zeros((B, N), np.float32); rb = np.ones((B, N), np.float32)
    cb[0], tb[0], rb[0] = coords, types, radii
    cb[2] = coords + 100.0
    tb[2], rb[2] = types, radii
    ns = torch.tensor([N, 0, N], dtype=torch.int32)
    outb = torch.full((B,) + dims, 7.0, device="cuda")
    cen = torch.zeros((B, 3), device="cuda")
    g.forward(cen, dev(cb), dev(tb), dev(rb), outb, n_atoms=ns)
    want = port.forward_index(og, (0, 0, 0), coords, types, radii, T)
    assert np.allclose(outb[0].cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    assert not outb[1].any() and not outb[2].any()
    agb = torch.full((B, N, 3), 7.0, device="cuda")
    diff = np.random.default_rng(2).normal(size=(B,) + dims).astype(np.float32)
    g.backward(cen, dev(cb), dev(tb), dev(rb), dev(diff), agb, n_atoms=ns)
    grad_close(agb[0].cpu().numpy(), port.backward_index(og, (0, 0, 0), coords, types, radii, diff[0]), "example 0")
    assert not agb[1].any() and not agb[2].any()


def test_extreme_shapes(port):
    """One channel, a grid of a single point, vector types without atoms, and one example with
    far more atoms than a launch dimension or a column buffer holds."""
    import libmolgrid_b200 as lmg
    # a single grid point (dimension 0): every atom either covers it or not
    g, og = gm_pair(port, resolution=0.5, dimension=0.0)
    assert g.grid_dimensions(1) == (1, 1, 1, 1)
    coords = np.array([[0.2, 0, 0], [3.0, 0, 0], [0, -0.4, 0.3]], np.float32)
    types = np.zeros(3, np.float32)
    radii = np.array([1.0, 1.0, 2.0], np.float32)
    out = torch.full((1, 1, 1, 1), 7.0, device="cuda")
    g.forward((0, 0, 0), dev(coords), dev(types), dev(radii), out)
    want = port.forward_index(og, (0, 0, 0), coords, types, radii, 1)
    assert np.allclose(out.cpu().numpy(), want, **DENS) and want[0, 0, 0, 0] > 0
    ag = torch.full((3, 3), 7.0, device="cuda")
    diff = np.ones((1, 1, 1, 1), np.float32)
    g.backward((0, 0, 0), dev(coords), dev(types), dev(radii), dev(diff), ag)
    grad_close(ag.cpu().numpy(), port.backward_index(og, (0, 0, 0), coords, types, radii, diff), "single point")
    # vector types, no atoms
    g, og = gm_pair(port, resolution=0.5, dimension=5.5)
    T = 3
    out = torch.full(g.grid_dimensions(T), 7.0, device="cuda")
    g.forward((0, 0, 0), torch.zeros((0, 3), device="cuda"), torch.zeros((0, T), device="cuda"),
              torch.zeros((0,), device="cuda"), out)
    assert not out.any()
    # 70000 atoms in one example (more than 65535), two channels
    rng = np.random.default_rng(12)
    n = 70000
    coords = rng.uniform(-3.5, 3.5, (n, 3)).astype(np.float32)
    types = rng.integers(0, 2, n).astype(np.float32)
    radii = rng.uniform(0.8, 1.4, n).astype(np.float32)
    out = torch.empty(g.grid_dimensions(2), device="cuda")
    g.forward((0, 0, 0), dev(coords), dev(types), dev(radii), out)
    want = port.forward_index(og, (0, 0, 0), coords, types, radii, 2)
    # thousands of terms per voxel in arbitrary order: the bound is relative to the voxel's value
    assert np.allclose(out.cpu().numpy(), want, rtol=2e-5, atol=1e-6)
    diff = rng.normal(size=g.grid_dimensions(2)).astype(np.float32)
    ag = torch.empty((n, 3), device="cuda")
    g.backward((0, 0, 0), dev(coords), dev(types), dev(radii), dev(diff), ag)
    grad_close(ag.cpu().numpy(), port.backward_index(og, (0, 0, 0), coords, types, radii, diff), "70000 atoms")
