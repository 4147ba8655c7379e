"""GPU parity at the shapes of the benchmark configurations, plus two safety nets.

* the vector-typed configuration (28 channels, 96^3 points at 0.25 A, radii indexed by type, dense
  Dirichlet type vectors) on a sub-sample of atoms the CPU checker finishes in seconds: forward,
  backward (atom and type gradients) and backward_gradients;
* backward_relevance on an example of the blob batch, where dozens of atoms overlap per voxel;
* one rotated 28x48^3 -> 28x48^3 interpolation against the checker directly;
* guard words around every output buffer of every pass (nothing may be written outside the output),
  also with buffers that are not 16-byte aligned;
* every pass that claims a fixed summation order gives bit-identical results when run twice.

Tolerances as everywhere: binary grids bit-exact, densities rel 1e-5 / abs 1e-6, gradients,
relevance and interpolated grids rel 1e-4 (abs floor 1e-5 x scale).
"""
import numpy as np
import pytest
import torch

from tests import cases
from tests.test_gridmaker_gpu import DENS, dev, gm_pair, grad_close

pytestmark = pytest.mark.gpu

T28 = 28


# ---- the vector-typed configuration at its own shape -------------------------------------------

@pytest.fixture(scope="module")
def c3(port):
    import libmolgrid_b200 as lmg  # noqa: F401
    g, og = gm_pair(port, resolution=0.25, dimension=23.75, radius_type_indexed=True)
    assert g.grid_dimensions(T28) == (28, 96, 96, 96)
    n = 40
    coords, tv, radii = cases.dense_vector_batch(1003, 1, n, T28)
    coords, tv, radii = coords[0], tv[0], radii[0]
    # a few atoms near a face of the box (clipped footprints) and one exactly on a grid point
    coords[0] = (11.6, 0.3, -0.2)
    coords[1] = (-11.8, -11.7, 11.9)
    coords[2] = (0.125, -0.125, 0.375)
    assert (tv == 0).sum() >= 0 and tv.shape == (n, T28)
    diff = np.random.default_rng(1003).normal(size=g.grid_dimensions(T28)).astype(np.float32)
    return g, og, coords, tv, radii, diff


def test_c3_forward(port, c3):
    g, og, coords, tv, radii, diff = c3
    want = port.forward_vector(og, (0, 0, 0), coords, tv, radii)
    out = torch.full(g.grid_dimensions(T28), -3.0, device="cuda")
    g.forward((0, 0, 0), dev(coords), dev(tv), dev(radii), out)
    got = out.cpu().numpy()
    assert np.allclose(got, want, **DENS), np.abs(got - want).max()
    assert want.max() > 0.1


def test_c3_backward_and_backward_gradients(port, c3):
    g, og, coords, tv, radii, diff = c3
    n = coords.shape[0]
    wag, wtg = port.backward_vector(og, (0, 0, 0), coords, tv, radii, diff)
    ag = torch.full((n, 3), 9.0, device="cuda")
    tg = torch.full((n, T28), 9.0, device="cuda")
    g.backward((0, 0, 0), dev(coords), dev(tv), dev(radii), dev(diff), ag, tg)
    grad_close(ag.cpu().numpy(), wag, "atom gradients")
    grad_close(tg.cpu().numpy(), wtg, "type gradients")

    # the second-order pass fed with the first-order results, as the configuration states
    wdd, wadd, wtdd = port.backward_gradients(og, (0, 0, 0), coords, tv, radii, diff, wag, wtg)
    dd = torch.full(g.grid_dimensions(T28), 5.0, device="cuda")
    add = torch.full((n, 3), 5.0, device="cuda")
    tdd = torch.full((n, T28), 5.0, device="cuda")
    g.backward_gradients((0, 0, 0), dev(coords), dev(tv), dev(radii), dev(diff), dev(wag), dev(wtg),
                         dd, add, tdd)
    grad_close(dd.cpu().numpy(), wdd, "diffdiff")
    grad_close(add.cpu().numpy(), wadd, "atom_diffdiff")
    assert not tdd.any() and not wtdd.any()


# ---- relevance where atoms overlap heavily -------------------------------------------------------

def test_relevance_on_a_blob_example(port):
    g, og = gm_pair(port)
    coords, types, radii, ns, tr = cases.blob_batch(1001, 1, 2000, 4000, T28)
    n = int(ns[0])
    moved = port.transform_forward(tr[0], coords[0, :n])
    dens = port.forward_index(og, (0, 0, 0), moved, types[0, :n], radii[0, :n], T28)
    assert dens.max() > 3.0          # the blob stacks many atoms on one voxel
    diff = np.random.default_rng(1002).normal(size=dens.shape).astype(np.float32)
    want = port.backward_relevance(og, (0, 0, 0), moved, types[0, :n], radii[0, :n], dens, diff)
    rel = torch.full((1, coords.shape[1]), 9.0, device="cuda")
    g.backward_relevance(dev(np.zeros((1, 3), np.float32)), dev(coords), dev(types), dev(radii),
                         dev(dens[None]), dev(diff[None]), rel, transforms=dev(tr),
                         n_atoms=torch.from_numpy(ns))
    grad_close(rel.cpu().numpy()[0, :n], want, "relevance")


# ---- interpolation at the benchmark's shape, against the checker directly ------------------------

def test_interpolate_28x48_rotated_against_oracle(port):
    import libmolgrid_b200 as lmg
    rng = np.random.default_rng(1005)
    grid = rng.uniform(0, 1, (T28, 48, 48, 48)).astype(np.float32)
    q = cases.random_quaternion(rng, 1)[0]
    tr = port.tr(q, (0, 0, 0), rng.uniform(-2, 2, 3))
    want = port.interpolate([0.5, 23.5, 0.5, 23.5], (0, 0, 0), grid, tr, (0, 0, 0))
    gi = lmg.GridInterpolater(0.5, 23.5, 0.5, 23.5)
    t = lmg.Transform(lmg.Quaternion(*q), (0, 0, 0), tuple(tr[7:10]))
    for tiled in (1, 0):
        from libmolgrid_b200 import _cabi
        _cabi.lib().lmg_set_interp_tiled(tiled)
        try:
            out = torch.full((T28, 48, 48, 48), -1.0, device="cuda")
            gi.forward((0, 0, 0), dev(grid), t, (0, 0, 0), out)
        finally:
            _cabi.lib().lmg_set_interp_tiled(1)
        got = out.cpu().numpy()
        assert np.array_equal(got, want), np.abs(got - want).max()
    assert _cabi.lib().lmg_tma_timeouts() == 0


@pytest.mark.parametrize("axis_angle", [((1.0, 0.0, 0.0), 0.0), ((0.0, 0.0, 1.0), 90.0), ((0.0, 0.0, 1.0), 45.0),
                                        ((1.0, -1.0, 0.0), 54.735610317245346), ((1.0, 1.0, 1.0), 60.0)])
def test_interpolate_48_cubed_special_rotations(port, axis_angle):
    """Rotations at the ends of the staged boxes' range: none (the smallest box), quarter turns (integer
    voxel positions: floor == ceil), 45 degrees, and the turn that puts a tile's diagonal along an
    axis (the largest box, a single staging slot); partly outside the input through the translation."""
    import libmolgrid_b200 as lmg
    from libmolgrid_b200 import _cabi
    (ax, ay, az), deg = axis_angle
    n = float(np.sqrt(ax * ax + ay * ay + az * az))
    h = np.deg2rad(deg) / 2
    q = (float(np.cos(h)), float(np.sin(h) * ax / n), float(np.sin(h) * ay / n), float(np.sin(h) * az / n))
    rng = np.random.default_rng(77)
    grid = rng.uniform(-1, 1, (3, 48, 48, 48)).astype(np.float32)
    tr = port.tr(q, (0, 0, 0), (1.5, -0.5, 3.0))
    want = port.interpolate([0.5, 23.5, 0.5, 23.5], (0, 0, 0), grid, tr, (0, 0, 0))
    gi = lmg.GridInterpolater(0.5, 23.5, 0.5, 23.5)
    t = lmg.Transform(lmg.Quaternion(*q), (0, 0, 0), (1.5, -0.5, 3.0))
    out = torch.full((3, 48, 48, 48), -1.0, device="cuda")
    gi.forward((0, 0, 0), dev(grid), t, (0, 0, 0), out)
    got = out.cpu().numpy()
    assert np.array_equal(got, want), np.abs(got - want).max()
    assert _cabi.lib().lmg_tma_timeouts() == 0


# ---- guard words around the outputs -----------------------------------------------------------------

GUARD = 0x7fc0dead  # a NaN payload no kernel produces


class Guarded:
    """A CUDA float buffer with `pad` guard words on either side of the part handed to the library.
    `shift` extra floats move the output off a 16-byte boundary (the kernels' unaligned paths)."""

    def __init__(self, shape, pad=64, shift=0):
        n = int(np.prod(shape))
        self.raw = torch.full((pad + shift + n + pad,), 0, dtype=torch.int32, device="cuda")
        self.raw.fill_(GUARD)
        self.lo, self.hi = pad + shift, pad + shift + n
        self.out = self.raw.view(torch.float32)[self.lo:self.hi].view(shape)
        assert self.out.data_ptr() % 16 == (4 * shift) % 16

    def check(self, what):
        r = self.raw.cpu().numpy()
        assert (r[:self.lo] == GUARD).all(), what + ": written before the output"
        assert (r[self.hi:] == GUARD).all(), what + ": written past the output"
        return self.out


@pytest.mark.parametrize("shift", [0, 1])
@pytest.mark.parametrize("binary", [False, True])
def test_guard_words_index_passes(port, binary, shift):
    g, og = gm_pair(port, resolution=0.5, dimension=11.5, binary=binary)
    T, B = 5, 2
    data = [cases.index_case(40 + b, 150, T, 7.0) for b in range(B)]
    coords, types, radii = (np.stack([x[i] for x in data]) for i in range(3))
    dims = g.grid_dimensions(T)
    centers = np.zeros((B, 3), np.float32)
    out = Guarded((B,) + dims, shift=shift)
    g.forward(dev(centers), dev(coords), dev(types), dev(radii), out.out)
    grid = out.check("forward").cpu().numpy()
    diffh = np.random.default_rng(3).normal(size=(B,) + dims).astype(np.float32)
    diff = Guarded((B,) + dims, shift=shift)          # inputs are moved off alignment as well
    diff.out.copy_(dev(diffh))
    ag = Guarded((B, 150, 3), shift=shift)
    g.backward(dev(centers), dev(coords), dev(types), dev(radii), diff.out, ag.out)
    got = ag.check("backward").cpu().numpy()
    rel = Guarded((B, 150), shift=shift)
    # the relevance divides by the density: both sides get the checker's grid, bit for bit
    wants = np.stack([port.forward_index(og, (0, 0, 0), coords[b], types[b], radii[b], T) for b in range(B)])
    dens = Guarded((B,) + dims, shift=shift)
    dens.out.copy_(dev(wants))
    g.backward_relevance(dev(centers), dev(coords), dev(types), dev(radii), dens.out, diff.out, rel.out)
    gotr = rel.check("relevance").cpu().numpy()
    diff.check("diff (input)")
    dens.check("density (input)")
    for b in range(B):
        want = wants[b]
        if binary:
            assert np.array_equal(grid[b], want)
        else:
            assert np.allclose(grid[b], want, **DENS)
        grad_close(got[b], port.backward_index(og, (0, 0, 0), coords[b], types[b], radii[b], diffh[b]),
                   "atom gradients")
        grad_close(gotr[b], port.backward_relevance(og, (0, 0, 0), coords[b], types[b], radii[b], want,
                                                    diffh[b]), "relevance")


@pytest.mark.parametrize("shift", [0, 1])
@pytest.mark.parametrize("rti", [False, True])
def test_guard_words_vector_passes(port, rti, shift):
    g, og = gm_pair(port, resolution=0.5, dimension=11.5, radius_type_indexed=rti)
    T, N = 6, 60
    coords, tv, radii = cases.vector_case(77, N, T, 7.0, rti=rti)
    dims = g.grid_dimensions(T)
    out = Guarded(dims, shift=shift)
    g.forward((0, 0, 0), dev(coords), dev(tv), dev(radii), out.out)
    grid = out.check("forward").cpu().numpy()
    assert np.allclose(grid, port.forward_vector(og, (0, 0, 0), coords, tv, radii), **DENS)
    rng = np.random.default_rng(4)
    diffh = rng.normal(size=dims).astype(np.float32)
    diff = Guarded(dims, shift=shift)
    diff.out.copy_(dev(diffh))
    ag, tg = Guarded((N, 3), shift=shift), Guarded((N, T), shift=shift)
    g.backward((0, 0, 0), dev(coords), dev(tv), dev(radii), diff.out, ag.out, tg.out)
    wag, wtg = port.backward_vector(og, (0, 0, 0), coords, tv, radii, diffh)
    grad_close(ag.check("atom gradients").cpu().numpy(), wag, "atom gradients")
    grad_close(tg.check("type gradients").cpu().numpy(), wtg, "type gradients")
    agi, tgi = rng.normal(size=(N, 3)).astype(np.float32), rng.normal(size=(N, T)).astype(np.float32)
    dd, add, tdd = Guarded(dims, shift=shift), Guarded((N, 3), shift=shift), Guarded((N, T), shift=shift)
    g.backward_gradients((0, 0, 0), dev(coords), dev(tv), dev(radii), diff.out, dev(agi), dev(tgi),
                         dd.out, add.out, tdd.out)
    wdd, wadd, _ = port.backward_gradients(og, (0, 0, 0), coords, tv, radii, diffh, agi, tgi)
    grad_close(dd.check("diffdiff").cpu().numpy(), wdd, "diffdiff")
    grad_close(add.check("atom_diffdiff").cpu().numpy(), wadd, "atom_diffdiff")
    assert not tdd.check("type_diffdiff").any()


def test_guard_words_transform_and_interpolation(port):
    import libmolgrid_b200 as lmg
    rng = np.random.default_rng(9)
    q = cases.random_quaternion(rng, 1)[0]
    t = lmg.Transform(lmg.Quaternion(*q), (0.5, 0, -0.5), (1.0, -1.0, 0.25))
    tr = port.tr(q, (0.5, 0, -0.5), (1.0, -1.0, 0.25))
    pts = rng.normal(size=(1001, 3)).astype(np.float32)
    fo, bo = Guarded((1001, 3)), Guarded((1001, 3))
    t.forward(dev(pts), fo.out)
    t.backward(dev(pts), bo.out)
    assert np.array_equal(fo.check("transform forward").cpu().numpy(), port.transform_forward(tr, pts))
    assert np.array_equal(bo.check("transform backward").cpu().numpy(), port.transform_backward(tr, pts))
    grid = rng.uniform(0, 1, (3, 24, 24, 24)).astype(np.float32)
    gi = lmg.GridInterpolater(0.5, 11.5, 0.5, 11.5)
    out = Guarded((3, 24, 24, 24))
    gi.forward((0, 0, 0), dev(grid), t, (0, 0, 0), out.out)
    want = port.interpolate([0.5, 11.5, 0.5, 11.5], (0, 0, 0), grid, tr, (0, 0, 0))
    assert np.array_equal(out.check("interpolate").cpu().numpy(), want)


# ---- run twice, compare bits ----------------------------------------------------------------------

def test_backward_passes_are_bitwise_reproducible(port):
    """The backward passes sum each atom's footprint in a fixed order (no atomics): two runs on
    the same inputs agree bit for bit.  The forward pass adds atoms into voxels in no fixed order;
    its run-to-run spread on the dense blob is bounded separately below."""
    g, og = gm_pair(port)
    B = 2
    coords, types, radii, ns, tr = cases.blob_batch(1002, B, 2000, 2500, T28)
    N = coords.shape[1]
    dims = (B,) + g.grid_dimensions(T28)
    diff = torch.randn(dims, device="cuda", generator=torch.Generator("cuda").manual_seed(5))
    dens = torch.empty(dims, device="cuda")
    cen = dev(np.zeros((B, 3), np.float32))
    args = (cen, dev(coords), dev(types), dev(radii))
    kw = dict(transforms=dev(tr), n_atoms=torch.from_numpy(ns))
    g.forward(*args, dens, **kw)
    runs = []
    for _ in range(2):
        ag = torch.empty((B, N, 3), device="cuda")
        rel = torch.empty((B, N), device="cuda")
        g.backward(*args, diff, ag, **kw)
        g.backward_relevance(*args, dens, diff, rel, **kw)
        runs.append((ag, rel))
    assert torch.equal(runs[0][0], runs[1][0])
    assert torch.equal(runs[0][1], runs[1][1])

    for rti in (False, True):
        gv, _ = gm_pair(port, resolution=0.5, dimension=11.5, radius_type_indexed=rti)
        T, n = 6, 300
        c, tv, r = cases.vector_case(31, n, T, 7.0, rti=rti)
        d = torch.randn(gv.grid_dimensions(T), device="cuda", generator=torch.Generator("cuda").manual_seed(6))
        agi = torch.randn((n, 3), device="cuda", generator=torch.Generator("cuda").manual_seed(7))
        tgi = torch.randn((n, T), device="cuda", generator=torch.Generator("cuda").manual_seed(8))
        runs = []
        for _ in range(2):
            ag, tg = torch.empty((n, 3), device="cuda"), torch.empty((n, T), device="cuda")
            gv.backward((0, 0, 0), dev(c), dev(tv), dev(r), d, ag, tg)
            dd = torch.empty(gv.grid_dimensions(T), device="cuda")
            add, tdd = torch.empty((n, 3), device="cuda"), torch.empty((n, T), device="cuda")
            gv.backward_gradients((0, 0, 0), dev(c), dev(tv), dev(r), d, agi, tgi, dd, add, tdd)
            runs.append((ag, tg, add))
        for x, y in zip(*runs):
            assert torch.equal(x, y)


def test_forward_spread_between_runs_on_the_dense_blob(port):
    """Voxels of the blob receive dozens of terms whose order of addition is not fixed: two runs may
    differ in the last bits, and by far less than the density tolerance."""
    g, og = gm_pair(port)
    coords, types, radii, ns, tr = cases.blob_batch(1001, 1, 3500, 4000, T28)
    args = (dev(np.zeros((1, 3), np.float32)), dev(coords), dev(types), dev(radii))
    kw = dict(transforms=dev(tr), n_atoms=torch.from_numpy(ns))
    a = torch.empty((1,) + g.grid_dimensions(T28), device="cuda")
    b = torch.empty_like(a)
    g.forward(*args, a, **kw)
    g.forward(*args, b, **kw)
    assert float(a.max()) > 3.0
    assert torch.equal(a != 0, b != 0)
    err = (a - b).abs()
    assert float((err / (1e-6 + 1e-5 * a.abs())).max()) < 0.1
    g.set_binary(True)
    g.forward(*args, a, **kw)
    g.forward(*args, b, **kw)
    assert torch.equal(a, b)
