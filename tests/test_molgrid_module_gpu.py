"""``import molgrid``: the reference's usage patterns running on the compiled module's classes
(C++ host layer), with the real-molecule known answers of test/test_gridmaker.py:72-103 and the
autograd bindings on top of the compiled GridMaker."""
import numpy as np
import pytest
import torch

from tests.golden.make_golden import molecule_diff
from tests.test_coord_cache import MOL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def molgrid():
    import molgrid
    return molgrid


def golden_example(molgrid):
    ex = molgrid.Example()
    ex.coord_sets.append(molgrid.CoordinateSet(MOL["rec_coords"], MOL["rec_types"], MOL["rec_radii"], 14))
    ex.coord_sets.append(molgrid.CoordinateSet(MOL["lig_coords"], MOL["lig_types"], MOL["lig_radii"], 14))
    ex.labels = [float(v) for v in MOL["labels"]]
    return ex


def test_classes_come_from_the_compiled_module(molgrid):
    for name in ("GridInterpolater", "Transform", "Quaternion", "float3", "CoordinateSet", "Example", "ExampleVec",
                 "Grid4f", "Grid4fCUDA", "MGrid4f", "MGrid5f"):
        assert getattr(molgrid, name).__module__.endswith("molgrid_native"), name
    assert issubclass(molgrid.GridMaker, molgrid.native.GridMaker)
    assert molgrid.Coords2Grid is not None and molgrid.ExampleProvider is not None


def test_molecule_known_answers_through_the_compiled_classes(molgrid):
    ex = golden_example(molgrid)
    c = ex.coord_sets[1]
    gmaker = molgrid.GridMaker()
    dims = gmaker.grid_dimensions(c.max_type)
    center = tuple(c.center())
    mgridgpu = molgrid.MGrid4f(*dims)
    npout = np.zeros(dims, dtype=np.float32)
    cudaout = torch.zeros(dims, dtype=torch.float32, device="cuda")
    gmaker.forward(center, c, mgridgpu.gpu())
    gmaker.forward(center, c, npout)
    gmaker.forward(center, c, cudaout)
    newt = gmaker.make_tensor(center, c)
    assert newt.is_cuda
    for got in (mgridgpu.tonumpy(), npout, cudaout.cpu().numpy(), newt.cpu().numpy(), gmaker.make_ndarray(center, c)):
        assert float(got.max()) == pytest.approx(1.438691, abs=2e-6)
    dims = gmaker.grid_dimensions(ex.num_types())
    mg = molgrid.MGrid4f(*dims)
    gmaker.forward(ex, molgrid.Transform(center, 0, False), mg.gpu())
    g = mg.tonumpy()
    assert float(g.max()) == pytest.approx(2.094017, abs=2e-6)
    want = MOL["ex_sample"]
    got = g.reshape(-1)[MOL["sample"]]
    assert np.all(np.abs(got - want) <= 1e-6 + 1e-5 * np.abs(want))
    mg2 = molgrid.MGrid4f(*dims)
    gmaker.forward(ex, mg2)                        # default centre = the last set's centre
    np.testing.assert_allclose(mg2.tonumpy(), g, rtol=1e-6, atol=1e-7)
    batch = torch.zeros((2,) + dims, device="cuda")
    gmaker.forward(molgrid.ExampleVec([ex, ex]), batch, 0.0, random_rotation=False)
    np.testing.assert_allclose(batch[1].cpu().numpy(), g, rtol=1e-6, atol=1e-7)

    m = ex.merge_coordinates()
    diff = torch.from_numpy(molecule_diff(gmaker.grid_dimensions(28))).cuda()
    grad = molgrid.MGrid2f(m.size(), 3)
    gmaker.backward(tuple(MOL["center"]), m, diff, grad.gpu())
    got, want = grad.tonumpy(), MOL["backward"]
    assert np.all(np.abs(got - want) <= 1e-5 + 1e-4 * np.abs(want))


def test_autograd_on_the_compiled_gridmaker(molgrid):
    """Coords2Grid over molgrid.GridMaker: the values and gradients of the Python layer's own."""
    import libmolgrid_b200 as layer
    rng = np.random.default_rng(4)
    B, N, T = 2, 30, 4
    coords = torch.tensor(rng.uniform(-4, 4, (B, N, 3)), dtype=torch.float32, device="cuda")
    types = torch.tensor(rng.dirichlet(np.ones(T), (B, N)), dtype=torch.float32, device="cuda")
    radii = torch.tensor(rng.uniform(1, 2, (B, N)), dtype=torch.float32, device="cuda")
    results = []
    for mod in (molgrid, layer):
        gm = mod.GridMaker(resolution=0.5, dimension=11.5)
        c = coords.clone().requires_grad_(True)
        t = types.clone().requires_grad_(True)
        out = mod.Coords2Grid(gm, center=(0, 0, 0))(c, t, radii)
        w = torch.linspace(0, 1, out.numel(), device="cuda").view(out.shape)
        (out * w).sum().backward()
        results.append((out.detach(), c.grad, t.grad))
        single = mod.Coords2Grid(gm, center=(0, 0, 0))(coords[0], types[0], radii[0])
        assert torch.allclose(single, out[0].detach(), rtol=1e-5, atol=1e-6)
    for a, b in zip(*results):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
    assert float(results[0][1].abs().max()) > 0


@pytest.mark.parametrize("vector", [False, True])
def test_resident_batches_take_the_compiled_route(molgrid, vector):
    """Batched CUDA tensors with per-example transforms and ragged atom counts: the compiled GridMaker
    serves them (forward and the batched backward), with the results of the Python layer's calls."""
    import libmolgrid_b200 as lmg
    from libmolgrid_b200 import synthetic as cases
    B, T = 3, 6
    coords, types, radii, ns, tr = cases.blob_batch(77, B, 200, 300, T)
    if vector:
        tv = np.zeros(types.shape + (T,), np.float32)
        np.put_along_axis(tv, types.astype(np.int64)[..., None], 0.75, axis=2)
        tv[..., 0] += 0.25
        types = tv
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    dc, dt, dr, dtr, dn = d(coords), d(types), d(radii), d(tr), d(ns)
    cen = torch.zeros((B, 3), device="cuda")
    gm, gp = molgrid.GridMaker(0.5, 11.5), lmg.GridMaker(0.5, 11.5)
    assert gm._resident_batch((cen, dc, dt, dr, None), dict(transforms=dtr, n_atoms=dn)) is False  # None is no tensor
    a = torch.full((B,) + gm.grid_dimensions(T), 3.0, device="cuda")
    b = torch.full_like(a, 4.0)
    assert gm._resident_batch((cen, dc, dt, dr, a), dict(transforms=dtr, n_atoms=dn))
    gm.forward(cen, dc, dt, dr, a, transforms=dtr, n_atoms=dn)
    gp.forward(cen, dc, dt, dr, b, transforms=dtr, n_atoms=dn)
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-6) and float(a.sum()) > 0
    diff = torch.randn_like(a)
    N = coords.shape[1]
    ag, ag2 = torch.full((B, N, 3), 9.0, device="cuda"), torch.full((B, N, 3), 8.0, device="cuda")
    if vector:
        tg, tg2 = torch.full((B, N, T), 9.0, device="cuda"), torch.full((B, N, T), 8.0, device="cuda")
        gm.backward(cen, dc, dt, dr, diff, ag, tg, transforms=dtr, n_atoms=dn)
        gp.backward(cen, dc, dt, dr, diff, ag2, tg2, transforms=dtr, n_atoms=dn)
        assert torch.equal(tg, tg2)
    else:
        gm.backward(cen, dc, dt, dr, diff, ag, transforms=dtr, n_atoms=dn)
        gp.backward(cen, dc, dt, dr, diff, ag2, transforms=dtr, n_atoms=dn)
    assert torch.equal(ag, ag2)            # the backward kernels sum in a fixed order
    with pytest.raises((TypeError, ValueError)):
        molgrid.native.GridMaker.forward(gm, cen, dc, dt, dr, a, transforms=dtr[:, :9].contiguous())


def test_provider_settings_feed_the_compiled_gridmaker(molgrid, tmp_path):
    """A shuffled, balanced provider with vector types and a data set with random access: their
    compiled Examples grid through the compiled GridMaker like the Python layer's do through its own."""
    import libmolgrid_b200 as lmg
    from libmolgrid_b200 import coord_cache
    rng = np.random.default_rng(9)
    lines = []
    for i in range(8):
        coord_cache.write_gninatypes(tmp_path / ("r%d.gninatypes" % i), rng.normal(size=(60, 3)) * 5, rng.integers(2, 14, 60))
        coord_cache.write_gninatypes(tmp_path / ("l%d.gninatypes" % i), rng.normal(size=(9, 3)) * 2, rng.integers(2, 14, 9))
        lines.append("%d %.2f r%d.gninatypes l%d.gninatypes" % (i % 2, i * 0.5, i, i))
    (tmp_path / "s.types").write_text("\n".join(lines) + "\n")
    kw = dict(data_root=str(tmp_path), shuffle=True, balanced=True, seed=5, default_batch_size=4)
    pn, pp = molgrid.ExampleProvider(**kw), lmg.ExampleProvider(**kw)
    for p in (pn, pp):
        p.populate(str(tmp_path / "s.types"))
    gn, gp = molgrid.GridMaker(0.5, 11.5), lmg.GridMaker(0.5, 11.5)
    bn, bp = pn.next_batch(), pp.next_batch()
    assert type(bn).__module__.endswith("molgrid_native") and [x.labels[0] for x in bn] == [1.0, 0.0, 1.0, 0.0]
    a = torch.zeros((4,) + gn.grid_dimensions(pn.num_types()), device="cuda")
    b = torch.zeros_like(a)
    gn.forward(bn, a, 0.0, False)
    gp.forward(bp, b, 0.0, False)
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-6) and float(a.max()) > 0
    ds = molgrid.ExampleDataset(data_root=str(tmp_path))
    ds.populate(str(tmp_path / "s.types"))
    ex = ds[3]
    one = torch.zeros(gn.grid_dimensions(ex.num_types()), device="cuda")
    gn.forward(ex, one)
    assert len(ds) == 8 and float(one.max()) > 0 and type(ex).__module__.endswith("molgrid_native")
