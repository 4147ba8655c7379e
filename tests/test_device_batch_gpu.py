"""Batch assembly on the device (lmg_decode_records) against the host-side path: the same atoms, the
same grid centres bit for bit, the same grids and gradients."""
import numpy as np
import pytest
import torch

import libmolgrid_b200 as molgrid
from libmolgrid_b200 import coord_cache

pytestmark = pytest.mark.gpu


@pytest.fixture()
def provider_dir(tmp_path):
    rng = np.random.default_rng(31)
    lines = []
    for i in range(7):
        nrec, nlig = int(rng.integers(150, 400)), int(rng.integers(5, 40))
        for name, n, spread in (("r%d.gninatypes" % i, nrec, 9.0), ("l%d.gninatypes" % i, nlig, 2.5)):
            coords = rng.normal(size=(n, 3)) * spread + (3.0, -2.0, 1.0)
            types = rng.integers(0, 30, n)     # includes hydrogens (dropped) and out-of-table numbers
            coord_cache.write_gninatypes(tmp_path / name, coords, types)
        lines.append("%d %.3f r%d.gninatypes l%d.gninatypes" % (i % 2, rng.normal(), i, i))
    # an example whose ligand has no mapped atom at all, and one with an empty ("none") ligand
    coord_cache.write_gninatypes(tmp_path / "h.gninatypes", rng.normal(size=(4, 3)), [0, 1, 0, 1])
    lines.append("0 0.5 r0.gninatypes h.gninatypes")
    lines.append("1 1.5 r1.gninatypes none")
    (tmp_path / "list.types").write_text("\n".join(lines) + "\n")
    return tmp_path


def providers(d):
    out = []
    for _ in range(2):
        p = coord_cache.ExampleProvider(data_root=str(d))
        p.populate(str(d / "list.types"))
        out.append(p)
    return out


def test_device_batch_matches_host_examples(provider_dir):
    pa, pb = providers(provider_dir)
    B = 9
    exs = pa.next_batch(B)
    batch = pb.next_device_batch(B)
    torch.cuda.synchronize()
    assert len(batch) == B and batch.num_types() == 28 and pb.pos == pa.pos
    labels = np.zeros((B, 2), np.float32)
    exs.extract_labels(labels)
    np.testing.assert_array_equal(batch.labels.cpu().numpy(), labels)
    coords, types, radii = (x.cpu().numpy() for x in (batch.coords, batch.type_index, batch.radii))
    ns = batch.n_atoms.cpu().numpy()
    for b, ex in enumerate(exs):
        m = ex.merge_coordinates()
        keep = types[b, :ns[b]] >= 0
        assert keep.sum() == m.size()
        np.testing.assert_array_equal(coords[b, :ns[b]][keep], m.coords.tonumpy())
        np.testing.assert_array_equal(types[b, :ns[b]][keep], m.type_index.tonumpy())
        np.testing.assert_array_equal(radii[b, :ns[b]][keep], m.radii.tonumpy())
        assert np.all(radii[b, :ns[b]][~keep] == 0)
        want = np.array(tuple(molgrid.GridMaker._default_center(ex)), np.float32)
        np.testing.assert_array_equal(batch.centers[b].cpu().numpy(), want)   # bit for bit
    assert np.all(batch.centers[7].cpu().numpy() == 0) and np.all(batch.centers[8].cpu().numpy() == 0)

    gm = molgrid.GridMaker(0.5, 15.5)
    dims = gm.grid_dimensions(28)
    a, c = torch.zeros((B,) + dims, device="cuda"), torch.zeros((B,) + dims, device="cuda")
    molgrid.set_random_seed(5)
    gm.forward(exs, a, random_translation=1.5, random_rotation=True)
    molgrid.set_random_seed(5)
    tr = gm.batch_transforms(batch, 1.5, True)
    gm.forward_arrays(batch.centers, batch.coords, batch.type_index, batch.radii, c, transforms=tr,
                      n_atoms=batch.n_atoms)
    assert float(a.sum()) > 100
    torch.testing.assert_close(a, c, rtol=1e-5, atol=1e-6)
    molgrid.set_random_seed(5)
    gm.forward(batch, c, 1.5, True)          # the overload that draws the transforms itself
    torch.testing.assert_close(a, c, rtol=1e-5, atol=1e-6)

    # backward on the batch equals backward on each merged example with the same transform
    diff = torch.randn((B,) + dims, device="cuda")
    grads = torch.zeros((B, batch.coords.shape[1], 3), device="cuda")
    gm.backward(batch, diff, grads, transforms=tr)
    trs = tr.cpu().numpy()
    for b in (0, 3, 6):
        m = exs[b].merge_coordinates()
        t = molgrid.Transform(molgrid.Quaternion(*trs[b, :4]), tuple(trs[b, 4:7]), tuple(trs[b, 7:]))
        moved = m.clone()
        t.forward(moved, moved)
        one = torch.zeros((m.size(), 3), device="cuda")
        gm.backward(t.get_rotation_center(), moved, diff[b], one)
        keep = (batch.type_index[b, :ns[b]] >= 0)
        got = grads[b, :ns[b]][keep]
        scale = max(1.0, float(one.abs().max()))
        # the batch path differentiates with respect to the transformed position as well
        assert torch.allclose(got, one, rtol=1e-4, atol=1e-5 * scale)
        assert float(grads[b, :ns[b]][~keep].abs().sum()) == 0


def test_empty_first_set_does_not_shift_the_channels(tmp_path):
    """'none lig' and a receptor whose atoms all map to nothing: the ligand keeps channels [0, 14) on
    both paths, as in Example::merge_coordinates (src/example.cpp:84-96), which ignores empty sets."""
    rng = np.random.default_rng(3)
    coord_cache.write_gninatypes(tmp_path / "lig.gninatypes", rng.normal(size=(12, 3)) * 2, rng.integers(2, 20, 12))
    coord_cache.write_gninatypes(tmp_path / "hyd.gninatypes", rng.normal(size=(5, 3)), [0, 1, 0, 1, 0])
    (tmp_path / "l.types").write_text("1 none lig.gninatypes\n0 hyd.gninatypes lig.gninatypes\n")
    pa, pb = (coord_cache.ExampleProvider(data_root=str(tmp_path)) for _ in range(2))
    for p in (pa, pb):
        p.populate(str(tmp_path / "l.types"))
    exs = pa.next_batch(2)
    batch = pb.next_device_batch(2).check()
    types = batch.type_index.cpu().numpy()
    ns = batch.n_atoms.cpu().numpy()
    for b, ex in enumerate(exs):
        m = ex.merge_coordinates()
        keep = types[b, :ns[b]] >= 0
        np.testing.assert_array_equal(types[b, :ns[b]][keep], m.type_index.tonumpy())
        assert m.size() > 0 and types[b, :ns[b]][keep].max() < pa.caches[1].num_types()
    with pytest.raises(ValueError):
        (tmp_path / "bad.types").write_text("1 0.5 none lig.gninatypes\n0 none lig.gninatypes\n")
        pc = coord_cache.ExampleProvider(data_root=str(tmp_path))
        pc.populate(str(tmp_path / "bad.types"))
        pc.next_device_batch(2)


def test_decode_reports_sets_that_do_not_fit(provider_dir):
    from libmolgrid_b200 import _cabi
    import ctypes
    rec = np.zeros(8, dtype=coord_cache.RECORD)
    rec["type"] = 2
    table = (_cabi.RecordSetStruct * 1)(_cabi.RecordSetStruct(0, 8, 0, 0, 0, 0, 1))
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    drec = d(rec.view(np.uint8))
    dtab = d(np.frombuffer(bytes(table), dtype=np.uint8).copy())
    tmap, trad = d(np.arange(28, dtype=np.int32)), d(np.ones(28, np.float32))
    coords, types, radii = (torch.zeros(s, device="cuda") for s in ((1, 4, 3), (1, 4), (1, 4)))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    vp = ctypes.c_void_p
    rc = _cabi.lib().lmg_decode_records(vp(drec.data_ptr()), vp(dtab.data_ptr()), 1, vp(tmap.data_ptr()),
                                        vp(trad.data_ptr()), 1, 4, 8, vp(coords.data_ptr()), vp(types.data_ptr()),
                                        vp(radii.data_ptr()), None, None, vp(status.data_ptr()), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 1 and float(types.sum()) == 8.0   # four atoms written, four refused
    with pytest.raises(ValueError):
        _cabi.check(_cabi.lib().lmg_decode_records(None, None, 1, None, None, 1, 4, 8, None, None, None, None,
                                                   None, None, None))


def test_sum_types_on_the_device_equals_the_host_sums():
    """lmg_sum_types against the host-side sums of the same sets: bit for bit with type vectors
    (same order of addition), exact counts with type indices, accumulation into the output, and the
    out-of-range report."""
    rng = np.random.default_rng(12)
    n, T = 3000, 28
    coords = rng.normal(size=(n, 3)).astype(np.float32)
    radii = np.ones(n, np.float32)
    tv = rng.dirichlet(np.ones(T) * 0.3, n).astype(np.float32)
    cs = molgrid.CoordinateSet(coords, tv, radii)
    start = rng.normal(size=T).astype(np.float32)
    host = start.copy()
    cs.sum_types(host, zerofirst=False)
    dev = torch.from_numpy(start.copy()).cuda()
    cs.sum_types(dev, zerofirst=False)
    np.testing.assert_array_equal(dev.cpu().numpy(), host)
    cs.sum_types(dev)                                   # cleared first
    host0 = np.zeros(T, np.float32)
    cs.sum_types(host0)
    np.testing.assert_array_equal(dev.cpu().numpy(), host0)

    ti = rng.integers(-1, T, n).astype(np.float32)
    ti[:10] += 0.4                                       # rounds down
    ti[10:20] -= 0.4                                     # rounds up; -1.4 stays negative
    ci = molgrid.CoordinateSet(coords, ti, radii, T)
    host = np.zeros(T, np.float32)
    ci.sum_types(host)
    dev = torch.full((T,), 3.0, device="cuda")
    ci.sum_types(dev)
    np.testing.assert_array_equal(dev.cpu().numpy(), host)
    assert host.sum() == (np.round(ti) >= 0).sum()
    ti[5] = T
    bad = molgrid.CoordinateSet(coords, ti, radii, T)
    with pytest.raises(IndexError):
        bad.sum_types(torch.zeros(T, device="cuda"))
    with pytest.raises(IndexError):
        bad.sum_types(np.zeros(T, np.float32))

    # an Example lays its sets side by side
    ex = molgrid.Example()
    ex.coord_sets += [ci, molgrid.CoordinateSet(coords[:50], ti[100:150], radii[:50], T)]
    both = torch.full((2 * T,), -1.0, device="cuda")
    ex.sum_types(both)
    hb = np.zeros(2 * T, np.float32)
    ex.sum_types(hb)
    np.testing.assert_array_equal(both.cpu().numpy(), hb)


def test_prefetched_batches_equal_sequential_batches(provider_dir):
    """device_batches (host assembly on worker threads, several staging buffers in flight) yields
    the batches next_device_batch yields, in the same order."""
    pa, pb = providers(provider_dir)
    got = []
    for batch in pb.device_batches(4, count=7, workers=3):
        got.append([x.clone() for x in (batch.coords, batch.type_index, batch.radii, batch.n_atoms,
                                        batch.centers, batch.labels)])
        batch.check()
    assert len(got) == 7 and pb.pos == (7 * 4) % pb.size()
    for g in got:
        want = pa.next_device_batch(4)
        ns = want.n_atoms.cpu().numpy()
        assert torch.equal(g[3], want.n_atoms) and torch.equal(g[4], want.centers) and torch.equal(g[5], want.labels)
        for b in range(4):
            for x, y in zip(g[:3], (want.coords, want.type_index, want.radii)):
                assert torch.equal(x[b, :ns[b]], y[b, :ns[b]])


@pytest.mark.parametrize("settings", [dict(shuffle=True, balanced=True), dict(stratify_receptor=True, num_copies=2),
                                      dict(duplicate_first=True)])
def test_device_batches_follow_the_order_settings(provider_dir, settings):
    """Shuffled, balanced, stratified or duplicated: the device batch holds the examples next_batch
    hands out for the same settings and seed."""
    ps = []
    for _ in range(2):
        p = coord_cache.ExampleProvider(data_root=str(provider_dir), seed=11, **settings)
        p.populate(str(provider_dir / "list.types"))
        ps.append(p)
    pa, pb = ps
    B = 6
    for _ in range(3):
        exs = pa.next_batch(B)
        batch = pb.next_device_batch(B).check()
        labels = np.zeros((B, 2), np.float32)
        exs.extract_labels(labels)
        np.testing.assert_array_equal(batch.labels.cpu().numpy(), labels)
        types = batch.type_index.cpu().numpy()
        coords = batch.coords.cpu().numpy()
        ns = batch.n_atoms.cpu().numpy()
        for b, ex in enumerate(exs):
            m = ex.merge_coordinates()
            keep = types[b, :ns[b]] >= 0
            np.testing.assert_array_equal(coords[b, :ns[b]][keep], m.coords.tonumpy())
            np.testing.assert_array_equal(types[b, :ns[b]][keep], m.type_index.tonumpy())


def test_vector_typed_examples_grid_like_index_typed_ones(provider_dir):
    """make_vector_types (one-hot vectors, radii by type) grids like the index-typed examples
    (test/test_gridmaker.py:281-340), into CUDA and host tensors alike."""
    ps = []
    for vec in (False, True):
        p = coord_cache.ExampleProvider(data_root=str(provider_dir), make_vector_types=vec)
        p.populate(str(provider_dir / "list.types"))
        ps.append(p)
    g = molgrid.GridMaker(0.5, 23.5)
    gv = molgrid.GridMaker(0.5, 23.5, radius_type_indexed=True)
    for _ in range(3):
        ex, exv = ps[0].next(), ps[1].next()
        assert exv.has_vector_types() and not ex.has_vector_types()
        dims = g.grid_dimensions(ex.num_types())
        a = torch.zeros(dims, device="cuda")
        b = torch.zeros(dims, device="cuda")
        host = torch.zeros(dims)
        g.forward(ex, a)
        gv.forward(exv, b)
        gv.forward(exv, host)
        assert float(a.max()) > 0
        assert torch.allclose(host, b.cpu(), rtol=1e-5, atol=1e-6)
        # channels that group types of different radii (4: the heavier halogens, 13: the metals) get
        # the mean radius of the group as their type radius, so only the other channels must agree
        same = [c for c in range(dims[0]) if c % 14 not in (4, 13)]
        assert torch.allclose(a[same], b[same], rtol=1e-5, atol=1e-6)
        assert not torch.allclose(a[[4, 13]], b[[4, 13]], rtol=1e-5, atol=1e-6)


def test_duplicated_first_set_grids_on_device_and_host(tmp_path):
    """duplicate_first with three files per line: four sets per example, the first one twice; grids
    into CUDA and host tensors agree (test/test_gridmaker.py:342-362)."""
    rng = np.random.default_rng(5)
    for name, n, spread in (("r.gninatypes", 200, 6.0), ("a.gninatypes", 12, 2.0), ("b.gninatypes", 9, 2.0)):
        coord_cache.write_gninatypes(tmp_path / name, rng.normal(size=(n, 3)) * spread, rng.integers(2, 14, n))
    (tmp_path / "dup.types").write_text("1 r.gninatypes a.gninatypes b.gninatypes\n")
    p = coord_cache.ExampleProvider(data_root=str(tmp_path), duplicate_first=True)
    p.populate(str(tmp_path / "dup.types"))
    batch = p.next_batch(1)
    assert len(batch[0].coord_sets) == 4 and p.num_types() == batch[0].num_types()
    g = molgrid.GridMaker(0.5, 23.5)
    shape = (1,) + g.grid_dimensions(p.num_types())
    dev_out, host_out = torch.zeros(shape, device="cuda"), torch.zeros(shape)
    g.forward(batch, dev_out, random_translation=0.0, random_rotation=False)
    g.forward(batch, host_out, random_translation=0.0, random_rotation=False)
    assert torch.allclose(dev_out.cpu(), host_out, rtol=1e-5, atol=1e-6) and 0 < float(dev_out.max()) < 75
    T0 = p.caches[0].num_types()
    T1 = p.caches[1].num_types()
    # the receptor's channels appear twice, before each ligand's
    assert torch.equal(dev_out[0, :T0], dev_out[0, T0 + T1:2 * T0 + T1]) or \
        torch.allclose(dev_out[0, :T0], dev_out[0, T0 + T1:2 * T0 + T1], rtol=1e-5, atol=1e-6)


def test_device_batch_with_a_null_typer(provider_dir):
    """The receptor typed by NullIndexTyper: no receptor atom survives, the ligand's channels start
    at zero, on the host path and in the device batch alike."""
    ps = []
    for _ in range(2):
        p = coord_cache.ExampleProvider(molgrid.NullIndexTyper(), molgrid.defaultGninaLigandTyper,
                                        data_root=str(provider_dir))
        p.populate(str(provider_dir / "list.types"))
        ps.append(p)
    assert ps[0].num_types() == 14
    exs = ps[0].next_batch(5)
    batch = ps[1].next_device_batch(5).check()
    types, ns = batch.type_index.cpu().numpy(), batch.n_atoms.cpu().numpy()
    coords = batch.coords.cpu().numpy()
    for b, ex in enumerate(exs):
        assert ex.coord_sets[0].size() == 0 and ex.num_types() == 14
        m = ex.merge_coordinates()
        keep = types[b, :ns[b]] >= 0
        np.testing.assert_array_equal(types[b, :ns[b]][keep], m.type_index.tonumpy())
        np.testing.assert_array_equal(coords[b, :ns[b]][keep], m.coords.tonumpy())
    g = molgrid.GridMaker(0.5, 23.5)
    a = torch.zeros((5,) + g.grid_dimensions(14), device="cuda")
    b = torch.zeros_like(a)
    g.forward(batch, a)
    g.forward(exs, b)
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-6) and float(a.max()) > 0
