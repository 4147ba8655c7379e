"""Pre-typed atom files, typers and the sequential provider (host only), and the real-molecule
golden case against the CPU oracle."""
import os

import numpy as np
import pytest

import libmolgrid_b200 as molgrid
from libmolgrid_b200 import atom_typing, coord_cache

HERE = os.path.dirname(os.path.abspath(__file__))
MOL = np.load(os.path.join(HERE, "golden", "molecule.npz"))
# the reference tree, where it is mounted (LMG_REFERENCE_ROOT overrides the usual place)
REF_DATA = os.path.join(os.environ.get("LMG_REFERENCE_ROOT", "/root/reference"), "test", "data")


def test_typers():
    g = atom_typing.GninaIndexTyper()
    assert g.num_types() == 28 and g.get_type_names()[26] == "GenericMetal"
    assert g.get_int_type(2) == (2, pytest.approx(1.9))
    assert g.get_int_type(500) == (26, pytest.approx(1.2))   # unknown numbers become GenericMetal
    assert atom_typing.GninaIndexTyper(True).get_int_type(2) == (2, pytest.approx(0.77))
    rec, lig = atom_typing.default_receptor_typer(), atom_typing.default_ligand_typer()
    assert rec.num_types() == 14 and lig.num_types() == 14
    assert rec.get_type_names()[4] == "Bromine_Iodine_Chlorine_Fluorine"
    assert rec.get_int_type(0)[0] == -1 and rec.get_int_type(1)[0] == -1      # hydrogens are unmapped
    assert rec.get_int_type(18) == (4, pytest.approx(1.8)) and lig.get_int_type(18) == (5, pytest.approx(1.8))
    assert lig.get_int_type(23)[0] == 13 and rec.get_int_type(23)[0] == 12    # zinc
    # the radius stays that of the original type; the per-type radius is the group's mean
    assert rec.get_type_radii()[4] == pytest.approx((2.0 + 2.2 + 1.8 + 1.5) / 4)
    t, r = lig.map_types([2, 0, 19, 99])
    assert list(t) == [0, -1, 4, 13] and r[2] == pytest.approx(2.0)
    with pytest.raises(ValueError):
        atom_typing.FileMappedGninaTyper("Carbon\n")


def test_gninatypes_and_molcache_round_trip(tmp_path):
    rng = np.random.default_rng(5)
    coords = rng.normal(size=(12, 3)).astype(np.float32)
    types = np.array([2, 3, 0, 6, 10, 1, 13, 19, 23, 40, 5, 2], np.int32)
    path = tmp_path / "a.gninatypes"
    coord_cache.write_gninatypes(path, coords, types)
    assert os.path.getsize(path) == 12 * 16
    c = coord_cache.read_gninatypes(str(path))            # ligand grouping by default
    keep = (types != 0) & (types != 1)
    assert c.size() == int(keep.sum()) == 10 and c.max_type == 14 and c.src == str(path)
    np.testing.assert_array_equal(c.coords.tonumpy(), coords[keep])
    np.testing.assert_array_equal(c.type_index.tonumpy(), [0, 1, 7, 9, 9, 4, 13, 13, 3, 0])
    np.testing.assert_allclose(c.radii.tonumpy(), [1.9, 1.9, 1.8, 1.7, 1.7, 2.0, 1.2, 1.2, 1.9, 1.9])
    with pytest.raises(ValueError):
        coord_cache.read_gninatypes(str(tmp_path / "missing.gninatypes"))

    cache = tmp_path / "m.molcache2"
    coord_cache.write_molcache2(cache, {"x/lig.gninatypes": (coords, types), "y": (coords[:3], types[:3])})
    mc = coord_cache.MolCache2(cache)
    assert "y" in mc and "z" not in mc
    np.testing.assert_array_equal(mc.records("x/lig.gninatypes")["type"], types)
    cc = coord_cache.CoordCache(atom_typing.default_ligand_typer(), str(tmp_path), "m.molcache2")
    c2 = cc.make_coords("x/lig.gninatypes")
    np.testing.assert_array_equal(c2.coords.tonumpy(), c.coords.tonumpy())
    assert cc.make_coords("none").size() == 0
    bad = tmp_path / "bad.molcache2"
    bad.write_bytes(b"\x00" * 32)
    with pytest.raises(ValueError):
        coord_cache.MolCache2(bad)


def test_provider_reads_example_lists(tmp_path):
    rng = np.random.default_rng(6)
    for name, n in (("r.gninatypes", 30), ("l1.gninatypes", 7), ("l2.gninatypes", 9)):
        coord_cache.write_gninatypes(tmp_path / name, rng.normal(size=(n, 3)), rng.integers(2, 20, n))
    lst = tmp_path / "list.types"
    lst.write_text("1 6.05 r.gninatypes l1.gninatypes\n\n0 -1.5 r.gninatypes l2.gninatypes # comment\n")
    p = coord_cache.ExampleProvider(data_root=str(tmp_path))
    p.populate(str(lst))
    assert p.size() == 2 and p.num_labels() == 2 and p.num_types() == 28
    batch = p.next_batch(3)   # wraps around
    assert [e.labels for e in batch] == [[1.0, 6.05], [0.0, -1.5], [1.0, 6.05]]
    assert [s.size() for s in batch[1].coord_sets] == [30, 9]
    assert batch[0].num_types() == 28 and batch[0].merge_coordinates().size() == 37
    labels = np.zeros((3, 2), np.float32)
    batch.extract_labels(labels)
    assert labels[1, 1] == -1.5
    ref = coord_cache.ExampleRef("3 1 0.5 a b", hasgroup=True)
    assert ref.group == 3 and ref.labels == [1.0, 0.5] and ref.files == ["a", "b"]
    with pytest.raises(ValueError):
        coord_cache.ExampleRef("1 2 3")


def golden_example():
    rec = molgrid.CoordinateSet(MOL["rec_coords"], MOL["rec_types"], MOL["rec_radii"], 14)
    lig = molgrid.CoordinateSet(MOL["lig_coords"], MOL["lig_types"], MOL["lig_radii"], 14)
    ex = molgrid.Example()
    ex.coord_sets += [rec, lig]
    return ex


def test_molecule_known_answers_oracle(port):
    """test/test_gridmaker.py:72-103 of the reference: maxima 1.438691 and 2.094017."""
    ex = golden_example()
    lig = ex.coord_sets[1]
    np.testing.assert_allclose(tuple(lig.center()), MOL["center"], rtol=0, atol=0)
    gm = port.gm(resolution=0.5, dimension=23.5)
    g = port.forward_index(gm, MOL["center"], MOL["lig_coords"], MOL["lig_types"], MOL["lig_radii"], 14)
    assert float(g.max()) == pytest.approx(1.438691, abs=1e-6)
    np.testing.assert_array_equal(g.reshape(14, -1).sum(1), MOL["lig_channel_sums"])
    m = ex.merge_coordinates()
    assert m.max_type == 28 and m.size() == 1791
    g = port.forward_index(gm, MOL["center"], m.coords.tonumpy(), m.type_index.tonumpy(), m.radii.tonumpy(), 28)
    assert float(g.max()) == pytest.approx(2.094017, abs=1e-6)
    np.testing.assert_array_equal(g.reshape(-1)[MOL["sample"]], MOL["ex_sample"])


@pytest.mark.skipif(not os.path.isdir(REF_DATA), reason="reference test data not mounted")
def test_reader_on_reference_fixtures():
    p = coord_cache.ExampleProvider(data_root=os.path.join(REF_DATA, "structs"))
    p.populate(os.path.join(REF_DATA, "small.types"))
    assert p.size() == 1000 and p.num_types() == 28
    ex = p.next()
    np.testing.assert_array_equal(ex.coord_sets[0].coords.tonumpy(), MOL["rec_coords"])
    np.testing.assert_array_equal(ex.coord_sets[1].type_index.tonumpy(), MOL["lig_types"])
    np.testing.assert_array_equal(np.array(ex.labels, dtype=np.float32), MOL["labels"])
    assert np.min(ex.coord_sets[1].type_index.tonumpy()) >= 0
    mc = coord_cache.MolCache2(os.path.join(REF_DATA, "lig.molcache2"))
    assert len(mc.offsets) > 100
    name = next(iter(mc.offsets))
    assert coord_cache.coordinate_set_from_records(mc.records(name), atom_typing.default_ligand_typer()).size() > 0


def _ligonly_first_example():
    p = coord_cache.ExampleProvider(data_root=os.path.join(REF_DATA, "structs"))
    p.populate(os.path.join(REF_DATA, "ligonly.types"))
    return p, p.next()


@pytest.mark.skipif(not os.path.isdir(REF_DATA), reason="reference fixtures not mounted")
def test_sum_types_known_answer_host():
    """Type counts of the first example of the reference's ligonly.types
    (test/test_example_provider.py:278-302 states them for one-hot type vectors; counting the
    type indices gives the same totals)."""
    p, ex = _ligonly_first_example()
    want = [0.] * 14 + [2., 3., 0., 0., 0., 0., 0., 0., 2., 2., 1., 0., 0., 0.]
    out = np.full(p.num_types(), 7.0, np.float32)
    ex.sum_types(out)
    np.testing.assert_array_equal(out, want)
    # shared range: not cleared first, sets must agree on the number of types
    shared = np.ones(14, np.float32)
    ex.sum_types(shared, False)
    np.testing.assert_array_equal(shared, np.array(want[14:]) + 1)
    with pytest.raises(ValueError):
        ex.sum_types(np.zeros(5, np.float32))
    # type vectors: column sums in atom order, added into the output
    cs = molgrid.CoordinateSet(np.zeros((3, 3), np.float32),
                               np.array([[0.5, 0, 0.25], [0.25, 1, 0], [0, 0, 0.125]], np.float32),
                               np.ones(3, np.float32))
    acc = np.array([1, 0, 0], np.float32)
    cs.sum_types(acc, zerofirst=False)
    np.testing.assert_array_equal(acc, [1.75, 1, 0.375])
