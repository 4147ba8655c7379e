"""Order of the examples an ExampleProvider hands out (no GPU needed): the guarantees of the
reference's providers (include/libmolgrid/exampleref_providers.h) and the checks its own tests make
(test/test_example_provider.py: grouped batches :185-233, copies :304-332, iterator :335-354,
duplicated first set :494-517, epoch sizes :520-560), on small synthetic pre-typed files."""
import math

import numpy as np
import pytest

import libmolgrid_b200 as molgrid
from libmolgrid_b200 import coord_cache


def _write_structs(d, nrec, nlig):
    rng = np.random.default_rng(0)
    for r in range(nrec):
        n = 5 + r
        coord_cache.write_gninatypes(str(d / ("rec%d.gninatypes" % r)), rng.normal(size=(n, 3)).astype(np.float32),
                                     rng.integers(0, 14, n))
    for l in range(nlig):
        n = 2 + l % 3
        coord_cache.write_gninatypes(str(d / ("lig%d.gninatypes" % l)), rng.normal(size=(n, 3)).astype(np.float32) + l,
                                     rng.integers(0, 14, n))


@pytest.fixture()
def lists(tmp_path):
    """40 lines: label (1 for every fourth), an affinity in [2, 10), receptor l % 4 ... except that
    receptor 3 has no actives."""
    _write_structs(tmp_path, 4, 40)
    lines = []
    for l in range(40):
        rec = l % 4
        label = 1 if (l % 8 == 0 or l % 8 == 1 or l % 8 == 2) and rec != 3 else 0
        aff = 2.0 + (l * 7 % 40) / 5.0
        lines.append("%d %.2f rec%d.gninatypes lig%d.gninatypes" % (label, aff, rec, l))
    f = tmp_path / "all.types"
    f.write_text("\n".join(lines) + "\n")
    return tmp_path, str(f), lines


def _provider(d, fname, **kw):
    p = molgrid.ExampleProvider(data_root=str(d), **kw)
    p.populate(fname)
    return p


def _lig(ex):
    return ex.coord_sets[1].src


def test_file_order_and_wrap(lists):
    d, f, lines = lists
    p = _provider(d, f)
    assert p.size() == 40 and p.small_epoch_size() == 40 and p.large_epoch_size() == 40
    got = [_lig(p.next()) for _ in range(45)]
    assert got[:40] == ["lig%d.gninatypes" % i for i in range(40)] and got[40:] == got[:5]
    assert p.get_small_epoch_num() == 1
    p.reset()
    assert _lig(p.next()) == "lig0.gninatypes"
    p.skip(9)
    assert _lig(p.next()) == "lig10.gninatypes"


def test_shuffle_is_a_permutation_per_pass(lists):
    d, f, _ = lists
    p = _provider(d, f, shuffle=True, seed=3)
    first = [_lig(p.next()) for _ in range(40)]
    second = [_lig(p.next()) for _ in range(40)]
    assert sorted(first) == sorted(second) == sorted("lig%d.gninatypes" % i for i in range(40))
    assert first != ["lig%d.gninatypes" % i for i in range(40)] and first != second
    q = _provider(d, f, shuffle=True, seed=3)
    assert [_lig(q.next()) for _ in range(40)] == first           # the seed fixes the order


def test_balanced_alternates(lists):
    d, f, _ = lists
    p = _provider(d, f, balanced=True)
    labels = [p.next().labels[0] for _ in range(30)]
    assert labels == [1.0, 0.0] * 15
    nact = 15   # lines with label 1 in the fixture
    assert p.small_epoch_size() == 2 * nact and p.large_epoch_size() == 2 * (40 - nact)
    with pytest.raises(ValueError):
        _provider(d, f, balanced=True, labelpos=5)


def test_receptor_stratified(lists):
    d, f, _ = lists
    p = _provider(d, f, stratify_receptor=True)
    recs = [p.next().coord_sets[0].src for _ in range(12)]
    assert recs == ["rec%d.gninatypes" % (i % 4) for i in range(12)]
    assert p.small_epoch_size() == 40 and p.large_epoch_size() == 40   # ten lines per receptor
    # balanced inside receptors: pairs (active, decoy) of one receptor; receptor 3 has no actives and is dropped
    p = _provider(d, f, stratify_receptor=True, balanced=True, shuffle=True)
    seen = set()
    for _ in range(20):
        a, b = p.next(), p.next()
        assert a.coord_sets[0].src == b.coord_sets[0].src and a.labels[0] == 1 and b.labels[0] == 0
        seen.add(a.coord_sets[0].src)
    assert seen == {"rec0.gninatypes", "rec1.gninatypes", "rec2.gninatypes"}
    assert p.size() == 30


def test_value_stratified(lists):
    d, f, _ = lists
    p = _provider(d, f, stratify_min=2, stratify_max=10, stratify_step=2, stratify_pos=1)
    bins = [int((p.next().labels[1] - 2) / 2) for _ in range(16)]
    assert bins == [0, 1, 2, 3] * 4
    with pytest.raises(ValueError):
        _provider(d, f, stratify_min=2, stratify_max=10, stratify_step=2, stratify_pos=4)
    with pytest.raises(ValueError):
        molgrid.ExampleProvider(stratify_min=2, stratify_max=3, stratify_step=2)   # a single bin


def test_copies_and_default_batch(lists):
    d, f, _ = lists
    p = _provider(d, f, num_copies=3, default_batch_size=6)
    b = p.next_batch()
    assert len(b) == 6
    assert [_lig(x) for x in b] == ["lig0.gninatypes"] * 3 + ["lig1.gninatypes"] * 3
    # the copies are separate objects
    c0 = b[0].coord_sets[1].coords.tonumpy().copy()
    b[1].coord_sets[1].coords.tonumpy()[:] += 1
    assert np.array_equal(b[0].coord_sets[1].coords.tonumpy(), c0)


def test_duplicate_first(tmp_path):
    _write_structs(tmp_path, 1, 4)
    f = tmp_path / "multi.types"
    f.write_text("1 rec0.gninatypes lig0.gninatypes lig1.gninatypes\n0 rec0.gninatypes lig2.gninatypes lig3.gninatypes\n")
    p = _provider(tmp_path, str(f))
    ex = p.next()
    assert len(ex.coord_sets) == 3 and p.num_types() == 14 + 2 * 14
    p = _provider(tmp_path, str(f), duplicate_first=True)
    ex = p.next()
    assert [c.src for c in ex.coord_sets] == ["rec0.gninatypes", "lig0.gninatypes", "rec0.gninatypes", "lig1.gninatypes"]
    assert np.array_equal(ex.coord_sets[0].coords.tonumpy(), ex.coord_sets[2].coords.tonumpy())
    assert p.num_types() == 4 * 14


def test_make_vector_types(lists):
    d, f, _ = lists
    p = _provider(d, f, make_vector_types=True)
    q = _provider(d, f)
    a, b = p.next(), q.next()
    for ca, cb in zip(a.coord_sets, b.coord_sets):
        assert ca.has_vector_types() and cb.has_indexed_types() and not cb.has_vector_types()
        assert ca.radii.size() == cb.num_types()          # radii by type now (src/coordinateset.cpp:205-211)
        tv = ca.type_vector.tonumpy()
        assert tv.shape == (cb.size(), cb.num_types()) and np.array_equal(tv.sum(1), np.ones(cb.size()))
        assert np.array_equal(tv.argmax(1), cb.type_index.tonumpy())


def test_grouped_batches(tmp_path):
    """Groups of 2 to 4 frames, batches of 3 groups, padded to 5 frames (the layout of the
    reference's grouped.types test)."""
    _write_structs(tmp_path, 3, 30)
    lines, l = [], 0
    for g in range(6):
        for t in range(2 + g % 3):
            lines.append("%d %d %.1f rec%d.gninatypes lig%d.gninatypes" % (g, g % 2, t, g % 3, l))
            l += 1
    f = tmp_path / "grouped.types"
    f.write_text("\n".join(lines) + "\n")
    B, T = 3, 5
    p = _provider(tmp_path, str(f), max_group_size=T, group_batch_size=B)
    assert p.size() == 6                                   # groups
    with pytest.raises(ValueError):
        p.next_batch(4)
    for _ in range(4):
        first = p.next_batch(B)
        groups = [x.group for x in first]
        assert all(not x.seqcont for x in first) and len(set(groups)) == B
        recs = [x.coord_sets[0].src for x in first]
        for t in range(1, T):
            b = p.next_batch(B)
            for x, g, r in zip(b, groups, recs):
                assert x.seqcont and x.group == g
                if t < 2 + g % 3:
                    assert x.coord_sets[0].src == r and x.labels[1] == float(t)
                else:                                       # padding: empty sets, NaN labels
                    assert all(c.size() == 0 for c in x.coord_sets) and all(math.isnan(v) for v in x.labels)


def test_epoch_iteration(lists):
    d, f, _ = lists
    p = _provider(d, f, default_batch_size=10, iteration_scheme=molgrid.IterationScheme.LargeEpoch)
    assert sum(1 for _ in p) == 4
    assert sum(1 for _ in p) == 4                          # and again for the next epoch
    p = _provider(d, f, default_batch_size=4, balanced=True, iteration_scheme="SmallEpoch")
    # 30 examples per small epoch; the counter runs one ahead (it names the epoch of the NEXT example)
    assert p.small_epoch_size() == 30 and sum(1 for _ in p) == 8
    p = _provider(d, f, default_batch_size=10)            # continuous: never ends by itself
    it = iter(p)
    assert [len(next(it)) for _ in range(9)] == [10] * 9


def test_dataset_random_access(lists):
    d, f, _ = lists
    ds = molgrid.ExampleDataset(data_root=str(d), shuffle=True)
    ds.populate(f)
    assert len(ds) == 40 and _lig(ds[7]) == "lig7.gninatypes" and _lig(ds[-1]) == "lig39.gninatypes"
    with pytest.raises(IndexError):
        ds[40]


def test_unknown_setting_is_refused():
    with pytest.raises(TypeError):
        molgrid.ExampleProvider(shufle=True)


def test_mem_caches_round_trip(lists, tmp_path_factory):
    d, f, _ = lists
    p = _provider(d, f)
    want = [(_lig(x), x.coord_sets[1].coords.tonumpy().copy()) for x in (p.next() for _ in range(40))]
    assert p.mem_caches_size() == 4 + 40
    cache = str(tmp_path_factory.mktemp("c") / "mem.cache")
    p.save_mem_caches(cache)
    empty = tmp_path_factory.mktemp("nofiles")             # no structure files here: only the cache can serve
    q = molgrid.ExampleProvider(data_root=str(empty))
    q.load_mem_caches(cache)
    q.populate(f)
    for name, coords in want:
        x = q.next()
        assert _lig(x) == name and np.array_equal(x.coord_sets[1].coords.tonumpy(), coords)


def test_null_typer_and_type_sums_of_a_batch(lists):
    """A receptor typed by NullIndexTyper takes no channels; provider and examples agree on the number
    of types; ExampleVec.sum_types counts the atoms of every type per example, the same into an MGrid
    and a numpy array (test/test_example_provider.py:236-302)."""
    d, f, _ = lists
    e = molgrid.ExampleProvider(molgrid.NullIndexTyper(), molgrid.defaultGninaLigandTyper, data_root=str(d),
                                make_vector_types=True)
    e.populate(f)
    b = e.next_batch(10)
    assert e.num_types() == 14 and b[0].num_types() == 14
    assert b[0].coord_sets[0].has_vector_types() and b[0].coord_sets[1].has_vector_types()
    c = b[0].merge_coordinates()
    tv = c.type_vector.tonumpy()
    assert tv.shape == (c.size(), 14) and np.array_equal(tv.sum(1), np.ones(c.size()))
    sums = molgrid.MGrid2f(10, e.num_types())
    b.sum_types(sums)
    sums2 = np.zeros((10, 14), np.float32)
    b.sum_types(sums2)
    assert np.array_equal(sums.tonumpy(), sums2)
    for i, ex in enumerate(b):
        assert sums2[i].sum() == ex.coord_sets[1].size()
        assert np.array_equal(sums2[i], ex.coord_sets[1].type_vector.tonumpy().sum(0))
    # with both default typers the example has 28 types and the sums fill the ligand's half as above
    e2 = molgrid.ExampleProvider(data_root=str(d), make_vector_types=True)
    e2.populate(f)
    b2 = e2.next_batch(10)
    assert e2.num_types() == b2[0].num_types() == 28
    s28 = np.zeros((10, 28), np.float32)
    b2.sum_types(s28)
    assert np.array_equal(s28[:, 14:], sums2)
