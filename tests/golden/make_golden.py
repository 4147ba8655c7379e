"""Generates tests/golden/golden.npz from the reference's own CPU code.

Needs oracle/_ref/liblmg_ref.so (``make -C oracle ref``, which compiles the reference's sources
where the reference tree is mounted).  The stored arrays are the reference's outputs on the small
seeded cases of :func:`golden_cases`; tests compare the C restatement (on CPU) and the CUDA path
(on a GPU) with them, so the vectors travel to machines that do not have the reference tree.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests import cases  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")

# name -> GridMaker settings
SETTINGS = {
    "g1": dict(resolution=0.5, dimension=5.5),
    "g1bin": dict(resolution=0.5, dimension=5.5, binary=True),
    "g3": dict(resolution=0.25, dimension=3.75, radius_scale=0.5, gaussian_radius_multiple=3.0),
    "gneg": dict(resolution=0.5, dimension=5.0, radius_scale=1.2, gaussian_radius_multiple=-2.0),
}
CENTER = (0.1, -0.2, 0.3)
NT = 4


def golden_inputs(name):
    """Inputs of one golden case, regenerated identically by the tests."""
    kw = SETTINGS[name]
    ext = kw["dimension"] / 2 + 1
    seed = sorted(SETTINGS).index(name) + 50
    coords, types, radii = cases.index_case(seed, 40, NT, ext, rmin=0.8, rmax=1.8)
    vcoords, tv, vradii = cases.vector_case(seed + 100, 30, NT, ext, rti=False)
    _, _, tradii = cases.vector_case(seed + 100, 30, NT, ext, rti=True)
    rng = np.random.default_rng(seed + 200)
    dim = int(np.round(np.float32(kw["dimension"]) / np.float32(kw["resolution"])) + 1)
    diff = rng.normal(size=(NT, dim, dim, dim)).astype(np.float32)
    return dict(coords=coords, types=types, radii=radii, vcoords=vcoords, tv=tv, vradii=vradii,
                tradii=tradii, diff=diff)


def transform_inputs():
    rng = np.random.default_rng(77)
    q = rng.normal(size=4).astype(np.float32)
    q2 = cases.random_quaternion(rng, 1)[0]
    c = rng.uniform(-2, 2, 3).astype(np.float32)
    t = rng.uniform(-2, 2, 3).astype(np.float32)
    pts = (rng.normal(size=(64, 3)) * 6).astype(np.float32)
    grid = rng.uniform(size=(3, 16, 16, 16)).astype(np.float32)
    return q, q2, c, t, pts, grid


def main():
    from oracle.oracle import CpuOracle
    R = CpuOracle("ref")
    out = {}
    for name, kw in SETTINGS.items():
        gm = R.gm(**kw)
        out[name + "/consts"] = R.consts(gm)
        x = golden_inputs(name)
        dens = R.forward_index(gm, CENTER, x["coords"], x["types"], x["radii"], NT)
        out[name + "/forward_index"] = dens
        out[name + "/backward_index"] = R.backward_index(gm, CENTER, x["coords"], x["types"], x["radii"], x["diff"])
        out[name + "/relevance"] = R.backward_relevance(gm, CENTER, x["coords"], x["types"], x["radii"], dens,
                                                        x["diff"])
        for rti in (0, 1):
            gmv = R.gm(**dict(kw, radii_type_indexed=bool(rti)))
            rad = x["tradii"] if rti else x["vradii"]
            tag = "%s/rti%d/" % (name, rti)
            out[tag + "forward_vector"] = R.forward_vector(gmv, CENTER, x["vcoords"], x["tv"], rad)
            ag, tg = R.backward_vector(gmv, CENTER, x["vcoords"], x["tv"], rad, x["diff"])
            out[tag + "atom_gradients"], out[tag + "type_gradients"] = ag, tg
            if not kw.get("binary"):
                dd, add, tdd = R.backward_gradients(gmv, CENTER, x["vcoords"], x["tv"], rad, x["diff"], ag, tg)
                out[tag + "diffdiff"], out[tag + "atom_diffdiff"], out[tag + "type_diffdiff"] = dd, add, tdd
    q, q2, c, t, pts, grid = transform_inputs()
    out["quat/ops"] = R.quaternion_ops(q, q2, pts[0])
    for name, qq in (("nonunit", q), ("unit", q2)):
        tr = R.tr(qq, c, t)
        for dt in (0, 1):
            out["transform/%s/forward%d" % (name, dt)] = R.transform_forward(tr, pts, bool(dt))
            out["transform/%s/backward%d" % (name, dt)] = R.transform_backward(tr, pts, bool(dt))
    out["interp/same"] = R.interpolate([0.5, 7.5, 0.5, 7.5], c, grid, R.tr(q2, c, t), c)
    out["interp/resample"] = R.interpolate([0.5, 7.5, 0.25, 5.0], (0, 0, 0), grid, R.tr(q2, (0, 0, 0), t), (0.5, 0, 0))
    # the reference's seeded random transforms: 4 draws with rotation, 2 without
    out["random/rot"] = R.random_transform(1234, (1, 2, 3), 2.5, True, 4)
    out["random/norot"] = R.random_transform(99, (0, 0, 0), 1.0, False, 2)
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(out), "arrays")
    molecule(R)


MOL_OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "molecule.npz")
REF_DATA = os.path.join(os.environ.get("LMG_REFERENCE_ROOT", "/root/reference"), "test", "data")


def molecule_diff(shape):
    """Grid gradient of the molecule case, regenerated identically by the tests."""
    return np.random.default_rng(4242).normal(size=shape).astype(np.float32)


def molecule(R):
    """The first example of the reference's test/data/small.types (receptor 4kqp_rec_0 and ligand
    4kqp_min_0, pre-typed records), decoded with this package's reader and gridded by the reference
    with its default GridMaker.  test/test_gridmaker.py:72-103 expects maxima 1.438691 (ligand about
    its centre) and 2.094017 (whole example); both are asserted here before anything is written."""
    from libmolgrid_b200 import coord_cache
    prov = coord_cache.ExampleProvider(data_root=os.path.join(REF_DATA, "structs"))
    prov.populate(os.path.join(REF_DATA, "small.types"))
    ex = prov.next()
    lig = ex.coord_sets[1]
    center = np.array(tuple(lig.center()), dtype=np.float32)
    gm = R.gm(resolution=0.5, dimension=23.5)
    m = ex.merge_coordinates()
    arr = lambda g: g.tonumpy()
    lig_grid = R.forward_index(gm, center, arr(lig.coords), arr(lig.type_index), arr(lig.radii), lig.max_type)
    ex_grid = R.forward_index(gm, center, arr(m.coords), arr(m.type_index), arr(m.radii), m.max_type)
    assert abs(float(lig_grid.max()) - 1.438691) < 1e-5 and abs(float(ex_grid.max()) - 2.094017) < 1e-5
    diff = molecule_diff(ex_grid.shape)
    grad = R.backward_index(gm, center, arr(m.coords), arr(m.type_index), arr(m.radii), diff)
    sample = np.random.default_rng(4243).choice(ex_grid.size, 8192, replace=False)
    out = dict(center=center, labels=np.array(ex.labels, dtype=np.float32),
               rec_coords=arr(ex.coord_sets[0].coords), rec_types=arr(ex.coord_sets[0].type_index),
               rec_radii=arr(ex.coord_sets[0].radii), lig_coords=arr(lig.coords), lig_types=arr(lig.type_index),
               lig_radii=arr(lig.radii), lig_max=lig_grid.max(), ex_max=ex_grid.max(),
               lig_channel_sums=lig_grid.reshape(lig.max_type, -1).sum(1),
               ex_channel_sums=ex_grid.reshape(m.max_type, -1).sum(1, dtype=np.float64),
               sample=sample, ex_sample=ex_grid.reshape(-1)[sample], backward=grad)
    np.savez_compressed(MOL_OUT, **out)
    print("wrote", MOL_OUT, os.path.getsize(MOL_OUT), "bytes")


if __name__ == "__main__":
    main()
