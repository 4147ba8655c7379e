"""The CUDA path against the committed golden vectors (outputs of the reference's own CPU code),
through the C ABI.  These run on machines that do not have the reference tree."""
import os

import numpy as np
import pytest
import torch

from tests.golden import make_golden as mg

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(mg.__file__)), "golden.npz"))
DENS = dict(rtol=1e-5, atol=1e-6)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def grad_close(a, b):
    scale = max(1.0, float(np.abs(b).max()))
    return np.allclose(a, b, rtol=1e-4, atol=1e-5 * scale)


def maker(kw, rti=False):
    import libmolgrid_b200 as lmg
    return lmg.GridMaker(kw["resolution"], kw["dimension"], kw.get("binary", False), rti,
                         kw.get("radius_scale", 1.0), kw.get("gaussian_radius_multiple", 1.0))


@pytest.mark.parametrize("name", sorted(mg.SETTINGS))
def test_index_paths(name):
    kw = mg.SETTINGS[name]
    x = mg.golden_inputs(name)
    g = maker(kw)
    out = torch.empty(g.grid_dimensions(mg.NT), device="cuda")
    g.forward(mg.CENTER, dev(x["coords"]), dev(x["types"]), dev(x["radii"]), out)
    got, want = out.cpu().numpy(), GOLD[name + "/forward_index"]
    if kw.get("binary"):
        assert np.array_equal(got, want)
    else:
        assert np.allclose(got, want, **DENS)
        assert np.array_equal(got != 0, want != 0)   # same footprint, including truncated Gaussians
    ag = torch.empty((40, 3), device="cuda")
    g.backward(mg.CENTER, dev(x["coords"]), dev(x["types"]), dev(x["radii"]), dev(x["diff"]), ag)
    assert grad_close(ag.cpu().numpy(), GOLD[name + "/backward_index"])
    rel = torch.empty((40,), device="cuda")
    g.backward_relevance(mg.CENTER, dev(x["coords"]), dev(x["types"]), dev(x["radii"]), dev(want), dev(x["diff"]), rel)
    assert grad_close(rel.cpu().numpy(), GOLD[name + "/relevance"])


@pytest.mark.parametrize("rti", [0, 1])
@pytest.mark.parametrize("name", sorted(mg.SETTINGS))
def test_vector_paths(name, rti):
    kw = mg.SETTINGS[name]
    x = mg.golden_inputs(name)
    g = maker(kw, bool(rti))
    rad = x["tradii"] if rti else x["vradii"]
    tag = "%s/rti%d/" % (name, rti)
    out = torch.empty(g.grid_dimensions(mg.NT), device="cuda")
    g.forward(mg.CENTER, dev(x["vcoords"]), dev(x["tv"]), dev(rad), out)
    assert np.allclose(out.cpu().numpy(), GOLD[tag + "forward_vector"], **DENS)
    ag = torch.empty((30, 3), device="cuda")
    tg = torch.empty((30, mg.NT), device="cuda")
    g.backward(mg.CENTER, dev(x["vcoords"]), dev(x["tv"]), dev(rad), dev(x["diff"]), ag, tg)
    assert grad_close(ag.cpu().numpy(), GOLD[tag + "atom_gradients"])
    assert grad_close(tg.cpu().numpy(), GOLD[tag + "type_gradients"])
    dd = torch.full(out.shape, 5.0, device="cuda")
    add = torch.full((30, 3), 5.0, device="cuda")
    tdd = torch.full((30, mg.NT), 5.0, device="cuda")
    args = (mg.CENTER, dev(x["vcoords"]), dev(x["tv"]), dev(rad), dev(x["diff"]),
            dev(GOLD[tag + "atom_gradients"]), dev(GOLD[tag + "type_gradients"]), dd, add, tdd)
    if kw.get("binary"):
        with pytest.raises(ValueError):          # "Binary densities not supported"
            g.backward_gradients(*args)
        return
    g.backward_gradients(*args)
    assert grad_close(dd.cpu().numpy(), GOLD[tag + "diffdiff"])
    assert grad_close(add.cpu().numpy(), GOLD[tag + "atom_diffdiff"])
    assert not tdd.any()


def test_transform_and_interpolation():
    import libmolgrid_b200 as lmg
    q, q2, c, t, pts, grid = mg.transform_inputs()
    for name, qq in (("nonunit", q), ("unit", q2)):
        tr = lmg.Transform(lmg.Quaternion(*qq), tuple(c), tuple(t))
        out = torch.empty((64, 3), device="cuda")
        for dt in (0, 1):
            tr.forward(dev(pts), out, bool(dt))
            assert np.array_equal(out.cpu().numpy(), GOLD["transform/%s/forward%d" % (name, dt)])
            tr.backward(dev(pts), out, bool(dt))
            assert np.array_equal(out.cpu().numpy(), GOLD["transform/%s/backward%d" % (name, dt)])
    gi = lmg.GridInterpolater(0.5, 7.5, 0.5, 7.5)
    out = torch.empty((3, 16, 16, 16), device="cuda")
    gi.forward(tuple(c), dev(grid), lmg.Transform(lmg.Quaternion(*q2), tuple(c), tuple(t)), tuple(c), out)
    assert np.array_equal(out.cpu().numpy(), GOLD["interp/same"])
    gi = lmg.GridInterpolater(0.5, 7.5, 0.25, 5.0)
    out = torch.empty((3, 21, 21, 21), device="cuda")
    gi.forward((0, 0, 0), dev(grid), lmg.Transform(lmg.Quaternion(*q2), (0, 0, 0), tuple(t)), (0.5, 0, 0), out)
    assert np.array_equal(out.cpu().numpy(), GOLD["interp/resample"])
