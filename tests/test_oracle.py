"""Pins the CPU oracle (oracle/lmg_oracle.c): bit-identical to the committed golden vectors that
the reference's own CPU code produced, bit-identical to the compiled reference where it is
present, and reproducing the known answers of the reference's test suite."""
import os

import numpy as np
import pytest

from tests import cases
from tests.golden import make_golden as mg

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(mg.__file__)), "golden.npz"))


def same(a, b):
    return np.array_equal(np.asarray(a), np.asarray(b), equal_nan=True)


@pytest.mark.parametrize("name", sorted(mg.SETTINGS))
def test_port_matches_golden(port, name):
    kw = mg.SETTINGS[name]
    gm = port.gm(**kw)
    x = mg.golden_inputs(name)
    assert same(port.consts(gm), GOLD[name + "/consts"])
    dens = port.forward_index(gm, mg.CENTER, x["coords"], x["types"], x["radii"], mg.NT)
    assert same(dens, GOLD[name + "/forward_index"])
    assert same(port.backward_index(gm, mg.CENTER, x["coords"], x["types"], x["radii"], x["diff"]),
                GOLD[name + "/backward_index"])
    assert same(port.backward_relevance(gm, mg.CENTER, x["coords"], x["types"], x["radii"], dens, x["diff"]),
                GOLD[name + "/relevance"])
    for rti in (0, 1):
        gmv = port.gm(**dict(kw, radii_type_indexed=bool(rti)))
        rad = x["tradii"] if rti else x["vradii"]
        tag = "%s/rti%d/" % (name, rti)
        assert same(port.forward_vector(gmv, mg.CENTER, x["vcoords"], x["tv"], rad), GOLD[tag + "forward_vector"])
        ag, tg = port.backward_vector(gmv, mg.CENTER, x["vcoords"], x["tv"], rad, x["diff"])
        assert same(ag, GOLD[tag + "atom_gradients"]) and same(tg, GOLD[tag + "type_gradients"])
        if not kw.get("binary"):
            dd, add, tdd = port.backward_gradients(gmv, mg.CENTER, x["vcoords"], x["tv"], rad, x["diff"], ag, tg)
            assert same(dd, GOLD[tag + "diffdiff"]) and same(add, GOLD[tag + "atom_diffdiff"])
            assert same(tdd, GOLD[tag + "type_diffdiff"]) and not tdd.any()


def test_port_transform_interp_golden(port):
    q, q2, c, t, pts, grid = mg.transform_inputs()
    assert same(port.quaternion_ops(q, q2, pts[0]), GOLD["quat/ops"])
    for name, qq in (("nonunit", q), ("unit", q2)):
        tr = port.tr(qq, c, t)
        for dt in (0, 1):
            assert same(port.transform_forward(tr, pts, bool(dt)), GOLD["transform/%s/forward%d" % (name, dt)])
            assert same(port.transform_backward(tr, pts, bool(dt)), GOLD["transform/%s/backward%d" % (name, dt)])
    assert same(port.interpolate([0.5, 7.5, 0.5, 7.5], c, grid, port.tr(q2, c, t), c), GOLD["interp/same"])
    assert same(port.interpolate([0.5, 7.5, 0.25, 5.0], (0, 0, 0), grid, port.tr(q2, (0, 0, 0), t), (0.5, 0, 0)),
                GOLD["interp/resample"])


def test_port_matches_compiled_reference(port, ref):
    """Random cases beyond the golden ones, when the compiled reference is present."""
    rng = np.random.default_rng(31)
    for kw in (dict(), dict(binary=True), dict(resolution=0.25, dimension=7.75, radius_scale=0.5,
                                               gaussian_radius_multiple=3.0),
               dict(resolution=0.5, dimension=11.5, gaussian_radius_multiple=-1.5)):
        gm = port.gm(**kw)
        T = 6
        ext = kw.get("dimension", 23.5) / 2 + 1
        coords, types, radii = cases.index_case(int(rng.integers(1 << 30)), 150, T, ext)
        a = ref.forward_index(gm, (0, 0, 0), coords, types, radii, T)
        assert same(a, port.forward_index(gm, (0, 0, 0), coords, types, radii, T))
        diff = rng.normal(size=a.shape).astype(np.float32)
        assert same(ref.backward_index(gm, (0, 0, 0), coords, types, radii, diff),
                    port.backward_index(gm, (0, 0, 0), coords, types, radii, diff))
        assert same(ref.backward_relevance(gm, (0, 0, 0), coords, types, radii, a, diff),
                    port.backward_relevance(gm, (0, 0, 0), coords, types, radii, a, diff))
        vc, tv, vr = cases.vector_case(int(rng.integers(1 << 30)), 60, T, ext, rti=True)
        gmv = port.gm(**dict(kw, radii_type_indexed=True))
        assert same(ref.forward_vector(gmv, (0, 0, 0), vc, tv, vr), port.forward_vector(gmv, (0, 0, 0), vc, tv, vr))
        ra, pa = ref.backward_vector(gmv, (0, 0, 0), vc, tv, vr, diff), port.backward_vector(gmv, (0, 0, 0), vc, tv, vr, diff)
        assert same(ra[0], pa[0]) and same(ra[1], pa[1])


# ---- known answers from the reference's own tests --------------------------------------------
def test_line_profile(port):
    """test/test_gridmaker.py:131-164: one atom, r=1, 0.1 A grid."""
    gm = port.gm(0.1, 6.0)
    out = port.forward_index(gm, (0, 0, 0), [[0, 0, 0]], [0], [1.0], 1)[0]
    c = out.shape[0] // 2
    assert out[c, c, c] == 1.0
    assert out[c + 5, c, c] == pytest.approx(0.60653066, abs=1e-6)
    assert out[c, c - 12, c] == pytest.approx(0.0487206, abs=1e-6)
    assert out[c, c, c + 15] == 0
    # gaussian_radius_multiple=3 with radius_scale=0.5, test/test_gridmaker.py:166-184
    gm = port.gm(0.1, 6.0, False, False, 0.5, 3.0)
    out = port.forward_index(gm, (0, 0, 0), [[0, 0, 0]], [0], [2.0], 1)[0]
    assert out[c + 10, c, c] == pytest.approx(np.exp(-2.0), rel=1e-6)
    assert out[c + 20, c, c] == pytest.approx(np.exp(-8.0), rel=1e-5)


def test_backward_single_atom(port):
    """test/test_gridmaker.py:186-214: -0.60653 along x."""
    gm = port.gm(0.5, 30.0)
    d = port.dim_of(gm)
    diff = np.zeros((1, d, d, d), np.float32)
    diff[0, d // 2, d // 2, d // 2] = 1
    ag = port.backward_index(gm, (0, 0, 0), [[1, 0, 0]], [0], [2.0], diff)
    assert ag[0, 0] == pytest.approx(-0.60653066, rel=1e-6)
    assert ag[0, 1] == 0 and ag[0, 2] == 0


def test_vector_type_gradient_signs(port):
    """test/test_gridmaker.py:364-391: two atoms either side of an upstream spike."""
    gm = port.gm(0.5, 6.0)
    d = port.dim_of(gm)
    diff = np.zeros((2, d, d, d), np.float32)
    diff[0, d // 2, d // 2, d // 2] = 1.0
    coords = np.array([[1, 0, 0], [-1, 0, 0]], np.float32)
    tv = np.array([[1, 0], [1, 0]], np.float32)
    ag, tg = port.backward_vector(gm, (0, 0, 0), coords, tv, [2.0, 2.0], diff)
    assert ag[0, 0] < 0 < ag[1, 0] and ag[0, 0] == pytest.approx(-ag[1, 0])
    assert tg[0, 0] > 0 and tg[0, 1] == 0


def test_backward_gradients_analytic(port):
    """test/test_gridmaker.py:439-487: truncated Gaussian (G=-2), second derivative along x."""
    gm = port.gm(0.1, 6.0, False, False, 1.0, -2.0)
    d = port.dim_of(gm)
    c = d // 2
    for dx in (3, 7):
        diff = np.zeros((1, d, d, d), np.float32)
        diff[0, c + dx, c, c] = 1.0
        coords = np.zeros((1, 3), np.float32)
        tv = np.ones((1, 1), np.float32)
        ag = np.array([[1.0, 0, 0]], np.float32)
        tg = np.zeros((1, 1), np.float32)
        dd, add, tdd = port.backward_gradients(gm, (0, 0, 0), coords, tv, [1.0], diff, ag, tg)
        x = dx * 0.1
        # d/dx of the atom gradient 4x e^{-2x^2}(grid minus atom convention): the reference's closed
        # form 16 x^2 e^{-2x^2} - 4 e^{-2x^2}
        want = 16 * x * x * np.exp(-2 * x * x) - 4 * np.exp(-2 * x * x)
        assert add[0, 0] == pytest.approx(want, rel=1e-4)
        assert not tdd.any()


def test_transform_points(port):
    """test/test_transform.py:30-97."""
    s = np.sqrt(0.5)
    tr = port.tr((s, 0, 0, s), (0, 1, 1), (2, 2, -3))
    out = port.transform_forward(tr, [[1, 1, 1]])
    assert np.allclose(out, [[2, 4, -2]], atol=1e-6)
    assert np.allclose(port.transform_backward(tr, out), [[1, 1, 1]], atol=1e-5)


def test_interpolation_identity_and_downsample(port):
    """test/test_gridinterp.py:15-30: identity resample is exact; so is 2x down-sampling."""
    rng = np.random.default_rng(0)
    g = rng.uniform(size=(2, 13, 13, 13)).astype(np.float32)
    same_res = port.interpolate([0.5, 6.0, 0.5, 6.0], (0, 0, 0), g, port.tr(), (0, 0, 0))
    assert np.array_equal(same_res, g)
    down = port.interpolate([0.5, 6.0, 1.0, 6.0], (0, 0, 0), g, port.tr(), (0, 0, 0))
    assert np.array_equal(down, g[:, ::2, ::2, ::2])


def test_interpolation_vs_scipy(port):
    """test/test_gridinterp.py: random rotations against scipy's RegularGridInterpolator (1e-4)."""
    from scipy.interpolate import RegularGridInterpolator
    from scipy.spatial.transform import Rotation
    rng = np.random.default_rng(2)
    d = 17
    g = rng.uniform(size=(1, d, d, d)).astype(np.float32)
    ax = np.arange(d) * 0.5 - 4.0
    f = RegularGridInterpolator((ax, ax, ax), g[0].astype(np.float64), bounds_error=False, fill_value=0)
    q = cases.random_quaternion(rng, 1)[0]
    out = port.interpolate([0.5, 8.0, 0.5, 8.0], (0, 0, 0), g, port.tr(q), (0, 0, 0))
    rot = Rotation.from_quat([q[1], q[2], q[3], q[0]])
    pts = np.stack(np.meshgrid(ax, ax, ax, indexing="ij"), -1).reshape(-1, 3)
    src = rot.inv().apply(pts)
    inside = np.all(np.abs(src) < 3.99, axis=1)
    want = f(src).reshape(d, d, d)
    assert np.allclose(out[0].reshape(-1)[inside], want.reshape(-1)[inside], atol=1e-4)
