"""GPU parity of Transform forward/backward and GridInterpolater against the CPU oracle,
through the C ABI.  Coordinates are bit-exact (same operation order, no fused multiply-add);
interpolated grids are held to rel 1e-4 as the path states, and checked for exact equality too
since the kernel keeps the reference's operation order."""
import numpy as np
import pytest
import torch

from tests import cases

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(autouse=True)
def _no_copy_timeouts():
    """No block of the tiled interpolation ever gave up waiting for its staged box."""
    yield
    from libmolgrid_b200 import _cabi
    torch.cuda.synchronize()
    assert _cabi.lib().lmg_tma_timeouts() == 0


def make_transform(q, c, t):
    import libmolgrid_b200 as lmg
    return lmg.Transform(lmg.Quaternion(*q), tuple(c), tuple(t))


@pytest.mark.parametrize("dotranslate", [True, False])
def test_transform_bit_exact(port, dotranslate):
    rng = np.random.default_rng(2)
    pts = (rng.normal(size=(1000, 3)) * 8).astype(np.float32)
    for q in (cases.random_quaternion(rng, 1)[0], rng.normal(size=4).astype(np.float32)):  # unit and not
        c, t = rng.uniform(-3, 3, 3).astype(np.float32), rng.uniform(-2, 2, 3).astype(np.float32)
        tr = make_transform(q, c, t)
        otr = port.tr(q, c, t)
        out = torch.empty((1000, 3), device="cuda")
        tr.forward(dev(pts), out, dotranslate)
        assert np.array_equal(out.cpu().numpy(), port.transform_forward(otr, pts, dotranslate))
        tr.backward(dev(pts), out, dotranslate)
        assert np.array_equal(out.cpu().numpy(), port.transform_backward(otr, pts, dotranslate))


def test_transform_known_points():
    """test/test_transform.py:30-97 of the reference: rotations by 90 degrees about axes."""
    import libmolgrid_b200 as lmg
    s = float(np.sqrt(0.5))
    pts = dev(np.array([[1, 1, 1]], np.float32))
    out = torch.empty_like(pts)
    tr = lmg.Transform(lmg.Quaternion(s, 0, 0, s), (0, 1, 1), (2, 2, -3))
    tr.forward(pts, out)
    # rotate (1,0,0) about z by 90 degrees around centre (0,1,1) -> (0,1,0)+(0,1,1), then translate
    assert np.allclose(out.cpu().numpy(), [[2, 4, -2]], atol=1e-6)
    back = torch.empty_like(pts)
    tr.backward(out, back)
    assert np.allclose(back.cpu().numpy(), [[1, 1, 1]], atol=1e-5)
    # in place is allowed
    tr.forward(pts, pts)
    assert torch.equal(pts, out)


def test_transform_roundtrip_large():
    import libmolgrid_b200 as lmg
    lmg.set_random_seed(0)
    rng = np.random.default_rng(1)
    pts = dev((rng.normal(size=(200000, 3)) * 10).astype(np.float32))
    tr = lmg.Transform((1.0, -2.0, 0.5), 3.0, True)
    a = torch.empty_like(pts)
    b = torch.empty_like(pts)
    tr.forward(pts, a)
    tr.backward(a, b)
    assert torch.allclose(b, pts, atol=1e-4)


@pytest.mark.parametrize("gi", [(0.5, 11.5, 0.5, 11.5), (0.5, 11.5, 0.25, 8.0), (0.25, 6.0, 0.5, 9.5)])
def test_interpolate(port, gi):
    import libmolgrid_b200 as lmg
    rng = np.random.default_rng(4)
    g = lmg.GridInterpolater(*gi)
    din, dout = g.s.in_dim, g.s.out_dim
    K = 5
    grid = rng.uniform(size=(K, din, din, din)).astype(np.float32)
    for q, c, t, ic, oc in [
        ((1, 0, 0, 0), (0, 0, 0), (0, 0, 0), (0, 0, 0), (0, 0, 0)),
        (cases.random_quaternion(rng, 1)[0], (0.5, 0, -1), (1, -0.5, 0.25), (0.5, 0, -1), (0.5, 0, -1)),
        (cases.random_quaternion(rng, 1)[0], (0, 0, 0), (0, 2, 0), (1, 0, 0), (0, 0.5, 0)),
    ]:
        want = port.interpolate(gi, ic, grid, port.tr(q, c, t), oc)
        out = torch.full((K, dout, dout, dout), -3.0, device="cuda")
        g.forward(ic, dev(grid), make_transform(q, c, t), oc, out)
        got = out.cpu().numpy()
        assert np.allclose(got, want, rtol=1e-4, atol=1e-6)
        assert np.array_equal(got, want)


def test_interpolate_batched_and_identity(port):
    import libmolgrid_b200 as lmg
    rng = np.random.default_rng(9)
    gi = (0.5, 5.5, 0.5, 5.5)
    g = lmg.GridInterpolater(*gi)
    B, K, d = 60, 3, 12   # more examples than one launch carries
    grids = rng.uniform(size=(B, K, d, d, d)).astype(np.float32)
    qs = cases.random_quaternion(rng, B)
    ts = rng.uniform(-1, 1, (B, 3)).astype(np.float32)
    trs = [make_transform(qs[b], (0, 0, 0), ts[b]) for b in range(B)]
    out = torch.empty((B, K, d, d, d), device="cuda")
    g.forward(dev(grids), trs, out)
    got = out.cpu().numpy()
    for b in (0, 17, 47, 48, 59):
        want = port.interpolate(gi, (0, 0, 0), grids[b], port.tr(qs[b], (0, 0, 0), ts[b]), (0, 0, 0))
        assert np.array_equal(got[b], want)
    # identity transform reproduces the input (test/test_gridinterp.py:15-30)
    one = torch.empty((K, d, d, d), device="cuda")
    g.forward(dev(grids[0]), lmg.Transform(), one)
    assert np.array_equal(one.cpu().numpy(), grids[0])
    with pytest.raises(ValueError):
        g.forward(one, lmg.Transform(), one)


def test_interpolate_tiled_equals_direct_at_benchmark_shape():
    """28x48^3 grids under random rotations: the kernel that stages input boxes with tensor copies
    and the direct-read kernel give identical bits, and no staged copy ever timed out."""
    import libmolgrid_b200 as lmg
    from libmolgrid_b200 import _cabi
    rng = np.random.default_rng(21)
    B, K, d = 6, 28, 48
    g = lmg.GridInterpolater(0.5, 23.5, 0.5, 23.5)
    src = torch.rand((B, K, d, d, d), device="cuda")
    qs = cases.random_quaternion(rng, B)
    qs[0] = (1, 0, 0, 0)
    qs[1] = np.array([0.5, 0.5, 0.5, 0.5], np.float32)   # 120 degrees about the diagonal
    ts = rng.uniform(-2, 2, (B, 3)).astype(np.float32)
    ts[2] = (40, 0, 0)                                    # mostly outside the input
    trs = [make_transform(qs[b], (0, 0, 0), ts[b]) for b in range(B)]
    tiled, direct = torch.full_like(src, -2.0), torch.empty_like(src)
    lib = _cabi.lib()
    g.forward(src, trs, tiled)
    try:
        lib.lmg_set_interp_tiled(0)
        g.forward(src, trs, direct)
    finally:
        lib.lmg_set_interp_tiled(1)
    torch.cuda.synchronize()
    assert torch.equal(tiled, direct)
    assert float(tiled[3].abs().sum()) > 0 and float(tiled[2].abs().sum()) < float(tiled[3].abs().sum())
    assert lib.lmg_tma_timeouts() == 0
    # an unaligned view of the same data takes the direct kernel and agrees as well
    shifted = torch.empty(src[0].numel() + 1, device="cuda")[1:].view_as(src[0])
    shifted.copy_(src[3])
    one = torch.empty_like(src[0])
    g.forward(shifted, trs[3], one)
    assert torch.equal(one, tiled[3])


@pytest.mark.parametrize("gi", [(0.5, 23.5, 0.6, 21.0), (0.5, 23.5, 0.41, 15.17), (0.5, 15.5, 1.5, 30.0)])
def test_interpolate_staged_resampling(port, gi):
    """Coarser and finer output grids than the input (input rows 16-byte aligned: the finer one
    takes the staged kernel, the coarser ones the direct kernel), against the oracle."""
    import libmolgrid_b200 as lmg
    rng = np.random.default_rng(33)
    g = lmg.GridInterpolater(*gi)
    din, dout = g.s.in_dim, g.s.out_dim
    assert din % 4 == 0
    K = 3
    grid = rng.uniform(size=(K, din, din, din)).astype(np.float32)
    q = cases.random_quaternion(rng, 1)[0]
    c, t = (0.25, -0.5, 0.75), (1.0, -2.0, 0.5)
    want = port.interpolate(gi, c, grid, port.tr(q, c, t), (0.0, 0.5, 0.0))
    out = torch.full((K, dout, dout, dout), -3.0, device="cuda")
    g.forward(c, dev(grid), make_transform(q, c, t), (0.0, 0.5, 0.0), out)
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("gi", [(0.5, 11.5, 0.5, 11.5), (0.5, 11.5, 0.25, 8.0), (0.25, 6.0, 0.5, 9.5)])
def test_interpolate_backward_is_the_adjoint(gi):
    """<forward(x), y> == <x, backward(y)> for random x, y, and backward of a one-hot output gradient
    reproduces the forward pass's weights (checked through a finite difference of the forward)."""
    import libmolgrid_b200 as lmg
    rng = np.random.default_rng(41)
    torch.manual_seed(41)          # the random grids below: the same on every run
    g = lmg.GridInterpolater(*gi)
    din, dout = g.s.in_dim, g.s.out_dim
    K = 3
    tr = make_transform(cases.random_quaternion(rng, 1)[0], (0.5, 0, -1), (1, -0.5, 0.25))
    x = torch.rand((K, din, din, din), device="cuda", dtype=torch.float32)
    y = torch.randn((K, dout, dout, dout), device="cuda", dtype=torch.float32)
    fx = torch.empty_like(y)
    g.forward(x, tr, fx)
    by = torch.full_like(x, 5.0)   # must be overwritten
    g.backward(y, tr, by)
    lhs = float((fx.double() * y.double()).sum())
    rhs = float((x.double() * by.double()).sum())
    # float32 accumulation on both sides: the bound is relative to the size of the terms, since
    # y has both signs and the sums may cancel
    scale = float((fx.double() * y.double()).abs().sum())
    assert scale > 1.0 and abs(lhs - rhs) <= 1e-5 * scale
    # linearity in x: forward(x + h e) - forward(x) = h * forward(e); <that, y> = h * by[e]
    e = (1, din // 2, din // 2 - 1, din // 2)
    x2 = x.clone()
    x2[e] += 1.0
    fx2 = torch.empty_like(y)
    g.forward(x2, tr, fx2)
    assert float(((fx2 - fx).double() * y.double()).sum()) == pytest.approx(float(by[e]), rel=1e-3, abs=1e-4)
    # batched, five-argument form
    xb = torch.rand((2, K, din, din, din), device="cuda")
    yb = torch.randn((2, K, dout, dout, dout), device="cuda")
    trs = [tr, make_transform(cases.random_quaternion(rng, 1)[0], (0, 0, 0), (0, 1, 0))]
    cen = np.zeros((2, 3), np.float32)
    fb, bb = torch.empty_like(yb), torch.empty_like(xb)
    g.forward(cen, xb, trs, cen, fb)
    g.backward(cen, yb, trs, cen, bb)
    scale = float((fb.double() * yb.double()).abs().sum())
    assert abs(float((fb.double() * yb.double()).sum()) - float((xb.double() * bb.double()).sum())) <= 1e-5 * scale
    with pytest.raises(ValueError):
        g.backward(y, tr, torch.empty_like(y) if din != dout else y)


@pytest.mark.parametrize("layer", ["python", "compiled"])
def test_transform_known_answers_on_host_arrays_and_in_place(layer):
    """The reference's worked example (test/test_transform.py:65-140): a quarter turn about z through
    (0,1,1) then a shift by (2,0,-3), on numpy arrays and MGrids, the input left unchanged; a random
    transform undone in place."""
    if layer == "python":
        import libmolgrid_b200 as mg
    else:
        import molgrid as mg
    from math import sqrt
    q = mg.Quaternion(sqrt(0.5), 0, 0, sqrt(0.5))
    nr = mg.Transform(q, mg.float3(0, 1, 1), mg.float3(2, 0, -3))
    data = np.array([[0, 0, 0], [1, 0, 0], [0, 1, 0], [0, 0, 1], [-1, .5, 3], [1, 1, 1], [0, 1, 1], [.333, .75, -9]],
                    np.float32)
    coords, out = data.copy(), np.zeros((8, 3), np.float32)
    nr.forward(coords, out)
    assert tuple(out[6]) == (2, 1, -2) and tuple(out[2]) == (2, 1, -3) and tuple(out[5]) == (2, 2, -2)
    assert np.array_equal(coords, data)
    m_in, m_out = mg.MGrid2f(8, 3), mg.MGrid2f(8, 3)
    m_in.copyFrom(data)
    nr.forward(m_in, m_out)
    assert np.array_equal(m_out.tonumpy(), out)
    r = mg.Transform(mg.float3(0, 1, 1), 10.0, True)
    r.forward(coords, out)
    assert not np.isclose(out, coords, atol=1e-5).all(axis=1).any()
    r.backward(out, out)                                   # in place
    assert np.allclose(out, coords, atol=1e-5)
