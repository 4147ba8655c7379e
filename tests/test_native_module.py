"""The compiled (pybind11) module over the C++ host layer: value types and argument checks on the
host, and on the GPU the same results as the ctypes module for every bound operation."""
import numpy as np
import pytest
import torch

import libmolgrid_b200 as molgrid
from tests import cases


@pytest.fixture(scope="module")
def native():
    from libmolgrid_b200 import build
    build.build_native_module()
    from libmolgrid_b200 import molgrid_native
    return molgrid_native


def test_value_types_and_settings(native):
    g = native.GridMaker(resolution=0.5, dimension=23.5, binary=True, radius_type_indexed=False,
                         radius_scale=1.0, gaussian_radius_multiple=1.0)
    assert g.grid_dimensions(28) == (28, 48, 48, 48) and g.spatial_grid_dimensions() == (48, 48, 48)
    assert g.get_binary() and not g.get_radii_type_indexed()
    g.set_resolution(0.25)
    assert g.grid_dimensions(1) == (1, 95, 95, 95)
    q = native.Quaternion(0.5, 0.5, 0.5, 0.5)
    p = q.rotate(1, 0, 0)
    assert (p.x, p.y, p.z) == pytest.approx((0, 1, 0))
    assert (q * q.inverse()).R_component_1() == pytest.approx(1.0)
    want = molgrid.Quaternion(0.3, -0.2, 0.9, 0.1) * molgrid.Quaternion(0.5, 0.5, -0.5, 0.5)
    got = native.Quaternion(0.3, -0.2, 0.9, 0.1) * native.Quaternion(0.5, 0.5, -0.5, 0.5)
    assert [got.R_component_1(), got.R_component_2(), got.R_component_3(), got.R_component_4()] == \
        [want.R_component_1(), want.R_component_2(), want.R_component_3(), want.R_component_4()]
    t = native.Transform(q, (0, 0, 0), (1, 2, 3))
    assert tuple(t.get_translation()) == (1.0, 2.0, 3.0) and len(native.float3((1, 2, 3))) == 3
    # the same seeded draws as the ctypes module (one engine behind both)
    native.set_random_seed(1234)
    a = native.Transform((1, 2, 3), 2.5, True)
    molgrid.set_random_seed(1234)
    b = molgrid.Transform((1, 2, 3), 2.5, True)
    assert a.get_quaternion().R_component_2() == b.get_quaternion().R_component_2()
    assert tuple(a.get_translation()) == tuple(b.get_translation())
    gi = native.GridInterpolater(in_resolution=0.5, in_dimension=11.5, out_resolution=0.25, out_dimension=8.0)
    assert gi.get_out_resolution() == 0.25
    with pytest.raises(TypeError):
        g.forward((0, 0, 0), [1, 2, 3], np.zeros(1, np.float32), np.zeros(1, np.float32), np.zeros((1, 2, 2, 2), np.float32))
    with pytest.raises(ValueError):
        g.forward((0, 0, 0), np.zeros((1, 3)), np.zeros(1, np.float32), np.zeros(1, np.float32),
                  np.zeros((1, 95, 95, 95), np.float32))   # float64 coordinates


@pytest.mark.gpu
def test_native_matches_ctypes_module(native):
    T, N = 5, 60
    coords, types, radii = cases.index_case(3, N, T, 7.0)
    vcoords, tv, vradii = cases.vector_case(4, N, T, 7.0)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    ga, gb = molgrid.GridMaker(0.5, 11.5), native.GridMaker(0.5, 11.5)
    dims = ga.grid_dimensions(T)
    center = (0.1, -0.2, 0.3)
    a, b = torch.zeros(dims, device="cuda"), torch.zeros(dims, device="cuda")
    ga.forward(center, d(coords), d(types), d(radii), a)
    gb.forward(center, d(coords), d(types), d(radii), b)
    torch.testing.assert_close(a, b, rtol=1e-6, atol=1e-7)
    assert float(a.sum()) > 10
    host = np.zeros(dims, np.float32)                   # host arrays are staged
    gb.forward(center, coords, types, radii, host)
    np.testing.assert_allclose(host, a.cpu().numpy(), rtol=1e-6, atol=1e-7)
    mg = molgrid.MGrid4f(*dims)                         # this package's MGrid converts to its GPU side
    gb.forward(center, coords, types, radii, mg)
    assert mg.ongpu()
    np.testing.assert_allclose(mg.tonumpy(), host, rtol=1e-6, atol=1e-7)
    ga.forward(center, d(vcoords), d(tv), d(vradii), a)
    gb.forward(center, d(vcoords), d(tv), d(vradii), b)
    torch.testing.assert_close(a, b, rtol=1e-6, atol=1e-7)
    # batched
    B = 3
    bc, bt, br, ns, _ = cases.blob_batch(5, B, 100, 150, T)
    cen = np.zeros((B, 3), np.float32)
    ba, bb = torch.zeros((B,) + dims, device="cuda"), torch.zeros((B,) + dims, device="cuda")
    ga.forward(d(cen), d(bc), d(bt), d(br), ba)
    gb.forward(d(cen), d(bc), d(bt), d(br), bb)
    torch.testing.assert_close(ba, bb, rtol=1e-6, atol=1e-7)
    # backward, index and vector types
    diff = torch.randn(dims, device="cuda")
    x, y = torch.zeros((N, 3), device="cuda"), torch.zeros((N, 3), device="cuda")
    ga.backward(center, d(coords), d(types), d(radii), diff, x)
    gb.backward(center, d(coords), d(types), d(radii), diff, y)
    assert torch.equal(x, y)
    xt, yt = torch.zeros((N, T), device="cuda"), torch.zeros((N, T), device="cuda")
    ga.backward(center, d(vcoords), d(tv), d(vradii), diff, x, xt)
    gb.backward(center, d(vcoords), d(tv), d(vradii), diff, y, yt)
    assert torch.equal(x, y) and torch.equal(xt, yt)
    # second order and relevance
    dd = [torch.zeros(dims, device="cuda") for _ in range(2)]
    ad = [torch.zeros((N, 3), device="cuda") for _ in range(2)]
    td = [torch.ones((N, T), device="cuda") for _ in range(2)]
    ga.backward_gradients(center, d(vcoords), d(tv), d(vradii), diff, x, xt, dd[0], ad[0], td[0])
    gb.backward_gradients(center, d(vcoords), d(tv), d(vradii), diff, x, xt, dd[1], ad[1], td[1])
    torch.testing.assert_close(dd[0], dd[1], rtol=1e-5, atol=1e-6)
    assert torch.equal(ad[0], ad[1]) and float(td[1].abs().sum()) == 0
    ga.forward(center, d(coords), d(types), d(radii), a)
    ra, rb = torch.zeros(N, device="cuda"), torch.zeros(N, device="cuda")
    ga.backward_relevance(center, d(coords), d(types), d(radii), a, diff, ra)
    gb.backward_relevance(center, d(coords), d(types), d(radii), a, diff, rb)
    assert torch.equal(ra, rb)
    # transform and interpolation
    q = [float(v) for v in cases.random_quaternion(np.random.default_rng(1), 1)[0]]
    ta = molgrid.Transform(molgrid.Quaternion(*q), (1, 0, -1), (0.5, 0.25, -2))
    tb = native.Transform(native.Quaternion(*q), (1, 0, -1), (0.5, 0.25, -2))
    pa, pb = torch.zeros((N, 3), device="cuda"), torch.zeros((N, 3), device="cuda")
    ta.forward(d(coords), pa)
    tb.forward(d(coords), pb)
    assert torch.equal(pa, pb)
    tb.backward(pb, pb, False)
    ta.backward(pa, pa, False)
    assert torch.equal(pa, pb)
    ia, ib = molgrid.GridInterpolater(0.5, 11.5, 0.5, 11.5), native.GridInterpolater(0.5, 11.5, 0.5, 11.5)
    src = torch.rand(dims, device="cuda")
    oa, ob = torch.zeros(dims, device="cuda"), torch.zeros(dims, device="cuda")
    ia.forward(src, ta, oa)
    ib.forward(src, tb, ob)
    assert torch.equal(oa, ob) and float(oa.sum()) > 1
    ia.backward(oa, ta, a)
    ib.backward(ob, tb, b)
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    # errors keep the reference's exception types
    with pytest.raises(IndexError):
        gb.forward(center, d(coords), d(types), d(radii), torch.zeros((T, 25, 24, 24), device="cuda"))
    with pytest.raises(ValueError):
        gb.forward(center, d(coords), d(types), d(radii), torch.zeros((T, 24, 24, 48), device="cuda")[..., ::2])
    with pytest.raises(ValueError):
        ib.forward(src, tb, src)
