"""Autograd bindings (Coords2Grid) on the GPU; follows the reference's test/test_torch.py:128-218."""
import numpy as np
import pytest
import torch

from tests import cases

pytestmark = pytest.mark.gpu


def test_coords2grid_gradients_single_atom():
    """One atom at (1,0,0), r=2, loss = grid value at the centre voxel: d/dx = -0.60653."""
    import libmolgrid_b200 as lmg
    gmaker = lmg.GridMaker(resolution=0.5, dimension=6.0, radius_scale=1.0)
    d = gmaker.spatial_grid_dimensions()[0]
    c2g = lmg.Coords2Grid(gmaker, center=(0, 0, 0))
    coords = torch.tensor([[1.0, 0, 0]], device="cuda", requires_grad=True)
    types = torch.tensor([[1.0]], device="cuda", requires_grad=True)
    radii = torch.tensor([2.0], device="cuda")
    grid = c2g(coords, types, radii)
    assert grid.shape == (1, d, d, d)
    centre = grid[0, d // 2, d // 2, d // 2]
    assert float(centre) == pytest.approx(0.60653066, rel=1e-5)
    centre.backward()
    assert coords.grad[0, 0].item() == pytest.approx(-0.60653066, rel=1e-4)
    assert coords.grad[0, 1].item() == 0 and coords.grad[0, 2].item() == 0
    assert types.grad[0, 0].item() == pytest.approx(0.60653066, rel=1e-4)


def test_batched_equals_single_and_oracle(port):
    import libmolgrid_b200 as lmg
    gmaker = lmg.GridMaker(resolution=0.5, dimension=11.5)
    og = port.gm(0.5, 11.5)
    B, N, T = 3, 50, 4
    data = [cases.vector_case(70 + b, N, T, 6.0) for b in range(B)]
    coords = torch.from_numpy(np.stack([x[0] for x in data])).cuda().requires_grad_()
    types = torch.from_numpy(np.stack([x[1] for x in data])).cuda().requires_grad_()
    radii = torch.from_numpy(np.stack([x[2] for x in data])).cuda()
    c2g = lmg.Coords2Grid(gmaker, center=(0.5, 0, -0.5))
    grid = c2g(coords, types, radii)
    w = torch.randn_like(grid)
    (grid * w).sum().backward()
    for b in range(B):
        want = port.forward_vector(og, (0.5, 0, -0.5), data[b][0], data[b][1], data[b][2])
        assert np.allclose(grid[b].detach().cpu().numpy(), want, rtol=1e-5, atol=1e-6)
        ag, tg = port.backward_vector(og, (0.5, 0, -0.5), data[b][0], data[b][1], data[b][2], w[b].cpu().numpy())
        assert np.allclose(coords.grad[b].cpu().numpy(), ag, rtol=1e-4, atol=1e-5 * max(1, np.abs(ag).max()))
        assert np.allclose(types.grad[b].cpu().numpy(), tg, rtol=1e-4, atol=1e-5 * max(1, np.abs(tg).max()))
        single = c2g(coords[b].detach(), types[b].detach(), radii[b])
        assert torch.allclose(single, grid[b].detach(), rtol=1e-6, atol=1e-7)
    assert "resolution 0.50" in repr(c2g)


def test_double_backward_matches_backward_gradients(port):
    """grad of (grad_coords . v + grad_types . u) w.r.t. the grid gradient, coords = backward_gradients."""
    import libmolgrid_b200 as lmg
    gmaker = lmg.GridMaker(resolution=0.5, dimension=7.5)
    og = port.gm(0.5, 7.5)
    N, T = 20, 3
    c, tv, r = cases.vector_case(91, N, T, 4.0)
    coords = torch.from_numpy(c).cuda().requires_grad_()
    types = torch.from_numpy(tv).cuda().requires_grad_()
    radii = torch.from_numpy(r).cuda()
    d = gmaker.spatial_grid_dimensions()[0]
    rng = np.random.default_rng(4)
    gg = torch.from_numpy(rng.normal(size=(T, d, d, d)).astype(np.float32)).cuda().requires_grad_()
    v = torch.from_numpy(rng.normal(size=(N, 3)).astype(np.float32)).cuda()
    u = torch.from_numpy(rng.normal(size=(N, T)).astype(np.float32)).cuda()
    gc, gt = lmg.Grid2CoordsGradientFunction.apply(gmaker, (0, 0, 0), coords, types, radii, gg)
    ((gc * v).sum() + (gt * u).sum()).backward()
    dd, add, tdd = port.backward_gradients(og, (0, 0, 0), c, tv, r, gg.detach().cpu().numpy(), v.cpu().numpy(),
                                           u.cpu().numpy())
    assert np.allclose(gg.grad.cpu().numpy(), dd, rtol=1e-4, atol=1e-5 * max(1, np.abs(dd).max()))
    assert np.allclose(coords.grad.cpu().numpy(), add, rtol=1e-4, atol=1e-5 * max(1, np.abs(add).max()))
    assert not types.grad.any()


def test_bad_ranks():
    import libmolgrid_b200 as lmg
    c2g = lmg.Coords2Grid(lmg.GridMaker(0.5, 5.5))
    with pytest.raises(RuntimeError):
        c2g(torch.zeros(2, 4, 3, device="cuda"), torch.zeros(4, 2, device="cuda"), torch.ones(4, device="cuda"))


def test_backward_skips_type_gradients_when_types_are_inputs(port):
    """Coordinates' gradients are the same whether or not the types ask for gradients."""
    import libmolgrid_b200 as lmg
    rng = np.random.default_rng(8)
    N, T = 40, 5
    coords = torch.tensor(rng.uniform(-4, 4, (N, 3)).astype(np.float32), device="cuda")
    types = torch.zeros((N, T), device="cuda")
    types[torch.arange(N), torch.arange(N) % T] = 1.0
    radii = torch.full((N,), 1.5, device="cuda")
    gm = lmg.GridMaker(0.5, 11.5)
    weight = torch.randn(gm.grid_dimensions(T), device="cuda")
    grads = []
    for types_need_grad in (False, True):
        c = coords.clone().requires_grad_(True)
        t = types.clone().requires_grad_(types_need_grad)
        out = lmg.Coords2GridFunction.apply(gm, (0, 0, 0), c, t, radii)
        (out * weight).sum().backward()
        grads.append(c.grad.clone())
        assert (t.grad is not None) == types_need_grad
    assert float(grads[1].abs().max()) > 0.1
    torch.testing.assert_close(grads[0], grads[1], rtol=1e-4, atol=1e-5)
