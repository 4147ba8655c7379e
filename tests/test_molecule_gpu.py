"""The reference's real-molecule known answers (test/test_gridmaker.py:72-103) on the GPU, from the
atoms stored in tests/golden/molecule.npz, through the Example / CoordinateSet / MGrid overloads."""
import os

import numpy as np
import pytest
import torch

import libmolgrid_b200 as molgrid
from tests.golden.make_golden import molecule_diff
from tests.test_coord_cache import MOL, golden_example

pytestmark = pytest.mark.gpu


def test_molecule_maxima_and_samples():
    ex = golden_example()
    c = ex.coord_sets[1]
    gmaker = molgrid.GridMaker()
    dims = gmaker.grid_dimensions(c.max_type)
    center = tuple(c.center())
    mgridgpu = molgrid.MGrid4f(*dims)
    npout = np.zeros(dims, dtype=np.float32)
    torchout = torch.zeros(dims, dtype=torch.float32)
    cudaout = torch.zeros(dims, dtype=torch.float32, device="cuda")
    gmaker.forward(center, c, mgridgpu.gpu())
    gmaker.forward(center, c, npout)
    gmaker.forward(center, c, torchout)
    gmaker.forward(center, c, cudaout)
    newt = gmaker.make_tensor(center, c)
    assert newt.is_cuda
    for got in (mgridgpu.tonumpy(), npout, torchout.numpy(), cudaout.cpu().numpy(), newt.cpu().numpy(),
                gmaker.make_ndarray(center, c)):
        assert float(got.max()) == pytest.approx(1.438691, abs=2e-6)
    np.testing.assert_allclose(npout.reshape(14, -1).sum(1), MOL["lig_channel_sums"], rtol=1e-5)

    dims = gmaker.grid_dimensions(ex.num_types())
    mg = molgrid.MGrid4f(*dims)
    gmaker.forward(ex, molgrid.Transform(center, 0, False), mg.gpu())
    g = mg.tonumpy()
    assert float(g.max()) == pytest.approx(2.094017, abs=2e-6)
    want = MOL["ex_sample"]
    got = g.reshape(-1)[MOL["sample"]]
    assert np.all(np.abs(got - want) <= 1e-6 + 1e-5 * np.abs(want))
    np.testing.assert_allclose(g.reshape(28, -1).sum(1, dtype=np.float64), MOL["ex_channel_sums"], rtol=1e-5)
    # default centre of forward(example, grid) is the last set's centre: the same grid again
    mg2 = molgrid.MGrid4f(*dims)
    gmaker.forward(ex, mg2)
    np.testing.assert_allclose(mg2.tonumpy(), g, rtol=1e-6, atol=1e-7)


def test_molecule_backward():
    ex = golden_example()
    m = ex.merge_coordinates()
    gmaker = molgrid.GridMaker()
    diff = torch.from_numpy(molecule_diff(gmaker.grid_dimensions(28))).cuda()
    grad = molgrid.MGrid2f(m.size(), 3)
    gmaker.backward(tuple(MOL["center"]), m, diff, grad.gpu())
    got, want = grad.tonumpy(), MOL["backward"]
    assert np.all(np.abs(got - want) <= 1e-5 + 1e-4 * np.abs(want))
    assert float(np.abs(want).max()) > 1.0
