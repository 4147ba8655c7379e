"""lmg_backward_static: the backward pass for hosts that cannot allocate device memory.

Called through the C ABI directly (ctypes), twice in a row, and compared with lmg_backward, the
entry point that takes a caller-provided workspace (the same kernels run, so bit for bit), and with
the CPU checker.  Kept in a file that pytest collects last so
that a run stopping at the first failure has already exercised everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

from tests import cases

pytestmark = pytest.mark.gpu


def _atoms(coords, types, radii, center, T):
    from libmolgrid_b200 import _cabi
    a = _cabi.AtomsStruct()
    a.batch, a.max_atoms, a.ntypes = coords.shape[0], coords.shape[1], T
    a.coords, a.type_index, a.radii = coords.data_ptr(), types.data_ptr(), radii.data_ptr()
    a.center_host[:] = list(center)
    return a


def test_static_backward_matches_workspace_backward(lib, port):
    from libmolgrid_b200 import _cabi
    torch.cuda.set_device(0)
    s = _cabi.GridMakerStruct()
    assert lib.lmg_gridmaker_init(ctypes.byref(s), 0.5, 11.5, 0, 0, 1.0, 1.0) == 0
    T, B, N = 6, 3, 200
    d = int(s.dim)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(123)
    for call in range(2):   # two calls in a row share the library's fixed scratch array
        data = [cases.index_case(900 + 10 * call + b, N, T, 6.5) for b in range(B)]
        coords = torch.from_numpy(np.stack([x[0] for x in data])).cuda()
        types = torch.from_numpy(np.stack([x[1] for x in data])).cuda()
        radii = torch.from_numpy(np.stack([x[2] for x in data])).cuda()
        diff = torch.from_numpy(rng.normal(size=(B, T, d, d, d)).astype(np.float32)).cuda()
        center = (0.25 * call, -0.5, 0.1)
        a = _atoms(coords, types, radii, center, T)

        want = torch.full((B, N, 3), 7.0, device="cuda")
        nbytes = lib.lmg_workspace_bytes(ctypes.byref(s), _cabi.OP_BACKWARD, B, N, T, 0)
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        rc = lib.lmg_backward(ctypes.byref(s), ctypes.byref(a), diff.data_ptr(), want.data_ptr(), None,
                              ws.data_ptr(), nbytes, stream)
        assert rc == 0, lib.lmg_last_error()

        got = torch.full((B, N, 3), -7.0, device="cuda")
        rc = lib.lmg_backward_static(ctypes.byref(s), ctypes.byref(a), diff.data_ptr(), got.data_ptr(), stream)
        assert rc == 0, lib.lmg_last_error()
        torch.cuda.synchronize()
        assert lib.lmg_static_check_status(stream) == 0, lib.lmg_last_error()
        assert torch.equal(got, want)
        w, g = want.cpu().numpy(), got.cpu().numpy()
        assert np.abs(w).max() > 0.1
        og = port.gm(0.5, 11.5)
        dh = diff.cpu().numpy()
        for b in range(B):
            ref = port.backward_index(og, center, data[b][0], data[b][1], data[b][2], dh[b])
            scale = max(1.0, float(np.abs(ref).max()))
            assert np.allclose(g[b], ref, rtol=1e-4, atol=1e-5 * scale), np.abs(g[b] - ref).max()


def test_static_backward_reports_out_of_range_types(lib):
    """A type index >= ntypes is dropped by the kernel and reported by lmg_static_check_status,
    as lmg_check_status does for the workspace entry point; the next clean call reports nothing."""
    from libmolgrid_b200 import _cabi
    torch.cuda.set_device(0)
    s = _cabi.GridMakerStruct()
    assert lib.lmg_gridmaker_init(ctypes.byref(s), 0.5, 5.5, 0, 0, 1.0, 1.0) == 0
    T, N, d = 3, 8, int(s.dim)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    coords = torch.zeros((1, N, 3), device="cuda")
    radii = torch.ones((1, N), device="cuda")
    diff = torch.ones((1, T, d, d, d), device="cuda")
    for bad in (True, False):
        types = torch.zeros((1, N), device="cuda")
        if bad:
            types[0, 3] = float(T)
        a = _atoms(coords, types, radii, (0, 0, 0), T)
        got = torch.full((1, N, 3), -7.0, device="cuda")
        rc = lib.lmg_backward_static(ctypes.byref(s), ctypes.byref(a), diff.data_ptr(), got.data_ptr(), stream)
        assert rc == 0, lib.lmg_last_error()
        rc = lib.lmg_static_check_status(stream)
        if bad:
            assert rc == _cabi.LMG_ERR_INVALID_ARGUMENT, rc
            assert float(got[0, 3].abs().sum()) == 0.0
        else:
            assert rc == 0, lib.lmg_last_error()


def test_static_backward_refuses_oversized_batches(lib):
    from libmolgrid_b200 import _cabi
    s = _cabi.GridMakerStruct()
    lib.lmg_gridmaker_init(ctypes.byref(s), 0.5, 11.5, 0, 0, 1.0, 1.0)
    limit = lib.lmg_static_max_atoms()
    a = _cabi.AtomsStruct()
    a.batch, a.max_atoms, a.ntypes = 2, limit // 2 + 1, 4
    a.coords = a.radii = a.type_index = 256   # never dereferenced: the size check comes first
    rc = lib.lmg_backward_static(ctypes.byref(s), ctypes.byref(a), 256, 256, None)
    assert rc == _cabi.LMG_ERR_WORKSPACE
    assert b"at most" in lib.lmg_last_error()
