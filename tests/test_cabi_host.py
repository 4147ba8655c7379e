"""Host-only checks of the C ABI library: it loads, exports every symbol include/lmg_b200.h
declares, computes GridMaker's constants and random transforms exactly as the reference does, and
rejects bad arguments before touching a GPU.  No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest

from tests.golden import make_golden as mg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))


def test_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "lmg_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(lmg_[a-z_0-9]+)\s*\(", header))
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(lib, name), name
    from libmolgrid_b200 import _cabi
    assert declared == {n for n, _, _ in _cabi.SYMBOLS}
    assert lib.lmg_version() >= 100
    tuning = open(os.path.join(ROOT, "include", "lmg_b200_tuning.h")).read()
    tuning = re.sub(r"/\*.*?\*/", "", tuning, flags=re.S)
    knobs = set(re.findall(r"\b(lmg_[a-z_0-9]+)\s*\(", tuning))
    assert knobs == {n for n, _, _ in _cabi.EXTRA_SYMBOLS}
    for name in knobs:
        assert hasattr(lib, name), name


def test_struct_layouts_match_header(lib):
    from libmolgrid_b200 import _cabi
    assert ctypes.sizeof(_cabi.GridMakerStruct) == 13 * 4
    assert ctypes.sizeof(_cabi.TransformStruct) == 40
    assert ctypes.sizeof(_cabi.InterpolaterStruct) == 24
    assert ctypes.sizeof(_cabi.RecordSetStruct) == 32
    assert ctypes.sizeof(_cabi.AtomsStruct) == 3 * 4 + 4 + 6 * 8 + 3 * 4 + 4 + 2 * 8


@pytest.mark.parametrize("grm", [1.0, 3.0, -2.0, -1.5, 0.7])
def test_gridmaker_constants_match_reference(lib, port, grm):
    from libmolgrid_b200 import _cabi
    s = _cabi.GridMakerStruct()
    assert lib.lmg_gridmaker_init(ctypes.byref(s), 0.5, 23.5, 0, 0, 1.0, grm) == 0
    want = port.consts(port.gm(0.5, 23.5, False, False, 1.0, grm))
    got = np.array([s.A, s.B, s.C, s.D, s.E, s.final_radius_multiple, s.dim, s.gaussian_radius_multiple],
                   np.float32)
    assert np.array_equal(got, want)
    assert s.dim == 48


def test_gridmaker_constants_match_golden(lib):
    from libmolgrid_b200 import _cabi
    for name, kw in mg.SETTINGS.items():
        s = _cabi.GridMakerStruct()
        lib.lmg_gridmaker_init(ctypes.byref(s), kw["resolution"], kw["dimension"], int(kw.get("binary", False)), 0,
                               kw.get("radius_scale", 1.0), kw.get("gaussian_radius_multiple", 1.0))
        got = np.array([s.A, s.B, s.C, s.D, s.E, s.final_radius_multiple, s.dim, s.gaussian_radius_multiple],
                       np.float32)
        assert np.array_equal(got, GOLD[name + "/consts"]), name


def test_random_transform_sequence_matches_reference(lib):
    """Seeded draws reproduce the reference's Transform(center, translate, rotate) constructor."""
    import libmolgrid_b200 as lmg
    lmg.set_random_seed(1234)
    want = GOLD["random/rot"]
    for i in range(want.shape[0]):
        t = lmg.Transform((1, 2, 3), 2.5, True)
        assert np.array_equal(np.array(t.as_row(), np.float32), want[i])
    lmg.set_random_seed(99)
    want = GOLD["random/norot"]
    for i in range(want.shape[0]):
        t = lmg.Transform(lmg.float3(0, 0, 0), random_translate=1.0)
        assert np.array_equal(np.array(t.as_row(), np.float32), want[i])
        assert t.get_quaternion() == lmg.Quaternion()


def test_python_quaternion_matches_reference():
    import libmolgrid_b200 as lmg
    q, q2, c, t, pts, grid = mg.transform_inputs()
    a, b = lmg.Quaternion(*q), lmg.Quaternion(*q2)
    got = []
    for r in (a * b, a / b, a.inverse()):
        got += [r.R_component_1(), r.R_component_2(), r.R_component_3(), r.R_component_4()]
    got += list(a.rotate(*pts[0]))
    assert np.array_equal(np.array(got, np.float32), GOLD["quat/ops"])
    want = GOLD["transform/nonunit/forward1"][0]
    assert np.array_equal(np.array(list(a.transform(*pts[0], c, t)), np.float32), want)


def test_argument_errors_need_no_gpu(lib):
    from libmolgrid_b200 import _cabi
    s = _cabi.GridMakerStruct()
    lib.lmg_gridmaker_init(ctypes.byref(s), 0.5, 23.5, 0, 1, 1.0, 1.0)
    a = _cabi.AtomsStruct()
    a.batch, a.max_atoms, a.ntypes = 1, 4, 2
    a.coords = a.radii = a.type_index = 16  # never dereferenced: the call fails before any launch
    ws = ctypes.c_void_p(16)
    rc = lib.lmg_forward(ctypes.byref(s), ctypes.byref(a), ws, ws, 1 << 20, None)
    assert rc == _cabi.LMG_ERR_INVALID_ARGUMENT   # type-indexed radii with index types
    assert b"Type indexed radii" in lib.lmg_last_error()
    s.radii_type_indexed = 0
    assert lib.lmg_forward(ctypes.byref(s), ctypes.byref(a), ws, None, 0, None) == _cabi.LMG_ERR_WORKSPACE
    a.ntypes = 0
    assert lib.lmg_forward(ctypes.byref(s), ctypes.byref(a), ws, ws, 1 << 20, None) == _cabi.LMG_ERR_INVALID_ARGUMENT
    assert lib.lmg_workspace_bytes(ctypes.byref(s), 0, 50, 4000, 28, 0) > 50 * 4000 * 64
    with pytest.raises(ValueError):
        _cabi.check(_cabi.LMG_ERR_INVALID_ARGUMENT)
    with pytest.raises(IndexError):
        _cabi.check(_cabi.LMG_ERR_OUT_OF_RANGE)


def test_no_cpu_fallback():
    """Without a CUDA device the Python layer refuses to run rather than compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import libmolgrid_b200 as lmg
    g = lmg.GridMaker()
    with pytest.raises(RuntimeError):
        g.forward((0, 0, 0), torch.zeros(1, 3), torch.zeros(1), torch.ones(1), torch.zeros(1, 48, 48, 48))
