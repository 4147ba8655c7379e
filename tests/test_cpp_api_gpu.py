"""The C++ host layer (libmolgrid_b200/cpp/include/libmolgrid/*.h): compile a program against it,
run it on the GPU and compare every array it produces with the CPU oracle."""
import os
import subprocess

import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def center_f32(coords):
    """CoordinateSet::center as the reference computes it: float accumulation in atom order."""
    s = np.zeros(3, np.float32)
    for row in coords:
        s = (s + row.astype(np.float32)).astype(np.float32)
    return (s / np.float32(len(coords))).astype(np.float32)


def test_cpp_layer_against_oracle(port, lib, tmp_path):
    exe = str(tmp_path / "test_cpp_api")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++14", "-O1", "-ffp-contract=off",
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "libmolgrid_b200", "cpp", "include"),
           "-I", os.path.join(cuda, "include"), os.path.join(ROOT, "tests", "cpp", "test_cpp_api.cpp"),
           "-L", os.path.join(ROOT, "libmolgrid_b200"), "-llmg_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart",
           "-Wl,-rpath," + os.path.join(ROOT, "libmolgrid_b200"), "-Wl,-rpath," + os.path.join(cuda, "lib64"),
           "-o", exe]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr

    N, T, NL, K, D = 150, 5, 40, 3, 24
    coords, types, radii = cases.index_case(61, N, T, 6.5)
    lcoords, ltypes, lradii = cases.index_case(62, NL, T, 3.0, ties=False)
    rng = np.random.default_rng(63)
    q = cases.random_quaternion(rng, 1)[0]
    tr = np.concatenate([q, [0.2, -0.1, 0.3], rng.uniform(-1, 1, 3)]).astype(np.float32)
    diff = rng.normal(size=(T, D, D, D)).astype(np.float32)
    ingrid = rng.uniform(size=(K, D, D, D)).astype(np.float32)
    inp, outp = str(tmp_path / "in.bin"), str(tmp_path / "out.bin")
    with open(inp, "wb") as f:
        np.array([N, T, NL, K], np.int32).tofile(f)
        for a in (coords, types, radii, lcoords, ltypes, lradii, tr, diff, ingrid):
            np.ascontiguousarray(a, np.float32).tofile(f)
    res = subprocess.run([exe, inp, outp], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "all checks passed" in res.stdout

    raw = np.fromfile(outp, np.float32)
    pos = [0]

    def take(*shape):
        n = int(np.prod(shape))
        a = raw[pos[0]:pos[0] + n].reshape(shape)
        pos[0] += n
        return a

    gm = port.gm(0.5, 11.5)
    center = (0.1, -0.2, 0.3)
    dens = dict(rtol=1e-5, atol=1e-6)
    # 1. forward
    assert np.allclose(take(T, D, D, D), port.forward_index(gm, center, coords, types, radii, T), **dens)
    # 3. backward
    want = port.backward_index(gm, center, coords, types, radii, diff)
    assert np.allclose(take(N, 3), want, rtol=1e-4, atol=1e-5 * max(1, np.abs(want).max()))
    # 4. Example + Transform: types of the second set are shifted past the first set's
    mcoords = np.concatenate([coords, lcoords])
    mtypes = np.concatenate([types, ltypes + T])
    mradii = np.concatenate([radii, lradii])
    moved = port.transform_forward(tr, mcoords)
    assert np.allclose(take(2 * T, D, D, D), port.forward_index(gm, tr[4:7], moved, mtypes, mradii, 2 * T), **dens)
    # 5. batched examples, identity transforms, centre of each example's last set
    got = take(2, 2 * T, D, D, D)
    c0 = center_f32(lcoords)
    assert np.allclose(got[0], port.forward_index(gm, c0, mcoords, mtypes, mradii, 2 * T), **dens)
    c1 = center_f32(coords)
    m1 = np.concatenate([coords, coords]), np.concatenate([types, types + T]), np.concatenate([radii, radii])
    assert np.allclose(got[1], port.forward_index(gm, c1, m1[0], m1[1], m1[2], 2 * T), **dens)
    assert np.array_equal(take(3), c0)
    # 6. transform and quaternion arithmetic are bit-exact
    assert np.array_equal(take(N, 3), port.transform_forward(tr, coords))
    assert np.array_equal(take(15), port.quaternion_ops(q, [0.5, -0.25, 0.75, 1.5], coords[0]))
    # 7. interpolation
    assert np.array_equal(take(K, D, D, D), port.interpolate([0.5, 11.5, 0.5, 11.5], tr[4:7], ingrid, tr, tr[4:7]))
    assert pos[0] == raw.size
