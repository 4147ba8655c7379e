"""Seeded synthetic inputs with the shapes and distributions of the benchmark configurations.

Used by bench.py / bench_ops.py (the workloads they time) and by the parity tests (the same inputs
go to the CPU checker and to the GPU)."""
import numpy as np


def sphere(rng, n, radius):
    """n points uniform in a ball."""
    v = rng.normal(size=(n, 3))
    v /= np.linalg.norm(v, axis=1, keepdims=True)
    r = radius * rng.uniform(size=(n, 1)) ** (1.0 / 3)
    return (v * r).astype(np.float32)


def random_quaternion(rng, n):
    q = rng.normal(size=(n, 4))
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    return q.astype(np.float32)


def index_case(seed, n, ntypes, extent, rmin=1.2, rmax=2.2, ties=True):
    """Index-typed atoms; per-type radii; a few atoms exactly on grid points, untyped atoms,
    a fractional type index and a zero radius to exercise the edge rules."""
    rng = np.random.default_rng(seed)
    coords = sphere(rng, n, extent)
    types = rng.integers(0, ntypes, n).astype(np.float32)
    R = rng.uniform(rmin, rmax, ntypes).astype(np.float32)
    radii = R[types.astype(int)].copy()
    if ties and n >= 12:
        coords[:6] = np.round(coords[:6] * 2) / 2 + 0.25
        radii[:6] = 1.0
        types[6] = -1
        types[7] = types[7] % (ntypes - 1) + 0.5  # floor and round give different channels
        radii[8] = 0
    return coords, types, radii


def vector_case(seed, n, ntypes, extent, alpha=0.3, rti=False):
    rng = np.random.default_rng(seed)
    coords = sphere(rng, n, extent)
    tv = rng.dirichlet(np.ones(ntypes) * alpha, n).astype(np.float32)
    tv[tv < 0.02] = 0
    if rti:
        radii = (1.7 * rng.uniform(0.8, 1.2, ntypes)).astype(np.float32)
    else:
        radii = rng.uniform(1.2, 2.2, n).astype(np.float32)
    return coords, tv, radii


def blob_batch(seed, batch, nmin, nmax, ntypes=28, layout_seed=None):
    """The benchmark's batch: 30% of atoms uniform in a 12 A ball, 70% in a 4 A blob whose centre
    is uniform in a 6 A ball; per-type radii U[1.2,2.2]; random rotation and +-2 A translation.

    With ``layout_seed`` the atom counts and the per-type radii come from that seed and only the
    coordinates, types and transforms from ``seed``: batches of equal size for weak scaling.  A batch
    whose two seeds are equal is the batch of ``seed`` alone."""
    rng = np.random.default_rng(seed)
    ns = rng.integers(nmin, nmax + 1, batch)
    if layout_seed is not None:
        ns = np.random.default_rng(layout_seed).integers(nmin, nmax + 1, batch)
    nmaxa = int(ns.max())
    coords = np.zeros((batch, nmaxa, 3), np.float32)
    types = np.zeros((batch, nmaxa), np.float32)
    radii = np.zeros((batch, nmaxa), np.float32)
    R = rng.uniform(1.2, 2.2, ntypes).astype(np.float32)
    if layout_seed is not None:
        lrng = np.random.default_rng(layout_seed)
        lrng.integers(nmin, nmax + 1, batch)
        R = lrng.uniform(1.2, 2.2, ntypes).astype(np.float32)
    for b in range(batch):
        n = int(ns[b])
        nblob = int(0.7 * n)
        c = sphere(rng, 1, 6.0)
        pts = np.concatenate([sphere(rng, n - nblob, 12.0), sphere(rng, nblob, 4.0) + c])
        rng.shuffle(pts)
        coords[b, :n] = pts
        t = rng.integers(0, ntypes, n)
        types[b, :n] = t
        radii[b, :n] = R[t]
    q = random_quaternion(rng, batch)
    tr = np.zeros((batch, 10), np.float32)
    tr[:, :4] = q
    tr[:, 7:] = rng.uniform(-2, 2, (batch, 3))
    return coords, types, radii, ns.astype(np.int32), tr


def dense_vector_batch(seed, batch, n, ntypes=28, alpha=0.3):
    """Vector-typed configuration: n atoms per example placed like the blob batch, a Dirichlet(alpha)
    type vector per atom (entries that underflow to zero stay zero) and one radius per type,
    1.7 A scaled by U[0.8, 1.2] (radii indexed by type)."""
    rng = np.random.default_rng(seed)
    coords = np.zeros((batch, n, 3), np.float32)
    for b in range(batch):
        nblob = int(0.7 * n)
        c = sphere(rng, 1, 6.0)
        pts = np.concatenate([sphere(rng, n - nblob, 12.0), sphere(rng, nblob, 4.0) + c])
        rng.shuffle(pts)
        coords[b] = pts
    tv = rng.dirichlet(np.ones(ntypes) * alpha, (batch, n)).astype(np.float32)
    radii = (1.7 * rng.uniform(0.8, 1.2, (batch, ntypes))).astype(np.float32)
    return coords, tv, radii


# ---- the blob workload example by example (so that a rank can make only its own slice) --------------

def blob_counts(seed, batch, nmin=2000, nmax=4000):
    """Atom counts of the examples of a blob batch."""
    return np.random.default_rng([seed, 0]).integers(nmin, nmax + 1, batch).astype(np.int32)


def type_radii(seed, ntypes=28):
    """One radius per type, U[1.2, 2.2]: a property of the typing scheme, the same for every example."""
    return np.random.default_rng([seed, 1]).uniform(1.2, 2.2, ntypes).astype(np.float32)


def blob_example(seed, index, n, R):
    """Example `index` of the blob workload: n atoms (30 % in a 12 A ball, 70 % in a 4 A blob whose
    centre is uniform in a 6 A ball), types uniform over len(R), radii by type, and the example's
    transform (random unit quaternion, centre 0, translation U[-2,2]^3) as a row of 10 floats."""
    rng = np.random.default_rng([seed, 2, index])
    nblob = int(0.7 * n)
    c = sphere(rng, 1, 6.0)
    pts = np.concatenate([sphere(rng, n - nblob, 12.0), sphere(rng, nblob, 4.0) + c])
    rng.shuffle(pts)
    t = rng.integers(0, len(R), n)
    tr = np.zeros(10, np.float32)
    tr[:4] = random_quaternion(rng, 1)[0]
    tr[7:] = rng.uniform(-2, 2, 3)
    return pts.astype(np.float32), t.astype(np.float32), R[t], tr


def blob_slice(seed, start, end, counts, R):
    """Examples [start, end) of the blob workload as padded arrays (coords, types, radii, n, transforms)."""
    nb = end - start
    nmaxa = int(counts[start:end].max()) if nb else 0
    coords = np.zeros((nb, nmaxa, 3), np.float32)
    types = np.zeros((nb, nmaxa), np.float32)
    radii = np.zeros((nb, nmaxa), np.float32)
    tr = np.zeros((nb, 10), np.float32)
    for i in range(nb):
        n = int(counts[start + i])
        coords[i, :n], types[i, :n], radii[i, :n], tr[i] = blob_example(seed, start + i, n, R)
    return coords, types, radii, counts[start:end].astype(np.int32), tr
