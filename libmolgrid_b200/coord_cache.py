"""Readers for the pre-typed atom files that feed the gridding path, and a sequential provider.

* ``.gninatypes``: a bare array of 16-byte records {float x, y, z; int type}
  (src/coord_cache.cpp:124-147).
* ``.molcache2``: int -1, the 8-byte offset of the name index, then per molecule an unsigned atom
  count followed by such records; the index holds (1-byte length, name, 8-byte offset) entries
  (src/coord_cache.cpp:31-76, 82-118).
* ``.types`` example lists: per line the labels, then the files of the example's coordinate sets
  (src/example.cpp:307-352).

Atoms whose mapped type is negative are dropped, as in the reference.  Records are decoded with
vectorised numpy on the host; the result is a CoordinateSet whose arrays go to the GPU in one copy.
Shuffling, balancing, stratification and molecule parsing (OpenBabel) are not part of this path.
"""
import os

import numpy as np

from .atom_typing import default_ligand_typer, default_receptor_typer
from .coordinates import CoordinateSet, Example, ExampleVec

RECORD = np.dtype([("x", "<f4"), ("y", "<f4"), ("z", "<f4"), ("type", "<i4")])


def coordinate_set_from_records(rec, typer, src=None):
    """CoordinateSet of the records whose mapped type is >= 0, in file order."""
    t, r = typer.map_types(rec["type"])
    keep = t >= 0
    coords = np.stack([rec["x"], rec["y"], rec["z"]], axis=1)[keep].astype(np.float32)
    c = CoordinateSet(np.ascontiguousarray(coords), t[keep].astype(np.float32),
                      np.asarray(r, dtype=np.float32)[keep], typer.num_types())
    c.src = src
    return c


def read_gninatypes(path, typer=None):
    """CoordinateSet from a .gninatypes file (trailing bytes short of a record are ignored)."""
    typer = typer or default_ligand_typer()
    try:
        raw = np.fromfile(path, dtype=np.uint8)
    except OSError:
        raise ValueError("Could not read " + str(path))
    n = raw.size // RECORD.itemsize
    return coordinate_set_from_records(raw[:n * RECORD.itemsize].view(RECORD), typer, src=str(path))


def write_gninatypes(path, coords, types):
    """Writes records in the .gninatypes layout (used by tests and for preparing inputs)."""
    rec = np.zeros(len(types), dtype=RECORD)
    c = np.asarray(coords, dtype=np.float32).reshape(-1, 3)
    rec["x"], rec["y"], rec["z"] = c[:, 0], c[:, 1], c[:, 2]
    rec["type"] = np.asarray(types, dtype=np.int32)
    rec.tofile(path)


class MolCache2(object):
    """Random access to the molecules of a .molcache2 file through a memory map."""

    def __init__(self, path):
        self.path = str(path)
        try:
            self.map = np.memmap(self.path, dtype=np.uint8, mode="r")
        except (OSError, ValueError):
            raise ValueError("Could not open file: " + self.path)
        if self.map.size < 12 or int(self.map[:4].view("<i4")[0]) != -1:
            raise ValueError(self.path + " is not a valid molcache2 file")
        start = int(self.map[4:12].view("<u8")[0])
        self.offsets = {}
        pos = start
        while pos < self.map.size:
            ln = int(self.map[pos])
            name = bytes(self.map[pos + 1:pos + 1 + ln]).decode()
            off = int(np.frombuffer(bytes(self.map[pos + 1 + ln:pos + 9 + ln]), dtype="<u8")[0])
            self.offsets[name] = off
            pos += 9 + ln

    def __contains__(self, name):
        return name in self.offsets

    def records(self, name):
        off = self.offsets[name]
        n = int(np.frombuffer(bytes(self.map[off:off + 4]), dtype="<u4")[0])
        return np.frombuffer(bytes(self.map[off + 4:off + 4 + n * RECORD.itemsize]), dtype=RECORD)


def write_molcache2(path, mols):
    """Writes {name: (coords, types)} in the .molcache2 layout."""
    body, offsets = bytearray(), {}
    for name, (coords, types) in mols.items():
        offsets[name] = 12 + len(body)
        rec = np.zeros(len(types), dtype=RECORD)
        c = np.asarray(coords, dtype=np.float32).reshape(-1, 3)
        rec["x"], rec["y"], rec["z"], rec["type"] = c[:, 0], c[:, 1], c[:, 2], np.asarray(types, np.int32)
        body += np.uint32(len(types)).tobytes() + rec.tobytes()
    with open(path, "wb") as f:
        f.write(np.int32(-1).tobytes() + np.uint64(12 + len(body)).tobytes() + bytes(body))
        for name, off in offsets.items():
            b = name.encode()
            f.write(bytes([len(b)]) + b + np.uint64(off).tobytes())


class CoordCache(object):
    """File name -> CoordinateSet with one typer (src/coord_cache.cpp:82-200 for pre-typed input)."""

    def __init__(self, typer=None, data_root="", molcache=""):
        self.typer = typer or default_ligand_typer()
        self.data_root = data_root
        self.cache = None
        if molcache:
            if not os.path.exists(molcache):
                molcache = os.path.join(data_root, molcache)
            self.cache = MolCache2(molcache)

    def num_types(self):
        return self.typer.num_types()

    def get_type_names(self):
        return self.typer.get_type_names()

    def make_coords(self, fname):
        if self.cache is not None and fname in self.cache:
            return coordinate_set_from_records(self.cache.records(fname), self.typer, src=fname)
        if fname.endswith("none"):  # reserved word: an empty set
            c = CoordinateSet()
            c.max_type = self.typer.num_types()
            return c
        if not fname.endswith(".gninatypes"):
            raise ValueError("Only pre-typed input (.gninatypes, .molcache2) is read here: " + fname)
        full = fname if os.path.isabs(fname) or not self.data_root else os.path.join(self.data_root, fname)
        c = read_gninatypes(full, self.typer)
        c.src = fname
        return c

    def set_coords(self, fname, cset):
        c = self.make_coords(fname)
        cset.coords, cset.type_index, cset.type_vector = c.coords, c.type_index, c.type_vector
        cset.radii, cset.max_type, cset.src = c.radii, c.max_type, c.src


def _is_numeric(tok):
    try:
        float(tok)
        return True
    except ValueError:
        return False


class ExampleRef(object):
    """One line of an example list: labels then file names (src/example.cpp:307-352)."""

    def __init__(self, line, numlabels=-1, hasgroup=False):
        tokens = line.split("#", 1)[0].split()
        if numlabels < 0:
            numlabels = 0
            while numlabels < len(tokens) and _is_numeric(tokens[numlabels]):
                numlabels += 1
            if hasgroup:
                numlabels -= 1
        self.group = -1
        if hasgroup:
            self.group = int(float(tokens[0]))
            tokens = tokens[1:]
        self.labels = [float(t) for t in tokens[:numlabels]]
        self.files = tokens[numlabels:]
        if not self.files:
            raise ValueError("Missing molecular data in line: " + line)


class ExampleProvider(object):
    """Examples in file order: ``populate`` reads example lists, ``next``/``next_batch`` walk them
    cyclically.  The typers apply to the files of a line in order, the last one repeating
    (src/example_extractor.cpp:21-37); the defaults are the receptor and ligand groupings."""

    def __init__(self, *typers, data_root="", recmolcache="", ligmolcache="", num_labels=-1):
        if not typers:
            typers = (default_receptor_typer(), default_ligand_typer())
        caches = [recmolcache, ligmolcache]
        self.caches = [CoordCache(t, data_root, caches[i] if i < 2 else "") for i, t in enumerate(typers)]
        self.refs = []
        self.pos = 0
        self._num_labels = num_labels

    def populate(self, fname, num_labels=-1):
        names = [fname] if isinstance(fname, str) else list(fname)
        nl = num_labels if num_labels >= 0 else self._num_labels
        for name in names:
            with open(name) as f:
                for line in f:
                    if line.strip():
                        self.refs.append(ExampleRef(line, nl))
        if not self.refs:
            raise ValueError("No valid examples found in training set.")

    def size(self):
        return len(self.refs)

    def num_labels(self):
        return len(self.refs[0].labels) if self.refs else 0

    def num_types(self):
        """Channels of a gridded example: one block of types per coordinate set of a line."""
        n = len(self.refs[0].files) if self.refs else len(self.caches)
        return sum(self.caches[min(i, len(self.caches) - 1)].num_types() for i in range(n))

    def get_type_names(self):
        out = []
        for i, c in enumerate(self.caches):
            out += ["%d_%s" % (i, n) for n in c.get_type_names()] if len(self.caches) > 1 else c.get_type_names()
        return out

    def reset(self):
        self.pos = 0

    def _make(self, ref):
        ex = Example()
        ex.labels = list(ref.labels)
        ex.group = ref.group
        for i, fname in enumerate(ref.files):
            ex.coord_sets.append(self.caches[min(i, len(self.caches) - 1)].make_coords(fname))
        return ex

    def next(self):
        if not self.refs:
            raise RuntimeError("No examples: populate() first")
        ex = self._make(self.refs[self.pos])
        self.pos = (self.pos + 1) % len(self.refs)
        return ex

    def next_batch(self, batch_size):
        return ExampleVec([self.next() for _ in range(int(batch_size))])
