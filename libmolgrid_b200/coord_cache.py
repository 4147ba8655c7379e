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
The order of the examples (shuffling, balancing, stratification, grouping) follows the reference's
settings (``example_order``); molecule parsing (OpenBabel) is not part of this path.
"""
import ctypes
import threading
import os

import numpy as np
import torch

from . import _cabi
from .atom_typing import default_ligand_typer, default_receptor_typer
from .coordinates import CoordinateSet, Example, ExampleVec
from .example_order import ExampleProviderSettings, IterationScheme, Uniform, create_provider

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
        self._raw = {}
        if molcache:
            if not os.path.exists(molcache):
                molcache = os.path.join(data_root, molcache)
            self.cache = MolCache2(molcache)

    def num_types(self):
        return self.typer.num_types()

    def get_type_names(self):
        return self.typer.get_type_names()

    def records(self, fname):
        """The raw records of ``fname`` (kept in memory after the first read)."""
        rec = self._raw.get(fname)
        if rec is None:
            if self.cache is not None and fname in self.cache:
                rec = self.cache.records(fname)
            elif fname.endswith("none"):
                rec = np.zeros(0, dtype=RECORD)
            elif fname.endswith(".gninatypes"):
                full = fname if os.path.isabs(fname) or not self.data_root else os.path.join(self.data_root, fname)
                try:
                    raw = np.fromfile(full, dtype=np.uint8)
                except OSError:
                    raise ValueError("Could not read " + full)
                rec = raw[:raw.size // RECORD.itemsize * RECORD.itemsize].view(RECORD)
            else:
                raise ValueError("Only pre-typed input (.gninatypes, .molcache2) is read here: " + fname)
            self._raw[fname] = rec
        return rec

    def mem_cache_size(self):
        return len(self._raw)

    def save_mem_cache(self, out):
        """Writes the records read so far (name, count, records) to the open binary file ``out``."""
        out.write(np.uint64(len(self._raw)).tobytes())
        for name, rec in self._raw.items():
            b = name.encode()
            out.write(np.uint32(len(b)).tobytes() + b + np.uint64(len(rec)).tobytes())
            out.write(np.ascontiguousarray(rec).tobytes())

    def load_mem_cache(self, inp):
        (n,) = np.frombuffer(inp.read(8), np.uint64)
        for _ in range(int(n)):
            (ln,) = np.frombuffer(inp.read(4), np.uint32)
            name = inp.read(int(ln)).decode()
            (cnt,) = np.frombuffer(inp.read(8), np.uint64)
            self._raw[name] = np.frombuffer(inp.read(int(cnt) * RECORD.itemsize), dtype=RECORD).copy()

    def tables(self):
        """(channel or -1, radius) for the record type numbers 0..27, as the device decoder wants them."""
        t, r = self.typer.map_types(np.arange(_cabi.RECORD_TYPES))
        return np.asarray(t, dtype=np.int32), np.asarray(r, dtype=np.float32)

    def make_coords(self, fname):
        if fname.endswith("none") and not (self.cache is not None and fname in self.cache):
            c = CoordinateSet()  # reserved word: an empty set
            c.max_type = self.typer.num_types()
            return c
        # through the in-memory records: a structure is read from its file once
        return coordinate_set_from_records(self.records(fname), self.typer, src=fname)

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


_SET_TABLE = np.dtype([("first", "<i8"), ("count", "<i4"), ("example", "<i4"), ("typer", "<i4"),
                       ("toff", "<i4"), ("dst", "<i4"), ("center", "<i4")])   # = lmg_record_set


class DeviceBatch(object):
    """A batch assembled on the GPU by ``ExampleProvider.next_device_batch``: padded
    ``coords (B,N,3)``, ``type_index (B,N)`` (-1 for atoms the typer does not map), ``radii (B,N)``,
    ``n_atoms (B)``, the default grid ``centers (B,3)`` and ``labels (B,L)``.  ``GridMaker.forward``
    and ``GridMaker.backward`` take it in place of a list of Examples."""

    def __init__(self, coords, type_index, radii, n_atoms, centers, labels, num_types, keep):
        self.coords, self.type_index, self.radii = coords, type_index, radii
        self.n_atoms, self.centers, self.labels = n_atoms, centers, labels
        self._num_types = num_types
        self._keep = keep  # staging buffers of this batch

    def __len__(self):
        return int(self.coords.shape[0])

    def num_types(self):
        return self._num_types

    def check(self):
        """Waits for the batch's assembly and raises if the decoder refused atoms (a coordinate set
        of the table did not fit the padded arrays).  Not called on the hot path: it synchronises."""
        status = self._keep[1]
        if int(status.item()) != 0:
            raise RuntimeError("batch assembly dropped atoms: a coordinate set does not fit max_atoms")
        return self


class ExampleProvider(object):
    """Examples from example lists: ``populate`` reads the lists, ``next`` / ``next_batch`` hand the
    examples out in the order the settings ask for (file order by default; ``shuffle``, ``balanced``,
    ``stratify_receptor``, ``stratify_min/max/step``, ``max_group_size`` as in the reference,
    src/example_provider.cpp:103-213).  The typers apply to the files of a line in order, the last
    one repeating (src/example_extractor.cpp:21-37); the defaults are the receptor and ligand
    groupings.  ``seed`` seeds the shuffles of this provider."""

    def __init__(self, *typers, num_labels=-1, seed=0, **settings):
        if typers and isinstance(typers[0], ExampleProviderSettings):
            self.settings, typers = typers[0], typers[1:]
            if settings:
                raise TypeError("settings given twice")
        else:
            self.settings = ExampleProviderSettings(**settings)
        st = self.settings
        if not typers:
            typers = (default_receptor_typer(), default_ligand_typer())
        caches = [st.recmolcache, st.ligmolcache]
        self.caches = [CoordCache(t, st.data_root, caches[i] if i < 2 else "") for i, t in enumerate(typers)]
        self.refs = []
        self._rng = np.random.default_rng(seed)
        self._order = create_provider(st, self._rng)
        self._grouped = bool(getattr(self._order, "has_group", False))
        self._pads = {}                  # (files, labels) of a line -> index of its padding frame
        self._last_epoch = 0
        self._num_labels = num_labels
        self._stage = [(None, None), (None, None)]   # two pinned staging buffers (+ "copy done" events)
        self._stage_slot = 0
        self._packs = {}
        self._tables = None
        self._ix = None                  # per-example staging index (see _index)
        self._ix_lock = threading.Lock()

    def populate(self, fname, num_labels=-1):
        names = [fname] if isinstance(fname, str) else list(fname)
        nl = num_labels if num_labels >= 0 else self._num_labels
        for name in names:
            try:
                f = open(name)
            except OSError:
                raise ValueError("Could not open file " + name)
            with f:
                for line in f:
                    if line.strip():
                        ref = ExampleRef(line, nl, self._grouped)
                        self.refs.append(ref)
                        self._order.addref(len(self.refs) - 1, ref)
        if not self.refs:
            raise ValueError("No valid examples found in training set.")
        self._order.setup()
        self._ix = None   # the staging index covers the examples known when it was built

    def size(self):
        return self._order.size()

    def num_labels(self):
        return len(self.refs[0].labels) if self.refs else 0

    def num_types(self):
        """Channels of a gridded example: one block of types per coordinate set of a line."""
        n = len(self.refs[0].files) if self.refs else len(self.caches)
        if self.settings.duplicate_first and n > 2:
            n = 2 * (n - 1)   # the first set again before every further one (count_types, :59-74)
            return sum(self.caches[0].num_types() if i % 2 == 0 else
                       self.caches[min(i // 2 + 1, len(self.caches) - 1)].num_types() for i in range(n))
        return sum(self.caches[min(i, len(self.caches) - 1)].num_types() for i in range(n))

    def get_type_names(self):
        out = []
        for i, c in enumerate(self.caches):
            out += ["%d_%s" % (i, n) for n in c.get_type_names()] if len(self.caches) > 1 else c.get_type_names()
        return out

    def reset(self):
        self._order.reset()
        self._last_epoch = 0

    def small_epoch_size(self):
        return self._order.small_epoch_size()

    def large_epoch_size(self):
        return self._order.large_epoch_size()

    def get_small_epoch_num(self):
        return self._order.get_small_epoch_num()

    def get_large_epoch_num(self):
        return self._order.get_large_epoch_num()

    def skip(self, n):
        for _ in range(int(n)):
            self._order.nextref()

    def mem_caches_size(self):
        """Coordinate sets held in memory (src/example_extractor.cpp:104-110)."""
        return sum(c.mem_cache_size() for c in self.caches)

    def save_mem_caches(self, fname):
        """Writes the structures read so far to ``fname``, one block per typer in order; a later
        ``load_mem_caches`` serves them without the structure files (include/libmolgrid/
        example_provider.h:166-193).  The layout is this library's own (records as read, before
        typing), not the reference's serialisation."""
        with open(fname, "wb") as f:
            for c in self.caches:
                c.save_mem_cache(f)

    def load_mem_caches(self, fname):
        with open(fname, "rb") as f:
            for c in self.caches:
                c.load_mem_cache(f)

    def at_new_epoch(self):
        """True once per epoch of the configured iteration scheme, when the next example belongs to a
        new epoch (include/libmolgrid/example_provider.h:135-152)."""
        sch = self.settings.iteration_scheme
        if sch == IterationScheme.LargeEpoch:
            e = self._order.get_large_epoch_num()
        elif sch == IterationScheme.SmallEpoch:
            e = self._order.get_small_epoch_num()
        else:
            return False
        if e != self._last_epoch:
            self._last_epoch = e
            return True
        return False

    def __iter__(self):
        return self

    def __next__(self):
        """Batches of ``default_batch_size`` until the epoch ends (never with the continuous scheme)."""
        if self.at_new_epoch():
            raise StopIteration("End of epoch.")
        return self.next_batch()

    @property
    def pos(self):
        """Position in the list while it is walked in file order."""
        return getattr(self._order, "current", 0)

    def _files(self, ref):
        """(file, typer index) of the coordinate sets of a line: the first file again before every
        further one with ``duplicate_first`` and three or more files (src/example_extractor.cpp:39-55)."""
        last = len(self.caches) - 1
        if self.settings.duplicate_first and len(ref.files) >= 3:
            out = []
            for i in range(1, len(ref.files)):
                out += [(ref.files[0], 0), (ref.files[i], min(i, last))]
            return out
        return [(f, min(i, last)) for i, f in enumerate(ref.files)]

    def _next_index(self):
        """Index of the next line, with a group's padding frames turned into lines of their own (the
        files of the group's last frame replaced by the empty set, labels NaN)."""
        r = self._order.nextref()
        if not self._grouped:
            return r, None
        i, padded, group, seqcont = r
        if padded:
            ref = self.refs[i]
            key = (len(ref.files), len(ref.labels))
            j = self._pads.get(key)
            if j is None:
                pad = ExampleRef.__new__(ExampleRef)
                pad.group, pad.labels, pad.files = -1, [float("nan")] * key[1], ["none"] * key[0]
                self.refs.append(pad)
                j = self._pads[key] = len(self.refs) - 1
                self._ix = None
            i = j
        return i, (group, seqcont)

    def _make(self, ref):
        ex = Example()
        ex.labels = list(ref.labels)
        ex.group = ref.group
        for fname, ci in self._files(ref):
            c = self.caches[ci].make_coords(fname)
            if self.settings.make_vector_types and c.has_indexed_types():
                c.make_vector_types(False, self.caches[ci].typer.get_type_radii())
            ex.coord_sets.append(c)
        return ex

    def next(self):
        if not self.refs:
            raise RuntimeError("No examples: populate() first")
        i, frame = self._next_index()
        ex = self._make(self.refs[i])
        if frame is not None:
            ex.group, ex.seqcont = frame
        return ex

    def next_batch(self, batch_size=0):
        B = int(batch_size) or int(self.settings.default_batch_size)
        if hasattr(self._order, "check_batch_size"):
            self._order.check_batch_size(B)
        return ExampleVec([self.next() for _ in range(B)])

    def _packed(self, i):
        """Example i ready for staging: the bytes of all its sets' records back to back, and per set
        the record count, typer, type offset and first atom slot (built once per example)."""
        p = self._packs.get(i)
        if p is None:
            ref = self.refs[i]
            recs, counts, typers, toffs, dst = [], [], [], [], []
            toffset = natoms = 0
            for fname, ci in self._files(ref):
                r = self.caches[ci].records(fname)
                recs.append(np.ascontiguousarray(r).view(np.uint8))
                counts.append(len(r)); typers.append(ci); toffs.append(toffset); dst.append(natoms)
                natoms += len(r)
                # a set without atoms after typing does not advance the type offset
                # (Example::merge_coordinates, src/example.cpp:84-96: "ignore empties")
                if len(r) and (np.asarray(self.caches[ci].typer.map_types(r["type"])[0]) >= 0).any():
                    toffset += self.caches[ci].num_types()
            p = (np.concatenate(recs) if recs else np.zeros(0, np.uint8), np.array(counts, np.int32),
                 np.array(typers, np.int32), np.array(toffs, np.int32), np.array(dst, np.int32))
            self._packs[i] = p
        return p

    def _take(self, batch_size):
        """Indices of the next ``batch_size`` examples."""
        if not self.refs:
            raise RuntimeError("No examples: populate() first")
        if self.settings.make_vector_types:
            raise ValueError("device batches carry index types; make_vector_types applies to next()/next_batch()")
        B = int(batch_size) or int(self.settings.default_batch_size)
        if hasattr(self._order, "check_batch_size"):
            self._order.check_batch_size(B)
        return [self._next_index()[0] for _ in range(B)]

    def _index(self, idx):
        """Per-example arrays for staging, built on first use and extended as examples are first
        seen: address and size of each example's packed records, its label row, and its
        coordinate sets in one flat table with a start offset per example."""
        ix = self._ix
        if ix is None:
            n = len(self.refs)
            ix = self._ix = dict(done=np.zeros(n, bool), ptr=np.zeros(n, np.uint64), nbytes=np.zeros(n, np.int64),
                                 nset=np.zeros(n, np.int64), start=np.zeros(n, np.int64),
                                 sets=np.zeros(0, dtype=_SET_TABLE), nlab=np.zeros(n, np.int64), labels=None)
        new = [i for i in set(idx) if not ix["done"][i]]
        if new:
            with self._ix_lock:
                rows = [ix["sets"]]
                at = len(ix["sets"])
                for i in new:
                    if ix["done"][i]:
                        continue
                    rec, counts, typers, toffs, dst = self._packed(i)
                    t = np.zeros(len(counts), dtype=_SET_TABLE)
                    t["count"], t["typer"], t["toff"], t["dst"] = counts, typers, toffs, dst
                    t["first"] = np.concatenate(([0], np.cumsum(counts[:-1]))) if len(counts) else 0
                    if len(counts):
                        t["center"][-1] = 1
                    rows.append(t)
                    ix["ptr"][i], ix["nbytes"][i] = rec.ctypes.data, rec.size
                    ix["nset"][i], ix["start"][i] = len(counts), at
                    at += len(counts)
                    lab = np.asarray(list(self.refs[i].labels), np.float32)
                    ix["nlab"][i] = lab.size
                    if ix["labels"] is None:
                        ix["labels"] = np.zeros((len(self.refs), lab.size), np.float32)
                    ix["labels"][i, :min(lab.size, ix["labels"].shape[1])] = lab[:ix["labels"].shape[1]]
                ix["sets"] = np.concatenate(rows)
                ix["done"][new] = True
        return ix

    def _assemble(self, idx, slot):
        """Host half of a device batch (no CUDA work besides waiting for the staging buffer): the raw
        records of the examples ``idx``, their set table, atom counts, typer tables and labels, laid
        out in the pinned buffer of staging slot ``slot``.  Safe to run on a worker thread; the copy
        of the records runs in native code without the interpreter lock."""
        B = len(idx)
        ix = self._index(idx)
        ia = np.asarray(idx, np.int64)
        nl = int(ix["nlab"][ia[0]])
        if (ix["nlab"][ia] != nl).any():
            raise ValueError("examples of one batch carry different numbers of labels: %s vs %d"
                             % (sorted(set(int(v) for v in ix["nlab"][ia])), nl))
        # the batch's set table: the cached rows of its examples, re-based
        nset = ix["nset"][ia]
        nsets = int(nset.sum())
        ends = np.cumsum(nset)
        flat = np.arange(nsets) - np.repeat(ends - nset, nset) + np.repeat(ix["start"][ia], nset)
        table = ix["sets"][flat]
        nbytes = ix["nbytes"][ia]
        rec_first = np.concatenate(([0], np.cumsum(nbytes[:-1]))) // RECORD.itemsize
        table["first"] += np.repeat(rec_first, nset)
        table["example"] = np.repeat(np.arange(B), nset)
        n_atoms = (nbytes // RECORD.itemsize).astype(np.int32)
        nmax = max(1, int(n_atoms.max()))
        labels = np.ascontiguousarray(ix["labels"][ia, :nl])
        if self._tables is None:
            tabs = [c.tables() for c in self.caches]
            self._tables = (np.concatenate([t for t, _ in tabs]).astype(np.int32).view(np.uint8),
                            np.concatenate([r for _, r in tabs]).astype(np.float32).view(np.uint8))
        # one pinned blob: records of every example | set table | atom counts | type tables | labels
        small = [table.view(np.uint8), n_atoms.view(np.uint8), self._tables[0], self._tables[1],
                 labels.view(np.uint8).reshape(-1)]
        rec_bytes = int(nbytes.sum())
        offs, total = [0], (rec_bytes + 15) // 16 * 16
        for p in small:
            offs.append(total)
            total += (p.size + 15) // 16 * 16
        host, busy = self._stage[slot]
        if busy is not None:
            busy.synchronize()               # the copy that last read this staging buffer has finished
        if host is None or host.numel() < total:
            host = torch.empty(max(2 * total, 1 << 20), dtype=torch.uint8).pin_memory()
            self._stage[slot] = (host, None)
        ptrs = np.ascontiguousarray(ix["ptr"][ia])
        nb = np.ascontiguousarray(nbytes)
        _cabi.check(_cabi.lib().lmg_gather_host(ctypes.c_void_p(host.data_ptr()), rec_bytes, B,
                                                ctypes.c_void_p(ptrs.ctypes.data), ctypes.c_void_p(nb.ctypes.data)))
        hv = host.numpy()
        for p, o in zip(small, offs[1:]):
            hv[o:o + p.size] = p
        return dict(B=B, nl=nl, nsets=nsets, nmax=nmax, offs=offs, total=total, slot=slot,
                    max_count=int(table["count"].max()) if nsets else 0)

    def _launch(self, m, dev):
        """Device half: one host-to-device copy of the staged blob and the decode kernels, queued
        on the current stream of ``dev``."""
        B, nl, nmax, offs, total, slot = m["B"], m["nl"], m["nmax"], m["offs"], m["total"], m["slot"]
        host = self._stage[slot][0]
        blob = torch.empty(total, dtype=torch.uint8, device=dev)
        blob.copy_(host[:total], non_blocking=True)
        busy = torch.cuda.Event()
        busy.record(torch.cuda.current_stream(dev))
        self._stage[slot] = (host, busy)
        coords = torch.empty((B, nmax, 3), dtype=torch.float32, device=dev)
        types = torch.empty((B, nmax), dtype=torch.float32, device=dev)
        radii = torch.empty((B, nmax), dtype=torch.float32, device=dev)
        centers = torch.empty((B, 3), dtype=torch.float32, device=dev)
        status = torch.empty(1, dtype=torch.int32, device=dev)
        base = blob.data_ptr()
        vp = ctypes.c_void_p
        _cabi.check(_cabi.lib().lmg_decode_records(
            vp(base + offs[0]), vp(base + offs[1]), m["nsets"], vp(base + offs[3]), vp(base + offs[4]), B, nmax,
            m["max_count"], vp(coords.data_ptr()), vp(types.data_ptr()),
            vp(radii.data_ptr()), vp(centers.data_ptr()), None, vp(status.data_ptr()),
            vp(torch.cuda.current_stream(dev).cuda_stream)))
        dn = blob[offs[2]:offs[2] + 4 * B].view(torch.int32)
        lab = blob[offs[5]:offs[5] + 4 * B * nl].view(torch.float32).view(B, nl)
        return DeviceBatch(coords, types, radii, dn, centers, lab, self.num_types(), (blob, status, host))

    @staticmethod
    def _device(device):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this library has no CPU path")
        return torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)

    def next_device_batch(self, batch_size, device=None):
        """The next ``batch_size`` examples as a DeviceBatch.  The raw records of all their files go
        to the GPU in ONE copy from pinned memory together with a table of their coordinate sets; a
        kernel does the type lookup, the merge of each example's sets with type offsets and the
        padding (``lmg_decode_records``).  Work is queued on the current stream of ``device``."""
        dev = self._device(device)
        idx = self._take(batch_size)
        slot = self._stage_slot
        self._stage_slot = (slot + 1) % len(self._stage)
        return self._launch(self._assemble(idx, slot), dev)

    def device_batches(self, batch_size, count=None, device=None, workers=2):
        """Generator of DeviceBatches in example order whose host half runs ahead on ``workers``
        threads: while the GPU grids batch k and the caller issues its kernels, batches k+1.. are
        being laid out in their own pinned buffers (src/example_provider.cpp:70-90 assembles
        batches on the calling thread).  ``count`` batches, or without end."""
        from concurrent.futures import ThreadPoolExecutor
        dev = self._device(device)
        workers = max(1, int(workers))
        depth = workers + 1
        while len(self._stage) < depth + 1:
            self._stage.append((None, None))
        nslots = len(self._stage)
        pending = []
        issued = 0
        with ThreadPoolExecutor(max_workers=workers) as pool:
            def submit():
                nonlocal issued
                slot = self._stage_slot
                self._stage_slot = (slot + 1) % nslots
                pending.append(pool.submit(self._assemble, self._take(batch_size), slot))
                issued += 1
            while (count is None or issued < count) and len(pending) < depth:
                submit()
            while pending:
                m = pending.pop(0).result()
                batch = self._launch(m, dev)
                if count is None or issued < count:
                    submit()
                yield batch


class ExampleDataset(ExampleProvider):
    """Random access to the examples of the lists, for map-style data sets: ``len(d)`` examples,
    ``d[i]`` the i-th line in file order (python/bindings.in.cpp: ExampleDataset; settings that
    concern iteration are ignored)."""

    def __init__(self, *typers, **kw):
        for k in ("shuffle", "balanced", "stratify_receptor", "stratify_min", "stratify_max", "stratify_step",
                  "max_group_size", "group_batch_size", "num_copies"):
            kw.pop(k, None)
        ExampleProvider.__init__(self, *typers, **kw)

    def __len__(self):
        return len(self.refs)

    def __getitem__(self, i):
        n = len(self.refs)
        if not -n <= i < n:
            raise IndexError("Invalid index: %d > %d" % (i, n))
        return self._make(self.refs[i % n])
