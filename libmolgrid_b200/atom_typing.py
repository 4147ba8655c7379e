"""Atom typing for pre-typed input (.gninatypes records, .molcache2 files).

The gridding path consumes (coordinates, type index, radius) triples.  On disk the reference keeps
atoms as 16-byte records {float x, y, z; int type} with ``type`` a gnina/smina atom type
(include/libmolgrid/atom_typer.h:125-156); a typer turns that integer into a channel index and a
radius (src/atom_typer.cpp:167-178, include/libmolgrid/atom_typer.h:363-368).  Typing molecules from
chemistry files needs OpenBabel and is outside this path.
"""
import os

import numpy as np

# (name, covalent radius, XS radius) in the order of GninaIndexTyper::type
# (src/atom_typer.cpp:33-64; the other legacy columns of that table are not used for gridding)
GNINA_TYPES = [
    ("Hydrogen", 0.37, 0.37),
    ("PolarHydrogen", 0.37, 0.37),
    ("AliphaticCarbonXSHydrophobe", 0.77, 1.9),
    ("AliphaticCarbonXSNonHydrophobe", 0.77, 1.9),
    ("AromaticCarbonXSHydrophobe", 0.77, 1.9),
    ("AromaticCarbonXSNonHydrophobe", 0.77, 1.9),
    ("Nitrogen", 0.75, 1.8),
    ("NitrogenXSDonor", 0.75, 1.8),
    ("NitrogenXSDonorAcceptor", 0.75, 1.8),
    ("NitrogenXSAcceptor", 0.75, 1.8),
    ("Oxygen", 0.73, 1.7),
    ("OxygenXSDonor", 0.73, 1.7),
    ("OxygenXSDonorAcceptor", 0.73, 1.7),
    ("OxygenXSAcceptor", 0.73, 1.7),
    ("Sulfur", 1.02, 2.0),
    ("SulfurAcceptor", 1.02, 2.0),
    ("Phosphorus", 1.06, 2.1),
    ("Fluorine", 0.71, 1.5),
    ("Chlorine", 0.99, 1.8),
    ("Bromine", 1.14, 2.0),
    ("Iodine", 1.33, 2.2),
    ("Magnesium", 1.30, 1.2),
    ("Manganese", 1.39, 1.2),
    ("Zinc", 1.31, 1.2),
    ("Calcium", 1.74, 1.2),
    ("Iron", 1.25, 1.2),
    ("GenericMetal", 1.75, 1.2),
    ("Boron", 0.90, 1.92),
]
GENERIC_METAL = 26


class GninaIndexTyper(object):
    """The 28 gnina atom types with their radii; ``get_int_type`` is the lookup used for pre-typed
    records (src/atom_typer.cpp:167-178): unknown type numbers become GenericMetal."""

    NumTypes = len(GNINA_TYPES)

    def __init__(self, use_covalent_radius=False):
        self.use_covalent = bool(use_covalent_radius)
        col = 1 if self.use_covalent else 2
        self._radii = np.array([t[col] for t in GNINA_TYPES], dtype=np.float32)

    def num_types(self):
        return self.NumTypes

    def get_type_names(self):
        return [t[0] for t in GNINA_TYPES]

    def get_type_radii(self):
        return [float(r) for r in self._radii]

    def get_int_type(self, t):
        t = int(t) if int(t) < self.NumTypes else GENERIC_METAL
        return t, float(self._radii[t])

    def is_vector_typer(self):
        return False

    def map_types(self, raw):
        """Vectorised get_int_type: (channel index or -1, radius) arrays for raw type numbers."""
        raw = np.asarray(raw, dtype=np.int64)
        t = np.where(raw < self.NumTypes, raw, GENERIC_METAL)
        return t.astype(np.int64), self._radii[t]


class FileAtomMapper(object):
    """Groups of old type names, one group per non-blank line, become the new types
    (src/atom_typer.cpp:419-475)."""

    def __init__(self, lines, old_type_names):
        if isinstance(lines, str):
            lines = lines.splitlines()
        old = {name: i for i, name in enumerate(old_type_names)}
        self.old_to_new = np.full(len(old_type_names), -1, dtype=np.int64)
        self.new_type_names = []
        for line in lines:
            names = line.split()
            if not names:
                continue
            nt = len(self.new_type_names)
            self.new_type_names.append("_".join(names))
            for name in names:
                if name not in old:
                    raise ValueError("Invalid atom type " + name)
                self.old_to_new[old[name]] = nt

    @classmethod
    def from_file(cls, fname, old_type_names):
        try:
            with open(fname) as f:
                return cls(f.read(), old_type_names)
        except OSError:
            raise ValueError("Could not open " + fname)

    def num_types(self):
        return len(self.new_type_names)

    def get_new_type(self, origt):
        return int(self.old_to_new[origt]) if 0 <= origt < len(self.old_to_new) else -1

    def get_type_names(self):
        return list(self.new_type_names)


class FileMappedGninaTyper(object):
    """GninaIndexTyper followed by a FileAtomMapper (include/libmolgrid/atom_typer.h:300-378): the
    channel is the mapped type, the radius stays that of the original gnina type."""

    def __init__(self, mapping, use_covalent_radius=False):
        self.typer = GninaIndexTyper(use_covalent_radius)
        names = self.typer.get_type_names()
        if isinstance(mapping, FileAtomMapper):
            self.mapper = mapping
        elif isinstance(mapping, str) and os.path.isfile(mapping):
            self.mapper = FileAtomMapper.from_file(mapping, names)
        else:
            self.mapper = FileAtomMapper(mapping, names)
        # per new type: mean radius of the old types it collects
        n = self.mapper.num_types()
        sums, counts = np.zeros(n), np.zeros(n)
        for ot in range(self.typer.num_types()):
            nt = self.mapper.get_new_type(ot)
            if nt >= 0:
                sums[nt] += self.typer.get_int_type(ot)[1]
                counts[nt] += 1
        self.type_radii = [float(s / c) if c else 0.0 for s, c in zip(sums, counts)]

    def num_types(self):
        return self.mapper.num_types()

    def get_type_names(self):
        return self.mapper.get_type_names()

    def get_type_radii(self):
        return list(self.type_radii)

    def is_vector_typer(self):
        return False

    def get_int_type(self, t):
        ot, r = self.typer.get_int_type(t)
        return self.mapper.get_new_type(ot), r

    def map_types(self, raw):
        ot, r = self.typer.map_types(raw)
        return self.mapper.old_to_new[ot], r


# the receptor and ligand groupings the reference builds in (src/atom_typer.cpp:530-562)
DEFAULT_RECMAP = """AliphaticCarbonXSHydrophobe
AliphaticCarbonXSNonHydrophobe
AromaticCarbonXSHydrophobe
AromaticCarbonXSNonHydrophobe
Bromine Iodine Chlorine Fluorine
Nitrogen NitrogenXSAcceptor
NitrogenXSDonor NitrogenXSDonorAcceptor
Oxygen OxygenXSAcceptor
OxygenXSDonorAcceptor OxygenXSDonor
Sulfur SulfurAcceptor
Phosphorus
Calcium
Zinc
GenericMetal Boron Manganese Magnesium Iron
"""
DEFAULT_LIGMAP = """AliphaticCarbonXSHydrophobe
AliphaticCarbonXSNonHydrophobe
AromaticCarbonXSHydrophobe
AromaticCarbonXSNonHydrophobe
Bromine Iodine
Chlorine
Fluorine
Nitrogen NitrogenXSAcceptor
NitrogenXSDonor NitrogenXSDonorAcceptor
Oxygen OxygenXSAcceptor
OxygenXSDonorAcceptor OxygenXSDonor
Sulfur SulfurAcceptor
Phosphorus
GenericMetal Boron Manganese Magnesium Zinc Calcium Iron
"""


def default_receptor_typer():
    return FileMappedGninaTyper(DEFAULT_RECMAP)


def default_ligand_typer():
    return FileMappedGninaTyper(DEFAULT_LIGMAP)


class NullIndexTyper(object):
    """No types at all: every atom is dropped and the coordinate sets it types take no channels
    (include/libmolgrid/atom_typer.h: NullIndexTyper).  For examples whose first file is only a
    place holder."""

    def num_types(self):
        return 0

    def get_type_names(self):
        return []

    def get_type_radii(self):
        return []

    def is_vector_typer(self):
        return False

    def get_int_type(self, t):
        return -1, 0.0

    def map_types(self, raw):
        raw = np.asarray(raw)
        return np.full(raw.shape, -1, dtype=np.int64), np.zeros(raw.shape, dtype=np.float32)


# the reference's module-level instances (python/bindings.in.cpp: defaultGninaLigandTyper, ...)
defaultGninaReceptorTyper = default_receptor_typer()
defaultGninaLigandTyper = default_ligand_typer()
