"""The order in which an ExampleProvider hands out the lines of its example lists: the reference's
ExampleRefProvider family (include/libmolgrid/exampleref_providers.h, src/exampleref_providers.cpp)
and the rules by which its settings choose among them (src/example_provider.cpp:103-213).

The providers here work on the indices of the lines in the ExampleProvider's list, not on copies of
the lines.  Shuffling draws from a numpy generator seeded by ``seed`` (the reference shuffles with its
C++ engine, whose sequence is specific to the standard library it was built with): the same
guarantees hold (every line once per pass, balance, stratification), not the same permutation.
"""
import math

import numpy as np

FLT_EPSILON = float(np.finfo(np.float32).eps)


class IterationScheme(object):
    """How ``for batch in provider`` ends (include/libmolgrid/example.h:18-22): never, after every
    example has been seen at least once, or at most once."""
    Continuous, LargeEpoch, SmallEpoch = 0, 1, 2
    _names = {"Continuous": 0, "LargeEpoch": 1, "SmallEpoch": 2}

    @classmethod
    def of(cls, v):
        if isinstance(v, str):
            return cls._names[v]
        return int(v)


class ExampleProviderSettings(object):
    """The reference's settings with their defaults (include/libmolgrid/example.h:24-45)."""

    DEFAULTS = dict(shuffle=False, balanced=False, stratify_receptor=False, labelpos=0, stratify_pos=1,
                    stratify_abs=True, stratify_min=0.0, stratify_max=0.0, stratify_step=0.0,
                    group_batch_size=1, max_group_size=0, default_batch_size=1, cache_structs=True,
                    add_hydrogens=True, duplicate_first=False, num_copies=1, make_vector_types=False,
                    iteration_scheme=IterationScheme.Continuous, data_root="", recmolcache="", ligmolcache="")

    def __init__(self, **kw):
        for k, v in self.DEFAULTS.items():
            setattr(self, k, kw.pop(k, v))
        if kw:
            raise TypeError("unknown example provider settings: " + ", ".join(sorted(kw)))
        self.iteration_scheme = IterationScheme.of(self.iteration_scheme)


class Uniform(object):
    """One list, walked in order, shuffled at set-up and at every wrap when ``shuffle`` is set, each
    entry handed out ``num_copies`` times in a row (UniformExampleRefProvider)."""

    def __init__(self, settings, rng, labels):
        self.all = []
        self.randomize = bool(settings.shuffle)
        self.ncopies = max(int(settings.num_copies), 1)
        self.rng = rng
        self.current = self.current_copy = self.epoch = 0
        self.cnt = 1

    def addref(self, i, ref):
        self.all.append(i)

    def setup(self):
        self.current = 0
        if self.randomize:
            self.rng.shuffle(self.all)
        if not self.all:
            raise ValueError("No valid examples found in training set.")

    def nextref(self):
        i = self.all[self.current]
        if self.ncopies > 1:
            self.current_copy += 1
            if self.current_copy >= self.ncopies:
                self.current += 1
                self.current_copy = 0
        else:
            self.current += 1
        if self.current >= len(self.all):
            self.setup()
            self.epoch += 1
        self.cnt += 1
        return i

    def size(self):
        return len(self.all)

    def small_epoch_size(self):
        return len(self.all)

    large_epoch_size = small_epoch_size

    def get_small_epoch_num(self):
        return self.epoch

    get_large_epoch_num = get_small_epoch_num

    def reset(self):
        self.cnt = 0
        self.current = self.current_copy = 0


class _Counting(object):
    def get_small_epoch_num(self):
        return self.cnt // self.small_epoch_size()

    def get_large_epoch_num(self):
        return self.cnt // self.large_epoch_size()


class Balanced(_Counting):
    """Alternates between the lines whose label at ``labelpos`` is non-zero and the others
    (BalancedExampleRefProvider)."""

    def __init__(self, settings, rng, labels):
        self.actives = Uniform(settings, rng, labels)
        self.decoys = Uniform(settings, rng, labels)
        self.labelpos = int(settings.labelpos)
        self.current = 0
        self.cnt = 1

    def addref(self, i, ref):
        if self.labelpos >= len(ref.labels):
            raise ValueError("Example has no label at position %d but a label is required to balance batches.  "
                             "There are only %d labels" % (self.labelpos, len(ref.labels)))
        (self.actives if ref.labels[self.labelpos] else self.decoys).addref(i, ref)

    def setup(self):
        self.current = 0
        self.actives.setup()
        self.decoys.setup()

    def nextref(self):
        i = (self.actives if self.current % 2 == 0 else self.decoys).nextref()
        self.current += 1
        self.cnt += 1
        return i

    def size(self):
        return self.actives.size() + self.decoys.size()

    def num_actives(self):
        return self.actives.size()

    def num_decoys(self):
        return self.decoys.size()

    def small_epoch_size(self):
        return 2 * min(self.actives.size(), self.decoys.size())

    def large_epoch_size(self):
        return 2 * max(self.actives.size(), self.decoys.size())

    def reset(self):
        self.actives.reset()
        self.decoys.reset()
        self.current = 0
        self.cnt = 0


class ReceptorStratified(_Counting):
    """One sub-provider per receptor (first file of a line); ``k`` lines from each receptor in turn,
    the receptors shuffled at every pass when ``shuffle`` is set (ReceptorStratifiedExampleRefProvider).
    With balanced sub-providers and k = 2, receptors that lack actives or decoys are dropped at set-up."""

    def __init__(self, settings, rng, labels, inner, k):
        self.settings, self.rng, self.labels = settings, rng, labels
        self.inner, self.k = inner, int(k)
        self.examples = []
        self.recmap = {}
        self.randomize = bool(settings.shuffle)
        self.currenti = self.currentk = 0
        self.cnt = 1

    def addref(self, i, ref):
        if not ref.files:
            raise ValueError("Missing receptor from line")
        pos = self.recmap.get(ref.files[0])
        if pos is None:
            pos = self.recmap[ref.files[0]] = len(self.examples)
            self.examples.append(self.inner(self.settings, self.rng, self.labels))
        self.examples[pos].addref(i, ref)

    def setup(self):
        if self.k <= 0:
            raise ValueError("Invalid sampling k for ReceptorStratifiedExampleRefProvider")
        self.currenti = self.currentk = 0
        if self.inner is Balanced and self.k == 2:
            self.examples = [e for e in self.examples if e.num_actives() > 0 and e.num_decoys() > 0]
        for e in self.examples:
            e.setup()
        if self.randomize:
            self.rng.shuffle(self.examples)

    def nextref(self):
        if not self.examples:
            raise ValueError("No valid stratified examples.")
        if self.currentk >= self.k:
            self.currentk = 0
            self.currenti += 1
        if self.currenti >= len(self.examples):
            self.currenti = 0
            if self.randomize:
                self.rng.shuffle(self.examples)
        e = self.examples[self.currenti]
        if e.size() == 0:
            raise RuntimeError("No valid sub-stratified examples.")
        i = e.nextref()
        self.currentk += 1
        self.cnt += 1
        return i

    def size(self):
        return sum(e.size() for e in self.examples)

    def small_epoch_size(self):
        if not self.examples:
            raise ValueError("No valid stratified examples.")
        return min(e.small_epoch_size() for e in self.examples) * len(self.examples)

    def large_epoch_size(self):
        if not self.examples:
            raise ValueError("No valid stratified examples.")
        return max(e.large_epoch_size() for e in self.examples) * len(self.examples)

    def reset(self):
        self.currenti = self.currentk = 0
        self.cnt = 0
        for e in self.examples:
            e.reset()


class ValueStratified(_Counting):
    """Bins the lines by the label at ``stratify_pos`` ([min, max) in steps of ``stratify_step``, by
    absolute value when ``stratify_abs``) and takes one line from each non-empty bin in turn
    (ValueStratifiedExampleRefProfider)."""

    def __init__(self, settings, rng, labels, inner):
        self.min, self.max = float(settings.stratify_min), float(settings.stratify_max)
        self.step, self.use_abs = float(settings.stratify_step), bool(settings.stratify_abs)
        self.valpos = int(settings.stratify_pos)
        if self.valpos < 0:
            raise ValueError("Negative position for stratification value")
        if self.min == self.max:
            raise ValueError("Empty range for value stratification")
        if not self.step > 0:
            raise ValueError("Not enough bins for value stratification")
        maxbin = self.bin(self.max)
        if maxbin == 0:
            raise ValueError("Not enough bins for value stratification")
        self.examples = [inner(settings, rng, labels) for _ in range(maxbin + 1)]
        self.currenti = 0
        self.cnt = 1

    def bin(self, val):
        if self.use_abs:
            val = math.fabs(val)
        if val < self.min:
            val = self.min
        if val >= self.max:
            val = self.max - FLT_EPSILON
        return int((val - self.min) / self.step)

    def addref(self, i, ref):
        if self.valpos >= len(ref.labels):
            raise ValueError("Invalid position for value stratification label")
        b = self.bin(ref.labels[self.valpos])
        if b >= len(self.examples):
            raise ValueError("Error with value stratification binning")
        self.examples[b].addref(i, ref)

    def setup(self):
        self.currenti = 0
        self.examples = [e for e in self.examples if e.size() > 0]
        for e in self.examples:
            e.setup()
        if not self.examples:
            raise ValueError("No examples in affinity stratification!")

    def nextref(self):
        i = self.examples[self.currenti].nextref()
        self.currenti = (self.currenti + 1) % len(self.examples)
        self.cnt += 1
        return i

    size = ReceptorStratified.size
    small_epoch_size = ReceptorStratified.small_epoch_size
    large_epoch_size = ReceptorStratified.large_epoch_size

    def reset(self):
        self.cnt = 0
        self.currenti = 0
        for e in self.examples:
            e.reset()


class Grouped(object):
    """Time series: the lines of a group (first column) are the frames of one example.  A batch of
    ``group_batch_size`` groups is chosen by the inner provider (from the first frame of each
    group); successive calls walk the batch frame by frame, T x N row-major, every group padded to
    ``max_group_size`` frames with empty frames whose labels are NaN (GroupedExampleRefProvider).
    ``nextref`` returns (index of the line, padded, group, continues-a-sequence)."""

    def __init__(self, settings, rng, labels, inner):
        self.examples = inner(settings, rng, labels)
        self.batch_size = int(settings.group_batch_size)
        self.maxgroupsize = int(settings.max_group_size)
        self.frame_groups = {}
        self._group_of = {}
        self.current_ts = self.current_group_index = 0
        self.current_groups = [self.maxgroupsize] * self.batch_size
        self.cnt = 1

    has_group = True

    def addref(self, i, ref):
        if ref.group not in self.frame_groups:
            self.examples.addref(i, ref)  # the inner provider chooses among the groups by their first frame
        self.frame_groups.setdefault(ref.group, []).append(i)
        self._group_of[i] = ref.group

    def setup(self):
        self.examples.setup()

    def check_batch_size(self, bsize):
        if bsize != self.batch_size:
            raise ValueError("Requested batch size %d does not match configured group batch size %d"
                             % (bsize, self.batch_size))

    def nextref(self):
        if self.current_group_index >= len(self.current_groups):
            self.current_group_index = 0
            self.current_ts += 1
        if self.current_ts >= self.maxgroupsize:
            self.current_ts = 0
        if self.current_ts == 0:
            first = self.examples.nextref()
            self.current_groups[self.current_group_index] = self._group_of[first]
        group = self.current_groups[self.current_group_index]
        series = self.frame_groups[group]
        padded = self.current_ts >= len(series)
        i = series[-1] if padded else series[self.current_ts]
        out = (i, padded, group, self.current_ts > 0)
        self.current_group_index += 1
        self.cnt += 1
        return out

    def size(self):
        return self.examples.size()

    def small_epoch_size(self):
        return self.examples.small_epoch_size()

    def large_epoch_size(self):
        return self.examples.large_epoch_size()

    def get_small_epoch_num(self):
        return self.cnt // self.small_epoch_size()

    def get_large_epoch_num(self):
        return self.cnt // self.large_epoch_size()

    def reset(self):
        self.cnt = 0
        self.current_ts = self.current_group_index = 0
        self.examples.reset()


def create_provider(settings, rng, labels=None):
    """The provider the settings ask for: value stratification outside receptor stratification outside
    balancing, all of it inside grouping (src/example_provider.cpp:103-213)."""
    strat_aff = settings.stratify_max != settings.stratify_min
    grouped = settings.max_group_size > 1

    def leaf(s, r, l):
        return (Balanced if s.balanced else Uniform)(s, r, l)

    inner = leaf
    if settings.stratify_receptor:
        k = 2 if settings.balanced else 1
        base = Balanced if settings.balanced else Uniform

        def inner(s, r, l, base=base, k=k):
            return ReceptorStratified(s, r, l, base, k)
    if strat_aff:
        below = inner

        def inner(s, r, l, below=below):
            return ValueStratified(s, r, l, below)
    # receptor stratification alone (neither balanced nor by value) is never grouped in the reference
    # (src/example_provider.cpp:186-196: the grouped branch there tests `balanced` again)
    ungrouped = settings.stratify_receptor and not settings.balanced and not strat_aff
    if grouped and not ungrouped:
        return Grouped(settings, rng, labels, inner)
    return inner(settings, rng, labels)
