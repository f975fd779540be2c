"""Choosing tile sizes for a `@dt.kernel`: a search over a small discrete space in which a
candidate only counts if the kernel it configures reproduces the eager run of the same
function, and the memory of past searches.

The protocol is the reference's (deuteron/runtime.py:220-303): check against the oracle, time
the correct ones, start from a seeded sample of the space and then walk to better neighbours
for up to three rounds; remember the winner per (kernel text, power-of-two bucketed shapes,
dtypes) in memory and in $DEUTERON_CACHE_DIR/configs.json.  What the sm_100a backend adds:
candidates that select the same hardware kernel are tried once, a candidate the backend
cannot run is dropped from its launch plan before anything is launched, and the file is
replaced atomically because one process per GPU tunes the same kernel at the same time.
"""

import itertools
import json
import os
import random
import tempfile

CACHE_VERSION = "sm100a-3"


class Config(dict):
    """Tile sizes by constexpr name, plus `num_warps` / `num_stages`."""

    @property
    def num_warps(self):
        return self.get("num_warps", 4)


# ---- the space --------------------------------------------------------------------------

def search_space(tunable, has_dot):
    """Options per knob.  A kernel with a matmul runs on tcgen05 tiles: 128-row MMAs (256 rows
    = a CTA pair), 64..256 columns (512 for a pair), and ring depths the GEMM has instances for;
    anything else is a generated kernel whose tiles may be any power of two."""
    if has_dot:
        space = {name: [64, 128, 256, 512] for name in tunable}
        space["num_warps"] = [4]
        space["num_stages"] = [2, 3, 4, 5, 6]
    else:
        space = {name: [1 << i for i in range(12)] for name in tunable}
        space["num_warps"] = [2, 4, 8]
    return space


def preferred(tunable, has_dot):
    """Configurations a search always times, whatever its sample holds: for a matmul written
    with three tile loops, the tiles the tensor-core kernels are at their best with (a CTA pair
    on 256 x 512 and on 256 x 256), so that the answer is never worse than the library's own
    choice."""
    if not has_dot or len(tunable) != 3:
        return []
    tm, tn, tk = tunable
    return [Config({tm: 256, tn: 512, tk: 64, "num_warps": 4, "num_stages": 4}),
            Config({tm: 256, tn: 256, tk: 128, "num_warps": 4, "num_stages": 3}),
            Config({tm: 256, tn: 256, tk: 64, "num_warps": 4, "num_stages": 6})]


def middle_of(space):
    return Config({knob: options[len(options) // 2] for knob, options in space.items()})


# ---- the search ---------------------------------------------------------------------------

class Search:
    """`measure(config)` returns milliseconds, or None for a candidate that is invalid or
    wrong; `identity(config)` returns what the backend would run for it (equal identities are
    measured once; None: every config is its own) or raises if the backend cannot run it."""

    def __init__(self, space, measure, identity=None, samples=12, rounds=3, seed=0, always=()):
        self.always = [c for c in always if all(c.get(k) in space[k] for k in space)]
        self.space = space
        self.knobs = list(space)
        self.measure = measure
        self.identity = identity
        self.samples, self.rounds, self.seed = samples, rounds, seed
        self.visited = set()
        self.identities = set()

    def config_at(self, point):
        return Config({k: self.space[k][i] for k, i in zip(self.knobs, point)})

    def point_of(self, config):
        return tuple(self.space[k].index(config[k]) if config[k] in self.space[k] else 0
                     for k in self.knobs)

    def distinct(self, point):
        """False for a point already visited or one the backend maps onto a kernel already
        tried or cannot run at all."""
        if point in self.visited:
            return False
        self.visited.add(point)
        if self.identity is None:
            return True
        try:
            ident = self.identity(self.config_at(point))
        except Exception:  # noqa: BLE001 - the backend's refusal, whatever its type
            return False
        if ident is None:
            return True
        if ident in self.identities:
            return False
        self.identities.add(ident)
        return True

    def starting_points(self):
        every = list(itertools.product(*[range(len(self.space[k])) for k in self.knobs]))
        if len(every) <= self.samples:
            return every
        if self.identity is not None:
            # many points share a hardware configuration: one of each is worth a slot
            seen, kept = set(), []
            for point in every:
                try:
                    ident = self.identity(self.config_at(point))
                except Exception:  # noqa: BLE001
                    continue
                if ident is None or ident not in seen:
                    seen.add(ident)
                    kept.append(point)
            every = kept or every
        if len(every) <= self.samples:
            return every
        return random.Random(self.seed).sample(every, self.samples)

    def neighbours(self, point):
        for axis in range(len(point)):
            for step in (-1, 1):
                moved = point[axis] + step
                if 0 <= moved < len(self.space[self.knobs[axis]]):
                    yield point[:axis] + (moved,) + point[axis + 1:]

    def run(self):
        """(best config, its time) or (None, None) when nothing valid was found."""
        best_point, best_ms = None, None
        first = [self.point_of(c) for c in self.always]
        for point in first + [p for p in self.starting_points() if p not in first]:
            if not self.distinct(point):
                continue
            ms = self.measure(self.config_at(point))
            if ms is not None and (best_ms is None or ms < best_ms):
                best_point, best_ms = point, ms
        if best_point is None:
            return None, None
        for _ in range(self.rounds):
            origin = best_point
            for point in self.neighbours(origin):
                if not self.distinct(point):
                    continue
                ms = self.measure(self.config_at(point))
                if ms is not None and ms < best_ms:
                    best_point, best_ms = point, ms
            if best_point == origin:
                break
        return self.config_at(best_point), best_ms


# ---- the memory ----------------------------------------------------------------------------

class ConfigFile:
    """configs.json under $DEUTERON_CACHE_DIR (default ~/.deuteron): key -> config."""

    @staticmethod
    def path():
        folder = os.environ.get("DEUTERON_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".deuteron")
        os.makedirs(folder, exist_ok=True)
        return os.path.join(folder, "configs.json")

    @classmethod
    def read(cls):
        try:
            with open(cls.path()) as f:
                data = json.load(f)
        except (OSError, ValueError):
            return {}
        return data if isinstance(data, dict) else {}

    @classmethod
    def lookup(cls, key):
        stored = cls.read().get(key)
        return Config(stored) if isinstance(stored, dict) else None

    @classmethod
    def remember(cls, key, config):
        """Merges one entry into the file and swaps the file in with a rename, so a reader in
        another process sees the old file or the new one, never half of either."""
        target = cls.path()
        data = cls.read()
        data[key] = dict(config)
        try:
            handle, scratch = tempfile.mkstemp(dir=os.path.dirname(target), suffix=".tmp")
            with os.fdopen(handle, "w") as f:
                json.dump(data, f, indent=1)
            os.replace(scratch, target)
        except OSError:
            pass      # a read-only cache directory costs a search next time, nothing else
