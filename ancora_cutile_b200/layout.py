"""Where every parameter lives in the two arenas of a rank, and the units a step walks.

Pure host arithmetic (no device, no library): given the parameter shapes, the Muon routing and
(rank, world) it fixes

  AdamW arena : every tensor at a 64-element-aligned global offset, the arena padded to
                world * per_rank; rank r owns the contiguous slice [r * per, (r + 1) * per).
  Muon arena  : [arena group][owner rank][matrix]; inside a group every rank's region has the
                same padded size ``per``, so a group is exchanged in place; the float32 state of
                the owned matrices is packed [arena group][matrix] (``m_own_off``).  An arena group
                is a shape group, except that with four or more ranks the largest shape group is
                cut into two parts (every rank's matrices of that shape, first half and second
                half): the exchange of the first part then runs while the second is computed,
                instead of the whole group's exchange starting when all of it is done.

and cuts a step into units, each a contiguous span of this rank's share of one arena.  The
reference keeps per-name buffers on one GPU (ancora/optim/adamw.py:76-87, optim/muon.py:236-254);
arenas exist here so that one launch covers all tensors and one exchange covers a unit.
"""
import os

import numpy as np

from .zero1 import partition_by_group, slice_bounds


def _numel(shape):
    return int(np.prod(shape, dtype=np.int64))


def _align_up(x, a):
    return -(-x // a) * a


class ArenaLayout:
    def __init__(self, shapes, muon_names, rank=0, world=1):
        """shapes: {name: shape} in registration order (identical on every rank)."""
        self.rank, self.world = int(rank), int(world)
        assert 0 <= self.rank < self.world
        mset = set(muon_names)
        self.shapes = {n: tuple(int(x) for x in s) for n, s in shapes.items()}
        self.muon_names = [n for n in self.shapes if n in mset]
        self.adamw_names = [n for n in self.shapes if n not in mset]
        W, R = self.world, self.rank

        # AdamW arena
        self.a_off, off = {}, 0
        for n in self.adamw_names:
            self.a_off[n] = off
            off = _align_up(off + _numel(self.shapes[n]), 64)
        self.a_total = off
        self.a_per, self.a_padded = slice_bounds(max(off, 64), W, 64)
        self.a_begin, self.a_end = R * self.a_per, (R + 1) * self.a_per

        # Muon arenas
        mshapes = [self.shapes[n] for n in self.muon_names]
        self.owner, self.load = partition_by_group(mshapes, W)
        self.m_owner = dict(zip(self.muon_names, self.owner))
        self.groups = []      # dicts: key, shape, plan_first, elems, per, base, names (by rank), own_base, total
        self.m_off, self.m_own_off = {}, {}
        base = own = 0
        shape_keys = sorted({(min(s), max(s)) for s in mshapes})
        members = {}
        for key in shape_keys:
            by_rank = [[] for _ in range(W)]
            for n, r in zip(self.muon_names, self.owner):
                if (min(self.shapes[n]), max(self.shapes[n])) == key:
                    by_rank[r].append(n)
            members[key] = by_rank
        self.parts = self._parts(members)
        for key in shape_keys:
            e = key[0] * key[1]
            whole = members[key]
            k = self.parts[key]
            cut = [[-(-len(x) * p // k) for p in range(k + 1)] for x in whole]     # per rank: part boundaries
            for p in range(k):
                by_rank = [x[c[p]:c[p + 1]] for x, c in zip(whole, cut)]
                per = max(max(len(x) for x in by_rank), 1) * e
                g = dict(key=key if p == 0 else key + (p,), shape=key, plan_first=cut[R][p], elems=e, per=per,
                         base=base, names=by_rank, own_base=own, total=sum(len(x) for x in by_rank) * e)
                for r in range(W):
                    for j, n in enumerate(by_rank[r]):
                        self.m_off[n] = base + r * per + j * e
                for j, n in enumerate(by_rank[R]):
                    self.m_own_off[n] = own + j * e
                base += W * per
                own += len(by_rank[R]) * e
                self.groups.append(g)
        self.m_total = max(base, 64)
        self.m_owned_elems = own
        self.gmap = {g["key"]: g for g in self.groups}

    def _parts(self, members):
        """{shape key: number of arena groups the shape group is cut into}.  The same on every rank:
        two for the largest shape group when there are at least four ranks and every rank owns at
        least eight of its matrices, else one (measured on the benchmark step: 3.08 against 3.22 ms at
        four ranks, no difference at two).  ANCORA_GROUP_PARTS=k cuts the largest group into k
        parts whatever the world size (for tests)."""
        parts = {key: 1 for key in members}
        if not members:
            return parts
        biggest = max(members, key=lambda k: (sum(len(x) for x in members[k]) * k[0] * k[1], k))
        forced = int(os.environ.get("ANCORA_GROUP_PARTS", "0"))
        if forced > 0:
            parts[biggest] = forced
        elif self.world >= 4 and min(len(x) for x in members[biggest]) >= 8:
            parts[biggest] = 2
        return parts

    def owned_range(self, name):
        """(start, stop) flat element range of ``name`` whose state this rank holds."""
        n = _numel(self.shapes[name])
        if name in self.a_off:
            o = self.a_off[name]
            lo, hi = max(o, self.a_begin), min(o + n, self.a_end)
            return (lo - o, hi - o) if lo < hi else (0, 0)
        return (0, n) if self.m_owner[name] == self.rank else (0, 0)

    def make_units(self, batch_cap=None, max_elems=None):
        """Units in execution order: ("adamw", begin, end) over arena-0 elements, then
        ("muon", group key, first, count) over this rank's matrices of each arena group (``first``
        counts inside the arena group; the group's ``plan_first`` places it inside the shape group), groups
        by descending size (the last unit's exchange or copy-out is the one nothing overlaps,
        so the smallest goes last).  ``batch_cap[key]`` bounds a Muon unit by the scratch batch
        of the plan; ``max_elems`` cuts units into sub-ranges of at most that many elements (host
        pipelining), and the sub-ranges of the last group then shrink toward the end (halves, down to
        a quarter of ``max_elems``): what nothing overlaps in the pipelined round trip is the last
        unit's compute and copy-out, so it is kept small, but not so small that the units' launches
        fall behind their uploads.  How many units a rank's share is cut into never matters
        to the exchange (``exchange_schedule``)."""
        units = []
        if max_elems is None:
            units.append(("adamw", self.a_begin, self.a_end))
        else:
            step = max(64, max_elems // 64 * 64)
            for lo in range(self.a_begin, self.a_end, step):
                units.append(("adamw", lo, min(lo + step, self.a_end)))
        order = [g for g in sorted(self.groups, key=lambda g: -g["total"]) if g["names"][self.rank]]
        for g in order:
            mine = len(g["names"][self.rank])
            cap = mine if batch_cap is None else batch_cap[g["shape"]]
            per = cap if max_elems is None else max(1, min(cap, max_elems // g["elems"]))
            first = 0
            while first < mine:
                left = mine - first
                count = min(per, left)
                if max_elems is not None and g is order[-1] and left <= per:
                    floor = max(1, max_elems // 4 // g["elems"])
                    if left > floor:
                        count = max(floor, (left + 1) // 2)
                units.append(("muon", g["key"], first, count))
                first += count
        return units

    def unit_span(self, unit):
        """(arena index, element offset, element count) of a unit's span in the bf16 parameter
        and gradient arenas (arena 0 = AdamW, 1 = Muon)."""
        if unit[0] == "adamw":
            return 0, unit[1], unit[2] - unit[1]
        g = self.gmap[unit[1]]
        return 1, g["base"] + self.rank * g["per"] + unit[2] * g["elems"], unit[3] * g["elems"]

    def exchange_schedule(self, unit_groups):
        """Interleaving of this rank's units with the per-group collectives of the overlapped
        exchange.  ``unit_groups[i]`` names the arena group of unit i ("adamw" or a shape key), in
        execution order.  Returns a list of ("compute", i) and ("gather", group) steps in which

          * every arena group -- the AdamW arena, then every shape group by descending size -- is
            gathered exactly once, in that order on every rank (a collective must be entered by
            all ranks in the same order, whether or not a rank owns anything of the group, and
            however many units its share was cut into);
          * a group's gather follows the last of this rank's units of that group.
        """
        order = ["adamw"] + [g["key"] for g in sorted(self.groups, key=lambda g: -g["total"])]
        steps, done = [], 0
        for grp in order:
            idx = [i for i, k in enumerate(unit_groups) if k == grp]
            if idx:
                assert idx[0] >= done, "units must come in arena-group order"
                steps += [("compute", i) for i in range(done, idx[-1] + 1)]
                done = idx[-1] + 1
            steps.append(("gather", grp))
        assert done == len(unit_groups), "a unit names an unknown arena group"
        return steps
