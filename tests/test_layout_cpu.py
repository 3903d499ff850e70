"""CPU: the arena layout and the unit lists of the ZeRO-1 engine (pure host arithmetic), for
1/2/4/8 ranks on the Qwen3-0.6B and MoE-family shapes, plus two gloo ranks that exchange their
spans and check that together they cover every parameter exactly once."""
import os

import numpy as np
import pytest

from ancora_cutile_b200 import shapes as S
from ancora_cutile_b200.hybrid import default_is_muon, muon_names_for
from ancora_cutile_b200.layout import ArenaLayout


def _family(which):
    shp = S.qwen3_0_6b_shapes() if which == "qwen3" else S.moe_family_shapes()
    mu = muon_names_for(shp)
    return shp, mu


def _numel(s):
    return int(np.prod(s, dtype=np.int64))


def _tiles(spans, lo, hi):
    """True when the (offset, count) spans tile [lo, hi) exactly, in any order."""
    pos = lo
    for o, n in sorted(spans):
        if o != pos or n <= 0:
            return False
        pos = o + n
    return pos == hi


@pytest.mark.parametrize("which", ["qwen3", "moe"])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_layout_is_the_same_on_every_rank_and_partitions_everything(which, world):
    shp, mu = _family(which)
    lays = [ArenaLayout(shp, mu, r, world) for r in range(world)]
    a = lays[0]
    for b in lays[1:]:
        assert b.a_off == a.a_off and b.m_off == a.m_off and b.owner == a.owner
        assert [(g["key"], g["base"], g["per"]) for g in b.groups] == [(g["key"], g["base"], g["per"]) for g in a.groups]
    # AdamW: 64-aligned offsets in registration order, slices tile the padded arena
    assert all(o % 64 == 0 for o in a.a_off.values())
    assert _tiles([(l.a_begin, l.a_end - l.a_begin) for l in lays], 0, a.a_padded)
    assert a.a_padded >= a.a_total and a.a_per % 64 == 0
    # Muon: every matrix inside its owner's region of its group, no two matrices overlap
    spans = []
    for n in mu:
        r = a.m_owner[n]
        g = next(g for g in a.groups if n in g["names"][r])
        assert g["shape"] == (min(shp[n]), max(shp[n]))
        lo = g["base"] + r * g["per"]
        assert lo <= a.m_off[n] and a.m_off[n] + _numel(shp[n]) <= lo + g["per"], n
        spans.append((a.m_off[n], _numel(shp[n])))
    spans.sort()
    assert all(spans[i][0] + spans[i][1] <= spans[i + 1][0] for i in range(len(spans) - 1))
    assert a.m_total >= spans[-1][0] + spans[-1][1]
    # state ownership: over all ranks the owned ranges of a tensor partition it
    for n in shp:
        got = [l.owned_range(n) for l in lays]
        assert _tiles([(s, e - s) for s, e in got if e > s], 0, _numel(shp[n])), n
    assert sum(l.m_owned_elems for l in lays) == sum(_numel(shp[n]) for n in mu)


@pytest.mark.parametrize("which", ["qwen3", "moe"])
@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("mode", ["plain", "host_chunks", "capped"])
def test_units_cover_exactly_what_the_rank_owns(which, world, mode):
    shp, mu = _family(which)
    for r in range(world):
        lay = ArenaLayout(shp, mu, r, world)
        caps = {g["key"]: max(1, min(8, len(g["names"][r]))) for g in lay.groups} if mode == "capped" else None
        units = lay.make_units(caps, 16 << 20 if mode == "host_chunks" else None)
        spans = {0: [], 1: []}
        for u in units:
            arena, off, n = lay.unit_span(u)
            spans[arena].append((off, n))
            if mode == "host_chunks":
                assert n <= 16 << 20 or (u[0] == "muon" and u[3] == 1)
            if caps and u[0] == "muon":
                assert u[3] <= caps[u[1]]
        assert _tiles(spans[0], lay.a_begin, lay.a_end)
        own = sorted((lay.m_off[n], _numel(shp[n])) for n in mu if lay.m_owner[n] == r)
        covered = sorted(spans[1])
        # the unit spans of a group are contiguous runs over this rank's matrices of the group
        assert sum(n for _, n in covered) == sum(n for _, n in own)
        merged = []
        for o, n in own:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + n)
            else:
                merged.append((o, n))
        for o, n in covered:
            assert any(mo <= o and o + n <= mo + mn for mo, mn in merged), (o, n)
        # AdamW first, then groups by descending size
        kinds = [u[0] for u in units]
        assert kinds == sorted(kinds, key=lambda k: k != "adamw")
        sizes = [lay.gmap[u[1]]["total"] for u in units if u[0] == "muon"]
        assert sizes == sorted(sizes, reverse=True)


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    shp, mu = _family("qwen3")
    lay = ArenaLayout(shp, mu, rank, world)
    mine = dict(rank=rank, spans=[lay.unit_span(u) for u in lay.make_units()], a_padded=lay.a_padded,
                groups=[(g["key"], g["base"], g["per"], [len(x) for x in g["names"]]) for g in lay.groups])
    box = [None] * world
    dist.all_gather_object(box, mine)
    if rank == 0:
        q.put(box)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("parts", [0, 2])
def test_two_gloo_ranks_exchange_complementary_spans(parts, monkeypatch):
    """What each rank would send in the exchange: the two ranks' AdamW spans tile the padded arena,
    and inside every arena group rank r's span starts at base + r * per (the in-place all-gather's
    slot) and holds exactly its matrices; also with the largest shape group cut into two arena groups."""
    import torch.multiprocessing as mp
    if parts:
        monkeypatch.setenv("ANCORA_GROUP_PARTS", str(parts))      # the spawned ranks inherit it
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [mpc.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    box = q.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert box[0]["groups"] == box[1]["groups"]
    assert len(box[0]["groups"]) == 3 + (1 if parts else 0)
    a_spans = [(o, n) for b in box for (arena, o, n) in b["spans"] if arena == 0]
    assert _tiles(a_spans, 0, box[0]["a_padded"])
    shp, _ = _family("qwen3")
    for key, base, per, counts in box[0]["groups"]:
        e = key[0] * key[1]
        for b in box:
            r = b["rank"]
            mine = [(o, n) for (arena, o, n) in b["spans"] if arena == 1 and base <= o < base + 2 * per]
            assert _tiles(mine, base + r * per, base + r * per + counts[r] * e), (key, r)


@pytest.mark.parametrize("world", [2, 8])
def test_every_rank_enters_the_same_collectives_in_the_same_order(world):
    """A small model whose groups do not divide evenly (one group has fewer matrices than ranks at
    world 8) and a scratch cap that cuts shares into different numbers of units per rank: the
    gather sequence is the same on every rank, once per arena group, after the rank's own units."""
    shp = S.qwen3_0_6b_shapes(n_layers=3, hidden=256, q_heads=4, kv_heads=2, head_dim=128, ffn=768, vocab=4096)
    mu = muon_names_for(shp)
    seqs = []
    for r in range(world):
        lay = ArenaLayout(shp, mu, r, world)
        caps = {g["key"]: 1 for g in lay.groups}                  # one matrix per unit
        units = lay.make_units(caps)
        names = ["adamw" if u[0] == "adamw" else u[1] for u in units]
        steps = lay.exchange_schedule(names)
        assert [i for op, i in steps if op == "compute"] == list(range(len(units)))
        gathers = [g for op, g in steps if op == "gather"]
        assert len(gathers) == 1 + len(lay.groups) and len(set(gathers)) == len(gathers)
        for i, n in enumerate(names):                              # a unit precedes its group's gather
            assert steps.index(("compute", i)) < steps.index(("gather", n))
        seqs.append(gathers)
    assert all(s == seqs[0] for s in seqs)
    if world == 8:                                                 # some rank really owns nothing of a group
        lays = [ArenaLayout(shp, mu, r, world) for r in range(world)]
        assert any(len(g["names"][l.rank]) == 0 for l in lays for g in l.groups)


def test_overlapped_step_issues_that_schedule(monkeypatch):
    """The engine's overlapped-exchange branch, driven on the CPU with stand-ins for the device
    calls: two ranks whose shares are cut into different numbers of units record the same
    all-gather sequence (pointer offsets and counts included), each gather after an event wait."""
    from ancora_cutile_b200 import resident

    shp = S.qwen3_0_6b_shapes(n_layers=3, hidden=256, q_heads=4, kv_heads=2, head_dim=128, ffn=768, vocab=4096)
    mu = muon_names_for(shp)

    class Ev:
        def __init__(self, log):
            self.log, self.handle = log, id(self)

        def record(self, stream):
            self.log.append(("record", stream))

    class Lib:
        def __init__(self, log):
            self.log = log

        def anc_stream_wait_event(self, stream, handle):
            self.log.append(("wait", stream))
            return 0

    class Comm:
        def __init__(self, log):
            self.log = log

        def allgather_bf16(self, ptr, per, stream):
            self.log.append(("gather", ptr, per, stream))

    class Buf:
        def __init__(self, ptr):
            self.ptr = ptr

    logs = []
    for r in range(2):
        log = []
        lay = ArenaLayout(shp, mu, r, 2)
        eng = resident.ResidentHybrid.__new__(resident.ResidentHybrid)
        eng.ctx, eng.world, eng.rank, eng.t = None, 2, r, 0
        eng.layout, eng._gmap, eng.a_per = lay, lay.gmap, lay.a_per
        eng.comm, eng.nccl_overlap, eng._comm_stream = Comm(log), True, 77
        eng.a_p16, eng.m_p16 = Buf(1 << 40), Buf(1 << 41)
        caps = {g["key"]: (2 if r == 0 else 3) for g in lay.groups}        # different cuts per rank
        eng.units = [("adamw", None, u[1], u[2]) if u[0] == "adamw" else ("muon", 0, u[2], u[3], u[1])
                     for u in lay.make_units(caps)]
        eng._compute_unit = lambda u, si, log=log: log.append(("compute", u[0], si))
        eng._events = lambda n, log=log: [Ev(log) for _ in range(n)]
        monkeypatch.setattr(resident.L, "lib", lambda log=log: Lib(log))
        eng.step(5)
        assert eng.t == 1
        assert sum(1 for e in log if e[0] == "compute") == len(eng.units)
        for i, e in enumerate(log):
            if e[0] == "gather":                       # record on the compute stream, wait on the comm stream
                assert log[i - 2] == ("record", 5) and log[i - 1] == ("wait", 77) and e[3] == 77
        assert log[-2:] == [("record", 77), ("wait", 5)]  # the step ends ordered after the last gather
        logs.append([e for e in log if e[0] == "gather"])
    assert logs[0] == logs[1]
    lay = ArenaLayout(shp, mu, 0, 2)
    want = [((1 << 40), lay.a_per)] + [((1 << 41) + g["base"] * 2, g["per"])
                                       for g in sorted(lay.groups, key=lambda g: -g["total"])]
    assert [(e[1], e[2]) for e in logs[0]] == want


def test_random_models_keep_the_layout_invariants():
    """Property test over random small models (any number of matrices per shape, fewer matrices
    than ranks included, AdamW tensors of ragged sizes) and world sizes 1..8."""
    from hypothesis import given, settings, strategies as st

    dims = st.sampled_from([128, 256, 384, 512])
    model = st.tuples(
        st.lists(st.tuples(dims, dims), min_size=0, max_size=14),          # Muon matrices (K, N)
        st.lists(st.integers(1, 5000), min_size=1, max_size=6),            # AdamW tensor sizes
        st.integers(1, 8),                                                 # world
        st.sampled_from([None, 1, 3]),                                     # scratch cap
        st.sampled_from([None, 1 << 16]),                                  # host chunk
    )

    @settings(max_examples=120, deadline=None)
    @given(model)
    def check(m):
        mats, vecs, world, cap, chunk = m
        shp = {f"v{i}": (n,) for i, n in enumerate(vecs)}
        shp.update({f"layers.{i}.q_proj": s for i, s in enumerate(mats)})
        mu = [n for n in shp if len(shp[n]) == 2]
        lays = [ArenaLayout(shp, mu, r, world) for r in range(world)]
        a = lays[0]
        assert _tiles([(l.a_begin, l.a_end - l.a_begin) for l in lays], 0, a.a_padded)
        for n in shp:
            got = [l.owned_range(n) for l in lays]
            assert _tiles([(s, e - s) for s, e in got if e > s], 0, _numel(shp[n])), n
        gathers = []
        for l in lays:
            caps = None if cap is None else {g["key"]: cap for g in l.groups}
            units = l.make_units(caps, chunk)
            spans = {0: [], 1: []}
            for u in units:
                arena, off, n = l.unit_span(u)
                spans[arena].append((off, n))
            assert _tiles(spans[0], l.a_begin, l.a_end)
            own = sum(_numel(shp[n]) for n in mu if l.m_owner[n] == l.rank)
            assert sum(n for _, n in spans[1]) == own
            assert len({o for o, _ in spans[1]}) == len(spans[1])
            steps = l.exchange_schedule(["adamw" if u[0] == "adamw" else u[1] for u in units])
            gathers.append([g for op, g in steps if op == "gather"])
        assert all(g == gathers[0] for g in gathers) and len(gathers[0]) == 1 + len(a.groups)

    check()


def test_routing_of_the_two_model_families():
    """Muon takes the tileable 2-D hidden matrices only: the MoE router (1024, 16) is 2-D and passes
    the reference's name rule (ancora/optim/hybrid.py:18-25) but cannot be tiled by 128, so it is
    stepped by AdamW; BASELINE config 5 counts 576 expert matrices of 768x1024."""
    q = S.qwen3_0_6b_shapes()
    mq = muon_names_for(q)
    assert len(mq) == 196 and sum(int(np.prod(q[n])) for n in q if n not in set(mq)) == 155_648_000
    m = S.moe_family_shapes()
    mm = muon_names_for(m)
    routers = [n for n in m if n.endswith(".router")]
    assert len(routers) == 12 and all(m[n] == (1024, 16) for n in routers)
    assert all(default_is_muon(n, np.empty((0, 0))) for n in routers)      # the name rule alone says Muon
    assert not set(routers) & set(mm)                                       # the tiling rule sends them to AdamW
    experts = [n for n in mm if ".experts." in n]
    assert len(experts) == 576 and all(sorted(m[n]) == [768, 1024] for n in experts)
    assert len(mm) == 576 + 24 * 4 + 12 * 3
    # the hybrid step host schedule: every rank gathers the same groups in the same order
    for world in (1, 8):
        orders = []
        for r in range(world):
            lay = ArenaLayout(m, mm, r, world)
            units = lay.make_units(None, 32 << 20)
            sched = lay.exchange_schedule(["adamw" if u[0] == "adamw" else u[1] for u in units])
            orders.append([w for op, w in sched if op == "gather"])
            assert [w for op, w in sched if op == "compute"] == list(range(len(units)))
        assert all(o == orders[0] for o in orders)


def test_host_units_of_the_last_group_shrink_toward_the_end():
    """Host pipelining: the last unit's compute and copy-out overlap nothing, so the last group's
    sub-ranges halve down to a quarter of the chunk size; every owned matrix is still in exactly one unit
    and the device-resident units (no max_elems) stay whole groups."""
    q = S.qwen3_0_6b_shapes()
    qm = muon_names_for(q)
    for world in (1, 2, 4, 8):
        for r in range(world):
            lay = ArenaLayout(q, qm, r, world)
            units = [u for u in lay.make_units(None, 32 << 20) if u[0] == "muon"]
            last_key = units[-1][1]
            per_key = {}
            for _, key, first, count in units:
                assert first == per_key.get(key, 0)              # contiguous, in order
                per_key[key] = first + count
            assert per_key == {g["key"]: len(g["names"][r]) for g in lay.groups if g["names"][r]}
            tail = [u[3] for u in units if u[1] == last_key]
            assert tail[-1] <= max(1, (32 << 20) // 4 // (last_key[0] * last_key[1])) or len(tail) == 1
            assert all(a >= b for a, b in zip(tail, tail[1:]))
            whole = [u for u in lay.make_units() if u[0] == "muon"]
            assert len(whole) == len(per_key) and all(u[2] == 0 for u in whole)


def test_the_largest_group_is_cut_in_two_from_four_ranks_on():
    """Arena groups: below four ranks one per shape; from four on the largest shape group becomes two
    arena groups (every rank's matrices of that shape, first and second half), each with its own
    region and exchange; ``plan_first`` places a part inside the rank's matrices of the shape."""
    for which in ("qwen3", "moe"):
        shp, mu = _family(which)
        for world in (1, 2):
            lay = ArenaLayout(shp, mu, 0, world)
            assert set(lay.parts.values()) == {1} and all(g["key"] == g["shape"] for g in lay.groups)
        assert sorted(ArenaLayout(shp, mu, 0, 4).parts.values())[-1] == 2
        lays = [ArenaLayout(shp, mu, r, 8) for r in range(8)]
        big = max(lays[0].parts, key=lambda k: lays[0].parts[k])
        assert lays[0].parts[big] == 2 and sum(lays[0].parts.values()) == len(lays[0].parts) + 1
        assert all(l.parts == lays[0].parts for l in lays)
        for r, lay in enumerate(lays):
            halves = [g for g in lay.groups if g["shape"] == big]
            assert [g["key"] for g in halves] == [big, big + (1,)]
            n0, n1 = len(halves[0]["names"][r]), len(halves[1]["names"][r])
            assert n0 - n1 in (0, 1) and halves[0]["plan_first"] == 0 and halves[1]["plan_first"] == n0
            # the two parts' names, in order, are the rank's matrices of the shape in registration order
            mine = [n for n in mu if lay.m_owner[n] == r and (min(shp[n]), max(shp[n])) == big]
            assert halves[0]["names"][r] + halves[1]["names"][r] == mine
            # owned state is packed [arena group][matrix]: part 1 follows part 0 directly
            assert halves[1]["own_base"] == halves[0]["own_base"] + n0 * halves[0]["elems"]
            # every rank enters the same gathers in the same order
            units = lay.make_units()
            sched = lay.exchange_schedule(["adamw" if u[0] == "adamw" else u[1] for u in units])
            assert [w for op, w in sched if op == "gather"] == \
                [w for op, w in lays[0].exchange_schedule(
                    ["adamw" if u[0] == "adamw" else u[1] for u in lays[0].make_units()]) if op == "gather"]
            assert sum(1 for op, w in sched if op == "gather") == 2 + len(lay.parts)


def test_forced_parts_with_empty_shares(monkeypatch):
    """ANCORA_GROUP_PARTS cuts the largest group whatever the world; a rank that owns one matrix of
    it gets an empty second part, still has a region there and still enters that part's gather."""
    monkeypatch.setenv("ANCORA_GROUP_PARTS", "2")
    shp = {f"l{i}.w": (128, 256) for i in range(5)}
    shp.update({f"l{i}.s": (128, 128) for i in range(2)})
    mu = list(shp)
    lays = [ArenaLayout(shp, mu, r, 4) for r in range(4)]
    assert lays[0].parts == {(128, 128): 1, (128, 256): 2}
    counts = [[len(g["names"][r]) for g in lays[r].groups if g["shape"] == (128, 256)] for r in range(4)]
    assert sorted(map(tuple, counts)) == [(1, 0), (1, 0), (1, 0), (1, 1)]
    orders = []
    for r, lay in enumerate(lays):
        units = lay.make_units()
        sched = lay.exchange_schedule(["adamw" if u[0] == "adamw" else u[1] for u in units])
        orders.append([w for op, w in sched if op == "gather"])
        assert all(g["per"] >= g["elems"] for g in lay.groups)
    assert all(o == orders[0] for o in orders)
    assert sorted(map(str, orders[0])) == sorted(map(str, ["adamw", (128, 128), (128, 256), (128, 256, 1)]))


def test_random_families_keep_the_layout_invariants():
    """Seeded random shape families and world sizes (with and without a forced cut of the largest group):
    arena groups tile the Muon arena, every matrix lies inside its owner's region of exactly one arena
    group, a rank's units cover exactly its matrices with plan ranges that follow each other inside a
    shape, and all ranks enter the same gathers in the same order."""
    rng = np.random.default_rng(2024)
    sides = [128, 256, 384, 512]
    for trial in range(40):
        world = int(rng.choice([1, 2, 3, 4, 8]))
        n = int(rng.integers(1, 40))
        shp = {}
        for i in range(n):
            k, m = int(rng.choice(sides)), int(rng.choice(sides))
            shp[f"w{i}"] = (k, m)
        shp["gain"] = (128,)
        shp["embed"] = (int(rng.integers(1, 50)) * 64 + int(rng.integers(0, 64)), 128)
        mu = [x for x in shp if x.startswith("w")]
        forced = int(rng.choice([0, 0, 2, 3]))
        if forced:
            os.environ["ANCORA_GROUP_PARTS"] = str(forced)
        try:
            lays = [ArenaLayout(shp, mu, r, world) for r in range(world)]
        finally:
            os.environ.pop("ANCORA_GROUP_PARTS", None)
        a = lays[0]
        # arena groups tile [0, m_total) in order; the same on every rank
        pos = 0
        for g in a.groups:
            assert g["base"] == pos and g["per"] % g["elems"] == 0 and g["per"] >= g["elems"]
            pos += world * g["per"]
        assert pos == a.m_total or (pos == 0 and a.m_total == 64)
        for b in lays[1:]:
            assert [(g["key"], g["base"], g["per"], g["names"]) for g in b.groups] == \
                   [(g["key"], g["base"], g["per"], g["names"]) for g in a.groups]
        seen = {}
        for g in a.groups:
            for r in range(world):
                for j, name in enumerate(g["names"][r]):
                    assert name not in seen and a.m_owner[name] == r
                    assert (min(shp[name]), max(shp[name])) == g["shape"]
                    assert a.m_off[name] == g["base"] + r * g["per"] + j * g["elems"]
                    seen[name] = g["key"]
        assert sorted(seen) == sorted(mu)
        gathers = []
        for r, lay in enumerate(lays):
            units = lay.make_units(None, int(rng.choice([0, 1 << 16, 1 << 18])) or None)
            nxt = {}
            for u in units:
                if u[0] != "muon":
                    continue
                g = lay.gmap[u[1]]
                assert u[2] == nxt.get(u[1], 0) and u[3] >= 1
                nxt[u[1]] = u[2] + u[3]
            assert nxt == {g["key"]: len(g["names"][r]) for g in lay.groups if g["names"][r]}
            # plan ranges of the parts of one shape follow each other
            by_shape = {}
            for g in lay.groups:
                assert g["plan_first"] == by_shape.get(g["shape"], 0)
                by_shape[g["shape"]] = g["plan_first"] + len(g["names"][r])
            sched = lay.exchange_schedule(["adamw" if u[0] == "adamw" else u[1] for u in units])
            assert [w for op, w in sched if op == "compute"] == list(range(len(units)))
            gathers.append([w for op, w in sched if op == "gather"])
        assert all(x == gathers[0] for x in gathers) and len(gathers[0]) == 1 + len(a.groups)
