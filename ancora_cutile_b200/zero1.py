"""ZeRO-1 partitioning and the NCCL communicator wrapper.

The reference is single-GPU (README.md:93); this module has no counterpart there.
* AdamW state: the flat arena is cut into ``world`` equal contiguous slices.
* Muon: whole matrices, greedy largest-first on the Newton-Schulz cost 4*M^2*N + 2*M^3,
  ties broken by registration order and lowest rank, so every rank computes the same
  assignment from the shapes alone.
* Exchange: all-gather of the updated bf16 parameters (anc_comm_allgather_bf16).
"""
import ctypes as C
import os

from . import _lib as L


def ns_cost(K, N):
    M, Nn = (K, N) if K <= N else (N, K)
    return 4 * M * M * Nn + 2 * M * M * M


def greedy_partition(costs, world):
    """owner[i] for each item; largest first onto the least-loaded rank."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    load = [0] * world
    owner = [0] * len(costs)
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        owner[i] = r
        load[r] += costs[i]
    return owner, load


def partition_by_group(shapes, world):
    """ZeRO-1 ownership of Muon matrices, balanced inside every Newton-Schulz shape group.

    shapes: list of (K, N) in registration order.  Matrices of one shape group cost the same,
    so each rank gets floor or ceil(n/world) of them as a contiguous run in registration
    order; groups are visited by descending total cost and the ranks that are least loaded so
    far take the extra matrices (ties to the lowest rank).  Equal per-group counts keep each
    group's slice of the parameter arena (and its all-gather) nearly padding-free.
    Returns (owner list, per-rank cost)."""
    groups = {}
    for i, (K, N) in enumerate(shapes):
        groups.setdefault((min(K, N), max(K, N)), []).append(i)
    load = [0] * world
    owner = [0] * len(shapes)
    order = sorted(groups, key=lambda k: (-ns_cost(*k) * len(groups[k]), k))
    for key in order:
        idx = groups[key]
        c = ns_cost(*key)
        base, extra = divmod(len(idx), world)
        takers = sorted(range(world), key=lambda r: (load[r], r))[:extra]
        counts = [base + (1 if r in takers else 0) for r in range(world)]
        pos = 0
        for r in range(world):
            for i in idx[pos:pos + counts[r]]:
                owner[i] = r
            pos += counts[r]
            load[r] += counts[r] * c
    return owner, load


def slice_bounds(total_elems, world, align=64):
    """Equal contiguous slices covering [0, total): returns (per_rank, padded_total)."""
    per = -(-total_elems // world)
    per = -(-per // align) * align
    return per, per * world


def find_nccl():
    """Path of an NCCL shared object: the venv's nvidia-nccl wheel if present, else the
    system library (resolved by the loader)."""
    try:
        import nvidia.nccl as n
        p = os.path.join(os.path.dirname(n.__file__ or n.__path__[0]), "lib", "libnccl.so.2")
        if os.path.exists(p):
            return p
    except Exception:
        pass
    try:
        import importlib.util
        spec = importlib.util.find_spec("nvidia")
        for base in (spec.submodule_search_locations or []):
            p = os.path.join(base, "nccl", "lib", "libnccl.so.2")
            if os.path.exists(p):
                return p
    except Exception:
        pass
    return None


def nccl_unique_id():
    p = find_nccl()
    L.check(L.lib().anc_nccl_load(p.encode() if p else None))
    buf = (C.c_char * 128)()
    L.check(L.lib().anc_nccl_unique_id(buf))
    return bytes(buf)


class Comm:
    """NCCL communicator over the library's C ABI.  ``uid`` is the 128-byte unique id made
    by rank 0 (``nccl_unique_id()``) and handed to every rank by the launcher's own means
    (a store, a file, torch.distributed's object broadcast)."""

    def __init__(self, ctx, uid, rank, world):
        self.ctx, self.rank, self.world = ctx, int(rank), int(world)
        p = find_nccl()
        L.check(L.lib().anc_nccl_load(p.encode() if p else None))
        h = C.c_void_p()
        buf = (C.c_char * 128).from_buffer_copy(uid)
        L.check(L.lib().anc_comm_create(ctx.handle, buf, self.rank, self.world, C.byref(h)))
        self.handle = h

    def allgather_bf16(self, arena_ptr, elems_per_rank, stream=None):
        L.check(L.lib().anc_comm_allgather_bf16(self.handle, arena_ptr, int(elems_per_rank),
                                                C.c_void_p(stream or None)))

    def reduce_scatter_grads(self, arena_ptr, elems_per_rank, grad_dtype="bf16", stream=None):
        L.check(L.lib().anc_comm_reduce_scatter_grads(self.handle, arena_ptr, int(elems_per_rank),
                                                      L.GRAD_BF16 if grad_dtype == "bf16" else L.GRAD_F32,
                                                      C.c_void_p(stream or None)))

    def barrier(self, stream=None):
        L.check(L.lib().anc_comm_barrier(self.handle, C.c_void_p(stream or None)))

    def destroy(self):
        if self.handle:
            L.lib().anc_comm_destroy(self.handle)
            self.handle = None


class P2PExchange:
    """All-gather of arena slices by copy-engine pushes into IPC-mapped peer arenas.

    Every rank owns two device arenas (bf16 AdamW parameters, bf16 Muon parameters) and a flag
    array of ``world`` counters.  ``local_handles()`` gives the three 64-byte IPC handles to
    hand to the other ranks; ``connect(all_handles)`` maps theirs.  ``push(arena, offset, bytes,
    after)`` copies this rank's bytes to the same offset of every peer on per-peer streams
    (so the copies run on separate copy engines) once event ``after`` has fired, then raises
    this rank's flag on each peer.  ``finish(stream)`` makes ``stream`` wait until all peers'
    pushes of the current step have landed here (bounded spin) and this rank's own pushes have
    drained.  No SM is used for the payload, so the transfer overlaps the GEMMs.
    """

    def __init__(self, ctx, rank, world, arena_ptrs):
        from .buffers import DBuf, Event
        import numpy as np
        self.ctx, self.rank, self.world = ctx, int(rank), int(world)
        self.local = list(arena_ptrs)
        self.flags = DBuf.zeros((64,), np.uint32, ctx)
        self.seq = 0
        self.peer = {}
        self.streams = {}
        self._events = {}
        self._Event = Event
        for p in range(self.world):
            if p != self.rank:
                s = C.c_void_p()
                L.check(L.lib().anc_stream_create(ctx.handle, C.byref(s)))
                self.streams[p] = s.value
                self._events[p] = Event()

    def local_handles(self):
        out = []
        for ptr in self.local + [self.flags.ptr]:
            buf = (C.c_char * 64)()
            L.check(L.lib().anc_ipc_export_mem(self.ctx.handle, ptr, buf))
            out.append(bytes(buf))
        return out

    def connect(self, all_handles):
        """all_handles[r] = rank r's ``local_handles()``."""
        for p in range(self.world):
            if p == self.rank:
                continue
            ptrs = []
            for h in all_handles[p]:
                q = C.c_void_p()
                L.check(L.lib().anc_ipc_open_mem(self.ctx.handle, (C.c_char * 64).from_buffer_copy(h), C.byref(q)))
                ptrs.append(q.value)
            self.peer[p] = ptrs

    def begin_step(self):
        pass

    def push(self, arena, offset_bytes, nbytes, after_event):
        """Arena index (0 or 1), byte offset of this rank's slice, its size."""
        self.seq = (self.seq + 1) & 0xFFFFFFFF
        lib = L.lib()
        for p, st in self.streams.items():
            L.check(lib.anc_stream_wait_event(st, after_event.handle))
            if nbytes:
                L.check(lib.anc_d2d(self.ctx.handle, self.peer[p][arena] + offset_bytes,
                                    self.local[arena] + offset_bytes, nbytes, st))
            L.check(lib.anc_p2p_signal(self.ctx.handle, self.peer[p][2] + 4 * self.rank, self.seq, st))
        return self.seq

    def wait_peers(self, stream, seq=None):
        """``stream`` waits until every peer's push number ``seq`` (default: latest) has landed."""
        L.check(L.lib().anc_p2p_wait_flags(self.ctx.handle, self.flags.ptr, self.world, self.rank,
                                           self.seq if seq is None else seq, C.c_void_p(stream or None)))

    def finish(self, stream):
        self.wait_peers(stream)
        for p, st in self.streams.items():
            self._events[p].record(st)
            L.check(L.lib().anc_stream_wait_event(C.c_void_p(stream or None), self._events[p].handle))

    def destroy(self):
        lib = L.lib()
        for p, ptrs in self.peer.items():
            for q in ptrs:
                lib.anc_ipc_close_mem(self.ctx.handle, q)
        self.peer = {}
        for st in self.streams.values():
            lib.anc_stream_destroy(self.ctx.handle, st)
        self.streams = {}
        if self.flags is not None:
            self.flags.free()
            self.flags = None
