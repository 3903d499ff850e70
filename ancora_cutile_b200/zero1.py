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
