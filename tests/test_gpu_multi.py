"""GPU (needs >= 2 GPUs, skipped otherwise): the ZeRO-1 step on two real ranks, one process per
GPU, with both exchange paths.  After the step every rank must hold, for every parameter, exactly
the bf16 bits the single-GPU engine produces (the sharded step must be bitwise identical to the 1-GPU
result).  Ranks are plain child processes; the NCCL id and the IPC handles travel through gloo."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
AKW = dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.1)


def _ngpu():
    from ancora_cutile_b200 import _lib
    n = C.c_int()
    _lib.lib().anc_device_count(C.byref(n))
    return n.value


def _small():
    from ancora_cutile_b200 import shapes as S
    return S.qwen3_0_6b_shapes(n_layers=3, hidden=256, q_heads=4, kv_heads=2, head_dim=128, ffn=768, vocab=4096)


def _run_engine(rank, world, mode, ctx, comm=None, all_gather=None):
    import ancora_cutile_b200 as anc
    from ancora_cutile_b200 import shapes as S
    shp = _small()
    params = S.synthetic_params(shp, seed=11)
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    eng = anc.ResidentHybrid(params, mu, nd, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=3,
                             rank=rank, world=world, comm=comm,
                             schedule=anc.PE_SCHEDULE, ctx=ctx)
    for k in range(3):
        eng.upload_grads(S.synthetic_grads_bf16(shp, seed=20 + k), ctx.stream)
        eng.step(ctx.stream)
    ctx.sync()
    status = ctx.status()
    bits, _ = eng.download_weights_bits()
    bits = {n: b.copy() for n, b in bits.items()}
    return eng, bits, status


def _worker(rank, world, port, mode, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    import ancora_cutile_b200 as anc
    from ancora_cutile_b200.zero1 import Comm, nccl_unique_id
    dist.init_process_group("gloo", rank=rank, world_size=world)
    anc.set_device(rank)
    ctx = anc.get_context()
    comm = None
    if mode == "nccl":
        box = [nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        comm = Comm(ctx, box[0], rank, world)

    def all_gather(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    eng, bits, status = _run_engine(rank, world, mode, ctx, comm, all_gather)
    dist.barrier()                      # nobody unmaps or frees while a peer may still push
    q.put((rank, status, {n: b.tobytes() for n, b in bits.items()}))
    dist.barrier()
    eng.free()
    if comm is not None:
        comm.destroy()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["nccl"])
def test_two_ranks_hold_the_single_gpu_bits(mode):
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    import ancora_cutile_b200 as anc
    ctx0 = anc.get_context()
    eng, want, status = _run_engine(0, 1, "single", ctx0)
    eng.free()
    assert status == 0
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    port = 29600 + (os.getpid() % 1000) + (7 if mode == "nccl" else 0)
    procs = [mpc.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for rank, status, bits in got:
        assert status == 0, (rank, status)
        for n, w in want.items():
            assert bits[n] == w.tobytes(), (mode, rank, n)


def _rs_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    import ancora_cutile_b200 as anc
    from ancora_cutile_b200 import shapes as S
    from ancora_cutile_b200.zero1 import Comm, nccl_unique_id
    dist.init_process_group("gloo", rank=rank, world_size=world)
    anc.set_device(rank)
    ctx = anc.get_context()
    box = [nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Comm(ctx, box[0], rank, world)
    shp = _small()
    params = S.synthetic_params(shp, seed=11)
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    eng = anc.ResidentHybrid(params, mu, nd, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=3,
                             rank=rank, world=world, comm=comm, schedule=anc.PE_SCHEDULE, ctx=ctx)
    eng.upload_full_grads(S.synthetic_grads_bf16(shp, seed=40 + rank), ctx.stream)     # rank-local gradients
    eng.reduce_scatter_grads(ctx.stream)
    ctx.sync()
    owned = {}
    for n in shp:
        s, e = eng.owned_range(n)
        if e > s:
            owned[n] = (s, e, eng.grad_view(n).to_numpy().reshape(-1)[s:e].tobytes())
    eng.step(ctx.stream)
    ctx.sync()
    bits, _ = eng.download_weights_bits()
    q.put((rank, ctx.status(), owned, {n: b.tobytes() for n, b in bits.items()}))
    dist.barrier()
    eng.free()
    comm.destroy()
    dist.barrier()
    dist.destroy_process_group()


def test_grad_reduce_scatter_feeds_the_sharded_step():
    """Two data-parallel replicas with different local gradients: after the reduce-scatter every
    owner holds bf16(g0 + g1) of its share (within one bf16 ulp: NCCL adds in its own precision),
    and the sharded step on those gradients leaves both ranks with identical parameters."""
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from ancora_cutile_b200 import shapes as S
    from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
    shp = _small()
    g0, g1 = S.synthetic_grads_bf16(shp, seed=40), S.synthetic_grads_bf16(shp, seed=41)
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    port = 29700 + (os.getpid() % 1000)
    procs = [mpc.Process(target=_rs_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted([q.get(timeout=300) for _ in range(2)], key=lambda x: x[0])
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    covered = {n: 0 for n in shp}
    for rank, status, owned, bits in got:
        assert status == 0
        for n, (s, e, raw) in owned.items():
            have = np.frombuffer(raw, np.uint16)
            want = f32_to_bf16_bits(bits_to_f32(g0[n]).reshape(-1)[s:e] + bits_to_f32(g1[n]).reshape(-1)[s:e])
            assert np.abs(have.astype(np.int32) - want.astype(np.int32)).max() <= 1, (rank, n)
            assert np.mean(have != want) < 1e-3, (rank, n)
            covered[n] += e - s
    for n, s in shp.items():
        assert covered[n] == int(np.prod(s)), n
    for n in shp:
        assert got[0][3][n] == got[1][3][n], n              # both ranks end with the same parameters


def _acc_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    import ancora_cutile_b200 as anc
    from ancora_cutile_b200 import shapes as S
    from ancora_cutile_b200.zero1 import Comm, nccl_unique_id
    dist.init_process_group("gloo", rank=rank, world_size=world)
    anc.set_device(rank)
    ctx = anc.get_context()
    box = [nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Comm(ctx, box[0], rank, world)
    shp = _small()
    params = S.synthetic_params(shp, seed=11)
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    eng = anc.ResidentHybrid(params, mu, nd, adamw_kw=AKW, grad_dtype="bf16", rounding="sr", seed=3,
                             rank=rank, world=world, comm=comm, schedule=anc.PE_SCHEDULE, ctx=ctx)
    eng.enable_grad_accumulation()
    for k in range(2):                                   # two micro-batches of rank-local gradients
        eng.upload_full_grads(S.synthetic_grads_bf16(shp, seed=70 + 2 * rank + k), ctx.stream)
        if k == 0:
            eng.accumulate_grads(ctx.stream)
        else:
            eng.finalize_grads(ctx.stream)               # reduce-scatter in float32, scale 1/4, SR
    ctx.sync()
    owned = {}
    for n in shp:
        s, e = eng.owned_range(n)
        if e > s:
            off = eng.a_off[n] if n in eng.a_off else eng.a_padded + eng.m_off[n]
            owned[n] = (s, e, off, eng.grad_view(n).to_numpy().reshape(-1)[s:e].tobytes())
    eng.step(ctx.stream)
    ctx.sync()
    bits, _ = eng.download_weights_bits()
    q.put((rank, ctx.status(), owned, {n: b.tobytes() for n, b in bits.items()}))
    dist.barrier()
    eng.free()
    comm.destroy()
    dist.barrier()
    dist.destroy_process_group()


def test_accumulated_gradients_reduce_in_float32_and_feed_the_sharded_step():
    """Two replicas, two micro-batches each: every owner ends with SR_bf16((acc_0 + acc_1) / 4) of
    its share, bit for bit against the oracle (a two-term float32 sum has one rounding whatever the
    order), and both ranks hold identical parameters after the step."""
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from ancora_cutile_b200 import shapes as S
    from oracle import grad_ref
    shp = _small()
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    port = 29700 + (os.getpid() % 1000)
    procs = [mpc.Process(target=_acc_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted([q.get(timeout=300) for _ in range(2)], key=lambda x: x[0])
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    acc = []
    for r in range(2):
        a = {n: np.zeros(int(np.prod(s)), np.float32) for n, s in shp.items()}
        for k in range(2):
            g = S.synthetic_grads_bf16(shp, seed=70 + 2 * r + k)
            for n in shp:
                a[n], _ = grad_ref.grad_accumulate(a[n], g[n].reshape(-1), want_g16=False)
        acc.append(a)
    covered = {n: 0 for n in shp}
    for rank, status, owned, bits in got:
        assert status == 0
        for n, (s, e, off, raw) in owned.items():
            tot = (acc[0][n] + acc[1][n])[s:e]
            _, want = grad_ref.grad_accumulate(tot, None, scale=0.25, rounding="sr", seed=4, step=1,
                                               elem_offset=off + s)
            assert np.array_equal(np.frombuffer(raw, np.uint16), want), (rank, n)
            covered[n] += e - s
    for n, s in shp.items():
        assert covered[n] == int(np.prod(s)), n
    for n in shp:
        assert got[0][3][n] == got[1][3][n], n
