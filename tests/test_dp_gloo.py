"""Data-parallel plumbing on CPU: world_size-2 gloo process groups (no GPU needed)."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


class _P:                                   # stand-in for QuantTensor: .shape and .grad
    def __init__(self, shape):
        self.shape = shape
        self.grad = None


def _init(rank, world, port, timeout_s=60):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _worker_allreduce(rank, world, port, q):
    from latentq_llm_b200.dp import GradArena, allreduce_mean, replicas_identical, shard_micro_batches
    _init(rank, world, port)
    params = [_P([96, 128]), _P([128, 64]), _P([40])]
    arena = GradArena(params, dtype=torch.bfloat16, device="cpu")
    arena.attach()
    assert all(p.grad.shape == tuple(p.shape) and p.grad.abs().sum() == 0 for p in params)
    # each rank accumulates its own micro-batches into the arena views, like the backward hook does
    g = torch.Generator().manual_seed(100)
    full = [[torch.randn(*p.shape, generator=g).to(torch.bfloat16) for p in params] for _ in range(4)]
    for mb in shard_micro_batches(4, rank, world):
        for p, t in zip(params, full[mb]):
            p.grad.add_(t)
    n_buckets = allreduce_mean(arena, bucket_bytes=8192)
    assert n_buckets == (arena.numel * 2 + 8191) // 8192
    want = []
    for i, p in enumerate(params):
        acc = [torch.zeros(*p.shape, dtype=torch.bfloat16) for _ in range(world)]
        for r in range(world):
            for mb in shard_micro_batches(4, r, world):
                acc[r].add_(full[mb][i])
        want.append((sum(a for a in acc) / world).to(torch.bfloat16))
    ok = all(torch.allclose(p.grad.float(), w.float(), rtol=2e-2, atol=1e-3) for p, w in zip(params, want))
    ident = replicas_identical([p.grad for p in params])
    differ = replicas_identical([torch.full((4,), float(rank))])
    # same multiset of bytes, same sum, different order on rank 1: a checksum of sums would pass, the hash must not
    swapped = torch.arange(64, dtype=torch.int8)
    if rank == 1:
        swapped[[5, 40]] = swapped[[40, 5]]
    differ = differ or replicas_identical([swapped])
    q.put((rank, ok, ident, differ))
    dist.destroy_process_group()


def test_bucketed_allreduce_mean_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_allreduce, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, ok, ident, differ in res:
        assert ok and ident and not differ


def _worker_chunk_reducer(rank, world, port, q):
    from latentq_llm_b200.dp import ChunkReducer, GradArena, allreduce_mean
    _init(rank, world, port)
    params = [_P([96, 128]), _P([128, 64]), _P([64, 64]), _P([40])]
    outs = []
    for chunked in (True, False):
        arena = GradArena(params, dtype=torch.bfloat16, device="cpu")
        arena.attach()
        g = torch.Generator().manual_seed(200 + rank)
        for p in params:
            p.grad.add_(torch.randn(*p.shape, generator=g).to(torch.bfloat16))
        if chunked:
            o = arena.offsets
            red = ChunkReducer(arena, [(o[0], o[1]), (o[1], o[3]), (o[3], o[3]), (o[3], arena.numel)])
            red.begin()
            for k in (1, 3):                         # ranges become final out of order, like layers in a backward pass
                red.launch(k)
            for k in range(4):                       # the rest; ranges already launched and the empty one are skipped
                red.launch(k)
            assert red.launched == 3
            red.wait(3); red.wait(0)                 # the optimizer waits range by range
            red.wait_all()
        else:
            allreduce_mean(arena, bucket_bytes=4096)
        outs.append(arena.flat.clone())
    q.put((rank, bool(torch.equal(outs[0], outs[1])), float(outs[0].float().abs().sum())))
    dist.destroy_process_group()


def test_chunk_reducer_equals_bucketed_allreduce_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_chunk_reducer, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert all(same and total > 0 for _, same, total in res)
    assert res[0][2] == res[1][2]


def _worker_dead_peer(rank, world, port, q):
    from latentq_llm_b200.dp import GradArena, PeerLostError, StepGate, allreduce_mean
    _init(rank, world, port)
    arena = GradArena([_P([64, 64])], dtype=torch.float32, device="cpu")
    arena.attach()
    gate = StepGate(timeout_s=3.0)
    gate.arrive_and_wait(0)                  # both ranks alive: passes
    allreduce_mean(arena)
    if rank == 1:
        q.put((rank, "left")); q.close(); q.join_thread()
        os._exit(0)                          # the peer leaves between steps, on the host, nothing in flight
    try:
        gate.arrive_and_wait(1)              # noticed here, before the next collective would be launched
        allreduce_mean(arena)
        q.put((rank, "no error"))
    except PeerLostError:
        q.put((rank, "peer lost"))
    q.close(); q.join_thread()
    os._exit(0)


def test_dead_peer_is_noticed_on_the_host_before_the_next_collective():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_dead_peer, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(30)
        if p.is_alive():
            p.kill()
    assert res == {1: "left", 0: "peer lost"}, res


def test_shard_micro_batches():
    from latentq_llm_b200.dp import shard_micro_batches
    assert shard_micro_batches(8, 1, 4) == [1, 5]
    assert sorted(sum((shard_micro_batches(8, r, 3) for r in range(3)), [])) == list(range(8))
