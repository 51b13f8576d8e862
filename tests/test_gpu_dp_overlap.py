"""Data-parallel fine-tune step on two GPUs (NCCL): the gradient reduction overlapped with the backward pass and the
optimizer step — eager (layer hooks launch the reductions) and captured (the replayed backward pass records external
events the reduction stream waits for) — must leave exactly the codes, residuals and losses of the plain
"backward, then one bucketed all-reduce, then step" route, on every rank.  Skipped with fewer than two GPUs."""
import datetime
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from latentq_llm_b200 import finetune as ft
    from latentq_llm_b200.dp import replicas_identical
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120),
                            device_id=torch.device("cuda", rank))
    results = []
    try:
        for chunks, use_graph in ((0, False), (3, False), (3, True), (4, True)):
            model = ft.build_model("llama-tiny", "cuda", seed=11, layers=4)
            swapped = ft.quantize_decoder(model, lbit=4, gbit=16)
            opt, groups = ft.build_optimizer(model, lr=2e-3)
            tuner = ft.LatentFineTuner(model, opt, groups, grad_accum=2, cuda_graph=use_graph, overlap_chunks=chunks,
                                       gate_timeout_s=60.0)
            assert (tuner._reducer is None) == (chunks == 0)
            if chunks:
                assert len(tuner._events) == chunks - 1 and len(tuner._reducer.ranges) == chunks + 1
            batches = ft.synthetic_batches(2, 2, 64, 1024, "cuda", seed=5 + rank)    # every rank its own data
            losses = [float(tuner.step(batches)) for _ in range(4)]
            if chunks:
                assert tuner._reducer.launched == chunks + 1
            codes = [m.weight.data.clone() for m in swapped]
            res = [m.weight.residual.residual_int.clone() for m in swapped]
            assert replicas_identical(codes) and replicas_identical(res)
            results.append((losses, codes, res))
        base = results[0]
        same = [r[0] == base[0] and all(torch.equal(a, b) for a, b in zip(r[1], base[1])) and
                all(torch.equal(a, b) for a, b in zip(r[2], base[2])) for r in results[1:]]
        q.put((rank, same, base[0]))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_overlapped_gradient_reduction_is_bit_identical_on_two_gpus():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        res = sorted(q.get(timeout=300) for _ in range(2))
    finally:
        for p in procs:
            p.join(60)
            if p.is_alive():
                p.kill()
    assert all(p.exitcode == 0 for p in procs)
    for rank, same, losses in res:
        assert all(same), (rank, same)
        assert losses[-1] < losses[0]
    assert res[0][2] != res[1][2]          # different data per rank, same weights
