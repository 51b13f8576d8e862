"""Data-parallel plumbing for the latent fine-tune step.

The reference never reduces the gradients of its quantized weights: they live on plain Python
`QuantTensor` objects, attached by a backward hook (utils/quant.py:398-411), invisible to DeepSpeed's
gradient all-reduce, and its default launch is world size 1 (main0.py:200-216).  Here every rank keeps the
bf16 weight gradients of all quantized linears in ONE flat arena; at the gradient-accumulation boundary the
arena is all-reduced in buckets (NCCL over NVLink on GPUs, gloo in the CPU tests), averaged, and every rank
then runs the same deterministic optimizer + requantize step, so packed codes, residuals and optimizer
states stay bit-identical across replicas without ever broadcasting weights (the stochastic-rounding
dither is keyed by seed / step / parameter, never by rank).
"""
from __future__ import annotations

from typing import Iterable, List, Sequence

import torch
import torch.distributed as dist


class GradArena:
    """Flat gradient buffer with one view per parameter.

    `params` are objects with `.shape` and a writable `.grad` attribute (QuantTensor, FPTensor) or plain
    tensors / nn.Parameters.  `attach()` points every `.grad` at its (zeroed) view, so the reference's backward
    hook — which adds into an existing `.grad` (utils/quant.py:408-411) — accumulates straight into the arena.
    """

    def __init__(self, params: Sequence, dtype=torch.bfloat16, device="cuda", align_elems: int = 128):
        self.params = list(params)
        self.offsets: List[int] = []
        n = 0
        for p in self.params:
            self.offsets.append(n)
            numel = 1
            for d in p.shape:
                numel *= int(d)
            n += (numel + align_elems - 1) // align_elems * align_elems
        self.numel = n
        self.flat = torch.zeros(n, dtype=dtype, device=device)
        self.views = []
        for p, off in zip(self.params, self.offsets):
            numel = 1
            for d in p.shape:
                numel *= int(d)
            self.views.append(self.flat[off:off + numel].view(*[int(d) for d in p.shape]))

    def attach(self) -> None:
        """Zero the arena and make every parameter's `.grad` its view (call at the start of an accumulation cycle)."""
        self.flat.zero_()
        for p, v in zip(self.params, self.views):
            p.grad = v

    def buckets(self, bucket_bytes: int) -> Iterable[torch.Tensor]:
        per = max(1, bucket_bytes // self.flat.element_size())
        for start in range(0, self.numel, per):
            yield self.flat[start:min(self.numel, start + per)]


def _mean_in_collective(flat: torch.Tensor, group) -> bool:
    """NCCL averages inside the collective (`ReduceOp.AVG`); gloo sums, and the caller divides afterwards."""
    return flat.is_cuda and dist.get_backend(group) == "nccl"


def allreduce_mean(arena: GradArena, group=None, bucket_bytes: int = 64 << 20) -> int:
    """Bucketed mean all-reduce of the arena, with the same reduction as `ChunkReducer` (NCCL: `AVG`; gloo: sum, then
    division by the world size), so that the two routes give the same bits at every world size.  Returns the bucket
    count.  NVSwitch gives every peer full bandwidth, so buckets are sized for launch latency / overlap (tens of MB)."""
    if not (dist.is_available() and dist.is_initialized()):
        return 0
    world = dist.get_world_size(group)
    if world == 1:
        return 0
    in_coll = _mean_in_collective(arena.flat, group)
    works = []
    for b in arena.buckets(bucket_bytes):
        works.append(dist.all_reduce(b, op=dist.ReduceOp.AVG if in_coll else dist.ReduceOp.SUM, group=group, async_op=True))
    for w in works:
        w.wait()
    if not in_coll:
        arena.flat.div_(world)
    return len(works)


class ChunkReducer:
    """Mean all-reduce of the arena, range by range, each range launched as soon as its gradients are final.

    `ranges` are (start, end) element ranges of `arena.flat`.  On a GPU every range is reduced on a side stream that
    waits either for the compute stream as it stands at the launch call, or for an event the backward pass records when
    the range is complete — so the transfer overlaps the rest of the backward pass — and `wait(k)` makes the compute
    stream wait for range k only, so the optimizer steps parameters whose gradients have arrived while later ranges
    are still in flight.  With NCCL the division by the world size happens inside the collective; gloo (CPU tests) sums
    and divides afterwards."""

    def __init__(self, arena: GradArena, ranges: Sequence, group=None):
        self.arena, self.group = arena, group
        self.ranges = [(int(a), int(b)) for a, b in ranges]
        self.world = dist.get_world_size(group)
        self.cuda = arena.flat.is_cuda
        self.in_collective_mean = _mean_in_collective(arena.flat, group)
        self.comm = torch.cuda.Stream(device=arena.flat.device) if self.cuda else None
        self.works = [None] * len(self.ranges)
        self.launched = 0

    def begin(self) -> None:
        self.works = [None] * len(self.ranges)
        self.launched = 0

    def launch(self, k: int, after_event=None) -> None:
        a, b = self.ranges[k]
        if b <= a or self.works[k] is not None:
            return
        view = self.arena.flat[a:b]
        op = dist.ReduceOp.AVG if self.in_collective_mean else dist.ReduceOp.SUM
        if self.cuda:
            if after_event is not None:
                self.comm.wait_event(after_event)
            else:
                self.comm.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm):
                self.works[k] = dist.all_reduce(view, op=op, group=self.group, async_op=True)
        else:
            self.works[k] = dist.all_reduce(view, op=op, group=self.group, async_op=True)
        self.launched += 1

    def wait(self, k: int) -> None:
        """Order everything launched on the compute stream from here on after range k's reduction (host-blocking on CPU)."""
        w = self.works[k]
        if w is None or w is True:
            return
        w.wait()
        if not self.in_collective_mean:
            a, b = self.ranges[k]
            self.arena.flat[a:b].div_(self.world)
        self.works[k] = True

    def wait_all(self) -> None:
        for k in range(len(self.ranges)):
            self.wait(k)


def shard_micro_batches(n_micro_batches: int, rank: int, world: int) -> List[int]:
    """DistributedSampler-style assignment (main0.py:387-392): rank r takes micro-batches r, r+W, r+2W, …"""
    return list(range(rank, n_micro_batches, world))


def tensor_hash64(t: torch.Tensor) -> torch.Tensor:
    """Position-sensitive 64-bit hash of a tensor's bytes (int64 scalar on the tensor's device): every 8-byte word is
    multiplied by an odd weight derived from its index and the products are summed modulo 2^64, so swapping two
    different words, or changing one, changes the hash."""
    b = t.detach().contiguous().reshape(-1).view(torch.uint8)
    pad = (-b.numel()) % 8
    if pad:
        b = torch.cat([b, torch.zeros(pad, dtype=torch.uint8, device=b.device)])
    w = b.view(torch.int64)
    idx = torch.arange(w.numel(), dtype=torch.int64, device=w.device)
    weight = (idx * -0x61C8864680B583EB + 0x2545F4914F6CDD1D) | 1         # int64 arithmetic wraps
    mixed = (w ^ (w >> 29)) * weight
    return mixed.sum() + w.numel()


def replicas_identical(tensors: Sequence[torch.Tensor], group=None) -> bool:
    """True when every given tensor holds the same bytes on every rank: one `tensor_hash64` per tensor, compared
    across ranks (max == min)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return True
    hashes = torch.stack([tensor_hash64(t) for t in tensors])
    hi, lo = hashes.clone(), hashes.clone()
    dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
    return bool(torch.equal(hi, lo))


class PeerLostError(RuntimeError):
    """A peer did not reach the step boundary in time (it crashed, hung or left)."""


class StepGate:
    """Host-side liveness check at the step boundary, before any collective is launched.

    Every rank publishes `gate/<run>/<step>/<rank>` in the process group's key-value store and waits (bounded) for the
    same key of every peer.  A rank that died between steps is therefore noticed on the host, with no kernel or
    collective in flight, instead of turning the next all-reduce into a hang.
    """

    def __init__(self, store=None, rank=None, world=None, timeout_s: float = 30.0, nonce: str = "0"):
        """`nonce` names the run: a restarted job that resumes at an earlier step number must not be let through by
        keys its previous incarnation left in a long-lived store."""
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.timeout_s = timeout_s
        self.nonce = str(nonce)

    def arrive_and_wait(self, step: int) -> None:
        import datetime
        self.store.set(f"gate/{self.nonce}/{step}/{self.rank}", "1")
        keys = [f"gate/{self.nonce}/{step}/{r}" for r in range(self.world) if r != self.rank]
        if not keys:
            return
        try:
            self.store.wait(keys, datetime.timedelta(seconds=self.timeout_s))
        except Exception as e:  # the store raises on timeout
            raise PeerLostError(f"rank {self.rank}: a peer did not reach step {step} within {self.timeout_s}s") from e
        # every peer has passed step-1 (it published `step`), so nobody can still be waiting for this rank's key of
        # step-2: drop it, the store does not grow with the run
        if step >= 2:
            try:
                self.store.delete_key(f"gate/{self.nonce}/{step - 2}/{self.rank}")
            except Exception:
                pass                                     # a store without delete support only keeps the key
