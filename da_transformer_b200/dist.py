"""Data-parallel glue of the hot path: one process per GPU, the batch of sentences is
sharded by rank and the only exchange is one SUM all-reduce of a few scalars.

The ops have no parameters and every sentence is independent, so no tensor ever crosses
GPUs; what the reference all-reduces after the loss is its logging buffer
(fairseq/trainer.py:1453-1491 -> fairseq/distributed/utils.py:634-680, one fp64 buffer).
``all_reduce_stats`` reproduces that collective for the quantities this path produces.
It works with any ``torch.distributed`` backend (NCCL on GPUs, gloo on CPU for tests).
"""
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [start, end) slice of ``n`` sentences owned by ``rank``."""
    per = (n + world - 1) // world
    return min(n, rank * per), min(n, (rank + 1) * per)


def sentence_stats(loss_result: torch.Tensor, target_length: torch.Tensor) -> torch.Tensor:
    """Per-shard statistics as an fp64 vector
    ``[sum_b loss_b / tl_b, sum_b tl_b, n_sentences, n_invalid]``.

    Mirrors fs_plugins/criterions/nat_dag_loss.py:190-194: sentences whose
    log-likelihood is inf/nan are zeroed and counted as invalid.  No host sync.
    The result is detached on every device: these are the LOGGING statistics that get
    all-reduced, not a differentiable loss (``criterion_glue.dag_loss_mean`` is the
    differentiable reduction).
    On the GPU this is one launch of the library (``dat_sentence_stats``) instead of a dozen
    elementwise and reduction launches; CPU tensors (the gloo tests of the multi-process glue)
    take the same expression in torch ops."""
    if loss_result.is_cuda:
        from . import _native
        loss32 = loss_result.detach().to(torch.float32).contiguous()
        tl64 = target_length.to(torch.int64).contiguous()
        stats = torch.empty(4, dtype=torch.float64, device=loss_result.device)
        _native.check(_native.lib().dat_sentence_stats(
            _native.ptr(loss32), _native.ptr(tl64), _native.ptr(stats), int(loss32.numel()),
            _native.stream_ptr(loss_result.device)), "dat_sentence_stats")
        return stats
    loss_result = loss_result.detach()
    invalid = loss_result.isinf().logical_or(loss_result.isnan())
    clean = loss_result.masked_fill(invalid, 0).to(torch.float64)
    tl = target_length.to(torch.float64)
    return torch.stack([
        (clean / tl).sum(),
        tl.sum(),
        clean.new_full((), float(loss_result.numel())),
        invalid.sum().to(torch.float64),
    ])


def all_reduce_stats(stats: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """SUM all-reduce of the statistics vector, enqueued on the current stream (no host
    sync).  A no-op when torch.distributed is not initialised."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.SUM, group=group)
    return stats


def global_loss(stats: torch.Tensor) -> torch.Tensor:
    """The criterion's scalar ``-(loss / target_length).mean()`` over the GLOBAL batch,
    from the reduced statistics."""
    return -(stats[0] / stats[2])


class OverlappedStatsReducer:
    """The statistics all-reduce kept off the compute stream.

    ``all_reduce_stats`` enqueues the collective on the current stream, where it sits between one
    step's last kernel and the next step's first: tens of microseconds of launch and wire latency per
    step for 32 bytes.  Nothing in the next step depends on the reduced numbers (they are logging
    statistics), so ``submit`` copies them into a slot of a small ring and reduces the slot on a side
    stream that only waits for the step that produced them; ``wait`` makes the current stream wait
    for everything submitted so far (call it before reading a returned slot, e.g. once per logging
    interval).  On CPU tensors, or without an initialised process group, ``submit`` reduces at once.
    """

    def __init__(self, device=None, slots: int = 4, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.device = torch.device(device) if device is not None else None
        self.cuda = self.device is not None and self.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.ring = [None] * max(1, int(slots))
        self.next = 0

    def submit(self, stats: torch.Tensor) -> torch.Tensor:
        if not (self.cuda and stats.is_cuda):
            return all_reduce_stats(stats.clone(), self.group)
        k = self.next
        self.next = (k + 1) % len(self.ring)
        if self.ring[k] is None or self.ring[k].shape != stats.shape or self.ring[k].dtype != stats.dtype:
            self.ring[k] = torch.empty_like(stats)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            self.ring[k].copy_(stats, non_blocking=True)
            all_reduce_stats(self.ring[k], self.group)
        return self.ring[k]

    def wait(self) -> None:
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
