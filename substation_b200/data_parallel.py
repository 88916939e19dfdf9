"""Data parallelism over batch for the encoder layer.

The reference has no multi-GPU path (no torch.distributed / NCCL / MPI call
anywhere; only its benchmark sweeps are sharded by rank,
pytorch_module/benchmark.py:42-83).  The layer shards naturally over batch:
every operator is independent across samples except the sums over tokens that
produce the 12 parameter gradients.  So each rank (one process per GPU) runs
the unmodified layer on its slice of the batch, and the per-rank gradients,
which the layer writes into ONE flat bucket (12 596 224 fp16 values for
BERT-large), are sum-allreduced.  Sums, not means: each rank's gradient is a
partial sum over its samples, so the reduced bucket equals the gradient of the
global batch; the caller scales if it wants a mean.

``GradientBucketReducer`` double-buffers the bucket so that the allreduce of
step i (NCCL, on its own stream) overlaps the forward/backward of step i+1
(or, in a stack, the backward of the next layer).  It works on any
torch.distributed backend, which is how the host logic is tested on CPU.
"""

import torch
import torch.distributed as dist


class BucketMismatch(RuntimeError):
    """Ranks disagree on the bucket they are about to reduce."""


class GradientBucketReducer:
    def __init__(self, nbytes, device, group=None, buffers=2, dtype=torch.float16, verify=True):
        if buffers < 1:
            raise ValueError('need at least one bucket')
        itemsize = torch.empty((), dtype=dtype).element_size()
        if nbytes % itemsize:
            raise ValueError('bucket size must be a multiple of the element size')
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.nbytes = nbytes
        self.dtype = dtype
        self.arenas = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(buffers)]
        self.pending = [None] * buffers
        self.reductions = 0
        self._side = None   # stream that waits for the mid-pass event of an early part
        if verify and self.world > 1:
            self._verify(device)

    def _verify(self, device):
        """All ranks must hold the same bucket size and dtype; checked with one tiny
        collective before any gradient is touched, so a mismatch is an error message
        on every rank instead of a hang or silent corruption in the data collective."""
        code = torch.tensor([self.nbytes, sum(ord(c) * (i + 1) for i, c in enumerate(str(self.dtype)))], dtype=torch.int64, device=device)
        lo, hi = code.clone(), code.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.group)
        if not torch.equal(lo, hi):
            raise BucketMismatch(f'gradient buckets differ between ranks: this rank has {self.nbytes} bytes of '
                                 f'{self.dtype}; min/max over ranks = {lo.tolist()} / {hi.tolist()}')

    def arena(self, i):
        """uint8 storage of bucket i (hand it to ``Encoder.views`` to lay the gradients into it).
        Waits for a reduction of the same bucket that is still in flight."""
        self.wait(i)
        return self.arenas[i % len(self.arenas)]

    def flat(self, i):
        return self.arenas[i % len(self.arenas)].view(self.dtype)

    def reduce_async(self, i, early=None):
        """Start the sum-allreduce of bucket i (ordered after work already queued on the
        current stream); returns at once.  ``early`` = (byte offset, event): the part of the bucket from that
        offset on is final as soon as ``event`` fires (an event recorded in the middle of the backward pass
        already queued), so its allreduce is queued behind the event only and runs beside the rest of the pass;
        the first part follows as usual."""
        b = i % len(self.arenas)
        if self.pending[b] is not None:
            raise RuntimeError(f'bucket {b} is already being reduced')
        if self.world > 1:
            flat = self.flat(b)
            works = []
            k = 0
            if early is not None:
                off, event = early
                itemsize = flat.element_size()
                if off % itemsize or not 0 <= off <= self.nbytes:
                    raise ValueError('early part must start on an element boundary inside the bucket')
                k = off // itemsize
            if early is not None and 0 < k < flat.numel():
                tail = flat[k:]
                if flat.is_cuda:
                    if self._side is None:
                        self._side = torch.cuda.Stream(flat.device)
                    self._side.wait_event(event)
                    with torch.cuda.stream(self._side):
                        works.append(dist.all_reduce(tail, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
                else:
                    works.append(dist.all_reduce(tail, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
                works.append(dist.all_reduce(flat[:k], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            else:
                works.append(dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            self.pending[b] = works
        self.reductions += 1

    def wait(self, i):
        """Make the current stream (or the host, on CPU backends) wait for bucket i's reduction."""
        b = i % len(self.arenas)
        if self.pending[b] is not None:
            for w in self.pending[b]:
                w.wait()
            self.pending[b] = None

    def drain(self):
        for b in range(len(self.arenas)):
            self.wait(b)


def shard_batch(global_batch, world, rank):
    """Samples [lo, hi) of the global batch that ``rank`` owns (contiguous, sizes differ by at most one)."""
    if not 0 <= rank < world:
        raise ValueError('rank out of range')
    base, extra = divmod(global_batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)
