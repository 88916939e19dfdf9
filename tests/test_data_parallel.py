"""Host-side logic of the data-parallel path, run as two gloo ranks on CPU: bucket
reduction, double buffering, batch sharding, and failures injected on the host
(mismatched buckets, a rank that never joins) that must surface as errors rather
than hangs.  No GPU is involved and nothing on a device is made to fail."""

import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from substation_b200.data_parallel import BucketMismatch, GradientBucketReducer, shard_batch


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=20):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))


def _worker_reduce(rank, world, port, q):
    try:
        _init(rank, world, port)
        n = 1000
        red = GradientBucketReducer(n * 4, 'cpu', buffers=2, dtype=torch.float32)
        for step in range(5):
            flat = red.arena(step).view(torch.float32)      # waits for this bucket's previous reduction
            flat.copy_(torch.arange(n, dtype=torch.float32) * (rank + 1) + step)
            red.reduce_async(step)
            if step >= 1:                                    # consume the previous step's result
                red.wait(step - 1)
                prev = red.flat(step - 1)
                want = torch.arange(n, dtype=torch.float32) * sum(r + 1 for r in range(world)) + world * (step - 1)
                assert torch.equal(prev, want), f'step {step - 1}'
        red.drain()
        assert red.reductions == 5
        q.put((rank, 'ok'))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _worker_reduce_in_two_parts(rank, world, port, q):
    """The bucket reduced as an early tail part and the rest gives the same sums as one allreduce."""
    try:
        _init(rank, world, port)
        n = 1000
        red = GradientBucketReducer(n * 4, 'cpu', buffers=2, dtype=torch.float32)
        for step in range(4):
            flat = red.arena(step).view(torch.float32)
            flat.copy_(torch.arange(n, dtype=torch.float32) * (rank + 1) + step)
            red.reduce_async(step, early=(4 * 300, None))     # elements 300.. first, then 0..299
            red.wait(step)
            want = torch.arange(n, dtype=torch.float32) * sum(r + 1 for r in range(world)) + world * step
            assert torch.equal(red.flat(step), want), f'step {step}'
        try:
            red.reduce_async(0, early=(3, None))
            raise AssertionError('an offset inside an element must be rejected')
        except ValueError:
            pass
        q.put((rank, 'ok'))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _worker_mismatch(rank, world, port, q):
    try:
        _init(rank, world, port)
        try:
            GradientBucketReducer(1024 if rank == 0 else 2048, 'cpu', dtype=torch.float32)
            q.put((rank, 'no error'))
        except BucketMismatch as e:
            q.put((rank, 'mismatch:' + str(e)[:40]))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _worker_absent_peer(rank, world, port, q):
    """Rank 1 never joins: rank 0's rendezvous must end with an error after its timeout."""
    if rank == 1:
        q.put((rank, 'stayed away'))
        return
    try:
        _init(rank, world, port, timeout_s=3)
        q.put((rank, 'joined?'))
    except Exception as e:
        q.put((rank, 'error:' + type(e).__name__))


def _run(worker, world=2, timeout=90):
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(world):
        r, msg = q.get(timeout=timeout)
        out[r] = msg
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    return out


def test_bucket_allreduce_two_ranks_double_buffered():
    assert _run(_worker_reduce) == {0: 'ok', 1: 'ok'}


def test_bucket_allreduce_in_an_early_part_and_the_rest():
    assert _run(_worker_reduce_in_two_parts) == {0: 'ok', 1: 'ok'}


def test_mismatched_buckets_are_rejected_on_every_rank_before_any_gradient_moves():
    out = _run(_worker_mismatch)
    assert all(v.startswith('mismatch:') for v in out.values()), out


def test_rank_that_never_joins_ends_in_an_error_not_a_hang():
    out = _run(_worker_absent_peer)
    assert out[1] == 'stayed away' and out[0].startswith('error:'), out


def test_single_process_reducer_is_a_no_op():
    red = GradientBucketReducer(64, 'cpu', dtype=torch.float16)
    red.flat(0).fill_(3)
    red.reduce_async(0)
    red.wait(0)
    assert (red.flat(0) == 3).all() and red.reductions == 1
    with pytest.raises(ValueError):
        GradientBucketReducer(63, 'cpu', dtype=torch.float16)


def test_shard_batch_covers_the_batch_once():
    for gb, w in ((96, 8), (10, 4), (7, 8), (64, 1)):
        spans = [shard_batch(gb, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == gb
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_batch(8, 2, 2)
