"""The data-parallel exchange of grad_w on CPU ranks (gloo, world size 2): bucket layout, sum
and mean semantics, and what a rank that raises does to the others (a failure made on the host)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

SHAPES = [[(6, 4), (4, 4), (8, 4), (4, 8)], [(6, 4), (4, 4), (8, 4), (4, 8)]]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, average, fail_rank, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=20))
    try:
        from hot_b200.dp import GradBuckets
        gb = GradBuckets(SHAPES, torch.float32, "cpu", average=average)
        assert gb.world_size == world and gb.message_bytes() == 2 * 4 * (24 + 16 + 32 + 32)
        for b in reversed(range(len(SHAPES))):                 # backward order
            for li in reversed(range(len(SHAPES[b]))):
                if rank == fail_rank and b == 0:
                    raise RuntimeError("injected host-side failure on rank %d" % rank)
                gb.view(b, li).fill_(float((rank + 1) * (10 * b + li + 1)))   # stands in for the GEMM epilogue
            gb.reduce_async(b)
        gb.wait_all()
        total = sum(r + 1 for r in range(world))
        for b in range(len(SHAPES)):
            for li, (o, i) in enumerate(SHAPES[b]):
                want = total * (10 * b + li + 1) / (world if average else 1)
                v = gb.view(b, li)
                assert v.shape == (o, i) and torch.all(v == want), (b, li, v.flatten()[0].item(), want)
            assert gb.buckets[b].data_ptr() == gb.view(b, 0).data_ptr()      # views alias the message
        out.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        out.put((rank, "error: %s" % e))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(average, fail_rank=-1):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, average, fail_rank, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    return res


@pytest.mark.parametrize("average", [False, True])
def test_bucketed_allreduce_two_ranks(average):
    assert _run(average) == {0: "ok", 1: "ok"}


def test_a_rank_that_raises_is_seen_by_its_peer():
    res = _run(False, fail_rank=1)
    assert res[1].startswith("error: injected")
    assert res[0].startswith("error")          # the peer's collective ends with an error, it does not hang


def test_single_process_is_a_no_op():
    from hot_b200.dp import GradBuckets
    gb = GradBuckets(SHAPES[:1], torch.float32, "cpu")
    gb.view(0, 2).fill_(3.0)
    gb.reduce_async(0)
    gb.wait_all()
    assert gb.world_size == 1 and float(gb.view(0, 2)[0, 0]) == 3.0
