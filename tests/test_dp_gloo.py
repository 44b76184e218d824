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


def test_hot_buffers_are_named_for_ddp_to_leave_alone():
    """apply_hot names the hadamard_out / hadamard_bs buffers of every layer it swapped in the attribute
    DistributedDataParallel reads from the module it wraps, so they are not broadcast at every forward; DDP over gloo
    then takes the list (its buffer set has none of them) and a model without HOT layers is left as it is."""
    import torch.nn as nn
    import hot_b200.args as hargs
    from hot_b200.quant_matmul import ddp_ignore_hot_buffers
    from hot_b200.vit import VisionTransformer, apply_hot
    hargs.transform_scheme = "gih_gwlr"
    hargs.lowRankPreset = "half16"
    model = VisionTransformer(img_size=32, patch=16, dim=32, depth=2, heads=2, num_classes=4)
    n = apply_hot(model)
    ignore = model._ddp_params_and_buffers_to_ignore
    assert n == 8 and len(ignore) == 16 and len(set(ignore)) == 16
    assert "blocks.0.attn.qkv.hadamard_out" in ignore and "blocks.1.mlp.fc2.hadamard_bs" in ignore
    buffers = dict(model.named_buffers())
    assert all(name in buffers for name in ignore)
    assert ddp_ignore_hot_buffers(model) == 16 and len(model._ddp_params_and_buffers_to_ignore) == 16   # idempotent
    plain = nn.Sequential(nn.Linear(4, 4))
    assert ddp_ignore_hot_buffers(plain) == 0 and plain._ddp_params_and_buffers_to_ignore == []
