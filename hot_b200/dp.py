"""Data-parallel plumbing for the weight gradients.

The HOT backward shards over the batch: every rank runs it on its own tokens with its own
(rank-local) quantisation scales, grad_x needs no communication, and grad_w is a partial sum
over tokens.  The one exchange is therefore an all-reduce of grad_w, as under the reference's
DistributedDataParallel wrapper (ViT_main.py:284-286).  ``GradBuckets`` lays the grad_w of the
layers of one transformer block out back to back in one flat buffer, so that the GEMM epilogues
write straight into the message and one collective per block moves it; the collective is
enqueued as soon as the block's kernels are, and overlaps the next block's backward.

Works with any ``torch.distributed`` backend (NCCL on GPUs; gloo in the CPU tests).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class GradBuckets:
    def __init__(self, block_shapes: Sequence[Sequence[Tuple[int, int]]], dtype: torch.dtype, device,
                 average: bool = False, group: Optional[dist.ProcessGroup] = None):
        """``block_shapes[b]`` lists the (out_features, in_features) of block b's layers in forward
        order.  ``average`` divides by the world size after the sum (DDP's mean)."""
        self.group = group
        self.average = average
        self.buckets: List[torch.Tensor] = []
        self.views: List[List[torch.Tensor]] = []
        for shapes in block_shapes:
            flat = torch.zeros((sum(o * i for o, i in shapes),), dtype=dtype, device=device)
            off, vs = 0, []
            for o, i in shapes:
                vs.append(flat[off:off + o * i].view(o, i))
                off += o * i
            self.buckets.append(flat)
            self.views.append(vs)
        self._works: list = []

    @property
    def world_size(self) -> int:
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def view(self, block: int, layer: int) -> torch.Tensor:
        """The [O, I] destination of one layer's grad_w inside its block's bucket."""
        return self.views[block][layer]

    def reduce_async(self, block: int) -> None:
        """Enqueue the all-reduce of one block's bucket behind the work already enqueued on the
        current stream; returns at once."""
        if self.world_size == 1:
            return
        self._works.append((block, dist.all_reduce(self.buckets[block], op=dist.ReduceOp.SUM, group=self.group,
                                                   async_op=True)))

    def wait_all(self) -> None:
        """Make the current stream (or the host, for CPU backends) wait for every pending
        all-reduce, then apply the averaging if asked for."""
        for block, work in self._works:
            work.wait()
            if self.average:
                self.buckets[block].div_(self.world_size)
        self._works = []

    def message_bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self.buckets)
