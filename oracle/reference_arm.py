"""Times the reference's own CPU implementation of the path: ``HQ_Linear`` forward + backward from
``utils/quant_matmul.py``, unmodified, imported from ``oracle/_ref/`` (see ``oracle/make_ref.py``).

BENCHMARK INFRASTRUCTURE ONLY.  Used by ``bench.py --impl reference`` and by the ``cpu_baseline``
leg of ``bench.py`` (which runs this file as a child process, so that the reference's top-level
``args`` and ``utils`` modules never share an interpreter with the product).

    python oracle/reference_arm.py --tokens 6304 --layers fc1 --steps 3 --warmup 1

prints one JSON object.  The layer runs with the flags of the reference's training script
(main.sh:13-25: gih_gwlr, all four transforms, 4/4/8/8 bits) and the per-tensor stochastic
quantiser on all four operands, on float32 tensors drawn as the single-layer configuration
describes them (activations N(0, 1) with 1 % of the channels scaled by 20, grad_out N(0, 1e-3),
nn.Linear's default weight init), with ``torch.bernoulli`` as it is.  The low-rank basis is the
one the reference derives from the token count (make_WHT: 10 of 32 rows at 6,304 tokens, 36 of 64
at 12,608).  Only the backward is timed; the forward (F.linear + the compressed activation
buffer) runs before the clock starts, as in the GPU arm.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHAPES = {"qkv": (768, 2304), "proj": (768, 768), "fc1": (768, 3072), "fc2": (3072, 768)}


def available() -> bool:
    return os.path.isfile(os.path.join(REF, "utils", "quant_matmul.py"))


def load():
    """(args module, utils.quant_matmul module) of the reference.  matplotlib, which only the
    plotting helpers need, is replaced by three empty stand-in modules when it is not installed."""
    try:
        import matplotlib  # noqa: F401
    except ImportError:
        for name in ("matplotlib", "matplotlib.pyplot", "matplotlib.ticker"):
            m = types.ModuleType(name)
            m.ScalarFormatter = m.LinearLocator = m.MaxNLocator = object
            sys.modules.setdefault(name, m)
        sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
        sys.modules["matplotlib"].ticker = sys.modules["matplotlib.ticker"]
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import args as ref_args
    import utils.quant_matmul as qm
    ref_args.transform_scheme = "gih_gwlr"
    ref_args.TransformGogi = ref_args.TransformWgt = ref_args.TransformGogw = ref_args.TransformInput = True
    ref_args.GogiQuantBit, ref_args.weightQuantBit, ref_args.GogwQuantBit, ref_args.actQuantBit = 4, 4, 8, 8
    ref_args.quantBWDGogi = ref_args.quantBWDWgt = ref_args.quantBWDGogw = ref_args.quantBWDAct = "stoch"
    ref_args.quantAuto = False
    ref_args.BATCH_SIZE = 128   # main.sh; a layer re-derives its basis from the live token count anyway
    return ref_args, qm


class Layer:
    """One reference HQ_Linear with its seeded input and output gradient."""

    def __init__(self, qm, tokens: int, i_f: int, o_f: int, seed: int = 0):
        import torch
        torch.manual_seed(seed)
        self.torch = torch
        self.lin = qm.HQ_Linear(i_f, o_f)
        self.x = torch.randn(tokens, i_f)
        self.x[:, torch.randperm(i_f)[:max(1, round(0.01 * i_f))]] *= 20.0
        self.go = torch.randn(tokens, o_f) * 1e-3

    def backward_seconds(self) -> float:
        x = self.x.clone().requires_grad_(True)
        self.lin.weight.grad = None
        y = self.lin(x)                       # forward: not timed
        t0 = time.perf_counter()
        y.backward(self.go)
        return time.perf_counter() - t0


def run(tokens: int, layers, steps: int, warmup: int, threads: int | None = None) -> dict:
    import torch
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    _, qm = load()
    built = [Layer(qm, tokens, *SHAPES[name]) for name in layers]
    for _ in range(max(warmup, 1)):
        for l in built:
            l.backward_seconds()
    per_step = []
    for _ in range(steps):
        per_step.append(sum(l.backward_seconds() for l in built))
    per_step.sort()
    sec = per_step[len(per_step) // 2]
    flops = float(sum(4 * tokens * SHAPES[n][0] * SHAPES[n][1] for n in layers))
    return {"seconds_per_step": sec, "effective_tops": flops / sec / 1e12, "threads": threads, "tokens": tokens,
            "layers": list(layers), "steps": steps, "warmup": warmup}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=6304)
    ap.add_argument("--layers", default="fc1")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--threads", type=int, default=0)
    a = ap.parse_args()
    if not available():
        print(json.dumps({"unavailable": "oracle/_ref is absent (run oracle/make_ref.py where the reference checkout is mounted)"}))
    else:
        print(json.dumps(run(a.tokens, a.layers.split(","), a.steps, a.warmup, a.threads or None)))
