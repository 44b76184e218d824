#!/usr/bin/env python
"""Benchmark of the HOT linear-layer backward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl hot|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload ("vit_b16_backward_48_linears_12608_tokens"): one step is the HOT backward of all 48
block linears of ViT-B/16 (12 x {qkv 768->2304, proj 768->768, fc1 768->3072, fc2 3072->768})
at batch 64 = 12,608 tokens per GPU, bf16 tensors, seeded synthetic data: weights with the
nn.Linear default init, grad_out ~ N(0, 1e-3), activations ~ N(0, 1) compressed ahead of time
(the activation buffer is produced in forward, not in backward).  Every layer has its own
grad_out / weight / buffer (2.1 GB per GPU in total, far more than the 126 MB L2), so no layer
finds its inputs in cache.  At N > 1 every rank runs the same step on its own tokens and the
weight gradients are summed over ranks by NCCL, one bucket per transformer block, overlapped
with the remaining backward ("weak" scaling).

The metric is effective TOPS = 4*L*O*I summed over the layers / step time (the FLOPs of the
two full-precision GEMMs the backward replaces), whole job.  ``e2e`` is the same metric
through the public plugin call ``HLQ_backward.backward(Go, W, X, ...)`` with Go and X starting
in pinned host memory and both gradients read back to the host.  One printed JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYERS = (("qkv", 768, 2304), ("proj", 768, 768), ("fc1", 768, 3072), ("fc2", 3072, 768))
METRIC, UNIT = "hot_backward_effective_tops", "TOPS"
WORKLOAD = "vit_b16_backward_48_linears_12608_tokens"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="hot", choices=["hot", "reference"])
    p.add_argument("--tokens", type=int, default=12608)
    p.add_argument("--blocks", type=int, default=12)
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    p.add_argument("--e2e-steps", type=int, default=2)
    p.add_argument("--gx-storage", default="auto", choices=["int4", "int8", "auto"],
                   help="how the 4-bit g_x codes of grad_out are stored between the quantiser and the GEMM: packed two per "
                        "byte and expanded in shared memory, one per byte, or (default) the library's policy "
                        "ops.gx_code_storage: packed where the contraction is 4096 or longer")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--sm-margin", type=int, default=-1,
                   help="SMs left out of the persistent kernels' grids for the all-reduce kernels (multi-GPU; default 0)")
    p.add_argument("--bucket-blocks", type=int, default=0,
                   help="transformer blocks per all-reduce bucket (multi-GPU); 0: three, six from 8 GPUs on (measured: "
                        "3.70 ms per step with three against 3.88 with one at 2 GPUs; 3.93 / 3.92 / 3.90 with three / four / six at 8)")
    p.add_argument("--dp-breakdown", action="store_true",
                   help="multi-GPU: also time the step without the all-reduces and the all-reduces alone")
    p.add_argument("--no-kernels", action="store_true", help="skip the per-kernel roofline legs")
    p.add_argument("--sweep", action="store_true",
                   help="instead of the step: the stand-alone fused Hadamard+quantise sweep (M x K x order x "
                        "format x rounding x scale x dtype), one JSON line with a table of GB/s")
    p.add_argument("--vit-train", action="store_true",
                   help="instead of the step: data-parallel ViT-B/16 training step (forward, HOT backward on the 48 "
                        "block linears, DDP all-reduce, SGD), images/s, beside the same model with plain nn.Linear")
    p.add_argument("--batch", type=int, default=256, help="images per GPU for --vit-train")
    p.add_argument("--one-layer", default=None, choices=["qkv", "proj", "fc1", "fc2"],
                   help="run --calls HOT backward calls of one ViT-B/16 linear shape and nothing else (for ncu captures)")
    p.add_argument("--calls", type=int, default=3)
    p.add_argument("--schemes", action="store_true", help="one fc1 backward under each built transform_scheme")
    p.add_argument("--per-sample", action="store_true",
                   help="the reference's 3-D semantics (one scale per image) on the ViT-B/16 linear shapes")
    p.add_argument("--large-mlp", action="store_true",
                   help="instead of the step: HOT backward vs bf16 matmul on large transformer MLP linears "
                        "(16384 tokens; 4096->11008, 11008->4096, 4096->4096; heavy-tailed outlier channels)")
    return p.parse_args()


# kernels one layer backward launches: grad_out abs-max pass + quantise pass (the weight's abs-max and codes come
# out of the same two launches) and one persistent kernel for both integer GEMMs (memset nodes are not kernels);
# in fp32 the weight has two kernels of its own on the helper stream
KERNELS_PER_LAYER = {"bf16": 3, "fp32": 5}


def step_flops(tokens: int, blocks: int) -> float:
    return float(sum(4 * tokens * o * i for _, i, o in LAYERS) * blocks)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm=float(d["hbm_gbs"]), bf16=float(d["bf16_tflops"]), bf16_sustained=float(d["bf16_tflops_sustained"]),
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi sampling SM clock and throttle reasons every 20 ms.  It is started well before the timed region
    (nvidia-smi takes a few hundred ms to begin, longer on a box with 8 GPUs, and the timed region of the default run
    is under 100 ms) and its lines carry a timestamp: `stop` reports the samples that fall between `mark_start` and
    `mark_end`, or, if the region was too short to catch one, the ones nearest to it."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        self.t0 = self.t1 = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime
        rows = []   # (time, sm MHz, max MHz, reasons)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            f = [v.strip() for v in line.split(",")]
            if len(f) < 8:
                continue
            try:
                t = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((t, float(f[1]), float(f[2]), {n for n, v in zip(names, f[4:8]) if v.lower().startswith("active")}))
            except ValueError:
                continue
        if not rows:
            return None
        window = "timed region"
        t0, t1 = self.t0 or rows[0][0], self.t1 or rows[-1][0]
        inside = [r for r in rows if t0 <= r[0] <= t1]
        if not inside:   # a region shorter than the sampling period: the two samples nearest to it
            mid = 0.5 * (t0 + t1)
            inside = sorted(rows, key=lambda r: abs(r[0] - mid))[:2]
            window = "nearest samples (%.0f ms from the region)" % (1e3 * min(abs(r[0] - mid) for r in inside))
        sm = [r[1] for r in inside]
        reasons = set().union(*[r[3] for r in inside])
        busy = [v for v in sm if v > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(r[2] for r in inside), "reasons": sorted(reasons),
                "samples": len(inside), "window": window}


# ---------------------------------------------------------------------------------------------
# the hot arm
# ---------------------------------------------------------------------------------------------
def build_layers(ops, tokens, blocks, dtype, device, rank, gx_storage="int4"):
    """Per block and layer: weight, grad_out, compressed activation, config."""
    from hot_b200.hadamard_matmul import biggest_power2_factor_max16, lowrank_selection
    gw_seed = torch.Generator(device=device).manual_seed(0)            # same weights on every rank
    gd = torch.Generator(device=device).manual_seed(1000 + rank)       # own data per rank
    order_l, sel = lowrank_selection(tokens, "half16")
    layers = []
    call = 0
    for b in range(blocks):
        blk = []
        for name, i_f, o_f in LAYERS:
            bound = 1.0 / (i_f ** 0.5)                                 # kaiming_uniform(a=sqrt(5)) == U(-1/sqrt(in), +)
            w = ((torch.rand((o_f, i_f), device=device, generator=gw_seed) * 2 - 1) * bound).to(dtype)
            go = (torch.randn((tokens, o_f), device=device, generator=gd) * 1e-3).to(dtype)
            x = torch.randn((tokens, i_f), device=device, generator=gd).to(dtype)
            call += 4
            cfg = ops.LinearConfig(order_o=biggest_power2_factor_max16(o_f), order_l=order_l, sel_l=sel,
                                   q_gx=ops.Quant(4, ops.gx_code_storage(4, o_f) if gx_storage == "auto" else gx_storage,
                                                  "philox", "tensor", 0, call + 1),
                                   q_w=ops.Quant(4, "int4", "philox", "tensor", 0, call + 2),
                                   q_gw=ops.Quant(8, "int8", "philox", "tensor", 0, call + 3),
                                   q_x=ops.Quant(8, "int8", "philox", "tensor", 0, call + 4))
            x_q_t, s_x = ops.abc_compress(x, cfg)
            del x
            blk.append(dict(name=name, w=w, go=go, x_q_t=x_q_t, s_x=s_x, cfg=cfg, I=i_f, O=o_f))
        layers.append(blk)
    torch.cuda.synchronize(device)
    return layers


def run_hot(a):
    import torch.distributed as dist
    from hot_b200 import ops
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the HOT kernels have no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    margin = 0 if a.sm_margin < 0 else a.sm_margin   # measured on 2 GPUs: leaving SMs to the collective costs more than it saves
    if world > 1:
        if margin > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(margin))   # the collective's kernels fit the SMs left free for them
        dist.init_process_group("nccl", device_id=device)
    ops.set_sm_margin(margin)
    dtype = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    pk = peaks()
    sampler = ClockSampler(local) if rank == 0 else None   # started here: it needs a while before its first line
    layers = build_layers(ops, a.tokens, a.blocks, dtype, device, rank, a.gx_storage)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    # gradient buffers: grad_x is consumed by the layer below (one reusable buffer per width);
    # grad_w lands in one flat bucket per block, the unit of the all-reduce
    from hot_b200.dp import GradBuckets
    gx_buf = {i_f: torch.empty((a.tokens, i_f), dtype=dtype, device=device) for _, i_f, _ in LAYERS}
    # a bucket holds the grad_w of `per` consecutive blocks (fewer, larger collectives); the blocks run from the top
    # down, so the bucket that ends the step is cut down to block 0 alone: its all-reduce has nothing to hide behind
    per = max(1, min(a.bucket_blocks if a.bucket_blocks > 0 else (6 if world >= 8 else 3), a.blocks))
    bounds = list(range(a.blocks, 0, -per))[::-1]            # upper ends, ascending: e.g. 3, 6, 9, 12
    lows = [max(hi - per, 0) for hi in bounds]
    if lows[0] == 0 and bounds[0] > 1:
        lows, bounds = [0, 1] + lows[1:], [1] + bounds       # [0, 1) and [1, first upper end)
    bucket_of, first_of = {}, {}
    for j, (lo, hi) in enumerate(zip(lows, bounds)):
        for b in range(lo, hi):
            bucket_of[b] = (j, b - lo)
        first_of[lo] = j
    n_buckets = len(bounds)
    grads = GradBuckets([[(o_f, i_f) for b in range(lo, hi) for _, i_f, o_f in LAYERS] for lo, hi in zip(lows, bounds)],
                        dtype, device)

    def block_backward(b):
        j, k = bucket_of[b]
        for li in reversed(range(len(LAYERS))):
            l = layers[b][li]
            ops.linear_backward(l["go"], l["w"], l["x_q_t"], l["s_x"], l["cfg"], status=status,
                                gx_out=gx_buf[l["I"]], gw_out=grads.view(j, k * len(LAYERS) + li))

    # one CUDA graph per transformer block: launch overhead off the critical path, and the
    # all-reduce of a block's bucket can be enqueued between graph launches
    side = torch.cuda.Stream(device)
    graphs = []
    with torch.cuda.stream(side):
        for b in range(a.blocks):
            block_backward(b)                       # warm-up outside capture (lazy init, attributes)
        torch.cuda.synchronize(device)
        for b in range(a.blocks):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                block_backward(b)
            graphs.append(g)
    torch.cuda.synchronize(device)

    def step(reduce=True):
        for b in reversed(range(a.blocks)):
            graphs[b].replay()
            if reduce and b in first_of:           # the bucket's last block (blocks run from the top down) is enqueued
                grads.reduce_async(first_of[b])
        grads.wait_all()

    def reduce_only():
        for j in reversed(range(n_buckets)):
            grads.reduce_async(j)
        grads.wait_all()

    def sync_all():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    for _ in range(max(a.warmup, 3)):
        step()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.mark_start()
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    sync_all()
    if sampler:
        sampler.mark_end()
    ms = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if sampler else None
    ms_step = float(ms.item()) / a.steps
    breakdown = None
    if world > 1 and a.dp_breakdown:
        def timed(fn):
            sync_all()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(a.steps):
                fn()
            t1.record()
            sync_all()
            v = torch.tensor([t0.elapsed_time(t1)], device=device)
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
            return round(float(v.item()) / a.steps, 4)
        breakdown = {"ms_step_without_all_reduce": timed(lambda: step(False)), "ms_all_reduce_alone": timed(reduce_only),
                     "ms_step": round(ms_step, 4)}
    if int(status.item()) != 0:
        raise SystemExit("a bounded device-side wait ran out during the benchmark (status %d)" % int(status.item()))
    flops = step_flops(a.tokens, a.blocks)
    value = flops * world / (ms_step * 1e-3) / 1e12
    n_layers = a.blocks * len(LAYERS)

    out = {"metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": a.steps,
           "warmup": max(a.warmup, 3), "ms_per_step": round(ms_step, 4), "ms_per_layer": round(ms_step / n_layers, 5),
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8/int4 codes, int32 accumulate",
           "data": "synthetic", "gpu_launches": n_layers * KERNELS_PER_LAYER[a.dtype] * a.steps,
           "config": {"workload": WORKLOAD, "tokens_per_gpu": a.tokens, "layers": n_layers, "tensor_dtype": a.dtype,
                      "hadamard_order": 16, "low_rank": "8 of 16 (lowest sequency)", "g_x": "INT4 x INT4, per-tensor, Philox stochastic" + {"int4": "; grad_out codes packed", "int8": "; grad_out codes stored one per byte", "auto": "; grad_out codes stored one per byte (packed only where the contraction is 4096 or longer)"}[a.gx_storage],
                      "g_w": "INT8 x INT8, per-tensor, Philox stochastic", "activation_buffer": "compressed in forward (not timed)",
                      "cache": "inputs 2.1 GB per GPU, distinct per layer (> 126 MB L2)",
                      "parallelism": ("dp%d, grad_w all-reduce (NCCL) in %d buckets of up to %d blocks (%.1f MB per block; the last one holds "
                                      "block 0 alone), %d SMs left to the collective"
                                      % (world, n_buckets, per, grads.message_bytes() / a.blocks / 1e6, margin))
                      if world > 1 else "single GPU"}}
    if breakdown:
        out["dp_breakdown"] = breakdown
    if clocks:
        out["clocks"] = clocks
    if rank == 0:
        # the per-kernel legs and the roofline at every GPU count (rank 0's GPU alone, the other ranks wait in the
        # end-to-end leg's first barrier); the CPU baseline at one GPU only
        if not a.no_kernels:
            out["kernels"], out["roofline"], out["fp_backward_bf16_cublas"] = kernel_legs(ops, layers, a, dtype, device, pk, status)
        if not a.no_cpu_baseline and world == 1:
            out["cpu_baseline"] = cpu_baseline(threads=os.cpu_count() or 1)
    out["e2e"] = e2e_leg(layers, a, dtype, device, flops, world) if a.e2e_steps > 0 else None   # every rank takes part
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_sweep(a):
    """Benchmark configuration 2 of the target: the fused transform + quantise kernel alone.  Algorithmic bytes per launch:
    M*K*sizeof(in) + M*K*bits/8 + 4 (per tensor) or + 4*M (per token), over the CUDA-event time."""
    from hot_b200 import ops
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    pk = peaks()
    rows = []
    g = torch.Generator(device=device).manual_seed(0)
    for dt_name, dt in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        for M in (4096, 16384, 65536):
            for K in (768, 1024, 4096, 8192):
                x = torch.randn((M, K), device=device, generator=g).to(dt)
                for order in (16, 32, 64):
                    for fmt, bits in (("int4", 4), ("int8", 8)):
                        for rounding in ("philox", "nearest"):
                            for scale in ("tensor", "row"):
                                q = ops.Quant(bits, fmt, rounding, scale, 0, 1)
                                fn = lambda: ops.row_ht_quant(x, order, q)
                                for _ in range(2):
                                    fn()
                                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                                torch.cuda.synchronize(device)
                                n_it = 5
                                e0.record()
                                for _ in range(n_it):
                                    fn()
                                e1.record()
                                torch.cuda.synchronize(device)
                                us = e0.elapsed_time(e1) * 1e3 / n_it
                                nbytes = M * K * x.element_size() + M * K * bits // 8 + (4 * M if scale == "row" else 4)
                                rows.append(dict(dtype=dt_name, M=M, K=K, order=order, fmt=fmt, rounding=rounding, scale=scale,
                                                 us=round(us, 1), gbs=round(nbytes / us / 1e3, 1)))
                del x
    best = max(rows, key=lambda r: r["gbs"])
    big = [r for r in rows if r["M"] * r["K"] >= 16384 * 4096]          # tensors larger than L2

    def med(sel):
        v = sorted(r["gbs"] for r in big if sel(r))
        return v[len(v) // 2] if v else None
    summary = {"%s_%s_%s" % (d, rd, sc): med(lambda r: r["dtype"] == d and r["rounding"] == rd and r["scale"] == sc)
               for d in ("bf16", "fp32") for rd in ("philox", "nearest") for sc in ("tensor", "row")}
    print(json.dumps({"metric": "fused_hadamard_quant_hbm_gbs", "unit": "GB/s", "value": best["gbs"], "best": best,
                      "median_gbs_large_tensors": summary, "peak": pk["hbm"], "peak_source": pk["source"] + " hbm_gbs",
                      "frac_best": round(best["gbs"] / pk["hbm"], 4), "cases": len(rows), "table": rows,
                      "note": "eager launches: cases under ~50 us include host launch latency"}), flush=True)


def run_large_mlp(a):
    """Benchmark configuration 4 of the target: large MLP linears in bf16 at 16384 tokens, activations with heavy-tailed
    outlier channels (1 % of channels scaled by |Student-t(3)| draws), compressed activation buffer."""
    from hot_b200 import ops
    from hot_b200.hadamard_matmul import lowrank_selection
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.manual_seed(0)
    M = 16384
    order_l, sel = lowrank_selection(M, "half16")
    status = torch.zeros(1, dtype=torch.int32, device=device)
    out = []
    for i_f, o_f in ((4096, 11008), (11008, 4096), (4096, 4096)):
        x = torch.randn((M, i_f), device=device)
        idx = torch.randperm(i_f, device=device)[:max(1, i_f // 100)]
        x[:, idx] *= torch.distributions.StudentT(3.0).sample((idx.numel(),)).abs().to(device) * 10.0
        x = x.to(torch.bfloat16)
        w = ((torch.rand((o_f, i_f), device=device) * 2 - 1) / i_f ** 0.5).to(torch.bfloat16)
        go = (torch.randn((M, o_f), device=device) * 1e-3).to(torch.bfloat16)
        cfg = ops.LinearConfig(order_o=16, order_l=order_l, sel_l=sel)
        x_q_t, s_x = ops.abc_compress(x, cfg)
        t_hot = _graph_time(lambda i: ops.linear_backward(go, w, x_q_t, s_x, cfg, status=status), 3, device, warm=1)
        t_fp = _graph_time(lambda i: (torch.matmul(go, w), torch.matmul(go.t(), x)), 3, device, warm=1)
        gx, gw = ops.linear_backward(go, w, x_q_t, s_x, cfg, status=status)
        ex, ew = torch.matmul(go, w).float(), torch.matmul(go.t(), x).float()
        cos = lambda p_, q_: float(torch.nn.functional.cosine_similarity(p_.float().flatten(), q_.flatten(), dim=0))
        flops = 4.0 * M * i_f * o_f
        out.append({"in": i_f, "out": o_f, "hot_us": round(t_hot, 1), "bf16_matmul_us": round(t_fp, 1),
                    "speedup_vs_bf16": round(t_fp / t_hot, 3), "hot_effective_tops": round(flops / t_hot / 1e6, 1),
                    "activation_buffer_bytes": int(x_q_t.numel()), "activation_bytes_bf16": int(x.numel() * 2),
                    "cos_gx_vs_fp": round(cos(gx, ex), 4), "cos_gw_vs_fp": round(cos(gw, ew), 4)})
        del x, w, go, x_q_t, gx, gw, ex, ew
    torch.cuda.synchronize(device)
    if int(status.item()) != 0:
        raise SystemExit("a bounded device-side wait ran out")
    print(json.dumps({"metric": "hot_backward_large_mlp", "tokens": M, "dtype": "bf16", "layers": out}), flush=True)


def run_schemes(a):
    """The four transform schemes built on the native path, on the fc1 shape (768 -> 3072) at --tokens
    tokens, bf16: time of one layer backward (CUDA graph replay) and agreement with the exact gradients."""
    from hot_b200 import ops
    from hot_b200.hadamard_matmul import lowrank_selection
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.manual_seed(0)
    L, i_f, o_f = a.tokens, 768, 3072
    x = torch.randn((L, i_f), device=device).to(torch.bfloat16)
    w = ((torch.rand((o_f, i_f), device=device) * 2 - 1) / i_f ** 0.5).to(torch.bfloat16)
    go = (torch.randn((L, o_f), device=device) * 1e-3).to(torch.bfloat16)
    ex, ew = torch.matmul(go, w).float(), torch.matmul(go.t(), x).float()
    cos = lambda p_, q_: float(torch.nn.functional.cosine_similarity(p_.float().flatten(), q_.flatten(), dim=0))
    n_lr, sel_lr = lowrank_selection(L, None, 50)          # the reference's make_WHT rows for this token count
    full16 = (16, list(range(16)))
    status = torch.zeros(1, dtype=torch.int32, device=device)
    out = []
    for scheme, gw_basis, gx_basis in (("gih_gwlr", (n_lr, sel_lr), None), ("hadamard", full16, None),
                                       ("low_rank", (n_lr, sel_lr), (n_lr, sel_lr)), ("gilr_gwh", full16, (n_lr, sel_lr))):
        cfg = ops.LinearConfig(order_o=16 if gx_basis is None else 1, order_l=gw_basis[0], sel_l=gw_basis[1])
        x_q_t, s_x = ops.abc_compress(x, cfg)

        def layer():
            if gx_basis is None:
                return ops.linear_backward(go, w, x_q_t, s_x, cfg, status=status)
            gw_ = ops.linear_backward(go, w, x_q_t, s_x, cfg, need_gx=False, status=status)[1]
            return ops.linear_backward_lowrank_gx(go, w, gx_basis[0], gx_basis[1], cfg.q_gx, cfg.q_w, status=status), gw_
        t = _graph_time(lambda i: layer(), 5, device, warm=2)
        gx, gw = layer()
        out.append({"scheme": scheme, "token_basis_gw": "%d of %d" % (len(gw_basis[1]), gw_basis[0]),
                    "token_basis_gx": None if gx_basis is None else "%d of %d" % (len(gx_basis[1]), gx_basis[0]),
                    "layer_us": round(t, 1), "cos_gx_vs_fp": round(cos(gx, ex), 4), "cos_gw_vs_fp": round(cos(gw, ew), 4)})
    torch.cuda.synchronize(device)
    if int(status.item()) != 0:
        raise SystemExit("a bounded device-side wait ran out")
    print(json.dumps({"metric": "hot_backward_schemes", "tokens": L, "in": i_f, "out": o_f, "dtype": "bf16", "layers": out}),
          flush=True)


def run_one_layer(a):
    """--calls HOT backward calls of one ViT-B/16 linear shape at --tokens tokens: a small, fixed
    launch sequence (per call: grad_out abs-max pass, grad_out quantise pass, weight abs-max and
    quantise, g_x GEMM, g_w GEMM) for profiler captures."""
    from hot_b200 import ops
    from hot_b200.hadamard_matmul import lowrank_selection
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.manual_seed(0)
    dtype = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    i_f, o_f = {"qkv": (768, 2304), "proj": (768, 768), "fc1": (768, 3072), "fc2": (3072, 768)}[a.one_layer]
    L = a.tokens
    order_l, sel = lowrank_selection(L, "half16")
    x = torch.randn((L, i_f), device=device).to(dtype)
    w = ((torch.rand((o_f, i_f), device=device) * 2 - 1) / i_f ** 0.5).to(dtype)
    go = (torch.randn((L, o_f), device=device) * 1e-3).to(dtype)
    storage = ops.gx_code_storage(4, o_f) if a.gx_storage == "auto" else a.gx_storage   # as the benchmark step stores them
    cfg = ops.LinearConfig(order_o=16, order_l=order_l, sel_l=sel, q_gx=ops.Quant(4, storage))
    x_q_t, s_x = ops.abc_compress(x, cfg)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    for _ in range(a.calls):
        ops.linear_backward(go, w, x_q_t, s_x, cfg, status=status)
    torch.cuda.synchronize(device)
    if int(status.item()) != 0:
        raise SystemExit("a bounded device-side wait ran out")
    print(json.dumps({"one_layer": a.one_layer, "tokens": L, "in": i_f, "out": o_f, "dtype": a.dtype, "calls": a.calls}), flush=True)


def run_per_sample(a):
    """The reference's 3-D semantics (one scale per image, grad_w summed over the batch) on the four
    linear shapes of ViT-B/16 at 64 images x 197 tokens, bf16, beside the flattened path (one scale for
    all 12,608 tokens, half16 low-rank) and the bf16 matmul backward.  With 197 tokens per image the
    reference's own low-rank basis is the identity (197 is odd), so this path carries no low-rank
    compression: its g_w GEMM contracts over 64 x 256 padded tokens."""
    from hot_b200 import ops
    from hot_b200.hadamard_matmul import lowrank_selection
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.manual_seed(0)
    B, L = 64, 197
    n_ps, sel_ps = lowrank_selection(L, None, 50)
    n_fl, sel_fl = lowrank_selection(B * L, "half16")
    status = torch.zeros(1, dtype=torch.int32, device=device)
    out = []
    for i_f, o_f in ((768, 2304), (768, 768), (768, 3072), (3072, 768)):
        x = torch.randn((B, L, i_f), device=device).to(torch.bfloat16)
        w = ((torch.rand((o_f, i_f), device=device) * 2 - 1) / i_f ** 0.5).to(torch.bfloat16)
        go = (torch.randn((B, L, o_f), device=device) * 1e-3).to(torch.bfloat16)
        cfg_ps = ops.LinearConfig(order_o=16, order_l=n_ps, sel_l=sel_ps)
        cfg_fl = ops.LinearConfig(order_o=16, order_l=n_fl, sel_l=sel_fl)
        xq_ps, sx_ps, _ = ops.abc_compress_batched(x, cfg_ps)
        xq_fl, sx_fl = ops.abc_compress(x.view(B * L, i_f), cfg_fl)
        go2, x2 = go.view(B * L, o_f), x.view(B * L, i_f)
        t_ps = _graph_time(lambda i: ops.linear_backward_batched(go, w, xq_ps, sx_ps, cfg_ps, status=status), 5, device, warm=2)
        t_fl = _graph_time(lambda i: ops.linear_backward(go2, w, xq_fl, sx_fl, cfg_fl, status=status), 5, device, warm=2)
        t_fp = _graph_time(lambda i: (torch.matmul(go2, w), torch.matmul(go2.t(), x2)), 5, device, warm=2)
        gx, gw = ops.linear_backward_batched(go, w, xq_ps, sx_ps, cfg_ps, status=status)
        ex, ew = torch.matmul(go2, w).float(), torch.matmul(go2.t(), x2).float()
        cos = lambda p_, q_: float(torch.nn.functional.cosine_similarity(p_.float().flatten(), q_.flatten(), dim=0))
        flops = 4.0 * B * L * i_f * o_f
        out.append({"in": i_f, "out": o_f, "per_sample_us": round(t_ps, 1), "flattened_us": round(t_fl, 1),
                    "bf16_matmul_us": round(t_fp, 1), "per_sample_effective_tops": round(flops / t_ps / 1e6, 1),
                    "cos_gx_vs_fp": round(cos(gx, ex), 4), "cos_gw_vs_fp": round(cos(gw, ew), 4)})
    torch.cuda.synchronize(device)
    if int(status.item()) != 0:
        raise SystemExit("a bounded device-side wait ran out")
    print(json.dumps({"metric": "hot_backward_per_sample", "images": B, "tokens_per_image": L, "dtype": "bf16",
                      "layers": out}), flush=True)


def run_vit_train(a):
    """Benchmark configuration 5 of the target: synthetic 224x224x3 images N(0,1), 100 random classes, random-init ViT-B/16
    in bf16, cross-entropy, SGD; per GPU `--batch` images (256 -> 50,432 tokens).  One process per
    GPU, gradients all-reduced by DistributedDataParallel over NCCL as in the reference."""
    import torch.distributed as dist
    import torch.nn as nn
    import hot_b200.args as hargs
    from hot_b200.vit import apply_hot, vit_base_patch16_224
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    margin = 0 if a.sm_margin < 0 else a.sm_margin
    if world > 1:
        if margin > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(margin))
        dist.init_process_group("nccl", device_id=device)
    from hot_b200 import ops as _ops
    _ops.set_sm_margin(margin)
    hargs.transform_scheme = "gih_gwlr"
    hargs.TransformGogi = hargs.TransformWgt = hargs.TransformGogw = hargs.TransformInput = True
    hargs.GogiQuantBit, hargs.weightQuantBit, hargs.GogwQuantBit, hargs.actQuantBit = 4, 4, 8, 8
    hargs.quantBWDGogi = hargs.quantBWDWgt = hargs.quantBWDGogw = hargs.quantBWDAct = "stoch"
    hargs.lowRankPreset = "half16"
    g = torch.Generator(device=device).manual_seed(1000 + rank)
    x = torch.randn((a.batch, 3, 224, 224), device=device, generator=g)
    y = torch.randint(0, 100, (a.batch,), device=device, generator=g)
    results = {}
    for mode in ("hot", "bf16"):
        torch.manual_seed(0)                                    # same weights on every rank and in both modes
        model = vit_base_patch16_224(100).to(device=device, dtype=torch.bfloat16)
        n_hot = apply_hot(model) if mode == "hot" else 0
        net = nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
        opt = torch.optim.SGD(net.parameters(), lr=1e-3)

        def step():
            opt.zero_grad(set_to_none=True)
            loss = nn.functional.cross_entropy(net(x.to(torch.bfloat16)).float(), y)
            loss.backward()
            opt.step()
            return loss

        for _ in range(max(a.warmup, 3)):
            step()
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        steps = min(a.steps, 10)
        e0.record()
        for _ in range(steps):
            loss = step()
        e1.record()
        torch.cuda.synchronize(device)
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        results[mode] = dict(ms_per_step=round(float(ms.item()), 3), images_per_s=round(a.batch * world / float(ms.item()) * 1e3, 1),
                             loss=round(float(loss.item()), 4), hot_layers=n_hot,
                             peak_mem_gb=round(torch.cuda.max_memory_allocated(device) / 2 ** 30, 2))
        del model, net, opt
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats(device)
    if rank == 0:
        print(json.dumps({"metric": "vit_b16_train_images_per_s", "unit": "images/s", "value": results["hot"]["images_per_s"],
                          "n_gpus": world, "scaling": "weak", "higher_is_better": True, "data": "synthetic", "dtype": "bf16",
                          "config": {"workload": "vit_b16_dp_train_step", "images_per_gpu": a.batch, "tokens_per_gpu": a.batch * 197,
                                     "optimizer": "SGD", "hot": "48 block linears, half16 low-rank, INT4 g_x / INT8 g_w, Philox"},
                          "hot": results["hot"], "plain_bf16_linear": results["bf16"],
                          "hot_vs_plain": round(results["hot"]["images_per_s"] / results["bf16"]["images_per_s"], 3)}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _graph_time(fn, iters, device, warm=3, replays=3):
    """Average device time of fn(i) in microseconds: the calls fn(0) .. fn(iters - 1) captured back to back in one
    CUDA graph (so that what is timed is the kernels as they follow one another in a step, not a graph launch per
    call), replayed `replays` times after `warm` warm-up replays."""
    side = torch.cuda.Stream(device)
    keep = []
    with torch.cuda.stream(side):
        fn(0)
        torch.cuda.synchronize(device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(iters):
                keep.append(fn(i))
        for _ in range(warm):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        e0.record(side)
        for _ in range(replays):
            g.replay()
        e1.record(side)
        torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) * 1e3 / (iters * replays)


def kernel_legs(ops, layers, a, dtype, device, pk, status):
    """Per-kernel device times on the fc1 layers (one distinct layer per launch, so inputs come
    from HBM), the roofline of the kernel with the largest share, and the bf16 cuBLAS backward
    of the same layer for comparison."""
    fc1 = [blk[2] for blk in layers]
    n = len(fc1)
    L, O, I = a.tokens, fc1[0]["O"], fc1[0]["I"]
    esz = 2 if dtype == torch.bfloat16 else 4
    cfg = fc1[0]["cfg"]
    lp = cfg.out_len(L)
    kern = {}
    # kernel A: Hadamard along O + INT4, per-tensor (two launches: abs-max, quantise)
    t = _graph_time(lambda i: ops.row_ht_quant(fc1[i % n]["go"], 16, cfg.q_gx), n, device)
    kern["row_ht_quant_int4_tensor"] = dict(us=t, bytes=L * O * esz + L * O // 2 + 4, bound="hbm")
    q_row = ops.Quant(4, "int4", "philox", "row", 0, 7)
    t = _graph_time(lambda i: ops.row_ht_quant(fc1[i % n]["go"], 16, q_row), n, device)
    kern["row_ht_quant_int4_token"] = dict(us=t, bytes=L * O * esz + L * O // 2 + 4 * L, bound="hbm")
    q_near = ops.Quant(8, "int8", "nearest", "row", 0, 7)
    t = _graph_time(lambda i: ops.row_ht_quant(fc1[i % n]["go"], 16, q_near), n, device)
    kern["row_ht_quant_int8_token_nearest"] = dict(us=t, bytes=L * O * esz + L * O + 4 * L, bound="hbm")
    # kernel B: low-rank along tokens + INT8, transposed out
    t = _graph_time(lambda i: ops.col_ht_quant(fc1[i % n]["go"], cfg.order_l, cfg.sel_l, cfg.q_gw, "transposed"), n, device)
    kern["col_hla_quant_int8_go"] = dict(us=t, bytes=L * O * esz + lp * O, bound="hbm")
    t = _graph_time(lambda i: ops.col_ht_quant(fc1[i % n]["w"], 16, list(range(16)), ops.Quant(4, "int8", "philox", "tensor", 0, 9), "natural"), n, device)
    kern["col_ht_quant_w"] = dict(us=t, bytes=O * I * esz + O * I, bound="hbm")
    # the fused pair the layer runs on grad_out (stats pass + quantise pass, both operands)
    t = _graph_time(lambda i: ops.go_dual_quant(fc1[i % n]["go"], cfg), n, device)
    gx_bytes = L * O // 2 if cfg.q_gx.storage == "int4" else L * O     # g_x codes packed two per byte, or one per byte
    kern["go_dual_quant"] = dict(us=t, bytes=L * O * esz + gx_bytes + lp * O + 8, bound="hbm")
    # kernel C: the two integer GEMMs
    q_go, s_go = ops.row_ht_quant(fc1[0]["go"], 16, cfg.q_gx)
    q_w8 = ops.Quant(4, "int8", "philox", "tensor", 0, 9)          # the layer keeps weight codes one per byte
    q_w, s_w, _ = ops.col_ht_quant(fc1[0]["w"], 16, list(range(16)), q_w8, "natural")
    q_gw, s_gw, _ = ops.col_ht_quant(fc1[0]["go"], cfg.order_l, cfg.sel_l, cfg.q_gw, "transposed")
    t = _graph_time(lambda i: ops.gemm_i8(q_go, cfg.q_gx.storage, q_w, "int8", L, I, O, s_go, s_w, 1 / 16, dtype, status), 8, device)
    kern["gemm_gx_4bit_codes_%s" % ("packed" if cfg.q_gx.storage == "int4" else "one_per_byte")] = dict(us=t, ops=2 * L * I * O, bound="tensor")
    t = _graph_time(lambda i: ops.gemm_i8(q_gw, "int8", fc1[0]["x_q_t"], "int8", O, I, lp, s_gw, fc1[0]["s_x"], 1 / 16, dtype, status), 8, device)
    kern["gemm_gw_int8"] = dict(us=t, ops=2 * O * I * lp, bound="tensor")
    # what the layer launches: both products in one persistent kernel
    g_main = dict(a=q_go, a_storage=cfg.q_gx.storage, b=q_w, M=L, N=I, K=O, scale_a=s_go, scale_b=s_w, post=1 / 16, out_dtype=dtype)
    g_rider = dict(a=q_gw, b=fc1[0]["x_q_t"], M=O, N=I, K=lp, scale_a=s_gw, scale_b=fc1[0]["s_x"], post=1 / 16, out_dtype=dtype)
    t = _graph_time(lambda i: ops.gemm_i8_dual(g_main, g_rider, status), 8, device)
    kern["gemm_gx_gw_one_launch"] = dict(us=t, ops=2 * L * I * O + 2 * O * I * lp, bound="tensor")
    t_layer = _graph_time(lambda i: ops.linear_backward(fc1[i % n]["go"], fc1[i % n]["w"], fc1[i % n]["x_q_t"], fc1[i % n]["s_x"], cfg, status=status), n, device)
    xs = [torch.randn((L, I), device=device).to(dtype) for _ in range(2)]
    # the forward side: the activation buffer of the layer's input (not part of the timed step)
    t = _graph_time(lambda i: ops.abc_compress(xs[i % 2], cfg), 8, device)
    kern["abc_compress_x"] = dict(us=t, bytes=L * I * esz + lp * I, bound="hbm")
    t_fp = _graph_time(lambda i: (torch.matmul(fc1[i % n]["go"], fc1[i % n]["w"]), torch.matmul(fc1[i % n]["go"].t(), xs[i % 2])), n, device)
    # the INT8 ceiling the GEMM fractions are quoted against: measured here, in this run, on a square 8192^3
    # problem by the library GEMM (torch._int_mm) and by this repo's kernel; the larger of the two
    int8 = int8_ceiling(ops, device, status)
    int8_peak = max(int8["torch_int_mm_tops"] or 0.0, int8["hot_gemm_i8_tops"] or 0.0) or 2.0 * pk["bf16"]
    for k, v in kern.items():
        v["us"] = round(v["us"], 2)
        if v["bound"] == "hbm":
            v["achieved"], v["unit"], v["peak"] = round(v["bytes"] / v["us"] / 1e3, 1), "GB/s", pk["hbm"]
        else:
            v["achieved"], v["unit"], v["peak"] = round(v["ops"] / v["us"] / 1e6, 1), "TOP/s", int8_peak
        v["frac"] = round(v["achieved"] / v["peak"], 4)
    # what a layer backward launches (in fp32 the weight has kernels of its own; in bf16 it is quantised inside the
    # two grad_out launches)
    in_layer = ["go_dual_quant", "gemm_gx_gw_one_launch"] + ([] if dtype == torch.bfloat16 else ["col_ht_quant_w"])
    top = max(in_layer, key=lambda k: kern[k]["us"])
    tk = kern[top]
    # DRAM traffic per launch pair, from ncu captures of this very workload (fc1 gradient, 12,608 x 3,072 bf16,
    # `bench.py --one-layer fc1`, cold caches).  g_x codes one per byte: pass 0 read 82.2 MB + wrote 2.4 MB, pass 1 read
    # 82.3 MB + wrote 20.5 MB (the rest of its 58 MB of codes were still in L2 when it ended), of which 11.8 MB are the
    # weight that the layer's launches carry and this leg does not: 175.6 MB for 135.6 MB of algorithmic bytes.  Packed
    # two per byte: 162.0 MB for 116.2 MB.  Scaled by the algorithmic bytes for other token counts.  No figure for the
    # other kernels.
    scale = 162.0 / 116.2 if cfg.q_gx.storage == "int4" else 175.6 / 135.6
    traffic = round(tk["bytes"] * scale) if top == "go_dual_quant" and dtype == torch.bfloat16 else None
    roof = {"kernel": top + (" (two launches: abs-max pass + quantise pass)" if top == "go_dual_quant" else ""),
            "bound": tk["bound"], "achieved": tk["achieved"], "peak": tk["peak"], "unit": tk["unit"],
            "frac": tk["frac"], "traffic": traffic, "launch_us": tk["us"],
            "peak_source": ("%s hbm_gbs" % pk["source"]) if tk["bound"] == "hbm" else
                           "INT8 ceiling measured in this run at 8192^3 (max of torch._int_mm and hot_gemm_i8)",
            "share_of_fc1_layer": round(tk["us"] / t_layer, 3)}
    kern["int8_ceiling_8192"] = int8
    # the other three linears of a block, and the block as a whole, against the same two cuBLAS products
    shapes = {"fc1": {"hot_us": round(t_layer, 2), "matmul_us": round(t_fp, 2)}}
    for li, name in ((0, "qkv"), (1, "proj"), (3, "fc2")):
        ls = [blk[li] for blk in layers]
        xs_l = [torch.randn((L, ls[0]["I"]), device=device).to(dtype) for _ in range(2)]
        th = _graph_time(lambda i: ops.linear_backward(ls[i % n]["go"], ls[i % n]["w"], ls[i % n]["x_q_t"], ls[i % n]["s_x"], ls[i % n]["cfg"], status=status), n, device)
        tf = _graph_time(lambda i: (torch.matmul(ls[i % n]["go"], ls[i % n]["w"]), torch.matmul(ls[i % n]["go"].t(), xs_l[i % 2])), n, device)
        shapes[name] = {"hot_us": round(th, 2), "matmul_us": round(tf, 2)}
        del xs_l
    blk_hot = sum(v["hot_us"] for v in shapes.values())
    blk_fp = sum(v["matmul_us"] for v in shapes.values())
    fp = {"fc1_hot_us": round(t_layer, 2), "fc1_bf16_matmul_us": round(t_fp, 2), "speedup": round(t_fp / t_layer, 3),
          "dtype": a.dtype, "per_linear": shapes,
          "block_hot_us": round(blk_hot, 1), "block_matmul_us": round(blk_fp, 1), "block_speedup": round(blk_fp / blk_hot, 3),
          "config1_fp32": config1_leg(ops, device, status)}
    return kern, roof, fp


def int8_ceiling(ops, device, status):
    """Dense INT8 throughput on an 8192 x 8192 x 8192 problem: torch._int_mm (the library GEMM) and this
    repo's hot_gemm_i8 (raw int32 output), TOP/s each (None where a path is not available)."""
    n = 8192
    a = torch.randint(-8, 8, (n, n), device=device, dtype=torch.int8)
    b = torch.randint(-8, 8, (n, n), device=device, dtype=torch.int8)
    out = {"torch_int_mm_tops": None, "hot_gemm_i8_tops": None, "ops": 2 * n ** 3}
    try:
        bt = b.t()                                                       # column-major second operand
        t = _graph_time(lambda i: torch._int_mm(a, bt), 4, device)
        out["torch_int_mm_tops"] = round(2.0 * n ** 3 / t / 1e6, 1)
    except Exception as e:                                               # pragma: no cover
        out["torch_int_mm_error"] = str(e)[:120]
    au, bu = a.view(torch.uint8), b.view(torch.uint8)
    t = _graph_time(lambda i: ops.gemm_i8(au, "int8", bu, "int8", n, n, n, None, None, out_dtype=torch.int32, status=status), 4, device)
    out["hot_gemm_i8_tops"] = round(2.0 * n ** 3 / t / 1e6, 1)
    return out


def config1_leg(ops, device, status):
    """Benchmark configuration 1 of the target: one ViT-B/16 fc1 backward in fp32, X [6304, 768] N(0,1) with 1 % of the
    channels scaled x20, W kaiming-uniform, grad_out N(0, 1e-3); Hadamard order 16, INT4 g_x with
    stochastic rounding, 8-of-16 low-rank INT8 g_w; beside the fp32 matmul backward (TF32 off)."""
    from hot_b200.hadamard_matmul import lowrank_selection
    g = torch.Generator(device=device).manual_seed(0)
    L, I, O = 6304, 768, 3072
    x = torch.randn((L, I), device=device, generator=g)
    x[:, torch.randperm(I, device=device, generator=g)[:8]] *= 20.0
    w = (torch.rand((O, I), device=device, generator=g) * 2 - 1) / I ** 0.5
    gos = [torch.randn((L, O), device=device, generator=g) * 1e-3 for _ in range(4)]   # 4 x 77 MB > L2
    order_l, sel = lowrank_selection(L, "half16")
    cfg = ops.LinearConfig(order_o=16, order_l=order_l, sel_l=sel)
    x_q_t, s_x = ops.abc_compress(x, cfg)
    t_hot = _graph_time(lambda i: ops.linear_backward(gos[i % 4], w, x_q_t, s_x, cfg, status=status), 4, device)
    t_fp32 = _graph_time(lambda i: (torch.matmul(gos[i % 4], w), torch.matmul(gos[i % 4].t(), x)), 4, device)
    return {"hot_us": round(t_hot, 1), "fp32_matmul_us": round(t_fp32, 1), "speedup_vs_fp32": round(t_fp32 / t_hot, 2),
            "effective_tops": round(4.0 * L * I * O / t_hot / 1e6, 1)}


def e2e_leg(layers, a, dtype, device, flops, world=1):
    """The same step through HLQ_backward.backward with Go and X in pinned host memory and both
    gradients copied back, every layer, every step; the copies of neighbouring layers overlap the
    call (two copy streams), as a caller streaming a model through the plugin would arrange it."""
    import torch.distributed as dist
    import HLQ_backward
    shapes = {}
    for name, i_f, o_f in LAYERS:
        shapes[name] = dict(go=torch.empty((a.tokens, o_f), dtype=dtype).pin_memory(),
                            x=torch.empty((a.tokens, i_f), dtype=dtype).pin_memory(),
                            gx=torch.empty((a.tokens, i_f), dtype=dtype).pin_memory(),
                            gw=torch.empty((o_f, i_f), dtype=dtype).pin_memory())
        shapes[name]["go"].normal_(0, 1e-3)
        shapes[name]["x"].normal_(0, 1)
    h2d = d2h = 0
    for name, i_f, o_f in LAYERS:
        h2d += (a.tokens * o_f + a.tokens * i_f) * shapes[name]["go"].element_size()
        d2h += (a.tokens * i_f + o_f * i_f) * shapes[name]["go"].element_size()
    h2d *= a.blocks
    d2h *= a.blocks

    # The caller's side of the pipeline: while layer k runs, the inputs of layer k + 1 come up on one
    # copy stream and the gradients of layer k - 1 go down on another (PCIe carries both directions).
    comp = torch.cuda.current_stream(device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    order = [(b, li) for b in reversed(range(a.blocks)) for li in reversed(range(len(LAYERS)))]

    def upload(k):
        l = layers[order[k][0]][order[k][1]]
        s = shapes[l["name"]]
        with torch.cuda.stream(s_in):
            go = s["go"].to(device, non_blocking=True)
            x = s["x"].to(device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(s_in)
        return l, s, go, x, ev

    def step():
        nxt = upload(0)
        for k in range(len(order)):
            l, s, go, x, ev = nxt
            if k + 1 < len(order):
                nxt = upload(k + 1)
            comp.wait_event(ev)
            go.record_stream(comp)
            x.record_stream(comp)
            gx, gw, _ = HLQ_backward.backward(go, l["w"], x, 0, 0, 16, False)   # returns with gx, gw complete
            with torch.cuda.stream(s_out):
                s["gx"].copy_(gx, non_blocking=True)
                s["gw"].copy_(gw, non_blocking=True)
            gx.record_stream(s_out)
            gw.record_stream(s_out)
        torch.cuda.synchronize(device)

    step()
    # timed on the device: the events sit on the compute stream, which joins both copy streams before
    # the closing one; with several ranks every rank streams its own shard and the slowest one counts
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(comp)
    for _ in range(a.e2e_steps):
        step()
    comp.wait_stream(s_in)
    comp.wait_stream(s_out)
    e1.record(comp)
    torch.cuda.synchronize(device)
    ms = torch.tensor([e0.elapsed_time(e1) / a.e2e_steps], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    dt = float(ms.item()) * 1e-3
    return {"value": round(flops * world / dt / 1e12, 3), "unit": UNIT, "ms_per_step": round(dt * 1e3, 3),
            "h2d_bytes_per_step": int(h2d) * world, "d2h_bytes_per_step": int(d2h) * world,
            "api": "HLQ_backward.backward(Go, W, X, 0, 0, 16, False)"}


# ---------------------------------------------------------------------------------------------
# the CPU arm: the oracle's restatement of the reference fake-quant path
# ---------------------------------------------------------------------------------------------
def cpu_layer_seconds(tokens, i_f, o_f, seed=0):
    import numpy as np
    from oracle import hot_oracle as oc
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((tokens, i_f)).astype(np.float32)
    w = ((rng.random((o_f, i_f)) * 2 - 1) / np.sqrt(i_f)).astype(np.float32)
    go = (rng.standard_normal((tokens, o_f)) * 1e-3).astype(np.float32)
    sel = oc.lowrank_preset(16, 8)
    lp = tokens // 16 * 8
    u = [rng.random(s, dtype=np.float32) for s in ((lp, i_f), (tokens, o_f), (o_f, i_f), (o_f, lp))]
    x_q, s_x = oc.abc_compress(x, 16, sel, 8, u[0])                     # forward side, not timed
    t0 = time.perf_counter()
    oc.linear_backward(go, w, x_q, s_x, n_o=oc.block_order(o_f), n_l=16, sel=sel, u_go=u[1], u_w=u[2], u_gw=u[3],
                       exact_matmul=False)
    return time.perf_counter() - t0


def cpu_baseline(threads):
    """The reference's own fake-quant backward on the host cores, on a bounded sample: one fc1 layer
    (768 -> 3072) at 6,304 tokens, float32 (the single-layer configuration).  Runs
    ``oracle/reference_arm.py`` as a child process (the reference's top-level ``args`` / ``utils``
    modules stay out of this interpreter); falls back to the numpy port when ``oracle/_ref`` is absent."""
    import subprocess
    tokens, (name, i_f, o_f) = 6304, LAYERS[2]
    root = os.path.dirname(os.path.abspath(__file__))
    if os.path.isfile(os.path.join(root, "oracle", "_ref", "utils", "quant_matmul.py")):
        r = subprocess.run([sys.executable, os.path.join(root, "oracle", "reference_arm.py"), "--tokens", str(tokens), "--layers",
                            "fc1", "--steps", "5", "--warmup", "1", "--threads", str(threads)], capture_output=True, text=True,
                           timeout=600)
        try:
            d = json.loads(r.stdout.strip().splitlines()[-1])
            return {"value": round(d["effective_tops"], 5), "unit": UNIT, "cores": d["threads"], "kind": "reference",
                    "seconds": round(d["seconds_per_step"], 3),
                    "sample": "one fc1 (768->3072) backward at 6304 tokens, fp32: the reference's HQ_Linear (utils/quant_matmul.py) "
                              "with its own low-rank basis (10 of 32 rows), stoch quantisers, median of 5 after 1 warm-up"}
        except Exception:                                 # fall through to the port, and say so
            pass
    from threadpoolctl import threadpool_limits
    with threadpool_limits(limits=threads):
        cpu_layer_seconds(256, i_f, o_f)
        sec = cpu_layer_seconds(tokens, i_f, o_f)
    return {"value": round(4.0 * tokens * i_f * o_f / sec / 1e12, 5), "unit": UNIT, "cores": threads, "kind": "port",
            "seconds": round(sec, 3),
            "sample": "one fc1 (768->3072) backward at 6304 tokens, fp32, oracle/hot_oracle.py linear_backward "
                      "(numpy restatement of utils/quant_matmul.py:214-348 with float32 BLAS matmuls as the reference runs)"}


def run_reference(a):
    """The reference arm: the reference's own CPU implementation of the path (``HQ_Linear`` of
    utils/quant_matmul.py, imported unmodified from ``oracle/_ref``) on all host threads; a step is one
    backward of each of the four layer shapes at the workload's token count, i.e. one of the 12
    transformer blocks (the token count is halved until a run of steps + warm-up fits a few minutes).
    Falls back to the numpy port where ``oracle/_ref`` is absent.  Rank 0 only."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    threads = os.cpu_count() or 1
    root = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, root)
    kind = "port"
    names = [n for n, _, _ in LAYERS]
    tokens = a.tokens
    if os.path.isfile(os.path.join(root, "oracle", "_ref", "utils", "quant_matmul.py")):
        from oracle import reference_arm
        kind = "reference"
        probe = reference_arm.run(1576, names, 1, 1, threads)["seconds_per_step"]       # 1/8 of the tokens
        budget = 200.0 / max(a.steps + max(a.warmup, 1), 1)
        while tokens > 1576 and probe * (tokens / 1576.0) > budget:
            tokens //= 2
        res = reference_arm.run(tokens, names, a.steps, a.warmup, threads)
        sec = res["seconds_per_step"]
        how = "the reference's HQ_Linear (utils/quant_matmul.py, unmodified, from oracle/_ref), its own low-rank basis"
    else:
        tokens = 1600
        for _, i_f, o_f in LAYERS:
            cpu_layer_seconds(64, i_f, o_f)
        for _ in range(max(a.warmup, 0)):
            for _, i_f, o_f in LAYERS:
                cpu_layer_seconds(tokens, i_f, o_f)
        t0 = time.perf_counter()
        for _ in range(a.steps):
            for _, i_f, o_f in LAYERS:
                cpu_layer_seconds(tokens, i_f, o_f)
        sec = (time.perf_counter() - t0) / a.steps
        how = "oracle/hot_oracle.py (numpy restatement; oracle/_ref absent)"
    flops = float(sum(4 * tokens * o * i for _, i, o in LAYERS))
    value = round(flops / sec / 1e12, 5)
    sample = ("per step: one backward of each of the 4 layer shapes (one of the 12 blocks) at %d tokens, fp32, %s"
              % (tokens, how))
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": a.gpus,
                      "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "f32 holding integer codes", "data": "synthetic",
                      "config": {"workload": WORKLOAD, "sample": sample},
                      "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
                      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.sweep:
        run_sweep(args)
    elif args.large_mlp:
        run_large_mlp(args)
    elif args.per_sample:
        run_per_sample(args)
    elif args.one_layer:
        run_one_layer(args)
    elif args.schemes:
        run_schemes(args)
    elif args.vit_train:
        run_vit_train(args)
    else:
        run_hot(args)
