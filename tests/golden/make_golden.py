"""Generate tests/golden/*.npz by running the UNMODIFIED reference implementation.

Usage (in a container where the reference checkout is mounted):

    python tests/golden/make_golden.py /path/to/reference [section ...]

With section names (``core``, ``lqs_batched``, ``precision``, ``conv``, ``gilro``, ``luq``) only those files are
rewritten; without, all of them.

The reference's ``args.py`` imports ``utils/plot.py`` which needs matplotlib; three
empty stand-in modules are registered before the import so that ``args``,
``utils.hadamard_matmul`` and ``utils.quant_matmul`` import and run as they are.
``torch.bernoulli`` is replaced by ``u < p`` for a supplied uniform tensor ``u`` (on
CPU the two are the same draw), which is what makes the stochastic quantisers
reproducible outside torch.  Nothing here is used at test time: the tests read only
the ``.npz`` files this script wrote.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch


def _import_reference(ref_root: str):
    for name in ("matplotlib", "matplotlib.pyplot", "matplotlib.ticker"):
        m = types.ModuleType(name)
        m.ScalarFormatter = m.LinearLocator = m.MaxNLocator = object
        sys.modules.setdefault(name, m)
    sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
    sys.modules["matplotlib"].ticker = sys.modules["matplotlib.ticker"]
    sys.path.insert(0, ref_root)
    import args as ref_args  # noqa: E402
    import utils.hadamard_matmul as hm  # noqa: E402
    import utils.quant_matmul as qm  # noqa: E402
    return ref_args, hm, qm


class NoiseQueue:
    """Stand-in for torch.bernoulli that consumes supplied uniforms in call order."""

    def __init__(self):
        self.queue: list[torch.Tensor] = []
        self._orig = torch.bernoulli

    def __enter__(self):
        torch.bernoulli = self._draw
        return self

    def __exit__(self, *exc):
        torch.bernoulli = self._orig

    def _draw(self, p):
        u = self.queue.pop(0)
        assert u.shape == p.shape, (u.shape, p.shape)
        return (u < p).to(p.dtype)


def main(ref_root: str, out_dir: str, only=()):
    ref_args, hm, qm = _import_reference(ref_root)
    extra = {"lqs_batched": lqs_batched, "precision": precision_schedule, "conv": conv2d, "gilro": gilro_and_big_order, "luq": luq}
    for name, fn in extra.items():
        if not only or name in only:
            fn(ref_args, hm, qm, out_dir)
    if only and "core" not in only:
        print("golden vectors written to", out_dir, "(sections: %s)" % ", ".join(only))
        return
    rng = np.random.default_rng(20250321)
    T = torch.from_numpy

    # ---- transforms ---------------------------------------------------------
    tr = {}
    for n in (1, 2, 4, 8, 16, 32, 64):
        tr["hadamard_%d" % n] = hm.hadamard(n).astype(np.int8)
    sizes = (768, 2304, 3072, 4096, 11008, 1000, 100, 197, 196, 48, 24)
    tr["make_hadamard_sizes"] = np.array(sizes)
    tr["make_hadamard_orders"] = np.array([hm.make_hadamard(s).shape[0] for s in sizes])
    tr["pow2_max16"] = np.array([hm.biggest_power2_factor_max16(s) for s in sizes])
    tr["pow2"] = np.array([hm.biggest_power2_factor(s) for s in sizes])
    wht_cases = [(6304, 50), (12608, 50), (196, 50), (197, 50), (160, 50), (48, 50), (48, 25), (48, 75),
                 (48, 100), (640, 50), (256, 50), (256, 25), (2, 50), (24, 50)]
    tr["wht_cases"] = np.array(wht_cases)
    for size, pct in wht_cases:
        tr["wht_%d_%d" % (size, pct)] = hm.make_WHT(size, pct).astype(np.int8)
    a = rng.standard_normal((64, 96)).astype(np.float32)
    h16 = torch.tensor(hm.hadamard(16), dtype=torch.float32)
    tr["lower_in"] = a
    tr["lower_front16"] = hm.lowering_matmul_front(T(a), h16).numpy()
    tr["lower_back16"] = hm.lowering_matmul_back(h16, T(a)).numpy()
    p = torch.tensor(hm.make_WHT(64, 50), dtype=torch.float32)       # [r, 64]
    tr["lower_back_wht64"] = hm.lowering_matmul_back(p, T(a)).numpy()
    np.savez_compressed(os.path.join(out_dir, "transforms.npz"), **tr)

    # ---- quantisers ---------------------------------------------------------
    q = {}
    x = (rng.standard_normal((48, 64)) * 1e-3).astype(np.float32)
    x[5] *= 40.0                                                      # an outlier token
    u = rng.random((48, 64), dtype=np.float32)
    q["x"], q["u"] = x, u
    for bits in (4, 8):
        with NoiseQueue() as nq:
            nq.queue.append(T(u))
            c, s = qm.stoch_quantizer(T(x), bits, False)
        q["stoch%d_codes" % bits], q["stoch%d_scale" % bits] = c.numpy(), s.numpy()
        c, s = qm.int_quantizer(T(x), bits, False)
        q["int%d_codes" % bits], q["int%d_scale" % bits] = c.numpy(), s.numpy()
        with NoiseQueue() as nq:
            nq.queue.append(T(u))
            d, one = qm.norm_quantizer(T(x), bits, False)
        q["norm%d_deq" % bits] = d.numpy()
        assert one == 1.0
        c, s = qm.sawb_quantizer(T(x), bits, False)
        q["sawb%d_codes" % bits], q["sawb%d_scale" % bits] = c.numpy(), s.numpy()
    np.savez_compressed(os.path.join(out_dir, "quantizers.npz"), **q)

    # ---- FLinearQ forward context + backward, scheme gih_gwlr ------------------
    for tag, (L, O, I, low_rank) in {"lr_ref": (160, 96, 48, "ref"), "lr_half16": (160, 96, 48, "half16")}.items():
        f = {}
        ref_args.transform_scheme = "gih_gwlr"
        ref_args.TransformGogi = ref_args.TransformWgt = ref_args.TransformGogw = ref_args.TransformInput = True
        ref_args.GogiQuantBit, ref_args.weightQuantBit, ref_args.GogwQuantBit, ref_args.actQuantBit = 4, 4, 8, 8
        ref_args.quantBWDGogi = ref_args.quantBWDWgt = ref_args.quantBWDGogw = ref_args.quantBWDAct = "stoch"
        ref_args.quantAuto = False
        xx = rng.standard_normal((L, I)).astype(np.float32)
        xx[:, 3] *= 20.0
        ww = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
        go = (rng.standard_normal((L, O)) * 1e-3).astype(np.float32)
        h_out = torch.tensor(hm.make_hadamard(O), dtype=torch.float32)
        if low_rank == "ref":
            pm = hm.make_WHT(L, 50)
        else:
            h = hm.hadamard(16)
            seq = [int(np.sum(r[:-1] != r[1:])) for r in h]
            pm = h[np.argsort(seq, kind="stable")[:8]]
        h_bs = torch.tensor(pm, dtype=torch.float32)
        r, n = pm.shape
        Lp = L * r // n
        u_x = rng.random((Lp, I), dtype=np.float32)
        u_go = rng.random((L, O), dtype=np.float32)
        u_w = rng.random((O, I), dtype=np.float32)
        u_gw = rng.random((O, Lp), dtype=np.float32)
        xt = T(xx).requires_grad_(True)
        wt = T(ww).requires_grad_(True)
        with NoiseQueue() as nq:
            nq.queue += [T(u_x), T(u_go), T(u_w), T(u_gw)]
            y = qm.FLinearQ.apply(xt, wt, h_out, h_bs, "layer")
            saved = y.grad_fn.saved_tensors
            y.backward(T(go))
            assert not nq.queue
        f.update(x=xx, w=ww, go=go, p=pm.astype(np.int8), u_x=u_x, u_go=u_go, u_w=u_w, u_gw=u_gw,
                 y=y.detach().numpy(), x_q=saved[0].numpy(), scale_x=saved[4].numpy(),
                 grad_input=xt.grad.numpy(), grad_w=wt.grad.numpy())
        np.savez_compressed(os.path.join(out_dir, "flinearq_%s.npz" % tag), **f)

    # ---- layer-wise quantiser selection rule (ViT_main.py:183-211, restated around
    #      the reference's own quantisers because ViT_main needs timm/peft) ----------
    l = {}
    for tag, g in {"flat": (rng.standard_normal((64, 48)) * 1e-3).astype(np.float32),
                   "outlier": (rng.standard_normal((64, 48)) * 1e-3).astype(np.float32)}.items():
        if tag == "outlier":
            g[7] *= 30.0
        u1 = rng.random(g.shape, dtype=np.float32)
        u2 = rng.random(g.shape, dtype=np.float32)
        errs = []
        with NoiseQueue() as nq:
            nq.queue += [T(u1), T(u2)]
            qg, sg = qm.stoch_quantizer(T(g), 4, False)
            errs.append(float(torch.dist(T(g), qg * sg)))
            qg, sg = qm.norm_quantizer(T(g), 4, False)
            errs.append(float(torch.dist(T(g), qg * sg)))
        choice = "stoch_quantizer"
        if errs[1] < errs[0] and (errs[0] - errs[1]) > errs[0] * 0.5:
            choice = "norm_quantizer"
        l[tag + "_g"], l[tag + "_u1"], l[tag + "_u2"] = g, u1, u2
        l[tag + "_errs"] = np.array(errs)
        l[tag + "_gx"] = np.array(choice)
    np.savez_compressed(os.path.join(out_dir, "lqs.npz"), **l)
    batched(ref_args, hm, qm, out_dir)
    scheme_hadamard(ref_args, hm, qm, out_dir)
    schemes_token_lowrank(ref_args, hm, qm, out_dir)
    schemes_token_lowrank_batched(ref_args, hm, qm, out_dir)
    print("golden vectors written to", out_dir)


def _per_sample(fn_bwd):
    """What torch.vmap over dim 0 of a reference ``*_BWD`` quantiser computes, as a loop (the explicit
    uniforms cannot be fed to torch.bernoulli inside vmap): per-sample results stacked."""
    def f(x, bits, is_batched):
        if not is_batched:
            return fn_bwd(x, bits)
        outs = [fn_bwd(x[b], bits) for b in range(x.shape[0])]
        return torch.stack([o[0] for o in outs]), torch.stack([o[1] for o in outs])
    return f


def schemes_token_lowrank_batched(ref_args, hm, qm, out_dir: str):
    """The token-low-rank schemes on a 3-D input [B, L, I]: projection and expansion run along the
    tokens of each sample, every quantiser of a batched tensor takes one scale per sample."""
    T = torch.from_numpy
    B, L, O, I = 2, 96, 64, 48
    for scheme, seed in (("low_rank", 20250326), ("gilr_gwh", 20250327)):
        rng = np.random.default_rng(seed)
        ref_args.transform_scheme = scheme
        ref_args.TransformGogi = ref_args.TransformWgt = ref_args.TransformGogw = ref_args.TransformInput = True
        ref_args.GogiQuantBit, ref_args.weightQuantBit, ref_args.GogwQuantBit, ref_args.actQuantBit = 4, 4, 8, 8
        ref_args.quantBWDGogi = ref_args.quantBWDWgt = ref_args.quantBWDGogw = ref_args.quantBWDAct = "stoch"
        ref_args.quantAuto = False
        xx = rng.standard_normal((B, L, I)).astype(np.float32)
        xx[1] *= 4.0
        ww = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
        go = (rng.standard_normal((B, L, O)) * 1e-3).astype(np.float32)
        go[0] *= 5.0
        lr = hm.make_WHT(L, 50)
        had = hm.make_hadamard(L)
        if scheme == "low_rank":
            h_out, h_bs = torch.zeros((1, 1)), torch.tensor(lr, dtype=torch.float32)
            Lx = Lw = L * lr.shape[0] // lr.shape[1]
        else:
            h_out, h_bs = torch.tensor(lr, dtype=torch.float32), torch.tensor(had, dtype=torch.float32)
            Lx = Lw = L
        Lg = L * lr.shape[0] // lr.shape[1]
        u_x = rng.random((B, Lx, I), dtype=np.float32)
        u_go = rng.random((B, Lg, O), dtype=np.float32)
        u_w = rng.random((O, I), dtype=np.float32)
        u_gw = rng.random((B, O, Lw), dtype=np.float32)
        xt = T(xx).requires_grad_(True)
        wt = T(ww).requires_grad_(True)
        keep = qm.stoch_quantizer
        qm.stoch_quantizer = _per_sample(qm.stoch_quantizer_BWD)
        try:
            with NoiseQueue() as nq:
                nq.queue += [T(u_x[b]) for b in range(B)] + [T(u_go[b]) for b in range(B)] + [T(u_w)] + \
                            [T(u_gw[b]) for b in range(B)]
                y = qm.FLinearQ.apply(xt, wt, h_out, h_bs, "layer")
                saved = y.grad_fn.saved_tensors
                y.backward(T(go))
                assert not nq.queue
        finally:
            qm.stoch_quantizer = keep
            ref_args.transform_scheme = "gih_gwlr"
        f = dict(x=xx, w=ww, go=go, lowrank=lr.astype(np.int8), hadamard=had.astype(np.int8), u_x=u_x, u_go=u_go, u_w=u_w,
                 u_gw=u_gw, x_q=saved[0].numpy(), scale_x=saved[4].numpy(), grad_input=xt.grad.numpy(),
                 grad_w=wt.grad.numpy())
        np.savez_compressed(os.path.join(out_dir, "flinearq_%s_batched.npz" % scheme), **f)


def schemes_token_lowrank(ref_args, hm, qm, out_dir: str):
    """FLinearQ under transform_scheme "low_rank" and "gilr_gwh": grad_output is projected along the
    tokens for the g_x product too, the weight stays untransformed and grad_input is expanded back
    (utils/quant_matmul.py:229-234, 261-266, 334-337)."""
    T = torch.from_numpy
    L, O, I = 96, 64, 48
    for scheme, seed in (("low_rank", 20250324), ("gilr_gwh", 20250325)):
        rng = np.random.default_rng(seed)
        ref_args.transform_scheme = scheme
        ref_args.TransformGogi = ref_args.TransformWgt = ref_args.TransformGogw = ref_args.TransformInput = True
        ref_args.GogiQuantBit, ref_args.weightQuantBit, ref_args.GogwQuantBit, ref_args.actQuantBit = 4, 4, 8, 8
        ref_args.quantBWDGogi = ref_args.quantBWDWgt = ref_args.quantBWDGogw = ref_args.quantBWDAct = "stoch"
        ref_args.quantAuto = False
        xx = rng.standard_normal((L, I)).astype(np.float32)
        xx[:, 7] *= 12.0
        ww = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
        go = (rng.standard_normal((L, O)) * 1e-3).astype(np.float32)
        lr = hm.make_WHT(L, 50)                                        # [r, n] low-rank rows for 96 tokens
        had = hm.make_hadamard(L)                                      # [16, 16]
        if scheme == "low_rank":
            h_out, h_bs = torch.zeros((1, 1)), torch.tensor(lr, dtype=torch.float32)
            Lx = L * lr.shape[0] // lr.shape[1]                        # tokens of the saved activation
            Lw = Lx                                                    # and of the g_w operand
        else:
            h_out, h_bs = torch.tensor(lr, dtype=torch.float32), torch.tensor(had, dtype=torch.float32)
            Lx = Lw = L
        Lg = L * lr.shape[0] // lr.shape[1]                            # tokens of the projected grad_output (g_x side)
        u_x = rng.random((Lx, I), dtype=np.float32)
        u_go = rng.random((Lg, O), dtype=np.float32)
        u_w = rng.random((O, I), dtype=np.float32)
        u_gw = rng.random((O, Lw), dtype=np.float32)
        xt = T(xx).requires_grad_(True)
        wt = T(ww).requires_grad_(True)
        try:
            with NoiseQueue() as nq:
                nq.queue += [T(u_x), T(u_go), T(u_w), T(u_gw)]
                y = qm.FLinearQ.apply(xt, wt, h_out, h_bs, "layer")
                saved = y.grad_fn.saved_tensors
                y.backward(T(go))
                assert not nq.queue
        finally:
            ref_args.transform_scheme = "gih_gwlr"
        f = dict(x=xx, w=ww, go=go, lowrank=lr.astype(np.int8), hadamard=had.astype(np.int8), u_x=u_x, u_go=u_go, u_w=u_w,
                 u_gw=u_gw, y=y.detach().numpy(), x_q=saved[0].numpy(), scale_x=saved[4].numpy(),
                 grad_input=xt.grad.numpy(), grad_w=wt.grad.numpy())
        np.savez_compressed(os.path.join(out_dir, "flinearq_%s.npz" % scheme), **f)


def scheme_hadamard(ref_args, hm, qm, out_dir: str):
    """FLinearQ under transform_scheme "hadamard": block Hadamard along the tokens (all rows kept)
    instead of the low-rank projection (utils/quant_matmul.py:183-184, 229-230, 261-262, 294-295, 330-331)."""
    rng = np.random.default_rng(20250323)
    T = torch.from_numpy
    L, O, I = 48, 96, 32
    ref_args.transform_scheme = "hadamard"
    ref_args.TransformGogi = ref_args.TransformWgt = ref_args.TransformGogw = ref_args.TransformInput = True
    ref_args.GogiQuantBit, ref_args.weightQuantBit, ref_args.GogwQuantBit, ref_args.actQuantBit = 4, 4, 8, 8
    ref_args.quantBWDGogi = ref_args.quantBWDWgt = ref_args.quantBWDGogw = ref_args.quantBWDAct = "stoch"
    ref_args.quantAuto = False
    xx = rng.standard_normal((L, I)).astype(np.float32)
    xx[:, 5] *= 15.0
    ww = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
    go = (rng.standard_normal((L, O)) * 1e-3).astype(np.float32)
    h_out = torch.tensor(hm.make_hadamard(O), dtype=torch.float32)
    pm = hm.make_hadamard(L)                                           # [16, 16] for 48 tokens
    h_bs = torch.tensor(pm, dtype=torch.float32)
    u_x = rng.random((L, I), dtype=np.float32)
    u_go = rng.random((L, O), dtype=np.float32)
    u_w = rng.random((O, I), dtype=np.float32)
    u_gw = rng.random((O, L), dtype=np.float32)
    xt = T(xx).requires_grad_(True)
    wt = T(ww).requires_grad_(True)
    try:
        with NoiseQueue() as nq:
            nq.queue += [T(u_x), T(u_go), T(u_w), T(u_gw)]
            y = qm.FLinearQ.apply(xt, wt, h_out, h_bs, "layer")
            saved = y.grad_fn.saved_tensors
            y.backward(T(go))
            assert not nq.queue
    finally:
        ref_args.transform_scheme = "gih_gwlr"
    f = dict(x=xx, w=ww, go=go, p=pm.astype(np.int8), u_x=u_x, u_go=u_go, u_w=u_w, u_gw=u_gw, y=y.detach().numpy(),
             x_q=saved[0].numpy(), scale_x=saved[4].numpy(), grad_input=xt.grad.numpy(), grad_w=wt.grad.numpy())
    np.savez_compressed(os.path.join(out_dir, "flinearq_hadamard.npz"), **f)


def batched(ref_args, hm, qm, out_dir: str):
    """FLinearQ on a 3-D input [B, L, I]: the reference quantises every sample with its own scale
    (torch.vmap over dim 0, utils/quant_matmul.py:102-106) and autograd sums the [B, O, I] weight
    gradient over the batch.  ``torch.bernoulli`` cannot be fed explicit uniforms inside vmap, so
    the vmapped wrappers are replaced by a loop that calls the reference's own per-sample
    ``*_BWD`` function on each sample and stacks the results, which is what vmap computes (checked
    below on the deterministic quantiser against the real vmap)."""
    rng = np.random.default_rng(20250322)
    T = torch.from_numpy

    def per_sample(fn_bwd):
        def f(x, bits, is_batched):
            if not is_batched:
                return fn_bwd(x, bits)
            outs = [fn_bwd(x[b], bits) for b in range(x.shape[0])]
            return torch.stack([o[0] for o in outs]), torch.stack([o[1] for o in outs])
        return f

    probe = T(rng.standard_normal((3, 10, 12)).astype(np.float32))
    c_v, s_v = qm.int_quantizer(probe, 8, True)                       # the real vmap
    c_l, s_l = per_sample(qm.int_quantizer_BWD)(probe, 8, True)
    assert torch.equal(c_v, c_l) and torch.equal(s_v, s_l)

    B, L, O, I = 3, 24, 96, 48
    ref_args.transform_scheme = "gih_gwlr"
    ref_args.TransformGogi = ref_args.TransformWgt = ref_args.TransformGogw = ref_args.TransformInput = True
    ref_args.GogiQuantBit, ref_args.weightQuantBit, ref_args.GogwQuantBit, ref_args.actQuantBit = 4, 4, 8, 8
    ref_args.quantBWDGogi = ref_args.quantBWDWgt = ref_args.quantBWDGogw = ref_args.quantBWDAct = "stoch"
    ref_args.quantAuto = False
    xx = rng.standard_normal((B, L, I)).astype(np.float32)
    xx[1] *= 3.0                                                       # samples of different magnitude
    xx[:, :, 3] *= 20.0
    ww = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
    go = (rng.standard_normal((B, L, O)) * 1e-3).astype(np.float32)
    go[2] *= 7.0
    h_out = torch.tensor(hm.make_hadamard(O), dtype=torch.float32)
    pm = hm.make_WHT(L, 50)
    h_bs = torch.tensor(pm, dtype=torch.float32)
    r, n = pm.shape
    Lp = L * r // n
    u_x = rng.random((B, Lp, I), dtype=np.float32)
    u_go = rng.random((B, L, O), dtype=np.float32)
    u_w = rng.random((O, I), dtype=np.float32)
    u_gw = rng.random((B, O, Lp), dtype=np.float32)
    xt = T(xx).requires_grad_(True)
    wt = T(ww).requires_grad_(True)
    keep = qm.stoch_quantizer
    qm.stoch_quantizer = per_sample(qm.stoch_quantizer_BWD)
    try:
        with NoiseQueue() as nq:
            nq.queue += [T(u_x[b]) for b in range(B)] + [T(u_go[b]) for b in range(B)] + [T(u_w)] + \
                        [T(u_gw[b]) for b in range(B)]
            y = qm.FLinearQ.apply(xt, wt, h_out, h_bs, "layer")
            saved = y.grad_fn.saved_tensors
            y.backward(T(go))
            assert not nq.queue
    finally:
        qm.stoch_quantizer = keep
    f = dict(x=xx, w=ww, go=go, p=pm.astype(np.int8), u_x=u_x, u_go=u_go, u_w=u_w, u_gw=u_gw, y=y.detach().numpy(),
             x_q=saved[0].numpy(), scale_x=saved[4].numpy(), grad_input=xt.grad.numpy(), grad_w=wt.grad.numpy())
    np.savez_compressed(os.path.join(out_dir, "flinearq_batched.npz"), **f)

    # the same call with the training script's defaults for the weight and the activation buffer
    # (sawb, ViT_main.py:102,104): the activation's clip is per sample through the reference's own
    # vmap (sawb draws no random numbers), the weight is 2-D and keeps one clip
    ref_args.quantBWDWgt = ref_args.quantBWDAct = "sawb"
    xt = T(xx).requires_grad_(True)
    wt = T(ww).requires_grad_(True)
    qm.stoch_quantizer = per_sample(qm.stoch_quantizer_BWD)
    try:
        with NoiseQueue() as nq:
            nq.queue += [T(u_go[b]) for b in range(B)] + [T(u_gw[b]) for b in range(B)]
            y = qm.FLinearQ.apply(xt, wt, h_out, h_bs, "layer")
            saved = y.grad_fn.saved_tensors
            y.backward(T(go))
            assert not nq.queue
    finally:
        qm.stoch_quantizer = keep
        ref_args.quantBWDWgt = ref_args.quantBWDAct = "stoch"
    f = dict(x=xx, w=ww, go=go, p=pm.astype(np.int8), u_go=u_go, u_gw=u_gw, y=y.detach().numpy(),
             x_q=saved[0].numpy(), scale_x=saved[4].numpy(), grad_input=xt.grad.numpy(), grad_w=wt.grad.numpy())
    np.savez_compressed(os.path.join(out_dir, "flinearq_batched_sawb.npz"), **f)

    # and with the training script's defaults on all four operands (ViT_main.py:101-104: nq, sawb, nq,
    # sawb), which is what runs while layer_quant_dict is still empty: the vmapped norm_quantizer takes
    # one scale per token of each sample on the g_x side and one per sample and output channel on the
    # g_w side, and returns dequantised values with scale 1
    def per_sample_nq(x, bits, is_batched):
        if not is_batched:
            return qm.norm_quantizer_BWD(x, bits), 1.
        return torch.stack([qm.norm_quantizer_BWD(x[b], bits) for b in range(x.shape[0])]), 1.

    ref_args.quantBWDWgt = ref_args.quantBWDAct = "sawb"
    ref_args.quantBWDGogi = ref_args.quantBWDGogw = "nq"
    xt = T(xx).requires_grad_(True)
    wt = T(ww).requires_grad_(True)
    keep_nq = qm.norm_quantizer
    qm.norm_quantizer = per_sample_nq
    try:
        with NoiseQueue() as nq:
            nq.queue += [T(u_go[b]) for b in range(B)] + [T(u_gw[b]) for b in range(B)]
            y = qm.FLinearQ.apply(xt, wt, h_out, h_bs, "layer")
            y.backward(T(go))
            assert not nq.queue
    finally:
        qm.norm_quantizer = keep_nq
        ref_args.quantBWDWgt = ref_args.quantBWDAct = ref_args.quantBWDGogi = ref_args.quantBWDGogw = "stoch"
    f = dict(x=xx, w=ww, go=go, p=pm.astype(np.int8), u_go=u_go, u_gw=u_gw, grad_input=xt.grad.numpy(),
             grad_w=wt.grad.numpy())
    np.savez_compressed(os.path.join(out_dir, "flinearq_batched_nq.npz"), **f)


def _gih_gwlr(ref_args, scheme="stoch"):
    ref_args.transform_scheme = "gih_gwlr"
    ref_args.TransformGogi = ref_args.TransformWgt = ref_args.TransformGogw = ref_args.TransformInput = True
    ref_args.GogiQuantBit, ref_args.weightQuantBit, ref_args.GogwQuantBit, ref_args.actQuantBit = 4, 4, 8, 8
    ref_args.quantBWDGogi = ref_args.quantBWDWgt = ref_args.quantBWDGogw = ref_args.quantBWDAct = scheme
    ref_args.quantAuto = False


def lqs_batched(ref_args, hm, qm, out_dir: str):
    """The selection rule on 3-D first-batch gradients [B, L, O], as the calibration loop applies it
    (ViT_main.py:190-211): both quantisers are called with is_batched=True, so the per-tensor
    quantiser takes one scale per SAMPLE and the error is torch.dist against q * s[:, None, None].
    Case "spread": samples of very different magnitude, where one scale for the whole batch would be
    poor but one per sample is not, so the per-token quantiser must not win.  Case "outlier": one
    outlier token in every sample, where it does."""
    rng = np.random.default_rng(20250328)
    T = torch.from_numpy
    out = {}
    for tag in ("spread", "outlier"):
        g = (rng.standard_normal((6, 24, 48)) * 1e-3).astype(np.float32)
        if tag == "spread":
            g *= np.array([1.0, 1.0, 1.0, 1.0, 1.0, 8.0], dtype=np.float32)[:, None, None]
        else:
            g[:, 5] *= 40.0
        u1 = rng.random(g.shape, dtype=np.float32)
        u2 = rng.random(g.shape, dtype=np.float32)
        errs = []
        with NoiseQueue() as nq:
            nq.queue += [T(u1[b]) for b in range(g.shape[0])] + [T(u2[b]) for b in range(g.shape[0])]
            qg, sg = _per_sample(qm.stoch_quantizer_BWD)(T(g), 4, True)
            errs.append(float(torch.dist(T(g), qg * sg.unsqueeze(1).unsqueeze(2))))
            qg = torch.stack([qm.norm_quantizer_BWD(T(g)[b], 4) for b in range(g.shape[0])])
            errs.append(float(torch.dist(T(g), qg * 1.)))
            assert not nq.queue
        choice = "stoch_quantizer"
        if errs[1] < errs[0] and (errs[0] - errs[1]) > errs[0] * 0.5:
            choice = "norm_quantizer"
        out[tag + "_g"], out[tag + "_u1"], out[tag + "_u2"] = g, u1, u2
        out[tag + "_errs"] = np.array(errs)
        out[tag + "_gx"] = np.array(choice)
    np.savez_compressed(os.path.join(out_dir, "lqs_batched.npz"), **out)


def precision_schedule(ref_args, hm, qm, out_dir: str):
    """utils/utils.py:149-159 run over epochs 0..11 for several flag settings: the four bit widths
    after each call."""
    import utils.utils as uu
    cases = [  # (quantBWDGogi, quantBWDWgt, max_bit, min_bit, milestones)
        ("stoch", "stoch", 8, 4, (3, 6)), ("int", "sawb", 8, 4, (2, 4, 5)), ("nq", "int", 8, 2, (1, 2, 3, 9)),
        ("nq", "sawb", 8, 4, (5,)), ("stoch", "int", 6, 3, (4, 8)), ("stoch", "stoch", 8, 4, ())]
    keep = {k: getattr(ref_args, k) for k in ("GogiQuantBit", "weightQuantBit", "GogwQuantBit", "actQuantBit",
                                              "quantBWDGogi", "quantBWDWgt")}
    table = np.zeros((len(cases), 12, 4), dtype=np.int32)
    for ci, (gogi, wgt, mx, mn, ms) in enumerate(cases):
        ref_args.quantBWDGogi, ref_args.quantBWDWgt = gogi, wgt
        ref_args.GogiQuantBit, ref_args.weightQuantBit, ref_args.GogwQuantBit, ref_args.actQuantBit = 4, 4, 8, 8
        for epoch in range(12):
            uu.precision_scheduler(epoch, mx, mn, list(ms))
            table[ci, epoch] = (ref_args.GogiQuantBit, ref_args.weightQuantBit, ref_args.GogwQuantBit, ref_args.actQuantBit)
    for k, v in keep.items():
        setattr(ref_args, k, v)
    np.savez_compressed(os.path.join(out_dir, "precision_scheduler.npz"), bits=table,
                        cases=np.array([("%s,%s,%d,%d,%s" % (c[0], c[1], c[2], c[3], " ".join(map(str, c[4])))) for c in cases]))


def conv2d(ref_args, hm, qm, out_dir: str):
    """HQ_Conv2d forward + backward (utils/quant_matmul.py:426-488) with the deterministic quantiser
    on all four operands (int_quantizer, vmapped per sample by the reference itself, so no random
    draws are involved): a stride-16 patch embedding (16 tokens per image, basis 10 of 16) and a 3x3
    convolution with padding 1 (64 positions per image, basis 36 of 64)."""
    T = torch.from_numpy
    out = {}
    for tag, (B, cin, cout, hw, k, stride, pad, seed) in {"patch": (4, 3, 64, 64, 16, 16, 0, 20250329),
                                                          "c3x3": (3, 8, 32, 8, 3, 1, 1, 20250330)}.items():
        rng = np.random.default_rng(seed)
        _gih_gwlr(ref_args, "int")
        torch.manual_seed(seed)
        conv = qm.HQ_Conv2d(cin, cout, k, stride=stride, padding=pad)
        x = rng.standard_normal((B, cin, hw, hw)).astype(np.float32)
        x[:, 1] *= 6.0
        xt = T(x).requires_grad_(True)
        y = conv(xt)
        go = (rng.standard_normal(tuple(y.shape)) * 1e-3).astype(np.float32)
        y.backward(T(go))
        out.update({tag + "_x": x, tag + "_w": conv.weight.detach().numpy(), tag + "_b": conv.bias.detach().numpy(),
                    tag + "_go": go, tag + "_y": y.detach().numpy(), tag + "_gx": xt.grad.numpy(),
                    tag + "_gw": conv.weight.grad.numpy(), tag + "_gb": conv.bias.grad.numpy(),
                    tag + "_p": conv.hadamard_bs.numpy().astype(np.int8),
                    tag + "_cfg": np.array([B, cin, cout, hw, k, stride, pad])})
    _gih_gwlr(ref_args, "stoch")
    np.savez_compressed(os.path.join(out_dir, "conv2d.npz"), **out)


def gilro_and_big_order(ref_args, hm, qm, out_dir: str):
    """(1) transform_scheme "gilro_gwh" as the reference can run it: TransformGogi / TransformWgt on (grad_output and
    the weight projected along the output features onto make_WHT(O), whose order is the whole 2-adic part of O),
    TransformInput / TransformGogw off (the reference has no branch for them and raises with them on).  Two widths:
    O = 96 (order 32, 10 rows) and O = 256 (order 256, 136 rows: above what one kernel launch takes).
    (2) gih_gwlr on 384 tokens: make_WHT gives an order-128 token basis (36 rows)."""
    T = torch.from_numpy
    for tag, (L, O, I, seed) in {"o96": (48, 96, 32, 20250331), "o256": (32, 256, 48, 20250401)}.items():
        rng = np.random.default_rng(seed)
        _gih_gwlr(ref_args, "stoch")
        ref_args.transform_scheme = "gilro_gwh"
        ref_args.TransformInput = ref_args.TransformGogw = False
        xx = rng.standard_normal((L, I)).astype(np.float32)
        xx[:, 2] *= 9.0
        ww = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
        go = (rng.standard_normal((L, O)) * 1e-3).astype(np.float32)
        lr = hm.make_WHT(O, 50)
        h_out = torch.tensor(lr, dtype=torch.float32)
        h_bs = torch.tensor(hm.make_hadamard(L), dtype=torch.float32)
        Op = O * lr.shape[0] // lr.shape[1]
        u_x = rng.random((L, I), dtype=np.float32)
        u_go = rng.random((L, Op), dtype=np.float32)
        u_w = rng.random((Op, I), dtype=np.float32)
        u_gw = rng.random((O, L), dtype=np.float32)
        xt = T(xx).requires_grad_(True)
        wt = T(ww).requires_grad_(True)
        try:
            with NoiseQueue() as nq:
                nq.queue += [T(u_x), T(u_go), T(u_w), T(u_gw)]
                y = qm.FLinearQ.apply(xt, wt, h_out, h_bs, "layer")
                saved = y.grad_fn.saved_tensors
                y.backward(T(go))
                assert not nq.queue
        finally:
            _gih_gwlr(ref_args, "stoch")
        np.savez_compressed(os.path.join(out_dir, "flinearq_gilro_%s.npz" % tag), x=xx, w=ww, go=go, lowrank=lr.astype(np.int8),
                            u_x=u_x, u_go=u_go, u_w=u_w, u_gw=u_gw, x_q=saved[0].numpy(), scale_x=saved[4].numpy(),
                            grad_input=xt.grad.numpy(), grad_w=wt.grad.numpy())
    rng = np.random.default_rng(20250402)
    _gih_gwlr(ref_args, "stoch")
    L, O, I = 384, 64, 32
    xx = rng.standard_normal((L, I)).astype(np.float32)
    xx[:, 4] *= 11.0
    ww = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
    go = (rng.standard_normal((L, O)) * 1e-3).astype(np.float32)
    pm = hm.make_WHT(L, 50)
    assert pm.shape[1] == 128
    Lp = L * pm.shape[0] // pm.shape[1]
    u_x, u_go = rng.random((Lp, I), dtype=np.float32), rng.random((L, O), dtype=np.float32)
    u_w, u_gw = rng.random((O, I), dtype=np.float32), rng.random((O, Lp), dtype=np.float32)
    xt = T(xx).requires_grad_(True)
    wt = T(ww).requires_grad_(True)
    with NoiseQueue() as nq:
        nq.queue += [T(u_x), T(u_go), T(u_w), T(u_gw)]
        y = qm.FLinearQ.apply(xt, wt, torch.tensor(hm.make_hadamard(O), dtype=torch.float32), torch.tensor(pm, dtype=torch.float32), "layer")
        saved = y.grad_fn.saved_tensors
        y.backward(T(go))
        assert not nq.queue
    np.savez_compressed(os.path.join(out_dir, "flinearq_lr_ref128.npz"), x=xx, w=ww, go=go, p=pm.astype(np.int8), u_x=u_x, u_go=u_go,
                        u_w=u_w, u_gw=u_gw, x_q=saved[0].numpy(), scale_x=saved[4].numpy(), grad_input=xt.grad.numpy(),
                        grad_w=wt.grad.numpy())


class UniformQueue:
    """Stand-ins for ``torch.rand`` and ``Tensor.uniform_`` that consume supplied uniforms in [0, 1) in call order
    (the two random draws of the reference's luq_quantizer_BWD)."""

    def __init__(self):
        self.queue: list[torch.Tensor] = []
        self._rand, self._uniform_ = torch.rand, torch.Tensor.uniform_

    def __enter__(self):
        q = self.queue

        def rand(*shape, **kw):
            u = q.pop(0)
            assert tuple(u.shape) == tuple(shape[0] if len(shape) == 1 and not isinstance(shape[0], int) else shape)
            return u.clone()

        def uniform_(t, a=0.0, b=1.0):
            u = q.pop(0)
            assert u.shape == t.shape
            return t.copy_(u * (b - a) + a)

        torch.rand, torch.Tensor.uniform_ = rand, uniform_
        return self

    def __exit__(self, *exc):
        torch.rand, torch.Tensor.uniform_ = self._rand, self._uniform_


def luq(ref_args, hm, qm, out_dir: str):
    """The logarithmic quantiser (utils/quant_matmul.py:58-83) alone, and FLinearQ with it on both grad_output
    sides (quantBWDGogi = quantBWDGogw = 'luq'; weight and activation keep the stochastic integer quantiser)."""
    T = torch.from_numpy
    rng = np.random.default_rng(20250403)
    out = {}
    x = (rng.standard_normal((40, 64)) * 1e-3).astype(np.float32)
    x[3] *= 25.0
    u1, u2 = rng.random(x.shape, dtype=np.float32), rng.random(x.shape, dtype=np.float32)
    for bits in (3, 4):
        with UniformQueue() as uq:
            uq.queue += [T(u1), T(u2)]
            q, s = qm.luq_quantizer(T(x), bits, False)
            assert not uq.queue
        out["luq%d_levels" % bits], out["luq%d_scale" % bits] = q.numpy(), s.numpy()
    out.update(x=x, u_prune=u1, u_round=u2)
    L, O, I = 64, 96, 32
    _gih_gwlr(ref_args, "stoch")
    ref_args.quantBWDGogi = ref_args.quantBWDGogw = "luq"
    ref_args.GogwQuantBit = 4      # the scale is mx / 2^(2^(bits-1)-1): at 8 bits the reference's own expression overflows
    xx = rng.standard_normal((L, I)).astype(np.float32)
    ww = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
    go = (rng.standard_normal((L, O)) * 1e-3).astype(np.float32)
    h = hm.hadamard(16)
    seq = [int(np.sum(r[:-1] != r[1:])) for r in h]
    pm = h[np.argsort(seq, kind="stable")[:8]]
    Lp = L // 2
    u_x, u_w = rng.random((Lp, I), dtype=np.float32), rng.random((O, I), dtype=np.float32)
    ug1, ug2 = rng.random((L, O), dtype=np.float32), rng.random((L, O), dtype=np.float32)
    uw1, uw2 = rng.random((O, Lp), dtype=np.float32), rng.random((O, Lp), dtype=np.float32)
    xt, wt = T(xx).requires_grad_(True), T(ww).requires_grad_(True)
    try:
        with NoiseQueue() as nq, UniformQueue() as uq:
            nq.queue += [T(u_x), T(u_w)]
            uq.queue += [T(ug1), T(ug2), T(uw1), T(uw2)]
            y = qm.FLinearQ.apply(xt, wt, torch.tensor(hm.make_hadamard(O), dtype=torch.float32), torch.tensor(pm, dtype=torch.float32), "layer")
            y.backward(T(go))
            assert not nq.queue and not uq.queue
    finally:
        _gih_gwlr(ref_args, "stoch")
    out.update(l_x=xx, l_w=ww, l_go=go, l_p=pm.astype(np.int8), l_u_x=u_x, l_u_w=u_w, l_ug1=ug1, l_ug2=ug2, l_uw1=uw1, l_uw2=uw2,
               l_grad_input=xt.grad.numpy(), l_grad_w=wt.grad.numpy())
    np.savez_compressed(os.path.join(out_dir, "luq.npz"), **out)


if __name__ == "__main__":
    main(sys.argv[1], os.path.dirname(os.path.abspath(__file__)), tuple(sys.argv[2:]))
