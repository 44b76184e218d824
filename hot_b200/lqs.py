"""Layer-wise quantiser selection (LQS): a calibration pass that decides, per HOT layer, whether
grad_output is quantised with one scale per tensor or one per token on the g_x path
(ViT_main.py:44-56, 133-215 and the first-batch capture of utils/plot.py:164-204).

The rule, unchanged: quantise the UN-transformed first-batch grad_output to 4 bits with the
per-tensor stochastic quantiser and with the per-token one; per-token wins for g_x only if it
cuts the L2 error by more than half; g_w always keeps the per-tensor quantiser.  A 3-D
grad_output [B, L, O] (every linear of a ViT block) is quantised "batched", as the reference
calls it there (ViT_main.py:190-201): the per-tensor quantiser then takes one scale per sample.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional

import torch
import torch.nn as nn

from .quant_matmul import HQ_Conv2d, HQ_Linear, _args, norm_quantizer, stoch_quantizer

quantScheme_gx = ["stoch_quantizer", "norm_quantizer"]


class FirstBatchCapture:
    """Keeps the first grad_output each named layer sees (the reference's ``Tensor_Dict``
    stores a tensor only while its slot still holds the initial sentinel)."""

    def __init__(self):
        self.grad_out: Dict[str, torch.Tensor] = {}
        self._handles = []

    def attach(self, model: nn.Module) -> "FirstBatchCapture":
        for name, layer in model.named_modules():
            if isinstance(layer, (HQ_Linear, HQ_Conv2d)):   # the reference hooks both (ViT_main.py:51-56)
                self._handles.append(layer.register_full_backward_hook(self._hook(name)))
        return self

    def _hook(self, name: str):
        def hook(module, grad_input, grad_output):
            if name not in self.grad_out and grad_output[0] is not None:
                self.grad_out[name] = grad_output[0].detach().clone()
        return hook

    def detach(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []


def _with_noise(g: torch.Tensor, bits: int, scale: str, u: torch.Tensor, is_batched: bool):
    """The quantiser call of the rule with caller-supplied uniforms instead of the Philox stream (the
    reference's predicate u < frac): dequantised values.  For reproducing a recorded calibration."""
    from . import ops
    g2 = g.reshape(-1, g.shape[-1])
    pad = (-g2.shape[1]) % 16
    un = u.reshape(g2.shape).float()
    if pad:
        g2, un = torch.nn.functional.pad(g2, (0, pad)), torch.nn.functional.pad(un, (0, pad))
    q = lambda noise: ops.Quant(bits, "int8", "noise", scale, 0, 0, noise.contiguous())
    if scale == "tensor" and is_batched:
        B = g.shape[0]
        codes, s = ops.row_ht_quant_batched(g2.view(B, -1, g2.shape[1]).contiguous(), 1, q(un))
        s = s.repeat_interleave(g2.shape[0] // B).unsqueeze(1)
    else:
        codes, s = ops.row_ht_quant(g2.contiguous(), 1, q(un))
        s = s.unsqueeze(1) if scale == "row" else s
    deq = codes.view(torch.int8)[:, :g2.shape[1] - pad].float() * s
    return deq.reshape(g.shape)


def select_quantizer(grad_out: torch.Tensor, bits: int = 4, noise=None):
    """(gx_name, gw_name, err_stoch, err_norm) for one layer's captured grad_output
    (ViT_main.py:183-211).  3-D [B, L, O]: batched quantisers, one scale per sample for the
    per-tensor one, error against q * s[:, None, None].  2-D: one scale.  4-D [B, C, H, W] (a
    convolution's gradient, which the reference does not treat as batched): one scale for the
    per-tensor quantiser and one per position (b, h, w) over the channels for the per-token one.
    ``noise`` = (u_stoch, u_norm), two float32 tensors of grad_out's shape with uniforms in [0, 1):
    round with them (u < frac, as torch.bernoulli does) instead of the Philox stream."""
    g = grad_out.float()
    if g.dim() == 4:
        g = g.permute(0, 2, 3, 1).reshape(-1, g.shape[1])
    elif g.dim() not in (2, 3):
        g = g.reshape(-1, g.shape[-1])
    g = g.contiguous()
    is_batched = g.dim() == 3
    choice_gx = choice_gw = None
    min_qerror = 9999.0
    errs = []
    for q_func in quantScheme_gx:
        if noise is not None:
            if g.shape != grad_out.shape:
                raise ValueError("explicit noise is taken for 2-D and 3-D gradients")
            q_grad = _with_noise(g, bits, "tensor" if q_func == "stoch_quantizer" else "row",
                                 noise[0 if q_func == "stoch_quantizer" else 1].to(g.device), is_batched)
            s_grad = 1.0
        elif q_func == "stoch_quantizer":
            q_grad, s_grad = stoch_quantizer(g, bits, is_batched)
            if is_batched:
                s_grad = s_grad.unsqueeze(1).unsqueeze(2)
        else:
            q_grad, s_grad = norm_quantizer(g, bits, is_batched)
        qerror = float(torch.dist(g, q_grad * s_grad))
        errs.append(qerror)
        if qerror < min_qerror and q_func != "norm_quantizer":
            min_qerror = qerror
            choice_gx = choice_gw = q_func
        elif qerror < min_qerror and q_func == "norm_quantizer":
            if (min_qerror - qerror) > (min_qerror * 0.5):
                min_qerror = qerror
                choice_gx, choice_gw = q_func, "stoch_quantizer"
    return choice_gx, choice_gw, errs[0], errs[1]


def calibrate(model: nn.Module, batches: Iterable, loss_fn: Callable, optimizer: Optional[torch.optim.Optimizer] = None,
              bits: int = 4) -> Dict[str, str]:
    """Run the calibration batches with quantisation switched off (the reference's calibration
    worker skips every ``quant*`` / ``Transform*`` flag, ViT_main.py:127-131, so its layers run in
    full precision), capture each layer's first grad_output, and fill
    ``args.layer_quant_dict`` with ``name_gx`` / ``name_gw`` entries.  With an optimizer the
    pass also trains, as the reference's does (ViT_main.py:167-181)."""
    a = _args()
    cap = FirstBatchCapture().attach(model)
    saved = _plain_linear_mode(model, True)
    try:
        for inputs, target in batches:
            if optimizer is not None:
                optimizer.zero_grad()
            loss = loss_fn(model(inputs), target)
            loss.backward()
            if optimizer is not None:
                optimizer.step()
    finally:
        _plain_linear_mode(model, False, saved)
        cap.detach()
    for name, g in cap.grad_out.items():
        gx, gw, _, _ = select_quantizer(g, bits)
        a.layer_quant_dict[name + "_gx"] = gx
        a.layer_quant_dict[name + "_gw"] = gw
    return dict(a.layer_quant_dict)


def _plain_linear_mode(model: nn.Module, on: bool, saved=None):
    """Temporarily route HQ_Linear / HQ_Conv2d forward through nn.Linear / nn.Conv2d (full precision)."""
    if on:
        saved = []
        for m in model.modules():
            if isinstance(m, HQ_Linear):
                saved.append(m)
                m.forward = nn.Linear.forward.__get__(m, nn.Linear)
            elif isinstance(m, HQ_Conv2d):
                saved.append(m)
                m.forward = nn.Conv2d.forward.__get__(m, nn.Conv2d)
        return saved
    for m in saved or []:
        m.__dict__.pop("forward", None)
    return None
