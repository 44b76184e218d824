"""Layer-wise quantiser selection (LQS): a calibration pass that decides, per HOT layer, whether
grad_output is quantised with one scale per tensor or one per token on the g_x path
(ViT_main.py:44-56, 133-215 and the first-batch capture of utils/plot.py:164-204).

The rule, unchanged: quantise the UN-transformed first-batch grad_output to 4 bits with the
per-tensor stochastic quantiser and with the per-token one; per-token wins for g_x only if it
cuts the L2 error by more than half; g_w always keeps the per-tensor quantiser.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional

import torch
import torch.nn as nn

from .quant_matmul import HQ_Linear, _args, norm_quantizer, stoch_quantizer

quantScheme_gx = ["stoch_quantizer", "norm_quantizer"]


class FirstBatchCapture:
    """Keeps the first grad_output each named layer sees (the reference's ``Tensor_Dict``
    stores a tensor only while its slot still holds the initial sentinel)."""

    def __init__(self):
        self.grad_out: Dict[str, torch.Tensor] = {}
        self._handles = []

    def attach(self, model: nn.Module) -> "FirstBatchCapture":
        for name, layer in model.named_modules():
            if isinstance(layer, HQ_Linear):
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


def select_quantizer(grad_out: torch.Tensor, bits: int = 4):
    """(gx_name, gw_name, err_stoch, err_norm) for one layer's captured grad_output."""
    g = grad_out.reshape(-1, grad_out.shape[-1]).float().contiguous()
    choice_gx = choice_gw = None
    min_qerror = 9999.0
    errs = []
    for q_func in quantScheme_gx:
        if q_func == "stoch_quantizer":
            q_grad, s_grad = stoch_quantizer(g, bits, False)
        else:
            q_grad, s_grad = norm_quantizer(g, bits, False)
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
    """Temporarily route HQ_Linear.forward through nn.Linear.forward (full precision)."""
    if on:
        saved = []
        for m in model.modules():
            if isinstance(m, HQ_Linear):
                saved.append(m)
                m.forward = nn.Linear.forward.__get__(m, nn.Linear)
        return saved
    for m in saved or []:
        m.__dict__.pop("forward", None)
    return None
