"""Drop-in for the reference's ``HLQ_backward`` torch extension
(cuda_measure/HLQ_backward.cpp:4-24, cuda_measure/HLQ_backward_kernel.cu:457-737).

    gx, gw, times = HLQ_backward.backward(Go, W, X, reorder_idx_go, reorder_idx_X, H_size, per_token)

Same argument list, same checks (RuntimeError for non-CUDA / non-contiguous / non-2-D
tensors), same return shape: ``gx [L, I]``, ``gw [O, I]`` in the dtype of ``Go`` and a list of
four stage times in seconds.  Unlike the prototype it computes real gradients: Hadamard-INT4
g_x, Hadamard-low-rank-INT8 g_w (the prototype multiplied zero dummies with scale 1).

Stage times: the transform and the quantiser are one fused kernel here, and so are the
integer GEMM and its dequantisation, so entries 0 and 2 carry the fused times and entries 1
and 3 are 0.0.  They are CUDA-event times, and the call returns when its
results are complete (it waits for its own stream; the prototype synchronises the whole device).
"""
from __future__ import annotations

import threading

import torch

from . import ops
from .hadamard_matmul import lowrank_selection

_call_counter = 0
_lock = threading.Lock()


def _check(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor!" % name)
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous!" % name)
    if t.dim() != 2:
        raise RuntimeError("%s must be 2D!" % name)


def backward(Go: torch.Tensor, W: torch.Tensor, X: torch.Tensor, reorder_idx_go=0, reorder_idx_X=0, H_size: int = 16,
             per_token: bool = False, *, seed: int = 0, stochastic: bool = True):
    """``reorder_idx_*`` are accepted and ignored, as in the prototype (its callers pass 0).
    ``H_size`` is the Hadamard block order along the output-channel dim; ``per_token`` switches
    the INT4 scale of ``Go`` from one per tensor to one per row."""
    global _call_counter
    _check(Go, "Go")
    _check(W, "Wt")
    _check(X, "X")
    L, O = Go.shape
    if W.shape[0] != O or X.shape[0] != L or X.shape[1] != W.shape[1]:
        raise RuntimeError("shape mismatch: Go %s, W %s, X %s" % (tuple(Go.shape), tuple(W.shape), tuple(X.shape)))
    if W.dtype != Go.dtype or X.dtype != Go.dtype:
        raise RuntimeError("Go, W and X must share a dtype")
    order_l, sel = lowrank_selection(L, "half")
    with _lock:
        _call_counter += 1
        base = _call_counter * 8
    rounding = "philox" if stochastic else "nearest"
    cfg = ops.LinearConfig(
        order_o=int(H_size), order_l=order_l, sel_l=sel,
        q_gx=ops.Quant(4, ops.gx_code_storage(4, O), rounding, "row" if per_token else "tensor", seed, base + 1),
        q_w=ops.Quant(4, "int4", rounding, "tensor", seed, base + 2),
        q_gw=ops.Quant(8, "int8", rounding, "tensor", seed, base + 3),
        q_x=ops.Quant(8, "int8", rounding, "tensor", seed, base + 4))
    n = order_l
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    status = torch.zeros(1, dtype=torch.int32, device=Go.device)
    I = W.shape[1]
    q_w8 = ops.Quant(4, "int8", rounding, "tensor", seed, base + 2)      # weight codes one per byte (B operand)
    ev[0].record()
    if order_l == 16 and L % 32 == 0 and O % 64 == 0:
        q_go, s_go, q_gw, s_gw = ops.go_dual_quant(Go, cfg, status)          # both operands from one read per pass
        lp = L // 2
    else:
        q_go, s_go = ops.row_ht_quant(Go, int(H_size), cfg.q_gx)
        q_gw, s_gw, lp = ops.col_ht_quant(Go, n, sel, cfg.q_gw, "transposed")
    q_w_t, s_w, _ = ops.col_ht_quant(W, int(H_size), list(range(int(H_size))), q_w8, "natural")
    x_q_t, s_x, _ = ops.col_ht_quant(X, n, sel, cfg.q_x, "natural")
    ev[1].record()
    # both products in one launch where the shapes suit it (else two launches, decided inside)
    gx, gw = ops.gemm_i8_dual(
        dict(a=q_go, a_storage=cfg.q_gx.storage, b=q_w_t, M=L, N=I, K=O, scale_a=s_go, scale_b=s_w, post=1.0 / int(H_size),
             out_dtype=Go.dtype, a_rows_per_scale=1),
        dict(a=q_gw, b=x_q_t, M=O, N=I, K=lp, scale_a=s_gw, scale_b=s_x, post=1.0 / n, out_dtype=Go.dtype), status)
    ev[2].record()
    # the prototype synchronises the device; here the call waits for its own stream, which gives the
    # caller the same guarantee (results complete on return) without stalling copies on other streams
    torch.cuda.current_stream(Go.device).synchronize()
    if int(status.item()) != 0:
        raise RuntimeError("HLQ_backward: a bounded device-side wait ran out (status %d)" % int(status.item()))
    return gx, gw, [ev[0].elapsed_time(ev[1]) * 1e-3, 0.0, ev[1].elapsed_time(ev[2]) * 1e-3, 0.0]
