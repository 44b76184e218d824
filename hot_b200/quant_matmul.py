"""The HOT layer: quantiser callables, the ``FLinearQ`` autograd function and the ``HQ_Linear``
module, with the public names, argument meaning and error behaviour of the reference's
``utils/quant_matmul.py`` -- and CUDA kernels underneath instead of fake-quant float ops.

What runs natively is the scheme the reference trains with: ``transform_scheme = "gih_gwlr"``
with all four transforms on (main.sh:13-25): Hadamard + INT4 for grad_input, Hadamard
low-rank + INT8 for grad_weight, the compressed activation buffer saved in forward.  Any
other combination of flags raises; nothing falls back to float emulation.
"""
from __future__ import annotations

import sys
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor
from torch.autograd.function import Function

from . import ops
from .hadamard_matmul import (Transform_Dict, biggest_power2_factor, biggest_power2_factor_max16, lowrank_selection,
                              make_hadamard, selection_from_matrix)


def _args():
    """The configuration module: a host program's own top-level ``args`` if it has one (the
    reference's scripts do), else ``hot_b200.args``."""
    mod = sys.modules.get("args")
    if mod is not None and hasattr(mod, "transform_scheme"):
        return mod
    from . import args as own
    return own


TD = Transform_Dict()
_philox_calls = 0


def _next_offset() -> int:
    """A fresh Philox stream offset per quantiser call, so no two calls share random bits."""
    global _philox_calls
    _philox_calls += 1
    return _philox_calls


def _seed() -> int:
    return int(getattr(_args(), "SEED", 0) or 0)


# ---------------------------------------------------------------------------------------------
# quantiser callables: f(x, quantBits, is_batched) -> (x_int as float tensor, scale)
# (utils/quant_matmul.py:19-37, 86-122, 160-166).  No transform is applied (block order 1).
# ---------------------------------------------------------------------------------------------
def _quantise_2d(x: Tensor, bits: int, rounding: str, scale: str):
    x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    pad = (-x2.shape[1]) % 16
    if pad:  # the kernels work on runs of 16; zero columns change neither abs-max nor codes
        x2 = F.pad(x2, (0, pad))
    q = ops.Quant(bits, "int8", rounding, scale, _seed(), _next_offset())
    codes, scales = ops.row_ht_quant(x2, 1, q)
    codes = codes.view(torch.int8)[:, :x2.shape[1] - pad].to(x.dtype).reshape(x.shape)
    return codes, scales


def _quantise_batched(x: Tensor, bits: int, rounding: str):
    """One scale per sample of x [B, ...] (what torch.vmap over dim 0 of the reference's quantisers
    gives, utils/quant_matmul.py:102-106,117-122): (codes like x, scales [B])."""
    if x.dim() < 2:
        raise ValueError("a batched quantiser takes a tensor with a batch dim")
    x3 = x.reshape(x.shape[0], -1, x.shape[-1]) if x.dim() >= 3 else x.reshape(x.shape[0], 1, x.shape[1])
    x3 = x3.contiguous()
    pad = (-x3.shape[2]) % 16
    if pad:
        x3 = F.pad(x3, (0, pad))
    q = ops.Quant(bits, "int8", rounding, "tensor", _seed(), _next_offset())
    codes, scales = ops.row_ht_quant_batched(x3, 1, q)
    codes = codes.view(torch.int8)[:, :x3.shape[2] - pad].to(x.dtype).reshape(x.shape)
    return codes, scales


def stoch_quantizer(x: Tensor, quantBits: int, is_batched: bool = False):
    """Abs-max scale (one per tensor, or one per sample when batched), stochastic rounding
    (utils/quant_matmul.py:86-106)."""
    if is_batched:
        return _quantise_batched(x, quantBits, "philox")
    codes, s = _quantise_2d(x, quantBits, "philox", "tensor")
    return codes, s[0]


def int_quantizer(x: Tensor, quantBits: int, is_batched: bool = False):
    """Abs-max scale (one per tensor, or one per sample when batched), round half to even
    (utils/quant_matmul.py:108-122)."""
    if is_batched:
        return _quantise_batched(x, quantBits, "nearest")
    codes, s = _quantise_2d(x, quantBits, "nearest", "tensor")
    return codes, s[0]


def norm_quantizer(x: Tensor, quantBits: int, is_batched: bool = False):
    """Per-row abs-max scale, stochastic rounding; returns the DEQUANTISED tensor and the scale
    1.0, as the reference does (utils/quant_matmul.py:19-37).  Batched [B, L, C] input: the rows of
    every sample are rows of the flattened tensor, so the batch changes nothing."""
    if x.dim() != (3 if is_batched else 2):
        raise NotImplementedError("norm_quantizer takes a 2-D tensor, or a 3-D one when batched")
    codes, s = _quantise_2d(x, quantBits, "philox", "row")
    return codes * s.to(x.dtype).reshape(x.shape[:-1]).unsqueeze(-1), 1.


def sawb_quantizer(x: Tensor, quantBits: int, is_batched: bool = False):
    """One scale from clip = 12.1*sqrt(mean(x^2)) - 12.2*mean(|x|), values clamped to +-clip, round to
    nearest (utils/quant_matmul.py:40-55).  Returns (codes as float, scale)."""
    if is_batched:   # one clip per sample of x [B, ...] (torch.vmap over dim 0, utils/quant_matmul.py:51-55)
        if x.dim() < 2:
            raise ValueError("a batched quantiser takes a tensor with a batch dim")
        x3 = (x.reshape(x.shape[0], -1, x.shape[-1]) if x.dim() >= 3 else x.reshape(x.shape[0], 1, x.shape[1])).contiguous()
        q = ops.Quant(quantBits, "int8", "nearest", "sawb")
        codes_t, s, n, pitch = ops.col_ht_quant_batched(x3, 1, [0], q, "natural")
        codes = codes_t.view(torch.int8).view(x3.shape[2], x3.shape[0], pitch)[:, :, :n].permute(1, 2, 0)
        return codes.to(x.dtype).reshape(x.shape), s
    x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    q = ops.Quant(quantBits, "int8", "nearest", "sawb")
    codes_t, s, n = ops.col_ht_quant(x2, 1, [0], q, "natural")      # identity transform, transposed codes
    codes = codes_t.view(torch.int8)[:, :n].t().to(x.dtype).reshape(x.shape)
    return codes, s[0]


def _luq_one(x: Tensor, quantBits: int, u_prune: Optional[Tensor] = None, u_round: Optional[Tensor] = None):
    """luq_quantizer_BWD (utils/quant_matmul.py:58-76), expression by expression, on the tensor's device.
    ``u_prune`` / ``u_round``: uniforms in [0, 1) to use instead of fresh draws (the reference draws torch.rand for
    the stochastic pruning below the smallest level and uniform_(-0.5, 0.5) for the rounding between powers of two)."""
    mx = torch.max(x)                                   # the signed maximum, as the reference takes it
    s = mx / (2 ** (2 ** (quantBits - 1) - 1))
    s_eps = s * (torch.rand(x.shape, device=x.device) if u_prune is None else u_prune)
    x_abs = x.abs()
    zero = torch.zeros((), dtype=torch.float32, device=x.device)
    out = torch.where(x_abs < s, s * torch.sign(x), x)
    out = torch.where(x_abs < s_eps, zero, out)
    half = (torch.rand(x.shape, device=x.device) if u_round is None else u_round) - 0.5
    level = 2 ** torch.floor(torch.log2(out.abs() / s))
    out_q = 2 ** torch.floor(torch.log2((out.abs() / s + level * half) * 4 / 3))
    out_q = torch.sign(out) * torch.where(out_q < level, level, out_q)
    out_q = torch.where(out == 0, zero, out_q)
    return out_q, s


def luq_quantizer(x: Tensor, quantBits: int, is_batched: bool = False, noise=None):
    """Logarithmic stochastic quantiser (utils/quant_matmul.py:58-83): values are sign * 2^k * s with
    k in [0, 2^(bits-1) - 1], those below the smallest level pruned stochastically.  Returns (levels as float:
    0 or +-2^k, s); batched: one s per sample.  The levels are not an integer code of ``quantBits`` bits, so this
    quantiser is a composition of elementwise device operations and its product is a float matmul
    (``FLinearQ`` does that when a grad_output side is set to 'luq'); ``noise`` = (u_prune, u_round)."""
    if x.dtype != torch.float32:
        x = x.float()
    if is_batched:
        outs = [_luq_one(x[b], quantBits, None if noise is None else noise[0][b], None if noise is None else noise[1][b])
                for b in range(x.shape[0])]
        return torch.stack([o[0] for o in outs]), torch.stack([o[1] for o in outs])
    return _luq_one(x, quantBits, None if noise is None else noise[0], None if noise is None else noise[1])


quant_scheme_dict = {
    "luq_quantizer": luq_quantizer,
    "sawb_quantizer": sawb_quantizer,
    "int_quantizer": int_quantizer,
    "stoch_quantizer": stoch_quantizer,
    "norm_quantizer": norm_quantizer,
}


# ---------------------------------------------------------------------------------------------
# configuration -> kernel modes
# ---------------------------------------------------------------------------------------------
def _storage(bits: int) -> str:
    return "int4" if bits <= 4 else "int8"


def _operand(kind: str, scheme, bits: int, what: str, row_ok: bool, k: int = 1 << 30) -> ops.Quant:
    if scheme == "stoch":
        rounding, scale = "philox", "tensor"
    elif scheme == "int":
        rounding, scale = "nearest", "tensor"
    elif scheme == "nq" and row_ok:
        rounding, scale = "philox", "row"
    elif scheme == "sawb" and kind in ("w", "x"):
        rounding, scale = "nearest", "sawb"
    elif scheme == "luq" and kind in ("gx", "gw"):
        return "luq"                                    # not an integer format: FLinearQ takes the float path for this side
    elif scheme in ("sawb", "luq", "no", False):
        raise NotImplementedError("%s rounding scheme %r is not built on the native path" % (what, scheme))
    else:
        raise Exception("%s rounding scheme not implemented: %s" % (what, scheme))
    if not 2 <= int(bits) <= 8:
        raise ValueError("%s: quantBits %r outside [2, 8]" % (what, bits))
    storage = ops.gx_code_storage(int(bits), k) if kind == "gx" else _storage(int(bits))
    return ops.Quant(int(bits), storage, rounding, scale, _seed(), _next_offset())


_BUILT_SCHEMES = ("gih_gwlr", "hadamard", "low_rank", "gilr_gwh", "gilro_gwh")
_TOKEN_GX_SCHEMES = ("low_rank", "gilr_gwh")   # grad_output is projected along the tokens for g_x too


def _token_basis(a, tokens: int, preset):
    """(n, sel) of the token-side transform of the configured scheme: the low-rank rows of make_WHT
    (or the preset) for ``gih_gwlr``; every row of the block Hadamard matrix H_n, n = min(16, 2-adic
    part of the token count), for ``hadamard`` (utils/quant_matmul.py:353-355, make_hadamard)."""
    if a.transform_scheme in ("hadamard", "gilr_gwh", "gilro_gwh"):
        n = biggest_power2_factor_max16(tokens)
        return n, list(range(n))
    return lowrank_selection(tokens, preset, a.vectorPercentile)


def _out_matrix(a, out_features: int, tokens: int, preset, dtype, device) -> Tensor:
    """What ``hadamard_out`` holds per scheme (utils/quant_matmul.py:353-370): the block Hadamard matrix
    of the output features (gih_gwlr, hadamard), a [1, 1] zero (low_rank) or the low-rank rows of the
    token count (gilr_gwh)."""
    from .hadamard_matmul import hadamard
    if a.transform_scheme == "low_rank":
        return torch.zeros((1, 1), dtype=dtype, device=device)
    if a.transform_scheme == "gilr_gwh":
        n, sel = lowrank_selection(tokens, preset, a.vectorPercentile)
        return torch.tensor(hadamard(n)[sel], dtype=dtype, device=device)
    if a.transform_scheme == "gilro_gwh":   # low-rank rows over the OUTPUT FEATURES, order = their whole 2-adic part (:365)
        return torch.tensor(TD.get_or_register("low_rank", out_features, a.vectorPercentile), dtype=dtype, device=device)
    return torch.tensor(TD.get_or_register("hadamard", out_features), dtype=dtype, device=device)


def _check_scheme(a) -> None:
    if a.transform_scheme not in _BUILT_SCHEMES:
        raise Exception("args.transform_scheme not implemented: " + str(a.transform_scheme))
    if a.transform_scheme == "gilro_gwh":
        # the reference has no activation / grad_out(g_w) transform for this scheme: it raises with them switched on
        # (utils/quant_matmul.py:192, 303), so the scheme runs with the g_w side untransformed
        if a.TransformInput:
            raise Exception("Activation transform scheme not implemented: gilro_gwh")
        if a.TransformGogw:
            raise Exception("GradHb transform scheme not implemented: gilro_gwh")
        if not (a.TransformGogi and a.TransformWgt):
            raise NotImplementedError("gilro_gwh on the native path needs TransformGogi and TransformWgt True")
        return
    if not (a.TransformGogi and a.TransformWgt and a.TransformGogw and a.TransformInput):
        raise NotImplementedError("the native path needs TransformGogi/Wgt/Gogw/Input all True")


_selection_cache: dict = {}


def _selection(h_bs: Tensor):
    """(n, sel) of the low-rank matrix a layer carries; cached on the matrix's identity."""
    key = (h_bs.data_ptr(), tuple(h_bs.shape), h_bs._version)
    hit = _selection_cache.get(key)
    if hit is None:
        hit = selection_from_matrix(h_bs)
        if len(_selection_cache) > 256:
            _selection_cache.clear()
        _selection_cache[key] = hit
    return hit


class FLinearQ(Function):
    """``FLinearQ.apply(x, w, h_out, h_bs, name)`` (utils/quant_matmul.py:169-348).

    forward: ``F.linear(x, w)`` in full precision.  Its context (the reference's setup_context): the activation buffer is the
    Hadamard low-rank projection of ``x`` along tokens, quantised to INT8 (what the reference
    saves), produced by one fused kernel.  backward: grad_input and grad_weight from the
    integer tensor-core path; exactly two real gradients are returned.
    3-D inputs [B, L, I] follow the reference: every quantiser of a batched tensor takes one scale
    per sample, the low-rank projection runs along the tokens of each sample, grad_weight is the sum
    over samples (utils/quant_matmul.py:180,223-225,288-290,322-324).  With ``args.lowRankPreset``
    set (not in the reference) the batch is flattened to B*L tokens with one scale instead, which
    is the faster path.
    An optional sixth argument is the layer's bias, added by the forward GEMM itself (``F.linear(x, w, bias)``);
    its gradient, the sum of grad_output over the tokens, then comes from this backward too.  The reference adds the
    bias after ``apply`` (utils/quant_matmul.py:420-421), a pass of its own over the output."""

    # forward(ctx, ...) rather than forward + setup_context as in the reference: torch binds the default arguments of a
    # forward that comes with a setup_context through inspect.signature on every call (67 us per layer call on the
    # benchmark host)
    @staticmethod
    def forward(ctx, x, w, h_out, h_bs, name, bias=None):
        FLinearQ._save_context(ctx, (x, w, h_out, h_bs, name) if bias is None else (x, w, h_out, h_bs, name, bias))
        return F.linear(x, w, bias)

    @staticmethod
    def _save_context(ctx, inputs):
        """What the reference's setup_context does (utils/quant_matmul.py:177-212)."""
        x, w, h_out, h_bs, name = inputs[:5]
        ctx.n_inputs = len(inputs)
        a = _args()
        _check_scheme(a)
        n_l, sel = _selection(h_bs)
        q_x = _operand("x", a.quantBWDAct, a.actQuantBit, "Activation", row_ok=False)
        ctx.scheme = a.transform_scheme
        ctx.gx_basis = None
        if ctx.scheme in _TOKEN_GX_SCHEMES:   # no transform along the output features; g_x takes token rows
            order_o = 1
            ctx.gx_basis = (n_l, sel) if ctx.scheme == "low_rank" else _selection(h_out)
        elif ctx.scheme == "gilro_gwh":       # low-rank rows over the output features for g_x; g_w untransformed
            order_o = 1
            ctx.gx_basis = _selection(h_out)
            n_l, sel = 1, [0]
        else:
            order_o = int(h_out.shape[0])
        cfg = ops.LinearConfig(order_o=order_o, order_l=n_l, sel_l=sel, q_x=q_x)
        ctx.per_sample = x.dim() == 3 and getattr(a, "lowRankPreset", None) is None
        if ctx.per_sample and ctx.scheme in _TOKEN_GX_SCHEMES and x.shape[1] % ctx.gx_basis[0]:
            raise ValueError("token count %d is not a multiple of the low-rank order %d" % (x.shape[1], ctx.gx_basis[0]))
        if ctx.per_sample:
            if x.shape[1] % n_l:
                raise ValueError("token count %d is not a multiple of the low-rank order %d" % (x.shape[1], n_l))
            x_q_t, scale_x, _ = ops.abc_compress_batched(x.detach().contiguous(), cfg)
        else:
            x2 = x.detach().reshape(-1, x.shape[-1])
            if not x2.is_contiguous():
                x2 = x2.contiguous()
            if x2.shape[0] % n_l:
                raise ValueError("token count %d is not a multiple of the low-rank order %d" % (x2.shape[0], n_l))
            x_q_t, scale_x = ops.abc_compress(x2, cfg)
        ctx.name = name
        ctx.x_shape = tuple(x.shape)
        ctx.order_o, ctx.order_l, ctx.sel = order_o, n_l, sel
        ctx.q_x = q_x
        ctx.save_for_backward(x_q_t, w, scale_x)

    @staticmethod
    def backward(ctx, grad_output):
        x_q_t, w, scale_x = ctx.saved_tensors
        a = _args()
        _check_scheme(a)
        name = ctx.name
        go = grad_output if ctx.per_sample else grad_output.reshape(-1, grad_output.shape[-1])
        if not go.is_contiguous():
            go = go.contiguous()
        if go.dtype != w.dtype:
            go = go.to(w.dtype)
        if a.quantAuto and len(a.layer_quant_dict) > 0:
            # layer-wise quantiser selection; both sides take GogiQuantBit here, as the reference
            # does (utils/quant_matmul.py:244-245, 307-308)
            pick = {"stoch_quantizer": "stoch", "norm_quantizer": "nq", "int_quantizer": "int", "luq_quantizer": "luq"}
            try:
                gx_scheme = pick[a.layer_quant_dict[name + "_gx"]]
                gw_scheme = pick[a.layer_quant_dict[name + "_gw"]]
            except KeyError as e:
                raise NotImplementedError("layer_quant_dict entry %s is not built on the native path" % e) from None
            q_gx = _operand("gx", gx_scheme, a.GogiQuantBit, "GradHo", row_ok=True, k=go.shape[-1])
            q_gw = _operand("gw", gw_scheme, a.GogiQuantBit, "GradHb", row_ok=True)
        else:
            q_gx = _operand("gx", a.quantBWDGogi, a.GogiQuantBit, "GradHo", row_ok=True, k=go.shape[-1])
            q_gw = _operand("gw", a.quantBWDGogw, a.GogwQuantBit, "GradHb", row_ok=True)
        q_w = _operand("w", a.quantBWDWgt, a.weightQuantBit, "Weight", row_ok=False)
        need_gx, need_gw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gx = gw = None
        # a grad_output side set to the logarithmic quantiser leaves the integer path: its product is a float matmul
        luq_gx, luq_gw = q_gx == "luq", q_gw == "luq"
        if luq_gx or luq_gw:
            if ctx.scheme not in ("gih_gwlr", "hadamard"):
                raise NotImplementedError("the logarithmic quantiser is built for transform_scheme gih_gwlr / hadamard")
            bits_gw = a.GogiQuantBit if (a.quantAuto and len(a.layer_quant_dict) > 0) else a.GogwQuantBit
            if luq_gx and need_gx:
                gx = _luq_grad_input(go, w.detach(), ctx.order_o, q_w, a.GogiQuantBit, ctx.per_sample)
            if luq_gw and need_gw:
                gw = _luq_grad_weight(go, x_q_t, scale_x, ctx.order_l, ctx.sel, bits_gw, ctx.per_sample, w.dtype)
            need_gx, need_gw = need_gx and not luq_gx, need_gw and not luq_gw
            if luq_gx:
                q_gx = _operand("gx", "stoch", a.GogiQuantBit, "GradHo", row_ok=True, k=go.shape[-1])   # placeholder, unused
            if luq_gw:
                q_gw = _operand("gw", "stoch", a.GogwQuantBit, "GradHb", row_ok=True)
        cfg = ops.LinearConfig(order_o=ctx.order_o, order_l=ctx.order_l, sel_l=ctx.sel, q_gx=q_gx, q_w=q_w, q_gw=q_gw,
                               q_x=ctx.q_x)
        gx_luq, gw_luq = gx, gw
        if ctx.scheme == "gilro_gwh":
            n_x, sel_x = ctx.gx_basis
            if need_gw:
                if ctx.per_sample:
                    _, gw = ops.linear_backward_batched(go, w.detach(), x_q_t, scale_x, cfg, need_gx=False, need_gw=True)
                else:
                    _, gw = ops.linear_backward(go, w.detach(), x_q_t, scale_x, cfg, need_gx=False, need_gw=True)
            if need_gx:
                B = go.shape[0] if ctx.per_sample else 1
                gx = ops.linear_backward_gilro_gx(go.reshape(-1, go.shape[-1]), w.detach(), n_x, sel_x, q_gx, q_w, batch=B)
        elif (need_gx or need_gw) and ctx.per_sample and ctx.gx_basis is not None:
            if need_gw:
                _, gw = ops.linear_backward_batched(go, w.detach(), x_q_t, scale_x, cfg, need_gx=False, need_gw=True)
            if need_gx:
                n_x, sel_x = ctx.gx_basis
                B, L, O = go.shape
                gx = ops.linear_backward_lowrank_gx(go.view(B * L, O), w.detach(), n_x, sel_x, q_gx, q_w, batch=B)
                gx = gx.view(B, L, -1)
        elif (need_gx or need_gw) and ctx.per_sample:
            gx, gw = ops.linear_backward_batched(go, w.detach(), x_q_t, scale_x, cfg, need_gx=need_gx, need_gw=need_gw)
        elif ctx.gx_basis is not None:
            if need_gw:
                _, gw = ops.linear_backward(go, w.detach(), x_q_t, scale_x, cfg, need_gx=False, need_gw=True)
            if need_gx:
                n_x, sel_x = ctx.gx_basis
                if go.shape[0] % n_x:
                    raise ValueError("token count %d is not a multiple of the low-rank order %d" % (go.shape[0], n_x))
                gx = ops.linear_backward_lowrank_gx(go, w.detach(), n_x, sel_x, q_gx, q_w)
        elif need_gx or need_gw:
            gx, gw = ops.linear_backward(go, w.detach(), x_q_t, scale_x, cfg, need_gx=need_gx, need_gw=need_gw)
        gx = gx_luq if gx_luq is not None else gx
        gw = gw_luq if gw_luq is not None else gw
        if gx is not None:
            gx = gx.reshape(ctx.x_shape)
        if ctx.n_inputs > 5:
            gb = grad_output.reshape(-1, grad_output.shape[-1]).sum(0) if ctx.needs_input_grad[5] else None
            return gx, gw, None, None, None, gb
        return gx, gw, None, None, None


def _luq_grad_input(go: Tensor, w: Tensor, order_o: int, q_w, bits: int, per_sample: bool, noise=None) -> Tensor:
    """grad_input with the logarithmic quantiser on grad_output (utils/quant_matmul.py:237-238, 250-251, 288-290, 342):
    block Hadamard of grad_output along the output features in float, luq levels, a float32 product with the
    weight's integer codes (which the integer kernel makes as usual), scales and the 1 / order factor."""
    from .hadamard_matmul import hadamard, lowering_matmul_front
    O = go.shape[-1]
    h = torch.tensor(hadamard(order_o), dtype=torch.float32, device=go.device)
    levels, s = luq_quantizer(lowering_matmul_front(go.float(), h), bits, per_sample, noise)
    q_w_t, s_w, _ = ops.col_ht_quant(w, order_o, list(range(order_o)), ops._one_per_byte(q_w), "natural")   # [I, O] codes
    wq = q_w_t.view(torch.int8)[:, :O].float()
    gi = torch.matmul(levels, wq.t()) * (s.view(-1, 1, 1) if per_sample else s) * s_w[0] / order_o
    return gi.to(go.dtype)


def _luq_grad_weight(go: Tensor, x_q_t: Tensor, scale_x: Tensor, order_l: int, sel, bits: int, per_sample: bool, dtype,
                     noise=None) -> Tensor:
    """grad_weight with the logarithmic quantiser on the projected grad_output (utils/quant_matmul.py:300-301, 313-314,
    322-324, 344): low-rank projection along the tokens in float, transposed, luq levels, a float32 product with the
    saved activation codes; per sample and summed over the batch for 3-D inputs."""
    O = go.shape[-1]
    go2 = go.reshape(-1, O)
    go_lr = ops.hla_project_any(go2, order_l, sel)                                   # [L', O] (all samples one after the other)
    if per_sample:
        B = go.shape[0]
        lp = go_lr.shape[0] // B
        levels, s = luq_quantizer(go_lr.view(B, lp, O).transpose(1, 2).contiguous(), bits, True, noise)     # [B, O, L']
        pitch = x_q_t.shape[1] // B
        xq = x_q_t.view(torch.int8).view(-1, B, pitch)[:, :, :lp].permute(1, 2, 0).float()                 # [B, L', I]
        gw = (torch.bmm(levels, xq) * (s * scale_x).view(-1, 1, 1)).sum(0) / order_l
    else:
        lp = go_lr.shape[0]
        levels, s = luq_quantizer(go_lr.t().contiguous(), bits, False, noise)                               # [O, L']
        xq = x_q_t.view(torch.int8)[:, :lp].t().float()                                                      # [L', I]
        gw = torch.matmul(levels, xq) * s * scale_x[0] / order_l
    return gw.to(dtype)


class HQ_Linear(nn.Linear):
    """Drop-in ``nn.Linear`` whose backward is HOT (utils/quant_matmul.py:350-422).  Buffers
    ``hadamard_out`` [n_O, n_O] and ``hadamard_bs`` [r, n_L] and the attribute ``layer_name``
    keep the reference's names so state dicts and the layer-naming loop carry over."""

    def __init__(self, in_features, out_features, bias=True) -> None:
        super().__init__(in_features, out_features, bias)
        a = _args()
        _check_scheme_name(a)
        self.register_buffer("hadamard_out", _out_matrix(a, self.out_features, max(int(a.BATCH_SIZE), 1), None,
                                                         self.weight.dtype, self.weight.device))
        n, sel = _token_basis(a, max(int(a.BATCH_SIZE), 1), None)
        self.register_buffer("hadamard_bs", self._basis(n, sel, self.weight.device))
        self._bs_tokens = None
        self.layer_name = " "

    def _basis(self, n, sel, device) -> Tensor:
        from .hadamard_matmul import hadamard
        return torch.tensor(hadamard(n)[sel], dtype=self.weight.dtype, device=device)

    def forward(self, input: Tensor) -> Tensor:
        a = _args()
        # the low-rank basis follows the live token count, as in the reference (:374-413); here it
        # is rebuilt only when that count changes, and straight on the device
        tokens = input.shape[0] if input.dim() == 2 else input.shape[0] * input.shape[1]
        if input.dim() == 3 and getattr(a, "lowRankPreset", None) is None:
            tokens = input.shape[1]   # the reference sizes the basis from the per-sample length
        key = (tokens, a.transform_scheme, getattr(a, "lowRankPreset", None), a.vectorPercentile)
        if key != self._bs_tokens or self.hadamard_bs.device != self.weight.device:
            n, sel = _token_basis(a, tokens, getattr(a, "lowRankPreset", None))
            self.hadamard_bs = self._basis(n, sel, self.weight.device)
            self.hadamard_out = _out_matrix(a, self.out_features, tokens, getattr(a, "lowRankPreset", None),
                                            self.weight.dtype, self.weight.device)
            self._bs_tokens = key
        # 16-bit tensors: the bias goes into the forward GEMM (one rounding of the output, no pass of its own over
        # it: at 50,432 x 3,072 that pass was 0.2 ms per layer); float32 keeps the reference's separate addition,
        # whose result the parity tests pin bit for bit
        if self.bias is not None and input.dtype in (torch.bfloat16, torch.float16) and self.bias.dtype == input.dtype:
            return FLinearQ.apply(input, self.weight, self.hadamard_out, self.hadamard_bs, self.layer_name, self.bias)
        output = FLinearQ.apply(input, self.weight, self.hadamard_out, self.hadamard_bs, self.layer_name)
        if self.bias is not None:
            output += self.bias.to(output.device)
        return output


class HQ_Conv2d(nn.Conv2d):
    """Drop-in ``nn.Conv2d`` whose backward is HOT (utils/quant_matmul.py:426-488): the input is
    unfolded to [B, H'*W', C*kh*kw] (im2col) and goes through the same ``FLinearQ`` as a linear
    layer, with the kernel viewed as a [C_out, C*kh*kw] weight.  Grouped (depth-wise) convolutions
    raise ``NotImplementedError``, as in the reference."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode="zeros") -> None:
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias, padding_mode)
        a = _args()
        _check_scheme_name(a)
        if a.transform_scheme in _TOKEN_GX_SCHEMES:
            raise NotImplementedError("HQ_Conv2d with transform_scheme %r is not built" % a.transform_scheme)
        self.register_buffer("hadamard_out", _out_matrix(a, self.out_channels, 1, None, self.weight.dtype, self.weight.device))
        self.register_buffer("hadamard_bs", torch.zeros((1, 1), dtype=self.weight.dtype))
        self._bs_tokens = None
        self.layer_name = " "

    def forward(self, input: Tensor) -> Tensor:
        if self.groups > 1:
            raise NotImplementedError
        a = _args()
        B = input.shape[0]
        cols = F.unfold(input, self.kernel_size, dilation=self.dilation, padding=self.padding,
                        stride=self.stride).transpose(1, 2)                      # [B, H'*W', C*kh*kw]
        weight = self.weight.view(self.weight.size(0), -1)
        preset = getattr(a, "lowRankPreset", None)
        tokens = cols.shape[1] if preset is None else cols.shape[0] * cols.shape[1]
        key = (tokens, a.transform_scheme, preset, a.vectorPercentile)
        if key != self._bs_tokens or self.hadamard_bs.device != self.weight.device:
            from .hadamard_matmul import hadamard
            n, sel = _token_basis(a, tokens, preset)
            self.hadamard_bs = torch.tensor(hadamard(n)[sel], dtype=self.weight.dtype, device=self.weight.device)
            self._bs_tokens = key
        out = FLinearQ.apply(cols, weight, self.hadamard_out, self.hadamard_bs, self.layer_name)   # [B, H'*W', C_out]
        h_out = (input.shape[-2] + 2 * self.padding[0] - self.dilation[0] * (self.kernel_size[0] - 1) - 1) // self.stride[0] + 1
        w_out = (input.shape[-1] + 2 * self.padding[1] - self.dilation[1] * (self.kernel_size[1] - 1) - 1) // self.stride[1] + 1
        out = out.transpose(1, 2).reshape(B, self.out_channels, h_out, w_out)
        if self.bias is not None:
            out = out + self.bias.view(1, -1, 1, 1)
        return out


def _check_scheme_name(a) -> None:
    if a.transform_scheme not in ("hadamard", "low_rank", "gilr_gwh", "gilro_gwh", "gih_gwlr"):
        raise Exception("Transformation method not implemented: " + str(a.transform_scheme))


def replace_layers(model: nn.Module, old, new) -> None:
    """Recursively swap ``nn.Linear`` children for ``new`` (``HQ_Linear``), sharing weight and
    bias storage with the replaced module (utils/utils.py:53-74).  LoRA sub-layers named
    ``base_layer`` / ``default`` are skipped unless ``args.HLQ_on_base`` / ``HLQ_on_decompose``."""
    a = _args()
    for n, module in model.named_children():
        if len(list(module.children())) > 0:
            replace_layers(module, old, new)
        if old == nn.Linear and isinstance(module, old) and not isinstance(module, new):
            if "base_layer" in n and not getattr(a, "HLQ_on_base", False):
                continue
            if "default" in n and not getattr(a, "HLQ_on_decompose", False):
                continue
            new_layer = new(module.in_features, module.out_features)   # always built with a bias (:73)
            new_layer = new_layer.to(device=module.weight.device, dtype=module.weight.dtype)
            new_layer.weight.data = module.weight.data
            new_layer.weight.requires_grad = module.weight.requires_grad
            if module.bias is not None:
                new_layer.bias.data = module.bias.data
            setattr(model, n, new_layer)
        elif old == nn.Conv2d and isinstance(module, old) and not isinstance(module, new) and module.groups == 1:
            new_layer = new(module.in_channels, module.out_channels, kernel_size=module.kernel_size, stride=module.stride,
                            padding=module.padding)
            new_layer = new_layer.to(device=module.weight.device, dtype=module.weight.dtype)
            new_layer.weight.data = module.weight.data
            new_layer.weight.requires_grad = module.weight.requires_grad
            if module.bias is not None:
                new_layer.bias.data = module.bias.data
            setattr(model, n, new_layer)


def ddp_ignore_hot_buffers(model: nn.Module) -> int:
    """Tell DistributedDataParallel (through the attribute it reads from the module it wraps) not to broadcast the
    ``hadamard_out`` / ``hadamard_bs`` buffers of the HOT layers under ``model`` at every forward: they are
    functions of the layer's shapes and the token count alone, hence identical on every rank, and two small
    tensors per layer (96 for ViT-B/16) cost more host time per step than the backward saves.  Call it on the module
    that will be wrapped, before wrapping.  Not in the reference, which lets DDP broadcast them.  Returns how many
    buffers were named."""
    names = [n + "." + b for n, m in model.named_modules() if isinstance(m, (HQ_Linear, HQ_Conv2d))
             for b in ("hadamard_out", "hadamard_bs")]
    names = [n.lstrip(".") for n in names]
    have = list(getattr(model, "_ddp_params_and_buffers_to_ignore", []))
    model._ddp_params_and_buffers_to_ignore = have + [n for n in names if n not in have]
    return len(names)


def precision_scheduler(current_epoch, max_bit=8, min_bit=4, milestones=()):
    """Bit-width schedule (utils/utils.py:149-159): everything at ``max_bit`` in epoch 0; at each
    milestone the grad_output (g_x side) and weight widths halve, if their scheme is stoch/int."""
    a = _args()
    if current_epoch == 0:
        a.GogiQuantBit = a.weightQuantBit = a.GogwQuantBit = a.actQuantBit = max_bit
    elif current_epoch in milestones and min(a.GogiQuantBit, a.weightQuantBit, a.GogwQuantBit, a.actQuantBit) > min_bit:
        if a.quantBWDGogi in ("stoch", "int"):
            a.GogiQuantBit = a.GogiQuantBit // 2
        if a.quantBWDWgt in ("stoch", "int"):
            a.weightQuantBit = a.weightQuantBit // 2
