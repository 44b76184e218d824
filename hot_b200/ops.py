"""Tensor-level wrappers over the C ABI: torch owns the memory and the stream, the library
does the work.  Every function launches on ``torch.cuda.current_stream()`` of the input's
device and returns without synchronising.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from . import _cabi as C

_DTYPES = {torch.float32: C.HOT_F32, torch.bfloat16: C.HOT_BF16}
_ROUNDING = {"nearest": C.ROUND_NEAREST, "philox": C.ROUND_STOCH_PHILOX, "noise": C.ROUND_STOCH_NOISE}


@dataclass
class Quant:
    """How one operand is quantised (mirrors ``hot_quant_t``)."""
    bits: int = 8
    storage: str = "int8"            # "int8" | "int4" (two codes per byte, in runs of 16: byte j = codes j and j + 8)
    rounding: str = "philox"         # "nearest" | "philox" | "noise"
    scale: str = "tensor"            # "tensor" | "row" | "sawb" (column kernel only, nearest rounding)
    seed: int = 0
    offset: int = 0
    noise: Optional[torch.Tensor] = field(default=None, repr=False)

    def to_c(self) -> C.HotQuant:
        q = C.HotQuant()
        q.bits = self.bits
        q.storage = C.STORE_INT4 if self.storage == "int4" else C.STORE_INT8
        q.rounding = _ROUNDING[self.rounding]
        q.scale_mode = {"tensor": C.SCALE_TENSOR, "row": C.SCALE_ROW, "sawb": C.SCALE_SAWB}[self.scale]
        q.seed, q.offset = self.seed & (2 ** 64 - 1), self.offset & (2 ** 64 - 1)
        if self.rounding == "noise":
            if self.noise is None or self.noise.dtype != torch.float32 or not self.noise.is_contiguous():
                raise ValueError("rounding='noise' needs a contiguous float32 noise tensor")
            q.noise = self.noise.data_ptr()
        else:
            q.noise = None
        return q


def check_status(status: torch.Tensor) -> None:
    """Reads a status word back (this synchronises with the stream that wrote it) and raises
    ``HotError`` (HOT_ERR_TIMEOUT) if a bounded device-side wait ran out in a launch that was given it."""
    C.check(C.lib().hot_check_status(int(status.item()) & 0xFFFFFFFF), "status word")


def set_wait_limit_ns(limit_ns: int) -> None:
    """Time limit of every device-side wait in launches made from now on (0 restores the default 1.5 s)."""
    C.lib().hot_set_wait_limit_ns(int(limit_ns))


def set_sm_margin(sms: int) -> None:
    """Leave ``sms`` SMs out of the persistent kernels' grids from now on (room for a collective's kernels)."""
    C.lib().hot_set_sm_margin(int(sms))


def wait_probe(status: torch.Tensor) -> None:
    """Launch the probe whose wait runs out (needs a limit of at most 100 ms): it ORs its bit into ``status``."""
    _require_cuda(status)
    with torch.cuda.device(status.device):
        C.check(C.lib().hot_wait_probe(status.data_ptr(), torch.cuda.current_stream(status.device).cuda_stream), "hot_wait_probe")


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("hot_b200 runs on CUDA tensors only (there is no CPU path)")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _dtype(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError("hot_b200 supports float32 and bfloat16 tensors, got %s" % t.dtype) from None


def _pitch16(nbytes: int) -> int:
    return (nbytes + 15) // 16 * 16


def row_ht_quant(x: torch.Tensor, order: int, q: Quant):
    """Block-Hadamard transform of the last dim of ``x`` [rows, cols] + quantisation.
    Returns (codes uint8 [rows, cols] or [rows, cols/2] packed (a view whose row pitch is a
    multiple of 16 bytes), scales float32 [1] or [rows])."""
    _require_cuda(x)
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be 2-D with a contiguous last dim")
    rows, cols = x.shape
    row_bytes = cols // 2 if q.storage == "int4" else cols
    codes = torch.empty((rows, _pitch16(row_bytes)), dtype=torch.uint8, device=x.device)[:, :row_bytes]
    scales = torch.empty((rows if q.scale == "row" else 1,), dtype=torch.float32, device=x.device)
    ws = torch.empty((16,), dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        C.check(C.lib().hot_row_ht_quant(x.data_ptr(), _dtype(x), rows, cols, x.stride(0), order, ctypes.byref(q.to_c()),
                                         codes.data_ptr(), codes.stride(0), scales.data_ptr(), ws.data_ptr(), _stream(x)),
                "hot_row_ht_quant")
    return codes, scales


def col_ht_quant(x: torch.Tensor, order: int, sel: Sequence[int], q: Quant, logical_layout: str = "natural"):
    """Block Walsh-Hadamard transform of the FIRST dim of ``x`` [rows, cols] keeping the rows
    ``sel`` of H_order, + quantisation, written transposed.  Returns (codes_t uint8
    [cols, pitch] whose first rows*r/order (int8) or half that (int4) bytes per row are codes,
    scales float32 [1] or [cols], out_len)."""
    _require_cuda(x)
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be 2-D with a contiguous last dim")
    rows, cols = x.shape
    r = len(sel)
    out_len = rows // order * r
    pitch = _pitch16((out_len + 1) // 2 if q.storage == "int4" else out_len)
    codes = torch.empty((cols, pitch), dtype=torch.uint8, device=x.device)
    scales = torch.empty((cols if q.scale == "row" else 1,), dtype=torch.float32, device=x.device)
    words = C.lib().hot_col_ht_quant_scratch_words(_dtype(x), rows, cols, order, r, q.to_c().scale_mode)
    ws = torch.empty((max(int(words), 16) + 1) // 2, dtype=torch.int64, device=x.device)   # 8-byte aligned
    sel_c = (C.c_i32 * r)(*[int(s) for s in sel])
    with torch.cuda.device(x.device):
        C.check(C.lib().hot_col_ht_quant(x.data_ptr(), _dtype(x), rows, cols, x.stride(0), order, sel_c, r,
                                         ctypes.byref(q.to_c()),
                                         C.LAYOUT_TRANSPOSED if logical_layout == "transposed" else C.LAYOUT_NATURAL,
                                         codes.data_ptr(), pitch, scales.data_ptr(), ws.data_ptr(), _stream(x)),
                "hot_col_ht_quant")
    return codes, scales, out_len


def col_ht_quant_static(x: torch.Tensor, order: int, sel: Sequence[int], q: Quant, logical_layout: str = "natural"):
    """``col_ht_quant`` through ``hot_col_ht_quant_static``: the library's built-in scratch array
    stands in for the abs-max workspace, so this wrapper hands the library nothing but the
    input and the two outputs.  Per-row scales are limited to 16384 columns.  Calls on one
    device share that array: keep them on one stream (or otherwise ordered)."""
    _require_cuda(x)
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be 2-D with a contiguous last dim")
    rows, cols = x.shape
    r = len(sel)
    out_len = rows // order * r
    pitch = _pitch16((out_len + 1) // 2 if q.storage == "int4" else out_len)
    codes = torch.empty((cols, pitch), dtype=torch.uint8, device=x.device)
    scales = torch.empty((cols if q.scale == "row" else 1,), dtype=torch.float32, device=x.device)
    sel_c = (C.c_i32 * r)(*[int(s) for s in sel])
    with torch.cuda.device(x.device):
        C.check(C.lib().hot_col_ht_quant_static(x.data_ptr(), _dtype(x), rows, cols, x.stride(0), order, sel_c, r,
                                                ctypes.byref(q.to_c()),
                                                C.LAYOUT_TRANSPOSED if logical_layout == "transposed" else C.LAYOUT_NATURAL,
                                                codes.data_ptr(), pitch, scales.data_ptr(), _stream(x)),
                "hot_col_ht_quant_static")
    return codes, scales, out_len


def gemm_i8(a: torch.Tensor, a_storage: str, b: torch.Tensor, b_storage: str, M: int, N: int, K: int,
            scale_a: Optional[torch.Tensor], scale_b: Optional[torch.Tensor], post: float = 1.0,
            out_dtype: torch.dtype = torch.float32, status: Optional[torch.Tensor] = None,
            stream_k: bool = False, a_rows_per_scale: int = 1) -> torch.Tensor:
    """out [M, N] = ((a . b^T) * scale_a[m or 0]) * scale_b[n or 0] * post on the tcgen05 integer path;
    ``a`` [M, pitch] and ``b`` [N, pitch] are uint8/int8 code matrices with K contiguous.
    ``out_dtype=torch.int32`` returns the raw accumulator.  ``stream_k=True`` hands the kernel a
    workspace so that it may balance k-blocks over the SMs (same results).  With
    ``a_rows_per_scale = k > 1``, ``scale_a`` holds one scale per k consecutive rows of ``a``."""
    _require_cuda(a, b)
    odt = {torch.float32: C.HOT_F32, torch.bfloat16: C.HOT_BF16, torch.int32: C.HOT_I32}[out_dtype]
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    sa = scale_a.data_ptr() if scale_a is not None else None
    sb = scale_b.data_ptr() if scale_b is not None else None
    with torch.cuda.device(a.device):
        ws = None
        if stream_k:
            ws = torch.empty((int(C.lib().hot_gemm_i8_workspace_bytes(M, N)),), dtype=torch.uint8, device=a.device)
        C.check(C.lib().hot_gemm_i8_ws(a.data_ptr(), C.STORE_INT4 if a_storage == "int4" else C.STORE_INT8, a.stride(0),
                                       b.data_ptr(), C.STORE_INT4 if b_storage == "int4" else C.STORE_INT8, b.stride(0),
                                       M, N, K, sa,
                                       int(a_rows_per_scale) if (scale_a is not None and scale_a.numel() > 1) else 0, sb,
                                       int(scale_b is not None and scale_b.numel() > 1), float(post), out.data_ptr(), odt,
                                       out.stride(0), ws.data_ptr() if ws is not None else None,
                                       ws.numel() if ws is not None else 0,
                                       status.data_ptr() if status is not None else None, _stream(a)),
                "hot_gemm_i8_ws")
    return out


def gemm_i8_dual(main: dict, rider: dict, status: Optional[torch.Tensor] = None):
    """Two ``gemm_i8`` problems in one launch (the rider's tiles fill the SMs the main problem's last
    wave leaves idle); each dict holds a, a_storage ("int8" | "int4"; rider: "int8"), b, M, N, K,
    scale_a, scale_b, post, out_dtype and optionally a_rows_per_scale.  Returns (out_main, out_rider)."""
    outs, probs = [], []
    odts = {torch.float32: C.HOT_F32, torch.bfloat16: C.HOT_BF16, torch.int32: C.HOT_I32}
    for g in (main, rider):
        a, b = g["a"], g["b"]
        _require_cuda(a, b)
        out = torch.empty((g["M"], g["N"]), dtype=g.get("out_dtype", torch.float32), device=a.device)
        sa, sb = g.get("scale_a"), g.get("scale_b")
        pr = C.HotGemmProblem()
        pr.a, pr.a_storage, pr.lda = a.data_ptr(), C.STORE_INT4 if g.get("a_storage", "int8") == "int4" else C.STORE_INT8, a.stride(0)
        pr.b, pr.ldb = b.data_ptr(), b.stride(0)
        pr.M, pr.N, pr.K = g["M"], g["N"], g["K"]
        pr.scale_a = sa.data_ptr() if sa is not None else None
        pr.scale_a_per_row = int(g.get("a_rows_per_scale", 1)) if (sa is not None and sa.numel() > 1) else 0
        pr.scale_b = sb.data_ptr() if sb is not None else None
        pr.scale_b_per_row = int(sb is not None and sb.numel() > 1)
        pr.post = float(g.get("post", 1.0))
        pr.out, pr.out_dtype, pr.ldo = out.data_ptr(), odts[out.dtype], out.stride(0)
        outs.append(out)
        probs.append(pr)
    with torch.cuda.device(main["a"].device):
        C.check(C.lib().hot_gemm_i8_dual(ctypes.byref(probs[0]), ctypes.byref(probs[1]),
                                         status.data_ptr() if status is not None else None, _stream(main["a"])),
                "hot_gemm_i8_dual")
    return outs[0], outs[1]


def row_ht_quant_batched(x: torch.Tensor, order: int, q: Quant):
    """``row_ht_quant`` on a batch ``x`` [B, rows, cols] with one scale per sample.  Returns (codes
    uint8 [B*rows, cols] or packed [B*rows, cols/2], scales float32 [B])."""
    _require_cuda(x)
    if x.dim() != 3 or not x.is_contiguous():
        raise ValueError("x must be a contiguous 3-D tensor")
    B, rows, cols = x.shape
    row_bytes = cols // 2 if q.storage == "int4" else cols
    codes = torch.empty((B * rows, _pitch16(row_bytes)), dtype=torch.uint8, device=x.device)[:, :row_bytes]
    scales = torch.empty((B,), dtype=torch.float32, device=x.device)
    ws = torch.empty((max(B, 16),), dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        C.check(C.lib().hot_row_ht_quant_batched(x.data_ptr(), _dtype(x), B, rows, cols, cols, order, ctypes.byref(q.to_c()),
                                                 codes.data_ptr(), codes.stride(0), scales.data_ptr(), ws.data_ptr(),
                                                 _stream(x)), "hot_row_ht_quant_batched")
    return codes, scales


def sample_pitch(out_len: int) -> int:
    """Bytes one sample takes along the contraction axis of a batched, transposed INT8 operand:
    its codes rounded up to whole 128-byte k-blocks of the integer GEMM."""
    return (out_len + 127) // 128 * 128


def col_ht_quant_batched(x: torch.Tensor, order: int, sel: Sequence[int], q: Quant, logical_layout: str = "natural"):
    """``col_ht_quant`` on a batch ``x`` [B, rows, cols], transform along the rows of each sample, one
    scale per sample (``q.scale`` "tensor" or "sawb") or one per sample and output row ("row").
    Returns (codes_t uint8 [cols, B * pitch] with sample b at byte b * pitch of each row, zero
    padded, scales float32 [B] or [B, cols], out_len per sample, pitch)."""
    _require_cuda(x)
    if x.dim() != 3 or not x.is_contiguous():
        raise ValueError("x must be a contiguous 3-D tensor")
    B, rows, cols = x.shape
    r = len(sel)
    out_len = rows // order * r
    pitch = sample_pitch(out_len)
    codes = torch.empty((cols, B * pitch), dtype=torch.uint8, device=x.device)
    scales = torch.empty((B, cols) if q.scale == "row" else (B,), dtype=torch.float32, device=x.device)
    words = B * cols if q.scale == "row" else B
    if q.scale == "sawb":
        words = B * int(C.lib().hot_col_ht_quant_scratch_words(_dtype(x), rows, cols, order, r, q.to_c().scale_mode))
    ws = torch.empty((max(words, 16) + 1) // 2, dtype=torch.int64, device=x.device)   # 8-byte aligned
    sel_c = (C.c_i32 * r)(*[int(v) for v in sel])
    with torch.cuda.device(x.device):
        C.check(C.lib().hot_col_ht_quant_batched(x.data_ptr(), _dtype(x), B, rows, cols, cols, order, sel_c, r,
                                                 ctypes.byref(q.to_c()),
                                                 C.LAYOUT_TRANSPOSED if logical_layout == "transposed" else C.LAYOUT_NATURAL,
                                                 codes.data_ptr(), codes.stride(0), pitch, scales.data_ptr(), ws.data_ptr(),
                                                 _stream(x)), "hot_col_ht_quant_batched")
    return codes, scales, out_len, pitch


def gemm_i8_grouped(a: torch.Tensor, b: torch.Tensor, M: int, N: int, groups: int, group_k: int, scale_a: torch.Tensor,
                    scale_b: torch.Tensor, post: float = 1.0, out_dtype: torch.dtype = torch.float32,
                    status: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out [M, N] = (sum_g ((a_g . b_g^T) * scale_a[g]) * scale_b[g]) * post, where group g is the
    columns [g * group_k, (g + 1) * group_k) of the INT8 code matrices ``a`` [M, .] and ``b`` [N, .]
    (group_k a multiple of 128); the sum over groups runs in fp32, group 0 first.  ``scale_a`` of
    shape [groups, M] gives every row of ``a`` its own scale within each group."""
    _require_cuda(a, b, scale_a, scale_b)
    odt = {torch.float32: C.HOT_F32, torch.bfloat16: C.HOT_BF16}[out_dtype]
    if out is None:  # the kernel stores through a tensor map: the row pitch must be a multiple of 16 bytes
        per16 = 16 // torch.empty((), dtype=out_dtype).element_size()
        out = torch.empty((M, (N + per16 - 1) // per16 * per16), dtype=out_dtype, device=a.device)[:, :N]
    with torch.cuda.device(a.device):
        per_row = scale_a.dim() == 2
        if per_row and (tuple(scale_a.shape) != (groups, M) or not scale_a.is_contiguous()):
            raise ValueError("per-row scale_a must be a contiguous [groups, M] tensor")
        C.check(C.lib().hot_gemm_i8_grouped(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), M, N, groups, group_k,
                                            scale_a.data_ptr(), 1 if per_row else 0, scale_b.data_ptr(), float(post),
                                            out.data_ptr(), odt,
                                            out.stride(0), status.data_ptr() if status is not None else None, _stream(a)),
                "hot_gemm_i8_grouped")
    return out


@dataclass
class LinearConfig:
    """Per-layer backward configuration (mirrors ``hot_linear_cfg_t``)."""
    order_o: int
    order_l: int
    sel_l: Sequence[int]
    q_gx: Quant = field(default_factory=lambda: Quant(4, "int4"))
    q_w: Quant = field(default_factory=lambda: Quant(4, "int4"))
    q_gw: Quant = field(default_factory=lambda: Quant(8, "int8"))
    q_x: Quant = field(default_factory=lambda: Quant(8, "int8"))

    def to_c(self, dtype: torch.dtype) -> C.HotLinearCfg:
        c = C.HotLinearCfg()
        c.dtype = _DTYPES[dtype]
        c.order_o, c.order_l, c.rank_l = self.order_o, self.order_l, len(self.sel_l)
        for i, s in enumerate(self.sel_l):
            c.sel_l[i] = int(s)
        c.q_gx, c.q_w, c.q_gw, c.q_x = self.q_gx.to_c(), self.q_w.to_c(), self.q_gw.to_c(), self.q_x.to_c()
        return c

    def out_len(self, L: int) -> int:
        return L // self.order_l * len(self.sel_l)


def abc_compress(x: torch.Tensor, cfg: LinearConfig):
    """Activation-buffer compression: x [L, I] -> (x_q_t uint8 [I, pitch], scale_x float32 [1])."""
    _require_cuda(x)
    if cfg.order_l > MAX_KERNEL_ORDER:   # project in two passes, then quantise the projected rows as they are
        return abc_compress(hla_project_any(x, cfg.order_l, cfg.sel_l), _identity_tokens(cfg))
    L, I = x.shape
    cc = cfg.to_c(x.dtype)
    pitch = C.lib().hot_abc_pitch(L, ctypes.byref(cc))
    if pitch <= 0:
        raise ValueError("token count %d is not a multiple of the low-rank order %d" % (L, cfg.order_l))
    x_q_t = torch.empty((I, pitch), dtype=torch.uint8, device=x.device)
    scale = torch.empty((1,), dtype=torch.float32, device=x.device)
    words = C.lib().hot_col_ht_quant_scratch_words(_DTYPES[x.dtype], L, I, cfg.order_l, len(cfg.sel_l), cc.q_x.scale_mode)
    ws = torch.empty((max(int(words), 16) * 4,), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        C.check(C.lib().hot_abc_compress(x.data_ptr(), L, I, x.stride(0), ctypes.byref(cc), x_q_t.data_ptr(),
                                         scale.data_ptr(), ws.data_ptr(), ws.numel(), _stream(x)), "hot_abc_compress")
    return x_q_t, scale


def _identity_tokens(cfg: "LinearConfig") -> "LinearConfig":
    """The same configuration with no transform along the tokens (order 1): for operands projected beforehand."""
    return LinearConfig(order_o=cfg.order_o, order_l=1, sel_l=[0], q_gx=cfg.q_gx, q_w=cfg.q_w, q_gw=cfg.q_gw, q_x=cfg.q_x)


def gx_code_storage(bits: int, k: int) -> str:
    """How the g_x codes of grad_out travel from the quantiser to the GEMM.  Codes of up to 4 bits are
    packed two per byte and expanded to int8 in the GEMM's shared memory when the contraction is very long
    (k >= 4096: the packed tensor saves 30-90 MB of HBM traffic per layer at 16,384 tokens); below that they are
    stored one per byte, which the GEMM takes as it is.  Measured on the 48 ViT-B/16 linears at 12,608 tokens with the
    tensor-core quantiser, whose stores are not what bounds it: 3.34 ms per step one per byte everywhere against 3.37 ms
    with qkv and fc1 (k = 2304, 3072) packed; the GEMM gains 2.8 us per such layer, the quantiser loses 1.7.  The
    codes, scales and results are the same either way."""
    return "int4" if bits <= 4 and k >= 4096 else "int8"


def go_dual_quant(go: torch.Tensor, cfg: LinearConfig, status: Optional[torch.Tensor] = None):
    """Both quantised operands of grad_out from the fused kernels (one HBM read per pass):
    returns (q_go codes [L, O/2 or O], s_gx [1] or [L], q_gw_t codes [O, pitch], s_gw [1] or [O]).
    Raises for configurations the fused kernels do not cover (see ``hot_go_dual_quant``)."""
    _require_cuda(go)
    L, O = go.shape
    cc = cfg.to_c(go.dtype)
    gx4 = cfg.q_gx.storage == "int4"
    q_go = torch.empty((L, _pitch16(O // 2 if gx4 else O)), dtype=torch.uint8, device=go.device)
    lp = cfg.out_len(L)
    q_gw = torch.empty((O, _pitch16(lp)), dtype=torch.uint8, device=go.device)
    s_gx = torch.empty((L if cfg.q_gx.scale == "row" else 1,), dtype=torch.float32, device=go.device)
    s_gw = torch.empty((O if cfg.q_gw.scale == "row" else 1,), dtype=torch.float32, device=go.device)
    ws = torch.empty((L + O + 64,), dtype=torch.int32, device=go.device)
    with torch.cuda.device(go.device):
        C.check(C.lib().hot_go_dual_quant(go.data_ptr(), L, O, go.stride(0), ctypes.byref(cc), q_go.data_ptr(), q_go.stride(0),
                                          s_gx.data_ptr(), q_gw.data_ptr(), q_gw.stride(0), s_gw.data_ptr(), ws.data_ptr(),
                                          status.data_ptr() if status is not None else None, _stream(go)),
                "hot_go_dual_quant")
    return q_go[:, :(O // 2 if gx4 else O)], s_gx, q_gw, s_gw


_workspaces: dict = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """One growing scratch buffer per (device, stream): kernels of consecutive layers on a
    stream run in order, so they can share it."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty((max(nbytes, 1 << 20),), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def linear_backward(go: torch.Tensor, w: torch.Tensor, x_q_t: torch.Tensor, scale_x: torch.Tensor, cfg: LinearConfig,
                    need_gx: bool = True, need_gw: bool = True, status: Optional[torch.Tensor] = None,
                    gx_out: Optional[torch.Tensor] = None, gw_out: Optional[torch.Tensor] = None):
    """HOT backward of one linear layer: returns (grad_x [L, I] or None, grad_w [O, I] or None).
    ``gx_out`` / ``gw_out`` are optional preallocated row-major destinations (e.g. a slice of a
    gradient bucket)."""
    _require_cuda(go, w, x_q_t)
    L, O = go.shape
    I = w.shape[1]
    if cfg.order_l > MAX_KERNEL_ORDER:
        # token basis of order above 64: grad_x does not involve it; for grad_w grad_out is projected in two passes
        # and quantised as it is (the activation buffer was made the same way by abc_compress)
        gx = gw = None
        if need_gx:
            gx, _ = linear_backward(go, w, x_q_t, scale_x, _identity_tokens(cfg), True, False, status, gx_out, None)
        if need_gw:
            go_lr = hla_project_any(go, cfg.order_l, cfg.sel_l)
            q_gw_t, s_gw, lp = col_ht_quant(go_lr, 1, [0], _one_per_byte(cfg.q_gw), "transposed")
            gw = gemm_i8(q_gw_t, "int8", x_q_t, "int8", O, I, lp, s_gw, scale_x, 1.0 / cfg.order_l, go.dtype, status=status)
            if gw_out is not None:
                gw_out.copy_(gw)
                gw = gw_out
        return gx, gw
    cc = cfg.to_c(go.dtype)
    nbytes = C.lib().hot_linear_workspace_bytes(L, O, I, ctypes.byref(cc))
    if nbytes == 0:
        raise ValueError("unsupported sizes L=%d O=%d I=%d for this configuration" % (L, O, I))
    ws = _workspace(go.device, nbytes)
    gx = (gx_out if gx_out is not None else torch.empty((L, I), dtype=go.dtype, device=go.device)) if need_gx else None
    gw = (gw_out if gw_out is not None else torch.empty((O, I), dtype=go.dtype, device=go.device)) if need_gw else None
    for t, shape in ((gx, (L, I)), (gw, (O, I))):
        if t is not None and (tuple(t.shape) != shape or t.dtype != go.dtype or t.stride(1) != 1):
            raise ValueError("gradient buffer must be %s %s with a contiguous last dim" % (shape, go.dtype))
    with torch.cuda.device(go.device):
        C.check(C.lib().hot_linear_backward(go.data_ptr(), go.stride(0), w.data_ptr(), w.stride(0), x_q_t.data_ptr(),
                                            scale_x.data_ptr(), L, O, I, ctypes.byref(cc),
                                            gx.data_ptr() if need_gx else None, gx.stride(0) if need_gx else I,
                                            gw.data_ptr() if need_gw else None, gw.stride(0) if need_gw else I,
                                            ws.data_ptr(), ws.numel(), status.data_ptr() if status is not None else None,
                                            _stream(go)), "hot_linear_backward")
    return gx, gw


def hla_project(x: torch.Tensor, order: int, sel: Sequence[int]) -> torch.Tensor:
    """Un-quantised low-rank projection along the first dim: x [rows, cols] -> float32 [rows*r/order, cols]."""
    _require_cuda(x)
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be 2-D with a contiguous last dim")
    rows, cols = x.shape
    r = len(sel)
    out = torch.empty((rows // order * r, cols), dtype=torch.float32, device=x.device)
    sel_c = (C.c_i32 * r)(*[int(v) for v in sel])
    with torch.cuda.device(x.device):
        C.check(C.lib().hot_hla_project(x.data_ptr(), _dtype(x), rows, cols, x.stride(0), order, sel_c, r, out.data_ptr(),
                                        out.stride(0), _stream(x)), "hot_hla_project")
    return out


MAX_KERNEL_ORDER = 64   # largest transform order a single kernel launch takes


def hla_project_any(x: torch.Tensor, order: int, sel: Sequence[int]) -> torch.Tensor:
    """``hla_project`` for any power-of-two order up to 4096.  Orders above 64 (a token count such as 128
    or 1024 under the reference's uncapped make_WHT, or the output-feature basis of ``gilro_gwh``) run as two
    passes of the order-<=64 kernel: H_(a*64) = H_a (x) H_64, so the 64-point butterflies run first on
    groups of 64 rows and the a-point ones then on rows 64 apart -- the same stage order h = 1, 2, 4, ... as a
    single butterfly, hence the same float32 results -- and the kept rows are gathered at the end."""
    if order <= MAX_KERNEL_ORDER:
        return hla_project(x, order, sel)
    if order & (order - 1) or order > MAX_KERNEL_ORDER ** 2:
        raise ValueError("transform order %d is not a power of two <= %d" % (order, MAX_KERNEL_ORDER ** 2))
    rows, cols = x.shape
    if rows % order:
        raise ValueError("rows %d not a multiple of order %d" % (rows, order))
    b, a = MAX_KERNEL_ORDER, order // MAX_KERNEL_ORDER
    y = hla_project(x, b, list(range(b)))                                   # [rows, cols]: index (blk, t_a, i_b)
    y = hla_project(y.view(rows // b, b * cols), a, list(range(a)))         # rows (blk, t_a) -> (blk, i_a)
    full = y.view(rows // order, order, cols)                               # natural row index i_a * 64 + i_b
    idx = torch.as_tensor([int(v) for v in sel], device=x.device, dtype=torch.long)
    return full.index_select(1, idx).reshape(-1, cols)


def hla_expand(y: torch.Tensor, order: int, sel: Sequence[int], scale: float, out_dtype: torch.dtype) -> torch.Tensor:
    """Transpose of ``hla_project``: y float32 [rows*r/order, cols] -> [rows, cols] of ``out_dtype``, times ``scale``."""
    _require_cuda(y)
    if y.dim() != 2 or y.stride(1) != 1 or y.dtype != torch.float32:
        raise ValueError("y must be a 2-D float32 tensor with a contiguous last dim")
    r = len(sel)
    rows = y.shape[0] // r * order
    cols = y.shape[1]
    out = torch.empty((rows, cols), dtype=out_dtype, device=y.device)
    sel_c = (C.c_i32 * r)(*[int(v) for v in sel])
    with torch.cuda.device(y.device):
        C.check(C.lib().hot_hla_expand(y.data_ptr(), y.stride(0), rows, cols, order, sel_c, r, float(scale), out.data_ptr(),
                                       _DTYPES[out_dtype], out.stride(0), _stream(y)), "hot_hla_expand")
    return out


def linear_backward_lowrank_gx(go: torch.Tensor, w: torch.Tensor, order: int, sel: Sequence[int], q_gx: Quant, q_w: Quant,
                               status: Optional[torch.Tensor] = None, batch: int = 1) -> torch.Tensor:
    """grad_input of the schemes that project grad_output along the TOKENS before the g_x product
    (transform_scheme low_rank / gilr_gwh, utils/quant_matmul.py:229-234, 261-266, 334-337):
    grad_x = expand( (Q(HLA(go)) . Q(w)) * s_go * s_w ) / order, the weight left untransformed.
    ``batch`` > 1: ``go`` holds that many samples of L / batch tokens each (a multiple of ``order``, so
    the projection blocks stay within a sample) and the quantiser takes one scale per sample."""
    _require_cuda(go, w)
    L, O = go.shape
    I = w.shape[1]
    if batch > 1 and (L % batch or (L // batch) % order):
        raise ValueError("tokens per sample must be a multiple of the low-rank order %d" % order)
    go_lr = hla_project(go, order, sel)                                     # [L', O] float32, natural layout
    rows_per_scale = 1
    if batch > 1 and q_gx.scale == "tensor":
        q_go, s_go = row_ht_quant_batched(go_lr.view(batch, -1, O), 1, q_gx)
        rows_per_scale = go_lr.shape[0] // batch
    else:
        q_go, s_go = row_ht_quant(go_lr, 1, q_gx)
    q_w_t, s_w, _ = col_ht_quant(w, 1, [0], _one_per_byte(q_w), "natural")  # [I, O] codes, no transform
    gi_lr = gemm_i8(q_go, q_gx.storage, q_w_t, "int8", go_lr.shape[0], I, O, s_go, s_w, 1.0, torch.float32, status=status,
                    a_rows_per_scale=rows_per_scale)
    return hla_expand(gi_lr, order, sel, 1.0 / order, go.dtype)


def linear_backward_gilro_gx(go: torch.Tensor, w: torch.Tensor, order: int, sel: Sequence[int], q_gx: Quant, q_w: Quant,
                             status: Optional[torch.Tensor] = None, batch: int = 1) -> torch.Tensor:
    """grad_input of transform_scheme ``gilro_gwh`` (utils/quant_matmul.py:235-236, 267-268, 288-290, 339-340):
    grad_output [L, O] and the weight [O, I] are both projected along the OUTPUT FEATURES onto the kept rows of
    H_order (order = the whole 2-adic part of O, up to 1024 for ViT widths), quantised, and multiplied over the
    shortened feature axis: grad_x = (Q(go . P^T) . Q(P w)) * s_go * s_w / order.  ``batch`` > 1: one scale per
    sample for grad_output, as the reference's batched quantiser gives."""
    import torch.nn.functional as F
    _require_cuda(go, w)
    L, O = go.shape
    I = w.shape[1]
    go_lr = hla_project_any(go.t().contiguous(), order, sel).t().contiguous()       # [L, O'] float32
    w_lr = hla_project_any(w, order, sel)                                            # [O', I] float32
    pad = (-go_lr.shape[1]) % 16      # the quantiser works on runs of 16; zero features add nothing to the product
    if pad:
        go_lr = F.pad(go_lr, (0, pad))
        w_lr = F.pad(w_lr, (0, 0, 0, pad))
    K = go_lr.shape[1]
    rows_per_scale = 1
    if batch > 1 and q_gx.scale == "tensor":
        q_go, s_go = row_ht_quant_batched(go_lr.view(batch, L // batch, K), 1, q_gx)
        rows_per_scale = L // batch
    else:
        q_go, s_go = row_ht_quant(go_lr, 1, q_gx)
    q_w_t, s_w, _ = col_ht_quant(w_lr, 1, [0], _one_per_byte(q_w), "natural")        # [I, O'] codes
    return gemm_i8(q_go, q_gx.storage, q_w_t, "int8", L, I, K, s_go, s_w, 1.0 / order, go.dtype, status=status,
                   a_rows_per_scale=rows_per_scale)


def abc_compress_batched(x: torch.Tensor, cfg: LinearConfig):
    """Activation buffer of a batch ``x`` [B, L, I] with one scale per sample, as the reference saves
    it for 3-D inputs: (x_q_t uint8 [I, B * pitch], scale_x float32 [B], pitch)."""
    if cfg.order_l > MAX_KERNEL_ORDER:   # projection blocks never straddle samples: project the flattened batch
        B, L, I = x.shape
        x_lr = hla_project_any(x.reshape(B * L, I), cfg.order_l, cfg.sel_l).view(B, -1, I)
        return abc_compress_batched(x_lr, _identity_tokens(cfg))
    codes, scales, _, pitch = col_ht_quant_batched(x, cfg.order_l, cfg.sel_l, _one_per_byte(cfg.q_x), "natural")
    return codes, scales, pitch


def _one_per_byte(q: Quant) -> Quant:
    """The same quantiser with its codes stored one per byte (the batched operands are INT8-stored)."""
    return Quant(q.bits, "int8", q.rounding, q.scale, q.seed, q.offset, q.noise)


def linear_backward_batched(go: torch.Tensor, w: torch.Tensor, x_q_t: torch.Tensor, scale_x: torch.Tensor,
                            cfg: LinearConfig, need_gx: bool = True, need_gw: bool = True,
                            status: Optional[torch.Tensor] = None):
    """HOT backward of one linear layer on a batch ``go`` [B, L, O] with the reference's 3-D
    semantics: every quantiser of grad_out and of the activation takes one scale per sample, the
    low-rank projection runs along the tokens of each sample, and grad_w is the fp32 sum over
    samples of the dequantised per-sample products (utils/quant_matmul.py:223-225, 288-290,
    322-324).  With ``scale="row"`` (the reference's norm_quantizer) the g_x side takes one scale per
    token and the g_w side one per sample and output channel.  ``x_q_t`` / ``scale_x`` come from
    ``abc_compress_batched``.  Returns
    (grad_x [B, L, I] or None, grad_w [O, I] or None)."""
    _require_cuda(go, w, x_q_t)
    if go.dim() != 3 or not go.is_contiguous():
        raise ValueError("go must be a contiguous [B, L, O] tensor")
    B, L, O = go.shape
    I = w.shape[1]
    gx = gw = None
    if need_gx:
        if cfg.q_gx.scale == "row":   # one scale per token: the samples' rows are the rows of the flattened tensor
            q_go, s_go = row_ht_quant(go.view(B * L, O), cfg.order_o, cfg.q_gx)
            rows_per_scale = 1
        else:
            q_go, s_go = row_ht_quant_batched(go, cfg.order_o, cfg.q_gx)
            rows_per_scale = L
        q_w_t, s_w, _ = col_ht_quant(w, cfg.order_o, list(range(cfg.order_o)), _one_per_byte(cfg.q_w), "natural")
        gx = gemm_i8(q_go, cfg.q_gx.storage, q_w_t, "int8", B * L, I, O, s_go, s_w, 1.0 / cfg.order_o, go.dtype,
                     status=status, a_rows_per_scale=rows_per_scale).view(B, L, I)
    if need_gw:
        go_w, order_w, sel_w = go, cfg.order_l, cfg.sel_l
        if cfg.order_l > MAX_KERNEL_ORDER:
            go_w, order_w, sel_w = hla_project_any(go.view(B * L, O), cfg.order_l, cfg.sel_l).view(B, -1, O), 1, [0]
        q_gw_t, s_gw, out_len, pitch = col_ht_quant_batched(go_w, order_w, sel_w, _one_per_byte(cfg.q_gw), "transposed")
        if x_q_t.shape[1] != B * pitch:
            raise ValueError("activation buffer does not match: %d bytes per row, expected %d" % (x_q_t.shape[1], B * pitch))
        gw = gemm_i8_grouped(q_gw_t, x_q_t, O, I, B, pitch, s_gw, scale_x, 1.0 / cfg.order_l, go.dtype, status=status)
    return gx, gw
