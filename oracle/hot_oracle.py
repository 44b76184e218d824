"""CPU oracle for the HOT linear-layer backward path.  TEST INFRASTRUCTURE ONLY.

This module restates, in numpy float32 arithmetic, the algorithm of the
reference's fake-quant path so that the CUDA kernels can be compared with it
bit for bit.  It is imported by the tests, by the smoke check and by the CPU
baseline leg of the benchmark, and by nothing that ships: the product path
never routes through this file.

Parity status: PINNED.  ``tests/golden/make_golden.py`` runs the unmodified
reference (utils/quant_matmul.py, utils/hadamard_matmul.py) on seeded inputs
and stores its outputs under ``tests/golden/``; ``tests/test_oracle_golden.py``
checks every function below against those files.

Where the reference leaves the floating-point summation order to a BLAS matmul
(the +-1 transforms of utils/hadamard_matmul.py:121-161) this oracle fixes the
order to the radix-2 butterfly ``h = 1, 2, 4, ...`` with ``(x + y, x - y)`` per
pair, the order of cuda_measure/HLQ_backward_kernel.cu:63-78.  Everything after
the transform (scale, division, rounding) follows the reference expression by
expression.
"""
from __future__ import annotations

import math

import numpy as np

F32 = np.float32
EPS = F32(1e-11)  # args.py:34 and the literal at utils/quant_matmul.py:22


# ----------------------------------------------------------------------------
# transform generators (utils/hadamard_matmul.py)
# ----------------------------------------------------------------------------
def pow2_factor(size: int) -> int:
    """Largest power of two dividing ``size`` (utils/hadamard_matmul.py:9-15)."""
    if size < 1:
        raise ValueError("size must be positive")
    return size & -size


def block_order(size: int) -> int:
    """Hadamard block order used along a dim of ``size``: the largest power of two
    dividing it, capped at 16 (utils/hadamard_matmul.py:17-27)."""
    p = pow2_factor(size)
    return 16 if (p > 16 and size > 16) else p


def hadamard(n: int) -> np.ndarray:
    """Sylvester Hadamard matrix in natural order, entries +-1, unnormalised
    (utils/hadamard_matmul.py:32-51).  H[i, j] = (-1)^popcount(i & j)."""
    if n < 1 or (n & (n - 1)):
        raise ValueError("n must be int and power of 2.")
    i = np.arange(n)
    bits = i[:, None] & i[None, :]
    par = np.zeros_like(bits)
    b = bits.copy()
    while b.any():
        par ^= b & 1
        b >>= 1
    return (1 - 2 * par).astype(np.int64)


def make_hadamard(size: int) -> np.ndarray:
    """utils/hadamard_matmul.py:57-59."""
    return hadamard(block_order(size))


def sequency(row: np.ndarray) -> int:
    """Number of sign changes along a +-1 row (utils/hadamard_matmul.py:211-212)."""
    return int(np.sum(row[:-1] != row[1:]))


def sequency_order(n: int) -> np.ndarray:
    """Natural-order row index of H_n for each sequency 0..n-1.  The sequencies of a
    Sylvester matrix are a permutation of 0..n-1, so the stable sort the reference
    uses (utils/hadamard_matmul.py:213) has no ties."""
    h = hadamard(n)
    seq = np.array([sequency(h[i]) for i in range(n)])
    return np.argsort(seq, kind="stable")


def wht_selection(size: int, percentile: float = 50) -> tuple[int, np.ndarray]:
    """(n, natural-order row indices) of the low-rank basis ``make_WHT(size, pct)``
    keeps (utils/hadamard_matmul.py:209-226): n = largest power of two dividing
    ``size`` (uncapped); rows sorted by sequency; the first q*q of them viewed as q
    groups of q (q*q = largest even power of two <= n); group i keeps q-(i+sf)
    rows, from the front for even i and from the back for odd i."""
    n = 1 if size == 1 else pow2_factor(size)
    order = sequency_order(n)
    # biggest_sqrt_factor: largest i <= n that is a perfect square and a power of two
    q2 = 1
    while q2 * 4 <= n:
        q2 *= 4
    q = int(math.isqrt(q2))
    sf = int(0.1 * (-np.sqrt(2 * q ** 2 * percentile + 25) + 10 * q + 5))
    kept: list[int] = []
    for i in range(q):
        if i % 2 == 0:
            lo, hi = q * i, q * (i + 1) - (i + sf)
        else:
            lo, hi = q * i + (i + sf), q * (i + 1)
        kept.extend(range(lo, max(lo, hi)))
    return n, order[np.array(kept, dtype=np.int64)] if kept else np.zeros(0, np.int64)


def make_WHT(size: int, percentile: float = 50) -> np.ndarray:
    n, sel = wht_selection(size, percentile)
    return hadamard(n)[sel]


def lowrank_preset(n: int, r: int) -> np.ndarray:
    """The r lowest-sequency rows of H_n as natural-order indices ("half16" is
    n=16, r=8: the analytic model's r=8 of n=16, utils/analysis_calculator.py:174-175)."""
    return sequency_order(n)[:r]


def selection_from_matrix(p: np.ndarray) -> tuple[int, np.ndarray]:
    """Recover (n, natural-order row indices) from an [r, n] +-1 matrix whose rows
    are rows of the Sylvester matrix H_n; raises ValueError otherwise."""
    p = np.asarray(p)
    r, n = p.shape
    h = hadamard(n)
    sel = np.empty(r, np.int64)
    for j in range(r):
        hit = np.nonzero((h == np.rint(p[j]).astype(np.int64)[None, :]).all(axis=1))[0]
        if hit.size != 1:
            raise ValueError("row %d is not a row of the order-%d Hadamard matrix" % (j, n))
        sel[j] = hit[0]
    return n, sel


# ----------------------------------------------------------------------------
# fixed-order transforms
# ----------------------------------------------------------------------------
def fwht_last(a: np.ndarray, n: int) -> np.ndarray:
    """Block transform of the LAST dim in blocks of n: out[..., c*n+k] =
    sum_t a[..., c*n+t] * H_n[t, k]  (lowering_matmul_front,
    utils/hadamard_matmul.py:121-141), evaluated as the butterfly
    h = 1, 2, 4, ...: (x, y) -> (x + y, x - y) in float32."""
    a = np.ascontiguousarray(a, dtype=F32)
    shp = a.shape
    v = a.reshape(-1, n).copy()
    h = 1
    while h < n:
        w = v.reshape(-1, n // (2 * h), 2, h)
        x = w[:, :, 0, :].copy()
        y = w[:, :, 1, :].copy()
        w[:, :, 0, :] = x + y
        w[:, :, 1, :] = x - y
        h *= 2
    return v.reshape(shp)


def fwht_first(a: np.ndarray, n: int) -> np.ndarray:
    """Block transform of the FIRST dim of a 2-D array in blocks of n:
    out[b*n+k, :] = sum_t H_n[k, t] * a[b*n+t, :]  (lowering_matmul_back with a
    square H, utils/hadamard_matmul.py:143-161), same butterfly order."""
    a = np.asarray(a, dtype=F32)
    return np.ascontiguousarray(fwht_last(np.ascontiguousarray(a.T), n).T)


def hla(a: np.ndarray, n: int, sel: np.ndarray) -> np.ndarray:
    """Hadamard low-rank projection along the first dim: out[b*r+j, :] =
    sum_t H_n[sel[j], t] * a[b*n+t, :]  (lowering_matmul_back with the [r, n]
    matrix of make_WHT, utils/hadamard_matmul.py:152), evaluated as the full
    order-n butterfly followed by the row selection."""
    a = np.asarray(a, dtype=F32)
    R, C = a.shape
    full = fwht_first(a, n).reshape(R // n, n, C)
    return np.ascontiguousarray(full[:, np.asarray(sel), :].reshape(-1, C))


# ----------------------------------------------------------------------------
# quantisers (utils/quant_matmul.py:19-122); codes are returned as int32
# ----------------------------------------------------------------------------
def _qmax(bits: int) -> F32:
    return F32(2 ** (bits - 1) - 1)


PHILOX_ROUNDS = 7
_K_MAGIC = 12582912  # 1.5 * 2^23: a float32 in [2^23, 2^24) holds an integer in its low mantissa bits


def rand_bits(bits: int) -> int:
    """Random bits per code of the kernels' production rounding: 4 for codes of up to 4 bits, else 8."""
    return 4 if bits <= 4 else 8


class PhiloxBytes(np.ndarray):
    """Marker type (uint16 per element) for the kernels' production rounding path.  The low byte
    is the element's 8-bit random number R8, the high byte its 4-bit one R4 (see ``philox_bytes``).
    With RB = rand_bits(bits), R the RB-bit random number, B = qmax + 1, d = s + eps and
    m = fl(2^RB / d) (one float32 division per scale):
        K = round_half_even(x * m) + 2^RB * B        (x * m exact: what fl(fma(x, m, 1.5 * 2^23 + 2^RB * B)) leaves
                                                      in the low mantissa bits)
        code = ((K + R) >> RB) - B
    i.e. x / d is rounded to RB fractional bits, a uniform RB-bit integer is added and the sum is
    floored: it rounds up with probability round(2^RB * frac) / 2^RB, unbiased.  |code| <= qmax holds
    without a clamp.  Plain float arrays keep the reference's predicate  u < frac."""


def _codes(xc: np.ndarray, d, u, qmax: F32) -> np.ndarray:
    """Codes of the clamped values ``xc`` for the divisor ``d`` = s + eps (scalar or broadcastable)."""
    d = np.asarray(d, dtype=F32)
    if isinstance(u, PhiloxBytes):
        bits = int(qmax).bit_length() + 1
        rb = rand_bits(bits)
        off = int(qmax) + 1
        m = (F32(1 << rb) / d).astype(F32)
        k = np.rint(xc.astype(np.float64) * m.astype(np.float64)).astype(np.int64) + (off << rb)
        r = np.asarray(u).astype(np.int64)
        r = (r >> 8) & 0xF if rb == 4 else r & 0xFF
        return (((k + r) >> rb) - off).astype(np.int32)
    y = (xc / d).astype(F32)
    if u is None:  # torch.round: half to even (utils/quant_matmul.py:47,115)
        return np.rint(y).astype(np.int32)
    a = np.abs(y)
    f = np.floor(a)
    frac = a - f
    flip = (np.asarray(u, dtype=F32) < frac).astype(F32)  # torch.bernoulli(frac) == (u < frac)
    return (np.sign(y) * (f + flip)).astype(np.int32)


def quant_tensor(x: np.ndarray, bits: int, u: np.ndarray | None):
    """stoch_quantizer_BWD (u given, :86-100) / int_quantizer_BWD (u None, :108-115):
    one abs-max scale for the whole tensor.  Returns (codes int32, s float32)."""
    x = np.asarray(x, dtype=F32)
    mx = np.max(np.abs(x)) if x.size else F32(0)
    s = F32(mx / _qmax(bits))
    return _codes(np.clip(x, -mx, mx), F32(s + EPS), u, _qmax(bits)), s


def quant_rows(x: np.ndarray, bits: int, u: np.ndarray | None):
    """norm_quantizer_BWD (:19-31): abs-max scale per row (dim=1).  Returns
    (codes int32, s float32[rows]); the reference returns codes*s and scale 1."""
    x = np.asarray(x, dtype=F32)
    mx = np.max(np.abs(x), axis=1, keepdims=True)
    s = (mx / _qmax(bits)).astype(F32)
    return _codes(np.clip(x, -mx, mx), (s + EPS).astype(F32), u, _qmax(bits)), s[:, 0]


def quant_sawb(x: np.ndarray, bits: int):
    """sawb_quantizer_BWD (:40-49): clip = 12.1*sqrt(mean(x^2)) - 12.2*mean(|x|),
    nearest rounding.  Means are taken in float64 and rounded once (the reference's
    float32 mean has an unspecified summation order)."""
    x = np.asarray(x, dtype=F32)
    xd = x.astype(np.float64)
    clip = F32(F32(12.1) * F32(np.sqrt(F32(np.mean(xd * xd)))) - F32(12.2) * F32(np.mean(np.abs(xd))))
    s = F32(clip / _qmax(bits))
    y = np.clip(x, -clip, clip) / F32(s + EPS)
    return np.rint(y).astype(np.int32), s


# ----------------------------------------------------------------------------
# counter-based random numbers (Philox4x32-7); mirrored bit for bit by the CUDA kernels
# ----------------------------------------------------------------------------
_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)


def philox4x32(c0, c1, c2, c3, k0: int, k1: int, rounds: int = PHILOX_ROUNDS):
    """Philox4x32 with ``rounds`` rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3";
    10 rounds is the paper's default, 7 the fewest it reports as passing BigCrush)."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) for c in (c0, c1, c2, c3))
    for _ in range(rounds):
        p0 = _M0 * c0
        p1 = _M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK
        c0, c1, c2, c3 = (hi1 ^ c1 ^ np.uint64(k0)) & _MASK, lo1, (hi0 ^ c3 ^ np.uint64(k1)) & _MASK, lo0
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def philox4x32_10(c0, c1, c2, c3, k0: int, k1: int):
    return philox4x32(c0, c1, c2, c3, k0, k1, 10)


def _philox_words(n_blocks: int, seed: int, offset: int) -> np.ndarray:
    """[n_blocks, 4] output words of the blocks with counter (g_lo, g_hi, offset_lo, offset_hi), key = seed."""
    g = np.arange(n_blocks, dtype=np.uint64)
    w = philox4x32(g & _MASK, g >> np.uint64(32), np.uint64(offset & 0xFFFFFFFF), np.uint64((offset >> 32) & 0xFFFFFFFF),
                   seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    return np.stack(w, axis=1).astype(np.uint64)


def philox_bytes(seed: int, offset: int, shape) -> np.ndarray:
    """The stochastic-rounding numbers of every element 0..N-1 of a tensor in row-major order, as a
    ``PhiloxBytes`` array: R8 | R4 << 8 per element.
    R8 (codes wider than 4 bits): elements 16g..16g+15 share Philox block g; element 16g + j takes
    byte j % 4 (little-endian) of output word j // 4.
    R4 (codes of up to 4 bits): elements 32g..32g+31 share block g; with j = e % 32, run h = j // 16
    and i = j % 16, element e takes nibble i // 8 of byte i % 4 of word 2h + (i % 8) // 4 -- so one
    word serves elements i..i+3 with its low nibbles and i+8..i+11 with its high ones."""
    n = int(np.prod(shape))
    e = np.arange(n, dtype=np.int64)
    w8 = _philox_words((n + 15) // 16, seed, offset)
    j = e & 15
    r8 = (w8[e >> 4, j >> 2] >> (8 * (j & 3)).astype(np.uint64)) & np.uint64(0xFF)
    w4 = w8[:(n + 31) // 32]
    i = e & 15
    word = 2 * ((e >> 4) & 1) + ((i & 7) >> 2)
    r4 = (w4[e >> 5, word] >> (8 * (i & 3) + 4 * (i >> 3)).astype(np.uint64)) & np.uint64(0xF)
    return (r8 | (r4 << np.uint64(8))).astype(np.uint16).reshape(shape).view(PhiloxBytes)


# ----------------------------------------------------------------------------
# int4 packing (cuda_measure/HLQ_backward_kernel.cu:140: low nibble = even element)
# ----------------------------------------------------------------------------
def pack_int4(codes: np.ndarray) -> np.ndarray:
    """The kernels' packed INT4 layout: the last dim is cut into runs of 16 codes (zero-padded), and
    byte j (0..7) of a run holds code j in its low nibble and code j + 8 in its high nibble, so that
    both halves of a run expand to consecutive int8 codes with one shift / mask each."""
    c = np.asarray(codes).astype(np.int32)
    n = c.shape[-1]
    pad = (-n) % 16
    if pad:
        c = np.concatenate([c, np.zeros(c.shape[:-1] + (pad,), np.int32)], axis=-1)
    g = c.reshape(c.shape[:-1] + (-1, 2, 8)) & 0xF                     # [..., run, half, 8]
    return (g[..., 0, :] | (g[..., 1, :] << 4)).astype(np.uint8).reshape(c.shape[:-1] + (-1,))


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    """Inverse of ``pack_int4`` (the byte count of the last dim must be a multiple of 8): two codes
    per byte, sign-extended; callers slice off the zero padding of the last run."""
    p = np.asarray(packed).astype(np.int32)
    if p.shape[-1] % 8:
        p = np.concatenate([p, np.zeros(p.shape[:-1] + ((-p.shape[-1]) % 8,), np.int32)], axis=-1)
    g = p.reshape(p.shape[:-1] + (-1, 8))
    lo = ((g & 0xF) ^ 8) - 8
    hi = (((g >> 4) & 0xF) ^ 8) - 8
    return np.concatenate([lo, hi], axis=-1).reshape(p.shape[:-1] + (-1,))


# ----------------------------------------------------------------------------
# FLinearQ forward context + backward, scheme gih_gwlr (utils/quant_matmul.py:177-348)
# ----------------------------------------------------------------------------
def abc_compress(x: np.ndarray, n_l: int, sel: np.ndarray, bits: int, u, mode: str = "stoch"):
    """setup_context (:177-212): HLA of x along tokens then quantisation to int8.
    mode: 'stoch' (u required), 'int', 'sawb'."""
    x_lr = hla(x, n_l, sel)
    if mode == "sawb":
        return quant_sawb(x_lr, bits)
    return quant_tensor(x_lr, bits, u if mode == "stoch" else None)


def _int_matmul(a: np.ndarray, b: np.ndarray, exact: bool) -> np.ndarray:
    """a @ b on integer codes.  exact: int64 (slow, no BLAS).  Otherwise float32 BLAS, which is
    what the reference runs (utils/quant_matmul.py:288,322) and is exact while |acc| < 2^24."""
    if exact:
        return a.astype(np.int64) @ b.astype(np.int64)
    return a.astype(F32) @ b.astype(F32)


def linear_backward(go, w, x_q, s_x, *, n_o: int, n_l: int, sel, bits_gx: int = 4, bits_w: int = 4,
                    bits_gw: int = 8, u_go=None, u_w=None, u_gw=None, gx_per_token: bool = False,
                    gw_per_channel: bool = False, w_mode: str = "stoch", exact_matmul: bool = True):
    """FLinearQ.backward (:214-348) for 2-D tensors.  ``u_*`` None selects nearest
    rounding for that operand.  Returns a dict with every intermediate the CUDA
    path can be compared on."""
    go = np.asarray(go, dtype=F32)
    w = np.asarray(w, dtype=F32)
    out = {}
    # g_x: Hadamard along O, INT4 x INT4 (:237-290)
    go_h = fwht_last(go, n_o)
    if gx_per_token:
        q_go, s_go = quant_rows(go_h, bits_gx, u_go)
    else:
        q_go, s_go = quant_tensor(go_h, bits_gx, u_go)
    w_h = fwht_first(w, n_o)
    if w_mode == "sawb":
        q_w, s_w = quant_sawb(w_h, bits_w)
    else:
        q_w, s_w = quant_tensor(w_h, bits_w, u_w if w_mode == "stoch" else None)
    acc_x = _int_matmul(q_go, q_w, exact_matmul)
    if gx_per_token:
        gx = (acc_x.astype(F32) * s_go[:, None]) * F32(s_w)
    else:
        gx = (acc_x.astype(F32) * F32(s_go)) * F32(s_w)
    gx = gx / F32(n_o)                                               # :342
    # g_w: low-rank along L, INT8 x INT8 (:300-324)
    go_lr_t = np.ascontiguousarray(hla(go, n_l, sel).T)              # [O, L']
    if gw_per_channel:
        q_gw, s_gw = quant_rows(go_lr_t, bits_gw, u_gw)
    else:
        q_gw, s_gw = quant_tensor(go_lr_t, bits_gw, u_gw)
    acc_w = _int_matmul(q_gw, np.asarray(x_q), exact_matmul)
    if gw_per_channel:
        gw = (acc_w.astype(F32) * s_gw[:, None]) * F32(s_x)
    else:
        gw = (acc_w.astype(F32) * F32(s_gw)) * F32(s_x)
    gw = gw / F32(n_l)                                               # :344
    out.update(q_go=q_go, s_go=s_go, q_w=q_w, s_w=s_w, acc_x=acc_x, grad_input=gx.astype(F32),
               q_gw=q_gw, s_gw=s_gw, acc_w=acc_w, grad_w=gw.astype(F32))
    return out


def hla_expand(y: np.ndarray, n: int, sel: np.ndarray, scale) -> np.ndarray:
    """lowering_matmul_back(P.mT, y) * scale for P = H_n[sel] (utils/quant_matmul.py:334,337): the kept
    rows go back to their places in a zero block and the butterfly (H_n is symmetric) runs over it."""
    y = np.asarray(y, dtype=F32)
    r = len(sel)
    nb = y.shape[0] // r
    full = np.zeros((nb, n, y.shape[1]), dtype=F32)
    full[:, np.asarray(sel), :] = y.reshape(nb, r, y.shape[1])
    return (fwht_first(full.reshape(nb * n, y.shape[1]), n) * F32(scale)).astype(F32)


def grad_input_lowrank(go, w, *, n: int, sel, bits_gx: int = 4, bits_w: int = 4, u_go=None, u_w=None,
                       gx_per_token: bool = False, w_mode: str = "stoch", exact_matmul: bool = True):
    """grad_input of transform_scheme low_rank / gilr_gwh (utils/quant_matmul.py:229-234, 261-266, 288-290,
    334-337): grad_output is projected along the tokens and quantised as [L', O], the weight is
    quantised untransformed, and the [L', I] product is expanded back to L tokens and divided by n."""
    go_lr = hla(np.asarray(go, dtype=F32), n, np.asarray(sel))
    q_go, s_go = (quant_rows if gx_per_token else quant_tensor)(go_lr, bits_gx, u_go)
    w = np.asarray(w, dtype=F32)
    q_w, s_w = quant_sawb(w, bits_w) if w_mode == "sawb" else quant_tensor(w, bits_w, u_w if w_mode == "stoch" else None)
    acc = _int_matmul(q_go, q_w, exact_matmul)
    gi_lr = (acc.astype(F32) * (s_go[:, None] if gx_per_token else F32(s_go))) * F32(s_w)
    return dict(q_go=q_go, s_go=s_go, q_w=q_w, s_w=s_w, grad_input=hla_expand(gi_lr, n, sel, F32(1.0) / F32(n)))


def grad_input_gilro(go, w, *, n: int, sel, bits_gx: int = 4, bits_w: int = 4, u_go=None, u_w=None,
                     w_mode: str = "stoch", exact_matmul: bool = True):
    """grad_input of transform_scheme gilro_gwh (utils/quant_matmul.py:235-236, 267-268, 288-290, 339-340):
    grad_output [L, O] and the weight [O, I] are projected along the output features onto the kept rows P of
    H_n (n = the whole 2-adic part of O): go_lr = go . P^T blockwise [L, O r/n], w_lr = P w blockwise
    [O r/n, I]; both quantised with one scale; grad_input = (q_go @ q_w) * s_go * s_w / n."""
    go = np.asarray(go, dtype=F32)
    w = np.asarray(w, dtype=F32)
    sel = np.asarray(sel)
    go_lr = np.ascontiguousarray(hla(np.ascontiguousarray(go.T), n, sel).T)
    w_lr = hla(w, n, sel)
    q_go, s_go = quant_tensor(go_lr, bits_gx, u_go)
    q_w, s_w = quant_sawb(w_lr, bits_w) if w_mode == "sawb" else quant_tensor(w_lr, bits_w, u_w if w_mode == "stoch" else None)
    acc = _int_matmul(q_go, q_w, exact_matmul)
    gi = ((acc.astype(F32) * F32(s_go)) * F32(s_w)) / F32(n)
    return dict(q_go=q_go, s_go=s_go, q_w=q_w, s_w=s_w, grad_input=gi.astype(F32))


# ----------------------------------------------------------------------------
# the same on 3-D tensors [B, L, .]: one scale per sample (torch.vmap over dim 0 of the
# quantisers, utils/quant_matmul.py:102-106,117-122), grad_w summed over the batch
# ----------------------------------------------------------------------------
def _sample(u, b):
    """Noise of sample b: a slice of a [B, ...] array (keeping the PhiloxBytes marker), or None."""
    if u is None:
        return None
    return u[b].view(type(u)) if isinstance(u, PhiloxBytes) else np.asarray(u)[b]


def abc_compress_batched(x: np.ndarray, n_l: int, sel: np.ndarray, bits: int, u, mode: str = "stoch"):
    """setup_context (:177-212) on x [B, L, I]: HLA along the tokens of each sample, one scale per
    sample.  Returns (codes int32 [B, L', I], s float32 [B])."""
    outs = [abc_compress(x[b], n_l, sel, bits, _sample(u, b), mode) for b in range(x.shape[0])]
    return np.stack([o[0] for o in outs]), np.array([o[1] for o in outs], dtype=F32)


def grad_input_lowrank_batched(go, w, *, n: int, sel, bits_gx: int = 4, bits_w: int = 4, u_go=None, u_w=None,
                               gx_per_token: bool = False, w_mode: str = "stoch", exact_matmul: bool = True):
    """grad_input_lowrank on go [B, L, O]: projection, quantiser (one scale per sample) and expansion
    run per sample; the weight is 2-D and is quantised once.  Returns grad_input [B, L, I]."""
    go = np.asarray(go, dtype=F32)
    outs = [grad_input_lowrank(go[b], w, n=n, sel=sel, bits_gx=bits_gx, bits_w=bits_w, u_go=_sample(u_go, b), u_w=u_w,
                               gx_per_token=gx_per_token, w_mode=w_mode, exact_matmul=exact_matmul)["grad_input"]
            for b in range(go.shape[0])]
    return np.stack(outs).astype(F32)


def linear_backward_batched(go, w, x_q, s_x, *, n_o: int, n_l: int, sel, bits_gx: int = 4, bits_w: int = 4,
                            bits_gw: int = 8, u_go=None, u_w=None, u_gw=None, w_mode: str = "stoch",
                            gx_per_token: bool = False, gw_per_channel: bool = False, exact_matmul: bool = True):
    """FLinearQ.backward (:214-348) for go [B, L, O], x_q [B, L', I], s_x [B].  Every quantiser of a
    batched tensor takes one scale per sample; the weight is 2-D and keeps one scale.  grad_input[b] =
    (q_go[b] @ q_w) * s_go[b] * s_w / n_o (:288-290, 342).  grad_w = sum_b (q_gw[b] @ x_q[b]) * s_gw[b]
    * s_x[b] / n_l (:322-324, 344; the sum over b is the reduction autograd applies to the
    [B, O, I] result); here it runs in float32 from sample 0 upwards, with the exact division by the
    power of two n_l after it.  gx_per_token / gw_per_channel: the vmapped norm_quantizer (:19-37) on
    that side, i.e. one scale per row of each sample's [L, O] / [O, L'] operand, applied to the
    integer product (the reference multiplies the scales in before its float matmul)."""
    go = np.asarray(go, dtype=F32)
    w = np.asarray(w, dtype=F32)
    B = go.shape[0]
    w_h = fwht_first(w, n_o)
    if w_mode == "sawb":
        q_w, s_w = quant_sawb(w_h, bits_w)
    else:
        q_w, s_w = quant_tensor(w_h, bits_w, u_w if w_mode == "stoch" else None)
    q_go, s_go, gx, q_gw, s_gw = [], [], [], [], []
    run = None
    for b in range(B):
        qg, sg = (quant_rows if gx_per_token else quant_tensor)(fwht_last(go[b], n_o), bits_gx, _sample(u_go, b))
        acc = _int_matmul(qg, q_w, exact_matmul)
        sg_b = sg[:, None] if gx_per_token else F32(sg)
        gx.append(((acc.astype(F32) * sg_b) * F32(s_w)) / F32(n_o))
        q_go.append(qg)
        s_go.append(sg)
        qw_, sw_ = (quant_rows if gw_per_channel else quant_tensor)(np.ascontiguousarray(hla(go[b], n_l, sel).T), bits_gw,
                                                                    _sample(u_gw, b))
        sw_b = sw_[:, None] if gw_per_channel else F32(sw_)
        v = ((_int_matmul(qw_, np.asarray(x_q[b]), exact_matmul).astype(F32) * sw_b) * F32(s_x[b])).astype(F32)
        run = v if run is None else (run + v).astype(F32)
        q_gw.append(qw_)
        s_gw.append(sw_)
    return dict(q_go=np.stack(q_go), s_go=np.array(s_go, dtype=F32), q_w=q_w, s_w=s_w,
                grad_input=np.stack(gx).astype(F32), q_gw=np.stack(q_gw), s_gw=np.array(s_gw, dtype=F32),
                grad_w=(run / F32(n_l)).astype(F32))


# ----------------------------------------------------------------------------
# layer-wise quantiser selection (ViT_main.py:183-211)
# ----------------------------------------------------------------------------
def lqs_select(grad_out: np.ndarray, u_stoch: np.ndarray, u_norm: np.ndarray, bits: int = 4):
    """Per-layer choice between per-tensor ('stoch_quantizer') and per-token
    ('norm_quantizer') quantisation of grad_out: the per-token quantiser is taken for
    g_x only when it cuts the per-tensor L2 error by more than half; g_w always keeps
    'stoch_quantizer'.  A 3-D grad_out [B, L, O] is quantised "batched", as the
    calibration loop does (ViT_main.py:190-201): the per-tensor quantiser takes one scale
    per sample and the error is the distance to q * s[:, None, None]; the per-token
    quantiser's rows are the tokens of every sample either way.  Returns (gx_name,
    gw_name, err_stoch, err_norm)."""
    g = np.asarray(grad_out, dtype=F32)
    if g.ndim == 3:
        deq = np.stack([(lambda q, s: q.astype(F32) * s)(*quant_tensor(g[b], bits, _sample(u_stoch, b)))
                        for b in range(g.shape[0])])
    else:
        q, s = quant_tensor(g, bits, u_stoch)
        deq = q.astype(F32) * s
    e_st = float(np.sqrt(np.sum((g.astype(np.float64) - deq.astype(np.float64)) ** 2)))
    g2 = g.reshape(-1, g.shape[-1])
    qn, sn = quant_rows(g2, bits, None if u_norm is None else np.asarray(u_norm).reshape(g2.shape))
    e_nq = float(np.sqrt(np.sum((g2.astype(np.float64) - (qn.astype(F32) * sn[:, None]).astype(np.float64)) ** 2)))
    gx = "stoch_quantizer"
    if e_nq < e_st and (e_st - e_nq) > e_st * 0.5:
        gx = "norm_quantizer"
    return gx, "stoch_quantizer", e_st, e_nq
