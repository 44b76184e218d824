"""Host-side transform generators and the transform cache, mirroring the public names of the
reference's ``utils/hadamard_matmul.py``.  The matrices are tiny +-1 integer tables built with
numpy on the host; the heavy lifting (applying them to activations and gradients) happens in
the CUDA kernels, which take the block order and the kept row indices rather than a matrix.
"""
from __future__ import annotations

import math
from collections import defaultdict

import numpy as np
import torch


def biggest_power2_factor(size_m: int) -> int:
    """Largest power of two dividing ``size_m`` (utils/hadamard_matmul.py:9-15)."""
    if size_m < 1:
        raise ValueError("size must be positive")
    return size_m & -size_m


def biggest_power2_factor_max16(size_m: int) -> int:
    """Same, capped at 16: the Hadamard block order (utils/hadamard_matmul.py:17-27)."""
    p = biggest_power2_factor(size_m)
    return 16 if (p > 16 and size_m > 16) else p


def hadamard(n: int) -> np.ndarray:
    """Sylvester Hadamard matrix of order n, natural order, +-1, unnormalised
    (utils/hadamard_matmul.py:32-51)."""
    if n < 1 or (n & (n - 1)):
        raise ValueError("n must be int and power of 2.")
    idx = np.arange(n)
    parity = np.zeros((n, n), dtype=np.int64)
    both = idx[:, None] & idx[None, :]
    while both.any():
        parity ^= both & 1
        both = both >> 1
    return 1 - 2 * parity


def make_hadamard(size_m: int) -> np.ndarray:
    """utils/hadamard_matmul.py:57-59."""
    return hadamard(biggest_power2_factor_max16(size_m))


def make_non_block_hadamard(size_m: int) -> np.ndarray:
    """utils/hadamard_matmul.py:167-170."""
    return hadamard(1 if size_m == 1 else biggest_power2_factor(size_m))


def _sequency_rank(n: int) -> np.ndarray:
    """Natural-order row index of H_n for sequency 0, 1, ..., n-1."""
    h = hadamard(n)
    changes = (h[:, 1:] != h[:, :-1]).sum(axis=1)
    return np.argsort(changes, kind="stable")


def wht_selection(size_m: int, percentile: float = 50):
    """(n, kept natural-order row indices) of ``make_WHT(size_m, percentile)``
    (utils/hadamard_matmul.py:209-226)."""
    n = 1 if size_m == 1 else biggest_power2_factor(size_m)
    by_seq = _sequency_rank(n)
    q2 = 1
    while q2 * 4 <= n:
        q2 *= 4
    q = math.isqrt(q2)
    sf = int(0.1 * (-np.sqrt(2 * q ** 2 * percentile + 25) + 10 * q + 5))
    keep: list = []
    for i in range(q):
        lo, hi = (q * i, q * (i + 1) - (i + sf)) if i % 2 == 0 else (q * i + (i + sf), q * (i + 1))
        keep.extend(range(lo, max(lo, hi)))
    return n, [int(by_seq[k]) for k in keep]


def make_WHT(size_m: int, percentile: float = 50) -> np.ndarray:
    """Low-rank Walsh-Hadamard basis [r, n] (utils/hadamard_matmul.py:209-226)."""
    n, sel = wht_selection(size_m, percentile)
    return hadamard(n)[sel]


def lowrank_selection(tokens: int, preset, percentile: float = 50):
    """(n, sel) for a token count.  preset None: what the reference's make_WHT gives;
    "half16": 8 lowest-sequency rows of H_16; "half": n = min(16, 2-adic part of tokens),
    the n/2 lowest-sequency rows (n = 1 keeps the single row)."""
    if preset is None:
        return wht_selection(tokens, percentile)
    if preset == "half16":
        if tokens % 16:
            raise ValueError("lowRankPreset 'half16' needs a token count divisible by 16 (got %d)" % tokens)
        return 16, [int(v) for v in _sequency_rank(16)[:8]]
    if preset == "half":
        n = biggest_power2_factor_max16(tokens)
        return n, [int(v) for v in _sequency_rank(n)[:max(1, n // 2)]]
    raise ValueError("unknown low-rank preset %r" % (preset,))


def selection_from_matrix(p) -> tuple:
    """(n, sel) from an [r, n] matrix whose rows are rows of H_n (what ``make_WHT`` returns and
    what ``HQ_Linear.hadamard_bs`` holds).  Raises ValueError for anything else."""
    p = np.asarray(p.detach().cpu().float().numpy() if isinstance(p, torch.Tensor) else p)
    if p.ndim != 2 or p.shape[1] < 1 or (p.shape[1] & (p.shape[1] - 1)):
        raise ValueError("expected an [r, n] matrix with n a power of two, got %s" % (p.shape,))
    r, n = p.shape
    signs = np.rint(p).astype(np.int64)
    # row i of the Sylvester matrix is t -> (-1)^popcount(i & t): bit k of i is the sign at t = 2^k
    sel = []
    t = np.arange(n)
    for j in range(r):
        i = 0
        k = 1
        while k < n:
            if signs[j, k] < 0:
                i |= k
            k <<= 1
        par = np.zeros(n, dtype=np.int64)
        both = i & t
        while both.any():
            par ^= both & 1
            both = both >> 1
        if not np.array_equal(signs[j], 1 - 2 * par):
            raise ValueError("row %d is not a row of the order-%d Hadamard matrix" % (j, n))
        sel.append(int(i))
    return n, sel


def lowering_matmul_front(A: torch.Tensor, H: torch.Tensor) -> torch.Tensor:
    """Block transform of the last dim, un-quantised (utils/hadamard_matmul.py:121-141).
    Kept for callers that want the plain float transform; the backward path does not use it."""
    n = H.shape[0]
    if A.dim() not in (2, 3):
        raise NotImplementedError
    if A.shape[-1] == n:
        return A @ H
    return (A.reshape(*A.shape[:-2], -1, n) @ H).reshape(*A.shape[:-1], -1)


def lowering_matmul_back(H: torch.Tensor, A: torch.Tensor) -> torch.Tensor:
    """Block transform of the token dim, un-quantised (utils/hadamard_matmul.py:143-161)."""
    n = H.shape[1]
    if A.dim() == 2:
        if A.shape[0] == n:
            return H @ A
        return (A.T.reshape(-1, n) @ H.T).reshape(A.shape[1], -1).T
    if A.dim() == 3:
        if A.shape[1] == n:
            return H.unsqueeze(0) @ A
        return (A.mT.reshape(A.shape[0], -1, n) @ H.mT).reshape(A.shape[0], A.shape[2], -1).mT
    raise NotImplementedError


class Transform_Dict:
    """Cache of generated matrices keyed by name + size (utils/hadamard_matmul.py:228-254)."""

    def __init__(self):
        self.transform_dict = defaultdict(np.array)

    def get(self, name, size):
        return self.transform_dict[name + str(size)]

    def register(self, name, size, vectorPercentile):
        if name == "hadamard":
            self.transform_dict[name + str(size)] = make_hadamard(size)
        elif name == "low_rank":
            self.transform_dict[name + str(size)] = make_WHT(size, vectorPercentile)
        else:
            raise NotImplementedError

    def get_or_register(self, name, size, vectorPercentile=50):
        if name + str(size) not in self.transform_dict:
            self.register(name, size, vectorPercentile)
        return self.get(name, size)
