"""The scratch-free entry point ``hot_col_ht_quant_static`` against ``hot_col_ht_quant``.

Some hosts of this library may not allocate device memory around the call (they work from a
fixed set of registered buffers, or sit in a region where an allocation would stall the
device), so they have no scratch buffer to pass.  For them the library keeps the abs-max words
in an array of its own.  That array is shared by every call and keeps what the last call
wrote, so the check here is two calls in a row whose abs-max values DEcrease: if the second
call saw anything left over from the first, its scales and codes would come out wrong.

Collected last on purpose (file name), so a failure here cannot hide the other tests' results.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from hot_b200 import ops as _ops
    return _ops


def _pair(ops, x, order, sel, q, layout):
    ref_codes, ref_scales, ref_len = ops.col_ht_quant(x, order, sel, q, layout)
    got_codes, got_scales, got_len = ops.col_ht_quant_static(x, order, sel, q, layout)
    torch.cuda.synchronize()
    assert got_len == ref_len
    nbytes = (ref_len + 1) // 2 if q.storage == "int4" else ref_len
    # bit-exact: same kernels, same arithmetic, only the scratch lives elsewhere
    assert torch.equal(got_scales.view(torch.int32), ref_scales.view(torch.int32))
    assert torch.equal(got_codes[:, :nbytes], ref_codes[:, :nbytes])
    return got_scales


@pytest.mark.parametrize("scale", ["tensor", "row"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_caller_scratch_twice_in_a_row(ops, scale, dtype):
    torch.manual_seed(7)
    sel = [0, 8, 12, 4, 6, 14, 10, 2]                      # 8 lowest-sequency rows of H_16
    q8 = ops.Quant(8, "int8", "philox", scale, 5, 1)
    q4 = ops.Quant(4, "int4", "nearest", scale, 5, 2)
    big = (torch.randn(16 * 24, 200, device="cuda") * 50.0).to(dtype)
    small = (torch.randn(16 * 24, 200, device="cuda") * 1e-3).to(dtype)
    s_big = _pair(ops, big, 16, sel, q8, "transposed")
    s_small = _pair(ops, small, 16, sel, q8, "transposed")  # stale maxima from `big` would inflate these
    assert float(s_small.max()) < float(s_big.min())
    _pair(ops, small, 16, list(range(16)), q4, "natural")   # and a different mode / width right after
    _pair(ops, big[:, :64].contiguous(), 16, sel, q8, "natural")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_sawb_mode_twice_in_a_row(ops, dtype):
    """The two-moment clip keeps four words per CTA in the array and clears nothing: every word the
    second kernel reads was written by the first kernel of the same call, so a call after a larger
    one (more CTAs, larger sums) must still agree with the caller-scratch variant bit for bit."""
    torch.manual_seed(9)
    q = ops.Quant(8, "int8", "nearest", "sawb")
    big = (torch.randn(16 * 40, 768, device="cuda") * 30.0).to(dtype)
    small = (torch.randn(16 * 6, 96, device="cuda") * 1e-2).to(dtype)
    sel = [0, 8, 12, 4, 6, 14, 10, 2]
    s_big = _pair(ops, big, 16, sel, q, "natural")
    s_small = _pair(ops, small, 16, sel, q, "natural")
    assert float(s_small[0]) < float(s_big[0])
    _pair(ops, small, 1, [0], ops.Quant(4, "int8", "nearest", "sawb"), "natural")   # the weight's form: no transform


def test_static_scratch_rejects_what_does_not_fit(ops):
    x = torch.zeros((16, 16400), device="cuda")             # one scratch word per column needed: 16400 > 16384
    sel = list(range(16))
    with pytest.raises(RuntimeError, match="built-in scratch holds 16384"):
        ops.col_ht_quant_static(x, 16, sel, ops.Quant(8, "int8", "nearest", "row"))
    big = torch.zeros((50432, 3072), device="cuda", dtype=torch.bfloat16)   # the clip needs four words per CTA: 18916 here
    with pytest.raises(RuntimeError, match="built-in scratch holds 16384"):
        ops.col_ht_quant_static(big, 16, [0, 8, 12, 4, 6, 14, 10, 2], ops.Quant(8, "int8", "nearest", "sawb"))
    del big
    codes, scales, n = ops.col_ht_quant_static(x, 16, sel, ops.Quant(8, "int8", "nearest", "tensor"))
    torch.cuda.synchronize()
    assert n == 16 and float(scales[0]) == 0.0 and int(codes[:, :16].max()) == 0
