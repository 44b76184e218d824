"""GPU parity tests of the per-sample (3-D) path: batched quantisation with one scale per sample,
the grouped integer GEMM that sums dequantised per-sample products, and the layer backward built
from them, against the CPU oracle and against the reference-generated fixture
``tests/golden/flinearq_batched.npz``.  Codes, scales and gradients are compared bit for bit.
"""
import os

import numpy as np
import pytest
import torch

from oracle import hot_oracle as oc

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from hot_b200 import ops as _ops
    return _ops


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def _as_f32(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).to(torch.float32).numpy()


def _bits(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32)).view(np.uint32)


def _codes(codes_t, storage, n):
    c = codes_t.cpu().numpy()
    if storage == "int4":
        return oc.unpack_int4(c)[..., :n]
    return c.view(np.int8).astype(np.int32)[..., :n]


def _noise(rounding, shape, rng, seed, offset):
    if rounding == "noise":
        return rng.random(shape, dtype=np.float32)
    if rounding == "philox":
        return oc.philox_bytes(seed, offset, shape)
    return None


def _slice(u, b):
    if u is None:
        return None
    return u[b].view(type(u)) if isinstance(u, oc.PhiloxBytes) else u[b]


@pytest.mark.parametrize("B,rows,cols,order", [(3, 24, 96, 16), (5, 197, 768, 16), (2, 7, 64, 1), (64, 197, 256, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("storage,bits", [("int4", 4), ("int8", 8)])
@pytest.mark.parametrize("rounding", ["nearest", "noise", "philox"])
def test_row_ht_quant_batched(ops, B, rows, cols, order, dtype, storage, bits, rounding):
    rng = np.random.default_rng(B * 7 + rows + cols)
    x = (rng.standard_normal((B, rows, cols)) * 1e-3).astype(np.float32)
    x *= (1.0 + 3.0 * rng.random((B, 1, 1))).astype(np.float32)          # a different range per sample
    seed, offset = 0xBEEF, 5
    u = _noise(rounding, (B, rows, cols), rng, seed, offset)
    q = ops.Quant(bits, storage, rounding, "tensor", seed, offset, _dev(u) if rounding == "noise" else None)
    codes, scales = ops.row_ht_quant_batched(_dev(x, dtype), order, q)
    torch.cuda.synchronize()
    got_c = _codes(codes, storage, cols).reshape(B, rows, cols)
    got_s = scales.cpu().numpy()
    xf = _as_f32(x, dtype)
    for b in range(B):
        ref_c, ref_s = oc.quant_tensor(oc.fwht_last(xf[b], order), bits, _slice(u, b))
        assert _bits(ref_s) == _bits(got_s[b]), b
        assert np.array_equal(got_c[b], ref_c), (b, int((got_c[b] != ref_c).sum()))


@pytest.mark.parametrize("B,rows,cols,order,sel", [
    (3, 24, 96, 8, list(oc.wht_selection(24, 50)[1])),
    (4, 197, 200, 1, [0]),                                            # odd token count: no transform
    (2, 196, 64, 4, list(oc.wht_selection(196, 50)[1])),
    (64, 32, 128, 16, list(oc.lowrank_preset(16, 8))),
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rounding,layout", [("nearest", "natural"), ("noise", "natural"), ("noise", "transposed"),
                                             ("philox", "transposed")])
def test_col_ht_quant_batched(ops, B, rows, cols, order, sel, dtype, rounding, layout):
    r = len(sel)
    out_len = rows // order * r
    rng = np.random.default_rng(B + rows * 3 + cols)
    x = rng.standard_normal((B, rows, cols)).astype(np.float32)
    x *= (1.0 + 5.0 * rng.random((B, 1, 1))).astype(np.float32)
    seed, offset = 31, 9
    if rounding == "noise":
        u_t = rng.random((B, cols, out_len), dtype=np.float32)        # as seen in the stored layout
        u_dev = _dev(u_t if layout == "transposed" else np.ascontiguousarray(u_t.transpose(0, 2, 1)))
    elif rounding == "philox":                                        # indexed by the position in the padded output
        pitch_ = ops.sample_pitch(out_len)
        u_t = np.ascontiguousarray(oc.philox_bytes(seed, offset, (cols, B, pitch_))[:, :, :out_len].transpose(1, 0, 2))
        u_t, u_dev = u_t.view(oc.PhiloxBytes), None
    else:
        u_t, u_dev = None, None
    q = ops.Quant(8, "int8", rounding, "tensor", seed, offset, u_dev)
    codes, scales, got_len, pitch = ops.col_ht_quant_batched(_dev(x, dtype), order, sel, q, layout)
    torch.cuda.synchronize()
    assert got_len == out_len and pitch % 128 == 0 and pitch >= out_len
    c = codes.cpu().numpy().view(np.int8).astype(np.int32).reshape(cols, B, pitch)
    got_s = scales.cpu().numpy()
    xf = _as_f32(x, dtype)
    for b in range(B):
        y_t = np.ascontiguousarray(oc.hla(xf[b], order, np.array(sel)).T)          # [cols, out_len]
        ref_c, ref_s = oc.quant_tensor(y_t, 8, _slice(u_t, b))
        assert _bits(ref_s) == _bits(got_s[b]), b
        assert np.array_equal(c[:, b, :out_len], ref_c), (b, int((c[:, b, :out_len] != ref_c).sum()))
        assert not c[:, b, out_len:].any(), "padding between samples must be zero"


@pytest.mark.parametrize("M,N,groups,glen", [(96, 48, 3, 9), (300, 130, 5, 197), (3072, 768, 64, 197), (128, 128, 1, 128),
                                             (257, 96, 7, 300)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("per_row", [False, True])
def test_gemm_i8_grouped(ops, M, N, groups, glen, out_dtype, per_row):
    rng = np.random.default_rng(M + N + groups)
    pitch = ops.sample_pitch(glen)
    a = np.zeros((M, groups, pitch), dtype=np.int8)
    b = np.zeros((N, groups, pitch), dtype=np.int8)
    a[:, :, :glen] = rng.integers(-127, 128, size=(M, groups, glen))
    b[:, :, :glen] = rng.integers(-127, 128, size=(N, groups, glen))
    sa = (rng.random((groups, M) if per_row else groups) * 1e-3 + 1e-4).astype(np.float32)   # [groups, M]: one per row too
    sb = (rng.random(groups) * 1e-2 + 1e-3).astype(np.float32)
    post = 0.125
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.gemm_i8_grouped(_dev(a.reshape(M, -1)).view(torch.uint8), _dev(b.reshape(N, -1)).view(torch.uint8), M, N,
                              groups, pitch, _dev(sa), _dev(sb), post, out_dtype, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    run = None
    for g in range(groups):
        acc = a[:, g].astype(np.int64) @ b[:, g].astype(np.int64).T
        v = ((acc.astype(np.float32) * (sa[g][:, None] if per_row else sa[g])) * sb[g]).astype(np.float32)
        run = v if run is None else (run + v).astype(np.float32)
    ref = torch.from_numpy((run * np.float32(post)).astype(np.float32)).to(out_dtype)
    assert torch.equal(out.cpu(), ref)


def test_gemm_rows_per_scale(ops):
    rng = np.random.default_rng(4)
    B, L, N, K = 5, 37, 80, 256
    M = B * L
    a = rng.integers(-7, 8, size=(M, K)).astype(np.int8)
    b = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    sa = (rng.random(B) + 0.5).astype(np.float32)
    sb = np.array([0.37], dtype=np.float32)
    out = ops.gemm_i8(_dev(a).view(torch.uint8), "int8", _dev(b).view(torch.uint8), "int8", M, N, K, _dev(sa), _dev(sb),
                      1.0 / 16, torch.float32, a_rows_per_scale=L)
    torch.cuda.synchronize()
    acc = (a.astype(np.int64) @ b.astype(np.int64).T).astype(np.float32)
    ref = ((acc * np.repeat(sa, L)[:, None]) * sb[0]) * np.float32(1.0 / 16)
    assert np.array_equal(_bits(out.cpu().numpy()), _bits(ref))


def _batched_layer(ops, go, w, x, n_o, n_l, sel, rounding, dtype, noise=None, seed=11):
    """Runs abc_compress_batched + linear_backward_batched; noise = dict of explicit uniforms."""
    def q(bits, storage, key, off):
        if rounding == "noise":
            return ops.Quant(bits, storage, "noise", "tensor", 0, 0, _dev(noise[key]))
        return ops.Quant(bits, storage, rounding, "tensor", seed, off)
    cfg = ops.LinearConfig(order_o=n_o, order_l=n_l, sel_l=list(sel), q_gx=q(4, "int4", "u_go", 2), q_w=q(4, "int4", "u_w", 3),
                           q_gw=q(8, "int8", "u_gw", 4), q_x=q(8, "int8", "u_x", 1))
    x_q_t, s_x, pitch = ops.abc_compress_batched(_dev(x, dtype), cfg)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gx, gw = ops.linear_backward_batched(_dev(go, dtype), _dev(w, dtype), x_q_t, s_x, cfg, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return x_q_t, s_x, pitch, gx, gw


def test_batched_backward_golden(ops):
    """The reference's own 3-D run (explicit noise): codes of the saved activation, its per-sample
    scales and both gradients."""
    g = np.load(os.path.join(GOLDEN, "flinearq_batched.npz"))
    n_l, sel = oc.selection_from_matrix(g["p"])
    B, L, O = g["go"].shape
    I = g["w"].shape[1]
    noise = {"u_x": g["u_x"], "u_go": g["u_go"], "u_w": g["u_w"], "u_gw": g["u_gw"]}
    x_q_t, s_x, pitch, gx, gw = _batched_layer(ops, g["go"], g["w"], g["x"], oc.block_order(O), n_l, sel, "noise",
                                               torch.float32, noise)
    out_len = L // n_l * len(sel)
    xq = x_q_t.cpu().numpy().view(np.int8).reshape(I, B, pitch)[:, :, :out_len].transpose(1, 2, 0)   # [B, L', I]
    assert np.array_equal(xq, g["x_q"])
    np.testing.assert_allclose(s_x.cpu().numpy(), g["scale_x"], rtol=1e-6)
    for got, name in ((gx, "grad_input"), (gw, "grad_w")):
        ref = g[name]
        rel = np.linalg.norm(got.cpu().numpy() - ref) / np.linalg.norm(ref)
        assert rel < 1e-3, (name, rel)
    # and bit for bit against the oracle on the same noise
    x_q, s_xo = oc.abc_compress_batched(g["x"], n_l, sel, 8, g["u_x"])
    ref = oc.linear_backward_batched(g["go"], g["w"], x_q, s_xo, n_o=oc.block_order(O), n_l=n_l, sel=sel, u_go=g["u_go"],
                                     u_w=g["u_w"], u_gw=g["u_gw"])
    assert np.array_equal(_bits(gx.cpu().numpy()), _bits(ref["grad_input"]))
    assert np.array_equal(_bits(gw.cpu().numpy()), _bits(ref["grad_w"]))


@pytest.mark.parametrize("B,rows,cols,order,sel", [
    (3, 24, 96, 8, list(oc.wht_selection(24, 50)[1])),
    (4, 197, 200, 1, [0]),
    (64, 32, 128, 16, list(oc.lowrank_preset(16, 8))),
    (5, 256, 768, 16, list(oc.lowrank_preset(16, 8))),                # several CTAs per sample
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_col_ht_quant_batched_sawb(ops, B, rows, cols, order, sel, dtype):
    """One SAWB clip per sample (the vmapped sawb_quantizer), nearest rounding."""
    r = len(sel)
    out_len = rows // order * r
    rng = np.random.default_rng(B * 7 + rows + cols)
    x = rng.standard_normal((B, rows, cols)).astype(np.float32)
    x *= (1.0 + 5.0 * rng.random((B, 1, 1))).astype(np.float32)
    q = ops.Quant(8, "int8", "nearest", "sawb")
    codes, scales, got_len, pitch = ops.col_ht_quant_batched(_dev(x, dtype), order, sel, q, "natural")
    torch.cuda.synchronize()
    c = codes.cpu().numpy().view(np.int8).astype(np.int32).reshape(cols, B, pitch)
    got_s = scales.cpu().numpy()
    xf = _as_f32(x, dtype)
    for b in range(B):
        y_t = np.ascontiguousarray(oc.hla(xf[b], order, np.array(sel)).T)
        ref_c, ref_s = oc.quant_sawb(y_t, 8)
        assert _bits(ref_s) == _bits(got_s[b]), (b, ref_s, got_s[b])
        assert np.array_equal(c[:, b, :out_len], ref_c), (b, int((c[:, b, :out_len] != ref_c).sum()))
        assert not c[:, b, out_len:].any()
    assert len(set(got_s.tolist())) == B


@pytest.mark.parametrize("B,rows,cols,order,sel", [
    (3, 24, 96, 8, list(oc.wht_selection(24, 50)[1])),
    (4, 197, 200, 1, [0]),
    (64, 32, 128, 16, list(oc.lowrank_preset(16, 8))),
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rounding", ["nearest", "noise", "philox"])
def test_col_ht_quant_batched_row_scales(ops, B, rows, cols, order, sel, dtype, rounding):
    """One scale per sample and output row (the vmapped norm_quantizer on [B, O, L'])."""
    r = len(sel)
    out_len = rows // order * r
    rng = np.random.default_rng(B * 11 + rows + cols)
    x = rng.standard_normal((B, rows, cols)).astype(np.float32)
    x *= (1.0 + 5.0 * rng.random((B, 1, cols))).astype(np.float32)
    seed, offset = 17, 5
    if rounding == "noise":
        u_t = rng.random((B, cols, out_len), dtype=np.float32)
        u_dev = _dev(u_t)
    elif rounding == "philox":
        pitch_ = ops.sample_pitch(out_len)
        u_t = np.ascontiguousarray(oc.philox_bytes(seed, offset, (cols, B, pitch_))[:, :, :out_len].transpose(1, 0, 2))
        u_t, u_dev = u_t.view(oc.PhiloxBytes), None
    else:
        u_t, u_dev = None, None
    q = ops.Quant(8, "int8", rounding, "row", seed, offset, u_dev)
    codes, scales, got_len, pitch = ops.col_ht_quant_batched(_dev(x, dtype), order, sel, q, "transposed")
    torch.cuda.synchronize()
    assert tuple(scales.shape) == (B, cols)
    c = codes.cpu().numpy().view(np.int8).astype(np.int32).reshape(cols, B, pitch)
    got_s = scales.cpu().numpy()
    xf = _as_f32(x, dtype)
    for b in range(B):
        y_t = np.ascontiguousarray(oc.hla(xf[b], order, np.array(sel)).T)
        ref_c, ref_s = oc.quant_rows(y_t, 8, _slice(u_t, b))
        assert np.array_equal(_bits(ref_s), _bits(got_s[b])), b
        assert np.array_equal(c[:, b, :out_len], ref_c), (b, int((c[:, b, :out_len] != ref_c).sum()))
        assert not c[:, b, out_len:].any()


def test_batched_backward_nq_golden(ops):
    """The reference's 3-D run with its default quantisers on all four operands (nq, sawb, nq, sawb):
    both gradients against its output, and bit for bit against the oracle on the same noise."""
    g = np.load(os.path.join(GOLDEN, "flinearq_batched_nq.npz"))
    n_l, sel = oc.selection_from_matrix(g["p"])
    B, L, O = g["go"].shape
    cfg = ops.LinearConfig(order_o=oc.block_order(O), order_l=n_l, sel_l=list(sel),
                           q_gx=ops.Quant(4, "int4", "noise", "row", 0, 0, _dev(g["u_go"])),
                           q_w=ops.Quant(4, "int4", "nearest", "sawb"),
                           q_gw=ops.Quant(8, "int8", "noise", "row", 0, 0, _dev(g["u_gw"])),
                           q_x=ops.Quant(8, "int8", "nearest", "sawb"))
    x_q_t, s_x, pitch = ops.abc_compress_batched(_dev(g["x"]), cfg)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gx, gw = ops.linear_backward_batched(_dev(g["go"]), _dev(g["w"]), x_q_t, s_x, cfg, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for got, name in ((gx, "grad_input"), (gw, "grad_w")):
        ref = g[name]
        rel = np.linalg.norm(got.cpu().numpy() - ref) / np.linalg.norm(ref)
        assert rel < 1e-3, (name, rel)
    x_q, s_xo = oc.abc_compress_batched(g["x"], n_l, sel, 8, None, "sawb")
    ref = oc.linear_backward_batched(g["go"], g["w"], x_q, s_xo, n_o=oc.block_order(O), n_l=n_l, sel=sel, u_go=g["u_go"],
                                     u_gw=g["u_gw"], w_mode="sawb", gx_per_token=True, gw_per_channel=True)
    assert np.array_equal(_bits(gx.cpu().numpy()), _bits(ref["grad_input"]))
    assert np.array_equal(_bits(gw.cpu().numpy()), _bits(ref["grad_w"]))


def test_batched_backward_sawb_golden(ops):
    """The reference's 3-D run with sawb on the weight and the activation buffer (its training
    defaults): saved codes, per-sample scales, both gradients; and bit for bit against the oracle."""
    g = np.load(os.path.join(GOLDEN, "flinearq_batched_sawb.npz"))
    n_l, sel = oc.selection_from_matrix(g["p"])
    B, L, O = g["go"].shape
    I = g["w"].shape[1]
    sawb = ops.Quant(8, "int8", "nearest", "sawb")
    cfg = ops.LinearConfig(order_o=oc.block_order(O), order_l=n_l, sel_l=list(sel),
                           q_gx=ops.Quant(4, "int4", "noise", "tensor", 0, 0, _dev(g["u_go"])),
                           q_w=ops.Quant(4, "int4", "nearest", "sawb"),
                           q_gw=ops.Quant(8, "int8", "noise", "tensor", 0, 0, _dev(g["u_gw"])), q_x=sawb)
    x_q_t, s_x, pitch = ops.abc_compress_batched(_dev(g["x"]), cfg)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gx, gw = ops.linear_backward_batched(_dev(g["go"]), _dev(g["w"]), x_q_t, s_x, cfg, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    out_len = L // n_l * len(sel)
    xq = x_q_t.cpu().numpy().view(np.int8).reshape(I, B, pitch)[:, :, :out_len].transpose(1, 2, 0)
    assert np.mean(xq != g["x_q"]) < 1e-3                              # float32 mean order differs in the reference
    np.testing.assert_allclose(s_x.cpu().numpy(), g["scale_x"], rtol=1e-5)
    for got, name in ((gx, "grad_input"), (gw, "grad_w")):
        ref = g[name]
        rel = np.linalg.norm(got.cpu().numpy() - ref) / np.linalg.norm(ref)
        assert rel < 1e-3, (name, rel)
    x_q, s_xo = oc.abc_compress_batched(g["x"], n_l, sel, 8, None, "sawb")
    assert np.array_equal(xq, x_q) and np.array_equal(_bits(s_x.cpu().numpy()), _bits(s_xo))
    ref = oc.linear_backward_batched(g["go"], g["w"], x_q, s_xo, n_o=oc.block_order(O), n_l=n_l, sel=sel, u_go=g["u_go"],
                                     u_gw=g["u_gw"], w_mode="sawb")
    assert np.array_equal(_bits(gx.cpu().numpy()), _bits(ref["grad_input"]))
    assert np.array_equal(_bits(gw.cpu().numpy()), _bits(ref["grad_w"]))


@pytest.mark.parametrize("B,L,O,I", [(4, 197, 768, 256), (6, 196, 256, 128), (8, 32, 128, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rounding", ["nearest", "philox"])
def test_batched_backward_vs_oracle(ops, B, L, O, I, dtype, rounding):
    rng = np.random.default_rng(B * L + O)
    x = rng.standard_normal((B, L, I)).astype(np.float32) * (1.0 + 2.0 * rng.random((B, 1, 1))).astype(np.float32)
    w = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
    go = (rng.standard_normal((B, L, O)) * 1e-3).astype(np.float32) * (1.0 + 4.0 * rng.random((B, 1, 1))).astype(np.float32)
    n_l, sel = oc.wht_selection(L, 50)
    n_o = oc.block_order(O)
    seed = 11
    x_q_t, s_x, pitch, gx, gw = _batched_layer(ops, go, w, x, n_o, n_l, sel, rounding, dtype, seed=seed)
    out_len = L // n_l * len(sel)

    def u(shape, off):
        return oc.philox_bytes(seed, off, shape) if rounding == "philox" else None
    xf, wf, gof = _as_f32(x, dtype), _as_f32(w, dtype), _as_f32(go, dtype)
    # Philox indices follow the stored layout: [I, B, pitch] for the activation, [I, O] for the weight
    u_x = u((I, B, pitch), 1)
    u_x = None if u_x is None else np.ascontiguousarray(u_x[:, :, :out_len].transpose(1, 2, 0)).view(oc.PhiloxBytes)
    u_w = u((I, O), 3)
    u_w = None if u_w is None else np.ascontiguousarray(u_w.T).view(oc.PhiloxBytes)
    u_gw = u((O, B, pitch), 4)
    u_gw = None if u_gw is None else np.ascontiguousarray(u_gw[:, :, :out_len].transpose(1, 0, 2)).view(oc.PhiloxBytes)
    mode = "stoch" if rounding == "philox" else "int"
    x_q, s_xo = oc.abc_compress_batched(xf, n_l, sel, 8, u_x, mode)
    assert np.array_equal(_bits(s_x.cpu().numpy()), _bits(s_xo))
    got_xq = x_q_t.cpu().numpy().view(np.int8).reshape(I, B, pitch)[:, :, :out_len].transpose(1, 2, 0)
    assert np.array_equal(got_xq, x_q)
    ref = oc.linear_backward_batched(gof, wf, x_q, s_xo, n_o=n_o, n_l=n_l, sel=sel, u_go=u((B, L, O), 2), u_w=u_w,
                                     u_gw=u_gw, w_mode=mode)
    tdt = dtype
    ref_gx = torch.from_numpy(ref["grad_input"]).to(tdt)
    ref_gw = torch.from_numpy(ref["grad_w"]).to(tdt)
    assert torch.equal(gx.cpu(), ref_gx)
    assert torch.equal(gw.cpu(), ref_gw)
