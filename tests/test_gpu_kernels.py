"""GPU parity tests of the three kernels, called through the C ABI and compared with the CPU
oracle on the same seeded inputs.  Integer artefacts (codes, accumulators) and scales must be
bit-exact; dequantised outputs are compared bit-for-bit too where the oracle evaluates the
same float expression, else to 1e-3 relative Frobenius error (the tolerance the target names).
"""
import numpy as np
import pytest
import torch

from oracle import hot_oracle as oc

pytestmark = pytest.mark.gpu


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
    """What the kernel sees: bf16 inputs are rounded to bf16 first, then widened exactly."""
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.to(dtype).to(torch.float32).numpy()


def _codes_from(codes_t, storage, n):
    c = codes_t.cpu().numpy()
    if storage == "int4":
        return oc.unpack_int4(c)[..., :n]
    return c.view(np.int8).astype(np.int32)[..., :n]


def _noise_for(rounding, shape, rng, seed, offset):
    if rounding == "noise":
        return rng.random(shape, dtype=np.float32)
    if rounding == "philox":
        return oc.philox_bytes(seed, offset, shape)
    return None


ROW_CASES = [
    # rows, cols, order
    (37, 768, 16), (5, 192, 32), (64, 1024, 64), (3, 64, 1), (9, 48, 8), (130, 3072, 16), (2, 16384, 16),
]


@pytest.mark.parametrize("rows,cols,order", ROW_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("storage,bits", [("int4", 4), ("int8", 8), ("int8", 4), ("int4", 3), ("int8", 6)])
@pytest.mark.parametrize("rounding", ["nearest", "noise", "philox"])
@pytest.mark.parametrize("scale", ["tensor", "row"])
def test_row_ht_quant(ops, rows, cols, order, dtype, storage, bits, rounding, scale):
    rng = np.random.default_rng(rows * 131 + cols + order)
    x = (rng.standard_normal((rows, cols)) * 1e-3).astype(np.float32)
    x[rows // 2] *= 25.0
    seed, offset = 0x1234ABCD5678, 77
    u = _noise_for(rounding, (rows, cols), rng, seed, offset)
    q = ops.Quant(bits, storage, rounding, scale, seed, offset, _dev(u) if rounding == "noise" else None)
    codes, scales = ops.row_ht_quant(_dev(x, dtype), order, q)
    torch.cuda.synchronize()
    xh = oc.fwht_last(_as_f32(x, dtype), order)
    ref_c, ref_s = (oc.quant_rows if scale == "row" else oc.quant_tensor)(xh, bits, u)
    got_c = _codes_from(codes, storage, cols)
    assert np.array_equal(np.atleast_1d(ref_s).astype(np.float32).view(np.uint32), scales.cpu().numpy().view(np.uint32))
    assert np.array_equal(got_c, ref_c), "%d codes differ" % int((got_c != ref_c).sum())


def _sel_cases():
    return [
        (16, list(range(16))),                         # plain Hadamard (weight side)
        (16, list(oc.lowrank_preset(16, 8))),          # half16
        (32, list(oc.wht_selection(6304, 50)[1])),     # the reference's 10 of 32
        (64, list(oc.wht_selection(12608, 50)[1])),    # 36 of 64
        (4, list(oc.wht_selection(196, 50)[1])),       # 3 of 4
        (1, [0]),                                      # identity (odd token counts)
        (8, list(range(8))),
    ]


@pytest.mark.parametrize("order,sel", _sel_cases())
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("storage,bits", [("int4", 4), ("int8", 8)])
@pytest.mark.parametrize("rounding,layout", [("nearest", "natural"), ("noise", "natural"), ("noise", "transposed"),
                                             ("philox", "natural")])
@pytest.mark.parametrize("scale", ["tensor", "row"])
def test_col_ht_quant(ops, order, sel, dtype, storage, bits, rounding, layout, scale):
    nblk = 21 if order <= 16 else 9
    rows, cols = order * nblk, 200
    r = len(sel)
    out_len = nblk * r
    rng = np.random.default_rng(order * 1000 + r)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    x[:, 7] *= 20.0
    seed, offset = 99, 3
    if rounding == "noise":
        u_t = rng.random((cols, out_len), dtype=np.float32)          # as seen in the stored layout
        u_dev = _dev(u_t if layout == "transposed" else np.ascontiguousarray(u_t.T))
    elif rounding == "philox":
        u_t, u_dev = oc.philox_bytes(seed, offset, (cols, out_len)), None
    else:
        u_t, u_dev = None, None
    q = ops.Quant(bits, storage, rounding, scale, seed, offset, u_dev)
    codes, scales, got_len = ops.col_ht_quant(_dev(x, dtype), order, sel, q, layout)
    torch.cuda.synchronize()
    assert got_len == out_len
    y_t = np.ascontiguousarray(oc.hla(_as_f32(x, dtype), order, np.array(sel)).T)   # [cols, out_len]
    ref_c, ref_s = (oc.quant_rows if scale == "row" else oc.quant_tensor)(y_t, bits, u_t)
    got_c = _codes_from(codes, storage, out_len)
    assert np.array_equal(np.atleast_1d(ref_s).astype(np.float32).view(np.uint32), scales.cpu().numpy().view(np.uint32))
    assert np.array_equal(got_c, ref_c), "%d codes differ" % int((got_c != ref_c).sum())


@pytest.mark.parametrize("order,sel", _sel_cases())
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_hla_project_and_expand(ops, order, sel, dtype):
    """The un-quantised projection along the first dim and its transpose, bit for bit."""
    nblk, cols = 13, 202
    rng = np.random.default_rng(order + len(sel))
    x = rng.standard_normal((order * nblk, cols)).astype(np.float32)
    y = ops.hla_project(_dev(x, dtype), order, sel)
    torch.cuda.synchronize()
    ref = oc.hla(_as_f32(x, dtype), order, np.array(sel))
    assert np.array_equal(y.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    z = ops.hla_expand(y, order, sel, 1.0 / order, dtype)
    torch.cuda.synchronize()
    want = torch.from_numpy(oc.hla_expand(ref, order, np.array(sel), np.float32(1.0 / order))).to(dtype)
    assert torch.equal(z.cpu(), want)


GEMM_CASES = [
    # M, N, K
    (128, 128, 128), (200, 96, 320), (37, 48, 96), (1000, 768, 3072), (384, 130, 50), (256, 256, 1970),
    (768, 768, 6304), (2500, 768, 1024), (19000, 256, 384),
]


@pytest.mark.parametrize("M,N,K", GEMM_CASES)
@pytest.mark.parametrize("a_storage,b_storage", [("int8", "int8"), ("int4", "int4"), ("int4", "int8"), ("int8", "int4")])
@pytest.mark.parametrize("schedule", ["tiles", "streamk", "pairs"])
def test_gemm_i8_accumulators_and_dequant(ops, M, N, K, a_storage, b_storage, schedule, monkeypatch):
    stream_k = schedule == "streamk"
    if stream_k:   # the cost model rarely picks stream-K at test sizes: force it wherever it applies
        monkeypatch.setenv("HOT_GEMM_SCHEDULE", "streamk")
    # CTA pairs (two CTAs per 256-row tile) are chosen by cost too: force them on, or off
    monkeypatch.setenv("HOT_GEMM_PAIR", "1" if schedule == "pairs" else "0")
    rng = np.random.default_rng(M + N + K)

    def make(rows, storage):
        lim = 7 if storage == "int4" else 127
        c = rng.integers(-lim, lim + 1, size=(rows, K)).astype(np.int32)
        if storage == "int4":
            kk = K + (K % 2)
            cp = np.zeros((rows, kk), np.int32)
            cp[:, :K] = c
            packed = oc.pack_int4(cp)
        else:
            packed = c.astype(np.int8).view(np.uint8)
        pitch = (packed.shape[1] + 15) // 16 * 16
        buf = np.full((rows, pitch), 0x5A, np.uint8)           # junk in the pitch padding must not leak in
        buf[:, :packed.shape[1]] = packed
        return c, _dev(buf)

    if (a_storage == "int4" or b_storage == "int4") and K % 2:
        pytest.skip("packed operands need an even K")
    a, a_dev = make(M, a_storage)
    b, b_dev = make(N, b_storage)
    ref = a.astype(np.int64) @ b.astype(np.int64).T
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acc = ops.gemm_i8(a_dev, a_storage, b_dev, b_storage, M, N, K, None, None, out_dtype=torch.int32, status=status,
                      stream_k=stream_k)
    sa = (rng.random(M, dtype=np.float32) + 0.5) * 1e-4
    sb = np.array([3.3e-3], np.float32)
    out = ops.gemm_i8(a_dev, a_storage, b_dev, b_storage, M, N, K, _dev(sa), _dev(sb), post=1.0 / 16, status=status,
                      stream_k=stream_k)
    out_bf = ops.gemm_i8(a_dev, a_storage, b_dev, b_storage, M, N, K, _dev(sa[:1]), _dev(sb), post=0.25,
                         out_dtype=torch.bfloat16, status=status, stream_k=stream_k)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded device-side wait ran out"
    assert np.array_equal(acc.cpu().numpy().astype(np.int64), ref)
    want = ((ref.astype(np.float32) * sa[:, None]) * sb[0]) * np.float32(1.0 / 16)
    assert np.array_equal(out.cpu().numpy(), want)
    want_bf = torch.from_numpy(((ref.astype(np.float32) * sa[0]) * sb[0]) * np.float32(0.25)).to(torch.bfloat16)
    assert torch.equal(out_bf.cpu(), want_bf)


@pytest.mark.parametrize("main_shape,rider_shape", [
    ((12608, 768, 3072), (3072, 768, 6304)),     # fc1: g_x and g_w
    ((12608, 768, 2304), (2304, 768, 6304)),     # qkv
    ((12608, 3072, 768), (768, 3072, 6304)),     # fc2
    ((19000, 256, 384), (256, 256, 1000)),       # ragged last row tile; rider K not a multiple of 128
    ((300, 100, 256), (128, 128, 128)),          # too few main tiles: falls back to two launches
])
@pytest.mark.parametrize("a_storage", ["int8", "int4"])
@pytest.mark.parametrize("force", ["1", None])
def test_gemm_i8_dual(ops, main_shape, rider_shape, a_storage, force, monkeypatch):
    """Two problems in one launch equal the two problems run separately, bit for bit."""
    if force:
        monkeypatch.setenv("HOT_GEMM_DUAL", force)
    rng = np.random.default_rng(sum(main_shape) + sum(rider_shape))

    def operand(rows, K, storage):
        lim = 7 if storage == "int4" else 127
        c = rng.integers(-lim, lim + 1, size=(rows, K)).astype(np.int32)
        packed = oc.pack_int4(c) if storage == "int4" else c.astype(np.int8).view(np.uint8)
        pitch = (packed.shape[1] + 15) // 16 * 16
        buf = np.zeros((rows, pitch), np.uint8)
        buf[:, :packed.shape[1]] = packed
        return c, _dev(buf)
    (M0, N0, K0), (M1, N1, K1) = main_shape, rider_shape
    a0, a0d = operand(M0, K0, a_storage)
    b0, b0d = operand(N0, K0, "int8")
    a1, a1d = operand(M1, K1, "int8")
    b1, b1d = operand(N1, K1, "int8")
    sa0 = (rng.random(M0, dtype=np.float32) + 0.5) * 1e-4
    sb0, sa1, sb1 = np.array([3.3e-3], np.float32), np.array([7.1e-5], np.float32), np.array([2.2e-2], np.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    main = dict(a=a0d, a_storage=a_storage, b=b0d, M=M0, N=N0, K=K0, scale_a=_dev(sa0), scale_b=_dev(sb0), post=1.0 / 16,
                out_dtype=torch.bfloat16)
    rider = dict(a=a1d, b=b1d, M=M1, N=N1, K=K1, scale_a=_dev(sa1), scale_b=_dev(sb1), post=1.0 / 16, out_dtype=torch.float32)
    o0, o1 = ops.gemm_i8_dual(main, rider, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded device-side wait ran out"
    # float64 BLAS is exact for these integer products (|acc| < 2^53) and far quicker than int64 matmul
    r0 = (a0.astype(np.float64) @ b0.astype(np.float64).T).astype(np.float32)
    r1 = (a1.astype(np.float64) @ b1.astype(np.float64).T).astype(np.float32)
    want0 = torch.from_numpy(((r0 * sa0[:, None]) * sb0[0]) * np.float32(1.0 / 16)).to(torch.bfloat16)
    want1 = ((r1 * sa1[0]) * sb1[0]) * np.float32(1.0 / 16)
    assert torch.equal(o0.cpu(), want0)
    assert np.array_equal(o1.cpu().numpy(), want1)


def _run_backward(ops, x, w, go, order_l, sel, dtype, *, gx_row=False, gw_row=False, rounding="noise", rng=None,
                  storage4="int4"):
    L, I = x.shape
    O = w.shape[0]
    n_o = oc.block_order(O)
    r = len(sel)
    Lp = L // order_l * r
    seeds = dict(x=(11, 1), go=(11, 2), w=(11, 3), gw=(11, 4))
    shapes = dict(x=(Lp, I), go=(L, O), w=(O, I), gw=(O, Lp))
    us, qs = {}, {}
    for k in shapes:
        if rounding == "noise":
            us[k] = rng.random(shapes[k], dtype=np.float32)
        elif rounding == "philox":
            # Philox streams are indexed in the stored layout: transposed for x and w
            if k in ("x", "w"):
                us[k] = np.ascontiguousarray(oc.philox_bytes(*seeds[k], shapes[k][::-1]).T).view(oc.PhiloxBytes)
            else:
                us[k] = oc.philox_bytes(*seeds[k], shapes[k])
        else:
            us[k] = None
    def mk(k, bits, storage, scale="tensor"):
        return ops.Quant(bits, storage, rounding, scale, seeds[k][0], seeds[k][1],
                         _dev(us[k]) if rounding == "noise" else None)
    cfg = ops.LinearConfig(order_o=n_o, order_l=order_l, sel_l=list(sel),
                           q_gx=mk("go", 4, storage4, "row" if gx_row else "tensor"), q_w=mk("w", 4, storage4),
                           q_gw=mk("gw", 8, "int8", "row" if gw_row else "tensor"), q_x=mk("x", 8, "int8"))
    xd, wd, god = _dev(x, dtype), _dev(w, dtype), _dev(go, dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x_q_t, s_x = ops.abc_compress(xd, cfg)
    gx, gw = ops.linear_backward(god, wd, x_q_t, s_x, cfg, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # oracle
    xf, wf, gof = _as_f32(x, dtype), _as_f32(w, dtype), _as_f32(go, dtype)
    xq_ref, sx_ref = oc.abc_compress(xf, order_l, np.array(sel), 8, us["x"], "stoch" if rounding != "nearest" else "int")
    ref = oc.linear_backward(gof, wf, xq_ref, sx_ref, n_o=n_o, n_l=order_l, sel=np.array(sel), u_go=us["go"],
                             u_w=us["w"], u_gw=us["gw"], gx_per_token=gx_row, gw_per_channel=gw_row,
                             w_mode="stoch" if rounding != "nearest" else "int")
    got_xq = x_q_t.cpu().numpy().view(np.int8).astype(np.int32)[:, :Lp].T
    assert np.array_equal(got_xq, xq_ref)
    assert np.float32(sx_ref).view(np.uint32) == s_x.cpu().numpy().view(np.uint32)[0]
    return gx, gw, ref


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rounding", ["noise", "philox", "nearest"])
@pytest.mark.parametrize("gx_row,gw_row", [(False, False), (True, True)])
@pytest.mark.parametrize("preset", ["half16", "ref32"])
@pytest.mark.parametrize("I", [136, 160])   # 160: a multiple of 32, so that in bf16 the weight is quantised by the grad_out kernels
def test_linear_backward_vs_oracle(ops, dtype, rounding, gx_row, gw_row, preset, I):
    rng = np.random.default_rng(5)
    L, O = 32 * 13, 384
    order_l, sel = (16, oc.lowrank_preset(16, 8)) if preset == "half16" else (32, oc.wht_selection(6304, 50)[1])
    x = rng.standard_normal((L, I)).astype(np.float32)
    x[:, 5] *= 20.0
    w = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
    go = (rng.standard_normal((L, O)) * 1e-3).astype(np.float32)
    go[17] *= 30.0
    gx, gw, ref = _run_backward(ops, x, w, go, order_l, sel, dtype, gx_row=gx_row, gw_row=gw_row, rounding=rounding,
                                rng=rng)
    for got, name in ((gx, "grad_input"), (gw, "grad_w")):
        want = ref[name]
        g = got.float().cpu().numpy()
        if dtype == torch.float32:
            assert np.array_equal(g, want), "%s: %d of %d values differ" % (name, (g != want).sum(), g.size)
        else:
            rel = np.linalg.norm(g - want) / np.linalg.norm(want)
            assert rel < 4e-3, (name, rel)     # bf16 output rounding: 2^-9 per element


@pytest.mark.parametrize("tag", ["lr_ref", "lr_half16"])
def test_linear_backward_vs_reference_golden(ops, golden, tag):
    """Against outputs of the unmodified reference (FLinearQ forward context + backward with
    explicit rounding noise).  The reference's transforms are BLAS matmuls, so a transformed
    value can differ in the last ulp and flip a code: the comparison is the 1e-3 relative
    Frobenius bound on the dequantised gradients."""
    g = golden("flinearq_" + tag)
    n_l, sel = oc.selection_from_matrix(g["p"])
    x, w, go = g["x"], g["w"], g["go"]
    L, I = x.shape
    O = w.shape[0]
    Lp = L // n_l * len(sel)
    q = lambda bits, storage, u: ops.Quant(bits, storage, "noise", "tensor", 0, 0, _dev(u))
    cfg = ops.LinearConfig(order_o=oc.block_order(O), order_l=n_l, sel_l=list(sel), q_gx=q(4, "int4", g["u_go"]),
                           q_w=q(4, "int4", g["u_w"]), q_gw=q(8, "int8", g["u_gw"]), q_x=q(8, "int8", g["u_x"]))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x_q_t, s_x = ops.abc_compress(_dev(x), cfg)
    gx, gw = ops.linear_backward(_dev(go), _dev(w), x_q_t, s_x, cfg, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got_xq = x_q_t.cpu().numpy().view(np.int8).astype(np.int32)[:, :Lp].T
    assert np.mean(got_xq != g["x_q"].astype(np.int32)) < 1e-3
    np.testing.assert_allclose(s_x.cpu().numpy()[0], g["scale_x"], rtol=1e-6)
    for got, name in ((gx, "grad_input"), (gw, "grad_w")):
        rel = np.linalg.norm(got.cpu().numpy() - g[name]) / np.linalg.norm(g[name])
        assert rel < 1e-3, (name, rel)


@pytest.mark.parametrize("basis", ["half16", "ref_10_of_32"])
def test_config1_fc1_full_size(ops, basis):
    """The single-layer configuration the targets are stated on, at its real size: ViT-B/16 fc1,
    X [6304, 768] ~ N(0, 1) with 8 of 768 channels scaled by 20, W [3072, 768] kaiming-uniform,
    grad_out [6304, 3072] ~ N(0, 1e-3), fp32, seed 0, explicit rounding noise; Hadamard order 16 +
    INT4 for g_x, low-rank (8 lowest-sequency rows of H_16, and the reference's own make_WHT(6304)
    rows) + INT8 for g_w.  Codes, scales, int32 accumulators and fp32 gradients are bit-exact
    against the oracle."""
    import math
    gen = torch.Generator().manual_seed(0)
    L, I, O = 6304, 768, 3072
    x = torch.randn(L, I, generator=gen)
    x[:, torch.randperm(I, generator=gen)[:8]] *= 20.0
    bound = 1.0 / math.sqrt(I)                                    # kaiming_uniform_(a=sqrt(5)) on [O, I]
    w = (torch.rand(O, I, generator=gen) * 2 - 1) * bound
    go = torch.randn(L, O, generator=gen) * 1e-3
    x, w, go = x.numpy(), w.numpy(), go.numpy()
    order_l, sel = (16, oc.lowrank_preset(16, 8)) if basis == "half16" else oc.wht_selection(L, 50)
    assert (order_l, len(sel)) == ((16, 8) if basis == "half16" else (32, 10))
    Lp = L // order_l * len(sel)
    rng = np.random.default_rng(0)
    u = {k: rng.random(shp, dtype=np.float32) for k, shp in dict(x=(Lp, I), go=(L, O), w=(O, I), gw=(O, Lp)).items()}
    mk = lambda k, bits, storage: ops.Quant(bits, storage, "noise", "tensor", 0, 0, _dev(u[k]))
    cfg = ops.LinearConfig(order_o=16, order_l=order_l, sel_l=[int(v) for v in sel], q_gx=mk("go", 4, "int4"),
                           q_w=mk("w", 4, "int4"), q_gw=mk("gw", 8, "int8"), q_x=mk("x", 8, "int8"))
    xd, wd, god = _dev(x), _dev(w), _dev(go)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x_q_t, s_x = ops.abc_compress(xd, cfg)
    gx, gw = ops.linear_backward(god, wd, x_q_t, s_x, cfg, status=status)
    # the operands one by one, for the integer artefacts
    q_go, s_go = ops.row_ht_quant(god, 16, cfg.q_gx)
    q_w_t, s_w, _ = ops.col_ht_quant(wd, 16, list(range(16)), mk("w", 4, "int8"), "natural")      # [I, O] codes
    q_gw_t, s_gw, lp = ops.col_ht_quant(god, order_l, [int(v) for v in sel], cfg.q_gw, "transposed")  # [O, L'] codes
    acc_x = ops.gemm_i8(q_go, "int4", q_w_t, "int8", L, I, O, None, None, out_dtype=torch.int32, status=status)
    acc_w = ops.gemm_i8(q_gw_t, "int8", x_q_t, "int8", O, I, Lp, None, None, out_dtype=torch.int32, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and lp == Lp
    xq_ref, sx_ref = oc.abc_compress(x, order_l, np.array(sel), 8, u["x"])
    ref = oc.linear_backward(go, w, xq_ref, sx_ref, n_o=16, n_l=order_l, sel=np.array(sel), u_go=u["go"], u_w=u["w"],
                             u_gw=u["gw"], exact_matmul=False)   # float32 BLAS on integer values: exact below 2^24
    bits32 = lambda a: np.atleast_1d(np.asarray(a, dtype=np.float32)).view(np.uint32)
    assert np.array_equal(x_q_t.cpu().numpy().view(np.int8).astype(np.int32)[:, :Lp].T, xq_ref)
    assert np.array_equal(bits32(sx_ref), s_x.cpu().numpy().view(np.uint32))
    assert np.array_equal(_codes_from(q_go, "int4", O), ref["q_go"])
    assert np.array_equal(_codes_from(q_w_t, "int8", O).T, ref["q_w"])
    assert np.array_equal(_codes_from(q_gw_t, "int8", Lp), ref["q_gw"])
    for got, want in ((s_go, ref["s_go"]), (s_w, ref["s_w"]), (s_gw, ref["s_gw"])):
        assert np.array_equal(got.cpu().numpy().view(np.uint32), bits32(want))
    assert np.abs(ref["acc_x"]).max() < 2 ** 24 and np.abs(ref["acc_w"]).max() < 2 ** 24
    assert np.array_equal(acc_x.cpu().numpy(), ref["acc_x"].astype(np.int32))
    assert np.array_equal(acc_w.cpu().numpy(), ref["acc_w"].astype(np.int32))
    assert np.array_equal(gx.cpu().numpy(), ref["grad_input"])
    assert np.array_equal(gw.cpu().numpy(), ref["grad_w"])


def test_a_bounded_wait_that_runs_out_is_reported_and_leaves_the_device_usable(ops):
    """One warp waits, with the kernels' own wait routine, on a barrier nothing ever arrives on, with the
    limit set to 2 ms: the kernel returns by itself, its bit is in the status word, the host side turns
    the word into HOT_ERR_TIMEOUT, and the next ordinary launch on the same stream is correct."""
    from hot_b200 import _cabi as C
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.set_wait_limit_ns(2_000_000)
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        ops.wait_probe(status)
        t1.record()
        torch.cuda.synchronize()
        assert 1.5 < t0.elapsed_time(t1) < 200.0                    # it waited about the limit, then gave up
        assert int(status.item()) == 8                               # HOT_STATUS_PROBE
        with pytest.raises(C.HotError, match="bounded device-side wait ran out.*wait probe") as err:
            ops.check_status(status)
        assert err.value.status == C.HOT_ERR_TIMEOUT
    finally:
        ops.set_wait_limit_ns(0)
    # the context is intact: a real launch with a clean status word right after
    status.zero_()
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((64, 128)) * 1e-3).astype(np.float32)
    codes, scales = ops.row_ht_quant(_dev(x), 16, ops.Quant(8, "int8", "nearest", "tensor"))
    a = torch.randint(-7, 8, (128, 256), device="cuda", dtype=torch.int8)
    b = torch.randint(-7, 8, (64, 256), device="cuda", dtype=torch.int8)
    acc = ops.gemm_i8(a.view(torch.uint8), "int8", b.view(torch.uint8), "int8", 128, 64, 256, None, None,
                      out_dtype=torch.int32, status=status)
    torch.cuda.synchronize()
    ops.check_status(status)                                         # 0: nothing ran out
    ref_c, ref_s = oc.quant_tensor(oc.fwht_last(x, 16), 8, None)
    assert np.array_equal(_codes_from(codes, "int8", 128), ref_c)
    assert torch.equal(acc.cpu(), (a.cpu().int() @ b.cpu().int().t()))


def test_errors_are_reported(ops):
    x = torch.zeros((4, 24), device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 16"):
        ops.row_ht_quant(x[:, :20].contiguous(), 4, ops.Quant(4, "int4"))
    with pytest.raises(RuntimeError, match="INT4 storage needs bits"):
        ops.row_ht_quant(x, 8, ops.Quant(8, "int4"))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.row_ht_quant(x.cpu(), 8, ops.Quant(8, "int8"))
    with pytest.raises(RuntimeError, match="not a multiple of order"):
        ops.col_ht_quant(torch.zeros((10, 8), device="cuda"), 4, [0, 1], ops.Quant(8, "int8"))
    # empty input is a no-op
    codes, scales = ops.row_ht_quant(torch.zeros((0, 64), device="cuda"), 16, ops.Quant(8, "int8", scale="row"))
    assert codes.shape == (0, 64)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rounding", ["philox", "nearest"])
@pytest.mark.parametrize("gx_scale,gw_scale", [("tensor", "tensor"), ("row", "row")])
@pytest.mark.parametrize("L,O,order_o,gx_storage", [(32 * 21, 192, 16, "int4"), (256 + 96, 128, 64, "int8"), (512, 64, 32, "int4")])
def test_go_dual_quant_matches_the_separate_kernels(ops, dtype, rounding, gx_scale, gw_scale, L, O, order_o, gx_storage):
    """The fused grad_out kernels against row_ht_quant + col_ht_quant (themselves checked against
    the oracle above): codes and scales bit-identical, ragged last token tile included."""
    torch.manual_seed(L + O)
    go = (torch.randn(L, O, device="cuda") * 1e-3).to(dtype)
    go[5] *= 30.0
    go[:, 3] *= 10.0
    sel = [int(v) for v in oc.lowrank_preset(16, 8)]
    bits_x = 4 if gx_storage == "int4" else 8
    cfg = ops.LinearConfig(order_o=order_o, order_l=16, sel_l=sel,
                           q_gx=ops.Quant(bits_x, gx_storage, rounding, gx_scale, 21, 5),
                           q_gw=ops.Quant(8, "int8", rounding, gw_scale, 21, 6))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    q_go, s_gx, q_gw, s_gw = ops.go_dual_quant(go, cfg, status)
    ref_go, ref_sx = ops.row_ht_quant(go, order_o, cfg.q_gx)
    ref_gw, ref_sw, lp = ops.col_ht_quant(go, 16, sel, cfg.q_gw, "transposed")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(s_gx.view(torch.int32), ref_sx.view(torch.int32))
    assert torch.equal(s_gw.view(torch.int32), ref_sw.view(torch.int32))
    assert torch.equal(q_go, ref_go)
    assert torch.equal(q_gw[:, :lp], ref_gw[:, :lp])


@pytest.mark.parametrize("rounding", ["philox", "nearest"])
@pytest.mark.parametrize("gx_scale,gw_scale", [("tensor", "tensor"), ("row", "row")])
@pytest.mark.parametrize("L,O,gx_storage,bits_x,bits_w", [(32 * 21, 384, "int4", 4, 8), (128 * 3 + 96, 128, "int8", 4, 8),
                                                          (256, 256, "int8", 8, 4), (32, 128, "int4", 3, 6),
                                                          (128 * 40, 768, "int4", 4, 8)])
def test_go_dual_quant_tensor_core_transforms(ops, rounding, gx_scale, gw_scale, L, O, gx_storage, bits_x, bits_w):
    """bf16 grad_out with channel order 16 takes the kernels that run both +-1 transforms on the tensor
    cores.  Their fp32 sums equal the butterflies' wherever a 16-term sum is exact in fp32; elsewhere a
    transformed value may differ in its last bit.  So: scales equal to the butterfly kernels' to within
    one ulp, and where they are bit-equal (the rule) at most a few codes in a million differ, by one."""
    torch.manual_seed(L * 7 + O)
    go = (torch.randn(L, O, device="cuda") * 1e-3).to(torch.bfloat16)
    go[5] *= 30.0
    go[:, 3] *= 10.0
    sel = [int(v) for v in oc.lowrank_preset(16, 8)]
    cfg = ops.LinearConfig(order_o=16, order_l=16, sel_l=sel,
                           q_gx=ops.Quant(bits_x, gx_storage, rounding, gx_scale, 21, 5),
                           q_gw=ops.Quant(bits_w, "int8", rounding, gw_scale, 21, 6))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    q_go, s_gx, q_gw, s_gw = ops.go_dual_quant(go, cfg, status)
    ref_go, ref_sx = ops.row_ht_quant(go, 16, cfg.q_gx)
    ref_gw, ref_sw, lp = ops.col_ht_quant(go, 16, sel, cfg.q_gw, "transposed")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for got_s, ref_s in ((s_gx, ref_sx), (s_gw, ref_sw)):
        ulps = (got_s.view(torch.int32).long() - ref_s.view(torch.int32).long()).abs()
        assert int(ulps.max()) <= 1, "a scale is more than one ulp from the butterfly kernels'"
    same_x = (s_gx.view(torch.int32) == ref_sx.view(torch.int32))
    same_w = (s_gw.view(torch.int32) == ref_sw.view(torch.int32))
    got_x, want_x = _codes_from(q_go, gx_storage, O), _codes_from(ref_go, gx_storage, O)
    got_w, want_w = _codes_from(q_gw, "int8", lp), _codes_from(ref_gw, "int8", lp)
    rows_x = same_x.cpu().numpy() if gx_scale == "row" else np.full(L, bool(same_x[0]))
    rows_w = same_w.cpu().numpy() if gw_scale == "row" else np.full(O, bool(same_w[0]))
    for got, want, rows in ((got_x, want_x, rows_x), (got_w, want_w, rows_w)):
        d = np.abs(got[rows] - want[rows])
        assert d.size == 0 or d.max() <= 1
        assert d.sum() <= max(2, 1e-5 * d.size), "%d of %d codes differ" % (int(d.sum()), d.size)
        assert np.abs(got - want).max() <= 1       # rows whose scale moved by an ulp: still neighbours
    assert rows_x.mean() > 0.99 and rows_w.mean() > 0.99


@pytest.mark.parametrize("rounding", ["philox", "nearest"])
@pytest.mark.parametrize("w_bits", [4, 8, 3])
@pytest.mark.parametrize("L,O,I", [(32 * 13, 384, 160), (256, 128, 32), (640, 256, 768), (128 * 150, 128, 64)])
def test_weight_quantised_by_the_grad_out_kernels_matches_its_own_kernels(ops, monkeypatch, rounding, w_bits, L, O, I):
    """In bf16 with the order-16 bases the weight is transformed and quantised inside the two grad_out kernels;
    HOT_WEIGHT_QUANT=separate sends it through hot_col_ht_quant instead.  Same codes and scale, hence the same
    accumulators: both gradients must be bit-identical."""
    rng = np.random.default_rng(L + O + I + w_bits)
    x = torch.from_numpy(rng.standard_normal((L, I)).astype(np.float32)).cuda().bfloat16()
    w = torch.from_numpy(((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)).cuda().bfloat16()
    w[5, 3] = 1.5   # one large entry decides the scale
    go = torch.from_numpy((rng.standard_normal((L, O)) * 1e-3).astype(np.float32)).cuda().bfloat16()
    sel = [int(v) for v in oc.lowrank_preset(16, 8)]
    cfg = ops.LinearConfig(order_o=16, order_l=16, sel_l=sel, q_gx=ops.Quant(4, "int4", rounding, "tensor", 3, 1),
                           q_w=ops.Quant(w_bits, "int4" if w_bits <= 4 else "int8", rounding, "tensor", 7, 2),
                           q_gw=ops.Quant(8, "int8", rounding, "tensor", 11, 3), q_x=ops.Quant(8, "int8", rounding, "tensor", 13, 4))
    x_q_t, s_x = ops.abc_compress(x, cfg)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = {}
    for mode in ("rides", "separate"):
        if mode == "separate":
            monkeypatch.setenv("HOT_WEIGHT_QUANT", "separate")
        else:
            monkeypatch.delenv("HOT_WEIGHT_QUANT", raising=False)
        gx, gw = ops.linear_backward(go, w, x_q_t, s_x, cfg, status=status)
        torch.cuda.synchronize()
        out[mode] = (gx.clone(), gw.clone())
    assert int(status.item()) == 0
    assert float(out["rides"][0].float().abs().max()) > 0
    assert torch.equal(out["rides"][0], out["separate"][0])
    assert torch.equal(out["rides"][1], out["separate"][1])


@pytest.mark.parametrize("L,O,I", [(128 * 50, 256, 768), (12608, 768, 768)])
def test_dual_gemm_with_g_w_tiles_cut_along_the_tokens(ops, monkeypatch, L, O, I):
    """The layer's GEMM launch may cut the few, long tiles of the g_w product into stretches of k-blocks that run on
    different SMs and are summed by whichever finishes last.  Integer sums: the gradients must be bit-identical to
    those of whole tiles, whatever the cut."""
    rng = np.random.default_rng(L + O)
    x = torch.from_numpy(rng.standard_normal((L, I)).astype(np.float32)).cuda().bfloat16()
    w = torch.from_numpy(((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)).cuda().bfloat16()
    go = torch.from_numpy((rng.standard_normal((L, O)) * 1e-3).astype(np.float32)).cuda().bfloat16()
    sel = [int(v) for v in oc.lowrank_preset(16, 8)]
    cfg = ops.LinearConfig(order_o=16, order_l=16, sel_l=sel, q_gx=ops.Quant(4, "int8", "philox", "tensor", 3, 1))
    x_q_t, s_x = ops.abc_compress(x, cfg)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    monkeypatch.setenv("HOT_GEMM_DUAL", "1")
    out = {}
    for split in ("1", "2", "3", "4"):
        monkeypatch.setenv("HOT_GEMM_RIDER_SPLIT", split)
        for rep in range(2):   # twice: the counters must come back to zero
            gx, gw = ops.linear_backward(go, w, x_q_t, s_x, cfg, status=status)
        torch.cuda.synchronize()
        out[split] = (gx.clone(), gw.clone())
    assert int(status.item()) == 0
    assert float(out["1"][1].float().abs().max()) > 0
    for split in ("2", "3", "4"):
        assert torch.equal(out[split][0], out["1"][0]), split
        assert torch.equal(out[split][1], out["1"][1]), split


@pytest.mark.parametrize("rounding", ["philox", "nearest"])
@pytest.mark.parametrize("bits", [8, 6])
@pytest.mark.parametrize("L,I", [(32 * 13, 128), (12608, 768), (640, 3072)])
def test_activation_buffer_from_the_tensor_core_kernels_matches_the_butterfly_kernel(ops, monkeypatch, rounding, bits, L, I):
    """bf16 with the order-16 token basis: hot_abc_compress runs the token side of the tensor-core grad_out kernels;
    HOT_ABC=butterfly keeps hot_col_ht_quant.  Same codes, same scale."""
    rng = np.random.default_rng(L + I + bits)
    x = torch.from_numpy(rng.standard_normal((L, I)).astype(np.float32)).cuda().bfloat16()
    x[:, 5] *= 20.0
    sel = [int(v) for v in oc.lowrank_preset(16, 8)]
    cfg = ops.LinearConfig(order_o=16, order_l=16, sel_l=sel, q_x=ops.Quant(bits, "int8", rounding, "tensor", 13, 4))
    out = {}
    for mode in ("tc", "butterfly"):
        if mode == "butterfly":
            monkeypatch.setenv("HOT_ABC", "butterfly")
        else:
            monkeypatch.delenv("HOT_ABC", raising=False)
        q, s = ops.abc_compress(x, cfg)
        torch.cuda.synchronize()
        out[mode] = (q.clone(), s.clone())
    lp = L // 2
    assert int(out["tc"][0][:, :lp].view(torch.int8).abs().max()) == (1 << (bits - 1)) - 1
    assert torch.equal(out["tc"][1], out["butterfly"][1])
    assert torch.equal(out["tc"][0][:, :lp], out["butterfly"][0][:, :lp])


def test_go_dual_quant_rejects_what_it_does_not_cover(ops):
    go = torch.zeros((64, 64), device="cuda")
    cfg = ops.LinearConfig(order_o=16, order_l=32, sel_l=list(oc.wht_selection(6304, 50)[1]))
    with pytest.raises(RuntimeError, match="hot_go_dual_quant covers"):
        ops.go_dual_quant(go, cfg)
