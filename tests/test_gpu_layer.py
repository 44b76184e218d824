"""GPU tests of the reference-facing layer: the quantiser callables, FLinearQ / HQ_Linear,
replace_layers, layer-wise quantiser selection and the HLQ_backward plugin call."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import hot_oracle as oc

pytestmark = pytest.mark.gpu


@pytest.fixture()
def hot():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import hot_b200.args as args
    import hot_b200.quant_matmul as qm
    saved = {k: getattr(args, k) for k in dir(args) if not k.startswith("_")}
    args.transform_scheme = "gih_gwlr"
    args.TransformGogi = args.TransformWgt = args.TransformGogw = args.TransformInput = True
    args.GogiQuantBit, args.weightQuantBit, args.GogwQuantBit, args.actQuantBit = 4, 4, 8, 8
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "stoch"
    args.quantAuto = False
    args.layer_quant_dict.clear()
    args.lowRankPreset = "half16"
    yield args, qm
    for k, v in saved.items():
        setattr(args, k, v)
    args.layer_quant_dict.clear()


def test_quantiser_callables_follow_the_reference_contract(hot):
    _, qm = hot
    g = torch.randn(48, 100, device="cuda") * 1e-3            # 100 columns: not a multiple of 8
    g[5] *= 40
    gn = g.cpu().numpy()
    q, s = qm.int_quantizer(g, 4, False)
    ref_q, ref_s = oc.quant_tensor(gn, 4, None)
    assert q.dtype == g.dtype and q.shape == g.shape
    assert np.array_equal(q.cpu().numpy().astype(np.int32), ref_q)
    assert np.float32(s.item()) == ref_s
    q, s = qm.stoch_quantizer(g, 4, False)
    qn = q.cpu().numpy()
    assert np.abs(qn).max() <= 7 and np.array_equal(qn, np.rint(qn))
    y = gn / (ref_s + np.float32(1e-11))
    assert np.all(np.abs(qn - y) < 1.0 + 1e-6)                 # each code is floor or ceil of the exact quotient
    assert abs(float((qn - y).mean())) < 0.02                  # and unbiased
    d, one = qm.norm_quantizer(g, 4, False)
    assert one == 1.0 and d.shape == g.shape
    row_err = (d - g).abs().amax(dim=1) / g.abs().amax(dim=1)
    assert float(row_err.max()) < 1.0 / 7 + 1e-3               # error bounded by one per-row step
    q, s = qm.sawb_quantizer(g.reshape(4, 12, 100), 4, True)   # one clip per sample
    assert q.shape == (4, 12, 100) and s.shape == (4,)
    for b in range(4):
        rq, rs = oc.quant_sawb(gn.reshape(4, 12, 100)[b], 4)
        assert np.float32(s[b].item()) == rs and np.array_equal(q[b].cpu().numpy().astype(np.int32), rq)
    assert set(qm.quant_scheme_dict) >= {"int_quantizer", "stoch_quantizer", "norm_quantizer"}


def test_hq_linear_matches_oracle_with_nearest_rounding(hot):
    args, qm = hot
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "int"   # deterministic
    torch.manual_seed(0)
    L, I, O = 320, 64, 96
    lin = qm.HQ_Linear(I, O).cuda()
    lin.layer_name = "blocks.0.mlp.fc1"
    x = torch.randn(L, I, device="cuda", requires_grad=True)
    go = torch.randn(L, O, device="cuda") * 1e-3
    y = lin(x)
    assert torch.allclose(y, torch.nn.functional.linear(x, lin.weight, lin.bias), atol=1e-5)
    y.backward(go)
    assert tuple(lin.hadamard_out.shape) == (16, 16) and tuple(lin.hadamard_bs.shape) == (8, 16)
    sel = np.array(oc.lowrank_preset(16, 8))
    xq, sx = oc.abc_compress(x.detach().cpu().numpy(), 16, sel, 8, None, "int")
    ref = oc.linear_backward(go.cpu().numpy(), lin.weight.detach().cpu().numpy(), xq, sx, n_o=16, n_l=16, sel=sel,
                             w_mode="int")
    assert np.array_equal(x.grad.cpu().numpy(), ref["grad_input"])
    assert np.array_equal(lin.weight.grad.cpu().numpy(), ref["grad_w"])
    assert torch.allclose(lin.bias.grad, go.sum(0), rtol=1e-4, atol=1e-6)   # bias grad is ordinary autograd


def test_hq_linear_3d_and_reference_low_rank_basis(hot):
    args, qm = hot
    args.lowRankPreset = None                                    # follow make_WHT(tokens, 50)
    lin = qm.HQ_Linear(64, 96).cuda()
    x = torch.randn(4, 160, 64, device="cuda", requires_grad=True)   # per-sample length 160 -> n=32, r=10
    y = lin(x)
    assert tuple(lin.hadamard_bs.shape) == (10, 32)
    y.backward(torch.randn_like(y) * 1e-3)
    assert x.grad.shape == x.shape and lin.weight.grad.shape == lin.weight.shape
    assert torch.isfinite(x.grad).all() and torch.isfinite(lin.weight.grad).all()
    x2 = torch.randn(3, 197, 64, device="cuda", requires_grad=True)  # ViT token count: identity basis
    lin(x2).sum().backward()
    assert tuple(lin.hadamard_bs.shape) == (1, 1)


def test_hq_linear_scheme_hadamard(hot):
    """transform_scheme "hadamard": full block Hadamard along the tokens; against the oracle bit for
    bit with nearest rounding, and against the reference's own run (golden, explicit noise)."""
    args, qm = hot
    args.transform_scheme = "hadamard"
    args.lowRankPreset = None
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "int"
    torch.manual_seed(5)
    L, I, O = 208, 64, 96                                        # 208 = 16 * 13 tokens
    lin = qm.HQ_Linear(I, O, bias=False).cuda()
    x = torch.randn(L, I, device="cuda", requires_grad=True)
    go = torch.randn(L, O, device="cuda") * 1e-3
    lin(x).backward(go)
    assert tuple(lin.hadamard_bs.shape) == (16, 16)
    sel = np.arange(16)
    xq, sx = oc.abc_compress(x.detach().cpu().numpy(), 16, sel, 8, None, "int")
    ref = oc.linear_backward(go.cpu().numpy(), lin.weight.detach().cpu().numpy(), xq, sx, n_o=16, n_l=16, sel=sel,
                             w_mode="int")
    assert np.array_equal(x.grad.cpu().numpy(), ref["grad_input"])
    assert np.array_equal(lin.weight.grad.cpu().numpy(), ref["grad_w"])
    # the reference's run of this scheme
    import os
    from hot_b200 import ops
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "flinearq_hadamard.npz"))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    q = lambda bits, st, u: ops.Quant(bits, st, "noise", "tensor", 0, 0, dev(u))
    cfg = ops.LinearConfig(order_o=16, order_l=16, sel_l=list(range(16)), q_gx=q(4, "int4", g["u_go"]), q_w=q(4, "int4", g["u_w"]),
                           q_gw=q(8, "int8", g["u_gw"]), q_x=q(8, "int8", g["u_x"]))
    x_q_t, s_x = ops.abc_compress(dev(g["x"]), cfg)
    gx, gw = ops.linear_backward(dev(g["go"]), dev(g["w"]), x_q_t, s_x, cfg)
    for got, name in ((gx, "grad_input"), (gw, "grad_w")):
        rel = np.linalg.norm(got.cpu().numpy() - g[name]) / np.linalg.norm(g[name])
        assert rel < 1e-3, (name, rel)


@pytest.mark.parametrize("scheme", ["low_rank", "gilr_gwh"])
def test_hq_linear_token_lowrank_schemes(hot, scheme):
    """transform_scheme low_rank / gilr_gwh: grad_output projected along the tokens for g_x, weight
    untransformed, grad_input expanded back; bit for bit against the oracle with nearest rounding, and
    against the reference's own run (golden, explicit noise)."""
    import os
    from hot_b200 import ops
    args, qm = hot
    args.transform_scheme = scheme
    args.lowRankPreset = None
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "int"
    torch.manual_seed(6)
    L, I, O = 192, 64, 96                                        # 192 tokens: low-rank order 64, block Hadamard order 16
    lin = qm.HQ_Linear(I, O, bias=False).cuda()
    x = torch.randn(L, I, device="cuda", requires_grad=True)
    go = torch.randn(L, O, device="cuda") * 1e-3
    lin(x).backward(go)
    n_x, sel_x = oc.wht_selection(L, 50)
    n_w, sel_w = (n_x, sel_x) if scheme == "low_rank" else (16, np.arange(16))
    xq, sx = oc.abc_compress(x.detach().cpu().numpy(), n_w, sel_w, 8, None, "int")
    wn, gon = lin.weight.detach().cpu().numpy(), go.cpu().numpy()
    ref_gx = oc.grad_input_lowrank(gon, wn, n=n_x, sel=sel_x, w_mode="int")["grad_input"]
    ref_gw = oc.linear_backward(gon, wn, xq, sx, n_o=1, n_l=n_w, sel=sel_w, w_mode="int")["grad_w"]
    assert np.array_equal(x.grad.cpu().numpy(), ref_gx)
    assert np.array_equal(lin.weight.grad.cpu().numpy(), ref_gw)
    # the reference's run of this scheme
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "flinearq_%s.npz" % scheme))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    q = lambda bits, st, u: ops.Quant(bits, st, "noise", "tensor", 0, 0, dev(u))
    n_x, sel_x = oc.selection_from_matrix(g["lowrank"])
    n_w, sel_w = (n_x, sel_x) if scheme == "low_rank" else oc.selection_from_matrix(g["hadamard"])
    cfg = ops.LinearConfig(order_o=1, order_l=n_w, sel_l=list(sel_w), q_gw=q(8, "int8", g["u_gw"]), q_x=q(8, "int8", g["u_x"]))
    x_q_t, s_x = ops.abc_compress(dev(g["x"]), cfg)
    _, gw = ops.linear_backward(dev(g["go"]), dev(g["w"]), x_q_t, s_x, cfg, need_gx=False)
    gx = ops.linear_backward_lowrank_gx(dev(g["go"]), dev(g["w"]), n_x, list(sel_x), q(4, "int4", g["u_go"]),
                                        q(4, "int4", np.ascontiguousarray(g["u_w"])))
    for got, name in ((gx, "grad_input"), (gw, "grad_w")):
        rel = np.linalg.norm(got.cpu().numpy() - g[name]) / np.linalg.norm(g[name])
        assert rel < 1e-3, (name, rel)


@pytest.mark.parametrize("scheme", ["low_rank", "gilr_gwh"])
def test_hq_linear_token_lowrank_schemes_3d(hot, scheme):
    """The token-low-rank schemes on a [B, L, I] input: projection, scales and expansion per sample;
    bit for bit against the oracle with nearest rounding, and against the reference's own 3-D run."""
    import os
    from hot_b200 import ops
    args, qm = hot
    args.transform_scheme = scheme
    args.lowRankPreset = None
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "int"
    torch.manual_seed(8)
    B, L, I, O = 3, 192, 64, 96
    lin = qm.HQ_Linear(I, O, bias=False).cuda()
    x = torch.randn(B, L, I, device="cuda") * torch.tensor([1.0, 4.0, 0.3], device="cuda").view(B, 1, 1)
    x.requires_grad_(True)
    go = torch.randn(B, L, O, device="cuda") * 1e-3 * torch.tensor([2.0, 0.5, 6.0], device="cuda").view(B, 1, 1)
    lin(x).backward(go)
    n_x, sel_x = oc.wht_selection(L, 50)
    n_w, sel_w = (n_x, sel_x) if scheme == "low_rank" else (16, np.arange(16))
    xq, sx = oc.abc_compress_batched(x.detach().cpu().numpy(), n_w, sel_w, 8, None, "int")
    wn, gon = lin.weight.detach().cpu().numpy(), go.cpu().numpy()
    ref_gx = oc.grad_input_lowrank_batched(gon, wn, n=n_x, sel=sel_x, w_mode="int")
    ref_gw = oc.linear_backward_batched(gon, wn, xq, sx, n_o=1, n_l=n_w, sel=sel_w, w_mode="int")["grad_w"]
    assert np.array_equal(x.grad.cpu().numpy(), ref_gx)
    assert np.array_equal(lin.weight.grad.cpu().numpy(), ref_gw)
    # the reference's 3-D run of this scheme (explicit noise)
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "flinearq_%s_batched.npz" % scheme))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    q = lambda bits, st, u: ops.Quant(bits, st, "noise", "tensor", 0, 0, dev(u))
    n_x, sel_x = oc.selection_from_matrix(g["lowrank"])
    n_w, sel_w = (n_x, sel_x) if scheme == "low_rank" else oc.selection_from_matrix(g["hadamard"])
    Bg, Lg, Og = g["go"].shape
    cfg = ops.LinearConfig(order_o=1, order_l=n_w, sel_l=list(sel_w), q_gw=q(8, "int8", g["u_gw"]), q_x=q(8, "int8", g["u_x"]))
    x_q_t, s_x, _ = ops.abc_compress_batched(dev(g["x"]), cfg)
    np.testing.assert_allclose(s_x.cpu().numpy(), g["scale_x"], rtol=1e-6)
    _, gw = ops.linear_backward_batched(dev(g["go"]), dev(g["w"]), x_q_t, s_x, cfg, need_gx=False)
    gx = ops.linear_backward_lowrank_gx(dev(g["go"]).view(Bg * Lg, Og), dev(g["w"]), n_x, list(sel_x), q(4, "int4", g["u_go"]),
                                        q(4, "int4", np.ascontiguousarray(g["u_w"])), batch=Bg).view(Bg, Lg, -1)
    for got, name in ((gx, "grad_input"), (gw, "grad_w")):
        rel = np.linalg.norm(got.cpu().numpy() - g[name]) / np.linalg.norm(g[name])
        assert rel < 1e-3, (name, rel)
    ref_gx = oc.grad_input_lowrank_batched(g["go"], g["w"], n=n_x, sel=sel_x, u_go=g["u_go"], u_w=g["u_w"])
    assert np.array_equal(gx.cpu().numpy(), ref_gx)


def test_hq_linear_3d_takes_one_scale_per_sample(hot):
    """Reference semantics of a [B, L, I] input (no preset): per-sample scales, per-sample low-rank
    projection, grad_weight summed over the batch; nearest rounding makes it reproducible."""
    args, qm = hot
    args.lowRankPreset = None
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "int"
    torch.manual_seed(3)
    B, L, I, O = 5, 24, 64, 96
    lin = qm.HQ_Linear(I, O, bias=False).cuda()
    x = torch.randn(B, L, I, device="cuda") * torch.tensor([1.0, 3.0, 0.5, 8.0, 2.0], device="cuda").view(B, 1, 1)
    x.requires_grad_(True)
    go = torch.randn(B, L, O, device="cuda") * 1e-3 * torch.tensor([1.0, 0.2, 6.0, 1.5, 3.0], device="cuda").view(B, 1, 1)
    lin(x).backward(go)
    n_l, sel = oc.wht_selection(L, 50)
    xq, sx = oc.abc_compress_batched(x.detach().cpu().numpy(), n_l, sel, 8, None, "int")
    ref = oc.linear_backward_batched(go.cpu().numpy(), lin.weight.detach().cpu().numpy(), xq, sx, n_o=16, n_l=n_l, sel=sel,
                                     w_mode="int")
    assert np.array_equal(x.grad.cpu().numpy(), ref["grad_input"])
    assert np.array_equal(lin.weight.grad.cpu().numpy(), ref["grad_w"])
    # the training script's defaults for the weight and the activation buffer (sawb), same 3-D call
    args.quantBWDWgt = args.quantBWDAct = "sawb"
    x.grad = None
    lin.weight.grad = None
    lin(x).backward(go)
    xq, sx = oc.abc_compress_batched(x.detach().cpu().numpy(), n_l, sel, 8, None, "sawb")
    ref = oc.linear_backward_batched(go.cpu().numpy(), lin.weight.detach().cpu().numpy(), xq, sx, n_o=16, n_l=n_l, sel=sel,
                                     w_mode="sawb")
    assert np.array_equal(x.grad.cpu().numpy(), ref["grad_input"])
    assert np.array_equal(lin.weight.grad.cpu().numpy(), ref["grad_w"])
    # all four of the training script's defaults (nq, sawb, nq, sawb): per-token / per-channel scales
    # within each sample, stochastic rounding; the gradients stay close to the exact ones
    args.quantBWDGogi = args.quantBWDGogw = "nq"
    x.grad = None
    lin.weight.grad = None
    lin(x).backward(go)
    exact_gx = go @ lin.weight.detach()
    cos = torch.nn.functional.cosine_similarity(x.grad.flatten(), exact_gx.flatten(), dim=0)
    assert torch.isfinite(lin.weight.grad).all() and float(cos) > 0.95, float(cos)
    # the batched quantiser callables: one scale per sample
    q, s = qm.int_quantizer(go, 4, True)
    assert q.shape == go.shape and s.shape == (B,)
    for b in range(B):
        rq, rs = oc.quant_tensor(go[b].cpu().numpy(), 4, None)
        assert np.array_equal(q[b].cpu().numpy(), rq.astype(np.float32)) and float(s[b]) == float(rs)
    q, s = qm.stoch_quantizer(go, 4, True)
    assert s.shape == (B,) and float((q * s.view(B, 1, 1) - go).abs().max()) <= float(s.max())
    d, one = qm.norm_quantizer(go, 4, True)
    assert one == 1. and d.shape == go.shape


def test_stochastic_backward_is_unbiased_enough(hot):
    """Against full precision the HOT gradients carry quantisation and low-rank error, not bias:
    grad_input correlates strongly with the exact one."""
    args, qm = hot
    torch.manual_seed(1)
    L, I, O = 1024, 128, 256
    lin = qm.HQ_Linear(I, O, bias=False).cuda()
    x = torch.randn(L, I, device="cuda", requires_grad=True)
    go = torch.randn(L, O, device="cuda") * 1e-3
    lin(x).backward(go)
    exact = go @ lin.weight.detach()
    cos = torch.nn.functional.cosine_similarity(x.grad.flatten(), exact.flatten(), dim=0)
    assert float(cos) > 0.85


def test_unbuilt_modes_raise(hot):
    args, qm = hot
    lin = qm.HQ_Linear(64, 64).cuda()
    x = torch.randn(32, 64, device="cuda", requires_grad=True)
    args.quantBWDAct = "luq"                                       # the logarithmic quantiser is for the grad_output sides
    with pytest.raises(NotImplementedError):
        lin(x)
    args.quantBWDAct, args.quantBWDGogi = "stoch", "sawb"       # sawb exists for W and X only
    with pytest.raises(NotImplementedError):
        lin(x).sum().backward()
    args.quantBWDGogi = "stoch"
    args.quantBWDAct = "bogus"
    with pytest.raises(Exception, match="rounding scheme not implemented"):
        lin(x)
    args.quantBWDAct = "stoch"
    args.transform_scheme = "gilro_gwh"                          # runs only with the g_w side untransformed, as in the reference
    with pytest.raises(Exception, match="Activation transform scheme not implemented: gilro_gwh"):
        lin(x)
    args.transform_scheme = "nonsense"
    with pytest.raises(Exception, match="not implemented"):
        qm.HQ_Linear(8, 8)


def test_replace_layers_and_lqs(hot):
    args, qm = hot
    from hot_b200 import lqs
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(64, 128), nn.GELU(), nn.Linear(128, 64)).cuda()
    w0 = model[0].weight
    qm.replace_layers(model, nn.Linear, qm.HQ_Linear)
    assert isinstance(model[0], qm.HQ_Linear) and isinstance(model[2], qm.HQ_Linear)
    assert model[0].weight.data_ptr() == w0.data_ptr()            # storage shared with the replaced layer
    for name, layer in model.named_modules():
        if isinstance(layer, qm.HQ_Linear):
            layer.layer_name = name
    x = torch.randn(64, 64, device="cuda")
    tgt = torch.randn(64, 64, device="cuda")
    picked = lqs.calibrate(model, [(x, tgt)], nn.functional.mse_loss)
    assert set(picked) == {"0_gx", "0_gw", "2_gx", "2_gw"}
    assert all(v in ("stoch_quantizer", "norm_quantizer") for v in picked.values())
    assert picked["0_gw"] == picked["2_gw"] == "stoch_quantizer"
    # the rule itself, on the golden cases' shapes: an outlier token flips g_x to per-token
    g = torch.randn(64, 48, device="cuda") * 1e-3
    assert lqs.select_quantizer(g)[0] == "stoch_quantizer"
    g[7] *= 30
    assert lqs.select_quantizer(g)[:2] == ("norm_quantizer", "stoch_quantizer")
    # the table drives the backward
    args.quantAuto = True
    args.layer_quant_dict["0_gx"] = "norm_quantizer"
    model.zero_grad()
    nn.functional.mse_loss(model(x), tgt).backward()
    assert torch.isfinite(model[0].weight.grad).all()


def test_hlq_backward_plugin_call(hot):
    import HLQ_backward
    torch.manual_seed(0)
    L, O, I = 784, 3072, 768                                       # 16 x 49 tokens, the harness's layer widths
    go = torch.randn(L, O, device="cuda") * 1e-3
    w = torch.randn(O, I, device="cuda") * 0.03
    x = torch.randn(L, I, device="cuda")
    for per_token in (True, False):
        gx, gw, times = HLQ_backward.backward(go, w, x, 0, 0, 16, per_token)
        assert gx.shape == (L, I) and gw.shape == (O, I) and gx.dtype == go.dtype
        assert len(times) == 4 and all(t >= 0 for t in times) and times[0] > 0 and times[2] > 0
        cos = torch.nn.functional.cosine_similarity(gx.flatten(), (go @ w).flatten(), dim=0)
        assert float(cos) > 0.85
        cosw = torch.nn.functional.cosine_similarity(gw.flatten(), (go.t() @ x).flatten(), dim=0)
        assert float(cosw) > 0.5                                   # half of the token basis is dropped
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        HLQ_backward.backward(go.cpu(), w, x, 0, 0, 16, False)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        HLQ_backward.backward(go.t().contiguous().t(), w, x, 0, 0, 16, False)
    with pytest.raises(RuntimeError, match="must be 2D"):
        HLQ_backward.backward(go[None], w, x, 0, 0, 16, False)


@pytest.mark.parametrize("per_token", [False, True])
@pytest.mark.parametrize("stochastic", [False, True])
@pytest.mark.parametrize("L", [16 * 27, 32 * 14])       # separate grad_out kernels / the fused pair
def test_hlq_backward_plugin_call_matches_the_oracle(hot, per_token, stochastic, L):
    """The plugin call composes its own launches, Philox offsets, post factors and low-rank preset:
    its fp32 gradients must equal the oracle's bit for bit, with nearest rounding and with the
    Philox streams at the offsets the call uses (8 * call number + 1..4 for grad_out/g_x, the
    weight, grad_out/g_w, the activation; weight and activation streams indexed in their stored,
    transposed layout)."""
    import HLQ_backward
    from hot_b200 import HLQ_backward as plugin
    rng = np.random.default_rng(7)
    O, I = 256, 96
    go = (rng.standard_normal((L, O)) * 1e-3).astype(np.float32)
    go[11] *= 25.0
    w = ((rng.random((O, I)) * 2 - 1) / np.sqrt(I)).astype(np.float32)
    x = rng.standard_normal((L, I)).astype(np.float32)
    x[:, 9] *= 15.0
    seed = 5
    base = (plugin._call_counter + 1) * 8
    gx, gw, times = HLQ_backward.backward(torch.from_numpy(go).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda(),
                                          0, 0, 16, per_token, seed=seed, stochastic=stochastic)
    sel = np.array(oc.lowrank_preset(16, 8))
    Lp = L // 2
    if stochastic:
        u_go = oc.philox_bytes(seed, base + 1, (L, O))
        u_w = np.ascontiguousarray(oc.philox_bytes(seed, base + 2, (I, O)).T).view(oc.PhiloxBytes)
        u_gw = oc.philox_bytes(seed, base + 3, (O, Lp))
        u_x = np.ascontiguousarray(oc.philox_bytes(seed, base + 4, (I, Lp)).T).view(oc.PhiloxBytes)
        mode = "stoch"
    else:
        u_go = u_w = u_gw = u_x = None
        mode = "int"
    xq, sx = oc.abc_compress(x, 16, sel, 8, u_x, mode)
    ref = oc.linear_backward(go, w, xq, sx, n_o=16, n_l=16, sel=sel, u_go=u_go, u_w=u_w, u_gw=u_gw,
                             gx_per_token=per_token, w_mode=mode)
    assert np.array_equal(gx.cpu().numpy(), ref["grad_input"])
    assert np.array_equal(gw.cpu().numpy(), ref["grad_w"])


@pytest.mark.parametrize("fixture,tags", [("lqs", ("flat", "outlier")), ("lqs_batched", ("spread", "outlier"))])
def test_lqs_select_quantizer_on_the_reference_cases(hot, golden, fixture, tags):
    """The product's selection on the first-batch gradients of the reference-generated cases.  With the
    recorded rounding noise: the reference's choice and its two quantisation errors to 1e-5 (the
    quantisers are bit-exact, the norm is summed in another order).  With the Philox stream: the same
    choice, and errors within the spread another draw of the noise has (one sample of 1,152 values, or a
    single outlier row of 48, carries most of an error: 10 % for the per-tensor error, 35 % for the
    per-token one).  "spread" is the case where one scale for the whole batch would give g_x to the
    per-token quantiser and the reference, with one scale per sample, does not."""
    from hot_b200 import lqs
    g = golden(fixture)
    for tag in tags:
        grad = torch.from_numpy(g[tag + "_g"]).cuda()
        noise = (torch.from_numpy(g[tag + "_u1"]).cuda(), torch.from_numpy(g[tag + "_u2"]).cuda())
        gx, gw, e_st, e_nq = lqs.select_quantizer(grad, noise=noise)
        assert (gx, gw) == (str(g[tag + "_gx"]), "stoch_quantizer"), (tag, gx, e_st, e_nq)
        np.testing.assert_allclose([e_st, e_nq], g[tag + "_errs"], rtol=1e-5)
        gx, gw, e_st, e_nq = lqs.select_quantizer(grad)
        assert (gx, gw) == (str(g[tag + "_gx"]), "stoch_quantizer"), (tag, gx, e_st, e_nq)
        np.testing.assert_allclose(e_st, g[tag + "_errs"][0], rtol=0.10)
        np.testing.assert_allclose(e_nq, g[tag + "_errs"][1], rtol=0.35)


@pytest.mark.parametrize("tag", ["patch", "c3x3"])
def test_hq_conv2d_against_the_reference(hot, golden, tag):
    """HQ_Conv2d forward + backward against the reference's own run (a stride-16 patch embedding and
    a padded 3x3 convolution, deterministic quantisers on all four operands, per-sample scales): the
    reference's transforms are BLAS matmuls, so the bound is the 1e-3 relative Frobenius error."""
    args, qm = hot
    args.lowRankPreset = None
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "int"
    g = golden("conv2d")
    B, cin, cout, hw, k, stride, pad = (int(v) for v in g[tag + "_cfg"])
    conv = qm.HQ_Conv2d(cin, cout, k, stride=stride, padding=pad).cuda()
    conv.weight.data = torch.from_numpy(g[tag + "_w"]).cuda()
    conv.bias.data = torch.from_numpy(g[tag + "_b"]).cuda()
    x = torch.from_numpy(g[tag + "_x"]).cuda().requires_grad_(True)
    y = conv(x)
    assert tuple(conv.hadamard_bs.shape) == tuple(g[tag + "_p"].shape)
    assert np.array_equal(conv.hadamard_bs.cpu().numpy().astype(np.int8), g[tag + "_p"])
    y.backward(torch.from_numpy(g[tag + "_go"]).cuda())
    for got, name in ((y.detach(), "y"), (x.grad, "gx"), (conv.weight.grad, "gw"), (conv.bias.grad, "gb")):
        want = g[tag + "_" + name]
        rel = np.linalg.norm(got.cpu().numpy() - want) / np.linalg.norm(want)
        assert rel < 1e-3, (name, rel)


@pytest.mark.parametrize("tag", ["o96", "o256"])
def test_scheme_gilro_gwh(hot, golden, tag):
    """transform_scheme "gilro_gwh": grad_input from grad_output and the weight projected along the output
    features (order 32, and order 256 = two passes of the order-64 kernel).  With the reference's recorded
    noise: bit-identical to the oracle, within 1e-3 of the reference's own run.  Through HQ_Linear with nearest
    rounding: bit-identical to the oracle; with the transforms the reference cannot run switched on, the
    reference's own exceptions."""
    args, qm = hot
    from hot_b200 import ops
    g = golden("flinearq_gilro_" + tag)
    n, sel = oc.selection_from_matrix(g["lowrank"])
    go, w, x = g["go"], g["w"], g["x"]
    L, O = go.shape
    Op = O * len(sel) // n
    pad = (-Op) % 16
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    u_go = np.pad(g["u_go"], ((0, 0), (0, pad)), constant_values=0.5)
    u_w = np.pad(g["u_w"], ((0, pad), (0, 0)), constant_values=0.5)
    q_gx = ops.Quant(4, "int4", "noise", "tensor", 0, 0, dev(u_go))
    q_w = ops.Quant(4, "int8", "noise", "tensor", 0, 0, dev(u_w))
    gx = ops.linear_backward_gilro_gx(dev(go), dev(w), n, [int(v) for v in sel], q_gx, q_w)
    ref = oc.grad_input_gilro(go, w, n=n, sel=sel, u_go=g["u_go"], u_w=g["u_w"])
    assert np.array_equal(gx.cpu().numpy(), ref["grad_input"])
    assert np.linalg.norm(gx.cpu().numpy() - g["grad_input"]) / np.linalg.norm(g["grad_input"]) < 1e-3
    # the layer
    args.transform_scheme = "gilro_gwh"
    args.lowRankPreset = None
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "int"
    lin = qm.HQ_Linear(w.shape[1], O, bias=False).cuda()
    lin.weight.data = dev(w)
    xin = dev(x).requires_grad_(True)
    with pytest.raises(Exception, match="Activation transform scheme not implemented: gilro_gwh"):
        lin(xin)
    args.TransformInput = False
    with pytest.raises(Exception, match="GradHb transform scheme not implemented: gilro_gwh"):
        lin(xin).backward(dev(go))
    args.TransformGogw = False
    lin.weight.grad = None
    xin.grad = None
    lin(xin).backward(dev(go))
    assert tuple(lin.hadamard_out.shape) == tuple(g["lowrank"].shape)
    xq, sx = oc.abc_compress(x, 1, np.array([0]), 8, None, "int")
    want_gx = oc.grad_input_gilro(go, w, n=n, sel=sel, w_mode="int")["grad_input"]
    want_gw = oc.linear_backward(go, w, xq, sx, n_o=1, n_l=1, sel=np.array([0]), w_mode="int")["grad_w"]
    assert np.array_equal(xin.grad.cpu().numpy(), want_gx)
    assert np.array_equal(lin.weight.grad.cpu().numpy(), want_gw)


def test_token_basis_of_order_128(hot, golden):
    """384 tokens give make_WHT an order-128 basis (36 rows): above what one kernel launch transforms, so
    the projection runs as two passes (64-point, then 2-point butterflies on rows 64 apart) and the projected
    rows are quantised as they are.  Bit-identical to the oracle with the recorded noise, within 1e-3 of the
    reference's run; and through HQ_Linear, which derives the basis from the live token count."""
    args, qm = hot
    from hot_b200 import ops
    g = golden("flinearq_lr_ref128")
    n_l, sel = oc.selection_from_matrix(g["p"])
    x, w, go = g["x"], g["w"], g["go"]
    L, I = x.shape
    O = w.shape[0]
    Lp = L // n_l * len(sel)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    q = lambda bits, storage, u: ops.Quant(bits, storage, "noise", "tensor", 0, 0, dev(u))
    cfg = ops.LinearConfig(order_o=16, order_l=n_l, sel_l=[int(v) for v in sel], q_gx=q(4, "int4", g["u_go"]),
                           q_w=q(4, "int4", g["u_w"]), q_gw=q(8, "int8", g["u_gw"]), q_x=q(8, "int8", g["u_x"]))
    x_q_t, s_x = ops.abc_compress(dev(x), cfg)
    gx, gw = ops.linear_backward(dev(go), dev(w), x_q_t, s_x, cfg)
    xq_ref, sx_ref = oc.abc_compress(x, n_l, sel, 8, g["u_x"])
    ref = oc.linear_backward(go, w, xq_ref, sx_ref, n_o=16, n_l=n_l, sel=sel, u_go=g["u_go"], u_w=g["u_w"], u_gw=g["u_gw"])
    assert np.array_equal(x_q_t.cpu().numpy().view(np.int8).astype(np.int32)[:, :Lp].T, xq_ref)
    assert np.array_equal(gx.cpu().numpy(), ref["grad_input"]) and np.array_equal(gw.cpu().numpy(), ref["grad_w"])
    for got, name in ((gx, "grad_input"), (gw, "grad_w")):
        assert np.linalg.norm(got.cpu().numpy() - g[name]) / np.linalg.norm(g[name]) < 1e-3, name
    args.lowRankPreset = None
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "int"
    lin = qm.HQ_Linear(I, O, bias=False).cuda()
    lin.weight.data = dev(w)
    xin = dev(x).requires_grad_(True)
    lin(xin).backward(dev(go))
    assert tuple(lin.hadamard_bs.shape) == (36, 128)
    xq_i, sx_i = oc.abc_compress(x, n_l, sel, 8, None, "int")
    ref_i = oc.linear_backward(go, w, xq_i, sx_i, n_o=16, n_l=n_l, sel=sel, w_mode="int")
    assert np.array_equal(xin.grad.cpu().numpy(), ref_i["grad_input"])
    assert np.array_equal(lin.weight.grad.cpu().numpy(), ref_i["grad_w"])
    # a 3-D input whose per-sample length has a 2-adic part above 64: one scale per sample, same projection
    x3 = torch.randn(2, 256, I, device="cuda", requires_grad=True)
    lin(x3).backward(torch.randn(2, 256, O, device="cuda") * 1e-3)
    assert tuple(lin.hadamard_bs.shape)[1] == 256 and torch.isfinite(x3.grad).all() and torch.isfinite(lin.weight.grad).all()


def test_luq_quantizer_and_layer(hot, golden):
    """The logarithmic quantiser against the reference's own run with the same two uniform draws (levels and
    scale; a level can differ where log2 lands on a power of two, hence the 1e-3 allowance), and FLinearQ with it
    on both grad_output sides (4-bit: at 8 bits the reference's scale expression overflows, and so does this one)."""
    args, qm = hot
    g = golden("luq")
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    for bits in (3, 4):
        lv, s = qm.luq_quantizer(dev(g["x"]), bits, False, noise=(dev(g["u_prune"]), dev(g["u_round"])))
        np.testing.assert_allclose(float(s), float(g["luq%d_scale" % bits]), rtol=1e-6)
        assert np.mean(lv.cpu().numpy() != g["luq%d_levels" % bits]) < 1e-3
    lv, s = qm.luq_quantizer(dev(g["x"]).reshape(4, 10, 64), 4, True)                   # batched: one scale per sample
    assert lv.shape == (4, 10, 64) and s.shape == (4,)
    assert set(np.unique(np.abs(lv.cpu().numpy()))) <= {0.0} | {2.0 ** k for k in range(0, 12)}
    with pytest.raises(OverflowError):
        qm.luq_quantizer(dev(g["x"]), 8, False)
    assert qm.quant_scheme_dict["luq_quantizer"] is qm.luq_quantizer
    # the layer: explicit draws through the two helpers the backward uses
    from hot_b200 import ops
    x, w, go = g["l_x"], g["l_w"], g["l_go"]
    n_l, sel = oc.selection_from_matrix(g["l_p"])
    q = lambda bits, storage, u: ops.Quant(bits, storage, "noise", "tensor", 0, 0, dev(u))
    cfg = ops.LinearConfig(order_o=16, order_l=n_l, sel_l=[int(v) for v in sel], q_x=q(8, "int8", g["l_u_x"]))
    x_q_t, s_x = ops.abc_compress(dev(x), cfg)
    gx = qm._luq_grad_input(dev(go), dev(w), 16, q(4, "int8", g["l_u_w"]), 4, False, noise=(dev(g["l_ug1"]), dev(g["l_ug2"])))
    gw = qm._luq_grad_weight(dev(go), x_q_t, s_x, n_l, [int(v) for v in sel], 4, False, torch.float32,
                             noise=(dev(g["l_uw1"]), dev(g["l_uw2"])))
    for got, name in ((gx, "l_grad_input"), (gw, "l_grad_w")):
        rel = np.linalg.norm(got.cpu().numpy() - g[name]) / np.linalg.norm(g[name])
        assert rel < 2e-3, (name, rel)
    # and through the module, 2-D and 3-D, with its own draws
    args.quantBWDGogi = args.quantBWDGogw = "luq"
    args.GogwQuantBit = 4
    lin = qm.HQ_Linear(w.shape[1], w.shape[0], bias=False).cuda()
    lin.weight.data = dev(w)
    xin = dev(x).requires_grad_(True)
    lin(xin).backward(dev(go))
    fp_gx, fp_gw = dev(go) @ dev(w), dev(go).t() @ dev(x)
    assert float(torch.nn.functional.cosine_similarity(xin.grad.flatten(), fp_gx.flatten(), dim=0)) > 0.8
    assert float(torch.nn.functional.cosine_similarity(lin.weight.grad.flatten(), fp_gw.flatten(), dim=0)) > 0.5
    args.lowRankPreset = None
    x3 = torch.randn(3, 32, w.shape[1], device="cuda", requires_grad=True)
    lin.weight.grad = None
    lin(x3).backward(torch.randn(3, 32, w.shape[0], device="cuda") * 1e-3)
    assert torch.isfinite(x3.grad).all() and torch.isfinite(lin.weight.grad).all()


def test_hq_linear_bf16_bias_goes_into_the_forward_gemm(hot):
    """In 16-bit dtypes HQ_Linear hands its bias to FLinearQ: the forward is F.linear(x, w, b) (what nn.Linear
    computes), the bias gradient is the sum of grad_output over the tokens, and the other two gradients are the HOT
    ones (close to the float gradients, as in the layer tests above)."""
    args, qm = hot
    args.transform_scheme = "gih_gwlr"
    args.lowRankPreset = "half16"
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "stoch"
    torch.manual_seed(3)
    layer = qm.HQ_Linear(96, 128).cuda().to(torch.bfloat16)
    x = torch.randn(4, 64, 96, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    go = (torch.randn(4, 64, 128, device="cuda") * 1e-2).to(torch.bfloat16)
    out = layer(x)
    assert torch.equal(out, nn.functional.linear(x, layer.weight, layer.bias))
    out.backward(go)
    torch.testing.assert_close(layer.bias.grad.float(), go.float().sum((0, 1)), rtol=2e-2, atol=1e-3)
    cos = lambda a, b: float(nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0))
    assert cos(x.grad, go.float() @ layer.weight.float()) > 0.9
    # (the low-rank projection keeps 8 of 16 token directions: on white noise that is half the energy, cos ~ 0.71)
    assert cos(layer.weight.grad, go.float().reshape(-1, 128).t() @ x.detach().float().reshape(-1, 96)) > 0.6
    # float32 keeps the separate addition
    layer32 = qm.HQ_Linear(96, 128).cuda()
    x32 = torch.randn(256, 96, device="cuda")
    assert torch.equal(layer32(x32), nn.functional.linear(x32, layer32.weight) + layer32.bias)


def test_vit_with_hot_linears_trains(hot):
    """A small ViT of the benchmark's architecture: apply_hot swaps exactly the block linears, a few
    SGD steps on a fixed batch reduce the loss, and gradients reach every parameter."""
    args, qm = hot
    from hot_b200.vit import VisionTransformer, apply_hot
    torch.manual_seed(0)
    model = VisionTransformer(img_size=64, patch=16, dim=64, depth=2, heads=4, num_classes=10).cuda()
    assert apply_hot(model) == 8
    assert isinstance(model.blocks[0].attn.qkv, qm.HQ_Linear) and model.blocks[1].mlp.fc2.layer_name == "blocks.1.mlp.fc2"
    assert type(model.head) is nn.Linear
    x = torch.randn(32, 3, 64, 64, device="cuda")            # 32 x 17 tokens = 544 = 16 * 34
    y = torch.randint(0, 10, (32,), device="cuda")
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    losses = []
    for _ in range(12):
        opt.zero_grad()
        loss = nn.functional.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    assert losses[-1] < losses[0] - 0.1, losses


def test_sawb_for_weight_and_activation(hot, golden):
    """The reference's default quantiser for W and X (ViT_main.py:102,104).  The clip value comes
    from two means whose summation order differs from torch's, so the scale is compared to 1e-6
    and the codes may differ in a vanishing fraction."""
    args, qm = hot
    g = golden("quantizers")
    x = torch.from_numpy(g["x"]).cuda()
    for bits in (4, 8):
        codes, s = qm.sawb_quantizer(x, bits, False)
        np.testing.assert_allclose(float(s), float(g["sawb%d_scale" % bits]), rtol=1e-6)
        assert np.mean(codes.cpu().numpy() != g["sawb%d_codes" % bits]) < 1e-3
    args.quantBWDWgt = args.quantBWDAct = "sawb"
    args.quantBWDGogi = args.quantBWDGogw = "int"
    torch.manual_seed(3)
    L, I, O = 512, 96, 128
    lin = qm.HQ_Linear(I, O, bias=False).cuda()
    xin = torch.randn(L, I, device="cuda", requires_grad=True)
    go = torch.randn(L, O, device="cuda") * 1e-3
    lin(xin).backward(go)
    sel = np.array(oc.lowrank_preset(16, 8))
    xq, sx = oc.abc_compress(xin.detach().cpu().numpy(), 16, sel, 8, None, "sawb")
    ref = oc.linear_backward(go.cpu().numpy(), lin.weight.detach().cpu().numpy(), xq, sx, n_o=16, n_l=16, sel=sel,
                             w_mode="sawb")
    for got, name in ((xin.grad, "grad_input"), (lin.weight.grad, "grad_w")):
        rel = np.linalg.norm(got.cpu().numpy() - ref[name]) / np.linalg.norm(ref[name])
        assert rel < 1e-3, (name, rel)
    # deterministic: the same call twice gives the same bytes
    a1, s1, n1 = hot_ops().col_ht_quant(xin.detach(), 16, list(sel), hot_ops().Quant(8, "int8", "nearest", "sawb"))
    a2, s2, _ = hot_ops().col_ht_quant(xin.detach(), 16, list(sel), hot_ops().Quant(8, "int8", "nearest", "sawb"))
    assert torch.equal(a1[:, :n1], a2[:, :n1]) and torch.equal(s1, s2)


def hot_ops():
    from hot_b200 import ops
    return ops


def test_hq_conv2d_matches_its_linear_form(hot):
    """HQ_Conv2d is im2col + the same FLinearQ: with nearest rounding its gradients equal those of an
    HQ_Linear fed the unfolded input, and its forward equals nn.Conv2d."""
    args, qm = hot
    args.quantBWDGogi = args.quantBWDWgt = args.quantBWDGogw = args.quantBWDAct = "int"
    torch.manual_seed(0)
    conv = qm.HQ_Conv2d(4, 32, kernel_size=4, stride=4).cuda()          # 4*4*4 = 64 input features per patch
    x = torch.randn(8, 4, 16, 16, device="cuda", requires_grad=True)     # 16 patches per image, 128 tokens
    y = conv(x)
    ref = torch.nn.functional.conv2d(x, conv.weight, conv.bias, stride=4)
    assert y.shape == ref.shape and torch.allclose(y, ref, atol=1e-5)
    go = torch.randn_like(y) * 1e-3
    y.backward(go)
    lin = qm.HQ_Linear(64, 32).cuda()
    lin.weight.data = conv.weight.data.view(32, 64).clone()
    lin.bias.data = conv.bias.data.clone()
    cols = torch.nn.functional.unfold(x.detach(), 4, stride=4).transpose(1, 2).reshape(-1, 64).requires_grad_(True)
    lin(cols).backward(go.flatten(2).transpose(1, 2).reshape(-1, 32))
    assert torch.equal(conv.weight.grad.view(32, 64), lin.weight.grad)
    gx_cols = cols.grad.reshape(8, 16, 64).transpose(1, 2)
    assert torch.allclose(x.grad, torch.nn.functional.fold(gx_cols, (16, 16), 4, stride=4), atol=1e-7)
    model = nn.Sequential(nn.Conv2d(3, 16, 3, padding=1), nn.Conv2d(16, 16, 3, groups=16)).cuda()
    qm.replace_layers(model, nn.Conv2d, qm.HQ_Conv2d)
    assert isinstance(model[0], qm.HQ_Conv2d) and type(model[1]) is nn.Conv2d      # depth-wise stays as it is
    with pytest.raises(NotImplementedError):
        qm.HQ_Conv2d(16, 16, 3, groups=16).cuda()(torch.randn(16, 16, 8, 8, device="cuda"))
