"""CPU-side checks of the boundary: the shared library loads without a GPU and exports every
symbol include/hot_b200.h declares; argument errors are reported without touching a device."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def cabi():
    from hot_b200 import build
    build.build()
    from hot_b200 import _cabi
    return _cabi


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "hot_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hot_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(cabi):
    lib = ctypes.CDLL(cabi.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), "missing export: " + n
    assert sorted(cabi.EXPORTS) == names, "ctypes table and header disagree"
    assert cabi.lib().hot_abi_version() >= 1
    assert cabi.lib().hot_status_string(cabi.HOT_ERR_TIMEOUT) == b"bounded device-side wait ran out"


def test_argument_errors_need_no_device(cabi):
    lib = cabi.lib()
    q = cabi.HotQuant(9, 0, 0, 0, 0, 0, None)
    buf = (ctypes.c_uint8 * 256)()
    p = ctypes.addressof(buf)
    rc = lib.hot_row_ht_quant(p, 0, 4, 64, 64, 16, ctypes.byref(q), p, 64, p, p, None)
    assert rc == cabi.HOT_ERR_ARG and b"bits" in lib.hot_last_error()
    q.bits = 4
    rc = lib.hot_row_ht_quant(p, 0, 4, 56, 64, 4, ctypes.byref(q), p, 64, p, p, None)
    assert rc == cabi.HOT_ERR_UNSUPPORTED
    rc = lib.hot_gemm_i8(None, 0, 16, p, 0, 16, 1, 1, 1, p, 0, p, 0, 1.0, p, 0, 1, None, None)
    assert rc == cabi.HOT_ERR_ARG
    cfg = cabi.HotLinearCfg()
    cfg.order_o, cfg.order_l, cfg.rank_l = 16, 16, 8
    assert lib.hot_linear_workspace_bytes(6304, 3072, 768, ctypes.byref(cfg)) > 6304 * 1536
    assert lib.hot_linear_workspace_bytes(6300, 3072, 768, ctypes.byref(cfg)) == 0      # tokens % 16 != 0
    assert lib.hot_abc_pitch(6304, ctypes.byref(cfg)) == 3152


def test_status_word_and_wait_limit(cabi):
    """The status word's host side needs no device: 0 is HOT_OK, any bit is HOT_ERR_TIMEOUT and the message
    names the kernels; the wait limit has a setter, and the probe refuses to run with a long limit."""
    C, lib = cabi, cabi.lib()
    assert lib.hot_check_status(0) == C.HOT_OK
    assert lib.hot_check_status(1 | 4) == C.HOT_ERR_TIMEOUT
    msg = lib.hot_last_error().decode()
    assert "integer GEMM" in msg and "tensor-core grad_out" in msg and "0x5" in msg and "wait probe" not in msg
    assert lib.hot_check_status(8) == C.HOT_ERR_TIMEOUT and "wait probe" in lib.hot_last_error().decode()
    assert lib.hot_get_wait_limit_ns() == 1500 * 1000 * 1000
    lib.hot_set_wait_limit_ns(2_000_000)
    assert lib.hot_get_wait_limit_ns() == 2_000_000
    lib.hot_set_wait_limit_ns(0)
    assert lib.hot_get_wait_limit_ns() == 1500 * 1000 * 1000
    import ctypes
    word = ctypes.c_uint32(0)
    assert lib.hot_wait_probe(ctypes.byref(word), None) == C.HOT_ERR_ARG        # limit too long for a probe
    assert "at most 100 ms" in lib.hot_last_error().decode()


def test_host_modules_without_a_device():
    import hot_b200.hadamard_matmul as hm
    g = np.load(os.path.join(ROOT, "tests", "golden", "transforms.npz"))
    for n in (1, 2, 16, 64):
        assert np.array_equal(hm.hadamard(n), g["hadamard_%d" % n])
    for size, pct in g["wht_cases"]:
        assert np.array_equal(hm.make_WHT(int(size), int(pct)), g["wht_%d_%d" % (size, pct)])
    assert [hm.biggest_power2_factor_max16(int(s)) for s in g["make_hadamard_sizes"]] == list(g["pow2_max16"])
    td = hm.Transform_Dict()
    assert td.get_or_register("hadamard", 3072).shape == (16, 16)
    assert td.get_or_register("low_rank", 6304, 50).shape == (10, 32)
    with pytest.raises(NotImplementedError):
        td.get_or_register("haar", 8)
    assert hm.selection_from_matrix(hm.make_WHT(160, 50)) == hm.wht_selection(160, 50)
    with pytest.raises(ValueError):
        hm.selection_from_matrix(np.ones((2, 6)))
    import torch
    from hot_b200 import ops
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.row_ht_quant(torch.zeros(4, 64), 16, ops.Quant(4, "int4"))
    # how the host layers store the 4-bit g_x codes: one per byte below a contraction of 4096, packed from there on
    assert [ops.gx_code_storage(4, k) for k in (768, 2304, 3072, 4095, 4096, 11008)] == ["int8"] * 4 + ["int4"] * 2
    assert ops.gx_code_storage(8, 11008) == "int8"
    # FLinearQ takes the bias as an optional sixth argument and runs on CPU as far as its forward product
    from hot_b200.quant_matmul import FLinearQ
    import inspect
    assert list(inspect.signature(FLinearQ.forward).parameters)[:7] == ["ctx", "x", "w", "h_out", "h_bs", "name", "bias"]
