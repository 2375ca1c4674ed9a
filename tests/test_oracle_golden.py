"""Checks the plain-C++ oracle bit-for-bit against fixtures produced by the reference's own
operator templates (tests/golden/make_golden.py). Runs everywhere, with or without the reference."""
import os

import numpy as np
import pytest

import oracle

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_ops.npz"))


def same(a, b):
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    if a.dtype == np.float32:
        a, b = a.view(np.uint32), b.view(np.uint32)
    assert np.array_equal(a, b)


def test_quant():
    q, s = oracle.quant_per_token(G["quant_x"])
    same(q, G["quant_q"]); same(s, G["quant_s"])
    assert s[3] == 1.0 and not q[3].any()


def test_gemm_dequant():
    acc = oracle.gemm_s8s8(G["gemm_a"], G["gemm_w"])
    same(acc, G["gemm_acc"])
    same(oracle.dequant(acc, G["deq_st"], G["deq_sc"]), G["deq_y"])
    same(oracle.gemm_u8s8(G["gemmu_a"], G["gemmu_w"]), G["gemmu_acc"])
    a2, y2 = oracle.linear_i8(G["gemm_a"], G["deq_st"], G["gemm_w"], G["deq_sc"])
    same(a2, G["gemm_acc"]); same(y2, G["deq_y"])


def test_fht():
    same(oracle.fht(G["fht64_x"], 8.0), G["fht64_y"])
    same(oracle.fht(G["fht8192_x"], 90.50966799), G["fht8192_y"])


def test_rope():
    x = G["rope_x"]
    same(oracle.rope(x, np.arange(x.shape[0]), G["rope_cos"], G["rope_sin"]), G["rope_y"])


def test_softmax():
    x = G["softmax_x"]
    same(oracle.softmax(x), G["softmax_full"])
    same(oracle.softmax(x, np.arange(1, x.shape[0] + 1)), G["softmax_causal"])
    same(oracle.softmax(G["softmax_dec_x"][None])[0], G["softmax_dec_p"])


def test_rmsnorm():
    x, gm = G["rms_x"], G["rms_gamma"]
    same(oracle.rmsnorm(x, gm, lanes=0), G["rms_prefill"])
    same(oracle.rmsnorm(x, gm, lanes=4), G["rms_dec4"])
    same(oracle.rmsnorm(x, gm, lanes=8), G["rms_dec8"])
    # the two phases really do use different summation orders
    assert not np.array_equal(G["rms_prefill"].view(np.uint32), G["rms_dec8"].view(np.uint32))


def test_elementwise():
    same(oracle.silu(G["silu_x"]), G["silu_y"])
    same(oracle.silu_mul(G["silu_x"], G["silu_u"]), G["silu_mul_y"])
    same(oracle.residual(G["silu_x"], G["silu_u"]), G["residual_y"])


def test_static_quant():
    same(oracle.static_quant(G["sq_x"], 0.01, 8.0, True), G["sq_signed"])
    same(oracle.static_quant(G["sq_p"], 1 / 255, 1.0, False), G["sq_unsigned"])
    assert G["sq_unsigned"].max() == 255


def test_argmax():
    same(oracle.argmax(G["argmax_x"]), G["argmax_i"])
    assert G["argmax_i"][1] == 77
