"""GPU parity of every operator against the CPU oracle, through the C ABI.

Bar: every output bit-exact (integers, int8 and fp32 alike) against the oracle evaluated with the
correctly rounded expf, which is what the kernels compute; against the oracle evaluated with the
build machine's libm expf (last-bit rounding left open by the C standard) the fp32 results that
pass through exp() agree to one ulp and the mismatch counts are printed.
"""
import numpy as np
import pytest
import torch

import oracle
from util import assert_same, max_abs_rel, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _correctly_rounded_exp():
    """The CUDA kernels evaluate the correctly rounded expf; pin them against the oracle in the same
    mode (bit for bit). Tests that quantify the distance to the build machine's libm switch modes
    themselves."""
    with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
        yield
TOL = 1e-3  # max-abs-rel tolerance for fp32 outputs that pass through exp()


@pytest.fixture(scope="module")
def F():
    import flexllm_b200
    flexllm_b200.lib()  # raises if the CUDA library is missing
    return flexllm_b200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rng(seed):
    return np.random.default_rng(seed)


# ------------------------------------------------------------------------------ quant / dequant
@pytest.mark.parametrize("M,K", [(1, 64), (7, 2048), (128, 2048), (5, 8192), (33, 512)])
def test_quant_per_token(F, M, K):
    x = (rng(1).standard_normal((M, K)) * 3).astype(np.float32)
    if M > 2:
        x[1] = 0
    q, s = F.pref_quant_layer_fp32_qint(dev(x))
    qo, so = oracle.quant_per_token(x)
    assert_same(to_np(s), so, "scale"); assert_same(to_np(q), qo, "q")


def test_quant_empty(F):
    q, s = F.pref_quant_layer_fp32_qint(torch.empty((0, 64), device="cuda"))
    assert q.shape == (0, 64)


def test_dequant(F):
    g = rng(2)
    acc = g.integers(-2**27, 2**27, (37, 512), dtype=np.int32)
    st = g.uniform(0.005, 0.05, 37).astype(np.float32); sc = g.uniform(0.001, 0.01, 512).astype(np.float32)
    y = F.pref_dequant_layer_qint_fp32(dev(acc), dev(st), dev(sc))
    assert_same(to_np(y), oracle.dequant(acc, st, sc))


def test_static_quant(F):
    g = rng(3)
    x = (g.standard_normal((9, 64)) * 2).astype(np.float32)
    s1 = np.array([0.01], np.float32)
    assert_same(to_np(F.pref_static_sym_quant_layer_fp32_qint(dev(x), dev(s1), 8.0, True)),
                oracle.static_quant(x, s1, 8.0, True))
    p = g.uniform(0, 1.3, (9, 64)).astype(np.float32)
    s2 = np.array([1 / 255], np.float32)
    assert_same(to_np(F.pref_static_sym_quant_layer_fp32_qint(dev(p), dev(s2), 1.0, False)),
                oracle.static_quant(p, s2, 1.0, False))
    sr = g.uniform(0.005, 0.05, 9).astype(np.float32)
    assert_same(to_np(F.pref_static_sym_quant_layer_fp32_qint(dev(x), dev(sr), 1.0, True)),
                oracle.static_quant(x, sr, 1.0, True))


# ------------------------------------------------------------------------------ FHT
@pytest.mark.parametrize("N,scale,rows", [(64, 8.0, 50), (2, 1.0, 3), (256, 16.0, 5), (8192, 90.50966799, 4), (4096, 64.0, 2)])
def test_fht(F, N, scale, rows):
    x = rng(4).standard_normal((rows, N)).astype(np.float32)
    y = F.pref_FHT(dev(x), scale)
    assert_same(to_np(y), oracle.fht(x, scale))


def test_fht_golden(F):
    import os
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_ops.npz"))
    assert_same(to_np(F.pref_FHT(dev(G["fht8192_x"]), 90.50966799)), G["fht8192_y"])
    assert_same(to_np(F.pref_FHT(dev(G["fht64_x"]), 8.0)), G["fht64_y"])


def test_swiglu_fht_quant(F):
    g_ = rng(5)
    M = 6
    g = (g_.standard_normal((M, 8192)) * 2).astype(np.float32); u = g_.standard_normal((M, 8192)).astype(np.float32)
    q, s, act = F.swiglu_fht_quant(dev(g), dev(u), want_act=True)
    act_o = oracle.silu_mul(g, u)
    assert_same(to_np(act), act_o, "silu(g)*u")
    qo, so = oracle.quant_per_token(oracle.fht(act_o, 90.50966799))
    assert_same(to_np(s), so, "scale"); assert_same(to_np(q), qo, "q")
    # distance to the libm flavour of the oracle: last-bit differences in act, +-1 at rounding ties in q
    with oracle.exp_mode(oracle.EXP_LIBM):
        act_l = oracle.silu_mul(g, u)
        ql, _ = oracle.quant_per_token(oracle.fht(act_l, 90.50966799))
    nbad = np.count_nonzero(act_l.view(np.uint32) != act_o.view(np.uint32))
    d = np.abs(to_np(q).astype(np.int32) - ql.astype(np.int32))
    print(f"vs libm expf: {nbad}/{act_o.size} fp32 values differ in the last bit, {np.count_nonzero(d)}/{d.size} int8 differ")
    assert max_abs_rel(act_l, act_o) < 1e-6 and d.max() <= 1


# ------------------------------------------------------------------------------ RoPE / qk_prepare
def test_rope(F):
    g = rng(6)
    cos_t, sin_t = oracle.rope_table(2048)
    T, H = 70, 5
    x = g.standard_normal((T, H, 64)).astype(np.float32); pos = g.integers(0, 2048, T).astype(np.int32)
    y = F.pref_RoPE_layer(dev(x), dev(pos), dev(cos_t), dev(sin_t))
    assert_same(to_np(y), oracle.rope(x, pos, cos_t, sin_t))


@pytest.mark.parametrize("T,H", [(1, 8), (100, 32), (33, 1)])
def test_qk_prepare(F, T, H):
    g = rng(7)
    cos_t, sin_t = oracle.rope_table(8200)
    q = g.integers(-127, 128, (T, H, 64), dtype=np.int8); s = g.uniform(0.005, 0.05, (T, H)).astype(np.float32)
    pos = g.integers(0, 8200, T).astype(np.int32)
    q2, s2 = F.qk_prepare(dev(q), dev(s), dev(pos), dev(cos_t), dev(sin_t))
    qo, so, _ = oracle.qk_prepare(q, s, pos, cos_t, sin_t)
    assert_same(to_np(s2), so, "scale"); assert_same(to_np(q2), qo, "q")


# ------------------------------------------------------------------------------ softmax
def test_softmax(F):
    g = rng(8)
    for rows, L in [(16, 64), (3, 1), (5, 1027), (2, 8193)]:
        x = (g.standard_normal((rows, L)) * 4).astype(np.float32)
        p = to_np(F.pref_Softmax(dev(x)))
        assert_same(p, oracle.softmax(x))
        assert np.abs(p.sum(-1) - 1).max() < 1e-5
        with oracle.exp_mode(oracle.EXP_LIBM):
            assert max_abs_rel(p, oracle.softmax(x)) < 1e-6
    x = (g.standard_normal((24, 24)) * 4).astype(np.float32)
    valid = np.arange(1, 25, dtype=np.int32)
    p = to_np(F.pref_Softmax(dev(x), dev(valid)))
    assert_same(p, oracle.softmax(x, valid))
    assert (np.triu(p, 1) == 0).all()


def test_softmax_summation_order_is_the_reference(F):
    """With exp() taken out of the picture (inputs whose exp is exact: x = max or masked), the row
    sum and the scaling are bit-exact."""
    L = 64
    x = np.full((1, L), -1e32, np.float32)
    x[0, [0, 5, 6, 63]] = 2.5          # four ones after exp, the rest exactly zero
    p = to_np(F.pref_Softmax(dev(x)))
    assert_same(p, oracle.softmax(x))


# ------------------------------------------------------------------------------ RMSNorm
@pytest.mark.parametrize("order", [0, 4, 8])
@pytest.mark.parametrize("M", [1, 64, 130])
def test_rmsnorm_quant(F, order, M):
    g = rng(9)
    x = g.standard_normal((M, 2048)).astype(np.float32); gamma = (1 + 0.02 * g.standard_normal(2048)).astype(np.float32)
    y, q, s = F.pref_Layer_Norm(dev(x), dev(gamma), 1e-5, order, quant=True)
    yo = oracle.rmsnorm(x, gamma, 1e-5, order)
    assert_same(to_np(y), yo, "y")
    qo, so = oracle.quant_per_token(yo)
    assert_same(to_np(s), so, "s"); assert_same(to_np(q), qo, "q")


def test_rmsnorm_golden(F):
    import os
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_ops.npz"))
    x, gm = dev(G["rms_x"]), dev(G["rms_gamma"])
    assert_same(to_np(F.pref_Layer_Norm(x, gm, 1e-5, 0)), G["rms_prefill"])
    assert_same(to_np(F.pref_Layer_Norm(x, gm, 1e-5, 8)), G["rms_dec8"])
    assert_same(to_np(F.pref_Layer_Norm(x, gm, 1e-5, 4)), G["rms_dec4"])


# ------------------------------------------------------------------------------ elementwise
def test_elementwise(F):
    g = rng(10)
    a = (g.standard_normal(10007) * 4).astype(np.float32); b = g.standard_normal(10007).astype(np.float32)
    a4, b4 = a[:10004], b[:10004]
    assert_same(to_np(F.pref_Gate_Layer_fp32xfp32(dev(a4), dev(b4))), a4 * b4)
    assert_same(to_np(F.pref_Residual_Layer(dev(a4), dev(b4))), oracle.residual(a4, b4))
    assert_same(to_np(F.pref_Residual_Layer(dev(a), dev(b))), oracle.residual(a, b))   # ragged tail
    sw = to_np(F.pref_Swish(dev(a)))
    assert_same(sw, oracle.silu(a))
    with oracle.exp_mode(oracle.EXP_LIBM):
        so = oracle.silu(a)
    ulp = np.abs(sw.view(np.int32).astype(np.int64) - so.view(np.int32).astype(np.int64))
    print(f"silu vs libm expf: {np.count_nonzero(ulp)}/{ulp.size} differ, max {ulp.max()} ulp")
    assert ulp.max() <= 2


def test_exp_dense(F):
    """The device exponential is the correctly rounded one: silu and 2-element softmax rows over
    millions of arguments, including the ranges where the fast path hands over (|x| >= 80), where
    exp overflows fp32 and where its result is subnormal."""
    g = rng(12)
    a = np.concatenate([g.uniform(-110, 110, 3_000_000), g.uniform(-1, 1, 500_000), g.standard_normal(500_000) * 8,
                        [0.0, -0.0, 79.99999, 80.0, -80.0, 88.72, 88.73, -87.3, -87.4, -103.9, -104.0, -150.0, 200.0]]).astype(np.float32)
    assert_same(to_np(F.pref_Swish(dev(a))), oracle.silu(a))
    x = np.zeros((a.size, 2), np.float32)
    x[:, 1] = -np.abs(a)
    assert_same(to_np(F.pref_Softmax(dev(x))), oracle.softmax(x))


def test_argmax(F):
    g = rng(11)
    l = g.standard_normal((5, 128256)).astype(np.float32)
    l[1, 77] = l[1, 100000] = 9.0
    l[2, :] = -3.0
    l[3, 128255] = 10.0
    idx = to_np(F.dec_Logits_argmax(dev(l)))
    assert_same(idx, oracle.argmax(l))
    assert idx[1] == 77 and idx[2] == 0 and idx[3] == 128255


# ------------------------------------------------------------------------------ linear layers
def lin_inputs(M, N, K, seed):
    g = rng(seed)
    a = g.integers(-127, 128, (M, K), dtype=np.int8); w = g.integers(-127, 128, (N, K), dtype=np.int8)
    st = g.uniform(0.005, 0.05, M).astype(np.float32); sc = g.uniform(0.001, 0.01, N).astype(np.float32)
    return a, st, w, sc


@pytest.mark.parametrize("M,N,K", [(1, 2048, 2048), (1, 8192, 2048), (1, 2048, 8192), (3, 512, 2048), (8, 64, 128),
                                   (5, 24, 64),
                                   # every token-count variant on wide and narrow matrices (whole-K warps and the K split over
                                   # the four warps of a CTA)
                                   (2, 16384, 2048), (4, 8192, 2048), (8, 2048, 8192), (7, 3072, 2048), (1, 4104, 1024), (3, 1032, 2048),
                                   (2, 9000, 640), (8, 16384, 2048), (1, 304, 8192), (6, 2056, 1152)])
def test_linear_decode_gemv(F, M, N, K):
    a, st, w, sc = lin_inputs(M, N, K, 20)
    acc, y = F.dec_Linear_Layer_i8xi8(dev(a), dev(st), dev(w), dev(sc), want_acc=True)
    acc_o, y_o = oracle.linear_i8(a, st, w, sc)
    assert_same(to_np(acc), acc_o, "acc"); assert_same(to_np(y), y_o, "y")


@pytest.mark.parametrize("M,N,K", [(128, 2048, 2048),      # the single prefill linear layer of the reference's own bench
                                   (128, 256, 128), (256, 512, 256), (100, 264, 144), (1, 16, 16), (300, 2048, 8192),
                                   (130, 128, 2048), (64, 64, 512), (17, 40, 1040)])
def test_linear_prefill_tcgen05(F, M, N, K):
    a, st, w, sc = lin_inputs(M, N, K, 21)
    acc, y = F.pref_Linear_Layer_i8xi8(dev(a), dev(st), dev(w), dev(sc), want_acc=True)
    torch.cuda.synchronize()
    acc_o, y_o = oracle.linear_i8(a, st, w, sc)
    assert_same(to_np(acc), acc_o, "acc"); assert_same(to_np(y), y_o, "y")


def test_linear_prefill_extremes(F):
    """Largest accumulator magnitude the path can see: |a|=|w|=128... here -128 * -128 * 8192."""
    M, N, K = 128, 128, 8192
    a = np.full((M, K), -128, np.int8); w = np.full((N, K), -128, np.int8)
    st = np.ones(M, np.float32); sc = np.ones(N, np.float32)
    acc, _ = F.pref_Linear_Layer_i8xi8(dev(a), dev(st), dev(w), dev(sc), want_acc=True)
    assert (to_np(acc) == 128 * 128 * 8192).all()


@pytest.mark.parametrize("M,N,K", [(64, 8192, 2048), (64, 2048, 8192), (32, 2048, 2048), (9, 512, 2048), (16, 128, 256),
                                   (33, 3072, 2048)])
def test_linear_decode_tcgen05(F, M, N, K):
    a, st, w, sc = lin_inputs(M, N, K, 22)
    acc, y = F.dec_Linear_Layer_i8xi8(dev(a), dev(st), dev(w), dev(sc), want_acc=True)
    torch.cuda.synchronize()
    acc_o, y_o = oracle.linear_i8(a, st, w, sc)
    assert_same(to_np(acc), acc_o, "acc"); assert_same(to_np(y), y_o, "y")
    _, y2 = F.dec_Linear_Layer_i8xi8(dev(a), dev(st), dev(w), dev(sc), want_acc=False)   # library scratch path
    assert_same(to_np(y2), y_o, "y (scratch)")


@pytest.mark.parametrize("M,N,K,decode", [(200, 2048, 2048, False), (130, 264, 144, False), (1, 2048, 2048, True), (5, 512, 2048, True),
                                            (32, 2048, 2048, True), (64, 2048, 8192, True), (20, 3072, 2048, True)])
def test_linear_fused_residual(F, M, N, K, decode):
    a, st, w, sc = lin_inputs(M, N, K, 24)
    res = rng(25).standard_normal((M, N)).astype(np.float32) * 50
    fn = F.dec_Linear_Layer_i8xi8 if decode else F.pref_Linear_Layer_i8xi8
    want = oracle.residual(res, oracle.linear_i8(a, st, w, sc)[1])
    for _ in range(3):   # repeated calls: the split-K scratch must come back zeroed every time
        _, y = fn(dev(a), dev(st), dev(w), dev(sc), residual=dev(res))
        assert_same(to_np(y), want, "residual + linear")
    # in place: y aliases the residual
    r = dev(res)
    lib = F.lib()
    name = "flexllm_linear_decode_i8_residual" if decode else "flexllm_linear_prefill_i8_residual"
    import ctypes as C
    p = lambda t: C.c_void_p(t.data_ptr())
    ad, std, wd, scd = dev(a), dev(st), dev(w), dev(sc)
    rc = getattr(lib, name)(p(ad), p(std), p(wd), p(scd), M, N, K, p(r), p(r), None)
    torch.cuda.synchronize()
    assert rc == 0
    assert_same(to_np(r), want, "in-place residual")


def test_linear_golden(F):
    import os
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_ops.npz"))
    acc, y = F.pref_Linear_Layer_i8xi8(dev(G["gemm_a"]), dev(G["deq_st"]), dev(G["gemm_w"]), dev(G["deq_sc"]), want_acc=True)
    assert_same(to_np(acc), G["gemm_acc"]); assert_same(to_np(y), G["deq_y"])


def test_linear_full_size_linearity(F):
    """Size-independent property at the prefill shape of the full model (M=32768 is too large for
    the CPU oracle): acc(a, w) is linear in a, and a column block equals the oracle."""
    M, N, K = 4096, 2048, 2048
    g = rng(23)
    a1 = g.integers(-63, 64, (M, K), dtype=np.int8); a2 = g.integers(-63, 64, (M, K), dtype=np.int8)
    w = g.integers(-127, 128, (N, K), dtype=np.int8)
    st = np.ones(M, np.float32); sc = np.ones(N, np.float32)
    wd = dev(w); std = dev(st); scd = dev(sc)
    acc1, _ = F.pref_Linear_Layer_i8xi8(dev(a1), std, wd, scd, want_acc=True, want_y=False)
    acc2, _ = F.pref_Linear_Layer_i8xi8(dev(a2), std, wd, scd, want_acc=True, want_y=False)
    acc12, _ = F.pref_Linear_Layer_i8xi8(dev((a1 + a2).astype(np.int8)), std, wd, scd, want_acc=True, want_y=False)
    assert torch.equal(acc1 + acc2, acc12)
    rows = g.choice(M, 16, replace=False)
    assert_same(to_np(acc1[torch.from_numpy(rows).cuda()]), oracle.gemm_s8s8(a1[rows], w))


@pytest.mark.parametrize("lanes,V", [(16, 16 * 250), (32, 128256), (32, 32 * 8)])
def test_topk_sampling(F, lanes, V):
    """Top-k sampling (Logits.h:145-279) against the oracle: sampled index and the merged top-5 list, on random
    logits, on logits with very few distinct values (ties inside and across lanes) and for random numbers that
    select every rank."""
    rng = np.random.default_rng(31 + lanes + V)
    B = 12
    x = (rng.standard_normal((B, V)) * 3).astype(np.float32)
    x[4:8] = rng.integers(-2, 3, (4, V)).astype(np.float32)
    x[8, 7] = 50.0; x[8, V - 3] = 50.0; x[8, V // 2 + 1] = 50.0
    x[9] = -1e33                      # nothing exceeds the initial -1e32: the list stays empty (index -1)
    x[10, :5] = [3, 3, 3, 3, 3]
    for rnd_value in [0.0, 0.2, 0.45, 0.7, 0.9, 0.9999]:
        rnd = np.full(B, rnd_value, np.float32); rnd[11] = rng.random()
        with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
            want, wi, wv, _ = oracle.topk_sample(x, rnd, lanes=lanes, details=True)
        got, gi, gv = F.dec_Sampling_Layer(torch.from_numpy(x).cuda(), torch.from_numpy(rnd).cuda(), lanes=lanes, details=True)
        assert np.array_equal(to_np(gi), wi), (rnd_value, to_np(gi)[:3], wi[:3])
        assert np.array_equal(to_np(gv).view(np.uint32), wv.view(np.uint32))
        assert np.array_equal(to_np(got), want), (rnd_value, to_np(got), want)


@pytest.mark.parametrize("M,N,K,decode", [(128, 2048, 2048, False), (37, 520, 400, False), (1, 2048, 2048, True), (40, 2048, 8192, True)])
def test_asymmetric_4bit_linear(F, M, N, K, decode):
    """The reference's shipped W4A4 configuration (asymmetric 4-bit activations, zero point in the dequantiser; quant.h:53-81,
    :146-148): quantiser, integer sums and dequantised output bit for bit against the oracle, whose functions are pinned
    against the reference templates. Inputs U(-1, 1) as in the reference's bench (Linear_Layer_Prefilling_tb.cpp:172-200)."""
    g = np.random.default_rng(42 + M)
    x = g.uniform(-1, 1, (M, K)).astype(np.float32)
    w = g.integers(-8, 8, (N, K), dtype=np.int8)
    sc = g.uniform(0.001, 0.01, N).astype(np.float32)
    wsum = (w.astype(np.float64) * sc[:, None]).sum(axis=1).astype(np.float32)
    q, s, b = F.pref_quant_layer_fp32_qint_asym(dev(x), 4)
    qo, so, bo = oracle.quant_per_token_asym(x, 4)
    assert_same(to_np(q), qo, "asymmetric quantiser"); assert_same(to_np(s), so, "scales"); assert_same(to_np(b), bo, "zero points")
    acc, y = F.pref_Linear_Layer_i4xi4(q, s, b, dev(w), dev(sc), dev(wsum), decode=decode)
    acco = oracle.gemm_s8s8(qo.astype(np.int8), w)
    assert_same(to_np(acc), acco, "integer sums")
    assert_same(to_np(y), oracle.dequant_asym(acco, so, bo, sc, wsum), "dequantised output")
