"""Pins the plain-C++ oracle (oracle/flexllm_oracle.cpp) bit-for-bit against the reference's own
operator templates compiled through the header shim (oracle/_ref). Skipped where the reference
sources, and hence oracle/_ref, are not available; tests/test_oracle_golden.py then carries the pin
through fixtures generated from the same library."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref not built (reference sources absent)")
R = oracle.ref


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a


def same(a, b):
    assert a.shape == b.shape and a.dtype == b.dtype
    assert np.array_equal(bits(a), bits(b)), f"{np.count_nonzero(bits(a) != bits(b))} of {a.size} differ"


def rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("M,K", [(8, 2048), (3, 64), (16, 8192), (1, 512)])
def test_quant_per_token(M, K):
    x = rng(1).standard_normal((M, K)).astype(np.float32) * 3
    x[0, :] = 0 if M > 1 else x[0, :]          # all-zero row -> scale forced to 1
    q, s = oracle.quant_per_token(x)
    q2, s2 = R.quant_per_token(x)
    same(q, q2); same(s, s2)
    if K % 8 == 0:
        q3, s3 = R.quant_per_token(x, decode=True)
        same(q, q3); same(s, s3)


def test_quant_ties_round_half_away():
    # x/s lands exactly on .5: scale = 127/127 = 1
    x = np.array([[127.0, 0.5, -0.5, 1.5, -2.5, 2.5, 63.5, -126.5]], np.float32)
    q, s = oracle.quant_per_token(x)
    assert s[0] == 1.0
    assert q.tolist() == [[127, 1, -1, 2, -3, 3, 64, -127]]
    q2, s2 = R.quant_per_token(x)
    same(q, q2)


@pytest.mark.parametrize("M,N,K", [(8, 16, 64), (16, 48, 2048), (5, 20, 8192)])
def test_gemm_s8s8(M, N, K):
    g = rng(2)
    a = g.integers(-127, 128, (M, K), dtype=np.int8); w = g.integers(-127, 128, (N, K), dtype=np.int8)
    acc = oracle.gemm_s8s8(a, w)
    same(acc, R.gemm_s8s8(a, w))
    same(acc, (a.astype(np.int64) @ w.astype(np.int64).T).astype(np.int32))


def test_gemm_extremes():
    a = np.full((8, 8192), -128, np.int8); w = np.full((16, 8192), -128, np.int8)
    acc = oracle.gemm_s8s8(a, w)
    assert (acc == 128 * 128 * 8192).all()
    same(acc, R.gemm_s8s8(a, w))


@pytest.mark.parametrize("M,N,K", [(8, 16, 1024), (16, 64, 128)])
def test_gemm_u8s8(M, N, K):
    g = rng(3)
    a = g.integers(0, 256, (M, K), dtype=np.uint8); w = g.integers(-128, 128, (N, K), dtype=np.int8)
    acc = oracle.gemm_u8s8(a, w)
    same(acc, R.gemm_u8s8(a, w))
    same(acc, (a.astype(np.int64) @ w.astype(np.int64).T).astype(np.int32))


def test_dequant():
    g = rng(4)
    acc = g.integers(-2**27, 2**27, (9, 300), dtype=np.int32)
    st = g.uniform(0.005, 0.05, 9).astype(np.float32); sc = g.uniform(0.001, 0.01, 300).astype(np.float32)
    same(oracle.dequant(acc, st, sc), R.dequant(acc, st, sc))
    same(oracle.dequant(acc, st, sc), R.scale_stream_dequant(acc, st, sc))


@pytest.mark.parametrize("N,scale", [(64, 8.0), (256, 16.0), (8192, 90.50966799)])
def test_fht(N, scale):
    x = rng(5).standard_normal((3, N)).astype(np.float32)
    y = oracle.fht(x, scale)
    same(y, R.fht(x, scale))
    if N == 8192:
        same(y, R.fht(x, scale, decode=True))
    # it is a Hadamard transform: applying it twice with scale sqrt(N) returns the input
    z = oracle.fht(oracle.fht(x, np.sqrt(N)), np.sqrt(N))
    assert np.allclose(z, x, rtol=1e-4, atol=1e-5)


def test_rope():
    g = rng(6)
    cos_t, sin_t = oracle.rope_table(1024)
    S, H = 40, 3
    x = g.standard_normal((S, H, 64)).astype(np.float32)
    y = oracle.rope(x, np.arange(S), cos_t, sin_t)
    same(y, R.rope_prefill(x, cos_t, sin_t))
    for pos in (0, 17, 1023):
        yd = oracle.rope(x[:1], np.array([pos]), cos_t, sin_t)
        same(yd[0], R.rope_decode(x[0], cos_t, sin_t, pos))


def test_softmax():
    g = rng(7)
    x = (g.standard_normal((24, 64)) * 4).astype(np.float32)
    same(oracle.softmax(x), R.softmax_prefill(x, causal=False))
    valid = np.arange(1, 25, dtype=np.int32)
    pc = oracle.softmax(x, valid)
    same(pc, R.softmax_prefill(x, causal=True))
    # the causal prefix alone gives the same bits as the padded masked row
    for t in (0, 1, 5, 23):
        same(oracle.softmax(x[t:t + 1, :t + 1])[0], pc[t, :t + 1])
        assert (pc[t, t + 1:] == 0).all()
    for L in (1, 2, 3, 7, 1025):
        r = (g.standard_normal(L) * 3).astype(np.float32)
        same(oracle.softmax(r[None])[0], R.softmax_decode(r))


def test_rmsnorm():
    g = rng(8)
    x = g.standard_normal((5, 2048)).astype(np.float32); gamma = (1 + 0.02 * g.standard_normal(2048)).astype(np.float32)
    same(oracle.rmsnorm(x, gamma, lanes=0), R.rmsnorm(x, gamma, lanes=0))
    same(oracle.rmsnorm(x, gamma, lanes=4), R.rmsnorm(x, gamma, lanes=4))
    same(oracle.rmsnorm(x, gamma, lanes=8), R.rmsnorm(x, gamma, lanes=8))


def test_silu_gate_residual():
    g = rng(9)
    a = (g.standard_normal(5000) * 4).astype(np.float32); b = g.standard_normal(5000).astype(np.float32)
    same(oracle.silu(a), R.silu(a))
    same(oracle.silu_mul(a, b), R.gate_mul(R.silu(a), b))
    same(oracle.residual(a, b), R.residual(a, b))


def test_static_quant():
    g = rng(10)
    x = (g.standard_normal((7, 64)) * 2).astype(np.float32)
    same(oracle.static_quant(x, 0.01, 8.0, True), R.static_quant(x, 0.01, 8.0, True))
    p = g.uniform(0, 1.2, (7, 64)).astype(np.float32)
    same(oracle.static_quant(p, 1 / 255, 1.0, False), R.static_quant(p, 1 / 255, 1.0, False))
    s = g.uniform(0.005, 0.05, 7).astype(np.float32)
    same(oracle.static_quant(x, s, 1.0, True), R.scale_stream_quant(x, s, True))


def test_head_quant():
    x = rng(11).standard_normal((6, 64)).astype(np.float32)
    q, s = oracle.quant_per_token(x)
    q2, s2 = R.head_quant(x)
    same(q, q2); same(s, s2)


def test_mha_integer_paths():
    g = rng(12)
    S, G = 32, 4
    q = g.integers(-127, 128, (S, G, 64), dtype=np.int8); k = g.integers(-127, 128, (S, 64), dtype=np.int8)
    acc = R.mha_qxk(q, k)
    same(acc, oracle.gemm_s8s8(q.reshape(S * G, 64), k).reshape(S, G, S))
    p = g.integers(0, 256, (S, G, S), dtype=np.uint8); v = g.integers(-127, 128, (S, 64), dtype=np.int8)
    acc2 = R.mha_axv(p, v)
    same(acc2, oracle.gemm_u8s8(p.reshape(S * G, S), np.ascontiguousarray(v.T)).reshape(S, G, 64))


def test_argmax_ties():
    l = np.zeros((3, 1000), np.float32)
    l[0, [5, 900]] = 2.0; l[1, 999] = 1.0; l[2, :] = -3.0
    a = oracle.argmax(l)
    assert a.tolist() == [5, 999, 0]
    same(a, R.argmax(l))


def test_attention_row_composition():
    """The build-specific composition (per-token value scales folded into P before its quantisation) is made of
    reference operators only: check each stage of one row against them."""
    g = rng(13)
    nk = 37
    q = g.integers(-127, 128, 64, dtype=np.int8); k = g.integers(-127, 128, (nk, 64), dtype=np.int8)
    v = g.integers(-127, 128, (nk, 64), dtype=np.int8)
    ks = g.uniform(0.005, 0.05, nk).astype(np.float32); vs = g.uniform(0.005, 0.05, nk).astype(np.float32)
    qs = np.float32(0.003); a_s = np.float32(0.05 / 255)
    r = oracle.attn_row(q, qs, k, ks, v, vs, a_s)
    acc = R.gemm_s8s8(q[None], k)
    score = R.scale_stream_dequant(acc, [qs], ks) * np.float32(0.125)
    same(r["score"], score[0])
    p = R.softmax_decode(score[0])
    pt = R.gate_mul(p, vs)
    pq = R.static_quant(pt[None], a_s, 1.0, False)
    same(r["p"], pq[0])
    oacc = R.gemm_u8s8(pq, np.ascontiguousarray(v.T))
    same(r["oacc"], oacc[0])
    same(r["out"], R.dequant(oacc, [a_s], np.ones(64, np.float32))[0])


@pytest.mark.parametrize("lanes", [16, 32])
def test_topk_sample_restatement_vs_reference(lanes):
    """Logits.h:145-279 top-k sampling: restatement vs the reference template, including exact ties inside and
    across lanes and every rank being picked by some random number."""
    if oracle.ref is None:
        pytest.skip("reference templates not built")
    rng = np.random.default_rng(90 + lanes)
    V = lanes * 96
    rows = []
    x = rng.standard_normal((6, V)).astype(np.float32) * 2
    rows.append(x)
    t = rng.integers(-3, 4, (6, V)).astype(np.float32)          # few distinct values: many ties everywhere
    rows.append(t)
    peak = rng.standard_normal((4, V)).astype(np.float32)
    peak[:, 5] = 9.0; peak[:, V - 7] = 9.0; peak[:, V // 2] = 9.0  # equal maxima in different lanes
    rows.append(peak)
    logits = np.concatenate(rows)
    for rnd_value in [0.0, 0.13, 0.37, 0.62, 0.81, 0.97, 0.999999]:
        rnd = np.full(len(logits), rnd_value, np.float32)
        with oracle.exp_mode(oracle.EXP_LIBM):                   # the reference calls the C library's exp
            got = oracle.topk_sample(logits, rnd, lanes=lanes)
        want = oracle.ref.topk_sample(logits, rnd, lanes=lanes)
        assert np.array_equal(got, want), (rnd_value, got, want)


def test_asymmetric_4bit_linear_path_matches_reference_templates():
    """The reference's shipped precision: 4-bit asymmetric activations (pref_quant_layer_fp32_qint<4, true>, quant.h:53-81),
    unsigned x signed 4-bit systolic array (Linear_Layer.h:9, is_uint_A), dequantiser with zero point (quant.h:146-148).
    Inputs as in the reference's own test bench: U(-1, 1) (Linear_Layer_Prefilling_tb.cpp:172-200)."""
    R = oracle.ref
    if R is None:
        pytest.skip("reference templates not built")
    g = np.random.default_rng(42)
    x = g.uniform(-1, 1, (24, 512)).astype(np.float32)
    x[5] = 0.25                                               # constant row: scale 0 -> 1
    q, s, b = oracle.quant_per_token_asym(x, 4)
    q2, s2, b2 = R.quant_per_token_asym4(x)
    assert np.array_equal(q, q2) and np.array_equal(s.view(np.uint32), s2.view(np.uint32)) and np.array_equal(b.view(np.uint32), b2.view(np.uint32))
    assert q.min() == 0 and q.max() == 15
    w = g.integers(-8, 8, (48, 512), dtype=np.int8)
    acc = oracle.gemm_s8s8(q.astype(np.int8), w)
    assert np.array_equal(acc, R.gemm_u4s4(q, w))
    sc = g.uniform(0.001, 0.01, 48).astype(np.float32)
    wsum = np.zeros(48, np.float32)
    ws = w.astype(np.float32) * sc[:, None]
    for j in range(512):
        wsum = (wsum + ws[:, j]).astype(np.float32)
    y = oracle.dequant_asym(acc, s, b, sc, wsum)
    assert np.array_equal(y.view(np.uint32), R.dequant_asym(acc, s, b, sc, wsum).view(np.uint32))
    # the reference bench's own tolerance check against the fake-quant product (rel 1e-2, Linear_Layer_Prefilling_tb.cpp:281)
    fq = (q.astype(np.float32) * s[:, None] + b[:, None]) @ ws.T
    assert np.abs(y - fq).max() <= 1e-2 * np.abs(fq).max()


def test_hmt_fp32_primitives_match_reference_templates():
    """The HMT cross-attention's linear unit (dec_Linear_Layer_fp32xfp32, Linear_Layer.h:1040; four interleaved chains,
    PE.h:655-756) and its softmax (dec_Softmax<float, 4, 64, scale, sub-max>, Softmax.h:261) against the restatement."""
    R = oracle.ref
    if R is None:
        pytest.skip("reference templates not built")
    g = np.random.default_rng(7)
    for N, K in [(2048, 2048), (64, 2048), (2048, 64)]:
        x = g.standard_normal(K).astype(np.float32); w = g.standard_normal((N, K)).astype(np.float32)
        assert np.array_equal(oracle.linear_fp32_chain4(x, w).view(np.uint32), R.linear_fp32(x, w).view(np.uint32))
    for trial in range(4):
        x = (g.standard_normal(64) * 40).astype(np.float32)
        x[16 * trial:] = 0                                      # empty memory slots score exactly 0
        with oracle.exp_mode(oracle.EXP_LIBM):                  # the template calls the C library's expf
            p = oracle.softmax_dec(x, 4, 45.2548339959)
        assert np.array_equal(p.view(np.uint32), R.softmax_dec4_64(x, 45.2548339959).view(np.uint32))
