"""GPU parity of the int8 attention kernels against the CPU oracle (the prefill-attention and paged decode-attention workloads at
sizes the oracle finishes in seconds, plus edge cases)."""
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


@pytest.fixture(scope="module")
def F():
    import flexllm_b200
    flexllm_b200.lib()
    return flexllm_b200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def attn_inputs(B, S, HQ, HKV, seed):
    g = np.random.default_rng(seed)
    q = g.integers(-127, 128, (B, S, HQ, 64), dtype=np.int8)
    k = g.integers(-127, 128, (B, S, HKV, 64), dtype=np.int8)
    v = g.integers(-127, 128, (B, S, HKV, 64), dtype=np.int8)
    qs = g.uniform(0.005, 0.05, (B, S, HQ)).astype(np.float32)
    ks = g.uniform(0.005, 0.05, (B, S, HKV)).astype(np.float32)
    vs = g.uniform(0.005, 0.05, (B, S, HKV)).astype(np.float32)
    a_s = np.full(HQ, 0.05 / 255, np.float32)
    return q, qs, k, ks, v, vs, a_s


def check_prefill(F, B, S, HQ, HKV, seed):
    q, qs, k, ks, v, vs, a_s = attn_inputs(B, S, HQ, HKV, seed)
    cos_t, sin_t = oracle.rope_table(max(S, 16))
    out, oacc = F.MHA_i8xi8_Prefilling(dev(q), dev(qs), dev(k), dev(ks), dev(v), dev(vs), dev(cos_t), dev(sin_t),
                                       dev(a_s), want_oacc=True)
    torch.cuda.synchronize()
    ref = oracle.mha_prefill(q, qs, k, ks, v, vs, cos_t, sin_t, a_s)
    out = to_np(out); oacc = to_np(oacc)
    assert_same(oacc, ref["oacc"], "int32 P.V accumulators")
    assert_same(out, ref["out"], "fp32 output")
    # distance to the libm flavour of the oracle (a last-bit difference in exp() can move a u8 across
    # a rounding boundary): count, and require the fp32 tolerance
    with oracle.exp_mode(oracle.EXP_LIBM):
        ref_l = oracle.mha_prefill(q, qs, k, ks, v, vs, cos_t, sin_t, a_s)
    bad = np.count_nonzero(oacc != ref_l["oacc"])
    err = max_abs_rel(out, ref_l["out"])
    print(f"prefill attn B={B} S={S}: exact; vs libm expf {bad}/{oacc.size} int32 accumulators differ, max-abs-rel {err:.2e}")
    assert err < 1e-3


@pytest.mark.parametrize("B,S,HQ,HKV", [(1, 128, 4, 1), (2, 256, 8, 2), (1, 16, 4, 4), (1, 144, 4, 1), (1, 400, 8, 2)])
def test_prefill_small(F, B, S, HQ, HKV):
    check_prefill(F, B, S, HQ, HKV, 30)


def test_prefill_config3_slice(F):
    """The prefill-attention workload's shapes (S=1024, 32/8 heads) on one batch element."""
    check_prefill(F, 1, 1024, 32, 8, 31)


def test_prefill_rows_sum_property(F):
    """Size-independent property at the full config-3 size (B=4): with V == 1 and vs == a_s * 255
    every output equals sum_k U[q][k] * a_s and U rows sum to about 255 (P sums to 1)."""
    B, S, HQ, HKV = 4, 1024, 32, 8
    q, qs, k, ks, v, vs, a_s = attn_inputs(B, S, HQ, HKV, 32)
    v[:] = 1
    vs[:] = a_s[0] * 255
    cos_t, sin_t = oracle.rope_table(S)
    out, oacc = F.MHA_i8xi8_Prefilling(dev(q), dev(qs), dev(k), dev(ks), dev(v), dev(vs), dev(cos_t), dev(sin_t),
                                       dev(a_s), want_oacc=True)
    oacc = to_np(oacc)
    # sum_k round(255 * P_k) <= 255 + (number of keys)/2; never negative
    nkeys = np.arange(1, S + 1)[None, :, None]
    assert oacc.min() >= 0 and (oacc <= 255 + nkeys / 2).all()
    # all 64 dims of a head see the same sum
    o = oacc.reshape(B, S, HQ, 64)
    assert (o == o[..., :1]).all()
    # first token attends to itself only: U = 255 exactly
    assert (o[:, 0] == 255).all()


def _float_attention(ref, v, vs):
    """Attention of the prepared int8 Q / K (after RoPE, FHT-64 and re-quantisation) and the int8 V in float64, with no
    quantisation of P: what both kernels approximate with their 8-bit P."""
    q2, qs2, k2, ks2 = ref["q2"], ref["qs2"], ref["k2"], ref["ks2"]
    B, S, HQ, _ = q2.shape; HKV = k2.shape[2]; G = HQ // HKV
    out = np.empty((B, S, HQ * 64))
    mask = np.tril(np.ones((S, S), bool))
    for b in range(B):
        for h in range(HQ):
            kv = h // G
            x = (q2[b, :, h].astype(np.float64) @ k2[b, :, kv].astype(np.float64).T) * qs2[b, :, h, None] * ks2[b, None, :, kv] * 0.125
            x = np.where(mask, x, -np.inf)
            p = np.exp(x - x.max(axis=1, keepdims=True)); p /= p.sum(axis=1, keepdims=True)
            out[b, :, h * 64:(h + 1) * 64] = p @ (v[b, :, kv].astype(np.float64) * vs[b, :, kv, None])
    return out


@pytest.mark.parametrize("B,S,HQ,HKV", [(1, 128, 4, 1), (2, 256, 8, 2), (1, 144, 4, 1), (1, 400, 8, 2), (1, 1024, 32, 8)])
def test_prefill_online_softmax_variant_is_close(F, B, S, HQ, HKV):
    """The single-sweep online-softmax variant is NOT bit-exact (it quantises P per key tile against a dynamic scale and
    uses fast exponentials). Both it and the exact kernel approximate the unquantised-P attention with an 8-bit P; the
    variant's distance to that float64 attention must stay within 3 % of the largest output (worst element) and 0.3 %
    (mean) -- the fp32-level tolerance an 8-bit P allows -- and is printed beside the exact kernel's own distance."""
    q, qs, k, ks, v, vs, a_s = attn_inputs(B, S, HQ, HKV, 33)
    cos_t, sin_t = oracle.rope_table(max(S, 16))
    args = [dev(q), dev(qs), dev(k), dev(ks), dev(v), dev(vs), dev(cos_t), dev(sin_t)]
    exact, _ = F.MHA_i8xi8_Prefilling(*args, dev(a_s))
    online = F.MHA_i8xi8_Prefilling_online(*args)
    torch.cuda.synchronize()
    assert F.lib().flexllm_device_status() == 0
    exact = to_np(exact); online = to_np(online)
    assert np.isfinite(online).all()
    ref = _float_attention(oracle.mha_prefill(q, qs, k, ks, v, vs, cos_t, sin_t, a_s), v, vs)
    scale = np.abs(ref).max()
    d_on = np.abs(online - ref) / scale; d_ex = np.abs(exact - ref) / scale
    print(f"online softmax B={B} S={S}: distance to float64 attention, of the largest output: online max {d_on.max():.2e} mean "
          f"{d_on.mean():.2e}; exact kernel max {d_ex.max():.2e} mean {d_ex.mean():.2e}")
    assert d_on.max() < 3e-2 and d_on.mean() < 3e-3


# ------------------------------------------------------------------------------ decode (config 4)
def decode_case(F, B, ctx, HQ=32, HKV=8, seed=40, steps=1):
    g = np.random.default_rng(seed)
    PAGE = 64
    ctx = np.asarray(ctx, np.int32)
    pages_per_seq = (ctx + steps + PAGE - 1) // PAGE + 1
    max_pages = int(pages_per_seq.max())
    n_pages = int(pages_per_seq.sum()) + 3
    perm = g.permutation(n_pages).astype(np.int32)            # seeded random page table
    page_table = np.zeros((B, max_pages), np.int32)
    o = 0
    for b in range(B):
        page_table[b, :pages_per_seq[b]] = perm[o:o + pages_per_seq[b]]; o += pages_per_seq[b]
    # cache contents for the already-present tokens (oracle layout: [n_pages][HKV][PAGE][64])
    k_pool = g.integers(-127, 128, (n_pages, HKV, PAGE, 64), dtype=np.int8)
    v_pool = g.integers(-127, 128, (n_pages, HKV, PAGE, 64), dtype=np.int8)
    ks_pool = g.uniform(0.005, 0.05, (n_pages, HKV, PAGE)).astype(np.float32)
    vs_pool = g.uniform(0.005, 0.05, (n_pages, HKV, PAGE)).astype(np.float32)
    max_ctx = int(ctx.max()) + steps
    cos_t, sin_t = oracle.rope_table(max_ctx + 1)
    a_s = np.full(HQ, 0.05 / 255, np.float32)
    cache = F.KVCache(1, n_pages, HKV)
    kd, ksd, vd, vsd = cache.pools(0)
    kd.copy_(dev(k_pool)); ksd.copy_(dev(ks_pool)); vsd.copy_(dev(vs_pool))
    vd.copy_(dev(np.ascontiguousarray(v_pool.transpose(0, 1, 3, 2))))
    cur = ctx.copy()
    for step in range(steps):
        q = g.integers(-127, 128, (B, HQ, 64), dtype=np.int8); k = g.integers(-127, 128, (B, HKV, 64), dtype=np.int8)
        v = g.integers(-127, 128, (B, HKV, 64), dtype=np.int8)
        qs = g.uniform(0.005, 0.05, (B, HQ)).astype(np.float32); ks = g.uniform(0.005, 0.05, (B, HKV)).astype(np.float32)
        vs = g.uniform(0.005, 0.05, (B, HKV)).astype(np.float32)
        out, oacc = F.MHA_i8xi8_Decoding(cache, 0, dev(q), dev(qs), dev(k), dev(ks), dev(v), dev(vs), dev(cos_t), dev(sin_t),
                                         dev(a_s), dev(page_table), dev(cur), max_ctx, want_oacc=True)
        torch.cuda.synchronize()
        out_o, oacc_o = oracle.mha_decode(q, qs, k, ks, v, vs, cos_t, sin_t, a_s, k_pool, ks_pool, v_pool, vs_pool,
                                          page_table, cur)
        assert_same(to_np(oacc), oacc_o, "int32 P.V accumulators")
        assert_same(to_np(out), out_o, "fp32 output")
        cur = cur + 1
    # the appended tokens landed in the cache exactly as in the oracle
    assert_same(to_np(kd), k_pool, "K cache"); assert_same(to_np(ksd), ks_pool, "K scales")
    assert_same(to_np(vd), np.ascontiguousarray(v_pool.transpose(0, 1, 3, 2)), "V cache"); assert_same(to_np(vsd), vs_pool, "V scales")
    cache.close()


def test_decode_small(F):
    decode_case(F, 3, [0, 5, 130], steps=2)


def test_decode_page_boundaries(F):
    decode_case(F, 6, [63, 64, 65, 511, 512, 513], seed=41, steps=2)


def test_decode_config4_slice(F):
    """The decode-attention workload's shapes: contexts drawn uniformly from [512, 8192], one layer, 8 sequences."""
    g = np.random.default_rng(42)
    decode_case(F, 8, g.integers(512, 8193, 8), seed=42)


def test_decode_max_context(F):
    decode_case(F, 2, [8192, 8191], seed=43)


def test_kv_append_alone(F):
    """The cache managers' append on its own: the new token's K row, transposed V column and both scales land at
    position ctx[b] of the right page; everything else in the pools is untouched."""
    g = np.random.default_rng(45)
    B, HKV, PAGE = 5, 8, 64
    ctx = np.array([0, 63, 64, 200, 777], np.int32)
    pages = (ctx + 1 + PAGE - 1) // PAGE
    max_pages = int(pages.max()); n_pages = int(pages.sum()) + 2
    perm = g.permutation(n_pages).astype(np.int32)
    pt = np.zeros((B, max_pages), np.int32); o = 0
    for b in range(B):
        pt[b, :pages[b]] = perm[o:o + pages[b]]; o += pages[b]
    cache = F.KVCache(2, n_pages, HKV)
    layer = 1
    kd, ksd, vd, vsd = cache.pools(layer)
    k_pool = g.integers(-127, 128, (n_pages, HKV, PAGE, 64), dtype=np.int8); v_pool = g.integers(-127, 128, (n_pages, HKV, 64, PAGE), dtype=np.int8)
    ks_pool = g.uniform(0.005, 0.05, (n_pages, HKV, PAGE)).astype(np.float32); vs_pool = g.uniform(0.005, 0.05, (n_pages, HKV, PAGE)).astype(np.float32)
    kd.copy_(dev(k_pool)); vd.copy_(dev(v_pool)); ksd.copy_(dev(ks_pool)); vsd.copy_(dev(vs_pool))
    k = g.integers(-127, 128, (B, HKV, 64), dtype=np.int8); v = g.integers(-127, 128, (B, HKV, 64), dtype=np.int8)
    ks = g.uniform(0.005, 0.05, (B, HKV)).astype(np.float32); vs = g.uniform(0.005, 0.05, (B, HKV)).astype(np.float32)
    F.dec_KV_cache_append(cache, layer, dev(k), dev(ks), dev(v), dev(vs), dev(pt), dev(ctx), int(ctx.max()))
    torch.cuda.synchronize()
    for b in range(B):
        pg, slot = pt[b, ctx[b] // PAGE], ctx[b] % PAGE
        k_pool[pg, :, slot, :] = k[b]; v_pool[pg, :, :, slot] = v[b]; ks_pool[pg, :, slot] = ks[b]; vs_pool[pg, :, slot] = vs[b]
    assert_same(to_np(kd), k_pool, "K pool"); assert_same(to_np(vd), v_pool, "V pool")
    assert_same(to_np(ksd), ks_pool, "K scales"); assert_same(to_np(vsd), vs_pool, "V scales")
    k0 = cache.pools(0)[0]
    assert int(k0.abs().max()) == 0          # the other layer was not touched
    cache.close()
