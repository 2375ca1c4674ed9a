"""ctypes bindings for the CPU oracle.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the repository's smoke check and by the CPU
baseline / reference arm of ``bench.py``. The product package (``flexllm_b200``) never imports it.

Two libraries:

* ``liboracle.so`` (``oracle/flexllm_oracle.cpp``) -- plain-C++ restatement of the reference's
  operator templates; functions ``orc_*``; exposed here as module-level functions.
* ``_ref/libflexllm_ref.so`` (``oracle/ref_wrap.cpp``) -- the reference's own templates compiled
  through the header shim; functions ``ref_*``; exposed through :data:`ref` when the file exists.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_REF = os.path.join(_HERE, "_ref", "libflexllm_ref.so")


def build(verbose=False):
    """Compile the oracle libraries with the Makefile beside this file."""
    r = subprocess.run(["make", "-C", _HERE], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stdout)


def _load(path):
    if not os.path.exists(path):
        return None
    return C.CDLL(path)


if not os.path.exists(_LIB):
    build()
_lib = _load(_LIB)
_ref = _load(_REF)


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i8(a):
    return np.ascontiguousarray(a, dtype=np.int8)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


# ------------------------------------------------------------------ Tier B (restatement)
EXP_LIBM, EXP_CORRECTLY_ROUNDED = 0, 1


def set_exp_mode(mode):
    """0: the build machine's libm expf (what a C simulation of the reference computes here);
    1: correctly rounded expf = (float)exp((double)x), which the CUDA kernels reproduce bit for bit."""
    _lib.orc_set_exp_mode(C.c_int(mode))


def set_threads(n):
    """Number of threads of the oracle's OpenMP loops (overrides an inherited OMP_NUM_THREADS)."""
    _lib.orc_set_threads(C.c_int(int(n)))


def get_threads():
    return int(_lib.orc_get_threads())


def get_exp_mode():
    return _lib.orc_get_exp_mode()


class exp_mode:
    """Context manager: ``with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED): ...``"""

    def __init__(self, mode):
        self.mode = mode

    def __enter__(self):
        self.prev = get_exp_mode(); set_exp_mode(self.mode)

    def __exit__(self, *a):
        set_exp_mode(self.prev)


def quant_per_token(x):
    x = _f32(x); M, K = x.shape
    q = np.empty((M, K), np.int8); s = np.empty(M, np.float32)
    _lib.orc_quant_per_token(_p(x), C.c_int(M), C.c_int(K), _p(q), _p(s))
    return q, s


def quant_per_token_asym(x, bits=4):
    """Asymmetric per-token quantiser (quant.h:53-81). Returns (q uint8 in [0, 2^bits-1], scale, zero point)."""
    x = _f32(x); M, K = x.shape
    q = np.empty((M, K), np.uint8); s = np.empty(M, np.float32); b = np.empty(M, np.float32)
    _lib.orc_quant_per_token_asym(_p(x), C.c_int(M), C.c_int(K), C.c_int(bits), _p(q), _p(s), _p(b))
    return q, s, b


def dequant_asym(acc, s_tok, b_tok, s_ch, wsum):
    """y = ((float)acc * s_tok) * s_ch + b_tok * wsum (quant.h:146-148)."""
    acc = _i32(acc); M, N = acc.shape; y = np.empty((M, N), np.float32)
    _lib.orc_dequant_asym(_p(acc), _p(_f32(s_tok)), _p(_f32(b_tok)), _p(_f32(s_ch)), _p(_f32(wsum)), C.c_int(M), C.c_int(N), _p(y))
    return y


def gemm_s8s8(a, w):
    a = _i8(a); w = _i8(w); M, K = a.shape; N = w.shape[0]
    acc = np.empty((M, N), np.int32)
    _lib.orc_gemm_s8s8(_p(a), _p(w), C.c_int(M), C.c_int(N), C.c_int(K), _p(acc))
    return acc


def gemm_u8s8(a, w):
    a = np.ascontiguousarray(a, dtype=np.uint8); w = _i8(w); M, K = a.shape; N = w.shape[0]
    acc = np.empty((M, N), np.int32)
    _lib.orc_gemm_u8s8(_p(a), _p(w), C.c_int(M), C.c_int(N), C.c_int(K), _p(acc))
    return acc


def dequant(acc, s_tok, s_ch):
    acc = _i32(acc); M, N = acc.shape
    y = np.empty((M, N), np.float32)
    _lib.orc_dequant(_p(acc), _p(_f32(s_tok)), _p(_f32(s_ch)), C.c_int(M), C.c_int(N), _p(y))
    return y


def fht(x, scale):
    x = _f32(x); N = x.shape[-1]; rows = x.size // N
    y = np.empty_like(x)
    _lib.orc_fht(_p(x), C.c_long(rows), C.c_int(N), C.c_float(scale), _p(y))
    return y


def rope_table(P):
    c = np.empty((P, 32), np.float32); s = np.empty((P, 32), np.float32)
    _lib.orc_rope_table(C.c_int(P), _p(c), _p(s))
    return c, s


def rope(x, pos, cos_t, sin_t):
    """x [T,H,64] fp32, pos [T] int32."""
    x = _f32(x); T, H, D = x.shape; assert D == 64
    pos = _i32(pos)
    y = np.empty_like(x)
    _lib.orc_rope(_p(x), _p(pos), _p(_f32(cos_t)), _p(_f32(sin_t)), C.c_long(T), C.c_int(H), _p(y))
    return y


def softmax(x, valid=None):
    x = _f32(x); L = x.shape[-1]; rows = x.size // L
    p = np.empty_like(x)
    v = None if valid is None else _i32(valid)
    _lib.orc_softmax(_p(x), C.c_long(rows), C.c_int(L), _p(v), _p(p))
    return p


def rmsnorm(x, gamma, eps=1e-5, lanes=0):
    x = _f32(x); M, D = x.shape
    y = np.empty_like(x)
    _lib.orc_rmsnorm(_p(x), _p(_f32(gamma)), C.c_int(M), C.c_int(D), C.c_float(eps), C.c_int(lanes), _p(y))
    return y


def silu(g):
    g = _f32(g); y = np.empty_like(g)
    _lib.orc_silu(_p(g), C.c_long(g.size), _p(y))
    return y


def silu_mul(g, u):
    g = _f32(g); u = _f32(u); y = np.empty_like(g)
    _lib.orc_silu_mul(_p(g), _p(u), C.c_long(g.size), _p(y))
    return y


def residual(a, b):
    a = _f32(a); b = _f32(b); y = np.empty_like(a)
    _lib.orc_residual(_p(a), _p(b), C.c_long(a.size), _p(y))
    return y


def static_quant(x, s, f=1.0, signed=True):
    """x [rows,n]; s scalar or [rows]. Returns int8 (signed) or uint8."""
    x = _f32(x); rows, n = x.shape
    s = _f32(np.atleast_1d(s)); stride = 0 if s.size == 1 else 1
    q = np.empty((rows, n), np.uint8)
    _lib.orc_static_quant(_p(x), C.c_long(rows), C.c_int(n), _p(s), C.c_int(stride), C.c_float(f),
                          C.c_int(1 if signed else 0), _p(q))
    return q.view(np.int8) if signed else q


def argmax(logits):
    logits = _f32(logits); B, V = logits.shape
    idx = np.empty(B, np.int32)
    _lib.orc_argmax(_p(logits), C.c_int(B), C.c_long(V), _p(idx))
    return idx


def topk_sample(logits, rnd, lanes=32, top_k=5, details=False):
    """Top-k sampling of Logits.h:145-279 with `lanes` lanes; rnd: one uniform number per row."""
    logits = _f32(logits); B, V = logits.shape
    rnd = _f32(np.asarray(rnd).reshape(B))
    idx = np.empty(B, np.int32); ti = np.empty((B, top_k), np.int32); tv = np.empty((B, top_k), np.float32); tp = np.empty((B, top_k), np.float32)
    rc = _lib.orc_topk_sample(_p(logits), C.c_int(B), C.c_long(V), C.c_int(lanes), C.c_int(top_k), _p(rnd), _p(idx), _p(ti), _p(tv), _p(tp))
    if rc != 0:
        raise ValueError("orc_topk_sample: unsupported shape")
    return (idx, ti, tv, tp) if details else idx


def linear_i8(a, s_tok, w, s_ch):
    a = _i8(a); w = _i8(w); M, K = a.shape; N = w.shape[0]
    acc = np.empty((M, N), np.int32); y = np.empty((M, N), np.float32)
    _lib.orc_linear_i8(_p(a), _p(_f32(s_tok)), _p(w), _p(_f32(s_ch)), C.c_int(M), C.c_int(N), C.c_int(K),
                       _p(acc), _p(y))
    return acc, y


def mlp_block(h, gamma, wg, sg, wu, su, wd, sd, eps=1e-5, lanes=0, fht_scale=90.50966799):
    """Returns dict(out, xq, xs, act, hq, hs, down_acc)."""
    h = _f32(h); M, D = h.shape; F = wg.shape[0]
    r = dict(out=np.empty((M, D), np.float32), xq=np.empty((M, D), np.int8), xs=np.empty(M, np.float32),
             act=np.empty((M, F), np.float32), hq=np.empty((M, F), np.int8), hs=np.empty(M, np.float32),
             down_acc=np.empty((M, D), np.int32))
    _lib.orc_mlp_block(_p(h), _p(_f32(gamma)), _p(_i8(wg)), _p(_f32(sg)), _p(_i8(wu)), _p(_f32(su)),
                       _p(_i8(wd)), _p(_f32(sd)), C.c_int(M), C.c_int(D), C.c_int(F), C.c_float(eps),
                       C.c_int(lanes), C.c_float(fht_scale), _p(r["out"]), _p(r["xq"]), _p(r["xs"]),
                       _p(r["act"]), _p(r["hq"]), _p(r["hs"]), _p(r["down_acc"]))
    return r


def qk_prepare(q, s, pos, cos_t, sin_t):
    """q [T,H,64] int8, s [T,H]; returns (q2 int8, s2, rotated fp32)."""
    q = _i8(q); T, H, D = q.shape; assert D == 64
    q2 = np.empty_like(q); s2 = np.empty((T, H), np.float32); rot = np.empty((T, H, 64), np.float32)
    _lib.orc_qk_prepare(_p(q), _p(_f32(s)), _p(_i32(pos)), _p(_f32(cos_t)), _p(_f32(sin_t)),
                        C.c_long(T), C.c_int(H), _p(q2), _p(s2), _p(rot))
    return q2, s2, rot


def mha_prefill(q, qs, k, ks, v, vs, cos_t, sin_t, a_s):
    """q [B,S,HQ,64] s8, qs [B,S,HQ]; k,v [B,S,HKV,64]; returns dict(out, q2, qs2, k2, ks2, oacc)."""
    q = _i8(q); k = _i8(k); v = _i8(v)
    B, S, HQ, _ = q.shape; HKV = k.shape[2]
    r = dict(out=np.empty((B, S, HQ * 64), np.float32), q2=np.empty_like(q), qs2=np.empty((B, S, HQ), np.float32),
             k2=np.empty_like(k), ks2=np.empty((B, S, HKV), np.float32), oacc=np.empty((B, S, HQ * 64), np.int32))
    _lib.orc_mha_prefill(_p(q), _p(_f32(qs)), _p(k), _p(_f32(ks)), _p(v), _p(_f32(vs)), _p(_f32(cos_t)),
                         _p(_f32(sin_t)), _p(_f32(a_s)), C.c_int(B), C.c_int(S), C.c_int(HQ), C.c_int(HKV),
                         _p(r["out"]), _p(r["q2"]), _p(r["qs2"]), _p(r["k2"]), _p(r["ks2"]), _p(r["oacc"]))
    return r


def mha_decode(q, qs, k, ks, v, vs, cos_t, sin_t, a_s, k_pool, ks_pool, v_pool, vs_pool, page_table, ctx):
    """One decode step; pools are modified in place (append). Returns (out [B,HQ*64], oacc)."""
    q = _i8(q); B, HQ, _ = q.shape; HKV = k.shape[1]
    n_pages, HKV2, PAGE, _ = k_pool.shape; assert HKV2 == HKV
    for a in (k_pool, ks_pool, v_pool, vs_pool):
        assert a.flags["C_CONTIGUOUS"]
    page_table = _i32(page_table); ctx = _i32(ctx)
    out = np.empty((B, HQ * 64), np.float32); oacc = np.empty((B, HQ * 64), np.int32)
    _lib.orc_mha_decode(_p(q), _p(_f32(qs)), _p(_i8(k)), _p(_f32(ks)), _p(_i8(v)), _p(_f32(vs)),
                        _p(_f32(cos_t)), _p(_f32(sin_t)), _p(_f32(a_s)), _p(k_pool), _p(ks_pool), _p(v_pool),
                        _p(vs_pool), _p(page_table), C.c_int(page_table.shape[1]), _p(ctx), C.c_int(B),
                        C.c_int(HQ), C.c_int(HKV), C.c_int(PAGE), _p(out), _p(oacc))
    return out, oacc


def attn_row(q, qs, k, ks, v, vs, a_s):
    """One attention row; returns dict(out[64], oacc[64], p[nk] u8, score[nk])."""
    k = _i8(k); nk = k.shape[0]
    r = dict(out=np.empty(64, np.float32), oacc=np.empty(64, np.int32), p=np.empty(nk, np.uint8),
             score=np.empty(nk, np.float32))
    _lib.orc_attn_row(_p(_i8(q)), C.c_float(qs), _p(k), _p(_f32(ks)), _p(_i8(v)), _p(_f32(vs)), C.c_int(nk),
                      C.c_float(a_s), _p(r["out"]), _p(r["oacc"]), _p(r["p"]), _p(r["score"]))
    return r


def linear_fp32_chain4(x, w):
    """y = W x in fp32 with the reference's accumulation order (dec_Linear_Layer_fp32xfp32, PE.h:655-756): four
    interleaved chains over k mod 4, combined (p0 + p1) + (p2 + p3). x [K], w [N,K] -> y [N]."""
    x = _f32(x); w = _f32(w); N, K = w.shape
    y = np.empty(N, np.float32)
    _lib.orc_linear_fp32_chain4(_p(x), _p(w), C.c_int(N), C.c_int(K), _p(y))
    return y


def softmax_dec(x, lanes=4, scale=1.0):
    """dec_Softmax with enable_scale and enable_sub_max (Softmax.h:261-363): p = softmax((x - max) / scale) with `lanes`
    block-partitioned lanes of four interleaved partial sums each."""
    x = _f32(x); p = np.empty_like(x)
    _lib.orc_softmax_dec(_p(x), C.c_int(x.size), C.c_int(lanes), C.c_float(scale), _p(p))
    return p


class _OrcModel(C.Structure):
    _PP = C.POINTER(C.c_void_p)
    _fields_ = ([("L", C.c_int), ("D", C.c_int), ("HQ", C.c_int), ("HKV", C.c_int), ("F", C.c_int), ("V", C.c_int),
                 ("eps", C.c_float), ("fht_scale", C.c_float)] +
                [(n, C.POINTER(C.c_void_p)) for n in ("wq", "wk", "wv", "wo", "wg", "wu", "wd", "sq", "sk", "sv", "so", "sg",
                                                       "su", "sd", "g0", "g1", "a_s")] +
                [("g_final", C.c_void_p), ("lm_w", C.c_void_p), ("lm_s", C.c_void_p), ("cos_t", C.c_void_p), ("sin_t", C.c_void_p)])


def _orc_model(weights):
    """(struct, keep-alive list) for the C model functions."""
    L = len(weights["wq"]); D = weights["wq"][0].shape[1]; F = weights["wg"][0].shape[0]; V = weights["lm_w"].shape[0]
    keep = []
    m = _OrcModel()
    m.L, m.D, m.HQ, m.HKV, m.F, m.V = L, D, weights["HQ"], weights["HKV"], F, V
    m.eps, m.fht_scale = 1e-5, float(np.float32(np.sqrt(F)))
    for name in ("wq", "wk", "wv", "wo", "wg", "wu", "wd"):
        arrs = [_i8(a) for a in weights[name]]; keep.append(arrs)
        ptrs = (C.c_void_p * L)(*[a.ctypes.data for a in arrs]); keep.append(ptrs)
        setattr(m, name, ptrs)
    for name in ("sq", "sk", "sv", "so", "sg", "su", "sd", "g0", "g1", "a_s"):
        arrs = [_f32(a) for a in weights[name]]; keep.append(arrs)
        ptrs = (C.c_void_p * L)(*[a.ctypes.data for a in arrs]); keep.append(ptrs)
        setattr(m, name, ptrs)
    for name, conv in (("g_final", _f32), ("lm_w", _i8), ("lm_s", _f32), ("cos_t", _f32), ("sin_t", _f32)):
        a = conv(weights[name]); keep.append(a)
        setattr(m, name, a.ctypes.data)
    return m, keep


def model_generate(weights, tokens, n_new, want_hidden=False, want_logits=False, sampling=None):
    """Full-model greedy generation on the CPU. `weights`: dict with per-layer lists under the keys
    wq wk wv wo wg wu wd (int8 [N,K]), sq sk sv so sg su sd g0 g1 a_s (fp32) and g_final, lm_w, lm_s,
    cos_t, sin_t, plus ints HQ, HKV. tokens [B,S] int32. sampling: None (greedy) or (lanes, top_k, rnd [n_new,B])
    for the reference's top-k sampling. Returns dict(tokens [B,n_new], hidden, logits_prefill, logits_last)."""
    tokens = _i32(tokens); B, S = tokens.shape
    m, keep = _orc_model(weights)
    D, V = m.D, m.V
    out = np.zeros((B, max(n_new, 1)), np.int32)
    hidden = np.empty((B * S, D), np.float32) if want_hidden else None
    lp = np.empty((B, V), np.float32) if want_logits else None
    ll = np.empty((B, V), np.float32) if (want_logits and n_new > 1) else None
    rnd = None
    if sampling is not None:
        rnd = _f32(np.asarray(sampling[2]).reshape(max(n_new, 1), B))
        _lib.orc_set_sampling(C.c_int(sampling[0]), C.c_int(sampling[1]), _p(rnd))
    try:
        _lib.orc_model_generate(C.byref(m), _p(tokens), C.c_int(B), C.c_int(S), C.c_int(n_new), _p(out), _p(hidden), _p(lp), _p(ll))
    finally:
        _lib.orc_set_sampling(C.c_int(0), C.c_int(0), None)
    return dict(tokens=out[:, :n_new], hidden=hidden, logits_prefill=lp, logits_last=ll)


def model_forward_embeds(weights, embeds, n_valid, n_new=0):
    """One sequence from embeddings [S,D] (rows from n_valid on are padding): returns (residual stream [S,D], tokens [n_new])."""
    embeds = _f32(embeds); S, D = embeds.shape
    m, keep = _orc_model(weights)
    hidden = np.empty((S, D), np.float32)
    out = np.zeros(max(n_new, 1), np.int32)
    _lib.orc_model_forward_embeds(C.byref(m), _p(embeds), C.c_int(S), C.c_int(n_valid), C.c_int(n_new), _p(hidden), _p(out))
    return hidden, out[:n_new]


def hmt_prefill(weights, embeds, t_embed, wq, wk, seg_len, sum_len, rec_len, mem_num, n_new=0, pad=16):
    """The HMT segment recurrence (Modules/HMT.h:8-195 segment loop, :278-355 cross-attention, :357-470 memory caches)
    for one long sequence given as embeddings [T,D]: per segment, stage 0 = prefill of [T_tok, first sum_len tokens, T_tok]
    whose last row S_n queries the memory (Q = Wq S_n, scores against the cached keys, dec_Softmax with scale sqrt(D),
    P_n = sum_s A_s M_s); stage 1 = prefill of [P_n, rec_len tail tokens of the previous segment, the segment, P_n] whose
    last row M_n and its key Wk M_n go into slot seg % mem_num. Returns dict(P, M, K per segment, hidden of the last
    stage-1 run, n_valid of that run, tokens)."""
    embeds = _f32(embeds); T, D = embeds.shape
    seg_num = (T + seg_len - 1) // seg_len
    mem = np.zeros((mem_num, D), np.float32); kmem = np.zeros((mem_num, D), np.float32)
    Pn = np.zeros(D, np.float32)
    scale = np.float32(np.sqrt(np.float32(D)))
    rec = dict(P=[], M=[], K=[], S=[])
    padded = lambda n: (n + pad - 1) // pad * pad
    hidden = None; tokens = None; n1 = 0
    for seg in range(seg_num):
        cur = seg_len if seg < seg_num - 1 else T - seg * seg_len
        sl = min(cur, sum_len); off = seg * seg_len
        if seg > 0:
            n0 = 1 + sl + 1
            x0 = np.zeros((padded(n0), D), np.float32)
            x0[0] = t_embed; x0[1:1 + sl] = embeds[off:off + sl]; x0[1 + sl] = t_embed
            h0, _ = model_forward_embeds(weights, x0, n0)
            Sn = h0[1 + sl]
            Qn = linear_fp32_chain4(Sn, wq)
            A = linear_fp32_chain4(Qn, kmem)
            Pa = softmax_dec(A, 4, scale)
            Pn = linear_fp32_chain4(Pa, np.ascontiguousarray(mem.T))
            rec["S"].append(Sn); rec["P"].append(Pn)
        last = seg == seg_num - 1
        n1 = 1 + rec_len + cur + (0 if last else 1)
        x1 = np.zeros((padded(n1), D), np.float32)
        x1[0] = Pn
        for i in range(rec_len):
            j = off - rec_len + i
            if j >= 0:
                x1[1 + i] = embeds[j]
        x1[1 + rec_len:1 + rec_len + cur] = embeds[off:off + cur]
        if not last:
            x1[1 + rec_len + cur] = Pn
        hidden, tokens = model_forward_embeds(weights, x1, n1, n_new if last else 0)
        if not last:
            Mn = hidden[1 + rec_len + cur].copy()
            Kn = linear_fp32_chain4(Mn, wk)
            mem[seg % mem_num] = Mn; kmem[seg % mem_num] = Kn
            rec["M"].append(Mn); rec["K"].append(Kn)
    rec.update(hidden=hidden, n_valid=n1, tokens=tokens)
    return rec


# ------------------------------------------------------------------ Tier A (reference templates)
class _Ref:
    """The reference's own operator templates (available only where oracle/_ref was built)."""

    def __init__(self, lib):
        self.lib = lib

    def quant_per_token(self, x, decode=False):
        x = _f32(x); M, K = x.shape
        q = np.empty((M, K), np.int8); s = np.empty(M, np.float32)
        fn = self.lib.ref_dec_quant_per_token if decode else self.lib.ref_quant_per_token
        fn(_p(x), C.c_int(M), C.c_int(K), _p(q), _p(s))
        return q, s

    def quant_per_token_asym4(self, x):
        x = _f32(x); M, K = x.shape
        q = np.empty((M, K), np.uint8); s = np.empty(M, np.float32); b = np.empty(M, np.float32)
        self.lib.ref_quant_per_token_asym4(_p(x), C.c_int(M), C.c_int(K), _p(q), _p(s), _p(b))
        return q, s, b

    def dequant_asym(self, acc, s_tok, b_tok, s_ch, wsum):
        acc = _i32(acc); M, N = acc.shape; y = np.empty((M, N), np.float32)
        self.lib.ref_dequant_asym(_p(acc), _p(_f32(s_tok)), _p(_f32(b_tok)), _p(_f32(s_ch)), _p(_f32(wsum)), C.c_int(M), C.c_int(N), _p(y))
        return y

    def gemm_u4s4(self, a, w):
        a = np.ascontiguousarray(a, dtype=np.uint8); w = _i8(w); M, K = a.shape; N = w.shape[0]; acc = np.empty((M, N), np.int32)
        self.lib.ref_gemm_u4s4(_p(a), _p(w), C.c_int(M), C.c_int(N), C.c_int(K), _p(acc))
        return acc

    def linear_fp32(self, x, w):
        x = _f32(x); w = _f32(w); N, K = w.shape; y = np.empty(N, np.float32)
        rc = self.lib.ref_linear_fp32(_p(x), _p(w), C.c_int(N), C.c_int(K), _p(y))
        assert rc == 0
        return y

    def softmax_dec4_64(self, x, scale):
        x = _f32(x); assert x.size == 64
        p = np.empty_like(x)
        self.lib.ref_softmax_dec4_64(_p(x), C.c_float(scale), _p(p))
        return p

    def dequant(self, acc, s_tok, s_ch):
        acc = _i32(acc); M, N = acc.shape; y = np.empty((M, N), np.float32)
        self.lib.ref_dequant(_p(acc), _p(_f32(s_tok)), _p(_f32(s_ch)), C.c_int(M), C.c_int(N), _p(y))
        return y

    def gemm_s8s8(self, a, w):
        a = _i8(a); w = _i8(w); M, K = a.shape; N = w.shape[0]; acc = np.empty((M, N), np.int32)
        self.lib.ref_gemm_s8s8(_p(a), _p(w), C.c_int(M), C.c_int(N), C.c_int(K), _p(acc))
        return acc

    def gemm_u8s8(self, a, w):
        a = np.ascontiguousarray(a, dtype=np.uint8); w = _i8(w); M, K = a.shape; N = w.shape[0]
        acc = np.empty((M, N), np.int32)
        self.lib.ref_gemm_u8s8(_p(a), _p(w), C.c_int(M), C.c_int(N), C.c_int(K), _p(acc))
        return acc

    def fht(self, x, scale, decode=False):
        x = _f32(x); N = x.shape[-1]; rows = x.size // N; y = np.empty_like(x)
        fn = self.lib.ref_dec_fht if decode else self.lib.ref_fht
        rc = fn(_p(x), C.c_long(rows), C.c_int(N), C.c_float(scale), _p(y))
        assert rc == 0
        return y

    def rope_prefill(self, x, cos_t, sin_t):
        x = _f32(x); S, H, _ = x.shape; y = np.empty_like(x)
        rc = self.lib.ref_rope_prefill(_p(x), _p(_f32(cos_t)), _p(_f32(sin_t)), C.c_int(S), C.c_int(H), _p(y))
        assert rc == 0
        return y

    def rope_decode(self, x, cos_t, sin_t, pos):
        x = _f32(x); H, _ = x.shape; y = np.empty_like(x); cos_t = _f32(cos_t)
        rc = self.lib.ref_rope_decode(_p(x), _p(cos_t), _p(_f32(sin_t)), C.c_int(cos_t.shape[0]), C.c_int(pos),
                                      C.c_int(H), _p(y))
        assert rc == 0
        return y

    def softmax_prefill(self, x, causal):
        x = _f32(x); S, L = x.shape; p = np.empty_like(x)
        rc = self.lib.ref_softmax_prefill(_p(x), C.c_int(S), C.c_int(L), C.c_int(1 if causal else 0), _p(p))
        assert rc == 0
        return p

    def softmax_decode(self, x):
        x = _f32(x); p = np.empty_like(x)
        rc = self.lib.ref_softmax_decode(_p(x), C.c_int(x.size), _p(p))
        assert rc == 0
        return p

    def rmsnorm(self, x, gamma, lanes=0):
        x = _f32(x); M, D = x.shape; y = np.empty_like(x)
        if lanes == 0:
            self.lib.ref_rmsnorm_prefill(_p(x), _p(_f32(gamma)), C.c_int(M), C.c_int(D), _p(y))
        else:
            rc = self.lib.ref_rmsnorm_decode(_p(x), _p(_f32(gamma)), C.c_int(M), C.c_int(D), C.c_int(lanes), _p(y))
            assert rc == 0
        return y

    def silu(self, g):
        g = _f32(g); y = np.empty_like(g)
        self.lib.ref_silu(_p(g), C.c_long(g.size), _p(y))
        return y

    def gate_mul(self, a, b):
        a = _f32(a); b = _f32(b); y = np.empty_like(a)
        self.lib.ref_gate_mul(_p(a), _p(b), C.c_long(a.size), _p(y))
        return y

    def residual(self, a, b):
        a = _f32(a); b = _f32(b); y = np.empty_like(a)
        self.lib.ref_residual(_p(a), _p(b), C.c_long(a.size), _p(y))
        return y

    def static_quant(self, x, s, f=1.0, signed=True):
        x = _f32(x); rows, n = x.shape; q = np.empty((rows, n), np.uint8)
        self.lib.ref_static_quant(_p(x), C.c_long(rows), C.c_int(n), C.c_float(s), C.c_float(f),
                                  C.c_int(1 if signed else 0), _p(q))
        return q.view(np.int8) if signed else q

    def scale_stream_quant(self, x, s, signed=True):
        x = _f32(x); rows, n = x.shape; q = np.empty((rows, n), np.uint8)
        self.lib.ref_scale_stream_quant(_p(x), C.c_long(rows), C.c_int(n), _p(_f32(s)), C.c_int(1 if signed else 0), _p(q))
        return q.view(np.int8) if signed else q

    def scale_stream_dequant(self, acc, s_row, s_col):
        acc = _i32(acc); M, N = acc.shape; y = np.empty((M, N), np.float32)
        self.lib.ref_scale_stream_dequant(_p(acc), _p(_f32(s_row)), _p(_f32(s_col)), C.c_int(M), C.c_int(N), _p(y))
        return y

    def head_quant(self, x):
        x = _f32(x); H, _ = x.shape; q = np.empty((H, 64), np.int8); s = np.empty(H, np.float32)
        self.lib.ref_head_quant(_p(x), C.c_int(H), _p(q), _p(s))
        return q, s

    def mha_qxk(self, q, k):
        q = _i8(q); k = _i8(k); S, G, _ = q.shape; acc = np.empty((S, G, S), np.int32)
        rc = self.lib.ref_mha_qxk(_p(q), _p(k), C.c_int(S), C.c_int(G), _p(acc))
        assert rc == 0
        return acc

    def mha_axv(self, p, v):
        p = np.ascontiguousarray(p, dtype=np.uint8); v = _i8(v); S, G, _ = p.shape
        acc = np.empty((S, G, 64), np.int32)
        rc = self.lib.ref_mha_axv(_p(p), _p(v), C.c_int(S), C.c_int(G), _p(acc))
        assert rc == 0
        return acc

    def topk_sample(self, logits, rnd, lanes=32):
        """The reference's dec_Sampling_Embedding_Layer (top_k = 5) row by row."""
        logits = _f32(logits); B, V = logits.shape; idx = np.empty(B, np.int32)
        one = np.empty(1, np.int32)
        for b in range(B):
            rc = self.lib.ref_topk_sample(_p(np.ascontiguousarray(logits[b])), C.c_int(V), C.c_int(lanes), C.c_float(float(rnd[b])), _p(one))
            if rc != 0:
                raise ValueError("ref_topk_sample: unsupported shape")
            idx[b] = one[0]
        return idx

    def argmax(self, logits):
        logits = _f32(logits); B, V = logits.shape; idx = np.empty(B, np.int32)
        self.lib.ref_argmax(_p(logits), C.c_int(B), C.c_long(V), _p(idx))
        return idx


ref = _Ref(_ref) if _ref is not None else None
