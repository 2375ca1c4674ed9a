"""Thin torch-tensor front end over the C ABI (one function per entry point of flexllm_b200.h).

Function names follow the reference's operator templates (``Modules/*.h``): ``pref_*`` for the
token-parallel (prefill) operators, ``dec_*`` for the single-token (decode) ones. Every function
takes CUDA tensors, allocates its outputs with torch, and launches on the current torch stream.
"""
import ctypes as C

import torch

from . import _lib

_handle = None


class FlexLLMError(RuntimeError):
    def __init__(self, fn, status):
        l = lib()
        msg = l.flexllm_status_string(status).decode()
        super().__init__(f"{fn} failed: {msg} (status {status}, cuda error {l.flexllm_last_cuda_error()})")
        self.status = status


def lib():
    global _handle
    if _handle is None:
        _handle = _lib.load()
    return _handle


def _check(fn, st):
    if st != 0:
        raise FlexLLMError(fn, st)


def _ptr(t):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "flexllm_b200 takes contiguous CUDA tensors"
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _call(name, *args):
    _check(name, getattr(lib(), name)(*args, _stream()))


# ------------------------------------------------------------------------------ linear layers
def pref_Linear_Layer_i8xi8(a, s_tok, w, s_ch, want_acc=False, want_y=True, residual=None):
    """Prefill W8A8 linear layer. a [M,K] int8, w [N,K] int8. Returns (acc int32 | None, y fp32 | None).
    With residual [M,N] the following Residual_Layer is fused: y = residual + dequant."""
    M, K = a.shape; N = w.shape[0]
    if residual is not None:
        y = torch.empty((M, N), dtype=torch.float32, device=a.device)
        _call("flexllm_linear_prefill_i8_residual", _ptr(a), _ptr(s_tok), _ptr(w), _ptr(s_ch), M, N, K, _ptr(residual), _ptr(y))
        return None, y
    acc = torch.empty((M, N), dtype=torch.int32, device=a.device) if want_acc else None
    y = torch.empty((M, N), dtype=torch.float32, device=a.device) if want_y else None
    _call("flexllm_linear_prefill_i8", _ptr(a), _ptr(s_tok), _ptr(w), _ptr(s_ch), M, N, K, _ptr(acc), _ptr(y))
    return acc, y


def dec_Linear_Layer_i8xi8(a, s_tok, w, s_ch, want_acc=False, want_y=True, residual=None):
    """Decode W8A8 linear layer, M <= 64 tokens (optionally fused with the residual add)."""
    M, K = a.shape; N = w.shape[0]
    if residual is not None:
        y = torch.empty((M, N), dtype=torch.float32, device=a.device)
        _call("flexllm_linear_decode_i8_residual", _ptr(a), _ptr(s_tok), _ptr(w), _ptr(s_ch), M, N, K, _ptr(residual), _ptr(y))
        return None, y
    acc = torch.empty((M, N), dtype=torch.int32, device=a.device) if want_acc else None
    y = torch.empty((M, N), dtype=torch.float32, device=a.device) if want_y else None
    _call("flexllm_linear_decode_i8", _ptr(a), _ptr(s_tok), _ptr(w), _ptr(s_ch), M, N, K, _ptr(acc), _ptr(y))
    return acc, y


# ------------------------------------------------------------------------------ quant.h
def pref_quant_layer_fp32_qint(x):
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    _call("flexllm_quant_per_token", _ptr(x), M, K, _ptr(q), _ptr(s))
    return q, s


dec_quant_layer_fp32_qint = pref_quant_layer_fp32_qint


def pref_quant_layer_fp32_qint_asym(x, bits=4):
    """Asymmetric per-token quantiser of the reference's shipped configuration (quant.h:53-81, is_act_asym = true).
    Returns (q uint8 [M,K] in [0, 2^bits-1], scale [M], zero point [M])."""
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.uint8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    b = torch.empty((M,), dtype=torch.float32, device=x.device)
    _call("flexllm_quant_per_token_asym", _ptr(x), M, K, bits, _ptr(q), _ptr(s), _ptr(b))
    return q, s, b


def pref_dequant_layer_qint_fp32_asym(acc, s_tok, b_tok, s_ch, wsum):
    """y = ((float)acc * s_tok) * s_ch + b_tok * wsum (quant.h:146-148)."""
    M, N = acc.shape
    y = torch.empty((M, N), dtype=torch.float32, device=acc.device)
    _call("flexllm_dequant_asym", _ptr(acc), _ptr(s_tok), _ptr(b_tok), _ptr(s_ch), _ptr(wsum), M, N, _ptr(y))
    return y


def pref_Linear_Layer_i4xi4(a, s_tok, b_tok, w, s_ch, wsum, decode=False):
    """The reference's asymmetric-activation linear layer (pref_/dec_Linear_Layer_i4xi4 with is_uint_input + the asymmetric
    dequantiser): a uint8 [M,K] from the asymmetric quantiser, w int8 [N,K]. Returns (acc int32, y fp32)."""
    M, K = a.shape; N = w.shape[0]
    acc = torch.empty((M, N), dtype=torch.int32, device=a.device)
    y = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _call("flexllm_linear_decode_asym" if decode else "flexllm_linear_prefill_asym", _ptr(a), _ptr(s_tok), _ptr(b_tok), _ptr(w),
          _ptr(s_ch), _ptr(wsum), M, N, K, _ptr(acc), _ptr(y))
    return acc, y


def dec_Linear_Layer_i4xi4(a, s_tok, b_tok, w, s_ch, wsum):
    return pref_Linear_Layer_i4xi4(a, s_tok, b_tok, w, s_ch, wsum, decode=True)


def pref_dequant_layer_qint_fp32(acc, s_tok, s_ch):
    M, N = acc.shape
    y = torch.empty((M, N), dtype=torch.float32, device=acc.device)
    _call("flexllm_dequant", _ptr(acc), _ptr(s_tok), _ptr(s_ch), M, N, _ptr(y))
    return y


def pref_static_sym_quant_layer_fp32_qint(x, s, f=1.0, signed=True):
    """s: tensor with one element (per-tensor) or one per row."""
    rows, n = x.shape
    q = torch.empty((rows, n), dtype=torch.uint8, device=x.device)
    stride = 0 if s.numel() == 1 else 1
    _call("flexllm_static_quant", _ptr(x), rows, n, _ptr(s), stride, float(f), 1 if signed else 0, _ptr(q))
    return q.view(torch.int8) if signed else q


# ------------------------------------------------------------------------------ FHT.h
def pref_FHT(x, scale):
    N = x.shape[-1]
    y = torch.empty_like(x)
    _call("flexllm_fht", _ptr(x), x.numel() // N, N, float(scale), _ptr(y))
    return y


dec_FHT = pref_FHT


def swiglu_fht_quant(g, u, scale=90.50966799, want_act=False):
    """silu(g)*u -> FHT-8192/scale -> per-token int8. Returns (q, s, act | None)."""
    M, N = g.shape
    q = torch.empty((M, N), dtype=torch.int8, device=g.device)
    s = torch.empty((M,), dtype=torch.float32, device=g.device)
    act = torch.empty_like(g) if want_act else None
    _call("flexllm_swiglu_fht_quant", _ptr(g), _ptr(u), M, N, float(scale), _ptr(q), _ptr(s), _ptr(act))
    return q, s, act


# ------------------------------------------------------------------------------ RoPE.h
def pref_RoPE_layer(x, pos, cos_t, sin_t):
    T, H, D = x.shape
    assert D == 64
    y = torch.empty_like(x)
    _call("flexllm_rope", _ptr(x), _ptr(pos), _ptr(cos_t), _ptr(sin_t), T, H, _ptr(y))
    return y


dec_RoPE_layer = pref_RoPE_layer


def qk_prepare(q, s, pos, cos_t, sin_t):
    T, H, D = q.shape
    assert D == 64
    q2 = torch.empty_like(q)
    s2 = torch.empty((T, H), dtype=torch.float32, device=q.device)
    _call("flexllm_qk_prepare", _ptr(q), _ptr(s), _ptr(pos), _ptr(cos_t), _ptr(sin_t), T, H, _ptr(q2), _ptr(s2))
    return q2, s2


# ------------------------------------------------------------------------------ Softmax.h
def pref_Softmax(x, valid=None):
    L = x.shape[-1]
    p = torch.empty_like(x)
    _call("flexllm_softmax", _ptr(x), x.numel() // L, L, _ptr(valid), _ptr(p))
    return p


dec_MHA_Softmax = pref_Softmax


# ------------------------------------------------------------------------------ LayerNorm.h
NORM_PREFILL, NORM_DECODE4, NORM_DECODE8 = 0, 4, 8


def pref_Layer_Norm(x, gamma, eps=1e-5, order=NORM_PREFILL, quant=False, want_y=True):
    """RMSNorm; with quant=True also returns the per-token int8 quantisation of the result."""
    M, D = x.shape
    y = torch.empty_like(x) if want_y else None
    q = torch.empty((M, D), dtype=torch.int8, device=x.device) if quant else None
    s = torch.empty((M,), dtype=torch.float32, device=x.device) if quant else None
    _call("flexllm_rmsnorm_quant", _ptr(x), _ptr(gamma), M, D, float(eps), order, _ptr(y), _ptr(q), _ptr(s))
    return (y, q, s) if quant else y


def dec_Layer_Norm(x, gamma, eps=1e-5, lanes=8, quant=False, want_y=True):
    return pref_Layer_Norm(x, gamma, eps, lanes, quant, want_y)


# ------------------------------------------------------------------------------ Swish / gate / residual
def pref_Swish(g):
    y = torch.empty_like(g)
    _call("flexllm_swish", _ptr(g), g.numel(), _ptr(y))
    return y


def pref_Gate_Layer_fp32xfp32(a, b):
    y = torch.empty_like(a)
    _call("flexllm_gate", _ptr(a), _ptr(b), a.numel(), _ptr(y))
    return y


def pref_Residual_Layer(a, b):
    y = torch.empty_like(a)
    _call("flexllm_residual", _ptr(a), _ptr(b), a.numel(), _ptr(y))
    return y


dec_Swish, dec_Gate_Layer_fp32xfp32, dec_Residual_Layer = pref_Swish, pref_Gate_Layer_fp32xfp32, pref_Residual_Layer


# ------------------------------------------------------------------------------ Logits.h
def dec_Logits_argmax(logits):
    B, V = logits.shape
    idx = torch.empty((B,), dtype=torch.int32, device=logits.device)
    _call("flexllm_logits_argmax", _ptr(logits), B, V, _ptr(idx))
    return idx


def dec_Sampling_Layer(logits, rnd, lanes=32, top_k=5, details=False):
    """Top-k sampling of dec_Sampling_Embedding_Layer (Logits.h:145-279) without the embedding gather.
    logits [B,V] fp32, rnd [B] uniform numbers in [0,1) -> token ids [B] (and the merged top-k list)."""
    B, V = logits.shape
    idx = torch.empty((B,), dtype=torch.int32, device=logits.device)
    ti = torch.empty((B, top_k), dtype=torch.int32, device=logits.device) if details else None
    tv = torch.empty((B, top_k), dtype=torch.float32, device=logits.device) if details else None
    _call("flexllm_topk_sample", _ptr(logits), B, V, lanes, top_k, _ptr(rnd), _ptr(idx), _ptr(ti) if details else None,
          _ptr(tv) if details else None)
    return (idx, ti, tv) if details else idx


# ------------------------------------------------------------------------------ MHA_i8xi8
def MHA_i8xi8_Prefilling(q, qs, k, ks, v, vs, cos_t, sin_t, a_s, want_oacc=False):
    """Prefill GQA attention. q [B,S,HQ,64] s8, qs [B,S,HQ]; k,v [B,S,HKV,64], ks,vs [B,S,HKV];
    a_s [HQ]. Returns (out fp32 [B,S,HQ*64], oacc int32 | None)."""
    B, S, HQ, D = q.shape
    HKV = k.shape[2]
    assert D == 64
    nbytes = lib().flexllm_mha_prefill_workspace(B, S, HQ, HKV)
    ws = torch.empty((nbytes,), dtype=torch.uint8, device=q.device)
    out = torch.empty((B, S, HQ * 64), dtype=torch.float32, device=q.device)
    oacc = torch.empty((B, S, HQ * 64), dtype=torch.int32, device=q.device) if want_oacc else None
    _call("flexllm_mha_i8xi8_prefill", _ptr(q), _ptr(qs), _ptr(k), _ptr(ks), _ptr(v), _ptr(vs), _ptr(cos_t),
          _ptr(sin_t), _ptr(a_s), B, S, HQ, HKV, _ptr(out), _ptr(oacc), _ptr(ws), nbytes)
    return out, oacc


def dec_MLP_block(x, gamma, w_gu, s_gu, w_d, s_d, eps=1e-5, order=8, fht_scale=90.50966799, out=None, workspace=None):
    """Decode MLP block in one call: RMSNorm + quant -> gate|up -> SiLU * up -> FHT-8192 -> quant -> down + residual.
    x [M,D] fp32; w_gu [2F,D] int8 (gate rows, then up rows); w_d [D,F]. Returns y [M,D] fp32."""
    M, D = x.shape
    Fd = w_d.shape[1]
    nbytes = lib().flexllm_mlp_block_workspace(M, D, Fd)
    ws = workspace if workspace is not None else torch.empty((nbytes,), dtype=torch.uint8, device=x.device)
    y = out if out is not None else torch.empty_like(x)
    _call("flexllm_mlp_block_decode", _ptr(x), _ptr(gamma), _ptr(w_gu), _ptr(s_gu), _ptr(w_d), _ptr(s_d), M, D, Fd, eps, order,
          fht_scale, _ptr(y), _ptr(ws), ws.numel())
    return y


def MHA_i8xi8_Prefilling_online(q, qs, k, ks, v, vs, cos_t, sin_t):
    """Prefill GQA attention in one sweep with an online softmax: close to, not bit-identical with,
    MHA_i8xi8_Prefilling (no static P scale). Returns out fp32 [B,S,HQ*64]."""
    B, S, HQ, D = q.shape
    HKV = k.shape[2]
    assert D == 64
    nbytes = lib().flexllm_mha_prefill_workspace(B, S, HQ, HKV)
    ws = torch.empty((nbytes,), dtype=torch.uint8, device=q.device)
    out = torch.empty((B, S, HQ * 64), dtype=torch.float32, device=q.device)
    _call("flexllm_mha_i8xi8_prefill_online", _ptr(q), _ptr(qs), _ptr(k), _ptr(ks), _ptr(v), _ptr(vs), _ptr(cos_t),
          _ptr(sin_t), B, S, HQ, HKV, _ptr(out), _ptr(ws), nbytes)
    return out


class KVCache:
    """Paged int8 KV cache (library-owned device memory). Pools of one layer are exposed as torch
    views: k [n_pages,HKV,64,64] (token-major rows), v [n_pages,HKV,64 dims,64 tokens] (transposed
    inside the page), ks/vs [n_pages,HKV,64]."""

    def __init__(self, layers, n_pages, hkv, page=64, device="cuda"):
        self.layers, self.n_pages, self.hkv, self.page = layers, n_pages, hkv, page
        self._h = C.c_void_p()
        _check("flexllm_kv_cache_create", lib().flexllm_kv_cache_create(C.byref(self._h), layers, n_pages, hkv, page))
        self.device = torch.device(device)

    def close(self):
        if self._h:
            lib().flexllm_kv_cache_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset(self):
        _check("flexllm_kv_cache_reset", lib().flexllm_kv_cache_reset(self._h, _stream()))

    def _view(self, ptr, shape, dtype):
        n = 1
        for d in shape:
            n *= d
        esz = torch.empty((), dtype=dtype).element_size()
        buf = (C.c_byte * (n * esz)).from_address(ptr)
        # wrap device memory: torch needs a CUDA array interface
        class _Holder:
            pass
        h = _Holder()
        typestr = {torch.int8: "|i1", torch.float32: "<f4"}[dtype]
        h.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}
        return torch.as_tensor(h, device=self.device)

    def pools(self, layer):
        k, ks, v, vs = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
        _check("flexllm_kv_cache_pools", lib().flexllm_kv_cache_pools(self._h, layer, C.byref(k), C.byref(ks), C.byref(v), C.byref(vs)))
        P, H, T = self.n_pages, self.hkv, self.page
        return (self._view(k.value, (P, H, T, 64), torch.int8), self._view(ks.value, (P, H, T), torch.float32),
                self._view(v.value, (P, H, 64, T), torch.int8), self._view(vs.value, (P, H, T), torch.float32))


def dec_KV_cache_append(cache, layer, k, ks, v, vs, page_table, ctx, max_ctx):
    """Stores k,v [B,HKV,64] int8 with scales ks,vs [B,HKV] at position ctx[b] of each sequence (the cache managers'
    append, Modules/MHA.h:484-513, :773-801)."""
    B = k.shape[0]
    _check("flexllm_kv_append", lib().flexllm_kv_append(cache._h, layer, _ptr(k), _ptr(ks), _ptr(v), _ptr(vs), _ptr(page_table),
                                                         page_table.shape[1], _ptr(ctx), max_ctx, B, _stream()))


def MHA_i8xi8_Decoding(cache, layer, q, qs, k, ks, v, vs, cos_t, sin_t, a_s, page_table, ctx, max_ctx, want_oacc=False):
    """One decode step of attention on `layer`. q [B,HQ,64] s8, qs [B,HQ]; k,v [B,HKV,64], ks,vs [B,HKV];
    page_table [B,max_pages] int32; ctx [B] int32 (tokens already cached, device); max_ctx >= max(ctx).
    The new k,v are appended to the cache. Returns (out fp32 [B,HQ*64], oacc | None)."""
    B, HQ, D = q.shape
    assert D == 64
    nbytes = lib().flexllm_mha_decode_workspace(B, HQ, max_ctx)
    ws = torch.empty((nbytes,), dtype=torch.uint8, device=q.device)
    out = torch.empty((B, HQ * 64), dtype=torch.float32, device=q.device)
    oacc = torch.empty((B, HQ * 64), dtype=torch.int32, device=q.device) if want_oacc else None
    _check("flexllm_mha_i8xi8_decode", lib().flexllm_mha_i8xi8_decode(
        cache._h, layer, _ptr(q), _ptr(qs), _ptr(k), _ptr(ks), _ptr(v), _ptr(vs), _ptr(cos_t), _ptr(sin_t), _ptr(a_s),
        _ptr(page_table), page_table.shape[1], _ptr(ctx), max_ctx, B, HQ, _ptr(out), _ptr(oacc), _ptr(ws), nbytes, _stream()))
    return out, oacc


def read_reference_layer(directory, layer, hidden, kv_hidden, ffn, heads_q):
    """One decoder layer of a checkpoint in the reference's on-disk format (its demo's parameters/ directory) as CPU
    tensors: keys wq wk wv wo wg wu wd (int8 [out,in]), sq.. sd (scales), sumq.. sumd (row sums of the asymmetric
    dequantiser), gamma0 gamma1 a_s. The first 17 are what Model.load_layer takes."""
    dims = dict(q=(hidden, hidden), k=(kv_hidden, hidden), v=(kv_hidden, hidden), o=(hidden, hidden), g=(ffn, hidden), u=(ffn, hidden),
                d=(hidden, ffn))
    out = {}
    for k, (n, kk) in dims.items():
        out["w" + k] = torch.empty((n, kk), dtype=torch.int8)
        out["s" + k] = torch.empty((n,), dtype=torch.float32)
        out["sum" + k] = torch.empty((n,), dtype=torch.float32)
    out["gamma0"] = torch.empty((hidden,), dtype=torch.float32); out["gamma1"] = torch.empty((hidden,), dtype=torch.float32)
    out["a_s"] = torch.empty((heads_q,), dtype=torch.float32)
    b = _lib.CkptLayerBuffers(*[C.c_void_p(out[n].data_ptr()) for n, _ in _lib.CkptLayerBuffers._fields_])
    _check("flexllm_ckpt_load_layer", lib().flexllm_ckpt_load_layer(str(directory).encode(), layer, hidden, kv_hidden, ffn, heads_q, C.byref(b)))
    return out


def read_reference_head(directory, layers, hidden, vocab, table_len, want_embed=False):
    """lm_head (int8 + scales + row sums), final RMSNorm weight, RoPE tables and optionally the fp32 embedding table."""
    out = dict(lm_w=torch.empty((vocab, hidden), dtype=torch.int8), lm_s=torch.empty((vocab,), dtype=torch.float32),
               lm_sum=torch.empty((vocab,), dtype=torch.float32), gamma_final=torch.empty((hidden,), dtype=torch.float32),
               cos_t=torch.empty((table_len, 32), dtype=torch.float32), sin_t=torch.empty((table_len, 32), dtype=torch.float32))
    if want_embed:
        out["embed"] = torch.empty((vocab, hidden), dtype=torch.float32)
    p = lambda n: C.c_void_p(out[n].data_ptr()) if n in out else None
    _check("flexllm_ckpt_load_head", lib().flexllm_ckpt_load_head(str(directory).encode(), layers, hidden, vocab, table_len, p("lm_w"), p("lm_s"),
                                                                  p("lm_sum"), p("gamma_final"), p("cos_t"), p("sin_t"), p("embed")))
    return out


class HMT:
    """HMT long-context plug-in (Modules/HMT.h) on a Model: segment recurrence with a ring of memory vectors."""

    def __init__(self, model, hidden, wq, wk, t_embed, seg_len=990, sum_len=495, rec_len=32, mem_num=64):
        self.model, self.hidden = model, hidden
        self.cfg = _lib.HmtConfig(seg_len, sum_len, rec_len, mem_num)
        self._h = C.c_void_p()
        p = lambda t: C.c_void_p(t.contiguous().data_ptr())
        _check("flexllm_hmt_create", lib().flexllm_hmt_create(C.byref(self._h), model._h, C.byref(self.cfg), hidden, p(wq), p(wk), p(t_embed)))

    def close(self):
        if self._h:
            lib().flexllm_hmt_destroy(self._h)
            self._h = C.c_void_p()

    def prefill(self, embeds, want_trace=False):
        """embeds [T,hidden] fp32 CUDA. Returns (first token [1], trace [segments,4,hidden] | None)."""
        T = embeds.shape[0]
        nseg = (T + self.cfg.seg_len - 1) // self.cfg.seg_len
        nxt = torch.empty((1,), dtype=torch.int32, device=embeds.device)
        tr = torch.zeros((nseg, 4, self.hidden), dtype=torch.float32, device=embeds.device) if want_trace else None
        _check("flexllm_hmt_prefill", lib().flexllm_hmt_prefill(self._h, _ptr(embeds), T, _ptr(nxt), _ptr(tr), _stream()))
        return nxt, tr


def tp_unique_id():
    """128-byte NCCL id made on one rank; hand it to the others (e.g. torch.distributed broadcast)."""
    from . import build
    buf = (C.c_ubyte * 128)()
    _check("flexllm_tp_unique_id", lib().flexllm_tp_unique_id(buf, build.nccl_library().encode()))
    return bytes(buf)


class TensorParallel:
    """Communicator of one tensor-parallel rank (one process per GPU; the current CUDA device is used)."""

    def __init__(self, rank, size, unique_id):
        from . import build
        self.rank, self.size = rank, size
        self._h = C.c_void_p()
        idbuf = (C.c_ubyte * 128).from_buffer_copy(unique_id)
        _check("flexllm_tp_init", lib().flexllm_tp_init(C.byref(self._h), rank, size, idbuf, build.nccl_library().encode()))

    @classmethod
    def local_group(cls, size):
        """`size` communicators whose ranks share the current GPU (one host thread per rank, one stream): the
        partitioned model of any rank count on a single device, for checking its arithmetic."""
        hs = (C.c_void_p * size)()
        _check("flexllm_tp_init_local", lib().flexllm_tp_init_local(hs, size))
        group = []
        for r in range(size):
            t = cls.__new__(cls)
            t.rank, t.size, t._h = r, size, C.c_void_p(hs[r])
            group.append(t)
        return group

    def close(self):
        if self._h:
            lib().flexllm_tp_destroy(self._h)
            self._h = C.c_void_p()

    def allreduce_s32(self, t):
        _check("flexllm_tp_allreduce_s32", lib().flexllm_tp_allreduce_s32(self._h, _ptr(t), t.numel(), _stream()))
        return t

    def allgather(self, t):
        out = torch.empty((self.size,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        _check("flexllm_tp_allgather", lib().flexllm_tp_allgather(self._h, _ptr(t), _ptr(out), t.numel() * t.element_size(), _stream()))
        return out

    def reduce_scatter_s32(self, t):
        """t int32 [size, n]: returns block `rank` of the sum over the ranks, [n]."""
        out = torch.empty(t.shape[1:], dtype=torch.int32, device=t.device)
        _check("flexllm_tp_reduce_scatter_s32", lib().flexllm_tp_reduce_scatter_s32(self._h, _ptr(t), _ptr(out), out.numel(), _stream()))
        return out

    def allreduce_max_f32(self, t):
        _check("flexllm_tp_allreduce_max_f32", lib().flexllm_tp_allreduce_max_f32(self._h, _ptr(t), t.numel(), _stream()))
        return t

    def alltoall(self, t):
        """t [size, ...]: block p goes to rank p; returns the blocks received, indexed by source rank."""
        out = torch.empty_like(t)
        _check("flexllm_tp_alltoall", lib().flexllm_tp_alltoall(self._h, _ptr(t), _ptr(out), t[0].numel() * t.element_size(), _stream()))
        return out


class Model:
    """Whole-model runner (SpinQuant_Prefilling + SpinQuant_Decoding graphs). Weights are given as
    CUDA or CPU torch tensors (the library copies them; with `tp` every rank passes the full weights
    and keeps its slice)."""

    def __init__(self, layers, hidden, heads_q, heads_kv, ffn, vocab, max_batch, max_prefill, max_ctx, eps=1e-5, tp=None):
        import math
        self.cfg = _lib.ModelConfig(layers, hidden, heads_q, heads_kv, ffn, vocab, eps, float(torch.tensor(math.sqrt(ffn), dtype=torch.float32)),
                                    max_batch, max_prefill, max_ctx)
        self._h = C.c_void_p()
        self.tp = tp
        _check("flexllm_model_create_tp", lib().flexllm_model_create_tp(C.byref(self._h), C.byref(self.cfg), tp._h if tp else None))

    def close(self):
        if self._h:
            lib().flexllm_model_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _p(t):
        assert t.is_contiguous()
        return C.c_void_p(t.data_ptr())

    def load_layer(self, layer, **w):
        """Keys: wq wk wv wo wg wu wd sq sk sv so sg su sd gamma0 gamma1 a_s."""
        lw = _lib.LayerWeights(*[self._p(w[n]) for n, _ in _lib.LayerWeights._fields_])
        _check("flexllm_model_load_layer", lib().flexllm_model_load_layer(self._h, layer, C.byref(lw), _stream()))
        torch.cuda.current_stream().synchronize()   # sources may be freed by the caller afterwards

    def load_head(self, lm_w, lm_s, gamma_final, cos_t, sin_t):
        _check("flexllm_model_load_head", lib().flexllm_model_load_head(
            self._h, self._p(lm_w), self._p(lm_s), self._p(gamma_final), self._p(cos_t), self._p(sin_t), cos_t.shape[0], _stream()))
        torch.cuda.current_stream().synchronize()

    def prefill(self, tokens):
        B, S = tokens.shape
        nxt = torch.empty((B,), dtype=torch.int32, device=tokens.device)
        _check("flexllm_model_prefill", lib().flexllm_model_prefill(self._h, _ptr(tokens), B, S, _ptr(nxt), _stream()))
        return nxt

    def prefill_embeds(self, embeds, n_valid=None):
        """embeds [B,S,hidden] fp32 CUDA; rows n_valid.. are padding. Returns the first tokens [B]."""
        B, S, _ = embeds.shape
        nxt = torch.empty((B,), dtype=torch.int32, device=embeds.device)
        _check("flexllm_model_prefill_embeds", lib().flexllm_model_prefill_embeds(self._h, _ptr(embeds), B, S, S if n_valid is None else n_valid,
                                                                                  _ptr(nxt), _stream()))
        return nxt

    def embed_tokens(self, tokens, hidden):
        out = torch.empty((tokens.numel(), hidden), dtype=torch.float32, device=tokens.device)
        _check("flexllm_model_embed_tokens", lib().flexllm_model_embed_tokens(self._h, _ptr(tokens), tokens.numel(), _ptr(out), _stream()))
        return out

    def begin(self, n_new):
        _check("flexllm_model_begin", lib().flexllm_model_begin(self._h, n_new, _stream()))

    def decode(self, n_steps, use_graph=True):
        _check("flexllm_model_decode", lib().flexllm_model_decode(self._h, n_steps, 1 if use_graph else 0, _stream()))

    def generate_host(self, tokens_cpu, n_new, use_graph=True, out=None):
        """tokens_cpu: pinned or pageable CPU int32 [B,S]. Returns CPU int32 [B,n_new]."""
        B, S = tokens_cpu.shape
        if out is None:
            out = torch.empty((B, n_new), dtype=torch.int32)
        _check("flexllm_model_generate_host", lib().flexllm_model_generate_host(
            self._h, C.c_void_p(tokens_cpu.data_ptr()), B, S, n_new, C.c_void_p(out.data_ptr()), 1 if use_graph else 0, _stream()))
        return out

    def set_sampling(self, lanes=0, top_k=0, rnd=None):
        """top_k == 0: greedy. Else top-k sampling with uniform numbers rnd [n_new, B] (CUDA fp32; kept alive here)."""
        self._rnd = rnd.contiguous() if rnd is not None else None
        _check("flexllm_model_set_sampling", lib().flexllm_model_set_sampling(self._h, lanes, top_k, _ptr(self._rnd) if self._rnd is not None else None))

    def buffer(self, which, shape, dtype):
        p = C.c_void_p()
        _check("flexllm_model_buffer", lib().flexllm_model_buffer(self._h, which, C.byref(p)))
        class _H:
            pass
        h = _H()
        typestr = {torch.int32: "<i4", torch.float32: "<f4"}[dtype]
        h.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (p.value, False), "version": 2}
        return torch.as_tensor(h, device="cuda")
