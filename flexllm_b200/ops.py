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
def pref_Linear_Layer_i8xi8(a, s_tok, w, s_ch, want_acc=False, want_y=True):
    """Prefill W8A8 linear layer. a [M,K] int8, w [N,K] int8. Returns (acc int32 | None, y fp32 | None)."""
    M, K = a.shape; N = w.shape[0]
    acc = torch.empty((M, N), dtype=torch.int32, device=a.device) if want_acc else None
    y = torch.empty((M, N), dtype=torch.float32, device=a.device) if want_y else None
    _call("flexllm_linear_prefill_i8", _ptr(a), _ptr(s_tok), _ptr(w), _ptr(s_ch), M, N, K, _ptr(acc), _ptr(y))
    return acc, y


def dec_Linear_Layer_i8xi8(a, s_tok, w, s_ch, want_acc=False, want_y=True):
    """Decode W8A8 linear layer, M <= 64 tokens."""
    M, K = a.shape; N = w.shape[0]
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
