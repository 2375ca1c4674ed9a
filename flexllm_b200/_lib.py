"""Loads libflexllm_b200.so and declares the C ABI of include/flexllm_b200.h for ctypes."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FLEXLLM_B200_LIB") or os.path.join(_HERE, "libflexllm_b200.so")   # the override is a development aid

OK, EINVAL, ECUDA, ETIMEDOUT, ENOTSUP, ENOMEM, ETOOBIG, EDEVDATA, EIO = 0, -1, -2, -3, -4, -5, -6, -7, -8

# name -> argument types, in the order of include/flexllm_b200.h (return type is int unless noted)
_P, _I, _L, _F, _SZ = C.c_void_p, C.c_int, C.c_long, C.c_float, C.c_size_t
SIGNATURES = {
    "flexllm_version": [],
    "flexllm_last_cuda_error": [],
    "flexllm_launch_count": [],
    "flexllm_device_status": [],
    "flexllm_linear_prefill_i8": [_P, _P, _P, _P, _I, _I, _I, _P, _P, _P],
    "flexllm_linear_decode_i8": [_P, _P, _P, _P, _I, _I, _I, _P, _P, _P],
    "flexllm_linear_prefill_i8_residual": [_P, _P, _P, _P, _I, _I, _I, _P, _P, _P],
    "flexllm_linear_decode_i8_residual": [_P, _P, _P, _P, _I, _I, _I, _P, _P, _P],
    "flexllm_linear_decode_i8_noalloc": [_P, _P, _P, _P, _I, _I, _I, _P, _P],
    "flexllm_quant_per_token": [_P, _I, _I, _P, _P, _P],
    "flexllm_dequant": [_P, _P, _P, _I, _I, _P, _P],
    "flexllm_quant_per_token_asym": [_P, _I, _I, _I, _P, _P, _P, _P],
    "flexllm_dequant_asym": [_P, _P, _P, _P, _P, _I, _I, _P, _P],
    "flexllm_linear_prefill_asym": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _P],
    "flexllm_linear_decode_asym": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _P],
    "flexllm_ckpt_read_bin": [C.c_char_p, _SZ, _SZ, _P],
    "flexllm_ckpt_read_c_array_f32": [C.c_char_p, C.c_char_p, _L, _L, _P],
    "flexllm_ckpt_load_layer": [C.c_char_p, _I, _I, _I, _I, _I, _P],
    "flexllm_ckpt_load_head": [C.c_char_p, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P],
    "flexllm_static_quant": [_P, _L, _I, _P, _I, _F, _I, _P, _P],
    "flexllm_fht": [_P, _L, _I, _F, _P, _P],
    "flexllm_rope": [_P, _P, _P, _P, _L, _I, _P, _P],
    "flexllm_softmax": [_P, _L, _I, _P, _P, _P],
    "flexllm_rmsnorm_quant": [_P, _P, _I, _I, _F, _I, _P, _P, _P, _P],
    "flexllm_swish": [_P, _L, _P, _P],
    "flexllm_gate": [_P, _P, _L, _P, _P],
    "flexllm_residual": [_P, _P, _L, _P, _P],
    "flexllm_swiglu_fht_quant": [_P, _P, _I, _I, _F, _P, _P, _P, _P],
    "flexllm_logits_argmax": [_P, _I, _L, _P, _P],
    "flexllm_topk_sample": [_P, _I, _L, _I, _I, _P, _P, _P, _P, _P],
    "flexllm_qk_prepare": [_P, _P, _P, _P, _P, _L, _I, _P, _P, _P],
    "flexllm_mha_prefill_workspace": [_I, _I, _I, _I],
    "flexllm_mlp_block_workspace": [_I, _I, _I],
    "flexllm_mlp_block_decode": [_P] * 6 + [_I, _I, _I, _F, _I, _F, _P, _P, _SZ, _P],
    "flexllm_mha_i8xi8_prefill": [_P] * 9 + [_I, _I, _I, _I, _P, _P, _P, _SZ, _P],
    "flexllm_mha_i8xi8_prefill_online": [_P] * 8 + [_I, _I, _I, _I, _P, _P, _SZ, _P],
    "flexllm_kv_cache_create": [_P, _I, _I, _I, _I],
    "flexllm_kv_cache_destroy": [_P],
    "flexllm_kv_cache_reset": [_P, _P],
    "flexllm_kv_cache_pools": [_P, _I, _P, _P, _P, _P],
    "flexllm_kv_append": [_P, _I, _P, _P, _P, _P, _P, _I, _P, _I, _I, _P],
    "flexllm_mha_decode_workspace": [_I, _I, _I],
    "flexllm_mha_i8xi8_decode": [_P, _I] + [_P] * 10 + [_I, _P, _I, _I, _I, _P, _P, _P, _SZ, _P],
    "flexllm_tp_unique_id": [_P, C.c_char_p],
    "flexllm_tp_init": [_P, _I, _I, _P, C.c_char_p],
    "flexllm_tp_init_local": [_P, _I],
    "flexllm_tp_is_local": [_P],
    "flexllm_tp_destroy": [_P],
    "flexllm_tp_rank": [_P],
    "flexllm_tp_size": [_P],
    "flexllm_tp_allreduce_s32": [_P, _P, _SZ, _P],
    "flexllm_tp_allgather": [_P, _P, _P, _SZ, _P],
    "flexllm_tp_reduce_scatter_s32": [_P, _P, _P, _SZ, _P],
    "flexllm_tp_allreduce_max_f32": [_P, _P, _SZ, _P],
    "flexllm_tp_alltoall": [_P, _P, _P, _SZ, _P],
    "flexllm_model_create": [_P, _P],
    "flexllm_model_create_tp": [_P, _P, _P],
    "flexllm_model_destroy": [_P],
    "flexllm_model_load_layer": [_P, _I, _P, _P],
    "flexllm_model_load_head": [_P, _P, _P, _P, _P, _P, _I, _P],
    "flexllm_model_prefill": [_P, _P, _I, _I, _P, _P],
    "flexllm_model_prefill_embeds": [_P, _P, _I, _I, _I, _P, _P],
    "flexllm_model_embed_tokens": [_P, _P, _I, _P, _P],
    "flexllm_hmt_create": [_P, _P, _P, _I, _P, _P, _P],
    "flexllm_hmt_destroy": [_P],
    "flexllm_hmt_prefill": [_P, _P, _I, _P, _P, _P],
    "flexllm_model_begin": [_P, _I, _P],
    "flexllm_model_decode": [_P, _I, _I, _P],
    "flexllm_model_generate_host": [_P, _P, _I, _I, _I, _P, _I, _P],
    "flexllm_model_set_sampling": [_P, _I, _I, _P],
    "flexllm_model_buffer": [_P, _I, _P],
    "flexllm_model_limits": [_P, _P, _P, _P],
    "flexllm_debug_hook": [_I, C.c_longlong],
    "flexllm_gemm_i8_mainloop_probe": [_P, _P, _I, _I, _I, _P],
}


class ModelConfig(C.Structure):
    _fields_ = [("layers", _I), ("hidden", _I), ("heads_q", _I), ("heads_kv", _I), ("ffn", _I), ("vocab", _I),
                ("eps", _F), ("fht_scale", _F), ("max_batch", _I), ("max_prefill", _I), ("max_ctx", _I)]


class CkptLayerBuffers(C.Structure):
    _fields_ = ([(n, _P) for n in ("wq", "wk", "wv", "wo", "wg", "wu", "wd")] + [(n, _P) for n in ("sq", "sk", "sv", "so", "sg", "su", "sd")] +
                [(n, _P) for n in ("sumq", "sumk", "sumv", "sumo", "sumg", "sumu", "sumd")] + [(n, _P) for n in ("gamma0", "gamma1", "a_s")])


class HmtConfig(C.Structure):
    _fields_ = [("seg_len", _I), ("sum_len", _I), ("rec_len", _I), ("mem_num", _I)]


class LayerWeights(C.Structure):
    _fields_ = [(n, _P) for n in ("wq", "wk", "wv", "wo", "wg", "wu", "wd", "sq", "sk", "sv", "so", "sg", "su", "sd",
                                  "gamma0", "gamma1", "a_s")]

RESTYPES = {"flexllm_status_string": C.c_char_p, "flexllm_launch_count": C.c_ulonglong, "flexllm_mha_prefill_workspace": C.c_size_t,
            "flexllm_mha_decode_workspace": C.c_size_t, "flexllm_mlp_block_workspace": C.c_size_t}


def load():
    """Returns the ctypes handle. Raises if the library has not been built: there is no fallback."""
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flexllm_b200.build` "
            "(flexllm_b200 has no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = RESTYPES.get(name, C.c_int)
    lib.flexllm_status_string.argtypes = [C.c_int]
    lib.flexllm_status_string.restype = C.c_char_p
    return lib
