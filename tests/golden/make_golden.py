"""Generates tests/golden/reference_ops.npz by running the reference's own operator templates
(oracle/_ref/libflexllm_ref.so, built from the reference sources through oracle/ref_shim).
Run from the repository root where the reference checkout is available:

    make -C oracle && python tests/golden/make_golden.py

Inputs are seeded; every array needed to replay a case is stored beside its expected output.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

R = oracle.ref
assert R is not None, "oracle/_ref/libflexllm_ref.so missing: build it with `make -C oracle`"
g = np.random.default_rng(20240)
out = {}

# per-token quantisation (quant.h:6), prefill and decode forms
x = (g.standard_normal((8, 256)) * 2.5).astype(np.float32); x[3] = 0
out["quant_x"] = x
out["quant_q"], out["quant_s"] = R.quant_per_token(x)
qd, sd = R.quant_per_token(x, decode=True)
assert np.array_equal(qd, out["quant_q"]) and np.array_equal(sd, out["quant_s"])

# integer matmuls through the systolic array (MHA.h:114) + dequant (quant.h:116)
a = g.integers(-127, 128, (8, 512), dtype=np.int8); w = g.integers(-127, 128, (32, 512), dtype=np.int8)
out["gemm_a"], out["gemm_w"] = a, w
out["gemm_acc"] = R.gemm_s8s8(a, w)
st = g.uniform(0.005, 0.05, 8).astype(np.float32); sc = g.uniform(0.001, 0.01, 32).astype(np.float32)
out["deq_st"], out["deq_sc"] = st, sc
out["deq_y"] = R.dequant(out["gemm_acc"], st, sc)
pu = g.integers(0, 256, (8, 128), dtype=np.uint8); wv = g.integers(-127, 128, (16, 128), dtype=np.int8)
out["gemmu_a"], out["gemmu_w"] = pu, wv
out["gemmu_acc"] = R.gemm_u8s8(pu, wv)

# FHT (FHT.h:8 / :70)
f64 = g.standard_normal((4, 64)).astype(np.float32)
out["fht64_x"], out["fht64_y"] = f64, R.fht(f64, 8.0)
f8k = g.standard_normal((1, 8192)).astype(np.float32)
out["fht8192_x"], out["fht8192_y"] = f8k, R.fht(f8k, 90.50966799)
assert np.array_equal(out["fht8192_y"].view(np.uint32), R.fht(f8k, 90.50966799, decode=True).view(np.uint32))

# RoPE (RoPE.h:9) with the llama3 table
cos_t, sin_t = oracle.rope_table(64)
rx = g.standard_normal((64, 2, 64)).astype(np.float32)
out["rope_cos"], out["rope_sin"], out["rope_x"] = cos_t, sin_t, rx
out["rope_y"] = R.rope_prefill(rx, cos_t, sin_t)

# causal mask + softmax (MHA.h:247, Softmax.h:7) and the ragged decode softmax (Softmax.h:457)
sx = (g.standard_normal((16, 16)) * 4).astype(np.float32)
out["softmax_x"] = sx
out["softmax_causal"] = R.softmax_prefill(sx, causal=True)
out["softmax_full"] = R.softmax_prefill(sx, causal=False)
sd_ = (g.standard_normal(1027) * 3).astype(np.float32)
out["softmax_dec_x"], out["softmax_dec_p"] = sd_, R.softmax_decode(sd_)

# RMSNorm, both summation orders (LayerNorm.h:29, :211)
nx = g.standard_normal((3, 2048)).astype(np.float32); gm = (1 + 0.02 * g.standard_normal(2048)).astype(np.float32)
out["rms_x"], out["rms_gamma"] = nx, gm
out["rms_prefill"] = R.rmsnorm(nx, gm, 0)
out["rms_dec4"] = R.rmsnorm(nx, gm, 4)
out["rms_dec8"] = R.rmsnorm(nx, gm, 8)

# SiLU, gate, residual (Swish.h:6, Linear_Layer.h:613, Residual_Layer.h:47)
sa = (g.standard_normal(2048) * 4).astype(np.float32); sb = g.standard_normal(2048).astype(np.float32)
out["silu_x"], out["silu_u"] = sa, sb
out["silu_y"] = R.silu(sa)
out["silu_mul_y"] = R.gate_mul(out["silu_y"], sb)
out["residual_y"] = R.residual(sa, sb)

# static quantisers (quant.h:253 signed/unsigned, :167 scale stream)
qx = (g.standard_normal((4, 64)) * 2).astype(np.float32)
out["sq_x"] = qx
out["sq_signed"] = R.static_quant(qx, 0.01, 8.0, True)
pp = g.uniform(0, 1.3, (4, 64)).astype(np.float32)
out["sq_p"] = pp
out["sq_unsigned"] = R.static_quant(pp, 1 / 255, 1.0, False)

# greedy token (Logits.h:6)
lg = g.standard_normal((4, 3000)).astype(np.float32); lg[1, 77] = lg[1, 2100] = 9.0
out["argmax_x"], out["argmax_i"] = lg, R.argmax(lg)

path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_ops.npz")
np.savez_compressed(path, **out)
print("wrote", path, os.path.getsize(path), "bytes")
