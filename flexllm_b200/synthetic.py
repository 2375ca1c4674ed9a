"""Seeded synthetic weights and inputs of the Llama-3.2-1B W8A8 shapes (there are no real
checkpoints in this project: parity and throughput are measured on random-init weights).

int8 weights uniform in [-127,127], per-channel scales uniform in [0.001,0.01], RMSNorm weights
N(1, 0.02), static attention-probability scale a_s, llama3 RoPE table (theta 500000, factor 32,
low 1, high 4, original context 8192) evaluated in double precision.
"""
import math

import numpy as np

LLAMA32_1B = dict(layers=16, hidden=2048, heads_q=32, heads_kv=8, ffn=8192, vocab=128256)


def rope_table(P):
    """cos/sin tables [P,32] fp32 for head_dim 64."""
    i = np.arange(32, dtype=np.float64)
    inv = np.power(500000.0, (2.0 * i) / 64.0)
    f = 1.0 / inv
    wl = 2.0 * math.pi * inv
    a = (8192.0 / wl - 1.0) / (4.0 - 1.0)
    sf = np.where(wl < 8192.0 / 4.0, f, np.where(wl > 8192.0, f / 32.0, (1 - a) * (f / 32.0) + a * f))
    th = np.arange(P, dtype=np.float64)[:, None] * sf[None, :]
    return np.cos(th).astype(np.float32), np.sin(th).astype(np.float32)


def numpy_weights(layers, hidden, heads_q, heads_kv, ffn, vocab, max_ctx, seed=0, a_s=2.0 / 255):
    """Weights as numpy arrays (small configurations, shared with the CPU oracle in the tests)."""
    g = np.random.default_rng(seed)
    D, Q, KV = hidden, heads_q * 64, heads_kv * 64

    def w8(n, k):
        return g.integers(-127, 128, (n, k), dtype=np.int8)

    def sc(n):
        return g.uniform(0.001, 0.01, n).astype(np.float32)

    def gam():
        return (1 + 0.02 * g.standard_normal(D)).astype(np.float32)

    W = dict(HQ=heads_q, HKV=heads_kv)
    for name, (n, k) in dict(wq=(Q, D), wk=(KV, D), wv=(KV, D), wo=(D, D), wg=(ffn, D), wu=(ffn, D), wd=(D, ffn)).items():
        W[name] = [w8(n, k) for _ in range(layers)]
        W["s" + name[1:]] = [sc(n) for _ in range(layers)]
    W["g0"] = [gam() for _ in range(layers)]
    W["g1"] = [gam() for _ in range(layers)]
    W["a_s"] = [np.full(heads_q, a_s, np.float32) for _ in range(layers)]
    W["g_final"] = gam()
    W["lm_w"] = w8(vocab, D)
    W["lm_s"] = sc(vocab)
    W["cos_t"], W["sin_t"] = rope_table(max_ctx + 1)
    return W


def load_numpy_weights(model, W):
    import torch
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    for l in range(len(W["wq"])):
        model.load_layer(l, wq=t(W["wq"][l]), wk=t(W["wk"][l]), wv=t(W["wv"][l]), wo=t(W["wo"][l]), wg=t(W["wg"][l]),
                         wu=t(W["wu"][l]), wd=t(W["wd"][l]), sq=t(W["sq"][l]), sk=t(W["sk"][l]), sv=t(W["sv"][l]),
                         so=t(W["so"][l]), sg=t(W["sg"][l]), su=t(W["su"][l]), sd=t(W["sd"][l]), gamma0=t(W["g0"][l]),
                         gamma1=t(W["g1"][l]), a_s=t(W["a_s"][l]))
    model.load_head(t(W["lm_w"]), t(W["lm_s"]), t(W["g_final"]), t(W["cos_t"]), t(W["sin_t"]))


def load_random_weights(model, layers, hidden, heads_q, heads_kv, ffn, vocab, max_ctx, seed=0, a_s=2.0 / 255, device="cuda"):
    """Full-size random weights generated on the device (throughput runs)."""
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    D, Q, KV = hidden, heads_q * 64, heads_kv * 64

    def w8(n, k):
        return torch.randint(-127, 128, (n, k), dtype=torch.int8, device=device, generator=gen)

    def sc(n):
        return torch.rand((n,), device=device, generator=gen) * 0.009 + 0.001

    def gam():
        return 1 + 0.02 * torch.randn((D,), device=device, generator=gen)

    for l in range(layers):
        model.load_layer(l, wq=w8(Q, D), wk=w8(KV, D), wv=w8(KV, D), wo=w8(D, D), wg=w8(ffn, D), wu=w8(ffn, D), wd=w8(D, ffn),
                         sq=sc(Q), sk=sc(KV), sv=sc(KV), so=sc(D), sg=sc(ffn), su=sc(ffn), sd=sc(D), gamma0=gam(), gamma1=gam(),
                         a_s=torch.full((heads_q,), a_s, device=device))
    cos_t, sin_t = rope_table(max_ctx + 1)
    model.load_head(w8(vocab, D), sc(vocab), gam(), torch.from_numpy(cos_t).to(device), torch.from_numpy(sin_t).to(device))


def write_reference_format(directory, W, embed=False):
    """Writes the weights W (as made by numpy_weights) in the on-disk format of the reference's demo (its parameters/
    directory): <proj>_L%02d.bin int8 [out][in], C headers with the scale / row-sum / norm / A_s / RoPE arrays,
    lm_head_L00.bin, optionally model_embed_tokens_fp32.bin. Row sums are accumulated in fp32 in index order, as the
    reference's test bench does (Linear_Layer_Prefilling_tb.cpp:222-237)."""
    import os
    os.makedirs(directory, exist_ok=True)
    L = len(W["wq"])
    names = dict(q="q_proj", k="k_proj", v="v_proj", o="o_proj", g="gate_proj", u="up_proj", d="down_proj")

    def rowsum(w, s):
        acc = np.zeros(w.shape[0], np.float32)
        ws = w.astype(np.float32) * s[:, None].astype(np.float32)
        for j in range(w.shape[1]):
            acc = (acc + ws[:, j]).astype(np.float32)
        return acc

    def c_array(name, a):
        a = np.asarray(a, np.float32)
        dims = "".join(f"[{d}]" for d in a.shape)
        flat = a.reshape(-1)
        body = ",\n".join(", ".join(f"{float(v):.9e}f" for v in flat[i:i + 8]) for i in range(0, flat.size, 8))
        return f"static const float {name}{dims} = {{\n{body}\n}};\n"

    sums = {}
    for k, nm in names.items():
        for l in range(L):
            W["w" + k][l].astype(np.int8).tofile(os.path.join(directory, f"{nm}_L{l:02d}.bin"))
        sc = np.stack([W["s" + k][l] for l in range(L)])
        sm = np.stack([rowsum(W["w" + k][l], W["s" + k][l]) for l in range(L)])
        sums[k] = sm
        with open(os.path.join(directory, f"w_{nm}_s_sum.h"), "w") as f:
            f.write(f"// per-channel scales and row sums of {nm}\n" + c_array(f"w_{nm}_s", sc) + c_array(f"w_{nm}_sum", sm))
    norm = np.stack([W["g0"][l // 2] if l % 2 == 0 else W["g1"][l // 2] for l in range(2 * L)] + [W["g_final"]])
    open(os.path.join(directory, "w_rmsnorm.h"), "w").write(c_array("RMSNorm_weight", norm))
    open(os.path.join(directory, "A_s.h"), "w").write(c_array("A_s", np.stack(W["a_s"])))
    open(os.path.join(directory, "RoPE_sin_cos.h"), "w").write(c_array("PE_sin", W["sin_t"]) + "/* cosines */\n" + c_array("PE_cos", W["cos_t"]))
    W["lm_w"].astype(np.int8).tofile(os.path.join(directory, "lm_head_L00.bin"))
    open(os.path.join(directory, "w_lm_head_lm_head.h"), "w").write(
        c_array("w_lm_head_lm_head_s", W["lm_s"]) + c_array("w_lm_head_lm_head_sum", rowsum(W["lm_w"], W["lm_s"])))
    if embed:
        (W["lm_w"].astype(np.float32) * W["lm_s"][:, None]).astype(np.float32).tofile(os.path.join(directory, "model_embed_tokens_fp32.bin"))
    return sums
