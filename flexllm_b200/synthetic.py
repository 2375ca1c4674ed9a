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
