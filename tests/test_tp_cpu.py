"""The tensor-parallel dataflow on CPU: two gloo ranks run one decoder layer with the partition the
GPU runner uses (column-parallel q/k/v and gate/up, all-gather of the fp32 activations, row-parallel
o/down with an int32 all-reduce, vocab-parallel argmax) on oracle primitives, and must reproduce the
single-process oracle bit for bit. This pins the claim that the partition changes no bits."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

CFGS = {2: dict(hidden=512, hq=8, hkv=2, ffn=8192, vocab=1024, T=12, seed=70),
        4: dict(hidden=1024, hq=16, hkv=4, ffn=8192, vocab=1024, T=6, seed=71)}
CFG = dict(CFGS[2])


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _layer_inputs():
    from flexllm_b200 import synthetic
    c = CFG
    W = synthetic.numpy_weights(1, c["hidden"], c["hq"], c["hkv"], c["ffn"], c["vocab"], c["T"] + 1, seed=c["seed"])
    x = np.random.default_rng(c["seed"] + 1).standard_normal((c["T"], c["hidden"])).astype(np.float32)
    return W, x


def _attention(oracle, W, qf, kf, vf, HQ, HKV, a_s, T):
    """Causal attention of one sequence on the given heads (positions 0..T-1)."""
    pos = np.arange(T, dtype=np.int32)
    prep = lambda f, H, rot: oracle.quant_per_token(
        (oracle.fht(oracle.rope(f.reshape(T, H, 64), pos, W["cos_t"], W["sin_t"]), 8.0) if rot else f.reshape(T, H, 64)).reshape(T * H, 64))
    q2, qs2 = prep(qf, HQ, True); k2, ks2 = prep(kf, HKV, True); v2, vs2 = prep(vf, HKV, False)
    q2 = q2.reshape(T, HQ, 64); k2 = k2.reshape(T, HKV, 64); v2 = v2.reshape(T, HKV, 64)
    qs2 = qs2.reshape(T, HQ); ks2 = ks2.reshape(T, HKV); vs2 = vs2.reshape(T, HKV)
    att = np.zeros((T, HQ * 64), np.float32)
    for t in range(T):
        for h in range(HQ):
            r = oracle.attn_row(q2[t, h], qs2[t, h], k2[:t + 1, h // 4], ks2[:t + 1, h // 4], v2[:t + 1, h // 4], vs2[:t + 1, h // 4], a_s[h])
            att[t, h * 64:(h + 1) * 64] = r["out"]
    return att


def _single(oracle):
    c = CFG; W, x = _layer_inputs(); T, D = c["T"], c["hidden"]
    xq, xs = oracle.quant_per_token(oracle.rmsnorm(x, W["g0"][0]))
    lin = lambda w, s: oracle.linear_i8(xq, xs, w, s)[1]
    att = _attention(oracle, W, lin(W["wq"][0], W["sq"][0]), lin(W["wk"][0], W["sk"][0]), lin(W["wv"][0], W["sv"][0]),
                     c["hq"], c["hkv"], W["a_s"][0], T)
    aq, as_ = oracle.quant_per_token(att)
    x1 = oracle.residual(x, oracle.linear_i8(aq, as_, W["wo"][0], W["so"][0])[1])
    out = oracle.mlp_block(x1, W["g1"][0], W["wg"][0], W["sg"][0], W["wu"][0], W["su"][0], W["wd"][0], W["sd"][0],
                           fht_scale=float(np.float32(np.sqrt(8192))))["out"]
    xq2, xs2 = oracle.quant_per_token(oracle.rmsnorm(out, W["g_final"]))
    logits = oracle.linear_i8(xq2, xs2, W["lm_w"], W["lm_s"])[1]
    return out, oracle.argmax(logits)


def _rank(rank, world, port, ret):
    CFG.clear(); CFG.update(CFGS[world])
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    oracle.set_exp_mode(oracle.EXP_CORRECTLY_ROUNDED)
    c = CFG; W, x = _layer_inputs(); T, D, F, V = c["T"], c["hidden"], c["ffn"], c["vocab"]
    g, r = world, rank
    HQl, HKVl, Dl, Fl, Vl = c["hq"] // g, c["hkv"] // g, D // g, F // g, V // g

    def gather(a):      # [g][T][W] rank-blocked, as an all-gather leaves it
        parts = [torch.empty_like(torch.from_numpy(a)) for _ in range(g)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(a)))
        return [p.numpy() for p in parts]

    def allreduce(acc):
        t = torch.from_numpy(np.ascontiguousarray(acc)); dist.all_reduce(t); return t.numpy()

    xq, xs = oracle.quant_per_token(oracle.rmsnorm(x, W["g0"][0]))
    rows = lambda w, n: w[r * n:(r + 1) * n]
    lin = lambda w, s, n: oracle.linear_i8(xq, xs, rows(w, n), rows(s, n))[1]
    att_l = _attention(oracle, W, lin(W["wq"][0], W["sq"][0], HQl * 64), lin(W["wk"][0], W["sk"][0], HKVl * 64),
                       lin(W["wv"][0], W["sv"][0], HKVl * 64), HQl, HKVl, W["a_s"][0][r * HQl:(r + 1) * HQl], T)
    att = np.concatenate(gather(att_l), axis=1)                     # logical rows again
    aq, as_ = oracle.quant_per_token(att)                            # scale from the whole row
    acc = oracle.gemm_s8s8(np.ascontiguousarray(aq[:, r * Dl:(r + 1) * Dl]), np.ascontiguousarray(W["wo"][0][:, r * Dl:(r + 1) * Dl]))
    x1 = oracle.residual(x, oracle.dequant(allreduce(acc), as_, W["so"][0]))
    xq1, xs1 = oracle.quant_per_token(oracle.rmsnorm(x1, W["g1"][0]))
    gt = oracle.linear_i8(xq1, xs1, rows(W["wg"][0], Fl), rows(W["sg"][0], Fl))[1]
    up = oracle.linear_i8(xq1, xs1, rows(W["wu"][0], Fl), rows(W["su"][0], Fl))[1]
    h = np.concatenate(gather(oracle.silu_mul(gt, up)), axis=1)
    hq, hs = oracle.quant_per_token(oracle.fht(h, float(np.float32(np.sqrt(8192)))))
    acc = oracle.gemm_s8s8(np.ascontiguousarray(hq[:, r * Fl:(r + 1) * Fl]), np.ascontiguousarray(W["wd"][0][:, r * Fl:(r + 1) * Fl]))
    out = oracle.residual(x1, oracle.dequant(allreduce(acc), hs, W["sd"][0]))
    # vocab-parallel greedy token
    xq2, xs2 = oracle.quant_per_token(oracle.rmsnorm(out, W["g_final"]))
    logits_l = oracle.linear_i8(xq2, xs2, rows(W["lm_w"], Vl), rows(W["lm_s"], Vl))[1]
    li = oracle.argmax(logits_l)
    pairs = np.stack([logits_l[np.arange(T), li], (li + r * Vl).astype(np.float32)], axis=1).astype(np.float32)
    allp = gather(pairs)
    best_v, best_i = allp[0][:, 0].copy(), allp[0][:, 1].copy()
    for p in allp[1:]:
        better = (p[:, 0] > best_v) | ((p[:, 0] == best_v) & (p[:, 1] < best_i))
        best_v[better] = p[better, 0]; best_i[better] = p[better, 1]
    ret[rank] = (out, best_i.astype(np.int32))
    dist.barrier(); dist.destroy_process_group()


def _rank_rows(rank, world, port, ret):
    """The token-row partition of the GPU runner's tensor-parallel prefill: each rank owns T / g rows of the residual
    stream; int8 rows are all-gathered for the column-parallel projections (q|k|v by heads, gate|up by FFN channels);
    the attention output is quantised per column slice with the all-reduced (max) row magnitude and its int8 columns
    go to the rows' owners (all-to-all), which run the o projection for their rows with the full weights; silu(gate) *
    up goes to the rows' owners in fp32 (all-to-all), which then run the 8192-point FHT, the quantiser and the down
    projection on whole rows."""
    CFG.clear(); CFG.update(CFGS_ROWS[world])
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    oracle.set_exp_mode(oracle.EXP_CORRECTLY_ROUNDED)
    c = CFG; W, x_all = _layer_inputs(); T, D, F = c["T"], c["hidden"], c["ffn"]
    g, r = world, rank
    HQl, HKVl, Fl, Tr = c["hq"] // g, c["hkv"] // g, F // g, T // g
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    rows = lambda w, n: w[r * n:(r + 1) * n]

    def allgather_rows(a):
        parts = [torch.empty_like(t(a)) for _ in range(g)]
        dist.all_gather(parts, t(a))
        return np.concatenate([p.numpy() for p in parts], axis=0)

    def allreduce_max(a):
        v = t(a); dist.all_reduce(v, op=dist.ReduceOp.MAX); return v.numpy()

    def alltoall(blocks):                   # blocks[p] goes to rank p; returns the list received (index = source)
        every = [None] * g                  # gloo has no all_to_all: gather everything, pick what is addressed to this rank
        dist.all_gather_object(every, [np.ascontiguousarray(b) for b in blocks])
        return [every[s][r] for s in range(g)]

    def quant_with(amax, v):                # the per-token quantiser given the row's largest magnitude (quant.h:84-109)
        s = (amax / np.float32(127.0)).astype(np.float32); s[s == 0] = 1
        return _round_half_away(v / s[:, None]).astype(np.int8), s

    own = slice(r * Tr, (r + 1) * Tr)
    x = x_all[own]                          # this rank's rows
    xq_l, xs_l = oracle.quant_per_token(oracle.rmsnorm(x, W["g0"][0]))
    xq, xs = allgather_rows(xq_l), allgather_rows(xs_l)
    lin = lambda w, s, n: oracle.linear_i8(xq, xs, rows(w, n), rows(s, n))[1]
    att_l = _attention(oracle, W, lin(W["wq"][0], W["sq"][0], HQl * 64), lin(W["wk"][0], W["sk"][0], HKVl * 64),
                       lin(W["wv"][0], W["sv"][0], HKVl * 64), HQl, HKVl, W["a_s"][0][r * HQl:(r + 1) * HQl], T)
    amax = allreduce_max(np.abs(att_l).max(axis=1).astype(np.float32))
    aq_l, as_ = quant_with(amax, att_l)                                          # this rank's columns of ALL rows
    aq = np.concatenate(alltoall([aq_l[p * Tr:(p + 1) * Tr] for p in range(g)]), axis=1)     # all columns of this rank's rows
    x1 = oracle.residual(x, oracle.linear_i8(aq, as_[own], W["wo"][0], W["so"][0])[1])
    xq_l, xs_l = oracle.quant_per_token(oracle.rmsnorm(x1, W["g1"][0]))
    xq, xs = allgather_rows(xq_l), allgather_rows(xs_l)
    gt = oracle.linear_i8(xq, xs, rows(W["wg"][0], Fl), rows(W["sg"][0], Fl))[1]
    up = oracle.linear_i8(xq, xs, rows(W["wu"][0], Fl), rows(W["su"][0], Fl))[1]
    h_l = oracle.silu_mul(gt, up)                                                # this rank's FFN channels of ALL rows
    h = np.concatenate(alltoall([h_l[p * Tr:(p + 1) * Tr] for p in range(g)]), axis=1)       # whole rows of this rank
    hq, hs = oracle.quant_per_token(oracle.fht(h, float(np.float32(np.sqrt(8192)))))
    out_l = oracle.residual(x1, oracle.linear_i8(hq, hs, W["wd"][0], W["sd"][0])[1])
    ret[rank] = (allgather_rows(out_l), None)
    dist.barrier(); dist.destroy_process_group()


def _round_half_away(x):
    """std::round on fp32 values (half away from zero)."""
    x = np.asarray(x, np.float32)
    return np.where(x >= 0, np.floor(x + np.float32(0.5)), np.ceil(x - np.float32(0.5))).astype(np.float32)


CFGS_ROWS = {2: dict(hidden=512, hq=8, hkv=2, ffn=8192, vocab=1024, T=12, seed=72),
             4: dict(hidden=1024, hq=16, hkv=4, ffn=8192, vocab=1024, T=8, seed=73)}

import pytest


@pytest.mark.parametrize("world", [2, 4])
def test_token_row_partition_is_bit_exact_on_cpu(world):
    import oracle
    CFG.clear(); CFG.update(CFGS_ROWS[world])
    with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
        want_out, _ = _single(oracle)
    mgr = mp.Manager(); ret = mgr.dict()
    mp.spawn(_rank_rows, args=(world, _free_port(), ret), nprocs=world, join=True)
    for rank in range(world):
        assert np.array_equal(ret[rank][0].view(np.uint32), want_out.view(np.uint32)), f"rank {rank}: residual stream differs"


@pytest.mark.parametrize("world", [2, 4])
def test_tp_partition_is_bit_exact_on_cpu(world):
    import oracle
    CFG.clear(); CFG.update(CFGS[world])
    with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
        want_out, want_tok = _single(oracle)
    mgr = mp.Manager(); ret = mgr.dict()
    mp.spawn(_rank, args=(world, _free_port(), ret), nprocs=world, join=True)
    for rank in range(world):
        out, tok = ret[rank]
        assert np.array_equal(out.view(np.uint32), want_out.view(np.uint32)), f"rank {rank}: residual stream differs"
        assert np.array_equal(tok, want_tok), f"rank {rank}: greedy tokens differ"
