"""Tensor-parallel model on 2, 4 and 8 GPUs (one process per GPU, NCCL): identical greedy tokens on every rank and a
bit-identical residual stream against the CPU oracle's single-device forward. Both partitions are covered: the
token-row partition with batch-parallel decode (batch divisible by the number of ranks; the 8-rank case leaves one KV
head per rank) and the all-gather partition (any batch, or FLEXLLM_TP_MODE=allgather). Cases that need more GPUs than
the box has are skipped."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, cfg, mode, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    if mode:
        os.environ["FLEXLLM_TP_MODE"] = mode
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)      # only to hand the NCCL id around
    import flexllm_b200 as F
    from flexllm_b200 import synthetic
    ids = [F.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    tp = F.TensorParallel(rank, world, ids[0])
    layers, hidden, hq, hkv, vocab, B, S, n_new, seed = cfg
    W = synthetic.numpy_weights(layers, hidden, hq, hkv, 8192, vocab, S + n_new, seed=seed)
    tokens = np.random.default_rng(seed + 1).integers(0, vocab, (B, S)).astype(np.int32)
    m = F.Model(layers, hidden, hq, hkv, 8192, vocab, max_batch=B, max_prefill=S, max_ctx=S + n_new, tp=tp)
    synthetic.load_numpy_weights(m, W)
    out = m.generate_host(torch.from_numpy(tokens), n_new, use_graph=True)
    m.prefill(torch.from_numpy(tokens).cuda()); torch.cuda.synchronize()
    hidden_gpu = m.buffer(0, (B * S, hidden), torch.float32).cpu().numpy()
    ret[f"tokens{rank}"] = out.numpy().copy()
    ret[f"status{rank}"] = F.lib().flexllm_device_status()
    if rank == 0:
        ret["hidden"] = hidden_gpu
    m.close(); tp.close()
    dist.barrier(); dist.destroy_process_group()


# cfg = (layers, hidden, heads_q, heads_kv, vocab, batch, prompt, generated, seed)
@pytest.mark.parametrize("world,cfg,mode", [
    (2, (2, 512, 8, 2, 1008, 2, 32, 4, 60), None),              # token rows, one sequence per rank
    (2, (2, 1024, 16, 4, 2000, 12, 48, 4, 61), None),           # token rows, six sequences per rank
    (2, (2, 1024, 16, 4, 2000, 12, 48, 4, 61), "allgather"),    # the same model on the all-gather partition
    (4, (2, 1024, 16, 4, 2016, 5, 32, 4, 62), None),            # batch 5 on 4 ranks: falls back to the all-gather partition
    (4, (2, 1024, 16, 4, 2016, 8, 32, 4, 64), None),            # token rows on 4 ranks
    (8, (1, 2048, 32, 8, 2048, 8, 32, 3, 63), None),            # 8 ranks: one KV head, four query heads, 1024 FFN channels each
])
def test_tp_matches_oracle(world, cfg, mode):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    import oracle
    from flexllm_b200 import synthetic
    layers, hidden, hq, hkv, vocab, B, S, n_new, seed = cfg
    mgr = mp.Manager(); ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), cfg, mode, ret), nprocs=world, join=True)
    W = synthetic.numpy_weights(layers, hidden, hq, hkv, 8192, vocab, S + n_new, seed=seed)
    tokens = np.random.default_rng(seed + 1).integers(0, vocab, (B, S)).astype(np.int32)
    with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
        ref = oracle.model_generate(W, tokens, n_new, want_hidden=True)
    for rank in range(world):
        assert ret[f"status{rank}"] == 0
        assert np.array_equal(ret[f"tokens{rank}"], ref["tokens"]), f"rank {rank}: tokens differ"
    assert np.array_equal(ret["hidden"].view(np.uint32), ref["hidden"].view(np.uint32))


def _shared_device_rank(tp, cfg, W, tokens, ret):
    import flexllm_b200 as F
    from flexllm_b200 import synthetic
    layers, hidden, hq, hkv, vocab, B, S, n_new, seed = cfg
    try:
        torch.cuda.set_device(0)
        m = F.Model(layers, hidden, hq, hkv, 8192, vocab, max_batch=B, max_prefill=S, max_ctx=S + n_new, tp=tp)
        synthetic.load_numpy_weights(m, W)
        ret[f"tokens{tp.rank}"] = m.generate_host(torch.from_numpy(tokens), n_new, use_graph=True).numpy().copy()
        m.prefill(torch.from_numpy(tokens).cuda())
        hidden_gpu = m.buffer(0, (B * S, hidden), torch.float32).cpu().numpy()      # a collective on the token-row partition
        if tp.rank == 0:
            ret["hidden"] = hidden_gpu
        m.close()
    except Exception as e:       # reported by the parent; the other ranks' rendezvous give up by themselves
        ret[f"error{tp.rank}"] = repr(e)


@pytest.mark.parametrize("world,cfg,mode", [
    (2, (2, 1024, 16, 4, 2000, 12, 48, 4, 61), None),
    (4, (2, 1024, 16, 4, 2016, 8, 32, 4, 64), None),
    (8, (1, 2048, 32, 8, 2048, 8, 32, 3, 63), None),            # one KV head, four query heads, 1024 FFN channels, one sequence per rank
    (8, (2, 2048, 32, 8, 2048, 16, 64, 3, 65), None),           # two sequences per rank, two layers
    (8, (1, 2048, 32, 8, 2048, 8, 32, 3, 63), "allgather"),
])
def test_tp_ranks_sharing_one_gpu_match_oracle(world, cfg, mode, monkeypatch):
    """The same partitioned dataflow with all ranks on ONE GPU (a host thread per rank, collectives as device copies in
    one stream): every rank count up to 8 is checked on any box."""
    import threading
    import oracle
    import flexllm_b200 as F
    from flexllm_b200 import synthetic
    if mode:
        monkeypatch.setenv("FLEXLLM_TP_MODE", mode)
    else:
        monkeypatch.delenv("FLEXLLM_TP_MODE", raising=False)
    layers, hidden, hq, hkv, vocab, B, S, n_new, seed = cfg
    W = synthetic.numpy_weights(layers, hidden, hq, hkv, 8192, vocab, S + n_new, seed=seed)
    tokens = np.random.default_rng(seed + 1).integers(0, vocab, (B, S)).astype(np.int32)
    group = F.TensorParallel.local_group(world)
    ret = {}
    threads = [threading.Thread(target=_shared_device_rank, args=(tp, cfg, W, tokens, ret)) for tp in group]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for tp in group:
        tp.close()
    assert not [k for k in ret if k.startswith("error")], {k: v for k, v in ret.items() if k.startswith("error")}
    assert F.lib().flexllm_device_status() == 0
    with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
        ref = oracle.model_generate(W, tokens, n_new, want_hidden=True)
    for rank in range(world):
        assert np.array_equal(ret[f"tokens{rank}"], ref["tokens"]), f"rank {rank}: tokens differ"
    assert np.array_equal(ret["hidden"].view(np.uint32), ref["hidden"].view(np.uint32))


@pytest.mark.parametrize("world", [2, 8])
def test_collectives_of_ranks_sharing_one_gpu(world):
    """Every collective of the device-sharing group against numpy: all-reduce (sum, max), reduce-scatter, all-gather,
    all-to-all, several in a row on one stream (the second rendezvous keeps a rank's next collective from overwriting
    buffers its peers still have to read)."""
    import threading
    import flexllm_b200 as F
    group = F.TensorParallel.local_group(world)
    rng = np.random.default_rng(90)
    n = 3000
    a = rng.integers(-1000, 1000, (world, world, n)).astype(np.int32)         # [rank][block][n]
    f = rng.standard_normal((world, n)).astype(np.float32)
    ret = {}

    def run(tp):
        try:
            torch.cuda.set_device(0)
            r = tp.rank
            mine = torch.from_numpy(a[r]).cuda()
            ret[("rs", r)] = tp.reduce_scatter_s32(mine).cpu().numpy()
            ret[("ar", r)] = tp.allreduce_s32(mine.clone()).cpu().numpy()
            ret[("mx", r)] = tp.allreduce_max_f32(torch.from_numpy(f[r]).cuda()).cpu().numpy()
            ret[("ag", r)] = tp.allgather(mine[0].contiguous()).cpu().numpy()
            ret[("aa", r)] = tp.alltoall(mine).cpu().numpy()
        except Exception as e:
            ret[("error", tp.rank)] = repr(e)

    threads = [threading.Thread(target=run, args=(tp,)) for tp in group]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for tp in group:
        tp.close()
    assert not [k for k in ret if k[0] == "error"], {k: v for k, v in ret.items() if k[0] == "error"}
    total = a.sum(axis=0)
    for r in range(world):
        assert np.array_equal(ret[("rs", r)], total[r])
        assert np.array_equal(ret[("ar", r)], total)
        assert np.array_equal(ret[("mx", r)], f.max(axis=0))
        assert np.array_equal(ret[("ag", r)], a[:, 0])
        assert np.array_equal(ret[("aa", r)], a[:, r])
