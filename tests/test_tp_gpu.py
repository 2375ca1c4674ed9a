"""Tensor-parallel model on 2 GPUs (one process per GPU, NCCL): identical greedy tokens and a
bit-identical residual stream / logits against the CPU oracle's single-device forward. Skipped on
boxes with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, cfg, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
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
    if rank == 0:
        ret["tokens"] = out.numpy().copy(); ret["hidden"] = hidden_gpu
    else:
        ret["tokens1"] = out.numpy().copy()
    m.close(); tp.close()
    dist.barrier(); dist.destroy_process_group()


@pytest.mark.parametrize("world,cfg", [(2, (2, 512, 8, 2, 1008, 2, 32, 4, 60)), (2, (2, 1024, 16, 4, 2000, 12, 48, 4, 61)),
                                       (4, (2, 1024, 16, 4, 2016, 5, 32, 4, 62))])
def test_tp_matches_oracle(world, cfg):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    import oracle
    from flexllm_b200 import synthetic
    layers, hidden, hq, hkv, vocab, B, S, n_new, seed = cfg
    mgr = mp.Manager(); ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), cfg, ret), nprocs=world, join=True)
    W = synthetic.numpy_weights(layers, hidden, hq, hkv, 8192, vocab, S + n_new, seed=seed)
    tokens = np.random.default_rng(seed + 1).integers(0, vocab, (B, S)).astype(np.int32)
    with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
        ref = oracle.model_generate(W, tokens, n_new, want_hidden=True)
    assert np.array_equal(ret["tokens"], ref["tokens"]) and np.array_equal(ret["tokens1"], ref["tokens"])
    assert np.array_equal(ret["hidden"].view(np.uint32), ref["hidden"].view(np.uint32))
