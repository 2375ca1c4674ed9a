"""The benchmark configurations at their full sizes, each against the CPU oracle (or, where the oracle
would take too long, against a second, independently coded GPU path of this library):

  decode MLP block at batch 1 and batch 64  (RMSNorm -> quant -> gate/up -> SiLU*up -> FHT-8192 -> quant ->
      down -> + residual; reference operator order SpinQuant_Decoding_mem_opt.h:1050-1126), bit for bit;
  decode attention at batch 64, context lengths drawn uniformly from [512, 8192], seeded random page table;
  the whole 16-layer model at batch 32, prompt 1024: persistent decode kernel against the kernel-per-operator
      decode path (the two share no host code beyond the weights), tokens and residual stream identical.
"""
import numpy as np
import pytest
import torch

import oracle
from util import assert_same, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _correctly_rounded_exp():
    with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
        yield


@pytest.fixture(scope="module")
def F():
    import flexllm_b200
    flexllm_b200.lib()
    return flexllm_b200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("B", [1, 64])
def test_decode_mlp_block(F, B):
    """h fp32 [B,2048] ~ N(0,1), gamma ~ N(1,0.02), int8 weights U[-127,127], per-channel scales U[0.001,0.01]."""
    D, Fdim = 2048, 8192
    g = np.random.default_rng(200 + B)
    h = g.standard_normal((B, D)).astype(np.float32)
    gamma = (1 + 0.02 * g.standard_normal(D)).astype(np.float32)
    wg, wu = g.integers(-127, 128, (Fdim, D), dtype=np.int8), g.integers(-127, 128, (Fdim, D), dtype=np.int8)
    wd = g.integers(-127, 128, (D, Fdim), dtype=np.int8)
    sg, su, sd = (g.uniform(0.001, 0.01, n).astype(np.float32) for n in (Fdim, Fdim, D))
    ref = oracle.mlp_block(h, gamma, wg, sg, wu, su, wd, sd, lanes=8)
    hd = dev(h)
    _, xq, xs = F.dec_Layer_Norm(hd, dev(gamma), lanes=8, quant=True, want_y=False)
    assert_same(to_np(xq), ref["xq"], "RMSNorm + quant"); assert_same(to_np(xs), ref["xs"], "token scales")
    _, gt = F.dec_Linear_Layer_i8xi8(xq, xs, dev(wg), dev(sg))
    _, up = F.dec_Linear_Layer_i8xi8(xq, xs, dev(wu), dev(su))
    hq, hs, act = F.swiglu_fht_quant(gt, up, want_act=True)
    assert_same(to_np(act), ref["act"], "silu(gate) * up")
    assert_same(to_np(hq), ref["hq"], "FHT-8192 + quant"); assert_same(to_np(hs), ref["hs"], "FHT row scales")
    acc, _ = F.dec_Linear_Layer_i8xi8(hq, hs, dev(wd), dev(sd), want_acc=True, want_y=False)
    assert_same(to_np(acc), ref["down_acc"], "down projection int32 sums")
    _, out = F.dec_Linear_Layer_i8xi8(hq, hs, dev(wd), dev(sd), residual=hd)
    assert_same(to_np(out), ref["out"], "block output")
    # the same block as ONE call (fused gate|up weights, dependent launches), twice in a row and in place the second time
    w_gu = dev(np.concatenate([wg, wu])); s_gu = dev(np.concatenate([sg, su]))
    y = F.dec_MLP_block(hd, dev(gamma), w_gu, s_gu, dev(wd), dev(sd), order=8)
    assert_same(to_np(y), ref["out"], "block output, one call")
    x2 = hd.clone()
    F.dec_MLP_block(x2, dev(gamma), w_gu, s_gu, dev(wd), dev(sd), order=8, out=x2)
    assert_same(to_np(x2), ref["out"], "block output, one call, in place")
    assert F.lib().flexllm_device_status() == 0


def test_decode_attention_batch64(F):
    """64 sequences, contexts ~ U{512..8192}: one decode step of one layer against the oracle."""
    from test_attention_gpu import decode_case
    g = np.random.default_rng(4)
    decode_case(F, 64, g.integers(512, 8193, 64), seed=44)


# which attention variant of the persistent kernel the decode steps of a case take (it is chosen per launch from the
# number of (sequence, KV head) items against the number of SMs and from the longest context against the staging areas)
@pytest.mark.parametrize("layers,B,S,n_new,what", [
    (16, 32, 1024, 8, "the full-model workload: two items per CTA, staged copies"),
    (2, 20, 1296, 3, "two items per CTA, contexts beyond half of the operand ring (per-thread loads)"),
    (2, 16, 1040, 3, "one item per CTA on all 512 threads, staged copies"),
    (2, 4, 2112, 3, "one item per CTA, contexts beyond the operand ring (per-thread loads)"),
])
def test_full_model_two_decode_paths(F, monkeypatch, layers, B, S, n_new, what):
    """Hidden 2048, 32/8 heads, FFN 8192, vocab 128256 -- 16 layers at batch 32, prompt 1024, 8 generated tokens, and
    2-layer stacks at the batch sizes and context lengths that select the persistent kernel's other attention
    variants: the persistent decode-step kernel and the kernel-per-operator decode path (FLEXLLM_MEGA=0) produce the
    same tokens, the same residual stream of the last step and the same logits."""
    from flexllm_b200 import synthetic
    cfg = dict(synthetic.LLAMA32_1B)
    cfg["layers"] = layers
    tok = torch.randint(0, cfg["vocab"], (B, S), dtype=torch.int32, generator=torch.Generator().manual_seed(77))
    res = {}
    for mega in ("1", "0"):
        monkeypatch.setenv("FLEXLLM_MEGA", mega)
        m = F.Model(max_batch=B, max_prefill=S, max_ctx=S + n_new, **cfg)
        synthetic.load_random_weights(m, max_ctx=S + n_new, seed=5, **cfg)
        out = m.generate_host(tok, n_new, use_graph=True)
        assert F.lib().flexllm_device_status() == 0
        res[mega] = (out.numpy().copy(), to_np(m.buffer(0, (B, cfg["hidden"]), torch.float32)),
                     to_np(m.buffer(1, (B, cfg["vocab"]), torch.float32)))
        m.close()
        del m
        torch.cuda.empty_cache()
    assert np.array_equal(res["1"][0], res["0"][0]), f"tokens differ between the two decode paths ({what})"
    assert_same(res["1"][1], res["0"][1], "residual stream of the last decode step")
    assert_same(res["1"][2], res["0"][2], "logits of the last decode step")
    # not a degenerate run: the sequences do not all emit one token
    assert len(np.unique(res["1"][0])) > min(B, 8)
