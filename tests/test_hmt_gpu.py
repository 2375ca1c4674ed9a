"""HMT long-context plug-in (Modules/HMT.h): the GPU driver against the oracle's restatement of the segment recurrence,
segment by segment (summary S_n, prompt vector P_n, memory M_n and its key K_n), then the residual stream of the last
segment and the tokens decoded after it. The oracle's two fp32 primitives (four-chain linear unit, four-lane softmax) are
pinned against the reference templates in tests/test_oracle_vs_reference.py. Small sizes in place of the reference's
990 / 495 / 32 / 64 so that the CPU side finishes in seconds; the ring wrap-around (more segments than memory slots) is
covered too."""
import numpy as np
import pytest
import torch

import oracle
from util import to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _correctly_rounded_exp():
    with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
        yield


@pytest.mark.parametrize("T,seg,summ,rec,mem", [(130, 40, 20, 8, 64), (75, 24, 24, 4, 16), (150, 8, 4, 2, 16)])
def test_hmt_segment_recurrence(T, seg, summ, rec, mem):
    import flexllm_b200 as F
    from flexllm_b200 import synthetic
    layers, hidden, hq, hkv, vocab, n_new, seed = 2, 512, 8, 2, 1000, 4, 95
    max_rows = (1 + rec + seg + 1 + 15) // 16 * 16
    W = synthetic.numpy_weights(layers, hidden, hq, hkv, 8192, vocab, max_rows + n_new, seed=seed)
    for l in range(layers):                     # moderate attention logits, so that the summaries depend on all tokens
        W["sq"][l] = (W["sq"][l] / 8).astype(np.float32); W["sk"][l] = (W["sk"][l] / 8).astype(np.float32)
    g = np.random.default_rng(seed + 1)
    tokens = g.integers(0, vocab, T).astype(np.int32)
    wq = (g.standard_normal((hidden, hidden)) / np.sqrt(hidden)).astype(np.float32)
    wk = (g.standard_normal((hidden, hidden)) / np.sqrt(hidden)).astype(np.float32)
    t_embed = g.standard_normal(hidden).astype(np.float32)
    m = F.Model(layers, hidden, hq, hkv, 8192, vocab, max_batch=1, max_prefill=max_rows, max_ctx=max_rows + n_new)
    synthetic.load_numpy_weights(m, W)
    emb = m.embed_tokens(torch.from_numpy(tokens).cuda(), hidden)
    emb_np = (W["lm_w"][tokens].astype(np.float32) * W["lm_s"][tokens][:, None]).astype(np.float32)
    assert np.array_equal(to_np(emb), emb_np)
    h = F.HMT(m, hidden, torch.from_numpy(wq), torch.from_numpy(wk), torch.from_numpy(t_embed), seg_len=seg, sum_len=summ, rec_len=rec, mem_num=mem)
    nxt, trace = h.prefill(emb, want_trace=True)
    m.begin(n_new); m.decode(n_new - 1, use_graph=False)
    torch.cuda.synchronize()
    assert F.lib().flexllm_device_status() == 0
    out = to_np(m.buffer(2, (1, n_new), torch.int32))[0]
    ref = oracle.hmt_prefill(W, emb_np, t_embed, wq, wk, seg, summ, rec, mem, n_new=n_new)
    trace = to_np(trace)
    nseg = (T + seg - 1) // seg
    same = lambda a, b: np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))
    for s in range(1, nseg):
        assert same(trace[s, 0], ref["S"][s - 1]), f"segment {s}: summary"
        assert same(trace[s, 1], ref["P"][s - 1]), f"segment {s}: prompt vector"
    for s in range(nseg - 1):
        assert same(trace[s, 2], ref["M"][s]), f"segment {s}: memory"
        assert same(trace[s, 3], ref["K"][s]), f"segment {s}: memory key"
    assert int(nxt.item()) == int(ref["tokens"][0])
    assert np.array_equal(out, ref["tokens"])
    # the memory does something: the prompt vector of the last segment is not zero and differs between segments
    assert np.abs(ref["P"][-1]).max() > 0 and (nseg < 3 or not same(ref["P"][-1], ref["P"][-2]))
    h.close(); m.close()


def test_hmt_needs_a_model_sized_for_one_stage():
    import flexllm_b200 as F
    from flexllm_b200 import _lib, synthetic
    from flexllm_b200.ops import FlexLLMError
    m = F.Model(1, 512, 8, 2, 8192, 1000, max_batch=1, max_prefill=32, max_ctx=64)
    z = torch.zeros((512, 512)); t = torch.zeros(512)
    with pytest.raises(FlexLLMError) as e:
        F.HMT(m, 512, z, z, t, seg_len=40, sum_len=20, rec_len=8, mem_num=64)
    assert e.value.status == _lib.ENOTSUP
    m.close()
