"""Reader of the reference's on-disk model format (its demo's parameters/ directory:
SpinQuant_Llama_32_1B_Ins/SpinQuant_Prefilling_Decoding_mem_opt_demo.cpp:21-74, :437-490). The parameter files themselves
are not part of the reference repository, so the test writes a small model in that format (int8 .bin rows, C headers
with the scale / row-sum / norm / RoPE arrays) and reads it back through the C ABI. Host code only: runs without a GPU."""
import numpy as np
import pytest
import torch


def _weights(four_bit):
    from flexllm_b200 import synthetic
    W = synthetic.numpy_weights(2, 256, 4, 1, 512, 300, 40, seed=80)
    if four_bit:        # the shipped model's range
        g = np.random.default_rng(81)
        for k in "qkvogud":
            W["w" + k] = [g.integers(-8, 8, w.shape, dtype=np.int8) for w in W["w" + k]]
    return W


@pytest.mark.parametrize("four_bit", [False, True])
def test_read_back_reference_format(tmp_path, four_bit):
    import flexllm_b200 as F
    from flexllm_b200 import synthetic
    W = _weights(four_bit)
    sums = synthetic.write_reference_format(tmp_path, W, embed=True)
    for l in range(2):
        got = F.read_reference_layer(tmp_path, l, hidden=256, kv_hidden=64, ffn=512, heads_q=4)
        for k in "qkvogud":
            assert np.array_equal(got["w" + k].numpy(), W["w" + k][l])
            assert np.array_equal(got["s" + k].numpy().view(np.uint32), W["s" + k][l].view(np.uint32))      # %.9e round-trips fp32
            assert np.array_equal(got["sum" + k].numpy().view(np.uint32), sums[k][l].view(np.uint32))
        assert np.array_equal(got["gamma0"].numpy(), W["g0"][l]) and np.array_equal(got["gamma1"].numpy(), W["g1"][l])
        assert np.array_equal(got["a_s"].numpy(), W["a_s"][l])
    head = F.read_reference_head(tmp_path, layers=2, hidden=256, vocab=300, table_len=41, want_embed=True)
    assert np.array_equal(head["lm_w"].numpy(), W["lm_w"]) and np.array_equal(head["lm_s"].numpy(), W["lm_s"])
    assert np.array_equal(head["gamma_final"].numpy(), W["g_final"])
    assert np.array_equal(head["cos_t"].numpy(), W["cos_t"]) and np.array_equal(head["sin_t"].numpy(), W["sin_t"])
    assert np.array_equal(head["embed"].numpy(), (W["lm_w"].astype(np.float32) * W["lm_s"][:, None]).astype(np.float32))


def test_missing_and_short_files_are_reported(tmp_path):
    import flexllm_b200 as F
    from flexllm_b200 import _lib, synthetic
    from flexllm_b200.ops import FlexLLMError
    with pytest.raises(FlexLLMError) as e:
        F.read_reference_layer(tmp_path, 0, hidden=256, kv_hidden=64, ffn=512, heads_q=4)
    assert e.value.status == _lib.EIO
    synthetic.write_reference_format(tmp_path, _weights(False))
    with pytest.raises(FlexLLMError) as e:                     # layer 2 does not exist
        F.read_reference_layer(tmp_path, 2, hidden=256, kv_hidden=64, ffn=512, heads_q=4)
    assert e.value.status == _lib.EIO
    with pytest.raises(FlexLLMError) as e:                     # rows are longer than the file
        F.read_reference_layer(tmp_path, 0, hidden=512, kv_hidden=64, ffn=512, heads_q=4)
    assert e.value.status == _lib.EIO
    buf = torch.empty(4)
    rc = F.lib().flexllm_ckpt_read_c_array_f32(str(tmp_path / "A_s.h").encode(), b"no_such_array", 0, 4, buf.data_ptr())
    assert rc == _lib.EINVAL


@pytest.mark.gpu
def test_model_from_checkpoint_directory(tmp_path):
    """A model loaded layer by layer from a directory in the reference's format generates the oracle's tokens."""
    import flexllm_b200 as F
    import oracle
    from flexllm_b200 import synthetic
    layers, hidden, hq, hkv, vocab, B, S, n_new = 2, 512, 8, 2, 1000, 2, 32, 4
    W = synthetic.numpy_weights(layers, hidden, hq, hkv, 8192, vocab, S + n_new, seed=82)
    g = np.random.default_rng(83)
    for k in "qkvogud":                                        # 4-bit weights, as the shipped model has
        W["w" + k] = [g.integers(-8, 8, w.shape, dtype=np.int8) for w in W["w" + k]]
    synthetic.write_reference_format(tmp_path, W)
    m = F.Model(layers, hidden, hq, hkv, 8192, vocab, max_batch=B, max_prefill=S, max_ctx=S + n_new)
    for l in range(layers):
        d = F.read_reference_layer(tmp_path, l, hidden=hidden, kv_hidden=hkv * 64, ffn=8192, heads_q=hq)
        m.load_layer(l, **{k: v for k, v in d.items() if not k.startswith("sum")})
    h = F.read_reference_head(tmp_path, layers, hidden, vocab, S + n_new + 1)
    m.load_head(h["lm_w"], h["lm_s"], h["gamma_final"], h["cos_t"], h["sin_t"])
    tokens = np.random.default_rng(84).integers(0, vocab, (B, S)).astype(np.int32)
    out = m.generate_host(torch.from_numpy(tokens), n_new, use_graph=False)
    with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
        ref = oracle.model_generate(W, tokens, n_new)
    assert np.array_equal(out.numpy(), ref["tokens"])
    m.close()
