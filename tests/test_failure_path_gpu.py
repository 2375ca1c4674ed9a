"""Failure paths that can be exercised without faulting, trapping or hanging the GPU.

A bounded device-side wait that runs out: the persistent decode-step kernel is told (test hook) to wait at
its first grid barrier for one arrival more than the grid delivers, with the wait limit cut to a few
milliseconds. Every CTA then gives up, leaves through the tear-down and the host reads FLEXLLM_ETIMEDOUT
from flexllm_device_status(); the context stays usable and the next generation is correct.
Requests the host can refuse before launching anything: decode steps past max_ctx, token ids outside the
vocabulary.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    import flexllm_b200
    flexllm_b200.lib()
    return flexllm_b200


def _small_model(F, B=4, S=32, n_new=6, seed=90):
    from flexllm_b200 import synthetic
    dims = dict(layers=2, hidden=512, heads_q=8, heads_kv=2, ffn=8192, vocab=1000)
    W = synthetic.numpy_weights(max_ctx=S + n_new, seed=seed, **dims)
    m = F.Model(max_batch=B, max_prefill=S, max_ctx=S + n_new, **dims)
    synthetic.load_numpy_weights(m, W)
    tokens = np.random.default_rng(seed + 1).integers(0, dims["vocab"], (B, S)).astype(np.int32)
    return m, W, tokens


def test_bounded_wait_runs_out_and_context_survives(F):
    from flexllm_b200 import _lib
    lib = F.lib()
    n_new = 6
    m, W, tokens = _small_model(F, n_new=n_new)
    with oracle.exp_mode(oracle.EXP_CORRECTLY_ROUNDED):
        want = oracle.model_generate(W, tokens, n_new)["tokens"]
    assert lib.flexllm_device_status() == 0
    try:
        assert lib.flexllm_debug_hook(0, 5_000_000) == 0        # 5 ms instead of 2 s
        m.prefill(torch.from_numpy(tokens).cuda()); m.begin(n_new)
        assert lib.flexllm_debug_hook(1, 1) == 0                # next step: first grid barrier can never complete
        m.decode(1, use_graph=False)
        torch.cuda.synchronize()                                # the kernel RETURNED: nothing hangs, nothing faults
        assert lib.flexllm_device_status() == _lib.ETIMEDOUT
        assert lib.flexllm_device_status() == 0                 # reading the status clears it
    finally:
        lib.flexllm_debug_hook(0, 0)
    # the same model object, a fresh generation: correct tokens
    out = m.generate_host(torch.from_numpy(tokens), n_new, use_graph=False)
    assert np.array_equal(out.numpy(), want)
    m.close()


def test_decode_past_max_ctx_is_refused_before_launch(F):
    from flexllm_b200.ops import FlexLLMError
    from flexllm_b200 import _lib
    lib = F.lib()
    n_new = 4
    m, W, tokens = _small_model(F, n_new=n_new, seed=91)      # max_ctx = S + 4
    m.prefill(torch.from_numpy(tokens).cuda()); m.begin(n_new)
    before = lib.flexllm_launch_count()
    with pytest.raises(FlexLLMError) as e:
        m.decode(n_new + 2, use_graph=False)                   # last step would append at position S + 5 > max_ctx
    assert e.value.status == _lib.EINVAL
    assert lib.flexllm_launch_count() == before                # nothing was launched
    m.decode(n_new - 1, use_graph=False)                       # the legal request still runs
    torch.cuda.synchronize()
    assert lib.flexllm_device_status() == 0
    m.close()


def test_token_ids_outside_the_vocabulary_are_refused(F):
    from flexllm_b200.ops import FlexLLMError
    from flexllm_b200 import _lib
    m, W, tokens = _small_model(F, seed=92)
    for bad in (-1, 1000):
        t = tokens.copy(); t[1, 3] = bad
        with pytest.raises(FlexLLMError) as e:
            m.generate_host(torch.from_numpy(t), 2, use_graph=False)
        assert e.value.status == _lib.EINVAL
    m.close()


def test_device_resident_bad_ids_and_lengths_are_clamped_and_reported(F):
    """Ids and context lengths that live in device memory cannot be vetted by the host: the kernels clamp them
    (no wild read) and raise the error word."""
    from flexllm_b200 import _lib
    lib = F.lib()
    m, W, tokens = _small_model(F, seed=93)
    t = tokens.copy(); t[0, 0] = 5000                          # device-resident prompt: goes straight to the kernel
    m.prefill(torch.from_numpy(t).cuda())
    torch.cuda.synchronize()
    assert lib.flexllm_device_status() == _lib.EDEVDATA
    assert lib.flexllm_device_status() == 0
    m.close()
