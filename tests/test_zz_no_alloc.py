"""The allocation-free decode linear layer (flexllm_linear_decode_i8_noalloc).

Some hosts cannot call cudaMalloc around a decode step (the device memory belongs to their own pool, or
an allocation would stall the other streams). For them the library offers one entry point whose split-K
scratch is a fixed array inside the library image. This test calls it through the C ABI and checks it
against the allocating entry point, twice in a row with different inputs (the shared array keeps the
previous call's contents, so the second call proves that it is cleared). The file is named so that
pytest collects it last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(M, N, K, seed):
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
    w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda", generator=g)
    st = torch.rand(M, device="cuda", generator=g) * 0.045 + 0.005
    sc = torch.rand(N, device="cuda", generator=g) * 0.009 + 0.001
    return a, st, w, sc


def _run(lib, name, a, st, w, sc, with_acc):
    M, K = a.shape; N = w.shape[0]
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    if with_acc:
        rc = getattr(lib, name)(p(a), p(st), p(w), p(sc), M, N, K, None, p(y), s)
    else:
        rc = getattr(lib, name)(p(a), p(st), p(w), p(sc), M, N, K, p(y), s)
    torch.cuda.synchronize()
    return rc, y


@pytest.mark.parametrize("M,N,K", [(32, 2048, 2048), (64, 16384, 2048), (12, 2048, 8192), (5, 1024, 2064), (40, 520, 400)])
def test_noalloc_matches_allocating_entry_point(M, N, K):
    """Also covers K that is not a multiple of 128 (the tensor maps zero-fill the ragged last K block) and
    M <= 8, where the allocating entry point takes the dp4a GEMV while this one stays on the tensor cores."""
    import flexllm_b200
    import oracle
    lib = flexllm_b200.lib()
    for call in range(2):                       # two calls in a row on the shared built-in scratch
        a, st, w, sc = _inputs(M, N, K, 100 + call)
        rc0, y0 = _run(lib, "flexllm_linear_decode_i8", a, st, w, sc, True)
        rc1, y1 = _run(lib, "flexllm_linear_decode_i8_noalloc", a, st, w, sc, False)
        assert rc0 == 0 and rc1 == 0, (rc0, rc1)
        # integer accumulation is exact and the dequant arithmetic identical: bit-for-bit equality
        assert torch.equal(y0.view(torch.int32), y1.view(torch.int32)), f"call {call}: outputs differ"
        # and both equal the CPU oracle's linear layer (exact int32 sums, then ((float)acc * s_tok) * s_ch)
        _, want = oracle.linear_i8(a.cpu().numpy(), st.cpu().numpy(), w.cpu().numpy(), sc.cpu().numpy())
        assert np.array_equal(y1.cpu().numpy().view(np.uint32), want.view(np.uint32)), f"call {call}: differs from the oracle"
    assert lib.flexllm_device_status() == 0     # no bounded wait ran out on the way


def test_noalloc_allocates_no_device_memory():
    """What the entry point is for: after the first call on the device (which only looks up addresses), further
    calls leave the amount of free device memory exactly as it was."""
    import flexllm_b200
    lib = flexllm_b200.lib()
    a, st, w, sc = _inputs(32, 4096, 2048, 9)
    rc, _ = _run(lib, "flexllm_linear_decode_i8_noalloc", a, st, w, sc, False)      # first call: set-up
    assert rc == 0
    y = torch.empty((32, 4096), dtype=torch.float32, device="cuda")
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(5):
        assert lib.flexllm_linear_decode_i8_noalloc(p(a), p(st), p(w), p(sc), 32, 4096, 2048, p(y), s) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0


def test_noalloc_rejects_oversize():
    import flexllm_b200
    from flexllm_b200 import _lib
    lib = flexllm_b200.lib()
    a, st, w, sc = _inputs(64, 16384 + 128, 128, 7)          # 64 x 16512 > 64 x 16384
    rc, y = _run(lib, "flexllm_linear_decode_i8_noalloc", a, st, w, sc, False)
    assert rc == _lib.ETOOBIG
    assert torch.isnan(y).all()                              # untouched
    assert b"built-in" in lib.flexllm_status_string(rc)
