#!/usr/bin/env python
"""Throughput of the quantized Llama-3.2-1B path on B200: prefill + greedy decode tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the full Llama-3.2-1B W8A8 model, 16 layers, hidden 2048, 32/8 heads, FFN 8192, vocab 128256, tied
embeddings; random-init int8 weights with per-channel scales, synthetic token ids; batch 32,
prefill 1024 tokens, greedy decode of 256 tokens. One "step" = one such request batch.

  value : tokens/s with the prompt ids already on the device (CUDA events on the launching stream)
  e2e   : the same request through flexllm_model_generate_host: prompt ids in pinned HOST memory,
          host->device copy, prefill, decode, device->host copy of the generated ids inside the
          timed region
  N > 1 : one process per GPU. Default (--parallel tp): ONE batch of 32 sequences on all N GPUs, prefill
          tensor-parallel, decode batch-parallel after the KV cache has been regrouped by sequence (strong
          scaling; rank 0 also checks the tokens against a single-GPU run: "tp_tokens_match"). --parallel dp:
          every rank serves its own batch of 32 (independent replicas, weak scaling). Time = max over ranks.

--impl reference times the reference's own operator templates (oracle/_ref, built from the FlexLLM
sources through the header shim) on the host cores, on a bounded sample of the same workload.
Prints one JSON line on rank 0.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(layers=16, hidden=2048, heads_q=32, heads_kv=8, ffn=8192, vocab=128256)
BATCH, PREFILL, NEW = 32, 1024, 256
METRIC = "llama32_1b_w8a8_prefill_decode_tokens_per_s"


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


# ------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": "nvmlClocksEventReasonHwSlowdown", "hw_thermal_slowdown": "nvmlClocksEventReasonHwThermalSlowdown",
                 "sw_thermal_slowdown": "nvmlClocksEventReasonSwThermalSlowdown", "sw_power_cap": "nvmlClocksEventReasonSwPowerCap"}
        fallback = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
                r = get(self.h)
                for k, attr in names.items():
                    if r & getattr(nv, attr, fallback[k]):
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.05)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def mark(self):
        """Start of the timed region: earlier samples are dropped."""
        self._first = len(self.samples)
        self.reasons.clear()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        s = sorted(self.samples[getattr(self, "_first", 0):])
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------------------------ CPU arms
def cpu_port_baseline():
    """The plain-C++ oracle (all host threads) on a bounded sample: the full 16-layer model,
    one sequence, 64 prompt tokens + 2 generated."""
    import numpy as np
    import oracle
    oracle.set_threads(os.cpu_count() or 1)      # a launcher (torchrun) may have exported OMP_NUM_THREADS=1
    from flexllm_b200 import synthetic
    S, n_new = 64, 2
    W = synthetic.numpy_weights(max_ctx=S + n_new, seed=0, **CFG)
    tok = np.random.default_rng(1).integers(0, CFG["vocab"], (1, S)).astype(np.int32)
    t0 = time.perf_counter()
    oracle.model_generate(W, tok, n_new)
    dt = time.perf_counter() - t0
    return {"value": (S + n_new) / dt, "unit": "tokens/s", "cores": oracle.get_threads(), "kind": "port",
            "sample": f"full 16-layer model, batch 1, {S} prompt + {n_new} generated tokens, {dt:.1f} s"}


def reference_arm(args):
    """The reference's own operator templates (oracle/_ref) over one decoder layer on one
    8-token block (the reference's TOKEN_PARALLEL), output channels split over the host threads;
    whole-model tokens/s = 8 / (16 layers x layer time + head time)."""
    import numpy as np
    import oracle
    from concurrent.futures import ThreadPoolExecutor
    from flexllm_b200 import synthetic
    R = oracle.ref
    kind = "reference" if R is not None else "port"
    T = 8
    threads = os.cpu_count() or 1
    oracle.set_threads(threads)                  # a launcher (torchrun) may have exported OMP_NUM_THREADS=1
    W = synthetic.numpy_weights(1, CFG["hidden"], CFG["heads_q"], CFG["heads_kv"], CFG["ffn"], 2048, T + 1, seed=0)
    g = np.random.default_rng(2)
    x = g.standard_normal((T, CFG["hidden"])).astype(np.float32)
    pool = ThreadPoolExecutor(threads)

    def gemm(aq, w):
        if R is None:
            return oracle.gemm_s8s8(aq, w)
        n = w.shape[0]
        step = max(16, (n // threads + 15) // 16 * 16)
        parts = list(pool.map(lambda i: R.gemm_s8s8(aq, w[i:i + step]), range(0, n, step)))
        return np.concatenate(parts, axis=1)

    O = R if R is not None else oracle

    def linear(xf, w, s):
        q, sc = O.quant_per_token(xf)
        return O.dequant(gemm(q, w), sc, s)

    def layer():
        HQ, HKV = CFG["heads_q"], CFG["heads_kv"]
        xn = O.rmsnorm(x, W["g0"][0], lanes=0) if R is not None else oracle.rmsnorm(x, W["g0"][0])
        qf = linear(xn, W["wq"][0], W["sq"][0]); kf = linear(xn, W["wk"][0], W["sk"][0]); vf = linear(xn, W["wv"][0], W["sv"][0])
        pos = np.arange(T, dtype=np.int32)
        if R is not None:           # RoPE, 64-point FHT and the per-head quantiser through the reference templates too
            qr = R.fht(R.rope_prefill(qf.reshape(T, HQ, 64), W["cos_t"], W["sin_t"]), 8.0)
            kr = R.fht(R.rope_prefill(kf.reshape(T, HKV, 64), W["cos_t"], W["sin_t"]), 8.0)
            hq_ = lambda x, H: [np.stack(z) for z in zip(*[R.head_quant(x.reshape(T, H, 64)[t]) for t in range(T)])]
            (q2, qs2), (k2, ks2), (v2, vs2) = hq_(qr, HQ), hq_(kr, HKV), hq_(vf, HKV)
        else:
            qr = oracle.fht(oracle.rope(qf.reshape(T, HQ, 64), pos, W["cos_t"], W["sin_t"]), 8.0)
            kr = oracle.fht(oracle.rope(kf.reshape(T, HKV, 64), pos, W["cos_t"], W["sin_t"]), 8.0)
            q2, qs2 = oracle.quant_per_token(qr.reshape(T * HQ, 64)); k2, ks2 = oracle.quant_per_token(kr.reshape(T * HKV, 64))
            v2, vs2 = oracle.quant_per_token(vf.reshape(T * HKV, 64))
        q2 = q2.reshape(T, HQ, 64); k2 = k2.reshape(T, HKV, 64); v2 = v2.reshape(T, HKV, 64)
        qs2 = qs2.reshape(T, HQ); ks2 = ks2.reshape(T, HKV); vs2 = vs2.reshape(T, HKV)
        att = np.zeros((T, HQ * 64), np.float32)
        for t in range(T):
            for h in range(HQ):
                r = oracle.attn_row(q2[t, h], qs2[t, h], k2[:t + 1, h // 4], ks2[:t + 1, h // 4], v2[:t + 1, h // 4],
                                    vs2[:t + 1, h // 4], W["a_s"][0][h])
                att[t, h * 64:(h + 1) * 64] = r["out"]
        x1 = O.residual(x, linear(att, W["wo"][0], W["so"][0]))
        xn1 = O.rmsnorm(x1, W["g1"][0], lanes=0) if R is not None else oracle.rmsnorm(x1, W["g1"][0])
        gq, gs = O.quant_per_token(xn1)
        gt = O.dequant(gemm(gq, W["wg"][0]), gs, W["sg"][0]); up = O.dequant(gemm(gq, W["wu"][0]), gs, W["su"][0])
        act = O.gate_mul(O.silu(gt), up) if R is not None else oracle.silu_mul(gt, up)
        hf = O.fht(act, 90.50966799)
        return O.residual(x1, linear(hf, W["wd"][0], W["sd"][0]))

    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        layer()
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    t_layer = sum(times) / len(times)
    tok_s = T / (t_layer * CFG["layers"])
    sample = (f"one decoder layer on one {T}-token block, {t_layer:.2f} s per layer, x{CFG['layers']} layers, lm_head not included; "
              + ("mixed: quantisers, int8 GEMMs, dequant, RMSNorm, RoPE, FHT, SiLU, gate and residual through the reference's own templates, "
                 "the 8 x 8 attention rows (scores, softmax, P.V) through the plain-C++ port" if R is not None else "everything through the plain-C++ port"))
    line = {"impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t_layer * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "s8", "data": "synthetic", "config": workload_config(),
            "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(world=1, parallel="dp"):
    tp = parallel == "tp" and world > 1
    return {"workload": "config5: Llama-3.2-1B W8A8 SpinQuant, random-init weights, batch 32" + (" in total" if tp else " per GPU") +
                        ", prefill 1024 + greedy decode 256",
            "global_batch": BATCH if tp else BATCH * world, "prefill_len": PREFILL, "decode_len": NEW, "layers": CFG["layers"],
            "l2": "weights (1.24 GB) and activations exceed the 126 MB L2; no flush needed",
            "parallelism": (f"tp{world}: prefill tensor-parallel (column-parallel q/k/v/gate/up by heads / FFN channels; token rows owned per "
                            f"rank in between: int8 attention columns and fp32 gated activations go to the rows' owners by all-to-all, which run "
                            f"the o and down projections for their rows with the full weights), then the KV cache regrouped "
                            f"by sequence and {BATCH // world} sequences decoded per rank (batch-parallel decode streams)"
                            if tp else ("single GPU" if world == 1 else f"dp{world}: batch-parallel replicas, no data-path collective"))}


# ------------------------------------------------------------------------------------ GPU arm
def kernel_roofline(F, torch, peaks):
    """Times the decode linear layers (the HBM-bound weight streaming that dominates a decode step)
    in isolation, with CUDA events on the launching stream, on the shapes of one layer. Algorithmic
    bytes per launch = weight bytes + scales + int8 activations in + fp32 out."""
    lib = F.lib()
    B = BATCH
    shapes = [("qkv", 3072, 2048), ("o", 2048, 2048), ("gate_up", 16384, 2048), ("down", 2048, 8192)]
    total_bytes, total_ms = 0, 0.0
    detail = {}
    # more weight sets than fit in L2, cycled, so that every launch streams from HBM
    for name, N, K in shapes:
        nset = max(2, int(300e6 // (N * K)) + 1)
        ws = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda") for _ in range(nset)]
        a = torch.randint(-127, 128, (B, K), dtype=torch.int8, device="cuda")
        st = torch.rand(B, device="cuda"); sc = torch.rand(N, device="cuda")
        y = torch.empty((B, N), dtype=torch.float32, device="cuda")
        s = torch.cuda.current_stream().cuda_stream

        def run(i):
            w = ws[i % nset]
            rc = lib.flexllm_linear_decode_i8(a.data_ptr(), st.data_ptr(), w.data_ptr(), sc.data_ptr(), B, N, K, None, y.data_ptr(), s)
            assert rc == 0, rc
        for i in range(5):
            run(i)
        torch.cuda.synchronize()
        # the n launches are replayed from a CUDA graph so that the figure is the kernels' own time
        # (back to back on the stream), not the host's cost of issuing them
        n = 40
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            s = side.cuda_stream
            with torch.cuda.graph(graph, stream=side):
                for i in range(n):
                    run(i)
            graph.replay()
            side.synchronize()
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(side)
            graph.replay()
            e1.record(side); side.synchronize()
        ms = e0.elapsed_time(e1) / n
        nbytes = N * K + 4 * N + B * K + 4 * B + 4 * B * N
        detail[name] = {"us": round(ms * 1e3, 2), "GB/s": round(nbytes / ms / 1e6, 1)}
        total_bytes += nbytes; total_ms += ms
    achieved = total_bytes / total_ms / 1e6
    return {"kernel": "decode linear layers as stand-alone launches (gemv / tcgen05 skinny GEMM), one layer's four projections, batch 32",
            "achieved": round(achieved, 1), "unit": "GB/s", "per_projection": detail}


# ------------------------------------------------------------------------------------ unit configurations
def unit_configs(F, torch, peaks, with_cpu=True):
    """The four operator-level configurations of the workload family, each timed on the device with CUDA events
    through the C ABI and set against its roofline; beside each, the CPU oracle (plain-C++ port, all host threads)
    on the same or a stated smaller case.

      config1  prefill linear layer 128 x 2048 x 2048 (int32 sums + fp32 dequant)
      config2  decode MLP block at batch 1 and batch 64 (RMSNorm, quant, gate, up, SiLU*up, FHT-8192, quant, down, +residual)
      config3  prefill GQA attention, batch 4 x 1024, 32/8 heads
      config4  decode attention, batch 64, contexts ~ U{512..8192}, 16 layers of paged int8 KV cache
    Inputs that must come from HBM are cycled through more copies than fit in the 126 MB L2."""
    import numpy as np
    lib = F.lib()
    dev = "cuda"
    if with_cpu:
        import oracle
        oracle.set_threads(os.cpu_count() or 1)  # a launcher (torchrun) may have exported OMP_NUM_THREADS=1
    hbm = peaks.get("hbm_gbs") or 6650.0
    i8_proxy = 2.0 * (peaks.get("bf16_tflops") or 1590.0)
    gen = torch.Generator(device=dev).manual_seed(11)
    r8 = lambda *sh: torch.randint(-127, 128, sh, dtype=torch.int8, device=dev, generator=gen)
    ru = lambda lo, hi, *sh: torch.rand(sh, device=dev, generator=gen) * (hi - lo) + lo
    P = lambda t: t.data_ptr()
    out = {}

    def graph_time(body, n_iter):
        """body(i, stream) issues iteration i; n_iter iterations are replayed from one CUDA graph."""
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for i in range(min(3, n_iter)):
                body(i, side.cuda_stream)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                for i in range(n_iter):
                    body(i, side.cuda_stream)
            g.replay(); side.synchronize()
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(side); g.replay(); e1.record(side); side.synchronize()
        return e0.elapsed_time(e1) / n_iter

    def cpu_time(fn, reps=1):
        if not with_cpu:
            return None
        import oracle  # noqa: F401  (the CPU leg is the only user of the oracle here)
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        return (time.perf_counter() - t0) / reps * 1e3

    # ---- int8 tensor-core ceiling of this library's own main loop (epilogue stores nothing)
    M, N, K = 8192, 8192, 2048
    a = r8(M, K); w = r8(N, K)
    ms = graph_time(lambda i, st: lib.flexllm_gemm_i8_mainloop_probe(P(a), P(w), M, N, K, st), 10)
    int8_peak = 2.0 * M * N * K / ms / 1e9
    out["int8_peak_measured"] = {"tops": round(int8_peak, 1), "how": "tcgen05.mma kind::i8 main loop of the prefill GEMM on 8192 x 8192 x 2048, "
                                 "accumulators drained, nothing stored", "proxy_2x_bf16_tops": round(i8_proxy, 1)}
    del a, w

    # ---- config 1
    M, N, K = 128, 2048, 2048
    nset = 40                                           # 40 x 4 MB of weights > L2
    ws = [r8(N, K) for _ in range(nset)]
    a = r8(M, K); st_ = ru(0.005, 0.05, M); sc = ru(0.001, 0.01, N)
    acc = torch.empty((M, N), dtype=torch.int32, device=dev); y = torch.empty((M, N), dtype=torch.float32, device=dev)
    ms = graph_time(lambda i, st: lib.flexllm_linear_prefill_i8(P(a), P(st_), P(ws[i % nset]), P(sc), M, N, K, None, P(y), st), nset)
    ops, nbytes = 2.0 * M * N * K, 262144 + 4194304 + 512 + 8192 + 1048576
    c1 = {"ms": round(ms, 5), "tops": round(ops / ms / 1e9, 2), "GB/s": round(nbytes / ms / 1e6, 1),
          "frac_hbm": round(nbytes / ms / 1e6 / hbm, 4), "frac_int8_proxy": round(ops / ms / 1e9 / i8_proxy, 4),
          "bound": "hbm + launch latency (16 output tiles on 148 SMs)", "algorithmic_bytes": nbytes, "ops": int(ops)}
    if with_cpu:
        import oracle
        an, wn = a.cpu().numpy(), ws[0].cpu().numpy(); sn, cn = st_.cpu().numpy(), sc.cpu().numpy()
        c1["cpu_port_ms"] = round(cpu_time(lambda: oracle.linear_i8(an, sn, wn, cn), 3), 2)
        if oracle.ref is not None:                       # the reference's own systolic-array template, 16 tokens of the 128
            t = cpu_time(lambda: oracle.ref.gemm_s8s8(an[:16], wn))
            c1["cpu_reference_ms"] = round(t * (M / 16), 1)
            c1["cpu_reference_sample"] = "reference template on 16 of the 128 tokens, one thread, scaled x8"
    out["config1_prefill_linear_128x2048x2048"] = c1
    del ws

    # ---- config 2
    D, Fd = 2048, 8192
    nset = 4                                            # 4 x 50 MB of weights > L2
    wg = [r8(Fd, D) for _ in range(nset)]; wu = [r8(Fd, D) for _ in range(nset)]; wd = [r8(D, Fd) for _ in range(nset)]
    sg, su, sd = ru(0.001, 0.01, Fd), ru(0.001, 0.01, Fd), ru(0.001, 0.01, D)
    gamma = 1 + 0.02 * torch.randn(D, device=dev, generator=gen)
    c2 = {}
    for B in (1, 64):
        h = torch.randn((B, D), device=dev, generator=gen)
        xq = torch.empty((B, D), dtype=torch.int8, device=dev); xs = torch.empty(B, device=dev)
        gt = torch.empty((B, Fd), device=dev); up = torch.empty((B, Fd), device=dev)
        hq = torch.empty((B, Fd), dtype=torch.int8, device=dev); hs = torch.empty(B, device=dev)
        o = torch.empty((B, D), device=dev)

        def block(i, st, B=B, h=h, xq=xq, xs=xs, gt=gt, up=up, hq=hq, hs=hs, o=o):
            j = i % nset
            rc = lib.flexllm_rmsnorm_quant(P(h), P(gamma), B, D, 1e-5, 8, None, P(xq), P(xs), st)
            rc |= lib.flexllm_linear_decode_i8(P(xq), P(xs), P(wg[j]), P(sg), B, Fd, D, None, P(gt), st)
            rc |= lib.flexllm_linear_decode_i8(P(xq), P(xs), P(wu[j]), P(su), B, Fd, D, None, P(up), st)
            rc |= lib.flexllm_swiglu_fht_quant(P(gt), P(up), B, Fd, 90.50966799, P(hq), P(hs), None, st)
            rc |= lib.flexllm_linear_decode_i8_residual(P(hq), P(hs), P(wd[j]), P(sd), B, D, Fd, P(h), P(o), st)
            assert rc == 0, rc
        ms5 = graph_time(block, 4 * nset)
        # the same block through the one-call entry point (fused gate|up weights, four dependent launches)
        wgu = [torch.cat([wg[j], wu[j]]) for j in range(nset)]; sgu = torch.cat([sg, su])
        ws_n = lib.flexllm_mlp_block_workspace(B, D, Fd)
        ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)

        def block1(i, st, B=B, h=h, o=o):
            j = i % nset
            rc = lib.flexllm_mlp_block_decode(P(h), P(gamma), P(wgu[j]), P(sgu), P(wd[j]), P(sd), B, D, Fd, 1e-5, 8, 90.50966799,
                                              P(o), P(ws), ws_n, st)
            assert rc == 0, rc
        ms = graph_time(block1, 4 * nset)
        del wgu
        nbytes = 50331648 + 73728 + 8192 + 2 * B * 8192
        e = {"ms": round(ms, 5), "GB/s": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / hbm, 4),
             "bound": "hbm (weights)", "algorithmic_bytes": nbytes, "launches_per_block": 4,
             "entry": "flexllm_mlp_block_decode", "ms_as_five_operator_calls": round(ms5, 5)}
        if with_cpu:
            import oracle
            hn = h.cpu().numpy()
            args = [hn, gamma.cpu().numpy(), wg[0].cpu().numpy(), sg.cpu().numpy(), wu[0].cpu().numpy(), su.cpu().numpy(),
                    wd[0].cpu().numpy(), sd.cpu().numpy()]
            e["cpu_port_ms"] = round(cpu_time(lambda: oracle.mlp_block(*args, lanes=8)), 2)
        c2[f"batch{B}"] = e
    out["config2_decode_mlp_block"] = c2
    del wg, wu, wd

    # ---- config 3
    from flexllm_b200 import synthetic
    B, S, HQ, HKV = 4, 1024, 32, 8
    q, k, v = r8(B, S, HQ, 64), r8(B, S, HKV, 64), r8(B, S, HKV, 64)
    qs, ks, vs = ru(0.005, 0.05, B, S, HQ), ru(0.005, 0.05, B, S, HKV), ru(0.005, 0.05, B, S, HKV)
    ct, sn_ = synthetic.rope_table(S); ct = torch.from_numpy(ct).to(dev); sn_ = torch.from_numpy(sn_).to(dev)
    a_s = torch.full((HQ,), 1.0 / 255, device=dev)
    for _ in range(3):
        F.MHA_i8xi8_Prefilling(q, qs, k, ks, v, vs, ct, sn_, a_s)
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    n = 5
    e0.record()
    for _ in range(n):
        F.MHA_i8xi8_Prefilling(q, qs, k, ks, v, vs, ct, sn_, a_s)
    e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    ops, nbytes = 17196646400.0, 47185920
    c3 = {"ms": round(ms, 4), "tops": round(ops / ms / 1e9, 2), "frac_int8_proxy": round(ops / ms / 1e9 / i8_proxy, 4),
          "GB/s": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / hbm, 4),
          "bound": "CUDA-core softmax arithmetic (exact ordered sums, correctly rounded exp)", "algorithmic_bytes": nbytes, "ops": int(ops),
          "l2": "working set 47 MB < L2: the operands of consecutive runs may hit L2 (the exp scratch is written and re-read each run)"}
    if with_cpu:
        import oracle
        an = [t.cpu().numpy() for t in (q[:1], qs[:1], k[:1], ks[:1], v[:1], vs[:1])]
        t = cpu_time(lambda: oracle.mha_prefill(*an, ct.cpu().numpy(), sn_.cpu().numpy(), a_s.cpu().numpy()))
        c3["cpu_port_ms"] = round(t * B, 1); c3["cpu_port_sample"] = "1 of the 4 sequences, scaled x4"
    out["config3_prefill_attention_b4_s1024"] = c3
    del q, k, v

    # ---- config 4
    B, L, HQ, HKV, PAGE = 64, 16, 32, 8, 64
    rng = np.random.default_rng(4)
    ctx = rng.integers(512, 8193, B).astype(np.int32)
    pages_per_seq = (ctx + 1 + PAGE - 1) // PAGE
    n_pages = int(pages_per_seq.sum()) + 3
    max_pages = int(pages_per_seq.max())
    perm = rng.permutation(n_pages).astype(np.int32)
    pt = np.zeros((B, max_pages), np.int32); o_ = 0
    for b in range(B):
        pt[b, :pages_per_seq[b]] = perm[o_:o_ + pages_per_seq[b]]; o_ += pages_per_seq[b]
    cache = F.KVCache(L, n_pages, HKV)
    for l in range(L):
        kd, ksd, vd, vsd = cache.pools(l)
        kd.copy_(r8(n_pages, HKV, PAGE, 64)); vd.copy_(r8(n_pages, HKV, 64, PAGE))
        ksd.copy_(ru(0.005, 0.05, n_pages, HKV, PAGE)); vsd.copy_(ru(0.005, 0.05, n_pages, HKV, PAGE))
    max_ctx = int(ctx.max()) + 1
    ct, sn_ = synthetic.rope_table(max_ctx + 1); ct = torch.from_numpy(ct).to(dev); sn_ = torch.from_numpy(sn_).to(dev)
    q, k, v = r8(B, HQ, 64), r8(B, HKV, 64), r8(B, HKV, 64)
    qs, ks, vs = ru(0.005, 0.05, B, HQ), ru(0.005, 0.05, B, HKV), ru(0.005, 0.05, B, HKV)
    ptd = torch.from_numpy(pt).to(dev); ctxd = torch.from_numpy(ctx).to(dev)
    nb = lib.flexllm_mha_decode_workspace(B, HQ, max_ctx)
    wsb = torch.empty(nb, dtype=torch.uint8, device=dev); o = torch.empty((B, HQ * 64), device=dev)

    def step(i, st):
        for l in range(L):
            rc = lib.flexllm_mha_i8xi8_decode(cache._h, l, P(q), P(qs), P(k), P(ks), P(v), P(vs), P(ct), P(sn_), P(a_s), P(ptd), max_pages,
                                              P(ctxd), max_ctx, B, HQ, P(o), None, P(wsb), nb, st)
            assert rc == 0, rc
    ms = graph_time(step, 3)                           # the step appends at the same slot every time: contents do not matter for time
    nbytes = 1088 * int((ctx.astype(np.int64) + 1).sum()) * L
    c4 = {"ms": round(ms, 4), "ms_per_layer": round(ms / L, 4), "GB/s": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / hbm, 4),
          "bound": "hbm (KV pages)", "algorithmic_bytes": nbytes, "sum_ctx_plus_1": int((ctx.astype(np.int64) + 1).sum())}
    if with_cpu:
        import oracle
        Bc = 8                                          # 8 of the 64 sequences, one layer
        npg = int(pages_per_seq[:Bc].sum()) + 1
        pt8 = np.zeros((Bc, max_pages), np.int32); o_ = 0
        for b in range(Bc):
            pt8[b, :pages_per_seq[b]] = np.arange(o_, o_ + pages_per_seq[b]); o_ += pages_per_seq[b]
        kp = rng.integers(-127, 128, (npg, HKV, PAGE, 64), dtype=np.int8); vp = rng.integers(-127, 128, (npg, HKV, PAGE, 64), dtype=np.int8)
        ksp = rng.uniform(0.005, 0.05, (npg, HKV, PAGE)).astype(np.float32); vsp = ksp.copy()
        hn = lambda t: t[:Bc].cpu().numpy()
        t = cpu_time(lambda: oracle.mha_decode(hn(q), hn(qs), hn(k), hn(ks), hn(v), hn(vs), ct.cpu().numpy(), sn_.cpu().numpy(),
                                               a_s.cpu().numpy(), kp, ksp, vp, vsp, pt8, ctx[:Bc]))
        share = float((ctx[:Bc].astype(np.int64) + 1).sum()) / float((ctx.astype(np.int64) + 1).sum())
        c4["cpu_port_ms"] = round(t / share * L, 1); c4["cpu_port_sample"] = "8 of the 64 sequences on one layer, scaled by cached tokens and x16 layers"
    out["config4_decode_attention_b64"] = c4
    cache.close()
    if with_cpu:
        import oracle
        out["cpu_threads"] = oracle.get_threads()
    return out


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_mega_kernel launch: ncu capture at context 131..136
# (1.358 GB read + 0.117 GB written, profiles/decode_mega_kernel_batch32_ctx131.md) plus the KV pages the
# bench's mean context of 1152 adds (16 layers x 1088 B x 32 sequences x 1019 tokens; KV traffic is proportional)
DRAM_TRAFFIC_PER_LAUNCH = int(1.358e9 + 0.117e9 + 16 * 1088 * 32 * 1019)


def prefill_ops(nb):
    """Integer operations of one prefill of nb sequences: 2 x tokens x weight elements of the 16 layers, the causal
    attention (4 x heads x 64 x S(S+1)/2 per sequence and layer) and the lm_head on each sequence's last token."""
    D, Fd, V, L = CFG["hidden"], CFG["ffn"], CFG["vocab"], CFG["layers"]
    qkv = (CFG["heads_q"] + 2 * CFG["heads_kv"]) * 64
    per_layer_w = qkv * D + D * D + 2 * Fd * D + D * Fd
    lin = 2.0 * nb * PREFILL * L * per_layer_w
    att = L * 4.0 * nb * CFG["heads_q"] * 64 * (PREFILL * (PREFILL + 1) / 2)
    return lin + att + 2.0 * nb * V * D


def decode_step_bytes(batch=None):
    """Algorithmic bytes one decode step has to read: every int8 weight once (layers + lm_head), the
    scales, and the int8 KV pages of all layers for the step's context lengths (K and V rows of 64
    bytes per KV head plus two fp32 scales per head: 1088 bytes per cached token and layer).
    batch: sequences the launch decodes (default: the whole batch)."""
    D, F, V, L = CFG["hidden"], CFG["ffn"], CFG["vocab"], CFG["layers"]
    qkv = (CFG["heads_q"] + 2 * CFG["heads_kv"]) * 64
    weights = L * (qkv * D + D * D + 2 * F * D + D * F) + V * D
    scales = 4 * (L * (qkv + D + 2 * F + D + 2 * D) + V + D)
    kv = L * 1088 * (BATCH if batch is None else batch) * (PREFILL + NEW / 2)
    return weights + scales + kv


def micro(args):
    """Runs one kernel a few times on a small fixed case (for ncu captures; prints its mean time)."""
    import torch
    import flexllm_b200 as F
    from flexllm_b200 import synthetic
    F.lib()
    name = args.micro
    dev = "cuda"
    if name in ("attn_prefill", "attn_prefill_online"):          # the prefill-attention workload: B=4, S=1024, 32/8 heads
        B, S, HQ, HKV = 4, 1024, 32, 8
        g = torch.Generator(device=dev).manual_seed(0)
        r8 = lambda *sh: torch.randint(-127, 128, sh, dtype=torch.int8, device=dev, generator=g)
        rs = lambda *sh: torch.rand(sh, device=dev, generator=g) * 0.045 + 0.005
        q, k, v, qs, ks, vs = r8(B, S, HQ, 64), r8(B, S, HKV, 64), r8(B, S, HKV, 64), rs(B, S, HQ), rs(B, S, HKV), rs(B, S, HKV)
        c, s_ = synthetic.rope_table(S); c = torch.from_numpy(c).to(dev); s_ = torch.from_numpy(s_).to(dev)
        a_s = torch.full((HQ,), 0.05 / 255, device=dev)
        fn = (lambda: F.MHA_i8xi8_Prefilling(q, qs, k, ks, v, vs, c, s_, a_s)) if name == "attn_prefill" else \
             (lambda: F.MHA_i8xi8_Prefilling_online(q, qs, k, ks, v, vs, c, s_))      # single-sweep variant, not bit-exact
    elif name in ("gemm_prefill", "gemm_prefill_k8192"):
        M, N, K = (8192, 8192, 2048) if name == "gemm_prefill" else (8192, 2048, 8192)
        a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev); w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev)
        st = torch.rand(M, device=dev); sc = torch.rand(N, device=dev)
        fn = lambda: F.pref_Linear_Layer_i8xi8(a, st, w, sc)
    elif name == "decode_linear":       # gate|up projection of one layer, batch 32; 5 weight sets > L2
        N, K, B = 16384, 2048, 32
        ws = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(5)]
        a = torch.randint(-127, 128, (B, K), dtype=torch.int8, device=dev); st = torch.rand(B, device=dev); sc = torch.rand(N, device=dev)
        it = [0]
        def fn():
            it[0] += 1
            return F.dec_Linear_Layer_i8xi8(a, st, ws[it[0] % 5], sc)
    elif name == "gemv_b1":             # decode linear layer for ONE token (dp4a weight streaming), gate projection, 8 weight sets > L2
        N, K, B = 8192, 2048, 1
        ws = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(8)]
        a = torch.randint(-127, 128, (B, K), dtype=torch.int8, device=dev); st = torch.rand(B, device=dev); sc = torch.rand(N, device=dev)
        it = [0]
        def fn():
            it[0] += 1
            return F.dec_Linear_Layer_i8xi8(a, st, ws[it[0] % 8], sc)
    elif name == "decode_attention":    # one layer of paged decode attention, batch 64, contexts ~ U{512..8192} (about 300 MB of KV pages)
        import numpy as np
        B, HQ, HKV, PAGE = 64, 32, 8, 64
        rng = np.random.default_rng(4)
        ctx = rng.integers(512, 8193, B).astype(np.int32)
        pages = (ctx + 1 + PAGE - 1) // PAGE
        n_pages, max_pages = int(pages.sum()) + 3, int(pages.max())
        perm = rng.permutation(n_pages).astype(np.int32)
        pt = np.zeros((B, max_pages), np.int32); o = 0
        for b in range(B):
            pt[b, :pages[b]] = perm[o:o + pages[b]]; o += pages[b]
        cache = F.KVCache(1, n_pages, HKV)
        kd, ksd, vd, vsd = cache.pools(0)
        kd.copy_(torch.randint(-127, 128, kd.shape, dtype=torch.int8, device=dev)); vd.copy_(torch.randint(-127, 128, vd.shape, dtype=torch.int8, device=dev))
        ksd.copy_(torch.rand(ksd.shape, device=dev) * 0.045 + 0.005); vsd.copy_(torch.rand(vsd.shape, device=dev) * 0.045 + 0.005)
        max_ctx = int(ctx.max()) + 1
        c, s_ = synthetic.rope_table(max_ctx + 1); c = torch.from_numpy(c).to(dev); s_ = torch.from_numpy(s_).to(dev)
        q = torch.randint(-127, 128, (B, HQ, 64), dtype=torch.int8, device=dev); k = torch.randint(-127, 128, (B, HKV, 64), dtype=torch.int8, device=dev)
        v = torch.randint(-127, 128, (B, HKV, 64), dtype=torch.int8, device=dev)
        qs = torch.rand((B, HQ), device=dev) * 0.045 + 0.005; ks = torch.rand((B, HKV), device=dev) * 0.045 + 0.005; vs = ks.clone()
        a_s = torch.full((HQ,), 1.0 / 255, device=dev)
        ptd, ctxd = torch.from_numpy(pt).to(dev), torch.from_numpy(ctx).to(dev)
        fn = lambda: F.MHA_i8xi8_Decoding(cache, 0, q, qs, k, ks, v, vs, c, s_, a_s, ptd, ctxd, max_ctx)
    elif name == "swiglu_fht":
        gg = torch.randn((4096, 8192), device=dev); uu = torch.randn((4096, 8192), device=dev)
        fn = lambda: F.swiglu_fht_quant(gg, uu)
    elif name == "rmsnorm_prefill":     # RMSNorm (prefill summation order) + per-token quantiser on 32768 x 2048 fp32 rows (268 MB)
        x = torch.randn((32768, 2048), device=dev); gam = torch.ones(2048, device=dev)
        fn = lambda: F.pref_Layer_Norm(x, gam, quant=True, want_y=False)
    elif name == "prefill_small":       # a 2-layer model's prefill of 8 x 1024 tokens: every prefill kernel at its model shapes, < 2 GB
        cfg2 = dict(CFG); cfg2["layers"] = 2
        m = F.Model(max_batch=8, max_prefill=1024, max_ctx=1040, **cfg2)
        synthetic.load_random_weights(m, max_ctx=1040, seed=0, **cfg2)
        tok = torch.randint(0, CFG["vocab"], (8, 1024), dtype=torch.int32).cuda()
        fn = lambda: m.prefill(tok)
    elif name == "decode_step":         # whole-model decode steps (one persistent kernel each) at a short context: small enough for ncu
        S, n = 128, 6
        m = F.Model(max_batch=BATCH, max_prefill=S, max_ctx=S + 16, **CFG)
        synthetic.load_random_weights(m, max_ctx=S + 16, seed=0, **CFG)
        tok = torch.randint(0, CFG["vocab"], (BATCH, S), dtype=torch.int32).cuda()
        m.prefill(tok); m.begin(16)
        m.decode(2, False); torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(); m.decode(n, False); e1.record(); torch.cuda.synchronize()
        print(json.dumps({"micro": name, "ms": e0.elapsed_time(e1) / n, "context": f"{S + 3}..{S + 2 + n}"}))
        m.close()
        return
    else:
        raise SystemExit(f"unknown --micro {name}")
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        fn()
    e1.record(); torch.cuda.synchronize()
    print(json.dumps({"micro": name, "ms": e0.elapsed_time(e1) / 3}))


def gpu_arm(args):
    import torch
    import torch.distributed as dist
    import flexllm_b200 as F
    from flexllm_b200 import synthetic
    rank, world = env_int("RANK", 0), env_int("WORLD_SIZE", 1)
    local = env_int("LOCAL_RANK", 0)
    torch.cuda.set_device(local)
    multi = world > 1
    if multi:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = F.lib()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    tp_comm = [None]

    def communicator():
        if tp_comm[0] is None:
            idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
            if rank == 0:
                idt.copy_(torch.frombuffer(bytearray(F.tp_unique_id()), dtype=torch.uint8))
            dist.broadcast(idt, src=0)
            tp_comm[0] = F.TensorParallel(rank, world, idt.cpu().numpy().tobytes())
        return tp_comm[0]

    def barrier():
        if multi:
            dist.barrier()
        torch.cuda.synchronize()

    def measure(use_tp, steps, with_e2e=True):
        """One partition of the N GPUs. Tensor parallel: every rank holds a slice of the SAME model and
        works on the same batch of 32 (total work fixed: strong scaling). Replicas: every rank runs its own
        model and batch with no data-path collective (weak scaling)."""
        seed = 0 if use_tp else rank
        m = F.Model(max_batch=BATCH, max_prefill=PREFILL, max_ctx=PREFILL + NEW, tp=communicator() if use_tp else None, **CFG)
        synthetic.load_random_weights(m, max_ctx=PREFILL + NEW, seed=seed, **CFG)
        gen = torch.Generator().manual_seed(1234 + seed)
        tok_host = torch.randint(0, CFG["vocab"], (BATCH, PREFILL), dtype=torch.int32, generator=gen).pin_memory()
        out_host = torch.empty((BATCH, NEW), dtype=torch.int32).pin_memory()
        tok_dev = tok_host.cuda()

        def step_device():
            m.prefill(tok_dev); m.begin(NEW); m.decode(NEW - 1, True)

        def step_host():
            m.generate_host(tok_host, NEW, True, out=out_host)

        def timed(fn):
            for _ in range(args.warmup):
                fn()
            # the sampler (NVML initialisation, thread start) comes up BEFORE the barrier: ranks that finish it at different
            # times would otherwise charge their skew to the timed region of the first collective
            sampler = ClockSampler(local); sampler.start()
            barrier()
            sampler.mark()              # only samples taken from here on count
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            l0 = lib.flexllm_launch_count()
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            barrier()
            launches = lib.flexllm_launch_count() - l0
            ms = e0.elapsed_time(e1)
            clocks = sampler.stop()
            if multi:
                t = torch.tensor([ms], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item())
            return ms, launches, clocks

        r = {}
        r["ms_dev"], r["launches"], r["clocks"] = timed(step_device)
        r["ms_e2e"] = timed(step_host)[0] if with_e2e else None
        # phase split (device-resident), one extra step
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record(); m.prefill(tok_dev); m.begin(NEW); ev[1].record(); m.decode(NEW - 1, True); ev[2].record(); torch.cuda.synchronize()
        tt = torch.tensor([ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])], device="cuda")
        if multi:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        r["t_pre"], r["t_dec"] = float(tt[0]), float(tt[1])
        r["units"] = BATCH * (PREFILL + NEW) * (1 if use_tp else world)
        r["value"] = r["units"] * steps / (r["ms_dev"] / 1e3)
        if use_tp:
            # parity carried by the bench itself: the tokens of the partitioned run against ONE GPU running the whole
            # model on the same seed (rank 0 only; the other ranks wait)
            tp_out = m.generate_host(tok_host, NEW, True).clone()
        m.close()
        del m
        torch.cuda.empty_cache()
        if use_tp:
            match = torch.ones(1, device="cuda")
            if rank == 0:
                one = F.Model(max_batch=BATCH, max_prefill=PREFILL, max_ctx=PREFILL + NEW, **CFG)
                synthetic.load_random_weights(one, max_ctx=PREFILL + NEW, seed=seed, **CFG)
                want = one.generate_host(tok_host, NEW, True)
                match[0] = float(torch.equal(want, tp_out))
                one.close()
                del one
                torch.cuda.empty_cache()
            dist.broadcast(match, src=0)
            r["tp_tokens_match"] = bool(match.item() == 1.0)
        return r

    def phases(r, nb):
        dec_bytes = decode_step_bytes(nb // world if nb % world == 0 else None)      # one rank's sequences against one GPU's bandwidth
        return {"prefill_ms": round(r["t_pre"], 3), "prefill_tokens_per_s": round(nb * PREFILL / r["t_pre"] * 1e3, 1),
                "prefill_tops": round(prefill_ops(nb) / r["t_pre"] / 1e9, 1),
                "decode_ms_per_step": round(r["t_dec"] / (NEW - 1), 4),
                "decode_tokens_per_s": round(nb * (NEW - 1) / r["t_dec"] * 1e3, 1),
                "decode_hbm_frac_of_measured": round(dec_bytes / (r["t_dec"] / (NEW - 1) / 1e3) / 1e9 / (peaks.get("hbm_gbs") or 6650.0), 4)}

    # N > 1: the headline partition is --parallel (tensor parallel by default: the partition the workload names;
    # strong scaling on a fixed batch of 32); the other partition (independent replicas, weak scaling) is measured
    # in the same run and reported beside it
    use_tp = multi and args.parallel == "tp"
    tp_error = None
    if use_tp:
        # if the partitioned run fails on any rank, all ranks fall back to independent replicas (and the line says so)
        try:
            main_r = measure(True, args.steps)
        except Exception as e:
            main_r, tp_error = None, f"{type(e).__name__}: {e}"
        ok = torch.tensor([0.0 if main_r is None else 1.0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() != 1.0:
            use_tp = False
            tp_error = tp_error or "failed on another rank"
            main_r = measure(False, args.steps)
    else:
        main_r = measure(False, args.steps)
    other = None
    if multi and not args.no_extras:
        other = {"parallelism": workload_config(world, "dp" if use_tp else "tp")["parallelism"],
                 "scaling": "weak" if use_tp else "strong"}
        try:
            o = measure(not use_tp, min(args.steps, 2), with_e2e=False)
            nb_o = BATCH if not use_tp else BATCH * world
            other.update({"value": round(o["value"], 1), "unit": "tokens/s",
                          "ms_per_step": round(o["ms_dev"] / min(args.steps, 2), 3), "phases": phases(o, nb_o)})
            if "tp_tokens_match" in o:
                other["tp_tokens_match"] = o["tp_tokens_match"]
        except Exception as e:      # the side measurement must not take the headline line down with it
            other.update({"value": None, "error": f"{type(e).__name__}: {e}"})

    if rank == 0:
        roof = cpu = None
        # the dominant kernel: one persistent launch per decode step (256 of the job's launches, ~3/4 of its
        # time); its duration is the CUDA-event time of the decode loop / launches, measured above
        hbm_peak = peaks.get("hbm_gbs") or 6650.0
        step_ms = main_r["t_dec"] / (NEW - 1)
        rows_mode = use_tp and BATCH % world == 0 and os.environ.get("FLEXLLM_TP_MODE", "") != "allgather"
        if not use_tp:
            kname = "decode_mega_kernel (whole decode step, batch 32, context 1024..1279)"
            nbytes, traffic = decode_step_bytes(), DRAM_TRAFFIC_PER_LAUNCH
        elif rows_mode:
            # after the tensor-parallel prefill every rank decodes its own BATCH / N sequences with the full (replicated)
            # weights: one persistent launch per rank and step; bytes, time and peak are ONE GPU's
            kname = f"decode_mega_kernel (one rank's launch: {BATCH // world} of the 32 sequences, replicated weights, context 1024..1279)"
            nbytes = decode_step_bytes(BATCH // world)
            traffic = int(1.358e9 + 0.117e9 + 16 * 1088 * (BATCH // world) * 1019)
        else:
            kname = "decode step (tensor-parallel kernel sequence; bytes of the whole step over all ranks / N)"
            nbytes, traffic = decode_step_bytes() / world, None
        roof = {"bound": "hbm", "kernel": kname, "achieved": round(nbytes / step_ms / 1e6, 1), "peak": hbm_peak, "unit": "GB/s",
                "frac": round(nbytes / step_ms / 1e6 / hbm_peak, 4), "traffic": traffic,
                "algorithmic_bytes_per_launch": int(nbytes), "us_per_launch": round(step_ms * 1e3, 1),
                "peak_source": "measured (MEASURED_PEAKS.json)" if peaks.get("hbm_gbs") else "fallback"}
        units = None
        if not args.no_extras and not multi:      # the operator-level configurations and the CPU baseline belong to the one-GPU line
            roof["standalone_linear"] = kernel_roofline(F, torch, peaks)
            try:
                units = unit_configs(F, torch, peaks)
            except Exception as e:  # the side measurements must not take the headline line down with them
                units = {"error": f"{type(e).__name__}: {e}"}
            try:
                cpu = cpu_port_baseline()
            except Exception as e:  # the CPU figure is a reported baseline only
                cpu = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port", "sample": f"failed: {e}"}
        r = main_r
        e2e = r["units"] * args.steps / (r["ms_e2e"] / 1e3)
        nb = BATCH if use_tp else BATCH * world
        line = {"metric": METRIC, "value": round(r["value"], 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(r["ms_dev"] / args.steps, 3), "higher_is_better": True,
                "scaling": "strong" if use_tp else "weak",
                "vs_baseline": None, "dtype": "s8", "data": "synthetic", "config": workload_config(world, "tp" if use_tp else "dp"),
                "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": BATCH * PREFILL * 4,
                        "d2h_bytes_per_step": BATCH * NEW * 4, "ms_per_step": round(r["ms_e2e"] / args.steps, 3)},
                "gpu_launches": int(r["launches"]), "clocks": r["clocks"], "roofline": roof, "cpu_baseline": cpu,
                "phases": phases(r, nb)}
        if "tp_tokens_match" in r:
            line["tp_tokens_match"] = r["tp_tokens_match"]
        if tp_error is not None:
            line["tensor_parallel_failed"] = tp_error
        if other is not None:
            line["other_partition"] = other
        if units is not None:
            line["unit_configs"] = units
        print(json.dumps(line))
    if tp_comm[0] is not None:
        tp_comm[0].close()
    if multi:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    # profiling aids (the headline workload is the default): shorter decode / skip the side measurements
    ap.add_argument("--parallel", default="tp", choices=["tp", "dp"],
                    help="N > 1: headline partition - tensor parallel over the N GPUs with a fixed total batch of 32 (default: the "
                         "partition the workload names), or independent batch-parallel replicas; the other one is reported under "
                         "other_partition")
    ap.add_argument("--decode-len", type=int, default=NEW)
    ap.add_argument("--no-extras", action="store_true", help="skip roofline kernel timing and the CPU baseline")
    ap.add_argument("--micro", default=None, help="run one kernel on a small case and exit (attn_prefill, attn_prefill_online, gemm_prefill, "
                                                  "gemm_prefill_k8192, decode_linear, gemv_b1, decode_attention, swiglu_fht, rmsnorm_prefill, prefill_small, decode_step)")
    args = ap.parse_args()
    globals()["NEW"] = args.decode_len
    args.warmup = max(args.warmup, 0)
    if args.micro:
        micro(args)
        return
    if args.impl == "reference":
        if env_int("RANK", 0) == 0:
            reference_arm(args)
        return
    if args.warmup < 3:
        args.warmup = 3   # timing rule: at least three warm-up steps
    gpu_arm(args)


if __name__ == "__main__":
    main()
