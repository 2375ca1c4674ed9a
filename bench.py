#!/usr/bin/env python
"""Throughput of the quantized Llama-3.2-1B path on B200: prefill + greedy decode tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config 5): 16 layers, hidden 2048, 32/8 heads, FFN 8192, vocab 128256, tied
embeddings; random-init int8 weights with per-channel scales, synthetic token ids; batch 32,
prefill 1024 tokens, greedy decode of 256 tokens. One "step" = one such request batch.

  value : tokens/s with the prompt ids already on the device (CUDA events on the launching stream)
  e2e   : the same request through flexllm_model_generate_host: prompt ids in pinned HOST memory,
          host->device copy, prefill, decode, device->host copy of the generated ids inside the
          timed region
  N > 1 : one process per GPU, every rank serves its own batch of 32 sequences (batch-parallel
          request streams, no data-path collective): weak scaling; time = max over ranks.

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

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------------------------ CPU arms
def cpu_port_baseline():
    """The plain-C++ oracle (all host threads) on a bounded sample: the full 16-layer model,
    one sequence, 64 prompt tokens + 2 generated."""
    import numpy as np
    import oracle
    from flexllm_b200 import synthetic
    S, n_new = 64, 2
    W = synthetic.numpy_weights(max_ctx=S + n_new, seed=0, **CFG)
    tok = np.random.default_rng(1).integers(0, CFG["vocab"], (1, S)).astype(np.int32)
    t0 = time.perf_counter()
    oracle.model_generate(W, tok, n_new)
    dt = time.perf_counter() - t0
    return {"value": (S + n_new) / dt, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
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
    sample = (f"one decoder layer (all projections, RoPE, FHT, attention, MLP) on one {T}-token block through the "
              f"{'reference templates' if R is not None else 'oracle port'}, {t_layer:.2f} s per layer; x{CFG['layers']} layers, lm_head not included")
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
            "parallelism": (f"tp{world}: column-parallel q/k/v/gate/up, row-parallel o/down + NCCL int32 all-reduce, vocab-parallel lm_head"
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


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_mega_kernel launch: ncu capture at context 131..136
# (1.358 GB read + 0.107 GB written, profiles/decode_mega_kernel_batch32_ctx131.md) plus the KV pages the
# bench's mean context of 1152 adds (16 layers x 1088 B x 32 sequences x 1019 tokens; KV traffic is proportional)
DRAM_TRAFFIC_PER_LAUNCH = int(1.358e9 + 0.107e9 + 16 * 1088 * 32 * 1019)


def decode_step_bytes():
    """Algorithmic bytes one decode step has to read: every int8 weight once (layers + lm_head), the
    scales, and the int8 KV pages of all layers for the step's context lengths (K and V rows of 64
    bytes per KV head plus two fp32 scales per head: 1088 bytes per cached token and layer)."""
    D, F, V, L = CFG["hidden"], CFG["ffn"], CFG["vocab"], CFG["layers"]
    qkv = (CFG["heads_q"] + 2 * CFG["heads_kv"]) * 64
    weights = L * (qkv * D + D * D + 2 * F * D + D * F) + V * D
    scales = 4 * (L * (qkv + D + 2 * F + D + 2 * D) + V + D)
    kv = L * 1088 * BATCH * (PREFILL + NEW / 2)
    return weights + scales + kv


def micro(args):
    """Runs one kernel a few times on a small fixed case (for ncu captures; prints its mean time)."""
    import torch
    import flexllm_b200 as F
    from flexllm_b200 import synthetic
    F.lib()
    name = args.micro
    dev = "cuda"
    if name == "attn_prefill":          # BASELINE config 3: B=4, S=1024, 32/8 heads
        B, S, HQ, HKV = 4, 1024, 32, 8
        g = torch.Generator(device=dev).manual_seed(0)
        r8 = lambda *sh: torch.randint(-127, 128, sh, dtype=torch.int8, device=dev, generator=g)
        rs = lambda *sh: torch.rand(sh, device=dev, generator=g) * 0.045 + 0.005
        q, k, v, qs, ks, vs = r8(B, S, HQ, 64), r8(B, S, HKV, 64), r8(B, S, HKV, 64), rs(B, S, HQ), rs(B, S, HKV), rs(B, S, HKV)
        c, s_ = synthetic.rope_table(S); c = torch.from_numpy(c).to(dev); s_ = torch.from_numpy(s_).to(dev)
        a_s = torch.full((HQ,), 0.05 / 255, device=dev)
        fn = lambda: F.MHA_i8xi8_Prefilling(q, qs, k, ks, v, vs, c, s_, a_s)
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
    elif name == "swiglu_fht":
        gg = torch.randn((4096, 8192), device=dev); uu = torch.randn((4096, 8192), device=dev)
        fn = lambda: F.swiglu_fht_quant(gg, uu)
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
            barrier()
            sampler = ClockSampler(local); sampler.start()
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
        m.close()
        del m
        torch.cuda.empty_cache()
        return r

    def phases(r, nb):
        dec_bytes = decode_step_bytes()
        return {"prefill_ms": round(r["t_pre"], 3), "prefill_tokens_per_s": round(nb * PREFILL / r["t_pre"] * 1e3, 1),
                "prefill_tops": round(6.60e13 * nb / BATCH / r["t_pre"] / 1e9, 1),
                "decode_ms_per_step": round(r["t_dec"] / (NEW - 1), 4),
                "decode_tokens_per_s": round(nb * (NEW - 1) / r["t_dec"] * 1e3, 1),
                "decode_hbm_frac_of_measured": round(dec_bytes / (r["t_dec"] / (NEW - 1) / 1e3) / 1e9 / (peaks.get("hbm_gbs") or 6650.0), 4)}

    # N > 1: the headline partition is --parallel (replicas by default: for a 1.2 GB model every
    # collective only adds latency, so independent batch-parallel replicas are the faster use of N
    # GPUs); the other partition is measured in the same run and reported beside it
    use_tp = multi and args.parallel == "tp"
    main_r = measure(use_tp, args.steps)
    other = None
    if multi and not args.no_extras:
        other = {"parallelism": workload_config(world, "dp" if use_tp else "tp")["parallelism"],
                 "scaling": "weak" if use_tp else "strong"}
        try:
            o = measure(not use_tp, min(args.steps, 2), with_e2e=False)
            nb_o = BATCH if not use_tp else BATCH * world
            other.update({"value": round(o["value"], 1), "unit": "tokens/s",
                          "ms_per_step": round(o["ms_dev"] / min(args.steps, 2), 3), "phases": phases(o, nb_o)})
        except Exception as e:      # the side measurement must not take the headline line down with it
            other.update({"value": None, "error": f"{type(e).__name__}: {e}"})

    if rank == 0:
        roof = cpu = None
        # the dominant kernel: one persistent launch per decode step (256 of the job's launches, ~3/4 of its
        # time); its duration is the CUDA-event time of the decode loop / launches, measured above
        hbm_peak = peaks.get("hbm_gbs") or 6650.0
        step_ms = main_r["t_dec"] / (NEW - 1)
        nbytes = decode_step_bytes()
        roof = {"bound": "hbm", "kernel": "decode_mega_kernel (whole decode step, batch 32, context 1024..1279)" if not use_tp
                else "decode step (tensor-parallel kernel sequence)", "achieved": round(nbytes / step_ms / 1e6, 1), "peak": hbm_peak, "unit": "GB/s",
                "frac": round(nbytes / step_ms / 1e6 / hbm_peak, 4), "traffic": DRAM_TRAFFIC_PER_LAUNCH,
                "algorithmic_bytes_per_launch": int(nbytes), "us_per_launch": round(step_ms * 1e3, 1),
                "peak_source": "measured (MEASURED_PEAKS.json)" if peaks.get("hbm_gbs") else "fallback"}
        if not args.no_extras:
            roof["standalone_linear"] = kernel_roofline(F, torch, peaks)
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
                "vs_baseline": None, "dtype": "s8", "data": "synthetic", "config": workload_config(world, args.parallel),
                "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": BATCH * PREFILL * 4,
                        "d2h_bytes_per_step": BATCH * NEW * 4, "ms_per_step": round(r["ms_e2e"] / args.steps, 3)},
                "gpu_launches": int(r["launches"]), "clocks": r["clocks"], "roofline": roof, "cpu_baseline": cpu,
                "phases": phases(r, nb)}
        if other is not None:
            line["other_partition"] = other
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
    ap.add_argument("--parallel", default="dp", choices=["tp", "dp"],
                    help="N > 1: headline partition - independent batch-parallel replicas (default) or tensor parallel over "
                         "the N GPUs with a fixed total batch; the other one is reported under other_partition")
    ap.add_argument("--decode-len", type=int, default=NEW)
    ap.add_argument("--no-extras", action="store_true", help="skip roofline kernel timing and the CPU baseline")
    ap.add_argument("--micro", default=None, help="run one kernel on a small case and exit (attn_prefill, gemm_prefill, "
                                                  "gemm_prefill_k8192, decode_linear, swiglu_fht, decode_step)")
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
