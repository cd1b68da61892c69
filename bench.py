#!/usr/bin/env python
"""Benchmark of the packed-ternary Linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[4], the largest one that fits a single GPU): the
ternary Linear layers of a Llama-3-8B-shaped decoder stack — 32 layers, each with
q/o 4096->4096, k/v 4096->1024, gate/up 4096->14336, down 14336->4096 — random
N(0, 0.02^2) weights quantised with the absmean rule (threshold 0.45) and packed
on the device; batch 8, a 2048-token prefill (16384 tokens through every Linear,
the tcgen05 kernel) followed by 128 decode steps (8 tokens, the streaming kernel).
Attention, norms and embeddings are not part of the path and are not run: every
Linear reads a resident synthetic bf16 activation buffer of its input width.
One "step" is that whole job; the metric is tokens/s = (8*2048 + 8*128) / step time.

With N > 1 (launched by torch.distributed.run) the job is the same size at every N
(strong scaling): in the prefill the output features of every Linear are sharded
across the ranks and one NCCL all-gather per Linear assembles the result; the
8-token decode calls are shorter than an all-gather, so every rank runs them whole.

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import contextlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYERS = 32
HIDDEN, KV, FFN = 4096, 1024, 14336
# (name, out_features, in_features)
LINEARS = [("q", HIDDEN, HIDDEN), ("k", KV, HIDDEN), ("v", KV, HIDDEN), ("o", HIDDEN, HIDDEN),
           ("gate", FFN, HIDDEN), ("up", FFN, HIDDEN), ("down", HIDDEN, FFN)]
INDEPENDENT = ("k", "v", "up")  # Linears of a decoder block that read what their predecessor reads
BATCH, PREFILL, DECODE = 8, 2048, 128
THRESHOLD = 0.45
WORKLOAD = ("llama3-8b-shaped ternary Linear stack: 32 layers x (q,o 4096x4096; k,v 1024x4096; gate,up 14336x4096; "
            "down 4096x14336), batch 8, 2048-token prefill + 128 decode steps, bf16 activations, absmean/0.45")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([f.strip() for f in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0])); mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------ reference arm


def run_reference(args):
    """The reference's own CPU implementation of the path, on the host cores of this box.

    The reference's Linear forward multiplies packed limbs by packed limbs
    (t81/torch/__init__.py:257-276 -> src/linalg/gemm_cpu.cpp:8-71): activations are
    thresholded to trits, column-packed, and gemm_ternary runs over limb values on one
    thread (the reference has no threading).  A bounded sample is timed through the
    compiled reference module (oracle/_ref) and scaled to the whole stack by limb products."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import oracle
    from oracle import ref as oracle_ref

    rng = np.random.default_rng(0)
    out_f, in_f, tokens = 256, HIDDEN, BATCH  # a 256-row slice of one 4096-wide Linear, one decode step's tokens
    w = rng.normal(0, 0.02, (out_f, in_f)).astype(np.float32)
    packed, _ = oracle.pack_dense_matrix_absmean(w, THRESHOLD)
    x = rng.normal(size=(in_f, tokens)).astype(np.float32)
    kl = packed.shape[1]
    xp = oracle.pack_trits_columnwise(oracle.quantize_to_trits(x, 0.5))
    products_sample = out_f * kl * tokens
    if oracle_ref.available():
        t81lib = oracle_ref.load()
        a = packed.reshape(-1, 16).view("V16").reshape(out_f, kl)
        b = xp.reshape(-1, 16).view("V16").reshape(kl, tokens)

        def once():
            c = np.zeros((out_f, tokens), np.float32)
            t81lib.gemm_ternary(a, b, c, out_f, tokens, kl * 48)
        kind, how = "reference", f"oracle/_ref ({oracle_ref.variant()} build) t81lib.gemm_ternary"
    else:
        def once():
            oracle.gemm_limb(packed, xp, np.zeros((out_f, tokens), np.float32), out_f, tokens, kl * 48)
        kind, how = "port", "oracle t81o_gemm_limb (oracle/_ref not present)"
    for _ in range(max(1, min(args.warmup, 1))):
        once()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter(); once(); times.append(time.perf_counter() - t0)
    per_product = statistics.mean(times) / products_sample
    weights_per_token_limbs = LAYERS * sum(o * ((i + 47) // 48) for _, o, i in LINEARS)
    job_tokens = BATCH * (PREFILL + DECODE)
    job_seconds = per_product * weights_per_token_limbs * job_tokens
    value = job_tokens / job_seconds
    sample = (f"{how}: {out_f}x{in_f} Linear slice x {tokens} tokens ({products_sample} limb products, "
              f"{statistics.mean(times):.2f} s per sample), scaled to the stack by limb products")
    line = {
        "impl": "reference", "metric": "t8.nn.Linear tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": job_seconds * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD, "semantics": "reference LIMB mode (activations thresholded to trits)"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": 1, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ our arm


def cpu_baseline(threads: int):
    """The CPU oracle (port of the TRIT-mode Linear) on a bounded sample, all host cores."""
    import numpy as np
    import oracle
    rng = np.random.default_rng(0)
    out_f, in_f, tokens = HIDDEN, HIDDEN, BATCH
    w = rng.normal(0, 0.02, (out_f, in_f)).astype(np.float32)
    packed, scale = oracle.pack_dense_matrix_absmean(w, THRESHOLD)
    x = rng.normal(size=(tokens, in_f)).astype(np.float32)
    oracle.set_num_threads(threads)
    oracle.linear_forward(packed, scale, None, x, in_f)
    reps, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < 10.0 and reps < 200:
        oracle.linear_forward(packed, scale, None, x, in_f)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    oracle.set_num_threads(1)
    weights_per_token = LAYERS * sum(o * i for _, o, i in LINEARS)
    job_tokens = BATCH * (PREFILL + DECODE)
    job_seconds = dt / (out_f * in_f * tokens) * weights_per_token * job_tokens
    return {"value": job_tokens / job_seconds, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"oracle linear_forward 4096x4096 x 8 tokens, {reps} repetitions, {dt*1e3:.1f} ms each, "
                      f"scaled to the stack by weight count"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    from t81lib_b200 import _capi, ops
    from t81lib_b200.nn import Linear
    from t81lib_b200.nn.sharded import PeerColumns, shard_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert _capi.device_available(), _capi.last_error()
    pk = peaks()

    # ---- build the stack: quantise + pack on the device, this rank's rows only
    gen = torch.Generator(device=dev).manual_seed(1234)
    layers = []
    for _ in range(LAYERS):
        mods = []
        for name, out_f, in_f in LINEARS:
            w = torch.randn(out_f, in_f, generator=gen, device=dev) * 0.02  # same on every rank
            # every rank packs the whole matrix and uses its own row slice of it (row-wise packing makes
            # the slice a contiguous view, byte for byte what packing the slice alone would give)
            packed, scale = ops.quantize_pack(w, THRESHOLD, "absmean")
            mods.append((name, out_f, in_f, packed, scale))
            del w
        layers.append(mods)
    torch.cuda.synchronize()

    ptok, dtok = BATCH * PREFILL, BATCH
    gin = torch.Generator(device=dev).manual_seed(99)
    x_in = {HIDDEN: torch.randn(ptok, HIDDEN, generator=gin, device=dev).to(torch.bfloat16),
            FFN: torch.randn(ptok, FFN, generator=gin, device=dev).to(torch.bfloat16)}
    xd_in = {HIDDEN: x_in[HIDDEN][:dtok].contiguous(), FFN: x_in[FFN][:dtok].contiguous()}
    out_widths = sorted({o for _, o, _ in LINEARS})
    y_loc = {o: torch.empty(ptok, o // world, dtype=torch.bfloat16, device=dev) for o in out_widths}
    yd_out = {name: torch.empty(dtok, o, dtype=torch.bfloat16, device=dev) for name, o, _ in LINEARS}  # one per Linear of a block
    # N > 1: full-width results of every rank, mapped into every process (copy-engine all-gather)
    y_peer = {o: PeerColumns(ptok, o, torch.bfloat16, dev) for o in out_widths} if world > 1 else None

    def shard(mod):
        name, out_f, in_f, packed, scale = mod
        lo, hi = shard_bounds(out_f, world, rank)
        return name, hi - lo, in_f, packed[lo:hi], scale[lo:hi]

    prefill_mods = [[shard(m) for m in mods] for mods in layers]

    # Prefill with N > 1: every GEMM computes this rank's output features and writes them into their
    # columns of its own full-width result AND of every peer's (TMA stores over NVLink from the kernel's
    # epilogue); flag words written behind the data order the exchange (each call waits for the peers'
    # stores of the previous call and signals its own; no collective, no host involvement).  One explicit
    # wait closes the phase.  Two result buffers per width are used in turn.

    def sharded_pass(x_by_width, bufs):
        for mods in prefill_mods:
            for name, out_l, in_f, packed, scale in mods:
                ex = bufs[out_l * world]
                idx = ex.next_index()
                lo, hi = rank * out_l, (rank + 1) * out_l
                ops.gemm_trit(packed, x_by_width[in_f], M=out_l, K=in_f, layout="nk", row_scale=scale,
                              C=ex.buffers[idx][:, lo:hi], peers=ex.peer_blocks(idx, lo, hi), sync=ex.flags)

    def prefill():
        if world == 1:
            for mods in layers:
                for name, out_f, in_f, packed, scale in mods:
                    ops.gemm_trit(packed, x_in[in_f], M=out_f, K=in_f, layout="nk", row_scale=scale, C=y_loc[out_f])
            return
        sharded_pass(x_in, y_peer)
        y_peer[HIDDEN].flags.wait()

    def decode_step():
        # decode runs whole on every rank at any N: the exchange adds ~8 us to a 5 us kernel (one system
        # fence, one flag flight over NVLink, one poll), more than the rows a rank would save
        # k, v read what q reads and up reads what gate reads: they need not wait for that predecessor
        # (the decoder block's own data flow; every other Linear runs behind the one before it)
        for mods in layers:
            for name, out_f, in_f, packed, scale in mods:
                with ops.independent_of_previous() if name in INDEPENDENT else contextlib.nullcontext():
                    ops.gemm_trit(packed, xd_in[in_f], M=out_f, K=in_f, layout="nk", row_scale=scale, C=yd_out[name])

    # the decode step is launch-bound: capture it once in a CUDA graph
    stream = torch.cuda.Stream(device=dev)
    graph = None
    with torch.cuda.stream(stream):
        decode_step()
        torch.cuda.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                decode_step()
            graph = g
        except Exception:
            graph = None
            torch.cuda.synchronize()
    torch.cuda.synchronize()

    def decode_all():
        for _ in range(DECODE):
            if graph is not None:
                graph.replay()
            else:
                decode_step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            prefill(); decode_all()
        barrier()
        step_ms, prefill_ms, decode_ms = [], [], []
        with ClockSampler(local_rank) as clocks:
            t_all0, t_all1 = ev(), ev()
            t_all0.record(stream)
            marks = []
            for _ in range(args.steps):
                a, b, c = ev(), ev(), ev()
                a.record(stream); prefill(); b.record(stream); decode_all(); c.record(stream)
                marks.append((a, b, c))
            t_all1.record(stream)
            barrier()
        total_ms = t_all0.elapsed_time(t_all1)
        for a, b, c in marks:
            prefill_ms.append(a.elapsed_time(b)); decode_ms.append(b.elapsed_time(c)); step_ms.append(a.elapsed_time(c))
    assert _capi.kernel_status(reset=True) == 0, "tensor-core kernel reported a timed-out wait"

    ms_per_step = total_ms / args.steps
    if world > 1:
        t = torch.tensor([ms_per_step, statistics.mean(prefill_ms), statistics.mean(decode_ms)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step, pre_ms, dec_ms = t.tolist()
    else:
        pre_ms, dec_ms = statistics.mean(prefill_ms), statistics.mean(decode_ms)
    job_tokens = BATCH * (PREFILL + DECODE)
    value = job_tokens / (ms_per_step * 1e-3)

    # ---- roofline of the dominant kernel (tcgen05 GEMM, prefill): algorithmic flops / time
    flops_prefill = 2.0 * ptok * LAYERS * sum(o * i for _, o, i in LINEARS) / world  # this rank's share
    tf = flops_prefill / (pre_ms * 1e-3) / 1e12
    roof = {"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
            "frac": tf / pk["bf16_tflops_sustained"], "traffic": None, "peak_source": pk["source"] + " (sustained bf16)",
            "kernel": "gemm_trit_tc_kernel", "note": "prefill phase: 224 launches per step, includes launch gaps"
                      + ("; includes the exchange" if world > 1 else "")}
    # decode: algorithmic bytes of the streaming kernel
    packed_bytes = sum(m[3].numel() for mods in layers for m in mods)  # decode runs whole on every rank
    bytes_decode = packed_bytes + sum(4 * m[1] + 2 * dtok * m[2] + 2 * dtok * m[1] for mods in layers for m in mods)
    gbs = bytes_decode * DECODE / (dec_ms * 1e-3) / 1e9
    gemv = {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
            "kernel": "gemv_trit_tma_kernel", "tokens": dtok, "cuda_graph": graph is not None,
            "note": "decode phase: 224 launches per step, includes launch gaps" + ("; whole on every rank" if world > 1 else "")}

    launches = args.steps * (1 + DECODE) * LAYERS * len(LINEARS)
    line = {
        "metric": "t8.nn.Linear tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": (f"prefill: output features of every Linear sharded x{world}, the GEMM epilogue also stores its output block into every peer's "
                                   f"result over NVLink, flag words order the exchange (no collective); decode: whole on every rank (the exchange "
                                   f"costs more than the rows saved)") if world > 1 else "single GPU",
                   "l2": "inputs larger than L2: 2.3 GB of packed weights and a 134 MB activation buffer are streamed each step",
                   "prefill_ms": pre_ms, "decode_ms": dec_ms, "prefill_tokens_per_s": ptok / (pre_ms * 1e-3),
                   "decode_tokens_per_s": dtok * DECODE / (dec_ms * 1e-3)},
        "roofline": roof, "gemv_roofline": gemv, "gpu_launches": launches,
    }

    if rank == 0:
        line["clocks"] = clocks.summary()

    # ---- end to end through the public API (t81lib_b200.nn.Linear), host buffers in and out
    if world == 1:
        line["e2e"] = e2e_public_api(torch, dev, Linear, layers, args)
        line["quantize_pack"] = quantize_pack_line(torch, dev, ops, pk)
        line["cpu_baseline"] = cpu_baseline(os.cpu_count() or 1)
    else:
        try:
            line["e2e"] = e2e_public_api(torch, dev, Linear, layers, args, world, rank)
        except Exception as exc:  # the device-resident figures above stand on their own
            line["e2e"] = {"value": None, "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                           "note": f"end-to-end pass failed: {type(exc).__name__}: {exc}"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # leave without tearing the process group down: with NCCL work captured in a CUDA graph the
        # teardown has been seen to wait forever; every rank has finished its work at this point
        graph = None
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def e2e_public_api(torch, dev, Linear, layers, args, world=1, rank=0):
    """Same job through nn.Module calls: pinned host activations are copied in for the
    prefill and for every decode step, the last Linear's output is copied back."""
    import t81lib_b200.torch as t81_torch
    from t81lib_b200 import ops
    mods = []
    for layer in layers:
        row = []
        for name, out_f, in_f, packed, scale in layer:
            m = Linear(in_f, out_f, bias=False, device="meta", threshold=THRESHOLD, rule="absmean")
            m.eval()
            m.ternary_weight = t81_torch.TernaryTensor(packed, (out_f, in_f), k_actual=in_f, k_limbs=packed.shape[1],
                                                       threshold=THRESHOLD, row_scale=scale, rule="absmean")
            row.append(m)
        mods.append(row)
    # N > 1: the prefill goes through ShardedLinear(exchange="p2p") modules over this rank's rows of the same
    # packed weights (waits deferred to the next call, one explicit wait before the result is read); the
    # decode pass uses the whole-matrix modules above on every rank.
    sharded = None
    if world > 1:
        from t81lib_b200.nn.sharded import ShardedLinear, shard_bounds
        sharded = []
        for layer in layers:
            row = []
            for name, out_f, in_f, packed, scale in layer:
                lo, hi = shard_bounds(out_f, world, rank)
                tt = t81_torch.TernaryTensor(packed[lo:hi], (hi - lo, in_f), k_actual=in_f, k_limbs=packed.shape[1],
                                             threshold=THRESHOLD, row_scale=scale[lo:hi], rule="absmean")
                m = ShardedLinear(torch.empty((out_f, in_f), device="meta"), None, threshold=THRESHOLD, rule="absmean",
                                  exchange="p2p", quantize=lambda w, t, r, tt=tt: tt,
                                  matmul=lambda x, b, tt=tt: tt.matmul_input(x, bias=b))
                m.defer_wait = True
                row.append(m)
            sharded.append(row)
    ptok, dtok = BATCH * PREFILL, BATCH
    host_p = {w: torch.randn(ptok, w).to(torch.bfloat16).pin_memory() for w in (HIDDEN, FFN)}
    host_d = {w: torch.randn(dtok, w).to(torch.bfloat16).pin_memory() for w in (HIDDEN, FFN)}
    out_p = torch.empty(ptok, HIDDEN, dtype=torch.bfloat16).pin_memory()
    out_d = torch.empty(dtok, HIDDEN, dtype=torch.bfloat16).pin_memory()

    def run_modules(x):
        y = None
        with torch.no_grad():
            for row in mods:
                keep = []  # a block's outputs stay alive together, so k/v (up) never reuse q's (gate's) memory
                for (name, out_f, in_f), m in zip(LINEARS, row):
                    with ops.independent_of_previous() if name in INDEPENDENT else contextlib.nullcontext():
                        y = m(x[in_f])
                    keep.append(y)
        return y

    def forward(host, out_host):
        x = {w: host[w].to(dev, non_blocking=True) for w in host}
        if sharded is None:
            out_host.copy_(run_modules(x), non_blocking=True)
            return
        y = None
        with torch.no_grad():
            for row in sharded:
                for (name, out_f, in_f), m in zip(LINEARS, row):
                    y = m(x[in_f])
        sharded[-1][-1].exchange_for(y.shape[0], y.dtype, dev).flags.wait()  # the peers' blocks of the last result
        out_host.copy_(y, non_blocking=True)

    # The decode pass (224 module calls on 8 tokens) is captured once in a CUDA graph, the way an
    # inference server drives nn.Modules: every step still copies its inputs in from pinned host
    # memory and its result back out.
    x_static = {w: torch.zeros(dtok, w, dtype=torch.bfloat16, device=dev) for w in (HIDDEN, FFN)}
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        run_modules(x_static)
        torch.cuda.synchronize()
        dgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(dgraph, stream=stream):
            y_static = run_modules(x_static)
    torch.cuda.synchronize()

    def decode_forward():
        for w in x_static:
            x_static[w].copy_(host_d[w], non_blocking=True)
        dgraph.replay()
        out_d.copy_(y_static, non_blocking=True)

    def job():
        forward(host_p, out_p)
        for _ in range(DECODE):
            decode_forward()

    steps = max(1, min(args.steps, 3))
    job()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        job()
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) * 1e-3 / steps
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([sec], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = t.item()
    h2d = 2 * (ptok + DECODE * dtok) * (HIDDEN + FFN)
    d2h = 2 * (ptok + DECODE * dtok) * HIDDEN
    return {"value": BATCH * (PREFILL + DECODE) / sec, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "steps": steps, "api": ("t81lib_b200.nn.Linear.forward" if world == 1 else "t81lib_b200.nn.sharded.ShardedLinear.forward (prefill, exchange='p2p') + t81lib_b200.nn.Linear.forward (decode)")
                   + " (prefill eager; decode pass replayed from a torch.cuda.CUDAGraph); host copies on every rank"}


def quantize_pack_line(torch, dev, ops, pk):
    """BASELINE config 2: 4096x4096 fp32 N(0, 0.02^2), absmean rule, threshold 0.45."""
    ws = [torch.randn(4096, 4096, device=dev) * 0.02 for _ in range(8)]  # 512 MB: rotates past L2
    outs = [ops.quantize_pack(w, THRESHOLD, "absmean") for w in ws]
    torch.cuda.synchronize()
    # one CUDA graph over the 8 matrices: the kernel is shorter than a Python-side launch
    graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for w, (p, s) in zip(ws, outs):
                ops.quantize_pack(w, THRESHOLD, "absmean", out=p, row_scale_out=s)
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) * 1e-3 / (reps * len(ws))
    alg = 4096 * 4096 * 4 + 4096 * 86 * 16 + 4096 * 4
    return {"bound": "hbm", "achieved": alg / sec / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": alg / sec / 1e9 / pk["hbm_gbs"], "us_per_launch": sec * 1e6, "kernel": "quantize_pack_row_kernel"}


def run_kernel_case(args):
    """One kernel alone on a small fixed case whose operands are larger than L2 (a few hundred MB):
    the command the ncu captures under profiles/ are taken with, and a quick per-kernel figure.
      gemv     : 14336 x 4096 (gate/up), 8 bf16 tokens, 16 distinct weight matrices, 2 passes
      gemm     : 4096 x 4096, 16384 bf16 tokens, 3 launches
      quantize : 4096 x 4096 fp32, absmean/0.45, 8 distinct matrices, 2 passes"""
    import torch
    from t81lib_b200 import _capi, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    assert _capi.device_available(), _capi.last_error()
    pk = peaks()
    gen = torch.Generator(device=dev).manual_seed(7)
    if args.kernel == "gemv":
        rows, k, tok = FFN, HIDDEN, BATCH
        kl = (k + 47) // 48
        mats = [torch.randint(0, 27, (rows, kl, 16), dtype=torch.uint8, device=dev, generator=gen) for _ in range(16)]
        scale = torch.rand(rows, device=dev, generator=gen)
        x = torch.randn(tok, k, device=dev, generator=gen).to(torch.bfloat16)
        y = torch.empty(tok, rows, dtype=torch.bfloat16, device=dev)
        calls = [lambda m=m: ops.gemm_trit(m, x, M=rows, K=k, layout="nk", row_scale=scale, C=y) for m in mats] * 2
        alg, unit, peak, name = rows * kl * 16 + 4 * rows + 2 * tok * k + 2 * tok * rows, "GB/s", pk["hbm_gbs"], "gemv_trit_tma_kernel"
    elif args.kernel == "gemm":
        rows, k, tok = HIDDEN, HIDDEN, BATCH * PREFILL
        kl = (k + 47) // 48
        m = torch.randint(0, 27, (rows, kl, 16), dtype=torch.uint8, device=dev, generator=gen)
        scale = torch.rand(rows, device=dev, generator=gen)
        x = torch.randn(tok, k, device=dev, generator=gen).to(torch.bfloat16)
        y = torch.empty(tok, rows, dtype=torch.bfloat16, device=dev)
        calls = [lambda: ops.gemm_trit(m, x, M=rows, K=k, layout="nk", row_scale=scale, C=y)] * 3
        alg, unit, peak, name = 2.0 * rows * k * tok, "TFLOP/s", pk["bf16_tflops"], "gemm_trit_tc_kernel"
    else:
        ws = [torch.randn(4096, 4096, device=dev, generator=gen) * 0.02 for _ in range(8)]
        outs = [ops.quantize_pack(w, THRESHOLD, "absmean") for w in ws]
        calls = [lambda w=w, o=o: ops.quantize_pack(w, THRESHOLD, "absmean", out=o[0], row_scale_out=o[1]) for w, o in zip(ws, outs)] * 2
        alg, unit, peak, name = 4096 * 4096 * 4 + 4096 * 86 * 16 + 4096 * 4, "GB/s", pk["hbm_gbs"], "quantize_pack_row_kernel"
    calls[0]()
    torch.cuda.synchronize()
    graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):  # the kernels are shorter than a Python-side launch
            for c in calls:
                c()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) * 1e-3 / len(calls)
    assert _capi.kernel_status(reset=True) == 0
    achieved = alg / sec / (1e12 if unit == "TFLOP/s" else 1e9)
    print(json.dumps({"kernel": name, "case": args.kernel, "launches": len(calls), "us_per_launch": sec * 1e6,
                      "achieved": achieved, "unit": unit, "peak": peak, "frac": achieved / peak,
                      "peak_source": pk["source"] + (" (burst bf16)" if unit == "TFLOP/s" else "")}), flush=True)


def run_sweep(args):
    """BASELINE configs 3 and 4: the ternary Linear layers of a Phi-3-mini-shaped block, decode-sized calls with
    1, 4 and 16 tokens (GB/s of algorithmic bytes against the HBM peak) and a 2048-token prefill with an fp32
    bias (TFLOP/s against the bf16 tensor peak).  One JSON line per shape and token count; every figure is a
    CUDA-graph replay over enough distinct weight matrices to exceed L2."""
    import torch
    from t81lib_b200 import _capi, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    assert _capi.device_available(), _capi.last_error()
    pk = peaks()
    gen = torch.Generator(device=dev).manual_seed(11)
    shapes = [("qkv", 9216, 3072), ("o", 3072, 3072), ("gate_up", 16384, 3072), ("down", 3072, 8192)]
    stream = torch.cuda.Stream(device=dev)
    for name, rows, k in shapes:
        kl = (k + 47) // 48
        nbytes = rows * kl * 16
        copies = max(2, int(400e6 // nbytes))
        ws = [torch.randn(rows, k, device=dev, generator=gen) * 0.02 for _ in range(2)]
        mats = [ops.quantize_pack(ws[i % 2], THRESHOLD, "absmean") for i in range(copies)]
        bias = torch.randn(rows, device=dev, generator=gen) * 0.01
        for tok in (1, 4, 16, 2048):
            x = torch.randn(tok, k, device=dev, generator=gen).to(torch.bfloat16)
            y = torch.empty(tok, rows, dtype=torch.bfloat16, device=dev)
            n = copies if tok <= 16 else 4
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                ops.gemm_trit(mats[0][0], x, M=rows, K=k, layout="nk", row_scale=mats[0][1], bias=bias, C=y)
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=stream):
                    for i in range(n):
                        m, sc = mats[i % copies]
                        ops.gemm_trit(m, x, M=rows, K=k, layout="nk", row_scale=sc, bias=bias, C=y)
                graph.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(3):
                    graph.replay()
                e1.record(stream)
                torch.cuda.synchronize()
            sec = e0.elapsed_time(e1) * 1e-3 / (3 * n)
            if tok <= 16:
                alg = nbytes + 8 * rows + 2 * tok * k + 2 * tok * rows
                line = {"achieved": alg / sec / 1e9, "unit": "GB/s", "peak": pk["hbm_gbs"], "bound": "hbm"}
            else:
                line = {"achieved": 2.0 * rows * k * tok / sec / 1e12, "unit": "TFLOP/s", "peak": pk["bf16_tflops"], "bound": "tensor"}
            line.update({"layer": name, "rows": rows, "k": k, "tokens": tok, "us_per_launch": sec * 1e6,
                         "frac": line["achieved"] / line["peak"]})
            print(json.dumps(line), flush=True)
        del mats, ws
    assert _capi.kernel_status(reset=True) == 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", choices=["gemv", "gemm", "quantize", "sweep"], default=None,
                    help="time one kernel alone on a small case instead of the whole job (used for ncu captures)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.kernel == "sweep":
        run_sweep(args)
    elif args.kernel:
        run_kernel_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
