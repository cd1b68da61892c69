#!/usr/bin/env python
"""Benchmark of the packed-ternary Linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the largest configuration that fits a single GPU): the ternary Linear layers of a
Llama-3-8B-shaped decoder stack — 32 layers, each with q/o 4096->4096, k/v 4096->1024,
gate/up 4096->14336, down 14336->4096 — random N(0, 0.02^2) weights quantised with the
absmean rule (threshold 0.45) and packed on the device; batch 8, a 2048-token prefill
(16384 tokens through every Linear, the tcgen05 kernel) followed by 128 decode steps
(8 tokens, the streaming kernel).  Attention, norms and embeddings are not part of the path
and are not run: every Linear reads a resident synthetic bf16 activation buffer of its input
width.  One "step" is that whole job; the metric is tokens/s = (8*2048 + 8*128) / step time.

With N > 1 (launched by torch.distributed.run) the job is the same size at every N (strong
scaling): in the prefill the output features of every Linear are sharded across the ranks and
the GEMM's epilogue stores its column block into every peer's result over NVLink, ordered by
flag words (no collective); the 8-token decode calls run whole on every rank.  After the timed
region every rank checks one sharded layer against the unsharded one (``parity_ok``).

At N = 1 the line also carries the smaller configurations as sub-objects of ``configs``
(gemm_ternary 512x512x256 in both semantics with the compiled reference timed beside it, the
Phi-3-mini-shaped decode sweep, the 2048-token prefill shapes) and the decode phase re-timed
with the Linears that share an input grouped into one launch.

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


NOMINAL_HBM_GBS, NOMINAL_BF16_TFLOPS = 8000.0, 2250.0  # data-sheet figures, reported beside the measured peaks


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


def _reference_sample(seed: int, steps: int, warmup: int):
    """One host process of the reference arm: ``steps`` timed gemm_ternary calls of the compiled reference on
    its own 256-row slice.  Returns (seconds, limb products, kind, how)."""
    import numpy as np
    import oracle
    from oracle import ref as oracle_ref

    rng = np.random.default_rng(seed)
    out_f, in_f, tokens = 256, HIDDEN, BATCH  # a 256-row slice of one 4096-wide Linear, one decode step's tokens
    w = rng.normal(0, 0.02, (out_f, in_f)).astype(np.float32)
    packed, _ = oracle.pack_dense_matrix_absmean(w, THRESHOLD)
    x = rng.normal(size=(in_f, tokens)).astype(np.float32)
    kl = packed.shape[1]
    xp = oracle.pack_trits_columnwise(oracle.quantize_to_trits(x, 0.5))
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
    for _ in range(max(1, min(warmup, 1))):
        once()
    t0 = time.perf_counter()
    for _ in range(steps):
        once()
    return time.perf_counter() - t0, steps * out_f * kl * tokens, kind, how


def run_reference(args):
    """The reference's own CPU implementation of the path, on the host cores of this box.

    The reference's Linear forward multiplies packed limbs by packed limbs
    (t81/torch/__init__.py:257-276 -> src/linalg/gemm_cpu.cpp:8-71): activations are
    thresholded to trits, column-packed, and gemm_ternary runs over limb values.  The reference
    has no threading, so every host core runs its own process on its own 256-row slice of a
    4096-wide Linear at the same time (output rows are independent); each timed step is one such
    slice per core, and the rate in limb products per second is scaled to the whole stack."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from concurrent.futures import ProcessPoolExecutor
    cores = max(1, min(os.cpu_count() or 1, 64))
    t0 = time.perf_counter()
    with ProcessPoolExecutor(max_workers=cores) as pool:
        results = list(pool.map(_reference_sample, range(cores), [args.steps] * cores, [args.warmup] * cores))
    wall = time.perf_counter() - t0
    busy = max(r[0] for r in results)          # the slowest worker bounds the rate
    products = sum(r[1] for r in results)
    kind, how = results[0][2], results[0][3]
    per_product = busy / products
    weights_per_token_limbs = LAYERS * sum(o * ((i + 47) // 48) for _, o, i in LINEARS)
    job_tokens = BATCH * (PREFILL + DECODE)
    job_seconds = per_product * weights_per_token_limbs * job_tokens
    value = job_tokens / job_seconds
    sample = (f"{how}: per step every one of {cores} host processes multiplies a 256x{HIDDEN} Linear slice by {BATCH} tokens "
              f"({products // args.steps} limb products per step, {busy / args.steps:.2f} s per step, {wall:.1f} s in all); "
              f"the rate is scaled to the stack by limb products — the whole job would take {job_seconds / 86400:.1f} days here")
    line = {
        "impl": "reference", "metric": "t8.nn.Linear tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": job_seconds * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD, "semantics": "reference LIMB mode (activations thresholded to trits)",
                   "extrapolated": True},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
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
        # the collectives here are barriers, small reductions and one broadcast: nothing in-switch reduction would
        # speed up, so NCCL is kept on plain peer transfers (no multicast objects bound to these processes' memory)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
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
    # decode-sized products read the decode-stream layout (made once per weight, like the packing itself)
    use_t2 = args.decode_layout == "t2"
    t2 = [{m[0]: ops.pack_t2(m[3], m[1], m[2]) for m in mods} for mods in layers] if use_t2 else None

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
        for li, mods in enumerate(layers):
            for name, out_f, in_f, packed, scale in mods:
                with ops.independent_of_previous() if name in INDEPENDENT else contextlib.nullcontext():
                    if use_t2:
                        ops.gemm_trit_t2([t2[li][name]], [out_f], xd_in[in_f], K=in_f, row_scales=[scale], outs=[yd_out[name]])
                    else:
                        ops.gemm_trit(packed, xd_in[in_f], M=out_f, K=in_f, layout="nk", row_scale=scale, C=yd_out[name])

    # N > 1: the decode step with every Linear's rows sharded like the prefill.  Each call multiplies this rank's
    # rows and stores them into its own result and every peer's (plain stores over NVLink from the kernel), with
    # no per-call ordering between the ranks: every Linear of a step writes its own rows of a per-name buffer, so
    # nothing is overwritten inside a step.  The last call of a step carries the flag exchange (its signal is
    # published after all earlier kernels of the stream have completed), and one wait closes the step: after it
    # every rank holds every result of the step, before the next step starts.  A consumer chained to a single
    # Linear would need the flags on that call (about 8 us); the stack's Linears read resident inputs.
    yd_peer = None
    if world > 1 and args.decode_shard:
        from t81lib_b200.nn.sharded import peer_order
        yd_peer = {name: PeerColumns(dtok * LAYERS, o, torch.bfloat16, dev, copies=1) for name, o, _ in LINEARS}
        t2_shard = [{m[0]: ops.pack_t2(m[3].contiguous(), m[1], m[2]) for m in mods} for mods in prefill_mods] if use_t2 else None

    def decode_step_sharded():
        last = LINEARS[-1][0]
        for li, mods in enumerate(prefill_mods):
            for name, out_l, in_f, packed, scale in mods:
                ex = yd_peer[name]
                lo, hi = rank * out_l, (rank + 1) * out_l
                rows = slice(li * dtok, (li + 1) * dtok)
                peers = [ex.peers[r][0][rows, lo:hi] for r in peer_order(rank, world)]
                closing = li == LAYERS - 1 and name == last
                with ops.independent_of_previous() if (name in INDEPENDENT and not closing) else contextlib.nullcontext():
                    if use_t2:
                        ops.gemm_trit_t2([t2_shard[li][name]], [out_l], xd_in[in_f], K=in_f, row_scales=[scale],
                                         outs=[ex.buffers[0][rows, lo:hi]], peers=peers, sync=ex.flags if closing else None)
                    else:
                        ops.gemm_trit(packed, xd_in[in_f], M=out_l, K=in_f, layout="nk", row_scale=scale,
                                      C=ex.buffers[0][rows, lo:hi], peers=peers, sync=ex.flags if closing else None)
        yd_peer[last].flags.wait()

    # The same step with the Linears that share an input in ONE launch each (q/k/v, gate/up): 4 launches per
    # block instead of 7, through the additive grouped entry point.  Reported beside the per-Linear figure.
    GROUPS = [("q", "k", "v"), ("o",), ("gate", "up"), ("down",)]
    ydg_out = {"qkv": torch.empty(dtok, HIDDEN + 2 * KV, dtype=torch.bfloat16, device=dev),
               "gate_up": torch.empty(dtok, 2 * FFN, dtype=torch.bfloat16, device=dev)}

    def split(buf, widths):
        outs, lo = [], 0
        for w_ in widths:
            outs.append(buf[:, lo:lo + w_]); lo += w_
        return outs

    def decode_step_grouped():
        for li, mods in enumerate(layers):
            by = {m[0]: m for m in mods}
            for names in GROUPS:
                ms = [by[n] for n in names]
                in_f = ms[0][2]
                outs = [yd_out[names[0]]] if len(ms) == 1 else split(ydg_out["qkv" if names[0] == "q" else "gate_up"], [m[1] for m in ms])
                if use_t2:
                    ops.gemm_trit_t2([t2[li][n] for n in names], [m[1] for m in ms], xd_in[in_f], K=in_f,
                                     row_scales=[m[4] for m in ms], outs=outs)
                elif len(ms) == 1:
                    name, out_f, _, packed, scale = ms[0]
                    ops.gemm_trit(packed, xd_in[in_f], M=out_f, K=in_f, layout="nk", row_scale=scale, C=yd_out[name])
                else:
                    ops.gemm_trit_grouped([m[3] for m in ms], xd_in[in_f], K=in_f, row_scales=[m[4] for m in ms], outs=outs)

    # the decode step is launch-bound: capture it once in a CUDA graph
    stream = torch.cuda.Stream(device=dev)

    def capture(step_fn):
        with torch.cuda.stream(stream):
            step_fn()
            torch.cuda.synchronize()
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    step_fn()
            except Exception:
                g = None
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        return g

    graph = capture(decode_step_sharded if yd_peer is not None else decode_step)

    def decode_all():
        for _ in range(DECODE):
            if graph is not None:
                graph.replay()
            else:
                (decode_step_sharded if yd_peer is not None else decode_step)()

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

    # ---- prefill: algorithmic flops / time of the tcgen05 GEMM
    flops_prefill = 2.0 * ptok * LAYERS * sum(o * i for _, o, i in LINEARS) / world  # this rank's share
    tf = flops_prefill / (pre_ms * 1e-3) / 1e12
    gemm = {"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
            "frac": tf / pk["bf16_tflops_sustained"], "frac_of_burst": tf / pk["bf16_tflops"],
            "frac_of_nominal": tf / NOMINAL_BF16_TFLOPS, "traffic": None,
            "peak_source": pk["source"] + " (sustained bf16: the kernel is timed inside a long step)",
            "kernel": "gemm_trit_tc_kernel", "share_of_step": pre_ms / (pre_ms + dec_ms),
            "note": "prefill phase: 224 launches per step, includes launch gaps" + ("; includes the exchange" if world > 1 else "")}
    # ---- decode: algorithmic bytes of the streaming kernel (the dominant kernel by time)
    # weight bytes the decode kernel streams: the decode-stream layout (0.25 byte per trit) or the limbs (0.33)
    limb_bytes = sum(m[3].numel() for mods in layers for m in mods)
    sharded_decode = yd_peer is not None
    if sharded_decode:  # this rank's rows; its outputs go to world results
        limb_bytes = limb_bytes // world
        packed_bytes = sum(t.numel() for d in t2_shard for t in d.values()) if use_t2 else limb_bytes
        other_bytes = sum(4 * m[1] // world + 2 * dtok * m[2] + 2 * dtok * m[1] for mods in layers for m in mods)
    else:               # whole on this rank
        packed_bytes = sum(t.numel() for d in t2 for t in d.values()) if use_t2 else limb_bytes
        other_bytes = sum(4 * m[1] + 2 * dtok * m[2] + 2 * dtok * m[1] for mods in layers for m in mods)
    bytes_decode = packed_bytes + other_bytes
    n_launch = LAYERS * len(LINEARS)
    gbs = bytes_decode * DECODE / (dec_ms * 1e-3) / 1e9
    # DRAM traffic per launch: the ncu capture of this kernel on the 14336 x 4096 layer reads exactly the packed
    # matrix (dram bytes / algorithmic bytes = 1.00, profiles/), so traffic scales with the algorithmic bytes
    roof = {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
            "frac_of_nominal": gbs / NOMINAL_HBM_GBS, "traffic": bytes_decode / n_launch,
            "traffic_note": "bytes per average launch; dram__bytes measured by ncu on one shape equals the algorithmic bytes there",
            "peak_source": pk["source"] + " (copy bandwidth)", "kernel": "gemv_trit_lut_kernel", "tokens": dtok,
            "algorithmic_bytes_per_launch": bytes_decode / n_launch, "us_per_launch": dec_ms * 1e3 / (DECODE * n_launch),
            "weight_layout": (("decode-stream layout" if use_t2 else "packed limbs") + ", rows sharded over the ranks (per-rank bytes and time)" if sharded_decode else
                              "decode-stream layout (2 bits per trit, made once per weight)" if use_t2 else "packed limbs"),
            "reference_layout_equivalent": {"bytes_per_launch": (limb_bytes + other_bytes) / n_launch,
                                            "achieved": (limb_bytes + other_bytes) * DECODE / (dec_ms * 1e-3) / 1e9, "unit": "GB/s",
                                            "frac": (limb_bytes + other_bytes) * DECODE / (dec_ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                                            "note": "the same time against the bytes the limb layout would have streamed"},
            "cuda_graph": graph is not None, "share_of_step": dec_ms / (pre_ms + dec_ms),
            "note": "decode phase: 224 launches per step (one per Linear), includes launch gaps" +
                    ("; rows sharded, results stored into every rank, one flag exchange per step" if sharded_decode else
                     "; whole on every rank" if world > 1 else "")}

    launches = args.steps * (1 + DECODE) * LAYERS * len(LINEARS)
    line = {
        "impl": "ours",
        "metric": "t8.nn.Linear tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": (f"prefill: output features of every Linear sharded x{world}, the GEMM epilogue also stores its output block into every peer's "
                                   f"result over NVLink, flag words order the exchange (no collective); decode: " +
                                   ("rows sharded the same way, plain peer stores from the kernel, one flag exchange per step"
                                    if sharded_decode else "whole on every rank")) if world > 1 else "single GPU",
                   "l2": "inputs larger than L2: 2.3 GB of packed weights and a 134 MB activation buffer are streamed each step",
                   "prefill_ms": pre_ms, "decode_ms": dec_ms, "prefill_tokens_per_s": ptok / (pre_ms * 1e-3),
                   "decode_tokens_per_s": dtok * DECODE / (dec_ms * 1e-3)},
        "roofline": roof, "gemm_roofline": gemm, "gpu_launches": launches,
    }

    # ---- the decode phase again with grouped launches (additive API; the headline stays per-Linear)
    ggraph = capture(decode_step_grouped)
    with torch.cuda.stream(stream):
        reps = max(1, min(args.steps, 5))
        for _ in range(DECODE):
            ggraph.replay() if ggraph is not None else decode_step_grouped()
        g0, g1 = ev(), ev()
        g0.record(stream)
        for _ in range(reps * DECODE):
            ggraph.replay() if ggraph is not None else decode_step_grouped()
        g1.record(stream)
        torch.cuda.synchronize()
    gdec_ms = g0.elapsed_time(g1) / reps
    if world > 1:
        t = torch.tensor([gdec_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gdec_ms = t.item()
    ggbs = bytes_decode * DECODE / (gdec_ms * 1e-3) / 1e9
    line["decode_grouped"] = {"launches_per_step": LAYERS * len(GROUPS), "decode_ms": gdec_ms, "achieved": ggbs, "unit": "GB/s",
                              "frac": ggbs / pk["hbm_gbs"], "frac_of_nominal": ggbs / NOMINAL_HBM_GBS,
                              "tokens_per_s_with_this_decode": job_tokens / ((pre_ms + gdec_ms) * 1e-3),
                              "api": ("t81b200_gemm_trit_t2" if use_t2 else "t81b200_gemm_trit_grouped") + ": q/k/v and gate/up in one launch each"}
    assert _capi.kernel_status(reset=True) == 0, "a kernel reported a timed-out wait"

    # ---- N > 1: an un-timed check that the exchange that produced these numbers is right on every rank
    if world > 1:
        line["parity_ok"] = sharded_parity_check(torch, dist, dev, layers, y_peer, world, rank)
        if yd_peer is not None:
            # the timed decode steps left every Linear's whole result on every rank: compare the first and the last
            # block's with the unsharded product computed here (same kernel family; order of the partial sums may
            # differ with the launch shape: 2^-7 of the largest magnitude, one bf16 rounding)
            ok = True
            for li in (0, LAYERS - 1):
                for name, out_f, in_f, packed, scale in layers[li]:
                    want = ops.gemm_trit(packed, xd_in[in_f], M=out_f, K=in_f, layout="nk", row_scale=scale).float()
                    got = yd_peer[name].buffers[0][li * dtok:(li + 1) * dtok].float()
                    ok = ok and bool((got - want).abs().max() <= 2.0 ** -7 * want.abs().max())
            flag = torch.tensor([1 if ok else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            line["parity_ok"] = bool(line["parity_ok"] and flag.item() == 1)

    if rank == 0:
        line["clocks"] = clocks.summary()

    # ---- end to end through the public API (t81lib_b200.nn.Linear), host buffers in and out
    if args.brief:
        pass
    elif world == 1:
        line["e2e"] = e2e_public_api(torch, dev, Linear, layers, args)
        line["quantize_pack"] = quantize_pack_line(torch, dev, ops, pk)
        line["configs"] = small_configs(torch, dev, ops, pk)
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

    def run_modules(x, ready=None):
        # ready: {width: event} — activations still on their way from the host; waited for at their first use
        y = None
        ready = dict(ready or {})
        with torch.no_grad():
            for row in mods:
                keep = []  # a block's outputs stay alive together, so k/v (up) never reuse q's (gate's) memory
                for (name, out_f, in_f), m in zip(LINEARS, row):
                    if in_f in ready:
                        torch.cuda.current_stream().wait_event(ready.pop(in_f))
                    with ops.independent_of_previous() if name in INDEPENDENT else contextlib.nullcontext():
                        y = m(x[in_f])
                    keep.append(y)
        return y

    copy_stream = torch.cuda.Stream(device=dev)

    def run_sharded_step(x):
        # decode-sized calls through the step-ordered exchange of the sharded modules: no ordering between the
        # ranks per call, one signal + wait closes the step
        y = None
        with torch.no_grad():
            for row in sharded:
                for (name, out_f, in_f), m in zip(LINEARS, row):
                    with ops.independent_of_previous() if name in INDEPENDENT else contextlib.nullcontext():
                        y = m(x[in_f])
        ShardedLinear.close_step(dev)
        return y

    def forward(host, out_host):
        if sharded is None:
            # the first Linears need the HIDDEN-wide activations only: the FFN-wide ones (3.5x the bytes) follow on a
            # second stream while those Linears run, and the first `down` waits for them
            main = torch.cuda.current_stream()
            x = {HIDDEN: host[HIDDEN].to(dev, non_blocking=True)}
            copy_stream.wait_stream(main)
            with torch.cuda.stream(copy_stream):
                x[FFN] = host[FFN].to(dev, non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(copy_stream)
            x[FFN].record_stream(main)
            out_host.copy_(run_modules(x, {FFN: arrived}), non_blocking=True)
            return
        # N > 1: the prefill activations (0.6 GB) enter through rank 0's host copy and reach the other ranks over
        # NVLink; the result leaves through rank 0.  Eight ranks copying the same bytes from the same host memory
        # at once take longer than the whole prefill.
        import torch.distributed as dist
        main = torch.cuda.current_stream()

        def bring(w):  # rank 0's host copy, then the broadcast, on the stream that is current
            t = host[w].to(dev, non_blocking=True) if rank == 0 else torch.empty(host[w].shape, dtype=host[w].dtype, device=dev)
            dist.broadcast(t, src=0)
            return t
        x = {HIDDEN: bring(HIDDEN)}
        copy_stream.wait_stream(main)
        with torch.cuda.stream(copy_stream):  # the FFN-wide activations follow while the first Linears run
            x[FFN] = bring(FFN)
            arrived = torch.cuda.Event()
            arrived.record(copy_stream)
        x[FFN].record_stream(main)
        ready = {FFN: arrived}
        y = None
        with torch.no_grad():
            for row in sharded:
                for (name, out_f, in_f), m in zip(LINEARS, row):
                    if in_f in ready:
                        main.wait_event(ready.pop(in_f))
                    y = m(x[in_f])
        sharded[-1][-1].exchange_for(y.shape[0], y.dtype, dev).flags.wait()  # the peers' blocks of the last result
        if rank == 0:
            out_host.copy_(y, non_blocking=True)

    # The decode pass (224 module calls on 8 tokens) is captured once in a CUDA graph, the way an
    # inference server drives nn.Modules: every step still copies its inputs in from pinned host
    # memory and its result back out.
    x_static = {w: torch.zeros(dtok, w, dtype=torch.bfloat16, device=dev) for w in (HIDDEN, FFN)}
    stream = torch.cuda.Stream(device=dev)
    step_sharded = sharded is not None and bool(getattr(args, "decode_shard", 1))
    if step_sharded:
        for row in sharded:
            for m in row:
                m.step_ordered = True
    decode_pass = run_sharded_step if step_sharded else run_modules
    with torch.cuda.stream(stream):
        decode_pass(x_static)  # also builds the per-layer result buffers (collective) before the capture
        torch.cuda.synchronize()
        dgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(dgraph, stream=stream):
            y_static = decode_pass(x_static)
    torch.cuda.synchronize()

    def decode_forward():
        for w in x_static:
            x_static[w].copy_(host_d[w], non_blocking=True)
        dgraph.replay()
        out_d.copy_(y_static, non_blocking=True)
        if step_sharded:
            ShardedLinear.release_step(dev)  # the peers' next step overwrites y_static: not before this copy has read it

    def job():
        forward(host_p, out_p)
        for _ in range(DECODE):
            decode_forward()

    steps = max(1, args.steps)
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
            "d2h_bytes_per_step": d2h, "steps": steps, "api": ("t81lib_b200.nn.Linear.forward" if world == 1 else
                                                                    "t81lib_b200.nn.sharded.ShardedLinear.forward (prefill: exchange='p2p'; decode: " +
                                                                    ("step_ordered + close_step" if step_sharded else "whole-matrix t81lib_b200.nn.Linear on every rank") + ")")
                   + " (prefill eager; decode pass replayed from a torch.cuda.CUDAGraph)" +
                   ("; prefill activations copied in by rank 0 and broadcast over NVLink, prefill result copied out by rank 0, decode "
                    "inputs and results copied on every rank" if world > 1 else "")}


def sharded_parity_check(torch, dist, dev, layers, y_peer, world, rank):
    """One sharded Linear of the stack per shape (q, k, gate, down of layer 0) through the same p2p exchange the
    timed prefill used, on a 512-token slice: the full-width result on every rank must equal what the unsharded
    kernel gives on that rank, bit for bit.  The verdicts are reduced with MIN over the ranks."""
    from t81lib_b200 import ops
    from t81lib_b200.nn.sharded import PeerColumns, shard_bounds
    gen = torch.Generator(device=dev).manual_seed(4321)  # same activations on every rank
    tokens = 512
    ok = True
    for name, out_f, in_f, packed, scale in layers[0]:
        if name not in ("q", "k", "gate", "down"):
            continue
        x = torch.randn(tokens, in_f, generator=gen, device=dev).to(torch.bfloat16)
        want = ops.gemm_trit(packed, x, M=out_f, K=in_f, layout="nk", row_scale=scale)
        ex = PeerColumns(tokens, out_f, torch.bfloat16, dev)
        lo, hi = shard_bounds(out_f, world, rank)
        for _ in range(2):
            idx = ex.next_index()
            ops.gemm_trit(packed[lo:hi], x, M=hi - lo, K=in_f, layout="nk", row_scale=scale[lo:hi],
                          C=ex.buffers[idx][:, lo:hi], peers=ex.peer_blocks(idx, lo, hi), sync=ex.flags)
            ex.flags.wait()
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(ex.buffers[idx], want))
            dist.barrier()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item() == 1)


def _graph_time(torch, stream, calls, reps=3):
    """Microseconds per call of a list of launches replayed from one CUDA graph."""
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        calls[0]()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for c in calls:
                c()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(calls))


def small_configs(torch, dev, ops, pk):
    """The smaller configurations, a few hundred milliseconds each: gemm_ternary 512x512x256 in both semantics
    (with the compiled reference's gemm_ternary timed once on the same LIMB-mode operands, one host thread), the
    Phi-3-mini-shaped decode sweep (1, 4, 16 tokens) and the 2048-token prefill of the same layers."""
    import numpy as np
    import oracle
    out = {}
    stream = torch.cuda.Stream(device=dev)
    # ---- gemm_ternary: A 512x512 uniform trits (K padded to 528 = 11 limbs), B 512x256, C 512x256, alpha 1, beta 0.5
    rng = np.random.default_rng(1)
    M, N, K = 512, 256, 528
    A = oracle.pack_trits_rowwise(np.pad(rng.integers(-1, 2, (M, 512)).astype(np.int8), ((0, 0), (0, 16))))
    Bf = np.zeros((K, N), np.float32); Bf[:512] = rng.normal(size=(512, N))
    C0 = rng.normal(size=(M, N)).astype(np.float32)
    Ad, Bd = torch.from_numpy(A).to(dev), torch.from_numpy(Bf).to(dev)
    Cs = [torch.from_numpy(C0).to(dev) for _ in range(32)]
    us = _graph_time(torch, stream, [lambda c=c: ops.gemm_trit(Ad, Bd, M=M, K=K, layout="kn", C=c, alpha=1.0, beta=0.5) for c in Cs])
    flops, nbytes = 2.0 * M * 512 * N, A.nbytes + 512 * N * 4 + 2 * M * N * 4
    cfg1 = {"shape": "A 512x512 trits (11 limbs per row), B 512x256 fp32, C 512x256 fp32, alpha 1, beta 0.5",
            "trit_mode": {"us": us, "tflops": flops / us / 1e6, "frac_of_bf16_peak": flops / us / 1e6 / pk["bf16_tflops"],
                          "frac_of_nominal_bf16": flops / us / 1e6 / NOMINAL_BF16_TFLOPS, "gbs": nbytes / us / 1e3,
                          "frac_of_hbm_peak": nbytes / us / 1e3 / pk["hbm_gbs"], "frac_of_nominal_hbm": nbytes / us / 1e3 / NOMINAL_HBM_GBS,
                          "note": "launch-bound: 134 MFLOP and 1.7 MB per call"}}
    # LIMB mode (the reference's literal semantics): B thresholded at 0.5 and column-packed, at most 10 non-zero
    # trits per limb so that limb values stay finite in fp32
    ta = np.zeros((M, K), np.int8); tb = np.zeros((K, N), np.int8)
    for l in range(11):
        ta[:, l * 48:l * 48 + 10] = rng.integers(-1, 2, (M, 10))
        tb[l * 48:l * 48 + 10] = rng.integers(-1, 2, (10, N))
    Al, Bl = oracle.pack_trits_rowwise(ta), oracle.pack_trits_columnwise(tb)
    Ald, Bld = torch.from_numpy(Al).to(dev), torch.from_numpy(Bl).to(dev)
    us_limb = _graph_time(torch, stream, [lambda c=c: ops.gemm_limb(Ald, Bld, c, M, N, K, 1.0, 0.5) for c in Cs[:8]])
    cfg1["limb_mode"] = {"us": us_limb, "limb_products_per_s": M * N * 11 / us_limb * 1e6}
    try:
        from oracle import ref as oracle_ref
        if oracle_ref.available():
            t81lib = oracle_ref.load()
            c = C0.copy()
            t0 = time.perf_counter()
            t81lib.gemm_ternary(Al.reshape(-1, 16).view("V16").reshape(M, 11), Bl.reshape(-1, 16).view("V16").reshape(11, N), c, M, N, K,
                                alpha=1.0, beta=0.5)
            sec = time.perf_counter() - t0
            got = Cs[0].cpu().numpy()  # the GPU's LIMB result after its last call (beta applied repeatedly): compare one fresh call
            fresh = torch.from_numpy(C0).to(dev)
            ops.gemm_limb(Ald, Bld, fresh, M, N, K, 1.0, 0.5)
            cfg1["limb_mode"].update({"reference_cpu_s": sec, "reference_cpu_cores": 1,
                                      "reference_cpu": f"oracle/_ref ({oracle_ref.variant()} build) t81lib.gemm_ternary, same operands, one call",
                                      "speedup_vs_reference_cpu": sec / (us_limb * 1e-6),
                                      "matches_reference": bool(np.allclose(fresh.cpu().numpy(), c, rtol=1e-6))})
    except Exception as exc:  # the reference module is test infrastructure: its absence does not stop the bench
        cfg1["limb_mode"]["reference_cpu"] = f"unavailable: {type(exc).__name__}: {exc}"
    out["gemm_ternary_512x512x256"] = cfg1
    # ---- Phi-3-mini-shaped layers: decode sweep and 2048-token prefill
    gen = torch.Generator(device=dev).manual_seed(11)
    decode, prefill = [], []
    for name, rows, k in [("qkv", 9216, 3072), ("o", 3072, 3072), ("gate_up", 16384, 3072), ("down", 3072, 8192)]:
        kl = (k + 47) // 48
        nbytes = rows * kl * 16
        copies = max(2, int(300e6 // nbytes))
        w = torch.randn(rows, k, device=dev, generator=gen) * 0.02
        mats = [ops.quantize_pack(w, THRESHOLD, "absmean") for _ in range(copies)]
        bias = torch.randn(rows, device=dev, generator=gen) * 0.01
        t2s = None
        for tok in (1, 4, 16, 2048):
            x = torch.randn(tok, k, device=dev, generator=gen).to(torch.bfloat16)
            y = torch.empty(tok, rows, dtype=torch.bfloat16, device=dev)
            use = mats if tok <= 16 else mats[:4]
            if tok <= 16:  # decode-sized: the decode-stream layout of the same weights
                if t2s is None:
                    t2s = [ops.pack_t2(m[0], rows, k) for m in mats]
                us = _graph_time(torch, stream, [lambda m=m, t=t: ops.gemm_trit_t2([t], [rows], x, K=k, row_scales=[m[1]], biases=[bias], outs=[y])
                                                for m, t in zip(mats, t2s)])
                alg = t2s[0].numel() + 8 * rows + 2 * tok * k + 2 * tok * rows
                ref_alg = nbytes + 8 * rows + 2 * tok * k + 2 * tok * rows
                decode.append({"layer": name, "rows": rows, "k": k, "tokens": tok, "us": us, "gbs": alg / us / 1e3,
                               "frac": alg / us / 1e3 / pk["hbm_gbs"], "frac_of_nominal": alg / us / 1e3 / NOMINAL_HBM_GBS,
                               "reference_layout_equivalent_gbs": ref_alg / us / 1e3})
                continue
            us = _graph_time(torch, stream, [lambda m=m: ops.gemm_trit(m[0], x, M=rows, K=k, layout="nk", row_scale=m[1], bias=bias, C=y)
                                            for m in use])
            if tok <= 16:
                alg = nbytes + 8 * rows + 2 * tok * k + 2 * tok * rows
                decode.append({"layer": name, "rows": rows, "k": k, "tokens": tok, "us": us, "gbs": alg / us / 1e3,
                               "frac": alg / us / 1e3 / pk["hbm_gbs"], "frac_of_nominal": alg / us / 1e3 / NOMINAL_HBM_GBS})
            else:
                tfl = 2.0 * rows * k * tok / us / 1e6
                prefill.append({"layer": name, "rows": rows, "k": k, "tokens": tok, "us": us, "tflops": tfl,
                                "frac_of_burst": tfl / pk["bf16_tflops"], "frac_of_nominal": tfl / NOMINAL_BF16_TFLOPS})
        del mats, w
    out["phi3_decode_sweep"] = {"peak_gbs": pk["hbm_gbs"], "weight_layout": "decode-stream layout (2 bits per trit); gbs and frac count its bytes",
                                "rotation": "distinct weight copies of 300 MB per shape (> L2) in one CUDA graph",
                                "cases": decode}
    out["phi3_prefill_2048"] = {"peak_tflops": pk["bf16_tflops"], "cases": prefill}
    return out


def quantize_pack_line(torch, dev, ops, pk):
    """Quantise + pack of a 4096x4096 fp32 N(0, 0.02^2) weight, absmean rule, threshold 0.45."""
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
            "frac": alg / sec / 1e9 / pk["hbm_gbs"], "us_per_launch": sec * 1e6, "kernel": "quantize_pack_ring_kernel"}


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
        if args.decode_layout == "t2":
            t2s = [ops.pack_t2(m, rows, k) for m in mats]
            calls = [lambda m=m: ops.gemm_trit_t2([m], [rows], x, K=k, row_scales=[scale], outs=[y]) for m in t2s] * 2
            wbytes = t2s[0].numel()
        else:
            calls = [lambda m=m: ops.gemm_trit(m, x, M=rows, K=k, layout="nk", row_scale=scale, C=y) for m in mats] * 2
            wbytes = rows * kl * 16
        alg, unit, peak, name = wbytes + 4 * rows + 2 * tok * k + 2 * tok * rows, "GB/s", pk["hbm_gbs"], "gemv_trit_lut_kernel"
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
        alg, unit, peak, name = 4096 * 4096 * 4 + 4096 * 86 * 16 + 4096 * 4, "GB/s", pk["hbm_gbs"], "quantize_pack_ring_kernel"
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
    """The ternary Linear layers of a Phi-3-mini-shaped block, decode-sized calls with
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
        t2s = None
        for tok in (1, 4, 16, 2048):
            x = torch.randn(tok, k, device=dev, generator=gen).to(torch.bfloat16)
            y = torch.empty(tok, rows, dtype=torch.bfloat16, device=dev)
            n = copies if tok <= 16 else 4
            use_t2 = tok <= 16 and args.decode_layout == "t2"
            if use_t2 and t2s is None:
                t2s = [ops.pack_t2(m[0], rows, k) for m in mats]

            def call(i):
                m, sc = mats[i % copies]
                if use_t2:
                    ops.gemm_trit_t2([t2s[i % copies]], [rows], x, K=k, row_scales=[sc], biases=[bias], outs=[y])
                else:
                    ops.gemm_trit(m, x, M=rows, K=k, layout="nk", row_scale=sc, bias=bias, C=y)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                call(0)
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=stream):
                    for i in range(n):
                        call(i)
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
                alg = (t2s[0].numel() if use_t2 else nbytes) + 8 * rows + 2 * tok * k + 2 * tok * rows
                line = {"achieved": alg / sec / 1e9, "unit": "GB/s", "peak": pk["hbm_gbs"], "bound": "hbm",
                        "weight_layout": "decode-stream" if use_t2 else "limbs"}
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
    ap.add_argument("--decode-layout", choices=["t2", "limb"], default="t2",
                    help="weight layout of the decode-sized calls: the decode-stream layout made once per weight (default) "
                         "or the reference's packed limbs")
    ap.add_argument("--decode-shard", type=int, default=1,
                    help="N > 1: 1 shards the rows of every decode-sized Linear over the ranks like the prefill (default), "
                         "0 runs the decode phase whole on every rank")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--brief", action="store_true",
                    help="timed region only: no end-to-end pass, no small configurations, no CPU baseline (profiling runs)")
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
