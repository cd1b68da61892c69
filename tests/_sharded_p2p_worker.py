"""One rank of tests/test_gpu_sharded_p2p.py (started by torch.distributed.run, one process per GPU):
the column-sharded Linear with exchange="p2p" must return, on every rank, exactly what the unsharded
layer returns, for the tensor-core path (stores into the peers from the GEMM), for fp32 activations
(per-element peer stores) and for decode-sized calls (copy-engine push after the streaming kernel)."""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main() -> int:
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from t81lib_b200 import _capi
    from t81lib_b200 import torch as t81_torch
    from t81lib_b200.nn.sharded import ShardedLinear

    # every product below, sharded or whole, runs on the packed limbs: the comparison is bit for bit, and the
    # decode-stream layout (used for <= 16 tokens otherwise) accumulates in another order than the peer-store kernel
    t81_torch.DECODE_STREAM_LAYOUT = False
    gen = torch.Generator(device=dev).manual_seed(5)  # same values on every rank
    w = torch.randn(1024, 520, generator=gen, device=dev) * 0.02
    b = torch.randn(1024, generator=gen, device=dev) * 0.01
    full = t81_torch.TernaryTensor.from_float(w, threshold=0.45, rule="absmean")
    ok = True
    for tokens, dtype in ((300, torch.bfloat16), (8, torch.bfloat16), (130, torch.float32), (700, torch.float16),
                          (20, torch.float32), (3, torch.float32)):
        x = torch.randn(tokens, 520, generator=gen, device=dev).to(dtype)
        want = full.matmul_input(x, bias=b)
        for exchange in ("collective", "p2p"):
            layer = ShardedLinear(w, b, threshold=0.45, rule="absmean", exchange=exchange)
            for _ in range(3):  # the p2p buffers are handed out round-robin: go around more than once
                got = layer(x)
                torch.cuda.synchronize()
                same = torch.equal(got, want)
                ok = ok and same
                if rank == 0 and not same:
                    print(f"MISMATCH tokens={tokens} dtype={dtype} exchange={exchange}", flush=True)
    # chained calls: each matmul waits for the peers' previous stores by itself, one wait at the end
    x = torch.randn(8, 520, generator=gen, device=dev).to(torch.bfloat16)
    want = full.matmul_input(x, bias=b)
    layer = ShardedLinear(w, b, threshold=0.45, rule="absmean", exchange="p2p")
    layer.defer_wait = True
    outs = [layer(x) for _ in range(40)]
    layer.exchange_for(8, torch.bfloat16, dev).flags.wait()
    torch.cuda.synchronize()
    ok = ok and torch.equal(outs[-1], want) and torch.equal(outs[-2], want)
    # A result is read AFTER the next same-shape call has been issued, while the peer runs ahead: rank 0 stalls
    # its stream before the read, the other ranks go on issuing calls that store into rank 0's buffers.  With
    # three buffers per shape the peers' stores of call j + 2 cannot land in the buffer that holds result j.
    x1 = torch.randn(8, 520, generator=gen, device=dev).to(torch.bfloat16)
    x2 = torch.randn(8, 520, generator=gen, device=dev).to(torch.bfloat16)
    want_sum = full.matmul_input(x1, bias=b).float() + full.matmul_input(x2, bias=b).float()
    for _ in range(4):
        ra = layer(x1)
        rb = layer(x2)
        if rank == 0:
            torch.cuda._sleep(20_000_000)  # ~10 ms: the peers get far ahead of this stream
        layer.exchange_for(8, torch.bfloat16, dev).flags.wait()  # the peers' blocks of call j + 1 have landed
        total = ra.float() + rb.float()    # reads result j after call j + 1 was issued
        layer(x)                           # call j + 2 (stores into a third buffer on every rank)
        layer.exchange_for(8, torch.bfloat16, dev).flags.wait()
        torch.cuda.synchronize()
        ok = ok and torch.equal(total, want_sum)
    # Step-ordered exchange: decode-sized calls store into every rank without per-call ordering, one signal + one
    # wait per rank closes the step.  Two layers, three steps; results against the unsharded product on the
    # decode-stream layout (same kernel, other launch shape: one rounding of the output type).
    from t81lib_b200 import ops
    w2 = torch.randn(768, 520, generator=gen, device=dev) * 0.02
    full2 = t81_torch.TernaryTensor.from_float(w2, threshold=0.45, rule="absmean")
    l1 = ShardedLinear(w, b, threshold=0.45, rule="absmean", exchange="p2p")
    l2 = ShardedLinear(w2, None, threshold=0.45, rule="absmean", exchange="p2p")
    l1.step_ordered = l2.step_ordered = True
    for tokens, dtype in ((8, torch.bfloat16), (3, torch.float32), (16, torch.float16)):
        for _ in range(3):
            xs = torch.randn(tokens, 520, generator=gen, device=dev).to(dtype)
            y1, y2 = l1(xs), l2(xs)
            ShardedLinear.close_step(dev)
            torch.cuda.synchronize()
            want1 = ops.gemm_trit_t2([ops.pack_t2(full.packed, 1024, 520)], [1024], xs, K=520, row_scales=[full.row_scale], biases=[b])[0]
            want2 = ops.gemm_trit_t2([ops.pack_t2(full2.packed, 768, 520)], [768], xs, K=520, row_scales=[full2.row_scale])[0]
            for got, want in ((y1, want1), (y2, want2)):
                tol = (2.0 ** -7 if dtype != torch.float32 else 1e-5) * float(want.float().abs().max())
                same = float((got.float() - want.float()).abs().max()) <= tol
                ok = ok and same
                if rank == 0 and not same:
                    print(f"STEP MISMATCH tokens={tokens} dtype={dtype}", flush=True)
            dist.barrier()  # nobody starts the next step's stores before every rank has compared
    ok = ok and _capi.kernel_status(reset=True) == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("SHARDED_P2P_OK" if flag.item() == 1 else "SHARDED_P2P_FAILED", flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0 if flag.item() == 1 else 1)  # no process-group teardown (it has been seen to wait forever)


if __name__ == "__main__":
    main()
