"""Host-side logic of the column-sharded Linear, on CPU: shard bounds, the
byte-for-byte identity of sharded and unsharded packing, and the all-gather path
with two gloo ranks.  The matmul and quantiser are injected (the CPU oracle stands
in as the checker's arithmetic); the device kernels are not involved here."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from t81lib_b200.nn.sharded import ShardedLinear, gather_columns, shard_bounds


def test_shard_bounds():
    assert shard_bounds(4096, 8, 0) == (0, 512)
    assert shard_bounds(4096, 8, 7) == (3584, 4096)
    assert shard_bounds(10, 1, 0) == (0, 10)
    with pytest.raises(ValueError, match="divisible"):
        shard_bounds(1000, 3, 0)
    with pytest.raises(ValueError, match="not in a group"):
        shard_bounds(8, 2, 2)
    covered = [shard_bounds(96, 4, r) for r in range(4)]
    assert covered == [(0, 24), (24, 48), (48, 72), (72, 96)]


def test_sharded_packing_equals_rows_of_unsharded_packing():
    rng = np.random.default_rng(0)
    w = rng.normal(0, 0.02, (64, 200)).astype(np.float32)
    full, full_scale = oracle.pack_dense_matrix_absmean(w, 0.45)
    for world in (2, 4, 8):
        for rank in range(world):
            lo, hi = shard_bounds(64, world, rank)
            part, scale = oracle.pack_dense_matrix_absmean(w[lo:hi], 0.45)
            assert np.array_equal(part, full[lo:hi]) and np.array_equal(scale, full_scale[lo:hi])


def _cpu_quantize(weight, threshold, rule):
    packed, scale = oracle.pack_dense_matrix_absmean(weight.numpy(), threshold)
    return packed, scale, weight.shape[1]


def _cpu_matmul_factory(holder):
    def matmul(x, bias):
        packed, scale, in_f = holder["w"]
        y = oracle.linear_forward(packed, scale, None if bias is None else bias.numpy(), x.numpy(), in_f)
        return torch.from_numpy(y)
    return matmul


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(7)  # same weights on every rank
        weight = torch.randn(48, 100, generator=gen) * 0.02
        bias = torch.randn(48, generator=gen) * 0.01
        x = torch.randn(5, 100, generator=gen)
        holder = {}
        layer = ShardedLinear(weight, bias, threshold=0.45, rule="absmean", quantize=_cpu_quantize,
                              matmul=_cpu_matmul_factory(holder))
        holder["w"] = layer.ternary_weight
        assert layer.rows == shard_bounds(48, world, rank)
        y = layer(x)
        y3 = layer(x.reshape(1, 5, 100))
        assert y3.shape == (1, 5, 48) and torch.equal(y3[0], y)
        # single-token case takes the reshape-only branch of the gather
        y1 = layer(x[:1])
        assert torch.equal(y1, y[:1])
        # a rank that brings a slice of the wrong width is caught by the collective's size check
        torch.save(y, os.path.join(out_dir, f"y{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_forward_matches_unsharded(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    gen = torch.Generator().manual_seed(7)
    weight = torch.randn(48, 100, generator=gen) * 0.02
    bias = torch.randn(48, generator=gen) * 0.01
    x = torch.randn(5, 100, generator=gen)
    packed, scale = oracle.pack_dense_matrix_absmean(weight.numpy(), 0.45)
    want = oracle.linear_forward(packed, scale, bias.numpy(), x.numpy(), 100)
    for rank in range(world):
        got = torch.load(os.path.join(tmp_path, f"y{rank}.pt")).numpy()
        assert np.array_equal(got, want)  # every rank ends with the full, identical result


def test_gather_columns_single_rank_is_identity():
    port = _free_port()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        t = torch.arange(12.0).reshape(3, 4)
        assert gather_columns(t) is t
    finally:
        dist.destroy_process_group()


def test_unknown_exchange_is_rejected():
    w = torch.zeros(8, 16)
    with pytest.raises(ValueError, match="unknown exchange"):
        ShardedLinear(w, None, world_size=1, rank=0, exchange="carrier-pigeon", quantize=_cpu_quantize,
                      matmul=lambda x, b: x)


def test_p2p_exchange_is_a_cuda_only_path_and_cpu_inputs_take_the_collective():
    # with CPU tensors (or injected kernels) exchange="p2p" must not try to map peer memory
    gen = torch.Generator().manual_seed(3)
    weight = torch.randn(12, 50, generator=gen) * 0.02
    x = torch.randn(4, 50, generator=gen)
    holder = {}
    layer = ShardedLinear(weight, None, threshold=0.45, rule="absmean", world_size=1, rank=0, exchange="p2p",
                          quantize=_cpu_quantize, matmul=_cpu_matmul_factory(holder))
    holder["w"] = layer.ternary_weight
    packed, scale = oracle.pack_dense_matrix_absmean(weight.numpy(), 0.45)
    want = oracle.linear_forward(packed, scale, None, x.numpy(), 50)
    assert np.array_equal(layer(x).numpy(), want)


def test_exchange_flag_slots_are_consistent_between_ranks():
    # Rank q waits on words 16 * (1 + j), j = 0 .. world-2, one per entry of ITS peer list; rank r must
    # publish into exactly the word that stands for r in q's list, and no two ranks may share a word.
    from t81lib_b200 import _capi
    from t81lib_b200.nn.sharded import flag_slot_word, peer_order
    for world in (2, 3, 4, 8):
        assert world - 1 <= _capi.MAX_PEERS
        for q in range(world):
            order = peer_order(q, world)
            assert sorted(order) == [r for r in range(world) if r != q]
            words = [flag_slot_word(r, q, world) for r in order]
            assert words == [16 * (1 + j) for j in range(world - 1)]  # q's j-th peer writes q's j-th wait word
            assert max(words) < _capi.SYNC_WORDS and len(set(words)) == world - 1
