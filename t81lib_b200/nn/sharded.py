"""Column-sharded ternary Linear: output features are split across the ranks of a
process group (one process per GPU); each rank quantises, packs and multiplies
only its slice of rows.  The result is assembled either by one all-gather
(``exchange="collective"``, any backend) or by the matmul kernel itself storing its
column block into every peer's result over NVLink, ordered by flag words
(``exchange="p2p"``, CUDA, one node).

Row-wise packing and per-row scales make a shard self-contained: the packed
bytes of rank r's slice equal rows [r*out/R, (r+1)*out/R) of the unsharded
packed matrix, byte for byte.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch import nn


def shard_bounds(out_features: int, world_size: int, rank: int) -> tuple[int, int]:
    """Rows [lo, hi) owned by ``rank``.  ``out_features`` must divide evenly so
    that every rank contributes an equal, contiguous chunk to the all-gather."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} is not in a group of {world_size}")
    if out_features % world_size != 0:
        raise ValueError(f"out_features ({out_features}) must be divisible by the group size ({world_size})")
    per = out_features // world_size
    return rank * per, (rank + 1) * per


def gather_columns(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather (tokens, out/R) slices into (tokens, out).  One collective; the
    rank-major gather buffer is re-viewed token-major with a single copy."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    tokens, per = local.shape
    flat = torch.empty((world * tokens, per), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, local.contiguous(), group=group)  # rank-major concatenation
    gathered = flat.view(world, tokens, per)
    if tokens == 1:
        return gathered.reshape(1, world * per)
    return gathered.permute(1, 0, 2).reshape(tokens, world * per)


def _open_on(device: torch.device, handles):
    """Rebuild tensors another rank exported with ``reduce_tensor``, opening the CUDA IPC handle in
    THIS rank's device context (argument 6 of torch's rebuild function is the device index): kernels
    and copies of this GPU then reach the peer's memory over NVLink."""
    return [fn(*(args[:6] + (device.index,) + args[7:])) for fn, args in handles]


def peer_order(rank: int, world: int) -> list:
    """The other ranks in the order this rank lists them (a different first peer on every rank, so
    that pushes do not all start on the same GPU)."""
    return [(rank + shift) % world for shift in range(1, world)]


def flag_slot_word(rank: int, peer: int, world: int) -> int:
    """Index, inside ``peer``'s flag words, of the word ``rank`` publishes its exchange count to:
    word 16 * (1 + i) where i is ``rank``'s position in ``peer``'s peer list."""
    return 16 * (1 + (rank - peer - 1) % world)


class ExchangeFlags:
    """The flag words that order the exchanges of column-sharded Linears between the GPUs of one
    node without a collective and without the host: every rank owns ``SYNC_WORDS`` words that its
    peers can write, and knows the address of its own slot in every peer's words (layout: see
    ``t81b200_gemm_trit_peers``).  One instance per (group, device), shared by every exchange on
    that device, because a call waits for the peers' PREVIOUS call whatever layer that was.
    Construction is collective."""

    _instances: dict = {}

    @classmethod
    def get(cls, device: torch.device, group=None) -> "ExchangeFlags":
        key = (device.index, id(group) if group is not None else None)
        inst = cls._instances.get(key)
        if inst is None:
            inst = cls._instances[key] = cls(device, group)
        return inst

    def __init__(self, device: torch.device, group=None):
        import ctypes
        from torch.multiprocessing.reductions import reduce_tensor
        from .. import _capi
        self.device, self.group = device, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world - 1 > _capi.MAX_PEERS:
            raise ValueError(f"at most {_capi.MAX_PEERS + 1} ranks are supported")
        self.words = torch.zeros(_capi.SYNC_WORDS, dtype=torch.int32, device=device)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, [reduce_tensor(self.words)], group=group)
        self.peer_ranks = peer_order(self.rank, self.world)
        self._peer_words = {r: _open_on(device, everyone[r])[0] for r in self.peer_ranks}
        slots = [self._peer_words[q].data_ptr() + 4 * flag_slot_word(self.rank, q, self.world) for q in self.peer_ranks]
        self.local_ptr = self.words.data_ptr()
        self.slot_ptrs = (ctypes.c_void_p * len(slots))(*slots)
        self.n_peers = len(slots)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def signal(self) -> None:
        """Queue, on torch's current stream, the publication of one more exchange of this rank: once everything
        queued before it has completed, the peers' next ``wait`` sees it.  Closes a step of calls issued
        without flags (``ShardedLinear.step_ordered``)."""
        from .. import _capi
        _capi.check(_capi.lib.t81b200_exchange_signal(self.local_ptr, self.slot_ptrs, self.n_peers,
                                                      torch.cuda.current_stream(self.device).cuda_stream))

    def wait(self) -> None:
        """Queue, on torch's current stream, the wait after which everything the peers stored for
        the calls issued so far is in this GPU's memory."""
        from .. import _capi
        _capi.check(_capi.lib.t81b200_exchange_wait(self.local_ptr, self.n_peers,
                                                    torch.cuda.current_stream(self.device).cuda_stream))


class PeerColumns:
    """Full-width (tokens, out_features) result buffers of every rank of one node, mapped into
    this process, for an all-gather made of copy-engine pushes.

    Each rank's matmul writes its output features straight into columns [lo, hi) of its own
    buffer (a strided C operand) and, from the same kernel, into the same place of every
    peer's buffer over NVLink (``ops.gemm_trit(..., peers=..., sync=flags)``); flag words written
    behind the data (``ExchangeFlags``) tell every rank when all blocks have landed.  Compared with
    ``all_gather_into_tensor`` there is no second pass over the result: no gather kernel and
    no token-major re-copy of a rank-major gather buffer.

    Construction is collective (handles are exchanged through the process group).  ``copies``
    buffers are handed out round-robin.  How long a result lives: the flag protocol lets a peer
    start call j + 1 as soon as this rank has COMPLETED call j, and that call j + 1 stores into
    buffer (j + 1) % copies of this rank.  Work this rank queues on its stream before it issues call
    j + c - 1 of this shape has finished by then, so with ``copies = c`` result j may be read by
    anything queued before the (c - 1)-th following call of the same shape; later readers must clone
    it first.  The default of three buffers gives every result a lifetime of two following calls
    (``a = L1(x); b = L2(a); out = a + b`` is safe).  CUDA only; ranks must be processes of one node
    that see the same GPUs in the same order."""

    def __init__(self, tokens: int, out_features: int, dtype: torch.dtype, device: torch.device, group=None,
                 copies: int = 3):
        from torch.multiprocessing.reductions import reduce_tensor
        if device.type != "cuda":
            raise ValueError("PeerColumns needs CUDA tensors (there is no CPU path)")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.tokens, self.out_features, self.dtype, self.device = tokens, out_features, dtype, device
        self.buffers = [torch.empty((tokens, out_features), dtype=dtype, device=device) for _ in range(copies)]
        mine = [reduce_tensor(b) for b in self.buffers]  # (rebuild function, CUDA IPC handle + geometry)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        self.peers = []  # peers[r][i]: rank r's buffer i as a tensor of this process (None for this rank)
        for r, handles in enumerate(everyone):
            self.peers.append(None if r == self.rank else _open_on(device, handles))
        self.flags = ExchangeFlags.get(device, group)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        self._next = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def next_index(self) -> int:
        i = self._next
        self._next = (i + 1) % len(self.buffers)
        return i

    def peer_blocks(self, index: int, lo: int, hi: int) -> list:
        """Columns [lo, hi) of every peer's buffer ``index`` (views of peer memory), in an order
        that starts with a different peer on every rank."""
        return [self.peers[r][index][:, lo:hi] for r in peer_order(self.rank, self.world)]

    def signal(self) -> None:
        """Collective alternative to the flag protocol: queue, on torch's current stream, an
        all-reduce after which every rank's buffers hold the column blocks that all ranks wrote
        before their own ``signal`` (for matmuls issued without ``sync=``)."""
        dist.all_reduce(self._flag, group=self.group)


class ShardedLinear(nn.Module):
    """Eval-only ternary Linear whose rows are sharded over ``group``.

    Built either from the full float weight (each rank keeps its slice) or from
    an ``nn.Linear`` via ``from_linear``.  Activations are replicated."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *, threshold: float = 0.45,
                 rule: str = "fixed", group=None, rank: Optional[int] = None, world_size: Optional[int] = None,
                 shard_min_tokens: int = 0, exchange: str = "collective", matmul=None, quantize=None):
        super().__init__()
        if weight.ndim != 2:
            raise ValueError("t81.trit tensors currently only support 2D matrices")
        self.group = group
        self.world_size = world_size if world_size is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self.out_features, self.in_features = weight.shape
        lo, hi = shard_bounds(self.out_features, self.world_size, self.rank)
        self.rows = (lo, hi)
        self.ternary_threshold = threshold
        self.ternary_rule = rule
        # Calls with fewer tokens than this run unsharded on every rank: an all-gather costs tens
        # of microseconds, a decode-sized matmul a few.  Needs the whole packed matrix on every
        # rank (2.67 bits per weight); the shard is then a view of it, not a second copy.
        self.shard_min_tokens = shard_min_tokens
        # "collective": one all_gather_into_tensor per call (any backend).  "p2p": stores into the peers'
        # results over NVLink (CUDA, one node); the result is then one of three shared buffers per shape:
        # it may be read by work queued before the second following p2p call of that shape is issued
        # (see PeerColumns); clone it to keep it longer.
        if exchange not in ("collective", "p2p"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.exchange = exchange
        # p2p only: True leaves the wait for the peers' blocks to the consumer — the next sharded matmul
        # waits at its start by itself; anything else calls ExchangeFlags.wait() first
        self.defer_wait = False
        # p2p only: True sends decode-sized calls (at most 16 tokens) through the step-ordered exchange — the call
        # multiplies this rank's rows (decode-stream layout) and stores them into a result buffer of ITS OWN on
        # every rank, with no ordering between the ranks per call; ``ShardedLinear.close_step(device)`` — one
        # signal and one wait per rank — then makes every result of the step whole on every rank.  For steps
        # whose Linears do not consume each other's results before the step is closed; a result is overwritten by
        # the layer's next call with that token count.
        self.step_ordered = False
        self._step_buffers: dict = {}
        self._full_matmul = None
        self._full_bias = None if bias is None or shard_min_tokens <= 0 else bias.detach().clone()
        # `quantize` / `matmul` are injection points for host-side tests of the sharding
        # logic; the defaults are the device kernels.
        if quantize is None:
            from .. import torch as t81_torch
            if shard_min_tokens > 0:
                full = t81_torch.TernaryTensor.from_float(weight.detach(), threshold=threshold, rule=rule)
                self.full_weight = full
                scale = None if full.row_scale is None else full.row_scale[lo:hi]
                self.ternary_weight = t81_torch.TernaryTensor(
                    full.packed[lo:hi], (hi - lo, self.in_features), k_actual=self.in_features, k_limbs=full.packed.shape[1],
                    threshold=threshold, row_scale=scale, rule=rule)
                self._full_matmul = lambda x, b: full.matmul_input(x, bias=b)
            else:
                self.ternary_weight = t81_torch.TernaryTensor.from_float(weight[lo:hi].detach(), threshold=threshold, rule=rule)
            self._matmul = lambda x, b: self.ternary_weight.matmul_input(x, bias=b)
        else:
            self.ternary_weight = quantize(weight[lo:hi].detach(), threshold, rule)
            self._matmul = matmul
        self.bias = None if bias is None else bias[lo:hi].detach().clone()

    @classmethod
    def from_linear(cls, linear: nn.Linear, **kwargs) -> "ShardedLinear":
        threshold = kwargs.pop("threshold", getattr(linear, "ternary_threshold", 0.45))
        return cls(linear.weight, linear.bias, threshold=threshold, **kwargs)

    def forward_local(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's (tokens, out/R) slice, no communication."""
        if x.ndim != 2:
            raise ValueError("t81.nn.Linear expects 2D or 3D inputs")
        bias = self.bias
        if bias is not None and bias.device != x.device:
            bias = self.bias = bias.to(x.device)
        return self._matmul(x, bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.ndim == 3:
            b, s, f = x.shape
            return self.forward(x.reshape(b * s, f)).reshape(b, s, -1)
        if self._full_matmul is not None and x.shape[0] < self.shard_min_tokens:
            bias = self._full_bias
            if bias is not None and bias.device != x.device:
                bias = self._full_bias = bias.to(x.device)
            return self._full_matmul(x, bias)
        if self.exchange == "p2p" and self.world_size > 1 and x.is_cuda and hasattr(self.ternary_weight, "packed"):
            return self._forward_p2p(x)
        local = self.forward_local(x)
        if self.world_size == 1:
            return local
        return gather_columns(local, self.group)

    # Result buffers are shared by every p2p layer of a process with the same (group, device, tokens, width,
    # dtype): a stack of layers needs three buffers per width, not three per layer.  A result stays valid
    # for readers queued before the second following call of that shape is issued (PeerColumns explains why
    # that takes three buffers under the flag protocol).
    _shared_exchanges: dict = {}

    def exchange_for(self, tokens: int, dtype: torch.dtype, device: torch.device) -> PeerColumns:
        key = (id(self.group) if self.group is not None else None, device.index, tokens, self.out_features, dtype)
        ex = ShardedLinear._shared_exchanges.get(key)
        if ex is None:  # collective: every rank reaches this with the same shape
            ex = ShardedLinear._shared_exchanges[key] = PeerColumns(tokens, self.out_features, dtype, device, self.group)
        return ex

    @staticmethod
    def close_step(device: torch.device, group=None) -> None:
        """Queue, on torch's current stream, the end of a step of ``step_ordered`` calls: after it every result
        returned by those calls is whole on this rank.  Every rank calls it once per step."""
        flags = ExchangeFlags.get(device, group)
        flags.signal()
        flags.wait()

    @staticmethod
    def release_step(device: torch.device, group=None) -> None:
        """Queue, on torch's current stream, the point after which the results of the closed step may be overwritten:
        the same signal + wait, issued by every rank AFTER the work that reads those results has been queued.  A
        faster rank's next step stores into this rank's result buffers, so a step is: calls, ``close_step``, readers,
        ``release_step``.  Not needed when nothing reads the results between two steps."""
        ShardedLinear.close_step(device, group)

    def _forward_step(self, x: torch.Tensor) -> torch.Tensor:
        from .. import ops
        tokens = x.shape[0]
        ex = self._step_buffers.get((tokens, x.dtype))
        if ex is None:  # collective: every rank reaches this with the same shape
            ex = self._step_buffers[(tokens, x.dtype)] = PeerColumns(tokens, self.out_features, x.dtype, x.device, self.group, copies=1)
        lo, hi = self.rows
        w = self.ternary_weight
        if w._t2 is None:
            w._t2 = ops.pack_t2(w.packed.contiguous(), hi - lo, self.in_features)
        bias = self.bias
        if bias is not None and bias.device != x.device:
            bias = self.bias = bias.to(x.device)
        ops.gemm_trit_t2([w._t2], [hi - lo], x, K=self.in_features, row_scales=[w.row_scale], biases=[bias],
                         outs=[ex.buffers[0][:, lo:hi]], peers=ex.peer_blocks(0, lo, hi))
        return ex.buffers[0]

    def _forward_p2p(self, x: torch.Tensor) -> torch.Tensor:
        from .. import ops
        tokens = x.shape[0]
        if self.step_ordered and 1 <= tokens <= 16:
            return self._forward_step(x)
        ex = self.exchange_for(tokens, x.dtype, x.device)
        i = ex.next_index()
        lo, hi = self.rows
        w = self.ternary_weight
        bias = self.bias
        if bias is not None and bias.device != x.device:
            bias = self.bias = bias.to(x.device)
        ops.gemm_trit(w.packed, x, M=hi - lo, K=self.in_features, layout="nk", row_scale=w.row_scale, bias=bias,
                      C=ex.buffers[i][:, lo:hi], peers=ex.peer_blocks(i, lo, hi), sync=ex.flags)
        if not self.defer_wait:
            ex.flags.wait()
        return ex.buffers[i]
