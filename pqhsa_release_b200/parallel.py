"""KV-head sharding across the GPUs of one node, in vLLM's tensor-parallel layout:
rank r owns KV heads [r * Hkv / W, (r + 1) * Hkv / W) and their G query heads; the
index, codes and pages of a head live only on its owner.  Streams are independent, so
the data path has exactly one collective: the all-gather of the output slices.

The reference has no distributed layer of its own (its only rank lookup is
benchmarks/vllm_backend/worker_hook.py:91-94); under vLLM each TP worker simply sees
its shard of heads, which is what these helpers reproduce for stand-alone use.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def kv_head_shard(num_kv_heads: int, rank: int, world: int) -> range:
    """KV heads owned by ``rank``."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} KV heads do not shard evenly over {world} ranks")
    per = num_kv_heads // world
    return range(rank * per, (rank + 1) * per)


def query_head_shard(num_kv_heads: int, group: int, rank: int, world: int) -> range:
    """Query heads owned by ``rank`` (the G heads of each owned KV head)."""
    kv = kv_head_shard(num_kv_heads, rank, world)
    return range(kv.start * group, kv.stop * group)


def gather_context(local: torch.Tensor, out: torch.Tensor | None = None, group=None) -> torch.Tensor:
    """All-gather of the per-rank contexts [B, Hq / W, D] into [B, Hq, D] (head order = rank
    order).  ``out`` may be a preallocated [W, B, Hq / W, D] staging tensor (needed when the call
    is captured in a CUDA graph).  With one rank this is the identity."""
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if world == 1:
        return local
    local = local.contiguous()
    if out is None:
        out = torch.empty((world, *local.shape), dtype=local.dtype, device=local.device)
    b, hl, d = local.shape
    # the output is the ranks' tensors concatenated along dim 0
    dist.all_gather_into_tensor(out.view(world * b, hl, d), local, group=group)
    return out.permute(1, 0, 2, 3).reshape(b, world * hl, d)


class PeerExchange:
    """The output exchange without a collective call: symmetric receive buffers of the ranks of one
    node, mapped into every process (``torch.distributed._symmetric_memory``), and their addresses
    installed in a pool's parameters.  The combine kernel of every step then sends its output rows to
    every rank as flagged words (8-byte stores of 4 bytes of the row and the step count);
    :meth:`wait` enqueues the receiving kernel, which waits (bounded) for every word of the step and
    unpacks the rows into the gathered buffer.  All ranks must run the same number of steps.

    Layout of a rank's gathered rows: ``[2, world, R, 128]`` - parity of the step, source rank, the
    source rank's query rows."""

    def __init__(self, pool, group=None):
        import torch.distributed._symmetric_memory as symm

        from . import _lib

        self.pool, self._lib = pool, _lib
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        R = pool.S * pool.G
        words = _lib.HEAD_DIM * torch.empty(0, dtype=pool.dtype).element_size() // 4
        self.recv = symm.empty(2, self.world, R, words, 2, dtype=torch.int32, device=pool.device)
        hb = symm.rendezvous(self.recv, group)
        self.recv.zero_()
        self.buf = torch.zeros(2, self.world, R, _lib.HEAD_DIM, dtype=pool.dtype, device=pool.device)
        self.ptr_out = torch.tensor([int(x) for x in hb.buffer_ptrs], dtype=torch.int64, device=pool.device)
        self.seq = torch.zeros(2, dtype=torch.int32, device=pool.device)  # steps exchanged, error flag
        p = pool.p
        p.peer_out, p.peer_gather, p.peer_seq = self.ptr_out.data_ptr(), self.buf.data_ptr(), self.seq.data_ptr()
        p.peer_world, p.peer_rank = self.world, self.rank
        self._handles = (hb,)
        torch.cuda.synchronize(pool.device)
        dist.barrier(group)  # nobody stores into a buffer that its owner has not cleared yet

    def wait(self) -> None:
        """Make the current stream receive the rows of the last step from every rank."""
        import ctypes as C

        self._lib.call("pqhsa_wait_peers", C.byref(self.pool.p), self.pool._stream())

    def result(self, steps_done: int) -> torch.Tensor:
        """Rows of all ranks after ``steps_done`` steps: ``[world, R, 128]`` (a view, valid until the
        step after next)."""
        return self.buf[(steps_done - 1) & 1]

    def timed_out(self) -> bool:
        return bool(int(self.seq[1].item()) != 0)


class LocalPeerGroup:
    """The same exchange between several pools that live in ONE process on ONE GPU (shards of a
    layer stepped one after the other on the same stream): every pool plays a rank, the receive
    buffers are ordinary device tensors.  Used to exercise the exchange protocol without a second
    GPU; the kernels are the ones the multi-GPU path runs."""

    def __init__(self, pools, wait_polls: int = 0):
        from . import _lib

        self._lib, self.pools = _lib, list(pools)
        self.world = len(self.pools)
        p0 = self.pools[0]
        R = p0.S * p0.G
        if any(p.S * p.G != R or p.dtype != p0.dtype or p.device != p0.device for p in self.pools):
            raise ValueError("all pools of a local peer group need the same row count, dtype and device")
        dev = p0.device
        words = _lib.HEAD_DIM * torch.empty(0, dtype=p0.dtype).element_size() // 4
        self.recv = [torch.zeros(2, self.world, R, words, 2, dtype=torch.int32, device=dev) for _ in self.pools]
        self.bufs = [torch.zeros(2, self.world, R, _lib.HEAD_DIM, dtype=p0.dtype, device=dev) for _ in self.pools]
        self.seqs = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in self.pools]
        self.ptr_out = torch.tensor([b.data_ptr() for b in self.recv], dtype=torch.int64, device=dev)
        for r, pool in enumerate(self.pools):
            p = pool.p
            p.peer_out, p.peer_gather, p.peer_seq = self.ptr_out.data_ptr(), self.bufs[r].data_ptr(), self.seqs[r].data_ptr()
            p.peer_world, p.peer_rank, p.peer_wait_polls = self.world, r, int(wait_polls)

    def wait(self, rank: int) -> None:
        import ctypes as C

        pool = self.pools[rank]
        self._lib.call("pqhsa_wait_peers", C.byref(pool.p), pool._stream())

    def result(self, rank: int, steps_done: int) -> torch.Tensor:
        return self.bufs[rank][(steps_done - 1) & 1]

    def timed_out(self, rank: int) -> bool:
        return bool(int(self.seqs[rank][1].item()) != 0)
