"""Multi-GPU decode: one process per GPU, ``torch.distributed`` (NCCL over NVLink) for the
only exchange the path has.

* KV-head sharding: a KV head and its query group never interact with another head
  (gqa_decode/gqa_decode.py:58-65 of the reference: each query head attends over its own KV
  head), so rank r simply runs the single-GPU kernels on its heads.  No collective.
* Sequence sharding: rank r holds a contiguous slice of the keys of every head, produces
  a normalised fp32 output and a log-sum-exp per query head, the ranks all-gather those
  (Hq * (D + 1) floats each) and every rank merges them with the LSE-weighted merge
  kernel - the same algebra as the reference's split-K reduction
  (gqa_decode/gqa_decode.py:661-669), one level up.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from ._native import trace_range as _trace_range


def next_epoch(epoch: int) -> int:
    """Epoch of the step after `epoch`.  Epochs are 32-bit, never 0 (0 means "no step yet" in
    the flag words) and alternate in parity (the parity selects one of two buffer halves):
    after 0xFFFFFFFF (odd) comes 2 (even), the same on every rank."""
    return epoch + 1 if epoch < 0xFFFFFFFF else 2


def _refuse_capture(what: str) -> None:
    """Steps that hand data to other GPUs carry a fresh epoch (and buffer half) chosen on the
    host each time; a CUDA graph would replay one epoch forever, find the flags already equal
    to it and read stale peer data.  Such steps must run eagerly."""
    if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        raise RuntimeError(f"{what} cannot be captured in a CUDA graph: every step needs a new epoch")


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced [begin, end) of `total` items for `rank` (first ranks get the
    remainder)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_kv_heads(num_q_heads: int, num_kv_heads: int, world: int, rank: int):
    """Slices of (query heads, KV heads) owned by `rank`; KV heads must divide evenly so
    every rank keeps whole query groups."""
    if num_kv_heads % world:
        raise ValueError("num_kv_heads must be divisible by the number of ranks")
    g = num_q_heads // num_kv_heads
    per = num_kv_heads // world
    return slice(rank * per * g, (rank + 1) * per * g), slice(rank * per, (rank + 1) * per)


def _native_local(q, k, v, seq_lens, **kw):
    from .gqa_decode import gqa_decode_attention_batched

    _, o32, lse = gqa_decode_attention_batched(q, k, v, seq_lens, return_f32=True, return_lse=True, **kw)
    return o32, lse


def _native_merge(o_parts, lse_parts, out_dtype):
    from .gqa_decode import merge_partials

    return merge_partials(o_parts, lse_parts, out_dtype=out_dtype)


class NvlinkExchange:
    """Symmetric receive buffers + the fused push/merge kernel (``gqa_exchange_merge``) for
    sequence-sharded decode: one kernel per rank replaces two NCCL all-gathers and a merge
    launch.  Collective constructor: every rank of ``group`` must create it with the same
    ``rows`` (= batch * num_q_heads) and ``head_dim``.  Ranks must be separate processes on
    separate GPUs of one NVLink domain.  Plain peer loads/stores only (no multicast)."""

    def __init__(self, rows: int, head_dim: int, device, group: Optional[dist.ProcessGroup] = None,
                 wait_limit_ns: int = 0):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import _native

        self._lib = _native.load()
        self._native = _native
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.rows, self.head_dim = int(rows), int(head_dim)
        self.device = torch.device(device)
        nbytes = int(self._lib.gqa_exchange_buffer_bytes(self.world, self.rows, self.head_dim))
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buf.zero_()  # flags start at 0; epochs start at 1
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.epoch = 0
        self.wait_limit_ns = int(wait_limit_ns)  # 0: the library's default of two seconds
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every buffer is zeroed before anybody pushes into it
        self._ctypes = ctypes

    def merge(self, o32: torch.Tensor, lse: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """o32 ``[rows, D]`` float32 and lse ``[rows]`` float32: this rank's partial.  Returns
        the merged ``[rows, D]`` in ``out_dtype`` (same on every rank)."""
        n = self._native
        o32, lse = o32.contiguous(), lse.contiguous()
        if o32.numel() != self.rows * self.head_dim or lse.numel() != self.rows:
            raise ValueError("partial does not match the exchange's rows/head_dim")
        if out is None:
            out = torch.empty(self.rows, self.head_dim, dtype=out_dtype, device=self.device)
        f32 = out.dtype == torch.float32
        _refuse_capture("NvlinkExchange.merge")
        self.epoch = next_epoch(self.epoch)
        code = {torch.bfloat16: n.DTYPE_BF16, torch.float16: n.DTYPE_FP16}.get(out.dtype, 0)
        with n.trace_range("gqa_decode:exchange_merge"):
            n.check(
                self._lib.gqa_exchange_merge(
                    o32.data_ptr(), lse.data_ptr(), self.handle.buffer_ptrs_dev, self.rank, self.world,
                    self.epoch, self.rows, self.head_dim, None if f32 else out.data_ptr(), code,
                    out.data_ptr() if f32 else None, None, self.status.data_ptr(), self.wait_limit_ns,
                    torch.cuda.current_stream(self.device).cuda_stream),
                "gqa_exchange_merge")
        return out

    def check(self) -> int:
        """Synchronise and return the status word (0 = ok, 16 = a peer never arrived)."""
        return int(self.status.item())


class HeadGather:
    """Head-sharded decode whose outputs land, inside the decode kernel itself, in every
    rank's ``[B, world * Hq_local, D]`` buffer (``gqa_decode_attention_gather``): the
    all-gather a tensor-parallel layer would run after attention disappears.  Final rows are
    written with plain peer stores; the kernel's last CTA raises this rank's flag on every
    peer and waits (bounded) for theirs, so ``decode()`` returns a tensor that is complete
    once the stream reaches that point.  Two output buffers alternate by step parity, so a
    rank may start step e+1 while a slower peer still reads step e.

    Collective constructor: every rank of ``group`` creates it with the same ``batch``,
    ``local_q_heads`` (query heads per rank), ``head_dim`` and ``dtype``.  One process per GPU,
    one NVLink domain, at most 8 ranks.  No multicast, no NVLS."""

    def __init__(self, batch: int, local_q_heads: int, head_dim: int, dtype: torch.dtype, device,
                 group: Optional[dist.ProcessGroup] = None):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import _native

        _native.load()
        self._native, self._ctypes = _native, ctypes
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("at most 8 ranks can gather head-sharded outputs")
        self.device = torch.device(device)
        self.shape = (int(batch), self.world * int(local_q_heads), int(head_dim))
        elems = self.shape[0] * self.shape[1] * self.shape[2]
        self.out = symm_mem.empty(2 * elems, dtype=dtype, device=self.device)
        self.flags = symm_mem.empty(2 * self.world, dtype=torch.int32, device=self.device)
        self.flags.zero_()  # epochs start at 1
        self._out_handle = symm_mem.rendezvous(self.out, self.group)
        self._flag_handle = symm_mem.rendezvous(self.flags, self.group)
        esz = self.out.element_size()
        ptr_array = ctypes.c_void_p * self.world
        # [parity] -> host array of every rank's output buffer for that parity
        self._peer_out = [
            ptr_array(*[int(self._out_handle.buffer_ptrs[r]) + par * elems * esz
                        for r in range(self.world)]) for par in (0, 1)]
        self._peer_flags = ptr_array(*[int(self._flag_handle.buffer_ptrs[r]) for r in range(self.world)])
        self.epoch = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every flag array is zeroed before anybody raises a flag in it

    def _next(self, g):
        """Advance to the next step: bump the epoch and point `g` at that parity's buffers."""
        ctypes = self._ctypes
        _refuse_capture("HeadGather")
        self.epoch = next_epoch(self.epoch)
        par = self.epoch & 1
        g.peer_out = ctypes.cast(self._peer_out[par], ctypes.POINTER(ctypes.c_void_p))
        g.peer_flags = ctypes.cast(self._peer_flags, ctypes.POINTER(ctypes.c_void_p))
        g.world, g.rank, g.epoch = self.world, self.rank, self.epoch
        g.mode = self._native.GATHER_HEADS
        elems = self.shape[0] * self.shape[1] * self.shape[2]
        return self.out[par * elems:(par + 1) * elems].view(self.shape)

    def plan(self, q_local, k_local, v_local, seq_lens=None, **kw):
        """Validate once; the returned callable runs one step (one C call) and returns the
        gathered ``[B, world * Hq_local, D]`` tensor of that step."""
        from .gqa_decode import plan_decode

        g = self._native.GatherArgs()
        before = self.epoch
        self._next(g)
        self.epoch = before  # nothing ran yet
        inner = plan_decode(q_local, k_local, v_local, seq_lens, _gather=g, **kw)

        def run():
            view = self._next(g)
            inner.run()
            return view

        run.status = inner.status  # synchronise and read the step's status word
        return run

    def decode(self, q_local, k_local, v_local, seq_lens=None, **kw) -> torch.Tensor:
        """q_local ``[B, Hq_local, D]``, k/v the local KV heads (any layout that
        :func:`gqa_decode_attention_batched` accepts).  Returns ``[B, world * Hq_local, D]``:
        rank r's heads at ``[:, r * Hq_local:(r + 1) * Hq_local]`` (valid until the step after
        next overwrites the buffer)."""
        from .gqa_decode import gqa_decode_attention_batched

        n = self._native
        if tuple(q_local.shape) != (self.shape[0], self.shape[1] // self.world, self.shape[2]):
            raise ValueError("q_local does not match the gather's batch / heads / head_dim")
        if q_local.dtype != self.out.dtype:
            raise ValueError("q dtype does not match the gather's dtype")
        g = n.GatherArgs()
        view = self._next(g)
        gqa_decode_attention_batched(q_local, k_local, v_local, seq_lens, _gather=g, **kw)
        return view


class FusedSequenceExchange:
    """Sequence-sharded decode in ONE kernel per rank and step
    (``gqa_decode_attention_gather`` with ``GQA_GATHER_SEQUENCE``): while a rank streams its
    slice of the keys, every finished row (normalised fp32 output + log-sum-exp) is pushed into
    all ranks' receive areas with plain peer stores, each value tagged with the step's epoch so
    that the data is its own arrival flag; the kernel's tail merges the ``world`` partials into
    the final output, waiting (bounded) for values that have not landed yet.  Replaces
    decode kernel + :class:`NvlinkExchange` kernel (or two NCCL all-gathers + merge).

    Collective constructor (same ``batch``, ``num_q_heads``, ``head_dim`` on every rank); one
    process per GPU of one NVLink domain, at most 8 ranks.  No multicast, no NVLS."""

    def __init__(self, batch: int, num_q_heads: int, head_dim: int, device,
                 group: Optional[dist.ProcessGroup] = None):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import _native

        _native.load()
        self._native, self._ctypes = _native, ctypes
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        self.device = torch.device(device)
        self.shape = (int(batch), int(num_q_heads), int(head_dim))
        rows = self.shape[0] * self.shape[1]
        nbytes = int(_native.load().gqa_sequence_exchange_bytes(self.world, rows, self.shape[2]))
        self.recv = symm_mem.empty(nbytes // 4, dtype=torch.float32, device=self.device)
        self.recv.zero_()  # every word's epoch tag starts at 0; epochs start at 1
        self.flags = symm_mem.empty(2 * self.world, dtype=torch.int32, device=self.device)
        self.flags.zero_()
        self._recv_handle = symm_mem.rendezvous(self.recv, self.group)
        self._flag_handle = symm_mem.rendezvous(self.flags, self.group)
        ptr_array = ctypes.c_void_p * self.world
        self._peer_recv = ptr_array(*[int(self._recv_handle.buffer_ptrs[r]) for r in range(self.world)])
        self._peer_flags = ptr_array(*[int(self._flag_handle.buffer_ptrs[r]) for r in range(self.world)])
        self.epoch = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def _next(self, g):
        ctypes = self._ctypes
        _refuse_capture("FusedSequenceExchange")
        self.epoch = next_epoch(self.epoch)
        g.peer_out = ctypes.cast(self._peer_recv, ctypes.POINTER(ctypes.c_void_p))
        g.peer_flags = ctypes.cast(self._peer_flags, ctypes.POINTER(ctypes.c_void_p))
        g.world, g.rank, g.epoch = self.world, self.rank, self.epoch
        g.mode = self._native.GATHER_SEQUENCE

    def decode(self, q, k_shard, v_shard, seq_lens_shard=None, **kw) -> torch.Tensor:
        """q ``[B, Hq, D]`` (identical on all ranks), k/v this rank's keys of every head,
        ``seq_lens_shard`` how many of them are valid (0 allowed).  Returns the full output
        ``[B, Hq, D]`` on every rank."""
        from .gqa_decode import gqa_decode_attention_batched

        if tuple(q.shape) != self.shape:
            raise ValueError("q does not match the exchange's batch / heads / head_dim")
        g = self._native.GatherArgs()
        self._next(g)
        return gqa_decode_attention_batched(q, k_shard, v_shard, seq_lens_shard, _gather=g, **kw)

    def plan(self, q, k_shard, v_shard, seq_lens_shard=None, **kw):
        """Validate once; the returned callable runs one step (one C call) and returns the
        output tensor (the same storage every step)."""
        from .gqa_decode import plan_decode

        g = self._native.GatherArgs()
        before = self.epoch
        self._next(g)
        self.epoch = before  # nothing ran yet
        inner = plan_decode(q, k_shard, v_shard, seq_lens_shard, _gather=g, **kw)

        def run():
            self._next(g)
            return inner.run()

        run.status = inner.status  # synchronise and read the step's status word
        return run


def sequence_sharded_decode(
    q: torch.Tensor,
    k_shard: torch.Tensor,
    v_shard: torch.Tensor,
    seq_lens_shard: Optional[torch.Tensor] = None,
    *,
    group: Optional[dist.ProcessGroup] = None,
    local_fn: Callable = _native_local,
    merge_fn: Callable = _native_merge,
    exchange: Optional["NvlinkExchange"] = None,
    **kw,
) -> torch.Tensor:
    """Decode step when every rank holds a contiguous slice of each sequence's keys.

    With ``exchange`` (an :class:`NvlinkExchange`) the partials travel by peer stores inside
    one fused push+merge kernel; otherwise by one NCCL all-gather followed by the merge kernel.

    q ``[B, Hq, D]`` (identical on all ranks); k_shard/v_shard ``[B, Hkv, S_r, D]`` (this
    rank's keys; ``seq_lens_shard`` gives how many of them are valid, 0 allowed).
    Returns the full output ``[B, Hq, D]`` on every rank.  ``local_fn`` / ``merge_fn``
    exist so the plumbing can be exercised on CPU ranks (gloo) in tests; the defaults are
    the CUDA kernels.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    with _trace_range("gqa_decode:local_partial"):
        o32, lse = local_fn(q, k_shard, v_shard, seq_lens_shard, **kw)
    b, hq, d = o32.shape
    if exchange is not None:
        return exchange.merge(o32.reshape(b * hq, d), lse.reshape(b * hq), q.dtype).view(b, hq, d)
    if world == 1:
        return merge_fn(o32.reshape(1, b * hq, d), lse.reshape(1, b * hq), q.dtype).view(b, hq, d)
    # one message per rank: [B*Hq, D+1] = normalised output with its log-sum-exp appended
    mine = torch.cat([o32.reshape(b * hq, d), lse.reshape(b * hq, 1)], dim=1).contiguous()
    flat = torch.empty((world * b * hq, d + 1), dtype=mine.dtype, device=mine.device)
    with _trace_range("gqa_decode:all_gather"):
        dist.all_gather_into_tensor(flat, mine, group=group)  # rank-major concatenation
    gathered = flat.view(world, b * hq, d + 1)
    with _trace_range("gqa_decode:merge_partials"):
        out = merge_fn(gathered[:, :, :d].contiguous(), gathered[:, :, d].contiguous(), q.dtype)
    return out.view(b, hq, d)


def head_sharded_decode(
    q_local: torch.Tensor,
    k_local: torch.Tensor,
    v_local: torch.Tensor,
    seq_lens: Optional[torch.Tensor] = None,
    *,
    gather_output: bool = False,
    group: Optional[dist.ProcessGroup] = None,
    local_fn: Optional[Callable] = None,
    **kw,
) -> torch.Tensor:
    """Decode step when rank r owns KV heads (and their query groups) ``shard_kv_heads``.
    The path needs no exchange; ``gather_output=True`` all-gathers the head-sharded
    outputs into ``[B, Hq, D]`` for callers that want the whole tensor."""
    if local_fn is None:
        from .gqa_decode import gqa_decode_attention_batched as local_fn
    out = local_fn(q_local, k_local, v_local, seq_lens, **kw)
    if not gather_output or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return out
    world = dist.get_world_size(group)
    flat = torch.empty((world * out.shape[0],) + tuple(out.shape[1:]), dtype=out.dtype, device=out.device)
    dist.all_gather_into_tensor(flat, out.contiguous(), group=group)  # rank-major concatenation
    parts = flat.view((world,) + tuple(out.shape))
    return parts.permute(1, 0, 2, 3).reshape(out.shape[0], world * out.shape[1], out.shape[2])
