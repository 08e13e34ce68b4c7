"""Multi-GPU decode steps: one process per GPU, ``torch.distributed`` for the plumbing.

The reference is single-process and single-GPU (src/diffcache/base.py:28); it scales context by
offloading to host memory.  On an 8-GPU box the same step shards instead:

* :class:`SequenceShardedStep` — one very long sequence (1M tokens): the retrieval region is cut
  into contiguous row ranges, one per rank.  Per step every rank scans its rows and selects a
  local top-k, sorted; the ranking keys are all-gathered (k*4 bytes per kv head and rank) and
  every rank counts how long a prefix of its own list belongs to the global top-k (same total
  order, ties to the smaller global id, which for contiguous shards means to the lower rank); each
  rank then attends over that prefix (rank 0 adds the sink rows, the last rank the local window and the new
  token) and the un-normalised partial results ``(acc, max, sum)`` are all-gathered and merged by
  log-sum-exp.  No K/V row ever crosses NVLink.
* :func:`shard_rows` / :func:`shard_heads` — the partition arithmetic, shared with the tests.

The numerical work is delegated to a *backend* object so that the host logic (partitioning,
gather layouts, offsets) can be exercised on CPU ranks over gloo with a stand-in backend;
:class:`GpuShardBackend` is the real one (CUDA kernels through the C ABI).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib

PAD = 0xFFFFFFFF


class PeerExchange:
    """Exchange buffers of all ranks mapped into one another (CUDA IPC over ``torch.distributed``), for the
    fused exchange kernels behind ``dc_xchg_*`` / ``dc_sharded_*``: producers store their block into every
    peer's buffer over NVLink as (word, epoch) pairs, consumers poll their own buffer.  ``slot_bytes[c]`` is the
    block size of channel ``c`` per rank (multiples of 16).

    Construction is collective.  If any rank cannot map a peer (no peer access, IPC not permitted) every
    rank raises ``RuntimeError`` and the caller keeps using the NCCL all-gathers."""

    def __init__(self, slot_bytes: Sequence[int], device: int, group: Optional["dist.ProcessGroup"] = None,
                 _rank_world: Optional[Tuple[int, int]] = None):
        self.lib = _lib.load()
        if _rank_world is not None:   # wired by in_process()
            self.rank, self.world = _rank_world
        else:
            self.world = dist.get_world_size(group) if dist.is_initialized() else 1
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = int(device)
        self.slot_bytes = [int(b) for b in slot_bytes]
        arr = (ctypes.c_int64 * len(self.slot_bytes))(*self.slot_bytes)
        handle = ctypes.c_void_p()
        _lib.check(self.lib.dc_xchg_create(self.rank, self.world, self.device, arr, len(self.slot_bytes),
                                           ctypes.byref(handle)))
        self._h = handle
        if self.world > 1 and _rank_world is None:
            ok, why = 1, ""
            try:
                mine = ctypes.create_string_buffer(self.lib.dc_xchg_handle_bytes())
                _lib.check(self.lib.dc_xchg_get_handle(self._h, mine))
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(mine.raw), group=group)
                for r, raw in enumerate(handles):
                    if r != self.rank:
                        _lib.check(self.lib.dc_xchg_open_peer(self._h, r, raw))
            except Exception as exc:  # keep going to the collective vote below
                ok, why = 0, str(exc)
            vote = torch.tensor([ok], dtype=torch.int32, device=torch.device("cuda", self.device))
            dist.all_reduce(vote, op=dist.ReduceOp.MIN, group=group)
            if int(vote[0]) == 0:
                self.close()
                raise RuntimeError(f"peer exchange unavailable on at least one rank ({why or 'another rank failed'})")
            dist.barrier(group)

    @classmethod
    def in_process(cls, slot_bytes: Sequence[int], devices: Sequence[int]) -> List["PeerExchange"]:
        """One exchange per entry of ``devices``, all owned by this process and wired to one another by plain
        pointers (no IPC): several GPUs driven by one process, or several ranks emulated on one GPU.  With
        emulated ranks the caller must run the ranks phase by phase (all pushes of a phase before any wait
        for it): kernels of one GPU that wait for one another cannot be relied on to run concurrently."""
        world = len(devices)
        xs = [cls(slot_bytes, devices[r], _rank_world=(r, world)) for r in range(world)]
        for a in xs:
            for b in xs:
                if a is not b:
                    _lib.check(a.lib.dc_xchg_set_peer(a._h, b.rank, a.lib.dc_xchg_local(b._h)))
        return xs

    def push(self, channel: int, src: torch.Tensor, stream=None) -> None:
        st = int(torch.cuda.current_stream().cuda_stream) if stream is None else int(stream)
        _lib.check(self.lib.dc_xchg_push(self._h, channel, src.data_ptr(), src.numel() * src.element_size(), st))

    def push_rows(self, channel: int, src: torch.Tensor, stream=None) -> None:
        """``src`` ``(rows, n)`` contiguous: afterwards every rank's channel reads ``(rows, world, n)``."""
        st = int(torch.cuda.current_stream().cuda_stream) if stream is None else int(stream)
        rows = src.shape[0]
        _lib.check(self.lib.dc_xchg_push_rows(self._h, channel, src.data_ptr(), rows,
                                              src.numel() // rows * src.element_size(), st))

    def collect(self, channel: int, dst: torch.Tensor, stream=None) -> None:
        """Waits for the blocks of all ranks and writes them densely into ``dst`` (``world`` slots after
        :meth:`push`, ``(rows, world, n)`` after :meth:`push_rows`); ``dst`` must be exactly what was pushed."""
        st = int(torch.cuda.current_stream().cuda_stream) if stream is None else int(stream)
        _lib.check(self.lib.dc_xchg_collect(self._h, channel, dst.data_ptr(), dst.numel() * dst.element_size(), st))

    def check(self) -> None:
        """Synchronises the current stream; raises if a wait for peer data ran out of time."""
        _lib.check(self.lib.dc_xchg_check(self._h, int(torch.cuda.current_stream().cuda_stream)))

    def set_timeout_ms(self, ms: int) -> None:
        _lib.check(self.lib.dc_xchg_set_timeout_ms(self._h, int(ms)))

    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self.lib.dc_xchg_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def shard_rows(n_rows: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous (start, length) row ranges, lengths differing by at most one 16-row block so
    that every shard start stays aligned; covers [0, n_rows) exactly."""
    block = 16
    blocks = (n_rows + block - 1) // block
    out, start = [], 0
    for r in range(world):
        nb = blocks // world + (1 if r < blocks % world else 0)
        length = max(0, min(n_rows - start, nb * block))
        out.append((start, length))
        start += length
    assert start == n_rows
    return out


def shard_heads(kv_heads: int, world: int) -> List[Tuple[int, int]]:
    """KV-head sharding (one layer stack replicated over ranks, each owning a head range)."""
    if kv_heads % world != 0:
        raise ValueError(f"kv_heads={kv_heads} is not divisible by world={world}")
    per = kv_heads // world
    return [(r * per, per) for r in range(world)]


def _adjacent(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``stack([a, b])``; free when ``b`` already sits right behind ``a`` in one allocation."""
    if (a.is_contiguous() and b.is_contiguous() and a.dtype == b.dtype and a.shape == b.shape
            and a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr()
            and b.storage_offset() == a.storage_offset() + a.numel()):
        return torch.as_strided(a, (2,) + tuple(a.shape), (a.numel(),) + tuple(a.stride()))
    return torch.stack([a, b])


def _adjacent_flat(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``cat([a.flatten(), b.flatten()])``; free when ``b`` sits right behind ``a`` in one allocation."""
    if (a.is_contiguous() and b.is_contiguous() and a.dtype == b.dtype
            and a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr()
            and b.storage_offset() == a.storage_offset() + a.numel()):
        return torch.as_strided(a, (a.numel() + b.numel(),), (1,))
    return torch.cat([a.reshape(-1), b.reshape(-1)])


class SequenceShardedStep:
    """Sequence-sharded fused decode step.  ``backend`` provides

    ``local_topk(q, k) -> (bits, gidx)``  int32/uint32-pattern tensors ``(P, k)``, padded with 0xFFFFFFFF
    ``merge(bits_all, gidx_all, k) -> sel``  ``(P, k)`` global row ids from ``(P, world*k)`` candidates
    ``merge_count(bits_all, k, rank) -> count``  ``(P,)`` int32 from the gathered ``(world, P, k)`` keys: how many
    leading entries of this rank's own list are among the global k best
    ``attend_owned(q, ids, count=None) -> (acc, ml)``  fp32 ``(P*G, D)`` and ``(P*G, 2)`` over the owned rows of
    ``ids`` (the first ``count[p]`` of them when given)
    ``combine_packed(parts, rows, D) -> out``  from ``(world, rows*D + rows*2)``: per rank the accumulators
    followed by the (max, sum) pairs
    """

    def __init__(self, backend, topk: int, group: Optional["dist.ProcessGroup"] = None, exchange: str = "nccl"):
        """``exchange``: "nccl" — two ``all_gather_into_tensor`` calls per step; "peer" — the exchanges are
        done by the step's own kernels with stores over NVLink (:class:`PeerExchange`; GPU backend only, the
        whole step is one C call); "auto" — "peer" when it can be set up, else "nccl"."""
        self.backend = backend
        self.topk = topk
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.xchg = None
        if exchange in ("peer", "auto") and hasattr(backend, "make_exchange"):
            try:
                self.xchg = backend.make_exchange(topk, group)
            except RuntimeError:
                if exchange == "peer":
                    raise
        elif exchange == "peer":
            raise ValueError("the peer exchange needs the GPU backend")
        self.exchange = "peer" if self.xchg is not None else "nccl"

    def _all_gather(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t.unsqueeze(0)
        flat = t.contiguous().view(-1)
        out = torch.empty(self.world * flat.numel(), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, flat, group=self.group)
        return out.view((self.world,) + tuple(t.shape))

    #: dc_merge_sorted_count keeps all ranks' lists in shared memory
    PREFIX_MERGE_MAX_BYTES = 200 * 1024

    def step(self, q: torch.Tensor, want_selection: bool = False) -> torch.Tensor:
        """Two exchanges per step: the candidates and the partial attention results (one buffer holding
        accumulators and (max, sum) pairs).

        Every rank's candidate list is sorted, so the global winners a rank owns are a prefix of its own
        list: only the ranking keys are exchanged, each rank computes the length of its prefix
        (``merge_count``) and attends over it.  ``want_selection`` (and lists too long for that kernel)
        also exchange the ids and run the full merge select, which leaves the global row list, identical
        on all ranks, in ``last_selection``."""
        k = self.topk
        if self.xchg is not None and not want_selection:
            return self.backend.peer_step(q, k, self.xchg)               # five kernels, no collective call
        bits, gidx = self.backend.local_topk(q, k)                       # (P, k) each, ascending, padded
        P = bits.shape[0]
        use_prefix = self.world * k * 4 <= self.PREFIX_MERGE_MAX_BYTES and hasattr(self.backend, "merge_count")
        sel = None
        bits_all = None
        if want_selection or not use_prefix:
            packed = _adjacent(bits, gidx)                               # (2, P, k) without a copy when possible
            cand = self._all_gather(packed)                              # (world, 2, P, k)
            bits_all = cand[:, 0]
            flat = cand.permute(1, 2, 0, 3).reshape(2, P, self.world * k).contiguous()
            sel = self.backend.merge(flat[0], flat[1], k)                # (P, k) global ids
            self.last_selection = sel
        if use_prefix:
            if bits_all is None:
                bits_all = self._all_gather(bits)                        # (world, P, k)
            count = self.backend.merge_count(bits_all.contiguous(), k, self.rank)   # (P,) int32
            self.last_owned = (gidx, count)
            acc, ml = self.backend.attend_owned(q, gidx, count)
        else:
            acc, ml = self.backend.attend_owned(q, sel)
        rows, D = acc.shape
        flat = _adjacent_flat(acc, ml)                                   # [acc | ml] as one flat buffer
        parts = self._all_gather(flat)                                   # (world, rows*D + rows*2)
        return self.backend.combine_packed(parts, rows, D)


class GpuShardBackend:
    """One rank's share of a sequence-sharded step on its GPU (kernels through the C ABI)."""

    def __init__(self, engine, row_offset: int, res_k=None, res_v=None, res_len: int = 0, k_new=None, v_new=None,
                 scale: float = 0.0):
        self.e = engine
        self.e.set_row_offset(row_offset)
        self.res_k, self.res_v, self.res_len = res_k, res_v, res_len
        self.k_new, self.v_new = k_new, v_new
        self.scale = scale
        self.lib = _lib.load()
        self.P = engine.bsz * engine.kv_head_num
        self.G = engine.group
        self.D = engine.head_dim
        dev = torch.device("cuda", engine.device)
        self.dev = dev
        self._bufs = {}
        self.status = torch.zeros(int(self.lib.dc_select_scratch_bytes(self.P)), dtype=torch.uint8, device=dev)

    def _buf(self, name, shape, dtype):
        key = (name, tuple(shape), dtype)
        if key not in self._bufs:
            self._bufs[key] = torch.empty(shape, dtype=dtype, device=self.dev)
        return self._bufs[key]

    @staticmethod
    def _stream() -> int:
        return int(torch.cuda.current_stream().cuda_stream)

    def make_exchange(self, topk: int, group=None) -> PeerExchange:
        need = (ctypes.c_int64 * 2)()
        _lib.check(self.lib.dc_sharded_slot_bytes(self.e._h, int(topk), need))
        return PeerExchange([int(need[0]), int(need[1])], self.e.device, group)

    def _res_args(self):
        sb = sh = 0
        if self.res_k is not None:
            st = tuple(self.res_k.stride())
            sb, sh = st[0], st[1]
        ptr = lambda t: None if t is None else t.data_ptr()  # noqa: E731
        return ptr(self.k_new), ptr(self.v_new), ptr(self.res_k), ptr(self.res_v), sb, sh, int(self.res_len)

    def peer_step(self, q, k, xchg: PeerExchange):
        """The whole step as one call: scan, select + key fan-out | prefix count (polls the keys), attention, split
        merge + partial fan-out + final merge (polls the partials).  ``k`` must be even.  Every rank must run on
        its own GPU: the last kernel waits for what the same kernel of the other ranks sends."""
        out = self._buf("out", (self.e.bsz, self.e.q_head_num, self.D), torch.bfloat16 if self.e.dtype == 0 else torch.float16)
        kn, vn, rk, rv, sb, sh, rl = self._res_args()
        _lib.check(self.lib.dc_sharded_decode_attend(self.e._h, xchg._h, q.data_ptr(), kn, vn, rk, rv, sb, sh, rl, int(k),
                                                     float(self.scale), out.data_ptr(), None, self._stream()))
        return out

    def peer_phase(self, phase: int, q, k, xchg: PeerExchange):
        """One of the three phases of :meth:`peer_step` (0 local, 1 attend, 2 combine), for drivers that
        hold several ranks in one process and must run them phase by phase."""
        if phase == 0:
            _lib.check(self.lib.dc_sharded_local(self.e._h, xchg._h, q.data_ptr(), int(k), self._stream()))
            return None
        if phase == 1:
            kn, vn, rk, rv, sb, sh, rl = self._res_args()
            _lib.check(self.lib.dc_sharded_attend(self.e._h, xchg._h, q.data_ptr(), kn, vn, rk, rv, sb, sh, rl,
                                                  float(self.scale), self._stream()))
            return None
        out = self._buf("out", (self.e.bsz, self.e.q_head_num, self.D), torch.bfloat16 if self.e.dtype == 0 else torch.float16)
        _lib.check(self.lib.dc_sharded_combine(self.e._h, xchg._h, out.data_ptr(), None, self._stream()))
        return out

    def trace_step(self, q, k, xchg: PeerExchange):
        """One peer step with an event after every kernel; returns the intervals in microseconds, in order:
        scan, select, key push, prefix count (incl. its wait for the keys), attention + split merge, partial
        push, merge (incl. its wait for the partials)."""
        _lib.check(self.lib.dc_trace_begin(self.e._h, 16))
        self.peer_step(q, k, xchg)
        vals = (ctypes.c_float * 16)()
        n = ctypes.c_int()
        _lib.check(self.lib.dc_trace_read(self.e._h, vals, ctypes.byref(n)))
        return [vals[i] * 1e3 for i in range(max(0, n.value - 1))]

    def local_topk(self, q, k):
        both = self._buf("cand", (2, self.P, k), torch.int32)
        bits, gidx = both[0], both[1]
        self.e.local_topk(q, k, bits, gidx)
        return bits, gidx

    def merge(self, bits_all, gidx_all, k):
        n = bits_all.shape[1]
        sel = self._buf("sel", (self.P, k), torch.int32)
        _lib.check(self.lib.dc_topk_select(bits_all.data_ptr(), gidx_all.data_ptr(), n, self.P, n, k, None, None,
                                           sel.data_ptr(), k, self.status.data_ptr(), self._stream()))
        return sel

    def merge_count(self, bits_all, k, rank):
        world = bits_all.shape[0]
        count = self._buf("count", (self.P,), torch.int32)
        _lib.check(self.lib.dc_merge_sorted_count(bits_all.data_ptr(), world, self.P, k, rank, count.data_ptr(),
                                                  self._stream()))
        return count

    def attend_owned(self, q, sel, count=None):
        rows = self.P * self.G
        flat = self._buf("partial", (rows * (self.D + 2),), torch.float32)
        acc = flat[:rows * self.D].view(rows, self.D)
        ml = flat[rows * self.D:].view(rows, 2)
        self.e.attend_owned(q, sel, sel.shape[1], acc, ml, res_k=self.res_k, res_v=self.res_v, res_len=self.res_len,
                            k_new=self.k_new, v_new=self.v_new, scale=self.scale, sel_count=count)
        return acc, ml

    def combine_packed(self, parts, rows, D):
        world = parts.shape[0]
        stride = rows * (D + 2)
        out = self._buf("out", (self.e.bsz, self.e.q_head_num, D), torch.bfloat16 if self.e.dtype == 0 else torch.float16)
        _lib.check(self.lib.dc_lse_combine(parts.data_ptr(), stride, parts.data_ptr() + rows * D * 4, stride, world, rows,
                                           D, self.e.dtype, out.data_ptr(), None, self._stream()))
        return out
