"""Host-side mirror of the reference engine class ``DiffCacheCPU``.

Same constructor, method names, argument meaning and error behaviour as the pyo3
class in diffcache_cpu/src/lib.rs:523-660, with the work done by the CUDA engine
behind the C ABI.  bf16 data crosses as ``uint16`` bit patterns exactly like the
reference (src/diffcache/kvcache/diffcache.py:81-84); every array argument may be
a numpy array (host) or a torch tensor (host or CUDA).
"""
from __future__ import annotations

import ctypes
import time
from typing import Optional, Sequence

import numpy as np

from . import _lib

BF16, FP16 = 0, 1

_OPTION_DEFAULTS = dict(  # diffcache_cpu/src/lib.rs:556-566
    max_ctx_len=1000000,
    m=16,
    ef_cons=200,
    r_sq=None,
    batch_search=False,
    name="l0",
    use_bruteforce=False,
    attn_mass_threshold=0.9,
    k_check_seq=[100, 200, 300, 400, 800, 1600, 3200, 6400, 12800, 25600],
)


def init_metrics() -> None:
    """Counterpart of ``diffcache._cpu.init_metrics`` (lib.rs:662-665).

    The reference installs a TCP exporter for its per-layer latency counters; this
    engine keeps the same counters, under the reference's names, in
    ``DiffCacheGPU.metrics`` instead, so there is nothing to install."""
    return None


def _metric_names(name: str) -> dict:
    """The reference's counters (microseconds for the latencies): ``{name}_num_searches`` and
    ``{name}_search_latency`` per (batch, kv-head) search (nsw.rs:595,618), ``{name}_collect_latency``
    (nsw.rs:660), ``{name}_total_query_latency`` per query call (lib.rs:403); ``{name}_num_queries``
    counts the calls."""
    return {f"{name}_{k}": 0 for k in ("num_queries", "num_searches", "search_latency", "collect_latency",
                                       "total_query_latency")}


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


def _ptr(x) -> Optional[int]:
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    if _is_torch(x):
        return x.data_ptr()
    if isinstance(x, int):
        return x
    raise TypeError(f"unsupported buffer type {type(x)}")


def _shape(x):
    return tuple(x.shape)


def _require_contiguous(x, what: str) -> None:
    ok = x.flags["C_CONTIGUOUS"] if isinstance(x, np.ndarray) else x.is_contiguous()
    if not ok:
        # the reference reshapes with into_shape_with_order(...).unwrap(), lib.rs:384-385
        raise ValueError(f"{what} must be C-contiguous")


def _require_u16(x, what: str) -> None:
    if isinstance(x, np.ndarray):
        if x.dtype != np.uint16:
            raise TypeError(f"{what}: expected uint16 bit patterns, got {x.dtype}")
    elif x.element_size() != 2:
        raise TypeError(f"{what}: expected a 16-bit element type, got {x.dtype}")


def _current_stream(stream) -> int:
    if stream is not None:
        return int(stream)
    import torch

    return int(torch.cuda.current_stream().cuda_stream)


class DiffCacheGPU:
    """``DiffCacheCPU(bsz, q_head_num, kv_head_num, head_dim, **kwargs)`` on a B200.

    Accepted kwargs are exactly the reference's (lib.rs:567-582): ``max_ctx_len, m,
    ef_cons, r_sq, batch_search, name, use_bruteforce, attn_mass_threshold,
    k_check_seq``; any other key raises (the reference panics with "Unknown option").
    The graph parameters are accepted and ignored: this engine always runs the exact
    scan, i.e. the reference's ``use_bruteforce=True`` semantics.  Two keyword-only
    additions select the element type and device: ``dtype`` ("bf16" | "fp16") and
    ``device`` (CUDA ordinal); ``adaptive_budget=True`` applies the reference's k-check
    (``k_check_seq``, ``attn_mass_threshold``) to the fused step."""

    def __init__(self, bsz: int, q_head_num: int, kv_head_num: int, head_dim: int, **kwargs):
        dtype = kwargs.pop("dtype", "bf16")
        device = kwargs.pop("device", None)
        adaptive = bool(kwargs.pop("adaptive_budget", False))
        opts = dict(_OPTION_DEFAULTS)
        for key, value in kwargs.items():
            if key not in opts:
                raise ValueError(f"Unknown option {key}")
            opts[key] = value
        if opts["r_sq"] is None:
            opts["r_sq"] = [4.0] * kv_head_num
        self.options = opts
        self.bsz, self.q_head_num, self.kv_head_num, self.head_dim = bsz, q_head_num, kv_head_num, head_dim
        self.dtype = {"bf16": BF16, "fp16": FP16, BF16: BF16, FP16: FP16}[dtype]
        if device is None:
            import torch

            device = torch.cuda.current_device()
        self.device = int(device)
        self.name = opts["name"]
        self.metrics = _metric_names(self.name)
        self._lib = _lib.load()
        handle = ctypes.c_void_p()
        _lib.check(self._lib.dc_create(bsz, q_head_num, kv_head_num, head_dim, int(opts["max_ctx_len"]), self.dtype,
                                       self.device, ctypes.byref(handle)))
        self._h = handle
        if adaptive:
            self.set_adaptive_budget(opts["k_check_seq"], opts["attn_mass_threshold"])

    # -- lifetime ------------------------------------------------------------------------
    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.dc_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def ctx_len(self) -> int:
        out = ctypes.c_int64()
        _lib.check(self._lib.dc_ctx_len(self._h, ctypes.byref(out)))
        return out.value

    @property
    def group(self) -> int:
        return self.q_head_num // self.kv_head_num

    # -- reference API ---------------------------------------------------------------------
    def prefill(self, keys, vals, neighbours=None, stream=None) -> None:
        """lib.rs:601-611.  keys/vals ``(bsz, kv_head_num, seq_len, head_dim)`` uint16
        (any strides whose last axis is contiguous); ``neighbours`` is accepted and
        ignored (it only feeds the reference's NSW graph)."""
        _require_u16(keys, "keys")
        _require_u16(vals, "vals")
        shp = _shape(keys)
        if len(shp) != 4 or shp[0] != self.bsz or shp[1] != self.kv_head_num or shp[3] != self.head_dim:
            raise ValueError(f"keys shape {shp} != (bsz, kv_head_num, seq_len, head_dim)")
        if _shape(vals) != shp:
            raise ValueError(f"vals shape {_shape(vals)} != keys shape {shp}")

        def strides(x):
            if isinstance(x, np.ndarray):
                st = tuple(s // x.itemsize for s in x.strides)
            else:
                st = tuple(x.stride())
            if st[3] != 1 and shp[3] > 1:
                raise ValueError("head_dim axis must be contiguous")
            return st

        sk, sv = strides(keys), strides(vals)
        if sk != sv:
            raise ValueError("keys and vals must share one stride pattern")
        _lib.check(self._lib.dc_prefill(self._h, _ptr(keys), _ptr(vals), shp[2], sk[0], sk[1], sk[2],
                                        _current_stream(stream)))

    def insert(self, keys, vals, stream=None) -> None:
        """lib.rs:591-599.  keys/vals ``(bsz, kv_head_num, head_dim)``."""
        for x, what in ((keys, "keys"), (vals, "vals")):
            _require_u16(x, what)
            _require_contiguous(x, what)
            if _shape(x) != (self.bsz, self.kv_head_num, self.head_dim):
                raise ValueError(f"{what} shape {_shape(x)} != (bsz, kv_head_num, head_dim)")
        _lib.check(self._lib.dc_insert(self._h, _ptr(keys), _ptr(vals), _current_stream(stream)))

    def query(self, out_keys, out_vals, queries, ef: int, out_idx=None, out_bits=None, stream=None) -> None:
        """lib.rs:613-624 with ``use_bruteforce`` semantics (nsw.rs:592-630).

        ``queries`` ``(bsz, kv_head_num, head_dim)``; ``out_keys/out_vals``
        ``(bsz, kv_head_num, min(ef, ctx_len), head_dim)`` C-contiguous; row ``i`` is the
        ``i``-th best key.  ``out_idx`` (int32) / ``out_bits`` (uint32) optionally receive the
        selected row ids and their ranking keys."""
        _require_u16(queries, "queries")
        _require_contiguous(queries, "queries")
        if _shape(queries) != (self.bsz, self.kv_head_num, self.head_dim):
            raise ValueError(f"queries shape {_shape(queries)} != (bsz, kv_head_num, head_dim)")
        ef_c = min(int(ef), self.ctx_len)
        for x, what in ((out_keys, "out_keys"), (out_vals, "out_vals")):
            if x is None:
                continue
            _require_u16(x, what)
            _require_contiguous(x, what)
            if _shape(x) != (self.bsz, self.kv_head_num, ef_c, self.head_dim):
                raise ValueError(f"{what} shape {_shape(x)} != (bsz, kv_head_num, {ef_c}, head_dim)")
        for x, what in ((out_idx, "out_idx"), (out_bits, "out_bits")):
            if x is not None:
                _require_contiguous(x, what)
                if _shape(x) != (self.bsz, self.kv_head_num, ef_c):
                    raise ValueError(f"{what} shape {_shape(x)} != (bsz, kv_head_num, {ef_c})")
        t0 = time.perf_counter()
        _lib.check(self._lib.dc_query(self._h, _ptr(queries), int(ef), _ptr(out_keys), _ptr(out_vals), _ptr(out_idx),
                                      _ptr(out_bits), _current_stream(stream)))
        # wall time of the call, as the reference measures it (lib.rs:378,403); with device outputs the call only
        # enqueues work, so device time has to come from set_phase_timing / phase_times
        self._count_query(int((time.perf_counter() - t0) * 1e6))

    def query_streaming(self, cuda_stream: int, out_keys_gpu: int, out_vals_gpu: int, queries, ef: int) -> None:
        """lib.rs:626-636: raw ``CUstream`` / device pointers as integers.  The reference
        streams chunks as its graph search converges; an exact scan has a single final
        answer, so this writes the complete result to the device buffers on ``cuda_stream``."""
        _require_u16(queries, "queries")
        _lib.check(self._lib.dc_query(self._h, _ptr(queries), int(ef), int(out_keys_gpu), int(out_vals_gpu), None, None,
                                      int(cuda_stream)))

    def _count_query(self, total_us: int = 0) -> None:
        m, n = self.metrics, self.name
        m[f"{n}_num_queries"] += 1
        m[f"{n}_num_searches"] += self.bsz * self.kv_head_num   # one search per (batch, kv head), nsw.rs:595
        m[f"{n}_total_query_latency"] += total_us

    def get_keys(self) -> np.ndarray:
        """lib.rs:646-649: stored keys as float32 ``(bsz, kv_head_num, ctx_len, head_dim)``."""
        out = np.empty((self.bsz, self.kv_head_num, self.ctx_len, self.head_dim), np.float32)
        _lib.check(self._lib.dc_get_keys(self._h, out.ctypes.data))
        return out

    def update_r_sq(self, r_sq: Sequence[float]) -> None:
        """lib.rs:651-659: validated and otherwise unused (r_sq never enters QKDist)."""
        arr = np.asarray(list(r_sq), np.float32)
        _lib.check(self._lib.dc_update_r_sq(self._h, arr.ctypes.data, int(arr.shape[0])))
        self.options["r_sq"] = [float(x) for x in arr]

    def save(self, path: str) -> None:
        """lib.rs:638-640.  Snapshot format: see :mod:`diffcache_b200.snapshot`."""
        from . import snapshot

        snapshot.save_engine(self, path)

    def load(self, path: str, ctx_len: int) -> None:
        """lib.rs:642-644."""
        from . import snapshot

        snapshot.load_engine(self, path, ctx_len)

    # -- fused device path -----------------------------------------------------------------
    def set_row_offset(self, row_offset: int) -> None:
        _lib.check(self._lib.dc_set_row_offset(self._h, int(row_offset)))

    def check_status(self, stream=None) -> None:
        _lib.check(self._lib.dc_check_status(self._h, _current_stream(stream)))

    def decode_attend(self, q, out, topk: int, res_k=None, res_v=None, res_len: int = 0, k_new=None, v_new=None,
                      scale: float = 0.0, out_idx=None, out_lse=None, stream=None) -> None:
        """One fused decode step on device tensors (see ``dc_decode_attend``).

        ``q``/``out`` ``(bsz, q_head_num, head_dim)``; ``res_k/res_v`` a view
        ``(bsz, kv_head_num, rows, head_dim)`` of the resident sink+window buffer whose first
        ``res_len`` rows are valid; ``k_new/v_new`` ``(bsz, kv_head_num, head_dim)``.  ``q``, ``k_new`` and
        ``v_new`` may be slices of a fused projection output: heads dense inside a batch, any batch stride
        (``k_new`` and ``v_new`` the same one)."""
        qsb = self._batch_stride(q, self.q_head_num, "q")
        nsb = 0
        if k_new is not None:
            nsb = self._batch_stride(k_new, self.kv_head_num, "k_new")
            if self._batch_stride(v_new, self.kv_head_num, "v_new") != nsb:
                raise ValueError("k_new and v_new must have the same batch stride")
        sb = sh = 0
        if res_k is not None:
            st = tuple(res_k.stride())
            if st != tuple(res_v.stride()) or st[3] != 1 or st[2] != self.head_dim:
                raise ValueError("res_k/res_v must share strides with contiguous rows of head_dim")
            sb, sh = st[0], st[1]
        _lib.check(self._lib.dc_decode_attend_strided(self._h, _ptr(q), qsb, _ptr(k_new), _ptr(v_new), nsb, _ptr(res_k),
                                                      _ptr(res_v), sb, sh, int(res_len), int(topk), float(scale),
                                                      _ptr(out), _ptr(out_idx), _ptr(out_lse), _current_stream(stream)))
        self._count_query()

    def set_output_exchange(self, exchange, channel: int = 0) -> None:
        """Head-sharded layers: every following ``decode_attend*`` call also stores its output slice into every
        rank's copy of ``channel`` of ``exchange`` (a :class:`diffcache_b200.sharded.PeerExchange`; ``None``
        switches it off), interleaved so that the channel reads ``(bsz, world, q_head_num * head_dim)``."""
        _lib.check(self._lib.dc_set_output_exchange(self._h, None if exchange is None else exchange._h, int(channel)))

    def set_output_gather(self, dense) -> None:
        """After :meth:`set_output_exchange`: the kernel that stores the slice also waits for every rank's slice
        and writes all of them to ``dense`` ``(bsz, world * q_head_num * head_dim)`` (a device tensor that must
        stay alive; ``None`` switches it off), so no separate ``PeerExchange.collect`` is needed.  Ranks must
        run on different GPUs."""
        _lib.check(self._lib.dc_set_output_gather(self._h, _ptr(dense)))
        self._out_dense = dense

    def window_push(self, k_new, v_new, res_k, res_v, window_state, stream=None) -> None:
        """Append the step's new token to this layer's window ring (see ``dc_window_push``): the oldest
        token is spilled into the scanned store once the window is full.  ``window_state`` is the int32
        device tensor of 8 words shared by all layers."""
        nsb = self._batch_stride(k_new, self.kv_head_num, "k_new")
        if self._batch_stride(v_new, self.kv_head_num, "v_new") != nsb:
            raise ValueError("k_new and v_new must have the same batch stride")
        st = tuple(res_k.stride())
        if st != tuple(res_v.stride()) or st[3] != 1 or st[2] != self.head_dim:
            raise ValueError("res_k/res_v must share strides with contiguous rows of head_dim")
        _lib.check(self._lib.dc_window_push(self._h, _ptr(k_new), _ptr(v_new), nsb, _ptr(res_k), _ptr(res_v), st[0], st[1],
                                            _ptr(window_state), _current_stream(stream)))

    def window_advance(self, window_state, stream=None) -> None:
        """Once per decode step, after the last layer's ``window_push``."""
        _lib.check(self._lib.dc_window_advance(_ptr(window_state), _current_stream(stream)))

    def decode_attend_dyn(self, q, out, topk: int, res_k, res_v, res_len_dev, res_cap: int, scale: float = 0.0,
                          out_idx=None, out_lse=None, stream=None) -> None:
        """``decode_attend`` with the resident length (``res_len_dev``, one int32 on the device) and the
        stored row count read on the device when the kernels run, so a captured graph of this call stays
        valid while the window and the store grow.  The new token must already be in the window."""
        qsb = self._batch_stride(q, self.q_head_num, "q")
        st = tuple(res_k.stride())
        if st != tuple(res_v.stride()) or st[3] != 1 or st[2] != self.head_dim:
            raise ValueError("res_k/res_v must share strides with contiguous rows of head_dim")
        _lib.check(self._lib.dc_decode_attend_dyn(self._h, _ptr(q), qsb, _ptr(res_k), _ptr(res_v), st[0], st[1],
                                                  _ptr(res_len_dev), int(res_cap), int(topk), float(scale), _ptr(out),
                                                  _ptr(out_idx), _ptr(out_lse), _current_stream(stream)))
        self._count_query()

    def _batch_stride(self, t, heads: int, what: str) -> int:
        """0 for a dense ``(bsz, heads, head_dim)`` tensor, else its batch stride in elements."""
        if not hasattr(t, "stride"):   # not a torch tensor: taken as dense
            return 0
        st, shape = tuple(t.stride()), tuple(t.shape)
        # the stride of a dimension of size 1 is never used and may hold anything
        if len(st) != 3 or (shape[2] != 1 and st[2] != 1) or (shape[1] != 1 and st[1] != self.head_dim):
            raise ValueError(f"{what} must be (bsz, {heads}, head_dim) with dense heads; strides {st}")
        return 0 if shape[0] == 1 or st[0] == heads * self.head_dim else int(st[0])

    def set_adaptive_budget(self, k_check_seq, attn_mass_threshold: float) -> None:
        """Switch the k-check on for ``decode_attend`` (``k_check_seq`` empty switches it off): per
        (batch, kv-head) the first checkpoint whose top-h keys already hold ``attn_mass_threshold`` of
        the estimated attention mass becomes the number of retrieved rows attended (nsw.rs:198-300)."""
        seq = np.asarray(sorted(int(x) for x in k_check_seq)[:16], np.int32)
        _lib.check(self._lib.dc_set_adaptive_budget(self._h, seq.ctypes.data if seq.size else None, int(seq.size),
                                                    float(attn_mass_threshold)))

    def last_budget(self) -> np.ndarray:
        """Budgets chosen by the last ``decode_attend`` step, ``(bsz, kv_head_num)`` int32."""
        out = np.zeros((self.bsz, self.kv_head_num), np.int32)
        _lib.check(self._lib.dc_get_budget(self._h, out.ctypes.data, _current_stream(None)))
        return out

    def set_phase_timing(self, max_steps: int) -> None:
        """Record CUDA events around the scan / select / attend phases of the next ``max_steps``
        ``decode_attend`` calls (the counterpart of the reference's per-layer latency counters)."""
        _lib.check(self._lib.dc_set_phase_timing(self._h, int(max_steps)))

    def phase_times(self) -> dict:
        """Summed milliseconds per phase over the recorded steps."""
        a, b, c, n = ctypes.c_float(), ctypes.c_float(), ctypes.c_float(), ctypes.c_int()
        _lib.check(self._lib.dc_get_phase_times(self._h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c),
                                                ctypes.byref(n)))
        # the device-timed phases under the reference's counter names: search = scan + select (nsw.rs:597-618),
        # collect = gather + attention of the selected rows (nsw.rs:620-629 and the attention that follows)
        m, nm = self.metrics, self.name
        m[f"{nm}_search_latency"] += int((a.value + b.value) * 1e3)
        m[f"{nm}_collect_latency"] += int(c.value * 1e3)
        m[f"{nm}_total_query_latency"] += int((a.value + b.value + c.value) * 1e3)
        return {"steps": n.value, "scan_ms": a.value, "select_ms": b.value, "attend_ms": c.value}

    def local_topk(self, q, topk: int, out_bits, out_gidx, stream=None) -> None:
        _lib.check(self._lib.dc_local_topk(self._h, _ptr(q), int(topk), _ptr(out_bits), _ptr(out_gidx),
                                           _current_stream(stream)))

    def attend_owned(self, q, sel_gidx, n_sel: int, out_acc, out_ml, res_k=None, res_v=None, res_len: int = 0,
                     k_new=None, v_new=None, scale: float = 0.0, stream=None, sel_count=None) -> None:
        sb = sh = 0
        if res_k is not None:
            st = tuple(res_k.stride())
            sb, sh = st[0], st[1]
        _lib.check(self._lib.dc_attend_owned(self._h, _ptr(q), _ptr(sel_gidx), int(n_sel), _ptr(k_new), _ptr(v_new),
                                             _ptr(res_k), _ptr(res_v), sb, sh, int(res_len), float(scale),
                                             _ptr(out_acc), _ptr(out_ml), _ptr(sel_count), _current_stream(stream)))
