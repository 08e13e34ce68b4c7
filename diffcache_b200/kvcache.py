"""``DiffCache`` — the KV-cache manager API of src/diffcache/kvcache/diffcache.py, on HBM.

Constructor arguments, method names and the GPU buffer layout
``[retrieved (right-aligned, budget rows) | prefix | suffix ...]`` per layer are the
reference's (diffcache.py:16-66), so the model runner (src/diffcache/base.py) keeps
calling the same methods.  What changes is where the retrieval region lives: instead of
host DRAM behind a CPU engine it is an HBM store inside one ``DiffCacheGPU`` per layer,
so the query never leaves the device:

* ``prefill_update_kv_cache`` ingests the middle region device-to-device straight from the
  model's ``(B, S, Hkv, D)`` layout (no ``.cpu().numpy()``, no CAGRA graph build);
* ``decode_pre_query_operation`` copies the query into a persistent device buffer (the
  reference's pinned ``qbuf_cpu``, without the D2H hop), so it can sit inside a captured graph;
* ``decode_query_kvcache`` + ``decode_post_query_operation`` reproduce the reference's
  two-call shape (retrieved rows land in ``kbuf[:, :, budget-ef:budget]``) for callers that
  still run their own attention kernel;
* ``decode_attention`` is the fused replacement for query + copy + ``flash_attn_with_kvcache``.

CUDA graphs.  The reference captures, per layer, one graph ending in ``decode_pre_query_operation``
and one starting with ``decode_post_query_operation`` (src/diffcache/base.py:116-155) and calls
``decode_query_kvcache`` between their replays; both methods here only enqueue copies between
buffers allocated before capture, so that pattern keeps working.  ``decode_attention`` can be
captured once per layer for the whole generation: every length it depends on (rows in the store,
resident rows, the slot of the new token) lives in device words that its kernels read when they
run.  The suffix region is a ring there: when it is full, the oldest generated token moves into
the scanned store and the new one takes its slot (the reference asserts instead,
diffcache.py:221).  Host attributes (``kvbuf_suffix_len``, ``retrieval_region_len``) follow calls
made from Python; after graph replays ``sync_lengths()`` refreshes them from the device.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional

import torch

from .engine import DiffCacheGPU, init_metrics

_TORCH_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16}


class DiffCache:
    def __init__(
        self,
        num_layers: int,
        batch_size: int,
        max_length: int,
        num_kv_heads: int,
        num_q_heads: int,
        head_dim: int,
        retrieval_budget: int,
        nsw_m: int = 16,
        nsw_ef_cons: int = 200,
        kvbuf_prefix_len: int = 128,
        kvbuf_suffix_len: int = 128,
        kvbuf_suffix_maxlen: int = 512,
        attn_mass_threshold: float = 0.9,
        k_check_seq: Optional[List[int]] = None,
        r_sq: Optional[List[List[float]]] = None,
        dtype: str = "bf16",
        device: Optional[int] = None,
        adaptive_budget: bool = False,
    ) -> None:
        self.num_layers = num_layers
        self.batch_size = batch_size
        self.max_length = max_length
        self.num_kv_heads = num_kv_heads
        self.num_q_heads = num_q_heads
        self.head_dim = head_dim
        self.retrieval_budget = retrieval_budget
        self.nsw_m = nsw_m
        self.nsw_ef_cons = nsw_ef_cons
        self.r_sq = r_sq if r_sq is not None else [[4.0] * num_kv_heads for _ in range(num_layers)]
        self.retrieval_region_len = 0
        self.kvbuf_suffix_maxlen = kvbuf_suffix_maxlen
        self.kvbuf_prefix_len = kvbuf_prefix_len
        self.kvbuf_suffix_len = kvbuf_suffix_len
        self.dtype = dtype
        self.torch_dtype = _TORCH_DTYPES[dtype]
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)

        buf_len = retrieval_budget + kvbuf_prefix_len + kvbuf_suffix_maxlen
        shape = (batch_size, num_kv_heads, buf_len, head_dim)
        self.kbuf = [torch.empty(shape, device=self.device, dtype=self.torch_dtype) for _ in range(num_layers)]
        self.vbuf = [torch.empty(shape, device=self.device, dtype=self.torch_dtype) for _ in range(num_layers)]
        # contiguous landing zone for the two-call query shape (the reference's pinned kbuf_cpu), allocated
        # when the retrieval length is known (end of prefill / load), i.e. before any graph capture
        self._stage_k = None
        self._stage_v = None
        # the reference's qbuf: decode_pre_query_operation copies into it, also when captured
        self._qbuf = torch.empty((batch_size, num_q_heads, head_dim), device=self.device, dtype=self.torch_dtype)
        # window-ring state read by the kernels of decode_attention:
        # {suffix_len, head, prefix_len, cap, res_len_now, steps, 0, 0}
        self._win = torch.zeros(8, dtype=torch.int32, device=self.device)

        self.data_layers = [
            DiffCacheGPU(
                bsz=batch_size,
                q_head_num=num_q_heads,
                kv_head_num=num_kv_heads,
                head_dim=head_dim,
                max_ctx_len=max_length,
                m=nsw_m,
                ef_cons=nsw_ef_cons,
                r_sq=self.r_sq[layer_idx],
                name=f"l{layer_idx:03d}",
                attn_mass_threshold=attn_mass_threshold,
                k_check_seq=k_check_seq if k_check_seq is not None else [1048576],
                use_bruteforce=True,
                adaptive_budget=adaptive_budget,
                dtype=dtype,
                device=self.device.index,
            )
            for layer_idx in range(num_layers)
        ]
        init_metrics()

    # ---- prefill -----------------------------------------------------------------------------
    def prefill_update_kv_cache(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int):
        """key/value_states ``(bsz, seq_len, num_kv_heads, head_dim)``; diffcache.py:149-184."""
        seq_len = key_states.size(1)
        budget = self.retrieval_budget
        r_sq = torch.einsum("bshd,bshd->bsh", key_states.float(), key_states.float()).amax(dim=(0, 1)).tolist()
        self.r_sq[layer_idx] = r_sq
        self.data_layers[layer_idx].update_r_sq(r_sq)

        prefix_len = min(self.kvbuf_prefix_len, seq_len)
        suffix_len = min(self.kvbuf_suffix_len, seq_len - prefix_len)
        for buf, states in ((self.kbuf[layer_idx], key_states), (self.vbuf[layer_idx], value_states)):
            buf[:, :, budget:budget + prefix_len].copy_(states[:, :prefix_len].permute(0, 2, 1, 3))
            buf[:, :, budget + prefix_len:budget + prefix_len + suffix_len].copy_(
                states[:, seq_len - suffix_len:seq_len].permute(0, 2, 1, 3))
        self.kvbuf_prefix_len = prefix_len
        self.kvbuf_suffix_len = suffix_len

        mid_k = key_states[:, prefix_len:seq_len - suffix_len]
        mid_v = value_states[:, prefix_len:seq_len - suffix_len]
        # (B, S', Hkv, D) -> logical (B, Hkv, S', D) view; the engine ingests it with strides
        self.data_layers[layer_idx].prefill(mid_k.permute(0, 2, 1, 3), mid_v.permute(0, 2, 1, 3), None)
        self.retrieval_region_len = mid_k.size(1)
        self._after_prefill()
        return key_states, value_states

    def _after_prefill(self) -> None:
        """Lengths are known: size the staging buffers and set the device-side window state."""
        ef = self._retrieval_len()
        if ef > 0 and (self._stage_k is None or self._stage_k.size(2) != ef):
            shape = (self.batch_size, self.num_kv_heads, ef, self.head_dim)
            self._stage_k = torch.empty(shape, device=self.device, dtype=self.torch_dtype)
            self._stage_v = torch.empty(shape, device=self.device, dtype=self.torch_dtype)
        p, sfx = self.kvbuf_prefix_len, self.kvbuf_suffix_len
        self._win.copy_(torch.tensor([sfx, 0, p, self.kvbuf_suffix_maxlen, p + sfx, 0, 0, 0], dtype=torch.int32))

    def sync_lengths(self) -> None:
        """Refresh the host attributes from the device words (after replays of a captured
        ``decode_attention`` graph, which advance the lengths without running any Python)."""
        w = self._win.cpu().tolist()
        self.kvbuf_suffix_len = int(w[0])
        self.retrieval_region_len = int(self.data_layers[0].ctx_len)

    # ---- views ---------------------------------------------------------------------------------
    def _retrieval_len(self) -> int:
        return min(self.retrieval_region_len, self.retrieval_budget)

    def get_kvcache(self, layer_idx: int):
        start = self.retrieval_budget - self._retrieval_len()
        return (self.kbuf[layer_idx][:, :, start:, :].permute(0, 2, 1, 3),
                self.vbuf[layer_idx][:, :, start:, :].permute(0, 2, 1, 3))

    def seq_len(self, layer_idx: int) -> int:
        return self.kvbuf_prefix_len + self.kvbuf_suffix_len + self.retrieval_region_len

    def seq_len_gpu(self, layer_idx: int) -> int:
        return self.kvbuf_prefix_len + self.kvbuf_suffix_len + self._retrieval_len()

    # ---- decode: the reference's three-call shape -------------------------------------------------
    def decode_pre_query_operation(self, queries: torch.Tensor) -> None:
        """diffcache.py:191-194 without the device->host hop: the query heads are copied into the
        persistent query buffer (the group mean is formed later, next to the scan).  The copy is an
        ordinary stream operation, so it is recorded when this call sits inside a graph capture
        (base.py:121-125) and every replay delivers that layer's fresh query."""
        self._qbuf.copy_(queries.view(self.batch_size, self.num_q_heads, self.head_dim), non_blocking=True)

    def decode_query_kvcache(self, layer_idx: int) -> None:
        """diffcache.py:211-223: top-``retrieval_len`` rows of this layer into the staging buffers.
        Called between the replays of the two per-layer graphs, like the reference's engine call."""
        ef = self._retrieval_len()
        if ef > 0:
            group = self.num_q_heads // self.num_kv_heads
            q = self._qbuf.view(self.batch_size, self.num_kv_heads, group, self.head_dim)
            q_mean = q.mean(dim=2).contiguous()
            if self._stage_k is None or self._stage_k.size(2) != ef:
                self._after_prefill()
            self.data_layers[layer_idx].query(self._stage_k, self._stage_v, q_mean, ef)
        assert self.kvbuf_suffix_len < self.kvbuf_suffix_maxlen
        if layer_idx == self.num_layers - 1:
            self.kvbuf_suffix_len += 1

    def decode_post_query_operation(self, layer_idx: int) -> None:
        """diffcache.py:196-209: retrieved rows into ``kbuf[:, :, budget-ef:budget]`` (device to device)."""
        ef = self._retrieval_len()
        if ef <= 0:
            return
        if self._stage_k is None or self._stage_k.size(2) != ef:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("decode_post_query_operation captured before prefill / load_prefill_cache")
            self._after_prefill()
        b = self.retrieval_budget
        self.kbuf[layer_idx][:, :, b - ef:b].copy_(self._stage_k[:, :, :ef], non_blocking=True)
        self.vbuf[layer_idx][:, :, b - ef:b].copy_(self._stage_v[:, :, :ef], non_blocking=True)

    # ---- decode: fused -------------------------------------------------------------------------
    def decode_attention(self, layer_idx: int, queries: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                         out: Optional[torch.Tensor] = None, out_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One call for query + gather + attention of a layer (replaces diffcache.py:191-223 and
        the ``flash_attn_with_kvcache`` call of base.py:134-142).  ``queries`` ``(bsz, 1, Hq*D)`` or
        ``(bsz, Hq, D)``; ``k_new/v_new`` ``(bsz, 1, Hkv, D)`` or ``(bsz, Hkv, D)``: the new token is
        appended to the suffix region in place and attended.  The suffix length is advanced after
        the last layer, like the reference; when the suffix region is full, the oldest generated
        token moves into the scanned store and the new one takes its slot.

        The call may be captured in a CUDA graph (one per layer, inputs in static tensors) and
        replayed for every generated token: the lengths it works with are device words."""
        q = queries.reshape(self.batch_size, self.num_q_heads, self.head_dim)
        kn = k_new.reshape(self.batch_size, self.num_kv_heads, self.head_dim)
        vn = v_new.reshape(self.batch_size, self.num_kv_heads, self.head_dim)
        if out is None:
            out = torch.empty_like(q)
        b = self.retrieval_budget
        eng = self.data_layers[layer_idx]
        res_k, res_v = self.kbuf[layer_idx][:, :, b:], self.vbuf[layer_idx][:, :, b:]
        eng.window_push(kn, vn, res_k, res_v, self._win)
        eng.decode_attend_dyn(q, out, topk=self._retrieval_len(), res_k=res_k, res_v=res_v, res_len_dev=self._win[4:5],
                              res_cap=self.kvbuf_prefix_len + self.kvbuf_suffix_maxlen, out_idx=out_idx)
        if layer_idx == self.num_layers - 1:
            eng.window_advance(self._win)
            # host mirrors of what the kernels just did (exact for calls made from Python)
            if self.kvbuf_suffix_len < self.kvbuf_suffix_maxlen:
                self.kvbuf_suffix_len += 1
            elif self.retrieval_region_len < self.max_length:
                self.retrieval_region_len += 1
        return out

    # ---- prefill cache (checkpoint) ----------------------------------------------------------------
    def save_prefill_cache(self, prefill_cache_path: str) -> None:
        """Directory layout of diffcache.py:225-259: ``metadata.txt``, ``p_l_XXX/{k,v}.pt``,
        ``s_l_XXX/{k,v}.pt`` and one engine snapshot per layer under the ``d_l_XXX`` prefix."""
        meta = {
            "r_sq": self.r_sq,
            "kvbuf_prefix_len": self.kvbuf_prefix_len,
            "kvbuf_suffix_len": self.kvbuf_suffix_len,
            "retrieval_region_len": self.retrieval_region_len,
        }
        with open(os.path.join(prefill_cache_path, "metadata.txt"), "w") as f:
            json.dump(meta, f)
        b, p, s = self.retrieval_budget, self.kvbuf_prefix_len, self.kvbuf_suffix_len
        for tag, lo, hi in (("p", b, b + p), ("s", b + p, b + p + s)):
            for layer_idx in range(self.num_layers):
                layer_path = os.path.join(prefill_cache_path, f"{tag}_l_{layer_idx:03d}")
                os.makedirs(layer_path, exist_ok=False)
                torch.save(self.kbuf[layer_idx][:, :, lo:hi, :], os.path.join(layer_path, "k.pt"))
                torch.save(self.vbuf[layer_idx][:, :, lo:hi, :], os.path.join(layer_path, "v.pt"))
        for layer_idx in range(self.num_layers):
            layer_path = os.path.join(prefill_cache_path, f"d_l_{layer_idx:03d}")
            os.makedirs(layer_path, exist_ok=False)
            self.data_layers[layer_idx].save(layer_path)

    def load_prefill_cache(self, inputs_ids: torch.Tensor, prefill_cache_path: str) -> None:
        """diffcache.py:261-293."""
        ctx_len = inputs_ids.size(1)
        with open(os.path.join(prefill_cache_path, "metadata.txt")) as f:
            meta = json.load(f)
        self.r_sq = meta["r_sq"]
        self.kvbuf_prefix_len = meta["kvbuf_prefix_len"]
        self.kvbuf_suffix_len = meta["kvbuf_suffix_len"]
        self.retrieval_region_len = meta["retrieval_region_len"]
        b, p, s = self.retrieval_budget, self.kvbuf_prefix_len, self.kvbuf_suffix_len
        for layer_idx in range(self.num_layers):
            self.data_layers[layer_idx].update_r_sq(self.r_sq[layer_idx])
            for tag, lo, hi in (("p", b, b + p), ("s", b + p, b + p + s)):
                layer_path = os.path.join(prefill_cache_path, f"{tag}_l_{layer_idx:03d}")
                self.kbuf[layer_idx][:, :, lo:hi, :] = torch.load(os.path.join(layer_path, "k.pt"))
                self.vbuf[layer_idx][:, :, lo:hi, :] = torch.load(os.path.join(layer_path, "v.pt"))
            self.data_layers[layer_idx].load(os.path.join(prefill_cache_path, f"d_l_{layer_idx:03d}"), ctx_len)
        self._after_prefill()
