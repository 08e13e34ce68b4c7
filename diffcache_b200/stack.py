"""Full-depth decode step: a Llama-3-8B-shaped attention stack over per-layer retrieval engines.

Every layer owns one ``DiffCacheGPU`` (as src/diffcache/kvcache/diffcache.py:87-100 owns one
engine per layer).  A decode step runs, per layer: RMSNorm -> fused q/k/v projection -> the fused
retrieval-attention step (scan, top-k, sparse attention incl. the new token) -> output projection
-> residual.  The projections are plain ``torch.nn.functional.linear`` calls with random-init
weights (they are not part of the retrieval path and the reference runs them through cuBLAS too,
src/diffcache/llama.py:181-195); the MLP is left out: the configuration asks for the attention stack.

With ``world > 1`` the stack is sharded by KV head: rank r owns kv heads
``[r*Hkv/world, (r+1)*Hkv/world)`` of every layer, the matching query heads and the matching
rows of the fused projection, so scan / select / attend are local; the per-layer exchange is one
all-gather of the attention output slice ``(B, Hq/world * D)`` before a replicated output
projection (deterministic: every rank computes the same residual stream).  That all-gather is
either an NCCL call or (``exchange="peer"``) done by the attention's own merge kernel: it stores the slice into
every rank's buffer over NVLink, interleaved so that the buffer reads ``(B, Hq*D)``, then waits for the other
ranks' slices and unpacks all of them for the projection (:class:`diffcache_b200.sharded.PeerExchange`,
``DiffCacheGPU.set_output_gather``); consecutive layers use different channels of the exchange so that a fast
rank never overwrites a block a slow rank is still reading.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import synth
from .engine import DiffCacheGPU
from .sharded import PeerExchange, shard_heads


class AttentionStack:
    def __init__(self, n_layers: int, hidden: int, batch: int, q_heads: int, kv_heads: int, head_dim: int,
                 context: int, topk: int, sink: int, window: int, dtype: str = "bf16", seed: int = 2000,
                 device: Optional[torch.device] = None, group: Optional["dist.ProcessGroup"] = None,
                 unsharded: bool = False, exchange: str = "nccl"):
        """``unsharded=True`` builds the whole stack on this device even inside a process group.
        ``exchange``: "nccl", "peer" or "auto" (peer when it can be set up)."""
        use_dist = dist.is_initialized() and not unsharded
        self.world = dist.get_world_size(group) if use_dist else 1
        self.rank = dist.get_rank(group) if use_dist else 0
        self.pg = group
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.n_layers, self.hidden, self.batch = n_layers, hidden, batch
        self.head_dim, self.topk = head_dim, topk
        h0, self.kv_local = shard_heads(kv_heads, self.world)[self.rank]
        g = q_heads // kv_heads
        self.q_local = self.kv_local * g
        self.q_heads, self.kv_heads = q_heads, kv_heads
        dt = synth.torch_dtype(dtype)
        n_r = context - sink - window
        self.res_rows = sink + window - 1
        self.engines, self.res_k, self.res_v, self.wqkv, self.wo, self.norm_w = [], [], [], [], [], []
        for layer in range(n_layers):
            wgen = torch.Generator(device=self.device).manual_seed(seed + 10 * layer + 5)
            # fused projection rows for the local heads: [q_local*D | kv_local*D | kv_local*D]
            full = torch.randn(((q_heads + 2 * kv_heads) * head_dim, hidden), generator=wgen, device=self.device) * 0.02
            qs = full[h0 * g * head_dim:(h0 + self.kv_local) * g * head_dim]
            ko = q_heads * head_dim
            ks = full[ko + h0 * head_dim:ko + (h0 + self.kv_local) * head_dim]
            vo = (q_heads + kv_heads) * head_dim
            vs = full[vo + h0 * head_dim:vo + (h0 + self.kv_local) * head_dim]
            self.wqkv.append(torch.cat([qs, ks, vs]).to(dt).contiguous())
            self.wo.append((torch.randn((hidden, q_heads * head_dim), generator=wgen, device=self.device) * 0.02).to(dt))
            self.norm_w.append(torch.ones(hidden, dtype=dt, device=self.device))
            del full
            # KV cache of this layer for the local heads, generated in place (same seed on every rank,
            # then the local head slice is kept)
            k, v = synth.make_kv(batch, kv_heads, context, head_dim, seed + layer, dtype, device=self.device)
            k, v = k[:, h0:h0 + self.kv_local], v[:, h0:h0 + self.kv_local]
            eng = DiffCacheGPU(batch, self.q_local, self.kv_local, head_dim, max_ctx_len=n_r, dtype=dtype,
                               device=self.device.index, use_bruteforce=True, name=f"l{layer:03d}")
            eng.prefill(k[:, :, sink:sink + n_r], v[:, :, sink:sink + n_r])
            rk = torch.zeros((batch, self.kv_local, sink + window + 8, head_dim), dtype=dt, device=self.device)
            rv = torch.zeros_like(rk)
            for dst, src in ((rk, k), (rv, v)):
                dst[:, :, :sink] = src[:, :, :sink]
                dst[:, :, sink:self.res_rows] = src[:, :, sink + n_r:context - 1]
            self.engines.append(eng)
            self.res_k.append(rk)
            self.res_v.append(rv)
            del k, v
        self.attn_local = torch.empty((batch, self.q_local, head_dim), dtype=dt, device=self.device)
        self.attn_full = torch.empty((self.world, batch, self.q_local * head_dim), dtype=dt, device=self.device)
        # Peer exchange: m channels used round-robin, m chosen so that the last layer of one step and the first
        # layer of the next (channel 0 again when the step is replayed from a graph) never share a channel.
        self.xchg, self.xchg_channels, self.xchg_views = None, 0, []
        if self.world > 1 and exchange in ("peer", "auto"):
            m = next((c for c in (2, 3, 4) if n_layers > 1 and (n_layers - 1) % c != 0), 0)
            if m == 0 and exchange == "peer":
                raise ValueError("the peer exchange needs at least two layers")
            if m:
                try:
                    slot = batch * self.q_local * head_dim * 2
                    self.xchg = PeerExchange([slot] * m, self.device.index, group)
                    self.xchg_channels = m
                    # where the wait kernel unpacks a layer's gathered slices: (B, world * q_local * D)
                    self.xchg_views = [torch.empty((batch, self.world * self.q_local * head_dim), dtype=dt,
                                                   device=self.device) for _ in range(m)]
                except RuntimeError:
                    if exchange == "peer":
                        raise
        self.exchange = "peer" if self.xchg is not None else ("nccl" if self.world > 1 else "none")
        # DC_STACK_FUSED_GATHER=0: the all-gather's consumer side stays a kernel of its own (PeerExchange.collect)
        self.fused_gather = os.environ.get("DC_STACK_FUSED_GATHER", "1") != "0"
        self._last_channel = -1
        torch.cuda.synchronize(self.device)

    def step(self, x: torch.Tensor, n_layers: Optional[int] = None, probe: Optional[dict] = None) -> torch.Tensor:
        """x ``(batch, hidden)`` -> ``(batch, hidden)`` after ``n_layers`` (default: all) layers.  The resident
        length is not advanced, so repeated calls time the same step.  ``probe`` (a dict) receives layer 0's
        query heads, new key/value rows and local attention output, for checks by the caller."""
        B, D = self.batch, self.head_dim
        nq, nkv = self.q_local * D, self.kv_local * D
        for layer in range(self.n_layers if n_layers is None else n_layers):
            h = F.rms_norm(x, (self.hidden,), self.norm_w[layer], 1e-5)
            qkv = F.linear(h, self.wqkv[layer])
            # slices of the fused projection output, passed as they are (batch stride = nq + 2*nkv)
            q = qkv[:, :nq].unflatten(1, (self.q_local, D))
            kn = qkv[:, nq:nq + nkv].unflatten(1, (self.kv_local, D))
            vn = qkv[:, nq + nkv:].unflatten(1, (self.kv_local, D))
            ch = layer % self.xchg_channels if self.xchg is not None else -1
            if self.xchg is not None and ch == self._last_channel:
                # two exchanges in a row on one channel (a call that stopped after an odd number of layers):
                # make sure every rank has finished reading the block this one overwrites
                if torch.cuda.is_current_stream_capturing():
                    raise RuntimeError("consecutive exchanges on one channel cannot be captured")
                torch.cuda.synchronize(self.device)
                dist.barrier(self.pg)
            self._last_channel = ch
            self.engines[layer].set_output_exchange(self.xchg if self.xchg is not None else None, max(ch, 0))
            # with the peer exchange the step's last kernel also stores the slice into every rank's buffer,
            # where it lands as (B, world, q_local*D), waits there for the other ranks' slices and unpacks all
            # of them into the dense buffer the projection reads
            if self.xchg is not None and self.fused_gather:
                self.engines[layer].set_output_gather(self.xchg_views[ch])
            self.engines[layer].decode_attend(q, self.attn_local, self.topk, res_k=self.res_k[layer],
                                              res_v=self.res_v[layer], res_len=self.res_rows, k_new=kn, v_new=vn)
            if probe is not None and layer == 0:
                probe.update(q=q.clone(), k_new=kn.clone(), v_new=vn.clone(), attn=self.attn_local.clone())
            if self.xchg is not None:
                attn = self.xchg_views[ch]
                if not self.fused_gather:
                    self.xchg.collect(ch, attn)                       # waits for all slices, unpacks them densely
            elif self.world > 1:
                dist.all_gather_into_tensor(self.attn_full.view(-1), self.attn_local.view(-1), group=self.pg)
                attn = self.attn_full.view(self.world, B, self.kv_local, -1).permute(1, 0, 2, 3).reshape(B, -1)
            else:
                attn = self.attn_local.view(B, -1)
            x = torch.addmm(x, attn, self.wo[layer].t())   # residual + output projection in one GEMM epilogue
        return x

    def close(self) -> None:
        for e in self.engines:
            e.close()
        self.engines = []
        if self.xchg is not None:
            self.xchg_views = []
            self.xchg.close()
            self.xchg = None
