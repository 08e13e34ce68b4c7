"""Seeded synthetic decode-step inputs with the shapes and value distributions of the
benchmark configurations: keys N(0,1) with four fixed outlier channels scaled x8 and a
slow per-position drift, values N(0,1), query = 0.3 * (a random cached key) + N(0,1).

They stand in for the needle-in-a-haystack / book-summarisation runs the reference is
exercised with (example/niah/run.py), whose model weights and texts are not available.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

OUTLIER_CHANNELS = (7, 45, 78, 101)


@dataclass
class StepConfig:
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    head_dim: int
    context: int
    topk: int
    sink: int
    window: int
    dtype: str = "bf16"

    @property
    def group(self) -> int:
        return self.q_heads // self.kv_heads

    @property
    def n_prob(self) -> int:
        return self.batch * self.kv_heads

    @property
    def n_retrieval(self) -> int:
        return self.context - self.sink - self.window

    def algorithmic_bytes(self) -> int:
        """Bytes one step must move: the key scan once, the attended K and V rows, q in, o out."""
        es = 2
        scan = self.n_prob * self.n_retrieval * self.head_dim * es
        rows = 2 * self.n_prob * (min(self.topk, self.n_retrieval) + self.sink + self.window) * self.head_dim * es
        qo = 2 * self.batch * self.q_heads * self.head_dim * es
        return scan + rows + qo

    def scan_bytes(self) -> int:
        return self.n_prob * self.n_retrieval * self.head_dim * 2


CONFIGS = {
    "cfg0": StepConfig("cfg0", 1, 32, 8, 128, 32768, 1024, 64, 256, "fp16"),
    "cfg1": StepConfig("cfg1", 16, 32, 8, 128, 131072, 2048, 64, 512, "bf16"),
    # configuration 1 with two sequences: same kernels and per-problem sizes, 0.5 GB of keys (still larger
    # than L2) — the case profiler captures are taken on
    "cfg1_b2": StepConfig("cfg1_b2", 2, 32, 8, 128, 131072, 2048, 64, 512, "bf16"),
    "cfg2_layer": StepConfig("cfg2_layer", 8, 32, 8, 128, 131072, 2048, 64, 512, "bf16"),
    "cfg3": StepConfig("cfg3", 1, 32, 8, 128, 1048576, 4096, 64, 1024, "bf16"),
    "cfg4": StepConfig("cfg4", 4, 32, 8, 128, 262144, 2048, 0, 0, "bf16"),
}


def torch_dtype(name: str) -> torch.dtype:
    return {"bf16": torch.bfloat16, "fp16": torch.float16}[name]


def make_kv(batch: int, kv_heads: int, n: int, head_dim: int, seed: int, dtype: str, device="cpu",
            pos_offset: int = 0, total: int | None = None, chunk: int = 1 << 16):
    """Keys/values ``(batch, kv_heads, n, head_dim)`` for positions ``[pos_offset, pos_offset+n)``
    of a sequence of ``total`` tokens.  Generated chunk-wise so the fp32 temporaries stay small."""
    total = n if total is None else total
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    dt = torch_dtype(dtype)
    k = torch.empty((batch, kv_heads, n, head_dim), dtype=dt, device=dev)
    v = torch.empty((batch, kv_heads, n, head_dim), dtype=dt, device=dev)
    drift_dir = torch.randn((kv_heads, head_dim), generator=gen, device=dev)
    for s in range(0, n, chunk):
        e = min(n, s + chunk)
        kc = torch.randn((batch, kv_heads, e - s, head_dim), generator=gen, device=dev)
        for c in OUTLIER_CHANNELS:
            if c < head_dim:
                kc[..., c] *= 8.0
        pos = (torch.arange(s, e, device=dev, dtype=torch.float32) + pos_offset) / float(total) - 0.5
        kc += 0.5 * pos[None, None, :, None] * drift_dir[None, :, None, :]
        k[:, :, s:e] = kc.to(dt)
        v[:, :, s:e] = torch.randn((batch, kv_heads, e - s, head_dim), generator=gen, device=dev).to(dt)
    return k, v


ROW_CHUNK = 1 << 16


def make_kv_rows(batch: int, kv_heads: int, row_start: int, n_rows: int, head_dim: int, seed: int, dtype: str,
                 device="cpu", total: int | None = None):
    """Rows ``[row_start, row_start + n_rows)`` of a sequence of ``total`` tokens whose contents depend only on
    (seed, global row), not on how the sequence is cut: every 65536-row chunk has its own generator seed, so
    ranks that hold different row ranges of one sequence generate exactly the rows a single holder would.
    Same distributions as :func:`make_kv`."""
    total = row_start + n_rows if total is None else total
    dev = torch.device(device)
    dt = torch_dtype(dtype)
    k = torch.empty((batch, kv_heads, n_rows, head_dim), dtype=dt, device=dev)
    v = torch.empty((batch, kv_heads, n_rows, head_dim), dtype=dt, device=dev)
    drift_dir = torch.randn((kv_heads, head_dim), generator=torch.Generator(device=dev).manual_seed(seed), device=dev)
    first, last = row_start // ROW_CHUNK, (row_start + n_rows - 1) // ROW_CHUNK if n_rows > 0 else -1
    for c in range(first, last + 1):
        gen = torch.Generator(device=dev).manual_seed(seed * 1_000_003 + 7 * c + 1)
        kc = torch.randn((batch, kv_heads, ROW_CHUNK, head_dim), generator=gen, device=dev)
        vc = torch.randn((batch, kv_heads, ROW_CHUNK, head_dim), generator=gen, device=dev)
        for ch in OUTLIER_CHANNELS:
            if ch < head_dim:
                kc[..., ch] *= 8.0
        pos = (torch.arange(c * ROW_CHUNK, (c + 1) * ROW_CHUNK, device=dev, dtype=torch.float32)) / float(total) - 0.5
        kc += 0.5 * pos[None, None, :, None] * drift_dir[None, :, None, :]
        lo, hi = max(row_start, c * ROW_CHUNK), min(row_start + n_rows, (c + 1) * ROW_CHUNK)
        k[:, :, lo - row_start:hi - row_start] = kc[:, :, lo - c * ROW_CHUNK:hi - c * ROW_CHUNK].to(dt)
        v[:, :, lo - row_start:hi - row_start] = vc[:, :, lo - c * ROW_CHUNK:hi - c * ROW_CHUNK].to(dt)
    return k, v


def make_query(keys: torch.Tensor, group: int, seed: int):
    """Query heads ``(batch, kv_heads*group, head_dim)``: 0.3 * a random cached key + N(0,1)."""
    batch, kv_heads, n, head_dim = keys.shape
    gen = torch.Generator(device=keys.device).manual_seed(seed + 7919)
    j = torch.randint(0, n, (batch, kv_heads), generator=gen, device=keys.device)
    picked = torch.gather(keys, 2, j[:, :, None, None].expand(batch, kv_heads, 1, head_dim)).float()  # (B,Hkv,1,D)
    noise = torch.randn((batch, kv_heads, group, head_dim), generator=gen, device=keys.device)
    q = 0.3 * picked + noise
    return q.reshape(batch, kv_heads * group, head_dim).to(keys.dtype)
