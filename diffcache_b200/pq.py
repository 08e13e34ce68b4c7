"""Product-quantisation baseline path (asymmetric-distance scorer + exact rerank).

The reference ships no PQ code (``evaluation/impl/pqcache`` is an empty directory); this is
the textbook scheme its evaluation compares against: keys are split into ``n_sub`` subspaces,
each quantised to 256 k-means centroids (uint8 codes).  A decode step builds a per-query
lookup table ``lut[m][c] = <q_m, centroid[m][c]>``, scores every key as
``sum_m lut[m][code_m]`` (ADC), keeps the best ``n_cand`` candidates, re-scores those exactly
against the stored keys and keeps the best ``topk`` — all four stages are CUDA kernels behind
the C ABI.  Codebook training and encoding are one-time set-up done with torch ops.
"""
from __future__ import annotations

import torch

from . import _lib


def _stream() -> int:
    return int(torch.cuda.current_stream().cuda_stream)


def train_codebooks(keys: torch.Tensor, n_sub: int = 16, iters: int = 8, seed: int = 0,
                    sample: int = 65536) -> torch.Tensor:
    """Seeded Lloyd k-means per (problem, subspace).  keys ``(P, n, D)`` (16-bit, CUDA) ->
    centroids ``(P, n_sub, 256, D / n_sub)`` float32.  A fixed number of iterations on a seeded
    subsample of at most ``sample`` rows; empty clusters keep their previous centroid."""
    P, n, D = keys.shape
    ds = D // n_sub
    gen = torch.Generator(device=keys.device).manual_seed(seed)
    take = min(n, sample)
    pick = torch.randperm(n, generator=gen, device=keys.device)[:take]
    x = keys[:, pick].float().reshape(P, take, n_sub, ds).permute(0, 2, 1, 3).contiguous()  # (P, M, take, ds)
    init = torch.randperm(take, generator=gen, device=keys.device)[:256]
    cen = x[:, :, init].clone()                                                               # (P, M, 256, ds)
    if take < 256:
        cen = torch.cat([cen, cen.new_zeros(P, n_sub, 256 - take, ds)], dim=2)
    for _ in range(iters):
        d = torch.cdist(x, cen)                       # (P, M, take, 256)
        assign = d.argmin(dim=-1)                     # (P, M, take)
        one = torch.zeros((P, n_sub, 256), device=keys.device).scatter_add_(2, assign, torch.ones_like(assign, dtype=torch.float32))
        sums = torch.zeros_like(cen).scatter_add_(2, assign[..., None].expand(-1, -1, -1, ds), x)
        new = sums / one.clamp_min(1.0)[..., None]
        cen = torch.where(one[..., None] > 0, new, cen)
    return cen.contiguous()


def encode(keys: torch.Tensor, centroids: torch.Tensor, chunk: int = 32768) -> torch.Tensor:
    """keys ``(P, n, D)`` -> codes ``(P, n, n_sub)`` uint8 (nearest centroid per subspace)."""
    P, n, D = keys.shape
    n_sub, ds = centroids.shape[1], centroids.shape[3]
    codes = torch.empty((P, n, n_sub), dtype=torch.uint8, device=keys.device)
    for s in range(0, n, chunk):
        e = min(n, s + chunk)
        x = keys[:, s:e].float().reshape(P, e - s, n_sub, ds).permute(0, 2, 1, 3)  # (P, M, c, ds)
        codes[:, s:e] = torch.cdist(x, centroids).argmin(dim=-1).permute(0, 2, 1).to(torch.uint8)
    return codes


class PQWorkspace:
    """Device buffers of one PQ decode step, allocated once."""

    def __init__(self, n_prob: int, n: int, n_sub: int, n_cand: int, topk: int, device):
        lib = _lib.load()
        i32 = torch.int32
        self.lut = torch.empty((n_prob, n_sub, 256), dtype=torch.float32, device=device)
        self.scores = torch.empty((n_prob, n), dtype=i32, device=device)
        self.minmax = torch.empty((n_prob, 2), dtype=i32, device=device)
        self.minmax_init = torch.tensor([[-1, 0]] * n_prob, dtype=i32, device=device)
        self.cand_idx = torch.empty((n_prob, n_cand), dtype=i32, device=device)
        self.cand_bits = torch.empty((n_prob, n_cand), dtype=i32, device=device)
        self.sel_idx = torch.empty((n_prob, topk), dtype=i32, device=device)
        self.sel_bits = torch.empty((n_prob, topk), dtype=i32, device=device)
        self.status = torch.zeros(int(lib.dc_select_scratch_bytes(n_prob)), dtype=torch.uint8, device=device)


def adc_rerank_topk(keys: torch.Tensor, codes: torch.Tensor, centroids: torch.Tensor, q: torch.Tensor, group: int,
                    n_cand: int, topk: int, ws: PQWorkspace | None = None, dtype: int = 0, mark=None):
    """One PQ retrieval: returns ``(sel_idx, sel_bits)`` ``(P, topk)`` int32 tensors holding the
    selected row ids (best first) and their exact ranking keys.  keys ``(P, n, D)``; codes
    ``(P, n, n_sub)``; q ``(B, Hq, D)`` query heads (group mean formed in the kernels).  ``mark``
    (optional callable) is called after every stage: table, ADC scan, candidate select, rerank, final
    select — for per-stage timing."""
    mark = mark or (lambda: None)
    lib = _lib.load()
    P, n, D = keys.shape
    n_sub = codes.shape[2]
    ws = ws or PQWorkspace(P, n, n_sub, n_cand, topk, keys.device)
    st = _stream()
    ws.minmax.copy_(ws.minmax_init)
    _lib.check(lib.dc_pq_build_lut(q.data_ptr(), 1, group, dtype, centroids.data_ptr(), P, D, n_sub,
                                   ws.lut.data_ptr(), st))
    mark()
    _lib.check(lib.dc_pq_adc_scan(codes.data_ptr(), n * n_sub, P, n, n_sub, ws.lut.data_ptr(), ws.scores.data_ptr(),
                                  n, ws.minmax.data_ptr(), st))
    mark()
    _lib.check(lib.dc_topk_select(ws.scores.data_ptr(), None, n, P, n, n_cand, ws.minmax.data_ptr(), None,
                                  ws.cand_idx.data_ptr(), n_cand, ws.status.data_ptr(), st))
    mark()
    _lib.check(lib.dc_rerank_scores(keys.data_ptr(), n * D, P, D, dtype, q.data_ptr(), 1, group,
                                    ws.cand_idx.data_ptr(), n_cand, n_cand, ws.cand_bits.data_ptr(), st))
    mark()
    _lib.check(lib.dc_topk_select(ws.cand_bits.data_ptr(), ws.cand_idx.data_ptr(), n_cand, P, n_cand, topk, None,
                                  ws.sel_bits.data_ptr(), ws.sel_idx.data_ptr(), topk, ws.status.data_ptr(), st))
    mark()
    return ws.sel_idx, ws.sel_bits
