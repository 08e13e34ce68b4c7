"""CPU oracle (test infrastructure, never on the product path).

ctypes binding of ``oracle/dc_oracle.c``, a restatement of the exact-scan path
of the reference engine (diffcache_cpu/src/nsw.rs:592-630,
diffcache_cpu/src/lib.rs:373-404) plus fp64 attention with the semantics of the
``flash_attn_with_kvcache`` call at src/diffcache/base.py:134-142.

Pinned against (1) outputs of the reference's own PyTorch statement of the path (exact branch of
``gqa_topk_attention``, tools/topk_test.py:303-470; ``tests/golden/spec_vectors.npz``) for the
chosen rows, their order and the attention output, and (2) the DualHeap test sequences for the
top-k ordering (``tests/golden/select_kat.json``).  Parity unpinned for the Rust engine's own
arithmetic: it has no tests or golden vectors for this path and cannot be built here, so the
last bit of ``dist`` is defined by this oracle (exact dot, rounded once).

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
reference legs may import this package.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libdc_oracle.so")
_SRC = os.path.join(_HERE, "dc_oracle.c")

BF16, FP16 = 0, 1


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (OpenMP, -O3 -march=native) into ``oracle/libdc_oracle.so``."""
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(_SRC):
        return _SO
    cmd = ["gcc", "-O3", "-march=native", "-fopenmp", "-shared", "-fPIC", "-std=c11", "-o", _SO, _SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        i64, i32, vp, f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_float
        _lib.dco_convert_to_f32.argtypes = [vp, i64, i32, vp]
        _lib.dco_convert_from_f32.argtypes = [vp, i64, i32, vp]
        _lib.dco_group_mean.argtypes = [vp, i32, i32, i32, i32, vp]
        _lib.dco_score_rows.argtypes = [vp, i64, i32, i32, vp, i32, vp]
        _lib.dco_topk_heap.argtypes = [vp, vp, i64, i64, vp, vp]
        _lib.dco_topk_heap.restype = i64
        _lib.dco_topk_sort.argtypes = [vp, vp, i64, i64, vp, vp]
        _lib.dco_topk_sort.restype = i64
        _lib.dco_query.argtypes = [vp, vp, i64, i32, i64, i32, i32, vp, i64, i32, i32, vp, vp, vp, vp]
        _lib.dco_query.restype = i64
        _lib.dco_attend.argtypes = [vp, vp, i32, i64, i32, i32, i32, vp, f32, i32, vp, vp, vp]
        _lib.dco_pq_build_lut.argtypes = [vp, i32, vp, i32, i32, i32, vp]
        _lib.dco_pq_adc_scores.argtypes = [vp, i64, i32, vp, vp]
        _lib.dco_rerank_scores.argtypes = [vp, i32, i32, vp, vp, i64, i32, vp]
        _lib.dco_k_check.argtypes = [vp, i32, i32, f32, vp, vp]
        _lib.dco_k_check.restype = i32
        _lib.dco_adaptive_budget.argtypes = [vp, i32, i32, vp, i32, f32]
        _lib.dco_adaptive_budget.restype = i32
        _lib.dco_max_threads.restype = i32
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


def max_threads() -> int:
    return int(lib().dco_max_threads())


def to_f32(x_u16: np.ndarray, dtype: int) -> np.ndarray:
    x = _c(x_u16, np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().dco_convert_to_f32(_p(x), x.size, dtype, _p(out))
    return out


def from_f32(x: np.ndarray, dtype: int) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().dco_convert_from_f32(_p(x), x.size, dtype, _p(out))
    return out


def group_mean(q_u16: np.ndarray, group: int, dtype: int) -> np.ndarray:
    """q (n_prob*group, D) -> (n_prob, D); diffcache.py:191-194."""
    q = _c(q_u16, np.uint16)
    rows, dim = q.shape
    out = np.empty((rows // group, dim), np.uint16)
    lib().dco_group_mean(_p(q), rows // group, group, dim, dtype, _p(out))
    return out


def score_rows(keys_u16: np.ndarray, q_u16: np.ndarray, dtype: int, exact: bool = True) -> np.ndarray:
    """dist bits of every row of ONE problem: keys (n, D), q (D,)."""
    k = _c(keys_u16, np.uint16)
    q = _c(q_u16, np.uint16)
    n, dim = k.shape
    out = np.empty(n, np.uint32)
    lib().dco_score_rows(_p(k), n, dim, dtype, _p(q), int(exact), _p(out))
    return out


def topk(bits: np.ndarray, ef: int, ids: np.ndarray | None = None, method: str = "heap"):
    """ef smallest (bits, id) ascending; returns (bits, ids)."""
    b = _c(bits, np.uint32)
    i = None if ids is None else _c(ids, np.uint32)
    n = b.shape[0]
    ob = np.empty(max(ef, 1), np.uint32)
    oi = np.empty(max(ef, 1), np.uint32)
    fn = lib().dco_topk_heap if method == "heap" else lib().dco_topk_sort
    kept = fn(_p(b), _p(i), n, ef, _p(ob), _p(oi))
    return ob[:kept].copy(), oi[:kept].copy()


def query(keys_u16, vals_u16, q_mean_u16, ef: int, dtype: int, n: int | None = None, exact: bool = True,
          n_threads: int = 0, gather: bool = True, out_keys=None, out_vals=None):
    """DataLayer::query, brute force.  keys/vals (n_prob, n_max, D); q_mean (n_prob, D).

    Returns dict(ef, keys, vals, idx, bits) with row i = i-th best.  ``out_keys``/``out_vals`` (uint16,
    (n_prob, min(ef, n), D), C-contiguous) are written in place when given, as the reference writes into
    the caller's pinned buffers (lib.rs:613-624)."""
    k = _c(keys_u16, np.uint16)
    v = None if vals_u16 is None else _c(vals_u16, np.uint16)
    q = _c(q_mean_u16, np.uint16)
    n_prob, n_max, dim = k.shape
    n = n_max if n is None else n
    ef_c = min(ef, n)
    for o in (out_keys, out_vals):
        assert o is None or (o.dtype == np.uint16 and o.shape == (n_prob, ef_c, dim) and o.flags["C_CONTIGUOUS"])
    ok = (out_keys if out_keys is not None else np.zeros((n_prob, ef_c, dim), np.uint16)) if gather else None
    ov = (out_vals if out_vals is not None else np.zeros((n_prob, ef_c, dim), np.uint16)) if (gather and v is not None) else None
    oi = np.zeros((n_prob, ef_c), np.uint32)
    ob = np.zeros((n_prob, ef_c), np.uint32)
    got = lib().dco_query(_p(k), _p(v), n_max * dim, n_prob, n, dim, dtype, _p(q), ef, int(exact), n_threads,
                          _p(ok), _p(ov), _p(oi), _p(ob))
    assert got == ef_c
    return dict(ef=ef_c, keys=ok, vals=ov, idx=oi, bits=ob)


def attend(k_rows_u16, v_rows_u16, q_u16, group: int, scale: float, dtype: int, n_threads: int = 0):
    """k_rows/v_rows (n_prob, n_rows, D) gathered rows; q (n_prob*group, D).

    Returns (out_f32, out_elem_u16, lse)."""
    k = _c(k_rows_u16, np.uint16)
    v = _c(v_rows_u16, np.uint16)
    q = _c(q_u16, np.uint16)
    n_prob, n_rows, dim = k.shape
    assert q.shape == (n_prob * group, dim)
    of = np.empty((n_prob * group, dim), np.float32)
    oe = np.empty((n_prob * group, dim), np.uint16)
    lse = np.empty(n_prob * group, np.float32)
    lib().dco_attend(_p(k), _p(v), n_prob, n_rows, group, dim, dtype, _p(q), scale, n_threads, _p(of), _p(oe), _p(lse))
    return of, oe, lse


def pq_build_lut(q_mean_u16, centroids_f32, n_sub: int, dtype: int) -> np.ndarray:
    q = _c(q_mean_u16, np.uint16)
    c = _c(centroids_f32, np.float32)
    n_prob, dim = q.shape
    lut = np.empty((n_prob, n_sub, 256), np.float32)
    lib().dco_pq_build_lut(_p(q), dtype, _p(c), n_prob, dim, n_sub, _p(lut))
    return lut


def pq_adc_scores(codes_u8, lut_f32) -> np.ndarray:
    """codes (n, M) of ONE problem, lut (M, 256) -> dist bits (n,)."""
    c = _c(codes_u8, np.uint8)
    lut = _c(lut_f32, np.float32)
    n, n_sub = c.shape
    out = np.empty(n, np.uint32)
    lib().dco_pq_adc_scores(_p(c), n, n_sub, _p(lut), _p(out))
    return out


def rerank_scores(keys_u16, q_u16, ids_u32, dtype: int, exact: bool = True) -> np.ndarray:
    k = _c(keys_u16, np.uint16)
    q = _c(q_u16, np.uint16)
    ids = _c(ids_u32, np.uint32)
    out = np.empty(ids.shape[0], np.uint32)
    lib().dco_rerank_scores(_p(k), k.shape[1], dtype, _p(q), _p(ids), ids.shape[0], int(exact), _p(out))
    return out


def k_check(dist_bits_sorted: np.ndarray, dim: int, threshold: float):
    """nsw.rs:285-300 on the best-first ranking keys; returns (stoppable, alpha, mass)."""
    b = _c(dist_bits_sorted, np.uint32)
    alpha = np.zeros(1, np.float32)
    mass = np.zeros(1, np.float32)
    ok = lib().dco_k_check(_p(b), b.shape[0], dim, threshold, _p(alpha), _p(mass))
    return bool(ok), float(alpha[0]), float(mass[0])


def adaptive_budget(dist_bits_sorted: np.ndarray, dim: int, seq, threshold: float) -> int:
    """First checkpoint of k_check_seq whose top-h keys pass the k-check, else k (nsw.rs:339-376)."""
    b = _c(dist_bits_sorted, np.uint32)
    sq = np.asarray(list(seq), np.int32)
    return int(lib().dco_adaptive_budget(_p(b), b.shape[0], dim, _p(sq), sq.shape[0], threshold))
