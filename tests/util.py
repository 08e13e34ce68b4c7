"""Shared helpers for the tests: seeded inputs and oracle-side composition of a decode step."""
import json
import os

import numpy as np
import torch

from diffcache_b200 import synth

KAT_OFFSET = 0x40000000 + 1000  # i32 test values in [-1000, 1000] -> bit patterns of positive floats
HERE = os.path.dirname(os.path.abspath(__file__))


def load_select_kat():
    with open(os.path.join(HERE, "golden", "select_kat.json")) as f:
        return json.load(f)


def u16(t: torch.Tensor) -> np.ndarray:
    """16-bit float tensor -> numpy uint16 bit patterns (host)."""
    return t.detach().cpu().contiguous().view(torch.uint16).numpy()


def dtype_code(name: str) -> int:
    return {"bf16": 0, "fp16": 1}[name]


def ulp_of_dist(bits: np.ndarray) -> np.ndarray:
    """Spacing of fp32 at the dist values whose bit patterns are given."""
    f = bits.view(np.float32).astype(np.float64)
    return np.spacing(np.abs(f).astype(np.float32)).astype(np.float64)


def check_selection_parity(gpu_idx, oracle_idx, oracle_all_bits):
    """BASELINE rule: the selected index SETS must match exactly, except for ties within one
    fp32 ulp of dist at the selection boundary.  `oracle_all_bits` are the oracle dist bits of
    every row.  Returns the number of boundary substitutions."""
    gs, os_ = set(int(i) for i in gpu_idx), set(int(i) for i in oracle_idx)
    assert len(gs) == len(gpu_idx), "duplicate rows selected"
    assert len(gs) == len(os_)
    if gs == os_:
        return 0
    kth = oracle_all_bits[np.asarray(oracle_idx, dtype=np.int64)].max()
    kth_f = np.array([kth], np.uint32).view(np.float32)[0]
    ulp = float(np.spacing(np.float32(abs(kth_f))))
    for i in (gs - os_) | (os_ - gs):
        d = np.array([oracle_all_bits[i]], np.uint32).view(np.float32)[0]
        assert abs(float(d) - float(kth_f)) <= ulp + 1e-12, (
            f"row {i}: dist {d} differs from the k-th dist {kth_f} by more than one ulp ({ulp})")
    return len(gs - os_)


def oracle_decode_step(oracle, k_store, v_store, q_heads, group, topk, res_k, res_v, k_new, v_new, scale, dtype):
    """Reference semantics of one fused step on host arrays (all uint16 bit patterns).

    k_store/v_store (P, n, D); q_heads (P*group, D); res_k/res_v (P, res_len, D) or None;
    k_new/v_new (P, D) or None.  Returns dict(idx, bits, all_bits, out_f32, out_elem, lse)."""
    P, n, D = k_store.shape
    q_mean = oracle.group_mean(q_heads, group, dtype)
    res = oracle.query(k_store, v_store, q_mean, topk, dtype, exact=True)
    all_bits = np.stack([oracle.score_rows(k_store[p], q_mean[p], dtype) for p in range(P)]) if n > 0 else np.zeros((P, 0), np.uint32)
    parts_k, parts_v = [], []
    if res["ef"] > 0:
        parts_k.append(res["keys"]); parts_v.append(res["vals"])
    if res_k is not None and res_k.shape[1] > 0:
        parts_k.append(res_k); parts_v.append(res_v)
    if k_new is not None:
        parts_k.append(k_new[:, None, :]); parts_v.append(v_new[:, None, :])
    kk = np.ascontiguousarray(np.concatenate(parts_k, axis=1))
    vv = np.ascontiguousarray(np.concatenate(parts_v, axis=1))
    of, oe, lse = oracle.attend(kk, vv, q_heads, group, scale, dtype)
    return dict(idx=res["idx"], bits=res["bits"], all_bits=all_bits, out_f32=of, out_elem=oe, lse=lse, q_mean=q_mean)


def small_problem(batch, kv_heads, group, n, head_dim, seed, dtype="bf16", device="cpu"):
    k, v = synth.make_kv(batch, kv_heads, n, head_dim, seed, dtype, device=device)
    q = synth.make_query(k, group, seed) if n > 0 else torch.randn(batch, kv_heads * group, head_dim).to(k.dtype)
    return k, v, q


def assert_attention_close(got_u16, want_f32, dtype, oracle, atol=1e-3, rtol=2e-3):
    """Output tolerance of the task (2e-3 relative / 1e-3 absolute) applied to the value the
    kernel computed; the final rounding to a 16-bit type can add up to half a unit in the last
    place of that type on top (2^-9 relative for bf16, 2^-12 for fp16), which no kernel can avoid."""
    got = oracle.to_f32(np.ascontiguousarray(got_u16), dtype).astype(np.float64)
    want = want_f32.astype(np.float64)
    mant = 8 if dtype == 0 else 11
    with np.errstate(divide="ignore"):
        half_ulp = np.where(want == 0, 0.0, 2.0 ** (np.floor(np.log2(np.abs(want) + 1e-300)) - mant))
    tol = atol + rtol * np.abs(want) + half_ulp
    bad = np.abs(got - want) > tol
    assert not bad.any(), f"{bad.sum()} outputs off; worst {np.max(np.abs(got - want) - tol):.3e} beyond tolerance"
