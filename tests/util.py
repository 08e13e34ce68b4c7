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
    """Parity rule of the task: the selected index SETS must match exactly, except for ties within one
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


def oracle_attention_over(oracle, k_store, v_store, sel_idx, q_heads, group, res_k, res_v, k_new, v_new, scale, dtype):
    """Oracle attention over the store rows `sel_idx` (P, k) — whatever rows were selected, e.g. the GPU's
    own choice when it differs from the oracle's by an allowed boundary tie — plus the resident rows and
    the new token.  Attention does not depend on the order of the rows.  Returns (out_f32, lse)."""
    P = k_store.shape[0]
    idx = np.asarray(sel_idx, dtype=np.int64).reshape(P, -1)
    parts_k, parts_v = [], []
    if idx.shape[1] > 0:
        parts_k.append(np.stack([k_store[p][idx[p]] for p in range(P)]))
        parts_v.append(np.stack([v_store[p][idx[p]] for p in range(P)]))
    if res_k is not None and res_k.shape[1] > 0:
        parts_k.append(res_k); parts_v.append(res_v)
    if k_new is not None:
        parts_k.append(k_new[:, None, :]); parts_v.append(v_new[:, None, :])
    kk = np.ascontiguousarray(np.concatenate(parts_k, axis=1))
    vv = np.ascontiguousarray(np.concatenate(parts_v, axis=1))
    of, _, lse = oracle.attend(kk, vv, q_heads, group, scale, dtype)
    return of, lse


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


# ---- inputs of the functional-spec fixtures (tests/golden/spec_vectors.npz) ----
# Generated with integer hashing only, so the same bytes come out on every platform, and
# quantised so that every value is exact in bf16 AND fp16, the group-mean query is exact, and
# every dot product is exact in fp32 in any summation order.

SPEC_CASES = {
    # name: batch, kv_heads, group, head_dim, kv_len, prefix_keep_len, suffix_keep_len, top_k, seed
    "c0": dict(batch=1, kv_heads=2, group=4, head_dim=64, kv_len=700, prefix=16, suffix=33, top_k=96, seed=11),
    "c1": dict(batch=2, kv_heads=2, group=2, head_dim=128, kv_len=1200, prefix=64, suffix=65, top_k=128, seed=72),
    "c2": dict(batch=1, kv_heads=1, group=8, head_dim=64, kv_len=300, prefix=0, suffix=1, top_k=500, seed=13),
    "c3": dict(batch=1, kv_heads=2, group=1, head_dim=128, kv_len=2500, prefix=4, suffix=17, top_k=256, seed=34),
}


def _hash_uniform(n: int, seed: int, salt: int) -> np.ndarray:
    """n doubles in [0, 1) from a splitmix64-style integer hash of (seed, salt, index)."""
    with np.errstate(over="ignore"):
        x = np.arange(n, dtype=np.uint64)
        x = x + np.uint64((seed * 0x9E3779B97F4A7C15 + salt * 0xD1B54A32D192ED03) & 0xFFFFFFFFFFFFFFFF)
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    return (x >> np.uint64(40)).astype(np.float64) / float(1 << 24)


def _hash_normal(shape, seed: int, salt: int) -> np.ndarray:
    """Roughly N(0, 1): centred sum of four uniforms (Irwin-Hall), scaled to unit variance."""
    n = int(np.prod(shape))
    s = sum(_hash_uniform(n, seed, salt * 4 + j) for j in range(4))
    return ((s - 2.0) * np.sqrt(3.0)).reshape(shape)


def spec_case_inputs(case: dict):
    """float32 arrays (query [B, H, 1, D], key [B, KV, kv_len, D], value [B, KV, kv_len, D]) in the
    layout of the attention function of tools/topk_test.py:303-311.

    keys/values: multiples of 1/32 in [-2, 2]; queries: multiples of 1/16 in [-3.9375, 3.9375],
    each head = 0.5 * (one cached key of its kv head) + noise, so the top-k is not arbitrary."""
    B, KV, G, D, N, seed = (case[k] for k in ("batch", "kv_heads", "group", "head_dim", "kv_len", "seed"))
    key = np.clip(np.round(_hash_normal((B, KV, N, D), seed, 1) * 32) / 32, -2, 2)
    val = np.clip(np.round(_hash_normal((B, KV, N, D), seed, 2) * 32) / 32, -2, 2)
    pick = (_hash_uniform(B * KV, seed, 99) * N).astype(np.int64).reshape(B, KV)
    anchor = np.take_along_axis(key, pick[:, :, None, None].repeat(D, axis=3), axis=2)  # [B, KV, 1, D]
    noise = _hash_normal((B, KV, G, D), seed, 3)
    q = np.clip(np.round((0.5 * anchor + noise) * 16) / 16, -3.9375, 3.9375)          # [B, KV, G, D]
    query = q.reshape(B, KV * G, 1, D)
    return query.astype(np.float32), key.astype(np.float32), val.astype(np.float32)


def load_spec_vectors():
    return np.load(os.path.join(HERE, "golden", "spec_vectors.npz"))


def spec_case_split(case: dict, query, key, value):
    """Maps the [prefix | retrieval | suffix] layout of tools/topk_test.py:355-364 onto the engine's
    inputs: the store holds the retrieval region, the resident rows are prefix + suffix without its
    last row, and that last row is the step's new token.  All float32 arrays; returns a dict."""
    B, KV, G, D, N = (case[k] for k in ("batch", "kv_heads", "group", "head_dim", "kv_len"))
    p_len = max(0, min(case["prefix"], N))
    s_len = max(0, min(case["suffix"], N - p_len))
    assert s_len >= 1, "the newest token is the last row of the suffix"
    return dict(
        store_k=np.ascontiguousarray(key[:, :, p_len:N - s_len]), store_v=np.ascontiguousarray(value[:, :, p_len:N - s_len]),
        res_k=np.ascontiguousarray(np.concatenate([key[:, :, :p_len], key[:, :, N - s_len:N - 1]], axis=2)),
        res_v=np.ascontiguousarray(np.concatenate([value[:, :, :p_len], value[:, :, N - s_len:N - 1]], axis=2)),
        k_new=np.ascontiguousarray(key[:, :, N - 1]), v_new=np.ascontiguousarray(value[:, :, N - 1]),
        q=np.ascontiguousarray(query.reshape(B, KV * G, D)), n_store=N - s_len - p_len, res_rows=p_len + s_len - 1)


# ---- inputs of the KV-cache-manager fixtures (tests/golden/kvcache_vectors.npz) ----

KVCACHE_CASES = {
    # long prompt: retrieval region (180) > budget (48); short prompt: retrieval region (20) < budget
    "long": dict(num_layers=2, batch=1, kv_heads=2, group=4, head_dim=64, seq_len=200, budget=48, prefix=8, suffix=12,
                 suffix_max=16, max_length=256, seed=21),
    "short": dict(num_layers=2, batch=2, kv_heads=2, group=4, head_dim=64, seq_len=40, budget=48, prefix=8, suffix=12,
                  suffix_max=16, max_length=256, seed=22),
}


def kvcache_case_inputs(case: dict, layer: int):
    """Per layer: key_states, value_states (B, S, Hkv, D) as the model hands them to
    prefill_update_kv_cache (diffcache.py:149-154) and the decode-step queries (B, 1, Hq*D);
    float32 arrays whose values are exact in bf16 (same quantisation as spec_case_inputs)."""
    B, KV, G, D, S = (case[k] for k in ("batch", "kv_heads", "group", "head_dim", "seq_len"))
    seed = case["seed"] * 100 + layer
    key = np.clip(np.round(_hash_normal((B, S, KV, D), seed, 1) * 32) / 32, -2, 2)
    val = np.clip(np.round(_hash_normal((B, S, KV, D), seed, 2) * 32) / 32, -2, 2)
    pick = (_hash_uniform(B * KV, seed, 99) * S).astype(np.int64).reshape(B, KV)
    anchor = np.stack([np.stack([key[b, pick[b, h], h] for h in range(KV)]) for b in range(B)])  # (B, KV, D)
    noise = _hash_normal((B, KV, G, D), seed, 3)
    q = np.clip(np.round((0.5 * anchor[:, :, None, :] + noise) * 16) / 16, -3.9375, 3.9375)
    return key.astype(np.float32), val.astype(np.float32), q.reshape(B, 1, KV * G * D).astype(np.float32)


def load_kvcache_vectors():
    return np.load(os.path.join(HERE, "golden", "kvcache_vectors.npz"))


# ---- inputs of the k-check fixtures (tests/golden/kcheck_vectors.json) ----

KCHECK_CASES = {
    # best-first ranking keys whose logits fall off like -alpha*ln(rank) plus noise
    "steep": dict(n=64, head_dim=128, alpha=2.5, noise=0.05, top=900.0, seed=31),
    "shallow": dict(n=256, head_dim=128, alpha=1.05, noise=0.10, top=400.0, seed=32),
    "short": dict(n=8, head_dim=64, alpha=1.8, noise=0.02, top=120.0, seed=33),
    "long": dict(n=2048, head_dim=128, alpha=1.4, noise=0.20, top=2000.0, seed=34),
    "flat": dict(n=100, head_dim=64, alpha=0.0, noise=0.0, top=50.0, seed=35),
}


def kcheck_case_bits(case: dict) -> np.ndarray:
    """uint32 ranking keys bits(65536 - dot), ascending (best first), of a list whose logits
    dot/sqrt(D) follow top/sqrt(D) - alpha*ln(rank) + noise."""
    n, D = case["n"], case["head_dim"]
    ranks = np.arange(1, n + 1, dtype=np.float64)
    logit = case["top"] / np.sqrt(D) - case["alpha"] * np.log(ranks) + case["noise"] * _hash_normal((n,), case["seed"], 7)
    dot = np.sort(logit * np.sqrt(D))[::-1]
    return (np.float32(65536.0) - dot.astype(np.float32)).astype(np.float32).view(np.uint32)


def load_kcheck_vectors():
    with open(os.path.join(HERE, "golden", "kcheck_vectors.json")) as f:
        return json.load(f)
