"""Writes tests/golden/spec_vectors.npz: outputs of the reference's own PyTorch statement of the
path, the exact (use_hnsw=False) branch of `gqa_topk_attention` in tools/topk_test.py:303-470,
on the seeded inputs of tests/util.py::spec_case_inputs.

The reference function is imported unmodified from a checkout of the reference (first argument,
or $DIFFCACHE_REFERENCE) and run on CPU in fp32.  It delegates the dense attention over the
gathered rows to whatever implementation is registered under `base_impl_name`
(topk_test.py:70,461-468); transformers' stock "sdpa" wrapper repeats the kv heads a second time
when the module carries `num_key_value_groups`, so a plain fp64 softmax attention is registered
through transformers' public `AttentionInterface.register` and named as the base instead.

Recorded per case: the positions chosen by the function's `torch.topk` (captured by wrapping
torch.topk for the duration of the call), the attention output, and the gap in q.k between the
last chosen and the first rejected row (the script refuses inputs where that gap is below
4 ulps of the engine's ranking key at 65536, so that the expected SET does not depend on how
ties are broken).

Run from the repository root:
    python tests/golden/make_spec_vectors.py /path/to/DiffCache
"""
import os
import sys
import types

import numpy as np
import torch

sys.dont_write_bytecode = True
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests.util import SPEC_CASES, spec_case_inputs  # noqa: E402


def dense_fp64_attention(module, query, key, value, attention_mask, scaling=None, **kwargs):
    """softmax(q k^T * scaling) v in fp64; returns [B, q_len, H, D] like the library wrappers."""
    q, k, v = query.double(), key.double(), value.double()
    s = torch.matmul(q, k.transpose(-1, -2)) * (scaling if scaling is not None else q.shape[-1] ** -0.5)
    if attention_mask is not None:
        s = s + attention_mask
    out = torch.matmul(torch.softmax(s, dim=-1), v)
    return out.transpose(1, 2).contiguous().to(query.dtype), None


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DIFFCACHE_REFERENCE", "")
    if not os.path.isfile(os.path.join(ref, "tools", "topk_test.py")):
        raise SystemExit("usage: make_spec_vectors.py <DiffCache checkout>")
    sys.path.insert(0, os.path.join(ref, "tools"))
    import topk_test  # the reference script, unmodified
    from transformers import AttentionInterface

    AttentionInterface.register("dense_fp64", dense_fp64_attention)
    out = {}
    for name, case in SPEC_CASES.items():
        query, key, value = (torch.from_numpy(a) for a in spec_case_inputs(case))
        D, G = case["head_dim"], case["group"]
        fn = topk_test.make_gqa_topk_attention(top_k=case["top_k"], base_impl_name="dense_fp64",
                                               prefix_keep_len=case["prefix"], suffix_keep_len=case["suffix"])
        module = types.SimpleNamespace(num_key_value_groups=G, scaling=D ** -0.5)
        seen = []
        real_topk = torch.topk

        def spy(*a, **kw):
            r = real_topk(*a, **kw)
            seen.append(r.indices.clone())
            return r

        torch.topk = spy
        try:
            attn, _ = fn(module, query, key, value, None, scaling=D ** -0.5)
        finally:
            torch.topk = real_topk
        assert len(seen) == 1
        top_local = seen[0]                      # [B, KV, k_eff], positions inside the retrieval region
        # boundary gap in q_mean . k units
        B, KV, N = case["batch"], case["kv_heads"], case["kv_len"]
        p_len = min(case["prefix"], N)
        s_len = min(case["suffix"], N - p_len)
        qm = query.view(B, KV, G, D).double().mean(2)
        dots = torch.einsum("bhd,bhnd->bhn", qm, key.double())[:, :, p_len:N - s_len]
        chosen = torch.zeros_like(dots, dtype=torch.bool).scatter_(2, top_local, True)
        worst_in = dots.masked_fill(~chosen, float("inf")).min(2).values
        best_out = dots.masked_fill(chosen, float("-inf")).max(2).values
        gap = float((worst_in - best_out).min()) if top_local.shape[2] < dots.shape[2] else float("inf")
        assert gap >= 4 * 2.0 ** -8, f"{name}: boundary gap {gap} too small, change the seed"
        out[f"{name}_top_local"] = top_local.numpy().astype(np.int32)
        out[f"{name}_attn"] = attn.numpy().astype(np.float32)    # [B, 1, H, D]
        out[f"{name}_gap"] = np.float64(gap)
        print(f"{name}: k_eff={top_local.shape[2]} gap={gap:.4f} attn {tuple(attn.shape)}")
    np.savez_compressed(os.path.join(HERE, "spec_vectors.npz"), **out)


if __name__ == "__main__":
    main()
