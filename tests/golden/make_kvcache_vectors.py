"""Writes tests/golden/kvcache_vectors.npz: the state the reference's KV-cache manager
(class DiffCache, src/diffcache/kvcache/diffcache.py:15-300) reaches after prefill and one decode
step on the seeded inputs of tests/util.py::kvcache_case_inputs.

The class is loaded unmodified from a checkout of the reference (first argument or
$DIFFCACHE_REFERENCE) and run on CPU.  What it imports but this machine lacks is stood in for,
outside the class: `diffcache._cpu` (the Rust engine; here a recorder that answers `query` with the
CPU oracle's exact top rows), `cuvs.neighbors.cagra` (graph build; returns an empty graph, which
only the engine would read), `codetiming.Timer` (no-op), and the CUDA placement of its buffers
(device='cuda' -> 'cpu', pin_memory -> identity, synchronize -> no-op).  Everything recorded is
produced by the reference's own statements: the region split, the buffer layout
[retrieved, right-aligned | prefix | suffix], get_kvcache, seq_len / seq_len_gpu, the arguments
it hands to the engine, and the suffix bookkeeping.

Run from the repository root:
    python tests/golden/make_kvcache_vectors.py /path/to/DiffCache
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

sys.dont_write_bytecode = True
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from tests.util import KVCACHE_CASES, kvcache_case_inputs  # noqa: E402


class RecordingEngine:
    """Stands in for diffcache._cpu.DiffCacheCPU (diffcache_cpu/src/lib.rs:523-660)."""

    def __init__(self, **kw):
        self.kw = kw
        self.calls = []

    def update_r_sq(self, r_sq):
        self.calls.append(("update_r_sq", len(r_sq)))

    def prefill(self, k, v, neighbours):
        assert k.dtype == np.uint16 and k.flags["C_CONTIGUOUS"] and neighbours.dtype == np.uint32
        self.k, self.v = k.copy(), v.copy()
        self.calls.append(("prefill", k.shape))

    def query(self, out_k, out_v, q, ef):
        B, H, n, D = self.k.shape
        self.calls.append(("query", tuple(out_k.shape), int(ef)))
        res = oracle.query(self.k.reshape(B * H, n, D), self.v.reshape(B * H, n, D), q.reshape(B * H, D), ef, oracle.BF16)
        got = res["ef"]
        out_k[:, :, :got, :] = res["keys"].reshape(B, H, got, D)
        out_v[:, :, :got, :] = res["vals"].reshape(B, H, got, D)
        self.last_idx = res["idx"].reshape(B, H, got)


def load_reference_class(ref):
    src = os.path.join(ref, "src", "diffcache")
    path = os.path.join(src, "kvcache", "diffcache.py")
    if not os.path.isfile(path):
        raise SystemExit("usage: make_kvcache_vectors.py <DiffCache checkout>")
    timer = types.ModuleType("codetiming")

    class Timer:
        def __init__(self, *a, **kw): pass
        def __enter__(self): return self
        def __exit__(self, *a): return False
    timer.Timer = Timer
    sys.modules["codetiming"] = timer

    cagra = types.ModuleType("cuvs.neighbors.cagra")
    cagra.IndexParams = lambda **kw: types.SimpleNamespace(**kw)
    cagra.build = lambda params, data: types.SimpleNamespace(graph=types.SimpleNamespace(
        copy_to_host=lambda: np.zeros((data.shape[0], params.graph_degree), np.uint32)))
    cuvs, neigh = types.ModuleType("cuvs"), types.ModuleType("cuvs.neighbors")
    neigh.cagra = cagra
    cuvs.neighbors = neigh
    sys.modules.update({"cuvs": cuvs, "cuvs.neighbors": neigh, "cuvs.neighbors.cagra": cagra})

    pkg, sub, eng = types.ModuleType("diffcache"), types.ModuleType("diffcache.kvcache"), types.ModuleType("diffcache._cpu")
    pkg.__path__, sub.__path__ = [src], [os.path.join(src, "kvcache")]
    eng.DiffCacheCPU, eng.init_metrics = RecordingEngine, (lambda: None)
    sys.modules.update({"diffcache": pkg, "diffcache.kvcache": sub, "diffcache._cpu": eng})
    spec = importlib.util.spec_from_file_location("diffcache.kvcache.diffcache", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod.DiffCache


def on_cpu(fn):
    def wrapped(*a, **kw):
        if kw.get("device") == "cuda":
            kw["device"] = "cpu"
        return fn(*a, **kw)
    return wrapped


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DIFFCACHE_REFERENCE", "")
    DiffCache = load_reference_class(ref)
    real_zeros = torch.zeros
    torch.zeros = on_cpu(real_zeros)
    torch.empty = on_cpu(real_zeros)          # defined contents for rows the class never writes
    torch.Tensor.pin_memory = lambda self: self
    torch.cuda.synchronize = lambda: None
    u16 = lambda t: t.contiguous().view(torch.uint16).numpy().copy()  # noqa: E731
    out = {}
    for name, c in KVCACHE_CASES.items():
        L, B, KV, G, D = c["num_layers"], c["batch"], c["kv_heads"], c["group"], c["head_dim"]
        cache = DiffCache(num_layers=L, batch_size=B, max_length=c["max_length"], num_kv_heads=KV, num_q_heads=KV * G,
                          head_dim=D, retrieval_budget=c["budget"], nsw_m=4, nsw_ef_cons=16,
                          kvbuf_prefix_len=c["prefix"], kvbuf_suffix_len=c["suffix"], kvbuf_suffix_maxlen=c["suffix_max"],
                          attn_mass_threshold=0.9, k_check_seq=[1048576], r_sq=[[4.0] * KV for _ in range(L)])
        ins = [kvcache_case_inputs(c, layer) for layer in range(L)]
        for layer in range(L):
            k, v, _ = ins[layer]
            cache.prefill_update_kv_cache(torch.from_numpy(k).bfloat16(), torch.from_numpy(v).bfloat16(), layer)
            eng = cache.data_layers[layer]
            p, s = cache.kvbuf_prefix_len, cache.kvbuf_suffix_len
            want = np.ascontiguousarray(k[:, p:c["seq_len"] - s].transpose(0, 2, 1, 3))
            assert np.array_equal(oracle.to_f32(eng.k, oracle.BF16), want)   # engine got the middle region, (B,Hkv,S',D)
            out[f"{name}_l{layer}_r_sq"] = np.asarray(cache.r_sq[layer], np.float64)
        out[f"{name}_after_prefill"] = np.asarray(
            [cache.kvbuf_prefix_len, cache.kvbuf_suffix_len, cache.retrieval_region_len, cache.seq_len(0), cache.seq_len_gpu(0)],
            np.int64)
        for layer in range(L):
            q = torch.from_numpy(ins[layer][2]).bfloat16()
            cache.decode_pre_query_operation(q)
            cache.decode_query_kvcache(layer)
            cache.decode_post_query_operation(layer)
            kk, vv = cache.get_kvcache(layer)                     # (B, rows, Hkv, D) views
            rows = min(cache.retrieval_region_len, c["budget"]) + c["prefix"] + c["suffix"]   # written rows
            out[f"{name}_l{layer}_k"] = u16(kk[:, :rows])
            out[f"{name}_l{layer}_v"] = u16(vv[:, :rows])
            out[f"{name}_l{layer}_shape"] = np.asarray(kk.shape, np.int64)
            out[f"{name}_l{layer}_idx"] = cache.data_layers[layer].last_idx.astype(np.int32)
            out[f"{name}_l{layer}_query_call"] = np.asarray(
                [x for call in cache.data_layers[layer].calls if call[0] == "query" for x in (*call[1], call[2])], np.int64)
        out[f"{name}_after_step"] = np.asarray(
            [cache.kvbuf_prefix_len, cache.kvbuf_suffix_len, cache.retrieval_region_len, cache.seq_len(0), cache.seq_len_gpu(0)],
            np.int64)
        print(name, out[f"{name}_after_prefill"], out[f"{name}_after_step"], out[f"{name}_l0_shape"],
              out[f"{name}_l0_query_call"])
    np.savez_compressed(os.path.join(HERE, "kvcache_vectors.npz"), **out)


if __name__ == "__main__":
    main()
