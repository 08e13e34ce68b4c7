"""Decode loops driven from CUDA graphs, the way the reference's model runner drives them
(src/diffcache/base.py:116-155): the three-call shape captured in two graphs per layer, and the fused
call captured once per layer and replayed past the point where the suffix region is full (window ring,
oldest token spilled into the scanned store)."""
import numpy as np
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-3, 2e-3


def _exact(shape, seed, salt, step, lim):
    """Values that are exact in bf16 (multiples of `step` within +-lim), so that every dot product is
    exact in fp32 and both sides rank rows identically."""
    return np.clip(np.round(util._hash_normal(shape, seed, salt) / step) * step, -lim, lim).astype(np.float32)


def _bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16)


class _OracleModel:
    """Host model of one layer's cache: sink rows, a window of the newest tokens (oldest first), and the
    scanned store that aged-out window tokens move into."""

    def __init__(self, oracle, k, v, prefix, suffix, cap, G):
        # k, v: (B, S, Hkv, D) float32 with bf16-exact values
        B, S, Hkv, D = k.shape
        self.o, self.G, self.P, self.D, self.cap = oracle, G, B * Hkv, D, cap
        to_p = lambda x: util.u16(_bf16(x).permute(0, 2, 1, 3).reshape(B * Hkv, -1, D))  # noqa: E731
        self.sink_k, self.sink_v = to_p(k[:, :prefix]), to_p(v[:, :prefix])
        self.store_k, self.store_v = to_p(k[:, prefix:S - suffix]), to_p(v[:, prefix:S - suffix])
        self.win_k = [to_p(k[:, S - suffix + i:S - suffix + i + 1])[:, 0] for i in range(suffix)]
        self.win_v = [to_p(v[:, S - suffix + i:S - suffix + i + 1])[:, 0] for i in range(suffix)]

    def step(self, q, k_new, v_new, topk):
        """q (B, Hq, D), k_new/v_new (B, Hkv, D) float32.  Returns (selected ids (P, k), out_f32 (P*G, D))."""
        P, D, G = self.P, self.D, self.G
        if len(self.win_k) == self.cap:  # window full: the oldest token moves into the store
            self.store_k = np.concatenate([self.store_k, self.win_k.pop(0)[:, None]], axis=1)
            self.store_v = np.concatenate([self.store_v, self.win_v.pop(0)[:, None]], axis=1)
        self.win_k.append(util.u16(_bf16(k_new).reshape(P, D)))
        self.win_v.append(util.u16(_bf16(v_new).reshape(P, D)))
        qh = util.u16(_bf16(q).reshape(P * G, D))
        qm = self.o.group_mean(qh, G, 0)
        ref = self.o.query(np.ascontiguousarray(self.store_k), np.ascontiguousarray(self.store_v), qm, topk, 0)
        rows_k = np.concatenate([ref["keys"], self.sink_k, np.stack(self.win_k, axis=1)], axis=1)
        rows_v = np.concatenate([ref["vals"], self.sink_v, np.stack(self.win_v, axis=1)], axis=1)
        of, _, _ = self.o.attend(np.ascontiguousarray(rows_k), np.ascontiguousarray(rows_v), qh, G, D ** -0.5, 0)
        return ref["idx"], of


def _make_cache(L, B, Hkv, G, D, S, budget, prefix, suffix, cap, max_length, seed):
    from diffcache_b200 import DiffCache

    cache = DiffCache(L, B, max_length, Hkv, Hkv * G, D, budget, kvbuf_prefix_len=prefix, kvbuf_suffix_len=suffix,
                      kvbuf_suffix_maxlen=cap)
    ks = [_exact((B, S, Hkv, D), seed, 10 + l, 1 / 32, 2.0) for l in range(L)]
    vs = [_exact((B, S, Hkv, D), seed, 20 + l, 1 / 32, 2.0) for l in range(L)]
    for l in range(L):
        cache.prefill_update_kv_cache(_bf16(ks[l]).cuda(), _bf16(vs[l]).cuda(), l)
    return cache, ks, vs


def test_fused_decode_loop_from_one_graph_per_layer(oracle_lib):
    """suffix_maxlen + 50 tokens through ONE captured graph per layer: the window fills, then every token
    spills the oldest one into the store.  Selection and output against a host model at three points, the
    device-side lengths at the end, and an eager run of the same loop bit for bit."""
    L, B, Hkv, G, D, S = 2, 2, 2, 4, 64, 300
    budget, prefix, suffix, cap = 32, 8, 8, 24
    n_tokens = cap + 50
    Hq, P = Hkv * G, B * Hkv
    cache, ks, vs = _make_cache(L, B, Hkv, G, D, S, budget, prefix, suffix, cap, S + n_tokens + 8, seed=5)
    eager, _, _ = _make_cache(L, B, Hkv, G, D, S, budget, prefix, suffix, cap, S + n_tokens + 8, seed=5)
    models = [_OracleModel(oracle_lib, ks[l], vs[l], prefix, suffix, cap, G) for l in range(L)]

    q_in = [torch.zeros((B, Hq, D), dtype=torch.bfloat16, device="cuda") for _ in range(L)]
    k_in = [torch.zeros((B, Hkv, D), dtype=torch.bfloat16, device="cuda") for _ in range(L)]
    v_in = [torch.zeros((B, Hkv, D), dtype=torch.bfloat16, device="cuda") for _ in range(L)]
    outs = [torch.zeros((B, Hq, D), dtype=torch.bfloat16, device="cuda") for _ in range(L)]
    idxs = [torch.zeros((B, Hkv, budget), dtype=torch.int32, device="cuda") for _ in range(L)]
    # warm-up outside capture happens on the twin cache (`eager`), so this one is captured untouched
    graphs = []
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for l in range(L):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                cache.decode_attention(l, q_in[l], k_in[l], v_in[l], out=outs[l], out_idx=idxs[l])
            graphs.append(g)
    torch.cuda.current_stream().wait_stream(side)
    # capture ran the Python side once (host mirrors moved); the device state is untouched
    cache.sync_lengths()
    assert cache.kvbuf_suffix_len == suffix and cache.retrieval_region_len == S - prefix - suffix

    check_at = {1, cap - suffix + 2, n_tokens - 1}  # before the window is full, just after the first spills, the end
    for t in range(n_tokens):
        for l in range(L):
            q = _exact((B, Hq, D), 900 + t, l, 1 / 16, 3.9375)
            kn = _exact((B, Hkv, D), 900 + t, 40 + l, 1 / 32, 2.0)
            vn = _exact((B, Hkv, D), 900 + t, 80 + l, 1 / 32, 2.0)
            q_in[l].copy_(_bf16(q)); k_in[l].copy_(_bf16(kn)); v_in[l].copy_(_bf16(vn))
            graphs[l].replay()
            want_idx, want_out = models[l].step(q, kn, vn, budget)
            e_out = eager.decode_attention(l, _bf16(q).cuda(), _bf16(kn).cuda(), _bf16(vn).cuda())
            if t in check_at:
                torch.cuda.synchronize()
                assert np.array_equal(idxs[l].cpu().numpy().reshape(P, budget), want_idx), f"token {t} layer {l}"
                util.assert_attention_close(util.u16(outs[l]).reshape(P * G, D), want_out, 0, oracle_lib, ATOL, RTOL)
                assert torch.equal(e_out, outs[l]), "graph replay and eager call differ"
    torch.cuda.synchronize()
    for c in (cache, eager):
        for eng in c.data_layers:
            eng.check_status()
    spills = n_tokens - (cap - suffix)
    cache.sync_lengths()
    assert cache.kvbuf_suffix_len == cap
    assert cache.retrieval_region_len == S - prefix - suffix + spills
    assert [e.ctx_len for e in cache.data_layers] == [S - prefix - suffix + spills] * L
    # the eager twin kept its host mirrors up to date without asking the device
    assert eager.kvbuf_suffix_len == cap and eager.retrieval_region_len == S - prefix - suffix + spills
    assert cache.seq_len(0) == S + n_tokens


def test_reference_capture_pattern_two_graphs_per_layer(oracle_lib):
    """The reference's own pattern (base.py:116-155): per layer a graph that ends with
    decode_pre_query_operation and a graph that starts with decode_post_query_operation followed by the
    attention over get_kvcache (here a plain torch attention with the append-at-cache_seqlens behaviour of
    flash_attn_with_kvcache), decode_query_kvcache called between their replays.  Three tokens, compared
    with the host model each time."""
    L, B, Hkv, G, D, S = 2, 1, 2, 4, 64, 260
    budget, prefix, suffix, cap = 48, 8, 12, 16
    Hq, P = Hkv * G, B * Hkv
    cache, ks, vs = _make_cache(L, B, Hkv, G, D, S, budget, prefix, suffix, cap, S + 16, seed=9)
    models = [_OracleModel(oracle_lib, ks[l], vs[l], prefix, suffix, cap, G) for l in range(L)]
    kv = [cache.get_kvcache(l) for l in range(L)]            # (B, rows, Hkv, D) views, fixed for the run
    rows = kv[0][0].shape[1]
    seqlens = torch.zeros(B, dtype=torch.int64, device="cuda")  # the reference's decode_cache_seqlens
    q_in = [torch.zeros((B, 1, Hq * D), dtype=torch.bfloat16, device="cuda") for _ in range(L)]
    k_in = [torch.zeros((B, 1, Hkv, D), dtype=torch.bfloat16, device="cuda") for _ in range(L)]
    v_in = [torch.zeros((B, 1, Hkv, D), dtype=torch.bfloat16, device="cuda") for _ in range(L)]
    outs = [torch.zeros((B, Hq, D), dtype=torch.float32, device="cuda") for _ in range(L)]
    ar_b, ar_r = torch.arange(B, device="cuda"), torch.arange(rows, device="cuda")

    def attention(l):
        kc, vc = kv[l]
        kc.index_put_((ar_b, seqlens), k_in[l][:, 0])        # append at cache_seqlens, in place
        vc.index_put_((ar_b, seqlens), v_in[l][:, 0])
        q = q_in[l].view(B, Hkv, G, D).float()
        s = torch.einsum("bhgd,brhd->bhgr", q, kc.float()) * D ** -0.5
        s = s.masked_fill(ar_r[None, None, None, :] > seqlens[:, None, None, None], float("-inf"))
        outs[l].copy_(torch.einsum("bhgr,brhd->bhgd", torch.softmax(s, dim=-1), vc.float()).reshape(B, Hq, D))

    pre, post = [], []
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for l in range(L):
            g1, g2 = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1, stream=side):
                cache.decode_pre_query_operation(q_in[l])
            with torch.cuda.graph(g2, stream=side):
                cache.decode_post_query_operation(l)
                attention(l)
            pre.append(g1); post.append(g2)
    torch.cuda.current_stream().wait_stream(side)

    for t in range(3):
        for l in range(L):
            q = _exact((B, Hq, D), 700 + t, l, 1 / 16, 3.9375)
            kn = _exact((B, Hkv, D), 700 + t, 40 + l, 1 / 32, 2.0)
            vn = _exact((B, Hkv, D), 700 + t, 80 + l, 1 / 32, 2.0)
            q_in[l].copy_(_bf16(q).reshape(B, 1, Hq * D)); k_in[l].copy_(_bf16(kn).reshape(B, 1, Hkv, D))
            v_in[l].copy_(_bf16(vn).reshape(B, 1, Hkv, D))
            seqlens.fill_(cache.seq_len_gpu(l))                  # base.py:149
            pre[l].replay()
            cache.decode_query_kvcache(l)
            post[l].replay()
            torch.cuda.synchronize()
            _, want_out = models[l].step(q, kn, vn, budget)
            got = outs[l].cpu().numpy().reshape(P * G, D)
            assert np.allclose(got, want_out, rtol=RTOL, atol=ATOL), f"token {t} layer {l}"
    assert cache.kvbuf_suffix_len == suffix + 3
