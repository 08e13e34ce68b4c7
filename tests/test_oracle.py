"""CPU tests: the oracle against the golden vectors and against independent restatements."""
import numpy as np
import pytest
import torch

from tests import util


def test_select_kat_heap_and_sort(oracle_lib):
    for case in util.load_select_kat():
        vals = np.asarray(case["values"], np.int64)
        # order-preserving map into positive-float bit patterns (the reference compares dist as
        # f32 and as raw bits, which agree only for dist >= 0: nsw.rs:127,136-137)
        bits = (vals + util.KAT_OFFSET).astype(np.uint32)
        for method in ("heap", "sort"):
            ob, oi = oracle_lib.topk(bits, case["cap"], method=method)
            got = (ob.astype(np.int64) - util.KAT_OFFSET).tolist()
            assert got == case["expected"], case["name"]
            # ties go to the smaller position, keys strictly ascending
            keys = (ob.astype(np.uint64) << np.uint64(32)) | oi.astype(np.uint64)
            assert np.all(keys[1:] > keys[:-1])
            assert np.array_equal(bits[oi], ob)


def test_heap_equals_sort_on_tie_heavy_streams(oracle_lib):
    rng = np.random.default_rng(1)
    for trial in range(200):
        n = int(rng.integers(1, 400))
        ef = int(rng.integers(1, 64))
        # quantised positive floats: many exact ties, like fp32(65536 - dot)
        d = (65536.0 - np.round(rng.normal(0, 3, n) * 4) / 4).astype(np.float32)
        bits = d.view(np.uint32)
        hb, hi = oracle_lib.topk(bits, ef, method="heap")
        sb, si = oracle_lib.topk(bits, ef, method="sort")
        assert np.array_equal(hb, sb) and np.array_equal(hi, si)


def test_conversions_match_torch_and_numpy(oracle_lib):
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(200000) * np.exp(rng.standard_normal(200000) * 4)).astype(np.float32)
    x[:8] = [0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 6e-8, -3e-5]
    want_bf = torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(oracle_lib.from_f32(x, 0), want_bf)
    with np.errstate(over="ignore"):
        want_h = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(oracle_lib.from_f32(x, 1), want_h)
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    got = oracle_lib.to_f32(allh, 1)
    ok = ~np.isnan(ref)
    assert np.array_equal(got.view(np.uint32)[ok], ref.view(np.uint32)[ok])
    assert np.array_equal(oracle_lib.to_f32(allh, 0).view(np.uint32), allh.astype(np.uint32) << 16)


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
def test_group_mean_matches_torch_mean(oracle_lib, dtype):
    """The reference forms the retrieval query with torch's CUDA mean over a 16-bit tensor
    (src/diffcache/kvcache/diffcache.py:193): fp32 sum, times 1/G, one rounding.  (torch's CPU
    kernel rounds the sum to 16 bits before dividing, so it is only compared where that is exact;
    the CUDA kernel is compared on a device in tests/test_gpu_parity.py.)"""
    td = {"bf16": torch.bfloat16, "fp16": torch.float16}[dtype]
    g = torch.Generator().manual_seed(3)
    for group in (1, 2, 4, 7, 8):
        q = (torch.randn(6, 4, group, 128, generator=g) * 3).to(td)
        got = oracle_lib.group_mean(util.u16(q.reshape(-1, 128)), group, util.dtype_code(dtype))
        acc = torch.zeros(6, 4, 128)
        for j in range(group):
            acc = acc + q[:, :, j].float()
        want = (acc * torch.tensor(1.0 / group, dtype=torch.float32)).to(td)
        assert np.array_equal(got, util.u16(want.reshape(-1, 128)))
        if group == 1:
            assert np.array_equal(got, util.u16(q.mean(dim=2).reshape(-1, 128)))


def test_scores_match_float64_definition(oracle_lib):
    g = torch.Generator().manual_seed(4)
    k = (torch.randn(3000, 128, generator=g) * 2).to(torch.bfloat16)
    q = (torch.randn(128, generator=g) * 2).to(torch.bfloat16)
    bits = oracle_lib.score_rows(util.u16(k), util.u16(q), 0)
    dot = (k.double() @ q.double()).numpy()
    want = (np.float32(65536.0) - dot.astype(np.float32)).astype(np.float32)
    assert np.array_equal(bits, want.view(np.uint32))
    fast = oracle_lib.score_rows(util.u16(k), util.u16(q), 0, exact=False)
    # fp32 accumulation may move a value by at most one dist ulp
    assert np.max(np.abs(fast.view(np.float32).astype(np.float64) - want.astype(np.float64))) <= 2 ** -7


def test_query_orders_and_gathers(oracle_lib):
    k, v, q = util.small_problem(2, 2, 4, 5000, 128, seed=5)
    P = 4
    ku, vu = util.u16(k).reshape(P, 5000, 128), util.u16(v).reshape(P, 5000, 128)
    qm = oracle_lib.group_mean(util.u16(q).reshape(-1, 128), 4, 0)
    res = oracle_lib.query(ku, vu, qm, 300, 0)
    for p in range(P):
        bits = oracle_lib.score_rows(ku[p], qm[p], 0)
        sb, si = oracle_lib.topk(bits, 300, method="sort")
        assert np.array_equal(res["idx"][p], si) and np.array_equal(res["bits"][p], sb)
        assert np.array_equal(res["keys"][p], ku[p][si]) and np.array_equal(res["vals"][p], vu[p][si])
    # ef larger than the store is clamped (lib.rs:374)
    res2 = oracle_lib.query(ku[:, :50].copy(), vu[:, :50].copy(), qm, 300, 0)
    assert res2["ef"] == 50 and res2["idx"].shape == (P, 50)


def test_attention_matches_torch_float64(oracle_lib):
    g = torch.Generator().manual_seed(6)
    P, G, n, D = 3, 4, 257, 128
    k = torch.randn(P, n, D, generator=g).to(torch.bfloat16)
    v = torch.randn(P, n, D, generator=g).to(torch.bfloat16)
    q = torch.randn(P * G, D, generator=g).to(torch.bfloat16)
    scale = D ** -0.5
    of, oe, lse = oracle_lib.attend(util.u16(k), util.u16(v), util.u16(q), G, scale, 0)
    s = torch.einsum("pgd,pnd->pgn", q.view(P, G, D).double(), k.double()) * scale
    want = torch.einsum("pgn,pnd->pgd", torch.softmax(s, -1), v.double()).reshape(P * G, D)
    assert np.allclose(of, want.float().numpy(), rtol=1e-6, atol=1e-7)
    assert np.array_equal(oe, util.u16(want.float().to(torch.bfloat16)))
    assert np.allclose(lse, torch.logsumexp(s, -1).reshape(-1).float().numpy(), rtol=1e-6)


def test_pq_definitions(oracle_lib):
    rng = np.random.default_rng(7)
    P, D, M, n = 2, 128, 16, 1000
    cen = rng.standard_normal((P, M, 256, D // M)).astype(np.float32)
    q = torch.randn(P, D).to(torch.bfloat16)
    lut = oracle_lib.pq_build_lut(util.u16(q), cen, M, 0)
    want = np.einsum("pmd,pmcd->pmc", q.float().numpy().reshape(P, M, D // M).astype(np.float64), cen.astype(np.float64))
    assert np.allclose(lut, want, rtol=1e-5, atol=1e-5)
    codes = rng.integers(0, 256, (n, M), dtype=np.uint8)
    bits = oracle_lib.pq_adc_scores(codes, lut[0])
    s = np.zeros(n, np.float32)
    for m in range(M):
        s = (s + lut[0, m, codes[:, m]]).astype(np.float32)
    assert np.array_equal(bits, (np.float32(65536.0) - s).astype(np.float32).view(np.uint32))


def test_k_check_against_numpy_fit(oracle_lib):
    """fit_alpha_from_logits / estimate_top_h_mass (nsw.rs:198-283) restated with numpy."""
    rng = np.random.default_rng(8)
    D = 128
    for alpha_true in (0.7, 1.3, 2.5):
        ranks = np.arange(1, 1025)
        z = (6.0 - alpha_true * np.log(ranks) + rng.normal(0, 0.05, ranks.size)).astype(np.float32)
        z = np.sort(z)[::-1].copy()
        dist = (np.float32(65536.0) - z * np.float32(np.sqrt(D))).astype(np.float32)
        zz = ((np.float32(65536.0) - dist) / np.float32(np.sqrt(D))).astype(np.float32)  # what the engine sees
        for h in (100, 400, 1024):
            ok, alpha, mass = oracle_lib.k_check(dist.view(np.uint32)[:h], D, 0.9)
            x = np.log(np.arange(5, h + 1, dtype=np.float64))
            slope = np.polyfit(x, zz[4:h].astype(np.float64), 1)[0]
            assert abs(alpha - (-slope)) < 1e-4
            if -slope > 1.0:
                head = np.exp(zz[:h].astype(np.float64) - zz[0]).sum()
                tail = np.exp(float(zz[h - 1]) - float(zz[0])) * h / (-slope - 1.0)
                assert abs(mass - head / (head + tail)) < 1e-4
                assert ok == (mass >= 0.9)
            else:
                assert not ok
        seq = [100, 200, 400, 800]
        got = oracle_lib.adaptive_budget(dist.view(np.uint32), D, seq, 0.9)
        want = next((h for h in seq if oracle_lib.k_check(dist.view(np.uint32)[:h], D, 0.9)[0]), 1024)
        assert got == want


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("name", sorted(util.SPEC_CASES))
def test_oracle_matches_reference_functional_spec(oracle_lib, name, dtype):
    """The oracle's decode step against outputs of the reference's own PyTorch statement of the path
    (exact branch of gqa_topk_attention, tools/topk_test.py:303-470; fixtures written by
    tests/golden/make_spec_vectors.py): same rows chosen per kv head inside the retrieval region,
    chosen rows ranked consistently with the reference's ordering, same attention output."""
    case = util.SPEC_CASES[name]
    gold = util.load_spec_vectors()
    top_local, attn = gold[f"{name}_top_local"], gold[f"{name}_attn"]
    sp = util.spec_case_split(case, *util.spec_case_inputs(case))
    B, KV, G, D = case["batch"], case["kv_heads"], case["group"], case["head_dim"]
    P, n = B * KV, sp["n_store"]
    enc = lambda a: oracle_lib.from_f32(np.ascontiguousarray(a, dtype=np.float32), dtype)  # noqa: E731
    for a in sp.values():  # the inputs are exact in both 16-bit types
        if isinstance(a, np.ndarray):
            assert np.array_equal(oracle_lib.to_f32(enc(a), dtype), a)
    ref = util.oracle_decode_step(
        oracle_lib, enc(sp["store_k"]).reshape(P, n, D), enc(sp["store_v"]).reshape(P, n, D),
        enc(sp["q"]).reshape(P * G, D), G, case["top_k"], enc(sp["res_k"]).reshape(P, -1, D),
        enc(sp["res_v"]).reshape(P, -1, D), enc(sp["k_new"]).reshape(P, D), enc(sp["v_new"]).reshape(P, D),
        D ** -0.5, dtype)
    want = top_local.reshape(P, -1)
    assert ref["idx"].shape == want.shape
    for p in range(P):
        assert set(ref["idx"][p].tolist()) == set(want[p].tolist())
        # the reference lists its rows best first; the engine's ranking key must not decrease along it
        keys_in_ref_order = ref["all_bits"][p][want[p]]
        assert np.all(np.diff(keys_in_ref_order.astype(np.int64)) >= 0)
        assert np.all(np.diff(ref["bits"][p].astype(np.int64)) >= 0)
    np.testing.assert_allclose(ref["out_f32"].reshape(B, 1, KV * G, D), attn, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("name", sorted(util.KVCACHE_CASES))
def test_reference_kvcache_layout_fixture(oracle_lib, name):
    """What the reference's KV-cache manager hands to attention after one decode step
    (tests/golden/kvcache_vectors.npz, written by running its class) is, per kv head,
    [top rows of the middle region, best first | first `prefix` tokens | last `suffix` tokens] in the
    (B, rows, Hkv, D) view of get_kvcache (diffcache.py:186-189), with the rows the oracle selects."""
    c = util.KVCACHE_CASES[name]
    gold = util.load_kvcache_vectors()
    B, KV, G, D, S = c["batch"], c["kv_heads"], c["group"], c["head_dim"], c["seq_len"]
    p, s = min(c["prefix"], S), min(c["suffix"], S - min(c["prefix"], S))
    for layer in range(c["num_layers"]):
        k, v, q = util.kvcache_case_inputs(c, layer)
        enc = lambda a: oracle_lib.from_f32(np.ascontiguousarray(a, dtype=np.float32), 0)  # noqa: E731
        mid_k = np.ascontiguousarray(k[:, p:S - s].transpose(0, 2, 1, 3)).reshape(B * KV, S - s - p, D)
        mid_v = np.ascontiguousarray(v[:, p:S - s].transpose(0, 2, 1, 3)).reshape(B * KV, S - s - p, D)
        qm = oracle_lib.group_mean(enc(q.reshape(B * KV * G, D)), G, 0)
        res = oracle_lib.query(enc(mid_k), enc(mid_v), qm, c["budget"], 0)
        ef = res["ef"]
        assert ef == min(c["budget"], S - s - p)
        assert np.array_equal(res["idx"].reshape(B, KV, ef), gold[f"{name}_l{layer}_idx"])
        for src, got, rows in ((k, gold[f"{name}_l{layer}_k"], res["keys"]), (v, gold[f"{name}_l{layer}_v"], res["vals"])):
            want = np.concatenate([rows.reshape(B, KV, ef, D).transpose(0, 2, 1, 3), enc(src[:, :p]), enc(src[:, S - s:])], axis=1)
            assert np.array_equal(got, want)


def test_k_check_alpha_matches_reference_prototype(oracle_lib):
    """The exponent the oracle's k-check fits (nsw.rs:198-240) against the reference's Python prototype
    of the same fit (fit_powerlaw_alpha_from_head, tools/analyze_attn_samples.ipynb; fixture written by
    tests/golden/make_kcheck_vectors.py)."""
    gold = util.load_kcheck_vectors()
    for name, case in util.KCHECK_CASES.items():
        bits = util.kcheck_case_bits(case)
        assert bits.shape[0] == gold[name]["n"] and np.all(np.diff(bits.astype(np.int64)) >= 0)
        _, alpha, _ = oracle_lib.k_check(bits, case["head_dim"], 0.9)
        assert abs(alpha - gold[name]["alpha"]) <= 1e-4 * max(1.0, abs(gold[name]["alpha"])), (name, alpha)
