"""Two real GPUs, NCCL: the sequence-sharded step of diffcache_b200.sharded against the single-GPU
fused step on the same data.  Skipped on boxes with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, tmpdir):
    import torch.distributed as dist

    from diffcache_b200 import DiffCacheGPU, sharded, synth

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        B, Hkv, G, D, n_r, sink, win, topk = 1, 4, 4, 128, 40000, 64, 128, 2048
        k, v = synth.make_kv(B, Hkv, sink + n_r + win, D, seed=5, dtype="bf16")
        q = synth.make_query(k[:, :, sink:sink + n_r], G, seed=5).cuda()
        start, length = sharded.shard_rows(n_r, world)[rank]
        eng = DiffCacheGPU(B, Hkv * G, Hkv, D, max_ctx_len=length, device=rank)
        eng.prefill(k[:, :, sink + start:sink + start + length].contiguous().cuda().view(torch.uint16),
                    v[:, :, sink + start:sink + start + length].contiguous().cuda().view(torch.uint16))
        res_k = res_v = kn = vn = None
        rows = 0
        if rank == 0 or rank == world - 1:
            lo, hi = (0, sink) if rank == 0 else (sink + n_r, sink + n_r + win - 1)
            rows = hi - lo
            res_k = torch.zeros((B, Hkv, rows + 2, D), dtype=torch.bfloat16, device="cuda")
            res_v = torch.zeros_like(res_k)
            res_k[:, :, :rows] = k[:, :, lo:hi].cuda(); res_v[:, :, :rows] = v[:, :, lo:hi].cuda()
            if rank == world - 1:
                kn, vn = k[:, :, -1].contiguous().cuda(), v[:, :, -1].contiguous().cuda()
        backend = sharded.GpuShardBackend(eng, start, res_k, res_v, rows, kn, vn)
        step = sharded.SequenceShardedStep(backend, topk)     # NCCL all-gathers
        fast = step.step(q).clone()                          # keys-only exchange, prefix counts
        out = step.step(q, want_selection=True).clone()      # also ids + the full merge select
        sel = step.last_selection.clone()
        assert torch.equal(fast, out)
        # the same step with both exchanges done by the step's own kernels over NVLink peer stores
        peer_step = sharded.SequenceShardedStep(backend, topk, exchange="peer")
        for _ in range(3):   # later rounds find the earlier rounds' blocks and epochs in the buffers
            assert torch.equal(peer_step.step(q), fast)
        g = torch.cuda.CUDAGraph()   # ... and replayed from a CUDA graph
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.cuda.graph(g, stream=side):
            captured = peer_step.step(q)
        torch.cuda.current_stream().wait_stream(side)
        dist.barrier()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        assert torch.equal(captured, fast)
        # soak: 200 replays back to back with a different query each time (no host synchronisation between most
        # of them, so the ranks drift apart as far as the protocol lets them); every checked output must equal
        # what the NCCL path gives for that query
        queries = [synth.make_query(k[:, :, sink:sink + n_r], G, seed=50 + i).cuda() for i in range(5)]
        wants = [step.step(qi).clone() for qi in queries]
        qbuf = queries[0].clone()
        g2 = torch.cuda.CUDAGraph()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.cuda.graph(g2, stream=side):
            soaked = peer_step.step(qbuf)
        torch.cuda.current_stream().wait_stream(side)
        dist.barrier()
        for it in range(200):
            qbuf.copy_(queries[it % 5])
            g2.replay()
            if it % 16 == 0 or it >= 195:
                assert torch.equal(soaked, wants[it % 5]), f"replay {it}"
        peer_step.xchg.check()
        eng.check_status()
        torch.cuda.synchronize()
        if rank == 0:  # single-GPU fused step on the whole sequence
            full = DiffCacheGPU(B, Hkv * G, Hkv, D, max_ctx_len=n_r, device=0)
            full.prefill(k[:, :, sink:sink + n_r].contiguous().cuda().view(torch.uint16),
                         v[:, :, sink:sink + n_r].contiguous().cuda().view(torch.uint16))
            rk = torch.zeros((B, Hkv, sink + win + 2, D), dtype=torch.bfloat16, device="cuda")
            rv = torch.zeros_like(rk)
            rk[:, :, :sink] = k[:, :, :sink].cuda(); rv[:, :, :sink] = v[:, :, :sink].cuda()
            rk[:, :, sink:sink + win - 1] = k[:, :, sink + n_r:-1].cuda(); rv[:, :, sink:sink + win - 1] = v[:, :, sink + n_r:-1].cuda()
            want = torch.empty_like(out)
            idx = torch.zeros((B, Hkv, topk), dtype=torch.int32, device="cuda")
            full.decode_attend(q, want, topk, res_k=rk, res_v=rv, res_len=sink + win - 1,
                               k_new=k[:, :, -1].contiguous().cuda(), v_new=v[:, :, -1].contiguous().cuda(), out_idx=idx)
            full.check_status()
            torch.cuda.synchronize()
            assert torch.equal(sel.view(B, Hkv, topk), idx), "sharded and single-GPU selections differ"
            assert torch.allclose(out.float(), want.float(), rtol=2e-3, atol=1e-3)
            full.close()
        eng.close()
        dist.barrier()
        open(os.path.join(tmpdir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def _stack_rank_main(rank, world, port, tmpdir):
    import torch.distributed as dist

    from diffcache_b200.stack import AttentionStack

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        kw = dict(n_layers=3, hidden=512, batch=2, q_heads=16, kv_heads=4, head_dim=128, context=6000, topk=512, sink=16,
                  window=48, dtype="bf16", seed=77, device=torch.device("cuda", rank))
        sharded_stack = AttentionStack(**kw)                       # kv heads split over the two ranks, NCCL all-gather
        x = torch.randn((2, 512), generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
        y = sharded_stack.step(x).clone()
        for e in sharded_stack.engines:
            e.check_status()
        torch.cuda.synchronize()
        # the all-gather done by peer stores instead: both sides inside the attention's merge kernel (default), and
        # with the consumer side left to the separate wait-and-unpack kernel
        for fused in ("1", "0"):
            os.environ["DC_STACK_FUSED_GATHER"] = fused
            peer_stack = AttentionStack(exchange="peer", **kw)
            assert peer_stack.exchange == "peer" and peer_stack.fused_gather == (fused == "1")
            for _ in range(3):
                assert torch.equal(peer_stack.step(x), y)
            peer_stack.xchg.check()
            dist.barrier()
            peer_stack.close()
        os.environ.pop("DC_STACK_FUSED_GATHER", None)
        if rank == 0:  # the same stack on one GPU: world of one
            solo = AttentionStack(unsharded=True, **kw)
            want = solo.step(x)
            torch.cuda.synchronize()
            assert torch.allclose(y.float(), want.float(), rtol=2e-2, atol=2e-2), (y.float() - want.float()).abs().max()
            solo.close()
        sharded_stack.close()
        dist.barrier()
        open(os.path.join(tmpdir, f"stack_ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_head_sharded_stack_on_two_gpus(tmp_path):
    """Configuration-2 shape in small: the kv-head-sharded attention stack on two GPUs (one all-gather of
    the attention output per layer) against the same stack on one GPU."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_stack_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "stack_ok0").exists() and (tmp_path / "stack_ok1").exists()


def test_sequence_sharded_step_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
