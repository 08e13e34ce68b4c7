"""CPU tests of the multi-GPU host logic: two gloo ranks run SequenceShardedStep with a numpy
stand-in backend built on the oracle, and the result must equal the unsharded oracle step."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from diffcache_b200 import sharded
from tests import util


def test_shard_rows_cover_and_align():
    for n in (0, 1, 15, 16, 17, 1000, 130496, 1047488):
        for world in (1, 2, 3, 4, 8):
            parts = sharded.shard_rows(n, world)
            assert len(parts) == world and sum(l for _, l in parts) == n
            pos = 0
            for start, length in parts:
                assert start == pos and (start % 16 == 0 or length == 0)
                pos += length
            lens = [l for _, l in parts]
            assert max(lens) - min(lens) <= 32 or n < 16 * world  # one block, plus the ragged last block
    assert sharded.shard_heads(8, 4) == [(0, 2), (2, 2), (4, 2), (6, 2)]
    with pytest.raises(ValueError):
        sharded.shard_heads(8, 3)


class OracleShardBackend:
    """What GpuShardBackend does, restated with the CPU oracle (fp64 attention partials)."""

    def __init__(self, oracle, k_shard, v_shard, row_offset, group, res_k, res_v, k_new, v_new, scale):
        self.o, self.k, self.v, self.off, self.G = oracle, k_shard, v_shard, row_offset, group
        self.res_k, self.res_v, self.k_new, self.v_new, self.scale = res_k, res_v, k_new, v_new, scale
        self.P, self.n, self.D = k_shard.shape

    def local_topk(self, q, k):
        qh = util.u16(q).reshape(self.P * self.G, self.D)
        qm = self.o.group_mean(qh, self.G, 0)
        bits = np.full((self.P, k), sharded.PAD, np.uint32)
        gidx = np.full((self.P, k), sharded.PAD, np.uint32)
        if self.n > 0:
            res = self.o.query(self.k, None, qm, k, 0, gather=False)
            bits[:, :res["ef"]] = res["bits"]
            gidx[:, :res["ef"]] = res["idx"] + self.off
        return torch.from_numpy(bits.view(np.int32)), torch.from_numpy(gidx.view(np.int32))

    def merge(self, bits_all, gidx_all, k):
        b = bits_all.numpy().view(np.uint32)
        g = gidx_all.numpy().view(np.uint32)
        sel = np.stack([self.o.topk(b[p], k, ids=g[p], method="sort")[1] for p in range(self.P)])
        return torch.from_numpy(sel.view(np.int32))

    def merge_count(self, bits_all, k, rank):
        """Order all candidates by (key, rank, position), keep the first k valid ones, count this rank's."""
        b = bits_all.numpy().view(np.uint32)                      # (world, P, k)
        world = b.shape[0]
        out = np.zeros(self.P, np.int32)
        for p in range(self.P):
            keys = [(int(b[r, p, i]), r, i) for r in range(world) for i in range(k) if b[r, p, i] != sharded.PAD]
            out[p] = sum(1 for _, r, _ in sorted(keys)[:k] if r == rank)
        return torch.from_numpy(out)

    def attend_owned(self, q, sel, count=None):
        qf = self.o.to_f32(util.u16(q).reshape(self.P * self.G, self.D), 0).astype(np.float64)
        s_ids = sel.numpy().view(np.uint32).astype(np.int64)
        if count is not None:
            s_ids = [s_ids[p][:int(count[p])] for p in range(self.P)]
        acc = np.zeros((self.P * self.G, self.D), np.float32)
        ml = np.zeros((self.P * self.G, 2), np.float32)
        for p in range(self.P):
            own = s_ids[p][(s_ids[p] >= self.off) & (s_ids[p] < self.off + self.n)] - self.off
            ks, vs = [self.k[p][own]], [self.v[p][own]]
            if self.res_k is not None:
                ks.append(self.res_k[p]); vs.append(self.res_v[p])
            if self.k_new is not None:
                ks.append(self.k_new[p][None]); vs.append(self.v_new[p][None])
            kk = self.o.to_f32(np.ascontiguousarray(np.concatenate(ks)), 0).astype(np.float64)
            vv = self.o.to_f32(np.ascontiguousarray(np.concatenate(vs)), 0).astype(np.float64)
            for g in range(self.G):
                r = p * self.G + g
                if kk.shape[0] == 0:
                    ml[r] = (-np.inf, 0.0)
                    continue
                s = kk @ qf[r] * self.scale * np.log2(np.e)
                m = s.max()
                w = np.exp2(s - m)
                acc[r] = w @ vv
                ml[r] = (m, w.sum())
        return torch.from_numpy(acc), torch.from_numpy(ml)

    def combine_packed(self, parts, rows, D):
        parts = parts.numpy()
        acc_all = parts[:, :rows * D].reshape(-1, rows, D)
        ml_all = parts[:, rows * D:].reshape(-1, rows, 2)
        a, m = acc_all.astype(np.float64), ml_all.astype(np.float64)
        mx = m[..., 0].max(axis=0)
        with np.errstate(invalid="ignore"):
            w = np.where(np.isinf(m[..., 0]), 0.0, np.exp2(m[..., 0] - mx))
        out = (a * w[..., None]).sum(0) / (m[..., 1] * w).sum(0)[:, None]
        return torch.from_numpy(out.astype(np.float32))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, tmpdir):
    import oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, Hkv, G, D, n_r, sink, win, topk = 1, 2, 4, 128, 3001, 16, 24, 700  # shard 2 holds fewer rows than top-k
        P = B * Hkv
        k, v, q = util.small_problem(B, Hkv, G, sink + n_r + win, D, seed=77)
        ku, vu = util.u16(k).reshape(P, -1, D), util.u16(v).reshape(P, -1, D)
        parts = sharded.shard_rows(n_r, world)
        start, length = parts[rank]
        ks = np.ascontiguousarray(ku[:, sink + start:sink + start + length])
        vs = np.ascontiguousarray(vu[:, sink + start:sink + start + length])
        res_k = res_v = k_new = v_new = None
        if rank == 0:
            res_k, res_v = ku[:, :sink], vu[:, :sink]
        if rank == world - 1:
            wk, wv = ku[:, sink + n_r:-1], vu[:, sink + n_r:-1]
            res_k = wk if res_k is None else np.concatenate([res_k, wk], 1)
            res_v = wv if res_v is None else np.concatenate([res_v, wv], 1)
            k_new, v_new = ku[:, -1], vu[:, -1]
        backend = OracleShardBackend(oracle, ks, vs, start, G, res_k, res_v, k_new, v_new, D ** -0.5)
        step = sharded.SequenceShardedStep(backend, topk)
        fast = step.step(q).numpy()                         # keys only: prefix counts
        out = step.step(q, want_selection=True).numpy()     # also the full merge with ids
        assert np.array_equal(fast, out)
        sel = step.last_selection.numpy().view(np.uint32)
        gidx, count = step.last_owned
        for p in range(P):                                  # my prefix = the selected rows in my range
            mine = set(int(x) for x in gidx.numpy().view(np.uint32)[p][:int(count[p])])
            assert mine == set(int(x) for x in sel[p] if start <= x < start + length)
        # unsharded reference
        ref = util.oracle_decode_step(
            oracle, np.ascontiguousarray(ku[:, sink:sink + n_r]), np.ascontiguousarray(vu[:, sink:sink + n_r]),
            util.u16(q).reshape(P * G, D), G, topk,
            np.ascontiguousarray(np.concatenate([ku[:, :sink], ku[:, sink + n_r:-1]], 1)),
            np.ascontiguousarray(np.concatenate([vu[:, :sink], vu[:, sink + n_r:-1]], 1)),
            np.ascontiguousarray(ku[:, -1]), np.ascontiguousarray(vu[:, -1]), D ** -0.5, 0)
        assert np.array_equal(sel, ref["idx"]), "merged selection differs from the unsharded top-k"
        assert np.allclose(out, ref["out_f32"], rtol=1e-5, atol=1e-6)
        open(os.path.join(tmpdir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_sharded_step_on_gloo_ranks(tmp_path, oracle_lib, world):
    port = _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
