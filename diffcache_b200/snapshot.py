"""Engine snapshots: the replacement for ``DiffCacheCPU.save`` / ``load``.

The reference writes one bincode ``IndexSnapshot{nodes, keys: f32, vals: f32, options, dim,
num_nodes}`` per (batch, kv-head) to ``{path}b{b:03}_h{h:03}.idx``
(diffcache_cpu/src/lib.rs:484-506, diffcache_cpu/src/nsw.rs:58-72,704-794).  The graph
(``nodes``) has no meaning for an exact scan and bincode/serde are Rust-only, so the file
keeps the reference's NAMES (same prefix rule: ``path`` is used as a string prefix, not a
directory) with this little-endian layout:

    offset  0  8 bytes  magic  b"DCB2IDX1"
    offset  8  u32      head_dim
    offset 12  u32      element type (0 = bf16, 1 = fp16)
    offset 16  u64      num_nodes
    offset 24  u16[num_nodes * head_dim]  keys (raw 16-bit patterns)
    then       u16[num_nodes * head_dim]  values
"""
from __future__ import annotations

import struct

import numpy as np

from . import _lib

MAGIC = b"DCB2IDX1"


def _file(path: str, b: int, h: int) -> str:
    return f"{path}b{b:03d}_h{h:03d}.idx"


def save_engine(engine, path: str) -> None:
    n = engine.ctx_len
    shape = (engine.bsz, engine.kv_head_num, n, engine.head_dim)
    k = np.empty(shape, np.uint16)
    v = np.empty(shape, np.uint16)
    _lib.check(engine._lib.dc_export_rows(engine._h, k.ctypes.data, v.ctypes.data))
    for b in range(engine.bsz):
        for h in range(engine.kv_head_num):
            with open(_file(path, b, h), "wb") as f:
                f.write(MAGIC)
                f.write(struct.pack("<IIQ", engine.head_dim, engine.dtype, n))
                f.write(k[b, h].tobytes())
                f.write(v[b, h].tobytes())


def load_engine(engine, path: str, ctx_len: int) -> None:
    """``ctx_len`` is the full prompt length the reference passes (lib.rs:496-506); the number of
    stored rows comes from the files themselves."""
    ks, vs, n_rows = [], [], None
    for b in range(engine.bsz):
        for h in range(engine.kv_head_num):
            with open(_file(path, b, h), "rb") as f:
                if f.read(8) != MAGIC:
                    raise ValueError(f"{_file(path, b, h)}: not a diffcache_b200 snapshot")
                dim, dtype, n = struct.unpack("<IIQ", f.read(16))
                if dim != engine.head_dim or dtype != engine.dtype:
                    raise ValueError("snapshot head_dim / element type do not match the engine")
                if n_rows is None:
                    n_rows = n
                if n != n_rows:
                    raise ValueError("snapshots of one layer disagree on the number of rows")
                ks.append(np.frombuffer(f.read(n * dim * 2), np.uint16).reshape(n, dim))
                vs.append(np.frombuffer(f.read(n * dim * 2), np.uint16).reshape(n, dim))
    if n_rows > ctx_len:
        raise ValueError("snapshot holds more rows than ctx_len")
    shape = (engine.bsz, engine.kv_head_num, n_rows, engine.head_dim)
    k = np.ascontiguousarray(np.stack(ks).reshape(shape))
    v = np.ascontiguousarray(np.stack(vs).reshape(shape))
    engine.prefill(k, v, None)
