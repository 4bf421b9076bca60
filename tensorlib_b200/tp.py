"""Tensor-parallel group set-up: one process per GPU, NCCL communicator created inside the native
library; ``torch.distributed`` (any backend, gloo is enough) is only the rendezvous that carries
the NCCL unique id from rank 0 to the others."""
from __future__ import annotations

import ctypes as C

import numpy as np

import tensorlib_b200 as tl

SHARD_REPLICATED, SHARD_ROWS, SHARD_COLS = 0, 1, 2
# how each checkpoint tensor of the Llama2 block is split (Megatron scheme: wq/wk/wv/w1/w3 by output rows,
# wo/w2 by input columns, classifier by vocabulary rows, embedding and norms replicated)
SHARD_KIND = {"tok_embeddings": SHARD_REPLICATED, "attention_norm": SHARD_REPLICATED, "ffn_norm": SHARD_REPLICATED,
              "norm": SHARD_REPLICATED, "wq": SHARD_ROWS, "wk": SHARD_ROWS, "wv": SHARD_ROWS, "w1": SHARD_ROWS,
              "w3": SHARD_ROWS, "output": SHARD_ROWS, "wo": SHARD_COLS, "w2": SHARD_COLS}


def shard(kind: int, rows: int, cols: int, rank: int, world: int):
    """(row0, nrows, col0, ncols) of the block rank `rank` keeps — the loader's own rule
    (tl_tp_shard, host-only)."""
    out = [C.c_int() for _ in range(4)]
    tl.check(tl.load().tl_tp_shard(kind, rows, cols, rank, world, *[C.byref(o) for o in out]), "tl_tp_shard")
    return tuple(o.value for o in out)


def shard_of(name: str, full: np.ndarray, rank: int, world: int) -> np.ndarray:
    r0, nr, c0, nc = shard(SHARD_KIND[name], full.shape[0], full.shape[1], rank, world)
    return np.ascontiguousarray(full[r0:r0 + nr, c0:c0 + nc])


def attach(model: "tl.Llama2", rank: int, world: int, dist) -> None:
    """Create the NCCL communicator (once per process) and hook it into `model`."""
    lib = tl.load()
    buf = (C.c_ubyte * 128)()
    if rank == 0:
        tl.check(lib.tl_tp_unique_id(buf, 128), "tl_tp_unique_id")
    payload = [bytes(buf)]
    dist.broadcast_object_list(payload, src=0)
    raw = (C.c_ubyte * 128).from_buffer_copy(payload[0])
    tl.check(lib.tl_tp_init(raw, 128, rank, world), "tl_tp_init")
    tl.check(lib.tl_tp_attach(model.h), "tl_tp_attach")


def open_fused_exchange(model: "tl.Llama2", rank: int, world: int, dist) -> None:
    """Switch the decode step from NCCL allreduces to the exchange fused into the GEMV kernels:
    every rank exports its receive region, the 64-byte IPC handles are gathered over `dist`,
    every rank maps all regions. Collective on the host side (all ranks must call it)."""
    lib = tl.load()
    buf = (C.c_ubyte * 64)()
    tl.check(lib.tl_tp_exchange_export(model.h, buf, 64), "tl_tp_exchange_export")
    gathered = [None] * world
    dist.all_gather_object(gathered, bytes(buf))
    allh = (C.c_ubyte * (64 * world)).from_buffer_copy(b"".join(gathered))
    tl.check(lib.tl_tp_exchange_open(model.h, allh, world), "tl_tp_exchange_open")
    dist.barrier()


def close_fused_exchange(model: "tl.Llama2", dist) -> None:
    tl.synchronize()
    dist.barrier()           # nobody unmaps while a peer may still push
    tl.load().tl_tp_exchange_close(model.h)
    dist.barrier()


def destroy() -> None:
    tl.load().tl_tp_destroy()
