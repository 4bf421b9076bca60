"""CPU suite, part 3: the tensor-parallel split, world size 2 and 4 over gloo.

No GPU: each rank takes its block of every weight with the loader's own rule (tl_tp_shard,
host-only), runs the block arithmetic of the Llama2 layer in numpy (float64, so that only the
algebra is under test) and exchanges partial results through torch.distributed/gloo exactly where
the GPU path calls NCCL: a sum after wo and after w2, a gather of the classifier slices. Rank 0
compares with the unsharded computation.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _silu(x):
    return x / (1.0 + np.exp(-x))


def _worker(rank: int, world: int, port: int, q):
    try:
        sys.path.insert(0, ROOT)
        import torch
        import torch.distributed as dist

        from tensorlib_b200 import synth, tp
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        dim, hid, heads, vocab, T = 64, 96, 8, 40, 3
        hd = dim // heads
        full = {n: synth.normal_f16(9, i + 1, r * c, 0.1).reshape(r, c).astype(np.float64)
                for i, (n, r, c) in enumerate([("wq", dim, dim), ("wk", dim, dim), ("wv", dim, dim), ("wo", dim, dim),
                                               ("w1", hid, dim), ("w3", hid, dim), ("w2", dim, hid),
                                               ("output", vocab, dim)])}
        x = synth.normal_f16(9, 50, T * dim, 1.0).reshape(T, dim).astype(np.float64)
        mine = {n: tp.shard_of(n, w, rank, world) for n, w in full.items()}

        # every element of every tensor is held by exactly one rank (or by all, if replicated)
        for n, w in full.items():
            cover = torch.zeros(w.shape, dtype=torch.float64)
            r0, nr, c0, nc = tp.shard(tp.SHARD_KIND[n], w.shape[0], w.shape[1], rank, world)
            cover[r0:r0 + nr, c0:c0 + nc] += 1
            dist.all_reduce(cover)
            assert bool((cover == 1).all()), f"{n}: shards overlap or leave holes"

        def allreduce(a):
            t = torch.from_numpy(np.ascontiguousarray(a))
            dist.all_reduce(t)
            return t.numpy()

        def attention(q, k, v, n_heads):   # (T, n_heads*hd) each, causal
            out = np.zeros_like(q)
            for h in range(n_heads):
                sl = slice(h * hd, (h + 1) * hd)
                s = q[:, sl] @ k[:, sl].T / np.sqrt(hd)
                s = np.where(np.tril(np.ones_like(s)) > 0, s, -np.inf)
                p = np.exp(s - s.max(axis=1, keepdims=True))
                out[:, sl] = (p / p.sum(axis=1, keepdims=True)) @ v[:, sl]
            return out

        # sharded layer: heads and hidden units are local, sums after wo and w2
        hl = heads // world
        att = attention(x @ mine["wq"].T, x @ mine["wk"].T, x @ mine["wv"].T, hl)
        h = x + allreduce(att @ mine["wo"].T)
        ff = (_silu(h @ mine["w1"].T) * (h @ mine["w3"].T)) @ mine["w2"].T
        out = h + allreduce(ff)
        logits_local = torch.from_numpy(np.ascontiguousarray(out @ mine["output"].T))
        gathered = [torch.empty_like(logits_local) for _ in range(world)]
        dist.all_gather(gathered, logits_local)
        logits = np.concatenate([g.numpy() for g in gathered], axis=1)

        if rank == 0:
            att_f = attention(x @ full["wq"].T, x @ full["wk"].T, x @ full["wv"].T, heads)
            h_f = x + att_f @ full["wo"].T
            out_f = h_f + (_silu(h_f @ full["w1"].T) * (h_f @ full["w3"].T)) @ full["w2"].T
            want = out_f @ full["output"].T
            err = float(np.abs(logits - want).max())
            assert err < 1e-9, err
            assert np.array_equal(logits.argmax(1), want.argmax(1))
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported to the parent
        import traceback
        q.put((rank, traceback.format_exc() + str(e)))


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_split_reproduces_the_unsharded_layer(world):
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_shard_rule_rejects_indivisible_shapes():
    sys.path.insert(0, ROOT)
    import tensorlib_b200 as tl
    from tensorlib_b200 import tp
    assert tp.shard(tp.SHARD_ROWS, 4096, 4096, 3, 8) == (1536, 512, 0, 4096)
    assert tp.shard(tp.SHARD_COLS, 4096, 11008, 7, 8) == (0, 4096, 9632, 1376)
    assert tp.shard(tp.SHARD_REPLICATED, 1, 4096, 1, 2) == (0, 1, 0, 4096)
    with pytest.raises(tl.TLError):
        tp.shard(tp.SHARD_ROWS, 30, 8, 0, 4)
