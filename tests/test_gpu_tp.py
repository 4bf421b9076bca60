"""GPU parity of the tensor-parallel forward (needs >= 2 GPUs; skipped on a single-GPU box).

Two ranks, one process per GPU, NCCL inside the library (gloo only carries the unique id). Each
rank loads its shard of the tiny model; prefill + decode logits must match the single-GPU fast
path within the matmul tolerance, and every rank must sample the same ids.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        import torch.distributed as dist

        import tensorlib_b200 as tl
        from tensorlib_b200 import synth, tp
        dist.init_process_group("gloo", rank=rank, world_size=world)
        tl.init(rank)
        payload = synth.llama2c_payload(synth.TINY, 20240229)
        prompt = synth.prompt_tokens(synth.TINY, 20240229, 16)
        m = tl.Llama2(synth.TINY, numerics=tl.FAST, tp_rank=rank, tp_world=world)
        tp.attach(m, rank, world, dist)
        m.load_payload(payload, shared_classifier=True)
        lg_prefill = m.forward(prompt, 0, all_logits=True)
        forced = synth.token_ids(20240229, 101, 6, synth.TINY.vocab_size)
        lg_decode = np.concatenate([m.forward(forced[i:i + 1], 16 + i, all_logits=True) for i in range(6)])
        m.forward(prompt, 0, all_logits=False)
        ids = m.decode_device(16, 12)                       # CUDA-graph decode with NCCL inside the graph
        status = tl.device_status()
        dist.barrier()
        # the same decode with the exchange fused into the GEMV kernels (peer stores, no NCCL)
        tp.open_fused_exchange(m, rank, world, dist)
        m.forward(prompt, 0, all_logits=False)               # prefill still reduces over NCCL
        lg_fused = np.concatenate([m.forward(forced[i:i + 1], 16 + i, all_logits=True) for i in range(6)])
        m.forward(prompt, 0, all_logits=False)
        ids_fused = m.decode_device(16, 12)
        status |= tl.device_status()
        tp.close_fused_exchange(m, dist)
        m.close()
        tp.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok", lg_prefill, lg_decode, ids, status, lg_fused, ids_fused))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc() + str(e), None, None, None, None, None, None))


def test_two_rank_tensor_parallel_matches_single_gpu(tl, tiny_payload):
    if tl.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from tensorlib_b200 import synth
    single = tl.Llama2(synth.TINY, numerics=tl.FAST)
    single.load_payload(tiny_payload, shared_classifier=True)
    prompt = synth.prompt_tokens(synth.TINY, 20240229, 16)
    forced = synth.token_ids(20240229, 101, 6, synth.TINY.vocab_size)
    want_prefill = single.forward(prompt, 0, all_logits=True).astype(np.float32)
    want_decode = np.concatenate([single.forward(forced[i:i + 1], 16 + i, all_logits=True) for i in range(6)]).astype(np.float32)
    single.close()

    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted((q.get(timeout=600) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
    for rank, msg, *_ in results:
        assert msg == "ok", f"rank {rank}: {msg}"
    for rank, _, lp, ld, ids, status, lf, ids_f in results:
        assert status == 0
        assert np.abs(lp.astype(np.float32) - want_prefill).max() <= 2e-2
        assert np.abs(ld.astype(np.float32) - want_decode).max() <= 2e-2
        assert np.abs(lf.astype(np.float32) - want_decode).max() <= 2e-2, "fused exchange"
    assert np.array_equal(results[0][4], results[1][4]), "ranks sampled different ids"
    assert np.array_equal(results[0][2].view(np.uint16), results[1][2].view(np.uint16)), "ranks disagree on logits"
    # fused exchange: every rank sums the same partials in the same (rank) order -> identical bits
    assert np.array_equal(results[0][6].view(np.uint16), results[1][6].view(np.uint16)), "ranks disagree (fused)"
    assert np.array_equal(results[0][7], results[1][7]), "ranks sampled different ids (fused)"
