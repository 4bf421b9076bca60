"""GPU parity of the tensor-parallel forward (needs >= 2 GPUs; cases that need more GPUs than the
box has are skipped).

One process per GPU, NCCL inside the library (gloo only carries the unique id and the IPC handles).
Each rank loads its shard; prefill and decode logits must match the single-GPU fast path within the
model tolerance, every rank must sample the same ids, and the exchange fused into the GEMV kernels
(peer stores, three launches per layer; the sum formed by every CTA or, `TL_TP_REDUCE=slice`, once per GPU as
eight ranks do by default) must agree with the NCCL form.
Configurations: the tiny model (world 2), a head_dim-128 model (world 2 and 4) and ONE layer of the
7B shape (dim 4096, hidden 11008, 32 heads; world 2 and 4), where a consumer gathers 4096 words.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
pytestmark = pytest.mark.gpu

N_PROMPT, N_FORCED, N_FREE = 16, 6, 12
N_LONG = 512      # a prompt long enough for the tcgen05 prefill path and divisible by 128 x world


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _config(name):
    sys.path.insert(0, ROOT)
    from tensorlib_b200 import synth
    if name == "tiny":
        cfg = synth.TINY
        return cfg, synth.llama2c_payload(cfg, 20240229)
    if name == "mid":
        cfg = synth.LlamaConfig(dim=512, hidden_dim=1408, n_layers=2, n_heads=4, vocab_size=1000, seq_len=640)
        return cfg, synth.llama2c_payload(cfg, 777)
    cfg = synth.LlamaConfig(dim=4096, hidden_dim=11008, n_layers=1, n_heads=32, vocab_size=2000, seq_len=640)
    payload = (np.random.default_rng(4096).standard_normal(cfg.payload_elems(), dtype=np.float32) * 0.02).astype(np.float16)
    V, d, L = cfg.vocab_size, cfg.dim, cfg.n_layers
    payload[V * d:V * d + L * d] = 1.0
    off = V * d + L * d + 4 * L * d * d
    payload[off:off + L * d] = 1.0
    payload[-d:] = 1.0
    return cfg, payload


def _tokens(cfg):
    from tensorlib_b200 import synth
    return synth.token_ids(20240229, 100, N_PROMPT, cfg.vocab_size), synth.token_ids(20240229, 101, N_FORCED, cfg.vocab_size)


def _long_prompt(cfg):
    from tensorlib_b200 import synth
    return synth.token_ids(20240229, 102, N_LONG, cfg.vocab_size) if cfg.seq_len > N_LONG and cfg.head_dim == 128 else None


def _worker(rank: int, world: int, port: int, name: str, q, reduce_form: str = ""):
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        if reduce_form:      # the form of the decode exchange's sum that eight ranks take by default
            os.environ["TL_TP_REDUCE"] = reduce_form
        import torch.distributed as dist

        import tensorlib_b200 as tl
        from tensorlib_b200 import tp
        dist.init_process_group("gloo", rank=rank, world_size=world)
        tl.init(rank)
        cfg, payload = _config(name)
        prompt, forced = _tokens(cfg)
        m = tl.Llama2(cfg, numerics=tl.FAST, tp_rank=rank, tp_world=world)
        tp.attach(m, rank, world, dist)
        m.load_payload(payload, shared_classifier=True)
        lg_prefill = m.forward(prompt, 0, all_logits=True)
        long_prompt = _long_prompt(cfg)
        lg_decode = np.concatenate([m.forward(forced[i:i + 1], N_PROMPT + i, all_logits=True) for i in range(N_FORCED)])
        m.forward(prompt, 0, all_logits=False)
        ids = m.decode_device(N_PROMPT, N_FREE)             # CUDA-graph decode with NCCL inside the graph
        status = tl.device_status()
        lg_long_nccl = m.forward(long_prompt, 0, all_logits=True)[-4:] if long_prompt is not None else None
        dist.barrier()
        # the same decode with the exchange fused into the GEMV kernels (peer stores, no NCCL)
        tp.open_fused_exchange(m, rank, world, dist)
        # long prompts: the K-split matmuls push their partial rows to the owning ranks, no NCCL in the layer loop
        lg_long_fused = None
        if long_prompt is not None:
            dist.barrier()
            lg_long_fused = m.forward(long_prompt, 0, all_logits=True)[-4:]
            status |= tl.device_status()
            dist.barrier()
            again = m.forward(long_prompt, 0, all_logits=True)[-4:]       # a second exchange round over the same buffers
            assert np.array_equal(again.view(np.uint16), lg_long_fused.view(np.uint16))
        m.forward(prompt, 0, all_logits=False)               # a 16-token prompt still reduces over NCCL
        lg_fused = np.concatenate([m.forward(forced[i:i + 1], N_PROMPT + i, all_logits=True) for i in range(N_FORCED)])
        m.forward(prompt, 0, all_logits=False)
        dist.barrier()
        ids_fused = m.decode_device(N_PROMPT, N_FREE)
        status |= tl.device_status()
        stamps = m.decode_profile(N_PROMPT + N_FREE)         # the timestamped step runs the same kernels
        status |= tl.device_status()
        tp.close_fused_exchange(m, dist)
        m.close()
        tp.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok", lg_prefill, lg_decode, ids, status, lg_fused, ids_fused, stamps.shape, lg_long_nccl, lg_long_fused))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc() + str(e), None, None, None, None, None, None, None, None, None))


def _rel_err(got, want):
    g, w = got.astype(np.float64), want.astype(np.float64)
    scale = np.sqrt((w * w).mean(axis=-1, keepdims=True)) + 1e-30
    return float((np.abs(g - w) / np.maximum(np.abs(w), scale)).max())


@pytest.mark.parametrize("name,world,reduce_form", [("tiny", 2, ""), ("mid", 2, ""), ("mid", 4, ""), ("layer7b", 2, ""),
                                                    ("layer7b", 4, ""), ("mid", 2, "slice"), ("layer7b", 2, "slice"),
                                                    ("layer7b", 4, "slice")])
def test_tensor_parallel_matches_single_gpu(tl, name, world, reduce_form):
    if tl.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cfg, payload = _config(name)
    prompt, forced = _tokens(cfg)
    single = tl.Llama2(cfg, numerics=tl.FAST)
    single.load_payload(payload, shared_classifier=True)
    want_prefill = single.forward(prompt, 0, all_logits=True)
    want_decode = np.concatenate([single.forward(forced[i:i + 1], N_PROMPT + i, all_logits=True) for i in range(N_FORCED)])
    long_prompt = _long_prompt(cfg)
    want_long = single.forward(long_prompt, 0, all_logits=True)[-4:] if long_prompt is not None else None
    single.close()

    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, name, q, reduce_form)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted((q.get(timeout=900) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
    for rank, msg, *_ in results:
        assert msg == "ok", f"rank {rank}: {msg}"
    tol = 2e-2          # relative to max(|logit|, row rms): the K-split changes the fp32 summation grouping only
    for rank, _, lp, ld, ids, status, lf, ids_f, stamp_shape, ll_nccl, ll_fused in results:
        assert status == 0
        if want_long is not None:
            assert _rel_err(ll_nccl, want_long) <= tol, (name, world, "512-token prefill, NCCL allreduce")
            assert _rel_err(ll_fused, want_long) <= tol, (name, world, "512-token prefill, fused exchange")
        assert _rel_err(lp, want_prefill) <= tol, (name, world, "prefill")
        assert _rel_err(ld, want_decode) <= tol, (name, world, "decode, NCCL exchange")
        assert _rel_err(lf, want_decode) <= tol, (name, world, "decode, fused exchange")
        assert stamp_shape == (4 * cfg.n_layers + 1, 3)
    first = results[0]
    for other in results[1:]:
        assert np.array_equal(first[4], other[4]), "ranks sampled different ids"
        assert np.array_equal(first[2].view(np.uint16), other[2].view(np.uint16)), "ranks disagree on logits"
        # fused exchange: every rank adds the same partials in the same (rank) order -> identical bits
        assert np.array_equal(first[6].view(np.uint16), other[6].view(np.uint16)), "ranks disagree (fused)"
        assert np.array_equal(first[7], other[7]), "ranks sampled different ids (fused)"
        if want_long is not None:
            assert np.array_equal(first[10].view(np.uint16), other[10].view(np.uint16)), "ranks disagree on the fused prefill"
    print(f"{name} x{world}: fused ids {first[7].tolist()}, NCCL ids {first[4].tolist()}")
