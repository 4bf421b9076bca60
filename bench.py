#!/usr/bin/env python
"""Headline benchmark: greedy decode tokens/s of a Llama2-7B-shaped fp16 model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decoded token (one pass over all weights). N = 1 runs the 7B shape on one B200
(128-token seeded prompt, then decode); N > 1 (under torchrun, one rank per GPU) runs the same
model tensor-parallel with a 512-token context. Weights are random N(0, 0.02) generated on the
device, norms = 1, token ids seeded: synthetic data of the benchmark's shape.

The JSON line:
  value      tokens/s with everything resident on the device: one CUDA-graph replay per token,
             the sampled id fed back in device memory; K steps timed with CUDA events on the
             launching stream, barrier + synchronize on both sides, max over ranks; repeated
             REPEATS times over the same positions, `value` is the median (spread in `repeats`).
  e2e        the same metric through the reference-facing call tl_llama2_generate: every step
             moves the token id host->device and the sampled id device->host, like
             Llama2::generate does; wall clock like the reference measures it.
  roofline   the dominant kernel (RMSNorm + w1|w3 GEMV + SiLU*up, 43 % of the weight bytes of a
             token), launched over all layers' weights (5.8 GB >> L2) and timed with CUDA events;
             its output for layer 0 is checked against an fp32 recomputation first.
             roofline.prefill_2048 is the compute-bound companion (one 2048-token prompt).
  checks     device status word after every timed region (a timed-out wait fails the run); for
             N > 1 the ids every rank sampled, compared across ranks and with the NCCL exchange.
  cpu_baseline / --impl reference
             the reference's own OpenMP CPU code (oracle/_ref) on all host cores: whole tokens of
             the full 32-layer model where host memory allows (about 30 GB), otherwise one decode
             step of a ONE-layer model with 1/32 of the classifier rows, 32 of which make a token
             (`extrapolation` says which).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from tensorlib_b200 import synth  # noqa: E402

SEED = 20240229
CFG = synth.LLAMA2_7B
METRIC = "decode tokens/s Llama2-7B fp16"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# -------------------------------------------------------------------------------------------------
# CPU arm: the reference's own code on the host cores
# -------------------------------------------------------------------------------------------------
def _cpu_lib():
    from oracle import ref_lib
    if ref_lib.have_ref():
        lib, kind = ref_lib.RefLib(), "reference"
    else:
        lib, kind = ref_lib.OracleLib(), "port"
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers: ask for the host's cores explicitly
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib.set_threads(max(1, cores))
    return lib, kind, lib.max_threads()


def _tiled_payload(cfg) -> np.ndarray:
    """Checkpoint payload for timing runs: values do not change the time of a dense pass, so one
    seeded block is tiled over it (norm weights = 1)."""
    block = synth.normal_f16(SEED, 1, 1 << 22, 0.02)
    payload = np.resize(block, cfg.payload_elems())
    d, L, V = cfg.dim, cfg.n_layers, cfg.vocab_size
    payload[V * d: V * d + L * d] = 1.0                                   # attention_norm
    off = V * d + L * d + 4 * L * d * d
    payload[off: off + L * d] = 1.0                                       # ffn_norm
    off += L * d + 3 * L * d * cfg.hidden_dim
    payload[off: off + d] = 1.0                                           # final norm
    return payload


def _host_memory_available() -> int:
    try:
        import psutil
        return int(psutil.virtual_memory().available)
    except Exception:
        return 0


def cpu_reference_decode(steps: int, warmup: int, budget_s: float, context: int):
    """Greedy decode steps on the reference's CPU backend, all host cores. Whole tokens of the full
    32-layer model when the host has the memory for it (payload + the reference's own copy of the
    weights, about 30 GB), else decode steps of a one-layer model with vocab/32 classifier rows,
    32 of which make a token. Returns a dict for the JSON line."""
    lib, kind, cores = _cpu_lib()
    full_bytes = 2 * CFG.payload_elems() * 2 + (4 << 30)
    full = os.environ.get("TL_BENCH_CPU_FULL", "auto")
    use_full = full == "1" or (full == "auto" and _host_memory_available() > full_bytes + (8 << 30))
    if use_full:
        cfg, factor = CFG, 1
    else:
        cfg = synth.LlamaConfig(dim=CFG.dim, hidden_dim=CFG.hidden_dim, n_layers=1, n_heads=CFG.n_heads,
                                vocab_size=CFG.vocab_size // CFG.n_layers, seq_len=CFG.seq_len, shared_classifier=True)
        factor = CFG.n_layers
    payload = _tiled_payload(cfg)
    model = lib.llama2(cfg, payload)
    del payload
    tok = np.array([1], dtype=np.int32)
    # the KV cache below `context` is zero: attention over it costs what it costs over real keys
    pos = min(context, cfg.seq_len - steps - warmup - 1)
    for _ in range(warmup):
        model.forward(tok, pos, 1); pos += 1
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        model.forward(tok, pos, 1); pos += 1; done += 1
        if time.perf_counter() - t0 > budget_s and done >= 3:
            break
    dt = (time.perf_counter() - t0) / done
    model.close()
    if use_full:
        sample = f"{done} whole tokens of the full 32-layer model at context {context}+ (no extrapolation)"
    else:
        sample = (f"{done} decode steps of a 1-layer 7B-shaped model with vocab/32 classifier rows at context "
                  f"{context}+; a token is {factor} such steps (extrapolated x{factor})")
    return {"tokens_per_s": 1.0 / (dt * factor), "ms_per_sample": dt * 1e3, "extrapolation": factor, "cores": cores,
            "kind": kind, "samples": done, "sample": sample}


def cpu_reference_matmul_and_prefill(budget_s: float = 25.0) -> dict:
    """The other two CPU baselines of the benchmark plan: the reference's OpenMP matmul2d
    (tensorLib/src/device/cpu/CPU.cpp:76-89) on the four sweep weight shapes, and the prefill of one
    7B-shaped layer. Every output row of a matmul is an independent dot-product loop, so the time is
    linear in M: M = 8 rows are timed and the rate is reported (a 2048-row point is that rate times 256).
    The prefill is timed at T = 64 on a one-layer model and scaled to 32 layers x 2048 tokens by the
    linear-layer flops (the attention part, quadratic in T, is 7 % of the flops at T = 2048)."""
    lib, kind, cores = _cpu_lib()
    out = {"cores": cores, "kind": kind, "matmul": []}
    t_start = time.perf_counter()
    for (K, N) in ((4096, 4096), (4096, 11008), (11008, 4096), (4096, 32000)):
        W = np.resize(synth.normal_f16(SEED, 2, 1 << 20, 0.02), N * K).reshape(N, K)
        x = synth.normal_f16(SEED, 3, 8 * K, 1.0).reshape(8, K)
        lib.matmul2d(x[:1], W[:64])
        t0 = time.perf_counter()
        lib.matmul2d(x, W)
        dt = time.perf_counter() - t0
        out["matmul"].append({"K": K, "N": N, "M_timed": 8, "ms": dt * 1e3, "gflops": 2.0 * 8 * N * K / dt / 1e9})
        if time.perf_counter() - t_start > budget_s:
            break
    T = 64
    cfg = synth.LlamaConfig(dim=CFG.dim, hidden_dim=CFG.hidden_dim, n_layers=1, n_heads=CFG.n_heads,
                            vocab_size=1000, seq_len=128, shared_classifier=True)
    model = lib.llama2(cfg, _tiled_payload(cfg))
    tokens = synth.token_ids(SEED, 9, T, cfg.vocab_size)
    t0 = time.perf_counter()
    model.forward(tokens, 0, 1)
    dt = time.perf_counter() - t0
    model.close()
    per_layer = 4 * CFG.dim * CFG.dim + 3 * CFG.dim * CFG.hidden_dim
    timed_flops = 2.0 * T * (per_layer + cfg.vocab_size * CFG.dim)
    full_flops = 2.0 * 2048 * (CFG.n_layers * per_layer) + 2.0 * 2048 * CFG.vocab_size * CFG.dim   # the reference computes all-position logits
    out["prefill_layer_T64_s"] = dt
    out["prefill_2048_extrapolated_s"] = dt * full_flops / timed_flops
    out["prefill_note"] = ("one 7B-shaped layer, 64 tokens, timed; scaled to 32 layers x 2048 tokens + all-position "
                           "classifier by linear-layer flops (labelled extrapolation)")
    return out


def bench_config(n_gpus: int) -> dict:
    """The workload description both arms print, key for key."""
    return {"workload": workload_name(n_gpus), "parallelism": f"tp{n_gpus}",
            "l2": "inputs larger than L2 (weights streamed per token >> 126 MB)"}


def run_reference_arm(args, rank: int):
    if rank != 0:
        return
    context = 128 if args.gpus == 1 else 512
    r = cpu_reference_decode(args.steps, max(args.warmup, 1), budget_s=120.0, context=context)
    line = {"impl": "reference", "metric": METRIC, "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": r["samples"], "warmup": max(args.warmup, 1), "ms_per_step": r["ms_per_sample"],
            "extrapolation": r["extrapolation"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": bench_config(args.gpus),
            "timing": "host wall clock around Transformer::forward, OpenMP on all host cores; ms_per_step is the "
                      "measured time of one sample, value = 1 / (extrapolation x that)",
            "cpu_baseline": {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"],
                             "sample": r["sample"]},
            "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_name(n_gpus: int) -> str:
    if n_gpus == 1:
        return ("Llama2-7B shape (dim 4096, hidden 11008, 32 layers, 32 heads, vocab 32000), batch 1, "
                "128-token prompt then greedy decode")
    return (f"Llama2-7B shape tensor-parallel over {n_gpus} GPUs (wq/wk/wv/w1/w3 row-split, wo/w2 column-split, "
            "allreduce after each K-split matmul), batch 1, 512-token context then greedy decode")


# -------------------------------------------------------------------------------------------------
# GPU arm
# -------------------------------------------------------------------------------------------------
REPEATS = 5   # the K timed steps are repeated this often over the same positions; value = median


class _DeviceArray:
    """A raw device pointer dressed as a CUDA array so that torch can view it without a copy."""

    def __init__(self, ptr: int, shape, typestr: str = "<f2"):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}


def require_clean_status(tl, where: str) -> None:
    """A kernel that gave up on a bounded wait leaves a status word behind: such a run measured
    wrong arithmetic, so it fails loudly instead of printing a number."""
    st = tl.device_status()
    if st != 0:
        raise SystemExit(f"bench.py: device status {st} after {where}: a bounded device-side wait ran out")


def roofline_gateup(tl, model, stream, torch, n_layers):
    """Time the dominant kernel over all layers' w1|w3 (distinct weights every launch), after
    checking what it computes for layer 0 against an fp32 recomputation."""
    lib = tl.load()
    dim, hid, L = CFG.dim, model.c.hidden_dim // model.c.tp_world, n_layers
    stream_ptr = stream.cuda_stream

    def tensor(name, layer):
        p, r, c = C.c_void_p(), C.c_int(), C.c_int()
        tl.check(lib.tl_llama2_tensor(model.h, name.encode(), layer, C.byref(p), C.byref(r), C.byref(c)), name)
        return p.value

    x = torch.randn(dim, device="cuda").half()
    out = torch.empty(hid, device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    ptrs = [(tensor("ffn_norm", l), tensor("w1", l), tensor("w3", l)) for l in range(L)]

    def sweep():
        for nw, w1, w3 in ptrs:
            tl.check(lib.tl_rmsnorm_gateup_swiglu_f16(x.data_ptr(), nw, 1e-5, w1, w3, out.data_ptr(), hid, dim,
                                                      stream_ptr), "gateup")
    # what the timed launch computes, layer 0: silu(w1 n) * (w3 n), n = x / rms(x) * norm weight
    nw0, w1p, w3p = ptrs[0]
    tl.check(lib.tl_rmsnorm_gateup_swiglu_f16(x.data_ptr(), nw0, 1e-5, w1p, w3p, out.data_ptr(), hid, dim, stream_ptr), "gateup")
    torch.cuda.synchronize()
    xf = x.float()
    n32 = xf * torch.rsqrt((xf * xf).mean() + 1e-5) * torch.as_tensor(_DeviceArray(nw0, (dim,)), device="cuda").float()
    g32 = torch.as_tensor(_DeviceArray(w1p, (hid, dim)), device="cuda").float() @ n32
    u32 = torch.as_tensor(_DeviceArray(w3p, (hid, dim)), device="cuda").float() @ n32
    want = torch.nn.functional.silu(g32) * u32
    err = float(((out.float() - want).abs() / want.abs().clamp_min(float(want.pow(2).mean().sqrt()))).max())
    if not err <= 2e-2:
        raise SystemExit(f"bench.py: the timed gate/up kernel is off by {err} (relative) against an fp32 recomputation")
    del g32, u32, want
    for _ in range(3):
        sweep()
    reps = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)          # events on the stream the kernels are launched on
    for _ in range(reps):
        sweep()
    e1.record(stream)
    torch.cuda.synchronize()
    require_clean_status(tl, "the roofline launches")
    sec = e0.elapsed_time(e1) * 1e-3 / (reps * L)
    bytes_per_launch = 2 * hid * dim * 2 + 2 * dim * 2 + hid * 2   # w1+w3, x + norm weight, out
    peak, peak_src = measured_peaks()
    achieved = bytes_per_launch / sec / 1e9
    traffic = NCU_TRAFFIC_GATEUP // model.c.tp_world   # weight rows per launch scale as 1 / ranks
    return {"bound": "hbm", "kernel": "k_gemv_ring<SWIGLU,NORM> (RMSNorm + w1|w3 GEMV + SiLU*up)",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
            "bytes_per_launch": bytes_per_launch, "us_per_launch": sec * 1e6, "traffic": traffic,
            "output_check_max_rel_err": err,
            "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one full-size launch "
                              "(profiles/gemv_ring_decode_llama2_7b.md)" + ("" if model.c.tp_world == 1 else
                                                                            f", divided by {model.c.tp_world} ranks")}


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the gate/up kernel (2 x 11008 x 4096
# fp16 weights) from the ncu capture summarised in profiles/gemv_ring_decode_llama2_7b.md:
# 180,431,872 B read + 3,465,984 B written
NCU_TRAFFIC_GATEUP = 183_897_856


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    import tensorlib_b200 as tl

    torch.cuda.set_device(local_rank)
    tl.init(local_rank)
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)  # rendezvous only; the data path is the library's own NCCL communicator
    cfg = CFG if args.layers == CFG.n_layers else synth.LlamaConfig(
        dim=CFG.dim, hidden_dim=CFG.hidden_dim, n_layers=args.layers, n_heads=CFG.n_heads,
        vocab_size=CFG.vocab_size, seq_len=CFG.seq_len, shared_classifier=False)
    one_kernel = args.decode_path == "kernel" and (world == 1 or args.tp_exchange == "fused")
    model = tl.Llama2(cfg, numerics=tl.FAST, tp_rank=rank, tp_world=world, one_kernel_decode=one_kernel)
    fused = world > 1 and args.tp_exchange == "fused"
    if world > 1:
        from tensorlib_b200 import tp
        tp.attach(model, rank, world, dist)
        if fused:
            tp.open_fused_exchange(model, rank, world, dist)
    model.init_random(SEED, 0.02)

    n_ctx = 128 if world == 1 else 512
    K, W = args.steps, args.warmup
    assert n_ctx + W + K + 2 <= CFG.seq_len, "steps + warmup exceed the 2048-token context"
    prompt = synth.prompt_tokens(CFG, SEED, n_ctx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def gather_ids(ids):
        """Every rank's copy of a sampled id sequence: (all ranks agree, rank 0's list)."""
        if world == 1:
            return True, [int(v) for v in ids]
        got = [None] * world
        dist.all_gather_object(got, [int(v) for v in ids])
        return all(g == got[0] for g in got), got[0]

    # prefill (untimed): leaves the first sampled id in the device slot
    checks = {}
    if args.skip_prefill:
        model.set_next_token(int(prompt[-1]))      # profiling runs: decode over a zero KV cache
        first_token = int(prompt[-1])
    else:
        first_token = int(model.forward(prompt, 0, all_logits=False)[0].astype(np.float32).argmax())
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    pos0 = n_ctx
    with torch.cuda.stream(stream):
        # correctness before speed: eight steps from the prompt, ids fetched and compared across the ranks
        barrier()
        ids8 = model.decode_device(pos0, min(8, K), fetch=True, stream=sp)
        require_clean_status(tl, "the first decode steps")
        agree, ids8_list = gather_ids(ids8)
        checks.update({"tp_ids_agree": agree, "first_ids": ids8_list, "exchange": args.tp_exchange if world > 1 else "none"})
        if not agree:
            raise SystemExit("bench.py: the ranks sampled different token ids")
        model.decode_device(pos0, W, fetch=False, stream=sp)          # warm-up over the positions that are timed
        barrier()
        launches0 = model.kernel_launches()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        times = []
        for _ in range(REPEATS):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record(stream)
            model.decode_device(pos0, K, fetch=False, stream=sp)     # the same K positions every repeat
            e1.record(stream)
            barrier()
            times.append(max_over_ranks(e0.elapsed_time(e1)))
        clocks = sampler.stop() if rank == 0 else None
        launches = (model.kernel_launches() - launches0) // REPEATS
        require_clean_status(tl, "the timed decode steps")
        barrier()      # rank 0 just spent host time stopping the clock sampler: the ranks must launch together
        ids_timed = model.decode_device(pos0 + K, 1, fetch=True, stream=sp)   # the id that followed the last timed step
        agree_timed, _ = gather_ids(ids_timed)
        checks["tp_ids_agree_after_timed_region"] = agree_timed
    ms = float(np.median(times))
    value = K / (ms * 1e-3)
    repeats = {"n": REPEATS, "ms_per_step_median": ms / K, "ms_per_step_min": min(times) / K,
               "ms_per_step_max": max(times) / K, "tokens_per_s_min": K / (max(times) * 1e-3),
               "tokens_per_s_max": K / (min(times) * 1e-3)}

    if args.profile_step:
        barrier()
        stamps = np.stack([model.decode_profile(pos0 + K, 0).astype(np.float64) for _ in range(3)])[-1]
        if rank == 0:
            L = cfg.n_layers
            if one_kernel:
                per, names = stamps[:5 * L].reshape(L, 5, 3), ["qkv", "attention", "wo", "gate/up", "w2"]
            elif world > 1 and fused:
                per, names = stamps[1:1 + 4 * L].reshape(L, 4, 3), ["wo", "gate/up", "w2", "qkv(next)"]
            else:
                per, names = stamps[:4 * L].reshape(L, 4, 3), ["qkv", "wo", "gate/up", "w2"]
            rep = {}
            for i, nm in enumerate(names):
                rep[nm] = {"wait_us": float(np.median(per[:, i, 1] - per[:, i, 0]) / 1e3),
                           "work_us": float(np.median(per[:, i, 2] - per[:, i, 1]) / 1e3)}
                if i + 1 < len(names):
                    rep[nm]["gap_to_next_us"] = float(np.median(per[:, i + 1, 0] - per[:, i, 2]) / 1e3)
            rep["layer_us"] = float(np.median(np.diff(per[:, 0, 0])) / 1e3)
            rep["step_us"] = float((stamps[-1, 2] - stamps[0, 0]) / 1e3)
            print(json.dumps({"profiling_only": True, "n_gpus": world, "decode_path": args.decode_path,
                              "decode_step_phases": rep}), flush=True)
    # end to end through the reference-facing generate(): id host->device->host every step
    barrier()
    if args.skip_prefill:
        print(json.dumps({"profiling_only": True, "layers": cfg.n_layers, "ms_per_step": ms / K,
                          "launches_per_step": launches / K}), flush=True)
        model.close()
        return
    ids, t_prefill, t_decode = model.generate(prompt, K + 1)
    e2e_ms = max_over_ranks(t_decode * 1e3)
    e2e = (len(ids) - 1) / (e2e_ms * 1e-3)
    agree_e2e, e2e_ids = gather_ids(ids[:8])
    checks["e2e_ids_agree"] = agree_e2e
    # generate() starts from the same prompt as the device-resident steps above: same kernels, same ids
    checks["e2e_ids_equal_device_resident"] = (e2e_ids[0] == first_token and
                                               e2e_ids[1:] == ids8_list[:len(e2e_ids) - 1])
    require_clean_status(tl, "generate()")

    roof = roofline_gateup(tl, model, stream, torch, cfg.n_layers) if rank == 0 else None
    weight_bytes = model.weight_bytes()
    # the compute-bound companion numbers: one 2048-token prefill (all ranks take part)
    prefill = prefill_2048(model, cfg, world, torch, dist) if cfg.n_layers == CFG.n_layers else None
    require_clean_status(tl, "the 2048-token prefill")
    if fused:
        # the same eight steps with the plain NCCL exchange: summation order differs (ring order against
        # rank order), so equal ids are reported, not required
        from tensorlib_b200 import tp
        model.forward(prompt, 0, all_logits=False)      # the same prefill as for the ids above, so only the decode exchange differs
        tp.close_fused_exchange(model, dist)
        with torch.cuda.stream(stream):
            ids_nccl = model.decode_device(pos0, min(8, K), fetch=True, stream=sp)
        require_clean_status(tl, "the NCCL-exchange decode steps")
        agree_nccl, ids_nccl_list = gather_ids(ids_nccl)
        checks.update({"nccl_ids_agree_across_ranks": agree_nccl, "nccl_first_ids": ids_nccl_list,
                       "fused_ids_equal_nccl_ids": ids_nccl_list == ids8_list})
    model.close()
    if rank == 0:
        peak, _ = measured_peaks()
        emb_bytes = cfg.vocab_size * cfg.dim * 2            # the embedding table is gathered, not streamed
        step_bytes = weight_bytes - emb_bytes
        if roof is not None and prefill is not None:
            roof["prefill_2048"] = {"ms": prefill["ms"], "tflops_per_gpu": prefill["tflops_per_gpu"],
                                    "frac_of_tensor_peak": prefill["frac_of_tensor_peak"], "bound": "tensor"}
        line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16", "data": "synthetic"}
        if world == 1 and cfg.n_layers == CFG.n_layers:
            line["matmul_sweep"] = matmul_sweep(tl, torch, with_baselines=not args.no_cpu)   # long: printed before the headline keys
        line.update({
            "prefill_2048": prefill,
            "config": bench_config(world) if cfg.n_layers == CFG.n_layers else
            {**bench_config(world), "workload": workload_name(world) + f" [PROFILING ONLY: {cfg.n_layers} layers]"},
            "details": {"context_at_start": n_ctx, "tp_exchange": (args.tp_exchange if world > 1 else "none"),
                        "decode_path": "one persistent dataflow kernel per token" if one_kernel else "CUDA graph of fused kernels",
                        "numerics": "fp16 storage, fp32 accumulate", "weight_bytes_per_token_per_gpu": step_bytes,
                        "timed_region": f"{REPEATS} x {K} steps over positions [{pos0}, {pos0 + K}); value = K / median"},
            "repeats": repeats, "checks": checks,
            "gpu_launches": int(launches), "clocks": clocks,
            "step_hbm_frac": (step_bytes / (ms / K * 1e-3) / 1e9) / peak})
        if world == 1 and not args.no_cpu:
            r = cpu_reference_decode(16, 1, budget_s=20.0, context=n_ctx)
            line["cpu_baseline"] = {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"],
                                    "sample": r["sample"], "extrapolation": r["extrapolation"]}
            line["cpu_baseline_other_configs"] = cpu_reference_matmul_and_prefill()
        line["e2e"] = {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8,
                       "prefill_s": t_prefill}
        line["roofline"] = roof
        print(json.dumps(line), flush=True)
    if world > 1:
        from tensorlib_b200 import tp
        tp.destroy()
        dist.destroy_process_group()
    return


def tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def prefill_2048(model, cfg, world, torch, dist, T: int = 2048):
    """Config 3/4 of the benchmark spec: one 2048-token prompt, batch 1, through
    tl_llama2_forward (token ids from the host, last-position logits back to the host)."""
    prompt = synth.prompt_tokens(cfg, SEED + 1, T)
    if world > 1:
        dist.barrier()          # rank 0 arrives late from its single-rank roofline measurement
    model.forward(prompt[:T], 0, all_logits=False)                       # warm-up (allocates score buffers)
    times = []
    for _ in range(3):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        model.forward(prompt, 0, all_logits=False)
        times.append(time.perf_counter() - t0)
    sec = min(times)
    if world > 1:
        t = torch.tensor([sec], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    per_layer = 4 * cfg.dim * cfg.dim + 3 * cfg.dim * cfg.hidden_dim
    linear = 2.0 * T * cfg.n_layers * per_layer + 2.0 * cfg.vocab_size * cfg.dim      # classifier: last row only
    attn = 2.0 * T * (T + 1) * cfg.dim * cfg.n_layers                                 # causal pairs only: 4 hd flops each
    peak, src = tensor_peak()
    tf = (linear + attn) / sec / 1e12
    out_sustained = {}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):      # the rate a seconds-long cuBLAS loop holds under the power cap, for context
        with open(path) as f:
            sustained = json.load(f).get("bf16_tflops_sustained")
        if sustained:
            out_sustained = {"frac_of_sustained_tensor_peak": tf / world / float(sustained)}
    return {"tokens": T, "ms": sec * 1e3, "tokens_per_s": T / sec, "algorithmic_tflop": (linear + attn) / 1e12,
            "tflops": tf, "tflops_per_gpu": tf / world, "frac_of_tensor_peak": tf / world / peak, "peak_source": src,
            **out_sustained,
            "note": "algorithmic flops: all linear layers + causal attention (T (T+1) / 2 query-key pairs per head); "
                    "wall clock through tl_llama2_forward including the host round trip"}


def matmul_sweep(tl, torch, m_list=(1, 8, 32, 128, 512, 2048),
                 kn_list=((4096, 4096), (4096, 11008), (11008, 4096), (4096, 32000)), with_baselines: bool = True):
    """Config 1: y = x W^T, fp16 in / fp32 accumulate, device-resident, through tl_linear_f16 (the weights are
    parameters), rotating over enough weight copies (>= 512 MB) that no launch finds its weights in L2.
    6 x 4 = 24 points, one row each
    (see `columns`). Two same-GPU baselines are timed beside every point, neither on the product
    path: cuBLAS through torch.matmul, and the reference's own CUDA route CUDA<half>::matmul2d
    (gemv_v6 at M = 1, cublasHgemm with a handle created per call otherwise; compiled from the
    reference sources into oracle/_ref) where that library is present."""
    lib = tl.load()
    hbm, _ = measured_peaks()
    tpk, _ = tensor_peak()
    sp = torch.cuda.current_stream().cuda_stream
    ref = None
    if with_baselines:
        try:
            from oracle import ref_lib
            if ref_lib.have_ref():
                ref = ref_lib.RefLib()
                if ref.cuda_device_count() < 1:
                    ref = None
        except Exception:
            ref = None
    rows = []

    def timed(fn, reps):
        for i in range(5):
            fn(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / reps

    for (K, N) in kn_list:
        copies = max(2, -(-512 * 2 ** 20 // (N * K * 2)))
        Ws = [torch.randn(N, K, device="cuda", dtype=torch.float16) * 0.02 for _ in range(copies)]
        W_host = Ws[0].cpu().numpy() if ref is not None else None
        for M in m_list:
            x = torch.randn(M, K, device="cuda", dtype=torch.float16)
            y = torch.empty(M, N, device="cuda", dtype=torch.float16)

            def run(i):      # y = x W^T with W a constant parameter: the nn::Linear form of the sweep
                tl.check(lib.tl_linear_f16(x.data_ptr(), Ws[i % copies].data_ptr(), y.data_ptr(), M, K, N, sp), "tl_linear_f16")
            sec = timed(run, 50)
            want = x[:4].float() @ Ws[49 % copies].float().t()        # the last timed launch, four rows in fp32
            err = float(((y[:4].float() - want).abs() / want.abs().clamp_min(float(want.pow(2).mean().sqrt()))).max())
            if not err <= 1e-2:
                raise SystemExit(f"bench.py: matmul sweep point M={M} K={K} N={N} is off by {err}")
            cublas_us = ref_us = None
            if with_baselines:
                cublas_us = timed(lambda i: torch.matmul(x, Ws[i % copies].t(), out=y), 50) * 1e6
            if ref is not None:
                _, ref_us = ref.cuda_matmul2d(x.cpu().numpy(), W_host, reps=20, b_copies=copies)
            flops, nbytes = 2.0 * M * N * K, 2.0 * (N * K + M * K + M * N)
            t_roof = max(nbytes / (hbm * 1e9), flops / (tpk * 1e12))
            bound = "hbm" if nbytes / (hbm * 1e9) > flops / (tpk * 1e12) else "tensor"
            rows.append([M, K, N, round(sec * 1e6, 2), round(t_roof / sec, 4), bound,
                         round(flops / sec / 1e12, 1) if bound == "tensor" else round(nbytes / sec / 1e9, 1),
                         None if cublas_us is None else round(cublas_us, 2), None if ref_us is None else round(ref_us, 2)])
        del Ws
    st = tl.device_status()
    if st != 0:
        raise SystemExit(f"bench.py: device status {st} after the matmul sweep")
    return {"columns": ["M", "K", "N", "us", "frac_of_roofline", "bound", "TFLOP/s or GB/s", "cublas_us (torch.matmul, baseline)",
                        "ref_cuda_us (the reference's CUDA<half>::matmul2d on this GPU, baseline)"],
            "rows": rows,
            "roofline": "max(2(NK+MK+MN) bytes / measured copy bandwidth, 2MNK flops / measured bf16 burst peak)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--layers", type=int, default=CFG.n_layers, help="profiling only: fewer layers of the 7B shape")
    ap.add_argument("--skip-prefill", action="store_true", help="profiling only: decode without a prompt pass")
    ap.add_argument("--sweep-only", default="", help="profiling only: time one matmul point 'M,K,N' and exit")
    ap.add_argument("--tp-exchange", default="fused", choices=["fused", "nccl"],
                    help="N>1 decode: partial sums exchanged by peer stores inside the GEMV kernels (default) "
                         "or by ncclAllReduce between them")
    ap.add_argument("--decode-path", default="graph", choices=["graph", "kernel"],
                    help="decode step as a CUDA graph of fused kernels (default, the faster one) or as one persistent dataflow kernel")
    ap.add_argument("--profile-step", action="store_true",
                    help="profiling only: after the timed region run one decode step with device timestamps and "
                         "print the per-phase microseconds of rank 0 (median over layers)")
    ap.add_argument("--prefill-only", action="store_true",
                    help="profiling only: just the 2048-token prefill (combine with --layers for a small capture)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.sweep_only:  # profiling only: one point of the matmul sweep, e.g. --sweep-only 2048,4096,4096
        import torch

        import tensorlib_b200 as tl
        torch.cuda.set_device(0)
        tl.init(0)
        M, K, N = (int(v) for v in args.sweep_only.split(","))
        print(json.dumps({"profiling_only": True, "matmul_sweep": matmul_sweep(tl, torch, (M,), ((K, N),), with_baselines=False)}), flush=True)
        return
    if args.prefill_only:
        import torch

        import tensorlib_b200 as tl
        torch.cuda.set_device(0)
        tl.init(0)
        cfg = synth.LlamaConfig(dim=CFG.dim, hidden_dim=CFG.hidden_dim, n_layers=args.layers, n_heads=CFG.n_heads,
                                vocab_size=CFG.vocab_size, seq_len=CFG.seq_len, shared_classifier=False)
        model = tl.Llama2(cfg, numerics=tl.FAST)
        model.init_random(SEED, 0.02)
        print(json.dumps({"profiling_only": True, "layers": args.layers,
                          "prefill_2048": prefill_2048(model, cfg, 1, torch, None)}), flush=True)
        model.close()
        return
    if args.warmup < 3:
        args.warmup = 3
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
