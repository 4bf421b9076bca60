#!/usr/bin/env python
"""Headline benchmark: greedy decode tokens/s of a Llama2-7B-shaped fp16 model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decoded token (one pass over all weights). N = 1 runs the 7B shape on one B200
(128-token seeded prompt, then decode); N > 1 (under torchrun, one rank per GPU) runs the same
model tensor-parallel with a 512-token context. Weights are random N(0, 0.02) generated on the
device, norms = 1, token ids seeded: synthetic data of the benchmark's shape.

The JSON line:
  value      tokens/s with everything resident on the device: one CUDA-graph replay per token,
             the sampled id fed back in device memory; timed with CUDA events on the launching
             stream, barrier + synchronize on both sides, max over ranks.
  e2e        the same metric through the reference-facing call tl_llama2_generate: every step
             moves the token id host->device and the sampled id device->host, like
             Llama2::generate does; wall clock like the reference measures it.
  roofline   the dominant kernel (RMSNorm + w1|w3 GEMV + SiLU*up, 43 % of the weight bytes of a
             token), launched over all layers' weights (5.8 GB >> L2) and timed with CUDA events.
  cpu_baseline / --impl reference
             the reference's own OpenMP CPU code (oracle/_ref) on the host cores, on a bounded
             sample: a ONE-layer 7B-shaped model with 1/32 of the classifier rows, one decode
             step per sample; a full token is 32 such samples.
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
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
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
def cpu_reference_decode(steps: int, warmup: int, budget_s: float):
    """Decode steps of a one-layer 7B-shaped model (vocab/32 classifier rows) on the reference's
    CPU backend. Returns (tokens_per_s_extrapolated, ms_per_step, cores, kind, steps_done)."""
    from oracle import ref_lib
    if ref_lib.have_ref():
        lib, kind = ref_lib.RefLib(), "reference"
    else:
        lib, kind = ref_lib.OracleLib(), "port"
    layers_full = CFG.n_layers
    cfg = synth.LlamaConfig(dim=CFG.dim, hidden_dim=CFG.hidden_dim, n_layers=1, n_heads=CFG.n_heads,
                            vocab_size=CFG.vocab_size // layers_full, seq_len=CFG.seq_len, shared_classifier=True)
    # values do not matter for timing: one seeded block tiled over the payload
    block = synth.normal_f16(SEED, 1, 1 << 22, 0.02)
    payload = np.resize(block, cfg.payload_elems())
    d, L, V = cfg.dim, cfg.n_layers, cfg.vocab_size
    payload[V * d: V * d + L * d] = 1.0                                   # attention_norm
    off = V * d + L * d + 4 * L * d * d
    payload[off: off + L * d] = 1.0                                       # ffn_norm
    payload[-d:] = 1.0                                                    # final norm
    model = lib.llama2(cfg, payload)
    tok = np.array([1], dtype=np.int32)
    pos = 0
    for _ in range(warmup):
        model.forward(tok, pos, 1); pos += 1
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        model.forward(tok, pos, 1); pos += 1; done += 1
        if time.perf_counter() - t0 > budget_s and done >= 3:
            break
    dt = (time.perf_counter() - t0) / done
    return 1.0 / (dt * layers_full), dt * 1e3, lib.max_threads(), kind, done


def run_reference_arm(args, rank: int):
    if rank != 0:
        return
    tps, ms, cores, kind, done = cpu_reference_decode(args.steps, max(args.warmup, 1), budget_s=150.0)
    sample = ("one decode step of a 1-layer 7B-shaped model with vocab/32 classifier rows "
              "(= 1/32 of a token) per step; tokens/s = 1 / (32 x step time)")
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": done, "warmup": max(args.warmup, 1), "ms_per_step": ms * CFG.n_layers,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": workload_name(args.gpus), "timing": "host wall clock, OpenMP on all host cores"},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
def roofline_gateup(tl, model, stream, torch, n_layers):
    """Time the dominant kernel over all layers' w1|w3 (distinct weights every launch)."""
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
    sec = e0.elapsed_time(e1) * 1e-3 / (reps * L)
    bytes_per_launch = 2 * hid * dim * 2 + 2 * dim * 2 + hid * 2   # w1+w3, x + norm weight, out
    peak, peak_src = measured_peaks()
    achieved = bytes_per_launch / sec / 1e9
    traffic = NCU_TRAFFIC_GATEUP // model.c.tp_world   # weight rows per launch scale as 1 / ranks
    return {"bound": "hbm", "kernel": "k_gemv_ring<SWIGLU,NORM> (RMSNorm + w1|w3 GEMV + SiLU*up)",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
            "bytes_per_launch": bytes_per_launch, "us_per_launch": sec * 1e6, "traffic": traffic,
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
    model = tl.Llama2(cfg, numerics=tl.FAST, tp_rank=rank, tp_world=world)
    if world > 1:
        from tensorlib_b200 import tp
        tp.attach(model, rank, world, dist)
        if args.tp_exchange == "fused":
            tp.open_fused_exchange(model, rank, world, dist)
    model.init_random(SEED, 0.02)

    n_ctx = 128 if world == 1 else 512
    K, W = args.steps, args.warmup
    assert n_ctx + W + 2 * K + 2 <= CFG.seq_len, "steps + warmup exceed the 2048-token context"
    prompt = synth.prompt_tokens(CFG, SEED, n_ctx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # prefill (untimed): leaves the first sampled id in the device slot
    if args.skip_prefill:
        model.set_next_token(int(prompt[-1]))      # profiling runs: decode over a zero KV cache
    else:
        model.forward(prompt, 0, all_logits=False)
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    pos = n_ctx
    with torch.cuda.stream(stream):
        model.decode_device(pos, W, fetch=False, stream=sp)           # warm-up (captures the graph)
        pos += W
        barrier()
        launches0 = model.kernel_launches()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        model.decode_device(pos, K, fetch=False, stream=sp)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop() if rank == 0 else None
        launches = model.kernel_launches() - launches0
        pos += K
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = K / (ms * 1e-3)

    # end to end through the reference-facing generate(): id host->device->host every step
    barrier()
    if args.skip_prefill:
        print(json.dumps({"profiling_only": True, "layers": cfg.n_layers, "ms_per_step": ms / K,
                          "launches_per_step": launches / K}), flush=True)
        model.close()
        return
    ids, t_prefill, t_decode = model.generate(prompt, K + 1)
    e2e_ms = t_decode * 1e3
    if world > 1:
        t = torch.tensor([e2e_ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e = (len(ids) - 1) / (e2e_ms * 1e-3)

    roof = roofline_gateup(tl, model, stream, torch, cfg.n_layers) if rank == 0 else None
    weight_bytes = model.weight_bytes()
    if rank == 0:
        peak, _ = measured_peaks()
        emb_bytes = cfg.vocab_size * cfg.dim * 2            # the embedding table is gathered, not streamed
        step_bytes = weight_bytes - emb_bytes
        line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16", "data": "synthetic",
                "config": {"workload": workload_name(world) + ("" if cfg.n_layers == CFG.n_layers else f" [PROFILING ONLY: {cfg.n_layers} layers]"),
                           "context_at_start": n_ctx + W,
                           "parallelism": f"tp{world}",
                           "tp_exchange": (args.tp_exchange if world > 1 else "none"), "numerics": "fp16 storage, fp32 accumulate",
                           "l2": "inputs larger than L2 (weights streamed per token >> 126 MB)",
                           "weight_bytes_per_token_per_gpu": step_bytes},
                "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4,
                        "prefill_s": t_prefill},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
                "step_hbm_frac": (step_bytes / (ms / K * 1e-3) / 1e9) / peak}
        if world == 1 and not args.no_cpu:
            tps, ms_cpu, cores, kind, done = cpu_reference_decode(64, 2, budget_s=20.0)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": kind,
                                    "sample": f"{done} decode steps of a 1-layer 7B-shaped model with vocab/32 "
                                              "classifier rows (1/32 of a token each), extrapolated x32"}
    # the compute-bound companion numbers: one 2048-token prefill (all ranks take part)
    prefill = prefill_2048(model, cfg, world, torch, dist) if cfg.n_layers == CFG.n_layers else None
    if world > 1 and args.tp_exchange == "fused":
        from tensorlib_b200 import tp
        tp.close_fused_exchange(model, dist)
    model.close()
    if rank == 0:
        line["prefill_2048"] = prefill
        if world == 1:
            line["matmul_sweep"] = matmul_sweep(tl, torch)
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
                 kn_list=((4096, 4096), (4096, 11008), (11008, 4096), (4096, 32000))):
    """Config 1: y = x W^T, fp16 in / fp32 accumulate, device-resident, rotating over enough
    weight copies (>= 512 MB) that no launch finds its weights in L2."""
    lib = tl.load()
    hbm, _ = measured_peaks()
    tpk, _ = tensor_peak()
    sp = torch.cuda.current_stream().cuda_stream
    out = []
    for (K, N) in kn_list:
        copies = max(2, -(-512 * 2 ** 20 // (N * K * 2)))
        Ws = [torch.randn(N, K, device="cuda", dtype=torch.float16) * 0.02 for _ in range(copies)]
        for M in m_list:
            x = torch.randn(M, K, device="cuda", dtype=torch.float16)
            y = torch.empty(M, N, device="cuda", dtype=torch.float16)

            def run(i):
                tl.check(lib.tl_matmul2d_f16(x.data_ptr(), Ws[i % copies].data_ptr(), y.data_ptr(), M, N, K,
                                             tl.FAST, sp), "tl_matmul2d_f16")
            for i in range(5):
                run(i)
            reps = 50
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for i in range(reps):
                run(i)
            e1.record()
            torch.cuda.synchronize()
            sec = e0.elapsed_time(e1) * 1e-3 / reps
            flops, nbytes = 2.0 * M * N * K, 2.0 * (N * K + M * K + M * N)
            t_roof = max(nbytes / (hbm * 1e9), flops / (tpk * 1e12))
            out.append({"M": M, "K": K, "N": N, "us": sec * 1e6, "tflops": flops / sec / 1e12,
                        "gbs": nbytes / sec / 1e9, "bound": "hbm" if nbytes / (hbm * 1e9) > flops / (tpk * 1e12) else "tensor",
                        "frac_of_roofline": t_roof / sec})
        del Ws
    return out


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
        print(json.dumps({"profiling_only": True, "matmul_sweep": matmul_sweep(tl, torch, (M,), ((K, N),))}), flush=True)
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
