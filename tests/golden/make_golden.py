"""Generate the golden fixtures in this folder from the REFERENCE ITSELF.

Runs the reference's own CPU code (oracle/_ref/libtl_ref.so, built by oracle/Makefile from the
unmodified reference sources, variable REF there) on seeded synthetic inputs and stores small outputs:

  tiny_llama2.npz   config 0 of the benchmark spec: tiny Llama2 (dim 288, hidden 768, 6 layers,
                    6 heads, vocab 32000, seq 256), weights N(0, 0.02) seed 20240229, norms = 1,
                    16 seeded prompt ids, 128 greedy ids; for both SiLU routes ("A" = CPU fp16
                    SiLU as shipped, "B" = SiLU through float as on the reference's CUDA path):
                    the ids, the last-position logits of four steps and a SHA-256 over the
                    logits of all steps; plus a teacher-forced pass over 24 seeded ids
                    (prefill of 16, then 8 single-token steps) with its logits hash and samples.
  ops.npz           single operators on seeded inputs: matmul (several shapes incl. odd ones),
                    rms_norm, rotary embedding, softmax, silu, argmax.
  matmul_sweep.npz  the four (K, N) pairs of the sweep at M = 1 and 8: SHA-256 of the outputs and
                    the first 64 values of each; at M = 32, 128, 512 and 2048: three rows (first,
                    one past the middle, last) x the first and last 32 columns.

Only this script needs the reference checkout (through the built library); the tests read the .npz
files. Usage:  make -C oracle ref && python tests/golden/make_golden.py
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from oracle.ref_lib import RefLib  # noqa: E402
from tensorlib_b200 import synth  # noqa: E402

SEED = 20240229
N_PROMPT, N_GEN = 16, 128
KEEP_STEPS = (0, 1, 64, 127)
SWEEP = ((4096, 4096), (4096, 11008), (11008, 4096), (4096, 32000))
SWEEP_LARGE_M = (32, 128, 512, 2048)


def sweep_sample(M: int, N: int):
    """Rows and columns of the large-M sweep points that the fixture pins."""
    return np.array([0, M // 2 + 1, M - 1]), np.concatenate([np.arange(32), np.arange(N - 32, N)])


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).view(np.uint8).tobytes()).hexdigest()


def op_inputs():
    """Seeded inputs of ops.npz; tests rebuild them with the same calls."""
    d = {}
    for name, (M, N, K) in {"mm_small": (5, 77, 300), "mm_odd": (3, 33, 37), "mm_tiny_qkv": (1, 288, 288),
                            "mm_tiny_ffn": (8, 768, 288), "mm_m1": (1, 512, 4096), "mm_m16": (16, 256, 1024),
                            "mm_m130": (130, 136, 264)}.items():
        d[name] = (synth.normal_f16(SEED, 301, M * K, 1.0).reshape(M, K),
                   synth.normal_f16(SEED, 302, N * K, 0.02).reshape(N, K))
    d["norm288"] = (synth.normal_f16(SEED, 310, 7 * 288, 1.0).reshape(7, 288), synth.normal_f16(SEED, 311, 288, 1.0))
    d["norm4096"] = (synth.normal_f16(SEED, 312, 3 * 4096, 2.0).reshape(3, 4096), synth.normal_f16(SEED, 313, 4096, 1.0))
    d["rope48"] = (synth.normal_f16(SEED, 320, 40 * 6 * 48, 1.0).reshape(40, 6, 48), 100)
    d["rope128"] = (synth.normal_f16(SEED, 321, 9 * 2 * 128, 1.0).reshape(9, 2, 128), 2000)
    sm = synth.normal_f16(SEED, 330, 50 * 333, 3.0).reshape(50, 333).copy()
    sm[3, 100:] = -np.inf
    d["softmax"] = (sm,)
    d["silu"] = (synth.normal_f16(SEED, 340, 4096, 4.0),)
    am = synth.normal_f16(SEED, 350, 4 * 32000, 1.0).reshape(4, 32000).copy()
    am[1, 500] = am[1].max()
    am[1, 20000] = am[1].max()
    d["argmax"] = (am,)
    return d


def main():
    ref = RefLib()
    if "--only-sweep" not in sys.argv:
        tiny_and_ops(ref)
    sweep(ref)


def tiny_and_ops(ref):
    # ---- tiny Llama2 ---------------------------------------------------------------------------
    cfg = synth.TINY
    payload = synth.llama2c_payload(cfg, SEED)
    prompt = synth.prompt_tokens(cfg, SEED, N_PROMPT)
    model = ref.llama2(cfg, payload)
    out = {"prompt": prompt, "seed": np.int64(SEED), "keep_steps": np.array(KEEP_STEPS, dtype=np.int32)}
    for mode, tag in ((0, "A"), (1, "B")):
        ids, logits = model.generate(prompt, N_GEN, silu_mode=mode, keep_logits=True)
        out[f"ids_{tag}"] = ids
        out[f"logits_{tag}"] = logits[list(KEEP_STEPS)]
        out[f"logits_sha_{tag}"] = np.array(sha(logits))
        s = np.sort(logits.astype(np.float32), axis=1)
        out[f"margin_{tag}"] = (s[:, -1] - s[:, -2]).astype(np.float32)
        print(tag, "ids", ids[:8], "...", "min margin", out[f"margin_{tag}"].min())
    forced = synth.token_ids(SEED, 101, 24, cfg.vocab_size)
    out["forced_tokens"] = forced
    for mode, tag in ((0, "A"), (1, "B")):
        lg = [model.forward(forced[:16], 0, mode)]
        for i in range(16, 24):
            lg.append(model.forward(forced[i:i + 1], i, mode))
        lg = np.concatenate(lg, axis=0)                      # (24, vocab)
        out[f"forced_sha_{tag}"] = np.array(sha(lg))
        out[f"forced_logits_{tag}"] = lg[[0, 15, 16, 23]]
        out[f"forced_argmax_{tag}"] = ref.argmax(np.ascontiguousarray(lg))
    np.savez_compressed(os.path.join(HERE, "tiny_llama2.npz"), **out)

    # ---- single operators -----------------------------------------------------------------------
    ins = op_inputs()
    ops = {}
    for name, args in ins.items():
        if name.startswith("mm_"):
            ops[name] = ref.matmul2d(*args)
        elif name.startswith("norm"):
            ops[name] = ref.rmsnorm(*args)
        elif name.startswith("rope"):
            ops[name] = ref.rope(*args)
        elif name == "softmax":
            ops[name] = ref.softmax(*args)
        elif name == "silu":
            ops["silu_float"] = ref.silu(args[0], True)
            ops["silu_half"] = ref.silu(args[0], False)
        elif name == "argmax":
            ops[name] = ref.argmax(*args)
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **ops)



def sweep(ref):
    # ---- matmul sweep at CPU-affordable M -------------------------------------------------------
    sw = {}
    for (K, N) in SWEEP:
        W = synth.normal_f16(SEED, synth.TID_SWEEP_W, N * K, 0.02).reshape(N, K)
        for M in (1, 8):
            x = synth.normal_f16(SEED, synth.TID_SWEEP_X, M * K, 1.0).reshape(M, K)
            y = ref.matmul2d(x, W)
            sw[f"sha_K{K}_N{N}_M{M}"] = np.array(sha(y))
            sw[f"head_K{K}_N{N}_M{M}"] = y.reshape(-1)[:64].copy()
            print("sweep", K, N, M, sha(y)[:12])
        for M in SWEEP_LARGE_M:       # every output element is an independent dot product: sample some
            x = synth.normal_f16(SEED, synth.TID_SWEEP_X, M * K, 1.0).reshape(M, K)
            rows, cols = sweep_sample(M, N)
            sw[f"sample_K{K}_N{N}_M{M}"] = ref.matmul2d(np.ascontiguousarray(x[rows]), np.ascontiguousarray(W[cols]))
    np.savez_compressed(os.path.join(HERE, "matmul_sweep.npz"), **sw)


if __name__ == "__main__":
    main()
