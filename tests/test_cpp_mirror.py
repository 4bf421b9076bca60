"""The C++ host mirror of the reference API (include/tensorlib_b200.hpp) over the C ABI.

tests/cpp/host_mirror_test.cpp is compiled with g++ against the header and the shared library.
Without a GPU it must refuse every call loudly; on a B200 it must reproduce the reference's CPU
matmul bit for bit (reference-order numerics) and its 128 greedy token ids on the tiny config.
"""
import os
import subprocess

import numpy as np
import pytest

from tensorlib_b200 import synth

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
SRC = os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp")
LIBDIR = os.path.join(ROOT, "tensorlib_b200")


@pytest.fixture(scope="module")
def mirror_binary(tmp_path_factory):
    import tensorlib_b200 as t
    if not os.path.exists(t.LIB_PATH):
        subprocess.run(["python", "-m", "tensorlib_b200.build"], cwd=ROOT, check=True)
    exe = str(tmp_path_factory.mktemp("cpp") / "host_mirror_test")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe,
           "-L", LIBDIR, "-ltensorlib_b200", f"-Wl,-rpath,{LIBDIR}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_cpp_mirror_compiles_and_refuses_without_a_device(mirror_binary):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present: the refusal path is the GPU-less one")
    r = subprocess.run([mirror_binary, "nogpu"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "no CPU path" in r.stdout and "FAIL" not in r.stdout


def test_cpp_tokenizer_matches_the_reference_tokenizer(mirror_binary, tmp_path):
    """Host only: every encoding and decoded piece of the committed fixture, which
    tests/golden/make_tokenizer_golden.py produced with the reference's own Tokenizer."""
    import json
    golden = os.path.join(ROOT, "tests", "golden")
    with open(os.path.join(golden, "tokenizer_cases.json")) as f:
        g = json.load(f)
    lines = [f"{g['vocab_size']} {len(g['cases'])}"]
    for c in g["cases"]:
        tb = list(c["text"].encode())
        parts = [c["bos"], c["eos"], len(tb), *tb, len(c["ids"]), *c["ids"], len(c["decode"])]
        for prev, tok, piece in c["decode"]:
            parts += [prev, tok, len(piece), *piece]
        lines.append(" ".join(str(int(v)) for v in parts))
    cases = tmp_path / "tok_cases.txt"
    cases.write_text("\n".join(lines) + "\n")
    r = subprocess.run([mirror_binary, "tokenizer", os.path.join(golden, "tokenizer.bin"), str(cases)],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "OK tokenizer" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_mirror_matches_reference_on_tiny_config(mirror_binary, oracle, golden_tiny, tmp_path):
    cfg = synth.TINY
    ckpt = str(tmp_path / "tiny.bin")
    synth.write_llama2c_file(ckpt, cfg, 20240229)          # same seed as the tiny_payload fixture
    M, N, K = 5, 96, 64
    A = synth.normal_f16(61, 1, M * K, 1.0).reshape(M, K)
    W = synth.normal_f16(61, 2, N * K, 0.02).reshape(N, K)
    want = oracle.matmul2d(A, W)
    prompt, ids = golden_tiny["prompt"], golden_tiny["ids_B"]
    case = tmp_path / "case.txt"
    with open(case, "w") as f:
        f.write(f"{cfg.dim} {cfg.hidden_dim} {cfg.n_layers} {cfg.n_heads} {cfg.vocab_size} {cfg.seq_len}\n")
        f.write(f"{len(prompt)} " + " ".join(str(int(v)) for v in prompt) + "\n")
        f.write(f"{len(ids)} " + " ".join(str(int(v)) for v in ids) + "\n")
        f.write(f"{M} {N} {K}\n")
        for a in (A, W, want):
            f.write(" ".join(str(int(v)) for v in np.ascontiguousarray(a).view(np.uint16).reshape(-1)) + "\n")
    r = subprocess.run([mirror_binary, "gpu", ckpt, str(case)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "FAIL" not in r.stdout and r.stdout.count("OK ") >= 7, r.stdout


@pytest.mark.gpu
def test_cpp_mirror_chat_carries_the_position_across_turns(mirror_binary, tmp_path):
    """Llama2::chat of the mirror (the reference's llama2.cpp:119-146): two user turns read from a stream, each
    rendered as [INST] .. [/INST]; the second turn must continue at the first turn's end position over the same KV
    cache. A small random model whose vocabulary is the synthetic tokenizer's."""
    import json
    golden = os.path.join(ROOT, "tests", "golden")
    with open(os.path.join(golden, "tokenizer_cases.json")) as f:
        vocab = int(json.load(f)["vocab_size"])
    cfg = synth.LlamaConfig(dim=64, hidden_dim=160, n_layers=2, n_heads=2, vocab_size=vocab, seq_len=128)
    ckpt = str(tmp_path / "chat.bin")
    synth.write_llama2c_file(ckpt, cfg, 4242)
    r = subprocess.run([mirror_binary, "chat", ckpt, os.path.join(golden, "tokenizer.bin"), str(cfg.dim), str(cfg.hidden_dim),
                        str(cfg.n_layers), str(cfg.n_heads), str(cfg.vocab_size), str(cfg.seq_len)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "FAIL" not in r.stdout and r.stdout.count("OK chat") == 3, r.stdout
