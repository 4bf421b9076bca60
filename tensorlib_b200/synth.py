"""Seeded synthetic inputs: weights, activations, prompts and llama2.c-layout checkpoints.

Counter-based, so any slice of any tensor can be produced independently of the rest (a
tensor-parallel rank can generate only its shard): element ``i`` of tensor ``tensor_id`` under
``seed`` is a pure function of ``(seed, tensor_id, i)``. The mixing function is splitmix64; normals
come from Box-Muller in float64 and are rounded once to fp16.

The checkpoint layout written by :func:`llama2c_payload` / :func:`write_llama2c_file` is the
llama2.c "legacy v0" fp16 layout the reference reads (model/llama2_7b/src/main.cpp:26-34 for the
7-int header, :36-190 for the tensor order; script/export.py:138-190 writes it): header
``dim, hidden_dim, n_layers, n_heads, n_kv_heads, +-vocab_size, seq_len`` (a positive vocab_size
means the classifier shares the embedding table), then tok_embeddings, attention_norm[L], wq[L],
wk[L], wv[L], wo[L], ffn_norm[L], w1[L], w2[L], w3[L], final norm, and for untied files
``seq_len*head_size`` RoPE values (written twice by the exporter, read once and skipped by the
reference) followed by wcls.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = x
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def _key(seed: int, tensor_id: int) -> np.uint64:
    with np.errstate(over="ignore"):
        k = _splitmix64(np.array([seed & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))
        k = _splitmix64(k ^ np.uint64(tensor_id & 0xFFFFFFFFFFFFFFFF))
    return k[0]


def uniform_bits(seed: int, tensor_id: int, start: int, count: int) -> np.ndarray:
    """64 random bits per element for elements [start, start+count)."""
    with np.errstate(over="ignore"):
        idx = np.arange(start, start + count, dtype=np.uint64)
        return _splitmix64(idx * np.uint64(0xD1342543DE82EF95) + _key(seed, tensor_id))


def normal_f16(seed: int, tensor_id: int, count: int, std: float, start: int = 0,
               chunk: int = 1 << 22) -> np.ndarray:
    """N(0, std^2) rounded to fp16, elements [start, start+count) of the stream."""
    out = np.empty(count, dtype=np.float16)
    for off in range(0, count, chunk):
        n = min(chunk, count - off)
        bits = uniform_bits(seed, tensor_id, start + off, n)
        u1 = ((bits >> np.uint64(32)).astype(np.float64) + 1.0) / 4294967296.0  # (0, 1]
        u2 = (bits & np.uint64(0xFFFFFFFF)).astype(np.float64) / 4294967296.0   # [0, 1)
        z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
        out[off:off + n] = (z * std).astype(np.float16)
    return out


def token_ids(seed: int, tensor_id: int, count: int, vocab: int) -> np.ndarray:
    """`count` token ids uniform in [0, vocab)."""
    bits = uniform_bits(seed, tensor_id, 0, count)
    return ((bits >> np.uint64(11)) % np.uint64(vocab)).astype(np.int32)


@dataclass(frozen=True)
class LlamaConfig:
    dim: int
    hidden_dim: int
    n_layers: int
    n_heads: int
    vocab_size: int
    seq_len: int
    shared_classifier: bool = True

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    def header(self) -> bytes:
        v = self.vocab_size if self.shared_classifier else -self.vocab_size
        return struct.pack("<7i", self.dim, self.hidden_dim, self.n_layers, self.n_heads,
                           self.n_heads, v, self.seq_len)

    def payload_elems(self) -> int:
        d, h, L, V = self.dim, self.hidden_dim, self.n_layers, self.vocab_size
        n = V * d + L * (2 * d + 4 * d * d + 3 * d * h) + d
        if not self.shared_classifier:
            n += self.seq_len * self.head_dim + V * d
        return n


TINY = LlamaConfig(dim=288, hidden_dim=768, n_layers=6, n_heads=6, vocab_size=32000, seq_len=256,
                   shared_classifier=True)
LLAMA2_7B = LlamaConfig(dim=4096, hidden_dim=11008, n_layers=32, n_heads=32, vocab_size=32000,
                        seq_len=2048, shared_classifier=False)

# tensor ids of the synthetic streams
TID_EMB, TID_WQ, TID_WK, TID_WV, TID_WO, TID_W1, TID_W2, TID_W3, TID_WCLS = range(1, 10)
TID_PROMPT = 100
TID_SWEEP_W, TID_SWEEP_X = 200, 201


def llama2c_payload(cfg: LlamaConfig, seed: int, std: float = 0.02) -> np.ndarray:
    """All weights in checkpoint order as one fp16 array (everything after the header).

    Linear and embedding weights ~ N(0, std^2); RMSNorm weights = 1."""
    d, h, L, V = cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.vocab_size
    parts = [normal_f16(seed, TID_EMB, V * d, std)]
    ones = np.ones(L * d, dtype=np.float16)
    parts.append(ones)                                     # attention_norm[L]
    for tid in (TID_WQ, TID_WK, TID_WV, TID_WO):           # layer l of a kind = slice l of one stream
        parts.append(normal_f16(seed, tid, L * d * d, std))
    parts.append(ones)                                     # ffn_norm[L]
    for tid in (TID_W1, TID_W2, TID_W3):
        parts.append(normal_f16(seed, tid, L * d * h, std))
    parts.append(np.ones(d, dtype=np.float16))             # final norm
    if not cfg.shared_classifier:
        parts.append(np.zeros(cfg.seq_len * cfg.head_dim, dtype=np.float16))  # skipped by readers
        parts.append(normal_f16(seed, TID_WCLS, V * d, std))
    out = np.concatenate(parts)
    assert out.size == cfg.payload_elems()
    return out


def write_llama2c_file(path: str, cfg: LlamaConfig, seed: int, std: float = 0.02) -> None:
    with open(path, "wb") as f:
        f.write(cfg.header())
        llama2c_payload(cfg, seed, std).tofile(f)


def prompt_tokens(cfg: LlamaConfig, seed: int, count: int) -> np.ndarray:
    return token_ids(seed, TID_PROMPT, count, cfg.vocab_size)
