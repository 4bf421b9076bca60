"""Generates tests/golden/tokenizer.bin (a small synthetic llama2.c-format vocabulary) and
tests/golden/tokenizer_cases.json (encodings / decodings produced by the reference's own
Tokenizer, compiled by `make -C oracle ref_tok`). Run in the build container, where the
reference sources exist:

    make -C oracle ref_tok && python tests/golden/make_tokenizer_golden.py

The vocabulary is synthetic (no real tokenizer model is reproduced): ids 0..2 are <unk>, <s>,
</s>; 3..258 the byte tokens <0x00>..<0xFF>; then single characters; then multi-character pieces
whose score decreases in listing order (the merge loop takes the highest score first).
"""
import ctypes as C
import json
import os
import struct

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))

SINGLES = list(" abcdefghijklmnopqrstuvwxyz") + list("ABCDEFGHIJKLM") + list("0123456789") + \
    list(".,!?'\"-:;()[]/\n") + ["é", "ü", "ß", "中", "文", "故", "事", "€"]
MERGES = [" t", "he", " a", "in", " the", "re", " s", "er", "on", " w", "at", "en", "it", "is", "an", "or", "es", " b",
          "ed", " c", "ing", " f", "ou", " p", "ar", "al", " m", " o", "le", " d", "ll", " h", " in", "nd", " to", "st",
          " of", " and", "hel", "hell", "hello", " hello", " wor", "ld", " world", "tell", " tell", " me", " sto",
          " story", "ry", " on", " once", "ce", " up", " upon", " time", "ti", "me", " [", "IN", "INS", "ST", "[/",
          " [/", "T]", " 中", "中文", " 故事", "故事", "!!", "...", " A", " I", "th", " th", " that", "ha"]


def write_vocab(path):
    pieces = ["<unk>", "<s>", "</s>"] + [f"<0x{i:02X}>" for i in range(256)]
    scores = [0.0] * len(pieces)
    for ch in SINGLES:
        pieces.append(ch)
        scores.append(-1000.0)
    for rank, m in enumerate(MERGES):
        pieces.append(m)
        scores.append(-float(rank + 1))
    assert len(set(pieces)) == len(pieces)
    with open(path, "wb") as f:
        f.write(struct.pack("<i", max(len(p.encode()) for p in pieces)))
        for p, s in zip(pieces, scores):
            b = p.encode()
            f.write(struct.pack("<fi", s, len(b)))
            f.write(b)
    return len(pieces)


TEXTS = ["hello world", "tell me a story", " the  thing in the hall", "once upon a time...", "[INST] hello [/INST]",
         "用中文讲一个故事", "中文 故事!!", "Zebra & Yak €5", "café über straße", "a", " ", "\n\nthat is it.", "hello" * 7,
         "😀 ok", "I said: 'on and on'"]


def main():
    vocab_path = os.path.join(HERE, "tokenizer.bin")
    n = write_vocab(vocab_path)
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libtl_ref_tok.so"))
    lib.reftok_create.restype = C.c_void_p
    lib.reftok_create.argtypes = [C.c_char_p, C.c_int]
    lib.reftok_encode.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int]
    lib.reftok_decode.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_char_p, C.c_int]
    lib.reftok_destroy.argtypes = [C.c_void_p]
    cases = []
    for text in TEXTS:
        for bos, eos in ((1, 0), (0, 0), (1, 1)):
            # a fresh tokenizer per case: the reference's decode() edits its vocabulary in place
            # (Tokenizer.cpp:155-167 assigns through a reference), so state must not leak
            t = lib.reftok_create(vocab_path.encode(), n)
            buf = (C.c_int * 4096)()
            cnt = lib.reftok_encode(t, text.encode(), bos, eos, buf, 4096)
            ids = [int(buf[i]) for i in range(cnt)]
            # decode every id once, in order, with the true predecessor (first use of each entry,
            # i.e. before the in-place edit can have touched it)
            seen, dec = set(), []
            prev = 0
            for tok in ids:
                if tok not in seen:
                    out = C.create_string_buffer(256)
                    ln = lib.reftok_decode(t, prev, tok, out, 256)
                    dec.append([prev, tok, list(out.raw[:ln])])
                    seen.add(tok)
                prev = tok
            lib.reftok_destroy(t)
            cases.append({"text": text, "bos": bos, "eos": eos, "ids": ids, "decode": dec})
    with open(os.path.join(HERE, "tokenizer_cases.json"), "w") as f:
        json.dump({"vocab_size": n, "cases": cases}, f, ensure_ascii=True, indent=0)
    print("vocab", n, "cases", len(cases))


if __name__ == "__main__":
    main()
