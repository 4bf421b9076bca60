"""GPU parity, Llama2 forward (tiny config of the benchmark spec), through the C ABI.

Reference-order numerics: logits bit-identical to the oracle / golden fixtures, hence the same
128 greedy ids. Fast numerics: logits within tolerance; greedy ids compared teacher-forced, and
the free-running match length is reported (top-2 logit margins of this random-weight model are
often 1-2 fp16 ulps, so the free-running sequence is a statement about rounding order).
"""
import hashlib
import os
import sys

import numpy as np
import pytest

from conftest import assert_bit_equal

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import N_GEN, SEED  # noqa: E402

from tensorlib_b200 import synth  # noqa: E402

pytestmark = pytest.mark.gpu


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).view(np.uint8).tobytes()).hexdigest()


def make_model(tl, payload, numerics, silu_via_float=True):
    m = tl.Llama2(synth.TINY, numerics=numerics, silu_via_float=silu_via_float)
    m.load_payload(payload, shared_classifier=True)
    return m


@pytest.mark.parametrize("tag,via_float", [("B", True), ("A", False)])
def test_refmode_greedy_ids_and_logits_match_reference(tl, golden_tiny, tiny_payload, tag, via_float):
    m = make_model(tl, tiny_payload, tl.REFERENCE_ORDER, via_float)
    prompt = golden_tiny["prompt"]
    ids, _, _ = m.generate(prompt, N_GEN)
    assert np.array_equal(ids, golden_tiny[f"ids_{tag}"]), "greedy token ids differ from the reference"
    # logits of every step, recomputed teacher-forced along the reference's own ids
    logits = [m.forward(prompt, 0, all_logits=True)[-1]]
    pos = prompt.size
    for t in golden_tiny[f"ids_{tag}"][:-1]:
        logits.append(m.forward(np.array([t], dtype=np.int32), pos, all_logits=True)[0])
        pos += 1
    logits = np.stack(logits)
    assert_bit_equal(logits[list(golden_tiny["keep_steps"])], golden_tiny[f"logits_{tag}"], "kept logits")
    assert sha(logits) == str(golden_tiny[f"logits_sha_{tag}"])
    m.close()


def test_refmode_teacher_forced_all_positions(tl, golden_tiny, tiny_payload):
    m = make_model(tl, tiny_payload, tl.REFERENCE_ORDER)
    forced = golden_tiny["forced_tokens"]
    lg = [m.forward(forced[:16], 0, all_logits=True)]
    for i in range(16, 24):
        lg.append(m.forward(forced[i:i + 1], i, all_logits=True))
    lg = np.concatenate(lg, axis=0)
    assert sha(lg) == str(golden_tiny["forced_sha_B"])
    assert np.array_equal(tl.argmax(lg), golden_tiny["forced_argmax_B"])
    m.close()


def test_refmode_device_decode_equals_host_loop(tl, golden_tiny, tiny_payload):
    m = make_model(tl, tiny_payload, tl.REFERENCE_ORDER)
    prompt = golden_tiny["prompt"]
    m.forward(prompt, 0, all_logits=False)               # leaves the sampled id in the device slot
    ids = m.decode_device(prompt.size, 24)
    assert np.array_equal(ids, golden_tiny["ids_B"][1:25])
    m.close()


def test_fast_logits_within_tolerance_and_teacher_forced_argmax(tl, oracle, golden_tiny, tiny_payload):
    m = make_model(tl, tiny_payload, tl.FAST)
    mo = oracle.llama2(synth.TINY, tiny_payload)
    forced = golden_tiny["forced_tokens"]
    got = [m.forward(forced[:16], 0, all_logits=True)]
    want = [mo.forward(forced[:16], 0, 1)]
    for i in range(16, 24):
        got.append(m.forward(forced[i:i + 1], i, all_logits=True))
        want.append(mo.forward(forced[i:i + 1], i, 1))
    got, want = np.concatenate(got).astype(np.float32), np.concatenate(want).astype(np.float32)
    err = np.abs(got - want).max()
    assert err <= 2e-2, f"max abs logit error {err} (logits are O(1))"
    # argmax must agree wherever the oracle's top-2 margin exceeds the error actually observed
    s = np.sort(want, axis=1)
    clear = (s[:, -1] - s[:, -2]) > 2 * err
    assert clear.sum() >= 12
    assert np.array_equal(got.argmax(1)[clear], want.argmax(1)[clear])
    m.close()


def test_fast_generate_graph_and_host_loop_agree(tl, golden_tiny, tiny_payload):
    """generate() (id round-trips through the host every step, like the reference) and
    decode_device() (CUDA-graph replay, id stays on the device) run the same kernels."""
    m = make_model(tl, tiny_payload, tl.FAST)
    prompt = golden_tiny["prompt"]
    ids, _, _ = m.generate(prompt, 64)
    m2 = make_model(tl, tiny_payload, tl.FAST)
    m2.forward(prompt, 0, all_logits=False)
    ids2 = m2.decode_device(prompt.size, 63)
    assert np.array_equal(ids[1:], ids2)
    ref_ids = golden_tiny["ids_B"][:64]
    match = int(np.argmax(np.concatenate([ids != ref_ids, [True]])))
    print(f"fast numerics: free-running greedy sequence matches the reference for {match}/64 steps")
    assert ids[0] == ref_ids[0]
    m.close(); m2.close()


def test_one_kernel_decode_step_matches_the_graph_of_kernels(tl, oracle, golden_tiny, tiny_payload):
    """one_kernel_decode=1 runs the whole step as one persistent cooperative kernel; same
    arithmetic up to fp32 summation order, so the logits agree within the fast-mode tolerance and
    stay within it against the oracle."""
    a = make_model(tl, tiny_payload, tl.FAST)
    b = tl.Llama2(synth.TINY, numerics=tl.FAST, one_kernel_decode=True)
    b.load_payload(tiny_payload, shared_classifier=True)
    mo = oracle.llama2(synth.TINY, tiny_payload)
    forced = golden_tiny["forced_tokens"]
    for m in (a, b, mo):
        m.forward(forced[:16], 0, *(() if m is not mo else (1,)))
    for i in range(16, 24):
        la = a.forward(forced[i:i + 1], i, all_logits=True).astype(np.float32)
        lb = b.forward(forced[i:i + 1], i, all_logits=True).astype(np.float32)
        lo = mo.forward(forced[i:i + 1], i, 1).astype(np.float32)
        assert np.abs(la - lb).max() <= 1e-2
        assert np.abs(lb - lo).max() <= 2e-2
    b.forward(forced[:16], 0, all_logits=False)
    ids = b.decode_device(16, 20)
    assert ids.shape == (20,) and tl.device_status() == 0
    a.close(); b.close()


def test_context_limits(tl, tiny_payload):
    m = make_model(tl, tiny_payload, tl.FAST)
    tok = synth.token_ids(5, 1, 256, synth.TINY.vocab_size)
    out = m.forward(tok, 0, all_logits=False)            # a prompt that fills the whole context
    assert out.shape == (1, synth.TINY.vocab_size) and np.isfinite(out.astype(np.float32)).all()
    with pytest.raises(tl.TLError):
        m.forward(tok[:2], 255)                          # would run past max_seq_len
    with pytest.raises(tl.TLError):
        m.forward(np.array([32000], dtype=np.int32), 0)  # id outside the vocabulary
    m.close()


def test_checkpoint_file_loader(tl, tmp_path, golden_tiny, tiny_payload):
    path = str(tmp_path / "tiny.bin")
    with open(path, "wb") as f:
        f.write(synth.TINY.header())
        tiny_payload.tofile(f)
    m = tl.Llama2(synth.TINY, numerics=tl.REFERENCE_ORDER)
    m.load_file(path)
    lg = m.forward(golden_tiny["prompt"], 0, all_logits=False)
    assert_bit_equal(lg[0], golden_tiny["logits_B"][0], "logits after loading from a file")
    with pytest.raises(tl.TLError):
        m.load_file(str(tmp_path / "missing.bin"))
    # a truncated file is refused before anything is uploaded: the weights stay as loaded
    short = str(tmp_path / "short.bin")
    with open(short, "wb") as f:
        f.write(synth.TINY.header())
        tiny_payload[: tiny_payload.size // 2].tofile(f)
    with pytest.raises(tl.TLError, match="truncated"):
        m.load_file(short)
    assert_bit_equal(m.forward(golden_tiny["prompt"], 0, all_logits=False)[0], golden_tiny["logits_B"][0], "after refusal")
    m.close()


def test_checkpoint_file_loader_untied_classifier_streams_in_chunks(tl, tmp_path):
    """Untied checkpoint (negative vocab in the header, RoPE block before wcls, main.cpp:160-190) with an
    embedding larger than one 64 MB staging chunk; file and in-memory loads must give the same logits."""
    cfg = synth.LlamaConfig(dim=1024, hidden_dim=2816, n_layers=1, n_heads=8, vocab_size=40000, seq_len=64,
                            shared_classifier=False)
    payload = synth.llama2c_payload(cfg, 99)
    path = str(tmp_path / "untied.bin")
    with open(path, "wb") as f:
        f.write(cfg.header())
        payload.tofile(f)
    tokens = synth.token_ids(99, 3, 24, cfg.vocab_size)
    a = tl.Llama2(cfg, numerics=tl.FAST)
    a.load_file(path)
    b = tl.Llama2(cfg, numerics=tl.FAST)
    b.load_payload(payload, shared_classifier=False)
    assert_bit_equal(a.forward(tokens, 0, all_logits=True), b.forward(tokens, 0, all_logits=True), "file vs memory")
    a.close(); b.close()


# head_dim 128 and 32-column-aligned widths: the shapes that take the fused prefill path
# (matmul epilogues with RoPE / KV write / residual / SiLU*up, attention in one kernel)
MID = synth.LlamaConfig(dim=512, hidden_dim=1408, n_layers=2, n_heads=4, vocab_size=1000, seq_len=384)


@pytest.mark.parametrize("T,tail", [(200, 3), (20, 2), (300, 2)])
def test_fast_fused_prefill_matches_oracle_at_head_dim_128(tl, oracle, T, tail):
    payload = synth.llama2c_payload(MID, 777)
    tokens = synth.token_ids(777, 5, T + tail, MID.vocab_size)
    m = tl.Llama2(MID, numerics=tl.FAST)
    m.load_payload(payload, shared_classifier=True)
    mo = oracle.llama2(MID, payload)
    got = [m.forward(tokens[:T], 0, all_logits=True)]
    want = [mo.forward(tokens[:T], 0, 1)]
    # a chunked continuation (start_pos > 0, T > 1) and single-token decode steps over the same cache
    got.append(m.forward(tokens[T:T + tail - 1], T, all_logits=True) if tail > 2 else np.zeros((0, MID.vocab_size), np.float16))
    want.append(mo.forward(tokens[T:T + tail - 1], T, 1) if tail > 2 else np.zeros((0, MID.vocab_size), np.float16))
    p = T + (tail - 1 if tail > 2 else 0)
    while p < T + tail:
        got.append(m.forward(tokens[p:p + 1], p, all_logits=True))
        want.append(mo.forward(tokens[p:p + 1], p, 1))
        p += 1
    got, want = np.concatenate(got).astype(np.float32), np.concatenate(want).astype(np.float32)
    assert tl.device_status() == 0
    err = np.abs(got - want).max()
    assert err <= 2e-2, f"max abs logit error {err} (logits are O(1))"
    s = np.sort(want, axis=1)
    clear = (s[:, -1] - s[:, -2]) > 2 * err
    assert np.array_equal(got.argmax(1)[clear], want.argmax(1)[clear])
    m.close()


_FUSED_CHILD = r"""
import sys, numpy as np
sys.path.insert(0, sys.argv[1])
import tensorlib_b200 as tl
from tensorlib_b200 import synth
tl.init(0)
MID = synth.LlamaConfig(dim=512, hidden_dim=1408, n_layers=2, n_heads=4, vocab_size=1000, seq_len=384)
m = tl.Llama2(MID, numerics=tl.FAST)
m.load_payload(synth.llama2c_payload(MID, 777), shared_classifier=True)
tokens = synth.token_ids(777, 5, 300, MID.vocab_size)
out = [m.forward(tokens, 0, all_logits=True) for _ in range(2)]     # twice: counters of the stream-K mode reset
assert tl.device_status() == 0
assert np.array_equal(out[0], out[1])
np.save(sys.argv[2], out[1])
"""


@pytest.mark.parametrize("mode", ["never", "always", "always512", "streamk", "streamk512"])
def test_fused_prefill_epilogues_under_every_hgemm_kernel(tl, oracle, tmp_path, mode):
    """The fused matmul epilogues of the prefill (RoPE + KV write, residual, SiLU*up) through the
    single-CTA kernel, the CTA-pair kernel with 256- and 512-row tiles, and both with stream-K ranges
    (partial tiles summed by the last arriver): all against the oracle's logits."""
    import subprocess, sys as _sys
    script, out = tmp_path / "child.py", tmp_path / "logits.npy"
    script.write_text(_FUSED_CHILD)
    root = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
    r = subprocess.run([_sys.executable, str(script), root, str(out)], capture_output=True, text=True,
                       env=dict(os.environ, TL_HGEMM_PAIR=mode), timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    got = np.load(out).astype(np.float32)
    tokens = synth.token_ids(777, 5, 300, MID.vocab_size)
    want = oracle.llama2(MID, synth.llama2c_payload(MID, 777)).forward(tokens, 0, 1).astype(np.float32)
    err = np.abs(got - want).max()
    assert err <= 2e-2, f"{mode}: max abs logit error {err}"


def test_multi_turn_generation_continues_over_the_kv_cache(tl, golden_tiny, tiny_payload):
    """Two turns (llama2.cpp keeps total_len across generate calls) equal one forward over the
    concatenated token stream, bit for bit in reference-order numerics."""
    m = make_model(tl, tiny_payload, tl.REFERENCE_ORDER)
    prompt = golden_tiny["prompt"]
    ids1, _, _ = m.generate(prompt, 5)
    assert np.array_equal(ids1, golden_tiny["ids_B"][:5])
    turn2 = synth.token_ids(SEED, 77, 4, synth.TINY.vocab_size)
    start = len(prompt) + len(ids1) - 1          # the last sampled id of turn 1 was never fed back
    ids2, _, _ = m.generate(np.concatenate([ids1[-1:], turn2]), 3, start_pos=start)
    whole = np.concatenate([prompt, ids1, turn2])
    m2 = make_model(tl, tiny_payload, tl.REFERENCE_ORDER)
    lg = m2.forward(whole, 0, all_logits=True)
    assert int(lg[-1].astype(np.float32).argmax()) == int(ids2[0])
    with pytest.raises(tl.TLError):
        m.generate(prompt, 8, start_pos=synth.TINY.seq_len - 4)
    m.close(); m2.close()


def test_long_context_decode_agrees_with_prefill_of_the_same_tokens(tl):
    """Context of ~2000 positions at head_dim 128: the decode path (GEMV ring + split attention over
    the in-place caches) must give the logits the fused prefill gives for the same token stream."""
    cfg = synth.LlamaConfig(dim=512, hidden_dim=1408, n_layers=2, n_heads=4, vocab_size=1000, seq_len=2048)
    payload = synth.llama2c_payload(cfg, 4242)
    tokens = synth.token_ids(4242, 9, 2043, cfg.vocab_size)
    a = tl.Llama2(cfg, numerics=tl.FAST)
    a.load_payload(payload, shared_classifier=True)
    a.forward(tokens[:2040], 0, all_logits=False)
    dec = np.concatenate([a.forward(tokens[p:p + 1], p, all_logits=True) for p in range(2040, 2043)]).astype(np.float32)
    ids = a.decode_device(2043, 3)            # graph path up to the last position of the context
    b = tl.Llama2(cfg, numerics=tl.FAST)
    b.load_payload(payload, shared_classifier=True)
    ref = b.forward(tokens, 0, all_logits=True)[2040:2043].astype(np.float32)
    assert tl.device_status() == 0
    assert np.abs(dec - ref).max() <= 2e-2
    assert ids.shape == (3,)
    with pytest.raises(tl.TLError):
        a.decode_device(2046, 3)              # would run past max_seq_len
    a.close(); b.close()


def test_growing_the_shared_rope_table_leaves_a_models_table_valid(tl, golden_tiny, tiny_payload):
    """A model keeps pointers into the cos/sin table of its head size (they are also baked into its
    decode graph). A later call that needs more rows for the same head size allocates a larger
    table; the model must go on reading valid memory and produce the same bits."""
    m = make_model(tl, tiny_payload, tl.FAST)
    prompt = golden_tiny["prompt"]
    before = m.forward(prompt, 0, all_logits=False)
    ids_before = m.decode_device(prompt.size, 12)
    hd = synth.TINY.head_dim
    x = synth.normal_f16(8, 1, 2 * 6 * hd, 1.0).reshape(2, 6, hd)
    for pos in (300, 700, 3000):                          # beyond the 256 rows the model asked for: three regrowths
        tl.apply_rotary_emb(x, pos)
    junk = [tl.DeviceBuffer(256 * (hd // 2) * 2) for _ in range(64)]    # would reuse a freed table's memory
    for j in junk:
        tl.check(tl.load().tl_memset(j.ptr, 0xFF, j.nbytes, None), "memset")
    tl.synchronize()
    after = m.forward(prompt, 0, all_logits=False)
    assert_bit_equal(after, before, "logits after the table grew")
    assert np.array_equal(m.decode_device(prompt.size, 12), ids_before)
    assert tl.device_status() == 0
    m.close()


def test_a_timed_out_device_wait_turns_into_an_error_return_of_the_model_call(tl, golden_tiny, tiny_payload):
    """The model calls that synchronise read the device status word: after a kernel gave up on a
    bounded wait they return TL_ERR_TIMEOUT instead of results, once, and then work again."""
    m = make_model(tl, tiny_payload, tl.FAST)
    prompt = golden_tiny["prompt"]
    good = m.forward(prompt, 0, all_logits=False)
    tl.check(tl.load().tl_selftest_unposted_exchange(256, None), "tl_selftest_unposted_exchange")
    with pytest.raises(tl.TLError) as err:
        m.forward(prompt, 0, all_logits=False)
    assert err.value.status == 6 and "bounded" in str(err.value)
    assert_bit_equal(m.forward(prompt, 0, all_logits=False), good, "next call")
    tl.check(tl.load().tl_selftest_unposted_exchange(256, None), "tl_selftest_unposted_exchange")
    with pytest.raises(tl.TLError) as err:
        m.generate(prompt, 4)
    assert err.value.status == 6
    ids, _, _ = m.generate(prompt, 4)
    assert ids.shape == (4,) and tl.device_status() == 0
    m.close()
