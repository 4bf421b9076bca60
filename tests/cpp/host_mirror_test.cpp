// Exercises the C++ host mirror (include/tensorlib_b200.hpp) the way the reference's own programs
// use its API: Tensor::matmul with a transposed weight view, nn::Linear::forward with a caller-owned
// result, Transformer::forward, Llama2::generate (model/llama2_7b/src/main.cpp:230-260).
//
//   host_mirror_test nogpu
//       no device: every entry point must refuse loudly (no CPU fallback), argument errors throw
//       std::invalid_argument before touching the device.
//   host_mirror_test gpu <checkpoint.bin> <case.txt>
//       case.txt: dim hidden layers heads vocab seq | n_prompt ids... | n_expected ids... |
//                 M N K | M*K A bits | N*K W bits | M*N expected C bits (reference CPU matmul)
//       prints "OK <what>" lines; exit code 0 only if all checks pass.
//   host_mirror_test chat <checkpoint.bin> <tokenizer.bin> dim hidden layers heads vocab seq
//       Llama2::chat over two lines of input against a replay of the same turns through generate_at:
//       the second turn must continue at the first turn's end position (the reference's total_len).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>

#include "tensorlib_b200.hpp"

using namespace tlb200;

static float half_to_float(uint16_t h) {
    const uint32_t s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023;
    if (e == 0) return (s ? -1.f : 1.f) * std::ldexp((float)m, -24);
    if (e == 31) return m ? NAN : (s ? -INFINITY : INFINITY);
    return (s ? -1.f : 1.f) * std::ldexp((float)(m | 1024), (int)e - 25);
}

static int run_nogpu() {
    int failures = 0;
    try { init(0); std::puts("FAIL init succeeded without a device"); failures++; }
    catch (const Error& e) { std::printf("OK init refused: %s\n", e.what()); }
    try { Tensor t({2, 8}); std::puts("FAIL allocation succeeded"); failures++; }
    catch (const Error& e) { std::printf("OK tensor refused (status %d)\n", e.status); }
    try {
        ModelArgs a; a.dim = 64; a.hidden_dim = 128; a.n_layers = 1; a.n_heads = 2; a.vocab_size = 100; a.max_seq_len = 16;
        Transformer m(a);
        std::puts("FAIL model creation succeeded"); failures++;
    } catch (const Error& e) { std::printf("OK model refused (status %d)\n", e.status); }
    return failures;
}

static int run_gpu(const char* ckpt, const char* case_path) {
    int failures = 0;
    std::ifstream in(case_path);
    ModelArgs a;
    in >> a.dim >> a.hidden_dim >> a.n_layers >> a.n_heads >> a.vocab_size >> a.max_seq_len;
    a.n_kv_heads = a.n_heads;
    int n_prompt, n_expected;
    in >> n_prompt;
    std::vector<int> prompt(n_prompt);
    for (int& v : prompt) in >> v;
    in >> n_expected;
    std::vector<int> expected(n_expected);
    for (int& v : expected) in >> v;
    int M, N, K;
    in >> M >> N >> K;
    std::vector<uint16_t> A((size_t)M * K), W((size_t)N * K), want((size_t)M * N);
    for (auto* vec : {&A, &W, &want}) for (uint16_t& v : *vec) { unsigned x; in >> x; v = (uint16_t)x; }
    if (!in) { std::puts("FAIL case file truncated"); return 1; }

    init(0);
    // Tensor::matmul + nn::Linear, fast numerics within 1e-2 and reference-order numerics bit-exact
    Tensor x({1, M, K}, A.data());
    nn::Linear lin(K, N, Tensor({N, K}, W.data()));
    Tensor out({1, M, N});
    Tensor y = lin.forward(x, out);                                       // caller-owned result
    if (y.data() != out.data()) { std::puts("FAIL result_opt not used"); failures++; }
    std::vector<uint16_t> got = y.to_host();
    double worst = 0, scale = 0;
    for (uint16_t v : want) scale += (double)half_to_float(v) * half_to_float(v);
    scale = std::sqrt(scale / want.size());
    for (size_t i = 0; i < got.size(); i++) {
        const double g = half_to_float(got[i]), w = half_to_float(want[i]);
        worst = std::max(worst, std::fabs(g - w) / std::max(std::fabs(w), scale));
    }
    if (worst <= 1e-2) std::printf("OK linear fast numerics, max rel err %.3g\n", worst);
    else { std::printf("FAIL linear fast numerics, max rel err %.3g\n", worst); failures++; }
    std::vector<uint16_t> exact = x.matmul(lin.weight.transpose(), std::nullopt, TL_NUMERICS_REFERENCE_ORDER).to_host();
    if (exact == want) std::puts("OK matmul reference-order numerics bit-identical");
    else { std::puts("FAIL matmul reference-order numerics differ"); failures++; }
    try { x.matmul(lin.weight); std::puts("FAIL untransposed weight accepted"); failures++; }
    catch (const std::invalid_argument&) { std::puts("OK untransposed weight rejected (std::invalid_argument)"); }
    try { Tensor bad({1, M, K + 8}); bad.matmul(lin.weight.transpose()); std::puts("FAIL shape mismatch accepted"); failures++; }
    catch (const std::invalid_argument&) { std::puts("OK inner-dimension mismatch rejected (std::invalid_argument)"); }

    // Llama2::generate in reference-order numerics: the greedy ids of the reference CPU run
    Llama2 llm(a, ckpt, TL_NUMERICS_REFERENCE_ORDER);
    GenerateResult r = llm.generate(prompt, n_expected, /*stop_on_eos=*/false);
    if (r.tokens == expected) std::printf("OK generate: %d greedy ids identical\n", n_expected);
    else { std::puts("FAIL generate: ids differ"); failures++; }
    // Transformer::forward: all-position logits, argmax of the last row is the first generated id
    std::vector<uint16_t> logits = llm.model.forward(prompt, 0);
    const uint16_t* last = logits.data() + (size_t)(n_prompt - 1) * a.vocab_size;
    int best = 0;
    for (int j = 1; j < a.vocab_size; j++) if (half_to_float(last[j]) > half_to_float(last[best])) best = j;
    if (best == expected[0]) std::puts("OK forward: last-position argmax is the first generated id");
    else { std::puts("FAIL forward argmax"); failures++; }
    try { llm.model.forward(prompt, a.max_seq_len); std::puts("FAIL context overflow accepted"); failures++; }
    catch (const std::invalid_argument&) { std::puts("OK context overflow rejected"); }
    return failures;
}

// tokenizer <tokenizer.bin> <cases.txt>: cases.txt holds, per case,
//   bos eos n_text_bytes bytes... n_ids ids... n_dec {prev tok n_bytes bytes...}...
// with the ids / pieces the reference's own Tokenizer produced (tests/golden/tokenizer_cases.json)
static int run_tokenizer(const char* vocab_path, const char* cases_path) {
    std::ifstream in(cases_path);
    int vocab_size = 0, n_cases = 0, failures = 0;
    in >> vocab_size >> n_cases;
    Tokenizer tok(vocab_path, vocab_size);
    for (int c = 0; c < n_cases; c++) {
        int bos, eos, nb, ni, nd;
        in >> bos >> eos >> nb;
        std::string text((size_t)nb, '\0');
        for (int i = 0; i < nb; i++) { int v; in >> v; text[(size_t)i] = (char)v; }
        in >> ni;
        std::vector<int> want((size_t)ni);
        for (int& v : want) in >> v;
        const std::vector<int> got = tok.encode(text, bos != 0, eos != 0);
        if (got != want) { std::printf("FAIL encode case %d\n", c); failures++; }
        in >> nd;
        for (int d = 0; d < nd; d++) {
            int prev, t, len;
            in >> prev >> t >> len;
            std::string piece((size_t)len, '\0');
            for (int i = 0; i < len; i++) { int v; in >> v; piece[(size_t)i] = (char)v; }
            if (tok.decode(prev, t) != piece) { std::printf("FAIL decode case %d token %d\n", c, t); failures++; }
        }
    }
    if (!in) { std::puts("FAIL cases file truncated"); return 1; }
    // decode must not change later encodes (the reference edits its vocabulary in place)
    const std::vector<int> before = tok.encode(" the", true, false);
    for (int t : before) tok.decode(1, t);
    if (tok.encode(" the", true, false) != before) { std::puts("FAIL decode changed the vocabulary"); failures++; }
    if (!tok.encode("", false, false).empty()) { std::puts("FAIL empty text"); failures++; }
    if (!failures) std::printf("OK tokenizer: %d cases identical to the reference\n", n_cases);
    return failures;
}

static int run_chat(int argc, char** argv) {
    int failures = 0;
    ModelArgs a;
    a.dim = std::atoi(argv[4]); a.hidden_dim = std::atoi(argv[5]); a.n_layers = std::atoi(argv[6]); a.n_heads = std::atoi(argv[7]);
    a.vocab_size = std::atoi(argv[8]); a.max_seq_len = std::atoi(argv[9]); a.n_kv_heads = a.n_heads;
    init(0);
    Tokenizer tok(argv[3], a.vocab_size);
    const int max_new = 12;
    const std::string turns[2] = {"the cat sat", "and then"};
    Llama2 llm(a, argv[2], TL_NUMERICS_REFERENCE_ORDER);
    std::istringstream in(turns[0] + "\n" + turns[1] + "\n");
    std::ostringstream out;
    const int answered = llm.chat(tok, in, out, max_new);
    // the same two turns by hand on a second model: positions carry over from turn to turn
    Llama2 replay(a, argv[2], TL_NUMERICS_REFERENCE_ORDER);
    std::string want;
    int pos = 0;
    for (int t = 0; t < 2; t++) {
        const std::vector<int> ids = tok.encode("[INST] " + turns[t] + " [/INST]", true, false);
        const GenerateResult r = replay.generate_at(pos, ids, max_new, true);
        pos += (int)ids.size() + (int)r.tokens.size() - 1;
        want += "> ";
        for (int id : r.tokens) { if (id == 1 || id == 2) break; want += tok.decode(-1, id); }
        want += "\n";
    }
    want += "> ";
    if (answered == 2 && out.str() == want) std::puts("OK chat: two turns, output identical to the replay through generate_at");
    else { std::printf("FAIL chat: answered %d turns, output differs\n", answered); failures++; }
    if (llm.total_len() == pos) std::printf("OK chat: running position %d = prompts + decode steps of both turns\n", pos);
    else { std::printf("FAIL chat: running position %d, expected %d\n", llm.total_len(), pos); failures++; }
    try { llm.generate_at(a.max_seq_len - 2, tok.encode("the", true, false), 8, true); std::puts("FAIL turn beyond the context accepted"); failures++; }
    catch (const std::invalid_argument&) { std::puts("OK chat: a turn beyond the context is rejected"); }
    return failures;
}

int main(int argc, char** argv) {
    try {
        if (argc >= 10 && !std::strcmp(argv[1], "chat")) return run_chat(argc, argv) ? 1 : 0;
        if (argc >= 4 && !std::strcmp(argv[1], "tokenizer")) return run_tokenizer(argv[2], argv[3]) ? 1 : 0;
        if (argc >= 2 && !std::strcmp(argv[1], "nogpu")) return run_nogpu() ? 1 : 0;
        if (argc >= 4 && !std::strcmp(argv[1], "gpu")) return run_gpu(argv[2], argv[3]) ? 1 : 0;
    } catch (const std::exception& e) {
        std::printf("FAIL unexpected exception: %s\n", e.what());
        return 1;
    }
    std::puts("usage: host_mirror_test nogpu | gpu <checkpoint> <case> | tokenizer <tokenizer.bin> <cases> | chat <checkpoint> <tokenizer.bin> dim hidden layers heads vocab seq");
    return 2;
}
