// TEST INFRASTRUCTURE — pointer-in/out wrappers around the reference's own Tokenizer
// (model/llama2_7b/src/Tokenizer.cpp, compiled unmodified next to this file by `make ref_tok`).
// Used only by tests/golden/make_tokenizer_golden.py to generate the committed fixture.
#include <cstring>
#include <string>
#include <vector>

#include "Tokenizer.hpp"

extern "C" {

void* reftok_create(const char* path, int vocab_size) {
    try { return new Tokenizer(path, vocab_size); } catch (...) { return nullptr; }
}
void reftok_destroy(void* t) { delete static_cast<Tokenizer*>(t); }
// returns the number of ids (written up to cap)
int reftok_encode(void* t, const char* text, int bos, int eos, int* out, int cap) {
    std::vector<int> ids = static_cast<Tokenizer*>(t)->encode(text, bos != 0, eos != 0);
    for (size_t i = 0; i < ids.size() && (int)i < cap; i++) out[i] = ids[i];
    return (int)ids.size();
}
// returns the byte length of the decoded piece (written up to cap, not NUL-terminated)
int reftok_decode(void* t, int prev, int token, char* out, int cap) {
    std::string s = static_cast<Tokenizer*>(t)->decode(prev, token);
    memcpy(out, s.data(), std::min<size_t>(s.size(), (size_t)cap));
    return (int)s.size();
}

}  // extern "C"
