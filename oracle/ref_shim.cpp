/*
 * C wrapper around the reference's own, unmodified ggml_file.cpp + utils.cpp
 * (compiled from the reference checkout where it lies; nothing is copied).
 * TEST INFRASTRUCTURE ONLY: used to validate the oracle's and the product's
 * ggjt parser and tokenizer and to generate the fixtures in tests/golden/.
 *
 * ggml_file keeps its header and mapping private but befriends
 * `llava_context` (ggml_file.h:45); this file defines a class of that name
 * to read them without touching the reference sources.
 *
 * The reference's classes share their names with the product's host classes,
 * so this library is built with hidden visibility and -Bsymbolic: only the
 * ref_* functions are exported and its internal calls can never be
 * interposed by (or interpose) another library in the same process.
 */
#include "ggml_file.h"
#include <cstring>

class llava_context {
public:
    static const ggml_header& header(const ggml_file& f) { return f.header; }
    static u32 ff_size(const ggml_file& f) { return f.ff_size; }
    static const std::vector<ggml_data_descriptor>& tables(const ggml_file& f) { return f.tables; }
    static bool is_open(const ggml_file& f) { return f.is_open(); }
};

#define REF_API __attribute__((visibility("default")))

extern "C" {

REF_API void* ref_open(const char* path) {
    auto* f = new ggml_file(path);
    if (!llava_context::is_open(*f)) { delete f; return nullptr; }
    return f;
}

REF_API void ref_close(void* h) { delete static_cast<ggml_file*>(h); }

/* out[0..8] = the nine header words (ggml_file.h:12-22), out[9] = ff_size */
REF_API void ref_header(void* h, uint32_t* out) {
    auto& f = *static_cast<ggml_file*>(h);
    std::memcpy(out, &llava_context::header(f), 36);
    out[9] = llava_context::ff_size(f);
}

REF_API uint32_t ref_n_tensors(void* h) { return (uint32_t)llava_context::tables(*static_cast<ggml_file*>(h)).size(); }

REF_API int ref_tensor(void* h, uint32_t i, char* name, size_t cap, uint32_t* type, uint64_t* offset,
               uint32_t* shape1, uint32_t* shape2, uint64_t* size) {
    auto& t = llava_context::tables(*static_cast<ggml_file*>(h));
    if (i >= t.size()) return -1;
    std::strncpy(name, t[i].name.c_str(), cap - 1);
    name[cap - 1] = 0;
    *type = (uint32_t)t[i].ftype; *offset = t[i].offset; *shape1 = t[i].shape1; *shape2 = t[i].shape2;
    *size = t[i].size;
    return 0;
}

/* get_buffer_descriptor (ggml_file.cpp:337-344); returns the table offset */
REF_API uint64_t ref_lookup_offset(void* h, const char* name) {
    return static_cast<ggml_file*>(h)->get_buffer_descriptor(name).offset;
}

REF_API uint32_t ref_tokenize(void* h, const char* text, size_t len, int bos, uint32_t* out, uint32_t cap) {
    std::vector<uint32_t> v;
    static_cast<ggml_file*>(h)->tokenize(v, std::string(text, len), bos != 0);
    for (uint32_t i = 0; i < v.size() && i < cap; i++) out[i] = v[i];
    return (uint32_t)v.size();
}

REF_API uint32_t ref_tokens_to_text(void* h, const uint32_t* toks, uint32_t n, char* out, uint32_t cap) {
    std::string s = static_cast<ggml_file*>(h)->tokens_to_text(toks, n);
    uint32_t m = (uint32_t)s.size() < cap ? (uint32_t)s.size() : cap;
    std::memcpy(out, s.data(), m);
    return (uint32_t)s.size();
}

REF_API uint32_t ref_token(void* h, uint32_t id, char* out, uint32_t cap, float* score) {
    auto& t = static_cast<ggml_file*>(h)->get_tokens().at(id);
    uint32_t m = (uint32_t)t.text.size() < cap ? (uint32_t)t.text.size() : cap;
    std::memcpy(out, t.text.data(), m);
    *score = t.score;
    return (uint32_t)t.text.size();
}

}
