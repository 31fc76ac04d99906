#include "ggml_file.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <iostream>
#include <queue>

#include "utils.h"

using namespace std;

ggml_data_descriptor::ggml_data_descriptor(string _name, ggml_value_type _ftype, u32 _model_version, size_t _offset,
                                           u32 _shape1, u32 _shape2)
    : name(std::move(_name)), ftype(_ftype), model_version(_model_version), offset(_offset), shape1(_shape1),
      shape2(_shape2), size(size_in_file(_ftype, _model_version, u64(_shape1) * _shape2)) {}

// Bytes of a tensor in the file (ggml_file.cpp:162-186 of the reference): f32 4 B and
// f16 2 B per element; quantised blocks of 32 elements take 20/36 B (f32 scale) in
// version-1 files and 18/34 B (f16 scale) otherwise.
size_t ggml_data_descriptor::size_in_file(ggml_value_type ftype, u32 model_version, u64 elements) {
    switch (ftype) {
        case ggml_value_type::f32: return elements * 4;
        case ggml_value_type::f16: return elements * 2;
        case ggml_value_type::q4_0: return elements % 32 ? 0 : elements / 32 * (model_version == 1 ? 20 : 18);
        case ggml_value_type::q8_0: return elements % 32 ? 0 : elements / 32 * (model_version == 1 ? 36 : 34);
        default: return 0;
    }
}

ggml_file::ggml_file(const char* filepath) {
    const int fd = ::open(filepath, O_RDONLY);
    if (fd < 0) {
        error_text = string("Cannot open ") + filepath + ": " + strerror(errno);
        cerr << error_text << endl;
        return;
    }
    struct stat st {};
    if (::fstat(fd, &st) < 0 || st.st_size <= 0) {
        error_text = string("Cannot stat ") + filepath;
        cerr << error_text << endl;
        ::close(fd);
        return;
    }
    mapping_size = static_cast<size_t>(st.st_size);
    void* m = ::mmap(nullptr, mapping_size, PROT_READ, MAP_SHARED, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) {
        error_text = string("Cannot mmap ") + filepath + ": " + strerror(errno);
        cerr << error_text << endl;
        mapping_size = 0;
        return;
    }
    mapping = static_cast<u8*>(m);
    if (!parse()) {
        cerr << "Bad model file " << filepath << ": " << error_text << endl;
        close_mapping();
    }
}

ggml_file::~ggml_file() { close_mapping(); }

void ggml_file::close_mapping() {
    if (mapping) ::munmap(mapping, mapping_size);
    mapping = nullptr;
    mapping_size = 0;
}

namespace {
// Bounds-checked little-endian reader over the mapping.
struct reader {
    const u8* base;
    size_t size, at;
    template <class T> bool get(T* out) {
        if (at + sizeof(T) > size) return false;
        memcpy(out, base + at, sizeof(T));
        at += sizeof(T);
        return true;
    }
};
}  // namespace

bool ggml_file::parse() {
    reader r{mapping, mapping_size, 0};
    if (!r.get(&header)) { error_text = "file shorter than its header"; return false; }
    if (header.magic != 0x67676a74u) { error_text = "not a ggjt file"; return false; }     // ggml_file.cpp:49
    if (!header.vocab_size || !header.n_heads || !header.n_layers || header.rot * header.n_heads != header.dim) {
        error_text = "inconsistent header";                                                 // ggml_file.cpp:50-53
        return false;
    }
    tokens.reserve(header.vocab_size);
    for (u32 i = 0; i < header.vocab_size; ++i) {                                           // ggml_file.cpp:67-77
        int32_t len;
        if (!r.get(&len) || len < 0 || r.at + size_t(len) + 4 > r.size) { error_text = "truncated vocabulary"; return false; }
        ggml_token& t = tokens.emplace_back();
        t.text.assign(reinterpret_cast<const char*>(mapping + r.at), size_t(len));
        r.at += size_t(len);
        r.get(&t.score);
        text_to_id.emplace(t.text, i);           // keeps the lowest id of duplicate strings
    }
    while (r.at != r.size) {                                                                // ggml_file.cpp:79-122
        const size_t record_at = r.at;
        u32 n_dims, name_len, ftype, shape1, shape2 = 1;
        if (!r.get(&n_dims) || !r.get(&name_len) || !r.get(&ftype) || !r.get(&shape1) || n_dims < 1 || n_dims > 2) {
            error_text = "bad tensor record at offset " + to_string(record_at);
            return false;
        }
        if (n_dims == 2) {               // the file stores (columns, rows)
            shape2 = shape1;
            if (!r.get(&shape1)) { error_text = "truncated tensor record"; return false; }
        }
        if (r.at + name_len > r.size) { error_text = "truncated tensor name"; return false; }
        string name(reinterpret_cast<const char*>(mapping + r.at), name_len);
        r.at += name_len;
        if (name.find('\0') != string::npos) { error_text = "NUL inside a tensor name"; return false; }
        if (!(ftype <= 3 || ftype == 8)) {                                                  // ggml_file.cpp:104-115
            const char* tn = ftype_name(static_cast<ggml_value_type>(ftype));
            error_text = "unsupported type " + (tn ? string(tn) : to_string(ftype)) + " for table " + name;
            return false;
        }
        const size_t offset = (r.at + 31) & ~size_t(31);                                    // ggml_file.cpp:117-118
        ggml_data_descriptor d(name, static_cast<ggml_value_type>(ftype), header.file_version, offset, shape1, shape2);
        if ((d.size == 0 && u64(shape1) * shape2 != 0) || offset + d.size > r.size) {
            error_text = "tensor " + name + " does not fit in the file";
            return false;
        }
        if (!name_to_index.emplace(name, u32(tables.size())).second) { error_text = "duplicate tensor " + name; return false; }
        tables.push_back(std::move(d));
        r.at = offset + tables.back().size;
    }
    const ggml_data_descriptor* w1 = find_buffer_descriptor("layers.0.feed_forward.w1");    // ggml_file.cpp:64
    if (!w1) { error_text = "layers.0.feed_forward.w1 missing"; return false; }
    ff_size = w1->shape1;
    return true;
}

void ggml_file::print_info() const {                                                        // ggml_file.cpp:132-145
    const u32 magic_copy[2] = {header.magic, 0};
    cout << "       magic: " << reinterpret_cast<const char*>(magic_copy) << "\n"
         << "file_version: " << header.file_version << "\n"
         << "  vocab_size: " << header.vocab_size << "\n"
         << "         dim: " << header.dim << "\n"
         << " multiple_of: " << header.multiple_of << "\n"
         << "     n_heads: " << header.n_heads << "\n"
         << "    n_layers: " << header.n_layers << "\n"
         << "per head dim: " << header.rot << "\n"
         << "       ftype: " << header.ftype << "\n"
         << "fast_forward: " << ff_size << endl;
}

const ggml_data_descriptor* ggml_file::find_buffer_descriptor(const string& s) const {      // ggml_file.cpp:337-344
    auto it = name_to_index.find(s);
    if (it == name_to_index.end()) it = name_to_index.find(s + ".weight");
    return it == name_to_index.end() ? nullptr : &tables[it->second];
}

const ggml_data_descriptor& ggml_file::get_buffer_descriptor(const string& s) const {
    const ggml_data_descriptor* d = find_buffer_descriptor(s);
    if (!d) {
        cerr << "[!] tensor " << s << " not found in the model file" << endl;
        abort();
    }
    return *d;
}

string ggml_file::tokens_to_text(const u32* ids, u32 count) const {                         // ggml_file.cpp:346-357
    string res;
    for (u32 j = 0; j < count; ++j) res += tokens.at(ids[j]).text;
    return res;
}

// ---- tokenizer ----------------------------------------------------------------------------
// Greedy bigram merging as in the reference (ggml_file.cpp:188-335): the text is cut into
// UTF-8 characters, every adjacent pair whose concatenation is a vocabulary entry is queued
// with that entry's score, the best pair (highest score, then leftmost) is merged and its new
// neighbours are queued, until nothing is left; pieces that are no vocabulary entry fall back
// to one token per byte (byte + 3).  The reference finds entries by a linear scan that returns
// the first match; the hash map built at load time returns the same id.
namespace {
struct piece {
    int prev, next;
    size_t at, n;          // byte range in the text; n == 0 once merged away
};
struct candidate {
    int left, right;
    float score;
    size_t size;
};
struct worse {
    bool operator()(const candidate& l, const candidate& r) const {
        return l.score < r.score || (l.score == r.score && l.left > r.left);
    }
};
}  // namespace

void ggml_file::tokenize(vector<uint32_t>& output, const string& text, bool bos) const {
    if (text.empty()) return;
    if (bos) output.push_back(1);                                                           // ggml_file.cpp:255-257

    static const size_t utf8_len[16] = {1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 2, 2, 3, 4};
    vector<piece> pieces;
    for (size_t at = 0; at < text.size();) {
        const size_t n = min(text.size() - at, utf8_len[static_cast<u8>(text[at]) >> 4]);
        pieces.push_back({int(pieces.size()) - 1, int(pieces.size()) + 1, at, n});
        at += n;
    }
    pieces.back().next = -1;

    priority_queue<candidate, vector<candidate>, worse> queue;
    string key;
    auto offer = [&](int left, int right) {
        if (left < 0 || right < 0) return;
        const size_t n = pieces[left].n + pieces[right].n;
        key.assign(text, pieces[left].at, n);
        const auto it = text_to_id.find(key);
        if (it != text_to_id.end()) queue.push({left, right, tokens[it->second].score, n});
    };
    for (int i = 1; i < int(pieces.size()); ++i) offer(i - 1, i);

    while (!queue.empty()) {
        const candidate c = queue.top();
        queue.pop();
        piece& l = pieces[c.left];
        piece& r = pieces[c.right];
        if (l.n == 0 || r.n == 0 || l.n + r.n != c.size) continue;      // one side was merged meanwhile
        l.n += r.n;
        r.n = 0;
        l.next = r.next;
        if (r.next >= 0) pieces[r.next].prev = c.left;
        offer(l.prev, c.left);
        offer(c.left, l.next);
    }

    for (int i = 0; i != -1; i = pieces[i].next) {
        key.assign(text, pieces[i].at, pieces[i].n);
        const auto it = text_to_id.find(key);
        if (it != text_to_id.end()) {
            output.push_back(it->second);
        } else {
            for (size_t j = 0; j < pieces[i].n; ++j) output.push_back(u32(static_cast<u8>(text[pieces[i].at + j])) + 3);   // :330
        }
    }
}
