#include "synth_ggjt.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <atomic>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "ggml_file.h"
#include "utils.h"

using namespace std;

namespace {

inline u64 mix64(u64 x) {                 // splitmix64 finaliser
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}

// Box-Muller on the two 24-bit halves of one hash; elements 2k and 2k+1 share a hash.
inline void normal_pair(u64 seed, u32 tensor, u64 pair, float* z0, float* z1) {
    const u64 h = mix64(mix64(seed ^ (u64(tensor) << 40)) + pair);
    const float u1 = (float((h >> 40) & 0xffffffu) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = (float(h & 0xffffffu) + 0.5f) * (1.0f / 16777216.0f);
    const float r = sqrtf(-2.0f * logf(u1));
    const float a = 6.28318530717958647692f * u2;
    *z0 = r * cosf(a);
    *z1 = r * sinf(a);
}

struct tensor_plan {
    string name;
    u32 rows, cols;        // cols == 1 for vectors
    ggml_value_type type;
    u64 header_at, data_at, data_bytes;
};

size_t block_bytes(ggml_value_type t, u32 version = 3) { return t == ggml_value_type::q4_0 ? (version == 1 ? 20 : 18) : 34; }

bool valid(const synth_config& c) {
    return c.dim && c.n_heads && c.n_layers && c.ff_size && c.vocab_size >= 259 && c.dim % c.n_heads == 0 &&
           c.dim % 32 == 0 && c.ff_size % 32 == 0 &&
           (c.wtype == ggml_value_type::q4_0 || c.wtype == ggml_value_type::q8_0) &&
           (c.file_version == 3 || (c.file_version == 1 && c.wtype == ggml_value_type::q4_0));
}

// Token strings: ids 0-2 specials, 3-258 the 256 single bytes (the tokenizer's byte fallback
// is byte + 3), the rest seeded random strings of 2 to 8 lower-case letters and spaces.
vector<ggml_token> make_vocab(const synth_config& c) {
    vector<ggml_token> v(c.vocab_size);
    v[0] = {"<unk>", 0.f};
    v[1] = {"<s>", 0.f};
    v[2] = {"</s>", 0.f};
    for (u32 b = 0; b < 256; ++b) v[3 + b] = {string(1, char(b)), 0.f};
    static const char alphabet[] = "abcdefghijklmnopqrstuvwxyz ";
    for (u32 i = 259; i < c.vocab_size; ++i) {
        u64 h = mix64(c.seed * 0x100000001b3ull + i);
        const u32 len = 2 + u32(h % 7);
        h = mix64(h);
        string s;
        for (u32 k = 0; k < len; ++k) {
            s.push_back(alphabet[h % 27]);
            h = mix64(h);
        }
        v[i] = {s, -10.0f * float(h & 0xffffffu) * (1.0f / 16777216.0f)};
    }
    return v;
}

vector<tensor_plan> make_plan(const synth_config& c, const vector<ggml_token>& vocab, u64* total) {
    vector<tensor_plan> plan;
    u64 at = sizeof(ggml_header);
    for (const auto& t : vocab) at += 4 + t.text.size() + 4;
    auto add = [&](const string& name, u32 rows, u32 cols, ggml_value_type type) {
        tensor_plan p{name, rows, cols, type, at, 0, 0};
        at += 4 * (cols == 1 ? 4 : 5) + name.size();
        at = (at + 31) & ~u64(31);
        p.data_at = at;
        p.data_bytes = type == ggml_value_type::f32 ? u64(rows) * cols * 4 : u64(rows) * cols / 32 * block_bytes(type, c.file_version);
        at += p.data_bytes;
        plan.push_back(p);
    };
    const auto W = c.wtype;
    const auto F = ggml_value_type::f32;
    add("tok_embeddings.weight", c.vocab_size, c.dim, c.f32_embeddings ? F : W);
    add("norm.weight", c.dim, 1, F);
    add("output.weight", c.vocab_size, c.dim, W);
    for (u32 l = 0; l < c.n_layers; ++l) {
        const string p = "layers." + to_string(l) + ".";
        add(p + "attention.wq.weight", c.dim, c.dim, W);
        add(p + "attention.wk.weight", c.dim, c.dim, W);
        add(p + "attention.wv.weight", c.dim, c.dim, W);
        add(p + "attention.wo.weight", c.dim, c.dim, W);
        add(p + "feed_forward.w1.weight", c.ff_size, c.dim, W);
        add(p + "feed_forward.w2.weight", c.dim, c.ff_size, W);
        add(p + "feed_forward.w3.weight", c.ff_size, c.dim, W);
        add(p + "attention_norm.weight", c.dim, 1, F);
        add(p + "ffn_norm.weight", c.dim, 1, F);
    }
    *total = at;
    return plan;
}

}  // namespace

float synth_normal(u64 seed, u32 tensor, u64 element) {
    float z0, z1;
    normal_pair(seed, tensor, element >> 1, &z0, &z1);
    return (element & 1) ? z1 : z0;
}

void synth_quantize_v1(const float* src, size_t count, u8* dst) {
    for (size_t b = 0; b < count / 32; ++b) {
        const float* w = src + b * 32;
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(w[j]));
        const float d = amax / 8.0f;
        const float inv = d > 0.f ? 1.0f / d : 0.f;
        u8* out = dst + b * 20;
        memcpy(out, &d, 4);
        u8 q[32];
        for (int j = 0; j < 32; ++j) q[j] = u8(fminf(15.f, fmaxf(0.f, rintf(w[j] * inv) + 8.f)));
        for (int j = 0; j < 16; ++j) out[4 + j] = u8(q[2 * j] | (q[2 * j + 1] << 4));
    }
}

void synth_quantize(const float* src, size_t count, ggml_value_type wtype, u8* dst) {
    for (size_t b = 0; b < count / 32; ++b) {
        const float* w = src + b * 32;
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(w[j]));
        if (wtype == ggml_value_type::q4_0) {
            const u16 d16 = float_to_half(amax / 8.0f);
            const float d = half_to_float(d16);
            const float inv = d > 0.f ? 1.0f / d : 0.f;
            u8* out = dst + b * 18;
            memcpy(out, &d16, 2);
            u8 q[32];
            for (int j = 0; j < 32; ++j) q[j] = u8(fminf(15.f, fmaxf(0.f, rintf(w[j] * inv) + 8.f)));
            for (int j = 0; j < 16; ++j) out[2 + j] = u8(q[j] | (q[j + 16] << 4));
        } else {
            const u16 d16 = float_to_half(amax / 127.0f);
            const float d = half_to_float(d16);
            const float inv = d > 0.f ? 1.0f / d : 0.f;
            u8* out = dst + b * 34;
            memcpy(out, &d16, 2);
            for (int j = 0; j < 32; ++j) out[2 + j] = u8(int8_t(fminf(127.f, fmaxf(-127.f, rintf(w[j] * inv)))));
        }
    }
}

u64 synth_file_size(const synth_config& cfg) {
    if (!valid(cfg)) return 0;
    u64 total = 0;
    make_plan(cfg, make_vocab(cfg), &total);
    return total;
}

bool synth_write_ggjt(const string& path, const synth_config& cfg, string* error) {
    auto fail = [&](const string& m) {
        if (error) *error = m;
        return false;
    };
    if (!valid(cfg)) return fail("invalid synthetic model configuration");
    const vector<ggml_token> vocab = make_vocab(cfg);
    u64 total = 0;
    const vector<tensor_plan> plan = make_plan(cfg, vocab, &total);

    const int fd = ::open(path.c_str(), O_RDWR | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) return fail("cannot create " + path + ": " + strerror(errno));
    if (::ftruncate(fd, off_t(total)) < 0) {
        ::close(fd);
        return fail("cannot size " + path + ": " + strerror(errno));
    }
    u8* map = static_cast<u8*>(::mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0));
    ::close(fd);
    if (map == MAP_FAILED) return fail("cannot map " + path + ": " + strerror(errno));

    // header, vocabulary and tensor records (ggjt layout: ggml_file.cpp:46-122 of the reference)
    ggml_header h{0x67676a74u, cfg.file_version, cfg.vocab_size, cfg.dim, 256, cfg.n_heads, cfg.n_layers, cfg.dim / cfg.n_heads, u32(cfg.wtype)};
    memcpy(map, &h, sizeof h);
    u64 at = sizeof h;
    for (const auto& t : vocab) {
        const int32_t len = int32_t(t.text.size());
        memcpy(map + at, &len, 4);
        memcpy(map + at + 4, t.text.data(), t.text.size());
        memcpy(map + at + 4 + t.text.size(), &t.score, 4);
        at += 8 + t.text.size();
    }
    for (const auto& p : plan) {
        u8* r = map + p.header_at;
        const u32 n_dims = p.cols == 1 ? 1 : 2, name_len = u32(p.name.size()), type = u32(p.type);
        memcpy(r, &n_dims, 4);
        memcpy(r + 4, &name_len, 4);
        memcpy(r + 8, &type, 4);
        if (n_dims == 1) {
            memcpy(r + 12, &p.rows, 4);
            memcpy(r + 16, p.name.data(), name_len);
        } else {                          // (columns, rows) order
            memcpy(r + 12, &p.cols, 4);
            memcpy(r + 16, &p.rows, 4);
            memcpy(r + 20, p.name.data(), name_len);
        }
    }

    // tensor data: work items of 64 rows, pulled by a pool of threads
    struct item { u32 tensor; u32 row0, row1; };
    vector<item> items;
    for (u32 t = 0; t < plan.size(); ++t) {
        const u32 step = plan[t].cols == 1 ? plan[t].rows : 64;
        for (u32 r0 = 0; r0 < plan[t].rows; r0 += step) items.push_back({t, r0, min(plan[t].rows, r0 + step)});
    }
    atomic<size_t> next{0};
    u32 nthreads = cfg.threads ? cfg.threads : thread::hardware_concurrency();
    if (nthreads == 0) nthreads = 1;
    auto worker = [&]() {
        vector<float> row;
        for (;;) {
            const size_t i = next.fetch_add(1);
            if (i >= items.size()) return;
            const tensor_plan& p = plan[items[i].tensor];
            if (p.type == ggml_value_type::f32 && p.cols != 1) {   // f32 embedding rows: the N(0, 0.02) values themselves
                float* out = reinterpret_cast<float*>(map + p.data_at);
                for (u32 r = items[i].row0; r < items[i].row1; ++r) {
                    const u64 e0 = u64(r) * p.cols;
                    for (u32 k = 0; k < p.cols; k += 2) {
                        float z0, z1;
                        normal_pair(cfg.seed, items[i].tensor, (e0 + k) >> 1, &z0, &z1);
                        out[e0 + k] = 0.02f * z0;
                        out[e0 + k + 1] = 0.02f * z1;
                    }
                }
                continue;
            }
            if (p.type == ggml_value_type::f32) {         // norm vectors: N(1, 0.01)
                float* out = reinterpret_cast<float*>(map + p.data_at);
                for (u32 e = items[i].row0; e < items[i].row1; ++e) out[e] = 1.0f + 0.01f * synth_normal(cfg.seed, items[i].tensor, e);
                continue;
            }
            row.resize(p.cols);
            const size_t rb = size_t(p.cols) / 32 * block_bytes(p.type, cfg.file_version);
            for (u32 r = items[i].row0; r < items[i].row1; ++r) {
                const u64 e0 = u64(r) * p.cols;            // cols is even: pairs never straddle rows
                for (u32 k = 0; k < p.cols; k += 2) {
                    float z0, z1;
                    normal_pair(cfg.seed, items[i].tensor, (e0 + k) >> 1, &z0, &z1);
                    row[k] = 0.02f * z0;
                    row[k + 1] = 0.02f * z1;
                }
                if (cfg.file_version == 1) synth_quantize_v1(row.data(), p.cols, map + p.data_at + size_t(r) * rb);
                else synth_quantize(row.data(), p.cols, p.type, map + p.data_at + size_t(r) * rb);
            }
        }
    };
    vector<thread> pool;
    for (u32 t = 1; t < nthreads; ++t) pool.emplace_back(worker);
    worker();
    for (auto& t : pool) t.join();

    const bool ok = ::msync(map, total, MS_ASYNC) == 0;
    ::munmap(map, total);
    return ok ? true : fail("msync failed");
}
