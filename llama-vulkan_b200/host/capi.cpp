// C wrappers declared in include/llava_host.h.
#include "../../include/llava_host.h"

#include <cstring>
#include <string>
#include <vector>

#include "ggml_file.h"
#include "llava_buffer.h"
#include "llava_context.h"
#include "llava_layer_session_data.h"
#include "llava_session.h"
#include <chrono>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>

#include "llava_session_group.h"
#include "server/session_wrapper.h"
#include "server/tlv_server.h"
#include "synth_ggjt.h"
#include "tp_shard.h"

namespace {
synth_config make_cfg(uint32_t dim, uint32_t n_heads, uint32_t n_layers, uint32_t ff, uint32_t vocab, int wtype) {
    synth_config c;
    c.dim = dim; c.n_heads = n_heads; c.n_layers = n_layers; c.ff_size = ff; c.vocab_size = vocab;
    c.wtype = static_cast<ggml_value_type>(wtype);
    return c;
}
ggml_file* F(void* p) { return static_cast<ggml_file*>(p); }
llava_session* S(void* p) { return static_cast<llava_session*>(p); }
uint32_t copy_out(const std::string& s, char* out, uint32_t cap) {
    if (out && cap) std::memcpy(out, s.data(), s.size() < cap ? s.size() : cap);
    return uint32_t(s.size());
}
}  // namespace

extern "C" {

int llava_synth_write(const char* path, uint32_t dim, uint32_t n_heads, uint32_t n_layers, uint32_t ff, uint32_t vocab,
                      int wtype, uint64_t seed, uint32_t threads) {
    synth_config c = make_cfg(dim, n_heads, n_layers, ff, vocab, wtype);
    c.seed = seed;
    c.threads = threads;
    std::string err;
    return synth_write_ggjt(path, c, &err) ? 1 : 0;
}

int llava_synth_write_ex(const char* path, uint32_t dim, uint32_t n_heads, uint32_t n_layers, uint32_t ff, uint32_t vocab,
                         int wtype, uint64_t seed, uint32_t threads, uint32_t file_version, int f32_embeddings) {
    synth_config c = make_cfg(dim, n_heads, n_layers, ff, vocab, wtype);
    c.seed = seed;
    c.threads = threads;
    c.file_version = file_version;
    c.f32_embeddings = f32_embeddings != 0;
    std::string err;
    return synth_write_ggjt(path, c, &err) ? 1 : 0;
}

void llava_synth_quantize_v1(const float* src, size_t count, uint8_t* dst) { synth_quantize_v1(src, count, dst); }

uint64_t llava_synth_file_size(uint32_t dim, uint32_t n_heads, uint32_t n_layers, uint32_t ff, uint32_t vocab, int wtype) {
    return synth_file_size(make_cfg(dim, n_heads, n_layers, ff, vocab, wtype));
}

float llava_synth_normal(uint64_t seed, uint32_t tensor, uint64_t element) { return synth_normal(seed, tensor, element); }

void llava_synth_quantize(const float* src, size_t count, int wtype, uint8_t* dst) {
    synth_quantize(src, count, static_cast<ggml_value_type>(wtype), dst);
}

void* ggml_file_open(const char* path) {
    auto* f = new ggml_file(path);
    if (!f->is_open()) {
        delete f;
        return nullptr;
    }
    return f;
}

void ggml_file_close(void* file) { delete F(file); }

void ggml_file_header(void* file, uint32_t* out10) {
    std::memcpy(out10, &F(file)->get_header(), sizeof(ggml_header));
    out10[9] = F(file)->get_ff_size();
}

uint32_t ggml_file_n_tensors(void* file) { return uint32_t(F(file)->get_tables().size()); }

int ggml_file_tensor(void* file, uint32_t index, char* name, size_t name_cap, uint32_t* type, uint64_t* offset,
                     uint32_t* shape1, uint32_t* shape2, uint64_t* size) {
    const auto& t = F(file)->get_tables();
    if (index >= t.size()) return 0;
    if (name && name_cap) {
        std::strncpy(name, t[index].name.c_str(), name_cap - 1);
        name[name_cap - 1] = 0;
    }
    if (type) *type = uint32_t(t[index].ftype);
    if (offset) *offset = t[index].offset;
    if (shape1) *shape1 = t[index].shape1;
    if (shape2) *shape2 = t[index].shape2;
    if (size) *size = t[index].size;
    return 1;
}

int ggml_file_find(void* file, const char* name, uint64_t* offset) {
    const ggml_data_descriptor* d = F(file)->find_buffer_descriptor(name);
    if (!d) return 0;
    if (offset) *offset = d->offset;
    return 1;
}

uint32_t ggml_file_tokenize(void* file, const char* text, size_t len, int bos, uint32_t* out, uint32_t cap) {
    std::vector<uint32_t> v;
    F(file)->tokenize(v, std::string(text, len), bos != 0);
    for (uint32_t i = 0; i < v.size() && i < cap; ++i) out[i] = v[i];
    return uint32_t(v.size());
}

uint32_t ggml_file_tokens_to_text(void* file, const uint32_t* tokens, uint32_t n, char* out, uint32_t cap) {
    for (uint32_t i = 0; i < n; ++i) if (tokens[i] >= F(file)->get_tokens().size()) return 0;
    return copy_out(F(file)->tokens_to_text(tokens, n), out, cap);
}

uint32_t ggml_file_token(void* file, uint32_t id, char* out, uint32_t cap, float* score) {
    if (id >= F(file)->get_tokens().size()) return 0;
    const ggml_token& t = F(file)->get_tokens()[id];
    if (score) *score = t.score;
    return copy_out(t.text, out, cap);
}

int llava_dequantize(const void* in, int type, uint32_t model_version, float* out, uint32_t count) {
    return dequantize_to_f32(in, static_cast<ggml_value_type>(type), model_version, out, count) ? 1 : 0;
}

void* llava_context_open(const char* model_path, int device) {
    auto* c = new llava_context();
    if (!c->open(model_path, device)) {
        delete c;
        return nullptr;
    }
    return c;
}

void* llava_context_open_model_only(const char* model_path) {
    auto* c = new llava_context();
    if (!c->open_model_only(model_path)) {
        delete c;
        return nullptr;
    }
    return c;
}

void* llava_context_open_sharded(const char* model_path, int device, uint32_t rank, uint32_t n_ranks, const uint8_t* nccl_id) {
    auto* c = new llava_context();
    if (!c->open_sharded(model_path, device, rank, n_ranks, nccl_id)) {
        delete c;
        return nullptr;
    }
    return c;
}

int llava_context_peer_window_create(void* ctx, uint8_t* handle64) {
    return static_cast<llava_context*>(ctx)->peer_window_create(handle64) ? 1 : 0;
}

int llava_context_peer_connect(void* ctx, const uint8_t* handles) {
    return static_cast<llava_context*>(ctx)->peer_connect(handles) ? 1 : 0;
}

int llava_tp_shape(int type, uint32_t rows, uint32_t cols, uint32_t how, uint32_t rank, uint32_t n_ranks, uint32_t* out_rows,
                   uint32_t* out_cols, uint32_t* out_cols_used, uint64_t* out_bytes) {
    const tp_shard_shape s = tp_shape(static_cast<ggml_value_type>(type), rows, cols, static_cast<tp_split>(how), rank, n_ranks);
    if (!s.valid) return 0;
    *out_rows = s.rows; *out_cols = s.cols; *out_cols_used = s.cols_used; *out_bytes = s.bytes;
    return 1;
}

int llava_tp_pack(const uint8_t* src, int type, uint32_t rows, uint32_t cols, uint32_t how, uint32_t rank, uint32_t n_ranks,
                  uint8_t* dst) {
    return tp_pack(src, static_cast<ggml_value_type>(type), rows, cols, static_cast<tp_split>(how), rank, n_ranks, dst) ? 1 : 0;
}

void llava_context_close(void* ctx) { delete static_cast<llava_context*>(ctx); }
void* llava_context_lv(void* ctx) { return static_cast<llava_context*>(ctx)->lv(); }

int llava_context_run(int argc, char** argv) {
    llava_context c;
    return c.run(argc, argv);
}

void* llava_session_create(void* ctx) { return new llava_session(static_cast<llava_context*>(ctx)); }
void llava_session_destroy(void* session) { delete S(session); }
int llava_session_set_text(void* s, const char* text, size_t len) { return S(s)->set_text(std::string(text, len)) ? 1 : 0; }
int llava_session_add_text(void* s, const char* text, size_t len) { return S(s)->add_text(std::string(text, len)) ? 1 : 0; }
int llava_session_push_token(void* s, uint32_t token) { return S(s)->push_token(token) ? 1 : 0; }
uint32_t llava_session_predict_next_token(void* s) { return S(s)->predict_next_token(); }
int llava_session_start_next_token_prediction(void* s) { return S(s)->start_next_token_prediction() ? 1 : 0; }
uint32_t llava_session_finish_next_token_prediction(void* s) { return S(s)->finish_next_token_prediction(); }
void llava_session_rewind(void* s, uint32_t n) { S(s)->rewind(n); }
uint32_t llava_session_set_options(void* s, uint32_t options) { return uint32_t(S(s)->set_options(options)); }
uint32_t llava_session_save_frame(void* s, const char* path) { return uint32_t(S(s)->save_frame(path)); }
uint32_t llava_session_snapshot(void* s, const char* path) { return uint32_t(S(s)->snapshot(path)); }
uint32_t llava_session_restore(void* s, const char* path) { return uint32_t(S(s)->restore(path)); }
uint32_t llava_session_get_token_count(void* s) { return S(s)->get_token_count(); }

uint32_t llava_session_get_tokens(void* s, uint32_t* out, uint32_t cap) {
    const auto& t = S(s)->get_token_buffer();
    for (uint32_t i = 0; i < t.size() && i < cap; ++i) out[i] = t[i];
    return uint32_t(t.size());
}

void llava_session_set_deterministic(void* s, int on) { S(s)->set_deterministic(on != 0); }
void llava_session_set_seed(void* s, uint32_t seed) { S(s)->set_seed(seed); }
int llava_session_set_max_batch(void* s, uint32_t n) { return S(s)->set_max_batch(n) ? 1 : 0; }

int llava_session_generate_greedy_on_device(void* s, uint32_t n, uint32_t* out) {
    std::vector<uint32_t> v;
    if (!S(s)->generate_greedy_on_device(n, &v)) return 0;
    for (uint32_t i = 0; i < v.size(); ++i) out[i] = v[i];
    return 1;
}

int llava_session_enqueue_greedy_on_device(void* s, uint32_t n) { return S(s)->enqueue_greedy_on_device(n) ? 1 : 0; }

int llava_session_collect_greedy_on_device(void* s, uint32_t* out, uint32_t cap) {
    std::vector<uint32_t> v;
    if (!S(s)->collect_greedy_on_device(&v)) return 0;
    for (uint32_t i = 0; i < v.size() && i < cap; ++i) out[i] = v[i];
    return 1;
}

int llava_session_get_logits(void* s, float* out, uint32_t cap) {
    std::vector<float> v;
    if (!S(s)->get_logits(&v) || v.size() > cap) return 0;
    std::memcpy(out, v.data(), v.size() * sizeof(float));
    return 1;
}

uint32_t llava_session_get_backlog_size(void* s) { return S(s)->get_backlog_size(); }
uint32_t llava_session_get_tokens_in_gpu(void* s) { return S(s)->get_tokens_in_gpu(); }
void llava_session_set_host_sampler(void* s, int on) { S(s)->set_host_sampler(on != 0); }
float llava_session_get_mirostat_mu(void* s) { return S(s)->get_mirostat_mu(); }
uint32_t llava_session_step_kernel_launches(void* s) { return S(s)->step_kernel_launches(); }
int llava_session_set_step_trace(void* s, int on) { return S(s)->set_step_trace(on != 0); }
uint64_t llava_session_read_step_trace(void* s, uint64_t* out, uint64_t cap, uint32_t* dims3) {
    std::vector<u64> v;
    if (!S(s)->read_step_trace(&v, &dims3[0], &dims3[1], &dims3[2])) return 0;
    const uint64_t n = uint64_t(dims3[0]) * dims3[1] * dims3[2];
    if (n > cap) return 0;
    memcpy(out, v.data(), n * 8);
    return n;
}

int llava_session_read_kv(void* s, uint32_t layer, int which, uint32_t row0, uint32_t nrows, uint16_t* out) {
    const auto& data = S(s)->get_layer_data();
    if (layer >= data.size()) return 0;
    llava_buffer* b = which == 0 ? data[layer]->get_k_cache() : data[layer]->get_v_cache();
    const size_t row_bytes = size_t(b->shape.second) * 2;
    return b->read_raw(row0 * row_bytes, out, nrows * row_bytes) ? 1 : 0;
}

// ---- lsrv::session_wrapper behind a collecting owner (what a front end would implement) ----
namespace {
struct collected { int kind; uint32_t who, opcode, request; std::vector<uint8_t> payload; };
class collecting_owner : public lsrv::session_owner {
public:
    explicit collecting_owner(llava_context* c) : ctx(c) {}
    llava_context* context() override { return ctx; }
    void receive_session_outbound_packets(std::list<lsrv::outbound_packet>& packets, std::list<lsrv::outbound_broadcast>& broadcasts) override {
        std::lock_guard<std::mutex> g(m);
        for (auto& p : packets) q.push_back({0, std::get<0>(p), uint32_t(std::get<1>(p)), std::get<2>(p), std::get<3>(p)});
        for (auto& b : broadcasts) q.push_back({1, std::get<0>(b), uint32_t(std::get<1>(b)), 0, std::get<2>(b)});
        packets.clear();
        broadcasts.clear();
        cv.notify_all();
    }
    void notify_session_death(uint32_t) override {
        std::lock_guard<std::mutex> g(m);
        ++dead;
        cv.notify_all();
    }
    llava_context* ctx;
    std::mutex m;
    std::condition_variable cv;
    std::deque<collected> q;
    uint32_t dead = 0;
};
}  // namespace

void* llava_wrapper_owner_create(void* ctx) { return new collecting_owner(static_cast<llava_context*>(ctx)); }
void llava_wrapper_owner_destroy(void* owner) { delete static_cast<collecting_owner*>(owner); }
uint32_t llava_wrapper_owner_dead_sessions(void* owner) {
    auto* o = static_cast<collecting_owner*>(owner);
    std::lock_guard<std::mutex> g(o->m);
    return o->dead;
}

int llava_wrapper_owner_pop(void* owner, int timeout_ms, uint32_t* kind, uint32_t* who, uint32_t* opcode, uint32_t* request,
                            uint8_t* payload, uint32_t cap, uint32_t* length) {
    auto* o = static_cast<collecting_owner*>(owner);
    std::unique_lock<std::mutex> g(o->m);
    if (!o->cv.wait_for(g, std::chrono::milliseconds(timeout_ms), [o]() { return !o->q.empty(); })) return 0;
    collected c = o->q.front();
    o->q.pop_front();
    *kind = uint32_t(c.kind); *who = c.who; *opcode = c.opcode; *request = c.request;
    *length = uint32_t(c.payload.size());
    std::memcpy(payload, c.payload.data(), c.payload.size() < cap ? c.payload.size() : cap);
    return 1;
}

void* llava_wrapper_create(void* owner, int deterministic) {
    lsrv::session_wrapper::set_deterministic_sessions(deterministic != 0);
    return new lsrv::session_wrapper(static_cast<collecting_owner*>(owner));
}
uint32_t llava_wrapper_session_id(void* w) { return static_cast<lsrv::session_wrapper*>(w)->session_id; }
void llava_wrapper_start(void* w) { static_cast<lsrv::session_wrapper*>(w)->start(); }
void llava_wrapper_join(void* w) { static_cast<lsrv::session_wrapper*>(w)->join(); }
void llava_wrapper_destroy(void* w) { delete static_cast<lsrv::session_wrapper*>(w); }
void llava_wrapper_push_order(void* w, uint32_t client_id, uint32_t request_id, uint32_t opcode, uint32_t arg1, const char* s, size_t len) {
    static_cast<lsrv::session_wrapper*>(w)->push_order(client_id, request_id, opcode, arg1, s ? std::string(s, len) : std::string());
}

uint64_t llava_tp_snapshot_slice_offset(uint32_t n_tokens, uint32_t dim, uint32_t layer, uint32_t which, uint32_t row, uint32_t rank,
                                        uint32_t n_ranks) {
    return tp_snapshot_slice_offset(n_tokens, dim, layer, which, row, rank, n_ranks);
}
uint64_t llava_tp_snapshot_file_size(uint32_t n_tokens, uint32_t dim, uint32_t n_layers) { return tp_snapshot_file_size(n_tokens, dim, n_layers); }

// ---- llava_session_group ----
void* llava_session_group_create(void* ctx, void* const* sessions, uint32_t n) {
    std::vector<llava_session*> members;
    for (uint32_t i = 0; i < n; ++i) members.push_back(static_cast<llava_session*>(sessions[i]));
    auto* g = new llava_session_group(static_cast<llava_context*>(ctx), members);
    if (!g->is_valid()) {
        delete g;
        return nullptr;
    }
    return g;
}
void llava_session_group_destroy(void* group) { delete static_cast<llava_session_group*>(group); }
int llava_session_group_step(void* group, uint32_t* next_tokens) {
    auto* g = static_cast<llava_session_group*>(group);
    std::vector<uint32_t> toks;
    if (!g->step(&toks)) return 0;
    if (next_tokens) std::memcpy(next_tokens, toks.data(), toks.size() * 4);
    return 1;
}
int llava_session_group_generate_greedy_on_device(void* group, uint32_t n, uint32_t* out) {
    auto* g = static_cast<llava_session_group*>(group);
    std::vector<std::vector<uint32_t>> toks;
    if (!g->generate_greedy_on_device(n, &toks)) return 0;
    if (out)
        for (size_t i = 0; i < toks.size(); ++i) std::memcpy(out + i * n, toks[i].data(), size_t(n) * 4);
    return 1;
}
int llava_session_group_get_logits(void* group, uint32_t member, float* out, uint32_t n) {
    std::vector<float> v;
    if (!static_cast<llava_session_group*>(group)->get_logits(member, &v) || v.size() != n) return 0;
    std::memcpy(out, v.data(), size_t(n) * sizeof(float));
    return 1;
}
uint32_t llava_session_group_kernel_launches(void* group) { return static_cast<llava_session_group*>(group)->kernel_launches(); }

// ---- lsrv::tlv_server on a thread of its own ----
namespace {
struct served {
    lsrv::tlv_server server;
    std::thread loop;
    served(llava_context* c, uint16_t port, const char* addr) : server(c, port, addr, false) {}
};
}  // namespace

void* llava_server_create(void* ctx, uint32_t port, const char* bind_address, int deterministic) {
    lsrv::session_wrapper::set_deterministic_sessions(deterministic != 0);
    auto* s = new served(static_cast<llava_context*>(ctx), uint16_t(port), bind_address ? bind_address : "127.0.0.1");
    s->server.set_announce(false);           // a library caller reads the port from llava_server_port
    if (!s->server.open()) {
        delete s;
        return nullptr;
    }
    return s;
}
uint32_t llava_server_port(void* server) { return static_cast<served*>(server)->server.port(); }
uint64_t llava_server_grouped_steps(void* server) { return static_cast<served*>(server)->server.grouped_steps(); }
uint64_t llava_server_scheduler_collect_us(void* server) { return static_cast<served*>(server)->server.scheduler_collect_us(); }
uint64_t llava_server_scheduler_device_us(void* server) { return static_cast<served*>(server)->server.scheduler_device_us(); }
uint64_t llava_server_steps_ahead(void* server) { return static_cast<served*>(server)->server.steps_ahead(); }
uint64_t llava_server_grouped_tokens(void* server) { return static_cast<served*>(server)->server.grouped_tokens(); }
void llava_server_start(void* server) {
    auto* s = static_cast<served*>(server);
    if (!s->loop.joinable()) s->loop = std::thread([s]() { s->server.serve_forever(); });
}
void llava_server_stop(void* server) {
    auto* s = static_cast<served*>(server);
    s->server.stop();
    if (s->loop.joinable()) s->loop.join();
}
void llava_server_destroy(void* server) {
    llava_server_stop(server);
    delete static_cast<served*>(server);
}

}  // extern "C"
