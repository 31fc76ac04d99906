#include "llava_session.h"

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <iostream>

#include "llava_buffer.h"
#include "llava_command_buffer.h"
#include "llava_context.h"
#include "llava_device_memory.h"
#include "llava_layer.h"
#include "tp_shard.h"
#include "llava_layer_session_data.h"
#include "utils.h"

using namespace std;

namespace {
// words of the pinned staging block after the token area
constexpr u32 kCfgWords = 0;      // 4 words: position to upload
constexpr u32 kArgmaxWord = 4;    // argmax written by the recorded step
constexpr u32 kSampleWord = 5;    // token drawn by the device sampler
constexpr u32 kStateWords = 8;    // 4 words: sampler state to upload / read back
constexpr u32 kPinnedExtra = 16;
}  // namespace

llava_session::llava_session(llava_context* _ctx)
    : ctx(_ctx), model(_ctx->get_model()), rng(u32(time(nullptr))), mirostat_mu(2 * mirostat_tau), sampler_seed(u32(time(nullptr))),
      backlog_size(min_backlog_size) {
    void* p = nullptr;
    if (lv_host_alloc(ctx->lv(), size_t(max_backlog_size + kPinnedExtra) * 4, &p) == LV_OK) {
        pinned = static_cast<u32*>(p);
        memset(pinned, 0, size_t(max_backlog_size + kPinnedExtra) * 4);
    } else {
        failed = true;
    }
}

llava_session::~llava_session() {
    lv_stream_sync(ctx->lv(), 0);
    drop_command_buffers();
    lv_step_plan_destroy(step_plan);
    for (auto* x : layer_data) delete x;
    reset_main_buffers();
    if (pinned) lv_host_free(ctx->lv(), pinned);
}

void llava_session::drop_command_buffers() {
    for (auto& kv : command_buffers) delete kv.second;
    command_buffers.clear();
    last_command_buffer = nullptr;
}

bool llava_session::ensure_buffers_created() {
    if (failed) return false;
    if (layer_data.empty()) {
        layer_data.reserve(ctx->get_layers().size());
        for (u32 i = 0; i < ctx->get_layers().size(); ++i) layer_data.push_back(new llava_layer_session_data(this));
    }
    ensure_step_plan();
    if (main_buffer_memory == nullptr) return recreate_buffers();
    return true;
}

// Binds the context's weights and this session's caches for lv_decode_step.  Failing to create a plan is not
// an error: the session then records one kernel per operation.
void llava_session::ensure_step_plan() {
    if (step_plan_tried) return;
    if (ctx->tp_size() != 1 && !ctx->fused_exchange()) return;      // ask again once the windows are connected
    step_plan_tried = true;
    const char* env = getenv("LV_DECODE_STEP");
    if (env == nullptr || env[0] != '1') return;          // opt-in while it is slower than one kernel per operation
    if (ctx->tp_size() != 1 && !ctx->fused_exchange()) return;      // sharded: the partial rows travel through the peer windows
    const ggml_header& h = model->get_header();
    const auto& layers = ctx->get_layers();
    std::vector<lv_step_layer> tab(layers.size());
    for (size_t i = 0; i < layers.size(); ++i) {
        const llava_layer* l = layers[i];
        lv_step_layer& t = tab[i];
        t.wq = l->wq()->device_ptr(); t.wk = l->wk()->device_ptr(); t.wv = l->wv()->device_ptr(); t.wo = l->wo()->device_ptr();
        t.w1 = l->w1()->device_ptr(); t.w2 = l->w2()->device_ptr(); t.w3 = l->w3()->device_ptr();
        t.attention_norm = static_cast<const float*>(l->attn_norm()->device_ptr());
        t.ffn_norm = static_cast<const float*>(l->ff_norm()->device_ptr());
        t.k_cache = layer_data[i]->get_k_cache()->device_ptr();
        t.v_cache = layer_data[i]->get_v_cache()->device_ptr();
        if (l->wq()->type != ctx->output_w->type) return;              // one matrix type per model
    }
    lv_step_model m{};
    m.dim = h.dim; m.ff = model->get_ff_size(); m.heads = h.n_heads; m.n_layers = u32(layers.size()); m.vocab = h.vocab_size;
    m.ctx_rows = max_backlog_size;
    if (ctx->tp_size() > 1) {
        m.tp_ranks = ctx->tp_size();
        m.tp_rank = ctx->tp_rank();
        m.shard_cols_o = layers[0]->wo()->shape.second;
        m.shard_cols_2 = layers[0]->w2()->shape.second;
    }
    m.wtype = ctx->output_w->kernel_type();
    m.emb_type = ctx->tok_embeddings->kernel_type();
    m.weights_base = ctx->weights_memory()->device_base();
    m.weights_bytes = ctx->weights_memory()->get_size();
    m.tok_embeddings = ctx->tok_embeddings->device_ptr();
    m.norm = static_cast<const float*>(ctx->norm_w->device_ptr());
    m.output = ctx->output_w->device_ptr();
    m.rope_table = ctx->rope_table;
    m.layers = tab.data();
    if (lv_step_plan_create(ctx->lv(), &m, &step_plan) != LV_OK) {
        cerr << "[?] no one-launch step for this model (one kernel per operation instead): " << lv_last_error_string() << endl;
        step_plan = nullptr;
    }
}

bool llava_session::recreate_buffers() {
    reset_main_buffers();
    const ggml_header& h = model->get_header();
    const u32 dim = h.dim, ff = model->get_ff_size(), B = max_batch;
    const u32 ranks = ctx->tp_size(), rank = ctx->tp_rank();
    // per-rank sizes: heads (and with them Q, K, V, the attention output) and the FFN width are
    // split; the inputs of the column-sharded wo and w2 are padded like their shards
    const u32 local_dim = dim / ranks;
    const auto Wt = ctx->output_w->type;
    const u32 vout_len = ranks == 1 ? dim : tp_shape(Wt, dim, dim, tp_split::columns, rank, ranks).cols;
    const u32 ff_len = ranks == 1 ? ff : tp_shape(Wt, dim, ff, tp_split::columns, rank, ranks).cols;
    const auto F = ggml_value_type::f32;
    main_buffer_memory = new llava_device_memory(ctx);
    llava_device_memory* m = main_buffer_memory;
    current_thought = new llava_buffer(ctx, F, dim, B, m);
    current_thought_sublayer = new llava_buffer(ctx, F, dim, B, m);
    current_thought_middle_normd = new llava_buffer(ctx, F, dim, B, m);
    main_ff_result = new llava_buffer(ctx, F, ff_len, B, m);
    current_Q = new llava_buffer(ctx, F, local_dim, B, m);
    current_K = new llava_buffer(ctx, F, local_dim, B, m);
    current_V = new llava_buffer(ctx, F, local_dim, B, m);
    current_Vout = new llava_buffer(ctx, F, vout_len, B, m);
    if (ranks > 1) tp_partial = new llava_buffer(ctx, F, dim, B, m);
    if (is_tracing_enabled()) main_attn_result = new llava_buffer(ctx, F, backlog_size, h.n_heads * B, m);
    config_buffer = new llava_buffer(ctx, F, 4, 1, m);
    output_probs = new llava_buffer(ctx, F, h.vocab_size, 1, m);
    token_log = new llava_buffer(ctx, F, max_backlog_size + kPinnedExtra, 1, m);
    argmax_result = new llava_buffer(ctx, F, 4, 1, m);
    sampler_state = new llava_buffer(ctx, F, 4, 1, m);
    sampler_state_dirty = true;
    const size_t scratch = lv_attention_scratch_bytes(h.n_heads / ranks, h.rot, max_backlog_size, B);
    if (scratch == 0) return false;
    attn_scratch = new llava_buffer(ctx, F, u32((scratch + 3) / 4), 1, m);
    if (B >= llava_command_buffer::kTensorCoreMinBatch)
        act_split = new llava_buffer(ctx, F, u32(lv_act_split_bytes(max(max(dim, ff_len), vout_len), B) / 4), 1, m);
    if (!m->freeze() || !m->zero(0, m->get_size())) return false;
    device_pos = ~0U;
    return true;
}

void llava_session::reset_main_buffers() {
    for (llava_buffer** b : {&current_thought, &current_thought_sublayer, &current_thought_middle_normd, &current_Q, &current_K,
                             &current_V, &current_Vout, &main_attn_result, &config_buffer, &output_probs, &main_ff_result,
                             &token_log, &argmax_result, &attn_scratch, &tp_partial, &act_split, &sampler_state}) {
        delete *b;
        *b = nullptr;
    }
    delete main_buffer_memory;
    main_buffer_memory = nullptr;
}

void llava_session::set_seed(u32 seed) {
    rng.seed(seed);
    sampler_seed = seed;
    sampler_state_dirty = true;
}

void llava_session::set_host_sampler(bool on) {
    if (on == host_sampler) return;
    get_mirostat_mu();              // bring mu over to the side that continues
    host_sampler = on;
    sampler_state_dirty = true;
}

// mu lives where the last token was drawn: on the device after device draws
float llava_session::get_mirostat_mu() {
    if (sampler_state != nullptr && !sampler_state_dirty && sampling_on_device()) {
        lv_stream_sync(ctx->lv(), 0);
        u32 words[4] = {0, 0, 0, 0};
        if (sampler_state->read_raw(0, words, sizeof words)) memcpy(&mirostat_mu, &words[0], 4);
    }
    return mirostat_mu;
}

// {mu, seed, draws so far, -} to the device, when the host copy is newer
bool llava_session::upload_sampler_state() {
    if (!sampler_state_dirty) return true;
    if (lv_stream_sync(ctx->lv(), 0) != LV_OK) return false;
    u32* w = pinned + max_backlog_size + kStateWords;
    memcpy(&w[0], &mirostat_mu, 4);
    w[1] = sampler_seed;
    w[2] = 0;
    w[3] = 0;
    if (lv_upload_async(ctx->lv(), sampler_state->device_ptr(), w, 16) != LV_OK) return false;
    sampler_state_dirty = false;
    return true;
}

llava_command_buffer* llava_session::get_command_buffer(u32 batch, bool with_head) {
    const bool sample = with_head && sampling_on_device();
    const u32 key = batch | (with_head ? 1u << 16 : 0u) | (sample ? 1u << 17 : 0u);
    auto it = command_buffers.find(key);
    if (it != command_buffers.end()) return it->second;
    auto* cb = new llava_command_buffer(this, batch, with_head, sample);
    if (!cb->record_execution()) {
        delete cb;
        return nullptr;
    }
    command_buffers[key] = cb;
    return cb;
}

bool llava_session::upload_pending_tokens(u32 first, u32 count) {
    memcpy(pinned + first, token_buffer.data() + first, size_t(count) * 4);
    return lv_upload_async(ctx->lv(), static_cast<u32*>(token_log->device_ptr()) + first, pinned + first, size_t(count) * 4) == LV_OK;
}

bool llava_session::sync_device_position(u32 pos) {
    if (device_pos == pos) return true;
    // rare (first step, rewind, restore): drain the stream so the staging words are free
    if (lv_stream_sync(ctx->lv(), 0) != LV_OK) return false;
    for (u32 i = 0; i < 4; ++i) pinned[max_backlog_size + kCfgWords + i] = pos;      // llava_session.cpp:224-225
    if (lv_upload_async(ctx->lv(), config_buffer->device_ptr(), pinned + max_backlog_size + kCfgWords, 16) != LV_OK) return false;
    device_pos = pos;
    return true;
}

bool llava_session::start_next_token_prediction() {
    if (!ensure_buffers_created()) return false;
    u32 to_process = u32(token_buffer.size()) - current_tokens_in_gpu;
    if (to_process == 0) {
        cerr << "GPU is already in sync" << endl;
        return false;
    }
    if (token_buffer.size() > backlog_size) {
        cerr << "Token buffer overflow" << endl;
        return false;
    }
    lock_guard<mutex> guard(ctx->queue_mutex);
    if (!sync_device_position(current_tokens_in_gpu)) return false;
    if (sampling_on_device() && !upload_sampler_state()) return false;
    if (!upload_pending_tokens(current_tokens_in_gpu, to_process)) return false;
    while (to_process > 0) {
        u32 n = min(to_process, max_batch);
        // sharded: a batch goes through the tensor-core step with its stand-alone exchanges; what is too short for that
        // goes token by token through the step with the exchange fused into the GEMVs
        if (ctx->tp_size() > 1 && n < llava_command_buffer::kTensorCoreMinBatch) n = 1;
        llava_command_buffer* cb = get_command_buffer(n, n == to_process);
        if (cb == nullptr || !cb->run()) return false;
        batch_size = n;
        last_command_buffer = cb;
        current_tokens_in_gpu += n;
        device_pos += n;
        to_process -= n;
    }
    return true;
}

u32 llava_session::finish_next_token_prediction() {
    if (last_command_buffer == nullptr || !last_command_buffer->wait_idle()) {
        cerr << "[!] evaluation failed: " << lv_last_error_string() << endl;
        return ~0U;
    }
    return get_last_predicted_token(deterministic);
}

u32 llava_session::predict_next_token() {
    if (!start_next_token_prediction()) return ~0U;
    return finish_next_token_prediction();
}

bool llava_session::set_step_trace(bool on) {
    if (!ensure_buffers_created() || step_plan == nullptr) return false;
    lv_stream_sync(ctx->lv(), 0);
    drop_command_buffers();                       // the trace buffer is an argument of the recorded launch
    return lv_step_plan_set_trace(step_plan, on ? 1 : 0) == LV_OK;
}

bool llava_session::read_step_trace(vector<u64>* out, u32* n_ops, u32* n_ctas, u32* n_points) {
    if (step_plan == nullptr) return false;
    out->resize(size_t(4 * ctx->get_layers().size() + 1) * 1024 * 8);
    return lv_step_plan_read_trace(step_plan, out->data(), out->size(), n_ops, n_ctas, n_points) == LV_OK;
}

u32 llava_session::step_kernel_launches() const {
    return last_command_buffer ? last_command_buffer->kernel_launches() : 0;
}

bool llava_session::get_logits(vector<float>* out) {
    if (output_probs == nullptr) return false;
    out->resize(model->get_header().vocab_size);
    return output_probs->read_raw(0, out->data(), out->size() * sizeof(float));
}

u32 llava_session::get_last_predicted_token(bool want_deterministic) {
    if (last_command_buffer && !last_command_buffer->wait_idle()) return ~0U;
    if (want_deterministic) {
        // first index of the largest logit (llava_session.cpp:144-152), computed on the device
        return pinned[max_backlog_size + kArgmaxWord];
    }
    if (!host_sampler) return pinned[max_backlog_size + kSampleWord];      // drawn by the recorded step (lv_sample_mirostat)
    vector<float> logits;
    if (!get_logits(&logits)) return ~0U;
    for (float x : logits) {
        if (std::isnan(x) || std::isinf(x)) {          // llava_session.cpp:137-142
            cerr << "NaN in output buffer" << endl;
            break;
        }
    }
    return sample_from_logits(logits);
}

// The reference's sampler (llava_session.cpp:154-194): repeat/frequency penalty applied to
// token 13 only, temperature, probabilities without max-subtraction, candidates with
// p >= 0.5^mu, one draw from them, mu moved by eta * (tau + log2(p_drawn / kept mass)).
u32 llava_session::sample_from_logits(vector<float>& p) {
    const u32 n_vocab = u32(p.size());
    u32 newline_count = 0;
    const size_t first = token_buffer.size() > repeat_last_n ? token_buffer.size() - repeat_last_n : 0;
    for (size_t i = first; i < token_buffer.size(); ++i) newline_count += token_buffer[i] == 13;
    if (newline_count != 0 && n_vocab > 13) {
        p[13] = p[13] <= 0 ? p[13] * repeat_penalty : p[13] / repeat_penalty;
        p[13] -= alpha_frequency * float(newline_count) + alpha_presence;
    }
    float total = 0;
    for (float& x : p) {
        x = expf(x / temp);
        total += x;
    }
    const float cut = powf(0.5f, mirostat_mu);
    vector<float> kept;
    vector<u32> kept_id;
    float kept_sum = 0;
    for (u32 i = 0; i < n_vocab; ++i) {
        const float q = p[i] / total;
        if (q >= cut) {
            kept.push_back(q);
            kept_id.push_back(i);
            kept_sum += q;
        }
    }
    if (kept.empty()) return ~0U;
    discrete_distribution<> dist(kept.begin(), kept.end());
    const int idx = dist(rng);
    mirostat_mu += mirostat_eta * (mirostat_tau + log2f(kept[idx] / kept_sum));
    return kept_id[idx];
}

bool llava_session::generate_greedy_on_device(u32 n, vector<u32>* out) {
    return enqueue_greedy_on_device(n) && collect_greedy_on_device(out);
}

bool llava_session::enqueue_greedy_on_device(u32 n) {
    if (n == 0 || enqueued_greedy != 0) return false;
    if (!ensure_buffers_created()) return false;
    if (token_buffer.empty() || token_buffer.size() - current_tokens_in_gpu != 1) return false;
    u32 need = backlog_size;
    while (token_buffer.size() + n > need) need <<= 1;
    if (need > max_backlog_size || !set_backlog_size(need)) return false;
    lock_guard<mutex> guard(ctx->queue_mutex);
    if (!sync_device_position(current_tokens_in_gpu)) return false;
    if (sampling_on_device() && !upload_sampler_state()) return false;
    if (!upload_pending_tokens(current_tokens_in_gpu, 1)) return false;
    llava_command_buffer* cb = get_command_buffer(1, true);
    if (cb == nullptr) return false;
    for (u32 i = 0; i < n; ++i) if (!cb->run()) return false;      // each step consumes the previous step's argmax
    batch_size = 1;
    last_command_buffer = cb;
    enqueued_greedy = n;
    return true;
}

bool llava_session::collect_greedy_on_device(vector<u32>* out) {
    const u32 n = enqueued_greedy;
    if (n == 0 || last_command_buffer == nullptr) return false;
    enqueued_greedy = 0;
    if (!last_command_buffer->wait_idle()) return false;
    const u32 start = u32(token_buffer.size());
    vector<u32> fresh(n);
    if (!token_log->read_raw(size_t(start) * 4, fresh.data(), size_t(n) * 4)) return false;
    token_buffer.insert(token_buffer.end(), fresh.begin(), fresh.end());
    current_tokens_in_gpu += n;
    device_pos += n;
    if (out) out->insert(out->end(), fresh.begin(), fresh.end());
    return true;
}

bool llava_session::set_text(const string& new_text) {
    vector<u32> fresh;
    model->tokenize(fresh, new_text, true);
    u32 next_backlog_size = backlog_size;
    while (fresh.size() > next_backlog_size) next_backlog_size <<= 1;        // llava_session.cpp:260-266
    if (next_backlog_size > max_backlog_size) return false;
    if (!set_backlog_size(next_backlog_size)) return false;
    // keep the evaluated prefix that the new token sequence shares with the old one (the
    // reference compares token ids with characters of the text here, llava_session.cpp:271,
    // which never matches; comparing token ids is what was meant and changes no result)
    u32 max_prefix = 0;
    while (max_prefix < fresh.size() && max_prefix < token_buffer.size() && max_prefix < current_tokens_in_gpu &&
           token_buffer[max_prefix] == fresh[max_prefix])
        max_prefix++;
    token_buffer = fresh;
    current_tokens_in_gpu = max_prefix;
    return true;
}

bool llava_session::add_text(const string& s) {
    return set_text(model->tokens_to_text(token_buffer.data(), u32(token_buffer.size())) + s);   // llava_session.cpp:279-282
}

bool llava_session::push_token(u32 new_token) {
    if (new_token >= model->get_tokens().size()) return false;
    if (token_buffer.size() == backlog_size) {                              // llava_session.cpp:286-294
        if (backlog_size == max_backlog_size) return false;
        if (!set_backlog_size(backlog_size * 2)) return false;
    }
    token_buffer.push_back(new_token);
    return true;
}

bool llava_session::set_backlog_size(u32 new_size) {
    if (new_size > max_backlog_size) return false;                          // llava_session.cpp:303-315
    if (new_size == backlog_size) return true;
    if (new_size < min_backlog_size) return false;
    if (new_size < current_tokens_in_gpu) return false;
    lv_stream_sync(ctx->lv(), 0);
    drop_command_buffers();
    backlog_size = new_size;
    // the caches already cover max_backlog_size rows; only buffers shaped by the backlog
    // (the trace scores) have to follow
    if (is_tracing_enabled() && main_buffer_memory != nullptr && !recreate_buffers()) return false;
    return flush_layers_data_buffers();
}

bool llava_session::tensor_core_shapes_ok() const {
    const u32 ranks = ctx->tp_size();
    if (ranks == 1) return true;
    return (model->get_header().dim / ranks) % 128 == 0 && (model->get_ff_size() / ranks) % 32 == 0;
}

bool llava_session::set_max_batch(u32 n) {
    if (n < 1 || n > max_batch_limit) return false;
    // sharded sessions evaluate prompt batches on the tensor cores (one exchange per sub-block for the whole batch) or,
    // where the shard shapes do not fit the tiles, token by token
    if (n > 1 && ctx->tp_size() > 1 && (n < llava_command_buffer::kTensorCoreMinBatch || !tensor_core_shapes_ok())) return false;
    if (n == max_batch) return true;
    lv_stream_sync(ctx->lv(), 0);
    drop_command_buffers();
    max_batch = n;
    if (main_buffer_memory != nullptr && !recreate_buffers()) return false;
    return flush_layers_data_buffers();
}

bool llava_session::flush_layers_data_buffers() {
    bool ok = true;
    for (llava_layer_session_data* l : layer_data) ok = l->flush_buffers_on_gpu() && ok;
    return ok;
}

void llava_session::rewind(u32 n) {
    if (n < token_buffer.size()) {                                          // llava_session.cpp:390-395
        token_buffer.resize(n);
        current_tokens_in_gpu = min(n, current_tokens_in_gpu);
    }
}

ReturnCode llava_session::set_options(u32 new_options) {
    if (options == new_options) return ReturnCode::ok;
    if (new_options != 0 && ctx->tp_size() > 1) return ReturnCode::nok;    // tracing records whole-model buffers
    lv_stream_sync(ctx->lv(), 0);
    options = new_options;
    drop_command_buffers();
    if (!ensure_buffers_created() || !recreate_buffers() || !flush_layers_data_buffers()) return ReturnCode::nok;
    return ReturnCode::ok;
}

ReturnCode llava_session::save_frame(const string& path) {
    if (!is_tracing_enabled()) return ReturnCode::not_tracing;
    if (last_command_buffer) last_command_buffer->wait_idle();
    const int fd = ::open(path.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) {
        perror("open");
        return ReturnCode::nok;
    }
    u32 i = 0;
    for (llava_layer_session_data* l : layer_data) l->dump_tracing_layers(fd, "layer." + to_string(i++));
    ::close(fd);
    return ReturnCode::ok;
}

// File layout (llava_session.cpp:447-495): u32 n; u32 tokens[n]; then per layer the first n
// rows of the K cache followed by the first n rows of the V cache, f16 [n][dim] each.
// File layout of the reference (llava_session.cpp:447-500): {u32 n; u32 tokens[n]; per layer: K rows [n][dim] f16, V rows
// [n][dim] f16}.  A tensor-parallel rank holds the columns [rank * dim / ranks, (rank + 1) * dim / ranks) of every row (its
// heads): each rank writes its column slices at their place in the same file, so that the file equals the one a single
// GPU writes.  Every rank sizes the file and writes the header; the caller waits for all ranks before reading it.
ReturnCode llava_session::snapshot(const string& path) {
    if (!ensure_buffers_created()) return ReturnCode::nok;
    if (last_command_buffer) last_command_buffer->wait_idle();
    const u32 n = current_tokens_in_gpu, dim = model->get_header().dim, ranks = ctx->tp_size(), width = dim / ranks;
    const size_t per_layer = size_t(2) * n * dim * 2, local = size_t(2) * n * width * 2;
    const int fd = ::open(path.c_str(), ranks > 1 ? (O_WRONLY | O_CREAT) : (O_WRONLY | O_CREAT | O_TRUNC), 0644);
    if (fd < 0) {
        perror("open");
        return ReturnCode::nok;
    }
    bool ok = ::ftruncate(fd, off_t(tp_snapshot_file_size(n, dim, u32(layer_data.size())))) == 0;
    ok = ok && pwrite_noshort(fd, &n, 4, 0) == 4 && pwrite_noshort(fd, token_buffer.data(), size_t(n) * 4, 4) == size_t(n) * 4;
    vector<u8> rows(local);
    const size_t row_bytes = size_t(width) * 2;
    u32 layer = 0;
    for (llava_layer_session_data* l : layer_data) {
        ok = ok && l->dump_kv_cache(rows.data(), n);
        if (ranks == 1) {
            ok = ok && pwrite_noshort(fd, rows.data(), per_layer, (long long)tp_snapshot_slice_offset(n, dim, layer, 0, 0, 0, 1)) == per_layer;
        } else {
            for (u32 which = 0; which < 2 && ok; ++which)           // K rows, then V rows
                for (u32 i = 0; i < n && ok; ++i)
                    ok = pwrite_noshort(fd, rows.data() + (size_t(which) * n + i) * row_bytes, row_bytes,
                                        (long long)tp_snapshot_slice_offset(n, dim, layer, which, i, ctx->tp_rank(), ranks)) == row_bytes;
        }
        ++layer;
    }
    if (::close(fd) < 0) ok = false;
    return ok ? ReturnCode::ok : ReturnCode::nok;
}

ReturnCode llava_session::restore(const string& path) {
    if (!ensure_buffers_created()) return ReturnCode::nok;
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) {
        perror("open");
        return ReturnCode::nok;
    }
    struct stat st {};
    u32 n = 0;
    auto bail = [&](const char* why) {
        cerr << why << endl;
        ::close(fd);
        return ReturnCode::nok;
    };
    if (::fstat(fd, &st) < 0 || !S_ISREG(st.st_mode)) return bail("Expected a regular file");
    if (st.st_size < 4 || read_noshort(fd, &n, 4) != 4) return bail("File too short");
    if (n > max_backlog_size) return bail("Too many tokens");                      // llava_session.cpp:543
    const u32 dim = model->get_header().dim;
    const size_t per_layer = size_t(2) * n * dim * 2;
    const size_t expected = layer_data.size() * per_layer + size_t(4) * n + 4;        // llava_session.cpp:559
    if (expected != size_t(st.st_size)) return bail("File size mismatch");
    u32 needed = min_backlog_size;
    while (needed < n) needed <<= 1;
    vector<u32> toks(n);
    if (read_noshort(fd, toks.data(), size_t(n) * 4) != size_t(n) * 4) return bail("Short read");
    for (u32 t : toks) if (t >= model->get_tokens().size()) return bail("Token id out of range");
    lv_stream_sync(ctx->lv(), 0);
    rewind(0);
    if (!set_backlog_size(needed)) return bail("Cannot set backlog size");
    // a tensor-parallel rank takes its column slice of every row (see snapshot)
    const u32 ranks = ctx->tp_size(), width = dim / ranks;
    const size_t row_bytes = size_t(width) * 2;
    vector<u8> rows(size_t(2) * n * row_bytes);
    u32 layer = 0;
    for (llava_layer_session_data* l : layer_data) {
        if (ranks == 1) {
            if (pread_noshort(fd, rows.data(), per_layer, (long long)tp_snapshot_slice_offset(n, dim, layer, 0, 0, 0, 1)) != per_layer) return bail("Short read");
        } else {
            for (u32 which = 0; which < 2; ++which)
                for (u32 i = 0; i < n; ++i)
                    if (pread_noshort(fd, rows.data() + (size_t(which) * n + i) * row_bytes, row_bytes,
                                      (long long)tp_snapshot_slice_offset(n, dim, layer, which, i, ctx->tp_rank(), ranks)) != row_bytes)
                        return bail("Short read");
        }
        if (!l->restore_kv_cache(rows.data(), n)) return bail("Cannot upload the cache rows");
        ++layer;
    }
    ::close(fd);
    token_buffer = toks;
    current_tokens_in_gpu = n;
    return ReturnCode::ok;
}
