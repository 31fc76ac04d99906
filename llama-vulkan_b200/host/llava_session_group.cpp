#include "llava_session_group.h"

#include <algorithm>
#include <cstring>
#include <iostream>
#include <mutex>

#include "llava_buffer.h"
#include "llava_command_buffer.h"
#include "llava_context.h"
#include "llava_device_memory.h"
#include "llava_layer.h"
#include "llava_layer_session_data.h"
#include "llava_session.h"

using namespace std;

namespace {
float* f32(llava_buffer* b) { return static_cast<float*>(b->device_ptr()); }
}  // namespace

llava_session_group::llava_session_group(llava_context* _ctx, vector<llava_session*> _members) : ctx(_ctx), members(std::move(_members)) {
    const u32 k = u32(members.size());
    if (ctx == nullptr || ctx->lv() == nullptr || ctx->tp_size() != 1 || k < 2 || k > llava_session::max_batch_limit) return;
    for (llava_session* s : members)
        if (s == nullptr || s->ctx != ctx || s->is_tracing_enabled()) return;
    for (u32 i = 0; i < k; ++i)
        for (u32 j = i + 1; j < k; ++j)
            if (members[i] == members[j]) return;
    // the batched products take ggjt-v3 blocks only
    if (!ctx->output_w->weight_buffer_is_f16() || ctx->get_layers().empty() || !ctx->get_layers()[0]->wq()->weight_buffer_is_f16()) return;
    const ggml_header& h = ctx->get_model()->get_header();
    const u32 dim = h.dim, ffn = ctx->get_model()->get_ff_size(), n_layers = u32(ctx->get_layers().size());
    if (h.vocab_size % 32 != 0) return;                        // what the batched product of the output matrix asks of its rows
    const auto F = ggml_value_type::f32;
    memory = new llava_device_memory(ctx);
    x = new llava_buffer(ctx, F, dim, k, memory, "group_x");
    q = new llava_buffer(ctx, F, dim, k, memory, "group_q");
    vout = new llava_buffer(ctx, F, dim, k, memory, "group_vout");
    ff = new llava_buffer(ctx, F, ffn, k, memory, "group_ff");
    split = new llava_buffer(ctx, F, u32(lv_act_split_bytes(max(dim, ffn), k) / 4), 1, memory, "group_split");
    logits = new llava_buffer(ctx, F, h.vocab_size, k, memory, "group_logits");
    const size_t scratch_bytes = lv_attention_scratch_bytes(h.n_heads, h.rot, max_backlog_size, k);
    if (scratch_bytes == 0) return;
    scratch = new llava_buffer(ctx, F, u32((scratch_bytes + 3) / 4), 1, memory, "group_attention_scratch");
    tables = new llava_buffer(ctx, F, u32(size_t(n_layers) * k * sizeof(lv_group_member) / 4), 1, memory, "group_members");
    tokens_dev = new llava_buffer(ctx, F, k, 1, memory, "group_tokens");
    sampler_backup = new llava_buffer(ctx, F, 4 * k, 1, memory, "group_sampler_backup");
    if (!memory->freeze() || !memory->zero(0, memory->get_size())) return;
    void* p = nullptr;
    if (lv_host_alloc(ctx->lv(), size_t(k) * 4, &p) != LV_OK) return;
    pinned_tokens = static_cast<u32*>(p);
    valid = true;
}

llava_session_group::~llava_session_group() {
    discard_ahead();
    drop_graph();
    if (pinned_tokens) lv_host_free(ctx->lv(), pinned_tokens);
    for (llava_buffer* b : {x, q, vout, ff, split, logits, scratch, tables, tokens_dev, sampler_backup}) delete b;
    delete memory;
}

void llava_session_group::drop_graph() {
    if (graph) {
        lv_stream_sync(ctx->lv(), 0);
        lv_graph_destroy(graph);
        graph = nullptr;
    }
}

// Checks the members, brings their device state up to date (position words, the pending token in the token log)
// and uploads the member tables if a member's buffers were (re)created since the step was recorded.
bool llava_session_group::prepare_members(u32* backlog) {
    const u32 k = size(), n_layers = u32(ctx->get_layers().size());
    u32 need = min_backlog_size;
    for (llava_session* s : members) {
        if (!s->ensure_buffers_created()) return false;
        if (s->token_buffer.empty() || s->token_buffer.size() - s->current_tokens_in_gpu != 1) {
            cerr << "[!] group step: every member needs exactly one token that is not evaluated yet" << endl;
            return false;
        }
        if (s->token_buffer.size() > s->backlog_size) return false;
        need = max(need, s->backlog_size);
    }
    vector<lv_group_member> table(size_t(n_layers) * k);
    for (u32 l = 0; l < n_layers; ++l) {
        for (u32 i = 0; i < k; ++i) {
            llava_session* s = members[i];
            lv_group_member& m = table[size_t(l) * k + i];
            m.k_cache = s->get_layer_data()[l]->get_k_cache()->device_ptr();
            m.v_cache = s->get_layer_data()[l]->get_v_cache()->device_ptr();
            m.pos = static_cast<u32*>(s->config_buffer->device_ptr());
            m.token_log = static_cast<u32*>(s->token_log->device_ptr());
        }
    }
    // written again only when a member recreated its buffers since the last step
    const size_t table_bytes = table.size() * sizeof(lv_group_member);
    if (uploaded_table.size() != table_bytes || memcmp(uploaded_table.data(), table.data(), table_bytes) != 0) {
        if (!tables->write_raw(0, table.data(), table_bytes)) return false;
        uploaded_table.assign(reinterpret_cast<const u8*>(table.data()), reinterpret_cast<const u8*>(table.data()) + table_bytes);
    }
    vector<bool> sampled_now;
    for (llava_session* s : members) {
        if (!s->sync_device_position(s->current_tokens_in_gpu)) return false;
        if (s->sampling_on_device() && !s->upload_sampler_state()) return false;
        if (!s->upload_pending_tokens(s->current_tokens_in_gpu, 1)) return false;
        if (!s->deterministic && s->host_sampler) {
            cerr << "[!] group step: a member samples on the host; only greedy members and the device sampler are supported" << endl;
            return false;
        }
        sampled_now.push_back(s->sampling_on_device());
    }
    if (sampled_now != sampled) {            // the sampler launches are part of the recorded step
        drop_graph();
        sampled = sampled_now;
    }
    *backlog = need;
    return true;
}

bool llava_session_group::record(u32 backlog) {
    if (graph != nullptr && graph_backlog == backlog) return true;
    drop_graph();
    const ggml_header& h = ctx->get_model()->get_header();
    const u32 k = size(), dim = h.dim, n_layers = u32(ctx->get_layers().size());
    lv_ctx* lv = ctx->lv();
    const lv_group_member* table = static_cast<const lv_group_member*>(tables->device_ptr());
    int rc = lv_graph_begin_capture(lv);
    auto note = [&](int r) { if (rc == LV_OK) rc = r; };
    note(lv_dequant_rows_group(lv, f32(x), ctx->tok_embeddings->device_ptr(), ctx->tok_embeddings->kernel_type(), table, dim, h.vocab_size, k));
    for (u32 l = 0; l < n_layers; ++l) {
        const llava_layer* L = ctx->get_layers()[l];
        const lv_group_member* tl = table + size_t(l) * k;
        const int wt = L->wq()->kernel_type();
        // the op sequence of llava_layer::execute for a batch, with the per-member forms of cache append and attention
        note(lv_act_split_f16(lv, split->device_ptr(), f32(x), static_cast<const float*>(L->attn_norm()->device_ptr()), dim, k));
        note(lv_gemm_tc_qkv_kvappend_group(lv, f32(q), L->wq()->device_ptr(), L->wk()->device_ptr(), L->wv()->device_ptr(), wt,
                                           split->device_ptr(), tl, dim, dim, k, max_backlog_size));
        note(lv_attention_fused_group(lv, f32(vout), f32(q), tl, ctx->rope_table, scratch->device_ptr(), h.n_heads, h.rot, backlog, k));
        note(lv_act_split_f16(lv, split->device_ptr(), f32(vout), nullptr, dim, k));
        note(lv_gemm_tc(lv, f32(x), L->wo()->device_ptr(), wt, split->device_ptr(), dim, dim, k, 1));
        note(lv_act_split_f16(lv, split->device_ptr(), f32(x), static_cast<const float*>(L->ff_norm()->device_ptr()), dim, k));
        note(lv_gemm_tc_silu(lv, f32(ff), L->w3()->device_ptr(), L->w1()->device_ptr(), wt, split->device_ptr(), L->w3()->shape.first, dim, k));
        note(lv_act_split_f16(lv, split->device_ptr(), f32(ff), nullptr, L->w3()->shape.first, k));
        note(lv_gemm_tc(lv, f32(x), L->w2()->device_ptr(), wt, split->device_ptr(), dim, L->w2()->shape.second, k, 1));
    }
    // every member needs its logits: final norm and output matrix for all rows (llava_command_buffer.cpp:38-39)
    note(lv_act_split_f16(lv, split->device_ptr(), f32(x), static_cast<const float*>(ctx->norm_w->device_ptr()), dim, k));
    note(lv_gemm_tc(lv, f32(logits), ctx->output_w->device_ptr(), ctx->output_w->kernel_type(), split->device_ptr(), h.vocab_size, dim, k, 0));
    note(lv_argmax_advance_group(lv, f32(logits), h.vocab_size, table, k, max_backlog_size + 1, static_cast<u32*>(tokens_dev->device_ptr()),
                                 pinned_tokens));
    // members that sample (the reference's default): the sampler of their own step, on their row of the logits;
    // it overwrites the greedy token in the member's token log and in the pinned word
    for (u32 i = 0; i < k; ++i) {
        if (!sampled[i]) continue;
        llava_session* s = members[i];
        u32* log = static_cast<u32*>(s->token_log->device_ptr());
        note(lv_sample_mirostat(lv, f32(logits) + size_t(i) * h.vocab_size, h.vocab_size, log, static_cast<u32*>(s->config_buffer->device_ptr()),
                                static_cast<u32*>(s->sampler_state->device_ptr()), -1.0f, log, max_backlog_size + 1,
                                static_cast<u32*>(tokens_dev->device_ptr()) + i, pinned_tokens + i, nullptr));
    }
    lv_graph* g = nullptr;
    const int end = lv_graph_end_capture(lv, &g);
    note(end);
    if (rc != LV_OK) {
        cerr << "[!] group step: recording failed: " << lv_last_error_string() << endl;
        if (g) lv_graph_destroy(g);
        return false;
    }
    graph = g;
    graph_backlog = backlog;
    launches = 0;
    lv_graph_kernel_nodes(graph, &launches);
    return true;
}

bool llava_session_group::step(vector<u32>* next_tokens) {
    if (!valid) return false;
    discard_ahead();
    lock_guard<mutex> guard(ctx->queue_mutex);
    u32 backlog = 0;
    if (!prepare_members(&backlog) || !record(backlog)) return false;
    if (lv_graph_launch(ctx->lv(), graph) != LV_OK || lv_stream_sync(ctx->lv(), 0) != LV_OK) {
        cerr << "[!] group step failed: " << lv_last_error_string() << endl;
        return false;
    }
    for (llava_session* s : members) {
        s->current_tokens_in_gpu += 1;
        s->device_pos += 1;
    }
    if (next_tokens) next_tokens->assign(pinned_tokens, pinned_tokens + size());
    return true;
}

bool llava_session_group::can_step_ahead() const {
    if (!valid || graph == nullptr || ahead) return false;
    for (llava_session* s : members)
        if (s->token_buffer.size() + 2 > s->backlog_size) return false;       // the backlog is about to grow: re-record first
    return true;
}

bool llava_session_group::launch_ahead() {
    if (!can_step_ahead()) return false;
    lock_guard<mutex> guard(ctx->queue_mutex);
    // a member that samples: its sampler state {mu, seed, draws} is kept, so that a dropped step leaves no trace in it
    for (u32 i = 0; i < size(); ++i)
        if (sampled[i] && lv_copy_d2d(ctx->lv(), static_cast<u8*>(sampler_backup->device_ptr()) + 16 * size_t(i),
                                      members[i]->sampler_state->device_ptr(), 16) != LV_OK)
            return false;
    if (lv_graph_launch(ctx->lv(), graph) != LV_OK) return false;
    ahead = true;
    return true;
}

bool llava_session_group::finish_ahead(vector<u32>* next_tokens) {
    if (!ahead) return false;
    lock_guard<mutex> guard(ctx->queue_mutex);
    ahead = false;
    if (lv_stream_sync(ctx->lv(), 0) != LV_OK) {
        cerr << "[!] group step failed: " << lv_last_error_string() << endl;
        for (llava_session* s : members) s->device_pos = ~0U;
        return false;
    }
    for (llava_session* s : members) {
        s->current_tokens_in_gpu += 1;
        s->device_pos += 1;
    }
    if (next_tokens) next_tokens->assign(pinned_tokens, pinned_tokens + size());
    return true;
}

void llava_session_group::discard_ahead() {
    if (!ahead) return;
    lock_guard<mutex> guard(ctx->queue_mutex);
    ahead = false;
    for (u32 i = 0; i < size(); ++i)
        if (sampled[i]) lv_copy_d2d(ctx->lv(), members[i]->sampler_state->device_ptr(),
                                    static_cast<const u8*>(sampler_backup->device_ptr()) + 16 * size_t(i), 16);
    lv_stream_sync(ctx->lv(), 0);
    for (llava_session* s : members) s->device_pos = ~0U;          // the device is one position further than the host's books
}

bool llava_session_group::generate_greedy_on_device(u32 n, vector<vector<u32>>* out) {
    if (!valid || n == 0) return false;
    discard_ahead();
    for (llava_session* s : members) {
        // room for the n tokens in every member (llava_session::enqueue_greedy_on_device)
        u32 need = s->backlog_size;
        while (s->token_buffer.size() + n > need) need <<= 1;
        if (need > max_backlog_size || !s->set_backlog_size(need)) return false;
    }
    lock_guard<mutex> guard(ctx->queue_mutex);
    u32 backlog = 0;
    if (!prepare_members(&backlog) || !record(backlog)) return false;
    for (u32 i = 0; i < n; ++i)
        if (lv_graph_launch(ctx->lv(), graph) != LV_OK) return false;           // each step consumes the previous step's tokens
    if (lv_stream_sync(ctx->lv(), 0) != LV_OK) {
        cerr << "[!] group steps failed: " << lv_last_error_string() << endl;
        return false;
    }
    if (out) out->assign(size(), {});
    for (u32 i = 0; i < size(); ++i) {
        llava_session* s = members[i];
        const u32 start = u32(s->token_buffer.size());
        vector<u32> fresh(n);
        if (!s->token_log->read_raw(size_t(start) * 4, fresh.data(), size_t(n) * 4)) return false;
        s->token_buffer.insert(s->token_buffer.end(), fresh.begin(), fresh.end());
        s->current_tokens_in_gpu += n;
        s->device_pos += n;
        if (out) (*out)[i] = fresh;
    }
    return true;
}

bool llava_session_group::get_logits(u32 member, vector<float>* out) {
    if (!valid || member >= size()) return false;
    const u32 vocab = ctx->get_model()->get_header().vocab_size;
    out->resize(vocab);
    return logits->read_raw(size_t(member) * vocab * sizeof(float), out->data(), size_t(vocab) * sizeof(float));
}
