#include "llava_command_buffer.h"

#include <iostream>

#include "llava_buffer.h"
#include "llava_context.h"
#include "llava_layer.h"
#include "llava_layer_session_data.h"
#include "llava_session.h"

using namespace std;

llava_command_buffer::llava_command_buffer(llava_session* _session, u32 _batch_size, bool _with_head, bool _sample)
    : session(_session), backlog_size(_session->backlog_size), workgroup_size(_session->ctx->workgroup_size),
      batch_size(_batch_size), with_head(_with_head), sample(_sample && _with_head) {}

llava_command_buffer::~llava_command_buffer() {
    wait_idle();
    lv_graph_destroy(graph);
}

lv_ctx* llava_command_buffer::lv() const { return session->ctx->lv(); }

void llava_command_buffer::note(int rc) {
    if (rc != LV_OK && first_error == LV_OK) {
        first_error = rc;
        cerr << "[!] recording failed: " << lv_last_error_string() << endl;
    }
}

// Shape contract of an op (the reference asserts these before each dispatch,
// e.g. llava_command_buffer.cpp:64-67,137-140,158-165).
bool llava_command_buffer::expect(bool cond, const char* what) {
    if (!cond && first_error == LV_OK) {
        first_error = LV_ERR_BAD_ARGUMENTS;
        cerr << "[!] shape check failed: " << what << endl;
    }
    return cond;
}

bool llava_command_buffer::wait_idle() const {
    // the reference waits on its fence for up to 1000 s and ignores the result
    // (llava_command_buffer.cpp:25-27); here the result is reported
    return lv_stream_sync(lv(), 1000 * 1000) == LV_OK;
}

u32 llava_command_buffer::kernel_launches() const {
    uint32_t n = 0;
    return (graph && lv_graph_kernel_nodes(graph, &n) == LV_OK) ? n : 0;
}

bool llava_command_buffer::run() {
    if (!graph) return false;
    return lv_graph_launch(lv(), graph) == LV_OK;
}

// The reference's sampler as the last kernel of the step (llava_session.cpp:154-194): reads the logits and the token
// history where they are, leaves the drawn token in the pinned staging word and -- for decoding without the host in
// the loop -- in the token log slot that the next step reads.
void llava_command_buffer::record_sampler() {
    llava_session* s = session;
    u32* config = static_cast<u32*>(s->config_buffer->device_ptr());
    u32* log = static_cast<u32*>(s->token_log->device_ptr());
    note(lv_sample_mirostat(lv(), static_cast<float*>(s->output_probs->device_ptr()), s->model->get_header().vocab_size, log, config,
                            static_cast<u32*>(s->sampler_state->device_ptr()), -1.0f, log, max_backlog_size + 1,
                            static_cast<u32*>(s->argmax_result->device_ptr()) + 1, s->pinned + max_backlog_size + 5, nullptr));
}

bool llava_command_buffer::record_execution() {
    if (graph) return false;
    llava_session* s = session;
    llava_context* c = s->ctx;
    const ggml_header& h = s->model->get_header();
    if (!expect(s->get_layer_data().size() == c->get_layers().size(), "one layer data per layer")) return false;
    if (lv_graph_begin_capture(lv()) != LV_OK) {
        note(LV_ERR_CUDA);
        return false;
    }
    u32* config = static_cast<u32*>(s->config_buffer->device_ptr());
    u32* log = static_cast<u32*>(s->token_log->device_ptr());
    if (batch_size == 1 && s->step_plan != nullptr && !s->is_tracing_enabled()) {
        // a single token: the whole list below as one persistent kernel
        note(lv_decode_step(lv(), s->step_plan, config, log, max_backlog_size + 1, static_cast<float*>(s->output_probs->device_ptr()),
                            static_cast<u32*>(s->argmax_result->device_ptr()), s->pinned + max_backlog_size + 4, with_head ? 1 : 0));
        if (sample) record_sampler();
        lv_graph* g1 = nullptr;
        note(lv_graph_end_capture(lv(), &g1));
        if (first_error != LV_OK) {
            lv_graph_destroy(g1);
            return false;
        }
        graph = g1;
        return true;
    }
    // embedding rows of the tokens at positions config.token_count .. + batch (the reference
    // dequantises them on the host, llava_session.cpp:219-223)
    note(lv_dequant_rows(lv(), static_cast<float*>(s->current_thought->device_ptr()), c->tok_embeddings->device_ptr(),
                         c->tok_embeddings->kernel_type(), log, config, h.dim, h.vocab_size, batch_size));
    llava_buffer* current = s->current_thought;
    for (u32 i = 0; i < c->get_layers().size(); ++i) current = c->get_layers()[i]->execute(this, s->get_layer_data()[i], current);
    if (with_head) {
        // final norm + output matrix on the last row only (llava_command_buffer.cpp:38-39; the
        // reference computes every row and reads the last, llava_session.cpp:129-135)
        const float* last = static_cast<const float*>(current->device_ptr()) + size_t(batch_size - 1) * h.dim;
        float* logits = static_cast<float*>(s->output_probs->device_ptr());
        // sharded with fused exchanges: the last layer's w2 pushed its partial rows; the head's
        // normalisation takes residual + the ranks' sum
        if (c->tp_size() > 1 && c->fused_exchange() && !use_tensor_cores(c->get_layers()[0]->wq()))
            tp_arm_pull(2 * u32(c->get_layers().size()) - 1, h.dim, current == s->current_thought ? s->current_thought_sublayer : s->current_thought);
        note(lv_norm_gemv(lv(), logits, c->output_w->device_ptr(), c->output_w->kernel_type(), last,
                          static_cast<const float*>(c->norm_w->device_ptr()), h.vocab_size, h.dim, 1));
        // greedy choice, token log and position word in one launch; the kernel stores the token
        // into the pinned staging word itself
        u32* am = static_cast<u32*>(s->argmax_result->device_ptr());
        note(lv_argmax_advance(lv(), logits, h.vocab_size, config, log, batch_size, max_backlog_size + 1, am,
                               s->pinned + max_backlog_size + 4));
        if (sample) record_sampler();
    } else {
        // leading chunk of a prompt: only the position advances
        note(lv_decode_advance(lv(), config, nullptr, nullptr, batch_size, 0));
    }
    lv_graph* g = nullptr;
    const int rc = lv_graph_end_capture(lv(), &g);
    note(rc);
    if (first_error != LV_OK) {
        lv_graph_destroy(g);
        return false;
    }
    graph = g;
    return true;
}

static inline float* f32(llava_buffer* b) { return static_cast<float*>(b->device_ptr()); }

void llava_command_buffer::normalize_logit(llava_buffer* outbuf, llava_buffer* inbuf, llava_buffer* weights) {
    if (!expect(outbuf->shape.first == inbuf->shape.first && weights->shape.first == inbuf->shape.first, "normalize shapes")) return;
    note(lv_norm_f32(lv(), f32(outbuf), f32(inbuf), f32(weights), inbuf->shape.first, batch_size));
}

void llava_command_buffer::matmul(llava_buffer* outbuf, llava_buffer* matrix, llava_buffer* inbuf) {
    if (!expect(inbuf->shape.first == matrix->shape.second && outbuf->shape.first == matrix->shape.first &&
                inbuf->shape.second >= batch_size && outbuf->shape.second >= batch_size, "matmul shapes")) return;
    note(lv_gemv(lv(), f32(outbuf), matrix->device_ptr(), matrix->kernel_type(), f32(inbuf), matrix->shape.first, matrix->shape.second, batch_size, 0));
}

void llava_command_buffer::matmul_add_inplace(llava_buffer* outbuf, llava_buffer* matrix, llava_buffer* inbuf) {
    if (!expect(inbuf->shape.first == matrix->shape.second && outbuf->shape.first == matrix->shape.first &&
                inbuf->shape.second >= batch_size && outbuf->shape.second >= batch_size, "matmul_add shapes")) return;
    note(lv_gemv(lv(), f32(outbuf), matrix->device_ptr(), matrix->kernel_type(), f32(inbuf), matrix->shape.first, matrix->shape.second, batch_size, 1));
}

void llava_command_buffer::matmul_silu_ff(llava_buffer* outbuf, llava_buffer* w3, llava_buffer* w1, llava_buffer* inbuf) {
    if (!expect(w3->shape == w1->shape && w3->type == w1->type && inbuf->shape.first == w3->shape.second &&
                outbuf->shape.first == w3->shape.first, "matmul_silu_ff shapes")) return;
    note(lv_gemv_silu(lv(), f32(outbuf), w3->device_ptr(), w1->device_ptr(), w3->kernel_type(), f32(inbuf), w3->shape.first, w3->shape.second, batch_size));
}

void llava_command_buffer::kv_copy(llava_buffer* cache, llava_buffer* line) {
    const u32 dim = session->model->get_header().dim;
    if (!expect(cache->shape.second == dim && line->shape.first == dim && cache->shape.first >= backlog_size, "kv_copy shapes")) return;
    note(lv_kv_append_f16(lv(), cache->device_ptr(), f32(line), static_cast<u32*>(session->config_buffer->device_ptr()), dim,
                          batch_size, cache->shape.first));
}

void llava_command_buffer::copy_logit(llava_buffer* out, llava_buffer* in) {
    const u32 dim = session->model->get_header().dim;
    if (!expect(out->shape.first == dim && in->shape.first == dim, "copy shapes")) return;
    note(lv_copy_f32(lv(), f32(out), f32(in), size_t(dim) * batch_size));
}

void llava_command_buffer::multi_head_attention(llava_buffer* attn_out, llava_buffer* k_cache, llava_buffer* query) {
    const ggml_header& h = session->model->get_header();
    if (!expect(k_cache->shape.second == h.dim && query->shape.first == h.dim && attn_out->shape.first == backlog_size &&
                attn_out->shape.second >= h.n_heads * batch_size, "mhsa shapes")) return;
    note(lv_attn_scores_rope(lv(), f32(attn_out), k_cache->device_ptr(), f32(query), static_cast<u32*>(session->config_buffer->device_ptr()),
                             session->ctx->rope_table, backlog_size, h.n_heads, h.rot, batch_size));
}

void llava_command_buffer::inplace_softmax(llava_buffer* buf) {
    const ggml_header& h = session->model->get_header();
    if (!expect(buf->shape.first == backlog_size && buf->shape.second >= h.n_heads * batch_size, "softmax shapes")) return;
    note(lv_softmax_masked(lv(), f32(buf), static_cast<u32*>(session->config_buffer->device_ptr()), backlog_size, h.n_heads, h.rot, batch_size));
}

void llava_command_buffer::perform_kqv_matching(llava_buffer* v_out, llava_buffer* v_cache, llava_buffer* softmax_out) {
    const ggml_header& h = session->model->get_header();
    if (!expect(v_out && v_cache && softmax_out && v_out->shape.first == h.dim && v_cache->shape.second == h.dim &&
                softmax_out->shape.first == backlog_size, "kqv shapes")) return;
    note(lv_attn_values(lv(), f32(v_out), v_cache->device_ptr(), f32(softmax_out), backlog_size, h.n_heads, h.rot, batch_size));
}

void llava_command_buffer::norm_qkv_kvappend(llava_buffer* q_out, llava_buffer* k_cache, llava_buffer* v_cache, llava_buffer* wq,
                                             llava_buffer* wk, llava_buffer* wv, llava_buffer* inbuf, llava_buffer* norm_weights) {
    const u32 dim = session->model->get_header().dim;
    if (!expect(wq->shape == wk->shape && wq->shape == wv->shape && wq->shape.second == dim && inbuf->shape.first == dim &&
                q_out->shape.first == wq->shape.first && k_cache->shape.second == wq->shape.first &&
                v_cache->shape.second == wq->shape.first, "qkv shapes")) return;
    note(lv_norm_qkv_kvappend(lv(), f32(q_out), k_cache->device_ptr(), v_cache->device_ptr(), wq->device_ptr(), wk->device_ptr(),
                              wv->device_ptr(), wq->kernel_type(), f32(inbuf), f32(norm_weights),
                              static_cast<u32*>(session->config_buffer->device_ptr()), wq->shape.first, dim, batch_size,
                              k_cache->shape.first));
}

void llava_command_buffer::attention_fused(llava_buffer* v_out, llava_buffer* query, llava_buffer* k_cache, llava_buffer* v_cache) {
    const ggml_header& h = session->model->get_header();
    const u32 local_heads = h.n_heads / session->ctx->tp_size();
    if (!expect(query->shape.first == local_heads * h.rot && v_out->shape.first >= local_heads * h.rot &&
                k_cache->shape.second == local_heads * h.rot, "attention shapes")) return;
    // the grid covers the current backlog only; a step is re-recorded when the backlog
    // doubles, like the reference re-specialises its pipelines (llava_session.cpp:303-327)
    note(lv_attention_fused(lv(), f32(v_out), f32(query), k_cache->device_ptr(), v_cache->device_ptr(),
                            static_cast<u32*>(session->config_buffer->device_ptr()), session->ctx->rope_table,
                            session->attn_scratch->device_ptr(), local_heads, h.rot, backlog_size, batch_size));
}

void llava_command_buffer::allreduce_add(llava_buffer* residual, llava_buffer* partial) {
    const u32 dim = session->model->get_header().dim;
    if (!expect(residual->shape.first == dim && partial->shape.first == dim, "allreduce shapes")) return;
    // one kernel over NVLink peer memory when the ranks have connected their windows, else NCCL + add
    note(lv_allreduce_add_f32(lv(), f32(residual), f32(partial), size_t(dim) * batch_size));
}

bool llava_command_buffer::use_tensor_cores(const llava_buffer* matrix) const {
    // from six tokens on one pass over the matrix on the tensor cores beats one GEMV per token
    // (4096x4096 q4_0: 17 us flat against 4.3 us per token)
    // sharded: the rank's rows of wq / wk / wv must fill 128-row tiles and its rows of w3 / w1 64-row halves
    return batch_size >= kTensorCoreMinBatch && batch_size <= 64 && matrix->weight_buffer_is_f16() &&        // v3 blocks only
           session->act_split != nullptr && session->tensor_core_shapes_ok();
}

void llava_command_buffer::act_split(llava_buffer* split, llava_buffer* inbuf, llava_buffer* norm_weights, u32 cols_used, u32 cols) {
    if (cols_used == 0) cols_used = cols = inbuf->shape.first;
    if (!expect(size_t(split->shape.first) * 4 >= lv_act_split_bytes(cols, batch_size) && cols_used <= inbuf->shape.first, "act_split shapes")) return;
    note(lv_act_split_f16_padded(lv(), split->device_ptr(), f32(inbuf), norm_weights ? f32(norm_weights) : nullptr, cols_used, cols, batch_size));
}

void llava_command_buffer::gemm(llava_buffer* outbuf, llava_buffer* matrix, llava_buffer* split) {
    if (!expect(outbuf->shape.first == matrix->shape.first, "gemm shapes")) return;
    note(lv_gemm_tc(lv(), f32(outbuf), matrix->device_ptr(), matrix->kernel_type(), split->device_ptr(), matrix->shape.first,
                    matrix->shape.second, batch_size, 0));
}

void llava_command_buffer::gemm_qkv_kvappend(llava_buffer* q_out, llava_buffer* k_cache, llava_buffer* v_cache, llava_buffer* wq,
                                             llava_buffer* wk, llava_buffer* wv, llava_buffer* split) {
    const u32 dim = session->model->get_header().dim;
    if (!expect(wq->shape == wk->shape && wq->shape == wv->shape && wq->shape.second == dim && q_out->shape.first == wq->shape.first &&
                k_cache->shape.second == wq->shape.first && v_cache->shape.second == wq->shape.first, "qkv shapes")) return;
    note(lv_gemm_tc_qkv_kvappend(lv(), f32(q_out), k_cache->device_ptr(), v_cache->device_ptr(), wq->device_ptr(), wk->device_ptr(),
                                 wv->device_ptr(), wq->kernel_type(), split->device_ptr(),
                                 static_cast<u32*>(session->config_buffer->device_ptr()), wq->shape.first, dim, batch_size,
                                 k_cache->shape.first));
}

void llava_command_buffer::gemm_add_inplace(llava_buffer* outbuf, llava_buffer* matrix, llava_buffer* split) {
    if (!expect(outbuf->shape.first == matrix->shape.first, "gemm_add_inplace shapes")) return;
    note(lv_gemm_tc(lv(), f32(outbuf), matrix->device_ptr(), matrix->kernel_type(), split->device_ptr(), matrix->shape.first,
                    matrix->shape.second, batch_size, 1));
}

void llava_command_buffer::gemm_silu_ff(llava_buffer* outbuf, llava_buffer* w3, llava_buffer* w1, llava_buffer* split) {
    if (!expect(w3->shape == w1->shape && w3->type == w1->type && outbuf->shape.first >= w3->shape.first, "gemm_silu_ff shapes")) return;
    note(lv_gemm_tc_silu(lv(), f32(outbuf), w3->device_ptr(), w1->device_ptr(), w3->kernel_type(), split->device_ptr(), w3->shape.first,
                         w3->shape.second, batch_size));
}

void llava_command_buffer::tp_arm_push(u32 exchange) {
    note(lv_tp_arm_push(lv(), int(exchange), 2 * u32(session->ctx->get_layers().size())));
}

void llava_command_buffer::tp_arm_pull(u32 exchange, u32 producer_rows, llava_buffer* x_out) {
    note(lv_tp_arm_pull(lv(), int(exchange), 2 * u32(session->ctx->get_layers().size()), producer_rows, f32(x_out)));
}

void llava_command_buffer::norm_matmul_silu_ff(llava_buffer* outbuf, llava_buffer* w3, llava_buffer* w1, llava_buffer* inbuf,
                                               llava_buffer* norm_weights) {
    if (!expect(w3->shape == w1->shape && w3->type == w1->type && inbuf->shape.first == w3->shape.second &&
                outbuf->shape.first >= w3->shape.first, "norm_matmul_silu_ff shapes")) return;
    note(lv_norm_gate_up_silu(lv(), f32(outbuf), w3->device_ptr(), w1->device_ptr(), w3->kernel_type(), f32(inbuf), f32(norm_weights),
                              w3->shape.first, w3->shape.second, batch_size));
}
