#include "llava_layer_session_data.h"

#include "llava_buffer.h"
#include "llava_context.h"
#include "llava_device_memory.h"
#include "llava_session.h"

using namespace std;

llava_layer_session_data::llava_layer_session_data(llava_session* _session) : session(_session) {
    const u32 dim = session->model->get_header().dim / session->ctx->tp_size();     // this rank's heads
    // both caches for the maximum context, zero filled (the reference zero-fills and regrows
    // them as the backlog doubles, llava_layer_session_data.cpp:100-127)
    cache_allocation = new llava_device_memory(session->ctx);
    k_cache = new llava_buffer(session->ctx, ggml_value_type::f16, max_backlog_size, dim, cache_allocation, "k_cache");
    v_cache = new llava_buffer(session->ctx, ggml_value_type::f16, max_backlog_size, dim, cache_allocation, "v_cache");
    if (cache_allocation->freeze()) cache_allocation->zero(0, cache_allocation->get_size());
    flush_buffers_on_gpu();
}

llava_layer_session_data::~llava_layer_session_data() {
    drop_trace_buffers();
    delete k_cache;
    delete v_cache;
    delete cache_allocation;
}

void llava_layer_session_data::drop_trace_buffers() {
    for (llava_buffer** b : {&attn_result, &ff_result, &normalized_input_logit, &post_attn_logit, &output_logit, &post_attn_norm_logit}) {
        delete *b;
        *b = nullptr;
    }
    delete trace_allocation;
    trace_allocation = nullptr;
    trace_batch = trace_backlog = 0;
}

bool llava_layer_session_data::flush_buffers_on_gpu() {
    const bool want = session->is_tracing_enabled() && session->max_batch != 0;
    const bool have = attn_result != nullptr;
    if (want == have && (!want || (trace_batch == session->max_batch && trace_backlog == session->backlog_size))) return true;
    drop_trace_buffers();
    if (!want) return true;
    const ggml_header& h = session->model->get_header();
    const u32 batch = session->max_batch, ff = session->model->get_ff_size();
    llava_context* c = session->ctx;
    trace_allocation = new llava_device_memory(c);
    const auto F = ggml_value_type::f32;
    // names and shapes of llava_layer_session_data.cpp:80-85
    attn_result = new llava_buffer(c, F, session->backlog_size, h.n_heads * batch, trace_allocation, "attn_result");
    ff_result = new llava_buffer(c, F, ff, batch, trace_allocation, "ff_result");
    normalized_input_logit = new llava_buffer(c, F, h.dim, batch, trace_allocation, "normalized_input_logit");
    post_attn_logit = new llava_buffer(c, F, h.dim, batch, trace_allocation, "post_attn_logit");
    post_attn_norm_logit = new llava_buffer(c, F, h.dim, batch, trace_allocation, "post_attn_norm_logit");
    output_logit = new llava_buffer(c, F, h.dim, batch, trace_allocation, "output_logit");
    trace_batch = batch;
    trace_backlog = session->backlog_size;
    return trace_allocation->freeze() && trace_allocation->zero(0, trace_allocation->get_size());
}

void llava_layer_session_data::dump_tracing_layers(int out_fd, const string& name) {
    if (trace_allocation) trace_allocation->dump_buffers(out_fd, name);
}

// The rows this rank holds: [token_count][dim / ranks] halves of K, then of V (the whole rows on one GPU).
bool llava_layer_session_data::dump_kv_cache(u8* dst, u32 token_count) {
    const size_t n = size_t(2) * (session->model->get_header().dim / session->ctx->tp_size()) * token_count;     // llava_layer_session_data.cpp:165-172
    return k_cache->read_raw(0, dst, n) && v_cache->read_raw(0, dst + n, n);
}

bool llava_layer_session_data::restore_kv_cache(const u8* src, u32 token_count) {
    const size_t n = size_t(2) * (session->model->get_header().dim / session->ctx->tp_size()) * token_count;     // llava_layer_session_data.cpp:174-181
    return k_cache->write_raw(0, src, n) && v_cache->write_raw(0, src + n, n);
}
