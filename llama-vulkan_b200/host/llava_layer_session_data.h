// Per-session, per-layer device state: the f16 K and V caches and, when
// tracing is on, the six intermediate buffers that make up a trace frame
// (llava_layer_session_data.h:17-44 of the reference).
#ifndef LLAVA_B200_LAYER_SESSION_DATA_H
#define LLAVA_B200_LAYER_SESSION_DATA_H

#include <string>

#include "types.h"

class llava_layer_session_data {
    friend class llava_layer;
public:
    explicit llava_layer_session_data(llava_session* session);
    ~llava_layer_session_data();
    llava_layer_session_data(const llava_layer_session_data&) = delete;
    llava_layer_session_data& operator=(const llava_layer_session_data&) = delete;

    void dump_tracing_layers(int out_fd, const std::string& name);
    // (Re)creates the trace buffers when tracing or the batch size changed; the
    // caches are allocated once for the maximum context and survive.
    bool flush_buffers_on_gpu();
    bool dump_kv_cache(u8* dst, u32 token_count);
    bool restore_kv_cache(const u8* src, u32 token_count);
    llava_buffer* get_k_cache() const { return k_cache; }
    llava_buffer* get_v_cache() const { return v_cache; }

    llava_session* const session;

private:
    llava_device_memory* cache_allocation = nullptr;
    llava_buffer* k_cache = nullptr;        // f16 [max_backlog][dim], un-rotated keys
    llava_buffer* v_cache = nullptr;

    llava_device_memory* trace_allocation = nullptr;
    llava_buffer* attn_result = nullptr;
    llava_buffer* ff_result = nullptr;
    llava_buffer* normalized_input_logit = nullptr;
    llava_buffer* post_attn_logit = nullptr;
    llava_buffer* output_logit = nullptr;
    llava_buffer* post_attn_norm_logit = nullptr;
    u32 trace_batch = 0, trace_backlog = 0;
    void drop_trace_buffers();
};

#endif
