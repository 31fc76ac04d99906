// One transformer layer: seven quantised matrices and two norm vectors
// (llava_layer.h:8-15, llava_layer.cpp:10-23 of the reference), placed in the
// context's weight arena.
#ifndef LLAVA_B200_LAYER_H
#define LLAVA_B200_LAYER_H

#include "types.h"

class llava_layer {
public:
    llava_layer(llava_context* context, u32 layer_id);
    ~llava_layer();
    llava_layer(const llava_layer&) = delete;
    llava_layer& operator=(const llava_layer&) = delete;

    // Records the layer's operations on cmd_buf; returns the buffer that holds
    // the layer output (llava_layer.cpp:39-75).
    llava_buffer* execute(llava_command_buffer* cmd_buf, llava_layer_session_data* layer_data, llava_buffer* raw_input_logit) const;
    bool freeze_storage();
    bool load_to_gpu();
    bool is_valid() const { return valid; }

    u32 const layer_id;
    llava_context* const context;

    // the tensors, for code that addresses a whole step at once (llava_session's step plan)
    const llava_buffer* wq() const { return attention_wq; }
    const llava_buffer* wk() const { return attention_wk; }
    const llava_buffer* wv() const { return attention_wv; }
    const llava_buffer* wo() const { return attention_wo; }
    const llava_buffer* w1() const { return feed_forward_w1; }
    const llava_buffer* w2() const { return feed_forward_w2; }
    const llava_buffer* w3() const { return feed_forward_w3; }
    const llava_buffer* attn_norm() const { return attention_norm; }
    const llava_buffer* ff_norm() const { return ffn_norm; }

private:
    llava_device_memory* layer_allocation = nullptr;     // the context's weight arena (not owned)
    llava_buffer* attention_wq = nullptr;
    llava_buffer* attention_wk = nullptr;
    llava_buffer* attention_wv = nullptr;
    llava_buffer* attention_wo = nullptr;
    llava_buffer* feed_forward_w1 = nullptr;
    llava_buffer* feed_forward_w2 = nullptr;
    llava_buffer* feed_forward_w3 = nullptr;
    llava_buffer* attention_norm = nullptr;
    llava_buffer* ffn_norm = nullptr;
    bool valid = false;
};

#endif
