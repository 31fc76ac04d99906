#include "llava_layer.h"

#include <iostream>

#include "llava_buffer.h"
#include "llava_command_buffer.h"
#include "llava_context.h"
#include "llava_device_memory.h"
#include "llava_layer_session_data.h"
#include "llava_session.h"

using namespace std;

llava_layer::llava_layer(llava_context* _context, u32 _layer_id) : layer_id(_layer_id), context(_context) {
    // every layer's tensors go into the context's one weight arena (the reference gives each layer a
    // device memory of its own, llava_layer.cpp:10-12); see llava_buffer.cpp for why
    layer_allocation = context->weights_memory();
    const ggml_file* model = context->get_model();
    const string prefix = "layers." + to_string(layer_id) + ".";
    bool ok = true;
    const u32 rank = context->tp_rank(), n_ranks = context->tp_size();
    auto make = [&](const char* leaf, tp_split how) -> llava_buffer* {
        const ggml_data_descriptor* d = model->find_buffer_descriptor(prefix + leaf);
        if (!d) {
            cerr << "[!] tensor " << prefix << leaf << " missing" << endl;
            ok = false;
            return nullptr;
        }
        if (n_ranks == 1 || how == tp_split::none) return new llava_buffer(context, *d, layer_allocation);
        auto* b = new llava_buffer(context, *d, layer_allocation, how, rank, n_ranks);
        if (b->byte_size() == 0) {
            cerr << "[!] tensor " << prefix << leaf << " cannot be split over " << n_ranks << " ranks" << endl;
            ok = false;
        }
        return b;
    };
    // Megatron-style split: output features of wq/wk/wv/w1/w3, input features of wo/w2
    attention_wq = make("attention.wq", tp_split::rows);
    attention_wk = make("attention.wk", tp_split::rows);
    attention_wv = make("attention.wv", tp_split::rows);
    attention_wo = make("attention.wo", tp_split::columns);
    feed_forward_w1 = make("feed_forward.w1", tp_split::rows);
    feed_forward_w2 = make("feed_forward.w2", tp_split::columns);
    feed_forward_w3 = make("feed_forward.w3", tp_split::rows);
    attention_norm = make("attention_norm", tp_split::none);
    ffn_norm = make("ffn_norm", tp_split::none);
    if (ok) {
        // norms must be f32 vectors, matrices q4_0 / q8_0 blocks of ggjt v3 or q4_0 blocks of ggjt v1 (the combinations
        // the reference loads, llava_buffer.cpp:63-99), all of one kind
        for (llava_buffer* m : {attention_wq, attention_wk, attention_wv, attention_wo, feed_forward_w1, feed_forward_w2, feed_forward_w3})
            ok = ok && m->weight_buffer_is_quantised() && m->kernel_type() == attention_wq->kernel_type();
        if (n_ranks > 1) ok = ok && attention_wq->weight_buffer_is_f16();      // shards are packed in v3 blocks only
        ok = ok && attention_norm->type == ggml_value_type::f32 && ffn_norm->type == ggml_value_type::f32;
        if (!ok) cerr << "[!] layer " << layer_id << ": unsupported tensor types (need q4_0/q8_0 ggjt v3 or q4_0 ggjt v1 matrices, f32 norms)" << endl;
    }
    valid = ok;
}

llava_layer::~llava_layer() {
    for (llava_buffer* b : {attention_wq, attention_wk, attention_wv, attention_wo, feed_forward_w1, feed_forward_w2,
                            feed_forward_w3, attention_norm, ffn_norm})
        delete b;
}

bool llava_layer::freeze_storage() { return valid && layer_allocation->is_frozen(); }     // the context froze the shared arena

bool llava_layer::load_to_gpu() {
    if (!valid) return false;
    for (llava_buffer* b : {attention_wq, attention_wk, attention_wv, attention_wo, feed_forward_w1, feed_forward_w2,
                            feed_forward_w3, attention_norm, ffn_norm})
        if (!b->load_to_gpu()) return false;
    return true;
}

llava_buffer* llava_layer::execute(llava_command_buffer* cmd_buf, llava_layer_session_data* layer_data,
                                   llava_buffer* raw_input_logit) const {
    llava_session* session = layer_data->session;
    const bool record = layer_data->attn_result != nullptr;

    if (!record) {
        // five launches: the residual stream is updated in place, as the reference does when
        // it is not tracing (llava_layer.cpp:45-51)
        llava_buffer* x = session->current_thought;
        if (cmd_buf->use_tensor_cores(attention_wq)) {
            // six or more tokens: every matrix is read once for the whole batch (tcgen05), nine launches
            llava_buffer* split = session->act_split;
            cmd_buf->act_split(split, x, attention_norm);
            cmd_buf->gemm_qkv_kvappend(session->current_Q, layer_data->k_cache, layer_data->v_cache, attention_wq, attention_wk,
                                       attention_wv, split);
            cmd_buf->attention_fused(session->current_Vout, session->current_Q, layer_data->k_cache, layer_data->v_cache);
            if (context->tp_size() > 1) {
                // this rank's heads and FFN rows; the column shards of wo and w2 have rows padded with zero blocks, so
                // their (dense) inputs are padded while they are split; the partial products of all tokens are summed
                // over the ranks by one exchange per sub-block
                cmd_buf->act_split(split, session->current_Vout, nullptr, attention_wq->shape.first, attention_wo->shape.second);
                cmd_buf->gemm(session->tp_partial, attention_wo, split);
                cmd_buf->allreduce_add(x, session->tp_partial);
                cmd_buf->act_split(split, x, ffn_norm);
                cmd_buf->gemm_silu_ff(session->main_ff_result, feed_forward_w3, feed_forward_w1, split);
                cmd_buf->act_split(split, session->main_ff_result, nullptr, feed_forward_w3->shape.first, feed_forward_w2->shape.second);
                cmd_buf->gemm(session->tp_partial, feed_forward_w2, split);
                cmd_buf->allreduce_add(x, session->tp_partial);
                return x;
            }
            cmd_buf->act_split(split, session->current_Vout, nullptr);
            cmd_buf->gemm_add_inplace(x, attention_wo, split);
            cmd_buf->act_split(split, x, ffn_norm);
            cmd_buf->gemm_silu_ff(session->main_ff_result, feed_forward_w3, feed_forward_w1, split);
            cmd_buf->act_split(split, session->main_ff_result, nullptr);
            cmd_buf->gemm_add_inplace(x, feed_forward_w2, split);
            return x;
        }
        if (context->tp_size() > 1 && context->fused_exchange() && layer_id > 0) {
            // the previous layer's w2 pushed exchange 2l-1: input = xb + the ranks' rows, sum kept in xa
            cmd_buf->tp_arm_pull(2 * layer_id - 1, context->get_model()->get_header().dim, session->current_thought);
            cmd_buf->norm_qkv_kvappend(session->current_Q, layer_data->k_cache, layer_data->v_cache, attention_wq, attention_wk,
                                       attention_wv, session->current_thought_sublayer, attention_norm);
        } else {
            cmd_buf->norm_qkv_kvappend(session->current_Q, layer_data->k_cache, layer_data->v_cache, attention_wq, attention_wk,
                                       attention_wv, x, attention_norm);
        }
        cmd_buf->attention_fused(session->current_Vout, session->current_Q, layer_data->k_cache, layer_data->v_cache);
        if (context->tp_size() == 1) {
            cmd_buf->matmul_add_inplace(x, attention_wo, session->current_Vout);
            cmd_buf->norm_matmul_silu_ff(session->main_ff_result, feed_forward_w3, feed_forward_w1, x, ffn_norm);
            cmd_buf->matmul_add_inplace(x, feed_forward_w2, session->main_ff_result);
        } else if (context->fused_exchange()) {
            // every rank holds a column shard of wo and w2.  Their partial products travel inside the
            // GEMVs: wo / w2 push their rows into every rank's window, the next normalising GEMV adds
            // the ranks' rows to the residual stream on its way in and leaves the sum in the other of
            // the two residual buffers (xa = current_thought, xb = current_thought_sublayer).
            // Exchange 2l follows wo of layer l, exchange 2l+1 follows w2.
            llava_buffer* xa = session->current_thought;
            llava_buffer* xb = session->current_thought_sublayer;
            const u32 dim = context->get_model()->get_header().dim;
            const bool last = layer_id + 1 == context->get_layers().size();
            // (the QKV launch above already consumed exchange 2l-1 when l > 0: see below)
            cmd_buf->tp_arm_push(2 * layer_id);
            cmd_buf->matmul(session->tp_partial, attention_wo, session->current_Vout);
            cmd_buf->tp_arm_pull(2 * layer_id, dim, xb);
            cmd_buf->norm_matmul_silu_ff(session->main_ff_result, feed_forward_w3, feed_forward_w1, xa, ffn_norm);
            if (last && !cmd_buf->with_head) {
                // nothing consumes the last exchange of a step without a head: use the stand-alone kernel
                cmd_buf->matmul(session->tp_partial, feed_forward_w2, session->main_ff_result);
                cmd_buf->allreduce_add(xb, session->tp_partial);
            } else {
                cmd_buf->tp_arm_push(2 * layer_id + 1);
                cmd_buf->matmul(session->tp_partial, feed_forward_w2, session->main_ff_result);
            }
            return xb;
        } else {
            // every rank holds a column shard of wo and w2: partial products, summed over the
            // ranks, then added to the (replicated) residual stream
            cmd_buf->matmul(session->tp_partial, attention_wo, session->current_Vout);
            cmd_buf->allreduce_add(x, session->tp_partial);
            cmd_buf->norm_matmul_silu_ff(session->main_ff_result, feed_forward_w3, feed_forward_w1, x, ffn_norm);
            cmd_buf->matmul(session->tp_partial, feed_forward_w2, session->main_ff_result);
            cmd_buf->allreduce_add(x, session->tp_partial);
        }
        return x;
    }

    // tracing: the reference's thirteen operations, each intermediate kept in its record buffer
    llava_buffer* normd = layer_data->normalized_input_logit;
    llava_buffer* post_attn = layer_data->post_attn_logit;
    llava_buffer* post_attn_normd = layer_data->post_attn_norm_logit;
    llava_buffer* output = layer_data->output_logit;
    cmd_buf->normalize_logit(normd, raw_input_logit, attention_norm);
    cmd_buf->matmul(session->current_K, attention_wk, normd);
    cmd_buf->matmul(session->current_Q, attention_wq, normd);
    cmd_buf->matmul(session->current_V, attention_wv, normd);
    cmd_buf->kv_copy(layer_data->k_cache, session->current_K);
    cmd_buf->kv_copy(layer_data->v_cache, session->current_V);
    cmd_buf->multi_head_attention(layer_data->attn_result, layer_data->k_cache, session->current_Q);
    cmd_buf->inplace_softmax(layer_data->attn_result);
    cmd_buf->perform_kqv_matching(session->current_Vout, layer_data->v_cache, layer_data->attn_result);
    cmd_buf->copy_logit(post_attn, raw_input_logit);
    cmd_buf->matmul_add_inplace(post_attn, attention_wo, session->current_Vout);
    cmd_buf->normalize_logit(post_attn_normd, post_attn, ffn_norm);
    cmd_buf->matmul_silu_ff(layer_data->ff_result, feed_forward_w3, feed_forward_w1, post_attn_normd);
    cmd_buf->copy_logit(output, post_attn);
    cmd_buf->matmul_add_inplace(output, feed_forward_w2, layer_data->ff_result);
    return output;
}
