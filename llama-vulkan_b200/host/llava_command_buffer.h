// Recorder of one evaluation step.  The reference records ~418 Vulkan command
// buffers with events between them and submits them with one fence
// (llava_command_buffer.cpp:29-55,196-280); here every op method enqueues one
// kernel through the C ABI while the context's stream is being captured, and
// the result is a CUDA graph that run() replays.
#ifndef LLAVA_B200_COMMAND_BUFFER_H
#define LLAVA_B200_COMMAND_BUFFER_H

#include "../../include/lv_b200.h"
#include "types.h"

class llava_command_buffer {
public:
    // with_head: record the final norm + output matrix + argmax (not needed for
    // the leading chunks of a long prompt)
    // sample: after the head, draw the next token on the device (the reference's sampler) as part of the step
    llava_command_buffer(llava_session* session, u32 batch_size, bool with_head, bool sample = false);
    ~llava_command_buffer();
    llava_command_buffer(const llava_command_buffer&) = delete;
    llava_command_buffer& operator=(const llava_command_buffer&) = delete;

    bool record_execution();
    bool run();
    bool wait_idle() const;
    u32 kernel_launches() const;       // kernel nodes of the recorded graph
    void record_sampler();

    // the reference's op set (llava_command_buffer.h:30-38)
    void normalize_logit(llava_buffer* outbuf, llava_buffer* inbuf, llava_buffer* weights);
    void matmul(llava_buffer* outbuf, llava_buffer* matrix, llava_buffer* inbuf);
    void matmul_add_inplace(llava_buffer* outbuf, llava_buffer* matrix, llava_buffer* inbuf);
    void kv_copy(llava_buffer* cache, llava_buffer* line);
    void copy_logit(llava_buffer* out, llava_buffer* in);
    void multi_head_attention(llava_buffer* attn_out, llava_buffer* k_cache, llava_buffer* query);
    void perform_kqv_matching(llava_buffer* v_out, llava_buffer* v_cache, llava_buffer* softmax_out);
    void inplace_softmax(llava_buffer* buf);
    void matmul_silu_ff(llava_buffer* outbuf, llava_buffer* w3_matrix, llava_buffer* w1_matrix, llava_buffer* inbuf);
    // fused forms used when tracing is off
    void norm_qkv_kvappend(llava_buffer* q_out, llava_buffer* k_cache, llava_buffer* v_cache, llava_buffer* wq,
                           llava_buffer* wk, llava_buffer* wv, llava_buffer* inbuf, llava_buffer* norm_weights);
    void attention_fused(llava_buffer* v_out, llava_buffer* query, llava_buffer* k_cache, llava_buffer* v_cache);
    void norm_matmul_silu_ff(llava_buffer* outbuf, llava_buffer* w3_matrix, llava_buffer* w1_matrix, llava_buffer* inbuf,
                             llava_buffer* norm_weights);

    // tensor-parallel: partial <- sum over ranks of partial; residual += partial
    void allreduce_add(llava_buffer* residual, llava_buffer* partial);
    // exchange fused into the neighbouring GEMVs (lv_tp_arm_push / lv_tp_arm_pull): the next matmul
    // pushes its rows to all ranks; the next normalising matmul takes inbuf + the ranks' sum as its
    // input and leaves that sum in x_out
    void tp_arm_push(u32 exchange);
    void tp_arm_pull(u32 exchange, u32 producer_rows, llava_buffer* x_out);
    static constexpr u32 kTensorCoreMinBatch = 6;
    // batched forms on the tensor cores (6..64 tokens per step): the activations are first
    // split into two fp16 planes (optionally normalised), then every matrix is read once
    bool use_tensor_cores(const llava_buffer* matrix) const;
    // cols_used != 0: the rows of inbuf are dense with cols_used values and meet a matrix of `cols` (padded) columns
    void act_split(llava_buffer* split, llava_buffer* inbuf, llava_buffer* norm_weights, u32 cols_used = 0, u32 cols = 0);
    void gemm(llava_buffer* outbuf, llava_buffer* matrix, llava_buffer* split);          // store, no residual
    void gemm_qkv_kvappend(llava_buffer* q_out, llava_buffer* k_cache, llava_buffer* v_cache, llava_buffer* wq, llava_buffer* wk,
                           llava_buffer* wv, llava_buffer* split);
    void gemm_add_inplace(llava_buffer* outbuf, llava_buffer* matrix, llava_buffer* split);
    void gemm_silu_ff(llava_buffer* outbuf, llava_buffer* w3_matrix, llava_buffer* w1_matrix, llava_buffer* split);

    int status() const { return first_error; }

    llava_session* const session;
    u32 const backlog_size;
    u32 const workgroup_size;
    u32 const batch_size;
    bool const with_head;
    bool const sample;

private:
    void note(int rc);
    bool expect(bool cond, const char* what);
    lv_ctx* lv() const;
    lv_graph* graph = nullptr;
    int first_error = LV_OK;
};

#endif
