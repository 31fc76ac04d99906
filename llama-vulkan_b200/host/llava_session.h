// One generation session: token buffer, KV caches, scratch buffers and the
// recorded evaluation step.  Public surface of the reference's llava_session
// (llava_session.h:44-62) plus the switches its CLI lacks (greedy decoding,
// seeding, decoding without the host in the loop).
#ifndef LLAVA_B200_SESSION_H
#define LLAVA_B200_SESSION_H

#include <map>
#include <random>
#include <string>
#include <vector>

#include "../../include/lv_b200.h"
#include "ggml_file.h"
#include "types.h"

const u32 min_backlog_size = 128;     // llava_session.cpp:23
const u32 max_backlog_size = 2048;    // llava_session.cpp:24

class llava_session {
    friend class llava_layer;
    friend class llava_layer_session_data;
    friend class llava_command_buffer;
    friend class llava_session_group;
public:
    explicit llava_session(llava_context* ctx);
    ~llava_session();
    llava_session(const llava_session&) = delete;
    llava_session& operator=(const llava_session&) = delete;

    const std::vector<llava_layer_session_data*>& get_layer_data() const { return layer_data; }
    bool set_text(const std::string& new_text);
    u32 get_token_count() const { return u32(token_buffer.size()); }
    const std::vector<u32>& get_token_buffer() const { return token_buffer; }
    bool push_token(u32 token);
    u32 predict_next_token();                   // ~0U on failure
    bool start_next_token_prediction();
    u32 finish_next_token_prediction();
    bool is_tracing_enabled() const { return options != 0; }
    void rewind(u32 n);
    ReturnCode set_options(u32 new_options);
    ReturnCode save_frame(const std::string& path);
    ReturnCode snapshot(const std::string& path);
    ReturnCode restore(const std::string& path);
    bool add_text(const std::string& s);

    // ---- additions --------------------------------------------------------------
    // true: finish_next_token_prediction returns the first index of the largest
    // logit (the argmax branch of the reference's get_last_predicted_token, which
    // its own callers never select); false: the reference's sampler.
    void set_deterministic(bool on) { deterministic = on; }
    void set_seed(u32 seed);
    // false (default): non-greedy tokens are drawn on the device (lv_sample_mirostat: 4 bytes come back instead of the
    // 128 KB of logits); true: on the host, with std::discrete_distribution over std::mt19937 as the reference does
    void set_host_sampler(bool on);
    float get_mirostat_mu();
    // tokens evaluated per recorded step while a prompt is ingested (1 ..
    // max_batch_limit); the reference evaluates the whole prompt as one batch
    bool set_max_batch(u32 n);
    // whether the batched (tensor-core) products can take this context's matrices: always on one GPU; sharded, the
    // rank's rows of wq / wk / wv must fill 128-row tiles and its rows of w3 / w1 64-row halves
    bool tensor_core_shapes_ok() const;
    // Greedy decoding of n tokens with no host round trip between tokens: the
    // recorded step feeds its own argmax back in.  Requires every token pushed
    // so far to be evaluated except the last one.  Appends to the token buffer.
    bool generate_greedy_on_device(u32 n, std::vector<u32>* out);
    // The two halves of generate_greedy_on_device, for callers that time the
    // device work themselves: enqueue returns as soon as the n steps are queued,
    // collect waits for them and appends the n tokens.
    bool enqueue_greedy_on_device(u32 n);
    bool collect_greedy_on_device(std::vector<u32>* out);
    // logits of the last evaluated token (vocab floats)
    bool get_logits(std::vector<float>* out);
    u32 get_backlog_size() const { return backlog_size; }
    u32 get_tokens_in_gpu() const { return current_tokens_in_gpu; }
    // timeline of the one-launch token step (lv_step_plan_set_trace); false when the session has no such step
    bool set_step_trace(bool on);
    bool read_step_trace(std::vector<u64>* out, u32* n_ops, u32* n_ctas, u32* n_points);
    u32 step_kernel_launches() const;          // kernel launches of one replay of the step evaluated last

    static constexpr u32 max_batch_limit = 64;

    llava_context* const ctx;
    ggml_file const* const model;

private:
    std::mt19937 rng;
    // sampler constants, llava_session.h:70-76
    const u32 repeat_last_n = 64;
    const float repeat_penalty = 1.1f;
    const float alpha_frequency = 0.1f;
    const float alpha_presence = 0.0f;
    const float temp = 0.8f;
    const float mirostat_tau = 5.0f;
    const float mirostat_eta = 0.1f;
    float mirostat_mu;
    bool deterministic = false;
    bool host_sampler = false;
    u32 sampler_seed;
    bool sampler_state_dirty = true;          // mu / seed on the host are newer than the device copy

    // scratch buffers, named as in the reference (llava_session.h:80-94); second dimension = max_batch
    llava_device_memory* main_buffer_memory = nullptr;
    llava_buffer* current_thought = nullptr;
    llava_buffer* current_thought_sublayer = nullptr;
    llava_buffer* current_thought_middle_normd = nullptr;
    llava_buffer* current_Q = nullptr;
    llava_buffer* current_K = nullptr;
    llava_buffer* current_V = nullptr;
    llava_buffer* current_Vout = nullptr;
    llava_buffer* main_attn_result = nullptr;     // only when tracing (separate attention ops)
    llava_buffer* config_buffer = nullptr;        // u32 x4: tokens already in the cache
    llava_buffer* output_probs = nullptr;         // raw logits of the last row, despite the name
    llava_buffer* main_ff_result = nullptr;
    // additions: device copy of the token buffer, argmax result, attention scratch
    llava_buffer* token_log = nullptr;
    llava_buffer* argmax_result = nullptr;
    llava_buffer* attn_scratch = nullptr;
    llava_buffer* sampler_state = nullptr;        // device sampler: {mu, seed, draws, -}
    llava_buffer* act_split = nullptr;            // max_batch >= 6: fp16 (hi, lo) planes of a batch of activations
    llava_buffer* tp_partial = nullptr;           // tensor-parallel only: this rank's partial wo / w2 product
    std::vector<llava_layer_session_data*> layer_data;

    u32 batch_size = 0;           // batch of the step recorded last
    u32 max_batch = 1;
    u32 backlog_size;
    u32 get_last_predicted_token(bool deterministic);
    u32 sample_from_logits(std::vector<float>& logits);

    void reset_main_buffers();
    bool recreate_buffers();
    bool set_backlog_size(u32 new_size);
    bool ensure_buffers_created();
    void drop_command_buffers();
    llava_command_buffer* get_command_buffer(u32 batch, bool with_head);
    bool sampling_on_device() const { return !deterministic && !host_sampler; }
public:
    bool samples_on_host() const { return !deterministic && host_sampler; }
private:
    bool upload_sampler_state();

    // key: batch | with_head << 16 | device sampler << 17
    std::map<u32, llava_command_buffer*> command_buffers;
    llava_command_buffer* last_command_buffer = nullptr;

    std::vector<u32> token_buffer;
    u32 current_tokens_in_gpu = 0;
    u32 device_pos = ~0U;         // value of config_buffer on the device as far as the host knows
    u32* pinned = nullptr;        // [max_backlog] token staging + [8] config/argmax words
    bool upload_pending_tokens(u32 first, u32 count);
    bool sync_device_position(u32 pos);

    // one-launch token step (lv_decode_step): weights of the context + caches of this session; null when
    // the session cannot use it (sharded contexts) or LV_DECODE_STEP=0 asks for one kernel per operation
    lv_step_plan* step_plan = nullptr;
    bool step_plan_tried = false;
    void ensure_step_plan();

    u32 enqueued_greedy = 0;      // steps queued by enqueue_greedy_on_device and not yet collected
    u32 options = 0;              // non-zero: tracing
    bool flush_layers_data_buffers();
    bool failed = false;
};

#endif
