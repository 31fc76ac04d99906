/*
 * llava_host -- plain-C wrappers around the C++ host surface (ggml_file,
 * llava_context, llava_session, the synthetic model writer) so that tests,
 * benchmarks and other languages can drive it.  Each wrapper forwards to the
 * C++ method of the same name; the C++ classes keep the public methods of the
 * reference's classes (ggml_file.h:51-57, llava_session.h:44-62,
 * llava_context.h:21-42).  Handles are opaque; functions that return int use
 * 1 = success, 0 = failure unless stated otherwise; ReturnCode values are
 * those of types.h:45-55.
 */
#ifndef LLAVA_HOST_H
#define LLAVA_HOST_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- synthetic ggjt-v3 models (seeded N(0,0.02) weights; q4_0 = 2, q8_0 = 8) */
int      llava_synth_write(const char* path, uint32_t dim, uint32_t n_heads, uint32_t n_layers, uint32_t ff_size,
                           uint32_t vocab_size, int wtype, uint64_t seed, uint32_t threads);
/* the same with a file version (3, or 1: q4_0 blocks with f32 scales and interleaved nibbles, as old ggjt files have
 * them) and, optionally, tok_embeddings stored as f32 */
int      llava_synth_write_ex(const char* path, uint32_t dim, uint32_t n_heads, uint32_t n_layers, uint32_t ff_size,
                              uint32_t vocab_size, int wtype, uint64_t seed, uint32_t threads, uint32_t file_version,
                              int f32_embeddings);
void     llava_synth_quantize_v1(const float* src, size_t count, uint8_t* dst);
uint64_t llava_synth_file_size(uint32_t dim, uint32_t n_heads, uint32_t n_layers, uint32_t ff_size,
                               uint32_t vocab_size, int wtype);
float    llava_synth_normal(uint64_t seed, uint32_t tensor, uint64_t element);
void     llava_synth_quantize(const float* src, size_t count, int wtype, uint8_t* dst);

/* ---- ggml_file (ggml_file.h:51-57) */
void*    ggml_file_open(const char* path);                 /* NULL if the file cannot be parsed */
void     ggml_file_close(void* file);
void     ggml_file_header(void* file, uint32_t* out10);    /* nine header words, then ff_size */
uint32_t ggml_file_n_tensors(void* file);
int      ggml_file_tensor(void* file, uint32_t index, char* name, size_t name_cap, uint32_t* type, uint64_t* offset,
                          uint32_t* shape1, uint32_t* shape2, uint64_t* size);
int      ggml_file_find(void* file, const char* name, uint64_t* offset);      /* get_buffer_descriptor */
uint32_t ggml_file_tokenize(void* file, const char* text, size_t len, int bos, uint32_t* out, uint32_t cap);
uint32_t ggml_file_tokens_to_text(void* file, const uint32_t* tokens, uint32_t n, char* out, uint32_t cap);
uint32_t ggml_file_token(void* file, uint32_t id, char* out, uint32_t cap, float* score);
/* llava_buffer::write_f32 arithmetic on the host (llava_buffer.cpp:339-401) */
int      llava_dequantize(const void* in, int type, uint32_t model_version, float* out, uint32_t count);

/* ---- llava_context (llava_context.h:21-42) */
void*    llava_context_open(const char* model_path, int device);   /* NULL on failure */
/* the model file only (vocabulary, tensor table), no device: serves the front end's session-independent requests */
void*    llava_context_open_model_only(const char* model_path);
/* tensor-parallel: this process is rank `rank` of `n_ranks`, one GPU each; nccl_id = the 128 bytes
 * of lv_comm_unique_id made by rank 0 (ignored when n_ranks == 1) */
void*    llava_context_open_sharded(const char* model_path, int device, uint32_t rank, uint32_t n_ranks,
                                    const uint8_t* nccl_id);
/* peer-memory all-reduce between the ranks (see lv_peer_window_create in lv_b200.h): make this
 * rank's window and 64-byte handle, exchange the handles of all ranks, connect (rank order) */
int      llava_context_peer_window_create(void* ctx, uint8_t* handle64);
int      llava_context_peer_connect(void* ctx, const uint8_t* handles);
/* shard geometry and packing (host/tp_shard.h): how = 1 rows, 2 columns */
int      llava_tp_shape(int type, uint32_t rows, uint32_t cols, uint32_t how, uint32_t rank, uint32_t n_ranks,
                        uint32_t* out_rows, uint32_t* out_cols, uint32_t* out_cols_used, uint64_t* out_bytes);
int      llava_tp_pack(const uint8_t* src, int type, uint32_t rows, uint32_t cols, uint32_t how, uint32_t rank,
                       uint32_t n_ranks, uint8_t* dst);
void     llava_context_close(void* ctx);
void*    llava_context_lv(void* ctx);                               /* the lv_ctx* behind it */
int      llava_context_run(int argc, char** argv);                  /* the command-line tool */

/* ---- llava_session (llava_session.h:44-62) */
void*    llava_session_create(void* ctx);
void     llava_session_destroy(void* session);
int      llava_session_set_text(void* session, const char* text, size_t len);
int      llava_session_add_text(void* session, const char* text, size_t len);
int      llava_session_push_token(void* session, uint32_t token);
uint32_t llava_session_predict_next_token(void* session);          /* 0xFFFFFFFF on failure */
int      llava_session_start_next_token_prediction(void* session);
uint32_t llava_session_finish_next_token_prediction(void* session);
void     llava_session_rewind(void* session, uint32_t n);
uint32_t llava_session_set_options(void* session, uint32_t options);    /* ReturnCode */
uint32_t llava_session_save_frame(void* session, const char* path);     /* ReturnCode */
uint32_t llava_session_snapshot(void* session, const char* path);       /* ReturnCode */
uint32_t llava_session_restore(void* session, const char* path);        /* ReturnCode */
uint32_t llava_session_get_token_count(void* session);
uint32_t llava_session_get_tokens(void* session, uint32_t* out, uint32_t cap);
/* additions of this build (see llava_session.h) */
void     llava_session_set_deterministic(void* session, int on);
void     llava_session_set_seed(void* session, uint32_t seed);
/* non-greedy tokens come from the device sampler (lv_sample_mirostat) unless on != 0 selects the host's
 * (std::discrete_distribution over std::mt19937, as the reference draws them) */
void     llava_session_set_host_sampler(void* session, int on);
float    llava_session_get_mirostat_mu(void* session);
int      llava_session_set_max_batch(void* session, uint32_t n);
int      llava_session_generate_greedy_on_device(void* session, uint32_t n, uint32_t* out);
int      llava_session_enqueue_greedy_on_device(void* session, uint32_t n);     /* returns once queued */
int      llava_session_collect_greedy_on_device(void* session, uint32_t* out, uint32_t cap);
int      llava_session_get_logits(void* session, float* out, uint32_t cap);
uint32_t llava_session_get_backlog_size(void* session);
uint32_t llava_session_get_tokens_in_gpu(void* session);
/* kernel launches of one replay of the step evaluated last (0 before the first step) */
uint32_t llava_session_step_kernel_launches(void* session);
/* timeline of the one-launch token step (lv_step_plan_set_trace / lv_step_plan_read_trace in lv_b200.h):
 * returns the number of words copied, dims3 = {operations, CTAs, points}; 0 when unavailable */
int      llava_session_set_step_trace(void* session, int on);
uint64_t llava_session_read_step_trace(void* session, uint64_t* out, uint64_t cap, uint32_t* dims3);
/* rows [row0, row0 + nrows) of one layer's K (which = 0) or V (1) cache, f16 bits */
int      llava_session_read_kv(void* session, uint32_t layer, int which, uint32_t row0, uint32_t nrows, uint16_t* out);

/* ---- llava_session_group: one decoding step for several sessions with one pass over the weights (greedy).
 * create: 2..64 sessions of one single-GPU context, NULL when that cannot work.  step: every member holds exactly one
 * token that is not evaluated yet; next_tokens[i] = member i's greedy next token (not pushed).  generate: n steps with
 * the tokens fed back on the device; out[i * n + j] = token j of member i (appended to the members' buffers). */
void*    llava_session_group_create(void* ctx, void* const* sessions, uint32_t n);
void     llava_session_group_destroy(void* group);
int      llava_session_group_step(void* group, uint32_t* next_tokens);
int      llava_session_group_generate_greedy_on_device(void* group, uint32_t n, uint32_t* out);
int      llava_session_group_get_logits(void* group, uint32_t member, float* out, uint32_t n);   /* of the last step */
uint32_t llava_session_group_kernel_launches(void* group);

/* where a rank's column slice of a cache row lives in a snapshot file (host/tp_shard.h), and the size of the file */
uint64_t llava_tp_snapshot_slice_offset(uint32_t n_tokens, uint32_t dim, uint32_t layer, uint32_t which, uint32_t row,
                                        uint32_t rank, uint32_t n_ranks);
uint64_t llava_tp_snapshot_file_size(uint32_t n_tokens, uint32_t dim, uint32_t n_layers);

/* ---- lsrv::session_wrapper (server/session_wrapper.h:17-23): one thread and one session per
 *      served session, driven by orders (opcodes of server/types.h:50-73).  The owner created
 *      here plays the reference's llava_server: it collects the outbound packets. */
void*    llava_wrapper_owner_create(void* ctx);
void     llava_wrapper_owner_destroy(void* owner);
uint32_t llava_wrapper_owner_dead_sessions(void* owner);
/* next outbound item (kind 0: packet to client `who` answering `request`; 1: broadcast of session
 * `who`); returns 0 when nothing arrived within timeout_ms */
int      llava_wrapper_owner_pop(void* owner, int timeout_ms, uint32_t* kind, uint32_t* who, uint32_t* opcode,
                                 uint32_t* request, uint8_t* payload, uint32_t cap, uint32_t* length);
void*    llava_wrapper_create(void* owner, int deterministic);
uint32_t llava_wrapper_session_id(void* wrapper);
void     llava_wrapper_start(void* wrapper);
void     llava_wrapper_push_order(void* wrapper, uint32_t client_id, uint32_t request_id, uint32_t opcode, uint32_t arg1,
                                  const char* s, size_t len);
void     llava_wrapper_join(void* wrapper);
void     llava_wrapper_destroy(void* wrapper);

/* ---- lsrv::tlv_server: the TCP front end of the session protocol (reference server/server.cpp:44-331,
 * server/client.cpp:43-313).  create binds and listens (port 0 = any free port; NULL address = 127.0.0.1) and
 * returns NULL on failure; start runs the event loop on a thread of its own; stop kills the sessions, waits
 * for them and joins the loop.  deterministic != 0: sessions decode greedily (the reference always samples). */
void*    llava_server_create(void* ctx, uint32_t port, const char* bind_address, int deterministic);
uint32_t llava_server_port(void* server);
/* sessions in the running state are stepped together (one pass over the weights per round): rounds that served two or
 * more sessions, and the tokens they produced */
uint64_t llava_server_grouped_steps(void* server);
uint64_t llava_server_grouped_tokens(void* server);
uint64_t llava_server_steps_ahead(void* server);
/* microseconds the scheduler's rounds spent waiting for their callers to arrive / for the device */
uint64_t llava_server_scheduler_collect_us(void* server);
uint64_t llava_server_scheduler_device_us(void* server);      /* grouped steps that were already queued when their sessions asked */
void     llava_server_start(void* server);
void     llava_server_stop(void* server);
void     llava_server_destroy(void* server);

#ifdef __cplusplus
}
#endif
#endif /* LLAVA_HOST_H */
