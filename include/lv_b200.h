/*
 * lv_b200 -- C ABI of the B200 (sm_100a) decode kernels that replace the
 * Vulkan compute path of aodenis/llama-vulkan.
 *
 * The reference has no FFI: its host code (llava_session / llava_layer /
 * llava_command_buffer / llava_buffer / llava_device_memory) calls Vulkan-Hpp
 * directly.  Each entry point below names the reference interface it stands
 * in for (file:line relative to the reference project root).
 *
 * Conventions: every function returns LV_OK (0) or an LV_ERR_* code and never
 * throws or aborts; lv_last_error_string() describes the last failure on the
 * calling thread.  All `void*`/`float*` arguments named as device memory are
 * device pointers obtained from lv_arena_create.  Kernels are enqueued on the
 * context's stream and run asynchronously; lv_stream_sync waits for them.
 * Quantised matrices keep the GGML ggjt-v3 block layout of the model file:
 * rows of K/32 blocks, a block being an f16 scale followed by 16 nibble bytes
 * (q4_0, 18 B) or 32 int8 (q8_0, 34 B).  `wtype` is the GGML type code
 * (2 = q4_0, 8 = q8_0).  K must be a multiple of 256 and matrix base
 * addresses 16-byte aligned (both hold for every tensor of a 7B/13B file
 * placed by lv_arena_create).
 */
#ifndef LV_B200_H
#define LV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  1..8 mirror ReturnCode (types.h:45-55) where they overlap. */
enum {
    LV_OK = 0,
    LV_ERR_NOK = 1,            /* generic failure (ReturnCode::nok) */
    LV_ERR_BAD_ARGUMENTS = 7,  /* ReturnCode::bad_arguments */
    LV_ERR_CUDA = 100,         /* a CUDA runtime call failed */
    LV_ERR_DEVICE_WAIT = 101,  /* a bounded device-side wait gave up (error word non-zero) */
    LV_ERR_TIMEOUT = 102,      /* lv_stream_sync timed out on the host */
    LV_ERR_COMM = 103          /* NCCL failure */
};

enum { LV_TYPE_F32 = 0, LV_TYPE_F16 = 1, LV_TYPE_Q4_0 = 2, LV_TYPE_Q8_0 = 8,
       /* the q4_0 blocks of ggjt version 1 files (llava_buffer.cpp:66-71,350-359): 20 bytes, f32 scale, byte j holding
        * elements 2j (low nibble) and 2j+1 (high); accepted by lv_gemv, lv_norm_gemv, lv_gemv_silu,
        * lv_norm_gate_up_silu, lv_norm_qkv_kvappend and lv_dequant_rows (the shaders matmul_dim.comp /
        * matmul_silu_ff.comp without the _fp16 suffix).  Not a GGML code: such files say "q4_0" too. */
       LV_TYPE_Q4_0_V1 = 258 };

typedef struct lv_ctx lv_ctx;
typedef struct lv_graph lv_graph;

/* ---- lifecycle: replaces the Vulkan instance/device/queue/pool bring-up of
 *      llava_context::run (llava_context.cpp:230-282) ---------------------- */
int lv_device_count(int* count);
int lv_ctx_create(int device, lv_ctx** out);
int lv_ctx_destroy(lv_ctx* ctx);
const char* lv_last_error_string(void);
/* cudaStream_t of the context, for callers that enqueue their own work */
void* lv_ctx_stream(lv_ctx* ctx);
int lv_ctx_sm_count(lv_ctx* ctx);

/* ---- memory: replaces llava_device_memory::freeze / map / unmap
 *      (llava_device_memory.cpp:23-73) and llava_buffer::load_to_gpu
 *      (llava_buffer.cpp:464-478).  One arena = one cudaMalloc. ------------ */
int lv_arena_create(lv_ctx* ctx, size_t bytes, void** dptr);
int lv_arena_free(lv_ctx* ctx, void* dptr);
int lv_host_alloc(lv_ctx* ctx, size_t bytes, void** hptr);        /* pinned */
int lv_host_free(lv_ctx* ctx, void* hptr);
int lv_upload(lv_ctx* ctx, void* dst, const void* host_src, size_t bytes);          /* blocking */
int lv_download(lv_ctx* ctx, void* host_dst, const void* src, size_t bytes);        /* blocking, after the stream drains */
int lv_upload_async(lv_ctx* ctx, void* dst, const void* pinned_src, size_t bytes);  /* on the stream */
int lv_download_async(lv_ctx* ctx, void* pinned_dst, const void* src, size_t bytes);
int lv_memset(lv_ctx* ctx, void* dst, int value, size_t bytes);                     /* on the stream */
int lv_copy_d2d(lv_ctx* ctx, void* dst, const void* src, size_t bytes);             /* on the stream */

/* ---- execution: replaces llava_command_buffer::record_execution / run /
 *      wait_idle (llava_command_buffer.cpp:25-55): the recorded command list
 *      becomes a CUDA graph captured from the context's stream. ------------ */
int lv_graph_begin_capture(lv_ctx* ctx);
int lv_graph_end_capture(lv_ctx* ctx, lv_graph** out);
int lv_graph_launch(lv_ctx* ctx, lv_graph* g);
/* number of kernel launches one replay of the graph performs */
int lv_graph_kernel_nodes(lv_graph* g, uint32_t* out);
int lv_graph_destroy(lv_graph* g);
/* Waits until the stream is idle (timeout_ms <= 0: no limit), then reads the
 * device error word; LV_ERR_DEVICE_WAIT if a kernel recorded a lost wait. */
int lv_stream_sync(lv_ctx* ctx, int timeout_ms);

/* ---- decode kernels, one per reference shader ---------------------------- */

/* shaders/normalize.comp via llava_command_buffer::normalize_logit
 * (llava_command_buffer.cpp:57-59): out = x * w * rsqrt(mean((x-mean x)^2)),
 * no epsilon.  x, out: f32 [batch][dim]; w: f32 [dim]. */
int lv_norm_f32(lv_ctx* ctx, float* out, const float* x, const float* w, uint32_t dim, uint32_t batch);

/* shaders/matmul_{dim,ff}{,_q8}_fp16.comp via llava_command_buffer::matmul
 * (llava_command_buffer.cpp:61-85); add != 0 selects matmul_add_* /
 * matmul_add_inplace (:87-111): out += W x.  W: [rows][cols] blocks;
 * x: f32 [batch][cols]; out: f32 [batch][rows].  rows % 4 == 0. */
int lv_gemv(lv_ctx* ctx, float* out, const void* W, int wtype, const float* x, uint32_t rows, uint32_t cols,
            uint32_t batch, int add);

/* shaders/matmul_silu_ff*.comp via llava_command_buffer::matmul_silu_ff
 * (llava_command_buffer.cpp:113-132): out = (w3 x) * (w1 x) / (1 + exp(-(w1 x))). */
int lv_gemv_silu(lv_ctx* ctx, float* out, const void* w3, const void* w1, int wtype, const float* x, uint32_t rows,
                 uint32_t cols, uint32_t batch);

/* shaders/copy_to_cache.comp via llava_command_buffer::kv_copy (:134-142):
 * cache[*pos + z][i] = f16(x[z][i]); no rotation.  cache: f16 [ctx_rows][dim];
 * pos: device u32 (the reference's config_buffer.token_count). */
int lv_kv_append_f16(lv_ctx* ctx, void* cache, const float* x, const uint32_t* pos, uint32_t dim, uint32_t batch,
                     uint32_t ctx_rows);

/* Builds the [max_ctx][rot/2] table of (cos, sin) of distance * 10000^(-i/(rot/2))
 * used by the two attention entry points below (angles in double on the host,
 * shaders/mhsa.comp:47-49). table: device f32 [max_ctx][rot/2][2]. */
int lv_rope_table_build(lv_ctx* ctx, float* table, uint32_t max_ctx, uint32_t rot);

/* shaders/mhsa.comp via llava_command_buffer::multi_head_attention (:154-168):
 * scores[z][p][h] = sum_i <q[z][h][i], R(-(P - p) theta_i) K[p][h][i]>, P = *pos + z,
 * for p <= P; slots above P (which the reference fills with values that its
 * softmax then zeroes) are written as 0.  scores: f32 [batch][backlog][heads]. */
int lv_attn_scores_rope(lv_ctx* ctx, float* scores, const void* k_cache, const float* q, const uint32_t* pos,
                        const float* rope_table, uint32_t backlog, uint32_t heads, uint32_t rot, uint32_t batch);

/* shaders/softmax.comp via llava_command_buffer::inplace_softmax (:170-177):
 * a = exp(s / sqrt(rot)), a = 0 for p > P, a /= sum_p a. */
int lv_softmax_masked(lv_ctx* ctx, float* scores, const uint32_t* pos, uint32_t backlog, uint32_t heads,
                      uint32_t rot, uint32_t batch);

/* shaders/kqv_matching.comp via llava_command_buffer::perform_kqv_matching
 * (:179-194): v_out[z][d] = sum_p f32(V[p][d]) * probs[z][p][d / rot]. */
int lv_attn_values(lv_ctx* ctx, float* v_out, const void* v_cache, const float* probs, uint32_t backlog,
                   uint32_t heads, uint32_t rot, uint32_t batch);

/* shaders/copy.comp via llava_command_buffer::copy_logit (:144-152). */
int lv_copy_f32(lv_ctx* ctx, float* dst, const float* src, size_t count);
/* shaders/add_logits.comp (no caller in the reference): a[i] += b[i]. */
int lv_add_f32(lv_ctx* ctx, float* a, const float* b, size_t count);

/* llava_buffer::write_f32 (llava_buffer.cpp:339-401) as used for the embedding
 * rows (llava_session.cpp:219-223): out[z][:] = dequant(table row ids[z]) with
 * ids = token_ids + (first ? *first : 0).  table: [vocab][cols] blocks (or f32);
 * token_ids: device u32; first: device u32 or null (lets a recorded step read
 * "the tokens at the current position" from a device copy of the token buffer);
 * ids >= vocab are reported through the error word and read as row 0. */
int lv_dequant_rows(lv_ctx* ctx, float* out, const void* table, int wtype, const uint32_t* token_ids,
                    const uint32_t* first, uint32_t cols, uint32_t vocab, uint32_t n);

/* The deterministic branch of llava_session::get_last_predicted_token
 * (llava_session.cpp:144-152): first index of the maximum. out: device u32. */
int lv_argmax_f32(lv_ctx* ctx, uint32_t* out_index, const float* v, uint32_t n);

/* Last node of a recorded token step: the four words of config (the
 * reference's config_buffer, token_count x4) grow by batch, and, when argmax
 * and token_log are given, token_log[old token_count + batch] = *argmax, i.e.
 * the predicted token becomes the input of the next step without a host round
 * trip.  The reference's host does both between submits
 * (llava_session.cpp:224-228, llava_context.cpp:355-359).  All pointers are
 * device memory; a log index >= log_capacity is reported, not written. */
int lv_decode_advance(lv_ctx* ctx, uint32_t* config, const uint32_t* argmax, uint32_t* token_log, uint32_t batch,
                      uint32_t log_capacity);

/* lv_argmax_f32 followed by lv_decode_advance in one launch, for the recorded
 * greedy step: token = first index of the maximum of v[0..n) (same rules as
 * lv_argmax_f32); token_log[old token_count + batch] = token; the four words
 * of config grow by batch.  The token is also stored to *argmax_out (device,
 * may be null) and to *host_token (may be null): a word of pinned host memory
 * from lv_host_alloc, written by the kernel itself so that the step needs no
 * separate device-to-host copy; it is valid after the stream has been
 * synchronised.  Replaces the host-side scan and bookkeeping of
 * llava_session.cpp:145-151,224-228. */
int lv_argmax_advance(lv_ctx* ctx, const float* v, uint32_t n, uint32_t* config, uint32_t* token_log, uint32_t batch,
                      uint32_t log_capacity, uint32_t* argmax_out, uint32_t* host_token);

/* The non-deterministic branch of llava_session::get_last_predicted_token (llava_session.cpp:154-194) on the
 * device, for the logits of one token: the repeat penalty of llava_session.cpp:157-167 (token 13 only, counted
 * over the last 64 of the n_tokens tokens in token_log), temperature 0.8, probabilities without subtracting the
 * maximum, the candidates with probability >= 0.5^mu, one draw among them in proportion to their probability, and
 * mu += 0.1 * (5 + log2(p_drawn / kept mass)).  The reference draws with std::discrete_distribution over a
 * std::mt19937; here the cumulative distribution of the same candidates (in index order) is inverted at a uniform
 * variate from a counter-based generator (Philox 4x32-10) keyed by state[1] and counted in state[2]; a
 * forced_uniform in [0, 1) replaces the generator (tests).  All pointers are device memory:
 *   logits f32 [n_vocab] (16-byte aligned, n_vocab <= 32768); token_log u32, *n_tokens tokens of history;
 *   state u32 [4] = {mu as f32 bits, seed, draws so far, unused}, updated;
 *   feed_token_log (may be null): the drawn token is also stored to feed_token_log[*n_tokens], where a recorded
 *   step that follows reads its input token (index checked against log_capacity);
 *   out_token (device, may be null), host_token (pinned host word, may be null) receive the token, 0xFFFFFFFF when
 *   no candidate is left (NaN logits; also reported through the error word);
 *   report (may be null) u32 [4] = {candidates kept, kept mass, p_drawn, uniform variate} (f32 bits). */
int lv_sample_mirostat(lv_ctx* ctx, const float* logits, uint32_t n_vocab, const uint32_t* token_log, const uint32_t* n_tokens,
                       uint32_t* state, float forced_uniform, uint32_t* feed_token_log, uint32_t log_capacity,
                       uint32_t* out_token, uint32_t* host_token, uint32_t* report);

/* ---- one step for several sessions (shared weight pass) ---------------------- */

/* The reference's server runs every session's steps on their own, streaming the weights once per
 * session and token (server/session_wrapper.cpp:55-105).  A group step evaluates one token of each
 * of up to 64 sessions with one pass over the weights: the batched products below take the rows of
 * all members; the entry points here are the operations that differ per member, because every
 * member has its own caches, position and token log.  `members` is a device array of `n` entries
 * (one array per layer: the caches differ, pos and token_log repeat). */
typedef struct lv_group_member {
    void* k_cache;          /* f16 [ctx_rows][dim] of the layer */
    void* v_cache;
    uint32_t* pos;          /* device words [4]: tokens of this member already in its caches */
    uint32_t* token_log;    /* device: the member's token ids by position */
} lv_group_member;

/* out[z] = embedding row of members[z].token_log[*members[z].pos] (lv_dequant_rows per member). */
int lv_dequant_rows_group(lv_ctx* ctx, float* out, const void* table, int wtype, const lv_group_member* members,
                          uint32_t cols, uint32_t vocab, uint32_t n);
/* lv_gemm_tc_qkv_kvappend with row z of K and V stored at row *members[z].pos of members[z]'s caches. */
int lv_gemm_tc_qkv_kvappend_group(lv_ctx* ctx, float* q_out, const void* wq, const void* wk, const void* wv, int wtype,
                                  const void* xh, const lv_group_member* members, uint32_t rows_each, uint32_t dim,
                                  uint32_t n, uint32_t ctx_rows);
/* lv_attention_fused with query row z attending over members[z]'s caches up to *members[z].pos. */
int lv_attention_fused_group(lv_ctx* ctx, float* out, const float* q, const lv_group_member* members, const float* rope_table,
                             void* scratch, uint32_t heads, uint32_t rot, uint32_t backlog, uint32_t n);
/* lv_argmax_advance per member: the first index of the largest of logits[z][0..vocab) goes to
 * members[z].token_log[*pos + 1], to out_tokens[z] and (when given) host_tokens[z] (pinned memory); pos advances by one. */
int lv_argmax_advance_group(lv_ctx* ctx, const float* logits, uint32_t vocab, const lv_group_member* members, uint32_t n,
                            uint32_t log_capacity, uint32_t* out_tokens, uint32_t* host_tokens);

/* ---- batched products on the tensor cores (prompt evaluation) -------------- */

/* When several tokens are evaluated together the reference dispatches its
 * matmul shaders with the batch in gl_WorkGroupID.z (llava_command_buffer.cpp:
 * 61-132), streaming every matrix once per token.  These entry points read the
 * matrix once for up to 64 tokens: q4_0 / q8_0 blocks are dequantised in the
 * kernel into exact fp16 (hi, lo) tiles and multiplied on the tcgen05 tensor
 * cores with fp32 accumulation.  The activations enter as the two fp16 planes that
 * lv_act_split_f16 writes.  rows: multiple of 32 (a CTA covers 128 rows, 64 of
 * each matrix of the SiLU pair; a last tile may be ragged); cols: multiple of 256; batch 1..64; wtype q4_0 (2) or q8_0 (8).
 *
 * There are two forms of the weight tiles.  The default writes one fp16 plane,
 * fp16((q - 8) * d) or fp16(q * d): the weight is rounded to 11 significant bits
 * (relative error <= 2^-12 per weight; the activations keep 22 bits), which is
 * what the stated logits tolerance allows and a third of the tensor-core and
 * shared-memory work.  lv_gemm_tc_set_exact(ctx, 1) (or LV_GEMM_TC_EXACT=1 in
 * the environment when the context is made) selects the exact (hi, lo) pair for
 * parity-checked runs. */
int lv_gemm_tc_set_exact(lv_ctx* ctx, int exact);

/* Bytes of the split-activation buffer for [batch][cols] inputs. */
size_t lv_act_split_bytes(uint32_t cols, uint32_t batch);

/* xh = (hi, lo) fp16 planes of x [batch][cols], hi + lo = x to 22 bits; with
 * norm_w the reference's normalisation (shaders/normalize.comp:39-63) is
 * applied first.  The buffer is private to the lv_gemm_tc* calls: it holds,
 * per 64 columns, one ready-to-copy operand tile of 2 * zpad rows of 128 bytes
 * (zpad = batch rounded up to 16; rows < zpad: hi of a token, then lo; a
 * row's 16-byte units at unit ^ (row & 7)); tokens >= batch are zero. */
int lv_act_split_f16(lv_ctx* ctx, void* xh, const float* x, const float* norm_w, uint32_t cols, uint32_t batch);
/* The same for an input of cols_used values per token (dense rows) that meets a matrix of cols >= cols_used columns:
 * columns from cols_used on are zero.  This is the input of a tensor-parallel column shard whose rows are padded with
 * zero blocks (host/tp_shard.h).  No normalisation with padding. */
int lv_act_split_f16_padded(lv_ctx* ctx, void* xh, const float* x, const float* norm_w, uint32_t cols_used, uint32_t cols,
                            uint32_t batch);

/* out[z][r] (+)= sum_k W[r][k] x[z][k]: matmul / matmul_add_inplace for a batch. */
int lv_gemm_tc(lv_ctx* ctx, float* out, const void* W, int wtype, const void* xh, uint32_t rows, uint32_t cols,
               uint32_t batch, int add);

/* matmul_silu_ff for a batch (shaders/matmul_silu_ff.comp:49-97). */
int lv_gemm_tc_silu(lv_ctx* ctx, float* out, const void* w3, const void* w1, int wtype, const void* xh, uint32_t ff,
                    uint32_t dim, uint32_t batch);

/* wk, wq, wv products of a batch with the K and V rows written as f16 into the
 * caches at rows *pos + z (llava_layer.cpp:53-58); xh holds the normalised input. */
int lv_gemm_tc_qkv_kvappend(lv_ctx* ctx, float* q_out, void* k_cache, void* v_cache, const void* wq, const void* wk,
                            const void* wv, int wtype, const void* xh, const uint32_t* pos, uint32_t rows_each,
                            uint32_t dim, uint32_t batch, uint32_t ctx_rows);

/* ---- fused forms used by the decode graph -------------------------------- */

/* normalize + matmul wk, wq, wv + two kv_copy (llava_layer.cpp:53-58) in one
 * launch: K and V rows go straight into the f16 caches at row *pos + z.
 * rows = output features of each of the three matrices (dim, or dim / n_ranks
 * for a row shard); q_out is f32 [batch][rows], the caches f16 [ctx_rows][rows]. */
int lv_norm_qkv_kvappend(lv_ctx* ctx, float* q_out, void* k_cache, void* v_cache, const void* wq, const void* wk,
                         const void* wv, int wtype, const float* x, const float* norm_w, const uint32_t* pos,
                         uint32_t rows, uint32_t dim, uint32_t batch, uint32_t ctx_rows);

/* Bytes of scratch lv_attention_fused needs for the given shape. */
size_t lv_attention_scratch_bytes(uint32_t heads, uint32_t rot, uint32_t max_ctx, uint32_t batch);

/* mhsa + softmax + kqv_matching (llava_layer.cpp:59-62) in one launch, reading
 * only the P + 1 filled cache rows (the reference's masked slots contribute
 * exactly 0).  out: f32 [batch][heads*rot].  scratch: device memory of
 * lv_attention_scratch_bytes, zero-filled once before first use.  Launches
 * of at most one CTA per SM (heads * ceil(max_ctx / 256) * batch) rotate with
 * the table rows themselves; larger ones form cos/sin of a distance 32A + B
 * from the rows of 32A and of B (a few units in the last place). */
int lv_attention_fused(lv_ctx* ctx, float* out, const float* q, const void* k_cache, const void* v_cache,
                       const uint32_t* pos, const float* rope_table, void* scratch, uint32_t heads, uint32_t rot,
                       uint32_t max_ctx, uint32_t batch);

/* Same computation as lv_attention_fused for callers that cannot allocate
 * device memory at the point where they need attention -- code that runs
 * inside a stream capture or behind a host that hands out no allocator, an
 * embedder whose memory budget was fixed at start-up, a plug-in that is only
 * given input and output buffers.  The chunk partials live in a buffer built
 * into the library image (lv_attention_static_scratch_limit() bytes, 1 MiB,
 * present on every GPU that loads the library until the process exits), so
 * the call performs no cudaMalloc/cudaFree and calls nothing that allocates.
 * Shapes whose scratch (lv_attention_scratch_bytes) exceeds that limit are
 * rejected with LV_ERR_BAD_ARGUMENTS: 7B and 13B geometry at 2048 rows fit
 * with a batch of up to 6.  The first call on a device looks up the buffer's device
 * address; make that call before any stream capture.  All calls on a device
 * share the one buffer: calls that overlap on the GPU (different streams or
 * contexts) race; calls on one stream are safe.  Stale contents of earlier
 * calls are harmless (the arrival counters are cleared by each call).
 * No counterpart in the reference. */
size_t lv_attention_static_scratch_limit(void);
int lv_attention_fused_static(lv_ctx* ctx, float* out, const float* q, const void* k_cache, const void* v_cache,
                              const uint32_t* pos, const float* rope_table, uint32_t heads, uint32_t rot,
                              uint32_t max_ctx, uint32_t batch);

/* normalize + matmul_silu_ff (llava_layer.cpp:68-69) in one launch. */
int lv_norm_gate_up_silu(lv_ctx* ctx, float* out, const void* w3, const void* w1, int wtype, const float* x,
                         const float* norm_w, uint32_t ff, uint32_t dim, uint32_t batch);

/* normalize + output matmul (llava_command_buffer.cpp:38-39) in one launch. */
int lv_norm_gemv(lv_ctx* ctx, float* out, const void* W, int wtype, const float* x, const float* norm_w,
                 uint32_t rows, uint32_t cols, uint32_t batch);

/* ---- one token in one launch ----------------------------------------------------------------
 *
 * The reference records, per evaluation step, the operations of every layer plus the final
 * normalisation and output matrix into a list of command buffers and submits the list
 * (llava_command_buffer::record_execution, llava_command_buffer.cpp:29-45, over
 * llava_layer::execute, llava_layer.cpp:39-75).  lv_decode_step runs that whole list for ONE token
 * as a single persistent kernel: embedding row (llava_session.cpp:219-223), every layer's
 * normalize / matmul wk, wq, wv / copy_to_cache / mhsa / softmax / kqv_matching / matmul_add wo /
 * normalize / matmul_silu_ff / matmul_add w2, final normalize and output matmul, then -- with_head --
 * the greedy choice and the position bookkeeping of lv_argmax_advance (without the head only the
 * position advances, as for the leading tokens of a prompt).  Arithmetic and results are those of
 * the per-operation entry points above.
 *
 * A plan binds a model's weights and one session's caches and owns a small workspace; it must be
 * created outside stream capture.  All quantised matrices (layers and output) must lie in ONE
 * device allocation [weights_base, weights_base + weights_bytes), each at a multiple of its row
 * size (cols / 32 * 18 or 34 bytes) from weights_base and 16-byte aligned -- they are then row
 * ranges of one 2-D view of the arena per row size, which one TMA tensor map addresses.  Matrices
 * that are not placed like this are still accepted (q4_0 falls back to 1-D bulk copies).
 * ctx_rows: rows of the f16 caches.  tok_embeddings: [vocab][dim] of emb_type (q4_0, q8_0 or f32). */
typedef struct lv_step_layer {
    const void *wq, *wk, *wv, *wo, *w1, *w2, *w3;     /* quantised [rows][cols] in GGML block layout */
    const float *attention_norm, *ffn_norm;         /* f32 [dim] */
    void *k_cache, *v_cache;                        /* f16 [ctx_rows][dim] */
} lv_step_layer;

typedef struct lv_step_model {
    uint32_t dim, ff, heads, n_layers, vocab, ctx_rows;     /* of the whole model */
    int wtype, emb_type;
    /* Tensor parallelism (all zero on one GPU): this context is rank tp_rank of tp_ranks and holds, per layer, row
     * shards of wq / wk / wv (dim / tp_ranks rows: whole heads) and of w1 / w3 (ff / tp_ranks rows), and column shards
     * of wo and w2 whose rows are padded with zero blocks to shard_cols_o / shard_cols_2 columns (multiples of 256); the
     * caches are [ctx_rows][dim / tp_ranks].  The peer windows of the context (lv_peer_connect) must be connected:
     * the partial rows of wo and w2 travel through them.  Every rank must launch the same steps. */
    uint32_t tp_ranks, tp_rank, shard_cols_o, shard_cols_2;
    const void* weights_base;
    size_t weights_bytes;
    const void* tok_embeddings;
    const float* norm;
    const void* output;
    const float* rope_table;                        /* from lv_rope_table_build, at least ctx_rows rows */
    const lv_step_layer* layers;                    /* host array of n_layers entries */
} lv_step_model;

typedef struct lv_step_plan lv_step_plan;
int lv_step_plan_create(lv_ctx* ctx, const lv_step_model* model, lv_step_plan** out);
int lv_step_plan_destroy(lv_step_plan* plan);
/* Timeline of the steps launched after the call (on != 0), for tuning: every CTA stamps the device's
 * nanosecond clock at five points of every weight operation (begin, attention done, input records ready,
 * work items done, rows handed over).  Steps recorded into a graph before the call are not traced.
 * lv_step_plan_read_trace copies [operation][CTA][point] of the last traced step (4 * n_layers + 1
 * operations: per layer QKV, wo, gate/up, w2; then the output head). */
int lv_step_plan_set_trace(lv_step_plan* plan, int on);
int lv_step_plan_read_trace(lv_step_plan* plan, uint64_t* out, size_t max_words, uint32_t* n_ops, uint32_t* n_ctas,
                            uint32_t* n_points);
/* config, token_log, logits, argmax_out: device memory as for lv_argmax_advance (config[0] = tokens
 * already in the caches = position of the token to evaluate, read from token_log[config[0]]);
 * host_token: pinned host word or null.  logits (f32 [vocab]) may be null without the head. */
int lv_decode_step(lv_ctx* ctx, const lv_step_plan* plan, uint32_t* config, uint32_t* token_log, uint32_t log_capacity,
                   float* logits, uint32_t* argmax_out, uint32_t* host_token, int with_head);

/* ---- multi-GPU: one process per GPU, one communicator per context.  The
 *      reference is single-device (llava_context.cpp:264-279 takes one queue of
 *      one device); these entry points add the exchange step of the
 *      tensor-parallel decoder: an fp32 sum all-reduce of `dim` floats after the
 *      wo and after the w2 product (the TP forms of matmul_add_inplace,
 *      llava_layer.cpp:67,73).  NCCL is loaded at run time. ------------------- */
/* rank 0 makes the 128-byte id and hands it to the other ranks by any means */
int lv_comm_unique_id(uint8_t* out128);
int lv_comm_init_rank(lv_ctx* ctx, const uint8_t* id128, int n_ranks, int rank);
/* in place, on the context's stream (capturable); a no-op without a communicator */
int lv_allreduce_f32(lv_ctx* ctx, float* buf, size_t count);
/* residual += sum over ranks of partial: the tensor-parallel form of the residual add that
 * matmul_add_inplace fuses (llava_layer.cpp:67,73).  With a connected peer window (below) this is
 * ONE kernel: peer stores of the partial vector into every rank's window over NVLink, arrival
 * flags, a bounded wait, and the sum in rank order from local memory (bit-identical on all
 * ranks).  Without one it is lv_allreduce_f32 followed by lv_add_f32.  partial is clobbered. */
int lv_allreduce_add_f32(lv_ctx* ctx, float* residual, float* partial, size_t count);

/* The same exchange without a kernel of its own: the all-reduce is split between the GEMV that
 * produces the partial vector and the GEMV that consumes the sum.
 *   lv_tp_arm_push: the next lv_gemv on this context (one matrix, batch 1) sends its finished rows
 *     into its slot of every rank's window with peer stores and publishes one flag per CTA,
 *     instead of writing `out` (which is ignored).
 *   lv_tp_arm_pull: the next lv_norm_gemv / lv_norm_gate_up_silu / lv_norm_qkv_kvappend (batch 1)
 *     waits, bounded, for the flags of all ranks' producer launches (producer_rows = rows of the
 *     pushed matrix, which fixes the number of producer CTAs), takes x + sum over ranks of the
 *     slots (rank order) as its input, and stores that sum -- the new residual stream -- to x_out
 *     (a buffer other than x).
 * exchange: index of the exchange inside one evaluation step, 0 .. epochs_per_step-1, the same on
 * every rank; consecutive exchanges must alternate in parity (two slot sets are used in turn) and
 * every pushed exchange must be pulled before the second next one is pushed.  Flags carry
 * step * epochs_per_step + exchange + 1, where step counts the lv_decode_advance /
 * lv_argmax_advance launches of the context, so every step must end with one of them on every
 * rank.  No counterpart in the reference (single device). */
int lv_tp_arm_push(lv_ctx* ctx, int exchange, uint32_t epochs_per_step);
int lv_tp_arm_pull(lv_ctx* ctx, int exchange, uint32_t epochs_per_step, uint32_t producer_rows, float* x_out);
/* Peer windows: every rank creates one (capacity_floats >= the longest vector, multiple of 4),
 * hands the 64-byte CUDA IPC handle to all ranks by any means, and connects with the handles
 * of all ranks in rank order (its own entry is ignored).  One process per GPU, same node. */
size_t lv_peer_window_bytes(int n_ranks, uint32_t capacity_floats);
int lv_peer_window_create(lv_ctx* ctx, int n_ranks, uint32_t capacity_floats, uint8_t* handle64);
int lv_peer_connect(lv_ctx* ctx, int rank, const uint8_t* handles);
int lv_peer_destroy(lv_ctx* ctx);
int lv_comm_status(lv_ctx* ctx);     /* LV_ERR_COMM if NCCL reported an asynchronous error */
int lv_comm_abort(lv_ctx* ctx);
int lv_comm_destroy(lv_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* LV_B200_H */
