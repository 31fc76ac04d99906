/*
 * CPU oracle for the per-token decode path of aodenis/llama-vulkan.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * shader arithmetic and host arithmetic; it exists so that the CUDA path can
 * be checked against it and so that a CPU baseline can be timed.  Nothing in
 * the shipped library links, loads or calls it.
 *
 * PARITY UNPINNED: the reference ships no tests, fixtures or golden vectors
 * for this path and its shaders cannot be executed here (they need Vulkan),
 * so this restatement is pinned only by hand-built known-answer cases, by the
 * reference's exact integer dequantisation formulas and, for file parsing and
 * tokenisation, by the reference's own ggml_file.cpp compiled unmodified.
 *
 * Every function cites the reference file:line it follows (paths are
 * relative to the reference project root).
 */
#ifndef LLAVA_ORACLE_H
#define LLAVA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml_value_type codes, types.h:28-43 */
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_Q4_0 = 2, ORC_Q8_0 = 8 };

/* ---- scalar helpers ---------------------------------------------------- */
float    orc_half_to_float(uint16_t h);              /* llava_buffer.cpp:142-177 */
uint16_t orc_float_to_half(float f);                 /* copy_to_cache.comp:35, round-to-nearest-even */

/* bytes of one row of `cols` weights, ggml_file.cpp:162-186 */
size_t orc_row_bytes(int type, int version, uint32_t cols);

/* ---- ops (one per reference shader / host routine) --------------------- */
/* llava_buffer.cpp:339-401: dequantise `count` (multiple of 32) weights */
int  orc_dequant(const void* in, int type, int version, float* out, uint32_t count);
/* shaders/normalize.comp:34-63, workgroup of `wgs` invocations */
void orc_norm(float* out, const float* x, const float* w, uint32_t dim, uint32_t wgs);
/* shaders/matmul.glsl:41-74 and matmul_q8.glsl:41-72; `workers` = MATMUL_Y,
 * add != 0 selects the matmul_add_* variant (out += result) */
int  orc_gemv(float* out, const void* W, int type, int version, const float* x,
              uint32_t rows, uint32_t cols, uint32_t workers, int add);
/* shaders/matmul_silu_ff.comp:49-97: out = (w3 x) * (w1 x) / (exp(-(w1 x)) + 1) */
int  orc_gemv_silu(float* out, const void* w3, const void* w1, int type, int version,
                   const float* x, uint32_t rows, uint32_t cols, uint32_t workers);
/* shaders/copy_to_cache.comp:29-37 */
void orc_kv_append(uint16_t* cache, const float* x, uint32_t pos, uint32_t dim);
/* shaders/mhsa.comp:32-60: scores[p*heads+h] for p in [0, n_slots) */
void orc_mhsa(float* scores, const uint16_t* k_cache, const float* q, uint32_t pos,
              uint32_t n_slots, uint32_t heads, uint32_t rot);
/* shaders/softmax.comp:26-44 over `backlog` slots (power of two) */
void orc_softmax(float* scores, uint32_t pos, uint32_t backlog, uint32_t heads, uint32_t rot);
/* shaders/kqv_matching.comp:27-42 */
void orc_kqv(float* v_out, const uint16_t* v_cache, const float* probs, uint32_t backlog,
             uint32_t heads, uint32_t rot);
/* llava_session.cpp:144-152: first index of the maximum */
uint32_t orc_argmax(const float* v, uint32_t n);
/* llava_session.cpp:154-194 up to (not including) the random draw: applies the
 * token-13 penalty, temperature and the 2^-mu cut.  Writes the kept
 * probabilities to probs_out and their token ids to ids_out; returns the kept
 * count and stores the kept mass in *kept_sum. */
uint32_t orc_sampler_candidates(const float* logits, uint32_t n_vocab, const uint32_t* tokens,
                                uint32_t n_tokens, float mu, float* probs_out, uint32_t* ids_out,
                                float* kept_sum);
/* llava_session.cpp:193: mu update after drawing candidate idx */
float orc_sampler_mu_update(float mu, float p_selected, float kept_sum);

/* ---- model + session (ggml_file.cpp:17-122, llava_session.cpp:197-327) -- */
typedef struct orc_model orc_model;
typedef struct orc_session orc_session;

typedef struct {
    uint32_t file_version, vocab_size, dim, multiple_of, n_heads, n_layers, rot, ftype, ff_size;
    uint32_t wtype;        /* type code of layers.0.attention.wq */
    uint32_t n_tensors;
} orc_model_info;

orc_model* orc_model_open(const char* path);
void       orc_model_close(orc_model* m);
void       orc_model_get_info(const orc_model* m, orc_model_info* out);
/* tensor table access; returns 0 on success.  rows = shape1, cols = shape2 as
 * the reference stores them (ggml_file.cpp:86-91) */
int        orc_model_tensor(const orc_model* m, uint32_t index, char* name, size_t name_cap,
                            uint32_t* type, uint64_t* offset, uint32_t* shape1, uint32_t* shape2,
                            uint64_t* size);
const void* orc_model_tensor_data(const orc_model* m, const char* name);
const char* orc_model_token(const orc_model* m, uint32_t id, uint32_t* len, float* score);

orc_session* orc_session_create(orc_model* m, uint32_t wgs);
void         orc_session_destroy(orc_session* s);
/* llava_session.cpp:284-297; returns 0 when the 2048-token limit is hit */
int          orc_session_push_token(orc_session* s, uint32_t token);
/* llava_session.cpp:390-395 */
void         orc_session_rewind(orc_session* s, uint32_t n);
uint32_t     orc_session_token_count(const orc_session* s);
uint32_t     orc_session_backlog(const orc_session* s);
/* Evaluates every token not yet in the cache (the reference evaluates them as
 * one batch whose rows are independent except through the cache, so token by
 * token is the same arithmetic) and leaves the last token's logits in
 * logits_out[vocab].  Returns 0 on success. */
int          orc_session_eval(orc_session* s, float* logits_out);
/* pointers into the session's state for layer-level parity checks */
const uint16_t* orc_session_k_cache(const orc_session* s, uint32_t layer);
const uint16_t* orc_session_v_cache(const orc_session* s, uint32_t layer);
/* residual stream after the last evaluated token's final layer, [dim] */
const float*    orc_session_residual(const orc_session* s);
/* per-layer residual stream captured after each layer for the last token,
 * [n_layers][dim]; valid after orc_session_eval */
const float*    orc_session_layer_outputs(const orc_session* s);

void orc_set_threads(int n);
int  orc_get_threads(void);

#ifdef __cplusplus
}
#endif
#endif
