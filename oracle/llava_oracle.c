/*
 * CPU oracle for the per-token decode path of aodenis/llama-vulkan.
 * TEST INFRASTRUCTURE ONLY -- see llava_oracle.h.  PARITY UNPINNED (the
 * reference has no golden vectors; its shaders cannot run without Vulkan).
 *
 * Conventions where the reference leaves behaviour to the Vulkan driver:
 *   - vec4/mat4 expressions are evaluated left to right without contraction
 *     (build with -ffp-contract=off);
 *   - shared-memory tree sums are restated literally (common.glsl:61-74);
 *   - float -> half is round-to-nearest-even;
 *   - pow/sin/cos are evaluated in double on float-rounded arguments and the
 *     result rounded to float; exp and 1/sqrt use float libm.
 */
#define _GNU_SOURCE
#include "llava_oracle.h"

#include <fcntl.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* scalar helpers                                                            */
/* ------------------------------------------------------------------------ */

/* llava_buffer.cpp:142-177 (halfToFloat) */
float orc_half_to_float(uint16_t half) {
    uint32_t s = (half >> 15) & 1u, single;
    int e = (half >> 10) & 0x1f;
    uint32_t m = half & 0x3ffu;
    if (e == 0) {
        if (m == 0) {
            single = s << 31;
        } else {
            while (!(m & 0x400u)) { m <<= 1; e -= 1; }
            e += 1;
            m &= ~0x400u;
            single = (s << 31) | ((uint32_t)(e + (127 - 15)) << 23) | (m << 13);
        }
    } else if (e == 31) {
        single = (s << 31) | 0x7f800000u | (m << 13);
    } else {
        single = (s << 31) | ((uint32_t)(e + (127 - 15)) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &single, 4);
    return f;
}

/* shaders/copy_to_cache.comp:35 float16_t(x); rounding fixed to nearest-even */
uint16_t orc_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) {                       /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0u));
    }
    if (absx >= 0x477ff000u) {                       /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x38800000u) {                        /* subnormal half or zero */
        if (absx < 0x33000000u) return (uint16_t)sign;      /* < 2^-25 -> 0 */
        int e = (int)(absx >> 23);                   /* biased exponent 102..112 */
        uint32_t man = (absx & 0x7fffffu) | 0x800000u;
        int shift = 126 - e;                         /* 14..24 */
        uint32_t q = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t e = (absx >> 23) - 112u;                /* 1..30 */
    uint32_t man = absx & 0x7fffffu;
    uint32_t q = (e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}

/* ggml_file.cpp:162-186 (size_in_file), per row */
size_t orc_row_bytes(int type, int version, uint32_t cols) {
    switch (type) {
        case ORC_F32: return (size_t)cols * 4;
        case ORC_F16: return (size_t)cols * 2;
        case ORC_Q4_0: return (size_t)cols / 32 * (version == 1 ? 20 : 18);
        case ORC_Q8_0: return (size_t)cols / 32 * (version == 1 ? 36 : 34);
        default: return 0;
    }
}

static int g_threads = 0;
void orc_set_threads(int n) {
    g_threads = n;
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#endif
}
int orc_get_threads(void) {
#ifdef _OPENMP
    return g_threads > 0 ? g_threads : omp_get_max_threads();
#else
    return 1;
#endif
}

/* common.glsl:61-74 local_sum: halving tree over n = 2^bits entries, in place */
static float tree_sum(float* buf, uint32_t n) {
    for (uint32_t cur = n >> 1; cur >= 1; cur >>= 1) {
        for (uint32_t i = 0; i < cur; i++) buf[i] += buf[cur + i];
    }
    return buf[0];
}

/* ------------------------------------------------------------------------ */
/* dequantisation: llava_buffer.cpp:339-401 (write_f32)                      */
/* ------------------------------------------------------------------------ */

/* 32 integer weight values of one block in natural element order plus its
 * scale.  q4_0 v3: element j in the low nibble of byte j, element j+16 in the
 * high nibble (llava_buffer.cpp:365-369); q4_0 v1: elements 2j, 2j+1 in byte j
 * with an f32 scale (:352-358); q8_0 v3: signed bytes (:387-394). */
static int block_ints(const uint8_t* blk, int type, int version, int* q, float* d) {
    if (type == ORC_Q4_0 && version == 3) {
        uint16_t h;
        memcpy(&h, blk, 2);
        *d = orc_half_to_float(h);
        for (int j = 0; j < 16; j++) {
            q[j] = (blk[2 + j] & 0xf) - 8;
            q[j + 16] = (blk[2 + j] >> 4) - 8;
        }
        return 0;
    }
    if (type == ORC_Q4_0 && version == 1) {
        memcpy(d, blk, 4);
        for (int j = 0; j < 16; j++) {
            q[2 * j] = (blk[4 + j] & 0xf) - 8;
            q[2 * j + 1] = (blk[4 + j] >> 4) - 8;
        }
        return 0;
    }
    if (type == ORC_Q8_0 && version == 3) {
        uint16_t h;
        memcpy(&h, blk, 2);
        *d = orc_half_to_float(h);
        for (int j = 0; j < 32; j++) {
            int v = blk[2 + j];
            if (v >= 128) v -= 256;
            q[j] = v;
        }
        return 0;
    }
    return -1;
}

int orc_dequant(const void* in, int type, int version, float* out, uint32_t count) {
    if (type == ORC_F32) {                     /* llava_buffer.cpp:377-381 */
        memcpy(out, in, (size_t)count * 4);
        return 0;
    }
    if (count % 32) return -1;
    size_t bsz = orc_row_bytes(type, version, 32);
    if (!bsz) return -1;
    const uint8_t* p = (const uint8_t*)in;
    for (uint32_t b = 0; b < count / 32; b++) {
        int q[32];
        float d;
        if (block_ints(p + b * bsz, type, version, q, &d)) return -1;
        for (int j = 0; j < 32; j++) out[b * 32 + j] = (float)q[j] * d;
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* shaders/normalize.comp:34-63                                              */
/* ------------------------------------------------------------------------ */
void orc_norm(float* out, const float* x, const float* w, uint32_t dim, uint32_t wgs) {
    uint32_t nvec = dim / 4;
    uint32_t managed = (nvec + wgs - 1) / wgs;          /* normalize.comp:23 */
    float* buf = (float*)malloc(sizeof(float) * wgs);
    for (uint32_t i = 0; i < wgs; i++) {
        float part = 0.f;
        for (uint32_t j = 0; j < managed; j++) {
            uint32_t v = managed * i + j;
            if (v < nvec) {
                const float* e = x + 4 * v;
                part += ((e[0] + e[1]) + e[2]) + e[3];   /* dot(element, vec4(1.)) */
            }
        }
        buf[i] = part;
    }
    float mean = tree_sum(buf, wgs) / (float)dim;        /* :47 */
    for (uint32_t i = 0; i < wgs; i++) {
        float part = 0.f;
        for (uint32_t j = 0; j < managed; j++) {
            uint32_t v = managed * i + j;
            if (v < nvec) {
                float a = x[4 * v] - mean, b = x[4 * v + 1] - mean;
                float c = x[4 * v + 2] - mean, d = x[4 * v + 3] - mean;
                part += ((a * a + b * b) + c * c) + d * d; /* dot(element, element) */
            }
        }
        buf[i] = part;
    }
    float factor = 1.0f / sqrtf(tree_sum(buf, wgs) / (float)dim);   /* :56 inversesqrt, no eps */
    for (uint32_t k = 0; k < dim; k++) out[k] = (x[k] * w[k]) * factor;   /* :58-62 */
    free(buf);
}

/* ------------------------------------------------------------------------ */
/* shaders/matmul.glsl:41-74, matmul_q8.glsl:41-72                           */
/* ------------------------------------------------------------------------ */

/* One row: per worker, blocks worker, worker+Y, ... ; inside a block the
 * integer weights times the input are summed in groups of four (the mat4 *
 * vec4 products), the block scale multiplies once (matmul.glsl:63), workers
 * are combined by the halving tree (:66). */
static float gemv_row(const uint8_t* row, int type, int version, const float* x, uint32_t nblocks,
                      uint32_t workers, float* wbuf) {
    size_t bsz = orc_row_bytes(type, version, 32);
    for (uint32_t w = 0; w < workers; w++) {
        float worker_sum = 0.f;
        for (uint32_t b = w; b < nblocks; b += workers) {
            int q[32];
            float d;
            block_ints(row + (size_t)b * bsz, type, version, q, &d);
            const float* xi = x + (size_t)b * 32;
            float block_val = 0.f;
            for (int g = 0; g < 8; g++) {
                float t = (float)q[4 * g] * xi[4 * g];
                t = t + (float)q[4 * g + 1] * xi[4 * g + 1];
                t = t + (float)q[4 * g + 2] * xi[4 * g + 2];
                t = t + (float)q[4 * g + 3] * xi[4 * g + 3];
                block_val += t;
            }
            worker_sum += block_val * d;
        }
        wbuf[w] = worker_sum;
    }
    return tree_sum(wbuf, workers);
}

static int gemv_args_ok(int type, int version, uint32_t cols, uint32_t workers) {
    if (cols % 32 || workers == 0 || (workers & (workers - 1))) return 0;
    if (type == ORC_Q4_0) return version == 1 || version == 3;
    if (type == ORC_Q8_0) return version == 3;
    return 0;
}

int orc_gemv(float* out, const void* W, int type, int version, const float* x, uint32_t rows,
             uint32_t cols, uint32_t workers, int add) {
    if (!gemv_args_ok(type, version, cols, workers)) return -1;
    size_t rb = orc_row_bytes(type, version, cols);
    const uint8_t* base = (const uint8_t*)W;
#pragma omp parallel
    {
        float* wbuf = (float*)malloc(sizeof(float) * workers);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < (int64_t)rows; r++) {
            float v = gemv_row(base + (size_t)r * rb, type, version, x, cols / 32, workers, wbuf);
            if (add) out[r] += v; else out[r] = v;           /* matmul.glsl:68-72 */
        }
        free(wbuf);
    }
    return 0;
}

/* shaders/matmul_silu_ff.comp:49-97 (mat1 = w3, mat2 = w1, llava_layer.cpp:69) */
int orc_gemv_silu(float* out, const void* w3, const void* w1, int type, int version, const float* x,
                  uint32_t rows, uint32_t cols, uint32_t workers) {
    if (!gemv_args_ok(type, version, cols, workers)) return -1;
    size_t rb = orc_row_bytes(type, version, cols);
    const uint8_t* b3 = (const uint8_t*)w3;
    const uint8_t* b1 = (const uint8_t*)w1;
#pragma omp parallel
    {
        float* wbuf = (float*)malloc(sizeof(float) * workers);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < (int64_t)rows; r++) {
            float r1 = gemv_row(b3 + (size_t)r * rb, type, version, x, cols / 32, workers, wbuf);
            float r2 = gemv_row(b1 + (size_t)r * rb, type, version, x, cols / 32, workers, wbuf);
            out[r] = r1 * r2 / (expf(-r2) + 1.0f);           /* :95 */
        }
        free(wbuf);
    }
    return 0;
}

/* shaders/copy_to_cache.comp:29-37: no rotation, plain cast */
void orc_kv_append(uint16_t* cache, const float* x, uint32_t pos, uint32_t dim) {
    for (uint32_t i = 0; i < dim; i++) cache[(size_t)pos * dim + i] = orc_float_to_half(x[i]);
}

/* RoPE angle pieces of shaders/mhsa.comp:47-49 for distance `delta`, pair i */
static void rope_cs(uint32_t delta, uint32_t i, uint32_t half_rot, float* ct, float* st) {
    float theta = (float)pow(10000.0, (double)(-(float)i / (float)half_rot));
    float d_theta = (float)delta * theta;
    *ct = (float)cos((double)d_theta);
    *st = (float)sin((double)d_theta);
}

static void mhsa_with_table(float* scores, const uint16_t* k_cache, const float* q, uint32_t pos,
                            uint32_t n_slots, uint32_t heads, uint32_t rot, const float* cs_table) {
    uint32_t dim = heads * rot, half_rot = rot / 2;
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < (int64_t)n_slots; p++) {
        uint32_t delta = pos - (uint32_t)p;      /* config.token_count + z - q_index, mhsa.comp:47 */
        for (uint32_t h = 0; h < heads; h++) {
            float result = 0.f;
            for (uint32_t i = 0; i < half_rot; i++) {
                float qx = q[h * rot + 2 * i], qy = q[h * rot + 2 * i + 1];     /* "raw_K": the query */
                float kx = orc_half_to_float(k_cache[(size_t)p * dim + h * rot + 2 * i]);
                float ky = orc_half_to_float(k_cache[(size_t)p * dim + h * rot + 2 * i + 1]);
                float ct, st;
                if (cs_table) {
                    ct = cs_table[((size_t)delta * half_rot + i) * 2];
                    st = cs_table[((size_t)delta * half_rot + i) * 2 + 1];
                } else {
                    rope_cs(delta, i, half_rot, &ct, &st);
                }
                /* rot_mat * raw_Q with columns (ct,-st) and (st,ct): mhsa.comp:50-54 */
                float rx = ct * kx + st * ky;
                float ry = (-st) * kx + ct * ky;
                result += qx * rx + qy * ry;
            }
            scores[(size_t)p * heads + h] = result;
        }
    }
}

/* shaders/mhsa.comp:32-60.  Slots above pos are not needed by any caller of
 * the oracle (the softmax zeroes them), so n_slots <= pos + 1 is expected. */
void orc_mhsa(float* scores, const uint16_t* k_cache, const float* q, uint32_t pos, uint32_t n_slots,
              uint32_t heads, uint32_t rot) {
    mhsa_with_table(scores, k_cache, q, pos, n_slots, heads, rot, NULL);
}

/* shaders/softmax.comp:26-44: exp without max-subtraction, masked slots 0,
 * tree sum over the whole backlog.  scores is [backlog][heads]; entries with
 * p > pos are overwritten with 0 and need not be initialised. */
void orc_softmax(float* scores, uint32_t pos, uint32_t backlog, uint32_t heads, uint32_t rot) {
    float main_factor = 1.0f / sqrtf((float)rot);
    float* buf = (float*)malloc(sizeof(float) * backlog);
    for (uint32_t h = 0; h < heads; h++) {
        for (uint32_t p = 0; p < backlog; p++) {
            float a = 0.f;
            if (p <= pos) a = expf(scores[(size_t)p * heads + h] * main_factor);
            scores[(size_t)p * heads + h] = a;
            buf[p] = a;
        }
        float total = tree_sum(buf, backlog);
        for (uint32_t p = 0; p < backlog; p++) scores[(size_t)p * heads + h] /= total;
    }
    free(buf);
}

/* shaders/kqv_matching.comp:27-42 */
void orc_kqv(float* v_out, const uint16_t* v_cache, const float* probs, uint32_t backlog,
             uint32_t heads, uint32_t rot) {
    uint32_t dim = heads * rot;
#pragma omp parallel
    {
        float* buf = (float*)malloc(sizeof(float) * backlog);
#pragma omp for schedule(static)
        for (int64_t d = 0; d < (int64_t)dim; d++) {
            for (uint32_t p = 0; p < backlog; p++) {
                float pr = probs[(size_t)p * heads + d / rot];
                /* masked slots have pr == 0 and a finite cache value */
                buf[p] = (pr == 0.f) ? 0.f : orc_half_to_float(v_cache[(size_t)p * dim + d]) * pr;
            }
            v_out[d] = tree_sum(buf, backlog);
        }
        free(buf);
    }
}

/* llava_session.cpp:144-152 */
uint32_t orc_argmax(const float* v, uint32_t n) {
    uint32_t m = 0;
    for (uint32_t i = 0; i < n; i++) if (v[i] > v[m]) m = i;
    return m;
}

/* llava_session.cpp:118-190 */
uint32_t orc_sampler_candidates(const float* logits, uint32_t n_vocab, const uint32_t* tokens,
                                uint32_t n_tokens, float mu, float* probs_out, uint32_t* ids_out,
                                float* kept_sum) {
    const uint32_t repeat_last_n = 64;                 /* llava_session.h:70-76 */
    const float repeat_penalty = 1.1f, alpha_frequency = 0.1f, alpha_presence = 0.0f, temp = 0.8f;
    float* p = (float*)malloc(sizeof(float) * n_vocab);
    memcpy(p, logits, sizeof(float) * n_vocab);
    uint32_t count13 = 0;
    uint32_t first = n_tokens > repeat_last_n ? n_tokens - repeat_last_n : 0;
    for (uint32_t i = first; i < n_tokens; i++) if (tokens[i] == 13) count13++;
    if (count13 && n_vocab > 13) {                     /* only token 13 is penalised, :157-167 */
        if (p[13] <= 0) p[13] *= repeat_penalty; else p[13] /= repeat_penalty;
        p[13] -= alpha_frequency * (float)count13 + alpha_presence;
    }
    float total = 0.f;
    for (uint32_t i = 0; i < n_vocab; i++) { p[i] = expf(p[i] / temp); total += p[i]; }
    float cut = powf(0.5f, mu), new_sum = 0.f;
    uint32_t kept = 0;
    for (uint32_t i = 0; i < n_vocab; i++) {
        p[i] /= total;
        if (p[i] >= cut) {
            new_sum += p[i];
            probs_out[kept] = p[i];
            ids_out[kept] = i;
            kept++;
        }
    }
    *kept_sum = new_sum;
    free(p);
    return kept;
}

float orc_sampler_mu_update(float mu, float p_selected, float kept_sum) {
    const float mirostat_tau = 5.0f, mirostat_eta = 0.1f;
    return mu + mirostat_eta * (mirostat_tau + log2f(p_selected / kept_sum));   /* :193 */
}

/* ------------------------------------------------------------------------ */
/* model file: ggml_file.cpp:17-122                                          */
/* ------------------------------------------------------------------------ */
typedef struct {
    char* name;
    uint32_t type, shape1, shape2;
    uint64_t offset, size;
} orc_tensor;

typedef struct {
    const char* text;
    uint32_t len;
    float score;
} orc_token;

struct orc_model {
    uint8_t* map;
    size_t map_size;
    uint32_t hdr[9];       /* magic, version, vocab, dim, multiple_of, heads, layers, rot, ftype */
    uint32_t ff_size;
    orc_token* tokens;
    orc_tensor* tensors;
    uint32_t n_tensors, cap_tensors;
};

static const orc_tensor* find_tensor(const orc_model* m, const char* name) {
    /* ggml_file.cpp:337-344: exact name, then name + ".weight" */
    for (uint32_t i = 0; i < m->n_tensors; i++) if (!strcmp(m->tensors[i].name, name)) return &m->tensors[i];
    size_t n = strlen(name);
    for (uint32_t i = 0; i < m->n_tensors; i++) {
        const char* t = m->tensors[i].name;
        if (strlen(t) == n + 7 && !memcmp(t, name, n) && !strcmp(t + n, ".weight")) return &m->tensors[i];
    }
    return NULL;
}

orc_model* orc_model_open(const char* path) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) return NULL;
    struct stat st;
    if (fstat(fd, &st) < 0) { close(fd); return NULL; }
    orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
    m->map_size = (size_t)st.st_size;
    m->map = (uint8_t*)mmap(NULL, m->map_size, PROT_READ, MAP_SHARED, fd, 0);
    close(fd);
    if (m->map == MAP_FAILED || m->map_size <= 36) { free(m); return NULL; }
    memcpy(m->hdr, m->map, 36);
    /* ggml_file.cpp:49-53 */
    if (m->hdr[0] != 0x67676a74u || !m->hdr[2] || !m->hdr[5] || !m->hdr[6] || m->hdr[7] * m->hdr[5] != m->hdr[3]) {
        orc_model_close(m);
        return NULL;
    }
    const uint8_t* cur = m->map + 36;
    const uint8_t* end = m->map + m->map_size;
    m->tokens = (orc_token*)calloc(m->hdr[2], sizeof(orc_token));
    for (uint32_t i = 0; i < m->hdr[2]; i++) {            /* ggml_file.cpp:67-77 */
        int32_t len;
        if (cur + 4 > end) { orc_model_close(m); return NULL; }
        memcpy(&len, cur, 4);
        cur += 4;
        if (len < 0 || cur + len + 4 > end) { orc_model_close(m); return NULL; }
        m->tokens[i].text = (const char*)cur;
        m->tokens[i].len = (uint32_t)len;
        cur += len;
        memcpy(&m->tokens[i].score, cur, 4);
        cur += 4;
    }
    while (cur != end) {                                   /* ggml_file.cpp:79-122 */
        uint32_t n_dims, name_len, ftype, shape1, shape2 = 1;
        if (cur + 16 > end) { orc_model_close(m); return NULL; }
        memcpy(&n_dims, cur, 4); memcpy(&name_len, cur + 4, 4); memcpy(&ftype, cur + 8, 4);
        memcpy(&shape1, cur + 12, 4);
        cur += 16;
        if (n_dims < 1 || n_dims > 2) { orc_model_close(m); return NULL; }
        if (n_dims == 2) { shape2 = shape1; memcpy(&shape1, cur, 4); cur += 4; }   /* :86-91 */
        if (!(ftype <= 3 || ftype == 8) || cur + name_len > end) { orc_model_close(m); return NULL; }
        if (m->n_tensors == m->cap_tensors) {
            m->cap_tensors = m->cap_tensors ? m->cap_tensors * 2 : 64;
            m->tensors = (orc_tensor*)realloc(m->tensors, m->cap_tensors * sizeof(orc_tensor));
        }
        orc_tensor* t = &m->tensors[m->n_tensors++];
        t->name = (char*)malloc(name_len + 1);
        memcpy(t->name, cur, name_len);
        t->name[name_len] = 0;
        cur += name_len;
        t->type = ftype; t->shape1 = shape1; t->shape2 = shape2;
        t->offset = ((uint64_t)(cur - m->map) + 31) & ~31ull;                     /* :117-118 */
        /* ggml_file.cpp:162-186: versions other than 1 use the f16-scale block sizes */
        size_t blk = orc_row_bytes((int)ftype, m->hdr[1] == 1 ? 1 : 3, 32);
        if (ftype == ORC_F32 || ftype == ORC_F16) t->size = (uint64_t)shape1 * shape2 * (ftype == ORC_F32 ? 4 : 2);
        else if ((ftype == ORC_Q4_0 || ftype == ORC_Q8_0) && ((uint64_t)shape1 * shape2) % 32 == 0)
            t->size = ((uint64_t)shape1 * shape2) / 32 * blk;
        else { orc_model_close(m); return NULL; }
        if (t->offset + t->size > m->map_size) { orc_model_close(m); return NULL; }
        cur = m->map + t->offset + t->size;
    }
    const orc_tensor* w1 = find_tensor(m, "layers.0.feed_forward.w1");            /* :64 */
    if (!w1) { orc_model_close(m); return NULL; }
    m->ff_size = w1->shape1;
    return m;
}

void orc_model_close(orc_model* m) {
    if (!m) return;
    for (uint32_t i = 0; i < m->n_tensors; i++) free(m->tensors[i].name);
    free(m->tensors);
    free(m->tokens);
    if (m->map && m->map != MAP_FAILED) munmap(m->map, m->map_size);
    free(m);
}

void orc_model_get_info(const orc_model* m, orc_model_info* o) {
    o->file_version = m->hdr[1]; o->vocab_size = m->hdr[2]; o->dim = m->hdr[3];
    o->multiple_of = m->hdr[4]; o->n_heads = m->hdr[5]; o->n_layers = m->hdr[6];
    o->rot = m->hdr[7]; o->ftype = m->hdr[8]; o->ff_size = m->ff_size;
    const orc_tensor* wq = find_tensor(m, "layers.0.attention.wq");
    o->wtype = wq ? wq->type : 0;
    o->n_tensors = m->n_tensors;
}

int orc_model_tensor(const orc_model* m, uint32_t index, char* name, size_t name_cap, uint32_t* type,
                     uint64_t* offset, uint32_t* shape1, uint32_t* shape2, uint64_t* size) {
    if (index >= m->n_tensors) return -1;
    const orc_tensor* t = &m->tensors[index];
    if (name && name_cap) { strncpy(name, t->name, name_cap - 1); name[name_cap - 1] = 0; }
    if (type) *type = t->type;
    if (offset) *offset = t->offset;
    if (shape1) *shape1 = t->shape1;
    if (shape2) *shape2 = t->shape2;
    if (size) *size = t->size;
    return 0;
}

const void* orc_model_tensor_data(const orc_model* m, const char* name) {
    const orc_tensor* t = find_tensor(m, name);
    return t ? m->map + t->offset : NULL;
}

const char* orc_model_token(const orc_model* m, uint32_t id, uint32_t* len, float* score) {
    if (id >= m->hdr[2]) return NULL;
    if (len) *len = m->tokens[id].len;
    if (score) *score = m->tokens[id].score;
    return m->tokens[id].text;
}

/* ------------------------------------------------------------------------ */
/* session: llava_session.cpp                                                */
/* ------------------------------------------------------------------------ */
#define ORC_MIN_BACKLOG 128u      /* llava_session.cpp:23 */
#define ORC_MAX_BACKLOG 2048u     /* llava_session.cpp:24 */

struct orc_session {
    orc_model* m;
    uint32_t wgs;
    uint32_t dim, ff, heads, rot, layers, vocab;
    int wtype, version;
    uint32_t backlog;
    uint32_t* tokens;
    uint32_t n_tokens, in_cache;
    uint16_t** k_cache;          /* per layer [ORC_MAX_BACKLOG][dim], zero filled (llava_layer_session_data.cpp:126-127) */
    uint16_t** v_cache;
    float *x, *h, *q, *k, *v, *vout, *ffr, *scores, *layer_out;
    float* cs_table;             /* [ORC_MAX_BACKLOG][rot/2][2]: cos, sin per (distance, pair) */
};

static uint32_t dim_workers(uint32_t dim) { return dim == 4096 ? 128 : 32; }   /* llava_session.cpp:357-363 */

orc_session* orc_session_create(orc_model* m, uint32_t wgs) {
    orc_model_info in;
    orc_model_get_info(m, &in);
    /* llava_session.cpp:357-375: only these geometries exist in the reference */
    if (!((in.dim == 4096 || in.dim == 5120) && (in.ff_size == 11008 || in.ff_size == 13824))) return NULL;
    if (wgs == 0 || (wgs & (wgs - 1))) return NULL;                          /* llava_context.cpp:259-260 */
    orc_session* s = (orc_session*)calloc(1, sizeof(orc_session));
    s->m = m; s->wgs = wgs;
    s->dim = in.dim; s->ff = in.ff_size; s->heads = in.n_heads; s->rot = in.rot;
    s->layers = in.n_layers; s->vocab = in.vocab_size;
    s->wtype = (int)in.wtype; s->version = (int)in.file_version;
    s->backlog = ORC_MIN_BACKLOG;
    s->tokens = (uint32_t*)calloc(ORC_MAX_BACKLOG, 4);
    s->k_cache = (uint16_t**)calloc(s->layers, sizeof(void*));
    s->v_cache = (uint16_t**)calloc(s->layers, sizeof(void*));
    for (uint32_t l = 0; l < s->layers; l++) {
        s->k_cache[l] = (uint16_t*)calloc((size_t)ORC_MAX_BACKLOG * s->dim, 2);
        s->v_cache[l] = (uint16_t*)calloc((size_t)ORC_MAX_BACKLOG * s->dim, 2);
    }
    s->x = (float*)calloc(s->dim, 4); s->h = (float*)calloc(s->dim, 4);
    s->q = (float*)calloc(s->dim, 4); s->k = (float*)calloc(s->dim, 4);
    s->v = (float*)calloc(s->dim, 4); s->vout = (float*)calloc(s->dim, 4);
    s->ffr = (float*)calloc(s->ff, 4);
    s->scores = (float*)calloc((size_t)ORC_MAX_BACKLOG * s->heads, 4);
    s->layer_out = (float*)calloc((size_t)s->layers * s->dim, 4);
    uint32_t half_rot = s->rot / 2;
    s->cs_table = (float*)malloc((size_t)ORC_MAX_BACKLOG * half_rot * 2 * sizeof(float));
    for (uint32_t d = 0; d < ORC_MAX_BACKLOG; d++)
        for (uint32_t i = 0; i < half_rot; i++)
            rope_cs(d, i, half_rot, &s->cs_table[((size_t)d * half_rot + i) * 2],
                    &s->cs_table[((size_t)d * half_rot + i) * 2 + 1]);
    return s;
}

void orc_session_destroy(orc_session* s) {
    if (!s) return;
    for (uint32_t l = 0; l < s->layers; l++) { free(s->k_cache[l]); free(s->v_cache[l]); }
    free(s->k_cache); free(s->v_cache); free(s->tokens);
    free(s->x); free(s->h); free(s->q); free(s->k); free(s->v); free(s->vout);
    free(s->ffr); free(s->scores); free(s->layer_out); free(s->cs_table);
    free(s);
}

/* llava_session.cpp:284-297 */
int orc_session_push_token(orc_session* s, uint32_t token) {
    if (token >= s->vocab) return 0;
    if (s->n_tokens == s->backlog) {
        if (s->backlog == ORC_MAX_BACKLOG) return 0;
        s->backlog *= 2;        /* grown caches keep their rows and zero the tail (llava_layer_session_data.cpp:100-106) */
    }
    s->tokens[s->n_tokens++] = token;
    return 1;
}

/* llava_session.cpp:390-395 */
void orc_session_rewind(orc_session* s, uint32_t n) {
    if (n < s->n_tokens) {
        s->n_tokens = n;
        if (s->in_cache > n) s->in_cache = n;
    }
}

uint32_t orc_session_token_count(const orc_session* s) { return s->n_tokens; }
uint32_t orc_session_backlog(const orc_session* s) { return s->backlog; }
const uint16_t* orc_session_k_cache(const orc_session* s, uint32_t l) { return s->k_cache[l]; }
const uint16_t* orc_session_v_cache(const orc_session* s, uint32_t l) { return s->v_cache[l]; }
const float* orc_session_residual(const orc_session* s) { return s->x; }
const float* orc_session_layer_outputs(const orc_session* s) { return s->layer_out; }

static const void* layer_tensor(const orc_session* s, uint32_t l, const char* leaf) {
    char name[128];
    snprintf(name, sizeof name, "layers.%u.%s", l, leaf);     /* llava_layer.cpp:13-22 */
    return orc_model_tensor_data(s->m, name);
}

/* One token at absolute position P: llava_layer.cpp:53-73 per layer. */
static int eval_token(orc_session* s, uint32_t P) {
    uint32_t dim = s->dim, ff = s->ff, B = s->backlog;
    uint32_t wd = dim_workers(dim), wf = 128;                 /* llava_session.cpp:357-371 */
    int T = s->wtype, V = s->version;
    /* llava_session.cpp:211-223: embedding row dequantised on the host */
    const orc_tensor* emb = find_tensor(s->m, "tok_embeddings");
    if (!emb) return -1;
    size_t erow = emb->size / s->vocab;
    if (orc_dequant(s->m->map + emb->offset + (size_t)s->tokens[P] * erow, (int)emb->type, V, s->x, dim)) return -1;
    for (uint32_t l = 0; l < s->layers; l++) {
        const float* an = (const float*)layer_tensor(s, l, "attention_norm");
        const float* fn = (const float*)layer_tensor(s, l, "ffn_norm");
        const void *wq = layer_tensor(s, l, "attention.wq"), *wk = layer_tensor(s, l, "attention.wk");
        const void *wv = layer_tensor(s, l, "attention.wv"), *wo = layer_tensor(s, l, "attention.wo");
        const void *w1 = layer_tensor(s, l, "feed_forward.w1"), *w2 = layer_tensor(s, l, "feed_forward.w2");
        const void* w3 = layer_tensor(s, l, "feed_forward.w3");
        if (!an || !fn || !wq || !wk || !wv || !wo || !w1 || !w2 || !w3) return -1;
        orc_norm(s->h, s->x, an, dim, s->wgs);
        if (orc_gemv(s->k, wk, T, V, s->h, dim, dim, wd, 0)) return -1;
        if (orc_gemv(s->q, wq, T, V, s->h, dim, dim, wd, 0)) return -1;
        if (orc_gemv(s->v, wv, T, V, s->h, dim, dim, wd, 0)) return -1;
        orc_kv_append(s->k_cache[l], s->k, P, dim);
        orc_kv_append(s->v_cache[l], s->v, P, dim);
        mhsa_with_table(s->scores, s->k_cache[l], s->q, P, P + 1, s->heads, s->rot, s->cs_table);
        orc_softmax(s->scores, P, B, s->heads, s->rot);
        orc_kqv(s->vout, s->v_cache[l], s->scores, B, s->heads, s->rot);
        if (orc_gemv(s->x, wo, T, V, s->vout, dim, dim, wd, 1)) return -1;
        orc_norm(s->h, s->x, fn, dim, s->wgs);
        if (orc_gemv_silu(s->ffr, w3, w1, T, V, s->h, ff, dim, wd)) return -1;
        if (orc_gemv(s->x, w2, T, V, s->ffr, dim, ff, wf, 1)) return -1;
        memcpy(s->layer_out + (size_t)l * dim, s->x, (size_t)dim * 4);
    }
    return 0;
}

int orc_session_eval(orc_session* s, float* logits_out) {
    if (s->in_cache >= s->n_tokens) return -1;                /* "GPU is already in sync", llava_session.cpp:200-203 */
    if (s->n_tokens > s->backlog) return -1;                  /* :214-217 */
    while (s->in_cache < s->n_tokens) {
        if (eval_token(s, s->in_cache)) return -1;
        s->in_cache++;
    }
    /* llava_command_buffer.cpp:38-39: final norm and output head */
    const float* nw = (const float*)orc_model_tensor_data(s->m, "norm");
    const orc_tensor* ow = find_tensor(s->m, "output");
    if (!nw || !ow) return -1;
    orc_norm(s->h, s->x, nw, s->dim, s->wgs);
    return orc_gemv(logits_out, s->m->map + ow->offset, (int)ow->type, s->version, s->h, s->vocab, s->dim,
                    dim_workers(s->dim), 0);
}
