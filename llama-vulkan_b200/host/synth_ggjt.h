// Writer of synthetic ggjt-v3 model files with LLaMA geometry: seeded N(0, 0.02)
// matrices quantised to q4_0 or q8_0, N(1, 0.01) norm vectors, and a synthetic
// vocabulary.  Stands in for real checkpoints in tests and benchmarks.
#ifndef LLAVA_B200_SYNTH_GGJT_H
#define LLAVA_B200_SYNTH_GGJT_H

#include <string>

#include "types.h"

struct synth_config {
    u32 dim = 4096;
    u32 n_heads = 32;
    u32 n_layers = 2;
    u32 ff_size = 11008;
    u32 vocab_size = 32000;
    ggml_value_type wtype = ggml_value_type::q4_0;    // q4_0 or q8_0
    u64 seed = 1234;
    u32 threads = 0;                                  // 0: all hardware threads
    u32 file_version = 3;                             // 1: q4_0 blocks of 20 bytes (f32 scale = absmax / 8, byte j = elements 2j, 2j+1)
    bool f32_embeddings = false;                      // tok_embeddings stored as f32 instead of quantised
};

// Standard normal sample number `element` of stream (`seed`, `tensor`): a pure
// function of its arguments, so files can be generated in parallel and tensors
// regenerated independently.
float synth_normal(u64 seed, u32 tensor, u64 element);

// Quantises `count` (multiple of 32) floats into ggjt-v3 blocks: scale =
// f16(absmax / 8) with 4-bit values offset by 8 (element j in the low nibble of
// byte j, element j + 16 in the high nibble), or f16(absmax / 127) with int8.
void synth_quantize(const float* src, size_t count, ggml_value_type wtype, u8* dst);
// The same values as version-1 q4_0 blocks (llava_buffer.cpp:350-359 of the reference).
void synth_quantize_v1(const float* src, size_t count, u8* dst);

// Total file size for a configuration (0 if the configuration is invalid).
u64 synth_file_size(const synth_config& cfg);

bool synth_write_ggjt(const std::string& path, const synth_config& cfg, std::string* error);

#endif
