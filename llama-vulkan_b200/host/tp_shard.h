// Tensor-parallel sharding of the decoder's matrices (one rank per GPU).
//   rows:    wq, wk, wv, w1, w3 -- rank r keeps rows [r*rows/n, (r+1)*rows/n): whole heads, a
//            contiguous byte range of the file tensor.
//   columns: wo, w2 -- rank r keeps blocks [r*nb/n, (r+1)*nb/n) of every row, re-packed into a
//            dense [rows][local blocks] matrix whose rows are padded with zero blocks to a
//            multiple of 8 blocks, so that every row starts on a 16-byte boundary (what the
//            bulk copies of the GEMV kernel need).  The matching activation slice is padded
//            with zeros to the same length.
// The reference is single-device; see llava_layer.cpp:10-23 for the tensors involved.
#ifndef LLAVA_B200_TP_SHARD_H
#define LLAVA_B200_TP_SHARD_H

#include <cstddef>

#include "types.h"

enum class tp_split : u32 { none = 0, rows = 1, columns = 2 };

struct tp_shard_shape {
    u32 rows = 0;          // local rows
    u32 cols = 0;          // local columns including padding
    u32 cols_used = 0;     // local columns that carry weights
    size_t bytes = 0;      // of the local matrix
    bool valid = false;
};

// false in .valid when the tensor cannot be split that way (rows or blocks not divisible)
tp_shard_shape tp_shape(ggml_value_type type, u32 rows, u32 cols, tp_split how, u32 rank, u32 n_ranks);
// writes the local matrix of `rank` to dst (tp_shape(...).bytes bytes) from the whole tensor at src
bool tp_pack(const u8* src, ggml_value_type type, u32 rows, u32 cols, tp_split how, u32 rank, u32 n_ranks, u8* dst);

#endif
