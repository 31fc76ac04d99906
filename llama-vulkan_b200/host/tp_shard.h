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

// Snapshot files keep the reference's layout (llava_session.cpp:447-500): {u32 n; u32 tokens[n]; per layer: K rows
// [n][dim] f16, V rows [n][dim] f16}.  A rank holds the columns [rank * dim / n_ranks, (rank + 1) * dim / n_ranks) of
// every cache row.  Byte offset of that slice of row `row` of cache `which` (0 = K, 1 = V) of layer `layer`, and the
// size of the whole file.
u64 tp_snapshot_slice_offset(u32 n_tokens, u32 dim, u32 layer, u32 which, u32 row, u32 rank, u32 n_ranks);
u64 tp_snapshot_file_size(u32 n_tokens, u32 dim, u32 n_layers);

#endif
