#include "tp_shard.h"

#include <cstring>

namespace {
u32 block_bytes(ggml_value_type t) { return t == ggml_value_type::q4_0 ? 18 : (t == ggml_value_type::q8_0 ? 34 : 0); }
}  // namespace

tp_shard_shape tp_shape(ggml_value_type type, u32 rows, u32 cols, tp_split how, u32 rank, u32 n_ranks) {
    tp_shard_shape s;
    const u32 bb = block_bytes(type);
    if (bb == 0 || n_ranks == 0 || rank >= n_ranks || cols % 32 != 0) return s;
    const u32 nb = cols / 32;
    switch (how) {
        case tp_split::none:
            s.rows = rows; s.cols = s.cols_used = cols;
            break;
        case tp_split::rows:
            if (rows % n_ranks != 0) return s;
            s.rows = rows / n_ranks; s.cols = s.cols_used = cols;
            break;
        case tp_split::columns: {
            if (nb % n_ranks != 0) return s;
            const u32 local = nb / n_ranks;
            s.rows = rows;
            s.cols_used = local * 32;
            s.cols = (local + 7) / 8 * 8 * 32;
            break;
        }
    }
    s.bytes = size_t(s.rows) * (s.cols / 32) * bb;
    s.valid = true;
    return s;
}

bool tp_pack(const u8* src, ggml_value_type type, u32 rows, u32 cols, tp_split how, u32 rank, u32 n_ranks, u8* dst) {
    const tp_shard_shape s = tp_shape(type, rows, cols, how, rank, n_ranks);
    if (!s.valid) return false;
    const u32 bb = block_bytes(type);
    const size_t src_row = size_t(cols / 32) * bb;
    if (how == tp_split::none) {
        memcpy(dst, src, s.bytes);
    } else if (how == tp_split::rows) {
        memcpy(dst, src + size_t(rank) * s.rows * src_row, s.bytes);
    } else {
        const u32 used = s.cols_used / 32, padded = s.cols / 32;
        const size_t dst_row = size_t(padded) * bb;
        for (u32 r = 0; r < rows; ++r) {
            u8* out = dst + size_t(r) * dst_row;
            memcpy(out, src + size_t(r) * src_row + size_t(rank) * used * bb, size_t(used) * bb);
            for (u32 b = used; b < padded; ++b) {          // zero blocks: scale 0, every weight 0
                u8* blk = out + size_t(b) * bb;
                blk[0] = blk[1] = 0;
                memset(blk + 2, type == ggml_value_type::q4_0 ? 0x88 : 0x00, bb - 2);
            }
        }
    }
    return true;
}

u64 tp_snapshot_slice_offset(u32 n_tokens, u32 dim, u32 layer, u32 which, u32 row, u32 rank, u32 n_ranks) {
    const u64 header = 4 + u64(n_tokens) * 4, per_cache = u64(n_tokens) * dim * 2;
    return header + (u64(layer) * 2 + which) * per_cache + u64(row) * dim * 2 + u64(rank) * (dim / n_ranks) * 2;
}

u64 tp_snapshot_file_size(u32 n_tokens, u32 dim, u32 n_layers) {
    return 4 + u64(n_tokens) * 4 + u64(n_layers) * 2 * n_tokens * dim * 2;
}
