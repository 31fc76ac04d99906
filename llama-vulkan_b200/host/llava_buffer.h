// Typed 2-D buffer inside a device arena.  Weight matrices keep the GGML block
// layout of the file (one sub-buffer), unlike the reference, which splits them
// into scale and quant sub-buffers and re-packs rows in groups of four
// (llava_buffer.cpp:179-325).
#ifndef LLAVA_B200_BUFFER_H
#define LLAVA_B200_BUFFER_H

#include <string>
#include <utility>

#include "ggml_file.h"
#include "tp_shard.h"
#include "types.h"

class llava_buffer {
public:
    // anonymous read-write f32 / f16 buffer of shape1 x shape2 elements
    llava_buffer(llava_context* context, ggml_value_type type, u32 shape1, u32 shape2 = 1,
                 llava_device_memory* device_memory = nullptr, std::string name = "");
    // tensor of the model file (shape1 rows of shape2 columns)
    llava_buffer(llava_context* context, const ggml_data_descriptor& table, llava_device_memory* device_memory = nullptr);
    // shard of a file matrix for rank `rank` of `n_ranks` (see tp_shard.h); shape = local shape
    llava_buffer(llava_context* context, const ggml_data_descriptor& table, llava_device_memory* device_memory,
                 tp_split how, u32 rank, u32 n_ranks);
    ~llava_buffer();
    llava_buffer(const llava_buffer&) = delete;
    llava_buffer& operator=(const llava_buffer&) = delete;

    bool is_allocated() const;
    void* device_ptr() const;                     // valid once the arena is frozen
    size_t byte_size() const { return bytes; }
    size_t arena_offset() const { return offset; }

    // Dequantises `f32_count` values from `in_buf` (type `intype`, file version
    // `model_version`) on the host and stores them at element `f32_offset`
    // (llava_buffer.cpp:339-401).  Only for f32 buffers.
    bool write_f32(const void* in_buf, ggml_value_type intype, u32 model_version, u32 f32_offset, u32 f32_count) const;
    bool write_full(const void* in_buf, ggml_value_type intype, u32 model_version) const;
    bool write_raw(size_t byte_offset, const void* src, size_t size) const;
    bool read_raw(size_t byte_offset, void* dst, size_t size) const;
    bool load_to_gpu();                           // file tensor -> device, layout unchanged
    void dump_raw(int out_fd, const std::string& name);   // one trace-frame record (llava_buffer.cpp:497-522)
    const std::string& get_pretty_name() const { return pretty_name; }
    bool weight_buffer_is_f16() const;            // block scale stored as f16 (every ggjt v3 file)
    bool weight_buffer_is_quantised() const;      // a block layout the kernels read: q4_0 / q8_0 of version 3, q4_0 of version 1
    int kernel_type() const;                      // type code for the lv_* entry points: the GGML code, or LV_TYPE_Q4_0_V1

    llava_context* const context;
    const std::string backing_buffer_name;
    const std::string pretty_name;
    const ggml_value_type type;
    const std::pair<u32, u32> shape;
    const bool device_memory_is_shared;
    llava_device_memory* const device_memory;
    const u32 model_version;
    const tp_split split = tp_split::none;
    const u32 tp_rank = 0, tp_ranks = 1;
    const std::pair<u32, u32> file_shape;      // shape of the whole tensor in the file
    u32 cols_used() const { return used_cols; }   // local columns that carry weights (< shape.second when padded)

private:
    u32 used_cols = 0;
    size_t bytes = 0;
    size_t offset = 0;
};

// Host-side dequantisation of `count` weights (llava_buffer.cpp:339-401); false for
// combinations the reference rejects as well.
bool dequantize_to_f32(const void* in_buf, ggml_value_type intype, u32 model_version, float* out, u32 count);

#endif
