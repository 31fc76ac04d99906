#include "llava_buffer.h"

#include <cstring>
#include <iostream>
#include <vector>

#include "llava_context.h"
#include "../../include/lv_b200.h"
#include "llava_device_memory.h"
#include "utils.h"

using namespace std;

namespace {
constexpr size_t kBufferAlignment = 256;      // keeps every tensor 16-byte aligned for bulk copies

size_t gcd_sz(size_t a, size_t b) { return b == 0 ? a : gcd_sz(b, a % b); }

// A quantised matrix starts at a multiple of its row size (and of 256 bytes) from the arena's base.  Every
// matrix of one row size in an arena is then a row range of ONE 2-D view [arena bytes / row size][row size]
// of the arena, so a single TMA tensor map per row size addresses them all (lv_step_plan_create).
size_t matrix_alignment(ggml_value_type type, u32 cols) {
    const size_t block = type == ggml_value_type::q4_0 ? 18 : type == ggml_value_type::q8_0 ? 34 : 0;
    if (block == 0 || cols % 32 != 0) return kBufferAlignment;
    const size_t row = size_t(cols / 32) * block;
    return row / gcd_sz(row, kBufferAlignment) * kBufferAlignment;
}
}

llava_buffer::llava_buffer(llava_context* _context, ggml_value_type _type, u32 shape1, u32 shape2,
                           llava_device_memory* _device_memory, string _name)
    : context(_context), pretty_name(std::move(_name)), type(_type), shape(shape1, shape2),
      device_memory_is_shared(_device_memory != nullptr),
      device_memory(_device_memory ? _device_memory : new llava_device_memory(_context)), model_version(0),
      file_shape(shape1, shape2), used_cols(shape2) {
    device_memory->register_llava_buffer(this);
    bytes = size_t(shape1) * shape2 * (type == ggml_value_type::f32 ? 4 : 2);
    offset = device_memory->register_buffer(kBufferAlignment, bytes);
    if (!device_memory_is_shared) device_memory->freeze();
}

llava_buffer::llava_buffer(llava_context* _context, const ggml_data_descriptor& table, llava_device_memory* _device_memory)
    : context(_context), backing_buffer_name(table.name), type(table.ftype), shape(table.shape1, table.shape2),
      device_memory_is_shared(_device_memory != nullptr),
      device_memory(_device_memory ? _device_memory : new llava_device_memory(_context)),
      model_version(table.model_version), file_shape(table.shape1, table.shape2), used_cols(table.shape2) {
    device_memory->register_llava_buffer(this);
    bytes = table.size;
    offset = device_memory->register_buffer(model_version == 3 ? matrix_alignment(type, shape.second) : kBufferAlignment, bytes);
    if (!device_memory_is_shared) device_memory->freeze();
}

static std::pair<u32, u32> local_shape(const ggml_data_descriptor& t, tp_split how, u32 rank, u32 n) {
    const tp_shard_shape s = tp_shape(t.ftype, t.shape1, t.shape2, how, rank, n);
    return s.valid ? std::make_pair(s.rows, s.cols) : std::make_pair(0u, 0u);
}

llava_buffer::llava_buffer(llava_context* _context, const ggml_data_descriptor& table, llava_device_memory* _device_memory,
                           tp_split how, u32 rank, u32 n_ranks)
    : context(_context), backing_buffer_name(table.name), type(table.ftype), shape(local_shape(table, how, rank, n_ranks)),
      device_memory_is_shared(_device_memory != nullptr),
      device_memory(_device_memory ? _device_memory : new llava_device_memory(_context)),
      model_version(table.model_version), split(how), tp_rank(rank), tp_ranks(n_ranks), file_shape(table.shape1, table.shape2) {
    device_memory->register_llava_buffer(this);
    const tp_shard_shape s = tp_shape(table.ftype, table.shape1, table.shape2, how, rank, n_ranks);
    bytes = s.bytes;
    used_cols = s.cols_used;
    offset = device_memory->register_buffer(model_version == 3 ? matrix_alignment(type, shape.second) : kBufferAlignment, bytes ? bytes : 16);
    if (!device_memory_is_shared) device_memory->freeze();
}

llava_buffer::~llava_buffer() {
    device_memory->forget_llava_buffer(this);
    if (!device_memory_is_shared) delete device_memory;
}

bool llava_buffer::is_allocated() const { return device_memory->is_frozen(); }

void* llava_buffer::device_ptr() const { return is_allocated() ? device_memory->device_base() + offset : nullptr; }

bool llava_buffer::write_raw(size_t byte_offset, const void* src, size_t size) const {
    return byte_offset + size <= bytes && device_memory->write(offset + byte_offset, src, size);
}

bool llava_buffer::read_raw(size_t byte_offset, void* dst, size_t size) const {
    return byte_offset + size <= bytes && device_memory->read(offset + byte_offset, dst, size);
}

// The dequantisation formulas of the reference's write_f32 (llava_buffer.cpp:350-397):
//   q4_0, version 1: f32 scale d, byte j holds elements 2j (low nibble) and 2j+1 (high)
//   q4_0, version 3: f16 scale d, byte j holds elements j (low nibble) and j+16 (high)
//   q8_0, version 3: f16 scale d, 32 signed bytes
// each weight being (integer value [- 8 for q4_0]) * d.
bool dequantize_to_f32(const void* in_buf, ggml_value_type intype, u32 model_version, float* out, u32 count) {
    const u8* in = static_cast<const u8*>(in_buf);
    if (intype == ggml_value_type::f32) {
        memcpy(out, in, size_t(count) * 4);
        return true;
    }
    if (count % 32 != 0) return false;
    const u32 blocks = count / 32;
    if (intype == ggml_value_type::q4_0 && (model_version == 1 || model_version == 3)) {
        const bool v1 = model_version == 1;
        for (u32 b = 0; b < blocks; ++b) {
            const u8* blk = in + size_t(b) * (v1 ? 20 : 18);
            float d;
            if (v1) {
                memcpy(&d, blk, 4);
            } else {
                u16 h;
                memcpy(&h, blk, 2);
                d = half_to_float(h);
            }
            const u8* qs = blk + (v1 ? 4 : 2);
            for (u32 j = 0; j < 16; ++j) {
                const float lo = float(int(qs[j] & 0xf) - 8) * d, hi = float(int(qs[j] >> 4) - 8) * d;
                if (v1) { out[b * 32 + 2 * j] = lo; out[b * 32 + 2 * j + 1] = hi; }
                else    { out[b * 32 + j] = lo;     out[b * 32 + j + 16] = hi; }
            }
        }
        return true;
    }
    if (intype == ggml_value_type::q8_0 && model_version == 3) {
        for (u32 b = 0; b < blocks; ++b) {
            const u8* blk = in + size_t(b) * 34;
            u16 h;
            memcpy(&h, blk, 2);
            const float d = half_to_float(h);
            for (u32 j = 0; j < 32; ++j) out[b * 32 + j] = float(int(int8_t(blk[2 + j]))) * d;
        }
        return true;
    }
    return false;
}

bool llava_buffer::write_f32(const void* in_buf, ggml_value_type intype, u32 version, u32 f32_offset, u32 f32_count) const {
    if (!is_allocated() || type != ggml_value_type::f32) return false;
    if (f32_count == 0) return true;
    const u64 capacity = u64(shape.first) * shape.second;
    if (f32_offset >= capacity || u64(f32_offset) + f32_count > capacity) return false;
    vector<float> tmp(f32_count);
    if (!dequantize_to_f32(in_buf, intype, version, tmp.data(), f32_count)) return false;
    return write_raw(size_t(f32_offset) * 4, tmp.data(), size_t(f32_count) * 4);
}

bool llava_buffer::write_full(const void* in_buf, ggml_value_type intype, u32 version) const {
    return write_f32(in_buf, intype, version, 0, shape.first * shape.second);
}

bool llava_buffer::load_to_gpu() {
    if (backing_buffer_name.empty()) return true;
    if (!is_allocated()) return false;
    const ggml_file* model = context->get_model();
    const ggml_data_descriptor& table = model->get_buffer_descriptor(backing_buffer_name);
    if (split == tp_split::none) return context->upload_from_host(device_ptr(), model->data() + table.offset, table.size);
    if (bytes == 0) return false;                      // the tensor cannot be split this way
    if (split == tp_split::rows)                       // a contiguous range of the file tensor
        return context->upload_from_host(device_ptr(), model->data() + table.offset + size_t(tp_rank) * bytes, bytes);
    std::vector<u8> packed(bytes);
    return tp_pack(model->data() + table.offset, type, file_shape.first, file_shape.second, split, tp_rank, tp_ranks, packed.data()) &&
           context->upload_from_host(device_ptr(), packed.data(), bytes);
}

void llava_buffer::dump_raw(int out_fd, const string& name) {
    if (type != ggml_value_type::f32) return;
    // record: shape.first, shape.second, type, name, NUL, zero padding to a multiple of 32 bytes, data
    const u32 header_size = u32((12 + name.size() + 1 + 31) & ~size_t(31));
    vector<u8> header(header_size, 0);
    const u32 t = u32(type);
    memcpy(header.data(), &shape.first, 4);
    memcpy(header.data() + 4, &shape.second, 4);
    memcpy(header.data() + 8, &t, 4);
    memcpy(header.data() + 12, name.data(), name.size());
    write_noshort(out_fd, header.data(), header.size());
    vector<u8> data(bytes);
    if (read_raw(0, data.data(), bytes)) write_noshort(out_fd, data.data(), data.size());
}

bool llava_buffer::weight_buffer_is_quantised() const {
    return weight_buffer_is_f16() || (type == ggml_value_type::q4_0 && model_version == 1);
}

// Version-1 files store q4_0 with an f32 scale and interleaved nibbles (llava_buffer.cpp:66-71,350-359 of the
// reference); the kernels take that layout under a code of its own.
int llava_buffer::kernel_type() const {
    return (type == ggml_value_type::q4_0 && model_version == 1) ? LV_TYPE_Q4_0_V1 : int(type);
}

bool llava_buffer::weight_buffer_is_f16() const {
    return (type == ggml_value_type::q4_0 || type == ggml_value_type::q8_0) && model_version != 1;
}
