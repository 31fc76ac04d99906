// Small helpers (counterpart of the reference's utils.h without the SPIR-V parts).
#ifndef LLAVA_B200_UTILS_H
#define LLAVA_B200_UTILS_H

#include <cstddef>
#include <string>

#include "types.h"

const char* ftype_name(ggml_value_type type);           // utils.cpp:6-38
inline u64 updiv(u64 a, u64 b) { return (a + b - 1) / b; }   // utils.h:9-11
// log2 of a power of two; returns false for 0 or a non power of two
// (the reference asserts instead, utils.cpp:52-61)
bool ulog2(u32 n, u32* out);
bool ends_with(const std::string& a, const std::string& b);
bool starts_with(const std::string& a, const std::string& b);
// read/write all of `sz` bytes unless the descriptor fails; return bytes moved (utils.cpp:63-90)
size_t read_noshort(int fd, void* dst, size_t sz);
size_t write_noshort(int fd, const void* src, size_t sz);
// the same at a file offset (the descriptor's position is left alone)
size_t pread_noshort(int fd, void* dst, size_t sz, long long offset);
size_t pwrite_noshort(int fd, const void* src, size_t sz, long long offset);
// IEEE binary16 <-> binary32 on the host
float half_to_float(u16 h);
u16 float_to_half(float f);        // round to nearest even

#endif
