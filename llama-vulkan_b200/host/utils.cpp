#include "utils.h"

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <unistd.h>

const char* ftype_name(ggml_value_type type) {
    static const struct { ggml_value_type t; const char* n; } names[] = {
        {ggml_value_type::f32, "f32"},   {ggml_value_type::f16, "f16"},   {ggml_value_type::q4_0, "q4_0"},
        {ggml_value_type::q4_1, "q4_1"}, {ggml_value_type::q5_0, "q5_0"}, {ggml_value_type::q5_1, "q5_1"},
        {ggml_value_type::q8_0, "q8_0"}, {ggml_value_type::q8_1, "q8_1"}, {ggml_value_type::q2_K, "q2_K"},
        {ggml_value_type::q3_K, "q3_K"}, {ggml_value_type::q4_K, "q4_K"}, {ggml_value_type::q5_K, "q5_K"},
        {ggml_value_type::q6_K, "q6_K"}, {ggml_value_type::q8_K, "q8_K"},
    };
    for (const auto& e : names) if (e.t == type) return e.n;
    return nullptr;
}

bool ulog2(u32 n, u32* out) {
    if (n == 0 || (n & (n - 1)) != 0) return false;
    u32 bits = 0;
    while ((n >> bits) != 1) ++bits;
    *out = bits;
    return true;
}

bool ends_with(const std::string& a, const std::string& b) {
    return a.size() >= b.size() && a.compare(a.size() - b.size(), b.size(), b) == 0;
}

bool starts_with(const std::string& a, const std::string& b) {
    return a.size() >= b.size() && a.compare(0, b.size(), b) == 0;
}

size_t read_noshort(int fd, void* dst, size_t sz) {
    size_t done = 0;
    while (done < sz) {
        const ssize_t r = ::read(fd, static_cast<u8*>(dst) + done, sz - done);
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) {
            if (r < 0) perror("read_noshort");
            break;
        }
        done += static_cast<size_t>(r);
    }
    return done;
}

size_t write_noshort(int fd, const void* src, size_t sz) {
    size_t done = 0;
    while (done < sz) {
        const ssize_t r = ::write(fd, static_cast<const u8*>(src) + done, sz - done);
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) {
            perror("write_noshort");
            break;
        }
        done += static_cast<size_t>(r);
    }
    return done;
}

size_t pread_noshort(int fd, void* dst, size_t sz, long long offset) {
    size_t done = 0;
    while (done < sz) {
        const ssize_t r = ::pread(fd, static_cast<u8*>(dst) + done, sz - done, static_cast<off_t>(offset) + static_cast<off_t>(done));
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) {
            if (r < 0) perror("pread_noshort");
            break;
        }
        done += static_cast<size_t>(r);
    }
    return done;
}

size_t pwrite_noshort(int fd, const void* src, size_t sz, long long offset) {
    size_t done = 0;
    while (done < sz) {
        const ssize_t r = ::pwrite(fd, static_cast<const u8*>(src) + done, sz - done, static_cast<off_t>(offset) + static_cast<off_t>(done));
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) {
            perror("pwrite_noshort");
            break;
        }
        done += static_cast<size_t>(r);
    }
    return done;
}

float half_to_float(u16 h) {
    const u32 sign = (h & 0x8000u) << 16;
    u32 exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {                                   // subnormal: renormalise
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            bits = sign | ((113u - shift) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

u16 float_to_half(float f) {
    u32 x;
    std::memcpy(&x, &f, 4);
    const u32 sign = (x >> 16) & 0x8000u, a = x & 0x7fffffffu;
    if (a >= 0x7f800000u) return static_cast<u16>(sign | 0x7c00u | (a > 0x7f800000u ? 0x200u : 0u));
    if (a >= 0x477ff000u) return static_cast<u16>(sign | 0x7c00u);
    if (a < 0x33000000u) return static_cast<u16>(sign);
    u32 q, rem, halfway;
    if (a < 0x38800000u) {
        const int shift = 126 - static_cast<int>(a >> 23);
        const u32 man = (a & 0x7fffffu) | 0x800000u;
        q = man >> shift;
        rem = man & ((1u << shift) - 1u);
        halfway = 1u << (shift - 1);
    } else {
        q = (((a >> 23) - 112u) << 10) | ((a & 0x7fffffu) >> 13);
        rem = a & 0x1fffu;
        halfway = 0x1000u;
    }
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    return static_cast<u16>(sign | q);
}
