// ggjt model file: memory-mapped header, vocabulary and tensor table, plus the
// SentencePiece-style tokenizer.  Same public surface as the reference's
// ggml_file (ggml_file.h:51-57); malformed files make is_open() false instead
// of tripping asserts.
#ifndef LLAVA_B200_GGML_FILE_H
#define LLAVA_B200_GGML_FILE_H

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "types.h"

struct ggml_header {               // ggml_file.h:12-22
    u32 magic;
    u32 file_version;
    u32 vocab_size;
    u32 dim;
    u32 multiple_of;
    u32 n_heads;
    u32 n_layers;
    u32 rot;
    u32 ftype;
} __attribute__((__packed__));

struct ggml_token {
    std::string text;
    float score;
};

class ggml_data_descriptor {       // ggml_file.h:29-41
public:
    ggml_data_descriptor(std::string name, ggml_value_type ftype, u32 model_version, size_t offset, u32 shape1, u32 shape2);
    std::string name;
    ggml_value_type ftype;
    u32 model_version;
    size_t offset;     // of the data in the file, 32-byte aligned
    u32 shape1;        // rows (length for 1-D tensors)
    u32 shape2;        // columns (1 for 1-D tensors)
    size_t size;       // bytes in the file; 0 for an unsupported type
    static size_t size_in_file(ggml_value_type ftype, u32 model_version, u64 elements);
};

class ggml_file {
public:
    explicit ggml_file(const char* filepath);
    ~ggml_file();
    ggml_file(const ggml_file&) = delete;
    ggml_file& operator=(const ggml_file&) = delete;

    void print_info() const;
    void tokenize(std::vector<uint32_t>& output, const std::string& text, bool bos) const;
    std::string tokens_to_text(u32 const* tokens, u32 count) const;
    // looks up `s`, then `s + ".weight"`; nullptr when absent
    const ggml_data_descriptor* find_buffer_descriptor(const std::string& s) const;
    // as the reference's accessor: the tensor must exist (aborts otherwise)
    const ggml_data_descriptor& get_buffer_descriptor(const std::string& s) const;
    const std::vector<ggml_token>& get_tokens() const { return tokens; }
    const std::vector<ggml_data_descriptor>& get_tables() const { return tables; }

    bool is_open() const { return mapping != nullptr; }
    const std::string& error() const { return error_text; }
    const ggml_header& get_header() const { return header; }
    u32 get_ff_size() const { return ff_size; }
    const u8* data() const { return mapping; }
    size_t data_size() const { return mapping_size; }

private:
    bool parse();
    void close_mapping();
    u8* mapping = nullptr;
    size_t mapping_size = 0;
    ggml_header header{};
    u32 ff_size = 0;
    std::vector<ggml_token> tokens;
    std::vector<ggml_data_descriptor> tables;
    std::map<std::string, u32> name_to_index;
    // token text -> lowest id with that text (what the reference's linear scan returns)
    std::unordered_map<std::string, u32> text_to_id;
    std::string error_text;
};

#endif
