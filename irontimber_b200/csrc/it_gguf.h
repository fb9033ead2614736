// GGUF v2/v3 container reader (host only): metadata, tensor directory and bounds-checked views of the tensor data in a
// read-only mapping of the file.  Stands where the reference's reader stands (src/gguf.rs:99-140).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

// ggml tensor type ids the model files use (src/gguf.rs:9-22); block = elements per quantisation block
enum { GG_F32 = 0, GG_F16 = 1, GG_Q8_0 = 8, GG_Q4_K = 12, GG_Q6_K = 14, GG_BF16 = 30, GG_PQ2_0 = 142, GG_PTQ1_0 = 143 };
bool it_gg_block(uint32_t type, size_t* block_elems, size_t* block_bytes);   // false: a type this library does not know
const char* it_gg_type_name(uint32_t type);

// metadata value type ids of the container
enum { GV_U8 = 0, GV_I8, GV_U16, GV_I16, GV_U32, GV_I32, GV_F32, GV_BOOL, GV_STR, GV_ARR, GV_U64, GV_I64, GV_F64 };

struct it_gguf_value {
    uint32_t type = 0, elem_type = 0;      // elem_type: element type of an array
    uint64_t u = 0; int64_t i = 0; double f = 0; std::string s;   // scalar, by kind
    uint64_t count = 0;                    // array length
    std::vector<int64_t> ints; std::vector<double> floats; std::vector<std::string> strs;   // array elements, by kind (empty when skipped)
    size_t raw_off = 0, raw_len = 0;       // the value's bytes in the file (type tag included)
    bool is_int() const { return type <= GV_F64 && ((1u << type) & 0x0C3Fu) != 0; }
    bool as_u64(uint64_t* v) const;        // any non-negative integer kind
    bool as_f32(float* v) const;           // f32 or f64
    bool as_bool(bool* v) const;
};
struct it_gguf_tensor { std::string name; std::vector<uint64_t> dims; uint32_t type; uint64_t offset, nelem, nbytes; };

class it_gguf {
public:
    it_gguf() {}
    ~it_gguf();
    it_gguf(const it_gguf&) = delete; it_gguf& operator=(const it_gguf&) = delete;
    // IT_* code; the message is left for it_last_error.  Arrays under `tokenizer.` are walked but not materialised.
    int open(const char* path);
    const it_gguf_value* get(const std::string& key) const;
    int u(const std::string& key, uint64_t* v) const;       // missing or non-integer key: IT_EFORMAT
    int f(const std::string& key, float* v) const;
    std::vector<std::string> strings(const std::string& key) const;   // empty when absent
    const it_gguf_tensor* tensor(const std::string& name) const;
    int need(const std::string& name, const it_gguf_tensor** t) const;   // missing tensor: IT_EFORMAT
    const uint8_t* data(const it_gguf_tensor& t) const { return base_ + data_off_ + t.offset; }
    const uint8_t* raw(const it_gguf_value& v) const { return base_ + v.raw_off; }
    const std::unordered_map<std::string, it_gguf_value>& kv() const { return kv_; }
    const std::vector<it_gguf_tensor>& tensors() const { return tensors_; }
    uint32_t version() const { return version_; }
    const std::string& path() const { return path_; }
private:
    std::string path_;
    const uint8_t* base_ = nullptr; size_t len_ = 0; size_t data_off_ = 0; uint32_t version_ = 0;
    std::unordered_map<std::string, it_gguf_value> kv_;
    std::vector<it_gguf_tensor> tensors_;
    std::unordered_map<std::string, size_t> index_;
};

// Element decoders (ggml's dequantize_row_* arithmetic, element order and float operation order as in
// src/quant.rs:51-62, :189-228): n elements, n a multiple of the type's block.
int it_gg_dequant(uint32_t type, const uint8_t* src, size_t n, float* out);
// PTQ1_0 blocks (24 base-3 bytes + 2 + f16 scale) rewritten as PQ2_0 blocks (f16 scale + 32 bytes of 2-bit codes) with
// the same codes and scale (ptq1_block_codes, src/quant.rs:37-49)
void it_gg_ptq1_to_pq2(const uint8_t* src, size_t nblocks, uint8_t* dst);
