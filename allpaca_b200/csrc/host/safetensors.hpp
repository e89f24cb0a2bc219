// Reader of one safetensors file: the header is parsed and checked, the file memory-mapped.
//
// Format (as the reference parses it, crates/allpaca-safetensors/src/parser.rs:93-159 and
// :181-188): an unsigned 64-bit little-endian header length (1 byte .. 100 MiB), a JSON
// object {name: {"dtype", "shape", "data_offsets": [begin, end]}} with an optional
// "__metadata__" object of strings, then the tensor bytes; offsets count from the end of the
// header.  Checked here: the header is UTF-8 and JSON, every entry is well formed, its type is
// known, its bytes lie inside the file and are exactly what shape and type need
// (parser.rs:95-123, :170-196).
#pragma once
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

namespace allpaca {

struct TensorEntry {
    std::string name;
    std::string dtype;            // "BF16", "F32", ...
    std::vector<int64_t> shape;
    int64_t begin = 0, end = 0;   // byte range within the data section
};

class SafetensorsFile {
public:
    static constexpr uint64_t kMaxHeaderBytes = 100ull * 1024 * 1024;   // parser.rs:11

    // nullptr and a message in *error when the file cannot be read as safetensors
    static SafetensorsFile* open(const std::string& path, std::string* error);
    ~SafetensorsFile();
    SafetensorsFile(const SafetensorsFile&) = delete;
    SafetensorsFile& operator=(const SafetensorsFile&) = delete;

    const std::vector<TensorEntry>& tensors() const { return tensors_; }
    const std::vector<std::pair<std::string, std::string>>& metadata() const { return metadata_; }
    const uint8_t* data() const { return map_ ? map_ + data_start_ : nullptr; }   // first data byte
    int64_t data_len() const { return data_len_; }

    // bytes of one element of a stored type, 0 if the type is not one safetensors defines here
    static int element_size(const std::string& dtype);

private:
    SafetensorsFile() = default;
    std::vector<TensorEntry> tensors_;
    std::vector<std::pair<std::string, std::string>> metadata_;
    uint8_t* map_ = nullptr;
    size_t map_len_ = 0;
    int64_t data_start_ = 0, data_len_ = 0;
};

}  // namespace allpaca
