// Reader for the safetensors container and the small JSON subset its header
// and the embedded TrainConfig use.  Container layout: u64 little-endian
// header length N, N bytes of JSON ({"__metadata__": {string: string},
// name: {"dtype", "shape", "data_offsets": [begin, end]}}), then the raw
// little-endian tensor bytes.  The reference reads these files through the
// `safetensors` crate (src/model.rs:3470-3477).
#pragma once
#include <stdint.h>

#include <map>
#include <memory>
#include <string>
#include <vector>

namespace ullis {

struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool boolean = false;
    double number = 0.0;
    std::string text;       // String value, or the literal text of a Number
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;

    const Json* get(const std::string& key) const;
    // unsigned integer value of a Number member; `fallback` when absent
    uint64_t u64(const std::string& key, uint64_t fallback, bool* present = nullptr) const;
};

// Throws ullis::Error(ULLIS_CUDA_ERR_CHECKPOINT) on malformed input.
Json parse_json(const char* data, size_t len);

struct TensorView {
    std::string dtype;  // "F16", "U32", "F32", ...
    const uint8_t* data = nullptr;
    size_t bytes = 0;
    size_t elements() const;
};

struct SafeTensors {
    std::map<std::string, std::string> metadata;
    bool has_metadata = false;
    std::map<std::string, TensorView> tensors;
};

SafeTensors parse_safetensors(const uint8_t* bytes, size_t len);

}  // namespace ullis
