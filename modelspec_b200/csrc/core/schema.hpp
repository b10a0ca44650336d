// The schema hash of a program's parameters: blake3 over the parameter paths, dtypes and shapes in
// declaration (ParamId) order, independent of the backend and the learning rate
// (crates/modelspec-core/src/artifact.rs:170-194 of the reference). Lowercase hex.
#pragma once

#include <string>
#include <vector>

#include "ir.hpp"
#include "rng.hpp"

namespace msx {

inline std::string schema_hash(const std::vector<Param>& params) {
    std::string bytes = "modelspec-schema/1\n";
    auto le64 = [&](uint64_t v) {
        for (int i = 0; i < 8; ++i) bytes.push_back(static_cast<char>(v >> (8 * i)));
    };
    for (const Param& p : params) {
        le64(p.path.size());
        bytes += p.path;
        bytes += p.ty.i32 ? "i32" : "f32";
        le64(p.ty.shape.size());
        for (uint64_t n : p.ty.shape) {
            bytes.push_back(0);  // a static dimension
            le64(n);
        }
    }
    uint8_t hash[32];
    blake3_hash(reinterpret_cast<const uint8_t*>(bytes.data()), bytes.size(), hash);
    static const char* digits = "0123456789abcdef";
    std::string out;
    for (uint8_t b : hash) {
        out += digits[b >> 4];
        out += digits[b & 15];
    }
    return out;
}

}  // namespace msx
