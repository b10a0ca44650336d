// Host-side initial values and synthetic draws, addressed by Philox counters
// (crates/modelspec-runtime/src/train/init.rs:167-242, :325-352). Both sides of a parity run
// start from these bits: a parameter's xavier_uniform draw is a (2u - 1) with a = sqrt(6 / (in +
// out)) and u word 0 of the element's block, computed in f64 and rounded once; `zeros` and `ones`
// draw nothing.
#pragma once

#include "ir.hpp"
#include "rng.hpp"

namespace msx {

inline std::vector<float> initial_parameter(const Param& p, uint64_t seed, uint32_t stream) {
    std::vector<float> out(p.ty.count());
    if (p.init != Init::XavierUniform) {
        std::fill(out.begin(), out.end(), p.init == Init::Ones ? 1.0f : 0.0f);
        return out;
    }
    if (p.ty.rank() != 2) throw Error("`" + p.path + "` is " + p.ty.str() + "; xavier_uniform needs rank 2");
    if (out.size() > (1ull << 32)) throw Error("`" + p.path + "` has more than 2^32 elements");
    double a = std::sqrt(6.0 / (static_cast<double>(p.ty.shape[0]) + static_cast<double>(p.ty.shape[1])));
    uint64_t id = canonical_id(p.path);
    for (size_t i = 0; i < out.size(); ++i) {
        uint32_t block[4];
        philox_block(seed, stream, id, static_cast<uint32_t>(i), block);
        out[i] = static_cast<float>(a * (2.0 * uniform01(block[0]) - 1.0));
    }
    return out;
}

// A standard normal tensor by Box-Muller over words 0 and 1, named `name` for its id.
inline std::vector<float> standard_normal_draw(uint64_t seed, uint32_t stream, const std::string& name, size_t n) {
    std::vector<float> out(n);
    uint64_t id = canonical_id(name);
    const double tau = 6.283185307179586476925286766559;
    for (size_t i = 0; i < n; ++i) {
        uint32_t block[4];
        philox_block(seed, stream, id, static_cast<uint32_t>(i), block);
        out[i] = static_cast<float>(std::sqrt(-2.0 * std::log(uniform01(block[0]))) * std::cos(tau * uniform01(block[1])));
    }
    return out;
}

}  // namespace msx
