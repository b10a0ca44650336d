// Counter-based random draws and the ids that address them.
//
// Every random value of a run is a Philox4x32-10 block (Salmon et al., SC 2011) addressed by
// key `[seed lo, seed hi]` and counter `[element index, stream tag, id lo, id hi]`, `id` the first
// 8 bytes, little-endian, of a BLAKE3 hash (crates/modelspec-runtime/src/train/init.rs:5-23,
// :91-165). BLAKE3 is the reference's third-party dependency `blake3 = "1"` (Cargo.lock pins
// 1.8.7); this file restates the published algorithm (the BLAKE3 paper, section 2) for inputs of
// any length, unkeyed, 32-byte output. The reference's own tests pin both: the Random123 Philox
// known answers (init.rs:423-449) and `blake3("")` (init.rs:453-456).
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace msx {

// Stream tags (init.rs:41-83).
enum Stream : uint32_t {
    kStreamInit = 0, kStreamTeacher = 1, kStreamData = 2, kStreamMasking = 3, kStreamDropout = 4,
    kStreamDataOrder = 5, kStreamProjection = 6,
    // Generators the reference does not have start at 16.
    kStreamSyntheticTokens = 16, kStreamSyntheticLabels = 17
};

inline void philox4x32_10(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
    uint32_t c0 = counter[0], c1 = counter[1], c2 = counter[2], c3 = counter[3];
    uint32_t k0 = key[0], k1 = key[1];
    for (int round = 0; round < 10; ++round) {
        if (round > 0) {
            k0 += W0;
            k1 += W1;
        }
        uint64_t p0 = static_cast<uint64_t>(M0) * c0;
        uint64_t p1 = static_cast<uint64_t>(M1) * c2;
        uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = static_cast<uint32_t>(p1);
        uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = static_cast<uint32_t>(p0);
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// The block of element `index` of the draw `id` on `stream` under `seed` (init.rs:122-128).
inline void philox_block(uint64_t seed, uint32_t stream, uint64_t id, uint32_t index, uint32_t out[4]) {
    uint32_t counter[4] = {index, stream, static_cast<uint32_t>(id), static_cast<uint32_t>(id >> 32)};
    uint32_t key[2] = {static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)};
    philox4x32_10(counter, key, out);
}

// A word as a uniform draw in (0, 1) (init.rs:130-133).
inline double uniform01(uint32_t word) { return (static_cast<double>(word) + 0.5) / 4294967296.0; }

// ---------------------------------------------------------------------------------------------
// BLAKE3, unkeyed hash, first 32 output bytes.

namespace blake3_detail {

constexpr uint32_t IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                            0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
constexpr int PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
constexpr uint32_t CHUNK_START = 1, CHUNK_END = 2, PARENT = 4, ROOT = 8;

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

inline void g(uint32_t* s, int a, int b, int c, int d, uint32_t mx, uint32_t my) {
    s[a] = s[a] + s[b] + mx; s[d] = rotr(s[d] ^ s[a], 16);
    s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 12);
    s[a] = s[a] + s[b] + my; s[d] = rotr(s[d] ^ s[a], 8);
    s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 7);
}

inline void compress(const uint32_t cv[8], const uint32_t block[16], uint64_t counter,
                     uint32_t block_len, uint32_t flags, uint32_t out[16]) {
    uint32_t s[16] = {cv[0], cv[1], cv[2], cv[3], cv[4], cv[5], cv[6], cv[7],
                      IV[0], IV[1], IV[2], IV[3],
                      static_cast<uint32_t>(counter), static_cast<uint32_t>(counter >> 32), block_len, flags};
    uint32_t m[16];
    std::memcpy(m, block, sizeof m);
    for (int round = 0; round < 7; ++round) {
        g(s, 0, 4, 8, 12, m[0], m[1]);   g(s, 1, 5, 9, 13, m[2], m[3]);
        g(s, 2, 6, 10, 14, m[4], m[5]);  g(s, 3, 7, 11, 15, m[6], m[7]);
        g(s, 0, 5, 10, 15, m[8], m[9]);  g(s, 1, 6, 11, 12, m[10], m[11]);
        g(s, 2, 7, 8, 13, m[12], m[13]); g(s, 3, 4, 9, 14, m[14], m[15]);
        uint32_t p[16];
        for (int i = 0; i < 16; ++i) p[i] = m[PERM[i]];
        std::memcpy(m, p, sizeof m);
    }
    for (int i = 0; i < 8; ++i) {
        out[i] = s[i] ^ s[i + 8];
        out[i + 8] = s[i + 8] ^ cv[i];
    }
}

inline void words_of(const uint8_t* bytes, size_t len, uint32_t block[16]) {
    uint8_t padded[64] = {0};
    std::memcpy(padded, bytes, len);
    for (int i = 0; i < 16; ++i)
        block[i] = static_cast<uint32_t>(padded[4 * i]) | (static_cast<uint32_t>(padded[4 * i + 1]) << 8) |
                   (static_cast<uint32_t>(padded[4 * i + 2]) << 16) | (static_cast<uint32_t>(padded[4 * i + 3]) << 24);
}

// What is left to compress as a root or to pass up as a chaining value.
struct Pending {
    uint32_t cv[8];
    uint32_t block[16];
    uint64_t counter;
    uint32_t block_len, flags;
    void chaining_value(uint32_t out[8]) const {
        uint32_t full[16];
        compress(cv, block, counter, block_len, flags, full);
        std::memcpy(out, full, 32);
    }
};

inline Pending chunk(const uint8_t* bytes, size_t len, uint64_t index) {
    Pending p;
    std::memcpy(p.cv, IV, sizeof p.cv);
    size_t blocks = len == 0 ? 1 : (len + 63) / 64;
    for (size_t b = 0; b < blocks; ++b) {
        size_t take = std::min<size_t>(64, len - b * 64);
        uint32_t flags = (b == 0 ? CHUNK_START : 0) | (b + 1 == blocks ? CHUNK_END : 0);
        words_of(bytes + b * 64, take, p.block);
        p.counter = index;
        p.block_len = static_cast<uint32_t>(take);
        p.flags = flags;
        if (b + 1 < blocks) {
            uint32_t full[16];
            compress(p.cv, p.block, index, p.block_len, flags, full);
            std::memcpy(p.cv, full, 32);
        }
    }
    return p;
}

inline Pending parent(const uint32_t left[8], const uint32_t right[8]) {
    Pending p;
    std::memcpy(p.cv, IV, sizeof p.cv);
    std::memcpy(p.block, left, 32);
    std::memcpy(p.block + 8, right, 32);
    p.counter = 0;
    p.block_len = 64;
    p.flags = PARENT;
    return p;
}

// The subtree over `len` bytes starting at chunk `index`: the left subtree takes the largest
// power of two of chunks that leaves at least one byte to the right.
inline Pending subtree(const uint8_t* bytes, size_t len, uint64_t index) {
    if (len <= 1024) return chunk(bytes, len, index);
    size_t chunks = (len + 1023) / 1024;
    size_t left_chunks = 1;
    while (left_chunks * 2 < chunks) left_chunks *= 2;
    size_t left_len = left_chunks * 1024;
    uint32_t l[8], r[8];
    subtree(bytes, left_len, index).chaining_value(l);
    subtree(bytes + left_len, len - left_len, index + left_chunks).chaining_value(r);
    return parent(l, r);
}

}  // namespace blake3_detail

inline void blake3_hash(const uint8_t* bytes, size_t len, uint8_t out[32]) {
    using namespace blake3_detail;
    Pending root = subtree(bytes, len, 0);
    uint32_t full[16];
    compress(root.cv, root.block, 0, root.block_len, root.flags | ROOT, full);
    for (int i = 0; i < 8; ++i) {
        out[4 * i] = static_cast<uint8_t>(full[i]);
        out[4 * i + 1] = static_cast<uint8_t>(full[i] >> 8);
        out[4 * i + 2] = static_cast<uint8_t>(full[i] >> 16);
        out[4 * i + 3] = static_cast<uint8_t>(full[i] >> 24);
    }
}

inline uint64_t first8_le(const uint8_t hash[32]) {
    uint64_t v = 0;
    for (int i = 7; i >= 0; --i) v = (v << 8) | hash[i];
    return v;
}

// The canonical id of a path (init.rs:113-120).
inline uint64_t canonical_id(const std::string& path) {
    uint8_t h[32];
    blake3_hash(reinterpret_cast<const uint8_t*>(path.data()), path.size(), h);
    return first8_le(h);
}

// The draw id of the dropout site `site` at step `step`: blake3(site bytes, then the step as 8
// little-endian bytes) (init.rs:135-145).
inline uint64_t dropout_id(const std::string& site, uint64_t step) {
    std::vector<uint8_t> bytes(site.begin(), site.end());
    for (int i = 0; i < 8; ++i) bytes.push_back(static_cast<uint8_t>(step >> (8 * i)));
    uint8_t h[32];
    blake3_hash(bytes.data(), bytes.size(), h);
    return first8_le(h);
}

// The i32[2] token a dropout site reads: id low word, id high word, as bit patterns
// (init.rs:147-153).
inline void dropout_token(const std::string& site, uint64_t step, int32_t token[2]) {
    uint64_t id = dropout_id(site, step);
    token[0] = static_cast<int32_t>(static_cast<uint32_t>(id));
    token[1] = static_cast<int32_t>(static_cast<uint32_t>(id >> 32));
}

// Whether element `index` of the dropout draw `id` is kept at drop probability `p`: u >= p with
// u = (w0 + 0.5) / 2^32, compared in f64 (init.rs:160-165).
inline bool dropout_keeps(uint64_t seed, uint64_t id, uint32_t index, float p) {
    uint32_t block[4];
    philox_block(seed, kStreamDropout, id, index, block);
    return uniform01(block[0]) >= static_cast<double>(p);
}

// The same test on the word alone: keep iff w0 >= threshold. u >= p is w0 + 0.5 >= p * 2^32, so
// the threshold is ceil(p * 2^32 - 0.5) clamped to [0, 2^32], computed exactly in f64 (p is an
// f32, so p * 2^32 is exact). The reference's GPU emitter uses the same integer form
// (crates/modelspec-runtime/src/spirv/emit/rowwise.rs:148-161).
inline uint64_t dropout_keep_threshold(float p) {
    double t = std::ceil(static_cast<double>(p) * 4294967296.0 - 0.5);
    if (t <= 0.0) return 0;
    if (t >= 4294967296.0) return 4294967296ull;
    return static_cast<uint64_t>(t);
}

}  // namespace msx
