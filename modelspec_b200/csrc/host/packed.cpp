// The packed masked-language-model feed of `train --data <packed directory>`: the directory the
// reference's `pack` writes, read and checked as the reference reads it, and the batch of every
// step as a pure function of the packed ids, the masking policy, the run seed and the step.
//
// Follows crates/modelspec-runtime/src/dataset/mlm.rs of the reference: `load` (:583-660),
// `epoch_order` (:662-675), `mlm_batch` (:708-788), `binding_id` (:161-184), and `uuid_of`
// (dataset/mod.rs:212-227); and the directory check of train/data.rs `source` (:1443-1483).
// Host code only: a batch is a few thousand Philox blocks, and the step uploads it with its other
// inputs.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>

#include "../../../include/msx.h"
#include "../core/json.hpp"
#include "../core/rng.hpp"

extern "C" void msx_internal_set_error(msx_device* device, const char* message);

namespace {

constexpr uint32_t kSpecials = 5;     // [PAD] [UNK] [CLS] [SEP] [MASK] head every vocabulary (tokenizer.rs:21)
constexpr int32_t kMaskTokenId = 4;   // tokenizer.rs:31

struct Refused {
    int status;
    std::string what;
};

std::string hex_of(const uint8_t* bytes, size_t n) {
    static const char* digits = "0123456789abcdef";
    std::string out;
    for (size_t i = 0; i < n; ++i) {
        out += digits[bytes[i] >> 4];
        out += digits[bytes[i] & 15];
    }
    return out;
}

// dataset/mod.rs:212-227: the first 16 bytes of a hash as a version-8 UUID.
std::string uuid_of(const uint8_t hash[32]) {
    uint8_t b[16];
    std::memcpy(b, hash, 16);
    b[6] = static_cast<uint8_t>((b[6] & 0x0f) | 0x80);
    b[8] = static_cast<uint8_t>((b[8] & 0x3f) | 0x80);
    std::string hex = hex_of(b, 16);
    return hex.substr(0, 8) + "-" + hex.substr(8, 4) + "-" + hex.substr(12, 4) + "-" + hex.substr(16, 4) + "-" + hex.substr(20, 12);
}

// mlm.rs:148-159: the 16 bytes of a hyphenated UUID, or false.
bool uuid_bytes(const std::string& text, uint8_t out[16]) {
    std::string hex;
    for (char c : text)
        if (c != '-') hex += c;
    if (hex.size() != 32 || text.size() != 36) return false;
    for (int i = 0; i < 16; ++i) {
        int v = 0;
        for (int k = 0; k < 2; ++k) {
            char c = hex[static_cast<size_t>(2 * i + k)];
            int d = c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : -1;
            if (d < 0) return false;
            v = v * 16 + d;
        }
        out[i] = static_cast<uint8_t>(v);
    }
    return true;
}

struct Policy {
    double selection_rate = 0.15, mask_fraction = 0.8, random_fraction = 0.1, keep_fraction = 0.1;
};

// mlm.rs:161-184.
bool binding_id_of(const std::string& dataset, const std::string& tokenizer, uint64_t seq_len, const Policy& p, std::string* out) {
    uint8_t bytes[16 + 16 + 8 + 32];
    if (!uuid_bytes(dataset, bytes) || !uuid_bytes(tokenizer, bytes + 16)) return false;
    for (int i = 0; i < 8; ++i) bytes[32 + i] = static_cast<uint8_t>(seq_len >> (8 * i));
    const double rates[4] = {p.selection_rate, p.mask_fraction, p.random_fraction, p.keep_fraction};
    for (int r = 0; r < 4; ++r) {
        uint64_t bits;
        std::memcpy(&bits, &rates[r], 8);
        for (int i = 0; i < 8; ++i) bytes[40 + 8 * r + i] = static_cast<uint8_t>(bits >> (8 * i));
    }
    uint8_t hash[32];
    msx::blake3_hash(bytes, sizeof(bytes), hash);
    *out = uuid_of(hash);
    return true;
}

std::string read_file(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw Refused{MSX_BAD_INPUT, path + ": cannot be read"};
    std::ostringstream buffer;
    buffer << in.rdbuf();
    return buffer.str();
}

msx::json::Value read_json(const std::string& path) {
    std::string text = read_file(path);
    try {
        return msx::json::parse(text);
    } catch (const std::exception& e) {
        throw Refused{MSX_BAD_INPUT, path + ": " + e.what()};
    }
}

}  // namespace

struct msx_packed {
    std::string dir, error;
    std::string binding_id, dataset_id, tokenizer_id, packed_id;
    uint64_t seq_len = 0, vocabulary = 0;
    Policy policy;
    std::vector<int32_t> ids[2];  // Train, HeldOut
    // The epoch order of the Train split last drawn (mlm.rs:565-582).
    bool have_order = false;
    uint64_t order_seed = 0, order_epoch = 0;
    std::vector<uint32_t> order;

    uint64_t sequences(int split) const { return ids[split].size() / seq_len; }
};

namespace {

// mlm.rs:662-675: ascending by the 64-bit key w1 * 2^32 + w0 of the block of sequence i on the
// data-order stream with the epoch as id, ties by i.
std::vector<uint32_t> epoch_order(uint64_t seed, uint64_t epoch, uint32_t n) {
    std::vector<std::pair<uint64_t, uint32_t>> keyed(n);
    for (uint32_t i = 0; i < n; ++i) {
        uint32_t w[4];
        msx::philox_block(seed, msx::kStreamDataOrder, epoch, i, w);
        keyed[i] = {(static_cast<uint64_t>(w[1]) << 32) | w[0], i};
    }
    std::sort(keyed.begin(), keyed.end());
    std::vector<uint32_t> out(n);
    for (uint32_t i = 0; i < n; ++i) out[i] = keyed[i].second;
    return out;
}

void load(msx_packed* p, const std::string& dir) {
    p->dir = dir;
    // train/data.rs:1443-1483: the binding, whose id is the id of its fields.
    const std::string binding_path = dir + "/binding.json";
    msx::json::Value binding = read_json(binding_path);
    try {
        p->binding_id = binding.at("binding_id").str();
        p->dataset_id = binding.at("dataset_id").str();
        p->tokenizer_id = binding.at("tokenizer_id").str();
        p->seq_len = binding.at("seq_len").u64();
        const msx::json::Value& policy = binding.at("masking_policy");
        p->policy.selection_rate = policy.at("selection_rate").f64();
        p->policy.mask_fraction = policy.at("mask_fraction").f64();
        p->policy.random_fraction = policy.at("random_fraction").f64();
        p->policy.keep_fraction = policy.at("keep_fraction").f64();
        if (binding.at("state").str() != "Recorded") throw std::runtime_error("unknown state `" + binding.at("state").str() + "`");
    } catch (const std::exception& e) {
        throw Refused{MSX_BAD_INPUT, binding_path + ": " + e.what()};
    }
    std::string id;
    if (p->seq_len == 0 || !binding_id_of(p->dataset_id, p->tokenizer_id, p->seq_len, p->policy, &id) || id != p->binding_id)
        throw Refused{MSX_BAD_INPUT, binding_path + ": binding_id " + p->binding_id +
                                         " is not the id of its dataset, tokenizer, seq_len and masking policy"};
    // mlm.rs:583-660: the record and the packed files it describes.
    const std::string record_path = dir + "/packed.json";
    msx::json::Value record = read_json(record_path);
    uint64_t record_seq_len = 0;
    std::string record_binding;
    std::vector<std::pair<uint64_t, std::string>> splits;
    try {
        p->packed_id = record.at("packed_id").str();
        record_binding = record.at("binding_id").str();
        record_seq_len = record.at("seq_len").u64();
        p->vocabulary = record.at("vocabulary_size").u64();
        const msx::json::Value& list = record.at("splits");
        bool roles = list.kind == msx::json::Value::Array && list.items.size() == 2 && list.items[0].at("role").str() == "Train" &&
                     list.items[1].at("role").str() == "HeldOut";
        if (!roles || record_seq_len == 0)
            throw Refused{MSX_BAD_INPUT, record_path + ": not a record of a Train and a HeldOut split of a positive sequence length"};
        for (const msx::json::Value& s : list.items) splits.emplace_back(s.at("sequence_count").u64(), s.at("content_hash").str());
    } catch (const Refused&) {
        throw;
    } catch (const std::exception& e) {
        throw Refused{MSX_BAD_INPUT, record_path + ": " + e.what()};
    }
    if (p->vocabulary <= kSpecials || p->vocabulary > (1ull << 31))
        throw Refused{MSX_BAD_INPUT, record_path + ": vocabulary_size " + std::to_string(p->vocabulary) + " is not between " +
                                         std::to_string(kSpecials + 1) + " and 2^31"};
    const char* files[2] = {"train.tokens", "heldout.tokens"};
    for (int split = 0; split < 2; ++split) {
        const std::string path = dir + "/" + files[split];
        std::string bytes = read_file(path);
        const uint64_t count = splits[static_cast<size_t>(split)].first;
        const bool fits = count <= 0xffffffffull && count <= UINT64_MAX / record_seq_len / 4 && count * record_seq_len * 4 == bytes.size();
        if (!fits)
            throw Refused{MSX_BAD_INPUT, path + ": " + std::to_string(bytes.size()) + " bytes, not " + std::to_string(count) + " sequences of " +
                                             std::to_string(record_seq_len) + " ids"};
        uint8_t hash[32];
        msx::blake3_hash(reinterpret_cast<const uint8_t*>(bytes.data()), bytes.size(), hash);
        if (hex_of(hash, 32) != splits[static_cast<size_t>(split)].second)
            throw Refused{MSX_BAD_INPUT, path + ": blake3 differs from the content_hash of packed.json"};
        std::vector<int32_t>& ids = p->ids[split];
        ids.resize(bytes.size() / 4);
        for (size_t i = 0; i < ids.size(); ++i) {
            const uint8_t* b = reinterpret_cast<const uint8_t*>(bytes.data()) + 4 * i;
            ids[i] = static_cast<int32_t>(static_cast<uint32_t>(b[0]) | (static_cast<uint32_t>(b[1]) << 8) | (static_cast<uint32_t>(b[2]) << 16) |
                                          (static_cast<uint32_t>(b[3]) << 24));
            if (ids[i] < 0 || static_cast<uint64_t>(ids[i]) >= p->vocabulary)
                throw Refused{MSX_BAD_INPUT, path + ": id " + std::to_string(ids[i]) + " outside a vocabulary of " + std::to_string(p->vocabulary)};
        }
    }
    // train/data.rs:1605-1613: the record belongs to the binding.
    if (record_binding != p->binding_id || record_seq_len != p->seq_len)
        throw Refused{MSX_BAD_INPUT, record_path + ": binding_id " + record_binding + " and seq_len " + std::to_string(record_seq_len) +
                                         " are not those of binding.json"};
}

template <class F> int guarded(msx_packed* p, F body) {
    try {
        body();
        return MSX_OK;
    } catch (const Refused& r) {
        p->error = r.what;
        return r.status;
    } catch (const std::exception& e) {
        p->error = e.what();
        return MSX_UNSUPPORTED;
    }
}

}  // namespace

extern "C" {

int msx_packed_open(const char* dir, msx_packed** out) {
    if (!dir || !out) return MSX_BAD_ARGUMENT;
    *out = nullptr;
    std::unique_ptr<msx_packed> p(new msx_packed);
    int rc = guarded(p.get(), [&] { load(p.get(), dir); });
    if (rc != MSX_OK) {
        msx_internal_set_error(nullptr, p->error.c_str());  // where msx_last_error(NULL) finds it
        return rc;
    }
    *out = p.release();
    return MSX_OK;
}

void msx_packed_close(msx_packed* p) { delete p; }
const char* msx_packed_last_error(const msx_packed* p) { return p ? p->error.c_str() : ""; }
uint64_t msx_packed_seq_len(const msx_packed* p) { return p ? p->seq_len : 0; }
uint64_t msx_packed_vocabulary(const msx_packed* p) { return p ? p->vocabulary : 0; }
uint64_t msx_packed_sequences(const msx_packed* p, int split) { return p && (split == 0 || split == 1) ? p->sequences(split) : 0; }
const char* msx_packed_binding_id(const msx_packed* p) { return p ? p->binding_id.c_str() : ""; }

// The `data` line a run on a packed directory prints first (crates/modelspec-cli/src/train.rs:
// 1506-1519): `data dataset <id> tokenizer <id> seq_len <n> masking <a>/<b>/<c>/<d> binding <id>`,
// the rates as Rust displays an f64.
uint64_t msx_packed_data_line(const msx_packed* p, char* out, uint64_t capacity) {
    if (!p) return 0;
    auto rate = [](double v) {
        std::string text = msx::json::f64_text(v);
        // Rust's Display never writes an exponent and drops a fraction of zero.
        if (text.size() > 2 && text.compare(text.size() - 2, 2, ".0") == 0) text.resize(text.size() - 2);
        return text;
    };
    const std::string line = "data dataset " + p->dataset_id + " tokenizer " + p->tokenizer_id + " seq_len " + std::to_string(p->seq_len) +
                             " masking " + rate(p->policy.selection_rate) + "/" + rate(p->policy.mask_fraction) + "/" +
                             rate(p->policy.random_fraction) + "/" + rate(p->policy.keep_fraction) + " binding " + p->binding_id + "\n";
    if (out && capacity) {
        const size_t n = std::min<size_t>(capacity - 1, line.size());
        std::memcpy(out, line.data(), n);
        out[n] = 0;
    }
    return line.size() + 1;
}

int msx_packed_epoch_order(msx_packed* p, uint64_t seed, uint64_t epoch, uint32_t* out, uint64_t count) {
    if (!p || !out) return MSX_BAD_ARGUMENT;
    return guarded(p, [&] {
        if (count != p->sequences(MSX_SPLIT_TRAIN)) throw Refused{MSX_BAD_ARGUMENT, "the Train split holds " + std::to_string(p->sequences(0)) + " sequences"};
        std::vector<uint32_t> order = epoch_order(seed, epoch, static_cast<uint32_t>(count));
        std::memcpy(out, order.data(), count * 4);
    });
}

int msx_packed_batch(msx_packed* p, int split, uint64_t seed, uint64_t step, uint64_t batch_size, int32_t* ids, int32_t* positions,
                     float* key_mask, int32_t* labels, float* weights) {
    if (!p || (split != MSX_SPLIT_TRAIN && split != MSX_SPLIT_HELDOUT)) return MSX_BAD_ARGUMENT;
    return guarded(p, [&] {
        // mlm.rs:708-788.
        const uint64_t seq_len = p->seq_len, sequences = p->sequences(split);
        if (batch_size == 0) throw Refused{MSX_BAD_INPUT, "a batch of 0 sequences"};
        if (batch_size > sequences)
            throw Refused{MSX_BAD_INPUT, "a batch of " + std::to_string(batch_size) + " sequences, more than the " + std::to_string(sequences) +
                                             " of the split"};
        const unsigned __int128 all_rows = static_cast<unsigned __int128>(batch_size) * seq_len;
        if (all_rows > (static_cast<unsigned __int128>(1) << 32))
            throw Refused{MSX_BAD_INPUT, "a batch of more than 2^32 rows; a draw addresses at most 2^32"};
        const uint64_t per_epoch = sequences / batch_size, batch = step % per_epoch;
        const uint64_t draw_id = split == MSX_SPLIT_TRAIN ? step : step + (1ull << 63);
        if (split == MSX_SPLIT_TRAIN) {
            const uint64_t epoch = step / per_epoch;
            if (!p->have_order || p->order_seed != seed || p->order_epoch != epoch) {
                p->order = epoch_order(seed, epoch, static_cast<uint32_t>(sequences));
                p->have_order = true;
                p->order_seed = seed;
                p->order_epoch = epoch;
            }
        }
        const std::vector<int32_t>& source = p->ids[split];
        const uint64_t random_tokens = p->vocabulary - kSpecials;
        for (uint64_t b = 0; b < batch_size; ++b) {
            const uint64_t sequence = split == MSX_SPLIT_TRAIN ? p->order[batch * batch_size + b] : batch * batch_size + b;
            const int32_t* from = source.data() + sequence * seq_len;
            for (uint64_t at = 0; at < seq_len; ++at) {
                const uint64_t row = b * seq_len + at;
                const int32_t label = from[at];
                uint32_t w[4];
                msx::philox_block(seed, msx::kStreamMasking, draw_id, static_cast<uint32_t>(row), w);
                const bool selected = label >= static_cast<int32_t>(kSpecials) && msx::uniform01(w[0]) < p->policy.selection_rate;
                int32_t id = label;
                if (selected) {
                    const double u = msx::uniform01(w[1]);
                    if (u < p->policy.mask_fraction) id = kMaskTokenId;
                    else if (u < p->policy.mask_fraction + p->policy.random_fraction)
                        id = static_cast<int32_t>(kSpecials + ((static_cast<uint64_t>(w[2]) * random_tokens) >> 32));
                }
                if (ids) ids[row] = id;
                if (positions) positions[row] = static_cast<int32_t>(at);
                if (key_mask) key_mask[row] = 1.0f;
                if (labels) labels[row] = label;
                if (weights) weights[row] = selected ? 1.0f : 0.0f;
            }
        }
    });
}

}  // extern "C"
