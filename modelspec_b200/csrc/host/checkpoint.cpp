// The `.msckpt` checkpoint: writer and validating reader, byte-compatible with the reference's
// format version 1 (crates/modelspec-runtime/src/train/checkpoint.rs:1-22 layout, :420-517 encode,
// :640-868 read, :870-921 invariants): a 56-byte little-endian header (magic MSCK, version, endian
// marker, a reserved zero word, the manifest size, a blake3 checksum over header and manifest with
// the checksum bytes counted as zero), a compact JSON manifest, and the payload: each tensor's
// little-endian f32 values at a multiple of 64, zero bytes between, the file ending with the last
// tensor. `payload_hash` is blake3 from the payload start to the end of the file; `checkpoint_id`
// is a version-8 UUID from blake3 over the manifest with the nil UUID in its place.
//
// One addition the format already has room for: the AdamW moments of a run are written as
// `optimizer_slots` records (slot "m" and "v" of each parameter path), which the reference's
// reader validates like parameters but its writer never emits, so the reference refuses to resume
// an AdamW run (train/runner.rs:335-347). Host code only.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <set>
#include <sstream>

#include "../../../include/msx.h"
#include "../core/json.hpp"
#include "../core/rng.hpp"

extern "C" void msx_internal_set_error(msx_device* device, const char* message);

namespace {

constexpr size_t kHeader = 56;
constexpr uint64_t kAlignment = 64;
constexpr size_t kMaxRank = 8;
const char* const kNilUuid = "00000000-0000-0000-0000-000000000000";

struct Refused {
    int status;
    std::string what;
};

struct Tensor {
    std::string path, slot;  // slot empty for a parameter
    std::vector<uint64_t> shape;
    std::vector<float> data;
    uint64_t count() const {
        uint64_t n = 1;
        for (uint64_t d : shape) n *= d;
        return n;
    }
};

struct Optimizer {
    int kind = MSX_OPTIMIZER_SGD;
    double learning_rate = 0.0, weight_decay = 0.0, beta1 = 0.0, beta2 = 0.0, epsilon = 0.0;
    uint64_t warmup_steps = 0;
    bool operator==(const Optimizer& o) const {
        if (kind != o.kind || learning_rate != o.learning_rate) return false;
        if (kind == MSX_OPTIMIZER_SGD) return true;
        return weight_decay == o.weight_decay && beta1 == o.beta1 && beta2 == o.beta2 && epsilon == o.epsilon && warmup_steps == o.warmup_steps;
    }
    std::string json() const {
        using msx::json::f64_text;
        std::string s = std::string("{\"kind\":\"") + (kind == MSX_OPTIMIZER_SGD ? "Sgd" : "AdamW") + "\",\"learning_rate\":" + f64_text(learning_rate);
        if (kind != MSX_OPTIMIZER_SGD)
            s += ",\"weight_decay\":" + f64_text(weight_decay) + ",\"beta1\":" + f64_text(beta1) + ",\"beta2\":" + f64_text(beta2) +
                 ",\"epsilon\":" + f64_text(epsilon) + ",\"schedule\":{\"warmup_steps\":" + std::to_string(warmup_steps) + "}";
        return s + "}";
    }
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

std::string blake3_hex(const void* data, size_t n) {
    uint8_t hash[32];
    msx::blake3_hash(static_cast<const uint8_t*>(data), n, hash);
    return hex_of(hash, 32);
}

// checkpoint.rs:611-627.
std::string uuid_of(const uint8_t hash[32]) {
    uint8_t b[16];
    std::memcpy(b, hash, 16);
    b[6] = static_cast<uint8_t>((b[6] & 0x0f) | 0x80);
    b[8] = static_cast<uint8_t>((b[8] & 0x3f) | 0x80);
    std::string hex = hex_of(b, 16);
    return hex.substr(0, 8) + "-" + hex.substr(8, 4) + "-" + hex.substr(12, 4) + "-" + hex.substr(16, 4) + "-" + hex.substr(20, 12);
}

bool is_uuid(const std::string& s) {
    if (s.size() != 36) return false;
    for (size_t i = 0; i < 36; ++i) {
        const bool dash = i == 8 || i == 13 || i == 18 || i == 23;
        if (dash ? s[i] != '-' : !std::isxdigit(static_cast<unsigned char>(s[i]))) return false;
    }
    return true;
}

uint64_t round_up(uint64_t n) { return (n + kAlignment - 1) / kAlignment * kAlignment; }

void put32(std::string& out, uint32_t v) {
    for (int i = 0; i < 4; ++i) out.push_back(static_cast<char>(v >> (8 * i)));
}
void put64(std::string& out, uint64_t v) {
    for (int i = 0; i < 8; ++i) out.push_back(static_cast<char>(v >> (8 * i)));
}
uint32_t get32(const uint8_t* p) { return static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) | (static_cast<uint32_t>(p[2]) << 16) | (static_cast<uint32_t>(p[3]) << 24); }
uint64_t get64(const uint8_t* p) { return static_cast<uint64_t>(get32(p)) | (static_cast<uint64_t>(get32(p + 4)) << 32); }

}  // namespace

struct msx_checkpoint {
    uint64_t step = 0, seed = 0, counter = 0;
    std::string schema_hash, checkpoint_id, error;
    Optimizer optimizer;
    std::vector<Tensor> parameters;  // in path order
    std::vector<Tensor> slots;       // in (path, slot) order
};

namespace {

void sort_tensors(msx_checkpoint* c) {
    auto by_name = [](const Tensor& a, const Tensor& b) { return a.path != b.path ? a.path < b.path : a.slot < b.slot; };
    std::sort(c->parameters.begin(), c->parameters.end(), by_name);
    std::sort(c->slots.begin(), c->slots.end(), by_name);
}

// checkpoint.rs:453-517: the file's bytes.
std::string encode(msx_checkpoint* c) {
    sort_tensors(c);
    std::string payload;
    std::vector<std::pair<uint64_t, uint64_t>> relative;
    auto place = [&](const Tensor& t) {
        const uint64_t at = round_up(payload.size());
        payload.resize(at, 0);
        for (float v : t.data) {
            uint32_t bits;
            std::memcpy(&bits, &v, 4);
            put32(payload, bits);
        }
        relative.emplace_back(at, payload.size() - at);
    };
    for (const Tensor& t : c->parameters) place(t);
    for (const Tensor& t : c->slots) place(t);
    const std::string payload_hash = blake3_hex(payload.data(), payload.size());
    auto record = [&](const Tensor& t, size_t at, uint64_t start) {
        std::string s = "{\"path\":" + msx::json::quoted(t.path);
        if (!t.slot.empty()) s += ",\"slot\":" + msx::json::quoted(t.slot);
        s += ",\"dtype\":\"F32\",\"shape\":[";
        for (size_t i = 0; i < t.shape.size(); ++i) s += (i ? "," : "") + std::to_string(t.shape[i]);
        return s + "],\"offset\":" + std::to_string(start + relative[at].first) + ",\"length\":" + std::to_string(relative[at].second) + "}";
    };
    auto manifest_at = [&](uint64_t start, const std::string& id) {
        std::string s = "{\"checkpoint_id\":\"" + id + "\",\"file_size\":" + std::to_string(start + payload.size()) + ",\"alignment\":" +
                        std::to_string(kAlignment) + ",\"schema_hash\":" + msx::json::quoted(c->schema_hash) + ",\"step\":" + std::to_string(c->step) +
                        ",\"payload_hash\":\"" + payload_hash + "\",\"optimizer\":" + c->optimizer.json() + ",\"optimizer_slots\":[";
        for (size_t i = 0; i < c->slots.size(); ++i) s += (i ? "," : "") + record(c->slots[i], c->parameters.size() + i, start);
        s += "],\"rng\":{\"algorithm\":\"Philox4x32x10\",\"seed\":" + std::to_string(c->seed) + ",\"counter\":" + std::to_string(c->counter) + "},\"parameters\":[";
        for (size_t i = 0; i < c->parameters.size(); ++i) s += (i ? "," : "") + record(c->parameters[i], i, start);
        return s + "]}";
    };
    // The payload start depends on the manifest's length, which holds the offsets: to a fixed point.
    uint64_t start = 0;
    std::string unnamed;
    for (;;) {
        unnamed = manifest_at(start, kNilUuid);
        const uint64_t next = round_up(kHeader + unnamed.size());
        if (next == start) break;
        start = next;
    }
    const std::string named = "modelspec-checkpoint-id/1\n" + unnamed;
    uint8_t hash[32];
    msx::blake3_hash(reinterpret_cast<const uint8_t*>(named.data()), named.size(), hash);
    c->checkpoint_id = uuid_of(hash);
    const std::string manifest = manifest_at(start, c->checkpoint_id);
    std::string bytes = "MSCK";
    put32(bytes, 1);
    put32(bytes, 0x01020304u);
    put32(bytes, 0);
    put64(bytes, manifest.size());
    bytes.append(32, '\0');
    bytes += manifest;
    msx::blake3_hash(reinterpret_cast<const uint8_t*>(bytes.data()), bytes.size(), hash);
    std::memcpy(&bytes[24], hash, 32);
    bytes.resize(start, '\0');
    bytes += payload;
    return bytes;
}

void only(const msx::json::Value& v, std::initializer_list<const char*> allowed, const char* what) {
    if (v.kind != msx::json::Value::Object) throw std::runtime_error(std::string(what) + " is not an object");
    std::set<std::string> seen;
    for (const auto& m : v.members) {
        if (std::find_if(allowed.begin(), allowed.end(), [&](const char* a) { return m.first == a; }) == allowed.end())
            throw std::runtime_error("unknown field `" + m.first + "` of " + what);
        if (!seen.insert(m.first).second) throw std::runtime_error("duplicate field `" + m.first + "` of " + what);
    }
}

struct Record {
    Tensor tensor;
    uint64_t offset = 0, length = 0;
    bool has_slot = false;
};

Record record_of(const msx::json::Value& v) {
    only(v, {"path", "slot", "dtype", "shape", "offset", "length"}, "a record");
    Record r;
    r.tensor.path = v.at("path").str();
    if (const msx::json::Value* slot = v.get("slot")) {
        if (slot->kind != msx::json::Value::Null) {
            r.tensor.slot = slot->str();
            r.has_slot = true;
        }
    }
    if (v.at("dtype").str() != "F32") throw std::runtime_error("unknown dtype `" + v.at("dtype").str() + "`");
    const msx::json::Value& shape = v.at("shape");
    if (shape.kind != msx::json::Value::Array) throw std::runtime_error("a shape is not a list");
    if (shape.items.size() > kMaxRank) throw std::runtime_error("a shape has more than " + std::to_string(kMaxRank) + " dimensions");
    for (const msx::json::Value& d : shape.items) r.tensor.shape.push_back(d.u64());
    r.offset = v.at("offset").u64();
    r.length = v.at("length").u64();
    return r;
}

// checkpoint.rs:640-868. Every refusal carries its E-CKPT code.
void read(msx_checkpoint* c, const std::string& path) {
    auto bad = [&](const std::string& m) { return Refused{MSX_BAD_INPUT, "E-CKPT-001: not a readable checkpoint: " + m + " (file " + path + ")"}; };
    auto outside = [&](const std::string& m) { return Refused{MSX_BAD_INPUT, "E-CKPT-002: " + m + " (file " + path + ")"}; };
    std::ifstream in(path, std::ios::binary);
    if (!in) throw bad("the file cannot be read");
    std::ostringstream buffer;
    buffer << in.rdbuf();
    const std::string file = buffer.str();
    const uint8_t* bytes = reinterpret_cast<const uint8_t*>(file.data());
    const uint64_t size = file.size();
    if (size < kHeader) throw outside("the file has " + std::to_string(size) + " bytes, fewer than the " + std::to_string(kHeader) + "-byte header");
    if (std::memcmp(bytes, "MSCK", 4) != 0) throw bad("the magic is not MSCK");
    if (get32(bytes + 4) != 1) throw bad("format version " + std::to_string(get32(bytes + 4)) + " is not 1");
    if (get32(bytes + 8) != 0x01020304u) {
        if (get32(bytes + 8) == 0x04030201u) throw bad("the endian marker is big-endian; the payload is little-endian");
        char text[16];
        std::snprintf(text, sizeof text, "%#010x", get32(bytes + 8));
        throw bad(std::string("the endian marker ") + text + " is unknown");
    }
    if (get32(bytes + 12) != 0) throw bad("the reserved header field is not zero");
    const uint64_t manifest_size = get64(bytes + 16);
    if (manifest_size == 0 || manifest_size > size - kHeader)
        throw outside("the manifest size " + std::to_string(manifest_size) + " does not fit the " + std::to_string(size) + "-byte file after its header");
    std::string signed_bytes = file.substr(0, kHeader + manifest_size);
    std::memset(&signed_bytes[24], 0, 32);
    uint8_t hash[32];
    msx::blake3_hash(reinterpret_cast<const uint8_t*>(signed_bytes.data()), signed_bytes.size(), hash);
    if (std::memcmp(hash, bytes + 24, 32) != 0) throw bad("the checksum differs from the header and manifest");
    const uint64_t manifest_end = kHeader + manifest_size;
    const uint64_t payload_start = std::min(round_up(manifest_end), size);
    // A valid file of n records has at least 124 n - 64 bytes: a manifest that lists more records
    // than a file of this size (plus 4,096 bytes of slack) could hold at 96 bytes a record in memory
    // is E-CKPT-002 before any of them is kept (checkpoint.rs:276-281, :711-716).
    const uint64_t most = (size + 4096) / 96;
    msx::json::Value manifest;
    std::vector<Record> parameters, slots;
    try {
        manifest = msx::json::parse(file.substr(kHeader, manifest_size));
        only(manifest, {"checkpoint_id", "file_size", "alignment", "schema_hash", "step", "payload_hash", "optimizer", "optimizer_slots", "rng", "parameters"},
             "the manifest");
        c->checkpoint_id = manifest.at("checkpoint_id").str();
        manifest.at("file_size").u64();
        manifest.at("alignment").u64();
        c->schema_hash = manifest.at("schema_hash").str();
        c->step = manifest.at("step").u64();
        manifest.at("payload_hash").str();
        const msx::json::Value& o = manifest.at("optimizer");
        only(o, {"kind", "learning_rate", "weight_decay", "beta1", "beta2", "epsilon", "schedule", "muon"}, "the optimizer");
        const std::string kind = o.at("kind").str();
        if (kind != "Sgd" && kind != "AdamW" && kind != "Muon") throw std::runtime_error("unknown optimizer kind `" + kind + "`");
        c->optimizer.kind = kind == "Sgd" ? MSX_OPTIMIZER_SGD : kind == "AdamW" ? MSX_OPTIMIZER_ADAMW : MSX_OPTIMIZER_OTHER;
        c->optimizer.learning_rate = o.at("learning_rate").f64();
        auto present = [&](const char* key) { return o.get(key) && o.get(key)->kind != msx::json::Value::Null; };
        const bool adamw_fields = present("weight_decay") && present("beta1") && present("beta2") && present("epsilon") && present("schedule");
        const bool none = !present("weight_decay") && !present("beta1") && !present("beta2") && !present("epsilon") && !present("schedule");
        // checkpoint.rs:155-172: the AdamW fields and the schedule exactly for AdamW and Muon, the Muon fields exactly for Muon.
        const bool fits = std::isfinite(c->optimizer.learning_rate) &&
                          (kind == "Sgd" ? none && !present("muon") : kind == "AdamW" ? adamw_fields && !present("muon") : adamw_fields && present("muon"));
        if (adamw_fields) {
            c->optimizer.weight_decay = o.at("weight_decay").f64();
            c->optimizer.beta1 = o.at("beta1").f64();
            c->optimizer.beta2 = o.at("beta2").f64();
            c->optimizer.epsilon = o.at("epsilon").f64();
            only(o.at("schedule"), {"warmup_steps"}, "the schedule");
            c->optimizer.warmup_steps = o.at("schedule").at("warmup_steps").u64();
        }
        const msx::json::Value& rng = manifest.at("rng");
        only(rng, {"algorithm", "seed", "counter"}, "the rng");
        if (rng.at("algorithm").str() != "Philox4x32x10") throw std::runtime_error("unknown rng algorithm `" + rng.at("algorithm").str() + "`");
        c->seed = rng.at("seed").u64();
        c->counter = rng.at("counter").u64();
        const msx::json::Value &ps = manifest.at("parameters"), &ss = manifest.at("optimizer_slots");
        if (ps.kind != msx::json::Value::Array || ss.kind != msx::json::Value::Array) throw std::runtime_error("a record list is not a list");
        if (ps.items.size() + ss.items.size() > most)
            throw outside("the manifest has " + std::to_string(ps.items.size() + ss.items.size()) + " records, more than the " + std::to_string(most) +
                          " a " + std::to_string(size) + "-byte file can hold");
        for (const msx::json::Value& v : ps.items) parameters.push_back(record_of(v));
        for (const msx::json::Value& v : ss.items) slots.push_back(record_of(v));
        // The invariants the manifest's own fields state (checkpoint.rs:870-921).
        if (!is_uuid(c->checkpoint_id)) throw bad("checkpoint_id \"" + c->checkpoint_id + "\" is not a UUID");
        if (!fits) throw bad("the optimizer's fields do not fit its kind");
        if (kind == "Sgd" && !slots.empty()) throw bad("an SGD checkpoint has optimizer slots");
        if (parameters.empty()) throw bad("the manifest has no parameter");
        std::set<std::string> paths;
        for (const Record& r : parameters) {
            if (r.has_slot) throw bad("parameter `" + r.tensor.path + "` has a slot name");
            if (!paths.insert(r.tensor.path).second) throw bad("parameter `" + r.tensor.path + "` is recorded twice");
        }
        std::set<std::pair<std::string, std::string>> named;
        for (const Record& r : slots) {
            if (!r.has_slot) throw bad("an optimizer slot of `" + r.tensor.path + "` has no name");
            if (!named.insert({r.tensor.path, r.tensor.slot}).second) throw bad("slot `" + r.tensor.slot + "` of `" + r.tensor.path + "` is recorded twice");
        }
        for (const std::vector<Record>* list : {&parameters, &slots})
            for (const Record& r : *list) {
                if (std::find(r.tensor.shape.begin(), r.tensor.shape.end(), 0ull) != r.tensor.shape.end())
                    throw bad("parameter `" + r.tensor.path + "` has a zero dimension");
                if (r.length == 0) throw bad("parameter `" + r.tensor.path + "` has length 0");
            }
    } catch (const Refused&) {
        throw;
    } catch (const std::exception& e) {
        throw bad(std::string("the manifest is not a checkpoint manifest: ") + e.what());
    }
    if (manifest.at("file_size").u64() != size)
        throw outside("the manifest's file_size " + std::to_string(manifest.at("file_size").u64()) + " is not the file's " + std::to_string(size) + " bytes");
    if (manifest.at("alignment").u64() != kAlignment)
        throw outside("the alignment " + std::to_string(manifest.at("alignment").u64()) + " is not " + std::to_string(kAlignment));
    struct Extent {
        uint64_t from, to;
        const std::string* path;
    };
    std::vector<Extent> extents;
    for (const std::vector<Record>* list : {&parameters, &slots})
        for (const Record& r : *list) {
            auto at = [&](const std::string& what) { return outside("parameter `" + r.tensor.path + "`: " + what); };
            if (r.offset % kAlignment != 0) throw at("offset " + std::to_string(r.offset) + " is not a multiple of " + std::to_string(kAlignment));
            if (r.offset < manifest_end)
                throw at("offset " + std::to_string(r.offset) + " lies inside the header or manifest, which end at " + std::to_string(manifest_end));
            if (r.length > UINT64_MAX - r.offset || r.offset + r.length > size)
                throw at("offset " + std::to_string(r.offset) + " and length " + std::to_string(r.length) + " end past the " + std::to_string(size) + "-byte file");
            unsigned __int128 expected = 4;
            bool fits = true;
            for (uint64_t d : r.tensor.shape) {
                expected *= d;
                if (expected > UINT64_MAX) fits = false, expected = 0;
            }
            if (!fits || static_cast<uint64_t>(expected) != r.length) {
                std::string shape = "[";
                for (size_t i = 0; i < r.tensor.shape.size(); ++i) shape += (i ? ", " : "") + std::to_string(r.tensor.shape[i]);
                throw at("length " + std::to_string(r.length) + " is not the shape " + shape + "] times 4 bytes");
            }
            extents.push_back({r.offset, r.offset + r.length, &r.tensor.path});
        }
    std::sort(extents.begin(), extents.end(), [](const Extent& a, const Extent& b) {
        return a.from != b.from ? a.from < b.from : a.to != b.to ? a.to < b.to : *a.path < *b.path;
    });
    for (size_t i = 1; i < extents.size(); ++i)
        if (extents[i].from < extents[i - 1].to) throw outside("parameters `" + *extents[i - 1].path + "` and `" + *extents[i].path + "` overlap");
    uint64_t last = manifest_end;
    for (const Extent& e : extents) last = std::max(last, e.to);
    if (last != size)
        throw outside("the file has " + std::to_string(size) + " bytes and does not end at the end of its last tensor, byte " + std::to_string(last));
    uint64_t cursor = manifest_end;
    for (const Extent& e : extents) {
        for (uint64_t i = cursor; i < e.from; ++i)
            if (bytes[i] != 0) throw outside("byte " + std::to_string(i) + " lies between tensors and is not zero");
        cursor = e.to;
    }
    if (blake3_hex(bytes + payload_start, size - payload_start) != manifest.at("payload_hash").str())
        throw Refused{MSX_BAD_INPUT, "E-CKPT-004: the payload hash differs from the payload (file " + path + ")"};
    auto take = [&](std::vector<Record>& list, std::vector<Tensor>& into) {
        for (Record& r : list) {
            r.tensor.data.resize(r.length / 4);
            for (size_t i = 0; i < r.tensor.data.size(); ++i) {
                const uint32_t bits = get32(bytes + r.offset + 4 * i);
                std::memcpy(&r.tensor.data[i], &bits, 4);
            }
            into.push_back(std::move(r.tensor));
        }
    };
    take(parameters, c->parameters);
    take(slots, c->slots);
}

template <class F> int guarded(msx_checkpoint* c, F body) {
    try {
        body();
        return MSX_OK;
    } catch (const Refused& r) {
        c->error = r.what;
        return r.status;
    } catch (const std::exception& e) {
        c->error = e.what();
        return MSX_UNSUPPORTED;
    }
}

const Tensor* tensor_at(const msx_checkpoint* c, int list, uint32_t index) {
    const std::vector<Tensor>& v = list == 0 ? c->parameters : c->slots;
    return index < v.size() ? &v[index] : nullptr;
}

}  // namespace

extern "C" {

int msx_checkpoint_new(uint64_t step, uint64_t seed, const char* schema_hash, msx_checkpoint** out) {
    if (!schema_hash || !out) return MSX_BAD_ARGUMENT;
    msx_checkpoint* c = new msx_checkpoint;
    c->step = step;
    c->seed = seed;
    c->schema_hash = schema_hash;
    *out = c;
    return MSX_OK;
}

void msx_checkpoint_destroy(msx_checkpoint* c) { delete c; }
const char* msx_checkpoint_last_error(const msx_checkpoint* c) { return c ? c->error.c_str() : ""; }

int msx_checkpoint_set_optimizer(msx_checkpoint* c, int kind, double learning_rate, double weight_decay, double beta1, double beta2,
                                 double epsilon, uint64_t warmup_steps) {
    if (!c || (kind != MSX_OPTIMIZER_SGD && kind != MSX_OPTIMIZER_ADAMW)) return MSX_BAD_ARGUMENT;
    c->optimizer = Optimizer{kind, learning_rate, weight_decay, beta1, beta2, epsilon, warmup_steps};
    return MSX_OK;
}

int msx_checkpoint_add(msx_checkpoint* c, const char* path, const char* slot, const uint64_t* shape, uint32_t rank, const float* data) {
    if (!c || !path || (rank && !shape) || !data) return MSX_BAD_ARGUMENT;
    return guarded(c, [&] {
        if (rank > kMaxRank)
            throw Refused{MSX_BAD_ARGUMENT, std::string("parameter `") + path + "` has " + std::to_string(rank) + " dimensions, more than the " +
                                                std::to_string(kMaxRank) + " a checkpoint holds"};
        Tensor t;
        t.path = path;
        t.slot = slot ? slot : "";
        t.shape.assign(shape, shape + rank);
        if (t.count() == 0) throw Refused{MSX_BAD_ARGUMENT, std::string("parameter `") + path + "` has a zero dimension"};
        t.data.assign(data, data + t.count());
        // Both lists stay in (path, slot) order, the order of the file.
        std::vector<Tensor>& list = t.slot.empty() ? c->parameters : c->slots;
        auto at = std::upper_bound(list.begin(), list.end(), t, [](const Tensor& a, const Tensor& b) { return a.path != b.path ? a.path < b.path : a.slot < b.slot; });
        list.insert(at, std::move(t));
    });
}

uint64_t msx_checkpoint_encode(msx_checkpoint* c, void* out, uint64_t capacity) {
    if (!c) return 0;
    std::string bytes = encode(c);
    if (out && capacity >= bytes.size()) std::memcpy(out, bytes.data(), bytes.size());
    return bytes.size();
}

// checkpoint.rs:629-665: the bytes go to `<path>.tmp` beside it, are synced and then renamed over
// `path`, so a write that fails part-way leaves the earlier file at `path`.
int msx_checkpoint_write(msx_checkpoint* c, const char* path) {
    if (!c || !path) return MSX_BAD_ARGUMENT;
    return guarded(c, [&] {
        const std::string bytes = encode(c), staged = std::string(path) + ".tmp";
        auto failed = [&](const std::string& why) { return Refused{MSX_BAD_INPUT, std::string("cannot write checkpoint ") + path + ": " + why}; };
        FILE* f = std::fopen(staged.c_str(), "wb");
        if (!f) throw failed(std::strerror(errno));
        const bool written = std::fwrite(bytes.data(), 1, bytes.size(), f) == bytes.size() && std::fflush(f) == 0;
        const int closed = std::fclose(f);
        if (!written || closed != 0 || std::rename(staged.c_str(), path) != 0) {
            const std::string why = std::strerror(errno);
            std::remove(staged.c_str());
            throw failed(why);
        }
    });
}

int msx_checkpoint_read(const char* path, msx_checkpoint** out) {
    if (!path || !out) return MSX_BAD_ARGUMENT;
    *out = nullptr;
    std::unique_ptr<msx_checkpoint> c(new msx_checkpoint);
    int rc = guarded(c.get(), [&] { read(c.get(), path); });
    if (rc != MSX_OK) {
        msx_internal_set_error(nullptr, c->error.c_str());  // where msx_last_error(NULL) finds it
        return rc;
    }
    *out = c.release();
    return MSX_OK;
}

uint64_t msx_checkpoint_step(const msx_checkpoint* c) { return c ? c->step : 0; }
uint64_t msx_checkpoint_seed(const msx_checkpoint* c) { return c ? c->seed : 0; }
const char* msx_checkpoint_schema_hash(const msx_checkpoint* c) { return c ? c->schema_hash.c_str() : ""; }
const char* msx_checkpoint_id(const msx_checkpoint* c) { return c ? c->checkpoint_id.c_str() : ""; }
int msx_checkpoint_optimizer(const msx_checkpoint* c, int* kind, double* learning_rate, double* weight_decay, double* beta1, double* beta2,
                             double* epsilon, uint64_t* warmup_steps) {
    if (!c) return MSX_BAD_ARGUMENT;
    if (kind) *kind = c->optimizer.kind;
    if (learning_rate) *learning_rate = c->optimizer.learning_rate;
    if (weight_decay) *weight_decay = c->optimizer.weight_decay;
    if (beta1) *beta1 = c->optimizer.beta1;
    if (beta2) *beta2 = c->optimizer.beta2;
    if (epsilon) *epsilon = c->optimizer.epsilon;
    if (warmup_steps) *warmup_steps = c->optimizer.warmup_steps;
    return MSX_OK;
}
uint64_t msx_checkpoint_optimizer_json(const msx_checkpoint* c, char* out, uint64_t capacity) {
    if (!c) return 0;
    std::string text = c->optimizer.json();
    if (out && capacity) {
        size_t n = std::min<size_t>(capacity - 1, text.size());
        std::memcpy(out, text.data(), n);
        out[n] = 0;
    }
    return text.size() + 1;
}
uint32_t msx_checkpoint_count(const msx_checkpoint* c, int list) { return c ? static_cast<uint32_t>((list == 0 ? c->parameters : c->slots).size()) : 0; }
const char* msx_checkpoint_path(const msx_checkpoint* c, int list, uint32_t index) {
    const Tensor* t = c ? tensor_at(c, list, index) : nullptr;
    return t ? t->path.c_str() : "";
}
const char* msx_checkpoint_slot(const msx_checkpoint* c, int list, uint32_t index) {
    const Tensor* t = c ? tensor_at(c, list, index) : nullptr;
    return t ? t->slot.c_str() : "";
}
uint32_t msx_checkpoint_rank(const msx_checkpoint* c, int list, uint32_t index) {
    const Tensor* t = c ? tensor_at(c, list, index) : nullptr;
    return t ? static_cast<uint32_t>(t->shape.size()) : 0;
}
const uint64_t* msx_checkpoint_shape(const msx_checkpoint* c, int list, uint32_t index) {
    const Tensor* t = c ? tensor_at(c, list, index) : nullptr;
    return t ? t->shape.data() : nullptr;
}
const float* msx_checkpoint_data(const msx_checkpoint* c, int list, uint32_t index) {
    const Tensor* t = c ? tensor_at(c, list, index) : nullptr;
    return t ? t->data.data() : nullptr;
}

}  // extern "C"
