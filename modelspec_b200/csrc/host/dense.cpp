// The dense feed of `train --data <directory>`: one headerless little-endian file per `input` and
// `target` declaration of the train block, `<dir>/<name>.f32` or `<dir>/<name>.i32`, and an
// optional `<dir>/order.u32`; the batch of every step as the reference assembles it.
//
// Follows crates/modelspec-runtime/src/train/data.rs of the reference: the layout and the sample
// rule (:14-35), `dense` with the order file and its two refusals (:513-577), `read_files` with the
// batch dimension B (:837-876), `read_tensor` and its refusals (:1232-1290), `non_finite`
// (:1328-1339), `refuse_out_of_range` (:957-1004) and `fill_step` (:446-454). Host code only: the
// step uploads a batch with its other inputs.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../../../include/msx.h"

extern "C" void msx_internal_set_error(msx_device* device, const char* message);

namespace {

struct Refused {
    int status;
    std::string what;
};

struct Tensor {
    std::string name;
    bool i32 = false;
    uint32_t role = 0;           // 0 an input, 1 a target, 2 an argument of an inference entry
    uint64_t sample = 0;         // values of one sample
    const char* role_name() const { return role == 1 ? "target" : role == 2 ? "argument" : "input"; }
    std::vector<char> values;    // the whole file: f32 or i32, 4 bytes a value
    uint64_t count() const { return values.size() / 4; }
};

// The file's bytes; false when it cannot be opened (errno names why).
bool read_file(const std::string& path, std::vector<char>* out) {
    std::ifstream in(path, std::ios::binary | std::ios::ate);
    if (!in) return false;
    const std::streamoff size = in.tellg();
    out->resize(static_cast<size_t>(size));
    in.seekg(0);
    if (size > 0) in.read(out->data(), size);
    return static_cast<bool>(in) || size == 0;
}

bool is_file(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    return static_cast<bool>(in);
}

// An f32 as the reference prints one in a diagnostic (`NaN`, `inf`, `-inf`).
std::string shown(float v) {
    if (v != v) return "NaN";
    if (std::isinf(v)) return v > 0 ? "inf" : "-inf";
    std::ostringstream s;
    s << v;
    return s.str();
}

}  // namespace

struct msx_dense {
    std::string dir;
    std::vector<Tensor> tensors;   // in source order
    uint64_t batch = 1, samples = 0;
    std::vector<uint32_t> order;   // empty: none
    bool has_order = false;
    std::string error;
};

namespace {

thread_local std::string g_error;

int refuse(msx_dense* d, const Refused& r) {
    g_error = r.what;
    if (d) d->error = r.what;
    msx_internal_set_error(nullptr, r.what.c_str());
    return r.status;
}

// read_tensor (data.rs:1232-1290).
void read_tensor(const std::string& dir, Tensor* t) {
    const char* role = t->role_name();
    const std::string ext = t->i32 ? "i32" : "f32", other = t->i32 ? "f32" : "i32";
    const std::string path = dir + "/" + t->name + "." + ext;
    const std::string what = std::string("the data file of the ") + role + " `" + t->name + "`";
    if (!read_file(path, &t->values)) {
        std::string message = "E-DATA-007: cannot read " + what + " (file " + path + ")";
        const std::string found = dir + "/" + t->name + "." + other;
        if (is_file(found))
            message += "; found " + found + ", the file of an " + other + " declaration; `" + t->name + "` is declared " + ext;
        throw Refused{MSX_BAD_INPUT, message};
    }
    if (t->values.size() % 4 != 0)
        throw Refused{MSX_BAD_INPUT, "E-DATA-007: cannot read " + what + " (file " + path + "): " + std::to_string(t->values.size()) +
                                         " bytes is not a whole number of " + ext + " values"};
    const uint64_t len = t->count();
    if (len == 0 || t->sample == 0 || len % t->sample != 0)
        throw Refused{MSX_BAD_INPUT, "E-DATA-007: " + what + " is not a whole number of samples (file " + path + ", values " + std::to_string(len) +
                                         ", sample " + std::to_string(t->sample) + " values)"};
    if (!t->i32) {
        const float* v = reinterpret_cast<const float*>(t->values.data());
        for (uint64_t i = 0; i < len; ++i)
            if (!std::isfinite(v[i]))
                throw Refused{MSX_BAD_INPUT, "E-DATA-007: " + what + " holds a value that is not finite (file " + path + ", index " + std::to_string(i) +
                                                 ", value " + shown(v[i]) + ")"};
    }
}

// `dense` and `dense_eval` (data.rs:513-600): the files of every declaration, then either the
// optional order of a run or the whole-batches rule of an evaluation.
int open_dense(const char* dir, uint32_t count, const char* const* names, const uint32_t* is_i32, const uint32_t* is_target,
               const uint32_t* ranks, const uint64_t* shapes, uint64_t steps, bool eval, msx_dense** out) {
    if (!dir || !out || (count && (!names || !is_i32 || !is_target || !ranks || !shapes))) return MSX_BAD_ARGUMENT;
    *out = nullptr;
    msx_dense* d = new msx_dense();
    d->dir = dir;
    try {
        if (count == 0) throw Refused{MSX_BAD_INPUT, "E-DATA-001: dense data needs an input or a target (inputs 0, targets 0)"};
        // read_files (data.rs:837-876): B is the leading dimension every declaration shares, else 1.
        std::vector<uint64_t> elements(count, 1), leading(count, 0);
        std::vector<bool> has_leading(count, false);
        const uint64_t* shape = shapes;
        for (uint32_t i = 0; i < count; ++i) {
            for (uint32_t a = 0; a < ranks[i]; ++a) elements[i] *= shape[a];
            if (ranks[i] > 0) {
                has_leading[i] = true;
                leading[i] = shape[0];
            }
            shape += ranks[i];
        }
        bool shared = has_leading[0];
        for (uint32_t i = 0; i < count && shared; ++i) shared = has_leading[i] && leading[i] == leading[0];
        d->batch = shared ? leading[0] : 1;
        if (d->batch == 0) throw Refused{MSX_BAD_INPUT, "E-INIT-001: the shape of `" + std::string(names[0]) + "` has no elements"};
        for (uint32_t i = 0; i < count; ++i) {
            Tensor t;
            t.name = names[i];
            t.i32 = is_i32[i] != 0;
            t.role = is_target[i] <= 2 ? is_target[i] : 0;
            t.sample = shared ? elements[i] / d->batch : elements[i];
            read_tensor(d->dir, &t);
            d->tensors.push_back(std::move(t));
        }
        d->samples = d->tensors[0].count() / d->tensors[0].sample;
        bool same = true;
        for (const Tensor& t : d->tensors) same = same && t.count() / t.sample == d->samples;
        if (!same) {
            std::string message = "E-DATA-007: the data files do not hold the same number of samples (directory " + d->dir;
            for (const Tensor& t : d->tensors) message += ", " + t.name + " " + std::to_string(t.count() / t.sample);
            throw Refused{MSX_BAD_INPUT, message + ")"};
        }
        // dense_eval (:588-595) and dense_function (:707-714) word the same rule differently.
        if (eval && d->samples % d->batch != 0)
            throw Refused{MSX_BAD_INPUT, std::string("E-DATA-009: ") + (d->tensors[0].role == 2 ? "the data is not a whole number of blocks"
                                                                                                 : "the eval data is not a whole number of batches") +
                                             " (directory " + d->dir + ", samples " + std::to_string(d->samples) + ", batch " + std::to_string(d->batch) + ")"};
        // dense (data.rs:513-577): the optional order, which an eval directory does not read.
        const std::string path = d->dir + "/order.u32";
        std::vector<char> bytes;
        if (!eval && read_file(path, &bytes)) {
            if (bytes.size() % 4 != 0)
                throw Refused{MSX_BAD_INPUT, "E-DATA-007: the order file is not a whole number of u32 indices (file " + path + ", bytes " +
                                                 std::to_string(bytes.size()) + ")"};
            d->order.resize(bytes.size() / 4);
            if (!bytes.empty()) std::memcpy(d->order.data(), bytes.data(), bytes.size());
            const unsigned __int128 needed = static_cast<unsigned __int128>(steps) * d->batch;
            if (static_cast<unsigned __int128>(d->order.size()) < needed || d->order.empty()) {
                const uint64_t shown_needed = needed > 0 ? static_cast<uint64_t>(needed) : 1;
                throw Refused{MSX_BAD_INPUT, "E-DATA-008: the order file holds fewer than steps · B indices (file " + path + ", indices " +
                                                 std::to_string(d->order.size()) + ", needed " + std::to_string(shown_needed) + ")"};
            }
            for (size_t p = 0; p < d->order.size(); ++p)
                if (d->order[p] >= d->samples)
                    throw Refused{MSX_BAD_INPUT, "E-DATA-008: the order file names a sample past the end of the data (file " + path + ", position " +
                                                     std::to_string(p) + ", index " + std::to_string(d->order[p]) + ", samples " +
                                                     std::to_string(d->samples) + ")"};
            d->has_order = true;
        }
    } catch (const Refused& r) {
        const int status = refuse(nullptr, r);
        delete d;
        return status;
    } catch (const std::exception& e) {
        const int status = refuse(nullptr, Refused{MSX_BAD_INPUT, e.what()});
        delete d;
        return status;
    }
    *out = d;
    return MSX_OK;
}

}  // namespace

extern "C" {

int msx_dense_open(const char* dir, uint32_t count, const char* const* names, const uint32_t* is_i32, const uint32_t* is_target,
                   const uint32_t* ranks, const uint64_t* shapes, uint64_t steps, msx_dense** out) {
    return open_dense(dir, count, names, is_i32, is_target, ranks, shapes, steps, false, out);
}

// dense_eval (data.rs:582-600): the same files, no order, a whole number of batches.
int msx_dense_open_eval(const char* dir, uint32_t count, const char* const* names, const uint32_t* is_i32, const uint32_t* is_target,
                        const uint32_t* ranks, const uint64_t* shapes, msx_dense** out) {
    return open_dense(dir, count, names, is_i32, is_target, ranks, shapes, 0, true, out);
}

void msx_dense_close(msx_dense* dense) { delete dense; }

const char* msx_dense_last_error(const msx_dense* dense) { return dense ? dense->error.c_str() : g_error.c_str(); }

uint64_t msx_dense_batch(const msx_dense* dense) { return dense ? dense->batch : 0; }
uint64_t msx_dense_samples(const msx_dense* dense) { return dense ? dense->samples : 0; }
int msx_dense_has_order(const msx_dense* dense) { return dense && dense->has_order ? 1 : 0; }
uint32_t msx_dense_tensors(const msx_dense* dense) { return dense ? static_cast<uint32_t>(dense->tensors.size()) : 0; }
uint64_t msx_dense_batch_bytes(const msx_dense* dense, uint32_t index) {
    return dense && index < dense->tensors.size() ? dense->tensors[index].sample * dense->batch * 4 : 0;
}

// refuse_out_of_range (data.rs:957-1004) for one declaration and the tightest bound that reads it.
int msx_dense_check_bound(msx_dense* dense, uint32_t index, uint64_t bound, const char* what) {
    if (!dense || index >= dense->tensors.size() || !what) return MSX_BAD_ARGUMENT;
    const Tensor& t = dense->tensors[index];
    if (!t.i32) return MSX_OK;
    const int32_t* v = reinterpret_cast<const int32_t*>(t.values.data());
    for (uint64_t p = 0; p < t.count(); ++p)
        if (v[p] < 0 || static_cast<uint64_t>(v[p]) >= bound)
            return refuse(dense, Refused{MSX_BAD_INPUT, std::string("E-DATA-011: the data file of the ") + t.role_name() + " `" + t.name +
                                                            "` holds " + std::to_string(v[p]) + ", outside " + what + " (file " + dense->dir + "/" + t.name +
                                                            ".i32, position " + std::to_string(p) + ", value " + std::to_string(v[p]) +
                                                            ", bound 0 <= value < " + std::to_string(bound) + ")"});
    return MSX_OK;
}

// fill_step (data.rs:446-454): the samples order[(k B + i) mod len] with an order, (k B + i) mod N
// without one, for i in 0 .. B.
int msx_dense_step(const msx_dense* dense, uint32_t index, uint64_t step, void* out, uint64_t capacity_bytes) {
    if (!dense || index >= dense->tensors.size() || !out) return MSX_BAD_ARGUMENT;
    const Tensor& t = dense->tensors[index];
    const uint64_t sample_bytes = t.sample * 4;
    if (capacity_bytes < sample_bytes * dense->batch) return MSX_BAD_ARGUMENT;
    const unsigned __int128 first = static_cast<unsigned __int128>(step) * dense->batch;
    for (uint64_t i = 0; i < dense->batch; ++i) {
        const unsigned __int128 position = first + i;
        const uint64_t sample = dense->has_order ? dense->order[static_cast<size_t>(position % dense->order.size())]
                                                 : static_cast<uint64_t>(position % dense->samples);
        std::memcpy(static_cast<char*>(out) + i * sample_bytes, t.values.data() + sample * sample_bytes, sample_bytes);
    }
    return MSX_OK;
}

// fill_eval_batch (data.rs:456-460): the samples b B .. (b + 1) B.
int msx_dense_eval_batch(const msx_dense* dense, uint32_t index, uint64_t batch, void* out, uint64_t capacity_bytes) {
    if (!dense || index >= dense->tensors.size() || !out) return MSX_BAD_ARGUMENT;
    const Tensor& t = dense->tensors[index];
    const uint64_t bytes = t.sample * 4 * dense->batch;
    if (capacity_bytes < bytes || batch >= dense->samples / dense->batch) return MSX_BAD_ARGUMENT;
    std::memcpy(out, t.values.data() + batch * bytes, bytes);
    return MSX_OK;
}

}  // extern "C"
