// The host loop of a training run, written against the msx C ABI alone (no CUDA call here): the
// counterpart of the reference's device runner vulkan::stepwise::train_stepwise_on_device
// (crates/modelspec-runtime/src/vulkan/stepwise.rs:289-296, :400-) and of the CPU loop
// train::runner::run_checked (crates/modelspec-runtime/src/train/runner.rs:365-512).
//
// Per step the host supplies what the reference's host supplies (stepwise.rs:475-543): the AdamW
// scalars of t = step + 1, the dropout token of every site at this step, the masked-row gather of
// the batch, and the batch itself. Parameters start from their initializers on Philox stream 0.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <set>

#include <fcntl.h>
#include <limits.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>

#include "../../../include/msx.h"
#include "../core/frontend.hpp"
#include "../core/init.hpp"
#include "../core/schema.hpp"

// Defined beside msx_last_error: records a message on the device handle.
extern "C" void msx_internal_set_error(msx_device* device, const char* message);

struct msx_training {
    msx_device* device = nullptr;
    msx::Compiled compiled;
    msx_plan* step = nullptr;
    msx_plan* forward = nullptr;
    msx_plan* infer = nullptr;  // the forward program with the prediction as a second output, made on first use
    // Held-out evaluation: the steps the prediction is computed from, the device reduction of its
    // logits, and the batches of the split, drawn once per run.
    msx_plan* predict = nullptr;
    msx_heldout* heldout = nullptr;
    std::string heldout_labels, heldout_weights;
    std::vector<std::map<std::string, std::vector<char>>> heldout_batches;
    std::vector<std::vector<float>> heldout_row_weights;  // per batch, once its targets are on the device
    std::set<std::string> predict_inputs;
    // A packed --data directory bound to the declarations (train/data.rs:1488-1500).
    // Restore and replay (stepwise.rs:84-92): a snapshot before every `window`-th step, and what
    // each step since was run on.
    uint32_t window = 0;
    struct Replayed {
        uint64_t step, end;
        std::map<std::string, std::vector<char>> batch;
    };
    std::vector<Replayed> since_snapshot;
    std::string report;  // the standard output of the last msx_training_run
    std::string schema;  // the schema hash of the training program's parameters, made on first use
    msx_dense* dense = nullptr;  // a dense --data directory, owned (train/data.rs:513-577)
    msx_packed* packed = nullptr;
    uint64_t packed_batch = 0;
    std::vector<std::string> packed_bound;  // the declared batch tensors, in source order
    uint32_t flags = 0;
    std::string error;
    std::map<std::string, std::vector<char>> batch;  // declared inputs and targets, by name
    std::vector<std::string> sites;                  // dropout token inputs of the step
    std::set<std::string> step_inputs, forward_inputs;
    bool submitted = false;
    std::map<uint64_t, uint64_t> submitted_as;  // run step -> submission number on the step plan
};

namespace {

struct Fail {
    int status;
    std::string what;
};

void ok(msx_training* t, int rc) {
    if (rc != MSX_OK) throw Fail{rc, msx_last_error(t->device)};
}

template <class F> int guarded(msx_training* t, F body) {
    try {
        body();
        return MSX_OK;
    } catch (const Fail& f) {
        t->error = f.what;
        return f.status;
    } catch (const std::exception& e) {
        t->error = e.what();
        return MSX_UNSUPPORTED;
    }
}

std::set<std::string> input_names(const msx_plan* plan) {
    std::set<std::string> out;
    for (uint32_t i = 0; i < msx_plan_input_count(plan); ++i) out.insert(msx_plan_input_name(plan, i));
    return out;
}

const msx::DataDecl* declared(const msx_training* t, const std::string& name) {
    for (const msx::DataDecl& d : t->compiled.config.data)
        if (d.name == name) return &d;
    return nullptr;
}

// The host side of the masked-row gather (crates/modelspec-runtime/src/train/masked.rs:88-128):
// the rows of non-zero weight in ascending order with their labels and weights, then padding
// rows of row 0, label 0 and weight +0.0; more selected rows than the capacity is refused.
void gather_masked(msx_training* t, uint64_t step, bool stage) {
    const msx::Compiled& c = t->compiled;
    if (!c.masked_rows) return;
    auto w = t->batch.find(c.masked_weights), l = t->batch.find(c.masked_labels);
    if (w == t->batch.end() || l == t->batch.end())
        throw Fail{MSX_BAD_INPUT, "E-DATA-012: the batch of step " + std::to_string(step) + " holds no `" +
                                      (w == t->batch.end() ? c.masked_weights : c.masked_labels) + "` to gather the masked rows from"};
    const float* weights = reinterpret_cast<const float*>(w->second.data());
    const int32_t* labels = reinterpret_cast<const int32_t*>(l->second.data());
    size_t rows = w->second.size() / 4, capacity = c.masked_rows;
    std::vector<int32_t> ids, lab;
    std::vector<float> wt;
    for (size_t r = 0; r < rows; ++r)
        if (weights[r] != 0.0f) {
            ids.push_back(static_cast<int32_t>(r));
            lab.push_back(r < l->second.size() / 4 ? labels[r] : 0);
            wt.push_back(weights[r]);
        }
    if (ids.size() > capacity)
        throw Fail{MSX_BAD_INPUT, "E-DATA-012: the batch of step " + std::to_string(step) + " has " + std::to_string(ids.size()) +
                                      " rows of non-zero `" + c.masked_weights + "`, more than the " + std::to_string(capacity) +
                                      " rows the masked-row gather holds"};
    if (!stage) return;
    ids.resize(capacity, 0);
    lab.resize(capacity, 0);
    wt.resize(capacity, 0.0f);
    ok(t, msx_set_input(t->step, "masked.rows", ids.data(), capacity * 4));
    ok(t, msx_set_input(t->step, ("masked.labels." + c.masked_labels).c_str(), lab.data(), capacity * 4));
    ok(t, msx_set_input(t->step, ("masked.weights." + c.masked_weights).c_str(), wt.data(), capacity * 4));
}

void stage_batch(msx_training* t, msx_plan* plan, const std::set<std::string>& reads) {
    for (const auto& [name, bytes] : t->batch)
        if (reads.count(name)) ok(t, msx_set_input(plan, name.c_str(), bytes.data(), bytes.size()));
}

}  // namespace

extern "C" {

extern "C++" {
namespace {

// The plans of a compiled entry (the train block, or a model function as an inference entry) and
// its parameters as the run's seed initialises them.
template <class Compile> int create_from(msx_device* device, uint32_t flags, msx_training** out, Compile compile) {
    *out = nullptr;
    msx_training* t = new msx_training;
    t->device = device;
    t->flags = flags;
    int rc = guarded(t, [&] {
        try {
            t->compiled = compile();
        } catch (const msx::Error& e) {
            const std::string what = e.what();
            throw Fail{what.rfind("E-DATA-", 0) == 0 ? MSX_BAD_INPUT : MSX_UNSUPPORTED, what};
        }
        const msx::Compiled& c = t->compiled;
        if (c.config.rule == msx::Rule::AdamW && c.config.steps > 0 && c.config.adamw.warmup_steps >= c.config.steps)
            throw Fail{MSX_BAD_ARGUMENT, "warmup_steps " + std::to_string(c.config.adamw.warmup_steps) +
                                             " is not below the run's " + std::to_string(c.config.steps) + " steps"};
        std::string step_ir = msx::print_program(c.step), forward_ir = msx::print_program(c.forward);
        ok(t, msx_plan_create(device, step_ir.c_str(), c.config.seed, flags, nullptr, &t->step));
        ok(t, msx_plan_create(device, forward_ir.c_str(), c.config.seed, flags, t->step, &t->forward));
        t->step_inputs = input_names(t->step);
        t->forward_inputs = input_names(t->forward);
        for (const std::string& name : t->step_inputs)
            if (name.find(".dropout#") != std::string::npos) t->sites.push_back(name);
        // A parameter the step does not hold (the loss does not reach it) lives in the forward
        // plan alone; both are initialised.
        for (uint32_t p = 0; p < c.step.params.size(); ++p) {
            std::vector<float> value = msx::initial_parameter(c.step.params[p], c.config.seed, msx::kStreamInit);
            int rs = msx_param_upload(t->step, p, value.data(), value.size() * 4);
            int rf = msx_param_upload(t->forward, p, value.data(), value.size() * 4);
            // (a model function as an entry may read a part of the file's parameters only)
            if (rs != MSX_OK && rf != MSX_OK && c.function.empty()) throw Fail{rs, msx_last_error(device)};
        }
    });
    if (rc != MSX_OK) {
        std::string why = t->error;
        msx_training_destroy(t);
        msx_internal_set_error(device, why.c_str());  // where msx_last_error(device) finds it
        return rc;
    }
    *out = t;
    return MSX_OK;
}

}  // namespace
}  // extern "C++"

int msx_training_create(msx_device* device, const char* source, uint64_t masked_rows, uint32_t flags, msx_training** out) {
    if (!device || !source || !out) return MSX_BAD_ARGUMENT;
    return create_from(device, flags, out, [&] { return msx::compile_training(source, masked_rows); });
}

int msx_training_create_function(msx_device* device, const char* source, const char* name, uint32_t flags, msx_training** out) {
    if (!device || !source || !name || !out) return MSX_BAD_ARGUMENT;
    return create_from(device, flags, out, [&] { return msx::compile_function(source, name); });
}

void msx_training_destroy(msx_training* t) {
    if (!t) return;
    if (t->dense) msx_dense_close(t->dense);
    if (t->heldout) msx_heldout_destroy(t->heldout);
    if (t->predict) msx_plan_destroy(t->predict);
    if (t->infer) msx_plan_destroy(t->infer);
    if (t->forward) msx_plan_destroy(t->forward);
    if (t->step) msx_plan_destroy(t->step);
    delete t;
}

msx_plan* msx_training_step_plan(msx_training* t) { return t ? t->step : nullptr; }
msx_plan* msx_training_forward_plan(msx_training* t) { return t ? t->forward : nullptr; }
uint64_t msx_training_steps(const msx_training* t) { return t ? t->compiled.config.steps : 0; }
uint64_t msx_training_seed(const msx_training* t) { return t ? t->compiled.config.seed : 0; }
const char* msx_training_last_error(const msx_training* t) { return t ? t->error.c_str() : ""; }

int msx_training_comm_init(msx_training* t, int rank, int world, const void* unique_id_128, uint64_t rows_per_rank) {
    if (!t || !unique_id_128) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        ok(t, msx_comm_init(t->step, rank, world, unique_id_128));
        ok(t, msx_comm_share(t->forward, t->step));
        ok(t, msx_set_shard(t->step, static_cast<uint64_t>(rank) * rows_per_rank, static_cast<uint64_t>(world) * rows_per_rank));
    });
}

int msx_training_set_input(msx_training* t, const char* name, const void* host, uint64_t bytes) {
    if (!t || !name || !host) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::DataDecl* d = declared(t, name);
        if (!d) throw Fail{MSX_BAD_ARGUMENT, std::string("the train block declares no `") + name + "`"};
        if (bytes != d->ty.count() * 4)
            throw Fail{MSX_BAD_ARGUMENT, std::string("`") + name + "` is " + d->ty.str() + ": " + std::to_string(d->ty.count() * 4) + " bytes"};
        const char* b = static_cast<const char*>(host);
        t->batch[name].assign(b, b + bytes);
    });
}

int msx_training_get_input(msx_training* t, const char* name, void* host, uint64_t bytes) {
    if (!t || !name || !host) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        auto it = t->batch.find(name);
        if (it == t->batch.end() || it->second.size() != bytes) throw Fail{MSX_BAD_ARGUMENT, std::string("no batch input `") + name + "` of that size"};
        std::memcpy(host, it->second.data(), bytes);
    });
}

int msx_training_synthetic(msx_training* t) {
    if (!t) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::Compiled& c = t->compiled;
        const msx::Program& fwd = c.forward;
        // Key masks: f32 inputs read only as the fourth operand of attention (data.rs:214-245).
        std::set<std::string> masks;
        for (uint32_t in : fwd.inputs) {
            const msx::Node& n = fwd.node(in);
            if (n.ty.i32) continue;
            bool any = false, only = true;
            for (const msx::Node& user : fwd.nodes)
                for (size_t k = 0; k < user.operands.size(); ++k)
                    if (user.operands[k] == in) {
                        any = true;
                        only = only && user.op == msx::Op::Attention && k == 3;
                    }
            if (any && only) masks.insert(n.name);
        }
        const msx::DataDecl *input = nullptr, *target = nullptr;
        int inputs = 0, targets = 0;
        for (const msx::DataDecl& d : c.config.data) {
            if (masks.count(d.name)) continue;
            if (d.target) { target = &d; ++targets; }
            else { input = &d; ++inputs; }
        }
        if (inputs != 1 || targets != 1)
            throw Fail{MSX_BAD_INPUT, "E-DATA-001: M0 synthetic data takes one input besides key masks and one target"};
        if (input->ty.i32 || target->ty.i32) throw Fail{MSX_BAD_INPUT, "E-DATA-004: M0 synthetic data cannot draw an i32 tensor"};
        if (target->ty != fwd.node(c.prediction).ty)
            throw Fail{MSX_BAD_INPUT, "E-DATA-002: the target is not of the model output type\n  target: " + target->ty.str() +
                                          "\n  model output: " + fwd.node(c.prediction).ty.str()};
        std::vector<float> x = msx::standard_normal_draw(c.config.seed, msx::kStreamData, input->name, input->ty.count());
        t->batch[input->name].assign(reinterpret_cast<char*>(x.data()), reinterpret_cast<char*>(x.data()) + x.size() * 4);
        for (const msx::DataDecl& d : c.config.data)
            if (masks.count(d.name)) {
                std::vector<float> ones(d.ty.count(), 1.0f);
                t->batch[d.name].assign(reinterpret_cast<char*>(ones.data()), reinterpret_cast<char*>(ones.data()) + ones.size() * 4);
            }
        // The teacher: the forward program up to the prediction, its own parameters drawn on the
        // teacher stream.
        msx::Program predict = fwd;
        predict.outputs = {msx::Output{c.prediction, msx::Role::Plain, 0, 0}};
        predict = msx::dce(std::move(predict));
        std::string ir = msx::print_program(predict);
        msx_plan* teacher = nullptr;
        ok(t, msx_plan_create(t->device, ir.c_str(), c.config.seed, MSX_PLAN_NO_GRAPH, nullptr, &teacher));
        try {
            for (uint32_t p = 0; p < predict.params.size(); ++p) {
                std::vector<float> value = msx::initial_parameter(predict.params[p], c.config.seed, msx::kStreamTeacher);
                int rc = msx_param_upload(teacher, p, value.data(), value.size() * 4);
                (void)rc;  // a parameter the prediction does not read has no buffer
            }
            stage_batch(t, teacher, input_names(teacher));
            ok(t, msx_run(teacher));
            std::vector<char> y(target->ty.count() * 4);
            ok(t, msx_value_download(teacher, c.prediction, y.data(), y.size()));
            t->batch[target->name] = std::move(y);
        } catch (...) {
            msx_plan_destroy(teacher);
            throw;
        }
        msx_plan_destroy(teacher);
    });
}

namespace {

// Step `step` of a run that ends at `end`, on the current batch: the host inputs of the step
// (stepwise.rs:475-543), then one submission.
void submit_step(msx_training* t, uint64_t step, uint64_t end) {
    const msx::Compiled& c = t->compiled;
    if (c.config.rule == msx::Rule::AdamW) {
        msx::StepScalars s = msx::adamw_scalars(c.config.adamw, c.config.lr, step + 1, end);
        if (t->step_inputs.count("optimizer.lr_t")) {
            ok(t, msx_set_input(t->step, "optimizer.lr_t", &s.lr_t, 4));
            ok(t, msx_set_input(t->step, "optimizer.c1", &s.c1, 4));
            ok(t, msx_set_input(t->step, "optimizer.c2", &s.c2, 4));
        }
    }
    stage_batch(t, t->step, t->step_inputs);
    gather_masked(t, step, true);
    for (const std::string& site : t->sites) {
        int32_t token[2];
        msx::dropout_token(site, step, token);
        ok(t, msx_set_input(t->step, site.c_str(), token, 8));
    }
    t->submitted_as[step] = msx_steps_submitted(t->step);
    if (t->submitted_as.size() > 64) t->submitted_as.erase(t->submitted_as.begin());
    ok(t, msx_run(t->step));
    t->submitted = true;
}

}  // namespace

int msx_training_step(msx_training* t, uint64_t step, uint64_t end) {
    if (!t) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        if (t->window) {
            if (t->since_snapshot.empty() || t->since_snapshot.size() >= t->window) {
                ok(t, msx_state_snapshot(t->step));
                t->since_snapshot.clear();
            }
            t->since_snapshot.push_back({step, end, t->batch});
        }
        submit_step(t, step, end);
    });
}

int msx_training_set_replay_window(msx_training* t, uint32_t steps) {
    if (!t) return MSX_BAD_ARGUMENT;
    t->window = steps;
    t->since_snapshot.clear();
    return MSX_OK;
}

int msx_training_rewind(msx_training* t, uint64_t step) {
    if (!t) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        size_t last = t->since_snapshot.size();
        for (size_t i = 0; i < t->since_snapshot.size(); ++i)
            if (t->since_snapshot[i].step == step) last = i;
        if (last == t->since_snapshot.size())
            throw Fail{MSX_BAD_ARGUMENT, "step " + std::to_string(step) + " was not run since the last snapshot" +
                                             (t->window ? "" : " (no replay window is set)")};
        // The steps in flight finish first (their status, a wait that gave up included, is dropped
        // with them), then the segment's start comes back and its steps run again through `step`.
        msx_sync(t->step, 0);
        ok(t, msx_state_restore(t->step));
        t->since_snapshot.resize(last + 1);
        for (const msx_training::Replayed& r : t->since_snapshot) {
            t->batch = r.batch;
            submit_step(t, r.step, r.end);
        }
        ok(t, msx_sync(t->step, 0));
    });
}

int msx_training_loss_of(msx_training* t, uint64_t step, float* loss) {
    if (!t || !loss) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        auto it = t->submitted_as.find(step);
        if (it == t->submitted_as.end()) throw Fail{MSX_BAD_ARGUMENT, "step " + std::to_string(step) + " was not submitted recently"};
        ok(t, msx_loss_of(t->step, it->second, loss, 0));
        if (!std::isfinite(*loss)) throw Fail{MSX_NON_FINITE, "E-TRAIN-001: the loss of step " + std::to_string(step) + " is not finite"};
    });
}

int msx_training_loss(msx_training* t, float* loss) {
    if (!t || !loss) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        ok(t, msx_loss(t->step, loss, 0));
        if (!std::isfinite(*loss)) throw Fail{MSX_NON_FINITE, "E-TRAIN-001: the loss is not finite"};
    });
}

int msx_training_final_loss(msx_training* t, float* loss) {
    if (!t || !loss) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        // The forward plan runs on its own stream: wait for the submitted updates first.
        ok(t, msx_sync(t->step, 0));
        // The final batch is held to the gather as every trained batch is (runner.rs:467-471).
        gather_masked(t, t->compiled.config.steps, false);
        stage_batch(t, t->forward, t->forward_inputs);
        ok(t, msx_run(t->forward));
        ok(t, msx_loss(t->forward, loss, 0));
    });
}

uint64_t msx_training_prediction_count(const msx_training* t) {
    return t ? t->compiled.forward.node(t->compiled.prediction).ty.count() : 0;
}

int msx_training_infer(msx_training* t, float* prediction, uint64_t bytes, float* loss) {
    if (!t || !prediction || !loss) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::Compiled& c = t->compiled;
        if (bytes != msx_training_prediction_count(t) * 4)
            throw Fail{MSX_BAD_ARGUMENT, "the prediction is " + c.forward.node(c.prediction).ty.str() + ": " +
                                             std::to_string(msx_training_prediction_count(t) * 4) + " bytes"};
        if (!t->infer) {
            // The forward program (dropout the identity) with the model's output kept beside the
            // loss, on the run's parameter buffers.
            msx::Program program = c.forward;
            // (a function entry whose result is rank 0: the loss is the prediction already)
            if (program.outputs.empty() || program.outputs[0].value != c.prediction)
                program.outputs.push_back(msx::Output{c.prediction, msx::Role::Plain, 0, 0});
            std::string ir = msx::print_program(program);
            ok(t, msx_plan_create(t->device, ir.c_str(), c.config.seed, t->flags, t->forward, &t->infer));
        }
        ok(t, msx_sync(t->step, 0));
        gather_masked(t, c.config.steps, false);
        stage_batch(t, t->infer, input_names(t->infer));
        ok(t, msx_run(t->infer));
        ok(t, msx_loss(t->infer, loss, 0));
        ok(t, msx_value_download(t->infer, c.prediction, prediction, bytes));
    });
}

uint64_t msx_training_infer_report(msx_training* t, char* out, uint64_t capacity) {
    if (!t) return 0;
    std::string text;
    std::vector<float> prediction(msx_training_prediction_count(t));
    float loss = 0.0f;
    if (msx_training_infer(t, prediction.data(), prediction.size() * 4, &loss) != MSX_OK) return 0;
    // `prediction: <type> = [v, ...]` and `loss <v>`, floats as Rust's Display prints them
    // (crates/modelspec-cli/src/infer.rs:251-262).
    text = "prediction: " + t->compiled.forward.node(t->compiled.prediction).ty.str() + " = [";
    for (size_t i = 0; i < prediction.size(); ++i) {
        if (i) text += ", ";
        text += msx::f32_display(prediction[i]);
    }
    text += "]\nloss " + msx::f32_display(loss) + "\n";
    if (out && capacity) {
        size_t n = std::min<size_t>(capacity - 1, text.size());
        std::memcpy(out, text.data(), n);
        out[n] = 0;
    }
    return text.size() + 1;
}

// ---- held-out evaluation (crates/modelspec-runtime/src/train/eval.rs:167-355) ---------------------

namespace {

// The steps the prediction is computed from, without the loss sum (stepwise.rs:32-35), on the
// run's parameter buffers, and the device reduction of its logits for `batches` batches of `rows`
// rows (eval.rs:143-163: the prediction is f32 logits [rows, V], one row per position).
void heldout_declare(msx_training* t, uint32_t batches, uint64_t rows) {
    const msx::Compiled& c = t->compiled;
    if (t->heldout) throw Fail{MSX_BAD_ARGUMENT, "the held-out batches of this run are already declared"};
    if (batches == 0) throw Fail{MSX_BAD_ARGUMENT, "a held-out split of no batch"};
    const msx::Type& ty = c.forward.node(c.prediction).ty;
    if (ty.i32 || ty.rank() != 2 || ty.shape[0] != rows || ty.shape[1] == 0)
        throw Fail{MSX_BAD_ARGUMENT, "--eval-every reads the prediction as f32 logits [" + std::to_string(rows) +
                                         ", V], one row per position of the batch; the model's prediction is " + ty.str()};
    msx::Program program = c.forward;
    program.outputs = {msx::Output{c.prediction, msx::Role::Plain, 0, 0}};
    program = msx::dce(std::move(program));
    std::string ir = msx::print_program(program);
    ok(t, msx_plan_create(t->device, ir.c_str(), c.config.seed, t->flags, t->forward, &t->predict));
    t->predict_inputs = input_names(t->predict);
    ok(t, msx_heldout_create(t->predict, c.prediction, batches, &t->heldout));
    t->heldout_batches.assign(batches, {});
    t->heldout_row_weights.assign(batches, {});
}

void heldout_targets(msx_training* t, uint32_t batch, const int32_t* labels, const float* weights, uint64_t rows) {
    ok(t, msx_heldout_targets(t->heldout, batch, labels, weights, rows));
    t->heldout_row_weights[batch].assign(weights, weights + rows);
}

}  // namespace

int msx_training_heldout_begin(msx_training* t, uint32_t batches, const char* labels, const char* weights) {
    if (!t || !labels || !weights) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::DataDecl *l = declared(t, labels), *w = declared(t, weights);
        if (!l || !l->ty.i32 || !w || w->ty.i32 || l->ty.count() != w->ty.count())
            throw Fail{MSX_BAD_ARGUMENT, std::string("`") + labels + "` and `" + weights + "` are not declared i32 labels and f32 weights of one row each"};
        heldout_declare(t, batches, l->ty.count());
        t->heldout_labels = labels;
        t->heldout_weights = weights;
    });
}

int msx_training_heldout_set(msx_training* t, uint32_t batch, const char* name, const void* host, uint64_t bytes) {
    if (!t || !name || !host) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        if (!t->heldout) throw Fail{MSX_BAD_ARGUMENT, "no held-out batches are declared"};
        if (batch >= t->heldout_batches.size())
            throw Fail{MSX_BAD_ARGUMENT, "held-out batch " + std::to_string(batch) + " of " + std::to_string(t->heldout_batches.size())};
        const msx::DataDecl* d = declared(t, name);
        if (!d) throw Fail{MSX_BAD_ARGUMENT, std::string("the train block declares no `") + name + "`"};
        if (bytes != d->ty.count() * 4)
            throw Fail{MSX_BAD_ARGUMENT, std::string("`") + name + "` is " + d->ty.str() + ": " + std::to_string(d->ty.count() * 4) + " bytes"};
        const char* b = static_cast<const char*>(host);
        auto& held = t->heldout_batches[batch];
        held[name].assign(b, b + bytes);
        // Both targets of a batch given: they go to the device, where they stay.
        auto l = held.find(t->heldout_labels), w = held.find(t->heldout_weights);
        if ((name == t->heldout_labels || name == t->heldout_weights) && l != held.end() && w != held.end())
            heldout_targets(t, batch, reinterpret_cast<const int32_t*>(l->second.data()), reinterpret_cast<const float*>(w->second.data()),
                            l->second.size() / 4);
    });
}

int msx_training_heldout_evaluate(msx_training* t, float* loss, float* accuracy) {
    if (!t || !loss || !accuracy) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        if (!t->heldout) throw Fail{MSX_BAD_ARGUMENT, "no held-out batches are declared"};
        // The prediction plan runs on its own stream: the submitted updates first.
        ok(t, msx_sync(t->step, 0));
        ok(t, msx_heldout_begin(t->heldout));
        // HeldOut::metrics_of_sums (eval.rs:325-355): the denominator and the selected rows are the
        // split's own weights, summed from the first term in batch and row order.
        bool any = false;
        double denominator = 0.0;
        uint64_t selected = 0;
        for (uint32_t b = 0; b < t->heldout_batches.size(); ++b) {
            const auto& held = t->heldout_batches[b];
            for (const std::string& name : t->predict_inputs) {
                auto it = held.find(name);
                if (it == held.end()) throw Fail{MSX_BAD_INPUT, "held-out batch " + std::to_string(b) + " holds no `" + name + "`"};
                ok(t, msx_set_input(t->predict, name.c_str(), it->second.data(), it->second.size()));
            }
            const std::vector<float>& weights = t->heldout_row_weights[b];
            if (weights.empty()) throw Fail{MSX_BAD_INPUT, "held-out batch " + std::to_string(b) + " holds no labels and weights"};
            ok(t, msx_run(t->predict));
            ok(t, msx_heldout_add(t->heldout, b));
            for (float weight : weights) {
                const double wide = static_cast<double>(weight);
                denominator = any ? denominator + wide : wide;
                any = true;
                if (weight > 0.0f) ++selected;
            }
        }
        double numerator = 0.0;
        uint64_t correct = 0;
        ok(t, msx_heldout_sums(t->heldout, &numerator, &correct, 0));
        *loss = denominator == 0.0 ? 0.0f : static_cast<float>(numerator / denominator);
        *accuracy = selected == 0 ? 0.0f : static_cast<float>(correct) / static_cast<float>(selected);
    });
}

// ---- packed --data (crates/modelspec-runtime/src/train/data.rs:1485-1760) ------------------------

namespace {

const char* const kBatchTensors[5] = {"ids", "positions", "key_mask", "labels", "weights"};
bool batch_tensor_is_i32(const std::string& name) { return name == "ids" || name == "positions" || name == "labels"; }
std::string batch_tensor_names() { return "ids, positions, key_mask, labels, weights"; }

// Draws batch `step` of a split as the declared tensors hold it, by declaration name.
void draw_packed(msx_training* t, int split, uint64_t step, std::map<std::string, std::vector<char>>* out, std::vector<int32_t>* labels,
                 std::vector<float>* weights) {
    const uint64_t rows = t->packed_batch * msx_packed_seq_len(t->packed);
    std::vector<int32_t> ids(rows), positions(rows);
    std::vector<float> key_mask(rows);
    labels->resize(rows);
    weights->resize(rows);
    if (msx_packed_batch(t->packed, split, t->compiled.config.seed, step, t->packed_batch, ids.data(), positions.data(), key_mask.data(),
                         labels->data(), weights->data()) != MSX_OK)
        throw Fail{MSX_BAD_INPUT, std::string(msx_packed_last_error(t->packed))};
    for (const std::string& name : t->packed_bound) {
        const void* from = name == "ids" ? static_cast<const void*>(ids.data())
                           : name == "positions" ? static_cast<const void*>(positions.data())
                           : name == "key_mask" ? static_cast<const void*>(key_mask.data())
                           : name == "labels" ? static_cast<const void*>(labels->data())
                                              : static_cast<const void*>(weights->data());
        const char* b = static_cast<const char*>(from);
        (*out)[name].assign(b, b + rows * 4);
    }
}

}  // namespace

int msx_training_bind_packed(msx_training* t, msx_packed* packed) {
    if (!t || !packed) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::Compiled& c = t->compiled;
        const uint64_t seq_len = msx_packed_seq_len(packed), vocabulary = msx_packed_vocabulary(packed);
        const auto& decls = c.config.data;  // in source order
        // bind (data.rs:1630-1745), its refusals in the reference's order.
        if (decls.empty()) throw Fail{MSX_BAD_INPUT, "E-DATA-005: a run on a packed directory declares no batch tensor (" + batch_tensor_names() + ")"};
        for (const msx::DataDecl& d : decls)
            if (std::find_if(std::begin(kBatchTensors), std::end(kBatchTensors), [&](const char* n) { return d.name == n; }) == std::end(kBatchTensors))
                throw Fail{MSX_BAD_INPUT, std::string("E-DATA-005: the ") + (d.target ? "target" : "input") + " `" + d.name +
                                              "` names no tensor of the masked-language-model batch (" + batch_tensor_names() + ")"};
        const msx::DataDecl* first = nullptr;
        for (const char* name : kBatchTensors) {
            for (const msx::DataDecl& d : decls)
                if (!first && d.name == name) first = &d;
        }
        auto type_text = [&](const std::string& name, const std::string& shape) {
            return std::string("Tensor<") + (batch_tensor_is_i32(name) ? "i32" : "f32") + ", [" + shape + "]>";
        };
        auto mismatch = [&](const msx::DataDecl& d, const std::string& expected) {
            return Fail{MSX_BAD_INPUT, std::string("E-DATA-006: the ") + (d.target ? "target" : "input") + " `" + d.name +
                                           "` is not of the type of the batch tensor `" + d.name + "`: it is " + d.ty.str() + ", expected " + expected};
        };
        uint64_t batch = 0;
        const auto& shape = first->ty.shape;
        const bool positive = std::all_of(shape.begin(), shape.end(), [](uint64_t n) { return n > 0; });
        if (positive && shape.size() == 2 && shape[1] == seq_len) batch = shape[0];
        else if (positive && shape.size() == 1 && shape[0] % seq_len == 0) batch = shape[0] / seq_len;
        if (batch == 0)
            throw mismatch(*first, type_text(first->name, "B, " + std::to_string(seq_len)) + " or " + type_text(first->name, "B·" + std::to_string(seq_len)));
        const uint64_t rows = batch * seq_len;
        for (const msx::DataDecl& d : decls) {
            const bool fits = d.ty.i32 == batch_tensor_is_i32(d.name) &&
                              ((d.ty.shape.size() == 2 && d.ty.shape[0] == batch && d.ty.shape[1] == seq_len) ||
                               (d.ty.shape.size() == 1 && d.ty.shape[0] == rows));
            if (!fits)
                throw mismatch(d, type_text(d.name, std::to_string(batch) + ", " + std::to_string(seq_len)) + " or " + type_text(d.name, std::to_string(rows)));
        }
        // refuse_unread (data.rs:307-338): every declaration has an Input node of the forward program.
        const msx::Program& fwd = c.forward_with_dropout;
        auto input_of = [&](const std::string& name) -> int64_t {
            for (uint32_t in : fwd.inputs)
                if (fwd.node(in).name == name) return in;
            return -1;
        };
        for (const msx::DataDecl& d : decls)
            if (input_of(d.name) < 0)
                throw Fail{MSX_BAD_INPUT, std::string("E-DATA-003: the ") + (d.target ? "target" : "input") + " `" + d.name + "` is not read by the loss"};
        // refuse_vocabulary (data.rs:1760-1840): the widths the packed vocabulary fixes.
        const int64_t ids = input_of("ids"), labels = input_of("labels");
        for (const msx::Node& n : fwd.nodes) {
            const bool table = n.op == msx::Op::Embedding && ids >= 0 && n.operands.size() > 1 && n.operands[1] == static_cast<uint32_t>(ids);
            const bool logits = n.op == msx::Op::CrossEntropy && labels >= 0 && n.operands.size() > 1 && n.operands[1] == static_cast<uint32_t>(labels);
            if (!table && !logits) continue;
            const msx::Node& value = fwd.node(n.operands[0]);
            const size_t axis = table ? 0 : 1;
            if (value.ty.shape.size() <= axis || value.ty.shape[axis] == vocabulary) continue;
            std::string named = "%" + std::to_string(value.id);
            if (value.op == msx::Op::ParamRead) named = fwd.params[value.param].path;
            throw Fail{MSX_BAD_INPUT, std::string("E-DATA-006: the ") + (table ? "table" : "logits") + " `" + named + "` of the `" +
                                          (table ? "embedding" : "cross_entropy") + "` that reads `" + (table ? "ids" : "labels") + "` has " +
                                          std::to_string(value.ty.shape[axis]) + (table ? " rows" : " classes") + ", not the " + std::to_string(vocabulary) +
                                          " tokens of the packed vocabulary"};
        }
        const uint64_t sequences = msx_packed_sequences(packed, MSX_SPLIT_TRAIN);
        if (batch > sequences)
            throw Fail{MSX_BAD_INPUT, "a batch of " + std::to_string(batch) + " sequences, more than the " + std::to_string(sequences) + " of the Train split"};
        t->packed = packed;
        t->packed_batch = batch;
        t->packed_bound.clear();
        for (const msx::DataDecl& d : decls) t->packed_bound.push_back(d.name);
    });
}

int msx_training_feed_packed(msx_training* t, uint64_t step) {
    if (!t) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        if (!t->packed) throw Fail{MSX_BAD_ARGUMENT, "no packed directory is bound"};
        std::vector<int32_t> labels;
        std::vector<float> weights;
        draw_packed(t, MSX_SPLIT_TRAIN, step, &t->batch, &labels, &weights);
    });
}

int msx_training_heldout_packed(msx_training* t, const char* dir_for_messages) {
    if (!t) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        if (!t->packed) throw Fail{MSX_BAD_ARGUMENT, "no packed directory is bound"};
        // HeldOut::new (eval.rs:167-199): the batches b = 0 .. n / B of the split, drawn once.
        const uint64_t sequences = msx_packed_sequences(t->packed, MSX_SPLIT_HELDOUT);
        if (sequences < t->packed_batch)
            throw Fail{MSX_BAD_INPUT, std::string("the HeldOut split of ") + (dir_for_messages ? dir_for_messages : "the packed directory") + " holds " +
                                          std::to_string(sequences) + " sequences, fewer than the batch of " + std::to_string(t->packed_batch) +
                                          " that --eval-every evaluates"};
        const uint64_t batches = sequences / t->packed_batch;
        if (batches > 0xffffffffull) throw Fail{MSX_BAD_INPUT, "too many held-out batches"};
        heldout_declare(t, static_cast<uint32_t>(batches), t->packed_batch * msx_packed_seq_len(t->packed));
        for (uint32_t b = 0; b < batches; ++b) {
            std::vector<int32_t> labels;
            std::vector<float> weights;
            draw_packed(t, MSX_SPLIT_HELDOUT, b, &t->heldout_batches[b], &labels, &weights);
            heldout_targets(t, b, labels.data(), weights.data(), labels.size());
        }
    });
}

uint32_t msx_training_heldout_batches(const msx_training* t) { return t ? static_cast<uint32_t>(t->heldout_batches.size()) : 0; }

// ---- dense data (crates/modelspec-runtime/src/train/data.rs:513-577, :627-671) ---------------------

namespace {

// The Input node of `program` that reads the declaration `name`, or -1.
int64_t input_named(const msx::Program& program, const std::string& name) {
    for (uint32_t in : program.inputs)
        if (program.node(in).name == name) return in;
    return -1;
}

// What read_dense refuses before it opens a file (data.rs:627-668), in its order: the one target
// the loss compares with the model output has the output's type (E-DATA-002), unless it is i32
// labels a cross_entropy reads or the loss is the value the forward call returns; every
// declaration is read by the loss (E-DATA-003, refuse_unread :307-338).
void refuse_dense_declarations(const msx::Compiled& c) {
    const auto& decls = c.config.data;  // in source order
    const msx::Program& fwd = c.forward_with_dropout;
    const msx::DataDecl* target = nullptr;
    uint32_t targets = 0;
    for (const msx::DataDecl& d : decls)
        if (d.target) {
            target = &d;
            ++targets;
        }
    const bool forward_value = !c.forward.outputs.empty() && c.forward.outputs[0].value == c.forward.node(c.prediction).id;
    if (targets == 1 && !forward_value) {
        bool labels = false;
        const int64_t input = input_named(fwd, target->name);
        if (target->ty.i32 && input >= 0)
            for (const msx::Node& n : fwd.nodes)
                if (n.op == msx::Op::CrossEntropy && n.operands.size() >= 2 && n.operands[1] == static_cast<uint32_t>(input)) labels = true;
        const msx::Type& output = c.forward.node(c.prediction).ty;
        if (!labels && target->ty != output)
            throw Fail{MSX_BAD_INPUT, "E-DATA-002: the target is not of the model output type\n  target: " + target->ty.str() +
                                          "\n  model output: " + output.str()};
    }
    for (const msx::DataDecl& d : decls)
        if (input_named(fwd, d.name) < 0)
            throw Fail{MSX_BAD_INPUT, std::string("E-DATA-003: the ") + (d.target ? "target" : "input") + " `" + d.name + "` is not read by the loss"};
}

// index_bounds (data.rs:899-939) over the files of `dense`, opened for the declarations of `c` in
// source order: the ids of an embedding lie below the rows of its table, the labels of a
// cross_entropy below the classes of its logits; the tightest bound of a declaration is the one
// its file is held to (refuse_out_of_range :957-1004, E-DATA-011).
void check_index_bounds(const msx::Compiled& c, msx_dense* dense) {
    const auto& decls = c.config.data;
    const msx::Program& fwd = c.forward_with_dropout;
    for (uint32_t i = 0; i < decls.size(); ++i) {
        if (!decls[i].ty.i32) continue;
        const int64_t input = input_named(fwd, decls[i].name);
        uint64_t tightest = 0;
        std::string what;
        for (const msx::Node& n : fwd.nodes) {
            const bool table = n.op == msx::Op::Embedding, logits = n.op == msx::Op::CrossEntropy;
            if ((!table && !logits) || n.operands.size() < 2 || input < 0 || n.operands[1] != static_cast<uint32_t>(input)) continue;
            const msx::Node& value = fwd.node(n.operands[0]);
            const size_t axis = table ? 0 : 1;
            if (value.ty.shape.size() <= axis) continue;
            const uint64_t bound = value.ty.shape[axis];
            if (!what.empty() && bound >= tightest) continue;
            std::string named = "%" + std::to_string(value.id);
            if (value.op == msx::Op::ParamRead) named = fwd.params[value.param].path;
            tightest = bound;
            what = "the " + std::to_string(bound) + (table ? " rows of the `embedding` table `" : " classes of the `cross_entropy` logits `") + named + "`";
        }
        if (what.empty()) continue;
        if (msx_dense_check_bound(dense, i, tightest, what.c_str()) != MSX_OK) throw Fail{MSX_BAD_INPUT, msx_dense_last_error(dense)};
    }
}

// The declarations of `c` as the dense reader takes them; `role` 0 / 1 by the declaration, or 2
// for the arguments of an inference entry.
struct DenseDeclarations {
    std::vector<const char*> names;
    std::vector<uint32_t> is_i32, roles, ranks;
    std::vector<uint64_t> shapes;
    explicit DenseDeclarations(const msx::Compiled& c) {
        for (const msx::DataDecl& d : c.config.data) {
            names.push_back(d.name.c_str());
            is_i32.push_back(d.ty.i32 ? 1u : 0u);
            roles.push_back(!c.function.empty() ? 2u : d.target ? 1u : 0u);
            ranks.push_back(static_cast<uint32_t>(d.ty.shape.size()));
            for (uint64_t n : d.ty.shape) shapes.push_back(n);
        }
    }
    uint32_t count() const { return static_cast<uint32_t>(names.size()); }
};

}  // namespace

int msx_training_bind_dense(msx_training* t, const char* dir) {
    if (!t || !dir) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::Compiled& c = t->compiled;
        refuse_dense_declarations(c);
        const DenseDeclarations d(c);
        msx_dense* dense = nullptr;
        if (msx_dense_open(dir, d.count(), d.names.data(), d.is_i32.data(), d.roles.data(), d.ranks.data(), d.shapes.data(), c.config.steps, &dense) !=
            MSX_OK)
            throw Fail{MSX_BAD_INPUT, msx_dense_last_error(nullptr)};
        try {
            check_index_bounds(c, dense);
        } catch (...) {
            msx_dense_close(dense);
            throw;
        }
        if (t->dense) msx_dense_close(t->dense);
        t->dense = dense;
    });
}

int msx_training_feed_dense(msx_training* t, uint64_t step) {
    if (!t) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        if (!t->dense) throw Fail{MSX_BAD_ARGUMENT, "no dense directory is bound"};
        const auto& decls = t->compiled.config.data;
        for (uint32_t i = 0; i < decls.size(); ++i) {
            std::vector<char>& bytes = t->batch[decls[i].name];
            bytes.resize(msx_dense_batch_bytes(t->dense, i));
            if (msx_dense_step(t->dense, i, step, bytes.data(), bytes.size()) != MSX_OK) throw Fail{MSX_BAD_ARGUMENT, "the dense batch does not fit its declaration"};
        }
    });
}

int msx_training_eval_dense(msx_training* t, const char* dir, double* loss, double* accuracy, int* has_accuracy) {
    if (!t || !dir || !loss || !accuracy || !has_accuracy) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::Compiled& c = t->compiled;
        const auto& decls = c.config.data;
        refuse_dense_declarations(c);
        const DenseDeclarations d(c);
        msx_dense* data = nullptr;
        if (msx_dense_open_eval(dir, d.count(), d.names.data(), d.is_i32.data(), d.roles.data(), d.ranks.data(), d.shapes.data(), &data) != MSX_OK)
            throw Fail{MSX_BAD_INPUT, msx_dense_last_error(nullptr)};
        std::unique_ptr<msx_dense, void (*)(msx_dense*)> owned(data, msx_dense_close);
        // compared_target (data.rs:419-425, read_dense :640-655): the one target, when it is f32 and
        // the loss is not the value the forward call returns.
        int compared = -1;
        uint32_t targets = 0;
        for (uint32_t i = 0; i < decls.size(); ++i)
            if (decls[i].target) {
                ++targets;
                compared = static_cast<int>(i);
            }
        const bool forward_value = !c.forward.outputs.empty() && c.forward.outputs[0].value == c.forward.node(c.prediction).id;
        if (targets != 1 || forward_value || decls[static_cast<size_t>(compared)].ty.i32) compared = -1;
        const uint64_t batches = msx_dense_samples(data) / msx_dense_batch(data);
        std::vector<float> prediction(msx_training_prediction_count(t));
        double sum = 0.0;
        uint64_t correct = 0, rows = 0;
        auto argmax = [](const float* row, uint64_t width, uint64_t* at) {
            for (uint64_t i = 0; i < width; ++i)
                if (row[i] != row[i]) return false;
            uint64_t best = 0;
            for (uint64_t i = 1; i < width; ++i)
                if (row[i] > row[best]) best = i;
            *at = best;
            return true;
        };
        for (uint64_t b = 0; b < batches; ++b) {
            for (uint32_t i = 0; i < decls.size(); ++i) {
                std::vector<char>& bytes = t->batch[decls[i].name];
                bytes.resize(msx_dense_batch_bytes(data, i));
                if (msx_dense_eval_batch(data, i, b, bytes.data(), bytes.size()) != MSX_OK) throw Fail{MSX_BAD_ARGUMENT, "the eval batch does not fit its declaration"};
            }
            float batch_loss = 0.0f;
            if (msx_training_infer(t, prediction.data(), prediction.size() * 4, &batch_loss) != MSX_OK) throw Fail{MSX_LAUNCH_FAILED, t->error};
            sum += static_cast<double>(batch_loss);
            if (compared < 0) continue;
            // correct_rows (runner.rs:626-636): rows along the target's leading dimension.
            const msx::DataDecl& target = decls[static_cast<size_t>(compared)];
            const std::vector<char>& held = t->batch[target.name];
            const float* wanted = reinterpret_cast<const float*>(held.data());
            const uint64_t count = held.size() / 4, target_rows = target.ty.shape.empty() ? 1 : target.ty.shape[0];
            const uint64_t width = target_rows ? count / target_rows : 0;
            for (uint64_t r = 0; r < target_rows && width; ++r) {
                uint64_t p = 0, w = 0;
                if (argmax(prediction.data() + r * width, width, &p) && argmax(wanted + r * width, width, &w) && p == w) ++correct;
            }
            rows += target_rows;
        }
        *loss = sum / static_cast<double>(batches);
        *has_accuracy = compared >= 0 ? 1 : 0;
        *accuracy = compared >= 0 ? static_cast<double>(correct) / static_cast<double>(rows) : 0.0;
    });
}

// ---- a model function over a dense directory (cli/src/infer.rs:306-470; train/data.rs:676-815) ----

namespace {

std::string listed_functions(const msx::Compiled& c) {
    std::string out;
    for (const std::string& f : c.functions) out += (out.empty() ? "" : ", ") + f;
    return out;
}

// `path` made canonical, or when it does not exist its canonical parent joined with its name
// (resolved, data.rs:800-815); empty when neither resolves.
std::string resolved(const std::string& path) {
    char buffer[PATH_MAX];
    if (realpath(path.c_str(), buffer)) return buffer;
    const size_t slash = path.find_last_of('/');
    const std::string parent = slash == std::string::npos ? "." : slash == 0 ? "/" : path.substr(0, slash);
    const std::string name = slash == std::string::npos ? path : path.substr(slash + 1);
    if (name.empty() || name == "." || name == "..") return "";
    if (!realpath(parent.c_str(), buffer)) return "";
    return std::string(buffer) + (std::string(buffer) == "/" ? "" : "/") + name;
}

bool same_file(const std::string& a, const std::string& b) {
    struct stat sa, sb;
    return stat(a.c_str(), &sa) == 0 && stat(b.c_str(), &sb) == 0 && sa.st_dev == sb.st_dev && sa.st_ino == sb.st_ino;
}

// replace (cli/src/infer.rs:455-490): the bytes go to `.<name>.<pid>.tmp` beside `out`, are synced
// and renamed over it; on an error the temporary file is removed and `out` keeps its bytes.
void replace_file(const std::string& out, const void* bytes, size_t size) {
    const size_t slash = out.find_last_of('/');
    const std::string dir = slash == std::string::npos ? "." : slash == 0 ? "/" : out.substr(0, slash);
    const std::string name = slash == std::string::npos ? out : out.substr(slash + 1);
    if (name.empty()) throw Fail{MSX_BAD_ARGUMENT, "cannot write " + out + ": the path names no file"};
    const std::string temporary = dir + "/." + name + "." + std::to_string(getpid()) + ".tmp";
    auto failed = [&](const char* what) {
        const std::string why = std::strerror(errno);
        unlink(temporary.c_str());
        return Fail{MSX_BAD_INPUT, "cannot write " + out + ": " + what + ": " + why};
    };
    const int fd = open(temporary.c_str(), O_WRONLY | O_CREAT | O_EXCL, 0644);
    if (fd < 0) throw Fail{MSX_BAD_INPUT, "cannot write " + out + ": " + temporary + ": " + std::strerror(errno)};
    const char* at = static_cast<const char*>(bytes);
    size_t left = size;
    while (left > 0) {
        const ssize_t wrote = write(fd, at, left);
        if (wrote < 0) {
            if (errno == EINTR) continue;
            const Fail f = failed("write");
            close(fd);
            throw f;
        }
        at += wrote;
        left -= static_cast<size_t>(wrote);
    }
    if (fsync(fd) != 0) {
        const Fail f = failed("sync");
        close(fd);
        throw f;
    }
    close(fd);
    if (rename(temporary.c_str(), out.c_str()) != 0) throw failed("rename");
}

}  // namespace

// refuse_out_reading (data.rs:773-798): `--out` resolves to a file the run reads.
int msx_training_refuse_out_reading(msx_training* t, const char* dir, const char* out, const char* model, const char* checkpoint) {
    if (!t || !dir || !out) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        std::vector<std::pair<std::string, std::string>> reads;
        if (model) reads.push_back({"model", model});
        if (checkpoint) reads.push_back({"checkpoint", checkpoint});
        for (const msx::DataDecl& d : t->compiled.config.data)
            reads.push_back({"argument `" + d.name + "`", std::string(dir) + "/" + d.name + (d.ty.i32 ? ".i32" : ".f32")});
        const std::string target = resolved(out);
        if (target.empty()) return;
        for (const auto& [what, file] : reads)
            if (resolved(file) == target || same_file(out, file))
                throw Fail{MSX_BAD_INPUT, std::string("E-DATA-010: `--out` names a file the run reads\n  --out: ") + out + "\n  " + what + ": " + file};
    });
}

int msx_training_infer_dense(msx_training* t, const char* dir, const char* out, uint64_t* blocks, uint64_t* rows) {
    if (!t || !dir || !out || !blocks || !rows) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::Compiled& c = t->compiled;
        if (c.function.empty()) throw Fail{MSX_BAD_ARGUMENT, "this run is the train block's, not a model function's (msx_training_create_function)"};
        // dense_function (data.rs:685-717).
        if (c.config.data.empty())
            throw Fail{MSX_BAD_INPUT, "E-DATA-010: the function `" + c.function + "` takes no argument a data file could bind\n  function: " + c.function +
                                          "\n  functions: " + listed_functions(c)};
        const DenseDeclarations d(c);
        msx_dense* data = nullptr;
        if (msx_dense_open_eval(dir, d.count(), d.names.data(), d.is_i32.data(), d.roles.data(), d.ranks.data(), d.shapes.data(), &data) != MSX_OK)
            throw Fail{MSX_BAD_INPUT, msx_dense_last_error(nullptr)};
        std::unique_ptr<msx_dense, void (*)(msx_dense*)> owned(data, msx_dense_close);
        check_index_bounds(c, data);
        // row_elements (data.rs:732-762): one row per sample of a block of B samples.
        const msx::Type& result = c.forward.node(c.prediction).ty;
        const uint64_t batch = msx_dense_batch(data), samples = msx_dense_samples(data);
        if (result.i32) throw Fail{MSX_UNSUPPORTED, "the result of the function `" + c.function + "` is " + result.str() + ", not f32"};
        if (batch != 1 && (result.shape.empty() || result.shape[0] != batch))
            throw Fail{MSX_BAD_INPUT, "E-DATA-010: the result of the function `" + c.function + "` is not one row per sample\n  function: " + c.function +
                                          "\n  result: " + result.str() + "\n  batch: " + std::to_string(batch) + "\n  functions: " + listed_functions(c)};
        const uint64_t per_block = result.count(), count = samples / batch;
        std::vector<float> values(static_cast<size_t>(per_block * count));
        for (uint64_t b = 0; b < count; ++b) {
            for (uint32_t i = 0; i < d.count(); ++i) {
                std::vector<char>& bytes = t->batch[c.config.data[i].name];
                bytes.resize(msx_dense_batch_bytes(data, i));
                if (msx_dense_eval_batch(data, i, b, bytes.data(), bytes.size()) != MSX_OK) throw Fail{MSX_BAD_ARGUMENT, "the block does not fit its argument"};
            }
            float loss = 0.0f;
            if (msx_training_infer(t, values.data() + b * per_block, per_block * 4, &loss) != MSX_OK) throw Fail{MSX_LAUNCH_FAILED, t->error};
        }
        replace_file(out, values.data(), values.size() * 4);
        *blocks = count;
        *rows = samples;
    });
}

uint64_t msx_training_eval_line(double loss, double accuracy, int has_accuracy, char* out, uint64_t capacity) {
    std::string text = "eval loss=" + msx::f64_display(loss);
    if (has_accuracy) text += " accuracy=" + msx::f64_display(accuracy);
    text += "\n";
    if (out && capacity) {
        const size_t n = std::min<size_t>(capacity - 1, text.size());
        std::memcpy(out, text.data(), n);
        out[n] = 0;
    }
    return text.size() + 1;
}

// ---- checkpoints (crates/modelspec-runtime/src/train/checkpoint.rs:420-451, :519-609) --------------

namespace {

// OptimizerConfig::of (checkpoint.rs:114-152): the f32 hyperparameters widened to f64.
void optimizer_of(const msx_training* t, int* kind, double v[5], uint64_t* warmup) {
    const msx::TrainConfig& c = t->compiled.config;
    *kind = c.rule == msx::Rule::AdamW ? MSX_OPTIMIZER_ADAMW : MSX_OPTIMIZER_SGD;
    v[0] = static_cast<double>(c.lr);
    v[1] = static_cast<double>(c.adamw.weight_decay);
    v[2] = static_cast<double>(c.adamw.beta1);
    v[3] = static_cast<double>(c.adamw.beta2);
    v[4] = static_cast<double>(c.adamw.eps);
    *warmup = c.adamw.warmup_steps;
}

std::string shape_text(const std::vector<uint64_t>& shape) {
    std::string s = "[";
    for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
    return s + "]";
}

}  // namespace

const char* msx_training_schema_hash(msx_training* t) {
    if (!t) return "";
    if (t->schema.empty()) t->schema = msx::schema_hash(t->compiled.step.params);
    return t->schema.c_str();
}

int msx_training_checkpoint(msx_training* t, uint64_t step, msx_checkpoint** out) {
    if (!t || !out) return MSX_BAD_ARGUMENT;
    *out = nullptr;
    return guarded(t, [&] {
        const msx::Compiled& c = t->compiled;
        ok(t, msx_sync(t->step, 0));
        msx_checkpoint* ckpt = nullptr;
        if (msx_checkpoint_new(step, c.config.seed, msx_training_schema_hash(t), &ckpt) != MSX_OK) throw Fail{MSX_UNSUPPORTED, "no checkpoint"};
        std::unique_ptr<msx_checkpoint, void (*)(msx_checkpoint*)> holder(ckpt, msx_checkpoint_destroy);
        int kind;
        double v[5];
        uint64_t warmup;
        optimizer_of(t, &kind, v, &warmup);
        msx_checkpoint_set_optimizer(ckpt, kind, v[0], v[1], v[2], v[3], v[4], warmup);
        auto add = [&](const msx::Param& p, const char* slot, const std::vector<float>& value) {
            if (msx_checkpoint_add(ckpt, p.path.c_str(), slot, p.ty.shape.data(), static_cast<uint32_t>(p.ty.shape.size()), value.data()) != MSX_OK)
                throw Fail{MSX_BAD_ARGUMENT, std::string("cannot write checkpoint: ") + msx_checkpoint_last_error(ckpt)};
        };
        const auto& params = c.forward.params;
        std::vector<float> value;
        for (uint32_t p = 0; p < params.size(); ++p) {
            value.resize(params[p].ty.count());
            // The forward plan holds every parameter the prediction or the loss reads (the step's own
            // buffers, shared); one that neither reads has no value to record.
            if (msx_param_download(t->forward, p, value.data(), value.size() * 4) != MSX_OK &&
                msx_param_download(t->step, p, value.data(), value.size() * 4) != MSX_OK)
                continue;
            add(params[p], nullptr, value);
            if (kind != MSX_OPTIMIZER_ADAMW) continue;
            for (char which : {'m', 'v'}) {
                if (msx_moment_download(t->step, p, which, value.data(), value.size() * 4) != MSX_OK) continue;
                const char slot[2] = {which, 0};
                add(params[p], slot, value);
            }
        }
        *out = holder.release();
    });
}

namespace {

Fail mismatch(const std::string& what) { return Fail{MSX_BAD_INPUT, "E-CKPT-003: the checkpoint does not match the compiled file: " + what}; }

// parameters_for (checkpoint.rs:519-585): both sides in path order, the first difference named,
// then the schema hash. Returns the run's parameters in path order.
std::vector<uint32_t> matched_parameters(msx_training* t, const msx_checkpoint* ckpt) {
    const msx::Compiled& c = t->compiled;
    std::vector<uint32_t> ours(c.forward.params.size());
    for (uint32_t p = 0; p < ours.size(); ++p) ours[p] = p;
    std::sort(ours.begin(), ours.end(), [&](uint32_t a, uint32_t b) { return c.forward.params[a].path < c.forward.params[b].path; });
    const uint32_t theirs = msx_checkpoint_count(ckpt, 0);
    for (uint32_t i = 0; i < std::max<uint32_t>(theirs, static_cast<uint32_t>(ours.size())); ++i) {
        const std::string their_path = i < theirs ? std::string("`") + msx_checkpoint_path(ckpt, 0, i) + "`" : "none";
        const std::string our_path = i < ours.size() ? "`" + c.forward.params[ours[i]].path + "`" : "none";
        if (their_path != our_path) throw mismatch("a parameter path differs (checkpoint " + their_path + ", compiled file " + our_path + ")");
        const msx::Param& p = c.forward.params[ours[i]];
        if (p.ty.i32) throw mismatch("parameter `" + p.path + "` has dtype f32 in the checkpoint and i32 in the compiled file");
        const uint64_t* shape = msx_checkpoint_shape(ckpt, 0, i);
        std::vector<uint64_t> their_shape(shape, shape + msx_checkpoint_rank(ckpt, 0, i));
        if (their_shape != p.ty.shape)
            throw mismatch("parameter `" + p.path + "` has another shape (checkpoint " + shape_text(their_shape) + ", compiled file " + p.ty.str() + ")");
    }
    if (std::string(msx_checkpoint_schema_hash(ckpt)) != msx_training_schema_hash(t))
        throw mismatch(std::string("the schema hash differs (checkpoint ") + msx_checkpoint_schema_hash(ckpt) + ", compiled file " + t->schema + ")");
    return ours;
}

}  // namespace

// The parameters of a checkpoint without its optimizer (`infer`: Checkpoint::parameters_for,
// checkpoint.rs:519-585; cli/src/infer.rs:361-363).
int msx_training_load_parameters(msx_training* t, const msx_checkpoint* ckpt, uint64_t* step) {
    if (!t || !ckpt) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::Compiled& c = t->compiled;
        const std::vector<uint32_t> ours = matched_parameters(t, ckpt);
        ok(t, msx_sync(t->step, 0));
        for (uint32_t i = 0; i < ours.size(); ++i) {
            const uint64_t bytes = c.forward.params[ours[i]].ty.count() * 4;
            int rs = msx_param_upload(t->step, ours[i], msx_checkpoint_data(ckpt, 0, i), bytes);
            int rf = msx_param_upload(t->forward, ours[i], msx_checkpoint_data(ckpt, 0, i), bytes);
            (void)rs;
            (void)rf;  // a parameter neither program reads has no buffer
        }
        if (step) *step = msx_checkpoint_step(ckpt);
    });
}

int msx_training_resume(msx_training* t, const msx_checkpoint* ckpt, uint64_t* start_step) {
    if (!t || !ckpt || !start_step) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::Compiled& c = t->compiled;
        const std::vector<uint32_t> ours = matched_parameters(t, ckpt);
        // resume_into (checkpoint.rs:587-609): the optimizer is that of the compiled file.
        int kind, their_kind;
        double v[5], w[5];
        uint64_t warmup, their_warmup;
        optimizer_of(t, &kind, v, &warmup);
        msx_checkpoint_optimizer(ckpt, &their_kind, &w[0], &w[1], &w[2], &w[3], &w[4], &their_warmup);
        bool same = kind == their_kind && v[0] == w[0];
        if (same && kind == MSX_OPTIMIZER_ADAMW) same = v[1] == w[1] && v[2] == w[2] && v[3] == w[3] && v[4] == w[4] && warmup == their_warmup;
        if (!same) {
            std::vector<char> text(msx_checkpoint_optimizer_json(ckpt, nullptr, 0));
            msx_checkpoint_optimizer_json(ckpt, text.data(), text.size());
            throw mismatch(std::string("the optimizer differs (checkpoint ") + text.data() + ")");
        }
        // The moments of an AdamW run: both of every parameter the step updates, or a step-0
        // checkpoint, whose moments are zero.
        const uint64_t step = msx_checkpoint_step(ckpt);
        std::map<std::pair<std::string, std::string>, uint32_t> slots;
        for (uint32_t i = 0; i < msx_checkpoint_count(ckpt, 1); ++i) slots[{msx_checkpoint_path(ckpt, 1, i), msx_checkpoint_slot(ckpt, 1, i)}] = i;
        ok(t, msx_sync(t->step, 0));
        for (uint32_t i = 0; i < ours.size(); ++i) {
            const uint32_t p = ours[i];
            const msx::Param& param = c.forward.params[p];
            const uint64_t bytes = param.ty.count() * 4;
            int rs = msx_param_upload(t->step, p, msx_checkpoint_data(ckpt, 0, i), bytes);
            int rf = msx_param_upload(t->forward, p, msx_checkpoint_data(ckpt, 0, i), bytes);
            if (rs != MSX_OK && rf != MSX_OK) continue;  // a parameter neither program reads
            if (kind != MSX_OPTIMIZER_ADAMW) continue;
            for (char which : {'m', 'v'}) {
                auto it = slots.find({param.path, std::string(1, which)});
                std::vector<float> zeros;
                const float* data = nullptr;
                if (it != slots.end()) {
                    const uint64_t* shape = msx_checkpoint_shape(ckpt, 1, it->second);
                    std::vector<uint64_t> their_shape(shape, shape + msx_checkpoint_rank(ckpt, 1, it->second));
                    if (their_shape != param.ty.shape) throw mismatch("slot `" + std::string(1, which) + "` of `" + param.path + "` has another shape");
                    data = msx_checkpoint_data(ckpt, 1, it->second);
                } else if (step == 0) {
                    zeros.assign(param.ty.count(), 0.0f);
                    data = zeros.data();
                } else {
                    throw Fail{MSX_BAD_INPUT, "the checkpoint of step " + std::to_string(step) + " holds no first and second moments of `" + param.path +
                                                  "`; an `adamw` run resumes only from a checkpoint that holds them, or from step 0"};
                }
                int rc = msx_moment_upload(t->step, p, which, data, bytes);
                (void)rc;  // a parameter the step does not update has no moments
            }
        }
        *start_step = step;
    });
}

// ---- a whole run (crates/modelspec-cli/src/train.rs:1494-1560; train/runner.rs:365-512) ---------------

namespace {

// `<label> @<path>: <type> = [v, ...]` for every parameter the run holds, in path order.
void parameter_lines(msx_training* t, const char* label, std::string* out) {
    const auto& params = t->compiled.forward.params;
    std::vector<uint32_t> order(params.size());
    for (uint32_t p = 0; p < order.size(); ++p) order[p] = p;
    std::sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return params[a].path < params[b].path; });
    std::vector<float> value;
    for (uint32_t p : order) {
        value.resize(params[p].ty.count());
        if (msx_param_download(t->forward, p, value.data(), value.size() * 4) != MSX_OK &&
            msx_param_download(t->step, p, value.data(), value.size() * 4) != MSX_OK)
            continue;
        *out += std::string(label) + " @" + params[p].path + ": " + params[p].ty.str() + " = [";
        for (size_t i = 0; i < value.size(); ++i) {
            if (i) *out += ", ";
            *out += msx::f32_display(value[i]);
        }
        *out += "]\n";
    }
}

constexpr uint64_t kLossEvery = 50;  // cli/src/train.rs LOSS_EVERY

}  // namespace

int msx_training_run(msx_training* t, uint64_t start, uint64_t eval_every) {
    if (!t) return MSX_BAD_ARGUMENT;
    t->report.clear();
    return guarded(t, [&] {
        const uint64_t steps = t->compiled.config.steps, end = start + steps;
        if (end < start) throw Fail{MSX_BAD_ARGUMENT, "the run's steps overflow the step counter"};
        std::string& out = t->report;
        if (t->packed) {
            std::vector<char> line(msx_packed_data_line(t->packed, nullptr, 0));
            msx_packed_data_line(t->packed, line.data(), line.size());
            out += line.data();
        }
        parameter_lines(t, "init", &out);
        const bool evaluating = eval_every > 0 && t->heldout != nullptr;
        auto evaluated = [&](uint64_t k) { return evaluating && (k % eval_every == 0 || k == end); };
        // Losses are read a few steps behind the submissions; the lines come out in step order.
        std::map<uint64_t, std::pair<float, float>> evals;
        auto lines_of = [&](uint64_t k, float loss, bool last = false) {
            if (k == start || k % kLossEvery == 0 || k == end || last || evals.count(k)) out += "step " + std::to_string(k) + " loss " + msx::f32_display(loss) + "\n";
            auto e = evals.find(k);
            if (e != evals.end())
                out += "eval " + std::to_string(k) + " loss " + msx::f32_display(e->second.first) + " accuracy " + msx::f32_display(e->second.second) + "\n";
        };
        auto read_loss = [&](uint64_t k) {
            float loss = 0.0f;
            const int rc = msx_training_loss_of(t, k, &loss);
            if (rc == MSX_NON_FINITE) {
                // The run stops at this step: its line is the last one (the last loss of a run
                // always has its line), and there are no `param` lines.
                ok(t, msx_loss_of(t->step, t->submitted_as.at(k), &loss, 0));
                lines_of(k, loss, true);
                throw Fail{MSX_NON_FINITE, t->error};
            }
            if (rc != MSX_OK) throw Fail{rc, t->error};
            lines_of(k, loss);
        };
        constexpr uint64_t kBehind = 4;
        uint64_t next_read = start;
        for (uint64_t k = start; k < end; ++k) {
            if (evaluated(k)) {
                float loss = 0.0f, accuracy = 0.0f;
                if (msx_training_heldout_evaluate(t, &loss, &accuracy) != MSX_OK) throw Fail{MSX_LAUNCH_FAILED, t->error};
                evals[k] = {loss, accuracy};
            }
            if (t->packed && msx_training_feed_packed(t, k) != MSX_OK) throw Fail{MSX_BAD_INPUT, t->error};
            if (t->dense && msx_training_feed_dense(t, k) != MSX_OK) throw Fail{MSX_BAD_INPUT, t->error};
            if (msx_training_step(t, k, end) != MSX_OK) throw Fail{MSX_LAUNCH_FAILED, t->error};
            while (next_read + kBehind <= k) read_loss(next_read++);
        }
        while (next_read < end) read_loss(next_read++);
        // The loss after the last update: the forward program without dropout on the batch of step
        // `end` (a packed run: the batch that step would train on; runner.rs:466-485).
        if (t->packed && msx_training_feed_packed(t, end) != MSX_OK) throw Fail{MSX_BAD_INPUT, t->error};
        if (t->dense && msx_training_feed_dense(t, end) != MSX_OK) throw Fail{MSX_BAD_INPUT, t->error};
        if (evaluated(end)) {
            float loss = 0.0f, accuracy = 0.0f;
            if (msx_training_heldout_evaluate(t, &loss, &accuracy) != MSX_OK) throw Fail{MSX_LAUNCH_FAILED, t->error};
            evals[end] = {loss, accuracy};
        }
        float last = 0.0f;
        if (msx_training_final_loss(t, &last) != MSX_OK) throw Fail{MSX_LAUNCH_FAILED, t->error};
        lines_of(end, last);
        if (!std::isfinite(last)) throw Fail{MSX_NON_FINITE, "E-TRAIN-001: the loss after the last update is not finite"};
        if (msx_training_check_finite(t) != MSX_OK) throw Fail{MSX_NON_FINITE, t->error};
        parameter_lines(t, "param", &out);
    });
}

uint64_t msx_training_report(const msx_training* t, char* out, uint64_t capacity) {
    if (!t) return 0;
    if (out && capacity) {
        const size_t n = std::min<size_t>(capacity - 1, t->report.size());
        std::memcpy(out, t->report.data(), n);
        out[n] = 0;
    }
    return t->report.size() + 1;
}

int msx_training_check_finite(msx_training* t) {
    if (!t) return MSX_BAD_ARGUMENT;
    return guarded(t, [&] {
        const msx::Program& p = t->compiled.step;
        std::vector<float> host;
        for (uint32_t i = 0; i < p.params.size(); ++i) {
            host.resize(p.params[i].ty.count());
            for (int which = 0; which < 3; ++which) {
                int rc = which == 0 ? msx_param_download(t->step, i, host.data(), host.size() * 4)
                                    : msx_moment_download(t->step, i, which == 1 ? 'm' : 'v', host.data(), host.size() * 4);
                if (rc != MSX_OK) continue;  // the step holds no such buffer
                for (float x : host)
                    if (!std::isfinite(x))
                        throw Fail{MSX_NON_FINITE, std::string("E-TRAIN-001: ") + (which == 0 ? "parameter" : which == 1 ? "moment m of" : "moment v of") +
                                                       " `" + p.params[i].path + "` is not finite"};
            }
        }
    });
}

}  // extern "C"
