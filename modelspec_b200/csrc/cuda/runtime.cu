// The msx C ABI (include/msx.h): devices, plans, transfers and step submission.
//
// A plan is built once from the text of a Tensor IR program: the scheduler below walks the live
// nodes in definition order and emits kernel launches (plan.hpp lists the fusions), a linear-scan
// allocator places every intermediate in one arena by liveness, and the launches are captured
// into one CUDA graph at the first step. A step is then one host-to-device copy of the staged
// inputs, one graph launch and one 4-byte read-back of the loss, all on the plan's stream; the
// host never waits inside msx_run unless all of its staging slots are still in flight.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <array>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <thread>

#include "../../../include/msx.h"
#include "../core/frontend.hpp"
#include "../core/rng.hpp"
#include "common.cuh"
#include "kernels.cuh"
#include "plan.hpp"

using msx::Launch;
using msx::Node;
using msx::Op;
using msx::Program;
using msx::Role;
using msx::Slot;
namespace k = msx::k;

namespace {

constexpr uint64_t kAlign = 256;
constexpr uint64_t kGuardBytes = 64;          // 16 sentinel words after every value of a MSX_PLAN_GUARD plan
constexpr uint32_t kGuardWord = 0xA5C3A5C3u;
constexpr int kStagingSlots = 8;  // steps in flight before msx_run waits (the reference's SUBMIT_STEPS)

uint64_t align_up(uint64_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

thread_local std::string g_open_error;

struct StatusError : std::runtime_error {
    int status;
    StatusError(int s, const std::string& what) : std::runtime_error(what), status(s) {}
};

}  // namespace

// NCCL, loaded on first use so that the library has no link-time dependency on it: a
// single-GPU host never needs it.
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    std::string error;

    bool load() {
        if (handle) return true;
        for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
            handle = dlopen(name, RTLD_NOW | RTLD_LOCAL);
            if (handle) break;
        }
        if (!handle) {
            error = std::string("cannot load libnccl.so.2: ") + dlerror();
            return false;
        }
        auto sym = [&](const char* n) { return dlsym(handle, n); };
        GetUniqueId = reinterpret_cast<decltype(GetUniqueId)>(sym("ncclGetUniqueId"));
        CommInitRank = reinterpret_cast<decltype(CommInitRank)>(sym("ncclCommInitRank"));
        CommDestroy = reinterpret_cast<decltype(CommDestroy)>(sym("ncclCommDestroy"));
        AllReduce = reinterpret_cast<decltype(AllReduce)>(sym("ncclAllReduce"));
        GetErrorString = reinterpret_cast<decltype(GetErrorString)>(sym("ncclGetErrorString"));
        if (!GetUniqueId || !CommInitRank || !CommDestroy || !AllReduce || !GetErrorString) {
            error = "libnccl.so.2 lacks an expected symbol";
            dlclose(handle);
            handle = nullptr;
            return false;
        }
        return true;
    }
};
static NcclApi g_nccl;

// A contiguous run of gradient bytes that is summed across ranks by one all-reduce, issued on
// the side stream as soon as the launch that writes its last gradient has been enqueued.
#ifndef MSX_DEFAULT_FUSIONS
#define MSX_DEFAULT_FUSIONS 127u
#endif

struct Bucket {
    uint64_t offset = 0, bytes = 0;  // within the arena
    int after_launch = -1;
    cudaEvent_t ready = nullptr, done = nullptr;
};

struct msx_device {
    int ordinal = 0;
    std::string error;
};

struct InputCheck {
    enum Kind { Ids, Labels, KeyMask, Weights } kind;
    uint64_t bound = 0;  // Ids: table rows; Labels: classes; KeyMask: keys per sequence
};

struct HostInput {
    std::string name;
    uint32_t pos = 0;  // node position
    uint64_t bytes = 0, offset = 0;
    bool i32 = false;
    std::vector<InputCheck> checks;
};

struct msx_plan {
    msx_device* device = nullptr;
    Program program;
    uint64_t seed = 0;
    uint32_t flags = 0;
    msx_plan* shares = nullptr;

    std::vector<Slot> slots;  // one per node, then scratch slots
    std::vector<Launch> launches;
    std::vector<HostInput> inputs;

    cudaStream_t stream = nullptr;
    char* arena = nullptr;
    uint64_t arena_bytes = 0, unshared_bytes = 0;
    std::vector<float*> params, m, v;  // by parameter index; null when the program has none
    std::vector<char> owns_param;
    // Mixed precision: the bf16 working copy of every matrix parameter, which the matmuls read; the
    // optimizer launch and msx_param_upload keep it equal to the rounded f32 master.
    std::vector<void*> params16;
    // msx_state_snapshot: a copy of every parameter and moment, one allocation, made on first use.
    float* backup = nullptr;
    uint64_t backup_floats = 0;
    bool backup_filled = false;
    std::vector<char> owns_param16;
    char* d_inputs = nullptr;
    uint64_t input_bytes = 0;
    std::vector<char> blob;  // the staged inputs, host side
    bool blob_dirty = true;  // staged since the last upload
    char* pinned[kStagingSlots] = {};
    float* pinned_loss = nullptr;  // kStagingSlots floats
    cudaEvent_t slot_begin[kStagingSlots] = {}, slot_done[kStagingSlots] = {};  // around each submitted step
    bool slot_used[kStagingSlots] = {};
    std::vector<float> consts;
    float* d_consts = nullptr;
    uint32_t* d_status = nullptr;
    uint32_t* pinned_status = nullptr;  // kStagingSlots words: the device status word as each step left it
    // Arrival counters of the one-launch two-stage reductions: zero between launches.
    uint32_t* d_counters = nullptr;
    uint32_t counters_used = 0;
    uint32_t* counter(uint32_t index) const { return d_counters + index; }
    void* d_update_tables = nullptr;
    void* d_sum_jobs = nullptr;  // k::SumJob table of the deferred second stages
    cudaStream_t side_stream = nullptr;              // launches with join_before >= 0 run here
    std::vector<cudaEvent_t> side_fork, side_done;   // per launch (null for launches on the main stream)
    void* d_row_sum_jobs = nullptr;  // k::RowSumJob table of the column sums that share one launch

    // What the plan did, counted as it ran: the fields of the reference's RunStats that have a
    // meaning here (vulkan/runner.rs:87-131). A step is one submit (a graph launch) of
    // launches.size() dispatches; barriers are stream order, so none are counted.
    uint64_t host_waits = 0, submits = 0, dispatches = 0, bytes_uploaded = 0, bytes_downloaded = 0;
    uint64_t device_allocations = 0, device_bytes = 0;
    double submitted_ms = 0.0;  // host time from the first submit to the end of the last wait
    std::chrono::steady_clock::time_point first_submit, last_wait;
    bool timing_begun = false;

    int loss_pos = -1;
    uint64_t steps = 0;
    uint64_t shard_rows_before = 0;

    cudaGraphExec_t graph = nullptr;
    cudaEvent_t clock_start = nullptr, clock_stop = nullptr;
    uint64_t clock_steps = 0;

    uint64_t live_nodes = 0, param_bytes = 0;

    // Data parallel (msx_comm_init): rank and size of the job, the communicator, the side stream
    // the gradient buckets are reduced on, and how gradients combine: summed when the loss divides
    // by a whole-batch weight sum (cross_entropy), averaged when it divides by a shard's element
    // count (mse).
    ncclComm_t comm = nullptr;
    bool owns_comm = false;
    int rank = 0, world = 1;
    cudaStream_t comm_stream = nullptr;
    std::vector<Bucket> buckets;
    uint64_t gradient_region_offset = 0, gradient_region_bytes = 0;
    std::vector<uint32_t> gradient_slots;  // in production order
    int optimizer_launch = -1;
    bool average_gradients = false;
    // The weight sum of the whole batch, which a data-parallel cross-entropy divides by, depends
    // only on a host input: it is summed and all-reduced on the side stream from the start of the
    // step, beside the forward pass, into a buffer of its own. The loss is all-reduced on the side
    // stream too; nothing on the device waits for it before the end of the step.
    int early_weights = -1;          // slot of the weights input, or -1
    uint64_t early_rows = 0;
    float* d_weight_total = nullptr;
    cudaEvent_t step_begun = nullptr, weights_summed = nullptr, loss_ready = nullptr, loss_reduced = nullptr;
    bool loss_in_flight = false;     // set while a step is being enqueued
    // msx_comm_exposed_ms: recorded on the main stream after the last launch before the optimizer
    // and right before the optimizer launch (after the waits for the buckets), when set.
    cudaEvent_t probe_backward_done = nullptr, probe_update_begins = nullptr;
    uint64_t bucket_bytes = 25u << 20;
    // Gradient buckets are summed by this backend's own kernel over peer memory when every rank
    // could map every other rank's arena (CUDA IPC, one process per GPU of one machine); otherwise
    // by the library's all-reduce. peer_arena[q] / peer_flags[q] are rank q's arena and flag words
    // as mapped here (this rank's own at q == rank); d_peer_words holds the channel's launch count,
    // block arrivals and failure mark.
    bool peer_ready = false;
    char* peer_arena[k::kPeerRanks] = {};
    uint32_t* peer_flags[k::kPeerRanks] = {};
    uint32_t* d_peer_flags = nullptr;
    uint32_t* d_peer_words = nullptr;

    void* ptr(uint32_t pos) const {
        const Slot& s = slots[pos];
        switch (s.kind) {
            case Slot::Arena: return arena + s.offset;
            case Slot::Param: return params[s.index];
            case Slot::Moment: return (s.moment == 'm' ? m : v)[s.index];
            case Slot::Input: return d_inputs + s.offset;
            case Slot::Const: return reinterpret_cast<char*>(d_consts) + s.offset;
            case Slot::View: return ptr(s.index);
            default: return nullptr;
        }
    }
    float* f(uint32_t pos) const { return static_cast<float*>(ptr(pos)); }
    // The same with the storage type, for the launchers that take either.
    bool half(uint32_t pos) const {
        const Slot& s = slots[pos];
        return s.kind == Slot::View ? half(s.index) : s.half;
    }
    k::In in(uint32_t pos) const { return k::In(ptr(pos), half(pos)); }
    k::Out out(uint32_t pos) const { return k::Out(ptr(pos), half(pos)); }
    // A matmul operand of a mixed-precision plan: a bf16 activation, or the working copy of a parameter.
    const void* h16(uint32_t pos) const {
        const Slot& s = slots[pos];
        if (s.kind == Slot::View) return h16(s.index);
        if (s.kind == Slot::Param) return params16[s.index];
        return s.kind == Slot::Arena && s.half ? arena + s.offset : nullptr;
    }
    int32_t* i(uint32_t pos) const { return static_cast<int32_t*>(ptr(pos)); }
    bool transposed(uint32_t pos) const {
        const Slot& s = slots[pos];
        return s.kind == Slot::View ? !transposed(s.index) : false;
    }
};

namespace {

void cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return;
    int status = e == cudaErrorMemoryAllocation ? MSX_OUT_OF_MEMORY : MSX_LAUNCH_FAILED;
    throw StatusError(status, std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}

void all_reduce(msx_plan* P, float* data, size_t count, bool average, cudaStream_t stream, bool exposed = true);
void close_peer_reduce(msx_plan* P);

// ---------------------------------------------------------------------------------------------
// The scheduler.

// Tuning switch: MSX_FUSE is a bit mask of optional fusions (default: all). 1 sublayer tails
// (dropout + residual + layer norm), 2 adjoint sums inside layer-norm backward, 4 weight-gradient
// matmuls as jobs of one launch, 8 heavy launches with late readers on a side stream, 16
// dropout_grad inside the layer-norm backward that makes or reads its operand, 32 the fused
// attention kernels of a mixed-precision plan (off: batched products with row kernels between),
// 64 the keep decisions of a dropout site stored by the forward launch that draws them, one bit
// per element, and read by the site's dropout_grad (off: every launch draws again).
inline uint32_t fusion_mask() {
    static const uint32_t mask = [] {
        const char* text = std::getenv("MSX_FUSE");
        return text ? static_cast<uint32_t>(std::strtoul(text, nullptr, 0)) : MSX_DEFAULT_FUSIONS;
    }();
    return mask;
}

struct Scheduler {
    msx_plan* P;
    const Program& prog;
    std::vector<char> live, handled;
    std::vector<std::vector<uint32_t>> users;  // live consumers of each node position

    explicit Scheduler(msx_plan* plan) : P(plan), prog(plan->program) {}

    uint32_t pos(uint32_t id) const {
        int at = prog.position(id);
        if (at < 0) throw StatusError(MSX_UNSUPPORTED, "value %" + std::to_string(id) + " is not defined");
        return static_cast<uint32_t>(at);
    }
    const Node& node(uint32_t position) const { return prog.nodes[position]; }
    [[noreturn]] void unsupported(const Node& n, const std::string& why) const {
        throw StatusError(MSX_UNSUPPORTED, "E-TARGET-011: %" + std::to_string(n.id) + " " + msx::op_name(n.op) +
                                               " has no CUDA kernel: " + why);
    }

    // Two-stage sums whose result only the optimizer (or nobody on the device) reads leave their
    // partial results in scratch; one launch before the optimizer finishes them all.
    struct Deferred {
        uint32_t partial;      // scratch slot of the partial results
        uint64_t offset;       // floats into it
        uint32_t chunks;
        uint64_t width;
        uint32_t out;          // node position of the result
    };
    std::vector<Deferred> deferred;
    // Column sums whose result only the optimizer reads wait for one launch that does the first
    // stage of all of them (a bias gradient is a 3 us kernel of its own otherwise); the matrix
    // they sum stays alive until then, so only matrices of a few MB wait.
    struct DeferredRows {
        uint32_t g, partial;
        uint64_t rows, width, ld;
    };
    std::vector<DeferredRows> deferred_rows;
    static constexpr uint64_t kDeferredRowsBytes = 16ull << 20;
    // Matmuls whose result only the optimizer reads (weight gradients) wait too: each would be a
    // launch of a few dozen CTAs for a few microseconds; together, as jobs of one launch per
    // storage form, they fill the device. Their operands stay alive until then, so the total is
    // capped.
    struct DeferredMatmul {
        uint32_t a, b, result;
        int workspace;
        uint64_t m, n, k;
    };
    std::vector<DeferredMatmul> deferred_matmuls[4];  // by storage form: 2 * a_t + b_t
    uint64_t deferred_matmul_bytes = 0;
    static constexpr uint64_t kDeferredMatmulBytes = 2ull << 30;
    static constexpr uint64_t kDeferredMatmulFlop = 2ull << 30;
    bool deferrable(uint32_t at) const {
        for (uint32_t u : users[at])
            if (node(u).tag != msx::Tag::Optimizer || !handled[u]) return false;
        return true;
    }
    // Moves the launch just emitted up to right after the last launch that writes something it
    // reads: it only feeds the finalize launch, so from there on it can run beside the rest of
    // the backward pass (mark_side_launches puts it on the side stream).
    void hoist_last_launch() {
        if (!(fusion_mask() & 8u) || P->launches.size() < 2) return;
        const size_t last = P->launches.size() - 1;
        size_t earliest = 0;
        for (size_t l = 0; l < last; ++l)
            for (uint32_t w : P->launches[l].writes)
                for (uint32_t r : P->launches[last].reads)
                    if (r == w) earliest = l + 1;
        if (earliest >= last) return;
        Launch moved = std::move(P->launches[last]);
        P->launches.pop_back();
        P->launches.insert(P->launches.begin() + static_cast<std::ptrdiff_t>(earliest), std::move(moved));
    }

    void emit_finalize() {
        for (int form = 0; form < 4; ++form) {
            const std::vector<DeferredMatmul>& all = deferred_matmuls[form];
            for (size_t begin = 0; begin < all.size(); begin += k::kMatmulJobs) {
                const std::vector<DeferredMatmul> part(all.begin() + begin, all.begin() + std::min(all.size(), begin + k::kMatmulJobs));
                std::vector<uint32_t> reads, writes;
                uint64_t flop = 0;
                for (const DeferredMatmul& d : part) {
                    reads.push_back(d.a);
                    reads.push_back(d.b);
                    writes.push_back(d.workspace >= 0 ? static_cast<uint32_t>(d.workspace) : d.result);
                    flop += 2 * d.m * d.n * d.k;
                }
                Node pseudo;
                pseudo.id = node(part[0].result).id;
                msx_plan* plan = P;
                const bool a_t = (form & 2) != 0, b_t = (form & 1) != 0;
                Launch& l = emit("matmul_jobs", pseudo, reads, writes, [=](cudaStream_t s) {
                    std::vector<k::MatmulJob> jobs;
                    for (const DeferredMatmul& d : part)
                        jobs.push_back({plan->f(d.a), plan->f(d.b), plan->f(static_cast<uint32_t>(d.workspace)),
                                        plan->f(static_cast<uint32_t>(d.workspace)), d.m, d.n, d.k});
                    k::matmul_tc_jobs(s, jobs.data(), static_cast<uint32_t>(jobs.size()), a_t, b_t, plan->d_status);
                });
                l.flop = flop;
                hoist_last_launch();
            }
        }
        finish_deferred_sums();
    }

    // The deferred sums entered since the last call, as one launch for the first stages of the
    // column sums and one for every second stage: the job tables are cut here, each launch
    // walking its own part.
    void finish_deferred_sums() {
        if (deferred_rows.size() > rows_finished) {
            std::vector<uint32_t> reads, writes;
            uint32_t blocks = 0;
            for (size_t i = rows_finished; i < deferred_rows.size(); ++i) {
                const DeferredRows& d = deferred_rows[i];
                reads.push_back(d.g);
                writes.push_back(d.partial);
                blocks += k::row_sum_job_blocks(d.rows, d.width);
            }
            Node pseudo;
            pseudo.id = node(deferred_rows[rows_finished].g).id;
            msx_plan* plan = P;
            const size_t first = rows_finished;
            const uint32_t jobs = static_cast<uint32_t>(deferred_rows.size() - rows_finished);
            emit("sum_rows_batched", pseudo, reads, writes, [=](cudaStream_t s) {
                k::sum_rows_batched(s, static_cast<const k::RowSumJob*>(plan->d_row_sum_jobs) + first, jobs, blocks);
            });
            hoist_last_launch();
            rows_cuts.push_back(rows_finished);
            rows_finished = deferred_rows.size();
        }
        if (deferred.size() == sums_finished) return;
        std::vector<uint32_t> reads, writes;
        uint32_t blocks = 0;
        for (size_t i = sums_finished; i < deferred.size(); ++i) {
            const Deferred& d = deferred[i];
            reads.push_back(d.partial);
            writes.push_back(d.out);
            blocks += k::sum_job_blocks(d.chunks, d.width);
        }
        Node pseudo;
        pseudo.id = node(deferred[sums_finished].out).id;
        msx_plan* plan = P;
        const size_t first = sums_finished;
        const uint32_t jobs = static_cast<uint32_t>(deferred.size() - sums_finished);
        emit("finalize_sums", pseudo, reads, writes, [=](cudaStream_t s) {
            k::finalize_sums(s, static_cast<const k::SumJob*>(plan->d_sum_jobs) + first, jobs, blocks);
        });
        // Issued as soon as the last partial sums exist: what follows them in the backward pass
        // does not read its results, so it runs beside that.
        hoist_last_launch();
        sums_cuts.push_back(sums_finished);
        sums_finished = deferred.size();
    }
    // Where each launch's part of the two job tables starts.
    std::vector<size_t> rows_cuts, sums_cuts;
    size_t rows_finished = 0, sums_finished = 0;
    // A large model's deferred sums are finished a layer's worth at a time rather than all at the
    // end of the backward pass: the gradients they complete can then be exchanged (a data-parallel
    // run reduces a bucket as soon as the launch that completes it has been issued) while the
    // layers below are still being differentiated. Products waiting as jobs of one launch write
    // partial sums of their own, so nothing is finished early while any wait.
    static constexpr uint64_t kFinishSumsBytes = 24ull << 20;
    void finish_deferred_sums_when_large() {
        for (int form = 0; form < 4; ++form)
            if (!deferred_matmuls[form].empty()) return;
        uint64_t pending = 0;
        for (size_t i = sums_finished; i < deferred.size(); ++i) pending += deferred[i].width * 4;
        if (pending >= kFinishSumsBytes) finish_deferred_sums();
    }

    // A matmul or column-sum launch whose results are first read at least `kSideGap` launches
    // later does not have to hold up the launches in between: it goes to the side stream.
    static constexpr int kSideGap = 4;
    void mark_side_launches() {
        if (!(fusion_mask() & 8u)) return;
        const int count = static_cast<int>(P->launches.size());
        // From the last launch back, so that a reader's own place is known: the side stream runs its
        // launches in order, so a result that another side launch reads is waited for where that
        // launch is, not where it is issued.
        for (int l = count - 1; l >= 0; --l) {
            Launch& launch = P->launches[static_cast<size_t>(l)];
            // finalize_sums writes outputs (gradients that the optimizer launch reads, and before it
            // a data-parallel bucket: the bucket waits for the side launches that wrote into it).
            // So does the scatter of a lookup table's gradient that nothing but the optimizer reads
            // (a position table's, beside the token table's).
            bool finalize = launch.kernel == "finalize_sums";
            if (launch.kernel == "embedding_grad" && !launch.writes.empty()) {
                bool all_outputs = true;
                for (uint32_t w : launch.writes)
                    if (w < prog.nodes.size() ? !is_output_value(w) : true) all_outputs = false;
                finalize = all_outputs;
                if (!all_outputs) continue;
            }
            if (launch.kernel != "matmul" && launch.kernel != "sum_rows" && launch.kernel != "embedding_order" &&
                launch.kernel != "matmul_jobs" && launch.kernel != "sum_rows_batched" && !finalize)
                continue;
            auto stored_as = [this](uint32_t v) {
                while (P->slots[v].kind == Slot::View) v = P->slots[v].index;
                return v;
            };
            bool eligible = !launch.writes.empty();
            for (uint32_t w : launch.writes) {
                const uint32_t home = stored_as(w);
                if (P->slots[home].kind != Slot::Arena) eligible = false;
                // An output is read by the host or a bucket, not by a launch; a value that a later
                // launch turns into an output in place is read by that launch.
                if (home == w && w < prog.nodes.size() && !finalize)
                    for (const msx::Output& o : prog.outputs)
                        if (pos(o.value) == w) eligible = false;
            }
            if (!eligible) continue;
            int first_reader = count;
            for (int later = l + 1; later < count; ++later) {
                const Launch& other = P->launches[static_cast<size_t>(later)];
                const int needed_at = other.join_before >= 0 ? other.join_before : later;
                for (uint32_t w : launch.writes) {
                    for (uint32_t r : other.reads)
                        if (stored_as(r) == stored_as(w)) first_reader = std::min(first_reader, needed_at);
                    for (uint32_t again : other.writes)
                        if (stored_as(again) == stored_as(w)) first_reader = std::min(first_reader, needed_at);
                }
            }
            if (first_reader == count || first_reader - l < (finalize ? 2 : kSideGap)) continue;
            launch.join_before = first_reader;
            launch.side_writes_outputs = finalize;
        }
    }

    uint32_t counters(uint64_t n) {
        uint32_t base = P->counters_used;
        P->counters_used += static_cast<uint32_t>(n);
        return base;
    }

    // A mixed-precision plan (MSX_PLAN_BF16) stores every rank-2 f32 intermediate as bf16;
    // program outputs (the loss, the gradients the optimizer and the buckets read), vectors,
    // scalars, partial sums and everything the host supplies stay f32.
    bool mixed() const { return (P->flags & MSX_PLAN_BF16) != 0; }
    bool stored_half(const Node& n) const {
        if (!mixed() || n.ty.rank() != 2 || n.ty.i32) return false;
        for (const msx::Output& o : prog.outputs)
            if (o.value == n.id) return false;
        return true;
    }
    void make_arena(Slot& slot, const Node& n) {
        slot.kind = Slot::Arena;
        slot.half = stored_half(n);
        slot.bytes = std::max<uint64_t>(n.ty.count() * (slot.half ? 2 : 4), 4);
    }
    // Every bf16 matrix a launch touches has rows of a multiple of 8 elements as stored (16 bytes:
    // what TMA and the 8-byte accesses of the row kernels need), by its width or by its pitch.
    void check_half_widths() const {
        for (const Launch& l : P->launches)
            for (const std::vector<uint32_t>* touched : {&l.reads, &l.writes})
                for (uint32_t t : *touched) {
                    const Slot& slot = P->slots[t];
                    if (t >= prog.nodes.size() || slot.kind != Slot::Arena || !slot.half) continue;
                    const Node& n = node(t);
                    if ((slot.pitch ? slot.pitch : n.ty.shape[1]) % 8 != 0)
                        throw StatusError(MSX_UNSUPPORTED, "E-TARGET-011: %" + std::to_string(n.id) + " " + msx::op_name(n.op) +
                                                               ": a bf16 plan stores matrices whose rows are a multiple of 8 elements");
                }
    }
    // The launches whose kernels read and write bf16 activations.
    static bool half_capable(const std::string& kernel) {
        static const char* const names[] = {"embedding", "embedding_grad", "add_layer_norm", "add_layer_norm_dropout", "dropout_add_layer_norm",
                                            "dropout_add", "gelu_layer_norm", "layer_norm", "matmul", "attention_forward", "attention_backward",
                                            "gelu", "unary", "gelu_grad", "dropout", "layer_norm_backward", "cross_entropy_with_grad",
                                            "cross_entropy", "sum_rows", "sum_rows_batched"};
        for (const char* name : names)
            if (kernel == name) return true;
        return false;
    }

    uint32_t scratch(uint64_t bytes) {
        Slot s;
        s.kind = Slot::Arena;
        s.bytes = std::max<uint64_t>(bytes, 4);
        P->slots.push_back(s);
        return static_cast<uint32_t>(P->slots.size() - 1);
    }

    Launch& emit(const char* kernel, const Node& n, std::vector<uint32_t> reads, std::vector<uint32_t> writes,
                 std::function<void(cudaStream_t)> run) {
        Launch l;
        l.kernel = kernel;
        l.value = n.id;
        // A folded Transpose is read through its source.
        for (uint32_t& r : reads)
            while (P->slots[r].kind == Slot::View) r = P->slots[r].index;
        l.reads = std::move(reads);
        l.writes = std::move(writes);
        l.run = std::move(run);
        if (mixed() && !half_capable(l.kernel))
            for (const std::vector<uint32_t>* touched : {&l.reads, &l.writes})
                for (uint32_t t : *touched)
                    if (P->slots[t].half) unsupported(n, std::string("its kernel (") + kernel + ") has no bf16 form, and a bf16 plan stores %" +
                                                             (t < prog.nodes.size() ? std::to_string(node(t).id) : std::string("scratch")) + " as bf16");
        P->launches.push_back(std::move(l));
        return P->launches.back();
    }

    bool is_output_value(uint32_t v) const {
        for (const msx::Output& o : prog.outputs)
            if (pos(o.value) == v) return true;
        return false;
    }

    bool is_scalar_operand(uint32_t operand_pos, const Node& result) const {
        return node(operand_pos).ty.rank() == 0 && result.ty.rank() > 0;
    }

    void run() {
        const size_t n = prog.nodes.size();
        P->slots.assign(n, Slot{});
        live.assign(n, 0);
        handled.assign(n, 0);
        users.assign(n, {});
        for (const msx::Output& o : prog.outputs) live[pos(o.value)] = 1;
        for (size_t at = n; at-- > 0;)
            if (live[at])
                for (uint32_t o : node(static_cast<uint32_t>(at)).operands) live[pos(o)] = 1;
        for (size_t at = 0; at < n; ++at)
            if (live[at]) {
                ++P->live_nodes;
                for (uint32_t o : node(static_cast<uint32_t>(at)).operands) users[pos(o)].push_back(static_cast<uint32_t>(at));
            }
        place_leaves();
        fold_constants();
        plan_optimizer();
        fold_transposes();
        for (uint32_t at = 0; at < n; ++at)
            if (live[at] && !handled[at]) {
                schedule(at);
                finish_deferred_sums_when_large();
            }
        emit_finalize();
        emit_optimizer();
        if (mixed()) check_half_widths();
        mark_side_launches();
        for (const msx::Output& o : prog.outputs) {
            Slot& s = P->slots[pos(o.value)];
            s.keep = true;
        }
        if (!prog.outputs.empty()) {
            const msx::Output* loss = nullptr;
            for (const msx::Output& o : prog.outputs)
                if (o.role == Role::Loss) loss = &o;
            if (!loss && node(pos(prog.outputs[0].value)).ty.rank() == 0) loss = &prog.outputs[0];
            if (loss) P->loss_pos = static_cast<int>(pos(loss->value));
        }
    }

    // Parameters, host inputs and moments get their storage class; inputs are laid out in the
    // upload region in node order.
    void place_leaves() {
        const size_t np = prog.params.size();
        P->params.assign(np, nullptr);
        P->m.assign(np, nullptr);
        P->v.assign(np, nullptr);
        P->owns_param.assign(np, 0);
        P->params16.assign(np, nullptr);
        P->owns_param16.assign(np, 0);
        uint64_t offset = 0;
        for (uint32_t at = 0; at < prog.nodes.size(); ++at) {
            const Node& nd = node(at);
            Slot& s = P->slots[at];
            s.bytes = nd.ty.count() * 4;
            if (nd.op == Op::ParamRead) {
                s.kind = Slot::Param;
                s.index = nd.param;
                handled[at] = 1;
            } else if (nd.op == Op::Input) {
                handled[at] = 1;
                bool moment = false;
                for (char which : {'m', 'v'}) {
                    std::string prefix = std::string("optimizer.") + which + "@";
                    if (nd.name.compare(0, prefix.size(), prefix) == 0) {
                        int param = prog.param_index(nd.name.substr(prefix.size()));
                        if (param < 0) throw StatusError(MSX_UNSUPPORTED, "moment input of an unknown parameter: " + nd.name);
                        s.kind = Slot::Moment;
                        s.index = static_cast<uint32_t>(param);
                        s.moment = which;
                        moment = true;
                    }
                }
                if (moment || !live[at]) continue;
                s.kind = Slot::Input;
                s.offset = offset;
                HostInput in;
                in.name = nd.name;
                in.pos = at;
                in.bytes = s.bytes;
                in.offset = offset;
                in.i32 = nd.ty.i32;
                P->inputs.push_back(in);
                offset += align_up(s.bytes);
            }
        }
        P->input_bytes = offset;
        // What the reference's interpreter checks before a run, by how each input is read.
        for (HostInput& in : P->inputs)
            for (uint32_t u : users[in.pos]) {
                const Node& user = node(u);
                auto operand_is = [&](size_t kth) { return user.operands.size() > kth && pos(user.operands[kth]) == in.pos; };
                if (user.op == Op::Embedding && operand_is(1))
                    in.checks.push_back({InputCheck::Ids, node(pos(user.operands[0])).ty.shape[0]});
                if (user.op == Op::EmbeddingGrad && operand_is(0)) in.checks.push_back({InputCheck::Ids, user.rows});
                if ((user.op == Op::CrossEntropy || user.op == Op::CrossEntropyGrad) && operand_is(1))
                    in.checks.push_back({InputCheck::Labels, node(pos(user.operands[0])).ty.shape[1]});
                if ((user.op == Op::CrossEntropy || user.op == Op::CrossEntropyGrad) && operand_is(2))
                    in.checks.push_back({InputCheck::Weights, 0});
                if ((user.op == Op::Attention || user.op == Op::AttentionGradQ || user.op == Op::AttentionGradK ||
                     user.op == Op::AttentionGradV) && operand_is(3))
                    in.checks.push_back({InputCheck::KeyMask, in.bytes / 4 / std::max<uint64_t>(1, node(in.pos).ty.shape[0])});
            }
    }

    void set_const(uint32_t at, float value) {
        Slot& s = P->slots[at];
        s.kind = Slot::Const;
        s.constant = value;
        s.offset = P->consts.size() * sizeof(float);
        s.bytes = 4;
        P->consts.push_back(value);
        handled[at] = 1;
    }

    // Rank-0 expressions over constants, each one rounded f32 operation as on the device.
    void fold_constants() {
        for (uint32_t at = 0; at < prog.nodes.size(); ++at) {
            const Node& nd = node(at);
            if (!live[at] || nd.ty.rank() != 0 || nd.ty.i32) continue;
            if (nd.op == Op::Scalar) {
                set_const(at, nd.scalar);
                continue;
            }
            bool all_const = !nd.operands.empty();
            for (uint32_t o : nd.operands) all_const = all_const && P->slots[pos(o)].kind == Slot::Const;
            if (!all_const) continue;
            auto c = [&](size_t kth) { return P->slots[pos(nd.operands[kth])].constant; };
            volatile float r;
            switch (nd.op) {
                case Op::Add: r = c(0) + c(1); break;
                case Op::Sub: r = c(0) - c(1); break;
                case Op::Mul: r = c(0) * c(1); break;
                case Op::Div: r = c(0) / c(1); break;
                case Op::Sqrt: r = std::sqrt(c(0)); break;
                case Op::StopGradient: r = c(0); break;
                default: continue;
            }
            set_const(at, r);
        }
    }

    // ---- the optimizer subgraph ------------------------------------------------------------
    struct Update {
        uint32_t param, grad_pos;
    };
    std::vector<Update> updates;

    void plan_optimizer() {
        if (prog.optimizer.rule == msx::Rule::None) return;
        std::map<uint32_t, uint32_t> grad_of;  // param -> gradient position
        std::set<uint32_t> stops;
        for (const msx::Output& o : prog.outputs)
            if (o.role == Role::Gradient) {
                grad_of[o.param] = pos(o.value);
                stops.insert(pos(o.value));
            }
        // Everything between the gradients and the update / next-moment outputs is the update
        // subgraph: it runs as one multi-tensor launch and its nodes get no storage.
        std::vector<uint32_t> work;
        for (const msx::Output& o : prog.outputs) {
            if (o.role != Role::Update && o.role != Role::Moment) continue;
            uint32_t at = pos(o.value);
            if (o.role == Role::Update) {
                const Node& nd = node(at);
                bool shape = nd.op == Op::Sub && nd.operands.size() == 2 && node(pos(nd.operands[0])).op == Op::ParamRead &&
                             node(pos(nd.operands[0])).param == o.param;
                if (!shape || !grad_of.count(o.param))
                    throw StatusError(MSX_UNSUPPORTED, "the update of @" + prog.params[o.param].path +
                                                           " is not `p - rate * step` over its gradient");
                updates.push_back({o.param, grad_of[o.param]});
                P->slots[at].kind = Slot::Param;
                P->slots[at].index = o.param;
            } else {
                P->slots[at].kind = Slot::Moment;
                P->slots[at].index = o.param;
                P->slots[at].moment = o.moment;
            }
            work.push_back(at);
        }
        while (!work.empty()) {
            uint32_t at = work.back();
            work.pop_back();
            if (handled[at] || stops.count(at)) continue;
            const Node& nd = node(at);
            if (nd.op == Op::ParamRead || nd.op == Op::Input || P->slots[at].kind == Slot::Const) continue;
            handled[at] = 1;
            for (uint32_t o : nd.operands) work.push_back(pos(o));
        }
        if (prog.optimizer.rule == msx::Rule::AdamW)
            for (const Update& u : updates) {
                bool has_m = false, has_v = false;
                for (const msx::Output& o : prog.outputs)
                    if (o.role == Role::Moment && o.param == u.param) (o.moment == 'm' ? has_m : has_v) = true;
                if (!has_m || !has_v)
                    throw StatusError(MSX_UNSUPPORTED, "an adamw step without both next moments of @" + prog.params[u.param].path);
            }
    }

    void emit_optimizer() {
        if (updates.empty()) return;
        msx_plan* plan = P;
        // Device tables: tensors, then the chunk -> (tensor, start) map.
        std::vector<uint32_t> chunk_tensor, chunk_start;
        for (uint32_t t = 0; t < updates.size(); ++t) {
            uint64_t count = prog.params[updates[t].param].ty.count();
            for (uint64_t c = 0; c * k::kUpdateChunk < count; ++c) {
                chunk_tensor.push_back(t);
                chunk_start.push_back(static_cast<uint32_t>(c));
            }
        }
        uint32_t chunks = static_cast<uint32_t>(chunk_tensor.size());
        const size_t n_updates = updates.size();
        update_chunk_tensor = chunk_tensor;
        update_chunk_start = chunk_start;
        std::vector<uint32_t> reads, writes;
        uint64_t elements = 0;
        for (const Update& u : updates) {
            reads.push_back(u.grad_pos);
            elements += prog.params[u.param].ty.count();
        }
        Node pseudo;
        pseudo.id = node(updates[0].grad_pos).id;
        bool adamw = prog.optimizer.rule == msx::Rule::AdamW;
        const msx::OptimizerInfo& o = prog.optimizer;
        if (adamw) {
            msx::AdamW a{o.weight_decay, o.beta1, o.beta2, o.eps, o.warmup_steps};
            std::vector<float> c = a.constants();
            k::AdamWConstants constants{c[0], c[1], c[2], c[3], c[4], c[5]};
            int lr_t = -1, c1 = -1, c2 = -1;
            for (uint32_t at = 0; at < prog.nodes.size(); ++at) {
                const Node& nd = node(at);
                if (nd.op != Op::Input) continue;
                if (nd.name == "optimizer.lr_t") lr_t = static_cast<int>(at);
                if (nd.name == "optimizer.c1") c1 = static_cast<int>(at);
                if (nd.name == "optimizer.c2") c2 = static_cast<int>(at);
            }
            if (lr_t < 0 || c1 < 0 || c2 < 0) throw StatusError(MSX_UNSUPPORTED, "an adamw step without its lr_t, c1, c2 inputs");
            reads.push_back(static_cast<uint32_t>(lr_t));
            reads.push_back(static_cast<uint32_t>(c1));
            reads.push_back(static_cast<uint32_t>(c2));
            Launch& l = emit("adamw_multi_tensor", pseudo, reads, writes, [=](cudaStream_t s) {
                auto* tensors = static_cast<k::UpdateTensor*>(plan->d_update_tables);
                auto* ct = reinterpret_cast<uint32_t*>(tensors + n_updates);
                k::adamw(s, tensors, ct, ct + chunks, chunks, constants, plan->f(static_cast<uint32_t>(lr_t)),
                         plan->f(static_cast<uint32_t>(c1)), plan->f(static_cast<uint32_t>(c2)));
            });
            l.flop = 16 * elements;
            optimizer_bytes = 28 * elements;
        } else {
            // The rate is the folded Scalar the update multiplies the gradient by.
            const Node& sub = node(update_node(updates[0].param));
            const Node& scaled = node(pos(sub.operands[1]));
            uint32_t rate = pos(scaled.operands[0]);
            if (scaled.op != Op::Mul || P->slots[rate].kind != Slot::Const)
                throw StatusError(MSX_UNSUPPORTED, "the sgd update is not `p - lr * g` with a constant rate");
            reads.push_back(rate);
            Launch& l = emit("sgd_multi_tensor", pseudo, reads, writes, [=](cudaStream_t s) {
                auto* tensors = static_cast<k::UpdateTensor*>(plan->d_update_tables);
                auto* ct = reinterpret_cast<uint32_t*>(tensors + n_updates);
                k::sgd(s, tensors, ct, ct + chunks, chunks, plan->f(rate));
            });
            l.flop = 2 * elements;
            optimizer_bytes = 12 * elements;
        }
    }
    std::vector<uint32_t> update_chunk_tensor, update_chunk_start;
    uint64_t optimizer_bytes = 0;
    uint32_t update_node(uint32_t param) const {
        for (const msx::Output& o : prog.outputs)
            if (o.role == Role::Update && o.param == param) return pos(o.value);
        throw StatusError(MSX_UNSUPPORTED, "no update");
    }

    // ---- transposes ------------------------------------------------------------------------
    // matmul_of[t] = position of the matmul a Transpose node t absorbs (its operands swapped).
    std::map<uint32_t, uint32_t> absorbed_matmul;

    // Whether the Transpose at `at` can be read in place by everything that reads it: matmuls,
    // and transposes that can themselves be read in place.
    bool folds(uint32_t at, std::map<uint32_t, bool>& memo) {
        auto known = memo.find(at);
        if (known != memo.end()) return known->second;
        bool ok = !users[at].empty();
        for (const msx::Output& o : prog.outputs) ok = ok && pos(o.value) != at;
        for (uint32_t u : users[at]) {
            if (!ok) break;
            const Node& user = node(u);
            if (handled[u]) ok = false;
            else if (user.op == Op::MatMul) continue;
            else if (user.op == Op::Transpose) ok = folds(u, memo);
            else ok = false;
        }
        memo[at] = ok;
        return ok;
    }

    void fold_transposes() {
        std::map<uint32_t, bool> memo;
        for (uint32_t at = 0; at < prog.nodes.size(); ++at) {
            const Node& nd = node(at);
            if (!live[at] || handled[at] || nd.op != Op::Transpose) continue;
            if (folds(at, memo)) {
                Slot& s = P->slots[at];
                s.kind = Slot::View;
                s.index = pos(nd.operands[0]);
                handled[at] = 1;
                continue;
            }
            uint32_t src = pos(nd.operands[0]);
            bool src_output = false;
            for (const msx::Output& o : prog.outputs) src_output = src_output || pos(o.value) == src;
            if (node(src).op == Op::MatMul && users[src].size() == 1 && !src_output && !handled[src]) {
                absorbed_matmul[at] = src;
                handled[src] = 1;  // never materialised
            }
        }
    }

    // ---- one node --------------------------------------------------------------------------
    void schedule(uint32_t at) {
        const Node& nd = node(at);
        msx_plan* plan = P;
        Slot& out = P->slots[at];
        make_arena(out, nd);
        std::vector<uint32_t> in;
        for (uint32_t o : nd.operands) in.push_back(pos(o));
        const uint64_t count = nd.ty.count();
        auto rows_of = [&](uint32_t p) { return node(p).ty.shape.at(0); };
        auto cols_of = [&](uint32_t p) { return node(p).ty.shape.at(1); };
        switch (nd.op) {
            case Op::Add:
            case Op::Sub:
            case Op::Mul:
            case Op::Div: {
                if (nd.op == Op::Add && joins_layer_norm_adjoint(at)) {
                    // The sum is formed inside the layer-norm backward launch that alone reads it.
                    std::vector<uint32_t> addends;
                    for (uint32_t operand : in) {
                        auto inner = adjoint_sums.find(operand);
                        if (inner != adjoint_sums.end()) addends.insert(addends.end(), inner->second.begin(), inner->second.end());
                        else addends.push_back(operand);
                    }
                    adjoint_sums[at] = addends;
                    out.kind = Slot::Dead;
                    break;
                }
                if (nd.op == Op::Add && schedule_add_layer_norm(at)) break;
                k::Binary op = nd.op == Op::Add ? k::Binary::Add : nd.op == Op::Sub ? k::Binary::Sub
                               : nd.op == Op::Mul ? k::Binary::Mul : k::Binary::Div;
                bool sa = is_scalar_operand(in[0], nd), sb = is_scalar_operand(in[1], nd);
                uint32_t a = in[0], b = in[1];
                emit("binary", nd, in, {at}, [=](cudaStream_t s) { k::binary(s, op, plan->f(a), sa, plan->f(b), sb, plan->f(at), count); });
                break;
            }
            case Op::Relu:
            case Op::Sqrt:
            case Op::Gelu:
            case Op::StopGradient: {
                k::Unary op = nd.op == Op::Relu ? k::Unary::Relu : nd.op == Op::Sqrt ? k::Unary::Sqrt
                              : nd.op == Op::Gelu ? k::Unary::Gelu : k::Unary::Copy;
                uint32_t a = in[0];
                // gelu with the layer norm of its result (a head's transform): one launch writes both.
                if (nd.op == Op::Gelu && (fusion_mask() & 1u) && nd.ty.rank() == 2 && k::layer_norm_backward_supported(nd.ty.shape[1])) {
                    int norm = -1;
                    for (uint32_t u : users[at]) {
                        const Node& ln = node(u);
                        if (ln.op == Op::LayerNorm && !handled[u] && pos(ln.operands[0]) == at && pos(ln.operands[1]) < at && pos(ln.operands[2]) < at) {
                            norm = static_cast<int>(u);
                            break;
                        }
                    }
                    if (norm >= 0) {
                        const uint32_t ln_at = static_cast<uint32_t>(norm);
                        const uint32_t gamma = pos(node(ln_at).operands[1]), beta = pos(node(ln_at).operands[2]);
                        handled[ln_at] = 1;
                        Slot& slot = P->slots[ln_at];
                        make_arena(slot, node(ln_at));
                        const uint64_t r = nd.ty.shape[0], h = nd.ty.shape[1];
                        emit("gelu_layer_norm", nd, {a, gamma, beta}, {at, ln_at}, [=](cudaStream_t s) {
                            k::add_layer_norm(s, plan->in(a), k::In(), nullptr, plan->f(gamma), plan->f(beta), plan->out(at), plan->out(ln_at), nullptr,
                                              k::Out(), r, h, true);
                        });
                        break;
                    }
                }
                emit(nd.op == Op::Gelu ? "gelu" : "unary", nd, in, {at}, [=](cudaStream_t s) { k::unary(s, op, plan->in(a), plan->out(at), count); });
                break;
            }
            case Op::ReluGrad:
            case Op::GeluGrad: {
                bool gelu = nd.op == Op::GeluGrad;
                uint32_t a = in[0], g = in[1];
                emit(gelu ? "gelu_grad" : "relu_grad", nd, in, {at}, [=](cudaStream_t s) {
                    if (gelu) k::gelu_grad(s, plan->in(a), plan->in(g), plan->out(at), count);
                    else k::relu_grad(s, plan->f(a), plan->f(g), plan->f(at), count);
                });
                break;
            }
            case Op::BroadcastScalar: {
                uint32_t a = in[0];
                emit("fill", nd, in, {at}, [=](cudaStream_t s) { k::fill_from_scalar(s, plan->f(a), plan->f(at), count); });
                break;
            }
            case Op::MatMul: {
                uint64_t m = nd.ty.shape[0], n = nd.ty.shape[1], kk = cols_of(in[0]);
                std::vector<Product> group = {claim_product(at)};
                const bool pitched = pitch_of(group[0].a) || pitch_of(group[0].b) || pitchable(group[0].result);
                if ((fusion_mask() & 4u) && !(P->flags & MSX_PLAN_EXACT_MATMUL) && !mixed() && !pitched && group[0].bias < 0 &&
                    nd.tag == msx::Tag::Gradient && deferrable(group[0].result)) {
                    const uint64_t operand_bytes = (m * kk + kk * n) * 4;
                    // Only products too small to fill the device on their own: a large one is better
                    // off with the tile the plan model picks for it.
                    if (2 * m * n * kk <= kDeferredMatmulFlop && deferred_matmul_bytes + operand_bytes <= kDeferredMatmulBytes) {
                        deferred_matmul_bytes += operand_bytes;
                        const Product& p = group[0];
                        const k::MatmulTcPlan job = k::matmul_tc_job_plan(m, n, kk);
                        // An unsplit job writes one "partial" tile too: the launch then touches no
                        // output, only scratch that the finalize launch reads, and may run beside others.
                        const int ws = static_cast<int>(scratch(std::max<uint64_t>(job.workspace_floats, m * n) * 4));
                        deferred.push_back({static_cast<uint32_t>(ws), 0, job.splits, m * n, p.result});
                        uint32_t a = p.a, b = p.b;
                        const int form = (P->transposed(a) ? 2 : 0) + (P->transposed(b) ? 1 : 0);
                        while (P->slots[a].kind == Slot::View) a = P->slots[a].index;
                        while (P->slots[b].kind == Slot::View) b = P->slots[b].index;
                        deferred_matmuls[form].push_back({a, b, p.result, ws, m, n, kk});
                        break;
                    }
                }
                // Later matmuls of the same shape and storage form whose operands already exist
                // (the three projections of an attention layer, their gradients) join the launch.
                if (!(P->flags & MSX_PLAN_EXACT_MATMUL) && !mixed() && !pitched)
                    for (uint32_t later = at + 1; later < prog.nodes.size() && later < at + 64 && group.size() < 4; ++later)
                        if (joins(later, group[0], at, m, n, kk)) group.push_back(claim_product(later));
                emit_matmul(nd, group, m, n, kk);
                break;
            }
            case Op::Transpose: {
                auto absorbed = absorbed_matmul.find(at);
                if (absorbed != absorbed_matmul.end()) {
                    // (A x B)^T = B^T x A^T: the same products summed over the same ascending k.
                    const Node& mm = node(absorbed->second);
                    uint32_t a = pos(mm.operands[0]), b = pos(mm.operands[1]);
                    uint64_t m = nd.ty.shape[0], n = nd.ty.shape[1], kk = cols_of(a);
                    std::vector<Product> one = {{at, at, b, a, true, true, -1}};
                    emit_matmul(nd, one, m, n, kk);
                } else {
                    uint32_t a = in[0];
                    uint64_t r = rows_of(a), c = cols_of(a);
                    if (P->slots[a].kind == Slot::View) unsupported(nd, "a transpose of a folded transpose that is not a matmul operand");
                    emit("transpose", nd, in, {at}, [=](cudaStream_t s) { k::transpose(s, plan->f(a), plan->f(at), r, c); });
                }
                break;
            }
            case Op::ReduceSum:
            case Op::ReduceMean: {
                uint32_t a = in[0], tmp = scratch(k::reduce_scratch_doubles() * 8);
                bool mean = nd.op == Op::ReduceMean;
                uint64_t n = node(a).ty.count();
                emit("reduce", nd, in, {at, tmp}, [=](cudaStream_t s) {
                    k::reduce_sum(s, plan->f(a), n, mean, static_cast<double*>(plan->ptr(tmp)), plan->f(at));
                });
                break;
            }
            case Op::Mse: {
                uint32_t a = in[0], b = in[1], tmp = scratch(k::reduce_scratch_doubles() * 8);
                uint64_t n = node(a).ty.count();
                emit("mse", nd, in, {at, tmp}, [=](cudaStream_t s) {
                    k::mse(s, plan->f(a), plan->f(b), n, static_cast<double*>(plan->ptr(tmp)), plan->f(at));
                    all_reduce(plan, plan->f(at), 1, true, s);  // the mean over equal shards
                });
                break;
            }
            case Op::Embedding: {
                uint32_t table = in[0], ids = in[1];
                uint64_t n = rows_of(ids), rows = rows_of(table), h = cols_of(table);
                emit("embedding", nd, in, {at}, [=](cudaStream_t s) {
                    k::embedding(s, plan->in(table), plan->i(ids), plan->out(at), n, rows, h, plan->d_status);
                });
                // The gradient of this lookup sorts the same ids: that half of it needs nothing
                // else, so it is issued here (and runs beside the forward pass).
                if ((fusion_mask() & 8u) && P->slots[ids].kind == Slot::Input && !orders.count({ids, rows}))
                    for (uint32_t u : users[ids]) {
                        const Node& grad = node(u);
                        if (grad.op != Op::EmbeddingGrad || handled[u] || pos(grad.operands[0]) != ids || grad.rows != rows) continue;
                        uint32_t tmp = scratch(k::embedding_grad_scratch_ints(n, rows) * 4);
                        orders[{ids, rows}] = tmp;
                        emit("embedding_order", nd, {ids}, {tmp}, [=](cudaStream_t s) {
                            k::embedding_order(s, plan->i(ids), n, rows, plan->i(tmp), plan->d_status);
                        });
                        break;
                    }
                break;
            }
            case Op::EmbeddingGrad: {
                uint32_t ids = in[0], g = in[1];
                uint64_t n = rows_of(ids), rows = nd.rows, h = cols_of(g);
                auto ordered = orders.find({ids, rows});
                const bool have_order = ordered != orders.end();
                uint32_t tmp = have_order ? ordered->second : scratch(k::embedding_grad_scratch_ints(n, rows) * 4);
                // other + embedding_grad(...) with nothing else reading the scatter (a tied weight's
                // dense gradient plus its lookup gradient): the scatter adds `other` as it writes.
                bool is_output = false;
                for (const msx::Output& o : prog.outputs) is_output = is_output || pos(o.value) == at;
                if (!is_output && users[at].size() == 1) {
                    uint32_t u = users[at][0];
                    const Node& add = node(u);
                    if (add.op == Op::Add && !handled[u] && add.ty.count() == nd.ty.count()) {
                        uint32_t other = pos(add.operands[0]) == at ? pos(add.operands[1]) : pos(add.operands[0]);
                        if (other < at && other != at && node(other).ty.count() == nd.ty.count()) {
                            handled[u] = 1;
                            out.kind = Slot::Dead;
                            Slot& sum = P->slots[u];
                            make_arena(sum, add);
                            // `other` is read by this sum alone and was written by an earlier launch:
                            // it is stored where the sum goes, and the scatter touches only the rows
                            // some id names (a table of 30,522 rows read by 4,096 ids: an eighth).
                            if (users[other].size() == 1 && P->slots[other].kind == Slot::Arena && P->slots[other].pitch == 0 &&
                                !is_output_value(other) && node(other).ty.shape == add.ty.shape) {
                                P->slots[other].kind = Slot::View;
                                P->slots[other].index = u;
                            }
                            if (have_order)
                                emit("embedding_grad", nd, {g, other, tmp}, {u}, [=](cudaStream_t s) {
                                    k::embedding_scatter(s, plan->in(g), plan->out(u), n, rows, h, plan->i(tmp), plan->f(other));
                                });
                            else
                                emit("embedding_grad", nd, {ids, g, other}, {u, tmp}, [=](cudaStream_t s) {
                                    k::embedding_grad(s, plan->i(ids), plan->in(g), plan->out(u), n, rows, h, plan->i(tmp), plan->d_status,
                                                      plan->f(other));
                                });
                            break;
                        }
                    }
                }
                if (have_order)
                    emit("embedding_grad", nd, {g, tmp}, {at}, [=](cudaStream_t s) {
                        k::embedding_scatter(s, plan->in(g), plan->out(at), n, rows, h, plan->i(tmp));
                    });
                else
                    emit("embedding_grad", nd, in, {at, tmp}, [=](cudaStream_t s) {
                        k::embedding_grad(s, plan->i(ids), plan->in(g), plan->out(at), n, rows, h, plan->i(tmp), plan->d_status);
                    });
                break;
            }
            case Op::AddRows: {
                uint32_t x = in[0], b = in[1];
                uint64_t r = rows_of(x), h = cols_of(x);
                emit("add_rows", nd, in, {at}, [=](cudaStream_t s) { k::add_rows(s, plan->f(x), plan->f(b), plan->f(at), r, h); });
                break;
            }
            case Op::SumRows: {
                uint32_t g = in[0];
                uint64_t r = rows_of(g), h = cols_of(g), ld = pitch_of(g);
                if (deferrable(at) && r * std::max<uint64_t>(ld, h) * 4 <= kDeferredRowsBytes) {
                    uint32_t tmp = scratch(k::sum_rows_scratch_floats(r, h) * 4);
                    uint32_t source = g;
                    while (P->slots[source].kind == Slot::View) source = P->slots[source].index;
                    deferred_rows.push_back({source, tmp, r, h, ld});
                    deferred.push_back({tmp, 0, k::sum_rows_chunks(r), h, at});
                    break;
                }
                if (deferrable(at)) {
                    uint32_t tmp = scratch(k::sum_rows_scratch_floats(r, h) * 4);
                    emit("sum_rows", nd, in, {tmp}, [=](cudaStream_t s) { k::sum_rows(s, plan->in(g), r, h, plan->f(tmp), nullptr, nullptr, ld); });
                    deferred.push_back({tmp, 0, k::sum_rows_chunks(r), h, at});
                    break;
                }
                uint32_t tmp = scratch(k::sum_rows_scratch_floats(r, h) * 4), ctr = counters(k::sum_rows_counters(h));
                emit("sum_rows", nd, in, {at, tmp},
                     [=](cudaStream_t s) { k::sum_rows(s, plan->in(g), r, h, plan->f(tmp), plan->f(at), plan->counter(ctr), ld); });
                break;
            }
            case Op::LayerNorm: {
                uint32_t x = in[0], gamma = in[1], beta = in[2];
                uint64_t r = rows_of(x), h = cols_of(x);
                if (out.half) {
                    // bf16 rows go through the kernel of the fused tails, with nothing fused to it.
                    if (!k::layer_norm_backward_supported(h)) unsupported(nd, "a bf16 layer norm of rows longer than 1,024");
                    emit("layer_norm", nd, in, {at}, [=](cudaStream_t s) {
                        k::add_layer_norm(s, plan->in(x), k::In(), nullptr, plan->f(gamma), plan->f(beta), k::Out(), plan->out(at), nullptr, k::Out(), r, h);
                    });
                    break;
                }
                emit("layer_norm", nd, in, {at}, [=](cudaStream_t s) {
                    k::layer_norm(s, plan->f(x), plan->f(gamma), plan->f(beta), plan->f(at), r, h);
                });
                break;
            }
            case Op::LayerNormGradX: {
                if (schedule_layer_norm_backward(at)) break;
                uint32_t x = in[0], gamma = in[1], g = in[2];
                uint64_t r = rows_of(x), h = cols_of(x);
                emit("layer_norm_grad_x", nd, in, {at}, [=](cudaStream_t s) {
                    k::layer_norm_grad_x(s, plan->f(x), plan->f(gamma), plan->f(g), plan->f(at), r, h);
                });
                break;
            }
            case Op::LayerNormGradGamma: {
                if (schedule_layer_norm_backward(at)) break;
                uint32_t x = in[0], g = in[1];
                uint64_t r = rows_of(x), h = cols_of(x);
                // The beta gradient is the SumRows of the same adjoint: one pass gives both.
                int beta = -1;
                for (uint32_t u : users[g])
                    if (u > at && node(u).op == Op::SumRows && !handled[u]) { beta = static_cast<int>(u); break; }
                std::vector<uint32_t> writes = {at};
                if (beta >= 0) {
                    handled[static_cast<size_t>(beta)] = 1;
                    Slot& b = P->slots[static_cast<size_t>(beta)];
                    b.kind = Slot::Arena;
                    b.bytes = h * 4;
                    writes.push_back(static_cast<uint32_t>(beta));
                }
                uint32_t tmp = scratch(k::layer_norm_grad_gamma_scratch_floats(r, h) * 4);
                writes.push_back(tmp);
                emit("layer_norm_grad_gamma", nd, in, writes, [=](cudaStream_t s) {
                    k::layer_norm_grad_gamma(s, plan->f(x), plan->f(g), plan->f(tmp), plan->f(at),
                                             beta >= 0 ? plan->f(static_cast<uint32_t>(beta)) : nullptr, r, h);
                });
                break;
            }
            case Op::Softmax: {
                uint32_t x = in[0];
                uint64_t r = rows_of(x), c = cols_of(x);
                emit("softmax", nd, in, {at}, [=](cudaStream_t s) { k::softmax(s, plan->f(x), plan->f(at), r, c); });
                break;
            }
            case Op::SoftmaxGrad: {
                uint32_t y = in[0], g = in[1];
                uint64_t r = rows_of(y), c = cols_of(y);
                emit("softmax_grad", nd, in, {at}, [=](cudaStream_t s) { k::softmax_grad(s, plan->f(y), plan->f(g), plan->f(at), r, c); });
                break;
            }
            case Op::Attention:
            case Op::AttentionGradQ:
            case Op::AttentionGradK:
            case Op::AttentionGradV: schedule_attention(at); break;
            case Op::CrossEntropy: {
                uint32_t logits = in[0], labels = in[1], weights = in[2];
                uint64_t r = rows_of(logits), v = cols_of(logits), ld = pitch_of(logits);
                uint32_t row_loss = scratch(std::max<uint64_t>(r, 1) * 4), den = scratch(4);
                // The gradient op of the same loss reads the same row maxima and sums: when its
                // incoming adjoint is a constant (the seed), one pass over the logits gives both.
                int grad = -1;
                for (uint32_t u : users[logits]) {
                    const Node& other = node(u);
                    if (other.op != Op::CrossEntropyGrad || handled[u] || u < at) continue;
                    if (pos(other.operands[0]) != logits || pos(other.operands[1]) != labels || pos(other.operands[2]) != weights) continue;
                    if (P->slots[pos(other.operands[3])].kind != Slot::Const) continue;
                    grad = static_cast<int>(u);
                    break;
                }
                if (grad >= 0) {
                    uint32_t gpos = static_cast<uint32_t>(grad), seed = pos(node(gpos).operands[3]);
                    handled[gpos] = 1;
                    Slot& gs = P->slots[gpos];
                    make_arena(gs, node(gpos));
                    if (pitchable(gpos)) set_pitch(gpos);
                    const uint64_t ld_grad = gs.pitch;
                    uint32_t ctr = counters(1);
                    if (P->slots[weights].kind == Slot::Input && P->early_weights < 0) {
                        P->early_weights = static_cast<int>(weights);
                        P->early_rows = r;
                    }
                    emit("cross_entropy_with_grad", nd, {logits, labels, weights, seed}, {at, gpos, row_loss, den}, [=](cudaStream_t s) {
                        float* total = plan->f(den);
                        const bool side = plan->comm && plan->comm_stream && plan->early_weights == static_cast<int>(weights);
                        if (side) {
                            total = plan->d_weight_total;  // summed and reduced since the start of the step
                            cuda_ok(cudaStreamWaitEvent(s, plan->weights_summed, 0), "cudaStreamWaitEvent");
                        } else if (plan->comm) {
                            k::weight_sum(s, plan->f(weights), r, total);
                            all_reduce(plan, total, 1, false, s);
                        }
                        k::cross_entropy_with_grad(s, plan->in(logits), plan->i(labels), plan->f(weights), plan->f(seed), plan->comm != nullptr,
                                                   total, plan->f(row_loss), plan->f(at), plan->out(gpos), r, v, plan->counter(ctr), ld,
                                                   ld_grad);
                        if (side) {
                            cuda_ok(cudaEventRecord(plan->loss_ready, s), "cudaEventRecord");
                            cuda_ok(cudaStreamWaitEvent(plan->comm_stream, plan->loss_ready, 0), "cudaStreamWaitEvent");
                            all_reduce(plan, plan->f(at), 1, false, plan->comm_stream);
                            cuda_ok(cudaEventRecord(plan->loss_reduced, plan->comm_stream), "cudaEventRecord");
                            plan->loss_in_flight = true;
                        } else {
                            all_reduce(plan, plan->f(at), 1, false, s);
                        }
                    });
                    break;
                }
                emit("cross_entropy", nd, in, {at, row_loss, den}, [=](cudaStream_t s) {
                    if (plan->comm) {
                        // The shard's numerator over the whole batch's weight sum, then summed.
                        k::weight_sum(s, plan->f(weights), r, plan->f(den));
                        all_reduce(plan, plan->f(den), 1, false, s);
                    }
                    k::cross_entropy(s, plan->in(logits), plan->i(labels), plan->f(weights), plan->f(row_loss),
                                     plan->comm ? plan->f(den) : nullptr, plan->f(at), r, v, ld);
                    all_reduce(plan, plan->f(at), 1, false, s);
                });
                break;
            }
            case Op::CrossEntropyGrad: {
                uint32_t logits = in[0], labels = in[1], weights = in[2], g = in[3];
                uint64_t r = rows_of(logits), v = cols_of(logits), ld = pitch_of(logits);
                if (pitchable(at)) set_pitch(at);
                const uint64_t ld_out = out.pitch;
                uint32_t den = scratch(4);
                emit("cross_entropy_grad", nd, in, {at, den}, [=](cudaStream_t s) {
                    if (plan->comm) {
                        k::weight_sum(s, plan->f(weights), r, plan->f(den));
                        all_reduce(plan, plan->f(den), 1, false, s);
                    }
                    k::cross_entropy_grad(s, plan->f(logits), plan->i(labels), plan->f(weights), plan->f(g), plan->comm != nullptr,
                                          plan->f(den), plan->f(at), r, v, ld, ld_out);
                });
                break;
            }
            case Op::Dropout:
            case Op::DropoutGrad: {
                uint32_t x = nd.op == Op::Dropout ? in[0] : in[1], token = nd.op == Op::Dropout ? in[1] : in[0];
                if (nd.op == Op::DropoutGrad && adjoint_draw_joins(at)) {
                    // Drawn inside the layer-norm backward launch that alone reads it.
                    adjoint_draws.insert(at);
                    out.kind = Slot::Dead;
                    break;
                }
                if (nd.ty.count() > (1ull << 32)) unsupported(nd, "a dropout draw addresses at most 2^32 elements");
                uint32_t threshold = static_cast<uint32_t>(msx::dropout_keep_threshold(nd.p));
                float scale = 1.0f / (1.0f - nd.p);
                uint64_t row_width = nd.ty.rank() > 0 && nd.ty.shape[0] > 0 ? count / nd.ty.shape[0] : 1;
                // residual + dropout(x) followed by the layer norm of that sum (the tail of every
                // transformer sublayer): one launch writes the sum and its layer norm.
                if ((fusion_mask() & 1u) && nd.op == Op::Dropout && nd.ty.rank() == 2 && users[at].size() == 1 &&
                    k::layer_norm_backward_supported(nd.ty.shape[1])) {
                    bool is_output = false;
                    for (const msx::Output& o : prog.outputs) is_output = is_output || pos(o.value) == at;
                    const uint32_t add_at = users[at][0];
                    const Node& add = node(add_at);
                    int norm = -1;
                    if (!is_output && add.op == Op::Add && !handled[add_at] && add.ty.shape == nd.ty.shape) {
                        const uint32_t residual = pos(add.operands[0]) == at ? pos(add.operands[1]) : pos(add.operands[0]);
                        if (residual < at && node(residual).ty.shape == nd.ty.shape) {
                            for (uint32_t u : users[add_at]) {
                                const Node& ln = node(u);
                                if (ln.op == Op::LayerNorm && !handled[u] && pos(ln.operands[0]) == add_at && pos(ln.operands[1]) < at &&
                                    pos(ln.operands[2]) < at) { norm = static_cast<int>(u); break; }
                            }
                            if (norm >= 0) {
                                const uint32_t ln_at = static_cast<uint32_t>(norm);
                                const uint32_t gamma = pos(node(ln_at).operands[1]), beta = pos(node(ln_at).operands[2]);
                                handled[add_at] = handled[ln_at] = 1;
                                out.kind = Slot::Dead;
                                for (uint32_t made : {add_at, ln_at}) {
                                    Slot& slot = P->slots[made];
                                    make_arena(slot, node(made));
                                }
                                const uint64_t r = nd.ty.shape[0], h = nd.ty.shape[1];
                                Draw draw = draw_of(at);
                                std::vector<uint32_t> made = {add_at, ln_at};
                                const int bits = store_bits(draw, r, h);
                                if (bits >= 0) made.push_back(static_cast<uint32_t>(bits));
                                emit("dropout_add_layer_norm", nd, {x, token, residual, gamma, beta}, made, [=](cudaStream_t s) {
                                    const k::DropoutDraw first = launch_draw(plan, draw, h);
                                    k::add_layer_norm(s, plan->in(x), plan->in(residual), &first, plan->f(gamma), plan->f(beta), plan->out(add_at),
                                                      plan->out(ln_at), nullptr, k::Out(), r, h);
                                });
                                break;
                            }
                            // No layer norm reads the sum: residual + dropout(x) alone is one launch.
                            handled[add_at] = 1;
                            out.kind = Slot::Dead;
                            Slot& slot = P->slots[add_at];
                            make_arena(slot, add);
                            const uint64_t r = nd.ty.shape[0], h = nd.ty.shape[1];
                            Draw draw = draw_of(at);
                            std::vector<uint32_t> made = {add_at};
                            const int bits = store_bits(draw, r, h);
                            if (bits >= 0) made.push_back(static_cast<uint32_t>(bits));
                            emit("dropout_add", nd, {x, token, residual}, made, [=](cudaStream_t s) {
                                const k::DropoutDraw first = launch_draw(plan, draw, h);
                                k::add_layer_norm(s, plan->in(x), plan->in(residual), &first, nullptr, nullptr, plan->out(add_at), k::Out(), nullptr,
                                                  k::Out(), r, h);
                            });
                            break;
                        }
                    }
                }
                emit("dropout", nd, in, {at}, [=](cudaStream_t s) {
                    k::dropout(s, plan->in(x), plan->i(token), plan->seed, threshold, scale, plan->shard_rows_before * row_width,
                               plan->out(at), count);
                });
                break;
            }
            default: unsupported(nd, "no kernel is written for it");
        }
    }

    // Chains of Adds that only the gradients of one layer norm read (the sum of the three input
    // gradients of the Q, K, V projections and the residual path): the backward launch adds them
    // as it loads its adjoint, in the program's nesting order, and the sums are never stored.
    std::map<uint32_t, std::vector<uint32_t>> adjoint_sums;
    size_t addend_count(uint32_t at) const {
        size_t n = 0;
        for (uint32_t o : node(at).operands) {
            auto inner = adjoint_sums.find(pos(o));
            n += inner != adjoint_sums.end() ? inner->second.size() : 1;
        }
        return n;
    }
    bool joins_layer_norm_adjoint(uint32_t at, size_t carried = 0) const {
        const Node& nd = node(at);
        if (!(fusion_mask() & 2u) || nd.op != Op::Add || nd.ty.rank() != 2 || nd.operands.size() != 2) return false;
        for (uint32_t o : nd.operands)
            if (node(pos(o)).ty.shape != nd.ty.shape) return false;
        for (const msx::Output& o : prog.outputs)
            if (pos(o.value) == at) return false;
        const size_t addends = carried ? carried + 1 : addend_count(at);
        if (addends > 4 || users[at].empty()) return false;
        // Either the next Add of the chain ...
        if (users[at].size() == 1 && node(users[at][0]).op == Op::Add)
            return pos(node(users[at][0]).operands[0]) != pos(node(users[at][0]).operands[1]) && joins_layer_norm_adjoint(users[at][0], addends);
        // ... or the dropout_grad that the same launch applies to the sum as it loads it ...
        if (users[at].size() == 1 && node(users[at][0]).op == Op::DropoutGrad)
            return pos(node(users[at][0]).operands[1]) == at && adjoint_draw_joins(users[at][0]);
        // ... or exactly the three gradient ops of one layer norm, which one launch will take.
        return feeds_one_layer_norm_backward(at);
    }
    bool feeds_one_layer_norm_backward(uint32_t at) const {
        const Node& nd = node(at);
        if (nd.ty.rank() != 2 || !k::layer_norm_backward_supported(nd.ty.shape[1]) || users[at].size() != 3) return false;
        int dx = -1, dgamma = -1, dbeta = -1;
        for (uint32_t u : users[at]) {
            const Node& un = node(u);
            if (un.op == Op::LayerNormGradX && pos(un.operands[2]) == at && pos(un.operands[0]) != at && pos(un.operands[1]) != at) dx = static_cast<int>(u);
            else if (un.op == Op::LayerNormGradGamma && pos(un.operands[1]) == at && pos(un.operands[0]) != at) dgamma = static_cast<int>(u);
            else if (un.op == Op::SumRows) dbeta = static_cast<int>(u);
        }
        if (dx < 0 || dgamma < 0 || dbeta < 0) return false;
        return pos(node(static_cast<uint32_t>(dx)).operands[0]) == pos(node(static_cast<uint32_t>(dgamma)).operands[0]);
    }

    // a + b with the layer norm of the sum and, when dropout is all that reads the layer norm, that
    // dropout: one launch (the embedding sum of an encoder; every residual sum of a forward pass
    // without dropout). The sum is stored as the separate kernel stores it.
    bool schedule_add_layer_norm(uint32_t at) {
        const Node& nd = node(at);
        if (!(fusion_mask() & 1u) || nd.ty.rank() != 2 || !k::layer_norm_backward_supported(nd.ty.shape[1])) return false;
        const uint32_t a = pos(nd.operands[0]), b = pos(nd.operands[1]);
        if (node(a).ty.shape != nd.ty.shape || node(b).ty.shape != nd.ty.shape) return false;
        auto is_output = [&](uint32_t v) {
            for (const msx::Output& o : prog.outputs)
                if (pos(o.value) == v) return true;
            return false;
        };
        int norm = -1;
        for (uint32_t u : users[at]) {
            const Node& ln = node(u);
            if (ln.op == Op::LayerNorm && !handled[u] && pos(ln.operands[0]) == at && pos(ln.operands[1]) < at && pos(ln.operands[2]) < at) {
                norm = static_cast<int>(u);
                break;
            }
        }
        if (norm < 0) return false;
        const uint32_t ln_at = static_cast<uint32_t>(norm);
        const uint32_t gamma = pos(node(ln_at).operands[1]), beta = pos(node(ln_at).operands[2]);
        int dropout = -1;
        if (users[ln_at].size() == 1 && !is_output(ln_at)) {
            const uint32_t u = users[ln_at][0];
            const Node& d = node(u);
            if (d.op == Op::Dropout && !handled[u] && pos(d.operands[0]) == ln_at && node(pos(d.operands[1])).op == Op::Input &&
                d.ty.shape == nd.ty.shape && d.ty.count() <= (1ull << 32))
                dropout = static_cast<int>(u);
        }
        std::vector<uint32_t> reads = {a, b, gamma, beta}, writes = {at};
        Draw draw;
        handled[ln_at] = 1;
        if (dropout >= 0) {
            draw = draw_of(static_cast<uint32_t>(dropout));
            handled[static_cast<uint32_t>(dropout)] = 1;
            P->slots[ln_at].kind = Slot::Dead;
            reads.push_back(static_cast<uint32_t>(draw.token));
            writes.push_back(static_cast<uint32_t>(dropout));
        } else {
            writes.push_back(ln_at);
        }
        for (uint32_t made : writes) {
            Slot& slot = P->slots[made];
            make_arena(slot, node(made));
        }
        msx_plan* plan = P;
        const uint64_t r = nd.ty.shape[0], h = nd.ty.shape[1];
        if (dropout >= 0) {
            // The decisions of the dropout behind the layer norm, kept for its gradient.
            const int bits = store_bits(draw, r, h);
            if (bits >= 0) writes.push_back(static_cast<uint32_t>(bits));
        }
        emit(dropout >= 0 ? "add_layer_norm_dropout" : "add_layer_norm", nd, reads, writes, [=](cudaStream_t s) {
            const k::DropoutDraw second = launch_draw(plan, draw, h);
            k::add_layer_norm(s, plan->in(a), plan->in(b), nullptr, plan->f(gamma), plan->f(beta), plan->out(at),
                              dropout >= 0 ? k::Out() : plan->out(ln_at), dropout >= 0 ? &second : nullptr,
                              dropout >= 0 ? plan->out(static_cast<uint32_t>(dropout)) : k::Out(), r, h);
        });
        return true;
    }

    // The draw of a Dropout or DropoutGrad node as a fused launch takes it: the token's position
    // now, its address, the seed and the shard's first element when the launch is issued.
    struct Draw { int token = -1; uint32_t threshold = 0; float scale = 1.0f; int bits = -1; bool stored = false; };
    // The keep decisions a forward launch stored for the dropout_grad of the same site: by the
    // site's token input, the scratch slot of the bits and the shape they were drawn for.
    struct KeptBits { uint32_t slot; uint64_t rows, width; };
    std::map<int, KeptBits> kept_bits;
    // A forward launch that draws `d` on [rows, width] stores its decisions (fusion bit 64) when a
    // row kernel can hold them a word per lane; the returned scratch slot joins the launch's writes.
    int store_bits(Draw& d, uint64_t rows, uint64_t width) {
        if (!(fusion_mask() & 64u) || d.token < 0 || width % 32 != 0 || width > 1024 || rows == 0 || kept_bits.count(d.token)) return -1;
        const uint32_t slot = scratch(rows * width / 8);
        kept_bits[d.token] = {slot, rows, width};
        d.bits = static_cast<int>(slot);
        d.stored = false;
        return d.bits;
    }
    // The dropout_grad of a site whose decisions were stored reads them; the slot joins the reads.
    int stored_bits(Draw& d, uint64_t rows, uint64_t width) const {
        auto kept = d.token < 0 ? kept_bits.end() : kept_bits.find(d.token);
        if (kept == kept_bits.end() || kept->second.rows != rows || kept->second.width != width) return -1;
        d.bits = static_cast<int>(kept->second.slot);
        d.stored = true;
        return d.bits;
    }
    Draw draw_of(uint32_t dropout) const {
        const Node& d = node(dropout);
        Draw draw;
        draw.token = static_cast<int>(pos(d.operands[d.op == Op::Dropout ? 1 : 0]));
        draw.threshold = static_cast<uint32_t>(msx::dropout_keep_threshold(d.p));
        draw.scale = 1.0f / (1.0f - d.p);
        return draw;
    }
    static k::DropoutDraw launch_draw(msx_plan* plan, const Draw& d, uint64_t row_width) {
        k::DropoutDraw draw;
        if (d.token < 0) return draw;
        draw.token = plan->i(static_cast<uint32_t>(d.token));
        draw.seed = plan->seed;
        draw.threshold = d.threshold;
        draw.scale = d.scale;
        draw.index_base = plan->shard_rows_before * row_width;
        if (d.bits >= 0) {
            draw.bits = static_cast<uint32_t*>(plan->ptr(static_cast<uint32_t>(d.bits)));
            draw.stored = d.stored;
        }
        return draw;
    }

    // A dropout_grad that only the gradients of one layer norm read: the backward launch draws the
    // mask on the adjoint it loads, and the masked matrix is never stored.
    std::set<uint32_t> adjoint_draws;
    bool draw_is_fusable(const Node& nd) const {
        return (fusion_mask() & 16u) && nd.op == Op::DropoutGrad && nd.ty.rank() == 2 && nd.ty.count() <= (1ull << 32) &&
               node(pos(nd.operands[0])).op == Op::Input && node(pos(nd.operands[1])).ty.shape == nd.ty.shape;
    }
    bool adjoint_draw_joins(uint32_t at) const {
        if (!draw_is_fusable(node(at))) return false;
        for (const msx::Output& o : prog.outputs)
            if (pos(o.value) == at) return false;
        return feeds_one_layer_norm_backward(at);
    }

    // The gradients of one layer_norm (dx, dgamma and, as the column sums of the same adjoint,
    // dbeta) read the same two matrices: whichever of them comes first in the program takes the
    // others along in one launch. False when the row width has no one-launch kernel.
    bool schedule_layer_norm_backward(uint32_t at) {
        const Node& nd = node(at);
        const bool from_dx = nd.op == Op::LayerNormGradX;
        const uint32_t x = pos(nd.operands[0]), g = pos(nd.operands[from_dx ? 2 : 1]);
        const uint64_t r = node(x).ty.shape.at(0), h = node(x).ty.shape.at(1);
        if (!k::layer_norm_backward_supported(h)) return false;
        int dx = from_dx ? static_cast<int>(at) : -1, dgamma = from_dx ? -1 : static_cast<int>(at), dbeta = -1;
        int gamma = from_dx ? static_cast<int>(pos(nd.operands[1])) : -1;
        for (uint32_t u : users[x]) {
            if (u <= at || handled[u]) continue;
            const Node& other = node(u);
            if (dx < 0 && other.op == Op::LayerNormGradX && pos(other.operands[0]) == x && pos(other.operands[2]) == g &&
                pos(other.operands[1]) < at) {
                dx = static_cast<int>(u);
                gamma = static_cast<int>(pos(other.operands[1]));
            } else if (dgamma < 0 && other.op == Op::LayerNormGradGamma && pos(other.operands[0]) == x && pos(other.operands[1]) == g) {
                dgamma = static_cast<int>(u);
            }
        }
        if (dgamma >= 0)
            for (uint32_t u : users[g])
                if (u > at && node(u).op == Op::SumRows && !handled[u]) { dbeta = static_cast<int>(u); break; }
        // An adjoint that is an absorbed chain of Adds is read as its addends.
        // ... and one that is an absorbed dropout_grad as the operand of that, drawn while loading.
        Draw adjoint_draw, dx_draw;
        uint32_t source = g;
        if (adjoint_draws.count(g)) {
            adjoint_draw = draw_of(g);
            source = pos(node(g).operands[1]);
        }
        std::vector<uint32_t> adjoint = {source};
        auto summed = adjoint_sums.find(source);
        if (summed != adjoint_sums.end()) adjoint = summed->second;
        // dropout_grad of dx (the adjoint of the projection under this sublayer's dropout) is a
        // second output of the launch.
        int dropped = -1;
        if (dx >= 0)
            for (uint32_t u : users[static_cast<uint32_t>(dx)]) {
                const Node& un = node(u);
                if (handled[u] || !draw_is_fusable(un) || pos(un.operands[1]) != static_cast<uint32_t>(dx) || adjoint_draw_joins(u)) continue;
                dropped = static_cast<int>(u);
                dx_draw = draw_of(u);
                break;
            }
        // gelu_grad of dx (the dense layer before a gelu and this layer norm) takes that place
        // instead; a dx that nothing else reads is then not stored.
        int pre_activation = -1;
        bool store_dx = true;
        if (dx >= 0 && dropped < 0 && (fusion_mask() & 16u))
            for (uint32_t u : users[static_cast<uint32_t>(dx)]) {
                const Node& un = node(u);
                if (handled[u] || un.op != Op::GeluGrad || pos(un.operands[1]) != static_cast<uint32_t>(dx) ||
                    pos(un.operands[0]) >= at || pos(un.operands[0]) == static_cast<uint32_t>(dx) || un.ty.shape != node(x).ty.shape)
                    continue;
                dropped = static_cast<int>(u);
                pre_activation = static_cast<int>(pos(un.operands[0]));
                store_dx = users[static_cast<uint32_t>(dx)].size() > 1 || is_output_value(static_cast<uint32_t>(dx));
                break;
            }
        std::vector<uint32_t> reads = {x}, writes;
        reads.insert(reads.end(), adjoint.begin(), adjoint.end());
        if (gamma >= 0) reads.push_back(static_cast<uint32_t>(gamma));
        if (adjoint_draw.token >= 0) reads.push_back(static_cast<uint32_t>(adjoint_draw.token));
        if (dx_draw.token >= 0) reads.push_back(static_cast<uint32_t>(dx_draw.token));
        for (Draw* d : {&adjoint_draw, &dx_draw}) {
            const int bits = stored_bits(*d, r, h);
            if (bits >= 0) reads.push_back(static_cast<uint32_t>(bits));
        }
        if (pre_activation >= 0) reads.push_back(static_cast<uint32_t>(pre_activation));
        if (!store_dx) {
            handled[static_cast<uint32_t>(dx)] = 1;
            P->slots[static_cast<uint32_t>(dx)].kind = Slot::Dead;
        }
        const int stored_dx = store_dx ? dx : -1;
        for (int other : {stored_dx, dropped, dgamma, dbeta}) {
            if (other < 0) continue;
            uint32_t u = static_cast<uint32_t>(other);
            handled[u] = 1;
            Slot& slot = P->slots[u];
            make_arena(slot, node(u));
            writes.push_back(u);
        }
        uint32_t tmp = scratch(k::layer_norm_backward_scratch_floats(r, h) * 4);
        msx_plan* plan = P;
        auto at_or_null = [plan](int p) -> float* { return p >= 0 ? plan->f(static_cast<uint32_t>(p)) : nullptr; };
        auto in_or_null = [plan](int p) { return p >= 0 ? plan->in(static_cast<uint32_t>(p)) : k::In(); };
        auto out_or_null = [plan](int p) { return p >= 0 ? plan->out(static_cast<uint32_t>(p)) : k::Out(); };
        auto draw_now = [plan, h](const Draw& d) { return launch_draw(plan, d, h); };
        const bool defer = (dgamma < 0 || deferrable(static_cast<uint32_t>(dgamma))) && (dbeta < 0 || deferrable(static_cast<uint32_t>(dbeta)));
        if (defer) {
            // dx is written here; the column sums stay as chunk sums until the finalize launch.
            std::vector<uint32_t> now;
            if (stored_dx >= 0) now.push_back(static_cast<uint32_t>(stored_dx));
            if (dropped >= 0) now.push_back(static_cast<uint32_t>(dropped));
            now.push_back(tmp);
            const uint32_t chunks = k::layer_norm_backward_chunks(r, h);
            if (dgamma >= 0) deferred.push_back({tmp, 0, chunks, h, static_cast<uint32_t>(dgamma)});
            if (dbeta >= 0) deferred.push_back({tmp, static_cast<uint64_t>(chunks) * h, chunks, h, static_cast<uint32_t>(dbeta)});
            float* const wanted = reinterpret_cast<float*>(uintptr_t{1});  // only null or not is read
            emit("layer_norm_backward", nd, reads, now, [=](cudaStream_t s) {
                const k::DropoutDraw in_draw = draw_now(adjoint_draw), out_draw = draw_now(dx_draw);
                k::layer_norm_backward(s, plan->in(x), at_or_null(gamma), plan->in(adjoint[0]), out_or_null(stored_dx), plan->f(tmp), nullptr,
                                       dgamma >= 0 ? wanted : nullptr, dbeta >= 0 ? wanted : nullptr, r, h,
                                       adjoint.size() > 1 ? plan->in(adjoint[1]) : k::In(), adjoint.size() > 2 ? plan->in(adjoint[2]) : k::In(),
                                       adjoint.size() > 3 ? plan->in(adjoint[3]) : k::In(), in_draw.token ? &in_draw : nullptr,
                                       out_draw.token ? &out_draw : nullptr, out_or_null(dropped), in_or_null(pre_activation));
            });
            return true;
        }
        uint32_t ctr = counters(1);
        writes.push_back(tmp);
        emit("layer_norm_backward", nd, reads, writes, [=](cudaStream_t s) {
            const k::DropoutDraw in_draw = draw_now(adjoint_draw), out_draw = draw_now(dx_draw);
            k::layer_norm_backward(s, plan->in(x), at_or_null(gamma), plan->in(adjoint[0]), out_or_null(stored_dx), plan->f(tmp), plan->counter(ctr),
                                   at_or_null(dgamma), at_or_null(dbeta), r, h,
                                   adjoint.size() > 1 ? plan->in(adjoint[1]) : k::In(), adjoint.size() > 2 ? plan->in(adjoint[2]) : k::In(),
                                   adjoint.size() > 3 ? plan->in(adjoint[3]) : k::In(), in_draw.token ? &in_draw : nullptr,
                                   out_draw.token ? &out_draw : nullptr, out_or_null(dropped), in_or_null(pre_activation));
        });
        return true;
    }

    // A matrix whose width is not a multiple of 4 floats (a 30,522-wide logits matrix) is stored
    // with its pitch rounded up when every kernel that touches it takes a pitch: rows then start
    // on 128-byte boundaries and are read and written 16 bytes at a time. The padding is never
    // read as data.
    bool pitchable(uint32_t v) const {
        if (P->flags & MSX_PLAN_EXACT_MATMUL) return false;
        const msx::Type& t = node(v).ty;
        if (t.rank() != 2 || t.i32 || t.shape[1] % (mixed() ? 8 : 4) == 0 || t.shape[1] < 8) return false;
        for (const msx::Output& o : prog.outputs)
            if (pos(o.value) == v) return false;
        for (uint32_t u : users[v]) {
            const Node& un = node(u);
            bool ok = false;
            if (un.op == Op::MatMul || un.op == Op::SumRows) ok = true;
            if ((un.op == Op::CrossEntropy || un.op == Op::CrossEntropyGrad) && pos(un.operands[0]) == v) {
                ok = true;
                for (size_t i = 1; i < un.operands.size(); ++i) ok = ok && pos(un.operands[i]) != v;
            }
            if (un.op == Op::Transpose && P->slots[u].kind == Slot::View) ok = true;  // folded: read only by matmuls
            if (!ok) return false;
        }
        return true;
    }
    void set_pitch(uint32_t v) {
        const msx::Type& t = node(v).ty;
        Slot& s = P->slots[v];
        // Rows start on 128-byte boundaries: 16 bytes is what the kernels need, whole cache lines
        // per row segment is what the TMA stores of the products want (the bf16 logits product
        // writes its 101 MB in 27 us instead of 58).
        const uint64_t unit = s.half ? 64 : 32;
        s.pitch = static_cast<uint32_t>((t.shape[1] + unit - 1) / unit * unit);
        s.bytes = t.shape[0] * s.pitch * (s.half ? 2 : 4);
    }
    uint32_t pitch_of(uint32_t p) const {
        const Slot& s = P->slots[p];
        return s.kind == Slot::View ? pitch_of(s.index) : s.pitch;
    }

    // One product of a matmul launch: `result` = the node whose slot receives it (the AddRows node
    // when the bias rides in the epilogue), `flip_*` reads the operand as the transpose of what its
    // slot says.
    struct Product {
        uint32_t node, result, a, b;
        bool flip_a, flip_b;
        int bias;
    };

    // The product of MatMul node `at`, with add_rows(matmul(x, w), b) folded when nothing else
    // reads the product: the bias rides in the matmul's epilogue and the product is never stored.
    Product describe_product(uint32_t at) const {
        const Node& nd = node(at);
        Product p = {at, at, pos(nd.operands[0]), pos(nd.operands[1]), false, false, -1};
        bool is_output = false;
        for (const msx::Output& o : prog.outputs) is_output = is_output || pos(o.value) == at;
        if (!is_output && users[at].size() == 1) {
            uint32_t u = users[at][0];
            const Node& add = node(u);
            if (add.op == Op::AddRows && !handled[u] && pos(add.operands[0]) == at && pos(add.operands[1]) < at) {
                p.bias = static_cast<int>(pos(add.operands[1]));
                p.result = u;
            }
        }
        return p;
    }
    Product claim_product(uint32_t at) {
        Product p = describe_product(at);
        handled[at] = 1;
        Slot& own = P->slots[at];
        make_arena(own, node(at));
        if (p.result != at) {
            handled[p.result] = 1;
            own.kind = Slot::Dead;
            Slot& r = P->slots[p.result];
            make_arena(r, node(p.result));
        }
        return p;
    }
    // Whether the storage behind operand position `p` exists before node `before` is scheduled.
    bool ready_before(uint32_t p, uint32_t before) const {
        const Slot& s = P->slots[p];
        if (s.kind == Slot::View) return ready_before(s.index, before);
        return p < before;
    }
    bool joins(uint32_t later, const Product& first, uint32_t at, uint64_t m, uint64_t n, uint64_t kk) const {
        const Node& nd = node(later);
        if (!live[later] || handled[later] || nd.op != Op::MatMul) return false;
        if (nd.ty.shape[0] != m || nd.ty.shape[1] != n || node(pos(nd.operands[0])).ty.shape.at(1) != kk) return false;
        Product p = describe_product(later);
        if (!ready_before(p.a, at) || !ready_before(p.b, at)) return false;
        if (pitch_of(p.a) || pitch_of(p.b) || pitchable(p.result)) return false;
        if (P->transposed(p.a) != P->transposed(first.a) || P->transposed(p.b) != P->transposed(first.b)) return false;
        if ((p.bias >= 0) != (first.bias >= 0)) return false;
        if (p.bias >= 0 && static_cast<uint32_t>(p.bias) >= at) return false;
        // A split k is either reduced by the launch or left for the finalize launch: one rule per launch.
        return deferrable(p.result) == deferrable(first.result);
    }

    // C[m, n] = op(a) x op(b) for every product of `group` (one shape, one storage form): the exact
    // f32 chain kernel under MSX_PLAN_EXACT_MATMUL (one product), else the tensor cores.
    void emit_matmul(const Node& nd, const std::vector<Product>& group, uint64_t m, uint64_t n, uint64_t kk) {
        msx_plan* plan = P;
        std::vector<uint32_t> reads, writes;
        for (const Product& p : group) {
            reads.push_back(p.a);
            reads.push_back(p.b);
            if (p.bias >= 0) reads.push_back(static_cast<uint32_t>(p.bias));
        }
        const Product first = group[0];
        const bool a_t_flip = first.flip_a, b_t_flip = first.flip_b;
        if (mixed()) {
            emit_matmul_bf16(nd, first, reads, m, n, kk);
            return;
        }
        if (P->flags & MSX_PLAN_EXACT_MATMUL) {
            const uint32_t a = first.a, b = first.b, at = first.result;
            const int bias = first.bias;
            Launch& l = emit("matmul", nd, reads, {at}, [=](cudaStream_t s) {
                k::matmul(s, plan->f(a), plan->transposed(a) != a_t_flip, plan->f(b), plan->transposed(b) != b_t_flip, plan->f(at), m, n, kk,
                          bias >= 0 ? plan->f(static_cast<uint32_t>(bias)) : nullptr);
            });
            l.flop = 2 * m * n * kk;
            return;
        }
        const uint32_t count = static_cast<uint32_t>(group.size());
        // (The same rule as the launch applies: the 128 x 128 tile wants TMA sources; every base
        // in a plan is on 256 bytes, so the row pitches decide.)
        const bool a_stored_t = P->transposed(first.a) != first.flip_a, b_stored_t = P->transposed(first.b) != first.flip_b;
        const uint64_t a_pitch = pitch_of(first.a) ? pitch_of(first.a) : (a_stored_t ? m : kk);
        const uint64_t b_pitch = pitch_of(first.b) ? pitch_of(first.b) : (b_stored_t ? kk : n);
        const k::MatmulTcPlan tc = k::matmul_tc_plan(m, n, kk, 1, count, a_pitch % 4 == 0 && b_pitch % 4 == 0);
        // A split k whose sum only the optimizer reads (a weight gradient) stays as partial
        // tiles: the finalize launch adds them with every other deferred sum.
        const bool defer = tc.workspace_floats != 0 && first.bias < 0 && deferrable(first.result);
        k::MatmulPitches pitches;
        pitches.a = pitch_of(first.a);
        pitches.b = pitch_of(first.b);
        if (count == 1 && tc.splits == 1 && pitchable(first.result)) {
            set_pitch(first.result);
            pitches.c = P->slots[first.result].pitch;
        }
        const std::vector<Product>& products = group;
        std::vector<int> workspaces;
        for (const Product& p : products) {
            int ws = -1;
            if (tc.workspace_floats) {
                ws = static_cast<int>(scratch(tc.workspace_floats * 4));
                writes.push_back(static_cast<uint32_t>(ws));
            }
            workspaces.push_back(ws);
            if (defer) deferred.push_back({static_cast<uint32_t>(ws), 0, tc.splits, m * n, p.result});
            else writes.push_back(p.result);
        }
        Launch& l = emit("matmul", nd, reads, writes, [=](cudaStream_t s) {
            k::MatmulOperands operands[4];
            for (uint32_t g = 0; g < count; ++g) {
                const Product& p = products[g];
                operands[g].a = plan->f(p.a);
                operands[g].b = plan->f(p.b);
                operands[g].c = plan->f(p.result);
                operands[g].bias = p.bias >= 0 ? plan->f(static_cast<uint32_t>(p.bias)) : nullptr;
                operands[g].workspace = workspaces[g] >= 0 ? plan->f(static_cast<uint32_t>(workspaces[g])) : nullptr;
            }
            k::matmul_tc_group(s, operands, count, plan->transposed(first.a) != a_t_flip, plan->transposed(first.b) != b_t_flip, m, n, kk,
                               plan->d_status, defer, pitches);
        });
        l.flop = 2 * m * n * kk * count;
    }

    // Attention and its gradients of a mixed-precision plan: the batched products on the bf16
    // kernel, probabilities kept as bf16 from the forward launch to the backward one, scores and
    // their adjoints as an f32 scratch matrix that lives inside one launch group.
    void schedule_attention_bf16(uint32_t at, k::AttentionShape shape, uint64_t pair_flop) {
        const Node& nd = node(at);
        msx_plan* plan = P;
        const uint32_t q = pos(nd.operands[0]), kk = pos(nd.operands[1]), v = pos(nd.operands[2]), mask = pos(nd.operands[3]);
        if (shape.k_len % 8 != 0 || shape.head_dim % 8 != 0) unsupported(nd, "a bf16 plan needs key counts and head widths that are multiples of 8");
        for (uint32_t operand : {q, kk, v})
            if (!P->half(operand)) unsupported(nd, "a bf16 plan's attention reads bf16 activations");
        // One kernel forward (O and the softmax statistics), one kernel for the three gradients,
        // when the shape fits them and the forward of the same attention is in the program.
        const std::array<uint32_t, 5> key = {q, kk, v, mask, static_cast<uint32_t>(nd.heads)};
        const bool fused = (fusion_mask() & 32u) && k::attention_fused_supported(shape);
        if (fused && nd.op == Op::Attention) {
            const uint32_t stats = scratch(k::attention_fused_stats_floats(shape) * 4);
            fused_forward[key] = {stats, at};
            Launch& l = emit("attention_forward", nd, {q, kk, v, mask}, {at, stats}, [=](cudaStream_t s) {
                k::attention_fused_forward(s, plan->ptr(q), plan->ptr(kk), plan->ptr(v), plan->f(mask), plan->ptr(at), plan->f(stats), shape,
                                           plan->d_status);
            });
            l.flop = 2 * pair_flop;
            return;
        }
        if (fused && nd.op != Op::Attention && fused_forward.count(key)) {
            const uint32_t g = pos(nd.operands[4]);
            if (!P->half(g)) unsupported(nd, "a bf16 plan's attention reads bf16 activations");
            const uint32_t stats = fused_forward[key].first, o = fused_forward[key].second;
            int dq = -1, dk = -1, dv = -1;
            for (uint32_t u : users[g]) {
                const Node& other = node(u);
                if (handled[u] && u != at) continue;
                if (other.op != Op::AttentionGradQ && other.op != Op::AttentionGradK && other.op != Op::AttentionGradV) continue;
                if (other.operands != nd.operands || other.heads != nd.heads) continue;
                int& target = other.op == Op::AttentionGradQ ? dq : other.op == Op::AttentionGradK ? dk : dv;
                if (target < 0) target = static_cast<int>(u);
            }
            std::vector<uint32_t> writes;
            for (int t : {dq, dk, dv})
                if (t >= 0) {
                    handled[static_cast<size_t>(t)] = 1;
                    make_arena(P->slots[static_cast<size_t>(t)], node(static_cast<uint32_t>(t)));
                    writes.push_back(static_cast<uint32_t>(t));
                }
            auto or_null = [plan](int p) -> void* { return p >= 0 ? plan->ptr(static_cast<uint32_t>(p)) : nullptr; };
            Launch& l = emit("attention_backward", nd, {q, kk, v, mask, g, stats, o}, writes, [=](cudaStream_t s) {
                k::attention_fused_backward(s, plan->ptr(q), plan->ptr(kk), plan->ptr(v), plan->f(mask), plan->ptr(g), plan->ptr(o),
                                            plan->f(stats), or_null(dq), or_null(dk), or_null(dv), shape, plan->d_status);
            });
            l.flop = pair_flop * 5;
            return;
        }
        const uint64_t count = k::attention_tc_scratch_floats(shape);
        auto half_scratch = [&](void) {
            const uint32_t slot = scratch(count * 2);
            P->slots[slot].half = true;
            return slot;
        };
        if (nd.op == Op::Attention) {
            const uint32_t probs = half_scratch(), scores = scratch(count * 4);
            forward_probabilities[{q, kk, v, mask, static_cast<uint32_t>(nd.heads)}] = probs;
            Launch& l = emit("attention_forward", nd, {q, kk, v, mask}, {at, probs, scores}, [=](cudaStream_t s) {
                k::attention_bf16_forward(s, plan->ptr(q), plan->ptr(kk), plan->ptr(v), plan->f(mask), plan->ptr(at), plan->ptr(probs),
                                          plan->f(scores), shape, plan->d_status);
            });
            l.flop = 2 * pair_flop;
            return;
        }
        const uint32_t g = pos(nd.operands[4]);
        if (!P->half(g)) unsupported(nd, "a bf16 plan's attention reads bf16 activations");
        int dq = -1, dk = -1, dv = -1;
        for (uint32_t u : users[g]) {
            const Node& other = node(u);
            if (handled[u] && u != at) continue;
            if (other.op != Op::AttentionGradQ && other.op != Op::AttentionGradK && other.op != Op::AttentionGradV) continue;
            if (other.operands != nd.operands || other.heads != nd.heads) continue;
            int& target = other.op == Op::AttentionGradQ ? dq : other.op == Op::AttentionGradK ? dk : dv;
            if (target < 0) target = static_cast<int>(u);
        }
        std::vector<uint32_t> reads = {q, kk, v, mask, g}, writes;
        for (int t : {dq, dk, dv})
            if (t >= 0) {
                handled[static_cast<size_t>(t)] = 1;
                make_arena(P->slots[static_cast<size_t>(t)], node(static_cast<uint32_t>(t)));
                writes.push_back(static_cast<uint32_t>(t));
            }
        auto kept = forward_probabilities.find({q, kk, v, mask, static_cast<uint32_t>(nd.heads)});
        const bool p_ready = kept != forward_probabilities.end();
        const uint32_t probs = p_ready ? kept->second : half_scratch();
        const uint32_t dscores = half_scratch(), scores = scratch(count * 4);
        writes.push_back(dscores);
        writes.push_back(scores);
        if (p_ready) reads.push_back(probs);
        else writes.push_back(probs);
        auto or_null = [plan](int p) -> void* { return p >= 0 ? plan->ptr(static_cast<uint32_t>(p)) : nullptr; };
        Launch& l = emit("attention_backward", nd, reads, writes, [=](cudaStream_t s) {
            k::attention_bf16_backward(s, plan->ptr(q), plan->ptr(kk), plan->ptr(v), plan->f(mask), plan->ptr(g), or_null(dq), or_null(dk),
                                       or_null(dv), plan->ptr(probs), plan->ptr(dscores), plan->f(scores), shape, plan->d_status, p_ready);
        });
        l.flop = pair_flop * (1 + (dv >= 0) + ((dq >= 0 || dk >= 0) ? 1 : 0) + (dq >= 0) + (dk >= 0));
    }

    // The product of a mixed-precision plan: bf16 operands in place (an activation, or the working
    // copy of a parameter), the result in the storage type of its slot, a split k reduced by the
    // launch or, for a weight gradient, left as f32 partial tiles for the finalize launch.
    void emit_matmul_bf16(const Node& nd, const Product& p, const std::vector<uint32_t>& reads, uint64_t m, uint64_t n, uint64_t kk) {
        msx_plan* plan = P;
        for (uint32_t operand : {p.a, p.b}) {
            uint32_t home = operand;
            while (P->slots[home].kind == Slot::View) home = P->slots[home].index;
            const Slot& slot = P->slots[home];
            const bool ok = (slot.kind == Slot::Arena && slot.half) || (slot.kind == Slot::Param && node(home).ty.rank() == 2);
            if (!ok) unsupported(nd, "a bf16 plan multiplies bf16 activations and matrix parameters; %" + std::to_string(node(home).id) + " is neither");
        }
        const k::MatmulBf16Plan tc = k::matmul_bf16_plan(m, n, kk);
        const bool defer = tc.workspace_floats != 0 && p.bias < 0 && deferrable(p.result);
        if (pitchable(p.result)) set_pitch(p.result);
        std::vector<uint32_t> writes;
        int ws = -1;
        if (tc.workspace_floats) {
            ws = static_cast<int>(scratch(tc.workspace_floats * 4));
            writes.push_back(static_cast<uint32_t>(ws));
        }
        if (defer) deferred.push_back({static_cast<uint32_t>(ws), 0, tc.splits, m * n, p.result});
        else writes.push_back(p.result);
        const bool a_t = P->transposed(p.a) != p.flip_a, b_t = P->transposed(p.b) != p.flip_b;
        const uint32_t a_pitch = pitch_of(p.a) ? pitch_of(p.a) : static_cast<uint32_t>(a_t ? m : kk);
        const uint32_t b_pitch = pitch_of(p.b) ? pitch_of(p.b) : static_cast<uint32_t>(b_t ? kk : n);
        const uint32_t c_pitch = P->slots[p.result].pitch;
        const uint32_t a = p.a, b = p.b, result = p.result;
        const int bias = p.bias;
        Launch& l = emit("matmul", nd, reads, writes, [=](cudaStream_t s) {
            const k::HalfMatrix A = {plan->h16(a), a_pitch, 0, 0, a_t};
            const k::HalfMatrix B = {plan->h16(b), b_pitch, 0, 0, b_t};
            const k::HalfResult C = {plan->ptr(result), plan->half(result), c_pitch, 0, 0};
            if (!A.base || !B.base) throw StatusError(MSX_LAUNCH_FAILED, "a matmul operand of a bf16 plan has no bf16 storage");
            k::matmul_bf16(s, A, B, C, m, n, kk, 1, 1, ws >= 0 ? plan->f(static_cast<uint32_t>(ws)) : nullptr,
                           bias >= 0 ? plan->f(static_cast<uint32_t>(bias)) : nullptr, plan->d_status, defer);
        });
        l.flop = 2 * m * n * kk;
    }

    std::map<std::array<uint32_t, 5>, uint32_t> forward_probabilities;  // (q, k, v, mask, heads) -> scratch slot
    std::map<std::array<uint32_t, 5>, std::pair<uint32_t, uint32_t>> fused_forward;  // -> (statistics scratch, the forward's output)
    std::map<std::pair<uint32_t, uint64_t>, uint32_t> orders;           // (ids, table rows) -> scratch slot of the sorted occurrences

    void schedule_attention(uint32_t at) {
        const Node& nd = node(at);
        msx_plan* plan = P;
        uint32_t q = pos(nd.operands[0]), kk = pos(nd.operands[1]), v = pos(nd.operands[2]), mask = pos(nd.operands[3]);
        const msx::Type& qt = node(q).ty;
        const msx::Type& mt = node(mask).ty;
        k::AttentionShape shape;
        shape.batch = static_cast<uint32_t>(mt.shape[0]);
        shape.k_len = static_cast<uint32_t>(mt.shape[1]);
        shape.q_len = static_cast<uint32_t>(qt.shape[0] / mt.shape[0]);
        shape.heads = static_cast<uint32_t>(nd.heads);
        shape.head_dim = static_cast<uint32_t>(qt.shape[1] / nd.heads);
        if (shape.k_len > 512) unsupported(nd, "more than 512 keys per sequence");
        if (shape.head_dim > 128) unsupported(nd, "a head wider than 128");
        const bool simt = (P->flags & MSX_PLAN_EXACT_MATMUL) != 0;
        const uint64_t pair_flop = 2ull * shape.batch * shape.q_len * shape.k_len * shape.heads * shape.head_dim;
        if (mixed()) {
            schedule_attention_bf16(at, shape, pair_flop);
            return;
        }
        if (nd.op == Op::Attention) {
            if (simt) {
                Launch& l = emit("attention_forward", nd, {q, kk, v, mask}, {at}, [=](cudaStream_t s) {
                    k::attention_forward(s, plan->f(q), plan->f(kk), plan->f(v), plan->f(mask), plan->f(at), shape);
                });
                l.flop = 2 * pair_flop;
            } else {
                uint32_t probs = scratch(k::attention_tc_scratch_floats(shape) * 4);
                // The backward of the same attention reads these probabilities instead of
                // computing them again: the scratch then lives until that launch.
                forward_probabilities[{q, kk, v, mask, static_cast<uint32_t>(nd.heads)}] = probs;
                Launch& l = emit("attention_forward", nd, {q, kk, v, mask}, {at, probs}, [=](cudaStream_t s) {
                    k::attention_tc_forward(s, plan->f(q), plan->f(kk), plan->f(v), plan->f(mask), plan->f(at), plan->f(probs), shape,
                                            plan->d_status);
                });
                l.flop = 2 * pair_flop;
            }
            return;
        }
        // The gradient ops of one attention read the same five operands: one launch group
        // recomputes the probabilities once for all three.
        uint32_t g = pos(nd.operands[4]);
        int dq = -1, dk = -1, dv = -1;
        for (uint32_t u : users[g]) {
            const Node& other = node(u);
            if (handled[u] && u != at) continue;
            if (other.op != Op::AttentionGradQ && other.op != Op::AttentionGradK && other.op != Op::AttentionGradV) continue;
            if (other.operands != nd.operands || other.heads != nd.heads) continue;
            int& target = other.op == Op::AttentionGradQ ? dq : other.op == Op::AttentionGradK ? dk : dv;
            if (target < 0) target = static_cast<int>(u);
        }
        for (int t : {dq, dk, dv})
            if (t >= 0) {
                handled[static_cast<size_t>(t)] = 1;
                Slot& s = P->slots[static_cast<size_t>(t)];
                make_arena(s, node(static_cast<uint32_t>(t)));
            }
        std::vector<uint32_t> reads = {q, kk, v, mask, g};
        if (!simt) {
            auto kept = forward_probabilities.find({q, kk, v, mask, static_cast<uint32_t>(nd.heads)});
            const bool p_ready = kept != forward_probabilities.end();
            uint32_t probs = p_ready ? kept->second : scratch(k::attention_tc_scratch_floats(shape) * 4);
            uint32_t dprobs = scratch(k::attention_tc_scratch_floats(shape) * 4);
            std::vector<uint32_t> writes = {dprobs};
            if (p_ready) reads.push_back(probs);
            else writes.push_back(probs);
            for (int t : {dq, dk, dv})
                if (t >= 0) writes.push_back(static_cast<uint32_t>(t));
            Launch& l = emit("attention_backward", nd, reads, writes, [=](cudaStream_t s) {
                k::attention_tc_backward(s, plan->f(q), plan->f(kk), plan->f(v), plan->f(mask), plan->f(g),
                                         dq >= 0 ? plan->f(static_cast<uint32_t>(dq)) : nullptr,
                                         dk >= 0 ? plan->f(static_cast<uint32_t>(dk)) : nullptr,
                                         dv >= 0 ? plan->f(static_cast<uint32_t>(dv)) : nullptr, plan->f(probs), plan->f(dprobs), shape,
                                         plan->d_status, p_ready);
            });
            l.flop = pair_flop * (1 + (dv >= 0) + ((dq >= 0 || dk >= 0) ? 1 : 0) + (dq >= 0) + (dk >= 0));
            return;
        }
        uint32_t stats = scratch(k::attention_stats_floats(shape) * 4);
        {
            std::vector<uint32_t> writes = {stats};
            if (dq >= 0) writes.push_back(static_cast<uint32_t>(dq));
            Launch& l = emit("attention_grad_q", nd, reads, writes, [=](cudaStream_t s) {
                k::attention_grad_q(s, plan->f(q), plan->f(kk), plan->f(v), plan->f(mask), plan->f(g), plan->f(stats),
                                    dq >= 0 ? plan->f(static_cast<uint32_t>(dq)) : nullptr, shape);
            });
            l.flop = pair_flop * (dq >= 0 ? 3 : 2);
        }
        if (dk >= 0 || dv >= 0) {
            std::vector<uint32_t> kv_reads = reads, writes;
            kv_reads.push_back(stats);
            if (dk >= 0) writes.push_back(static_cast<uint32_t>(dk));
            if (dv >= 0) writes.push_back(static_cast<uint32_t>(dv));
            Launch& l = emit("attention_grad_kv", nd, kv_reads, writes, [=](cudaStream_t s) {
                k::attention_grad_kv(s, plan->f(q), plan->f(kk), plan->f(v), plan->f(mask), plan->f(g), plan->f(stats),
                                     dk >= 0 ? plan->f(static_cast<uint32_t>(dk)) : nullptr,
                                     dv >= 0 ? plan->f(static_cast<uint32_t>(dv)) : nullptr, shape);
            });
            l.flop = pair_flop * 4;
        }
    }
};

// ---------------------------------------------------------------------------------------------
// Arena placement by liveness: launches run in order on one stream, so a value's storage is free
// after the last launch that reads it.

struct FreeList {
    std::vector<std::pair<uint64_t, uint64_t>> blocks;  // (offset, size), sorted by offset
    uint64_t end = 0;

    uint64_t take(uint64_t bytes) {
        bytes = align_up(bytes);
        for (size_t b = 0; b < blocks.size(); ++b)
            if (blocks[b].second >= bytes) {
                uint64_t at = blocks[b].first;
                blocks[b].first += bytes;
                blocks[b].second -= bytes;
                if (blocks[b].second == 0) blocks.erase(blocks.begin() + static_cast<long>(b));
                return at;
            }
        // Grow: extend a free block that touches the end, else append.
        if (!blocks.empty() && blocks.back().first + blocks.back().second == end) {
            uint64_t at = blocks.back().first;
            end = at + bytes;
            blocks.pop_back();
            return at;
        }
        uint64_t at = end;
        end += bytes;
        return at;
    }
    void give(uint64_t offset, uint64_t bytes) {
        bytes = align_up(bytes);
        auto it = std::lower_bound(blocks.begin(), blocks.end(), std::make_pair(offset, uint64_t{0}));
        it = blocks.insert(it, {offset, bytes});
        if (it + 1 != blocks.end() && it->first + it->second == (it + 1)->first) {
            it->second += (it + 1)->second;
            blocks.erase(it + 1);
        }
        if (it != blocks.begin() && (it - 1)->first + (it - 1)->second == it->first) {
            (it - 1)->second += it->second;
            blocks.erase(it);
        }
    }
};

void place_arena(msx_plan* P) {
    std::vector<Slot>& slots = P->slots;
    // A value stored as another one is that one, wherever a launch names it.
    auto stored_as = [&slots](uint32_t v) {
        while (slots[v].kind == Slot::View) v = slots[v].index;
        return v;
    };
    for (Launch& launch : P->launches) {
        for (uint32_t& w : launch.writes) w = stored_as(w);
        for (uint32_t& r : launch.reads) r = stored_as(r);
    }
    for (size_t l = 0; l < P->launches.size(); ++l) {
        const Launch& launch = P->launches[l];
        for (uint32_t w : launch.writes)
            if (slots[w].kind == Slot::Arena) {
                if (slots[w].first < 0) slots[w].first = static_cast<int>(l);
                slots[w].last = std::max(slots[w].last, static_cast<int>(l));
                slots[w].last_write = std::max(slots[w].last_write, static_cast<int>(l));
            }
        for (uint32_t r : launch.reads)
            if (slots[r].kind == Slot::Arena) {
                if (slots[r].first < 0)
                    throw StatusError(MSX_UNSUPPORTED, "scheduling bug: launch " + std::to_string(l) + " (" + launch.kernel +
                                                           ") reads a value no earlier launch wrote");
                slots[r].last = std::max(slots[r].last, static_cast<int>(l));
            }
    }
    // A launch on the side stream may still be running until the launch that waits for it: what it
    // reads and writes stays allocated until then.
    for (const Launch& launch : P->launches) {
        if (launch.join_before < 0) continue;
        for (const std::vector<uint32_t>* touched : {&launch.reads, &launch.writes})
            for (uint32_t t : *touched)
                if (slots[t].kind == Slot::Arena) slots[t].last = std::max(slots[t].last, launch.join_before);
    }
    // Gradients live side by side, in the order the step produces them, so that a bucket of
    // consecutive gradients is one contiguous all-reduce.
    std::vector<char> is_gradient(slots.size(), 0);
    P->gradient_slots.clear();
    for (const msx::Output& o : P->program.outputs)
        if (o.role == Role::Gradient) {
            int at = P->program.position(o.value);
            if (at >= 0 && slots[static_cast<size_t>(at)].kind == Slot::Arena && slots[static_cast<size_t>(at)].first >= 0 &&
                !is_gradient[static_cast<size_t>(at)]) {
                is_gradient[static_cast<size_t>(at)] = 1;
                P->gradient_slots.push_back(static_cast<uint32_t>(at));
            }
        }
    std::stable_sort(P->gradient_slots.begin(), P->gradient_slots.end(),
                     [&](uint32_t a, uint32_t b) { return slots[a].first < slots[b].first; });
    std::vector<std::vector<uint32_t>> starts(P->launches.size()), ends(P->launches.size());
    for (uint32_t s = 0; s < slots.size(); ++s)
        if (slots[s].kind == Slot::Arena && slots[s].first >= 0 && !is_gradient[s]) {
            starts[static_cast<size_t>(slots[s].first)].push_back(s);
            if (!slots[s].keep) ends[static_cast<size_t>(slots[s].last)].push_back(s);
            P->unshared_bytes += align_up(slots[s].bytes);
        }
    // MSX_PLAN_GUARD: every value keeps storage of its own for the whole step, followed by 64
    // bytes of a sentinel that no kernel may touch (msx_plan_check_guards looks at them).
    const bool guarded_plan = (P->flags & MSX_PLAN_GUARD) != 0;
    FreeList free;
    for (size_t l = 0; l < P->launches.size(); ++l) {
        for (uint32_t s : starts[l]) slots[s].offset = free.take(slots[s].bytes + (guarded_plan ? kGuardBytes : 0));
        if (!guarded_plan)
            for (uint32_t s : ends[l]) free.give(slots[s].offset, slots[s].bytes);
    }
    P->gradient_region_offset = align_up(free.end);
    uint64_t at = P->gradient_region_offset;
    for (uint32_t g : P->gradient_slots) {
        slots[g].offset = at;
        at += align_up(slots[g].bytes + (guarded_plan ? kGuardBytes : 0));
        P->unshared_bytes += align_up(slots[g].bytes);
    }
    P->gradient_region_bytes = at - P->gradient_region_offset;
    P->arena_bytes = std::max<uint64_t>(at, kAlign);
    for (size_t l = 0; l < P->launches.size(); ++l)
        if (P->launches[l].kernel == "adamw_multi_tensor" || P->launches[l].kernel == "sgd_multi_tensor") P->optimizer_launch = static_cast<int>(l);
}

// Cuts the gradient region into buckets of about `bucket_bytes`, each closed by the launch that
// writes its last gradient.
void plan_buckets(msx_plan* P) {
    P->buckets.clear();
    Bucket open;
    bool any = false;
    for (uint32_t g : P->gradient_slots) {
        const Slot& s = P->slots[g];
        if (!any) {
            open = Bucket{};
            open.offset = s.offset;
            any = true;
        }
        open.bytes = s.offset + align_up(s.bytes) - open.offset;
        open.after_launch = std::max(open.after_launch, s.last_write);
        if (open.bytes >= P->bucket_bytes) {
            P->buckets.push_back(open);
            any = false;
        }
    }
    if (any) P->buckets.push_back(open);
}

// cudaMalloc for a plan, counted (device_allocations, peak_device_bytes of the run statistics).
template <class T> cudaError_t plan_malloc(msx_plan* P, T** out, size_t bytes) {
    cudaError_t e = cudaMalloc(out, bytes);
    if (e == cudaSuccess) {
        ++P->device_allocations;
        P->device_bytes += bytes;
    }
    return e;
}

void allocate(msx_plan* P, const Scheduler& sched) {
    const Program& prog = P->program;
    cuda_ok(cudaStreamCreateWithFlags(&P->stream, cudaStreamNonBlocking), "cudaStreamCreate");
    cuda_ok(plan_malloc(P, &P->arena, P->arena_bytes), "cudaMalloc(arena)");
    // The gaps between gradients are summed with them across ranks: keep them finite.
    if (P->gradient_region_bytes)
        cuda_ok(cudaMemset(P->arena + P->gradient_region_offset, 0, P->gradient_region_bytes), "cudaMemset(gradients)");
    if (P->flags & MSX_PLAN_GUARD) {
        std::vector<uint32_t> sentinel(kGuardBytes / 4, kGuardWord);
        for (const Slot& s : P->slots)
            if (s.kind == Slot::Arena && s.first >= 0)
                cuda_ok(cudaMemcpy(P->arena + s.offset + (s.bytes + 3) / 4 * 4, sentinel.data(), kGuardBytes, cudaMemcpyHostToDevice), "cudaMemcpy(guard)");
    }
    std::vector<char> param_used(prog.params.size(), 0), moment_used(prog.params.size(), 0);
    for (const Slot& s : P->slots) {
        if (s.kind == Slot::Param) param_used[s.index] = 1;
        if (s.kind == Slot::Moment) moment_used[s.index] = 1;
    }
    for (size_t p = 0; p < prog.params.size(); ++p) {
        uint64_t bytes = std::max<uint64_t>(prog.params[p].ty.count() * 4, 4);
        if (param_used[p]) {
            float* shared = nullptr;
            if (P->shares) {
                int at = P->shares->program.param_index(prog.params[p].path);
                if (at >= 0 && P->shares->program.params[static_cast<size_t>(at)].ty == prog.params[p].ty)
                    shared = P->shares->params[static_cast<size_t>(at)];
            }
            if (shared) {
                P->params[p] = shared;
            } else {
                cuda_ok(plan_malloc(P, &P->params[p], bytes), "cudaMalloc(parameter)");
                cuda_ok(cudaMemset(P->params[p], 0, bytes), "cudaMemset(parameter)");
                P->owns_param[p] = 1;
                P->param_bytes += bytes;
            }
        }
        // Mixed precision: every matrix parameter gets the bf16 working copy the matmuls read
        // (the owner's, for a plan that shares its parameters).
        if (param_used[p] && (P->flags & MSX_PLAN_BF16) && prog.params[p].ty.rank() == 2) {
            void* shared16 = nullptr;
            if (P->shares && !P->owns_param[p]) {
                int at = P->shares->program.param_index(prog.params[p].path);
                if (at >= 0) shared16 = P->shares->params16[static_cast<size_t>(at)];
            }
            if (shared16) {
                P->params16[p] = shared16;
            } else {
                cuda_ok(plan_malloc(P, &P->params16[p], bytes / 2), "cudaMalloc(parameter working copy)");
                P->owns_param16[p] = 1;
                P->param_bytes += bytes / 2;
                k::working_copy(P->stream, P->params[p], P->params16[p], prog.params[p].ty.count());
            }
        }
        if (moment_used[p]) {
            cuda_ok(plan_malloc(P, &P->m[p], bytes), "cudaMalloc(moment)");
            cuda_ok(plan_malloc(P, &P->v[p], bytes), "cudaMalloc(moment)");
            cuda_ok(cudaMemset(P->m[p], 0, bytes), "cudaMemset(moment)");
            cuda_ok(cudaMemset(P->v[p], 0, bytes), "cudaMemset(moment)");
            P->param_bytes += 2 * bytes;
        }
    }
    uint64_t in_bytes = std::max<uint64_t>(P->input_bytes, kAlign);
    cuda_ok(plan_malloc(P, &P->d_inputs, in_bytes), "cudaMalloc(inputs)");
    cuda_ok(cudaMemset(P->d_inputs, 0, in_bytes), "cudaMemset(inputs)");
    P->blob.assign(in_bytes, 0);
    for (int s = 0; s < kStagingSlots; ++s) {
        cuda_ok(cudaMallocHost(&P->pinned[s], in_bytes), "cudaMallocHost(staging)");
        cuda_ok(cudaEventCreate(&P->slot_begin[s]), "cudaEventCreate");
        cuda_ok(cudaEventCreate(&P->slot_done[s]), "cudaEventCreate");
    }
    cuda_ok(cudaMallocHost(&P->pinned_loss, kStagingSlots * sizeof(float)), "cudaMallocHost(loss)");
    cuda_ok(cudaMallocHost(&P->pinned_status, kStagingSlots * sizeof(uint32_t)), "cudaMallocHost(status)");
    std::memset(P->pinned_status, 0, kStagingSlots * sizeof(uint32_t));
    uint64_t const_bytes = std::max<uint64_t>(P->consts.size() * 4, 4);
    cuda_ok(plan_malloc(P, &P->d_consts, const_bytes), "cudaMalloc(constants)");
    if (!P->consts.empty())
        cuda_ok(cudaMemcpy(P->d_consts, P->consts.data(), P->consts.size() * 4, cudaMemcpyHostToDevice), "cudaMemcpy(constants)");
    cuda_ok(plan_malloc(P, &P->d_status, 4), "cudaMalloc(status)");
    cuda_ok(cudaMemset(P->d_status, 0, 4), "cudaMemset(status)");
    uint64_t counter_bytes = std::max<uint64_t>(P->counters_used, 1) * 4;
    cuda_ok(plan_malloc(P, &P->d_counters, counter_bytes), "cudaMalloc(counters)");
    cuda_ok(cudaMemset(P->d_counters, 0, counter_bytes), "cudaMemset(counters)");
    cuda_ok(cudaEventCreate(&P->clock_start), "cudaEventCreate");
    cuda_ok(cudaEventCreate(&P->clock_stop), "cudaEventCreate");
    P->side_fork.assign(P->launches.size(), nullptr);
    P->side_done.assign(P->launches.size(), nullptr);
    for (size_t l = 0; l < P->launches.size(); ++l) {
        if (P->launches[l].join_before < 0) continue;
        if (!P->side_stream) cuda_ok(cudaStreamCreateWithFlags(&P->side_stream, cudaStreamNonBlocking), "cudaStreamCreate");
        cuda_ok(cudaEventCreateWithFlags(&P->side_fork[l], cudaEventDisableTiming), "cudaEventCreate");
        cuda_ok(cudaEventCreateWithFlags(&P->side_done[l], cudaEventDisableTiming), "cudaEventCreate");
    }
    if (!sched.deferred_rows.empty()) {
        std::vector<k::RowSumJob> jobs;
        uint32_t first_block = 0;
        for (const Scheduler::DeferredRows& d : sched.deferred_rows) {
            // A launch counts its blocks from the start of its own part of the table.
            if (std::find(sched.rows_cuts.begin(), sched.rows_cuts.end(), jobs.size()) != sched.rows_cuts.end()) first_block = 0;
            jobs.push_back(k::row_sum_job(P->in(d.g), static_cast<float*>(P->ptr(d.partial)), d.rows, d.width,
                                          d.ld, first_block));
            first_block += k::row_sum_job_blocks(d.rows, d.width);
        }
        cuda_ok(plan_malloc(P, &P->d_row_sum_jobs, jobs.size() * sizeof(k::RowSumJob)), "cudaMalloc(row sum jobs)");
        cuda_ok(cudaMemcpy(P->d_row_sum_jobs, jobs.data(), jobs.size() * sizeof(k::RowSumJob), cudaMemcpyHostToDevice), "cudaMemcpy(row sum jobs)");
    }
    if (!sched.deferred.empty()) {
        std::vector<k::SumJob> jobs;
        uint32_t first_block = 0;
        for (const Scheduler::Deferred& d : sched.deferred) {
            if (std::find(sched.sums_cuts.begin(), sched.sums_cuts.end(), jobs.size()) != sched.sums_cuts.end()) first_block = 0;
            k::SumJob job = {};
            job.partial = static_cast<const float*>(P->ptr(d.partial)) + d.offset;
            job.out = static_cast<float*>(P->ptr(d.out));
            job.chunks = d.chunks;
            job.width = static_cast<uint32_t>(d.width);
            job.first_block = first_block;
            first_block += k::sum_job_blocks(d.chunks, d.width);
            jobs.push_back(job);
        }
        cuda_ok(plan_malloc(P, &P->d_sum_jobs, jobs.size() * sizeof(k::SumJob)), "cudaMalloc(sum jobs)");
        cuda_ok(cudaMemcpy(P->d_sum_jobs, jobs.data(), jobs.size() * sizeof(k::SumJob), cudaMemcpyHostToDevice), "cudaMemcpy(sum jobs)");
    }
    if (!sched.updates.empty()) {
        std::vector<k::UpdateTensor> tensors;
        for (const Scheduler::Update& u : sched.updates) {
            k::UpdateTensor t;
            t.p = P->params[u.param];
            t.g = static_cast<const float*>(P->ptr(u.grad_pos));
            t.m = P->m[u.param];
            t.v = P->v[u.param];
            t.count = prog.params[u.param].ty.count();
            t.p16 = P->params16[u.param];
            tensors.push_back(t);
        }
        size_t table_bytes = tensors.size() * sizeof(k::UpdateTensor);
        size_t chunk_bytes = sched.update_chunk_tensor.size() * 4;
        cuda_ok(plan_malloc(P, &P->d_update_tables, table_bytes + 2 * chunk_bytes), "cudaMalloc(update tables)");
        char* base = static_cast<char*>(P->d_update_tables);
        cuda_ok(cudaMemcpy(base, tensors.data(), table_bytes, cudaMemcpyHostToDevice), "cudaMemcpy(update tables)");
        cuda_ok(cudaMemcpy(base + table_bytes, sched.update_chunk_tensor.data(), chunk_bytes, cudaMemcpyHostToDevice), "cudaMemcpy");
        cuda_ok(cudaMemcpy(base + table_bytes + chunk_bytes, sched.update_chunk_start.data(), chunk_bytes, cudaMemcpyHostToDevice), "cudaMemcpy");
    }
}

void release(msx_plan* P) {
    if (!P) return;
    cudaSetDevice(P->device->ordinal);
    if (P->stream) cudaStreamSynchronize(P->stream);
    if (P->graph) cudaGraphExecDestroy(P->graph);
    if (P->comm_stream) cudaStreamSynchronize(P->comm_stream);
    for (Bucket& b : P->buckets) {
        if (b.ready) cudaEventDestroy(b.ready);
        if (b.done) cudaEventDestroy(b.done);
    }
    close_peer_reduce(P);
    if (P->comm && P->owns_comm) g_nccl.CommDestroy(P->comm);
    if (P->comm_stream) cudaStreamDestroy(P->comm_stream);
    for (cudaEvent_t e : {P->step_begun, P->weights_summed, P->loss_ready, P->loss_reduced})
        if (e) cudaEventDestroy(e);
    cudaFree(P->d_weight_total);
    cudaFree(P->arena);
    for (size_t p = 0; p < P->params.size(); ++p) {
        if (P->owns_param[p]) cudaFree(P->params[p]);
        if (P->owns_param16[p]) cudaFree(P->params16[p]);
        cudaFree(P->m[p]);
        cudaFree(P->v[p]);
    }
    cudaFree(P->d_inputs);
    cudaFree(P->d_consts);
    cudaFree(P->d_status);
    cudaFree(P->d_counters);
    cudaFree(P->d_update_tables);
    cudaFree(P->d_sum_jobs);
    if (P->side_stream) {
        cudaStreamSynchronize(P->side_stream);
        cudaStreamDestroy(P->side_stream);
    }
    for (cudaEvent_t e : P->side_fork)
        if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : P->side_done)
        if (e) cudaEventDestroy(e);
    cudaFree(P->d_row_sum_jobs);
    for (int s = 0; s < kStagingSlots; ++s) {
        if (P->pinned[s]) cudaFreeHost(P->pinned[s]);
        if (P->slot_begin[s]) cudaEventDestroy(P->slot_begin[s]);
        if (P->slot_done[s]) cudaEventDestroy(P->slot_done[s]);
    }
    if (P->backup) cudaFree(P->backup);
    if (P->pinned_loss) cudaFreeHost(P->pinned_loss);
    if (P->pinned_status) cudaFreeHost(P->pinned_status);
    if (P->clock_start) cudaEventDestroy(P->clock_start);
    if (P->clock_stop) cudaEventDestroy(P->clock_stop);
    if (P->stream) cudaStreamDestroy(P->stream);
    delete P;
}

void nccl_ok(ncclResult_t r, const char* what);

// Maps every rank's arena and flag words into this process (CUDA IPC handles, exchanged through
// the communicator as integers summed with zeros). The mapping is used only when it worked on
// every rank; MSX_PEER_REDUCE=0 (set for all ranks alike) leaves it off.
void setup_peer_reduce(msx_plan* P) {
    const char* wanted = std::getenv("MSX_PEER_REDUCE");
    if (wanted && std::strtol(wanted, nullptr, 0) == 0) return;
    if (P->world < 2 || P->world > k::kPeerRanks || !P->arena) return;
    constexpr size_t kWords = 2 * sizeof(cudaIpcMemHandle_t) / 4 + 1;  // two handles and a success mark
    static_assert(sizeof(cudaIpcMemHandle_t) % 4 == 0, "handles travel as 32-bit words");
    const size_t flag_bytes = k::kPeerRanks * sizeof(uint32_t);
    cuda_ok(cudaMalloc(&P->d_peer_flags, flag_bytes), "cudaMalloc(peer flags)");
    cuda_ok(cudaMemset(P->d_peer_flags, 0, flag_bytes), "cudaMemset(peer flags)");
    cuda_ok(cudaMalloc(&P->d_peer_words, 4 * sizeof(uint32_t)), "cudaMalloc(peer words)");
    cuda_ok(cudaMemset(P->d_peer_words, 0, 4 * sizeof(uint32_t)), "cudaMemset(peer words)");
    std::vector<uint32_t> table(kWords * static_cast<size_t>(P->world), 0u);
    uint32_t* mine = table.data() + kWords * static_cast<size_t>(P->rank);
    cudaIpcMemHandle_t arena_handle, flag_handle;
    bool ok = cudaIpcGetMemHandle(&arena_handle, P->arena) == cudaSuccess && cudaIpcGetMemHandle(&flag_handle, P->d_peer_flags) == cudaSuccess;
    cudaGetLastError();
    if (ok) {
        std::memcpy(mine, &arena_handle, sizeof arena_handle);
        std::memcpy(mine + sizeof(arena_handle) / 4, &flag_handle, sizeof flag_handle);
        mine[kWords - 1] = 1;
    }
    uint32_t* d_table = nullptr;
    cuda_ok(cudaMalloc(&d_table, table.size() * 4), "cudaMalloc(handle table)");
    auto exchange = [&]() {
        cuda_ok(cudaMemcpy(d_table, table.data(), table.size() * 4, cudaMemcpyHostToDevice), "cudaMemcpy(handle table)");
        nccl_ok(g_nccl.AllReduce(d_table, d_table, table.size(), ncclUint32, ncclSum, P->comm, P->comm_stream), "ncclAllReduce(handles)");
        cuda_ok(cudaStreamSynchronize(P->comm_stream), "cudaStreamSynchronize");
        cuda_ok(cudaMemcpy(table.data(), d_table, table.size() * 4, cudaMemcpyDeviceToHost), "cudaMemcpy(handle table)");
    };
    exchange();
    for (int q = 0; q < P->world && ok; ++q) ok = table[kWords * static_cast<size_t>(q) + kWords - 1] == 1;
    for (int q = 0; q < P->world && ok; ++q) {
        if (q == P->rank) {
            P->peer_arena[q] = P->arena;
            P->peer_flags[q] = P->d_peer_flags;
            continue;
        }
        const uint32_t* theirs = table.data() + kWords * static_cast<size_t>(q);
        std::memcpy(&arena_handle, theirs, sizeof arena_handle);
        std::memcpy(&flag_handle, theirs + sizeof(arena_handle) / 4, sizeof flag_handle);
        void* arena = nullptr;
        void* flags = nullptr;
        ok = cudaIpcOpenMemHandle(&arena, arena_handle, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
        if (ok) P->peer_arena[q] = static_cast<char*>(arena);
        ok = ok && cudaIpcOpenMemHandle(&flags, flag_handle, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
        if (ok) P->peer_flags[q] = static_cast<uint32_t*>(flags);
        cudaGetLastError();
    }
    // Every rank must agree: one that could not map a peer switches all of them to the library.
    std::fill(table.begin(), table.end(), 0u);
    table[static_cast<size_t>(P->rank)] = ok ? 1u : 0u;
    exchange();
    bool all = true;
    for (int q = 0; q < P->world; ++q) all = all && table[static_cast<size_t>(q)] == 1;
    cudaFree(d_table);
    P->peer_ready = all;
}

void close_peer_reduce(msx_plan* P) {
    for (int q = 0; q < k::kPeerRanks; ++q) {
        if (q == P->rank) continue;
        if (P->peer_arena[q]) cudaIpcCloseMemHandle(P->peer_arena[q]);
        if (P->peer_flags[q]) cudaIpcCloseMemHandle(P->peer_flags[q]);
    }
    cudaFree(P->d_peer_flags);
    cudaFree(P->d_peer_words);
}

void nccl_ok(ncclResult_t r, const char* what) {
    if (r != ncclSuccess) throw StatusError(MSX_LAUNCH_FAILED, std::string(what) + ": " + g_nccl.GetErrorString(r));
}

// Sums (or averages) `count` floats in place across the ranks, on `stream`. A no-op for a plan
// that is not data parallel.
void all_reduce(msx_plan* P, float* data, size_t count, bool average, cudaStream_t stream, bool exposed) {
    if (!P->comm) return;
    const char* at = reinterpret_cast<const char*>(data);
    // A reduction that the step waits for goes through the backend's own kernel (lower latency, all
    // links at once); one that runs behind the rest of the backward pass through the library, whose
    // kernel leaves more of the device to the launches beside it.
    if (exposed && P->peer_ready && stream == P->comm_stream && at >= P->arena && at + count * 4 <= P->arena + P->arena_bytes) {
        // One channel: every reduction of arena data on the communication stream, which every
        // rank issues in the same order.
        k::PeerReduceArgs args = {};
        const uint64_t offset = static_cast<uint64_t>(at - P->arena);
        for (int q = 0; q < P->world; ++q) {
            args.buffers[q] = reinterpret_cast<float*>(P->peer_arena[q] + offset);
            args.flags[q] = P->peer_flags[q];
        }
        args.epoch = P->d_peer_words;
        args.arrivals = P->d_peer_words + 1;
        args.failed = P->d_peer_words + 2;
        args.status = P->d_status;
        args.rank = static_cast<uint32_t>(P->rank);
        args.world = static_cast<uint32_t>(P->world);
        args.count = count;
        args.scale = average ? 1.0f / static_cast<float>(P->world) : 1.0f;
        k::peer_all_reduce(stream, args);
        return;
    }
    nccl_ok(g_nccl.AllReduce(data, data, count, ncclFloat, average ? ncclAvg : ncclSum, P->comm, stream), "ncclAllReduce");
}

// Data parallel: what a step starts on the side stream before its first launch, and how the side
// stream rejoins. Used by the step itself and by the launch-by-launch profile.
void begin_side_work(msx_plan* P) {
    P->loss_in_flight = false;
    if (!(P->comm && P->comm_stream) || P->early_weights < 0) return;
    cuda_ok(cudaEventRecord(P->step_begun, P->stream), "cudaEventRecord");
    cuda_ok(cudaStreamWaitEvent(P->comm_stream, P->step_begun, 0), "cudaStreamWaitEvent");
    k::weight_sum(P->comm_stream, P->f(static_cast<uint32_t>(P->early_weights)), P->early_rows, P->d_weight_total);
    all_reduce(P, P->d_weight_total, 1, false, P->comm_stream);
    cuda_ok(cudaEventRecord(P->weights_summed, P->comm_stream), "cudaEventRecord");
}
void join_loss(msx_plan* P) {
    if (!P->loss_in_flight) return;
    cuda_ok(cudaStreamWaitEvent(P->stream, P->loss_reduced, 0), "cudaStreamWaitEvent");
    P->loss_in_flight = false;
}

// A bucket closed this few launches before the optimizer has nothing left to hide behind.
constexpr int kExposedLaunches = 6;

void enqueue_all(msx_plan* P) {
    begin_side_work(P);
    std::vector<char> joined(P->launches.size(), 0);
    for (size_t l = 0; l < P->launches.size(); ++l) {
        // Side launches that this launch is the first to read: wait for them.
        for (size_t earlier = 0; earlier < l; ++earlier)
            if (P->launches[earlier].join_before == static_cast<int>(l) && P->side_done[earlier] && !joined[earlier]) {
                cuda_ok(cudaStreamWaitEvent(P->stream, P->side_done[earlier], 0), "cudaStreamWaitEvent");
                joined[earlier] = 1;
            }
        if (P->comm && static_cast<int>(l) == P->optimizer_launch) {
            if (P->probe_backward_done) cuda_ok(cudaEventRecord(P->probe_backward_done, P->stream), "cudaEventRecord");
            for (Bucket& b : P->buckets) cuda_ok(cudaStreamWaitEvent(P->stream, b.done, 0), "cudaStreamWaitEvent");
            join_loss(P);
            if (P->probe_update_begins) cuda_ok(cudaEventRecord(P->probe_update_begins, P->stream), "cudaEventRecord");
        }
        if (P->launches[l].join_before >= 0 && P->side_stream && P->side_fork[l]) {
            cuda_ok(cudaEventRecord(P->side_fork[l], P->stream), "cudaEventRecord");
            cuda_ok(cudaStreamWaitEvent(P->side_stream, P->side_fork[l], 0), "cudaStreamWaitEvent");
            P->launches[l].run(P->side_stream);
            cuda_ok(cudaEventRecord(P->side_done[l], P->side_stream), "cudaEventRecord");
        } else {
            P->launches[l].run(P->stream);
        }
        if (!P->comm) continue;
        for (Bucket& b : P->buckets) {
            if (b.after_launch != static_cast<int>(l)) continue;
            // Launches that run beside the main stream and have not been waited for yet may have
            // written gradients of this bucket: the main stream waits for them first.
            for (size_t earlier = 0; earlier <= l; ++earlier)
                if (P->launches[earlier].join_before > static_cast<int>(l) && P->side_done[earlier] && !joined[earlier] &&
                    P->launches[earlier].side_writes_outputs) {
                    cuda_ok(cudaStreamWaitEvent(P->stream, P->side_done[earlier], 0), "cudaStreamWaitEvent");
                    joined[earlier] = 1;
                }
            // The bucket's gradients are complete in stream order: reduce them on the side stream
            // while the rest of backward runs.
            cuda_ok(cudaEventRecord(b.ready, P->stream), "cudaEventRecord");
            cuda_ok(cudaStreamWaitEvent(P->comm_stream, b.ready, 0), "cudaStreamWaitEvent");
            const bool exposed = P->optimizer_launch < 0 || P->optimizer_launch - b.after_launch <= kExposedLaunches;
            all_reduce(P, reinterpret_cast<float*>(P->arena + b.offset), b.bytes / 4, P->average_gradients, P->comm_stream, exposed);
            cuda_ok(cudaEventRecord(b.done, P->comm_stream), "cudaEventRecord");
        }
    }
    join_loss(P);  // a plan without an optimizer launch: the side stream rejoins here
}

// Waits for `event` at most `timeout_ms`, polling: never an unbounded wait.
int wait_event(cudaEvent_t event, uint32_t timeout_ms) {
    auto start = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t e = cudaEventQuery(event);
        if (e == cudaSuccess) return MSX_OK;
        if (e != cudaErrorNotReady) cuda_ok(e, "cudaEventQuery");
        auto waited = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - start).count();
        if (timeout_ms != 0 && waited >= static_cast<long long>(timeout_ms)) return MSX_TIMEOUT;
        if (waited > 2) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

// The device status word as the step of staging slot `slot` left it (copied out behind the step's
// loss): a raised bit means the results of that step, and of every later one, are not valid. The
// word is sticky on the device until this clears it.
void check_status(msx_plan* P, int slot) {
    const uint32_t bits = P->pinned_status[slot];
    if (!bits) return;
    for (int s = 0; s < kStagingSlots; ++s) P->pinned_status[s] = 0;
    cuda_ok(cudaMemsetAsync(P->d_status, 0, 4, P->stream), "cudaMemsetAsync");
    if (bits & 2u) throw StatusError(MSX_TIMEOUT, "a bounded wait on the device ran out (tensor-core matmul, or a peer rank of the gradient all-reduce); the step's results are not valid");
    throw StatusError(MSX_BAD_INPUT, "an embedding id computed on the device is outside its table");
}

int wait_all(msx_plan* P, uint32_t timeout_ms) {
    ++P->host_waits;
    struct Stamp {
        msx_plan* plan;
        ~Stamp() { plan->last_wait = std::chrono::steady_clock::now(); }
    } stamp{P};
    if (P->steps == 0) {
        cuda_ok(cudaStreamSynchronize(P->stream), "cudaStreamSynchronize");
        return MSX_OK;
    }
    int slot = static_cast<int>((P->steps - 1) % kStagingSlots);
    int rc = wait_event(P->slot_done[slot], timeout_ms == 0 ? 600000u : timeout_ms);
    if (rc != MSX_OK) return rc;
    check_status(P, slot);
    return MSX_OK;
}

template <class F> int guarded(msx_device* device, F body) {
    try {
        return body();
    } catch (const StatusError& e) {
        if (device) device->error = e.what();
        else g_open_error = e.what();
        return e.status;
    } catch (const k::CudaError& e) {
        if (device) device->error = e.what();
        else g_open_error = e.what();
        return e.code == cudaErrorMemoryAllocation ? MSX_OUT_OF_MEMORY : MSX_LAUNCH_FAILED;
    } catch (const std::exception& e) {
        if (device) device->error = e.what();
        else g_open_error = e.what();
        return MSX_UNSUPPORTED;
    }
}

int check_input(const HostInput& in, const void* host, std::string* why) {
    const uint64_t n = in.bytes / 4;
    for (const InputCheck& c : in.checks) {
        if (c.kind == InputCheck::Ids || c.kind == InputCheck::Labels) {
            const int32_t* v = static_cast<const int32_t*>(host);
            for (uint64_t e = 0; e < n; ++e)
                if (v[e] < 0 || static_cast<uint64_t>(v[e]) >= c.bound) {
                    *why = "`" + in.name + "`[" + std::to_string(e) + "] = " + std::to_string(v[e]) + " is outside [0, " +
                           std::to_string(c.bound) + ")";
                    return MSX_BAD_INPUT;
                }
        } else if (c.kind == InputCheck::Weights) {
            const float* v = static_cast<const float*>(host);
            for (uint64_t e = 0; e < n; ++e)
                if (!(v[e] * 0.0f == 0.0f) || v[e] < 0.0f) {
                    *why = "`" + in.name + "`[" + std::to_string(e) + "] is negative or not finite";
                    return MSX_BAD_INPUT;
                }
        } else {
            const float* v = static_cast<const float*>(host);
            for (uint64_t seq = 0; seq * c.bound < n; ++seq) {
                bool any = false;
                for (uint64_t j = 0; j < c.bound; ++j) {
                    float mk = v[seq * c.bound + j];
                    if (mk != 0.0f && mk != 1.0f) {
                        *why = "`" + in.name + "`: sequence " + std::to_string(seq) + " key " + std::to_string(j) + " is neither 0 nor 1";
                        return MSX_BAD_INPUT;
                    }
                    any = any || mk == 1.0f;
                }
                if (!any) {
                    *why = "`" + in.name + "`: sequence " + std::to_string(seq) + " has no unmasked key";
                    return MSX_BAD_INPUT;
                }
            }
        }
    }
    return MSX_OK;
}

}  // namespace

// ---------------------------------------------------------------------------------------------

extern "C" {

int msx_open(int ordinal, msx_device** out) {
    return guarded(nullptr, [&]() -> int {
        if (!out) throw StatusError(MSX_BAD_ARGUMENT, "msx_open: null output");
        *out = nullptr;
        int count = 0;
        cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess || count == 0) throw StatusError(MSX_NO_DEVICE, std::string("no CUDA device: ") + cudaGetErrorString(e));
        if (ordinal < 0 || ordinal >= count)
            throw StatusError(MSX_NO_DEVICE, "no CUDA device " + std::to_string(ordinal) + " (" + std::to_string(count) + " present)");
        cudaDeviceProp prop;
        cuda_ok(cudaGetDeviceProperties(&prop, ordinal), "cudaGetDeviceProperties");
        if (prop.major != 10)
            throw StatusError(MSX_NO_DEVICE, std::string("device ") + prop.name + " is sm_" + std::to_string(prop.major * 10 + prop.minor) +
                                                 "; the kernels are built for sm_100a only");
        cuda_ok(cudaSetDevice(ordinal), "cudaSetDevice");
        msx_device* d = new msx_device;
        d->ordinal = ordinal;
        *out = d;
        return MSX_OK;
    });
}

void msx_close(msx_device* device) { delete device; }

const char* msx_last_error(const msx_device* device) { return device ? device->error.c_str() : g_open_error.c_str(); }

// For the host loop above this file, which reports its own failures through the device handle.
void msx_internal_set_error(msx_device* device, const char* message) {
    if (device) device->error = message ? message : "";
    else g_open_error = message ? message : "";
}

// For the tests: sets the low byte of the plan's device status word in stream order, as a kernel
// whose bounded wait ran out (bit 1) or that met a bad id (bit 0) would, without any kernel
// misbehaving. Not part of the ABI.
int msx_internal_raise_status(msx_plan* plan, uint32_t bits) {
    if (!plan) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        cuda_ok(cudaMemsetAsync(plan->d_status, static_cast<int>(bits & 0xffu), 1, plan->stream), "cudaMemsetAsync(status)");
        return MSX_OK;
    });
}

int msx_plan_create(msx_device* device, const char* ir_text, uint64_t seed, uint32_t flags, msx_plan* shares,
                    msx_plan** out) {
    if (!device || !ir_text || !out) return MSX_BAD_ARGUMENT;
    *out = nullptr;
    msx_plan* P = new msx_plan;
    int rc = guarded(device, [&]() -> int {
        cuda_ok(cudaSetDevice(device->ordinal), "cudaSetDevice");
        P->device = device;
        P->seed = seed;
        P->flags = flags;
        if ((flags & MSX_PLAN_BF16) && (flags & MSX_PLAN_EXACT_MATMUL))
            throw StatusError(MSX_BAD_ARGUMENT, "msx_plan_create: MSX_PLAN_BF16 and MSX_PLAN_EXACT_MATMUL exclude each other");
        P->shares = shares;
        try {
            P->program = msx::parse_program(ir_text);
        } catch (const msx::Error& e) {
            throw StatusError(MSX_UNSUPPORTED, e.what());
        }
        if (P->program.outputs.empty()) throw StatusError(MSX_UNSUPPORTED, "the program has no output");
        Scheduler sched(P);
        sched.run();
        place_arena(P);
        allocate(P, sched);
        return MSX_OK;
    });
    if (rc != MSX_OK) {
        std::string keep = device->error;
        release(P);
        device->error = keep;
        return rc;
    }
    *out = P;
    return MSX_OK;
}

void msx_plan_destroy(msx_plan* plan) { release(plan); }

uint32_t msx_plan_input_count(const msx_plan* plan) { return plan ? static_cast<uint32_t>(plan->inputs.size()) : 0; }
const char* msx_plan_input_name(const msx_plan* plan, uint32_t index) {
    return plan && index < plan->inputs.size() ? plan->inputs[index].name.c_str() : nullptr;
}
uint64_t msx_plan_input_bytes(const msx_plan* plan, uint32_t index) {
    return plan && index < plan->inputs.size() ? plan->inputs[index].bytes : 0;
}
int msx_plan_input_is_i32(const msx_plan* plan, uint32_t index) {
    return plan && index < plan->inputs.size() && plan->inputs[index].i32 ? 1 : 0;
}
uint32_t msx_plan_param_count(const msx_plan* plan) { return plan ? static_cast<uint32_t>(plan->program.params.size()) : 0; }
const char* msx_plan_param_path(const msx_plan* plan, uint32_t index) {
    return plan && index < plan->program.params.size() ? plan->program.params[index].path.c_str() : nullptr;
}
uint64_t msx_plan_param_bytes(const msx_plan* plan, uint32_t index) {
    return plan && index < plan->program.params.size() ? plan->program.params[index].ty.count() * 4 : 0;
}

static int transfer(msx_plan* plan, float* device_ptr, uint64_t expect, void* host, uint64_t bytes, bool upload, const char* what) {
    if (!plan || !host) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        if (!device_ptr) throw StatusError(MSX_BAD_ARGUMENT, std::string(what) + ": the plan holds no such buffer");
        if (bytes != expect)
            throw StatusError(MSX_BAD_ARGUMENT, std::string(what) + ": " + std::to_string(bytes) + " bytes given, " + std::to_string(expect) + " expected");
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        if (upload) cuda_ok(cudaMemcpyAsync(device_ptr, host, bytes, cudaMemcpyHostToDevice, plan->stream), what);
        else cuda_ok(cudaMemcpyAsync(host, device_ptr, bytes, cudaMemcpyDeviceToHost, plan->stream), what);
        (upload ? plan->bytes_uploaded : plan->bytes_downloaded) += bytes;
        cuda_ok(cudaStreamSynchronize(plan->stream), what);
        return MSX_OK;
    });
}

int msx_param_upload(msx_plan* plan, uint32_t index, const void* host, uint64_t bytes) {
    if (!plan || index >= plan->program.params.size()) return MSX_BAD_ARGUMENT;
    int rc = transfer(plan, plan->params[index], msx_plan_param_bytes(plan, index), const_cast<void*>(host), bytes, true, "msx_param_upload");
    if (rc != MSX_OK || !plan->params16[index]) return rc;
    // The bf16 working copy follows its f32 master.
    return guarded(plan->device, [&]() -> int {
        k::working_copy(plan->stream, plan->params[index], plan->params16[index], plan->program.params[index].ty.count());
        cuda_ok(cudaStreamSynchronize(plan->stream), "cudaStreamSynchronize");
        return MSX_OK;
    });
}
int msx_param_download(msx_plan* plan, uint32_t index, void* host, uint64_t bytes) {
    if (!plan || index >= plan->program.params.size()) return MSX_BAD_ARGUMENT;
    return transfer(plan, plan->params[index], msx_plan_param_bytes(plan, index), host, bytes, false, "msx_param_download");
}
int msx_moment_upload(msx_plan* plan, uint32_t index, char which, const void* host, uint64_t bytes) {
    if (!plan || index >= plan->program.params.size() || (which != 'm' && which != 'v')) return MSX_BAD_ARGUMENT;
    return transfer(plan, (which == 'm' ? plan->m : plan->v)[index], msx_plan_param_bytes(plan, index), const_cast<void*>(host), bytes, true,
                    "msx_moment_upload");
}
int msx_moment_download(msx_plan* plan, uint32_t index, char which, void* host, uint64_t bytes) {
    if (!plan || index >= plan->program.params.size() || (which != 'm' && which != 'v')) return MSX_BAD_ARGUMENT;
    return transfer(plan, (which == 'm' ? plan->m : plan->v)[index], msx_plan_param_bytes(plan, index), host, bytes, false,
                    "msx_moment_download");
}

}  // extern "C"

// The state a later step overwrites: every parameter, then every moment, in parameter order.
template <class F> static void for_each_state_tensor(msx_plan* plan, F visit) {
    for (size_t p = 0; p < plan->program.params.size(); ++p) {
        const uint64_t count = plan->program.params[p].ty.count();
        if (plan->params[p]) visit(plan->params[p], count, static_cast<int>(p));
        if (plan->m[p]) visit(plan->m[p], count, -1);
        if (plan->v[p]) visit(plan->v[p], count, -1);
    }
}

extern "C" {

int msx_state_snapshot(msx_plan* plan) {
    if (!plan) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        if (!plan->backup) {
            uint64_t floats = 0;
            for_each_state_tensor(plan, [&](float*, uint64_t count, int) { floats += (count + 3) / 4 * 4; });
            cuda_ok(plan_malloc(plan, &plan->backup, std::max<uint64_t>(floats, 4) * 4), "cudaMalloc(state backup)");
            plan->backup_floats = floats;
        }
        uint64_t at = 0;
        for_each_state_tensor(plan, [&](float* from, uint64_t count, int) {
            cuda_ok(cudaMemcpyAsync(plan->backup + at, from, count * 4, cudaMemcpyDeviceToDevice, plan->stream), "cudaMemcpyAsync(state backup)");
            at += (count + 3) / 4 * 4;
        });
        plan->backup_filled = true;
        return MSX_OK;
    });
}

int msx_state_restore(msx_plan* plan) {
    if (!plan) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        if (!plan->backup_filled) throw StatusError(MSX_BAD_ARGUMENT, "msx_state_restore: no snapshot was taken");
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        uint64_t at = 0;
        for_each_state_tensor(plan, [&](float* to, uint64_t count, int param) {
            cuda_ok(cudaMemcpyAsync(to, plan->backup + at, count * 4, cudaMemcpyDeviceToDevice, plan->stream), "cudaMemcpyAsync(state restore)");
            at += (count + 3) / 4 * 4;
            // The bf16 working copy follows its f32 master.
            if (param >= 0 && plan->params16[static_cast<size_t>(param)])
                k::working_copy(plan->stream, to, plan->params16[static_cast<size_t>(param)], count);
        });
        // The status word of the abandoned steps goes with them.
        cuda_ok(cudaMemsetAsync(plan->d_status, 0, 4, plan->stream), "cudaMemsetAsync(status)");
        return MSX_OK;
    });
}

int msx_set_input(msx_plan* plan, const char* name, const void* host, uint64_t bytes) {
    if (!plan || !name || !host) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        for (const HostInput& in : plan->inputs) {
            if (in.name != name) continue;
            if (bytes != in.bytes)
                throw StatusError(MSX_BAD_ARGUMENT, "msx_set_input: `" + in.name + "` takes " + std::to_string(in.bytes) + " bytes, " +
                                                        std::to_string(bytes) + " given");
            std::string why;
            int rc = check_input(in, host, &why);
            if (rc != MSX_OK) throw StatusError(rc, why);
            std::memcpy(plan->blob.data() + in.offset, host, bytes);
            plan->blob_dirty = true;
            return MSX_OK;
        }
        throw StatusError(MSX_BAD_ARGUMENT, std::string("msx_set_input: the step reads no input `") + name + "`");
    });
}

int msx_set_shard(msx_plan* plan, uint64_t rows_before, uint64_t global_rows) {
    if (!plan) return MSX_BAD_ARGUMENT;
    (void)global_rows;
    return guarded(plan->device, [&]() -> int {
        if (plan->shard_rows_before != rows_before && plan->graph) {
            cuda_ok(cudaStreamSynchronize(plan->stream), "cudaStreamSynchronize");
            cuda_ok(cudaGraphExecDestroy(plan->graph), "cudaGraphExecDestroy");
            plan->graph = nullptr;
        }
        plan->shard_rows_before = rows_before;
        return MSX_OK;
    });
}

int msx_run(msx_plan* plan) {
    if (!plan) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        int slot = static_cast<int>(plan->steps % kStagingSlots);
        if (plan->slot_used[slot]) {
            int rc = wait_event(plan->slot_done[slot], 600000u);
            if (rc != MSX_OK) throw StatusError(rc, "msx_run: a step submitted " + std::to_string(kStagingSlots) + " steps ago has not finished");
        }
        if (plan->clock_steps == 0) cuda_ok(cudaEventRecord(plan->clock_start, plan->stream), "cudaEventRecord");
        cuda_ok(cudaEventRecord(plan->slot_begin[slot], plan->stream), "cudaEventRecord");
        if (!plan->timing_begun) {
            plan->timing_begun = true;
            plan->first_submit = plan->last_wait = std::chrono::steady_clock::now();
        }
        ++plan->submits;
        plan->dispatches += plan->launches.size();
        plan->bytes_downloaded += (plan->loss_pos >= 0 ? 4 : 0) + 4;
        if (plan->input_bytes && plan->blob_dirty) {
            plan->bytes_uploaded += plan->input_bytes;
            plan->blob_dirty = false;
            std::memcpy(plan->pinned[slot], plan->blob.data(), plan->input_bytes);
            cuda_ok(cudaMemcpyAsync(plan->d_inputs, plan->pinned[slot], plan->input_bytes, cudaMemcpyHostToDevice, plan->stream),
                    "cudaMemcpyAsync(inputs)");
        }
        if (plan->flags & MSX_PLAN_NO_GRAPH) {
            enqueue_all(plan);
        } else {
            if (!plan->graph) {
                cudaGraph_t graph = nullptr;
                cuda_ok(cudaStreamBeginCapture(plan->stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
                try {
                    enqueue_all(plan);
                } catch (...) {
                    cudaStreamEndCapture(plan->stream, &graph);
                    if (graph) cudaGraphDestroy(graph);
                    throw;
                }
                cuda_ok(cudaStreamEndCapture(plan->stream, &graph), "cudaStreamEndCapture");
                cudaError_t e = cudaGraphInstantiate(&plan->graph, graph, 0);
                cudaGraphDestroy(graph);
                cuda_ok(e, "cudaGraphInstantiate");
            }
            cuda_ok(cudaGraphLaunch(plan->graph, plan->stream), "cudaGraphLaunch");
        }
        if (plan->loss_pos >= 0)
            cuda_ok(cudaMemcpyAsync(plan->pinned_loss + slot, plan->ptr(static_cast<uint32_t>(plan->loss_pos)), 4, cudaMemcpyDeviceToHost,
                                    plan->stream),
                    "cudaMemcpyAsync(loss)");
        cuda_ok(cudaMemcpyAsync(plan->pinned_status + slot, plan->d_status, 4, cudaMemcpyDeviceToHost, plan->stream), "cudaMemcpyAsync(status)");
        cuda_ok(cudaEventRecord(plan->clock_stop, plan->stream), "cudaEventRecord");
        cuda_ok(cudaEventRecord(plan->slot_done[slot], plan->stream), "cudaEventRecord");
        plan->slot_used[slot] = true;
        ++plan->steps;
        ++plan->clock_steps;
        return MSX_OK;
    });
}

int msx_sync(msx_plan* plan, uint32_t timeout_ms) {
    if (!plan) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int { return wait_all(plan, timeout_ms); });
}

int msx_loss(msx_plan* plan, float* loss, uint32_t timeout_ms) {
    if (!plan || !loss) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        if (plan->steps == 0) throw StatusError(MSX_BAD_ARGUMENT, "msx_loss: no step has run");
        if (plan->loss_pos < 0) throw StatusError(MSX_BAD_ARGUMENT, "msx_loss: the program has no rank-0 loss");
        int rc = wait_all(plan, timeout_ms);
        if (rc != MSX_OK) return rc;
        *loss = plan->pinned_loss[(plan->steps - 1) % kStagingSlots];
        return MSX_OK;
    });
}

int msx_loss_of(msx_plan* plan, uint64_t step_number, float* loss, uint32_t timeout_ms) {
    if (!plan || !loss) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        if (step_number >= plan->steps || step_number + kStagingSlots < plan->steps)
            throw StatusError(MSX_BAD_ARGUMENT, "msx_loss_of: only the last " + std::to_string(kStagingSlots) + " submitted steps keep their loss");
        if (plan->loss_pos < 0) throw StatusError(MSX_BAD_ARGUMENT, "msx_loss_of: the program has no rank-0 loss");
        int slot = static_cast<int>(step_number % kStagingSlots);
        int rc = wait_event(plan->slot_done[slot], timeout_ms == 0 ? 600000u : timeout_ms);
        if (rc != MSX_OK) return rc;
        check_status(plan, slot);
        *loss = plan->pinned_loss[slot];
        return MSX_OK;
    });
}

uint64_t msx_steps_submitted(const msx_plan* plan) { return plan ? plan->steps : 0; }

int msx_profile_step(msx_plan* plan, float* launch_ms, uint32_t capacity) {
    return msx_profile_step_repeated(plan, 1, launch_ms, capacity);
}

int msx_profile_step_repeated(msx_plan* plan, uint32_t repeats, float* launch_ms, uint32_t capacity) {
    if (!plan || !launch_ms || repeats == 0) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        if (capacity < plan->launches.size()) throw StatusError(MSX_BAD_ARGUMENT, "msx_profile_step: room for every launch is needed");
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        int rc = wait_all(plan, 0);
        if (rc != MSX_OK) return rc;
        // A data-parallel step holds collectives (the loss and weight sums inside the cross-entropy
        // launch, the gradient buckets before the update): every launch is then issued once, and
        // the buckets are summed across the ranks before the optimizer launch, so that the
        // replicas stay equal as after any other step.
        if (plan->comm) repeats = 1;
        const size_t count = plan->launches.size();
        std::vector<cudaEvent_t> events(2 * count);
        for (cudaEvent_t& e : events) cuda_ok(cudaEventCreate(&e), "cudaEventCreate");
        if (plan->input_bytes) {
            std::memcpy(plan->pinned[0], plan->blob.data(), plan->input_bytes);
            cuda_ok(cudaMemcpyAsync(plan->d_inputs, plan->pinned[0], plan->input_bytes, cudaMemcpyHostToDevice, plan->stream), "cudaMemcpyAsync");
        }
        begin_side_work(plan);
        for (size_t l = 0; l < count; ++l) {
            const std::string& kernel = plan->launches[l].kernel;
            const bool in_place = kernel == "adamw_multi_tensor" || kernel == "sgd_multi_tensor";
            if (plan->comm && static_cast<int>(l) == plan->optimizer_launch) {
                for (const Bucket& b : plan->buckets)
                    all_reduce(plan, reinterpret_cast<float*>(plan->arena + b.offset), b.bytes / 4, plan->average_gradients, plan->stream, false);
                join_loss(plan);
            }
            cuda_ok(cudaEventRecord(events[2 * l], plan->stream), "cudaEventRecord");
            for (uint32_t r = 0; r < (in_place ? 1u : repeats); ++r) plan->launches[l].run(plan->stream);
            cuda_ok(cudaEventRecord(events[2 * l + 1], plan->stream), "cudaEventRecord");
        }
        join_loss(plan);
        cuda_ok(cudaStreamSynchronize(plan->stream), "cudaStreamSynchronize");
        for (size_t l = 0; l < count; ++l) {
            cuda_ok(cudaEventElapsedTime(&launch_ms[l], events[2 * l], events[2 * l + 1]), "cudaEventElapsedTime");
            const std::string& kernel = plan->launches[l].kernel;
            if (kernel != "adamw_multi_tensor" && kernel != "sgd_multi_tensor") launch_ms[l] /= static_cast<float>(repeats);
        }
        for (cudaEvent_t e : events) cudaEventDestroy(e);
        return MSX_OK;
    });
}

int msx_step_ms(msx_plan* plan, uint64_t step_number, float* ms) {
    if (!plan || !ms) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        if (step_number >= plan->steps || step_number + kStagingSlots < plan->steps)
            throw StatusError(MSX_BAD_ARGUMENT, "msx_step_ms: only the last " + std::to_string(kStagingSlots) + " submitted steps keep their time");
        int slot = static_cast<int>(step_number % kStagingSlots);
        int rc = wait_event(plan->slot_done[slot], 600000u);
        if (rc != MSX_OK) return rc;
        cuda_ok(cudaEventElapsedTime(ms, plan->slot_begin[slot], plan->slot_done[slot]), "cudaEventElapsedTime");
        return MSX_OK;
    });
}

int msx_comm_exposed_ms(msx_plan* plan, float* ms) {
    if (!plan || !ms) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        *ms = 0.0f;
        if (!plan->comm || plan->optimizer_launch < 0) return MSX_OK;
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        int rc = wait_all(plan, 0);
        if (rc != MSX_OK) return rc;
        cudaEvent_t before = nullptr, after = nullptr;
        cuda_ok(cudaEventCreate(&before), "cudaEventCreate");
        cuda_ok(cudaEventCreate(&after), "cudaEventCreate");
        plan->probe_backward_done = before;
        plan->probe_update_begins = after;
        try {
            enqueue_all(plan);
            cuda_ok(cudaStreamSynchronize(plan->stream), "cudaStreamSynchronize");
            cuda_ok(cudaEventElapsedTime(ms, before, after), "cudaEventElapsedTime");
        } catch (...) {
            plan->probe_backward_done = plan->probe_update_begins = nullptr;
            cudaEventDestroy(before);
            cudaEventDestroy(after);
            throw;
        }
        plan->probe_backward_done = plan->probe_update_begins = nullptr;
        cudaEventDestroy(before);
        cudaEventDestroy(after);
        return MSX_OK;
    });
}

uint64_t msx_launch_bytes(const msx_plan* plan, uint32_t launch) {
    if (!plan || launch >= plan->launches.size()) return 0;
    const Launch& l = plan->launches[launch];
    uint64_t bytes = 0;
    for (uint32_t r : l.reads) bytes += plan->slots[r].bytes;
    for (uint32_t w : l.writes) bytes += plan->slots[w].bytes;
    if (l.kernel == "adamw_multi_tensor") bytes += l.flop / 16 * 24;
    if (l.kernel == "sgd_multi_tensor") bytes += l.flop / 2 * 8;
    return bytes;
}

uint64_t msx_launch_flop(const msx_plan* plan, uint32_t launch) {
    return plan && launch < plan->launches.size() ? plan->launches[launch].flop : 0;
}

const char* msx_launch_kernel(const msx_plan* plan, uint32_t launch) {
    return plan && launch < plan->launches.size() ? plan->launches[launch].kernel.c_str() : nullptr;
}

int msx_value_download(msx_plan* plan, uint32_t value_id, void* host, uint64_t bytes) {
    if (!plan || !host) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        int at = plan->program.position(value_id);
        if (at < 0) throw StatusError(MSX_BAD_ARGUMENT, "msx_value_download: %" + std::to_string(value_id) + " is not defined");
        const Slot& s = plan->slots[static_cast<size_t>(at)];
        bool readable = s.keep || s.kind == Slot::Param || s.kind == Slot::Moment || s.kind == Slot::Input || s.kind == Slot::Const;
        if (!readable || s.kind == Slot::Dead || s.kind == Slot::View)
            throw StatusError(MSX_BAD_ARGUMENT, "msx_value_download: %" + std::to_string(value_id) + " is not an output; its storage is reused");
        uint64_t expect = plan->program.nodes[static_cast<size_t>(at)].ty.count() * 4;
        if (bytes != expect) throw StatusError(MSX_BAD_ARGUMENT, "msx_value_download: " + std::to_string(expect) + " bytes expected");
        int rc = wait_all(plan, 0);
        if (rc != MSX_OK) return rc;
        cuda_ok(cudaMemcpyAsync(host, plan->ptr(static_cast<uint32_t>(at)), bytes, cudaMemcpyDeviceToHost, plan->stream), "cudaMemcpyAsync");
        cuda_ok(cudaStreamSynchronize(plan->stream), "cudaStreamSynchronize");
        return MSX_OK;
    });
}

// ---- held-out reduction ---------------------------------------------------------------------
}  // extern "C"

struct msx_heldout {
    msx_plan* plan = nullptr;
    uint32_t at = 0;           // position of the logits in the plan's program
    uint64_t rows = 0, classes = 0;
    uint32_t batches = 0;
    int32_t* d_labels = nullptr;   // [batches][rows], resident for the run
    float* d_weights = nullptr;    // [batches][rows]
    double* d_terms = nullptr;     // [rows] scratch
    uint32_t* d_hits = nullptr;    // [rows] scratch
    k::HeldOutState* d_state = nullptr;
    k::HeldOutState* pinned = nullptr;
    cudaEvent_t done = nullptr;
    std::vector<char> given;       // which batches have their targets
    bool begun = false;
};

extern "C" {

int msx_heldout_create(msx_plan* plan, uint32_t logits, uint32_t batches, msx_heldout** out) {
    if (!plan || !out) return MSX_BAD_ARGUMENT;
    *out = nullptr;
    return guarded(plan->device, [&]() -> int {
        int at = plan->program.position(logits);
        if (at < 0) throw StatusError(MSX_BAD_ARGUMENT, "msx_heldout_create: %" + std::to_string(logits) + " is not defined");
        const Slot& s = plan->slots[static_cast<size_t>(at)];
        const msx::Type& ty = plan->program.nodes[static_cast<size_t>(at)].ty;
        if (ty.i32 || ty.rank() != 2 || ty.shape[0] == 0 || ty.shape[1] == 0 || ty.count() > 0xffffffffull)
            throw StatusError(MSX_BAD_ARGUMENT, "msx_heldout_create: the logits are " + ty.str() + ", not f32 [rows, classes] of 1 to 2^32 - 1 elements");
        if (!s.keep || s.kind != Slot::Arena || s.half)
            throw StatusError(MSX_BAD_ARGUMENT, "msx_heldout_create: %" + std::to_string(logits) + " is not an f32 output of the plan");
        if (batches == 0) throw StatusError(MSX_BAD_ARGUMENT, "msx_heldout_create: no batches");
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        std::unique_ptr<msx_heldout> h(new msx_heldout());
        h->plan = plan;
        h->at = static_cast<uint32_t>(at);
        h->rows = ty.shape[0];
        h->classes = ty.shape[1];
        h->batches = batches;
        h->given.assign(batches, 0);
        const size_t all = static_cast<size_t>(batches) * h->rows;
        cudaError_t e = plan_malloc(plan, &h->d_labels, all * 4);
        if (e == cudaSuccess) e = plan_malloc(plan, &h->d_weights, all * 4);
        if (e == cudaSuccess) e = plan_malloc(plan, &h->d_terms, h->rows * 8);
        if (e == cudaSuccess) e = plan_malloc(plan, &h->d_hits, h->rows * 4);
        if (e == cudaSuccess) e = plan_malloc(plan, &h->d_state, sizeof(k::HeldOutState));
        if (e == cudaSuccess) e = cudaMallocHost(&h->pinned, sizeof(k::HeldOutState));
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->done, cudaEventDisableTiming);
        if (e != cudaSuccess) {
            msx_heldout_destroy(h.release());
            cuda_ok(e, "msx_heldout_create");
        }
        *out = h.release();
        return MSX_OK;
    });
}

void msx_heldout_destroy(msx_heldout* h) {
    if (!h) return;
    cudaSetDevice(h->plan->device->ordinal);
    cudaStreamSynchronize(h->plan->stream);
    cudaFree(h->d_labels);
    cudaFree(h->d_weights);
    cudaFree(h->d_terms);
    cudaFree(h->d_hits);
    cudaFree(h->d_state);
    if (h->pinned) cudaFreeHost(h->pinned);
    if (h->done) cudaEventDestroy(h->done);
    delete h;
}

int msx_heldout_targets(msx_heldout* h, uint32_t batch, const int32_t* labels, const float* weights, uint64_t rows) {
    if (!h || !labels || !weights) return MSX_BAD_ARGUMENT;
    msx_plan* plan = h->plan;
    return guarded(plan->device, [&]() -> int {
        if (batch >= h->batches) throw StatusError(MSX_BAD_ARGUMENT, "msx_heldout_targets: batch " + std::to_string(batch) + " of " + std::to_string(h->batches));
        if (rows != h->rows)
            throw StatusError(MSX_BAD_ARGUMENT, "msx_heldout_targets: held-out batch " + std::to_string(batch) + " has not " + std::to_string(h->rows) + " rows");
        for (uint64_t n = 0; n < rows; ++n)
            if (labels[n] < 0 || static_cast<uint64_t>(labels[n]) >= h->classes)
                throw StatusError(MSX_BAD_INPUT, "held-out batch " + std::to_string(batch) + ", row " + std::to_string(n) + ": label " +
                                                     std::to_string(labels[n]) + " is not below the " + std::to_string(h->classes) + " classes");
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        // Ordered on the plan's stream behind any evaluation still reading the old targets.
        cuda_ok(cudaMemcpyAsync(h->d_labels + batch * rows, labels, rows * 4, cudaMemcpyHostToDevice, plan->stream), "cudaMemcpyAsync(labels)");
        cuda_ok(cudaMemcpyAsync(h->d_weights + batch * rows, weights, rows * 4, cudaMemcpyHostToDevice, plan->stream), "cudaMemcpyAsync(weights)");
        cuda_ok(cudaStreamSynchronize(plan->stream), "cudaStreamSynchronize");
        plan->bytes_uploaded += rows * 8;
        h->given[batch] = 1;
        return MSX_OK;
    });
}

int msx_heldout_begin(msx_heldout* h) {
    if (!h) return MSX_BAD_ARGUMENT;
    return guarded(h->plan->device, [&]() -> int {
        cuda_ok(cudaSetDevice(h->plan->device->ordinal), "cudaSetDevice");
        cuda_ok(cudaMemsetAsync(h->d_state, 0, sizeof(k::HeldOutState), h->plan->stream), "cudaMemsetAsync(held-out state)");
        h->begun = true;
        return MSX_OK;
    });
}

int msx_heldout_add(msx_heldout* h, uint32_t batch) {
    if (!h) return MSX_BAD_ARGUMENT;
    msx_plan* plan = h->plan;
    return guarded(plan->device, [&]() -> int {
        if (!h->begun) throw StatusError(MSX_BAD_ARGUMENT, "msx_heldout_add: no evaluation was begun");
        if (batch >= h->batches || !h->given[batch])
            throw StatusError(MSX_BAD_ARGUMENT, "msx_heldout_add: held-out batch " + std::to_string(batch) + " has no labels and weights");
        if (plan->steps == 0) throw StatusError(MSX_BAD_ARGUMENT, "msx_heldout_add: the plan has not run the batch");
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        k::heldout_rows(plan->stream, static_cast<const float*>(plan->ptr(h->at)), plan->slots[h->at].pitch, h->d_labels + static_cast<size_t>(batch) * h->rows,
                        h->d_weights + static_cast<size_t>(batch) * h->rows, h->rows, h->classes, h->d_terms, h->d_hits, h->d_state);
        ++plan->dispatches;
        return MSX_OK;
    });
}

int msx_heldout_sums(msx_heldout* h, double* numerator, uint64_t* correct, uint32_t timeout_ms) {
    if (!h || !numerator || !correct) return MSX_BAD_ARGUMENT;
    msx_plan* plan = h->plan;
    return guarded(plan->device, [&]() -> int {
        if (!h->begun) throw StatusError(MSX_BAD_ARGUMENT, "msx_heldout_sums: no evaluation was begun");
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        cuda_ok(cudaMemcpyAsync(h->pinned, h->d_state, sizeof(k::HeldOutState), cudaMemcpyDeviceToHost, plan->stream), "cudaMemcpyAsync(held-out state)");
        cuda_ok(cudaEventRecord(h->done, plan->stream), "cudaEventRecord");
        int rc = wait_event(h->done, timeout_ms == 0 ? 600000u : timeout_ms);
        ++plan->host_waits;
        plan->last_wait = std::chrono::steady_clock::now();
        if (rc != MSX_OK) return rc;
        plan->bytes_downloaded += sizeof(k::HeldOutState);
        // The batches' own steps were waited for with the state: a wait of theirs that gave up shows here.
        if (plan->steps) check_status(plan, static_cast<int>((plan->steps - 1) % kStagingSlots));
        *numerator = h->pinned->numerator;
        *correct = h->pinned->correct;
        h->begun = false;
        return MSX_OK;
    });
}

int msx_plan_check_guards(msx_plan* plan) {
    if (!plan) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        if (!(plan->flags & MSX_PLAN_GUARD)) throw StatusError(MSX_BAD_ARGUMENT, "msx_plan_check_guards: the plan was not made with MSX_PLAN_GUARD");
        int rc = wait_all(plan, 0);
        if (rc != MSX_OK) return rc;
        std::vector<uint32_t> words(kGuardBytes / 4);
        for (uint32_t at = 0; at < plan->slots.size(); ++at) {
            const Slot& s = plan->slots[at];
            if (s.kind != Slot::Arena || s.first < 0) continue;
            cuda_ok(cudaMemcpy(words.data(), plan->arena + s.offset + (s.bytes + 3) / 4 * 4, kGuardBytes, cudaMemcpyDeviceToHost), "cudaMemcpy(guard)");
            for (size_t w = 0; w < words.size(); ++w)
                if (words[w] != kGuardWord) {
                    const std::string name = at < plan->program.nodes.size() ? "%" + std::to_string(plan->program.nodes[at].id)
                                                                             : "scratch" + std::to_string(at - plan->program.nodes.size());
                    std::string writer = "?";
                    if (s.last_write >= 0) writer = plan->launches[static_cast<size_t>(s.last_write)].kernel;
                    throw StatusError(MSX_LAUNCH_FAILED, "guard word " + std::to_string(w) + " after " + name + " (" + std::to_string(s.bytes) +
                                                             " bytes, last written by " + writer + ") was overwritten");
                }
        }
        return MSX_OK;
    });
}

int msx_plan_stats(const msx_plan* plan, msx_stats* out) {
    if (!plan || !out) return MSX_BAD_ARGUMENT;
    std::memset(out, 0, sizeof *out);
    out->launches_per_step = plan->launches.size();
    out->nodes = plan->program.nodes.size();
    out->live_nodes = plan->live_nodes;
    out->arena_bytes = plan->arena_bytes;
    out->unshared_bytes = plan->unshared_bytes;
    out->param_bytes = plan->param_bytes;
    out->upload_bytes_per_step = plan->input_bytes;
    out->steps_run = plan->steps;
    for (const Launch& l : plan->launches) {
        for (uint32_t r : l.reads) out->algorithmic_bytes_per_step += plan->slots[r].bytes;
        for (uint32_t w : l.writes) out->algorithmic_bytes_per_step += plan->slots[w].bytes;
        if (l.kernel == "matmul") out->matmul_flop_per_step += l.flop;
        if (l.kernel == "adamw_multi_tensor") out->algorithmic_bytes_per_step += l.flop / 16 * 24;  // p, m, v read and written
        if (l.kernel == "sgd_multi_tensor") out->algorithmic_bytes_per_step += l.flop / 2 * 8;
    }
    return MSX_OK;
}

namespace {
uint64_t copy_text(const std::string& text, char* out, uint64_t capacity) {
    if (out && capacity) {
        size_t n = std::min<size_t>(capacity - 1, text.size());
        std::memcpy(out, text.data(), n);
        out[n] = 0;
    }
    return text.size() + 1;
}
std::string fixed3(double v) {
    char buf[64];
    std::snprintf(buf, sizeof buf, "%.3f", v);
    return buf;
}
}  // namespace

int msx_plan_run_stats(const msx_plan* plan, msx_run_stats* out) {
    if (!plan || !out) return MSX_BAD_ARGUMENT;
    std::memset(out, 0, sizeof *out);
    out->steps = plan->steps;
    out->host_waits = plan->host_waits;
    out->submits = plan->submits;
    out->dispatches = plan->dispatches;
    out->dispatches_per_step = plan->launches.size();
    out->barriers_per_step = 0;
    out->bytes_uploaded = plan->bytes_uploaded;
    out->bytes_downloaded = plan->bytes_downloaded;
    out->device_allocations = plan->device_allocations;
    out->peak_device_bytes = plan->device_bytes;
    out->tolerance_class = (plan->flags & MSX_PLAN_EXACT_MATMUL) ? 0u : 1u;
    out->elapsed_us = plan->timing_begun ? std::chrono::duration<double, std::micro>(plan->last_wait - plan->first_submit).count() : 0.0;
    return MSX_OK;
}

uint64_t msx_stats_report(const msx_plan* plan, char* out, uint64_t capacity) {
    msx_run_stats s;
    if (msx_plan_run_stats(plan, &s) != MSX_OK) return 0;
    // The lines of `train --stats`, field for field (vulkan/runner.rs:143-163). A CUDA plan has no
    // pipelines to create: its kernels are compiled into the library.
    std::string text;
    text += "steps: " + std::to_string(s.steps) + "\n";
    text += "host waits: " + std::to_string(s.host_waits) + "\n";
    text += "submits: " + std::to_string(s.submits) + "\n";
    text += "dispatches: " + std::to_string(s.dispatches) + "\n";
    text += "dispatches per step: " + std::to_string(s.dispatches_per_step) + "\n";
    text += "barriers per step: " + std::to_string(s.barriers_per_step) + "\n";
    text += "bytes uploaded: " + std::to_string(s.bytes_uploaded) + "\n";
    text += "bytes downloaded: " + std::to_string(s.bytes_downloaded) + "\n";
    text += "device allocations: " + std::to_string(s.device_allocations) + "\n";
    text += "peak device bytes: " + std::to_string(s.peak_device_bytes) + "\n";
    text += std::string("numerics class: ") + (s.tolerance_class ? "tolerance" : "bit-for-bit") + "\n";
    text += "us per step: " + fixed3(s.steps ? s.elapsed_us / static_cast<double>(s.steps) : 0.0) + "\n";
    text += "pipelines: 0\n";
    text += "pipeline creation us: 0.000\n";
    return copy_text(text, out, capacity);
}

uint64_t msx_profile_report(msx_plan* plan, msx_plan* final_plan, uint32_t repeats, char* out, uint64_t capacity) {
    if (!plan) return 0;
    std::string text;
    int rc = guarded(plan->device, [&]() -> int {
        // One `profile dispatch` line per launch of the step plan, then of the final-loss plan, in
        // the reference's format (vulkan/profile.rs:237-338): the kernel's number is its rank among
        // the plan's distinct kernels, its entry the kernel's name.
        double step_us = 0.0;
        unsigned long long step_flop = 0, step_bytes = 0;
        for (msx_plan* which : {plan, final_plan}) {
            if (!which) continue;
            std::vector<float> ms(which->launches.size());
            int r = msx_profile_step_repeated(which, repeats ? repeats : 1, ms.data(), static_cast<uint32_t>(ms.size()));
            if (r != MSX_OK) return r;
            std::vector<std::string> kernels;
            for (size_t l = 0; l < which->launches.size(); ++l) {
                const Launch& launch = which->launches[l];
                size_t id = std::find(kernels.begin(), kernels.end(), launch.kernel) - kernels.begin();
                if (id == kernels.size()) kernels.push_back(launch.kernel);
                const double us = static_cast<double>(ms[l]) * 1e3;
                const unsigned long long flop = msx_launch_flop(which, static_cast<uint32_t>(l)), bytes = msx_launch_bytes(which, static_cast<uint32_t>(l));
                text += std::string("profile dispatch ") + (which == plan ? "step " : "final ") + std::to_string(l) + " " + std::to_string(id) + " " +
                        launch.kernel + " calls 1 total_us " + fixed3(us) + " mean_us " + fixed3(us) + " flop " + std::to_string(flop) + " bytes " +
                        std::to_string(bytes);
                if (us > 0.0) text += " gflop_per_s " + fixed3(static_cast<double>(flop) / us / 1e3) + " gb_per_s " + fixed3(static_cast<double>(bytes) / us / 1e3);
                else text += " gflop_per_s unavailable gb_per_s unavailable";
                text += "\n";
                if (which == plan) {
                    step_us += us;
                    step_flop += flop;
                    step_bytes += bytes;
                }
            }
        }
        text += "profile pipeline statistics: not reported\n";
        msx_run_stats s;
        msx_plan_run_stats(plan, &s);
        text += "profile dispatches " + std::to_string(s.dispatches) + "\n";
        text += "profile submits " + std::to_string(s.submits) + "\n";
        text += "profile host_waits " + std::to_string(s.host_waits) + "\n";
        text += "profile barriers_per_step " + std::to_string(s.barriers_per_step) + "\n";
        text += "profile bytes_uploaded " + std::to_string(s.bytes_uploaded) + "\n";
        text += "profile bytes_downloaded " + std::to_string(s.bytes_downloaded) + "\n";
        text += "profile device_allocations " + std::to_string(s.device_allocations) + "\n";
        text += "profile peak_device_bytes " + std::to_string(s.peak_device_bytes) + "\n";
        text += "profile pipeline_creation_us 0.000\n";
        text += "profile compile_us 0.000\n";
        // The steady time of a step: the profiled launches one after another (the graph replay of a
        // step is shorter: msx_elapsed_ms, msx_step_ms).
        text += "profile steady_us_per_step " + fixed3(step_us) + "\n";
        text += "profile step_total flop " + std::to_string(step_flop) + " bytes " + std::to_string(step_bytes);
        if (step_us > 0.0) text += " gflop_per_s " + fixed3(static_cast<double>(step_flop) / step_us / 1e3) + " gb_per_s " + fixed3(static_cast<double>(step_bytes) / step_us / 1e3);
        else text += " gflop_per_s unavailable gb_per_s unavailable";
        text += " uncounted_sites 0\n";
        return MSX_OK;
    });
    if (rc != MSX_OK) return 0;
    return copy_text(text, out, capacity);
}

uint64_t msx_plan_describe(const msx_plan* plan, char* out, uint64_t capacity) {
    if (!plan) return 0;
    std::string text;
    auto name = [&](uint32_t slot) {
        // A value a mixed-precision plan stores as bf16 carries the suffix `h`.
        const std::string suffix = plan->half(slot) ? "h" : "";
        if (slot < plan->program.nodes.size()) return "%" + std::to_string(plan->program.nodes[slot].id) + suffix;
        return "scratch" + std::to_string(slot - plan->program.nodes.size()) + suffix;
    };
    for (size_t l = 0; l < plan->launches.size(); ++l) {
        const Launch& launch = plan->launches[l];
        text += std::to_string(l) + ": " + launch.kernel + " %" + std::to_string(launch.value) + " reads";
        for (uint32_t r : launch.reads) text += " " + name(r);
        text += " writes";
        for (uint32_t w : launch.writes) text += " " + name(w);
        if (launch.flop) text += " flop " + std::to_string(launch.flop);
        if (launch.join_before >= 0) text += " beside " + std::to_string(launch.join_before);
        text += "\n";
    }
    if (out && capacity) {
        size_t n = std::min<size_t>(capacity - 1, text.size());
        std::memcpy(out, text.data(), n);
        out[n] = 0;
    }
    return text.size() + 1;
}

int msx_elapsed_ms(msx_plan* plan, double* total_ms, uint64_t* steps) {
    if (!plan || !total_ms || !steps) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        *total_ms = 0.0;
        *steps = plan->clock_steps;
        if (plan->clock_steps == 0) return MSX_OK;
        int rc = wait_all(plan, 0);
        if (rc != MSX_OK) return rc;
        cuda_ok(cudaEventSynchronize(plan->clock_stop), "cudaEventSynchronize");
        float ms = 0.0f;
        cuda_ok(cudaEventElapsedTime(&ms, plan->clock_start, plan->clock_stop), "cudaEventElapsedTime");
        *total_ms = ms;
        plan->clock_steps = 0;
        return MSX_OK;
    });
}

int msx_op_matmul(const float* a, int a_transposed, const float* b, int b_transposed, float* c, uint64_t m, uint64_t n, uint64_t k,
                  float* workspace, uint64_t workspace_floats, uint32_t* status, void* stream, int exact) {
    if (!a || !b || !c) return MSX_BAD_ARGUMENT;
    return guarded(nullptr, [&]() -> int {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        if (exact) {
            k::matmul(s, a, a_transposed != 0, b, b_transposed != 0, c, m, n, k);
            return MSX_OK;
        }
        const bool wide_ok = (a_transposed ? m : k) % 4 == 0 && (b_transposed ? k : n) % 4 == 0 &&
                             reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0;
        uint64_t need = k::matmul_tc_plan(m, n, k, 1, 1, wide_ok).workspace_floats;
        if (need > workspace_floats || (need && !workspace) || !status)
            throw StatusError(MSX_BAD_ARGUMENT, "msx_op_matmul: the tensor-core kernel needs " + std::to_string(need) +
                                                    " workspace floats and a status word");
        k::matmul_tc(s, a, a_transposed != 0, b, b_transposed != 0, c, m, n, k, workspace, status);
        return MSX_OK;
    });
}

uint64_t msx_op_matmul_workspace(uint64_t m, uint64_t n, uint64_t k) {
    // Enough for either choice of tile (which one runs depends on how the operands are stored).
    return std::max(k::matmul_tc_plan(m, n, k, 1, 1, true).workspace_floats, k::matmul_tc_plan(m, n, k, 1, 1, false).workspace_floats);
}

int msx_op_matmul_bf16(const void* a, int a_transposed, const void* b, int b_transposed, void* c, int c_is_bf16, uint64_t m, uint64_t n,
                       uint64_t k, float* workspace, uint64_t workspace_floats, uint32_t* status, void* stream) {
    if (!a || !b || !c || !status) return MSX_BAD_ARGUMENT;
    return guarded(nullptr, [&]() -> int {
        const uint64_t need = k::matmul_bf16_plan(m, n, k).workspace_floats;
        if (need > workspace_floats || (need && !workspace))
            throw StatusError(MSX_BAD_ARGUMENT, "msx_op_matmul_bf16: the product needs " + std::to_string(need) + " workspace floats");
        try {
            k::HalfMatrix A = {a, static_cast<uint32_t>(a_transposed ? m : k), 0, 0, a_transposed != 0};
            k::HalfMatrix B = {b, static_cast<uint32_t>(b_transposed ? k : n), 0, 0, b_transposed != 0};
            k::HalfResult C = {c, c_is_bf16 != 0, static_cast<uint32_t>(n), 0, 0};
            k::matmul_bf16(static_cast<cudaStream_t>(stream), A, B, C, m, n, k, 1, 1, workspace, nullptr, status);
        } catch (const std::invalid_argument& e) {
            throw StatusError(MSX_BAD_ARGUMENT, e.what());
        }
        return MSX_OK;
    });
}

uint64_t msx_op_matmul_bf16_workspace(uint64_t m, uint64_t n, uint64_t k) { return k::matmul_bf16_plan(m, n, k).workspace_floats; }

int msx_op_attention_bf16(const void* q, const void* k, const void* v, const float* mask, const void* g, void* out, void* dq, void* dk,
                          void* dv, float* stats, uint32_t batch, uint32_t q_len, uint32_t k_len, uint32_t heads, uint32_t head_dim,
                          uint32_t* status, void* stream) {
    if (!q || !k || !v || !mask || !out || !stats || !status) return MSX_BAD_ARGUMENT;
    return guarded(nullptr, [&]() -> int {
        k::AttentionShape shape = {batch, q_len, k_len, heads, head_dim};
        if (!k::attention_fused_supported(shape))
            throw StatusError(MSX_UNSUPPORTED, "msx_op_attention_bf16: heads of up to 64 columns (a multiple of 8), up to 512 keys and queries");
        try {
            cudaStream_t s = static_cast<cudaStream_t>(stream);
            k::attention_fused_forward(s, q, k, v, mask, out, stats, shape, status);
            if (g) k::attention_fused_backward(s, q, k, v, mask, g, out, stats, dq, dk, dv, shape, status);
        } catch (const std::invalid_argument& e) {
            throw StatusError(MSX_BAD_ARGUMENT, e.what());
        }
        return MSX_OK;
    });
}

int msx_op_heldout_rows(const float* logits, uint64_t pitch, const int32_t* labels, const float* weights, uint64_t rows, uint64_t classes,
                        void* scratch, void* state, void* stream) {
    if (!logits || !labels || !weights || !scratch || !state) return MSX_BAD_ARGUMENT;
    static_assert(sizeof(k::HeldOutState) == 24, "the state the header describes");
    return guarded(nullptr, [&]() -> int {
        if (rows == 0 || classes == 0 || rows * classes > 0xffffffffull || (pitch && pitch < classes))
            throw StatusError(MSX_BAD_ARGUMENT, "msx_op_heldout_rows: logits of 1 to 2^32 - 1 elements, rows at least `classes` floats apart");
        double* terms = static_cast<double*>(scratch);
        k::heldout_rows(static_cast<cudaStream_t>(stream), logits, pitch, labels, weights, rows, classes, terms,
                        reinterpret_cast<uint32_t*>(terms + rows), static_cast<k::HeldOutState*>(state));
        return MSX_OK;
    });
}

uint64_t msx_schedule_describe(const char* ir_text, char* out, uint64_t capacity) {
    return msx_schedule_describe_with(ir_text, MSX_PLAN_DEFAULT, out, capacity);
}

uint64_t msx_schedule_describe_with(const char* ir_text, uint32_t flags, char* out, uint64_t capacity) {
    if (!ir_text) return 0;
    msx_plan* P = new msx_plan;
    P->flags = flags;
    std::string text;
    int rc = guarded(nullptr, [&]() -> int {
        try {
            P->program = msx::parse_program(ir_text);
        } catch (const msx::Error& e) {
            throw StatusError(MSX_UNSUPPORTED, e.what());
        }
        if (P->program.outputs.empty()) throw StatusError(MSX_UNSUPPORTED, "the program has no output");
        Scheduler sched(P);
        sched.run();
        place_arena(P);
        uint64_t need = msx_plan_describe(P, nullptr, 0);
        text.resize(need);
        msx_plan_describe(P, &text[0], need);
        text.resize(need - 1);
        text += "arena " + std::to_string(P->arena_bytes) + " bytes, unshared " + std::to_string(P->unshared_bytes) +
                " bytes, inputs " + std::to_string(P->input_bytes) + " bytes, launches " + std::to_string(P->launches.size()) + "\n";
        return MSX_OK;
    });
    delete P;
    if (rc != MSX_OK) return 0;
    if (out && capacity) {
        size_t n = std::min<size_t>(capacity - 1, text.size());
        std::memcpy(out, text.data(), n);
        out[n] = 0;
    }
    return text.size() + 1;
}

int msx_comm_unique_id(void* unique_id_128) {
    if (!unique_id_128) return MSX_BAD_ARGUMENT;
    return guarded(nullptr, [&]() -> int {
        static_assert(sizeof(ncclUniqueId) == 128, "the ABI hands a 128-byte id around");
        if (!g_nccl.load()) throw StatusError(MSX_UNSUPPORTED, g_nccl.error);
        ncclUniqueId id;
        nccl_ok(g_nccl.GetUniqueId(&id), "ncclGetUniqueId");
        std::memcpy(unique_id_128, &id, sizeof id);
        return MSX_OK;
    });
}

int msx_comm_init(msx_plan* plan, int rank, int world, const void* unique_id_128) {
    if (!plan || !unique_id_128 || world < 1 || rank < 0 || rank >= world) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        if (plan->comm) throw StatusError(MSX_BAD_ARGUMENT, "msx_comm_init: the plan already has a communicator");
        if (plan->steps) throw StatusError(MSX_BAD_ARGUMENT, "msx_comm_init: call it before the first step");
        if (!g_nccl.load()) throw StatusError(MSX_UNSUPPORTED, g_nccl.error);
        cuda_ok(cudaSetDevice(plan->device->ordinal), "cudaSetDevice");
        ncclUniqueId id;
        std::memcpy(&id, unique_id_128, sizeof id);
        nccl_ok(g_nccl.CommInitRank(&plan->comm, world, id, rank), "ncclCommInitRank");
        plan->owns_comm = true;
        plan->rank = rank;
        plan->world = world;
        cuda_ok(cudaStreamCreateWithFlags(&plan->comm_stream, cudaStreamNonBlocking), "cudaStreamCreate");
        // An mse-style loss divides by the shard's own element count, so gradients are averaged;
        // a weighted cross_entropy divides by the whole batch's weight sum, so they are summed.
        plan->average_gradients = true;
        for (const Node& n : plan->program.nodes)
            if (n.op == Op::CrossEntropy) plan->average_gradients = false;
        for (cudaEvent_t* e : {&plan->step_begun, &plan->weights_summed, &plan->loss_ready, &plan->loss_reduced})
            cuda_ok(cudaEventCreateWithFlags(e, cudaEventDisableTiming), "cudaEventCreate");
        cuda_ok(cudaMalloc(&plan->d_weight_total, sizeof(float)), "cudaMalloc(weight total)");
        plan_buckets(plan);
        setup_peer_reduce(plan);
        for (Bucket& b : plan->buckets) {
            cuda_ok(cudaEventCreateWithFlags(&b.ready, cudaEventDisableTiming), "cudaEventCreate");
            cuda_ok(cudaEventCreateWithFlags(&b.done, cudaEventDisableTiming), "cudaEventCreate");
        }
        return MSX_OK;
    });
}

int msx_comm_share(msx_plan* plan, msx_plan* owner) {
    if (!plan || !owner) return MSX_BAD_ARGUMENT;
    return guarded(plan->device, [&]() -> int {
        if (!owner->comm) throw StatusError(MSX_BAD_ARGUMENT, "msx_comm_share: the other plan has no communicator");
        if (plan->comm || plan->steps) throw StatusError(MSX_BAD_ARGUMENT, "msx_comm_share: call it once, before the first step");
        plan->comm = owner->comm;
        plan->rank = owner->rank;
        plan->world = owner->world;
        plan->average_gradients = owner->average_gradients;
        return MSX_OK;
    });
}

uint32_t msx_comm_bucket_count(const msx_plan* plan) { return plan ? static_cast<uint32_t>(plan->buckets.size()) : 0; }
uint32_t msx_comm_uses_peer_memory(const msx_plan* plan) { return plan && plan->peer_ready ? 1u : 0u; }

int msx_peer_reduce_check(msx_device* device, uint32_t world, uint64_t count, float* const* host_copies, float scale,
                          int peers_present, uint32_t wait_ms, uint32_t* status_bits) {
    if (!device || !host_copies || !status_bits || world < 2 || world > static_cast<uint32_t>(k::kPeerRanks) || count == 0)
        return MSX_BAD_ARGUMENT;
    return guarded(device, [&]() -> int {
        cuda_ok(cudaSetDevice(device->ordinal), "cudaSetDevice");
        // One allocation: the copies (each on a 256-byte boundary), then per rank eight flag words
        // and four channel words, then the status word.
        const uint64_t pitch = align_up(count * 4);
        const uint64_t words_at = pitch * world, bytes = words_at + (static_cast<uint64_t>(world) * 12 + 1) * 4;
        char* base = nullptr;
        cuda_ok(cudaMalloc(&base, bytes), "cudaMalloc(peer check)");
        struct Free { char* p; ~Free() { cudaFree(p); } } release{base};
        cuda_ok(cudaMemset(base, 0, bytes), "cudaMemset(peer check)");
        for (uint32_t q = 0; q < world; ++q) {
            if (!host_copies[q]) return MSX_BAD_ARGUMENT;
            cuda_ok(cudaMemcpy(base + pitch * q, host_copies[q], count * 4, cudaMemcpyHostToDevice), "cudaMemcpy(copy)");
        }
        uint32_t* words = reinterpret_cast<uint32_t*>(base + words_at);
        uint32_t* status = words + static_cast<uint64_t>(world) * 12;
        if (peers_present) {
            // Flag values only grow, so one large value stands for "arrived" at every rendezvous.
            std::vector<uint32_t> arrived(static_cast<size_t>(world) * 12, 0u);
            for (uint32_t q = 0; q < world; ++q)
                for (uint32_t r = 0; r < world; ++r) arrived[static_cast<size_t>(q) * 12 + r] = 1u << 20;
            cuda_ok(cudaMemcpy(words, arrived.data(), arrived.size() * 4, cudaMemcpyHostToDevice), "cudaMemcpy(flags)");
        }
        const uint32_t launches = peers_present ? world : 2u;  // without peers: rank 0 twice
        for (uint32_t l = 0; l < launches; ++l) {
            const uint32_t rank = peers_present ? l : 0u;
            k::PeerReduceArgs args = {};
            for (uint32_t q = 0; q < world; ++q) {
                args.buffers[q] = reinterpret_cast<float*>(base + pitch * q);
                args.flags[q] = words + static_cast<uint64_t>(q) * 12;
            }
            args.epoch = words + static_cast<uint64_t>(rank) * 12 + 8;
            args.arrivals = args.epoch + 1;
            args.failed = args.epoch + 2;
            args.status = status;
            args.rank = rank;
            args.world = world;
            args.count = count;
            args.scale = scale;
            args.wait_nanoseconds = static_cast<uint64_t>(wait_ms ? wait_ms : 1u) * 1000000ull;
            k::peer_all_reduce(nullptr, args);
            cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        }
        cuda_ok(cudaMemcpy(status_bits, status, 4, cudaMemcpyDeviceToHost), "cudaMemcpy(status)");
        for (uint32_t q = 0; q < world; ++q)
            cuda_ok(cudaMemcpy(host_copies[q], base + pitch * q, count * 4, cudaMemcpyDeviceToHost), "cudaMemcpy(copy)");
        return MSX_OK;
    });
}

uint64_t msx_compile(const char* source, const char* which, uint64_t masked_rows, char* out, uint64_t capacity) {
    if (!source || !which) return 0;
    std::string text;
    try {
        msx::Compiled c = msx::compile_training(source, masked_rows);
        std::string w = which;
        if (w == "step") text = msx::print_program(c.step);
        else if (w == "forward") text = msx::print_program(c.forward);
        else if (w == "tensor") text = msx::print_program(c.forward_with_dropout);
        else throw msx::Error("msx_compile: `which` is step, forward or tensor");
    } catch (const std::exception& e) {
        g_open_error = e.what();
        return 0;
    }
    if (out && capacity) {
        size_t n = std::min<size_t>(capacity - 1, text.size());
        std::memcpy(out, text.data(), n);
        out[n] = 0;
    }
    return text.size() + 1;
}

uint64_t msx_compile_function(const char* source, const char* name, const char* which, char* out, uint64_t capacity) {
    if (!source || !name || !which) return 0;
    std::string text;
    try {
        msx::Compiled c = msx::compile_function(source, name);
        std::string w = which;
        if (w == "step") text = msx::print_program(c.step);
        else if (w == "forward") text = msx::print_program(c.forward);
        else if (w == "prediction") text = "%" + std::to_string(c.prediction);
        else throw msx::Error("msx_compile_function: `which` is step, forward or prediction");
    } catch (const std::exception& e) {
        g_open_error = e.what();
        return 0;
    }
    if (out && capacity) {
        size_t n = std::min<size_t>(capacity - 1, text.size());
        std::memcpy(out, text.data(), n);
        out[n] = 0;
    }
    return text.size() + 1;
}

}  // extern "C"
