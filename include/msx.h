/* msx: the C ABI of the B200 CUDA backend for ModelSpec's compiled training step.
 *
 * This is the boundary a `cuda` sibling of the reference's `vulkan` runtime module binds: plain
 * C, opaque handles, host pointers and byte counts, an int status from every call, no
 * exceptions. The library's own waits are bounded: host waits on events take a timeout, and the
 * spin waits inside its kernels (tensor-core pipeline barriers, the peer-memory all-reduce) give
 * up after a limit and raise a status bit. Calls into NCCL (communicator set-up, its all-reduce
 * kernels) are bounded only by NCCL's own settings. The shim owns every device allocation,
 * stream, graph and communicator; the caller owns host memory, which is copied before a call
 * returns.
 *
 * What crosses the boundary is the training step in the text form the reference already prints
 * (`modelspec ir --stage training`, crates/modelspec-core/src/ir/print.rs:55-166): the tensor-SSA
 * program with its parameter table, optimizer line, subgraph tags and output roles. The shim
 * does its own fusion, liveness and buffer reuse over that program, as the reference's scheduler
 * does for Vulkan (crates/modelspec-core/src/schedule.rs:759-1484), and refuses a program holding
 * an op it has no kernel for (the reference's E-TARGET-011, schedule.rs:155-159).
 */
#ifndef MSX_H
#define MSX_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct msx_device msx_device;
typedef struct msx_plan msx_plan;

/* Status codes. The message of the last failure on a handle is msx_last_error(). */
enum {
    MSX_OK = 0,
    MSX_BAD_ARGUMENT = 1,   /* null handle, unknown name, wrong byte count */
    MSX_NO_DEVICE = 2,      /* no CUDA device at that ordinal, or it is not sm_100 */
    MSX_OUT_OF_MEMORY = 3,
    MSX_UNSUPPORTED = 4,    /* an op with no CUDA kernel, or malformed IR */
    MSX_LAUNCH_FAILED = 5,  /* a CUDA call failed; the message holds its name */
    MSX_NON_FINITE = 6,     /* reserved for the host loop's E-TRAIN-001 check */
    MSX_TIMEOUT = 7,        /* a bounded wait ran out */
    MSX_BAD_INPUT = 8       /* an input the reference's interpreter refuses: id or label out of
                               range, key mask not 0/1, negative or non-finite loss weight */
};

/* Plan flags. */
enum {
    MSX_PLAN_DEFAULT = 0,
    MSX_PLAN_NO_GRAPH = 1,  /* launch kernels one by one instead of through one CUDA graph */
    MSX_PLAN_EXACT_MATMUL = 2, /* matmuls as f32 fused chains in ascending k, the bits of the
                                  reference's CPU loop, instead of 3xTF32 on the tensor cores */
    MSX_PLAN_GUARD = 8,        /* for tests: every intermediate value keeps storage of its own for the
                                  whole step (no reuse by liveness), followed by 16 sentinel words
                                  that msx_plan_check_guards inspects: the guard words the reference's
                                  device tests keep after every output
                                  (crates/modelspec-runtime/tests/common/mod.rs:100-117) */
    MSX_PLAN_BF16 = 4          /* mixed precision, an extension: the reference's IR has f32 and i32
                                  only (ir/tensor.rs:38-51). Every rank-2 intermediate (activations
                                  and their adjoints) is stored as bf16 and every product runs as
                                  bf16 x bf16 with f32 accumulation on TMA-fed tcgen05.mma; parameters,
                                  AdamW moments, gradients, row statistics, losses and all sums stay
                                  f32, and the optimizer launch writes a bf16 working copy of every
                                  matrix parameter beside its f32 master. Tolerance class against the
                                  f32 CPU run: losses within 2e-2 relative over 100 steps of the
                                  BERT twin. Refused (MSX_UNSUPPORTED) for a program with an op that
                                  has no bf16 kernel, a matmul operand that is a host input, or a
                                  matrix whose row width is not a multiple of 8 (vocabulary-wide
                                  logits are padded). Not combinable with MSX_PLAN_EXACT_MATMUL. */
};

typedef struct msx_stats {
    uint64_t launches_per_step;   /* kernels of one step, as scheduled */
    uint64_t nodes;               /* IR nodes of the program */
    uint64_t live_nodes;          /* nodes an output depends on */
    uint64_t arena_bytes;         /* intermediate values after liveness reuse */
    uint64_t unshared_bytes;      /* the same values with one buffer each */
    uint64_t param_bytes;         /* parameters (and moments, when the step has them) */
    uint64_t upload_bytes_per_step;
    uint64_t steps_run;
    uint64_t algorithmic_bytes_per_step; /* sum over launches of bytes read + written, the
                                            reference's counting rule (ir/kernel.rs:1562-1579) */
    uint64_t matmul_flop_per_step;       /* 2 m k n over the step's matmuls */
} msx_stats;

/* What a plan did, counted as it ran: RunStats of the reference (vulkan/runner.rs:87-131). One
 * submitted step is one submit (a CUDA graph launch) of `dispatches_per_step` kernels; kernels
 * of a stream run in order, so there are no barriers to count; `peak_device_bytes` is what the plan
 * allocated at creation (it allocates nothing afterwards). */
typedef struct msx_run_stats {
    uint64_t steps, host_waits, submits, dispatches, dispatches_per_step, barriers_per_step;
    uint64_t bytes_uploaded, bytes_downloaded, device_allocations, peak_device_bytes;
    uint32_t tolerance_class;   /* 0 bit-for-bit matmuls (MSX_PLAN_EXACT_MATMUL), 1 tolerance */
    double elapsed_us;          /* host time from the first submit to the end of the last wait */
} msx_run_stats;

/* Replaces the device-selection half of vulkan::runner::on_device
 * (crates/modelspec-runtime/src/vulkan/runner.rs:412-436). */
int msx_open(int ordinal, msx_device** out);
void msx_close(msx_device* device);

/* The message of the last failure: of `device`, or of the last msx_open when `device` is null. */
const char* msx_last_error(const msx_device* device);

/* Builds the execution plan of one program: the part of train_stepwise_profiled that creates
 * buffers and pipelines (vulkan/stepwise.rs:548-642). `ir_text` is a training step or a bare
 * tensor program (a forward program for the final loss line and for `infer`). `seed` keys the
 * dropout masks. `shares`, when not null, is a plan of the same device whose parameter buffers
 * this plan reads by canonical path instead of allocating its own (the reference runs its loss
 * and prediction steps on the training run's buffers, vulkan/runner.rs:541-566). */
int msx_plan_create(msx_device* device, const char* ir_text, uint64_t seed, uint32_t flags,
                    msx_plan* shares, msx_plan** out);
void msx_plan_destroy(msx_plan* plan);

/* Host inputs of a step, in node order: the data declarations, masked-row inputs, dropout tokens
 * and optimizer scalars (schedule::host_inputs, schedule.rs:723-750). AdamW moments are not
 * among them: they live on the device (msx_moment_upload). */
uint32_t msx_plan_input_count(const msx_plan* plan);
const char* msx_plan_input_name(const msx_plan* plan, uint32_t index);
uint64_t msx_plan_input_bytes(const msx_plan* plan, uint32_t index);
int msx_plan_input_is_i32(const msx_plan* plan, uint32_t index);

uint32_t msx_plan_param_count(const msx_plan* plan);
const char* msx_plan_param_path(const msx_plan* plan, uint32_t index);
uint64_t msx_plan_param_bytes(const msx_plan* plan, uint32_t index);

/* Parameter and moment transfer; `which` is 'm' or 'v'. Uploads and downloads are ordered after
 * every step already submitted. Replaces the upload at vulkan/stepwise.rs:605-642 and the
 * read-back of Run::state. */
int msx_param_upload(msx_plan* plan, uint32_t index, const void* host, uint64_t bytes);
int msx_param_download(msx_plan* plan, uint32_t index, void* host, uint64_t bytes);
int msx_moment_upload(msx_plan* plan, uint32_t index, char which, const void* host, uint64_t bytes);
int msx_moment_download(msx_plan* plan, uint32_t index, char which, void* host, uint64_t bytes);

/* Stages one host input of the next step. The bytes are checked the way the reference's
 * interpreter checks them before a run (cpu/interpreter.rs:700-715, :1146-1170, :1238-1254) and
 * copied; MSX_BAD_INPUT names the first offending element. An input not staged again keeps its
 * last value. */
int msx_set_input(msx_plan* plan, const char* name, const void* host, uint64_t bytes);

/* First element index of this plan's rows in the global batch, for dropout masks that must
 * match a single-device run over the whole batch (cpu/interpreter.rs:848-849); 0 by default.
 * `rows_before` counts rows of the leading dimension held by lower ranks. */
int msx_set_shard(msx_plan* plan, uint64_t rows_before, uint64_t global_rows);

/* Submits one step: the staged inputs are copied to the device and every kernel of the plan is
 * enqueued; returns without waiting. The loss of the step is read by msx_loss. Replaces one
 * recorded step of a segment (vulkan/stepwise.rs:975-1100). */
int msx_run(msx_plan* plan);

/* Waits for every submitted step (bounded by `timeout_ms`, MSX_TIMEOUT past it) and returns the
 * loss of the last one. */
int msx_loss(msx_plan* plan, float* loss, uint32_t timeout_ms);

/* The loss of submitted step `step_number` (counted from 0 over the plan's life) without waiting
 * for later steps; the last 8 submitted steps keep theirs. Lets a host read losses a few steps
 * behind the one it submits, as the reference observes a segment while the next one runs
 * (vulkan/stepwise.rs:976-1100). */
int msx_loss_of(msx_plan* plan, uint64_t step_number, float* loss, uint32_t timeout_ms);
uint64_t msx_steps_submitted(const msx_plan* plan);

/* Device time of submitted step `step_number` in milliseconds, between CUDA events recorded on
 * the plan's stream before its input copy and after its loss read-back; the last 8 submitted
 * steps keep theirs. With steps submitted back to back these times add up to the run's: the
 * per-step view of the reference's training clock (cli/src/train.rs:17-33), from which a host
 * takes the median step time the reference's benchmarks quote (vulkan/profile.rs:25). */
int msx_step_ms(msx_plan* plan, uint64_t step_number, float* ms);

/* Waits for every submitted step. */
int msx_sync(msx_plan* plan, uint32_t timeout_ms);

/* Reads the value `%value_id` of the last step. Every output of the program can be read (the
 * loss, the gradients; of a bare program, its outputs); other values are refused because their
 * storage is reused. */
int msx_value_download(msx_plan* plan, uint32_t value_id, void* host, uint64_t bytes);

int msx_plan_stats(const msx_plan* plan, msx_stats* out);
int msx_plan_run_stats(const msx_plan* plan, msx_run_stats* out);

/* The lines `train --stats` prints for a device run, field for field as RunStats displays them
 * (vulkan/runner.rs:143-163: `steps: N`, `host waits: N`, ... `pipeline creation us: T`). Copies at
 * most `capacity` bytes, NUL-terminated; returns the bytes needed. */
uint64_t msx_stats_report(const msx_plan* plan, char* out, uint64_t capacity);

/* The lines `train --profile` prints (Profile::report, vulkan/profile.rs:237-338): one
 * `profile dispatch <plan> <position> <kernel> <entry> calls <n> total_us <t> mean_us <m> flop <f>
 * bytes <b> gflop_per_s <g> gb_per_s <h>` line per launch of `plan` (named `step`) and, when not
 * null, of `final_plan` (named `final`), the counters of the run as `profile <counter> <value>`
 * lines, and `profile step_total ...`. The times come from msx_profile_step_repeated (a real
 * step runs on each plan; `repeats` as there). Returns 0 on failure (message in msx_last_error). */
uint64_t msx_profile_report(msx_plan* plan, msx_plan* final_plan, uint32_t repeats, char* out, uint64_t capacity);

/* For a plan made with MSX_PLAN_GUARD: waits for the submitted steps and checks the 16 sentinel
 * words after every intermediate value and scratch area. MSX_LAUNCH_FAILED names the first value
 * whose guard a kernel overwrote and the launch that last wrote that value. */
int msx_plan_check_guards(msx_plan* plan);

/* One line per scheduled kernel: `<index> <kernel> <value> reads ... writes ...`, the CUDA
 * counterpart of the `plan step` listing of `modelspec ir --stage kernel` (ir/print.rs:226-266).
 * Copies at most `capacity` bytes, NUL-terminated; returns the bytes needed. */
uint64_t msx_plan_describe(const msx_plan* plan, char* out, uint64_t capacity);

/* Per-launch device times of one step run kernel by kernel with a CUDA event after each launch
 * (not through the graph): the counterpart of the reference's `--profile` timestamps
 * (vulkan/profile.rs:1-60). `launch_ms` takes launches_per_step floats. The step is a real one:
 * parameters are updated. On a data-parallel plan every rank must make the call together: the
 * gradient buckets are summed across the ranks (on the plan's stream, outside any launch's time)
 * before the optimizer launch, so the replicas stay equal, and the launches that hold a
 * collective make the call run every launch once whatever `repeats` says. msx_launch_kernel / _bytes / _flop give each launch's kernel name and
 * its bytes read + written and FLOP by the reference's counting rule (ir/kernel.rs:1221-1306,
 * :1562-1579). */
int msx_profile_step(msx_plan* plan, float* launch_ms, uint32_t capacity);
/* The same with every launch issued `repeats` times back to back between its two events and the
 * time divided by `repeats`: a launch of a few microseconds is then timed at the rate the device
 * runs it rather than the rate the host can issue single launches. Every kernel of a step writes
 * a function of what it reads, so repeating it leaves the step's values unchanged; the optimizer
 * launch, which updates in place, is issued once. */
int msx_profile_step_repeated(msx_plan* plan, uint32_t repeats, float* launch_ms, uint32_t capacity);
const char* msx_launch_kernel(const msx_plan* plan, uint32_t launch);
uint64_t msx_launch_bytes(const msx_plan* plan, uint32_t launch);
uint64_t msx_launch_flop(const msx_plan* plan, uint32_t launch);

/* The same listing for a program without building a plan (no device needed), followed by one
 * line of totals: what `modelspec ir --stage kernel` is to the Vulkan backend. Returns 0 with
 * the reason in msx_last_error(NULL) when the program cannot be scheduled. */
uint64_t msx_schedule_describe(const char* ir_text, char* out, uint64_t capacity);
/* The same under plan flags (MSX_PLAN_EXACT_MATMUL, MSX_PLAN_BF16): a value that a mixed-precision
 * plan stores as bf16 is listed with the suffix `h`. */
uint64_t msx_schedule_describe_with(const char* ir_text, uint32_t flags, char* out, uint64_t capacity);

/* Device time of the steps run since the last call, in milliseconds, measured with CUDA events
 * on the plan's stream around each msx_run: the reference's training clock (cli/src/train.rs:
 * 17-33). Waits for the submitted steps. */
int msx_elapsed_ms(msx_plan* plan, double* total_ms, uint64_t* steps);

/* Data-parallel training over the GPUs of one box: every rank holds a plan of the same step
 * compiled for its shard of the batch; gradients are summed across ranks in buckets on a side
 * stream before the update. The reference has no counterpart (it is single-device).
 * `unique_id` is 128 bytes, made by rank 0 with msx_comm_unique_id and handed to the others by
 * the caller. */
int msx_comm_unique_id(void* unique_id_128);
int msx_comm_init(msx_plan* plan, int rank, int world, const void* unique_id_128);
/* Lets `plan` (a forward plan) use the communicator of `owner` for its loss reductions; `owner`
 * must outlive it, and the two must not run concurrently. */
int msx_comm_share(msx_plan* plan, msx_plan* owner);
/* How many all-reduces one step issues for its gradients (about 25 MB each). */
uint32_t msx_comm_bucket_count(const msx_plan* plan);
/* 1 when the gradient buckets are summed by this library's own kernel over peer memory (every
 * rank mapped every other rank's arena through CUDA IPC), 0 when by the NCCL all-reduce (a rank
 * could not map a peer, more than 8 ranks, or MSX_PEER_REDUCE=0 in the environment). */
uint32_t msx_comm_uses_peer_memory(const msx_plan* plan);
/* How long the optimizer launch of a data-parallel step waits for the gradient exchange after
 * the backward pass has ended, in milliseconds: runs ONE real step launch by launch (not through
 * the graph) on the staged inputs, with CUDA events on the plan's stream after the last launch
 * before the optimizer and right before the optimizer launch. Every rank makes the call together.
 * 0 for a plan that is not data parallel. */
int msx_comm_exposed_ms(msx_plan* plan, float* ms);
/* A check of the peer-memory all-reduce on ONE device: the launches of all `world` (2 to 8)
 * ranks of an emulated job run one after the other over `world` copies of `count` floats.
 * `host_copies[q]` is rank q's copy on the host, replaced by what the copy holds afterwards.
 * With `peers_present` non-zero the flag words start as if every rank had already arrived at
 * both rendezvous, so each launch goes straight to its slice; every copy must then hold
 * scale x the sum of the copies. With 0 only rank 0's launch runs and waits for ranks that never
 * come: it gives up after `wait_ms`, sums nothing, and a second launch returns at once because
 * the channel is marked failed. `*status_bits` receives the status word the launches left
 * (bit 1: a wait ran out). Nothing here needs a second GPU, and no launch waits for another. */
int msx_peer_reduce_check(msx_device* device, uint32_t world, uint64_t count, float* const* host_copies, float scale,
                          int peers_present, uint32_t wait_ms, uint32_t* status_bits);

/* ---- The training run above the plan -------------------------------------------------------
 *
 * The host loop of `train --backend cuda`, mirroring the reference's device runner
 * vulkan::stepwise::train_stepwise_on_device (crates/modelspec-runtime/src/vulkan/stepwise.rs:
 * 289-296, :400-) and the CPU loop it is compared with, train::runner::run_checked
 * (crates/modelspec-runtime/src/train/runner.rs:365-512): parameters drawn by their
 * initializers, per step the AdamW scalars of t = step + 1, the dropout token of every site,
 * the masked-row gather of the batch, one submitted step; the loss of step k is the loss before
 * update k; the final loss is the dropout-free forward program on the final parameters. */
typedef struct msx_training msx_training;

/* Compiles `source` (`.mspec`), builds the step plan and the forward plan on shared parameter
 * buffers, and uploads the initial parameters (Philox stream 0 under the train block's seed).
 * `masked_rows` as in msx_compile; `flags` are plan flags. */
int msx_training_create(msx_device* device, const char* source, uint64_t masked_rows, uint32_t flags,
                        msx_training** out);
void msx_training_destroy(msx_training* training);
msx_plan* msx_training_step_plan(msx_training* training);
msx_plan* msx_training_forward_plan(msx_training* training);
uint64_t msx_training_steps(const msx_training* training);   /* `steps` of the train block */
uint64_t msx_training_seed(const msx_training* training);
/* The message of the last failure of a msx_training_* call on `training`. */
const char* msx_training_last_error(const msx_training* training);

/* Makes the run one rank of a data-parallel job: joins the step plan to the communicator
 * (msx_comm_init), lets the forward plan use it, and offsets the dropout element indices by the
 * rows of the lower ranks (`rows_per_rank` rows of the leading dimension each), so that the
 * masks are those of one device running the whole batch. Call before the first step. */
int msx_training_comm_init(msx_training* training, int rank, int world, const void* unique_id_128,
                           uint64_t rows_per_rank);

/* Sets one declared `input` or `target` of the batch for the steps that follow (the dense feed
 * of train/data.rs:14-35; block k of a `--data` file is what the caller passes before step k). */
int msx_training_set_input(msx_training* training, const char* name, const void* host, uint64_t bytes);

/* The reference's synthetic batch (train/data.rs:189-212): the one f32 input standard normal,
 * key masks all ones, the target the prediction of a teacher drawn on the teacher stream, run on
 * the device. Refused unless the block declares one f32 input besides key masks and one f32
 * target. */
int msx_training_synthetic(msx_training* training);

/* Copies the current batch's declared input `name` out (after msx_training_synthetic). */
int msx_training_get_input(msx_training* training, const char* name, void* host, uint64_t bytes);

/* Submits step `step` of a run that ends at `end` (steps are counted from 0; `end` is
 * start + steps); returns without waiting. MSX_BAD_INPUT when the batch selects more rows than
 * the masked-row gather holds (the reference's E-DATA-012). */
int msx_training_step(msx_training* training, uint64_t step, uint64_t end);

/* Loss of run step `step` (as passed to msx_training_step), readable while later steps are in
 * flight; only the last 8 submitted steps keep theirs. */
int msx_training_loss_of(msx_training* training, uint64_t step, float* loss);

/* Loss of the last submitted step (waits for it). MSX_NON_FINITE when it is NaN or infinite
 * (the reference's E-TRAIN-001, train/runner.rs:162-228). */
int msx_training_loss(msx_training* training, float* loss);

/* The final loss line: the forward program, dropout the identity, on the current parameters and
 * the current batch. */
int msx_training_final_loss(msx_training* training, float* loss);

/* `infer --backend cuda`: the forward program, dropout the identity, on the current parameters and
 * the current batch, as the reference runs the loss steps of its plan once on the device
 * (vulkan/runner.rs:381-386; cli/src/infer.rs:1-60). `prediction` receives the output of the one
 * `model.forward(...)` call, row-major (msx_training_prediction_count elements), `loss` the loss of
 * the batch. msx_training_infer_report formats the two lines the CLI prints:
 * `prediction: <type> = [v, ...]` and `loss <v>`, numbers as Rust displays an f32
 * (infer.rs:251-262); returns the bytes needed, 0 on failure. */
uint64_t msx_training_prediction_count(const msx_training* training);
int msx_training_infer(msx_training* training, float* prediction, uint64_t bytes, float* loss);
uint64_t msx_training_infer_report(msx_training* training, char* out, uint64_t capacity);

/* ---- restore and replay --------------------------------------------------------------------------
 * The reference runs its steps in segments of several per submission, and when a step's loss is
 * not finite it stops the run at that step with the parameters and moments after that step, as
 * one step per submission leaves them: each segment first copies the state it starts from into a
 * device buffer of its own, and the failing segment copies it back and runs its steps through the
 * failing one again (crates/modelspec-runtime/src/vulkan/stepwise.rs:84-92, :1024-1082).
 *
 * msx_state_snapshot copies every parameter and moment of `plan` into a device buffer of the
 * plan's (allocated by the first call), msx_state_restore copies them back (and rewrites the bf16
 * working copies of a mixed-precision plan); both are ordered on the plan's stream and wait for
 * nothing. msx_training_set_replay_window(training, n) takes a snapshot before every n-th step and
 * keeps the batches of the steps since (n = 0, the default, takes none);
 * msx_training_rewind(training, step) then leaves the run as it was after the update of `step`, a
 * step at or after the last snapshot: snapshot restored, the steps from it through `step` run
 * again on their own batches, tokens and scalars. The steps after `step` are forgotten. */
int msx_state_snapshot(msx_plan* plan);
int msx_state_restore(msx_plan* plan);
int msx_training_set_replay_window(msx_training* training, uint32_t steps);
int msx_training_rewind(msx_training* training, uint64_t step);

/* ---- held-out evaluation (`--eval-every`) --------------------------------------------------------
 * Replaces the device side of the reference's held-out evaluation: every batch of the HeldOut
 * split runs the steps of the plan the prediction is computed from, dropout off, without the loss
 * sum, and the logits are reduced on the device to the weighted sum of the row losses and the
 * count of correct rows; one small state comes down per evaluation
 * (crates/modelspec-runtime/src/vulkan/stepwise.rs:32-46, :1648-1790;
 * spirv/emit/heldout.rs:1-24; train/eval.rs:167-355).
 *
 * The plan-level piece. `logits` names a rank-2 f32 output [rows, classes] of `plan` (a program
 * whose outputs hold the prediction). The labels and weights of all `batches` batches are
 * uploaded once (msx_heldout_targets; a label outside the classes is MSX_BAD_INPUT with the
 * reference's message, train/eval.rs:86-93) and stay on the device. An evaluation is
 * msx_heldout_begin, then for every batch in order: msx_set_input of its tensors, msx_run,
 * msx_heldout_add (all without a host wait), then msx_heldout_sums, the evaluation's one wait.
 * `numerator` is the f64 sum over every row, in batch and row order, of f64(weight) x f64(nll)
 * with nll = max + ln(sum exp(x - max)) - x[label] in f32 (rows of weight +0 and finite logits add
 * +0 without their softmax, eval.rs:436-442); `correct` counts the rows of positive weight whose
 * first largest logit (the lowest class among ties) is their label in a row without a NaN. */
typedef struct msx_heldout msx_heldout;
int msx_heldout_create(msx_plan* plan, uint32_t logits, uint32_t batches, msx_heldout** out);
void msx_heldout_destroy(msx_heldout* heldout);
int msx_heldout_targets(msx_heldout* heldout, uint32_t batch, const int32_t* labels, const float* weights, uint64_t rows);
int msx_heldout_begin(msx_heldout* heldout);
int msx_heldout_add(msx_heldout* heldout, uint32_t batch);
int msx_heldout_sums(msx_heldout* heldout, double* numerator, uint64_t* correct, uint32_t timeout_ms);

/* The whole evaluation of a training run. msx_training_heldout_begin declares `batches` held-out
 * batches and names the declared tensors that hold each row's label (i32) and weight (f32), which
 * the reduction reads whether or not the prediction depends on them; the prediction must be f32
 * logits [rows, V], one row per label (the reference's EvalError::Prediction otherwise).
 * msx_training_heldout_set gives batch `batch` its declared tensor `name` (every declared input the
 * prediction reads, and the labels and weights); the batches are drawn once per run and read by
 * every evaluation. msx_training_heldout_evaluate evaluates the current parameters:
 * loss = f32(numerator / sum of the weights), both whole-split f64 sums, 0 when the weights sum
 * to 0; accuracy = correct / selected in f32 over the rows of positive weight, 0 when none is
 * selected (HeldOut::metrics_of_sums, train/eval.rs:325-355). */
int msx_training_heldout_begin(msx_training* training, uint32_t batches, const char* labels, const char* weights);
int msx_training_heldout_set(msx_training* training, uint32_t batch, const char* name, const void* host, uint64_t bytes);
int msx_training_heldout_evaluate(msx_training* training, float* loss, float* accuracy);

/* ---- packed masked-language-model data (`train --data <packed directory>`) ----------------------
 * The directory the reference's `pack` writes: binding.json, packed.json, train.tokens and
 * heldout.tokens (little-endian i32 ids, sequences of exactly seq_len ids, no padding).
 * msx_packed_open reads and checks it as the reference does (dataset/mlm.rs:583-660,
 * train/data.rs:1443-1483, :1605-1613): the binding's id is the id of its fields, the record
 * lists a Train and a HeldOut split, 5 < vocabulary_size <= 2^31, every file has the length and
 * the blake3 hash of its record, every id is inside the vocabulary, and the record belongs to the
 * binding. MSX_BAD_INPUT with the reference's reason otherwise (msx_last_error(NULL)). */
typedef struct msx_packed msx_packed;
#define MSX_SPLIT_TRAIN 0
#define MSX_SPLIT_HELDOUT 1
int msx_packed_open(const char* dir, msx_packed** out);
void msx_packed_close(msx_packed* packed);
const char* msx_packed_last_error(const msx_packed* packed);
uint64_t msx_packed_seq_len(const msx_packed* packed);
uint64_t msx_packed_vocabulary(const msx_packed* packed);
uint64_t msx_packed_sequences(const msx_packed* packed, int split);
const char* msx_packed_binding_id(const msx_packed* packed);

/* The `data` line a run on a packed directory prints first (cli/src/train.rs:1506-1519); returns
 * the bytes needed. */
uint64_t msx_packed_data_line(const msx_packed* packed, char* out, uint64_t capacity);

/* The order in which epoch `epoch` of a run with seed `seed` visits the Train sequences
 * (dataset/mlm.rs:662-675); `count` is msx_packed_sequences(packed, MSX_SPLIT_TRAIN). */
int msx_packed_epoch_order(msx_packed* packed, uint64_t seed, uint64_t epoch, uint32_t* out, uint64_t count);

/* `mlm_batch` (dataset/mlm.rs:708-788): the batch of step `step` of a split for a run with seed
 * `seed` and `batch_size` sequences per step, flattened to batch_size * seq_len rows. Train step k
 * is batch k mod (n / B) of epoch k / (n / B) in epoch order; HeldOut step k is batch k mod (n / B)
 * in stored order, its masking drawn with id k + 2^63. Any output may be null. */
int msx_packed_batch(msx_packed* packed, int split, uint64_t seed, uint64_t step, uint64_t batch_size, int32_t* ids, int32_t* positions,
                     float* key_mask, int32_t* labels, float* weights);

/* Binds a packed directory to the run's declarations as the reference's `packed` does
 * (train/data.rs:1588-1745): every declaration names a batch tensor (E-DATA-005), has its dtype
 * and the shape [B, S] or [B*S] (E-DATA-006), is read by the loss (E-DATA-003); an embedding table
 * that reads `ids` and the logits of the cross_entropy that reads `labels` are as wide as the
 * packed vocabulary (E-DATA-006); the Train split holds at least B sequences. `packed` must
 * outlive the training. msx_training_feed_packed makes the Train batch of step `step` the current
 * batch (then msx_training_step). msx_training_heldout_packed draws the batches 0 .. n / B of the
 * HeldOut split once and declares them for msx_training_heldout_evaluate; fewer than B sequences is
 * the reference's EvalError::TooFewSequences (`dir` is named in that message). */
int msx_training_bind_packed(msx_training* training, msx_packed* packed);
int msx_training_feed_packed(msx_training* training, uint64_t step);
int msx_training_heldout_packed(msx_training* training, const char* dir);
uint32_t msx_training_heldout_batches(const msx_training* training);

/* ---- dense data (`train --data <directory>` without a binding file) ------------------------------
 * The reference's dense directory (train/data.rs:14-35): `<dir>/<name>.f32` or `<dir>/<name>.i32`
 * for every `input` and `target` declaration, row-major little-endian values without a header,
 * and an optional `<dir>/order.u32`. msx_dense_open takes the declarations in source order (name,
 * dtype, role, rank and shape: `is_target` is 0 for an input, 1 for a target and 2 for an argument
 * of a model function run as an inference entry, which the messages name so; `shapes` holds the
 * ranks[0] + ranks[1] + ... extents one after another) and the run's step count, and reads and checks the files as the reference does
 * (read_files :837-876, read_tensor :1232-1290, dense :513-577): B is the leading dimension all
 * declarations share, else 1; a file is a whole number of samples of finite values (E-DATA-007);
 * all files hold the same number N of samples (E-DATA-007); an order holds at least steps x B
 * indices, each below N (E-DATA-008). MSX_BAD_INPUT with the reference's reason otherwise
 * (msx_dense_last_error(NULL)). msx_dense_check_bound refuses an i32 file that holds a value
 * outside 0 .. bound - 1 (E-DATA-011, refuse_out_of_range :957-1004; `what` names the bound in
 * the message: "the 6 rows of the `embedding` table `Named.table`"). msx_dense_step copies the
 * batch of step `step` of declaration `index`: the samples order[(step B + i) mod len] with an
 * order, (step B + i) mod N without one (fill_step :446-454). */
typedef struct msx_dense msx_dense;
int msx_dense_open(const char* dir, uint32_t count, const char* const* names, const uint32_t* is_i32, const uint32_t* is_target,
                   const uint32_t* ranks, const uint64_t* shapes, uint64_t steps, msx_dense** out);
void msx_dense_close(msx_dense* dense);
const char* msx_dense_last_error(const msx_dense* dense);
uint64_t msx_dense_batch(const msx_dense* dense);
uint64_t msx_dense_samples(const msx_dense* dense);
int msx_dense_has_order(const msx_dense* dense);
uint32_t msx_dense_tensors(const msx_dense* dense);
uint64_t msx_dense_batch_bytes(const msx_dense* dense, uint32_t index);
int msx_dense_check_bound(msx_dense* dense, uint32_t index, uint64_t bound, const char* what);
int msx_dense_step(const msx_dense* dense, uint32_t index, uint64_t step, void* out, uint64_t capacity_bytes);
/* The directory of `--eval <dir>` (dense_eval, train/data.rs:582-600): the same files, `order.u32`
 * is not read, and N is a multiple of B (E-DATA-009). msx_dense_eval_batch copies batch `batch`:
 * the samples batch x B .. (batch + 1) x B (fill_eval_batch :456-460). */
int msx_dense_open_eval(const char* dir, uint32_t count, const char* const* names, const uint32_t* is_i32, const uint32_t* is_target,
                        const uint32_t* ranks, const uint64_t* shapes, msx_dense** out);
int msx_dense_eval_batch(const msx_dense* dense, uint32_t index, uint64_t batch, void* out, uint64_t capacity_bytes);

/* Binds a dense directory to the run's declarations (dense, read_dense :627-671): a declaration
 * the loss does not read is E-DATA-003; then the files as msx_dense_open reads them; then every
 * i32 file against the rows of the embedding table or the classes of the cross_entropy logits
 * that read it (E-DATA-011). The training owns the data it read. msx_training_feed_dense makes
 * the batch of step `step` the current batch (then msx_training_step); msx_training_run feeds a
 * bound dense directory as it feeds a packed one. */
int msx_training_bind_dense(msx_training* training, const char* dir);
int msx_training_feed_dense(msx_training* training, uint64_t step);
/* `--eval <dir>` (evaluate_dense, train/runner.rs:571-624): the forward program, dropout the
 * identity, on the current parameters over every batch of an eval directory. `loss` = the mean of
 * the batch losses, summed in f64; `accuracy` = the fraction of target rows whose prediction row
 * has its first maximum where the target row has its (a prediction row holding a NaN is never
 * correct), defined (`has_accuracy` = 1) when the block declares exactly one target, that target is
 * f32 and the loss is not the value `model.forward(...)` returns. The current batch is left as
 * the last eval batch. msx_training_eval_line formats the line the CLI prints last:
 * `eval loss=<loss>` and, when defined, ` accuracy=<accuracy>` (cli/src/train.rs:1553-1559). */
int msx_training_eval_dense(msx_training* training, const char* dir, double* loss, double* accuracy, int* has_accuracy);
uint64_t msx_training_eval_line(double loss, double accuracy, int has_accuracy, char* out, uint64_t capacity);

/* ---- a whole run and its standard output --------------------------------------------------------
 * `train --backend cuda` as one call: the steps `start` .. `start + steps` of the train block (the
 * run's `steps`; `start` > 0 after msx_training_resume), fed from the bound packed directory when
 * there is one and from the current batch otherwise (the reference's synthetic feed trains on one
 * batch), the held-out split evaluated at every multiple of `eval_every` and at the last step when
 * held-out batches are declared and `eval_every` > 0, and the loss after the last update from the
 * forward program without dropout. The text is the reference's standard output for the run
 * (crates/modelspec-cli/src/train.rs:7-17, :1494-1560): the `data` line of a packed run,
 * `init @<path>: <type> = [v, ...]` for every parameter in path order, `step <k> loss <v>` at the
 * first step, every 50 steps, the last step and every evaluated step, `eval <k> loss <l> accuracy
 * <a>` after an evaluated step's line, and `param @<path>: ...` for every parameter after the last
 * step; every f32 in its shortest round-trip form. A loss that is not finite stops the run at that
 * step (MSX_NON_FINITE, E-TRAIN-001): the text then ends with that step's line and has no `param`
 * lines. msx_training_report copies the text of the last run (returns the bytes needed). */
int msx_training_run(msx_training* training, uint64_t start, uint64_t eval_every);
uint64_t msx_training_report(const msx_training* training, char* out, uint64_t capacity);

/* ---- `.msckpt` checkpoints ------------------------------------------------------------------------
 * Writer and validating reader of the reference's checkpoint format version 1, byte for byte
 * (crates/modelspec-runtime/src/train/checkpoint.rs:1-22, :420-517, :640-921): 56-byte header,
 * compact JSON manifest, 64-byte-aligned little-endian f32 payloads in path order, blake3 checksum,
 * payload hash and checkpoint id. msx_checkpoint_read refuses what the reference's reader refuses,
 * with its codes in the message: E-CKPT-001 (header, checksum, manifest, invariants), E-CKPT-002
 * (sizes, offsets, alignment, overlap, non-zero gap bytes), E-CKPT-004 (payload hash);
 * MSX_BAD_INPUT, text from msx_last_error(NULL). A checkpoint is built with msx_checkpoint_new,
 * msx_checkpoint_set_optimizer and one msx_checkpoint_add per tensor (`slot` NULL for a parameter,
 * "m" / "v" for an AdamW moment, written as the manifest's optimizer_slots, which the reference's
 * format defines and its writer leaves empty). Lists: 0 the parameters, 1 the optimizer slots. */
typedef struct msx_checkpoint msx_checkpoint;
#define MSX_OPTIMIZER_SGD 0
#define MSX_OPTIMIZER_ADAMW 1
#define MSX_OPTIMIZER_OTHER 2 /* a kind this backend reads but does not run (Muon) */
int msx_checkpoint_new(uint64_t step, uint64_t seed, const char* schema_hash, msx_checkpoint** out);
void msx_checkpoint_destroy(msx_checkpoint* checkpoint);
const char* msx_checkpoint_last_error(const msx_checkpoint* checkpoint);
int msx_checkpoint_set_optimizer(msx_checkpoint* checkpoint, int kind, double learning_rate, double weight_decay, double beta1, double beta2,
                                 double epsilon, uint64_t warmup_steps);
int msx_checkpoint_add(msx_checkpoint* checkpoint, const char* path, const char* slot, const uint64_t* shape, uint32_t rank, const float* data);
/* The file's bytes: returns their count; copies them when `capacity` holds them. */
uint64_t msx_checkpoint_encode(msx_checkpoint* checkpoint, void* out, uint64_t capacity);
/* Writes `<path>.tmp`, then renames it over `path` (checkpoint.rs:629-665). */
int msx_checkpoint_write(msx_checkpoint* checkpoint, const char* path);
int msx_checkpoint_read(const char* path, msx_checkpoint** out);
uint64_t msx_checkpoint_step(const msx_checkpoint* checkpoint);
uint64_t msx_checkpoint_seed(const msx_checkpoint* checkpoint);
const char* msx_checkpoint_schema_hash(const msx_checkpoint* checkpoint);
const char* msx_checkpoint_id(const msx_checkpoint* checkpoint); /* set by encode, write and read */
int msx_checkpoint_optimizer(const msx_checkpoint* checkpoint, int* kind, double* learning_rate, double* weight_decay, double* beta1,
                             double* beta2, double* epsilon, uint64_t* warmup_steps);
uint64_t msx_checkpoint_optimizer_json(const msx_checkpoint* checkpoint, char* out, uint64_t capacity);
uint32_t msx_checkpoint_count(const msx_checkpoint* checkpoint, int list);
const char* msx_checkpoint_path(const msx_checkpoint* checkpoint, int list, uint32_t index);
const char* msx_checkpoint_slot(const msx_checkpoint* checkpoint, int list, uint32_t index);
uint32_t msx_checkpoint_rank(const msx_checkpoint* checkpoint, int list, uint32_t index);
const uint64_t* msx_checkpoint_shape(const msx_checkpoint* checkpoint, int list, uint32_t index);
const float* msx_checkpoint_data(const msx_checkpoint* checkpoint, int list, uint32_t index);

/* The checkpoint of a run after `step` updates (Checkpoint::of_state, checkpoint.rs:420-451): every
 * parameter read back from the device in path order, the schema hash of the training program's
 * parameters, the optimizer of the train block, the run's seed at counter 0; for AdamW also both
 * moments of every parameter. msx_training_resume loads it into a run (Checkpoint::resume_into,
 * checkpoint.rs:519-609): E-CKPT-003 at the first parameter path or shape that differs in path
 * order, then at a differing schema hash, then at a differing optimizer; an AdamW checkpoint of a
 * step above 0 without moments is refused as the reference refuses it (train/runner.rs:335-347).
 * `start_step` receives the checkpoint's step: the run continues with msx_training_step(start_step,
 * end), and equals the run that never stopped. */
int msx_training_checkpoint(msx_training* training, uint64_t step, msx_checkpoint** out);
int msx_training_resume(msx_training* training, const msx_checkpoint* checkpoint, uint64_t* start_step);
const char* msx_training_schema_hash(msx_training* training);

/* E-TRAIN-001 over the state: MSX_NON_FINITE naming the first parameter or moment that holds a
 * NaN or an infinity. Reads every parameter back; call it at the cadence the host can afford. */
int msx_training_check_finite(msx_training* training);

/* One matmul on the caller's device buffers, outside any plan: C[m, n] = op(A) x op(B) with
 * `a_transposed` meaning A is stored [k, m] and `b_transposed` meaning B is stored [n, k]
 * (the operand flags of the reference's matmul kernel, ir/kernel.rs:1013-1046). `exact` selects
 * the f32 fused-chain kernel; otherwise the tensor-core kernel runs, which needs
 * msx_op_matmul_workspace(m, n, k) floats of device scratch (0 when k is not split) and a device
 * status word (bit 1 is raised if a bounded wait inside the kernel runs out). Enqueues on
 * `stream` (a cudaStream_t) and returns. For profiling a single kernel on a small case and for
 * hosts that schedule themselves. */
int msx_op_matmul(const float* a, int a_transposed, const float* b, int b_transposed, float* c, uint64_t m, uint64_t n,
                  uint64_t k, float* workspace, uint64_t workspace_floats, uint32_t* status, void* stream, int exact);
uint64_t msx_op_matmul_workspace(uint64_t m, uint64_t n, uint64_t k);

/* The same for the mixed-precision kernel: `a` and `b` are bf16 device matrices (dense, on 16-byte
 * boundaries, row widths multiples of 8 elements), `c` is bf16 or f32 by `c_is_bf16`; the product
 * is formed by tcgen05.mma kind::f16 from TMA-loaded tiles with f32 accumulation. The reference
 * has no 16-bit type (ir/tensor.rs:38-51); this is the product a plan made with MSX_PLAN_BF16 runs.
 * `workspace` holds msx_op_matmul_bf16_workspace(m, n, k) floats (a split k; 0 otherwise). */
int msx_op_matmul_bf16(const void* a, int a_transposed, const void* b, int b_transposed, void* c, int c_is_bf16, uint64_t m,
                       uint64_t n, uint64_t k, float* workspace, uint64_t workspace_floats, uint32_t* status, void* stream);
uint64_t msx_op_matmul_bf16_workspace(uint64_t m, uint64_t n, uint64_t k);

/* The fused attention kernels of a mixed-precision plan on the caller's device buffers: q, k, v
 * (and g, the adjoint of the result) are bf16 [batch * len, heads * head_dim], `mask` is f32
 * [batch, k_len] of 0 / 1. Writes `out` (bf16) and `stats` (2 floats per (row, head): the softmax
 * maximum and sum); with `g` not null also dq, dk, dv (bf16, each may be null). The op is the
 * reference's Attention / AttentionGradQ/K/V (cpu/interpreter.rs:1035-1119); the score matrix
 * stays on the SM. Heads of up to 64 columns (a multiple of 8), up to 512 keys and queries. */
int msx_op_attention_bf16(const void* q, const void* k, const void* v, const float* mask, const void* g, void* out, void* dq, void* dk,
                          void* dv, float* stats, uint32_t batch, uint32_t q_len, uint32_t k_len, uint32_t heads, uint32_t head_dim,
                          uint32_t* status, void* stream);

/* The held-out row reduction on the caller's device buffers: the rows of `logits` (f32
 * [rows, classes], `pitch` floats between rows, 0 = classes) with their labels and weights are
 * added to `state`, 24 bytes {f64 numerator, u64 correct, u32 started, u32 arrived} that are zero
 * before the first batch of an evaluation. `scratch` holds 12 * rows bytes. One launch; what
 * msx_heldout_add runs (spirv/emit/heldout.rs:1-24 of the reference). */
int msx_op_heldout_rows(const float* logits, uint64_t pitch, const int32_t* labels, const float* weights, uint64_t rows, uint64_t classes,
                        void* scratch, void* state, void* stream);

/* Column sums without any allocation: out[c] = sum over rows of g[r, c] for a row-major
 * [rows, columns] device matrix, the `SumRows` of a bias gradient. This function has no
 * counterpart in the reference. It exists for hosts that cannot allocate device memory once they
 * run (all memory handed to their own pool, a loop that may not enter the allocator, a host
 * application that forbids it): it calls no cudaMalloc, cudaFree or allocating library routine.
 * Its partial sums live in a 1 MiB device array that is part of the library image on every GPU
 * that loads the library, until the process exits.
 *   - `device_g` and `device_out` are the caller's device buffers; `stream` is a cudaStream_t
 *     (null for the default stream). The call enqueues two kernels and returns.
 *   - `columns` must be between 1 and 4096; more is MSX_BAD_ARGUMENT, as are null pointers.
 *     The message is msx_static_last_error().
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture.
 *   - All calls on a device share the one array. Calls whose kernels can overlap on the GPU
 *     (different streams without an ordering between them) race on it: order them. Nothing in
 *     the array has to be cleared between calls, since each call writes every partial sum it
 *     later reads.
 * The result has the bits of a plan's `sum_rows`: the same first-stage kernels, the chunk sums
 * added in the same ascending order (here by a second launch). */
int msx_sum_rows_static(const float* device_g, uint64_t rows, uint64_t columns, float* device_out, void* stream);
const char* msx_static_last_error(void);

/* The `.mspec` front door, for hosts without the reference's compiler: lowers the train block
 * of `source`, differentiates it and attaches its optimizer. `which` is "step", "forward" (the
 * dropout-free program of the final loss line) or "tensor". `masked_rows` is the capacity of
 * the masked-row gather (passes/masked_rows.rs:117-206), 0 for none. Copies at most `capacity`
 * bytes; returns the bytes needed, or 0 on failure with the message in msx_last_error(NULL).
 * Mirrors compile::compile_training_with (crates/modelspec-core/src/compile.rs:85-116). */
uint64_t msx_compile(const char* source, const char* which, uint64_t masked_rows, char* out,
                     uint64_t capacity);

/* `infer --data <dir> --function <name> --out <path>` (crates/modelspec-cli/src/infer.rs:306-470):
 * msx_training_create_function makes a run of the model function `name` as an inference entry
 * (msx_compile_function below) instead of the train block: its arguments are the run's inputs, its
 * result the prediction. A name the model does not declare is E-DATA-010 naming its functions
 * (MSX_BAD_INPUT, text in msx_last_error(device)). msx_training_load_parameters loads a
 * checkpoint's parameters without its optimizer (Checkpoint::parameters_for, checkpoint.rs:519-585:
 * E-CKPT-003 at the first path, dtype or shape that differs in path order, then at a differing
 * schema hash); `step` (may be NULL) receives the checkpoint's step.
 * msx_training_refuse_out_reading refuses, before anything is read, an `out` that resolves to a
 * file the run reads: `model`, `checkpoint` (either may be NULL) or an argument's file of `dir`
 * (refuse_out_reading, train/data.rs:773-798; E-DATA-010; by canonical path, or by device and
 * inode for a hard link). msx_training_infer_dense binds every argument to `<dir>/<name>.f32|.i32`
 * as --eval binds a declaration (dense_function, train/data.rs:685-717: E-DATA-010 for a function
 * without arguments, E-DATA-007, E-DATA-011, E-DATA-009 when the samples are no whole number of
 * blocks of B), holds the result to one row per sample (row_elements :732-762, E-DATA-010), runs
 * the function on every block in block order and writes the results, row-major little-endian f32
 * without a header, to `out` through `.<name>.<pid>.tmp` beside it, synced and renamed over it, so
 * an existing `out` is replaced whole or not at all. `blocks` and `rows` are what the CLI prints:
 * `function <name> blocks <blocks> rows <rows> out <path>`. */
int msx_training_create_function(msx_device* device, const char* source, const char* name, uint32_t flags, msx_training** out);
int msx_training_load_parameters(msx_training* training, const msx_checkpoint* checkpoint, uint64_t* step);
int msx_training_refuse_out_reading(msx_training* training, const char* dir, const char* out, const char* model, const char* checkpoint);
int msx_training_infer_dense(msx_training* training, const char* dir, const char* out, uint64_t* blocks, uint64_t* rows);

/* A model function as an inference entry (compile::compile_function,
 * crates/modelspec-core/src/compile.rs:173-223): one input per argument, the function's result the
 * prediction, the result itself (rank 0) or its mean the loss, every dropout the identity, sgd at
 * the block's learning rate. `which` is "step", "forward" or "prediction" (the prediction's value
 * id, `%n`). A name the model does not declare fails with E-DATA-010 naming its functions. */
uint64_t msx_compile_function(const char* source, const char* name, const char* which, char* out, uint64_t capacity);

#ifdef __cplusplus
}
#endif

#endif /* MSX_H */
