// Launchers of the sm_100a kernels of the training step. Every launcher enqueues on `stream` and
// returns; none allocates or synchronises. Pointers are device pointers unless named `h_`.
//
// The translation units are compiled with -fmad=false: a multiply and an add written apart stay
// two rounded operations, and every fused multiply-add is written as fmaf. That keeps each
// kernel's rounding sequence the one its comment states.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace msx {
namespace k {

// A device array whose elements are f32 or, in a mixed-precision plan, bf16. The launchers that
// take these compute in f32 whatever the storage; the activation operands of one launch are all of
// one type (parameters, partial sums and whole-tensor results are always f32). A plain float
// pointer converts to either.
struct In {
    const void* p = nullptr;
    bool half = false;
    In() = default;
    In(const float* f) : p(f) {}
    In(const void* q, bool h) : p(q), half(h) {}
    explicit operator bool() const { return p != nullptr; }
    const float* f32() const { return static_cast<const float*>(p); }
};
struct Out {
    void* p = nullptr;
    bool half = false;
    Out() = default;
    Out(float* f) : p(f) {}
    Out(void* q, bool h) : p(q), half(h) {}
    explicit operator bool() const { return p != nullptr; }
    float* f32() const { return static_cast<float*>(p); }
    operator In() const { return In(p, half); }
};

// ---- pointwise (pointwise.cu) -----------------------------------------------------------------
enum class Binary : int { Add, Sub, Mul, Div };
// out[i] = a[i] op b[i]; an operand with `*_scalar` set is one element read for every i.
void binary(cudaStream_t s, Binary op, const float* a, bool a_scalar, const float* b, bool b_scalar,
            float* out, uint64_t n);
enum class Unary : int { Relu, Sqrt, Gelu, Copy };
void unary(cudaStream_t s, Unary op, In a, Out out, uint64_t n);
// out[i] = a[i] > 0 ? g[i] : 0 (relu) or gelu'(a[i]) * g[i] (gelu).
void relu_grad(cudaStream_t s, const float* a, const float* g, float* out, uint64_t n);
void gelu_grad(cudaStream_t s, In a, In g, Out out, uint64_t n);
void fill_from_scalar(cudaStream_t s, const float* scalar, float* out, uint64_t n);
// out[r, c] = x[r, c] + b[c]
void add_rows(cudaStream_t s, const float* x, const float* b, float* out, uint64_t rows, uint64_t h);
// out[c, r] = a[r, c]
void transpose(cudaStream_t s, const float* a, float* out, uint64_t rows, uint64_t cols);

// Philox4x32-10 dropout: element i (global index index_base + i) is kept iff word 0 of
// philox([index, 4, token[0], token[1]], [seed lo, seed hi]) >= threshold; kept -> x * scale,
// dropped -> +0. `token` is the i32[2] device input of the site.
void dropout(cudaStream_t s, In x, const int32_t* token, uint64_t seed, uint32_t threshold,
             float scale, uint64_t index_base, Out out, uint64_t n);

// ---- reductions (reduce.cu) -------------------------------------------------------------------
// Whole-tensor sums in f64, rounded to f32 once. `scratch` holds at least reduce_scratch_doubles()
// doubles.
uint64_t reduce_scratch_doubles();
void reduce_sum(cudaStream_t s, const float* a, uint64_t n, bool mean, double* scratch, float* out);
void mse(cudaStream_t s, const float* a, const float* b, uint64_t n, double* scratch, float* out);
// out[c] = sum over rows of g[r, c]. `scratch` holds sum_rows_scratch_floats(rows, h) floats.
uint32_t sum_rows_chunks(uint64_t rows);
uint64_t sum_rows_scratch_floats(uint64_t rows, uint64_t h);
// `counters`, when not null, is sum_rows_counters(h) words that are zero before the first launch
// and left zero by every launch: the chunk sums are then combined by the same launch (same order,
// same result) instead of a second one.
// With `out` null only the chunk sums are written, as scratch[chunk][h]: finalize_sums adds them.
uint64_t sum_rows_counters(uint64_t h);
void sum_rows(cudaStream_t s, In g, uint64_t rows, uint64_t h, float* scratch, float* out,
              uint32_t* counters = nullptr, uint64_t ld = 0);

// The first stages of many column sums (the bias gradients of a step) in one launch: job j sums
// the rows of g ([rows, width], pitch ld) in sum_rows_chunks(rows) chunks into
// partial[chunk][width], as sum_rows with a null `out` does; finalize_sums adds the chunks.
// `first_block` = the blocks (row_sum_job_blocks each) of the jobs before this one.
struct RowSumJob {
    const void* g;
    float* partial;
    uint32_t rows, width, ld, rows_per_chunk, first_block, half;  // half: g holds bf16 elements
};
RowSumJob row_sum_job(In g, float* partial, uint64_t rows, uint64_t h, uint64_t ld, uint32_t first_block);
uint32_t row_sum_job_blocks(uint64_t rows, uint64_t h);
void sum_rows_batched(cudaStream_t s, const RowSumJob* d_jobs, uint32_t jobs, uint32_t blocks);

// Deferred second stages. A kernel that leaves `chunks` partial results of `width` floats each,
// stored [chunk][width], is finished by one launch over all such jobs of a step: up to 64 chunks
// are added in ascending order; beyond that thread y of 8 adds chunks y, y + 8, ... in ascending
// order and the eight sums are added in ascending y (deterministic; tolerance class against a
// sequential sum). `first_block` = the blocks
// (sum_job_blocks each) of the jobs before this one.
struct SumJob {
    const float* partial;
    float* out;
    uint32_t chunks, width, first_block, reserved;
};
inline uint32_t sum_job_blocks(uint32_t chunks, uint64_t width) {
    return static_cast<uint32_t>(chunks <= 64 ? (width + 255) / 256 : (width + 31) / 32);
}
void finalize_sums(cudaStream_t s, const SumJob* d_jobs, uint32_t jobs, uint32_t blocks);

// ---- row kernels (rowwise.cu) -----------------------------------------------------------------
// `ld`, `ld_out`, `ld_grad`: elements between the rows of the logits and of the gradient as stored
// (0 = the row width v). A width that is not a multiple of 4 is stored with the pitch rounded up,
// so that rows start on 16-byte boundaries; the padding is never read as data.
void layer_norm(cudaStream_t s, const float* x, const float* gamma, const float* beta, float* out,
                uint64_t rows, uint64_t h);
void layer_norm_grad_x(cudaStream_t s, const float* x, const float* gamma, const float* g, float* out,
                       uint64_t rows, uint64_t h);
// dgamma[c] = sum_r g[r, c] * xhat[r, c]; dbeta[c] = sum_r g[r, c] when dbeta is not null.
// `scratch` holds layer_norm_grad_gamma_scratch_floats(rows, h) floats.
uint64_t layer_norm_grad_gamma_scratch_floats(uint64_t rows, uint64_t h);
void layer_norm_grad_gamma(cudaStream_t s, const float* x, const float* g, float* scratch,
                           float* dgamma, float* dbeta, uint64_t rows, uint64_t h);
// layer_norm_grad_x (into dx, with gamma), layer_norm_grad_gamma (dgamma) and the column sums of g
// (dbeta) in one launch, for rows of up to 1,024 elements. dx, dgamma and dbeta may each be null.
// `scratch` holds layer_norm_backward_scratch_floats(rows, h) floats; `counter` is one word that
// is zero before the first launch and left zero by every launch.
// With `counter` null the chunk sums stay in `scratch` for finalize_sums: dgamma's as
// scratch[chunk][h], dbeta's after them, layer_norm_backward_chunks(rows, h) chunks each; the dgamma
// and dbeta pointers then only say which are wanted.
bool layer_norm_backward_supported(uint64_t h);
uint32_t layer_norm_backward_chunks(uint64_t rows, uint64_t h);
uint64_t layer_norm_backward_scratch_floats(uint64_t rows, uint64_t h);
// g1, g2, g3, when not null, are further addends of the adjoint: the kernel reads ((g + g1) + g2) + g3
// where the program has a chain of Adds that nothing else reads.
// A dropout draw for `dropout`'s element numbering: element i of the matrix is kept iff word 0 of
// its Philox block is at least `threshold`, and is then multiplied by `scale`.
struct DropoutDraw {
    const int32_t* token = nullptr;
    uint64_t seed = 0;
    uint32_t threshold = 0;
    float scale = 1.0f;
    uint64_t index_base = 0;
    // The keep decisions of the site as one bit per element, 32 consecutive columns of a row per
    // word (rows of a multiple of 32 columns only). A launch that draws the site writes them when
    // `bits` is set and `stored` is not; a later launch of the same step (the dropout_grad of the
    // site) given `stored` reads them instead of drawing again. Null: every launch draws.
    uint32_t* bits = nullptr;
    bool stored = false;
};
// `adjoint_draw`, when not null: the adjoint is dropout_grad of that sum. `dx_draw` and `dx_dropped`,
// when not null: dropout_grad of dx is written to dx_dropped beside dx. `pre_activation` and
// `dx_dropped`: gelu_grad(pre_activation, dx) is written to dx_dropped instead; dx may then be null.
void layer_norm_backward(cudaStream_t s, In x, const float* gamma, In g, Out dx, float* scratch,
                         uint32_t* counter, float* dgamma, float* dbeta, uint64_t rows, uint64_t h, In g1 = In(),
                         In g2 = In(), In g3 = In(), const DropoutDraw* adjoint_draw = nullptr,
                         const DropoutDraw* dx_draw = nullptr, Out dx_dropped = Out(), In pre_activation = In());
// sum_out = residual + dropout(x), out = layer_norm(sum_out, gamma, beta), rows of up to 1,024
// elements (layer_norm_backward_supported(h)); the dropout draw is that of `dropout`.
void dropout_add_layer_norm(cudaStream_t s, In x, In residual, const int32_t* token, uint64_t seed,
                            uint32_t threshold, float scale, uint64_t index_base, const float* gamma, const float* beta,
                            Out sum_out, Out out, uint64_t rows, uint64_t h);
// The general form: sum_out = residual + x (x through `x_draw` first when not null); with gamma
// and beta, out = layer_norm(sum_out) (out may be null when only the next output is wanted) and,
// with `out_draw`, out_dropped = dropout(out).
// With `gelu_first`, gelu(x) stands where the sum does (residual is null then): sum_out = gelu(x).
// sum_out may be null when only the layer norm is wanted (a plain layer norm: residual null too).
void add_layer_norm(cudaStream_t s, In x, In residual, const DropoutDraw* x_draw, const float* gamma,
                    const float* beta, Out sum_out, Out out, const DropoutDraw* out_draw, Out out_dropped, uint64_t rows,
                    uint64_t h, bool gelu_first = false);
void softmax(cudaStream_t s, const float* x, float* out, uint64_t rows, uint64_t k);
void softmax_grad(cudaStream_t s, const float* y, const float* g, float* out, uint64_t rows, uint64_t k);
// Row losses max + ln(sum exp(x - max)) - x[label] into row_loss[rows], then
// loss = sum w * l / sum w (f64 sums, one rounding; 0 when the weights sum to 0).
// `global_den`, when not null, is a device float that replaces the weight sum in the division:
// a data-parallel shard divides its own numerator by the weight sum of the whole batch.
void cross_entropy(cudaStream_t s, In logits, const int32_t* labels, const float* weights,
                   float* row_loss, const float* global_den, float* loss, uint64_t rows, uint64_t v, uint64_t ld = 0);
// out[0] = f32(sum of the weights in f64).
void weight_sum(cudaStream_t s, const float* weights, uint64_t rows, float* out);
// out[n, c] = g * w[n] / f32(sum w) * (softmax(logits[n])[c] - [c == labels[n]]); all 0 when the
// weights sum to 0. `denominator` is a one-float scratch the launcher fills with the weight sum,
// unless `denominator_ready` says the caller already put the (whole-batch) sum there.
void cross_entropy_grad(cudaStream_t s, const float* logits, const int32_t* labels, const float* weights,
                        const float* g, bool denominator_ready, float* denominator, float* out, uint64_t rows,
                        uint64_t v, uint64_t ld = 0, uint64_t ld_out = 0);

// Both at once, one visit of each logits row: `loss` as cross_entropy gives it, `grad` as
// cross_entropy_grad gives it. `denominator` as in cross_entropy_grad; when it is ready (data
// parallel) the loss divides by it too. `counter`, when not null, is one word that is zero before
// the first launch and left zero by every launch: rows of up to 32,768 logits then take one
// launch in all (weight sum and final loss included) and one read of the logits from memory.
void cross_entropy_with_grad(cudaStream_t s, In logits, const int32_t* labels, const float* weights,
                             const float* g, bool denominator_ready, float* denominator, float* row_loss, float* loss,
                             Out grad, uint64_t rows, uint64_t v, uint32_t* counter = nullptr, uint64_t ld = 0,
                             uint64_t ld_grad = 0);

// ---- held-out reduction (heldout.cu) -----------------------------------------------------------
// The running sums of one evaluation, all zero before its first batch.
struct HeldOutState {
    double numerator;            // sum of f64(w) x f64(nll) over every row so far, in batch and row order
    unsigned long long correct;  // rows of positive weight whose first largest logit is their label
    uint32_t started;            // whether the numerator holds a term yet (the first term starts the sum)
    uint32_t arrived;            // rows of the batch in flight that are done; zero between launches
};
// Adds the rows of one batch of logits [rows, classes] (row pitch `pitch` floats, 0 = classes) to
// `state`: one launch. `terms[rows]` and `hits[rows]` are scratch. A label outside the classes
// reads class 0: the host refuses such a batch before it is evaluated.
void heldout_rows(cudaStream_t s, const float* logits, uint64_t pitch, const int32_t* labels, const float* weights, uint64_t rows,
                  uint64_t classes, double* terms, uint32_t* hits, HeldOutState* state);

// ---- all-reduce over peer memory (peer_reduce.cu) ---------------------------------------------
// `buffers[q]` is rank q's copy of the same `count` floats (this rank's own for q == rank, the
// others mapped through CUDA IPC), `flags[q]` rank q's flag words (one per rank, zero before the
// first launch). `epoch`, `arrivals` and `failed` are words of this rank's own, zero before the
// first launch; every rank launches the same sequence of reductions on a channel (one stream),
// one channel per set of these words. After the launch every copy holds scale x the sum over the
// ranks, added in rank order by the rank that owns the element's slice. A wait that runs out
// (10 s unless `wait_nanoseconds` says otherwise) raises bit 1 of *status and sets *failed, after which launches on the channel return
// without waiting or summing.
constexpr int kPeerRanks = 8;
struct PeerReduceArgs {
    float* buffers[kPeerRanks];
    uint32_t* flags[kPeerRanks];
    uint32_t* epoch;
    uint32_t* arrivals;
    uint32_t* failed;
    uint32_t* status;
    uint32_t rank, world;
    uint64_t count;
    float scale;
    uint64_t wait_nanoseconds;  // 0: the default limit
};
void peer_all_reduce(cudaStream_t s, const PeerReduceArgs& args);

// ---- embedding (embedding.cu) -----------------------------------------------------------------
// out[n, :] = table[ids[n], :]; an id outside [0, rows) writes zeros and raises bit 0 of *status.
void embedding(cudaStream_t s, In table, const int32_t* ids, Out out, uint64_t n,
               uint64_t rows, uint64_t h, uint32_t* status);
// out = zeros[rows, h] with g[n, :] added to row ids[n] in ascending n: bit-exact with a
// sequential loop. `scratch` holds embedding_grad_scratch_ints(n, rows) ints. With `base`
// ([rows, h]) the result is base + that tensor, element by element.
uint64_t embedding_grad_scratch_ints(uint64_t n, uint64_t rows);
void embedding_grad(cudaStream_t s, const int32_t* ids, In g, Out out, uint64_t n,
                    uint64_t rows, uint64_t h, int32_t* scratch, uint32_t* status, const float* base = nullptr);
// Its two halves: the order of the occurrences depends on the ids alone and can be computed as
// soon as they are on the device (beside the forward pass); the scatter needs g.
void embedding_order(cudaStream_t s, const int32_t* ids, uint64_t n, uint64_t rows, int32_t* scratch, uint32_t* status);
void embedding_scatter(cudaStream_t s, In g, Out out, uint64_t n, uint64_t rows, uint64_t h, const int32_t* scratch,
                       const float* base = nullptr);

// ---- matmul (gemm.cu) -------------------------------------------------------------------------
// C[m, n] = op(A) x op(B) (+ bias[n]) with each element one ascending-k fused chain starting
// from its first product. `a_t`: A is stored [k, m] and read transposed; `b_t`: B stored [n, k].
// `bias`, when not null, is a row of n floats added to every row of the product (one more
// rounding per element, the add_rows the reference runs as its own kernel).
void matmul(cudaStream_t s, const float* a, bool a_t, const float* b, bool b_t, float* c,
            uint64_t m, uint64_t n, uint64_t k, const float* bias = nullptr);

// ---- matmul on tensor cores (gemm_tc.cu) ------------------------------------------------------
// The same product by tcgen05.mma with a 3xTF32 operand split and f32 accumulation in tensor
// memory: tolerance class (about 2^-21 of each |a||b| term). `workspace` holds
// matmul_tc_plan(m, n, k).workspace_floats floats (split-K partial tiles; 0 when k is not split).
// A wait that runs out inside the kernel raises bit 1 of *status instead of hanging. With
// `leave_partials` a split k stops at the partial tiles, workspace[split][m][n], for
// finalize_sums (no bias then).
struct MatmulTcPlan {
    uint32_t bm, bn, splits, kblocks_per_split;  // tile rows (64 or 128) and width, k split
    uint64_t workspace_floats;
};
// `problems` > 1: that many independent batched products in one launch (k is then not split);
// `group` > 1: that many products of this shape in one launch of matmul_tc_group (the workspace
// size is per product).
// `wide_ok`: the operands can be TMA sources (bases on 16 bytes, row pitches multiples of 4
// floats), which the 128 x 128 tile needs.
MatmulTcPlan matmul_tc_plan(uint64_t m, uint64_t n, uint64_t k, uint64_t problems = 1, uint64_t group = 1, bool wide_ok = true);
void matmul_tc(cudaStream_t s, const float* a, bool a_t, const float* b, bool b_t, float* c, uint64_t m,
               uint64_t n, uint64_t k, float* workspace, uint32_t* status, const float* bias = nullptr,
               bool leave_partials = false);

// Up to 4 products of one shape and one storage form in one launch (the query, key and value
// projections of a layer, their input gradients, their weight gradients): the CTAs of all of them
// share the SMs, where each alone fills a fraction of the device.
struct MatmulOperands {
    const float* a;
    const float* b;
    float* c;
    const float* bias;   // may be null
    float* workspace;    // matmul_tc_plan(m, n, k, 1, count).workspace_floats floats, or null when that is 0
};
// Elements between the rows of A, B and C as stored; 0 = dense (the row width). A pitched C needs
// an unsplit k (matmul_tc_plan(...).splits == 1).
struct MatmulPitches {
    uint32_t a = 0, b = 0, c = 0;
};
void matmul_tc_group(cudaStream_t s, const MatmulOperands* products, uint32_t count, bool a_t, bool b_t, uint64_t m, uint64_t n,
                     uint64_t k, uint32_t* status, bool leave_partials = false, MatmulPitches pitches = {});

// Products of different shapes, one storage form, in one launch (the weight gradients of a step,
// which only the optimizer reads and which would each fill a fraction of the device for a few
// microseconds). A job whose k is split (matmul_tc_job_plan(m, n, k).splits > 1) leaves its partial
// tiles in `workspace`, [split][m][n], for finalize_sums; otherwise it writes `c`.
struct MatmulJob {
    const float* a;
    const float* b;
    float* c;
    float* workspace;  // matmul_tc_job_plan(m, n, k).workspace_floats floats, or null when that is 0
    uint64_t m, n, k;
};
constexpr uint32_t kMatmulJobs = 24;  // jobs one launch carries
MatmulTcPlan matmul_tc_job_plan(uint64_t m, uint64_t n, uint64_t k);
void matmul_tc_jobs(cudaStream_t s, const MatmulJob* jobs, uint32_t count, bool a_t, bool b_t, uint32_t* status);

// outer x inner independent products through one launch (grid.z = problem): matrix z of an
// operand starts at base + (z / inner) * stride_outer + (z % inner) * stride_inner elements and
// has `pitch` elements between rows as stored; `transposed` as in matmul (A stored [k, m], B
// stored [n, k]). k is not split.
struct BatchedOperand {
    const float* base;
    uint32_t pitch;
    uint64_t stride_outer, stride_inner;
    bool transposed;
};
void matmul_tc_batched(cudaStream_t s, const BatchedOperand& a, const BatchedOperand& b, const BatchedOperand& c,
                       uint64_t m, uint64_t n, uint64_t k, uint32_t outer, uint32_t inner, uint32_t* status);

// ---- matmul on bf16 operands (gemm_bf16.cu) ---------------------------------------------------
// Mixed-precision plans: operands stored as bf16, products by tcgen05.mma kind::f16 fed by TMA,
// f32 accumulation, the result stored as bf16 or f32. An operand is `outer` x `inner` matrices of
// `pitch` elements between rows; matrix (o, i) starts stride_outer * o + stride_inner * i elements
// after `base`. `transposed`: A is stored [k, m], B is stored [n, k] (as for the f32 kernels).
// TMA sources: base on a 16-byte boundary, pitch and strides multiples of 8 elements.
struct HalfMatrix {
    const void* base;  // bf16 elements
    uint32_t pitch;
    uint64_t stride_outer, stride_inner;
    bool transposed;
};
struct HalfResult {
    void* base;
    bool half;       // bf16 elements, else f32
    uint32_t pitch;  // 0 = n
    uint64_t stride_outer, stride_inner;
};
struct MatmulBf16Plan {
    uint32_t bn, splits, kblocks_per_split;
    uint64_t workspace_floats;  // split-k partial tiles [split][m][n]; 0 when k is not split
};
MatmulBf16Plan matmul_bf16_plan(uint64_t m, uint64_t n, uint64_t k, uint64_t problems = 1);
// `workspace` holds matmul_bf16_plan(m, n, k, outer * inner).workspace_floats floats. With
// `leave_partials` a split k stops at the partial tiles for finalize_sums (no bias then). A wait
// that runs out inside the kernel raises bit 1 of *status.
void matmul_bf16(cudaStream_t s, const HalfMatrix& a, const HalfMatrix& b, const HalfResult& c, uint64_t m, uint64_t n, uint64_t k,
                 uint32_t outer, uint32_t inner, float* workspace, const float* bias, uint32_t* status, bool leave_partials = false);

// ---- attention (attention.cu) -----------------------------------------------------------------
struct AttentionShape {
    uint32_t batch, q_len, k_len, heads, head_dim;  // q rows = batch * q_len, k rows = batch * k_len
};
// Row statistics shared by the backward kernels: stats[(row * heads + head) * 3 + {0, 1, 2}] =
// max score, sum of exp(score - max), sum_j P[row, j] dP[row, j].
uint64_t attention_stats_floats(AttentionShape shape);
void attention_forward(cudaStream_t s, const float* q, const float* k, const float* v, const float* mask,
                       float* out, AttentionShape shape);
// Writes `stats`; `dq` may be null when only the statistics are wanted.
void attention_grad_q(cudaStream_t s, const float* q, const float* k, const float* v, const float* mask,
                      const float* g, float* stats, float* dq, AttentionShape shape);
// Reads the `stats` attention_grad_q wrote for the same operands; dk and dv may each be null.
void attention_grad_kv(cudaStream_t s, const float* q, const float* k, const float* v, const float* mask,
                       const float* g, const float* stats, float* dk, float* dv, AttentionShape shape);

// The same ops as batched tensor-core matmuls with row kernels between them (attention_tc.cu):
// tolerance class. `p` and `dp` each hold attention_tc_scratch_floats(shape) floats.
uint64_t attention_tc_scratch_floats(AttentionShape shape);
void attention_tc_forward(cudaStream_t s, const float* q, const float* k, const float* v, const float* mask,
                          float* out, float* p, AttentionShape shape, uint32_t* status);
// dq, dk and dv may each be null. `p_ready`: `p` still holds what attention_tc_forward left there
// for the same operands (the probabilities are then not computed again); it is only read.
void attention_tc_backward(cudaStream_t s, const float* q, const float* k, const float* v, const float* mask,
                           const float* g, float* dq, float* dk, float* dv, float* p, float* dp,
                           AttentionShape shape, uint32_t* status, bool p_ready = false);

// The same for a mixed-precision plan: q, k, v, g, out and the gradients are bf16 [rows, H], `p`
// (kept for the backward) and `ds` hold attention_tc_scratch_floats(shape) bf16 elements, `scores`
// as many floats (the f32 scores, then the f32 score adjoints; dead after the call).
void attention_bf16_forward(cudaStream_t s, const void* q, const void* k, const void* v, const float* mask, void* out, void* p,
                            float* scores, AttentionShape shape, uint32_t* status);
void attention_bf16_backward(cudaStream_t s, const void* q, const void* k, const void* v, const float* mask, const void* g, void* dq,
                             void* dk, void* dv, void* p, void* ds, float* scores, AttentionShape shape, uint32_t* status,
                             bool p_ready = false);

// Fused attention for mixed-precision plans (attention_fused.cu): the forward as one kernel that
// never stores the scores (it writes O and, per (row, head), the softmax maximum and sum:
// attention_fused_stats_floats(shape) floats), the three gradients as one kernel that reads those
// statistics and O. Heads of up to 64 columns (a multiple of 8), up to 512 keys and queries a
// sequence; attention_fused_supported says whether a shape qualifies. dq, dk, dv may each be null.
bool attention_fused_supported(AttentionShape shape);
uint64_t attention_fused_stats_floats(AttentionShape shape);
void attention_fused_forward(cudaStream_t s, const void* q, const void* k, const void* v, const float* mask, void* out, float* stats,
                             AttentionShape shape, uint32_t* status);
void attention_fused_backward(cudaStream_t s, const void* q, const void* k, const void* v, const float* mask, const void* g, const void* o,
                              const float* stats, void* dq, void* dk, void* dv, AttentionShape shape, uint32_t* status);

// ---- optimizer (optimizer.cu) -----------------------------------------------------------------
struct UpdateTensor {
    float* p;
    const float* g;
    float* m;
    float* v;
    uint64_t count;
    void* p16;  // the bf16 working copy of p that a mixed-precision plan's matmuls read, or null
};
struct AdamWConstants {
    float beta1, rest1, beta2, rest2, eps, weight_decay;
};
// One launch over every tensor of `d_tensors` (a device array of `tensors` entries; `chunks` =
// d_chunk_tensor/d_chunk_start entries of kUpdateChunk elements each). p, m, v are updated in
// place with the reference's 16 rounded f32 operations per element.
constexpr uint32_t kUpdateChunk = 4096;
void adamw(cudaStream_t s, const UpdateTensor* d_tensors, const uint32_t* d_chunk_tensor,
           const uint32_t* d_chunk_start, uint32_t chunks, AdamWConstants c, const float* lr_t,
           const float* c1, const float* c2);
// p16[i] = bf16(p[i]): the working copy of a parameter after its f32 master was uploaded.
void working_copy(cudaStream_t s, const float* p, void* p16, uint64_t n);
// p -= lr * g, `lr` a device scalar.
void sgd(cudaStream_t s, const UpdateTensor* d_tensors, const uint32_t* d_chunk_tensor,
         const uint32_t* d_chunk_start, uint32_t chunks, const float* lr);

}  // namespace k
}  // namespace msx
