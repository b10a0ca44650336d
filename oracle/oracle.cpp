// TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the test suite, the smoke check and the benchmark's
// CPU-baseline leg load this library; the CUDA backend never does.
//
// A CPU restatement of ModelSpec's reference interpreter and training loop: the arithmetic the
// CUDA backend is held to. The reference is Rust and cannot be built where this runs, so this is
// a port ("kind: port"), pinned by the reference's own recorded outputs: the Philox and BLAKE3
// known answers, the linear-regression training log (initial parameters, losses, final
// parameters), the 501 and 201 per-step losses of two recorded runs, and the transformer-block
// first-step loss. No recorded CPU output exists for the BERT-only ops (embedding, dropout,
// cross-entropy, AdamW); for those, parity is pinned by restatement and known answers, not by
// recorded vectors.
//
// Each function cites what it follows under crates/modelspec-runtime/src/ of the reference:
//   cpu/interpreter.rs:8-56     the reduction-order contract
//   cpu/interpreter.rs:860-1139 every op (eval_node)
//   cpu/matmul.rs:268-292       the portable matmul loop
//   train/init.rs:91-352        draws and initialisation
//   train/data.rs:189-212       the synthetic teacher batch
//   train/optimizer.rs:443-568  one prepared step and its application
//   train/runner.rs:365-512     the run loop
//   train/masked.rs:88-128      the host side of the masked-row gather
//
// The IR data structures, the `.mspec` front door and the RNG id helpers are shared with the
// backend's host code (modelspec_b200/csrc/core); all tensor arithmetic is in this file. Rows are
// evaluated in parallel only where every output element keeps its own sequential sum, so the bits
// do not depend on the thread count.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include <atomic>
#include <thread>

#include "../modelspec_b200/csrc/core/frontend.hpp"
#include "../modelspec_b200/csrc/core/rng.hpp"

namespace orc {

using msx::Node;
using msx::Op;
using msx::Program;
using msx::Type;

template <class T> inline T fma_t(T a, T b, T c);
template <> inline float fma_t<float>(float a, float b, float c) { return __builtin_fmaf(a, b, c); }
template <> inline double fma_t<double>(double a, double b, double c) { return __builtin_fma(a, b, c); }

// Runs f(i) for i in [0, n) on up to `g_threads` threads, in blocks of `grain` handed out in
// order. Callers use it only where iterations write disjoint outputs.
static int g_threads = 1;

template <class F> void parallel_for(int64_t n, int64_t grain, F f) {
    int threads = static_cast<int>(std::min<int64_t>(g_threads, (n + grain - 1) / std::max<int64_t>(grain, 1)));
    if (threads <= 1) {
        for (int64_t i = 0; i < n; ++i) f(i);
        return;
    }
    std::atomic<int64_t> next{0};
    auto work = [&] {
        for (;;) {
            int64_t start = next.fetch_add(grain);
            if (start >= n) return;
            int64_t stop = std::min(n, start + grain);
            for (int64_t i = start; i < stop; ++i) f(i);
        }
    };
    std::vector<std::thread> pool;
    for (int t = 1; t < threads; ++t) pool.emplace_back(work);
    work();
    for (std::thread& t : pool) t.join();
}

// `a * b` when first, else fused into acc (interpreter.rs:1292-1296).
template <class T> inline T fused(bool first, T a, T b, T acc) { return first ? a * b : fma_t(a, b, acc); }

template <class T> struct Interp {
    const Program* program = nullptr;
    std::map<std::string, std::vector<float>> inputs;    // f32 inputs by name
    std::map<std::string, std::vector<int32_t>> ids;     // i32 inputs by name
    std::vector<std::vector<float>> params;              // by parameter index
    bool has_seed = false;
    uint64_t seed = 0;
    std::vector<std::vector<T>> values;                  // by node position
    std::vector<char> live;

    void fail(const std::string& what) const { throw msx::Error(what); }

    const std::vector<T>& val(uint32_t id) const { return values[static_cast<size_t>(program->position(id))]; }
    const Node& node_of(uint32_t id) const { return program->node(id); }
    const std::vector<int32_t>& ids_of(uint32_t id) const {
        const Node& n = node_of(id);
        auto it = ids.find(n.name);
        if (n.op != Op::Input || it == ids.end()) fail("no i32 input `" + n.name + "`");
        if (it->second.size() != n.ty.count()) fail("i32 input `" + n.name + "` has the wrong length");
        return it->second;
    }

    // Sequential sum from the first term (interpreter.rs:1905-1911).
    static T sum(const T* x, size_t n, size_t stride = 1) {
        if (n == 0) return T(0);
        T acc = x[0];
        for (size_t i = 1; i < n; ++i) acc = acc + x[i * stride];
        return acc;
    }
    // Whole-tensor sum in f64 (interpreter.rs:1913-1921).
    static double wide_sum(const std::vector<T>& x) {
        if (x.empty()) return 0.0;
        double acc = static_cast<double>(x[0]);
        for (size_t i = 1; i < x.size(); ++i) acc = acc + static_cast<double>(x[i]);
        return acc;
    }
    // Mean and 1/sqrt(var + eps) of one layer_norm row, two passes (interpreter.rs:1513-1527).
    static void row_moments(const T* row, size_t h, T* mean, T* rstd) {
        T width = static_cast<T>(static_cast<double>(h));
        T m = sum(row, h) / width;
        T acc = T(0);
        for (size_t j = 0; j < h; ++j) {
            T d = row[j] - m;
            acc = fused(j == 0, d, d, acc);
        }
        T variance = acc / width;
        *mean = m;
        *rstd = T(1) / std::sqrt(variance + static_cast<T>(1e-12f));
    }
    // GELU constants: f32(high) + f32(low) of the f64 value (interpreter.rs:1538-1551).
    static T constant(double value) {
        float high = static_cast<float>(value);
        float low = static_cast<float>(value - static_cast<double>(high));
        return static_cast<T>(high) + static_cast<T>(low);
    }
    static T gelu_twice_inner(T x) {
        return T(2) * constant(0.7978845608028654) * (x + constant(0.044715) * x * x * x);
    }
    static T logistic(T v) { return T(1) / (T(1) + std::exp(T(0) - v)); }
    static T gelu(T x) { return x * logistic(gelu_twice_inner(x)); }
    static T gelu_grad(T x, T g) {
        T v = gelu_twice_inner(x);
        T s = logistic(v), r = logistic(T(0) - v);
        T slope = constant(0.7978845608028654) * (T(1) + T(3) * constant(0.044715) * x * x);
        return (s + T(2) * (s * x) * r * slope) * g;
    }
    // Row max (first element, replaced only by a greater one) and sum of exp(x - max)
    // (interpreter.rs:1172-1180).
    static void row_softmax(const T* row, size_t v, T* max, T* total) {
        T m = row[0];
        for (size_t c = 1; c < v; ++c)
            if (row[c] > m) m = row[c];
        T acc = std::exp(row[0] - m);
        for (size_t c = 1; c < v; ++c) acc = acc + std::exp(row[c] - m);
        *max = m;
        *total = acc;
    }

    // The operands of one attention op (interpreter.rs:1308-1510), key-mask form.
    struct Attend {
        const T *q, *k, *v, *mask;
        size_t h, d, heads, s, l, b;
        T scale;
        T score(size_t i, size_t j, size_t head) const {
            const T* qi = q + i * h + head * d;
            const T* kj = k + j * h + head * d;
            T acc = qi[0] * kj[0];
            for (size_t c = 1; c < d; ++c) acc = fma_t(qi[c], kj[c], acc);
            return acc * scale;
        }
        bool unmasked(size_t j) const { return mask[j] != T(0); }
        void softmax(size_t i, size_t head, T* max, T* total) const {
            size_t start = i / l * s;
            bool first = true;
            T m = T(0);
            for (size_t j = start; j < start + s; ++j) {
                if (!unmasked(j)) continue;
                T x = score(i, j, head);
                if (first) { m = x; first = false; }
                else if (x > m) m = x;
            }
            first = true;
            T acc = T(0);
            for (size_t j = start; j < start + s; ++j) {
                if (!unmasked(j)) continue;
                T e = std::exp(score(i, j, head) - m);
                acc = first ? e : acc + e;
                first = false;
            }
            *max = m;
            *total = acc;
        }
        T probability(size_t i, size_t j, size_t head, T max, T total) const {
            return std::exp(score(i, j, head) - max) / total;
        }
        T probability_grad(size_t i, size_t j, size_t head, const T* g) const {
            const T* gi = g + i * h + head * d;
            const T* vj = v + j * h + head * d;
            T acc = gi[0] * vj[0];
            for (size_t c = 1; c < d; ++c) acc = fma_t(gi[c], vj[c], acc);
            return acc;
        }
        T row_dot(size_t i, size_t head, T max, T total, const T* g) const {
            size_t start = i / l * s;
            bool first = true;
            T acc = T(0);
            for (size_t j = start; j < start + s; ++j) {
                if (!unmasked(j)) continue;
                acc = fused(first, probability(i, j, head, max, total), probability_grad(i, j, head, g), acc);
                first = false;
            }
            return acc;
        }
        T score_grad(size_t i, size_t j, size_t head, T max, T total, T dd, const T* g) const {
            return probability(i, j, head, max, total) * (probability_grad(i, j, head, g) - dd);
        }
    };

    Attend attend(const Node& n) const {
        const Type& qt = node_of(n.operands[0]).ty;
        const Type& mt = node_of(n.operands[3]).ty;
        Attend a;
        a.q = val(n.operands[0]).data();
        a.k = val(n.operands[1]).data();
        a.v = val(n.operands[2]).data();
        a.mask = val(n.operands[3]).data();
        a.h = qt.shape[1];
        a.heads = n.heads;
        a.d = a.h / a.heads;
        a.b = mt.shape[0];
        a.s = mt.shape[1];
        a.l = qt.shape[0] / a.b;
        a.scale = T(1) / std::sqrt(static_cast<T>(static_cast<double>(a.d)));
        // interpreter.rs:1238-1254: every value 0 or 1, one unmasked key per sequence.
        for (size_t b = 0; b < a.b; ++b) {
            bool any = false;
            for (size_t j = 0; j < a.s; ++j) {
                T m = a.mask[b * a.s + j];
                if (m != T(0) && m != T(1)) fail("key mask value is neither 0 nor 1");
                any = any || m == T(1);
            }
            if (!any) fail("a sequence has no unmasked key");
        }
        return a;
    }

    void masked(std::vector<T>& out, const std::vector<T>& x, uint32_t token_node, float p) {
        if (!has_seed) fail("a program with a dropout runs without a seed");
        const std::vector<int32_t>& token = ids_of(token_node);
        uint64_t id = static_cast<uint64_t>(static_cast<uint32_t>(token[0])) |
                      (static_cast<uint64_t>(static_cast<uint32_t>(token[1])) << 32);
        T scale = static_cast<T>(1.0f / (1.0f - p));
        out.resize(x.size());
        int64_t n = static_cast<int64_t>(x.size());
        parallel_for(n, 64, [&](int64_t i) {
            out[static_cast<size_t>(i)] = msx::dropout_keeps(seed, id, static_cast<uint32_t>(i), p) ? x[static_cast<size_t>(i)] * scale : T(0);
        });
    }

    template <class F> void elementwise(std::vector<T>& out, const Node& n, F f) {
        const std::vector<T>& a = val(n.operands[0]);
        const std::vector<T>& b = val(n.operands[1]);
        const Type& ta = node_of(n.operands[0]).ty;
        const Type& tb = node_of(n.operands[1]).ty;
        if (ta.shape == tb.shape) {
            out.resize(a.size());
            for (size_t i = 0; i < a.size(); ++i) out[i] = f(a[i], b[i]);
        } else if (tb.rank() == 0) {
            out.resize(a.size());
            for (size_t i = 0; i < a.size(); ++i) out[i] = f(a[i], b[0]);
        } else {
            out.resize(b.size());
            for (size_t i = 0; i < b.size(); ++i) out[i] = f(a[0], b[i]);
        }
    }

    void eval(size_t at) {
        const Node& n = program->nodes[at];
        std::vector<T>& out = values[at];
        out.clear();
        size_t count = n.ty.count();
        auto arg = [&](size_t k) -> const std::vector<T>& { return val(n.operands[k]); };
        auto ty = [&](size_t k) -> const Type& { return node_of(n.operands[k]).ty; };
        switch (n.op) {
            case Op::Input: {
                if (n.ty.i32) break;  // read through ids_of by its consumers
                auto it = inputs.find(n.name);
                if (it == inputs.end()) fail("no f32 input `" + n.name + "`");
                if (it->second.size() != count) fail("f32 input `" + n.name + "` has the wrong length");
                out.assign(it->second.begin(), it->second.end());
                break;
            }
            case Op::ParamRead: {
                const std::vector<float>& p = params.at(n.param);
                if (p.size() != count) fail("parameter has the wrong length");
                out.assign(p.begin(), p.end());
                break;
            }
            case Op::Scalar: out.push_back(static_cast<T>(n.scalar)); break;
            case Op::Add: elementwise(out, n, [](T a, T b) { return a + b; }); break;
            case Op::Sub: elementwise(out, n, [](T a, T b) { return a - b; }); break;
            case Op::Mul: elementwise(out, n, [](T a, T b) { return a * b; }); break;
            case Op::Div: elementwise(out, n, [](T a, T b) { return a / b; }); break;
            case Op::Sqrt: {
                const auto& a = arg(0);
                out.resize(a.size());
                for (size_t i = 0; i < a.size(); ++i) out[i] = std::sqrt(a[i]);
                break;
            }
            case Op::MatMul: {
                // cpu/matmul.rs:268-292: loop order i, k, j; the k = 0 products start each sum,
                // every later product is fused into it.
                const T* a = arg(0).data();
                const T* b = arg(1).data();
                int64_t m = static_cast<int64_t>(ty(0).shape[0]);
                size_t k = ty(0).shape[1], nn = ty(1).shape[1];
                out.assign(static_cast<size_t>(m) * nn, T(0));
                if (k == 0) break;
                T* o = out.data();
                parallel_for(m, 64, [&](int64_t i) {
                    T* row = o + static_cast<size_t>(i) * nn;
                    T x = a[static_cast<size_t>(i) * k];
                    for (size_t j = 0; j < nn; ++j) row[j] = x * b[j];
                    for (size_t p = 1; p < k; ++p) {
                        T xp = a[static_cast<size_t>(i) * k + p];
                        const T* brow = b + p * nn;
                        for (size_t j = 0; j < nn; ++j) row[j] = fma_t(xp, brow[j], row[j]);
                    }
                });
                break;
            }
            case Op::Relu: {
                const auto& a = arg(0);
                out.resize(a.size());
                for (size_t i = 0; i < a.size(); ++i) out[i] = a[i] > T(0) ? a[i] : T(0);
                break;
            }
            case Op::ReluGrad: {
                const auto &a = arg(0), &g = arg(1);
                out.resize(a.size());
                for (size_t i = 0; i < a.size(); ++i) out[i] = a[i] > T(0) ? g[i] : T(0);
                break;
            }
            case Op::Transpose: {
                const T* a = arg(0).data();
                size_t m = ty(0).shape[0], nn = ty(0).shape[1];
                out.resize(m * nn);
                for (size_t i = 0; i < m; ++i)
                    for (size_t j = 0; j < nn; ++j) out[j * m + i] = a[i * nn + j];
                break;
            }
            case Op::ReduceSum: out.push_back(static_cast<T>(wide_sum(arg(0)))); break;
            case Op::ReduceMean:
                out.push_back(static_cast<T>(wide_sum(arg(0)) / static_cast<double>(arg(0).size())));
                break;
            case Op::Mse: {
                // interpreter.rs:910-917: differences and products in f64, first product rounded,
                // later ones fused, one division by the count, one rounding.
                const auto &a = arg(0), &b = arg(1);
                double acc = 0.0;
                for (size_t i = 0; i < a.size(); ++i) {
                    double d = static_cast<double>(a[i]) - static_cast<double>(b[i]);
                    acc = i == 0 ? d * d : __builtin_fma(d, d, acc);
                }
                out.push_back(static_cast<T>(acc / static_cast<double>(a.size())));
                break;
            }
            case Op::BroadcastScalar: out.assign(count, arg(0)[0]); break;
            case Op::Embedding: {
                const T* table = arg(0).data();
                size_t rows = ty(0).shape[0], h = ty(0).shape[1];
                const auto& idv = ids_of(n.operands[1]);
                out.resize(idv.size() * h);
                for (size_t r = 0; r < idv.size(); ++r) {
                    if (idv[r] < 0 || static_cast<uint64_t>(idv[r]) >= rows) fail("an embedding id is out of range");
                    std::memcpy(out.data() + r * h, table + static_cast<size_t>(idv[r]) * h, h * sizeof(T));
                }
                break;
            }
            case Op::EmbeddingGrad: {
                const T* g = arg(1).data();
                size_t h = ty(1).shape[1];
                const auto& idv = ids_of(n.operands[0]);
                out.assign(count, T(0));
                for (size_t r = 0; r < idv.size(); ++r) {
                    if (idv[r] < 0 || static_cast<uint64_t>(idv[r]) >= n.rows) fail("an embedding id is out of range");
                    T* row = out.data() + static_cast<size_t>(idv[r]) * h;
                    for (size_t c = 0; c < h; ++c) row[c] = row[c] + g[r * h + c];
                }
                break;
            }
            case Op::AddRows: {
                const auto &x = arg(0), &b = arg(1);
                size_t h = b.size();
                out.resize(x.size());
                for (size_t i = 0; i < x.size(); ++i) out[i] = x[i] + b[i % h];
                break;
            }
            case Op::SumRows: {
                const T* g = arg(0).data();
                size_t rows = ty(0).shape[0];
                int64_t h = static_cast<int64_t>(count);
                out.assign(count, T(0));
                if (rows == 0) break;
                parallel_for(h, 64, [&](int64_t c) {
                    T acc = g[c];
                    for (size_t r = 1; r < rows; ++r) acc = acc + g[r * static_cast<size_t>(h) + static_cast<size_t>(c)];
                    out[static_cast<size_t>(c)] = acc;
                });
                break;
            }
            case Op::Gelu: {
                const auto& a = arg(0);
                out.resize(a.size());
                int64_t m = static_cast<int64_t>(a.size());
                parallel_for(m, 64, [&](int64_t i) {
                    out[static_cast<size_t>(i)] = gelu(a[static_cast<size_t>(i)]);
                });
                break;
            }
            case Op::GeluGrad: {
                const auto &a = arg(0), &g = arg(1);
                out.resize(a.size());
                int64_t m = static_cast<int64_t>(a.size());
                parallel_for(m, 64, [&](int64_t i) {
                    out[static_cast<size_t>(i)] = gelu_grad(a[static_cast<size_t>(i)], g[static_cast<size_t>(i)]);
                });
                break;
            }
            case Op::LayerNorm: {
                const T *x = arg(0).data(), *gamma = arg(1).data(), *beta = arg(2).data();
                size_t h = ty(1).shape[0];
                int64_t rows = static_cast<int64_t>(ty(0).shape[0]);
                out.resize(static_cast<size_t>(rows) * h);
                parallel_for(rows, 64, [&](int64_t r) {
                    const T* row = x + static_cast<size_t>(r) * h;
                    T mean, rstd;
                    row_moments(row, h, &mean, &rstd);
                    for (size_t j = 0; j < h; ++j)
                        out[static_cast<size_t>(r) * h + j] = (row[j] - mean) * rstd * gamma[j] + beta[j];
                });
                break;
            }
            case Op::LayerNormGradX: {
                const T *x = arg(0).data(), *gamma = arg(1).data(), *g = arg(2).data();
                size_t h = ty(1).shape[0];
                int64_t rows = static_cast<int64_t>(ty(0).shape[0]);
                T width = static_cast<T>(static_cast<double>(h));
                out.resize(static_cast<size_t>(rows) * h);
                parallel_for(rows, 64, [&](int64_t r) {
                    const T* row = x + static_cast<size_t>(r) * h;
                    const T* grow = g + static_cast<size_t>(r) * h;
                    T mean, rstd;
                    row_moments(row, h, &mean, &rstd);
                    T s1 = T(0), s2 = T(0);
                    for (size_t j = 0; j < h; ++j) {
                        T gx = grow[j] * gamma[j];
                        T xhat = (row[j] - mean) * rstd;
                        s1 = j == 0 ? gx : s1 + gx;
                        s2 = fused(j == 0, gx, xhat, s2);
                    }
                    T mean_gx = s1 / width, mean_gx_xhat = s2 / width;
                    for (size_t j = 0; j < h; ++j) {
                        T gx = grow[j] * gamma[j];
                        T xhat = (row[j] - mean) * rstd;
                        out[static_cast<size_t>(r) * h + j] = rstd * ((gx - mean_gx) - xhat * mean_gx_xhat);
                    }
                });
                break;
            }
            case Op::LayerNormGradGamma: {
                const T *x = arg(0).data(), *g = arg(1).data();
                size_t h = count, rows = ty(0).shape[0];
                out.assign(count, T(0));
                std::vector<T> means(rows), rstds(rows);
                for (size_t r = 0; r < rows; ++r) row_moments(x + r * h, h, &means[r], &rstds[r]);
                int64_t hh = static_cast<int64_t>(h);
                parallel_for(hh, 64, [&](int64_t c) {
                    T acc = T(0);
                    for (size_t r = 0; r < rows; ++r) {
                        T xhat = (x[r * h + static_cast<size_t>(c)] - means[r]) * rstds[r];
                        acc = fused(r == 0, g[r * h + static_cast<size_t>(c)], xhat, acc);
                    }
                    out[static_cast<size_t>(c)] = acc;
                });
                break;
            }
            case Op::Softmax: {
                const T* x = arg(0).data();
                size_t k = ty(0).shape[1], rows = ty(0).shape[0];
                out.resize(rows * k);
                for (size_t r = 0; r < rows; ++r) {
                    const T* row = x + r * k;
                    T m = row[0];
                    for (size_t c = 1; c < k; ++c)
                        if (row[c] > m) m = row[c];
                    T* o = out.data() + r * k;
                    for (size_t c = 0; c < k; ++c) o[c] = std::exp(row[c] - m);
                    T total = sum(o, k);
                    for (size_t c = 0; c < k; ++c) o[c] = o[c] / total;
                }
                break;
            }
            case Op::SoftmaxGrad: {
                const T *y = arg(0).data(), *g = arg(1).data();
                size_t k = ty(0).shape[1], rows = ty(0).shape[0];
                out.resize(rows * k);
                for (size_t r = 0; r < rows; ++r) {
                    T d = T(0);
                    for (size_t c = 0; c < k; ++c) d = fused(c == 0, g[r * k + c], y[r * k + c], d);
                    for (size_t c = 0; c < k; ++c) out[r * k + c] = y[r * k + c] * (g[r * k + c] - d);
                }
                break;
            }
            case Op::Attention: {
                Attend at = attend(n);
                out.assign(count, T(0));
                int64_t rows = static_cast<int64_t>(at.b * at.l);
                parallel_for(rows, 16, [&](int64_t ii) {
                    size_t i = static_cast<size_t>(ii), start = i / at.l * at.s;
                    for (size_t head = 0; head < at.heads; ++head) {
                        T max, total;
                        at.softmax(i, head, &max, &total);
                        bool first = true;
                        for (size_t j = start; j < start + at.s; ++j) {
                            if (!at.unmasked(j)) continue;
                            T p = at.probability(i, j, head, max, total);
                            for (size_t c = head * at.d; c < (head + 1) * at.d; ++c)
                                out[i * at.h + c] = fused(first, p, at.v[j * at.h + c], out[i * at.h + c]);
                            first = false;
                        }
                    }
                });
                break;
            }
            case Op::AttentionGradQ: {
                Attend at = attend(n);
                const T* g = arg(4).data();
                out.assign(count, T(0));
                int64_t rows = static_cast<int64_t>(at.b * at.l);
                parallel_for(rows, 16, [&](int64_t ii) {
                    size_t i = static_cast<size_t>(ii), start = i / at.l * at.s;
                    for (size_t head = 0; head < at.heads; ++head) {
                        T max, total;
                        at.softmax(i, head, &max, &total);
                        T dd = at.row_dot(i, head, max, total, g);
                        bool first = true;
                        for (size_t j = start; j < start + at.s; ++j) {
                            if (!at.unmasked(j)) continue;
                            T ds = at.score_grad(i, j, head, max, total, dd, g);
                            for (size_t c = head * at.d; c < (head + 1) * at.d; ++c)
                                out[i * at.h + c] = fused(first, ds, at.k[j * at.h + c], out[i * at.h + c]);
                            first = false;
                        }
                        for (size_t c = head * at.d; c < (head + 1) * at.d; ++c)
                            out[i * at.h + c] = out[i * at.h + c] * at.scale;
                    }
                });
                break;
            }
            case Op::AttentionGradK:
            case Op::AttentionGradV: {
                Attend at = attend(n);
                const T* g = arg(4).data();
                bool is_k = n.op == Op::AttentionGradK;
                out.assign(count, T(0));
                int64_t seqs = static_cast<int64_t>(at.b);
                parallel_for(seqs, 1, [&](int64_t bb) {
                    size_t b = static_cast<size_t>(bb), start = b * at.s;
                    for (size_t i = b * at.l; i < (b + 1) * at.l; ++i) {
                        bool first = i % at.l == 0;
                        for (size_t head = 0; head < at.heads; ++head) {
                            T max, total;
                            at.softmax(i, head, &max, &total);
                            T dd = is_k ? at.row_dot(i, head, max, total, g) : T(0);
                            for (size_t j = start; j < start + at.s; ++j) {
                                if (!at.unmasked(j)) continue;
                                T w = is_k ? at.score_grad(i, j, head, max, total, dd, g)
                                           : at.probability(i, j, head, max, total);
                                const T* src = is_k ? at.q : g;
                                for (size_t c = head * at.d; c < (head + 1) * at.d; ++c)
                                    out[j * at.h + c] = fused(first, w, src[i * at.h + c], out[j * at.h + c]);
                            }
                        }
                    }
                    if (is_k)
                        for (size_t j = start; j < start + at.s; ++j)
                            if (at.unmasked(j))
                                for (size_t c = 0; c < at.h; ++c) out[j * at.h + c] = out[j * at.h + c] * at.scale;
                });
                break;
            }
            case Op::CrossEntropy:
            case Op::CrossEntropyGrad: {
                // interpreter.rs:1146-1233.
                const T* logits = arg(0).data();
                const auto& labels = ids_of(n.operands[1]);
                const auto& weights = arg(2);
                size_t v = ty(0).shape[1];
                int64_t rows = static_cast<int64_t>(ty(0).shape[0]);
                for (int64_t r = 0; r < rows; ++r) {
                    if (labels[static_cast<size_t>(r)] < 0 || static_cast<uint64_t>(labels[static_cast<size_t>(r)]) >= v)
                        fail("a label is out of range");
                    T w = weights[static_cast<size_t>(r)];
                    if (!(w * T(0) == T(0)) || w < T(0)) fail("a loss weight is negative or not finite");
                }
                if (n.op == Op::CrossEntropy) {
                    std::vector<double> losses(static_cast<size_t>(rows));
                    parallel_for(rows, 64, [&](int64_t r) {
                        const T* row = logits + static_cast<size_t>(r) * v;
                        T max, total;
                        row_softmax(row, v, &max, &total);
                        losses[static_cast<size_t>(r)] =
                            static_cast<double>(max + std::log(total) - row[labels[static_cast<size_t>(r)]]);
                    });
                    double numerator = 0.0;
                    for (int64_t r = 0; r < rows; ++r) {
                        double w = static_cast<double>(weights[static_cast<size_t>(r)]);
                        numerator = r == 0 ? w * losses[0] : __builtin_fma(w, losses[static_cast<size_t>(r)], numerator);
                    }
                    double denominator = wide_sum(weights);
                    out.push_back(denominator == 0.0 ? T(0) : static_cast<T>(numerator / denominator));
                } else {
                    T gg = arg(3)[0];
                    T denominator = static_cast<T>(wide_sum(weights));
                    out.assign(count, T(0));
                    if (denominator == T(0)) break;
                    parallel_for(rows, 64, [&](int64_t r) {
                        const T* row = logits + static_cast<size_t>(r) * v;
                        T max, total;
                        row_softmax(row, v, &max, &total);
                        T scale = gg * weights[static_cast<size_t>(r)] / denominator;
                        size_t label = static_cast<size_t>(labels[static_cast<size_t>(r)]);
                        for (size_t c = 0; c < v; ++c) {
                            T target = c == label ? T(1) : T(0);
                            out[static_cast<size_t>(r) * v + c] = scale * (std::exp(row[c] - max) / total - target);
                        }
                    });
                }
                break;
            }
            case Op::Dropout: masked(out, arg(0), n.operands[1], n.p); break;
            case Op::DropoutGrad: masked(out, arg(1), n.operands[0], n.p); break;
            case Op::StopGradient: out = arg(0); break;
            default: fail(std::string("the oracle has no ") + msx::op_name(n.op));
        }
    }

    // Evaluates every node an output depends on, in definition order. Values stay until the next
    // run so a test can read any of them.
    void run(const Program& p) {
        program = &p;
        values.assign(p.nodes.size(), {});
        live.assign(p.nodes.size(), 0);
        for (const msx::Output& o : p.outputs) live[static_cast<size_t>(p.position(o.value))] = 1;
        for (size_t i = p.nodes.size(); i-- > 0;)
            if (live[i])
                for (uint32_t o : p.nodes[i].operands) live[static_cast<size_t>(p.position(o))] = 1;
        // Free each value after its last reader to bound memory (the reference plans the same
        // reuse, interpreter.rs:341-494); outputs are kept.
        std::vector<size_t> last(p.nodes.size(), 0);
        for (size_t i = 0; i < p.nodes.size(); ++i)
            if (live[i])
                for (uint32_t o : p.nodes[i].operands) last[static_cast<size_t>(p.position(o))] = i;
        std::vector<char> is_output(p.nodes.size(), 0);
        for (const msx::Output& o : p.outputs) is_output[static_cast<size_t>(p.position(o.value))] = 1;
        std::vector<std::vector<size_t>> frees(p.nodes.size());
        for (size_t i = 0; i < p.nodes.size(); ++i)
            if (live[i] && !is_output[i] && keep_all == false) frees[last[i]].push_back(i);
        for (size_t i = 0; i < p.nodes.size(); ++i) {
            if (!live[i]) continue;
            eval(i);
            for (size_t f : frees[i]) std::vector<T>().swap(values[f]);
        }
    }
    bool keep_all = false;
};

// ---------------------------------------------------------------------------------------------
// Initialisation and data (train/init.rs).

inline std::vector<float> initial_value(const msx::Param& p, uint64_t seed, uint32_t stream) {
    size_t n = p.ty.count();
    std::vector<float> out(n);
    if (p.init == msx::Init::Zeros) { std::fill(out.begin(), out.end(), 0.0f); return out; }
    if (p.init == msx::Init::Ones) { std::fill(out.begin(), out.end(), 1.0f); return out; }
    // xavier_uniform (init.rs:207-225): a (2u - 1), a = sqrt(6 / (in + out)), in f64.
    double a = std::sqrt(6.0 / (static_cast<double>(p.ty.shape[0]) + static_cast<double>(p.ty.shape[1])));
    uint64_t id = msx::canonical_id(p.path);
    for (size_t i = 0; i < n; ++i) {
        uint32_t block[4];
        msx::philox_block(seed, stream, id, static_cast<uint32_t>(i), block);
        out[i] = static_cast<float>(a * (2.0 * msx::uniform01(block[0]) - 1.0));
    }
    return out;
}

// Box-Muller standard normal of each element (init.rs:228-242).
inline std::vector<float> standard_normal(uint64_t seed, uint32_t stream, const std::string& name, size_t n) {
    std::vector<float> out(n);
    uint64_t id = msx::canonical_id(name);
    const double tau = 6.283185307179586;
    for (size_t i = 0; i < n; ++i) {
        uint32_t block[4];
        msx::philox_block(seed, stream, id, static_cast<uint32_t>(i), block);
        out[i] = static_cast<float>(std::sqrt(-2.0 * std::log(msx::uniform01(block[0]))) *
                                    std::cos(tau * msx::uniform01(block[1])));
    }
    return out;
}

// One training run's state: the reference's PreparedStep + ParamState (train/optimizer.rs).
struct Trainer {
    msx::Compiled compiled;
    Interp<float> step, forward;
    std::vector<std::vector<float>> params, m, v;
    std::vector<std::vector<float>> gradients;  // of the last step, by parameter index (empty: none)
    std::map<std::string, std::vector<float>> inputs;
    std::map<std::string, std::vector<int32_t>> ids;
    std::vector<std::string> sites;

    Trainer(const std::string& source, uint64_t masked_rows) : compiled(msx::compile_training(source, masked_rows)) {
        const Program& fwd = compiled.forward;
        for (const msx::Param& p : fwd.params) {
            params.push_back(initial_value(p, compiled.config.seed, msx::kStreamInit));
            m.emplace_back(p.ty.count(), 0.0f);
            v.emplace_back(p.ty.count(), 0.0f);
        }
        gradients.resize(params.size());
        for (const Node& n : compiled.step.nodes)
            if (n.op == Op::Input && n.ty.i32 && n.ty.shape == std::vector<uint64_t>{2} &&
                n.name.find(".dropout#") != std::string::npos)
                sites.push_back(n.name);
    }

    // The reference's synthetic batch (train/data.rs:189-212): the one drawn input standard
    // normal, key masks all ones, the target the prediction of a teacher initialised on the
    // teacher stream.
    void synthetic() {
        const Program& fwd = compiled.forward;
        std::set<std::string> masks;
        for (uint32_t in : fwd.inputs) {
            const Node& n = fwd.node(in);
            if (n.ty.i32) continue;
            bool any = false, only = true;
            for (const Node& user : fwd.nodes)
                for (size_t k = 0; k < user.operands.size(); ++k)
                    if (user.operands[k] == in) {
                        any = true;
                        only = only && user.op == Op::Attention && k == 3;
                    }
            if (any && only) masks.insert(n.name);
        }
        const msx::DataDecl *input = nullptr, *target = nullptr;
        for (const msx::DataDecl& d : compiled.config.data) {
            if (masks.count(d.name)) continue;
            if (d.target) { if (target) throw msx::Error("synthetic data takes one target"); target = &d; }
            else { if (input) throw msx::Error("synthetic data takes one input"); input = &d; }
        }
        if (!input || !target || input->ty.i32 || target->ty.i32)
            throw msx::Error("synthetic data takes one f32 input and one f32 target");
        uint64_t seed = compiled.config.seed;
        inputs[input->name] = standard_normal(seed, msx::kStreamData, input->name, input->ty.count());
        inputs[target->name] = std::vector<float>(target->ty.count(), 0.0f);
        for (const msx::DataDecl& d : compiled.config.data)
            if (masks.count(d.name)) inputs[d.name] = std::vector<float>(d.ty.count(), 1.0f);
        Interp<float> teacher;
        for (const msx::Param& p : fwd.params) teacher.params.push_back(initial_value(p, seed, msx::kStreamTeacher));
        teacher.inputs = inputs;
        teacher.ids = ids;
        Program predict = fwd;
        predict.outputs = {msx::Output{compiled.prediction, msx::Role::Plain, 0, 0}};
        teacher.run(predict);
        inputs[target->name] = teacher.val(compiled.prediction);
    }

    // The host side of the masked-row gather (train/masked.rs:88-128).
    void gather_masked() {
        if (!compiled.masked_rows) return;
        size_t capacity = compiled.masked_rows;
        const std::vector<float>& weights = inputs.at(compiled.masked_weights);
        const std::vector<int32_t>& labels = ids.at(compiled.masked_labels);
        std::vector<int32_t> rows, lab;
        std::vector<float> w;
        for (size_t r = 0; r < weights.size(); ++r)
            if (weights[r] != 0.0f) {
                rows.push_back(static_cast<int32_t>(r));
                lab.push_back(r < labels.size() ? labels[r] : 0);
                w.push_back(weights[r]);
            }
        if (rows.size() > capacity) throw msx::Error("E-DATA-012: more selected rows than the masked-row gather holds");
        rows.resize(capacity, 0);
        lab.resize(capacity, 0);
        w.resize(capacity, 0.0f);
        ids["masked.rows"] = rows;
        ids["masked.labels." + compiled.masked_labels] = lab;
        inputs["masked.weights." + compiled.masked_weights] = w;
    }

    // Step `k` of a run that ends at `end` (runner.rs:417-463): scalars of t = k + 1, tokens of
    // step k, one evaluation, then every update and next moment applied.
    float train_step(uint64_t k, uint64_t end) {
        const Program& p = compiled.step;
        if (p.optimizer.rule == msx::Rule::AdamW) {
            msx::StepScalars s = msx::adamw_scalars(compiled.config.adamw, compiled.config.lr, k + 1, end);
            inputs["optimizer.lr_t"] = {s.lr_t};
            inputs["optimizer.c1"] = {s.c1};
            inputs["optimizer.c2"] = {s.c2};
            for (size_t i = 0; i < params.size(); ++i) {
                inputs["optimizer.m@" + p.params[i].path] = m[i];
                inputs["optimizer.v@" + p.params[i].path] = v[i];
            }
        }
        gather_masked();
        for (const std::string& site : sites) {
            int32_t token[2];
            msx::dropout_token(site, k, token);
            ids[site] = {token[0], token[1]};
        }
        step.inputs = inputs;
        step.ids = ids;
        step.params = params;
        step.has_seed = true;
        step.seed = compiled.config.seed;
        step.run(p);
        float loss = 0.0f;
        for (const msx::Output& o : p.outputs) {
            const std::vector<float>& value = step.val(o.value);
            switch (o.role) {
                case msx::Role::Loss: loss = value[0]; break;
                case msx::Role::Gradient: gradients[o.param] = value; break;
                case msx::Role::Update: params[o.param] = value; break;
                case msx::Role::Moment: (o.moment == 'm' ? m : v)[o.param] = value; break;
                default: break;
            }
        }
        return loss;
    }

    // The dropout-free forward loss on the current parameters (runner.rs:466-485).
    float final_loss() {
        forward.inputs = inputs;
        forward.ids = ids;
        forward.params = params;
        forward.run(compiled.forward);
        return forward.val(compiled.forward.outputs[0].value)[0];
    }

    // The model's prediction for the current batch on the current parameters, from the forward
    // program (dropout the identity), as held-out evaluation reads it (train/eval.rs:279-296).
    std::vector<float> predict() {
        forward.inputs = inputs;
        forward.ids = ids;
        forward.params = params;
        Program program = compiled.forward;
        program.outputs = {msx::Output{compiled.prediction, msx::Role::Plain, 0, 0}};
        forward.run(program);
        return forward.val(compiled.prediction);
    }
};

// The held-out reduction (crates/modelspec-runtime/src/train/eval.rs:409-499): the running sums
// over every row of every batch, in batch order and then row order.
struct Tally {
    bool has_numerator = false, has_denominator = false;
    double numerator = 0.0, denominator = 0.0;
    uint64_t correct = 0, selected = 0, softmaxes = 0;

    // eval.rs:490-499: the maximum the first element replaced by each later greater one, the sum
    // in ascending order from its first term.
    static float row_nll(const float* row, size_t v, size_t label) {
        float max = row[0];
        for (size_t c = 1; c < v; ++c)
            if (row[c] > max) max = row[c];
        float total = std::exp(row[0] - max);
        for (size_t c = 1; c < v; ++c) total = total + std::exp(row[c] - max);
        return max + std::log(total) - row[label];
    }
    // eval.rs:481-484.
    static bool nll_is_finite(const float* row, size_t v) {
        bool small = true;
        for (size_t c = 0; c < v; ++c) small = small & (std::fabs(row[c]) < 5.0e37f);
        return small;
    }
    // train/runner.rs:631-638: the first maximum, or none when the row holds a NaN.
    static long argmax(const float* row, size_t v) {
        for (size_t c = 0; c < v; ++c)
            if (std::isnan(row[c])) return -1;
        size_t best = 0;
        for (size_t c = 1; c < v; ++c)
            if (row[c] > row[best]) best = c;
        return static_cast<long>(best);
    }
    // eval.rs:421-457. `skipping` false is the tally "as it was before it skipped rows"
    // (eval.rs:514-547), which the reference's tests hold the skipping one to.
    void add(const float* logits, const int32_t* labels, const float* weights, size_t rows, size_t v, bool skipping) {
        for (size_t n = 0; n < rows; ++n) {
            const float* row = logits + n * v;
            if (labels[n] < 0 || static_cast<size_t>(labels[n]) >= v)
                throw msx::Error("held-out row " + std::to_string(n) + ": label " + std::to_string(labels[n]) + " is not below the " +
                                 std::to_string(v) + " classes");
            const size_t target = static_cast<size_t>(labels[n]);
            const float weight = weights[n];
            uint32_t bits;
            std::memcpy(&bits, &weight, 4);
            if (skipping && bits == 0 && nll_is_finite(row, v)) {
                numerator = has_numerator ? numerator + 0.0 : 0.0;
                denominator = has_denominator ? denominator + 0.0 : 0.0;
                has_numerator = has_denominator = true;
                continue;
            }
            ++softmaxes;
            const double wide = static_cast<double>(weight), nll = static_cast<double>(row_nll(row, v, target));
            numerator = has_numerator ? std::fma(wide, nll, numerator) : wide * nll;
            denominator = has_denominator ? denominator + wide : wide;
            has_numerator = has_denominator = true;
            if (weight > 0.0f) {
                ++selected;
                if (argmax(row, v) == static_cast<long>(target)) ++correct;
            }
        }
    }
    // eval.rs:459-475.
    void metrics(float* loss, float* accuracy) const {
        *loss = denominator == 0.0 ? 0.0f : static_cast<float>(numerator / denominator);
        *accuracy = selected == 0 ? 0.0f : static_cast<float>(correct) / static_cast<float>(selected);
    }
};

// A bare program evaluated once, for op-level checks; f32 or f64 arithmetic.
struct Session {
    Program program;
    bool wide = false;
    Interp<float> f;
    Interp<double> d;
};

}  // namespace orc

// ---------------------------------------------------------------------------------------------
// C ABI for the tests (ctypes).

static thread_local std::string g_error;

template <class F> static int guarded(F f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}

extern "C" {

const char* orc_last_error() { return g_error.c_str(); }

void orc_set_threads(int n) { orc::g_threads = n > 0 ? n : 1; }

void orc_philox(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]) { msx::philox4x32_10(counter, key, out); }
void orc_blake3(const uint8_t* bytes, uint64_t len, uint8_t out[32]) { msx::blake3_hash(bytes, len, out); }
uint64_t orc_canonical_id(const char* path) { return msx::canonical_id(path); }
uint64_t orc_dropout_id(const char* site, uint64_t step) { return msx::dropout_id(site, step); }
int orc_dropout_keeps(uint64_t seed, uint64_t id, uint32_t index, float p) { return msx::dropout_keeps(seed, id, index, p) ? 1 : 0; }

void* orc_trainer_create(const char* source, uint64_t masked_rows) {
    orc::Trainer* t = nullptr;
    if (guarded([&] { t = new orc::Trainer(source, masked_rows); })) return nullptr;
    return t;
}
void orc_trainer_destroy(void* h) { delete static_cast<orc::Trainer*>(h); }

// Copies the text of the step ("step"), the forward program ("forward") or the lowered program
// with dropout ("tensor") into `out` (capacity `cap`); returns the length needed.
uint64_t orc_trainer_ir(void* h, const char* which, char* out, uint64_t cap) {
    orc::Trainer* t = static_cast<orc::Trainer*>(h);
    std::string w = which;
    std::string text = msx::print_program(w == "step" ? t->compiled.step : w == "forward" ? t->compiled.forward
                                                                                           : t->compiled.forward_with_dropout);
    if (out && cap) {
        size_t n = std::min<size_t>(cap - 1, text.size());
        std::memcpy(out, text.data(), n);
        out[n] = 0;
    }
    return text.size() + 1;
}
uint64_t orc_trainer_steps(void* h) { return static_cast<orc::Trainer*>(h)->compiled.config.steps; }
uint64_t orc_trainer_seed(void* h) { return static_cast<orc::Trainer*>(h)->compiled.config.seed; }
int orc_trainer_synthetic(void* h) { return guarded([&] { static_cast<orc::Trainer*>(h)->synthetic(); }); }
int orc_trainer_set_f32(void* h, const char* name, const float* data, uint64_t n) {
    return guarded([&] { static_cast<orc::Trainer*>(h)->inputs[name].assign(data, data + n); });
}
int orc_trainer_set_i32(void* h, const char* name, const int32_t* data, uint64_t n) {
    return guarded([&] { static_cast<orc::Trainer*>(h)->ids[name].assign(data, data + n); });
}
int orc_trainer_get_f32(void* h, const char* name, float* out, uint64_t n) {
    return guarded([&] {
        const std::vector<float>& v = static_cast<orc::Trainer*>(h)->inputs.at(name);
        if (v.size() != n) throw msx::Error("input length mismatch");
        std::memcpy(out, v.data(), n * sizeof(float));
    });
}
int orc_trainer_step(void* h, uint64_t k, uint64_t end, float* loss) {
    return guarded([&] { *loss = static_cast<orc::Trainer*>(h)->train_step(k, end); });
}
int orc_trainer_final_loss(void* h, float* loss) {
    return guarded([&] { *loss = static_cast<orc::Trainer*>(h)->final_loss(); });
}
uint64_t orc_trainer_param_count(void* h) { return static_cast<orc::Trainer*>(h)->params.size(); }
const char* orc_trainer_param_path(void* h, uint64_t i) { return static_cast<orc::Trainer*>(h)->compiled.forward.params.at(i).path.c_str(); }
uint64_t orc_trainer_param_len(void* h, uint64_t i) { return static_cast<orc::Trainer*>(h)->params.at(i).size(); }
// which: 0 parameter, 1 first moment, 2 second moment, 3 gradient of the last step.
int orc_trainer_read(void* h, int which, uint64_t i, float* out, uint64_t n) {
    return guarded([&] {
        orc::Trainer* t = static_cast<orc::Trainer*>(h);
        const std::vector<float>& v = (which == 0 ? t->params : which == 1 ? t->m : which == 2 ? t->v : t->gradients).at(i);
        if (v.size() != n) throw msx::Error("length mismatch");
        std::memcpy(out, v.data(), n * sizeof(float));
    });
}
int orc_trainer_predict(void* h, float* out, uint64_t n) {
    return guarded([&] {
        std::vector<float> v = static_cast<orc::Trainer*>(h)->predict();
        if (v.size() != n) throw msx::Error("length mismatch");
        std::memcpy(out, v.data(), n * sizeof(float));
    });
}
// The held-out tally: create, add batches of logits [rows, classes] in order, read the metrics.
void* orc_tally_create() { return new orc::Tally(); }
void orc_tally_destroy(void* h) { delete static_cast<orc::Tally*>(h); }
int orc_tally_add(void* h, const float* logits, const int32_t* labels, const float* weights, uint64_t rows, uint64_t classes, int skipping) {
    return guarded([&] { static_cast<orc::Tally*>(h)->add(logits, labels, weights, rows, classes, skipping != 0); });
}
// sums: numerator, denominator; counts: correct, selected, softmaxes.
void orc_tally_read(void* h, float* loss, float* accuracy, double sums[2], uint64_t counts[3]) {
    const orc::Tally* t = static_cast<orc::Tally*>(h);
    t->metrics(loss, accuracy);
    sums[0] = t->numerator;
    sums[1] = t->denominator;
    counts[0] = t->correct;
    counts[1] = t->selected;
    counts[2] = t->softmaxes;
}
int orc_trainer_write_param(void* h, uint64_t i, const float* data, uint64_t n) {
    return guarded([&] {
        orc::Trainer* t = static_cast<orc::Trainer*>(h);
        if (t->params.at(i).size() != n) throw msx::Error("length mismatch");
        t->params[i].assign(data, data + n);
    });
}

void* orc_session_create(const char* ir_text, int wide) {
    orc::Session* s = nullptr;
    if (guarded([&] {
            s = new orc::Session;
            s->program = msx::parse_program(ir_text);
            s->wide = wide != 0;
            s->f.params.resize(s->program.params.size());
            s->d.params.resize(s->program.params.size());
            s->f.keep_all = s->d.keep_all = true;
        }))
        return nullptr;
    return s;
}
void orc_session_destroy(void* h) { delete static_cast<orc::Session*>(h); }
int orc_session_set_f32(void* h, const char* name, const float* data, uint64_t n) {
    return guarded([&] {
        orc::Session* s = static_cast<orc::Session*>(h);
        s->f.inputs[name].assign(data, data + n);
        s->d.inputs[name].assign(data, data + n);
    });
}
int orc_session_set_i32(void* h, const char* name, const int32_t* data, uint64_t n) {
    return guarded([&] {
        orc::Session* s = static_cast<orc::Session*>(h);
        s->f.ids[name].assign(data, data + n);
        s->d.ids[name].assign(data, data + n);
    });
}
int orc_session_set_param(void* h, uint64_t i, const float* data, uint64_t n) {
    return guarded([&] {
        orc::Session* s = static_cast<orc::Session*>(h);
        s->f.params.at(i).assign(data, data + n);
        s->d.params.at(i).assign(data, data + n);
    });
}
void orc_session_set_seed(void* h, uint64_t seed) {
    orc::Session* s = static_cast<orc::Session*>(h);
    s->f.has_seed = s->d.has_seed = true;
    s->f.seed = s->d.seed = seed;
}
int orc_session_run(void* h) {
    return guarded([&] {
        orc::Session* s = static_cast<orc::Session*>(h);
        if (s->wide) s->d.run(s->program);
        else s->f.run(s->program);
    });
}
// The value %id after a run, as f64 (exact for an f32 run).
int orc_session_value(void* h, uint32_t id, double* out, uint64_t n) {
    return guarded([&] {
        orc::Session* s = static_cast<orc::Session*>(h);
        if (s->wide) {
            const std::vector<double>& v = s->d.val(id);
            if (v.size() != n) throw msx::Error("length mismatch");
            std::memcpy(out, v.data(), n * sizeof(double));
        } else {
            const std::vector<float>& v = s->f.val(id);
            if (v.size() != n) throw msx::Error("length mismatch");
            for (size_t i = 0; i < n; ++i) out[i] = static_cast<double>(v[i]);
        }
    });
}

}  // extern "C"
