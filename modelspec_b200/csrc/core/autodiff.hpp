// Reverse-mode differentiation of a forward Tensor IR program and the attachment of the SGD and
// AdamW update subgraphs: what turns a lowered `train` block into the training step a backend
// runs.
//
// `differentiate` follows crates/modelspec-core/src/autodiff.rs:59-105 (driver), :115-158 (the
// reverse walk), :462-532 (the sink: ids, subgraph tags, adjoint sums in contribution order) with
// the gradient rules of crates/modelspec-core/src/ops.rs:752-975. `attach_sgd` and `attach_adamw`
// follow crates/modelspec-core/src/ir/training.rs:737-797 and :822-980; the AdamW constants and
// per-step scalars are training.rs:190-227.
#pragma once

#include <algorithm>
#include <set>

#include "ops.hpp"

namespace msx {

namespace detail {

struct Sink {
    Builder b;
    bool has_seed = false;
    uint32_t seed = 0;
    Tag tag = Tag::Gradient;

    explicit Sink(Program p) : b(std::move(p)) {}

    const Type& type_of(uint32_t v) const { return b.type_of(v); }

    uint32_t emit(Node n) {
        bool on_seed = false;
        for (uint32_t o : n.operands)
            if ((has_seed && o == seed) || b.program.node(o).tag == Tag::Gradient) on_seed = true;
        n.tag = (on_seed || tag == Tag::Loss) ? tag : Tag::Forward;
        return b.push(std::move(n));
    }
    uint32_t emit(Op op, std::vector<uint32_t> operands) {
        Node n;
        n.op = op;
        n.operands = std::move(operands);
        return emit(std::move(n));
    }
    uint32_t scalar(float v) {
        Node n;
        n.op = Op::Scalar;
        n.scalar = v;
        return emit(std::move(n));
    }
    // The sum of `values` in order, each added once; the value itself when there is one.
    uint32_t sum(const std::vector<uint32_t>& values) {
        uint32_t acc = values.at(0);
        for (size_t i = 1; i < values.size(); ++i) acc = emit(Op::Add, {acc, values[i]});
        return acc;
    }
};

inline uint32_t unbroadcast(Sink& s, uint32_t c, uint32_t operand) {
    if (s.type_of(operand).rank() == 0 && s.type_of(c).rank() > 0) return s.emit(Op::ReduceSum, {c});
    return c;
}

inline uint32_t broadcast(Sink& s, uint32_t v, uint32_t operand) {
    std::vector<uint64_t> shape = s.type_of(operand).shape;
    if (shape.empty()) return v;
    Node n;
    n.op = Op::BroadcastScalar;
    n.bshape = shape;
    n.operands = {v};
    return s.emit(std::move(n));
}

inline uint32_t negate(Sink& s, uint32_t c) {
    uint32_t minus_one = s.scalar(-1.0f);
    return s.emit(Op::Mul, {c, minus_one});
}

inline float per_element(const Type& ty, double factor) {
    return static_cast<float>(factor / static_cast<double>(ty.count()));
}

constexpr uint32_t kNone = 0xffffffffu;

// The gradient rule of `node` (ops.rs:752-930): the contribution to each wanted operand's
// adjoint, kNone for the others. Returns false for an op with no rule.
inline bool gradient(Sink& s, const Node& node, uint32_t g, const std::vector<bool>& wanted,
                     std::vector<uint32_t>* out) {
    const std::vector<uint32_t>& in = node.operands;
    out->assign(in.size(), kNone);
    auto want = [&](size_t i) { return i < wanted.size() && wanted[i]; };
    switch (node.op) {
        case Op::Input:
        case Op::ParamRead:
        case Op::Scalar:
        case Op::StopGradient: return true;
        case Op::Add:
            for (size_t i = 0; i < in.size(); ++i)
                if (want(i)) (*out)[i] = unbroadcast(s, g, in[i]);
            return true;
        case Op::Sub:
            if (want(0)) (*out)[0] = unbroadcast(s, g, in[0]);
            if (want(1)) (*out)[1] = negate(s, unbroadcast(s, g, in[1]));
            return true;
        case Op::Mul:
            if (want(0)) (*out)[0] = unbroadcast(s, s.emit(Op::Mul, {g, in[1]}), in[0]);
            if (want(1)) (*out)[1] = unbroadcast(s, s.emit(Op::Mul, {g, in[0]}), in[1]);
            return true;
        case Op::MatMul:
            if (want(0)) {
                uint32_t bt = s.emit(Op::Transpose, {in[1]});
                (*out)[0] = s.emit(Op::MatMul, {g, bt});
            }
            if (want(1)) {
                uint32_t at = s.emit(Op::Transpose, {in[0]});
                (*out)[1] = s.emit(Op::MatMul, {at, g});
            }
            return true;
        case Op::Relu:
            if (want(0)) (*out)[0] = s.emit(Op::ReluGrad, {in[0], g});
            return true;
        case Op::Transpose:
            if (want(0)) (*out)[0] = s.emit(Op::Transpose, {g});
            return true;
        case Op::ReduceSum:
            if (want(0)) (*out)[0] = broadcast(s, g, in[0]);
            return true;
        case Op::ReduceMean:
            if (want(0)) {
                uint32_t c = s.scalar(per_element(s.type_of(in[0]), 1.0));
                uint32_t scaled = s.emit(Op::Mul, {g, c});
                (*out)[0] = broadcast(s, scaled, in[0]);
            }
            return true;
        case Op::Mse:
            if (want(0) || want(1)) {
                float scale = per_element(s.type_of(in[0]), 2.0);
                uint32_t d = s.emit(Op::Sub, {in[0], in[1]});
                uint32_t c = s.scalar(scale);
                uint32_t scaled = s.emit(Op::Mul, {g, c});
                uint32_t dy = s.emit(Op::Mul, {d, scaled});
                if (want(0)) (*out)[0] = dy;
                if (want(1)) (*out)[1] = negate(s, dy);
            }
            return true;
        case Op::Embedding:
            if (want(0)) {
                Node n;
                n.op = Op::EmbeddingGrad;
                n.rows = s.type_of(in[0]).shape[0];
                n.operands = {in[1], g};
                (*out)[0] = s.emit(std::move(n));
            }
            return true;
        case Op::AddRows:
            if (want(0)) (*out)[0] = g;
            if (want(1)) (*out)[1] = s.emit(Op::SumRows, {g});
            return true;
        case Op::Gelu:
            if (want(0)) (*out)[0] = s.emit(Op::GeluGrad, {in[0], g});
            return true;
        case Op::LayerNorm:
            if (want(0)) (*out)[0] = s.emit(Op::LayerNormGradX, {in[0], in[1], g});
            if (want(1)) (*out)[1] = s.emit(Op::LayerNormGradGamma, {in[0], g});
            if (want(2)) (*out)[2] = s.emit(Op::SumRows, {g});
            return true;
        case Op::Softmax:
            if (want(0)) (*out)[0] = s.emit(Op::SoftmaxGrad, {node.id, g});
            return true;
        case Op::Attention: {
            Op rules[3] = {Op::AttentionGradQ, Op::AttentionGradK, Op::AttentionGradV};
            for (size_t i = 0; i < 3; ++i) {
                if (!want(i)) continue;
                Node n;
                n.op = rules[i];
                n.heads = node.heads;
                n.operands = {in[0], in[1], in[2], in[3], g};
                (*out)[i] = s.emit(std::move(n));
            }
            return true;
        }
        case Op::CrossEntropy:
            if (want(0)) (*out)[0] = s.emit(Op::CrossEntropyGrad, {in[0], in[1], in[2], g});
            return true;
        case Op::Dropout:
            if (want(0)) {
                Node n;
                n.op = Op::DropoutGrad;
                n.p = node.p;
                n.operands = {in[1], g};
                (*out)[0] = s.emit(std::move(n));
            }
            return true;
        default: return false;
    }
}

}  // namespace detail

// Differentiates `forward` with respect to its parameters from its one rank-0 output, the loss.
// The result keeps the forward nodes (tagged forward, the loss tagged loss), then the seed and
// the backward nodes; its outputs are the loss and each reachable parameter's gradient in
// parameter order.
inline Program differentiate(const Program& forward) {
    if (forward.outputs.size() != 1) throw Error("the forward program has not one output");
    uint32_t loss = forward.outputs[0].value;
    int loss_at = forward.position(loss);
    if (loss_at < 0) throw Error("the loss is not defined");
    if (forward.nodes[static_cast<size_t>(loss_at)].ty.rank() != 0)
        throw Error("the loss is not rank 0");
    Program start = forward;
    start.tagged = true;
    for (Node& n : start.nodes) n.tag = n.id == loss ? Tag::Loss : Tag::Forward;
    const std::vector<Node>& nodes = forward.nodes;
    std::map<uint32_t, size_t> position;
    for (size_t i = 0; i < nodes.size(); ++i) position[nodes[i].id] = i;
    // Which nodes depend on a parameter read (autodiff.rs:160-175).
    std::vector<bool> reaches(nodes.size(), false);
    for (size_t i = 0; i < nodes.size(); ++i) {
        bool any = nodes[i].op == Op::ParamRead;
        for (uint32_t o : nodes[i].operands) any = any || reaches[position.at(o)];
        reaches[i] = nodes[i].op != Op::StopGradient && any;
    }
    detail::Sink sink(std::move(start));
    std::map<uint32_t, std::vector<uint32_t>> adjoints;
    std::vector<std::pair<uint32_t, uint32_t>> leaves;
    if (reaches[static_cast<size_t>(loss_at)]) {
        sink.tag = Tag::Loss;
        uint32_t seed = sink.scalar(1.0f);
        sink.tag = Tag::Gradient;
        sink.has_seed = true;
        sink.seed = seed;
        adjoints[loss] = {seed};
    }
    for (size_t i = static_cast<size_t>(loss_at) + 1; i-- > 0;) {
        const Node node = nodes[i];  // a copy: the sink's node vector grows
        auto found = adjoints.find(node.id);
        if (found == adjoints.end()) continue;
        std::vector<uint32_t> contributions = std::move(found->second);
        adjoints.erase(found);
        uint32_t g = sink.sum(contributions);
        if (node.op == Op::ParamRead || node.op == Op::Input) {
            leaves.emplace_back(node.id, g);
            continue;
        }
        std::vector<bool> wanted;
        for (uint32_t o : node.operands) wanted.push_back(reaches[position.at(o)]);
        std::vector<uint32_t> per_operand;
        if (!detail::gradient(sink, node, g, wanted, &per_operand))
            throw Error(std::string(op_name(node.op)) + " has no gradient rule");
        for (size_t k = 0; k < node.operands.size(); ++k)
            if (per_operand[k] != detail::kNone) adjoints[node.operands[k]].push_back(per_operand[k]);
    }
    std::map<uint32_t, std::vector<uint32_t>> reads;  // param -> adjoints of its reads
    for (auto& [leaf, g] : leaves) {
        const Node& n = nodes[position.at(leaf)];
        if (n.op == Op::ParamRead) reads[n.param].push_back(g);
    }
    Program& out = sink.b.program;
    out.outputs.clear();
    out.outputs.push_back(Output{loss, Role::Loss, 0, 0});
    for (auto& [param, gs] : reads) {
        uint32_t g = sink.sum(gs);
        out.outputs.push_back(Output{g, Role::Gradient, param, 0});
    }
    return std::move(sink.b.program);
}

// Each use of a `StopGradient` reads its operand instead and the node goes
// (crates/modelspec-core/src/passes/stop_gradient.rs:38,61).
inline Program without_stop_gradient(Program program) {
    std::map<uint32_t, uint32_t> identity;
    std::vector<Node> kept;
    for (Node& n : program.nodes) {
        for (uint32_t& o : n.operands) {
            auto it = identity.find(o);
            if (it != identity.end()) o = it->second;
        }
        if (n.op == Op::StopGradient) identity[n.id] = n.operands.at(0);
        else kept.push_back(std::move(n));
    }
    program.nodes = std::move(kept);
    for (Output& o : program.outputs) {
        auto it = identity.find(o.value);
        if (it != identity.end()) o.value = it->second;
    }
    return program;
}

// ---------------------------------------------------------------------------------------------
// Optimizer attachment.

struct AdamW {
    float weight_decay = 0.0f, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f;
    uint64_t warmup_steps = 0;

    // beta1, 1 - beta1, beta2, 1 - beta2, eps, weight_decay; each complement computed in f64 and
    // rounded once (training.rs:190-203).
    std::vector<float> constants() const {
        auto complement = [](float beta) { return static_cast<float>(1.0 - static_cast<double>(beta)); };
        return {beta1, complement(beta1), beta2, complement(beta2), eps, weight_decay};
    }
};

struct StepScalars {
    float lr_t, c1, c2;
};

// `x^n` by repeated squaring, the way Rust's `f64::powi` (LLVM `powi`) multiplies it out.
inline double powi(double x, int n) {
    bool recip = n < 0;
    unsigned int m = recip ? static_cast<unsigned int>(-(static_cast<long long>(n))) : static_cast<unsigned int>(n);
    double r = 1.0;
    for (;;) {
        if (m & 1u) r *= x;
        m >>= 1;
        if (m == 0) break;
        x *= x;
    }
    return recip ? 1.0 / r : r;
}

// The host inputs of AdamW step `t`, counted from 1, of a run of `steps` steps at peak rate `lr`
// (training.rs:205-227): linear warm-up from 0, linear decay to 0 at the last step, and the two
// bias corrections, each computed in f64 and rounded once.
inline StepScalars adamw_scalars(const AdamW& a, float lr, uint64_t t, uint64_t steps) {
    double peak = static_cast<double>(lr);
    uint64_t warmup = a.warmup_steps;
    double rate;
    if (t <= warmup) {
        rate = peak * static_cast<double>(t) / static_cast<double>(warmup);
    } else {
        uint64_t span = steps > warmup ? steps - warmup : 0;
        uint64_t left = steps > t ? steps - t : 0;
        rate = span == 0 ? 0.0 : peak * static_cast<double>(left) / static_cast<double>(span);
    }
    int power = t > 0x7fffffffull ? 0x7fffffff : static_cast<int>(t);
    auto correction = [&](float beta) {
        return static_cast<float>(1.0 / (1.0 - powi(static_cast<double>(beta), power)));
    };
    return StepScalars{static_cast<float>(rate), correction(a.beta1), correction(a.beta2)};
}

namespace detail {

inline uint32_t first_read(const Program& p, uint32_t param) {
    for (const Node& n : p.nodes)
        if (n.op == Op::ParamRead && n.param == param) return n.id;
    throw Error("a parameter with a gradient is not read");
}

inline std::vector<std::pair<uint32_t, uint32_t>> gradients_of(const Program& p) {
    std::vector<std::pair<uint32_t, uint32_t>> out;
    for (const Output& o : p.outputs)
        if (o.role == Role::Gradient) out.emplace_back(o.param, o.value);
    std::sort(out.begin(), out.end());
    return out;
}

inline void check_lr(float lr) {
    if (!(std::isfinite(lr) && lr > 0.0f)) throw Error("the learning rate is not positive and finite");
}

}  // namespace detail

// `p_next = p - lr * grad` per parameter with a gradient, in parameter order.
inline Program attach_sgd(Program training, float lr) {
    detail::check_lr(lr);
    Builder b(std::move(training));
    b.tag = Tag::Optimizer;
    auto gradients = detail::gradients_of(b.program);
    std::vector<std::pair<uint32_t, uint32_t>> updates;
    if (!gradients.empty()) {
        uint32_t rate = b.scalar(lr);
        for (auto [param, grad] : gradients) {
            uint32_t read = detail::first_read(b.program, param);
            uint32_t scaled = b.op(Op::Mul, {rate, grad});
            uint32_t update = b.op(Op::Sub, {read, scaled});
            updates.emplace_back(param, update);
        }
    }
    Program& p = b.program;
    uint32_t token = 0;
    for (Node& n : p.nodes)
        if (n.op == Op::ParamRead)
            n.effect = "{!" + std::to_string(token++) + " read @" + p.params[n.param].path + " v0}";
    for (auto [param, update] : updates) {
        p.outputs.push_back(Output{update, Role::Update, param, 0});
        p.nodes[static_cast<size_t>(p.position(update))].effect =
            "{!" + std::to_string(token++) + " write @" + p.params[param].path + " v1}";
    }
    p.optimizer = OptimizerInfo{};
    p.optimizer.rule = Rule::Sgd;
    p.optimizer.lr = lr;
    return std::move(b.program);
}

// The AdamW step, each line one rounded f32 operation in this order (training.rs:925-980):
//   m' = beta1 * m + (1 - beta1) * g
//   v' = beta2 * v + ((1 - beta2) * g) * g
//   p' = p - lr_t * ((m' * c1) / (sqrt(v' * c2) + eps) + weight_decay * p)
inline Program attach_adamw(Program training, float lr, const AdamW& a) {
    detail::check_lr(lr);
    auto beta = [](float x) { return x >= 0.0f && x < 1.0f; };
    if (!(std::isfinite(a.weight_decay) && a.weight_decay >= 0.0f && beta(a.beta1) &&
          beta(a.beta2) && std::isfinite(a.eps) && a.eps > 0.0f))
        throw Error("an adamw hyperparameter is out of range");
    Builder b(std::move(training));
    b.tag = Tag::Optimizer;
    auto gradients = detail::gradients_of(b.program);
    struct State {
        uint32_t param, update, m, v, m_next, v_next;
    };
    std::vector<State> states;
    if (!gradients.empty()) {
        std::vector<uint32_t> k;
        for (float c : a.constants()) k.push_back(b.scalar(c));
        uint32_t lr_t = b.input("optimizer.lr_t", Type::f32({}));
        uint32_t c1 = b.input("optimizer.c1", Type::f32({}));
        uint32_t c2 = b.input("optimizer.c2", Type::f32({}));
        for (auto [param, g] : gradients) {
            const Param decl = b.program.params[param];
            uint32_t p = detail::first_read(b.program, param);
            uint32_t m = b.input("optimizer.m@" + decl.path, decl.ty);
            uint32_t v = b.input("optimizer.v@" + decl.path, decl.ty);
            uint32_t decayed_m = b.op(Op::Mul, {k[0], m});
            uint32_t new_m = b.op(Op::Mul, {k[1], g});
            uint32_t m_next = b.op(Op::Add, {decayed_m, new_m});
            uint32_t decayed_v = b.op(Op::Mul, {k[2], v});
            uint32_t scaled_g = b.op(Op::Mul, {k[3], g});
            uint32_t new_v = b.op(Op::Mul, {scaled_g, g});
            uint32_t v_next = b.op(Op::Add, {decayed_v, new_v});
            uint32_t m_hat = b.op(Op::Mul, {m_next, c1});
            uint32_t v_hat = b.op(Op::Mul, {v_next, c2});
            uint32_t root = b.op(Op::Sqrt, {v_hat});
            uint32_t denominator = b.op(Op::Add, {root, k[4]});
            uint32_t direction = b.op(Op::Div, {m_hat, denominator});
            uint32_t shrink = b.op(Op::Mul, {k[5], p});
            uint32_t step = b.op(Op::Add, {direction, shrink});
            uint32_t scaled = b.op(Op::Mul, {lr_t, step});
            uint32_t update = b.op(Op::Sub, {p, scaled});
            states.push_back(State{param, update, m, v, m_next, v_next});
        }
    }
    Program& p = b.program;
    auto at = [&](uint32_t v) -> Node& { return p.nodes[static_cast<size_t>(p.position(v))]; };
    uint32_t token = 0;
    auto effect = [&](const char* access, const std::string& what, int version) {
        return "{!" + std::to_string(token++) + " " + access + " " + what + " v" +
               std::to_string(version) + "}";
    };
    for (Node& n : p.nodes)
        if (n.op == Op::ParamRead) n.effect = effect("read", "@" + p.params[n.param].path, 0);
    for (const State& s : states) {
        at(s.m).effect = effect("read", "m@" + p.params[s.param].path, 0);
        at(s.v).effect = effect("read", "v@" + p.params[s.param].path, 0);
    }
    for (const State& s : states) {
        at(s.update).effect = effect("write", "@" + p.params[s.param].path, 1);
        p.outputs.push_back(Output{s.update, Role::Update, s.param, 0});
    }
    for (const State& s : states) {
        at(s.m_next).effect = effect("write", "m@" + p.params[s.param].path, 1);
        at(s.v_next).effect = effect("write", "v@" + p.params[s.param].path, 1);
        p.outputs.push_back(Output{s.m_next, Role::Moment, s.param, 'm'});
        p.outputs.push_back(Output{s.v_next, Role::Moment, s.param, 'v'});
    }
    p.optimizer = OptimizerInfo{Rule::AdamW, lr, a.weight_decay, a.beta1, a.beta2, a.eps, a.warmup_steps};
    return std::move(b.program);
}

}  // namespace msx
