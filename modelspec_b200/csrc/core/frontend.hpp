// The `.mspec` front door: reads a model and its `train` block, lowers the loss to Tensor IR and
// runs the passes that precede a backend: dead-code elimination, the masked-row gather of a
// weighted cross-entropy, differentiation, optimizer attachment, and the dropout-free forward
// program of the final loss line.
//
// The lowering follows crates/modelspec-core/src/lower.rs:1-37 (node order: inputs and targets
// in declaration order, one ParamRead per parameter in source order, then the loss, operands
// before the operation, model functions inlined), :375-414 (dropout sites and their token
// inputs), :165-196 (without_dropout); the passes follow passes/dce.rs:16-26 and
// passes/masked_rows.rs:117-292; the pipeline order is compile.rs:85-116 and :381-404. The
// language subset is what the shipped examples use (examples/*.mspec): one `model` with `param`
// and `fn` items, `let` and `return`, operator calls with the named arguments `heads` and `p`,
// and one `train` block. Generic modules (`module`, `layer`) are not read.
#pragma once

#include <cctype>
#include <memory>

#include "autodiff.hpp"

namespace msx {

struct DataDecl {
    std::string name;
    Type ty;
    bool target = false;
};

struct TrainConfig {
    std::string model;
    std::vector<DataDecl> data;  // inputs and targets in declaration order
    Rule rule = Rule::Sgd;
    float lr = 0.0f;
    AdamW adamw;
    uint64_t steps = 0;
    uint64_t seed = 0;
};

struct Compiled {
    Program forward_with_dropout;  // lowered + dce; the loss its one output
    Program forward;               // dropout the identity: the final loss line and inference
    Program step;                  // the training step
    uint32_t prediction = 0;       // the value of the one model.forward(...) call
    TrainConfig config;
    uint64_t masked_rows = 0;      // capacity of the gather, 0 for none
    std::string masked_labels, masked_weights;
    std::string function;                // compile_function: the entry; empty for the train block
    std::vector<std::string> functions;  // compile_function: the model's functions in source order
};

namespace detail {

struct Token {
    enum Kind { Ident, Number, Punct, End } kind = End;
    std::string text;
    int line = 0;
};

inline std::vector<Token> lex(const std::string& src) {
    std::vector<Token> out;
    int line = 1;
    size_t i = 0;
    while (i < src.size()) {
        char c = src[i];
        if (c == '\n') { ++line; ++i; continue; }
        if (std::isspace(static_cast<unsigned char>(c))) { ++i; continue; }
        if (c == '/' && i + 1 < src.size() && src[i + 1] == '/') {
            while (i < src.size() && src[i] != '\n') ++i;
            continue;
        }
        if (std::isalpha(static_cast<unsigned char>(c)) || c == '_') {
            size_t s = i;
            while (i < src.size() && (std::isalnum(static_cast<unsigned char>(src[i])) || src[i] == '_')) ++i;
            out.push_back({Token::Ident, src.substr(s, i - s), line});
            continue;
        }
        if (std::isdigit(static_cast<unsigned char>(c)) ||
            (c == '-' && i + 1 < src.size() && std::isdigit(static_cast<unsigned char>(src[i + 1])) )) {
            size_t s = i++;
            while (i < src.size() &&
                   (std::isalnum(static_cast<unsigned char>(src[i])) || src[i] == '.' ||
                    ((src[i] == '-' || src[i] == '+') && (src[i - 1] == 'e' || src[i - 1] == 'E'))))
                ++i;
            out.push_back({Token::Number, src.substr(s, i - s), line});
            continue;
        }
        if (c == '-' && i + 1 < src.size() && src[i + 1] == '>') {
            out.push_back({Token::Punct, "->", line});
            i += 2;
            continue;
        }
        out.push_back({Token::Punct, std::string(1, c), line});
        ++i;
    }
    out.push_back({Token::End, "", line});
    return out;
}

struct Expr {
    enum Kind { Name, Scalar, Call, ModelCall } kind = Name;
    std::string name;                 // Name: identifier; Call/ModelCall: callee
    float value = 0.0f;               // Scalar
    std::vector<std::unique_ptr<Expr>> args;
    std::map<std::string, std::string> named;  // named compile-time arguments, as written
    int dropout_index = -1;           // index of a dropout call in its body, source order
    int line = 0;
};

struct Function {
    std::string name;
    std::vector<std::pair<std::string, Type>> args;
    std::vector<std::pair<std::string, std::unique_ptr<Expr>>> lets;
    std::unique_ptr<Expr> result;
};

struct Source {
    std::string model;
    std::vector<Param> params;  // path = Model.name
    std::vector<std::string> param_names;
    std::vector<Function> functions;
    TrainConfig train;
    std::unique_ptr<Expr> loss;
};

struct Parser {
    std::vector<Token> t;
    size_t at = 0;
    int dropouts = 0;  // dropout calls seen in the body being parsed

    [[noreturn]] void fail(const std::string& what) const {
        throw Error("line " + std::to_string(t[at].line) + ": " + what + " at `" + t[at].text + "`");
    }
    bool is(const std::string& text) const { return t[at].kind != Token::End && t[at].text == text; }
    bool eat(const std::string& text) {
        if (is(text)) { ++at; return true; }
        return false;
    }
    void expect(const std::string& text) {
        if (!eat(text)) fail("expected `" + text + "`");
    }
    std::string ident() {
        if (t[at].kind != Token::Ident) fail("expected a name");
        return t[at++].text;
    }
    std::string number() {
        if (t[at].kind != Token::Number) fail("expected a number");
        return t[at++].text;
    }
    Type type() {
        expect("Tensor");
        expect("<");
        Type ty;
        std::string d = ident();
        if (d == "f32") ty.i32 = false;
        else if (d == "i32") ty.i32 = true;
        else fail("unknown element type `" + d + "`");
        expect(",");
        expect("[");
        while (!is("]")) {
            ty.shape.push_back(std::strtoull(number().c_str(), nullptr, 10));
            if (!eat(",")) break;
        }
        expect("]");
        expect(">");
        return ty;
    }
    std::unique_ptr<Expr> expr() {
        auto e = std::make_unique<Expr>();
        e->line = t[at].line;
        if (t[at].kind == Token::Number) {
            e->kind = Expr::Scalar;
            e->value = std::strtof(number().c_str(), nullptr);
            return e;
        }
        std::string name = ident();
        if ((name == "model" || name == "self") && eat(".")) {
            e->kind = Expr::ModelCall;
            e->name = ident();
        } else if (is("(")) {
            e->kind = Expr::Call;
            e->name = name;
        } else {
            e->kind = Expr::Name;
            e->name = name;
            return e;
        }
        if (e->kind == Expr::Call && e->name == "dropout") e->dropout_index = dropouts++;
        expect("(");
        while (!is(")")) {
            if (t[at].kind == Token::Ident && t[at + 1].kind == Token::Punct && t[at + 1].text == "=") {
                std::string key = ident();
                expect("=");
                e->named[key] = t[at].kind == Token::Number ? number() : ident();
            } else {
                e->args.push_back(expr());
            }
            if (!eat(",")) break;
        }
        expect(")");
        return e;
    }
    Source parse() {
        Source s;
        while (t[at].kind != Token::End) {
            if (eat("model")) {
                s.model = ident();
                expect("{");
                while (!eat("}")) {
                    if (eat("param")) {
                        Param p;
                        std::string name = ident();
                        expect(":");
                        p.ty = type();
                        expect("=");
                        std::string init = ident();
                        expect("(");
                        expect(")");
                        expect(";");
                        if (init == "xavier_uniform") p.init = Init::XavierUniform;
                        else if (init == "zeros") p.init = Init::Zeros;
                        else if (init == "ones") p.init = Init::Ones;
                        else fail("unknown initializer `" + init + "`");
                        if (p.ty.i32) fail("a parameter is f32");
                        if (p.init == Init::XavierUniform && p.ty.rank() != 2)
                            fail("xavier_uniform needs rank 2");
                        p.path = s.model + "." + name;
                        s.params.push_back(p);
                        s.param_names.push_back(name);
                    } else if (eat("fn")) {
                        Function f;
                        f.name = ident();
                        expect("(");
                        while (!is(")")) {
                            std::string arg = ident();
                            expect(":");
                            f.args.emplace_back(arg, type());
                            if (!eat(",")) break;
                        }
                        expect(")");
                        expect("->");
                        type();
                        expect("{");
                        dropouts = 0;
                        while (eat("let")) {
                            std::string name = ident();
                            expect("=");
                            auto value = expr();
                            expect(";");
                            f.lets.emplace_back(name, std::move(value));
                        }
                        expect("return");
                        f.result = expr();
                        expect(";");
                        expect("}");
                        s.functions.push_back(std::move(f));
                    } else {
                        fail("expected `param` or `fn`");
                    }
                }
            } else if (eat("train")) {
                ident();
                expect("{");
                while (!eat("}")) {
                    std::string key = ident();
                    if (key == "input" || key == "target") {
                        DataDecl d;
                        d.name = ident();
                        expect(":");
                        d.ty = type();
                        d.target = key == "target";
                        expect(";");
                        s.train.data.push_back(d);
                        continue;
                    }
                    expect("=");
                    if (key == "model") s.train.model = ident();
                    else if (key == "loss") { dropouts = 0; s.loss = expr(); }
                    else if (key == "optimizer") {
                        auto o = expr();
                        auto f = [&](const char* k, float fallback, bool required) {
                            auto it = o->named.find(k);
                            if (it == o->named.end()) {
                                if (required) fail(std::string("optimizer needs `") + k + "`");
                                return fallback;
                            }
                            return std::strtof(it->second.c_str(), nullptr);
                        };
                        s.train.lr = f("lr", 0.0f, true);
                        if (o->name == "sgd") s.train.rule = Rule::Sgd;
                        else if (o->name == "adamw") {
                            s.train.rule = Rule::AdamW;
                            AdamW& a = s.train.adamw;
                            a.weight_decay = f("weight_decay", 0.0f, true);
                            a.beta1 = f("beta1", 0.0f, true);
                            a.beta2 = f("beta2", 0.0f, true);
                            a.eps = f("eps", 0.0f, true);
                            auto w = o->named.find("warmup_steps");
                            a.warmup_steps = w == o->named.end() ? 0 : std::strtoull(w->second.c_str(), nullptr, 10);
                        } else fail("the optimizer `" + o->name + "` has no CUDA kernel");
                    }
                    else if (key == "steps") s.train.steps = std::strtoull(number().c_str(), nullptr, 10);
                    else if (key == "seed") s.train.seed = std::strtoull(number().c_str(), nullptr, 10);
                    else if (key == "device") { ident(); if (eat("(")) { number(); expect(")"); } }
                    else fail("unknown train item `" + key + "`");
                    expect(";");
                }
            } else {
                fail("expected `model` or `train`");
            }
        }
        if (!s.loss) throw Error("the train block has no loss");
        if (s.train.model != s.model) throw Error("the train block names another model");
        return s;
    }
};

struct Frame {
    const Function* function = nullptr;     // null: the train block
    std::vector<uint32_t> args, lets;
    std::string site_prefix;                // `<Model>.<fn>` or `<Model>.<fn>@<c>`
};

struct Lowering {
    const Source& src;
    Builder b;
    std::vector<uint32_t> data, reads;
    std::vector<size_t> inlined;
    std::vector<const Function*> inlining;
    std::map<std::string, uint32_t> tokens;
    std::vector<uint32_t> predictions;

    explicit Lowering(const Source& s) : src(s), inlined(s.functions.size(), 0) {}

    uint32_t name(const Expr& e, const Frame& f) {
        if (f.function) {
            for (size_t i = f.function->lets.size(); i-- > 0;)
                if (i < f.lets.size() && f.function->lets[i].first == e.name) return f.lets[i];
            for (size_t i = 0; i < f.function->args.size(); ++i)
                if (f.function->args[i].first == e.name) return f.args[i];
        } else {
            for (size_t i = 0; i < src.train.data.size(); ++i)
                if (src.train.data[i].name == e.name) return data[i];
        }
        if (f.function)
            for (size_t i = 0; i < src.param_names.size(); ++i)
                if (src.param_names[i] == e.name) return reads[i];
        throw Error("line " + std::to_string(e.line) + ": unknown name `" + e.name + "`");
    }

    uint32_t inline_call(const Expr& e, std::vector<uint32_t> values) {
        size_t fi = 0;
        for (; fi < src.functions.size(); ++fi)
            if (src.functions[fi].name == e.name) break;
        if (fi == src.functions.size())
            throw Error("line " + std::to_string(e.line) + ": the model has no function `" + e.name + "`");
        const Function& fn = src.functions[fi];
        for (const Function* open : inlining)
            if (open == &fn) throw Error("`" + fn.name + "` calls itself");
        if (values.size() != fn.args.size())
            throw Error("line " + std::to_string(e.line) + ": `" + fn.name + "` takes " +
                        std::to_string(fn.args.size()) + " arguments");
        for (size_t i = 0; i < values.size(); ++i)
            if (b.type_of(values[i]) != fn.args[i].second)
                throw Error("line " + std::to_string(e.line) + ": argument `" + fn.args[i].first +
                            "` is " + b.type_of(values[i]).str() + ", not " + fn.args[i].second.str());
        Frame frame;
        frame.function = &fn;
        frame.args = std::move(values);
        size_t instance = inlined[fi]++;
        frame.site_prefix = src.model + "." + fn.name + (instance ? "@" + std::to_string(instance) : "");
        inlining.push_back(&fn);
        for (const auto& binding : fn.lets) frame.lets.push_back(expr(*binding.second, frame));
        uint32_t value = expr(*fn.result, frame);
        inlining.pop_back();
        if (fn.name == "forward") predictions.push_back(value);
        return value;
    }

    uint32_t expr(const Expr& e, const Frame& f) {
        switch (e.kind) {
            case Expr::Name: return name(e, f);
            case Expr::Scalar: return b.scalar(e.value);
            case Expr::ModelCall: {
                std::vector<uint32_t> values;
                for (const auto& a : e.args) values.push_back(expr(*a, f));
                return inline_call(e, std::move(values));
            }
            case Expr::Call: break;
        }
        static const std::pair<const char*, Op> operators[] = {
            {"matmul", Op::MatMul}, {"add", Op::Add}, {"sub", Op::Sub}, {"mul", Op::Mul},
            {"relu", Op::Relu}, {"transpose", Op::Transpose}, {"sum", Op::ReduceSum},
            {"mean", Op::ReduceMean}, {"mse", Op::Mse}, {"embedding", Op::Embedding},
            {"add_rows", Op::AddRows}, {"gelu", Op::Gelu}, {"layer_norm", Op::LayerNorm},
            {"softmax", Op::Softmax}, {"attention", Op::Attention},
            {"cross_entropy", Op::CrossEntropy}, {"dropout", Op::Dropout},
            {"stop_gradient", Op::StopGradient}};
        const Op* op = nullptr;
        for (const auto& entry : operators)
            if (e.name == entry.first) op = &entry.second;
        if (!op) {
            // A bare call of a model function from inside the model.
            std::vector<uint32_t> values;
            for (const auto& a : e.args) values.push_back(expr(*a, f));
            for (const Function& fn : src.functions)
                if (fn.name == e.name) return inline_call(e, std::move(values));
            throw Error("line " + std::to_string(e.line) + ": the operator `" + e.name +
                        "` has no CUDA kernel");
        }
        Node n;
        n.op = *op;
        for (const auto& a : e.args) n.operands.push_back(expr(*a, f));
        auto named = [&](const char* key) -> const std::string& {
            auto it = e.named.find(key);
            if (it == e.named.end())
                throw Error("line " + std::to_string(e.line) + ": `" + e.name + "` needs `" + key + " = ...`");
            return it->second;
        };
        if (*op == Op::Attention) n.heads = std::strtoull(named("heads").c_str(), nullptr, 10);
        if (*op == Op::Dropout) {
            n.p = std::strtof(named("p").c_str(), nullptr);
            if (!(n.p >= 0.0f && n.p < 1.0f)) throw Error("dropout p is outside [0, 1)");
            if (n.operands.size() != 1) throw Error("dropout takes 1 operand");
            if (n.p == 0.0f) return n.operands[0];
            std::string site = (f.function ? f.site_prefix : src.model + ".train") + ".dropout#" +
                               std::to_string(e.dropout_index);
            auto it = tokens.find(site);
            uint32_t token = it != tokens.end() ? it->second : (tokens[site] = b.input(site, Type::ids({2})));
            n.operands.push_back(token);
        }
        return b.push(std::move(n));
    }
};

}  // namespace detail

// Removes every node no output reaches (passes/dce.rs:16-26).
inline Program dce(Program program) {
    std::set<uint32_t> live;
    for (const Output& o : program.outputs) live.insert(o.value);
    for (size_t i = program.nodes.size(); i-- > 0;)
        if (live.count(program.nodes[i].id))
            for (uint32_t o : program.nodes[i].operands) live.insert(o);
    std::vector<Node> kept;
    for (Node& n : program.nodes)
        if (live.count(n.id)) kept.push_back(std::move(n));
    program.nodes = std::move(kept);
    program.refresh_inputs();
    return program;
}

// Every Dropout the identity (lower.rs:165-196).
inline Program without_dropout(Program program) {
    std::map<uint32_t, uint32_t> identity;
    std::vector<Node> kept;
    for (Node& n : program.nodes) {
        for (uint32_t& o : n.operands) {
            auto it = identity.find(o);
            if (it != identity.end()) o = it->second;
        }
        if (n.op == Op::Dropout) identity[n.id] = n.operands.at(0);
        else kept.push_back(std::move(n));
    }
    program.nodes = std::move(kept);
    for (Output& o : program.outputs) {
        auto it = identity.find(o.value);
        if (it != identity.end()) o.value = it->second;
    }
    return dce(std::move(program));
}

// The capacity of the masked-row gather for `rows` rows each selected with probability `rate`:
// the expected count plus 8 standard deviations, rounded up to a multiple of 64, at most `rows`
// (crates/modelspec-cli/src/train.rs:379-388).
inline uint64_t default_masked_rows(uint64_t rows, double rate) {
    double n = static_cast<double>(rows);
    rate = std::min(1.0, std::max(0.0, rate));
    double bound = n * rate + 8.0 * std::sqrt(n * rate * (1.0 - rate));
    uint64_t capacity = (static_cast<uint64_t>(std::ceil(bound)) + 63) / 64 * 64;
    return std::min(capacity, rows);
}

// The masked-row gather of a weighted cross-entropy loss (passes/masked_rows.rs:117-206,
// :232-292): a copy of the row-local head on `capacity` gathered rows, read by the loss with the
// gathered labels and weights. Returns the program unchanged when it has no such site.
inline Program masked_rows_gather(Program program, uint64_t capacity, std::string* labels_name,
                                  std::string* weights_name) {
    if (program.outputs.size() != 1) return program;
    int loss_at = program.position(program.outputs[0].value);
    if (loss_at < 0) return program;
    const Node loss = program.nodes[static_cast<size_t>(loss_at)];
    if (loss.op != Op::CrossEntropy) return program;
    auto input_name = [&](uint32_t v, std::string* out) {
        const Node& n = program.node(v);
        if (n.op != Op::Input) return false;
        *out = n.name;
        return true;
    };
    std::string labels, weights;
    if (!input_name(loss.operands[1], &labels) || !input_name(loss.operands[2], &weights)) return program;
    const Type& logits_ty = program.node(loss.operands[0]).ty;
    if (logits_ty.rank() != 2) return program;
    uint64_t rows = logits_ty.shape[0];
    if (capacity == 0 || capacity >= rows) return program;
    // Values that depend on no input: the same for every row of a batch (:294-).
    std::set<uint32_t> row_free;
    for (const Node& n : program.nodes) {
        bool leaf = n.op == Op::ParamRead || n.op == Op::Scalar;
        bool derived = !n.operands.empty();
        for (uint32_t o : n.operands) derived = derived && row_free.count(o);
        if (leaf || derived) row_free.insert(n.id);
    }
    std::map<uint32_t, int> consumers;
    for (const Node& n : program.nodes)
        for (uint32_t o : n.operands) consumers[o]++;
    for (const Output& o : program.outputs) consumers[o.value]++;
    std::vector<Node> chain;  // head nodes, logits first while walking back
    const Node* current = &program.node(loss.operands[0]);
    for (;;) {
        bool row_local = current->op == Op::AddRows || current->op == Op::MatMul ||
                         current->op == Op::Gelu || current->op == Op::LayerNorm;
        bool rest_free = true;
        for (size_t i = 1; i < current->operands.size(); ++i)
            rest_free = rest_free && row_free.count(current->operands[i]);
        if (!row_local || consumers[current->id] != 1 || !rest_free) break;
        chain.push_back(*current);
        current = &program.node(current->operands[0]);
    }
    if (chain.empty() || current->ty.i32 || current->ty.rank() != 2) return program;
    uint32_t frontier = current->id;
    std::reverse(chain.begin(), chain.end());

    std::vector<Node> before(program.nodes.begin(), program.nodes.begin() + loss_at);
    std::vector<Node> after(program.nodes.begin() + loss_at + 1, program.nodes.end());
    Program head = program;
    head.nodes = before;
    Builder b(std::move(head));
    b.next = program.next_id();
    uint32_t rows_in = b.input("masked.rows", Type::ids({capacity}));
    uint32_t labels_in = b.input("masked.labels." + labels, Type::ids({capacity}));
    uint32_t weights_in = b.input("masked.weights." + weights, Type::f32({capacity}));
    uint32_t value = b.op(Op::Embedding, {frontier, rows_in});
    for (const Node& link : chain) {
        Node n = link;
        n.operands[0] = value;
        n.tag = Tag::None;
        value = b.push(std::move(n));
    }
    Node gathered_loss = loss;
    gathered_loss.operands = {value, labels_in, weights_in};
    b.program.nodes.push_back(gathered_loss);
    for (Node& n : after) b.program.nodes.push_back(std::move(n));
    b.program.refresh_inputs();
    if (labels_name) *labels_name = labels;
    if (weights_name) *weights_name = weights;
    return std::move(b.program);
}

// Compiles `.mspec` source to its training step and forward program. `masked_rows` is the
// capacity of the masked-row gather, 0 for none.
inline Compiled compile_training(const std::string& source, uint64_t masked_rows = 0) {
    detail::Parser parser;
    parser.t = detail::lex(source);
    detail::Source src = parser.parse();
    detail::Lowering lo(src);
    lo.b.program.params = src.params;
    for (const DataDecl& d : src.train.data) lo.data.push_back(lo.b.input(d.name, d.ty));
    for (size_t i = 0; i < src.params.size(); ++i)
        lo.reads.push_back(lo.b.param_read(static_cast<uint32_t>(i)));
    detail::Frame train_frame;
    uint32_t loss = lo.expr(*src.loss, train_frame);
    if (lo.b.type_of(loss).rank() != 0) throw Error("the loss is not rank 0");
    if (lo.predictions.size() != 1) throw Error("the loss does not call model.forward exactly once");
    lo.b.program.outputs = {Output{loss, Role::Plain, 0, 0}};

    Compiled out;
    out.config = src.train;
    out.prediction = lo.predictions[0];
    out.forward_with_dropout = dce(std::move(lo.b.program));
    Program differentiated = out.forward_with_dropout;
    if (masked_rows) {
        size_t before = differentiated.nodes.size();
        differentiated = masked_rows_gather(std::move(differentiated), masked_rows,
                                            &out.masked_labels, &out.masked_weights);
        if (differentiated.nodes.size() != before) out.masked_rows = masked_rows;
    }
    Program training = without_stop_gradient(differentiate(differentiated));
    out.step = src.train.rule == Rule::AdamW ? attach_adamw(std::move(training), src.train.lr, src.train.adamw)
                                             : attach_sgd(std::move(training), src.train.lr);
    Program fwd = without_stop_gradient(without_dropout(out.forward_with_dropout));
    // The prediction may have been a Dropout: follow it to its operand.
    {
        uint32_t p = out.prediction;
        while (fwd.position(p) < 0) {
            const Node& n = out.forward_with_dropout.node(p);
            if (n.op != Op::Dropout && n.op != Op::StopGradient) break;
            p = n.operands[0];
        }
        out.prediction = p;
    }
    out.forward = dce(std::move(fwd));
    return out;
}

// The model function `name` as an inference entry (compile.rs:173-223, function_entry :239-288 of
// the reference): one `input` per argument, named and typed as the argument; the prediction is the
// function's result; the loss is the result itself when it is rank 0 and its mean otherwise; every
// dropout is the identity; the parameter table is the file's, so a checkpoint of the file supplies
// the parameters. The step differentiates that loss and attaches sgd at the block's learning rate
// whatever the block's optimizer; nothing runs its update. The configuration keeps the block's
// seed and steps. A name the model does not declare is E-DATA-010 with the functions it declares
// (train/data.rs:719-730).
inline Compiled compile_function(const std::string& source, const std::string& name) {
    detail::Parser parser;
    parser.t = detail::lex(source);
    detail::Source src = parser.parse();
    Compiled out;
    for (const detail::Function& f : src.functions) out.functions.push_back(f.name);
    const detail::Function* entry = nullptr;
    for (const detail::Function& f : src.functions)
        if (f.name == name) entry = &f;
    if (!entry) {
        std::string listed;
        for (const std::string& f : out.functions) listed += (listed.empty() ? "" : ", ") + f;
        throw Error("E-DATA-010: the model declares no function `" + name + "`\n  function: " + name + "\n  functions: " + listed);
    }
    src.train.data.clear();
    for (const auto& arg : entry->args) src.train.data.push_back(DataDecl{arg.first, arg.second, false});
    src.train.rule = Rule::Sgd;
    detail::Lowering lo(src);
    lo.b.program.params = src.params;
    for (const DataDecl& d : src.train.data) lo.data.push_back(lo.b.input(d.name, d.ty));
    for (size_t i = 0; i < src.params.size(); ++i) lo.reads.push_back(lo.b.param_read(static_cast<uint32_t>(i)));
    detail::Expr call;
    call.kind = detail::Expr::ModelCall;
    call.name = name;
    uint32_t result = lo.inline_call(call, lo.data);
    uint32_t loss = result;
    if (lo.b.type_of(result).rank() != 0) {
        Node mean;
        mean.op = Op::ReduceMean;
        mean.operands = {result};
        loss = lo.b.push(std::move(mean));
    }
    lo.b.program.outputs = {Output{loss, Role::Plain, 0, 0}};
    const Program with_dropout = dce(std::move(lo.b.program));
    Program lowered = without_dropout(with_dropout);
    // The result may have been a Dropout: follow it to its operand.
    while (lowered.position(result) < 0) {
        const Node& n = with_dropout.node(result);
        if (n.op != Op::Dropout) break;
        result = n.operands[0];
    }
    out.config = src.train;
    out.function = name;
    out.prediction = result;
    out.forward_with_dropout = lowered;
    out.step = attach_sgd(without_stop_gradient(differentiate(lowered)), src.train.lr);
    Program fwd = without_stop_gradient(lowered);
    while (fwd.position(out.prediction) < 0) {
        const Node& n = lowered.node(out.prediction);
        if (n.op != Op::StopGradient) break;
        out.prediction = n.operands[0];
    }
    out.forward = dce(std::move(fwd));
    return out;
}

}  // namespace msx
