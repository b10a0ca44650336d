// Tensor IR: the typed SSA program a ModelSpec training step is, with the text form the
// reference prints for `modelspec ir --stage tensor|training` and a reader of that text.
//
// The text form is the interchange at the backend boundary: the reference's printer
// (crates/modelspec-core/src/ir/print.rs:55-166, write_training and write_node :269-307) writes
// it, `parse_program` reads it back. The op set is the reference's TensorOp
// (crates/modelspec-core/src/ir/tensor.rs:129-273) without the `sigreg` family, which is not part
// of the BERT operator set.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace msx {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

enum class Op : uint8_t {
    Input, ParamRead, Scalar, Add, Sub, Mul, MatMul, Relu, Transpose, ReduceSum, ReduceMean, Mse,
    ReluGrad, BroadcastScalar, Embedding, EmbeddingGrad, AddRows, SumRows, Gelu, GeluGrad,
    LayerNorm, LayerNormGradX, LayerNormGradGamma, Softmax, SoftmaxGrad, Attention,
    AttentionGradQ, AttentionGradK, AttentionGradV, CrossEntropy, CrossEntropyGrad, Dropout,
    DropoutGrad, StopGradient, Sqrt, Div, Count
};

inline const char* op_name(Op op) {
    static const char* names[] = {
        "Input", "ParamRead", "Scalar", "Add", "Sub", "Mul", "MatMul", "Relu", "Transpose",
        "ReduceSum", "ReduceMean", "Mse", "ReluGrad", "BroadcastScalar", "Embedding",
        "EmbeddingGrad", "AddRows", "SumRows", "Gelu", "GeluGrad", "LayerNorm", "LayerNormGradX",
        "LayerNormGradGamma", "Softmax", "SoftmaxGrad", "Attention", "AttentionGradQ",
        "AttentionGradK", "AttentionGradV", "CrossEntropy", "CrossEntropyGrad", "Dropout",
        "DropoutGrad", "StopGradient", "Sqrt", "Div"};
    return op < Op::Count ? names[static_cast<int>(op)] : "?";
}

inline bool op_from_name(const std::string& name, Op* out) {
    for (int i = 0; i < static_cast<int>(Op::Count); ++i) {
        if (name == op_name(static_cast<Op>(i))) {
            *out = static_cast<Op>(i);
            return true;
        }
    }
    return false;
}

// A tensor type, printed `Tensor<f32, [8, 1]>`; rank 0 is a scalar (tensor.rs:82-126).
struct Type {
    bool i32 = false;
    std::vector<uint64_t> shape;

    uint64_t count() const {
        uint64_t n = 1;
        for (uint64_t d : shape) n *= d;
        return n;
    }
    size_t rank() const { return shape.size(); }
    bool operator==(const Type& o) const { return i32 == o.i32 && shape == o.shape; }
    bool operator!=(const Type& o) const { return !(*this == o); }

    std::string str() const {
        std::string s = i32 ? "Tensor<i32, [" : "Tensor<f32, [";
        for (size_t i = 0; i < shape.size(); ++i) {
            if (i) s += ", ";
            s += std::to_string(shape[i]);
        }
        return s + "]>";
    }
    static Type f32(std::vector<uint64_t> shape) { return Type{false, std::move(shape)}; }
    static Type ids(std::vector<uint64_t> shape) { return Type{true, std::move(shape)}; }
};

enum class Init : uint8_t { XavierUniform, Zeros, Ones };

inline const char* init_name(Init i) {
    return i == Init::XavierUniform ? "xavier_uniform" : i == Init::Zeros ? "zeros" : "ones";
}

struct Param {
    std::string path;  // canonical path, `Model.name`
    Type ty;
    Init init = Init::Zeros;
};

// The subgraph tag a training program prints before each node (training.rs Subgraph).
enum class Tag : uint8_t { None, Forward, Loss, Gradient, Optimizer };

inline const char* tag_name(Tag t) {
    switch (t) {
        case Tag::Forward: return "forward";
        case Tag::Loss: return "loss";
        case Tag::Gradient: return "gradient";
        case Tag::Optimizer: return "optimizer";
        default: return "";
    }
}

struct Node {
    uint32_t id = 0;
    Op op = Op::Input;
    std::vector<uint32_t> operands;
    Type ty;
    std::string name;             // Input: its name
    uint32_t param = 0;           // ParamRead: index into Program::params
    float scalar = 0.0f;          // Scalar: its value
    uint64_t heads = 0;           // Attention and its gradient ops
    uint64_t rows = 0;            // EmbeddingGrad: rows of the table
    float p = 0.0f;               // Dropout, DropoutGrad
    std::vector<uint64_t> bshape; // BroadcastScalar
    Tag tag = Tag::None;
    std::string effect;           // `{!0 read @M.w v0}` of a training step, braces included
};

enum class Role : uint8_t { Plain, Loss, Gradient, Update, Moment };

struct Output {
    uint32_t value = 0;
    Role role = Role::Plain;
    uint32_t param = 0;  // Gradient, Update, Moment: index into Program::params
    char moment = 0;     // Moment: 'm' or 'v'
};

enum class Rule : uint8_t { None, Sgd, AdamW };

// The optimizer line of a training step (print.rs:75-84).
struct OptimizerInfo {
    Rule rule = Rule::None;
    float lr = 0.0f;
    float weight_decay = 0.0f, beta1 = 0.0f, beta2 = 0.0f, eps = 0.0f;
    uint64_t warmup_steps = 0;
};

struct Program {
    std::vector<Param> params;
    std::vector<Node> nodes;
    std::vector<uint32_t> inputs;  // ids of the Input nodes, in node order
    std::vector<Output> outputs;
    OptimizerInfo optimizer;
    bool tagged = false;  // a training program: nodes print their subgraph tag

    int position(uint32_t id) const {
        // Ids are dense and ascending in practice; fall back to a scan.
        if (id < nodes.size() && nodes[id].id == id) return static_cast<int>(id);
        for (size_t i = 0; i < nodes.size(); ++i)
            if (nodes[i].id == id) return static_cast<int>(i);
        return -1;
    }
    const Node& node(uint32_t id) const {
        int at = position(id);
        if (at < 0) throw Error("value %" + std::to_string(id) + " is not defined");
        return nodes[static_cast<size_t>(at)];
    }
    int param_index(const std::string& path) const {
        for (size_t i = 0; i < params.size(); ++i)
            if (params[i].path == path) return static_cast<int>(i);
        return -1;
    }
    uint32_t next_id() const {
        uint32_t m = 0;
        for (const Node& n : nodes) m = std::max(m, n.id + 1);
        return m;
    }
    void refresh_inputs() {
        inputs.clear();
        for (const Node& n : nodes)
            if (n.op == Op::Input) inputs.push_back(n.id);
    }
};

// ---------------------------------------------------------------------------------------------
// f32 text, as Rust prints it. `{:?}` (Debug) is the shortest digits that read back to the same
// f32, with `.0` after an integer and exponent form below 1e-4 and from 1e16; `{}` (Display) is
// the same digits, never in exponent form.

inline void shortest_digits(float v, std::string* digits, int* exp10) {
    // digits d1d2...dn and exponent e such that v = 0.d1d2...dn * 10^e, n minimal.
    char buf[64];
    for (int prec = 0; prec < 9; ++prec) {
        std::snprintf(buf, sizeof buf, "%.*e", prec, static_cast<double>(v));
        if (std::strtof(buf, nullptr) == v) break;
    }
    std::string s(buf);
    size_t e = s.find('e');
    std::string mant = s.substr(0, e);
    int ex = std::atoi(s.c_str() + e + 1);
    digits->clear();
    for (char c : mant)
        if (c >= '0' && c <= '9') digits->push_back(c);
    while (digits->size() > 1 && digits->back() == '0') digits->pop_back();
    *exp10 = ex + 1;
}

inline std::string plain_decimal(const std::string& digits, int exp10, bool force_fraction) {
    std::string out;
    int n = static_cast<int>(digits.size());
    if (exp10 <= 0) {
        out = "0.";
        out.append(static_cast<size_t>(-exp10), '0');
        out += digits;
    } else if (exp10 >= n) {
        out = digits;
        out.append(static_cast<size_t>(exp10 - n), '0');
        if (force_fraction) out += ".0";
    } else {
        out = digits.substr(0, static_cast<size_t>(exp10)) + "." +
              digits.substr(static_cast<size_t>(exp10));
    }
    return out;
}

inline std::string f32_special(float v) {
    if (std::isnan(v)) return "NaN";
    if (std::isinf(v)) return v < 0 ? "-inf" : "inf";
    return "";
}

// Rust `{:?}` of an f32.
inline std::string f32_debug(float v) {
    std::string special = f32_special(v);
    if (!special.empty()) return special;
    std::string sign = std::signbit(v) ? "-" : "";
    float a = std::fabs(v);
    if (a == 0.0f) return sign + "0.0";
    std::string digits;
    int exp10;
    shortest_digits(a, &digits, &exp10);
    if (a >= 1e16f || a < 1e-4f) {
        std::string out = sign + digits.substr(0, 1);
        if (digits.size() > 1) out += "." + digits.substr(1);
        return out + "e" + std::to_string(exp10 - 1);
    }
    return sign + plain_decimal(digits, exp10, true);
}

// Rust `{}` of an f64: the shortest digits that read back to the same f64, as a plain decimal.
inline std::string f64_display(double v) {
    if (std::isnan(v)) return "NaN";
    if (std::isinf(v)) return v < 0 ? "-inf" : "inf";
    std::string sign = std::signbit(v) ? "-" : "";
    double a = std::fabs(v);
    if (a == 0.0) return sign + "0";
    char buf[64];
    for (int prec = 0; prec < 17; ++prec) {
        std::snprintf(buf, sizeof buf, "%.*e", prec, a);
        if (std::strtod(buf, nullptr) == a) break;
    }
    std::string text(buf);
    const size_t e = text.find('e');
    std::string digits;
    for (char c : text.substr(0, e))
        if (c >= '0' && c <= '9') digits.push_back(c);
    while (digits.size() > 1 && digits.back() == '0') digits.pop_back();
    return sign + plain_decimal(digits, std::atoi(text.c_str() + e + 1) + 1, false);
}

// Rust `{}` of an f32.
inline std::string f32_display(float v) {
    std::string special = f32_special(v);
    if (!special.empty()) return special;
    std::string sign = std::signbit(v) ? "-" : "";
    float a = std::fabs(v);
    if (a == 0.0f) return sign + "0";
    std::string digits;
    int exp10;
    shortest_digits(a, &digits, &exp10);
    return sign + plain_decimal(digits, exp10, false);
}

// ---------------------------------------------------------------------------------------------
// Printer (print.rs:55-166, :269-307).

inline std::string node_text(const Program& program, const Node& node) {
    std::string s = "%" + std::to_string(node.id) + ": " + node.ty.str() + " = " + op_name(node.op);
    switch (node.op) {
        case Op::Input: s += " \"" + node.name + "\""; break;
        case Op::ParamRead: s += " @" + program.params.at(node.param).path; break;
        case Op::Scalar: s += " " + f32_debug(node.scalar); break;
        case Op::BroadcastScalar: {
            s += " [";
            for (size_t i = 0; i < node.bshape.size(); ++i) {
                if (i) s += ", ";
                s += std::to_string(node.bshape[i]);
            }
            s += "]";
            break;
        }
        case Op::EmbeddingGrad: s += " [" + std::to_string(node.rows) + "]"; break;
        case Op::Attention:
        case Op::AttentionGradQ:
        case Op::AttentionGradK:
        case Op::AttentionGradV: s += " [heads = " + std::to_string(node.heads) + "]"; break;
        case Op::Dropout:
        case Op::DropoutGrad: {
            size_t token_at = node.op == Op::Dropout ? 1 : 0;
            std::string site = "?";
            if (token_at < node.operands.size()) {
                int at = program.position(node.operands[token_at]);
                if (at >= 0 && program.nodes[static_cast<size_t>(at)].op == Op::Input)
                    site = program.nodes[static_cast<size_t>(at)].name;
            }
            s += " [p = " + f32_debug(node.p) + ", site = " + site + "]";
            break;
        }
        default: break;
    }
    for (size_t i = 0; i < node.operands.size(); ++i) {
        s += i ? ", %" : " %";
        s += std::to_string(node.operands[i]);
    }
    return s;
}

inline std::string print_program(const Program& program) {
    std::string out;
    bool step = program.optimizer.rule != Rule::None;
    for (const Param& p : program.params) {
        out += "param @" + p.path + ": " + p.ty.str() + " = " + init_name(p.init);
        if (step) out += " {v0}";
        out += "\n";
    }
    const OptimizerInfo& o = program.optimizer;
    if (o.rule == Rule::Sgd) {
        out += "optimizer sgd lr = " + f32_debug(o.lr) + "\n";
    } else if (o.rule == Rule::AdamW) {
        out += "optimizer adamw lr = " + f32_debug(o.lr) + " weight_decay = " +
               f32_debug(o.weight_decay) + " beta1 = " + f32_debug(o.beta1) + " beta2 = " +
               f32_debug(o.beta2) + " eps = " + f32_debug(o.eps) + " warmup_steps = " +
               std::to_string(o.warmup_steps) + "\n";
    }
    for (const Node& n : program.nodes) {
        if (program.tagged && n.tag != Tag::None) out += std::string(tag_name(n.tag)) + " ";
        out += node_text(program, n);
        if (!n.effect.empty()) out += " " + n.effect;
        out += "\n";
    }
    for (const Output& o2 : program.outputs) {
        out += "output %" + std::to_string(o2.value);
        switch (o2.role) {
            case Role::Loss: out += " loss"; break;
            case Role::Gradient: out += " gradient @" + program.params.at(o2.param).path; break;
            case Role::Update: out += " update @" + program.params.at(o2.param).path; break;
            case Role::Moment:
                out += std::string(" moment ") + o2.moment + " @" + program.params.at(o2.param).path;
                break;
            default: break;
        }
        out += "\n";
    }
    return out;
}

// ---------------------------------------------------------------------------------------------
// Reader of the text form.

namespace detail {

struct Cursor {
    const std::string& s;
    size_t at = 0;
    int line_no;

    [[noreturn]] void fail(const std::string& what) const {
        throw Error("IR line " + std::to_string(line_no) + ": " + what + " in `" + s + "`");
    }
    void skip_ws() {
        while (at < s.size() && s[at] == ' ') ++at;
    }
    bool eat(const std::string& lit) {
        skip_ws();
        if (s.compare(at, lit.size(), lit) == 0) {
            at += lit.size();
            return true;
        }
        return false;
    }
    void expect(const std::string& lit) {
        if (!eat(lit)) fail("expected `" + lit + "`");
    }
    bool done() {
        skip_ws();
        return at >= s.size();
    }
    uint64_t number() {
        skip_ws();
        size_t start = at;
        while (at < s.size() && s[at] >= '0' && s[at] <= '9') ++at;
        if (start == at) fail("expected a number");
        return std::strtoull(s.substr(start, at - start).c_str(), nullptr, 10);
    }
    std::string word() {  // up to a space, comma, or bracket
        skip_ws();
        size_t start = at;
        while (at < s.size() && s[at] != ' ' && s[at] != ',' && s[at] != ']' && s[at] != ':') ++at;
        if (start == at) fail("expected a word");
        return s.substr(start, at - start);
    }
    float f32() {
        std::string w = word();
        if (w == "NaN") return std::nanf("");
        if (w == "inf") return INFINITY;
        if (w == "-inf") return -INFINITY;
        char* end = nullptr;
        float v = std::strtof(w.c_str(), &end);
        if (end == w.c_str() || *end) fail("`" + w + "` is not an f32");
        return v;
    }
    std::vector<uint64_t> dims() {
        expect("[");
        std::vector<uint64_t> out;
        if (eat("]")) return out;
        for (;;) {
            out.push_back(number());
            if (eat("]")) break;
            expect(",");
        }
        return out;
    }
    Type type() {
        expect("Tensor<");
        Type t;
        if (eat("f32")) t.i32 = false;
        else if (eat("i32")) t.i32 = true;
        else fail("expected f32 or i32");
        expect(",");
        t.shape = dims();
        expect(">");
        return t;
    }
    uint32_t value() {
        expect("%");
        return static_cast<uint32_t>(number());
    }
    std::string path() {  // @Model.name, up to a space or `:`
        expect("@");
        return word();
    }
};

}  // namespace detail

inline Program parse_program(const std::string& text) {
    Program program;
    size_t start = 0;
    int line_no = 0;
    while (start < text.size()) {
        size_t end = text.find('\n', start);
        if (end == std::string::npos) end = text.size();
        std::string line = text.substr(start, end - start);
        start = end + 1;
        ++line_no;
        while (!line.empty() && (line.back() == '\r' || line.back() == ' ')) line.pop_back();
        if (line.empty()) continue;
        detail::Cursor c{line, 0, line_no};
        if (c.eat("param ")) {
            Param p;
            p.path = c.path();
            c.expect(":");
            p.ty = c.type();
            c.expect("=");
            std::string init = c.word();
            if (init == "xavier_uniform") p.init = Init::XavierUniform;
            else if (init == "zeros") p.init = Init::Zeros;
            else if (init == "ones") p.init = Init::Ones;
            else c.fail("unknown initializer `" + init + "`");
            program.params.push_back(p);
            continue;
        }
        if (c.eat("optimizer sgd")) {
            c.expect("lr");
            c.expect("=");
            program.optimizer.rule = Rule::Sgd;
            program.optimizer.lr = c.f32();
            continue;
        }
        if (c.eat("optimizer adamw")) {
            OptimizerInfo& o = program.optimizer;
            o.rule = Rule::AdamW;
            c.expect("lr"); c.expect("="); o.lr = c.f32();
            c.expect("weight_decay"); c.expect("="); o.weight_decay = c.f32();
            c.expect("beta1"); c.expect("="); o.beta1 = c.f32();
            c.expect("beta2"); c.expect("="); o.beta2 = c.f32();
            c.expect("eps"); c.expect("="); o.eps = c.f32();
            c.expect("warmup_steps"); c.expect("="); o.warmup_steps = c.number();
            continue;
        }
        if (c.eat("optimizer muon"))
            c.fail("the muon optimizer has no CUDA kernel");
        if (c.eat("output ")) {
            Output o;
            o.value = c.value();
            if (c.eat("loss")) o.role = Role::Loss;
            else if (c.eat("gradient")) o.role = Role::Gradient;
            else if (c.eat("update")) o.role = Role::Update;
            else if (c.eat("moment")) {
                o.role = Role::Moment;
                std::string m = c.word();
                if (m != "m" && m != "v") c.fail("unknown moment `" + m + "`");
                o.moment = m[0];
            }
            if (o.role == Role::Gradient || o.role == Role::Update || o.role == Role::Moment) {
                std::string path = c.path();
                int at = program.param_index(path);
                if (at < 0) c.fail("unknown parameter @" + path);
                o.param = static_cast<uint32_t>(at);
            }
            program.outputs.push_back(o);
            continue;
        }
        Node n;
        for (Tag t : {Tag::Forward, Tag::Loss, Tag::Gradient, Tag::Optimizer}) {
            if (c.eat(std::string(tag_name(t)) + " %")) {
                n.tag = t;
                program.tagged = true;
                c.at -= 1;
                break;
            }
        }
        n.id = c.value();
        c.expect(":");
        n.ty = c.type();
        c.expect("=");
        std::string opname = c.word();
        if (!op_from_name(opname, &n.op)) c.fail("no CUDA kernel for the op `" + opname + "`");
        switch (n.op) {
            case Op::Input: {
                c.expect("\"");
                size_t close = line.find('"', c.at);
                if (close == std::string::npos) c.fail("unterminated input name");
                n.name = line.substr(c.at, close - c.at);
                c.at = close + 1;
                break;
            }
            case Op::ParamRead: {
                std::string path = c.path();
                int at = program.param_index(path);
                if (at < 0) c.fail("unknown parameter @" + path);
                n.param = static_cast<uint32_t>(at);
                break;
            }
            case Op::Scalar: n.scalar = c.f32(); break;
            case Op::BroadcastScalar: n.bshape = c.dims(); break;
            case Op::EmbeddingGrad:
                c.expect("[");
                n.rows = c.number();
                c.expect("]");
                break;
            case Op::Attention:
            case Op::AttentionGradQ:
            case Op::AttentionGradK:
            case Op::AttentionGradV:
                c.expect("[");
                c.expect("heads");
                c.expect("=");
                n.heads = c.number();
                c.expect("]");
                break;
            case Op::Dropout:
            case Op::DropoutGrad: {
                c.expect("[");
                c.expect("p");
                c.expect("=");
                n.p = c.f32();
                c.expect(",");
                c.expect("site");
                c.expect("=");
                size_t close = line.find(']', c.at);
                if (close == std::string::npos) c.fail("unterminated dropout site");
                c.at = close + 1;
                break;
            }
            default: break;
        }
        while (!c.done()) {
            if (line[c.at] == '{') {
                if (!n.effect.empty()) n.effect += " ";
                size_t close = line.find('}', c.at);
                if (close == std::string::npos) c.fail("unterminated effect");
                n.effect += line.substr(c.at, close - c.at + 1);
                c.at = close + 1;
                continue;
            }
            n.operands.push_back(c.value());
            c.eat(",");
        }
        program.nodes.push_back(std::move(n));
    }
    program.refresh_inputs();
    return program;
}

}  // namespace msx
