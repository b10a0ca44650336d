// The operator registry: operand counts and result types of every Tensor IR op, and a builder
// that types each node it appends through it.
//
// Follows the reference's registry (crates/modelspec-core/src/ops.rs:260-297 arity, :334-572
// shape inference, :610-658 attention shapes) for the ops of the BERT operator set.
#pragma once

#include "ir.hpp"

namespace msx {

inline std::string op_error(Op op, const std::string& what) {
    return std::string(op_name(op)) + ": " + what;
}

// The result type of `node.op` over operands of types `in`. `node` carries the op's attributes.
inline Type infer(const Node& node, const std::vector<const Type*>& in) {
    Op op = node.op;
    auto need = [&](size_t n) {
        if (in.size() != n)
            throw Error(op_error(op, "takes " + std::to_string(n) + " operands, got " +
                                         std::to_string(in.size())));
    };
    auto f32 = [&](size_t i) {
        if (in[i]->i32) throw Error(op_error(op, "operand " + std::to_string(i) + " is i32"));
    };
    auto ids = [&](size_t i) {
        if (!in[i]->i32) throw Error(op_error(op, "operand " + std::to_string(i) + " is not i32"));
    };
    auto rank = [&](size_t i, size_t r) {
        if (in[i]->rank() != r)
            throw Error(op_error(op, "operand " + std::to_string(i) + " is " + in[i]->str() +
                                         ", not rank " + std::to_string(r)));
    };
    auto same = [&](size_t i, size_t j) {
        if (*in[i] != *in[j])
            throw Error(op_error(op, in[i]->str() + " against " + in[j]->str()));
    };
    auto row_of = [&](size_t x, size_t r) {
        f32(r);
        rank(r, 1);
        if (in[r]->shape[0] != in[x]->shape[1])
            throw Error(op_error(op, in[x]->str() + " against row " + in[r]->str()));
    };
    switch (op) {
        case Op::Input:
        case Op::ParamRead: need(0); return node.ty;
        case Op::Scalar: need(0); return Type::f32({});
        case Op::Add:
        case Op::Sub:
        case Op::Mul:
        case Op::Div:
            need(2); f32(0); f32(1);
            if (in[0]->shape == in[1]->shape) return *in[0];
            if (in[1]->rank() == 0) return *in[0];
            if (in[0]->rank() == 0) return *in[1];
            throw Error(op_error(op, in[0]->str() + " against " + in[1]->str()));
        case Op::MatMul:
            need(2); f32(0); f32(1); rank(0, 2); rank(1, 2);
            if (in[0]->shape[1] != in[1]->shape[0])
                throw Error(op_error(op, in[0]->str() + " x " + in[1]->str()));
            return Type::f32({in[0]->shape[0], in[1]->shape[1]});
        case Op::Relu:
        case Op::Gelu:
        case Op::StopGradient:
        case Op::Sqrt: need(1); f32(0); return *in[0];
        case Op::Transpose:
            need(1); f32(0); rank(0, 2);
            return Type::f32({in[0]->shape[1], in[0]->shape[0]});
        case Op::ReduceSum:
        case Op::ReduceMean: need(1); f32(0); return Type::f32({});
        case Op::Mse: need(2); f32(0); same(0, 1); return Type::f32({});
        case Op::ReluGrad:
        case Op::GeluGrad: need(2); f32(0); same(0, 1); return *in[0];
        case Op::BroadcastScalar: need(1); f32(0); rank(0, 0); return Type::f32(node.bshape);
        case Op::Embedding:
            need(2); f32(0); rank(0, 2); ids(1); rank(1, 1);
            return Type::f32({in[1]->shape[0], in[0]->shape[1]});
        case Op::EmbeddingGrad:
            need(2); ids(0); rank(0, 1); f32(1); rank(1, 2);
            if (in[0]->shape[0] != in[1]->shape[0])
                throw Error(op_error(op, in[0]->str() + " against " + in[1]->str()));
            return Type::f32({node.rows, in[1]->shape[1]});
        case Op::AddRows: need(2); f32(0); rank(0, 2); row_of(0, 1); return *in[0];
        case Op::SumRows: need(1); f32(0); rank(0, 2); return Type::f32({in[0]->shape[1]});
        case Op::LayerNorm:
            need(3); f32(0); rank(0, 2); row_of(0, 1); row_of(0, 2); return *in[0];
        case Op::LayerNormGradX:
            need(3); f32(0); rank(0, 2); row_of(0, 1); same(0, 2); return *in[0];
        case Op::LayerNormGradGamma:
            need(2); f32(0); rank(0, 2); same(0, 1); return Type::f32({in[0]->shape[1]});
        case Op::Softmax: need(1); f32(0); rank(0, 2); return *in[0];
        case Op::SoftmaxGrad: need(2); f32(0); rank(0, 2); same(0, 1); return *in[0];
        case Op::Attention:
        case Op::AttentionGradQ:
        case Op::AttentionGradK:
        case Op::AttentionGradV: {
            need(op == Op::Attention ? 4 : 5);
            f32(0); f32(1); f32(2); f32(3);
            rank(0, 2); rank(1, 2); rank(2, 2); rank(3, 2);
            same(1, 2);
            uint64_t h = in[0]->shape[1];
            uint64_t b = in[3]->shape[0], s = in[3]->shape[1];
            if (in[1]->shape[1] != h || node.heads == 0 || h % node.heads != 0)
                throw Error(op_error(op, "heads do not divide the width of " + in[0]->str()));
            if (b == 0 || in[1]->shape[0] != b * s || in[0]->shape[0] % b != 0)
                throw Error(op_error(op, "key mask " + in[3]->str() + " against keys " +
                                             in[1]->str()));
            uint64_t l = in[0]->shape[0] / b;
            if (l < 1 || l > s) throw Error(op_error(op, "query rows per sequence out of range"));
            if (op != Op::Attention) same(0, 4);
            return op == Op::AttentionGradQ || op == Op::Attention ? *in[0] : *in[1];
        }
        case Op::CrossEntropy:
        case Op::CrossEntropyGrad: {
            need(op == Op::CrossEntropy ? 3 : 4);
            f32(0); rank(0, 2); ids(1); rank(1, 1); f32(2); rank(2, 1);
            if (in[1]->shape[0] != in[0]->shape[0] || in[2]->shape[0] != in[0]->shape[0])
                throw Error(op_error(op, "labels or weights against " + in[0]->str()));
            if (op == Op::CrossEntropy) return Type::f32({});
            f32(3); rank(3, 0);
            return *in[0];
        }
        case Op::Dropout:
            need(2); f32(0); ids(1);
            if (in[1]->shape != std::vector<uint64_t>{2}) throw Error(op_error(op, "token is not i32[2]"));
            return *in[0];
        case Op::DropoutGrad:
            need(2); ids(0); f32(1);
            if (in[0]->shape != std::vector<uint64_t>{2}) throw Error(op_error(op, "token is not i32[2]"));
            return *in[1];
        default: break;
    }
    throw Error(op_error(op, "not in the registry"));
}

// Appends typed nodes to a program, ids counting up from the program's largest.
struct Builder {
    Program program;
    uint32_t next = 0;
    Tag tag = Tag::None;

    explicit Builder(Program p = {}) : program(std::move(p)), next(program.next_id()) {}

    const Type& type_of(uint32_t v) const { return program.node(v).ty; }

    uint32_t push(Node n) {
        std::vector<const Type*> in;
        for (uint32_t o : n.operands) in.push_back(&type_of(o));
        n.ty = infer(n, in);
        n.id = next++;
        if (n.tag == Tag::None) n.tag = tag;
        program.nodes.push_back(std::move(n));
        if (program.nodes.back().op == Op::Input) program.inputs.push_back(program.nodes.back().id);
        return program.nodes.back().id;
    }
    uint32_t op(Op o, std::vector<uint32_t> operands) {
        Node n;
        n.op = o;
        n.operands = std::move(operands);
        return push(std::move(n));
    }
    uint32_t input(const std::string& name, Type ty) {
        Node n;
        n.op = Op::Input;
        n.name = name;
        n.ty = std::move(ty);
        return push(std::move(n));
    }
    uint32_t param_read(uint32_t param) {
        Node n;
        n.op = Op::ParamRead;
        n.param = param;
        n.ty = program.params.at(param).ty;
        return push(std::move(n));
    }
    uint32_t scalar(float v) {
        Node n;
        n.op = Op::Scalar;
        n.scalar = v;
        return push(std::move(n));
    }
};

}  // namespace msx
