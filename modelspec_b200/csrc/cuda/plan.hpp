// The execution plan of one Tensor IR program on one GPU: which kernel runs for which nodes, in
// what order, and where every value lives.
//
// This is the CUDA counterpart of the reference's scheduler
// (crates/modelspec-core/src/schedule.rs:412-678 fusions, :759-1484 schedule_with) with two
// differences the reference names as open work: values share storage by liveness (the reference
// gives every stored value its own buffer, schedule.rs:97-104), and the optimizer is one launch
// over all parameters (the reference dispatches once per parameter, ir/kernel.rs:869-894).
//
// Fusions made here. Those marked (=) leave the arithmetic of every element unchanged; the others
// change only the order in which a sum's terms are added (deterministic, tolerance class):
//   * (=) rank-0 constant expressions are folded on the host (one rounded f32 op each, as on device);
//   * (=) a Transpose read only by matmuls is folded into their operand flags; a Transpose of a
//     matmul's result swaps and flips the matmul's operands instead (same products, same order);
//   * (=) add_rows(matmul(x, w), b): the bias is added in the matmul's epilogue;
//   * (=) up to four matmuls of one shape and storage form whose operands exist (the Q, K, V
//     projections of a layer, their input gradients) are one launch;
//   * gradient-tagged matmuls whose result only the optimizer reads (weight gradients) wait for
//     the end of the backward pass and run as jobs of one launch per storage form (their k split
//     left as partial tiles for the finalize launch);
//   * (=) residual + dropout(x) followed by the layer norm of the sum is one launch;
//   * (=) a chain of Adds that only the gradients of one layer norm read is added as that launch
//     loads its adjoint;
//   * (=) other + embedding_grad(...): the scatter adds `other` as it writes;
//   * the attention forward keeps its probabilities for the backward of the same attention, and
//     the three attention gradient ops are one launch group;
//   * cross_entropy and cross_entropy_grad of the same logits are one launch;
//   * LayerNormGradX, LayerNormGradGamma and the SumRows of the same adjoint are one launch;
//   * column sums, layer-norm parameter gradients and split-k weight gradients that only the
//     optimizer reads leave chunk partials; one launch per step adds them all, and the first
//     stages of the small column sums share one launch too;
//   * (=) the SGD / AdamW update subgraph of every parameter is one multi-tensor launch, in place;
//   * (=) nodes no output depends on (the ungathered head beside a masked-row gather) are not run.
// A heavy launch whose result is first read many launches later (the weight gradient of the tied
// table, the 30,522-wide bias gradient) runs on a side stream beside the small launches between
// it and its first reader; what it reads and writes stays allocated until that reader.
// A matrix whose width is not a multiple of 4 floats and that only pitch-aware kernels touch is
// stored with padded rows (Slot::pitch).
#pragma once

#include <functional>
#include <string>
#include <vector>

#include "../core/ir.hpp"

namespace msx {

struct Slot {
    enum Kind : uint8_t {
        Dead,      // not computed
        Arena,     // an intermediate in the shared arena
        Param,     // a parameter buffer (ParamRead, and an update written in place)
        Moment,    // an AdamW moment buffer (its input and its next value)
        Input,     // a host input in the upload region
        Const,     // a folded rank-0 constant in the constant table
        View       // stored as another value: a Transpose folded away (read with the transposed flag
                   // flipped), or an addend that the launch which adds to it updates in place
    } kind = Dead;
    uint64_t bytes = 0;
    uint32_t pitch = 0;        // elements between rows as stored; 0 = the row width
    bool half = false;         // stored as bf16 (a mixed-precision plan's activations), else 4-byte elements
    uint64_t offset = 0;       // Arena, Input: byte offset; Const: index into the constant table
    uint32_t index = 0;        // Param, Moment: parameter index; View: position of the source
    char moment = 0;           // Moment: 'm' or 'v'
    float constant = 0.0f;     // Const
    int first = -1, last = -1; // launches that define and last read an Arena value
    int last_write = -1;       // the last launch that writes it (a value updated in place has two)
    bool keep = false;         // an output: never reused
};

struct Launch {
    std::string kernel;
    uint32_t value = 0;                  // id of the node this launch is scheduled for
    std::vector<uint32_t> reads, writes; // slot positions (nodes first, then scratch slots)
    uint64_t flop = 0;
    // >= 0: the launch runs on the plan's side stream from its place in the list, beside the
    // launches that follow it, and the launch with this index is the first to wait for it.
    int join_before = -1;
    // A side launch that writes outputs (gradients): a data-parallel bucket that holds them waits
    // for it before it is reduced.
    bool side_writes_outputs = false;
    std::function<void(cudaStream_t)> run;
};

}  // namespace msx
