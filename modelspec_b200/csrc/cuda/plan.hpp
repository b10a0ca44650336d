// The execution plan of one Tensor IR program on one GPU: which kernel runs for which nodes, in
// what order, and where every value lives.
//
// This is the CUDA counterpart of the reference's scheduler
// (crates/modelspec-core/src/schedule.rs:412-678 fusions, :759-1484 schedule_with) with two
// differences the reference names as open work: values share storage by liveness (the reference
// gives every stored value its own buffer, schedule.rs:97-104), and the optimizer is one launch
// over all parameters (the reference dispatches once per parameter, ir/kernel.rs:869-894).
//
// Fusions made here, each leaving the arithmetic of every element unchanged:
//   * rank-0 constant expressions are folded on the host (one rounded f32 op each, as on device);
//   * a Transpose read only by matmuls is folded into their operand flags; a Transpose of a
//     matmul's result swaps and flips the matmul's operands instead (same products, same order);
//   * the three attention gradient ops of one attention share one statistics pass;
//   * LayerNormGradGamma and the SumRows of the same adjoint (the beta gradient) are one launch;
//   * the SGD / AdamW update subgraph of every parameter is one multi-tensor launch, in place;
//   * nodes no output depends on (the ungathered head beside a masked-row gather) are not run.
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
        View       // a Transpose folded away: reads its source with the transposed flag flipped
    } kind = Dead;
    uint64_t bytes = 0;
    uint32_t pitch = 0;        // elements between rows as stored; 0 = the row width
    uint64_t offset = 0;       // Arena, Input: byte offset; Const: index into the constant table
    uint32_t index = 0;        // Param, Moment: parameter index; View: position of the source
    char moment = 0;           // Moment: 'm' or 'v'
    float constant = 0.0f;     // Const
    int first = -1, last = -1; // launches that define and last read an Arena value
    bool keep = false;         // an output: never reused
};

struct Launch {
    std::string kernel;
    uint32_t value = 0;                  // id of the node this launch is scheduled for
    std::vector<uint32_t> reads, writes; // slot positions (nodes first, then scratch slots)
    uint64_t flop = 0;
    std::function<void(cudaStream_t)> run;
};

}  // namespace msx
