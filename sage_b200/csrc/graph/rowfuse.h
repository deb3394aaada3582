// Whole-row programs: a graph of maps, row reductions, gathers and scatters along the row, all over one
// [R, C] space, evaluated by ONE generated kernel that keeps each row on chip.
//
// The reference runs such a graph (e.g. softmax_cross_entropy of a fused map and its gradient,
// examples/basics.rs:28-36, src/ops/nn.rs:58-82) as one kernel per map chain / reduction / gather /
// scatter, each reading and writing full [R, C] tensors (Program::compile, src/session.rs:62-206,
// decides which values are materialised).  Here every value of the graph lives in registers for the
// row being processed: a block loads the row of each input once, walks the graph in topological
// order (block reductions where the graph reduces along the row), and writes only the requested
// outputs.  DRAM traffic is the compulsory one: inputs once, outputs once.
#pragma once
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "graph.h"

namespace sage {

struct RowProgram;

// Null when the graph below `targets` (cut at `evaluated` and at data variables) is not a row program.
// `whole_program`: the targets are a whole evaluation; then a graph of maps alone is left to the
// ordinary map kernels (they already run at the HBM peak).  Without it (a region inside a larger
// program) maps alone qualify.  `emit_source` false: analysis only, the result cannot be run.
std::shared_ptr<RowProgram> row_program_build(const std::vector<Var> &evaluated, const std::vector<Var> &targets, bool whole_program = true,
                                              bool emit_source = true);
// Allocates the targets, launches the kernel, stores the results in `s.data`.
sage_status row_program_exec(RowProgram &p, Context &ctx, Session &s);
// The same with the caller's own lookup of the (non-data) inputs; `outs` are the targets in order.
// `planes` (optional, one flag per target): also write the tf32 hi / lo planes of that (f32, full-size) target.
sage_status row_program_run(RowProgram &p, Context &ctx, const std::function<bool(const Var &, Tensor *)> &fetch, std::vector<Tensor> *outs,
                            const std::vector<char> *planes = nullptr);
void row_program_space(const RowProgram &p, long long *rows, long long *cols);
std::vector<Var> row_program_inputs(const RowProgram &p);
int row_program_exchanges(const RowProgram &p);  // reductions + gathers + scatters in the program
// Are the evaluated values the program was cut at still held by the session?
bool row_program_ready(const RowProgram &p, const Session &s);
std::string row_program_describe(const RowProgram &p);
// The generated CUDA source (for tests).
const std::string &row_program_source(const RowProgram &p);

}  // namespace sage
