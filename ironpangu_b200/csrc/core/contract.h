// Engine-side re-validation of a serialized token program and its initialization plans.
//
// The compiler checks what it emits; an engine must not trust a file. Before any device memory is allocated the
// decoded program is checked again, independently of the lowering code: every instruction names an operation the kernel
// library implements and one of the entry points registered for it, the kinds of its inputs and of its result fit the
// operation, the attributes the kernel reads are present and within limits, views stay inside their input, and the
// fused all-reduce operations do not alias the buffers they read from other instructions. `validate_bindings` then checks
// the program against one rank's initialization plan: every weight attribute resolves to a parameter of the plan whose
// dimensions fit the instruction, and the plan carries no parameter the program never reads.
// Reference: native/include/ascend_token_contract.h:36-557 (validate_kernels, validate_bindings).
#pragma once
#include "initplan.h"
#include "program.h"

namespace ifab::contract {

// throws Error(Invalid) naming the instruction and the violated rule
void validate_kernels(const program::Program& p);
void validate_bindings(const program::Program& p, const init::Plan& plan);

// both checks over a bundle directory (execution.bin + every rank-N.bin found); returns a JSON summary
Json validate_bundle(const std::string& dir);

}  // namespace ifab::contract
