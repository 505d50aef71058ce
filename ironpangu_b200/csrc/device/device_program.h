// Native device executor of a compiled bundle: the program-engine contract on a GPU, with no Python in the process.
//
//   DeviceProgram     one rank of a bundle on one GPU (this build: bundles compiled for tp = 1): parses device-program.json,
//                     re-checks the bundle's contracts, loads the rank's parameters by executing its init plan through a
//                     bounded pinned staging buffer (init::execute over CudaMemory), places every instruction result at the
//                     compiler's offset inside ONE device block (the frozen arena + workspace, fingerprint and row count checked),
//                     keeps the latent KV pages per resident sequence slot beside it, dispatches instructions to the kernel
//                     library's C entry points - the group {q_b linear, cache write, absorb, attention} as the one-launch
//                     cluster-per-head kernel for steps of one or two rows and short contexts, the grouped-query group as a packed
//                     projection + rotate-and-append + attention, hyper-connections / token convolutions / sink rows of the
//                     hyper-connected programs - and replays one CUDA graph per step width after the first eager run of that width
//   make_device_program_engine
//                     the same executor as a server engine (`ifab-server --program BUNDLE CHECKPOINT --gpus 1`): packed steps
//                     of prompt slices and decode rows in launch groups of up to eight rows, greedy tokens
//   ifab_device_program_*  C ABI over DeviceProgram (open / info / step / reset / close / error), for hosts that are not C++
//
// After `ready()` a step allocates nothing: control inputs travel through one pinned block, tokens come back through another.
// Reference: native/src/program_engine.cpp:86-258 (rank workers over a bundle), native/src/token_dispatch.inc:19-294 (dispatch),
// native/src/prepared_execution.h:189-239 (arena), native/include/program_engine.h (the contract).
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "../core/serve.h"

namespace ifab::device {

struct Options {
  int device = 0;
  uint32_t residents = 0;        // 0 = the bundle's resident_sequences
  uint32_t context = 0;          // 0 = the bundle's max_context (a smaller value only shrinks the KV pages)
  size_t staging_bytes = 64 << 20;
  bool graphs = true;
  int fused_head = -1;           // -1: by context (<= 2048 keys), 0 / 1: forced
};

class DeviceProgram {
 public:
  DeviceProgram(const std::string& bundle_dir, const std::string& checkpoint_dir, const Options& opt = {});
  ~DeviceProgram();
  DeviceProgram(const DeviceProgram&) = delete;
  DeviceProgram& operator=(const DeviceProgram&) = delete;

  uint32_t context() const;
  uint32_t vocab() const;
  uint32_t eos() const;
  uint32_t residents() const;
  uint32_t max_rows() const;       // query rows per launch group (what the arena was planned for, at most 8)
  const std::string& name() const;

  // One launch group: `rows` (<= max_rows) query rows with their positions and resident slots -> the greedy next token of
  // every row. Rows of one sequence must be in position order. Throws Backend when a kernel reports through the status word.
  void run_rows(const int32_t* tokens, const int32_t* positions, const int32_t* slots, int rows, int32_t* next_tokens);
  void reset();                    // every KV page back to zero
  Json audit() const;              // launches, graph widths, arena, bytes moved each way, allocations after readiness

 private:
  struct Impl;
  std::unique_ptr<Impl> p_;
};

std::shared_ptr<serve::ResidentEngine> make_device_program_engine(const std::string& bundle, const std::string& checkpoint, const Options& opt);

}  // namespace ifab::device

extern "C" {
const char* ifab_device_program_error(void);
int ifab_device_program_open(const char* bundle, const char* checkpoint, int device, uint32_t residents, void** out);
int ifab_device_program_info(void* engine, uint32_t* context, uint32_t* vocabulary, uint32_t* eos, uint32_t* residents, uint32_t* max_rows);
int ifab_device_program_rows(void* engine, const int32_t* tokens, const int32_t* positions, const int32_t* slots, uint32_t rows, int32_t* next_tokens);
int ifab_device_program_reset(void* engine);
int ifab_device_program_audit(void* engine, char* out_json, uint64_t capacity);
int ifab_device_program_close(void* engine);
/* a heap-allocated std::shared_ptr<ifab::serve::ResidentEngine>* (the caller moves from it and deletes it), or NULL */
void* ifab_device_program_engine_new(const char* bundle, const char* checkpoint, int device, uint32_t residents, uint32_t context);
}
