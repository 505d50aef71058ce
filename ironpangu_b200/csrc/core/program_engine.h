/* Program engine C ABI, version 1: one engine = one compiled bundle + its checkpoint, a fixed number of resident sequence
 * slots, token-in / token-out. No activation crosses the boundary; calls on one handle are serialised by the caller.
 * The function set mirrors the reference's (native/include/program_engine.h) under the `ifab_program_` prefix, so a
 * front end written against that contract ports by renaming.
 *
 * This build of the ABI executes the bundle's logical program on the host with the CPU interpreter (all tensor-parallel
 * ranks simulated, same bf16 rounding points as the device plan): it is the portable reference executor and what the
 * server's `--program ... --cpu` mode runs. Device execution goes through the engine worker protocol instead
 * (runtime/engine_worker.py), which needs no C ABI because it is another process.
 *
 * Every function returns 0 on success and a non-zero code on failure; ifab_program_error() then describes the last
 * failure of the calling thread. */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

uint32_t ifab_program_abi_version(void);
/* preparation = 1 is an offline qualification mode: the engine opens but refuses generation calls. */
int ifab_program_open(const char* bundle, const char* checkpoint, uint32_t preparation, void** out);
int ifab_program_close(void* engine);
const char* ifab_program_error(void);

int ifab_program_info(void* engine, uint32_t* context, uint32_t* vocabulary, uint32_t* eos);
int ifab_program_reset(void* engine);                                   /* all residents back to position 0 */
int ifab_program_resident_capacity(void* engine, uint32_t* count);
int ifab_program_select_resident(void* engine, uint32_t slot);          /* the slot `token` / `prefill` act on */
int ifab_program_reset_resident(void* engine, uint32_t slot);
/* Complete-state copy: `source` must stand exactly at `boundary`, `destination` must be reset. */
int ifab_program_copy_resident(void* engine, uint32_t source, uint32_t destination, uint32_t boundary);
/* Page bindings are metadata of the device executors; here they are validated (non-negative, unique) and recorded. */
int ifab_program_bind_pages(void* engine, uint32_t rank, const char* component, const int32_t* pages, uint32_t count);
int ifab_program_bind_state(void* engine, uint32_t rank, uint32_t logical_node, const int32_t* pages, uint32_t count);
int ifab_program_shared_pages(void* engine, uint32_t* enabled);

int ifab_program_token(void* engine, uint32_t token, uint32_t position, uint32_t sample, uint32_t* output);
int ifab_program_prefill_capacity(void* engine, uint32_t* count);
int ifab_program_prefill_mode(void* engine, uint32_t* mode);            /* 1: any query length up to the capacity */
int ifab_program_prefill_variants(void* engine, uint32_t* mask);
int ifab_program_prefill_sizes(void* engine, uint32_t* sizes, uint32_t capacity, uint32_t* count);
int ifab_program_prefill(void* engine, const uint32_t* tokens, uint32_t count, uint32_t position, uint32_t sample, uint32_t* output);

typedef struct IfabProgramSequenceV1 {
  uint32_t resident, position, token_count, sample;
} IfabProgramSequenceV1;
/* Packed batch: tokens concatenate in sequence order; one output per sample = 1 member, in sequence order. */
int ifab_program_batch(void* engine, const IfabProgramSequenceV1* sequences, uint32_t sequence_count, const uint32_t* tokens,
                       uint32_t token_count, uint32_t* outputs, uint32_t output_capacity, uint32_t* output_count);
int ifab_program_batch_capacity(void* engine, uint32_t* capacity);

#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
#include <memory>

#include "serve.h"

namespace ifab::serve {
/* The same executor as a server engine: `ifab-server --program BUNDLE CHECKPOINT --cpu`. */
std::shared_ptr<ResidentEngine> make_cpu_program_engine(const std::string& bundle, const std::string& checkpoint, uint32_t residents,
                                                        uint32_t context);
}  // namespace ifab::serve
#endif
