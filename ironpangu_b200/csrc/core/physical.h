// Backend-neutral physical inspection plan: which implementation candidate runs every operation of a graph, why, what it
// is allowed to touch, and what it is expected to cost - with the plan re-derivable from itself (`verify`).
//
// An Operation carries one or more Candidates. A candidate states where it runs (only device-resident candidates are
// admitted: a host or opaque implementation, or one with a host<->device copy among its boundaries, is refused BEFORE any
// cost is looked at), its numerical contract (all legal candidates of an operation must share it), whether it is eligible
// (an ineligible one says why), its workspace bound (absent = unresolved, never zero) and a Cost with provenance. `choose`
// picks the cheapest eligible candidate by its conservative bound when every legal candidate has a complete cost, and the
// stable lowest id otherwise - an unknown cost is never treated as zero. `serial_plan` lays the operations out in order on
// stream 0 with one value per operation, lifetimes from first definition to last use, no arena reuse claimed; `verify`
// recomputes selections, dependencies, lifetimes, payload sizes, the collective sequence and the cost summary.
// Reference: crates/inferfabric-plan/src/physical.rs:9-457.
#pragma once
#include <optional>

#include "base.h"

namespace ifab::physical {

constexpr const char* kFormat = "inferfabric.physical.v1";
constexpr const char* kPolicy = "serial-device-resident-v1";

enum class CostSource { Unknown, Analytical, Measured, Interpolated };
struct Cost {
  CostSource source = CostSource::Unknown;
  std::optional<uint64_t> estimate_ns, upper_ns;
  std::string evidence;           // sample identity or model revision; empty only for Unknown
};
enum class Location { Host, Device, Opaque };
enum class BoundaryKind {
  HostToDevice, DeviceToHost, ControlUpload, ParameterUpload, ParameterReadback, RequestOutput, Synchronize, DynamicAllocation,
  InternalLaunches, PersistentState
};
struct Boundary {
  BoundaryKind kind;
  std::string detail;
};
struct Candidate {
  std::string id, contract_revision, numerical_contract;
  Location location = Location::Device;
  bool eligible = true;
  std::string rejection;                          // why not, when ineligible
  std::optional<uint64_t> workspace_bound_bytes;  // absent = unresolved
  bool capture_qualified = false;
  std::vector<Boundary> boundaries;
  std::vector<std::string> unresolved;
  Cost cost;
};
struct Value {
  size_t logical_node = 0;
  std::string dtype;                              // empty = not known
  std::vector<uint64_t> shape;
  std::string layout = "row_major";
  Location location = Location::Device;
  std::optional<uint64_t> payload_bytes, alignment, arena_offset;
  size_t first = 0, last = 0;                     // lifetime in steps
};
struct Collective {
  std::string group = "all_ranks", operation, dtype;
  uint64_t elements_per_rank = 0;
  size_t sequence = 0;
};
struct Operation {
  std::string name;
  std::vector<size_t> logical_nodes, inputs;
  std::vector<Candidate> candidates;
  std::optional<Collective> collective;
};
struct Step {
  size_t id = 0;
  Operation operation;
  size_t selected = 0;
  std::string selection_reason;
  size_t stream = 0;
  std::vector<size_t> data_dependencies, order_dependencies, reuse_dependencies;
};
struct Schedule {
  std::vector<Step> steps;
  std::vector<Value> values;
  std::vector<size_t> outputs;
  uint64_t known_host_payload_peak_bytes = 0;
  bool memory_complete = false, cost_complete = false;
  std::string activation_policy;
  std::optional<uint64_t> estimated_serial_ns;
};
struct Plan {
  std::string format = kFormat, name, target, logical_digest, policy = kPolicy;
  bool executable = false;
  std::vector<uint32_t> devices;                  // rank i runs on devices[i]; all ranks share the one schedule
  Schedule schedule;
  std::vector<std::string> limitations;
  Json to_json() const;
  static Plan from_json(const Json& j);
};

struct Choice {
  size_t index = 0;
  std::string reason;
};
Choice choose(const std::vector<Candidate>& candidates);
Plan serial_plan(std::string name, std::string target, std::string logical_digest, const std::vector<uint32_t>& devices,
                 std::vector<Operation> operations, std::vector<Value> values, std::vector<size_t> outputs);
void verify(const Plan& plan);

}  // namespace ifab::physical
