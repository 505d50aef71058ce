// Unit tests of the host runtime services (no device needed). Exit code 0 = all passed.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <unistd.h>
#include <functional>
#include <iostream>

#include "bundle.h"
#include "interp.h"
#include "chat_parse.h"
#include "contract.h"
#include "cpu_plan.h"
#include "device_buffer.h"
#include "physical.h"
#include "initplan.h"
#include "paging.h"
#include "prefix_index.h"
#include "rankplan.h"
#include "runtime.h"
#include "scheduler.h"
#include "state_pool.h"

using namespace ifab;

static int failures = 0, checks = 0;
#define CHECK(cond)                                                            \
  do {                                                                         \
    ++checks;                                                                  \
    if (!(cond)) {                                                             \
      ++failures;                                                              \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);              \
    }                                                                          \
  } while (0)
template <typename F>
static bool throws(F&& f, ErrorKind kind) {
  try {
    f();
  } catch (const Error& e) {
    return e.kind() == kind;
  } catch (...) {
    return false;
  }
  return false;
}
#define CHECK_THROWS(kind, expr) CHECK(throws([&] { expr; }, ErrorKind::kind))

static serving::Manifest manifest(bool sliding) {
  serving::Manifest m;
  m.identity = {"m", std::string(64, 'a'), "b200_token_v1", 2};
  m.max_context = 4096;
  m.vocab = 1000;
  m.eos = 1;
  m.resident_sequences = 4;
  m.max_batched_tokens = 64;
  serving::Variant d;
  d.name = "decode";
  d.numerics = "gemv";
  m.variants.push_back(d);
  serving::Variant p;
  p.name = "prefill_chunk";
  p.phase = serving::Phase::Prefill;
  p.max_query_tokens = 64;
  p.captured = false;
  p.numerics = "tc";
  m.variants.push_back(p);
  serving::State kv;
  kv.name = "kv16";
  kv.component = 0;
  kv.dtype = "bf16";
  kv.storage = {serving::Storage::Kind::Pages, 16, 1152, 0};
  if (sliding) kv.retention = {serving::Retention::Kind::SlidingWindow, 512};
  m.states.push_back(kv);
  serving::State slot;
  slot.name = "conv";
  slot.component = 1;
  slot.dtype = "bf16";
  slot.storage = {serving::Storage::Kind::Slot, 0, 0, 4096};
  m.states.push_back(slot);
  m.validate();
  return m;
}

static void test_state_pool() {
  using namespace runtime;
  auto m = manifest(false);
  std::map<StatePool::Key, uint32_t> cap;
  for (uint32_t r = 0; r < 2; ++r) {
    cap[{"kv16", r}] = 8;
    cap[{"conv", r}] = 2;
  }
  StatePool p(m, 7, 2, cap);
  auto baseline = p.usage();
  Lease a = p.reserve(7, 1, 32);
  CHECK(p.bindings(7, a).size() == 4);
  CHECK(p.page_address(7, a, "kv16", 1, 17).row == 1);
  CHECK(p.page_address(7, a, "kv16", 0, 17).byte_offset == (uint64_t)p.bindings(7, a)[0].units[1] * 16 * 1152 + 1152);
  CHECK_THROWS(Capacity, p.page_address(7, a, "kv16", 0, 32));
  CHECK_THROWS(Stale, p.reserve(8, 2, 16));
  Ticket t = p.submit(7, {a}, {});
  CHECK_THROWS(Invalid, p.seal(7, a));
  p.complete(7, t, 0);
  CHECK_THROWS(Invalid, p.seal(7, a));      // every rank must complete
  CHECK_THROWS(Invalid, p.complete(7, t, 0));
  p.complete(7, t, 1);
  SealedLease s = p.seal(7, a);
  CHECK_THROWS(Invalid, p.submit(7, {a}, {}));   // sealed = read-only
  Borrow pin = p.borrow_sealed(7, s);
  p.retire(7, a);
  Borrow reader = p.borrow_sealed(7, s);          // snapshot survives the owner's retirement
  Ticket restore = p.submit(7, {}, {reader});
  p.release(7, pin);
  p.release(7, reader);
  p.complete(7, restore, 1);
  bool occupied = false;
  for (auto& u : p.usage()) occupied |= u.occupied_units > 0;
  CHECK(occupied);                                 // still in flight on rank 0
  p.complete(7, restore, 0);
  CHECK(p.usage() == baseline);                    // deferred reclaim happened
  CHECK_THROWS(Stale, p.borrow_sealed(7, s));
  // all-or-nothing reservation
  Lease big = p.reserve(7, 3, 8 * 16);
  auto before = p.usage();
  CHECK_THROWS(Capacity, p.reserve(7, 4, 16));
  CHECK(p.usage() == before);
  p.retire(7, big);
  // slot pinning
  Lease s1 = p.reserve_at_slot(7, 5, 16, 1);
  for (auto& b : p.bindings(7, s1))
    if (b.component == "conv") CHECK(b.units[0] == 1);
  CHECK_THROWS(Capacity, p.reserve_at_slot(7, 6, 16, 1));
  p.poison();
  CHECK_THROWS(Backend, p.reserve(7, 9, 16));
  // sliding window ring
  auto ms = manifest(true);
  std::map<StatePool::Key, uint32_t> cap2;
  for (uint32_t r = 0; r < 2; ++r) {
    cap2[{"kv16", r}] = 80;
    cap2[{"conv", r}] = 2;
  }
  StatePool q(ms, 1, 2, cap2);
  Lease lg = q.reserve(1, 1, 4096);
  const auto& bs = q.bindings(1, lg);
  CHECK(bs[0].ring_tokens == 544 && bs[0].units.size() == 34);
  std::set<uint64_t> live;
  for (uint32_t pos = 2000; pos < 2000 + 512; ++pos) CHECK(live.insert(q.page_address(1, lg, "kv16", 0, pos).byte_offset).second);
  Lease sh = q.reserve(1, 2, 17);
  CHECK(q.bindings(1, sh)[0].units.size() == 2 && q.bindings(1, sh)[0].ring_tokens == 0);
}

static void test_prefix_index() {
  using namespace runtime;
  serving::PrefixIdentity id{"p", "w", "ns", "", 16};
  PrefixIndex ix(id, 4);
  std::vector<uint32_t> a{1, 2, 3, 4, 5, 6, 7, 8}, b{1, 2, 3, 4, 9, 9, 9, 9}, c{1, 2, 3, 4};
  CHECK(ix.insert(id, a, {1}));
  CHECK(ix.insert(id, b, {2}));
  CHECK(ix.insert(id, c, {3}));
  CHECK(!ix.insert(id, c, {4}));
  CHECK_THROWS(Invalid, ix.insert(id, {1, 2, 3}, {5}));
  CHECK(ix.size() == 3);
  auto m = ix.lookup(id, {1, 2, 3, 4, 5, 6, 7, 8, 10});
  CHECK(m && m->id.value == 1 && m->tokens == 8);
  m = ix.lookup(id, {1, 2, 3, 4, 5, 6, 7, 8});     // must leave one token to compute
  CHECK(m && m->id.value == 3 && m->tokens == 4);
  m = ix.lookup(id, {1, 2, 3, 4, 9, 9, 0});
  CHECK(m && m->id.value == 3);
  CHECK(!ix.lookup(id, {2, 2, 3, 4, 5}));
  serving::PrefixIdentity other = id;
  other.salt = "x";
  CHECK(!ix.lookup(other, {1, 2, 3, 4, 5, 6, 7, 8, 10}));
  CHECK(ix.remove({3}));
  CHECK(!ix.remove({3}));
  m = ix.lookup(id, {1, 2, 3, 4, 5, 6, 7, 8, 10});
  CHECK(m && m->id.value == 1);
  CHECK(ix.remove({1}) && ix.remove({2}) && ix.empty() && ix.token_units() == 0);
  // LRU cache
  PrefixCache cache(id, 4, 2);
  serving::ArithmeticHistory h4, h8;
  h4.append_completed(0, 4, "tc");
  h8.append_completed(0, 8, "tc");
  std::vector<SealedLease> ev;
  auto i1 = cache.publish(c, {1, 1}, h4, &ev);
  auto i2 = cache.publish(a, {2, 2}, h8, &ev);
  CHECK(i1 && i2 && ev.empty());
  const auto* hit = cache.restore({1, 2, 3, 4, 5, 6, 7, 8, 9});
  CHECK(hit && hit->tokens.size() == 8);
  auto i3 = cache.publish(b, {3, 3}, h8, &ev);       // evicts the LRU unpinned entry (prefix c)
  CHECK(i3 && ev.size() == 1 && ev[0].lease == 1);
  cache.unpin(hit->id);
  serving::ArithmeticHistory other_hist;
  other_hist.append_completed(0, 8, "gemv");
  CHECK(cache.restore({1, 2, 3, 4, 9, 9, 9, 9, 1}, &other_hist) == nullptr);   // different numerics: no reuse
  CHECK(cache.clear().size() == 2);
}

static void test_paging() {
  using namespace paging;
  auto sp = page_spans(14, 20, 16);
  CHECK(sp.size() == 3 && sp[0].page == 0 && sp[0].first_row == 14 && sp[0].rows == 2 && sp[1].rows == 16 && sp[2].rows == 2);
  ResidentPages rp({16, 1152, 8, 4}, 2);
  rp.bind(0, {5, 2, 7});       // permuted, non-contiguous pages
  rp.bind(1, {0, 1, 3});
  CHECK_THROWS(Invalid, rp.bind(1, {5}));
  CHECK(rp.row_offset(0, 17) == ((uint64_t)2 * 16 + 1) * 1152);
  auto t = rp.batch_table();
  CHECK(t.size() == 8 && t[0] == 5 && t[3] == -1 && t[4] == 0);
  auto cp = rp.copy_plan(0, 1, 40);
  CHECK(cp.size() == 3 && cp[2].bytes == 8 * 1152);
  CHECK_THROWS(Capacity, rp.copy_plan(0, 1, 64));
  rp.release(0);
  rp.append(0, 5);
  CHECK_THROWS(Invalid, rp.append(0, 0));
  auto b = SequenceBatch::make({{1, 10, 3, true}, {0, 0, 2, false}}, {7, 8, 9, 1, 2}, 8, 2, 64);
  CHECK(b.tokens.size() == 5 && b.positions[2] == 12 && b.slots[3] == 0 && b.sample_rows[0] == 2 && b.sample_rows[1] == -1);
  CHECK_THROWS(Invalid, SequenceBatch::make({{1, 0, 1, true}, {1, 1, 1, true}}, {1, 2}, 8, 2, 64));
  CHECK_THROWS(Capacity, SequenceBatch::make({{0, 62, 4, true}}, {1, 2, 3, 4}, 8, 2, 64));
  auto w = SlidingWindowLayout::make(65536, 512, 4, 16);
  CHECK(w.capacity == 544 && w.ring_row(544) == 0 && w.first_visible(1000) == 489);
  CHECK(w.append_is_safe(5000, 4) && w.append_is_safe(5000, 32) && !w.append_is_safe(5000, 64));
  BoundedBuffers bb(1024, 2);
  uint32_t x = bb.acquire(1000);
  bb.acquire(8);
  CHECK_THROWS(Capacity, bb.acquire(8));
  CHECK_THROWS(Capacity, BoundedBuffers(16, 1).acquire(32));
  bb.release(x);
  CHECK_THROWS(Invalid, bb.release(x));
}

static rankplan::Spec spec(uint32_t tp, uint32_t cp, bool sp) {
  rankplan::Spec s;
  s.model = {"hybrid", 2048, 6144, 248320, 8, 2, 256, 16, 128, 4, {rankplan::Layer::Delta, rankplan::Layer::Delta, rankplan::Layer::Delta, rankplan::Layer::Full}};
  s.prefill = {tp, cp, sp};
  s.decode = {tp, 1, false};
  s.page_tokens = 128;
  s.token_budget = 1024;
  s.batch_buckets = {1, 2, 4, 8};
  s.context_buckets = {128, 512, 2048, 8192};
  return s;
}

static void test_rankplan_and_runtime() {
  using namespace rankplan;
  using namespace runtime;
  Artifact a = compile(spec(2, 2, true));
  size_t n_prefill = 0, n_decode = 0;
  for (auto& p : a.plans) (p.role == Role::Prefill ? n_prefill : n_decode)++;
  CHECK(n_prefill == 4 && n_decode == 2 && a.buckets.size() == 16);
  auto count = [&](const RankPlan& p, CommKind k, const std::string& g) {
    size_t n = 0;
    for (auto& i : p.instructions) n += i.kind == Instruction::Kind::Communication && i.comm == k && i.group == g;
    return n;
  };
  const RankPlan& p0 = a.plans[0];
  CHECK(count(p0, CommKind::ReduceScatter, "tp") == 8 && count(p0, CommKind::AllReduce, "tp") == 0);   // SP: RS instead of AR
  CHECK(count(p0, CommKind::AllGather, "tp") == 8 + 1 + 1);
  CHECK(count(p0, CommKind::Send, "cp") == 1 + 3 && count(p0, CommKind::Receive, "cp") == 1);           // ring on the full layer; delta hand-off
  const RankPlan& dec = a.plans[4];
  CHECK(dec.role == Role::Decode && count(dec, CommKind::AllReduce, "tp") == 8 && count(dec, CommKind::Send, "cp") == 0);
  CHECK(dec.states.size() == 3 * 2 + 1);
  Artifact back = decode(encode(a));
  CHECK(back.key == a.key && back.plans.size() == a.plans.size());
  std::string bytes = encode(a);
  bytes[100] ^= 1;
  CHECK_THROWS(Stale, decode(bytes));
  auto bad = spec(2, 1, false);
  bad.decode.cp = 2;
  CHECK_THROWS(Invalid, bad.validate());
  bad = spec(1, 1, true);
  CHECK_THROWS(Invalid, bad.validate());
  bad = spec(2, 1, false);
  bad.batch_buckets = {4, 2};
  CHECK_THROWS(Invalid, bad.validate());
  // every start-up stage failure prevents readiness
  for (Stage st : {Stage::Validate, Stage::Compile, Stage::Prepare, Stage::Warmup, Stage::Capture, Stage::ValidateReplay, Stage::Reset, Stage::Ready}) {
    auto tr = std::make_shared<Trace>();
    Runtime rt(compile(spec(2, 1, false)), Role::Decode, 0, std::make_unique<MockBackend>(tr));
    CHECK_THROWS(Backend, rt.start("w", st));
    CHECK(rt.stage() == Stage::Failed && !rt.ready());
    CHECK_THROWS(Backend, rt.step({{1, {1}, 0}}));
  }
  auto tr = std::make_shared<Trace>();
  Runtime rt(compile(spec(2, 1, false)), Role::Decode, 1, std::make_unique<MockBackend>(tr, 1));
  rt.start("w");
  CHECK(rt.ready() && tr->count("capture") == 16);
  auto out = rt.step({{5, {3}, 100}, {6, {4}, 600}});
  CHECK(out.size() == 2 && out[0].token == MockBackend::token_for(5, 101, 248320));
  CHECK(tr->count("comm all_reduce tp") == 8);
  CHECK_THROWS(Capacity, rt.step({{5, {3}, 9000}}));
  rt.close();
  CHECK(rt.stage() == Stage::Closed);
  // thread-per-rank worker group: a failing rank fails the group for good
  std::atomic<int> ran{0};
  {
    WorkerGroup g(4, [&](uint32_t rank, uint64_t gen) {
      ++ran;
      if (gen == 2 && rank == 3) throw std::runtime_error("boom");
    });
    g.step();
    CHECK(ran == 4 && g.healthy());
    CHECK_THROWS(Backend, g.step());
    CHECK(!g.healthy() && g.failure().find("rank 3") != std::string::npos);
    CHECK_THROWS(Backend, g.step());
  }
  HealthGuard hg;
  hg.fail("first");
  hg.fail("second");
  CHECK(!hg.healthy() && hg.reason() == "first");
}

static void test_transfer() {
  using namespace runtime;
  InMemoryTransport t("key", 8, 2, 16);
  TransferLease l = t.reserve(1, 5, 40);
  CHECK(l.pages.size() == 3);
  TransferManifest m{1, 5, "key", 40, 77, {1, 2}, 0, 0};
  CHECK_THROWS(Invalid, t.commit(l));
  t.transfer(m);
  t.transfer(m);                                   // idempotent duplicate
  TransferManifest other = m;
  other.next_token = 78;
  CHECK_THROWS(Invalid, t.transfer(other));
  TransferManifest stale = m;
  stale.epoch = 4;
  CHECK_THROWS(Stale, t.transfer(stale));
  t.complete(l);
  CHECK(t.commit(l).next_token == 77 && t.commit(l).next_token == 77);
  CHECK_THROWS(Invalid, t.finish(l));
  t.acknowledge(l);
  t.acknowledge(l);
  t.finish(l);
  CHECK(t.pending() == 0 && t.pool().retired() == 3 && t.pool().free_pages() == 5);
  TransferLease old = l;
  CHECK_THROWS(Stale, t.complete(old));
  t.completion_fence();
  CHECK(t.pool().free_pages() == 8);
  TransferLease l2 = t.reserve(1, 5, 16);
  CHECK(l2.generation != l.generation);
  CHECK_THROWS(Stale, t.pool().check(l));
  TransferLease grown = t.pool().ensure(l2, 50);
  CHECK(grown.pages.size() == 4);
  CHECK_THROWS(NotImplemented, UnavailableTransport().poll(1));
}

static void test_scheduler() {
  using namespace sched;
  size_t cur = 0;
  auto pick = select_round({4, 4, 4, 4}, &cur, 10);
  CHECK(pick.size() == 2 && pick[0] == 0 && cur == 2);
  pick = select_round({4, 4, 4, 4}, &cur, 10);
  CHECK(pick[0] == 2 && pick[1] == 3 && cur == 0);
  LiveScheduler s({2, 8, 4, 64, 3, 100});
  s.submit({1, {1, 2, 3, 4, 5, 6}, 3, {99}});
  s.submit({2, {7, 8}, 2, {}});
  s.submit({3, {9}, 1, {}});
  CHECK_THROWS(Invalid, s.submit({3, {9}, 1, {}}));
  CHECK_THROWS(Invalid, s.submit({4, {1000}, 1, {}}));
  CHECK_THROWS(Capacity, s.submit({5, std::vector<uint32_t>(63, 1), 4, {}}));
  auto p = s.plan();                                 // seq1 chunk of 4, seq2 whole prompt (2)
  CHECK(p.batch.slices.size() == 2 && p.batch.slices[0].token_count == 4 && !p.batch.slices[0].sample && p.batch.slices[1].sample);
  CHECK(s.queued() == 1 && s.running() == 2);
  auto ev = s.commit(p, {0, 50});
  CHECK(ev.size() == 1 && ev[0].request == 2 && *ev[0].token == 50 && !ev[0].finish);
  p = s.plan();                                      // seq1 rest of prompt (2 rows), seq2 decode (service order rotates)
  CHECK(p.batch.tokens.size() == 3);
  std::vector<uint32_t> sampled;
  for (size_t k = 0; k < p.batch.slices.size(); ++k) {
    if (p.requests[k] == 1) CHECK(p.batch.slices[k].position == 4 && p.batch.slices[k].token_count == 2 && p.batch.slices[k].sample);
    sampled.push_back(p.requests[k] == 1 ? 60 : 51);
  }
  ev = s.commit(p, sampled);
  CHECK(ev.size() == 2);
  for (auto& e : ev) CHECK(e.request == 1 ? (!e.finish && *e.token == 60) : (e.finish && *e.finish == Finish::Length));
  p = s.plan();                                      // resident of seq2 is reused by request 3
  CHECK(p.released.size() == 1 && p.requests.size() == 2);
  s.set_backpressure(1, true);
  sampled.clear();
  for (auto r : p.requests) sampled.push_back(r == 1 ? 99 : 5);
  ev = s.commit(p, sampled);                         // seq1 hits its stop token
  bool stop_seen = false;
  for (auto& e : ev) stop_seen |= e.request == 1 && e.finish && *e.finish == Finish::Stop;
  CHECK(stop_seen);
  p = s.plan();
  CHECK(s.idle() || !p.empty());
  // cancellation while a step is in flight
  LiveScheduler c({1, 4, 4, 64, 4, 0});
  c.submit({9, {1, 2}, 5, {}});
  auto pc = c.plan();
  auto ce = c.cancel(9);
  CHECK(ce && *ce->finish == Finish::Cancelled && c.running() == 1);
  CHECK(c.commit(pc, {3}).empty() && c.running() == 0 && c.idle());
  c.submit({10, {1}, 2, {}});
  c.plan();
  CHECK(c.fail_all().size() == 1 && c.idle());
  // PD simulation over the mock runtime
  auto tr = std::make_shared<runtime::Trace>();
  auto rep = run_mock(rankplan::compile(spec(1, 1, false)), {{1, 300, 4, 0, std::nullopt}, {2, 2000, 3, 0, std::nullopt}, {3, 50, 5, 2, 4u}}, {4, 64, 128}, tr);
  CHECK(rep.completed == 2 && rep.cancelled == 1 && rep.transfers == 3 && rep.leaked_allocations == 0);
  CHECK(rep.outputs.at(1).size() == 4 && rep.prefill_steps >= 3);
  auto rep2 = run_mock(rankplan::compile(spec(1, 1, false)), {{1, 300, 4, 0, std::nullopt}, {2, 2000, 3, 0, std::nullopt}}, {4, 64, 128});
  CHECK(rep2.outputs.at(1) == rep.outputs.at(1));     // repeatable
}

static void test_cpu_plan() {
  using namespace cpu;
  LogicalGraph g = from_dsl(R"(language inferfabric 1;
model Acc { input x: tensor<f32>[2, 2]; const w: tensor<f32>[2, 2] = [1, 2, 3, 4]; const one: tensor<f32>[2, 2] = [1, 1, 1, 1];
  state hist: tensor<f32>[2, 2] = [0, 0, 0, 0];
  let scale = add(one, one); let p = matmul(x, w); let q = mul(p, scale); let r = relu(q); let dead = mul(p, p);
  let out = add(r, hist); update hist = out; yield out; }
plan Cpu for Acc { target = cpu_f32_v1; })");
  PhysicalPlan plan = compile(g);
  verify(plan);
  CHECK(plan.folded_constants == 1 && plan.eliminated_nodes == 1 && plan.steps.size() == 4);
  Executor ex(plan);
  auto r1 = ex.run({{"x", {1, 0, 0, 1}}});
  CHECK(r1.outputs.at("out") == (std::vector<float>{2, 4, 6, 8}));
  auto r2 = ex.run({{"x", {1, 0, 0, 1}}});
  CHECK(r2.outputs.at("out") == (std::vector<float>{4, 8, 12, 16}));   // state committed after the first run
  PhysicalPlan back = decode_plan(encode_plan(plan));
  CHECK(back.steps.size() == plan.steps.size() && back.arena_bytes == plan.arena_bytes);
  PhysicalPlan broken = plan;
  broken.steps[1].dependencies.clear();
  CHECK_THROWS(Invalid, verify(broken));
  broken = plan;
  for (auto& b : broken.buffers)
    if (b.storage == Storage::Temporary) b.offset = 0;   // everything aliased
  CHECK_THROWS(Invalid, verify(broken));
  Options o;
  o.override_kernels["p"] = Kernel::MatmulBlockedF32V1;
  CHECK(compile(g, o).steps[0].selection_reason == "forced by override");
  o.override_kernels["p"] = Kernel::AddF32V1;
  CHECK_THROWS(Invalid, compile(g, o));
  CHECK_THROWS(Invalid, ex.run({{"y", {1}}}));
}

#include "serve_tests.h"
#include "kernel_plugin.h"

static void test_kernel_plugin_loader() {
  using namespace ifab::plugin;
  const char* dir = std::getenv("IFAB_PLUGIN_DIR");
  if (!dir) {
    std::printf("skip kernel_plugin (IFAB_PLUGIN_DIR not set)\n");
    return;
  }
  const std::string so = std::string(dir) + "/libifab_plugin_swiglu_cpu.so";
  CHECK_THROWS(Io, PluginKernel("/nonexistent/plugin.so", "inferfabric.swiglu.bf16.v1", "cpu"));
  CHECK_THROWS(Stale, PluginKernel(so, "inferfabric.other.v1", "cpu"));
  CHECK_THROWS(Stale, PluginKernel(so, "inferfabric.swiglu.bf16.v1", kCudaTarget));      // built for another target
  std::vector<uint16_t> x(3 * 8, 0x3f80), y(3 * 4, 0);                                  // bf16 1.0 everywhere
  {
    PluginKernel k(so, "inferfabric.swiglu.bf16.v1", "cpu");
    CHECK_THROWS(Invalid, k.enqueue(nullptr, 0, nullptr));                               // before prepare
    IFKernelTensorV1 in = make_tensor(x.data(), 2, {3, 8}, 1), out = make_tensor(y.data(), 2, {3, 4}, 2);
    IFKernelTensorV1 ro = out;
    ro.access = 1;
    CHECK_THROWS(Invalid, k.prepare({in}, {ro}));                                        // output not writable
    IFKernelTensorV1 alias = make_tensor(x.data() + 4, 2, {3, 4}, 2);
    CHECK_THROWS(Invalid, k.prepare({in}, {alias}));                                     // output overlaps the input
    IFKernelTensorV1 small = in;
    small.allocation_bytes = 8;
    CHECK_THROWS(Invalid, k.prepare({small}, {out}));                                    // view larger than its allocation
    IFKernelTensorV1 wrong = make_tensor(y.data(), 2, {3, 5}, 2, 64);
    CHECK_THROWS(Backend, k.prepare({in}, {wrong}));                                     // the plugin itself refuses the shapes
    k.prepare({in}, {out});
    CHECK_THROWS(Invalid, k.prepare({in}, {out}));                                       // only once
    k.enqueue(nullptr, 0, nullptr);
    CHECK_THROWS(Invalid, k.enqueue(nullptr, 0, nullptr));                               // single-enqueue guard
    k.completed();
    k.enqueue(nullptr, 0, nullptr);
    k.completed();
  }
  // silu(1) * 1 = 0.7310586 -> bf16 0x3f3b
  CHECK(y[0] == 0x3f3b && y[11] == 0x3f3b);
}

// ---- engine-side contract validator: a correct program passes, each tampering is refused -----------------------
static void test_contract_validator() {
  // path of a model source (the two-layer example of the repository), handed over by the harness
  const char* src_path = std::getenv("IFAB_EXAMPLE_MODEL");
  if (!src_path) { std::printf("skip contract_validator (IFAB_EXAMPLE_MODEL not set)\n"); return; }
  graph::Graph g = graph::compile_source(read_file(src_path, 1 << 20));
  program::Program p = program::lower(g);
  init::Checkpoint ck = init::Checkpoint::synthetic(init::required_tensors(p));
  std::vector<init::Plan> plans = init::plan_all(p, ck);
  contract::validate_kernels(p);
  contract::validate_bindings(p, plans.at(0));
  auto find = [&](const char* op) -> size_t {
    for (size_t i = 0; i < p.instructions.size(); ++i) if (p.instructions[i].op == op) return i;
    return p.instructions.size();
  };
  auto drop_attr = [](program::Instruction& i, const char* key) {
    for (size_t k = 0; k < i.attrs.size(); ++k) if (i.attrs[k].first == key) { i.attrs.erase(i.attrs.begin() + (long)k); return; }
  };
  auto set_attr = [](program::Instruction& i, const char* key, const char* value) {
    for (auto& a : i.attrs) if (a.first == key) a.second = value;
  };
  { program::Program q = p; q.instructions[find("linear")].kernel = "cublasGemmEx"; CHECK_THROWS(Invalid, contract::validate_kernels(q)); }
  { program::Program q = p; q.instructions[find("router_topk")].kernel = "unsupported"; CHECK_THROWS(Invalid, contract::validate_kernels(q)); }
  { program::Program q = p; drop_attr(q.instructions[find("mla_q_absorb")], "theta"); CHECK_THROWS(Invalid, contract::validate_kernels(q)); }
  { program::Program q = p; set_attr(q.instructions[find("router_topk")], "topk", "4096"); CHECK_THROWS(Invalid, contract::validate_kernels(q)); }
  { program::Program q = p; set_attr(q.instructions[find("mla_attention")], "latent", "256"); CHECK_THROWS(Invalid, contract::validate_kernels(q)); }
  { program::Program q = p; set_attr(q.instructions[find("view")], "start", "100000"); CHECK_THROWS(Invalid, contract::validate_kernels(q)); }
  { program::Program q = p; q.instructions[find("moe_gate_up")].inputs.pop_back(); CHECK_THROWS(Invalid, contract::validate_kernels(q)); }
  { program::Program q = p; q.instructions[find("lm_head")].kind = 2; CHECK_THROWS(Invalid, contract::validate_kernels(q)); }
  { program::Program q = p; q.instructions[find("linear")].op = "conv3d"; CHECK_THROWS(Invalid, contract::validate_kernels(q)); }
  // bindings: a weight the rank does not load, a parameter nobody reads, a wrong leading dimension, a short load
  { program::Program q = p; set_attr(q.instructions[find("lm_head")], "weight", "lm_tail"); CHECK_THROWS(Invalid, contract::validate_bindings(q, plans[0])); }
  { init::Plan b = plans[0]; b.parameters.push_back(b.parameters[0]); b.parameters.back().name = "orphan"; CHECK_THROWS(Invalid, contract::validate_bindings(p, b)); }
  { init::Plan b = plans[0];
    const std::string head = *p.instructions[find("lm_head")].attr("weight");
    for (auto& prm : b.parameters) if (prm.name == head) prm.dims[0] += 8;
    CHECK_THROWS(Invalid, contract::validate_bindings(p, b)); }
  { init::Plan b = plans[0]; b.loads.pop_back(); CHECK_THROWS(Invalid, contract::validate_bindings(p, b)); }
  { init::Plan b = plans[0]; b.loads[0].dest = 100000; CHECK_THROWS(Invalid, contract::validate_bindings(p, b)); }
}

// ---- a hyper-connected program: residual streams mixed by mHC modules, token convolutions, attention sinks ----------------
static const char* kHyperSource = R"SRC(language inferfabric 1;
module Attn(x, w) {
    let qkv = linear(x, weight = w.qa, paired_weight = w.kva, width = 128, paired_width = 576, placement = "replicated");
    let qc = mome(slice(qkv, start = 0, width = 128), weight = w.q_conv, taps = 3);
    let q = linear(norm(qc, weight = w.q_norm, eps = 1e-5), weight = w.qb, width = 384, placement = "tp_rows");
    let kc = mome(slice(qkv, start = 128, width = 512), weight = w.kv_conv, taps = 3);
    let kr = slice(qkv, start = 640, width = 64);
    let sinks = sink_normalize(weight = w, norm = w.kv_norm, count = 3, latent = 512, rope = 64, eps = 1e-5);
    let cache = cache_norm_rope_append(kc, kr, sinks, weight = w.kv_norm, eps = 1e-5, theta = 10000);
    let query = mla_query(q, weight = w.kvb, theta = 10000, heads = 2, nope = 128, rope = 64, latent = 512, value = 128, input_layout = "rank_local");
    let att = latent_attention(query, cache, scale_dim = 192, window = 0, selection = "all_causal_within_window");
    let value = mla_value(att, weight = w.kvb, heads = 2, latent = 512, value = 128, nope = 128);
    let out = allreduce(linear(mome(value, weight = w.o_conv, taps = 3, placement = "tp_channels"), weight = w.o, width = 64, placement = "tp_columns"));
    yield out;
}
model Hyper {
    context = 32;
    eos = 2;
    let w = weights("m");
    let streams = repeat(embedding(weight = w.embed, width = 64, vocab = 96), count = 4);
    let hc = mhc_pre(streams, weight = w.mhc, streams = 4, sinkhorn = 20, eps = 1e-6);
    let branch = Attn(norm(mhc_input(hc), weight = w.in_norm, eps = 1e-5), w.attn);
    let mixed = mhc_post(hc, norm(branch, weight = w.out_norm, eps = 1e-5));
    let passed = optional_norm(mixed, weight = w.block_norm, eps = 1e-5);
    let merged = mhc_input(mhc_merge(passed, weight = w.merge, streams = 4, sinkhorn = 20, eps = 1e-6));
    let logits = gather(linear(norm(merged, weight = w.final_norm, eps = 1e-5), weight = weights("head"), width = 96, placement = "tp_rows"));
    yield logits;
}
plan P for Hyper { target = b200_token_v1; tp = 1; ep = 1; devices = [0]; max_num_seqs = 1; max_num_batched_tokens = 1; max_model_len = 32; }
)SRC";

static void test_hyper_connected_program() {
  graph::Graph g = graph::compile_source(kHyperSource);
  program::Program p = program::lower(g);
  auto find = [&](const char* op) -> size_t {
    for (size_t i = 0; i < p.instructions.size(); ++i) if (p.instructions[i].op == op) return i;
    return p.instructions.size();
  };
  // the checkpoint must hold the mixing tensors (f32, no ".weight" suffix), the taps of every convolution and the sink rows
  auto need = init::required_tensors(p);
  CHECK(need.count("m.mhc.phi") && need.at("m.mhc.phi").second == (std::vector<uint64_t>{24, 256}) && need.at("m.mhc.phi").first == init::DType::F32);
  CHECK(need.count("m.mhc.gamma") && need.count("m.mhc.alpha") && need.count("m.merge.beta") && need.at("m.merge.beta").second == (std::vector<uint64_t>{24}));
  CHECK(need.count("m.attn.q_conv.weight") && need.at("m.attn.q_conv.weight").second == (std::vector<uint64_t>{128, 1, 3}));
  CHECK(need.count("m.attn.o_conv.weight") && need.at("m.attn.o_conv.weight").second == (std::vector<uint64_t>{256, 1, 3}));
  CHECK(need.count("m.attn.param_sink_compressed_kv") && need.at("m.attn.param_sink_k_pe").second == (std::vector<uint64_t>{3, 64}));
  CHECK(!need.count("m.block_norm.weight"));                           // optional
  init::Checkpoint ck = init::Checkpoint::synthetic(need);
  std::vector<init::Plan> plans = init::plan_all(p, ck);
  const init::Parameter* taps = nullptr;
  for (auto& prm : plans.at(0).parameters) if (prm.name == "m.attn.kv_conv") taps = &prm;
  CHECK(taps && taps->dims == (std::vector<uint64_t>{512, 3}) && taps->dtype == init::DType::F32);   // [channels, 1, taps] loads as [channels, taps]
  contract::validate_kernels(p);
  contract::validate_bindings(p, plans[0]);
  { init::Plan b = plans[0];                                           // a mixing tensor the rank does not load
    for (size_t k = 0; k < b.parameters.size(); ++k) if (b.parameters[k].name == "m.mhc.phi") b.parameters[k].name = "m.mhc.psi";
    CHECK_THROWS(Invalid, contract::validate_bindings(p, b)); }
  { program::Program q = p;                                            // sink rows must come from a sink_normalize
    q.instructions[find("mla_kv_write")].inputs[2] = q.instructions[find("mla_kv_write")].inputs[0];
    CHECK_THROWS(Invalid, contract::validate_kernels(q)); }
  // lowering: the branch norm is folded into the return of the hyper-connection, which also names the streams it mixes
  const program::Instruction& post = p.instructions[find("mhc_post")];
  CHECK(post.inputs.size() == 3 && post.attr("norm_weight") && *post.attr("norm_weight") == "m.out_norm");
  CHECK(p.instructions[post.inputs[0]].op == "mhc_pre" && p.instructions[post.inputs[0]].inputs[0] == post.inputs[2]);
  size_t norms = 0;
  for (auto& i : p.instructions) norms += i.op == "norm";
  CHECK(norms == 0);
  // arena: an optional norm that passes its rows through gets no slot and keeps its source alive as long as it is read
  const uint32_t opt = (uint32_t)find("optional_norm");
  bundle::Arena plain = bundle::plan_arena(p, 8), aliased = bundle::plan_arena(p, 8, {opt});
  auto slot_of = [](const bundle::Arena& a, uint32_t ins) -> const bundle::ArenaSlot* {
    for (auto& sl : a.slots) if (sl.instruction == ins) return &sl;
    return nullptr;
  };
  CHECK(slot_of(plain, opt) != nullptr && slot_of(aliased, opt) == nullptr);
  const uint32_t src = p.instructions[opt].inputs[0];
  uint32_t last_reader = 0;
  for (uint32_t k = 0; k < p.instructions.size(); ++k)
    for (uint32_t in : p.instructions[k].inputs) if (in == opt) last_reader = k;
  CHECK(slot_of(aliased, src) && slot_of(aliased, src)->last >= last_reader && slot_of(plain, src)->last == opt);
  aliased.verify();
  // the oracle runs it: finite logits, and the convolution history makes a repeated token see a different past
  interp::Weights w = interp::Weights::random(need, 7);
  interp::Interpreter it(g, w);
  std::vector<float> l0, l2;
  it.step(5, 0, &l0);
  it.step(5, 1, nullptr);
  it.step(5, 2, &l2);
  bool finite = l0.size() == 96, differs = false;
  for (size_t i = 0; i < l0.size(); ++i) {
    finite = finite && std::isfinite(l0[i]) && std::isfinite(l2[i]);
    differs = differs || std::fabs(l0[i] - l2[i]) > 1e-4f;
  }
  CHECK(finite && differs);
}

// ---- a dense grouped-query program at tp = 2: lowering, sharded init plans, contracts, arena ---------------------------------
static const char* kDenseSource = R"SRC(language inferfabric 1;
module Attn(x, w) {
    let q = rotary_prefix(linear(x, weight = w.q, width = div(256, 2), placement = "tp_rows"), heads = div(4, 2), head_dim = 64, rotary_dim = 64, theta = 10000);
    let k = rotary_prefix(linear(x, weight = w.k, width = div(128, 2), placement = "tp_rows"), heads = div(2, 2), head_dim = 64, rotary_dim = 64, theta = 10000);
    let v = linear(x, weight = w.v, width = div(128, 2), placement = "tp_rows");
    let cache = kv_cache_append(k, v, kv_heads = 2, head_dim = 64);
    let att = paged_attention(q, cache, heads = 4, kv_heads = 2, head_dim = 64, scale = 0.125);
    yield allreduce(linear(att, weight = w.o, width = 128, placement = "tp_columns"));
}
model Dense {
    context = 64;
    eos = 2;
    let w = weights("m");
    let x = embedding(weight = w.embed, width = 128, vocab = 256);
    let h = add(x, Attn(norm(x, weight = w.n1, eps = 1e-6), w.attn));
    let act = swiglu(linear(norm(h, weight = w.n2, eps = 1e-6), weight = w.gate, paired_weight = w.up, width = div(192, 2), paired_width = div(192, 2), placement = "tp_rows"));
    let y = add(h, allreduce(linear(act, weight = w.down, width = 128, placement = "tp_columns")));
    let logits = gather(linear(norm(y, weight = w.nf, eps = 1e-6), weight = weights("head"), width = div(256, 2), placement = "tp_rows"));
    yield logits;
}
plan P for Dense { target = b200_token_v1; tp = 2; ep = 2; devices = [0, 1]; max_num_seqs = 1; max_num_batched_tokens = 1; max_model_len = 64; }
)SRC";

static void test_dense_program_at_two_ranks() {
  graph::Graph g = graph::compile_source(kDenseSource);
  program::Program p = program::lower(g);
  std::vector<std::string> ops;
  for (auto& i : p.instructions) ops.push_back(i.op);
  const std::vector<std::string> want = {"embedding", "linear", "rotary_prefix", "linear", "rotary_prefix", "linear", "kv_cache_append", "paged_attention",
                                         "linear_allreduce", "linear", "linear_allreduce", "lm_head"};
  CHECK(ops == want);                                                   // norms folded, residuals absorbed, SwiGLU fused, head fused
  const program::Instruction& gu = p.instructions[9];
  CHECK(gu.attr("activation") && *gu.attr("activation") == "swiglu" && gu.attr("paired_width") && *gu.attr("paired_width") == "96");
  CHECK(p.instructions[8].inputs.size() == 2 && p.instructions[10].inputs.size() == 2);      // residual operands of the fused all-reduces
  init::Checkpoint ck = init::Checkpoint::synthetic(init::required_tensors(p));
  std::vector<init::Plan> plans = init::plan_all(p, ck);
  CHECK(plans.size() == 2);
  for (auto& pl : plans) {
    contract::validate_bindings(p, pl);
    for (auto& prm : pl.parameters) {
      if (prm.name == "m.attn.q") CHECK(prm.dims == (std::vector<uint64_t>{128, 128}));                  // 2 of 4 heads
      if (prm.name == "m.attn.o") CHECK(prm.dims == (std::vector<uint64_t>{128, 128}));                  // half of the input columns
      if (prm.name == "m.gate|m.up") CHECK(prm.dims == (std::vector<uint64_t>{192, 128}));               // gate rows, then up rows, of this rank
      if (prm.name == "head") CHECK(prm.dims == (std::vector<uint64_t>{128, 128}));
    }
  }
  contract::validate_kernels(p);
  auto load_of = [](const init::Plan& pl, const std::string& tensor) -> const init::LoadSlice* {
    for (auto& l : pl.loads) if (l.tensor == tensor) return &l;
    return nullptr;
  };
  const init::LoadSlice *q0 = load_of(plans[0], "m.attn.q.weight"), *q1 = load_of(plans[1], "m.attn.q.weight");
  CHECK(q0 && q1 && q0->tag == 1 && q1->offset == q0->offset + q0->bytes);                                 // row shards: consecutive byte ranges
  const init::LoadSlice *o0 = load_of(plans[0], "m.attn.o.weight"), *o1 = load_of(plans[1], "m.attn.o.weight");
  CHECK(o0 && o1 && o0->tag == 2 && o0->row_bytes == 256 && o0->stride_bytes == 512 && o1->offset == o0->offset + 256);   // column shards: strided rows
  bundle::Arena a = bundle::plan_arena(p, 8);
  a.verify();
  CHECK(a.tokens == 8 && a.bytes > 0 && a.workspace_bytes > 0);
  for (auto& sl : a.slots) CHECK(p.instructions[sl.instruction].op != "kv_cache_append");                 // sequence state lives outside the arena
  // the oracle simulates both ranks
  interp::Weights w = interp::Weights::random(init::required_tensors(p), 3);
  interp::Interpreter it(g, w);
  std::vector<float> logits;
  it.step(7, 0, &logits);
  it.step(9, 1, &logits);
  bool finite = logits.size() == 256;
  for (float v : logits) finite = finite && std::isfinite(v);
  CHECK(finite);
}

// ---- chat post-processing: reasoning sections and tool calls ---------------------------------------------------------
static void test_chat_parsers() {
  using namespace ifab::chat;
  Parsed a = parse_assistant("<think>\nadd the numbers\n</think>\n\nThe sum is 4.");
  CHECK(a.has_reasoning && a.reasoning == "add the numbers" && a.content == "The sum is 4." && a.tool_calls.empty());
  Parsed b = parse_assistant("plan first</think>answer");          // the template opened the section in the prompt
  CHECK(b.has_reasoning && b.reasoning == "plan first" && b.content == "answer");
  Parsed c = parse_assistant("no sections here");
  CHECK(!c.has_reasoning && c.content == "no sections here");
  Parsed d = parse_assistant("Let me look.\n<tool_call>\n{\"name\": \"get_weather\", \"arguments\": {\"city\": \"Oslo\", \"days\": 2}}\n</tool_call>\n"
                             "<tool_call>{\"name\":\"now\"}</tool_call>");
  CHECK(d.tool_calls.size() == 2 && d.tool_calls[0].name == "get_weather" && d.tool_calls[1].name == "now" && d.tool_calls[1].arguments == "{}");
  CHECK(Json::parse(d.tool_calls[0].arguments).at("days").as_int() == 2 && d.content == "Let me look.");
  Parsed e = parse_assistant("<tool_call>{\"name\": 7}</tool_call> and <tool_call>{broken</tool_call> <tool_call>{\"name\":\"x\"}");
  CHECK(e.tool_calls.empty() && e.content.find("{broken") != std::string::npos && e.content.find("<tool_call>{\"name\":\"x\"}") != std::string::npos);
  Parsed f = parse_assistant("<tool_call>{\"name\":\"f\",\"arguments\":\"{\\\"k\\\": 1}\"}</tool_call>");   // arguments as a JSON string
  CHECK(f.tool_calls.size() == 1 && Json::parse(f.tool_calls[0].arguments).at("k").as_int() == 1);
  Parsed g = parse_assistant("<think>x</think><tool_call>{\"name\":\"f\"}</tool_call>", false, false);     // both parsers off: verbatim
  CHECK(!g.has_reasoning && g.tool_calls.empty() && g.content.find("<think>") == 0);
  Json m = message_json(d, "chatcmpl-9");
  CHECK(m.at("tool_calls").size() == 2 && m.at("tool_calls").as_array()[0].at("id").as_string() == "chatcmpl-9-call-0");
  CHECK(m.at("tool_calls").as_array()[0].at("function").at("arguments").is_string() && m.at("content").as_string() == "Let me look.");
  Json only_calls = message_json(parse_assistant("<tool_call>{\"name\":\"f\"}</tool_call>"), "id");
  CHECK(only_calls.at("content").is_null());
  Json tools = Json::parse("[{\"type\":\"function\",\"function\":{\"name\":\"get_weather\",\"parameters\":{\"type\":\"object\"}}}]");
  const std::string block = render_tools(tools);
  CHECK(block.find("\"get_weather\"") != std::string::npos && block.find("<tool_call>") != std::string::npos);
  CHECK_THROWS(Invalid, render_tools(Json::parse("[{\"type\":\"retrieval\"}]")));
  CHECK_THROWS(Invalid, render_tools(Json::parse("{}")));
}

// An initialization plan laid out byte for byte as the reference's encoder writes it (crates/inferfabric-compiler/src/
// initialization.rs:8-49): magic, rank, device, length-prefixed sha256 text, parameters {id, name, dtype, rank, dims},
// instructions {tag, destination, shard FILE name, absolute file offset, bytes, source dtype [, row_bytes, stride_bytes]}.
// Built here by hand, decoded by the library, executed against a shard file, and re-encoded to the same bytes.
static void test_init_plan_reference_layout() {
  namespace fs = std::filesystem;
  const fs::path dir = fs::temp_directory_path() / ("ifab_init_" + std::to_string((unsigned long)::getpid()));
  fs::create_directories(dir);
  // one shard with a [4, 6] bf16 matrix (values 0..23 as raw u16) and a [3] bf16 vector (100..102)
  init::TensorInfo a, b;
  a.name = "w"; a.dtype = init::DType::Bf16; a.shape = {4, 6};
  b.name = "v"; b.dtype = init::DType::Bf16; b.shape = {3};
  std::string da, db;
  for (uint16_t i = 0; i < 24; ++i) { da.push_back((char)(i & 0xff)); da.push_back((char)(i >> 8)); }
  for (uint16_t i = 100; i < 103; ++i) { db.push_back((char)(i & 0xff)); db.push_back((char)(i >> 8)); }
  init::write_safetensors((dir / "model-00001-of-00001.safetensors").string(), {{a, da}, {b, db}});
  const init::Checkpoint ck = init::Checkpoint::inspect(dir.string());
  const uint64_t w_at = ck.need("w").file_offset(), v_at = ck.need("v").file_offset();
  CHECK(w_at >= 8 && v_at == w_at + 48);

  std::string bytes = "IFINIT01";
  auto u32 = [&](uint32_t v) { for (int i = 0; i < 4; ++i) bytes.push_back((char)((v >> (8 * i)) & 0xff)); };
  auto u64 = [&](uint64_t v) { for (int i = 0; i < 8; ++i) bytes.push_back((char)((v >> (8 * i)) & 0xff)); };
  auto str = [&](const std::string& t) { u32((uint32_t)t.size()); bytes += t; };
  u32(1);                          // rank
  u32(1);                          // device
  str(std::string(64, 'c'));       // checkpoint metadata sha256 (provenance text)
  u32(3);                          // parameters
  u32(0); str("w.cols"); u32(2); u32(2); u64(4); u64(3);   // columns 3..5 of every row: strided source rows
  u32(1); str("v");      u32(3); u32(1); u64(3);           // bf16 source widened to f32
  u32(2); str("w.rows"); u32(2); u32(2); u64(2); u64(6);   // rows 2..3: one contiguous range
  u32(3);                          // instructions, one per parameter, in parameter order
  u32(2); u32(0); str("model-00001-of-00001.safetensors"); u64(w_at + 6); u64(24); u32(2); u64(6); u64(12);
  u32(1); u32(1); str("model-00001-of-00001.safetensors"); u64(v_at); u64(6); u32(2);
  u32(1); u32(2); str("model-00001-of-00001.safetensors"); u64(w_at + 24); u64(24); u32(2);

  init::Plan plan = init::Plan::decode(bytes);
  CHECK(plan.rank == 1 && plan.parameters.size() == 3 && plan.loads.size() == 3 && plan.reference_form());
  CHECK(plan.loads[0].shard == "model-00001-of-00001.safetensors" && plan.loads[0].offset == w_at + 6 && plan.loads[0].stride_bytes == 12);
  CHECK(plan.encode() == bytes);   // the same bytes come back
  init::Checkpoint files;          // execution needs the directory only: no tensor table, no fingerprint
  files.dir = dir.string();
  init::HostMemory mem;
  init::ExecuteOptions opt;
  opt.staging_bytes = 4096;
  opt.verify_upload = true;
  CHECK(init::execute(plan, files, mem, opt) == 24 + 12 + 24);
  auto u16_at = [&](uint32_t param, size_t i) { return (uint16_t)((uint8_t)mem.store[param][2 * i] | ((uint8_t)mem.store[param][2 * i + 1] << 8)); };
  const uint16_t want_cols[12] = {3, 4, 5, 9, 10, 11, 15, 16, 17, 21, 22, 23};
  for (size_t i = 0; i < 12; ++i) CHECK(u16_at(0, i) == want_cols[i]);
  for (size_t i = 0; i < 12; ++i) CHECK(u16_at(2, i) == 12 + i);
  uint32_t f0;
  memcpy(&f0, mem.store[1].data(), 4);
  CHECK(f0 == (100u << 16));       // bf16 bits moved to the upper half of the f32
  // what the reference's validate() refuses is refused here too under the IFINIT01 magic
  {
    std::string two = bytes;       // claim a second load for parameter 0 by rewriting the destination of the last load
    init::Plan bad = plan;
    bad.loads[2].dest = 0;
    CHECK(!bad.reference_form() && bad.encode().compare(0, 8, "IFINIT02") == 0);
    std::string forged = bad.encode();
    forged.replace(0, 8, "IFINIT01");
    CHECK_THROWS(Invalid, init::Plan::decode(forged));
  }
  {
    init::Plan bad = plan;
    bad.loads[1].shard = "../outside.safetensors";
    CHECK_THROWS(Invalid, init::Plan::decode(bad.encode()));
    bad = plan;
    bad.loads[2].offset = w_at + 1000;   // past the end of the shard
    CHECK_THROWS(Invalid, init::execute(bad, files, mem, opt));
  }
  fs::remove_all(dir);
}

static physical::Candidate device_candidate(const std::string& id, std::optional<uint64_t> est = std::nullopt, std::optional<uint64_t> upper = std::nullopt) {
  physical::Candidate c;
  c.id = id;
  c.contract_revision = "kernels@1";
  c.numerical_contract = "bf16 in, f32 accumulate, bf16 out";
  if (est) {
    c.cost.source = physical::CostSource::Analytical;
    c.cost.estimate_ns = est;
    c.cost.upper_ns = upper ? upper : est;
    c.cost.evidence = "stream-model-1";
  }
  return c;
}

static void test_physical_inspection_plan() {
  using namespace physical;
  // choice: complete costs -> cheapest conservative bound; any unknown cost -> stable baseline, never "unknown = free"
  std::vector<Candidate> cs = {device_candidate("b_fast", 900, 1000), device_candidate("a_slow", 800, 2000)};
  Choice c = choose(cs);
  CHECK(c.index == 0 && c.reason.find("cheapest") != std::string::npos);
  cs.push_back(device_candidate("c_unknown"));
  c = choose(cs);
  CHECK(cs[c.index].id == "a_slow" && c.reason.find("no latency is compared") != std::string::npos);
  // an ineligible candidate is skipped but must say why
  cs[1].eligible = false;
  CHECK_THROWS(Invalid, choose(cs));
  cs[1].rejection = "needs at least 9 rows";
  CHECK(cs[choose(cs).index].id == "b_fast");
  // residency is checked before cost: a host candidate, or one that copies through the host, is refused even if rejected
  auto host = cs;
  host[2].location = Location::Host;
  host[2].eligible = false;
  host[2].rejection = "cpu fallback";
  CHECK_THROWS(Invalid, choose(host));
  auto copy = cs;
  copy[0].boundaries.push_back({BoundaryKind::DeviceToHost, "reads the routing table back"});
  CHECK_THROWS(Invalid, choose(copy));
  auto numerics = cs;
  numerics[2].numerical_contract = "fp8";
  CHECK_THROWS(Invalid, choose(numerics));
  auto cost = cs;
  cost[0].cost.upper_ns = 100;   // bound below the estimate
  CHECK_THROWS(Invalid, choose(cost));
  CHECK_THROWS(Invalid, choose({}));

  // a three-step plan: embedding -> linear (+ all-reduce) -> head; one value per step
  auto op = [&](const char* name, size_t node, std::vector<size_t> in, std::vector<Candidate> cand) {
    Operation o;
    o.name = name;
    o.logical_nodes = {node};
    o.inputs = std::move(in);
    o.candidates = std::move(cand);
    return o;
  };
  auto val = [&](size_t node, uint64_t cols) {
    Value v;
    v.logical_node = node;
    v.dtype = "bf16";
    v.shape = {1, cols};
    v.payload_bytes = 2 * cols;
    v.alignment = 256;
    return v;
  };
  std::vector<Operation> ops = {op("embed", 0, {}, {device_candidate("ifab_embedding_bf16", 2000)}),
                                op("o_proj", 3, {0}, {device_candidate("ifab_gemv_allreduce_bf16", 8000, 9000)}),
                                op("head", 7, {1}, {device_candidate("ifab_lm_head_argmax", 60000)})};
  ops[1].collective = Collective{"all_ranks", "all_reduce_sum", "f32", 4096, 0};
  Plan p = serial_plan("toy", "b200_token_v1", std::string(64, 'd'), {0, 1}, ops, {val(0, 4096), val(3, 4096), val(7, 8)}, {2});
  CHECK(p.schedule.estimated_serial_ns && *p.schedule.estimated_serial_ns == 70000 && p.schedule.cost_complete && !p.executable);
  CHECK(p.schedule.values[0].last == 1 && p.schedule.values[1].last == 2 && p.schedule.values[2].last == 3);
  CHECK(p.schedule.steps[2].order_dependencies == std::vector<size_t>{1});
  // JSON round trip, then tampering: every derived fact is recomputed by verify
  Plan q = Plan::from_json(Json::parse(p.to_json().dump()));
  verify(q);
  CHECK(q.to_json().dump() == p.to_json().dump());
  { Plan t = q; t.schedule.steps[1].selected = 5; CHECK_THROWS(Invalid, verify(t)); }
  { Plan t = q; t.schedule.values[0].last = 2; CHECK_THROWS(Invalid, verify(t)); }
  { Plan t = q; t.schedule.values[1].payload_bytes = 9000; CHECK_THROWS(Invalid, verify(t)); }
  { Plan t = q; t.schedule.estimated_serial_ns = 1; CHECK_THROWS(Invalid, verify(t)); }
  { Plan t = q; t.schedule.steps[1].operation.collective->sequence = 1; CHECK_THROWS(Invalid, verify(t)); }
  { Plan t = q; t.executable = true; CHECK_THROWS(Invalid, verify(t)); }
  { Plan t = q; t.devices = {3, 3}; CHECK_THROWS(Invalid, verify(t)); }
  { Plan t = q; t.schedule.steps[2].operation.logical_nodes = {3}; CHECK_THROWS(Invalid, verify(t)); }
  { Plan t = q; t.schedule.steps[1].stream = 1; CHECK_THROWS(Invalid, verify(t)); }
  // a cost of unknown source makes the summary incomplete rather than smaller
  ops[2].candidates = {device_candidate("ifab_lm_head_argmax")};
  Plan u = serial_plan("toy", "b200_token_v1", std::string(64, 'd'), {0}, ops, {val(0, 4096), val(3, 4096), val(7, 8)}, {2});
  CHECK(!u.schedule.cost_complete && !u.schedule.estimated_serial_ns);
  ops[1].inputs = {2};
  CHECK_THROWS(Invalid, serial_plan("toy", "t", "d", {0}, ops, {val(0, 4096), val(3, 4096), val(7, 8)}, {2}));
}

static void test_device_buffer_contract() {
  using namespace device_buffer;
  Invocation call;
  call.implementation = "swiglu_cuda";
  call.binary_sha256 = std::string(64, 'a');
  call.numerical_contract = "inferfabric.swiglu.bf16.v1";
  call.rank = 1;
  call.device = 1;
  call.allocations = {{7, 1, 1, 1 << 20, 256, MemoryClass::Activation, false}, {9, 1, 1, 4096, 256, MemoryClass::Workspace, false},
                      {3, 1, 1, 1 << 16, 256, MemoryClass::Weight, true}};
  TensorView x{7, 0, DType::Bf16, {4, 256}, {256, 1}, 16, Access::Read};
  TensorView w{3, 512, DType::Bf16, {128}, {1}, 16, Access::Read};
  TensorView y{7, 4096, DType::Bf16, {4, 128}, {128, 1}, 16, Access::Write};
  call.inputs = {x, w};
  call.outputs = {y};
  call.workspace = Workspace{9, 0, 2048, 256};
  call.verify();
  CHECK(x.byte_span() == 2048);
  Invocation again = Invocation::from_json(Json::parse(call.to_json().dump()));
  again.verify();
  CHECK(again.to_json().dump() == call.to_json().dump());
  { Invocation c = call; c.outputs[0].offset = 1024; CHECK_THROWS(Invalid, c.verify()); }                       // output overlaps an input
  { Invocation c = call; c.outputs.push_back(y); CHECK_THROWS(Invalid, c.verify()); }                            // two outputs overlap
  { Invocation c = call; c.inputs[0].strides = {512, 1}; CHECK_THROWS(Invalid, c.verify()); }                    // not contiguous
  { Invocation c = call; c.outputs[0].allocation = 3; c.outputs[0].offset = 0; CHECK_THROWS(Invalid, c.verify()); }   // write into weights
  { Invocation c = call; c.allocations[2].read_only = false; CHECK_THROWS(Invalid, c.verify()); }                // writable weight
  { Invocation c = call; c.inputs[1].offset = 513; CHECK_THROWS(Invalid, c.verify()); }                          // misaligned
  { Invocation c = call; c.inputs[0].shape = {4096, 256}; c.inputs[0].strides = {256, 1}; CHECK_THROWS(Invalid, c.verify()); }   // outside
  { Invocation c = call; c.allocations.push_back({11, 1, 1, 64, 64, MemoryClass::State, false}); CHECK_THROWS(Invalid, c.verify()); }   // unused
  { Invocation c = call; c.allocations[0].device = 2; CHECK_THROWS(Invalid, c.verify()); }                       // other device
  { Invocation c = call; c.workspace->allocation = 7; c.workspace->offset = 4096; CHECK_THROWS(Invalid, c.verify()); }   // workspace on a tensor
  { Invocation c = call; c.binary_sha256 = "xyz"; CHECK_THROWS(Invalid, c.verify()); }
  call.verify_prepared(std::string(64, 'a'), "inferfabric.swiglu.bf16.v1", 1024, 128);
  CHECK_THROWS(Invalid, call.verify_prepared(std::string(64, 'a'), "inferfabric.swiglu.bf16.v1", 4096, 128));   // larger than frozen
  CHECK_THROWS(Invalid, call.verify_prepared(std::string(64, 'b'), "inferfabric.swiglu.bf16.v1", 0, 1));        // another binary
  { Invocation c = call; c.workspace.reset(); c.allocations.erase(c.allocations.begin() + 1); c.verify_prepared(std::string(64, 'a'), "inferfabric.swiglu.bf16.v1", 0, 1);
    CHECK_THROWS(Invalid, c.verify_prepared(std::string(64, 'a'), "inferfabric.swiglu.bf16.v1", 16, 16)); }
  // binding: descriptors carry absolute addresses (simulated here: they are never dereferenced)
  char* base = (char*)(uintptr_t)0x7f0000000000ull;
  std::vector<ResidentAllocation> res = {{7, base, 1 << 20, 1, 1}, {9, base + (2 << 20), 4096, 1, 1}, {3, base + (4 << 20), 1 << 16, 1, 1}};
  BoundInvocation b = device_buffer::bind(call, res);
  CHECK(b.inputs.size() == 2 && b.outputs.size() == 1 && b.outputs[0].data == base + 4096 && b.outputs[0].access == 2 && b.outputs[0].dtype == 2);
  CHECK(b.inputs[0].shape[1] == 256 && b.inputs[0].strides[0] == 256 && b.inputs[0].allocation_bytes == (1u << 20) && b.workspace == base + (2 << 20) && b.workspace_bytes == 2048);
  { auto r = res; r[1].base = base + 4096; CHECK_THROWS(Invalid, device_buffer::bind(call, r)); }          // another id, same memory as the output
  { auto r = res; r[0].bytes = 1 << 10; CHECK_THROWS(Invalid, device_buffer::bind(call, r)); }             // smaller than recorded
  { auto r = res; r[2].device = 0; CHECK_THROWS(Invalid, device_buffer::bind(call, r)); }
  { auto r = res; r[0].base = base + 8; CHECK_THROWS(Invalid, device_buffer::bind(call, r)); }             // misaligned base
  { auto r = res; r.pop_back(); CHECK_THROWS(Invalid, device_buffer::bind(call, r)); }
  CHECK(support().at("kernel_abi").as_string() == "IFKernelTensorV1");
}

int main() {
  std::pair<const char*, std::function<void()>> tests[] = {
      {"physical_inspection_plan", test_physical_inspection_plan}, {"device_buffer_contract", test_device_buffer_contract},
      {"init_plan_reference_layout", test_init_plan_reference_layout},
      {"serve_batching", test_serve_batching_matches_sequential}, {"serve_admission", test_serve_validation_and_admission},
      {"serve_backpressure_cancel", test_serve_backpressure_cancel_and_eos}, {"serve_failure_shutdown", test_serve_engine_failure_and_shutdown},
      {"api_tokenizer", test_api_tokenizer_and_sampling_json}, {"kernel_plugin", test_kernel_plugin_loader},
      {"state_pool", test_state_pool}, {"prefix_index", test_prefix_index}, {"paging", test_paging},
      {"rankplan_runtime", test_rankplan_and_runtime}, {"transfer", test_transfer}, {"scheduler", test_scheduler}, {"cpu_plan", test_cpu_plan},
      {"contract_validator", test_contract_validator}, {"hyper_connected_program", test_hyper_connected_program},
      {"dense_program_two_ranks", test_dense_program_at_two_ranks},
      {"chat_parsers", test_chat_parsers}};
  for (auto& t : tests) {
    int before = failures;
    try {
      t.second();
    } catch (const std::exception& e) {
      ++failures;
      std::printf("FAIL %s: unexpected exception: %s\n", t.first, e.what());
    }
    std::printf("%s %s\n", failures == before ? "ok  " : "FAIL", t.first);
  }
  std::printf("%d checks, %d failures\n", checks, failures);
  return failures ? 1 : 0;
}
