// ifab-server: OpenAI-compatible HTTP front end (loopback only).
//
//   ifab-server --mock [options]                      deterministic CPU engine (tests, smoke runs, load tools)
//   ifab-server --engine-socket PATH [options]        engine worker(s) started by someone else connect to PATH
//   ifab-server --spawn "CMD" [options]               start CMD with IFAB_ENGINE_SOCKET set, wait for it to connect
//   ifab-server --program BUNDLE CHECKPOINT [--gpus N] [options]
//                                                     sugar for --spawn of the Python engine worker on a compiled bundle
//   ifab-server --program BUNDLE CHECKPOINT --cpu     run the bundle on the host with the CPU interpreter (no device needed)
//   ifab-server --program BUNDLE CHECKPOINT --native [--device N]   run a tp = 1 bundle on GPU N through the native device
//                                                     executor (csrc/device, loaded on demand): no Python in the serving path
// Options: --port P (0 = pick one, printed), --max-num-seqs N, --max-num-batched-tokens B, --max-model-len C,
//          --vocab V, --max-queue Q, --stream-capacity S, --step-micros U (mock), --accept-seconds S, --temperature T,
//          --top-k K, --presence-penalty X (server-side sampling defaults), --sampling-defaults model-card|DIR|FILE (the
//          model-card recommendation, overridden by DIR/generation_config.json).
// Prints "listening on 127.0.0.1:PORT" once ready; SIGINT / SIGTERM drain and exit.
// Reference: frontend/src/main.rs (modes --mock / --program / --native), frontend/src/shutdown.rs.
#include <dlfcn.h>
#include <signal.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>

#include "api.h"
#include "program_engine.h"

using namespace ifab;

namespace {

struct Args {
  std::string mode, socket, spawn, bundle, checkpoint, tokenizer = "bytes", chat_template = "auto", device_lib;
  int port = 8000, gpus = 1, device = 0;
  bool cpu = false, native = false, seqs_given = false, len_given = false;
  serve::EngineInfo info;
  serve::ServiceOptions opt;
  uint32_t step_micros = 0;
  double accept_seconds = 600;
  serve::SamplingParams defaults;
};

[[noreturn]] void usage(const char* why) {
  std::fprintf(stderr, "ifab-server: %s\nmodes: --mock | --engine-socket PATH | --spawn CMD | --program BUNDLE CHECKPOINT [--gpus N]\n", why);
  std::exit(2);
}

Args parse(int argc, char** argv) {
  Args a;
  a.info.model = "ifab-mock";
  a.info.residents = 4;
  a.info.token_budget = 8;
  a.info.chunk = 8;
  a.info.context = 512;
  a.info.vocab = 1024;
  a.info.eos = api::ByteTokenizer::kEos;
  a.info.has_eos = true;
  auto need = [&](int& i) -> const char* {
    if (i + 1 >= argc) usage((std::string("missing value after ") + argv[i]).c_str());
    return argv[++i];
  };
  for (int i = 1; i < argc; ++i) {
    const std::string f = argv[i];
    if (f == "--mock") a.mode = "mock";
    else if (f == "--engine-socket") { a.mode = "socket"; a.socket = need(i); }
    else if (f == "--spawn") { a.mode = "spawn"; a.spawn = need(i); }
    else if (f == "--program") { a.mode = "program"; a.bundle = need(i); a.checkpoint = need(i); }
    else if (f == "--gpus") a.gpus = std::atoi(need(i));
    else if (f == "--cpu") a.cpu = true;
    else if (f == "--native") a.native = true;                     // --program on the GPU through libifab_device.so (tp = 1 bundles)
    else if (f == "--device") a.device = std::atoi(need(i));
    else if (f == "--device-lib") a.device_lib = need(i);
    else if (f == "--tokenizer") a.tokenizer = need(i);            // "bytes" or the path of a tokenizer.json (byte-level BPE)
    else if (f == "--chat-template") a.chat_template = need(i);    // auto | chatml | plain
    else if (f == "--port") a.port = std::atoi(need(i));
    else if (f == "--max-num-seqs") { a.info.residents = (uint32_t)std::atoi(need(i)); a.seqs_given = true; }
    else if (f == "--max-num-batched-tokens") a.info.token_budget = a.info.chunk = (uint32_t)std::atoi(need(i));
    else if (f == "--max-model-len") { a.info.context = (uint32_t)std::atoi(need(i)); a.len_given = true; }
    else if (f == "--vocab") a.info.vocab = (uint32_t)std::atoi(need(i));
    else if (f == "--max-queue") a.opt.queue = (uint32_t)std::atoi(need(i));
    else if (f == "--stream-capacity") a.opt.stream_capacity = (uint32_t)std::atoi(need(i));
    else if (f == "--step-micros") a.step_micros = (uint32_t)std::atoi(need(i));
    else if (f == "--accept-seconds") a.accept_seconds = std::atof(need(i));
    else if (f == "--sampling-defaults") {
      // "model-card": temperature 1, top-k 20, presence penalty 2; a directory or file: those, overridden by its generation_config.json
      const std::string v = need(i);
      a.defaults = v == "model-card" ? serve::SamplingParams::model_card() : serve::SamplingParams::deployment_defaults(v);
    }
    else if (f == "--temperature") a.defaults.temperature = std::atof(need(i));
    else if (f == "--top-k") a.defaults.top_k = std::atoi(need(i));
    else if (f == "--presence-penalty") a.defaults.presence_penalty = std::atof(need(i));
    else if (f == "--model-name") a.info.model = need(i);
    else usage(("unknown flag " + f).c_str());
  }
  if (a.mode.empty()) usage("no mode given");
  return a;
}

// libifab_device.so next to this binary's directory: <dir>/../device/libifab_device.so
std::string default_device_lib(const char* argv0) {
  char buf[4096];
  const ssize_t n = ::readlink("/proc/self/exe", buf, sizeof buf - 1);
  std::string exe = n > 0 ? std::string(buf, (size_t)n) : std::string(argv0);
  const size_t slash = exe.find_last_of('/');
  return (slash == std::string::npos ? std::string(".") : exe.substr(0, slash)) + "/../device/libifab_device.so";
}

pid_t spawn_shell(const std::string& cmd, const std::string& socket_path) {
  const pid_t pid = ::fork();
  if (pid < 0) return -1;
  if (pid == 0) {
    ::setenv("IFAB_ENGINE_SOCKET", socket_path.c_str(), 1);
    ::setpgid(0, 0);
    ::execl("/bin/sh", "sh", "-c", cmd.c_str(), (char*)nullptr);
    ::_exit(127);
  }
  return pid;
}

}  // namespace

int main(int argc, char** argv) {
  Args a = parse(argc, argv);
  // block the termination signals in every thread; one thread waits for them
  sigset_t set;
  sigemptyset(&set);
  sigaddset(&set, SIGINT);
  sigaddset(&set, SIGTERM);
  pthread_sigmask(SIG_BLOCK, &set, nullptr);
  ::signal(SIGPIPE, SIG_IGN);

  pid_t child = -1;
  std::shared_ptr<serve::ResidentEngine> engine;
  std::shared_ptr<tok::Tokenizer> tokenizer;
  try {
    tokenizer = tok::load_tokenizer(a.tokenizer);
    if (a.mode == "mock" && a.tokenizer != "bytes") {
      // the stand-in engine speaks the tokenizer's vocabulary: its end-of-sequence id and width come from the file
      if (tokenizer->eos() >= 0) a.info.eos = (uint32_t)tokenizer->eos();
      a.info.vocab = std::max<uint32_t>(a.info.vocab, tokenizer->vocab_size());
    }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ifab-server: cannot load the tokenizer: %s\n", e.what());
    return 1;
  }
  try {
    if (a.mode == "mock") {
      engine = std::make_shared<serve::MockEngine>(a.info, a.step_micros);
    } else if (a.mode == "program" && a.cpu) {
      engine = serve::make_cpu_program_engine(a.bundle, a.checkpoint, a.seqs_given ? a.info.residents : 0, a.len_given ? a.info.context : 0);
    } else if (a.mode == "program" && a.native) {
      // the native device executor, loaded on demand so that this binary needs no CUDA: no Python, no worker process
      const std::string lib = a.device_lib.empty() ? default_device_lib(argv[0]) : a.device_lib;
      void* h = ::dlopen(lib.c_str(), RTLD_NOW | RTLD_GLOBAL);
      if (!h) throw Error(ErrorKind::Io, std::string("cannot load the device executor: ") + ::dlerror());
      using New = void* (*)(const char*, const char*, int, uint32_t, uint32_t);
      using Err = const char* (*)();
      auto make = reinterpret_cast<New>(::dlsym(h, "ifab_device_program_engine_new"));
      auto why = reinterpret_cast<Err>(::dlsym(h, "ifab_device_program_error"));
      if (!make || !why) throw Error(ErrorKind::Io, "the device executor library lacks its entry points");
      void* made = make(a.bundle.c_str(), a.checkpoint.c_str(), a.device, a.seqs_given ? a.info.residents : 0, a.len_given ? a.info.context : 0);
      if (!made) throw Error(ErrorKind::Backend, why());
      auto* holder = static_cast<std::shared_ptr<serve::ResidentEngine>*>(made);
      engine = std::move(*holder);
      delete holder;
    } else {
      if (a.socket.empty()) a.socket = "/tmp/ifab-engine-" + std::to_string((long)::getpid()) + ".sock";
      if (a.mode == "program") {
        const std::string worker = "-m ironpangu_b200.runtime.engine_worker --bundle '" + a.bundle + "' --checkpoint '" + a.checkpoint +
                                   "' --max-num-seqs " + std::to_string(a.info.residents) + " --max-model-len " + std::to_string(a.info.context);
        a.spawn = a.gpus > 1 ? "python -m torch.distributed.run --nnodes=1 --nproc-per-node " + std::to_string(a.gpus) +
                                   " --master-addr 127.0.0.1 --master-port 29577 " + worker
                             : "python " + worker;
      }
      if (!a.spawn.empty()) {
        child = spawn_shell(a.spawn, a.socket);
        if (child < 0) throw Error(ErrorKind::Io, "cannot start the engine worker");
      }
      engine = std::make_shared<serve::PipeEngine>(a.socket, a.accept_seconds, 120.0, (long)child);
    }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ifab-server: engine start-up failed: %s\n", e.what());
    if (child > 0) ::kill(-child, SIGTERM);
    return 1;
  }
  serve::Service service(engine, a.opt);
  if (service.info().greedy_only) a.defaults.temperature = 0.0;
  api::Api api(service, a.defaults, tokenizer, a.chat_template);
  std::unique_ptr<http::Server> server;
  try {
    server = std::make_unique<http::Server>((uint16_t)a.port, [&](const http::Request& r, http::ResponseWriter& w) { api.handle(r, w); });
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ifab-server: %s\n", e.what());
    service.shutdown();
    if (child > 0) ::kill(-child, SIGTERM);
    return 1;
  }
  std::printf("listening on 127.0.0.1:%u\n", (unsigned)server->port());
  std::printf("engine %s residents=%u token_budget=%u context=%u vocab=%u world=%u\n", service.info().model.c_str(), service.info().residents,
              service.info().token_budget, service.info().context, service.info().vocab, service.info().world);
  std::fflush(stdout);
  int sig = 0;
  sigwait(&set, &sig);
  std::fprintf(stderr, "ifab-server: signal %d, draining\n", sig);
  server->stop();
  service.shutdown();
  if (child > 0) {
    int status = 0;
    for (int i = 0; i < 100; ++i) {
      if (::waitpid(child, &status, WNOHANG) != 0) break;
      ::usleep(100000);
      if (i == 50) ::kill(-child, SIGTERM);
    }
  }
  return 0;
}
