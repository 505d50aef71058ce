// Minimal HTTP/1.1 server for the inference front end: loopback only, one thread per connection (bounded), keep-alive,
// Content-Length bodies with a size limit, fixed responses or chunked streaming (used for server-sent events).
// No external dependencies; everything the OpenAI-compatible routes need and nothing more.
#pragma once
#include <atomic>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace ifab::http {

struct Request {
  std::string method, path, query, body;
  std::map<std::string, std::string> headers;   // lower-case names
};

class ResponseWriter {
 public:
  explicit ResponseWriter(int fd) : fd_(fd) {}
  // a complete response with Content-Length
  void send(int status, const std::string& content_type, const std::string& body);
  // chunked transfer: begin, any number of chunks, end. write_chunk returns false once the peer is gone.
  bool begin_stream(const std::string& content_type);
  bool write_chunk(const std::string& data);
  void end_stream();
  bool client_gone();          // non-blocking probe: the peer closed its side
  bool started() const { return started_; }
  bool broken() const { return broken_; }

 private:
  bool write_all(const char* p, size_t n);
  int fd_;
  bool started_ = false, streaming_ = false, broken_ = false;
};

using Handler = std::function<void(const Request&, ResponseWriter&)>;

class Server {
 public:
  // port 0 picks a free port (see port()). Binds 127.0.0.1 only.
  Server(uint16_t port, Handler handler, size_t max_connections = 256, size_t max_body_bytes = (size_t)32 << 20);
  ~Server();
  uint16_t port() const { return port_; }
  void stop();

 private:
  void accept_loop();
  void serve(int fd);
  Handler handler_;
  size_t max_connections_, max_body_;
  int listen_fd_ = -1;
  uint16_t port_ = 0;
  std::atomic<bool> stop_{false};
  std::atomic<size_t> active_{0};
  std::thread acceptor_;
  std::mutex mu_;
  std::vector<int> open_fds_;
};

const char* status_text(int status);

}  // namespace ifab::http
