#include "http.h"

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <stdexcept>

namespace ifab::http {

const char* status_text(int s) {
  switch (s) {
    case 200: return "OK";
    case 400: return "Bad Request";
    case 404: return "Not Found";
    case 405: return "Method Not Allowed";
    case 413: return "Payload Too Large";
    case 429: return "Too Many Requests";
    case 500: return "Internal Server Error";
    case 503: return "Service Unavailable";
    default: return "Status";
  }
}

bool ResponseWriter::write_all(const char* p, size_t n) {
  while (n > 0 && !broken_) {
    const ssize_t w = ::send(fd_, p, n, MSG_NOSIGNAL);
    if (w <= 0) {
      broken_ = true;
      return false;
    }
    p += w;
    n -= (size_t)w;
  }
  return !broken_;
}

void ResponseWriter::send(int status, const std::string& content_type, const std::string& body) {
  if (started_) return;
  started_ = true;
  std::string head = "HTTP/1.1 " + std::to_string(status) + " " + status_text(status) + "\r\nContent-Type: " + content_type +
                     "\r\nContent-Length: " + std::to_string(body.size()) + "\r\nConnection: keep-alive\r\n\r\n";
  write_all(head.data(), head.size());
  write_all(body.data(), body.size());
}

bool ResponseWriter::begin_stream(const std::string& content_type) {
  if (started_) return false;
  started_ = streaming_ = true;
  const std::string head = "HTTP/1.1 200 OK\r\nContent-Type: " + content_type +
                           "\r\nCache-Control: no-cache\r\nTransfer-Encoding: chunked\r\nConnection: keep-alive\r\n\r\n";
  return write_all(head.data(), head.size());
}

bool ResponseWriter::write_chunk(const std::string& data) {
  if (!streaming_ || data.empty()) return !broken_;
  char len[32];
  const int n = std::snprintf(len, sizeof(len), "%zx\r\n", data.size());
  return write_all(len, (size_t)n) && write_all(data.data(), data.size()) && write_all("\r\n", 2);
}

void ResponseWriter::end_stream() {
  if (streaming_) write_all("0\r\n\r\n", 5);
  streaming_ = false;
}

bool ResponseWriter::client_gone() {
  if (broken_) return true;
  pollfd p{fd_, POLLIN | POLLRDHUP, 0};
  if (::poll(&p, 1, 0) > 0) {
    if (p.revents & (POLLRDHUP | POLLHUP | POLLERR)) return broken_ = true;
    if (p.revents & POLLIN) {
      char c;
      if (::recv(fd_, &c, 1, MSG_PEEK | MSG_DONTWAIT) == 0) return broken_ = true;
    }
  }
  return false;
}

Server::Server(uint16_t port, Handler handler, size_t max_connections, size_t max_body)
    : handler_(std::move(handler)), max_connections_(max_connections), max_body_(max_body) {
  listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
  if (listen_fd_ < 0) throw std::runtime_error("http: cannot create socket");
  int one = 1;
  ::setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  addr.sin_port = htons(port);
  if (::bind(listen_fd_, (sockaddr*)&addr, sizeof(addr)) != 0 || ::listen(listen_fd_, 128) != 0) {
    ::close(listen_fd_);
    throw std::runtime_error("http: cannot bind 127.0.0.1:" + std::to_string(port));
  }
  socklen_t len = sizeof(addr);
  ::getsockname(listen_fd_, (sockaddr*)&addr, &len);
  port_ = ntohs(addr.sin_port);
  acceptor_ = std::thread([this] { accept_loop(); });
}

Server::~Server() { stop(); }

void Server::stop() {
  if (stop_.exchange(true)) return;
  if (listen_fd_ >= 0) ::shutdown(listen_fd_, SHUT_RDWR);
  if (acceptor_.joinable()) acceptor_.join();
  if (listen_fd_ >= 0) ::close(listen_fd_);
  listen_fd_ = -1;
  {
    std::lock_guard<std::mutex> lk(mu_);
    for (int fd : open_fds_) ::shutdown(fd, SHUT_RDWR);
  }
  for (int i = 0; i < 500 && active_.load() > 0; ++i) ::usleep(10000);
}

void Server::accept_loop() {
  while (!stop_.load()) {
    pollfd p{listen_fd_, POLLIN, 0};
    if (::poll(&p, 1, 100) <= 0) continue;
    const int fd = ::accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) continue;
    if (active_.load() >= max_connections_) {
      ResponseWriter w(fd);
      w.send(503, "text/plain", "too many connections\n");
      ::close(fd);
      continue;
    }
    int one = 1;
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    ++active_;
    {
      std::lock_guard<std::mutex> lk(mu_);
      open_fds_.push_back(fd);
    }
    std::thread([this, fd] {
      serve(fd);
      {
        std::lock_guard<std::mutex> lk(mu_);
        open_fds_.erase(std::remove(open_fds_.begin(), open_fds_.end(), fd), open_fds_.end());
      }
      ::close(fd);
      --active_;
    }).detach();
  }
}

static std::string lower(std::string s) {
  for (auto& c : s) c = (char)std::tolower((unsigned char)c);
  return s;
}

void Server::serve(int fd) {
  std::string buf;
  char tmp[16384];
  while (!stop_.load()) {
    // read the header block
    size_t hend;
    while ((hend = buf.find("\r\n\r\n")) == std::string::npos) {
      if (buf.size() > 65536) return;
      pollfd p{fd, POLLIN, 0};
      const int pr = ::poll(&p, 1, 30000);
      if (pr <= 0 || stop_.load()) return;
      const ssize_t n = ::recv(fd, tmp, sizeof(tmp), 0);
      if (n <= 0) return;
      buf.append(tmp, (size_t)n);
    }
    Request req;
    const std::string head = buf.substr(0, hend);
    buf.erase(0, hend + 4);
    size_t line_end = head.find("\r\n");
    const std::string first = head.substr(0, line_end);
    const size_t sp1 = first.find(' '), sp2 = first.rfind(' ');
    ResponseWriter w(fd);
    if (sp1 == std::string::npos || sp2 == sp1) {
      w.send(400, "text/plain", "malformed request line\n");
      return;
    }
    req.method = first.substr(0, sp1);
    std::string target = first.substr(sp1 + 1, sp2 - sp1 - 1);
    const size_t qm = target.find('?');
    req.path = target.substr(0, qm);
    if (qm != std::string::npos) req.query = target.substr(qm + 1);
    size_t pos = line_end == std::string::npos ? head.size() : line_end + 2;
    while (pos < head.size()) {
      size_t e = head.find("\r\n", pos);
      if (e == std::string::npos) e = head.size();
      const std::string line = head.substr(pos, e - pos);
      const size_t colon = line.find(':');
      if (colon != std::string::npos) {
        size_t v = colon + 1;
        while (v < line.size() && line[v] == ' ') ++v;
        req.headers[lower(line.substr(0, colon))] = line.substr(v);
      }
      pos = e + 2;
    }
    size_t need = 0;
    if (auto it = req.headers.find("content-length"); it != req.headers.end()) need = (size_t)std::strtoull(it->second.c_str(), nullptr, 10);
    if (need > max_body_) {
      w.send(413, "text/plain", "body too large\n");
      return;
    }
    while (buf.size() < need) {
      pollfd p{fd, POLLIN, 0};
      if (::poll(&p, 1, 30000) <= 0 || stop_.load()) return;
      const ssize_t n = ::recv(fd, tmp, sizeof(tmp), 0);
      if (n <= 0) return;
      buf.append(tmp, (size_t)n);
    }
    req.body = buf.substr(0, need);
    buf.erase(0, need);
    try {
      handler_(req, w);
    } catch (const std::exception& e) {
      if (!w.started()) w.send(500, "text/plain", std::string("internal error: ") + e.what() + "\n");
    }
    if (!w.started()) w.send(404, "text/plain", "not found\n");
    if (w.broken()) return;
    auto conn = req.headers.find("connection");
    if (conn != req.headers.end() && lower(conn->second) == "close") return;
  }
}

}  // namespace ifab::http
