// Client side of the remote memory pool: see RemotePool in staged_lane.hpp for the
// protocol. Sockets are blocking with send/receive timeouts, so that a daemon that
// stops answering turns into an I/O error (and the runtime's failure latch) instead
// of a hang.
#include "staged_lane.hpp"

#include <arpa/inet.h>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

namespace ssc {

namespace {

constexpr int IO_TIMEOUT_SECONDS = 30;

int send_all(int fd, const char* p, int64_t n) {
  while (n > 0) {
    ssize_t k = ::send(fd, p, static_cast<size_t>(n), MSG_NOSIGNAL);
    if (k < 0) {
      if (errno == EINTR) continue;
      return -1;
    }
    p += k; n -= k;
  }
  return 0;
}

int recv_all(int fd, char* p, int64_t n) {
  while (n > 0) {
    ssize_t k = ::recv(fd, p, static_cast<size_t>(n), 0);
    if (k < 0) {
      if (errno == EINTR) continue;
      return -1;
    }
    if (k == 0) return -1;       // the peer closed
    p += k; n -= k;
  }
  return 0;
}

// Reads one '\n'-terminated line (without the newline), byte by byte: replies are short.
int recv_line(int fd, std::string& line) {
  line.clear();
  char c;
  while (line.size() < 256) {
    if (recv_all(fd, &c, 1) != 0) return -1;
    if (c == '\n') return 0;
    line.push_back(c);
  }
  return -1;
}

int dial(const std::string& host, int port) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  char service[16];
  std::snprintf(service, sizeof service, "%d", port);
  if (::getaddrinfo(host.c_str(), service, &hints, &res) != 0) return -1;
  int fd = -1;
  for (addrinfo* a = res; a; a = a->ai_next) {
    fd = ::socket(a->ai_family, a->ai_socktype | SOCK_CLOEXEC, a->ai_protocol);
    if (fd < 0) continue;
    timeval tv{IO_TIMEOUT_SECONDS, 0};
    ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
    ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
    int one = 1;
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
    if (::connect(fd, a->ai_addr, a->ai_addrlen) == 0) break;
    ::close(fd);
    fd = -1;
  }
  ::freeaddrinfo(res);
  return fd;
}

// Sends `request` and expects a reply line that starts with "OK"; the rest of it is returned.
int exchange(int fd, const std::string& request, std::string& rest) {
  if (send_all(fd, request.data(), static_cast<int64_t>(request.size())) != 0) return -1;
  std::string line;
  if (recv_line(fd, line) != 0) return -1;
  if (line.compare(0, 2, "OK") != 0) return -1;
  rest = line.size() > 3 ? line.substr(3) : "";
  return 0;
}

}  // namespace

int RemotePool::open(const char* address, int64_t bytes, std::string& error) {
  close();
  if (!address || bytes <= 0) { error = "remote pool needs host:port and a positive size"; return SS_INVALID_ARGUMENT; }
  const std::string a(address);
  const size_t colon = a.rfind(':');
  if (colon == std::string::npos) { error = "remote pool address must be host:port"; return SS_INVALID_ARGUMENT; }
  host_ = a.substr(0, colon);
  port_ = std::atoi(a.c_str() + colon + 1);
  const int fd = dial(host_, port_);
  if (fd < 0) { error = "cannot reach the memory daemon at " + a; return SS_IO_ERROR; }
  std::string rest;
  if (exchange(fd, "ALLOCATE " + std::to_string(bytes) + "\n", rest) != 0) {
    ::close(fd);
    error = "the memory daemon at " + a + " refused " + std::to_string(bytes) + " bytes";
    return SS_OUT_OF_MEMORY;
  }
  region_ = std::atoll(rest.c_str());
  control_fd_ = fd;
  bytes_ = bytes;
  return SS_OK;
}

void RemotePool::close() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    for (int fd : idle_) ::close(fd);
    idle_.clear();
  }
  if (control_fd_ >= 0) {
    std::string rest;
    exchange(control_fd_, "FREE " + std::to_string(region_) + "\n", rest);   // best effort: closing frees too
    ::close(control_fd_);
  }
  control_fd_ = -1;
  region_ = -1;
  bytes_ = 0;
}

int RemotePool::connect_data() {
  const int fd = dial(host_, port_);
  if (fd < 0) return -1;
  std::string rest;
  if (exchange(fd, "CONNECT " + std::to_string(region_) + "\n", rest) != 0) { ::close(fd); return -1; }
  return fd;
}

int RemotePool::borrow() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (!idle_.empty()) {
      const int fd = idle_.back();
      idle_.pop_back();
      return fd;
    }
  }
  return connect_data();
}

void RemotePool::give_back(int fd) {
  std::lock_guard<std::mutex> lk(mu_);
  idle_.push_back(fd);
}

int RemotePool::chunk_io(bool write, void* buf, int64_t off, int64_t n) {
  if (control_fd_ < 0 || off < 0 || n < 0 || off + n > bytes_) return SS_INVALID_ARGUMENT;
  if (n == 0) return SS_OK;
  const int fd = borrow();
  if (fd < 0) return SS_IO_ERROR;
  char head[96];
  std::snprintf(head, sizeof head, "%s %lld %lld\n", write ? "WRITE" : "READ",
                static_cast<long long>(off), static_cast<long long>(n));
  bool ok = send_all(fd, head, static_cast<int64_t>(std::strlen(head))) == 0;
  std::string line;
  if (ok && write) ok = send_all(fd, static_cast<const char*>(buf), n) == 0;
  ok = ok && recv_line(fd, line) == 0 && line.compare(0, 2, "OK") == 0;
  if (ok && !write) ok = recv_all(fd, static_cast<char*>(buf), n) == 0;
  if (!ok) { ::close(fd); return SS_IO_ERROR; }      // the stream position is unknown: drop it
  give_back(fd);
  return SS_OK;
}

}  // namespace ssc
