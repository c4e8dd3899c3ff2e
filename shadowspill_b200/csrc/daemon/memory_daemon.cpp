// ss_memory_daemon: holds host memory for training runs on other machines (the far
// side of RemotePool, staged_lane.hpp).
//
//   ss_memory_daemon --port 7070 [--bind 0.0.0.0] [--capacity-gib 512] [--lock]
//
// One thread per connection. A region is created by ALLOCATE on a connection and lives
// as long as that connection (a trainer that dies frees its memory); CONNECT attaches
// further connections of the same client to it for data. Prints "listening <port>" on
// stdout once it accepts connections (port 0 picks a free one). The reference's daemon
// answers the same allocate/connect/free requests for RDMA-registered memory
// (packages/engine/csrc/daemon/src/daemon.c, daemon/README.md:36-42); this one serves
// the bytes over the connection itself.
#include <arpa/inet.h>
#include <atomic>
#include <cerrno>
#include <csignal>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <string>
#include <sys/mman.h>
#include <sys/socket.h>
#include <thread>
#include <unistd.h>

namespace {

struct Region {
  char* base = nullptr;
  int64_t bytes = 0;
  ~Region() { if (base) ::munmap(base, static_cast<size_t>(bytes)); }
};

std::mutex g_mu;
std::map<int64_t, std::shared_ptr<Region>> g_regions;
int64_t g_next_region = 1;
int64_t g_held = 0, g_capacity = 0;
bool g_lock = false;

bool send_all(int fd, const char* p, int64_t n) {
  while (n > 0) {
    ssize_t k = ::send(fd, p, static_cast<size_t>(n), MSG_NOSIGNAL);
    if (k < 0) { if (errno == EINTR) continue; return false; }
    p += k; n -= k;
  }
  return true;
}
bool recv_all(int fd, char* p, int64_t n) {
  while (n > 0) {
    ssize_t k = ::recv(fd, p, static_cast<size_t>(n), 0);
    if (k < 0) { if (errno == EINTR) continue; return false; }
    if (k == 0) return false;
    p += k; n -= k;
  }
  return true;
}
bool recv_line(int fd, std::string& line) {
  line.clear();
  char c;
  while (line.size() < 256) {
    if (!recv_all(fd, &c, 1)) return false;
    if (c == '\n') return true;
    line.push_back(c);
  }
  return false;
}
bool reply(int fd, const std::string& s) { return send_all(fd, s.data(), static_cast<int64_t>(s.size())); }

std::shared_ptr<Region> allocate(int64_t bytes, int64_t* id) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (bytes <= 0 || (g_capacity > 0 && g_held + bytes > g_capacity)) return nullptr;
  void* p = ::mmap(nullptr, static_cast<size_t>(bytes), PROT_READ | PROT_WRITE,
                   MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (p == MAP_FAILED) return nullptr;
  if (g_lock) ::mlock(p, static_cast<size_t>(bytes));      // best effort
  auto r = std::make_shared<Region>();
  r->base = static_cast<char*>(p);
  r->bytes = bytes;
  *id = g_next_region++;
  g_regions[*id] = r;
  g_held += bytes;
  return r;
}

void release(int64_t id) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_regions.find(id);
  if (it == g_regions.end()) return;
  g_held -= it->second->bytes;
  g_regions.erase(it);          // memory goes when the last data connection lets go of it
}

void serve(int fd) {
  int one = 1;
  ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
  std::shared_ptr<Region> region;     // what WRITE / READ address
  int64_t owned = -1;                 // the region this connection allocated
  std::string line;
  while (recv_line(fd, line)) {
    char verb[16] = {0};
    long long a = 0, b = 0;
    const int fields = std::sscanf(line.c_str(), "%15s %lld %lld", verb, &a, &b);
    if (fields < 1) break;
    if (!std::strcmp(verb, "ALLOCATE") && fields >= 2 && owned < 0) {
      region = allocate(a, &owned);
      if (!region) { owned = -1; if (!reply(fd, "ERR out of memory\n")) break; continue; }
      if (!reply(fd, "OK " + std::to_string(owned) + "\n")) break;
    } else if (!std::strcmp(verb, "CONNECT") && fields >= 2) {
      {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_regions.find(a);
        region = it == g_regions.end() ? nullptr : it->second;
      }
      if (!reply(fd, region ? "OK " + std::to_string(region->bytes) + "\n" : "ERR no such region\n")) break;
    } else if (!std::strcmp(verb, "WRITE") && fields >= 3) {
      if (!region || a < 0 || b < 0 || b > region->bytes || a > region->bytes - b) { reply(fd, "ERR range\n"); break; }
      if (!recv_all(fd, region->base + a, b)) break;
      if (!reply(fd, "OK\n")) break;
    } else if (!std::strcmp(verb, "READ") && fields >= 3) {
      if (!region || a < 0 || b < 0 || b > region->bytes || a > region->bytes - b) { reply(fd, "ERR range\n"); break; }
      if (!reply(fd, "OK " + std::to_string(b) + "\n")) break;
      if (!send_all(fd, region->base + a, b)) break;
    } else if (!std::strcmp(verb, "FREE") && fields >= 2) {
      if (a == owned) { release(owned); owned = -1; region.reset(); }
      if (!reply(fd, "OK\n")) break;
    } else if (!std::strcmp(verb, "STAT")) {
      std::lock_guard<std::mutex> lk(g_mu);
      if (!reply(fd, "OK " + std::to_string(g_regions.size()) + " " + std::to_string(g_held) + "\n")) break;
    } else {
      if (!reply(fd, "ERR unknown request\n")) break;
    }
  }
  if (owned >= 0) release(owned);     // the lease ends with the connection
  ::close(fd);
}

}  // namespace

int main(int argc, char** argv) {
  int port = 7070;
  std::string bind_to = "127.0.0.1";
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--port" && i + 1 < argc) port = std::atoi(argv[++i]);
    else if (a == "--bind" && i + 1 < argc) bind_to = argv[++i];
    else if (a == "--capacity-gib" && i + 1 < argc) g_capacity = static_cast<int64_t>(std::atof(argv[++i]) * (1ll << 30));
    else if (a == "--lock") g_lock = true;
    else { std::fprintf(stderr, "usage: ss_memory_daemon --port P [--bind ADDR] [--capacity-gib G] [--lock]\n"); return 2; }
  }
  std::signal(SIGPIPE, SIG_IGN);
  const int ls = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (ls < 0) { std::perror("socket"); return 1; }
  int one = 1;
  ::setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (::inet_pton(AF_INET, bind_to.c_str(), &addr.sin_addr) != 1) { std::fprintf(stderr, "bad --bind address\n"); return 2; }
  if (::bind(ls, reinterpret_cast<sockaddr*>(&addr), sizeof addr) != 0 || ::listen(ls, 64) != 0) {
    std::perror("bind/listen");
    return 1;
  }
  socklen_t len = sizeof addr;
  ::getsockname(ls, reinterpret_cast<sockaddr*>(&addr), &len);
  std::printf("listening %d\n", ntohs(addr.sin_port));
  std::fflush(stdout);
  for (;;) {
    const int fd = ::accept4(ls, nullptr, nullptr, SOCK_CLOEXEC);
    if (fd < 0) { if (errno == EINTR) continue; break; }
    std::thread(serve, fd).detach();
  }
  return 0;
}
