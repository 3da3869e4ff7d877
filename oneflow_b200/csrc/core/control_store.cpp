// Control plane: a TCP key-value store with counters, barriers and a heartbeat-based failure detector.
//
// One rank hosts the server (a poll() loop on one thread); every rank holds a client connection whose
// requests are serialised by a mutex. A heartbeat thread per client stamps "hb/<rank>" with the server's
// clock at a fixed interval; any client can ask which ranks have not stamped for longer than a limit, which
// is how a rank that died or stalled is noticed on the host before the next collective is launched.
// Blocking reads (get, barrier) carry a deadline and report a time-out instead of waiting forever.
//
// Plays the role of the reference's CtrlServer / CtrlClient (oneflow/core/control/ctrl_client.cpp:27-58:
// PushKV / PullKV / Barrier / IncreaseCount and the heartbeat thread that reports "Machine i lost").
//
// Wire format (little endian): request = u32 op, u32 key_len, u32 val_len, i64 arg, key bytes, value bytes;
// response = i64 status_or_value, u32 val_len, value bytes.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "common.h"
#include "ofc_core.h"

namespace {

enum Op : uint32_t { kSet = 1, kGet = 2, kAdd = 3, kStamp = 4, kAges = 5, kDel = 6, kCas = 7, kCount = 8, kHas = 9 };

int64_t now_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

bool send_all(int fd, const void* p, size_t n) {
  const char* c = static_cast<const char*>(p);
  while (n) {
    ssize_t w = ::send(fd, c, n, MSG_NOSIGNAL);
    if (w <= 0) return false;
    c += w;
    n -= static_cast<size_t>(w);
  }
  return true;
}
bool recv_all(int fd, void* p, size_t n) {
  char* c = static_cast<char*>(p);
  while (n) {
    ssize_t r = ::recv(fd, c, n, 0);
    if (r <= 0) return false;
    c += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

struct Header {
  uint32_t op, key_len, val_len;
  int64_t arg;
} __attribute__((packed));
struct RespHeader {
  int64_t status;
  uint32_t val_len;
} __attribute__((packed));

struct Server {
  int listen_fd = -1;
  int port = 0;
  int world = 0;
  std::thread th;
  std::atomic<bool> stop{false};
  std::map<std::string, std::string> kv;
  std::map<std::string, int64_t> counters;
  std::map<int64_t, int64_t> stamps;  // rank -> last heartbeat (server clock)
  int64_t start_ms = 0;

  void handle(int fd, const Header& h, const std::string& key, const std::string& val) {
    RespHeader r{0, 0};
    std::string out;
    switch (h.op) {
      case kSet: kv[key] = val; break;
      case kGet: {
        auto it = kv.find(key);
        if (it == kv.end()) r.status = -1; else out = it->second;
        break;
      }
      case kAdd: {
        // counters are visible as decimal-string values too, so that a reader of the key (the process-group
        // rendezvous reads what another rank added) sees the count
        auto it = counters.find(key);
        if (it == counters.end()) {
          auto kvit = kv.find(key);
          int64_t base = 0;
          if (kvit != kv.end()) base = std::strtoll(kvit->second.c_str(), nullptr, 10);
          it = counters.emplace(key, base).first;
        }
        r.status = (it->second += h.arg);
        kv[key] = std::to_string(it->second);
        break;
      }
      case kDel: r.status = static_cast<int64_t>(kv.erase(key)); counters.erase(key); break;
      case kCas: {
        // value = u32 length of `expected` + expected + desired. An absent key matches an empty `expected`.
        uint32_t el = 0;
        if (val.size() >= 4) std::memcpy(&el, val.data(), 4);
        if (val.size() < 4 + static_cast<size_t>(el)) { r.status = -100; break; }
        const std::string expected = val.substr(4, el), desired = val.substr(4 + el);
        auto it = kv.find(key);
        if ((it == kv.end() && expected.empty()) || (it != kv.end() && it->second == expected)) {
          kv[key] = desired;
          counters.erase(key);
          out = desired;
        } else if (it != kv.end()) {
          out = it->second;
        } else {
          out = expected;
        }
        break;
      }
      case kCount: r.status = static_cast<int64_t>(kv.size()); break;
      case kHas: r.status = kv.count(key) ? 1 : 0; break;
      case kStamp: stamps[h.arg] = now_ms(); break;
      case kAges: {
        // value = world x i64 ages in ms (time since last stamp, or since server start if never stamped)
        std::vector<int64_t> ages(static_cast<size_t>(world));
        const int64_t t = now_ms();
        for (int i = 0; i < world; ++i) {
          auto it = stamps.find(i);
          ages[static_cast<size_t>(i)] = it == stamps.end() ? -(t - start_ms) - 1 : t - it->second;
        }
        out.assign(reinterpret_cast<const char*>(ages.data()), ages.size() * sizeof(int64_t));
        break;
      }
      default: r.status = -100;
    }
    r.val_len = static_cast<uint32_t>(out.size());
    send_all(fd, &r, sizeof(r));
    if (!out.empty()) send_all(fd, out.data(), out.size());
  }

  void loop() {
    std::vector<pollfd> fds;
    fds.push_back({listen_fd, POLLIN, 0});
    while (!stop.load()) {
      int n = ::poll(fds.data(), fds.size(), 100);
      if (n <= 0) continue;
      if (fds[0].revents & POLLIN) {
        int c = ::accept(listen_fd, nullptr, nullptr);
        if (c >= 0) {
          int one = 1;
          setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
          fds.push_back({c, POLLIN, 0});
        }
      }
      for (size_t i = 1; i < fds.size();) {
        if (fds[i].revents & (POLLIN | POLLHUP | POLLERR)) {
          Header h;
          bool ok = recv_all(fds[i].fd, &h, sizeof(h));
          std::string key, val;
          if (ok && h.key_len < (1u << 20) && h.val_len < (1u << 30)) {
            key.resize(h.key_len);
            val.resize(h.val_len);
            ok = (h.key_len == 0 || recv_all(fds[i].fd, &key[0], h.key_len)) &&
                 (h.val_len == 0 || recv_all(fds[i].fd, &val[0], h.val_len));
          } else {
            ok = false;
          }
          if (!ok) {
            ::close(fds[i].fd);
            fds.erase(fds.begin() + static_cast<long>(i));
            continue;
          }
          handle(fds[i].fd, h, key, val);
        }
        ++i;
      }
    }
    for (size_t i = 1; i < fds.size(); ++i) ::close(fds[i].fd);
  }
};

struct Client {
  int fd = -1;
  int rank = 0;
  std::mutex mu;
  std::thread hb;
  std::atomic<bool> stop{false};
  int hb_interval_ms = 0;

  int64_t request(Op op, const std::string& key, const void* val, uint32_t val_len, int64_t arg, std::string* out) {
    std::lock_guard<std::mutex> g(mu);
    Header h{op, static_cast<uint32_t>(key.size()), val_len, arg};
    if (!send_all(fd, &h, sizeof(h)) || (!key.empty() && !send_all(fd, key.data(), key.size())) ||
        (val_len && !send_all(fd, val, val_len)))
      return ofc::fail("control store: connection lost while sending", -10);
    RespHeader r;
    if (!recv_all(fd, &r, sizeof(r))) return ofc::fail("control store: connection lost while receiving", -10);
    std::string v(r.val_len, '\0');
    if (r.val_len && !recv_all(fd, &v[0], r.val_len)) return ofc::fail("control store: connection lost while receiving", -10);
    if (out) *out = std::move(v);
    return r.status;
  }
};

}  // namespace

OFC_API void* ofc_store_server_start(int port, int world_size) {
  auto* s = new Server();
  s->world = world_size;
  s->listen_fd = ::socket(AF_INET, SOCK_STREAM, 0);
  int one = 1;
  setsockopt(s->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (::bind(s->listen_fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(s->listen_fd, 128) != 0) {
    ofc::fail("control store: cannot bind/listen on the requested port");
    ::close(s->listen_fd);
    delete s;
    return nullptr;
  }
  socklen_t len = sizeof(addr);
  getsockname(s->listen_fd, reinterpret_cast<sockaddr*>(&addr), &len);
  s->port = ntohs(addr.sin_port);
  s->start_ms = now_ms();
  s->th = std::thread([s] { s->loop(); });
  return s;
}
OFC_API int ofc_store_server_port(void* server) { return static_cast<Server*>(server)->port; }
OFC_API void ofc_store_server_stop(void* server) {
  auto* s = static_cast<Server*>(server);
  s->stop.store(true);
  if (s->th.joinable()) s->th.join();
  ::close(s->listen_fd);
  delete s;
}

OFC_API void* ofc_store_client_connect(const char* host, int port, int rank, int timeout_ms) {
  const int64_t deadline = now_ms() + timeout_ms;
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (inet_pton(AF_INET, host, &addr.sin_addr) != 1) {
    ofc::fail("control store: host must be a dotted IPv4 address");
    return nullptr;
  }
  while (true) {
    int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) {
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      auto* c = new Client();
      c->fd = fd;
      c->rank = rank;
      return c;
    }
    ::close(fd);
    if (now_ms() > deadline) {
      ofc::fail("control store: could not reach the server before the deadline");
      return nullptr;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(50));
  }
}
OFC_API void ofc_store_client_close(void* client) {
  auto* c = static_cast<Client*>(client);
  c->stop.store(true);
  if (c->hb.joinable()) c->hb.join();
  ::close(c->fd);
  delete c;
}
OFC_API int ofc_store_set(void* client, const char* key, const void* value, int len) {
  return static_cast<int>(static_cast<Client*>(client)->request(kSet, key, value, static_cast<uint32_t>(len), 0, nullptr));
}
OFC_API int ofc_store_get(void* client, const char* key, void* out, int cap, int timeout_ms) {
  auto* c = static_cast<Client*>(client);
  const int64_t deadline = now_ms() + timeout_ms;
  while (true) {
    std::string v;
    int64_t st = c->request(kGet, key, nullptr, 0, 0, &v);
    if (st == 0) {
      if (static_cast<int>(v.size()) > cap) return ofc::fail("control store: value larger than the caller's buffer", -3);
      std::memcpy(out, v.data(), v.size());
      return static_cast<int>(v.size());
    }
    if (st <= -10) return static_cast<int>(st);
    if (now_ms() > deadline) return ofc::fail(std::string("control store: timed out waiting for key ") + key, -2);
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
}
OFC_API int ofc_store_delete(void* client, const char* key) {
  return static_cast<int>(static_cast<Client*>(client)->request(kDel, key, nullptr, 0, 0, nullptr));
}
OFC_API int64_t ofc_store_num_keys(void* client) { return static_cast<Client*>(client)->request(kCount, "", nullptr, 0, 0, nullptr); }
OFC_API int ofc_store_has(void* client, const char* key) {
  return static_cast<int>(static_cast<Client*>(client)->request(kHas, key, nullptr, 0, 0, nullptr));
}
// Sets key to `desired` if its current value equals `expected` (an absent key equals an empty `expected`); the value
// the key holds afterwards is copied to out. Returns its length or a negative error.
OFC_API int ofc_store_compare_set(void* client, const char* key, const void* expected, int elen, const void* desired, int dlen,
                                  void* out, int cap) {
  std::string payload(4 + static_cast<size_t>(elen) + static_cast<size_t>(dlen), '\0');
  const uint32_t el = static_cast<uint32_t>(elen);
  std::memcpy(&payload[0], &el, 4);
  if (elen) std::memcpy(&payload[4], expected, static_cast<size_t>(elen));
  if (dlen) std::memcpy(&payload[4 + static_cast<size_t>(elen)], desired, static_cast<size_t>(dlen));
  std::string v;
  int64_t st = static_cast<Client*>(client)->request(kCas, key, payload.data(), static_cast<uint32_t>(payload.size()), 0, &v);
  if (st < 0) return static_cast<int>(st);
  if (static_cast<int>(v.size()) > cap) return ofc::fail("control store: value larger than the caller's buffer", -3);
  std::memcpy(out, v.data(), v.size());
  return static_cast<int>(v.size());
}
OFC_API int64_t ofc_store_add(void* client, const char* key, int64_t delta) {
  return static_cast<Client*>(client)->request(kAdd, key, nullptr, 0, delta, nullptr);
}
OFC_API int ofc_store_barrier(void* client, const char* name, int world_size, int timeout_ms) {
  auto* c = static_cast<Client*>(client);
  const std::string key = std::string("barrier/") + name;
  const int64_t arrived = c->request(kAdd, key, nullptr, 0, 1, nullptr);
  if (arrived < 0) return static_cast<int>(arrived);
  // generation = which use of this barrier name the caller belongs to
  const int64_t target = ((arrived + world_size - 1) / world_size) * world_size;
  const int64_t deadline = now_ms() + timeout_ms;
  while (true) {
    const int64_t cur = c->request(kAdd, key, nullptr, 0, 0, nullptr);
    if (cur < 0) return static_cast<int>(cur);
    if (cur >= target) return 0;
    if (now_ms() > deadline)
      return ofc::fail(std::string("control store: barrier '") + name + "' timed out: " + std::to_string(cur % world_size) + " of " +
                       std::to_string(world_size) + " ranks arrived (maybe executing different code in different ranks)", -2);
    std::this_thread::sleep_for(std::chrono::milliseconds(2));
  }
}
OFC_API int ofc_store_heartbeat_start(void* client, int interval_ms) {
  auto* c = static_cast<Client*>(client);
  if (c->hb.joinable()) return 0;
  c->hb_interval_ms = interval_ms;
  c->request(kStamp, "", nullptr, 0, c->rank, nullptr);
  c->hb = std::thread([c] {
    int64_t next = now_ms() + c->hb_interval_ms;
    while (!c->stop.load()) {
      std::this_thread::sleep_for(std::chrono::milliseconds(10));
      if (now_ms() >= next) {
        if (c->request(kStamp, "", nullptr, 0, c->rank, nullptr) < 0) return;
        next += c->hb_interval_ms;
      }
    }
  });
  return 0;
}
OFC_API int ofc_store_lost_ranks(void* client, int max_age_ms, int* lost_out, int cap) {
  std::string v;
  int64_t st = static_cast<Client*>(client)->request(kAges, "", nullptr, 0, 0, &v);
  if (st < 0) return static_cast<int>(st);
  const int64_t* ages = reinterpret_cast<const int64_t*>(v.data());
  const int n = static_cast<int>(v.size() / sizeof(int64_t));
  int lost = 0;
  for (int i = 0; i < n; ++i) {
    // negative age: never stamped; -(age) - 1 is the time since the server started
    const int64_t age = ages[i] >= 0 ? ages[i] : -(ages[i] + 1);
    if (age > max_age_ms) {
      if (lost < cap) lost_out[lost] = i;
      ++lost;
    }
  }
  return lost;
}
