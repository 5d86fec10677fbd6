// Experiment store: a small in-memory key/value + list server that the processes of one experiment
// (trainers, generation workers, router, evaluation workers) use to find each other and to pass work.
// It plays the role the reference gives to a spawned redis-server
// (steptronoss/utils/comm_utils.py:33-250): strings, counters, lists with push/pop at both ends,
// scored sets for load balancing, prefix key listing and expiry.
//
// Wire format (little endian), request:  u32 body_len | u8 op | u32 klen | key | payload
//                              response: u32 body_len | u8 status (0 ok, 1 nil, 2 error) | payload
// One epoll loop, non-blocking sockets, no threads: every command is atomic with respect to the others,
// which is what the queue and balance operations rely on.
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/epoll.h>
#include <sys/socket.h>
#include <time.h>
#include <unistd.h>

#include <deque>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

enum Op : uint8_t {
  kPing = 0, kSet = 1, kGet = 2, kDel = 3, kIncr = 4, kLPush = 5, kRPush = 6, kLPop = 7, kRPop = 8,
  kLLen = 9, kKeys = 10, kSetNx = 11, kExpire = 12, kZAdd = 13, kZIncr = 14, kZPopMinIncr = 15,
  kShutdown = 16, kLRange = 17,
};

struct Conn {
  int fd = -1;
  std::string in, out;
};

std::unordered_map<std::string, std::string> g_strings;
std::unordered_map<std::string, std::deque<std::string>> g_lists;
std::unordered_map<std::string, std::map<std::string, double>> g_zsets;
std::unordered_map<std::string, double> g_expiry;  // key -> absolute monotonic seconds
bool g_stop = false;

double now_s() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}

void erase_key(const std::string& k) {
  g_strings.erase(k);
  g_lists.erase(k);
  g_zsets.erase(k);
  g_expiry.erase(k);
}

void expire_if_due(const std::string& k) {
  auto it = g_expiry.find(k);
  if (it != g_expiry.end() && it->second <= now_s()) erase_key(k);
}

void reply(Conn& c, uint8_t status, const std::string& payload = std::string()) {
  uint32_t len = static_cast<uint32_t>(payload.size() + 1);
  c.out.append(reinterpret_cast<const char*>(&len), 4);
  c.out.push_back(static_cast<char>(status));
  c.out.append(payload);
}

std::string i64(int64_t v) { return std::string(reinterpret_cast<const char*>(&v), 8); }

void handle(Conn& c, uint8_t op, const std::string& key, const std::string& val) {
  expire_if_due(key);
  switch (op) {
    case kPing: reply(c, 0, "PONG"); break;
    case kSet: g_strings[key] = val; reply(c, 0); break;
    case kSetNx:
      if (g_strings.count(key)) reply(c, 1);
      else { g_strings[key] = val; reply(c, 0); }
      break;
    case kGet: {
      auto it = g_strings.find(key);
      if (it == g_strings.end()) reply(c, 1); else reply(c, 0, it->second);
      break;
    }
    case kDel: {
      const bool had = g_strings.count(key) || g_lists.count(key) || g_zsets.count(key);
      erase_key(key);
      reply(c, had ? 0 : 1);
      break;
    }
    case kIncr: {
      int64_t delta = 1;
      if (val.size() == 8) memcpy(&delta, val.data(), 8);
      int64_t cur = 0;
      auto it = g_strings.find(key);
      if (it != g_strings.end()) cur = strtoll(it->second.c_str(), nullptr, 10);
      cur += delta;
      g_strings[key] = std::to_string(cur);
      reply(c, 0, i64(cur));
      break;
    }
    case kLPush: case kRPush: {
      auto& q = g_lists[key];
      if (op == kLPush) q.push_front(val); else q.push_back(val);
      reply(c, 0, i64(static_cast<int64_t>(q.size())));
      break;
    }
    case kLPop: case kRPop: {
      auto it = g_lists.find(key);
      if (it == g_lists.end() || it->second.empty()) { reply(c, 1); break; }
      std::string v;
      if (op == kLPop) { v = std::move(it->second.front()); it->second.pop_front(); }
      else { v = std::move(it->second.back()); it->second.pop_back(); }
      if (it->second.empty()) g_lists.erase(it);
      reply(c, 0, v);
      break;
    }
    case kLLen: {
      auto it = g_lists.find(key);
      reply(c, 0, i64(it == g_lists.end() ? 0 : static_cast<int64_t>(it->second.size())));
      break;
    }
    case kLRange: {  // whole list, elements length-prefixed
      std::string out;
      auto it = g_lists.find(key);
      if (it != g_lists.end())
        for (const auto& e : it->second) {
          uint32_t n = static_cast<uint32_t>(e.size());
          out.append(reinterpret_cast<const char*>(&n), 4);
          out.append(e);
        }
      reply(c, 0, out);
      break;
    }
    case kKeys: {  // keys starting with `key`, newline separated
      std::string out;
      const double t = now_s();
      auto add = [&](const std::string& k) {
        auto e = g_expiry.find(k);
        if (e != g_expiry.end() && e->second <= t) return;
        if (k.compare(0, key.size(), key) == 0) { out.append(k); out.push_back('\n'); }
      };
      for (const auto& kv : g_strings) add(kv.first);
      for (const auto& kv : g_lists) add(kv.first);
      for (const auto& kv : g_zsets) add(kv.first);
      reply(c, 0, out);
      break;
    }
    case kExpire: {
      double secs = 0;
      if (val.size() == 8) memcpy(&secs, val.data(), 8);
      g_expiry[key] = now_s() + secs;
      reply(c, 0);
      break;
    }
    case kZAdd: case kZIncr: {  // payload: f64 score | member
      if (val.size() < 8) { reply(c, 2, "short zset payload"); break; }
      double score;
      memcpy(&score, val.data(), 8);
      const std::string member = val.substr(8);
      auto& z = g_zsets[key];
      if (op == kZAdd) { if (!z.count(member)) z[member] = score; } else z[member] += score;
      reply(c, 0);
      break;
    }
    case kZPopMinIncr: {  // member with the lowest score gets +1 and is returned (least-loaded sub-queue)
      auto it = g_zsets.find(key);
      if (it == g_zsets.end() || it->second.empty()) { reply(c, 1); break; }
      auto best = it->second.begin();
      for (auto m = it->second.begin(); m != it->second.end(); ++m)
        if (m->second < best->second) best = m;
      best->second += 1.0;
      reply(c, 0, best->first);
      break;
    }
    case kShutdown: reply(c, 0); g_stop = true; break;
    default: reply(c, 2, "unknown op");
  }
}

// Consume complete frames from c.in. Returns false on a malformed frame.
bool drain(Conn& c) {
  size_t off = 0;
  while (c.in.size() - off >= 4) {
    uint32_t len;
    memcpy(&len, c.in.data() + off, 4);
    if (len < 5 || len > (1u << 30)) return false;
    if (c.in.size() - off - 4 < len) break;
    const char* p = c.in.data() + off + 4;
    const uint8_t op = static_cast<uint8_t>(p[0]);
    uint32_t klen;
    memcpy(&klen, p + 1, 4);
    if (klen > len - 5) return false;
    handle(c, op, std::string(p + 5, klen), std::string(p + 5 + klen, len - 5 - klen));
    off += 4 + len;
  }
  c.in.erase(0, off);
  return true;
}

void set_nonblock(int fd) { fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK); }

}  // namespace

int main(int argc, char** argv) {
  int port = argc > 1 ? atoi(argv[1]) : 0;
  signal(SIGPIPE, SIG_IGN);
  int lfd = socket(AF_INET, SOCK_STREAM, 0);
  int one = 1;
  setsockopt(lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (bind(lfd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || listen(lfd, 512) != 0) {
    perror("expstore: bind/listen");
    return 1;
  }
  socklen_t alen = sizeof(addr);
  getsockname(lfd, reinterpret_cast<sockaddr*>(&addr), &alen);
  printf("EXPSTORE_PORT %d\n", ntohs(addr.sin_port));  // the parent reads the port from this line
  fflush(stdout);
  set_nonblock(lfd);
  int ep = epoll_create1(0);
  epoll_event ev{};
  ev.events = EPOLLIN;
  ev.data.fd = lfd;
  epoll_ctl(ep, EPOLL_CTL_ADD, lfd, &ev);
  std::unordered_map<int, Conn> conns;
  std::vector<epoll_event> events(256);
  const pid_t parent = getppid();
  while (!g_stop) {
    int n = epoll_wait(ep, events.data(), static_cast<int>(events.size()), 1000);
    if (n < 0 && errno != EINTR) break;
    if (getppid() != parent) break;  // the process that started the store is gone
    for (int i = 0; i < n; ++i) {
      const int fd = events[i].data.fd;
      if (fd == lfd) {
        for (;;) {
          int cfd = accept(lfd, nullptr, nullptr);
          if (cfd < 0) break;
          set_nonblock(cfd);
          setsockopt(cfd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
          epoll_event cev{};
          cev.events = EPOLLIN;
          cev.data.fd = cfd;
          epoll_ctl(ep, EPOLL_CTL_ADD, cfd, &cev);
          conns[cfd].fd = cfd;
        }
        continue;
      }
      Conn& c = conns[fd];
      bool alive = true;
      if (events[i].events & (EPOLLHUP | EPOLLERR)) alive = false;
      if (alive && (events[i].events & EPOLLIN)) {
        char buf[65536];
        for (;;) {
          ssize_t r = read(fd, buf, sizeof(buf));
          if (r > 0) c.in.append(buf, static_cast<size_t>(r));
          else if (r == 0) { alive = false; break; }
          else { if (errno != EAGAIN && errno != EWOULDBLOCK) alive = false; break; }
        }
        if (alive && !drain(c)) alive = false;
      }
      if (alive && !c.out.empty()) {
        ssize_t w = write(fd, c.out.data(), c.out.size());
        if (w > 0) c.out.erase(0, static_cast<size_t>(w));
        else if (w < 0 && errno != EAGAIN && errno != EWOULDBLOCK) alive = false;
        epoll_event mev{};
        mev.events = EPOLLIN | (c.out.empty() ? 0 : EPOLLOUT);
        mev.data.fd = fd;
        epoll_ctl(ep, EPOLL_CTL_MOD, fd, &mev);
      }
      if (!alive) {
        epoll_ctl(ep, EPOLL_CTL_DEL, fd, nullptr);
        close(fd);
        conns.erase(fd);
      }
    }
  }
  for (auto& kv : conns) close(kv.first);
  close(lfd);
  return 0;
}
