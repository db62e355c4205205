// Heartbeat / quorum service for replica-group fault tolerance, and its client.
//
// One "lighthouse" per job; every replica group (a separate launcher invocation) keeps one client per rank-0.
// Wire protocol: newline-terminated text over TCP.
//   HB <replica> <step>                                   -> (no reply) liveness + progress
//   QUORUM <replica> <step> <min_replicas> <timeout_ms> <address>
//        -> OK <quorum_id> <n> <id,id,...> <addr,addr,...> <max_step> <max_step_replica>
//        -> ERR <reason>
//   STATUS                                                 -> one line of counters
// An <address> ending in '!' means "my previous cross-replica group is unusable": the quorum id is then bumped even if
// the membership is unchanged, so that every member rebuilds its group under a fresh id.
// A quorum forms when every replica that has heartbeat within `hb_timeout_ms` has asked for one, or when
// `join_timeout_ms` has passed since the first request and at least `min_replicas` have asked. Members are
// reported in ascending id order; the quorum id increases whenever the membership differs from the last one.
//
// This plays the role that the external torchft lighthouse (a separate native service) plays for
// torchtitan/experiments/ft/manager.py:91-115. Plain C ABI for ctypes; no CUDA.

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

namespace {
using Clock = std::chrono::steady_clock;
using Ms = std::chrono::milliseconds;

struct Member {
  Clock::time_point last_hb;
  long long step = 0;
  bool asking = false;
  long long ask_step = 0;
  std::string address;
  bool wants_fresh = false;
};

struct Lighthouse {
  int listen_fd = -1;
  int port = 0;
  int hb_timeout_ms = 5000;
  int join_timeout_ms = 1000;
  std::atomic<bool> stop{false};
  std::thread acceptor;
  std::vector<std::thread> workers;
  std::mutex mu;
  std::condition_variable cv;
  std::map<std::string, Member> members;
  Clock::time_point first_ask{};
  bool any_ask = false;
  long long quorum_id = 0;
  long long generation = 0;        // bumps every time a quorum is published
  std::string last_members;
  std::string published;           // reply line of the latest quorum
  std::vector<std::string> published_ids;
  long long n_quorums = 0, n_heartbeats = 0;
};

bool send_all(int fd, const std::string& s) {
  size_t off = 0;
  while (off < s.size()) {
    ssize_t n = ::send(fd, s.data() + off, s.size() - off, MSG_NOSIGNAL);
    if (n <= 0) return false;
    off += size_t(n);
  }
  return true;
}

// reads one line (without '\n'); false on EOF / error / timeout
bool read_line(int fd, std::string& line, std::string& pending) {
  for (;;) {
    auto pos = pending.find('\n');
    if (pos != std::string::npos) {
      line = pending.substr(0, pos);
      pending.erase(0, pos + 1);
      return true;
    }
    char buf[1024];
    ssize_t n = ::recv(fd, buf, sizeof buf, 0);
    if (n <= 0) return false;
    pending.append(buf, size_t(n));
  }
}

// caller holds lh.mu
bool try_form(Lighthouse& lh, int min_replicas) {
  auto now = Clock::now();
  std::vector<std::string> alive, asking;
  for (auto& kv : lh.members) {
    bool live = now - kv.second.last_hb <= Ms(lh.hb_timeout_ms);
    if (live) alive.push_back(kv.first);
    if (live && kv.second.asking) asking.push_back(kv.first);
  }
  if (asking.empty() || int(asking.size()) < min_replicas) return false;
  bool everyone = asking.size() == alive.size();
  bool waited = lh.any_ask && now - lh.first_ask >= Ms(lh.join_timeout_ms);
  if (!everyone && !waited) return false;
  std::string ids, addrs, best;
  long long max_step = -1;
  bool fresh = false;
  for (auto& id : asking) {   // std::map iteration => ascending ids
    auto& m = lh.members[id];
    fresh = fresh || m.wants_fresh;
    m.wants_fresh = false;
    ids += (ids.empty() ? "" : ",") + id;
    addrs += (addrs.empty() ? "" : ",") + (m.address.empty() ? std::string("-") : m.address);
    if (m.ask_step > max_step) { max_step = m.ask_step; best = id; }
    m.asking = false;
  }
  if (ids != lh.last_members || fresh) { lh.quorum_id++; lh.last_members = ids; }
  std::ostringstream os;
  os << "OK " << lh.quorum_id << " " << asking.size() << " " << ids << " " << addrs << " " << max_step << " " << best << "\n";
  lh.published = os.str();
  lh.published_ids = asking;
  lh.generation++;
  lh.n_quorums++;
  lh.any_ask = false;
  return true;
}

void serve(Lighthouse* lh, int fd) {
  std::string pending, line;
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
  while (!lh->stop.load() && read_line(fd, line, pending)) {
    std::istringstream is(line);
    std::string cmd;
    is >> cmd;
    if (cmd == "HB") {
      std::string id; long long step = 0;
      is >> id >> step;
      std::lock_guard<std::mutex> g(lh->mu);
      auto& m = lh->members[id];
      m.last_hb = Clock::now();
      m.step = step;
      lh->n_heartbeats++;
      lh->cv.notify_all();
    } else if (cmd == "QUORUM") {
      std::string id, addr; long long step = 0; int min_rep = 1; int timeout_ms = 10000;
      is >> id >> step >> min_rep >> timeout_ms >> addr;
      std::unique_lock<std::mutex> g(lh->mu);
      auto& m = lh->members[id];
      m.last_hb = Clock::now();
      bool fresh = !addr.empty() && addr.back() == '!';
      if (fresh) addr.pop_back();
      m.asking = true; m.ask_step = step; m.step = step; m.address = addr; m.wants_fresh = fresh;
      if (!lh->any_ask) { lh->any_ask = true; lh->first_ask = Clock::now(); }
      long long gen0 = lh->generation;
      auto deadline = Clock::now() + Ms(timeout_ms);
      std::string reply;
      for (;;) {
        if (lh->generation != gen0 &&
            std::find(lh->published_ids.begin(), lh->published_ids.end(), id) != lh->published_ids.end()) {
          reply = lh->published; break;
        }
        if (lh->generation != gen0) gen0 = lh->generation;   // a quorum formed without us: keep waiting for the next
        if (lh->members[id].asking && try_form(*lh, min_rep)) { lh->cv.notify_all(); continue; }
        if (lh->stop.load()) { reply = "ERR stopped\n"; break; }
        if (Clock::now() >= deadline) { lh->members[id].asking = false; reply = "ERR timeout\n"; break; }
        lh->members[id].last_hb = Clock::now();   // a replica blocked in QUORUM is alive
        lh->cv.wait_for(g, Ms(50));
      }
      g.unlock();
      if (!send_all(fd, reply)) break;
    } else if (cmd == "STATUS") {
      std::ostringstream os;
      {
        std::lock_guard<std::mutex> g(lh->mu);
        auto now = Clock::now();
        int alive = 0;
        for (auto& kv : lh->members) alive += (now - kv.second.last_hb <= Ms(lh->hb_timeout_ms));
        os << "STATUS members=" << lh->members.size() << " alive=" << alive << " quorum_id=" << lh->quorum_id
           << " quorums=" << lh->n_quorums << " heartbeats=" << lh->n_heartbeats << "\n";
      }
      if (!send_all(fd, os.str())) break;
    } else {
      if (!send_all(fd, "ERR unknown command\n")) break;
    }
  }
  ::close(fd);
}

struct Client {
  int fd = -1;
  std::string pending;
  std::mutex mu;                 // one request at a time on the command socket
  // heartbeat thread has its own socket
  int hb_fd = -1;
  std::thread hb;
  std::atomic<bool> hb_stop{false};
  std::atomic<long long> step{0};
  std::atomic<bool> hb_paused{false};
  std::string id;
};

int dial(const char* host, int port, int timeout_ms) {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons(uint16_t(port));
  if (inet_pton(AF_INET, host, &a.sin_addr) != 1) { ::close(fd); return -1; }
  timeval tv{timeout_ms / 1000, (timeout_ms % 1000) * 1000};
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
  if (::connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof a) != 0) { ::close(fd); return -1; }
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
  return fd;
}
}  // namespace

extern "C" {

// ---- server ------------------------------------------------------------------------------------------
void* tt_lighthouse_start(int port, int hb_timeout_ms, int join_timeout_ms) {
  auto* lh = new Lighthouse();
  lh->hb_timeout_ms = hb_timeout_ms;
  lh->join_timeout_ms = join_timeout_ms;
  lh->listen_fd = ::socket(AF_INET, SOCK_STREAM, 0);
  int one = 1;
  setsockopt(lh->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_addr.s_addr = htonl(INADDR_ANY);
  a.sin_port = htons(uint16_t(port));
  if (::bind(lh->listen_fd, reinterpret_cast<sockaddr*>(&a), sizeof a) != 0 || ::listen(lh->listen_fd, 128) != 0) {
    ::close(lh->listen_fd);
    delete lh;
    return nullptr;
  }
  socklen_t len = sizeof a;
  getsockname(lh->listen_fd, reinterpret_cast<sockaddr*>(&a), &len);
  lh->port = ntohs(a.sin_port);
  lh->acceptor = std::thread([lh] {
    while (!lh->stop.load()) {
      int fd = ::accept(lh->listen_fd, nullptr, nullptr);
      if (fd < 0) break;
      std::lock_guard<std::mutex> g(lh->mu);
      lh->workers.emplace_back(serve, lh, fd);
    }
  });
  return lh;
}

int tt_lighthouse_port(void* h) { return h ? static_cast<Lighthouse*>(h)->port : -1; }

void tt_lighthouse_stop(void* h) {
  if (!h) return;
  auto* lh = static_cast<Lighthouse*>(h);
  lh->stop.store(true);
  ::shutdown(lh->listen_fd, SHUT_RDWR);
  ::close(lh->listen_fd);
  { std::lock_guard<std::mutex> g(lh->mu); lh->cv.notify_all(); }
  if (lh->acceptor.joinable()) lh->acceptor.join();
  // workers exit when their peers close; detach so that stop never blocks on a silent client
  std::vector<std::thread> ws;
  { std::lock_guard<std::mutex> g(lh->mu); ws.swap(lh->workers); }
  for (auto& t : ws) t.detach();
  // the object is leaked on purpose: detached workers may still touch it
}

// ---- client ------------------------------------------------------------------------------------------
void* tt_ft_connect(const char* host, int port, const char* replica_id, int heartbeat_interval_ms) {
  auto* c = new Client();
  c->id = replica_id;
  c->fd = dial(host, port, 5000);
  c->hb_fd = heartbeat_interval_ms > 0 ? dial(host, port, 5000) : -1;
  if (c->fd < 0 || (heartbeat_interval_ms > 0 && c->hb_fd < 0)) {
    if (c->fd >= 0) ::close(c->fd);
    if (c->hb_fd >= 0) ::close(c->hb_fd);
    delete c;
    return nullptr;
  }
  if (heartbeat_interval_ms > 0) {
    c->hb = std::thread([c, heartbeat_interval_ms] {
      while (!c->hb_stop.load()) {
        if (!c->hb_paused.load()) {
          std::string msg = "HB " + c->id + " " + std::to_string(c->step.load()) + "\n";
          if (!send_all(c->hb_fd, msg)) break;
        }
        for (int waited = 0; waited < heartbeat_interval_ms && !c->hb_stop.load(); waited += 10)
          std::this_thread::sleep_for(Ms(10));
      }
    });
  }
  return c;
}

void tt_ft_set_step(void* h, long long step) { static_cast<Client*>(h)->step.store(step); }

// test hook: a paused client stops sending heartbeats (a "silent" replica) without exiting
void tt_ft_pause_heartbeat(void* h, int paused) { static_cast<Client*>(h)->hb_paused.store(paused != 0); }

// Blocks until a quorum containing this replica forms. Writes the reply line (without '\n') to `out`.
// Returns 0 on OK, 1 on ERR reply, -1 on connection failure.
int tt_ft_quorum(void* h, long long step, int min_replicas, int timeout_ms, const char* address, char* out, int out_len) {
  auto* c = static_cast<Client*>(h);
  std::lock_guard<std::mutex> g(c->mu);
  c->step.store(step);
  std::string addr = (address && *address) ? address : "-";
  std::string msg = "QUORUM " + c->id + " " + std::to_string(step) + " " + std::to_string(min_replicas) + " " +
                    std::to_string(timeout_ms) + " " + addr + "\n";
  if (!send_all(c->fd, msg)) return -1;
  timeval tv{(timeout_ms + 2000) / 1000, ((timeout_ms + 2000) % 1000) * 1000};
  setsockopt(c->fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  std::string line;
  if (!read_line(c->fd, line, c->pending)) return -1;
  std::snprintf(out, size_t(out_len), "%s", line.c_str());
  return line.rfind("OK", 0) == 0 ? 0 : 1;
}

int tt_ft_status(void* h, char* out, int out_len) {
  auto* c = static_cast<Client*>(h);
  std::lock_guard<std::mutex> g(c->mu);
  if (!send_all(c->fd, "STATUS\n")) return -1;
  std::string line;
  if (!read_line(c->fd, line, c->pending)) return -1;
  std::snprintf(out, size_t(out_len), "%s", line.c_str());
  return 0;
}

void tt_ft_close(void* h) {
  if (!h) return;
  auto* c = static_cast<Client*>(h);
  c->hb_stop.store(true);
  if (c->hb.joinable()) c->hb.join();
  if (c->hb_fd >= 0) ::close(c->hb_fd);
  if (c->fd >= 0) ::close(c->fd);
  delete c;
}

}  // extern "C"
