// hmp2pd — the transport daemon of hivemind_b200 (single-threaded epoll event loop, C++17).
//
// It plays the part that the external Go `p2pd` (go-libp2p-daemon) plays for the reference
// (spawned at hivemind/p2p/p2p_daemon.py:205-262, driven through hivemind/p2p/p2p_daemon_bindings/control.py):
//   * a control socket (unix) for local clients: IDENTIFY, CONNECT, LIST_PEERS, DISCONNECT,
//     STREAM_OPEN, STREAM_HANDLER (optionally balanced between several clients), REMOVE_STREAM_HANDLER and
//     a PERSISTENT upgrade that multiplexes unary calls (add/remove handler, call, response, cancel)
//     keyed by a 16-byte call id;
//   * a peer listener (TCP or unix) for other daemons: one persistent connection per peer carries unary
//     requests/responses/cancels and address gossip; every stream gets a connection of its own whose bytes
//     are spliced between the two local clients, so the kernel provides flow control;
//   * an address book filled by CONNECT, by handshakes and by gossip, with a WHO-HAS query to connected
//     peers for ids it has never seen (the reference relies on libp2p peer routing for this).
// Not provided (one box, trusted network): encryption, NAT traversal, relays, QUIC.
//
// Framing on control and persistent peer connections: u32 big-endian length, u8 type, body.
// Body fields: blob = u32 length + bytes; list = u32 count + items.
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/epoll.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

constexpr uint32_t MAX_FRAME = 64u << 20;
constexpr size_t SPLICE_HIGH_WATER = 4u << 20;  // stop reading a stream side while this much is queued for its partner

enum MsgType : uint8_t {
  // client -> daemon (first frame of a control connection)
  C_IDENTIFY = 1, C_CONNECT = 2, C_LIST_PEERS = 3, C_DISCONNECT = 4, C_PERSISTENT = 5, C_STREAM_OPEN = 6,
  C_STREAM_HANDLER = 7, C_REMOVE_STREAM_HANDLER = 8,
  // replies
  REPLY_OK = 20, REPLY_ERR = 21,
  // persistent control channel
  P_ADD_UNARY_HANDLER = 30, P_REMOVE_UNARY_HANDLER = 31, P_CALL_UNARY = 32, P_UNARY_RESPONSE = 33, P_CANCEL = 34,
  P_REQUEST = 35, P_RESPONSE = 36, P_ACK = 37,
  // daemon <-> daemon
  D_HELLO = 50, D_UNARY_REQ = 51, D_UNARY_RESP = 52, D_CANCEL = 53, D_ADDRS = 54, D_WHOHAS = 55, D_WHOHAS_REPLY = 56,
  S_OK = 60, S_ERR = 61, S_INFO = 62,
};

double now_s() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}

struct Writer {
  std::string buf;
  explicit Writer(uint8_t type) { buf.assign(5, '\0'); buf[4] = (char)type; }
  void u8(uint8_t v) { buf.push_back((char)v); }
  void u32(uint32_t v) { uint32_t be = htonl(v); buf.append((const char*)&be, 4); }
  void blob(const std::string& s) { u32((uint32_t)s.size()); buf.append(s); }
  std::string finish() {
    uint32_t be = htonl((uint32_t)(buf.size() - 4));
    memcpy(&buf[0], &be, 4);
    return std::move(buf);
  }
};

struct Reader {
  const char* p;
  const char* end;
  bool ok = true;
  Reader(const char* b, size_t n) : p(b), end(b + n) {}
  uint8_t u8() { if (end - p < 1) { ok = false; return 0; } return (uint8_t)*p++; }
  uint32_t u32() { if (end - p < 4) { ok = false; return 0; } uint32_t be; memcpy(&be, p, 4); p += 4; return ntohl(be); }
  std::string blob() {
    uint32_t n = u32();
    if (!ok || (size_t)(end - p) < n) { ok = false; return {}; }
    std::string s(p, n);
    p += n;
    return s;
  }
};

enum class Kind {
  LISTEN_CONTROL, LISTEN_PEER,
  CONTROL,        // local client, frame protocol (before classification or one-shot command)
  PERSISTENT,     // local client after C_PERSISTENT
  PEER_IN,        // inbound daemon connection, waiting for D_HELLO
  PEER,           // persistent daemon <-> daemon link
  STREAM_WAIT,    // outbound stream connection waiting for S_OK / S_ERR from the remote daemon
  SPLICE,         // raw byte pipe with a partner
};

struct Conn {
  uint64_t id = 0;
  int fd = -1;
  Kind kind = Kind::CONTROL;
  bool connecting = false;
  bool rd_closed = false, wr_shutdown_pending = false, wr_closed = false;
  bool read_paused = false;
  std::string in;
  std::string out;
  size_t out_off = 0;
  uint64_t partner = 0;          // SPLICE / STREAM_WAIT: the other side
  std::string peer_id;           // PEER: remote daemon id
  std::string pending_hello;     // bytes to send right after connect
  std::vector<std::string> protos;  // STREAM_WAIT: requested protocols
};

struct StreamHandler { std::string listen_path; bool balanced; };
struct UnaryHandler { uint64_t client; bool balanced; };
struct OutCall { uint64_t client; uint64_t peer_conn; };
struct InCall { uint64_t peer_conn; uint64_t client; };
struct Parked { std::string peer_id; std::string frame; uint64_t client; std::string call_id; double deadline; };
struct ParkedStream { uint64_t client; std::string peer_id; std::vector<std::string> protos; double deadline; };

struct Daemon {
  int ep = -1;
  uint64_t next_id = 1;
  std::unordered_map<uint64_t, std::unique_ptr<Conn>> conns;
  std::unordered_map<int, uint64_t> by_fd;
  std::string peer_id;
  std::vector<std::string> listen_addrs;
  std::map<std::string, std::set<std::string>> addr_book;          // peer id -> addresses
  std::map<std::string, uint64_t> peer_links;                      // peer id -> PEER conn
  std::map<std::string, std::vector<StreamHandler>> stream_handlers;  // protocol -> handlers
  std::map<std::string, size_t> stream_rr;
  std::map<std::string, std::vector<UnaryHandler>> unary_handlers;
  std::map<std::string, size_t> unary_rr;
  std::map<std::string, OutCall> out_calls;                         // call id -> origin client / link
  std::map<std::string, InCall> in_calls;                           // call id -> requesting link / serving client
  std::deque<Parked> parked;                                        // frames waiting for an address
  std::deque<ParkedStream> parked_streams;                          // stream opens waiting for an address
  bool verbose = false;

  // ---------------------------------------------------------------- fd plumbing
  static void set_nonblock(int fd) { fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK); }

  Conn* add(int fd, Kind kind) {
    auto c = std::make_unique<Conn>();
    c->id = next_id++;
    c->fd = fd;
    c->kind = kind;
    set_nonblock(fd);
    int sockbuf = 4 << 20;  // large tensors move through these sockets: ask for deep kernel buffers (best effort)
    setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &sockbuf, sizeof(sockbuf));
    setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &sockbuf, sizeof(sockbuf));
    epoll_event ev{};
    ev.events = EPOLLIN;
    ev.data.u64 = c->id;
    epoll_ctl(ep, EPOLL_CTL_ADD, fd, &ev);
    by_fd[fd] = c->id;
    Conn* raw = c.get();
    conns[raw->id] = std::move(c);
    return raw;
  }
  Conn* get(uint64_t id) {
    auto it = conns.find(id);
    return it == conns.end() ? nullptr : it->second.get();
  }
  void rearm(Conn* c) {
    epoll_event ev{};
    ev.events = 0;
    if (!c->rd_closed && !c->read_paused && !c->connecting) ev.events |= EPOLLIN;
    if (c->connecting || c->out_off < c->out.size()) ev.events |= EPOLLOUT;
    ev.data.u64 = c->id;
    epoll_ctl(ep, EPOLL_CTL_MOD, c->fd, &ev);
  }
  void send_bytes(Conn* c, const std::string& data) { send_raw(c, data.data(), data.size()); }
  // Queue bytes for a connection. With an empty queue the bytes go straight to the socket and only what the kernel
  // did not take is copied into the queue (the common case for spliced streams moving large tensors).
  void send_raw(Conn* c, const char* data, size_t len) {
    if (c->wr_closed) return;
    if (c->out_off > 0 && c->out_off == c->out.size()) { c->out.clear(); c->out_off = 0; }
    if (!c->connecting && c->out_off == c->out.size()) {
      while (len > 0) {
        ssize_t n = ::send(c->fd, data, len, MSG_NOSIGNAL);
        if (n > 0) { data += n; len -= (size_t)n; continue; }
        if (n < 0 && errno == EINTR) continue;
        if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) break;
        close_conn(c->id, "send failed");
        return;
      }
      if (len == 0) return;
    }
    c->out.append(data, len);
    if (!c->connecting) flush(c);
    else rearm(c);
  }
  void flush(Conn* c) {
    while (c->out_off < c->out.size()) {
      ssize_t n = ::send(c->fd, c->out.data() + c->out_off, c->out.size() - c->out_off, MSG_NOSIGNAL);
      if (n > 0) { c->out_off += (size_t)n; continue; }
      if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) break;
      if (n < 0 && errno == EINTR) continue;
      close_conn(c->id, "send failed");
      return;
    }
    if (c->out_off == c->out.size()) {
      c->out.clear();
      c->out_off = 0;
      if (c->wr_shutdown_pending && !c->wr_closed) {
        ::shutdown(c->fd, SHUT_WR);
        c->wr_closed = true;
        if (c->rd_closed) { close_conn(c->id, "both directions finished"); return; }
      }
    }
    // back-pressure for spliced streams: resume the partner's reads once our queue has drained
    if (c->kind == Kind::SPLICE) {
      Conn* p = get(c->partner);
      if (p && p->read_paused && c->out.size() - c->out_off < SPLICE_HIGH_WATER / 2) {
        p->read_paused = false;
        rearm(p);
      }
    }
    rearm(c);
  }

  void close_conn(uint64_t id, const char* why) {
    auto it = conns.find(id);
    if (it == conns.end()) return;
    std::unique_ptr<Conn> c = std::move(it->second);
    conns.erase(it);
    if (verbose) fprintf(stderr, "[hmp2pd] close conn %llu kind %d: %s\n", (unsigned long long)id, (int)c->kind, why);
    epoll_ctl(ep, EPOLL_CTL_DEL, c->fd, nullptr);
    by_fd.erase(c->fd);
    ::close(c->fd);
    if (c->kind == Kind::SPLICE || c->kind == Kind::STREAM_WAIT) {
      Conn* p = get(c->partner);
      if (p) {
        p->partner = 0;
        if (p->kind == Kind::SPLICE) {
          // let queued bytes drain, then finish the partner's write side
          const uint64_t partner_id = p->id;
          p->wr_shutdown_pending = true;
          p->rd_closed = true;
          flush(p);
          // if the partner's write side had been finished earlier (its stream had already sent EOF), flush() has
          // nothing left to trigger on: close it here, so that the far end learns that nobody reads any more
          Conn* q = get(partner_id);
          if (q && q->wr_closed && q->out_off == q->out.size()) close_conn(partner_id, "stream partner closed");
        } else {
          close_conn(p->id, "stream partner closed");
        }
      }
    } else if (c->kind == Kind::PEER) {
      auto pl = peer_links.find(c->peer_id);
      if (pl != peer_links.end() && pl->second == id) peer_links.erase(pl);
      // fail calls that were routed through this link
      for (auto oc = out_calls.begin(); oc != out_calls.end();) {
        if (oc->second.peer_conn == id) {
          respond_to_client(oc->second.client, oc->first, true, "connection to the peer was lost");
          oc = out_calls.erase(oc);
        } else ++oc;
      }
      for (auto ic = in_calls.begin(); ic != in_calls.end();) {
        if (ic->second.peer_conn == id) {
          Conn* cl = get(ic->second.client);
          if (cl) { Writer w(P_CANCEL); w.blob(ic->first); send_bytes(cl, w.finish()); }
          ic = in_calls.erase(ic);
        } else ++ic;
      }
    } else if (c->kind == Kind::PERSISTENT) {
      for (auto& kv : unary_handlers) {
        auto& v = kv.second;
        for (size_t i = 0; i < v.size();) { if (v[i].client == id) v.erase(v.begin() + i); else ++i; }
      }
      for (auto ic = in_calls.begin(); ic != in_calls.end();) {
        if (ic->second.client == id) {
          Conn* link = get(ic->second.peer_conn);
          if (link) { Writer w(D_UNARY_RESP); w.blob(ic->first); w.u8(1); w.blob("handler process went away"); send_bytes(link, w.finish()); }
          ic = in_calls.erase(ic);
        } else ++ic;
      }
      for (auto oc = out_calls.begin(); oc != out_calls.end();) {
        if (oc->second.client == id) {
          Conn* link = get(oc->second.peer_conn);
          if (link) { Writer w(D_CANCEL); w.blob(oc->first); send_bytes(link, w.finish()); }
          oc = out_calls.erase(oc);
        } else ++oc;
      }
    }
  }

  // ---------------------------------------------------------------- addresses
  static bool parse_addr(const std::string& maddr, sockaddr_storage& ss, socklen_t& len) {
    // "/ip4/A.B.C.D/tcp/PORT[/p2p/ID]" or "/unix/PATH"
    if (maddr.rfind("/unix/", 0) == 0) {
      auto* un = (sockaddr_un*)&ss;
      memset(un, 0, sizeof(*un));
      un->sun_family = AF_UNIX;
      std::string path = maddr.substr(5);
      size_t cut = path.find("/p2p/");
      if (cut != std::string::npos) path = path.substr(0, cut);
      if (path.size() >= sizeof(un->sun_path)) return false;
      strcpy(un->sun_path, path.c_str());
      len = sizeof(sockaddr_un);
      return true;
    }
    if (maddr.rfind("/ip4/", 0) == 0) {
      size_t a = 5, b = maddr.find('/', a);
      if (b == std::string::npos) return false;
      std::string host = maddr.substr(a, b - a);
      if (maddr.compare(b, 5, "/tcp/") != 0) return false;
      size_t c = b + 5, d = maddr.find('/', c);
      int port = atoi(maddr.substr(c, d == std::string::npos ? std::string::npos : d - c).c_str());
      auto* in = (sockaddr_in*)&ss;
      memset(in, 0, sizeof(*in));
      in->sin_family = AF_INET;
      in->sin_port = htons((uint16_t)port);
      if (host == "0.0.0.0") host = "127.0.0.1";
      if (inet_pton(AF_INET, host.c_str(), &in->sin_addr) != 1) return false;
      len = sizeof(sockaddr_in);
      return true;
    }
    return false;
  }

  int start_connect(const std::string& maddr, bool& in_progress) {
    sockaddr_storage ss;
    socklen_t len;
    if (!parse_addr(maddr, ss, len)) return -1;
    int fd = ::socket(ss.ss_family, SOCK_STREAM, 0);
    if (fd < 0) return -1;
    set_nonblock(fd);
    if (ss.ss_family == AF_INET) { int one = 1; setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one)); }
    int rc = ::connect(fd, (sockaddr*)&ss, len);
    in_progress = false;
    if (rc < 0) {
      if (errno == EINPROGRESS || errno == EAGAIN) in_progress = true;
      else { ::close(fd); return -1; }
    }
    return fd;
  }

  std::string hello_frame(uint8_t kind, const std::vector<std::string>& protos) {
    Writer w(D_HELLO);
    w.blob(peer_id);
    w.u32((uint32_t)listen_addrs.size());
    for (auto& a : listen_addrs) w.blob(a);
    w.u8(kind);  // 0 = persistent link, 1 = stream
    w.u32((uint32_t)protos.size());
    for (auto& p : protos) w.blob(p);
    return w.finish();
  }

  void learn(const std::string& pid, const std::string& addr) {
    if (pid.empty() || addr.empty() || pid == peer_id) return;
    addr_book[pid].insert(addr);
  }

  std::string addrs_frame() {
    Writer w(D_ADDRS);
    uint32_t n = 0;
    for (auto& kv : addr_book) n += (uint32_t)kv.second.size();
    w.u32(n);
    for (auto& kv : addr_book) for (auto& a : kv.second) { w.blob(kv.first); w.blob(a); }
    return w.finish();
  }

  // persistent link to a peer, creating it if an address is known; nullptr if not reachable right now
  Conn* link_to(const std::string& pid) {
    auto it = peer_links.find(pid);
    if (it != peer_links.end()) { Conn* c = get(it->second); if (c) return c; peer_links.erase(it); }
    auto ab = addr_book.find(pid);
    if (ab == addr_book.end()) return nullptr;
    for (auto& addr : ab->second) {
      bool prog;
      int fd = start_connect(addr, prog);
      if (fd < 0) continue;
      Conn* c = add(fd, Kind::PEER);
      c->peer_id = pid;
      c->connecting = prog;
      peer_links[pid] = c->id;
      send_bytes(c, hello_frame(0, {}));
      send_bytes(c, addrs_frame());
      return c;
    }
    return nullptr;
  }

  void ask_who_has(const std::string& pid) {
    Writer w(D_WHOHAS);
    w.blob(pid);
    std::string f = w.finish();
    for (auto& kv : peer_links) { Conn* c = get(kv.second); if (c) send_bytes(c, f); }
  }

  // ---------------------------------------------------------------- replies to clients
  void reply_ok(Conn* c, const std::string& body = std::string()) { Writer w(REPLY_OK); w.buf.append(body); send_bytes(c, w.finish()); }
  void reply_err(Conn* c, const std::string& msg) { Writer w(REPLY_ERR); w.blob(msg); send_bytes(c, w.finish()); }
  void respond_to_client(uint64_t client, const std::string& call_id, bool is_err, const std::string& data) {
    Conn* c = get(client);
    if (!c) return;
    Writer w(P_RESPONSE);
    w.blob(call_id);
    w.u8(is_err ? 1 : 0);
    w.blob(data);
    send_bytes(c, w.finish());
  }

  // ---------------------------------------------------------------- frame handlers
  void on_control_frame(Conn* c, uint8_t type, Reader& r) {
    switch (type) {
      case C_IDENTIFY: {
        Writer w(REPLY_OK);
        w.blob(peer_id);
        w.u32((uint32_t)listen_addrs.size());
        for (auto& a : listen_addrs) w.blob(a);
        send_bytes(c, w.finish());
        break;
      }
      case C_CONNECT: {
        std::string pid = r.blob();
        uint32_t n = r.u32();
        for (uint32_t i = 0; i < n && r.ok; ++i) learn(pid, r.blob());
        if (!r.ok) { reply_err(c, "malformed CONNECT"); break; }
        if (pid == peer_id) { reply_ok(c); break; }
        Conn* link = link_to(pid);
        if (link) reply_ok(c); else reply_err(c, "failed to connect: no reachable address for the peer");
        break;
      }
      case C_LIST_PEERS: {
        Writer w(REPLY_OK);
        w.u32((uint32_t)peer_links.size());
        for (auto& kv : peer_links) {
          w.blob(kv.first);
          auto ab = addr_book.find(kv.first);
          w.blob(ab != addr_book.end() && !ab->second.empty() ? *ab->second.begin() : std::string());
        }
        send_bytes(c, w.finish());
        break;
      }
      case C_DISCONNECT: {
        std::string pid = r.blob();
        auto it = peer_links.find(pid);
        if (it != peer_links.end()) close_conn(it->second, "DISCONNECT requested");
        reply_ok(c);
        break;
      }
      case C_PERSISTENT:
        c->kind = Kind::PERSISTENT;
        reply_ok(c);
        break;
      case C_STREAM_HANDLER: {
        std::string path = r.blob();
        uint8_t balanced = r.u8();
        uint32_t n = r.u32();
        std::vector<std::string> protos;
        for (uint32_t i = 0; i < n && r.ok; ++i) protos.push_back(r.blob());
        if (!r.ok) { reply_err(c, "malformed STREAM_HANDLER"); break; }
        std::string clash;
        for (auto& p : protos) {
          auto& v = stream_handlers[p];
          bool same = false;
          for (auto& h : v) if (h.listen_path == path) same = true;
          if (same) continue;
          if (!v.empty() && !(balanced && v[0].balanced)) { clash = p; break; }
        }
        if (!clash.empty()) { reply_err(c, "handler for protocol " + clash + " already set"); break; }
        for (auto& p : protos) {
          auto& v = stream_handlers[p];
          bool same = false;
          for (auto& h : v) if (h.listen_path == path) same = true;
          if (!same) v.push_back({path, balanced != 0});
        }
        reply_ok(c);
        break;
      }
      case C_REMOVE_STREAM_HANDLER: {
        std::string path = r.blob();
        uint32_t n = r.u32();
        for (uint32_t i = 0; i < n && r.ok; ++i) {
          std::string p = r.blob();
          auto it = stream_handlers.find(p);
          if (it == stream_handlers.end()) continue;
          auto& v = it->second;
          for (size_t k = 0; k < v.size();) { if (v[k].listen_path == path) v.erase(v.begin() + k); else ++k; }
          if (v.empty()) stream_handlers.erase(it);
        }
        reply_ok(c);
        break;
      }
      case C_STREAM_OPEN: {
        std::string pid = r.blob();
        uint32_t n = r.u32();
        std::vector<std::string> protos;
        for (uint32_t i = 0; i < n && r.ok; ++i) protos.push_back(r.blob());
        if (!r.ok || protos.empty()) { reply_err(c, "malformed STREAM_OPEN"); break; }
        if (pid == peer_id) { open_local_stream(c, protos); break; }
        c->read_paused = true;  // no client bytes are consumed until the remote side accepted the stream
        rearm(c);
        auto ab = addr_book.find(pid);
        if (ab == addr_book.end() || ab->second.empty()) {
          parked_streams.push_back({c->id, pid, protos, now_s() + 3.0});
          ask_who_has(pid);
          break;
        }
        start_remote_stream(c, pid, protos);
        break;
      }
      default:
        reply_err(c, "unknown command");
    }
  }

  void start_remote_stream(Conn* c, const std::string& pid, const std::vector<std::string>& protos) {
    Conn* out = nullptr;
    auto ab = addr_book.find(pid);
    if (ab != addr_book.end()) {
      for (auto& addr : ab->second) {
        bool prog;
        int fd = start_connect(addr, prog);
        if (fd < 0) continue;
        out = add(fd, Kind::STREAM_WAIT);
        out->connecting = prog;
        break;
      }
    }
    if (!out) {
      c->read_paused = false;
      reply_err(c, "failed to open stream: peer is unreachable");
      return;
    }
    out->partner = c->id;
    out->protos = protos;
    c->partner = out->id;
    send_bytes(out, hello_frame(1, protos));
  }

  // pick a handler for the first supported protocol; returns the listen path (empty if none)
  std::string pick_stream_handler(const std::vector<std::string>& protos, std::string& chosen) {
    for (auto& p : protos) {
      auto it = stream_handlers.find(p);
      if (it == stream_handlers.end() || it->second.empty()) continue;
      auto& v = it->second;
      size_t idx = v.size() > 1 ? (stream_rr[p]++ % v.size()) : 0;
      chosen = p;
      return v[idx].listen_path;
    }
    return {};
  }

  // connect to a local handler client and announce the stream; returns the new connection or nullptr
  Conn* connect_handler(const std::string& path, const std::string& from_peer, const std::string& from_addr,
                        const std::string& proto) {
    bool prog;
    int fd = start_connect("/unix" + path, prog);
    if (fd < 0) return nullptr;
    Conn* h = add(fd, Kind::SPLICE);
    h->connecting = prog;
    Writer w(S_INFO);
    w.blob(from_peer);
    w.blob(from_addr);
    w.blob(proto);
    send_bytes(h, w.finish());
    return h;
  }

  void drop_dead_handler(const std::string& proto, const std::string& path) {
    auto it = stream_handlers.find(proto);
    if (it == stream_handlers.end()) return;
    auto& v = it->second;
    for (size_t k = 0; k < v.size();) { if (v[k].listen_path == path) v.erase(v.begin() + k); else ++k; }
    if (v.empty()) stream_handlers.erase(it);
  }

  void open_local_stream(Conn* client, const std::vector<std::string>& protos) {
    std::string chosen;
    std::string path = pick_stream_handler(protos, chosen);
    if (path.empty()) { reply_err(client, "protocol not supported"); return; }
    Conn* h = connect_handler(path, peer_id, listen_addrs.empty() ? "" : listen_addrs[0], chosen);
    if (!h) { drop_dead_handler(chosen, path); reply_err(client, "handler is not reachable"); return; }
    Writer w(REPLY_OK);
    w.blob(chosen);
    send_bytes(client, w.finish());
    client->kind = Kind::SPLICE;
    client->partner = h->id;
    h->partner = client->id;
    pump_leftover(client);
  }

  // bytes that arrived behind a command frame belong to the stream
  void pump_leftover(Conn* c) {
    if (c->in.empty()) return;
    Conn* p = get(c->partner);
    if (p) send_bytes(p, c->in);
    c->in.clear();
  }

  void on_persistent_frame(Conn* c, uint8_t type, Reader& r) {
    switch (type) {
      case P_ADD_UNARY_HANDLER: {
        std::string call_id = r.blob(), proto = r.blob();
        uint8_t balanced = r.u8();
        auto& v = unary_handlers[proto];
        bool err = false;
        bool mine = false;
        for (auto& h : v) if (h.client == c->id) mine = true;
        if (!mine) {
          if (!v.empty() && !(balanced && v[0].balanced)) err = true;
          else v.push_back({c->id, balanced != 0});
        }
        Writer w(P_ACK);
        w.blob(call_id);
        w.u8(err ? 1 : 0);
        w.blob(err ? "handler for protocol " + proto + " already registered" : std::string());
        send_bytes(c, w.finish());
        break;
      }
      case P_REMOVE_UNARY_HANDLER: {
        std::string call_id = r.blob(), proto = r.blob();
        auto it = unary_handlers.find(proto);
        bool found = false;
        if (it != unary_handlers.end()) {
          auto& v = it->second;
          for (size_t k = 0; k < v.size();) { if (v[k].client == c->id) { v.erase(v.begin() + k); found = true; } else ++k; }
          if (v.empty()) unary_handlers.erase(it);
        }
        Writer w(P_ACK);
        w.blob(call_id);
        w.u8(found ? 0 : 1);
        w.blob(found ? std::string() : "handler for protocol " + proto + " does not exist");
        send_bytes(c, w.finish());
        break;
      }
      case P_CALL_UNARY: {
        std::string call_id = r.blob(), pid = r.blob(), proto = r.blob(), data = r.blob();
        if (!r.ok) break;
        Writer w(D_UNARY_REQ);
        w.blob(call_id);
        w.blob(proto);
        w.blob(data);
        std::string frame = w.finish();
        if (pid == peer_id) { deliver_request(0, peer_id, call_id, proto, data, c->id); break; }
        Conn* link = link_to(pid);
        if (link) {
          out_calls[call_id] = {c->id, link->id};
          send_bytes(link, frame);
        } else {
          parked.push_back({pid, std::move(frame), c->id, call_id, now_s() + 3.0});
          ask_who_has(pid);
        }
        break;
      }
      case P_UNARY_RESPONSE: {
        std::string call_id = r.blob();
        uint8_t is_err = r.u8();
        std::string data = r.blob();
        auto it = in_calls.find(call_id);
        if (it == in_calls.end()) break;  // cancelled in the meantime
        InCall ic = it->second;
        in_calls.erase(it);
        if (ic.peer_conn == 0) {  // loopback call: the requester is a local client stored in out_calls
          auto oc = out_calls.find(call_id);
          if (oc != out_calls.end()) { respond_to_client(oc->second.client, call_id, is_err != 0, data); out_calls.erase(oc); }
          break;
        }
        Conn* link = get(ic.peer_conn);
        if (!link) break;
        Writer w(D_UNARY_RESP);
        w.blob(call_id);
        w.u8(is_err);
        w.blob(data);
        send_bytes(link, w.finish());
        break;
      }
      case P_CANCEL: {
        std::string call_id = r.blob();
        auto oc = out_calls.find(call_id);
        if (oc != out_calls.end()) {
          if (oc->second.peer_conn == 0) {
            auto ic = in_calls.find(call_id);
            if (ic != in_calls.end()) {
              Conn* cl = get(ic->second.client);
              if (cl) { Writer w(P_CANCEL); w.blob(call_id); send_bytes(cl, w.finish()); }
              in_calls.erase(ic);
            }
          } else {
            Conn* link = get(oc->second.peer_conn);
            if (link) { Writer w(D_CANCEL); w.blob(call_id); send_bytes(link, w.finish()); }
          }
          out_calls.erase(oc);
        }
        for (auto it = parked.begin(); it != parked.end(); ++it) if (it->call_id == call_id) { parked.erase(it); break; }
        break;
      }
      default:
        break;
    }
  }

  // hand a unary request to a local handler client; `link` = 0 means the request came from a local client
  void deliver_request(uint64_t link, const std::string& from_peer, const std::string& call_id, const std::string& proto,
                       const std::string& data, uint64_t local_origin) {
    auto fail = [&](const std::string& msg) {
      if (link == 0) respond_to_client(local_origin, call_id, true, msg);
      else { Conn* l = get(link); if (l) { Writer w(D_UNARY_RESP); w.blob(call_id); w.u8(1); w.blob(msg); send_bytes(l, w.finish()); } }
    };
    auto it = unary_handlers.find(proto);
    if (it == unary_handlers.end() || it->second.empty()) { fail("protocol not supported: " + proto); return; }
    auto& v = it->second;
    Conn* cl = nullptr;
    for (size_t tries = 0; tries < v.size() && !cl; ++tries) {
      size_t idx = v.size() > 1 ? (unary_rr[proto]++ % v.size()) : 0;
      cl = get(v[idx].client);
    }
    if (!cl) { fail("handler is gone"); return; }
    in_calls[call_id] = {link, cl->id};
    if (link == 0) out_calls[call_id] = {local_origin, 0};
    Writer w(P_REQUEST);
    w.blob(call_id);
    w.blob(from_peer);
    w.blob(proto);
    w.blob(data);
    send_bytes(cl, w.finish());
  }

  void on_peer_frame(Conn* c, uint8_t type, Reader& r) {
    switch (type) {
      case D_UNARY_REQ: {
        std::string call_id = r.blob(), proto = r.blob(), data = r.blob();
        if (r.ok) deliver_request(c->id, c->peer_id, call_id, proto, data, 0);
        break;
      }
      case D_UNARY_RESP: {
        std::string call_id = r.blob();
        uint8_t is_err = r.u8();
        std::string data = r.blob();
        auto it = out_calls.find(call_id);
        if (it == out_calls.end()) break;
        respond_to_client(it->second.client, call_id, is_err != 0, data);
        out_calls.erase(it);
        break;
      }
      case D_CANCEL: {
        std::string call_id = r.blob();
        auto it = in_calls.find(call_id);
        if (it == in_calls.end()) break;
        Conn* cl = get(it->second.client);
        if (cl) { Writer w(P_CANCEL); w.blob(call_id); send_bytes(cl, w.finish()); }
        in_calls.erase(it);
        break;
      }
      case D_ADDRS: {
        uint32_t n = r.u32();
        for (uint32_t i = 0; i < n && r.ok; ++i) { std::string pid = r.blob(), a = r.blob(); if (r.ok) learn(pid, a); }
        retry_parked();
        break;
      }
      case D_WHOHAS: {
        std::string pid = r.blob();
        auto ab = addr_book.find(pid);
        Writer w(D_WHOHAS_REPLY);
        w.blob(pid);
        w.u32(ab == addr_book.end() ? 0 : (uint32_t)ab->second.size());
        if (ab != addr_book.end()) for (auto& a : ab->second) w.blob(a);
        send_bytes(c, w.finish());
        break;
      }
      case D_WHOHAS_REPLY: {
        std::string pid = r.blob();
        uint32_t n = r.u32();
        for (uint32_t i = 0; i < n && r.ok; ++i) learn(pid, r.blob());
        retry_parked();
        break;
      }
      default:
        break;
    }
  }

  void retry_parked() {
    for (size_t i = 0; i < parked.size();) {
      Conn* link = link_to(parked[i].peer_id);
      if (link) {
        out_calls[parked[i].call_id] = {parked[i].client, link->id};
        send_bytes(link, parked[i].frame);
        parked.erase(parked.begin() + i);
      } else ++i;
    }
    for (size_t i = 0; i < parked_streams.size();) {
      auto ab = addr_book.find(parked_streams[i].peer_id);
      if (ab != addr_book.end() && !ab->second.empty()) {
        ParkedStream ps = parked_streams[i];
        parked_streams.erase(parked_streams.begin() + i);
        Conn* c = get(ps.client);
        if (c) start_remote_stream(c, ps.peer_id, ps.protos);
      } else ++i;
    }
  }
  void expire_parked() {
    double t = now_s();
    for (size_t i = 0; i < parked_streams.size();) {
      if (parked_streams[i].deadline < t) {
        Conn* c = get(parked_streams[i].client);
        if (c) { c->read_paused = false; reply_err(c, "failed to open stream: unknown peer"); }
        parked_streams.erase(parked_streams.begin() + i);
      } else ++i;
    }
    for (size_t i = 0; i < parked.size();) {
      if (parked[i].deadline < t) {
        respond_to_client(parked[i].client, parked[i].call_id, true, "failed to reach the peer: address unknown");
        parked.erase(parked.begin() + i);
      } else ++i;
    }
  }

  // first frame of an inbound daemon connection
  void on_hello(Conn* c, Reader& r) {
    std::string pid = r.blob();
    uint32_t n = r.u32();
    std::vector<std::string> addrs;
    for (uint32_t i = 0; i < n && r.ok; ++i) addrs.push_back(r.blob());
    uint8_t kind = r.u8();
    uint32_t np = r.u32();
    std::vector<std::string> protos;
    for (uint32_t i = 0; i < np && r.ok; ++i) protos.push_back(r.blob());
    if (!r.ok) { close_conn(c->id, "malformed HELLO"); return; }
    for (auto& a : addrs) learn(pid, a);
    if (kind == 0 && !addrs.empty()) {  // tell the peers we already know about the newcomer
      Writer g(D_ADDRS);
      g.u32((uint32_t)addrs.size());
      for (auto& a : addrs) { g.blob(pid); g.blob(a); }
      std::string gf = g.finish();
      for (auto& kv : peer_links) { Conn* l = get(kv.second); if (l && kv.first != pid) send_bytes(l, gf); }
    }
    if (kind == 0) {
      c->kind = Kind::PEER;
      c->peer_id = pid;
      if (!peer_links.count(pid) || !get(peer_links[pid])) peer_links[pid] = c->id;
      send_bytes(c, addrs_frame());
      retry_parked();
      return;
    }
    // stream request
    std::string chosen;
    std::string path = pick_stream_handler(protos, chosen);
    if (path.empty()) {
      Writer w(S_ERR); w.blob("protocol not supported"); send_bytes(c, w.finish());
      c->wr_shutdown_pending = true; flush(c);
      return;
    }
    Conn* h = connect_handler(path, pid, addrs.empty() ? std::string() : addrs[0], chosen);
    if (!h) {
      drop_dead_handler(chosen, path);
      Writer w(S_ERR); w.blob("handler is not reachable"); send_bytes(c, w.finish());
      c->wr_shutdown_pending = true; flush(c);
      return;
    }
    Writer w(S_OK);
    w.blob(chosen);
    send_bytes(c, w.finish());
    c->kind = Kind::SPLICE;
    c->partner = h->id;
    h->partner = c->id;
    pump_leftover(c);
  }

  void on_stream_reply(Conn* c, uint8_t type, Reader& r) {
    Conn* client = get(c->partner);
    if (!client) { close_conn(c->id, "client went away"); return; }
    if (type == S_OK) {
      std::string proto = r.blob();
      Writer w(REPLY_OK);
      w.blob(proto);
      send_bytes(client, w.finish());
      c->kind = Kind::SPLICE;
      client->kind = Kind::SPLICE;
      client->read_paused = false;
      rearm(client);
      pump_leftover(c);
      pump_leftover(client);
    } else {
      std::string msg = r.blob();
      client->partner = 0;
      c->partner = 0;
      client->read_paused = false;
      reply_err(client, msg.empty() ? "stream refused" : msg);
      close_conn(c->id, "stream refused");
    }
  }

  // ---------------------------------------------------------------- io events
  void consume_frames(Conn* c) {
    uint64_t id = c->id;
    while (true) {
      c = get(id);
      if (!c || c->kind == Kind::SPLICE) return;
      if (c->kind == Kind::CONTROL && (c->partner != 0 || c->read_paused)) return;  // a stream open is pending
      if (c->in.size() < 5) return;
      uint32_t be;
      memcpy(&be, c->in.data(), 4);
      uint32_t len = ntohl(be);
      if (len < 1 || len > MAX_FRAME) { close_conn(id, "bad frame length"); return; }
      if (c->in.size() < 4 + (size_t)len) return;
      std::string frame = c->in.substr(4, len);
      c->in.erase(0, 4 + (size_t)len);
      uint8_t type = (uint8_t)frame[0];
      Reader r(frame.data() + 1, frame.size() - 1);
      switch (c->kind) {
        case Kind::CONTROL: on_control_frame(c, type, r); break;
        case Kind::PERSISTENT: on_persistent_frame(c, type, r); break;
        case Kind::PEER_IN: if (type == D_HELLO) on_hello(c, r); else close_conn(id, "expected HELLO"); break;
        case Kind::PEER: on_peer_frame(c, type, r); break;
        case Kind::STREAM_WAIT: on_stream_reply(c, type, r); break;
        default: return;
      }
    }
  }

  void on_readable(Conn* c) {
    static char buf[1 << 20];  // the daemon is single-threaded and on_readable never nests
    uint64_t id = c->id;
    while (true) {
      c = get(id);
      if (!c || c->read_paused) return;
      ssize_t n = ::recv(c->fd, buf, sizeof(buf), 0);
      if (n > 0) {
        if (c->kind == Kind::SPLICE) {
          Conn* p = get(c->partner);
          if (!p) continue;  // partner gone: discard
          send_raw(p, buf, (size_t)n);
          c = get(id);
          p = c ? get(c->partner) : nullptr;
          if (c && p && p->out.size() - p->out_off > SPLICE_HIGH_WATER) { c->read_paused = true; rearm(c); return; }
        } else {
          c->in.append(buf, (size_t)n);
          consume_frames(c);
        }
        continue;
      }
      if (n == 0) {
        c->rd_closed = true;
        if (c->kind == Kind::SPLICE) {
          Conn* p = get(c->partner);
          if (p) { p->wr_shutdown_pending = true; flush(p); }
          c = get(id);
          if (c && (c->wr_closed || !p)) { close_conn(id, "stream finished"); return; }
          if (c) rearm(c);
        } else {
          close_conn(id, "peer closed");
        }
        return;
      }
      if (errno == EAGAIN || errno == EWOULDBLOCK) return;
      if (errno == EINTR) continue;
      close_conn(id, "recv failed");
      return;
    }
  }

  void on_writable(Conn* c) {
    if (c->connecting) {
      int err = 0;
      socklen_t len = sizeof(err);
      getsockopt(c->fd, SOL_SOCKET, SO_ERROR, &err, &len);
      if (err != 0) {
        uint64_t id = c->id;
        if (c->kind == Kind::STREAM_WAIT) {
          Conn* client = get(c->partner);
          if (client) { client->partner = 0; client->read_paused = false; c->partner = 0; reply_err(client, "failed to open stream: connection refused"); }
        }
        close_conn(id, "connect failed");
        return;
      }
      c->connecting = false;
    }
    flush(c);
  }

  void accept_all(Conn* l) {
    while (true) {
      int fd = ::accept(l->fd, nullptr, nullptr);
      if (fd < 0) return;
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      add(fd, l->kind == Kind::LISTEN_CONTROL ? Kind::CONTROL : Kind::PEER_IN);
    }
  }

  int run() {
    epoll_event evs[256];
    double last_sweep = now_s();
    while (true) {
      int n = epoll_wait(ep, evs, 256, 500);
      if (n < 0 && errno != EINTR) return 1;
      for (int i = 0; i < n; ++i) {
        Conn* c = get(evs[i].data.u64);
        if (!c) continue;
        if (c->kind == Kind::LISTEN_CONTROL || c->kind == Kind::LISTEN_PEER) { accept_all(c); continue; }
        uint64_t id = c->id;
        if (evs[i].events & EPOLLOUT) on_writable(c);
        c = get(id);
        if (c && (evs[i].events & (EPOLLIN | EPOLLHUP | EPOLLERR))) on_readable(c);
      }
      if (now_s() - last_sweep > 0.5) { expire_parked(); last_sweep = now_s(); }
      if (parent_watch && getppid() != initial_parent) return 0;  // the process that spawned us is gone
    }
  }
  bool parent_watch = true;
  pid_t initial_parent = getppid();
};

int listen_unix(const std::string& path) {
  int fd = ::socket(AF_UNIX, SOCK_STREAM, 0);
  sockaddr_un un{};
  un.sun_family = AF_UNIX;
  if (path.size() >= sizeof(un.sun_path)) return -1;
  strcpy(un.sun_path, path.c_str());
  ::unlink(path.c_str());
  if (::bind(fd, (sockaddr*)&un, sizeof(un)) < 0 || ::listen(fd, 1024) < 0) { ::close(fd); return -1; }
  return fd;
}

int listen_tcp(const std::string& host, int port, int& bound_port) {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in in{};
  in.sin_family = AF_INET;
  in.sin_port = htons((uint16_t)port);
  if (inet_pton(AF_INET, host.c_str(), &in.sin_addr) != 1) { ::close(fd); return -1; }
  if (::bind(fd, (sockaddr*)&in, sizeof(in)) < 0 || ::listen(fd, 1024) < 0) { ::close(fd); return -1; }
  socklen_t len = sizeof(in);
  getsockname(fd, (sockaddr*)&in, &len);
  bound_port = ntohs(in.sin_port);
  return fd;
}

}  // namespace

int main(int argc, char** argv) {
  signal(SIGPIPE, SIG_IGN);
  Daemon d;
  std::string control_path, host = "127.0.0.1", peer_unix;
  int port = 0;
  bool no_tcp = false;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() -> std::string { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--control") control_path = next();
    else if (a == "--peer-id") d.peer_id = next();
    else if (a == "--host") host = next();
    else if (a == "--port") port = atoi(next().c_str());
    else if (a == "--peer-unix") peer_unix = next();
    else if (a == "--no-tcp") no_tcp = true;
    else if (a == "--verbose") d.verbose = true;
    else if (a == "--no-parent-watch") d.parent_watch = false;
    else if (a == "--help") {
      printf("hmp2pd --control PATH --peer-id ID [--host IP] [--port N] [--peer-unix PATH] [--no-tcp] [--verbose]\n");
      return 0;
    }
  }
  if (control_path.empty() || d.peer_id.empty()) { fprintf(stderr, "hmp2pd: --control and --peer-id are required\n"); return 2; }
  d.ep = epoll_create1(0);
  int cfd = listen_unix(control_path);
  if (cfd < 0) { fprintf(stderr, "hmp2pd: cannot listen on %s: %s\n", control_path.c_str(), strerror(errno)); return 3; }
  d.add(cfd, Kind::LISTEN_CONTROL);
  if (!no_tcp) {
    int bound = 0;
    int pfd = listen_tcp(host, port, bound);
    if (pfd < 0) { fprintf(stderr, "hmp2pd: cannot listen on %s:%d: %s\n", host.c_str(), port, strerror(errno)); return 4; }
    d.add(pfd, Kind::LISTEN_PEER);
    d.listen_addrs.push_back("/ip4/" + (host == "0.0.0.0" ? std::string("127.0.0.1") : host) + "/tcp/" + std::to_string(bound));
  }
  if (!peer_unix.empty()) {
    int ufd = listen_unix(peer_unix);
    if (ufd < 0) { fprintf(stderr, "hmp2pd: cannot listen on %s\n", peer_unix.c_str()); return 5; }
    d.add(ufd, Kind::LISTEN_PEER);
    d.listen_addrs.push_back("/unix" + peer_unix);
  }
  printf("Peer ID: %s\n", d.peer_id.c_str());
  for (auto& a : d.listen_addrs) printf("Listening: %s\n", a.c_str());
  printf("Ready\n");
  fflush(stdout);
  int rc = d.run();
  ::unlink(control_path.c_str());
  if (!peer_unix.empty()) ::unlink(peer_unix.c_str());
  return rc;
}
