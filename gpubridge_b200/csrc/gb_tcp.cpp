// Native tagged-message worker over several TCP streams per peer: the host-staged bridge
// transport for links that leave the NVSwitch box (cross-node fallback).
//
// Contract (the reference's multi-stream TCP worker, written there in Rust:
// src/gpubridge/multitcp/crate/src/lib.rs:656-840): a worker listens on one port; for every
// pair of members the lower index dials `streams` connections to the higher; a message is a
// 16-byte header {tag, length} followed by its bytes and travels on one connection, chosen by
// its tag (the chunk number sits in the tag's low bits, so the chunks of a message fan out over
// the connections like a round robin would, while messages that share a tag share a connection
// and so arrive in the order sent); every connection has a sender thread (fed by a queue) and
// a receiver thread;
// a receive is matched by (peer, tag), and a message that arrives before its receive is
// posted is buffered - and stays receivable after its sender has closed: a member that ends
// its connections between two messages has left, which fails what still waits for it and what
// is posted towards it later, but is not a wreck of the whole worker (a connection that ends
// in the middle of a message is); send() and recv() return operation ids at once and wait() blocks until
// the listed operations are done or a deadline passes.  A failed wait stops every thread
// before it returns, so no thread touches the caller's memory afterwards.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "gb_tagged.h"

namespace {

using Clock = std::chrono::steady_clock;

struct Header { uint64_t tag, length; };

struct Op {
    bool sending = false;
    int peer = 0;
    uint64_t tag = 0;
    char* data = nullptr;
    uint64_t length = 0;
    int state = 0;                 // 0 pending, 1 done, 2 failed
};

struct Conn {
    int fd = -1;
    int peer = -1;
    std::thread sender, receiver;
    std::deque<long> queue;        // ids of sends waiting for this connection
    std::condition_variable wake;
};

struct Worker {
    int index = 0, members = 0, streams = 1;
    int listener = -1;
    uint16_t port = 0;
    std::string host = "127.0.0.1";
    std::mutex mu;
    std::condition_variable done;
    std::map<long, Op> ops;
    long next_id = 1;
    std::vector<std::unique_ptr<Conn>> conns;
    std::vector<std::vector<int>> by_peer;         // connection indices of each peer
    std::map<std::pair<int, uint64_t>, long> posted;                  // receives waiting
    std::map<std::pair<int, uint64_t>, std::deque<std::vector<char>>> early;   // unexpected messages
    std::vector<int> open_conns;                   // per peer: connections that have not ended
    std::atomic<bool> stopping{false};
    std::mutex stop_mu;                            // one thread at a time stops (and joins) the others
    bool broken = false;
    std::string error;
    bool gone(int peer) const { return !by_peer[peer].empty() && open_conns[peer] == 0; }
};

thread_local std::string g_error;

void set_error(Worker* w, const std::string& text) {
    if (w != nullptr && w->error.empty()) w->error = text;
    g_error = text;
}

bool read_all(int fd, char* p, uint64_t n, std::atomic<bool>& stop, bool* ended_cleanly = nullptr) {
    const uint64_t wanted = n;
    if (ended_cleanly != nullptr) *ended_cleanly = false;
    while (n > 0) {
        pollfd pfd{fd, POLLIN, 0};
        int ready = poll(&pfd, 1, 100);
        if (stop.load()) return false;
        if (ready == 0) continue;
        if (ready < 0) { if (errno == EINTR) continue; return false; }
        ssize_t got = ::recv(fd, p, n > (1u << 30) ? (1u << 30) : n, 0);
        if (got <= 0) {
            if (got < 0 && (errno == EINTR || errno == EAGAIN)) continue;
            if (got == 0 && n == wanted && ended_cleanly != nullptr) *ended_cleanly = true;
            return false;
        }
        p += got; n -= (uint64_t)got;
    }
    return true;
}

bool write_all(int fd, const char* p, uint64_t n, std::atomic<bool>& stop) {
    while (n > 0) {
        if (stop.load()) return false;
        ssize_t put = ::send(fd, p, n > (1u << 30) ? (1u << 30) : n, MSG_NOSIGNAL);
        if (put < 0) { if (errno == EINTR || errno == EAGAIN) continue; return false; }
        p += put; n -= (uint64_t)put;
    }
    return true;
}

void fail_all(Worker* w, const std::string& why) {
    // called with w->mu held
    w->broken = true;
    if (w->error.empty()) w->error = why;
    for (auto& entry : w->ops)
        if (entry.second.state == 0) entry.second.state = 2;
    w->done.notify_all();
    for (auto& c : w->conns) c->wake.notify_all();
}

void sender_loop(Worker* w, Conn* c) {
    for (;;) {
        long id;
        Op op;
        {
            std::unique_lock<std::mutex> lock(w->mu);
            c->wake.wait(lock, [&] { return w->stopping.load() || w->broken || !c->queue.empty(); });
            if (w->stopping.load() || w->broken) return;
            id = c->queue.front();
            c->queue.pop_front();
            op = w->ops[id];
        }
        Header h{op.tag, op.length};
        bool ok = write_all(c->fd, reinterpret_cast<const char*>(&h), sizeof(h), w->stopping) &&
                  write_all(c->fd, op.data, op.length, w->stopping);
        std::lock_guard<std::mutex> lock(w->mu);
        if (!ok) {
            if (!w->stopping.load()) fail_all(w, "send to member " + std::to_string(c->peer) + " failed");
            return;
        }
        auto it = w->ops.find(id);
        if (it != w->ops.end() && it->second.state == 0) it->second.state = 1;
        w->done.notify_all();
    }
}

// The member at the other end of `c` closed it between two messages.  What it sent before is
// still here and can be received; when its last connection has ended, receives that wait for
// more from it fail, and so does everything posted towards it later.  Called with w->mu held.
void member_left(Worker* w, Conn* c) {
    if (--w->open_conns[c->peer] > 0) return;
    const std::string why = "member " + std::to_string(c->peer) + " closed its connections";
    if (w->error.empty()) w->error = why;
    for (auto it = w->posted.begin(); it != w->posted.end();) {
        if (it->first.first == c->peer) {
            auto op = w->ops.find(it->second);
            if (op != w->ops.end() && op->second.state == 0) op->second.state = 2;
            it = w->posted.erase(it);
        } else ++it;
    }
    for (auto& entry : w->ops)
        if (entry.second.sending && entry.second.peer == c->peer && entry.second.state == 0) entry.second.state = 2;
    w->done.notify_all();
}

void receiver_loop(Worker* w, Conn* c) {
    for (;;) {
        Header h{};
        bool ended_cleanly = false;
        if (!read_all(c->fd, reinterpret_cast<char*>(&h), sizeof(h), w->stopping, &ended_cleanly)) {
            if (ended_cleanly && !w->stopping.load()) {
                std::lock_guard<std::mutex> lock(w->mu);
                member_left(w, c);
                return;
            }
            break;
        }
        long id = 0;
        char* target = nullptr;
        {
            std::lock_guard<std::mutex> lock(w->mu);
            auto it = w->posted.find({c->peer, h.tag});
            if (it != w->posted.end()) {
                id = it->second;
                w->posted.erase(it);
                Op& op = w->ops[id];
                if (op.length != h.length) {
                    fail_all(w, "message of " + std::to_string(h.length) + " bytes from member " +
                                std::to_string(c->peer) + " for a receive of " +
                                std::to_string(op.length));
                    return;
                }
                target = op.data;
            }
        }
        if (id != 0) {
            if (!read_all(c->fd, target, h.length, w->stopping)) break;
            std::lock_guard<std::mutex> lock(w->mu);
            auto it = w->ops.find(id);
            if (it != w->ops.end() && it->second.state == 0) it->second.state = 1;
            w->done.notify_all();
        } else {
            std::vector<char> body(h.length);
            if (!read_all(c->fd, body.data(), h.length, w->stopping)) break;
            std::lock_guard<std::mutex> lock(w->mu);
            // a receive may have been posted while the body was read
            auto it = w->posted.find({c->peer, h.tag});
            if (it != w->posted.end()) {
                Op& op = w->ops[it->second];
                if (op.length == h.length) {
                    std::memcpy(op.data, body.data(), h.length);
                    op.state = 1;
                } else {
                    op.state = 2;
                    w->error = "length mismatch on a buffered message";
                }
                w->posted.erase(it);
                w->done.notify_all();
            } else {
                w->early[{c->peer, h.tag}].push_back(std::move(body));
            }
        }
    }
    std::lock_guard<std::mutex> lock(w->mu);
    if (!w->stopping.load()) fail_all(w, "connection to member " + std::to_string(c->peer) + " closed");
}

void stop_threads(Worker* w) {
    // A failed wait stops the worker, and so may an abort or a close from another thread at the
    // same moment: the second one waits here and then finds nothing left to join.
    std::lock_guard<std::mutex> one_at_a_time(w->stop_mu);
    w->stopping.store(true);
    {
        std::lock_guard<std::mutex> lock(w->mu);
        w->broken = true;                              // nothing can be posted on a stopped worker
        if (w->error.empty()) w->error = "the worker was stopped";
        for (auto& c : w->conns) {
            if (c->fd >= 0) ::shutdown(c->fd, SHUT_RDWR);
            c->wake.notify_all();
        }
        w->done.notify_all();
    }
    for (auto& c : w->conns) {
        if (c->sender.joinable()) c->sender.join();
        if (c->receiver.joinable()) c->receiver.join();
    }
    std::lock_guard<std::mutex> lock(w->mu);
    for (auto& c : w->conns) {
        if (c->fd >= 0) { ::close(c->fd); c->fd = -1; }
    }
    for (auto& entry : w->ops)
        if (entry.second.state == 0) entry.second.state = 2;
}

bool split_address(const std::string& text, std::string& host, uint16_t& port) {
    size_t colon = text.rfind(':');
    if (colon == std::string::npos) return false;
    host = text.substr(0, colon);
    port = (uint16_t)std::stoi(text.substr(colon + 1));
    return true;
}

}  // namespace

extern "C" {

int gb_tcp_protocol() { return 1; }

const char* gb_tcp_last_error(void* handle) {
    Worker* w = static_cast<Worker*>(handle);
    if (w != nullptr) {
        std::lock_guard<std::mutex> lock(w->mu);
        g_error = w->error.empty() ? g_error : w->error;
    }
    return g_error.c_str();
}

// A worker for member `index` of `members`, listening on `host` (an address of this machine).
void* gb_tcp_create(int index, int members, int streams, const char* host) {
    auto w = std::make_unique<Worker>();
    w->index = index; w->members = members; w->streams = streams < 1 ? 1 : streams;
    if (host != nullptr && host[0] != 0) w->host = host;
    w->by_peer.resize(members);
    w->open_conns.assign(members, 0);
    w->listener = ::socket(AF_INET, SOCK_STREAM, 0);
    if (w->listener < 0) { set_error(nullptr, "socket() failed"); return nullptr; }
    int one = 1;
    ::setsockopt(w->listener, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = 0;
    if (::inet_pton(AF_INET, w->host.c_str(), &addr.sin_addr) != 1) {
        set_error(nullptr, "not an IPv4 address: " + w->host);
        ::close(w->listener);
        return nullptr;
    }
    if (::bind(w->listener, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 ||
        ::listen(w->listener, 128) != 0) {
        set_error(nullptr, "bind/listen on " + w->host + " failed");
        ::close(w->listener);
        return nullptr;
    }
    socklen_t len = sizeof(addr);
    ::getsockname(w->listener, reinterpret_cast<sockaddr*>(&addr), &len);
    w->port = ntohs(addr.sin_port);
    return w.release();
}

int gb_tcp_address(void* handle, char* out, int capacity) {
    Worker* w = static_cast<Worker*>(handle);
    std::string text = w->host + ":" + std::to_string(w->port);
    if ((int)text.size() + 1 > capacity) return -1;
    std::memcpy(out, text.c_str(), text.size() + 1);
    return 0;
}

// `addresses`: "host:port" of every member, by index.  The lower index of a pair dials.
int gb_tcp_connect(void* handle, const char** addresses, double timeout_s) {
    Worker* w = static_cast<Worker*>(handle);
    const auto deadline = Clock::now() + std::chrono::duration<double>(timeout_s);
    int expected = w->index * w->streams;               // lower members dial us
    // dial the higher members
    for (int peer = w->index + 1; peer < w->members; ++peer) {
        std::string host; uint16_t port = 0;
        if (!split_address(addresses[peer], host, port)) { set_error(w, "bad address"); return -1; }
        for (int s = 0; s < w->streams; ++s) {
            int fd = -1;
            for (;;) {
                fd = ::socket(AF_INET, SOCK_STREAM, 0);
                sockaddr_in addr{};
                addr.sin_family = AF_INET;
                addr.sin_port = htons(port);
                ::inet_pton(AF_INET, host.c_str(), &addr.sin_addr);
                if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) break;
                ::close(fd);
                fd = -1;
                if (Clock::now() > deadline) { set_error(w, "connect to " + std::string(addresses[peer]) + " timed out"); return -1; }
                std::this_thread::sleep_for(std::chrono::milliseconds(20));
            }
            int one = 1;
            ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
            int32_t hello[2] = {w->index, s};
            if (!write_all(fd, reinterpret_cast<const char*>(hello), sizeof(hello), w->stopping)) {
                set_error(w, "handshake write failed"); ::close(fd); return -1;
            }
            auto c = std::make_unique<Conn>();
            c->fd = fd; c->peer = peer;
            w->by_peer[peer].push_back((int)w->conns.size());
            w->conns.push_back(std::move(c));
        }
    }
    // accept the lower members
    while (expected > 0) {
        pollfd pfd{w->listener, POLLIN, 0};
        int ready = poll(&pfd, 1, 100);
        if (Clock::now() > deadline) { set_error(w, "waiting for lower members to connect timed out"); return -1; }
        if (ready <= 0) continue;
        int fd = ::accept(w->listener, nullptr, nullptr);
        if (fd < 0) continue;
        int one = 1;
        ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        int32_t hello[2] = {-1, -1};
        if (!read_all(fd, reinterpret_cast<char*>(hello), sizeof(hello), w->stopping) ||
            hello[0] < 0 || hello[0] >= w->index) {
            ::close(fd);
            continue;
        }
        auto c = std::make_unique<Conn>();
        c->fd = fd; c->peer = hello[0];
        w->by_peer[hello[0]].push_back((int)w->conns.size());
        w->conns.push_back(std::move(c));
        --expected;
    }
    w->open_conns.assign(w->members, 0);
    for (auto& c : w->conns) ++w->open_conns[c->peer];
    for (auto& c : w->conns) {
        Conn* raw = c.get();
        raw->sender = std::thread(sender_loop, w, raw);
        raw->receiver = std::thread(receiver_loop, w, raw);
    }
    return 0;
}

long gb_tcp_send(void* handle, int peer, const void* data, uint64_t length, uint64_t tag) {
    Worker* w = static_cast<Worker*>(handle);
    std::lock_guard<std::mutex> lock(w->mu);
    if (w->broken || peer < 0 || peer >= w->members || w->by_peer[peer].empty() || w->gone(peer)) {
        set_error(w, "send: the worker is broken or has no connection to that member");
        return -1;
    }
    long id = w->next_id++;
    Op op;
    op.sending = true; op.peer = peer; op.tag = tag;
    op.data = const_cast<char*>(static_cast<const char*>(data)); op.length = length;
    w->ops[id] = op;
    auto& list = w->by_peer[peer];
    Conn* c = w->conns[list[(size_t)((tag ^ (tag >> 28)) % list.size())]].get();
    c->queue.push_back(id);
    c->wake.notify_one();
    return id;
}

long gb_tcp_recv(void* handle, int peer, void* data, uint64_t length, uint64_t tag) {
    Worker* w = static_cast<Worker*>(handle);
    std::lock_guard<std::mutex> lock(w->mu);
    if (w->broken || peer < 0 || peer >= w->members) {
        set_error(w, "recv: the worker is broken or the member does not exist");
        return -1;
    }
    long id = w->next_id++;
    Op op;
    op.peer = peer; op.tag = tag; op.data = static_cast<char*>(data); op.length = length;
    auto found = w->early.find({peer, tag});
    if (found != w->early.end() && !found->second.empty()) {
        std::vector<char>& body = found->second.front();
        if (body.size() == length) { std::memcpy(data, body.data(), length); op.state = 1; }
        else { op.state = 2; w->error = "length mismatch on a buffered message"; }
        found->second.pop_front();
        if (found->second.empty()) w->early.erase(found);
    } else if (w->gone(peer)) {
        set_error(w, "recv: member " + std::to_string(peer) + " closed its connections and sent nothing more");
        return -1;
    } else {
        w->posted[{peer, tag}] = id;
    }
    w->ops[id] = op;
    return id;
}

// 0: every listed operation finished.  -1: one failed or the deadline passed; every thread of
// the worker has been stopped before this returns.
int gb_tcp_wait(void* handle, const long* ids, int count, double timeout_s) {
    Worker* w = static_cast<Worker*>(handle);
    const auto deadline = Clock::now() + std::chrono::duration<double>(timeout_s);
    bool failed = false;
    {
        std::unique_lock<std::mutex> lock(w->mu);
        for (;;) {
            bool all = true;
            for (int i = 0; i < count; ++i) {
                auto it = w->ops.find(ids[i]);
                if (it == w->ops.end()) continue;
                if (it->second.state == 2) failed = true;
                if (it->second.state == 0) all = false;
            }
            if (failed || w->broken) { failed = true; break; }
            if (all) break;
            if (w->done.wait_until(lock, deadline) == std::cv_status::timeout) {
                set_error(w, "timed out waiting for a bridge message");
                failed = true;
                break;
            }
        }
        if (!failed)
            for (int i = 0; i < count; ++i) w->ops.erase(ids[i]);
    }
    if (failed) { stop_threads(w); return -1; }
    return 0;
}

// ---- collectives over the worker ----------------------------------------------------------------
// The algorithms live in gb_tagged.cpp, written against an interface this worker implements.

}  // extern "C"

namespace {

struct TcpTagged : GbTaggedWorker {
    Worker* w;
    explicit TcpTagged(Worker* worker) : w(worker) {}
    int members() const override { return w->members; }
    int index() const override { return w->index; }
    long send(int peer, const void* data, uint64_t length, uint64_t tag) override {
        return gb_tcp_send(w, peer, data, length, tag);
    }
    long recv(int peer, void* data, uint64_t length, uint64_t tag) override {
        return gb_tcp_recv(w, peer, data, length, tag);
    }
    int wait(const long* ids, int count, double timeout_s) override { return gb_tcp_wait(w, ids, count, timeout_s); }
    void stop() override { stop_threads(w); }
    void fail(const char* why) override { set_error(w, why); }
};

}  // namespace

extern "C" {

// In-place all-reduce of `count` elements over every member of the worker.  0 on success;
// -1 after a failure (the worker's threads are stopped; gb_tcp_last_error says why).
int gb_tcp_all_reduce(void* handle, void* data, uint64_t count, int dtype, int op,
                      uint64_t chunk_elems, uint64_t seq, double timeout_s) {
    TcpTagged worker(static_cast<Worker*>(handle));
    return gb_tagged_all_reduce(worker, data, count, dtype, op, chunk_elems, seq, timeout_s);
}

// Broadcast `nbytes` from member `root` to every other member.
int gb_tcp_broadcast(void* handle, void* data, uint64_t nbytes, int root, uint64_t chunk_bytes,
                     uint64_t seq, double timeout_s) {
    TcpTagged worker(static_cast<Worker*>(handle));
    return gb_tagged_broadcast(worker, data, nbytes, root, chunk_bytes, seq, timeout_s);
}

void gb_tcp_abort(void* handle) { stop_threads(static_cast<Worker*>(handle)); }

void gb_tcp_close(void* handle) {
    Worker* w = static_cast<Worker*>(handle);
    if (w == nullptr) return;
    stop_threads(w);
    if (w->listener >= 0) ::close(w->listener);
    delete w;
}

}  // extern "C"
