// An RDMA-style tagged-message endpoint: the host-staged bridge for links that are reliable
// connected queue pairs (InfiniBand / RoCE verbs), with everything above the wire written
// against a small provider interface so that it runs - and is tested, faults included - on an
// in-process fabric.  Role of the reference's ibverbs bridge (src/gpubridge/verbs/crate: endpoint,
// protocol, memory-registration cache, mock fabric); the design here is this library's own.
//
// Provider: what reliable connections give - post a receive buffer, post a two-sided send, post
// a one-sided write into memory the peer registered, poll completions, register memory.  Every
// pair of members has two connections ("lanes"): one for data-class messages, one for control,
// each with its own receive queue, so that a control message can never land in a slot posted
// for data; writes travel on the control lane, where the FIN that follows them keeps its place.  `MockFabric` implements it inside one process (one provider per member, completions
// through per-member queues, writes validated against the peer's registrations) and can be told
// to misbehave: fail, drop, delay or corrupt the n-th operation on a link, or kill a member.
// A provider over libibverbs has the same five calls; its headers are not in this image, so
// none is built here and `bridge="verbs"` reports that.
//
// Wire protocol, version 1.  Every two-sided message starts with a 48-byte header:
//     0  u32 magic 'GBR1'      4  u8 kind   5  u8 reserved   6  u16 sender index
//     8  u32 sequence of the message this belongs to (per sender and peer, from 1)
//    12  u32 payload bytes that follow the header in this send (EAGER only)
//    16  u32 data slots the sender has re-posted for this peer, cumulative
//    20  u32 control slots the sender has re-posted for this peer, cumulative
//    24  u64 tag            32  u64 length of the whole message
//    40  u64 GRANT: address to write to   (the remote key travels in the first payload word)
// Kinds: EAGER (header + the whole message, up to eager_max bytes), RTS (a large message is
// ready), GRANT (the receiver matched it: write here), FIN (written), CREDIT (counters only),
// BYE (the sender leaves in good order: it has sent what it owed, nothing more goes to it, and
// the end of its link is no failure; a member that vanishes without it breaks its peers).
// Flow control: every member pre-posts `data_slots` receive buffers per peer for EAGER and RTS
// and `ctrl_slots` for GRANT, FIN and CREDIT; a sender may only have as many unreturned
// messages of a class in flight as the peer has slots, and learns of re-posted slots from the
// cumulative counters every header carries.  One control slot is kept for CREDIT alone, so a
// member can always report; without that reserve two members that had filled each other's
// slots could wait for each other's report for ever.
// Large messages (more than eager_max bytes) are never copied: the receiver registers the
// user's buffer (cached, LRU, bounded), the sender writes into it in pieces, FIN follows the
// last piece on the same connection and therefore arrives after the data.
// Messages that arrive before their receive is posted are kept (EAGER: a copy, bounded by
// unexpected_max bytes; RTS: the request) and matched when it is.
//
// Failure rule: the first completion with an error, malformed header, overrun or deadline puts
// the endpoint into a broken state that fails every pending and future operation with the
// first reason; wait() never returns while the fabric may still touch the caller's memory.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <cerrno>
#include <cstdlib>
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <pthread.h>
#include <sched.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include "gb_tagged.h"

namespace {

using Clock = std::chrono::steady_clock;

enum Status { ST_OK = 0, ST_ERROR = 1, ST_REMOTE_ACCESS = 2, ST_FLUSHED = 3, ST_LENGTH = 4 };
enum Opcode { OC_SEND = 0, OC_RECV = 1, OC_WRITE = 2 };

struct Completion {
    uint64_t wr_id = 0;
    int status = ST_OK;
    int opcode = OC_SEND;
    uint32_t bytes = 0;
    int peer = -1;
};

struct Provider {
    virtual ~Provider() {}
    virtual int post_recv(int peer, int lane, uint64_t wr_id, void* buf, uint32_t len) = 0;
    virtual int post_send(int peer, int lane, uint64_t wr_id, const void* buf, uint32_t len) = 0;
    virtual int post_write(int peer, uint64_t wr_id, const void* local, uint64_t remote, uint32_t rkey,
                           uint32_t len) = 0;
    virtual int poll(Completion* out, int max, int timeout_ms) = 0;
    virtual int reg(void* addr, size_t len, uint32_t* rkey) = 0;
    virtual int dereg(uint32_t rkey) = 0;
    virtual void wake() = 0;
};

// ---- the in-process fabric ---------------------------------------------------------------------------
// F_SPURIOUS: both ends' polls are woken with nothing to report, `arg` times, and the operation
// goes through.  F_LATE: the operation is carried out at once but its completion reaches the
// poster `arg` milliseconds later - so the peer's answer may come back before it.
enum FaultKind { F_NONE = 0, F_ERROR = 1, F_DROP = 2, F_DELAY = 3, F_CORRUPT = 4, F_KILL = 5, F_SPURIOUS = 6,
                 F_LATE = 7 };

struct Fault {
    int kind = F_NONE, src = -1, dst = -1, opcode = -1;
    long nth = 0;                 // fires on the nth matching operation from now (1 = the next)
    int arg = 0;                  // F_DELAY: milliseconds
};

struct MockFabric;

struct MockProvider : Provider {
    MockFabric* fabric;
    int index;
    std::mutex mu;
    std::condition_variable cv;
    std::deque<Completion> cq;
    std::deque<std::pair<Clock::time_point, Completion>> late;    // completions held back by F_LATE
    struct Posted { uint64_t wr_id; char* buf; uint32_t len; };
    std::map<std::pair<int, int>, std::deque<Posted>> recvs; // by (source, lane)
    struct Region { char* base; size_t len; };
    std::map<uint32_t, Region> regions;
    uint32_t next_key = 0x1000;
    bool woken = false;

    MockProvider(MockFabric* f, int i) : fabric(f), index(i) {}
    void complete(const Completion& c) {
        { std::lock_guard<std::mutex> hold(mu); cq.push_back(c); }
        cv.notify_all();
    }
    void complete_later(const Completion& c, int milliseconds) {
        std::lock_guard<std::mutex> hold(mu);
        late.emplace_back(Clock::now() + std::chrono::milliseconds(milliseconds), c);
    }
    int post_recv(int peer, int lane, uint64_t wr_id, void* buf, uint32_t len) override;
    int post_send(int peer, int lane, uint64_t wr_id, const void* buf, uint32_t len) override;
    int post_write(int peer, uint64_t wr_id, const void* local, uint64_t remote, uint32_t rkey,
                   uint32_t len) override;
    // mu held.  Completions that were held back and are due now join the queue.
    void release_due() {
        const auto now = Clock::now();
        for (auto it = late.begin(); it != late.end();) {
            if (it->first <= now) { cq.push_back(it->second); it = late.erase(it); } else ++it;
        }
    }
    int poll(Completion* out, int max, int timeout_ms) override {
        std::unique_lock<std::mutex> hold(mu);
        release_due();
        if (cq.empty() && timeout_ms > 0) {
            auto until = Clock::now() + std::chrono::milliseconds(timeout_ms);
            for (auto& held : late) until = std::min(until, held.first);       // wake for the next one that falls due
            cv.wait_until(hold, until, [&] { return !cq.empty() || woken; });
            release_due();
        }
        woken = false;
        int n = 0;
        while (n < max && !cq.empty()) { out[n++] = cq.front(); cq.pop_front(); }
        return n;
    }
    int reg(void* addr, size_t len, uint32_t* rkey) override {
        std::lock_guard<std::mutex> hold(mu);
        *rkey = next_key++;
        regions[*rkey] = Region{static_cast<char*>(addr), len};
        return 0;
    }
    int dereg(uint32_t rkey) override {
        std::lock_guard<std::mutex> hold(mu);
        return regions.erase(rkey) ? 0 : -1;
    }
    void wake() override {
        { std::lock_guard<std::mutex> hold(mu); woken = true; }
        cv.notify_all();
    }
};

struct MockFabric {
    std::mutex mu;                                    // orders deliveries and fault bookkeeping
    std::vector<std::unique_ptr<MockProvider>> members;
    std::vector<Fault> faults;
    std::vector<bool> dead;
    struct Held { int src, dst, lane; uint64_t wr_id; std::vector<char> bytes; };
    std::deque<Held> waiting;                         // sends that found no receive posted (RNR)
    std::atomic<long> rnr{0}, sends{0}, writes{0}, dropped{0};

    explicit MockFabric(int n) : dead(n, false) {
        for (int i = 0; i < n; ++i) members.emplace_back(new MockProvider(this, i));
    }
    // mu held.  The fault that fires for this operation, if any.
    Fault take_fault(int src, int dst, int opcode) {
        for (size_t i = 0; i < faults.size(); ++i) {
            Fault& f = faults[i];
            if ((f.src >= 0 && f.src != src) || (f.dst >= 0 && f.dst != dst)) continue;
            if (f.opcode >= 0 && f.opcode != opcode) continue;
            if (--f.nth > 0) continue;
            Fault fired = f;
            faults.erase(faults.begin() + (long)i);
            return fired;
        }
        return Fault();
    }
    // mu held.
    void deliver(int src, int dst, int lane, uint64_t wr_id, const char* bytes, uint32_t len, bool corrupt,
                 int late_ms = 0) {
        MockProvider& to = *members[dst];
        MockProvider::Posted slot;
        {
            std::lock_guard<std::mutex> hold(to.mu);
            slot = to.recvs[{src, lane}].front();
            to.recvs[{src, lane}].pop_front();
        }
        Completion s, r;
        s.wr_id = wr_id; s.opcode = OC_SEND; s.peer = dst;
        r.wr_id = slot.wr_id; r.opcode = OC_RECV; r.peer = src;
        if (len > slot.len) {
            s.status = r.status = ST_LENGTH;
        } else {
            std::memcpy(slot.buf, bytes, len);
            if (corrupt && len > 0) slot.buf[0] ^= 0x5A;
            r.bytes = len;
        }
        if (late_ms > 0) members[src]->complete_later(s, late_ms); else members[src]->complete(s);
        to.complete(r);
    }
    void spurious(int a, int b, int times) {
        for (int i = 0; i < (times > 0 ? times : 1); ++i) { members[a]->wake(); members[b]->wake(); }
    }
};

int MockProvider::post_recv(int peer, int lane, uint64_t wr_id, void* buf, uint32_t len) {
    std::lock_guard<std::mutex> order(fabric->mu);
    if (fabric->dead[index] || fabric->dead[peer]) {
        Completion c; c.wr_id = wr_id; c.status = ST_FLUSHED; c.opcode = OC_RECV; c.peer = peer;
        complete(c);
        return 0;
    }
    { std::lock_guard<std::mutex> hold(mu); recvs[{peer, lane}].push_back(Posted{wr_id, static_cast<char*>(buf), len}); }
    // a send that was waiting for this receive goes through now
    for (auto it = fabric->waiting.begin(); it != fabric->waiting.end(); ++it) {
        if (it->src == peer && it->dst == index && it->lane == lane) {
            MockFabric::Held held = std::move(*it);
            fabric->waiting.erase(it);
            fabric->deliver(held.src, held.dst, lane, held.wr_id, held.bytes.data(), (uint32_t)held.bytes.size(), false);
            break;
        }
    }
    return 0;
}

int MockProvider::post_send(int peer, int lane, uint64_t wr_id, const void* buf, uint32_t len) {
    std::unique_lock<std::mutex> order(fabric->mu);
    fabric->sends.fetch_add(1);
    Completion c; c.wr_id = wr_id; c.opcode = OC_SEND; c.peer = peer;
    if (fabric->dead[index] || fabric->dead[peer]) { c.status = ST_FLUSHED; complete(c); return 0; }
    const Fault f = fabric->take_fault(index, peer, OC_SEND);
    if (f.kind == F_ERROR) { c.status = ST_ERROR; complete(c); return 0; }
    if (f.kind == F_DROP) { fabric->dropped.fetch_add(1); return 0; }
    if (f.kind == F_KILL) {
        fabric->dead[peer] = true;
        c.status = ST_FLUSHED; complete(c);
        fabric->members[peer]->wake();
        return 0;
    }
    if (f.kind == F_DELAY) {
        order.unlock();
        std::this_thread::sleep_for(std::chrono::milliseconds(f.arg));
        order.lock();
    }
    if (f.kind == F_SPURIOUS) fabric->spurious(index, peer, f.arg);
    bool posted;
    {
        std::lock_guard<std::mutex> hold(fabric->members[peer]->mu);
        posted = !fabric->members[peer]->recvs[{index, lane}].empty();
    }
    if (!posted) {                                    // receiver not ready: the link retries
        fabric->rnr.fetch_add(1);
        MockFabric::Held held{index, peer, lane, wr_id, std::vector<char>((const char*)buf, (const char*)buf + len)};
        fabric->waiting.push_back(std::move(held));
        return 0;
    }
    fabric->deliver(index, peer, lane, wr_id, static_cast<const char*>(buf), len, f.kind == F_CORRUPT,
                    f.kind == F_LATE ? f.arg : 0);
    return 0;
}

int MockProvider::post_write(int peer, uint64_t wr_id, const void* local, uint64_t remote, uint32_t rkey,
                             uint32_t len) {
    std::unique_lock<std::mutex> order(fabric->mu);
    fabric->writes.fetch_add(1);
    Completion c; c.wr_id = wr_id; c.opcode = OC_WRITE; c.peer = peer; c.bytes = len;
    if (fabric->dead[index] || fabric->dead[peer]) { c.status = ST_FLUSHED; complete(c); return 0; }
    const Fault f = fabric->take_fault(index, peer, OC_WRITE);
    if (f.kind == F_ERROR) { c.status = ST_ERROR; complete(c); return 0; }
    if (f.kind == F_DROP) { fabric->dropped.fetch_add(1); return 0; }
    if (f.kind == F_KILL) { fabric->dead[peer] = true; c.status = ST_FLUSHED; complete(c); fabric->members[peer]->wake(); return 0; }
    if (f.kind == F_DELAY) {
        order.unlock();
        std::this_thread::sleep_for(std::chrono::milliseconds(f.arg));
        order.lock();
    }
    if (f.kind == F_SPURIOUS) fabric->spurious(index, peer, f.arg);
    MockProvider& to = *fabric->members[peer];
    {
        std::lock_guard<std::mutex> hold(to.mu);
        auto it = to.regions.find(rkey);
        const char* at = reinterpret_cast<const char*>(remote);
        if (it == to.regions.end() || at < it->second.base || at + len > it->second.base + it->second.len) {
            c.status = ST_REMOTE_ACCESS;
        } else {
            std::memcpy(const_cast<char*>(at), local, len);
        }
    }
    if (f.kind == F_LATE) complete_later(c, f.arg); else complete(c);
    return 0;
}

// ---- a provider over stream sockets: members in different processes ----------------------------------
//
// Names: a plain string is an abstract Unix-domain socket name (the processes of one host);
// "tcp://a.b.c.d:port" is a TCP address (port 0 when listening: the system picks one, and
// bound_name() says which), so the same provider also joins processes on different hosts -
// the endpoint's protocol over an ordinary network, where no adapter exists.
//
// The same queue-pair semantics as the in-process fabric, carried over one stream socket per
// pair of members (abstract socket names, so nothing is left in the file system): a SEND is
// matched to the receive posted for (source, lane) and completes at both ends; a WRITE names a
// registered region of the destination and lands there without the destination's endpoint
// taking part, completing at the source when the destination has acknowledged it (refused, with
// "remote access", when the key or the range is not registered any more).  A reader and a
// writer thread per connection: posting never blocks the caller, and a reader never waits for
// the endpoint above it (credits guarantee a posted receive for every SEND), so the sockets
// always drain.  A peer that goes away flushes everything posted for it.  This is what lets the
// whole bridge run between processes where no adapter exists; it is not a fast path.
struct SocketProvider : Provider {
    enum Frame : uint32_t { FR_SEND = 1, FR_WRITE = 2, FR_ACK = 3 };
    struct Wire { uint32_t type, lane; uint64_t wr_id, remote; uint32_t rkey, len; };   // 32 bytes
    struct Out { Wire w; const char* data; int opcode; };
    struct Link {
        int fd = -1;
        std::thread reader, writer;
        std::mutex mu;
        std::condition_variable cv;
        std::deque<Out> queue;
        bool gone = false;                 // nothing can be sent on this link any more
        bool eof = false;                  // ... and nothing will arrive on it: the reader has ended
        bool busy = false;                 // the writer is putting a frame on the wire
    };
    int index, count;
    int listener = -1;
    std::vector<std::unique_ptr<Link>> links;
    std::mutex mu;
    std::condition_variable cv, posted_cv;
    std::deque<Completion> cq;
    std::deque<std::pair<Clock::time_point, Completion>> late;    // completions held back by F_LATE
    struct Posted { uint64_t wr_id; char* buf; uint32_t len; };
    std::map<std::pair<int, int>, std::deque<Posted>> recvs;
    struct Region { char* base; size_t len; };
    std::map<uint32_t, Region> regions;
    uint32_t next_key = 0x2000;
    bool woken = false, closing = false;

    SocketProvider(int i, int n) : index(i), count(n) {
        for (int p = 0; p < n; ++p) links.emplace_back(new Link());
    }
    ~SocketProvider() override { shutdown_all(); }

    std::string bound;                                 // the name peers can reach this member under
    static bool is_tcp(const std::string& name) { return name.rfind("tcp://", 0) == 0; }
    static bool tcp_address(const std::string& name, sockaddr_in* a) {
        const std::string rest = name.substr(6);
        const size_t colon = rest.rfind(':');
        if (colon == std::string::npos) return false;
        std::memset(a, 0, sizeof(*a));
        a->sin_family = AF_INET;
        a->sin_port = htons((uint16_t)std::atoi(rest.c_str() + colon + 1));
        return ::inet_pton(AF_INET, rest.substr(0, colon).c_str(), &a->sin_addr) == 1;
    }
    static sockaddr_un address(const std::string& name, socklen_t* len) {
        sockaddr_un a;
        std::memset(&a, 0, sizeof(a));
        a.sun_family = AF_UNIX;
        const size_t n = name.size() < sizeof(a.sun_path) - 2 ? name.size() : sizeof(a.sun_path) - 2;
        std::memcpy(a.sun_path + 1, name.data(), n);            // leading NUL: the abstract namespace
        *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
        return a;
    }
    bool listen_on(const std::string& name) {
        bound = name;
        if (is_tcp(name)) {
            sockaddr_in a;
            if (!tcp_address(name, &a)) return false;
            listener = ::socket(AF_INET, SOCK_STREAM, 0);
            if (listener < 0) return false;
            const int yes = 1;
            ::setsockopt(listener, SOL_SOCKET, SO_REUSEADDR, &yes, sizeof(yes));
            if (::bind(listener, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0 || ::listen(listener, 64) != 0)
                return false;
            socklen_t len = sizeof(a);
            ::getsockname(listener, reinterpret_cast<sockaddr*>(&a), &len);     // the port the system chose
            char ip[INET_ADDRSTRLEN];
            ::inet_ntop(AF_INET, &a.sin_addr, ip, sizeof(ip));
            bound = std::string("tcp://") + ip + ":" + std::to_string(ntohs(a.sin_port));
            return true;
        }
        listener = ::socket(AF_UNIX, SOCK_STREAM, 0);
        if (listener < 0) return false;
        socklen_t len;
        sockaddr_un a = address(name, &len);
        return ::bind(listener, reinterpret_cast<sockaddr*>(&a), len) == 0 && ::listen(listener, 64) == 0;
    }
    // A connected socket to `name`, or -1.
    static int dial(const std::string& name) {
        if (is_tcp(name)) {
            sockaddr_in a;
            if (!tcp_address(name, &a)) return -1;
            const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
            if (fd >= 0 && ::connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) == 0) {
                const int yes = 1;
                ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &yes, sizeof(yes));
                return fd;
            }
            if (fd >= 0) ::close(fd);
            return -1;
        }
        socklen_t len;
        sockaddr_un a = address(name, &len);
        const int fd = ::socket(AF_UNIX, SOCK_STREAM, 0);
        if (fd >= 0 && ::connect(fd, reinterpret_cast<sockaddr*>(&a), len) == 0) return fd;
        if (fd >= 0) ::close(fd);
        return -1;
    }
    static bool write_all(int fd, const void* data, size_t n) {
        const char* p = static_cast<const char*>(data);
        while (n) {
            const ssize_t k = ::send(fd, p, n, MSG_NOSIGNAL);
            if (k <= 0) { if (k < 0 && errno == EINTR) continue; return false; }
            p += k; n -= (size_t)k;
        }
        return true;
    }
    static bool read_all(int fd, void* data, size_t n) {
        char* p = static_cast<char*>(data);
        while (n) {
            const ssize_t k = ::recv(fd, p, n, 0);
            if (k <= 0) { if (k < 0 && errno == EINTR) continue; return false; }
            p += k; n -= (size_t)k;
        }
        return true;
    }
    // Members with a lower index dial; every connection opens with the dialler's index.
    bool connect_all(const std::vector<std::string>& names, double timeout_s, std::string* why) {
        const auto deadline = Clock::now() + std::chrono::duration<double>(timeout_s);
        for (int p = index + 1; p < count; ++p) {
            int fd = -1;
            for (;;) {
                fd = dial(names[p]);
                if (fd >= 0) break;
                if (Clock::now() > deadline) { *why = "member " + std::to_string(p) + " never listened"; return false; }
                std::this_thread::sleep_for(std::chrono::milliseconds(20));
            }
            const uint32_t me = (uint32_t)index;
            if (!write_all(fd, &me, 4)) { *why = "handshake failed"; ::close(fd); return false; }
            links[p]->fd = fd;
        }
        for (int got = 0; got < index; ++got) {
            pollfd wait{listener, POLLIN, 0};
            const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count();
            if (left <= 0 || ::poll(&wait, 1, (int)left) <= 0) { *why = "a lower member never dialled"; return false; }
            const int fd = ::accept(listener, nullptr, nullptr);
            if (fd >= 0 && is_tcp(bound)) {
                const int yes = 1;
                ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &yes, sizeof(yes));
            }
            uint32_t who = 0;
            if (fd < 0 || !read_all(fd, &who, 4) || (int)who >= index || links[who]->fd >= 0) {
                if (fd >= 0) ::close(fd);
                *why = "a connection with no valid member index";
                return false;
            }
            links[who]->fd = fd;
        }
        ::close(listener);
        listener = -1;
        for (int p = 0; p < count; ++p) {
            if (p == index) continue;
            Link* l = links[p].get();
            l->reader = std::thread([this, p] { read_loop(p); });
            l->writer = std::thread([this, p] { write_loop(p); });
        }
        return true;
    }
    void complete(const Completion& c) {
        { std::lock_guard<std::mutex> hold(mu); cq.push_back(c); }
        cv.notify_all();
    }
    void complete_later(const Completion& c, int milliseconds) {
        std::lock_guard<std::mutex> hold(mu);
        late.emplace_back(Clock::now() + std::chrono::milliseconds(milliseconds), c);
    }
    void flush_peer(int peer) {
        std::deque<Posted> lost;
        {
            std::lock_guard<std::mutex> hold(mu);
            for (int lane = 0; lane < 2; ++lane) {
                auto& q = recvs[{peer, lane}];
                while (!q.empty()) { lost.push_back(q.front()); q.pop_front(); }
            }
        }
        for (const Posted& r : lost) {
            Completion c; c.wr_id = r.wr_id; c.status = ST_FLUSHED; c.opcode = OC_RECV; c.peer = peer;
            complete(c);
        }
        { std::lock_guard<std::mutex> hold(links[peer]->mu); links[peer]->eof = true; }
        send_side_dead(peer);
        posted_cv.notify_all();
    }
    // Nothing more can be sent to `peer` (a write failed, or its stream ended): what is queued
    // fails.  What the peer sent before it went may still be unread - the reader decides when
    // the receives are lost, not the writer.
    void send_side_dead(int peer) {
        Link& l = *links[peer];
        std::deque<Out> unsent;
        { std::lock_guard<std::mutex> hold(l.mu); l.gone = true; unsent.swap(l.queue); }
        l.cv.notify_all();
        for (const Out& o : unsent) {
            if (o.w.type == FR_ACK) continue;
            Completion c; c.wr_id = o.w.wr_id; c.status = ST_FLUSHED; c.opcode = o.opcode; c.peer = peer;
            complete(c);
        }
    }
    void write_loop(int peer) {
        Link& l = *links[peer];
        for (;;) {
            Out o;
            {
                std::unique_lock<std::mutex> hold(l.mu);
                l.cv.wait(hold, [&] { return l.gone || !l.queue.empty(); });
                if (l.gone) return;
                o = l.queue.front();
                l.queue.pop_front();
                l.busy = true;
            }
            const bool ok = write_all(l.fd, &o.w, sizeof(Wire)) && (o.w.len == 0 || o.data == nullptr ||
                                                                    write_all(l.fd, o.data, o.w.len));
            { std::lock_guard<std::mutex> hold(l.mu); l.busy = false; }
            l.cv.notify_all();
            if (o.w.type == FR_ACK) { if (!ok) { send_side_dead(peer); return; } continue; }
            if (!ok) {
                Completion c; c.wr_id = o.w.wr_id; c.status = ST_FLUSHED; c.opcode = o.opcode; c.peer = peer;
                complete(c);
                send_side_dead(peer);
                return;
            }
            if (o.w.type == FR_SEND) {                 // a WRITE completes when its acknowledgement arrives
                Completion c; c.wr_id = o.w.wr_id; c.opcode = OC_SEND; c.peer = peer;
                complete(c);
            }
        }
    }
    void read_loop(int peer) {
        Link& l = *links[peer];
        std::vector<char> sink;
        for (;;) {
            Wire w;
            if (!read_all(l.fd, &w, sizeof(Wire))) break;
            if (w.type == FR_SEND) {
                Posted slot{0, nullptr, 0};
                {
                    std::unique_lock<std::mutex> hold(mu);
                    posted_cv.wait(hold, [&] { return closing || !recvs[{peer, (int)w.lane}].empty(); });
                    if (closing) return;
                    slot = recvs[{peer, (int)w.lane}].front();
                    recvs[{peer, (int)w.lane}].pop_front();
                }
                Completion c; c.wr_id = slot.wr_id; c.opcode = OC_RECV; c.peer = peer;
                if (w.len > slot.len) {
                    sink.resize(w.len);
                    if (!read_all(l.fd, sink.data(), w.len)) break;
                    c.status = ST_LENGTH;
                } else {
                    if (w.len && !read_all(l.fd, slot.buf, w.len)) { c.status = ST_FLUSHED; complete(c); break; }
                    c.bytes = w.len;
                }
                complete(c);
            } else if (w.type == FR_WRITE) {
                char* at = reinterpret_cast<char*>(w.remote);
                bool allowed;
                {
                    // the registration is held for the length of the copy: a region that is
                    // dropped while data lands would be memory the caller already reuses
                    std::unique_lock<std::mutex> hold(mu);
                    auto it = regions.find(w.rkey);
                    allowed = it != regions.end() && at >= it->second.base &&
                              at + w.len <= it->second.base + it->second.len;
                    if (allowed) {
                        if (w.len && !read_all(l.fd, at, w.len)) { hold.unlock(); goto out; }
                    }
                }
                if (!allowed) {
                    sink.resize(w.len);
                    if (w.len && !read_all(l.fd, sink.data(), w.len)) break;
                }
                Out ack;
                ack.w = Wire{FR_ACK, (uint32_t)(allowed ? ST_OK : ST_REMOTE_ACCESS), w.wr_id, 0, 0, 0};
                ack.data = nullptr; ack.opcode = OC_WRITE;
                { std::lock_guard<std::mutex> hold(l.mu); if (!l.gone) l.queue.push_back(ack); }
                l.cv.notify_all();
            } else if (w.type == FR_ACK) {
                Completion c; c.wr_id = w.wr_id; c.opcode = OC_WRITE; c.peer = peer; c.status = (int)w.lane;
                complete(c);
            } else {
                break;                                 // not this protocol
            }
        }
    out:
        if (!closing) flush_peer(peer);
    }
    int enqueue(int peer, const Out& o) {
        Link& l = *links[peer];
        bool gone;
        { std::lock_guard<std::mutex> hold(l.mu); gone = l.gone || l.fd < 0; if (!gone) l.queue.push_back(o); }
        if (gone) {
            Completion c; c.wr_id = o.w.wr_id; c.status = ST_FLUSHED; c.opcode = o.opcode; c.peer = peer;
            complete(c);
        } else {
            l.cv.notify_all();
        }
        return 0;
    }
    int post_recv(int peer, int lane, uint64_t wr_id, void* buf, uint32_t len) override {
        bool gone;
        { std::lock_guard<std::mutex> hold(links[peer]->mu); gone = links[peer]->eof; }
        if (gone) {
            Completion c; c.wr_id = wr_id; c.status = ST_FLUSHED; c.opcode = OC_RECV; c.peer = peer;
            complete(c);
            return 0;
        }
        { std::lock_guard<std::mutex> hold(mu); recvs[{peer, lane}].push_back(Posted{wr_id, static_cast<char*>(buf), len}); }
        posted_cv.notify_all();
        return 0;
    }
    int post_send(int peer, int lane, uint64_t wr_id, const void* buf, uint32_t len) override {
        Out o;
        o.w = Wire{FR_SEND, (uint32_t)lane, wr_id, 0, 0, len};
        o.data = static_cast<const char*>(buf); o.opcode = OC_SEND;
        return enqueue(peer, o);
    }
    int post_write(int peer, uint64_t wr_id, const void* local, uint64_t remote, uint32_t rkey,
                   uint32_t len) override {
        Out o;
        o.w = Wire{FR_WRITE, 0, wr_id, remote, rkey, len};
        o.data = static_cast<const char*>(local); o.opcode = OC_WRITE;
        return enqueue(peer, o);
    }
    // mu held.  Completions that were held back and are due now join the queue.
    void release_due() {
        const auto now = Clock::now();
        for (auto it = late.begin(); it != late.end();) {
            if (it->first <= now) { cq.push_back(it->second); it = late.erase(it); } else ++it;
        }
    }
    int poll(Completion* out, int max, int timeout_ms) override {
        std::unique_lock<std::mutex> hold(mu);
        release_due();
        if (cq.empty() && timeout_ms > 0) {
            auto until = Clock::now() + std::chrono::milliseconds(timeout_ms);
            for (auto& held : late) until = std::min(until, held.first);       // wake for the next one that falls due
            cv.wait_until(hold, until, [&] { return !cq.empty() || woken; });
            release_due();
        }
        woken = false;
        int n = 0;
        while (n < max && !cq.empty()) { out[n++] = cq.front(); cq.pop_front(); }
        return n;
    }
    int reg(void* addr, size_t len, uint32_t* rkey) override {
        std::lock_guard<std::mutex> hold(mu);
        *rkey = next_key++;
        regions[*rkey] = Region{static_cast<char*>(addr), len};
        return 0;
    }
    int dereg(uint32_t rkey) override {
        std::lock_guard<std::mutex> hold(mu);              // waits for a copy into the region to end
        return regions.erase(rkey) ? 0 : -1;
    }
    void wake() override {
        { std::lock_guard<std::mutex> hold(mu); woken = true; }
        cv.notify_all();
    }
    // Give what is queued for the wire (acknowledgements of the peers' last writes among it)
    // the time to leave: a member that closes right after its last operation completed must
    // not take its peers' last messages with it.
    void drain(double seconds) {
        const auto until = Clock::now() + std::chrono::duration<double>(seconds);
        for (auto& l : links) {
            std::unique_lock<std::mutex> hold(l->mu);
            l->cv.wait_until(hold, until, [&] { return l->gone || (l->queue.empty() && !l->busy); });
        }
    }
    void shutdown_all() {
        { std::lock_guard<std::mutex> hold(mu); if (closing) return; closing = true; regions.clear(); recvs.clear(); }
        posted_cv.notify_all();
        if (listener >= 0) { ::close(listener); listener = -1; }
        for (auto& l : links) {
            if (l->fd >= 0) ::shutdown(l->fd, SHUT_RDWR);
            { std::lock_guard<std::mutex> hold(l->mu); l->gone = true; }
            l->cv.notify_all();
        }
        for (auto& l : links) {
            if (l->reader.joinable()) l->reader.join();
            if (l->writer.joinable()) l->writer.join();
            if (l->fd >= 0) { ::close(l->fd); l->fd = -1; }
        }
    }
};

// ---- registrations of user memory, cached ---------------------------------------------------------------
struct MrCache {
    struct Entry { char* base; size_t len; uint32_t rkey; };
    Provider* provider;
    size_t capacity;
    std::list<Entry> lru;                               // most recently used first
    long hits = 0, misses = 0, evictions = 0;

    MrCache(Provider* p, size_t cap) : provider(p), capacity(cap ? cap : 1) {}
    // The remote key of a registration that covers [addr, addr + len); registers on a miss.
    bool lookup(void* addr, size_t len, uint32_t* rkey) {
        char* a = static_cast<char*>(addr);
        for (auto it = lru.begin(); it != lru.end(); ++it) {
            if (a >= it->base && a + len <= it->base + it->len) {
                ++hits;
                *rkey = it->rkey;
                lru.splice(lru.begin(), lru, it);
                return true;
            }
        }
        ++misses;
        uint32_t key = 0;
        if (provider->reg(addr, len, &key) != 0) return false;
        lru.push_front(Entry{a, len, key});
        while (lru.size() > capacity) {
            provider->dereg(lru.back().rkey);
            lru.pop_back();
            ++evictions;
        }
        *rkey = key;
        return true;
    }
    // The caller is about to free or reuse [addr, addr + len): forget what overlaps it.
    int invalidate(void* addr, size_t len) {
        char* a = static_cast<char*>(addr);
        int dropped = 0;
        for (auto it = lru.begin(); it != lru.end();) {
            if (a < it->base + it->len && it->base < a + len) {
                provider->dereg(it->rkey);
                it = lru.erase(it);
                ++dropped;
            } else ++it;
        }
        return dropped;
    }
    void clear() {
        for (auto& e : lru) provider->dereg(e.rkey);
        lru.clear();
    }
};

// ---- the protocol ---------------------------------------------------------------------------------------------
constexpr uint32_t MAGIC = 0x31524247u;          // "GBR1"
constexpr int HEADER_BYTES = 48;
enum Kind { K_EAGER = 1, K_RTS = 2, K_GRANT = 3, K_FIN = 4, K_CREDIT = 5, K_BYE = 6 };

struct Header {
    uint8_t kind = 0;
    uint16_t sender = 0;
    uint32_t seq = 0, payload = 0, data_freed = 0, ctrl_freed = 0;
    uint64_t tag = 0, length = 0, address = 0;
};

void encode(const Header& h, char* out) {
    std::memset(out, 0, HEADER_BYTES);
    std::memcpy(out, &MAGIC, 4);
    out[4] = (char)h.kind;
    std::memcpy(out + 6, &h.sender, 2);
    std::memcpy(out + 8, &h.seq, 4);
    std::memcpy(out + 12, &h.payload, 4);
    std::memcpy(out + 16, &h.data_freed, 4);
    std::memcpy(out + 20, &h.ctrl_freed, 4);
    std::memcpy(out + 24, &h.tag, 8);
    std::memcpy(out + 32, &h.length, 8);
    std::memcpy(out + 40, &h.address, 8);
}

// Empty string when the bytes are a well-formed message of `received` bytes.
std::string decode(const char* in, uint32_t received, Header* h) {
    if (received < HEADER_BYTES) return "a message shorter than its header";
    uint32_t magic;
    std::memcpy(&magic, in, 4);
    if (magic != MAGIC) return "a message without the protocol's magic number";
    h->kind = (uint8_t)in[4];
    std::memcpy(&h->sender, in + 6, 2);
    std::memcpy(&h->seq, in + 8, 4);
    std::memcpy(&h->payload, in + 12, 4);
    std::memcpy(&h->data_freed, in + 16, 4);
    std::memcpy(&h->ctrl_freed, in + 20, 4);
    std::memcpy(&h->tag, in + 24, 8);
    std::memcpy(&h->length, in + 32, 8);
    std::memcpy(&h->address, in + 40, 8);
    if (h->kind < K_EAGER || h->kind > K_BYE) return "a message of unknown kind " + std::to_string(h->kind);
    if (received != HEADER_BYTES + h->payload) return "a message whose length disagrees with its header";
    if (h->kind == K_EAGER && h->payload != h->length) return "an eager message that is not whole";
    if (h->kind == K_GRANT && (h->payload != 4 || h->address == 0)) return "a write grant without key or address";
    if (h->kind != K_EAGER && h->kind != K_GRANT && h->payload != 0) return "a control message with a payload";
    if ((h->kind == K_RTS || h->kind == K_GRANT || h->kind == K_FIN) && h->length == 0)
        return "a rendezvous for an empty message";
    return "";
}

struct Config {
    uint32_t eager_max = 16384;          // larger messages go by rendezvous
    uint32_t data_slots = 16, ctrl_slots = 8;
    uint32_t max_write = 1u << 20;       // bytes per one-sided write
    uint64_t unexpected_max = 64ull << 20;
    uint32_t mr_cache = 64;
    int poll_ms = 5;                     // how long the progress thread sleeps in poll
    int spin = 0;                        // "latency" progress: poll without sleeping, this many
                                         // empty rounds before a short sleep is allowed again
    int cpu = -1;                        // pin the progress thread to this CPU (-1: leave it)
};

struct Op {
    bool sending = false;
    int peer = 0;
    uint64_t tag = 0;
    char* data = nullptr;
    uint64_t length = 0;
    int state = 0;                       // 0 pending, 1 done, 2 failed
    uint32_t seq = 0;                    // rendezvous: the sender's message number
    uint32_t writes_left = 0;
};

struct Endpoint : GbTaggedWorker {
    Provider* provider = nullptr;
    MockFabric* mock = nullptr;
    std::unique_ptr<Provider> owned;               // a provider that lives and dies with this endpoint
    int me = 0, count = 0;
    Config cfg;
    std::mutex mu;
    std::condition_variable done;
    std::map<long, Op> ops;
    long next_id = 1;
    bool broken = false, closing = false;
    std::string error;
    std::thread progress;
    std::unique_ptr<MrCache> mrs;

    struct Peer {
        std::vector<std::vector<char>> data_slots, ctrl_slots;       // receive buffers
        uint32_t sent_data = 0, sent_ctrl = 0;                        // messages of each class sent
        uint32_t seen_data_freed = 0, seen_ctrl_freed = 0;            // the peer's counters, last seen
        uint32_t freed_data = 0, freed_ctrl = 0;                      // slots re-posted here, cumulative
        uint32_t reported_data = 0, reported_ctrl = 0;                // ... and last told to the peer
        uint32_t next_seq = 1;
        bool departed = false;                                        // it said goodbye: nothing more goes to it
        std::deque<long> posted;                                      // receives waiting, in order
        struct Early { Header h; std::vector<char> bytes; };
        std::deque<Early> early;                                      // messages waiting for a receive
        std::deque<std::vector<char>> backlog_data, backlog_ctrl;     // encoded, waiting for a credit
        std::map<uint32_t, long> sends_by_seq, recvs_by_seq;          // rendezvous in flight
    };
    std::vector<Peer> peers;
    std::map<uint64_t, std::vector<char>> in_flight;                  // send buffers until completed
    std::map<uint64_t, bool> reports;                                 // sends that carry counters only
    uint64_t next_wr = 1;
    uint64_t unexpected_bytes = 0;
    // wr_id layout: bit 63 receive, bit 62 control class, bits 32-47 peer, low 32 slot / serial
    struct Counters {
        long eager_sent = 0, rndv_sent = 0, eager_recv = 0, rndv_recv = 0, bytes_sent = 0, bytes_recv = 0;
        long unexpected = 0, credit_msgs = 0, credit_stalls = 0, completions = 0, errors = 0, writes = 0;
    } n;

    // -- GbTaggedWorker ---------------------------------------------------------------------------------------
    int members() const override { return count; }
    int index() const override { return me; }
    long send(int peer, const void* data, uint64_t length, uint64_t tag) override;
    long recv(int peer, void* data, uint64_t length, uint64_t tag) override;
    int wait(const long* ids, int n_ids, double timeout_s) override;
    void stop() override { std::unique_lock<std::mutex> hold(mu); break_locked("stopped after a failed post"); }
    void fail(const char* why) override { std::unique_lock<std::mutex> hold(mu); break_locked(why); }

    // -- internals (mu held unless said otherwise) ------------------------------------------------------------
    void break_locked(const std::string& why) {
        if (!broken) {
            broken = true; error = why; ++n.errors;
            // Revoke every registration: a peer's late write is then refused by the fabric
            // instead of landing in memory the caller is about to reuse.  (A provider over real
            // queue pairs also moves them to the error state here, which flushes what is posted.)
            if (mrs) mrs->clear();
        }
        for (auto& kv : ops) if (kv.second.state == 0) kv.second.state = 2;
        done.notify_all();
    }
    uint32_t data_credits(const Peer& p) const { return cfg.data_slots - (p.sent_data - p.seen_data_freed); }
    uint32_t ctrl_credits(const Peer& p) const { return cfg.ctrl_slots - (p.sent_ctrl - p.seen_ctrl_freed); }

    void post_slot(int peer, bool ctrl, uint32_t slot) {
        Peer& p = peers[peer];
        std::vector<char>& buf = ctrl ? p.ctrl_slots[slot] : p.data_slots[slot];
        const uint64_t wr = (1ull << 63) | (ctrl ? 1ull << 62 : 0) | ((uint64_t)peer << 32) | slot;
        provider->post_recv(peer, ctrl ? 1 : 0, wr, buf.data(), (uint32_t)buf.size());
    }
    // Put an encoded message on the wire, or queue it until the peer has a slot for its class.
    void transmit(int peer, bool ctrl, std::vector<char>&& bytes, bool is_credit = false) {
        Peer& p = peers[peer];
        if (p.departed) {
            if (!ctrl || !is_credit) break_locked("member " + std::to_string(peer) + " has left the bridge");
            return;
        }
        std::deque<std::vector<char>>& backlog = ctrl ? p.backlog_ctrl : p.backlog_data;
        const uint32_t have = ctrl ? ctrl_credits(p) : data_credits(p);
        const uint32_t need = ctrl && !is_credit ? 2u : 1u;             // the last control slot is CREDIT's
        if (!backlog.empty() || have < need) {
            if (is_credit) return;                                       // a later report says the same
            ++n.credit_stalls;
            backlog.push_back(std::move(bytes));
            return;
        }
        put(peer, ctrl, std::move(bytes));
    }
    uint64_t put(int peer, bool ctrl, std::vector<char>&& bytes) {
        Peer& p = peers[peer];
        // every header carries the latest counters
        std::memcpy(bytes.data() + 16, &p.freed_data, 4);
        std::memcpy(bytes.data() + 20, &p.freed_ctrl, 4);
        p.reported_data = p.freed_data;
        p.reported_ctrl = p.freed_ctrl;
        (ctrl ? p.sent_ctrl : p.sent_data)++;
        const uint64_t wr = next_wr++;
        auto& kept = in_flight[wr] = std::move(bytes);
        provider->post_send(peer, ctrl ? 1 : 0, wr, kept.data(), (uint32_t)kept.size());
        return wr;
    }
    void drain_backlogs(int peer) {
        Peer& p = peers[peer];
        while (!p.backlog_ctrl.empty() && ctrl_credits(p) >= 2) {
            std::vector<char> bytes = std::move(p.backlog_ctrl.front());
            p.backlog_ctrl.pop_front();
            put(peer, true, std::move(bytes));
        }
        while (!p.backlog_data.empty() && data_credits(p) >= 1) {
            std::vector<char> bytes = std::move(p.backlog_data.front());
            p.backlog_data.pop_front();
            put(peer, false, std::move(bytes));
        }
    }
    void maybe_report(int peer) {
        Peer& p = peers[peer];
        const bool due = p.freed_data - p.reported_data >= (cfg.data_slots + 1) / 2 ||
                         p.freed_ctrl - p.reported_ctrl >= (cfg.ctrl_slots + 1) / 2;
        if (!due || p.departed || ctrl_credits(p) < 1 || !p.backlog_ctrl.empty()) return;
        Header h;
        h.kind = K_CREDIT; h.sender = (uint16_t)me;
        std::vector<char> bytes(HEADER_BYTES);
        encode(h, bytes.data());
        ++n.credit_msgs;
        reports[put(peer, true, std::move(bytes))] = true;
    }
    // Leaving in good order: tell every peer that nothing more comes from here and that nothing
    // more should be sent here.  A peer that has read this neither reports to this member any
    // more nor takes the end of its stream for a failure.
    void say_goodbye() {
        for (int peer = 0; peer < count; ++peer) {
            Peer& p = peers[peer];
            if (peer == me || p.departed || ctrl_credits(p) < 1) continue;
            Header h;
            h.kind = K_BYE; h.sender = (uint16_t)me;
            std::vector<char> bytes(HEADER_BYTES);
            encode(h, bytes.data());
            reports[put(peer, true, std::move(bytes))] = true;
        }
    }
    void send_control(int peer, const Header& h, const char* payload = nullptr, uint32_t payload_len = 0) {
        std::vector<char> bytes(HEADER_BYTES + payload_len);
        encode(h, bytes.data());
        if (payload_len) std::memcpy(bytes.data() + HEADER_BYTES, payload, payload_len);
        transmit(peer, true, std::move(bytes));
    }
    void grant(int peer, const Header& rts, long op_id) {
        Op& op = ops[op_id];
        if (rts.length != op.length) {
            break_locked("message of " + std::to_string(rts.length) + " bytes from member " + std::to_string(peer) +
                         " met a receive of " + std::to_string(op.length) + " (tag " + std::to_string(rts.tag) + ")");
            return;
        }
        uint32_t rkey = 0;
        if (!mrs->lookup(op.data, op.length, &rkey)) { break_locked("memory registration failed"); return; }
        peers[peer].recvs_by_seq[rts.seq] = op_id;
        Header h;
        h.kind = K_GRANT; h.sender = (uint16_t)me; h.seq = rts.seq; h.payload = 4;
        h.tag = rts.tag; h.length = rts.length; h.address = reinterpret_cast<uint64_t>(op.data);
        send_control(peer, h, reinterpret_cast<const char*>(&rkey), 4);
    }
    void finish(long op_id, bool ok) {
        auto it = ops.find(op_id);
        if (it == ops.end() || it->second.state != 0) return;
        it->second.state = ok ? 1 : 2;
        done.notify_all();
    }
    void on_message(int peer, const Header& h, const char* payload);
    void on_completion(const Completion& c);
    void loop();
    std::string telemetry();
};

long Endpoint::send(int peer, const void* data, uint64_t length, uint64_t tag) {
    std::unique_lock<std::mutex> hold(mu);
    if (broken || closing || peer < 0 || peer >= count || peer == me) return -1;
    const long id = next_id++;
    Op& op = ops[id];
    op.sending = true; op.peer = peer; op.tag = tag;
    op.data = static_cast<char*>(const_cast<void*>(data)); op.length = length;
    Peer& p = peers[peer];
    Header h;
    h.sender = (uint16_t)me; h.tag = tag; h.length = length; h.seq = p.next_seq++;
    op.seq = h.seq;
    n.bytes_sent += (long)length;
    if (length <= cfg.eager_max) {
        ++n.eager_sent;
        h.kind = K_EAGER; h.payload = (uint32_t)length;
        std::vector<char> bytes(HEADER_BYTES + length);
        encode(h, bytes.data());
        if (length) std::memcpy(bytes.data() + HEADER_BYTES, data, length);
        transmit(peer, false, std::move(bytes));
        op.state = 1;                    // the bytes were copied: the caller's buffer is free
    } else {
        ++n.rndv_sent;
        h.kind = K_RTS;
        p.sends_by_seq[h.seq] = id;
        std::vector<char> bytes(HEADER_BYTES);
        encode(h, bytes.data());
        transmit(peer, false, std::move(bytes));
    }
    return id;
}

long Endpoint::recv(int peer, void* data, uint64_t length, uint64_t tag) {
    std::unique_lock<std::mutex> hold(mu);
    if (broken || closing || peer < 0 || peer >= count || peer == me) return -1;
    const long id = next_id++;
    Op& op = ops[id];
    op.sending = false; op.peer = peer; op.tag = tag; op.data = static_cast<char*>(data); op.length = length;
    Peer& p = peers[peer];
    if (p.departed && p.early.empty()) {
        break_locked("member " + std::to_string(peer) + " has left the bridge");
        return id;
    }
    for (auto it = p.early.begin(); it != p.early.end(); ++it) {       // did it arrive first?
        if (it->h.tag != tag) continue;
        Peer::Early early = std::move(*it);
        p.early.erase(it);
        if (early.h.kind == K_EAGER) {
            unexpected_bytes -= early.bytes.size();
            if (early.h.length != length) {
                break_locked("message of " + std::to_string(early.h.length) + " bytes from member " +
                             std::to_string(peer) + " met a receive of " + std::to_string(length));
                return id;
            }
            if (length) std::memcpy(data, early.bytes.data(), length);
            n.bytes_recv += (long)length;
            op.state = 1;
        } else {
            grant(peer, early.h, id);
        }
        return id;
    }
    p.posted.push_back(id);
    return id;
}

void Endpoint::on_message(int peer, const Header& h, const char* payload) {
    Peer& p = peers[peer];
    p.seen_data_freed = h.data_freed;
    p.seen_ctrl_freed = h.ctrl_freed;
    switch (h.kind) {
    case K_EAGER: case K_RTS: {
        long match = -1;
        for (auto it = p.posted.begin(); it != p.posted.end(); ++it) {
            if (ops[*it].tag == h.tag) { match = *it; p.posted.erase(it); break; }
        }
        if (h.kind == K_EAGER) ++n.eager_recv; else ++n.rndv_recv;
        if (match < 0) {
            ++n.unexpected;
            Peer::Early early;
            early.h = h;
            if (h.kind == K_EAGER) {
                unexpected_bytes += h.payload;
                if (unexpected_bytes > cfg.unexpected_max) {
                    break_locked("more than " + std::to_string(cfg.unexpected_max) +
                                 " bytes arrived before their receives were posted");
                    return;
                }
                early.bytes.assign(payload, payload + h.payload);
            }
            p.early.push_back(std::move(early));
        } else if (h.kind == K_EAGER) {
            Op& op = ops[match];
            if (op.length != h.length) {
                break_locked("message of " + std::to_string(h.length) + " bytes from member " + std::to_string(peer) +
                             " met a receive of " + std::to_string(op.length) + " (tag " + std::to_string(h.tag) + ")");
                return;
            }
            if (h.length) std::memcpy(op.data, payload, h.length);
            n.bytes_recv += (long)h.length;
            finish(match, true);
        } else {
            grant(peer, h, match);
        }
        break;
    }
    case K_GRANT: {
        auto it = p.sends_by_seq.find(h.seq);
        if (it == p.sends_by_seq.end()) { break_locked("a write grant for a message that was never offered"); return; }
        Op& op = ops[it->second];
        uint32_t rkey;
        std::memcpy(&rkey, payload, 4);
        const uint64_t pieces = (op.length + cfg.max_write - 1) / cfg.max_write;
        op.writes_left = (uint32_t)pieces;
        for (uint64_t i = 0; i < pieces; ++i) {
            const uint64_t off = i * cfg.max_write;
            const uint32_t len = (uint32_t)(op.length - off < cfg.max_write ? op.length - off : cfg.max_write);
            // wr_id: bit 61 marks a write; the message number finds the operation again
            const uint64_t wr = (1ull << 61) | ((uint64_t)peer << 32) | h.seq;
            ++n.writes;
            provider->post_write(peer, wr, op.data + off, h.address + off, rkey, len);
        }
        break;
    }
    case K_FIN: {
        auto it = p.recvs_by_seq.find(h.seq);
        if (it == p.recvs_by_seq.end()) { break_locked("an end-of-write for a message that was never granted"); return; }
        n.bytes_recv += (long)ops[it->second].length;
        finish(it->second, true);
        p.recvs_by_seq.erase(it);
        break;
    }
    case K_BYE: {
        // The peer leaves in good order.  It owes this member nothing (it sent what it had
        // first); anything this member still expects of it can never come.
        p.departed = true;
        p.backlog_data.clear();
        p.backlog_ctrl.clear();
        if (!p.posted.empty() || !p.sends_by_seq.empty() || !p.recvs_by_seq.empty())
            break_locked("member " + std::to_string(peer) + " left the bridge with operations pending");
        break;
    }
    default: break;                                       // CREDIT: the counters were all it carried
    }
}

void Endpoint::on_completion(const Completion& c) {
    ++n.completions;
    if (c.status != ST_OK) {
        // After a goodbye the link's end is no failure, and a report (counters only, or this
        // member's own goodbye) that could not be delivered costs nothing: if its peer is really
        // dead, the end of that peer's stream will say so.
        const bool receive = (c.wr_id >> 63) & 1, piece = (c.wr_id >> 61) & 1;
        const int about = receive || piece ? (int)((c.wr_id >> 32) & 0xFFFF) : c.peer;
        const bool report = !receive && !piece && reports.count(c.wr_id) != 0;
        if (closing || report || (about >= 0 && about < count && peers[about].departed)) {
            if (!receive && !piece) { in_flight.erase(c.wr_id); reports.erase(c.wr_id); }
            return;
        }
        static const char* names[] = {"ok", "a transport error", "a refused remote access", "a flushed connection",
                                      "a message longer than its receive buffer"};
        break_locked(std::string("the link to member ") + std::to_string(c.peer) + " reported " +
                     names[c.status <= ST_LENGTH ? c.status : 1]);
        return;
    }
    if (c.wr_id & (1ull << 63)) {                         // a receive slot was filled
        const bool ctrl = (c.wr_id >> 62) & 1;
        const int peer = (int)((c.wr_id >> 32) & 0xFFFF);
        const uint32_t slot = (uint32_t)(c.wr_id & 0xFFFFFFFFu);
        Peer& p = peers[peer];
        std::vector<char>& buf = ctrl ? p.ctrl_slots[slot] : p.data_slots[slot];
        Header h;
        const std::string problem = decode(buf.data(), c.bytes, &h);
        if (!problem.empty()) { break_locked("member " + std::to_string(peer) + " sent " + problem); return; }
        const bool control_kind = h.kind >= K_GRANT;
        if (control_kind != ctrl || h.sender != peer) { break_locked("a message in the wrong class of slot"); return; }
        on_message(peer, h, buf.data() + HEADER_BYTES);
        if (broken || p.departed) return;
        post_slot(peer, ctrl, slot);
        (ctrl ? p.freed_ctrl : p.freed_data)++;
        drain_backlogs(peer);
        maybe_report(peer);
        return;
    }
    if (c.wr_id & (1ull << 61)) {                         // one piece of a large message is written
        const int peer = (int)((c.wr_id >> 32) & 0xFFFF);
        const uint32_t seq = (uint32_t)(c.wr_id & 0xFFFFFFFFu);
        Peer& p = peers[peer];
        auto it = p.sends_by_seq.find(seq);
        if (it == p.sends_by_seq.end()) return;
        Op& op = ops[it->second];
        if (--op.writes_left == 0) {
            Header h;
            h.kind = K_FIN; h.sender = (uint16_t)me; h.seq = seq; h.tag = op.tag; h.length = op.length;
            send_control(peer, h);
            finish(it->second, true);                     // the data has left the caller's buffer
            p.sends_by_seq.erase(it);
        }
        return;
    }
    in_flight.erase(c.wr_id);                             // a send buffer is free again
    reports.erase(c.wr_id);
}

// How the progress thread waits for completions - GPUBRIDGE_VERBS_PROGRESS, read once per
// endpoint: "economy" sleeps up to 50 ms in poll (an idle bridge costs nothing), "balanced" (the
// default) up to 5 ms, "latency" polls without sleeping while completions keep coming and
// only sleeps 1 ms after 2000 empty rounds.  GPUBRIDGE_VERBS_PROGRESS_CPU pins the thread.
void Endpoint::loop() {
    Completion batch[32];
    if (cfg.cpu >= 0) {
        cpu_set_t set;
        CPU_ZERO(&set);
        CPU_SET(cfg.cpu, &set);
        pthread_setaffinity_np(pthread_self(), sizeof(set), &set);       // best effort
    }
    int empty = 0;
    for (;;) {
        const int sleep_ms = cfg.spin > 0 ? (empty < cfg.spin ? 0 : 1) : cfg.poll_ms;
        const int got = provider->poll(batch, 32, sleep_ms);
        empty = got ? 0 : empty + 1;
        if (cfg.spin > 0 && !got && sleep_ms == 0) std::this_thread::yield();
        std::unique_lock<std::mutex> hold(mu);
        if (closing) return;
        for (int i = 0; i < got && !broken; ++i) on_completion(batch[i]);
    }
}

int Endpoint::wait(const long* ids, int n_ids, double timeout_s) {
    std::unique_lock<std::mutex> hold(mu);
    const auto deadline = Clock::now() + std::chrono::duration_cast<Clock::duration>(
        std::chrono::duration<double>(timeout_s));
    for (;;) {
        bool all = true, failed = broken;
        for (int i = 0; i < n_ids; ++i) {
            auto it = ops.find(ids[i]);
            if (it == ops.end()) continue;
            if (it->second.state == 0) all = false;
            if (it->second.state == 2) failed = true;
        }
        if (failed) {
            break_locked(error.empty() ? "an operation failed" : error);
            return -1;
        }
        if (all) {
            for (int i = 0; i < n_ids; ++i) ops.erase(ids[i]);
            return 0;
        }
        if (done.wait_until(hold, deadline) == std::cv_status::timeout) {
            break_locked("operations did not complete within " + std::to_string(timeout_s) + " s");
            return -1;
        }
    }
}

std::string Endpoint::telemetry() {
    std::unique_lock<std::mutex> hold(mu);
    char text[1024];
    std::snprintf(text, sizeof(text),
        "{\"protocol\": 1, \"member\": %d, \"members\": %d, \"broken\": %s, \"eager_sent\": %ld, \"rndv_sent\": %ld, "
        "\"eager_recv\": %ld, \"rndv_recv\": %ld, \"bytes_sent\": %ld, \"bytes_recv\": %ld, \"unexpected\": %ld, "
        "\"unexpected_bytes_now\": %llu, \"credit_msgs\": %ld, \"credit_stalls\": %ld, \"completions\": %ld, "
        "\"errors\": %ld, \"writes\": %ld, \"mr_hits\": %ld, \"mr_misses\": %ld, \"mr_evictions\": %ld, "
        "\"mr_entries\": %zu, \"pending_ops\": %zu, \"progress\": \"%s\", \"progress_cpu\": %d}",
        me, count, broken ? "true" : "false", n.eager_sent, n.rndv_sent, n.eager_recv, n.rndv_recv, n.bytes_sent,
        n.bytes_recv, n.unexpected, (unsigned long long)unexpected_bytes, n.credit_msgs, n.credit_stalls,
        n.completions, n.errors, n.writes, mrs->hits, mrs->misses, mrs->evictions, mrs->lru.size(), ops.size(),
        cfg.spin > 0 ? "latency" : cfg.poll_ms >= 50 ? "economy" : "balanced", cfg.cpu);
    return text;
}

thread_local std::string g_text;

}  // namespace

extern "C" {

int gb_rdma_protocol() { return 1; }

// An in-process fabric of `members` connected members (tests, and development without a NIC).
void* gb_rdma_mock_fabric(int members) {
    if (members < 1 || members > 64) return nullptr;
    return new MockFabric(members);
}

void gb_rdma_mock_free(void* fabric) { delete static_cast<MockFabric*>(fabric); }

// Make the fabric misbehave: `kind` 1 fail, 2 drop, 3 delay by `arg` ms, 4 corrupt, 5 kill the
// destination - on the `nth` next operation of `opcode` (0 send, 2 write, -1 any) from `src` to
// `dst` (-1: any).
void gb_rdma_mock_inject(void* fabric, int kind, int src, int dst, int opcode, long nth, int arg) {
    MockFabric* f = static_cast<MockFabric*>(fabric);
    std::lock_guard<std::mutex> hold(f->mu);
    Fault fault;
    fault.kind = kind; fault.src = src; fault.dst = dst; fault.opcode = opcode; fault.nth = nth < 1 ? 1 : nth;
    fault.arg = arg;
    f->faults.push_back(fault);
}

// {"rnr": sends that found no receive posted, "sends", "writes", "dropped"}
const char* gb_rdma_mock_stats(void* fabric) {
    MockFabric* f = static_cast<MockFabric*>(fabric);
    char text[200];
    std::snprintf(text, sizeof(text), "{\"rnr\": %ld, \"sends\": %ld, \"writes\": %ld, \"dropped\": %ld}",
                  f->rnr.load(), f->sends.load(), f->writes.load(), f->dropped.load());
    g_text = text;
    return g_text.c_str();
}

// A provider over Unix-domain sockets for member `index` of `members`, listening under `name`
// (an abstract socket name; every member publishes its own and connects with all of them).
void* gb_rdma_socket_provider(int index, int members, const char* name) {
    if (members < 1 || members > 64 || index < 0 || index >= members || name == nullptr) return nullptr;
    SocketProvider* p = new SocketProvider(index, members);
    if (!p->listen_on(name)) { delete p; return nullptr; }
    return p;
}

// Connect with every member (names[i]: member i's socket name).  0, or -1 with the reason in
// gb_rdma_socket_error().
int gb_rdma_socket_connect(void* provider, const char* const* names, double timeout_s) {
    SocketProvider* p = static_cast<SocketProvider*>(provider);
    std::vector<std::string> all;
    for (int i = 0; i < p->count; ++i) all.push_back(names[i] ? names[i] : "");
    std::string why;
    if (p->connect_all(all, timeout_s, &why)) return 0;
    g_text = why;
    return -1;
}
const char* gb_rdma_socket_error() { return g_text.c_str(); }
// The name peers reach this member under (for "tcp://host:0": with the port the system chose).
const char* gb_rdma_socket_name(void* provider) {
    g_text = static_cast<SocketProvider*>(provider)->bound;
    return g_text.c_str();
}
void gb_rdma_socket_free(void* provider) { delete static_cast<SocketProvider*>(provider); }

namespace {
Endpoint* make_endpoint(Provider* provider, MockFabric* fabric, int index, int count, unsigned eager_max,
                        unsigned data_slots, unsigned ctrl_slots, unsigned max_write,
                        unsigned long long unexpected_max, unsigned mr_cache);
}

// An endpoint over a connected socket provider; it owns the provider from here on.
void* gb_rdma_create_on(void* provider, unsigned eager_max, unsigned data_slots, unsigned ctrl_slots,
                        unsigned max_write, unsigned long long unexpected_max, unsigned mr_cache) {
    SocketProvider* p = static_cast<SocketProvider*>(provider);
    if (p == nullptr) return nullptr;
    Endpoint* e = make_endpoint(p, nullptr, p->index, p->count, eager_max, data_slots, ctrl_slots, max_write,
                                unexpected_max, mr_cache);
    e->owned.reset(p);
    return e;
}

// Member `index` of the fabric.  Zero for a setting keeps its default.
void* gb_rdma_create(void* fabric, int index, unsigned eager_max, unsigned data_slots, unsigned ctrl_slots,
                     unsigned max_write, unsigned long long unexpected_max, unsigned mr_cache) {
    MockFabric* f = static_cast<MockFabric*>(fabric);
    if (f == nullptr || index < 0 || index >= (int)f->members.size()) return nullptr;
    return make_endpoint(f->members[index].get(), f, index, (int)f->members.size(), eager_max, data_slots,
                         ctrl_slots, max_write, unexpected_max, mr_cache);
}

}  // extern "C"

namespace {
Endpoint* make_endpoint(Provider* provider, MockFabric* fabric, int index, int count, unsigned eager_max,
                        unsigned data_slots, unsigned ctrl_slots, unsigned max_write,
                        unsigned long long unexpected_max, unsigned mr_cache) {
    Endpoint* e = new Endpoint();
    e->provider = provider;
    e->mock = fabric;
    e->me = index;
    e->count = count;
    if (eager_max) e->cfg.eager_max = eager_max;
    if (data_slots) e->cfg.data_slots = data_slots;
    if (ctrl_slots) e->cfg.ctrl_slots = ctrl_slots < 2 ? 2 : ctrl_slots;
    if (max_write) e->cfg.max_write = max_write;
    if (unexpected_max) e->cfg.unexpected_max = unexpected_max;
    if (mr_cache) e->cfg.mr_cache = mr_cache;
    if (const char* mode = std::getenv("GPUBRIDGE_VERBS_PROGRESS")) {
        const std::string m(mode);
        if (m == "economy") e->cfg.poll_ms = 50;
        else if (m == "latency") e->cfg.spin = 2000;
    }
    if (const char* cpu = std::getenv("GPUBRIDGE_VERBS_PROGRESS_CPU")) e->cfg.cpu = std::atoi(cpu);
    e->mrs.reset(new MrCache(e->provider, e->cfg.mr_cache));
    e->peers.resize(e->count);
    for (int p = 0; p < e->count; ++p) {
        if (p == index) continue;
        Endpoint::Peer& peer = e->peers[p];
        peer.data_slots.assign(e->cfg.data_slots, std::vector<char>(HEADER_BYTES + e->cfg.eager_max));
        peer.ctrl_slots.assign(e->cfg.ctrl_slots, std::vector<char>(HEADER_BYTES + 8));
        for (uint32_t s = 0; s < e->cfg.data_slots; ++s) e->post_slot(p, false, s);
        for (uint32_t s = 0; s < e->cfg.ctrl_slots; ++s) e->post_slot(p, true, s);
    }
    e->progress = std::thread([e] { e->loop(); });
    return e;
}
}  // namespace

extern "C" {

long gb_rdma_send(void* ep, int peer, const void* data, unsigned long long length, unsigned long long tag) {
    return static_cast<Endpoint*>(ep)->send(peer, data, length, tag);
}
long gb_rdma_recv(void* ep, int peer, void* data, unsigned long long length, unsigned long long tag) {
    return static_cast<Endpoint*>(ep)->recv(peer, data, length, tag);
}
int gb_rdma_wait(void* ep, const long* ids, int count, double timeout_s) {
    return static_cast<Endpoint*>(ep)->wait(ids, count, timeout_s);
}
int gb_rdma_all_reduce(void* ep, void* data, unsigned long long count, int dtype, int op,
                       unsigned long long chunk_elems, unsigned long long seq, double timeout_s) {
    return gb_tagged_all_reduce(*static_cast<Endpoint*>(ep), data, count, dtype, op, chunk_elems, seq, timeout_s);
}
int gb_rdma_broadcast(void* ep, void* data, unsigned long long nbytes, int root, unsigned long long chunk_bytes,
                      unsigned long long seq, double timeout_s) {
    return gb_tagged_broadcast(*static_cast<Endpoint*>(ep), data, nbytes, root, chunk_bytes, seq, timeout_s);
}
// Forget cached registrations that overlap [addr, addr + length): call before freeing memory
// that large messages were received into.  Returns how many were dropped.
int gb_rdma_invalidate(void* ep, void* addr, unsigned long long length) {
    Endpoint* e = static_cast<Endpoint*>(ep);
    std::unique_lock<std::mutex> hold(e->mu);
    return e->mrs->invalidate(addr, length);
}
const char* gb_rdma_last_error(void* ep) {
    Endpoint* e = static_cast<Endpoint*>(ep);
    std::unique_lock<std::mutex> hold(e->mu);
    g_text = e->error;
    return g_text.c_str();
}
const char* gb_rdma_telemetry(void* ep) {
    g_text = static_cast<Endpoint*>(ep)->telemetry();
    return g_text.c_str();
}
void gb_rdma_abort(void* ep) { static_cast<Endpoint*>(ep)->fail("aborted by the caller"); }
void gb_rdma_close(void* ep) {
    Endpoint* e = static_cast<Endpoint*>(ep);
    if (e == nullptr) return;
    {
        // Leave in good order: messages this member still owes its peers (queued for a credit,
        // or handed to the provider and not yet completed) go out first, for a bounded time.
        std::unique_lock<std::mutex> hold(e->mu);
        const auto until = Clock::now() + std::chrono::seconds(5);
        while (!e->broken && Clock::now() < until) {
            bool owed = !e->in_flight.empty();
            for (const Endpoint::Peer& p : e->peers) owed = owed || !p.backlog_data.empty() || !p.backlog_ctrl.empty();
            if (!owed) break;
            e->done.wait_for(hold, std::chrono::milliseconds(5));
        }
        const bool clean = !e->broken;
        if (clean) {
            e->say_goodbye();
            const auto last = Clock::now() + std::chrono::seconds(2);
            while (!e->broken && !e->in_flight.empty() && Clock::now() < last)
                e->done.wait_for(hold, std::chrono::milliseconds(5));
        }
        hold.unlock();
        if (clean && e->owned) static_cast<SocketProvider*>(e->owned.get())->drain(5.0);
        hold.lock();
        e->closing = true;
        e->break_locked("the endpoint was closed");
    }
    e->provider->wake();
    if (e->progress.joinable()) e->progress.join();
    e->mrs->clear();
    if (e->owned) static_cast<SocketProvider*>(e->owned.get())->shutdown_all();   // nothing lands any more
    if (e->mock != nullptr) {                              // nothing may land in this member's buffers any more
        std::lock_guard<std::mutex> order(e->mock->mu);
        e->mock->dead[e->me] = true;
        MockProvider* mine = e->mock->members[e->me].get();
        std::lock_guard<std::mutex> hold(mine->mu);
        mine->recvs.clear();
        mine->regions.clear();
    }
    delete e;
}

}  // extern "C"
