// The stand-in UCP library of the tests: the part of the API declared in include/ucp/api/ucp.h,
// over Unix-domain stream sockets between the processes of one host.
//
// A worker listens on an abstract socket whose name is its address.  An endpoint is a
// one-directional connection to the peer's worker: the first frame says who is calling, every
// message is a frame (tag, length, payload) and an orderly close ends with a BYE frame.
// Everything is non-blocking and happens inside ucp_worker_progress (and inside the calls that
// post or cancel), as with the real library: a send completes once the kernel has all its bytes,
// a receive when a matching message has arrived whole; a message nobody waits for yet is kept
// until a receive matches it.  A connection that ends without BYE is a vanished peer: the
// endpoint to that peer reports UCS_ERR_CONNECTION_RESET to its error handler, and so does an
// endpoint whose write fails.
#include <ucp/api/ucp.h>

#include <atomic>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <list>
#include <string>
#include <vector>

#include <fcntl.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace {

enum : uint32_t { HELLO = 1, MESSAGE = 2, BYE = 3 };
struct Header { uint32_t kind, pad; uint64_t tag, length; };
struct Address { char magic[8]; char name[96]; };
const char MAGIC[8] = {'F', 'A', 'K', 'E', 'U', 'C', 'P', '1'};

struct Request {
    enum Kind { SEND, RECV, CLOSE } kind = SEND;
    bool done = false, released = false;
    ucs_status_t status = UCS_INPROGRESS;
    ucp_send_nbx_callback_t on_send = nullptr;
    ucp_tag_recv_nbx_callback_t on_recv = nullptr;
    void* user = nullptr;
    // a receive
    char* buffer = nullptr;
    size_t room = 0;
    ucp_tag_t tag = 0, mask = 0;
    ucp_tag_recv_info_t info = {0, 0};
};

void finish(Request* r, ucs_status_t status) {
    r->status = status;
    r->done = true;
    if (r->kind == Request::RECV && r->on_recv != nullptr) r->on_recv(r, status, &r->info, r->user);
    if (r->kind == Request::SEND && r->on_send != nullptr) r->on_send(r, status, r->user);
    if (r->released) delete r;
}

struct Outgoing {
    Header header;
    const char* payload = nullptr;
    std::string own;                     // payload the library itself owns (HELLO)
    size_t written = 0;                  // of header + payload
    Request* request = nullptr;
};

struct Incoming {
    int fd = -1;
    Header header;
    size_t header_got = 0, payload_got = 0;
    Request* target = nullptr;           // the posted receive this message lands in
    std::vector<char> held;              // or the library's own copy
    std::string caller;
    bool bye = false, dead = false;
};

struct Kept { ucp_tag_t tag; std::vector<char> bytes; };

}  // namespace

struct ucp_context { uint64_t memory_types; };
struct ucp_config { int unused; };

struct ucp_ep {
    ucp_worker_h worker = nullptr;
    int fd = -1;
    std::string remote;
    std::deque<Outgoing> queue;
    ucp_err_handler_t handler = {nullptr, nullptr};
    bool failed = false, closing = false;
    Request* closed = nullptr;
};

struct ucp_worker {
    ucp_context_h context = nullptr;
    int listener = -1;
    std::string name;
    std::list<ucp_ep*> endpoints;
    std::list<Incoming> callers;
    std::deque<Request*> posted;
    std::deque<Kept> kept;
};

namespace {

std::atomic<unsigned> serial{0};

void unblock(int fd) { fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK); }

sockaddr_un abstract(const std::string& name, socklen_t* length) {
    sockaddr_un where;
    std::memset(&where, 0, sizeof where);
    where.sun_family = AF_UNIX;
    std::memcpy(where.sun_path + 1, name.data(), name.size());       // leading NUL: abstract namespace
    *length = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
    return where;
}

void break_endpoint(ucp_ep* ep, ucs_status_t status) {
    if (ep->failed) return;
    ep->failed = true;
    while (!ep->queue.empty()) {
        Request* r = ep->queue.front().request;
        ep->queue.pop_front();
        if (r != nullptr) finish(r, status);
    }
    if (ep->closed != nullptr) { finish(ep->closed, UCS_OK); ep->closed = nullptr; }
    if (ep->handler.cb != nullptr && !ep->closing) ep->handler.cb(ep->handler.arg, ep, status);
}

unsigned flush(ucp_ep* ep) {
    unsigned events = 0;
    while (!ep->failed && !ep->queue.empty()) {
        Outgoing& out = ep->queue.front();
        const size_t total = sizeof(Header) + out.header.length;
        const char* from;
        size_t n;
        if (out.written < sizeof(Header)) {
            from = reinterpret_cast<const char*>(&out.header) + out.written;
            n = sizeof(Header) - out.written;
        } else {
            from = out.payload + (out.written - sizeof(Header));
            n = total - out.written;
        }
        if (n > 0) {
            const ssize_t put = send(ep->fd, from, n, MSG_NOSIGNAL);
            if (put < 0) {
                if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) break;
                break_endpoint(ep, UCS_ERR_CONNECTION_RESET);
                return events + 1;
            }
            out.written += (size_t)put;
            ++events;
        }
        if (out.written == total) {
            Request* r = out.request;
            ep->queue.pop_front();
            if (r != nullptr) finish(r, UCS_OK);
        }
    }
    if (ep->closing && !ep->failed && ep->queue.empty() && ep->fd >= 0) {
        close(ep->fd);
        ep->fd = -1;
        if (ep->closed != nullptr) { finish(ep->closed, UCS_OK); ep->closed = nullptr; }
        ++events;
    }
    return events;
}

bool matches(const Request* r, ucp_tag_t tag) { return (r->tag & r->mask) == (tag & r->mask); }

void deliver(Request* r, ucp_tag_t tag, const char* bytes, size_t length) {
    r->info.sender_tag = tag;
    r->info.length = length;
    if (bytes != nullptr) std::memcpy(r->buffer, bytes, length < r->room ? length : r->room);
    finish(r, length > r->room ? UCS_ERR_MESSAGE_TRUNCATED : UCS_OK);
}

void vanished(ucp_worker* w, Incoming& in) {
    in.dead = true;
    if (in.target != nullptr) { Request* r = in.target; in.target = nullptr; finish(r, UCS_ERR_CONNECTION_RESET); }
    if (in.bye) return;
    for (ucp_ep* ep : w->endpoints)
        if (!in.caller.empty() && ep->remote == in.caller) break_endpoint(ep, UCS_ERR_CONNECTION_RESET);
}

unsigned drain(ucp_worker* w, Incoming& in) {
    unsigned events = 0;
    char spill[4096];
    while (!in.dead) {
        if (in.header_got < sizeof(Header)) {
            const ssize_t got = recv(in.fd, reinterpret_cast<char*>(&in.header) + in.header_got,
                                     sizeof(Header) - in.header_got, 0);
            if (got == 0 || (got < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) {
                vanished(w, in);
                return events + 1;
            }
            if (got < 0) return events;
            in.header_got += (size_t)got;
            ++events;
            if (in.header_got < sizeof(Header)) continue;
            in.payload_got = 0;
            in.target = nullptr;
            in.held.clear();
            if (in.header.kind == MESSAGE) {
                for (auto it = w->posted.begin(); it != w->posted.end(); ++it)
                    if (matches(*it, in.header.tag)) { in.target = *it; w->posted.erase(it); break; }
            }
            if (in.target == nullptr) in.held.resize(in.header.length);
        }
        // the payload
        while (in.payload_got < in.header.length) {
            char* into;
            size_t room;
            if (in.target != nullptr && in.payload_got < in.target->room) {
                into = in.target->buffer + in.payload_got;
                room = (in.header.length < in.target->room ? in.header.length : in.target->room) - in.payload_got;
            } else if (in.target != nullptr) {
                into = spill;
                room = in.header.length - in.payload_got < sizeof spill ? in.header.length - in.payload_got : sizeof spill;
            } else {
                into = in.held.data() + in.payload_got;
                room = in.header.length - in.payload_got;
            }
            const ssize_t got = recv(in.fd, into, room, 0);
            if (got == 0 || (got < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) {
                vanished(w, in);
                return events + 1;
            }
            if (got < 0) return events;
            in.payload_got += (size_t)got;
            ++events;
        }
        // a whole frame
        in.header_got = 0;
        if (in.header.kind == HELLO) {
            in.caller.assign(in.held.begin(), in.held.end());
        } else if (in.header.kind == BYE) {
            in.bye = true;
        } else if (in.target != nullptr) {
            Request* r = in.target;
            in.target = nullptr;
            deliver(r, in.header.tag, nullptr, in.header.length);
        } else {
            bool taken = false;
            for (auto it = w->posted.begin(); it != w->posted.end(); ++it)
                if (matches(*it, in.header.tag)) {
                    Request* r = *it;
                    w->posted.erase(it);
                    deliver(r, in.header.tag, in.held.data(), in.held.size());
                    taken = true;
                    break;
                }
            if (!taken) w->kept.push_back(Kept{in.header.tag, std::move(in.held)});
            in.held = std::vector<char>();
        }
    }
    return events;
}

}  // namespace

extern "C" {

const char* ucs_status_string(ucs_status_t status) {
    switch (status) {
        case UCS_OK: return "Success";
        case UCS_INPROGRESS: return "Operation in progress";
        case UCS_ERR_NO_MEMORY: return "Out of memory";
        case UCS_ERR_INVALID_PARAM: return "Invalid parameter";
        case UCS_ERR_UNREACHABLE: return "Destination is unreachable";
        case UCS_ERR_NO_DEVICE: return "No such device";
        case UCS_ERR_CANCELED: return "Operation canceled";
        case UCS_ERR_MESSAGE_TRUNCATED: return "Message truncated";
        case UCS_ERR_CONNECTION_RESET: return "Connection reset by remote peer";
        case UCS_ERR_ENDPOINT_TIMEOUT: return "Endpoint timeout";
        default: return "Unknown error";
    }
}

void ucp_get_version(unsigned* major, unsigned* minor, unsigned* release) {
    unsigned a = UCP_API_MAJOR, b = UCP_API_MINOR, c = 0;
    const char* forced = std::getenv("FAKE_UCP_VERSION");
    if (forced != nullptr) std::sscanf(forced, "%u.%u.%u", &a, &b, &c);
    *major = a; *minor = b; *release = c;
}

ucs_status_t ucp_config_read(const char*, const char*, ucp_config_t** config) {
    *config = new ucp_config{0};
    return UCS_OK;
}
void ucp_config_release(ucp_config_t* config) { delete config; }

ucs_status_t ucp_init(const ucp_params_t* params, const ucp_config_t*, ucp_context_h* context) {
    const char* fail = std::getenv("FAKE_UCP_FAIL_INIT");
    if (fail != nullptr && fail[0] == '1') return UCS_ERR_NO_DEVICE;
    if (params == nullptr || !(params->field_mask & UCP_PARAM_FIELD_FEATURES) || !(params->features & UCP_FEATURE_TAG))
        return UCS_ERR_INVALID_PARAM;
    uint64_t types = UCS_BIT(UCS_MEMORY_TYPE_HOST);
    const char* listed = std::getenv("FAKE_UCP_MEMORY_TYPES");
    if (listed != nullptr && std::strstr(listed, "cuda") != nullptr) types |= UCS_BIT(UCS_MEMORY_TYPE_CUDA);
    *context = new ucp_context{types};
    return UCS_OK;
}
void ucp_cleanup(ucp_context_h context) { delete context; }

ucs_status_t ucp_context_query(ucp_context_h context, ucp_context_attr_t* attr) {
    if (attr->field_mask & UCP_ATTR_FIELD_MEMORY_TYPES) attr->memory_types = context->memory_types;
    return UCS_OK;
}

ucs_status_t ucp_worker_create(ucp_context_h context, const ucp_worker_params_t*, ucp_worker_h* worker) {
    auto* w = new ucp_worker;
    w->context = context;
    char name[96];
    std::snprintf(name, sizeof name, "fake-ucp-%d-%u-%08x", (int)getpid(), serial++, (unsigned)std::rand());
    w->name = name;
    w->listener = socket(AF_UNIX, SOCK_STREAM, 0);
    socklen_t length;
    sockaddr_un where = abstract(w->name, &length);
    if (w->listener < 0 || bind(w->listener, reinterpret_cast<sockaddr*>(&where), length) != 0 ||
        listen(w->listener, 64) != 0) {
        if (w->listener >= 0) close(w->listener);
        delete w;
        return UCS_ERR_NO_DEVICE;
    }
    unblock(w->listener);
    *worker = w;
    return UCS_OK;
}

void ucp_worker_destroy(ucp_worker_h w) {
    for (ucp_ep* ep : w->endpoints) { if (ep->fd >= 0) close(ep->fd); delete ep; }
    for (Incoming& in : w->callers) if (in.fd >= 0) close(in.fd);
    close(w->listener);
    delete w;
}

ucs_status_t ucp_worker_get_address(ucp_worker_h w, ucp_address_t** address, size_t* length) {
    auto* a = new Address;
    std::memset(a, 0, sizeof *a);
    std::memcpy(a->magic, MAGIC, sizeof MAGIC);
    std::snprintf(a->name, sizeof a->name, "%s", w->name.c_str());
    *address = reinterpret_cast<ucp_address_t*>(a);
    *length = sizeof(Address);
    return UCS_OK;
}
void ucp_worker_release_address(ucp_worker_h, ucp_address_t* address) { delete reinterpret_cast<Address*>(address); }

unsigned ucp_worker_progress(ucp_worker_h w) {
    unsigned events = 0;
    for (;;) {
        const int fd = accept(w->listener, nullptr, nullptr);
        if (fd < 0) break;
        unblock(fd);
        w->callers.emplace_back();
        w->callers.back().fd = fd;
        ++events;
    }
    for (auto it = w->endpoints.begin(); it != w->endpoints.end();) {
        ucp_ep* ep = *it;
        events += flush(ep);
        if (ep->closing && (ep->fd < 0 || ep->failed)) {
            if (ep->fd >= 0) close(ep->fd);
            delete ep;
            it = w->endpoints.erase(it);
        } else {
            ++it;
        }
    }
    for (auto it = w->callers.begin(); it != w->callers.end();) {
        events += drain(w, *it);
        if (it->dead) { close(it->fd); it = w->callers.erase(it); } else { ++it; }
    }
    return events;
}

ucs_status_t ucp_ep_create(ucp_worker_h w, const ucp_ep_params_t* params, ucp_ep_h* out) {
    if (!(params->field_mask & UCP_EP_PARAM_FIELD_REMOTE_ADDRESS)) return UCS_ERR_INVALID_PARAM;
    const auto* address = reinterpret_cast<const Address*>(params->address);
    if (std::memcmp(address->magic, MAGIC, sizeof MAGIC) != 0) return UCS_ERR_INVALID_PARAM;
    auto* ep = new ucp_ep;
    ep->worker = w;
    ep->remote = std::string(address->name, strnlen(address->name, sizeof address->name));
    if (params->field_mask & UCP_EP_PARAM_FIELD_ERR_HANDLER) ep->handler = params->err_handler;
    ep->fd = socket(AF_UNIX, SOCK_STREAM, 0);
    socklen_t length;
    sockaddr_un where = abstract(ep->remote, &length);
    if (ep->fd < 0 || connect(ep->fd, reinterpret_cast<sockaddr*>(&where), length) != 0) {
        if (ep->fd >= 0) close(ep->fd);
        delete ep;
        return UCS_ERR_UNREACHABLE;
    }
    unblock(ep->fd);
    Outgoing hello;
    hello.header = Header{HELLO, 0, 0, w->name.size()};
    hello.own = w->name;
    ep->queue.push_back(std::move(hello));
    ep->queue.back().payload = ep->queue.back().own.data();
    w->endpoints.push_back(ep);
    *out = ep;
    return UCS_OK;
}

ucs_status_ptr_t ucp_ep_close_nbx(ucp_ep_h ep, const ucp_request_param_t* param) {
    const bool force = param != nullptr && (param->op_attr_mask & UCP_OP_ATTR_FIELD_FLAGS) &&
                       (param->flags & UCP_EP_CLOSE_FLAG_FORCE);
    ep->closing = true;
    if (force || ep->failed) {
        while (!ep->queue.empty()) {
            Request* r = ep->queue.front().request;
            ep->queue.pop_front();
            if (r != nullptr) finish(r, UCS_ERR_CANCELED);
        }
        if (ep->fd >= 0) { close(ep->fd); ep->fd = -1; }
        return nullptr;                                   // the worker's next progress frees it
    }
    Outgoing bye;
    bye.header = Header{BYE, 0, 0, 0};
    ep->queue.push_back(std::move(bye));
    auto* r = new Request;
    r->kind = Request::CLOSE;
    ep->closed = r;
    return r;
}

ucs_status_ptr_t ucp_tag_send_nbx(ucp_ep_h ep, const void* buffer, size_t count, ucp_tag_t tag,
                                  const ucp_request_param_t* param) {
    if (ep->failed || ep->closing) return UCS_STATUS_PTR(UCS_ERR_CONNECTION_RESET);
    auto* r = new Request;
    r->kind = Request::SEND;
    if (param->op_attr_mask & UCP_OP_ATTR_FIELD_CALLBACK) r->on_send = param->cb.send;
    if (param->op_attr_mask & UCP_OP_ATTR_FIELD_USER_DATA) r->user = param->user_data;
    Outgoing out;
    out.header = Header{MESSAGE, 0, tag, count};
    out.payload = static_cast<const char*>(buffer);
    out.request = r;
    ep->queue.push_back(std::move(out));
    flush(ep);
    return r;
}

ucs_status_ptr_t ucp_tag_recv_nbx(ucp_worker_h w, void* buffer, size_t count, ucp_tag_t tag,
                                  ucp_tag_t mask, const ucp_request_param_t* param) {
    auto* r = new Request;
    r->kind = Request::RECV;
    if (param->op_attr_mask & UCP_OP_ATTR_FIELD_CALLBACK) r->on_recv = param->cb.recv;
    if (param->op_attr_mask & UCP_OP_ATTR_FIELD_USER_DATA) r->user = param->user_data;
    r->buffer = static_cast<char*>(buffer);
    r->room = count;
    r->tag = tag;
    r->mask = mask;
    for (auto it = w->kept.begin(); it != w->kept.end(); ++it)
        if (matches(r, it->tag)) {
            Kept message = std::move(*it);
            w->kept.erase(it);
            deliver(r, message.tag, message.bytes.data(), message.bytes.size());
            return r;
        }
    w->posted.push_back(r);
    return r;
}

ucs_status_t ucp_request_check_status(void* request) {
    auto* r = static_cast<Request*>(request);
    return r->done ? r->status : UCS_INPROGRESS;
}

void ucp_request_cancel(ucp_worker_h w, void* request) {
    auto* r = static_cast<Request*>(request);
    if (r->done) return;
    if (r->kind == Request::RECV) {
        for (auto it = w->posted.begin(); it != w->posted.end(); ++it)
            if (*it == r) { w->posted.erase(it); finish(r, UCS_ERR_CANCELED); return; }
        return;                                          // a message is landing in it: it completes
    }
    if (r->kind == Request::SEND) {
        for (ucp_ep* ep : w->endpoints)
            for (auto it = ep->queue.begin(); it != ep->queue.end(); ++it)
                if (it->request == r && it->written == 0) { ep->queue.erase(it); finish(r, UCS_ERR_CANCELED); return; }
    }
}

void ucp_request_free(void* request) {
    auto* r = static_cast<Request*>(request);
    if (r->done) delete r; else r->released = true;
}

}  // extern "C"
