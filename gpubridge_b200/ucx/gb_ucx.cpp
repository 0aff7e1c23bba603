// The worker of bridge="ucx": tagged messages between the bridge members over UCX's UCP layer,
// as a GbTaggedWorker, so that the chunked exchange / ring / broadcast of gb_tagged.cpp run on it
// natively like they do on the TCP worker and on the RDMA-style endpoint.
//
// This file is not part of the package's own library: it is compiled on first use against the
// UCX installation of the machine (python -m gpubridge_b200.ucx build), because UCX is a system
// library whose headers an image may or may not have.  It uses only the public UCP API:
//   ucp_init / ucp_context_query / ucp_worker_create / ucp_worker_get_address / ucp_ep_create
//   ucp_tag_send_nbx / ucp_tag_recv_nbx / ucp_worker_progress / ucp_request_cancel /
//   ucp_request_free / ucp_ep_close_nbx
//
// Rules of this worker:
//  * One thread at a time per worker (UCS_THREAD_MODE_SERIALIZED); a mutex enforces it.
//  * A receive names no peer: the tag (sequence | step | sender | chunk) says whose message it is.
//  * Completion is reported by UCP's callbacks into a table of operations; wait() drives
//    ucp_worker_progress until its operations are complete, a peer's endpoint reported an error,
//    or the deadline passed.  A receive that completed SHORTER than posted is an error, never
//    silently accepted; a longer message is UCX's own truncation error.
//  * After a timeout, a peer failure or stop() the worker is broken: outstanding operations are
//    cancelled and progressed until UCX has let go of the caller's buffers (bounded), and every
//    later call fails with the first reason.
//  * abort() may come from another thread while one is inside wait(): a flag read without the
//    mutex ends that wait, then the worker is stopped.
//  * close() closes the endpoints with a flush first and by force when that takes longer than
//    the limit; it never blocks past the limit.
// (Role of the reference's src/gpubridge/ucx/bridge.cpp, whose collectives run in Python.)
#include <ucp/api/ucp.h>

#include <sched.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "gb_tagged.h"

namespace {

constexpr int GB_UCX_FAILED = -1, GB_UCX_TIMED_OUT = -2, GB_UCX_PEER_FAILED = -3;
constexpr int MEM_HOST = 0, MEM_CUDA = 1, MEM_DETECT = -1;

double seconds_now() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct UcxWorker;

struct Operation {
    UcxWorker* owner = nullptr;
    long id = 0;
    void* request = nullptr;          // UCX's handle while it is in flight
    bool done = false;
    bool receive = false;
    ucs_status_t status = UCS_OK;
    uint64_t posted = 0, arrived = 0;
};

struct Link {
    ucp_ep_h ep = nullptr;
    UcxWorker* owner = nullptr;
    int member = -1;
    ucs_status_t failure = UCS_OK;
};

struct UcxWorker final : GbTaggedWorker {
    int count = 0, me = 0;
    int memory = MEM_HOST;                     // memory type given to the next posts
    ucp_context_h context = nullptr;
    ucp_worker_h worker = nullptr;
    std::vector<Link> links;
    std::unordered_map<long, Operation*> table;
    long next_id = 1;
    bool broken = false;
    int broken_code = 0;
    std::string reason;
    std::mutex gate;
    std::atomic<bool> asked_to_stop{false};    // set without the gate, so that it reaches a thread inside wait()
    unsigned long long sends = 0, receives = 0, bytes_out = 0, bytes_in = 0, progress_calls = 0;

    int members() const override { return count; }
    int index() const override { return me; }

    // An argument error: the call is refused, the worker stays usable.
    int refuse(const std::string& why) {
        if (!broken) reason = why;
        return GB_UCX_FAILED;
    }
    // The worker is broken from here on; the first reason stays.
    int wreck(int code, const std::string& why) {
        if (!broken) { broken = true; broken_code = code; reason = why; }
        return broken_code;
    }

    // ---- callbacks (called by UCX from inside our own calls into it) --------------------------
    static void sent(void* request, ucs_status_t status, void* user) {
        auto* op = static_cast<Operation*>(user);
        op->status = status;
        op->done = true;
        (void)request;
    }
    static void received(void* request, ucs_status_t status, const ucp_tag_recv_info_t* info, void* user) {
        auto* op = static_cast<Operation*>(user);
        op->status = status;
        if (status == UCS_OK && info != nullptr) op->arrived = info->length;
        op->done = true;
        (void)request;
    }
    static void link_failed(void* arg, ucp_ep_h, ucs_status_t status) {
        static_cast<Link*>(arg)->failure = status;
    }

    ucs_memory_type_t memory_type() const {
        return memory == MEM_CUDA ? UCS_MEMORY_TYPE_CUDA
             : memory == MEM_DETECT ? UCS_MEMORY_TYPE_UNKNOWN : UCS_MEMORY_TYPE_HOST;
    }

    long post(bool receive, int peer, void* data, uint64_t length, uint64_t tag) {
        if (broken) return broken_code;
        if (!receive && (peer < 0 || peer >= count || peer == me || links[peer].ep == nullptr))
            return refuse("send to member " + std::to_string(peer) + ", which is not connected");
        auto* op = new Operation;
        op->owner = this;
        op->id = next_id++;
        op->receive = receive;
        op->posted = length;
        ucp_request_param_t param;
        std::memset(&param, 0, sizeof param);
        param.op_attr_mask = UCP_OP_ATTR_FIELD_CALLBACK | UCP_OP_ATTR_FIELD_USER_DATA |
                             UCP_OP_ATTR_FIELD_MEMORY_TYPE | UCP_OP_ATTR_FLAG_NO_IMM_CMPL;
        param.user_data = op;
        param.memory_type = memory_type();
        ucs_status_ptr_t handle;
        if (receive) {
            param.cb.recv = &UcxWorker::received;
            handle = ucp_tag_recv_nbx(worker, data, length, tag, ~0ull, &param);
        } else {
            param.cb.send = &UcxWorker::sent;
            handle = ucp_tag_send_nbx(links[peer].ep, data, length, tag, &param);
        }
        if (UCS_PTR_IS_ERR(handle)) {
            const ucs_status_t status = UCS_PTR_STATUS(handle);
            delete op;
            return wreck(GB_UCX_FAILED, std::string(receive ? "posting a receive" : "posting a send") +
                         " failed: " + ucs_status_string(status));
        }
        if (handle == nullptr) op->done = true;         // finished before the call returned
        op->request = handle;
        table[op->id] = op;
        if (receive) { ++receives; bytes_in += length; } else { ++sends; bytes_out += length; }
        return op->id;
    }

    void retire(Operation* op) {
        if (op->request != nullptr) ucp_request_free(op->request);
        table.erase(op->id);
        delete op;
    }

    // Cancel what is in flight and progress until UCX has completed (with whatever status) every
    // operation: afterwards nothing of UCX points into a caller's buffer.  Bounded.
    void let_go(double limit_s) {
        for (auto& entry : table)
            if (!entry.second->done && entry.second->request != nullptr)
                ucp_request_cancel(worker, entry.second->request);
        const double until = seconds_now() + limit_s;
        for (;;) {
            bool open = false;
            for (auto& entry : table) open = open || !entry.second->done;
            if (!open || seconds_now() > until) break;
            ucp_worker_progress(worker);
        }
        std::vector<Operation*> finished;
        for (auto& entry : table) if (entry.second->done) finished.push_back(entry.second);
        for (auto* op : finished) retire(op);
        // what is still not done after the limit stays in the table: its memory is never reused
    }

    int check_links() {
        for (auto& link : links)
            if (link.failure != UCS_OK)
                return wreck(GB_UCX_PEER_FAILED, "the endpoint to member " + std::to_string(link.member) +
                               " failed: " + ucs_status_string(link.failure));
        return 0;
    }

    // ---- GbTaggedWorker ----------------------------------------------------------------------------
    long send(int peer, const void* data, uint64_t length, uint64_t tag) override {
        return post(false, peer, const_cast<void*>(data), length, tag);
    }
    long recv(int peer, void* data, uint64_t length, uint64_t tag) override {
        (void)peer;
        return post(true, -1, data, length, tag);
    }
    // Collect what has completed among `ids`; `open` says whether any is still in flight.
    // < 0: one of them failed (the worker is broken and has let go of everything).
    int sweep(const long* ids, int n, bool* open) {
        *open = false;
        for (int i = 0; i < n; ++i) {
            auto found = table.find(ids[i]);
            if (found == table.end()) continue;                  // completed and collected before
            Operation* op = found->second;
            if (!op->done) { *open = true; continue; }
            if (op->status != UCS_OK) {
                const std::string why = std::string(op->receive ? "a receive" : "a send") + " failed: " +
                                        ucs_status_string(op->status);
                retire(op);
                wreck(GB_UCX_PEER_FAILED, why);
                let_go(2.0);
                return broken_code;
            }
            if (op->receive && op->arrived != op->posted) {
                const std::string why = "a message of " + std::to_string(op->arrived) + " bytes arrived for a "
                    "receive of " + std::to_string(op->posted) + ": the members disagree about the call";
                retire(op);
                wreck(GB_UCX_FAILED, why);
                let_go(2.0);
                return broken_code;
            }
            retire(op);
        }
        if (*open && check_links() != 0) { let_go(2.0); return broken_code; }
        return 0;
    }

    int wait(const long* ids, int n, double timeout_s) override {
        if (broken) return broken_code;
        const double until = seconds_now() + (timeout_s > 0 ? timeout_s : 0);
        unsigned spins = 0;
        for (;;) {
            bool open = false;
            const int rc = sweep(ids, n, &open);
            if (rc != 0) return rc;
            if (!open) return 0;
            if (asked_to_stop.load()) {
                wreck(GB_UCX_FAILED, "stopped from another thread while operations were outstanding");
                let_go(2.0);
                return broken_code;
            }
            if (seconds_now() > until) {
                wreck(GB_UCX_TIMED_OUT, "operations were still outstanding at the deadline "
                      "(a member that never joined, or a slower link than the timeout allows)");
                let_go(2.0);
                return broken_code;
            }
            ++progress_calls;
            if (ucp_worker_progress(worker) == 0 && ++spins > 2000) { sched_yield(); spins = 0; }
        }
    }
    // Without waiting: progress a little, then 0 (all complete), 1 (some in flight) or < 0.
    int poll(const long* ids, int n) {
        if (broken) return broken_code;
        for (int round = 0; round < 8; ++round) {
            ++progress_calls;
            if (ucp_worker_progress(worker) == 0) break;
        }
        bool open = false;
        const int rc = sweep(ids, n, &open);
        return rc != 0 ? rc : (open ? 1 : 0);
    }
    void stop() override {
        wreck(GB_UCX_FAILED, reason.empty() ? "stopped after a failed call" : reason);
        if (worker != nullptr) let_go(2.0);
    }
    void fail(const char* why) override { refuse(why); }

    int shut(double limit_s) {
        int late = 0;
        if (worker != nullptr) {
            let_go(limit_s < 2.0 ? limit_s : 2.0);
            std::vector<void*> closing;
            for (auto& link : links) {
                if (link.ep == nullptr) continue;
                ucp_request_param_t param;
                std::memset(&param, 0, sizeof param);
                if (broken || link.failure != UCS_OK) {
                    param.op_attr_mask = UCP_OP_ATTR_FIELD_FLAGS;
                    param.flags = UCP_EP_CLOSE_FLAG_FORCE;
                }
                ucs_status_ptr_t handle = ucp_ep_close_nbx(link.ep, &param);
                link.ep = nullptr;
                if (UCS_PTR_IS_PTR(handle)) closing.push_back(handle);
            }
            const double until = seconds_now() + limit_s;
            for (void* handle : closing) {
                while (ucp_request_check_status(handle) == UCS_INPROGRESS) {
                    if (seconds_now() > until) { late = 1; break; }
                    ucp_worker_progress(worker);
                }
                if (!late) ucp_request_free(handle);
            }
            ucp_worker_destroy(worker);
            worker = nullptr;
        }
        if (context != nullptr) { ucp_cleanup(context); context = nullptr; }
        for (auto& entry : table) delete entry.second;
        table.clear();
        return late;
    }
};

void say(char* error, size_t room, const std::string& text) {
    if (error != nullptr && room > 0) std::snprintf(error, room, "%s", text.c_str());
}

}  // namespace

extern "C" {

void gb_ucx_version(unsigned* major, unsigned* minor, unsigned* patch) { ucp_get_version(major, minor, patch); }

// The UCX version this file was COMPILED against (the headers'), as major << 16 | minor.
unsigned gb_ucx_built_against(void) { return (UCP_API_MAJOR << 16) | UCP_API_MINOR; }

void* gb_ucx_create(int members, int index, char* error, size_t room) {
    if (members < 1 || index < 0 || index >= members) { say(error, room, "bad member count or index"); return nullptr; }
    auto* w = new UcxWorker;
    w->count = members;
    w->me = index;
    w->links.resize(members);
    for (int m = 0; m < members; ++m) { w->links[m].owner = w; w->links[m].member = m; }
    ucp_params_t params;
    std::memset(&params, 0, sizeof params);
    params.field_mask = UCP_PARAM_FIELD_FEATURES;
    params.features = UCP_FEATURE_TAG;
    ucp_config_t* config = nullptr;
    ucs_status_t status = ucp_config_read(nullptr, nullptr, &config);
    if (status == UCS_OK) {
        status = ucp_init(&params, config, &w->context);
        ucp_config_release(config);
    }
    if (status != UCS_OK) {
        say(error, room, std::string("UCX did not start (ucp_init): ") + ucs_status_string(status));
        delete w;
        return nullptr;
    }
    ucp_worker_params_t wparams;
    std::memset(&wparams, 0, sizeof wparams);
    wparams.field_mask = UCP_WORKER_PARAM_FIELD_THREAD_MODE;
    wparams.thread_mode = UCS_THREAD_MODE_SERIALIZED;
    status = ucp_worker_create(w->context, &wparams, &w->worker);
    if (status != UCS_OK) {
        say(error, room, std::string("UCX made no worker (ucp_worker_create): ") + ucs_status_string(status));
        ucp_cleanup(w->context);
        delete w;
        return nullptr;
    }
    return w;
}

// Bit 0: host, bit 1: CUDA memory can be handed to UCX as it lies.
int gb_ucx_memory_types(void* handle, unsigned long long* bits) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    ucp_context_attr_t attr;
    std::memset(&attr, 0, sizeof attr);
    attr.field_mask = UCP_ATTR_FIELD_MEMORY_TYPES;
    const ucs_status_t status = ucp_context_query(w->context, &attr);
    if (status != UCS_OK) return w->refuse(std::string("ucp_context_query: ") + ucs_status_string(status));
    *bits = 1ull | ((attr.memory_types & UCS_BIT(UCS_MEMORY_TYPE_CUDA)) ? 2ull : 0ull);
    return 0;
}

int gb_ucx_address(void* handle, void* into, size_t room, size_t* length) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    ucp_address_t* address = nullptr;
    size_t size = 0;
    const ucs_status_t status = ucp_worker_get_address(w->worker, &address, &size);
    if (status != UCS_OK) return w->refuse(std::string("ucp_worker_get_address: ") + ucs_status_string(status));
    *length = size;
    int rc = 0;
    if (size <= room) std::memcpy(into, address, size); else rc = 1;      // 1: call again with more room
    ucp_worker_release_address(w->worker, address);
    return rc;
}

int gb_ucx_connect(void* handle, int member, const void* address) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    if (member < 0 || member >= w->count || member == w->me) return w->refuse("connect: no such member");
    if (w->links[member].ep != nullptr) return w->refuse("connect: member " + std::to_string(member) + " is connected already");
    ucp_ep_params_t params;
    std::memset(&params, 0, sizeof params);
    params.field_mask = UCP_EP_PARAM_FIELD_REMOTE_ADDRESS | UCP_EP_PARAM_FIELD_ERR_HANDLING_MODE |
                        UCP_EP_PARAM_FIELD_ERR_HANDLER;
    params.address = static_cast<const ucp_address_t*>(address);
    params.err_mode = UCP_ERR_HANDLING_MODE_PEER;
    params.err_handler.cb = &UcxWorker::link_failed;
    params.err_handler.arg = &w->links[member];
    const ucs_status_t status = ucp_ep_create(w->worker, &params, &w->links[member].ep);
    if (status != UCS_OK) {
        w->links[member].ep = nullptr;
        return w->refuse("ucp_ep_create to member " + std::to_string(member) + ": " + ucs_status_string(status));
    }
    return 0;
}

// Memory type of the buffers of the posts that follow: 0 host, 1 CUDA, -1 let UCX find out.
void gb_ucx_set_memory(void* handle, int memory) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    w->memory = memory;
}

long long gb_ucx_send(void* handle, int member, const void* data, unsigned long long length, unsigned long long tag) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    return w->send(member, data, length, tag);
}

long long gb_ucx_recv(void* handle, void* data, unsigned long long length, unsigned long long tag) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    return w->recv(-1, data, length, tag);
}

int gb_ucx_wait(void* handle, const long long* ids, int count, double timeout_s) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    std::vector<long> own(ids, ids + count);
    return w->wait(own.data(), count, timeout_s);
}

// The same without waiting: 0 all complete, 1 some still in flight, < 0 failed.  Lets several
// threads share one worker without one of them holding it for the length of a wait.
int gb_ucx_poll(void* handle, const long long* ids, int count) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    std::vector<long> own(ids, ids + count);
    return w->poll(own.data(), count);
}

int gb_ucx_all_reduce(void* handle, void* data, unsigned long long count, int dtype, int op,
                      unsigned long long chunk_elems, unsigned long long seq, double timeout_s) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    if (w->broken) return w->broken_code;
    const int rc = gb_tagged_all_reduce(*w, data, count, dtype, op, chunk_elems, seq, timeout_s);
    return rc == 0 ? 0 : (w->broken ? w->broken_code : GB_UCX_FAILED);
}

int gb_ucx_broadcast(void* handle, void* data, unsigned long long nbytes, int root,
                     unsigned long long chunk_bytes, unsigned long long seq, double timeout_s) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    if (w->broken) return w->broken_code;
    const int rc = gb_tagged_broadcast(*w, data, nbytes, root, chunk_bytes, seq, timeout_s);
    return rc == 0 ? 0 : (w->broken ? w->broken_code : GB_UCX_FAILED);
}

// May be called while another thread is inside a wait: the flag ends that wait, which frees
// the gate for the rest.
void gb_ucx_abort(void* handle) {
    auto* w = static_cast<UcxWorker*>(handle);
    w->asked_to_stop.store(true);
    std::lock_guard<std::mutex> hold(w->gate);
    w->stop();
}

// Writes the reason of the last failure; returns its length.
int gb_ucx_last_error(void* handle, char* into, size_t room) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    say(into, room, w->reason);
    return (int)w->reason.size();
}

// sends, receives, bytes out, bytes in, calls of ucp_worker_progress, operations still in the table, broken
void gb_ucx_counters(void* handle, unsigned long long* seven) {
    auto* w = static_cast<UcxWorker*>(handle);
    std::lock_guard<std::mutex> hold(w->gate);
    seven[0] = w->sends; seven[1] = w->receives; seven[2] = w->bytes_out; seven[3] = w->bytes_in;
    seven[4] = w->progress_calls; seven[5] = w->table.size(); seven[6] = w->broken ? 1 : 0;
}

// 0: closed in time; 1: endpoints were still flushing at the limit and were torn down anyway.
int gb_ucx_close(void* handle, double limit_s) {
    auto* w = static_cast<UcxWorker*>(handle);
    int late;
    {
        std::lock_guard<std::mutex> hold(w->gate);
        late = w->shut(limit_s);
    }
    delete w;
    return late;
}

}  // extern "C"
