// Registering device memory for an adapter that reads and writes it in place (GPUDirect RDMA):
// which way a range of device memory can be registered, a bounded cache of such registrations
// keyed by the identity of the ALLOCATION (not by address), and the one-receive "windows" a peer
// may write into.  Part of the RDMA-style bridge (gb_rdma.cpp is its endpoint); kept apart
// because it talks to two other parties - the GPU driver and the adapter's registration calls -
// through interfaces of their own, so that all of it runs and is tested without either
// (MockGpu, MockAdapter below).  (Role of the reference's verbs crate: direct.rs and gpu.rs.)
//
// Selection for a range of device memory, in order, each only where its checks pass:
//   1. dma-buf      the device exports dma-bufs, the range lies inside ONE allocation, the export
//                   of the page-rounded range succeeds and the adapter imports it;
//   2. peer memory  a peer-memory kernel module is loaded (nvidia_peermem / nv_peer_mem), the
//                   device allows it and the adapter registers the device pointer itself.
// If neither succeeds the caller gets EVERY reason ("dma-buf: ...; peer memory: ...") and stages
// through host memory; nothing is reported direct that is not.
//
// Identity and lifetime.  A cached registration belongs to the allocation's buffer id, which the
// driver never reuses within a process: the same address in a later allocation is another owner,
// and the stale entry is dropped when it is met (or the call is refused while posted work still
// holds it).  The cached range is the asked-for range rounded out to 2 MiB inside the
// allocation, so neighbouring tensors of one allocator segment share a registration.  A dma-buf
// entry owns its descriptor and closes it exactly once, after deregistering.
//
// Remote writes.  Nothing cached is remotely writable.  A receive that the peer writes into gets
// a window: an uncached registration of exactly its bytes, with remote write, made for that one
// receive and released when the peer has said "written".  The time spent making and releasing
// windows is counted.
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include <dlfcn.h>
#include <unistd.h>

namespace {

constexpr uint64_t ROUND = 2ull << 20;
enum Method { M_NONE = 0, M_DMABUF = 1, M_PEER = 2 };
enum Access { A_LOCAL = 1, A_REMOTE_WRITE = 2 };

uint64_t ns_now() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
        std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct Allocation { uint64_t base = 0, size = 0, buffer_id = 0; int device = -1; };

// ---- the GPU driver, as far as registration needs it ---------------------------------------------
struct GpuMemory {
    virtual ~GpuMemory() {}
    virtual bool dmabuf_support(int device, std::string* why) = 0;
    virtual bool peer_support(int device, std::string* why) = 0;
    virtual bool allocation(uint64_t va, Allocation* out, std::string* why) = 0;
    virtual int export_dmabuf(uint64_t va, uint64_t len, std::string* why) = 0;      // a descriptor, or -1
    virtual void close_descriptor(int fd) = 0;
    virtual uint64_t page() const { return 4096; }
};

// Pretend device memory for tests: allocations with never-reused buffer ids, descriptors that are
// plain numbers, and switches to make each step fail.
struct MockGpu final : GpuMemory {
    std::mutex mu;
    std::map<uint64_t, Allocation> live;               // by base
    uint64_t next_va = 0x7000'0000'0000ull, next_id = 1;
    int next_fd = 1000;
    std::map<int, int> closes;                         // descriptor -> times closed
    std::vector<int> open;
    std::string no_dmabuf, no_peer, no_export;
    uint64_t exports = 0;

    bool dmabuf_support(int, std::string* why) override {
        std::lock_guard<std::mutex> hold(mu);
        if (!no_dmabuf.empty()) { *why = no_dmabuf; return false; }
        return true;
    }
    bool peer_support(int, std::string* why) override {
        std::lock_guard<std::mutex> hold(mu);
        if (!no_peer.empty()) { *why = no_peer; return false; }
        return true;
    }
    bool allocation(uint64_t va, Allocation* out, std::string* why) override {
        std::lock_guard<std::mutex> hold(mu);
        auto it = live.upper_bound(va);
        if (it != live.begin()) {
            --it;
            if (va < it->second.base + it->second.size) { *out = it->second; return true; }
        }
        *why = "the address is not device memory of this process";
        return false;
    }
    int export_dmabuf(uint64_t, uint64_t, std::string* why) override {
        std::lock_guard<std::mutex> hold(mu);
        if (!no_export.empty()) { *why = no_export; return -1; }
        ++exports;
        open.push_back(next_fd);
        return next_fd++;
    }
    void close_descriptor(int fd) override {
        std::lock_guard<std::mutex> hold(mu);
        ++closes[fd];
        open.erase(std::remove(open.begin(), open.end(), fd), open.end());
    }
    uint64_t alloc(int device, uint64_t size, uint64_t at = 0) {
        std::lock_guard<std::mutex> hold(mu);
        Allocation a;
        a.base = at ? at : next_va;
        a.size = size;
        a.buffer_id = next_id++;
        a.device = device;
        if (!at) next_va += (size + ROUND - 1) / ROUND * ROUND + ROUND;
        live[a.base] = a;
        return a.base;
    }
    void release(uint64_t va) {
        std::lock_guard<std::mutex> hold(mu);
        live.erase(va);
    }
};

// The CUDA driver, loaded at run time (this library does not link against it): pointer attributes
// for the allocation's identity, the device's dma-buf attribute, and the export call.
struct DriverGpu final : GpuMemory {
    void* lib = nullptr;
    typedef int (*PointerAttr)(void*, int, unsigned long long);
    typedef int (*DeviceAttr)(int*, int, int);
    typedef int (*HandleForRange)(void*, unsigned long long, size_t, int, unsigned long long);
    PointerAttr pointer_attr = nullptr;
    DeviceAttr device_attr = nullptr;
    HandleForRange handle_for_range = nullptr;
    std::string problem;
    // numeric values of the driver API's enumerators (public header cuda.h)
    static constexpr int ATTR_DEVICE_ORDINAL = 9, ATTR_BUFFER_ID = 7, ATTR_RANGE_START = 11, ATTR_RANGE_SIZE = 12;
    static constexpr int DEV_ATTR_DMA_BUF = 124, DEV_ATTR_GDR = 116, HANDLE_DMA_BUF_FD = 1;

    DriverGpu() {
        lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
        if (lib == nullptr) { problem = "libcuda.so.1 cannot be loaded"; return; }
        pointer_attr = reinterpret_cast<PointerAttr>(dlsym(lib, "cuPointerGetAttribute"));
        device_attr = reinterpret_cast<DeviceAttr>(dlsym(lib, "cuDeviceGetAttribute"));
        handle_for_range = reinterpret_cast<HandleForRange>(dlsym(lib, "cuMemGetHandleForAddressRange"));
        if (pointer_attr == nullptr || device_attr == nullptr) { problem = "the driver lacks the pointer attribute calls"; return; }
        typedef int (*Init)(unsigned);
        Init init = reinterpret_cast<Init>(dlsym(lib, "cuInit"));
        const int rc = init != nullptr ? init(0) : -1;            // attribute queries need an initialised driver
        if (rc != 0) problem = "the CUDA driver did not initialise (cuInit: code " + std::to_string(rc) + ")";
    }
    ~DriverGpu() override { if (lib != nullptr) dlclose(lib); }
    bool ready(std::string* why) { if (!problem.empty()) { *why = problem; return false; } return true; }
    bool dmabuf_support(int device, std::string* why) override {
        if (!ready(why)) return false;
        if (handle_for_range == nullptr) { *why = "this driver has no cuMemGetHandleForAddressRange"; return false; }
        int value = 0;
        if (device_attr(&value, DEV_ATTR_DMA_BUF, device) != 0 || value == 0) {
            *why = "the device does not export dma-bufs (needs the open kernel modules)";
            return false;
        }
        return true;
    }
    bool peer_support(int device, std::string* why) override {
        if (!ready(why)) return false;
        int value = 0;
        if (device_attr(&value, DEV_ATTR_GDR, device) != 0 || value == 0) {
            *why = "the device does not support GPUDirect RDMA";
            return false;
        }
        return true;
    }
    bool allocation(uint64_t va, Allocation* out, std::string* why) override {
        if (!ready(why)) return false;
        unsigned long long id = 0, base = 0;
        size_t size = 0;
        int device = -1;
        if (pointer_attr(&id, ATTR_BUFFER_ID, va) != 0 || pointer_attr(&base, ATTR_RANGE_START, va) != 0 ||
            pointer_attr(&size, ATTR_RANGE_SIZE, va) != 0 || pointer_attr(&device, ATTR_DEVICE_ORDINAL, va) != 0) {
            *why = "the driver does not know this address as device memory";
            return false;
        }
        out->base = base; out->size = size; out->buffer_id = id; out->device = device;
        return true;
    }
    int export_dmabuf(uint64_t va, uint64_t len, std::string* why) override {
        int fd = -1;
        const int rc = handle_for_range(&fd, va, len, HANDLE_DMA_BUF_FD, 0);
        if (rc != 0) { *why = "cuMemGetHandleForAddressRange failed with code " + std::to_string(rc); return -1; }
        return fd;
    }
    void close_descriptor(int fd) override { if (fd >= 0) ::close(fd); }
    uint64_t page() const override { const long p = sysconf(_SC_PAGESIZE); return p > 0 ? (uint64_t)p : 4096; }
};

// Which peer-memory module is loaded, from <root>/proc/modules.
bool peer_module(const std::string& root, std::string* name) {
    std::ifstream modules(root + "/proc/modules");
    std::string line;
    while (std::getline(modules, line)) {
        const std::string first = line.substr(0, line.find(' '));
        if (first == "nvidia_peermem" || first == "nv_peer_mem") { *name = first; return true; }
    }
    return false;
}

// ---- the adapter's registration calls --------------------------------------------------------------
struct Adapter {
    virtual ~Adapter() {}
    virtual bool reg_dmabuf(int fd, uint64_t offset, uint64_t len, uint64_t iova, int access, uint32_t* key,
                            std::string* why) = 0;
    virtual bool reg_pointer(uint64_t va, uint64_t len, int access, uint32_t* key, std::string* why) = 0;
    virtual void dereg(uint32_t key) = 0;
};

struct MockAdapter final : Adapter {
    struct Made { uint32_t key; int method; uint64_t va, len; int access; int fd; };
    std::mutex mu;
    std::map<uint32_t, Made> live;
    uint32_t next_key = 0x5000;
    std::string no_dmabuf, no_pointer;
    uint64_t registrations = 0, deregistrations = 0;
    bool reg_dmabuf(int fd, uint64_t, uint64_t len, uint64_t iova, int access, uint32_t* key, std::string* why) override {
        std::lock_guard<std::mutex> hold(mu);
        if (!no_dmabuf.empty()) { *why = no_dmabuf; return false; }
        *key = next_key++;
        live[*key] = Made{*key, M_DMABUF, iova, len, access, fd};
        ++registrations;
        return true;
    }
    bool reg_pointer(uint64_t va, uint64_t len, int access, uint32_t* key, std::string* why) override {
        std::lock_guard<std::mutex> hold(mu);
        if (!no_pointer.empty()) { *why = no_pointer; return false; }
        *key = next_key++;
        live[*key] = Made{*key, M_PEER, va, len, access, -1};
        ++registrations;
        return true;
    }
    void dereg(uint32_t key) override {
        std::lock_guard<std::mutex> hold(mu);
        live.erase(key);
        ++deregistrations;
    }
};

// ---- the registrar -------------------------------------------------------------------------------------
struct Region {
    uint32_t key = 0;
    int method = M_NONE, device = -1, fd = -1;
    uint64_t lo = 0, hi = 0, buffer_id = 0;
    int held = 0;                                      // posted work that still uses it
    bool doomed = false;                               // invalidated while held: goes at the last release
};

struct Registrar {
    std::mutex mu;
    GpuMemory* gpu;
    Adapter* adapter;
    std::string modules_root;
    size_t capacity;
    std::list<std::shared_ptr<Region>> lru;            // most recently used first
    std::map<uint64_t, std::shared_ptr<Region>> windows;
    uint64_t next_window = 1;
    uint64_t hits = 0, misses = 0, evictions = 0, stale = 0, refusals = 0;
    uint64_t windows_made = 0, window_register_ns = 0, window_release_ns = 0;
    std::string dmabuf_off, peer_off;                  // a method the user switched off, with the reason to give

    void drop(const std::shared_ptr<Region>& r) {
        adapter->dereg(r->key);
        if (r->fd >= 0) gpu->close_descriptor(r->fd);  // after deregistering, exactly once
        r->fd = -1;
    }

    // Register [lo, hi) of allocation `a` with `access`; which method worked, or every reason.
    bool make(const Allocation& a, uint64_t lo, uint64_t hi, int access, Region* out, std::string* reasons) {
        std::string why, all;
        if (!dmabuf_off.empty()) {
            why = dmabuf_off;
        } else if (gpu->dmabuf_support(a.device, &why)) {
            const uint64_t page = gpu->page();
            const uint64_t from = lo / page * page, to = std::min(a.base + a.size, (hi + page - 1) / page * page);
            const int fd = gpu->export_dmabuf(from, to - from, &why);
            if (fd >= 0) {
                uint32_t key = 0;
                if (adapter->reg_dmabuf(fd, lo - from, hi - lo, lo, access, &key, &why)) {
                    out->key = key; out->method = M_DMABUF; out->fd = fd;
                    return true;
                }
                gpu->close_descriptor(fd);
            }
        }
        all += "dma-buf: " + why;
        why.clear();
        std::string module;
        if (!peer_off.empty()) {
            why = peer_off;
        } else if (!peer_module(modules_root, &module)) {
            why = "neither nvidia_peermem nor nv_peer_mem is loaded";
        } else if (gpu->peer_support(a.device, &why)) {
            uint32_t key = 0;
            if (adapter->reg_pointer(lo, hi - lo, access, &key, &why)) {
                out->key = key; out->method = M_PEER; out->fd = -1;
                return true;
            }
        }
        all += "; peer memory: " + why;
        *reasons = all;
        return false;
    }

    // A cached, locally-writable registration that covers [va, va + len).  The caller holds it
    // until release().
    std::shared_ptr<Region> acquire(uint64_t va, uint64_t len, std::string* reasons) {
        std::lock_guard<std::mutex> hold(mu);
        Allocation a;
        if (len == 0) { *reasons = "an empty range needs no registration"; return nullptr; }
        if (!gpu->allocation(va, &a, reasons)) return nullptr;
        if (va + len > a.base + a.size) {
            *reasons = "the range runs past the end of its allocation: it spans more than one";
            return nullptr;
        }
        for (auto it = lru.begin(); it != lru.end();) {
            Region& r = **it;
            const bool overlaps = va < r.hi && r.lo < va + len;
            if (overlaps && r.buffer_id != a.buffer_id) {         // the same addresses, another owner
                if (r.held > 0) {
                    ++refusals;
                    *reasons = "a registration of freed memory at this address is still held by posted work";
                    return nullptr;
                }
                ++stale;
                drop(*it);
                it = lru.erase(it);
                continue;
            }
            if (r.buffer_id == a.buffer_id && va >= r.lo && va + len <= r.hi && !r.doomed) {
                ++hits;
                ++r.held;
                auto found = *it;
                lru.splice(lru.begin(), lru, it);
                return found;
            }
            ++it;
        }
        ++misses;
        const uint64_t lo = std::max(a.base, va / ROUND * ROUND);
        const uint64_t hi = std::min(a.base + a.size, (va + len + ROUND - 1) / ROUND * ROUND);
        auto region = std::make_shared<Region>();
        if (!make(a, lo, hi, A_LOCAL, region.get(), reasons)) return nullptr;
        region->lo = lo; region->hi = hi; region->buffer_id = a.buffer_id; region->device = a.device;
        region->held = 1;
        lru.push_front(region);
        for (auto it = lru.end(); lru.size() > capacity && it != lru.begin();) {
            --it;
            if ((*it)->held > 0) continue;                        // in use: skip, try an older idle one
            ++evictions;
            drop(*it);
            it = lru.erase(it);
        }
        return region;
    }

    void release(const std::shared_ptr<Region>& region) {
        std::lock_guard<std::mutex> hold(mu);
        if (region->held > 0) --region->held;
        if (region->held == 0 && region->doomed) {
            drop(region);
            lru.remove(region);
        }
    }

    // The owner is about to free [va, va + len): forget what overlaps it (at once, or when the
    // last holder lets go).
    int invalidate(uint64_t va, uint64_t len) {
        std::lock_guard<std::mutex> hold(mu);
        int count = 0;
        for (auto it = lru.begin(); it != lru.end();) {
            Region& r = **it;
            if (va < r.hi && r.lo < va + len) {
                ++count;
                if (r.held > 0) { r.doomed = true; ++it; continue; }
                drop(*it);
                it = lru.erase(it);
            } else ++it;
        }
        return count;
    }

    // A window for ONE receive: exactly [va, va + len), remotely writable, never cached.
    uint64_t expose(uint64_t va, uint64_t len, uint32_t* key, std::string* reasons) {
        const uint64_t began = ns_now();
        std::lock_guard<std::mutex> hold(mu);
        Allocation a;
        if (!gpu->allocation(va, &a, reasons)) return 0;
        if (len == 0 || va + len > a.base + a.size) { *reasons = "the window does not lie inside one allocation"; return 0; }
        auto region = std::make_shared<Region>();
        if (!make(a, va, va + len, A_LOCAL | A_REMOTE_WRITE, region.get(), reasons)) return 0;
        region->lo = va; region->hi = va + len; region->buffer_id = a.buffer_id; region->device = a.device;
        const uint64_t id = next_window++;
        windows[id] = region;
        *key = region->key;
        ++windows_made;
        window_register_ns += ns_now() - began;
        return id;
    }
    bool close_window(uint64_t id) {
        const uint64_t began = ns_now();
        std::lock_guard<std::mutex> hold(mu);
        auto it = windows.find(id);
        if (it == windows.end()) return false;
        drop(it->second);
        windows.erase(it);
        window_release_ns += ns_now() - began;
        return true;
    }
    void clear() {
        std::lock_guard<std::mutex> hold(mu);
        for (auto& r : lru) drop(r);
        lru.clear();
        for (auto& w : windows) drop(w.second);
        windows.clear();
    }
    std::string capabilities(int device) {
        std::string why, module, out = "dma-buf: ";
        if (!dmabuf_off.empty()) out += "no (" + dmabuf_off + ")";
        else out += gpu->dmabuf_support(device, &why) ? "yes" : "no (" + why + ")";
        why.clear();
        out += "; peer memory: ";
        if (!peer_off.empty()) out += "no (" + peer_off + ")";
        else if (!peer_module(modules_root, &module)) out += "no (no peer-memory module is loaded)";
        else out += gpu->peer_support(device, &why) ? "yes (" + module + ")" : "no (" + why + ")";
        return out;
    }
    std::string telemetry() {
        std::lock_guard<std::mutex> hold(mu);
        int held = 0;
        for (auto& r : lru) held += r->held > 0;
        std::ostringstream s;
        s << "{\"cached\": " << lru.size() << ", \"held\": " << held << ", \"hits\": " << hits << ", \"misses\": " << misses
          << ", \"evictions\": " << evictions << ", \"stale_dropped\": " << stale << ", \"refusals\": " << refusals
          << ", \"windows_open\": " << windows.size() << ", \"windows_made\": " << windows_made
          << ", \"write_window_register_ns\": " << window_register_ns
          << ", \"write_window_release_ns\": " << window_release_ns << "}";
        return s.str();
    }
};

struct Handle {                                         // what the C interface hands out
    std::unique_ptr<GpuMemory> gpu;
    std::unique_ptr<Adapter> adapter;
    std::unique_ptr<Registrar> registrar;
    std::map<uint64_t, std::shared_ptr<Region>> taken;  // registrations handed to the caller, by ticket
    uint64_t next_ticket = 1;
    std::mutex mu;
};

void put(char* into, size_t room, const std::string& text) {
    if (into != nullptr && room > 0) std::snprintf(into, room, "%s", text.c_str());
}

}  // namespace

extern "C" {

// A registrar over pretend device memory and a pretend adapter (tests), or over the CUDA driver
// (`real` != 0; the adapter is still the pretend one until a provider over real queue pairs
// brings its own).  `modules_root` is where /proc is looked for ("" = the machine's).
void* gb_direct_new(int real, const char* modules_root, unsigned long long capacity) {
    auto* h = new Handle;
    if (real) h->gpu.reset(new DriverGpu); else h->gpu.reset(new MockGpu);
    h->adapter.reset(new MockAdapter);
    h->registrar.reset(new Registrar);
    h->registrar->gpu = h->gpu.get();
    h->registrar->adapter = h->adapter.get();
    h->registrar->modules_root = modules_root ? modules_root : "";
    h->registrar->capacity = capacity ? capacity : 1;
    return h;
}
void gb_direct_free(void* handle) {
    auto* h = static_cast<Handle*>(handle);
    h->taken.clear();
    h->registrar->clear();
    delete h;
}

// -- the pretend device (no-ops on a real one)
unsigned long long gb_direct_mock_alloc(void* handle, int device, unsigned long long size, unsigned long long at) {
    auto* gpu = dynamic_cast<MockGpu*>(static_cast<Handle*>(handle)->gpu.get());
    return gpu ? gpu->alloc(device, size, at) : 0;
}
void gb_direct_mock_release(void* handle, unsigned long long va) {
    auto* gpu = dynamic_cast<MockGpu*>(static_cast<Handle*>(handle)->gpu.get());
    if (gpu) gpu->release(va);
}
// what: 0 device has no dma-buf, 1 device refuses peer memory, 2 exports fail, 3 adapter refuses
// dma-bufs, 4 adapter refuses device pointers.  An empty reason switches the failure off.
void gb_direct_mock_fail(void* handle, int what, const char* reason) {
    auto* h = static_cast<Handle*>(handle);
    auto* gpu = dynamic_cast<MockGpu*>(h->gpu.get());
    auto* adapter = dynamic_cast<MockAdapter*>(h->adapter.get());
    const std::string why = reason ? reason : "";
    if (gpu && what == 0) gpu->no_dmabuf = why;
    if (gpu && what == 1) gpu->no_peer = why;
    if (gpu && what == 2) gpu->no_export = why;
    if (adapter && what == 3) adapter->no_dmabuf = why;
    if (adapter && what == 4) adapter->no_pointer = why;
}
// exports made, descriptors still open, descriptors closed more than once, adapter registrations
// alive, made, released
void gb_direct_mock_counts(void* handle, unsigned long long* six) {
    auto* h = static_cast<Handle*>(handle);
    std::memset(six, 0, 6 * sizeof *six);
    if (auto* gpu = dynamic_cast<MockGpu*>(h->gpu.get())) {
        std::lock_guard<std::mutex> hold(gpu->mu);
        six[0] = gpu->exports;
        six[1] = gpu->open.size();
        for (auto& c : gpu->closes) six[2] += c.second > 1;
    }
    if (auto* adapter = dynamic_cast<MockAdapter*>(h->adapter.get())) {
        std::lock_guard<std::mutex> hold(adapter->mu);
        six[3] = adapter->live.size(); six[4] = adapter->registrations; six[5] = adapter->deregistrations;
    }
}

// Switch a method off for this registrar (1 dma-buf, 2 peer memory), with the reason to report;
// an empty reason switches it back on.
void gb_direct_switch_off(void* handle, int method, const char* reason) {
    auto* r = static_cast<Handle*>(handle)->registrar.get();
    std::lock_guard<std::mutex> hold(r->mu);
    (method == M_DMABUF ? r->dmabuf_off : r->peer_off) = reason ? reason : "";
}

// -- registrations.  Returns a ticket (> 0) and fills method (1 dma-buf, 2 peer memory), key and the
// registered range; 0 with every reason in `why` when the range cannot be registered.
unsigned long long gb_direct_acquire(void* handle, unsigned long long va, unsigned long long len, int* method,
                                     unsigned* key, unsigned long long* lo, unsigned long long* hi,
                                     char* why, size_t room) {
    auto* h = static_cast<Handle*>(handle);
    std::string reasons;
    auto region = h->registrar->acquire(va, len, &reasons);
    if (!region) { put(why, room, reasons); return 0; }
    *method = region->method; *key = region->key; *lo = region->lo; *hi = region->hi;
    std::lock_guard<std::mutex> hold(h->mu);
    h->taken[h->next_ticket] = region;
    return h->next_ticket++;
}
int gb_direct_release(void* handle, unsigned long long ticket) {
    auto* h = static_cast<Handle*>(handle);
    std::shared_ptr<Region> region;
    {
        std::lock_guard<std::mutex> hold(h->mu);
        auto it = h->taken.find(ticket);
        if (it == h->taken.end()) return -1;
        region = it->second;
        h->taken.erase(it);
    }
    h->registrar->release(region);
    return 0;
}
int gb_direct_invalidate(void* handle, unsigned long long va, unsigned long long len) {
    return static_cast<Handle*>(handle)->registrar->invalidate(va, len);
}
unsigned long long gb_direct_expose(void* handle, unsigned long long va, unsigned long long len, unsigned* key,
                                    char* why, size_t room) {
    std::string reasons;
    const uint64_t id = static_cast<Handle*>(handle)->registrar->expose(va, len, key, &reasons);
    if (id == 0) put(why, room, reasons);
    return id;
}
int gb_direct_close_window(void* handle, unsigned long long window) {
    return static_cast<Handle*>(handle)->registrar->close_window(window) ? 0 : -1;
}
void gb_direct_capabilities(void* handle, int device, char* into, size_t room) {
    put(into, room, static_cast<Handle*>(handle)->registrar->capabilities(device));
}
void gb_direct_telemetry(void* handle, char* into, size_t room) {
    put(into, room, static_cast<Handle*>(handle)->registrar->telemetry());
}

}  // extern "C"
