// The collectives of gb_tagged.h and the element-wise folds they use (see the header).
#include "gb_tagged.h"

#include <cstring>
#include <vector>

namespace {

enum Dtype { F32 = 0, BF16 = 1, F16 = 2, F64 = 3, I8 = 4, U8 = 5, I32 = 6, I64 = 7 };
enum Fold { SUM = 0, MAX = 1, MIN = 2 };

inline uint64_t make_tag_(uint64_t seq, uint64_t step, uint64_t sender, uint64_t chunk) {
    return ((seq & 0xFFFFFFull) << 40) | ((step & 0xFFFull) << 28) | ((sender & 0xFFull) << 20) |
           (chunk & 0xFFFFFull);
}

inline float bf16_to_float(uint16_t v) {
    uint32_t bits = (uint32_t)v << 16;
    float f; std::memcpy(&f, &bits, 4); return f;
}
inline uint16_t float_to_bf16(float f) {                       // round to nearest even
    uint32_t bits; std::memcpy(&bits, &f, 4);
    if ((bits & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)0x7FC0u;                  // NaN, as torch rounds it
    bits += 0x7FFFu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}
inline float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            bits = sign | ((uint32_t)(113 - shift) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f; std::memcpy(&f, &bits, 4); return f;
}
inline uint16_t float_to_half(float f) {                        // round to nearest even
    uint32_t bits; std::memcpy(&bits, &f, 4);
    uint32_t sign = (bits >> 16) & 0x8000u;
    int32_t exp = (int32_t)((bits >> 23) & 0xFFu) - 127 + 15;
    uint32_t man = bits & 0x7FFFFFu;
    if (((bits >> 23) & 0xFFu) == 0xFFu) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u | (man >> 13) : 0u));
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - exp);
        uint32_t half = man >> shift, rest = man & ((1u << shift) - 1u), mid = 1u << (shift - 1);
        if (rest > mid || (rest == mid && (half & 1u))) ++half;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)exp << 10) | (man >> 13), rest = man & 0x1FFFu;
    if (rest > 0x1000u || (rest == 0x1000u && (half & 1u))) ++half;
    return (uint16_t)(sign | half);
}

template <typename T> inline T fold_one(T a, T b, int op) {
    if (op == SUM) return (T)(a + b);
    if (a != a) return a;                                       // NaN wins, as torch.maximum does
    if (b != b) return b;
    if (op == MAX) return a > b ? a : b;
    return a < b ? a : b;
}

template <typename T> void fold_plain(void* into, const void* from, size_t n, int op) {
    T* a = static_cast<T*>(into);
    const T* b = static_cast<const T*>(from);
    for (size_t i = 0; i < n; ++i) a[i] = fold_one<T>(a[i], b[i], op);
}

template <float (*Up)(uint16_t), uint16_t (*Down)(float)>
void fold_16(void* into, const void* from, size_t n, int op) {
    uint16_t* a = static_cast<uint16_t*>(into);
    const uint16_t* b = static_cast<const uint16_t*>(from);
    for (size_t i = 0; i < n; ++i) a[i] = Down(fold_one<float>(Up(a[i]), Up(b[i]), op));
}

size_t dtype_size_(int dtype) {
    switch (dtype) {
        case F32: case I32: return 4;
        case BF16: case F16: return 2;
        case F64: case I64: return 8;
        case I8: case U8: return 1;
    }
    return 0;
}

void fold_(int dtype, void* into, const void* from, size_t n, int op) {
    switch (dtype) {
        case F32: fold_plain<float>(into, from, n, op); break;
        case F64: fold_plain<double>(into, from, n, op); break;
        case I8: fold_plain<int8_t>(into, from, n, op); break;
        case U8: fold_plain<uint8_t>(into, from, n, op); break;
        case I32: fold_plain<int32_t>(into, from, n, op); break;
        case I64: fold_plain<int64_t>(into, from, n, op); break;
        case BF16: fold_16<bf16_to_float, float_to_bf16>(into, from, n, op); break;
        case F16: fold_16<half_to_float, float_to_half>(into, from, n, op); break;
    }
}

// Post `count` elements starting at `base` as chunks; the ids go to `ids`.
bool post_chunks(GbTaggedWorker& w, bool sending, int peer, char* base, size_t count, size_t esize,
                 size_t chunk, uint64_t seq, uint64_t step, uint64_t sender, std::vector<long>& ids) {
    size_t index = 0;
    for (size_t start = 0; start < count || (count == 0 && index == 0); start += chunk, ++index) {
        const size_t n = count - start < chunk ? count - start : chunk;
        const uint64_t t = make_tag_(seq, step, sender, index);
        long id = sending ? w.send(peer, base + start * esize, n * esize, t)
                          : w.recv(peer, base + start * esize, n * esize, t);
        if (id < 0) return false;
        ids.push_back(id);
        if (count == 0) break;
    }
    return true;
}

}  // namespace

size_t gb_tagged_dtype_size(int dtype) { return dtype_size_(dtype); }
void gb_tagged_fold(int dtype, void* into, const void* from, size_t n, int op) { fold_(dtype, into, from, n, op); }
uint64_t gb_tagged_tag(uint64_t seq, uint64_t step, uint64_t sender, uint64_t chunk) {
    return make_tag_(seq, step, sender, chunk);
}

int gb_tagged_all_reduce(GbTaggedWorker& w, void* data, uint64_t count, int dtype, int op,
                         uint64_t chunk_elems, uint64_t seq, double timeout_s) {
    const size_t esize = gb_tagged_dtype_size(dtype);
    if (esize == 0 || op < SUM || op > MIN) { w.fail("all_reduce: unsupported dtype or op"); return -1; }
    const int size = w.members(), me = w.index();
    if (size == 1 || count == 0) return 0;
    if (chunk_elems == 0) chunk_elems = 1;
    char* flat = static_cast<char*>(data);
    if (size == 2) {
        const int peer = 1 - me;
        std::vector<char> scratch(count * esize);
        std::vector<long> got, sent;
        if (!post_chunks(w, false, peer, scratch.data(), count, esize, chunk_elems, seq, 0, peer, got) ||
            !post_chunks(w, true, peer, flat, count, esize, chunk_elems, seq, 0, me, sent)) {
            w.stop();
            return -1;
        }
        size_t index = 0;
        for (size_t start = 0; start < count; start += chunk_elems, ++index) {
            const size_t n = count - start < chunk_elems ? count - start : chunk_elems;
            long pair[2] = {got[index], sent[index]};
            if (w.wait(pair, 2, timeout_s) != 0) return -1;
            gb_tagged_fold(dtype, flat + start * esize, scratch.data() + start * esize, n, op);
        }
        return 0;
    }
    const int right = (me + 1) % size, left = (me + size - 1) % size;
    const size_t base = count / size, extra = count % size;
    auto seg_start = [&](int i) { i = ((i % size) + size) % size; return (size_t)i * base + ((size_t)i < extra ? (size_t)i : extra); };
    auto seg_len = [&](int i) { i = ((i % size) + size) % size; return base + ((size_t)i < extra ? 1 : 0); };
    std::vector<char> scratch((base + 1) * esize);
    for (int step = 0; step < size - 1; ++step) {               // reduce-scatter
        const int in_seg = me - step - 1, out_seg = me - step;
        std::vector<long> ids;
        if (!post_chunks(w, false, left, scratch.data(), seg_len(in_seg), esize, chunk_elems, seq, step, left, ids) ||
            !post_chunks(w, true, right, flat + seg_start(out_seg) * esize, seg_len(out_seg), esize,
                         chunk_elems, seq, step, me, ids)) {
            w.stop();
            return -1;
        }
        if (w.wait(ids.data(), (int)ids.size(), timeout_s) != 0) return -1;
        gb_tagged_fold(dtype, flat + seg_start(in_seg) * esize, scratch.data(), seg_len(in_seg), op);
    }
    for (int step = 0; step < size - 1; ++step) {               // all-gather: I own segment me + 1
        const int in_seg = me - step, out_seg = me + 1 - step;
        std::vector<long> ids;
        if (!post_chunks(w, false, left, flat + seg_start(in_seg) * esize, seg_len(in_seg), esize,
                         chunk_elems, seq, size + step, left, ids) ||
            !post_chunks(w, true, right, flat + seg_start(out_seg) * esize, seg_len(out_seg), esize,
                         chunk_elems, seq, size + step, me, ids)) {
            w.stop();
            return -1;
        }
        if (w.wait(ids.data(), (int)ids.size(), timeout_s) != 0) return -1;
    }
    return 0;
}

int gb_tagged_broadcast(GbTaggedWorker& w, void* data, uint64_t nbytes, int root, uint64_t chunk_bytes,
                        uint64_t seq, double timeout_s) {
    if (w.members() == 1) return 0;
    if (chunk_bytes == 0) chunk_bytes = 1;
    char* flat = static_cast<char*>(data);
    std::vector<long> ids;
    bool ok = true;
    if (w.index() == root) {
        for (int peer = 0; peer < w.members() && ok; ++peer)
            if (peer != root)
                ok = post_chunks(w, true, peer, flat, nbytes, 1, chunk_bytes, seq, 0, root, ids);
    } else {
        ok = post_chunks(w, false, root, flat, nbytes, 1, chunk_bytes, seq, 0, root, ids);
    }
    if (!ok) { w.stop(); return -1; }
    return w.wait(ids.data(), (int)ids.size(), timeout_s);
}

