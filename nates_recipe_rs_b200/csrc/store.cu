// Weight residency: a three-tier store (device memory, pinned host memory, file) with stream-ordered
// staging, for models larger than one GPU's memory and for banks of experts.
//
// Counterpart of the upstream's Waterfall (gpu-core/src/waterfall.rs:86-168: ONE device claim carved
// hottest-first, then host memory down to a floor, the rest stays on disk and is never read at placement)
// and of the streaming glue of its example (examples/gemma4.rs:363-400: a resident blob is used in
// place, a host blob bounces through a staging buffer, a disk blob is read into it first; expert slots the
// same three ways).  Differences that follow from the hardware: staging is asynchronous on the caller's
// stream out of pinned memory (the upstream's copies are synchronous), two staging windows alternate so a
// prefetch of the next blob can run on a copy stream while kernels consume the current one, and blobs that
// do not live in device memory can be kept in a small least-recently-used cache of device slots (the
// upstream re-stages an expert on every use).
#include "qmm_common.cuh"
#include "../../include/qmm_store.h"
#include <fcntl.h>
#include <unistd.h>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace qmm {

struct StoreBlob {
    int tier = QMM_TIER_DISK;
    size_t bytes = 0;
    uint8_t* dev = nullptr;    // tier VRAM: inside the slab
    uint8_t* host = nullptr;   // tier RAM
    std::string path;          // tier DISK
    uint64_t file_offset = 0;
    int cache_slot = -1;       // device cache slot currently holding this blob, or -1
};

struct Store {
    size_t vram_budget = 0, vram_used = 0, ram_budget = 0, ram_used = 0, disk_bytes = 0;
    uint8_t* slab = nullptr;
    bool pinned = false;       // host copies live in pinned memory (false only when no CUDA device is present)
    // staging: two device windows and two pinned bounce buffers, used alternately
    size_t stage_bytes = 0;
    uint8_t* window[2] = {nullptr, nullptr};
    uint8_t* bounce[2] = {nullptr, nullptr};
    cudaEvent_t bounce_free[2] = {nullptr, nullptr};  // the copy out of the bounce buffer has finished
    cudaEvent_t prefetched = nullptr;
    cudaStream_t copy_stream = nullptr;
    int next_window = 0;
    std::string prefetch_name;  // blob whose bytes are (being) copied into window[prefetch_window]
    int prefetch_window = -1;
    // least-recently-used cache of device slots for blobs that are not resident
    size_t slot_bytes = 0;
    int n_slots = 0;
    uint8_t* slots = nullptr;
    std::vector<std::string> slot_owner;
    std::vector<unsigned long long> slot_stamp;
    unsigned long long clock = 0;
    std::map<std::string, StoreBlob> blobs;
    unsigned long long fetches[3] = {0, 0, 0}, cache_hits = 0, staged_bytes = 0;
};

static void store_free_host(Store* s, uint8_t* p) {
    if (!p) return;
    if (s->pinned) cudaFreeHost(p);
    else std::free(p);
}

static void store_destroy(Store* s) {
    if (!s) return;
    for (auto& kv : s->blobs) store_free_host(s, kv.second.host);
    for (int i = 0; i < 2; ++i) {
        if (s->window[i]) cudaFree(s->window[i]);
        store_free_host(s, s->bounce[i]);
        if (s->bounce_free[i]) cudaEventDestroy(s->bounce_free[i]);
    }
    if (s->prefetched) cudaEventDestroy(s->prefetched);
    if (s->copy_stream) cudaStreamDestroy(s->copy_stream);
    if (s->slots) cudaFree(s->slots);
    if (s->slab) cudaFree(s->slab);
    delete s;
}

static bool read_file_range(const std::string& path, uint64_t off, void* dst, size_t n) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) return false;
    size_t done = 0;
    while (done < n) {
        const ssize_t r = pread(fd, static_cast<char*>(dst) + done, n - done, (off_t)(off + done));
        if (r <= 0) break;
        done += (size_t)r;
    }
    close(fd);
    return done == n;
}

// Places one blob, hottest first: device memory while the claim lasts, then host memory while its budget lasts,
// else the blob stays in its file.  The bytes are read (from `host_src`, or from the file) only when the blob
// lands in device or host memory.
static int store_place(Store* s, const char* name, const void* host_src, const char* path, uint64_t file_offset, size_t bytes) {
    if (s->blobs.count(name)) return QMM_ERR_SHAPE;  // placed already
    if (!host_src && !path) return QMM_ERR_NULL;
    StoreBlob b;
    b.bytes = bytes;
    if (path) b.path = path, b.file_offset = file_offset;
    const size_t padded = (bytes + 255) & ~size_t(255);
    std::vector<uint8_t> tmp;
    auto source = [&]() -> const void* {
        if (host_src) return host_src;
        tmp.resize(bytes);
        return read_file_range(b.path, file_offset, tmp.data(), bytes) ? tmp.data() : nullptr;
    };
    if (s->slab && s->vram_used + padded <= s->vram_budget) {
        const void* src = source();
        if (!src) return QMM_ERR_IO;
        b.tier = QMM_TIER_VRAM;
        b.dev = s->slab + s->vram_used;
        QMM_CUDA_TRY(cudaMemcpy(b.dev, src, bytes, cudaMemcpyHostToDevice));
        s->vram_used += padded;
    } else if (s->ram_used + bytes <= s->ram_budget) {
        const void* src = source();
        if (!src) return QMM_ERR_IO;
        b.tier = QMM_TIER_RAM;
        if (s->pinned) {
            void* p = nullptr;
            QMM_CUDA_TRY(cudaMallocHost(&p, bytes));
            b.host = static_cast<uint8_t*>(p);
        } else {
            b.host = static_cast<uint8_t*>(std::malloc(bytes));
            if (!b.host) return QMM_ERR_IO;
        }
        std::memcpy(b.host, src, bytes);
        s->ram_used += bytes;
    } else {
        if (!path) return QMM_ERR_SCRATCH;  // nowhere to keep bytes that have no file behind them
        b.tier = QMM_TIER_DISK;
        s->disk_bytes += bytes;
    }
    s->blobs[name] = b;
    return QMM_OK;
}

// Starts the copy of a non-resident blob into window w on `stream` (bounce buffer w; its previous copy has
// finished before it is overwritten).
static int store_stage(Store* s, const StoreBlob& b, int w, cudaStream_t stream) {
    if (b.bytes > s->stage_bytes) return QMM_ERR_SCRATCH;
    const uint8_t* src = b.host;
    if (b.tier == QMM_TIER_DISK) {
        QMM_CUDA_TRY(cudaEventSynchronize(s->bounce_free[w]));
        if (!read_file_range(b.path, b.file_offset, s->bounce[w], b.bytes)) return QMM_ERR_IO;
        src = s->bounce[w];
    }
    QMM_CUDA_TRY(cudaMemcpyAsync(s->window[w], src, b.bytes, cudaMemcpyHostToDevice, stream));
    if (b.tier == QMM_TIER_DISK) QMM_CUDA_TRY(cudaEventRecord(s->bounce_free[w], stream));
    s->staged_bytes += b.bytes;
    return QMM_OK;
}

}  // namespace qmm

using namespace qmm;

extern "C" {

int qmm_store_create(long vram_budget_bytes, long ram_budget_bytes, long stage_bytes, int cache_slots, long cache_slot_bytes, void** store) {
    if (!store) return QMM_ERR_NULL;
    if (vram_budget_bytes < 0 || ram_budget_bytes < 0 || stage_bytes < 0 || cache_slots < 0 || cache_slot_bytes < 0) return QMM_ERR_SHAPE;
    Store* s = new Store();
    int n_dev = 0;
    s->pinned = cudaGetDeviceCount(&n_dev) == cudaSuccess && n_dev > 0;
    if (!s->pinned) cudaGetLastError();
    s->ram_budget = (size_t)ram_budget_bytes;
    auto fail = [&](cudaError_t e) {
        store_destroy(s);
        return cuda_fail(e);
    };
    if ((vram_budget_bytes > 0 || stage_bytes > 0 || cache_slots > 0) && !s->pinned) {
        store_destroy(s);
        return QMM_ERR_UNSUPPORTED;  // device tiers need a device
    }
    if (vram_budget_bytes > 0) {  // the one claim: every resident blob is carved from it
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, (size_t)vram_budget_bytes);
        if (e != cudaSuccess) return fail(e);
        s->slab = static_cast<uint8_t*>(p);
        s->vram_budget = (size_t)vram_budget_bytes;
    }
    if (stage_bytes > 0) {
        s->stage_bytes = (size_t)stage_bytes;
        for (int i = 0; i < 2; ++i) {
            void *w = nullptr, *b = nullptr;
            cudaError_t e = cudaMalloc(&w, s->stage_bytes);
            if (e == cudaSuccess) e = cudaMallocHost(&b, s->stage_bytes);
            s->window[i] = static_cast<uint8_t*>(w), s->bounce[i] = static_cast<uint8_t*>(b);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->bounce_free[i], cudaEventDisableTiming);
            if (e != cudaSuccess) return fail(e);
        }
        cudaError_t e = cudaEventCreateWithFlags(&s->prefetched, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s->copy_stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) return fail(e);
    }
    if (cache_slots > 0 && cache_slot_bytes > 0) {
        s->n_slots = cache_slots;
        s->slot_bytes = ((size_t)cache_slot_bytes + 255) & ~size_t(255);
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, s->slot_bytes * cache_slots);
        if (e != cudaSuccess) return fail(e);
        s->slots = static_cast<uint8_t*>(p);
        s->slot_owner.assign(cache_slots, std::string());
        s->slot_stamp.assign(cache_slots, 0);
    }
    *store = s;
    return QMM_OK;
}

int qmm_store_destroy(void* store) {
    if (!store) return QMM_ERR_NULL;
    if (static_cast<Store*>(store)->pinned) cudaDeviceSynchronize();
    store_destroy(static_cast<Store*>(store));
    return QMM_OK;
}

int qmm_store_place_host(void* store, const char* name, const void* host_src, long bytes) {
    if (!store || !name || !host_src) return QMM_ERR_NULL;
    if (bytes <= 0) return QMM_ERR_SHAPE;
    return store_place(static_cast<Store*>(store), name, host_src, nullptr, 0, (size_t)bytes);
}

int qmm_store_place_file(void* store, const char* name, const char* path, long file_offset, long bytes) {
    if (!store || !name || !path) return QMM_ERR_NULL;
    if (bytes <= 0 || file_offset < 0) return QMM_ERR_SHAPE;
    return store_place(static_cast<Store*>(store), name, nullptr, path, (uint64_t)file_offset, (size_t)bytes);
}

int qmm_store_home(void* store, const char* name) {
    if (!store || !name) return QMM_ERR_NULL;
    Store* s = static_cast<Store*>(store);
    auto it = s->blobs.find(name);
    return it == s->blobs.end() ? QMM_ERR_SHAPE : it->second.tier;
}

int qmm_store_stats(void* store, qmm_store_stats_t* out) {
    if (!store || !out) return QMM_ERR_NULL;
    Store* s = static_cast<Store*>(store);
    out->vram_bytes = (long)s->vram_used, out->ram_bytes = (long)s->ram_used, out->disk_bytes = (long)s->disk_bytes;
    out->fetches_vram = (long)s->fetches[0], out->fetches_ram = (long)s->fetches[1], out->fetches_disk = (long)s->fetches[2];
    out->cache_hits = (long)s->cache_hits, out->staged_bytes = (long)s->staged_bytes;
    return QMM_OK;
}

// A device pointer to the blob's bytes, valid for work enqueued on `stream` until the second fetch after
// this one (the staging windows alternate).  Resident blob: the pointer into the claim, nothing is copied.
int qmm_store_fetch(void* store, const char* name, void* stream, void** device_ptr) {
    if (!store || !name || !device_ptr) return QMM_ERR_NULL;
    Store* s = static_cast<Store*>(store);
    auto it = s->blobs.find(name);
    if (it == s->blobs.end()) return QMM_ERR_SHAPE;
    StoreBlob& b = it->second;
    s->fetches[b.tier]++;
    if (b.tier == QMM_TIER_VRAM) {
        *device_ptr = b.dev;
        return QMM_OK;
    }
    cudaStream_t st = as_stream(stream);
    if (s->prefetch_window >= 0 && s->prefetch_name == name) {  // its copy is already under way on the copy stream
        QMM_CUDA_TRY(cudaStreamWaitEvent(st, s->prefetched, 0));
        *device_ptr = s->window[s->prefetch_window];
        s->next_window = 1 - s->prefetch_window;
        s->prefetch_window = -1;
        return QMM_OK;
    }
    if (!s->stage_bytes) return QMM_ERR_SCRATCH;
    const int w = s->next_window;
    if (int rc = store_stage(s, b, w, st)) return rc;
    s->next_window = 1 - w;
    *device_ptr = s->window[w];
    return QMM_OK;
}

// Starts staging a non-resident blob on the store's copy stream, into the window the next fetch would use,
// while kernels enqueued on `after_stream` so far still run; the next qmm_store_fetch of the same name only waits
// for the copy.  `after_stream`: the stream whose already enqueued work last read that window (two fetches ago).
int qmm_store_prefetch(void* store, const char* name, void* after_stream) {
    if (!store || !name) return QMM_ERR_NULL;
    Store* s = static_cast<Store*>(store);
    auto it = s->blobs.find(name);
    if (it == s->blobs.end()) return QMM_ERR_SHAPE;
    StoreBlob& b = it->second;
    if (b.tier == QMM_TIER_VRAM) return QMM_OK;
    if (!s->stage_bytes) return QMM_ERR_SCRATCH;
    const int w = s->next_window;
    // the window may still be read by kernels enqueued before this call: order the copy after them
    QMM_CUDA_TRY(cudaEventRecord(s->prefetched, as_stream(after_stream)));
    QMM_CUDA_TRY(cudaStreamWaitEvent(s->copy_stream, s->prefetched, 0));
    if (int rc = store_stage(s, b, w, s->copy_stream)) return rc;
    QMM_CUDA_TRY(cudaEventRecord(s->prefetched, s->copy_stream));
    s->prefetch_name = name;
    s->prefetch_window = w;
    return QMM_OK;
}

// The same through the cache of device slots: a blob used recently is found in its slot and nothing is copied;
// otherwise the least recently used slot is overwritten (stream-ordered on `stream`: its earlier readers were
// enqueued on the same stream).  The pointer stays valid until cache_slots other blobs have been fetched.
int qmm_store_fetch_cached(void* store, const char* name, void* stream, void** device_ptr) {
    if (!store || !name || !device_ptr) return QMM_ERR_NULL;
    Store* s = static_cast<Store*>(store);
    auto it = s->blobs.find(name);
    if (it == s->blobs.end()) return QMM_ERR_SHAPE;
    StoreBlob& b = it->second;
    if (b.tier == QMM_TIER_VRAM) {
        s->fetches[0]++;
        *device_ptr = b.dev;
        return QMM_OK;
    }
    if (!s->n_slots || b.bytes > s->slot_bytes) return QMM_ERR_SCRATCH;
    ++s->clock;
    if (b.cache_slot >= 0 && s->slot_owner[b.cache_slot] == name) {
        s->cache_hits++;
        s->slot_stamp[b.cache_slot] = s->clock;
        *device_ptr = s->slots + (size_t)b.cache_slot * s->slot_bytes;
        return QMM_OK;
    }
    s->fetches[b.tier]++;
    int victim = 0;
    for (int i = 1; i < s->n_slots; ++i)
        if (s->slot_stamp[i] < s->slot_stamp[victim]) victim = i;
    if (!s->slot_owner[victim].empty()) {
        auto old = s->blobs.find(s->slot_owner[victim]);
        if (old != s->blobs.end()) old->second.cache_slot = -1;
    }
    uint8_t* dst = s->slots + (size_t)victim * s->slot_bytes;
    cudaStream_t st = as_stream(stream);
    const uint8_t* src = b.host;
    if (b.tier == QMM_TIER_DISK) {
        if (!s->stage_bytes || b.bytes > s->stage_bytes) return QMM_ERR_SCRATCH;
        QMM_CUDA_TRY(cudaEventSynchronize(s->bounce_free[0]));
        if (!read_file_range(b.path, b.file_offset, s->bounce[0], b.bytes)) return QMM_ERR_IO;
        src = s->bounce[0];
    }
    QMM_CUDA_TRY(cudaMemcpyAsync(dst, src, b.bytes, cudaMemcpyHostToDevice, st));
    if (b.tier == QMM_TIER_DISK) QMM_CUDA_TRY(cudaEventRecord(s->bounce_free[0], st));
    s->staged_bytes += b.bytes;
    s->slot_owner[victim] = name;
    s->slot_stamp[victim] = s->clock;
    b.cache_slot = victim;
    *device_ptr = dst;
    return QMM_OK;
}

}  // extern "C"
