/*
 * qmm_store.h — C ABI of libqmm's tiered weight store.
 *
 * Counterpart of the upstream's Waterfall (gpu-core/src/waterfall.rs:86-168) and of the streaming glue of its
 * example (examples/gemma4.rs:363-400).  Blobs (tensors, expert slots) are placed hottest first: into ONE
 * device claim while it lasts, then into pinned host memory while its budget lasts, and what is left stays in
 * its file and is not read at placement.  A fetch returns a device pointer: into the claim for a resident blob
 * (nothing is copied), else into one of two staging windows that alternate, filled by an asynchronous copy on
 * the caller's stream (a file blob is read into a pinned bounce buffer first).  qmm_store_prefetch starts that
 * copy early on the store's own copy stream; qmm_store_fetch_cached keeps non-resident blobs in a small
 * least-recently-used cache of device slots (the upstream re-stages an expert on every use).
 * Single host thread per store, as upstream.
 */
#ifndef QMM_STORE_H
#define QMM_STORE_H
#include "qmm.h"
#ifdef __cplusplus
extern "C" {
#endif

#define QMM_TIER_VRAM 0
#define QMM_TIER_RAM 1
#define QMM_TIER_DISK 2

typedef struct {
    long vram_bytes, ram_bytes, disk_bytes;            /* placed per tier */
    long fetches_vram, fetches_ram, fetches_disk;      /* fetches served per tier (cache hits not included) */
    long cache_hits, staged_bytes;                     /* slot-cache hits; bytes copied host -> device by fetches */
} qmm_store_stats_t;

/* vram_budget_bytes: the device claim (0: none); ram_budget_bytes: host memory for blobs that do not fit it;
 * stage_bytes: size of each of the two staging windows (0: non-resident blobs cannot be fetched);
 * cache_slots x cache_slot_bytes: the device slot cache (0: none).  Without a CUDA device only a store with
 * all device sizes 0 can be created (placement into host memory and files still works). */
int qmm_store_create(long vram_budget_bytes, long ram_budget_bytes, long stage_bytes, int cache_slots, long cache_slot_bytes, void** store);
int qmm_store_destroy(void* store);
/* place a blob whose bytes are in host memory now (QMM_ERR_SCRATCH when neither device nor host budget has room) */
int qmm_store_place_host(void* store, const char* name, const void* host_src, long bytes);
/* place a blob that lives in a file (bytes [file_offset, file_offset + bytes)); read only if it lands in memory */
int qmm_store_place_file(void* store, const char* name, const char* path, long file_offset, long bytes);
int qmm_store_home(void* store, const char* name);     /* QMM_TIER_*, or a negative status */
int qmm_store_stats(void* store, qmm_store_stats_t* out);
/* device pointer valid for work enqueued on `stream` until the second fetch after this one */
int qmm_store_fetch(void* store, const char* name, void* stream, void** device_ptr);
int qmm_store_prefetch(void* store, const char* name, void* after_stream);
/* device pointer valid until cache_slots other blobs have been fetched through the cache */
int qmm_store_fetch_cached(void* store, const char* name, void* stream, void** device_ptr);

#ifdef __cplusplus
}
#endif
#endif
