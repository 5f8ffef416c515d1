/*
 * qmm_gguf.h — C ABI of libqmm's GGUF container reader and writer.
 *
 * Counterpart of the upstream's weight-file side (recipe-infer/src/safetensors.rs:98-143:
 * parse_safetensors_header keeps name, dtype, shape and byte range per tensor and decodes nothing; a
 * tensor's bytes are fetched when it is placed) for the container the block formats of this library
 * come in.  Opening a file parses the header and the tensor table only; tensor bytes are read on demand,
 * straight into caller memory or, through a pinned bounce buffer in 64 MiB chunks (the upstream's upload
 * path, gpu-core/src/memory.rs:405-453), into device memory.  Array-valued metadata (vocabularies) is
 * skipped.  Byte compatibility with files written by other tools is unverified (no such file was
 * available); files written by the writer below round-trip.
 */
#ifndef QMM_GGUF_H
#define QMM_GGUF_H
#include "qmm.h"
#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    char name[128];
    int type;          /* GGUF type number: 0 F32, 1 F16, QMM_TYPE_* for the block formats */
    int n_dims;
    long dims[4];      /* dims[0] = row length (k), dims[1] = rows (n) */
    long file_offset;  /* absolute offset of the tensor's bytes in the file */
    long bytes;        /* 0: a type this library does not handle (listed, not readable) */
} qmm_gguf_tensor;

int qmm_gguf_open(const char* path, void** file);
int qmm_gguf_close(void* file);
long qmm_gguf_tensor_count(void* file);
long qmm_gguf_find(void* file, const char* name);                       /* index, or -1 */
int qmm_gguf_tensor_info(void* file, long index, qmm_gguf_tensor* out);
int qmm_gguf_read_tensor(void* file, long index, void* host_dst, long capacity);
int qmm_gguf_upload_tensor(void* file, long index, void* device_dst, long capacity, void* stream);
/* scalar metadata: QMM_ERR_SHAPE when the key is absent, QMM_ERR_TYPE when it holds another kind of value */
int qmm_gguf_meta_u64(void* file, const char* key, unsigned long long* out);
int qmm_gguf_meta_f64(void* file, const char* key, double* out);
long qmm_gguf_meta_str(void* file, const char* key, char* out, long capacity);   /* returns the string's length */

/* writer: metadata and tensors are collected in memory and written by qmm_gguf_writer_finish (which also
 * frees the writer).  dims as in qmm_gguf_tensor; bytes must equal rows * packed row bytes. */
int qmm_gguf_writer_create(const char* path, void** writer);
int qmm_gguf_writer_meta_u32(void* writer, const char* key, unsigned value);
int qmm_gguf_writer_meta_f32(void* writer, const char* key, float value);
int qmm_gguf_writer_meta_str(void* writer, const char* key, const char* value);
int qmm_gguf_writer_add_tensor(void* writer, const char* name, int type, int n_dims, const long* dims, const void* host_data, long bytes);
int qmm_gguf_writer_finish(void* writer);

#ifdef __cplusplus
}
#endif
#endif
