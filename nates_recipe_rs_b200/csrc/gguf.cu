// GGUF container: header-only parse with seek-on-demand tensor reads, and a writer for synthetic files.
//
// The upstream's on-disk side of inference is safetensors, read the same way: parse only the header, keep
// (name, dtype, shape, byte range) per tensor, and fetch a tensor's bytes when it is placed
// (recipe-infer/src/safetensors.rs:98-143; upload through a pinned bounce buffer in chunks,
// gpu-core/src/memory.rs:405-453).  GGUF is the container the block formats of this library come in; the
// layout below restates its published description (version 3, little endian):
//   u32 magic "GGUF", u32 version, u64 tensor_count, u64 metadata_kv_count,
//   metadata: { string key, u32 value_type, value }          string = u64 length + bytes (no terminator)
//       value types 0..12: u8 i8 u16 i16 u32 i32 f32 bool string array u64 i64 f64;  array = u32 element
//       type, u64 count, elements
//   tensor infos: { string name, u32 n_dims, u64 dims[n_dims] (dims[0] = row length), u32 type, u64 offset }
//   padding to `general.alignment` (default 32), then the tensor data; offsets are relative to its start.
// No real GGUF file was available to check against, so byte compatibility with files written by other tools
// is unverified; files written by the writer below round-trip.
#include "qmm_common.cuh"
#include "../../include/qmm_gguf.h"
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace qmm {

constexpr uint32_t GGUF_MAGIC = 0x46554747u;  // "GGUF"
constexpr size_t GGUF_BOUNCE_BYTES = 64u << 20;

struct GgufMeta {
    uint32_t type = 0;
    uint64_t u = 0;      // integer and bool values
    double f = 0.0;      // float values
    std::string s;       // string values
    uint64_t array_count = 0;  // arrays are skipped, only their length is kept
};

struct GgufTensor {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint32_t type = 0;
    uint64_t offset = 0;  // relative to the data section
    uint64_t bytes = 0;
};

struct GgufFile {
    int fd = -1;
    uint64_t file_size = 0, data_start = 0, alignment = 32;
    uint32_t version = 0;
    std::vector<GgufTensor> tensors;
    std::map<std::string, long> by_name;
    std::map<std::string, GgufMeta> meta;
    void* bounce = nullptr;  // pinned staging for uploads, allocated on first use
};

// bytes of `elems` elements of a ggml type, or 0 when the type is not one this library handles
static uint64_t gguf_type_bytes(uint32_t type, uint64_t elems) {
    switch (type) {
    case 0: return elems * 4;                                           // F32
    case 1: return elems * 2;                                           // F16
    case QMM_TYPE_Q8_0: return elems % 32 ? 0 : elems / 32 * Q8_0_BYTES;
    case QMM_TYPE_Q8_1: return elems % 32 ? 0 : elems / 32 * Q8_1_BYTES;
    case QMM_TYPE_Q4_K: return elems % 256 ? 0 : elems / 256 * Q4_K_BYTES;
    case QMM_TYPE_Q6_K: return elems % 256 ? 0 : elems / 256 * Q6_K_BYTES;
    }
    return 0;
}

// sequential reader over the header with a refillable window (headers of real models carry megabytes of vocabulary)
struct GgufCursor {
    int fd;
    uint64_t pos, size;
    bool ok = true;
    bool read(void* dst, size_t n) {
        if (!ok || pos + n > size) return ok = false;
        size_t done = 0;
        while (done < n) {
            const ssize_t r = pread(fd, static_cast<char*>(dst) + done, n - done, (off_t)(pos + done));
            if (r <= 0) return ok = false;
            done += (size_t)r;
        }
        pos += n;
        return true;
    }
    template <typename T>
    T get() {
        T v{};
        read(&v, sizeof(T));
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > (1u << 24)) {
            ok = false;
            return {};
        }
        std::string s(n, '\0');
        if (n) read(&s[0], n);
        return s;
    }
    void skip(uint64_t n) {
        if (pos + n > size) ok = false;
        pos += n;
    }
};

static uint64_t gguf_scalar_size(uint32_t t) {
    switch (t) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    }
    return 0;
}

static bool gguf_read_value(GgufCursor& c, uint32_t type, GgufMeta& m, int depth) {
    m.type = type;
    switch (type) {
    case 0: m.u = c.get<uint8_t>(); break;
    case 1: m.u = (uint64_t)(int64_t)c.get<int8_t>(); break;
    case 2: m.u = c.get<uint16_t>(); break;
    case 3: m.u = (uint64_t)(int64_t)c.get<int16_t>(); break;
    case 4: m.u = c.get<uint32_t>(); break;
    case 5: m.u = (uint64_t)(int64_t)c.get<int32_t>(); break;
    case 6: m.f = c.get<float>(); break;
    case 7: m.u = c.get<uint8_t>() != 0; break;
    case 8: m.s = c.str(); break;
    case 10: m.u = c.get<uint64_t>(); break;
    case 11: m.u = (uint64_t)c.get<int64_t>(); break;
    case 12: m.f = c.get<double>(); break;
    case 9: {  // array: element type, count, elements (skipped)
        if (depth > 2) return c.ok = false;
        const uint32_t et = c.get<uint32_t>();
        const uint64_t n = c.get<uint64_t>();
        m.array_count = n;
        if (const uint64_t sz = gguf_scalar_size(et)) {
            c.skip(n * sz);
        } else if (et == 8) {
            for (uint64_t i = 0; i < n && c.ok; ++i) c.skip(c.get<uint64_t>());
        } else if (et == 9) {
            for (uint64_t i = 0; i < n && c.ok; ++i) {
                GgufMeta inner;
                gguf_read_value(c, 9, inner, depth + 1);
            }
        } else {
            return c.ok = false;
        }
        break;
    }
    default: return c.ok = false;
    }
    return c.ok;
}

static int gguf_open(const char* path, GgufFile** out) {
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return QMM_ERR_IO;
    struct stat st;
    if (fstat(fd, &st) != 0) {
        close(fd);
        return QMM_ERR_IO;
    }
    GgufFile* f = new GgufFile();
    f->fd = fd;
    f->file_size = (uint64_t)st.st_size;
    GgufCursor c{fd, 0, f->file_size};
    auto fail = [&](int code) {
        close(fd);
        delete f;
        return code;
    };
    if (c.get<uint32_t>() != GGUF_MAGIC || !c.ok) return fail(QMM_ERR_FORMAT);
    f->version = c.get<uint32_t>();
    if (f->version < 2 || f->version > 3) return fail(QMM_ERR_FORMAT);
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (!c.ok || n_tensors > (1u << 20) || n_kv > (1u << 20)) return fail(QMM_ERR_FORMAT);
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string key = c.str();
        const uint32_t vt = c.get<uint32_t>();
        GgufMeta m;
        if (!c.ok || !gguf_read_value(c, vt, m, 0)) return fail(QMM_ERR_FORMAT);
        f->meta[key] = m;
    }
    auto al = f->meta.find("general.alignment");
    if (al != f->meta.end() && al->second.u >= 8 && (al->second.u & (al->second.u - 1)) == 0) f->alignment = al->second.u;
    f->tensors.resize(n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        GgufTensor& t = f->tensors[i];
        t.name = c.str();
        t.n_dims = c.get<uint32_t>();
        if (!c.ok || t.n_dims < 1 || t.n_dims > 4) return fail(QMM_ERR_FORMAT);
        uint64_t elems = 1;
        for (uint32_t d = 0; d < t.n_dims; ++d) {
            t.dims[d] = c.get<uint64_t>();
            if (t.dims[d] == 0 || t.dims[d] > (1ull << 40)) return fail(QMM_ERR_FORMAT);
            elems *= t.dims[d];
        }
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) return fail(QMM_ERR_FORMAT);
        // rows are whole blocks: the row length decides, not the element count
        const uint64_t row = gguf_type_bytes(t.type, t.dims[0]);
        t.bytes = row ? row * (elems / t.dims[0]) : 0;  // 0: a type this library does not handle (listed, not readable)
        f->by_name[t.name] = (long)i;
    }
    f->data_start = (c.pos + f->alignment - 1) / f->alignment * f->alignment;
    for (const GgufTensor& t : f->tensors)
        if (t.bytes && (t.offset % f->alignment != 0 || f->data_start + t.offset + t.bytes > f->file_size)) return fail(QMM_ERR_FORMAT);
    *out = f;
    return QMM_OK;
}

static void gguf_close(GgufFile* f) {
    if (!f) return;
    if (f->bounce) cudaFreeHost(f->bounce);
    if (f->fd >= 0) close(f->fd);
    delete f;
}

static bool pread_all(int fd, void* dst, size_t n, uint64_t off) {
    size_t done = 0;
    while (done < n) {
        const ssize_t r = pread(fd, static_cast<char*>(dst) + done, n - done, (off_t)(off + done));
        if (r <= 0) return false;
        done += (size_t)r;
    }
    return true;
}

// Rows [row0, row0 + rows) and bytes [col_off, col_off + width) of every such row of a 2-D tensor, to device
// memory as a dense (rows, width) block: read in chunks of whole rows into the pinned bounce buffer, one
// strided copy per chunk.  (A row range of a column-parallel shard: col_off = 0, width = the row; a column
// range of a row-parallel shard: whole blocks out of every row.)
int gguf_upload_rows(GgufFile* f, long index, uint64_t row0, uint64_t rows, uint64_t col_off, uint64_t width, void* device_dst,
                     cudaStream_t stream) {
    if (index < 0 || index >= (long)f->tensors.size()) return QMM_ERR_SHAPE;
    const GgufTensor& t = f->tensors[index];
    if (!t.bytes) return QMM_ERR_TYPE;
    const uint64_t n_rows = t.bytes / gguf_type_bytes(t.type, t.dims[0]);
    const uint64_t row_bytes = t.bytes / n_rows;
    if (row0 + rows > n_rows || col_off + width > row_bytes || width == 0 || rows == 0) return QMM_ERR_SHAPE;
    if (!f->bounce) QMM_CUDA_TRY(cudaMallocHost(&f->bounce, GGUF_BOUNCE_BYTES));
    if (row_bytes > GGUF_BOUNCE_BYTES) return QMM_ERR_UNSUPPORTED;
    const uint64_t rows_per = GGUF_BOUNCE_BYTES / row_bytes;
    uint8_t* dst = static_cast<uint8_t*>(device_dst);
    for (uint64_t r = 0; r < rows; r += rows_per) {
        const uint64_t nr = rows - r < rows_per ? rows - r : rows_per;
        if (!pread_all(f->fd, f->bounce, nr * row_bytes, f->data_start + t.offset + (row0 + r) * row_bytes)) return QMM_ERR_IO;
        QMM_CUDA_TRY(cudaMemcpy2DAsync(dst + r * width, width, static_cast<uint8_t*>(f->bounce) + col_off, row_bytes, width, nr,
                                       cudaMemcpyHostToDevice, stream));
        QMM_CUDA_TRY(cudaStreamSynchronize(stream));  // the bounce buffer is reused by the next chunk
    }
    return QMM_OK;
}

// ---- writer -------------------------------------------------------------------------------------------
struct GgufWriter {
    std::string path;
    struct Kv {
        std::string key;
        uint32_t type;
        uint64_t u;
        float f;
        std::string s;
    };
    struct Pending {
        GgufTensor info;
        std::vector<uint8_t> data;
    };
    std::vector<Kv> kvs;
    std::vector<Pending> tensors;
    uint64_t alignment = 32;
};

static void put(std::vector<uint8_t>& b, const void* p, size_t n) {
    const uint8_t* s = static_cast<const uint8_t*>(p);
    b.insert(b.end(), s, s + n);
}
template <typename T>
static void put_v(std::vector<uint8_t>& b, T v) {
    put(b, &v, sizeof(T));
}
static void put_str(std::vector<uint8_t>& b, const std::string& s) {
    put_v<uint64_t>(b, s.size());
    put(b, s.data(), s.size());
}

static int gguf_writer_finish(GgufWriter* w) {
    std::vector<uint8_t> head;
    put_v<uint32_t>(head, GGUF_MAGIC);
    put_v<uint32_t>(head, 3);
    put_v<uint64_t>(head, w->tensors.size());
    put_v<uint64_t>(head, w->kvs.size() + 1);
    put_str(head, "general.alignment");
    put_v<uint32_t>(head, 4);
    put_v<uint32_t>(head, (uint32_t)w->alignment);
    for (const auto& kv : w->kvs) {
        put_str(head, kv.key);
        put_v<uint32_t>(head, kv.type);
        if (kv.type == 4) put_v<uint32_t>(head, (uint32_t)kv.u);
        else if (kv.type == 6) put_v<float>(head, kv.f);
        else if (kv.type == 10) put_v<uint64_t>(head, kv.u);
        else put_str(head, kv.s);
    }
    uint64_t off = 0;
    for (auto& t : w->tensors) {
        t.info.offset = off;
        off = (off + t.data.size() + w->alignment - 1) / w->alignment * w->alignment;
        put_str(head, t.info.name);
        put_v<uint32_t>(head, t.info.n_dims);
        for (uint32_t d = 0; d < t.info.n_dims; ++d) put_v<uint64_t>(head, t.info.dims[d]);
        put_v<uint32_t>(head, t.info.type);
        put_v<uint64_t>(head, t.info.offset);
    }
    FILE* fp = std::fopen(w->path.c_str(), "wb");
    if (!fp) return QMM_ERR_IO;
    bool ok = std::fwrite(head.data(), 1, head.size(), fp) == head.size();
    const std::vector<uint8_t> zeros(w->alignment, 0);
    uint64_t pos = head.size();
    auto pad = [&]() {
        const uint64_t want = (pos + w->alignment - 1) / w->alignment * w->alignment;
        if (want > pos) ok = ok && std::fwrite(zeros.data(), 1, want - pos, fp) == want - pos;
        pos = want;
    };
    pad();
    for (const auto& t : w->tensors) {
        ok = ok && std::fwrite(t.data.data(), 1, t.data.size(), fp) == t.data.size();
        pos += t.data.size();
        pad();
    }
    ok = std::fclose(fp) == 0 && ok;
    return ok ? QMM_OK : QMM_ERR_IO;
}

}  // namespace qmm

using namespace qmm;

extern "C" {

int qmm_gguf_open(const char* path, void** file) {
    if (!path || !file) return QMM_ERR_NULL;
    GgufFile* f = nullptr;
    if (int st = gguf_open(path, &f)) return st;
    *file = f;
    return QMM_OK;
}
int qmm_gguf_close(void* file) {
    if (!file) return QMM_ERR_NULL;
    gguf_close(static_cast<GgufFile*>(file));
    return QMM_OK;
}
long qmm_gguf_tensor_count(void* file) { return file ? (long)static_cast<GgufFile*>(file)->tensors.size() : QMM_ERR_NULL; }
long qmm_gguf_find(void* file, const char* name) {
    if (!file || !name) return QMM_ERR_NULL;
    GgufFile* f = static_cast<GgufFile*>(file);
    auto it = f->by_name.find(name);
    return it == f->by_name.end() ? -1 : it->second;
}
int qmm_gguf_tensor_info(void* file, long index, qmm_gguf_tensor* out) {
    if (!file || !out) return QMM_ERR_NULL;
    GgufFile* f = static_cast<GgufFile*>(file);
    if (index < 0 || index >= (long)f->tensors.size()) return QMM_ERR_SHAPE;
    const GgufTensor& t = f->tensors[index];
    std::memset(out, 0, sizeof(*out));
    std::strncpy(out->name, t.name.c_str(), sizeof(out->name) - 1);
    out->type = (int)t.type;
    out->n_dims = (int)t.n_dims;
    for (int d = 0; d < 4; ++d) out->dims[d] = (long)t.dims[d];
    out->file_offset = (long)(f->data_start + t.offset);
    out->bytes = (long)t.bytes;
    return QMM_OK;
}
int qmm_gguf_read_tensor(void* file, long index, void* host_dst, long capacity) {
    if (!file || !host_dst) return QMM_ERR_NULL;
    GgufFile* f = static_cast<GgufFile*>(file);
    if (index < 0 || index >= (long)f->tensors.size()) return QMM_ERR_SHAPE;
    const GgufTensor& t = f->tensors[index];
    if (!t.bytes) return QMM_ERR_TYPE;
    if ((long)t.bytes > capacity) return QMM_ERR_SHAPE;
    return pread_all(f->fd, host_dst, t.bytes, f->data_start + t.offset) ? QMM_OK : QMM_ERR_IO;
}
int qmm_gguf_upload_tensor(void* file, long index, void* device_dst, long capacity, void* stream) {
    if (!file || !device_dst) return QMM_ERR_NULL;
    GgufFile* f = static_cast<GgufFile*>(file);
    if (index < 0 || index >= (long)f->tensors.size()) return QMM_ERR_SHAPE;
    const GgufTensor& t = f->tensors[index];
    if (!t.bytes) return QMM_ERR_TYPE;
    if ((long)t.bytes > capacity) return QMM_ERR_SHAPE;
    const uint64_t row_bytes = gguf_type_bytes(t.type, t.dims[0]);
    return gguf_upload_rows(f, index, 0, t.bytes / row_bytes, 0, row_bytes, device_dst, as_stream(stream));
}
int qmm_gguf_meta_u64(void* file, const char* key, unsigned long long* out) {
    if (!file || !key || !out) return QMM_ERR_NULL;
    GgufFile* f = static_cast<GgufFile*>(file);
    auto it = f->meta.find(key);
    if (it == f->meta.end()) return QMM_ERR_SHAPE;
    const uint32_t t = it->second.type;
    if (t == 6 || t == 12 || t == 8 || t == 9) return QMM_ERR_TYPE;
    *out = it->second.u;
    return QMM_OK;
}
int qmm_gguf_meta_f64(void* file, const char* key, double* out) {
    if (!file || !key || !out) return QMM_ERR_NULL;
    GgufFile* f = static_cast<GgufFile*>(file);
    auto it = f->meta.find(key);
    if (it == f->meta.end()) return QMM_ERR_SHAPE;
    if (it->second.type != 6 && it->second.type != 12) return QMM_ERR_TYPE;
    *out = it->second.f;
    return QMM_OK;
}
long qmm_gguf_meta_str(void* file, const char* key, char* out, long capacity) {
    if (!file || !key) return QMM_ERR_NULL;
    GgufFile* f = static_cast<GgufFile*>(file);
    auto it = f->meta.find(key);
    if (it == f->meta.end()) return QMM_ERR_SHAPE;
    if (it->second.type != 8) return QMM_ERR_TYPE;
    const std::string& s = it->second.s;
    if (out && capacity > 0) {
        const size_t n = s.size() < (size_t)capacity - 1 ? s.size() : (size_t)capacity - 1;
        std::memcpy(out, s.data(), n);
        out[n] = '\0';
    }
    return (long)s.size();
}

int qmm_gguf_writer_create(const char* path, void** writer) {
    if (!path || !writer) return QMM_ERR_NULL;
    GgufWriter* w = new GgufWriter();
    w->path = path;
    *writer = w;
    return QMM_OK;
}
int qmm_gguf_writer_meta_u32(void* writer, const char* key, unsigned value) {
    if (!writer || !key) return QMM_ERR_NULL;
    static_cast<GgufWriter*>(writer)->kvs.push_back({key, 4, value, 0.f, {}});
    return QMM_OK;
}
int qmm_gguf_writer_meta_f32(void* writer, const char* key, float value) {
    if (!writer || !key) return QMM_ERR_NULL;
    static_cast<GgufWriter*>(writer)->kvs.push_back({key, 6, 0, value, {}});
    return QMM_OK;
}
int qmm_gguf_writer_meta_str(void* writer, const char* key, const char* value) {
    if (!writer || !key || !value) return QMM_ERR_NULL;
    static_cast<GgufWriter*>(writer)->kvs.push_back({key, 8, 0, 0.f, value});
    return QMM_OK;
}
int qmm_gguf_writer_add_tensor(void* writer, const char* name, int type, int n_dims, const long* dims, const void* host_data, long bytes) {
    if (!writer || !name || !dims || !host_data) return QMM_ERR_NULL;
    if (n_dims < 1 || n_dims > 4 || bytes <= 0) return QMM_ERR_SHAPE;
    GgufWriter::Pending p;
    p.info.name = name;
    p.info.n_dims = (uint32_t)n_dims;
    uint64_t elems = 1;
    for (int d = 0; d < n_dims; ++d) {
        if (dims[d] <= 0) return QMM_ERR_SHAPE;
        p.info.dims[d] = (uint64_t)dims[d];
        elems *= (uint64_t)dims[d];
    }
    p.info.type = (uint32_t)type;
    const uint64_t row = gguf_type_bytes((uint32_t)type, p.info.dims[0]);
    if (!row) return QMM_ERR_TYPE;
    if (row * (elems / p.info.dims[0]) != (uint64_t)bytes) return QMM_ERR_SHAPE;
    p.data.assign(static_cast<const uint8_t*>(host_data), static_cast<const uint8_t*>(host_data) + bytes);
    static_cast<GgufWriter*>(writer)->tensors.push_back(std::move(p));
    return QMM_OK;
}
int qmm_gguf_writer_finish(void* writer) {
    if (!writer) return QMM_ERR_NULL;
    GgufWriter* w = static_cast<GgufWriter*>(writer);
    const int st = gguf_writer_finish(w);
    delete w;
    return st;
}

}  // extern "C"
