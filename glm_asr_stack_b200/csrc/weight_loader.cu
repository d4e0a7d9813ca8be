// safetensors -> device weight store (reference: safetensors_load / safetensors_free,
// Infer-engine/src/safetensors.c:57-193; header Infer-engine/include/safetensors.h).
//
// Same result as the reference loader -- every tensor of the file whose dtype the engine knows
// (BF16, F32, F16, U8, F8_E4M3) becomes one WeightStore entry, in header order, with its name, dtype
// tag, shape (at most 4 dims) and byte count, at most 2048 of them; "__metadata__" and tensors of other
// dtypes are skipped -- but built for a 1361-tensor, multi-gigabyte checkpoint that eight replicas load
// at start-up:
//   * ONE device allocation per file: tensors sit at 256-byte aligned offsets of an arena (the
//     reference calls cudaMalloc once per tensor, which gives the same 256-byte alignment the TMA
//     descriptors of the GEMMs rely on);
//   * the file is read straight into two pinned staging buffers, already in arena layout, by a few
//     reader threads, and leaves them as 64 MiB host-to-device copies that overlap the next window's
//     reads (the reference does malloc + fread + synchronous cudaMemcpy + free per tensor);
//   * nothing is parsed twice: glmasr_safetensors_inspect() exposes the header pass on its own (no CUDA
//     call), which is also what the CPU tests exercise.
// safetensors_free releases the arena and the names, and makes the library forget what it cached about
// these weights (re-tiled scales, the decoder's pointer table).
#include <cuda_runtime.h>
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../../include/glmasr_engine_types.h"
#include "../../include/glmasr_fp4.h"

namespace {

constexpr size_t kAlign = 256;                 // arena alignment of every tensor (what cudaMalloc would give)
constexpr size_t kWindow = 64ull << 20;        // bytes per staging buffer / host-to-device copy
constexpr int kReaders = 4;                    // reader threads per window

struct Entry {
    std::string name;
    int dtype = -1;
    int ndim = 0;
    int64_t shape[GLMASR_MAX_DIMS] = {0, 0, 0, 0};
    uint64_t file_off = 0;                     // offset of the tensor's bytes in the file
    size_t nbytes = 0;                         // as the reference computes it (0 stays 0)
    size_t copy_bytes = 0;                     // bytes actually read (the reference reads 4 for an empty tensor)
    size_t arena_off = 0;
};

// ---- the small JSON subset a safetensors header uses -------------------------------------------------
struct Cursor {
    const char *p, *end;
    void ws() { while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p; }
    bool at(char c) { ws(); return p < end && *p == c; }
    bool take(char c) { if (at(c)) { ++p; return true; } return false; }
};

static bool parse_string(Cursor &c, std::string *out) {
    if (!c.take('"')) return false;
    out->clear();
    while (c.p < c.end && *c.p != '"') {
        if (*c.p == '\\' && c.p + 1 < c.end) ++c.p;          // the reference keeps the escaped character as is
        out->push_back(*c.p++);
    }
    if (c.p < c.end) ++c.p;
    return true;
}

static int64_t parse_int(Cursor &c) {
    c.ws();
    bool neg = false;
    if (c.p < c.end && *c.p == '-') neg = true, ++c.p;
    int64_t v = 0;
    while (c.p < c.end && *c.p >= '0' && *c.p <= '9') v = v * 10 + (*c.p++ - '0');
    return neg ? -v : v;
}

static void skip_value(Cursor &c) {
    c.ws();
    if (c.p >= c.end) return;
    if (*c.p == '"') {
        std::string s;
        parse_string(c, &s);
    } else if (*c.p == '{' || *c.p == '[') {
        const char open = *c.p, close = open == '{' ? '}' : ']';
        int depth = 0;
        bool in_str = false;
        for (; c.p < c.end; ++c.p) {
            if (in_str) {
                if (*c.p == '\\') ++c.p;
                else if (*c.p == '"') in_str = false;
            } else if (*c.p == '"') in_str = true;
            else if (*c.p == open) ++depth;
            else if (*c.p == close && --depth == 0) { ++c.p; break; }
        }
    } else {
        while (c.p < c.end && *c.p != ',' && *c.p != '}' && *c.p != ']') ++c.p;
    }
}

static int dtype_tag(const std::string &s) {       // Infer-engine/src/safetensors.c:48-55
    if (s == "BF16") return GLMASR_DTYPE_BF16;
    if (s == "F32") return GLMASR_DTYPE_FP32;
    if (s == "F16") return GLMASR_DTYPE_FP16;
    if (s == "U8") return GLMASR_DTYPE_UINT8;
    if (s == "F8_E4M3") return GLMASR_DTYPE_FP8;
    return -1;
}

static size_t dtype_bytes(int tag) {                // Infer-engine/include/types.h:14-23
    switch (tag) {
        case GLMASR_DTYPE_FP32: return 4;
        case GLMASR_DTYPE_BF16: case GLMASR_DTYPE_FP16: return 2;
        case GLMASR_DTYPE_UINT8: case GLMASR_DTYPE_FP8: return 1;
        default: return 0;
    }
}

// Header pass: entries in header order with their arena layout.  Returns false with a message on stderr.
static bool read_index(const char *path, std::vector<Entry> *out, size_t *arena_bytes, uint64_t *file_size, int *fd_out) {
    const int fd = open(path, O_RDONLY);
    if (fd < 0) {
        fprintf(stderr, "Cannot open %s\n", path);           // the reference's message (safetensors.c:59)
        return false;
    }
    struct stat sb;
    uint64_t header_size = 0;
    if (fstat(fd, &sb) != 0 || pread(fd, &header_size, 8, 0) != 8 || header_size > (uint64_t)sb.st_size - 8) {
        fprintf(stderr, "%s: not a safetensors file (bad header length)\n", path);
        close(fd);
        return false;
    }
    std::string json(header_size, '\0');
    for (size_t got = 0; got < header_size;) {
        const ssize_t n = pread(fd, &json[got], header_size - got, 8 + got);
        if (n <= 0) {
            fprintf(stderr, "%s: short read of the header\n", path);
            close(fd);
            return false;
        }
        got += (size_t)n;
    }
    const uint64_t data_start = 8 + header_size;
    Cursor c{json.data(), json.data() + json.size()};
    c.take('{');
    size_t cursor = 0;
    while (c.p < c.end && !c.at('}') && (int)out->size() < GLMASR_MAX_WEIGHTS) {
        c.take(',');
        if (c.at('}') || c.p >= c.end) break;
        std::string key;
        if (!parse_string(c, &key)) break;
        c.take(':');
        if (key == "__metadata__" || !c.at('{')) {
            skip_value(c);
            continue;
        }
        c.take('{');
        Entry e;
        e.name = key;
        std::string dtype;
        int64_t off0 = 0, off1 = 0;
        while (c.p < c.end && !c.at('}')) {
            c.take(',');
            if (c.at('}')) break;
            std::string field;
            if (!parse_string(c, &field)) break;
            c.take(':');
            if (field == "dtype") {
                parse_string(c, &dtype);
            } else if (field == "shape" && c.take('[')) {
                while (!c.at(']') && c.p < c.end) {
                    const int64_t d = parse_int(c);
                    if (e.ndim < GLMASR_MAX_DIMS) e.shape[e.ndim++] = (int)d;     // the reference keeps 4 dims of int
                    else break;
                    c.take(',');
                }
                // dims beyond the fourth are dropped (the reference's parser loses its place in the header there;
                // no tensor of the checkpoint has more than four)
                while (c.p < c.end && !c.at(']')) ++c.p;
                c.take(']');
            } else if (field == "data_offsets" && c.take('[')) {
                off0 = parse_int(c);
                c.take(',');
                off1 = parse_int(c);
                c.take(']');
            } else {
                skip_value(c);
            }
        }
        c.take('}');
        e.dtype = dtype_tag(dtype);
        if (e.dtype < 0) continue;                            // unknown dtype: no entry (safetensors.c:141)
        e.nbytes = (size_t)(off1 - off0);
        if (e.nbytes == 0 && e.ndim == 0) e.nbytes = dtype_bytes(e.dtype);      // safetensors.c:143-146
        e.copy_bytes = e.nbytes > 0 ? e.nbytes : 4;           // the reference allocates and reads 4 bytes for nothing
        e.file_off = data_start + (uint64_t)off0;
        if (off1 < off0 || e.file_off > (uint64_t)sb.st_size) {
            fprintf(stderr, "%s: tensor %s lies outside the file\n", path, key.c_str());
            close(fd);
            return false;
        }
        // bytes past the end of the file (only possible for the 4-byte read of an empty tensor) are not read
        if (e.file_off + e.copy_bytes > (uint64_t)sb.st_size) e.copy_bytes = (size_t)((uint64_t)sb.st_size - e.file_off);
        e.arena_off = cursor;
        cursor += ((e.copy_bytes > 4 ? e.copy_bytes : 4) + kAlign - 1) / kAlign * kAlign;
        out->push_back(std::move(e));
    }
    *arena_bytes = cursor;
    *file_size = (uint64_t)sb.st_size;
    if (fd_out != nullptr) *fd_out = fd;
    else close(fd);
    return true;
}

static void fill_store(glmasr_WeightStore *ws, const std::vector<Entry> &idx, uint8_t *arena) {
    ws->count = 0;
    for (const Entry &e : idx) {
        const int i = ws->count++;
        ws->names[i] = strdup(e.name.c_str());
        glmasr_Tensor &t = ws->tensors[i];
        t.data = arena + e.arena_off;
        t.dtype = e.dtype;
        t.ndim = e.ndim;
        for (int d = 0; d < GLMASR_MAX_DIMS; ++d) t.shape[d] = d < e.ndim ? e.shape[d] : 0;
        t.nbytes = e.nbytes;
    }
}

// arenas by the store that points into them
static std::unordered_map<const glmasr_WeightStore *, void *> g_arenas;

static bool pread_all(int fd, uint8_t *dst, size_t n, uint64_t off) {
    while (n > 0) {
        const ssize_t r = pread(fd, dst, n, (off_t)off);
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) return false;
        dst += r, n -= (size_t)r, off += (uint64_t)r;
    }
    return true;
}

struct Piece {
    size_t stage_off;      // where in the staging window
    uint64_t file_off;
    size_t bytes;
};

}  // namespace

// Header pass only: fills names, dtype tags, shapes and byte counts exactly as safetensors_load would and
// stores every tensor's OFFSET inside the arena in `data` (no device memory is touched, no CUDA call is
// made); *arena_bytes = size of the one allocation safetensors_load makes.  Names are malloc'd: release them
// with glmasr_safetensors_release_index.  Returns 0, or -1 like safetensors_load.
extern "C" int glmasr_safetensors_inspect(const char *path, void *ws_v, size_t *arena_bytes) {
    glmasr_WeightStore *ws = (glmasr_WeightStore *)ws_v;
    if (path == nullptr || ws == nullptr) return -1;
    std::vector<Entry> idx;
    size_t arena = 0;
    uint64_t fsize = 0;
    ws->count = 0;
    if (!read_index(path, &idx, &arena, &fsize, nullptr)) return -1;
    fill_store(ws, idx, nullptr);
    if (arena_bytes != nullptr) *arena_bytes = arena;
    return 0;
}

extern "C" void glmasr_safetensors_release_index(void *ws_v) {
    glmasr_WeightStore *ws = (glmasr_WeightStore *)ws_v;
    if (ws == nullptr) return;
    for (int i = 0; i < ws->count; ++i) {
        free(ws->names[i]);
        ws->names[i] = nullptr;
    }
    ws->count = 0;
}

// Infer-engine/include/safetensors.h:6, Infer-engine/src/safetensors.c:57-181.
extern "C" int safetensors_load(const char *path, void *ws_v) {
    glmasr_WeightStore *ws = (glmasr_WeightStore *)ws_v;
    if (path == nullptr || ws == nullptr) return -1;
    std::vector<Entry> idx;
    size_t arena_bytes = 0;
    uint64_t fsize = 0;
    int fd = -1;
    ws->count = 0;
    if (!read_index(path, &idx, &arena_bytes, &fsize, &fd)) return -1;

    uint8_t *arena = nullptr;
    uint8_t *stage[2] = {nullptr, nullptr};
    cudaStream_t copy = nullptr;
    cudaEvent_t done[2] = {nullptr, nullptr};
    bool ok = true;
    auto fail = [&](const char *what, cudaError_t e) {
        fprintf(stderr, "safetensors_load(%s): %s%s%s\n", path, what, e != cudaSuccess ? ": " : "",
                e != cudaSuccess ? cudaGetErrorString(e) : "");
        ok = false;
    };
    cudaError_t e = cudaMalloc(&arena, arena_bytes > 0 ? arena_bytes : kAlign);
    if (e != cudaSuccess) fail("cudaMalloc of the weight arena failed", e);
    const size_t window = arena_bytes < kWindow ? (arena_bytes > 0 ? arena_bytes : kAlign) : kWindow;
    for (int b = 0; b < 2 && ok; ++b) {
        if ((e = cudaHostAlloc(&stage[b], window, cudaHostAllocDefault)) != cudaSuccess) fail("pinned staging buffer", e);
        else if ((e = cudaEventCreateWithFlags(&done[b], cudaEventDisableTiming)) != cudaSuccess) fail("event", e);
    }
    if (ok && (e = cudaStreamCreateWithFlags(&copy, cudaStreamNonBlocking)) != cudaSuccess) fail("stream", e);

    // windows of the arena; a tensor larger than a window, or one that straddles a boundary, is read in pieces
    size_t next = 0;           // index of the first tensor that may reach into the current window
    int buf = 0;
    for (size_t w0 = 0; ok && w0 < arena_bytes; w0 += window, buf ^= 1) {
        const size_t w1 = w0 + window < arena_bytes ? w0 + window : arena_bytes;
        std::vector<Piece> pieces;
        while (next < idx.size() && idx[next].arena_off + idx[next].copy_bytes <= w0) ++next;
        for (size_t i = next; i < idx.size() && idx[i].arena_off < w1; ++i) {
            const Entry &t = idx[i];
            const size_t a0 = t.arena_off > w0 ? t.arena_off : w0;
            const size_t a1 = t.arena_off + t.copy_bytes < w1 ? t.arena_off + t.copy_bytes : w1;
            if (a1 > a0) pieces.push_back({a0 - w0, t.file_off + (a0 - t.arena_off), a1 - a0});
        }
        // the staging buffer is free once the copy that last used it has finished
        if ((e = cudaEventSynchronize(done[buf])) != cudaSuccess) { fail("waiting for a staging buffer", e); break; }
        // spread the window's bytes over the reader threads (large pieces are cut, so that one 243 MB
        // embedding table does not serialise on one thread)
        std::vector<Piece> cut;
        const size_t grain = 4ull << 20;
        for (const Piece &p : pieces)
            for (size_t o = 0; o < p.bytes; o += grain)
                cut.push_back({p.stage_off + o, p.file_off + o, p.bytes - o < grain ? p.bytes - o : grain});
        bool read_ok[kReaders];
        std::vector<std::thread> readers;
        for (int r = 0; r < kReaders; ++r) {
            read_ok[r] = true;
            readers.emplace_back([&, r]() {
                for (size_t i = (size_t)r; i < cut.size(); i += kReaders)
                    if (!pread_all(fd, stage[buf] + cut[i].stage_off, cut[i].bytes, cut[i].file_off)) read_ok[r] = false;
            });
        }
        for (auto &t : readers) t.join();
        for (int r = 0; r < kReaders; ++r)
            if (!read_ok[r]) fail("short read of tensor data", cudaSuccess);
        if (!ok) break;
        if ((e = cudaMemcpyAsync(arena + w0, stage[buf], w1 - w0, cudaMemcpyHostToDevice, copy)) != cudaSuccess) fail("host-to-device copy", e);
        else if ((e = cudaEventRecord(done[buf], copy)) != cudaSuccess) fail("event record", e);
    }
    if (ok && copy != nullptr && (e = cudaStreamSynchronize(copy)) != cudaSuccess) fail("host-to-device copies", e);

    close(fd);
    for (int b = 0; b < 2; ++b) {
        if (stage[b]) cudaFreeHost(stage[b]);
        if (done[b]) cudaEventDestroy(done[b]);
    }
    if (copy) cudaStreamDestroy(copy);
    if (!ok) {
        if (arena) cudaFree(arena);
        return -1;
    }
    fill_store(ws, idx, arena);
    g_arenas[ws] = arena;
    return 0;
}

// Infer-engine/include/safetensors.h:7, Infer-engine/src/safetensors.c:183-193.  Stores that safetensors_load
// did not fill (tensors allocated one by one by someone else) are released tensor by tensor as the reference does.
extern "C" void safetensors_free(void *ws_v) {
    glmasr_WeightStore *ws = (glmasr_WeightStore *)ws_v;
    if (ws == nullptr) return;
    glmasr_decoder_forget_weights();
    for (int i = 0; i < ws->count; ++i)
        if (ws->tensors[i].dtype == GLMASR_DTYPE_FP8 && ws->tensors[i].data != nullptr) glmasr_fp4_forget(ws->tensors[i].data);
    auto it = g_arenas.find(ws);
    if (it != g_arenas.end()) {
        cudaDeviceSynchronize();
        cudaFree(it->second);
        g_arenas.erase(it);
    } else {
        for (int i = 0; i < ws->count; ++i)
            if (ws->tensors[i].data) cudaFree(ws->tensors[i].data);
    }
    for (int i = 0; i < ws->count; ++i) {
        if (ws->names[i]) free(ws->names[i]);
        ws->names[i] = nullptr;
        ws->tensors[i].data = nullptr;
    }
    ws->count = 0;
}
