// Reader of safetensors files: host code (no kernels), part of the library so that weights go from the
// file to the device without passing through Python objects.
//
// Format: an 8-byte little-endian header length, a JSON header that maps each tensor name to
// {"dtype", "shape", "data_offsets": [begin, end]} (offsets relative to the end of the header; the key
// "__metadata__" holds string pairs), then the raw little-endian data.  rb_st_open reads and checks the
// header (every tensor's span against its shape and type and against the file's size) and keeps the file
// open; rb_st_read copies one tensor's bytes to host memory, or to device memory through two pinned
// staging buffers: while one is on its way to the device the next piece of the file is read into the other.
//
// It stands where the reference has its GGUF reader (rocml-core/src/gguf/mod.rs:47-236: open, look a
// tensor up by name, know its shape and type, typed errors for truncated or malformed files).
#include <cuda_runtime.h>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <utility>
#include <vector>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>
#include "common.cuh"
#include "api.h"

namespace {

constexpr long long MAX_HEADER = 100ll * 1024 * 1024;
constexpr size_t STAGE_BYTES = 64u << 20;
constexpr size_t READ_THREADS = 8;

struct Entry {
    std::string name, dtype;
    std::vector<long long> shape;
    long long begin = 0, end = 0;
};

struct File {
    int fd = -1;
    long long size = 0, base = 0;
    std::string path;
    std::vector<Entry> entries;
    std::vector<std::pair<std::string, std::string>> metadata;
};

// The pinned staging buffers: made at the first copy to a device and kept for the life of the process (pinning
// 128 MB costs as much as copying a gigabyte), shared by all open files under a lock.
struct Staging {
    std::mutex lock;
    void* pinned[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    bool in_flight[2] = {false, false};
    int next = 0;
};
Staging g_staging;

int element_size(const std::string& d) {
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
    return 0;
}

// ---- a JSON reader for headers: objects, arrays, strings, integers; other values are skipped --------
struct Json {
    const char* p;
    const char* end;
    std::string err;

    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool fail(const char* what) {
        if (err.empty()) err = std::string(what) + " at byte " + std::to_string((long long)(p - start));
        return false;
    }
    const char* start;
    bool eat(char c) {
        ws();
        if (p < end && *p == c) { ++p; return true; }
        return false;
    }
    static void utf8(std::string& out, unsigned cp) {
        if (cp < 0x80) out += (char)cp;
        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) {
            out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F));
        } else {
            out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F));
            out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F));
        }
    }
    bool hex4(unsigned& v) {
        if (end - p < 4) return fail("short \\u escape");
        v = 0;
        for (int i = 0; i < 4; ++i, ++p) {
            const char c = *p;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (unsigned)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (unsigned)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (unsigned)(c - 'A' + 10);
            else return fail("bad \\u escape");
        }
        return true;
    }
    bool string(std::string& out) {
        ws();
        if (p >= end || *p != '"') return fail("expected a string");
        ++p;
        out.clear();
        while (p < end && *p != '"') {
            if ((unsigned char)*p < 0x20) return fail("control character in a string");
            if (*p != '\\') { out += *p++; continue; }
            if (++p >= end) return fail("unterminated escape");
            const char c = *p++;
            switch (c) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    unsigned cp = 0;
                    if (!hex4(cp)) return false;
                    if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                        p += 2;
                        unsigned lo = 0;
                        if (!hex4(lo)) return false;
                        if (lo >= 0xDC00 && lo < 0xE000) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        else return fail("unpaired surrogate");
                    }
                    utf8(out, cp);
                    break;
                }
                default: return fail("unknown escape");
            }
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }
    bool integer(long long& v) {
        ws();
        const char* s = p;
        bool neg = false;
        if (p < end && *p == '-') { neg = true; ++p; }
        if (p >= end || *p < '0' || *p > '9') { p = s; return fail("expected an integer"); }
        unsigned long long u = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            if (u > (0x7FFFFFFFFFFFFFFFull - 9) / 10) return fail("integer too large");
            u = u * 10 + (unsigned)(*p++ - '0');
        }
        if (p < end && (*p == '.' || *p == 'e' || *p == 'E')) return fail("expected an integer, found a fraction");
        v = neg ? -(long long)u : (long long)u;
        return true;
    }
    bool skip() {   // any value
        ws();
        if (p >= end) return fail("unexpected end");
        if (*p == '"') { std::string s; return string(s); }
        if (*p == '{') {
            ++p;
            if (eat('}')) return true;
            do {
                std::string k;
                if (!string(k) || !eat(':')) return fail("expected ':'");
                if (!skip()) return false;
            } while (eat(','));
            return eat('}') || fail("expected '}'");
        }
        if (*p == '[') {
            ++p;
            if (eat(']')) return true;
            do { if (!skip()) return false; } while (eat(','));
            return eat(']') || fail("expected ']'");
        }
        const char* s = p;
        while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n' && *p != '\t' && *p != '\r') ++p;
        return p > s || fail("expected a value");
    }
};

bool parse_entry(Json& j, Entry& e) {
    if (!j.eat('{')) return j.fail("tensor entry is not an object");
    bool have_dtype = false, have_shape = false, have_off = false;
    if (!j.eat('}')) {
        do {
            std::string k;
            if (!j.string(k) || !j.eat(':')) return j.fail("expected ':'");
            if (k == "dtype") {
                if (!j.string(e.dtype)) return false;
                have_dtype = true;
            } else if (k == "shape") {
                if (!j.eat('[')) return j.fail("shape is not an array");
                e.shape.clear();
                if (!j.eat(']')) {
                    do {
                        long long v;
                        if (!j.integer(v)) return false;
                        if (v < 0) return j.fail("negative extent");
                        e.shape.push_back(v);
                    } while (j.eat(','));
                    if (!j.eat(']')) return j.fail("expected ']'");
                }
                have_shape = true;
            } else if (k == "data_offsets") {
                if (!j.eat('[') || !j.integer(e.begin) || !j.eat(',') || !j.integer(e.end) || !j.eat(']'))
                    return j.fail("data_offsets is not [begin, end]");
                have_off = true;
            } else if (!j.skip()) {
                return false;
            }
        } while (j.eat(','));
        if (!j.eat('}')) return j.fail("expected '}'");
    }
    if (!have_dtype || !have_shape || !have_off) return j.fail("tensor entry lacks dtype, shape or data_offsets");
    return true;
}

void say(char* err, int err_len, const std::string& msg) {
    if (err != nullptr && err_len > 0) {
        std::snprintf(err, (size_t)err_len, "%s", msg.c_str());
    }
}

bool read_exact(int fd, void* dst, size_t n, long long off) {
    uint8_t* d = static_cast<uint8_t*>(dst);
    while (n > 0) {
        const ssize_t r = pread(fd, d, n, (off_t)off);
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) return false;
        d += r; n -= (size_t)r; off += r;
    }
    return true;
}

// The same with several threads, each reading its own part: one thread copies out of the page cache at a
// fraction of what the link to the device takes.
bool read_parallel(int fd, void* dst, size_t n, long long off) {
    constexpr size_t MIN_PART = 4u << 20;
    unsigned hw = std::thread::hardware_concurrency();
    size_t parts = n / MIN_PART;
    if (parts > READ_THREADS) parts = READ_THREADS;
    if (hw > 0 && parts > hw) parts = hw;
    if (parts < 2) return read_exact(fd, dst, n, off);
    const size_t each = (n / parts + 4095) & ~(size_t)4095;
    std::vector<std::thread> workers;
    std::vector<char> ok(parts, 1);
    for (size_t k = 1; k < parts; ++k) {
        const size_t lo = k * each, hi = (k + 1 == parts || (k + 1) * each > n) ? n : (k + 1) * each;
        if (lo >= n) { parts = k; break; }
        workers.emplace_back([=, &ok] { ok[k] = read_exact(fd, static_cast<uint8_t*>(dst) + lo, hi - lo, off + (long long)lo) ? 1 : 0; });
    }
    ok[0] = read_exact(fd, dst, each < n ? each : n, off) ? 1 : 0;
    for (auto& w : workers) w.join();
    for (size_t k = 0; k < ok.size(); ++k)
        if (!ok[k]) return false;
    return true;
}

void release(File* f) {
    if (f->fd >= 0) close(f->fd);
    delete f;
}

}  // namespace

// Opens `path` and checks its header.  Returns a handle, or null with the reason in err (at most err_len bytes).
extern "C" void* rb_st_open(const char* path, char* err, int err_len) {
    File* f = new File();
    f->path = path;
    f->fd = open(path, O_RDONLY | O_CLOEXEC);
    if (f->fd < 0) {
        say(err, err_len, std::string(path) + ": cannot open: " + std::strerror(errno));
        release(f);
        return nullptr;
    }
    struct stat st;
    if (fstat(f->fd, &st) != 0 || st.st_size < 8) {
        say(err, err_len, std::string(path) + ": too short for a header");
        release(f);
        return nullptr;
    }
    f->size = (long long)st.st_size;
    uint8_t len8[8];
    if (!read_exact(f->fd, len8, 8, 0)) {
        say(err, err_len, std::string(path) + ": cannot read the header length");
        release(f);
        return nullptr;
    }
    unsigned long long hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | len8[i];
    if (hlen > (unsigned long long)MAX_HEADER || 8 + (long long)hlen > f->size) {
        say(err, err_len, std::string(path) + ": header length " + std::to_string(hlen) + " does not fit the file of " +
                              std::to_string(f->size) + " bytes (truncated?)");
        release(f);
        return nullptr;
    }
    std::string header((size_t)hlen, '\0');
    if (hlen > 0 && !read_exact(f->fd, &header[0], (size_t)hlen, 8)) {
        say(err, err_len, std::string(path) + ": cannot read the header");
        release(f);
        return nullptr;
    }
    f->base = 8 + (long long)hlen;
    const long long data_size = f->size - f->base;
    Json j{header.data(), header.data() + header.size(), std::string(), header.data()};
    bool ok = j.eat('{');
    if (!ok) j.fail("header is not a JSON object");
    if (ok && !j.eat('}')) {
        do {
            std::string name;
            if (!j.string(name) || !j.eat(':')) { ok = j.fail("expected ':'"); break; }
            if (name == "__metadata__") {
                j.ws();
                if (j.p < j.end && *j.p == '{') {
                    ++j.p;
                    if (!j.eat('}')) {
                        do {
                            std::string k, v;
                            if (!j.string(k) || !j.eat(':')) { ok = j.fail("expected ':'"); break; }
                            j.ws();
                            if (j.p < j.end && *j.p == '"') {
                                if (!j.string(v)) { ok = false; break; }
                                f->metadata.emplace_back(k, v);
                            } else if (!j.skip()) { ok = false; break; }
                        } while (j.eat(','));
                        if (ok && !j.eat('}')) ok = j.fail("expected '}'");
                    }
                } else if (!j.skip()) {
                    ok = false;
                }
                if (!ok) break;
                continue;
            }
            Entry e;
            e.name = name;
            if (!parse_entry(j, e)) { ok = false; break; }
            const int esz = element_size(e.dtype);
            if (esz == 0) {
                say(err, err_len, f->path + ": tensor '" + name + "' has the unknown element type '" + e.dtype + "'");
                release(f);
                return nullptr;
            }
            unsigned long long n = 1;
            bool overflow = false;
            for (long long s : e.shape) {
                if (s != 0 && n > 0xFFFFFFFFFFFFull / (unsigned long long)s) overflow = true;
                n *= (unsigned long long)s;
            }
            const long long want = (long long)n * esz;
            if (overflow || e.begin < 0 || e.end - e.begin != want || e.end > data_size) {
                say(err, err_len, f->path + ": tensor '" + name + "' spans bytes [" + std::to_string(e.begin) + ", " +
                                      std::to_string(e.end) + ") but its shape needs " + std::to_string(want) +
                                      " and the data section holds " + std::to_string(data_size) + " (truncated?)");
                release(f);
                return nullptr;
            }
            f->entries.push_back(std::move(e));
        } while (j.eat(','));
        if (ok && !j.eat('}')) ok = j.fail("expected '}'");
    }
    if (ok) {
        j.ws();
        if (j.p != j.end) ok = j.fail("text after the header object");
    }
    if (!ok) {
        say(err, err_len, f->path + ": header is not valid: " + j.err);
        release(f);
        return nullptr;
    }
    return f;
}

extern "C" int rb_st_count(const void* handle) { return (int)static_cast<const File*>(handle)->entries.size(); }

// Tensor i: its name and element type (strings owned by the handle), rank, extents (at most 8) and bytes.
extern "C" int rb_st_entry(const void* handle, int i, const char** name, const char** dtype, int* rank,
                           long long* shape, long long* nbytes) {
    const File* f = static_cast<const File*>(handle);
    if (i < 0 || i >= (int)f->entries.size()) return RB_ERR_BAD_SIZE;
    const Entry& e = f->entries[(size_t)i];
    if (e.shape.size() > 8) return RB_ERR_BAD_SIZE;
    *name = e.name.c_str();
    *dtype = e.dtype.c_str();
    *rank = (int)e.shape.size();
    for (size_t d = 0; d < e.shape.size(); ++d) shape[d] = e.shape[d];
    *nbytes = e.end - e.begin;
    return RB_OK;
}

extern "C" int rb_st_metadata_count(const void* handle) { return (int)static_cast<const File*>(handle)->metadata.size(); }
extern "C" int rb_st_metadata(const void* handle, int i, const char** key, const char** value) {
    const File* f = static_cast<const File*>(handle);
    if (i < 0 || i >= (int)f->metadata.size()) return RB_ERR_BAD_SIZE;
    *key = f->metadata[(size_t)i].first.c_str();
    *value = f->metadata[(size_t)i].second.c_str();
    return RB_OK;
}

// Copies tensor i's bytes to dst (dst_bytes must equal the tensor's size).  on_device = 0: dst is host memory,
// the copy is done when the call returns.  on_device = 1: dst is device memory; the bytes travel through
// pinned buffers on `stream`, and the last pieces may still be on their way when the call returns (work
// enqueued later on the same stream sees them).  RB_ERR_BAD_SIZE for a wrong
// size or index, RB_ERR_IO when the file cannot be read, else a cudaError_t value.
extern "C" int rb_st_read(void* handle, int i, void* dst, long long dst_bytes, int on_device, void* stream) {
    File* f = static_cast<File*>(handle);
    if (i < 0 || i >= (int)f->entries.size()) return RB_ERR_BAD_SIZE;
    const Entry& e = f->entries[(size_t)i];
    const long long n = e.end - e.begin;
    if (dst_bytes != n) return RB_ERR_BAD_SIZE;
    if (n == 0) return RB_OK;
    const long long off = f->base + e.begin;
    if (!on_device) return read_exact(f->fd, dst, (size_t)n, off) ? RB_OK : RB_ERR_IO;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t ce;
    Staging& g = g_staging;
    std::lock_guard<std::mutex> hold(g.lock);
    for (int b = 0; b < 2; ++b) {
        if (g.pinned[b] == nullptr) {
            if ((ce = cudaHostAlloc(&g.pinned[b], STAGE_BYTES, cudaHostAllocDefault)) != cudaSuccess) return (int)ce;
            if ((ce = cudaEventCreateWithFlags(&g.done[b], cudaEventDisableTiming)) != cudaSuccess) return (int)ce;
        }
    }
    for (long long at = 0; at < n; at += (long long)STAGE_BYTES) {
        const size_t piece = (size_t)((n - at) < (long long)STAGE_BYTES ? (n - at) : (long long)STAGE_BYTES);
        const int b = g.next;
        g.next ^= 1;
        if (g.in_flight[b]) {       // the copy that last used this buffer has to be off it
            if ((ce = cudaEventSynchronize(g.done[b])) != cudaSuccess) return (int)ce;
            g.in_flight[b] = false;
        }
        if (!read_parallel(f->fd, g.pinned[b], piece, off + at)) return RB_ERR_IO;
        if ((ce = cudaMemcpyAsync(static_cast<uint8_t*>(dst) + at, g.pinned[b], piece, cudaMemcpyHostToDevice, s)) != cudaSuccess)
            return (int)ce;
        if ((ce = cudaEventRecord(g.done[b], s)) != cudaSuccess) return (int)ce;
        g.in_flight[b] = true;
    }
    return RB_OK;
}

// Closes the file.  Copies to a device that are still on their way are not waited for: they read the
// staging buffers, not the file, and work enqueued later on their stream sees them.
extern "C" void rb_st_close(void* handle) {
    if (handle != nullptr) release(static_cast<File*>(handle));
}
