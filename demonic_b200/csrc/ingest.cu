// ingest.cu -- weights from a .npz archive straight into HBM.
//
// The reference's `vault.load_npz[bf16, [K, N]](path, key = "w")` opens the archive, finds the entry
// `<key>.npy` (or `<key>`), skips the NPY v1/v2 header and copies `numel * elem_bytes` raw
// little-endian bytes into a fresh host buffer (compiler/src/jit.rs:29836-29927); the GPU backend
// then uploads that buffer at the first matmul.  Here the bytes go from the file through a small
// ring of pinned buffers (filled by a few reader threads) directly to the device (and, if the caller
// wants the host copy the JIT expects, into its buffer on the way), each rank of a sharded weight
// reading only its own rows.
//
// Differences from the reference, on purpose: an entry shorter than the tensor is an error (the
// reference fills what it has "for debugging"), the header's item size and storage order are
// checked against the request (the reference ignores them), and a deflated entry needs libz at run
// time (resolved with dlopen; NumPy's savez writes stored entries, savez_compressed deflated ones).
#include <dlfcn.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>
#include <zlib.h>

#include <algorithm>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "runtime.h"

namespace dmc {
namespace {

inline uint16_t rd16(const unsigned char *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
inline uint32_t rd32(const unsigned char *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
inline uint64_t rd64(const unsigned char *p) { return (uint64_t)rd32(p) | ((uint64_t)rd32(p + 4) << 32); }

bool pread_all(int fd, void *dst, size_t bytes, uint64_t off) {
    unsigned char *d = static_cast<unsigned char *>(dst);
    while (bytes) {
        ssize_t r = pread(fd, d, bytes, (off_t)off);
        if (r <= 0) return false;
        d += r;
        off += (uint64_t)r;
        bytes -= (size_t)r;
    }
    return true;
}

struct ZipEntry {
    uint64_t local_off = 0, comp = 0, uncomp = 0;
    int method = 0;
};

// Walk the central directory (zip64 aware: NumPy forces zip64 local headers) for `name`.
int zip_find(int fd, uint64_t file_size, const std::string &name, ZipEntry *out, std::string *why) {
    const uint64_t tail = std::min<uint64_t>(file_size, 65557 + 20);  // EOCD + longest comment + zip64 locator
    std::vector<unsigned char> buf((size_t)tail);
    if (tail < 22 || !pread_all(fd, buf.data(), (size_t)tail, file_size - tail)) { *why = "not a zip file (too short)"; return 1; }
    int64_t e = -1;
    for (int64_t i = (int64_t)tail - 22; i >= 0; --i)
        if (rd32(&buf[(size_t)i]) == 0x06054b50u) { e = i; break; }
    if (e < 0) { *why = "not a zip file (no end-of-central-directory record)"; return 1; }
    uint64_t entries = rd16(&buf[(size_t)e + 10]), cd_size = rd32(&buf[(size_t)e + 12]), cd_off = rd32(&buf[(size_t)e + 16]);
    if (entries == 0xFFFF || cd_size == 0xFFFFFFFFu || cd_off == 0xFFFFFFFFu) {
        if (e < 20 || rd32(&buf[(size_t)e - 20]) != 0x07064b50u) { *why = "zip64 archive without a zip64 locator"; return 1; }
        const uint64_t e64 = rd64(&buf[(size_t)e - 20 + 8]);
        unsigned char r[56];
        if (e64 + 56 > file_size || !pread_all(fd, r, 56, e64) || rd32(r) != 0x06064b50u) { *why = "bad zip64 end record"; return 1; }
        entries = rd64(r + 32);
        cd_size = rd64(r + 40);
        cd_off = rd64(r + 48);
    }
    if (cd_off + cd_size > file_size) { *why = "central directory outside the file"; return 1; }
    std::vector<unsigned char> cd((size_t)cd_size);
    if (!pread_all(fd, cd.data(), (size_t)cd_size, cd_off)) { *why = "cannot read the central directory"; return 1; }
    size_t p = 0;
    for (uint64_t i = 0; i < entries && p + 46 <= cd.size(); ++i) {
        if (rd32(&cd[p]) != 0x02014b50u) break;
        const int method = rd16(&cd[p + 10]);
        uint64_t comp = rd32(&cd[p + 20]), uncomp = rd32(&cd[p + 24]), loff = rd32(&cd[p + 42]);
        const size_t nlen = rd16(&cd[p + 28]), xlen = rd16(&cd[p + 30]), clen = rd16(&cd[p + 32]);
        if (p + 46 + nlen + xlen + clen > cd.size()) break;
        const std::string nm(reinterpret_cast<const char *>(&cd[p + 46]), nlen);
        // zip64 extra field: the values that overflowed, in the order uncompressed, compressed, offset
        size_t x = p + 46 + nlen;
        const size_t xend = x + xlen;
        while (x + 4 <= xend) {
            const uint16_t id = rd16(&cd[x]), sz = rd16(&cd[x + 2]);
            if (id == 0x0001) {
                size_t q = x + 4;
                if (uncomp == 0xFFFFFFFFu && q + 8 <= xend) { uncomp = rd64(&cd[q]); q += 8; }
                if (comp == 0xFFFFFFFFu && q + 8 <= xend) { comp = rd64(&cd[q]); q += 8; }
                if (loff == 0xFFFFFFFFu && q + 8 <= xend) { loff = rd64(&cd[q]); q += 8; }
            }
            x += 4 + (size_t)sz;
        }
        if (nm == name) {
            out->local_off = loff;
            out->comp = comp;
            out->uncomp = uncomp;
            out->method = method;
            return 0;
        }
        p += 46 + nlen + xlen + clen;
    }
    *why = "no such entry";
    return 2;
}

// zlib, resolved at run time so the library carries no link dependency on it
struct Zlib {
    int (*inflateInit2_)(z_streamp, int, const char *, int) = nullptr;
    int (*inflate)(z_streamp, int) = nullptr;
    int (*inflateEnd)(z_streamp) = nullptr;
    bool ok = false;
};
Zlib &zlib() {
    static Zlib z;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *h = dlopen("libz.so.1", RTLD_NOW | RTLD_LOCAL);
        if (!h) h = dlopen("libz.so", RTLD_NOW | RTLD_LOCAL);
        if (h) {
            z.inflateInit2_ = reinterpret_cast<int (*)(z_streamp, int, const char *, int)>(dlsym(h, "inflateInit2_"));
            z.inflate = reinterpret_cast<int (*)(z_streamp, int)>(dlsym(h, "inflate"));
            z.inflateEnd = reinterpret_cast<int (*)(z_streamp)>(dlsym(h, "inflateEnd"));
            z.ok = z.inflateInit2_ && z.inflate && z.inflateEnd;
        }
    }
    return z;
}

// Sequential reader of an entry's uncompressed bytes (stored or deflated).
class EntryStream {
  public:
    EntryStream(int fd, uint64_t data_off, const ZipEntry &e) : fd_(fd), off_(data_off), e_(e) {}
    ~EntryStream() {
        if (zinit_) zlib().inflateEnd(&zs_);
    }
    // the next `bytes` uncompressed bytes into dst (dst == nullptr: skip them); false on a short or bad stream
    bool read(void *dst, uint64_t bytes) {
        if (e_.method == 0) {
            if (pos_ + bytes > e_.uncomp) return false;
            const bool ok = !dst || pread_all(fd_, dst, (size_t)bytes, off_ + pos_);
            pos_ += bytes;
            return ok;
        }
        if (e_.method != 8 || !zlib().ok) return false;
        if (!zinit_) {
            memset(&zs_, 0, sizeof zs_);
            if (zlib().inflateInit2_(&zs_, -15, ZLIB_VERSION, (int)sizeof(z_stream)) != Z_OK) return false;
            zinit_ = true;
            in_.resize(1 << 20);
        }
        std::vector<unsigned char> sink;
        while (bytes) {
            unsigned char *o;
            size_t want;
            if (dst) {
                o = static_cast<unsigned char *>(dst);
                want = (size_t)std::min<uint64_t>(bytes, 1u << 30);
            } else {
                if (sink.empty()) sink.resize(1 << 20);
                o = sink.data();
                want = (size_t)std::min<uint64_t>(bytes, sink.size());
            }
            zs_.next_out = o;
            zs_.avail_out = (uInt)want;
            while (zs_.avail_out) {
                if (zs_.avail_in == 0) {
                    const uint64_t left = e_.comp - cpos_;
                    if (!left) return false;
                    const size_t n = (size_t)std::min<uint64_t>(left, in_.size());
                    if (!pread_all(fd_, in_.data(), n, off_ + cpos_)) return false;
                    cpos_ += n;
                    zs_.next_in = in_.data();
                    zs_.avail_in = (uInt)n;
                }
                const int r = zlib().inflate(&zs_, Z_NO_FLUSH);
                if (r == Z_STREAM_END && zs_.avail_out) return false;
                if (r != Z_OK && r != Z_STREAM_END) return false;
            }
            if (dst) dst = static_cast<unsigned char *>(dst) + want;
            bytes -= want;
            pos_ += want;
        }
        return true;
    }

  private:
    int fd_;
    uint64_t off_;
    ZipEntry e_;
    uint64_t pos_ = 0, cpos_ = 0;
    z_stream zs_;
    bool zinit_ = false;
    std::vector<unsigned char> in_;
};

// Value of 'key': in the NPY header dictionary text (a Python literal written by NumPy).
bool npy_field(const std::string &h, const char *key, std::string *val) {
    const std::string k = std::string("'") + key + "'";
    size_t p = h.find(k);
    if (p == std::string::npos) return false;
    p = h.find(':', p + k.size());
    if (p == std::string::npos) return false;
    ++p;
    while (p < h.size() && h[p] == ' ') ++p;
    size_t q = p;
    if (p < h.size() && h[p] == '(') q = h.find(')', p);
    else if (p < h.size() && h[p] == '\'') q = h.find('\'', p + 1);
    else {
        while (q < h.size() && h[q] != ',' && h[q] != '}') ++q;
        --q;
    }
    if (q == std::string::npos) return false;
    *val = h.substr(p, q - p + 1);
    return true;
}

struct Located {
    ZipEntry ze;
    uint64_t payload_off = 0;  // first byte of the entry's (possibly compressed) data in the file
    uint64_t npy_header = 0;   // bytes of NPY preamble + header before the array data
    dmc_npz_entry info;
};

int locate(int fd, const char *key, Located *L, std::string *why) {
    struct stat st;
    if (fstat(fd, &st) != 0) { *why = "cannot stat the file"; return 1; }
    int rc = zip_find(fd, (uint64_t)st.st_size, std::string(key) + ".npy", &L->ze, why);
    if (rc == 2) rc = zip_find(fd, (uint64_t)st.st_size, key, &L->ze, why);  // some savers omit the extension
    if (rc) {
        if (rc == 2) *why = std::string("key `") + key + "` not found";
        return rc;
    }
    unsigned char lh[30];
    if (!pread_all(fd, lh, 30, L->ze.local_off) || rd32(lh) != 0x04034b50u) { *why = "bad local file header"; return 1; }
    L->payload_off = L->ze.local_off + 30 + rd16(lh + 26) + rd16(lh + 28);
    if (L->ze.method != 0 && L->ze.method != 8) { *why = "entry uses a compression method other than stored / deflate"; return 1; }
    if (L->ze.method == 8 && !zlib().ok) { *why = "entry is deflated and libz.so.1 is not available"; return 1; }
    EntryStream s(fd, L->payload_off, L->ze);
    unsigned char pre[12];
    if (!s.read(pre, 10) || memcmp(pre, "\x93NUMPY", 6) != 0) { *why = "entry is not a valid .npy file"; return 1; }
    const int major = pre[6];
    uint64_t hlen;
    if (major == 1) {
        hlen = rd16(pre + 8);
        L->npy_header = 10 + hlen;
    } else {
        if (!s.read(pre + 10, 2)) { *why = "truncated .npy header"; return 1; }
        hlen = rd32(pre + 8);
        L->npy_header = 12 + hlen;
    }
    if (hlen > (1u << 20)) { *why = "unreasonable .npy header length"; return 1; }
    std::string h((size_t)hlen, '\0');
    if (!s.read(&h[0], hlen)) { *why = "truncated .npy header"; return 1; }
    dmc_npz_entry &o = L->info;
    memset(&o, 0, sizeof o);
    o.method = L->ze.method;
    o.data_offset = L->ze.method == 0 ? (int64_t)(L->payload_off + L->npy_header) : -1;
    o.data_bytes = (int64_t)(L->ze.uncomp - L->npy_header);
    std::string v;
    if (npy_field(h, "descr", &v)) {
        const std::string d = v.size() >= 2 ? v.substr(1, v.size() - 2) : v;  // strip the quotes
        strncpy(o.descr, d.c_str(), sizeof o.descr - 1);
        size_t i = 0;
        while (i < d.size() && !(d[i] >= '0' && d[i] <= '9')) ++i;
        o.itemsize = i < d.size() ? atoi(d.c_str() + i) : 0;
        if (d.find("bfloat16") != std::string::npos) o.itemsize = 2;
    }
    if (npy_field(h, "fortran_order", &v)) o.fortran_order = v.find("True") != std::string::npos;
    if (npy_field(h, "shape", &v)) {
        const char *p = v.c_str();
        while (*p && o.ndim < 4) {
            while (*p && !(*p >= '0' && *p <= '9')) ++p;
            if (!*p) break;
            o.shape[o.ndim++] = strtoll(p, const_cast<char **>(&p), 10);
        }
    }
    return 0;
}

constexpr size_t kRingBytes = 8u << 20;
constexpr int kRingSlots = 8;    // two groups of kReaders slots: one being filled while the other drains
constexpr int kReaders = 4;      // a single thread copies out of the page cache at only ~6 GB/s

}  // namespace
}  // namespace dmc

using namespace dmc;

extern "C" int dmc_npz_locate(const char *path, const char *key, dmc_npz_entry *out) {
    if (!path || !key || !out) return DMC_CUDA_ERR_BAD_ARG;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return DMC_CUDA_ERR_IO;
    Located L;
    std::string why;
    const int rc = locate(fd, key, &L, &why);
    close(fd);
    if (rc) return DMC_CUDA_ERR_IO;
    *out = L.info;
    return DMC_CUDA_OK;
}

extern "C" int dmc_cuda_load_npz(const char *path, const char *key, int64_t rows, int64_t cols, int wdtype, int rank,
                                 int world, int64_t host_dst, void **dev_out, int64_t *rows_out) {
    std::lock_guard<std::mutex> lock(ctx_mutex());
    if (dev_out) *dev_out = nullptr;
    if (rows_out) *rows_out = 0;
    if (dmc::status()) return dmc::status();
    if (!path || !key || !dev_out || rows <= 0 || cols <= 0 || world < 1 || rank < 0 || rank >= world ||
        (wdtype != DMC_W_BF16 && wdtype != DMC_W_F32))
        return fail(DMC_CUDA_ERR_BAD_ARG, "load_npz: need a path, a key, rows, cols > 0, a weight type and 0 <= rank < world");
    int rc = ensure_init();
    if (rc) return rc;
    Context &c = ctx();
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(DMC_CUDA_ERR_IO, "vault.load_npz: cannot open `%s`", path);
    Located L;
    std::string why;
    if (locate(fd, key, &L, &why)) {
        close(fd);
        return fail(DMC_CUDA_ERR_IO, "vault.load_npz: `%s`: %s", path, why.c_str());
    }
    const size_t esz = wdtype == DMC_W_BF16 ? 2 : 4;
    if (L.info.itemsize != (int)esz || L.info.fortran_order) {
        close(fd);
        return fail(DMC_CUDA_ERR_IO, "vault.load_npz: entry `%s` holds `%s`%s, not row-major %zu-byte elements", key,
                    L.info.descr, L.info.fortran_order ? " in Fortran order" : "", esz);
    }
    if ((uint64_t)L.info.data_bytes < (uint64_t)rows * (uint64_t)cols * esz) {
        close(fd);
        return fail(DMC_CUDA_ERR_IO, "vault.load_npz: entry `%s` data is %lld bytes but expected %llu", key,
                    (long long)L.info.data_bytes, (unsigned long long)((uint64_t)rows * cols * esz));
    }
    int64_t r0 = 0, r1 = rows;
    dmc_cuda_shard_range(rows, rank, world, &r0, &r1);
    const uint64_t first = (uint64_t)r0 * cols * esz, total = (uint64_t)(r1 - r0) * cols * esz;

    unsigned char *ring = nullptr, *dev = nullptr;
    cudaEvent_t ev[kRingSlots] = {};
    auto cleanup = [&](bool keep_dev) {
        for (cudaEvent_t e : ev)
            if (e) cudaEventDestroy(e);
        if (dev && !keep_dev) cudaFree(dev);
        close(fd);
    };
    cudaError_t ce = dmc_malloc((void **)&dev, std::max<uint64_t>(total, 16));
    // the ring outlives the call: pinning 64 MiB costs as much as reading a few hundred MiB
    if (ce == cudaSuccess && !c.ingest_ring) ce = dmc_malloc_host((void **)&c.ingest_ring, kRingBytes * kRingSlots);
    ring = c.ingest_ring;
    for (int i = 0; i < kRingSlots && ce == cudaSuccess; ++i) ce = cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming);
    if (ce != cudaSuccess) {
        cleanup(false);
        return fail(ce == cudaErrorMemoryAllocation ? DMC_CUDA_ERR_OOM : DMC_CUDA_ERR_CUDA, "load_npz: %s", cudaGetErrorString(ce));
    }
    bool ok = true;
    uint64_t done = 0;
    if (L.ze.method == 0) {
        // stored entry: any byte range can be read directly, so kReaders threads fill a group of ring
        // slots at once while the previous group's copies to the device are still running
        const uint64_t base = L.payload_off + L.npy_header + first;
        for (int group = 0; ok && ce == cudaSuccess && done < total; group ^= 1) {
            std::thread th[kReaders];
            bool good[kReaders];
            size_t len[kReaders];
            int used = 0;
            uint64_t off = done;
            for (int j = 0; j < kReaders && off < total; ++j, ++used) {
                const int slot = group * kReaders + j;
                if ((ce = cudaEventSynchronize(ev[slot])) != cudaSuccess) break;  // the slot's previous copy has left it
                len[j] = (size_t)std::min<uint64_t>(kRingBytes, total - off);
                unsigned char *h = ring + (size_t)slot * kRingBytes;
                unsigned char *hd = host_dst ? reinterpret_cast<unsigned char *>(host_dst) + off : nullptr;
                const uint64_t src = base + off;
                const size_t n = len[j];
                bool *g = &good[j];
                th[j] = std::thread([=]() {
                    *g = pread_all(fd, h, n, src);
                    if (*g && hd) memcpy(hd, h, n);
                });
                off += len[j];
            }
            for (int j = 0; j < used; ++j) th[j].join();
            for (int j = 0; j < used && ok && ce == cudaSuccess; ++j) {
                const int slot = group * kReaders + j;
                ok = good[j];
                if (!ok) break;
                ce = cudaMemcpyAsync(dev + done, ring + (size_t)slot * kRingBytes, len[j], cudaMemcpyHostToDevice, c.stream);
                if (ce == cudaSuccess) ce = cudaEventRecord(ev[slot], c.stream);
                done += len[j];
            }
        }
    } else {
        // deflated entry: one sequential stream, inflated chunk by chunk into the ring
        EntryStream s(fd, L.payload_off, L.ze);
        ok = s.read(nullptr, L.npy_header + first);
        for (int slot = 0; ok && done < total; slot = (slot + 1) % kRingSlots) {
            const size_t n = (size_t)std::min<uint64_t>(kRingBytes, total - done);
            unsigned char *h = ring + (size_t)slot * kRingBytes;
            if ((ce = cudaEventSynchronize(ev[slot])) != cudaSuccess) break;  // the slot's previous copy has left it
            ok = s.read(h, n);
            if (!ok) break;
            if (host_dst) memcpy(reinterpret_cast<unsigned char *>(host_dst) + done, h, n);
            if ((ce = cudaMemcpyAsync(dev + done, h, n, cudaMemcpyHostToDevice, c.stream)) != cudaSuccess) break;
            if ((ce = cudaEventRecord(ev[slot], c.stream)) != cudaSuccess) break;
            done += n;
        }
    }
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(c.stream);
    if (!ok || ce != cudaSuccess) {
        cleanup(false);
        if (!ok) return fail(DMC_CUDA_ERR_IO, "vault.load_npz: read error for `%s` in `%s`", key, path);
        return fail(DMC_CUDA_ERR_CUDA, "load_npz: upload failed: %s", cudaGetErrorString(ce));
    }
    if (host_dst) {
        // the host copy the JIT keeps stands for this device buffer from now on
        for (const RegisteredRange &rg : c.registered)
            if ((uintptr_t)host_dst < rg.host + rg.bytes && rg.host < (uintptr_t)host_dst + total) {
                cleanup(false);
                return fail(DMC_CUDA_ERR_BAD_ARG, "load_npz: host range overlaps a registered range");
            }
        c.registered.push_back(RegisteredRange{(uintptr_t)host_dst, (size_t)total, dev, wdtype});
        c.resident_bytes += (int64_t)total;
    }
    cleanup(true);
    *dev_out = dev;
    if (rows_out) *rows_out = r1 - r0;
    return DMC_CUDA_OK;
}
