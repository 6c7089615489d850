// Edge list -> CSR, and the reader of GNNAdvisor-style `.npz` graph files (host only).
//
// Native counterpart of the reference's converters (scripts/npz_to_csr.py:13-28,
// scripts/fetch_dataset.py:11-21): those build scipy's coo_matrix from (src, dst), call tocsr() -
// which sums duplicate entries and leaves every row's columns sorted - and write indptr / indices as
// text, cell by cell in Python.  Here the same CSR structure is built by all cores: histogram of the
// rows, stable scatter, then sort + unique inside each row.
#include "mps.h"

#include <zlib.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "mps_internal.h"

using mps::fail;

namespace {

int thread_count(int requested, size_t work) {
    int n = requested > 0 ? requested : (int)std::thread::hardware_concurrency();
    if (n < 1) n = 1;
    const size_t by_size = work / (1 << 16) + 1;
    if ((size_t)n > by_size) n = (int)by_size;
    return n;
}

template <typename F>
void parallel_ranges(size_t n, int nt, F f) {  // f(thread, begin, end)
    std::vector<std::thread> th;
    for (int t = 1; t < nt; ++t) th.emplace_back(f, t, n * (size_t)t / nt, n * (size_t)(t + 1) / nt);
    f(0, (size_t)0, n / (size_t)nt);
    for (auto &x : th) x.join();
}

}  // namespace

extern "C" int mps_coo_to_csr(int32_t n_nodes, int64_t n_edges, const int64_t *src, const int64_t *dst, int n_threads, mps_csr *out) {
    if (!out || n_edges < 0 || (n_edges > 0 && (!src || !dst)) || n_nodes < 0) return fail(MPS_ERR_ARG, "mps_coo_to_csr: bad argument");
    memset(out, 0, sizeof *out);
    int nt = thread_count(n_threads, (size_t)n_edges);
    // size of the (square) matrix: given, or largest index + 1
    std::vector<int64_t> hi((size_t)nt, -1), lo((size_t)nt, 0);
    parallel_ranges((size_t)n_edges, nt, [&](int t, size_t b, size_t e) {
        int64_t mx = -1, mn = 0;
        for (size_t i = b; i < e; ++i) {
            mx = std::max(mx, std::max(src[i], dst[i]));
            mn = std::min(mn, std::min(src[i], dst[i]));
        }
        hi[(size_t)t] = mx; lo[(size_t)t] = mn;
    });
    const int64_t max_index = *std::max_element(hi.begin(), hi.end());
    if (*std::min_element(lo.begin(), lo.end()) < 0) return fail(MPS_ERR_ARG, "mps_coo_to_csr: negative node index");
    int64_t n = n_nodes > 0 ? n_nodes : max_index + 1;
    if (max_index >= n) return fail(MPS_ERR_ARG, "mps_coo_to_csr: node index %lld outside [0, %lld)", (long long)max_index, (long long)n);
    if (n + 1 + n_edges >= (int64_t)1 << 31) return fail(MPS_ERR_UNSUPPORTED, "mps_coo_to_csr: N+1+edges does not fit 31 bits");

    while (nt > 1 && (size_t)nt * (size_t)n > ((size_t)1 << 28)) nt /= 2;  // one histogram of n ints per thread
    // rows: per-thread histograms -> per-thread write cursors (stable: thread order = edge order)
    std::vector<std::vector<int32_t>> hist((size_t)nt, std::vector<int32_t>((size_t)n + 1, 0));
    parallel_ranges((size_t)n_edges, nt, [&](int t, size_t b, size_t e) {
        int32_t *h = hist[(size_t)t].data();
        for (size_t i = b; i < e; ++i) ++h[src[i]];
    });
    std::vector<int64_t> row_start((size_t)n + 1, 0);
    for (int64_t r = 0; r < n; ++r) {
        int64_t sum = 0;
        for (int t = 0; t < nt; ++t) { const int32_t c = hist[(size_t)t][(size_t)r]; hist[(size_t)t][(size_t)r] = (int32_t)sum; sum += c; }
        row_start[(size_t)r + 1] = row_start[(size_t)r] + sum;
    }
    std::vector<int32_t> cols((size_t)(n_edges ? n_edges : 1));
    parallel_ranges((size_t)n_edges, nt, [&](int t, size_t b, size_t e) {
        int32_t *cur = hist[(size_t)t].data();
        for (size_t i = b; i < e; ++i) cols[(size_t)(row_start[(size_t)src[i]] + cur[src[i]]++)] = (int32_t)dst[i];
    });
    hist.clear();
    hist.shrink_to_fit();
    // inside each row: sort, drop duplicates (tocsr() sums them into one entry), count what is left
    std::vector<int32_t> kept((size_t)n + 1, 0);
    parallel_ranges((size_t)n, thread_count(n_threads, (size_t)n_edges), [&](int, size_t b, size_t e) {
        for (size_t r = b; r < e; ++r) {
            int32_t *first = cols.data() + row_start[r], *last = cols.data() + row_start[r + 1];
            std::sort(first, last);
            kept[r] = (int32_t)(std::unique(first, last) - first);
        }
    });
    int32_t *rp = (int32_t *)malloc(sizeof(int32_t) * ((size_t)n + 1));
    if (!rp) return fail(MPS_ERR_NOMEM, "mps_coo_to_csr: out of memory");
    rp[0] = 0;
    for (int64_t r = 0; r < n; ++r) rp[r + 1] = rp[r] + kept[(size_t)r];
    const int32_t nnz = rp[n];
    int32_t *ci = (int32_t *)malloc(sizeof(int32_t) * (size_t)(nnz ? nnz : 1));
    if (!ci) { free(rp); return fail(MPS_ERR_NOMEM, "mps_coo_to_csr: out of memory"); }
    parallel_ranges((size_t)n, thread_count(n_threads, (size_t)n_edges), [&](int, size_t b, size_t e) {
        for (size_t r = b; r < e; ++r) memcpy(ci + rp[r], cols.data() + row_start[r], sizeof(int32_t) * (size_t)kept[r]);
    });
    out->n_rows = (int32_t)n; out->nnz = nnz; out->row_ptr = rp; out->col_idx = ci;
    return MPS_OK;
}

// ------------------------------------------------------------------------------------- .npz

namespace {

uint16_t rd16(const unsigned char *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
uint32_t rd32(const unsigned char *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
uint64_t rd64(const unsigned char *p) { return (uint64_t)rd32(p) | ((uint64_t)rd32(p + 4) << 32); }

struct ZipEntry { std::string name; uint16_t method; uint64_t comp, uncomp, local; };

// Central directory of a zip archive (zip64 sizes and offsets included), read from the end of the file.
int zip_entries(const std::vector<unsigned char> &f, std::vector<ZipEntry> &out) {
    if (f.size() < 22) return -1;
    size_t eocd = f.size() - 22;
    while (true) {
        if (rd32(&f[eocd]) == 0x06054b50u) break;
        if (eocd == 0 || f.size() - eocd > 22 + 65535) return -1;
        --eocd;
    }
    uint64_t count = rd16(&f[eocd + 10]), cd_off = rd32(&f[eocd + 16]);
    if (eocd >= 20 && rd32(&f[eocd - 20]) == 0x07064b50u) {  // zip64 locator
        const uint64_t e64 = rd64(&f[eocd - 20 + 8]);
        if (e64 + 56 <= f.size() && rd32(&f[e64]) == 0x06064b50u) { count = rd64(&f[e64 + 32]); cd_off = rd64(&f[e64 + 48]); }
    }
    size_t p = (size_t)cd_off;
    for (uint64_t i = 0; i < count; ++i) {
        if (p + 46 > f.size() || rd32(&f[p]) != 0x02014b50u) return -1;
        ZipEntry e;
        e.method = rd16(&f[p + 10]);
        e.comp = rd32(&f[p + 20]); e.uncomp = rd32(&f[p + 24]);
        const uint16_t nlen = rd16(&f[p + 28]), xlen = rd16(&f[p + 30]), clen = rd16(&f[p + 32]);
        e.local = rd32(&f[p + 42]);
        if (p + 46 + nlen + xlen > f.size()) return -1;
        e.name.assign((const char *)&f[p + 46], nlen);
        size_t x = p + 46 + nlen;
        const size_t xend = x + xlen;
        while (x + 4 <= xend) {  // zip64 extra: the fields that overflowed, in this order
            const uint16_t id = rd16(&f[x]), sz = rd16(&f[x + 2]);
            if (id == 0x0001) {
                size_t q = x + 4;
                if (e.uncomp == 0xFFFFFFFFu && q + 8 <= xend) { e.uncomp = rd64(&f[q]); q += 8; }
                if (e.comp == 0xFFFFFFFFu && q + 8 <= xend) { e.comp = rd64(&f[q]); q += 8; }
                if (e.local == 0xFFFFFFFFu && q + 8 <= xend) { e.local = rd64(&f[q]); q += 8; }
            }
            x += 4 + sz;
        }
        out.push_back(e);
        p += 46 + (size_t)nlen + xlen + clen;
    }
    return 0;
}

int zip_read(const std::vector<unsigned char> &f, const ZipEntry &e, std::vector<unsigned char> &out) {
    const size_t l = (size_t)e.local;
    if (l + 30 > f.size() || rd32(&f[l]) != 0x04034b50u) return -1;
    const size_t data = l + 30 + rd16(&f[l + 26]) + rd16(&f[l + 28]);
    if (data + e.comp > f.size()) return -1;
    out.resize((size_t)e.uncomp);
    if (e.method == 0) {
        if (e.comp != e.uncomp) return -1;
        memcpy(out.data(), &f[data], (size_t)e.uncomp);
        return 0;
    }
    if (e.method != 8) return -2;
    z_stream z;
    memset(&z, 0, sizeof z);
    if (inflateInit2(&z, -MAX_WBITS) != Z_OK) return -1;
    size_t in_at = 0, out_at = 0;
    int rc = Z_OK;
    while (rc != Z_STREAM_END) {  // avail_in / avail_out are 32-bit: feed in pieces
        const size_t in_n = std::min<size_t>((size_t)e.comp - in_at, 1u << 30), out_n = std::min<size_t>(out.size() - out_at, 1u << 30);
        z.next_in = const_cast<unsigned char *>(&f[data + in_at]); z.avail_in = (uInt)in_n;
        z.next_out = out.data() + out_at; z.avail_out = (uInt)out_n;
        rc = inflate(&z, Z_NO_FLUSH);
        in_at += in_n - z.avail_in; out_at += out_n - z.avail_out;
        if (rc != Z_OK && rc != Z_STREAM_END) break;
        if (rc == Z_OK && in_n - z.avail_in == 0 && out_n - z.avail_out == 0) break;  // no progress
    }
    inflateEnd(&z);
    return (rc == Z_STREAM_END && out_at == out.size()) ? 0 : -1;
}

// One-dimensional little-endian integer array from a .npy image -> int64.
int npy_to_i64(const std::vector<unsigned char> &b, std::vector<int64_t> &out, std::string &why) {
    if (b.size() < 10 || memcmp(b.data(), "\x93NUMPY", 6) != 0) { why = "not a .npy member"; return -1; }
    size_t hlen, hoff;
    if (b[6] == 1) { hlen = rd16(&b[8]); hoff = 10; } else { if (b.size() < 12) return -1; hlen = rd32(&b[8]); hoff = 12; }
    if (hoff + hlen > b.size()) { why = "truncated .npy header"; return -1; }
    const std::string h((const char *)&b[hoff], hlen);
    int width = 0;
    bool is_unsigned = false;
    for (const char *d : {"<i8", "<i4", "<u4", "<u8", "|i8", "<i2", "<u2"})
        if (h.find(std::string("'") + d + "'") != std::string::npos) { width = d[2] - '0'; is_unsigned = d[1] == 'u'; }
    if (!width) { why = "unsupported dtype (need little-endian integers): " + h; return -1; }
    const size_t sp = h.find("'shape': (");
    if (sp == std::string::npos) { why = "no shape in .npy header"; return -1; }
    const long long n = atoll(h.c_str() + sp + 10);
    const size_t close = h.find(')', sp);
    const std::string shape = h.substr(sp + 10, close - sp - 10);
    const size_t comma = shape.find(',');  // numpy writes a one-dimensional shape as "(n,)"
    if (comma == std::string::npos || shape.find_first_of("0123456789", comma + 1) != std::string::npos) {
        why = "array is not one-dimensional: (" + shape + ")";
        return -1;
    }
    const unsigned char *p = &b[hoff + hlen];
    if (n < 0 || hoff + hlen + (size_t)n * width > b.size()) { why = "truncated .npy data"; return -1; }
    out.resize((size_t)n);
    for (long long i = 0; i < n; ++i) {
        const unsigned char *q = p + (size_t)i * width;
        int64_t v;
        if (width == 8) v = (int64_t)rd64(q);
        else if (width == 4) v = is_unsigned ? (int64_t)rd32(q) : (int64_t)(int32_t)rd32(q);
        else v = is_unsigned ? (int64_t)rd16(q) : (int64_t)(int16_t)rd16(q);
        out[(size_t)i] = v;
    }
    return 0;
}

}  // namespace

extern "C" int mps_npz_to_csr(const char *path, int n_threads, mps_csr *out) {
    if (!path || !out) return fail(MPS_ERR_ARG, "mps_npz_to_csr: NULL argument");
    memset(out, 0, sizeof *out);
    FILE *fp = fopen(path, "rb");
    if (!fp) return fail(MPS_ERR_IO, "cannot open %s: %s", path, strerror(errno));
    std::vector<unsigned char> file;
    fseek(fp, 0, SEEK_END);
    const long size = ftell(fp);
    fseek(fp, 0, SEEK_SET);
    if (size > 0) file.resize((size_t)size);
    const bool ok = size > 0 && fread(file.data(), 1, (size_t)size, fp) == (size_t)size;
    fclose(fp);
    if (!ok) return fail(MPS_ERR_IO, "cannot read %s", path);
    std::vector<ZipEntry> entries;
    if (zip_entries(file, entries) != 0) return fail(MPS_ERR_FORMAT, "%s: not a zip (.npz) archive", path);
    std::vector<int64_t> src, dst;
    for (const char *want : {"src_li.npy", "dst_li.npy"}) {
        const ZipEntry *hit = nullptr;
        for (const ZipEntry &e : entries)
            if (e.name == want) hit = &e;
        if (!hit) return fail(MPS_ERR_FORMAT, "%s: no member %s (the reference's converter reads src_li and dst_li)", path, want);
        std::vector<unsigned char> raw;
        const int rc = zip_read(file, *hit, raw);
        if (rc == -2) return fail(MPS_ERR_UNSUPPORTED, "%s: member %s uses zip method %d", path, want, (int)hit->method);
        if (rc != 0) return fail(MPS_ERR_FORMAT, "%s: member %s is damaged", path, want);
        std::string why;
        if (npy_to_i64(raw, want[0] == 's' ? src : dst, why) != 0) return fail(MPS_ERR_FORMAT, "%s: member %s: %s", path, want, why.c_str());
    }
    if (src.size() != dst.size()) return fail(MPS_ERR_FORMAT, "%s: src_li has %zu entries, dst_li %zu", path, src.size(), dst.size());
    return mps_coo_to_csr(0, (int64_t)src.size(), src.data(), dst.data(), n_threads, out);
}
