// `.csr` text files and the binary sidecar (host only).
//
// Text grammar = what the reference's loader accepts and its writers emit
// (src/MergePathSpMM.cu:130-173; scripts/npz_to_csr.py:21-28): two lines of decimal integers
// separated by ','.  The reference makes two passes with getline/stringstream/stoi on one thread
// and holds two copies of each line; here the file is mapped once and the cells of a line are
// counted and parsed by all cores in place.
#include "mps.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

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

struct Span { const char *b, *e; };

int worker_count(int requested, size_t bytes) {
    int n = requested > 0 ? requested : (int)std::thread::hardware_concurrency();
    if (n < 1) n = 1;
    const size_t by_size = bytes / (1 << 16) + 1;  // no point in a thread per few KB
    if ((size_t)n > by_size) n = (int)by_size;
    return n;
}

// Cuts [b,e) into n pieces that end just after a ','.
std::vector<Span> cut_at_commas(const char *b, const char *e, int n) {
    std::vector<Span> out;
    const char *at = b;
    for (int i = 1; i <= n && at < e; ++i) {
        const char *stop = i == n ? e : b + (size_t)(e - b) * i / n;
        if (stop < at) stop = at;
        if (i != n) {
            const void *c = memchr(stop, ',', (size_t)(e - stop));
            stop = c ? (const char *)c + 1 : e;
        }
        if (stop > at) out.push_back({at, stop});
        at = stop;
    }
    return out;
}

// A piece holds one cell per ',' plus one more if text follows its last ','.
size_t count_cells(Span s) {
    size_t n = 0;
    const char *last = nullptr;
    for (const char *b = s.b; b < s.e;) {  // blocks keep the per-byte sum in a narrow counter: the loop vectorises
        const char *stop = s.e - b > 4096 ? b + 4096 : s.e;
        unsigned hits = 0;
        for (const char *p = b; p < stop; ++p) hits += *p == ',';
        n += hits;
        b = stop;
    }
    for (const char *p = s.e; p > s.b; --p)
        if (p[-1] == ',') { last = p - 1; break; }
    if (s.e > s.b && (!last || last + 1 < s.e)) ++n;  // text after the last ',' (or no ',' at all) is one more cell
    return n;
}

// Eight ASCII digits, first digit in the lowest byte -> their value (three multiplications, no loop).
inline uint32_t eight_digits(uint64_t v) {
    const uint64_t mask = 0x000000FF000000FFull;
    const uint64_t mul1 = 0x000F424000000064ull;  // 100 + (1000000 << 32)
    const uint64_t mul2 = 0x0000271000000001ull;  // 1 + (10000 << 32)
    v = (v * 10) + (v >> 8);
    v = (((v & mask) * mul1) + (((v >> 16) & mask) * mul2)) >> 32;
    return (uint32_t)v;
}

// Plain cells - one to eight digits and a ',' with nothing else - eight bytes at a time: the position of the ',' from a
// zero-byte test, the digits checked and converted in the same word.  Stops at the first cell that is anything else
// (blanks, a sign, nine or ten digits, a bad byte) or too near the end of the piece for an 8-byte read, and leaves
// it to the byte-wise loop of parse_cells.  Little-endian hosts (the first character is the lowest byte).
inline const char *parse_plain_cells(const char *p, const char *e, int32_t *&out) {
    const uint64_t ones = 0x0101010101010101ull, high = 0x8080808080808080ull;
    while (e - p >= 16) {
        uint64_t x;
        memcpy(&x, p, 8);
        const uint64_t c = x ^ 0x2C2C2C2C2C2C2C2Cull;               // a zero byte where a ',' stands
        const uint64_t comma = (c - ones) & ~c & high;
        unsigned len;
        if (comma) {
            len = (unsigned)__builtin_ctzll(comma) >> 3;            // digits before the first ','
            if (len == 0) return p;                                  // empty cell: the byte-wise loop reports it
        } else {
            if (p[8] != ',') return p;                               // nine digits or more, or something else
            len = 8;
        }
        const uint64_t keep = len == 8 ? ~0ull : (1ull << (8 * len)) - 1;
        const uint64_t d = (x & keep) - (0x3030303030303030ull & keep);  // digit values, if digits they are
        // every byte of d must be 0..9: no high nibble, and adding 6 must not carry into one
        if (((d | (d + 0x0606060606060606ull)) & 0xF0F0F0F0F0F0F0F0ull) != 0) return p;
        // (a byte below '0' made the subtraction borrow: its own byte then reads >= 0xF0 or it spoilt its neighbour - both
        // show as a high nibble)
        *out++ = (int32_t)eight_digits(len == 8 ? d : d << (8 * (8 - len)));  // shifted up: the missing digits lead as zeros
        p += len + 1;
    }
    return p;
}

// Parses the cells of a piece into out[]; returns the offset of the first bad byte or -1.
long parse_cells(Span s, int32_t *out) {
    const char *p = s.b;
    while (p < s.e) {
        p = parse_plain_cells(p, s.e, out);  // runs of plain cells; what follows is one cell the long way
        if (p >= s.e) break;
        while (p < s.e && (*p == ' ' || *p == '\t')) ++p;
        bool neg = false;
        if (p < s.e && (*p == '-' || *p == '+')) { neg = *p == '-'; ++p; }
        if (p >= s.e || *p < '0' || *p > '9') return (long)(p - s.b);
        int64_t v = 0;
        while (p < s.e && *p >= '0' && *p <= '9') {
            v = v * 10 + (*p - '0');
            if (v > (int64_t)INT32_MAX + 1) return (long)(p - s.b);
            ++p;
        }
        if (neg) v = -v;
        if (v > INT32_MAX || v < INT32_MIN) return (long)(p - s.b);
        *out++ = (int32_t)v;
        while (p < s.e && (*p == ' ' || *p == '\t')) ++p;  // blanks after a cell: stoi stops at them, getline cut at the ','
        if (p < s.e) {
            if (*p != ',') return (long)(p - s.b);
            ++p;
        }
    }
    return -1;
}

// One line -> malloc'ed int32 array.
int parse_line(const char *b, const char *e, int n_threads, int32_t **out, size_t *count, const char *what) {
    std::vector<Span> pieces = cut_at_commas(b, e, worker_count(n_threads, (size_t)(e - b)));
    const size_t np = pieces.size();
    std::vector<size_t> cells(np + 1, 0);
    {
        std::vector<std::thread> th;
        for (size_t i = 1; i < np; ++i) th.emplace_back([&, i] { cells[i + 1] = count_cells(pieces[i]); });
        if (np) cells[1] = count_cells(pieces[0]);
        for (auto &t : th) t.join();
    }
    for (size_t i = 0; i < np; ++i) cells[i + 1] += cells[i];
    const size_t total = cells[np];
    if (total > (size_t)INT32_MAX) return fail(MPS_ERR_UNSUPPORTED, "%s has %zu cells, more than int32 holds", what, total);
    int32_t *arr = (int32_t *)malloc(sizeof(int32_t) * (total ? total : 1));
    if (!arr) return fail(MPS_ERR_NOMEM, "out of memory for %zu cells of %s", total, what);
    std::atomic<long> bad_at(-1);
    auto run = [&](size_t i) {
        long r = parse_cells(pieces[i], arr + cells[i]);
        if (r >= 0) {
            long want = -1;
            bad_at.compare_exchange_strong(want, (long)(pieces[i].b - b) + r);
        }
    };
    {
        std::vector<std::thread> th;
        for (size_t i = 1; i < np; ++i) th.emplace_back(run, i);
        if (np) run(0);
        for (auto &t : th) t.join();
    }
    if (bad_at.load() >= 0) {
        free(arr);
        return fail(MPS_ERR_FORMAT, "%s: not a decimal int32 cell at byte %ld of the line", what, bad_at.load());
    }
    *out = arr;
    *count = total;
    return MPS_OK;
}

struct Mapping {
    const char *data = nullptr;
    size_t size = 0;
    int fd = -1;
    ~Mapping() {
        if (data && size) munmap((void *)data, size);
        if (fd >= 0) close(fd);
    }
};

}  // namespace

extern "C" void mps_csr_free(mps_csr *csr) {
    if (!csr) return;
    free(csr->row_ptr);
    free(csr->col_idx);
    csr->row_ptr = csr->col_idx = nullptr;
    csr->n_rows = csr->nnz = 0;
}

// n_cols == nullptr: the square matrix of the reference program (every column index below n_rows); otherwise any
// non-negative column index is accepted and *n_cols receives max(n_rows, largest index + 1).
static int load_text(const char *path, int n_threads, mps_csr *out, int32_t *n_cols) {
    if (!path || !out) return fail(MPS_ERR_ARG, "mps_csr_load: NULL argument");
    memset(out, 0, sizeof *out);
    Mapping m;
    m.fd = open(path, O_RDONLY);
    if (m.fd < 0) return fail(MPS_ERR_IO, "cannot open %s: %s", path, strerror(errno));
    struct stat st;
    if (fstat(m.fd, &st) != 0) return fail(MPS_ERR_IO, "cannot stat %s: %s", path, strerror(errno));
    m.size = (size_t)st.st_size;
    if (m.size == 0) return fail(MPS_ERR_FORMAT, "%s is empty", path);
    void *map = mmap(nullptr, m.size, PROT_READ, MAP_PRIVATE, m.fd, 0);
    if (map == MAP_FAILED) { m.size = 0; return fail(MPS_ERR_IO, "cannot map %s: %s", path, strerror(errno)); }
    m.data = (const char *)map;
    madvise(map, m.size, MADV_SEQUENTIAL);

    const char *end = m.data + m.size;
    const char *nl1 = (const char *)memchr(m.data, '\n', m.size);
    const char *l1e = nl1 ? nl1 : end;
    const char *l2b = nl1 ? nl1 + 1 : end;
    const char *nl2 = l2b < end ? (const char *)memchr(l2b, '\n', (size_t)(end - l2b)) : nullptr;
    const char *l2e = nl2 ? nl2 : end;

    int32_t *rp = nullptr, *col = nullptr;
    size_t n_rp = 0, n_col = 0;
    if (int rc = parse_line(m.data, l1e, n_threads, &rp, &n_rp, "line 1 (row_ptr)")) return rc;
    if (n_rp == 0) { free(rp); return fail(MPS_ERR_FORMAT, "%s: line 1 holds no row_ptr cell", path); }
    if (int rc = parse_line(l2b, l2e, n_threads, &col, &n_col, "line 2 (col_idx)")) { free(rp); return rc; }

    const int64_t n_rows = (int64_t)n_rp - 1, nnz = rp[n_rp - 1];
    int rc = MPS_OK;
    if (nnz < 0 || (size_t)nnz != n_col)
        rc = fail(MPS_ERR_FORMAT, "%s: last row_ptr cell says %lld non-zeros, line 2 has %zu cells", path, (long long)nnz, n_col);
    else if (rp[0] != 0)
        rc = fail(MPS_ERR_FORMAT, "%s: row_ptr[0] is %d, expected 0", path, rp[0]);
    else if (n_rows + 1 + nnz >= (int64_t)1 << 31)
        rc = fail(MPS_ERR_UNSUPPORTED, "%s: N+1+nnz = %lld does not fit 31 bits", path, (long long)(n_rows + 1 + nnz));
    int32_t width = (int32_t)n_rows;
    if (rc == MPS_OK) {
        const long long bad_row = mps::first_decreasing_row(rp, n_rows, n_threads);
        if (bad_row >= 0) rc = fail(MPS_ERR_FORMAT, "%s: row_ptr decreases at row %lld", path, bad_row);
    }
    if (rc == MPS_OK && n_cols) {
        const int32_t top = mps::max_column(col, nnz, n_threads);
        if (top >= width) width = top == INT32_MAX ? top : top + 1;
    }
    if (rc == MPS_OK) {
        const long long bad = mps::first_bad_column(col, nnz, width, n_threads);
        if (bad >= 0) rc = fail(MPS_ERR_FORMAT, "%s: col_idx[%lld] = %d outside [0, %d)", path, bad, col[bad], width);
    }
    if (rc != MPS_OK) { free(rp); free(col); return rc; }
    if (n_cols) *n_cols = width;
    out->n_rows = (int32_t)n_rows;
    out->nnz = (int32_t)nnz;
    out->row_ptr = rp;
    out->col_idx = col;
    return MPS_OK;
}

extern "C" int mps_csr_load(const char *path, int n_threads, mps_csr *out) { return load_text(path, n_threads, out, nullptr); }

extern "C" int mps_csr_load_rect(const char *path, int n_threads, mps_csr *out, int32_t *n_cols) {
    if (!n_cols) return fail(MPS_ERR_ARG, "mps_csr_load_rect: n_cols is NULL");
    return load_text(path, n_threads, out, n_cols);
}

namespace {
// Formats cells [b,e) of a, each followed by ','.
void format_cells(const int32_t *a, size_t b, size_t e, std::string &s) {
    s.resize((e - b) * 12);  // "-2147483648," is the longest cell
    char *out = &s[0];
    for (size_t i = b; i < e; ++i) {
        int64_t v = a[i];
        if (v < 0) { *out++ = '-'; v = -v; }
        char digits[12];
        int n = 0;
        do { digits[n++] = (char)('0' + v % 10); v /= 10; } while (v);
        while (n) *out++ = digits[--n];
        *out++ = ',';
    }
    s.resize((size_t)(out - &s[0]));
}
int write_line(FILE *f, const int32_t *a, size_t n) {
    const size_t block = 1 << 20;
    const int nt = worker_count(0, n * 8);
    std::vector<std::string> bufs((size_t)nt);
    for (size_t base = 0; base < n; base += block * (size_t)nt) {
        std::vector<std::thread> th;
        for (int t = 0; t < nt; ++t) {
            const size_t b = base + block * (size_t)t, e = b + block < n ? b + block : n;
            if (b >= n) { bufs[(size_t)t].clear(); continue; }
            th.emplace_back(format_cells, a, b, e, std::ref(bufs[(size_t)t]));
        }
        for (auto &t : th) t.join();
        for (int t = 0; t < nt; ++t)
            if (!bufs[(size_t)t].empty() && fwrite(bufs[(size_t)t].data(), 1, bufs[(size_t)t].size(), f) != bufs[(size_t)t].size()) return -1;
    }
    return 0;
}
}  // namespace

extern "C" int mps_csr_save(const char *path, int32_t n_rows, const int32_t *row_ptr, const int32_t *col_idx) {
    if (!path || !row_ptr || n_rows < 0) return fail(MPS_ERR_ARG, "mps_csr_save: bad argument");
    const int32_t nnz = row_ptr[n_rows];
    if (nnz < 0 || (nnz > 0 && !col_idx)) return fail(MPS_ERR_ARG, "mps_csr_save: bad nnz / col_idx");
    FILE *f = fopen(path, "wb");
    if (!f) return fail(MPS_ERR_IO, "cannot create %s: %s", path, strerror(errno));
    int bad = write_line(f, row_ptr, (size_t)n_rows + 1);
    if (!bad) bad = fputc('\n', f) == EOF;
    if (!bad) bad = write_line(f, col_idx, (size_t)nnz);
    if (fclose(f) != 0) bad = 1;
    if (bad) return fail(MPS_ERR_IO, "short write to %s", path);
    return MPS_OK;
}

namespace {
struct BinHeader {
    char magic[8];
    int32_t n_rows, nnz, val_bytes;
    int32_t reserved[3];
};
static_assert(sizeof(BinHeader) == 32, "sidecar header is 32 bytes");
const char kMagic[8] = {'M', 'P', 'S', 'C', 'S', 'R', '0', '1'};
}  // namespace

extern "C" int mps_csr_save_bin(const char *path, int32_t n_rows, const int32_t *row_ptr, const int32_t *col_idx, const void *val,
                                int val_bytes) {
    if (!path || !row_ptr || n_rows < 0) return fail(MPS_ERR_ARG, "mps_csr_save_bin: bad argument");
    if (!(val_bytes == 0 || val_bytes == 2 || val_bytes == 4) || (val_bytes && !val)) return fail(MPS_ERR_ARG, "mps_csr_save_bin: val_bytes must be 0, 2 or 4");
    BinHeader h;
    memset(&h, 0, sizeof h);
    memcpy(h.magic, kMagic, 8);
    h.n_rows = n_rows; h.nnz = row_ptr[n_rows]; h.val_bytes = val_bytes;
    FILE *f = fopen(path, "wb");
    if (!f) return fail(MPS_ERR_IO, "cannot create %s: %s", path, strerror(errno));
    bool ok = fwrite(&h, sizeof h, 1, f) == 1;
    ok = ok && fwrite(row_ptr, 4, (size_t)n_rows + 1, f) == (size_t)n_rows + 1;
    ok = ok && (h.nnz == 0 || fwrite(col_idx, 4, (size_t)h.nnz, f) == (size_t)h.nnz);
    ok = ok && (!val_bytes || h.nnz == 0 || fwrite(val, (size_t)val_bytes, (size_t)h.nnz, f) == (size_t)h.nnz);
    if (fclose(f) != 0) ok = false;
    if (!ok) return fail(MPS_ERR_IO, "short write to %s", path);
    return MPS_OK;
}

extern "C" int mps_csr_load_bin(const char *path, mps_csr *out, void **val, int *val_bytes) {
    if (!path || !out) return fail(MPS_ERR_ARG, "mps_csr_load_bin: NULL argument");
    memset(out, 0, sizeof *out);
    if (val) *val = nullptr;
    if (val_bytes) *val_bytes = 0;
    FILE *f = fopen(path, "rb");
    if (!f) return fail(MPS_ERR_IO, "cannot open %s: %s", path, strerror(errno));
    BinHeader h;
    if (fread(&h, sizeof h, 1, f) != 1 || memcmp(h.magic, kMagic, 8) != 0 || h.n_rows < 0 || h.nnz < 0 ||
        !(h.val_bytes == 0 || h.val_bytes == 2 || h.val_bytes == 4)) {
        fclose(f);
        return fail(MPS_ERR_FORMAT, "%s: not a csr sidecar", path);
    }
    int32_t *rp = (int32_t *)malloc(4 * ((size_t)h.n_rows + 1));
    int32_t *col = (int32_t *)malloc(4 * ((size_t)h.nnz ? (size_t)h.nnz : 1));
    void *v = (h.val_bytes && val) ? malloc((size_t)h.val_bytes * ((size_t)h.nnz ? (size_t)h.nnz : 1)) : nullptr;
    bool ok = rp && col && (!(h.val_bytes && val) || v);
    ok = ok && fread(rp, 4, (size_t)h.n_rows + 1, f) == (size_t)h.n_rows + 1;
    ok = ok && (h.nnz == 0 || fread(col, 4, (size_t)h.nnz, f) == (size_t)h.nnz);
    if (ok && v) ok = h.nnz == 0 || fread(v, (size_t)h.val_bytes, (size_t)h.nnz, f) == (size_t)h.nnz;
    fclose(f);
    if (ok && (rp[0] != 0 || rp[h.n_rows] != h.nnz)) ok = false;
    if (!ok) { free(rp); free(col); free(v); return fail(MPS_ERR_FORMAT, "%s: truncated or inconsistent sidecar", path); }
    // the same checks the text loader applies: a damaged sidecar must not hand the kernels an index they would follow
    const long long bad_row = mps::first_decreasing_row(rp, h.n_rows, 0);
    const long long bad_col = bad_row >= 0 ? -1 : mps::first_bad_column(col, h.nnz, h.n_rows, 0);
    if (bad_row >= 0 || bad_col >= 0 || (long long)h.n_rows + 1 + h.nnz >= 1ll << 31) {
        int rc = bad_row >= 0 ? fail(MPS_ERR_FORMAT, "%s: row_ptr decreases at row %lld", path, bad_row)
               : bad_col >= 0 ? fail(MPS_ERR_FORMAT, "%s: col_idx[%lld] = %d outside [0, %d)", path, bad_col, col[bad_col], h.n_rows)
                              : fail(MPS_ERR_UNSUPPORTED, "%s: N+1+nnz does not fit 31 bits", path);
        free(rp); free(col); free(v);
        return rc;
    }
    out->n_rows = h.n_rows; out->nnz = h.nnz; out->row_ptr = rp; out->col_idx = col;
    if (val) *val = v;
    if (val_bytes) *val_bytes = v ? h.val_bytes : 0;
    return MPS_OK;
}
