// Host-side data formats either side of the SDDMM path: the Matrix Market loader,
// the column-sorted -> row-sorted conversion and the multi-GPU row partitioner.
// Pure host C++ (no CUDA), exported through the C ABI of include/sddmm_b200.h.
#include <algorithm>
#include <cctype>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <numeric>
#include <string>
#include <vector>

#include "mtx_holder.hpp"
#include "sddmm_b200.h"


namespace {

void set_err(char *buf, int len, const std::string &msg)
{
    if (buf && len > 0) {
        std::snprintf(buf, (size_t)len, "%s", msg.c_str());
    }
}

inline const char *skip_ws(const char *p, const char *end)
{
    while (p < end && (*p == ' ' || *p == '\t' || *p == '\r' || *p == '\n')) ++p;
    return p;
}
inline const char *skip_blank_in_line(const char *p, const char *end)
{
    while (p < end && (*p == ' ' || *p == '\t' || *p == '\r')) ++p;
    return p;
}

// Decimal integer; returns nullptr when no digits are present.
inline const char *parse_i64(const char *p, const char *end, int64_t *out)
{
    bool neg = false;
    if (p < end && (*p == '-' || *p == '+')) { neg = (*p == '-'); ++p; }
    if (p >= end || !std::isdigit((unsigned char)*p)) return nullptr;
    int64_t v = 0;
    while (p < end && std::isdigit((unsigned char)*p)) { v = v * 10 + (*p - '0'); ++p; }
    *out = neg ? -v : v;
    return p;
}

// Floating-point token -> float, same rounding as the reference's `fp >> float`
// (both end in strtof/strtod-quality conversion).
inline const char *parse_f32(const char *p, const char *end, float *out)
{
    char tmp[64];
    size_t n = 0;
    while (p + n < end && n < sizeof(tmp) - 1 && !std::isspace((unsigned char)p[n])) { tmp[n] = p[n]; ++n; }
    if (n == 0) return nullptr;
    tmp[n] = 0;
    char *e = nullptr;
    errno = 0;
    float v = std::strtof(tmp, &e);
    if (e == tmp || *e != 0) return nullptr;
    *out = v;
    return p + n;
}

// ---- binary form of a COO matrix: header, rows, cols, [vals]; little-endian ----
const char BIN_MAGIC[8] = {'S', 'D', 'D', 'M', 'M', 'C', 'O', 'O'};
struct BinHeader {
    char magic[8];
    uint32_t version, flags;  // flags bit 0: values present
    int64_t M, N, nnz;
    uint64_t checksum;        // over rows, cols, vals as stored
};
static_assert(sizeof(BinHeader) == 48, "binary header layout");

// 64-bit multiply-xorshift over 8-byte words (tail bytes zero-extended), chained through `h`.
uint64_t checksum(uint64_t h, const void *data, size_t bytes)
{
    const unsigned char *p = (const unsigned char *)data;
    size_t i = 0;
    for (; i + 8 <= bytes; i += 8) {
        uint64_t w;
        std::memcpy(&w, p + i, 8);
        h = (h ^ w) * 0x9E3779B97F4A7C15ull;
        h ^= h >> 29;
    }
    if (i < bytes) {
        uint64_t w = 0;
        std::memcpy(&w, p + i, bytes - i);
        h = (h ^ w) * 0x9E3779B97F4A7C15ull;
        h ^= h >> 29;
    }
    return h;
}

// `f` is positioned after the magic.
int load_binary(FILE *f, sddmm_mtx_s **out, char *errbuf, int errbuf_len)
{
    BinHeader h;
    if (std::fread((char *)&h + 8, sizeof(h) - 8, 1, f) != 1) {
        set_err(errbuf, errbuf_len, "binary matrix: truncated header");
        return SDDMM_PARSE_ERROR;
    }
    if (h.version != 1 || h.M < 0 || h.N < 0 || h.nnz < 0 || h.M > INT32_MAX || h.N > INT32_MAX || h.nnz >= INT32_MAX) {
        set_err(errbuf, errbuf_len, "binary matrix: unsupported version or sizes out of range");
        return SDDMM_PARSE_ERROR;
    }
    sddmm_mtx_s *mx = new (std::nothrow) sddmm_mtx_s;
    if (!mx) return SDDMM_OUT_OF_MEMORY;
    mx->M = h.M; mx->N = h.N; mx->nnz = h.nnz;
    const size_t z = (size_t)h.nnz;
    try {
        mx->rows.resize(z);
        mx->cols.resize(z);
        mx->vals.assign(z, 1.0f);
    } catch (...) {
        delete mx;
        return SDDMM_OUT_OF_MEMORY;
    }
    bool ok = z == 0 || std::fread(mx->rows.data(), sizeof(int32_t), z, f) == z;
    ok = ok && (z == 0 || std::fread(mx->cols.data(), sizeof(int32_t), z, f) == z);
    if (h.flags & 1u) ok = ok && (z == 0 || std::fread(mx->vals.data(), sizeof(float), z, f) == z);
    if (!ok) {
        set_err(errbuf, errbuf_len, "binary matrix: truncated payload");
        delete mx;
        return SDDMM_PARSE_ERROR;
    }
    uint64_t sum = 0;
    sum = checksum(sum, mx->rows.data(), sizeof(int32_t) * z);
    sum = checksum(sum, mx->cols.data(), sizeof(int32_t) * z);
    if (h.flags & 1u) sum = checksum(sum, mx->vals.data(), sizeof(float) * z);
    if (sum != h.checksum) {
        set_err(errbuf, errbuf_len, "binary matrix: checksum mismatch");
        delete mx;
        return SDDMM_PARSE_ERROR;
    }
    for (size_t i = 0; i < z; ++i)
        if (mx->rows[i] < 0 || mx->rows[i] >= h.M || mx->cols[i] < 0 || mx->cols[i] >= h.N) {
            set_err(errbuf, errbuf_len, "binary matrix: index out of range");
            delete mx;
            return SDDMM_INDEX_OUT_OF_RANGE;
        }
    *out = mx;
    return SDDMM_OK;
}

// What the open flags ask for after the triples are in memory.
int finish_open(sddmm_mtx_s *mx, uint32_t flags, int symmetric, char *errbuf, int errbuf_len)
{
    try {
        if ((flags & SDDMM_MTX_EXPAND_SYMMETRIC) && symmetric != 0) {
            // a symmetric file stores one triangle: add the mirror image of every off-diagonal entry
            if (mx->M != mx->N) {
                set_err(errbuf, errbuf_len, "a symmetric matrix must be square");
                return SDDMM_PARSE_ERROR;
            }
            const size_t z = (size_t)mx->nnz;
            size_t extra = 0;
            for (size_t i = 0; i < z; ++i) extra += mx->rows[i] != mx->cols[i];
            if (z + extra >= (size_t)INT32_MAX) {
                set_err(errbuf, errbuf_len, "matrix too large for 32-bit indices once expanded");
                return SDDMM_PARSE_ERROR;
            }
            mx->rows.reserve(z + extra);
            mx->cols.reserve(z + extra);
            mx->vals.reserve(z + extra);
            for (size_t i = 0; i < z; ++i)
                if (mx->rows[i] != mx->cols[i]) {
                    mx->rows.push_back(mx->cols[i]);
                    mx->cols.push_back(mx->rows[i]);
                    mx->vals.push_back(symmetric < 0 ? -mx->vals[i] : mx->vals[i]);
                }
            mx->nnz = (int64_t)(z + extra);
        }
        if (flags & SDDMM_MTX_SORT_ROWS) {
            bool sorted = true;
            for (int64_t i = 1; i < mx->nnz && sorted; ++i)
                sorted = mx->rows[(size_t)i - 1] < mx->rows[(size_t)i] ||
                         (mx->rows[(size_t)i - 1] == mx->rows[(size_t)i] && mx->cols[(size_t)i - 1] <= mx->cols[(size_t)i]);
            if (!sorted) {
                const int st = sddmm_coo_sort_rows(&mx->M, &mx->N, mx->nnz, mx->rows.data(), mx->cols.data(),
                                                   mx->vals.data(), 0);
                if (st != SDDMM_OK) return st;
            }
        }
    } catch (const std::bad_alloc &) {
        return SDDMM_OUT_OF_MEMORY;
    }
    return SDDMM_OK;
}

}  // namespace

extern "C" {

int sddmm_mtx_open(const char *path, sddmm_mtx_t *out, int64_t *M, int64_t *N, int64_t *nnz, char *errbuf,
                   int errbuf_len)
{
    return sddmm_mtx_open_ex(path, 0u, out, M, N, nnz, errbuf, errbuf_len);
}

int sddmm_mtx_open_ex(const char *path, uint32_t flags, sddmm_mtx_t *out, int64_t *M, int64_t *N, int64_t *nnz,
                      char *errbuf, int errbuf_len)
{
    if (!path || !out) return SDDMM_INVALID_ARG;
    *out = nullptr;
    FILE *f = std::fopen(path, "rb");
    if (!f) {
        set_err(errbuf, errbuf_len, std::string("cannot open ") + path + ": " + std::strerror(errno));
        return SDDMM_IO_ERROR;
    }
    {
        // the binary form written by sddmm_coo_save_binary is recognised by its first eight bytes
        char magic[8] = {0};
        const size_t got = std::fread(magic, 1, 8, f);
        if (got == 8 && std::memcmp(magic, BIN_MAGIC, 8) == 0) {
            sddmm_mtx_s *mx = nullptr;
            int st = load_binary(f, &mx, errbuf, errbuf_len);
            std::fclose(f);
            if (st != SDDMM_OK) return st;
            st = finish_open(mx, flags, /*symmetric*/0, errbuf, errbuf_len);
            if (st != SDDMM_OK) { delete mx; return st; }
            if (M) *M = mx->M;
            if (N) *N = mx->N;
            if (nnz) *nnz = mx->nnz;
            *out = mx;
            return SDDMM_OK;
        }
        std::fseek(f, 0, SEEK_SET);
    }
    std::vector<char> text;
    {
        std::fseek(f, 0, SEEK_END);
        long sz = std::ftell(f);
        std::fseek(f, 0, SEEK_SET);
        if (sz < 0) { std::fclose(f); return SDDMM_IO_ERROR; }
        text.resize((size_t)sz);
        size_t got = sz ? std::fread(text.data(), 1, (size_t)sz, f) : 0;
        std::fclose(f);
        if (got != (size_t)sz) {
            set_err(errbuf, errbuf_len, "short read");
            return SDDMM_IO_ERROR;
        }
    }
    const char *p = text.data(), *end = p + text.size();

    // Banner and comments.  The reference skips every line until one whose first
    // character is a digit (sddmm.cu:257-261); here a line is skipped when it is
    // empty or starts with '%', and the banner's field / symmetry words are read.
    bool pattern = false;
    int symmetric = 0;  // 0 general, +1 symmetric (or hermitian), -1 skew-symmetric
    while (true) {
        p = skip_ws(p, end);
        if (p >= end) {
            set_err(errbuf, errbuf_len, "no size line found");
            return SDDMM_PARSE_ERROR;
        }
        if (*p != '%') break;
        const char *eol = (const char *)std::memchr(p, '\n', (size_t)(end - p));
        if (!eol) eol = end;
        if (end - p >= 14 && std::strncmp(p, "%%MatrixMarket", 14) == 0) {
            std::string line(p, eol);
            std::transform(line.begin(), line.end(), line.begin(), [](unsigned char c) { return (char)std::tolower(c); });
            if (line.find("coordinate") == std::string::npos) {
                set_err(errbuf, errbuf_len, "only 'coordinate' Matrix Market files are supported");
                return SDDMM_PARSE_ERROR;
            }
            if (line.find("complex") != std::string::npos) {
                set_err(errbuf, errbuf_len, "complex matrices are not supported");
                return SDDMM_PARSE_ERROR;
            }
            pattern = line.find("pattern") != std::string::npos;
            if (line.find("skew-symmetric") != std::string::npos) symmetric = -1;
            else if (line.find("symmetric") != std::string::npos || line.find("hermitian") != std::string::npos) symmetric = 1;
        }
        p = eol;
    }

    int64_t m = 0, n = 0, z = 0;
    const char *q = parse_i64(p, end, &m);
    // the three sizes may sit on one line (Matrix Market) or on three (headerless bag-of-words
    // "docword" files: documents, words, entries) -- the reference's other readers take both
    // (`fp >> n_rows >> n_cols >> nnz`, other_ideas/our_work/sparse_dense_split/sddmm.cu:356)
    if (q) q = parse_i64(skip_ws(q, end), end, &n);
    if (q) q = parse_i64(skip_ws(q, end), end, &z);
    if (!q || m < 0 || n < 0 || z < 0) {
        set_err(errbuf, errbuf_len, "malformed size line (expected: rows cols nnz)");
        return SDDMM_PARSE_ERROR;
    }
    if (m > INT32_MAX || n > INT32_MAX || z >= INT32_MAX) {
        set_err(errbuf, errbuf_len, "matrix too large for 32-bit indices");
        return SDDMM_PARSE_ERROR;
    }
    p = q;

    sddmm_mtx_s *mx = new (std::nothrow) sddmm_mtx_s;
    if (!mx) return SDDMM_OUT_OF_MEMORY;
    mx->M = m; mx->N = n; mx->nnz = z;
    try {
        mx->rows.resize((size_t)z);
        mx->cols.resize((size_t)z);
        mx->vals.resize((size_t)z);
    } catch (...) {
        delete mx;
        return SDDMM_OUT_OF_MEMORY;
    }
    for (int64_t i = 0; i < z; ++i) {
        int64_t r = 0, c = 0;
        float v = 1.0f;
        p = skip_ws(p, end);
        const char *t = parse_i64(p, end, &r);
        if (t) t = parse_i64(skip_blank_in_line(t, end), end, &c);
        if (t && !pattern) {
            const char *u = skip_blank_in_line(t, end);
            // a missing value column is what the reference mis-parses silently
            t = (u < end && *u != '\n') ? parse_f32(u, end, &v) : nullptr;
        }
        if (!t) {
            char msg[128];
            std::snprintf(msg, sizeof(msg), "malformed or missing entry %lld of %lld", (long long)(i + 1), (long long)z);
            set_err(errbuf, errbuf_len, msg);
            delete mx;
            return SDDMM_PARSE_ERROR;
        }
        if (r < 1 || r > m || c < 1 || c > n) {
            char msg[128];
            std::snprintf(msg, sizeof(msg), "entry %lld: index (%lld,%lld) outside %lld x %lld", (long long)(i + 1),
                          (long long)r, (long long)c, (long long)m, (long long)n);
            set_err(errbuf, errbuf_len, msg);
            delete mx;
            return SDDMM_INDEX_OUT_OF_RANGE;
        }
        mx->rows[(size_t)i] = (int32_t)(r - 1);  // 1-based -> 0-based, sddmm.cu:277-278
        mx->cols[(size_t)i] = (int32_t)(c - 1);
        mx->vals[(size_t)i] = v;
        p = t;
    }
    {
        const int st = finish_open(mx, flags, symmetric, errbuf, errbuf_len);
        if (st != SDDMM_OK) { delete mx; return st; }
    }
    if (M) *M = mx->M;
    if (N) *N = mx->N;
    if (nnz) *nnz = mx->nnz;
    *out = mx;
    return SDDMM_OK;
}

int sddmm_coo_save_binary(const char *path, int64_t M, int64_t N, int64_t nnz, const int32_t *rows, const int32_t *cols,
                          const float *vals)
{
    if (!path || M < 0 || N < 0 || nnz < 0 || (nnz > 0 && (!rows || !cols))) return SDDMM_INVALID_ARG;
    FILE *f = std::fopen(path, "wb");
    if (!f) return SDDMM_IO_ERROR;
    BinHeader h;
    std::memcpy(h.magic, BIN_MAGIC, 8);
    h.version = 1;
    h.flags = vals ? 1u : 0u;
    h.M = M; h.N = N; h.nnz = nnz;
    uint64_t sum = 0;
    sum = checksum(sum, rows, sizeof(int32_t) * (size_t)nnz);
    sum = checksum(sum, cols, sizeof(int32_t) * (size_t)nnz);
    if (vals) sum = checksum(sum, vals, sizeof(float) * (size_t)nnz);
    h.checksum = sum;
    bool ok = std::fwrite(&h, sizeof(h), 1, f) == 1;
    ok = ok && (nnz == 0 || std::fwrite(rows, sizeof(int32_t), (size_t)nnz, f) == (size_t)nnz);
    ok = ok && (nnz == 0 || std::fwrite(cols, sizeof(int32_t), (size_t)nnz, f) == (size_t)nnz);
    ok = ok && (nnz == 0 || !vals || std::fwrite(vals, sizeof(float), (size_t)nnz, f) == (size_t)nnz);
    ok = (std::fclose(f) == 0) && ok;
    return ok ? SDDMM_OK : SDDMM_IO_ERROR;
}

int sddmm_mtx_read(sddmm_mtx_t f, int32_t *rows, int32_t *cols, float *vals)
{
    if (!f) return SDDMM_INVALID_ARG;
    const size_t z = (size_t)f->nnz;
    if (rows && z) std::memcpy(rows, f->rows.data(), z * sizeof(int32_t));
    if (cols && z) std::memcpy(cols, f->cols.data(), z * sizeof(int32_t));
    if (vals && z) std::memcpy(vals, f->vals.data(), z * sizeof(float));
    return sddmm_mtx_close(f);
}

int sddmm_mtx_close(sddmm_mtx_t f)
{
    delete f;
    return SDDMM_OK;
}

int sddmm_coo_is_row_sorted(int64_t nnz, const int32_t *rows)
{
    for (int64_t i = 1; i < nnz; ++i)
        if (rows[i - 1] > rows[i]) return 0;
    return 1;
}

int sddmm_mtx_write(const char *path, int64_t M, int64_t N, int64_t nnz, const int32_t *rows, const int32_t *cols,
                    const float *vals)
{
    if (!path || (nnz > 0 && (!rows || !cols))) return SDDMM_INVALID_ARG;
    FILE *f = std::fopen(path, "wb");
    if (!f) return SDDMM_IO_ERROR;
    std::fprintf(f, "%%%%MatrixMarket matrix coordinate real general\n%lld %lld %lld\n", (long long)M, (long long)N,
                 (long long)nnz);
    for (int64_t i = 0; i < nnz; ++i)
        std::fprintf(f, "%d %d %.9g\n", rows[i] + 1, cols[i] + 1, vals ? (double)vals[i] : 1.0);
    return std::fclose(f) == 0 ? SDDMM_OK : SDDMM_IO_ERROR;
}

int sddmm_coo_sort_rows(int64_t *M, int64_t *N, int64_t nnz, int32_t *rows, int32_t *cols, float *vals, int transpose)
{
    if (!M || !N || nnz < 0 || (nnz > 0 && (!rows || !cols || !vals))) return SDDMM_INVALID_ARG;
    struct Triple { int32_t a, b; float v; };
    std::vector<Triple> items;
    try {
        items.resize((size_t)nnz);
    } catch (...) {
        return SDDMM_OUT_OF_MEMORY;
    }
    for (int64_t i = 0; i < nnz; ++i) {
        items[(size_t)i].a = transpose ? cols[i] : rows[i];
        items[(size_t)i].b = transpose ? rows[i] : cols[i];
        items[(size_t)i].v = vals[i];
    }
    if (transpose) {
        // the reference sorts whole (col,row,val) tuples (util.h:88-95)
        std::sort(items.begin(), items.end(), [](const Triple &x, const Triple &y) {
            if (x.a != y.a) return x.a < y.a;
            if (x.b != y.b) return x.b < y.b;
            return x.v < y.v;
        });
    } else {
        std::stable_sort(items.begin(), items.end(), [](const Triple &x, const Triple &y) {
            if (x.a != y.a) return x.a < y.a;
            return x.b < y.b;
        });
    }
    for (int64_t i = 0; i < nnz; ++i) {
        rows[i] = items[(size_t)i].a;
        cols[i] = items[(size_t)i].b;
        vals[i] = items[(size_t)i].v;
    }
    if (transpose) std::swap(*M, *N);
    return SDDMM_OK;
}

int sddmm_partition_rows(int64_t M, int64_t nnz, const int32_t *rows, int n_parts, int align_rows, int64_t *cuts,
                         int64_t *nnz_cuts)
{
    return sddmm_partition_rows_weighted(M, nnz, rows, n_parts, align_rows, 0.0, cuts, nnz_cuts);
}

int sddmm_partition_rows_shares(int64_t M, int64_t nnz, const int32_t *rows, int n_parts, int align_rows,
                                const double *shares, int64_t *cuts, int64_t *nnz_cuts)
{
    if (!shares) return sddmm_partition_rows(M, nnz, rows, n_parts, align_rows, cuts, nnz_cuts);
    if (M < 0 || nnz < 0 || n_parts < 1 || !cuts || (nnz > 0 && !rows)) return SDDMM_INVALID_ARG;
    if (align_rows < 1) align_rows = 1;
    double total = 0;
    for (int g = 0; g < n_parts; ++g) {
        if (!(shares[g] >= 0)) return SDDMM_INVALID_ARG;
        total += shares[g];
    }
    if (!(total > 0)) return SDDMM_INVALID_ARG;
    cuts[0] = 0;
    double acc = 0;
    for (int g = 1; g < n_parts; ++g) {
        acc += shares[g - 1];
        int64_t target = (int64_t)((double)nnz * (acc / total));
        if (target > nnz) target = nnz;
        int64_t r = target > 0 ? (int64_t)rows[target - 1] + 1 : 0;
        r = ((r + align_rows - 1) / align_rows) * align_rows;
        if (r > M) r = M;
        if (r < cuts[g - 1]) r = cuts[g - 1];
        cuts[g] = r;
    }
    cuts[n_parts] = M;
    if (nnz_cuts) {
        for (int g = 0; g <= n_parts; ++g) {
            const int32_t *lb = std::lower_bound(rows, rows + nnz, cuts[g], [](int32_t a, int64_t b) { return (int64_t)a < b; });
            nnz_cuts[g] = (int64_t)(lb - rows);
        }
    }
    return SDDMM_OK;
}

int sddmm_partition_rows_weighted(int64_t M, int64_t nnz, const int32_t *rows, int n_parts, int align_rows,
                                  double row_cost, int64_t *cuts, int64_t *nnz_cuts)
{
    if (M < 0 || nnz < 0 || n_parts < 1 || !cuts || (nnz > 0 && !rows) || row_cost < 0) return SDDMM_INVALID_ARG;
    if (align_rows < 1) align_rows = 1;
    cuts[0] = 0;
    if (row_cost == 0.0) {
        for (int g = 1; g < n_parts; ++g) {
            const int64_t target = (int64_t)(((__int128)nnz * g) / n_parts);
            // smallest row r whose prefix (nonzeros in rows < r) reaches the target
            int64_t r = target > 0 ? (int64_t)rows[target - 1] + 1 : 0;
            r = ((r + align_rows - 1) / align_rows) * align_rows;
            if (r > M) r = M;
            if (r < cuts[g - 1]) r = cuts[g - 1];
            cuts[g] = r;
        }
    } else {
        // cost of a prefix = its nonzeros + row_cost per non-empty row in it
        int64_t n_rows_ne = 0;
        for (int64_t i = 0; i < nnz; ++i) n_rows_ne += (i == 0 || rows[i] != rows[i - 1]);
        const double total = (double)nnz + row_cost * (double)n_rows_ne;
        int g = 1;
        double acc = 0;
        for (int64_t i = 0; i < nnz && g < n_parts; ++i) {
            acc += 1.0 + ((i == 0 || rows[i] != rows[i - 1]) ? row_cost : 0.0);
            while (g < n_parts && acc >= total * g / n_parts) {
                int64_t r = (int64_t)rows[i] + 1;
                r = ((r + align_rows - 1) / align_rows) * align_rows;
                if (r > M) r = M;
                if (r < cuts[g - 1]) r = cuts[g - 1];
                cuts[g++] = r;
            }
        }
        for (; g < n_parts; ++g) cuts[g] = cuts[g - 1] > 0 ? cuts[g - 1] : 0;
    }
    cuts[n_parts] = M;
    if (nnz_cuts) {
        for (int g = 0; g <= n_parts; ++g) {
            const int32_t *lb = std::lower_bound(rows, rows + nnz, cuts[g],
                                                 [](int32_t a, int64_t b) { return (int64_t)a < b; });
            nnz_cuts[g] = (int64_t)(lb - rows);
        }
    }
    return SDDMM_OK;
}

}  // extern "C"
