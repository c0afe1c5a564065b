// Seeded synthetic sparse matrices (host), row-sorted COO, for the command line's
// "gen:" inputs and for benchmarks without a dataset.  The reference ships no
// matrix (its dataset/ folder is empty and its scripts name public corpora and
// graphs); these generators produce matrices with the shapes, sizes and value
// distributions of the benchmark configurations, never a record of any dataset.
//
// One counter-based generator serves everything: value = mix(seed, stream, index),
// so a matrix depends only on its spec and seed, not on thread count or order.
//
//   uniform:M:N:density      floor(density*M*N) distinct cells, uniform; values 1
//   zipf:M:N:nnz             row lengths ~ Zipf(1.1) over a random row order, scaled to
//                            hit nnz exactly; columns without replacement with
//                            popularity ~ Zipf(1.0); values integer 1..20
//   rmat:scale:edge_factor   R-MAT (0.57, 0.19, 0.19, 0.05), edge_factor * 2^scale draws,
//                            duplicates removed; values normal(0, 1)
//   band:M:half_width:g      |i - j| <= half_width plus g full rows and g full columns
//                            at seeded positions; values 1
//   c1 .. c5                 the five benchmark configurations (with their seeds)
// An optional trailing ":seed=S" overrides the seed.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <numeric>
#include <string>
#include <thread>
#include <vector>

#include "mtx_holder.hpp"
#include "sddmm_b200.h"

namespace {

inline uint64_t mix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
struct Rng {
    uint64_t key;
    Rng(uint64_t seed, uint64_t stream) : key(mix64(seed ^ mix64(stream * 0xD1342543DE82EF95ull + 1))) {}
    uint64_t u64(uint64_t i) const { return mix64(key + i * 0x9E3779B97F4A7C15ull); }
    double u01(uint64_t i) const { return (double)(u64(i) >> 11) * (1.0 / 9007199254740992.0); }  // [0, 1)
};
enum Stream : uint64_t { S_STRUCT = 3, S_VALUES = 4, S_PERM = 5, S_GLOBAL = 6 };

enum class Vals { One, Int20, Normal };

void set_err(char *buf, int len, const std::string &msg)
{
    if (buf && len > 0) std::snprintf(buf, (size_t)len, "%s", msg.c_str());
}

std::vector<std::string> split(const std::string &s, char sep)
{
    std::vector<std::string> out;
    size_t a = 0;
    while (true) {
        size_t b = s.find(sep, a);
        out.push_back(s.substr(a, b == std::string::npos ? b : b - a));
        if (b == std::string::npos) break;
        a = b + 1;
    }
    return out;
}

void fill_values(sddmm_mtx_s &m, Vals kind, uint64_t seed)
{
    const Rng r(seed, S_VALUES);
    m.vals.resize((size_t)m.nnz);
    for (int64_t i = 0; i < m.nnz; ++i) {
        float v = 1.0f;
        if (kind == Vals::Int20) {
            v = (float)(1 + (int)(r.u64((uint64_t)i) % 20));
        } else if (kind == Vals::Normal) {  // Box-Muller on two counter-based uniforms
            const double u1 = 1.0 - r.u01(2 * (uint64_t)i), u2 = r.u01(2 * (uint64_t)i + 1);
            v = (float)(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
        }
        m.vals[(size_t)i] = v;
    }
}

void keys_to_coo(const std::vector<uint64_t> &keys, sddmm_mtx_s &m)
{
    m.nnz = (int64_t)keys.size();
    m.rows.resize(keys.size());
    m.cols.resize(keys.size());
    for (size_t i = 0; i < keys.size(); ++i) {
        m.rows[i] = (int32_t)(keys[i] >> 32);
        m.cols[i] = (int32_t)(keys[i] & 0xffffffffu);
    }
}

// floor(density * M * N) distinct cells: draw, sort, dedup, top up until enough, then
// drop the surplus cells with the largest hash (keeps the choice uniform and seeded).
int gen_uniform(int64_t M, int64_t N, double density, uint64_t seed, sddmm_mtx_s &m)
{
    const double cells = (double)M * (double)N;
    const int64_t target = (int64_t)std::floor(density * cells);
    if (target < 0 || (double)target > cells || target >= INT32_MAX) return SDDMM_INVALID_ARG;
    const Rng r(seed, S_STRUCT);
    const uint64_t total = (uint64_t)M * (uint64_t)N;
    // more than half of the cells: draw the cells that stay EMPTY instead (drawing without replacement by
    // rejection slows down as the matrix fills up)
    const bool complement = (uint64_t)target * 2 > total;
    const int64_t want_cells = complement ? (int64_t)(total - (uint64_t)target) : target;
    std::vector<uint64_t> keys;  // linear cell ids, sorted, distinct
    uint64_t drawn = 0;
    while ((int64_t)keys.size() < want_cells) {
        const uint64_t want = (uint64_t)(want_cells - (int64_t)keys.size());
        const uint64_t batch = want + want / 16 + 16;
        for (uint64_t i = 0; i < batch; ++i) keys.push_back(r.u64(drawn++) % total);
        std::sort(keys.begin(), keys.end());
        keys.erase(std::unique(keys.begin(), keys.end()), keys.end());
    }
    if ((int64_t)keys.size() > want_cells) {
        // drop the surplus cells with the largest hash: keeps the choice uniform and seeded
        std::vector<std::pair<uint64_t, uint64_t>> h(keys.size());
        for (size_t i = 0; i < keys.size(); ++i) h[i] = {mix64(keys[i] ^ seed), keys[i]};
        std::nth_element(h.begin(), h.begin() + want_cells, h.end());
        keys.resize((size_t)want_cells);
        for (int64_t i = 0; i < want_cells; ++i) keys[(size_t)i] = h[(size_t)i].second;
        std::sort(keys.begin(), keys.end());
    }
    if (complement) {
        std::vector<uint64_t> kept;
        kept.reserve((size_t)target);
        size_t j = 0;
        for (uint64_t c = 0; c < total; ++c) {
            if (j < keys.size() && keys[j] == c) { ++j; continue; }
            kept.push_back(c);
        }
        keys.swap(kept);
    }
    for (auto &c : keys) c = ((c / (uint64_t)N) << 32) | (c % (uint64_t)N);  // row-major cell id -> (row, col) key, order kept
    keys_to_coo(keys, m);
    return SDDMM_OK;
}

int gen_zipf(int64_t M, int64_t N, int64_t nnz, uint64_t seed, sddmm_mtx_s &m)
{
    if (nnz > M * N || nnz >= INT32_MAX) return SDDMM_INVALID_ARG;
    // row lengths: Zipf(1.1) weights over a seeded random order of the rows
    std::vector<int64_t> order((size_t)M);
    std::iota(order.begin(), order.end(), 0);
    const Rng rp(seed, S_PERM);
    for (int64_t i = M - 1; i > 0; --i) std::swap(order[(size_t)i], order[(size_t)(rp.u64((uint64_t)i) % (uint64_t)(i + 1))]);
    std::vector<double> w((size_t)M);
    double wsum = 0;
    for (int64_t i = 0; i < M; ++i) wsum += (w[(size_t)i] = std::pow((double)(i + 1), -1.1));
    std::vector<int64_t> len((size_t)M);
    int64_t have = 0;
    for (int64_t i = 0; i < M; ++i) {
        int64_t l = (int64_t)std::llround(w[(size_t)i] / wsum * (double)nnz);
        if (l > N) l = N;
        len[(size_t)order[(size_t)i]] = l;
        have += l;
    }
    // hit nnz exactly: walk the rows from the heaviest rank, one nonzero at a time
    for (int64_t pass = 0; have != nnz && pass < 4 * (N + 1); ++pass)
        for (int64_t i = 0; i < M && have != nnz; ++i) {
            int64_t &l = len[(size_t)order[(size_t)i]];
            if (have < nnz && l < N) { ++l; ++have; }
            else if (have > nnz && l > 0) { --l; --have; }
        }
    if (have != nnz) return SDDMM_INVALID_ARG;
    // columns of a row: weighted sampling without replacement (smallest exponential keys win)
    std::vector<double> cw((size_t)N);
    for (int64_t c = 0; c < N; ++c) cw[(size_t)c] = (double)(c + 1);  // 1 / weight of Zipf(1.0)
    m.rows.resize((size_t)nnz);
    m.cols.resize((size_t)nnz);
    const Rng rs(seed, S_STRUCT);
    std::vector<std::pair<double, int32_t>> key((size_t)N);
    int64_t out = 0;
    for (int64_t r = 0; r < M; ++r) {
        const int64_t l = len[(size_t)r];
        if (l == 0) continue;
        for (int64_t c = 0; c < N; ++c) {
            const double u = 1.0 - rs.u01((uint64_t)r * (uint64_t)N + (uint64_t)c);
            key[(size_t)c] = {-std::log(u) * cw[(size_t)c], (int32_t)c};
        }
        if (l < N) std::nth_element(key.begin(), key.begin() + l, key.end());
        std::vector<int32_t> chosen((size_t)l);
        for (int64_t j = 0; j < l; ++j) chosen[(size_t)j] = key[(size_t)j].second;
        std::sort(chosen.begin(), chosen.end());
        for (int64_t j = 0; j < l; ++j) {
            m.rows[(size_t)out] = (int32_t)r;
            m.cols[(size_t)out] = chosen[(size_t)j];
            ++out;
        }
    }
    m.nnz = nnz;
    return SDDMM_OK;
}

int gen_rmat(int scale, int64_t edge_factor, uint64_t seed, sddmm_mtx_s &m)
{
    if (scale < 1 || scale > 30 || edge_factor < 1) return SDDMM_INVALID_ARG;
    const int64_t n = (int64_t)1 << scale;
    const int64_t E = edge_factor * n;
    if (E >= INT32_MAX) return SDDMM_INVALID_ARG;
    std::vector<uint64_t> keys((size_t)E);
    const Rng r(seed, S_STRUCT);
    // quadrant thresholds on 16 bits: a, a+b, a+b+c of (0.57, 0.19, 0.19, 0.05)
    const uint32_t ta = (uint32_t)(0.57 * 65536), tb = (uint32_t)(0.76 * 65536), tc = (uint32_t)(0.95 * 65536);
    const int words = (scale + 3) / 4;  // four levels per 64-bit word
    auto work = [&](int64_t e0, int64_t e1) {
        for (int64_t e = e0; e < e1; ++e) {
            uint64_t row = 0, col = 0;
            int level = 0;
            for (int wi = 0; wi < words; ++wi) {
                uint64_t bits = r.u64((uint64_t)e * (uint64_t)words + (uint64_t)wi);
                for (int j = 0; j < 4 && level < scale; ++j, ++level, bits >>= 16) {
                    const uint32_t u = (uint32_t)(bits & 0xffffu);
                    const uint64_t rb = u >= tb ? 1 : 0;                       // quadrants c, d: lower half
                    const uint64_t cb = (u >= ta && u < tb) || u >= tc ? 1 : 0;  // quadrants b, d: right half
                    row = (row << 1) | rb;
                    col = (col << 1) | cb;
                }
            }
            keys[(size_t)e] = (row << 32) | col;
        }
    };
    unsigned nt = std::thread::hardware_concurrency();
    if (nt == 0) nt = 1;
    if (nt > 32) nt = 32;
    std::vector<std::thread> pool;
    for (unsigned t = 0; t < nt; ++t) pool.emplace_back(work, E * t / nt, E * (t + 1) / nt);
    for (auto &t : pool) t.join();
    std::sort(keys.begin(), keys.end());
    keys.erase(std::unique(keys.begin(), keys.end()), keys.end());
    keys_to_coo(keys, m);
    return SDDMM_OK;
}

int gen_band(int64_t M, int64_t hw, int64_t g, uint64_t seed, sddmm_mtx_s &m)
{
    if (hw < 0 || g < 0 || g > M) return SDDMM_INVALID_ARG;
    // g distinct global indices for rows, g for columns (seeded partial shuffles)
    auto pick = [&](uint64_t stream) {
        std::vector<char> mark((size_t)M, 0);
        const Rng r(seed, stream);
        int64_t got = 0;
        for (uint64_t i = 0; got < g; ++i) {
            const int64_t v = (int64_t)(r.u64(i) % (uint64_t)M);
            if (!mark[(size_t)v]) { mark[(size_t)v] = 1; ++got; }
        }
        return mark;
    };
    const std::vector<char> grow = pick(S_GLOBAL), gcol = pick(S_GLOBAL + 1);
    std::vector<int32_t> gcols;
    for (int64_t c = 0; c < M; ++c) if (gcol[(size_t)c]) gcols.push_back((int32_t)c);
    int64_t nnz = 0;
    for (int pass = 0; pass < 2; ++pass) {
        int64_t out = 0;
        for (int64_t i = 0; i < M; ++i) {
            const int64_t lo = std::max<int64_t>(0, i - hw), hi = std::min<int64_t>(M - 1, i + hw);
            if (grow[(size_t)i]) {
                if (pass) for (int64_t c = 0; c < M; ++c) { m.rows[(size_t)out] = (int32_t)i; m.cols[(size_t)out] = (int32_t)c; ++out; }
                else out += M;
                continue;
            }
            // global columns left of the band, the band, global columns right of it
            size_t gi = 0;
            for (; gi < gcols.size() && gcols[gi] < lo; ++gi) {
                if (pass) { m.rows[(size_t)out] = (int32_t)i; m.cols[(size_t)out] = gcols[gi]; }
                ++out;
            }
            for (int64_t c = lo; c <= hi; ++c) {
                if (pass) { m.rows[(size_t)out] = (int32_t)i; m.cols[(size_t)out] = (int32_t)c; }
                ++out;
            }
            for (; gi < gcols.size(); ++gi) {
                if (gcols[gi] <= hi) continue;
                if (pass) { m.rows[(size_t)out] = (int32_t)i; m.cols[(size_t)out] = gcols[gi]; }
                ++out;
            }
        }
        if (!pass) {
            if (out >= INT32_MAX) return SDDMM_INVALID_ARG;
            nnz = out;
            m.rows.resize((size_t)nnz);
            m.cols.resize((size_t)nnz);
        }
    }
    m.nnz = nnz;
    return SDDMM_OK;
}

bool to_i64(const std::string &s, int64_t *v)
{
    if (s.empty()) return false;
    char *end = nullptr;
    const long long x = std::strtoll(s.c_str(), &end, 10);
    if (*end) return false;
    *v = x;
    return true;
}
bool to_f64(const std::string &s, double *v)
{
    if (s.empty()) return false;
    char *end = nullptr;
    const double x = std::strtod(s.c_str(), &end);
    if (*end) return false;
    *v = x;
    return true;
}

}  // namespace

extern "C" int sddmm_gen_open(const char *spec, sddmm_mtx_t *out, int64_t *M, int64_t *N, int64_t *nnz, char *err,
                              int err_len)
{
    if (!spec || !out || !M || !N || !nnz) return SDDMM_INVALID_ARG;
    *out = nullptr;
    std::string s(spec);
    static const struct { const char *name, *spec; uint64_t seed; } presets[] = {
        {"c1", "uniform:4096:4096:0.001", 1001}, {"c2", "zipf:12419:1500:746316", 1002}, {"c3", "rmat:20:16", 1003},
        {"c4", "rmat:22:24", 1004},              {"c5", "band:65536:256:80", 1005},
    };
    std::vector<std::string> f = split(s, ':');
    uint64_t seed = 1;
    bool seed_given = false;
    if (!f.empty() && f.back().rfind("seed=", 0) == 0) {
        int64_t v = 0;
        if (!to_i64(f.back().substr(5), &v) || v < 0) {
            set_err(err, err_len, "bad seed in '" + s + "'");
            return SDDMM_INVALID_ARG;
        }
        seed = (uint64_t)v;
        seed_given = true;
        f.pop_back();
    }
    if (f.size() == 1)
        for (const auto &p : presets)
            if (f[0] == p.name) {
                f = split(p.spec, ':');
                if (!seed_given) seed = p.seed;
                break;
            }
    sddmm_mtx_s *m = new (std::nothrow) sddmm_mtx_s;
    if (!m) return SDDMM_OUT_OF_MEMORY;
    int st = SDDMM_INVALID_ARG;
    Vals vals = Vals::One;
    try {
        int64_t a = 0, b = 0, c = 0;
        double d = 0;
        if (f.size() == 4 && f[0] == "uniform" && to_i64(f[1], &a) && to_i64(f[2], &b) && to_f64(f[3], &d) && a > 0 && b > 0 &&
            a <= INT32_MAX && b <= INT32_MAX && d >= 0 && d <= 1) {
            m->M = a; m->N = b;
            st = gen_uniform(a, b, d, seed, *m);
        } else if (f.size() == 4 && f[0] == "zipf" && to_i64(f[1], &a) && to_i64(f[2], &b) && to_i64(f[3], &c) && a > 0 &&
                   b > 0 && c >= 0 && a <= INT32_MAX && b <= INT32_MAX) {
            m->M = a; m->N = b;
            vals = Vals::Int20;
            st = gen_zipf(a, b, c, seed, *m);
        } else if (f.size() == 3 && f[0] == "rmat" && to_i64(f[1], &a) && to_i64(f[2], &b)) {
            m->M = m->N = a >= 1 && a <= 30 ? (int64_t)1 << a : 0;
            vals = Vals::Normal;
            st = gen_rmat((int)a, b, seed, *m);
        } else if (f.size() == 4 && f[0] == "band" && to_i64(f[1], &a) && to_i64(f[2], &b) && to_i64(f[3], &c) && a > 0 &&
                   a <= INT32_MAX) {
            m->M = m->N = a;
            st = gen_band(a, b, c, seed, *m);
        } else {
            set_err(err, err_len, "unknown generator spec '" + s + "' (uniform:M:N:density, zipf:M:N:nnz, "
                                  "rmat:scale:edge_factor, band:M:half_width:g, c1..c5, optional :seed=S)");
        }
        if (st == SDDMM_OK) fill_values(*m, vals, seed);
    } catch (const std::bad_alloc &) {
        st = SDDMM_OUT_OF_MEMORY;
    }
    if (st != SDDMM_OK) {
        if (st == SDDMM_INVALID_ARG && err && err_len > 0 && !err[0]) set_err(err, err_len, "generator parameters out of range in '" + s + "'");
        delete m;
        return st;
    }
    *M = m->M; *N = m->N; *nnz = m->nnz;
    *out = m;
    return SDDMM_OK;
}
