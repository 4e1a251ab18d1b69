// host_encode.cpp -- weight generators and the host-side encoder.
//
// The reference generates and encodes its weights on the device, one thread per column
// (prepareW_map, main.cu:202-489).  Here both run on the host, column-parallel over
// std::thread, and emit either the reference's layouts byte-for-byte or the native ones.
#include <algorithm>
#include <cstring>
#include <thread>

#include "internal.h"

namespace sptmm {

static thread_local std::string g_err;

int fail(int code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

template <typename F>
static void parallel_columns(uint32_t N, F &&body)
{
    unsigned hw = std::max(1u, std::thread::hardware_concurrency());
    unsigned nt = std::min<unsigned>(hw, std::max(1u, N / 64));
    if (nt <= 1) { body(0u, N); return; }
    std::vector<std::thread> th;
    for (unsigned t = 0; t < nt; t++)
        th.emplace_back([&, t] { body((uint32_t)((uint64_t)N * t / nt), (uint32_t)((uint64_t)N * (t + 1) / nt)); });
    for (auto &x : th) x.join();
}

static inline uint32_t xs32(uint32_t &s)       // macro.cuh:69-76
{
    s ^= s << 13; s ^= s >> 17; s ^= s << 5;
    return s;
}

static inline uint64_t sm64(uint64_t &s)
{
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

struct Lists {                       // per-column sorted row indices of the +1 / -1 entries
    std::vector<std::vector<uint16_t>> pos, neg;
    uint32_t max_count = 0;
    uint64_t nnz = 0;
    bool uniform = true;             // every list has the same length
};

static int build_lists(const int8_t *W, uint32_t K, uint32_t N, Lists &L)
{
    L.pos.assign(N, {});
    L.neg.assign(N, {});
    std::vector<int> bad(N, 0);
    parallel_columns(N, [&](uint32_t c0, uint32_t c1) {
        for (uint32_t c = c0; c < c1; c++) {
            const int8_t *w = W + (size_t)c * K;
            auto &p = L.pos[c]; auto &n = L.neg[c];
            for (uint32_t k = 0; k < K; k++) {       // ascending rows, as main.cu:267-274
                if (w[k] == 1) p.push_back((uint16_t)k);
                else if (w[k] == -1) n.push_back((uint16_t)k);
                else if (w[k] != 0) bad[c] = 1;
            }
        }
    });
    const size_t first = N ? L.pos[0].size() : 0;
    for (uint32_t c = 0; c < N; c++) {
        if (bad[c]) return fail(SPTMM_ERR_INVALID, "W has an entry outside {-1,0,+1} in column %u", c);
        L.max_count = std::max<uint32_t>(L.max_count, (uint32_t)std::max(L.pos[c].size(), L.neg[c].size()));
        L.nnz += L.pos[c].size() + L.neg[c].size();
        if (L.pos[c].size() != first || L.neg[c].size() != first) L.uniform = false;
    }
    return SPTMM_OK;
}

static HostArray make_array(const char *name, size_t bytes, bool streamed, uint8_t fill = 0)
{
    HostArray a;
    a.name = name;
    a.data.assign(bytes, fill);
    a.streamed = streamed;
    return a;
}

// Reference chunk-interleaved layout: element (entry e, column c) at
// (e/split)*(split*N) + c*split + e%split   (main.cu:345-373).
static void encode_u16_div(const Lists &L, sptmm_weights &w, uint32_t cap)
{
    const uint32_t N = w.N, split = w.split;
    const char *names[2][3] = {{"W_map_8_div", "W_map_16_div", "W_map_32_div"},
                               {"W_map_negative_8_div", "W_map_negative_16_div", "W_map_negative_32_div"}};
    const int si = split == 8 ? 0 : split == 16 ? 1 : 2;
    for (int sign = 0; sign < 2; sign++) {
        w.arrays.push_back(make_array(names[sign][si], (size_t)cap * N * 2, true));
        uint16_t *out = (uint16_t *)w.arrays.back().data.data();
        parallel_columns(N, [&](uint32_t c0, uint32_t c1) {
            for (uint32_t c = c0; c < c1; c++) {
                const auto &l = sign ? L.neg[c] : L.pos[c];
                for (uint32_t e = 0; e < cap; e++) {
                    uint16_t v = e < l.size() ? l[e] : (uint16_t)w.K;    // pad -> zero row K
                    out[(size_t)(e / split) * ((size_t)split * N) + (size_t)c * split + e % split] = v;
                }
            }
        });
    }
    w.S = 2 * cap;
    w.stream_bytes = (uint64_t)cap * N * 2 * 2;
}

// Reference gap layout: gap[0] = first index, gap[i] = idx[i]-idx[i-1], each stored in 8 bits
// (main.cu:376-394); element (entry e, column c) at (e/256)*(256*N) + c*256 + e%256
// (main.cu:400-413).  The unwritten tail of the last block is zero here.
static void encode_delta_div256(const Lists &L, sptmm_weights &w, uint32_t cap)
{
    const uint32_t N = w.N;
    const size_t blocks = (cap + 255) / 256;
    std::vector<uint64_t> lossy(N, 0);
    const char *names[2] = {"W_map_delta2_div256", "W_map_negative_delta2_div256"};
    for (int sign = 0; sign < 2; sign++) {
        w.arrays.push_back(make_array(names[sign], blocks * 256 * N, true));
        uint8_t *out = w.arrays.back().data.data();
        parallel_columns(N, [&](uint32_t c0, uint32_t c1) {
            for (uint32_t c = c0; c < c1; c++) {
                const auto &l = sign ? L.neg[c] : L.pos[c];
                for (uint32_t e = 0; e < cap; e++) {
                    uint32_t gap = e == 0 ? l[0] : (uint32_t)(l[e] - l[e - 1]);
                    if (gap > 255) lossy[c]++;
                    out[(size_t)(e / 256) * ((size_t)256 * N) + (size_t)c * 256 + e % 256] = (uint8_t)gap;
                }
            }
        });
    }
    for (uint32_t c = 0; c < N; c++) w.lossy += lossy[c];
    w.S = 2 * cap;
    w.stream_bytes = (uint64_t)cap * N * 2;      // the tail padding is never read
}

// Native u16 layout.  Each list, in the order bank_order() gives it, is cut into blocks of 256
// entries (the last one padded with index K, which addresses a zero row the kernels append to
// X).  Inside a block the entry that lane l consumes at step t, entry 32*t + l, sits at
// position 8*l + t, so that one 16-byte load per lane brings eight entries.
//
// Order of a list's entries inside the native format.  A sum does not depend on the order of its
// terms, so the encoder is free to choose which 32 entries a warp gathers in one step (entries
// 32t..32t+31 of a block) and which lane gets which.  The kernels keep MT rows of X side by side,
// RB = MT*sizeof(element) bytes per matrix row, so a gathered row r occupies shared-memory banks
// (r*RB/4) mod 32.  Sorted order is ideal for RB = 1 (32 neighbouring rows share a few words) but
// random for wider tiles: 2.9 / 5.1 / 9.1 bank cycles per step at RB = 4 / 8 / 16 where 1 / 2 / 4
// would do.  The order chosen here gives lane l an entry with r = l (mod 32) whenever the next
// kWindow unused entries of the sorted list hold one: then the 32 rows differ mod 32 (RB = 4), the
// rows of a half warp differ mod 16 (RB = 8) and those of a quarter warp mod 8 (RB = 16).  Lanes
// left empty fall back to r = l (mod 16), then (mod 8), then to the smallest unused row.  Every
// choice must also keep the step conflict-free for RB = 1: two rows of a step may share a bank
// ((r/4) mod 32) only if they share the word.  Measured on the reference generator's lists
// (K=6912, 2048 entries): 1.10 / 1.46 / 2.56 / 4.6 cycles per step at RB = 1 / 4 / 8 / 16 (a
// window of 192 entries gave 1.07 / 2.0 / 3.0 / 4.8; beyond 768 nothing changes).
// `rows` is ascending; `out` receives the same rows, 32 per step, in step order; a step's unused
// lanes (possible only in the last steps of a list) hold `pad`.
static void bank_order(const std::vector<uint16_t> &rows, uint16_t pad, std::vector<uint16_t> &out)
{
    constexpr size_t kWindow = 768;
    const size_t n = rows.size();
    out.clear();
    out.reserve((n + 31) / 32 * 32);
    std::vector<uint16_t> bucket[32];         // window entries by r mod 32, ascending
    size_t next = 0, in_window = 0, remaining = n;
    while (remaining) {
        while (in_window < kWindow && next < n) { bucket[rows[next] & 31].push_back(rows[next]); next++; in_window++; }
        uint16_t step[32];
        bool filled[32] = {};
        int32_t bank_word[32];
        for (int i = 0; i < 32; i++) bank_word[i] = -1;
        auto fits = [&](uint16_t r) { const int32_t wd = r >> 2; return bank_word[wd & 31] < 0 || bank_word[wd & 31] == wd; };
        auto take = [&](int lane, int b, size_t j) {
            const uint16_t r = bucket[b][j];
            bucket[b].erase(bucket[b].begin() + (ptrdiff_t)j);
            step[lane] = r; filled[lane] = true; bank_word[(r >> 2) & 31] = r >> 2;
        };
        for (int mod = 32; mod >= 8; mod >>= 1)
            for (int lane = 0; lane < 32; lane++) {
                if (filled[lane]) continue;
                for (int b = lane % mod; b < 32 && !filled[lane]; b += mod)
                    for (size_t j = 0; j < bucket[b].size(); j++)
                        if (fits(bucket[b][j])) { take(lane, b, j); break; }
            }
        for (int strict = 1; strict >= 0; strict--)
            for (int lane = 0; lane < 32; lane++) {
                if (filled[lane]) continue;
                int best_b = -1; size_t best_j = 0; uint32_t best_r = 0xffffffffu;
                for (int b = 0; b < 32; b++)
                    for (size_t j = 0; j < bucket[b].size(); j++)
                        if (!strict || fits(bucket[b][j])) {
                            if (bucket[b][j] < best_r) { best_r = bucket[b][j]; best_b = b; best_j = j; }
                            break;
                        }
                if (best_b >= 0) take(lane, best_b, best_j);
            }
        for (int lane = 0; lane < 32; lane++) {
            out.push_back(filled[lane] ? step[lane] : pad);
            if (filled[lane]) { remaining--; in_window--; }
        }
    }
}

// Blocks are stored list after list in the order pos(0), neg(0), pos(1), ...; blk_off[2c+s]
// is the first block of list (column c, sign s).
static void encode_u16_v256(const Lists &L, sptmm_weights &w)
{
    const uint32_t N = w.N;
    std::vector<uint32_t> off(2 * (size_t)N + 1, 0);
    uint32_t maxblk = 0;
    for (uint32_t c = 0; c < N; c++) {
        uint32_t bp = (uint32_t)(L.pos[c].size() + 255) / 256, bn = (uint32_t)(L.neg[c].size() + 255) / 256;
        off[2 * c + 1] = off[2 * c] + bp;
        off[2 * c + 2] = off[2 * c + 1] + bn;
        maxblk = std::max(maxblk, std::max(bp, bn));
    }
    w.total_blocks = off[2 * (size_t)N];
    w.entries_per_block = 256;
    w.uniform_nbl = off[1] - off[0];
    for (size_t l = 0; l < 2 * (size_t)N; l++)
        if (off[l + 1] - off[l] != w.uniform_nbl) { w.uniform_nbl = 0; break; }
    w.arrays.push_back(make_array("idx_v256", (size_t)w.total_blocks * 512, true));
    uint16_t *out = (uint16_t *)w.arrays.back().data.data();
    parallel_columns(N, [&](uint32_t c0, uint32_t c1) {
        std::vector<uint16_t> l;
        for (uint32_t c = c0; c < c1; c++)
            for (int sign = 0; sign < 2; sign++) {
                bank_order(sign ? L.neg[c] : L.pos[c], (uint16_t)w.K, l);
                uint16_t *dst = out + (size_t)off[2 * c + sign] * 256;
                const uint32_t nb = off[2 * c + sign + 1] - off[2 * c + sign];
                for (uint32_t b = 0; b < nb; b++)
                    for (uint32_t lane = 0; lane < 32; lane++)
                        for (uint32_t t = 0; t < 8; t++) {
                            size_t e = (size_t)b * 256 + 32 * t + lane;
                            dst[(size_t)b * 256 + 8 * lane + t] = e < l.size() ? l[e] : (uint16_t)w.K;
                        }
            }
    });
    w.arrays.push_back(make_array("blk_off", off.size() * 4, true));
    memcpy(w.arrays.back().data.data(), off.data(), off.size() * 4);
    w.S = 2 * 256 * maxblk;
    w.stream_bytes = (uint64_t)w.total_blocks * 512 + off.size() * 4;
}

// Native narrow-integer layout (SPTMM_FMT_DELTA_LANE).  A list's sorted rows are cut into gather
// STEPS of up to 32 entries: a step takes the next entries while they lie within 255 rows of its
// first one (its base), so every entry is base + an 8-bit offset, exactly; in lists denser than
// one entry per eight rows nearly every step is full.  Eight steps make a 304-byte block:
//   [0,256)    offsets: byte 8*lane + t is lane's offset in step t (one 8-byte load per lane)
//   [256,288)  eight 32-bit bases
//   [288,296)  eight counts (entries of the step; lanes at or beyond it gather nothing)
//   [296,304)  zero
// Blocks are stored list after list like the u16 format's, with the same blk_off array.  Unlike
// the reference's gap lists (main.cu:376-394) nothing is truncated and no scan across lanes is
// needed to decode: a lane adds its offset to the step's base.
static void encode_delta_lane(const Lists &L, sptmm_weights &w)
{
    constexpr size_t BB = 304;
    const uint32_t N = w.N;
    auto steps_of = [](const std::vector<uint16_t> &l) {
        uint32_t steps = 0;
        for (size_t i = 0; i < l.size();) {
            size_t j = i;
            while (j < l.size() && j - i < 32 && (uint32_t)(l[j] - l[i]) <= 255u) j++;
            steps++;
            i = j;
        }
        return steps;
    };
    std::vector<uint32_t> off(2 * (size_t)N + 1, 0);
    uint32_t maxblk = 0;
    for (uint32_t c = 0; c < N; c++) {
        const uint32_t bp = (steps_of(L.pos[c]) + 7) / 8, bn = (steps_of(L.neg[c]) + 7) / 8;
        off[2 * c + 1] = off[2 * c] + bp;
        off[2 * c + 2] = off[2 * c + 1] + bn;
        maxblk = std::max(maxblk, std::max(bp, bn));
    }
    w.total_blocks = off[2 * (size_t)N];
    w.entries_per_block = 256;
    w.uniform_nbl = off[1] - off[0];
    for (size_t l = 0; l < 2 * (size_t)N; l++)
        if (off[l + 1] - off[l] != w.uniform_nbl) { w.uniform_nbl = 0; break; }
    w.arrays.push_back(make_array("idx_delta_lane", (size_t)w.total_blocks * BB, true));     // zero-filled
    uint8_t *out = w.arrays.back().data.data();
    parallel_columns(N, [&](uint32_t c0, uint32_t c1) {
        for (uint32_t c = c0; c < c1; c++)
            for (int sign = 0; sign < 2; sign++) {
                const auto &l = sign ? L.neg[c] : L.pos[c];
                uint8_t *dst = out + (size_t)off[2 * c + sign] * BB;
                uint32_t step = 0;
                for (size_t i = 0; i < l.size(); step++) {
                    uint8_t *blk = dst + (size_t)(step / 8) * BB;
                    const uint32_t t = step % 8;
                    size_t j = i;
                    while (j < l.size() && j - i < 32 && (uint32_t)(l[j] - l[i]) <= 255u) {
                        blk[8 * (j - i) + t] = (uint8_t)(l[j] - l[i]);
                        j++;
                    }
                    const uint32_t base = l[i];
                    memcpy(blk + 256 + 4 * t, &base, 4);
                    blk[288 + t] = (uint8_t)(j - i);
                    i = j;
                }
            }
    });
    w.arrays.push_back(make_array("blk_off", off.size() * 4, true));
    memcpy(w.arrays.back().data.data(), off.data(), off.size() * 4);
    w.S = 2 * 256 * maxblk;
    w.stream_bytes = (uint64_t)w.total_blocks * BB + off.size() * 4;
}

// Comparator packing: word j of column c carries rows 16j..16j+15 as 2-bit codes w+2; row
// 16j+e sits at bit 8*(e%4) + 2*(e/4)  (the decode order of bitnet_kernels.cuh:57-71).
static void encode_i2s(const int8_t *W, sptmm_weights &w)
{
    const uint32_t K = w.K, N = w.N, words = K / 16;
    w.arrays.push_back(make_array("i2s", (size_t)words * N * 4, true));
    uint32_t *out = (uint32_t *)w.arrays.back().data.data();
    parallel_columns(N, [&](uint32_t c0, uint32_t c1) {
        for (uint32_t c = c0; c < c1; c++)
            for (uint32_t j = 0; j < words; j++) {
                uint32_t word = 0;
                for (uint32_t e = 0; e < 16; e++) {
                    uint32_t code = (uint32_t)(W[(size_t)c * K + 16 * j + e] + 2) & 3u;
                    word |= code << (8 * (e % 4) + 2 * (e / 4));
                }
                out[(size_t)c * words + j] = word;
            }
    });
    w.stream_bytes = (uint64_t)words * N * 4;
}

}  // namespace sptmm

using namespace sptmm;

extern "C" const char *sptmm_last_error(void) { return g_err.c_str(); }
extern "C" int sptmm_version(void) { return 100; }

extern "C" int sptmm_gen_ternary_fixed(uint32_t K, uint32_t N, uint32_t S, int8_t *W)
{
    if (!W || K == 0 || N == 0) return fail(SPTMM_ERR_INVALID, "gen_ternary_fixed: null W or empty shape");
    if ((S & 1) || S > K) return fail(SPTMM_ERR_INVALID, "gen_ternary_fixed: S=%u must be even and <= K=%u", S, K);
    parallel_columns(N, [&](uint32_t c0, uint32_t c1) {
        for (uint32_t c = c0; c < c1; c++) {
            int8_t *w = W + (size_t)c * K;
            std::fill(w, w + S / 2, (int8_t)-1);
            std::fill(w + S / 2, w + S, (int8_t)1);
            std::fill(w + S, w + K, (int8_t)0);
            uint32_t state = 0xCAFEBABEu ^ c;
            for (uint32_t i = K - 1; i > 0; --i)
                std::swap(w[i], w[xs32(state) % (i + 1)]);
        }
    });
    return SPTMM_OK;
}

extern "C" int sptmm_gen_ternary_iid(uint32_t K, uint32_t N, double p_zero, uint64_t seed, int8_t *W)
{
    if (!W || K == 0 || N == 0) return fail(SPTMM_ERR_INVALID, "gen_ternary_iid: null W or empty shape");
    if (!(p_zero >= 0.0 && p_zero <= 1.0)) return fail(SPTMM_ERR_INVALID, "gen_ternary_iid: p_zero=%g outside [0,1]", p_zero);
    const uint64_t full = 1ull << 53;
    uint64_t t0 = std::min(full, (uint64_t)(p_zero * (double)full));
    const uint64_t t1 = t0 + (full - t0) / 2;
    parallel_columns(N, [&](uint32_t c0, uint32_t c1) {
        for (uint32_t c = c0; c < c1; c++) {
            uint64_t t = seed ^ ((uint64_t)(c + 1) * 0xD1342543DE82EF95ull);
            uint64_t s = sm64(t);             // hashed, so column streams are unrelated
            int8_t *w = W + (size_t)c * K;
            for (uint32_t k = 0; k < K; k++) {
                uint64_t r = sm64(s) >> 11;
                w[k] = r < t0 ? 0 : (r < t1 ? 1 : -1);
            }
        }
    });
    return SPTMM_OK;
}

extern "C" int sptmm_encode(const int8_t *W, uint32_t K, uint32_t N, uint32_t format, uint32_t split,
                            uint32_t S, sptmm_weights **out)
{
    if (!W || !out) return fail(SPTMM_ERR_INVALID, "encode: null pointer");
    *out = nullptr;
    if (K == 0 || N == 0) return fail(SPTMM_ERR_INVALID, "encode: empty shape K=%u N=%u", K, N);
    if (K > 65535) return fail(SPTMM_ERR_INVALID, "encode: K=%u does not fit 16-bit row indices (K must be < 65536)", K);
    if (S & 1) return fail(SPTMM_ERR_INVALID, "encode: S=%u must be even (S/2 entries per sign)", S);

    sptmm_weights *w = new (std::nothrow) sptmm_weights();
    if (!w) return fail(SPTMM_ERR_NOMEM, "encode: out of host memory");
    w->K = K; w->N = N; w->format = format; w->split = split;

    int rc = SPTMM_OK;
    if (format == SPTMM_FMT_I2S) {
        if (K % 16) rc = fail(SPTMM_ERR_INVALID, "encode: i2s packs 16 rows per word, K=%u is not a multiple of 16", K);
        else {
            for (size_t i = 0; i < (size_t)K * N && rc == SPTMM_OK; i++) {
                if (W[i] < -1 || W[i] > 1) rc = fail(SPTMM_ERR_INVALID, "W has an entry outside {-1,0,+1}");
                else w->nnz += W[i] != 0;
            }
            if (rc == SPTMM_OK) { w->split = 0; encode_i2s(W, *w); }
        }
    } else {
        Lists L;
        rc = build_lists(W, K, N, L);
        if (rc == SPTMM_OK) {
            w->max_count = L.max_count;
            w->nnz = L.nnz;
            if (S && L.max_count > S / 2)
                rc = fail(SPTMM_ERR_INVALID, "encode: a column has %u entries of one sign, more than S/2=%u", L.max_count, S / 2);
        }
        if (rc == SPTMM_OK) switch (format) {
            case SPTMM_FMT_U16_DIV: {
                if (split != 8 && split != 16 && split != 32) { rc = fail(SPTMM_ERR_INVALID, "Wrong split size"); break; }
                if (N % (32 / split)) { rc = fail(SPTMM_ERR_INVALID, "encode: N=%u must be a multiple of %u for split %u", N, 32 / split, split); break; }
                uint32_t cap = S ? S / 2 : (L.max_count + split - 1) / split * split;
                if (cap % split) { rc = fail(SPTMM_ERR_INVALID, "encode: S/2=%u must be a multiple of split=%u", cap, split); break; }
                if (cap == 0) cap = split;
                encode_u16_div(L, *w, cap);
                break;
            }
            case SPTMM_FMT_DELTA_DIV256: {
                uint32_t cap = S ? S / 2 : L.max_count;
                if (!L.uniform || cap != L.max_count || cap == 0) {
                    rc = fail(SPTMM_ERR_UNSUPPORTED, "encode: the 8-bit gap layout has no padding value; every list must hold exactly S/2 entries");
                    break;
                }
                w->split = 32;
                encode_delta_div256(L, *w, cap);
                break;
            }
            case SPTMM_FMT_U16_V256:
                w->split = 32;
                encode_u16_v256(L, *w);
                break;
            case SPTMM_FMT_DELTA_LANE:
                w->split = 32;
                encode_delta_lane(L, *w);
                break;
            default:
                rc = fail(SPTMM_ERR_UNSUPPORTED, "encode: unknown format %u", format);
        }
    }
    if (rc != SPTMM_OK) { delete w; return rc; }
    *out = w;
    return SPTMM_OK;
}

// A K-tiled matrix: the rows are cut into tiles of k_tile rows and every tile is encoded as a
// native u16 matrix of its own (row numbers counted from the tile's first row).  The reference's
// "split-K" is lane striding over one list (main.cu:581-584); a K range that can be multiplied on
// its own is what a kernel needs to keep sixteen rows of a long activation in shared memory, and
// what a GPU needs to own one K range of a matrix split across GPUs.
extern "C" int sptmm_encode_ktiled(const int8_t *W, uint32_t K, uint32_t N, uint32_t k_tile, sptmm_weights **out)
{
    if (!W || !out) return fail(SPTMM_ERR_INVALID, "encode_ktiled: null pointer");
    *out = nullptr;
    if (K == 0 || N == 0 || K >= 65536) return fail(SPTMM_ERR_INVALID, "encode_ktiled: bad shape K=%u N=%u", K, N);
    if (k_tile == 0 || (k_tile & 15)) return fail(SPTMM_ERR_INVALID, "encode_ktiled: k_tile=%u must be a positive multiple of 16", k_tile);
    sptmm_weights *w = new (std::nothrow) sptmm_weights();
    if (!w) return fail(SPTMM_ERR_NOMEM, "encode_ktiled: out of host memory");
    w->K = K; w->N = N; w->format = SPTMM_FMT_U16_V256; w->split = 32; w->k_tile = k_tile;
    std::vector<int8_t> slice;
    for (uint32_t k0 = 0; k0 < K; k0 += k_tile) {
        const uint32_t kt = std::min(k_tile, K - k0);
        slice.resize((size_t)kt * N);
        for (uint32_t c = 0; c < N; c++) memcpy(slice.data() + (size_t)c * kt, W + (size_t)c * K + k0, kt);
        sptmm_weights *t = nullptr;
        const int rc = sptmm_encode(slice.data(), kt, N, SPTMM_FMT_U16_V256, 32, 0, &t);
        if (rc != SPTMM_OK) { sptmm_weights_free(w); return rc; }
        w->tiles.push_back(t);
        w->nnz += t->nnz; w->stream_bytes += t->stream_bytes;
        w->max_count = std::max(w->max_count, t->max_count);
    }
    *out = w;
    return SPTMM_OK;
}

extern "C" int sptmm_weights_tile(const sptmm_weights *w, uint32_t tile, sptmm_weights **out)
{
    if (!w || !out) return fail(SPTMM_ERR_INVALID, "weights_tile: null pointer");
    if (tile >= w->tiles.size()) return fail(SPTMM_ERR_INVALID, "weights_tile: tile %u of %zu", tile, w->tiles.size());
    *out = w->tiles[tile];
    return SPTMM_OK;
}

extern "C" int sptmm_weights_info_get(const sptmm_weights *w, sptmm_weights_info *info)
{
    if (!w || !info) return fail(SPTMM_ERR_INVALID, "weights_info: null pointer");
    info->K = w->K; info->N = w->N; info->format = w->format; info->split = w->split; info->S = w->S;
    info->max_count = w->max_count; info->nnz = w->nnz; info->stream_bytes = w->stream_bytes;
    info->lossy_entries = w->lossy; info->n_arrays = (uint32_t)w->arrays.size(); info->device = w->device;
    info->k_tile = w->k_tile; info->n_tiles = (uint32_t)w->tiles.size();
    return SPTMM_OK;
}

extern "C" int sptmm_weights_array(const sptmm_weights *w, uint32_t i, const void **host_ptr,
                                   const void **device_ptr, uint64_t *bytes, const char **name)
{
    if (!w) return fail(SPTMM_ERR_INVALID, "weights_array: null handle");
    if (i >= w->arrays.size()) return fail(SPTMM_ERR_INVALID, "weights_array: index %u of %zu", i, w->arrays.size());
    if (host_ptr) *host_ptr = w->arrays[i].data.data();
    if (device_ptr) *device_ptr = (!w->dev.empty() && i < w->dev[0].size()) ? w->dev[0][i] : nullptr;
    if (bytes) *bytes = w->arrays[i].data.size();
    if (name) *name = w->arrays[i].name.c_str();
    return SPTMM_OK;
}
