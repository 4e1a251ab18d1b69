// weights_file.cpp -- encoded weights on disk: sptmm_weights_save / sptmm_weights_load.
//
// The reference re-generates and re-encodes its matrix on the GPU at every start (prepareW_map,
// main.cu:202-489, called at main.cu:972) and has no file format.  Encoding a large matrix on the
// host takes seconds, so an encoded matrix can be written once and mapped back in.
//
// File layout (little-endian, every array starts on a 64-byte boundary of the file):
//   0    8   magic "SPTMMW\0\1"
//   8    4   version (1)
//   12   4   header bytes (offset of the array table)
//   16   ..  K, N, format, split, S, max_count, total_blocks, entries_per_block, uniform_nbl   (9 x u32)
//        ..  nnz, stream_bytes, lossy_entries                                                    (3 x u64)
//        4   n_arrays
//   then per array: u32 name length, name bytes, u8 streamed, u64 data offset, u64 data bytes
//   then the arrays' bytes, and last a u64 FNV-1a hash of everything before it.
// Loading checks magic, version, every offset and size against the file length, and the hash.
#include <cstdio>
#include <cstring>
#include <memory>

#include "internal.h"

using namespace sptmm;

namespace {

constexpr char kMagic[8] = {'S', 'P', 'T', 'M', 'M', 'W', 0, 1};
constexpr uint32_t kVersion = 1;

uint64_t fnv1a(const uint8_t *p, size_t n, uint64_t h = 1469598103934665603ull)
{
    for (size_t i = 0; i < n; i++) { h ^= p[i]; h *= 1099511628211ull; }
    return h;
}

template <class T> void put(std::vector<uint8_t> &b, T v)
{
    const uint8_t *p = reinterpret_cast<const uint8_t *>(&v);
    b.insert(b.end(), p, p + sizeof(T));
}

struct Reader {
    const uint8_t *p; size_t n, at = 0; bool ok = true;
    template <class T> T get()
    {
        T v{};
        if (at + sizeof(T) > n) { ok = false; return v; }
        memcpy(&v, p + at, sizeof(T));
        at += sizeof(T);
        return v;
    }
};

struct FileCloser { void operator()(FILE *f) const { if (f) fclose(f); } };

}  // namespace

extern "C" int sptmm_weights_save(const sptmm_weights *w, const char *path)
{
    if (!w || !path) return fail(SPTMM_ERR_INVALID, "weights_save: null pointer");
    if (w->k_tile) return fail(SPTMM_ERR_UNSUPPORTED, "weights_save: a K-tiled matrix is saved tile by tile (sptmm_weights_tile)");
    std::vector<uint8_t> head;
    head.insert(head.end(), kMagic, kMagic + 8);
    put<uint32_t>(head, kVersion);
    put<uint32_t>(head, 0);                                    // header bytes, patched below
    for (uint32_t v : {w->K, w->N, w->format, w->split, w->S, w->max_count, w->total_blocks, w->entries_per_block, w->uniform_nbl})
        put<uint32_t>(head, v);
    for (uint64_t v : {w->nnz, w->stream_bytes, w->lossy}) put<uint64_t>(head, v);
    put<uint32_t>(head, (uint32_t)w->arrays.size());
    const uint32_t header_bytes = (uint32_t)head.size();
    memcpy(head.data() + 12, &header_bytes, 4);
    size_t table = 0;
    for (const HostArray &a : w->arrays) table += 4 + a.name.size() + 1 + 8 + 8;
    size_t at = (head.size() + table + 63) & ~(size_t)63;
    std::vector<uint64_t> offs;
    for (const HostArray &a : w->arrays) {
        put<uint32_t>(head, (uint32_t)a.name.size());
        head.insert(head.end(), a.name.begin(), a.name.end());
        put<uint8_t>(head, a.streamed ? 1 : 0);
        put<uint64_t>(head, (uint64_t)at);
        put<uint64_t>(head, (uint64_t)a.data.size());
        offs.push_back(at);
        at = (at + a.data.size() + 63) & ~(size_t)63;
    }
    std::unique_ptr<FILE, FileCloser> f(fopen(path, "wb"));
    if (!f) return fail(SPTMM_ERR_INVALID, "weights_save: cannot open %s for writing", path);
    uint64_t h = 1469598103934665603ull;
    size_t written = 0;
    auto emit = [&](const uint8_t *p, size_t n) {
        h = fnv1a(p, n, h);
        written += n;
        return fwrite(p, 1, n, f.get()) == n;
    };
    static const uint8_t zeros[64] = {};
    bool ok = emit(head.data(), head.size());
    for (size_t i = 0; ok && i < w->arrays.size(); i++) {
        ok = emit(zeros, offs[i] - written);
        ok = ok && emit(w->arrays[i].data.data(), w->arrays[i].data.size());
    }
    ok = ok && emit(zeros, at - written);
    ok = ok && fwrite(&h, 1, 8, f.get()) == 8;
    if (!ok) return fail(SPTMM_ERR_INVALID, "weights_save: short write to %s", path);
    return SPTMM_OK;
}

extern "C" int sptmm_weights_load(const char *path, sptmm_weights **out)
{
    if (!path || !out) return fail(SPTMM_ERR_INVALID, "weights_load: null pointer");
    *out = nullptr;
    std::unique_ptr<FILE, FileCloser> f(fopen(path, "rb"));
    if (!f) return fail(SPTMM_ERR_INVALID, "weights_load: cannot open %s", path);
    if (fseek(f.get(), 0, SEEK_END) != 0) return fail(SPTMM_ERR_INVALID, "weights_load: cannot seek in %s", path);
    const long len = ftell(f.get());
    if (len < 64) return fail(SPTMM_ERR_INVALID, "weights_load: %s is not an encoded-weights file (too short)", path);
    rewind(f.get());
    std::vector<uint8_t> buf((size_t)len);
    if (fread(buf.data(), 1, buf.size(), f.get()) != buf.size()) return fail(SPTMM_ERR_INVALID, "weights_load: short read from %s", path);
    if (memcmp(buf.data(), kMagic, 8) != 0) return fail(SPTMM_ERR_INVALID, "weights_load: %s is not an encoded-weights file (bad magic)", path);
    uint64_t stored;
    memcpy(&stored, buf.data() + buf.size() - 8, 8);
    if (fnv1a(buf.data(), buf.size() - 8) != stored) return fail(SPTMM_ERR_INVALID, "weights_load: %s is damaged (checksum mismatch)", path);

    Reader r{buf.data(), buf.size() - 8};
    r.at = 8;
    const uint32_t version = r.get<uint32_t>();
    if (version != kVersion) return fail(SPTMM_ERR_UNSUPPORTED, "weights_load: %s has file version %u, this build reads %u", path, version, kVersion);
    (void)r.get<uint32_t>();                                   // header bytes
    std::unique_ptr<sptmm_weights> w(new (std::nothrow) sptmm_weights());
    if (!w) return fail(SPTMM_ERR_NOMEM, "weights_load: out of host memory");
    w->K = r.get<uint32_t>(); w->N = r.get<uint32_t>(); w->format = r.get<uint32_t>(); w->split = r.get<uint32_t>();
    w->S = r.get<uint32_t>(); w->max_count = r.get<uint32_t>(); w->total_blocks = r.get<uint32_t>();
    w->entries_per_block = r.get<uint32_t>(); w->uniform_nbl = r.get<uint32_t>();
    w->nnz = r.get<uint64_t>(); w->stream_bytes = r.get<uint64_t>(); w->lossy = r.get<uint64_t>();
    const uint32_t n_arrays = r.get<uint32_t>();
    if (!r.ok || n_arrays > 64 || w->format < SPTMM_FMT_U16_DIV || w->format > SPTMM_FMT_I2S || w->K == 0 || w->N == 0 || w->K >= 65536)
        return fail(SPTMM_ERR_INVALID, "weights_load: %s has an inconsistent header", path);
    for (uint32_t i = 0; i < n_arrays; i++) {
        const uint32_t nl = r.get<uint32_t>();
        if (!r.ok || nl > 256 || r.at + nl > r.n) return fail(SPTMM_ERR_INVALID, "weights_load: %s has a damaged array table", path);
        HostArray a;
        a.name.assign(reinterpret_cast<const char *>(buf.data() + r.at), nl);
        r.at += nl;
        a.streamed = r.get<uint8_t>() != 0;
        const uint64_t off = r.get<uint64_t>(), bytes = r.get<uint64_t>();
        if (!r.ok || off > r.n || bytes > r.n - off) return fail(SPTMM_ERR_INVALID, "weights_load: array %u of %s lies outside the file", i, path);
        a.data.assign(buf.data() + off, buf.data() + off + bytes);
        w->arrays.push_back(std::move(a));
    }
    // what the kernels index with must agree with the array sizes
    const bool native = w->format == SPTMM_FMT_U16_V256 || w->format == SPTMM_FMT_DELTA_LANE;
    if (native) {
        const size_t bb = w->format == SPTMM_FMT_U16_V256 ? 512 : 304;
        bool good = w->arrays.size() == 2 && w->arrays[1].data.size() == (2 * (size_t)w->N + 1) * 4 &&
                    w->arrays[0].data.size() == (size_t)w->total_blocks * bb;
        if (good) {
            const uint32_t *off = reinterpret_cast<const uint32_t *>(w->arrays[1].data.data());
            good = off[0] == 0 && off[2 * (size_t)w->N] == w->total_blocks;
            for (size_t l = 0; good && l < 2 * (size_t)w->N; l++) good = off[l] <= off[l + 1];
        }
        if (!good) return fail(SPTMM_ERR_INVALID, "weights_load: the block table of %s does not match its arrays", path);
        // The kernels divide block numbers by uniform_nbl to find a column, so it is never taken from
        // the file: it follows from the block table exactly as the encoder derives it.
        const uint32_t *off = reinterpret_cast<const uint32_t *>(w->arrays[1].data.data());
        uint32_t nbl = off[1] - off[0];
        for (size_t l = 0; l < 2 * (size_t)w->N; l++)
            if (off[l + 1] - off[l] != nbl) { nbl = 0; break; }
        if (w->uniform_nbl != nbl || w->entries_per_block != 256)
            return fail(SPTMM_ERR_INVALID, "weights_load: the header of %s disagrees with its block table", path);
    } else {
        const size_t half = w->S / 2;
        size_t want = 0, count = 2;
        if (w->format == SPTMM_FMT_U16_DIV) want = half * w->N * 2;
        else if (w->format == SPTMM_FMT_DELTA_DIV256) want = (half + 255) / 256 * 256 * w->N;
        else { want = (size_t)(w->K / 16) * w->N * 4; count = 1; }
        bool good = w->arrays.size() == count && (w->format != SPTMM_FMT_I2S || w->K % 16 == 0);
        for (size_t i = 0; good && i < count; i++) good = w->arrays[i].data.size() == want;
        if (!good) return fail(SPTMM_ERR_INVALID, "weights_load: the arrays of %s do not have the size K, N and S imply", path);
    }
    // row indices address shared memory directly: none may exceed K (K itself is the zero row)
    bool in_range = true;
    if (w->format == SPTMM_FMT_U16_V256 || w->format == SPTMM_FMT_U16_DIV) {
        for (size_t a = 0; a < (w->format == SPTMM_FMT_U16_DIV ? 2u : 1u); a++) {
            const uint16_t *v = reinterpret_cast<const uint16_t *>(w->arrays[a].data.data());
            for (size_t i = 0, n = w->arrays[a].data.size() / 2; i < n && in_range; i++) in_range = v[i] <= w->K;
        }
    } else if (w->format == SPTMM_FMT_DELTA_LANE) {
        const uint8_t *blk = w->arrays[0].data.data();
        for (uint32_t b = 0; b < w->total_blocks && in_range; b++, blk += 304)
            for (int t = 0; t < 8 && in_range; t++) {
                uint32_t base;
                memcpy(&base, blk + 256 + 4 * t, 4);
                const uint32_t cnt = blk[288 + t];
                in_range = cnt <= 32 && (cnt == 0 || base < w->K);
                for (uint32_t l = 0; l < cnt && in_range; l++) in_range = base + blk[8 * l + t] < w->K;
            }
    }
    if (!in_range) return fail(SPTMM_ERR_INVALID, "weights_load: %s holds a row index beyond K=%u", path, w->K);
    *out = w.release();
    return SPTMM_OK;
}
