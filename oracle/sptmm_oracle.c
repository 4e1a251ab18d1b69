/*
 * sptmm_oracle.c -- CPU restatement of the SpTMM reference's ternary sparse matmul path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA library, never the product:
 * only the test-suite, the smoke check and the benchmark's CPU-baseline leg may load it.
 *
 * The reference (Ogiwara-CostlierRain464/SpTMM) has no CPU implementation and no tests, so
 * every function here restates, in scalar C, what one piece of the reference's CUDA code
 * computes; the citation above each function names the reference lines it follows.
 * Parity pinning: the reference ships no golden vectors.  The functions here are pinned
 * against outputs of the reference's own kernels (built unmodified by ref_harness.cu and
 * run on a B200); the resulting fixtures live in tests/golden/.
 *
 * Matrix conventions (reference macro.cuh:24-61):
 *   AT_0 row-major  mat[row*col_dim + col];   AT_1 col-major  mat[col*row_dim + row].
 * W (dense ternary, K x N) and the plain index lists W_map (S/2 x N) are column-major in
 * both reference builds (W_MAJOR = MAJOR_COL, script/make_rcr.sh:6, script/make_ccc.sh:6).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>

/* ---------------------------------------------------------------- PRNGs */

/* macro.cuh:69-76 (state must be non-zero) */
uint32_t oracle_xorshift32(uint32_t *state)
{
    uint32_t x = *state;
    x ^= x << 13;
    x ^= x >> 17;
    x ^= x << 5;
    *state = x;
    return x;
}

/* Harness-defined (the reference's make_X, main.cu:787-797, is unseeded): int8 activations
 * uniform on [-127,127] from xorshift32; seed 0 is mapped to a non-zero state. */
void oracle_gen_x_i8(int8_t *X, uint64_t count, uint32_t seed)
{
    uint32_t s = seed ? seed : 0x9E3779B9u;
    for (uint64_t i = 0; i < count; i++)
        X[i] = (int8_t)((int)(oracle_xorshift32(&s) % 255u) - 127);
}

static uint64_t splitmix64(uint64_t *s)
{
    uint64_t z = (*s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* ---------------------------------------------------------------- generators */

/* main.cu:248-265: column c = S/2 times -1, then S/2 times +1, then zeros; Fisher-Yates from
 * the last row down with xorshift32 seeded 0xCAFEBABE ^ c.  W is column-major K x N. */
int oracle_gen_fixed(uint32_t K, uint32_t N, uint32_t S, int8_t *W)
{
    if (S > K || (S & 1)) return -1;
    for (uint32_t c = 0; c < N; c++) {
        int8_t *w = W + (uint64_t)c * K;
        for (uint32_t i = 0; i < K; i++) w[i] = 0;
        for (uint32_t i = 0; i < S / 2; i++) w[i] = -1;
        for (uint32_t i = S / 2; i < S; i++) w[i] = 1;
        uint32_t seed = (uint32_t)(0xCAFEBABEu ^ c);
        for (int i = (int)K - 1; i > 0; --i) {
            int j = (int)(oracle_xorshift32(&seed) % (uint32_t)(i + 1));
            int8_t t = w[i]; w[i] = w[j]; w[j] = t;
        }
    }
    return 0;
}

/* Not in the reference (its generator is fixed-count only): i.i.d. ternary entries with
 * P(0) = p_zero and P(+1) = P(-1).  Column c draws from a splitmix64 stream whose state is the
 * splitmix64 hash of seed ^ (c+1)*0xD1342543DE82EF95; each row takes the top 53 bits r and compares against integer
 * thresholds t0 = floor(p_zero * 2^53), t1 = t0 + (2^53 - t0)/2:  r<t0 -> 0, r<t1 -> +1, else -1. */
int oracle_gen_iid(uint32_t K, uint32_t N, double p_zero, uint64_t seed, int8_t *W)
{
    if (p_zero < 0.0 || p_zero > 1.0) return -1;
    const uint64_t full = 1ull << 53;
    uint64_t t0 = (uint64_t)(p_zero * (double)full);
    if (t0 > full) t0 = full;
    uint64_t t1 = t0 + (full - t0) / 2;
    for (uint32_t c = 0; c < N; c++) {
        uint64_t t = seed ^ ((uint64_t)(c + 1) * 0xD1342543DE82EF95ull);
        uint64_t s = splitmix64(&t);          /* hashed, so column streams are unrelated */
        int8_t *w = W + (uint64_t)c * K;
        for (uint32_t k = 0; k < K; k++) {
            uint64_t r = splitmix64(&s) >> 11;
            w[k] = (r < t0) ? 0 : (r < t1 ? 1 : -1);
        }
    }
    return 0;
}

/* ---------------------------------------------------------------- index lists */

/* main.cu:267-274: scan rows ascending; +1 rows go to W_map[.][c], -1 rows to
 * W_map_negative[.][c].  Lists are column-major cap x N (cap = S/2 in the reference).
 * Extension for variable-length columns: entries past a column's count are filled with
 * `sentinel`; counts are returned per column.  Returns the largest count seen, or -1 if a
 * column overflows cap. */
int64_t oracle_build_lists(const int8_t *W, uint32_t K, uint32_t N, uint32_t cap,
                           uint16_t sentinel, uint16_t *pos, uint16_t *neg,
                           uint32_t *npos, uint32_t *nneg)
{
    int64_t maxc = 0;
    for (uint32_t c = 0; c < N; c++) {
        const int8_t *w = W + (uint64_t)c * K;
        uint32_t c1 = 0, cm1 = 0;
        for (uint32_t i = 0; i < K; i++) {
            if (w[i] == 1) {
                if (c1 >= cap) return -1;
                pos[(uint64_t)c * cap + c1++] = (uint16_t)i;
            } else if (w[i] == -1) {
                if (cm1 >= cap) return -1;
                neg[(uint64_t)c * cap + cm1++] = (uint16_t)i;
            }
        }
        for (uint32_t i = c1; i < cap; i++) pos[(uint64_t)c * cap + i] = sentinel;
        for (uint32_t i = cm1; i < cap; i++) neg[(uint64_t)c * cap + i] = sentinel;
        if (npos) npos[c] = c1;
        if (nneg) nneg[c] = cm1;
        if (c1 > maxc) maxc = c1;
        if (cm1 > maxc) maxc = cm1;
    }
    return maxc;
}

/* main.cu:345-373 (W_map_32_div / _16_div / _8_div): viewed as a column-major matrix of
 * split*N rows by (S/2)/split columns, row i = col*split + lane, column j = chunk; the
 * element is list entry j*split + lane of column `col`.  Flat offset of (entry e, column c):
 *   (e / split) * (split * N) + c * split + (e % split). */
void oracle_encode_div(const uint16_t *list, uint32_t half_s, uint32_t N, uint32_t split,
                       uint16_t *out)
{
    uint32_t chunks = half_s / split;
    for (uint64_t i = 0; i < (uint64_t)split * N; i++) {
        for (uint32_t j = 0; j < chunks; j++) {
            uint32_t original_row = j * split + (uint32_t)(i % split);
            uint32_t original_col = (uint32_t)(i / split);
            out[(uint64_t)j * ((uint64_t)split * N) + i] =
                list[(uint64_t)original_col * half_s + original_row];
        }
    }
}

/* main.cu:376-394: gap list of one sign, column-major S/2 x N, element type unsigned char:
 * entry 0 is the first index, entry i is idx[i]-idx[i-1]; both are TRUNCATED to 8 bits by the
 * store.  Returns how many entries lost information (value > 255). */
uint64_t oracle_delta_lists(const uint16_t *list, uint32_t half_s, uint32_t N, uint8_t *gaps)
{
    uint64_t lossy = 0;
    for (uint32_t c = 0; c < N; c++) {
        for (uint32_t i = 0; i < half_s; i++) {
            uint32_t v = (i == 0) ? list[(uint64_t)c * half_s]
                                  : (uint32_t)(list[(uint64_t)c * half_s + i] -
                                               list[(uint64_t)c * half_s + i - 1]);
            if (v > 255) lossy++;
            gaps[(uint64_t)c * half_s + i] = (uint8_t)v;
        }
    }
    return lossy;
}

/* main.cu:400-413 (W_map_delta2_div256): column-major 256*N rows by ceil((S/2)/256) columns;
 * flat offset of (entry e, column c) = (e/256)*(256*N) + c*256 + (e%256).  Entries with
 * e >= S/2 in the last block are never written by the reference (uninitialised device
 * memory); this restatement leaves `out` untouched there so the caller chooses the fill. */
void oracle_encode_delta_div256(const uint8_t *gaps, uint32_t half_s, uint32_t N, uint8_t *out)
{
    uint32_t blocks = (half_s + 255) / 256;
    for (uint64_t i = 0; i < (uint64_t)256 * N; i++) {
        for (uint32_t j = 0; j < blocks; j++) {
            uint32_t original_row = j * 256 + (uint32_t)(i % 256);
            uint32_t original_col = (uint32_t)(i / 256);
            if (original_row < half_s)
                out[(uint64_t)j * ((uint64_t)256 * N) + i] =
                    gaps[(uint64_t)original_col * half_s + original_row];
        }
    }
}

/* ---------------------------------------------------------------- the matmul itself */

/* main.cu:556-594 rowWiseSplit3Small4: X row-major M x K, C row-major M x N;
 * column c = blockIdx.x*(32/split) + threadIdx.y; lane walks i = lane, lane+split*N, ...
 * over the 32-wide base &W[32*blockIdx.x].  int32 adds commute, so the scalar loop below,
 * which visits the same elements, is bit-exact. */
void oracle_gemv_i8_div(const int8_t *X, const uint16_t *wpos, const uint16_t *wneg, int32_t *C,
                        uint32_t M, uint32_t K, uint32_t N, uint32_t S, uint32_t split)
{
    uint32_t chunks = (S / 2) / split;
    for (uint32_t m = 0; m < M; m++) {
        const int8_t *x = X + (uint64_t)m * K;
        for (uint32_t c = 0; c < N; c++) {
            int32_t acc = 0;
            for (uint32_t j = 0; j < chunks; j++) {
                uint64_t base = (uint64_t)j * ((uint64_t)split * N) + (uint64_t)c * split;
                for (uint32_t l = 0; l < split; l++) {
                    acc += x[wpos[base + l]];
                    acc -= x[wneg[base + l]];
                }
            }
            C[(uint64_t)m * N + c] = acc;
        }
    }
}

/* main.cu:599-764 rowWiseSplit2DeltaSmallAsync2/3: indices are rebuilt as a running sum of the
 * 8-bit gaps in `ushort` arithmetic carried across the whole column (main.cu:650-665), entries
 * e < S/2 only (main.cu:735).  A lossy (truncated) gap therefore yields the reference's wrong
 * index, faithfully. */
void oracle_gemv_i8_delta256(const int8_t *X, const uint8_t *dpos, const uint8_t *dneg, int32_t *C,
                             uint32_t M, uint32_t K, uint32_t N, uint32_t S)
{
    uint32_t half_s = S / 2;
    (void)K;
    for (uint32_t m = 0; m < M; m++) {
        const int8_t *x = X + (uint64_t)m * K;
        for (uint32_t c = 0; c < N; c++) {
            int32_t acc = 0;
            uint16_t ip = 0, in = 0;
            for (uint32_t e = 0; e < half_s; e++) {
                uint64_t off = (uint64_t)(e / 256) * ((uint64_t)256 * N) + (uint64_t)c * 256 + (e % 256);
                ip = (uint16_t)(ip + dpos[off]);
                in = (uint16_t)(in + dneg[off]);
                acc += x[ip];
                acc -= x[in];
            }
            C[(uint64_t)m * N + c] = acc;
        }
    }
}

/* Independent check that shares no code with the list path: C = X * W on the dense matrix. */
void oracle_gemv_i8_dense(const int8_t *X, const int8_t *W, int32_t *C,
                          uint32_t M, uint32_t K, uint32_t N)
{
    for (uint32_t m = 0; m < M; m++)
        for (uint32_t c = 0; c < N; c++) {
            const int8_t *w = W + (uint64_t)c * K;
            const int8_t *x = X + (uint64_t)m * K;
            int32_t acc = 0;
            for (uint32_t k = 0; k < K; k++) acc += (int32_t)x[k] * (int32_t)w[k];
            C[(uint64_t)m * N + c] = acc;
        }
}

/* Plain (un-interleaved) list form, variable length: pos/neg column-major cap x N with
 * per-column counts.  This is the loop main.cu:577-584 runs, stated on W_map itself. */
void oracle_gemv_i8_lists(const int8_t *X, const uint16_t *pos, const uint16_t *neg,
                          const uint32_t *npos, const uint32_t *nneg, uint32_t cap,
                          int32_t *C, uint32_t M, uint32_t K, uint32_t N)
{
    for (uint32_t m = 0; m < M; m++) {
        const int8_t *x = X + (uint64_t)m * K;
        for (uint32_t c = 0; c < N; c++) {
            int32_t acc = 0;
            for (uint32_t i = 0; i < npos[c]; i++) acc += x[pos[(uint64_t)c * cap + i]];
            for (uint32_t i = 0; i < nneg[c]; i++) acc -= x[neg[(uint64_t)c * cap + i]];
            C[(uint64_t)m * N + c] = acc;
        }
    }
}

/* Floating-point activations are an extension (every reference kernel is int8 -> int32,
 * main.cu:558-561).  Two results per output: `Cref` follows the reference's summation order in
 * fp32 (32 lane-strided partial sums, main.cu:581-584, then the shfl_down tree,
 * main.cu:586-589); `Cdbl` is the same sum in double.  `Cabs` is sum |x| over the gathered
 * entries, the scale a relative tolerance is normalised by.  X is fp32 here (fp16 inputs are
 * widened by the caller; widening is exact). */
void oracle_gemv_f32_lists(const float *X, const uint16_t *pos, const uint16_t *neg,
                           const uint32_t *npos, const uint32_t *nneg, uint32_t cap,
                           float *Cref, double *Cdbl, double *Cabs,
                           uint32_t M, uint32_t K, uint32_t N)
{
    for (uint32_t m = 0; m < M; m++) {
        const float *x = X + (uint64_t)m * K;
        for (uint32_t c = 0; c < N; c++) {
            float lane[32];
            for (int l = 0; l < 32; l++) lane[l] = 0.0f;
            double d = 0.0, a = 0.0;
            uint32_t np = npos[c], nn = nneg[c];
            uint32_t n = np > nn ? np : nn;
            for (uint32_t i = 0; i < n; i++) {
                if (i < np) {
                    float v = x[pos[(uint64_t)c * cap + i]];
                    lane[i & 31] += v; d += v; a += v < 0 ? -v : v;
                }
                if (i < nn) {
                    float v = x[neg[(uint64_t)c * cap + i]];
                    lane[i & 31] -= v; d -= v; a += v < 0 ? -v : v;
                }
            }
            for (int s = 16; s > 0; s >>= 1)
                for (int l = 0; l < s; l++) lane[l] += lane[l + s];
            if (Cref) Cref[(uint64_t)m * N + c] = lane[0];
            if (Cdbl) Cdbl[(uint64_t)m * N + c] = d;
            if (Cabs) Cabs[(uint64_t)m * N + c] = a;
        }
    }
}

/* ---------------------------------------------------------------- i2s comparator */

/* bitnet_kernels.cuh:52-72 decode_i2s_to_i8s: one 32-bit word carries 16 weights as 2-bit
 * codes (code = w + 2, so 1,2,3 <-> -1,0,+1); output byte e of the 16 decoded bytes comes from
 * bits [8*(e%4) + 2*(e/4), +2).  This packs 16 consecutive rows k0..k0+15 of one column. */
uint32_t oracle_i2s_pack16(const int8_t *w16)
{
    uint32_t word = 0;
    for (int e = 0; e < 16; e++) {
        uint32_t code = (uint32_t)(w16[e] + 2) & 3u;
        word |= code << (8 * (e % 4) + 2 * (e / 4));
    }
    return word;
}

void oracle_i2s_unpack16(uint32_t word, int8_t *w16)
{
    for (int e = 0; e < 16; e++)
        w16[e] = (int8_t)((int)((word >> (8 * (e % 4) + 2 * (e / 4))) & 3u) - 2);
}

/* ---------------------------------------------------------------- timed CPU baseline */

/* The "reference's scalar CPU add/sub path" named by the benchmark contract does not exist in
 * the reference; this is the loop of main.cu:577-584 over the chunk-interleaved u16 layout, with
 * columns partitioned over `threads` pthreads. */
struct slice { const int8_t *X; const uint16_t *wp, *wn; int32_t *C;
               uint32_t M, K, N, S, split, c0, c1; };

static void *slice_run(void *p)
{
    struct slice *s = (struct slice *)p;
    uint32_t chunks = (s->S / 2) / s->split;
    for (uint32_t m = 0; m < s->M; m++) {
        const int8_t *x = s->X + (uint64_t)m * s->K;
        for (uint32_t c = s->c0; c < s->c1; c++) {
            int32_t acc = 0;
            for (uint32_t j = 0; j < chunks; j++) {
                uint64_t base = (uint64_t)j * ((uint64_t)s->split * s->N) + (uint64_t)c * s->split;
                for (uint32_t l = 0; l < s->split; l++) {
                    acc += x[s->wp[base + l]];
                    acc -= x[s->wn[base + l]];
                }
            }
            s->C[(uint64_t)m * s->N + c] = acc;
        }
    }
    return NULL;
}

int oracle_gemv_i8_div_mt(const int8_t *X, const uint16_t *wpos, const uint16_t *wneg, int32_t *C,
                          uint32_t M, uint32_t K, uint32_t N, uint32_t S, uint32_t split,
                          uint32_t threads)
{
    if (threads == 0) threads = 1;
    if (threads > 256) threads = 256;
    pthread_t th[256];
    struct slice sl[256];
    for (uint32_t t = 0; t < threads; t++) {
        sl[t] = (struct slice){ X, wpos, wneg, C, M, K, N, S, split,
                                (uint32_t)((uint64_t)N * t / threads),
                                (uint32_t)((uint64_t)N * (t + 1) / threads) };
        if (t + 1 < threads && pthread_create(&th[t], NULL, slice_run, &sl[t]) != 0) return -1;
    }
    slice_run(&sl[threads - 1]);
    for (uint32_t t = 0; t + 1 < threads; t++) pthread_join(th[t], NULL);
    return 0;
}

/* FNV-1a 64-bit, the checksum the golden fixtures record for arrays too large to commit. */
uint64_t oracle_fnv1a64(const void *p, uint64_t n)
{
    const unsigned char *b = (const unsigned char *)p;
    uint64_t h = 0xcbf29ce484222325ull;
    for (uint64_t i = 0; i < n; i++) { h ^= b[i]; h *= 0x100000001b3ull; }
    return h;
}

/* Not in the reference (it has no activation quantiser; its X is drawn as int8 directly,
 * main.cu:787-797).  Defines the quantiser a layer stack needs between matmuls: per row,
 * amax = max |a+b|, q = clamp(rint((float)(a+b) * (127.0f/(float)amax)), -127, 127) with
 * single-precision arithmetic and round-to-nearest-even; amax == 0 gives zeros.
 * scale[m] = amax/127.  B may be NULL. */
#include <math.h>
void oracle_quant_absmax_i8(const int32_t *A, uint32_t lda, const int32_t *B, uint32_t ldb,
                            uint32_t M, uint32_t K, int8_t *out, float *scale)
{
    for (uint32_t m = 0; m < M; m++) {
        int amax = 0;
        for (uint32_t k = 0; k < K; k++) {
            int v = A[(uint64_t)m * lda + k] + (B ? B[(uint64_t)m * ldb + k] : 0);
            int a = v < 0 ? -v : v;
            if (a > amax) amax = a;
        }
        volatile float s = amax ? 127.0f / (float)amax : 0.0f;
        for (uint32_t k = 0; k < K; k++) {
            int v = A[(uint64_t)m * lda + k] + (B ? B[(uint64_t)m * ldb + k] : 0);
            volatile float prod = (float)v * s;
            int q = (int)rintf(prod);
            if (q > 127) q = 127;
            if (q < -127) q = -127;
            out[(uint64_t)m * K + k] = (int8_t)q;
        }
        if (scale) scale[m] = (float)amax / 127.0f;
    }
}

/* Absmean ternarisation of real-valued weights (BitNet b1.58): scale = mean(|W|) over the matrix,
 * W_t = clamp(round_half_even(W / (scale + 1e-5)), -1, +1).  The reference has no such step (its
 * matrices are synthetic, main.cu:248-265); this restates the rule the library's
 * sptmm_ternarise_absmean implements, for the tests.  W: K x N fp32, column-major; the mean is a
 * double-precision sum per column, the columns added in order. */
void oracle_ternarise_absmean(const float *W, uint32_t K, uint32_t N, int8_t *out, float *scale)
{
    double total = 0.0;
    for (uint32_t c = 0; c < N; c++) {
        double s = 0.0;
        for (uint32_t k = 0; k < K; k++) s += fabs((double)W[(uint64_t)c * K + k]);
        total += s;
    }
    volatile float mean = (float)(total / ((double)K * N));
    volatile float inv = 1.0f / (mean + 1e-5f);
    for (uint64_t i = 0; i < (uint64_t)K * N; i++) {
        volatile float prod = W[i] * inv;
        float q = rintf(prod);
        out[i] = (int8_t)(q > 1.0f ? 1 : (q < -1.0f ? -1 : (int)q));
    }
    if (scale) *scale = mean;
}
