// stack.cpp -- a BitNet-b1.58-shaped stack of ternary layers behind the C ABI (host C++ only: it
// is written against include/sptmm.h like any other caller and needs no CUDA header).
//
// The reference has no layer stack, no quantiser and no multi-GPU path; the shapes are the ones
// its dispatch ladders hard-code (main.cu:1107-1190: fused qkv N = hidden + 2 kv and gate|up
// N = 2 ffn at K = hidden, down ffn x hidden).  Per layer, four dependent steps on int8
// activations with int32 results, the per-row absmax re-quantisation fused into the next step:
//     qkv  = Wqkv(x)                 x: the previous layer's `down` output
//     o    = Wo(qkv[:, :hidden])     (stand-in for attention: the q part)
//     gu   = Wgu(o)                  gate | up fused along N with their columns interleaved; the
//                                    step stores gate_j + up_j
//     down = Wdown(gu)
// Every matrix is sharded by contiguous column ranges over the ranks of one node.  A forward pass
// is one persistent kernel per rank (sptmm_seq_*); across GPUs each rank's kernel stores its
// output columns into every rank's copy of the activation buffers, which therefore live in an
// arena the CALLER allocates so that every rank can address every rank's copy (CUDA IPC, the
// virtual memory API, a symmetric-memory allocator: the caller's choice).
#include <algorithm>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "internal.h"

using namespace sptmm;

namespace {

struct Shape { const char *name; uint32_t K, N; };

std::vector<Shape> layer_shapes(uint32_t hidden, uint32_t ffn, uint32_t kv)
{
    return {{"qkv", hidden, hidden + 2 * kv}, {"o", hidden, hidden}, {"gu", hidden, 2 * ffn}, {"down", ffn, hidden}};
}

uint64_t matrix_seed(uint64_t seed, uint32_t layer, uint32_t which) { return seed * 1000003ull + (uint64_t)layer * 16 + which; }

void shard_range(uint32_t n, uint32_t rank, uint32_t world, uint32_t &c0, uint32_t &c1)
{
    c0 = (uint32_t)((uint64_t)n * rank / world);
    c1 = (uint32_t)((uint64_t)n * (rank + 1) / world);
}

uint64_t align256(uint64_t v) { return (v + 255) & ~(uint64_t)255; }

}  // namespace

struct sptmm_stack_weights {
    sptmm_stack_config cfg{};
    std::vector<sptmm_weights *> w;          // 4 per layer, this rank's columns
    uint64_t stream_bytes = 0, params = 0;
    ~sptmm_stack_weights() { for (sptmm_weights *x : w) sptmm_weights_free(x); }
};

struct sptmm_stack {
    sptmm_stack_weights *weights = nullptr;  // not owned
    uint32_t M = 0, exchange = 0, n_steps = 0, chains = 1, rows = 0;
    bool tagged = false;                     // the intermediate buffers hold tagged words
    sptmm_seq *seq = nullptr;
    void *own_arena = nullptr;               // allocated here (one rank, no arena given)
    char *mine = nullptr;                    // this rank's arena
    uint64_t off_counters = 0, off_x = 0, off_scales = 0;
    uint64_t off_buf[2][5] = {};             // per half-batch: qkv, o, gu, down, out
    uint32_t width[5] = {};
    ~sptmm_stack()
    {
        if (seq) sptmm_seq_free(seq);
        if (own_arena) sptmm_dev_free(own_arena);
    }
};

static int check_config(const sptmm_stack_config *c, const char *who)
{
    if (!c) return fail(SPTMM_ERR_INVALID, "%s: null configuration", who);
    if (c->layers == 0 || c->hidden == 0 || c->ffn == 0 || c->world == 0 || c->world > 8 || c->rank >= c->world)
        return fail(SPTMM_ERR_INVALID, "%s: layers=%u hidden=%u ffn=%u rank %u of %u", who, c->layers, c->hidden, c->ffn, c->rank, c->world);
    if (c->hidden >= 65536 || c->ffn >= 65536) return fail(SPTMM_ERR_INVALID, "%s: rows are indexed with 16 bits (hidden=%u, ffn=%u)", who, c->hidden, c->ffn);
    if ((2 * c->ffn) % (2 * c->world)) return fail(SPTMM_ERR_INVALID, "%s: the fused gate|up columns (2 x %u) must split into even shards over %u ranks", who, c->ffn, c->world);
    return SPTMM_OK;
}

extern "C" int sptmm_stack_weights_create(const sptmm_stack_config *cfg, sptmm_stack_weights **out)
{
    if (!out) return fail(SPTMM_ERR_INVALID, "stack_weights_create: null pointer");
    *out = nullptr;
    int rc = check_config(cfg, "stack_weights_create");
    if (rc != SPTMM_OK) return rc;
    std::unique_ptr<sptmm_stack_weights> sw(new (std::nothrow) sptmm_stack_weights());
    if (!sw) return fail(SPTMM_ERR_NOMEM, "stack_weights_create: out of host memory");
    sw->cfg = *cfg;
    const auto shapes = layer_shapes(cfg->hidden, cfg->ffn, cfg->kv);
    std::vector<int8_t> W, Wi;
    for (uint32_t l = 0; l < cfg->layers; l++)
        for (uint32_t i = 0; i < 4; i++) {
            const uint32_t K = shapes[i].K, N = shapes[i].N;
            W.resize((size_t)K * N);
            rc = sptmm_gen_ternary_iid(K, N, cfg->p_zero, matrix_seed(cfg->seed, l, i), W.data());     // identical on every rank
            if (rc != SPTMM_OK) return rc;
            const int8_t *src = W.data();
            if (i == 2) {            // columns g0,u0,g1,u1,...: a pair-summing step adds gate_j and up_j
                Wi.resize(W.size());
                for (uint32_t j = 0; j < cfg->ffn; j++) {
                    memcpy(Wi.data() + (size_t)(2 * j) * K, W.data() + (size_t)j * K, K);
                    memcpy(Wi.data() + (size_t)(2 * j + 1) * K, W.data() + (size_t)(cfg->ffn + j) * K, K);
                }
                src = Wi.data();
            }
            uint32_t c0, c1;
            shard_range(N, cfg->rank, cfg->world, c0, c1);
            sptmm_weights *w = nullptr;
            rc = sptmm_encode(src + (size_t)c0 * K, K, c1 - c0, SPTMM_FMT_U16_V256, 32, 0, &w);
            if (rc == SPTMM_OK) {
                sw->w.push_back(w);
                rc = sptmm_weights_upload(w);
            }
            if (rc != SPTMM_OK) return rc;
            sptmm_weights_info info;
            sptmm_weights_info_get(w, &info);
            sw->stream_bytes += info.stream_bytes;
            sw->params += (uint64_t)K * N;
        }
    *out = sw.release();
    return SPTMM_OK;
}

extern "C" int sptmm_stack_weights_info(const sptmm_stack_weights *w, uint64_t *stream_bytes, uint64_t *params)
{
    if (!w) return fail(SPTMM_ERR_INVALID, "stack_weights_info: null handle");
    if (stream_bytes) *stream_bytes = w->stream_bytes;
    if (params) *params = w->params;
    return SPTMM_OK;
}

extern "C" int sptmm_stack_weights_matrix(const sptmm_stack_weights *w, uint32_t index, const sptmm_weights **out)
{
    if (!w || !out || index >= w->w.size()) return fail(SPTMM_ERR_INVALID, "stack_weights_matrix: bad handle or index %u", index);
    *out = w->w[index];
    return SPTMM_OK;
}

extern "C" int sptmm_stack_weights_free(sptmm_stack_weights *w)
{
    delete w;
    return SPTMM_OK;
}

// Which exchange a stack uses when the caller leaves it open (exchange 0), from measurements on B200:
// the settled exchange wins across GPUs at every M and on one GPU from eight rows upward; below that
// the step counters with the reader-side quantiser do.  Across GPUs, twelve rows or more are run as
// two half-batches whose steps alternate (SPTMM_STACK_SETTLED_HALVES): the settle phase of one half
// then runs in warps of its own while the other half is gathered, which hides the hand-over almost
// entirely (the tile is ready 6-10 us before it is needed) -- but two 8-row gathers cost 1.3x one
// 16-row gather and every step's weights are streamed twice, so it nets 8-10 % at M=16 (2 GPUs 2 384
// against 2 602 us per pass, 4 GPUs 1 888 against 2 109) and loses below (M=8: 1 566 against 1 521,
// M=4: 1 592 against 1 371 at 4 GPUs).
static uint32_t pick_exchange(uint32_t exchange, uint32_t M, uint32_t world)
{
    if (exchange) return exchange;
    if (world > 1 && M >= 12 && M % 2 == 0) return SPTMM_STACK_SETTLED_HALVES;
    return (world > 1 || M >= 8) ? SPTMM_STACK_SETTLED : SPTMM_STACK_COUNTERS;
}

struct StackPlan {                 // everything that depends on the configuration, M and the exchange only
    uint32_t chains = 1, rows = 0;              // independent half-batches and the rows of each
    std::vector<sptmm_seq_step> steps;          // X / C hold OFFSETS into a rank's arena until create() adds the base
    std::vector<uint64_t> c_off;                // per step: offset of this rank's first output column
    uint64_t off_counters = 0, off_x = 0, off_scales = 0, off_buf[2][5] = {}, bytes = 0;
    uint32_t width[5] = {};
};

static int make_plan(const sptmm_stack_weights *sw, uint32_t M, uint32_t exchange, StackPlan &pl)
{
    const sptmm_stack_config &c = sw->cfg;
    const uint32_t layer_steps = 4 * c.layers, hidden = c.hidden, ffn = c.ffn;
    const auto shapes = layer_shapes(hidden, ffn, c.kv);
    uint32_t xk, xw;               // readers of part of a row / of a whole row
    pl.chains = 1;
    switch (exchange) {
        case SPTMM_STACK_COUNTERS: xk = xw = 1; break;
        case SPTMM_STACK_TAGGED: xk = xw = 2; break;
        case SPTMM_STACK_ROW_MAXIMA: xk = 1; xw = 3; break;
        case SPTMM_STACK_PRODUCER_QUANT: xk = xw = 4; break;
        case SPTMM_STACK_SETTLED: xk = xw = 5; break;
        case SPTMM_STACK_SETTLED_HALVES:
            xk = xw = 5; pl.chains = 2;
            if (M < 2 || (M & 1)) return fail(SPTMM_ERR_INVALID, "stack: two half-batches need an even number of rows (M=%u)", M);
            break;
        default: return fail(SPTMM_ERR_INVALID, "stack: unknown exchange %u", exchange);
    }
    const uint32_t chains = pl.chains, rows = M / chains, n_steps = layer_steps * chains;
    pl.rows = rows;
    pl.width[0] = shapes[0].N; pl.width[1] = hidden; pl.width[2] = ffn; pl.width[3] = hidden; pl.width[4] = hidden;
    pl.steps.assign(n_steps, sptmm_seq_step{});
    pl.c_off.assign(n_steps, 0);
    // Step t = chains * s + h is layer step s of half-batch h; it reads what step t - chains wrote.
    // Sizes first: the synchronisation area depends on the step kinds and shapes only.
    for (uint32_t t = 0; t < n_steps; t++) {
        sptmm_seq_step &st = pl.steps[t];
        const uint32_t s = t / chains, i = s % 4;
        st.w = sw->w[s];
        st.dep = s == 0 ? -1 : (int32_t)(t - chains);
        st.x_kind = s == 0 ? 0 : (i == 1 ? xk : xw);
        st.c_kind = i == 2 ? 1 : 0;
        st.X = reinterpret_cast<const void *>((uintptr_t)16);       // placeholders: the layout does not look at addresses
        st.C = reinterpret_cast<void *>((uintptr_t)16);
    }
    uint64_t cur = 0;
    pl.off_counters = cur;
    cur += sptmm_seq_shared_bytes_for(pl.steps.data(), n_steps, rows);
    for (uint32_t h = 0; h < chains; h++)
        for (int b = 0; b < 5; b++) {
            cur = align256(cur);
            pl.off_buf[h][b] = cur;
            cur += (uint64_t)rows * pl.width[b] * 4;
        }
    cur = align256(cur);
    pl.off_x = cur; cur += align256((uint64_t)rows * hidden) * chains;
    cur = align256(cur);
    pl.off_scales = cur; cur += (uint64_t)n_steps * rows * 4;
    pl.bytes = align256(cur);
    // the steps, with offsets where addresses will go
    static const int src_of[4] = {3, 0, 1, 2};       // qkv reads down, o reads qkv, gu reads o, down reads gu
    for (uint32_t t = 0; t < n_steps; t++) {
        sptmm_seq_step &st = pl.steps[t];
        const uint32_t s = t / chains, h = t % chains, i = s % 4;
        const int dst = s == layer_steps - 1 ? 4 : (int)i;  // the last step's result: never tagged, no reader inside the kernel
        uint32_t c0, c1;
        shard_range(shapes[i].N, c.rank, c.world, c0, c1);
        const uint32_t o0 = i == 2 ? c0 / 2 : c0;           // where this rank's first output column lands
        pl.c_off[t] = pl.off_buf[h][dst] + (uint64_t)o0 * 4;
        st.ldc = pl.width[dst];
        if (s == 0) {
            st.X = reinterpret_cast<const void *>((uintptr_t)(pl.off_x + h * align256((uint64_t)rows * hidden)));
            st.ldx = hidden;
        } else {
            st.X = reinterpret_cast<const void *>((uintptr_t)pl.off_buf[h][src_of[i]]);
            st.ldx = pl.width[src_of[i]];
        }
        st.scale_out = reinterpret_cast<float *>((uintptr_t)(pl.off_scales + (uint64_t)t * rows * 4));
    }
    return SPTMM_OK;
}

extern "C" uint64_t sptmm_stack_arena_bytes(const sptmm_stack_weights *w, uint32_t M, uint32_t exchange)
{
    if (!w || M == 0 || M > 16) return 0;
    StackPlan pl;
    if (make_plan(w, M, pick_exchange(exchange, M, w->cfg.world), pl) != SPTMM_OK) return 0;
    return pl.bytes;
}

extern "C" int sptmm_stack_create(sptmm_stack_weights *w, uint32_t M, uint32_t exchange, void *const *arena_peers,
                                  sptmm_stack **out)
{
    if (!w || !out) return fail(SPTMM_ERR_INVALID, "stack_create: null pointer");
    *out = nullptr;
    if (M == 0 || M > 16) return fail(SPTMM_ERR_UNSUPPORTED, "stack_create: M=%u, the sequence kernel blocks 1..16 rows", M);
    const sptmm_stack_config &c = w->cfg;
    if (c.world > 1 && !arena_peers) return fail(SPTMM_ERR_INVALID, "stack_create: %u ranks need every rank's arena", c.world);
    std::unique_ptr<sptmm_stack> st(new (std::nothrow) sptmm_stack());
    if (!st) return fail(SPTMM_ERR_NOMEM, "stack_create: out of host memory");
    st->weights = w; st->M = M;
    st->exchange = pick_exchange(exchange, M, c.world);
    st->tagged = st->exchange == SPTMM_STACK_TAGGED || st->exchange == SPTMM_STACK_SETTLED || st->exchange == SPTMM_STACK_SETTLED_HALVES;
    StackPlan pl;
    int rc = make_plan(w, M, st->exchange, pl);
    if (rc != SPTMM_OK) return rc;
    st->n_steps = (uint32_t)pl.steps.size(); st->chains = pl.chains; st->rows = pl.rows;
    std::vector<char *> bases(c.world, nullptr);
    if (arena_peers) {
        for (uint32_t r = 0; r < c.world; r++) {
            if (!arena_peers[r]) return fail(SPTMM_ERR_INVALID, "stack_create: no arena for rank %u", r);
            bases[r] = static_cast<char *>(arena_peers[r]);
        }
    } else {
        rc = sptmm_dev_alloc(&st->own_arena, pl.bytes);
        if (rc != SPTMM_OK) return rc;
        std::vector<char> zero(pl.bytes, 0);
        rc = sptmm_memcpy_h2d(st->own_arena, zero.data(), pl.bytes);
        if (rc != SPTMM_OK) return rc;
        bases[0] = static_cast<char *>(st->own_arena);
    }
    st->mine = bases[c.rank];
    st->off_counters = pl.off_counters; st->off_x = pl.off_x; st->off_scales = pl.off_scales;
    for (int h = 0; h < 2; h++)
        for (int b = 0; b < 5; b++) st->off_buf[h][b] = pl.off_buf[h][b];
    for (int b = 0; b < 5; b++) st->width[b] = pl.width[b];
    std::vector<void *> c_peers((size_t)st->n_steps * c.world), counter_peers(c.world);
    for (uint32_t s = 0; s < st->n_steps; s++) {
        sptmm_seq_step &sd = pl.steps[s];
        sd.X = st->mine + (uintptr_t)sd.X;
        sd.scale_out = reinterpret_cast<float *>(st->mine + (uintptr_t)sd.scale_out);
        sd.C = st->mine + pl.c_off[s];
        for (uint32_t r = 0; r < c.world; r++) c_peers[(size_t)s * c.world + r] = bases[r] + pl.c_off[s];
    }
    for (uint32_t r = 0; r < c.world; r++) counter_peers[r] = bases[r] + pl.off_counters;
    if (c.world > 1)
        rc = sptmm_seq_create_shared(pl.steps.data(), st->n_steps, pl.rows, c_peers.data(), counter_peers.data(), c.world, c.rank, &st->seq);
    else            // one rank: the sequence keeps its counters itself (device scope, no peer stores)
        rc = sptmm_seq_create(pl.steps.data(), st->n_steps, pl.rows, &st->seq);
    if (rc != SPTMM_OK) return rc;
    *out = st.release();
    return SPTMM_OK;
}

extern "C" int sptmm_stack_set_input(sptmm_stack *st, const int8_t *x_host)
{
    if (!st || !x_host) return fail(SPTMM_ERR_INVALID, "stack_set_input: null pointer");
    const uint64_t half = (uint64_t)st->rows * st->weights->cfg.hidden;      // rows 0..rows-1 go to the first half-batch, the rest to the second
    for (uint32_t h = 0; h < st->chains; h++) {
        const int rc = sptmm_memcpy_h2d(st->mine + st->off_x + h * align256(half), x_host + h * half, half);
        if (rc != SPTMM_OK) return rc;
    }
    return SPTMM_OK;
}

extern "C" int sptmm_stack_forward(sptmm_stack *st, void *stream)
{
    if (!st) return fail(SPTMM_ERR_INVALID, "stack_forward: null handle");
    return sptmm_seq_run(st->seq, stream);
}

extern "C" int sptmm_stack_status(sptmm_stack *st, uint32_t *status)
{
    if (!st || !status) return fail(SPTMM_ERR_INVALID, "stack_status: null pointer");
    return sptmm_seq_status(st->seq, status, nullptr);
}

extern "C" int sptmm_stack_exchange(const sptmm_stack *st, uint32_t *exchange)
{
    if (!st || !exchange) return fail(SPTMM_ERR_INVALID, "stack_exchange: null pointer");
    *exchange = st->exchange;
    return SPTMM_OK;
}

extern "C" int sptmm_stack_sequence(sptmm_stack *st, sptmm_seq **seq)
{
    if (!st || !seq) return fail(SPTMM_ERR_INVALID, "stack_sequence: null pointer");
    *seq = st->seq;
    return SPTMM_OK;
}

extern "C" int sptmm_stack_wait_limit(sptmm_stack *st, uint32_t polls)
{
    if (!st) return fail(SPTMM_ERR_INVALID, "stack_wait_limit: null handle");
    return sptmm_seq_set_wait_limit(st->seq, polls);
}

extern "C" int sptmm_stack_buffer(sptmm_stack *st, const char *name, int32_t *host_out, uint32_t *width)
{
    if (!st || !name) return fail(SPTMM_ERR_INVALID, "stack_buffer: null pointer");
    static const char *names[4] = {"qkv", "o", "gu", "down"};
    int b = -1;
    for (int i = 0; i < 4; i++) if (strcmp(name, names[i]) == 0) b = i;
    if (b < 0) return fail(SPTMM_ERR_INVALID, "stack_buffer: no buffer called %s (qkv, o, gu, down)", name);
    const int src = b == 3 ? 4 : b;                   // "down" = the stack's final result
    if (width) *width = st->width[src];
    if (!host_out) return SPTMM_OK;
    const size_t n = (size_t)st->M * st->width[src], per_half = (size_t)st->rows * st->width[src];
    int rc = sptmm_device_sync();
    for (uint32_t h = 0; h < st->chains && rc == SPTMM_OK; h++)
        rc = sptmm_memcpy_d2h(host_out + h * per_half, st->mine + st->off_buf[h][src], per_half * 4);
    if (rc != SPTMM_OK) return rc;
    if (st->tagged && src != 4)
        for (size_t i = 0; i < n; i++) host_out[i] = (int32_t)((uint32_t)host_out[i] << 8) >> 8;     // drop the tag byte, sign-extend 24 bits
    return SPTMM_OK;
}

extern "C" int sptmm_stack_free(sptmm_stack *st)
{
    delete st;
    return SPTMM_OK;
}
