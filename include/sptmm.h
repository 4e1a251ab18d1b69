/*
 * sptmm.h -- C ABI of the B200 (sm_100a) ternary sparse matmul library.
 *
 * Computes C = X * W for W in {-1,0,+1}^(K x N) stored as per-column sorted row-index lists
 * (one list for the +1 rows, one for the -1 rows) with add/subtract-only gathers.
 * It replaces, for that one path, the reference program Ogiwara-CostlierRain464/SpTMM
 * (a single main.cu); each entry point cites the reference lines it stands in for.
 *
 * Conventions
 *  - every function returns 0 on success or a negative sptmm_status; sptmm_last_error()
 *    gives the message of the calling thread's last failure.  Nothing here calls exit/abort.
 *  - "device pointer" = memory of the CUDA device current at the call; `stream` is a
 *    cudaStream_t passed as void* (NULL = default stream, which is what the reference uses,
 *    main.cu:1861).  Launches are asynchronous unless stated otherwise.
 *  - X is M x K, C is M x N.  Row-major unless a layout flag says otherwise
 *    (reference "rcr" build, script/make_rcr.sh:6).
 */
#ifndef SPTMM_H
#define SPTMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum sptmm_status {
    SPTMM_OK = 0,
    SPTMM_ERR_INVALID = -1,      /* bad argument / shape constraint violated              */
    SPTMM_ERR_CUDA = -2,         /* a CUDA runtime call failed                            */
    SPTMM_ERR_UNSUPPORTED = -3,  /* valid request this build cannot serve                 */
    SPTMM_ERR_LOSSY = -4,        /* encoding cannot represent the matrix exactly          */
    SPTMM_ERR_NOMEM = -5,
    SPTMM_ERR_STATE = -6         /* e.g. weights not uploaded to the current device       */
} sptmm_status;

typedef enum sptmm_format {
    /* reference layout W_map_{8,16,32}_div (main.cu:345-373): u16, [chunk][column][split]   */
    SPTMM_FMT_U16_DIV = 1,
    /* reference layout W_map_delta2_div256 (main.cu:376-413): u8 gaps, [block][column][256] */
    SPTMM_FMT_DELTA_DIV256 = 2,
    /* native: u16, 256-entry blocks pre-interleaved for 16-byte-per-lane loads              */
    SPTMM_FMT_U16_V256 = 3,
    /* native narrow-integer variant: 304-byte blocks of eight 32-lane gather steps; a step is
     * a 32-bit base row, a count and one 8-bit offset per lane (1.19 bytes per entry, exact:
     * a step that would span more than 255 rows is cut short instead)                        */
    SPTMM_FMT_DELTA_LANE = 4,
    /* comparator: 2-bit codes, 16 rows per 32-bit word (bitnet_kernels.cuh:52-72)           */
    SPTMM_FMT_I2S = 5
} sptmm_format;

typedef enum sptmm_dtype { SPTMM_I8 = 0, SPTMM_F16 = 1, SPTMM_F32 = 2 } sptmm_dtype;

/* bit flags for the `flags` argument of the launch functions */
enum {
    SPTMM_X_COLMAJOR = 1,   /* X(m,k) at k*M+m  (reference "ccc" build, script/make_ccc.sh:6) */
    SPTMM_C_COLMAJOR = 2,   /* C(m,n) at n*M+m                                               */
    SPTMM_LAUNCH_PDL = 4    /* programmatic dependent launch: this call's weight prefetch may
                               overlap the tail of the previous kernel in the stream; X is read
                               and C written only after that kernel has completed             */
};

typedef struct sptmm_weights sptmm_weights;   /* opaque, host-owned encoded matrix */

typedef struct sptmm_weights_info {
    uint32_t K, N;
    uint32_t format;        /* sptmm_format                                                  */
    uint32_t split;         /* U16_DIV: 8/16/32; native formats: 32 (lanes per gather step)  */
    uint32_t S;             /* 2 x padded per-sign list capacity (reference -S) where uniform */
    uint32_t max_count;     /* longest single-sign list                                      */
    uint64_t nnz;           /* non-zeros of W                                                */
    uint64_t stream_bytes;  /* bytes of encoded arrays one matmul reads (roofline numerator) */
    uint64_t lossy_entries; /* DELTA_DIV256: entries whose 8-bit store lost information      */
    uint32_t n_arrays;      /* number of encoded arrays, see sptmm_weights_array             */
    int32_t  device;        /* device the arrays are uploaded to, -1 if none                 */
    uint32_t k_tile;        /* rows per K-tile of a K-tiled matrix, else 0                   */
    uint32_t n_tiles;       /* number of K-tiles, else 0                                     */
} sptmm_weights_info;

const char *sptmm_last_error(void);
int sptmm_version(void);

/* ---- weight generation (host).  W is column-major K x N int8 (W_MAJOR = MAJOR_COL).        */

/* Reference generator, bit-exact: S/2 entries -1 and S/2 entries +1 per column, Fisher-Yates
 * with xorshift32 seeded 0xCAFEBABE ^ column (main.cu:248-265, macro.cuh:69-76). */
int sptmm_gen_ternary_fixed(uint32_t K, uint32_t N, uint32_t S, int8_t *W);

/* No counterpart in the reference: i.i.d. entries, P(0)=p_zero, P(+1)=P(-1), splitmix64 per column. */
int sptmm_gen_ternary_iid(uint32_t K, uint32_t N, double p_zero, uint64_t seed, int8_t *W);

/* Real-valued weights -> ternary, the absmean rule of BitNet b1.58 (no counterpart in the reference,
 * whose matrices are synthetic, main.cu:248-265): scale = mean(|W|) over the matrix,
 * W_t = clamp(round_half_even(W / (scale + 1e-5)), -1, +1), so that W ~ scale * W_t.
 * W: K x N column-major like every matrix here, `dtype` SPTMM_F16 or SPTMM_F32 (host memory);
 * W_ternary: K x N int8 ready for sptmm_encode; *scale (optional): the factor a de-quantising
 * epilogue multiplies by (sptmm_gemv_scaled's w_scale). */
int sptmm_ternarise_absmean(const void *W, uint32_t dtype, uint32_t K, uint32_t N, int8_t *W_ternary, float *scale);

/* ---- encoding (host).  Replaces the device-side encoder prepareW_map (main.cu:202-489).    */

/* S = 0 derives the per-sign capacity from the longest list (rounded up as the format needs);
 * S > 0 fixes it at S/2 as the reference's -S flag does and fails if a column has more.
 * `split`: U16_DIV 8|16|32 (reference -row_split3_small values, main.cu:998-1059);
 *          the other formats ignore it. */
int sptmm_encode(const int8_t *W, uint32_t K, uint32_t N, uint32_t format, uint32_t split,
                 uint32_t S, sptmm_weights **out);
/* The same matrix cut along K ("chunked for split-K"): tile t holds rows t*k_tile .. of W as a
 * native u16 matrix of its own, row numbers counted from the tile's first row (k_tile a multiple
 * of 16).  The reference splits K only by striding lanes over one list (main.cu:581-584).
 *  - sptmm_gemv on the handle multiplies tile after tile on the stream, the first storing C and
 *    the others adding to it: the activation tile in shared memory is k_tile rows long instead of
 *    K, so up to sixteen rows of X share one pass over the indices however long K is (int sums
 *    exact as ever; float sums are added tile by tile).
 *  - sptmm_weights_tile hands out one tile as a handle of its own (owned by the parent), e.g. for
 *    the rank that owns that K range in sptmm_gemv_reduce: one encoding serves every rank, each
 *    uploads only its tile.
 * sptmm_weights_upload on the parent uploads every tile; save/load take single tiles. */
int sptmm_encode_ktiled(const int8_t *W, uint32_t K, uint32_t N, uint32_t k_tile, sptmm_weights **out);
int sptmm_weights_tile(const sptmm_weights *w, uint32_t tile, sptmm_weights **out);
int sptmm_weights_info_get(const sptmm_weights *w, sptmm_weights_info *info);
/* Encoded array `i` on the host (byte-for-byte what is uploaded).  For U16_DIV: 0 = +1 lists,
 * 1 = -1 lists; DELTA_DIV256 likewise.  Native formats: 0 = payload, then metadata arrays. */
int sptmm_weights_array(const sptmm_weights *w, uint32_t i, const void **host_ptr,
                        const void **device_ptr, uint64_t *bytes, const char **name);
/* Copy the arrays to the current device (one cudaMalloc per array; synchronous). */
int sptmm_weights_upload(sptmm_weights *w);
/* Upload `copies` independent replicas (for cold-cache timing); replica r is selected per call. */
int sptmm_weights_upload_replicas(sptmm_weights *w, uint32_t copies);
int sptmm_weights_free(sptmm_weights *w);

/* Encoded weights on disk (no counterpart in the reference, which re-encodes on the GPU at every
 * start, main.cu:972).  save writes the host-side arrays with a header (shape, format, counts)
 * and a checksum; load rebuilds a handle ready for sptmm_weights_upload and rejects files whose
 * header, array sizes, row indices or checksum do not fit together. */
int sptmm_weights_save(const sptmm_weights *w, const char *path);
int sptmm_weights_load(const char *path, sptmm_weights **out);

/* ---- the matmul ---------------------------------------------------------------------------- */

/* C = X*W with uploaded weights of any format.  X: device, `dtype` elements; C: device, int32
 * for SPTMM_I8 (exact), float for F16/F32 (fp32 accumulation).  `replica` picks the weight copy
 * (0 unless upload_replicas was used).  No allocation, no synchronisation on this path.
 * Stands in for the launches of main.cu:993-1460 / 1463-1846 / 1864-1961. */
int sptmm_gemv(const sptmm_weights *w, const void *X, uint32_t dtype, uint32_t M, void *C,
               uint32_t flags, uint32_t replica, void *stream);

/* The steps either side of the matmul in a quantised layer; the reference has neither (its
 * activations start as int8, main.cu:787-797, and its results stay raw int32, main.cu:591-593).
 *
 * sptmm_quantize_absmax: int32 rows -> int8 with one scale per row,
 *     q = clamp(rint(v * (127 / absmax)), -127, 127),  scale[m] = absmax / 127   (fp32 throughout;
 *     a row of zeros gives zeros and scale 0).
 *   X: device int32; element (m, k) at X[m*ldx + k] (ldx 0 = the row length), or, with shard > 0,
 *   where an all-gather of per-rank column shards leaves it: rank r's M x shard block after rank
 *   r-1's.  pair != 0: the value quantised is X(m, 2k) + X(m, 2k+1) (a fused gate | up output with
 *   its columns interleaved).  Xq: device int8, M x K row-major.  scale: device float[M] or NULL.
 * sptmm_gemv_scaled: the matmul on int8 activations with the de-quantisation fused into its
 *   epilogue: C (device float, M x N) = float(sum) * (row_scale[m] * w_scale); row_scale is a device
 *   float[M] (NULL = 1), e.g. the scale sptmm_quantize_absmax wrote; native formats only. */
int sptmm_quantize_absmax(const int32_t *X, uint32_t M, uint32_t K, uint32_t ldx, uint32_t shard, uint32_t pair,
                          int8_t *Xq, float *scale, uint32_t flags, void *stream);
int sptmm_gemv_scaled(const sptmm_weights *w, const int8_t *X, uint32_t M, float *C, const float *row_scale,
                      float w_scale, uint32_t flags, uint32_t replica, void *stream);

/* The kernels behind sptmm_gemv bound every wait they make (on a bulk copy's barrier); if one runs
 * out the kernel stores a non-zero word in device memory and finishes with whatever sums it has
 * (the reference's kernels have no waits and no such word; main.cu:556-594).  This waits for the
 * device and reads that word: 0 = every call on this handle since upload completed normally.
 * The host-buffer calls below check it by themselves and return SPTMM_ERR_STATE. */
int sptmm_gemv_status(const sptmm_weights *w, uint32_t *status);

/* Split-K across the GPUs of one node: the matmul fused with the reduce-scatter of its partial
 * sums.  No counterpart in the reference (single GPU).  Every rank holds the rows k0..k1 of W
 * (encoded as a (k1-k0) x N matrix, native u16 format) and the matching slice of X, and calls this
 * with the same C_peers: C_peers[r] is rank r's buffer of M x (N*(r+1)/n_peers - N*r/n_peers)
 * int32 / float, row-major, holding columns N*r/n_peers .. of the result.  Instead of storing a
 * column's partial sum the kernel ADDS it (red.global.add) to its owner's buffer, over NVLink for a
 * peer: when all ranks' kernels are done, rank r's buffer holds its columns of X*W summed over the
 * whole K.  The caller zeroes the buffers and separates zeroing, the calls and reading with a
 * barrier on the stream (e.g. a collective).  int32 sums are exact; float sums depend on the
 * order the additions arrive in (last-bit differences between runs).  Peer pointers only ever
 * see plain reductions -- no multicast or bulk loads touch them. */
int sptmm_gemv_reduce(const sptmm_weights *w, const void *X, uint32_t dtype, uint32_t M,
                      void *const *C_peers, uint32_t n_peers, uint32_t flags, uint32_t replica,
                      void *stream);

/* Same, but X and C are HOST buffers: copies X in, runs, copies C out, waits.  Uses pinned
 * staging owned by the handle (slot 0 of the asynchronous form below; not re-entrant per handle). */
int sptmm_gemv_host(sptmm_weights *w, const void *X_host, uint32_t dtype, uint32_t M, void *C_host,
                    uint32_t flags, uint32_t replica);

/* The host-buffer call in two halves, so that independent calls overlap: _async copies X into the
 * slot's pinned staging, enqueues the copy to the device and the kernel on the slot's own stream
 * and returns; _wait blocks until that call is done and copies the result (which the kernel stored
 * straight into mapped pinned memory) to the C_host given to _async.  Sixteen slots per handle;
 * issuing on a busy slot waits for it first.  X_host may be reused as soon as _async returns,
 * C_host must stay valid until _wait.  A slot belongs to one host thread at a time; different
 * slots of one handle may be driven from different host threads at once (each with the handle's
 * device current), which is how a host gets past one thread's launch rate. */
int sptmm_gemv_host_async(sptmm_weights *w, const void *X_host, uint32_t dtype, uint32_t M, void *C_host,
                          uint32_t flags, uint32_t replica, uint32_t slot);
int sptmm_gemv_host_wait(sptmm_weights *w, uint32_t slot);

/* A list of n independent host-buffer calls on one handle: call i takes X_hosts[i] (M rows each),
 * delivers to C_hosts[i] and streams weight copy replicas[i] (copy 0 when replicas is null).  The
 * calls go round the slots slot0 .. slot0+nslots-1 (nslots of them in flight at once) and all have
 * delivered when the function returns; on an error the calls issued so far are waited for and the
 * first error is returned.  Two host threads may each run a list on their own slots. */
int sptmm_gemv_host_batch(sptmm_weights *w, uint32_t n, const void *const *X_hosts, void *const *C_hosts,
                          const uint32_t *replicas, uint32_t dtype, uint32_t M, uint32_t flags,
                          uint32_t slot0, uint32_t nslots);

/* Raw-pointer forms with the reference's kernel argument convention (X, W_pos, W_neg, C), for a
 * caller that built the reference layouts itself.
 * rowWiseSplit3Small4<M,K,N,S,SPLIT><<<...>>>(X, W_map_SPLIT_div, W_map_negative_SPLIT_div, C)
 * (main.cu:556-594, launches main.cu:1000-1448). */
int sptmm_row_split3_small(const int8_t *X, const uint16_t *W_pos_div, const uint16_t *W_neg_div,
                           int32_t *C, uint32_t M, uint32_t K, uint32_t N, uint32_t S,
                           uint32_t split, void *stream);
/* rowWiseSplit2DeltaSmallAsync2/3<M,K,N,S,32><<<...>>>(X, W_map_delta2_div256,
 * W_map_negative_delta2_div256, C) (main.cu:599-764, launches main.cu:1468-1830).  Indices are
 * rebuilt modulo 65536 exactly as the reference does; a rebuilt index >= K contributes 0. */
int sptmm_row_split_delta2(const int8_t *X, const uint8_t *W_pos_delta, const uint8_t *W_neg_delta,
                           int32_t *C, uint32_t M, uint32_t K, uint32_t N, uint32_t S,
                           uint32_t split, void *stream);

/* ---- comparators --------------------------------------------------------------------------- */

/* Dense int8 x int8 -> int32 through cublasGemmEx, column-major operands as main.cu:856-867
 * (X: M x K lda=M, W: K x N ldb=K, C: M x N ldc=M).  W_dense is a device pointer the caller
 * filled (the reference passes a null W, main.cu:837,863).  Reported reference only. */
int sptmm_dense_cublas_gemm(const int8_t *X_colmajor, const int8_t *W_dense, int32_t *C_colmajor,
                            uint32_t M, uint32_t K, uint32_t N, void *stream);
/* The same with fp16 X and W (W holds -1, 0, +1 as fp16), fp32 accumulation and output: the dense
 * comparator of the large fp16 sweeps.  No counterpart in the reference. */
int sptmm_dense_cublas_gemm_f16(const void *X_colmajor, const void *W_dense, float *C_colmajor,
                                uint32_t M, uint32_t K, uint32_t N, void *stream);

/* ---- sequences of matmuls in one launch ----------------------------------------------------- */

/* No counterpart in the reference, which launches one kernel per matmul and synchronises the host
 * after each (main.cu:994-1458).  A sequence is a fixed list of steps C = X*W (native u16 format,
 * int8 activations, int32 results, M <= 16) that one persistent kernel runs back to back, with
 * the next step's weights streaming from HBM while the current one is gathered. */
typedef struct sptmm_seq sptmm_seq;

typedef struct sptmm_seq_step {
    const sptmm_weights *w;  /* uploaded to the current device                                   */
    uint32_t replica;        /* which uploaded copy of w                                          */
    uint32_t x_kind;         /* 0: X is int8.  1: X (and X2, if set) are int32 results of earlier
                                steps; their sum is quantised per row to int8 with
                                q = clamp(rint(v * (127/absmax)), -127, 127) before the matmul.
                                2: as 1, with the tagged exchange: X (and X2) lie in the output of
                                step `dep`, which then stores every result as
                                (tag << 24) | (value & 0xffffff) -- the tag changes with every
                                write of the buffer -- and this step waits for the words
                                themselves to turn current instead of for a step counter (no
                                fence, one memory round trip less per step).  Every step that
                                writes that buffer must feed an x_kind 2 reader; the host sees
                                tagged words there ((int32)(w << 8) >> 8 recovers the value; it
                                always fits, since |value| <= 127*K < 2^23).  A buffer may be
                                rewritten by the second step after the one that reads it, not
                                by the next one.
                                3: as 1 with no X2, and X is the WHOLE output row of step `dep`
                                (all columns, all ranks' shards, ldx = that step's ldc).  The
                                producing step then also records every row's largest magnitude
                                while it stores its results, and this step quantises in one pass
                                over X instead of two (absmax first, values second).
                                4: as 1 with no X2, but the PRODUCING step `dep` does the quantising:
                                X names the first of the K columns inside that step's output (any
                                column range of it), every CTA of that step publishes the row maxima
                                of its own columns, and once it knows the rows' maxima over the
                                whole range it rounds its own columns and stores them as int8 --
                                three rows and a tag to a 32-bit word -- where this step picks them
                                up.  Readers then fetch M*K bytes instead of quantising M*K int32
                                each, which is what pays from a few rows upward (and across GPUs,
                                where every rank's kernel stores its columns into every rank's
                                copy).  The producer still stores its int32 results as usual.
                                All steps that read one producer this way must read the same range.
                                5: as 2 (tagged words in the output of step `dep`, no X2), with the
                                "settled" hand-over: each word is watched by ONE CTA per GPU instead
                                of by all of them (every CTA owns K/CTAs columns), the CTAs of a GPU
                                meet at a local counter once their columns have arrived, and --
                                for two rows or more -- each CTA quantises only its own columns
                                into a local int8 tile that all CTAs then fetch with one bulk copy.
                                Nothing but the producer's tagged words crosses NVLink.            */
    const void *X;           /* device, M rows of K elements, row stride ldx (0 = K)              */
    const void *X2;          /* optional second int32 source, row stride ldx2 (0 = K)             */
    void *C;                 /* device int32, M rows of N, row stride ldc (0 = N)                 */
    float *scale_out;        /* optional device float[M]: absmax/127 of the quantised rows        */
    uint32_t ldx, ldx2, ldc;
    int32_t dep;             /* index of the earlier step whose output this step reads, or -1.
                                A step starts reading X only after step `dep` has finished on the
                                whole device.  Buffers are the caller's: a step must not overwrite
                                memory that a step it does not (transitively) depend on may still
                                be reading.                                                       */
    uint32_t c_kind;         /* 0: C holds the N results of a row.  1: pair sums -- C holds N/2
                                values per row, C[m][j] = result[2j] + result[2j+1] (a fused
                                "gate | up" matrix with its columns interleaved hands the next
                                step one source instead of two); N even, ldc counts output
                                elements.  2: the de-quantising epilogue -- C holds FLOATS,
                                C[m][n] = float(result) * s[m] with s[m] the absmax/127 this step's
                                input stage quantised row m with (1 for int8 inputs, x_kind 0); for
                                the last step of a chain, whose output no later step reads      */
} sptmm_seq_step;

int sptmm_seq_create(const sptmm_seq_step *steps, uint32_t n_steps, uint32_t M, sptmm_seq **out);

/* The same over several GPUs of one node, one process per GPU, each holding a column shard of
 * every matrix (the reference is single-GPU; no counterpart).  Instead of an all-gather after a
 * step, every rank's kernel stores its output columns directly into each peer's copy of the
 * output buffer over NVLink and adds to each peer's step counter; a dependent step waits until
 * all ranks have reported.  No collective call and no NCCL kernel sits on the data path.
 *  - C_peers[s*n_peers + p]: where step s's shard starts in rank p's buffer (peer-mapped device
 *    pointer valid in THIS process, e.g. from CUDA IPC / symmetric memory; p = own rank too).
 *    Each points at column 0 of this rank's shard inside the full-width row (stride ldc).
 *  - counter_peers[p]: rank p's synchronisation area of sptmm_seq_shared_bytes(n_steps) bytes
 *    (step counters, then the row maxima of x_kind 3; sptmm_seq_shared_bytes_for() bytes when
 *    there are x_kind 4 steps), zeroed once before first use, peer-mapped likewise.  All ranks must create the same sequence and run it equally often.
 * steps[].C is ignored when n_peers > 0. */
uint64_t sptmm_seq_shared_bytes(uint32_t n_steps);
/* The same for a sequence with x_kind 4 steps, whose producers keep their row maxima and packed
 * int8 outputs in that area as well: the size depends on the steps and on M (0 on bad arguments). */
uint64_t sptmm_seq_shared_bytes_for(const sptmm_seq_step *steps, uint32_t n_steps, uint32_t M);
int sptmm_seq_create_shared(const sptmm_seq_step *steps, uint32_t n_steps, uint32_t M,
                            void *const *C_peers, void *const *counter_peers, uint32_t n_peers,
                            uint32_t my_rank, sptmm_seq **out);
/* One cooperative launch on `stream`; asynchronous.  Runs of one sequence must not overlap. */
int sptmm_seq_run(sptmm_seq *seq, void *stream);
/* status (if not NULL): waits for the device, then reads the error word a run raises when one of
 * its bounded waits ran out (0 = all good).  stream_bytes (if not NULL): encoded bytes per run. */
int sptmm_seq_status(sptmm_seq *seq, uint32_t *status, uint64_t *stream_bytes);
/* How often a waiting thread reloads a step counter (or a word of the settled exchange) before it
 * gives up, raises the status word and lets the run finish without further waiting.  0 restores
 * the default of 2^21 reloads (seconds).  A host that supervises several GPUs sets this to what
 * its own timeout allows; the status word tells it that a peer never delivered:
 * bit 0 a weight copy never arrived, bit 1 a producer's output never arrived, bit 2 a ring slot
 * was never freed, bit 3 row maxima never arrived, bit 4 a local arrival counter never filled. */
int sptmm_seq_set_wait_limit(sptmm_seq *seq, uint32_t polls);
/* No counterpart in the reference.  Runs a sequence of at most 16 steps WITHOUT allocating any
 * device memory: for callers that cannot call cudaMalloc when they need the result -- code inside
 * a closed, pre-sized memory pool, a real-time loop that may not block on the allocator, a host
 * framework that owns the whole device.  The sequence kernel's scratch (step descriptors, per-CTA
 * plan, step counters, status word; about 36 KB) lives in a fixed array inside the library image
 * instead, which every GPU that loads the library holds until the process exits.
 *  - steps / M / stream as for sptmm_seq_create + sptmm_seq_run; weights must already be uploaded
 *    (that upload allocates; this call does not).  More than 16 steps, or a device with more than
 *    256 SMs, is refused with SPTMM_ERR_INVALID / SPTMM_ERR_UNSUPPORTED.
 *  - The first call on a device looks the array's device address up and sets kernel attributes
 *    (host threads making first calls at the same time are serialised).  Every call copies its
 *    step tables from host memory that dies with the call, so a stream that is being captured
 *    into a graph is refused with SPTMM_ERR_STATE.
 *  - All calls share the one array and it keeps the previous call's contents (the counters and the
 *    status word are cleared at every call): two calls whose kernels overlap on the GPU race.
 *    Serialise them on one stream.
 *  - status_out == NULL: asynchronous.  Otherwise the call waits for the stream, stores the error
 *    word there (0 = all bounded waits were met) and returns SPTMM_ERR_STATE if it is not 0. */
int sptmm_seq_run_static(const sptmm_seq_step *steps, uint32_t n_steps, uint32_t M, void *stream,
                         uint32_t *status_out);

int sptmm_seq_free(sptmm_seq *seq);

/* ---- a stack of ternary layers over the GPUs of one node ----------------------------------------- */

/* No counterpart in the reference (one matmul per launch on one GPU, main.cu:994-1458, 1861); the
 * layer shapes are the ones its dispatch ladders hard-code (main.cu:1107-1190).  `layers` layers of
 * four dependent steps -- qkv (hidden -> hidden + 2 kv), o (hidden -> hidden, on the q part of
 * qkv), gate|up fused (hidden -> 2 ffn, stored as gate_j + up_j) and down (ffn -> hidden) -- on
 * int8 activations with int32 results and the per-row absmax quantiser between the steps.  Every
 * matrix is sharded by contiguous column ranges over `world` ranks (one process or host thread per
 * GPU); a forward pass is one persistent kernel per rank.  Weights are synthetic: i.i.d. ternary
 * with P(0) = p_zero, a seed per matrix derived from `seed`, identical on every rank. */
typedef struct sptmm_stack_config {
    uint32_t layers, hidden, ffn, kv;
    double p_zero;
    uint64_t seed;
    uint32_t rank, world;
} sptmm_stack_config;

/* how a step's int32 output becomes the next step's int8 input (sptmm_seq_step::x_kind) */
enum {
    SPTMM_STACK_AUTO = 0,            /* across GPUs: settled, as two half-batches from twelve (even) rows
                                        upward; one GPU: settled from eight rows upward, else counters */
    SPTMM_STACK_COUNTERS = 1,        /* x_kind 1: step counters, readers quantise                    */
    SPTMM_STACK_TAGGED = 2,          /* x_kind 2: tagged words polled by every reader                */
    SPTMM_STACK_ROW_MAXIMA = 3,      /* x_kind 3 for readers of whole rows (1 otherwise)             */
    SPTMM_STACK_PRODUCER_QUANT = 4,  /* x_kind 4: producers quantise, packed int8 travels            */
    SPTMM_STACK_SETTLED = 5,         /* x_kind 5: one watcher per word, local counters, int8 tile    */
    SPTMM_STACK_SETTLED_HALVES = 6   /* the same with the M rows (even) run as two half-batches whose
                                        steps alternate in the one kernel: while one half's outputs
                                        travel and settle -- in warps of their own, one step ahead -- the
                                        other half is gathered (each step's weights are streamed twice;
                                        pays at M=16 across GPUs, see csrc/stack.cpp)                  */
};

typedef struct sptmm_stack_weights sptmm_stack_weights;   /* this rank's shard of every matrix, uploaded */
typedef struct sptmm_stack sptmm_stack;

/* Generates, shards, encodes and uploads (to the current device) this rank's columns of every
 * matrix.  Independent of the batch size: stacks for several M may share one set. */
int sptmm_stack_weights_create(const sptmm_stack_config *cfg, sptmm_stack_weights **out);
int sptmm_stack_weights_info(const sptmm_stack_weights *w, uint64_t *stream_bytes, uint64_t *params);
/* matrix `index` (4 per layer: qkv, o, gate|up interleaved, down) as an encoded, uploaded handle */
int sptmm_stack_weights_matrix(const sptmm_stack_weights *w, uint32_t index, const sptmm_weights **out);
int sptmm_stack_weights_free(sptmm_stack_weights *w);

/* Bytes of one rank's arena (activation buffers, synchronisation area, input, scales) for M rows.
 * With several ranks the caller allocates one arena per rank, zeroes it, maps every rank's arena
 * into every rank's address space (CUDA IPC, the virtual memory API, a symmetric-memory
 * allocator) and passes the `world` base addresses, valid in THIS process, as arena_peers; only
 * the library's own kernels touch peer memory, with plain stores.  With one rank arena_peers may
 * be NULL and the library allocates. */
uint64_t sptmm_stack_arena_bytes(const sptmm_stack_weights *w, uint32_t M, uint32_t exchange);
int sptmm_stack_create(sptmm_stack_weights *w, uint32_t M, uint32_t exchange, void *const *arena_peers,
                       sptmm_stack **out);
int sptmm_stack_set_input(sptmm_stack *st, const int8_t *x_host);        /* M x hidden int8, host memory */
int sptmm_stack_forward(sptmm_stack *st, void *stream);                   /* asynchronous, one launch */
/* This rank's copy of "qkv", "o", "gu" (pair sums) or "down" (the final result) of the last layer,
 * int32 M x *width, after waiting for the device; host_out may be NULL to ask for the width. */
int sptmm_stack_buffer(sptmm_stack *st, const char *name, int32_t *host_out, uint32_t *width);
int sptmm_stack_status(sptmm_stack *st, uint32_t *status);                /* see sptmm_seq_status */
int sptmm_stack_exchange(const sptmm_stack *st, uint32_t *exchange);      /* the exchange in use */
int sptmm_stack_sequence(sptmm_stack *st, sptmm_seq **seq);               /* the stack's sequence (not to be freed) */
int sptmm_stack_wait_limit(sptmm_stack *st, uint32_t polls);              /* see sptmm_seq_set_wait_limit */
int sptmm_stack_free(sptmm_stack *st);

/* ---- split-K over the GPUs of one node as an object (csrc/splitk.cu) ------------------------ */
/* The host side around sptmm_gemv_reduce: shard arithmetic, the per-rank arena and the phases of
 * a pass.  No counterpart in the reference (one device, one stream, main.cu:1861; its only split
 * of K is the lane striding of main.cu:581-584).
 *  - sptmm_splitk_k_range: the rows of W (and elements of every row of X) rank r holds --
 *    contiguous, boundaries on multiples of 16.  sptmm_splitk_col_range: the result columns rank r
 *    owns after the reduce-scatter, N*r/world .. N*(r+1)/world.
 *  - The arena of a rank (sptmm_splitk_arena_bytes; 256-byte aligned, zeroed by the caller, every
 *    rank's mapped into every rank's address space like the stack's) holds the rank's result block
 *    and one flag word per rank.  With one rank arena_peers may be NULL and the library allocates.
 *  - `w`: this rank's K range encoded as a native u16 matrix and uploaded (or its tile of a K-tiled
 *    encoding, sptmm_weights_tile); stays the caller's.
 *  - sptmm_splitk_forward queues a whole pass on the stream: clear my block | barrier | add the
 *    partial sums to their owners (sptmm_gemv_reduce) | barrier.  Every rank calls it the same
 *    number of times.  The barrier is a one-warp kernel of this library -- each rank stores its pass
 *    counter into every rank's flag words and polls its own -- so a pass needs no collective of
 *    another library and no host round trip; its poll is bounded (sptmm_splitk_set_wait_limit,
 *    reloads; 0 = default) and a poll that runs out sets bit 0 of sptmm_splitk_status (bit 1: the
 *    matmul kernel's own status word, see sptmm_gemv_status).  Creation must have finished on every
 *    rank before the first pass starts on any (a host-side barrier of the caller's).
 *  - The phases are also callable one by one (clear, barrier, accumulate) for a caller that brings
 *    its own barrier, or that runs several ranks one after another on one device, where the
 *    library's barrier kernel must not be used: its ranks would wait for kernels queued behind them.
 *  - sptmm_splitk_output: this rank's block, M x width row-major int32 / float, valid once the
 *    stream has run the pass. */
typedef struct sptmm_splitk sptmm_splitk;
int sptmm_splitk_k_range(uint32_t K, uint32_t rank, uint32_t world, uint32_t *k0, uint32_t *k1);
int sptmm_splitk_col_range(uint32_t N, uint32_t rank, uint32_t world, uint32_t *c0, uint32_t *c1);
uint64_t sptmm_splitk_arena_bytes(uint32_t M, uint32_t N, uint32_t world);
int sptmm_splitk_create(const sptmm_weights *w, uint32_t dtype, uint32_t M, uint32_t rank, uint32_t world,
                        void *const *arena_peers, sptmm_splitk **out);
int sptmm_splitk_forward(sptmm_splitk *s, const void *X_slice, uint32_t flags, void *stream);
int sptmm_splitk_clear(sptmm_splitk *s, void *stream);
int sptmm_splitk_barrier(sptmm_splitk *s, void *stream);
int sptmm_splitk_accumulate(sptmm_splitk *s, const void *X_slice, uint32_t flags, void *stream);
int sptmm_splitk_output(const sptmm_splitk *s, void **C, uint32_t *width);
int sptmm_splitk_status(sptmm_splitk *s, uint32_t *status);
int sptmm_splitk_set_wait_limit(sptmm_splitk *s, uint64_t polls);
int sptmm_splitk_free(sptmm_splitk *s);

/* ---- small device helpers so a C caller needs no CUDA headers ------------------------------ */
int sptmm_device_count(int *count);
int sptmm_set_device(int device);
int sptmm_dev_alloc(void **ptr, uint64_t bytes);
int sptmm_dev_free(void *ptr);
int sptmm_memcpy_h2d(void *dst, const void *src, uint64_t bytes);
int sptmm_memcpy_d2h(void *dst, const void *src, uint64_t bytes);
int sptmm_device_sync(void);
/* Wait until `stream` (NULL = the default stream) has finished: polls first, which returns sooner
 * than the blocking wait for work of a few microseconds (the reference waits with
 * cudaDeviceSynchronize after every launch, main.cu:1456). */
int sptmm_stream_wait(void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SPTMM_H */
