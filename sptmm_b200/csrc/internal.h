// internal.h -- structures shared by the host encoder, the device API and the kernel launchers.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/sptmm.h"

namespace sptmm {

int fail(int code, const char *fmt, ...);        // records the message, returns `code`

struct HostArray {
    std::string name;
    std::vector<uint8_t> data;
    bool streamed;      // read once per matmul (counts toward stream_bytes)
};

// Most CTAs a launch plan may have.  The plan travels in the kernel parameters, and a launch
// copies all of them: 384 entries (two arrays, 3 KB) cover two CTAs per SM on 192 SMs.
constexpr uint32_t kMaxPlanCtas = 384;

// One CTA's share of a native-format matrix: columns [c0,c1) and their blocks [b0,b1).
struct CtaPlan { uint32_t c0, c1, b0, b1; };

struct LaunchPlan {                   // derived at upload time from the device's SM count
    uint32_t grid = 0;                // CTAs along x
    uint32_t threads = 0;             // threads per CTA
    uint32_t max_cols = 0;            // most columns any CTA owns
    std::vector<uint32_t> cta_blk;    // grid+1 block boundaries (passed in kernel parameters)
    std::vector<uint32_t> cta_col;    // grid+1 column boundaries (passed in kernel parameters)
    void *d_status = nullptr;         // device word set by a kernel whose bounded wait ran out
    uint32_t max_cta_blocks = 0;      // most blocks any CTA owns
};

}  // namespace sptmm

struct sptmm_weights {
    uint32_t K = 0, N = 0, format = 0, split = 0, S = 0, max_count = 0;
    uint64_t nnz = 0, stream_bytes = 0, lossy = 0;
    uint32_t total_blocks = 0;        // native formats
    uint32_t entries_per_block = 0;
    uint32_t uniform_nbl = 0;         // blocks per list if every list has the same count, else 0
    std::vector<sptmm::HostArray> arrays;
    // A K-tiled matrix (sptmm_encode_ktiled) carries no arrays itself: tile t is a native u16 matrix
    // of rows [t*k_tile, min(K, (t+1)*k_tile)), with its own lists, owned by this handle.
    uint32_t k_tile = 0;
    std::vector<sptmm_weights *> tiles;

    int device = -1;
    uint32_t sm_count = 0;
    std::vector<std::vector<void *>> dev;   // [replica][array]
    sptmm::LaunchPlan plan;           // small activation tiles: several CTAs per SM (see Tune)
    sptmm::LaunchPlan plan_wide;      // tiles of tens of KB: one 512-thread CTA per SM

    // Host-buffer calls (sptmm_gemv_host*): each slot has its own pinned input, mapped pinned
    // output, device copy of X and stream, so that independent calls overlap.
    struct HostSlot {
        void *pin_x = nullptr, *dev_x = nullptr;      // pinned host copy of X and its device copy
        void *pin_c = nullptr, *dev_c = nullptr;      // mapped pinned result and the device's address of it
        void *pin_status = nullptr, *dev_status = nullptr;   // mapped pinned word a kernel sets when a bounded wait runs out
        size_t x_bytes = 0, c_bytes = 0;              // capacities
        void *stream = nullptr;
        void *user_c = nullptr;                       // where the pending call's result goes
        size_t user_c_bytes = 0;
        bool busy = false;
    };
    static constexpr uint32_t kHostSlots = 16;
    HostSlot slots[kHostSlots];
};

namespace sptmm {

// Launch constants of the per-call kernel.  smem_kb = shared memory one CTA of the small-tile plan
// may use beside its activation tile.
struct Tune { int ctas_per_sm; int threads; int prefetch; int smem_kb; };
const Tune &tune();

// A build with -DSPTMM_TUNING (build.py --tuning, a separate library used for sweeps and kernel
// timelines) lets the environment override the constants below; the product library has them fixed.
#ifdef SPTMM_TUNING
long tuning_knob(const char *name, long dflt);
#else
constexpr long tuning_knob(const char *, long dflt) { return dflt; }
#endif

struct GemvArgs {
    const sptmm_weights *w;
    const void *const *arrays;        // device arrays of the chosen replica
    const void *X; void *C;
    uint32_t dtype, M, flags;
    void *stream;
    void *const *C_peers = nullptr;   // split-K: per-rank output buffers the partial sums are added to
    uint32_t n_peers = 0;
    uint32_t *status = nullptr;       // where a bounded wait that ran out is reported (null: the handle's device word)
    uint32_t ldx = 0;                 // elements between rows of a row-major X (0 = K)
    bool accumulate = false;          // add to C instead of storing
    bool scaled = false;              // int8 activations, float output: C = sum * row_scale[m] * out_scale
    const float *row_scale = nullptr; // device float[M], or null for 1
    float out_scale = 1.0f;
};

int launch_native_u16(const GemvArgs &a);
int launch_native_delta(const GemvArgs &a);
int launch_i2s(const GemvArgs &a);
int launch_div(const void *X, const uint16_t *wp, const uint16_t *wn, void *C, uint32_t dtype,
               uint32_t M, uint32_t K, uint32_t N, uint32_t S, uint32_t split, uint32_t flags,
               void *stream);
int launch_delta256(const void *X, const uint8_t *dp, const uint8_t *dn, void *C, uint32_t dtype,
                    uint32_t M, uint32_t K, uint32_t N, uint32_t S, uint32_t flags, void *stream);
#ifdef SPTMM_TUNING
void set_trace_buffer(unsigned long long *dev_ptr);
#endif
void plan_columns(const uint32_t *off, uint32_t N, uint32_t grid, std::vector<uint32_t> &cta_blk,
                  std::vector<uint32_t> &cta_col, uint32_t &max_cols, uint32_t &max_cta_blocks,
                  uint32_t col_align = 1);

inline size_t dtype_size(uint32_t d) { return d == SPTMM_I8 ? 1 : d == SPTMM_F16 ? 2 : 4; }

}  // namespace sptmm
