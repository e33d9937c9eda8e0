// C ABI of the B200 scan (see include/fm_scan_b200.h): argument checks, choice of the aligned
// or the masked instantiation, kernel launches.  No allocation, no synchronisation, no torch.
#include "fm_scan_b200.h"

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "btd_kernels.cuh"
#include "fm_kernels.cuh"
#include "scan_kernels.cuh"

#define FMS_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

thread_local int g_last_cuda_error = 0;

inline int record(cudaError_t e) {
    if (e == cudaSuccess) return FMS_OK;
    g_last_cuda_error = static_cast<int>(e);
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver ||
        e == cudaErrorNoKernelImageForDevice || e == cudaErrorInvalidDeviceFunction)
        return FMS_ERR_NO_DEVICE;
    return FMS_ERR_LAUNCH;
}

inline int check_launch() { return record(cudaGetLastError()); }

inline bool aligned_to(const void *p, size_t a) {
    return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

inline size_t elem_size(int dtype) { return dtype == FMS_F32 ? 4 : 2; }

// rows * T must be addressable with int64 byte offsets.
inline bool sizes_ok(int64_t rows, int64_t T) {
    if (rows < 0 || T < 0) return false;
    if (rows == 0 || T == 0) return true;
    return rows <= (INT64_MAX / 8) / T;
}

// Tuning knobs (FMS_TUNE_* environment variables): warps per row K, tiles per warp and step U,
// the persistent walk, a cap on the grid.  The environment is read ONCE, at the first launch of
// the process (getenv on every launch would sit on the host critical path of 30-60 us kernels and
// race with setenv); fms_tune_reload() reads it again.  Unset, the choices made below apply, which
// are the measured best on B200.
struct Tune {
    int fwd_k = 0, bwd_k = 0, fwd_u = 0, bwd_u = 0;  // 0 = choose from the shape
    int max_ctas = 0x7fffffff;                       // test knob: forces the multi-row walk
    int persist = -1;                                // -1 = choose from the shape, 0 = off, 1 = on
    int fm_blocked = 1, fm_ring = 3, fm_dc = 0, btd_warps_per_sm = 32;
    int bwd_descending = 1;  // backward visits rows last-to-first (re-reads the forward's latest rows from L2)
    int fwd_keep = 0;        // L2 policy of the forward's state stores: 0 evict-first, 1 normal, 2 evict-last
};

Tune g_tune;
std::once_flag g_tune_once;

void load_tune() {
    auto get = [](const char *name, int dflt) {
        const char *s = std::getenv(name);
        return s ? std::atoi(s) : dflt;
    };
    Tune t;
    t.fwd_k = get("FMS_TUNE_FWD_K", 0);
    t.bwd_k = get("FMS_TUNE_BWD_K", 0);
    t.fwd_u = get("FMS_TUNE_FWD_U", 0);
    t.bwd_u = get("FMS_TUNE_BWD_U", 0);
    t.max_ctas = std::max(1, get("FMS_TUNE_MAX_CTAS", 0x7fffffff));
    t.persist = get("FMS_TUNE_PERSIST", -1);
    t.fm_blocked = get("FMS_TUNE_FM_BLOCKED", 1);
    t.fm_ring = get("FMS_TUNE_FM_RING", 3);
    t.fm_dc = get("FMS_TUNE_FM_DC", 0);
    t.btd_warps_per_sm = std::max(1, get("FMS_TUNE_BTD_WARPS_PER_SM", 32));
    t.bwd_descending = get("FMS_TUNE_BWD_DESCENDING", 1);
    t.fwd_keep = get("FMS_TUNE_FWD_KEEP", 0);
    g_tune = t;
}

inline const Tune &tune() {
    std::call_once(g_tune_once, load_tune);
    return g_tune;
}

// The default build holds the launch shapes the choices below can reach; -DFMS_ALL_VARIANTS adds
// every (warps per row, tiles per step) combination the FMS_TUNE_* knobs can name (tuning builds).
#ifdef FMS_ALL_VARIANTS
constexpr bool kAllVariants = true;
#else
constexpr bool kAllVariants = false;
#endif

struct Problem {
    int64_t rows, T;
    bool aligned;  // every row of every tensor starts on a 16-byte boundary
};

template <typename... Ptrs>
int make_problem(Problem &pb, int64_t rows, int64_t T, int dtype, Ptrs... big) {
    if (dtype != FMS_F32 && dtype != FMS_F16 && dtype != FMS_BF16) return FMS_ERR_BAD_DTYPE;
    if (!sizes_ok(rows, T)) return FMS_ERR_BAD_SHAPE;
    pb.rows = rows;
    pb.T = T;
    if (rows == 0 || T == 0) {
        pb.aligned = true;
        return FMS_OK;
    }
    const size_t es = elem_size(dtype);
    const void *ptrs[] = {big...};
    bool all16 = (static_cast<uint64_t>(T) * es) % 16 == 0;
    for (const void *p : ptrs) {
        if (!p) return FMS_ERR_NULL_POINTER;
        if (!aligned_to(p, es)) return FMS_ERR_MISALIGNED;
        all16 = all16 && aligned_to(p, 16);
    }
    pb.aligned = all16;
    return FMS_OK;
}

__global__ void copy_or_zero_kernel(const float *__restrict__ src, float *__restrict__ dst, int64_t n,
                                    float fill) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src ? src[i] : fill;
}

int copy_or_zero(const float *src, float *dst, int64_t n, float fill, cudaStream_t st) {
    if (!dst || n == 0) return FMS_OK;
    const int64_t blocks = (n + 255) / 256;
    copy_or_zero_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(src, dst, n, fill);
    return check_launch();
}

// Number of SMs of the current device, asked once (every GPU of a box is alike); 148 on B200.
int sm_count() {
    static const int count = []() {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 148;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
        return n;
    }();
    return count;
}

template <typename Kernel>
int64_t resident_ctas(Kernel kernel, int threads) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess || per_sm <= 0)
        per_sm = 1;
    return static_cast<int64_t>(per_sm) * sm_count();
}

// Grid of a persistent launch.  Every CTA walks the same number q of units, q being the fewest
// whole passes over the work that the resident capacity allows: all CTAs are then resident from
// the first cycle, carry the load pipeline across their unit boundaries, and finish together.
// One unit per CTA under the hardware block scheduler instead leaves the last, partly filled
// wave (2.77 and 4.61 waves for 4096 rows of 16 KB forward and backward) running at a fraction
// of the bandwidth.
inline int64_t balanced_grid(int64_t ctas, int64_t resident) {
    const int64_t q = (ctas + resident - 1) / resident;
    return (ctas + q - 1) / q;
}

// Whether a launch of `ctas` one-unit CTAs walks persistently instead.  FMS_TUNE_PERSIST forces
// either answer.
inline bool use_persistent(int64_t ctas, int64_t resident) {
    const int forced = tune().persist;
    if (forced >= 0) return forced != 0;
    return ctas > resident;
}

// How a launch is cut into scan units and how many warps share a unit.
struct Split {
    int64_t nseg = 1;     // segments per row (1 = whole rows)
    int64_t seg_len = 0;  // positions per segment (T when nseg == 1)
};

// Warps per unit.  A CTA of K warps per row reads K*U*512 contiguous bytes per tensor per step
// and lets the block scheduler balance at a finer grain (all rows have the same length, so whole
// waves finish together); each row then takes fewer loop iterations to prefetch across.
int choose_coop(int64_t units, int64_t T, size_t es, int forced, bool finer_for_small_launches = true) {
    if (forced == 1 || forced == 2 || forced == 4 || forced == 8) return forced;
    // Measured on B200 (CUDA events, fwd+bwd GB/s): 16 KB rows x 32768 rows: K=2 6306, K=4 6182,
    // K=1 5797; 16 KB rows x 8192 rows: K=4 6026, K=2 5761; 128 KB rows x 4096 rows: K=8 6284,
    // K=4 6143; 8 KB rows x 65536 rows: K=2 6374, K=1 6196, K=4 5770; 12 KB rows: K=2 6474,
    // K=1 6217.  Rows shorter than 16 tiles keep one warp each.
    const int64_t tiles = (T * static_cast<int64_t>(es) + 511) / 512;
    int k = tiles >= 128 ? 8 : tiles >= 64 ? 4 : tiles >= 16 ? 2 : 1;
    // small launches: finer-grained CTAs shorten the tail.  With the balanced persistent grid this
    // still pays forward (4096 / 8192 rows of 16 KB: 33.0 / 63.4 us with K=4, 33.0 / 66.0 with K=2)
    // but not backward (59.5 / 111.1 us with K=4 against 57.0 / 108.1 with K=2)
    if (finer_for_small_launches && tiles >= 32 && k < 8 && units <= 8192) k *= 2;
    return k;
}

// Tiles per warp and step: 4 unless the row is too short to fill K*4 tiles.
int choose_unroll(int64_t T, size_t es, int K, int forced) {
    if (forced == 1 || forced == 2 || forced == 4) return forced;
    const int64_t tiles = (T * static_cast<int64_t>(es) + 511) / 512;
    if (tiles >= 4 * K) return 4;
    if (tiles >= 2 * K) return 2;
    return 1;
}

template <typename S, bool WRITE>
int launch_forward(const Problem &pb, const Split &sp, const void *gates, const void *tokens,
                   const float *h0, void *states, float *h_last, float *P, cudaStream_t st) {
    const int64_t units = pb.rows * sp.nseg;
    int K = sp.nseg > 1 ? 1 : choose_coop(units, pb.T, sizeof(S), tune().fwd_k);
    // masked path (measured on 2304 rows x 16385 fp16): one warp per row is fastest forward when
    // rows are plentiful; with few rows the warps-per-row choice above keeps the GPU filled
    if (!pb.aligned && tune().fwd_k == 0 && units >= 1024) K = 1;
    int unroll = choose_unroll(pb.T, sizeof(S), K, tune().fwd_u);
    if (!kAllVariants && K > 1) unroll = 4;
    const int64_t ctas = K == 1 ? (units + fms::kWarpsPerCta - 1) / fms::kWarpsPerCta : units;
    if (ctas > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
    const int64_t seg_len = sp.nseg == 1 ? pb.T : sp.seg_len;
    const int64_t max_ctas = tune().max_ctas;
#define FMS_LAUNCH_FWD_S(G, UU, KK, SS)                                                            \
    do {                                                                                           \
        auto kern = fms::plain_forward_kernel<S, G, UU, WRITE, KK, SS, false>;                            \
        int64_t nctas = ctas;                                                                      \
        if (!(G) && !(SS)) { /* instantiation that can walk several units */                       \
            static const int64_t resident = resident_ctas(kern, fms::Coop<KK>::kThreads);          \
            if (use_persistent(ctas, resident)) nctas = balanced_grid(ctas, resident);             \
            nctas = std::min(nctas, max_ctas);                                                     \
        }                                                                                          \
        kern<<<static_cast<unsigned>(nctas), fms::Coop<KK>::kThreads, 0, st>>>(                    \
            static_cast<const S *>(gates), static_cast<const S *>(tokens), h0,                     \
            static_cast<S *>(states), h_last, P, units, pb.T, sp.nseg, seg_len, 0, 0,              \
            tune().fwd_keep);                                                                      \
    } while (0)
#define FMS_LAUNCH_FWD(G, UU, KK) FMS_LAUNCH_FWD_S(G, UU, KK, false)
#define FMS_LAUNCH_FWD_K(G, UU)                                                                    \
    switch (K) {                                                                                   \
        case 1: FMS_LAUNCH_FWD(G, UU, 1); break;                                                   \
        case 2: FMS_LAUNCH_FWD(G, UU, 2); break;                                                   \
        case 4: FMS_LAUNCH_FWD(G, UU, 4); break;                                                   \
        default: FMS_LAUNCH_FWD(G, UU, 8); break;                                                  \
    }
#ifdef FMS_ALL_VARIANTS
#define FMS_LAUNCH_FWD_KLOW(G, UU) FMS_LAUNCH_FWD_K(G, UU)
#else  // fewer than 4 tiles per step is only ever chosen with one warp per row
#define FMS_LAUNCH_FWD_KLOW(G, UU) FMS_LAUNCH_FWD(G, UU, 1);
#endif
    if (sp.nseg > 1) {  // split path: units are plentiful by construction, one warp each
        if (pb.aligned) FMS_LAUNCH_FWD_S(false, 2, 1, true);
        else FMS_LAUNCH_FWD_S(true, 2, 1, true);
    } else if (pb.aligned) {
        if (unroll == 4) { FMS_LAUNCH_FWD_K(false, 4) }
        else if (unroll == 2) { FMS_LAUNCH_FWD_KLOW(false, 2) }
        else { FMS_LAUNCH_FWD_KLOW(false, 1) }
    } else {
        FMS_LAUNCH_FWD_K(true, 2)
    }
#undef FMS_LAUNCH_FWD_KLOW
#undef FMS_LAUNCH_FWD_K
#undef FMS_LAUNCH_FWD
#undef FMS_LAUNCH_FWD_S
    return check_launch();
}

template <typename S, bool WRITE>
int launch_backward(const Problem &pb, const Split &sp, const void *gates, const void *states,
                    const void *grad_states, const float *h0, const float *carry_in, void *grad_gates,
                    void *grad_tokens, float *grad_h0, float *P, cudaStream_t st) {
    const int64_t units = pb.rows * sp.nseg;
    int K = sp.nseg > 1 ? 1 : choose_coop(units, pb.T, sizeof(S), tune().bwd_k, false);
    // masked path (same measurement): two warps per row are fastest backward when rows are plentiful
    if (!pb.aligned && tune().bwd_k == 0 && units >= 1024) K = std::min(K, 2);
    // one warp per row: 2 tiles per step (4 costs occupancy: 141+ registers for three inputs)
    int unroll = K == 1 ? std::min(2, choose_unroll(pb.T, sizeof(S), K, tune().bwd_u))
                        : choose_unroll(pb.T, sizeof(S), K, tune().bwd_u);
    if (!kAllVariants && K > 1) unroll = 4;
    const int64_t ctas = K == 1 ? (units + fms::kWarpsPerCta - 1) / fms::kWarpsPerCta : units;
    if (ctas > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
    const int64_t seg_len = sp.nseg == 1 ? pb.T : sp.seg_len;
    const int64_t max_ctas = tune().max_ctas;
#define FMS_LAUNCH_BWD_S(G, UU, KK, SS)                                                            \
    do {                                                                                           \
        auto kern = fms::plain_backward_kernel<S, G, UU, WRITE, KK, SS, false>;                           \
        int64_t nctas = ctas;                                                                      \
        if (!(G) && !(SS)) {                                                                       \
            static const int64_t resident = resident_ctas(kern, fms::Coop<KK>::kThreads);          \
            if (use_persistent(ctas, resident)) nctas = balanced_grid(ctas, resident);             \
            nctas = std::min(nctas, max_ctas);                                                     \
        }                                                                                          \
        kern<<<static_cast<unsigned>(nctas), fms::Coop<KK>::kThreads, 0, st>>>(                    \
            static_cast<const S *>(gates), static_cast<const S *>(states),                         \
            static_cast<const S *>(grad_states), h0, carry_in, static_cast<S *>(grad_gates),       \
            static_cast<S *>(grad_tokens), grad_h0, P, units, pb.T, sp.nseg, seg_len, nullptr,     \
            nullptr, nullptr, 0, 0, tune().bwd_descending);                                        \
    } while (0)
#define FMS_LAUNCH_BWD(G, UU, KK) FMS_LAUNCH_BWD_S(G, UU, KK, false)
#define FMS_LAUNCH_BWD_K(G, UU)                                                                    \
    switch (K) {                                                                                   \
        case 1: FMS_LAUNCH_BWD(G, UU, 1); break;                                                   \
        case 2: FMS_LAUNCH_BWD(G, UU, 2); break;                                                   \
        case 4: FMS_LAUNCH_BWD(G, UU, 4); break;                                                   \
        default: FMS_LAUNCH_BWD(G, UU, 8); break;                                                  \
    }
#ifdef FMS_ALL_VARIANTS
#define FMS_LAUNCH_BWD_KLOW(G, UU) FMS_LAUNCH_BWD_K(G, UU)
#define FMS_LAUNCH_BWD_KHIGH(G, UU) FMS_LAUNCH_BWD_K(G, UU)
#else  // one warp per row walks at most 2 tiles per step, several warps per row always 4
#define FMS_LAUNCH_BWD_KLOW(G, UU) FMS_LAUNCH_BWD(G, UU, 1);
#define FMS_LAUNCH_BWD_KHIGH(G, UU)                                                                \
    switch (K) {                                                                                   \
        case 2: FMS_LAUNCH_BWD(G, UU, 2); break;                                                   \
        case 4: FMS_LAUNCH_BWD(G, UU, 4); break;                                                   \
        default: FMS_LAUNCH_BWD(G, UU, 8); break;                                                  \
    }
#endif
    if (sp.nseg > 1) {
        if (pb.aligned) FMS_LAUNCH_BWD_S(false, 2, 1, true);
        else FMS_LAUNCH_BWD_S(true, 1, 1, true);
    } else if (pb.aligned) {
        if (unroll == 4) { FMS_LAUNCH_BWD_KHIGH(false, 4) }
        else if (unroll == 2) { FMS_LAUNCH_BWD_KLOW(false, 2) }
        else { FMS_LAUNCH_BWD_KLOW(false, 1) }
    } else {
        FMS_LAUNCH_BWD_K(true, 1)
    }
#undef FMS_LAUNCH_BWD_KHIGH
#undef FMS_LAUNCH_BWD_KLOW
#undef FMS_LAUNCH_BWD_K
#undef FMS_LAUNCH_BWD
#undef FMS_LAUNCH_BWD_S
    return check_launch();
}

int launch_combine(const float *P, const float *S, const float *carry0, float *carry_out, float *total,
                   int64_t nchunks, int64_t rows, int reverse, int64_t chunk_stride, int64_t row_stride,
                   cudaStream_t st) {
    const int64_t blocks = (rows + 127) / 128;
    if (blocks > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
    fms::combine_carries_kernel<<<static_cast<unsigned>(blocks), 128, 0, st>>>(
        P, S, carry0, carry_out, total, nchunks, rows, reverse ? 1 : 0, chunk_stride, row_stride);
    return check_launch();
}

#define FMS_DISPATCH_DTYPE(dtype, CALL)                                  \
    switch (dtype) {                                                     \
        case FMS_F32: { using S = float; return CALL; }                  \
        case FMS_F16: { using S = __half; return CALL; }                 \
        case FMS_BF16: { using S = __nv_bfloat16; return CALL; }         \
        default: return FMS_ERR_BAD_DTYPE;                               \
    }

}  // namespace

FMS_EXPORT int fms_version(void) { return 200; }

FMS_EXPORT void fms_tune_reload(void) {
    tune();  // make sure the one-time load has happened, then read the environment again
    load_tune();
}

FMS_EXPORT const char *fms_status_string(int status) {
    switch (status) {
        case FMS_OK: return "ok";
        case FMS_ERR_BAD_SHAPE: return "bad shape: negative size or size overflow";
        case FMS_ERR_BAD_DTYPE: return "unsupported dtype: expecting float32, float16 or bfloat16";
        case FMS_ERR_NULL_POINTER: return "a required pointer is NULL";
        case FMS_ERR_MISALIGNED: return "a pointer is not aligned to its element size";
        case FMS_ERR_LAUNCH: return "CUDA launch or copy failed (see fms_last_cuda_error)";
        case FMS_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case FMS_ERR_TOO_LARGE: return "problem exceeds a fixed capacity of this entry point";
        case FMS_ERR_NO_DEVICE: return "no usable CUDA device (this library holds sm_100a code only)";
        default: return "unknown status";
    }
}

FMS_EXPORT int fms_last_cuda_error(void) { return g_last_cuda_error; }

FMS_EXPORT int fms_plain_forward(const void *gates, const void *tokens, const float *h0, void *states,
                                 float *h_last, int64_t rows, int64_t T, int dtype,
                                 fms_stream_t stream) {
    Problem pb;
    if (int rc = make_problem(pb, rows, T, dtype, gates, tokens, static_cast<const void *>(states)))
        return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) return FMS_OK;
    if (T == 0) return copy_or_zero(h0, h_last, rows, 0.f, st);
    FMS_DISPATCH_DTYPE(dtype, (launch_forward<S, true>(pb, Split{}, gates, tokens, h0, states, h_last, nullptr, st)));
}

FMS_EXPORT int fms_plain_reduce(const void *gates, const void *tokens, float *P, float *S_out,
                                int64_t rows, int64_t T, int dtype, fms_stream_t stream) {
    Problem pb;
    if (int rc = make_problem(pb, rows, T, dtype, gates, tokens)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) return FMS_OK;
    if (!P || !S_out) return FMS_ERR_NULL_POINTER;
    if (T == 0) {
        if (int rc = copy_or_zero(nullptr, P, rows, 1.f, st)) return rc;
        return copy_or_zero(nullptr, S_out, rows, 0.f, st);
    }
    FMS_DISPATCH_DTYPE(dtype, (launch_forward<S, false>(pb, Split{}, gates, tokens, nullptr, nullptr, S_out, P, st)));
}

FMS_EXPORT int fms_plain_backward(const void *gates, const void *states, const void *grad_states,
                                  const float *h0, const float *carry_in, void *grad_gates,
                                  void *grad_tokens, float *grad_h0, int64_t rows, int64_t T,
                                  int dtype, fms_stream_t stream) {
    Problem pb;
    if (int rc = make_problem(pb, rows, T, dtype, gates, states, grad_states,
                              static_cast<const void *>(grad_gates),
                              static_cast<const void *>(grad_tokens)))
        return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) return FMS_OK;
    if (T == 0) return copy_or_zero(carry_in, grad_h0, rows, 0.f, st);
    FMS_DISPATCH_DTYPE(dtype, (launch_backward<S, true>(pb, Split{}, gates, states, grad_states, h0, carry_in,
                                                        grad_gates, grad_tokens, grad_h0, nullptr, st)));
}

FMS_EXPORT int fms_plain_reduce_reverse(const void *gates, const void *grad_states, float *P,
                                        float *S_rev, int64_t rows, int64_t T, int dtype,
                                        fms_stream_t stream) {
    Problem pb;
    if (int rc = make_problem(pb, rows, T, dtype, gates, grad_states)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) return FMS_OK;
    if (!S_rev) return FMS_ERR_NULL_POINTER;
    if (T == 0) {
        if (int rc = copy_or_zero(nullptr, P, rows, 1.f, st)) return rc;
        return copy_or_zero(nullptr, S_rev, rows, 0.f, st);
    }
    FMS_DISPATCH_DTYPE(dtype, (launch_backward<S, false>(pb, Split{}, gates, nullptr, grad_states, nullptr, nullptr,
                                                         nullptr, nullptr, S_rev, P, st)));
}

FMS_EXPORT int fms_combine_carries(const float *P, const float *S, const float *carry0,
                                   float *carry_out, float *total, int64_t nchunks, int64_t rows,
                                   int reverse, fms_stream_t stream) {
    if (nchunks < 0 || rows < 0) return FMS_ERR_BAD_SHAPE;
    if (rows == 0) return FMS_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (nchunks == 0) return copy_or_zero(carry0, total, rows, 0.f, st);
    if (!P || !S || !carry_out) return FMS_ERR_NULL_POINTER;
    return launch_combine(P, S, carry0, carry_out, total, nchunks, rows, reverse, rows, 1, st);
}

// ------------------------------------------------------------------ FM mode -----------------
namespace {

struct FmShape {
    int64_t B, M, D, L, rows;  // rows = B*M*D output rows
};

int make_fm_shape(FmShape &sh, int64_t B, int64_t M, int64_t D, int64_t L, int dtype) {
    if (dtype != FMS_F32 && dtype != FMS_F16 && dtype != FMS_BF16) return FMS_ERR_BAD_DTYPE;
    if (B < 0 || M < 0 || D < 0 || L < 0) return FMS_ERR_BAD_SHAPE;
    sh = FmShape{B, M, D, L, 0};
    if (B == 0 || M == 0 || D == 0) return FMS_OK;
    if (B > INT64_MAX / M || B * M > INT64_MAX / D) return FMS_ERR_BAD_SHAPE;
    sh.rows = B * M * D;
    if (!sizes_ok(sh.rows, L)) return FMS_ERR_BAD_SHAPE;
    return FMS_OK;
}

template <typename S>
int launch_fm_forward(const FmShape &sh, bool aligned, const void *gates, const void *tokens, const float *h0,
                      void *states, cudaStream_t st) {
    const int K = choose_coop(sh.rows, sh.L, sizeof(S), tune().fwd_k);
    int unroll = std::min(2, choose_unroll(sh.L, sizeof(S), K, tune().fwd_u));
    if (!kAllVariants && K > 1) unroll = 2;
    const int64_t ctas = K == 1 ? (sh.rows + fms::kWarpsPerCta - 1) / fms::kWarpsPerCta : sh.rows;
    if (ctas > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
#define FMS_LAUNCH_FM_FWD(G, UU, KK)                                                               \
    fms::plain_forward_kernel<S, G, UU, true, KK, false, true>                                     \
        <<<static_cast<unsigned>(ctas), fms::Coop<KK>::kThreads, 0, st>>>(                         \
            static_cast<const S *>(gates), static_cast<const S *>(tokens), h0,                     \
            static_cast<S *>(states), nullptr, nullptr, sh.rows, sh.L, 1, sh.L, sh.M, sh.D, 0)
#define FMS_LAUNCH_FM_FWD_K(G, UU)                                                                 \
    switch (K) {                                                                                   \
        case 1: FMS_LAUNCH_FM_FWD(G, UU, 1); break;                                                \
        case 2: FMS_LAUNCH_FM_FWD(G, UU, 2); break;                                                \
        case 4: FMS_LAUNCH_FM_FWD(G, UU, 4); break;                                                \
        default: FMS_LAUNCH_FM_FWD(G, UU, 8); break;                                               \
    }
    if (!aligned) { FMS_LAUNCH_FM_FWD_K(true, 1) }
    else if (unroll == 2) { FMS_LAUNCH_FM_FWD_K(false, 2) }
#ifdef FMS_ALL_VARIANTS
    else { FMS_LAUNCH_FM_FWD_K(false, 1) }
#else
    else { FMS_LAUNCH_FM_FWD(false, 1, 1); }
#endif
#undef FMS_LAUNCH_FM_FWD_K
#undef FMS_LAUNCH_FM_FWD
    return check_launch();
}

// full_gates / full_tokens non-null: store the per-row terms into (B,M,D,L) tensors instead of
// accumulating the sums (acc_* are then unused).
template <typename S>
int launch_fm_backward(const FmShape &sh, bool aligned, const void *gates, const void *tokens,
                       const void *states, const void *grad_states, const float *h0, float *acc_gates,
                       float *acc_tokens, float *grad_h0, cudaStream_t st, void *full_gates = nullptr,
                       void *full_tokens = nullptr) {
    const int K = choose_coop(sh.rows, sh.L, sizeof(S), tune().bwd_k);
    int unroll = std::min(2, choose_unroll(sh.L, sizeof(S), K, tune().bwd_u));
    if (!kAllVariants && K > 1) unroll = 2;
    const int64_t ctas = K == 1 ? (sh.rows + fms::kWarpsPerCta - 1) / fms::kWarpsPerCta : sh.rows;
    if (ctas > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
#define FMS_LAUNCH_FM_BWD(G, UU, KK)                                                               \
    fms::plain_backward_kernel<S, G, UU, true, KK, false, true>                                    \
        <<<static_cast<unsigned>(ctas), fms::Coop<KK>::kThreads, 0, st>>>(                         \
            static_cast<const S *>(gates), static_cast<const S *>(states),                         \
            static_cast<const S *>(grad_states), h0, nullptr, static_cast<S *>(full_gates),        \
            static_cast<S *>(full_tokens), grad_h0, nullptr, sh.rows, sh.L, 1, sh.L,               \
            static_cast<const S *>(tokens), acc_gates, acc_tokens, sh.M, sh.D, 0)
#define FMS_LAUNCH_FM_BWD_K(G, UU)                                                                 \
    switch (K) {                                                                                   \
        case 1: FMS_LAUNCH_FM_BWD(G, UU, 1); break;                                                \
        case 2: FMS_LAUNCH_FM_BWD(G, UU, 2); break;                                                \
        case 4: FMS_LAUNCH_FM_BWD(G, UU, 4); break;                                                \
        default: FMS_LAUNCH_FM_BWD(G, UU, 8); break;                                               \
    }
    if (!aligned) { FMS_LAUNCH_FM_BWD_K(true, 1) }
    else if (unroll == 2) { FMS_LAUNCH_FM_BWD_K(false, 2) }
#ifdef FMS_ALL_VARIANTS
    else { FMS_LAUNCH_FM_BWD_K(false, 1) }
#else
    else { FMS_LAUNCH_FM_BWD(false, 1, 1); }
#endif
#undef FMS_LAUNCH_FM_BWD_K
#undef FMS_LAUNCH_FM_BWD
    return check_launch();
}

// Blocked forward (fm_kernels.cuh): 8 gate rows x 8 token rows per CTA, aligned tensors only.
template <typename S>
int launch_fm_forward_blocked(const FmShape &sh, const void *gates, const void *tokens, const float *h0,
                              void *states, cudaStream_t st) {
    constexpr int MC = 8, DC = 8;
    const int64_t m_blocks = (sh.M + MC - 1) / MC, d_blocks = (sh.D + DC - 1) / DC;
    if (sh.B > 0x7fffffffLL / m_blocks || sh.B * m_blocks > 0x7fffffffLL / d_blocks) return FMS_ERR_BAD_SHAPE;
    const unsigned grid = static_cast<unsigned>(sh.B * m_blocks * d_blocks);
    fms::fm_forward_blocked_kernel<S, MC, DC><<<grid, MC * 32, 0, st>>>(
        static_cast<const S *>(gates), static_cast<const S *>(tokens), h0, static_cast<S *>(states), sh.M, sh.D,
        sh.L, m_blocks, d_blocks);
    return check_launch();
}

// Blocked backward (fm_kernels.cuh): 8 gate rows (one warp each) x DC token rows per CTA, aligned
// tensors only.  Every CTA walks the whole sequence, so the launch is a few waves of equal CTAs
// whose last one may be nearly empty: DC is 8, or 7 when that makes (waves, rounded up) x DC
// smaller (measured: 3-4 % at (1,32,1024,8192) and (2,16,1000,4096), nothing at (1,32,2048,8192),
// where the kernel is bound by the memory system and a thin last wave simply runs faster).
template <typename S>
int launch_fm_backward_blocked(const FmShape &sh, const void *gates, const void *tokens, const void *states,
                               const void *grad_states, const float *h0, float *acc_gates, float *acc_tokens,
                               float *grad_h0, cudaStream_t st) {
    constexpr int MC = 8;
    const int64_t m_blocks = (sh.M + MC - 1) / MC;
    const int64_t slots = 2LL * sm_count();  // two CTAs per SM (registers and shared memory)
    int dc = 8;
    int64_t best = -1;
    for (int cand = 8; cand >= 7; --cand) {
        const int64_t d_blocks = (sh.D + cand - 1) / cand;
        if (sh.B > 0x7fffffffLL / m_blocks || sh.B * m_blocks > 0x7fffffffLL / d_blocks) return FMS_ERR_BAD_SHAPE;
        const int64_t ctas = sh.B * m_blocks * d_blocks;
        const int64_t cost = ((ctas + slots - 1) / slots) * cand;
        if (best < 0 || cost < best) {
            best = cost;
            dc = cand;
        }
    }
    if (tune().fm_dc >= 7 && tune().fm_dc <= 8) dc = tune().fm_dc;
    const int64_t d_blocks = (sh.D + dc - 1) / dc;
    const unsigned grid = static_cast<unsigned>(sh.B * m_blocks * d_blocks);
    // the shared-memory opt-in is per device, so it is (cheaply) repeated on every launch
#define FMS_LAUNCH_FM_RING(DCV, PDV)                                                                \
    do {                                                                                            \
        auto kern = fms::fm_backward_ring_kernel<S, MC, DCV, PDV>;                                  \
        constexpr size_t smem = fms::fm_backward_ring_smem<S, MC, DCV, PDV>();                      \
        const cudaError_t attr = cudaFuncSetAttribute(                                              \
            kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));             \
        if (int rc = record(attr)) return rc;                                                       \
        kern<<<grid, MC * 32, smem, st>>>(                                                          \
            static_cast<const S *>(gates), static_cast<const S *>(tokens),                          \
            static_cast<const S *>(states), static_cast<const S *>(grad_states), h0, acc_gates,     \
            acc_tokens, grad_h0, sh.M, sh.D, sh.L, m_blocks, d_blocks);                             \
    } while (0)
#ifdef FMS_ALL_VARIANTS
    if (dc == 8 && tune().fm_ring == 2) FMS_LAUNCH_FM_RING(8, 2);
    else if (dc == 8 && tune().fm_ring == 4) FMS_LAUNCH_FM_RING(8, 4);
    else if (dc == 8 && tune().fm_ring == 5) FMS_LAUNCH_FM_RING(8, 5);
    else
#endif
    if (dc == 8) FMS_LAUNCH_FM_RING(8, 3);
    else FMS_LAUNCH_FM_RING(7, 3);
#undef FMS_LAUNCH_FM_RING
    return check_launch();
}

template <typename S>
int launch_cast(const float *src, void *dst, int64_t n, cudaStream_t st) {
    if (n == 0) return FMS_OK;
    const int64_t blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
    fms::cast_from_f32_kernel<S><<<static_cast<unsigned>(blocks), 256, 0, st>>>(src, static_cast<S *>(dst), n);
    return check_launch();
}

// 16-byte alignment of every row of every tensor involved (rows are L elements long).
template <typename... Ptrs>
int fm_alignment(bool &aligned, int64_t L, int dtype, Ptrs... big) {
    const size_t es = elem_size(dtype);
    const void *ptrs[] = {big...};
    aligned = (static_cast<uint64_t>(L) * es) % 16 == 0;
    for (const void *p : ptrs) {
        if (!p) return FMS_ERR_NULL_POINTER;
        if (!aligned_to(p, es)) return FMS_ERR_MISALIGNED;
        aligned = aligned && aligned_to(p, 16);
    }
    return FMS_OK;
}

inline size_t fm_acc_elems(const FmShape &sh) {
    return static_cast<size_t>(sh.B) * static_cast<size_t>(sh.M + sh.D) * static_cast<size_t>(sh.L);
}

}  // namespace

FMS_EXPORT int fms_fm_forward(const void *gates, const void *tokens, const float *h0, void *states,
                              int64_t B, int64_t M, int64_t D, int64_t L, int dtype, fms_stream_t stream) {
    FmShape sh;
    if (int rc = make_fm_shape(sh, B, M, D, L, dtype)) return rc;
    if (sh.rows == 0 || L == 0) return FMS_OK;
    bool aligned = false;
    if (int rc = fm_alignment(aligned, L, dtype, gates, tokens, static_cast<const void *>(states))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (aligned && tune().fm_blocked != 0) {
        FMS_DISPATCH_DTYPE(dtype, (launch_fm_forward_blocked<S>(sh, gates, tokens, h0, states, st)));
    }
    FMS_DISPATCH_DTYPE(dtype, (launch_fm_forward<S>(sh, aligned, gates, tokens, h0, states, st)));
}

FMS_EXPORT size_t fms_fm_backward_workspace_bytes(int64_t B, int64_t M, int64_t D, int64_t L, int dtype) {
    FmShape sh;
    if (make_fm_shape(sh, B, M, D, L, dtype) != FMS_OK || sh.rows == 0 || L == 0) return 0;
    if (dtype == FMS_F32) return 0;  // fp32 outputs are accumulated in place
    return (fm_acc_elems(sh) * sizeof(float) + 255) / 256 * 256;
}

FMS_EXPORT int fms_fm_backward(const void *gates, const void *tokens, const void *states,
                               const void *grad_states, const float *h0, void *grad_gates, void *grad_tokens,
                               float *grad_h0, int64_t B, int64_t M, int64_t D, int64_t L, int dtype,
                               void *workspace, size_t workspace_bytes, fms_stream_t stream) {
    FmShape sh;
    if (int rc = make_fm_shape(sh, B, M, D, L, dtype)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t es = elem_size(dtype);
    const size_t n_g = static_cast<size_t>(B) * M * L, n_x = static_cast<size_t>(B) * D * L;
    if (sh.rows == 0 || L == 0) {
        // a sum over an empty axis is zero; with no positions nothing depends on h0 either
        if (grad_gates && n_g) if (int rc = record(cudaMemsetAsync(grad_gates, 0, n_g * es, st))) return rc;
        if (grad_tokens && n_x) if (int rc = record(cudaMemsetAsync(grad_tokens, 0, n_x * es, st))) return rc;
        if (grad_h0 && sh.rows) return copy_or_zero(nullptr, grad_h0, sh.rows, 0.f, st);
        return FMS_OK;
    }
    bool aligned = false;
    if (int rc = fm_alignment(aligned, L, dtype, gates, tokens, states, grad_states,
                              static_cast<const void *>(grad_gates), static_cast<const void *>(grad_tokens)))
        return rc;
    float *acc_g, *acc_x;
    if (dtype == FMS_F32) {
        acc_g = static_cast<float *>(grad_gates);
        acc_x = static_cast<float *>(grad_tokens);
        if (int rc = record(cudaMemsetAsync(acc_g, 0, n_g * sizeof(float), st))) return rc;
        if (int rc = record(cudaMemsetAsync(acc_x, 0, n_x * sizeof(float), st))) return rc;
    } else {
        const size_t need = fms_fm_backward_workspace_bytes(B, M, D, L, dtype);
        if (!workspace || !aligned_to(workspace, 16) || workspace_bytes < need) return FMS_ERR_WORKSPACE;
        acc_g = static_cast<float *>(workspace);
        acc_x = acc_g + n_g;
        if (int rc = record(cudaMemsetAsync(acc_g, 0, (n_g + n_x) * sizeof(float), st))) return rc;
    }
    // vector reductions need 16-byte aligned fp32 rows as well
    aligned = aligned && (static_cast<uint64_t>(L) * sizeof(float)) % 16 == 0 && aligned_to(acc_g, 16) &&
              aligned_to(acc_x, 16);
    {
        // rows that share a gate or a token row are reduced inside a CTA before any global
        // atomic when everything is 16-byte aligned; the row-per-CTA kernel covers the rest
        const bool blocked = aligned && tune().fm_blocked != 0;
        auto pass = [&]() -> int {
            if (blocked) {
                FMS_DISPATCH_DTYPE(dtype, (launch_fm_backward_blocked<S>(sh, gates, tokens, states, grad_states,
                                                                         h0, acc_g, acc_x, grad_h0, st)));
            }
            FMS_DISPATCH_DTYPE(dtype, (launch_fm_backward<S>(sh, aligned, gates, tokens, states, grad_states, h0,
                                                             acc_g, acc_x, grad_h0, st)));
        };
        if (int rc = pass()) return rc;
    }
    if (dtype == FMS_F32) return FMS_OK;
    {
        auto cast_g = [&]() -> int { FMS_DISPATCH_DTYPE(dtype, (launch_cast<S>(acc_g, grad_gates, n_g, st))); };
        if (int rc = cast_g()) return rc;
    }
    FMS_DISPATCH_DTYPE(dtype, (launch_cast<S>(acc_x, grad_tokens, n_x, st)));
}

FMS_EXPORT int fms_fm_backward_unreduced(const void *gates, const void *tokens, const void *states,
                                         const void *grad_states, const float *h0, void *grad_gates_full,
                                         void *grad_tokens_full, float *grad_h0, int64_t B, int64_t M, int64_t D,
                                         int64_t L, int dtype, fms_stream_t stream) {
    FmShape sh;
    if (int rc = make_fm_shape(sh, B, M, D, L, dtype)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (sh.rows == 0) return FMS_OK;
    if (L == 0) return copy_or_zero(nullptr, grad_h0, sh.rows, 0.f, st);
    bool aligned = false;
    if (int rc = fm_alignment(aligned, L, dtype, gates, tokens, states, grad_states,
                              static_cast<const void *>(grad_gates_full), static_cast<const void *>(grad_tokens_full)))
        return rc;
    FMS_DISPATCH_DTYPE(dtype, (launch_fm_backward<S>(sh, aligned, gates, tokens, states, grad_states, h0, nullptr,
                                                     nullptr, grad_h0, st, grad_gates_full, grad_tokens_full)));
}

// ------------------------------------------------------------------ FM layer read-out -------
namespace {

// states_out / rnorm_out non-null: the training forward (normalised states and the norm factor are
// kept for the backward); null: inference read-out, nothing of size (B,M,D,L) is written.
template <typename S>
int launch_fm_readout(const FmShape &sh, const void *gates, const void *tokens, const void *weight,
                      const float *h0, float *scale, float *out32, void *out, int mem_norm, float eps,
                      void *states_out, float *rnorm_out, cudaStream_t st) {
    constexpr int MC = 8, DC = 8;
    const int64_t m_blocks = (sh.M + MC - 1) / MC, d_blocks = (sh.D + DC - 1) / DC;
    if (sh.B > 0x7fffffffLL / m_blocks || sh.B * m_blocks > 0x7fffffffLL / d_blocks) return FMS_ERR_BAD_SHAPE;
    const unsigned grid = static_cast<unsigned>(sh.B * m_blocks * d_blocks);
    constexpr size_t smem = fms::fm_readout_smem<S, MC, DC>();
    const int64_t n_g = sh.B * sh.M * sh.L, n_x = sh.B * sh.D * sh.L;
    auto k0 = fms::fm_readout_blocked_kernel<S, MC, DC, 0>;
    auto k1 = fms::fm_readout_blocked_kernel<S, MC, DC, 1>;
    auto k2 = fms::fm_readout_blocked_kernel<S, MC, DC, 2>;
    const cudaError_t a2 =
        cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (int rc = record(a2)) return rc;
    const cudaError_t a0 =
        cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    const cudaError_t a1 =
        cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (int rc = record(a0)) return rc;
    if (int rc = record(a1)) return rc;
    if (int rc = record(cudaMemsetAsync(scale, 0, static_cast<size_t>(n_g + n_x) * sizeof(float), st))) return rc;
    if (mem_norm) {
        k0<<<grid, MC * 32, smem, st>>>(static_cast<const S *>(gates), static_cast<const S *>(tokens), h0, nullptr,
                                        scale, nullptr, nullptr, nullptr, sh.M, sh.D, sh.L, m_blocks, d_blocks);
        if (int rc = check_launch()) return rc;
    }
    const int64_t blocks = (n_g + 255) / 256;
    if (blocks > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
    fms::fm_readout_scale_kernel<S><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        scale, static_cast<const S *>(weight), mem_norm ? rnorm_out : nullptr, n_g,
        1.f / static_cast<float>(sh.D), eps, mem_norm ? 1 : 0);
    if (int rc = check_launch()) return rc;
    if (states_out)
        k2<<<grid, MC * 32, smem, st>>>(static_cast<const S *>(gates), static_cast<const S *>(tokens), h0, scale,
                                        nullptr, out32, mem_norm ? rnorm_out : nullptr,
                                        static_cast<S *>(states_out), sh.M, sh.D, sh.L, m_blocks, d_blocks);
    else
        k1<<<grid, MC * 32, smem, st>>>(static_cast<const S *>(gates), static_cast<const S *>(tokens), h0, scale,
                                        nullptr, out32, nullptr, nullptr, sh.M, sh.D, sh.L, m_blocks, d_blocks);
    if (int rc = check_launch()) return rc;
    return launch_cast<S>(out32, out, n_x, st);
}

}  // namespace

FMS_EXPORT size_t fms_fm_readout_workspace_bytes(int64_t B, int64_t M, int64_t D, int64_t L, int dtype) {
    FmShape sh;
    if (make_fm_shape(sh, B, M, D, L, dtype) != FMS_OK || sh.rows == 0 || L == 0) return 0;
    return (fm_acc_elems(sh) * sizeof(float) + 255) / 256 * 256;
}

FMS_EXPORT int fms_fm_readout(const void *gates, const void *tokens, const void *out_weight, const float *h0,
                              void *out, int64_t B, int64_t M, int64_t D, int64_t L, int dtype, int mem_norm,
                              float eps, void *workspace, size_t workspace_bytes, fms_stream_t stream) {
    FmShape sh;
    if (int rc = make_fm_shape(sh, B, M, D, L, dtype)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (B == 0 || D == 0 || L == 0) return FMS_OK;
    if (M == 0) {
        if (!out) return FMS_ERR_NULL_POINTER;
        return record(cudaMemsetAsync(out, 0, static_cast<size_t>(B) * D * L * elem_size(dtype), st));
    }
    bool aligned = false;
    if (int rc = fm_alignment(aligned, L, dtype, gates, tokens, out_weight, static_cast<const void *>(out)))
        return rc;
    if (!aligned || (static_cast<uint64_t>(L) * sizeof(float)) % 16 != 0) return FMS_ERR_MISALIGNED;
    const size_t need = fms_fm_readout_workspace_bytes(B, M, D, L, dtype);
    if (!workspace || !aligned_to(workspace, 16) || workspace_bytes < need) return FMS_ERR_WORKSPACE;
    float *scale = static_cast<float *>(workspace);
    float *out32 = scale + static_cast<size_t>(B) * M * L;
    if (!aligned_to(out32, 16)) return FMS_ERR_WORKSPACE;
    FMS_DISPATCH_DTYPE(dtype, (launch_fm_readout<S>(sh, gates, tokens, out_weight, h0, scale, out32, out, mem_norm,
                                                    eps, nullptr, nullptr, st)));
}

// ------------------------------------------------------------------ FM layer, training -----
namespace {

template <typename S>
int launch_fm_layer_backward(const FmShape &sh, const void *gates, const void *tokens, const void *weight,
                             const void *hn, const void *dout, const void *ext, const float *rnorm,
                             const float *h0, float *ws, void *grad_gates, void *grad_tokens, void *grad_weight,
                             float *grad_h0, cudaStream_t st) {
    constexpr int MC = 8, DC = 8;
    const int64_t m_blocks = (sh.M + MC - 1) / MC, d_blocks = (sh.D + DC - 1) / DC;
    if (sh.B > 0x7fffffffLL / m_blocks || sh.B * m_blocks > 0x7fffffffLL / d_blocks) return FMS_ERR_BAD_SHAPE;
    const unsigned grid = static_cast<unsigned>(sh.B * m_blocks * d_blocks);
    const int64_t n_g = sh.B * sh.M * sh.L, n_x = sh.B * sh.D * sh.L;
    float *dotc = ws, *dw = dotc + n_g, *p1 = dw + n_g, *rinv = p1 + n_g, *acc_g = rinv + n_g, *acc_x = acc_g + n_g;
    if (int rc = record(cudaMemsetAsync(ws, 0, static_cast<size_t>(5 * n_g + n_x) * sizeof(float), st))) return rc;
    const S *hn_ = static_cast<const S *>(hn), *dout_ = static_cast<const S *>(dout), *ext_ = static_cast<const S *>(ext);
    const S *w_ = static_cast<const S *>(weight);
#define FMS_LAUNCH_LAYER_DOTS(EXTV)                                                                     \
    do {                                                                                                \
        constexpr int PDD = 6;                                                                          \
        auto kern = fms::fm_layer_dots_kernel<S, MC, DC, PDD, EXTV>;                                    \
        constexpr size_t smem = fms::fm_layer_dots_smem<S, MC, DC, PDD, EXTV>();                        \
        const cudaError_t attr = cudaFuncSetAttribute(                                                  \
            kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));                 \
        if (int rc = record(attr)) return rc;                                                           \
        kern<<<grid, MC * 32, smem, st>>>(hn_, dout_, ext_, w_, dotc, dw, sh.M, sh.D, sh.L, m_blocks, d_blocks); \
    } while (0)
    if (ext) FMS_LAUNCH_LAYER_DOTS(true);
    else FMS_LAUNCH_LAYER_DOTS(false);
#undef FMS_LAUNCH_LAYER_DOTS
    if (int rc = check_launch()) return rc;
    const int64_t blocks = (n_g + 255) / 256;
    if (blocks > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
    fms::fm_layer_factors_kernel<S><<<static_cast<unsigned>(blocks), 256, 0, st>>>(rnorm, w_, dotc, p1, rinv, n_g,
                                                                                   1.f / static_cast<float>(sh.D));
    if (int rc = check_launch()) return rc;
#define FMS_LAUNCH_LAYER_BWD(EXTV, PDV)                                                                 \
    do {                                                                                                \
        auto kern = fms::fm_layer_backward_ring_kernel<S, MC, DC, PDV, EXTV>;                           \
        constexpr size_t smem = fms::fm_layer_backward_smem<S, MC, DC, PDV, EXTV>();                    \
        const cudaError_t attr = cudaFuncSetAttribute(                                                  \
            kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));                 \
        if (int rc = record(attr)) return rc;                                                           \
        kern<<<grid, MC * 32, smem, st>>>(static_cast<const S *>(gates), static_cast<const S *>(tokens), hn_, dout_, \
                                          ext_, p1, dotc, rinv, rnorm, h0, acc_g, acc_x, grad_h0, sh.M, sh.D,    \
                                          sh.L, m_blocks, d_blocks);                                    \
    } while (0)
    const int ring = tune().fm_ring;
    (void)ring;
    if (ext) {
#ifdef FMS_ALL_VARIANTS
        if (ring == 2) FMS_LAUNCH_LAYER_BWD(true, 2);
        else if (ring == 4) FMS_LAUNCH_LAYER_BWD(true, 4);
        else
#endif
            FMS_LAUNCH_LAYER_BWD(true, 3);
    } else {
#ifdef FMS_ALL_VARIANTS
        if (ring == 2) FMS_LAUNCH_LAYER_BWD(false, 2);
        else if (ring == 4) FMS_LAUNCH_LAYER_BWD(false, 4);
        else if (ring == 5) FMS_LAUNCH_LAYER_BWD(false, 5);
        else
#endif
            FMS_LAUNCH_LAYER_BWD(false, 3);
    }
#undef FMS_LAUNCH_LAYER_BWD
    if (int rc = check_launch()) return rc;
    if (int rc = launch_cast<S>(acc_g, grad_gates, n_g, st)) return rc;
    if (int rc = launch_cast<S>(dw, grad_weight, n_g, st)) return rc;
    return launch_cast<S>(acc_x, grad_tokens, n_x, st);
}

}  // namespace

FMS_EXPORT int fms_fm_layer_forward(const void *gates, const void *tokens, const void *out_weight, const float *h0,
                                    void *out, void *states_norm, float *rnorm, int64_t B, int64_t M, int64_t D,
                                    int64_t L, int dtype, int mem_norm, float eps, void *workspace,
                                    size_t workspace_bytes, fms_stream_t stream) {
    FmShape sh;
    if (int rc = make_fm_shape(sh, B, M, D, L, dtype)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (sh.rows == 0 || L == 0) return FMS_OK;
    bool aligned = false;
    if (int rc = fm_alignment(aligned, L, dtype, gates, tokens, out_weight, static_cast<const void *>(out),
                              static_cast<const void *>(states_norm)))
        return rc;
    if (mem_norm && !rnorm) return FMS_ERR_NULL_POINTER;
    if (!aligned || (static_cast<uint64_t>(L) * sizeof(float)) % 16 != 0 || (rnorm && !aligned_to(rnorm, 16)))
        return FMS_ERR_MISALIGNED;
    const size_t need = fms_fm_readout_workspace_bytes(B, M, D, L, dtype);
    if (!workspace || !aligned_to(workspace, 16) || workspace_bytes < need) return FMS_ERR_WORKSPACE;
    float *scale = static_cast<float *>(workspace);
    float *out32 = scale + static_cast<size_t>(B) * M * L;
    FMS_DISPATCH_DTYPE(dtype, (launch_fm_readout<S>(sh, gates, tokens, out_weight, h0, scale, out32, out, mem_norm,
                                                    eps, states_norm, rnorm, st)));
}

FMS_EXPORT size_t fms_fm_layer_backward_workspace_bytes(int64_t B, int64_t M, int64_t D, int64_t L, int dtype) {
    FmShape sh;
    if (make_fm_shape(sh, B, M, D, L, dtype) != FMS_OK || sh.rows == 0 || L == 0) return 0;
    const size_t elems = static_cast<size_t>(B) * static_cast<size_t>(5 * M + D) * static_cast<size_t>(L);
    return (elems * sizeof(float) + 255) / 256 * 256;
}

FMS_EXPORT int fms_fm_layer_backward(const void *gates, const void *tokens, const void *out_weight,
                                     const void *states_norm, const float *rnorm, const void *grad_out,
                                     const void *grad_states_norm, const float *h0, void *grad_gates,
                                     void *grad_tokens, void *grad_out_weight, float *grad_h0, int64_t B, int64_t M,
                                     int64_t D, int64_t L, int dtype, void *workspace, size_t workspace_bytes,
                                     fms_stream_t stream) {
    FmShape sh;
    if (int rc = make_fm_shape(sh, B, M, D, L, dtype)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (sh.rows == 0 || L == 0) return FMS_OK;
    bool aligned = false;
    if (int rc = fm_alignment(aligned, L, dtype, gates, tokens, out_weight, states_norm, grad_out,
                              static_cast<const void *>(grad_gates), static_cast<const void *>(grad_tokens),
                              static_cast<const void *>(grad_out_weight)))
        return rc;
    if (grad_states_norm && !aligned_to(grad_states_norm, 16)) aligned = false;
    if (!aligned || (static_cast<uint64_t>(L) * sizeof(float)) % 16 != 0 || (rnorm && !aligned_to(rnorm, 16)))
        return FMS_ERR_MISALIGNED;
    const size_t need = fms_fm_layer_backward_workspace_bytes(B, M, D, L, dtype);
    if (!workspace || !aligned_to(workspace, 16) || workspace_bytes < need) return FMS_ERR_WORKSPACE;
    FMS_DISPATCH_DTYPE(dtype, (launch_fm_layer_backward<S>(sh, gates, tokens, out_weight, states_norm, grad_out,
                                                           grad_states_norm, rnorm, h0,
                                                           static_cast<float *>(workspace), grad_gates, grad_tokens,
                                                           grad_out_weight, grad_h0, st)));
}

// ------------------------------------------------------------------ channel-last layout -----
namespace {

bool make_btd_geom(fms::BtdGeom &g, int64_t B, int64_t T, int64_t D, int dtype) {
    const int64_t E = 16 / static_cast<int64_t>(elem_size(dtype));
    g.B = B;
    g.T = T;
    g.D = D;
    g.dtiles = (D + 32 * E - 1) / (32 * E);
    // enough warps to fill the GPU, chunks of at least 16 steps
    const int64_t target = tune().btd_warps_per_sm;
    int64_t want = (sm_count() * target + B * g.dtiles - 1) / (B * g.dtiles);
    want = std::max<int64_t>(1, std::min<int64_t>(want, (T + 15) / 16));
    g.chunk = (T + want - 1) / want;
    g.nchunks = (T + g.chunk - 1) / g.chunk;
    return true;
}

int btd_check(int64_t B, int64_t T, int64_t D, int dtype) {
    if (dtype != FMS_F32 && dtype != FMS_F16 && dtype != FMS_BF16) return FMS_ERR_BAD_DTYPE;
    if (B < 0 || T < 0 || D < 0) return FMS_ERR_BAD_SHAPE;
    if (B && D && (B > INT64_MAX / 8 / D || (T && B * D > INT64_MAX / 8 / T))) return FMS_ERR_BAD_SHAPE;
    return FMS_OK;
}

inline int64_t btd_ctas(const fms::BtdGeom &g) {
    return (g.B * g.nchunks * g.dtiles + fms::kBtdWarps - 1) / fms::kBtdWarps;
}

template <typename S>
int launch_btd_forward(const fms::BtdGeom &g, const void *gates, const void *tokens, const float *h0, void *states,
                       float *h_last, float *wP, float *wS, float *wC, cudaStream_t st) {
    const int64_t ctas = btd_ctas(g);
    if (ctas > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
    const unsigned grid = static_cast<unsigned>(ctas), block = fms::kBtdWarps * 32;
    constexpr size_t ring2 = fms::btd_ring_bytes<2>();
    auto kr = fms::btd_reduce_kernel<S, false>;
    auto kf = fms::btd_forward_kernel<S>;
    if (int rc = record(cudaFuncSetAttribute(kr, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ring2))))
        return rc;
    if (int rc = record(cudaFuncSetAttribute(kf, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ring2))))
        return rc;
    kr<<<grid, block, ring2, st>>>(static_cast<const S *>(gates), static_cast<const S *>(tokens), wP, wS, g);
    if (int rc = check_launch()) return rc;
    const int64_t fb = (g.B * g.D + 255) / 256;
    fms::btd_fold_kernel<<<static_cast<unsigned>(fb), 256, 0, st>>>(wP, wS, wC, h0, h_last, g, 0);
    if (int rc = check_launch()) return rc;
    kf<<<grid, block, ring2, st>>>(static_cast<const S *>(gates), static_cast<const S *>(tokens), wC,
                                   static_cast<S *>(states), g);
    return check_launch();
}

template <typename S>
int launch_btd_backward(const fms::BtdGeom &g, const void *gates, const void *states, const void *grad_states,
                        const float *h0, void *grad_gates, void *grad_tokens, float *grad_h0, float *wP, float *wS,
                        float *wC, cudaStream_t st) {
    const int64_t ctas = btd_ctas(g);
    if (ctas > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
    const unsigned grid = static_cast<unsigned>(ctas), block = fms::kBtdWarps * 32;
    constexpr size_t ring2 = fms::btd_ring_bytes<2>(), ring3 = fms::btd_ring_bytes<3>();
    auto kr = fms::btd_reduce_kernel<S, true>;
    auto kb = fms::btd_backward_kernel<S>;
    if (int rc = record(cudaFuncSetAttribute(kr, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ring2))))
        return rc;
    if (int rc = record(cudaFuncSetAttribute(kb, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ring3))))
        return rc;
    kr<<<grid, block, ring2, st>>>(static_cast<const S *>(gates), static_cast<const S *>(grad_states), wP, wS, g);
    if (int rc = check_launch()) return rc;
    const int64_t fb = (g.B * g.D + 255) / 256;
    fms::btd_fold_kernel<<<static_cast<unsigned>(fb), 256, 0, st>>>(wP, wS, wC, nullptr, grad_h0, g, 1);
    if (int rc = check_launch()) return rc;
    kb<<<grid, block, ring3, st>>>(static_cast<const S *>(gates), static_cast<const S *>(states),
                                   static_cast<const S *>(grad_states), h0, wC, static_cast<S *>(grad_gates),
                                   static_cast<S *>(grad_tokens), g);
    return check_launch();
}

}  // namespace

FMS_EXPORT size_t fms_btd_workspace_bytes(int64_t B, int64_t T, int64_t D, int dtype) {
    if (btd_check(B, T, D, dtype) != FMS_OK || B == 0 || T == 0 || D == 0) return 0;
    fms::BtdGeom g;
    make_btd_geom(g, B, T, D, dtype);
    return (static_cast<size_t>(3) * B * g.nchunks * D * sizeof(float) + 255) / 256 * 256;  // P, S, carries
}

FMS_EXPORT int fms_btd_forward(const void *gates, const void *tokens, const float *h0, void *states, float *h_last,
                               int64_t B, int64_t T, int64_t D, int dtype, void *workspace, size_t workspace_bytes,
                               fms_stream_t stream) {
    if (int rc = btd_check(B, T, D, dtype)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (B == 0 || D == 0) return FMS_OK;
    if (T == 0) return copy_or_zero(h0, h_last, B * D, 0.f, st);
    bool aligned = false;
    if (int rc = fm_alignment(aligned, D, dtype, gates, tokens, static_cast<const void *>(states))) return rc;
    if (!aligned) return FMS_ERR_MISALIGNED;  // D * element size must be a multiple of 16 bytes
    const size_t need = fms_btd_workspace_bytes(B, T, D, dtype);
    if (!workspace || !aligned_to(workspace, 16) || workspace_bytes < need) return FMS_ERR_WORKSPACE;
    fms::BtdGeom g;
    make_btd_geom(g, B, T, D, dtype);
    float *wP = static_cast<float *>(workspace), *wS = wP + B * g.nchunks * D, *wC = wS + B * g.nchunks * D;
    FMS_DISPATCH_DTYPE(dtype, (launch_btd_forward<S>(g, gates, tokens, h0, states, h_last, wP, wS, wC, st)));
}

FMS_EXPORT int fms_btd_backward(const void *gates, const void *states, const void *grad_states, const float *h0,
                                void *grad_gates, void *grad_tokens, float *grad_h0, int64_t B, int64_t T, int64_t D,
                                int dtype, void *workspace, size_t workspace_bytes, fms_stream_t stream) {
    if (int rc = btd_check(B, T, D, dtype)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (B == 0 || D == 0) return FMS_OK;
    if (T == 0) return copy_or_zero(nullptr, grad_h0, B * D, 0.f, st);
    bool aligned = false;
    if (int rc = fm_alignment(aligned, D, dtype, gates, states, grad_states, static_cast<const void *>(grad_gates),
                              static_cast<const void *>(grad_tokens)))
        return rc;
    if (!aligned) return FMS_ERR_MISALIGNED;
    const size_t need = fms_btd_workspace_bytes(B, T, D, dtype);
    if (!workspace || !aligned_to(workspace, 16) || workspace_bytes < need) return FMS_ERR_WORKSPACE;
    fms::BtdGeom g;
    make_btd_geom(g, B, T, D, dtype);
    float *wP = static_cast<float *>(workspace), *wS = wP + B * g.nchunks * D, *wC = wS + B * g.nchunks * D;
    FMS_DISPATCH_DTYPE(dtype, (launch_btd_backward<S>(g, gates, states, grad_states, h0, grad_gates, grad_tokens,
                                                      grad_h0, wP, wS, wC, st)));
}

// ------------------------------------------------------------------ split inside one GPU ----
namespace {

constexpr int64_t kSplitTargetUnits = 148 * 32;  // one-warp units that fill a B200 (148 SMs x 32 warps); a
                                                 // constant so that plans and workspace sizes do not
                                                 // depend on which device happens to be current
constexpr int64_t kSplitMinLength = 8192;        // rows shorter than this are never split
constexpr int64_t kSplitMinSegment = 2048;       // positions; shorter segments only add carries
constexpr int64_t kSplitQuantum = 1024;          // segment lengths are multiples of this, so
                                                 // segments of aligned rows stay 16-byte aligned

struct SplitPlan {
    int64_t nseg, seg_len, units;
    size_t bytes;
};

SplitPlan plan_split(int64_t rows, int64_t T) {
    SplitPlan p{1, T, rows, 0};
    if (rows <= 0 || T < kSplitMinLength || rows >= kSplitTargetUnits / 2) return p;
    int64_t want = (kSplitTargetUnits + rows - 1) / rows;
    want = std::min<int64_t>(want, T / kSplitMinSegment);
    if (want < 2) return p;
    int64_t seg = (T + want - 1) / want;
    seg = (seg + kSplitQuantum - 1) / kSplitQuantum * kSplitQuantum;
    p.nseg = (T + seg - 1) / seg;
    if (p.nseg < 2) return SplitPlan{1, T, rows, 0};
    p.seg_len = seg;
    p.units = rows * p.nseg;
    p.bytes = (static_cast<size_t>(p.units) * 3 * sizeof(float) + 255) / 256 * 256;
    return p;
}

}  // namespace

FMS_EXPORT int64_t fms_plain_split_segments(int64_t rows, int64_t T, int dtype) {
    if (dtype != FMS_F32 && dtype != FMS_F16 && dtype != FMS_BF16) return 1;
    if (!sizes_ok(rows, T)) return 1;
    return plan_split(rows, T).nseg;
}

// Measured on B200 (fwd+bwd, CUDA events, L2 flushed): with K warps sharing a row the unsplit
// kernels beat the three-launch split down to 64 rows at every length tried (8192 ... 131072;
// e.g. 64 rows x 131072 fp32: 99 us against 110 us; 256 x 32768: 52 against 97; 2304 x 16385 fp16:
// 127 against 242).  The split pays only when there are too few rows to give every SM a CTA of
// K warps.
FMS_EXPORT int fms_plain_split_recommended(int64_t rows, int64_t T, int dtype) {
    if (dtype != FMS_F32 && dtype != FMS_F16 && dtype != FMS_BF16) return 0;
    if (!sizes_ok(rows, T)) return 0;
    if (plan_split(rows, T).nseg < 2) return 0;
    return rows * 4 <= sm_count() ? 1 : 0;
}

FMS_EXPORT size_t fms_plain_split_workspace_bytes(int64_t rows, int64_t T, int dtype) {
    if (dtype != FMS_F32 && dtype != FMS_F16 && dtype != FMS_BF16) return 0;
    if (!sizes_ok(rows, T)) return 0;
    return plan_split(rows, T).bytes;
}

FMS_EXPORT int fms_plain_forward_split(const void *gates, const void *tokens, const float *h0, void *states,
                                       float *h_last, int64_t rows, int64_t T, int dtype, void *workspace,
                                       size_t workspace_bytes, fms_stream_t stream) {
    Problem pb;
    if (int rc = make_problem(pb, rows, T, dtype, gates, tokens, static_cast<const void *>(states)))
        return rc;
    const SplitPlan plan = plan_split(rows, T);
    if (plan.nseg == 1)
        return fms_plain_forward(gates, tokens, h0, states, h_last, rows, T, dtype, stream);
    if (!workspace || !aligned_to(workspace, 16) || workspace_bytes < plan.bytes) return FMS_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *wP = static_cast<float *>(workspace), *wS = wP + plan.units, *wC = wS + plan.units;
    const Split sp{plan.nseg, plan.seg_len};
    {
        auto pass1 = [&]() -> int {
            FMS_DISPATCH_DTYPE(dtype, (launch_forward<S, false>(pb, sp, gates, tokens, nullptr, nullptr, wS, wP, st)));
        };
        if (int rc = pass1()) return rc;
    }
    if (int rc = launch_combine(wP, wS, h0, wC, h_last, plan.nseg, rows, 0, 1, plan.nseg, st)) return rc;
    FMS_DISPATCH_DTYPE(dtype, (launch_forward<S, true>(pb, sp, gates, tokens, wC, states, nullptr, nullptr, st)));
}

FMS_EXPORT int fms_plain_backward_split(const void *gates, const void *states, const void *grad_states,
                                        const float *h0, const float *carry_in, void *grad_gates,
                                        void *grad_tokens, float *grad_h0, int64_t rows, int64_t T,
                                        int dtype, void *workspace, size_t workspace_bytes,
                                        fms_stream_t stream) {
    Problem pb;
    if (int rc = make_problem(pb, rows, T, dtype, gates, states, grad_states,
                              static_cast<const void *>(grad_gates),
                              static_cast<const void *>(grad_tokens)))
        return rc;
    const SplitPlan plan = plan_split(rows, T);
    if (plan.nseg == 1)
        return fms_plain_backward(gates, states, grad_states, h0, carry_in, grad_gates, grad_tokens, grad_h0,
                                  rows, T, dtype, stream);
    if (!workspace || !aligned_to(workspace, 16) || workspace_bytes < plan.bytes) return FMS_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *wP = static_cast<float *>(workspace), *wS = wP + plan.units, *wC = wS + plan.units;
    const Split sp{plan.nseg, plan.seg_len};
    {
        auto pass1 = [&]() -> int {
            FMS_DISPATCH_DTYPE(dtype, (launch_backward<S, false>(pb, sp, gates, nullptr, grad_states, nullptr,
                                                                 nullptr, nullptr, nullptr, wS, wP, st)));
        };
        if (int rc = pass1()) return rc;
    }
    if (int rc = launch_combine(wP, wS, carry_in, wC, grad_h0, plan.nseg, rows, 1, 1, plan.nseg, st)) return rc;
    FMS_DISPATCH_DTYPE(dtype, (launch_backward<S, true>(pb, sp, gates, states, grad_states, h0, wC, grad_gates,
                                                        grad_tokens, nullptr, nullptr, st)));
}

// ------------------------------------------------- split forward with built-in scratch ----
// The carries of fms_plain_forward_split_static live here, in the library's device image, so
// the entry point never touches the allocator.  In host code the name below is only a handle:
// the address kernels may use is looked up per device with cudaGetSymbolAddress.
static __device__ __align__(256) float g_static_scratch[3 * FMS_STATIC_SCRATCH_MAX_UNITS];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
float *g_static_scratch_ptr[kMaxDevices] = {};

// Device address of g_static_scratch on the current device (resolved once per device).
int static_scratch_on_current_device(float **out) {
    int dev = -1;
    if (int rc = record(cudaGetDevice(&dev))) return rc;
    if (dev < 0 || dev >= kMaxDevices) return FMS_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_scratch_ptr[dev]) {
        void *p = nullptr;
        if (int rc = record(cudaGetSymbolAddress(&p, g_static_scratch))) return rc;
        if (!p) return FMS_ERR_LAUNCH;
        g_static_scratch_ptr[dev] = static_cast<float *>(p);
    }
    *out = g_static_scratch_ptr[dev];
    return FMS_OK;
}

}  // namespace

FMS_EXPORT int fms_plain_forward_split_static(const void *gates, const void *tokens, const float *h0,
                                              void *states, float *h_last, int64_t rows, int64_t T,
                                              int dtype, fms_stream_t stream) {
    Problem pb;
    if (int rc = make_problem(pb, rows, T, dtype, gates, tokens, static_cast<const void *>(states)))
        return rc;
    SplitPlan plan = plan_split(rows, T);
    if (plan.nseg == 1)  // no scratch involved
        return fms_plain_forward(gates, tokens, h0, states, h_last, rows, T, dtype, stream);
    if (plan.units > FMS_STATIC_SCRATCH_MAX_UNITS) {
        // The library's own plan aims a little above the array's capacity.  Re-plan inside it with
        // fewer, longer segments; refuse only when not even two segments per row fit.
        if (rows * 2 > FMS_STATIC_SCRATCH_MAX_UNITS) return FMS_ERR_TOO_LARGE;
        const int64_t want = std::min<int64_t>(plan.nseg, FMS_STATIC_SCRATCH_MAX_UNITS / rows);
        int64_t seg = (T + want - 1) / want;
        seg = (seg + kSplitQuantum - 1) / kSplitQuantum * kSplitQuantum;
        plan.nseg = (T + seg - 1) / seg;
        plan.seg_len = seg;
        plan.units = rows * plan.nseg;
        if (plan.nseg < 2) return fms_plain_forward(gates, tokens, h0, states, h_last, rows, T, dtype, stream);
    }
    float *scratch = nullptr;
    if (int rc = static_scratch_on_current_device(&scratch)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *wP = scratch, *wS = wP + plan.units, *wC = wS + plan.units;
    const Split sp{plan.nseg, plan.seg_len};
    {
        auto pass1 = [&]() -> int {
            FMS_DISPATCH_DTYPE(dtype, (launch_forward<S, false>(pb, sp, gates, tokens, nullptr, nullptr, wS, wP, st)));
        };
        if (int rc = pass1()) return rc;
    }
    if (int rc = launch_combine(wP, wS, h0, wC, h_last, plan.nseg, rows, 0, 1, plan.nseg, st)) return rc;
    FMS_DISPATCH_DTYPE(dtype, (launch_forward<S, true>(pb, sp, gates, tokens, wC, states, nullptr, nullptr, st)));
}
