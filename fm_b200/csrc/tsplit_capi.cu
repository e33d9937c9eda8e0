// C ABI of the fused split-along-T scan (tsplit_kernels.cuh); declared in include/fm_scan_b200.h.
#include <algorithm>
#include <cstdlib>

#include "fm_scan_b200.h"
#include "tsplit_kernels.cuh"
#include "tsplit_tma_kernels.cuh"

#define FMS_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

inline bool dtype_ok(int dtype) { return dtype == FMS_F32 || dtype == FMS_F16 || dtype == FMS_BF16; }
inline size_t elem_size(int dtype) { return dtype == FMS_F32 ? 4 : 2; }
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool layout_ok(int64_t rows, int world, int rank) {
    return rows >= 0 && world >= 1 && world <= FMS_MAX_PEERS && rank >= 0 && rank < world;
}

long long wait_cycles(double max_wait_seconds) {
    if (!(max_wait_seconds > 0.0) || max_wait_seconds > 30.0) max_wait_seconds = 2.0;
    static const int khz = []() {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, dev) != cudaSuccess ||
            v <= 0)
            v = 1965000;
        return v;
    }();
    return static_cast<long long>(max_wait_seconds * 1e3 * static_cast<double>(khz));
}

int env_int(const char *name, int dflt) {
    const char *s = std::getenv(name);
    return s ? std::atoi(s) : dflt;
}

// Launch shape: K warps per row, U tiles per warp and step, CTAs per SM.  Fewer, larger CTAs keep
// fewer rows in flight, which is what lets pass B find its operands in L2 (rows in flight x row
// bytes x tensors must stay well inside the 126 MB).  Read once per process.
struct TsTune {
    int k, u, bwd_u, ctas_per_sm, staged, l2_hint, look;
};
const TsTune &ts_tune() {
    // staged = 1 (default): operands come through the bulk-copy shared-memory ring, one CTA per SM
    // (K defaults to 16 there); 0: the register-prefetch kernels (K defaults to 8, two CTAs per SM)
    static const TsTune t = []() {
        TsTune v;
        v.staged = env_int("FMS_TUNE_TSPLIT_STAGED", 1);
        v.k = env_int("FMS_TUNE_TSPLIT_K", v.staged ? 16 : 8);
        v.u = env_int("FMS_TUNE_TSPLIT_U", 4);
        v.bwd_u = env_int("FMS_TUNE_TSPLIT_BWD_U", 2);
        v.ctas_per_sm = env_int("FMS_TUNE_TSPLIT_CTAS_PER_SM", 2);
        v.l2_hint = env_int("FMS_TUNE_TSPLIT_L2_HINT", 0);
        v.look = env_int("FMS_TUNE_TSPLIT_LOOK", -1);  // -1: chosen from the number of ranks
        return v;
    }();
    return t;
}

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
int64_t grid_for(Kernel kernel, int threads, int64_t rows) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess || per_sm <= 0)
        per_sm = 1;
    per_sm = std::min(per_sm, std::max(1, ts_tune().ctas_per_sm));
    const int64_t resident = static_cast<int64_t>(per_sm) * sm_count();
    // every CTA walks the same number of rows, all CTAs resident (they wait on peers)
    const int64_t q = (rows + resident - 1) / resident;
    return (rows + q - 1) / q;
}

int make_exchange(fms::TsExchange &ex, void *const *peer_buffers, int64_t rows, int world, int rank, uint32_t exchange,
                  double max_wait_seconds) {
    if (!layout_ok(rows, world, rank) || exchange == 0) return FMS_ERR_BAD_SHAPE;
    if (!peer_buffers) return FMS_ERR_NULL_POINTER;
    for (int p = 0; p < world; ++p) {
        if (!peer_buffers[p]) return FMS_ERR_NULL_POINTER;
        if (!aligned16(peer_buffers[p])) return FMS_ERR_MISALIGNED;
        ex.buf[p] = static_cast<char *>(peer_buffers[p]);
    }
    ex.lay = fms::TsLayout{rows, world};
    ex.rank = rank;
    ex.epoch = exchange;
    ex.max_wait_cycles = wait_cycles(max_wait_seconds);
    ex.l2_hint = ts_tune().l2_hint;
    // Look-ahead of one super-tile pays once the exchange latency of several ranks stacks up
    // (configuration 4, fwd+bwd: 8 GPUs 0.842 -> 0.833 ms; 2 GPUs with the same block 0.754 -> 0.773 ms).
    ex.look = ts_tune().look >= 0 ? ts_tune().look : (world >= 4 ? 1 : 0);
    return FMS_OK;
}

// Staged kernels: one CTA per SM, every CTA the same number of rows.
inline int64_t staged_grid(int64_t rows) {
    const int64_t resident = sm_count();
    const int64_t q = (rows + resident - 1) / resident;
    return (rows + q - 1) / q;
}

template <typename S>
int launch_forward_staged(const void *gates, const void *tokens, const float *h0, void *states, float *h_in_out,
                          const fms::TsExchange &ex, int64_t rows, int64_t T, cudaStream_t st) {
#define FMS_TS_FWD_STAGED(UU, KK, NS)                                                                         \
    do {                                                                                                     \
        auto kern = fms::tsplit_forward_tma_kernel<S, UU, KK, NS>;                                           \
        constexpr size_t smem = fms::TsRing<S, UU, KK, 2, NS>::kBytes;                                       \
        constexpr int64_t super = fms::TsRing<S, UU, KK, 2, NS>::SUPER;                                      \
        if ((T + super - 1) / super * KK > fms::kTsMaxAgg) return FMS_ERR_TOO_LARGE;                         \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != \
            cudaSuccess)                                                                                     \
            return FMS_ERR_LAUNCH;                                                                           \
        kern<<<static_cast<unsigned>(staged_grid(rows)), (KK + 1) * 32, smem, st>>>(                         \
            static_cast<const S *>(gates), static_cast<const S *>(tokens), h0, static_cast<S *>(states), h_in_out, \
            ex, rows, T);                                                                                    \
    } while (0)
    if (ts_tune().k == 8) FMS_TS_FWD_STAGED(4, 8, 6);
    else if (ts_tune().k == 24) FMS_TS_FWD_STAGED(2, 24, 4);
    else if (ts_tune().u == 2) FMS_TS_FWD_STAGED(2, 16, 6);
    else FMS_TS_FWD_STAGED(4, 16, 3);
#undef FMS_TS_FWD_STAGED
    return cudaGetLastError() == cudaSuccess ? FMS_OK : FMS_ERR_LAUNCH;
}

template <typename S>
int launch_backward_staged(const void *gates, const void *states, const void *grad_states, const float *h_in,
                           void *grad_gates, void *grad_tokens, float *grad_h0, const fms::TsExchange &ex,
                           int64_t rows, int64_t T, cudaStream_t st) {
#define FMS_TS_BWD_STAGED(UU, KK, NS)                                                                         \
    do {                                                                                                     \
        auto kern = fms::tsplit_backward_tma_kernel<S, UU, KK, NS>;                                          \
        constexpr size_t smem = fms::TsRing<S, UU, KK, 3, NS>::kBytes;                                       \
        constexpr int64_t super = fms::TsRing<S, UU, KK, 3, NS>::SUPER;                                      \
        if ((T + super - 1) / super * KK > fms::kTsMaxAgg) return FMS_ERR_TOO_LARGE;                         \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != \
            cudaSuccess)                                                                                     \
            return FMS_ERR_LAUNCH;                                                                           \
        kern<<<static_cast<unsigned>(staged_grid(rows)), (KK + 1) * 32, smem, st>>>(                         \
            static_cast<const S *>(gates), static_cast<const S *>(states), static_cast<const S *>(grad_states), \
            h_in, static_cast<S *>(grad_gates), static_cast<S *>(grad_tokens), grad_h0, ex, rows, T);        \
    } while (0)
    if (ts_tune().k == 8) FMS_TS_BWD_STAGED(4, 8, 4);
    else if (ts_tune().k == 24) FMS_TS_BWD_STAGED(2, 24, 3);
    else FMS_TS_BWD_STAGED(2, 16, 4);
#undef FMS_TS_BWD_STAGED
    return cudaGetLastError() == cudaSuccess ? FMS_OK : FMS_ERR_LAUNCH;
}

template <typename S>
int launch_forward(const void *gates, const void *tokens, const float *h0, void *states, float *h_in_out,
                   const fms::TsExchange &ex, int64_t rows, int64_t T, cudaStream_t st) {
    if (ts_tune().staged) {
        // blocks too long for the staged kernels' per-row aggregate table use the register kernels
        const int rc = launch_forward_staged<S>(gates, tokens, h0, states, h_in_out, ex, rows, T, st);
        if (rc != FMS_ERR_TOO_LARGE) return rc;
    }
    const int K = ts_tune().k == 16 ? 16 : 8, U = ts_tune().u;
#define FMS_TS_FWD(UU, KK)                                                                                   \
    do {                                                                                                     \
        auto kern = fms::tsplit_forward_kernel<S, UU, KK>;                                                   \
        const int64_t grid = grid_for(kern, KK * 32, rows);                                                  \
        kern<<<static_cast<unsigned>(grid), KK * 32, 0, st>>>(static_cast<const S *>(gates),                 \
                                                              static_cast<const S *>(tokens), h0,            \
                                                              static_cast<S *>(states), h_in_out, ex, rows, T); \
    } while (0)
    if (K == 16) {
        if (U == 2) FMS_TS_FWD(2, 16);
        else FMS_TS_FWD(4, 16);
    } else {
        if (U == 2) FMS_TS_FWD(2, 8);
        else FMS_TS_FWD(4, 8);
    }
#undef FMS_TS_FWD
    return cudaGetLastError() == cudaSuccess ? FMS_OK : FMS_ERR_LAUNCH;
}

template <typename S>
int launch_backward(const void *gates, const void *states, const void *grad_states, const float *h_in,
                    void *grad_gates, void *grad_tokens, float *grad_h0, const fms::TsExchange &ex, int64_t rows,
                    int64_t T, cudaStream_t st) {
    if (ts_tune().staged) {
        const int rc = launch_backward_staged<S>(gates, states, grad_states, h_in, grad_gates, grad_tokens, grad_h0,
                                                 ex, rows, T, st);
        if (rc != FMS_ERR_TOO_LARGE) return rc;
    }
    // three input streams: 4 tiles per step need 189 registers (one CTA of 8 warps per SM), 2 need 128
    const int K = ts_tune().k == 16 ? 16 : 8, U = ts_tune().bwd_u;
#define FMS_TS_BWD(UU, KK)                                                                                   \
    do {                                                                                                     \
        auto kern = fms::tsplit_backward_kernel<S, UU, KK>;                                                  \
        const int64_t grid = grid_for(kern, KK * 32, rows);                                                  \
        kern<<<static_cast<unsigned>(grid), KK * 32, 0, st>>>(                                               \
            static_cast<const S *>(gates), static_cast<const S *>(states), static_cast<const S *>(grad_states), \
            h_in, static_cast<S *>(grad_gates), static_cast<S *>(grad_tokens), grad_h0, ex, rows, T);        \
    } while (0)
    if (K == 16) {
        FMS_TS_BWD(2, 16);  // 4 tiles per step would not fit the registers of 512 threads
    } else {
        if (U == 2) FMS_TS_BWD(2, 8);
        else FMS_TS_BWD(4, 8);
    }
#undef FMS_TS_BWD
    return cudaGetLastError() == cudaSuccess ? FMS_OK : FMS_ERR_LAUNCH;
}

#define FMS_TS_DISPATCH(dtype, CALL)                          \
    switch (dtype) {                                          \
        case FMS_F32: { using S = float; return CALL; }       \
        case FMS_F16: { using S = __half; return CALL; }      \
        default: { using S = __nv_bfloat16; return CALL; }    \
    }

int check_rows(int64_t rows, int64_t T, int dtype, std::initializer_list<const void *> big) {
    if (!dtype_ok(dtype)) return FMS_ERR_BAD_DTYPE;
    if (rows < 0 || T < 0 || (rows > 0 && T > 0 && rows > (INT64_MAX / 8) / T)) return FMS_ERR_BAD_SHAPE;
    if (rows == 0 || T == 0) return FMS_OK;
    for (const void *p : big)
        if (!p) return FMS_ERR_NULL_POINTER;
    // the fused kernels use 16-byte vectors only: callers with other layouts use the three-step path
    if ((static_cast<uint64_t>(T) * elem_size(dtype)) % 16 != 0) return FMS_ERR_MISALIGNED;
    for (const void *p : big)
        if (!aligned16(p)) return FMS_ERR_MISALIGNED;
    return FMS_OK;
}

}  // namespace

FMS_EXPORT size_t fms_tsplit_exchange_bytes(int64_t rows, int world) {
    if (!layout_ok(rows, world, 0)) return 0;
    return fms::TsLayout{rows, world}.total_bytes();
}

FMS_EXPORT size_t fms_tsplit_exchange_status_offset(int64_t rows, int world) {
    if (!layout_ok(rows, world, 0)) return 0;
    return fms::TsLayout{rows, world}.status_offset();
}

FMS_EXPORT int fms_tsplit_forward(const void *gates, const void *tokens, const float *h0, void *states,
                                  float *h_in_out, int64_t rows, int64_t T, int dtype, void *const *peer_buffers,
                                  int world, int rank, uint32_t exchange, double max_wait_seconds,
                                  fms_stream_t stream) {
    if (int rc = check_rows(rows, T, dtype, {gates, tokens, static_cast<const void *>(states)})) return rc;
    fms::TsExchange ex;
    if (int rc = make_exchange(ex, peer_buffers, rows, world, rank, exchange, max_wait_seconds)) return rc;
    if (rows == 0) return FMS_OK;
    if (T == 0) return FMS_ERR_BAD_SHAPE;  // an empty block has nothing to publish from: not supported
    if (!h_in_out) return FMS_ERR_NULL_POINTER;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    FMS_TS_DISPATCH(dtype, (launch_forward<S>(gates, tokens, h0, states, h_in_out, ex, rows, T, st)));
}

FMS_EXPORT int fms_tsplit_backward(const void *gates, const void *states, const void *grad_states,
                                   const float *h_in, void *grad_gates, void *grad_tokens, float *grad_h0,
                                   int64_t rows, int64_t T, int dtype, void *const *peer_buffers, int world,
                                   int rank, uint32_t exchange, double max_wait_seconds, fms_stream_t stream) {
    if (int rc = check_rows(rows, T, dtype,
                            {gates, states, grad_states, static_cast<const void *>(grad_gates),
                             static_cast<const void *>(grad_tokens)}))
        return rc;
    fms::TsExchange ex;
    if (int rc = make_exchange(ex, peer_buffers, rows, world, rank, exchange, max_wait_seconds)) return rc;
    if (rows == 0) return FMS_OK;
    if (T == 0) return FMS_ERR_BAD_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    FMS_TS_DISPATCH(dtype, (launch_backward<S>(gates, states, grad_states, h_in, grad_gates, grad_tokens, grad_h0, ex,
                                               rows, T, st)));
}
