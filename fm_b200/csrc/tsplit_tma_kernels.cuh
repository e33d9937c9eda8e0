// The fused split-along-T kernels of tsplit_kernels.cuh with their operands staged through a
// shared-memory ring by bulk asynchronous copies (cp.async.bulk + mbarrier, the 1-D form of TMA).
//
// Why: the second pass of a row finds its operands in L2 only while few rows are in flight (148
// rows x 256 KB on the long-sequence workload; with 296 rows most of it has been evicted).  One
// CTA per SM with register prefetch keeps too few bytes in flight to fill HBM from so few rows.
// Here a producer warp streams the row into a ring of STAGES x (one super-tile of every operand)
// -- up to ~200 KB per SM in flight, independent of the consumers' barriers, of the peer wait
// between the two passes and of row boundaries -- and K consumer warps take their tiles from
// shared memory.  A stage is K*U tiles of 512 B per operand; consumers release a stage as soon as
// its tiles are in registers.
//
// The copies read THIS GPU's memory only and are not multicast.  Every mbarrier wait is bounded;
// a wait that runs out raises the CTA's fault flag, every role stops at its next wait, the
// producer drains the copies still in flight (bounded) and the kernel ends with the fault in the
// status word.
#pragma once

#include "tsplit_kernels.cuh"

namespace fms {

constexpr int FMS_TSPLIT_ERR_PIPELINE = 5;  // status word: an mbarrier wait of the staging ring ran out
constexpr unsigned kTsMbarSpins = 1u << 26;  // try_wait polls before a ring wait gives up (seconds)

__device__ __forceinline__ unsigned ts_smem_addr(const void *p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void ts_mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ts_smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void ts_mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ts_smem_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void ts_mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ts_smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool ts_mbar_try_wait(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(ts_smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false = gave up (or another role already raised the ring fault).
__device__ __forceinline__ bool ts_mbar_wait(uint64_t *bar, unsigned parity, volatile int *fault) {
    for (unsigned spin = 0; spin < kTsMbarSpins; ++spin) {
        if (ts_mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *fault == FMS_TSPLIT_ERR_PIPELINE) return false;
    }
    return false;
}
// A role whose ring wait ran out: raise the CTA's fault flag and record it in the status word.
__device__ __forceinline__ void ts_ring_fault(const TsExchange &ex, volatile int *fault) {
    *fault = FMS_TSPLIT_ERR_PIPELINE;
    atomicCAS(reinterpret_cast<uint32_t *>(ex.buf[ex.rank] + ex.lay.status_offset()), 0u,
              static_cast<uint32_t>(FMS_TSPLIT_ERR_PIPELINE));
}
// Bulk copy global -> shared of this CTA, completion counted in bytes on `bar`.
__device__ __forceinline__ void ts_bulk_load(void *smem_dst, const void *gmem_src, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     ts_smem_addr(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(ts_smem_addr(bar))
                 : "memory");
}
// The same copy with an L2 eviction policy: the first pass of a row asks L2 to keep the lines
// (evict-last), the second pass releases them (evict-first).
__device__ __forceinline__ void ts_bulk_load_hint(void *smem_dst, const void *gmem_src, unsigned bytes, uint64_t *bar,
                                                  uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
            "r"(ts_smem_addr(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(ts_smem_addr(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t ts_policy(bool keep) {
    uint64_t pol;
    if (keep) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    else asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void ts_consumer_sync(int threads) {
    asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

// Aggregates of one row's block, one (P, S) pair per (super-tile, warp) in walk order.  The first
// pass writes them (each warp its own, no barrier); then ONE warp turns them, in place, into
// exclusive prefixes -- the pair that maps the block's carry-in to the carry entering that warp's
// tiles -- and returns the block's total.  The second pass then needs no barrier at all: every
// warp starts each super-tile from  fma(prefix.P, carry_in, prefix.S).
constexpr int kTsMaxAgg = 512;  // (super-tiles per block) x K must fit (two tables: this row's and the next
                                // row's); longer blocks use the register kernels

__device__ __forceinline__ float2 ts_scan_aggregates(float2 *aggs, int n, int lane) {
    float rp = 1.f, rs = 0.f;  // running total of the chunks done so far
    for (int base = 0; base < n; base += 32) {
        const int i = base + lane;
        const float2 v = i < n ? aggs[i] : make_float2(1.f, 0.f);
        float P = v.x, Sv = v.y;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const float pP = __shfl_up_sync(kFullMask, P, d);
            const float pS = __shfl_up_sync(kFullMask, Sv, d);
            if (lane >= d) {
                Sv = fmaf(P, pS, Sv);
                P *= pP;
            }
        }
        float eP = __shfl_up_sync(kFullMask, P, 1), eS = __shfl_up_sync(kFullMask, Sv, 1);
        if (lane == 0) {
            eP = 1.f;
            eS = 0.f;
        }
        if (i < n) aggs[i] = make_float2(eP * rp, fmaf(eP, rs, eS));
        const float tP = __shfl_sync(kFullMask, P, 31), tS = __shfl_sync(kFullMask, Sv, 31);
        rs = fmaf(tP, rs, tS);
        rp *= tP;
    }
    return make_float2(rp, rs);
}

// Order in which a CTA visits (pass, row, super-tile).  Between the two passes of a row the
// first `look` super-tiles of the NEXT row's first pass are slipped in: a row's carries are then
// published that much earlier relative to the moment the other ranks need them, which hides the
// NVLink latency of the exchange (with look = 0 every rank meets every row's carries one hop
// late).  The price is L2 footprint: (1 + look / super-tiles-per-row) rows per CTA in flight.
//   A(r0) | [A(r1) first `look`]  B(r0)  [A(r1) rest] | [A(r2) first `look`]  B(r1)  [A(r2) rest] | ...
// Producer and consumers run the same walk; `fn(pass, i, step)` is called for the i-th row of
// the CTA and the step-th super-tile in walk order of that pass.
template <typename F>
__device__ __forceinline__ void ts_walk(int64_t m, int64_t ngroups, int64_t look, F &&fn) {
    if (m <= 0) return;
    for (int64_t g = 0; g < ngroups; ++g) fn(0, static_cast<int64_t>(0), g);
    for (int64_t i = 0; i < m; ++i) {
        if (i + 1 < m)
            for (int64_t g = 0; g < look; ++g) fn(0, i + 1, g);
        for (int64_t g = 0; g < ngroups; ++g) fn(1, i, g);
        if (i + 1 < m)
            for (int64_t g = look; g < ngroups; ++g) fn(0, i + 1, g);
    }
}

// Shared memory of one CTA: NT operands per stage, each SUPER elements of S.
template <typename S, int U, int K, int NT, int STAGES>
struct TsRing {
    static constexpr int E = Store<S>::E;
    static constexpr int TILE = 32 * E;
    static constexpr int SUPER = TILE * U * K;
    static constexpr size_t kStageBytes = static_cast<size_t>(NT) * SUPER * sizeof(S);
    static constexpr size_t kBytes = STAGES * kStageBytes + 2 * STAGES * sizeof(uint64_t) + 256;
};

// ---------------------------------------------------------------- forward --------------------
template <typename S, int U, int K, int STAGES>
__global__ void __launch_bounds__((K + 1) * 32, 1)
tsplit_forward_tma_kernel(const S *__restrict__ gates, const S *__restrict__ tokens, const float *__restrict__ h0,
                          S *__restrict__ states, float *__restrict__ h_in_out, TsExchange ex, int64_t R, int64_t T) {
    using Ring = TsRing<S, U, K, 2, STAGES>;
    constexpr int E = Ring::E, TILE = Ring::TILE;
    constexpr int64_t SUPER = Ring::SUPER;
    extern __shared__ __align__(128) unsigned char ts_smem[];
    S *stage_base = reinterpret_cast<S *>(ts_smem);
    uint64_t *full = reinterpret_cast<uint64_t *>(ts_smem + STAGES * Ring::kStageBytes);
    uint64_t *empty = full + STAGES;
    __shared__ float2 aggs[2][kTsMaxAgg];  // by parity of the CTA's row counter
    __shared__ float s_carry;
    __shared__ int s_fault;
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ts_mbar_init(full + s, 1);
            ts_mbar_init(empty + s, K);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_fault = ts_wait_acks(ex, 0);
        if (s_fault)
            atomicCAS(reinterpret_cast<uint32_t *>(ex.buf[ex.rank] + ex.lay.status_offset()), 0u,
                      static_cast<uint32_t>(s_fault));
    }
    __syncthreads();
    const bool publish_ok = s_fault == 0;
    const int64_t ngroups = (T + SUPER - 1) / SUPER;
    const int64_t m = (R - blockIdx.x + gridDim.x - 1) / gridDim.x;  // rows of this CTA
    const int64_t look = min(static_cast<int64_t>(ex.look), ngroups);

    if (w == K) {
        // ---------------- producer: one lane streams the walk in consumption order
        if (lane == 0) {
            unsigned n = 0;
            bool alive = true;
            const uint64_t pol_keep = ts_policy(true), pol_release = ts_policy(false);
            ts_walk(m, ngroups, look, [&](int pass, int64_t i, int64_t g) {
                if (!alive) return;
                const int s = static_cast<int>(n % STAGES);
                if (!ts_mbar_wait(empty + s, ((n / STAGES) & 1u) ^ 1u, &s_fault)) {
                    alive = false;
                    return;
                }
                const int64_t off = (blockIdx.x + i * gridDim.x) * T, e0 = g * SUPER;
                const unsigned bytes = static_cast<unsigned>(min(SUPER, T - e0) * sizeof(S));
                S *dst = stage_base + static_cast<size_t>(s) * 2 * SUPER;
                ts_mbar_expect_tx(full + s, 2 * bytes);
                if (ex.l2_hint) {
                    const uint64_t pol = pass == 0 ? pol_keep : pol_release;
                    ts_bulk_load_hint(dst, gates + off + e0, bytes, full + s, pol);
                    ts_bulk_load_hint(dst + SUPER, tokens + off + e0, bytes, full + s, pol);
                } else {
                    ts_bulk_load(dst, gates + off + e0, bytes, full + s);
                    ts_bulk_load(dst + SUPER, tokens + off + e0, bytes, full + s);
                }
                ++n;
            });
            if (!alive) {
                ts_ring_fault(ex, &s_fault);
                // drain: every stage that was filled completes its copies within the bound
                for (unsigned k = n > STAGES ? n - STAGES : 0; k < n; ++k) {
                    const int s = static_cast<int>(k % STAGES);
                    for (unsigned spin = 0; spin < kTsMbarSpins && !ts_mbar_try_wait(full + s, (k / STAGES) & 1u); ++spin) {
                    }
                }
            }
        }
    } else {
        // ---------------- consumers: K warps, the arithmetic of tsplit_forward_kernel.
        // Inside a pass the warps run free (the ring's barriers are the only coupling); the CTA
        // meets at two named barriers per row: when the row's first pass is complete (warp 0 then
        // scans the aggregates and publishes) and before its second pass (warp 0 has the carry-in).
        // A warp whose ring wait ran out keeps walking (every warp must meet every named barrier)
        // but touches neither the ring nor global memory any more.
        const int64_t e_lane = static_cast<int64_t>(w) * (TILE * U) + lane * E;  // element offset inside a stage
        unsigned n = 0;
        bool alive = true;
        float hin = 0.f;
        ts_walk(m, ngroups, look, [&](int pass, int64_t i, int64_t g) {
            const int64_t row = blockIdx.x + i * gridDim.x, off = row * T;
            float2 *tab = aggs[i & 1];
            if (pass == 1 && g == 0) {
                // the carry entering this row's block: wait for the earlier blocks (published long ago
                // when look > 0) and fold them
                if (w == 0 && alive) {
                    float c_in = ts_wait_row(ex, 0, row, lane, &s_fault);
                    if (ex.rank == 0) c_in = h0 ? h0[row] : 0.f;
                    if (lane == 0) {
                        s_carry = c_in;
                        h_in_out[row] = c_in;
                    }
                }
                ts_consumer_sync(K * 32);  // prefixes (scanned after the first pass) and the carry-in are visible
                hin = s_carry;
            }
            if (alive) {
                const int s = static_cast<int>(n % STAGES);
                if (!ts_mbar_wait(full + s, (n / STAGES) & 1u, &s_fault)) {
                    alive = false;
                    if (lane == 0) ts_ring_fault(ex, &s_fault);
                }
            }
            if (alive) {
                const int s = static_cast<int>(n % STAGES);
                const S *sa = stage_base + static_cast<size_t>(s) * 2 * SUPER;
                const S *sx = sa + SUPER;
                const int64_t v = g * SUPER + e_lane;
                uint4 ra[U], rx[U];
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    const bool in = v + j * TILE < T;
                    ra[j] = in ? *reinterpret_cast<const uint4 *>(sa + e_lane + j * TILE)
                               : make_uint4(Store<S>::kOne, Store<S>::kOne, Store<S>::kOne, Store<S>::kOne);
                    rx[j] = in ? *reinterpret_cast<const uint4 *>(sx + e_lane + j * TILE) : make_uint4(0u, 0u, 0u, 0u);
                }
                __syncwarp();
                if (lane == 0) ts_mbar_arrive(empty + s);  // this warp's tiles are in registers

                float fa[U][E], fx[U][E], A[U], H[U];
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    Store<S>::unpack(ra[j], fa[j]);
                    Store<S>::unpack(rx[j], fx[j]);
                    A[j] = fa[j][0];
                    H[j] = fx[j][0];
#pragma unroll
                    for (int k = 1; k < E; ++k) {
                        H[j] = fmaf(fa[j][k], H[j], fx[j][k]);
                        A[j] *= fa[j][k];
                    }
                }
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
                    for (int j = 0; j < U; ++j) {
                        const float pA = __shfl_up_sync(kFullMask, A[j], d);
                        const float pH = __shfl_up_sync(kFullMask, H[j], d);
                        if (lane >= d) {
                            H[j] = fmaf(A[j], pH, H[j]);
                            A[j] *= pA;
                        }
                    }
                }
                const int slot = static_cast<int>(g) * K + w;
                if (pass == 0) {
                    float WA = __shfl_sync(kFullMask, A[0], 31), WH = __shfl_sync(kFullMask, H[0], 31);
#pragma unroll
                    for (int j = 1; j < U; ++j) {
                        const float tA = __shfl_sync(kFullMask, A[j], 31);
                        WH = fmaf(tA, WH, __shfl_sync(kFullMask, H[j], 31));
                        WA *= tA;
                    }
                    if (lane == 0) tab[slot] = make_float2(WA, WH);
                } else {
                    const float2 pre = tab[slot];
                    float c = fmaf(pre.x, hin, pre.y);  // state entering this warp's first tile
#pragma unroll
                    for (int j = 0; j < U; ++j) {
                        const float tA = __shfl_sync(kFullMask, A[j], 31);
                        const float tH = __shfl_sync(kFullMask, H[j], 31);
                        float eA = __shfl_up_sync(kFullMask, A[j], 1);
                        float eH = __shfl_up_sync(kFullMask, H[j], 1);
                        if (lane == 0) {
                            eA = 1.f;
                            eH = 0.f;
                        }
                        float st = fmaf(eA, c, eH);
                        float out[E];
#pragma unroll
                        for (int k = 0; k < E; ++k) {
                            st = fmaf(fa[j][k], st, fx[j][k]);
                            out[k] = st;
                        }
                        store_vec<S, false>(states + off, v + j * TILE, T, true, Store<S>::pack(out));
                        c = fmaf(tA, c, tH);
                    }
                }
            }
            ++n;
            if (pass == 0 && g == ngroups - 1) {
                ts_consumer_sync(K * 32);  // every warp's aggregates of this row are in shared memory
                if (w == 0 && alive) {
                    const float2 total = ts_scan_aggregates(tab, static_cast<int>(ngroups) * K, lane);
                    float S_pub = total.y;
                    if (ex.rank == 0 && h0) S_pub = fmaf(total.x, h0[row], total.y);  // the first block folds h0 in
                    ts_publish_row(ex, 0, row, total.x, S_pub, publish_ok, lane);
                }
            }
        });
    }
    __syncthreads();
    if (threadIdx.x == 0) ts_finish(ex, 0);
}

// ---------------------------------------------------------------- backward -------------------
template <typename S, int U, int K, int STAGES>
__global__ void __launch_bounds__((K + 1) * 32, 1)
tsplit_backward_tma_kernel(const S *__restrict__ gates, const S *__restrict__ states,
                           const S *__restrict__ grad_states, const float *__restrict__ h_in,
                           S *__restrict__ grad_gates, S *__restrict__ grad_tokens, float *__restrict__ grad_h0,
                           TsExchange ex, int64_t R, int64_t T) {
    using Ring = TsRing<S, U, K, 3, STAGES>;
    constexpr int E = Ring::E, TILE = Ring::TILE;
    constexpr int64_t SUPER = Ring::SUPER;
    extern __shared__ __align__(128) unsigned char ts_smem[];
    S *stage_base = reinterpret_cast<S *>(ts_smem);
    uint64_t *full = reinterpret_cast<uint64_t *>(ts_smem + STAGES * Ring::kStageBytes);
    uint64_t *empty = full + STAGES;
    __shared__ float2 aggs[2][kTsMaxAgg];
    __shared__ float s_carry;
    __shared__ int s_fault;
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ts_mbar_init(full + s, 1);
            ts_mbar_init(empty + s, K);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_fault = ts_wait_acks(ex, 1);
        if (s_fault)
            atomicCAS(reinterpret_cast<uint32_t *>(ex.buf[ex.rank] + ex.lay.status_offset()), 0u,
                      static_cast<uint32_t>(s_fault));
    }
    __syncthreads();
    const bool publish_ok = s_fault == 0;
    const int64_t ngroups = (T + SUPER - 1) / SUPER;
    const int64_t m = (R - blockIdx.x + gridDim.x - 1) / gridDim.x;
    const int64_t look = min(static_cast<int64_t>(ex.look), ngroups);

    if (w == K) {
        if (lane == 0) {
            unsigned n = 0;
            bool alive = true;
            const uint64_t pol_keep = ts_policy(true), pol_release = ts_policy(false);
            ts_walk(m, ngroups, look, [&](int pass, int64_t i, int64_t step) {
                if (!alive) return;
                const int s = static_cast<int>(n % STAGES);
                if (!ts_mbar_wait(empty + s, ((n / STAGES) & 1u) ^ 1u, &s_fault)) {
                    alive = false;
                    return;
                }
                const int64_t g = ngroups - 1 - step;  // time runs backwards
                const int64_t off = (blockIdx.x + i * gridDim.x) * T, e0 = g * SUPER;
                const unsigned bytes = static_cast<unsigned>(min(SUPER, T - e0) * sizeof(S));
                S *dst = stage_base + static_cast<size_t>(s) * 3 * SUPER;
                ts_mbar_expect_tx(full + s, (pass == 1 ? 3 : 2) * bytes);
                if (ex.l2_hint) {
                    const uint64_t pol = pass == 0 ? pol_keep : pol_release;
                    ts_bulk_load_hint(dst, gates + off + e0, bytes, full + s, pol);
                    ts_bulk_load_hint(dst + SUPER, grad_states + off + e0, bytes, full + s, pol);
                    if (pass == 1) ts_bulk_load_hint(dst + 2 * SUPER, states + off + e0, bytes, full + s, pol_release);
                } else {
                    ts_bulk_load(dst, gates + off + e0, bytes, full + s);
                    ts_bulk_load(dst + SUPER, grad_states + off + e0, bytes, full + s);
                    if (pass == 1) ts_bulk_load(dst + 2 * SUPER, states + off + e0, bytes, full + s);
                }
                ++n;
            });
            if (!alive) {
                ts_ring_fault(ex, &s_fault);
                for (unsigned k = n > STAGES ? n - STAGES : 0; k < n; ++k) {
                    const int s = static_cast<int>(k % STAGES);
                    for (unsigned spin = 0; spin < kTsMbarSpins && !ts_mbar_try_wait(full + s, (k / STAGES) & 1u); ++spin) {
                    }
                }
            }
        }
    } else {
        const int64_t e_lane = static_cast<int64_t>(w) * (TILE * U) + lane * E;
        unsigned n = 0;
        bool alive = true;
        float cin = 0.f, h_before = 0.f;
        ts_walk(m, ngroups, look, [&](int pass, int64_t i, int64_t step) {
            const int64_t row = blockIdx.x + i * gridDim.x, off = row * T;
            const int64_t g = ngroups - 1 - step;
            float2 *tab = aggs[i & 1];
            if (pass == 1 && step == 0) {
                if (w == 0 && alive) {
                    const float c_in = ts_wait_row(ex, 1, row, lane, &s_fault);
                    if (lane == 0) s_carry = c_in;
                }
                ts_consumer_sync(K * 32);
                cin = s_carry;
                h_before = h_in ? h_in[row] : 0.f;
            }
            const int64_t v = g * SUPER + e_lane;
            // the state just before this group sits outside the stage: one scalar from global memory,
            // asked for before the wait (only the first lane of the group's first tile)
            float group_halo = 0.f;
            if (alive && pass == 1 && w == 0 && lane == 0 && g > 0)
                group_halo = Store<S>::to_float(states[off + g * SUPER - 1]);
            if (alive) {
                const int s = static_cast<int>(n % STAGES);
                if (!ts_mbar_wait(full + s, (n / STAGES) & 1u, &s_fault)) {
                    alive = false;
                    if (lane == 0) ts_ring_fault(ex, &s_fault);
                }
            }
            if (alive) {
                const int s = static_cast<int>(n % STAGES);
                const S *sa = stage_base + static_cast<size_t>(s) * 3 * SUPER;
                const S *sg = sa + SUPER, *sh = sa + 2 * SUPER;
                uint4 ra[U], rg[U], rh[U];
                float halo[U];
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    const bool in = v + j * TILE < T;
                    ra[j] = in ? *reinterpret_cast<const uint4 *>(sa + e_lane + j * TILE)
                               : make_uint4(Store<S>::kOne, Store<S>::kOne, Store<S>::kOne, Store<S>::kOne);
                    rg[j] = in ? *reinterpret_cast<const uint4 *>(sg + e_lane + j * TILE) : make_uint4(0u, 0u, 0u, 0u);
                    rh[j] = make_uint4(0u, 0u, 0u, 0u);
                    halo[j] = 0.f;
                    if (pass == 1 && in) {
                        rh[j] = *reinterpret_cast<const uint4 *>(sh + e_lane + j * TILE);
                        if (lane == 0) {
                            const int64_t ee = e_lane + j * TILE;  // first element of this tile inside the stage
                            halo[j] = ee > 0 ? Store<S>::to_float(sh[ee - 1]) : group_halo;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) ts_mbar_arrive(empty + s);

                float fa[U][E], fg[U][E], A[U], C[U];
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    Store<S>::unpack(ra[j], fa[j]);
                    Store<S>::unpack(rg[j], fg[j]);
                    A[j] = fa[j][E - 1];
                    C[j] = fa[j][E - 1] * fg[j][E - 1];
#pragma unroll
                    for (int k = E - 2; k >= 0; --k) {
                        C[j] = fa[j][k] * (fg[j][k] + C[j]);
                        A[j] *= fa[j][k];
                    }
                }
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
                    for (int j = 0; j < U; ++j) {
                        const float pA = __shfl_down_sync(kFullMask, A[j], d);
                        const float pC = __shfl_down_sync(kFullMask, C[j], d);
                        if (lane + d < 32) {
                            C[j] = fmaf(A[j], pC, C[j]);
                            A[j] *= pA;
                        }
                    }
                }
                // walk order: super-tiles from the last one down, warps from K-1 down
                const int slot = static_cast<int>(step) * K + (K - 1 - w);
                if (pass == 0) {
                    float WA = __shfl_sync(kFullMask, A[U - 1], 0), WC = __shfl_sync(kFullMask, C[U - 1], 0);
#pragma unroll
                    for (int j = U - 2; j >= 0; --j) {
                        const float tA = __shfl_sync(kFullMask, A[j], 0);
                        WC = fmaf(tA, WC, __shfl_sync(kFullMask, C[j], 0));
                        WA *= tA;
                    }
                    if (lane == 0) tab[slot] = make_float2(WA, WC);
                } else {
                    const float2 pre = tab[slot];
                    float cw = fmaf(pre.x, cin, pre.y);  // c just after this warp's last tile
#pragma unroll
                    for (int j = U - 1; j >= 0; --j) {
                        const float tA = __shfl_sync(kFullMask, A[j], 0);
                        const float tC = __shfl_sync(kFullMask, C[j], 0);
                        float eA = __shfl_down_sync(kFullMask, A[j], 1);
                        float eC = __shfl_down_sync(kFullMask, C[j], 1);
                        if (lane == 31) {
                            eA = 1.f;
                            eC = 0.f;
                        }
                        float fh[E];
                        Store<S>::unpack(rh[j], fh);
                        float hprev0 = __shfl_up_sync(kFullMask, fh[E - 1], 1);
                        if (lane == 0) hprev0 = (v + j * TILE - 1 >= 0) ? halo[j] : h_before;
                        float c = fmaf(eA, cw, eC);
                        float dx[E], da[E];
#pragma unroll
                        for (int k = E - 1; k >= 0; --k) {
                            const float delta = fg[j][k] + c;
                            c = fa[j][k] * delta;
                            const float hp = (k > 0) ? fh[k > 0 ? k - 1 : 0] : hprev0;
                            dx[k] = delta;
                            da[k] = delta * hp;
                        }
                        store_vec<S, false>(grad_tokens + off, v + j * TILE, T, true, Store<S>::pack(dx));
                        store_vec<S, false>(grad_gates + off, v + j * TILE, T, true, Store<S>::pack(da));
                        cw = fmaf(tA, cw, tC);
                    }
                    // the warp that owns the block's first tile ends with c at the block start
                    if (grad_h0 && g == 0 && w == 0 && lane == 0) grad_h0[row] = cw;
                }
            }
            ++n;
            if (pass == 0 && step == ngroups - 1) {
                ts_consumer_sync(K * 32);
                if (w == 0 && alive) {
                    const float2 total = ts_scan_aggregates(tab, static_cast<int>(ngroups) * K, lane);
                    ts_publish_row(ex, 1, row, total.x, total.y, publish_ok, lane);
                }
            }
        });
    }
    __syncthreads();
    if (threadIdx.x == 0) ts_finish(ex, 1);
}

}  // namespace fms
