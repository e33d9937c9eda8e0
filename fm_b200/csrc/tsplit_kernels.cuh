// Split-along-T scan as ONE kernel per direction: carry pass, carry exchange over peer memory and
// scan pass fused, row by row.
//
// Rank k of `world` owns time block k of every row.  The three-launch scheme (carry pass over the
// whole block -> exchange -> scan pass over the whole block) reads gates and tokens twice from
// HBM.  Here a CTA of K warps takes ONE row at a time and runs
//     pass A  carries of the row's block, (P, S) = (prod a, state from a zero start)   reads a, x
//     publish (P, S) into the buffers of the ranks that scan later blocks (one 16-byte peer store
//             per row and peer, value and exchange number together), then
//     wait    (bounded, polling LOCAL memory) for the (P, S) of the earlier blocks and fold them
//     pass B  the ordinary scan of the block from the true carry-in          re-reads a, x; writes h
// so that a row's operands are read again a few microseconds after they were first read, while
// they are still in the 126 MB L2: per element the block costs 2 reads + 1 write of HBM traffic
// forward (3 + 2 backward: the states are read once), the same as an unsplit scan.  The peer
// latency of one row hides behind the other CTAs of the SM and the loads of pass B that are already
// in flight.  The backward kernel mirrors this in reverse time order with c_t = a_t * delta_t as
// the carried quantity (see scan_kernels.cuh).
//
// Peer traffic is plain stores into the peers' buffers and local loads: no multicast, no multimem,
// no remote loads.  Every wait is bounded by a clock; a wait that runs out records a fault in the
// local status word, the CTA stops waiting (carry-in 0 from then on) and the kernel still ends.
//
// Exchange buffer of a rank (all ranks map all buffers), e = exchange number, two slot generations:
//   slots [2 parity][2 direction][world src][rows]  16 bytes {P, e, S, e}
//   acks  [2 direction][world consumer]             uint32: last exchange that rank finished
//   done  [2 direction]                             uint32: CTAs of the running kernel that ended
//   status                                          uint32: 0, or the first fault
// A kernel of exchange e starts by waiting until the ranks that read its slots have acknowledged
// e-2 (same generation), and ends by acknowledging e to every rank.
#pragma once

#include "fm_scan_b200.h"
#include "scan_kernels.cuh"

namespace fms {

struct TsLayout {
    int64_t rows;
    int world;
    __host__ __device__ size_t slot_index(int parity, int dir, int src, int64_t row) const {
        return ((static_cast<size_t>(parity) * 2 + dir) * world + src) * static_cast<size_t>(rows) + row;
    }
    __host__ __device__ size_t slots_bytes() const { return static_cast<size_t>(4) * world * rows * 16; }
    __host__ __device__ size_t acks_offset() const { return (slots_bytes() + 255) / 256 * 256; }
    __host__ __device__ size_t done_offset() const { return acks_offset() + static_cast<size_t>(2) * world * 4; }
    __host__ __device__ size_t status_offset() const { return done_offset() + 8; }
    __host__ __device__ size_t total_bytes() const { return (status_offset() + 4 + 255) / 256 * 256; }
};

struct TsExchange {
    char *buf[FMS_MAX_PEERS];  // every rank's buffer as mapped here; buf[rank] is local
    TsLayout lay;
    int rank;
    uint32_t epoch;
    long long max_wait_cycles;
    int l2_hint;  // staged kernels: first pass evict-last, second pass evict-first
    int look;     // staged kernels: super-tiles of the NEXT row's first pass run before a row's second pass
};

__device__ __forceinline__ void st_slot(void *p, float P, float S, uint32_t e) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(__float_as_uint(P)), "r"(e),
                 "r"(__float_as_uint(S)), "r"(e)
                 : "memory");
}

__device__ __forceinline__ uint4 ld_slot(const void *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

// Kernel prologue, thread 0 of every CTA: the slot generation of this exchange was last used by
// exchange epoch-2; wait until its readers are done with it.  Returns a fault code or 0.
__device__ __forceinline__ int ts_wait_acks(const TsExchange &ex, int dir) {
    if (ex.epoch <= 2u) return 0;
    volatile uint32_t *acks = reinterpret_cast<volatile uint32_t *>(ex.buf[ex.rank] + ex.lay.acks_offset());
    const int first = dir == 0 ? ex.rank + 1 : 0, last = dir == 0 ? ex.lay.world : ex.rank;
    const long long start = clock64();
    for (int c = first; c < last; ++c) {
        while (static_cast<int32_t>(acks[dir * ex.lay.world + c] - (ex.epoch - 2u)) < 0) {
            if (clock64() - start > ex.max_wait_cycles) return FMS_PEER_ERR_ACK_TIMEOUT;
            __nanosleep(200);
        }
    }
    return 0;
}

// Kernel epilogue, thread 0 of every CTA: the last CTA to finish acknowledges the exchange to every
// rank -- unless a fault was recorded, in which case the publishers stop at their own bounded wait.
__device__ __forceinline__ void ts_finish(const TsExchange &ex, int dir) {
    char *local = ex.buf[ex.rank];
    uint32_t *done = reinterpret_cast<uint32_t *>(local + ex.lay.done_offset()) + dir;
    __threadfence();
    if (atomicAdd(done, 1u) == gridDim.x - 1) {
        __threadfence();
        *done = 0;
        if (*reinterpret_cast<volatile uint32_t *>(local + ex.lay.status_offset()) == 0u) {
            for (int p = 0; p < ex.lay.world; ++p)
                reinterpret_cast<volatile uint32_t *>(ex.buf[p] + ex.lay.acks_offset())[dir * ex.lay.world + ex.rank] =
                    ex.epoch;
        }
    }
}

// Warp 0 of a CTA, after pass A of `row`: store this block's (P, S) into the buffers of the ranks
// that need it (one lane per peer).  `publish` is false after an acknowledgement timeout (the
// slots may still be in use).
__device__ __forceinline__ void ts_publish_row(const TsExchange &ex, int dir, int64_t row, float P, float S,
                                               bool publish, int lane) {
    const int world = ex.lay.world, rank = ex.rank;
    const int parity = static_cast<int>(ex.epoch & 1u);
    // forward: later blocks read this one; backward: earlier blocks do
    const bool is_reader = dir == 0 ? (lane > rank && lane < world) : (lane < rank);
    if (is_reader && publish)
        st_slot(ex.buf[lane] + ex.lay.slot_index(parity, dir, rank, row) * 16, P, S, ex.epoch);
}

// Warp 0 of a CTA, before pass B of `row`: wait (bounded, local polls) for the blocks this rank
// needs and fold them in scan order.  Returns the carry entering this rank's block (every lane).
// `fault` is the CTA's sticky fault flag: once set, nothing waits and the carry is 0.
__device__ __forceinline__ float ts_wait_row(const TsExchange &ex, int dir, int64_t row, int lane,
                                             volatile int *fault) {
    const int world = ex.lay.world, rank = ex.rank;
    const int parity = static_cast<int>(ex.epoch & 1u);
    const bool is_source = dir == 0 ? (lane < rank) : (lane > rank && lane < world);
    float Pq = 1.f, Sq = 0.f;
    bool ok = !is_source;
    if (!*fault) {
        const char *slot = ex.buf[rank] + ex.lay.slot_index(parity, dir, is_source ? lane : 0, row) * 16;
        const long long start = clock64();
        int code = 0;
        for (;;) {
            if (!ok) {
                const uint4 s = ld_slot(slot);
                if (s.y == ex.epoch && s.w == ex.epoch) {
                    Pq = __uint_as_float(s.x);
                    Sq = __uint_as_float(s.z);
                    ok = true;
                } else if (static_cast<int32_t>(s.y - ex.epoch) > 0 && s.y == s.w) {
                    code = FMS_PEER_ERR_OVERRUN;  // a later exchange already sits in the slot
                }
            }
            if (__all_sync(kFullMask, ok)) break;
            if (clock64() - start > ex.max_wait_cycles)
                code = dir == 0 ? FMS_PEER_ERR_WAIT_TIMEOUT : FMS_PEER_ERR_WAIT_TIMEOUT_REVERSE;
            code = __reduce_max_sync(kFullMask, code);
            if (code) {
                if (lane == 0) {
                    *fault = code;
                    atomicCAS(reinterpret_cast<uint32_t *>(ex.buf[rank] + ex.lay.status_offset()), 0u,
                              static_cast<uint32_t>(code));
                }
                break;
            }
            __nanosleep(100);
        }
    }
    const bool good = __all_sync(kFullMask, ok);
    float c = 0.f;
    if (good) {
        if (dir == 0) {
            for (int q = 0; q < rank; ++q)
                c = fmaf(__shfl_sync(kFullMask, Pq, q), c, __shfl_sync(kFullMask, Sq, q));
        } else {
            for (int q = world - 1; q > rank; --q)
                c = fmaf(__shfl_sync(kFullMask, Pq, q), c, __shfl_sync(kFullMask, Sq, q));
        }
    }
    return c;
}

// Publish, then wait and fold (the register-prefetch kernels do both at the same point).
__device__ __forceinline__ float ts_exchange_row(const TsExchange &ex, int dir, int64_t row, float P, float S,
                                                 bool publish, int lane, volatile int *fault) {
    ts_publish_row(ex, dir, row, P, S, publish, lane);
    return ts_wait_row(ex, dir, row, lane, fault);
}

// ---------------------------------------------------------------- forward --------------------
// gates, tokens, states: (R, T) of this rank's block, rows 16-byte aligned.  h0 (rank 0 only,
// nullable): the state before the first block.  h_in_out (R) receives the carry that entered this
// block (the backward needs it as h_{t-1} of the block's first position).
template <typename S, int U, int K>
__global__ void __launch_bounds__(K * 32)
tsplit_forward_kernel(const S *__restrict__ gates, const S *__restrict__ tokens, const float *__restrict__ h0,
                      S *__restrict__ states, float *__restrict__ h_in_out, TsExchange ex, int64_t R, int64_t T) {
    constexpr int E = Store<S>::E;
    constexpr int TILE = 32 * E;
    constexpr int64_t SUPER = static_cast<int64_t>(TILE) * U * K;
    __shared__ float2 agg[2][K];
    __shared__ float s_carry;
    __shared__ int s_fault;
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        s_fault = ts_wait_acks(ex, 0);
        if (s_fault)
            atomicCAS(reinterpret_cast<uint32_t *>(ex.buf[ex.rank] + ex.lay.status_offset()), 0u,
                      static_cast<uint32_t>(s_fault));
    }
    __syncthreads();
    const bool publish_ok = s_fault == 0;  // after an ack timeout the slots may still be in use

    const int64_t ngroups = (T + SUPER - 1) / SUPER;
    const int64_t v0 = static_cast<int64_t>(w) * (TILE * U) + lane * E;
    int64_t row = blockIdx.x;  // the grid never exceeds R
    int pass = 0;
    float carry = 0.f, prod = 1.f;
    int64_t off = row * T, v = v0, g = 0;
    uint4 ra[U], rx[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        ra[j] = load_vec<S, false>(gates + off, v + j * TILE, T, true, Store<S>::kOne);
        rx[j] = load_vec<S, false>(tokens + off, v + j * TILE, T, true, 0u);
    }
    for (unsigned it = 0;; ++it) {
        const bool last_group = (g + 1 == ngroups);
        int64_t noff = off, nv = v + SUPER;
        bool more = true;
        if (last_group) {
            if (pass == 0) {
                nv = v0;  // pass B of the same row: these loads hit L2
            } else if (row + gridDim.x < R) {
                noff = (row + gridDim.x) * T;
                nv = v0;
            } else {
                more = false;
                nv = T;  // outside: identity, no memory access
            }
        }
        uint4 na[U], nx[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            na[j] = load_vec<S, false>(gates + noff, nv + j * TILE, T, true, Store<S>::kOne);
            nx[j] = load_vec<S, false>(tokens + noff, nv + j * TILE, T, true, 0u);
        }
        float fa[U][E], fx[U][E], A[U], H[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            Store<S>::unpack(ra[j], fa[j]);
            Store<S>::unpack(rx[j], fx[j]);
            A[j] = fa[j][0];
            H[j] = fx[j][0];
#pragma unroll
            for (int i = 1; i < E; ++i) {
                H[j] = fmaf(fa[j][i], H[j], fx[j][i]);
                A[j] *= fa[j][i];
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
        float WA = __shfl_sync(kFullMask, A[0], 31), WH = __shfl_sync(kFullMask, H[0], 31);
#pragma unroll
        for (int j = 1; j < U; ++j) {
            const float tA = __shfl_sync(kFullMask, A[j], 31);
            WH = fmaf(tA, WH, __shfl_sync(kFullMask, H[j], 31));
            WA *= tA;
        }
        const int buf = static_cast<int>(it & 1u);
        if (lane == 0) agg[buf][w] = make_float2(WA, WH);
        __syncthreads();
        float run = carry, mine = carry;
#pragma unroll
        for (int ww = 0; ww < K; ++ww) {
            if (ww == w) mine = run;
            const float2 p = agg[buf][ww];
            run = fmaf(p.x, run, p.y);
            prod *= p.x;
        }
        if (pass == 1) {
            float c = mine;
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
                float s = fmaf(eA, c, eH);
                float out[E];
#pragma unroll
                for (int i = 0; i < E; ++i) {
                    s = fmaf(fa[j][i], s, fx[j][i]);
                    out[i] = s;
                }
                store_vec<S, false>(states + off, v + j * TILE, T, true, Store<S>::pack(out));
                c = fmaf(tA, c, tH);
            }
        }
        carry = run;

        if (last_group) {
            if (pass == 0) {
                // (prod, carry) = (P, S) of this row's block, identical in every thread
                if (w == 0) {
                    float S_pub = carry, h_first = 0.f;
                    if (ex.rank == 0 && h0) {  // the first block folds the initial state into what it publishes
                        h_first = h0[row];
                        S_pub = fmaf(prod, h_first, carry);
                    }
                    float hin = ts_exchange_row(ex, 0, row, prod, S_pub, publish_ok, lane, &s_fault);
                    if (ex.rank == 0) hin = h_first;
                    if (lane == 0) {
                        s_carry = hin;
                        h_in_out[row] = hin;
                    }
                }
                __syncthreads();
                carry = s_carry;
                prod = 1.f;
                pass = 1;
                g = 0;
            } else {
                if (!more) break;
                row += gridDim.x;
                carry = 0.f;
                prod = 1.f;
                pass = 0;
                g = 0;
            }
        } else {
            ++g;
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            ra[j] = na[j];
            rx[j] = nx[j];
        }
        off = noff;
        v = nv;
    }
    __syncthreads();
    if (threadIdx.x == 0) ts_finish(ex, 0);
}

// ---------------------------------------------------------------- backward -------------------
// Reverse scan of c_t = a_t * (G_t + c_{t+1}); grad_tokens = delta, grad_gates = delta * h_{t-1}.
// h_in (R): the carry that entered this block in forward (h_{t-1} of the block's first position).
// grad_h0 (rank 0 only, nullable) receives c at the block start = dL/d(initial state).
template <typename S, int U, int K>
__global__ void __launch_bounds__(K * 32)
tsplit_backward_kernel(const S *__restrict__ gates, const S *__restrict__ states, const S *__restrict__ grad_states,
                       const float *__restrict__ h_in, S *__restrict__ grad_gates, S *__restrict__ grad_tokens,
                       float *__restrict__ grad_h0, TsExchange ex, int64_t R, int64_t T) {
    constexpr int E = Store<S>::E;
    constexpr int TILE = 32 * E;
    constexpr int64_t SUPER = static_cast<int64_t>(TILE) * U * K;
    __shared__ float2 agg[2][K];
    __shared__ float s_carry;
    __shared__ int s_fault;
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        s_fault = ts_wait_acks(ex, 1);
        if (s_fault)
            atomicCAS(reinterpret_cast<uint32_t *>(ex.buf[ex.rank] + ex.lay.status_offset()), 0u,
                      static_cast<uint32_t>(s_fault));
    }
    __syncthreads();
    const bool publish_ok = s_fault == 0;

    const int64_t ngroups = (T + SUPER - 1) / SUPER;
    const int64_t v_last = (ngroups - 1) * SUPER + static_cast<int64_t>(w) * (TILE * U) + lane * E;
    int64_t row = blockIdx.x;
    int pass = 0;
    float carry = 0.f, prod = 1.f;
    int64_t off = row * T, v = v_last, g = ngroups - 1;

    auto load_halo = [&](int64_t o, int64_t vt) -> float {
        if (lane != 0) return 0.f;
        const int64_t t = vt - 1;
        return (t >= 0 && t < T) ? Store<S>::to_float(states[o + t]) : 0.f;
    };

    uint4 ra[U], rg[U], rh[U];
    float halo[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        ra[j] = load_vec<S, false>(gates + off, v + j * TILE, T, true, Store<S>::kOne);
        rg[j] = load_vec<S, false>(grad_states + off, v + j * TILE, T, true, 0u);
        rh[j] = make_uint4(0u, 0u, 0u, 0u);
        halo[j] = 0.f;
    }
    float h_before = 0.f;
    for (unsigned it = 0;; ++it) {
        const bool last_group = (g == 0);
        int64_t noff = off, nv = v - SUPER;
        bool more = true;
        int npass = pass;
        if (last_group) {
            if (pass == 0) {
                nv = v_last;  // pass B of the same row: a and G hit L2, the states come from HBM
                npass = 1;
            } else if (row + gridDim.x < R) {
                noff = (row + gridDim.x) * T;
                nv = v_last;
                npass = 0;
            } else {
                more = false;
            }
        }
        uint4 na[U], ng[U], nh[U];
        float nhalo[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int64_t vv = more ? nv + j * TILE : T;
            na[j] = load_vec<S, false>(gates + noff, vv, T, true, Store<S>::kOne);
            ng[j] = load_vec<S, false>(grad_states + noff, vv, T, true, 0u);
            if (npass == 1 && more) {
                nh[j] = load_vec<S, false>(states + noff, vv, T, true, 0u);
                nhalo[j] = load_halo(noff, vv);
            } else {
                nh[j] = make_uint4(0u, 0u, 0u, 0u);
                nhalo[j] = 0.f;
            }
        }
        float fa[U][E], fg[U][E], A[U], C[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            Store<S>::unpack(ra[j], fa[j]);
            Store<S>::unpack(rg[j], fg[j]);
            A[j] = fa[j][E - 1];
            C[j] = fa[j][E - 1] * fg[j][E - 1];
#pragma unroll
            for (int i = E - 2; i >= 0; --i) {
                C[j] = fa[j][i] * (fg[j][i] + C[j]);
                A[j] *= fa[j][i];
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
        float WA = __shfl_sync(kFullMask, A[U - 1], 0), WC = __shfl_sync(kFullMask, C[U - 1], 0);
#pragma unroll
        for (int j = U - 2; j >= 0; --j) {
            const float tA = __shfl_sync(kFullMask, A[j], 0);
            WC = fmaf(tA, WC, __shfl_sync(kFullMask, C[j], 0));
            WA *= tA;
        }
        const int buf = static_cast<int>(it & 1u);
        if (lane == 0) agg[buf][w] = make_float2(WA, WC);
        __syncthreads();
        float run = carry, mine = carry;
#pragma unroll
        for (int ww = K - 1; ww >= 0; --ww) {
            if (ww == w) mine = run;
            const float2 p = agg[buf][ww];
            run = fmaf(p.x, run, p.y);
            prod *= p.x;
        }
        if (pass == 1) {
            float cw = mine;
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
                for (int i = E - 1; i >= 0; --i) {
                    const float delta = fg[j][i] + c;
                    c = fa[j][i] * delta;
                    const float hp = (i > 0) ? fh[i > 0 ? i - 1 : 0] : hprev0;
                    dx[i] = delta;
                    da[i] = delta * hp;
                }
                store_vec<S, false>(grad_tokens + off, v + j * TILE, T, true, Store<S>::pack(dx));
                store_vec<S, false>(grad_gates + off, v + j * TILE, T, true, Store<S>::pack(da));
                cw = fmaf(tA, cw, tC);
            }
        }
        carry = run;

        if (last_group) {
            if (pass == 0) {
                if (w == 0) {
                    const float cin = ts_exchange_row(ex, 1, row, prod, carry, publish_ok, lane, &s_fault);
                    if (lane == 0) s_carry = cin;
                }
                __syncthreads();
                carry = s_carry;
                prod = 1.f;
                h_before = h_in ? h_in[row] : 0.f;
                pass = 1;
                g = ngroups - 1;
            } else {
                if (grad_h0 && threadIdx.x == 0) grad_h0[row] = carry;
                if (!more) break;
                row += gridDim.x;
                carry = 0.f;
                prod = 1.f;
                pass = 0;
                g = ngroups - 1;
            }
        } else {
            --g;
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            ra[j] = na[j];
            rg[j] = ng[j];
            rh[j] = nh[j];
            halo[j] = nhalo[j];
        }
        off = noff;
        v = nv;
    }
    __syncthreads();
    if (threadIdx.x == 0) ts_finish(ex, 1);
}

}  // namespace fms
