// Device code of the B200 scan: forward, backward and carry-only (reduce) kernels.
//
// Work decomposition
//   K warps own one scan unit (a row, or a segment of a row) and walk it along time in
//   super-tiles of K*U tiles.  A tile is 32 lanes x one 16-byte vector (E = 4 fp32 or 8 fp16/bf16
//   elements per lane), i.e. 512 contiguous bytes per tensor per warp instruction, so every
//   global access is a fully coalesced 128-bit access and a CTA reads K*U*512 contiguous bytes
//   per tensor per step.  The loads of step g+1 are issued into registers before step g is
//   computed, which keeps U x (number of input tensors) x 512 B in flight per warp across the
//   serial carry.  K == 1 packs four independent units into a CTA and uses no block barrier;
//   K > 1 exchanges the warps' aggregates through double-buffered shared memory with one
//   __syncthreads per super-tile.
//
//   Inside a tile: each lane scans its E elements sequentially to an aggregate pair
//   (A, H) = (prod a, state from a zero start); the 32 pairs are combined with a 5-step
//   warp-shuffle scan under the associative operator
//        (A2, H2) o (A1, H1) = (A2*A1, A2*H1 + H2)          ("1" earlier in time than "2");
//   the lane's carry-in follows from the exclusive prefix and the running carry, and the lane
//   re-runs its E elements sequentially from that carry-in to produce the outputs.  Only
//   multiply-add pairs are used, so gates that are exactly 0 or 1 need no special case.
//
//   Backward uses the substitution c_t = a_t * delta_t (delta_t = G_t + c_{t+1}), which turns the
//   "reverse scan with the gate shifted by one" (fm/scan/fm_scan.cuh:86-88,103-108) into a
//   reverse scan with UNSHIFTED gates and tokens a_t*G_t: every vector load stays aligned, and
//   the only halo is the single state h_{t-1} before a tile (one scalar load by lane 0).
//
// Rows whose start is not 16-byte aligned (odd T with 2-byte elements, sliced views) use the
// GENERIC instantiation: tiles are laid on the 16-byte grid of the gates row, vectors that
// straddle a row end or belong to a tensor with a different phase are read/written element by
// element under a mask, and masked positions carry the identity (a = 1, x = 0).
//
// Other template flags: WRITE (false = carries only), SEG (units are segments of rows: the split
// path for few long rows), FM (the reference's (B,M,L) x (B,D,L) -> (B,M,D,L) operator with the
// 1 - gate token weight; its blocked variants live in fm_kernels.cuh).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fms {

#ifndef FMS_WARPS_PER_CTA
#define FMS_WARPS_PER_CTA 4
#endif
constexpr int kWarpsPerCta = FMS_WARPS_PER_CTA;
constexpr unsigned kFullMask = 0xffffffffu;

// ---------------------------------------------------------------- storage <-> fp32 ----------
// Mirrors the role of cast_to_float / cast_from_float (fm/scan/fm_scan.cuh:14-40): all
// arithmetic is fp32, storage is fp32 / fp16 / bf16 with round-to-nearest-even on the way out.
template <typename S>
struct Store;

template <>
struct Store<float> {
    static constexpr int E = 4;
    static constexpr uint32_t kOne = 0x3f800000u;
    static __device__ __forceinline__ void unpack(const uint4 &v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
    static __device__ __forceinline__ uint4 pack(const float (&f)[4]) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                          __float_as_uint(f[3]));
    }
    static __device__ __forceinline__ float to_float(float s) { return s; }
};

template <>
struct Store<__nv_bfloat16> {
    static constexpr int E = 8;
    static constexpr uint32_t kOne = 0x3f803f80u;
    static __device__ __forceinline__ void unpack(const uint4 &v, float (&f)[8]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            f[2 * k] = __uint_as_float(w[k] << 16);
            f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
            w[k] = *reinterpret_cast<uint32_t *>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ float to_float(__nv_bfloat16 s) { return __bfloat162float(s); }
};

template <>
struct Store<__half> {
    static constexpr int E = 8;
    static constexpr uint32_t kOne = 0x3c003c00u;
    static __device__ __forceinline__ void unpack(const uint4 &v, float (&f)[8]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
            f[2 * k] = p.x;
            f[2 * k + 1] = p.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            __half2 p = __floats2half2_rn(f[2 * k], f[2 * k + 1]);
            w[k] = *reinterpret_cast<uint32_t *>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ float to_float(__half s) { return __half2float(s); }
};

// ---------------------------------------------------------------- global memory access ------
// Streaming 128-bit accesses: every byte is touched once per kernel, so loads bypass L1
// allocation and stores are marked evict-first.
__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void stg_stream(void *p, const uint4 &v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

// The same store under an L2 eviction policy chosen at run time (one instruction either way, no
// branch): evict-first for write-once streams, evict-normal / evict-last for data the NEXT kernel
// reads back soon (the states a forward writes and the backward of the same step re-reads, latest
// rows first).  mode: 0 evict-first, 1 evict-normal, 2 evict-last.
__device__ __forceinline__ uint64_t make_store_policy(int mode) {
    uint64_t pol;
    if (mode == 2) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    else if (mode == 1) asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
    else asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void stg_policy(void *p, const uint4 &v, uint64_t pol) {
    asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w), "l"(pol)
                 : "memory");
}

// One lane's vector of a row: positions [v, v+E).  `fill` is the 32-bit pattern returned for
// positions outside [0, T) (packed ones for gates, zero otherwise).  In the aligned
// instantiation a vector is either wholly inside the row or wholly outside it.
template <typename S, bool GENERIC>
__device__ __forceinline__ uint4 load_vec(const S *__restrict__ row, int64_t v, int64_t T,
                                          bool same_phase, uint32_t fill) {
    constexpr int E = Store<S>::E;
    if constexpr (!GENERIC) {
        if (v < T) return ldg_stream(row + v);
        return make_uint4(fill, fill, fill, fill);
    } else {
        if (same_phase && v >= 0 && v + E <= T) return ldg_stream(row + v);
        union {
            uint4 q;
            S s[E];
        } u;
        u.q = make_uint4(fill, fill, fill, fill);
#pragma unroll
        for (int i = 0; i < E; ++i) {
            const int64_t t = v + i;
            if (t >= 0 && t < T) u.s[i] = row[t];
        }
        return u.q;
    }
}

template <typename S, bool GENERIC>
__device__ __forceinline__ void store_vec(S *__restrict__ row, int64_t v, int64_t T,
                                          bool same_phase, const uint4 &q) {
    constexpr int E = Store<S>::E;
    if constexpr (!GENERIC) {
        if (v < T) stg_stream(row + v, q);
    } else {
        if (same_phase && v >= 0 && v + E <= T) {
            stg_stream(row + v, q);
            return;
        }
        union {
            uint4 q;
            S s[E];
        } u;
        u.q = q;
#pragma unroll
        for (int i = 0; i < E; ++i) {
            const int64_t t = v + i;
            if (t >= 0 && t < T) row[t] = u.s[i];
        }
    }
}

// store_vec whose full-vector stores carry an L2 eviction policy (make_store_policy).
template <typename S, bool GENERIC>
__device__ __forceinline__ void store_vec_policy(S *__restrict__ row, int64_t v, int64_t T, bool same_phase,
                                                 const uint4 &q, uint64_t pol) {
    if constexpr (!GENERIC) {
        if (v < T) stg_policy(row + v, q, pol);
    } else {
        store_vec<S, GENERIC>(row, v, T, same_phase, q);
    }
}

// Accumulate one lane's E fp32 values into an fp32 buffer (FM-mode gradient reductions): vector
// reductions (red.global.add.v4.f32) when the vector is wholly inside the row and 16-byte
// aligned, scalar atomics under the mask otherwise.
template <int E, bool GENERIC>
__device__ __forceinline__ void red_vec(float *__restrict__ row, int64_t v, int64_t T, const float (&f)[E]) {
    bool whole = (v >= 0) && (v + E <= T);
    if constexpr (GENERIC) whole = whole && ((reinterpret_cast<uintptr_t>(row + v) & 15u) == 0);
    if (whole) {
#pragma unroll
        for (int k = 0; k < E; k += 4)
            asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(row + v + k), "f"(f[k]),
                         "f"(f[k + 1]), "f"(f[k + 2]), "f"(f[k + 3])
                         : "memory");
    } else if constexpr (GENERIC) {
#pragma unroll
        for (int i = 0; i < E; ++i) {
            const int64_t t = v + i;
            if (t >= 0 && t < T) atomicAdd(row + t, f[i]);
        }
    }
}

// Row geometry shared by all kernels: where the first (virtual) vector of the row starts and
// how many groups of U tiles cover it.
template <typename S, bool GENERIC>
__device__ __forceinline__ int64_t row_phase(const S *row) {
    if constexpr (GENERIC)
        return -static_cast<int64_t>((reinterpret_cast<uintptr_t>(row) & 15u) / sizeof(S));
    else
        return 0;
}

__device__ __forceinline__ bool same_phase16(const void *p, const void *q) {
    return ((reinterpret_cast<uintptr_t>(p) ^ reinterpret_cast<uintptr_t>(q)) & 15u) == 0;
}

// ---------------------------------------------------------------- row geometry ------------
// A launch covers `R` scan units.  A unit is a whole row (SEG = false) or one of `nseg` consecutive
// segments of `seg_len` positions of a row (SEG = true: the split path for few, long rows);
// carries are indexed by unit.  K warps cooperate on one unit: K == 1 packs kWarpsPerCta independent units
// into a CTA (no block barrier at all); K > 1 gives a CTA of K warps per unit, which walk
// "super-tiles" of K*U tiles and exchange their aggregates through shared memory with one
// __syncthreads per super-tile (double-buffered slots).
struct Unit {
    int64_t offset;  // element offset of the unit's first position
    int64_t len;     // number of positions
    bool first;      // unit starts at t = 0 of its row
};

template <bool SEG>
__device__ __forceinline__ Unit unit_of(int64_t u, int64_t T, int64_t nseg, int64_t seg_len) {
    Unit q;
    if constexpr (!SEG) {
        q.offset = u * T;
        q.len = T;
        q.first = true;
    } else {
        const int64_t r = u / nseg, k = u - r * nseg;
        q.offset = r * T + k * seg_len;
        q.len = min(seg_len, T - k * seg_len);
        q.first = (k == 0);
    }
    return q;
}

template <int K>
struct Coop {
    static constexpr int kThreads = (K == 1 ? kWarpsPerCta : K) * 32;
    // Index of the first unit this warp (K == 1) or CTA (K > 1) works on, and the distance to
    // its next one when the grid is smaller than the number of units.
    static __device__ __forceinline__ int64_t first_unit() {
        return K == 1 ? static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5)
                      : static_cast<int64_t>(blockIdx.x);
    }
    static __device__ __forceinline__ int64_t unit_stride() {
        return K == 1 ? static_cast<int64_t>(gridDim.x) * kWarpsPerCta : static_cast<int64_t>(gridDim.x);
    }
    static __device__ __forceinline__ int warp_in_unit() { return K == 1 ? 0 : (threadIdx.x >> 5); }
};

// ---------------------------------------------------------------- forward / reduce ----------
// WRITE = true : states (and optionally h_last) are produced            -> fms_plain_forward
// WRITE = false: only the carries P = prod a and S = h_last are produced -> fms_plain_reduce
//
// Aligned whole-row launches (!GENERIC && !SEG) are persistent: the grid is sized to what the
// GPU holds at once, each warp (or CTA) walks units first, first+stride, ... and the prefetch
// at the last group of a unit already fetches the first group of the next one, so the load
// pipeline never drains at a row boundary.  The masked and the segmented instantiations get one
// unit per warp/CTA (their geometry changes from unit to unit).
//
// FM = true is the reference's literal operator (fm/scan/fm_pytorch.py:19-42): unit (b,m,d) reads
// gate row (b,m) and token row (b,d), the token is weighted by 1 - gate as it is unpacked
// (fm/scan/fm_scan.cuh:116), and the state row (b,m,d) is written.  The gate and token rows are
// re-read D and M times, from L2.
template <typename S, bool GENERIC, int U, bool WRITE, int K, bool SEG, bool FM>
__global__ void __launch_bounds__(Coop<K>::kThreads)
plain_forward_kernel(const S *__restrict__ gates, const S *__restrict__ tokens,
                     const float *__restrict__ h0, S *__restrict__ states,
                     float *__restrict__ h_last, float *__restrict__ P_out, int64_t R, int64_t T,
                     int64_t nseg, int64_t seg_len, int64_t M, int64_t D, int keep_states) {
    static_assert(!(FM && SEG), "FM mode has no segmented variant");
    constexpr int E = Store<S>::E;
    constexpr int TILE = 32 * E;
    constexpr bool PERSIST = !GENERIC && !SEG && !FM;
    constexpr int64_t SUPER = static_cast<int64_t>(TILE) * U * K;
    __shared__ float2 agg[2][K > 1 ? K : 1];
    const int lane = threadIdx.x & 31;
    const int w = Coop<K>::warp_in_unit();
    int64_t unit = Coop<K>::first_unit();
    if (unit >= R) return;  // K == 1 only: with K > 1 the grid never exceeds R CTAs
    const int64_t stride = Coop<K>::unit_stride();

    const Unit q = unit_of<SEG>(unit, T, nseg, seg_len);
    const int64_t L = q.len;  // PERSIST: every unit has length T
    int64_t off = q.offset;   // element offset of the current unit (states; also gates/tokens unless FM)
    int64_t goff_fm = 0, toff_fm = 0;
    if constexpr (FM) {
        const int64_t bm = unit / D, d = unit - bm * D, b = bm / M;
        goff_fm = bm * T;
        toff_fm = (b * D + d) * T;
    }
#define FMS_GOFF (FM ? goff_fm : off)
#define FMS_TOFF (FM ? toff_fm : off)
    const int64_t vbase = row_phase<S, GENERIC>(gates + FMS_GOFF);
    const bool ph_x = !GENERIC || same_phase16(gates + FMS_GOFF, tokens + FMS_TOFF);
    const bool ph_h = !GENERIC || !WRITE || same_phase16(gates + FMS_GOFF, states + off);
    const int64_t ngroups = (L - vbase + SUPER - 1) / SUPER;
    const int64_t v0 = vbase + static_cast<int64_t>(w) * (TILE * U) + lane * E;

    float carry = h0 ? h0[unit] : 0.f;  // state entering the current super-tile
    float prod = 1.f;                   // product of the unit's gates so far (reduce only)
    uint64_t store_pol = 0;
    if constexpr (WRITE && !GENERIC) store_pol = make_store_policy(keep_states);

    int64_t v = v0;  // this lane's first vector of the current group, relative to the unit
    int64_t g = 0;
    uint4 ra[U], rx[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        ra[j] = load_vec<S, GENERIC>(gates + FMS_GOFF, v + j * TILE, L, true, Store<S>::kOne);
        rx[j] = load_vec<S, GENERIC>(tokens + FMS_TOFF, v + j * TILE, L, ph_x, 0u);
    }

    for (unsigned it = 0;; ++it) {
        // Where the next group lives: same unit, or the first group of this warp's next unit.
        const bool last_group = (g + 1 == ngroups);
        int64_t noff = off, nv = v + SUPER;
        bool more = true;
        if (last_group) {
            if (PERSIST && unit + stride < R) {
                noff = (unit + stride) * T;
                nv = v0;
            } else {
                more = false;
                nv = L;  // "outside": the prefetch below returns the identity, no memory access
            }
        }
        uint4 na[U], nx[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            na[j] = load_vec<S, GENERIC>(gates + (FM ? goff_fm : noff), nv + j * TILE, L, true, Store<S>::kOne);
            nx[j] = load_vec<S, GENERIC>(tokens + (FM ? toff_fm : noff), nv + j * TILE, L, ph_x, 0u);
        }

        float fa[U][E], fx[U][E], A[U], H[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            Store<S>::unpack(ra[j], fa[j]);
            Store<S>::unpack(rx[j], fx[j]);
            if constexpr (FM) {
#pragma unroll
                for (int i = 0; i < E; ++i) fx[j][i] = (1.f - fa[j][i]) * fx[j][i];
            }
            A[j] = fa[j][0];
            H[j] = fx[j][0];
#pragma unroll
            for (int i = 1; i < E; ++i) {
                H[j] = fmaf(fa[j][i], H[j], fx[j][i]);
                A[j] *= fa[j][i];
            }
        }
        // Inclusive warp scan of the U independent tiles (interleaved for ILP).
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
        float next_carry = 0.f;
        if constexpr (K > 1) {
            // Publish this warp's aggregate over its U tiles, then fold the K aggregates in time
            // order: `carry` becomes the state entering this warp's first tile, `next_carry` the
            // state leaving the super-tile (every warp computes the same value).
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
            float run = carry;
#pragma unroll
            for (int ww = 0; ww < K; ++ww) {
                if (ww == w) carry = run;
                const float2 p = agg[buf][ww];
                run = fmaf(p.x, run, p.y);
                if constexpr (!WRITE) prod *= p.x;
            }
            next_carry = run;
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const float tA = __shfl_sync(kFullMask, A[j], 31);
            const float tH = __shfl_sync(kFullMask, H[j], 31);
            if constexpr (WRITE) {
                float eA = __shfl_up_sync(kFullMask, A[j], 1);
                float eH = __shfl_up_sync(kFullMask, H[j], 1);
                if (lane == 0) {
                    eA = 1.f;
                    eH = 0.f;
                }
                float s = fmaf(eA, carry, eH);  // state entering this lane's elements
                float out[E];
#pragma unroll
                for (int i = 0; i < E; ++i) {
                    s = fmaf(fa[j][i], s, fx[j][i]);
                    out[i] = s;
                }
                store_vec_policy<S, GENERIC>(states + off, v + j * TILE, L, ph_h, Store<S>::pack(out), store_pol);
            } else if constexpr (K == 1) {
                prod *= tA;
            }
            carry = fmaf(tA, carry, tH);
        }
        if constexpr (K > 1) carry = next_carry;

        if (last_group) {  // the unit is complete
            if (lane == 0 && w == 0) {
                if (h_last) h_last[unit] = carry;
                if (!WRITE && P_out) P_out[unit] = prod;
            }
            if (!more) break;
            unit += stride;
            carry = h0 ? h0[unit] : 0.f;
            prod = 1.f;
            g = 0;
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
#undef FMS_GOFF
#undef FMS_TOFF
}

// ---------------------------------------------------------------- backward / reverse reduce -
// c_t = a_t * (G_t + c_{t+1}) scanned from the row end; delta_t = G_t + c_{t+1};
// grad_tokens_t = delta_t; grad_gates_t = delta_t * h_{t-1}; grad_h0 = c_0.
// WRITE = false produces only S_rev = c_0 (from carry_in = 0) and P = prod a.
// Same persistence rule as the forward kernel.
//
// FM = true (needs WRITE): unit (b,m,d) additionally reads token row (b,d); instead of storing two
// full rows it ACCUMULATES into fp32 buffers
//     acc_gates [b,m,t] += (h_{t-1} - x_t) * delta_t     (sum over d; fm/scan/fm_scan.cuh:188-207
//                                                          followed by fm/scan/fm_scan.py:76)
//     acc_tokens[b,d,t] += (1 - g_t) * delta_t           (sum over m; fm_scan.cuh:184-185, fm_scan.py:78)
// with vector reductions, so the reference's two (B,M,D,L) temporaries never exist.  When the
// caller does pass (B,M,D,L) outputs in grad_gates / grad_tokens (the unmodified reference caller,
// fm/scan/fm_scan.py:70-73, which sums them itself), the per-row terms are stored there instead.
template <typename S, bool GENERIC, int U, bool WRITE, int K, bool SEG, bool FM>
__global__ void __launch_bounds__(Coop<K>::kThreads)
plain_backward_kernel(const S *__restrict__ gates, const S *__restrict__ states,
                      const S *__restrict__ grad_states, const float *__restrict__ h0,
                      const float *__restrict__ carry_in, S *__restrict__ grad_gates,
                      S *__restrict__ grad_tokens, float *__restrict__ grad_h0,
                      float *__restrict__ P_out, int64_t R, int64_t T, int64_t nseg,
                      int64_t seg_len, const S *__restrict__ tokens_fm, float *__restrict__ acc_gates,
                      float *__restrict__ acc_tokens, int64_t M, int64_t D, int descending) {
    static_assert(!(FM && SEG) && !(FM && !WRITE), "FM mode: whole rows, full backward only");
    constexpr int E = Store<S>::E;
    constexpr int TILE = 32 * E;
    constexpr bool PERSIST = !GENERIC && !SEG && !FM;
    constexpr int64_t SUPER = static_cast<int64_t>(TILE) * U * K;
    __shared__ float2 agg[2][K > 1 ? K : 1];
    const int lane = threadIdx.x & 31;
    const int w = Coop<K>::warp_in_unit();
    int64_t unit = Coop<K>::first_unit();
    if (unit >= R) return;
    // descending: units are visited from the last one down, so that the rows a forward over the
    // same tensors touched last (still in L2) are re-read first
    int64_t stride = Coop<K>::unit_stride();
    if (descending) {
        unit = R - 1 - unit;
        stride = -stride;
    }

    const Unit q = unit_of<SEG>(unit, T, nseg, seg_len);
    const int64_t L = q.len;
    int64_t off = q.offset;
    int64_t goff_fm = 0, toff_fm = 0;
    if constexpr (FM) {
        const int64_t bm = unit / D, d = unit - bm * D, b = bm / M;
        goff_fm = bm * T;
        toff_fm = (b * D + d) * T;
    }
#define FMS_GOFF (FM ? goff_fm : off)
    const int64_t vbase = row_phase<S, GENERIC>(gates + FMS_GOFF);
    const bool ph_g = !GENERIC || same_phase16(gates + FMS_GOFF, grad_states + off);
    const bool ph_h = !GENERIC || !WRITE || same_phase16(gates + FMS_GOFF, states + off);
    // FM mode stores per-row gradients only when the caller passed (B,M,D,L) outputs
    const bool fm_unreduced = FM && grad_gates != nullptr;
    const bool ph_ga = !GENERIC || !WRITE || (FM && !fm_unreduced) || same_phase16(gates + FMS_GOFF, grad_gates + off);
    const bool ph_gx = !GENERIC || !WRITE || (FM && !fm_unreduced) || same_phase16(gates + FMS_GOFF, grad_tokens + off);
    const bool ph_x = !GENERIC || !FM || same_phase16(gates + FMS_GOFF, tokens_fm + toff_fm);
    const int64_t ngroups = (L - vbase + SUPER - 1) / SUPER;
    // this lane's first vector in the LAST group of a unit (the first one the reverse walk visits)
    const int64_t v_last = vbase + (ngroups - 1) * SUPER + static_cast<int64_t>(w) * (TILE * U) + lane * E;

    // State just before the unit: the row's initial state, or (split path) the last state of
    // the previous segment of the same row.
    auto state_before = [&](int64_t u, int64_t o) -> float {
        if constexpr (!WRITE) return 0.f;
        if constexpr (SEG) {
            if (!q.first) return Store<S>::to_float(states[o - 1]);
            return h0 ? h0[u / nseg] : 0.f;
        }
        return h0 ? h0[u] : 0.f;
    };
    float h_before = state_before(unit, off);
    float carry = carry_in ? carry_in[unit] : 0.f;  // c at the first position after the super-tile
    float prod = 1.f;

    // State just before a tile (h_{t-1} of the tile's first element), read by lane 0; positions
    // before the unit are replaced by h_before when the tile is computed.
    auto load_halo = [&](int64_t o, int64_t vt) -> float {
        if (!WRITE || lane != 0) return 0.f;
        const int64_t t = vt - 1;
        return (t >= 0 && t < L) ? Store<S>::to_float(states[o + t]) : 0.f;
    };

    int64_t v = v_last;
    int64_t g = ngroups - 1;
    uint4 ra[U], rg[U], rh[U], rx[FM ? U : 1];
    float halo[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        ra[j] = load_vec<S, GENERIC>(gates + FMS_GOFF, v + j * TILE, L, true, Store<S>::kOne);
        rg[j] = load_vec<S, GENERIC>(grad_states + off, v + j * TILE, L, ph_g, 0u);
        if constexpr (WRITE) {
            rh[j] = load_vec<S, GENERIC>(states + off, v + j * TILE, L, ph_h, 0u);
            halo[j] = load_halo(off, v + j * TILE);
        }
        if constexpr (FM) rx[j] = load_vec<S, GENERIC>(tokens_fm + toff_fm, v + j * TILE, L, ph_x, 0u);
    }

    for (unsigned it = 0;; ++it) {
        const bool last_group = (g == 0);  // last in walking order = first in time
        int64_t noff = off, nv = v - SUPER;
        bool more = true;
        if (last_group) {
            if (PERSIST && unit + stride < R && unit + stride >= 0) {
                noff = (unit + stride) * T;
                nv = v_last;
            } else {
                more = false;
            }
        }
        uint4 na[U], ng[U], nh[U], nx[FM ? U : 1];
        float nhalo[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int64_t vv = more ? nv + j * TILE : L;  // L = "outside" for every path
            na[j] = load_vec<S, GENERIC>(gates + (FM ? goff_fm : noff), vv, L, true, Store<S>::kOne);
            ng[j] = load_vec<S, GENERIC>(grad_states + noff, vv, L, ph_g, 0u);
            if constexpr (WRITE) {
                nh[j] = load_vec<S, GENERIC>(states + noff, vv, L, ph_h, 0u);
                nhalo[j] = more ? load_halo(noff, vv) : 0.f;
            }
            if constexpr (FM) nx[j] = load_vec<S, GENERIC>(tokens_fm + toff_fm, vv, L, ph_x, 0u);
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
        // Inclusive warp scan towards lane 0 (later positions combine into earlier ones).
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
        float next_carry = 0.f;
        if constexpr (K > 1) {
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
            float run = carry;
#pragma unroll
            for (int ww = K - 1; ww >= 0; --ww) {
                if (ww == w) carry = run;
                const float2 p = agg[buf][ww];
                run = fmaf(p.x, run, p.y);
                if constexpr (!WRITE) prod *= p.x;
            }
            next_carry = run;
        }
#pragma unroll
        for (int j = U - 1; j >= 0; --j) {
            const float tA = __shfl_sync(kFullMask, A[j], 0);
            const float tC = __shfl_sync(kFullMask, C[j], 0);
            if constexpr (WRITE) {
                float eA = __shfl_down_sync(kFullMask, A[j], 1);
                float eC = __shfl_down_sync(kFullMask, C[j], 1);
                if (lane == 31) {
                    eA = 1.f;
                    eC = 0.f;
                }
                float fh[E];
                Store<S>::unpack(rh[j], fh);
                // h_{t-1} of this lane's first element: last state of the lane below, or the halo.
                float hprev0 = __shfl_up_sync(kFullMask, fh[E - 1], 1);
                if (lane == 0) hprev0 = (v + j * TILE - 1 >= 0) ? halo[j] : h_before;
                float c = fmaf(eA, carry, eC);  // c just after this lane's elements
                float dx[E], da[E];
                float fxm[FM ? E : 1];
                if constexpr (FM) Store<S>::unpack(rx[j], fxm);
#pragma unroll
                for (int i = E - 1; i >= 0; --i) {
                    const float delta = fg[j][i] + c;
                    c = fa[j][i] * delta;
                    float hp = (i > 0) ? fh[i > 0 ? i - 1 : 0] : hprev0;
                    if constexpr (GENERIC) {
                        if (v + j * TILE + i == 0) hp = h_before;  // unit start inside a vector
                    }
                    if constexpr (FM) {
                        dx[i] = (1.f - fa[j][i]) * delta;
                        da[i] = delta * (hp - fxm[i]);
                    } else {
                        dx[i] = delta;
                        da[i] = delta * hp;
                    }
                }
                if (FM && !fm_unreduced) {
                    red_vec<E, GENERIC>(acc_tokens + toff_fm, v + j * TILE, L, dx);
                    red_vec<E, GENERIC>(acc_gates + goff_fm, v + j * TILE, L, da);
                } else {
                    store_vec<S, GENERIC>(grad_tokens + off, v + j * TILE, L, ph_gx, Store<S>::pack(dx));
                    store_vec<S, GENERIC>(grad_gates + off, v + j * TILE, L, ph_ga, Store<S>::pack(da));
                }
            } else if constexpr (K == 1) {
                prod *= tA;
            }
            carry = fmaf(tA, carry, tC);
        }
        if constexpr (K > 1) carry = next_carry;

        if (last_group) {
            if (lane == 0 && w == 0) {
                if (grad_h0) grad_h0[unit] = carry;
                if (!WRITE && P_out) P_out[unit] = prod;
            }
            if (!more) break;
            unit += stride;
            h_before = state_before(unit, noff);
            carry = carry_in ? carry_in[unit] : 0.f;
            prod = 1.f;
            g = ngroups - 1;
        } else {
            --g;
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            ra[j] = na[j];
            rg[j] = ng[j];
            if constexpr (WRITE) {
                rh[j] = nh[j];
                halo[j] = nhalo[j];
            }
            if constexpr (FM) rx[j] = nx[j];
        }
        off = noff;
        v = nv;
    }
#undef FMS_GOFF
}

// fp32 accumulators -> storage type (FM-mode gradients with 16-bit storage).
template <typename S>
__global__ void cast_from_f32_kernel(const float *__restrict__ src, S *__restrict__ dst, int64_t n) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) {
        if constexpr (sizeof(S) == 4) dst[i] = src[i];
        else if constexpr (Store<S>::kOne == 0x3f803f80u) dst[i] = __float2bfloat16(src[i]);
        else dst[i] = __float2half(src[i]);
    }
}

// ---------------------------------------------------------------- carry combination ---------
// One thread per row folds the per-block carries serially in scan order (nchunks is the number
// of ranks or time blocks: small).
// Element (chunk k, row r) of P, S and carry_out lives at k*chunk_stride + r*row_stride:
// (R, 1) for the chunk-major layout an all-gather produces, (1, nchunks) for the row-major
// layout of the one-GPU split path.
static __global__ void combine_carries_kernel(const float *__restrict__ P, const float *__restrict__ S,
                                       const float *__restrict__ carry0,
                                       float *__restrict__ carry_out, float *__restrict__ total,
                                       int64_t nchunks, int64_t R, int reverse,
                                       int64_t chunk_stride, int64_t row_stride) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r >= R) return;
    float c = carry0 ? carry0[r] : 0.f;
    for (int64_t i = 0; i < nchunks; ++i) {
        const int64_t k = reverse ? nchunks - 1 - i : i;
        const int64_t at = k * chunk_stride + r * row_stride;
        carry_out[at] = c;
        c = fmaf(P[at], c, S[at]);
    }
    if (total) total[r] = c;
}

}  // namespace fms
