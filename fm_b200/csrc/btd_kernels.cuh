// Channel-last scan: tensors (B, T, D), one recurrence per (b, d) along T.
//
// The layer of the reference receives its inputs as (B, L, .) and transposes them to (B, ., L)
// before every call of the scan (fm/scan/fm_scan.py:118-119).  These kernels scan the (B, T, D)
// layout directly.  Lanes run across channels (a lane owns E = 16 bytes of consecutive channels,
// a warp 512 contiguous bytes of one time step), time is walked sequentially with the loads of
// the next PF steps already in flight as cp.async copies into a per-lane shared-memory ring,
// and T is cut into chunks so that the machine is filled:
//   pass 1  per (b, chunk, channel): P = prod a, S = state from a zero start     reads a, x
//   pass 2  fold the chunks of every (b, channel) in time order                  tiny
//   pass 3  scan every chunk from its true carry-in                              reads a, x; writes h
// Backward mirrors it with c_t = a_t * (G_t + c_{t+1}) walked from the end; h_{t-1} of a step is
// simply the state vector of the previous time step (row t-1 of the same channels).
#pragma once

#include "scan_kernels.cuh"

namespace fms {

#ifndef FMS_BTD_WARPS
#define FMS_BTD_WARPS 4
#endif
#ifndef FMS_BTD_PF
#define FMS_BTD_PF 16
#endif
constexpr int kBtdWarps = FMS_BTD_WARPS;  // warps per CTA = adjacent channel tiles of one (b, chunk)
constexpr int kBtdPF = FMS_BTD_PF;        // time steps in flight per lane

struct BtdGeom {
    int64_t B, T, D, nchunks, chunk, dtiles;  // dtiles = ceil(D / (32*E))
};

// which (b, chunk, channel vector) this lane works on; returns false for lanes past D
template <int E>
__device__ __forceinline__ bool btd_lane(const BtdGeom &g, int64_t &b, int64_t &c, int64_t &d) {
    const int64_t warp = static_cast<int64_t>(blockIdx.x) * kBtdWarps + (threadIdx.x >> 5);
    const int64_t dt = warp % g.dtiles, rest = warp / g.dtiles;
    c = rest % g.nchunks;
    b = rest / g.nchunks;
    d = dt * (32 * E) + (threadIdx.x & 31) * E;
    return b < g.B && d < g.D;
}

// ---- per-lane asynchronous ring ------------------------------------------------------------
// A lane's loads of the next kBtdPF time steps are in flight as 16-byte cp.async copies into a
// shared-memory ring that only this lane reads back, so the depth costs no registers and needs no
// barrier: the lane waits on its own copy groups (one group per time step).
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ring slot of (tensor, step) for this thread: [tensor][step % PF][thread]
template <int NT>
struct BtdRing {
    uint4 *base;
    __device__ __forceinline__ uint4 *slot(int tensor, int64_t step) const {
        return base + (static_cast<size_t>(tensor) * kBtdPF + static_cast<size_t>(step % kBtdPF)) * (kBtdWarps * 32) +
               threadIdx.x;
    }
};
template <int NT>
constexpr size_t btd_ring_bytes() {
    return sizeof(uint4) * NT * kBtdPF * kBtdWarps * 32;
}

// REVERSE = false: P, S of the forward recurrence;  true: P and the reverse carry c at the chunk
// start from a zero carry-in (second operand = grad of the states).
template <typename S, bool REVERSE>
__global__ void __launch_bounds__(kBtdWarps * 32)
btd_reduce_kernel(const S *__restrict__ gates, const S *__restrict__ second, float *__restrict__ P_out,
                  float *__restrict__ S_out, BtdGeom g) {
    constexpr int E = Store<S>::E;
    extern __shared__ __align__(16) unsigned char btd_smem[];
    const BtdRing<2> ring{reinterpret_cast<uint4 *>(btd_smem)};
    int64_t b, c, d;
    if (!btd_lane<E>(g, b, c, d)) return;
    const int64_t t0 = c * g.chunk, t1 = min(g.T, t0 + g.chunk), n = t1 - t0;
    const int64_t step = REVERSE ? -g.D : g.D;
    const S *ap = gates + (b * g.T + (REVERSE ? t1 - 1 : t0)) * g.D + d;
    const S *sp = second + (b * g.T + (REVERSE ? t1 - 1 : t0)) * g.D + d;
    float prod[E], acc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
        prod[e] = 1.f;
        acc[e] = 0.f;
    }
    auto issue = [&](int64_t i) {
        if (i < n) {
            cp_async16(ring.slot(0, i), ap + i * step);
            cp_async16(ring.slot(1, i), sp + i * step);
        }
        cp_async_commit();  // an empty group past the end keeps the group count in step
    };
    for (int64_t i = 0; i < kBtdPF; ++i) issue(i);
    for (int64_t i = 0; i < n; ++i) {
        cp_async_wait<kBtdPF - 1>();
        float fa[E], fs[E];
        Store<S>::unpack(*ring.slot(0, i), fa);
        Store<S>::unpack(*ring.slot(1, i), fs);
        issue(i + kBtdPF);
#pragma unroll
        for (int e = 0; e < E; ++e) {
            prod[e] *= fa[e];
            acc[e] = REVERSE ? fa[e] * (fs[e] + acc[e]) : fmaf(fa[e], acc[e], fs[e]);
        }
    }
    const int64_t o = (b * g.nchunks + c) * g.D + d;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        P_out[o + e] = prod[e];
        S_out[o + e] = acc[e];
    }
}

// Fold the chunks of every (b, channel): carry[b,c,d] = the carry entering chunk c (in scan
// order); the carry leaving the last chunk goes to `total` (nullable).  P and S are read in
// batches ahead of the serial fold.
__global__ void btd_fold_kernel(const float *__restrict__ P, const float *__restrict__ S,
                                float *__restrict__ carry, const float *__restrict__ carry0,
                                float *__restrict__ total, BtdGeom g, int reverse) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= g.B * g.D) return;
    const int64_t b = i / g.D, d = i - b * g.D;
    float c = carry0 ? carry0[i] : 0.f;
    constexpr int BATCH = 8;
    for (int64_t k0 = 0; k0 < g.nchunks; k0 += BATCH) {
        float p[BATCH], s[BATCH];
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
            const int64_t k = k0 + j;
            if (k < g.nchunks) {
                const int64_t o = (b * g.nchunks + (reverse ? g.nchunks - 1 - k : k)) * g.D + d;
                p[j] = P[o];
                s[j] = S[o];
            }
        }
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
            const int64_t k = k0 + j;
            if (k < g.nchunks) {
                const int64_t o = (b * g.nchunks + (reverse ? g.nchunks - 1 - k : k)) * g.D + d;
                carry[o] = c;
                c = fmaf(p[j], c, s[j]);
            }
        }
    }
    if (total) total[i] = c;
}

template <typename S>
__global__ void __launch_bounds__(kBtdWarps * 32)
btd_forward_kernel(const S *__restrict__ gates, const S *__restrict__ tokens, const float *__restrict__ carry,
                   S *__restrict__ states, BtdGeom g) {
    constexpr int E = Store<S>::E;
    extern __shared__ __align__(16) unsigned char btd_smem[];
    const BtdRing<2> ring{reinterpret_cast<uint4 *>(btd_smem)};
    int64_t b, c, d;
    if (!btd_lane<E>(g, b, c, d)) return;
    const int64_t t0 = c * g.chunk, t1 = min(g.T, t0 + g.chunk), n = t1 - t0;
    const int64_t base = (b * g.T + t0) * g.D + d;
    const S *ap = gates + base, *xp = tokens + base;
    S *hp = states + base;
    float s[E];
    const int64_t o = (b * g.nchunks + c) * g.D + d;
#pragma unroll
    for (int e = 0; e < E; ++e) s[e] = carry[o + e];
    auto issue = [&](int64_t i) {
        if (i < n) {
            cp_async16(ring.slot(0, i), ap + i * g.D);
            cp_async16(ring.slot(1, i), xp + i * g.D);
        }
        cp_async_commit();
    };
    for (int64_t i = 0; i < kBtdPF; ++i) issue(i);
    for (int64_t i = 0; i < n; ++i) {
        cp_async_wait<kBtdPF - 1>();
        float fa[E], fx[E], out[E];
        Store<S>::unpack(*ring.slot(0, i), fa);
        Store<S>::unpack(*ring.slot(1, i), fx);
        issue(i + kBtdPF);
#pragma unroll
        for (int e = 0; e < E; ++e) {
            s[e] = fmaf(fa[e], s[e], fx[e]);
            out[e] = s[e];
        }
        stg_stream(hp + i * g.D, Store<S>::pack(out));
    }
}

// grad_tokens_t = delta_t = G_t + c_{t+1};  c_t = a_t * delta_t;  grad_gates_t = delta_t * h_{t-1}.
template <typename S>
__global__ void __launch_bounds__(kBtdWarps * 32)
btd_backward_kernel(const S *__restrict__ gates, const S *__restrict__ states, const S *__restrict__ grad_states,
                    const float *__restrict__ h0, const float *__restrict__ carry, S *__restrict__ grad_gates,
                    S *__restrict__ grad_tokens, BtdGeom g) {
    constexpr int E = Store<S>::E;
    extern __shared__ __align__(16) unsigned char btd_smem[];
    const BtdRing<3> ring{reinterpret_cast<uint4 *>(btd_smem)};
    int64_t b, c, d;
    if (!btd_lane<E>(g, b, c, d)) return;
    const int64_t t0 = c * g.chunk, t1 = min(g.T, t0 + g.chunk), n = t1 - t0;
    const int64_t last = (b * g.T + t1 - 1) * g.D + d;  // walk from the chunk end
    const S *ap = gates + last, *gp = grad_states + last, *hp = states + last - g.D;  // hp: state of step t-1
    S *gap = grad_gates + last, *gxp = grad_tokens + last;
    float cc[E];
    const int64_t o = (b * g.nchunks + c) * g.D + d;
#pragma unroll
    for (int e = 0; e < E; ++e) cc[e] = carry[o + e];
    auto issue = [&](int64_t i) {
        if (i < n) {
            cp_async16(ring.slot(0, i), ap - i * g.D);
            cp_async16(ring.slot(1, i), gp - i * g.D);
            if (t1 - 1 - i > 0) cp_async16(ring.slot(2, i), hp - i * g.D);  // h_{-1} is patched in below
        }
        cp_async_commit();
    };
    for (int64_t i = 0; i < kBtdPF; ++i) issue(i);
    for (int64_t i = 0; i < n; ++i) {
        cp_async_wait<kBtdPF - 1>();
        float fa[E], fg[E], fh[E], dx[E], da[E];
        Store<S>::unpack(*ring.slot(0, i), fa);
        Store<S>::unpack(*ring.slot(1, i), fg);
        if (t1 - 1 - i > 0) {
            Store<S>::unpack(*ring.slot(2, i), fh);
        } else {  // the initial state, kept in fp32
#pragma unroll
            for (int e = 0; e < E; ++e) fh[e] = h0 ? h0[b * g.D + d + e] : 0.f;
        }
        issue(i + kBtdPF);
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float delta = fg[e] + cc[e];
            cc[e] = fa[e] * delta;
            dx[e] = delta;
            da[e] = delta * fh[e];
        }
        stg_stream(gxp - i * g.D, Store<S>::pack(dx));
        stg_stream(gap - i * g.D, Store<S>::pack(da));
    }
}

}  // namespace fms
