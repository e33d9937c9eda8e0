// Channel-last scan: tensors (B, T, D), one recurrence per (b, d) along T.
//
// The layer of the reference receives its inputs as (B, L, .) and transposes them to (B, ., L)
// before every call of the scan (fm/scan/fm_scan.py:118-119).  These kernels scan the (B, T, D)
// layout directly.  Lanes run across channels (a lane owns E = 16 bytes of consecutive channels,
// a warp 512 contiguous bytes of one time step), time is walked sequentially with the loads of
// the next PF steps already in flight, and T is cut into chunks so that the machine is filled:
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
#define FMS_BTD_PF 4
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

// REVERSE = false: P, S of the forward recurrence;  true: P and the reverse carry c at the chunk
// start from a zero carry-in (second operand = grad of the states).
template <typename S, bool REVERSE>
__global__ void __launch_bounds__(kBtdWarps * 32)
btd_reduce_kernel(const S *__restrict__ gates, const S *__restrict__ second, float *__restrict__ P_out,
                  float *__restrict__ S_out, BtdGeom g) {
    constexpr int E = Store<S>::E;
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
    uint4 qa[kBtdPF], qs[kBtdPF];
#pragma unroll
    for (int k = 0; k < kBtdPF; ++k)
        if (k < n) {
            qa[k] = ldg_stream(ap + k * step);
            qs[k] = ldg_stream(sp + k * step);
        }
    for (int64_t i = 0; i < n; i += kBtdPF) {
#pragma unroll
        for (int k = 0; k < kBtdPF; ++k) {
            if (i + k < n) {
                float fa[E], fs[E];
                Store<S>::unpack(qa[k], fa);
                Store<S>::unpack(qs[k], fs);
                if (i + k + kBtdPF < n) {
                    qa[k] = ldg_stream(ap + (i + k + kBtdPF) * step);
                    qs[k] = ldg_stream(sp + (i + k + kBtdPF) * step);
                }
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    prod[e] *= fa[e];
                    acc[e] = REVERSE ? fa[e] * (fs[e] + acc[e]) : fmaf(fa[e], acc[e], fs[e]);
                }
            }
        }
    }
    const int64_t o = (b * g.nchunks + c) * g.D + d;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        P_out[o + e] = prod[e];
        S_out[o + e] = acc[e];
    }
}

// Fold the chunks of every (b, channel): S[b,c,d] becomes the carry entering chunk c (in scan
// order); the carry leaving the last chunk goes to `total` (nullable).
__global__ void btd_fold_kernel(const float *__restrict__ P, float *__restrict__ S_to_carry,
                                const float *__restrict__ carry0, float *__restrict__ total, BtdGeom g,
                                int reverse) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= g.B * g.D) return;
    const int64_t b = i / g.D, d = i - b * g.D;
    float c = carry0 ? carry0[i] : 0.f;
    for (int64_t k = 0; k < g.nchunks; ++k) {
        const int64_t ch = reverse ? g.nchunks - 1 - k : k;
        const int64_t o = (b * g.nchunks + ch) * g.D + d;
        const float s = S_to_carry[o];
        S_to_carry[o] = c;
        c = fmaf(P[o], c, s);
    }
    if (total) total[i] = c;
}

template <typename S>
__global__ void __launch_bounds__(kBtdWarps * 32)
btd_forward_kernel(const S *__restrict__ gates, const S *__restrict__ tokens, const float *__restrict__ carry,
                   S *__restrict__ states, BtdGeom g) {
    constexpr int E = Store<S>::E;
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
    uint4 qa[kBtdPF], qx[kBtdPF];
#pragma unroll
    for (int k = 0; k < kBtdPF; ++k)
        if (k < n) {
            qa[k] = ldg_stream(ap + k * g.D);
            qx[k] = ldg_stream(xp + k * g.D);
        }
    for (int64_t i = 0; i < n; i += kBtdPF) {
#pragma unroll
        for (int k = 0; k < kBtdPF; ++k) {
            if (i + k < n) {
                float fa[E], fx[E], out[E];
                Store<S>::unpack(qa[k], fa);
                Store<S>::unpack(qx[k], fx);
                if (i + k + kBtdPF < n) {
                    qa[k] = ldg_stream(ap + (i + k + kBtdPF) * g.D);
                    qx[k] = ldg_stream(xp + (i + k + kBtdPF) * g.D);
                }
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    s[e] = fmaf(fa[e], s[e], fx[e]);
                    out[e] = s[e];
                }
                stg_stream(hp + (i + k) * g.D, Store<S>::pack(out));
            }
        }
    }
}

// grad_tokens_t = delta_t = G_t + c_{t+1};  c_t = a_t * delta_t;  grad_gates_t = delta_t * h_{t-1}.
template <typename S>
__global__ void __launch_bounds__(kBtdWarps * 32)
btd_backward_kernel(const S *__restrict__ gates, const S *__restrict__ states, const S *__restrict__ grad_states,
                    const float *__restrict__ h0, const float *__restrict__ carry, S *__restrict__ grad_gates,
                    S *__restrict__ grad_tokens, BtdGeom g) {
    constexpr int E = Store<S>::E;
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
    auto load_hprev = [&](int64_t k) -> uint4 {  // state before step t1-1-k (h0 is patched in at t = 0)
        return (t1 - 1 - k > 0) ? ldg_stream(hp - k * g.D) : make_uint4(0u, 0u, 0u, 0u);
    };
    uint4 qa[kBtdPF], qg[kBtdPF], qh[kBtdPF];
#pragma unroll
    for (int k = 0; k < kBtdPF; ++k)
        if (k < n) {
            qa[k] = ldg_stream(ap - k * g.D);
            qg[k] = ldg_stream(gp - k * g.D);
            qh[k] = load_hprev(k);
        }
    for (int64_t i = 0; i < n; i += kBtdPF) {
#pragma unroll
        for (int k = 0; k < kBtdPF; ++k) {
            if (i + k < n) {
                float fa[E], fg[E], fh[E], dx[E], da[E];
                Store<S>::unpack(qa[k], fa);
                Store<S>::unpack(qg[k], fg);
                Store<S>::unpack(qh[k], fh);
                if (t1 - 1 - (i + k) == 0) {  // h_{-1} is the initial state, kept in fp32
#pragma unroll
                    for (int e = 0; e < E; ++e) fh[e] = h0 ? h0[b * g.D + d + e] : 0.f;
                }
                if (i + k + kBtdPF < n) {
                    qa[k] = ldg_stream(ap - (i + k + kBtdPF) * g.D);
                    qg[k] = ldg_stream(gp - (i + k + kBtdPF) * g.D);
                    qh[k] = load_hprev(i + k + kBtdPF);
                }
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const float delta = fg[e] + cc[e];
                    cc[e] = fa[e] * delta;
                    dx[e] = delta;
                    da[e] = delta * fh[e];
                }
                stg_stream(gxp - (i + k) * g.D, Store<S>::pack(dx));
                stg_stream(gap - (i + k) * g.D, Store<S>::pack(da));
            }
        }
    }
}

}  // namespace fms
