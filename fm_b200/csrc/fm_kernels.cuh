// FM-mode kernels blocked over rows that share a gate row or a token row.
//
// FM mode is the reference's own operator (fm/scan/fm_pytorch.py:19-42):
//     h[b,m,d,t] = g[b,m,t] * h[b,m,d,t-1] + (1 - g[b,m,t]) * x[b,d,t]
// Its backward needs, besides one reverse scan per output row (b,m,d),
//     d_gates [b,m,t] = sum_d (h[b,m,d,t-1] - x[b,d,t]) * delta[b,m,d,t]
//     d_tokens[b,d,t] = sum_m (1 - g[b,m,t])            * delta[b,m,d,t]
// which the reference obtains from two (B,M,D,L) temporaries and two torch sums
// (fm/scan/fm_scan.cuh:184-207, fm/scan/fm_scan.py:70-78).
//
// Here a CTA owns MC gate rows x DC token rows of one batch element (MC*DC output rows) and
// walks time backwards one tile (32 lanes x 16 bytes) per step.  Warp w owns gate row m0+w:
//   * the gate tile is loaded and unpacked once per step and the gate half of the pair scan
//     (the five levels of prefix products) is computed once, then reused for all DC rows;
//   * the DC token tiles of the step are staged in shared memory once for all warps;
//   * the sum over d is accumulated in registers (same warp); for the sum over m every warp
//     publishes its tile to shared memory and, after a barrier, warp d adds the MC tiles of
//     token row d (plain 128-bit shared accesses, no shared atomics, fixed summation order);
//   * per step each warp issues ONE vector reduction row for d_gates and the CTA DC rows for
//     d_tokens: global atomics drop by DC and MC against one-row-per-CTA.
// Only the big streams h and G (grad of the states) come from HBM; they are prefetched PD rows
// ahead into registers.
#pragma once

#include "scan_kernels.cuh"

namespace fms {

template <typename S, int MC, int DC, int PD>
__global__ void __launch_bounds__(MC * 32, 2)
fm_backward_blocked_kernel(const S *__restrict__ gates, const S *__restrict__ tokens,
                           const S *__restrict__ states, const S *__restrict__ grad_states,
                           const float *__restrict__ h0, float *__restrict__ acc_gates,
                           float *__restrict__ acc_tokens, float *__restrict__ grad_h0, int64_t M,
                           int64_t D, int64_t L, int64_t m_blocks, int64_t d_blocks) {
    static_assert(DC % PD == 0 && PD <= DC, "DC must be a multiple of the prefetch distance");
    constexpr int E = Store<S>::E;
    constexpr int W = 32 * E;  // positions per tile
    // dynamic shared memory (more than the 48 KB static limit): token tiles, then the partial tiles
    extern __shared__ __align__(16) unsigned char fm_smem[];
    uint4(*xs)[DC][32] = reinterpret_cast<uint4(*)[DC][32]>(fm_smem);  // [2][DC][32] token tiles, raw
    // every warp's (1-g)*delta tile of every token row; summed over warps after the step.
    // [warp][row][E/4][lane] float4: a lane's two vectors sit in different halves, so both the
    // stores and the loads are conflict-free 128-bit accesses
    float4(*part)[DC][E / 4][32] =
        reinterpret_cast<float4(*)[DC][E / 4][32]>(fm_smem + sizeof(uint4) * 2 * DC * 32);  // [MC][DC][E/4][32]
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;

    // block -> (b, m block, d block); d blocks vary fastest so neighbours share the gate rows in L2
    const int64_t blk = blockIdx.x;
    const int64_t db = blk % d_blocks, mb = (blk / d_blocks) % m_blocks, b = blk / (d_blocks * m_blocks);
    const int64_t m = mb * MC + w, d0 = db * DC;
    const bool have_m = m < M;
    const int64_t ntiles = (L + W - 1) / W;

    const S *grow = gates + (b * M + (have_m ? m : 0)) * L;
    const int64_t row0 = ((b * M + (have_m ? m : 0)) * D + d0);  // first output row of this warp
    float carry[DC], dh_before[DC];
#pragma unroll
    for (int d = 0; d < DC; ++d) {
        carry[d] = 0.f;
        dh_before[d] = (h0 && have_m && d0 + d < D) ? h0[row0 + d] : 0.f;
    }
    // register ring of the big streams: slot = d % PD
    uint4 rG[PD], rH[PD];
    float rhalo[PD];
    auto fetch = [&](int slot, int64_t tile, int d) {
        const int64_t t = tile * W + lane * E;
        const bool ok = have_m && tile >= 0 && d0 + d < D && t < L;
        const int64_t base = (row0 + d) * L;
        rG[slot] = ok ? ldg_stream(grad_states + base + t) : make_uint4(0u, 0u, 0u, 0u);
        rH[slot] = ok ? ldg_stream(states + base + t) : make_uint4(0u, 0u, 0u, 0u);
        rhalo[slot] = (ok && lane == 0 && t > 0) ? Store<S>::to_float(states[base + t - 1]) : 0.f;
    };
#pragma unroll
    for (int p = 0; p < PD; ++p) fetch(p, ntiles - 1, p);

    // Token tiles and the gate tile of a step are fetched one step ahead into registers; the token
    // tiles then go to the shared buffer the NEXT step reads (two buffers, so a step needs only
    // two barriers).
    auto load_x = [&](int64_t tile, int d) -> uint4 {
        const int64_t tt = tile * W + lane * E;
        return (tile >= 0 && tt < L && d < DC && d0 + d < D) ? ldg_stream(tokens + (b * D + d0 + d) * L + tt)
                                                   : make_uint4(0u, 0u, 0u, 0u);
    };
    auto load_g = [&](int64_t tile) -> uint4 {
        const int64_t tt = tile * W + lane * E;
        return (tile >= 0 && tt < L && have_m)
                   ? ldg_stream(grow + tt)
                   : make_uint4(Store<S>::kOne, Store<S>::kOne, Store<S>::kOne, Store<S>::kOne);
    };
    constexpr int XPW = (DC + MC - 1) / MC;  // token rows staged per warp
    uint4 gq = load_g(ntiles - 1), xq[XPW];
#pragma unroll
    for (int k = 0; k < XPW; ++k)
        if (w + k * MC < DC) xs[0][w + k * MC][lane] = load_x(ntiles - 1, w + k * MC);

    unsigned step = 0;
    for (int64_t tile = ntiles - 1; tile >= 0; --tile, ++step) {
        const int64_t t = tile * W + lane * E;  // this lane's first position
        const bool in = t < L;
        const unsigned buf = step & 1u;
        __syncthreads();  // previous step's flush is complete and xs[buf] is staged
        float fa[E], om[E];
        Store<S>::unpack(gq, fa);
        gq = load_g(tile - 1);
#pragma unroll
        for (int k = 0; k < XPW; ++k) xq[k] = load_x(tile - 1, w + k * MC);
        float A = fa[E - 1];
#pragma unroll
        for (int i = E - 2; i >= 0; --i) A *= fa[i];
#pragma unroll
        for (int i = 0; i < E; ++i) om[i] = 1.f - fa[i];
        float Alvl[5];
#pragma unroll
        for (int k = 0; k < 5; ++k) {
            Alvl[k] = A;
            const float pA = __shfl_down_sync(kFullMask, A, 1 << k);
            if (lane + (1 << k) < 32) A *= pA;
        }
        float eA = __shfl_down_sync(kFullMask, A, 1);
        if (lane == 31) eA = 1.f;
        const float tA = __shfl_sync(kFullMask, A, 0);
        float dg[E];
#pragma unroll
        for (int i = 0; i < E; ++i) dg[i] = 0.f;

#pragma unroll
        for (int d = 0; d < DC; ++d) {
            const int slot = d % PD;
            float fg[E], fh[E], fx[E];
            Store<S>::unpack(rG[slot], fg);
            Store<S>::unpack(rH[slot], fh);
            const float halo = rhalo[slot];
            // refill the slot: PD rows ahead, wrapping into the next (earlier) tile
            if (d + PD < DC) fetch(slot, tile, d + PD);
            else fetch(slot, tile - 1, d + PD - DC);
            Store<S>::unpack(xs[buf][d][lane], fx);

            float C = fa[E - 1] * fg[E - 1];
#pragma unroll
            for (int i = E - 2; i >= 0; --i) C = fa[i] * (fg[i] + C);
#pragma unroll
            for (int k = 0; k < 5; ++k) {
                const float pC = __shfl_down_sync(kFullMask, C, 1 << k);
                if (lane + (1 << k) < 32) C = fmaf(Alvl[k], pC, C);
            }
            float eC = __shfl_down_sync(kFullMask, C, 1);
            if (lane == 31) eC = 0.f;
            const float tC = __shfl_sync(kFullMask, C, 0);
            float hprev0 = __shfl_up_sync(kFullMask, fh[E - 1], 1);
            if (lane == 0) hprev0 = (t > 0) ? halo : dh_before[d];
            float c = fmaf(eA, carry[d], eC);
            carry[d] = fmaf(tA, carry[d], tC);
            float dxv[E];  // zero for masked rows and lanes (G = 0, carry = 0 there)
#pragma unroll
            for (int i = E - 1; i >= 0; --i) {
                const float delta = fg[i] + c;
                c = fa[i] * delta;
                const float hp = (i > 0) ? fh[i > 0 ? i - 1 : 0] : hprev0;
                dg[i] = fmaf(delta, hp - fx[i], dg[i]);
                dxv[i] = om[i] * delta;
            }
#pragma unroll
            for (int k = 0; k < E / 4; ++k)
                part[w][d][k][lane] = make_float4(dxv[4 * k], dxv[4 * k + 1], dxv[4 * k + 2], dxv[4 * k + 3]);
        }
        if (in && have_m) red_vec<E, false>(acc_gates + (b * M + m) * L, t, L, dg);
#pragma unroll
        for (int k = 0; k < XPW; ++k)
            if (w + k * MC < DC) xs[buf ^ 1u][w + k * MC][lane] = xq[k];
        __syncthreads();  // every warp has published its tiles (and staged the next token tiles)
#pragma unroll
        for (int d = w; d < DC; d += MC) {
            float v[E];
#pragma unroll
            for (int i = 0; i < E; ++i) v[i] = 0.f;
#pragma unroll
            for (int ww = 0; ww < MC; ++ww)
#pragma unroll
                for (int k = 0; k < E / 4; ++k) {
                    const float4 p = part[ww][d][k][lane];
                    v[4 * k] += p.x;
                    v[4 * k + 1] += p.y;
                    v[4 * k + 2] += p.z;
                    v[4 * k + 3] += p.w;
                }
            if (in && d0 + d < D) red_vec<E, false>(acc_tokens + (b * D + d0 + d) * L, t, L, v);
        }
    }
    if (grad_h0 && have_m && lane == 0) {
#pragma unroll
        for (int d = 0; d < DC; ++d)
            if (d0 + d < D) grad_h0[row0 + d] = carry[d];
    }
}

// FM-mode forward with the same blocking: warp w owns gate row m0+w and produces the DC state
// rows (m0+w, d0..d0+DC-1).  The gate tile is unpacked and its prefix products are taken once per
// step; the DC token tiles are staged in shared memory one step ahead (two buffers, one barrier
// per step); each state row costs one 5-shuffle scan of its token half and one 16-byte store per
// lane.  Nothing but the states goes to HBM; gates and tokens are read once per CTA block.
template <typename S, int MC, int DC>
__global__ void __launch_bounds__(MC * 32)
fm_forward_blocked_kernel(const S *__restrict__ gates, const S *__restrict__ tokens,
                          const float *__restrict__ h0, S *__restrict__ states, int64_t M, int64_t D,
                          int64_t L, int64_t m_blocks, int64_t d_blocks) {
    constexpr int E = Store<S>::E;
    constexpr int W = 32 * E;
    __shared__ uint4 xs[2][DC][32];
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const int64_t blk = blockIdx.x;
    const int64_t db = blk % d_blocks, mb = (blk / d_blocks) % m_blocks, b = blk / (d_blocks * m_blocks);
    const int64_t m = mb * MC + w, d0 = db * DC;
    const bool have_m = m < M;
    const int64_t ntiles = (L + W - 1) / W;
    const S *grow = gates + (b * M + (have_m ? m : 0)) * L;
    const int64_t row0 = ((b * M + (have_m ? m : 0)) * D + d0);

    float carry[DC];
#pragma unroll
    for (int d = 0; d < DC; ++d) carry[d] = (h0 && have_m && d0 + d < D) ? h0[row0 + d] : 0.f;

    auto load_x = [&](int64_t tile, int d) -> uint4 {
        const int64_t tt = tile * W + lane * E;
        return (tile < ntiles && tt < L && d < DC && d0 + d < D)
                   ? ldg_stream(tokens + (b * D + d0 + d) * L + tt)
                   : make_uint4(0u, 0u, 0u, 0u);
    };
    auto load_g = [&](int64_t tile) -> uint4 {
        const int64_t tt = tile * W + lane * E;
        return (tile < ntiles && tt < L && have_m)
                   ? ldg_stream(grow + tt)
                   : make_uint4(Store<S>::kOne, Store<S>::kOne, Store<S>::kOne, Store<S>::kOne);
    };
    constexpr int XPW = (DC + MC - 1) / MC;
    uint4 gq = load_g(0), xq[XPW];
#pragma unroll
    for (int k = 0; k < XPW; ++k)
        if (w + k * MC < DC) xs[0][w + k * MC][lane] = load_x(0, w + k * MC);

    for (int64_t tile = 0; tile < ntiles; ++tile) {
        const int64_t t = tile * W + lane * E;
        const bool in = t < L;
        const unsigned buf = static_cast<unsigned>(tile) & 1u;
        __syncthreads();  // xs[buf] is staged; xs[buf^1] is no longer read
        float fa[E], om[E];
        Store<S>::unpack(gq, fa);
        gq = load_g(tile + 1);
#pragma unroll
        for (int k = 0; k < XPW; ++k) xq[k] = load_x(tile + 1, w + k * MC);
        float A = fa[0];
#pragma unroll
        for (int i = 1; i < E; ++i) A *= fa[i];
#pragma unroll
        for (int i = 0; i < E; ++i) om[i] = 1.f - fa[i];
        float Alvl[5];
#pragma unroll
        for (int k = 0; k < 5; ++k) {
            Alvl[k] = A;
            const float pA = __shfl_up_sync(kFullMask, A, 1 << k);
            if (lane >= (1 << k)) A *= pA;
        }
        float eA = __shfl_up_sync(kFullMask, A, 1);
        if (lane == 0) eA = 1.f;
        const float tA = __shfl_sync(kFullMask, A, 31);

#pragma unroll
        for (int d = 0; d < DC; ++d) {
            float fx[E];
            Store<S>::unpack(xs[buf][d][lane], fx);
#pragma unroll
            for (int i = 0; i < E; ++i) fx[i] *= om[i];
            float H = fx[0];
#pragma unroll
            for (int i = 1; i < E; ++i) H = fmaf(fa[i], H, fx[i]);
#pragma unroll
            for (int k = 0; k < 5; ++k) {
                const float pH = __shfl_up_sync(kFullMask, H, 1 << k);
                if (lane >= (1 << k)) H = fmaf(Alvl[k], pH, H);
            }
            float eH = __shfl_up_sync(kFullMask, H, 1);
            if (lane == 0) eH = 0.f;
            const float tH = __shfl_sync(kFullMask, H, 31);
            float s_ = fmaf(eA, carry[d], eH);
            carry[d] = fmaf(tA, carry[d], tH);
            float out[E];
#pragma unroll
            for (int i = 0; i < E; ++i) {
                s_ = fmaf(fa[i], s_, fx[i]);
                out[i] = s_;
            }
            if (in && have_m && d0 + d < D) stg_stream(states + (row0 + d) * L + t, Store<S>::pack(out));
        }
#pragma unroll
        for (int k = 0; k < XPW; ++k)
            if (w + k * MC < DC) xs[buf ^ 1u][w + k * MC][lane] = xq[k];
    }
}

// The layer's read-out without materialising the states (fm/scan/fm_scan.py:122-131 computes
// states (B,M,D,L), RMS-normalises them over D and contracts them with the output weight over
// M).  Two launches of this kernel recompute the scan instead of storing it:
//   MODE 0: sumsq[b,m,t]  += sum over the CTA's token rows of h[b,m,d,t]^2
//   MODE 1: out32[b,d,t]  += sum over the CTA's gate rows of scale[b,m,t] * h[b,m,d,t]
// with scale = output_weight * rsqrt(sumsq / D + eps) formed in between (or just the output
// weight when the norm is off).  Same blocking as fm_forward_blocked_kernel; HBM sees only the
// gate, token, scale and output rows -- the (B,M,D,L) tensor never exists.
template <typename S, int MC, int DC, int MODE>
__global__ void __launch_bounds__(MC * 32)
fm_readout_blocked_kernel(const S *__restrict__ gates, const S *__restrict__ tokens,
                          const float *__restrict__ h0, const float *__restrict__ scale,
                          float *__restrict__ sumsq, float *__restrict__ out32, int64_t M, int64_t D,
                          int64_t L, int64_t m_blocks, int64_t d_blocks) {
    constexpr int E = Store<S>::E;
    constexpr int W = 32 * E;
    extern __shared__ __align__(16) unsigned char fm_smem[];
    uint4(*xs)[DC][32] = reinterpret_cast<uint4(*)[DC][32]>(fm_smem);
    float4(*part)[DC][E / 4][32] =
        reinterpret_cast<float4(*)[DC][E / 4][32]>(fm_smem + sizeof(uint4) * 2 * DC * 32);  // MODE 1 only
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const int64_t blk = blockIdx.x;
    const int64_t db = blk % d_blocks, mb = (blk / d_blocks) % m_blocks, b = blk / (d_blocks * m_blocks);
    const int64_t m = mb * MC + w, d0 = db * DC;
    const bool have_m = m < M;
    const int64_t ntiles = (L + W - 1) / W;
    const int64_t grow_off = (b * M + (have_m ? m : 0)) * L;
    const S *grow = gates + grow_off;
    const int64_t row0 = ((b * M + (have_m ? m : 0)) * D + d0);

    float carry[DC];
#pragma unroll
    for (int d = 0; d < DC; ++d) carry[d] = (h0 && have_m && d0 + d < D) ? h0[row0 + d] : 0.f;

    auto load_x = [&](int64_t tile, int d) -> uint4 {
        const int64_t tt = tile * W + lane * E;
        return (tile < ntiles && tt < L && d < DC && d0 + d < D)
                   ? ldg_stream(tokens + (b * D + d0 + d) * L + tt)
                   : make_uint4(0u, 0u, 0u, 0u);
    };
    auto load_g = [&](int64_t tile) -> uint4 {
        const int64_t tt = tile * W + lane * E;
        return (tile < ntiles && tt < L && have_m)
                   ? ldg_stream(grow + tt)
                   : make_uint4(Store<S>::kOne, Store<S>::kOne, Store<S>::kOne, Store<S>::kOne);
    };
    constexpr int XPW = (DC + MC - 1) / MC;
    uint4 gq = load_g(0), xq[XPW];
#pragma unroll
    for (int k = 0; k < XPW; ++k)
        if (w + k * MC < DC) xs[0][w + k * MC][lane] = load_x(0, w + k * MC);

    for (int64_t tile = 0; tile < ntiles; ++tile) {
        const int64_t t = tile * W + lane * E;
        const bool in = t < L;
        const unsigned buf = static_cast<unsigned>(tile) & 1u;
        __syncthreads();  // xs[buf] staged; previous flush done
        float fa[E], om[E], sc[E], ss[E];
        Store<S>::unpack(gq, fa);
        gq = load_g(tile + 1);
#pragma unroll
        for (int k = 0; k < XPW; ++k) xq[k] = load_x(tile + 1, w + k * MC);
#pragma unroll
        for (int i = 0; i < E; ++i) {
            sc[i] = 0.f;
            ss[i] = 0.f;
        }
        if constexpr (MODE == 1) {
            if (in && have_m) {
#pragma unroll
                for (int k = 0; k < E / 4; ++k) {
                    const float4 q4 = *reinterpret_cast<const float4 *>(scale + grow_off + t + 4 * k);
                    sc[4 * k] = q4.x;
                    sc[4 * k + 1] = q4.y;
                    sc[4 * k + 2] = q4.z;
                    sc[4 * k + 3] = q4.w;
                }
            }
        }
        float A = fa[0];
#pragma unroll
        for (int i = 1; i < E; ++i) A *= fa[i];
#pragma unroll
        for (int i = 0; i < E; ++i) om[i] = 1.f - fa[i];
        float Alvl[5];
#pragma unroll
        for (int k = 0; k < 5; ++k) {
            Alvl[k] = A;
            const float pA = __shfl_up_sync(kFullMask, A, 1 << k);
            if (lane >= (1 << k)) A *= pA;
        }
        float eA = __shfl_up_sync(kFullMask, A, 1);
        if (lane == 0) eA = 1.f;
        const float tA = __shfl_sync(kFullMask, A, 31);

#pragma unroll
        for (int d = 0; d < DC; ++d) {
            float fx[E];
            Store<S>::unpack(xs[buf][d][lane], fx);
#pragma unroll
            for (int i = 0; i < E; ++i) fx[i] *= om[i];
            float H = fx[0];
#pragma unroll
            for (int i = 1; i < E; ++i) H = fmaf(fa[i], H, fx[i]);
#pragma unroll
            for (int k = 0; k < 5; ++k) {
                const float pH = __shfl_up_sync(kFullMask, H, 1 << k);
                if (lane >= (1 << k)) H = fmaf(Alvl[k], pH, H);
            }
            float eH = __shfl_up_sync(kFullMask, H, 1);
            if (lane == 0) eH = 0.f;
            const float tH = __shfl_sync(kFullMask, H, 31);
            float s_ = fmaf(eA, carry[d], eH);
            carry[d] = fmaf(tA, carry[d], tH);
            const bool row_ok = have_m && d0 + d < D;
            float contrib[E];
#pragma unroll
            for (int i = 0; i < E; ++i) {
                s_ = fmaf(fa[i], s_, fx[i]);
                if constexpr (MODE == 0) {
                    if (row_ok) ss[i] = fmaf(s_, s_, ss[i]);
                } else {
                    contrib[i] = sc[i] * s_;  // sc is zero for lanes and gate rows outside the problem
                }
            }
            if constexpr (MODE == 1) {
#pragma unroll
                for (int k = 0; k < E / 4; ++k)
                    part[w][d][k][lane] =
                        make_float4(contrib[4 * k], contrib[4 * k + 1], contrib[4 * k + 2], contrib[4 * k + 3]);
            }
        }
        if constexpr (MODE == 0) {
            if (in && have_m) red_vec<E, false>(sumsq + grow_off, t, L, ss);
        }
#pragma unroll
        for (int k = 0; k < XPW; ++k)
            if (w + k * MC < DC) xs[buf ^ 1u][w + k * MC][lane] = xq[k];
        if constexpr (MODE == 1) {
            __syncthreads();  // every warp has published its tiles
#pragma unroll
            for (int d = w; d < DC; d += MC) {
                float v[E];
#pragma unroll
                for (int i = 0; i < E; ++i) v[i] = 0.f;
#pragma unroll
                for (int ww = 0; ww < MC; ++ww)
#pragma unroll
                    for (int k = 0; k < E / 4; ++k) {
                        const float4 p = part[ww][d][k][lane];
                        v[4 * k] += p.x;
                        v[4 * k + 1] += p.y;
                        v[4 * k + 2] += p.z;
                        v[4 * k + 3] += p.w;
                    }
                if (in && d0 + d < D) red_vec<E, false>(out32 + (b * D + d0 + d) * L, t, L, v);
            }
        }
    }
}

// scale[b,m,t] = weight[b,m,t] * rsqrt(sumsq[b,m,t] / D + eps)   (in place over sumsq)
template <typename S>
__global__ void fm_readout_scale_kernel(float *__restrict__ sumsq_to_scale, const S *__restrict__ weight,
                                        int64_t n, float inv_d, float eps, int use_norm) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) {
        const float wgt = Store<S>::to_float(weight[i]);
        sumsq_to_scale[i] = use_norm ? wgt * rsqrtf(sumsq_to_scale[i] * inv_d + eps) : wgt;
    }
}

// Dynamic shared memory fm_backward_blocked_kernel and fm_readout_blocked_kernel need.
template <typename S, int MC, int DC>
constexpr size_t fm_backward_blocked_smem() {
    return sizeof(uint4) * 2 * DC * 32 + sizeof(float4) * MC * DC * (Store<S>::E / 4) * 32;
}

}  // namespace fms
