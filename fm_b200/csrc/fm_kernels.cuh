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
// Only the big streams h and G (grad of the states) come from HBM; they are kept PD rows ahead as
// cp.async copies into a per-thread shared-memory ring (fm_backward_ring_kernel).
#pragma once

#include "scan_kernels.cuh"

namespace fms {

// 16-byte asynchronous copy global -> shared that writes zeros instead when `ok` is false (the
// source is then not read).  Completion is awaited per thread with cp.async.wait_group.
__device__ __forceinline__ void fm_cp_async16(void *smem_dst, const void *gmem_src, bool ok) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    const int bytes = ok ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fm_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void fm_cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// The backward.  The two big streams (states and their gradient) are kept PD rows ahead as 16-byte
// cp.async copies into a per-thread shared-memory ring rather than in registers: the copies are
// issued where the source says, whatever the register allocator would prefer (a register ring of
// the same depth waited on its loads for 4 of every 9 stall cycles and ran at 0.96 ms where this
// kernel needs 0.62 ms at (1,32,2048,8192) bf16), and the depth costs no registers.  A thread
// reads back only what it copied itself, so the ring needs no barrier, only the thread's own wait
// on its copy groups (one group per row).  The token tiles of the next step travel the same way,
// straight into the buffer the next step reads.
//
// Per row the lane first scans its own E positions from a zero carry (dl), the warp scans the
// lanes' aggregates, and delta_i = dl_i + q_i * c with q_i = prod_{j>i} a_j shared by the DC rows.
//
// The state just before a tile (needed by lane 0 for d_gates at the tile's first position) is not
// fetched separately: walking backwards, it is the last element of the NEXT tile this warp
// processes.  Lane 0 therefore leaves that one product out, keeps delta of the first position
// per row (`pend`), and adds  sum_d pend[d] * h_last[d]  one step later with a single scalar
// reduction per warp and step.
template <typename S, int MC, int DC, int PD>
__global__ void __launch_bounds__(MC * 32, 2)
fm_backward_ring_kernel(const S *__restrict__ gates, const S *__restrict__ tokens,
                        const S *__restrict__ states, const S *__restrict__ grad_states,
                        const float *__restrict__ h0, float *__restrict__ acc_gates,
                        float *__restrict__ acc_tokens, float *__restrict__ grad_h0, int64_t M, int64_t D,
                        int64_t L, int64_t m_blocks, int64_t d_blocks) {
    static_assert(PD >= 1 && PD < DC, "the token tiles of the next step must land within the step");
    constexpr int E = Store<S>::E;
    constexpr int W = 32 * E;  // positions per tile
    constexpr int NT = MC * 32;
    extern __shared__ __align__(16) unsigned char fm_smem[];
    uint4(*xs)[DC][32] = reinterpret_cast<uint4(*)[DC][32]>(fm_smem);  // [2][DC][32] token tiles, raw
    float4(*part)[DC][E / 4][32] =
        reinterpret_cast<float4(*)[DC][E / 4][32]>(fm_smem + sizeof(uint4) * 2 * DC * 32);  // [MC][DC][E/4][32]
    // [PD][2][NT]: slot, {gradient, state}, thread
    uint4 *ring = reinterpret_cast<uint4 *>(fm_smem + sizeof(uint4) * 2 * DC * 32 +
                                            sizeof(float4) * MC * DC * (E / 4) * 32) + threadIdx.x;
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;

    const int64_t blk = blockIdx.x;
    // m blocks vary fastest: the CTAs that add into the same d_tokens rows (and read the same token
    // tiles) run at the same time, so those reductions meet their lines in L2
    const int64_t mb = blk % m_blocks, db = (blk / m_blocks) % d_blocks, b = blk / (d_blocks * m_blocks);
    const int64_t m = mb * MC + w, d0 = db * DC;
    const bool have_m = m < M;
    const int64_t ntiles = (L + W - 1) / W;

    const S *grow = gates + (b * M + (have_m ? m : 0)) * L;
    const int64_t row0 = ((b * M + (have_m ? m : 0)) * D + d0);  // first output row of this warp
    float carry[DC], pend[DC];
#pragma unroll
    for (int d = 0; d < DC; ++d) carry[d] = pend[d] = 0.f;

    auto fetch = [&](int slot, int64_t tile, int d) {
        const int64_t t = tile * W + lane * E;
        const bool ok = have_m && tile >= 0 && d0 + d < D && t < L;
        const int64_t off = ok ? (row0 + d) * L + t : 0;
        fm_cp_async16(ring + (slot * 2) * NT, grad_states + off, ok);
        fm_cp_async16(ring + (slot * 2 + 1) * NT, states + off, ok);
        fm_cp_async_commit();
    };
    constexpr int XPW = (DC + MC - 1) / MC;  // token rows staged per warp
    auto stage_x = [&](unsigned buf, int64_t tile) {
        const int64_t tt = tile * W + lane * E;
#pragma unroll
        for (int k = 0; k < XPW; ++k) {
            const int r = w + k * MC;
            if (r < DC) {
                const bool ok = tile >= 0 && tt < L && d0 + r < D;
                fm_cp_async16(&xs[buf][r][lane], tokens + (ok ? (b * D + d0 + r) * L + tt : 0), ok);
            }
        }
    };
    auto load_g = [&](int64_t tile) -> uint4 {
        const int64_t tt = tile * W + lane * E;
        return (tile >= 0 && tt < L && have_m)
                   ? ldg_stream(grow + tt)
                   : make_uint4(Store<S>::kOne, Store<S>::kOne, Store<S>::kOne, Store<S>::kOne);
    };
    stage_x(0, ntiles - 1);
    fm_cp_async_commit();
#pragma unroll
    for (int p = 0; p < PD; ++p) fetch(p, ntiles - 1, p);
    uint4 gq = load_g(ntiles - 1);
    fm_cp_async_wait<PD>();  // the first token tiles have landed (made visible by the barrier below)

    unsigned step = 0;
    int run = 0;  // ring position when PD does not divide DC (otherwise static per row)
    for (int64_t tile = ntiles - 1; tile >= 0; --tile, ++step) {
        const int64_t t = tile * W + lane * E;  // this lane's first position
        const bool in = t < L;
        const unsigned buf = step & 1u;
        __syncthreads();  // previous step's flush is complete and xs[buf] is staged
        float fa[E];
        Store<S>::unpack(gq, fa);
        gq = load_g(tile - 1);
        stage_x(buf ^ 1u, tile - 1);  // rides in the copy group of the first row below
        // Per-lane factors shared by the DC rows: Q_i = prod_{j>i} a_j carries a later lane's
        // contribution down to element i, A = prod_j a_j is the lane's gate aggregate.
        float q[E];
        q[E - 1] = 1.f;
#pragma unroll
        for (int i = E - 2; i >= 0; --i) q[i] = q[i + 1] * fa[i + 1];
        float A = q[0] * fa[0];
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
        float defer = 0.f;

#pragma unroll
        for (int d = 0; d < DC; ++d) {
            const int slot = (DC % PD == 0) ? d % PD : run;
            if (DC % PD != 0) run = (run + 1 == PD) ? 0 : run + 1;
            float fg[E], fh[E], fx[E];
            fm_cp_async_wait<PD - 1>();  // this row's copies (the oldest group) have landed
            Store<S>::unpack(ring[(slot * 2) * NT], fg);
            Store<S>::unpack(ring[(slot * 2 + 1) * NT], fh);
            // refill the slot: PD rows ahead, wrapping into the next (earlier) tile
            if (d + PD < DC) fetch(slot, tile, d + PD);
            else fetch(slot, tile - 1, d + PD - DC);
            Store<S>::unpack(xs[buf][d][lane], fx);

            // the lane's own reverse scan from a zero carry: dl_i = G_i + a_{i+1} * dl_{i+1}
            float dl[E];
            dl[E - 1] = fg[E - 1];
#pragma unroll
            for (int i = E - 2; i >= 0; --i) dl[i] = fmaf(fa[i + 1], dl[i + 1], fg[i]);
            float C = fa[0] * dl[0];
#pragma unroll
            for (int k = 0; k < 5; ++k) {
                const float pC = __shfl_down_sync(kFullMask, C, 1 << k);
                if (lane + (1 << k) < 32) C = fmaf(Alvl[k], pC, C);
            }
            float eC = __shfl_down_sync(kFullMask, C, 1);
            if (lane == 31) eC = 0.f;
            const float tC = __shfl_sync(kFullMask, C, 0);
            // the state before this lane's vector: lane 0 receives lane 31's last state, which is
            // the one in front of the tile processed one step ago
            float hprev0 = __shfl_sync(kFullMask, fh[E - 1], (lane + 31) & 31);
            if (lane == 0) {
                defer = fmaf(pend[d], hprev0, defer);
                hprev0 = (tile == 0 && h0 && have_m && d0 + d < D) ? h0[row0 + d] : 0.f;
            }
            const float c = fmaf(eA, carry[d], eC);  // a_{t+1} * delta_{t+1} just behind this lane
            carry[d] = fmaf(tA, carry[d], tC);
            float dxv[E];  // zero for masked rows and lanes (G = 0, carry = 0 there)
#pragma unroll
            for (int i = 0; i < E; ++i) {
                const float delta = fmaf(q[i], c, dl[i]);
                const float hp = (i > 0) ? fh[i > 0 ? i - 1 : 0] : hprev0;
                dg[i] = fmaf(delta, hp - fx[i], dg[i]);
                dxv[i] = fmaf(-fa[i], delta, delta);  // (1 - a) * delta, one rounding
                if (i == 0) pend[d] = delta;
            }
#pragma unroll
            for (int k = 0; k < E / 4; ++k)
                part[w][d][k][lane] = make_float4(dxv[4 * k], dxv[4 * k + 1], dxv[4 * k + 2], dxv[4 * k + 3]);
        }
        if (in && have_m) red_vec<E, false>(acc_gates + (b * M + m) * L, t, L, dg);
        if (lane == 0 && have_m && tile + 1 < ntiles) atomicAdd(acc_gates + (b * M + m) * L + (tile + 1) * W, defer);
        __syncthreads();  // every warp has published its tiles; the next token tiles have landed
#pragma unroll
        for (int d = w; d < DC; d += MC) {
            float2 v2[E / 2];  // pairs of neighbouring positions: add.f32x2, one issue slot for two sums
#pragma unroll
            for (int k = 0; k < E / 2; ++k) v2[k] = make_float2(0.f, 0.f);
#pragma unroll
            for (int ww = 0; ww < MC; ++ww)
#pragma unroll
                for (int k = 0; k < E / 4; ++k) {
                    const float4 p = part[ww][d][k][lane];
                    v2[2 * k] = __fadd2_rn(v2[2 * k], make_float2(p.x, p.y));
                    v2[2 * k + 1] = __fadd2_rn(v2[2 * k + 1], make_float2(p.z, p.w));
                }
            float v[E];
#pragma unroll
            for (int k = 0; k < E / 2; ++k) {
                v[2 * k] = v2[k].x;
                v[2 * k + 1] = v2[k].y;
            }
            if (in && d0 + d < D) red_vec<E, false>(acc_tokens + (b * D + d0 + d) * L, t, L, v);
        }
    }
    fm_cp_async_wait<0>();
    if (grad_h0 && have_m && lane == 0) {
#pragma unroll
        for (int d = 0; d < DC; ++d)
            if (d0 + d < D) grad_h0[row0 + d] = carry[d];
    }
}

template <typename S, int MC, int DC, int PD>
constexpr size_t fm_backward_ring_smem() {
    return sizeof(uint4) * 2 * DC * 32 + sizeof(float4) * MC * DC * (Store<S>::E / 4) * 32 +
           sizeof(uint4) * PD * 2 * MC * 32;
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

        // Rows go through the scan two at a time, stage by stage, so that the shuffle chain of one
        // row covers the latency of the other's.
        constexpr int R2 = 2;
#pragma unroll
        for (int d = 0; d < DC; d += R2) {
            float fx[R2][E], H[R2];
#pragma unroll
            for (int r = 0; r < R2; ++r) {
                if (d + r < DC) Store<S>::unpack(xs[buf][d + r < DC ? d + r : 0][lane], fx[r]);
            }
#pragma unroll
            for (int r = 0; r < R2; ++r) {
#pragma unroll
                for (int i = 0; i < E; ++i) fx[r][i] *= om[i];
                H[r] = fx[r][0];
#pragma unroll
                for (int i = 1; i < E; ++i) H[r] = fmaf(fa[i], H[r], fx[r][i]);
            }
#pragma unroll
            for (int k = 0; k < 5; ++k) {
#pragma unroll
                for (int r = 0; r < R2; ++r) {
                    const float pH = __shfl_up_sync(kFullMask, H[r], 1 << k);
                    if (lane >= (1 << k)) H[r] = fmaf(Alvl[k], pH, H[r]);
                }
            }
            float eH[R2], tH[R2];
#pragma unroll
            for (int r = 0; r < R2; ++r) {
                eH[r] = __shfl_up_sync(kFullMask, H[r], 1);
                if (lane == 0) eH[r] = 0.f;
                tH[r] = __shfl_sync(kFullMask, H[r], 31);
            }
#pragma unroll
            for (int r = 0; r < R2; ++r) {
                if (d + r < DC) {
                    const int dd = d + r < DC ? d + r : 0;
                    float s_ = fmaf(eA, carry[dd], eH[r]);
                    carry[dd] = fmaf(tA, carry[dd], tH[r]);
                    float out[E];
#pragma unroll
                    for (int i = 0; i < E; ++i) {
                        s_ = fmaf(fa[i], s_, fx[r][i]);
                        out[i] = s_;
                    }
                    if (in && have_m && d0 + dd < D) stg_stream(states + (row0 + dd) * L + t, Store<S>::pack(out));
                }
            }
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
//   MODE 2: MODE 1 and the normalised states h * rnorm are written (the training forward of the
//           layer, which hands the normalised states back to the caller)
// with scale = output_weight * rsqrt(sumsq / D + eps) formed in between (or just the output
// weight when the norm is off).  Same blocking as fm_forward_blocked_kernel; HBM sees only the
// gate, token, scale and output rows -- the (B,M,D,L) tensor never exists.
template <typename S, int MC, int DC, int MODE>
__global__ void __launch_bounds__(MC * 32)
fm_readout_blocked_kernel(const S *__restrict__ gates, const S *__restrict__ tokens,
                          const float *__restrict__ h0, const float *__restrict__ scale,
                          float *__restrict__ sumsq, float *__restrict__ out32,
                          const float *__restrict__ rnorm, S *__restrict__ states_out, int64_t M,
                          int64_t D, int64_t L, int64_t m_blocks, int64_t d_blocks) {
    constexpr bool READOUT = MODE >= 1;
    constexpr bool STORE = MODE == 2;
    constexpr int E = Store<S>::E;
    constexpr int W = 32 * E;
    extern __shared__ __align__(16) unsigned char fm_smem[];
    uint4(*xs)[DC][32] = reinterpret_cast<uint4(*)[DC][32]>(fm_smem);
    float4(*part)[DC][E / 4][32] =
        reinterpret_cast<float4(*)[DC][E / 4][32]>(fm_smem + sizeof(uint4) * 2 * DC * 32);  // MODE 1 only
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const int64_t blk = blockIdx.x;
    // m blocks fastest: the CTAs that add into the same output rows run side by side (L2)
    const int64_t mb = blk % m_blocks, db = (blk / m_blocks) % d_blocks, b = blk / (d_blocks * m_blocks);
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
        float rn[STORE ? E : 1];
        if constexpr (READOUT) {
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
        if constexpr (STORE) {
#pragma unroll
            for (int i = 0; i < E; ++i) rn[i] = 1.f;
            if (rnorm && in && have_m) {
#pragma unroll
                for (int k = 0; k < E / 4; ++k) {
                    const float4 q4 = *reinterpret_cast<const float4 *>(rnorm + grow_off + t + 4 * k);
                    rn[4 * k] = q4.x;
                    rn[4 * k + 1] = q4.y;
                    rn[4 * k + 2] = q4.z;
                    rn[4 * k + 3] = q4.w;
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

        // two rows at a time, stage by stage: one row's shuffle chain covers the other's latency
        constexpr int R2 = 2;
#pragma unroll
        for (int d = 0; d < DC; d += R2) {
            float fx[R2][E], H[R2];
#pragma unroll
            for (int r = 0; r < R2; ++r)
                if (d + r < DC) Store<S>::unpack(xs[buf][d + r < DC ? d + r : 0][lane], fx[r]);
#pragma unroll
            for (int r = 0; r < R2; ++r) {
#pragma unroll
                for (int i = 0; i < E; ++i) fx[r][i] *= om[i];
                H[r] = fx[r][0];
#pragma unroll
                for (int i = 1; i < E; ++i) H[r] = fmaf(fa[i], H[r], fx[r][i]);
            }
#pragma unroll
            for (int k = 0; k < 5; ++k) {
#pragma unroll
                for (int r = 0; r < R2; ++r) {
                    const float pH = __shfl_up_sync(kFullMask, H[r], 1 << k);
                    if (lane >= (1 << k)) H[r] = fmaf(Alvl[k], pH, H[r]);
                }
            }
            float eH[R2], tH[R2];
#pragma unroll
            for (int r = 0; r < R2; ++r) {
                eH[r] = __shfl_up_sync(kFullMask, H[r], 1);
                if (lane == 0) eH[r] = 0.f;
                tH[r] = __shfl_sync(kFullMask, H[r], 31);
            }
#pragma unroll
            for (int r = 0; r < R2; ++r) {
                if (d + r < DC) {
                    const int dd = d + r < DC ? d + r : 0;
                    float s_ = fmaf(eA, carry[dd], eH[r]);
                    carry[dd] = fmaf(tA, carry[dd], tH[r]);
                    const bool row_ok = have_m && d0 + dd < D;
                    float contrib[E], hn[STORE ? E : 1];
#pragma unroll
                    for (int i = 0; i < E; ++i) {
                        s_ = fmaf(fa[i], s_, fx[r][i]);
                        if constexpr (MODE == 0) {
                            if (row_ok) ss[i] = fmaf(s_, s_, ss[i]);
                        } else {
                            contrib[i] = sc[i] * s_;  // sc is zero for lanes and gate rows outside the problem
                        }
                        if constexpr (STORE) hn[i] = s_ * rn[i];
                    }
                    if constexpr (STORE) {
                        if (in && row_ok) stg_stream(states_out + (row0 + dd) * L + t, Store<S>::pack(hn));
                    }
                    if constexpr (READOUT) {
#pragma unroll
                        for (int k = 0; k < E / 4; ++k)
                            part[w][dd][k][lane] =
                                make_float4(contrib[4 * k], contrib[4 * k + 1], contrib[4 * k + 2], contrib[4 * k + 3]);
                    }
                }
            }
        }
        if constexpr (MODE == 0) {
            if (in && have_m) red_vec<E, false>(sumsq + grow_off, t, L, ss);
        }
#pragma unroll
        for (int k = 0; k < XPW; ++k)
            if (w + k * MC < DC) xs[buf ^ 1u][w + k * MC][lane] = xq[k];
        if constexpr (READOUT) {
            __syncthreads();  // every warp has published its tiles
#pragma unroll
            for (int d = w; d < DC; d += MC) {
                float2 v2[E / 2];  // pairs of neighbouring positions: add.f32x2
#pragma unroll
                for (int k = 0; k < E / 2; ++k) v2[k] = make_float2(0.f, 0.f);
#pragma unroll
                for (int ww = 0; ww < MC; ++ww)
#pragma unroll
                    for (int k = 0; k < E / 4; ++k) {
                        const float4 p = part[ww][d][k][lane];
                        v2[2 * k] = __fadd2_rn(v2[2 * k], make_float2(p.x, p.y));
                        v2[2 * k + 1] = __fadd2_rn(v2[2 * k + 1], make_float2(p.z, p.w));
                    }
                float v[E];
#pragma unroll
                for (int k = 0; k < E / 2; ++k) {
                    v[2 * k] = v2[k].x;
                    v[2 * k + 1] = v2[k].y;
                }
                if (in && d0 + d < D) red_vec<E, false>(out32 + (b * D + d0 + d) * L, t, L, v);
            }
        }
    }
}

// scale[b,m,t] = weight[b,m,t] * rsqrt(sumsq[b,m,t] / D + eps)   (in place over sumsq)
// rnorm_out (nullable) receives the norm factor itself (kept for the layer's backward).
template <typename S>
__global__ void fm_readout_scale_kernel(float *__restrict__ sumsq_to_scale, const S *__restrict__ weight,
                                        float *__restrict__ rnorm_out, int64_t n, float inv_d, float eps,
                                        int use_norm) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) {
        const float wgt = Store<S>::to_float(weight[i]);
        const float r = use_norm ? rsqrtf(sumsq_to_scale[i] * inv_d + eps) : 1.f;
        sumsq_to_scale[i] = wgt * r;
        if (rnorm_out) rnorm_out[i] = r;
    }
}

// Dynamic shared memory fm_readout_blocked_kernel needs (token tiles and the per-warp partial tiles).
template <typename S, int MC, int DC>
constexpr size_t fm_readout_smem() {
    return sizeof(uint4) * 2 * DC * 32 + sizeof(float4) * MC * DC * (Store<S>::E / 4) * 32;
}

// ---------------------------------------------------------------- layer backward ------------
// Training backward of the layer (scan -> RMS norm over D -> read-out over M), given
//   hn   (B,M,D,L)  the normalised states the forward returned, hn = h * r,  r = rsqrt(mean_d h^2 + eps)
//   dout (B,D,L)    gradient of the layer output,  ext (B,M,D,L) optional gradient of the returned states
//   w    (B,M,L)    output weight
// With Ghn = ext + w * dout the gradient that reaches the raw states is
//   G = r * (Ghn - hn * c),   c[b,m,t] = (1/D) sum_d Ghn * hn          (c = 0 without the norm)
// and the weight gradient is dw[b,m,t] = sum_d dout * hn.
//
// Pass 1 (this kernel): the two sums over d, accumulated in registers over the CTA's DC token
// rows and reduced into fp32 (B,M,L) buffers.  No recurrence here: pure streaming of hn.
// hn (and ext) stream through a per-thread cp.async ring PD rows ahead, the dout tiles of the next
// step go straight into the buffer the next step reads (two buffers, one barrier per step).
template <typename S, int MC, int DC, int PD, bool EXT>
__global__ void __launch_bounds__(MC * 32, 3)
fm_layer_dots_kernel(const S *__restrict__ hn, const S *__restrict__ dout, const S *__restrict__ ext,
                     const S *__restrict__ weight, float *__restrict__ dotc, float *__restrict__ dw,
                     int64_t M, int64_t D, int64_t L, int64_t m_blocks, int64_t d_blocks) {
    static_assert(PD >= 1 && PD < DC, "the dout tiles of the next step must land within the step");
    constexpr int E = Store<S>::E;
    constexpr int W = 32 * E;
    constexpr int NT = MC * 32;
    constexpr int NS = EXT ? 2 : 1;
    extern __shared__ __align__(16) unsigned char fm_smem[];
    uint4(*ds)[DC][32] = reinterpret_cast<uint4(*)[DC][32]>(fm_smem);  // [2][DC][32] dout tiles
    uint4 *ring = reinterpret_cast<uint4 *>(fm_smem + sizeof(uint4) * 2 * DC * 32) + threadIdx.x;  // [PD][NS][NT]
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const int64_t blk = blockIdx.x;
    const int64_t mb = blk % m_blocks, db = (blk / m_blocks) % d_blocks, b = blk / (d_blocks * m_blocks);
    const int64_t m = mb * MC + w, d0 = db * DC;
    const bool have_m = m < M;
    const int64_t ntiles = (L + W - 1) / W;
    const int64_t grow_off = (b * M + (have_m ? m : 0)) * L;
    const int64_t row0 = ((b * M + (have_m ? m : 0)) * D + d0);

    auto fetch = [&](int slot, int64_t tile, int d) {
        const int64_t t = tile * W + lane * E;
        const bool ok = have_m && tile < ntiles && d0 + d < D && t < L;
        const int64_t off = ok ? (row0 + d) * L + t : 0;
        fm_cp_async16(ring + (slot * NS) * NT, hn + off, ok);
        if constexpr (EXT) fm_cp_async16(ring + (slot * NS + 1) * NT, ext + off, ok);
        fm_cp_async_commit();
    };
    constexpr int XPW = (DC + MC - 1) / MC;
    auto stage_d = [&](unsigned buf, int64_t tile) {
        const int64_t tt = tile * W + lane * E;
#pragma unroll
        for (int k = 0; k < XPW; ++k) {
            const int r = w + k * MC;
            if (r < DC) {
                const bool ok = tile < ntiles && tt < L && d0 + r < D;
                fm_cp_async16(&ds[buf][r][lane], dout + (ok ? (b * D + d0 + r) * L + tt : 0), ok);
            }
        }
    };
    auto load_w = [&](int64_t tile) -> uint4 {
        const int64_t tt = tile * W + lane * E;
        return (tile < ntiles && tt < L && have_m) ? ldg_stream(weight + grow_off + tt) : make_uint4(0u, 0u, 0u, 0u);
    };
    stage_d(0, 0);
    fm_cp_async_commit();
#pragma unroll
    for (int p = 0; p < PD; ++p) fetch(p, 0, p);
    uint4 wq = load_w(0);
    fm_cp_async_wait<PD>();  // the first dout tiles have landed

    int run = 0;  // ring position when PD does not divide DC (otherwise static per row)
    for (int64_t tile = 0; tile < ntiles; ++tile) {
        const int64_t t = tile * W + lane * E;
        const bool in = t < L;
        const unsigned buf = static_cast<unsigned>(tile) & 1u;
        __syncthreads();  // ds[buf] is staged; ds[buf^1] is no longer read
        float fw[E], a1[E], a2[E];
        Store<S>::unpack(wq, fw);
        wq = load_w(tile + 1);
        stage_d(buf ^ 1u, tile + 1);  // rides in the copy group of the first row below
#pragma unroll
        for (int i = 0; i < E; ++i) a1[i] = a2[i] = 0.f;
#pragma unroll
        for (int d = 0; d < DC; ++d) {
            const int slot = (DC % PD == 0) ? d % PD : run;
            if (DC % PD != 0) run = (run + 1 == PD) ? 0 : run + 1;
            float fh[E], fd[E];
            float fe[EXT ? E : 1];
            fm_cp_async_wait<PD - 1>();  // this row's copies (the oldest group) have landed
            Store<S>::unpack(ring[(slot * NS) * NT], fh);
            if constexpr (EXT) Store<S>::unpack(ring[(slot * NS + 1) * NT], fe);
            if (d + PD < DC) fetch(slot, tile, d + PD);
            else fetch(slot, tile + 1, d + PD - DC);
            Store<S>::unpack(ds[buf][d][lane], fd);
#pragma unroll
            for (int i = 0; i < E; ++i) {
                float ghn = fw[i] * fd[i];
                if constexpr (EXT) ghn += fe[i];
                a1[i] = fmaf(ghn, fh[i], a1[i]);
                a2[i] = fmaf(fd[i], fh[i], a2[i]);
            }
        }
        if (in && have_m) {
            red_vec<E, false>(dotc + grow_off, t, L, a1);
            red_vec<E, false>(dw + grow_off, t, L, a2);
        }
    }
    fm_cp_async_wait<0>();
}

template <typename S, int MC, int DC, int PD, bool EXT>
constexpr size_t fm_layer_dots_smem() {
    return sizeof(uint4) * 2 * DC * 32 + sizeof(uint4) * PD * (EXT ? 2 : 1) * MC * 32;
}

// Small per-(b,m,t) factors for pass 2, in place:  p1 = r*w,  p2 = r*c = r*dotc/D,  rinv = 1/r.
// Without the norm r = 1 and c = 0.
template <typename S>
__global__ void fm_layer_factors_kernel(const float *__restrict__ rnorm, const S *__restrict__ weight,
                                        float *__restrict__ dotc_to_p2, float *__restrict__ p1,
                                        float *__restrict__ rinv, int64_t n, float inv_d) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) {
        const float r = rnorm ? rnorm[i] : 1.f;
        p1[i] = r * Store<S>::to_float(weight[i]);
        dotc_to_p2[i] = rnorm ? r * dotc_to_p2[i] * inv_d : 0.f;
        rinv[i] = 1.f / r;
    }
}

// Pass 2: fm_backward_ring_kernel with the gradient of the raw states GENERATED per tile
//   G = p1 * dout - hn * p2 (+ r * ext)     and the raw states recovered as h = hn * rinv,
// so the only (B,M,D,L) stream read is hn (and ext when the caller used the returned states).
template <typename S, int MC, int DC, int PD, bool EXT>
__global__ void __launch_bounds__(MC * 32, 2)
fm_layer_backward_ring_kernel(const S *__restrict__ gates, const S *__restrict__ tokens,
                              const S *__restrict__ hn, const S *__restrict__ dout,
                              const S *__restrict__ ext, const float *__restrict__ p1,
                              const float *__restrict__ p2, const float *__restrict__ rinv,
                              const float *__restrict__ rnorm, const float *__restrict__ h0,
                              float *__restrict__ acc_gates, float *__restrict__ acc_tokens,
                              float *__restrict__ grad_h0, int64_t M, int64_t D, int64_t L,
                              int64_t m_blocks, int64_t d_blocks) {
    static_assert(PD >= 1 && PD < DC, "the tiles of the next step must land within the step");
    constexpr int E = Store<S>::E;
    constexpr int W = 32 * E;
    constexpr int NT = MC * 32;
    constexpr int NS = EXT ? 2 : 1;  // big streams in the ring: hn (and ext)
    extern __shared__ __align__(16) unsigned char fm_smem[];
    uint4(*xs)[DC][32] = reinterpret_cast<uint4(*)[DC][32]>(fm_smem);                        // [2] tokens
    uint4(*ds)[DC][32] = reinterpret_cast<uint4(*)[DC][32]>(fm_smem + sizeof(uint4) * 2 * DC * 32);  // [2] dout
    float4(*part)[DC][E / 4][32] =
        reinterpret_cast<float4(*)[DC][E / 4][32]>(fm_smem + sizeof(uint4) * 4 * DC * 32);
    // [PD][NS][NT]: slot, {hn, ext}, thread -- read back only by the thread that copied
    uint4 *ring = reinterpret_cast<uint4 *>(fm_smem + sizeof(uint4) * 4 * DC * 32 +
                                            sizeof(float4) * MC * DC * (E / 4) * 32) + threadIdx.x;
    // The step's fp32 factor rows p1, p2 ([2][E/4][NT] float4) travel one step ahead the same way
    // (without ext only: with it the second ring stream takes the shared memory).
    constexpr bool FACPF = !EXT;
    float4 *fac = reinterpret_cast<float4 *>(ring - threadIdx.x + PD * NS * NT) + threadIdx.x;
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const int64_t blk = blockIdx.x;
    const int64_t mb = blk % m_blocks, db = (blk / m_blocks) % d_blocks, b = blk / (d_blocks * m_blocks);
    const int64_t m = mb * MC + w, d0 = db * DC;
    const bool have_m = m < M;
    const int64_t ntiles = (L + W - 1) / W;
    const int64_t grow_off = (b * M + (have_m ? m : 0)) * L;
    const S *grow = gates + grow_off;
    const int64_t row0 = ((b * M + (have_m ? m : 0)) * D + d0);
    // delta of lane 0's first position per row, kept for one step (used by lane 0 only)
    constexpr size_t kPendOff = sizeof(uint4) * 4 * DC * 32 + sizeof(float4) * MC * DC * (E / 4) * 32 +
                                sizeof(uint4) * PD * NS * NT +
                                (EXT ? 0 : sizeof(float4) * 2 * (E / 4) * NT);  // behind the ring and the factors
    float *pend = reinterpret_cast<float *>(fm_smem + kPendOff) + w * DC;
    float carry[DC];
#pragma unroll
    for (int d = 0; d < DC; ++d) carry[d] = 0.f;
    if (lane < DC) pend[lane] = 0.f;
    __syncwarp();

    auto fetch = [&](int slot, int64_t tile, int d) {
        const int64_t t = tile * W + lane * E;
        const bool ok = have_m && tile >= 0 && d0 + d < D && t < L;
        const int64_t off = ok ? (row0 + d) * L + t : 0;
        fm_cp_async16(ring + (slot * NS) * NT, hn + off, ok);
        if constexpr (EXT) fm_cp_async16(ring + (slot * NS + 1) * NT, ext + off, ok);
        fm_cp_async_commit();
    };
    constexpr int XPW = (DC + MC - 1) / MC;
    auto stage_rows = [&](unsigned buf, int64_t tile) {  // this warp's share of the token and dout tiles
        const int64_t tt = tile * W + lane * E;
#pragma unroll
        for (int k = 0; k < XPW; ++k) {
            const int r = w + k * MC;
            if (r < DC) {
                const bool ok = tile >= 0 && tt < L && d0 + r < D;
                const int64_t off = ok ? (b * D + d0 + r) * L + tt : 0;
                fm_cp_async16(&xs[buf][r][lane], tokens + off, ok);
                fm_cp_async16(&ds[buf][r][lane], dout + off, ok);
            }
        }
    };
    auto load_g = [&](int64_t tile) -> uint4 {
        const int64_t tt = tile * W + lane * E;
        return (tile >= 0 && tt < L && have_m)
                   ? ldg_stream(grow + tt)
                   : make_uint4(Store<S>::kOne, Store<S>::kOne, Store<S>::kOne, Store<S>::kOne);
    };
    auto stage_factors = [&](int64_t tile) {
        const int64_t tt = tile * W + lane * E;
        const bool ok = tile >= 0 && tt < L && have_m;
#pragma unroll
        for (int k = 0; k < E / 4; ++k) {
            fm_cp_async16(fac + k * NT, p1 + (ok ? grow_off + tt + 4 * k : 0), ok);
            fm_cp_async16(fac + (E / 4 + k) * NT, p2 + (ok ? grow_off + tt + 4 * k : 0), ok);
        }
    };
    stage_rows(0, ntiles - 1);
    if constexpr (FACPF) stage_factors(ntiles - 1);
    fm_cp_async_commit();
#pragma unroll
    for (int p = 0; p < PD; ++p) fetch(p, ntiles - 1, p);
    uint4 gq = load_g(ntiles - 1);
    fm_cp_async_wait<PD>();  // the first token / dout tiles have landed

    auto load_f32 = [&](const float *src, int64_t t, bool ok, float fill, float (&f)[E]) {
#pragma unroll
        for (int k = 0; k < E / 4; ++k) {
            const float4 q4 = ok ? *reinterpret_cast<const float4 *>(src + grow_off + t + 4 * k)
                                 : make_float4(fill, fill, fill, fill);
            f[4 * k] = q4.x;
            f[4 * k + 1] = q4.y;
            f[4 * k + 2] = q4.z;
            f[4 * k + 3] = q4.w;
        }
    };

    unsigned step = 0;
    int run = 0;  // ring position when PD does not divide DC (otherwise static per row)
    for (int64_t tile = ntiles - 1; tile >= 0; --tile, ++step) {
        const int64_t t = tile * W + lane * E;
        const bool in = t < L;
        const unsigned buf = step & 1u;
        __syncthreads();  // previous flush complete; xs[buf], ds[buf] staged
        float fa[E], f1[E], f2[E];
        Store<S>::unpack(gq, fa);
        gq = load_g(tile - 1);
        stage_rows(buf ^ 1u, tile - 1);  // rides in the copy group of the first row below
        if constexpr (FACPF) {
            // landed with an earlier group of this thread (zeros outside the problem)
#pragma unroll
            for (int k = 0; k < E / 4; ++k) {
                const float4 a4 = fac[k * NT], b4 = fac[(E / 4 + k) * NT];
                f1[4 * k] = a4.x, f1[4 * k + 1] = a4.y, f1[4 * k + 2] = a4.z, f1[4 * k + 3] = a4.w;
                f2[4 * k] = b4.x, f2[4 * k + 1] = b4.y, f2[4 * k + 2] = b4.z, f2[4 * k + 3] = b4.w;
            }
            stage_factors(tile - 1);  // rides in the copy group of the first row below
        } else {
            load_f32(p1, t, in && have_m, 0.f, f1);
            load_f32(p2, t, in && have_m, 0.f, f2);
        }
        float frn[EXT ? E : 1];
        if constexpr (EXT) {
            if (rnorm) load_f32(rnorm, t, in && have_m, 1.f, frn);
            else {
#pragma unroll
                for (int i = 0; i < E; ++i) frn[i] = 1.f;
            }
        }
        float q[E];  // q_i = prod_{j>i} a_j
        q[E - 1] = 1.f;
#pragma unroll
        for (int i = E - 2; i >= 0; --i) q[i] = q[i + 1] * fa[i + 1];
        float A = q[0] * fa[0];
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
        // d_gates[t] = (1/r[t-1]) * sum_d delta * hn[t-1] - sum_d delta * x[t]: the raw state is
        // hn / r, and 1/r does not depend on d, so the two sums run over the NORMALISED states and
        // the tokens and 1/r is applied once per step
        float dgh[E], dgx[E];
#pragma unroll
        for (int i = 0; i < E; ++i) dgh[i] = dgx[i] = 0.f;
        float defer = 0.f;

#pragma unroll
        for (int d = 0; d < DC; ++d) {
            const int slot = (DC % PD == 0) ? d % PD : run;
            if (DC % PD != 0) run = (run + 1 == PD) ? 0 : run + 1;
            float fg[E], fh[E], fx[E], fd[E];
            float fe[EXT ? E : 1];
            fm_cp_async_wait<PD - 1>();  // this row's copies (the oldest group) have landed
            Store<S>::unpack(ring[(slot * NS) * NT], fh);  // normalised states
            if constexpr (EXT) Store<S>::unpack(ring[(slot * NS + 1) * NT], fe);
            if (d + PD < DC) fetch(slot, tile, d + PD);
            else fetch(slot, tile - 1, d + PD - DC);
            Store<S>::unpack(xs[buf][d][lane], fx);
            Store<S>::unpack(ds[buf][d][lane], fd);
#pragma unroll
            for (int i = 0; i < E; ++i) {
                float gi = fmaf(f1[i], fd[i], -fh[i] * f2[i]);  // r*w*dout - hn*r*c
                if constexpr (EXT) gi = fmaf(frn[i], fe[i], gi);
                fg[i] = gi;
            }
            // the lane's own reverse scan from a zero carry: dl_i = G_i + a_{i+1} * dl_{i+1}
            float dl[E];
            dl[E - 1] = fg[E - 1];
#pragma unroll
            for (int i = E - 2; i >= 0; --i) dl[i] = fmaf(fa[i + 1], dl[i + 1], fg[i]);
            float C = fa[0] * dl[0];
#pragma unroll
            for (int k = 0; k < 5; ++k) {
                const float pC = __shfl_down_sync(kFullMask, C, 1 << k);
                if (lane + (1 << k) < 32) C = fmaf(Alvl[k], pC, C);
            }
            float eC = __shfl_down_sync(kFullMask, C, 1);
            if (lane == 31) eC = 0.f;
            const float tC = __shfl_sync(kFullMask, C, 0);
            // normalised state before this lane's vector; lane 0 gets lane 31's last one, which
            // belongs in front of the tile processed one step ago (see fm_backward_ring_kernel).
            // At the very first position the state before is the RAW initial state (factor 1 below).
            float hprev0 = __shfl_sync(kFullMask, fh[E - 1], (lane + 31) & 31);
            if (lane == 0) {
                defer = fmaf(pend[d], hprev0, defer);
                hprev0 = (tile == 0 && h0 && have_m && d0 + d < D) ? h0[row0 + d] : 0.f;
            }
            const float c = fmaf(eA, carry[d], eC);
            carry[d] = fmaf(tA, carry[d], tC);
            float dxv[E];
#pragma unroll
            for (int i = 0; i < E; ++i) {
                const float delta = fmaf(q[i], c, dl[i]);
                const float hp = (i > 0) ? fh[i > 0 ? i - 1 : 0] : hprev0;
                dgh[i] = fmaf(delta, hp, dgh[i]);
                dgx[i] = fmaf(delta, fx[i], dgx[i]);
                dxv[i] = fmaf(-fa[i], delta, delta);  // (1 - a) * delta, one rounding
                if (i == 0 && lane == 0) pend[d] = delta;
            }
#pragma unroll
            for (int k = 0; k < E / 4; ++k)
                part[w][d][k][lane] = make_float4(dxv[4 * k], dxv[4 * k + 1], dxv[4 * k + 2], dxv[4 * k + 3]);
        }
        {
            float fri[E], dg[E];
            load_f32(rinv, t, in && have_m, 1.f, fri);
            // 1/r of the position before each element: the previous lane's last one for element 0
            // (lane 0 receives lane 31's, which is the factor of its deferred sum)
            const float rrot = __shfl_sync(kFullMask, fri[E - 1], (lane + 31) & 31);
            dg[0] = fmaf((lane == 0) ? 1.f : rrot, dgh[0], -dgx[0]);
#pragma unroll
            for (int i = 1; i < E; ++i) dg[i] = fmaf(fri[i - 1], dgh[i], -dgx[i]);
            if (in && have_m) red_vec<E, false>(acc_gates + grow_off, t, L, dg);
            if (lane == 0 && have_m && tile + 1 < ntiles)
                atomicAdd(acc_gates + grow_off + (tile + 1) * W, defer * rrot);
        }
        __syncthreads();  // every warp has published its tiles; the next token / dout tiles have landed
#pragma unroll
        for (int d = w; d < DC; d += MC) {
            float2 v2[E / 2];  // pairs of neighbouring positions: add.f32x2
#pragma unroll
            for (int k = 0; k < E / 2; ++k) v2[k] = make_float2(0.f, 0.f);
#pragma unroll
            for (int ww = 0; ww < MC; ++ww)
#pragma unroll
                for (int k = 0; k < E / 4; ++k) {
                    const float4 p = part[ww][d][k][lane];
                    v2[2 * k] = __fadd2_rn(v2[2 * k], make_float2(p.x, p.y));
                    v2[2 * k + 1] = __fadd2_rn(v2[2 * k + 1], make_float2(p.z, p.w));
                }
            float v[E];
#pragma unroll
            for (int k = 0; k < E / 2; ++k) {
                v[2 * k] = v2[k].x;
                v[2 * k + 1] = v2[k].y;
            }
            if (in && d0 + d < D) red_vec<E, false>(acc_tokens + (b * D + d0 + d) * L, t, L, v);
        }
    }
    fm_cp_async_wait<0>();
    if (grad_h0 && have_m && lane == 0) {
#pragma unroll
        for (int d = 0; d < DC; ++d)
            if (d0 + d < D) grad_h0[row0 + d] = carry[d];
    }
}

template <typename S, int MC, int DC, int PD, bool EXT>
constexpr size_t fm_layer_backward_smem() {
    return sizeof(uint4) * 4 * DC * 32 + sizeof(float4) * MC * DC * (Store<S>::E / 4) * 32 +
           sizeof(uint4) * PD * (EXT ? 2 : 1) * MC * 32 +
           (EXT ? 0 : sizeof(float4) * 2 * (Store<S>::E / 4) * MC * 32) + sizeof(float) * MC * DC;
}

}  // namespace fms
