// Carry exchange of the split-along-T scan over peer-mapped memory (NVLink / NVSwitch), without
// a collective library.  Declared in include/fm_scan_b200.h.
//
// Every rank owns one buffer that all ranks of the box have mapped (symmetric memory).  A rank
// PUBLISHES its block's carries by storing them into every peer's buffer and then raising a
// flag there; a rank CONSUMES by polling flags in its OWN memory (never a remote load in the
// wait loop), then folding the carries of the blocks before (forward) or after (backward) it.
// Only plain peer stores and local loads are used: no multicast, no multimem.
//
// Buffer layout (floats unless noted), P = parity of the exchange number (two generations, so a
// fast rank publishing exchange e+1 cannot overwrite what a slow rank still reads for e):
//   data [2 parity][2 direction][world src][2 (P, S)][rows]
//   flags[2 parity][2 direction][world src]      uint32, value = exchange number
//   status                                       uint32, 0 = ok, else a timeout was recorded
#include <cuda_runtime.h>

#include "fm_scan_b200.h"

#define FMS_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kMaxWorld = FMS_MAX_PEERS;

struct Layout {
    int64_t rows;
    int world;
    __host__ __device__ size_t data_floats() const { return static_cast<size_t>(2) * 2 * world * 2 * rows; }
    __host__ __device__ size_t data_index(int parity, int dir, int src, int which) const {
        return ((((static_cast<size_t>(parity) * 2 + dir) * world + src) * 2 + which) * rows);
    }
    __host__ __device__ size_t flag_index(int parity, int dir, int src) const {
        return (static_cast<size_t>(parity) * 2 + dir) * world + src;
    }
    __host__ __device__ size_t flags_offset_bytes() const { return (data_floats() * sizeof(float) + 255) / 256 * 256; }
    __host__ __device__ size_t status_offset_bytes() const {
        return flags_offset_bytes() + static_cast<size_t>(2) * 2 * world * sizeof(uint32_t);
    }
    __host__ __device__ size_t total_bytes() const { return (status_offset_bytes() + sizeof(uint32_t) + 255) / 256 * 256; }
};

struct Peers {
    char *buf[kMaxWorld];
};

// One CTA: copy this rank's (P, S) into slot `rank` of every peer's buffer, make the stores
// visible system-wide, then raise the flag on every peer.
__global__ void publish_kernel(const float *__restrict__ P, const float *__restrict__ S, Peers peers, Layout lay,
                               int rank, int dir, uint32_t epoch) {
    const int parity = static_cast<int>(epoch & 1u);
    const size_t iP = lay.data_index(parity, dir, rank, 0), iS = lay.data_index(parity, dir, rank, 1);
    for (int p = 0; p < lay.world; ++p) {
        float *dst = reinterpret_cast<float *>(peers.buf[p]);
        for (int64_t r = threadIdx.x; r < lay.rows; r += blockDim.x) {
            dst[iP + r] = P[r];
            dst[iS + r] = S[r];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < lay.world) {
        volatile uint32_t *flags =
            reinterpret_cast<volatile uint32_t *>(peers.buf[threadIdx.x] + lay.flags_offset_bytes());
        flags[lay.flag_index(parity, dir, rank)] = epoch;
    }
}

// Wait (bounded) for the flags of the blocks this rank depends on, then fold their carries per
// row: forward takes the blocks before `rank` in time order, backward the blocks after it.
// On a timeout the status word is set and the kernel still terminates normally.
__global__ void wait_fold_kernel(char *local, Layout lay, int rank, int dir, uint32_t epoch,
                                 const float *__restrict__ carry0, float *__restrict__ carry_out,
                                 long long max_wait_cycles) {
    const int parity = static_cast<int>(epoch & 1u);
    volatile uint32_t *flags = reinterpret_cast<volatile uint32_t *>(local + lay.flags_offset_bytes());
    uint32_t *status = reinterpret_cast<uint32_t *>(local + lay.status_offset_bytes());
    __shared__ int timed_out;
    if (threadIdx.x == 0) {
        timed_out = 0;
        const long long start = clock64();
        const int first = dir == 0 ? 0 : rank + 1, last = dir == 0 ? rank : lay.world;
        for (int src = first; src < last; ++src) {
            // flags only grow; the slot of this parity holds e, e+2, ...
            while (static_cast<int32_t>(flags[lay.flag_index(parity, dir, src)] - epoch) < 0) {
                if (clock64() - start > max_wait_cycles) {
                    timed_out = 1;
                    break;
                }
                __nanosleep(200);
            }
            if (timed_out) break;
        }
        if (timed_out) atomicExch(status, 1u + static_cast<uint32_t>(dir));
        __threadfence_system();
    }
    __syncthreads();
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r >= lay.rows) return;
    const float *data = reinterpret_cast<const float *>(local);
    float c = carry0 ? carry0[r] : 0.f;
    if (!timed_out) {
        if (dir == 0) {
            for (int src = 0; src < rank; ++src)
                c = fmaf(__ldcv(data + lay.data_index(parity, dir, src, 0) + r), c,
                         __ldcv(data + lay.data_index(parity, dir, src, 1) + r));
        } else {
            for (int src = lay.world - 1; src > rank; --src)
                c = fmaf(__ldcv(data + lay.data_index(parity, dir, src, 0) + r), c,
                         __ldcv(data + lay.data_index(parity, dir, src, 1) + r));
        }
    }
    carry_out[r] = c;
}

bool layout_ok(int64_t rows, int world, int rank) {
    return rows >= 0 && world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world;
}

}  // namespace

FMS_EXPORT size_t fms_peer_exchange_bytes(int64_t rows, int world) {
    if (!layout_ok(rows, world, 0)) return 0;
    return Layout{rows, world}.total_bytes();
}

FMS_EXPORT size_t fms_peer_exchange_status_offset(int64_t rows, int world) {
    if (!layout_ok(rows, world, 0)) return 0;
    return Layout{rows, world}.status_offset_bytes();
}

FMS_EXPORT int fms_peer_publish(const float *P, const float *S, int64_t rows, void *const *peer_buffers, int world,
                                int rank, int reverse, uint32_t exchange, fms_stream_t stream) {
    if (!layout_ok(rows, world, rank)) return FMS_ERR_BAD_SHAPE;
    if (rows == 0) return FMS_OK;
    if (!P || !S || !peer_buffers) return FMS_ERR_NULL_POINTER;
    Peers peers;
    for (int p = 0; p < world; ++p) {
        if (!peer_buffers[p]) return FMS_ERR_NULL_POINTER;
        peers.buf[p] = static_cast<char *>(peer_buffers[p]);
    }
    publish_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(P, S, peers, Layout{rows, world}, rank,
                                                                     reverse ? 1 : 0, exchange);
    return cudaGetLastError() == cudaSuccess ? FMS_OK : FMS_ERR_LAUNCH;
}

FMS_EXPORT int fms_peer_wait_fold(void *local_buffer, const float *carry0, float *carry_out, int64_t rows, int world,
                                  int rank, int reverse, uint32_t exchange, double max_wait_seconds,
                                  fms_stream_t stream) {
    if (!layout_ok(rows, world, rank)) return FMS_ERR_BAD_SHAPE;
    if (rows == 0) return FMS_OK;
    if (!local_buffer || !carry_out) return FMS_ERR_NULL_POINTER;
    if (!(max_wait_seconds > 0.0) || max_wait_seconds > 30.0) max_wait_seconds = 2.0;
    // the clock-rate attribute is a slow driver query: ask once (all GPUs of a box are alike)
    static const int khz = []() {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, dev) != cudaSuccess ||
            v <= 0)
            v = 1965000;
        return v;
    }();
    const long long cycles = static_cast<long long>(max_wait_seconds * 1e3 * static_cast<double>(khz));
    const int64_t blocks = (rows + 255) / 256;
    if (blocks > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
    wait_fold_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<char *>(local_buffer), Layout{rows, world}, rank, reverse ? 1 : 0, exchange, carry0, carry_out,
        cycles);
    return cudaGetLastError() == cudaSuccess ? FMS_OK : FMS_ERR_LAUNCH;
}
