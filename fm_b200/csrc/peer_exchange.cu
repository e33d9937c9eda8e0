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
// rank may publish exchange e+1 while a slower rank still reads e):
//   data [2 parity][2 direction][world src][2 (P, S)][rows]
//   flags[2 parity][2 direction][world src]      uint32, value = exchange number published
//   acks [2 direction][world consumer]           uint32, value = last exchange that consumer folded
//   done [2 direction]                           uint32, CTAs of the running fold that have finished
//   status                                       uint32, 0 = ok, else the code of the first fault
//
// Back-pressure: slot generation e&1 is reused by exchange e+2.  After its fold of exchange e a
// consumer stores e into its ack word in EVERY rank's buffer (peer stores); a publisher does not
// write exchange e before the ranks that read its slot have acknowledged e-2 (bounded wait on
// LOCAL ack words).  A rank therefore runs at most one exchange ahead of the slowest rank that
// reads from it, in forward-only sequences too.
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
    __host__ __device__ size_t acks_offset_bytes() const {
        return flags_offset_bytes() + static_cast<size_t>(2) * 2 * world * sizeof(uint32_t);
    }
    __host__ __device__ size_t ack_index(int dir, int consumer) const { return static_cast<size_t>(dir) * world + consumer; }
    __host__ __device__ size_t done_offset_bytes() const {
        return acks_offset_bytes() + static_cast<size_t>(2) * world * sizeof(uint32_t);
    }
    __host__ __device__ size_t status_offset_bytes() const { return done_offset_bytes() + 2 * sizeof(uint32_t); }
    __host__ __device__ size_t total_bytes() const { return (status_offset_bytes() + sizeof(uint32_t) + 255) / 256 * 256; }
};

struct Peers {
    char *buf[kMaxWorld];
};

// Ranks that read what `rank` publishes: the later blocks forward, the earlier ones in reverse.
__host__ __device__ inline void readers_of(int rank, int dir, int world, int &first, int &last) {
    first = dir == 0 ? rank + 1 : 0;
    last = dir == 0 ? world : rank;
}

// One CTA: wait (bounded, local polls) until the readers of this rank's slot have folded exchange
// epoch-2, which used the same slot generation; then copy this rank's (P, S) into slot `rank` of
// every peer's buffer, make the stores visible system-wide and raise the flag on every peer.
// If the wait runs out, FMS_PEER_ERR_ACK_TIMEOUT goes into the LOCAL status word and nothing is
// published (the slot may still be in use).
__global__ void publish_kernel(const float *__restrict__ P, const float *__restrict__ S, Peers peers, Layout lay,
                               int rank, int dir, uint32_t epoch, long long max_wait_cycles) {
    const int parity = static_cast<int>(epoch & 1u);
    __shared__ int give_up;
    if (threadIdx.x == 0) {
        give_up = 0;
        if (epoch > 2u) {
            char *local = peers.buf[rank];
            volatile uint32_t *acks = reinterpret_cast<volatile uint32_t *>(local + lay.acks_offset_bytes());
            int first, last;
            readers_of(rank, dir, lay.world, first, last);
            const long long start = clock64();
            for (int c = first; c < last && !give_up; ++c) {
                while (static_cast<int32_t>(acks[lay.ack_index(dir, c)] - (epoch - 2u)) < 0) {
                    if (clock64() - start > max_wait_cycles) {
                        give_up = 1;
                        break;
                    }
                    __nanosleep(200);
                }
            }
            if (give_up)
                atomicCAS(reinterpret_cast<uint32_t *>(local + lay.status_offset_bytes()), 0u,
                          static_cast<uint32_t>(FMS_PEER_ERR_ACK_TIMEOUT));
        }
    }
    __syncthreads();
    if (give_up) return;
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
// On a timeout, or when a slot already holds a LATER exchange than the one asked for (its data was
// overwritten: the caller broke the numbering), the status word is set, carry0 is passed through
// and the kernel still terminates normally.  The last CTA to finish acknowledges the exchange to
// every rank, which releases the slot generation for exchange epoch+2.
__global__ void wait_fold_kernel(Peers peers, Layout lay, int rank, int dir, uint32_t epoch,
                                 const float *__restrict__ carry0, float *__restrict__ carry_out,
                                 long long max_wait_cycles) {
    char *local = peers.buf[rank];
    const int parity = static_cast<int>(epoch & 1u);
    volatile uint32_t *flags = reinterpret_cast<volatile uint32_t *>(local + lay.flags_offset_bytes());
    uint32_t *status = reinterpret_cast<uint32_t *>(local + lay.status_offset_bytes());
    __shared__ int fault;
    if (threadIdx.x == 0) {
        fault = 0;
        const long long start = clock64();
        const int first = dir == 0 ? 0 : rank + 1, last = dir == 0 ? rank : lay.world;
        for (int src = first; src < last && !fault; ++src) {
            int32_t ahead;
            while ((ahead = static_cast<int32_t>(flags[lay.flag_index(parity, dir, src)] - epoch)) < 0) {
                if (clock64() - start > max_wait_cycles) {
                    fault = dir == 0 ? FMS_PEER_ERR_WAIT_TIMEOUT : FMS_PEER_ERR_WAIT_TIMEOUT_REVERSE;
                    break;
                }
                __nanosleep(200);
            }
            if (!fault && ahead > 0) fault = FMS_PEER_ERR_OVERRUN;
        }
        if (fault) atomicCAS(status, 0u, static_cast<uint32_t>(fault));
        __threadfence_system();
    }
    __syncthreads();
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r < lay.rows) {
        const float *data = reinterpret_cast<const float *>(local);
        float c = carry0 ? carry0[r] : 0.f;
        if (!fault) {
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
    // Acknowledge once every CTA of this fold has read its slots.  A fold that saw a fault does
    // not acknowledge: its publishers then stop at their own bounded wait instead of overwriting.
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t *done = reinterpret_cast<uint32_t *>(local + lay.done_offset_bytes()) + dir;
        __threadfence();
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            __threadfence();
            *done = 0;
            if (!fault && *reinterpret_cast<volatile uint32_t *>(status) == 0u) {
                for (int p = 0; p < lay.world; ++p) {
                    volatile uint32_t *acks =
                        reinterpret_cast<volatile uint32_t *>(peers.buf[p] + lay.acks_offset_bytes());
                    acks[lay.ack_index(dir, rank)] = epoch;
                }
            }
        }
    }
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

namespace {

// Clock cycles of a wait bound given in seconds (<= 30; 2 if out of range).
long long wait_cycles(double max_wait_seconds) {
    if (!(max_wait_seconds > 0.0) || max_wait_seconds > 30.0) max_wait_seconds = 2.0;
    // the clock-rate attribute is a slow driver query: ask once (all GPUs of a box are alike)
    static const int khz = []() {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, dev) != cudaSuccess ||
            v <= 0)
            v = 1965000;
        return v;
    }();
    return static_cast<long long>(max_wait_seconds * 1e3 * static_cast<double>(khz));
}

int make_peers(Peers &peers, void *const *peer_buffers, int world) {
    if (!peer_buffers) return FMS_ERR_NULL_POINTER;
    for (int p = 0; p < world; ++p) {
        if (!peer_buffers[p]) return FMS_ERR_NULL_POINTER;
        peers.buf[p] = static_cast<char *>(peer_buffers[p]);
    }
    return FMS_OK;
}

}  // namespace

FMS_EXPORT int fms_peer_publish(const float *P, const float *S, int64_t rows, void *const *peer_buffers, int world,
                                int rank, int reverse, uint32_t exchange, double max_wait_seconds,
                                fms_stream_t stream) {
    if (!layout_ok(rows, world, rank) || exchange == 0) return FMS_ERR_BAD_SHAPE;
    if (rows == 0) return FMS_OK;
    if (!P || !S) return FMS_ERR_NULL_POINTER;
    Peers peers;
    if (int rc = make_peers(peers, peer_buffers, world)) return rc;
    publish_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(P, S, peers, Layout{rows, world}, rank,
                                                                     reverse ? 1 : 0, exchange,
                                                                     wait_cycles(max_wait_seconds));
    return cudaGetLastError() == cudaSuccess ? FMS_OK : FMS_ERR_LAUNCH;
}

FMS_EXPORT int fms_peer_wait_fold(void *const *peer_buffers, const float *carry0, float *carry_out, int64_t rows,
                                  int world, int rank, int reverse, uint32_t exchange, double max_wait_seconds,
                                  fms_stream_t stream) {
    if (!layout_ok(rows, world, rank) || exchange == 0) return FMS_ERR_BAD_SHAPE;
    if (rows == 0) return FMS_OK;
    if (!carry_out) return FMS_ERR_NULL_POINTER;
    Peers peers;
    if (int rc = make_peers(peers, peer_buffers, world)) return rc;
    const int64_t blocks = (rows + 255) / 256;
    if (blocks > 0x7fffffffLL) return FMS_ERR_BAD_SHAPE;
    wait_fold_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        peers, Layout{rows, world}, rank, reverse ? 1 : 0, exchange, carry0, carry_out,
        wait_cycles(max_wait_seconds));
    return cudaGetLastError() == cudaSuccess ? FMS_OK : FMS_ERR_LAUNCH;
}
