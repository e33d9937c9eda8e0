// Host-buffer pipeline: blocks of rows stream host -> device -> kernels -> host on three streams.
// Declared in include/fm_scan_b200.h.  Allocates no device memory (staging is the caller's).
#include <cuda_runtime.h>

#include <algorithm>
#include <new>

#include "fm_scan_b200.h"

#define FMS_EXPORT extern "C" __attribute__((visibility("default")))

struct fms_pipeline {
    int device = -1;
    char *workspace = nullptr;
    size_t workspace_bytes = 0;
    cudaStream_t s_in = nullptr, s_compute = nullptr, s_out = nullptr;
    cudaEvent_t start = nullptr, done_in = nullptr, done_compute = nullptr, done_out = nullptr;
    cudaEvent_t in_ready[2] = {}, in_free[2] = {}, out_ready[2] = {}, out_free[2] = {};
};

namespace {

constexpr size_t kAlign = 256;
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline size_t elem_size(int dtype) { return dtype == FMS_F32 ? 4 : 2; }
inline bool dtype_ok(int dtype) { return dtype == FMS_F32 || dtype == FMS_F16 || dtype == FMS_BF16; }

#define FMS_CUDA(call)                                  \
    do {                                                \
        cudaError_t e_ = (call);                        \
        if (e_ != cudaSuccess) return FMS_ERR_LAUNCH;   \
    } while (0)

int destroy(fms_pipeline *p) {
    if (!p) return FMS_OK;
    int rc = FMS_OK;
    auto ev = [&](cudaEvent_t e) { if (e && cudaEventDestroy(e) != cudaSuccess) rc = FMS_ERR_LAUNCH; };
    auto st = [&](cudaStream_t s) { if (s && cudaStreamDestroy(s) != cudaSuccess) rc = FMS_ERR_LAUNCH; };
    ev(p->start); ev(p->done_in); ev(p->done_compute); ev(p->done_out);
    for (int i = 0; i < 2; ++i) { ev(p->in_ready[i]); ev(p->in_free[i]); ev(p->out_ready[i]); ev(p->out_free[i]); }
    st(p->s_in); st(p->s_compute); st(p->s_out);
    delete p;
    return rc;
}

}  // namespace

FMS_EXPORT size_t fms_pipeline_workspace_bytes(int64_t rows_per_block, int64_t T, int dtype) {
    if (rows_per_block <= 0 || T <= 0 || !dtype_ok(dtype)) return 0;
    return 12 * round_up(static_cast<size_t>(rows_per_block) * static_cast<size_t>(T) * elem_size(dtype), kAlign);
}

FMS_EXPORT int fms_pipeline_create(fms_pipeline **out, void *workspace, size_t workspace_bytes) {
    if (!out) return FMS_ERR_NULL_POINTER;
    *out = nullptr;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & (kAlign - 1)) || workspace_bytes < 12 * kAlign)
        return FMS_ERR_WORKSPACE;
    fms_pipeline *p = new (std::nothrow) fms_pipeline();
    if (!p) return FMS_ERR_LAUNCH;
    p->workspace = static_cast<char *>(workspace);
    p->workspace_bytes = workspace_bytes;
    bool ok = cudaGetDevice(&p->device) == cudaSuccess;
    auto mk_stream = [&](cudaStream_t *s) { ok = ok && cudaStreamCreateWithFlags(s, cudaStreamNonBlocking) == cudaSuccess; };
    auto mk_event = [&](cudaEvent_t *e) { ok = ok && cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess; };
    mk_stream(&p->s_in); mk_stream(&p->s_compute); mk_stream(&p->s_out);
    mk_event(&p->start); mk_event(&p->done_in); mk_event(&p->done_compute); mk_event(&p->done_out);
    for (int i = 0; i < 2; ++i) {
        mk_event(&p->in_ready[i]); mk_event(&p->in_free[i]);
        mk_event(&p->out_ready[i]); mk_event(&p->out_free[i]);
    }
    if (!ok) {
        destroy(p);
        return FMS_ERR_LAUNCH;
    }
    *out = p;
    return FMS_OK;
}

FMS_EXPORT int fms_pipeline_destroy(fms_pipeline *pipe) { return destroy(pipe); }

namespace {

// kernels = false: the copies and their ordering only (what the PCIe links allow on their own).
int run_pipeline(fms_pipeline *p, const void *gates_h, const void *tokens_h, const void *grad_states_h,
                 void *states_h, void *grad_gates_h, void *grad_tokens_h, int64_t rows, int64_t T, int dtype,
                 fms_stream_t stream, bool kernels) {
    if (!p) return FMS_ERR_NULL_POINTER;
    if (!dtype_ok(dtype)) return FMS_ERR_BAD_DTYPE;
    if (rows < 0 || T < 0) return FMS_ERR_BAD_SHAPE;
    if (rows == 0 || T == 0) return FMS_OK;
    if (!gates_h || !tokens_h || !grad_states_h || !states_h || !grad_gates_h || !grad_tokens_h)
        return FMS_ERR_NULL_POINTER;
    const size_t row_bytes = static_cast<size_t>(T) * elem_size(dtype);
    // Largest block whose 12 staging buffers fit; buffers start on 256-byte boundaries.
    int64_t block_rows = static_cast<int64_t>((p->workspace_bytes / 12 / kAlign * kAlign) / row_bytes);
    if (block_rows < 1) return FMS_ERR_WORKSPACE;
    block_rows = std::min(block_rows, rows);
    // Many blocks keep the fill (first block on its way in) and the drain (last block on its way
    // out) short against the steady state in which both copy directions run at once.
    constexpr int64_t kBlocks = 32, kMinBlockRows = 64;
    if (rows >= kBlocks * kMinBlockRows && block_rows > rows / kBlocks) block_rows = (rows + kBlocks - 1) / kBlocks;
    else if (rows >= 8 && block_rows > rows / 8) block_rows = (rows + 7) / 8;
    const size_t slot = round_up(static_cast<size_t>(block_rows) * row_bytes, kAlign);
    char *in_buf[2][3], *out_buf[2][3];
    for (int s = 0; s < 2; ++s)
        for (int k = 0; k < 3; ++k) {
            in_buf[s][k] = p->workspace + (static_cast<size_t>(s) * 3 + k) * slot;
            out_buf[s][k] = p->workspace + (6 + static_cast<size_t>(s) * 3 + k) * slot;
        }
    cudaStream_t user = static_cast<cudaStream_t>(stream);
    FMS_CUDA(cudaEventRecord(p->start, user));
    FMS_CUDA(cudaStreamWaitEvent(p->s_in, p->start, 0));
    FMS_CUDA(cudaStreamWaitEvent(p->s_compute, p->start, 0));
    FMS_CUDA(cudaStreamWaitEvent(p->s_out, p->start, 0));

    const char *src[3] = {static_cast<const char *>(gates_h), static_cast<const char *>(tokens_h),
                          static_cast<const char *>(grad_states_h)};
    char *dst[3] = {static_cast<char *>(states_h), static_cast<char *>(grad_gates_h),
                    static_cast<char *>(grad_tokens_h)};
    int64_t b = 0;
    for (int64_t r0 = 0; r0 < rows; r0 += block_rows, ++b) {
        const int s = static_cast<int>(b & 1);
        const int64_t nr = std::min(block_rows, rows - r0);
        const size_t off = static_cast<size_t>(r0) * row_bytes, bytes = static_cast<size_t>(nr) * row_bytes;
        // host -> device
        if (b >= 2) FMS_CUDA(cudaStreamWaitEvent(p->s_in, p->in_free[s], 0));
        for (int k = 0; k < 3; ++k)
            FMS_CUDA(cudaMemcpyAsync(in_buf[s][k], src[k] + off, bytes, cudaMemcpyHostToDevice, p->s_in));
        FMS_CUDA(cudaEventRecord(p->in_ready[s], p->s_in));
        // kernels
        FMS_CUDA(cudaStreamWaitEvent(p->s_compute, p->in_ready[s], 0));
        if (b >= 2) FMS_CUDA(cudaStreamWaitEvent(p->s_compute, p->out_free[s], 0));
        if (kernels) {
            int rc = fms_plain_forward(in_buf[s][0], in_buf[s][1], nullptr, out_buf[s][0], nullptr, nr, T, dtype,
                                       p->s_compute);
            if (rc != FMS_OK) return rc;
            rc = fms_plain_backward(in_buf[s][0], out_buf[s][0], in_buf[s][2], nullptr, nullptr, out_buf[s][1],
                                    out_buf[s][2], nullptr, nr, T, dtype, p->s_compute);
            if (rc != FMS_OK) return rc;
        }
        FMS_CUDA(cudaEventRecord(p->in_free[s], p->s_compute));
        FMS_CUDA(cudaEventRecord(p->out_ready[s], p->s_compute));
        // device -> host
        FMS_CUDA(cudaStreamWaitEvent(p->s_out, p->out_ready[s], 0));
        for (int k = 0; k < 3; ++k)
            FMS_CUDA(cudaMemcpyAsync(dst[k] + off, out_buf[s][k], bytes, cudaMemcpyDeviceToHost, p->s_out));
        FMS_CUDA(cudaEventRecord(p->out_free[s], p->s_out));
    }
    FMS_CUDA(cudaEventRecord(p->done_in, p->s_in));
    FMS_CUDA(cudaEventRecord(p->done_compute, p->s_compute));
    FMS_CUDA(cudaEventRecord(p->done_out, p->s_out));
    FMS_CUDA(cudaStreamWaitEvent(user, p->done_in, 0));
    FMS_CUDA(cudaStreamWaitEvent(user, p->done_compute, 0));
    FMS_CUDA(cudaStreamWaitEvent(user, p->done_out, 0));
    return FMS_OK;
}

}  // namespace

FMS_EXPORT int fms_plain_forward_backward_host(fms_pipeline *p, const void *gates_h, const void *tokens_h,
                                               const void *grad_states_h, void *states_h,
                                               void *grad_gates_h, void *grad_tokens_h, int64_t rows,
                                               int64_t T, int dtype, fms_stream_t stream) {
    return run_pipeline(p, gates_h, tokens_h, grad_states_h, states_h, grad_gates_h, grad_tokens_h, rows, T, dtype,
                        stream, true);
}

FMS_EXPORT int fms_pipeline_copy_probe(fms_pipeline *p, const void *gates_h, const void *tokens_h,
                                       const void *grad_states_h, void *states_h, void *grad_gates_h,
                                       void *grad_tokens_h, int64_t rows, int64_t T, int dtype,
                                       fms_stream_t stream) {
    return run_pipeline(p, gates_h, tokens_h, grad_states_h, states_h, grad_gates_h, grad_tokens_h, rows, T, dtype,
                        stream, false);
}
