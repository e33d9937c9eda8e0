// Thin torch C++ extension over the C ABI (include/fm_scan_b200.h).
//
// It exports the two functions the reference binds into Python (fm/scan/fm_scan.py:8-16,34-35)
// with the same names, argument order and conventions:
//   at::Tensor fm_scan_forward (gates, tokens, initial_state, out)         fm/scan/fm_scan.cuh:344-358
//   void       fm_scan_backward(gates, outGrad, firstPropGrad, tokenGradOut,
//                               cached_output, input_tokens, gateGradOut)  fm/scan/fm_scan.cuh:361-381
// Every tensor, outputs included, is allocated by the caller; failures surface as c10::Error
// (RuntimeError in Python) exactly like the reference's TORCH_CHECKs.  Unlike the reference it
// installs a device guard, launches on the current stream of the tensors' device, and checks
// the launch.
//
// Layout: all big tensors are (B, D, T) -- one independent scan per (b, d) row -- or, when the
// output has one more axis than the gates, the reference's own FM layout
// gates (B,M,L) x tokens (B,D,L) -> states (B,M,D,L) with the 1 - gate token weight.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "fm_scan_b200.h"

namespace {

int dtype_tag(const at::Tensor &t) {
    switch (t.scalar_type()) {
        case at::ScalarType::Float: return FMS_F32;
        case at::ScalarType::Half: return FMS_F16;
        case at::ScalarType::BFloat16: return FMS_BF16;
        default:
            TORCH_CHECK(false, "Unsupported tensor dtype: expecting bfloat16, float16 or float32");
    }
}

void check_status(int rc, const char *what) {
    TORCH_CHECK(rc == FMS_OK, what, " failed: ", fms_status_string(rc), " (status ", rc,
                ", cuda error ", fms_last_cuda_error(), ")");
}

void check_big(const at::Tensor &t, const at::Tensor &like, const char *name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(t.scalar_type() == like.scalar_type(), name, " must have the dtype of gates");
    TORCH_CHECK(t.device() == like.device(), name, " must be on the device of gates");
    TORCH_CHECK(t.sizes() == like.sizes(), name, " must have the shape of gates");
}

// Per-row fp32 carry vector from an optional tensor of `rows` elements (any float dtype).
// Returns an fp32 contiguous tensor (possibly the argument itself) or an undefined tensor.
at::Tensor carry_f32(const c10::optional<at::Tensor> &t, int64_t rows, const at::Tensor &like,
                     const char *name) {
    if (!t.has_value() || !t->defined() || t->numel() == 0) return at::Tensor();
    TORCH_CHECK(t->is_cuda() && t->device() == like.device(), name, " must be on the device of gates");
    TORCH_CHECK(t->numel() == rows, name, " must have one element per row (", rows, "), got ",
                t->numel());
    return t->to(at::kFloat).contiguous();
}

const float *fptr(const at::Tensor &t) { return t.defined() ? t.data_ptr<float>() : nullptr; }


int64_t rows_of_shape(const at::Tensor &t) {
    int64_t r = 1;
    for (int64_t i = 0; i + 1 < t.dim(); ++i) r *= t.size(i);
    return r;
}

}  // namespace

// Forward.  gates, tokens, out: (..., T) of one dtype; initial_state: (...), None or empty (= zeros,
// which is what fm/scan/fm_scan.py:48 passes by default).  Returns `out`.
// FM mode (the reference's own shapes): gates (B,M,L), tokens (B,D,L), initial_state (B,M,D) or
// empty, out (B,M,D,L).  Selected when `out` has one more axis than `gates`.
static at::Tensor fm_mode_forward(const at::Tensor &gates, const at::Tensor &tokens,
                                  const c10::optional<at::Tensor> &initial_state, const at::Tensor &out) {
    TORCH_CHECK(gates.dim() == 3 && tokens.dim() == 3 && out.dim() == 4,
                "FM mode expects gates (B,M,L), tokens (B,D,L), out (B,M,D,L)");
    const int64_t B = gates.size(0), M = gates.size(1), L = gates.size(2), D = tokens.size(1);
    TORCH_CHECK(tokens.size(0) == B && tokens.size(2) == L, "tokens must be (B,D,L) with the B and L of gates");
    TORCH_CHECK(out.size(0) == B && out.size(1) == M && out.size(2) == D && out.size(3) == L,
                "out must be (B,M,D,L)");
    for (const at::Tensor *t : {&tokens, &out}) {
        TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == gates.scalar_type() &&
                        t->device() == gates.device(),
                    "tokens and out must be contiguous CUDA tensors with the dtype and device of gates");
    }
    const int dtype = dtype_tag(gates);
    const c10::cuda::CUDAGuard guard(gates.device());
    at::Tensor h0 = carry_f32(initial_state, B * M * D, gates, "initial_state");
    check_status(fms_fm_forward(gates.data_ptr(), tokens.data_ptr(), fptr(h0), out.data_ptr(), B, M, D, L, dtype,
                                at::cuda::getCurrentCUDAStream().stream()),
                 "fm_scan_forward");
    return out;
}

at::Tensor fm_scan_forward(const at::Tensor &gates, const at::Tensor &tokens,
                           const c10::optional<at::Tensor> &initial_state, const at::Tensor &out) {
    TORCH_CHECK(gates.is_cuda(), "gates must be a CUDA tensor");
    TORCH_CHECK(gates.is_contiguous(), "gates must be contiguous");
    if (out.dim() == gates.dim() + 1) return fm_mode_forward(gates, tokens, initial_state, out);
    check_big(tokens, gates, "tokens");
    check_big(out, gates, "out");
    const int dtype = dtype_tag(gates);
    const int64_t rows = rows_of_shape(gates), T = gates.size(-1);
    const c10::cuda::CUDAGuard guard(gates.device());
    at::Tensor h0 = carry_f32(initial_state, rows, gates, "initial_state");
    auto stream = at::cuda::getCurrentCUDAStream().stream();
    // A handful of very long rows: cut them into segments so the whole GPU works (needs scratch).
    const size_t scratch = fms_plain_split_recommended(rows, T, dtype) ? fms_plain_split_workspace_bytes(rows, T, dtype) : 0;
    if (scratch > 0) {
        at::Tensor ws = at::empty({static_cast<int64_t>(scratch)}, gates.options().dtype(at::kByte));
        check_status(fms_plain_forward_split(gates.data_ptr(), tokens.data_ptr(), fptr(h0), out.data_ptr(),
                                             nullptr, rows, T, dtype, ws.data_ptr(), scratch, stream),
                     "fm_scan_forward");
        return out;
    }
    check_status(fms_plain_forward(gates.data_ptr(), tokens.data_ptr(), fptr(h0), out.data_ptr(),
                                   nullptr, rows, T, dtype, stream),
                 "fm_scan_forward");
    return out;
}

// Backward with every carry exposed.
//   carry_in           (...) or empty: a_T*delta_T entering from beyond the block (the reference's
//                      firstPropGrad, fm/scan/fm_scan.cuh:120-122)
//   initial_state      (...) or empty: the forward h0, i.e. h_{-1} for grad_gates at t = 0
//   grad_initial_state (...) fp32 or empty: receives dL/dh0
void fm_scan_backward_ex(const at::Tensor &gates, const at::Tensor &outGrad,
                         const c10::optional<at::Tensor> &carry_in, const at::Tensor &tokenGradOut,
                         const at::Tensor &cached_output, const at::Tensor &gateGradOut,
                         const c10::optional<at::Tensor> &initial_state,
                         const c10::optional<at::Tensor> &grad_initial_state_opt) {
    TORCH_CHECK(gates.is_cuda(), "gates must be a CUDA tensor");
    TORCH_CHECK(gates.is_contiguous(), "gates must be contiguous");
    check_big(outGrad, gates, "outGrad");
    check_big(cached_output, gates, "cached_output");
    check_big(tokenGradOut, gates, "tokenGradOut");
    check_big(gateGradOut, gates, "gateGradOut");
    const int dtype = dtype_tag(gates);
    const int64_t rows = rows_of_shape(gates), T = gates.size(-1);
    const c10::cuda::CUDAGuard guard(gates.device());
    at::Tensor cin = carry_f32(carry_in, rows, gates, "firstPropGrad");
    at::Tensor h0 = carry_f32(initial_state, rows, gates, "initial_state");
    float *gh0 = nullptr;
    const at::Tensor grad_initial_state =
        grad_initial_state_opt.has_value() ? *grad_initial_state_opt : at::Tensor();
    if (grad_initial_state.defined() && grad_initial_state.numel() > 0) {
        TORCH_CHECK(grad_initial_state.is_cuda() && grad_initial_state.is_contiguous() &&
                        grad_initial_state.scalar_type() == at::kFloat &&
                        grad_initial_state.numel() == rows,
                    "grad_initial_state must be a contiguous fp32 CUDA tensor with one element per row");
        gh0 = grad_initial_state.data_ptr<float>();
    }
    auto stream = at::cuda::getCurrentCUDAStream().stream();
    const size_t scratch = fms_plain_split_recommended(rows, T, dtype) ? fms_plain_split_workspace_bytes(rows, T, dtype) : 0;
    if (scratch > 0) {
        at::Tensor ws = at::empty({static_cast<int64_t>(scratch)}, gates.options().dtype(at::kByte));
        check_status(fms_plain_backward_split(gates.data_ptr(), cached_output.data_ptr(), outGrad.data_ptr(),
                                              fptr(h0), fptr(cin), gateGradOut.data_ptr(),
                                              tokenGradOut.data_ptr(), gh0, rows, T, dtype, ws.data_ptr(),
                                              scratch, stream),
                     "fm_scan_backward");
        return;
    }
    check_status(fms_plain_backward(gates.data_ptr(), cached_output.data_ptr(), outGrad.data_ptr(),
                                    fptr(h0), fptr(cin), gateGradOut.data_ptr(),
                                    tokenGradOut.data_ptr(), gh0, rows, T, dtype, stream),
                 "fm_scan_backward");
}

// FM-mode backward.  tokenGradOut (B,D,L), gateGradOut (B,M,L): the reductions are fused -- the
// shapes the reference's Python reaches only after materialising two (B,M,D,L) tensors and summing
// them (fm/scan/fm_scan.py:70-78).  tokenGradOut, gateGradOut both (B,M,D,L): the reference's own
// contract, per-row terms for a caller that sums them itself.  initial_state is the forward h0;
// grad_initial_state (B,M,D) fp32.
void fm_scan_backward_fm(const at::Tensor &gates, const at::Tensor &outGrad, const at::Tensor &tokenGradOut,
                         const at::Tensor &cached_output, const at::Tensor &input_tokens,
                         const at::Tensor &gateGradOut, const c10::optional<at::Tensor> &initial_state,
                         const c10::optional<at::Tensor> &grad_initial_state_opt) {
    TORCH_CHECK(gates.is_cuda() && gates.is_contiguous() && gates.dim() == 3, "gates must be a contiguous CUDA (B,M,L) tensor");
    TORCH_CHECK(input_tokens.dim() == 3 && cached_output.dim() == 4, "expected tokens (B,D,L) and states (B,M,D,L)");
    const int64_t B = gates.size(0), M = gates.size(1), L = gates.size(2), D = input_tokens.size(1);
    auto same = [&](const at::Tensor &t, at::IntArrayRef shape, const char *name) {
        TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == gates.scalar_type() &&
                        t.device() == gates.device() && t.sizes() == shape,
                    name, " must be a contiguous CUDA tensor of shape ", shape, " with the dtype of gates");
    };
    same(input_tokens, {B, D, L}, "input_tokens");
    same(cached_output, {B, M, D, L}, "cached_output");
    same(outGrad, {B, M, D, L}, "outGrad");
    // (B,M,D,L) outputs: the reference's own contract -- per-row terms, summed by the caller
    // (fm/scan/fm_scan.py:70-78); reduced shapes: the sums are fused into the kernel.
    const bool unreduced = tokenGradOut.dim() == 4 && gateGradOut.dim() == 4;
    if (unreduced) {
        same(tokenGradOut, {B, M, D, L}, "tokenGradOut");
        same(gateGradOut, {B, M, D, L}, "gateGradOut");
    } else {
        same(tokenGradOut, {B, D, L}, "tokenGradOut (fused reduction over M)");
        same(gateGradOut, {B, M, L}, "gateGradOut (fused reduction over D)");
    }
    const int dtype = dtype_tag(gates);
    const c10::cuda::CUDAGuard guard(gates.device());
    at::Tensor h0 = carry_f32(initial_state, B * M * D, gates, "initial_state");
    float *gh0 = nullptr;
    if (grad_initial_state_opt.has_value() && grad_initial_state_opt->defined() && grad_initial_state_opt->numel() > 0) {
        const at::Tensor &g = *grad_initial_state_opt;
        TORCH_CHECK(g.is_cuda() && g.is_contiguous() && g.scalar_type() == at::kFloat && g.numel() == B * M * D,
                    "grad_initial_state must be a contiguous fp32 CUDA tensor of B*M*D elements");
        gh0 = g.data_ptr<float>();
    }
    if (unreduced) {
        check_status(fms_fm_backward_unreduced(gates.data_ptr(), input_tokens.data_ptr(), cached_output.data_ptr(),
                                               outGrad.data_ptr(), fptr(h0), gateGradOut.data_ptr(),
                                               tokenGradOut.data_ptr(), gh0, B, M, D, L, dtype,
                                               at::cuda::getCurrentCUDAStream().stream()),
                     "fm_scan_backward");
        return;
    }
    const size_t scratch = fms_fm_backward_workspace_bytes(B, M, D, L, dtype);
    at::Tensor ws;
    if (scratch > 0) ws = at::empty({static_cast<int64_t>(scratch)}, gates.options().dtype(at::kByte));
    check_status(fms_fm_backward(gates.data_ptr(), input_tokens.data_ptr(), cached_output.data_ptr(),
                                 outGrad.data_ptr(), fptr(h0), gateGradOut.data_ptr(), tokenGradOut.data_ptr(),
                                 gh0, B, M, D, L, dtype, scratch ? ws.data_ptr() : nullptr, scratch,
                                 at::cuda::getCurrentCUDAStream().stream()),
                 "fm_scan_backward");
}

// Layer read-out without the states (inference): out (B,D,L) = sum_m weight * [rms-norm] * states.
// gates, weight (B,M,L); tokens, out (B,D,L); initial_state (B,M,D) or None.
void fm_memory_readout(const at::Tensor &gates, const at::Tensor &tokens, const at::Tensor &weight,
                       const c10::optional<at::Tensor> &initial_state, const at::Tensor &out, bool mem_norm,
                       double eps) {
    TORCH_CHECK(gates.is_cuda() && gates.is_contiguous() && gates.dim() == 3, "gates must be a contiguous CUDA (B,M,L) tensor");
    TORCH_CHECK(tokens.dim() == 3, "tokens must be (B,D,L)");
    const int64_t B = gates.size(0), M = gates.size(1), L = gates.size(2), D = tokens.size(1);
    auto same = [&](const at::Tensor &t, at::IntArrayRef shape, const char *name) {
        TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == gates.scalar_type() &&
                        t.device() == gates.device() && t.sizes() == shape,
                    name, " must be a contiguous CUDA tensor of shape ", shape, " with the dtype of gates");
    };
    same(tokens, {B, D, L}, "tokens");
    same(weight, {B, M, L}, "weight");
    same(out, {B, D, L}, "out");
    const int dtype = dtype_tag(gates);
    const c10::cuda::CUDAGuard guard(gates.device());
    at::Tensor h0 = carry_f32(initial_state, B * M * D, gates, "initial_state");
    const size_t scratch = fms_fm_readout_workspace_bytes(B, M, D, L, dtype);
    at::Tensor ws = at::empty({static_cast<int64_t>(std::max<size_t>(scratch, 16))}, gates.options().dtype(at::kByte));
    check_status(fms_fm_readout(gates.data_ptr(), tokens.data_ptr(), weight.data_ptr(), fptr(h0), out.data_ptr(), B,
                                M, D, L, dtype, mem_norm ? 1 : 0, static_cast<float>(eps), ws.data_ptr(), scratch,
                                at::cuda::getCurrentCUDAStream().stream()),
                 "fm_memory_readout");
}

// Training forward of the layer: writes out (B,D,L), the normalised states (B,M,D,L) and the norm
// factor rnorm (B,M,L) fp32 (ignored when mem_norm is false).
void fm_memory_forward_train(const at::Tensor &gates, const at::Tensor &tokens, const at::Tensor &weight,
                             const c10::optional<at::Tensor> &initial_state, const at::Tensor &out,
                             const at::Tensor &states_norm, const at::Tensor &rnorm, bool mem_norm, double eps) {
    TORCH_CHECK(gates.is_cuda() && gates.is_contiguous() && gates.dim() == 3 && tokens.dim() == 3,
                "gates must be a contiguous CUDA (B,M,L) tensor and tokens (B,D,L)");
    const int64_t B = gates.size(0), M = gates.size(1), L = gates.size(2), D = tokens.size(1);
    auto same = [&](const at::Tensor &t, at::IntArrayRef shape, const char *name) {
        TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == gates.scalar_type() &&
                        t.device() == gates.device() && t.sizes() == shape,
                    name, " must be a contiguous CUDA tensor of shape ", shape, " with the dtype of gates");
    };
    same(tokens, {B, D, L}, "tokens");
    same(weight, {B, M, L}, "weight");
    same(out, {B, D, L}, "out");
    same(states_norm, {B, M, D, L}, "states_norm");
    TORCH_CHECK(rnorm.is_cuda() && rnorm.is_contiguous() && rnorm.scalar_type() == at::kFloat &&
                    rnorm.numel() == B * M * L, "rnorm must be a contiguous fp32 CUDA tensor of B*M*L elements");
    const int dtype = dtype_tag(gates);
    const c10::cuda::CUDAGuard guard(gates.device());
    at::Tensor h0 = carry_f32(initial_state, B * M * D, gates, "initial_state");
    const size_t scratch = fms_fm_readout_workspace_bytes(B, M, D, L, dtype);
    at::Tensor ws = at::empty({static_cast<int64_t>(std::max<size_t>(scratch, 16))}, gates.options().dtype(at::kByte));
    check_status(fms_fm_layer_forward(gates.data_ptr(), tokens.data_ptr(), weight.data_ptr(), fptr(h0), out.data_ptr(),
                                      states_norm.data_ptr(), rnorm.data_ptr<float>(), B, M, D, L, dtype,
                                      mem_norm ? 1 : 0, static_cast<float>(eps), ws.data_ptr(), scratch,
                                      at::cuda::getCurrentCUDAStream().stream()),
                 "fm_memory_forward");
}

// Training backward of the layer.  grad_states_norm: None when the returned states were not used.
void fm_memory_backward(const at::Tensor &gates, const at::Tensor &tokens, const at::Tensor &weight,
                        const at::Tensor &states_norm, const at::Tensor &rnorm, bool mem_norm,
                        const at::Tensor &grad_out, const c10::optional<at::Tensor> &grad_states_norm,
                        const c10::optional<at::Tensor> &initial_state, const at::Tensor &d_gates,
                        const at::Tensor &d_tokens, const at::Tensor &d_weight,
                        const c10::optional<at::Tensor> &d_initial_state) {
    TORCH_CHECK(gates.is_cuda() && gates.is_contiguous() && gates.dim() == 3 && tokens.dim() == 3,
                "gates must be a contiguous CUDA (B,M,L) tensor and tokens (B,D,L)");
    const int64_t B = gates.size(0), M = gates.size(1), L = gates.size(2), D = tokens.size(1);
    auto same = [&](const at::Tensor &t, at::IntArrayRef shape, const char *name) {
        TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == gates.scalar_type() &&
                        t.device() == gates.device() && t.sizes() == shape,
                    name, " must be a contiguous CUDA tensor of shape ", shape, " with the dtype of gates");
    };
    same(tokens, {B, D, L}, "tokens");
    same(weight, {B, M, L}, "weight");
    same(states_norm, {B, M, D, L}, "states_norm");
    same(grad_out, {B, D, L}, "grad_out");
    same(d_gates, {B, M, L}, "d_gates");
    same(d_tokens, {B, D, L}, "d_tokens");
    same(d_weight, {B, M, L}, "d_weight");
    const void *ext = nullptr;
    if (grad_states_norm.has_value() && grad_states_norm->defined()) {
        same(*grad_states_norm, {B, M, D, L}, "grad_states_norm");
        ext = grad_states_norm->data_ptr();
    }
    const float *rn = nullptr;
    if (mem_norm) {
        TORCH_CHECK(rnorm.is_cuda() && rnorm.is_contiguous() && rnorm.scalar_type() == at::kFloat &&
                        rnorm.numel() == B * M * L, "rnorm must be a contiguous fp32 CUDA tensor of B*M*L elements");
        rn = rnorm.data_ptr<float>();
    }
    float *gh0 = nullptr;
    if (d_initial_state.has_value() && d_initial_state->defined() && d_initial_state->numel() > 0) {
        TORCH_CHECK(d_initial_state->is_cuda() && d_initial_state->is_contiguous() &&
                        d_initial_state->scalar_type() == at::kFloat && d_initial_state->numel() == B * M * D,
                    "d_initial_state must be a contiguous fp32 CUDA tensor of B*M*D elements");
        gh0 = d_initial_state->data_ptr<float>();
    }
    const int dtype = dtype_tag(gates);
    const c10::cuda::CUDAGuard guard(gates.device());
    at::Tensor h0 = carry_f32(initial_state, B * M * D, gates, "initial_state");
    const size_t scratch = fms_fm_layer_backward_workspace_bytes(B, M, D, L, dtype);
    at::Tensor ws = at::empty({static_cast<int64_t>(std::max<size_t>(scratch, 16))}, gates.options().dtype(at::kByte));
    check_status(fms_fm_layer_backward(gates.data_ptr(), tokens.data_ptr(), weight.data_ptr(), states_norm.data_ptr(),
                                       rn, grad_out.data_ptr(), ext, fptr(h0), d_gates.data_ptr(), d_tokens.data_ptr(),
                                       d_weight.data_ptr(), gh0, B, M, D, L, dtype, ws.data_ptr(), scratch,
                                       at::cuda::getCurrentCUDAStream().stream()),
                 "fm_memory_backward");
}

// Channel-last layout: gates, tokens, out (B, T, D); initial_state (B, D) or None.
at::Tensor fm_scan_btd_forward(const at::Tensor &gates, const at::Tensor &tokens,
                               const c10::optional<at::Tensor> &initial_state, const at::Tensor &out) {
    TORCH_CHECK(gates.is_cuda() && gates.is_contiguous() && gates.dim() == 3, "gates must be a contiguous CUDA (B,T,D) tensor");
    check_big(tokens, gates, "tokens");
    check_big(out, gates, "out");
    const int64_t B = gates.size(0), T = gates.size(1), D = gates.size(2);
    const int dtype = dtype_tag(gates);
    const c10::cuda::CUDAGuard guard(gates.device());
    at::Tensor h0 = carry_f32(initial_state, B * D, gates, "initial_state");
    const size_t scratch = fms_btd_workspace_bytes(B, T, D, dtype);
    at::Tensor ws = at::empty({static_cast<int64_t>(std::max<size_t>(scratch, 16))}, gates.options().dtype(at::kByte));
    check_status(fms_btd_forward(gates.data_ptr(), tokens.data_ptr(), fptr(h0), out.data_ptr(), nullptr, B, T, D, dtype,
                                 ws.data_ptr(), scratch, at::cuda::getCurrentCUDAStream().stream()),
                 "fm_scan_forward (B,T,D)");
    return out;
}

void fm_scan_btd_backward(const at::Tensor &gates, const at::Tensor &outGrad, const at::Tensor &tokenGradOut,
                          const at::Tensor &cached_output, const at::Tensor &gateGradOut,
                          const c10::optional<at::Tensor> &initial_state,
                          const c10::optional<at::Tensor> &grad_initial_state) {
    TORCH_CHECK(gates.is_cuda() && gates.is_contiguous() && gates.dim() == 3, "gates must be a contiguous CUDA (B,T,D) tensor");
    check_big(outGrad, gates, "outGrad");
    check_big(cached_output, gates, "cached_output");
    check_big(tokenGradOut, gates, "tokenGradOut");
    check_big(gateGradOut, gates, "gateGradOut");
    const int64_t B = gates.size(0), T = gates.size(1), D = gates.size(2);
    const int dtype = dtype_tag(gates);
    const c10::cuda::CUDAGuard guard(gates.device());
    at::Tensor h0 = carry_f32(initial_state, B * D, gates, "initial_state");
    float *gh0 = nullptr;
    if (grad_initial_state.has_value() && grad_initial_state->defined() && grad_initial_state->numel() > 0) {
        TORCH_CHECK(grad_initial_state->is_cuda() && grad_initial_state->is_contiguous() &&
                        grad_initial_state->scalar_type() == at::kFloat && grad_initial_state->numel() == B * D,
                    "grad_initial_state must be a contiguous fp32 CUDA tensor of B*D elements");
        gh0 = grad_initial_state->data_ptr<float>();
    }
    const size_t scratch = fms_btd_workspace_bytes(B, T, D, dtype);
    at::Tensor ws = at::empty({static_cast<int64_t>(std::max<size_t>(scratch, 16))}, gates.options().dtype(at::kByte));
    check_status(fms_btd_backward(gates.data_ptr(), cached_output.data_ptr(), outGrad.data_ptr(), fptr(h0),
                                  gateGradOut.data_ptr(), tokenGradOut.data_ptr(), gh0, B, T, D, dtype, ws.data_ptr(),
                                  scratch, at::cuda::getCurrentCUDAStream().stream()),
                 "fm_scan_backward (B,T,D)");
}

// Backward with the reference's seven arguments.  firstPropGrad seeds the reverse scan
// (fm/scan/fm_scan.cuh:120-122); the reference passes zeros (fm/scan/fm_scan.py:65).
// input_tokens is accepted for signature compatibility and not read: with the token weight
// dropped, grad_gates_t = delta_t * h_{t-1} needs no tokens.  h_{-1} is taken as zero, which is
// what the reference's call amounts to (its h_{-1} is firstPropGrad = zeros,
// fm/scan/fm_scan.cuh:195-196).
void fm_scan_backward(const at::Tensor &gates, const at::Tensor &outGrad,
                      const c10::optional<at::Tensor> &firstPropGrad, const at::Tensor &tokenGradOut,
                      const at::Tensor &cached_output, const c10::optional<at::Tensor> &input_tokens,
                      const at::Tensor &gateGradOut) {
    if (cached_output.dim() == gates.dim() + 1) {  // FM mode, h_{-1} = 0; outputs reduced or (B,M,D,L)
        TORCH_CHECK(input_tokens.has_value() && input_tokens->defined(), "FM mode needs input_tokens");
        fm_scan_backward_fm(gates, outGrad, tokenGradOut, cached_output, *input_tokens, gateGradOut,
                            c10::nullopt, c10::nullopt);
        return;
    }
    fm_scan_backward_ex(gates, outGrad, firstPropGrad, tokenGradOut, cached_output, gateGradOut,
                        c10::nullopt, c10::nullopt);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "fm_scan for B200: torch shim over the C ABI libfm_scan_b200.so";
    m.def("fm_scan_forward", &fm_scan_forward, "scan forward (writes and returns out)");
    m.def("fm_scan_backward", &fm_scan_backward, "scan backward, reference signature");
    m.def("fm_scan_backward_ex", &fm_scan_backward_ex, "scan backward with h0 / carry_in / grad_h0");
    m.def("fm_scan_backward_fm", &fm_scan_backward_fm, "FM-mode backward with fused reductions");
    m.def("fm_scan_btd_forward", &fm_scan_btd_forward, "scan forward on (B,T,D) tensors");
    m.def("fm_scan_btd_backward", &fm_scan_btd_backward, "scan backward on (B,T,D) tensors");
    m.def("fm_memory_forward_train", &fm_memory_forward_train, "layer forward: output + normalised states");
    m.def("fm_memory_backward", &fm_memory_backward, "layer backward with the state gradient generated in-kernel");
    m.def("fm_memory_readout", &fm_memory_readout, "layer read-out without materialising the states");
    m.def("abi_version", []() { return fms_version(); });
}
