// PyTorch operator shim over the C ABI of libmam_b200.so.
//
// Defines the same operator schemas as the reference's extension modules
//   mamtorch/kernel/v1/csrc/register_functions.cpp:21-24
//   mamtorch/kernel/v2/csrc/register_functions.cpp:28-32
//   mamtorch/kernel/v3/csrc/register_functions.cpp:30-34
//   mamtorch/kernel/v4/csrc/register_functions.cpp:10-14
//   mamtorch/sparse/kernel/v1/csrc/cuda/register_functions.cu:18-28
// so torch.ops.mamtorch_kernel_v{1,2,3,4}.* keep their names, argument order and return types,
// plus a `mamtorch_b200` namespace with the weight-as-stored ([N,K]) forms the nn modules use to
// skip the reference's per-call transposes.  Only CUDA implementations are registered: a CPU
// tensor gets the dispatcher's NotImplementedError instead of the reference's "print a warning and
// return uninitialised memory" (mamtorch/kernel/v1/csrc/fullyconnected.cpp:24-32).
// Nothing here computes: it validates, allocates outputs and workspace with the caching
// allocator, and forwards raw pointers and the current stream to the C ABI.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <vector>

#include "../../include/mam_b200.h"

namespace {

void check_status(int st, const char* what) {
    if (st == MAM_OK) return;
    if (st == MAM_ERR_CUDA) {
        TORCH_CHECK(false, what, ": ", mam_status_str(st), ": ", mam_last_cuda_error());
    }
    TORCH_CHECK(false, what, ": ", mam_status_str(st));
}

void check_matrix(const at::Tensor& t, const char* name, at::ScalarType dt = at::kFloat) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.dim() == 2, name, " must be 2-D");
    TORCH_CHECK(t.scalar_type() == dt, name, " has the wrong dtype");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

struct Fwd {
    at::Tensor y, argmax, argmin;
};

// b_layout: MAM_B_KN -> w is b[K,N]; MAM_B_NK -> w is W[N,K]
Fwd forward_impl(const at::Tensor& a, const at::Tensor& w, int b_layout, const c10::optional<at::Tensor>& bias,
                 const c10::optional<at::Tensor>& dense, bool blend, double alpha, double beta, bool want_idx,
                 double drop_rate = 0.0, int64_t drop_seed = 0) {
    check_matrix(a, "a");
    check_matrix(w, "b");
    const int64_t M = a.size(0), K = a.size(1);
    const int64_t N = b_layout == MAM_B_KN ? w.size(1) : w.size(0);
    TORCH_CHECK((b_layout == MAM_B_KN ? w.size(0) : w.size(1)) == K, "inner dimensions of a and b differ");
    TORCH_CHECK(a.device() == w.device(), "a and b must be on the same device");
    TORCH_CHECK(K > 0, "the reduction dimension must not be empty");
    c10::cuda::CUDAGuard guard(a.device());
    Fwd out;
    out.y = at::empty({M, N}, a.options());
    if (want_idx) {
        out.argmax = at::empty({M, N}, a.options().dtype(at::kInt));
        out.argmin = at::empty({M, N}, a.options().dtype(at::kInt));
    }
    if (M == 0 || N == 0) return out;
    const float* bias_p = nullptr;
    at::Tensor bias_c;
    if (bias.has_value() && bias->defined()) {
        TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kFloat && bias->numel() == N,
                    "bias must be a float CUDA tensor with one value per output");
        bias_c = bias->contiguous();
        bias_p = bias_c.data_ptr<float>();
    }
    const float* dense_p = nullptr;
    at::Tensor dense_c;
    if (dense.has_value() && dense->defined()) {
        TORCH_CHECK(dense->sizes() == out.y.sizes() && dense->scalar_type() == at::kFloat, "dense term shape");
        dense_c = dense->contiguous();
        dense_p = dense_c.data_ptr<float>();
    }
    const size_t ws_bytes = mam_fwd_workspace_bytes(M, K, N, b_layout, want_idx);
    at::Tensor ws;
    void* ws_p = nullptr;
    if (ws_bytes) {
        ws = at::empty({(int64_t)ws_bytes}, a.options().dtype(at::kByte));
        ws_p = ws.data_ptr();
    }
    auto stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(drop_rate >= 0.0 && drop_rate < 1.0, "drop_rate must be in [0, 1)");
    const int st = mam_fwd_drop_f32(a.data_ptr<float>(), w.data_ptr<float>(), b_layout, bias_p, dense_p, blend ? 1 : 0,
                                    (float)alpha, (float)beta, (float)drop_rate, (uint64_t)drop_seed,
                                    out.y.data_ptr<float>(), want_idx ? out.argmax.data_ptr<int32_t>() : nullptr,
                                    want_idx ? out.argmin.data_ptr<int32_t>() : nullptr, M, K, N, ws_p, ws_bytes,
                                    stream.stream());
    check_status(st, "mam_fwd_drop_f32");
    return out;
}

std::vector<at::Tensor> backward_impl(const at::Tensor& a, const at::Tensor& w, int b_layout, const at::Tensor& grad,
                                      const at::Tensor& argmax, const at::Tensor& argmin, double scale,
                                      bool count = false, bool da_km = false) {
    check_matrix(a, "a");
    check_matrix(w, "b");
    check_matrix(grad, "grad");
    check_matrix(argmax, "argmax", at::kInt);
    check_matrix(argmin, "argmin", at::kInt);
    const int64_t M = a.size(0), K = a.size(1);
    const int64_t N = b_layout == MAM_B_KN ? w.size(1) : w.size(0);
    TORCH_CHECK((b_layout == MAM_B_KN ? w.size(0) : w.size(1)) == K, "inner dimensions of a and b differ");
    TORCH_CHECK(grad.size(0) == M && grad.size(1) == N, "grad must be [M,N]");
    TORCH_CHECK(argmax.sizes() == grad.sizes() && argmin.sizes() == grad.sizes(), "index shapes must match grad");
    c10::cuda::CUDAGuard guard(a.device());
    auto da = da_km ? at::empty({K, M}, a.options()) : at::empty_like(a);   // da_km: gradient of a, transposed
    auto dw = at::empty_like(w);
    at::Tensor hmax, hmin;
    if (count) {
        hmax = at::zeros({N, K}, argmax.options());
        hmin = at::zeros({N, K}, argmax.options());
    }
    if (M == 0 || N == 0 || K == 0) {
        da.zero_();
        dw.zero_();
    } else {
        auto stream = at::cuda::getCurrentCUDAStream();
        // with counting: scratch for the 16-byte {dW, max hits, min hits} records, so that the hits ride on the
        // dW reductions instead of costing a second sweep over the indices
        const size_t ws_bytes = count ? mam_bwd_count_workspace_bytes(M, K, N) : 0;
        at::Tensor ws;
        if (ws_bytes) ws = at::empty({(int64_t)ws_bytes}, a.options().dtype(at::kByte));
        const int st = mam_bwd_count_ws_f32(a.data_ptr<float>(), w.data_ptr<float>(), b_layout, grad.data_ptr<float>(),
                                            argmax.data_ptr<int32_t>(), argmin.data_ptr<int32_t>(), da.data_ptr<float>(),
                                            da_km ? MAM_DA_KM : MAM_DA_MK, dw.data_ptr<float>(),
                                            count ? hmax.data_ptr<int32_t>() : nullptr,
                                            count ? hmin.data_ptr<int32_t>() : nullptr, (float)scale, M, K, N,
                                            ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, stream.stream());
        check_status(st, "mam_bwd_count_ws_f32");
    }
    if (count) return {da, dw, hmax, hmin};
    return {da, dw};
}

// ------------------------------------------------------------------ dense (sum-of-products) term
// 1: tcgen05 TF32 kernel of this library; 0: torch/cuBLAS in full fp32, what the reference computes
// (at::linalg_matmul / F.linear and its own dense.cu); -1 (default): follow torch's own switch for TF32
// matrix products (torch.backends.cuda.matmul.allow_tf32, off unless the user turned it on), so that the
// reference-named operators return full-fp32 results unless reduced precision was asked for.
int g_dense_backend = -1;

void set_dense_backend(int64_t backend) { g_dense_backend = backend < 0 ? -1 : (backend ? 1 : 0); }
int64_t get_dense_backend() { return g_dense_backend; }
bool dense_tf32_wanted() {
    if (g_dense_backend >= 0) return g_dense_backend == 1;
    return at::globalContext().allowTF32CuBLAS();
}
bool ptr16(const at::Tensor& t) { return reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0; }

// The flag a kernel of the library sets when one of its bounded waits gave up (its outputs are then invalid).
// check_device_flag synchronises the device and raises if the flag is set.  poll_device_flag does not wait:
// it raises if the copy of the flag fetched by an EARLIER poll shows a time-out, then queues the next fetch
// on the current stream -- cheap enough to sit in every module call, one call late at most.
void check_device_flag() { check_status(mam_check_device_flag(), "a kernel of mamtorch_b200"); }
void poll_device_flag() {
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_poll_device_flag(stream.stream()), "a kernel of mamtorch_b200");
}

// a[M,K] . w[N,K]^T -> [M,N]
at::Tensor dense_nt(const at::Tensor& a, const at::Tensor& w) {
    check_matrix(a, "a");
    check_matrix(w, "w");
    TORCH_CHECK(a.size(1) == w.size(1), "inner dimensions differ");
    c10::cuda::CUDAGuard guard(a.device());
    const int64_t M = a.size(0), K = a.size(1), N = w.size(0);
    const bool tf32_ok = dense_tf32_wanted() && M > 0 && N > 0 && K > 0 && K % 4 == 0 && ptr16(a) && ptr16(w);
    if (!tf32_ok) return at::matmul(a, w.t());
    auto out = at::empty({M, N}, a.options());
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_dense_tf32(a.data_ptr<float>(), w.data_ptr<float>(), out.data_ptr<float>(), 1.0f, 0.0f, M, K, N,
                                stream.stream()),
                 "mam_dense_tf32");
    return out;
}

// ------------------------------------------------------------------ reference-named operators
std::vector<at::Tensor> fullyconnected(const at::Tensor& a, const at::Tensor& b) {
    auto r = forward_impl(a, b, MAM_B_KN, c10::nullopt, c10::nullopt, false, 1.0, 0.0, true);
    return {r.y, r.argmax, r.argmin};
}
at::Tensor fullyconnected_fast(const at::Tensor& a, const at::Tensor& b) {
    return forward_impl(a, b, MAM_B_KN, c10::nullopt, c10::nullopt, false, 1.0, 0.0, false).y;
}
std::vector<at::Tensor> fullyconnected_backward(const at::Tensor& a, const at::Tensor& b, const at::Tensor& grad,
                                                const at::Tensor& argmax, const at::Tensor& argmin) {
    return backward_impl(a, b, MAM_B_KN, grad, argmax, argmin, 1.0);
}

// v2/v3: C = (1-beta)*mam + beta*(a.b) + bias  (mamtorch/kernel/v3/csrc/cuda/fullyconnected.cu:153-160)
at::Tensor dense(const at::Tensor& a, const at::Tensor& b) {
    check_matrix(a, "a");
    check_matrix(b, "b");
    TORCH_CHECK(a.size(1) == b.size(0), "inner dimensions differ");
    if (!dense_tf32_wanted()) return at::matmul(a, b);
    return dense_nt(a, b.t().contiguous());
}
// The K-contiguous copy of b serves both the tensor-core product and the MAM kernels, so the
// blended operators transpose once instead of once per kernel.
Fwd blended_impl(const at::Tensor& a, const at::Tensor& b, const at::Tensor& bias, double beta, bool want_idx) {
    check_matrix(a, "a");
    check_matrix(b, "b");
    TORCH_CHECK(a.size(1) == b.size(0), "inner dimensions of a and b differ");
    if (beta == 0.0) return forward_impl(a, b, MAM_B_KN, bias, c10::nullopt, true, 1.0, 0.0, want_idx);
    auto bt = b.t().contiguous();  // W[N,K]
    c10::optional<at::Tensor> d = dense_nt(a, bt);
    return forward_impl(a, bt, MAM_B_NK, bias, d, true, 1.0 - beta, beta, want_idx);
}
std::vector<at::Tensor> fullyconnected_beta(const at::Tensor& a, const at::Tensor& b, const at::Tensor& bias,
                                            double beta) {
    auto r = blended_impl(a, b, bias, beta, true);
    return {r.y, r.argmax, r.argmin};
}
at::Tensor fullyconnected_fast_beta(const at::Tensor& a, const at::Tensor& b, const at::Tensor& bias, double beta) {
    return blended_impl(a, b, bias, beta, false).y;
}
// (mamtorch/kernel/v3/csrc/cuda/fullyconnected_backward.cu:138-145)
std::vector<at::Tensor> fullyconnected_backward_beta(const at::Tensor& a, const at::Tensor& b, const at::Tensor& grad,
                                                     const at::Tensor& argmax, const at::Tensor& argmin, double beta) {
    auto r = backward_impl(a, b, MAM_B_KN, grad, argmax, argmin, 1.0 - beta);
    if (beta != 0.0) {
        const int64_t M = a.size(0), K = a.size(1), N = b.size(1);
        bool tf32_ok = dense_tf32_wanted() && M % 4 == 0 && N % 4 == 0 && K % 4 == 0 && M > 0 && N > 0 && K > 0 &&
                       ptr16(grad) && ptr16(b) && ptr16(r[0]) && ptr16(r[1]);
        at::Tensor at_, gt;
        if (tf32_ok) {
            at_ = a.t().contiguous();
            gt = grad.t().contiguous();
            tf32_ok = ptr16(at_) && ptr16(gt);
        }
        if (tf32_ok) {
            // da[M,K] += beta * grad[M,N] . b[K,N]^T      (reduction over N: both operands N-contiguous)
            // db[K,N] += beta * a^T[K,M] . grad^T[N,M]^T  (reduction over M: transposed copies)
            auto stream = at::cuda::getCurrentCUDAStream();
            check_status(mam_dense_tf32(grad.data_ptr<float>(), b.data_ptr<float>(), r[0].data_ptr<float>(),
                                        (float)beta, 1.0f, M, N, K, stream.stream()),
                         "mam_dense_tf32");
            check_status(mam_dense_tf32(at_.data_ptr<float>(), gt.data_ptr<float>(), r[1].data_ptr<float>(),
                                        (float)beta, 1.0f, K, M, N, stream.stream()),
                         "mam_dense_tf32");
        } else {
            r[0].addmm_(grad, b.t(), 1.0, beta);
            r[1].addmm_(a.t(), grad, 1.0, beta);
        }
    }
    return r;
}

// ------------------------------------------------------------------ weight-as-stored forms
std::vector<at::Tensor> linear_forward(const at::Tensor& x, const at::Tensor& weight,
                                       const c10::optional<at::Tensor>& bias, const c10::optional<at::Tensor>& dense_t,
                                       double alpha, double beta, bool want_idx) {
    const bool blend = !(alpha == 1.0 && beta == 0.0);
    auto r = forward_impl(x, weight, MAM_B_NK, bias, dense_t, blend, alpha, beta, want_idx);
    if (!want_idx) return {r.y};
    return {r.y, r.argmax, r.argmin};
}
// linear_forward with the output dropout applied in the kernel epilogue: every element is dropped with
// probability drop_rate by a counter-based generator keyed by (drop_seed, element index), kept ones are scaled
// by 1 / (1 - drop_rate).  drop_apply forms the same mask again (the backward uses it on the upstream gradient).
std::vector<at::Tensor> linear_forward_drop(const at::Tensor& x, const at::Tensor& weight,
                                            const c10::optional<at::Tensor>& bias,
                                            const c10::optional<at::Tensor>& dense_t, double alpha, double beta,
                                            bool want_idx, double drop_rate, int64_t drop_seed) {
    const bool blend = !(alpha == 1.0 && beta == 0.0);
    auto r = forward_impl(x, weight, MAM_B_NK, bias, dense_t, blend, alpha, beta, want_idx, drop_rate, drop_seed);
    if (!want_idx) return {r.y};
    return {r.y, r.argmax, r.argmin};
}
// out = t * scale where element i (row-major) is kept under (seed, rate), else 0
at::Tensor drop_apply(const at::Tensor& t, double rate, double scale, int64_t seed) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat, "t must be a float32 CUDA tensor");
    TORCH_CHECK(rate >= 0.0 && rate < 1.0, "rate must be in [0, 1)");
    auto tc = t.contiguous();
    c10::cuda::CUDAGuard guard(t.device());
    auto out = at::empty_like(tc);
    if (tc.numel() == 0) return out;
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_drop_f32(tc.data_ptr<float>(), out.data_ptr<float>(), tc.numel(), (float)rate, (float)scale,
                              (uint64_t)seed, stream.stream()),
                 "mam_drop_f32");
    return out;
}
// y[M,N] with K cut into slices of split_width columns, each contributing its own max + min; an empty tensor
// where the single-launch form does not apply (the caller then goes slice by slice)
at::Tensor linear_forward_splits(const at::Tensor& x, const at::Tensor& weight, const c10::optional<at::Tensor>& bias,
                                 const c10::optional<at::Tensor>& dense_t, double alpha, double beta,
                                 int64_t split_width) {
    check_matrix(x, "x");
    check_matrix(weight, "weight");
    const int64_t M = x.size(0), K = x.size(1), N = weight.size(0);
    TORCH_CHECK(weight.size(1) == K, "weight must be [N, K]");
    const float* bias_p = nullptr;
    const float* dense_p = nullptr;
    at::Tensor bias_c;
    if (bias.has_value() && bias->defined()) {
        TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kFloat && bias->numel() == N, "bias must be float32 [N]");
        bias_c = bias->contiguous();
        bias_p = bias_c.data_ptr<float>();
    }
    if (dense_t.has_value() && dense_t->defined()) {
        check_matrix(*dense_t, "dense");
        TORCH_CHECK(dense_t->size(0) == M && dense_t->size(1) == N, "dense must be [M, N]");
        dense_p = dense_t->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    if (M == 0 || N == 0) return at::empty({M, N}, x.options());
    auto y = at::empty({M, N}, x.options());
    const bool blend = !(alpha == 1.0 && beta == 0.0);
    auto stream = at::cuda::getCurrentCUDAStream();
    const int st = mam_fwd_splits_f32(x.data_ptr<float>(), weight.data_ptr<float>(), bias_p, dense_p, blend ? 1 : 0,
                                      (float)alpha, (float)beta, y.data_ptr<float>(), M, K, N, split_width,
                                      stream.stream());
    if (st == MAM_ERR_UNSUPPORTED) return at::empty({0}, x.options());
    check_status(st, "mam_fwd_splits_f32");
    return y;
}
// {y[M,N], argmax[S,M,N], argmin[S,M,N]} with K cut into S slices of split_width columns, every slice keeping its
// own selected pairs (indices in the numbering of the whole row); {} (no tensors) where the single-launch form
// does not apply and the caller goes slice by slice
std::vector<at::Tensor> linear_forward_splits_idx(const at::Tensor& x, const at::Tensor& weight,
                                                  const c10::optional<at::Tensor>& bias,
                                                  const c10::optional<at::Tensor>& dense_t, double alpha, double beta,
                                                  int64_t split_width) {
    check_matrix(x, "x");
    check_matrix(weight, "weight");
    const int64_t M = x.size(0), K = x.size(1), N = weight.size(0);
    TORCH_CHECK(weight.size(1) == K, "weight must be [N, K]");
    TORCH_CHECK(split_width > 0, "split_width must be positive");
    const float* bias_p = nullptr;
    const float* dense_p = nullptr;
    at::Tensor bias_c;
    if (bias.has_value() && bias->defined()) {
        TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kFloat && bias->numel() == N, "bias must be float32 [N]");
        bias_c = bias->contiguous();
        bias_p = bias_c.data_ptr<float>();
    }
    if (dense_t.has_value() && dense_t->defined()) {
        check_matrix(*dense_t, "dense");
        TORCH_CHECK(dense_t->size(0) == M && dense_t->size(1) == N, "dense must be [M, N]");
        dense_p = dense_t->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    if (M == 0 || N == 0 || K == 0) return {};
    const int64_t S = (K + split_width - 1) / split_width;
    auto y = at::empty({M, N}, x.options());
    auto amax = at::empty({S, M, N}, x.options().dtype(at::kInt));
    auto amin = at::empty({S, M, N}, x.options().dtype(at::kInt));
    const bool blend = !(alpha == 1.0 && beta == 0.0);
    auto stream = at::cuda::getCurrentCUDAStream();
    const int st = mam_fwd_splits_idx_f32(x.data_ptr<float>(), weight.data_ptr<float>(), bias_p, dense_p, blend ? 1 : 0,
                                          (float)alpha, (float)beta, y.data_ptr<float>(), amax.data_ptr<int32_t>(),
                                          amin.data_ptr<int32_t>(), M, K, N, split_width, stream.stream());
    if (st == MAM_ERR_UNSUPPORTED) return {};
    check_status(st, "mam_fwd_splits_idx_f32");
    return {y, amax, amin};
}
// {dx, dw} through the selected pairs of every slice (argmax / argmin [S,M,N])
std::vector<at::Tensor> linear_backward_splits(const at::Tensor& x, const at::Tensor& weight, const at::Tensor& grad,
                                               const at::Tensor& argmax, const at::Tensor& argmin, double scale) {
    check_matrix(x, "x");
    check_matrix(weight, "weight");
    check_matrix(grad, "grad");
    TORCH_CHECK(argmax.is_cuda() && argmax.dim() == 3 && argmax.scalar_type() == at::kInt && argmax.is_contiguous(),
                "argmax must be a contiguous int32 CUDA [S,M,N] tensor");
    TORCH_CHECK(argmin.sizes() == argmax.sizes() && argmin.scalar_type() == at::kInt && argmin.is_contiguous(),
                "argmin must match argmax");
    const int64_t M = x.size(0), K = x.size(1), N = weight.size(0), S = argmax.size(0);
    TORCH_CHECK(weight.size(1) == K && grad.size(0) == M && grad.size(1) == N, "shape mismatch");
    TORCH_CHECK(argmax.size(1) == M && argmax.size(2) == N && S >= 1, "index shapes must be [S,M,N]");
    c10::cuda::CUDAGuard guard(x.device());
    auto da = at::empty_like(x);
    auto dw = at::empty_like(weight);
    if (M == 0 || N == 0 || K == 0) {
        da.zero_();
        dw.zero_();
        return {da, dw};
    }
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_bwd_splits_f32(x.data_ptr<float>(), weight.data_ptr<float>(), MAM_B_NK, grad.data_ptr<float>(),
                                    argmax.data_ptr<int32_t>(), argmin.data_ptr<int32_t>(), (int)S, da.data_ptr<float>(),
                                    MAM_DA_MK, dw.data_ptr<float>(), nullptr, nullptr, (float)scale, M, K, N, nullptr, 0,
                                    stream.stream()),
                 "mam_bwd_splits_f32");
    return {da, dw};
}
std::vector<at::Tensor> linear_backward(const at::Tensor& x, const at::Tensor& weight, const at::Tensor& grad,
                                        const at::Tensor& argmax, const at::Tensor& argmin, double scale) {
    return backward_impl(x, weight, MAM_B_NK, grad, argmax, argmin, scale);
}
// {dx, dw, hit_max[N,K], hit_min[N,K]}: the backward with this pass's selection hits counted on the way
std::vector<at::Tensor> linear_backward_count(const at::Tensor& x, const at::Tensor& weight, const at::Tensor& grad,
                                              const at::Tensor& argmax, const at::Tensor& argmin, double scale) {
    return backward_impl(x, weight, MAM_B_NK, grad, argmax, argmin, scale, true);
}
// ------------------------------------------------------------------ convolution as patch rows
// rows[B*Ho*Wo, C*kH*kW] of x[B,C,H,W]
at::Tensor conv_im2col(const at::Tensor& x, int64_t kH, int64_t kW, int64_t sh, int64_t sw, int64_t ph, int64_t pw) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.dim() == 4, "x must be a float32 CUDA [B,C,H,W] tensor");
    auto xc = x.contiguous();
    const int64_t B = xc.size(0), C = xc.size(1), H = xc.size(2), W = xc.size(3);
    TORCH_CHECK(H + 2 * ph >= kH && W + 2 * pw >= kW, "kernel larger than the padded input");
    const int64_t Ho = (H + 2 * ph - kH) / sh + 1, Wo = (W + 2 * pw - kW) / sw + 1;
    c10::cuda::CUDAGuard guard(x.device());
    auto rows = at::empty({B * Ho * Wo, C * kH * kW}, xc.options());
    if (rows.numel() == 0) return rows;
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_im2col_f32(xc.data_ptr<float>(), rows.data_ptr<float>(), B, C, H, W, (int)kH, (int)kW, (int)sh,
                                (int)sw, (int)ph, (int)pw, stream.stream()),
                 "mam_im2col_f32");
    return rows;
}
// A fresh [B,H,W,C] contiguous copy of x[B,C,H,W].  (A caller whose x already is channels-last in memory
// uses x.permute(0, 2, 3, 1) as it is and does not come here.)
at::Tensor conv_channels_last(const at::Tensor& x) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.dim() == 4, "x must be a float32 CUDA [B,C,H,W] tensor");
    auto view = x.permute({0, 2, 3, 1});
    auto xc = x.contiguous();
    const int64_t B = xc.size(0), C = xc.size(1), H = xc.size(2), W = xc.size(3);
    c10::cuda::CUDAGuard guard(x.device());
    auto out = at::empty({B, H, W, C}, xc.options());
    if (out.numel() == 0) return out;
    if (B > 65535 || C > 65535 * 32) return view.contiguous();
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_nchw_to_nhwc_f32(xc.data_ptr<float>(), out.data_ptr<float>(), B, C, H, W, stream.stream()),
                 "mam_nchw_to_nhwc_f32");
    return out;
}
// A fresh contiguous [C,R] transpose of the matrix a[R,C] (the same batched-transpose kernel, one image of R
// channels and C pixels); several times faster than a strided torch copy.
at::Tensor transpose2d(const at::Tensor& a) {
    TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kFloat && a.dim() == 2, "a must be a float32 CUDA matrix");
    auto ac = a.contiguous();
    const int64_t R = ac.size(0), C = ac.size(1);
    c10::cuda::CUDAGuard guard(a.device());
    auto out = at::empty({C, R}, ac.options());
    if (out.numel() == 0) return out;
    if (R > 65535LL * 32) return ac.t().contiguous();
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_nchw_to_nhwc_f32(ac.data_ptr<float>(), out.data_ptr<float>(), 1, R, 1, C, stream.stream()),
                 "mam_nchw_to_nhwc_f32");
    return out;
}
// Whether conv_forward_implicit can take a convolution of this geometry (no device needed).
bool conv_implicit_applies(int64_t B, int64_t C, int64_t H, int64_t W, int64_t kH, int64_t kW, int64_t sh, int64_t sw,
                           int64_t ph, int64_t pw) {
    return mam_conv_fwd_applies(B, C, H, W, (int)kH, (int)kW, (int)sh, (int)sw, (int)ph, (int)pw) != 0;
}
// {y[B*Ho*Wo, N]} or {y, argmax, argmin}: forward straight from the channels-last input x_nhwc[B,H,W,C] with the
// weight in tap order w_taps[N, kH*kW*C] (weight.permute(0, 3, 2, 1)); indices numbered as weight.view(N, -1)
std::vector<at::Tensor> conv_forward_implicit(const at::Tensor& x_nhwc, const at::Tensor& w_taps,
                                              const c10::optional<at::Tensor>& bias,
                                              const c10::optional<at::Tensor>& dense_t, double alpha, double beta,
                                              int64_t kH, int64_t kW, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                                              bool want_idx) {
    TORCH_CHECK(x_nhwc.is_cuda() && x_nhwc.scalar_type() == at::kFloat && x_nhwc.dim() == 4 && x_nhwc.is_contiguous(),
                "x_nhwc must be a contiguous float32 CUDA [B,H,W,C] tensor");
    check_matrix(w_taps, "w_taps");
    const int64_t B = x_nhwc.size(0), H = x_nhwc.size(1), W = x_nhwc.size(2), C = x_nhwc.size(3);
    TORCH_CHECK(H + 2 * ph >= kH && W + 2 * pw >= kW, "kernel larger than the padded input");
    const int64_t Ho = (H + 2 * ph - kH) / sh + 1, Wo = (W + 2 * pw - kW) / sw + 1;
    const int64_t M = B * Ho * Wo, K = C * kH * kW, N = w_taps.size(0);
    TORCH_CHECK(w_taps.size(1) == K, "w_taps must be [N, kH*kW*C]");
    const float* bias_p = nullptr;
    const float* dense_p = nullptr;
    at::Tensor bias_c, dense_c;
    if (bias.has_value() && bias->defined()) {
        TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kFloat && bias->numel() == N, "bias must be float32 [N]");
        bias_c = bias->contiguous();
        bias_p = bias_c.data_ptr<float>();
    }
    if (dense_t.has_value() && dense_t->defined()) {
        check_matrix(*dense_t, "dense");
        TORCH_CHECK(dense_t->size(0) == M && dense_t->size(1) == N, "dense must be [B*Ho*Wo, N]");
        dense_c = *dense_t;
        dense_p = dense_c.data_ptr<float>();
    }
    const bool blend = !(alpha == 1.0 && beta == 0.0);
    c10::cuda::CUDAGuard guard(x_nhwc.device());
    auto y = at::empty({M, N}, x_nhwc.options());
    at::Tensor amax, amin;
    if (want_idx) {
        amax = at::empty({M, N}, x_nhwc.options().dtype(at::kInt));
        amin = at::empty({M, N}, x_nhwc.options().dtype(at::kInt));
    }
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_conv_fwd_f32(x_nhwc.data_ptr<float>(), w_taps.data_ptr<float>(), bias_p, dense_p, blend ? 1 : 0,
                                  (float)alpha, (float)beta, y.data_ptr<float>(),
                                  want_idx ? amax.data_ptr<int32_t>() : nullptr,
                                  want_idx ? amin.data_ptr<int32_t>() : nullptr, B, C, H, W, (int)kH, (int)kW, (int)sh,
                                  (int)sw, (int)ph, (int)pw, N, stream.stream()),
                 "mam_conv_fwd_f32");
    if (!want_idx) return {y};
    return {y, amax, amin};
}
// dx[B,C,H,W] from the transposed row gradients cols_t[C*kH*kW, B*Ho*Wo]
at::Tensor conv_col2im(const at::Tensor& cols_t, int64_t B, int64_t C, int64_t H, int64_t W, int64_t kH, int64_t kW,
                       int64_t sh, int64_t sw, int64_t ph, int64_t pw) {
    check_matrix(cols_t, "cols_t");
    const int64_t Ho = (H + 2 * ph - kH) / sh + 1, Wo = (W + 2 * pw - kW) / sw + 1;
    TORCH_CHECK(cols_t.size(0) == C * kH * kW && cols_t.size(1) == B * Ho * Wo, "cols_t must be [C*kH*kW, B*Ho*Wo]");
    c10::cuda::CUDAGuard guard(cols_t.device());
    auto dx = at::empty({B, C, H, W}, cols_t.options());
    if (dx.numel() == 0) return dx;
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_col2im_f32(cols_t.data_ptr<float>(), dx.data_ptr<float>(), B, C, H, W, (int)kH, (int)kW, (int)sh,
                                (int)sw, (int)ph, (int)pw, stream.stream()),
                 "mam_col2im_f32");
    return dx;
}
// {cols_t [C*kH*kW, B*Ho*Wo], dw [N, C*kH*kW]}: convolution backward reading the selected activations from x itself
std::vector<at::Tensor> conv_backward(const at::Tensor& x, const at::Tensor& w2d, const at::Tensor& grad,
                                      const at::Tensor& argmax, const at::Tensor& argmin, double scale, int64_t kH,
                                      int64_t kW, int64_t sh, int64_t sw, int64_t ph, int64_t pw) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.dim() == 4, "x must be a float32 CUDA [B,C,H,W] tensor");
    check_matrix(w2d, "weight");
    check_matrix(grad, "grad");
    check_matrix(argmax, "argmax", at::kInt);
    check_matrix(argmin, "argmin", at::kInt);
    auto xc = x.contiguous();
    const int64_t B = xc.size(0), C = xc.size(1), H = xc.size(2), W = xc.size(3);
    const int64_t Ho = (H + 2 * ph - kH) / sh + 1, Wo = (W + 2 * pw - kW) / sw + 1;
    const int64_t M = B * Ho * Wo, K = C * kH * kW, N = w2d.size(0);
    TORCH_CHECK(w2d.size(1) == K, "weight must be [N, C*kH*kW]");
    TORCH_CHECK(grad.size(0) == M && grad.size(1) == N, "grad must be [B*Ho*Wo, N]");
    TORCH_CHECK(argmax.sizes() == grad.sizes() && argmin.sizes() == grad.sizes(), "index shapes must match grad");
    c10::cuda::CUDAGuard guard(x.device());
    auto cols_t = at::empty({K, M}, xc.options());
    auto dw = at::empty_like(w2d);
    if (M == 0 || N == 0 || K == 0) {
        cols_t.zero_();
        dw.zero_();
        return {cols_t, dw};
    }
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_conv_bwd_f32(xc.data_ptr<float>(), w2d.data_ptr<float>(), grad.data_ptr<float>(),
                                  argmax.data_ptr<int32_t>(), argmin.data_ptr<int32_t>(), cols_t.data_ptr<float>(),
                                  dw.data_ptr<float>(), (float)scale, B, C, H, W, (int)kH, (int)kW, (int)sh, (int)sw,
                                  (int)ph, (int)pw, N, stream.stream()),
                 "mam_conv_bwd_f32");
    return {cols_t, dw};
}
// Whether conv_backward_direct can take a convolution of this geometry (no device needed).
bool conv_direct_applies(int64_t B, int64_t C, int64_t H, int64_t W, int64_t kH, int64_t kW, int64_t sh, int64_t sw,
                         int64_t ph, int64_t pw) {
    return mam_conv_bwd_direct_applies(B, C, H, W, (int)kH, (int)kW, (int)sh, (int)sw, (int)ph, (int)pw) != 0;
}
// {dx [B,C,H,W], dw [N, C*kH*kW]}: convolution backward in one kernel, dx summed per tile of output rows
std::vector<at::Tensor> conv_backward_direct(const at::Tensor& x, const at::Tensor& w2d, const at::Tensor& grad,
                                             const at::Tensor& argmax, const at::Tensor& argmin, double scale,
                                             int64_t kH, int64_t kW, int64_t sh, int64_t sw, int64_t ph, int64_t pw) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.dim() == 4, "x must be a float32 CUDA [B,C,H,W] tensor");
    check_matrix(w2d, "weight");
    check_matrix(grad, "grad");
    check_matrix(argmax, "argmax", at::kInt);
    check_matrix(argmin, "argmin", at::kInt);
    auto xc = x.contiguous();
    const int64_t B = xc.size(0), C = xc.size(1), H = xc.size(2), W = xc.size(3);
    const int64_t Ho = (H + 2 * ph - kH) / sh + 1, Wo = (W + 2 * pw - kW) / sw + 1;
    const int64_t M = B * Ho * Wo, K = C * kH * kW, N = w2d.size(0);
    TORCH_CHECK(w2d.size(1) == K, "weight must be [N, C*kH*kW]");
    TORCH_CHECK(grad.size(0) == M && grad.size(1) == N, "grad must be [B*Ho*Wo, N]");
    TORCH_CHECK(argmax.sizes() == grad.sizes() && argmin.sizes() == grad.sizes(), "index shapes must match grad");
    c10::cuda::CUDAGuard guard(x.device());
    auto dx = at::empty_like(xc);
    auto dw = at::empty_like(w2d);
    if (M == 0 || N == 0 || K == 0) {
        dx.zero_();
        dw.zero_();
        return {dx, dw};
    }
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_conv_bwd_direct_f32(xc.data_ptr<float>(), w2d.data_ptr<float>(), grad.data_ptr<float>(),
                                         argmax.data_ptr<int32_t>(), argmin.data_ptr<int32_t>(), dx.data_ptr<float>(),
                                         dw.data_ptr<float>(), (float)scale, B, C, H, W, (int)kH, (int)kW, (int)sh,
                                         (int)sw, (int)ph, (int)pw, N, stream.stream()),
                 "mam_conv_bwd_direct_f32");
    return {dx, dw};
}
// {dx transposed [K,M], dw}: the backward of linear_forward with the row gradients laid out for conv_col2im
std::vector<at::Tensor> linear_backward_km(const at::Tensor& x, const at::Tensor& weight, const at::Tensor& grad,
                                           const at::Tensor& argmax, const at::Tensor& argmin, double scale) {
    return backward_impl(x, weight, MAM_B_NK, grad, argmax, argmin, scale, false, true);
}

// hits[0] = hit_max[N,K], hits[1] = hit_min[N,K]: how many rows selected each weight
std::vector<at::Tensor> selection_hits(const at::Tensor& argmax, const at::Tensor& argmin, int64_t K) {
    check_matrix(argmax, "argmax", at::kInt);
    check_matrix(argmin, "argmin", at::kInt);
    TORCH_CHECK(argmax.sizes() == argmin.sizes(), "argmax/argmin shapes differ");
    c10::cuda::CUDAGuard guard(argmax.device());
    const int64_t M = argmax.size(0), N = argmax.size(1);
    auto hmax = at::zeros({N, K}, argmax.options());
    auto hmin = at::zeros({N, K}, argmax.options());
    if (M == 0 || N == 0 || K == 0) return {hmax, hmin};
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_selcount_i32(argmax.data_ptr<int32_t>(), argmin.data_ptr<int32_t>(), hmax.data_ptr<int32_t>(),
                                  hmin.data_ptr<int32_t>(), M, K, N, stream.stream()),
                 "mam_selcount_i32");
    return {hmax, hmin};
}
// count += (hit_max>0) + (hit_min>0), in place; returns count
at::Tensor selection_count_update_(at::Tensor count, const at::Tensor& hit_max, const at::Tensor& hit_min) {
    TORCH_CHECK(count.is_cuda() && count.scalar_type() == at::kInt && count.is_contiguous(), "count: int32 CUDA");
    TORCH_CHECK(hit_max.sizes() == count.sizes() && hit_min.sizes() == count.sizes(), "shape mismatch");
    c10::cuda::CUDAGuard guard(count.device());
    if (count.numel() == 0) return count;
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_selcount_indicator_i32(hit_max.data_ptr<int32_t>(), hit_min.data_ptr<int32_t>(),
                                            count.data_ptr<int32_t>(), count.numel(), stream.stream()),
                 "mam_selcount_indicator_i32");
    return count;
}

// ------------------------------------------------------------------ pruned weights (CSR)
// y (and indices) of the dense layer on W with zeros at the positions that are not stored
std::vector<at::Tensor> csr_linear_forward(const at::Tensor& x, const at::Tensor& crow, const at::Tensor& col,
                                           const at::Tensor& val, const c10::optional<at::Tensor>& bias,
                                           bool want_idx) {
    check_matrix(x, "x");
    TORCH_CHECK(crow.is_cuda() && col.is_cuda() && val.is_cuda(), "CSR components must be CUDA tensors");
    TORCH_CHECK(crow.scalar_type() == at::kLong && col.scalar_type() == at::kLong, "CSR indices must be int64");
    TORCH_CHECK(val.scalar_type() == at::kFloat, "CSR values must be float32");
    TORCH_CHECK(crow.dim() == 1 && crow.numel() >= 1 && col.numel() == val.numel(), "malformed CSR components");
    const int64_t M = x.size(0), K = x.size(1), N = crow.numel() - 1;
    c10::cuda::CUDAGuard guard(x.device());
    auto y = at::empty({M, N}, x.options());
    at::Tensor amax, amin;
    if (want_idx) {
        amax = at::empty({M, N}, x.options().dtype(at::kInt));
        amin = at::empty({M, N}, x.options().dtype(at::kInt));
    }
    if (M > 0 && N > 0) {
        TORCH_CHECK(K > 0, "the reduction dimension must not be empty");
        auto crow_c = crow.contiguous(), col_c = col.contiguous(), val_c = val.contiguous();
        const float* bias_p = nullptr;
        at::Tensor bias_c;
        if (bias.has_value() && bias->defined()) {
            TORCH_CHECK(bias->numel() == N && bias->scalar_type() == at::kFloat && bias->is_cuda(), "bias");
            bias_c = bias->contiguous();
            bias_p = bias_c.data_ptr<float>();
        }
        // col may be empty (everything pruned): pass a valid dummy pointer, it is never dereferenced
        const int64_t* col_p = col_c.numel() ? col_c.data_ptr<int64_t>() : crow_c.data_ptr<int64_t>();
        const float* val_p = val_c.numel() ? val_c.data_ptr<float>() : x.data_ptr<float>();
        auto stream = at::cuda::getCurrentCUDAStream();
        // scratch for the tiled kernels (transposed activations + regrouped entries); 0 = not applicable
        const int64_t nnz = val_c.numel();
        const size_t wsb = mam_csr_fwd_workspace_bytes(M, K, N, nnz);
        at::Tensor ws;
        if (wsb) ws = at::empty({(int64_t)wsb}, x.options().dtype(at::kByte));
        check_status(mam_csr_fwd_ws_f32(x.data_ptr<float>(), crow_c.data_ptr<int64_t>(), col_p, val_p, nnz, bias_p,
                                        y.data_ptr<float>(), want_idx ? amax.data_ptr<int32_t>() : nullptr,
                                        want_idx ? amin.data_ptr<int32_t>() : nullptr, M, K, N,
                                        wsb ? ws.data_ptr() : nullptr, wsb, stream.stream()),
                     "mam_csr_fwd_ws_f32");
    }
    if (!want_idx) return {y};
    return {y, amax, amin};
}

// Bytes of scratch the tiled CSR forward wants for [M,K] activations and this weight (0: the tiled kernels do not
// apply), and how many of them hold the regrouped weight (independent of M).
std::vector<int64_t> csr_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t nnz) {
    return {(int64_t)mam_csr_fwd_workspace_bytes(M, K, N, nnz), (int64_t)mam_csr_fwd_entries_bytes(K, N, nnz)};
}
// csr_linear_forward on a scratch buffer the caller keeps: with entries_ready = 1 the regrouped weight found in
// `workspace` (left there by an earlier call on the same CSR contents) is used as is; with 2 only the sparsity
// pattern is taken as unchanged and the stored values are regrouped again (a training step: same mask, new values)
std::vector<at::Tensor> csr_linear_forward_ws(const at::Tensor& x, const at::Tensor& crow, const at::Tensor& col,
                                              const at::Tensor& val, const c10::optional<at::Tensor>& bias,
                                              bool want_idx, at::Tensor workspace, int64_t entries_ready) {
    check_matrix(x, "x");
    TORCH_CHECK(crow.is_cuda() && col.is_cuda() && val.is_cuda(), "CSR components must be CUDA tensors");
    TORCH_CHECK(crow.scalar_type() == at::kLong && col.scalar_type() == at::kLong, "CSR indices must be int64");
    TORCH_CHECK(val.scalar_type() == at::kFloat, "CSR values must be float32");
    TORCH_CHECK(crow.dim() == 1 && crow.numel() >= 1 && col.numel() == val.numel(), "malformed CSR components");
    TORCH_CHECK(crow.is_contiguous() && col.is_contiguous() && val.is_contiguous(), "CSR components must be contiguous");
    TORCH_CHECK(workspace.is_cuda() && workspace.scalar_type() == at::kByte && workspace.is_contiguous(),
                "workspace must be a contiguous uint8 CUDA tensor");
    const int64_t M = x.size(0), K = x.size(1), N = crow.numel() - 1, nnz = val.numel();
    TORCH_CHECK(M > 0 && N > 0 && K > 0 && nnz > 0, "empty problem: use csr_linear_forward");
    const size_t need = mam_csr_fwd_workspace_bytes(M, K, N, nnz);
    TORCH_CHECK(need > 0 && (size_t)workspace.numel() >= need, "workspace too small for this call");
    c10::cuda::CUDAGuard guard(x.device());
    auto y = at::empty({M, N}, x.options());
    at::Tensor amax, amin;
    if (want_idx) {
        amax = at::empty({M, N}, x.options().dtype(at::kInt));
        amin = at::empty({M, N}, x.options().dtype(at::kInt));
    }
    const float* bias_p = nullptr;
    at::Tensor bias_c;
    if (bias.has_value() && bias->defined()) {
        TORCH_CHECK(bias->numel() == N && bias->scalar_type() == at::kFloat && bias->is_cuda(), "bias");
        bias_c = bias->contiguous();
        bias_p = bias_c.data_ptr<float>();
    }
    auto stream = at::cuda::getCurrentCUDAStream();
    check_status(mam_csr_fwd_ws_ex_f32(x.data_ptr<float>(), crow.data_ptr<int64_t>(), col.data_ptr<int64_t>(),
                                       val.data_ptr<float>(), nnz, bias_p, y.data_ptr<float>(),
                                       want_idx ? amax.data_ptr<int32_t>() : nullptr,
                                       want_idx ? amin.data_ptr<int32_t>() : nullptr, M, K, N, workspace.data_ptr(),
                                       (size_t)workspace.numel(), (int)entries_ready, stream.stream()),
                 "mam_csr_fwd_ws_ex_f32");
    if (!want_idx) return {y};
    return {y, amax, amin};
}

// c[N,Mc] = A . b for A given by its CSR components
at::Tensor spmm_components(const at::Tensor& crow, const at::Tensor& col, const at::Tensor& val, int64_t N, int64_t K,
                           const at::Tensor& b) {
    c10::cuda::CUDAGuard guard(b.device());
    const int64_t Mc = b.size(1);
    auto c = at::zeros({N, Mc}, b.options());
    if (N == 0 || Mc == 0 || K == 0) return c;
    if (val.numel() == 0) return c;
    auto bc = b.contiguous();
    auto stream = at::cuda::getCurrentCUDAStream();
    const int64_t nnz = val.numel();
    const size_t wsb = mam_spmm_csr_workspace_bytes(N, K, Mc, nnz);   // 0: the tiled kernel does not apply
    at::Tensor ws;
    if (wsb) ws = at::empty({(int64_t)wsb}, bc.options().dtype(at::kByte));
    check_status(mam_spmm_csr_ws_f32(crow.data_ptr<int64_t>(), col.data_ptr<int64_t>(), val.data_ptr<float>(), nnz,
                                     bc.data_ptr<float>(), c.data_ptr<float>(), N, K, Mc, wsb ? ws.data_ptr() : nullptr,
                                     wsb, stream.stream()),
                 "mam_spmm_csr_ws_f32");
    return c;
}
// cusparsemm(a_sparse[N,K], b[K,M]) -> dense [N,M], a in CSR layout
at::Tensor spmm_csr(const at::Tensor& a, const at::Tensor& b) {
    TORCH_CHECK(b.is_cuda() && b.dim() == 2 && b.scalar_type() == at::kFloat, "b must be a 2-D float CUDA tensor");
    TORCH_CHECK(a.dim() == 2 && a.size(1) == b.size(0), "inner dimensions differ");
    return spmm_components(a.crow_indices().to(at::kLong).contiguous(), a.col_indices().to(at::kLong).contiguous(),
                           a.values().to(at::kFloat).contiguous(), a.size(0), a.size(1), b);
}
// The same for a COO operand.  A coalesced COO tensor keeps its entries sorted by (row, column), which is CSR
// order already: the column indices and the values are used where they are and only the N+1 row offsets are
// formed (one small kernel), instead of converting the whole tensor on every call.
at::Tensor spmm_coo(const at::Tensor& a, const at::Tensor& b) {
    TORCH_CHECK(b.is_cuda() && b.dim() == 2 && b.scalar_type() == at::kFloat, "b must be a 2-D float CUDA tensor");
    TORCH_CHECK(a.dim() == 2 && a.size(1) == b.size(0), "inner dimensions differ");
    if (!a.is_coalesced() || a.sparse_dim() != 2 || a.dense_dim() != 0) return spmm_csr(a.to_sparse_csr(), b);
    auto idx = a._indices();                                   // [2, nnz] int64
    auto crow = at::_convert_indices_from_coo_to_csr(idx.select(0, 0).contiguous(), a.size(0), /*out_int32=*/false);
    return spmm_components(crow, idx.select(0, 1).contiguous(), a._values().to(at::kFloat).contiguous(), a.size(0),
                           a.size(1), b);
}

}  // namespace

// The MAM layer on a pruned weight, beside the reference's one sparse operator and in its namespace: forward on
// the CSR components of W[N,K] (crow, col, val as torch.Tensor.to_sparse_csr() gives them), backward through the
// selected pairs into a DENSE weight gradient (a pruned position whose zero product was selected receives one).
std::vector<at::Tensor> fullyconnected_csr(const at::Tensor& a, const at::Tensor& crow, const at::Tensor& col,
                                           const at::Tensor& val, const c10::optional<at::Tensor>& bias) {
    return csr_linear_forward(a, crow, col, val, bias, true);
}
std::vector<at::Tensor> fullyconnected_csr_backward(const at::Tensor& a, const at::Tensor& w_dense,
                                                    const at::Tensor& grad, const at::Tensor& argmax,
                                                    const at::Tensor& argmin) {
    return backward_impl(a, w_dense, MAM_B_NK, grad, argmax, argmin, 1.0);
}

TORCH_LIBRARY(mamtorch_kernel_sparsev1, m) {
    m.def("cusparsemm(Tensor a, Tensor b) -> Tensor");
    m.def("fullyconnected_csr(Tensor a, Tensor crow, Tensor col, Tensor val, Tensor? bias) -> Tensor[]");
    m.def("fullyconnected_csr_backward(Tensor a, Tensor w_dense, Tensor grad, Tensor argmax, Tensor argmin) -> Tensor[]");
}
TORCH_LIBRARY_IMPL(mamtorch_kernel_sparsev1, SparseCUDA, m) { m.impl("cusparsemm", &spmm_coo); }
TORCH_LIBRARY_IMPL(mamtorch_kernel_sparsev1, SparseCsrCUDA, m) { m.impl("cusparsemm", &spmm_csr); }
TORCH_LIBRARY_IMPL(mamtorch_kernel_sparsev1, CUDA, m) {
    m.impl("fullyconnected_csr", &fullyconnected_csr);
    m.impl("fullyconnected_csr_backward", &fullyconnected_csr_backward);
}

TORCH_LIBRARY(mamtorch_kernel_v1, m) {
    m.def("fullyconnected(Tensor a, Tensor b) -> Tensor[]");
    m.def("fullyconnected_backward(Tensor a, Tensor b, Tensor grad, Tensor argmax, Tensor argmin) -> Tensor[]");
}
TORCH_LIBRARY_IMPL(mamtorch_kernel_v1, CUDA, m) {
    m.impl("fullyconnected", &fullyconnected);
    m.impl("fullyconnected_backward", &fullyconnected_backward);
}

TORCH_LIBRARY(mamtorch_kernel_v2, m) {
    m.def("fullyconnected(Tensor a, Tensor b, Tensor bias, float beta) -> Tensor[]");
    m.def("fullyconnected_backward(Tensor a, Tensor b, Tensor grad, Tensor argmax, Tensor argmin, float beta) -> Tensor[]");
    m.def("dense(Tensor a, Tensor b) -> Tensor");
}
TORCH_LIBRARY_IMPL(mamtorch_kernel_v2, CUDA, m) {
    m.impl("fullyconnected", &fullyconnected_beta);
    m.impl("fullyconnected_backward", &fullyconnected_backward_beta);
    m.impl("dense", &dense);
}

TORCH_LIBRARY(mamtorch_kernel_v3, m) {
    m.def("fullyconnected(Tensor a, Tensor b, Tensor bias, float beta) -> Tensor[]");
    m.def("fullyconnected_fast(Tensor a, Tensor b, Tensor bias, float beta) -> Tensor");
    m.def("fullyconnected_backward(Tensor a, Tensor b, Tensor grad, Tensor argmax, Tensor argmin, float beta) -> Tensor[]");
}
TORCH_LIBRARY_IMPL(mamtorch_kernel_v3, CUDA, m) {
    m.impl("fullyconnected", &fullyconnected_beta);
    m.impl("fullyconnected_fast", &fullyconnected_fast_beta);
    m.impl("fullyconnected_backward", &fullyconnected_backward_beta);
}

TORCH_LIBRARY(mamtorch_kernel_v4, m) {
    m.def("fullyconnected(Tensor a, Tensor b) -> Tensor[]");
    m.def("fullyconnected_fast(Tensor a, Tensor b) -> Tensor");
    m.def("fullyconnected_backward(Tensor a, Tensor b, Tensor grad, Tensor argmax, Tensor argmin) -> Tensor[]");
}
TORCH_LIBRARY_IMPL(mamtorch_kernel_v4, CUDA, m) {
    m.impl("fullyconnected", &fullyconnected);
    m.impl("fullyconnected_fast", &fullyconnected_fast);
    m.impl("fullyconnected_backward", &fullyconnected_backward);
}

TORCH_LIBRARY(mamtorch_b200, m) {
    m.def("linear_forward(Tensor x, Tensor weight, Tensor? bias, Tensor? dense, float alpha, float beta, bool want_idx) -> Tensor[]");
    m.def("linear_forward_drop(Tensor x, Tensor weight, Tensor? bias, Tensor? dense, float alpha, float beta, bool want_idx, float drop_rate, int drop_seed) -> Tensor[]");
    m.def("drop_apply(Tensor t, float rate, float scale, int seed) -> Tensor");
    m.def("linear_backward(Tensor x, Tensor weight, Tensor grad, Tensor argmax, Tensor argmin, float scale) -> Tensor[]");
    m.def("linear_backward_count(Tensor x, Tensor weight, Tensor grad, Tensor argmax, Tensor argmin, float scale) -> Tensor[]");
    m.def("linear_backward_km(Tensor x, Tensor weight, Tensor grad, Tensor argmax, Tensor argmin, float scale) -> Tensor[]");
    m.def("conv_backward(Tensor x, Tensor weight, Tensor grad, Tensor argmax, Tensor argmin, float scale, int kH, int kW, int sh, int sw, int ph, int pw) -> Tensor[]");
    m.def("conv_im2col(Tensor x, int kH, int kW, int sh, int sw, int ph, int pw) -> Tensor");
    m.def("conv_backward_direct(Tensor x, Tensor weight, Tensor grad, Tensor argmax, Tensor argmin, float scale, int kH, int kW, int sh, int sw, int ph, int pw) -> Tensor[]");
    m.def("conv_direct_applies(int B, int C, int H, int W, int kH, int kW, int sh, int sw, int ph, int pw) -> bool", &conv_direct_applies);
    m.def("linear_forward_splits(Tensor x, Tensor weight, Tensor? bias, Tensor? dense, float alpha, float beta, int split_width) -> Tensor");
    m.def("linear_forward_splits_idx(Tensor x, Tensor weight, Tensor? bias, Tensor? dense, float alpha, float beta, int split_width) -> Tensor[]");
    m.def("linear_backward_splits(Tensor x, Tensor weight, Tensor grad, Tensor argmax, Tensor argmin, float scale) -> Tensor[]");
    m.def("conv_channels_last(Tensor x) -> Tensor");
    m.def("transpose2d(Tensor a) -> Tensor");
    m.def("conv_forward_implicit(Tensor x_nhwc, Tensor w_taps, Tensor? bias, Tensor? dense, float alpha, float beta, int kH, int kW, int sh, int sw, int ph, int pw, bool need_indices) -> Tensor[]");
    m.def("conv_implicit_applies(int B, int C, int H, int W, int kH, int kW, int sh, int sw, int ph, int pw) -> bool", &conv_implicit_applies);
    m.def("conv_col2im(Tensor cols_t, int B, int C, int H, int W, int kH, int kW, int sh, int sw, int ph, int pw) -> Tensor");
    m.def("selection_hits(Tensor argmax, Tensor argmin, int K) -> Tensor[]");
    m.def("selection_count_update_(Tensor(a!) count, Tensor hit_max, Tensor hit_min) -> Tensor(a!)");
    m.def("dense_nt(Tensor a, Tensor w) -> Tensor");
    m.def("set_dense_backend(int backend) -> ()");
    m.def("get_dense_backend() -> int");
    m.def("check_device_flag() -> ()");
    m.def("poll_device_flag() -> ()");
    m.def("csr_linear_forward(Tensor x, Tensor crow, Tensor col, Tensor val, Tensor? bias, bool want_idx) -> Tensor[]");
    m.def("csr_linear_forward_ws(Tensor x, Tensor crow, Tensor col, Tensor val, Tensor? bias, bool want_idx, Tensor(a!) workspace, int entries_ready) -> Tensor[]");
    m.def("csr_workspace_bytes(int M, int K, int N, int nnz) -> int[]", &csr_workspace_bytes);
}
TORCH_LIBRARY_IMPL(mamtorch_b200, CUDA, m) {
    m.impl("linear_forward", &linear_forward);
    m.impl("linear_forward_drop", &linear_forward_drop);
    m.impl("drop_apply", &drop_apply);
    m.impl("linear_backward", &linear_backward);
    m.impl("linear_backward_count", &linear_backward_count);
    m.impl("linear_backward_km", &linear_backward_km);
    m.impl("conv_backward", &conv_backward);
    m.impl("conv_backward_direct", &conv_backward_direct);
    m.impl("conv_im2col", &conv_im2col);
    m.impl("conv_forward_implicit", &conv_forward_implicit);
    m.impl("conv_channels_last", &conv_channels_last);
    m.impl("transpose2d", &transpose2d);
    m.impl("linear_forward_splits", &linear_forward_splits);
    m.impl("linear_forward_splits_idx", &linear_forward_splits_idx);
    m.impl("linear_backward_splits", &linear_backward_splits);
    m.impl("conv_col2im", &conv_col2im);
    m.impl("selection_hits", &selection_hits);
    m.impl("selection_count_update_", &selection_count_update_);
    m.impl("csr_linear_forward", &csr_linear_forward);
    m.impl("csr_linear_forward_ws", &csr_linear_forward_ws);
    m.impl("dense_nt", &dense_nt);
}
TORCH_LIBRARY_IMPL(mamtorch_b200, CompositeExplicitAutograd, m) {
    m.impl("set_dense_backend", &set_dense_backend);
    m.impl("get_dense_backend", &get_dense_backend);
    m.impl("check_device_flag", &check_device_flag);
    m.impl("poll_device_flag", &poll_device_flag);
}
