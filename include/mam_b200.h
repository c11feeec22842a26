/* mam_b200.h -- C ABI of the B200 (sm_100a) Multiply-And-Max/min library, libmam_b200.so.
 *
 * Plain C types only: device pointers, sizes, a CUDA stream passed as void*.  No entry point
 * allocates or frees device memory; the caller owns every buffer, including the workspace whose
 * size the *_workspace_bytes queries return -- with one exception, mam_fwd_kn_static_f32, whose
 * scratch is a fixed buffer compiled into the library.  Every entry point returns a mam_status
 * code; text for it comes from mam_status_str().  All launches go to the stream given (0 = legacy default
 * stream) on the device that is current for the calling thread.
 *
 * Each function names the interface of SSIGPRO/mamtorch it stands in for (path:line inside that
 * project).  Layout notation: a[M,K] activations, row-major; the weight operand is either
 * b[K,N] row-major (MAM_B_KN, what the torch ops receive) or W[N,K] row-major (MAM_B_NK, how
 * nn.FullyConnected stores its parameter); y, grad, argmax, argmin are [M,N] row-major.
 */
#ifndef MAM_B200_H
#define MAM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MAM_ABI_VERSION 1

enum mam_status {
    MAM_OK = 0,
    MAM_ERR_INVALID_ARGUMENT = 1, /* null pointer, non-positive extent, bad layout code          */
    MAM_ERR_UNSUPPORTED = 2,      /* extent beyond what the kernels index (see each function)     */
    MAM_ERR_WORKSPACE = 3,        /* workspace missing, too small or not 256-byte aligned         */
    MAM_ERR_CUDA = 4,             /* a CUDA runtime/driver call failed; see mam_last_cuda_error() */
    MAM_ERR_DEVICE_TIMEOUT = 5,   /* a bounded wait inside a kernel gave up (results invalid)     */
    MAM_ERR_NOT_SM100 = 6,        /* the current device is not compute capability 10.x            */
    MAM_ERR_STATIC_SCRATCH = 7    /* problem needs more scratch than the built-in static buffer   */
};

#define MAM_B_KN 0
#define MAM_B_NK 1

/* Text for a status code (static storage). */
const char* mam_status_str(int status);
/* MAM_ABI_VERSION the library was built with. */
int mam_abi_version(void);
/* cudaGetErrorString of the last CUDA error seen by this library on the calling thread. */
const char* mam_last_cuda_error(void);
/* Synchronises the device and returns MAM_ERR_DEVICE_TIMEOUT if any kernel of this library has
 * recorded a wait that ran out since the flag was last cleared (it clears the flag). */
int mam_check_device_flag(void);

/* The same check without waiting for the device, for callers that must not stall their stream: returns
 * MAM_ERR_DEVICE_TIMEOUT if the copy of the flag that an EARLIER call of this function fetched shows a
 * wait that ran out (and then clears flag and copy), else queues the next fetch of the flag on `stream`
 * (4 bytes into pinned host memory the library keeps per device) and returns MAM_OK.  A time-out is thus
 * reported one call late at most.  No counterpart in the reference, whose kernels have no bounded waits. */
int mam_poll_device_flag(void* stream);

/* Per-kernel timing without a profiler.  While armed, every launch of the kernel class `kernel_id`
 * is bracketed by cudaEventRecord(starts[i]) / cudaEventRecord(stops[i]) on the launch stream,
 * i = 0,1,... up to `capacity` (later launches are not timed).  The caller creates the events
 * (cudaEvent_t passed as void*), synchronises, and reads cudaEventElapsedTime itself.
 * mam_timer_disarm() returns how many pairs were recorded.  Process-wide; not thread-safe. */
#define MAM_KERNEL_FWD_TILED 0   /* mam_fwd_tiled_kernel, the main forward loop       */
#define MAM_KERNEL_FWD_RESOLVE 1 /* chunk id -> exact index                              */
#define MAM_KERNEL_FWD_GENERIC 2 /* any-shape forward                                    */
#define MAM_KERNEL_BWD 3         /* selected-pair scatter                                */
#define MAM_KERNEL_SELCOUNT 4    /* selection hits                                       */
#define MAM_KERNEL_DENSE_TF32 5  /* tcgen05 TF32 product of the beta term                */
int mam_timer_arm(void** starts, void** stops, int capacity, int kernel_id);
int mam_timer_disarm(void);

/* Workspace needed by mam_fwd_f32 for these extents (0 is possible). */
size_t mam_fwd_workspace_bytes(int64_t M, int64_t K, int64_t N, int b_layout, int want_indices);

/* MAM forward.
 *   s[m,n] = max_k fl32(a[m,k]*b[k,n]) + min_k fl32(a[m,k]*b[k,n])
 *   y[m,n] = s                                   if blend == 0
 *          = alpha*s + beta*dense[m,n]           if blend != 0   (dense may be NULL: alpha*s)
 *          (+ bias[n] when bias != NULL)
 *   argmax/argmin: the k attaining max/min, lowest k on ties, int32.  Pass both NULL for the
 *   values-only form.
 * Stands in for fullyconnected_cuda (mamtorch/kernel/v1/csrc/cuda/fullyconnected.cu:177-291 and
 * mamtorch/kernel/v4/csrc/cuda/fullyconnected.cu:41-149), fullyconnected_fast_cuda
 * (mamtorch/kernel/v4/csrc/cuda/fullyconnected_fast.cu:39-137) and, through alpha/beta/bias/dense,
 * the blend of the v2/v3 host code (mamtorch/kernel/v3/csrc/cuda/fullyconnected.cu:153-160).
 * Limits: M*N < 2^31 * 64, K < 2^31; K == 0 is MAM_ERR_INVALID_ARGUMENT (a maximum over nothing). */
int mam_fwd_f32(const float* a, const float* b, int b_layout,
                const float* bias, const float* dense, int blend, float alpha, float beta,
                float* y, int32_t* argmax, int32_t* argmin,
                int64_t M, int64_t K, int64_t N,
                void* workspace, size_t workspace_bytes, void* stream);

/* mam_fwd_f32 with the module's output dropout (torch.nn.functional.dropout in training,
 * mamtorch/nn/v4/fullyconnected.py:204-206) applied in the kernel epilogue, after the bias: element
 * i = m*N + n of y is set to 0 with probability drop_rate and multiplied by 1 / (1 - drop_rate) otherwise
 * (0 <= drop_rate < 1; 0 is mam_fwd_f32).  The decision for element i is a pure function of (drop_seed, i) --
 * a counter-based generator -- so no mask is stored: mam_drop_f32 with the same seed and rate forms it again
 * for the backward.  The random stream is this library's own, not torch's. */
int mam_fwd_drop_f32(const float* a, const float* b, int b_layout,
                     const float* bias, const float* dense, int blend, float alpha, float beta,
                     float drop_rate, uint64_t drop_seed,
                     float* y, int32_t* argmax, int32_t* argmin,
                     int64_t M, int64_t K, int64_t N,
                     void* workspace, size_t workspace_bytes, void* stream);
/* out[i] = in[i] * scale where the generator above keeps element i under (seed, rate), else 0; i < n, in == out
 * allowed.  Three uses: the backward of the epilogue dropout (scale = 1 / (1 - rate) on the upstream gradient),
 * the module's weight drop (mamtorch/nn/v4/fullyconnected.py:143-148: scale = 1 on the weight, one pass in
 * place of bernoulli + multiply and their two [N,K] temporaries) and its backward (scale = 1 on dW). */
int mam_drop_f32(const float* in, float* out, int64_t n, float rate, float scale, uint64_t seed, void* stream);

/* Values-only forward with K cut into consecutive slices of split_width columns (the last one may be
 * shorter): y[m,n] = sum over slices, in ascending order, of (max + min over the slice's products), then the
 * blend / bias epilogue of mam_fwd_f32.  One launch for what the reference module's `splits` option does with
 * one kernel call and one addition pass per slice (mamtorch/nn/v4/fullyconnected.py:164-176).  a[M,K] and
 * w[N,K] (the weight as stored).  MAM_ERR_UNSUPPORTED unless split_width % 32 == 0, split_width < K, K % 4 == 0
 * and both operands are 16-byte aligned: callers then run slice by slice. */
int mam_fwd_splits_f32(const float* a, const float* w, const float* bias, const float* dense, int blend,
                       float alpha, float beta, float* y, int64_t M, int64_t K, int64_t N,
                       int64_t split_width, void* stream);

/* The same with indices, for training: argmax / argmin receive one [M,N] matrix PER SLICE ([slices][M][N],
 * slices = ceil(K / split_width)), each holding the slice's selected k in the numbering of the whole row.  One
 * launch of the index-producing forward for all slices (their partial sums are banked in y on the way) and one
 * index-resolver launch per slice, in place of one forward call, one addition pass and one autograd node per
 * slice (mamtorch/nn/v4/fullyconnected.py:164-176).  Same preconditions and MAM_ERR_UNSUPPORTED rule as
 * mam_fwd_splits_f32.  mam_bwd_splits_f32 is its backward. */
int mam_fwd_splits_idx_f32(const float* a, const float* w, const float* bias, const float* dense, int blend,
                           float alpha, float beta, float* y, int32_t* argmax, int32_t* argmin,
                           int64_t M, int64_t K, int64_t N, int64_t split_width, void* stream);

/* Forward for callers that cannot allocate device memory.  (No counterpart in the reference:
 * its host code allocates freely through ATen.)
 *
 * mam_fwd_f32 with the torch-op operand layout b[K,N] needs a K*N-float workspace for the
 * K-contiguous copy of b that the tiled kernels read.  Some hosts have nowhere to get one: code
 * running inside a stream capture or a real-time callback where cudaMalloc is forbidden, a plugin
 * whose host framework owns the allocator and exposes no scratch interface, a process that runs
 * with a fixed, fully committed memory plan.  For them this entry point keeps that copy in a
 * buffer compiled into the library: MAM_STATIC_SCRATCH_BYTES of device memory that every GPU
 * loading the library holds until the process exits, whether or not this function is ever called.
 *
 *   - Same results as mam_fwd_f32(a, b, MAM_B_KN, NULL, NULL, 0, ...): y = max+min, int32 indices
 *     (pass both NULL for values only).  It calls no cudaMalloc/cudaFree and no allocating
 *     library routine.
 *   - K*N*4 (rounded up to 256) must not exceed MAM_STATIC_SCRATCH_BYTES, otherwise
 *     MAM_ERR_STATIC_SCRATCH is returned and nothing is launched.
 *   - The first call on each device looks up the buffer's device address (with that device
 *     current).  Make that first call outside any stream capture.
 *   - All calls on a device share the one buffer and it keeps the previous call's contents.  Each
 *     call rewrites the part it uses before reading it, so nothing needs clearing, but two calls
 *     whose kernels overlap on the GPU (different streams, no ordering between them) race on it:
 *     serialise them. */
#define MAM_STATIC_SCRATCH_BYTES (8u << 20)
int mam_fwd_kn_static_f32(const float* a, const float* b, float* y, int32_t* argmax, int32_t* argmin,
                          int64_t M, int64_t K, int64_t N, void* stream);

/* MAM backward through the selected pairs.
 *   da[m,k]  = scale * sum_n grad[m,n] * b[k,n] * ([k==argmax[m,n]] + [k==argmin[m,n]])
 *   db (same layout as b) = scale * sum_m grad[m,n] * a[m,k] * (same selector)
 * Both outputs are overwritten.  Stands in for fullyconnected_backward_cuda
 * (mamtorch/kernel/v4/csrc/cuda/fullyconnected_backward.cu:80-135); scale carries the (1-beta)
 * of the v2/v3 variant (mamtorch/kernel/v3/csrc/cuda/fullyconnected_backward.cu:138-145).
 * Limit: K*4 bytes must fit the shared memory of one CTA (K <= 56000). */
int mam_bwd_f32(const float* a, const float* b, int b_layout, const float* grad,
                const int32_t* argmax, const int32_t* argmin,
                float* da, float* db, float scale,
                int64_t M, int64_t K, int64_t N, void* stream);

/* The same backward with the selection hits of this pass delivered too: hit_max[n,k] += #rows with
 * argmax[m,n]==k, hit_min likewise ([N,K] int32, added into; pass both NULL for no counting).  Without
 * scratch memory (this entry point and mam_bwd_count_ex_f32) the hits come from a second sweep over the two
 * index matrices after the gradient kernel, as mam_selcount_i32 does it.  mam_bwd_count_ws_f32 below makes it
 * ONE sweep: given 16 bytes of 256-byte aligned scratch per weight, every dW term goes to L2 together with
 * its hit as one 16-byte vector reduction {term, max hit, min hit, -} and a short pass splits the records into
 * db and the hit matrices.  mam_bwd_count_workspace_bytes(M, K, N) returns the scratch size where that form is
 * the faster one on B200 and 0 where it is not (the wider reduction costs more than the second sweep once the
 * records outgrow L2, or where the gradient kernel's time is its L2 reductions already: K in 640..832) or is
 * not available (M >= 2^24: the hits ride as fp32 sums of 1.0).  A caller that passes scratch of 16*K*N bytes
 * although the query answered 0 for speed still gets the one-sweep form.  With workspace == NULL it is
 * mam_bwd_count_ex_f32.  The device-side form of the bookkeeping in
 * FullyConnected.update_selection_count (mamtorch/nn/v4/fullyconnected.py:114-131) riding on
 * fullyconnected_backward_cuda (mamtorch/kernel/v4/csrc/cuda/fullyconnected_backward.cu:80-135). */
int mam_bwd_count_f32(const float* a, const float* b, int b_layout, const float* grad,
                      const int32_t* argmax, const int32_t* argmin,
                      float* da, float* db, int32_t* hit_max, int32_t* hit_min, float scale,
                      int64_t M, int64_t K, int64_t N, void* stream);

/* The same with a choice of layout for da: MAM_DA_MK is da[m*K + k] (as above), MAM_DA_KM is the
 * transpose da[k*M + m], which is what mam_col2im_f32 reads. */
#define MAM_DA_MK 0
#define MAM_DA_KM 1
int mam_bwd_count_ex_f32(const float* a, const float* b, int b_layout, const float* grad,
                         const int32_t* argmax, const int32_t* argmin,
                         float* da, int da_layout, float* db, int32_t* hit_max, int32_t* hit_min, float scale,
                         int64_t M, int64_t K, int64_t N, void* stream);
/* mam_bwd_count_ws_f32 for `slices` pairs of index matrices ([slices][M][N], as mam_fwd_splits_idx_f32 leaves
 * them): every slice routes the same upstream gradient through its own selected pairs, all in one pass over
 * the rows; hits (optional) are counted over all slices.  slices == 1 is mam_bwd_count_ws_f32. */
int mam_bwd_splits_f32(const float* a, const float* b, int b_layout, const float* grad,
                       const int32_t* argmax, const int32_t* argmin, int slices,
                       float* da, int da_layout, float* db, int32_t* hit_max, int32_t* hit_min, float scale,
                       int64_t M, int64_t K, int64_t N, void* workspace, size_t workspace_bytes, void* stream);
size_t mam_bwd_count_workspace_bytes(int64_t M, int64_t K, int64_t N);
int mam_bwd_count_ws_f32(const float* a, const float* b, int b_layout, const float* grad,
                         const int32_t* argmax, const int32_t* argmin,
                         float* da, int da_layout, float* db, int32_t* hit_max, int32_t* hit_min, float scale,
                         int64_t M, int64_t K, int64_t N, void* workspace, size_t workspace_bytes, void* stream);

/* Patch rows of a convolution input: rows[m][k] = x[b][c][ho*sh-ph+kh][wo*sw-pw+kw] (0 outside the image),
 * m = (b*Ho+ho)*Wo+wo, k = (c*kH+kh)*kW+kw, Ho = (H+2*ph-kH)/sh+1, Wo likewise; x is [B,C,H,W], rows is
 * [B*Ho*Wo, C*kH*kW].  Feeds mam_fwd_f32 (MAM_B_NK with weight.view(F, C*kH*kW)); one pass, no transposes.
 * Stands in for the per-call permutes of the reference's (never compiled) convolution host code,
 * mamtorch/kernel/backup/mamconv2d.txt:70-100, and the F.pad of mamtorch/nn/backup/mamconv2d.txt:133-139. */
int mam_im2col_f32(const float* x, float* rows, int64_t B, int64_t C, int64_t H, int64_t W,
                   int kH, int kW, int sh, int sw, int ph, int pw, void* stream);
/* Input gradient of the convolution from the TRANSPOSED row gradients cols_t[K][M] that
 * mam_bwd_count_ex_f32(..., MAM_DA_KM, ...) writes: dx[b][c][h][w] = sum of the (up to kH*kW) entries that
 * patch element came from.  dx is overwritten; no atomics.  Counterpart of the input-gradient scatter in
 * mamtorch/kernel/backup/mamconv2d_backward.txt:21-124. */
int mam_col2im_f32(const float* cols_t, float* dx, int64_t B, int64_t C, int64_t H, int64_t W,
                   int kH, int kW, int sh, int sw, int ph, int pw, void* stream);

/* Backward of the MAM convolution straight from the input: like mam_bwd_count_ex_f32(..., MAM_B_NK,
 * MAM_DA_KM, ...) on the patch rows of x, but the two selected activations per output are read where they
 * live in x[B,C,H,W] (zero in the padding), so the patch rows need not be kept after the forward.
 * w is the weight viewed as [N, C*kH*kW], grad / argmax / argmin are [B*Ho*Wo, N], cols_t receives the
 * transposed row gradients [C*kH*kW, B*Ho*Wo] (feed it to mam_col2im_f32), dw like w.  Stands in for
 * mamconv2d_backward of the reference's text backups (mamtorch/kernel/backup/mamconv2d_backward.txt:21-124). */
int mam_conv_bwd_f32(const float* x, const float* w, const float* grad,
                     const int32_t* argmax, const int32_t* argmin,
                     float* cols_t, float* dw, float scale,
                     int64_t B, int64_t C, int64_t H, int64_t W,
                     int kH, int kW, int sh, int sw, int ph, int pw, int64_t N, void* stream);

/* The same backward WITHOUT the transposed row gradients: dx[B,C,H,W] and dw[N, C*kH*kW] in one kernel.  A CTA
 * owns a few consecutive output rows of one image, sums in shared memory the part of dx they reach (all
 * channels x the input rows under those output rows x W) and adds it into dx with reductions (dx and dw are
 * zero-filled by the call; sums are formed in another order than mam_conv_bwd_f32 + mam_col2im_f32, so the
 * two agree to rounding).  mam_conv_bwd_direct_applies() answers without a device whether the geometry fits:
 * C * kH * W * 4 bytes plus the 16-byte-per-k table must fit one CTA's shared memory (226 KiB); otherwise
 * MAM_ERR_UNSUPPORTED and the caller takes the two-step form.  Stands in for the same reference text as
 * mam_conv_bwd_f32 (mamtorch/kernel/backup/mamconv2d_backward.txt:21-124). */
int mam_conv_bwd_direct_applies(int64_t B, int64_t C, int64_t H, int64_t W, int kH, int kW, int sh, int sw,
                                int ph, int pw);
int mam_conv_bwd_direct_f32(const float* x, const float* w, const float* grad,
                            const int32_t* argmax, const int32_t* argmin,
                            float* dx, float* dw, float scale,
                            int64_t B, int64_t C, int64_t H, int64_t W,
                            int kH, int kW, int sh, int sw, int ph, int pw, int64_t N, void* stream);

/* Forward of the MAM convolution WITHOUT materialised patch rows: the tiled kernels fetch every 32-channel
 * chunk of the patch rows from the channels-last input x_nhwc[B,H,W,C] by im2col-mode TMA
 * (cp.async.bulk.tensor.4d...im2col: the copy engine walks the output pixels, applies stride, padding and
 * the filter tap, and zero-fills outside the image).  w_taps is the weight as [N][(kw*kH + kh)*C + c], i.e.
 * weight.permute(0, 3, 2, 1) made contiguous: channels fastest, then kh, then kw -- the reduction order of the
 * reference's convolution text (k = c + C*(kh + kH*kw), mamtorch/kernel/backup/mamconv2d_forward.txt:128).
 * y / argmax / argmin are [B*Ho*Wo, N] (both index pointers NULL: values only); bias, dense, blend, alpha,
 * beta as in mam_fwd_f32.  Indices are RETURNED in the numbering k = (c*kH + kh)*kW + kw of
 * weight.view(N, -1), the one mam_conv_bwd_f32 and mam_col2im_f32 use; among equal products the one that
 * comes first in the reduction order above is chosen (with mam_im2col_f32 + mam_fwd_f32 it is the lowest k).
 * MAM_ERR_UNSUPPORTED where the copy engine cannot express the problem -- C % 32 != 0, padding > 127,
 * kernel extent > 128, stride > 8, pointers not 16-byte aligned, an input below 128 KiB, or a device
 * without the driver entry point: mam_conv_fwd_applies() answers that (pointer alignment apart) without a
 * device, and callers then take the patch-row route.  Stands in for mamconv2d_forward of the reference's
 * text backups (mamtorch/kernel/backup/mamconv2d_forward.txt:25-175) and the permutes around it
 * (mamtorch/kernel/backup/mamconv2d.txt:70-100). */
/* out[B,H,W,C] = x[B,C,H,W]: the channels-last copy mam_conv_fwd_f32 reads (one pass; B <= 65535). */
int mam_nchw_to_nhwc_f32(const float* x, float* out, int64_t B, int64_t C, int64_t H, int64_t W, void* stream);
int mam_conv_fwd_applies(int64_t B, int64_t C, int64_t H, int64_t W, int kH, int kW, int sh, int sw, int ph, int pw);
int mam_conv_fwd_f32(const float* x_nhwc, const float* w_taps, const float* bias, const float* dense, int blend,
                     float alpha, float beta, float* y, int32_t* argmax, int32_t* argmin,
                     int64_t B, int64_t C, int64_t H, int64_t W,
                     int kH, int kW, int sh, int sw, int ph, int pw, int64_t N, void* stream);

/* Selection hits: hit_max[n,k] += #rows m with argmax[m,n]==k, hit_min likewise ([N,K] int32,
 * accumulated into, so zero them first for per-call counts).  The device-side form of the
 * bookkeeping in FullyConnected.update_selection_count (mamtorch/nn/v4/fullyconnected.py:114-131). */
int mam_selcount_i32(const int32_t* argmax, const int32_t* argmin,
                     int32_t* hit_max, int32_t* hit_min,
                     int64_t M, int64_t K, int64_t N, void* stream);
/* count[i] += (hit_max[i]>0) + (hit_min[i]>0): exactly what one update_selection_count() call of
 * the reference adds to max_selection_count (mamtorch/nn/v4/fullyconnected.py:125-129). */
int mam_selcount_indicator_i32(const int32_t* hit_max, const int32_t* hit_min,
                               int32_t* count, int64_t n_elems, void* stream);

/* Dense product on the tcgen05 tensor cores: out[M,N] = c_out*out + c_acc*(a[M,K] . w[N,K]^T), TF32
 * inputs (10-bit mantissa), fp32 accumulation: the beta term of the blended layer.  Stands in for the
 * cuBLAS products in mamtorch/kernel/v3/csrc/cuda/fullyconnected.cu:153-160 and for dense_cuda
 * (mamtorch/kernel/v2/csrc/cuda/dense.cu:146-260).  Needs K % 4 == 0 and 16-byte aligned a, w
 * (otherwise MAM_ERR_UNSUPPORTED).  Agreement with an fp32 product: 1e-3 relative. */
int mam_dense_tf32(const float* a, const float* w, float* out, float c_acc, float c_out,
                   int64_t M, int64_t K, int64_t N, void* stream);

/* MAM forward on a pruned weight stored as CSR rows of W[N,K] (crow[N+1], col[nnz] ascending within
 * a row, val[nnz]; 64-bit indices as torch.Tensor.to_sparse_csr() produces).  Result = the dense
 * forward on W with zeros at the positions that are not stored: a missing position contributes a
 * product of 0 at its k (lowest-k tie rule included).  bias, argmax, argmin may be NULL.
 * The reference has no sparse MAM kernel; it runs the dense kernels on zeroed weights
 * (examples/vitb16_imagenet1k/pruning_utils.py:105-116).  Limit: K <= 50000. */
int mam_csr_fwd_f32(const float* a, const int64_t* crow, const int64_t* col, const float* val,
                    const float* bias, float* y, int32_t* argmax, int32_t* argmin,
                    int64_t M, int64_t K, int64_t N, void* stream);

/* The same forward through the tiled kernels, which need scratch memory from the caller: the
 * activations transposed (K x M floats), and the stored entries regrouped into 64-column stages
 * (16 bytes per entry plus 24 bytes per (row, stage) pair).  mam_csr_fwd_workspace_bytes returns the
 * size for these extents and nnz stored entries (0 when the tiled form does not apply: fewer than 32
 * rows of a, or extents beyond its 32-bit segment offsets); the workspace must be 256-byte aligned.
 * With workspace == NULL, or where the tiled form does not apply, the call runs mam_csr_fwd_f32.
 * Results are identical to mam_csr_fwd_f32; at 90 % sparsity and thousands of rows it is several
 * times faster (rows of a ride on the lanes, the stored weights are broadcast).  No counterpart in
 * the reference beyond the one named at mam_csr_fwd_f32. */
size_t mam_csr_fwd_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t nnz);
/* The same call for a weight that stays put between calls (inference on a pruned layer).  The workspace holds
 * the regrouped weight first -- mam_csr_fwd_entries_bytes(K, N, nnz) bytes, independent of M -- and the
 * transposed activations after it.  With entries_ready != 0 the regrouping kernels are skipped: the caller
 * vouches that this workspace was last written by a call with the same crow / col / val contents, K, N and
 * nnz (M may differ; the workspace must hold mam_csr_fwd_workspace_bytes for the M of this call).  With
 * entries_ready == 2 the caller vouches for crow, col, K, N and nnz only -- the sparsity pattern -- and the
 * stored values are regrouped again in one pass: a training step, where the mask stays and the values move.
 * With entries_ready == 0 it is mam_csr_fwd_ws_f32. */
size_t mam_csr_fwd_entries_bytes(int64_t K, int64_t N, int64_t nnz);
int mam_csr_fwd_ws_ex_f32(const float* a, const int64_t* crow, const int64_t* col, const float* val, int64_t nnz,
                          const float* bias, float* y, int32_t* argmax, int32_t* argmin,
                          int64_t M, int64_t K, int64_t N,
                          void* workspace, size_t workspace_bytes, int entries_ready, void* stream);
int mam_csr_fwd_ws_f32(const float* a, const int64_t* crow, const int64_t* col, const float* val, int64_t nnz,
                       const float* bias, float* y, int32_t* argmax, int32_t* argmin,
                       int64_t M, int64_t K, int64_t N,
                       void* workspace, size_t workspace_bytes, void* stream);

/* c[N,Mc] = A_csr[N,K] . b[K,Mc], ordinary sum.  Stands in for cusparsemm_csr / cusparsemm_coo
 * (mamtorch/sparse/kernel/v1/csrc/cuda/cusparsemm_csr.cu:19-77, cusparsemm_coo.cu:19-76). */
int mam_spmm_csr_f32(const int64_t* crow, const int64_t* col, const float* val, const float* b,
                     float* c, int64_t N, int64_t K, int64_t Mc, void* stream);

/* The same product through the tiled kernel, which wants scratch from the caller for the regrouped
 * entries (8 bytes per entry plus 12 bytes per (row, 64-column stage) pair; 256-byte aligned;
 * mam_spmm_csr_workspace_bytes returns 0 where the tiled form does not apply or does not pay: Mc < 64,
 * Mc % 4 != 0, fewer than two stored entries per (row, stage) pair on average, less than ~1e9
 * multiply-adds, or extents beyond its 32-bit offsets).  With workspace == NULL, or where the tiled
 * form cannot run (Mc < 64, Mc % 4 != 0, b or c not 16-byte aligned), the call runs mam_spmm_csr_f32; a
 * caller that passes a large enough workspace although the query answered 0 for lack of work still
 * gets the tiled kernel.  Entries of a row are summed in ascending column order in both. */
size_t mam_spmm_csr_workspace_bytes(int64_t N, int64_t K, int64_t Mc, int64_t nnz);
int mam_spmm_csr_ws_f32(const int64_t* crow, const int64_t* col, const float* val, int64_t nnz,
                        const float* b, float* c, int64_t N, int64_t K, int64_t Mc,
                        void* workspace, size_t workspace_bytes, void* stream);

/* out[C,R] = transpose(in[R,C]); replaces the .T.contiguous() copies of the reference's glue
 * (mamtorch/nn/v4/fullyconnected.py:141, mamtorch/kernel/v4/csrc/cuda/fullyconnected.cu:66). */
int mam_transpose_f32(const float* in, float* out, int64_t R, int64_t C, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MAM_B200_H */
