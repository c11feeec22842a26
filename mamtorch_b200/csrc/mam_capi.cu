// C ABI of libmam_b200.so: argument checking, path selection, tensor-map encoding and launches.
// Declarations and the reference interfaces each entry point replaces are in include/mam_b200.h.
#include <cstdio>
#include <cstring>
#include <mutex>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/mam_b200.h"
#include "../../include/mam_b200_tuning.h"
#include "mam_bwd.cuh"
#include "mam_conv.cuh"
#include "mam_csr.cuh"
#include "mam_csr_tiled.cuh"
#include "mam_dense_tf32.cuh"
#include "mam_fwd_generic.cuh"
#include "mam_fwd_tiled.cuh"

using namespace mamb200;

namespace {

thread_local cudaError_t t_last_cuda = cudaSuccess;
__device__ int g_wait_gave_up = 0;  // set by kernels whose bounded wait ran out

int cuda_fail(cudaError_t e) {
    t_last_cuda = e;
    return MAM_ERR_CUDA;
}
#define MAM_CUDA(x)                                  \
    do {                                             \
        cudaError_t e_ = (x);                        \
        if (e_ != cudaSuccess) return cuda_fail(e_); \
    } while (0)

struct DevInfo {
    int valid = 0, sms = 0, major = 0, minor = 0, max_smem = 0;
};
DevInfo g_dev[64];

int device_info(const DevInfo** out) {
    int dev = 0;
    MAM_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return MAM_ERR_UNSUPPORTED;
    DevInfo& d = g_dev[dev];
    if (!d.valid) {
        MAM_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev));
        MAM_CUDA(cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev));
        MAM_CUDA(cudaDeviceGetAttribute(&d.minor, cudaDevAttrComputeCapabilityMinor, dev));
        MAM_CUDA(cudaDeviceGetAttribute(&d.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        d.valid = 1;
    }
    *out = &d;
    return d.major == 10 ? MAM_OK : MAM_ERR_NOT_SM100;
}

// ---- optional per-kernel event timing (mam_timer_arm) ----
struct KernelTimer {
    void** starts = nullptr;
    void** stops = nullptr;
    int capacity = 0, count = 0, kernel_id = -1;
} g_timer;

struct TimedLaunch {
    bool on;
    cudaStream_t st;
    TimedLaunch(int kernel_id, cudaStream_t s) : st(s) {
        on = g_timer.kernel_id == kernel_id && g_timer.count < g_timer.capacity;
        if (on) cudaEventRecord((cudaEvent_t)g_timer.starts[g_timer.count], st);
    }
    ~TimedLaunch() {
        if (on) {
            cudaEventRecord((cudaEvent_t)g_timer.stops[g_timer.count], st);
            ++g_timer.count;
        }
    }
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_encode() {
    if (g_encode) return MAM_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    MAM_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || !fn) return cuda_fail(cudaErrorNotSupported);
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return MAM_OK;
}

// [rows, K] fp32 row-major matrix -> boxes of [box_rows][32 floats], 128-byte swizzle (or none), zero fill.
// pitch: floats between the starts of consecutive rows (0: K), for a matrix that is a column slice of a wider one
int encode_rows_k(CUtensorMap* tm, const float* base, long long rows, long long K, int box_rows,
                  bool swizzle = true, long long pitch = 0) {
    int st = get_encode();
    if (st != MAM_OK) return st;
    cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t gstr[1] = {(cuuint64_t)(pitch ? pitch : K) * 4};
    cuuint32_t box[2] = {(cuuint32_t)FWD_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), gdim, gstr, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
    return MAM_OK;
}

// [outer][inner] fp32 matrix with a row pitch in bytes -> boxes of [box_outer][box_inner], no swizzle, zero fill.
int encode_2d_plain(CUtensorMap* tm, const float* base, long long inner, long long outer, long long pitch_bytes,
                    int box_inner, int box_outer) {
    int st = get_encode();
    if (st != MAM_OK) return st;
    cuuint64_t gdim[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t gstr[1] = {(cuuint64_t)pitch_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), gdim, gstr, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
    return MAM_OK;
}

typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeIm2colFn g_encode_im2col = nullptr;

// The convolution input the patch rows are read from: channels-last [B][H][W][C] floats.
struct ConvSrc {
    const float* x_nhwc;
    ConvGeom g;
};

// Im2col-mode map over the channels-last input: boxes of `pixels` consecutive output pixels x 32
// channels.  The pixel box is the set of base pixels (top-left patch corners): from -pad to
// extent + pad - (k - 1) exclusive, walked with the convolution stride; the filter tap comes with
// every load as an offset.  Zero fill outside the image.
int encode_im2col_rows(CUtensorMap* tm, const ConvSrc& cv, int pixels, bool swizzle) {
    if (!g_encode_im2col) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        MAM_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !fn) return cuda_fail(cudaErrorNotSupported);
        g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
    }
    const ConvGeom& g = cv.g;
    cuuint64_t gdim[4] = {(cuuint64_t)g.C, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.B};
    cuuint64_t gstr[3] = {(cuuint64_t)g.C * 4, (cuuint64_t)g.W * g.C * 4, (cuuint64_t)g.H * g.W * g.C * 4};
    int lower[2] = {-g.pw, -g.ph};
    int upper[2] = {g.pw - (g.kW - 1), g.ph - (g.kH - 1)};
    cuuint32_t estr[4] = {1, (cuuint32_t)g.sw, (cuuint32_t)g.sh, 1};
    CUresult r = g_encode_im2col(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(cv.x_nhwc), gdim, gstr,
                                 lower, upper, (cuuint32_t)FWD_BK, (cuuint32_t)pixels, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
    return MAM_OK;
}

template <class Cfg, bool CONV = false>
int launch_tiled(const float* a, const float* w, const FwdParams& prm, const DevInfo& d, cudaStream_t st,
                 const ConvSrc* cv = nullptr) {
    if (Cfg::SMEM_BYTES > d.max_smem) return MAM_ERR_UNSUPPORTED;
    if (CONV != (cv != nullptr)) return MAM_ERR_INVALID_ARGUMENT;
    CUtensorMap tmA, tmW;
    int s = CONV ? encode_im2col_rows(&tmA, *cv, Cfg::BM, true) : encode_rows_k(&tmA, a, prm.M, prm.K, Cfg::BM);
    if (s != MAM_OK) return s;
    s = encode_rows_k(&tmW, w, prm.N, prm.K, Cfg::BN);
    if (s != MAM_OK) return s;
    MAM_CUDA(cudaFuncSetAttribute(mam_fwd_tiled_kernel<Cfg, CONV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  Cfg::SMEM_BYTES));
    const long long ntiles = ((prm.M + Cfg::BM - 1) / Cfg::BM) * ((prm.N + Cfg::BN - 1) / Cfg::BN);
    const int grid = (int)(ntiles < d.sms ? ntiles : d.sms);
    {
        TimedLaunch t(MAM_KERNEL_FWD_TILED, st);
        mam_fwd_tiled_kernel<Cfg, CONV><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(tmA, tmW, prm);
    }
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

//                         TM TN WM WN ST track UQ batch mul2
using ValCfg0 = FwdCfg<8, 8, 4, 2, 4, false, 1, false, false>;  // 128x128 tile, 256 threads, scalar multiplies
using ValCfg1 = FwdCfg<8, 8, 4, 2, 4, false, 2, false>;
using ValCfg2 = FwdCfg<8, 8, 4, 2, 4, false, 1, false>;
using ValCfg3 = FwdCfg<4, 8, 6, 2, 4, false, 2, false>;         // 96x128 tile, 384 threads
using ValCfg4 = FwdCfg<4, 8, 4, 3, 4, false, 2, false>;         // 64x192 tile, 384 threads
using ValCfg5 = FwdCfg<4, 8, 4, 2, 4, false, 2, false, false>;  // 64x128 tile, 256 threads, scalar multiplies
using ValCfg6 = FwdCfg<4, 8, 4, 2, 4, false, 2, true>;          // 64x128 tile, 256 threads
using ValCfg7 = FwdCfg<4, 4, 8, 2, 6, false, 4, false>;         // 128x64 tile, 512 threads
using SplitCfg = FwdCfg<4, 8, 4, 2, 4, false, 2, false, true, true>;   // 64x128 tile, slices of K summed in the kernel
using SplitIdxCfg = FwdCfg<4, 8, 4, 2, 4, true, 2, false, true, true>;  // the same with chunk ids per slice
using IdxCfg0 = FwdCfg<4, 8, 4, 2, 4, true, 1, false, true, false, true>;   // as IdxCfg2 with the paired-warp row mapping
using IdxCfg1 = FwdCfg<4, 8, 4, 2, 4, true, 2, false, true, false, true>;   // as IdxCfg0, k loop unrolled twice
using IdxCfg2 = FwdCfg<4, 8, 4, 2, 4, true, 1, false>;
using IdxCfg3 = FwdCfg<4, 4, 4, 4, 4, true, 1, false>;          // 64x128 tile, 512 threads
using IdxCfg4 = FwdCfg<8, 4, 2, 4, 4, true, 1, false, true, false, true>;   // 8x4 outputs per thread, paired-warp rows
using IdxCfg5 = FwdCfg<8, 4, 2, 4, 4, true, 2, false>;          // 64x128 tile, 256 threads, A-heavy
using IdxCfg6 = FwdCfg<4, 4, 4, 4, 4, true, 4, false>;          // 64x128 tile, 512 threads
using IdxCfg7 = FwdCfg<4, 4, 4, 4, 4, true, 1, false, true, false, true>;   // 64x128 tile, 512 threads, paired-warp rows
constexpr int N_VARIANTS = 8;
const char* kValNames[N_VARIANTS] = {"val_8x8_t128x128_c256_u1_scalar", "val_8x8_t128x128_c256_u2",
                                     "val_8x8_t128x128_c256_u1", "val_4x8_t96x128_c384_u2", "val_4x8_t64x192_c384_u2",
                                     "val_4x8_t64x128_c256_u2_scalar", "val_4x8_t64x128_c256_u2b",
                                     "val_4x4_t128x64_c512_u4"};
const char* kIdxNames[N_VARIANTS] = {"idx_4x8_t64x128_c256_u1_row8", "idx_4x8_t64x128_c256_u2_row8",
                                     "idx_4x8_t64x128_c256_u1", "idx_4x4_t64x128_c512_u1",
                                     "idx_8x4_t64x128_c256_u1_row8", "idx_8x4_t64x128_c256_u2",
                                     "idx_4x4_t64x128_c512_u4", "idx_4x4_t64x128_c512_u1_row8"};
int g_variant[2] = {-1, -1};  // [with_indices]
int g_resolve_simple = 0;      // 1: use the thread-per-output resolver (cross-check)

// Scratch for mam_fwd_kn_static_f32: lives in the library image, one copy per device.
static __device__ __align__(256) unsigned char g_static_scratch[MAM_STATIC_SCRATCH_BYTES];
void* g_static_scratch_addr[64] = {nullptr};  // device address per device, looked up on first use
std::mutex g_static_scratch_mutex;

int bad_ptr(const void* p) { return p == nullptr; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
size_t round256(size_t x) { return (x + 255) & ~size_t(255); }

template <int R>
int launch_csr(const float* a, const int64_t* crow, const int64_t* col, const float* val, const float* bias,
                      float* y, int32_t* argmax, int32_t* argmin, int64_t M, int64_t K, int64_t N, cudaStream_t cs) {
    const size_t smem = ((size_t)R * (size_t)K + (size_t)CSR_WARPS * 3 * R * 32) * 4;
    MAM_CUDA(cudaFuncSetAttribute(mam_csr_fwd_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long grid = (M + R - 1) / R;
    if (grid > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    mam_csr_fwd_kernel<R><<<(unsigned)grid, CSR_WARPS * 32, smem, cs>>>(
        a, reinterpret_cast<const long long*>(crow), reinterpret_cast<const long long*>(col), val, bias, y, argmax,
        argmin, M, K, N);
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

// Tile configuration of the tiled forward for an M x N problem.
int auto_variant(bool want_idx, int64_t M, int64_t N, const DevInfo& d) {
    // 4x8 outputs per thread, 64x128 tile, the k loop not unrolled beyond one 16-byte group, paired-warp row
    // mapping: the fastest of the index-producing forms at 12608x768x3072, 12608x3072x768 and 4096^3 alike
    // (2.70 / 2.60 / 6.00 ms; the same without the row mapping 2.76 / 2.65 / 6.13; the 512-thread 4x4 form wins
    // only the first of the three, 2.67)
    if (want_idx) return 0;
    // Candidates differ in speed per unit (measured, units/clk/SM) and in how well their tile
    // count fills whole waves of SMs; pick the best product of the two.
    struct Cand { int variant; long long bm, bn; double rate; };
    const Cand cands[3] = {{2, 128, 128, 42.9}, {3, 96, 128, 40.4}, {6, 64, 128, 41.0}};
    double best = -1.0;
    int variant = 2;
    for (const Cand& c : cands) {
        const long long tiles = ((M + c.bm - 1) / c.bm) * ((N + c.bn - 1) / c.bn);
        const long long waves = (tiles + d.sms - 1) / d.sms;
        // work actually executed includes the padding of edge tiles
        const double useful = (double)M * (double)N / ((double)waves * d.sms * c.bm * c.bn);
        if (useful * c.rate > best) {
            best = useful * c.rate;
            variant = c.variant;
        }
    }
    return variant;
}

// What the im2col-mode loads can express: whole 32-channel chunks, corners and tap offsets inside the
// instruction's fields ([-128, 127] and [0, 255] for two spatial dimensions), strides up to 8, and an
// input of at least 128 KiB (smaller im2col maps are not encoded reliably by current drivers).
bool conv_implicit_applies(const ConvGeom& g, const float* x_nhwc) {
    if (g.C % 32 != 0 || !aligned16(x_nhwc)) return false;
    if (g.pw > 127 || g.ph > 127 || g.kW > 128 || g.kH > 128 || g.sw > 8 || g.sh > 8) return false;
    if (g.pw - (g.kW - 1) < -128 || g.ph - (g.kH - 1) < -128) return false;
    if ((long long)g.B * g.H * g.W * g.C * 4 < 131072) return false;
    if ((long long)g.C * g.kH * g.kW / FWD_BK >= 65535) return false;
    return true;
}

int run_resolver(const float* a, const float* w, int32_t* argmax, int32_t* argmin, int64_t M, int64_t K, int64_t N,
                 int64_t pitch, int k_offset, int* flag, const Im2colRows& conv, cudaStream_t cs, const ConvSrc* cv);

// The tiled forward (and, with indices, the resolver behind it) on K-contiguous operands a[M,K] (or,
// with `cv`, patch rows read from a channels-last convolution input) and w[N,K].
int run_tiled(const float* a, const float* w, float* y, int32_t* argmax, int32_t* argmin, int64_t M, int64_t K,
              int64_t N, const EpilogueArgs& ep, int variant, const DevInfo& d, cudaStream_t cs, const ConvSrc* cv) {
    const bool want_idx = argmax != nullptr;
    int st = MAM_OK;
    int* flag = nullptr;
    MAM_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&flag), g_wait_gave_up));
    FwdParams prm{y, argmax, argmin, M, K, N, ep, 1.0f, flag, Im2colRows{}, 0};
    if (cv) {
        const ConvGeom& g = cv->g;
        prm.conv = Im2colRows{g.C / 32, g.C, g.kH, g.kW, g.Ho, g.Wo, g.sh, g.sw, g.ph, g.pw};
    }
    if (cv) {
        // patch rows by im2col-mode TMA: the configurations the automatic choice makes (the tuning
        // selector of mam_tune_set applies to the matrix form only)
        if (!want_idx) {
            switch (auto_variant(false, M, N, d)) {
                case 3: return launch_tiled<ValCfg3, true>(a, w, prm, d, cs, cv);
                case 6: return launch_tiled<ValCfg6, true>(a, w, prm, d, cs, cv);
                default: return launch_tiled<ValCfg2, true>(a, w, prm, d, cs, cv);
            }
        }
        st = g_variant[1] == 1 ? launch_tiled<IdxCfg1, true>(a, w, prm, d, cs, cv)
                               : launch_tiled<IdxCfg0, true>(a, w, prm, d, cs, cv);
    } else if (!want_idx) {
        switch (variant) {
            case 0: st = launch_tiled<ValCfg0>(a, w, prm, d, cs); break;
            case 1: st = launch_tiled<ValCfg1>(a, w, prm, d, cs); break;
            case 2: st = launch_tiled<ValCfg2>(a, w, prm, d, cs); break;
            case 3: st = launch_tiled<ValCfg3>(a, w, prm, d, cs); break;
            case 4: st = launch_tiled<ValCfg4>(a, w, prm, d, cs); break;
            case 5: st = launch_tiled<ValCfg5>(a, w, prm, d, cs); break;
            case 6: st = launch_tiled<ValCfg6>(a, w, prm, d, cs); break;
            default: st = launch_tiled<ValCfg7>(a, w, prm, d, cs); break;
        }
        return st;
    } else {
        switch (variant) {
            case 0: st = launch_tiled<IdxCfg0>(a, w, prm, d, cs); break;
            case 1: st = launch_tiled<IdxCfg1>(a, w, prm, d, cs); break;
            case 2: st = launch_tiled<IdxCfg2>(a, w, prm, d, cs); break;
            case 3: st = launch_tiled<IdxCfg3>(a, w, prm, d, cs); break;
            case 4: st = launch_tiled<IdxCfg4>(a, w, prm, d, cs); break;
            case 5: st = launch_tiled<IdxCfg5>(a, w, prm, d, cs); break;
            case 6: st = launch_tiled<IdxCfg6>(a, w, prm, d, cs); break;
            default: st = launch_tiled<IdxCfg7>(a, w, prm, d, cs); break;
        }
    }
    if (st != MAM_OK) return st;
    return run_resolver(a, w, argmax, argmin, M, K, N, 0, 0, flag, prm.conv, cs, cv);
}

// Chunk ids -> exact indices.  pitch / k_offset: the operands are the column slice [k_offset, k_offset + K) of
// matrices whose rows are `pitch` floats apart (0: K); a and w already point at the slice's first column.
int run_resolver(const float* a, const float* w, int32_t* argmax, int32_t* argmin, int64_t M, int64_t K, int64_t N,
                 int64_t pitch, int k_offset, int* flag, const Im2colRows& conv, cudaStream_t cs, const ConvSrc* cv) {
    int st = MAM_OK;
    const int nkc = (int)((K + FWD_BK - 1) / FWD_BK);
    if (cv && nkc > ResolveCfg::NK_MAX) return MAM_ERR_UNSUPPORTED;
    if (pitch && (nkc > ResolveCfg::NK_MAX || g_resolve_simple != 0)) return MAM_ERR_UNSUPPORTED;
    if ((nkc <= ResolveCfg::NK_MAX && g_resolve_simple == 0) || cv) {
        CUtensorMap tmA, tmW;
        st = cv ? encode_im2col_rows(&tmA, *cv, ResolveCfg::RM, false)
                : encode_rows_k(&tmA, a, M, K, ResolveCfg::RM, false, pitch);
        if (st != MAM_OK) return st;
        st = encode_rows_k(&tmW, w, N, K, ResolveCfg::RN, false, pitch);
        if (st != MAM_OK) return st;
        const long long tiles = ((M + ResolveCfg::RM - 1) / ResolveCfg::RM) * ((N + ResolveCfg::RN - 1) / ResolveCfg::RN);
        if (tiles > 2147483647LL) return MAM_ERR_UNSUPPORTED;
        const int rsmem = ResolveCfg::smem_bytes(nkc);
        TimedLaunch t(MAM_KERNEL_FWD_RESOLVE, cs);
        if (cv) {
            MAM_CUDA(cudaFuncSetAttribute(mam_resolve_tiled_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          rsmem));
            mam_resolve_tiled_kernel<true><<<(unsigned)tiles, ResolveCfg::THREADS, rsmem, cs>>>(
                tmA, tmW, argmax, argmin, M, K, N, flag, conv, 0);
        } else {
            MAM_CUDA(cudaFuncSetAttribute(mam_resolve_tiled_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          rsmem));
            mam_resolve_tiled_kernel<false><<<(unsigned)tiles, ResolveCfg::THREADS, rsmem, cs>>>(
                tmA, tmW, argmax, argmin, M, K, N, flag, conv, k_offset);
        }
    } else {
        const long long total = M * N;
        const long long blocks = (total + 255) / 256;
        if (blocks > 2147483647LL) return MAM_ERR_UNSUPPORTED;
        TimedLaunch t(MAM_KERNEL_FWD_RESOLVE, cs);
        mam_resolve_kernel<<<(unsigned)blocks, 256, 0, cs>>>(a, w, argmax, argmin, M, K, N);
    }
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int g_dense_split = 1;  // 0: the TF32 product runs whole tiles only (cross-check / timing selector)
int g_conv_direct_rows = 0;  // 0 auto, else output rows per CTA of mam_conv_bwd_direct_kernel (if they fit)
int g_bwd_mode = 0;  // 0 auto, 1 CTA-shared rows, 2 two kernels, 3 row per warp (a parked in shared memory where it fits), 4 row per warp (a read from L1)

// K for which the automatic choice takes the row-per-warp gradient kernel (measured, see mam_bwd_count_ws_f32)
bool bwd_rowwarp_band(int64_t K) { return g_bwd_mode == 0 && K >= 640 && K <= 832; }

template <bool NK>
int launch_bwd_split(const float* a, const float* b, const float* grad, const int32_t* argmax, const int32_t* argmin,
                     float* da, float* db, int32_t* hit_max, int32_t* hit_min, float scale, int64_t M, int64_t K,
                     int64_t N, int rows, int cols, cudaStream_t cs) {
    const size_t smem_dx = (size_t)rows * (size_t)K * 4;
    MAM_CUDA(cudaFuncSetAttribute(mam_bwd_dx_kernel<NK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dx));
    {
        TimedLaunch t(MAM_KERNEL_BWD, cs);
        mam_bwd_dx_kernel<NK><<<(unsigned)((M + rows - 1) / rows), BWD_THREADS, smem_dx, cs>>>(
            b, grad, argmax, argmin, da, M, K, N, rows, scale);
    }
    MAM_CUDA(cudaGetLastError());
    const bool count = hit_max != nullptr;
    const size_t smem_dw = (size_t)cols * (size_t)K * 4 * (count ? 3 : 1);
    const unsigned grid = (unsigned)((N + cols - 1) / cols);
    TimedLaunch t(MAM_KERNEL_BWD, cs);
    if (count) {
        MAM_CUDA(cudaFuncSetAttribute(mam_bwd_dw_kernel<NK, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem_dw));
        mam_bwd_dw_kernel<NK, true><<<grid, BWD_THREADS, smem_dw, cs>>>(a, grad, argmax, argmin, db, hit_max, hit_min,
                                                                        M, K, N, cols, scale);
    } else {
        MAM_CUDA(cudaFuncSetAttribute(mam_bwd_dw_kernel<NK, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem_dw));
        mam_bwd_dw_kernel<NK, false><<<grid, BWD_THREADS, smem_dw, cs>>>(a, grad, argmax, argmin, db, nullptr, nullptr,
                                                                         M, K, N, cols, scale);
    }
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}
}  // namespace

extern "C" {

const char* mam_status_str(int status) {
    switch (status) {
        case MAM_OK: return "ok";
        case MAM_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, non-positive extent or bad layout code)";
        case MAM_ERR_UNSUPPORTED: return "extent outside what the kernels support";
        case MAM_ERR_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
        case MAM_ERR_CUDA: return "a CUDA call failed (see mam_last_cuda_error)";
        case MAM_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up; results are invalid";
        case MAM_ERR_NOT_SM100: return "the current device is not compute capability 10.x (B200)";
        case MAM_ERR_STATIC_SCRATCH:
            return "the problem needs more scratch than the library's built-in static buffer "
                   "(MAM_STATIC_SCRATCH_BYTES); use mam_fwd_f32 with a caller-provided workspace";
        default: return "unknown status";
    }
}

int mam_abi_version(void) { return MAM_ABI_VERSION; }

const char* mam_last_cuda_error(void) { return cudaGetErrorString(t_last_cuda); }

int mam_check_device_flag(void) {
    MAM_CUDA(cudaDeviceSynchronize());
    int flag = 0;
    MAM_CUDA(cudaMemcpyFromSymbol(&flag, g_wait_gave_up, sizeof(int)));
    if (flag) {
        int zero = 0;
        MAM_CUDA(cudaMemcpyToSymbol(g_wait_gave_up, &zero, sizeof(int)));
        return MAM_ERR_DEVICE_TIMEOUT;
    }
    return MAM_OK;
}

int mam_poll_device_flag(void* stream) {
    int dev = 0;
    MAM_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return MAM_ERR_UNSUPPORTED;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    MAM_CUDA(cudaStreamIsCapturing((cudaStream_t)stream, &cap));
    if (cap != cudaStreamCaptureStatusNone) return MAM_OK;   // nothing is fetched or reported inside a capture
    // one pinned int per device: the landing place of the asynchronous fetches
    static int* mirror[64] = {nullptr};
    if (mirror[dev] == nullptr) {
        int* p = nullptr;
        MAM_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&p), sizeof(int), cudaHostAllocDefault));
        *p = 0;
        mirror[dev] = p;
    }
    const int seen = *reinterpret_cast<volatile int*>(mirror[dev]);
    if (seen) {
        // report once: clear the device flag and the copy (this path may wait for the device)
        int zero = 0;
        MAM_CUDA(cudaMemcpyToSymbol(g_wait_gave_up, &zero, sizeof(int)));
        *mirror[dev] = 0;
        return MAM_ERR_DEVICE_TIMEOUT;
    }
    MAM_CUDA(cudaMemcpyFromSymbolAsync(mirror[dev], g_wait_gave_up, sizeof(int), 0, cudaMemcpyDeviceToHost,
                                       (cudaStream_t)stream));
    return MAM_OK;
}

int mam_timer_arm(void** starts, void** stops, int capacity, int kernel_id) {
    if (!starts || !stops || capacity <= 0) return MAM_ERR_INVALID_ARGUMENT;
    g_timer.starts = starts;
    g_timer.stops = stops;
    g_timer.capacity = capacity;
    g_timer.count = 0;
    g_timer.kernel_id = kernel_id;
    return MAM_OK;
}

int mam_timer_disarm(void) {
    const int n = g_timer.count;
    g_timer = KernelTimer();
    return n;
}

int mam_tune_set(int knob, int value) {
    switch (knob) {
        case MAM_TUNE_FWD_VALUES:
        case MAM_TUNE_FWD_INDICES:
            if (value < -2 || value >= N_VARIANTS) return MAM_ERR_INVALID_ARGUMENT;
            g_variant[knob == MAM_TUNE_FWD_INDICES ? 1 : 0] = value;
            return MAM_OK;
        case MAM_TUNE_RESOLVER:
            g_resolve_simple = value ? 1 : 0;
            return MAM_OK;
        case MAM_TUNE_BWD_FORM:
            if (value < 0 || value > 4) return MAM_ERR_INVALID_ARGUMENT;
            g_bwd_mode = value;
            return MAM_OK;
        case MAM_TUNE_DENSE_SPLIT:
            g_dense_split = value ? 1 : 0;
            return MAM_OK;
        case MAM_TUNE_CONV_DIRECT_ROWS:
            if (value < 0 || value > 64) return MAM_ERR_INVALID_ARGUMENT;
            g_conv_direct_rows = value;
            return MAM_OK;
        default:
            return MAM_ERR_INVALID_ARGUMENT;
    }
}

const char* mam_fwd_variant_name(int with_indices, int variant) {
    if (variant == -1) return "auto";
    if (variant == -2) return "generic";
    if (variant < 0 || variant >= N_VARIANTS) return "";
    return with_indices ? kIdxNames[variant] : kValNames[variant];
}

size_t mam_fwd_workspace_bytes(int64_t M, int64_t K, int64_t N, int b_layout, int want_indices) {
    (void)M;
    (void)want_indices;
    if (b_layout == MAM_B_KN && K > 0 && N > 0 && K % 4 == 0) return round256((size_t)K * (size_t)N * 4);
    return 0;
}

int mam_transpose_f32(const float* in, float* out, int64_t R, int64_t C, void* stream) {
    if (bad_ptr(in) || bad_ptr(out) || R <= 0 || C <= 0) return MAM_ERR_INVALID_ARGUMENT;
    const long long gx = (C + 31) / 32, gy = (R + 31) / 32;
    if (gy > 65535 || gx > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    mam_transpose_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, (cudaStream_t)stream>>>(in, out, R, C);
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int mam_nchw_to_nhwc_f32(const float* x, float* out, int64_t B, int64_t C, int64_t H, int64_t W, void* stream) {
    if (bad_ptr(x) || bad_ptr(out) || B <= 0 || C <= 0 || H <= 0 || W <= 0) return MAM_ERR_INVALID_ARGUMENT;
    const long long hw = H * W;
    const long long gx = (hw + 31) / 32, gy = (C + 31) / 32;
    if (gy > 65535 || B > 65535 || gx > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    mam_transpose_batched_kernel<<<dim3((unsigned)gx, (unsigned)gy, (unsigned)B), 256, 0, (cudaStream_t)stream>>>(
        x, out, C, hw);
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

namespace {
// rate in [0, 1) -> threshold on a 32-bit draw; false if the rate is out of range
bool drop_threshold(float rate, unsigned* thr) {
    if (!(rate >= 0.f && rate < 1.f)) return false;
    const double t = (double)rate * 4294967296.0;
    *thr = t >= 4294967295.0 ? 4294967295u : (unsigned)t;
    return true;
}
}  // namespace

int mam_fwd_f32(const float* a, const float* b, int b_layout, const float* bias, const float* dense, int blend,
                float alpha, float beta, float* y, int32_t* argmax, int32_t* argmin, int64_t M, int64_t K,
                int64_t N, void* workspace, size_t workspace_bytes, void* stream) {
    return mam_fwd_drop_f32(a, b, b_layout, bias, dense, blend, alpha, beta, 0.f, 0, y, argmax, argmin, M, K, N,
                            workspace, workspace_bytes, stream);
}

int mam_drop_f32(const float* in, float* out, int64_t n, float rate, float scale, uint64_t seed, void* stream) {
    unsigned thr = 0;
    if (bad_ptr(in) || bad_ptr(out) || n <= 0 || !drop_threshold(rate, &thr)) return MAM_ERR_INVALID_ARGUMENT;
    const long long blocks = (n + 255) / 256;
    if (blocks > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    mam_drop_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(in, out, n, seed, thr, scale);
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int mam_fwd_drop_f32(const float* a, const float* b, int b_layout, const float* bias, const float* dense, int blend,
                     float alpha, float beta, float drop_rate, uint64_t drop_seed, float* y, int32_t* argmax,
                     int32_t* argmin, int64_t M, int64_t K, int64_t N, void* workspace, size_t workspace_bytes,
                     void* stream) {
    if (bad_ptr(a) || bad_ptr(b) || bad_ptr(y) || M <= 0 || K <= 0 || N <= 0) return MAM_ERR_INVALID_ARGUMENT;
    if (b_layout != MAM_B_KN && b_layout != MAM_B_NK) return MAM_ERR_INVALID_ARGUMENT;
    if ((argmax == nullptr) != (argmin == nullptr)) return MAM_ERR_INVALID_ARGUMENT;
    if (K >= (1LL << 31) || N >= (1LL << 31) || M >= (1LL << 31)) return MAM_ERR_UNSUPPORTED;
    const DevInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MAM_OK) return st;
    cudaStream_t cs = (cudaStream_t)stream;
    const bool want_idx = argmax != nullptr;
    EpilogueArgs ep{bias, dense, alpha, beta, blend};
    if (drop_rate != 0.f) {
        if (!drop_threshold(drop_rate, &ep.drop_threshold)) return MAM_ERR_INVALID_ARGUMENT;
        ep.drop_seed = drop_seed;
        ep.drop_scale = 1.0f / (1.0f - drop_rate);
    }

    int variant = g_variant[want_idx ? 1 : 0];
    const bool tma_ok = (K % 4 == 0) && aligned16(a) && aligned16(b) && K / FWD_BK < 65535;
    if (variant == -1) {
        if (!(tma_ok && M * N >= 4096)) {
            variant = -2;
        } else {
            variant = auto_variant(want_idx, M, N, *d);
        }
    }
    if (variant >= 0 && !tma_ok) variant = -2;

    if (variant == -2) {
        const long long gx = (N + GEN_TILE - 1) / GEN_TILE, gy = (M + GEN_TILE - 1) / GEN_TILE;
        if (gy > 65535) return MAM_ERR_UNSUPPORTED;
        dim3 grid((unsigned)gx, (unsigned)gy);
        TimedLaunch t(MAM_KERNEL_FWD_GENERIC, cs);
        if (b_layout == MAM_B_NK)
            mam_fwd_generic_kernel<true><<<grid, 256, 0, cs>>>(a, b, y, argmax, argmin, M, K, N, ep);
        else
            mam_fwd_generic_kernel<false><<<grid, 256, 0, cs>>>(a, b, y, argmax, argmin, M, K, N, ep);
        MAM_CUDA(cudaGetLastError());
        return MAM_OK;
    }

    const float* w = b;
    if (b_layout == MAM_B_KN) {
        const size_t need = round256((size_t)K * (size_t)N * 4);
        if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
            return MAM_ERR_WORKSPACE;
        st = mam_transpose_f32(b, static_cast<float*>(workspace), K, N, stream);
        if (st != MAM_OK) return st;
        w = static_cast<const float*>(workspace);
    }
    return run_tiled(a, w, y, argmax, argmin, M, K, N, ep, variant, *d, cs, nullptr);
}

int mam_fwd_splits_f32(const float* a, const float* w, const float* bias, const float* dense, int blend, float alpha,
                       float beta, float* y, int64_t M, int64_t K, int64_t N, int64_t split_width, void* stream) {
    if (bad_ptr(a) || bad_ptr(w) || bad_ptr(y) || M <= 0 || K <= 0 || N <= 0 || split_width <= 0)
        return MAM_ERR_INVALID_ARGUMENT;
    if (K >= (1LL << 31) || N >= (1LL << 31) || M >= (1LL << 31)) return MAM_ERR_UNSUPPORTED;
    // slices must end on chunk boundaries and there must be more than one of them
    if (split_width % FWD_BK != 0 || split_width >= K || K % 4 != 0 || !aligned16(a) || !aligned16(w) ||
        K / FWD_BK >= 65535)
        return MAM_ERR_UNSUPPORTED;
    const DevInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MAM_OK) return st;
    int* flag = nullptr;
    MAM_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&flag), g_wait_gave_up));
    EpilogueArgs ep{bias, dense, alpha, beta, blend};
    FwdParams prm{y, nullptr, nullptr, M, K, N, ep, 1.0f, flag, Im2colRows{}, (int)(split_width / FWD_BK)};
    return launch_tiled<SplitCfg>(a, w, prm, *d, (cudaStream_t)stream);
}

int mam_fwd_splits_idx_f32(const float* a, const float* w, const float* bias, const float* dense, int blend,
                           float alpha, float beta, float* y, int32_t* argmax, int32_t* argmin, int64_t M, int64_t K,
                           int64_t N, int64_t split_width, void* stream) {
    if (bad_ptr(a) || bad_ptr(w) || bad_ptr(y) || bad_ptr(argmax) || bad_ptr(argmin) || M <= 0 || K <= 0 || N <= 0 ||
        split_width <= 0)
        return MAM_ERR_INVALID_ARGUMENT;
    if (K >= (1LL << 31) || N >= (1LL << 31) || M >= (1LL << 31)) return MAM_ERR_UNSUPPORTED;
    if (split_width % FWD_BK != 0 || split_width >= K || K % 4 != 0 || !aligned16(a) || !aligned16(w) ||
        K / FWD_BK >= 65535 || split_width / FWD_BK > ResolveCfg::NK_MAX || g_resolve_simple != 0)
        return MAM_ERR_UNSUPPORTED;
    const DevInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MAM_OK) return st;
    cudaStream_t cs = (cudaStream_t)stream;
    int* flag = nullptr;
    MAM_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&flag), g_wait_gave_up));
    EpilogueArgs ep{bias, dense, alpha, beta, blend};
    FwdParams prm{y, argmax, argmin, M, K, N, ep, 1.0f, flag, Im2colRows{}, (int)(split_width / FWD_BK)};
    st = launch_tiled<SplitIdxCfg>(a, w, prm, *d, cs);
    if (st != MAM_OK) return st;
    // every slice is a problem of its own for the resolver: its columns of a and w, its pair of index matrices
    const int64_t slices = (K + split_width - 1) / split_width;
    for (int64_t sl = 0; sl < slices; ++sl) {
        const int64_t k0 = sl * split_width, width = (k0 + split_width <= K) ? split_width : K - k0;
        st = run_resolver(a + k0, w + k0, argmax + sl * M * N, argmin + sl * M * N, M, width, N, K, (int)k0, flag,
                          Im2colRows{}, cs, nullptr);
        if (st != MAM_OK) return st;
    }
    return MAM_OK;
}

int mam_fwd_kn_static_f32(const float* a, const float* b, float* y, int32_t* argmax, int32_t* argmin, int64_t M,
                          int64_t K, int64_t N, void* stream) {
    if (M <= 0 || K <= 0 || N <= 0) return MAM_ERR_INVALID_ARGUMENT;
    const size_t need = mam_fwd_workspace_bytes(M, K, N, MAM_B_KN, argmax != nullptr);
    if (need > MAM_STATIC_SCRATCH_BYTES || (double)K * (double)N * 4.0 > (double)MAM_STATIC_SCRATCH_BYTES)
        return MAM_ERR_STATIC_SCRATCH;
    int dev = 0;
    MAM_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return MAM_ERR_UNSUPPORTED;
    void* scratch = nullptr;
    {
        // In host code `g_static_scratch` is only a handle for the symbol, not a device address:
        // ask the runtime where the array lives on the current device, once (first callers on several
        // host threads take turns).
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (g_static_scratch_addr[dev] == nullptr) {
            void* p = nullptr;
            MAM_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
            g_static_scratch_addr[dev] = p;
        }
        scratch = g_static_scratch_addr[dev];
    }
    return mam_fwd_f32(a, b, MAM_B_KN, nullptr, nullptr, 0, 1.0f, 0.0f, y, argmax, argmin, M, K, N, scratch,
                       MAM_STATIC_SCRATCH_BYTES, stream);
}

int mam_bwd_count_f32(const float* a, const float* b, int b_layout, const float* grad, const int32_t* argmax,
                      const int32_t* argmin, float* da, float* db, int32_t* hit_max, int32_t* hit_min, float scale,
                      int64_t M, int64_t K, int64_t N, void* stream) {
    return mam_bwd_count_ex_f32(a, b, b_layout, grad, argmax, argmin, da, MAM_DA_MK, db, hit_max, hit_min, scale, M, K,
                                N, stream);
}

int mam_bwd_count_ex_f32(const float* a, const float* b, int b_layout, const float* grad, const int32_t* argmax,
                         const int32_t* argmin, float* da, int da_layout, float* db, int32_t* hit_max,
                         int32_t* hit_min, float scale, int64_t M, int64_t K, int64_t N, void* stream) {
    return mam_bwd_count_ws_f32(a, b, b_layout, grad, argmax, argmin, da, da_layout, db, hit_max, hit_min, scale, M, K,
                                N, nullptr, 0, stream);
}

size_t mam_bwd_count_workspace_bytes(int64_t M, int64_t K, int64_t N) {
    // counts ride as sums of 1.0f: exact while no weight can be hit 2^24 times in one call
    if (M <= 0 || K <= 0 || N <= 0 || M >= (1LL << 24)) return 0;
    // Where the 16-byte records pay (B200, 12608 rows unless said otherwise; gradient kernel + hits, separate
    // sweep vs riding along): with the CTA-shared gradient kernel and records that stay in L2, K x N = 3072 x 768:
    // 0.304 -> 0.273 ms.  Not in the row-per-warp band, whose time IS its L2 reductions and where the wider
    // reduction costs more than the second sweep saves (768 x 3072: 0.889 -> 0.960 ms), and not once the records
    // outgrow L2 (4096 rows, 4096 x 4096, 268 MB of records: 0.644 -> 0.725 ms).  The query answers 0 there and
    // callers run the second sweep.
    if (bwd_rowwarp_band(K) || (double)K * (double)N * 16.0 > 64.0 * 1024 * 1024) return 0;
    return round256((size_t)K * (size_t)N * 16);
}

int mam_bwd_count_ws_f32(const float* a, const float* b, int b_layout, const float* grad, const int32_t* argmax,
                         const int32_t* argmin, float* da, int da_layout, float* db, int32_t* hit_max,
                         int32_t* hit_min, float scale, int64_t M, int64_t K, int64_t N, void* workspace,
                         size_t workspace_bytes, void* stream) {
    return mam_bwd_splits_f32(a, b, b_layout, grad, argmax, argmin, 1, da, da_layout, db, hit_max, hit_min, scale, M, K,
                              N, workspace, workspace_bytes, stream);
}

int mam_bwd_splits_f32(const float* a, const float* b, int b_layout, const float* grad, const int32_t* argmax,
                       const int32_t* argmin, int slices, float* da, int da_layout, float* db, int32_t* hit_max,
                       int32_t* hit_min, float scale, int64_t M, int64_t K, int64_t N, void* workspace,
                       size_t workspace_bytes, void* stream) {
    if (slices < 1 || (long long)slices * M >= (1LL << 31)) return MAM_ERR_INVALID_ARGUMENT;
    if (da_layout != MAM_DA_MK && da_layout != MAM_DA_KM) return MAM_ERR_INVALID_ARGUMENT;
    if (bad_ptr(a) || bad_ptr(b) || bad_ptr(grad) || bad_ptr(argmax) || bad_ptr(argmin) || bad_ptr(da) ||
        bad_ptr(db) || M <= 0 || K <= 0 || N <= 0)
        return MAM_ERR_INVALID_ARGUMENT;
    if (b_layout != MAM_B_KN && b_layout != MAM_B_NK) return MAM_ERR_INVALID_ARGUMENT;
    if ((hit_max == nullptr) != (hit_min == nullptr)) return MAM_ERR_INVALID_ARGUMENT;
    const DevInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MAM_OK) return st;
    if (K * 4 > d->max_smem - 1024) return MAM_ERR_UNSUPPORTED;
    cudaStream_t cs = (cudaStream_t)stream;
    int rows = (int)((32 * 1024) / (K * 4));
    if (rows < 1) rows = 1;
    if (rows > 8) rows = 8;
    // transposed da: every k receives `rows` consecutive floats from a CTA, so take more rows per CTA
    // (16 = one 64-byte run) when their accumulators still leave room for several CTAs per SM
    if (da_layout == MAM_DA_KM && 16 * K * 4 <= 48 * 1024) rows = 16;
    const bool count = hit_max != nullptr;
    // the hits travel with the dW terms when the caller brought the scratch for the 16-byte records
    // (a caller that brings the scratch gets the records whatever the query's advice, except beyond 2^24 rows)
    const size_t fused_need = M < (1LL << 24) ? round256((size_t)K * (size_t)N * 16) : 0;
    const bool fused = count && workspace != nullptr && fused_need != 0 && g_bwd_mode != 2 && slices == 1;
    if (fused && (workspace_bytes < fused_need || (reinterpret_cast<uintptr_t>(workspace) & 255u)))
        return MAM_ERR_WORKSPACE;
    float* dw_dst = fused ? static_cast<float*>(workspace) : db;
    const size_t dw_fill = fused ? (size_t)K * (size_t)N * 16 : (size_t)K * (size_t)N * 4;
    auto unpack = [&]() -> int {
        const long long blocks = (K * N + 255) / 256;
        if (blocks > 2147483647LL) return MAM_ERR_UNSUPPORTED;
        TimedLaunch t(MAM_KERNEL_SELCOUNT, cs);
        if (b_layout == MAM_B_NK)
            mam_bwd_unpack_kernel<true><<<(unsigned)blocks, 256, 0, cs>>>(static_cast<const float4*>(workspace), db,
                                                                          hit_max, hit_min, K, N);
        else
            mam_bwd_unpack_kernel<false><<<(unsigned)blocks, 256, 0, cs>>>(static_cast<const float4*>(workspace), db,
                                                                           hit_max, hit_min, K, N);
        MAM_CUDA(cudaGetLastError());
        return MAM_OK;
    };
    // columns owned per CTA in the two-kernel form: at most 8, shared memory permitting, and enough
    // CTAs to cover the SMs twice
    const long long per_col = K * 4 * (count ? 3 : 1);
    int cols = (int)(((long long)d->max_smem - 1024) / per_col);
    if (cols > 8) cols = 8;
    while (cols > 1 && (N + cols - 1) / cols < 2LL * d->sms) cols >>= 1;
    // Measured on B200 the single-kernel form is faster at every benchmarked shape (0.87 vs 1.32 ms at
    // 12608x768x3072): the column-owned sweep is latency-bound.  The two-kernel form stays selectable.
    const bool split = g_bwd_mode == 2 && da_layout == MAM_DA_MK && slices == 1;
    if (split && cols >= 1) {
        if (b_layout == MAM_B_NK)
            return launch_bwd_split<true>(a, b, grad, argmax, argmin, da, db, hit_max, hit_min, scale, M, K, N, rows,
                                          cols, cs);
        return launch_bwd_split<false>(a, b, grad, argmax, argmin, da, db, hit_max, hit_min, scale, M, K, N, rows, cols,
                                       cs);
    }
    // Row-per-warp form: every warp keeps its own row of da (and, where 8 rows of each still leave room for
    // two CTAs per SM, of a) in shared memory and needs no floating-point shared-memory atomics.
    constexpr int RW_ROWS = BWD_THREADS / 32;
    const size_t rw_row = (size_t)K * 4;
    const bool rw_fits = da_layout == MAM_DA_MK && RW_ROWS * rw_row <= (size_t)d->max_smem - 1024;
    // Measured on B200 against the CTA-shared form (NK layout, 12608 rows): K x N = 768 x 3072 0.76 vs 0.88 ms
    // (its 155 M scattered L2 sector operations -- weight gathers + fp32 reductions -- at the 2.0e11/s the probe
    // measures), 1024 x 4096 1.12 vs 1.22; but 512 x 2048 0.62 vs 0.58 (per row the zero / stage / write-out of K
    // floats weighs more), 896 x 3584 1.10 vs 1.03, 1280 x 5120 1.95 vs 1.30, 3072 x 768 0.42 vs 0.23 (a warp's rows
    // leave room for too few warps per SM).  The automatic choice takes this form only in the band where it won.
    const bool rw_auto = bwd_rowwarp_band(K);
    if (rw_fits && (rw_auto || g_bwd_mode == 3 || g_bwd_mode == 4)) {
        const bool a_smem = g_bwd_mode != 4 && 2 * RW_ROWS * rw_row <= ((size_t)d->max_smem - 2048) / 2;
        const size_t smem_rw = RW_ROWS * rw_row * (a_smem ? 2 : 1);
        const long long grid_rw = (M + RW_ROWS - 1) / RW_ROWS;
        if (grid_rw > 2147483647LL) return MAM_ERR_UNSUPPORTED;
        MAM_CUDA(cudaMemsetAsync(dw_dst, 0, dw_fill, cs));
        auto launch = [&](auto kern) -> int {
            MAM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rw));
            TimedLaunch t(MAM_KERNEL_BWD, cs);
            kern<<<(unsigned)grid_rw, BWD_THREADS, smem_rw, cs>>>(a, b, grad, argmax, argmin, da, dw_dst, M, K, N, scale,
                                                                   slices);
            return MAM_OK;
        };
        const bool nk = b_layout == MAM_B_NK;
        if (slices > 1)   // (the sliced form always takes the plain reductions and, for hits, the second sweep)
            st = nk ? (a_smem ? launch(mam_bwd_rowwarp_kernel<true, true, false, true>) : launch(mam_bwd_rowwarp_kernel<true, false, false, true>))
                    : (a_smem ? launch(mam_bwd_rowwarp_kernel<false, true, false, true>) : launch(mam_bwd_rowwarp_kernel<false, false, false, true>));
        else if (fused)
            st = nk ? (a_smem ? launch(mam_bwd_rowwarp_kernel<true, true, true>) : launch(mam_bwd_rowwarp_kernel<true, false, true>))
                    : (a_smem ? launch(mam_bwd_rowwarp_kernel<false, true, true>) : launch(mam_bwd_rowwarp_kernel<false, false, true>));
        else
            st = nk ? (a_smem ? launch(mam_bwd_rowwarp_kernel<true, true>) : launch(mam_bwd_rowwarp_kernel<true, false>))
                    : (a_smem ? launch(mam_bwd_rowwarp_kernel<false, true>) : launch(mam_bwd_rowwarp_kernel<false, false>));
        if (st != MAM_OK) return st;
        MAM_CUDA(cudaGetLastError());
        if (fused) return unpack();
        if (count) return mam_selcount_i32(argmax, argmin, hit_max, hit_min, M * slices, K, N, stream);
        return MAM_OK;
    }
    const size_t smem = (size_t)rows * (size_t)K * 4;
    const long long grid = (M + rows - 1) / rows;
    if (grid > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    MAM_CUDA(cudaMemsetAsync(dw_dst, 0, dw_fill, cs));
    {
        auto launch = [&](auto kern) -> int {
            MAM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            TimedLaunch t(MAM_KERNEL_BWD, cs);
            kern<<<(unsigned)grid, BWD_THREADS, smem, cs>>>(a, b, grad, argmax, argmin, da, dw_dst, M, K, N, rows, scale,
                                                            ConvGeom{}, slices);
            return MAM_OK;
        };
        const bool nk = b_layout == MAM_B_NK, km = da_layout == MAM_DA_KM;
        if (slices > 1)
            st = nk ? (km ? launch(mam_bwd_kernel<true, true, false, false, true>) : launch(mam_bwd_kernel<true, false, false, false, true>))
                    : (km ? launch(mam_bwd_kernel<false, true, false, false, true>) : launch(mam_bwd_kernel<false, false, false, false, true>));
        else if (fused)
            st = nk ? (km ? launch(mam_bwd_kernel<true, true, false, true>) : launch(mam_bwd_kernel<true, false, false, true>))
                    : (km ? launch(mam_bwd_kernel<false, true, false, true>) : launch(mam_bwd_kernel<false, false, false, true>));
        else
            st = nk ? (km ? launch(mam_bwd_kernel<true, true>) : launch(mam_bwd_kernel<true, false>))
                    : (km ? launch(mam_bwd_kernel<false, true>) : launch(mam_bwd_kernel<false, false>));
        if (st != MAM_OK) return st;
    }
    MAM_CUDA(cudaGetLastError());
    if (fused) return unpack();
    if (count) return mam_selcount_i32(argmax, argmin, hit_max, hit_min, M * slices, K, N, stream);
    return MAM_OK;
}

int mam_bwd_f32(const float* a, const float* b, int b_layout, const float* grad, const int32_t* argmax,
                const int32_t* argmin, float* da, float* db, float scale, int64_t M, int64_t K, int64_t N,
                void* stream) {
    return mam_bwd_count_f32(a, b, b_layout, grad, argmax, argmin, da, db, nullptr, nullptr, scale, M, K, N, stream);
}

namespace {
int conv_geom(ConvGeom* g, int64_t B, int64_t C, int64_t H, int64_t W, int kH, int kW, int sh, int sw, int ph, int pw) {
    if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || kH <= 0 || kW <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0)
        return MAM_ERR_INVALID_ARGUMENT;
    if (H + 2LL * ph < kH || W + 2LL * pw < kW) return MAM_ERR_INVALID_ARGUMENT;
    const long long Ho = (H + 2LL * ph - kH) / sh + 1, Wo = (W + 2LL * pw - kW) / sw + 1;
    if (B >= (1LL << 31) || C * (long long)kH * kW >= (1LL << 31) || H >= (1LL << 30) || W >= (1LL << 30))
        return MAM_ERR_UNSUPPORTED;
    *g = ConvGeom{(int)B, (int)C, (int)H, (int)W, kH, kW, sh, sw, ph, pw, (int)Ho, (int)Wo};
    return MAM_OK;
}
// Shared memory of mam_conv_bwd_direct_kernel for `th` output rows per CTA: the region of dx they reach plus
// the per-k table.
size_t conv_direct_smem(const ConvGeom& g, int th) {
    const size_t region = (size_t)g.C * (size_t)((th - 1) * g.sh + g.kH) * (size_t)g.W * 4;
    return ((region + 15) & ~size_t(15)) + (size_t)g.C * g.kH * g.kW * sizeof(ConvDirectEntry);
}
// Output rows per CTA: as many as keep the CTA under 84 KB (two CTAs per SM with room to spare, so that one
// CTA's flush overlaps the other's sweep; measured at [128,64,56,56] 3x3 -> 128: 1 to 3 rows 1.54-1.55 ms,
// 4 rows 1.63, 8 rows 1.83), at most 8; a single row may use the whole SM; 0 = the region does not fit.
int conv_direct_rows(const ConvGeom& g) {
    if ((long long)g.C * g.H * g.W >= (1LL << 31) || (long long)g.kW >= 32768 || (long long)g.kH >= 65536) return 0;
    if (g_conv_direct_rows > 0 && conv_direct_smem(g, g_conv_direct_rows) <= 226 * 1024)
        return g_conv_direct_rows < g.Ho ? g_conv_direct_rows : g.Ho;
    int th = 0;
    for (int t = 1; t <= 8 && t <= g.Ho; ++t)
        if (conv_direct_smem(g, t) <= 84 * 1024) th = t;
    if (th == 0 && conv_direct_smem(g, 1) <= 226 * 1024) th = 1;
    return th;
}
}  // namespace

int mam_conv_bwd_f32(const float* x, const float* w, const float* grad, const int32_t* argmax, const int32_t* argmin,
                     float* cols_t, float* dw, float scale, int64_t B, int64_t C, int64_t H, int64_t W, int kH, int kW,
                     int sh, int sw, int ph, int pw, int64_t N, void* stream) {
    if (bad_ptr(x) || bad_ptr(w) || bad_ptr(grad) || bad_ptr(argmax) || bad_ptr(argmin) || bad_ptr(cols_t) ||
        bad_ptr(dw) || N <= 0)
        return MAM_ERR_INVALID_ARGUMENT;
    ConvGeom g;
    int st = conv_geom(&g, B, C, H, W, kH, kW, sh, sw, ph, pw);
    if (st != MAM_OK) return st;
    const long long M = (long long)g.B * g.Ho * g.Wo, K = (long long)g.C * g.kH * g.kW;
    const DevInfo* d = nullptr;
    st = device_info(&d);
    if (st != MAM_OK) return st;
    if (K * 4 > d->max_smem - 1024) return MAM_ERR_UNSUPPORTED;
    cudaStream_t cs = (cudaStream_t)stream;
    int rows = (int)((32 * 1024) / (K * 4));
    if (rows < 1) rows = 1;
    if (rows > 8) rows = 8;
    if (16 * K * 4 <= 48 * 1024) rows = 16;   // transposed row gradients: longer runs per patch element
    const size_t smem = (size_t)rows * (size_t)K * 4;
    const long long grid = (M + rows - 1) / rows;
    if (grid > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    MAM_CUDA(cudaMemsetAsync(dw, 0, (size_t)K * (size_t)N * 4, cs));
    MAM_CUDA(cudaFuncSetAttribute(mam_bwd_kernel<true, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)smem));
    {
        TimedLaunch t(MAM_KERNEL_BWD, cs);
        mam_bwd_kernel<true, true, true><<<(unsigned)grid, BWD_THREADS, smem, cs>>>(x, w, grad, argmax, argmin, cols_t,
                                                                                     dw, M, K, N, rows, scale, g, 1);
    }
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int mam_conv_fwd_applies(int64_t B, int64_t C, int64_t H, int64_t W, int kH, int kW, int sh, int sw, int ph, int pw) {
    ConvGeom g;
    if (conv_geom(&g, B, C, H, W, kH, kW, sh, sw, ph, pw) != MAM_OK) return 0;
    return conv_implicit_applies(g, nullptr) ? 1 : 0;
}

int mam_conv_fwd_f32(const float* x_nhwc, const float* w_taps, const float* bias, const float* dense, int blend,
                     float alpha, float beta, float* y, int32_t* argmax, int32_t* argmin, int64_t B, int64_t C,
                     int64_t H, int64_t W, int kH, int kW, int sh, int sw, int ph, int pw, int64_t N, void* stream) {
    if (bad_ptr(x_nhwc) || bad_ptr(w_taps) || bad_ptr(y) || N <= 0) return MAM_ERR_INVALID_ARGUMENT;
    if ((argmax == nullptr) != (argmin == nullptr)) return MAM_ERR_INVALID_ARGUMENT;
    ConvGeom g;
    int st = conv_geom(&g, B, C, H, W, kH, kW, sh, sw, ph, pw);
    if (st != MAM_OK) return st;
    if (!conv_implicit_applies(g, x_nhwc) || !aligned16(w_taps)) return MAM_ERR_UNSUPPORTED;
    const long long M = (long long)g.B * g.Ho * g.Wo, K = (long long)g.C * g.kH * g.kW;
    if (M >= (1LL << 31) || N >= (1LL << 31)) return MAM_ERR_UNSUPPORTED;
    const DevInfo* d = nullptr;
    st = device_info(&d);
    if (st != MAM_OK) return st;
    const bool want_idx = argmax != nullptr;
    int variant = g_variant[want_idx ? 1 : 0];
    if (variant < 0) variant = auto_variant(want_idx, M, N, *d);
    ConvSrc cv{x_nhwc, g};
    EpilogueArgs ep{bias, dense, alpha, beta, blend};
    return run_tiled(nullptr, w_taps, y, argmax, argmin, M, K, N, ep, variant, *d, (cudaStream_t)stream, &cv);
}

int mam_im2col_f32(const float* x, float* rows, int64_t B, int64_t C, int64_t H, int64_t W, int kH, int kW, int sh,
                   int sw, int ph, int pw, void* stream) {
    if (bad_ptr(x) || bad_ptr(rows)) return MAM_ERR_INVALID_ARGUMENT;
    ConvGeom g;
    int st = conv_geom(&g, B, C, H, W, kH, kW, sh, sw, ph, pw);
    if (st != MAM_OK) return st;
    if ((long long)g.C * g.H * g.W >= (1LL << 31)) return MAM_ERR_UNSUPPORTED;   // per-image offsets are 32-bit
    const long long blocks = (long long)g.B * g.Ho;
    if (blocks > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    mam_im2col_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(x, rows, g);
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int mam_conv_bwd_direct_applies(int64_t B, int64_t C, int64_t H, int64_t W, int kH, int kW, int sh, int sw, int ph,
                                int pw) {
    ConvGeom g;
    if (conv_geom(&g, B, C, H, W, kH, kW, sh, sw, ph, pw) != MAM_OK) return 0;
    return conv_direct_rows(g) > 0 ? 1 : 0;
}

int mam_conv_bwd_direct_f32(const float* x, const float* w, const float* grad, const int32_t* argmax,
                            const int32_t* argmin, float* dx, float* dw, float scale, int64_t B, int64_t C, int64_t H,
                            int64_t W, int kH, int kW, int sh, int sw, int ph, int pw, int64_t N, void* stream) {
    if (bad_ptr(x) || bad_ptr(w) || bad_ptr(grad) || bad_ptr(argmax) || bad_ptr(argmin) || bad_ptr(dx) ||
        bad_ptr(dw) || N <= 0)
        return MAM_ERR_INVALID_ARGUMENT;
    ConvGeom g;
    int st = conv_geom(&g, B, C, H, W, kH, kW, sh, sw, ph, pw);
    if (st != MAM_OK) return st;
    const long long K = (long long)g.C * g.kH * g.kW;
    if (N >= (1LL << 31) / K) return MAM_ERR_UNSUPPORTED;
    const int th = conv_direct_rows(g);
    if (th <= 0) return MAM_ERR_UNSUPPORTED;
    const long long grid = (long long)g.B * ((g.Ho + th - 1) / th);
    if (grid > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    const size_t smem = conv_direct_smem(g, th);
    cudaStream_t cs = (cudaStream_t)stream;
    MAM_CUDA(cudaMemsetAsync(dw, 0, (size_t)K * (size_t)N * 4, cs));
    MAM_CUDA(cudaMemsetAsync(dx, 0, (size_t)g.B * g.C * g.H * g.W * 4, cs));
    MAM_CUDA(cudaFuncSetAttribute(mam_conv_bwd_direct_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    {
        TimedLaunch t(MAM_KERNEL_BWD, cs);
        mam_conv_bwd_direct_kernel<<<(unsigned)grid, CONV_DIRECT_THREADS, smem, cs>>>(
            x, w, grad, argmax, argmin, dx, dw, g, N, th, scale, (g.W % 4 == 0 && aligned16(dx)) ? 1 : 0);
    }
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int mam_col2im_f32(const float* cols_t, float* dx, int64_t B, int64_t C, int64_t H, int64_t W, int kH, int kW, int sh,
                   int sw, int ph, int pw, void* stream) {
    if (bad_ptr(cols_t) || bad_ptr(dx)) return MAM_ERR_INVALID_ARGUMENT;
    ConvGeom g;
    int st = conv_geom(&g, B, C, H, W, kH, kW, sh, sw, ph, pw);
    if (st != MAM_OK) return st;
    const long long M = (long long)g.B * g.Ho * g.Wo;
    // input rows per CTA: whole planes when that still gives a few CTAs per SM, else split the height
    const DevInfo* d = nullptr;
    st = device_info(&d);
    if (st != MAM_OK) return st;
    int hrows = g.H;
    while (hrows > 4 && (long long)g.B * g.C * ((g.H + hrows - 1) / hrows) < 4LL * d->sms) hrows = (hrows + 1) / 2;
    const long long blocks = (long long)g.B * g.C * ((g.H + hrows - 1) / hrows);
    if (blocks > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    if (g.sh == 1 && g.sw == 1)
        mam_col2im_kernel<true><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(cols_t, dx, g, M, hrows);
    else
        mam_col2im_kernel<false><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(cols_t, dx, g, M, hrows);
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int mam_selcount_i32(const int32_t* argmax, const int32_t* argmin, int32_t* hit_max, int32_t* hit_min, int64_t M,
                     int64_t K, int64_t N, void* stream) {
    if (bad_ptr(argmax) || bad_ptr(argmin) || bad_ptr(hit_max) || bad_ptr(hit_min) || M <= 0 || K <= 0 || N <= 0)
        return MAM_ERR_INVALID_ARGUMENT;
    const DevInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MAM_OK) return st;
    const long long budget = (long long)d->max_smem - 1024;
    if (2 * K * 4 > budget) return MAM_ERR_UNSUPPORTED;
    // Columns per CTA: 8 ints = one 32-byte sector of every index row; fewer only when the
    // counters of 8 columns would not leave room for two CTAs per SM (or would not fit at all).
    int cols = 8;
    while (cols > 1 && 2LL * cols * K * 4 > budget / 2) cols >>= 1;
    const size_t smem = 2ull * cols * (size_t)K * 4;
    const long long col_blocks = (N + cols - 1) / cols;
    if (col_blocks > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    // Row slices: enough CTAs for ~3 rounds over the SMs, each slice at least 512 rows.
    long long ctas_per_sm = (long long)(budget / (long long)smem);
    if (ctas_per_sm > 8) ctas_per_sm = 8;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    long long slices = (3LL * d->sms * ctas_per_sm + col_blocks - 1) / col_blocks;
    const long long max_slices = (M + 511) / 512;
    if (slices > max_slices) slices = max_slices;
    if (slices < 1) slices = 1;
    if (slices > 65535) slices = 65535;
    const long long rows_per_slice = (M + slices - 1) / slices;
    slices = (M + rows_per_slice - 1) / rows_per_slice;
    const dim3 grid((unsigned)col_blocks, (unsigned)slices);
    cudaStream_t cs = (cudaStream_t)stream;
    auto launch = [&](auto kern) -> int {
        MAM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TimedLaunch t(MAM_KERNEL_SELCOUNT, cs);
        kern<<<grid, SEL_THREADS, smem, cs>>>(argmax, argmin, hit_max, hit_min, M, K, N, rows_per_slice);
        return MAM_OK;
    };
    switch (cols) {
        case 8: st = launch(mam_selcount_kernel<8>); break;
        case 4: st = launch(mam_selcount_kernel<4>); break;
        case 2: st = launch(mam_selcount_kernel<2>); break;
        default: st = launch(mam_selcount_kernel<1>); break;
    }
    if (st != MAM_OK) return st;
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int mam_dense_tf32(const float* a, const float* w, float* out, float c_acc, float c_out, int64_t M, int64_t K,
                   int64_t N, void* stream) {
    if (bad_ptr(a) || bad_ptr(w) || bad_ptr(out) || M <= 0 || K <= 0 || N <= 0) return MAM_ERR_INVALID_ARGUMENT;
    if (K % 4 != 0 || !aligned16(a) || !aligned16(w)) return MAM_ERR_UNSUPPORTED;
    const DevInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MAM_OK) return st;
    CUtensorMap tmA, tmW;
    st = encode_rows_k(&tmA, a, M, K, DG_BM);
    if (st != MAM_OK) return st;
    st = encode_rows_k(&tmW, w, N, K, DG_BN);
    if (st != MAM_OK) return st;
    CUtensorMap tmW64;   // 64-row boxes of W for the column slices of the last partial wave
    st = encode_rows_k(&tmW64, w, N, K, 64);
    if (st != MAM_OK) return st;
    const long long tiles = ((M + DG_BM - 1) / DG_BM) * ((N + DG_BN - 1) / DG_BN);
    if (tiles > 2147483647LL) return MAM_ERR_UNSUPPORTED;
    int* flag = nullptr;
    MAM_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&flag), g_wait_gave_up));
    MAM_CUDA(cudaFuncSetAttribute(mam_dense_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DG_SMEM_BYTES));
    {
        TimedLaunch t(MAM_KERNEL_DENSE_TF32, (cudaStream_t)stream);
        // persistent, one CTA per SM; the tiles of the last partial wave are cut into 2 or 4 column slices
        // when that many more work items still fit one wave
        const long long rem = tiles % d->sms;
        int split = rem == 0 ? 1 : (rem * 4 <= d->sms ? 4 : (rem * 2 <= d->sms ? 2 : 1));
        if (!g_dense_split) split = 1;
        const long long full = split > 1 ? tiles - rem : tiles;
        const long long items = full + (tiles - full) * split;
        const unsigned grid = (unsigned)(items < d->sms ? items : d->sms);
        mam_dense_tf32_kernel<<<grid, DG_THREADS, DG_SMEM_BYTES, (cudaStream_t)stream>>>(
            tmA, tmW, tmW64, out, M, K, N, c_acc, c_out, flag, full, split);
    }
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int mam_csr_fwd_f32(const float* a, const int64_t* crow, const int64_t* col, const float* val, const float* bias,
                    float* y, int32_t* argmax, int32_t* argmin, int64_t M, int64_t K, int64_t N, void* stream) {
    if (bad_ptr(a) || bad_ptr(crow) || bad_ptr(y) || M <= 0 || K <= 0 || N <= 0) return MAM_ERR_INVALID_ARGUMENT;
    if ((argmax == nullptr) != (argmin == nullptr)) return MAM_ERR_INVALID_ARGUMENT;
    if (K >= (1LL << 31)) return MAM_ERR_UNSUPPORTED;
    const DevInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MAM_OK) return st;
    cudaStream_t cs = (cudaStream_t)stream;
    const long long budget = ((long long)d->max_smem - 1024) / 4;  // floats
    auto fits = [&](int R) { return (long long)R * K + (long long)CSR_WARPS * 3 * R * 32 <= budget; };
    // rows parked per CTA: as many as shared memory holds (each CTA streams the whole CSR once)
    if (fits(8) && M >= 8) return launch_csr<8>(a, crow, col, val, bias, y, argmax, argmin, M, K, N, cs);
    if (fits(4) && M >= 4) return launch_csr<4>(a, crow, col, val, bias, y, argmax, argmin, M, K, N, cs);
    if (fits(2) && M >= 2) return launch_csr<2>(a, crow, col, val, bias, y, argmax, argmin, M, K, N, cs);
    if (fits(1)) return launch_csr<1>(a, crow, col, val, bias, y, argmax, argmin, M, K, N, cs);
    return MAM_ERR_UNSUPPORTED;
}

namespace {
struct CsrWs {
    size_t at_off, counts_off, seg_off, k0_off, list_off, rlist_off, total;
    long long pitch;  // floats per row of the transposed activations
    int nks;
};
CsrWs csr_ws_layout(int64_t M, int64_t K, int64_t N, int64_t nnz) {
    CsrWs w{};
    w.nks = (int)((K + CT_KS - 1) / CT_KS);
    w.pitch = (M + 3) & ~3LL;
    const size_t segs = (size_t)w.nks * (size_t)N;
    // the regrouped weight first (nothing in it depends on M, so it can be kept from call to call while the
    // weight stays the same), the transposed activations last
    size_t off = 0;
    w.counts_off = off; off += round256(segs * 4);
    w.seg_off = off;    off += round256((segs + 1) * 4);
    w.k0_off = off;     off += round256((size_t)N * 4);
    w.list_off = off;   off += round256(((size_t)nnz + segs) * sizeof(CsrEntry));
    w.rlist_off = off;  off += round256(((size_t)nnz + segs) * sizeof(CsrColEntry));
    w.at_off = off;     off += round256((size_t)K * (size_t)w.pitch * 4);
    w.total = off;
    return w;
}
bool csr_tiled_applies(int64_t M, int64_t K, int64_t N, int64_t nnz) {
    const long long nks = (K + CT_KS - 1) / CT_KS;
    return M >= 32 && nks * N < (1LL << 30) && nnz + nks * N < (1LL << 30) && K < (1LL << 31) &&
           (N + CT_BN - 1) / CT_BN < (1LL << 31) && (M + CT_BM - 1) / CT_BM <= 65535;
}
}  // namespace

size_t mam_csr_fwd_entries_bytes(int64_t K, int64_t N, int64_t nnz) {
    if (K <= 0 || N <= 0 || nnz < 0 || !csr_tiled_applies(32, K, N, nnz)) return 0;
    return csr_ws_layout(32, K, N, nnz).at_off;
}

size_t mam_csr_fwd_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t nnz) {
    if (M <= 0 || K <= 0 || N <= 0 || nnz < 0 || !csr_tiled_applies(M, K, N, nnz)) return 0;
    return csr_ws_layout(M, K, N, nnz).total;
}

int mam_csr_fwd_ws_f32(const float* a, const int64_t* crow, const int64_t* col, const float* val, int64_t nnz,
                       const float* bias, float* y, int32_t* argmax, int32_t* argmin, int64_t M, int64_t K,
                       int64_t N, void* workspace, size_t workspace_bytes, void* stream) {
    return mam_csr_fwd_ws_ex_f32(a, crow, col, val, nnz, bias, y, argmax, argmin, M, K, N, workspace, workspace_bytes,
                                 0, stream);
}

int mam_csr_fwd_ws_ex_f32(const float* a, const int64_t* crow, const int64_t* col, const float* val, int64_t nnz,
                          const float* bias, float* y, int32_t* argmax, int32_t* argmin, int64_t M, int64_t K,
                          int64_t N, void* workspace, size_t workspace_bytes, int entries_ready, void* stream) {
    if (bad_ptr(a) || bad_ptr(crow) || bad_ptr(y) || M <= 0 || K <= 0 || N <= 0 || nnz < 0)
        return MAM_ERR_INVALID_ARGUMENT;
    if ((argmax == nullptr) != (argmin == nullptr)) return MAM_ERR_INVALID_ARGUMENT;
    if (!csr_tiled_applies(M, K, N, nnz) || workspace == nullptr)
        return mam_csr_fwd_f32(a, crow, col, val, bias, y, argmax, argmin, M, K, N, stream);
    const CsrWs w = csr_ws_layout(M, K, N, nnz);
    if (workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return MAM_ERR_WORKSPACE;
    const DevInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MAM_OK) return st;
    if (CT_SMEM_BYTES > d->max_smem) return MAM_ERR_UNSUPPORTED;
    cudaStream_t cs = (cudaStream_t)stream;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    float* at = reinterpret_cast<float*>(ws + w.at_off);
    int* counts = reinterpret_cast<int*>(ws + w.counts_off);
    int* seg = reinterpret_cast<int*>(ws + w.seg_off);
    int* k0 = reinterpret_cast<int*>(ws + w.k0_off);
    CsrEntry* list = reinterpret_cast<CsrEntry*>(ws + w.list_off);
    CsrColEntry* rlist = reinterpret_cast<CsrColEntry*>(ws + w.rlist_off);
    const long long segs = (long long)w.nks * N;

    // activations transposed: aT[K][pitch]
    {
        const long long gx = (K + 31) / 32, gy = (M + 31) / 32;
        if (gy > 65535) return MAM_ERR_UNSUPPORTED;
        mam_transpose_pitch_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, cs>>>(a, at, M, K, w.pitch);
    }
    // stored entries regrouped by stage (kept from an earlier call when the caller says so)
    const unsigned seg_blocks = (unsigned)((segs + 255) / 256);
    const long long* crow_ll = reinterpret_cast<const long long*>(crow);
    const long long* col_ll = reinterpret_cast<const long long*>(col);
    if (entries_ready == 2) {
        // same sparsity pattern as the call that left seg / k0 here, new values: one pass over the entries
        csr_tile_fill_kernel<<<seg_blocks, 256, 0, cs>>>(crow_ll, col_ll, val, seg, list, rlist, N, w.nks, 0);
    } else if (!entries_ready) {
        csr_tile_count_kernel<<<seg_blocks, 256, 0, cs>>>(crow_ll, col_ll, counts, k0, N, K, w.nks);
        // counts -> seg (exclusive scan); the first words of the list area hold the per-block sums
        // until the fill kernel overwrites them
        int* block_sums = reinterpret_cast<int*>(list);
        const long long nb = (segs + 1 + CSR_SCAN_BLOCK - 1) / CSR_SCAN_BLOCK;
        csr_scan_block_sums_kernel<<<(unsigned)nb, 1024, 0, cs>>>(counts, block_sums, segs);
        csr_scan_sums_kernel<<<1, 1024, 0, cs>>>(block_sums, nb);
        csr_scan_apply_kernel<<<(unsigned)nb, 1024, 0, cs>>>(counts, block_sums, seg, segs);
        csr_tile_fill_kernel<<<seg_blocks, 256, 0, cs>>>(crow_ll, col_ll, val, seg, list, rlist, N, w.nks, 0);
    }
    MAM_CUDA(cudaGetLastError());

    CUtensorMap tmAT;
    st = encode_2d_plain(&tmAT, at, M, K, w.pitch * 4, CT_BM, CT_KS);
    if (st != MAM_OK) return st;
    int* flag = nullptr;
    MAM_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&flag), g_wait_gave_up));
    CsrTiledParams prm{seg, list, k0, bias, y, argmax, argmin, M, K, N, w.nks, 1.0f, flag};
    const dim3 grid((unsigned)((N + CT_BN - 1) / CT_BN), (unsigned)((M + CT_BM - 1) / CT_BM));
    if (argmax) {
        MAM_CUDA(cudaFuncSetAttribute(mam_csr_tiled_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      CT_SMEM_BYTES));
        mam_csr_tiled_kernel<true><<<grid, CT_THREADS, CT_SMEM_BYTES, cs>>>(tmAT, prm);
    } else {
        MAM_CUDA(cudaFuncSetAttribute(mam_csr_tiled_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      CT_SMEM_BYTES));
        mam_csr_tiled_kernel<false><<<grid, CT_THREADS, CT_SMEM_BYTES, cs>>>(tmAT, prm);
    }
    MAM_CUDA(cudaGetLastError());
    if (!argmax) return MAM_OK;
    // recorded segments -> indices; rows parked per CTA so that three CTAs share an SM
    auto launch_resolve = [&](auto kern, int R) -> int {
        const size_t smem = (size_t)R * (size_t)K * 4;
        MAM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const long long g = (M + R - 1) / R;
        if (g > 2147483647LL) return MAM_ERR_UNSUPPORTED;
        kern<<<(unsigned)g, 512, smem, cs>>>(a, rlist, k0, argmax, argmin, M, K, N);
        return MAM_OK;
    };
    const long long row_bytes = K * 4;
    if (row_bytes > d->max_smem - 1024) return MAM_ERR_UNSUPPORTED;
    if (2 * row_bytes <= 110 * 1024) st = launch_resolve(mam_csr_resolve_kernel<2>, 2);
    else st = launch_resolve(mam_csr_resolve_kernel<1>, 1);
    if (st != MAM_OK) return st;
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

namespace {
struct SpmmWs {
    size_t counts_off, seg_off, k0_off, list_off, total;
    int nks;
};
SpmmWs spmm_ws_layout(int64_t N, int64_t K, int64_t nnz) {
    SpmmWs w{};
    w.nks = (int)((K + CT_KS - 1) / CT_KS);
    const size_t segs = (size_t)w.nks * (size_t)N;
    size_t off = 0;
    w.counts_off = off; off += round256(segs * 4);
    w.seg_off = off;    off += round256((segs + 1) * 4);
    w.k0_off = off;     off += round256((size_t)N * 4);
    w.list_off = off;   off += round256(((size_t)nnz + segs) * sizeof(CsrEntry));
    w.total = off;
    return w;
}
bool spmm_tiled_applies(int64_t N, int64_t K, int64_t Mc, int64_t nnz, const float* b, const float* c) {
    const long long nks = (K + CT_KS - 1) / CT_KS;
    return Mc >= 64 && Mc % 4 == 0 && (b == nullptr || aligned16(b)) && (c == nullptr || aligned16(c)) &&
           nks * N < (1LL << 30) && nnz + nks * N < (1LL << 30) && K < (1LL << 31) &&
           (N + SP_BN - 1) / SP_BN < (1LL << 31) && (Mc + CT_BM - 1) / CT_BM <= 65535;
}
}  // namespace

size_t mam_spmm_csr_workspace_bytes(int64_t N, int64_t K, int64_t Mc, int64_t nnz) {
    if (N <= 0 || K <= 0 || Mc <= 0 || nnz < 0 || !spmm_tiled_applies(N, K, Mc, nnz, nullptr, nullptr)) return 0;
    // The tiled kernel pays only with enough entries per (row, stage) segment and enough work to cover the
    // regrouping launches: below ~3 % density or ~1e9 multiply-adds the thread-per-output kernel wins
    // (measured: 4096^2 x 4096 at 90 % sparsity 1.29 vs 3.2 ms, at 99 % 0.59 vs 0.39 ms).  Answering 0 here
    // steers callers to it; a caller that passes a workspace anyway gets the tiled kernel.
    const long long nks = (K + CT_KS - 1) / CT_KS;
    if (nnz < 2 * N * nks || (double)nnz * (double)Mc < 1e9) return 0;
    return spmm_ws_layout(N, K, nnz).total;
}

int mam_spmm_csr_ws_f32(const int64_t* crow, const int64_t* col, const float* val, int64_t nnz, const float* b,
                        float* c, int64_t N, int64_t K, int64_t Mc, void* workspace, size_t workspace_bytes,
                        void* stream) {
    if (bad_ptr(crow) || bad_ptr(b) || bad_ptr(c) || N <= 0 || K <= 0 || Mc <= 0 || nnz < 0)
        return MAM_ERR_INVALID_ARGUMENT;
    if (workspace == nullptr || !spmm_tiled_applies(N, K, Mc, nnz, b, c))
        return mam_spmm_csr_f32(crow, col, val, b, c, N, K, Mc, stream);
    const SpmmWs w = spmm_ws_layout(N, K, nnz);
    if (workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return MAM_ERR_WORKSPACE;
    const DevInfo* d = nullptr;
    int st = device_info(&d);
    if (st != MAM_OK) return st;
    if (SP_SMEM_BYTES > d->max_smem) return MAM_ERR_UNSUPPORTED;
    cudaStream_t cs = (cudaStream_t)stream;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    int* counts = reinterpret_cast<int*>(ws + w.counts_off);
    int* seg = reinterpret_cast<int*>(ws + w.seg_off);
    int* k0 = reinterpret_cast<int*>(ws + w.k0_off);
    CsrEntry* list = reinterpret_cast<CsrEntry*>(ws + w.list_off);
    const long long segs = (long long)w.nks * N;
    const unsigned seg_blocks = (unsigned)((segs + 255) / 256);
    const long long* crow_ll = reinterpret_cast<const long long*>(crow);
    const long long* col_ll = reinterpret_cast<const long long*>(col);
    csr_tile_count_kernel<<<seg_blocks, 256, 0, cs>>>(crow_ll, col_ll, counts, k0, N, K, w.nks);
    {
        int* block_sums = reinterpret_cast<int*>(list);
        const long long nb = (segs + 1 + CSR_SCAN_BLOCK - 1) / CSR_SCAN_BLOCK;
        csr_scan_block_sums_kernel<<<(unsigned)nb, 1024, 0, cs>>>(counts, block_sums, segs);
        csr_scan_sums_kernel<<<1, 1024, 0, cs>>>(block_sums, nb);
        csr_scan_apply_kernel<<<(unsigned)nb, 1024, 0, cs>>>(counts, block_sums, seg, segs);
    }
    csr_tile_fill_kernel<<<seg_blocks, 256, 0, cs>>>(crow_ll, col_ll, val, seg, list, nullptr, N, w.nks, 1);
    MAM_CUDA(cudaGetLastError());
    CUtensorMap tmB;
    st = encode_2d_plain(&tmB, b, Mc, K, Mc * 4, CT_BM, CT_KS);
    if (st != MAM_OK) return st;
    int* flag = nullptr;
    MAM_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&flag), g_wait_gave_up));
    SpmmTiledParams prm{seg, list, c, N, K, Mc, w.nks, flag};
    const dim3 grid((unsigned)((N + SP_BN - 1) / SP_BN), (unsigned)((Mc + CT_BM - 1) / CT_BM));
    MAM_CUDA(cudaFuncSetAttribute(mam_spmm_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SP_SMEM_BYTES));
    mam_spmm_tiled_kernel<<<grid, CT_THREADS, SP_SMEM_BYTES, cs>>>(tmB, prm);
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int mam_spmm_csr_f32(const int64_t* crow, const int64_t* col, const float* val, const float* b, float* c, int64_t N,
                     int64_t K, int64_t Mc, void* stream) {
    if (bad_ptr(crow) || bad_ptr(b) || bad_ptr(c) || N <= 0 || K <= 0 || Mc <= 0) return MAM_ERR_INVALID_ARGUMENT;
    // four columns per thread where rows of b and c can be read and written 16 bytes at a time
    const bool v4 = Mc % 4 == 0 && aligned16(b) && aligned16(c);
    const long long per_cta = v4 ? 512 : 128;
    for (int64_t n0 = 0; n0 < N; n0 += 65535) {   // grid.y limit: row blocks
        const int64_t nn = N - n0 < 65535 ? N - n0 : 65535;
        dim3 grid((unsigned)((Mc + per_cta - 1) / per_cta), (unsigned)nn);
        if (v4)
            mam_spmm_csr_v4_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(
                reinterpret_cast<const long long*>(crow) + n0, reinterpret_cast<const long long*>(col), val, b,
                c + n0 * Mc, nn, Mc);
        else
            mam_spmm_csr_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(
                reinterpret_cast<const long long*>(crow) + n0, reinterpret_cast<const long long*>(col), val, b,
                c + n0 * Mc, nn, Mc);
    }
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

int mam_selcount_indicator_i32(const int32_t* hit_max, const int32_t* hit_min, int32_t* count, int64_t n_elems,
                               void* stream) {
    if (bad_ptr(hit_max) || bad_ptr(hit_min) || bad_ptr(count) || n_elems <= 0) return MAM_ERR_INVALID_ARGUMENT;
    const long long blocks = (n_elems + 255) / 256;
    mam_selcount_indicator_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(hit_max, hit_min, count,
                                                                                      n_elems);
    MAM_CUDA(cudaGetLastError());
    return MAM_OK;
}

}  // extern "C"
