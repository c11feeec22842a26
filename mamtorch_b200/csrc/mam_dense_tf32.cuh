// Dense term of the beta-blended MAM layer on the 5th-generation tensor cores:
//     out[M,N] = c_out * out + c_acc * (a[M,K] . W[N,K]^T),   TF32 inputs, fp32 accumulation.
//
// Replaces the cuBLAS calls behind `at::linalg_matmul` in the reference's host code
// (mamtorch/kernel/v3/csrc/cuda/fullyconnected.cu:153-160, .../fullyconnected_backward.cu:138-145) and its
// SIMT `dense_cuda_kernel` (mamtorch/kernel/v2/csrc/cuda/dense.cu:33-144).  The max/min semiring of
// the MAM term cannot use tensor cores; this sum-of-products term can.
//
// One 128x128 output tile per CTA, 192 threads in three roles:
//   warp 0, one lane : TMA producer -- [128 rows][32 floats] boxes of a and W (both K-contiguous, 128-byte
//                      swizzle) into a STAGES-deep full/empty mbarrier ring;
//   warp 1, one lane : issues tcgen05.mma.cta_group::1.kind::tf32 (M=128, N=128, K=8; four per stage,
//                      stepping the shared-memory descriptors 32 bytes along K), accumulating in
//                      128 columns of tensor memory that warp 1 allocates and frees; tcgen05.commit
//                      hands each stage back to the producer and finally signals the epilogue;
//   warps 2..5       : epilogue -- tcgen05.ld (32 lanes x 32 columns per instruction), scale/blend, store.
// Rows and columns beyond M, N and the k tail are zero-filled by TMA (zeros are neutral for a sum)
// and masked at the store.  Every mbarrier wait is bounded; on expiry the kernel raises the
// device flag, still frees its tensor memory and returns.
#pragma once
#include <cuda.h>
#include "mam_ptx.cuh"

namespace mamb200 {

constexpr int DG_BM = 128, DG_BN = 128, DG_BK = 32, DG_STAGES = 6;
constexpr int DG_THREADS = 192;
constexpr int DG_A_BYTES = DG_BM * DG_BK * 4, DG_B_BYTES = DG_BN * DG_BK * 4;
constexpr int DG_STAGE_BYTES = DG_A_BYTES + DG_B_BYTES;
constexpr int DG_SMEM_BYTES = 1024 + DG_STAGES * DG_STAGE_BYTES + (2 * DG_STAGES + 1) * 8 + 16;
constexpr int DG_TMEM_COLS = 128;

// Instruction descriptor of tcgen05.mma kind::tf32: fp32 accumulator (bits 4-5 = 1), TF32 A and B
// (bits 7-9 and 10-12 = 2), both operands K-major (bits 15, 16 = 0), N>>3 at bit 17, M>>4 at bit 24.
__host__ __device__ constexpr uint32_t dg_idesc() {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(DG_BN >> 3) << 17) | ((uint32_t)(DG_BM >> 4) << 24);
}

// Shared-memory matrix descriptor for a K-major operand stored as rows of 128 bytes in the 128-byte
// swizzle: start address >> 4 in bits 0-13, leading byte offset (unused for this layout) = 1 in
// bits 16-29, stride between 8-row groups = 1024 bytes >> 4 in bits 32-45, descriptor version 1 in
// bits 46-47, swizzle mode 2 (128 bytes) in bits 61-63.
__device__ __forceinline__ uint64_t dg_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__global__ void __launch_bounds__(DG_THREADS, 1)
mam_dense_tf32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                      float* __restrict__ out, long long M, long long K, long long N, float c_acc, float c_out,
                      int* error) {
    extern __shared__ unsigned char dg_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(dg_smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + DG_STAGES * DG_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + DG_STAGES;
    uint64_t* accum_bar = empty_bar + DG_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntn = (int)((N + DG_BN - 1) / DG_BN);
    const int tm = blockIdx.x / ntn, tn = blockIdx.x % ntn;
    const int nk = (int)((K + DG_BK - 1) / DG_BK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < DG_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(accum_bar, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(DG_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmW);
            int stage = 0;
            uint32_t phase = 0;
            for (int kc = 0; kc < nk; ++kc) {
                if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u)) {
                    atomicExch(error, 1);
                    break;
                }
                mbar_expect_tx(&full_bar[stage], DG_STAGE_BYTES);
                unsigned char* sa = smem + stage * DG_STAGE_BYTES;
                tma_load_2d(sa, &tmA, &full_bar[stage], kc * DG_BK, tm * DG_BM);
                tma_load_2d(sa + DG_A_BYTES, &tmW, &full_bar[stage], kc * DG_BK, tn * DG_BN);
                if (++stage == DG_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kc = 0; kc < nk && ok; ++kc) {
                if (!mbar_wait_bounded(&full_bar[stage], phase)) {
                    atomicExch(error, 1);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + stage * DG_STAGE_BYTES);
                const uint32_t b_addr = a_addr + DG_A_BYTES;
#pragma unroll
                for (int k = 0; k < DG_BK / 8; ++k) {
                    // 8 tf32 = 32 bytes along K inside the 128-byte swizzle span: +2 in the address field
                    const uint64_t adesc = dg_smem_desc(a_addr + k * 32);
                    const uint64_t bdesc = dg_smem_desc(b_addr + k * 32);
                    tc_mma_tf32(tmem_base, adesc, bdesc, dg_idesc(), (kc | k) ? 1u : 0u);
                }
                tc_commit(&empty_bar[stage]);  // stage is free once these MMAs have read it
                if (++stage == DG_STAGES) { stage = 0; phase ^= 1u; }
            }
            tc_commit(accum_bar);  // arrives when every MMA issued so far has completed
        }
    } else {
        // epilogue warps 2..5: TMEM lane quarter = warp % 4
        const int quarter = warp & 3;
        const bool ready = mbar_wait_bounded(accum_bar, 0);
        if (!ready) atomicExch(error, 1);
        tc_fence_after();
        const long long m = (long long)tm * DG_BM + quarter * 32 + lane;
        if (ready) {
#pragma unroll 1
            for (int cg = 0; cg < DG_BN / 32; ++cg) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cg * 32);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                      "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
                      "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
                      "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (m < M) {
                    const long long n0 = (long long)tn * DG_BN + cg * 32;
                    float* o = out + m * N + n0;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (n0 + i < N) {
                            float v = __uint_as_float(r[i]) * c_acc;
                            if (c_out != 0.f) v = fmaf(c_out, o[i], v);
                            o[i] = v;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(DG_TMEM_COLS)
                     : "memory");
    }
}

}  // namespace mamb200
