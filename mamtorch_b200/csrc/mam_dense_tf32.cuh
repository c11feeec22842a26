// Dense term of the beta-blended MAM layer on the 5th-generation tensor cores:
//     out[M,N] = c_out * out + c_acc * (a[M,K] . W[N,K]^T),   TF32 inputs, fp32 accumulation.
//
// Replaces the cuBLAS calls behind `at::linalg_matmul` in the reference's host code
// (mamtorch/kernel/v3/csrc/cuda/fullyconnected.cu:153-160, .../fullyconnected_backward.cu:138-145) and its
// SIMT `dense_cuda_kernel` (mamtorch/kernel/v2/csrc/cuda/dense.cu:33-144).  The max/min semiring of
// the MAM term cannot use tensor cores; this sum-of-products term can.
//
// Persistent kernel, one CTA of 192 threads per SM walking 128x256 output tiles, three roles:
//   warp 0, one lane : TMA producer -- [128][32 floats] of a and [256][32 floats] of W per stage (both
//                      K-contiguous, 128-byte swizzle) into a 4-deep full/empty mbarrier ring that
//                      runs straight across tile boundaries;
//   warp 1, one lane : issues tcgen05.mma.cta_group::1.kind::tf32 (M=128, N=256, K=8; four per stage,
//                      stepping the shared-memory descriptors 32 bytes along K).  The accumulator
//                      alternates between the two 256-column halves of tensor memory, so the MMAs of
//                      tile i+1 run while the epilogue drains tile i; tcgen05.commit hands each stage
//                      back to the producer and each finished accumulator to the epilogue;
//   warps 2..5       : epilogue -- tcgen05.ld (32 lanes x 32 columns per instruction), a turn through a
//                      padded shared-memory block so that global accesses are whole 128-byte row
//                      segments, scale/blend, store, then release of the accumulator half.
// 128x256 rather than 128x128 because the product is fed from L2: a 128x128 tile needs 32 KB of
// operands per 1.05 MFLOP, a 128x256 tile 48 KB per 2.1 MFLOP.
// Rows and columns beyond M, N and the k tail are zero-filled by TMA (zeros are neutral for a sum)
// and masked at the store.  Every mbarrier wait is bounded; on expiry the kernel raises the
// device flag, still frees its tensor memory and returns.
#pragma once
#include <cuda.h>
#include "mam_ptx.cuh"

namespace mamb200 {

constexpr int DG_BM = 128, DG_BN = 256, DG_BK = 32, DG_STAGES = 4;
constexpr int DG_THREADS = 192;
constexpr int DG_A_BYTES = DG_BM * DG_BK * 4, DG_B_BYTES = DG_BN * DG_BK * 4;
constexpr int DG_STAGE_BYTES = DG_A_BYTES + DG_B_BYTES;
constexpr int DG_EPI_BYTES = 4 * 32 * 33 * 4;  // one padded 32x32 fp32 block per epilogue warp
constexpr int DG_SMEM_BYTES = 1024 + DG_STAGES * DG_STAGE_BYTES + (2 * DG_STAGES + 4) * 8 + 16 + DG_EPI_BYTES;
constexpr int DG_TMEM_COLS = 2 * DG_BN;  // two accumulators of 256 fp32 columns: all of tensor memory

// Instruction descriptor of tcgen05.mma kind::tf32: fp32 accumulator (bits 4-5 = 1), TF32 A and B
// (bits 7-9 and 10-12 = 2), both operands K-major (bits 15, 16 = 0), N>>3 at bit 17, M>>4 at bit 24.
__host__ __device__ constexpr uint32_t dg_idesc(int n = DG_BN) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(DG_BM >> 4) << 24);
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

// Tile order: bands of DG_BAND tile-rows, walked row-fastest inside a band, so that the CTAs running
// at the same time share a few row-tiles of a and a run of adjacent column-tiles of W in L2.
constexpr int DG_BAND = 8;
__device__ __forceinline__ void dg_tile_coords(long long tile, int ntm, int ntn, int& tm, int& tn) {
    const long long per_band = (long long)DG_BAND * ntn;
    const int band = (int)(tile / per_band);
    const int r = (int)(tile - (long long)band * per_band);
    const int rows = min(DG_BAND, ntm - band * DG_BAND);
    tm = band * DG_BAND + r % rows;
    tn = r / rows;
}

// Work items.  The first `full` tiles (a whole number of waves of the grid) are whole 128x256 tiles; the tiles
// of the last, partial wave are cut into `split` column slices of 256/split columns each, one item per
// slice, so that the tail keeps (nearly) every SM busy for 1/split of a tile time instead of a few SMs
// for a whole one.  A slice loads the same operand boxes as its tile and multiplies against the rows
// [ncol0, ncol0 + ncols) of the W box (N = ncols in the instruction descriptor).
struct DgItem {
    int tm, tn, ncol0, ncols;
};
__device__ __forceinline__ DgItem dg_item(long long g, long long full, int split, int ntm, int ntn) {
    DgItem it;
    long long tile = g;
    it.ncol0 = 0;
    it.ncols = DG_BN;
    if (g >= full) {
        const long long s = g - full;
        tile = full + s / split;
        it.ncols = DG_BN / split;
        it.ncol0 = (int)(s % split) * it.ncols;
    }
    dg_tile_coords(tile, ntm, ntn, it.tm, it.tn);
    return it;
}

__global__ void __launch_bounds__(DG_THREADS, 1)
mam_dense_tf32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                      const __grid_constant__ CUtensorMap tmW64, float* __restrict__ out, long long M, long long K, long long N, float c_acc, float c_out,
                      int* error, long long full, int split) {
    extern __shared__ unsigned char dg_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(dg_smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + DG_STAGES * DG_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + DG_STAGES;
    uint64_t* acc_full = empty_bar + DG_STAGES;  // [2] accumulator half holds a finished tile
    uint64_t* acc_empty = acc_full + 2;          // [2] accumulator half has been drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntn = (int)((N + DG_BN - 1) / DG_BN);
    const int ntm = (int)((M + DG_BM - 1) / DG_BM);
    const long long ntiles = (long long)ntm * ntn;
    const long long nitems = full + (ntiles - full) * split;
    const int nk = (int)((K + DG_BK - 1) / DG_BK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < DG_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
        }
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
            bool ok = true;
            for (long long g = blockIdx.x; g < nitems && ok; g += gridDim.x) {
                const DgItem item = dg_item(g, full, split, ntm, ntn);
                const int tm = item.tm, tn = item.tn;
                for (int kc = 0; kc < nk; ++kc) {
                    if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u)) {
                        atomicExch(error, 1);
                        ok = false;
                        break;
                    }
                    unsigned char* sa = smem + stage * DG_STAGE_BYTES;
                    if (item.ncols == DG_BN) {
                        mbar_expect_tx(&full_bar[stage], DG_STAGE_BYTES);
                        tma_load_2d(sa, &tmA, &full_bar[stage], kc * DG_BK, tm * DG_BM);
                        tma_load_2d(sa + DG_A_BYTES, &tmW, &full_bar[stage], kc * DG_BK, tn * DG_BN);
                    } else {
                        // a column slice: only its rows of W, in 64-row boxes, at their place in the stage
                        mbar_expect_tx(&full_bar[stage], DG_A_BYTES + item.ncols * DG_BK * 4);
                        tma_load_2d(sa, &tmA, &full_bar[stage], kc * DG_BK, tm * DG_BM);
                        for (int r = item.ncol0; r < item.ncol0 + item.ncols; r += 64)
                            tma_load_2d(sa + DG_A_BYTES + r * (DG_BK * 4), &tmW64, &full_bar[stage], kc * DG_BK,
                                        tn * DG_BN + r);
                    }
                    if (++stage == DG_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long it = 0;  // tiles done by this CTA
            for (long long g = blockIdx.x; g < nitems && ok; g += gridDim.x, ++it) {
                const DgItem item = dg_item(g, full, split, ntm, ntn);
                const uint32_t idesc = dg_idesc(item.ncols);
                const uint32_t b_rows_off = (uint32_t)item.ncol0 * 128u;   // W rows are 128-byte rows of the box
                const int buf = (int)(it & 1);
                // the half must have been drained by the epilogue of the tile two steps back
                if (!mbar_wait_bounded(&acc_empty[buf], (uint32_t)((it >> 1) & 1) ^ 1u)) {
                    atomicExch(error, 1);
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * DG_BN);
                for (int kc = 0; kc < nk; ++kc) {
                    if (!mbar_wait_bounded(&full_bar[stage], phase)) {
                        atomicExch(error, 1);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + stage * DG_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + DG_A_BYTES + b_rows_off;
#pragma unroll
                    for (int k = 0; k < DG_BK / 8; ++k) {
                        // 8 tf32 = 32 bytes along K inside the 128-byte swizzle span: +2 in the address field
                        const uint64_t adesc = dg_smem_desc(a_addr + k * 32);
                        const uint64_t bdesc = dg_smem_desc(b_addr + k * 32);
                        tc_mma_tf32(tmem_d, adesc, bdesc, idesc, (kc | k) ? 1u : 0u);
                    }
                    tc_commit(&empty_bar[stage]);  // stage is free once these MMAs have read it
                    if (++stage == DG_STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) tc_commit(&acc_full[buf]);  // arrives when every MMA of this tile has completed
            }
        }
    } else {
        // epilogue warps 2..5: TMEM lane quarter = warp % 4
        const int quarter = warp & 3;
        float* stage_s = reinterpret_cast<float*>(tmem_slot + 4) + (warp - 2) * (32 * 33);
        long long it = 0;
        for (long long g = blockIdx.x; g < nitems; g += gridDim.x, ++it) {
            const DgItem item = dg_item(g, full, split, ntm, ntn);
            const int tm = item.tm, tn = item.tn;
            const int buf = (int)(it & 1);
            if (!mbar_wait_bounded(&acc_full[buf], (uint32_t)((it >> 1) & 1))) {
                atomicExch(error, 1);
                break;
            }
            tc_fence_after();
#pragma unroll 1
            for (int cg = 0; cg < item.ncols / 32; ++cg) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * DG_BN + cg * 32);
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
                // thread = row here; turn the 32x32 block through shared memory so that every global
                // access of the warp is one 128-byte row segment
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 32; ++i) stage_s[lane * 33 + i] = __uint_as_float(r[i]) * c_acc;
                __syncwarp();
                const long long n = (long long)tn * DG_BN + item.ncol0 + cg * 32 + lane;
                const long long mrow0 = (long long)tm * DG_BM + quarter * 32;
                if (n < N) {
#pragma unroll 8
                    for (int rr = 0; rr < 32; ++rr) {
                        if (mrow0 + rr < M) {
                            float* o = out + (mrow0 + rr) * N + n;
                            float v = stage_s[rr * 33 + lane];
                            if (c_out != 0.f) v = fmaf(c_out, *o, v);
                            *o = v;
                        }
                    }
                }
            }
            // every tcgen05.ld of this half has completed (wait::ld above): hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
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
