// Issue-rate probe for the instruction mixes a Multiply-And-Max/min inner loop can be built
// from on sm_100a.  It answers, by measurement, how many (mul, max, min) units per clock per SM
// each formulation can sustain when every operand already sits in shared memory -- the ceiling
// the real forward kernels are judged against.  Nothing here touches global memory inside the
// timed loop except one final store that keeps the work alive.
//
// Build:  nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o pipe_probe pipe_probe.cu
// Run:    ./pipe_probe            (prints one JSON object per line)
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "mam_ptx.cuh"

using namespace mamb200;

#define CK(x)                                                                        \
    do {                                                                             \
        cudaError_t e_ = (x);                                                        \
        if (e_ != cudaSuccess) {                                                     \
            fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, \
                    __LINE__);                                                       \
            exit(1);                                                                 \
        }                                                                            \
    } while (0)

constexpr int THREADS = 256;
constexpr int KSM = 256;  // k extent resident in shared memory (floats per row)

// Shared layout: A rows [32][KSM], W rows [64][KSM]; each thread owns TM rows of A and TN rows of W.
// Row addresses are spread like the real kernel (4 row-lanes x 8 col-lanes per warp).

// Operand layout inside shared memory mirrors the real kernels' TMA stages: k is cut into chunks
// of 32 floats; a chunk holds [rows][32] with the 16-byte groups of each 128-byte row XOR-swizzled
// by (row & 7) (the 128-byte TMA swizzle), which makes every LDS.128 below bank-conflict free.
__device__ __forceinline__ const ulonglong2* opnd(const float* base, int rows, int row, int k) {
    const int kc = k >> 5, q = (k >> 2) & 7;
    return reinterpret_cast<const ulonglong2*>(base + kc * rows * 32 + row * 32 + ((q ^ (row & 7)) << 2));
}

enum Mode {
    PURE_FMUL = 0,
    PURE_FFMA,
    PURE_FMUL2,
    PURE_FMNMX,
    PURE_FMNMX3,
    PURE_SETP_SEL,
    MIX_SCALAR,       // FMUL + FMNMX + FMNMX per unit
    MIX_MAX3,         // 2 FMUL + max3 + min3 per 2 units
    MIX_MUL2_MAX3,    // FMUL2 + max3 + min3 per 2 units
    MIX_NAIVE_INDEX,  // per-k compare/select index tracking (what a direct port would do)
    MIX_BLOCKTRACK,   // MIX_MUL2_MAX3 on block-local extremes + merge every 32 k (4x8 tile)
    N_MODES
};

static const char* mode_name[N_MODES] = {
    "pure_fmul", "pure_ffma", "pure_fmul2", "pure_fmnmx", "pure_fmnmx3", "pure_setp_sel",
    "mix_fmul_fmnmx_fmnmx", "mix_fmul_max3_min3", "mix_fmul2_max3_min3", "mix_naive_index",
    "mix_blocktrack_4x8_merge32"};

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
probe_kernel(float* out, int iters, long long* clk_out) {
    extern __shared__ __align__(16) float smem[];
    float* As = smem;               // [32][KSM]
    float* Ws = smem + 32 * KSM;    // [64][KSM]
    for (int i = threadIdx.x; i < 96 * KSM; i += THREADS)
        smem[i] = __int_as_float(0x3f000000 + ((i * 2654435761u) >> 12));  // values in [0.5, 1)
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lane_m = lane >> 3, lane_n = lane & 7;
    long long t0 = clock64();

    if constexpr (MODE <= PURE_SETP_SEL) {
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = As[(threadIdx.x + i * 7) % (32 * KSM)];
        float c = Ws[threadIdx.x];
        int sel[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) sel[i] = i;
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int r = 0; r < 16; ++r) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if constexpr (MODE == PURE_FMUL) {
                        asm volatile("mul.rn.f32 %0, %0, %1;" : "+f"(acc[i]) : "f"(c));
                    } else if constexpr (MODE == PURE_FFMA) {
                        asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(acc[i]) : "f"(c));
                    } else if constexpr (MODE == PURE_FMUL2) {
                        if (i % 2 == 0) {
                            f32x2_t v = pack2(acc[i], acc[i + 1]);
                            f32x2_t cc = pack2(c, c);
                            asm volatile("mul.rn.f32x2 %0, %0, %1;" : "+l"(v) : "l"(cc));
                            unpack2(v, acc[i], acc[i + 1]);
                        }
                    } else if constexpr (MODE == PURE_FMNMX) {
                        asm volatile("max.f32 %0, %0, %1;" : "+f"(acc[i]) : "f"(acc[(i + 1) & 15]));
                    } else if constexpr (MODE == PURE_FMNMX3) {
                        asm volatile("max.f32 %0, %0, %1, %2;"
                                     : "+f"(acc[i])
                                     : "f"(acc[(i + 1) & 15]), "f"(acc[(i + 2) & 15]));
                    } else {  // setp + selp pair
                        asm volatile(
                            "{\n\t.reg .pred p;\n\t"
                            "setp.gt.f32 p, %2, %0;\n\t"
                            "selp.f32 %0, %2, %0, p;\n\t"
                            "selp.s32 %1, %3, %1, p;\n\t}"
                            : "+f"(acc[i]), "+r"(sel[i])
                            : "f"(acc[(i + 1) & 15]), "r"(it));
                    }
                }
            }
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) s += acc[i] + (float)sel[i];
        out[blockIdx.x * THREADS + threadIdx.x] = s;
    } else if constexpr (MODE == MIX_BLOCKTRACK) {
        constexpr int TM = 4, TN = 8;
        float vmax[TM][TN], vmin[TM][TN];
        unsigned bmax[TM][TN / 2], bmin[TM][TN / 2];  // two 16-bit block ids per register
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                vmax[i][j] = -INFINITY;
                vmin[i][j] = INFINITY;
                if (j < TN / 2) bmax[i][j] = bmin[i][j] = 0;
            }
        int arow[TM], wrow[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) arow[i] = (warp & 1) * 16 + i * 4 + lane_m;
#pragma unroll
        for (int j = 0; j < TN; ++j) wrow[j] = j * 8 + lane_n;
        for (int it = 0; it < iters; ++it) {
            for (int kb = 0; kb < KSM / 32; ++kb) {
                float lmax[TM][TN], lmin[TM][TN];
#pragma unroll
                for (int ks = 0; ks < 32; ks += 4) {
                    const int k = kb * 32 + ks;
                    ulonglong2 av[TM];
#pragma unroll
                    for (int i = 0; i < TM; ++i) av[i] = *opnd(As, 32, arow[i], k);
#pragma unroll
                    for (int j = 0; j < TN; ++j) {
                        ulonglong2 wv = *opnd(Ws, 64, wrow[j], k);
#pragma unroll
                        for (int i = 0; i < TM; ++i) {
                            float p0, p1, p2, p3;
                            unpack2(mul2(av[i].x, wv.x), p0, p1);
                            unpack2(mul2(av[i].y, wv.y), p2, p3);
                            if (ks == 0) {
                                lmax[i][j] = fmaxf(p0, p1);
                                lmin[i][j] = fminf(p0, p1);
                            } else {
                                lmax[i][j] = fmax3(lmax[i][j], p0, p1);
                                lmin[i][j] = fmin3(lmin[i][j], p0, p1);
                            }
                            lmax[i][j] = fmax3(lmax[i][j], p2, p3);
                            lmin[i][j] = fmin3(lmin[i][j], p2, p3);
                        }
                    }
                }
                const unsigned kid = (unsigned)(it * (KSM / 32) + kb) & 0xffffu;
                const unsigned kid2 = kid | (kid << 16);
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) {
                        const bool gt = lmax[i][j] > vmax[i][j];
                        const bool lt = lmin[i][j] < vmin[i][j];
                        vmax[i][j] = fmaxf(vmax[i][j], lmax[i][j]);
                        vmin[i][j] = fminf(vmin[i][j], lmin[i][j]);
                        const unsigned selhalf = (j & 1) ? 0x7610u : 0x3254u;  // replace hi / lo half
                        if (gt) bmax[i][j / 2] = __byte_perm(bmax[i][j / 2], kid2, selhalf);
                        if (lt) bmin[i][j / 2] = __byte_perm(bmin[i][j / 2], kid2, selhalf);
                    }
            }
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j)
                s += vmax[i][j] + vmin[i][j] + (float)(bmax[i][j / 2] ^ bmin[i][j / 2]);
        out[blockIdx.x * THREADS + threadIdx.x] = s;
    } else {
        constexpr int TM = 8, TN = 8;
        float vmax[TM][TN], vmin[TM][TN];
        int imax[MODE == MIX_NAIVE_INDEX ? TM : 1][MODE == MIX_NAIVE_INDEX ? TN : 1];
        int imin[MODE == MIX_NAIVE_INDEX ? TM : 1][MODE == MIX_NAIVE_INDEX ? TN : 1];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                vmax[i][j] = -INFINITY;
                vmin[i][j] = INFINITY;
                if constexpr (MODE == MIX_NAIVE_INDEX) imax[i][j] = imin[i][j] = 0;
            }
        int arow[TM], wrow[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) arow[i] = i * 4 + lane_m;
#pragma unroll
        for (int j = 0; j < TN; ++j) wrow[j] = j * 8 + lane_n;
        for (int it = 0; it < iters; ++it) {
#pragma unroll 2
            for (int k = 0; k < KSM; k += 4) {
                ulonglong2 av[TM];
#pragma unroll
                for (int i = 0; i < TM; ++i) av[i] = *opnd(As, 32, arow[i], k);
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    ulonglong2 wv = *opnd(Ws, 64, wrow[j], k);
#pragma unroll
                    for (int i = 0; i < TM; ++i) {
                        float p0, p1, p2, p3;
                        if constexpr (MODE == MIX_MUL2_MAX3) {
                            unpack2(mul2(av[i].x, wv.x), p0, p1);
                            unpack2(mul2(av[i].y, wv.y), p2, p3);
                        } else {
                            float a0, a1, a2, a3, w0, w1, w2, w3;
                            unpack2(av[i].x, a0, a1);
                            unpack2(av[i].y, a2, a3);
                            unpack2(wv.x, w0, w1);
                            unpack2(wv.y, w2, w3);
                            p0 = __fmul_rn(a0, w0);
                            p1 = __fmul_rn(a1, w1);
                            p2 = __fmul_rn(a2, w2);
                            p3 = __fmul_rn(a3, w3);
                        }
                        if constexpr (MODE == MIX_SCALAR) {
                            vmax[i][j] = fmaxf(fmaxf(fmaxf(fmaxf(vmax[i][j], p0), p1), p2), p3);
                            vmin[i][j] = fminf(fminf(fminf(fminf(vmin[i][j], p0), p1), p2), p3);
                        } else if constexpr (MODE == MIX_NAIVE_INDEX) {
                            const float pp[4] = {p0, p1, p2, p3};
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                if (pp[q] > vmax[i][j]) { vmax[i][j] = pp[q]; imax[i][j] = k + q; }
                                if (pp[q] < vmin[i][j]) { vmin[i][j] = pp[q]; imin[i][j] = k + q; }
                            }
                        } else {
                            vmax[i][j] = fmax3(fmax3(vmax[i][j], p0, p1), p2, p3);
                            vmin[i][j] = fmin3(fmin3(vmin[i][j], p0, p1), p2, p3);
                        }
                    }
                }
            }
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                s += vmax[i][j] + vmin[i][j];
                if constexpr (MODE == MIX_NAIVE_INDEX) s += (float)(imax[i][j] + imin[i][j]);
            }
        out[blockIdx.x * THREADS + threadIdx.x] = s;
    }
    long long t1 = clock64();
    if (threadIdx.x == 0) clk_out[blockIdx.x] = t1 - t0;
}

template <int MODE>
static void run(int sms, float* d_out, long long* d_clk) {
    const size_t smem = 96 * KSM * sizeof(float);
    CK(cudaFuncSetAttribute(probe_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int iters = (MODE <= PURE_SETP_SEL) ? 4000 : 200;
    // lane-ops the timed loop issues per thread (the unit that matters for each mode)
    double per_thread;
    const char* what;
    if (MODE <= PURE_SETP_SEL) {
        per_thread = (double)iters * 16 * 16 * ((MODE == PURE_FMUL2) ? 0.5 : 1.0);
        what = (MODE == PURE_SETP_SEL) ? "setp+selp+selp triples" : "instructions";
    } else if (MODE == MIX_BLOCKTRACK) {
        per_thread = (double)iters * KSM * 4 * 8;
        what = "units";
    } else {
        per_thread = (double)iters * KSM * 8 * 8;
        what = "units";
    }
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    for (int ctas_per_sm = 1; ctas_per_sm <= ((MODE <= PURE_SETP_SEL) ? 2 : 1); ++ctas_per_sm) {
        const int grid = sms * ctas_per_sm;
        probe_kernel<MODE><<<grid, THREADS, smem>>>(d_out, iters / 10 + 1, d_clk);  // warm-up
        CK(cudaDeviceSynchronize());
        CK(cudaEventRecord(e0));
        probe_kernel<MODE><<<grid, THREADS, smem>>>(d_out, iters, d_clk);
        CK(cudaEventRecord(e1));
        CK(cudaDeviceSynchronize());
        float ms;
        CK(cudaEventElapsedTime(&ms, e0, e1));
        std::vector<long long> clk(grid);
        CK(cudaMemcpy(clk.data(), d_clk, grid * sizeof(long long), cudaMemcpyDeviceToHost));
        double mean_clk = 0;
        for (auto c : clk) mean_clk += (double)c;
        mean_clk /= grid;
        const double per_sm = per_thread * THREADS * ctas_per_sm;
        printf("{\"probe\": \"%s\", \"counted\": \"%s\", \"threads_per_sm\": %d, \"ms\": %.4f, "
               "\"sm_clocks\": %.0f, \"per_clk_per_sm\": %.2f, \"total_per_s\": %.4e, "
               "\"implied_sm_mhz\": %.0f}\n",
               mode_name[MODE], what, THREADS * ctas_per_sm, ms, mean_clk, per_sm / mean_clk,
               per_sm * sms / (ms * 1e-3), mean_clk / (ms * 1e-3) * 1e-6);
        fflush(stdout);
    }
}

// ---------------------------------------------------------------- datapath-sharing probes
// Register-only streams with NO dependency between the max/min instructions and the multiplies:
// whatever slows the mix down here is the hardware's issue/datapath structure, not latency.
//   0  max.f32 (3-input) alone, all three sources distinct registers
//   1  2 max3 : 1 mul.rn.f32x2 with register operands      (the instruction mix of the MAM loop)
//   2  2 max3 : 2 scalar mul.rn.f32 with register operands (same work, scalar multiplies)
//   3  2 max3 : 1 scalar mul.rn.f32 by an immediate         (multiplies the compiler can keep scalar)
// Reported: max3 instructions per clock per SM (64 = the ALU pipe saturated).
template <int VAR>
__global__ void __launch_bounds__(THREADS, 1)
share_probe_kernel(float* out, int iters, long long* clk_out) {
    float m[32];
    f32x2_t s[16], f[16], g[16];
#pragma unroll
    for (int i = 0; i < 32; ++i) m[i] = out[i] + threadIdx.x;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        s[i] = pack2(out[i + 32] + threadIdx.x, out[i + 33]);
        f[i] = pack2(out[i + 48] * 0.f + 1.f, 1.0f + out[i + 49] * 0.f);
        g[i] = pack2(1.f + out[i + 50] * 0.f, 1.f + out[i + 51] * 0.f);
    }
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float lo, hi;
                unpack2(s[(i * 5 + r * 3) & 15], lo, hi);
                asm volatile("max.f32 %0, %0, %1, %2;" : "+f"(m[i]) : "f"(lo), "f"(hi));
                if ((i & 1) == 0) {
                    const int fi = i >> 1, gi = ((i >> 1) * 3 + r) & 15;
                    if constexpr (VAR == 1) {
                        asm volatile("mul.rn.f32x2 %0, %0, %1;" : "+l"(f[fi]) : "l"(g[gi]));
                    } else if constexpr (VAR == 2) {
                        float a0, a1, b0, b1;
                        unpack2(f[fi], a0, a1);
                        unpack2(g[gi], b0, b1);
                        asm volatile("mul.rn.f32 %0, %0, %1;" : "+f"(a0) : "f"(b0));
                        asm volatile("mul.rn.f32 %0, %0, %1;" : "+f"(a1) : "f"(b1));
                        f[fi] = pack2(a0, a1);
                    } else if constexpr (VAR == 3) {
                        float a0, a1;
                        unpack2(f[fi], a0, a1);
                        asm volatile("mul.rn.f32 %0, %0, 0f3F800001;" : "+f"(a0));
                        f[fi] = pack2(a0, a1);
                    }
                }
            }
        }
    }
    long long t1 = clock64();
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) acc += m[i];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float lo, hi;
        unpack2(f[i], lo, hi);
        acc += lo + hi;
    }
    out[blockIdx.x * THREADS + threadIdx.x + 64] = acc;
    if (threadIdx.x == 0) clk_out[blockIdx.x] = t1 - t0;
}

template <int VAR>
static void run_share(int sms, float* d_out, long long* d_clk) {
    static const char* nm[4] = {"share_max3_only", "share_2max3_1fmul2_reg", "share_2max3_2fmul_reg",
                                "share_2max3_1fmul_imm"};
    const int iters = 2000;
    share_probe_kernel<VAR><<<sms, THREADS>>>(d_out, 20, d_clk);
    CK(cudaDeviceSynchronize());
    share_probe_kernel<VAR><<<sms, THREADS>>>(d_out, iters, d_clk);
    CK(cudaDeviceSynchronize());
    std::vector<long long> clk(sms);
    CK(cudaMemcpy(clk.data(), d_clk, sms * sizeof(long long), cudaMemcpyDeviceToHost));
    double mean_clk = 0;
    for (auto c : clk) mean_clk += (double)c;
    mean_clk /= sms;
    printf("{\"probe\": \"%s\", \"counted\": \"max3 instructions\", \"threads_per_sm\": %d, "
           "\"per_clk_per_sm\": %.2f}\n",
           nm[VAR], THREADS, (double)iters * 4 * 32 * THREADS / mean_clk);
    fflush(stdout);
}

// ---------------------------------------------------------------- scatter-add probes
// SPACE 0: fp32 atomic add into shared memory bins; 1: fp32 red.global.add into an L2-resident
// matrix; 2: int32 atomic add into shared memory.  Addresses are pseudo-random with no
// intra-warp structure, the access pattern of the selected-pair backward scatter.
template <int SPACE>
__global__ void __launch_bounds__(THREADS, 1)
scatter_probe_kernel(float* gbuf, unsigned gmask, int iters, long long* clk_out) {
    extern __shared__ __align__(16) float smem[];
    constexpr int BINS = 12288;  // 48 KB of fp32 bins
    for (int i = threadIdx.x; i < BINS; i += THREADS) smem[i] = 0.f;
    __syncthreads();
    unsigned h = (blockIdx.x * THREADS + threadIdx.x) * 2654435761u + 12345u;
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            h = h * 1664525u + 1013904223u;
            const unsigned r = h >> 8;
            if constexpr (SPACE == 0) {
                atomicAdd(&smem[r % BINS], 1.0f);
            } else if constexpr (SPACE == 1) {
                atomicAdd(&gbuf[r & gmask], 1.0f);
            } else {
                atomicAdd(reinterpret_cast<int*>(smem) + (r % BINS), 1);
            }
        }
    }
    __syncthreads();
    long long t1 = clock64();
    if (threadIdx.x == 0) {
        clk_out[blockIdx.x] = t1 - t0;
        gbuf[blockIdx.x] += smem[5];
    }
}

template <int SPACE>
static void run_scatter(int sms, long long* d_clk) {
    const size_t smem = 12288 * sizeof(float);
    CK(cudaFuncSetAttribute(scatter_probe_kernel<SPACE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const unsigned gelems = 1u << 22;  // 16 MB fp32, stays in L2
    float* gbuf;
    CK(cudaMalloc(&gbuf, gelems * sizeof(float)));
    CK(cudaMemset(gbuf, 0, gelems * sizeof(float)));
    const int iters = 2000;
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    scatter_probe_kernel<SPACE><<<sms, THREADS, smem>>>(gbuf, gelems - 1, 50, d_clk);
    CK(cudaDeviceSynchronize());
    CK(cudaEventRecord(e0));
    scatter_probe_kernel<SPACE><<<sms, THREADS, smem>>>(gbuf, gelems - 1, iters, d_clk);
    CK(cudaEventRecord(e1));
    CK(cudaDeviceSynchronize());
    float ms;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    std::vector<long long> clk(sms);
    CK(cudaMemcpy(clk.data(), d_clk, sms * sizeof(long long), cudaMemcpyDeviceToHost));
    double mean_clk = 0;
    for (auto c : clk) mean_clk += (double)c;
    mean_clk /= sms;
    const double per_sm = (double)iters * 8 * THREADS;
    static const char* nm[3] = {"scatter_smem_f32_atomic", "scatter_global_f32_red", "scatter_smem_i32_atomic"};
    printf("{\"probe\": \"%s\", \"counted\": \"atomic lane-ops\", \"threads_per_sm\": %d, \"ms\": %.4f, "
           "\"sm_clocks\": %.0f, \"per_clk_per_sm\": %.3f, \"total_per_s\": %.4e}\n",
           nm[SPACE], THREADS, ms, mean_clk, per_sm / mean_clk, per_sm * sms / (ms * 1e-3));
    fflush(stdout);
    CK(cudaFree(gbuf));
}

int main() {
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, 0));
    const int sms = prop.multiProcessorCount;
    printf("{\"device\": \"%s\", \"sms\": %d, \"cc\": \"%d.%d\"}\n", prop.name, sms, prop.major, prop.minor);
    float* d_out;
    long long* d_clk;
    CK(cudaMalloc(&d_out, (size_t)sms * 2 * THREADS * sizeof(float)));
    CK(cudaMalloc(&d_clk, (size_t)sms * 2 * sizeof(long long)));
    run<PURE_FMUL>(sms, d_out, d_clk);
    run<PURE_FFMA>(sms, d_out, d_clk);
    run<PURE_FMUL2>(sms, d_out, d_clk);
    run<PURE_FMNMX>(sms, d_out, d_clk);
    run<PURE_FMNMX3>(sms, d_out, d_clk);
    run<PURE_SETP_SEL>(sms, d_out, d_clk);
    run<MIX_SCALAR>(sms, d_out, d_clk);
    run<MIX_MAX3>(sms, d_out, d_clk);
    run<MIX_MUL2_MAX3>(sms, d_out, d_clk);
    run<MIX_NAIVE_INDEX>(sms, d_out, d_clk);
    run<MIX_BLOCKTRACK>(sms, d_out, d_clk);
    run_share<0>(sms, d_out, d_clk);
    run_share<1>(sms, d_out, d_clk);
    run_share<2>(sms, d_out, d_clk);
    run_share<3>(sms, d_out, d_clk);
    run_scatter<0>(sms, d_clk);
    run_scatter<1>(sms, d_clk);
    run_scatter<2>(sms, d_clk);
    CK(cudaFree(d_out));
    CK(cudaFree(d_clk));
    return 0;
}
