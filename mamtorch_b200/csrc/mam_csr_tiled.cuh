// Pruned-weight MAM forward, tiled form: rows of a ride on the lanes, stored weights are broadcast.
//
// Same contract as mam_csr_fwd_kernel (mam_csr.cuh): the result of the dense layer on W with zeros
// at the positions that are not stored, indices with the lowest-k tie rule.  The reference has no
// sparse MAM kernel (its pruning example zeroes dense weights,
// examples/vitb16_imagenet1k/pruning_utils.py:105-116); what it does have for sparse operands is the
// cuSPARSE wrapper in mamtorch/sparse/kernel/v1/csrc/cuda/cusparsemm_csr.cu:19-77.
//
// Why a second form: with one stored entry per lane every product needs its own gather from a row of
// a in shared memory (random banks) plus per-entry index tracking, and the kernel runs at ~4.5
// (m, stored k) units/clk/SM.  Here a CTA owns 128 rows of a and 64 rows of W.  The activations are
// used TRANSPOSED (aT[K][M], built once per call): for one stored entry (n, k, v) a warp reads
// aT[k][m0 .. m0+127] as one conflict-free LDS.128 per lane -- four rows of a per lane -- multiplies
// by the broadcast v with mul.rn.f32x2 and folds two entries per three-input max/min, the instruction
// mix of the dense kernel.  Each warp keeps 4 rows of W x 4 rows of a x (max, min) in registers and
// walks the stored entries of its 4 rows; aT arrives by TMA in stages of 64 columns, shared by the
// 16 warps (every staged value is used by ~0.1 * 64 stored entries at 90 % sparsity).
//
// The stored entries are regrouped once per call into stage-major segments -- all entries of W row n
// whose column falls into stage s, padded to an even count by repeating the last entry (max/min are
// idempotent) -- so that the entries a warp needs for one stage are one contiguous run.
//
// Indices: like the dense kernel, the loop tracks only WHICH STAGE last raised the running maximum
// (lowered the minimum): one compare, one predicated move and one predicated 16-bit store per
// accumulator and stage; what it stores is where that stage's entries of row n begin in the list.
// (Tracking per pair of entries was tried: it triples the instruction count of a loop that is
// issue-bound.)  mam_csr_resolve_kernel then rescans those entries (about 6 at 90 % sparsity) with
// strict compares in ascending k, and applies the rule for the implicit zero product of a pruned
// position (value 0 at k0 = the lowest column that is not stored).
#pragma once
#include <cuda.h>
#include "mam_csr.cuh"
#include "mam_fwd_tiled.cuh"

namespace mamb200 {

constexpr int CT_KS = 64;            // columns of a per TMA stage
constexpr int CT_BM = 128;           // rows of a per CTA: 4 per lane
constexpr int CT_WARPS = 16;
constexpr int CT_WROWS = 4;          // rows of W per warp
constexpr int CT_BN = CT_WARPS * CT_WROWS;
constexpr int CT_THREADS = CT_WARPS * 32;
constexpr int CT_STAGES = 4;
constexpr int CT_LOOKAHEAD = CT_STAGES - 2;
constexpr int CT_STAGE_BYTES = CT_KS * CT_BM * 4;
constexpr int CT_ID_BYTES = 2 * CT_WROWS * 4 * CT_THREADS * 4;   // one 32-bit list offset per accumulator
constexpr int CT_EB_PAIRS = 32;                                  // entry pairs staged per warp at a time
constexpr int CT_EB_BYTES = CT_WARPS * CT_EB_PAIRS * 16;
constexpr int CT_SMEM_BYTES = 1024 + CT_STAGES * CT_STAGE_BYTES + CT_ID_BYTES + CT_EB_BYTES + 2 * CT_STAGES * 8;
static_assert(CT_BM * (CT_BN + 1) * 4 <= CT_STAGES * CT_STAGE_BYTES, "output staging reuses the stage ring");

struct CsrEntry {
    int koff;   // (k - first column of the stage) * CT_BM * 4: byte offset of row k inside the stage
    float v;
};
// The same entries as the resolver wants them: the column itself, with the top bit set on the last
// true entry of a (row, stage) segment (the padding entry behind it is never looked at).
struct CsrColEntry {
    unsigned k;
    float v;
};
constexpr unsigned CSR_LAST = 0x80000000u;
constexpr int CSR_NO_ENTRY = -1;   // list offset recorded for an output whose row stores nothing

// first position in [lo, hi) whose column is >= key
__device__ __forceinline__ long long csr_lower_bound(const long long* __restrict__ col, long long lo, long long hi,
                                                     long long key) {
    while (lo < hi) {
        const long long mid = (lo + hi) >> 1;
        if (col[mid] < key) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// counts[s * N + n] = stored entries of row n inside stage s, rounded up to even;
// k0[n] = lowest column of row n that is not stored (K when the row is full)
__global__ void __launch_bounds__(256)
csr_tile_count_kernel(const long long* __restrict__ crow, const long long* __restrict__ col,
                      int* __restrict__ counts, int* __restrict__ k0, long long N, long long K, int nks) {
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= (long long)nks * N) return;
    const int s = (int)(idx / N);
    const long long n = idx - (long long)s * N;
    const long long rs = crow[n], re = crow[n + 1];
    const long long lo = csr_lower_bound(col, rs, re, (long long)s * CT_KS);
    const long long hi = csr_lower_bound(col, lo, re, (long long)(s + 1) * CT_KS);
    counts[idx] = (int)((hi - lo + 1) & ~1LL);
    if (s == 0) {
        // columns are ascending and distinct: col[rs + t] == t holds for a prefix and fails from the
        // first missing column on
        long long a = 0, b = re - rs;
        while (a < b) {
            const long long mid = (a + b) >> 1;
            if (col[rs + mid] == mid) a = mid + 1; else b = mid;
        }
        k0[n] = (int)min(a, K);
    }
}

// Exclusive scan seg[i] = sum of counts[0..i), seg[n] = total, in three launches: per-block sums
// (CSR_SCAN_BLOCK elements each), a one-CTA scan of those sums, and the block-local scans offset by them.
// The grid covers n + 1 positions so that some block writes seg[n].
constexpr int CSR_SCAN_ROUND = 4096;                    // elements per 1024-thread round (one int4 each)
constexpr int CSR_SCAN_BLOCK = 4 * CSR_SCAN_ROUND;      // elements per CTA

__global__ void __launch_bounds__(1024)
csr_scan_block_sums_kernel(const int* __restrict__ counts, int* __restrict__ block_sums, long long n) {
    __shared__ int warp_sums[32];
    const long long base = (long long)blockIdx.x * CSR_SCAN_BLOCK;
    int sum = 0;
    for (int i = threadIdx.x; i < CSR_SCAN_BLOCK; i += 1024) sum += base + i < n ? counts[base + i] : 0;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x < 32) {
        int v = warp_sums[threadIdx.x];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
        if (threadIdx.x == 0) block_sums[blockIdx.x] = v;
    }
}

// in place: sums[i] <- sum of sums[0..i); one CTA, any length
__global__ void __launch_bounds__(1024)
csr_scan_sums_kernel(int* __restrict__ sums, long long nb) {
    __shared__ int warp_sums[32];
    __shared__ int carry_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) carry_s = 0;
    __syncthreads();
    for (long long base = 0; base < nb; base += 1024) {
        const int v = base + tid < nb ? sums[base + tid] : 0;
        int incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        int wbase = 0;
        for (int w2 = 0; w2 < warp; ++w2) wbase += warp_sums[w2];
        const int excl = carry_s + wbase + incl - v;
        if (base + tid < nb) sums[base + tid] = excl;
        __syncthreads();
        if (tid == 1023) carry_s = excl + v;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(1024)
csr_scan_apply_kernel(const int* __restrict__ counts, const int* __restrict__ block_offsets, int* __restrict__ seg,
                      long long n) {
    __shared__ int warp_sums[32];
    __shared__ int carry_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) carry_s = block_offsets[blockIdx.x];
    __syncthreads();
    const long long block_base = (long long)blockIdx.x * CSR_SCAN_BLOCK;
    for (int round = 0; round < CSR_SCAN_BLOCK / CSR_SCAN_ROUND; ++round) {
        const long long base = block_base + (long long)round * CSR_SCAN_ROUND + (long long)tid * 4;
        int v[4], sum = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = base + i < n ? counts[base + i] : 0;
            sum += v[i];
        }
        int incl = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        int wbase = 0;
        for (int w2 = 0; w2 < warp; ++w2) wbase += warp_sums[w2];
        int run = carry_s + wbase + incl - sum;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (base + i <= n) seg[base + i] = run;   // position n receives the grand total
            run += v[i];
        }
        __syncthreads();
        if (tid == 1023) carry_s = run;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256)
csr_tile_fill_kernel(const long long* __restrict__ crow, const long long* __restrict__ col,
                     const float* __restrict__ val, const int* __restrict__ seg, CsrEntry* __restrict__ list,
                     CsrColEntry* __restrict__ rlist, long long N, int nks, int pad_with_zero) {
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= (long long)nks * N) return;
    const int s = (int)(idx / N);
    const long long n = idx - (long long)s * N;
    const long long rs = crow[n], re = crow[n + 1];
    const long long lo = csr_lower_bound(col, rs, re, (long long)s * CT_KS);
    const long long hi = csr_lower_bound(col, lo, re, (long long)(s + 1) * CT_KS);
    long long p = seg[idx];
    CsrEntry last{0, 0.f};
    CsrColEntry rlast{0u, 0.f};
    for (long long t = lo; t < hi; ++t) {
        last.koff = (int)(col[t] - (long long)s * CT_KS) * (CT_BM * 4);
        last.v = val[t];
        rlast.k = (unsigned)col[t] | (t + 1 == hi ? CSR_LAST : 0u);
        rlast.v = last.v;
        list[p] = last;
        if (rlist) rlist[p] = rlast;
        ++p;
    }
    if ((hi - lo) & 1) {
        // max/min are idempotent, so their padding repeats the last entry; a sum needs a zero instead
        if (pad_with_zero) last.v = 0.f;
        list[p] = last;
        if (rlist) rlist[p] = rlast;
    }
}

// out[c * pitch + r] = in[r * C + c]
__global__ void __launch_bounds__(256)
mam_transpose_pitch_kernel(const float* __restrict__ in, float* __restrict__ out, long long R, long long C,
                           long long pitch) {
    __shared__ float t[32][33];
    const long long c0 = (long long)blockIdx.x * 32, r0 = (long long)blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const long long r = r0 + ty + 8 * p, c = c0 + tx;
        if (r < R && c < C) t[ty + 8 * p][tx] = in[r * C + c];
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const long long c = c0 + ty + 8 * p, r = r0 + tx;
        if (r < R && c < C) out[c * pitch + r] = t[tx][ty + 8 * p];
    }
}

struct CsrTiledParams {
    const int* seg;        // [nks * N + 1] stage-major segment offsets into list
    const CsrEntry* list;
    const int* k0;         // [N]
    const float* bias;     // [N] or nullptr
    float* y;
    int* cid_max;          // TRACK: list offsets of the recorded segments, resolved in place by mam_csr_resolve_kernel
    int* cid_min;
    long long M, K, N;
    int nks;
    float one;             // 1.0f kept opaque to the compiler
    int* error;
};

template <bool TRACK>
__global__ void __launch_bounds__(CT_THREADS, 1)
mam_csr_tiled_kernel(const __grid_constant__ CUtensorMap tmAT, const CsrTiledParams prm) {
    extern __shared__ unsigned char ct_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(ct_smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* ids = smem + CT_STAGES * CT_STAGE_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ids + CT_ID_BYTES + CT_EB_BYTES);   // entry staging sits in between
    uint64_t* empty_bar = full_bar + CT_STAGES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long N = prm.N;
    const long long n_cta = (long long)blockIdx.x * CT_BN;
    const long long m0 = (long long)blockIdx.y * CT_BM;
    const int nks = prm.nks;

    if (tid == 0) {
        for (int s = 0; s < CT_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], CT_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();

    // producer: stage p_ks of aT, columns [p_ks*64, +64) x rows [m0, m0+128).  Every thread steps the position;
    // the warp that issues the copy changes from stage to stage, so that no warp is permanently the slowest.
    int p_ks = 0, p_stage = 0;
    uint32_t p_phase = 0;
    auto produce_one = [&](const bool issue) -> bool {
        if (p_ks >= nks) return true;
        bool good = true;
        if (issue) {
            good = mbar_wait_bounded(&empty_bar[p_stage], p_phase ^ 1u);
            if (good) {
                mbar_expect_tx(&full_bar[p_stage], CT_STAGE_BYTES);
                tma_load_2d(smem + p_stage * CT_STAGE_BYTES, &tmAT, &full_bar[p_stage], (int)m0, p_ks * CT_KS);
            }
        }
        if (++p_stage == CT_STAGES) { p_stage = 0; p_phase ^= 1u; }
        ++p_ks;
        return good;
    };
    if (tid == 0) tma_prefetch_desc(&tmAT);
    for (int i = 0; i < CT_LOOKAHEAD; ++i) produce_one(tid == 0);

    const long long n_w = n_cta + warp * CT_WROWS;          // first W row of this warp
    const uint32_t id_addr = smem_u32(ids) + (uint32_t)tid * 4u;
    int4* eb = reinterpret_cast<int4*>(ids + CT_ID_BYTES) + warp * CT_EB_PAIRS;   // this warp's staged entry pairs
    const int4* list4 = reinterpret_cast<const int4*>(prm.list);
    float cmax[CT_WROWS][4], cmin[CT_WROWS][4];              // running extremes
    float pmax[TRACK ? CT_WROWS : 1][4], pmin[TRACK ? CT_WROWS : 1][4];  // their values at the last stage boundary
#pragma unroll
    for (int j = 0; j < CT_WROWS; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            cmax[j][i] = -INFINITY;
            cmin[j][i] = INFINITY;
            if constexpr (TRACK) {
                pmax[j][i] = -INFINITY;
                pmin[j][i] = INFINITY;
            }
        }
    if constexpr (TRACK) {
#pragma unroll
        for (int s = 0; s < 2 * CT_WROWS * 4; ++s) {
            const uint32_t addr = id_addr + (uint32_t)(s * CT_THREADS * 4);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(CSR_NO_ENTRY) : "memory");
        }
    }

    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // segment offsets of this warp's rows for one stage: lane j holds the start of row j (lane
    // CT_WROWS the end of the last row); rows beyond N read the start of the next stage's first row,
    // i.e. form empty segments.  Offsets are even (segments are padded), so /2 gives pair indices.
    auto load_seg = [&](int ks) -> int {
        const long long r = min(n_w + (long long)lane, N);
        return (lane <= CT_WROWS && ks < nks) ? __ldg(prm.seg + (long long)ks * N + r) : 0;
    };
    int seg_next = load_seg(0);
    // the pair this lane will stage for the coming stage, fetched one stage ahead
    int4 pre = make_int4(0, 0, 0, 0);
    {
        const int p0 = __shfl_sync(0xffffffffu, seg_next, 0) >> 1, p1 = __shfl_sync(0xffffffffu, seg_next, CT_WROWS) >> 1;
        if (p0 + lane < p1) pre = __ldg(list4 + p0 + lane);
    }
    for (int ks = 0; ks < nks; ++ks) {
        const int seg_cur = seg_next;
        seg_next = load_seg(ks + 1);
        int bnd[CT_WROWS + 1];   // pair-index boundaries of the 4 rows: one contiguous run of the list
#pragma unroll
        for (int j = 0; j <= CT_WROWS; ++j) bnd[j] = __shfl_sync(0xffffffffu, seg_cur, j) >> 1;
        int4 mine = pre;
        {
            const int p0 = __shfl_sync(0xffffffffu, seg_next, 0) >> 1, p1 = __shfl_sync(0xffffffffu, seg_next, CT_WROWS) >> 1;
            pre = make_int4(0, 0, 0, 0);
            if (p0 + lane < p1) pre = __ldg(list4 + p0 + lane);
        }
        if (!produce_one(lane == 0 && warp == ks % CT_WARPS)) atomicExch(prm.error, 1);
        if (!mbar_wait_bounded(&full_bar[stage], phase)) {
            atomicExch(prm.error, 1);
            ok = false;
            break;
        }
        const uint32_t xs = smem_u32(smem) + (uint32_t)(stage * CT_STAGE_BYTES) + (uint32_t)lane * 16u;
        const uint32_t ebs = smem_u32(eb);
        for (int off = bnd[0]; off < bnd[CT_WROWS]; off += CT_EB_PAIRS) {
            if (off > bnd[0]) {   // a run longer than the staging buffer: fetch the next batch directly
                mine = make_int4(0, 0, 0, 0);
                if (off + lane < bnd[CT_WROWS]) mine = __ldg(list4 + off + lane);
            }
            __syncwarp();
            eb[lane] = mine;
            __syncwarp();
            // one pair of entries (the same for every lane), then the two rows of aT they name
            auto fetch = [&](int q, int4& e, ulonglong2& x0, ulonglong2& x1) {
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(e.x), "=r"(e.y), "=r"(e.z), "=r"(e.w)
                             : "r"(ebs + (uint32_t)q * 16u)
                             : "memory");   // stays behind the staging store above
                x0 = lds128_at<0>(xs + (uint32_t)e.x);
                x1 = lds128_at<0>(xs + (uint32_t)e.z);
            };
            static_for<0, CT_WROWS>([&](auto jc) {
                constexpr int j = decltype(jc)::value;
                const int lo = max(bnd[j], off) - off, hi = min(bnd[j + 1], off + CT_EB_PAIRS) - off;
                auto consume = [&](const int4& e, const ulonglong2& x0, const ulonglong2& x1) {
                    const float v0 = __int_as_float(e.y), v1 = __int_as_float(e.w);
                    const f32x2_t vv0 = pack2(v0, v0), vv1 = pack2(v1, v1);
                    float pa[4], pb[4];
                    unpack2(mul2(x0.x, vv0), pa[0], pa[1]);
                    unpack2(mul2(x0.y, vv0), pa[2], pa[3]);
                    unpack2(mul2(x1.x, vv1), pb[0], pb[1]);
                    unpack2(mul2(x1.y, vv1), pb[2], pb[3]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        cmax[j][i] = fmax3(cmax[j][i], pa[i], pb[i]);
                        cmin[j][i] = fmin3(cmin[j][i], pa[i], pb[i]);
                    }
                };
#pragma unroll 2
                for (int q = lo; q < hi; ++q) {
                    int4 e;
                    ulonglong2 x0, x1;
                    fetch(q, e, x0, x1);
                    consume(e, x0, x1);
                }
            });
        }
        if constexpr (TRACK) {
            // did the running extreme move inside this stage?  One compare per accumulator; the
            // snapshot is refreshed through a multiply by an opaque 1.0 so that the move issues on the
            // FMA pipe.  (No "memory" clobber: the slots are read only after the loop, behind a barrier.)
            static_for<0, CT_WROWS * 4>([&](auto slot) {
                constexpr int S = decltype(slot)::value;
                constexpr int j = S / 4, i = S % 4;
                const int t0 = bnd[j] * 2;   // where this stage's entries of row j begin
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.gt.f32 p, %1, %0;\n\t"
                    "@p mul.rn.f32 %0, %1, %2;\n\t"
                    "@p st.shared.u32 [%3+%5], %4;\n\t}"
                    : "+f"(pmax[j][i])
                    : "f"(cmax[j][i]), "f"(prm.one), "r"(id_addr), "r"(t0), "n"((S * 2 + 0) * CT_THREADS * 4));
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.lt.f32 p, %1, %0;\n\t"
                    "@p mul.rn.f32 %0, %1, %2;\n\t"
                    "@p st.shared.u32 [%3+%5], %4;\n\t}"
                    : "+f"(pmin[j][i])
                    : "f"(cmin[j][i]), "f"(prm.one), "r"(id_addr), "r"(t0), "n"((S * 2 + 1) * CT_THREADS * 4));
            });
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == CT_STAGES) { stage = 0; phase ^= 1u; }
    }
    // every warp is done with the ring (and every TMA write has landed) before it is reused below;
    // a wait that gave up in any warp ends the whole CTA here
    if (__syncthreads_or(ok ? 0 : 1)) return;

    // ---- epilogue: the 128 x 64 output tile goes through shared memory so that rows are written
    // as 256-byte runs.  Row of the tile = 4*lane + i, column = 4*warp + j.
    float* tile = reinterpret_cast<float*>(smem);
    constexpr int TP = CT_BN + 1;
    auto flush = [&](auto* dst) {
        __syncthreads();
        for (int idx = tid; idx < CT_BM * CT_BN; idx += CT_THREADS) {
            const int r = idx / CT_BN, c = idx % CT_BN;
            const long long m = m0 + r, n = n_cta + c;
            if (m < prm.M && n < N) {
                using T = std::remove_pointer_t<decltype(dst)>;
                T v;
                if constexpr (std::is_same_v<T, float>) v = tile[r * TP + c];
                else v = (T)__float_as_int(tile[r * TP + c]);
                dst[m * N + n] = v;
            }
        }
        __syncthreads();
    };
#pragma unroll
    for (int j = 0; j < CT_WROWS; ++j) {
        const long long n = n_w + j;
        const bool implicit = n < N && __ldg(prm.k0 + min(n, N - 1)) < prm.K;
        const float b = (prm.bias && n < N) ? __ldg(prm.bias + n) : 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float vmax = cmax[j][i], vmin = cmin[j][i];
            if (implicit) {
                if (0.f > vmax) vmax = 0.f;
                if (0.f < vmin) vmin = 0.f;
            }
            float out = __fadd_rn(vmax, vmin);
            if (prm.bias) out = __fadd_rn(out, b);
            tile[(4 * lane + i) * TP + 4 * warp + j] = out;
        }
    }
    flush(prm.y);
    if constexpr (TRACK) {
#pragma unroll
        for (int side = 0; side < 2; ++side) {
#pragma unroll
            for (int j = 0; j < CT_WROWS; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    int c;
                    const uint32_t addr = id_addr + (uint32_t)((((j * 4 + i) * 2 + side) * CT_THREADS) * 4);
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(c) : "r"(addr) : "memory");
                    tile[(4 * lane + i) * TP + 4 * warp + j] = __int_as_float(c);
                }
            flush(side == 0 ? prm.cid_max : prm.cid_min);
        }
    }
}

// Recorded segments -> exact indices for the tiled CSR forward.  A CTA parks R rows of a in shared
// memory; each thread takes one column n at a time and resolves the max and the min of all R rows
// together: the 2R segment walks advance in lockstep, so that their (L2-latency-bound) entry loads
// are in flight at the same time.  A walk reads the entries of the recorded (row, stage) segment two
// at a time in ascending k with strict compares, up to the entry flagged as the segment's last; the
// result is then weighed against the implicit zero of a pruned position.
template <int R>
__global__ void __launch_bounds__(512)
mam_csr_resolve_kernel(const float* __restrict__ a, const CsrColEntry* __restrict__ rlist,
                       const int* __restrict__ k0, int* __restrict__ argmax, int* __restrict__ argmin,
                       long long M, long long K, long long N) {
    extern __shared__ float cr_smem[];  // [R][K]
    const long long m0 = (long long)blockIdx.x * R;
    const int rows = (int)min((long long)R, M - m0);
    for (long long i = threadIdx.x; i < (long long)rows * K; i += 512) cr_smem[i] = a[m0 * K + i];
    __syncthreads();
    const unsigned NONE = 0x7fffffffu;
    const uint4* pairs = reinterpret_cast<const uint4*>(rlist);
    constexpr int T = 2 * R;   // walks per thread: task q = row q/2, side q%2 (0 = max, 1 = min)
    for (long long n = threadIdx.x; n < N; n += 512) {
        const unsigned kk0 = (unsigned)__ldg(k0 + n);
        const bool implicit = kk0 < (unsigned long long)K;
        int t[T];
        float best[T];
        unsigned bk[T];
        unsigned active = 0;
#pragma unroll
        for (int q = 0; q < T; ++q) {
            best[q] = (q & 1) ? INFINITY : -INFINITY;
            bk[q] = NONE;
            t[q] = CSR_NO_ENTRY;
            if (q / 2 < rows) {
                const long long o = (m0 + q / 2) * N + n;
                t[q] = (q & 1) ? argmin[o] : argmax[o];
                if (t[q] != CSR_NO_ENTRY) active |= 1u << q;
            }
            t[q] >>= 1;   // segments start on even offsets: entries come as 16-byte pairs
        }
        for (int step = 0; step < CT_KS / 2 && active; ++step) {
            uint4 e[T];
#pragma unroll
            for (int q = 0; q < T; ++q)
                if (active & (1u << q)) e[q] = __ldg(pairs + t[q] + step);
#pragma unroll
            for (int q = 0; q < T; ++q) {
                if (active & (1u << q)) {
                    const float* ar = cr_smem + (long long)(q / 2) * K;
                    const unsigned ka = e[q].x & ~CSR_LAST, kb = e[q].z & ~CSR_LAST;
                    const float pa = __fmul_rn(ar[ka], __uint_as_float(e[q].y));
                    if ((q & 1) ? pa < best[q] : pa > best[q]) { best[q] = pa; bk[q] = ka; }
                    if (e[q].x & CSR_LAST) {
                        active &= ~(1u << q);
                    } else {
                        const float pb = __fmul_rn(ar[kb], __uint_as_float(e[q].w));
                        if ((q & 1) ? pb < best[q] : pb > best[q]) { best[q] = pb; bk[q] = kb; }
                        if (e[q].z & CSR_LAST) active &= ~(1u << q);
                    }
                }
            }
        }
#pragma unroll
        for (int q = 0; q < T; ++q) {
            if (q / 2 < rows) {
                if (implicit) {
                    const bool zero_wins = (q & 1) ? 0.f < best[q] : 0.f > best[q];
                    if (zero_wins) bk[q] = kk0; else if (0.f == best[q]) bk[q] = min(bk[q], kk0);
                }
                const long long o = (m0 + q / 2) * N + n;
                ((q & 1) ? argmin : argmax)[o] = (int)min(bk[q], (unsigned)(K - 1));
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// C[N, Mc] = A_csr[N, K] . B[K, Mc] in the ordinary sum semiring, on the same machinery: B is already
// "k-major with the other index contiguous", exactly what the MAM kernel above wants of the transposed
// activations, so a CTA takes 128 columns of B/C and 128 rows of A; B arrives by TMA in stages of 64
// rows, every lane owns 4 adjacent columns, every warp 8 rows of A whose stored entries are broadcast
// and applied with fma.rn.f32x2.  Entries of a row are applied in ascending column order, so a result
// does not depend on the tiling.  Stands in for cusparsemm_csr / cusparsemm_coo of the reference
// (mamtorch/sparse/kernel/v1/csrc/cuda/cusparsemm_csr.cu:19-77, cusparsemm_coo.cu:19-76).
constexpr int SP_WROWS = 8;
constexpr int SP_BN = CT_WARPS * SP_WROWS;
constexpr int SP_STAGES = 6;
constexpr int SP_LOOKAHEAD = SP_STAGES - 2;
constexpr int SP_SMEM_BYTES = 1024 + SP_STAGES * CT_STAGE_BYTES + CT_EB_BYTES + 2 * SP_STAGES * 8;

struct SpmmTiledParams {
    const int* seg;
    const CsrEntry* list;
    float* c;
    long long N, K, Mc;
    int nks;
    int* error;
};

__device__ __forceinline__ f32x2_t fma2(f32x2_t a, f32x2_t b, f32x2_t c) {
    f32x2_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__global__ void __launch_bounds__(CT_THREADS, 1)
mam_spmm_tiled_kernel(const __grid_constant__ CUtensorMap tmB, const SpmmTiledParams prm) {
    extern __shared__ unsigned char sp_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(sp_smem_raw) + 1023) & ~uintptr_t(1023));
    int4* eb_all = reinterpret_cast<int4*>(smem + SP_STAGES * CT_STAGE_BYTES);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SP_STAGES * CT_STAGE_BYTES + CT_EB_BYTES);
    uint64_t* empty_bar = full_bar + SP_STAGES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long N = prm.N;
    const long long n_cta = (long long)blockIdx.x * SP_BN;
    const long long j0 = (long long)blockIdx.y * CT_BM;
    const int nks = prm.nks;

    if (tid == 0) {
        for (int s = 0; s < SP_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], CT_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();

    // producer: every thread steps the position, the issuing warp rotates (see mam_csr_tiled_kernel)
    int p_ks = 0, p_stage = 0;
    uint32_t p_phase = 0;
    auto produce_one = [&](const bool issue) -> bool {
        if (p_ks >= nks) return true;
        bool good = true;
        if (issue) {
            good = mbar_wait_bounded(&empty_bar[p_stage], p_phase ^ 1u);
            if (good) {
                mbar_expect_tx(&full_bar[p_stage], CT_STAGE_BYTES);
                tma_load_2d(smem + p_stage * CT_STAGE_BYTES, &tmB, &full_bar[p_stage], (int)j0, p_ks * CT_KS);
            }
        }
        if (++p_stage == SP_STAGES) { p_stage = 0; p_phase ^= 1u; }
        ++p_ks;
        return good;
    };
    if (tid == 0) tma_prefetch_desc(&tmB);
    for (int i = 0; i < SP_LOOKAHEAD; ++i) produce_one(tid == 0);

    const long long n_w = n_cta + warp * SP_WROWS;
    int4* eb = eb_all + warp * CT_EB_PAIRS;
    const int4* list4 = reinterpret_cast<const int4*>(prm.list);
    f32x2_t acc[SP_WROWS][2];   // 4 adjacent columns of C per row of A, as two packed pairs
#pragma unroll
    for (int j = 0; j < SP_WROWS; ++j) acc[j][0] = acc[j][1] = pack2(0.f, 0.f);

    auto load_seg = [&](int ks) -> int {
        const long long r = min(n_w + (long long)lane, N);
        return (lane <= SP_WROWS && ks < nks) ? __ldg(prm.seg + (long long)ks * N + r) : 0;
    };
    int seg_next = load_seg(0);
    int4 pre = make_int4(0, 0, 0, 0);
    {
        const int p0 = __shfl_sync(0xffffffffu, seg_next, 0) >> 1, p1 = __shfl_sync(0xffffffffu, seg_next, SP_WROWS) >> 1;
        if (p0 + lane < p1) pre = __ldg(list4 + p0 + lane);
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int ks = 0; ks < nks; ++ks) {
        const int seg_cur = seg_next;
        seg_next = load_seg(ks + 1);
        int bnd[SP_WROWS + 1];
#pragma unroll
        for (int j = 0; j <= SP_WROWS; ++j) bnd[j] = __shfl_sync(0xffffffffu, seg_cur, j) >> 1;
        int4 mine = pre;
        {
            const int p0 = __shfl_sync(0xffffffffu, seg_next, 0) >> 1, p1 = __shfl_sync(0xffffffffu, seg_next, SP_WROWS) >> 1;
            pre = make_int4(0, 0, 0, 0);
            if (p0 + lane < p1) pre = __ldg(list4 + p0 + lane);
        }
        if (!produce_one(lane == 0 && warp == ks % CT_WARPS)) atomicExch(prm.error, 1);
        if (!mbar_wait_bounded(&full_bar[stage], phase)) {
            atomicExch(prm.error, 1);
            ok = false;
            break;
        }
        const uint32_t xs = smem_u32(smem) + (uint32_t)(stage * CT_STAGE_BYTES) + (uint32_t)lane * 16u;
        const uint32_t ebs = smem_u32(eb);
        for (int off = bnd[0]; off < bnd[SP_WROWS]; off += CT_EB_PAIRS) {
            if (off > bnd[0]) {
                mine = make_int4(0, 0, 0, 0);
                if (off + lane < bnd[SP_WROWS]) mine = __ldg(list4 + off + lane);
            }
            __syncwarp();
            eb[lane] = mine;
            __syncwarp();
            static_for<0, SP_WROWS>([&](auto jc) {
                constexpr int j = decltype(jc)::value;
                const int lo = max(bnd[j], off) - off, hi = min(bnd[j + 1], off + CT_EB_PAIRS) - off;
#pragma unroll 2
                for (int q = lo; q < hi; ++q) {
                    int4 e;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(e.x), "=r"(e.y), "=r"(e.z), "=r"(e.w)
                                 : "r"(ebs + (uint32_t)q * 16u)
                                 : "memory");
                    const ulonglong2 x0 = lds128_at<0>(xs + (uint32_t)e.x);
                    const ulonglong2 x1 = lds128_at<0>(xs + (uint32_t)e.z);
                    const float v0 = __int_as_float(e.y), v1 = __int_as_float(e.w);
                    const f32x2_t vv0 = pack2(v0, v0), vv1 = pack2(v1, v1);
                    acc[j][0] = fma2(x1.x, vv1, fma2(x0.x, vv0, acc[j][0]));
                    acc[j][1] = fma2(x1.y, vv1, fma2(x0.y, vv0, acc[j][1]));
                }
            });
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == SP_STAGES) { stage = 0; phase ^= 1u; }
    }
    if (!ok) return;   // nothing after the loop needs the whole CTA
    // each lane writes its 4 adjacent columns of every row: 512 contiguous bytes per row and warp
    const long long j = j0 + 4 * lane;
#pragma unroll
    for (int r = 0; r < SP_WROWS; ++r) {
        const long long n = n_w + r;
        if (n >= N) break;
        float v[4];
        unpack2(acc[r][0], v[0], v[1]);
        unpack2(acc[r][1], v[2], v[3]);
        float* o = prm.c + n * prm.Mc + j;
        if (j + 3 < prm.Mc) {
            *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (j + i < prm.Mc) o[i] = v[i];
        }
    }
}

}  // namespace mamb200
