// Patch (im2col) and fold (col2im) kernels around the MAM convolution.
//
// A MAM convolution is the fully-connected MAM problem over one row per output pixel:
// rows[m][k] = x[b][c][ho*sh - ph + kh][wo*sw - pw + kw], m = (b*Ho + ho)*Wo + wo,
// k = (c*kH + kh)*kW + kw, zero outside the image.  The reference keeps convolution only as
// never-compiled text: its host code permutes input, weight and output to column-major on every call
// (mamtorch/kernel/backup/mamconv2d.txt:70-100) and its module pads with F.pad
// (mamtorch/nn/backup/mamconv2d.txt:133-139).  Here
//   * mam_im2col_kernel writes the patch rows in one pass, K-contiguous, exactly the operand layout
//     the tiled forward reads by TMA (no unfold + transpose copies);
//   * the backward leaves the row gradients TRANSPOSED ([K][M], see mam_bwd_kernel), so that
//     mam_col2im_kernel reads them with unit stride along the image width: every input pixel sums its
//     (up to kH*kW) contributions from coalesced loads and is written once, without atomics.
#pragma once
#include <cuda_runtime.h>

namespace mamb200 {

struct ConvGeom {
    int B, C, H, W, kH, kW, sh, sw, ph, pw, Ho, Wo;
};

constexpr int IM2COL_KPT = 4;   // patch columns per thread held across a row of output pixels

// One CTA per (image, output row): every thread decodes its (up to IM2COL_KPT) patch columns k once and
// then walks the Wo pixels of the row; the writes of a pixel are one contiguous run of K floats, the
// reads of neighbouring pixels overlap and come from L1.
__global__ void __launch_bounds__(256)
mam_im2col_kernel(const float* __restrict__ x, float* __restrict__ rows, ConvGeom g) {
    const int K = g.C * g.kH * g.kW, taps = g.kH * g.kW;
    const int ho = blockIdx.x % g.Ho;
    const long long b = blockIdx.x / g.Ho;
    const float* xb = x + b * (long long)g.C * g.H * g.W;
    float* out = rows + ((b * g.Ho + ho) * (long long)g.Wo) * K;
    const int h0 = ho * g.sh - g.ph;
    for (int kbase = 0; kbase < K; kbase += 256 * IM2COL_KPT) {
        int off[IM2COL_KPT], kw_[IM2COL_KPT];   // offset of (c, h) inside the image (or -1), and kw
#pragma unroll
        for (int j = 0; j < IM2COL_KPT; ++j) {
            const int k = kbase + j * 256 + threadIdx.x;
            off[j] = -1;
            kw_[j] = 0;
            if (k < K) {
                const int c = k / taps, r = k - c * taps;
                const int kh = r / g.kW;
                kw_[j] = r - kh * g.kW;
                const int h = h0 + kh;
                if ((unsigned)h < (unsigned)g.H) off[j] = (c * g.H + h) * g.W;
            }
        }
        for (int wo = 0; wo < g.Wo; ++wo) {
            const int w0 = wo * g.sw - g.pw;
#pragma unroll
            for (int j = 0; j < IM2COL_KPT; ++j) {
                const int k = kbase + j * 256 + threadIdx.x;
                if (k < K) {
                    const int w = w0 + kw_[j];
                    float v = 0.f;
                    if (off[j] >= 0 && (unsigned)w < (unsigned)g.W) v = __ldg(xb + off[j] + w);
                    out[(long long)wo * K + k] = v;
                }
            }
        }
    }
}

// dx[b][c][h][w] = sum over the taps (kh, kw) whose output pixel exists of colsT[(c*kH+kh)*kW+kw][m].
// One CTA per (image, channel, block of `hrows` input rows): its reads of every tap row k are one long
// run of consecutive output pixels m, and threads run along (h, w) so each warp load is contiguous.
template <bool UNIT_STRIDE>
__global__ void __launch_bounds__(256)
mam_col2im_kernel(const float* __restrict__ colsT, float* __restrict__ dx, ConvGeom g, long long M, int hrows) {
    const int hblocks = (g.H + hrows - 1) / hrows;
    const int hb = blockIdx.x % hblocks;
    const long long bc = blockIdx.x / hblocks;      // b * C + c
    const int c = (int)(bc % g.C);
    const long long b = bc / g.C;
    const int h_first = hb * hrows;
    const int nh = min(hrows, g.H - h_first);
    float* dplane = dx + (bc * g.H + h_first) * (long long)g.W;
    for (int i = threadIdx.x; i < nh * g.W; i += 256) {
        const int dh = i / g.W, w = i - dh * g.W;
        const int h = h_first + dh;
        float acc = 0.f;
        for (int kh = 0; kh < g.kH; ++kh) {
            int ho = h + g.ph - kh;
            if (ho < 0) continue;
            if (!UNIT_STRIDE) {
                if (ho % g.sh) continue;
                ho /= g.sh;
            }
            if (ho >= g.Ho) continue;
            for (int kw = 0; kw < g.kW; ++kw) {
                int wo = w + g.pw - kw;
                if (wo < 0) continue;
                if (!UNIT_STRIDE) {
                    if (wo % g.sw) continue;
                    wo /= g.sw;
                }
                if (wo >= g.Wo) continue;
                const long long m = (b * g.Ho + ho) * g.Wo + wo;
                const long long k = ((long long)c * g.kH + kh) * g.kW + kw;
                acc += __ldg(colsT + k * M + m);
            }
        }
        dplane[i] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// Convolution backward without row gradients: dx accumulated where it lives.
//
// The patch-row form above hands every output pixel's K row gradients to the fold kernel through
// memory ([K][M] floats, nine times the size of dx for a 3x3 kernel).  Here a CTA owns `th` consecutive
// output rows of one image and keeps, in shared memory, the part of dx those rows can reach: all C
// channels x ((th-1)*sh + kH) input rows x W columns.  Every selected pair adds its term g*w there
// (shared-memory atomics: different outputs reach the same input pixel) and its term g*x to dW in L2;
// at the end the region is added into dx, four floats per reduction where the rows allow it --
// neighbouring CTAs overlap by kH - sh input rows, so dx is zero-filled first and every CTA adds.
// Per selected k the channel / tap arithmetic comes from a table built once per CTA.
struct ConvDirectEntry {
    int roff;   // (c*RH + kh)*W + kw : offset inside the region, before the pixel's own (row, column) shift
    int goff;   // (c*H + kh)*W + kw  : the same inside the image
    int khkw;   // kh | kw << 16
    int pad;
};
constexpr int CONV_DIRECT_THREADS = 512;
constexpr int CONV_DIRECT_UNROLL = 2;   // outputs in flight per lane

__global__ void __launch_bounds__(CONV_DIRECT_THREADS, 2)
mam_conv_bwd_direct_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ g,
                           const int* __restrict__ argmax, const int* __restrict__ argmin,
                           float* __restrict__ dx, float* __restrict__ dw, ConvGeom cg, long long N, int th,
                           float scale, int vec4) {
    extern __shared__ __align__(16) unsigned char cd_smem[];
    const int K = cg.C * cg.kH * cg.kW, taps = cg.kH * cg.kW;
    const int RH = (th - 1) * cg.sh + cg.kH;
    const int region = cg.C * RH * cg.W;
    float* reg = reinterpret_cast<float*>(cd_smem);
    ConvDirectEntry* tab = reinterpret_cast<ConvDirectEntry*>(cd_smem + (((size_t)region * 4 + 15) & ~(size_t)15));
    const int hblocks = (cg.Ho + th - 1) / th;
    const int ho0 = (blockIdx.x % hblocks) * th;
    const long long b = blockIdx.x / hblocks;
    const int nrows = min(th, cg.Ho - ho0);
    const int h_lo = ho0 * cg.sh - cg.ph;               // image row of region row 0 (may be negative)
    for (int i = threadIdx.x; i < region; i += CONV_DIRECT_THREADS) reg[i] = 0.f;
    for (int k = threadIdx.x; k < K; k += CONV_DIRECT_THREADS) {
        const int c = k / taps, r = k - c * taps;
        const int kh = r / cg.kW, kw = r - kh * cg.kW;
        tab[k] = ConvDirectEntry{(c * RH + kh) * cg.W + kw, (c * cg.H + kh) * cg.W + kw, kh | (kw << 16), 0};
    }
    __syncthreads();
    const float* xb = x + b * (long long)cg.C * cg.H * cg.W;
    const long long m0 = (b * cg.Ho + ho0) * (long long)cg.Wo;
    const float* gt = g + m0 * N;
    const int* r1 = argmax + m0 * N;
    const int* r2 = argmin + m0 * N;
    // a warp takes one output pixel at a time and its lanes walk the pixel's N outputs (one coalesced run)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npix = nrows * cg.Wo;
    for (int p = warp; p < npix; p += CONV_DIRECT_THREADS / 32) {
        const int hl = p / cg.Wo, wo = p - hl * cg.Wo;
        const int hs = hl * cg.sh;                      // region row of the patch's first row
        const int w0 = wo * cg.sw - cg.pw;              // image column of the patch's first column
        const int rshift = hs * cg.W + w0;              // the pixel's shift inside the region ...
        const int gshift = (h_lo + hs) * cg.W + w0;     // ... and inside the image
        const long long row = (long long)p * N;
        // CONV_DIRECT_UNROLL outputs per lane at a time, in three phases -- the streamed reads, the four
        // gathers per output, the additions -- so that the loads of a phase are in flight together
        // (atomics in between would keep the compiler from hoisting them)
        constexpr int U = CONV_DIRECT_UNROLL;
        const int Ni = (int)N;   // N * K < 2^31 (checked by the host): 32-bit offsets into w / dw
        for (int nb = 0; nb < Ni; nb += 32 * U) {
            float gv[U];
            int ks[2 * U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int n = nb + u * 32 + lane;
                gv[u] = 0.f;
                ks[2 * u] = -1;
                ks[2 * u + 1] = -1;
                if (n < Ni) {
                    gv[u] = __fmul_rn(gt[row + n], scale);
                    ks[2 * u] = r1[row + n];
                    ks[2 * u + 1] = r2[row + n];
                }
            }
            int ra[2 * U];          // index inside the region, -1 = nothing to add
            int wi[2 * U];
            float wv[2 * U], xv[2 * U];
#pragma unroll
            for (int j = 0; j < 2 * U; ++j) {
                const int k = ks[j];
                const int n = nb + (j >> 1) * 32 + lane;
                ra[j] = -1;
                wi[j] = 0;
                wv[j] = 0.f;
                xv[j] = 0.f;
                // an index outside [0,K) cannot come from the forward; skip it rather than fault
                if ((unsigned)k < (unsigned)K) {
                    const ConvDirectEntry e = tab[k];
                    const int kh = e.khkw & 0xffff, kw = e.khkw >> 16;
                    const int h = h_lo + hs + kh, ww = w0 + kw;
                    // a selected padding position multiplied a zero: it has no pixel to send a gradient to
                    if ((unsigned)h < (unsigned)cg.H && (unsigned)ww < (unsigned)cg.W) {
                        ra[j] = e.roff + rshift;
                        wi[j] = n * K + k;
                        wv[j] = w[wi[j]];
                        xv[j] = xb[e.goff + gshift];
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 2 * U; ++j) {
                if (ra[j] >= 0) {
                    atomicAdd(&reg[ra[j]], __fmul_rn(wv[j], gv[j >> 1]));
                    atomicAdd(&dw[wi[j]], __fmul_rn(xv[j], gv[j >> 1]));
                }
            }
        }
    }
    __syncthreads();
    // region -> dx: rows of the region that lie inside the image, all channels
    float* dxb = dx + b * (long long)cg.C * cg.H * cg.W;
    const int rh_first = max(0, -h_lo), rh_last = min(RH, cg.H - h_lo);   // [first, last)
    const int live = rh_last - rh_first;
    if (live <= 0) return;
    if (vec4) {   // W % 4 == 0 and dx 16-byte aligned: every row of the region starts on a 16-byte boundary
        const int w4 = cg.W >> 2, per_c = live * w4;
        for (int i = threadIdx.x; i < cg.C * per_c; i += CONV_DIRECT_THREADS) {
            const int c = i / per_c, r = i - c * per_c;
            const int rh = rh_first + r / w4, q = r - (r / w4) * w4;
            const float4 v = *reinterpret_cast<const float4*>(reg + (c * RH + rh) * cg.W + q * 4);
            if (v.x == 0.f && v.y == 0.f && v.z == 0.f && v.w == 0.f) continue;
            float* dst = dxb + ((long long)c * cg.H + (h_lo + rh)) * cg.W + q * 4;
            asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z),
                         "f"(v.w)
                         : "memory");
        }
    } else {
        const int per_c = live * cg.W;
        for (int i = threadIdx.x; i < cg.C * per_c; i += CONV_DIRECT_THREADS) {
            const int c = i / per_c, r = i - c * per_c;
            const int rh = rh_first + r / cg.W, ww = r - (r / cg.W) * cg.W;
            const float v = reg[(c * RH + rh) * cg.W + ww];
            if (v != 0.f) atomicAdd(dxb + ((long long)c * cg.H + (h_lo + rh)) * cg.W + ww, v);
        }
    }
}

}  // namespace mamb200
