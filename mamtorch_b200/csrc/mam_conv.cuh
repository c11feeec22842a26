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

}  // namespace mamb200
