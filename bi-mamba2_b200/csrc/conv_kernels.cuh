// Depthwise, non-causal ("same" padding) conv1d over the sequence followed by SiLU, channels-last, forward and
// backward - the front end of BiMamba2 (src/ssd/modules.py:164-167: conv1d on the transposed tensor, transposed
// back, then the activation).  Working channels-last on (batch, seqlen, channels) removes both transposes and hands
// x / B / C to the scan as strided views of one contiguous tensor, which its TMA maps read in place.
//
//   pre[b,l,c] = bias[c] + sum_k w[c,k] x[b, l + k - K/2, c]      (zero outside 0 <= l < L),   out = silu(pre)
//   dpre = dout silu'(pre);  dx[b,l,c] = sum_k w[c,k] dpre[b, l - k + K/2, c];
//   dw[c,k] = sum_{b,l} dpre[b,l,c] x[b, l + k - K/2, c];  dbias[c] = sum_{b,l} dpre[b,l,c]
//
// HBM-bound: every thread owns 8 adjacent channels (one 16-byte access per row) and walks a run of rows; the K
// neighbouring rows of a window are re-read from L1 / L2.  The backward recomputes pre instead of saving it and runs
// as three light kernels (dpre; weight / bias gradient partials; dx) rather than one register-heavy one.  Weight
// and bias gradients: per-thread accumulators over the thread's rows, one partial row per (batch, row block) in the
// workspace, summed in a fixed order by conv_bwd_reduce - no float atomics.  Width K <= 8.
#pragma once
#include "norm_kernels.cuh"

namespace bissd {
namespace conv {

constexpr int kMaxK = 8;
constexpr int kRows = 64;                        // rows per thread run (and per partial row of dw / dbias)

struct ConvDims {
    int batch, seqlen, channels, width;
    long long xsb, xsl;                          // x and dx: batch and row strides in elements; channel stride 1
    long long osb, osl;                          // out, dout and dpre
    int has_bias;
};

using norm::load8;
using norm::store8;
using norm::sigmoidn;

// grid (channels / 8 / 128 rounded up, ceil(L / kRows), batch); block 128: thread = 8 channels, kRows rows.
template <class T, class W>
__global__ void __launch_bounds__(128, 4) dwconv_silu_fwd(ConvDims d, const void *x, const void *weight, const void *bias,
                                                       void *out) {
    const int c0 = (blockIdx.x * 128 + threadIdx.x) * 8;
    if (c0 >= d.channels) return;
    const int b = blockIdx.z, l0 = blockIdx.y * kRows, l1 = min(d.seqlen, l0 + kRows), pad = d.width / 2;
    float w[kMaxK][8], bv[8];
#pragma unroll
    for (int k = 0; k < kMaxK; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j)
            w[k][j] = (k < d.width) ? (sizeof(W) == 4 ? static_cast<const float *>(weight)[(long long)(c0 + j) * d.width + k]
                                                       : static_cast<float>(static_cast<const W *>(weight)[(long long)(c0 + j) * d.width + k]))
                                    : 0.f;
    if (d.has_bias) load8<W>(bias, c0, bv);
    else
#pragma unroll
        for (int j = 0; j < 8; ++j) bv[j] = 0.f;
    for (int l = l0; l < l1; ++l) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = bv[j];
#pragma unroll
        for (int k = 0; k < kMaxK; ++k) {
            const int ls = l + k - pad;
            if (k < d.width && ls >= 0 && ls < d.seqlen) {
                float xv[8];
                load8<T>(x, b * d.xsb + ls * d.xsl + c0, xv);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = fmaf(w[k][j], xv[j], acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= sigmoidn(acc[j]);
        store8<T>(out, b * d.osb + l * d.osl + c0, acc);
    }
}

// Backward, first pass: dpre = dout silu'(pre), pre recomputed, stored in the activation dtype.
template <class T, class W>
__global__ void __launch_bounds__(128, 4) dwconv_silu_bwd_pre(ConvDims d, const void *x, const void *weight, const void *bias,
                                                              const void *dout, void *dpre) {
    const int c0 = (blockIdx.x * 128 + threadIdx.x) * 8;
    if (c0 >= d.channels) return;
    const int b = blockIdx.z, l0 = blockIdx.y * kRows, l1 = min(d.seqlen, l0 + kRows), pad = d.width / 2;
    float w[kMaxK][8], bv[8];
#pragma unroll
    for (int k = 0; k < kMaxK; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j)
            w[k][j] = (k < d.width) ? (sizeof(W) == 4 ? static_cast<const float *>(weight)[(long long)(c0 + j) * d.width + k]
                                                       : static_cast<float>(static_cast<const W *>(weight)[(long long)(c0 + j) * d.width + k]))
                                    : 0.f;
    if (d.has_bias) load8<W>(bias, c0, bv);
    else
#pragma unroll
        for (int j = 0; j < 8; ++j) bv[j] = 0.f;
    for (int l = l0; l < l1; ++l) {
        float acc[8], g[8];
        load8<T>(dout, b * d.osb + l * d.osl + c0, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = bv[j];
#pragma unroll
        for (int k = 0; k < kMaxK; ++k) {
            const int ls = l + k - pad;
            if (k < d.width && ls >= 0 && ls < d.seqlen) {
                float xv[8];
                load8<T>(x, b * d.xsb + ls * d.xsl + c0, xv);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = fmaf(w[k][j], xv[j], acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float sg = sigmoidn(acc[j]);
            g[j] *= sg * (1.f + acc[j] * (1.f - sg));
        }
        store8<T>(dpre, b * d.osb + l * d.osl + c0, g);
    }
}

// Backward, weight / bias gradients from dpre and x.
// part: [batch * row blocks][channels][kMaxK + 1] fp32 (slot kMaxK holds the bias gradient).
template <class T>
__global__ void __launch_bounds__(128, 4) dwconv_silu_bwd_dw(ConvDims d, const void *x, const void *dpre, float *part) {
    const int c0 = (blockIdx.x * 128 + threadIdx.x) * 8;
    if (c0 >= d.channels) return;
    const int b = blockIdx.z, l0 = blockIdx.y * kRows, l1 = min(d.seqlen, l0 + kRows), pad = d.width / 2;
    float dw[kMaxK][8], db[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        db[j] = 0.f;
#pragma unroll
        for (int k = 0; k < kMaxK; ++k) dw[k][j] = 0.f;
    }
    for (int l = l0; l < l1; ++l) {
        float g[8];
        load8<T>(dpre, b * d.osb + l * d.osl + c0, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) db[j] += g[j];
#pragma unroll
        for (int k = 0; k < kMaxK; ++k) {
            const int ls = l + k - pad;
            if (k < d.width && ls >= 0 && ls < d.seqlen) {
                float xv[8];
                load8<T>(x, b * d.xsb + ls * d.xsl + c0, xv);
#pragma unroll
                for (int j = 0; j < 8; ++j) dw[k][j] = fmaf(g[j], xv[j], dw[k][j]);
            }
        }
    }
    float *p = part + ((long long)(b * gridDim.y + blockIdx.y) * d.channels + c0) * (kMaxK + 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int k = 0; k < kMaxK; ++k) p[j * (kMaxK + 1) + k] = dw[k][j];
        p[j * (kMaxK + 1) + kMaxK] = db[j];
    }
}

// Backward, second pass: dx = correlation of dpre with the weights.  Same grid as the forward.
template <class T, class W>
__global__ void __launch_bounds__(128, 4) dwconv_silu_bwd_dx(ConvDims d, const void *dpre, const void *weight, void *dx) {
    const int c0 = (blockIdx.x * 128 + threadIdx.x) * 8;
    if (c0 >= d.channels) return;
    const int b = blockIdx.z, l0 = blockIdx.y * kRows, l1 = min(d.seqlen, l0 + kRows), pad = d.width / 2;
    float w[kMaxK][8];
#pragma unroll
    for (int k = 0; k < kMaxK; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j)
            w[k][j] = (k < d.width) ? (sizeof(W) == 4 ? static_cast<const float *>(weight)[(long long)(c0 + j) * d.width + k]
                                                       : static_cast<float>(static_cast<const W *>(weight)[(long long)(c0 + j) * d.width + k]))
                                    : 0.f;
    for (int l = l0; l < l1; ++l) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
        for (int k = 0; k < kMaxK; ++k) {
            const int ls = l - k + pad;
            if (k < d.width && ls >= 0 && ls < d.seqlen) {
                float gv[8];
                load8<T>(dpre, b * d.osb + ls * d.osl + c0, gv);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = fmaf(w[k][j], gv[j], acc[j]);
            }
        }
        store8<T>(dx, b * d.xsb + l * d.xsl + c0, acc);
    }
}

// dweight[c][k] and dbias[c] = sums of the partial rows, in row order.  One thread per (channel, k <= K).
template <class W>
__global__ void __launch_bounds__(256) conv_bwd_reduce(const float *part, int nparts, int channels, int width, void *dweight,
                                                       void *dbias) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)channels * (kMaxK + 1)) return;
    const int c = (int)(i / (kMaxK + 1)), k = (int)(i % (kMaxK + 1));
    if (k >= width && k != kMaxK) return;
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
    int p = 0;
    for (; p + 3 < nparts; p += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) s4[u] += part[((long long)(p + u) * channels + c) * (kMaxK + 1) + k];
    }
    for (; p < nparts; ++p) s4[0] += part[((long long)p * channels + c) * (kMaxK + 1) + k];
    const float v = (s4[0] + s4[1]) + (s4[2] + s4[3]);
    if (k == kMaxK) {
        if (dbias) {
            if constexpr (sizeof(W) == 4) static_cast<float *>(dbias)[c] = v;
            else static_cast<W *>(dbias)[c] = static_cast<W>(v);
        }
    } else {
        if constexpr (sizeof(W) == 4) static_cast<float *>(dweight)[(long long)c * width + k] = v;
        else static_cast<W *>(dweight)[(long long)c * width + k] = static_cast<W>(v);
    }
}

}  // namespace conv
}  // namespace bissd
