// Depthwise, non-causal ("same" padding) conv1d over the sequence followed by SiLU, channels-last, forward and
// backward - the front end of BiMamba2 (src/ssd/modules.py:164-167: conv1d on the transposed tensor, transposed
// back, then the activation).  Working channels-last on (batch, seqlen, channels) removes both transposes and hands
// x / B / C to the scan as strided views of one contiguous tensor, which its TMA maps read in place.
//
//   pre[b,l,c] = bias[c] + sum_k w[c,k] x[b, l + k - K/2, c]      (zero outside 0 <= l < L),   out = silu(pre)
//   dpre = dout silu'(pre);  dx[b,l,c] = sum_k w[c,k] dpre[b, l - k + K/2, c];
//   dw[c,k] = sum_{b,l} dpre[b,l,c] x[b, l + k - K/2, c];  dbias[c] = sum_{b,l} dpre[b,l,c]
//
// HBM-bound: every thread owns 8 adjacent channels (one 16-byte access per row) and walks a run of rows.  Two forms:
// the general one (any dtype, any K <= 8) re-reads the K neighbouring rows of a window from L1 / L2; 16-bit
// activations with K = 3, 5, 7 use the rolling-window kernel further down.  The backward recomputes pre instead of saving it and runs
// as three light kernels (dpre; weight / bias gradient partials; dx) rather than one register-heavy one.  Weight
// and bias gradients: per-thread accumulators over the thread's rows, one partial row per (batch, row block) in the
// workspace, summed in a fixed order by conv_bwd_reduce - no float atomics.  Width K <= 8.
#pragma once
#include "norm_kernels.cuh"

namespace bissd {
namespace conv {

constexpr int kMaxK = 8;
constexpr int kRows = 64;                        // rows per thread run (and per partial row of dw / dbias)
constexpr int kRowsDw = 256;                     // the same for the rolling-window dw pass: fewer partial rows to reduce

struct ConvDims {
    int batch, seqlen, channels, width;
    long long xsb, xsl;                          // x and dx: batch and row strides in elements; channel stride 1
    long long osb, osl;                          // out, dout and dpre
    int has_bias;
};

using norm::load8;
using norm::store8;
using norm::sigmoidn;
using norm::unpack8n;

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

// ---------------------------------------------------------------------------------------------------------
// Odd width K, 16-bit activations: the same four passes with a rolling window.  A thread keeps the K - 1 previous rows
// of its 8 channels in registers (packed, as loaded) and fetches each row of the source once, U rows per round with
// all U loads in flight before the first is used - the row-at-a-time kernels above have one new row in flight per
// thread and are bound by load latency, not by HBM.  MODE 0: out = silu(pre).  MODE 1: dpre = dout silu'(pre).
// MODE 2: partial dw / dbias from x (window) and dpre.  MODE 3: dx from dpre (same window, weights reversed).
//   src: x (MODE 0-2) or dpre (MODE 3);  aux: dout (MODE 1) or dpre (MODE 2);  dst: out, dpre, -, dx.
template <class T>
__device__ __forceinline__ uint4 conv_row(const void *base, long long rowoff, int l, int seqlen) {
    return (l >= 0 && l < seqlen) ? __ldg(reinterpret_cast<const uint4 *>(static_cast<const T *>(base) + rowoff)) : make_uint4(0u, 0u, 0u, 0u);
}

template <class T, class W, int MODE, int K>
__global__ void __launch_bounds__(128, 3) dwconv_win(ConvDims d, const void *src, const void *weight, const void *bias,
                                                     const void *aux, void *dst, float *part) {
    constexpr int U = 4, PAD = K / 2;                            // the window covers rows l - PAD .. l + PAD
    constexpr int ROWS = MODE == 2 ? kRowsDw : kRows;
    const int c0 = (blockIdx.x * 128 + threadIdx.x) * 8;
    if (c0 >= d.channels) return;
    const int b = blockIdx.z, l0 = blockIdx.y * ROWS, l1 = min(d.seqlen, l0 + ROWS);
    const long long ssb = MODE == 3 ? d.osb : d.xsb, ssl = MODE == 3 ? d.osl : d.xsl;      // source strides
    const long long dsb = MODE == 3 ? d.xsb : d.osb, dsl = MODE == 3 ? d.xsl : d.osl;      // destination strides
    float w[K][8], bv[8];                                        // w[o]: weight of window slot o; MODE 2: the dw accumulators
#pragma unroll
    for (int o = 0; o < K; ++o)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long wi = (long long)(c0 + j) * K + (MODE == 3 ? K - 1 - o : o);
            if (MODE == 2) w[o][j] = 0.f;
            else if constexpr (sizeof(W) == 4) w[o][j] = static_cast<const float *>(weight)[wi];
            else w[o][j] = static_cast<float>(static_cast<const W *>(weight)[wi]);
        }
#pragma unroll
    for (int j = 0; j < 8; ++j) bv[j] = 0.f;                     // MODE 2: the dbias accumulator
    if (MODE <= 1 && d.has_bias) load8<W>(bias, c0, bv);
    uint4 win[K - 1];
#pragma unroll
    for (int o = 0; o < K - 1; ++o) win[o] = conv_row<T>(src, b * ssb + (long long)(l0 - PAD + o) * ssl + c0, l0 - PAD + o, d.seqlen);
    for (int lb = l0; lb < l1; lb += U) {
        uint4 nw[U], au[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int ln = lb + u + PAD;
            nw[u] = conv_row<T>(src, b * ssb + (long long)ln * ssl + c0, ln, d.seqlen);
            if (MODE == 1 || MODE == 2) au[u] = conv_row<T>(aux, b * d.osb + (long long)(lb + u) * d.osl + c0, lb + u, l1);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int l = lb + u;
            if (l < l1) {
                float t[8];
                if (MODE == 2) {
                    float g[8];
                    unpack8n<T>(au[u], g);
#pragma unroll
                    for (int o = 0; o < K; ++o) {
                        unpack8n<T>(o < K - 1 ? win[o < K - 1 ? o : 0] : nw[u], t);
#pragma unroll
                        for (int j = 0; j < 8; ++j) w[o][j] = fmaf(g[j], t[j], w[o][j]);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) bv[j] += g[j];
                } else {
                    float acc[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] = bv[j];
#pragma unroll
                    for (int o = 0; o < K; ++o) {
                        unpack8n<T>(o < K - 1 ? win[o < K - 1 ? o : 0] : nw[u], t);
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[j] = fmaf(w[o][j], t[j], acc[j]);
                    }
                    if (MODE == 0) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[j] *= sigmoidn(acc[j]);
                    } else if (MODE == 1) {
                        unpack8n<T>(au[u], t);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float sg = sigmoidn(acc[j]);
                            acc[j] = t[j] * sg * (1.f + acc[j] * (1.f - sg));
                        }
                    }
                    store8<T>(dst, b * dsb + (long long)l * dsl + c0, acc);
                }
            }
#pragma unroll
            for (int o = 0; o + 1 < K - 1; ++o) win[o] = win[o + 1];
            win[K - 2] = nw[u];
        }
    }
    if (MODE == 2) {
        float *p = part + ((long long)(b * gridDim.y + blockIdx.y) * d.channels + c0) * (kMaxK + 1);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int k = 0; k < K; ++k) p[j * (kMaxK + 1) + k] = w[k][j];
            p[j * (kMaxK + 1) + kMaxK] = bv[j];
        }
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
