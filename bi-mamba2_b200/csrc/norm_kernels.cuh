// Gated RMSNorm, forward and backward, for the layer that follows the scan in BiMamba2
// (takes over _layer_norm_fwd_1pass_kernel / _layer_norm_bwd_kernel of src/ssd/bi/layernorm_gated.py:45-105, :155-268
// in their RMS form; the arithmetic follows rms_norm_ref, :18-41):
//   norm_before_gate:  y = x rstd w;  out = y silu(z)
//   otherwise:         u = x silu(z);  out = u rstd w
// (no bias: the reference's RMSNorm registers none, src/ssd/bi/layernorm_gated.py:424)
//   rstd = rsqrt(mean over the group of (x or u)^2 + eps), one value per (row, group).
// HBM-bound element-wise work with two small reductions per row, so: one warp per row, 16-byte accesses, the row kept
// in registers between the statistics pass and the output pass (hidden <= 4096), statistics by warp shuffles only.
// Groups must be whole multiples of 256 channels (or the whole row), so that the 32 x 8 channels a
// warp touches in one step always belong to one group.
// Weight gradient: per-lane accumulators over the rows of a warp, combined over the warps of a CTA in a fixed
// order through shared memory, one partial row per CTA in the workspace, summed by norm_bwd_reduce - no float atomics.
#pragma once
#include "common.cuh"

namespace bissd {
namespace norm {

constexpr int kThreads = 256, kWarps = 8;

struct NormDims {
    long long rows;
    int hidden, group, ngroups;                  // group = channels per statistics group
    long long sx, sz, so;                        // row strides (elements) of x (and dx), z (and dz), out (and dout)
    int has_z, norm_before_gate;
    float eps;
};

template <class T> __device__ __forceinline__ void unpack8n(uint4 u, float (&v)[8]);
template <> __device__ __forceinline__ void unpack8n<__nv_bfloat16>(uint4 u, float (&v)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
template <> __device__ __forceinline__ void unpack8n<__half>(uint4 u, float (&v)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
template <> __device__ __forceinline__ void unpack8n<float>(uint4, float (&)[8]) {}
template <class T> __device__ __forceinline__ uint4 pack8n(const float (&v)[8]);
template <> __device__ __forceinline__ uint4 pack8n<__nv_bfloat16>(const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t *>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ uint4 pack8n<__half>(const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 p = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t *>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// 8 consecutive channels of one row, as fp32
template <class T> __device__ __forceinline__ void load8(const void *base, long long off, float (&v)[8]) {
    if constexpr (sizeof(T) == 4) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(base) + off));
        const float4 b = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(base) + off) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        unpack8n<T>(__ldg(reinterpret_cast<const uint4 *>(static_cast<const T *>(base) + off)), v);
    }
}
template <class T> __device__ __forceinline__ void store8(void *base, long long off, const float (&v)[8]) {
    if constexpr (sizeof(T) == 4) {
        float4 *p = reinterpret_cast<float4 *>(static_cast<float *>(base) + off);
        p[0] = make_float4(v[0], v[1], v[2], v[3]);
        p[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        *reinterpret_cast<uint4 *>(static_cast<T *>(base) + off) = pack8n<T>(v);
    }
}
template <class T> __device__ __forceinline__ uint4 ldq(const void *base, long long off) {   // 8 packed 16-bit values
    return __ldg(reinterpret_cast<const uint4 *>(static_cast<const T *>(base) + off));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float sigmoidn(float v) { return __fdividef(1.f, 1.f + __expf(-v)); }

// grid: any; each warp walks rows  blockIdx.x * kWarps + warp,  + gridDim.x * kWarps, ...
// NS: register-resident steps of 256 channels (hidden <= NS * 256).  W: dtype of the weight (fp32 or as x).
template <class T, class W, int NS>
__global__ void __launch_bounds__(kThreads) rmsnorm_gated_fwd(NormDims d, const void *x, const void *z, const void *weight,
                                                              void *out, float *rstd) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsteps = d.hidden / 256, spg = d.group / 256;          // steps per statistics group
    for (long long row = (long long)blockIdx.x * kWarps + warp; row < d.rows; row += (long long)gridDim.x * kWarps) {
        float xv[NS][8], ss[NS], rs[NS];
        if constexpr (sizeof(T) == 2) {
            // all loads of the row are issued before the first is used (a load per step followed by its use costs one
            // memory round trip per step)
            const bool gate_first = d.has_z && !d.norm_before_gate;
            uint4 xq[NS], zq[NS];
#pragma unroll
            for (int k = 0; k < NS; ++k) {
                const long long c0 = k * 256 + lane * 8;
                xq[k] = k < nsteps ? ldq<T>(x, row * d.sx + c0) : make_uint4(0u, 0u, 0u, 0u);
                zq[k] = (k < nsteps && gate_first) ? ldq<T>(z, row * d.sz + c0) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int k = 0; k < NS; ++k) {
                ss[k] = 0.f;
                rs[k] = 0.f;
                unpack8n<T>(xq[k], xv[k]);
                if (gate_first) {
                    float zz[8];
                    unpack8n<T>(zq[k], zz);
#pragma unroll
                    for (int j = 0; j < 8; ++j) xv[k][j] *= zz[j] * sigmoidn(zz[j]);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) ss[k] = fmaf(xv[k][j], xv[k][j], ss[k]);
            }
        } else
#pragma unroll
        for (int k = 0; k < NS; ++k) {
            ss[k] = 0.f;
            rs[k] = 0.f;
            if (k < nsteps) {
                const int c0 = k * 256 + lane * 8;
                load8<T>(x, row * d.sx + c0, xv[k]);
                if (d.has_z && !d.norm_before_gate) {
                    float zz[8];
                    load8<T>(z, row * d.sz + c0, zz);
#pragma unroll
                    for (int j = 0; j < 8; ++j) xv[k][j] *= zz[j] * sigmoidn(zz[j]);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) ss[k] = fmaf(xv[k][j], xv[k][j], ss[k]);
            }
        }
        for (int g = 0; g < d.ngroups; ++g) {
            float gs = 0.f;
#pragma unroll
            for (int k = 0; k < NS; ++k) gs += (k / spg == g) ? ss[k] : 0.f;
            const float r = rsqrtf(warp_sum(gs) / (float)d.group + d.eps);
            if (lane == 0) rstd[row * d.ngroups + g] = r;
#pragma unroll
            for (int k = 0; k < NS; ++k) rs[k] = (k / spg == g) ? r : rs[k];
        }
#pragma unroll
        for (int k = 0; k < NS; ++k) {
            if (k < nsteps) {
                const int c0 = k * 256 + lane * 8;
                float wv[8], o[8];
                load8<W>(weight, c0, wv);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = xv[k][j] * rs[k] * wv[j];
                if (d.has_z && d.norm_before_gate) {
                    float zz[8];
                    load8<T>(z, row * d.sz + c0, zz);
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] *= zz[j] * sigmoidn(zz[j]);
                }
                store8<T>(out, row * d.so + c0, o);
            }
        }
    }
}

// Backward.  dw_part: [gridDim.x][hidden] fp32, one partial row per CTA.
// dynamic shared memory: kWarps * hidden floats - every warp accumulates its rows' weight gradient in a row of its own
// (registers would cost 8 * NS per thread and halve the occupancy of a kernel that lives on memory latency).
//   xhat = u rstd,  dy = dout (silu(z) if the gate follows the norm),  du = rstd (dy w - xhat mean_group(dy w xhat))
//   gate after the norm:  dx = du,  dz = dout (xhat w) silu'(z);   gate before:  dx = du silu(z),  dz = du x silu'(z)
//   dw = sum over rows of dy xhat
template <class T, class W, int NS>
__global__ void __launch_bounds__(kThreads, 2) rmsnorm_gated_bwd(NormDims d, const void *x, const void *z, const void *weight,
                                                              const void *dout, const float *rstd, void *dx, void *dz,
                                                              float *dw_part) {
    extern __shared__ float red[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsteps = d.hidden / 256, spg = d.group / 256;
    float *mine = red + warp * d.hidden;
    for (int cidx = lane * 8; cidx < d.hidden; cidx += 256) {
        *reinterpret_cast<float4 *>(mine + cidx) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4 *>(mine + cidx + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (long long row = (long long)blockIdx.x * kWarps + warp; row < d.rows; row += (long long)gridDim.x * kWarps) {
        // pass 1: per step, the sum of (dy w) xhat; per group its mean
        float dot[NS], mean[NS];
#pragma unroll
        for (int h0 = 0; h0 < NS; h0 += 4) {
        // four steps at a time: their twelve loads are issued before the first is used
        uint4 xq[4], gq[4], zq[4];
        if constexpr (sizeof(T) == 2) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const long long c0 = (h0 + q) * 256 + lane * 8;
                const bool on = h0 + q < nsteps;
                xq[q] = on ? ldq<T>(x, row * d.sx + c0) : make_uint4(0u, 0u, 0u, 0u);
                gq[q] = on ? ldq<T>(dout, row * d.so + c0) : make_uint4(0u, 0u, 0u, 0u);
                zq[q] = (on && d.has_z) ? ldq<T>(z, row * d.sz + c0) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int k = h0; k < h0 + 4; ++k) {
            dot[k] = 0.f;
            mean[k] = 0.f;
            if (k < nsteps) {
                const int c0 = k * 256 + lane * 8;
                const float r = rstd[row * d.ngroups + k / spg];
                float xv[8], gv[8], wv[8], zz[8];
                if constexpr (sizeof(T) == 2) {
                    unpack8n<T>(xq[k - h0], xv);
                    unpack8n<T>(gq[k - h0], gv);
                    unpack8n<T>(zq[k - h0], zz);
                } else {
                    load8<T>(x, row * d.sx + c0, xv);
                    load8<T>(dout, row * d.so + c0, gv);
                    if (d.has_z) load8<T>(z, row * d.sz + c0, zz);
                }
                load8<W>(weight, c0, wv);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float u = xv[j], dy = gv[j];
                    if (d.has_z) {
                        const float sl = zz[j] * sigmoidn(zz[j]);
                        if (d.norm_before_gate) dy *= sl;
                        else u *= sl;
                    }
                    dot[k] = fmaf(dy * wv[j], u * r, dot[k]);
                }
            }
        }
        }
        for (int g = 0; g < d.ngroups; ++g) {
            float gs = 0.f;
#pragma unroll
            for (int k = 0; k < NS; ++k) gs += (k / spg == g) ? dot[k] : 0.f;
            const float m = warp_sum(gs) / (float)d.group;
#pragma unroll
            for (int k = 0; k < NS; ++k) mean[k] = (k / spg == g) ? m : mean[k];
        }
        // pass 2: gradients (the operands come from L1 / L2 the second time), again four steps at a time
#pragma unroll
        for (int h0 = 0; h0 < NS; h0 += 4) {
        uint4 xq[4], gq[4], zq[4];
        if constexpr (sizeof(T) == 2) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const long long c0 = (h0 + q) * 256 + lane * 8;
                const bool on = h0 + q < nsteps;
                xq[q] = on ? ldq<T>(x, row * d.sx + c0) : make_uint4(0u, 0u, 0u, 0u);
                gq[q] = on ? ldq<T>(dout, row * d.so + c0) : make_uint4(0u, 0u, 0u, 0u);
                zq[q] = (on && d.has_z) ? ldq<T>(z, row * d.sz + c0) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int k = h0; k < h0 + 4; ++k) {
            if (k < nsteps) {
                const int c0 = k * 256 + lane * 8;
                const float r = rstd[row * d.ngroups + k / spg];
                float xv[8], gv[8], wv[8], zz[8], ox[8], oz[8], dwv[8];
                if constexpr (sizeof(T) == 2) {
                    unpack8n<T>(xq[k - h0], xv);
                    unpack8n<T>(gq[k - h0], gv);
                    unpack8n<T>(zq[k - h0], zz);
                } else {
                    load8<T>(x, row * d.sx + c0, xv);
                    load8<T>(dout, row * d.so + c0, gv);
                    if (d.has_z) load8<T>(z, row * d.sz + c0, zz);
                }
                load8<W>(weight, c0, wv);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float sl = 1.f, dsl = 0.f;
                    if (d.has_z) {
                        const float sg = sigmoidn(zz[j]);
                        sl = zz[j] * sg;
                        dsl = sg * (1.f + zz[j] * (1.f - sg));
                    }
                    const bool after = d.has_z && d.norm_before_gate, before = d.has_z && !d.norm_before_gate;
                    const float u = before ? xv[j] * sl : xv[j];
                    const float xhat = u * r;
                    const float dy = after ? gv[j] * sl : gv[j];
                    const float du = r * (dy * wv[j] - xhat * mean[k]);
                    ox[j] = before ? du * sl : du;
                    oz[j] = after ? gv[j] * xhat * wv[j] * dsl : (before ? du * xv[j] * dsl : 0.f);
                    dwv[j] = dy * xhat;
                }
                {
                    float4 *acc4 = reinterpret_cast<float4 *>(mine + c0);
                    float4 a0 = acc4[0], a1 = acc4[1];
                    a0.x += dwv[0]; a0.y += dwv[1]; a0.z += dwv[2]; a0.w += dwv[3];
                    a1.x += dwv[4]; a1.y += dwv[5]; a1.z += dwv[6]; a1.w += dwv[7];
                    acc4[0] = a0;
                    acc4[1] = a1;
                }
                store8<T>(dx, row * d.sx + c0, ox);
                if (d.has_z) store8<T>(dz, row * d.sz + c0, oz);
            }
        }
        }
    }
    // the eight warps' rows are added in warp order and written as this CTA's partial row
    __syncthreads();
    for (int cidx = threadIdx.x; cidx < d.hidden; cidx += kThreads) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) v += red[w * d.hidden + cidx];
        dw_part[(long long)blockIdx.x * d.hidden + cidx] = v;
    }
}

// dw[c] = sum over the partial rows, in row order.  grid ceil(hidden / 256).
template <class W>
__global__ void __launch_bounds__(kThreads) norm_bwd_reduce(const float *dw_part, int nparts, int hidden, void *dw) {
    const int cidx = blockIdx.x * kThreads + threadIdx.x;
    if (cidx >= hidden) return;
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
    int p = 0;
    for (; p + 3 < nparts; p += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) s4[u] += dw_part[(long long)(p + u) * hidden + cidx];
    }
    for (; p < nparts; ++p) s4[0] += dw_part[(long long)p * hidden + cidx];
    const float v = (s4[0] + s4[1]) + (s4[2] + s4[3]);
    if constexpr (sizeof(W) == 4) static_cast<float *>(dw)[cidx] = v;
    else static_cast<W *>(dw)[cidx] = static_cast<W>(v);
}

}  // namespace norm
}  // namespace bissd
