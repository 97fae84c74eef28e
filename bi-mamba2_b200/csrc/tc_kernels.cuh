// Tensor-core (tcgen05 / TMEM) kernels for the contractions of the bidirectional SSD chunk scan, 16-bit inputs.
//
// Each kernel maps one or more K-segments onto tc::umma_gemm: the operand functors read global memory in
// 16-byte pieces, apply the decay / mask / gate factors in registers and hand back 8 packed 16-bit values that the
// engine places into the swizzled shared-memory tiles the tensor core reads.  Accumulators live in TMEM and are
// read back one 32-column strip per thread-row for the epilogue.
//
// Requirements checked on the host (tc_eligible): 16-bit x/B/C, headdim % 8 == 0, dstate % 8 == 0, chunk % 8 == 0,
// headdim <= 256, dstate <= 256, 16-byte aligned pointers and strides.
//
// Notation as in simt_kernels.cuh.
#pragma once
#include "tc_engine.cuh"

namespace bissd {
namespace tc {

__host__ __device__ inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
__host__ __device__ inline int b_stage_bytes(int n_tile) { return ((n_tile + 63) / 64) * 8192; }
// dynamic shared memory of a kernel with B tiles of n_tile rows and `floats` table entries
inline size_t smem_bytes(int n_tile, int floats) { return 1024 + 2 * kAStageBytes + 2 * b_stage_bytes(n_tile) + floats * 4; }
__host__ __device__ inline uint32_t tmem_cols(int n) { uint32_t c = 32; while ((int)c < n) c <<= 1; return c; }

struct Carve {
    uint8_t *stage;
    float *tab;
};
__device__ __forceinline__ Carve carve(uint8_t *dyn, int n_tile) {
    Carve c;
    c.stage = smem_align1024(dyn);
    c.tab = reinterpret_cast<float *>(c.stage + 2 * kAStageBytes + 2 * b_stage_bytes(n_tile));
    return c;
}

template <class T> __device__ __forceinline__ uint4 ld8v(const View &t, int b, int l, int h, int i) {
    return ldg8(t.ptr, b * t.sb + l * t.sl + h * t.sh + i);
}
template <class T> __device__ __forceinline__ uint4 scale8(uint4 u, float s) {
    float v[8];
    unpack8<T>(u, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= s;
    return pack8<T>(v);
}
// 8 values of g = dout (* silu(z)) along the head dimension
template <class T>
__device__ __forceinline__ uint4 gate8(const Dims &d, const View &dout, const View &z, int b, int l, int h, int p) {
    uint4 u = ld8v<T>(dout, b, l, h, p);
    if (!d.has_z) return u;
    float g[8], zz[8];
    unpack8<T>(u, g);
    unpack8<T>(ld8v<T>(z, b, l, h, p), zz);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= zz[j] * sigmoidf_(zz[j]);
    return pack8<T>(g);
}
template <class T> __device__ __forceinline__ uint4 pack8f(const float *p) {
    float v[8];
    ldg8f(p, v);
    return pack8<T>(v);
}

// ---------------------------------------------------------------------------------------------------------
// CB[b,c,g,l,s] = C[l].B[s].   grid (b*nc*G, ceil(Q/128)); n_tile = round16(Q); tables: none.
// Outputs, each optional: CB (fp32), CBt (fp32, transposed), CB16 / CBt16 (the same two rounded to bf16, for the
// kernels that take the tile by TMA and only use it as a factor of a 16-bit MMA operand), CBs (fp32 in strips of 16
// columns, [Q/16][Q rows][16]: a thread that owns a row reads 64 contiguous bytes per strip, a warp 2 KB).
template <class T>
__global__ void __launch_bounds__(kThreads) bmm_cb(Dims d, View Cm, View Bm, float *CB, float *CBt, __nv_bfloat16 *CB16,
                                                   __nv_bfloat16 *CBt16, float *CBs, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ PipeShared sh;
    const int nt = round_up(d.Q, 16);
    Carve cv = carve(dyn, nt);
    Pipe p;
    const uint32_t ncols = tmem_cols(nt);
    pipe_init(p, &sh, cv.stage, b_stage_bytes(nt), ncols, status);
    const int g = blockIdx.x % d.G, c = (blockIdx.x / d.G) % d.nc, b = blockIdx.x / (d.G * d.nc);
    const int lim = min(d.Q, d.L - c * d.Q);
    const int l0 = blockIdx.y * kTileM;
    auto fa = [&](int r, int k) -> uint4 {
        return (l0 + r < lim && k < d.N) ? ld8v<T>(Cm, b, c * d.Q + l0 + r, g, k) : zero8();
    };
    auto fb = [&](int r, int k) -> uint4 { return (r < lim && k < d.N) ? ld8v<T>(Bm, b, c * d.Q + r, g, k) : zero8(); };
    bool ok = umma_gemm<T, false, false>(p, p.tmem, nt, d.N, 0u, fa, fb);
    ok = ok && umma_drain(p);
    if (ok) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int l = l0 + (warp & 3) * 32 + lane;
        const long long tile = ((long long)(b * d.nc + c) * d.G + g) * d.Q * d.Q;
        for (int c0 = (warp >> 2) * 32; c0 < nt; c0 += 64) {
            float v[32];
            tmem_ld32(tmem_lane_base(p.tmem) + c0, v);
            if (l < d.Q) {
                if (CB) {
                    float *out = CB + tile + (long long)l * d.Q;
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        if (c0 + j < d.Q) *reinterpret_cast<float4 *>(out + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
                if (CBt) {                                              // transposed copy: lanes write consecutive l
                    float *ot = CBt + tile + l;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c0 + j < d.Q) ot[(long long)(c0 + j) * d.Q] = v[j];
                }
                if (CBs) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        if (c0 + j < d.Q)
                            *reinterpret_cast<float4 *>(CBs + tile + (long long)((c0 + j) >> 4) * d.Q * 16 + l * 16 + ((c0 + j) & 15)) =
                                make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
                if (CB16) {
                    __nv_bfloat16 *out = CB16 + tile + (long long)l * d.Q;
#pragma unroll
                    for (int j = 0; j < 32; j += 8)
                        if (c0 + j < d.Q) {
                            const float o[8] = {v[j], v[j + 1], v[j + 2], v[j + 3], v[j + 4], v[j + 5], v[j + 6], v[j + 7]};
                            *reinterpret_cast<uint4 *>(out + c0 + j) = pack8<__nv_bfloat16>(o);
                        }
                }
                if (CBt16) {
                    __nv_bfloat16 *ot = CBt16 + tile + l;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c0 + j < d.Q) ot[(long long)(c0 + j) * d.Q] = __float2bfloat16_rn(v[j]);
                }
            }
        }
    }
    pipe_destroy(p, ncols);
}

// ---------------------------------------------------------------------------------------------------------
// Local chunk states / local state gradients, both directions stacked along M:
//   MODE 0 (chunk_state): out[dir][p][n] = sum_l (B[l,n] Delta[l] e^{T-cs_dir[l]}) x[l,p]
//   MODE 1 (dstates):     out[dir][p][n] = sum_l (C[l,n] e^{cs_dir[l]})            g[l,p]
// D rows m = dir*N + n, D columns p.   grid (b*nc*H, ceil(2N/128)); n_tile = round16(P); tables: 2*Q floats.
template <class T, int MODE, int BCH>
__global__ void __launch_bounds__(kThreads, BCH <= 2 ? 2 : 1) state_gemm(Dims d, View rowsrc /* B or C */, View colsrc /* x or dout */,
                                                       View z, const float *dt_out, const float *cs_f,
                                                       const float *cs_b, float *out, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ PipeShared sh;
    const int nt = round_up(d.P, 16);
    Carve cv = carve(dyn, nt);
    float *wf = cv.tab, *wb = cv.tab + d.Q;
    const int h = blockIdx.x % d.H, c = (blockIdx.x / d.H) % d.nc, b = blockIdx.x / (d.H * d.nc);
    const int g = h / d.R;
    const int lim = min(d.Q, d.L - c * d.Q);
    const long long base = ((long long)(b * d.H + h) * d.nc + c) * d.Q;
    {
        const float Tf = cs_f[base + d.Q - 1], Tb = cs_b[base];
        for (int l = threadIdx.x; l < d.Q; l += kThreads) {
            if (MODE == 0) {
                const float dl = dt_out[base + l];
                wf[l] = __expf(Tf - cs_f[base + l]) * dl;
                wb[l] = __expf(Tb - cs_b[base + l]) * dl;
            } else {
                wf[l] = __expf(cs_f[base + l]);
                wb[l] = __expf(cs_b[base + l]);
            }
        }
    }
    Pipe p;
    const uint32_t ncols = tmem_cols(nt);
    pipe_init(p, &sh, cv.stage, b_stage_bytes(nt), ncols, status);     // contains the __syncthreads for the tables
    const int m0 = blockIdx.y * kTileM;
    const int N = d.N;
    auto fa = [&](int r, int k) -> uint4 {                              // MN-major: rows m..m+7 at sequence index k
        const int m = m0 + r;
        if (m >= 2 * N || k >= lim) return zero8();
        const int dir = m >= N, n = m - dir * N;
        return scale8<T>(ld8v<T>(rowsrc, b, c * d.Q + k, g, n), dir ? wb[k] : wf[k]);
    };
    auto fb = [&](int r, int k) -> uint4 {                              // MN-major: p..p+7 at sequence index k
        if (r >= d.P || k >= lim) return zero8();
        return MODE == 0 ? ld8v<T>(colsrc, b, c * d.Q + k, h, r) : gate8<T>(d, colsrc, z, b, c * d.Q + k, h, r);
    };
    bool ok = umma_gemm<T, true, true, BCH>(p, p.tmem, nt, d.Q, 0u, fa, fb);
    ok = ok && umma_drain(p);
    if (ok) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int m = m0 + (warp & 3) * 32 + lane;
        const int dir = m >= N, n = m - dir * N;
        const long long per_dir = (long long)d.b * d.nc * d.H * d.P * N;
        float *o = out + dir * per_dir + ((long long)(b * d.nc + c) * d.H + h) * d.P * N + n;
        for (int c0 = (warp >> 2) * 32; c0 < nt; c0 += 64) {
            float v[32];
            tmem_ld32(tmem_lane_base(p.tmem) + c0, v);
            if (m < 2 * N) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (c0 + j < d.P) o[(long long)(c0 + j) * N] = v[j];
            }
        }
    }
    pipe_destroy(p, ncols);
}

// ---------------------------------------------------------------------------------------------------------
// Forward output (see simt::chunk_scan for the formula).  One accumulator, three K-segments:
//   [C e^{cs_f} | S_f]  [C e^{cs_b} | S_b]  [CB Delta (L_f+L_b) | x]
// grid (b*nc*H, ceil(Q/128)); n_tile = round16(P); tables: 3*Q floats.
template <class T, int BCH>
__global__ void __launch_bounds__(kThreads, BCH <= 2 ? 2 : 1) chunk_scan(Dims d, View x, View Cm, View z, const float *D,
                                                       const float *dt_out, const float *cs_f, const float *cs_b,
                                                       const float *CB, const void *states_f, const void *states_b,
                                                       MutView out, MutView out_x, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ PipeShared sh;
    const int nt = round_up(d.P, 16);
    Carve cv = carve(dyn, nt);
    float *sf = cv.tab, *sb = cv.tab + d.Q, *sd = cv.tab + 2 * d.Q;
    const int h = blockIdx.x % d.H, c = (blockIdx.x / d.H) % d.nc, b = blockIdx.x / (d.H * d.nc);
    const int g = h / d.R;
    const int Q = d.Q, N = d.N;
    const int lim = min(Q, d.L - c * Q);
    const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
    for (int l = threadIdx.x; l < Q; l += kThreads) {
        sf[l] = cs_f[base + l];
        sb[l] = cs_b[base + l];
        sd[l] = dt_out[base + l];
    }
    Pipe p;
    const uint32_t ncols = tmem_cols(nt);
    pipe_init(p, &sh, cv.stage, b_stage_bytes(nt), ncols, status);
    const int l0 = blockIdx.y * kTileM;
    const float *cb = CB + ((long long)(b * d.nc + c) * d.G + g) * Q * Q;
    const long long st_base = ((long long)(b * d.nc + c) * d.H + h) * d.P * N;
    bool ok = true;
#pragma unroll 1
    for (int dir = 0; dir < 2 && ok; ++dir) {
        const float *cs = dir ? sb : sf;
        const void *st = dir ? states_b : states_f;
        auto fa = [&](int r, int k) -> uint4 {
            const int l = l0 + r;
            if (l >= lim || k >= N) return zero8();
            return scale8<T>(ld8v<T>(Cm, b, c * Q + l, g, k), __expf(cs[l]));
        };
        auto fb = [&](int r, int k) -> uint4 {
            return (r < d.P && k < N) ? ldg8(st, st_base + (long long)r * N + k) : zero8();
        };
        ok = umma_gemm<T, false, false, BCH>(p, p.tmem, nt, N, dir ? 1u : 0u, fa, fb);
    }
    if (ok) {
        auto fa = [&](int r, int k) -> uint4 {                          // K-major: M[l][s..s+7]
            const int l = l0 + r;
            if (l >= lim || k >= lim) return zero8();
            float v[8];
            ldg8f(cb + (long long)l * Q + k, v);
            const float fl = sf[l], bl = sb[l];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int s = k + j;
                const float e = (s <= l) ? fl - sf[s] : bl - sb[s];
                float w = __expf(e);
                if (s == l) w = 2.f;
                v[j] = (s < lim) ? v[j] * sd[s] * w : 0.f;
            }
            return pack8<T>(v);
        };
        auto fb = [&](int r, int k) -> uint4 {                          // MN-major: x[s][p..p+7]
            return (r < d.P && k < lim) ? ld8v<T>(x, b, c * Q + k, h, r) : zero8();
        };
        ok = umma_gemm<T, false, true, BCH>(p, p.tmem, nt, Q, 1u, fa, fb);
    }
    ok = ok && umma_drain(p);
    if (ok) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int l = l0 + (warp & 3) * 32 + lane;
        for (int c0 = (warp >> 2) * 32; c0 < nt; c0 += 64) {
            float v[32];
            tmem_ld32(tmem_lane_base(p.tmem) + c0, v);
            if (l < lim) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    const int p0 = c0 + j;
                    if (p0 >= d.P) continue;
                    float y[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) y[i] = v[j + i];
                    if (d.has_D) {
                        float xv[8];
                        unpack8<T>(ld8v<T>(x, b, c * Q + l, h, p0), xv);
#pragma unroll
                        for (int i = 0; i < 8; ++i) y[i] += (d.D_hdim ? D[h * d.P + p0 + i] : D[h]) * xv[i];
                    }
                    const long long oo = b * out.sb + (long long)(c * Q + l) * out.sl + h * out.sh + p0;
                    if (d.has_z) {
                        const long long ox = b * out_x.sb + (long long)(c * Q + l) * out_x.sl + h * out_x.sh + p0;
                        *reinterpret_cast<uint4 *>(static_cast<T *>(out_x.ptr) + ox) = pack8<T>(y);
                        float zz[8];
                        unpack8<T>(ld8v<T>(z, b, c * Q + l, h, p0), zz);
#pragma unroll
                        for (int i = 0; i < 8; ++i) y[i] *= zz[i] * sigmoidf_(zz[i]);
                    }
                    *reinterpret_cast<uint4 *>(static_cast<T *>(out.ptr) + oo) = pack8<T>(y);
                }
            }
        }
    }
    pipe_destroy(p, ncols);
}

// ---------------------------------------------------------------------------------------------------------
// dx, ddt_out, dz, dD partials (see simt::dx_kernel).  One accumulator, three K-segments:
//   [B e^{T-cs_f} | E_f]  [B e^{T-cs_b} | E_b]  [CB^T (L_f+L_b)^T | g]
// grid (b*nc*H, ceil(Q/128)); n_tile = round16(P); tables: 3*Q floats.
template <class T, int BCH>
__global__ void __launch_bounds__(kThreads, BCH <= 2 ? 2 : 1) dx_kernel(Dims d, View x, View Bm, View z, View dout, View out_x,
                                                      const float *D, const float *dt_out, const float *cs_f,
                                                      const float *cs_b, const float *CB, const void *E16, void *dx,
                                                      void *dz, float *ddt_out, float *dDpart, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ PipeShared sh;
    __shared__ float rowred[kTileM];
    __shared__ float colred[4][256];
    const int nt = round_up(d.P, 16);
    Carve cv = carve(dyn, nt);
    float *sf = cv.tab, *sb = cv.tab + d.Q, *sd = cv.tab + 2 * d.Q;
    const int h = blockIdx.x % d.H, c = (blockIdx.x / d.H) % d.nc, b = blockIdx.x / (d.H * d.nc);
    const int g = h / d.R;
    const int Q = d.Q, N = d.N;
    const int lim = min(Q, d.L - c * Q);
    const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
    for (int l = threadIdx.x; l < Q; l += kThreads) {
        sf[l] = cs_f[base + l];
        sb[l] = cs_b[base + l];
        sd[l] = dt_out[base + l];
    }
    Pipe p;
    const uint32_t ncols = tmem_cols(nt);
    pipe_init(p, &sh, cv.stage, b_stage_bytes(nt), ncols, status);
    const float Tf = sf[Q - 1], Tb = sb[0];
    const int l0 = blockIdx.y * kTileM;
    const float *cb = CB + ((long long)(b * d.nc + c) * d.G + g) * Q * Q;
    const long long per_dir = (long long)d.b * d.nc * d.H * d.P * N;
    const long long st_base = ((long long)(b * d.nc + c) * d.H + h) * d.P * N;
    bool ok = true;
#pragma unroll 1
    for (int dir = 0; dir < 2 && ok; ++dir) {
        const float *cs = dir ? sb : sf;
        const float T0 = dir ? Tb : Tf;
        const long long eoff = dir * per_dir + st_base;
        auto fa = [&](int r, int k) -> uint4 {
            const int l = l0 + r;
            if (l >= lim || k >= N) return zero8();
            return scale8<T>(ld8v<T>(Bm, b, c * Q + l, g, k), __expf(T0 - cs[l]));
        };
        auto fb = [&](int r, int k) -> uint4 { return (r < d.P && k < N) ? ldg8(E16, eoff + (long long)r * N + k) : zero8(); };
        ok = umma_gemm<T, false, false, BCH>(p, p.tmem, nt, N, dir ? 1u : 0u, fa, fb);
    }
    if (ok) {
        auto fa = [&](int r, int k) -> uint4 {                          // MN-major: rows l..l+7 at column s = k
            const int lb = l0 + r, s = k;
            if (lb >= lim || s >= lim) return zero8();
            float v[8];
            ldg8f(cb + (long long)s * Q + lb, v);
            const float fs = sf[s], bs = sb[s];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int l = lb + j;
                const float e = (s >= l) ? fs - sf[l] : bs - sb[l];
                float w = __expf(e);
                if (s == l) w = 2.f;
                v[j] = (l < lim) ? v[j] * w : 0.f;
            }
            return pack8<T>(v);
        };
        auto fb = [&](int r, int k) -> uint4 {                          // MN-major: g[s][p..p+7]
            return (r < d.P && k < lim) ? gate8<T>(d, dout, z, b, c * Q + k, h, r) : zero8();
        };
        ok = umma_gemm<T, true, true, BCH>(p, p.tmem, nt, Q, 1u, fa, fb);
    }
    ok = ok && umma_drain(p);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quad = warp & 3, half = warp >> 2;
    const int r = quad * 32 + lane, l = l0 + r;
    float rowsum = 0.f;
    if (ok) {
        for (int c0 = half * 32; c0 < nt; c0 += 64) {
            float v[32];
            tmem_ld32(tmem_lane_base(p.tmem) + c0, v);
            float cs8[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) cs8[j] = 0.f;
            if (l < lim) {
                const int ls = c * Q + l;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    const int p0 = c0 + j;
                    if (p0 >= d.P) continue;
                    float xv[8], gv[8], o[8];
                    unpack8<T>(ld8v<T>(x, b, ls, h, p0), xv);
                    unpack8<T>(ld8v<T>(dout, b, ls, h, p0), gv);
                    const long long oo = ((long long)(b * d.L + ls) * d.H + h) * d.P + p0;
                    if (d.has_z) {
                        float zz[8], ox[8], dzv[8];
                        unpack8<T>(ld8v<T>(z, b, ls, h, p0), zz);
                        unpack8<T>(ld8v<T>(out_x, b, ls, h, p0), ox);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float sg = sigmoidf_(zz[i]);
                            dzv[i] = gv[i] * ox[i] * sg * (1.f + zz[i] * (1.f - sg));
                            gv[i] *= zz[i] * sg;
                        }
                        *reinterpret_cast<uint4 *>(static_cast<T *>(dz) + oo) = pack8<T>(dzv);
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        o[i] = v[j + i] * sd[l];
                        if (d.has_D) o[i] += (d.D_hdim ? D[h * d.P + p0 + i] : D[h]) * gv[i];
                        rowsum += v[j + i] * xv[i];
                        cs8[j + i] = gv[i] * xv[i];
                    }
                    *reinterpret_cast<uint4 *>(static_cast<T *>(dx) + oo) = pack8<T>(o);
                }
            }
            if (d.has_D) {                                              // column sums of g*x over this warp's 32 rows
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float s = cs8[j];
#pragma unroll
                    for (int o2 = 16; o2 > 0; o2 >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
                    if (lane == 0) colred[quad][c0 + j] = s;
                }
            }
        }
    }
    if (half == 1) rowred[r] = rowsum;
    __syncthreads();
    if (ok) {
        if (half == 0 && l < Q) ddt_out[base + l] = rowsum + rowred[r];
        if (d.has_D && threadIdx.x < d.P) {
            const int pcol = threadIdx.x;
            const int nlt = gridDim.y;
            dDpart[(((long long)(b * d.nc + c) * d.H + h) * nlt + blockIdx.y) * d.P + pcol] =
                colred[0][pcol] + colred[1][pcol] + colred[2][pcol] + colred[3][pcol];
        }
    }
    pipe_destroy(p, ncols);
}

// ---------------------------------------------------------------------------------------------------------
// "States" parts of dB / dC summed over the heads of a group, and the decay-gradient row sums per head
// (see simt::dbc_states).  blockIdx.z: 0 = dB (A = x, B-operand = E, scale Delta e^{T-cs}), 1 = dC (A = g,
// B-operand = entering states, scale e^{cs}).  Per head two accumulators (forward / reverse direction) in TMEM;
// the head sum is kept in registers.  part layout [b, nc*Q, G, N] fp32; row sums [split][b,H,nc,Q].
// grid (b*nc*G*nsplit, ceil(Q/128), 2), nsplit = ceil(N/128); n_tile = min(round16(N), 128).
template <class T>
__global__ void __launch_bounds__(kThreads) dbc_states(Dims d, View x, View Bm, View Cm, View z, View dout,
                                                       const float *dt_out, const float *cs_f, const float *cs_b,
                                                       const void *E16, const void *states_f, const void *states_b,
                                                       float *dB_part, float *dC_part, float *nf, float *nb, float *pf,
                                                       float *pb, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ PipeShared sh;
    __shared__ float rowred[2][kTileM];
    const int N = d.N, Q = d.Q;
    const int nsplit = (N + 127) / 128;
    const int nt = min(round_up(N, 16), 128);
    Carve cv = carve(dyn, nt);
    Pipe p;
    pipe_init(p, &sh, cv.stage, b_stage_bytes(nt), 256, status);
    const int split = blockIdx.x % nsplit;
    const int bx = blockIdx.x / nsplit;
    const int g = bx % d.G, c = (bx / d.G) % d.nc, b = bx / (d.G * d.nc);
    const int which = blockIdx.z;
    const int lim = min(Q, d.L - c * Q);
    const int l0 = blockIdx.y * kTileM, n0 = split * 128;
    const int nvalid = min(nt, N - n0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quad = warp & 3, half = warp >> 2;
    const int r = quad * 32 + lane, l = l0 + r;
    const long long per_dir = (long long)d.b * d.nc * d.H * d.P * N;
    const View &other = which ? Cm : Bm;
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    bool ok = true;
#pragma unroll 1
    for (int hr = 0; hr < d.R && ok; ++hr) {
        const int h = g * d.R + hr;
        const long long st_base = ((long long)(b * d.nc + c) * d.H + h) * d.P * N;
        auto fa = [&](int rr, int k) -> uint4 {                         // K-major over the head dimension
            const int ll = l0 + rr;
            if (ll >= lim || k >= d.P) return zero8();
            return which ? gate8<T>(d, dout, z, b, c * Q + ll, h, k) : ld8v<T>(x, b, c * Q + ll, h, k);
        };
#pragma unroll 1
        for (int dir = 0; dir < 2 && ok; ++dir) {
            auto fb = [&](int rr, int k) -> uint4 {                     // MN-major: n..n+7 at head-dim index k
                if (rr >= nvalid || k >= d.P) return zero8();
                const long long o = st_base + (long long)k * N + n0 + rr;
                if (which) return ldg8(dir ? states_b : states_f, o);
                return ldg8(E16, dir * per_dir + o);
            };
            ok = umma_gemm<T, false, true, 4>(p, p.tmem + dir * 128, nt, d.P, 0u, fa, fb);
        }
        ok = ok && umma_drain(p);
        float rs_f = 0.f, rs_b = 0.f;
        if (ok) {
            const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
            float scf = 0.f, scb = 0.f;
            if (l < lim) {
                if (which) {
                    scf = __expf(cs_f[base + l]);
                    scb = __expf(cs_b[base + l]);
                } else {
                    const float dl = dt_out[base + l];
                    scf = dl * __expf(cs_f[base + Q - 1] - cs_f[base + l]);
                    scb = dl * __expf(cs_b[base] - cs_b[base + l]);
                }
            }
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                const int c0 = half * 32 + ch * 64;
                if (c0 >= nt) continue;
                float vf[32], vb[32];
                tmem_ld32(tmem_lane_base(p.tmem) + c0, vf);
                tmem_ld32(tmem_lane_base(p.tmem) + 128 + c0, vb);
                if (l < lim) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (c0 + j >= nvalid) continue;
                        float o[8];
                        unpack8<T>(ld8v<T>(other, b, c * Q + l, g, n0 + c0 + j), o);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float a = vf[j + i] * scf, bb = vb[j + i] * scb;
                            rs_f += a * o[i];
                            rs_b += bb * o[i];
                            acc[ch * 32 + j + i] += a + bb;
                        }
                    }
                }
            }
        }
        if (half == 1) {
            rowred[0][r] = rs_f;
            rowred[1][r] = rs_b;
        }
        tmem_reads_done();
        if (ok && half == 0 && l < Q) {
            const long long o = (long long)split * d.b * d.H * d.nc * Q + ((long long)(b * d.H + h) * d.nc + c) * Q + l;
            (which ? pf : nf)[o] = rs_f + rowred[0][r];
            (which ? pb : nb)[o] = rs_b + rowred[1][r];
        }
    }
    if (ok && l < lim) {
        float *part = (which ? dC_part : dB_part) + (((long long)b * d.nc * Q + c * Q + l) * d.G + g) * N + n0;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
            const int c0 = half * 32 + ch * 64;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                if (c0 + j < nvalid)
                    *reinterpret_cast<float4 *>(part + c0 + j) =
                        make_float4(acc[ch * 32 + j], acc[ch * 32 + j + 1], acc[ch * 32 + j + 2], acc[ch * 32 + j + 3]);
        }
    }
    pipe_destroy(p, 256);
}

// ---------------------------------------------------------------------------------------------------------
// dB[s,n] = sum_l dCB[l,s] C[l,n] + sum_r dB_part[s,r,n];  dC[l,n] = sum_s dCB[l,s] B[s,n] + sum_r dC_part[l,r,n]
// (see simt::bmm_bwd).  dCB is rounded to the 16-bit input type for the product, as the reference's kernel does.
// part layout [b, nc*Q, part_heads, N], part_heads / G entries are summed per group.
// grid (b*nc*G*2, ceil(Q/128), nsplit); n_tile = min(round16(N), 128).
template <class T>
__global__ void __launch_bounds__(kThreads) bmm_bwd(Dims d, View Bm, View Cm, const float *dCB, const float *dB_part,
                                                    const float *dC_part, int part_heads, void *dB, void *dC,
                                                    int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ PipeShared sh;
    const int N = d.N, Q = d.Q;
    const int nt = min(round_up(N, 16), 128);
    Carve cv = carve(dyn, nt);
    Pipe p;
    pipe_init(p, &sh, cv.stage, b_stage_bytes(nt), 128, status);
    const int which = blockIdx.x & 1;
    const int bx = blockIdx.x >> 1;
    const int g = bx % d.G, c = (bx / d.G) % d.nc, b = bx / (d.G * d.nc);
    const int lim = min(Q, d.L - c * Q);
    const int r0 = blockIdx.y * kTileM, n0 = blockIdx.z * 128;
    const int nvalid = min(nt, N - n0);
    const float *dcb = dCB + ((long long)(b * d.nc + c) * d.G + g) * Q * Q;
    const View &src = which ? Bm : Cm;
    auto fb = [&](int rr, int k) -> uint4 {                             // MN-major: n..n+7 at sequence index k
        return (rr < nvalid && k < lim) ? ld8v<T>(src, b, c * Q + k, g, n0 + rr) : zero8();
    };
    bool ok;
    if (which == 0) {
        auto fa = [&](int rr, int k) -> uint4 {                         // MN-major: dCB[l = k][s..s+7]
            return (r0 + rr < Q && k < lim) ? pack8f<T>(dcb + (long long)k * Q + r0 + rr) : zero8();
        };
        ok = umma_gemm<T, true, true, 4>(p, p.tmem, nt, Q, 0u, fa, fb);
    } else {
        auto fa = [&](int rr, int k) -> uint4 {                         // K-major: dCB[l][s..s+7]
            return (r0 + rr < lim && k < Q) ? pack8f<T>(dcb + (long long)(r0 + rr) * Q + k) : zero8();
        };
        ok = umma_gemm<T, false, true, 4>(p, p.tmem, nt, Q, 0u, fa, fb);
    }
    ok = ok && umma_drain(p);
    if (ok) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int row = r0 + (warp & 3) * 32 + lane;
        const int rp = part_heads / d.G;
        const float *part = (which ? dC_part : dB_part) + (((long long)b * d.nc * Q + c * Q + row) * part_heads + g * rp) * N + n0;
        T *out = static_cast<T *>(which ? dC : dB) + (((long long)b * d.L + c * Q + row) * d.G + g) * N + n0;
        for (int c0 = (warp >> 2) * 32; c0 < nt; c0 += 64) {
            float v[32];
            tmem_ld32(tmem_lane_base(p.tmem) + c0, v);
            if (row < lim) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    if (c0 + j >= nvalid) continue;
                    float o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = v[j + i];
                    for (int q = 0; q < rp; ++q) {
                        float t[8];
                        ldg8f(part + (long long)q * N + c0 + j, t);
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] += t[i];
                    }
                    *reinterpret_cast<uint4 *>(out + c0 + j) = pack8<T>(o);
                }
            }
        }
    }
    pipe_destroy(p, 128);
}

}  // namespace tc
}  // namespace bissd
