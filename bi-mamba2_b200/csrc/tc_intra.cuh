// Tensor-core kernels for the two backward products built on G2[l,s] = g[l].x[s] (per head):
//   * dcb_kernel       - dCB[l,s] = sum_{h in group} G2_h[l,s] Delta_h[s] ([s<=l] e^{cs_f[l]-cs_f[s]} + [s>=l] e^{cs_b[l]-cs_b[s]})
//   * intra_decay_grad - the intra-chunk decay gradients da_f + da_b (see simt::intra_decay_grad), where the masked
//     column sums over the rows of the prefix/suffix matrices are themselves done on the tensor core (a ones-row
//     times the bf16-rounded matrix).
#pragma once
#include "tc_kernels.cuh"
#include "tc_tma.cuh"

namespace bissd {
namespace tc {

// ---------------------------------------------------------------------------------------------------------
// grid (b*nc*G, ceil(Q/128) row tiles, ceil(Q/128) column tiles); n_tile = min(round16(Q), 128); tables 3*Q floats.
template <class T>
__global__ void __launch_bounds__(kThreads) dcb_kernel(Dims d, View x, View z, View dout, const float *dt_out,
                                                       const float *cs_f, const float *cs_b, float *dCB, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ PipeShared sh;
    const int Q = d.Q;
    const int nt = min(round_up(Q, 16), 128);
    Carve cv = carve(dyn, nt);
    float *sf = cv.tab, *sb = cv.tab + Q, *sd = cv.tab + 2 * Q;
    Pipe p;
    pipe_init(p, &sh, cv.stage, b_stage_bytes(nt), 128, status);
    const int g = blockIdx.x % d.G, c = (blockIdx.x / d.G) % d.nc, b = blockIdx.x / (d.G * d.nc);
    const int lim = min(Q, d.L - c * Q);
    const int l0 = blockIdx.y * kTileM, s0 = blockIdx.z * 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = warp >> 2;
    const int l = l0 + (warp & 3) * 32 + lane;
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    bool ok = true;
#pragma unroll 1
    for (int hr = 0; hr < d.R && ok; ++hr) {
        const int h = g * d.R + hr;
        const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
        for (int i = threadIdx.x; i < Q; i += kThreads) {
            sf[i] = cs_f[base + i];
            sb[i] = cs_b[base + i];
            sd[i] = dt_out[base + i];
        }
        auto fa = [&](int r, int k) -> uint4 {
            return (l0 + r < lim && k < d.P) ? gate8<T>(d, dout, z, b, c * Q + l0 + r, h, k) : zero8();
        };
        auto fb = [&](int r, int k) -> uint4 {
            return (s0 + r < lim && k < d.P) ? ld8v<T>(x, b, c * Q + s0 + r, h, k) : zero8();
        };
        ok = umma_gemm<T, false, false, 4>(p, p.tmem, nt, d.P, 0u, fa, fb);  // its barrier also publishes the tables
        ok = ok && umma_drain(p);
        if (ok) {
            const float fl = (l < lim) ? sf[l] : 0.f, bl = (l < lim) ? sb[l] : 0.f;
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                const int c0 = half * 32 + ch * 64;
                if (c0 >= nt) continue;
                float v[32];
                tmem_ld32(tmem_lane_base(p.tmem) + c0, v);
                if (l < lim) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int s = s0 + c0 + j;
                        if (s < lim) {
                            float w = __expf((s <= l) ? fl - sf[s] : bl - sb[s]);
                            if (s == l) w = 2.f;
                            acc[ch * 32 + j] += v[j] * sd[s] * w;
                        }
                    }
                }
            }
        }
        tmem_reads_done();
    }
    if (ok && l < Q) {
        float *out = dCB + ((long long)(b * d.nc + c) * d.G + g) * Q * Q + (long long)l * Q + s0;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
            const int c0 = half * 32 + ch * 64;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                if (c0 + j < nt && s0 + c0 + j < Q)
                    *reinterpret_cast<float4 *>(out + c0 + j) =
                        make_float4(acc[ch * 32 + j], acc[ch * 32 + j + 1], acc[ch * 32 + j + 2], acc[ch * 32 + j + 3]);
        }
    }
    pipe_destroy(p, 128);
}

// One 16-column strip of a row of the intra-chunk sweep.  DIR 0: left to right, W[s] counted for s < l, rm[j] = sum of
// W left of column j (kept for j <= l).  DIR 1: right to left, W[s] for s > l, rm[j] = sum right of j (kept for j >= l).
// tt: the strip's 16 table entries (tf or tb); rl: f2[l] or b2[l].
template <int DIR>
__device__ __forceinline__ void sweep_strip(const float (&v)[16], const float (&cbv)[16], float (&rm)[16], float &run,
                                            const float *tt, float rl, int c0, int l, int Q) {
    const bool whole = DIR ? (c0 > l) : (c0 + 15 < l);          // strip entirely inside this row's triangle
#pragma unroll
    for (int gq = 0; gq < 2; ++gq) {
        const int j0 = DIR ? 8 - 8 * gq : 8 * gq;
        float tv[8];
        if (c0 + j0 < Q) {
            const float4 t0 = *reinterpret_cast<const float4 *>(tt + j0), t1 = *reinterpret_cast<const float4 *>(tt + j0 + 4);
            tv[0] = t0.x; tv[1] = t0.y; tv[2] = t0.z; tv[3] = t0.w; tv[4] = t1.x; tv[5] = t1.y; tv[6] = t1.z; tv[7] = t1.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) tv[i] = 1e30f;
        }
#pragma unroll
        for (int ii = 0; ii < 8; ++ii) {
            const int i = DIR ? 7 - ii : ii, j = j0 + i, s = c0 + j;
            const float w = v[j] * cbv[j] * ex2_approx(rl - tv[i]);
            if (whole) {
                rm[j] = run;
                run += w;
            } else if (DIR == 0) {
                rm[j] = (s <= l) ? run : 0.f;
                if (s < l) run += w;
            } else {
                rm[j] = (s >= l) ? run : 0.f;
                if (s > l) run += w;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Intra-chunk decay gradients for one (batch, chunk, head) and one tile of 128 rows l:
//   W_f[l,s] = G2 CB Delta[s] e^{cs_f[l]-cs_f[s]} (s<l),  R_f[l,j] = sum_{s<j} W_f[l,s],  da_f[j] = sum_{l>=j} R_f[l,j]
//   W_b[l,s] = G2 CB Delta[s] e^{cs_b[l]-cs_b[s]} (s>l),  R_b[l,j] = sum_{s>j} W_b[l,s],  da_b[j] = sum_{l<=j} R_b[l,j]
// Warps 0-3 sweep their rows left to right (prefix, forward direction), warps 4-7 right to left (suffix, reverse
// direction); the masked matrices [j<=l] R_f + [j>=l] R_b are written as bf16 into a shared-memory tile and summed
// over l by an MMA with a ones matrix.  Output: partial da over this row tile, out_part[row tile][b,H,nc,Q]
// (the two row tiles of a 256-chunk are added by the consumer); tile 0 zero-fills part 1 when there is only one tile.
// grid (b*nc*H, ceil(Q/128)); n_tile = round16(Q); tables 3*Q floats + 128*8 exchange floats.
template <class T, bool TMA>
__global__ void __launch_bounds__(kThreads, 2) intra_decay_grad(Dims d, const __grid_constant__ CUtensorMap tmG,
                                                             const __grid_constant__ CUtensorMap tmX, View x, View z,
                                                             View dout, const float *dt_out,
                                                             const float *cs_f, const float *cs_b, const float *CB,
                                                             float *da_part0, float *da_part1, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ PipeShared sh;
    const int Q = d.Q;
    const int nt = round_up(Q, 16);
    Carve cv = carve(dyn, nt);
    // log2-domain tables: f2 = cs_f log2e, b2 = cs_b log2e, tf = f2 - log2 Delta, tb = b2 - log2 Delta
    float *sf = cv.tab, *sb = cv.tab + Q, *tf = cv.tab + 2 * Q, *tb = cv.tab + 3 * Q, *xch = cv.tab + 4 * Q;   // xch[128][8]
    const int h = blockIdx.x % d.H, c = (blockIdx.x / d.H) % d.nc, b = blockIdx.x / (d.H * d.nc);
    const int g = h / d.R;
    const int lim = min(Q, d.L - c * Q);
    const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
    for (int i = threadIdx.x; i < Q; i += kThreads) {
        const float cf = cs_f[base + i] * 1.4426950408889634f, cb_ = cs_b[base + i] * 1.4426950408889634f;
        const float lg = __log2f(dt_out[base + i]);           // -inf on the zero-padded tail: those columns vanish
        sf[i] = cf;
        sb[i] = cb_;
        tf[i] = cf - lg;
        tb[i] = cb_ - lg;
    }
    Pipe p;
    const uint32_t ncols = tmem_cols(nt);
    pipe_init(p, &sh, cv.stage, b_stage_bytes(nt), ncols, status);
    const int l0 = blockIdx.y * kTileM;
    auto fa = [&](int r, int k) -> uint4 {
        return (l0 + r < lim && k < d.P) ? gate8<T>(d, dout, z, b, c * Q + l0 + r, h, k) : zero8();
    };
    auto fb = [&](int r, int k) -> uint4 { return (r < lim && k < d.P) ? ld8v<T>(x, b, c * Q + r, h, k) : zero8(); };
    bool ok;
    if (TMA) {
        // g (128 rows) and x (Q rows) tiles by TMA into the engine's stage buffers, one 64-wide headdim slab per buffer
        const int npb = d.P / 64;
        if (threadIdx.x == 0) {
            mbar_expect_tx(&sh.free_bar[0], (uint32_t)(npb * (16384 + Q * 128)));
            for (int j = 0; j < npb; ++j) {
                tma_load4(p.a_stage[j], &tmG, j * 64, h, c * Q + l0, b, &sh.free_bar[0]);
                tma_load4(p.b_stage[j], &tmX, j * 64, h, c * Q, b, &sh.free_bar[0]);
            }
            ok = mbar_wait(&sh.free_bar[0], 0);
            if (ok) {
                tc_fence_after();
                const uint32_t idesc = instr_desc(AbFmt<T>::v, false, false, nt);
                for (int j = 0; j < npb; ++j)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma(p.tmem, smem_desc(smem_u32(p.a_stage[j]) + kk * 32, 16, 1024),
                             smem_desc(smem_u32(p.b_stage[j]) + kk * 32, 16, 1024), idesc, (j > 0 || kk > 0) ? 1u : 0u);
            }
        } else {
            ok = true;
        }
        ok = __syncthreads_and(ok);
    } else {
        ok = umma_gemm<T, false, false>(p, p.tmem, nt, d.P, 0u, fa, fb);
    }
    ok = ok && umma_drain(p);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dirn = warp >> 2;
    const int r = (warp & 3) * 32 + lane, l = l0 + r;
    const int wl_min = l0 + (warp & 3) * 32, wl_max = wl_min + 31;      // rows handled by this warp
    uint8_t *btile = p.b_stage[r >> 6];
    const int kl = r & 63;
    const int qd = l >> 3;                                              // 8-column group holding the diagonal
    auto store8 = [&](int jc, uint4 v) {                                // columns 8*jc..8*jc+7 of row l
        *reinterpret_cast<uint4 *>(btile + (jc >> 3) * 8192 + (kl >> 3) * 1024 + (kl & 7) * 128 +
                                   (((jc & 7) ^ (kl & 7)) << 4)) = v;
    };
    if (ok) {
        const float *cbrow = CB + ((long long)(b * d.nc + c) * d.G + g) * Q * Q + (long long)min(l, Q - 1) * Q;
        const bool row_on = l < lim;
        float run = 0.f;
        float diag[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) diag[i] = 0.f;
        // 16-column strips; the CB values of the next strip are requested before the current one is processed
        const int nstrip = nt / 16;
        auto strip_c0 = [&](int t) { return (dirn ? nstrip - 1 - t : t) * 16; };
        auto strip_live = [&](int c0) { return dirn ? (c0 + 15 > wl_min) : (c0 < wl_max); };
        float4 cbn[4];
        auto load_cb = [&](int c0) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                cbn[q] = (row_on && c0 + q * 4 < Q) ? __ldg(reinterpret_cast<const float4 *>(cbrow + c0 + q * 4))
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
        };
        if (strip_live(strip_c0(0))) load_cb(strip_c0(0));
        for (int t = 0; t < nstrip; ++t) {
            const int c0 = strip_c0(t);
            // a strip contributes only where it overlaps this warp's triangle (s < l forward, s > l reverse)
            const bool live = strip_live(c0);
            float rm[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) rm[j] = 0.f;
            if (live) {
                float v[16], cbv[16];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    cbv[4 * q] = cbn[q].x; cbv[4 * q + 1] = cbn[q].y; cbv[4 * q + 2] = cbn[q].z; cbv[4 * q + 3] = cbn[q].w;
                }
                tmem_ld16(tmem_lane_base(p.tmem) + c0, v);
                if (t + 1 < nstrip && strip_live(strip_c0(t + 1))) load_cb(strip_c0(t + 1));
                if (row_on) {
                    if (!dirn) sweep_strip<0>(v, cbv, rm, run, tf + c0, sf[l], c0, l, Q);
                    else sweep_strip<1>(v, cbv, rm, run, tb + c0, sb[l], c0, l, Q);
                }
            } else if (t + 1 < nstrip && strip_live(strip_c0(t + 1))) {
                load_cb(strip_c0(t + 1));
            }
            // forward warps own the 8-column groups left of the diagonal group, reverse warps those right of it
#pragma unroll
            for (int j = 0; j < 16; j += 8) {
                const int jc = (c0 + j) >> 3;
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = rm[j + i];
                if (jc == qd) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) diag[i] = o[i];
                } else if (dirn ? (jc > qd) : (jc < qd)) {
                    store8(jc, pack8<__nv_bfloat16>(o));
                }
            }
        }
        if (dirn) {
#pragma unroll
            for (int i = 0; i < 8; ++i) xch[r * 8 + i] = diag[i];
        }
        __syncthreads();
        if (!dirn) {
            if (qd * 8 < nt) {
#pragma unroll
                for (int i = 0; i < 8; ++i) diag[i] += xch[r * 8 + i];
                store8(qd, pack8<__nv_bfloat16>(diag));
            }
        }
        // ones matrix as the A operand (K-major, one stage reused for both K halves)
        for (int q = threadIdx.x; q < kTileM * 8; q += kThreads)
            *reinterpret_cast<uint4 *>(p.a_stage[0] + q * 16) = make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
        fence_async_smem();
    }
    tmem_reads_done();
    if (ok) {
        if (threadIdx.x == 0) {
            tc_fence_after();
            umma_issue_stage<false, true>(p.tmem, nt, 1, p.a_stage[0], p.b_stage[0], 0u);
            umma_issue_stage<false, true>(p.tmem, nt, 1, p.a_stage[0], p.b_stage[1], 1u);
        }
        ok = umma_drain(p);
    }
    if (ok && (warp & 3) == 0) {                                        // row 0 of the result holds the column sums
        float *out = (blockIdx.y == 0 ? da_part0 : da_part1) + base;
        for (int c0 = dirn * 32; c0 < nt; c0 += 64) {
            float v[32];
            tmem_ld32(tmem_lane_base(p.tmem) + c0, v);
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (c0 + j < Q) out[c0 + j] = v[j];
            }
        }
        if (gridDim.y == 1 && warp == 0)
            for (int j = lane; j < Q; j += 32) da_part1[base + j] = 0.f;
    }
    pipe_destroy(p, ncols);
}

}  // namespace tc
}  // namespace bissd
