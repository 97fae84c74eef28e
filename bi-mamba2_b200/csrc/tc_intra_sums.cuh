// Intra-chunk decay gradients from row and column sums (TMA-fed; replaces the prefix-sweep kernel where it applies).
//
// With  W_f[l,s] = (g[l].x[s]) CB[l,s] Delta[s] e^{cs_f[l]-cs_f[s]}  (s < l)  and  W_b  likewise with cs_b (s > l),
// the two dominance sums the decay gradient needs,
//     da_f[j] = sum_{l>=j} sum_{s<j} W_f[l,s],      da_b[j] = sum_{l<=j} sum_{s>j} W_b[l,s],
// telescope:  da_f[j+1] - da_f[j] = C_f[j] - R_f[j]  and  da_b[j-1] - da_b[j] = C_b[j] - R_b[j]  with the column sums
// C[j] = sum_l W[l,j] and the row sums R[j] = sum_s W[j,s].  So this kernel only forms
//     u_f[j] = C_f[j] - R_f[j],    u_b[j] = C_b[j] - R_b[j]
// and the consumer (cumsum_bwd) adds u_f to the terms it prefix-sums exclusively and u_b to those it suffix-sums.
//
// Per CTA: one (batch, chunk, head) and 128 rows l.  G2 = g.x^T by tcgen05 into TMEM; every thread turns its row into
// V[l,s] = W_f (s<l) | 0 (s=l) | W_b (s>l), accumulating the row sums in registers and writing V as bf16 into shared
// memory; one more MMA with a lower-triangular ones matrix, D[m,s] = sum_{l<=m} V[l,s], then gives at once the column
// totals (row 127) and, on its diagonal, the split of each column into its part above the diagonal (= D[m, l0+m])
// and below it.  Output: u4[(row tile*2 + dir)][b,H,nc,Q], the two row tiles being added by the consumer.
//
// Shapes: chunk 128 or 256, headdim 64 or 128 (as the other TMA-fed kernels), 16-bit inputs.
#pragma once
#include "tc_kernels.cuh"
#include "tc_tma.cuh"

namespace bissd {
namespace tc {

inline size_t intra_sums_smem(int Q) { return smem_bytes(Q, 6 * Q); }

// grid (b*nc*H, Q/128)
template <class T>
__global__ void __launch_bounds__(kThreads, 2)
intra_sums(Dims d, const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmX, const float *dt_out,
           const float *cs_f, const float *cs_b, const float *CBs, float *u4, long long hq, int *status) {
    pdl_begin();
    extern __shared__ uint8_t dyn[];
    __shared__ PipeShared sh;
    __shared__ float rsum[2][2][kTileM];                          // [column half][direction][row]
    __shared__ float dg[kTileM];                                  // D[m, l0+m]
    __shared__ float tot[256];                                    // D[127, s]
    const int Q = d.Q, nt = Q;
    Carve cv = carve(dyn, nt);
    // log2-domain tables: f2 = cs_f log2e, b2 = cs_b log2e, tf = f2 - log2 Delta, tb = b2 - log2 Delta
    // and, per 16-column strip, the column factors of the factorised decay: a strip wholly left of a row's diagonal has
    // 2^(f2[l] - tf[s]) = 2^(f2[l] - f2[last column of the strip]) * colF[s], one wholly right of it
    // 2^(b2[l] - tb[s]) = 2^(b2[l] - b2[first column of the strip]) * colB[s]; both exponents stay <= 0.
    float *sf = cv.tab, *sb = cv.tab + Q, *tf = cv.tab + 2 * Q, *tb = cv.tab + 3 * Q, *colF = cv.tab + 4 * Q, *colB = cv.tab + 5 * Q;
    const int h = blockIdx.x % d.H, c = (blockIdx.x / d.H) % d.nc, b = blockIdx.x / (d.H * d.nc);
    const int g = h / d.R;
    const int lim = min(Q, d.L - c * Q);
    const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
    Pipe p;
    const uint32_t ncols = tmem_cols(nt);
    pipe_init(p, &sh, cv.stage, b_stage_bytes(nt), ncols, status);
    const int l0 = blockIdx.y * kTileM;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    bool ok = true;
    {
        // g (128 rows) and x (Q rows) by TMA into the stage buffers, one 64-wide headdim slab per buffer; the decay
        // tables are built while the tiles are in flight
        const int npb = d.P / 64;
        if (tid == 0) {
            mbar_expect_tx(&sh.free_bar[0], (uint32_t)(npb * (16384 + Q * 128)));
            for (int j = 0; j < npb; ++j) {
                tma_load4(p.a_stage[j], &tmG, j * 64, h, c * Q + l0, b, &sh.free_bar[0]);
                tma_load4(p.b_stage[j], &tmX, j * 64, h, c * Q, b, &sh.free_bar[0]);
            }
        }
        for (int i = threadIdx.x; i < Q; i += kThreads) {
            const float cf = cs_f[base + i] * 1.4426950408889634f, cb_ = cs_b[base + i] * 1.4426950408889634f;
            const float lg = __log2f(dt_out[base + i]);               // -inf on the zero-padded tail: those columns vanish
            sf[i] = cf;
            sb[i] = cb_;
            tf[i] = cf - lg;
            tb[i] = cb_ - lg;
            colF[i] = ex2_approx(cs_f[base + (i | 15)] * 1.4426950408889634f - (cf - lg));
            colB[i] = ex2_approx(cs_b[base + (i & ~15)] * 1.4426950408889634f - (cb_ - lg));
        }
        if (tid == 0) {
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
        }
        ok = __syncthreads_and(ok);
    }
    ok = ok && umma_drain(p);
    const int quarter = warp & 3, colhalf = warp >> 2;
    const int r = quarter * 32 + lane, l = l0 + r;
    if (ok) {
        // the operand tiles of the first product are dead: the lower-triangular ones matrix A[m,k] = [k <= m] takes the
        // place of g (two K slabs of 64), V will take the place of x
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int q = tid + i * kThreads;
            const int slab = q >> 10, m = (q & 1023) >> 3, cch = q & 7, k0 = slab * 64 + cch * 8;
            uint32_t wv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
                wv[e] = ((k0 + 2 * e <= m) ? 0x3F80u : 0u) | ((k0 + 2 * e + 1 <= m) ? 0x3F800000u : 0u);
            *reinterpret_cast<uint4 *>(p.a_stage[slab] + m * 128 + ((cch ^ (m & 7)) << 4)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        }
        const int wl_min = l0 + quarter * 32, wl_max = wl_min + 31;      // rows handled by this warp
        uint8_t *btile = p.b_stage[r >> 6];
        const int kl = r & 63;
        auto store8 = [&](int jc, uint4 v) {                             // columns 8*jc..8*jc+7 of row l
            *reinterpret_cast<uint4 *>(btile + (jc >> 3) * 8192 + (kl >> 3) * 1024 + (kl & 7) * 128 +
                                       (((jc & 7) ^ (kl & 7)) << 4)) = v;
        };
        const bool row_on = l < lim;
        // C.B^T is read from its copy in strips of 16 columns ([Q/16][Q][16]): this thread's 16 values of a strip are 64
        // contiguous bytes and the 32 rows of a warp 2 KB, whereas 32 row pieces of the row-major matrix are 32
        // separate lines
        const float *cbstrip = CBs + ((long long)(b * d.nc + c) * d.G + g) * Q * Q + min(l, Q - 1) * 16;
        const float fl = sf[min(l, Q - 1)], bl = sb[min(l, Q - 1)];
        float rf = 0.f, rb = 0.f;
        const int cbeg = colhalf * (Q / 2), cend = cbeg + Q / 2;
        float4 cbn[4];
        auto load_cb = [&](int c0) {
            const float4 *src = reinterpret_cast<const float4 *>(cbstrip + (long long)(c0 >> 4) * Q * 16);
#pragma unroll
            for (int q = 0; q < 4; ++q) cbn[q] = row_on ? __ldg(src + q) : make_float4(0.f, 0.f, 0.f, 0.f);
        };
        // the accumulator columns and the CB values of strip k+1 are requested before strip k is worked on
        uint32_t rn[16];
        tmem_ld16_nowait(tmem_lane_base(p.tmem) + cbeg, rn);
        load_cb(cbeg);
#pragma unroll 1
        for (int c0 = cbeg; c0 < cend; c0 += 16) {
            float v[16], cbv[16], w[16];
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(rn[j]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                cbv[4 * q] = cbn[q].x; cbv[4 * q + 1] = cbn[q].y; cbv[4 * q + 2] = cbn[q].z; cbv[4 * q + 3] = cbn[q].w;
            }
            if (c0 + 16 < cend) {
                tmem_ld16_nowait(tmem_lane_base(p.tmem) + c0 + 16, rn);
                load_cb(c0 + 16);
            }
            // The row sums are taken over the values as rounded to bf16 for the column-sum MMA: only then do row and
            // column sums telescope exactly and the rounding errors stay local instead of accumulating along the scan.
            const int side = (c0 + 15 < wl_min) ? 0 : (c0 > wl_max) ? 1 : 2;   // left of every diagonal / right / mixed
            if (side != 2) {
                const float *col = (side ? colB : colF) + c0;
                const float rfac = row_on ? ex2_approx(side ? bl - sb[c0] : fl - sf[c0 + 15]) : 0.f;
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    const float4 cf4 = *reinterpret_cast<const float4 *>(col + j);
                    w[j] = v[j] * cbv[j] * cf4.x * rfac;
                    w[j + 1] = v[j + 1] * cbv[j + 1] * cf4.y * rfac;
                    w[j + 2] = v[j + 2] * cbv[j + 2] * cf4.z * rfac;
                    w[j + 3] = v[j + 3] * cbv[j + 3] * cf4.w * rfac;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int s = c0 + j;
                    const float e = ex2_approx(s < l ? fl - tf[s] : bl - tb[s]);
                    w[j] = (!row_on || s == l) ? 0.f : v[j] * cbv[j] * e;
                }
            }
            const uint4 q0 = make_uint4(pack2<__nv_bfloat16>(w[0], w[1]), pack2<__nv_bfloat16>(w[2], w[3]),
                                        pack2<__nv_bfloat16>(w[4], w[5]), pack2<__nv_bfloat16>(w[6], w[7]));
            const uint4 q1 = make_uint4(pack2<__nv_bfloat16>(w[8], w[9]), pack2<__nv_bfloat16>(w[10], w[11]),
                                        pack2<__nv_bfloat16>(w[12], w[13]), pack2<__nv_bfloat16>(w[14], w[15]));
            store8(c0 >> 3, q0);
            store8((c0 >> 3) + 1, q1);
            float rq[16];
            unpack2<__nv_bfloat16>(q0.x, rq[0], rq[1]);
            unpack2<__nv_bfloat16>(q0.y, rq[2], rq[3]);
            unpack2<__nv_bfloat16>(q0.z, rq[4], rq[5]);
            unpack2<__nv_bfloat16>(q0.w, rq[6], rq[7]);
            unpack2<__nv_bfloat16>(q1.x, rq[8], rq[9]);
            unpack2<__nv_bfloat16>(q1.y, rq[10], rq[11]);
            unpack2<__nv_bfloat16>(q1.z, rq[12], rq[13]);
            unpack2<__nv_bfloat16>(q1.w, rq[14], rq[15]);
            if (side == 0) {
#pragma unroll
                for (int j = 0; j < 16; ++j) rf += rq[j];
            } else if (side == 1) {
#pragma unroll
                for (int j = 0; j < 16; ++j) rb += rq[j];
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    rf += (c0 + j < l) ? rq[j] : 0.f;
                    rb += (c0 + j > l) ? rq[j] : 0.f;
                }
            }
        }
        rsum[colhalf][0][r] = row_on ? rf : 0.f;
        rsum[colhalf][1][r] = row_on ? rb : 0.f;
        fence_async_smem();
    }
    tmem_reads_done();
    if (ok) {
        if (tid == 0) {
            tc_fence_after();
            umma_issue_stage<false, true>(p.tmem, nt, 1, p.a_stage[0], p.b_stage[0], 0u);
            umma_issue_stage<false, true>(p.tmem, nt, 1, p.a_stage[1], p.b_stage[1], 1u);
        }
        ok = umma_drain(p);
    }
    if (ok) {
        const uint32_t tl = tmem_lane_base(p.tmem);
        if (colhalf == 0) {                                              // the diagonal element of this thread's row
            float v[32];
            tmem_ld32(tl + l0 + quarter * 32, v);
            float x = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) x = (lane == j) ? v[j] : x;
            dg[r] = x;
        }
        if (quarter == 3) {                                              // lane 31 of these two warps holds row 127
            for (int c0 = colhalf * (Q / 2); c0 < (colhalf + 1) * (Q / 2); c0 += 32) {
                float v[32];
                tmem_ld32(tl + c0, v);
                if (lane == 31) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) tot[c0 + j] = v[j];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (ok && tid < Q) {
        const int s = tid, m = s - l0;
        const bool in = m >= 0 && m < kTileM;
        const float T_ = tot[s];
        const float above = in ? dg[m] : 0.f;                            // sum over rows l < s of column s
        const float Cf = in ? T_ - above : (s < l0 ? T_ : 0.f);
        const float Cb = in ? above : (s >= l0 + kTileM ? T_ : 0.f);
        const float Rf = in ? rsum[0][0][m] + rsum[1][0][m] : 0.f;
        const float Rb = in ? rsum[0][1][m] + rsum[1][1][m] : 0.f;
        u4[(blockIdx.y * 2 + 0) * hq + base + s] = Cf - Rf;
        u4[(blockIdx.y * 2 + 1) * hq + base + s] = Cb - Rb;
        if (gridDim.y == 1) {
            u4[2 * hq + base + s] = 0.f;
            u4[3 * hq + base + s] = 0.f;
        }
    }
    if (threadIdx.x < 32) tmem_dealloc(p.tmem, ncols);
}

}  // namespace tc
}  // namespace bissd
