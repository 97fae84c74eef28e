// dCB and the intra-chunk decay gradients from ONE product per head: a CTA walks the heads of a group.
//
// Both quantities start from G2_h = g_h x_h^T and the same masked decay weights
//     w_h[l,s] = Delta_h[s] ([s<l] e^{cs_f[l]-cs_f[s]} + [s>l] e^{cs_b[l]-cs_b[s]}),   2 Delta_h[l] on the diagonal:
//     dCB[l,s]   = sum_{h in group} G2_h[l,s] w_h[l,s]                       (see simt::dcb_kernel)
//     V_h[l,s]   = G2_h[l,s] w_h[l,s] CB[l,s]  for s != l,  0 on the diagonal
//     u_f[j] = (column sum - row sum) of the part of V_h below the diagonal, u_b[j] the same above it - the
//     differences of the two dominance sums the decay gradient needs (derivation in tc_intra_sums.cuh; cumsum_bwd
//     scans them).
// One CTA per (batch, chunk, group) and 128 x 128 tile of (l, s), 256 threads, two CTAs per SM: the bf16 C.B^T tile
// stays in shared memory; for each head g [128 x P] and x [128 x P] arrive by TMA, one tcgen05 chain gives G2 in
// tensor memory, the warps weight it (row x column factors everywhere; in a 16-column strip the diagonal crosses the
// factors are taken around the strip's own end columns and chosen per element, and only a strip whose decay across its
// 16 columns would leave fp32's range pays one ex2 per element), add it to the dCB tile they keep in registers, and write V as bf16 into shared
// memory - over g and x, which are dead once G2 exists; a second chain with a lower-triangular ones matrix,
// D[m,s] = sum_{l<=m} V[l,s], yields the column totals (row 127) and, in tiles on the diagonal, their split at the
// diagonal (D[m,m]).  Row sums are taken over the values as rounded for that chain, so that row and column sums
// telescope exactly.  While one CTA weights a head the other one's loads and products are in flight.  A tile writes two
// Q-long vectors (forward / reverse part): + column sums at its columns, - row sums at its rows, zero elsewhere;
// cumsum_bwd adds the vectors of a chunk's tiles.  Tiles off the diagonal hold one direction only and no mixed strip.
//
// Tried and measured at the benchmark shape (this form: 175 us at first, 140 us since the strips are dealt alternately,
// the diagonal strips factorised and the per-head read-out trimmed; the two separate kernels it replaces: 138 + 66 us):
// a 128 x Q tile per CTA with sixteen warps and the loads of the next head in flight (183 us); the 128 x 128 tile
// with one CTA per SM and every stage of the chain double-buffered (232 us - the kernel is bound by instruction
// issue, about twenty instructions per element and head, not by the chain's latencies).
//
// Shapes: headdim 64, chunk 128 or 256, 16-bit inputs.
#pragma once
#include "tc_scan_tma.cuh"

namespace bissd {
namespace tc {

struct IntraGrpShared {
    uint64_t bar_cb, bar_in, bar_m1, bar_m2;
    uint32_t tmem_base;
};

constexpr int kIntraTileThreads = 256;
constexpr float kMixedSpan = 60.f;                              // log2 of the largest decay across 16 columns the fast form takes
inline size_t intra_tile_smem(int Q) { return 1024 + 32768 + 32768 + 32768 + 6 * (size_t)Q * 4; }
inline bool intra_tile_ok(int P, int Q) { return P == 64 && (Q == 128 || Q == 256); }

template <class T>
__global__ void __launch_bounds__(kIntraTileThreads, 2)
intra_dcb_tile(Dims d, const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmX,
               const __grid_constant__ CUtensorMap tmCB, const float *dt_out, const float *cs_f, const float *cs_b,
               float *u4, long long hq, void *dCB16, int *status) {
    pdl_begin();
    extern __shared__ uint8_t dyn[];
    __shared__ IntraGrpShared sh;
    __shared__ float rsum[2][2][kTileM];                          // [column half][direction][row]
    __shared__ float dg[kTileM];                                  // D[m, m] of a diagonal tile
    __shared__ __align__(16) float tot[kTileM];                   // D[127, s]
    const int Q = d.Q, R = d.R;
    uint8_t *base_sm = smem_align1024(dyn);
    uint8_t *smCB = base_sm;                                      // two slabs [128 x 64] bf16, K-major
    uint8_t *smG = smCB + 32768;                                  // [128 x 64], K-major
    uint8_t *smX = smG + 16384;                                   // [128 x 64], K-major
    uint8_t *smV = smG;                                           // two K slabs [64 x 128] bf16 MN-major, over g and x
    uint8_t *smTri = smG + 32768;                                 // two slabs [128 x 64] bf16, K-major
    float *tab = reinterpret_cast<float *>(smTri + 32768);        // [6][Q]: f2, b2, tf, tb, colF, colB
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = blockIdx.x % d.G, c = (blockIdx.x / d.G) % d.nc, b = blockIdx.x / (d.G * d.nc);
    // Launch order (x, then y, then z) puts the tiles on the diagonal first: they carry the dearer strips, and the
    // second CTA an SM receives is then mostly one off the diagonal.
    const int ty = blockIdx.y ^ blockIdx.z, tz = blockIdx.y;
    const int l0 = ty * kTileM, s0 = tz * kTileM;
    const int quad = warp & 3, chalf = warp >> 2;
    const int r = quad * 32 + lane, l = l0 + r;
    const int lim = min(Q, d.L - c * Q);
    const bool row_on = l < lim;
    const int wl_min = l0 + quad * 32, wl_max = wl_min + 31;      // rows handled by this warp
    const int tile = ty * gridDim.z + tz;
    if (warp == 0) tmem_alloc(&sh.tmem_base, 256);
    auto load_head = [&](int hr) {                                // one thread: g and x of head hr
        const int h = g * R + hr;
        mbar_expect_tx(&sh.bar_in, 32768u);
        tma_load4(smG, &tmG, 0, h, c * Q + l0, b, &sh.bar_in);
        tma_load4(smX, &tmX, 0, h, c * Q + s0, b, &sh.bar_in);
    };
    if (tid == 32) {                                              // barriers and first loads by the same thread
        mbar_init(&sh.bar_cb, 1);
        mbar_init(&sh.bar_in, 1);
        mbar_init(&sh.bar_m1, 1);
        mbar_init(&sh.bar_m2, 1);
        fence_mbar_init();
        mbar_expect_tx(&sh.bar_cb, 32768u);
        const int row = ((b * d.nc + c) * d.G + g) * Q + l0;
        for (int k = 0; k < 2; ++k) tma_load2(smCB + k * 16384, &tmCB, s0 + k * 64, row, &sh.bar_cb);
        load_head(0);
    }
    float pcf = 0.f, pcb = 0.f, pdt = 1.f, pcfr = 0.f, pcbr = 0.f;
    auto fetch_tab = [&](int hr) {
        const int h = g * R + hr;
        const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
        if (tid < Q) {
            pcf = cs_f[base + tid];
            pcb = cs_b[base + tid];
            pdt = dt_out[base + tid];
            pcfr = cs_f[base + (tid | 15)];                       // reference columns of the factorised form
            pcbr = cs_b[base + (tid & ~15)];
        }
    };
    auto write_tab = [&]() {
        if (tid < Q) {
            const float cf = pcf * 1.4426950408889634f, cb_ = pcb * 1.4426950408889634f;
            const float lg = __log2f(pdt);                        // -inf on the zero-padded tail: those columns vanish
            tab[tid] = cf;
            tab[Q + tid] = cb_;
            tab[2 * Q + tid] = cf - lg;
            tab[3 * Q + tid] = cb_ - lg;
            tab[4 * Q + tid] = ex2_approx(pcfr * 1.4426950408889634f - (cf - lg));
            tab[5 * Q + tid] = ex2_approx(pcbr * 1.4426950408889634f - (cb_ - lg));
        }
    };
#pragma unroll
    for (int i = 0; i < 8; ++i) {                                 // lower-triangular ones matrix A[m,k] = [k <= m]
        const int q = tid + i * kIntraTileThreads;
        const int slab = q >> 10, m = (q & 1023) >> 3, cch = q & 7, k0 = slab * 64 + cch * 8;
        uint32_t wv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            wv[e] = ((k0 + 2 * e <= m) ? 0x3F80u : 0u) | ((k0 + 2 * e + 1 <= m) ? 0x3F800000u : 0u);
        *reinterpret_cast<uint4 *>(smTri + slab * 16384 + m * 128 + ((cch ^ (m & 7)) << 4)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
    }
    fetch_tab(0);
    write_tab();
    if (R > 1) fetch_tab(1);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    const uint32_t tG2 = tmem, tD2 = tmem + 128;
    auto issue_g2 = [&](int hr) -> bool {                         // thread 0: G2 of head hr
        if (!mbar_wait(&sh.bar_in, hr & 1)) return false;
        tc_fence_after();
        const uint32_t idesc = instr_desc(AbFmt<T>::v, false, false, 128);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
            umma(tG2, smem_desc(smem_u32(smG) + kk * 32, 16, 1024), smem_desc(smem_u32(smX) + kk * 32, 16, 1024), idesc,
                 kk > 0 ? 1u : 0u);
        umma_commit(&sh.bar_m1);
        return true;
    };
    bool ok = true;
    if (tid == 0) ok = issue_g2(0) && mbar_wait(&sh.bar_cb, 0);
    float acc[64];                                                // this thread's piece of the dCB tile: row l, 64 columns
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    const uint32_t tl = tmem_lane_base(tmem);
    const int cbeg = chalf * 64;                                  // first column of this warp's share of the read-out of row 127
    uint8_t *vtile = smV + (r >> 6) * 16384;
    const int kl = r & 63;
    auto store_v8 = [&](int jc, uint4 v) {                        // tile columns 8 jc .. 8 jc + 7 of row l
        *reinterpret_cast<uint4 *>(vtile + (jc >> 3) * 8192 + (kl >> 3) * 1024 + (kl & 7) * 128 +
                                   (((jc & 7) ^ (kl & 7)) << 4)) = v;
    };
#pragma unroll 1
    for (int hr = 0; hr < R; ++hr) {
        ok = mbar_wait_cta(&sh.bar_m1, hr & 1, ok);               // G2 of head hr is in tensor memory
        tc_fence_after();
        if (hr == 0 && ok && ty == tz && chalf == ((r >> 4) & 1)) {
            // V has no diagonal: the one thread that reads C.B^T[r, r] (its strip r / 16) clears it in the resident tile
            *reinterpret_cast<__nv_bfloat16 *>(smCB + (r >> 6) * 16384 + r * 128 + ((((r & 63) >> 3) ^ (r & 7)) << 4) +
                                               (r & 7) * 2) = __float2bfloat16(0.f);
        }
        float rf = 0.f, rb = 0.f;
        if (ok) {
            const float *sf = tab, *sb = tab + Q, *tf = tab + 2 * Q, *tb = tab + 3 * Q, *colF = tab + 4 * Q, *colB = tab + 5 * Q;
            const float fl = sf[min(l, Q - 1)], bl = sb[min(l, Q - 1)];
#pragma unroll
            for (int st = 0; st < 4; ++st) {                      // strips of 16 columns, dealt alternately to the two
                // warps of a row quarter: in a tile on the diagonal each then holds one of the two strips the diagonal crosses
                const int ct = (st * 2 + chalf) * 16, c0 = s0 + ct;   // within the tile / within the chunk
                float v[16], cbv[16], w[16];
                tmem_ld16(tl + ct, v);
                {
                    const uint8_t *rowp = smCB + (ct >> 6) * 16384 + r * 128;
                    const int ch = (ct & 63) >> 3;
                    float lo[8], hi[8];
                    unpack8<__nv_bfloat16>(*reinterpret_cast<const uint4 *>(rowp + ((ch ^ (r & 7)) << 4)), lo);
                    unpack8<__nv_bfloat16>(*reinterpret_cast<const uint4 *>(rowp + (((ch + 1) ^ (r & 7)) << 4)), hi);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        cbv[j] = lo[j];
                        cbv[8 + j] = hi[j];
                    }
                }
                const int side = (c0 + 15 < wl_min) ? 0 : (c0 > wl_max) ? 1 : 2;   // left of every diagonal / right / mixed
                if (side != 2) {
                    const float *col = (side ? colB : colF) + c0;
                    const float rfac = row_on ? ex2_approx(side ? bl - sb[c0] : fl - sf[c0 + 15]) : 0.f;
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const float4 cf4 = *reinterpret_cast<const float4 *>(col + j);
                        const float t0 = v[j] * cf4.x * rfac, t1 = v[j + 1] * cf4.y * rfac, t2 = v[j + 2] * cf4.z * rfac,
                                    t3 = v[j + 3] * cf4.w * rfac;
                        acc[st * 16 + j] += t0;
                        acc[st * 16 + j + 1] += t1;
                        acc[st * 16 + j + 2] += t2;
                        acc[st * 16 + j + 3] += t3;
                        w[j] = t0 * cbv[j];
                        w[j + 1] = t1 * cbv[j + 1];
                        w[j + 2] = t2 * cbv[j + 2];
                        w[j + 3] = t3 * cbv[j + 3];
                    }
                } else if (sf[c0] - sf[c0 + 15] <= kMixedSpan && sb[c0 + 15] - sb[c0] <= kMixedSpan) {
                    // The strip the diagonal crosses, factorised as well: the forward weights around the strip's last
                    // column, the reverse ones around its first (the column factors of the tables), a row factor each.
                    // A row inside the strip then has a row factor above one - bounded by the decay across the 16
                    // columns, which the test above keeps within fp32's range; the side a row does not use may
                    // overflow and is never selected.
                    const float rF = row_on ? ex2_approx(fl - sf[c0 + 15]) : 0.f;
                    const float rB = row_on ? ex2_approx(bl - sb[c0]) : 0.f;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int s = c0 + j;
                        const float wf = colF[s] * rF, wb = colB[s] * rB;
                        float wt = (s < l) ? wf : wb;
                        if (s == l) wt = wf + wf;                 // the diagonal counts once per direction in dCB
                        const float tj = v[j] * wt;               // rF = rB = 0 for a row past the sequence
                        acc[st * 16 + j] += tj;
                        w[j] = tj * cbv[j];                       // ... and not at all in the decay gradient: C.B^T's diagonal is zeroed
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int s = c0 + j;
                        float a = (s <= l) ? fl - tf[s] : bl - tb[s];
                        if (s == l) a += 1.f;                     // the diagonal counts once per direction in dCB
                        const float tj = row_on ? v[j] * ex2_approx(a) : 0.f;
                        acc[st * 16 + j] += tj;
                        w[j] = tj * cbv[j];                       // ... and not at all in the decay gradient: C.B^T's diagonal is zeroed
                    }
                }
                const uint4 q0 = make_uint4(pack2<__nv_bfloat16>(w[0], w[1]), pack2<__nv_bfloat16>(w[2], w[3]),
                                            pack2<__nv_bfloat16>(w[4], w[5]), pack2<__nv_bfloat16>(w[6], w[7]));
                const uint4 q1 = make_uint4(pack2<__nv_bfloat16>(w[8], w[9]), pack2<__nv_bfloat16>(w[10], w[11]),
                                            pack2<__nv_bfloat16>(w[12], w[13]), pack2<__nv_bfloat16>(w[14], w[15]));
                float rq[16];
                unpack8<__nv_bfloat16>(q0, *reinterpret_cast<float(*)[8]>(&rq[0]));
                unpack8<__nv_bfloat16>(q1, *reinterpret_cast<float(*)[8]>(&rq[8]));
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
                // V takes the place of g and x: both were consumed when bar_m1 completed (G2 is in tensor memory)
                store_v8(ct >> 3, q0);
                store_v8((ct >> 3) + 1, q1);
            }
        }
        rsum[chalf][0][r] = rf;
        rsum[chalf][1][r] = rb;
        fence_async_smem();
        tc_fence_before();
        ok = __syncthreads_and(ok);                               // V complete, G2 fully read, tables free
        if (tid == 0 && ok) {
            tc_fence_after();
            umma_issue_stage<false, true>(tD2, 128, 1, smTri, smV, 0u);
            umma_issue_stage<false, true>(tD2, 128, 1, smTri + 16384, smV + 16384, 1u);
            umma_commit(&sh.bar_m2);
        }
        if (hr + 1 < R) {                                         // single set of tables: the next head's go in here,
            write_tab();                                          // while the triangular product runs
            if (hr + 2 < R) fetch_tab(hr + 2);
        }
        ok = mbar_wait_cta(&sh.bar_m2, hr & 1, ok);               // column sums done: V (= g, x) may be overwritten
        tc_fence_after();
        if (tid == 0 && ok && hr + 1 < R) load_head(hr + 1);
        if (ok) {
            if (ty == tz && chalf == (quad >> 1)) {   // the diagonal element of this thread's row
                float v[32];
                tmem_ld32(tl + 128 + quad * 32, v);
                float x = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) x = (lane == j) ? v[j] : x;
                dg[r] = x;
            }
            if (quad == 3) {                                      // lane 31 of these two warps holds row 127
#pragma unroll
                for (int c0 = 0; c0 < 64; c0 += 32) {
                    float v[32];
                    tmem_ld32(tl + 128 + cbeg + c0, v);
                    if (lane == 31) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4 *>(&tot[cbeg + c0 + j]) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    }
                }
            }
        }
        tc_fence_before();
        ok = __syncthreads_and(ok);
        if (!ok) break;
        if (tid == 0 && hr + 1 < R) ok = issue_g2(hr + 1);        // its loads have had the read-out above to land
        if (tid < Q) {
            const int h = g * R + hr;
            const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
            const int j = tid, mc = j - s0, mr = j - l0;          // position as a column / as a row of this tile
            const bool incol = mc >= 0 && mc < kTileM, inrow = mr >= 0 && mr < kTileM;
            float uf = 0.f, ub = 0.f;
            if (incol) {
                const float T_ = tot[mc];
                if (ty == tz) {
                    const float above = dg[mc];                   // rows l < s of column s
                    uf += T_ - above;
                    ub += above;
                } else if (ty > tz) {
                    uf += T_;                                     // every row of the tile lies below its columns
                } else {
                    ub += T_;
                }
            }
            if (inrow) {
                uf -= rsum[0][0][mr] + rsum[1][0][mr];
                ub -= rsum[0][1][mr] + rsum[1][1][mr];
            }
            u4[(tile * 2 + 0) * hq + base + j] = uf;
            u4[(tile * 2 + 1) * hq + base + j] = ub;
        }
    }
    if (!ok && tid == 0) atomicExch(status, kErrMmaTimeout);
    if (ok && l < Q) {                                            // the rounded dCB tile; zero outside the sequence
        T *out = static_cast<T *>(dCB16) + ((long long)(b * d.nc + c) * d.G + g) * Q * Q + (long long)l * Q + s0;
#pragma unroll
        for (int j0 = 0; j0 < 64; j0 += 8) {
            const int col = ((j0 >> 4) * 2 + chalf) * 16 + (j0 & 8);   // acc[16 st + j] is tile column 16 (2 st + chalf) + j
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = (l < lim && s0 + col + i < lim) ? acc[j0 + i] : 0.f;
            *reinterpret_cast<uint4 *>(out + col) = pack8<T>(o);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace tc
}  // namespace bissd
