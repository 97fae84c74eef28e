// Persistent warp-specialised kernels for the two "masked-decay tile times activations" passes:
//   MODE 0  forward chunk scan (see simt::chunk_scan for the formula): operands C, C.B^T, entering states, x
//   MODE 1  backward dx / ddt_out / "next" terms / dD (see simt::dx_kernel): operands B, (C.B^T)^T, passed state
//           gradients, g = gated output gradient
// Both have the shape  acc[l,:] = rf[l] (A.S_f^T)[l,:] + rb[l] (A.S_b^T)[l,:] + sum_s M[l,s] X[s,:]  and differ in
// the decay tables behind M and in the epilogue.  The description below uses the forward names.
//
// One CTA per SM walks a contiguous range of (batch, chunk, row tile, head) tiles.  Consecutive tiles of one group
// share the C rows [128 x N] and the 16-bit C.B^T rows [128 x Q]; both stay resident in shared memory while the heads
// of the group stream through:
//
//   warp 0 (one lane)   issues every tcgen05.mma
//   warp 1 (one lane)   issues every TMA load
//   warps 2-9           epilogue: TMEM -> registers -> out_x / out in 32-byte pieces (row factors, gate);
//                       warps w and w+4 share 32 rows and take 32 columns each
//   warps 10-17         build the masked-decay tile M 64 columns at a time into a ring of stages
//
// The rows the epilogue reads beside the accumulators - z (MODE 0) or x (MODE 1), a [128 x 64] tile per step - come
// by TMA into one more buffer, requested by a lane of the first epilogue warp a tile ahead: as per-lane loads (32 row
// pieces, 32 different lines per instruction) they cost the backward kernel 12 us at the benchmark shape.  g, which the
// backward epilogue needs too, still comes by per-lane loads: there is no room for a second buffer, and reading it out
// of the MMA's operand pieces (same rows, same layout) ties the loader to the epilogue and measured slower.
//
// Accumulators are double-buffered in TMEM (2 x 3P columns), so the epilogue of tile i overlaps the MMAs of tile i+1
// and the M build of tile i+1/i+2.  The entering states of tile i+1 are requested as soon as the state products of
// tile i have completed; x of tile i+1 arrives in 64-row pieces, each requested once the MMAs that read the same
// piece of tile i have completed.
//
// M[l,s] = CB[l,s] w[l,s] with w = Delta[s] (L_f + L_b)[l,s].  In blocks of 32 rows x 64 columns that lie entirely
// below (above) the diagonal, w factorises around a reference index between s and l - both exponents stay <= 0 -
// into a row factor and a column factor, so only the blocks the diagonal crosses pay one ex2 per element.  A per-head
// scalar D is folded into the diagonal of M.
//
// Every blocking point is an mbarrier wait with an attempt limit; a wait that runs out raises a CTA-wide flag that
// every other wait polls, the status word is set and all roles leave their loops.
//
// Shapes: headdim 64, dstate 64 or 128, chunk 128 or 256, 16-bit inputs.
#pragma once
#include "tc_kernels.cuh"
#include "tc_tma.cuh"

namespace bissd {
namespace tc {

constexpr int kWsBuilderWarps = 8, kWsEpiWarps = 8;
constexpr int kWsFirstEpi = 2, kWsFirstBuilder = kWsFirstEpi + kWsEpiWarps;
constexpr int kWsThreads = 32 * (kWsFirstBuilder + kWsBuilderWarps);
constexpr int kWsMaxMStages = 3;
// Ring of built M stages: three where shared memory allows (dstate 64), two beside the row tile at dstate 128 (two
// and three measured the same there: scan 112 / 114, dx 139 / 141 us).
__host__ __device__ constexpr int ws_m_stages(int nsl) { return nsl == 1 ? 3 : 2; }
constexpr int kWsRowBytes = kTileM * 128;                       // the epilogue's rows of one tile: [128 x 64] 16-bit

struct WsShared {
    uint64_t grp_full, grp_done, st_full, st_done, tab_bar, fin_bar;
    // MODE 1: row sums of the upper column half are in place; one barrier per (row quarter, rowred slot).  The upper
    // half can run two tiles ahead of its partner, so a single barrier per quarter could be two phases ahead of a
    // waiter - which a parity wait cannot tell from "not yet" (and at the end of the tile list nothing would follow
    // to release it).  With one barrier per slot it is at most zero phases ahead.
    uint64_t red_bar[4][3];
    uint64_t x_full[4], x_free[4];
    uint64_t m_full[kWsMaxMStages], m_free[kWsMaxMStages];
    uint64_t acc_full[2], acc_free[2];
    uint64_t r_full, r_free;     // the epilogue's row tile (z or x) has landed / every epilogue warp has taken its rows
    uint32_t tmem_base;
    int fail;
};

inline size_t scan_ws_smem(int P, int N, int Q) {
    return 1024 + (size_t)(N / 64) * 16384 + (size_t)(Q / 64) * 16384 + 2 * (size_t)(N / 64) * P * 128 + (size_t)Q * 128 +
           (size_t)ws_m_stages(N / 64) * kAStageBytes + kWsRowBytes + 2 * 6 * (size_t)Q * 4;
}
inline bool scan_ws_ok(int P, int N, int Q) {
    if (P != 64 || (N != 64 && N != 128) || (Q != 128 && Q != 256)) return false;
    return scan_ws_smem(P, N, Q) <= 227 * 1024;
}

// Walks (batch, chunk, row tile, head) tiles in the order head fastest; grp numbers the (batch, chunk, row tile,
// group) sets whose tiles share C and C.B^T.
struct WsIter {
    int b, c, rt, h, hr, g, grp;
    __device__ __forceinline__ void init(const Dims &d, int nrt, int t) {
        h = t % d.H;
        int r = t / d.H;
        rt = r % nrt;
        r /= nrt;
        c = r % d.nc;
        b = r / d.nc;
        g = h / d.R;
        hr = h - g * d.R;
        grp = ((b * d.nc + c) * nrt + rt) * d.G + g;
    }
    __device__ __forceinline__ void next(const Dims &d, int nrt) {
        ++h;
        if (++hr == d.R) {
            hr = 0;
            ++g;
            ++grp;
        }
        if (h == d.H) {
            h = 0;
            g = 0;
            if (++rt == nrt) {
                rt = 0;
                if (++c == d.nc) {
                    c = 0;
                    ++b;
                }
            }
        }
    }
};

__device__ __forceinline__ float tanh_approx(float v) {
    float r;
    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
// 16 consecutive 16-bit elements (32-byte aligned) from global memory in one access
__device__ __forceinline__ void ldg16(const void *p, uint4 &lo, uint4 &hi) {
    asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
                 : "l"(p));
}

// 16 consecutive 16-bit elements to global memory: one 32-byte store when the address allows it
__device__ __forceinline__ void stg16(void *p, const uint4 &lo, const uint4 &hi, bool wide) {
    if (wide) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(lo.x), "r"(lo.y), "r"(lo.z),
                     "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                     : "memory");
    } else {
        reinterpret_cast<uint4 *>(p)[0] = lo;
        reinterpret_cast<uint4 *>(p)[1] = hi;
    }
}
// Position in the ring of M stages and the parity of each stage's next "free" phase.
struct WsRing {
    uint32_t mb = 0, par = 0, used = 0;
};

// raw (8 bf16) * rf * col[j], as the operand type T.  bf16: the product is formed in packed bf16 arithmetic (one more
// rounding than the fp32 route, a third of the instructions); f16: through fp32.
template <class T>
__device__ __forceinline__ uint4 ws_scale8(const uint4 &raw, float rf, const float (&col)[8]);
template <>
__device__ __forceinline__ uint4 ws_scale8<__nv_bfloat16>(const uint4 &raw, float rf, const float (&col)[8]) {
    uint4 o;
    const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t out[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 w = __floats2bfloat162_rn(rf * col[2 * k], rf * col[2 * k + 1]);
        const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&in[k]), w);
        out[k] = *reinterpret_cast<const uint32_t *>(&v);
    }
    o.x = out[0]; o.y = out[1]; o.z = out[2]; o.w = out[3];
    return o;
}
template <>
__device__ __forceinline__ uint4 ws_scale8<__half>(const uint4 &raw, float rf, const float (&col)[8]) {
    float v[8];
    unpack8<__nv_bfloat16>(raw, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= rf * col[j];
    return pack8<__half>(v);
}

// All stages of one tile whose rows start at l0.  Deliberately a compact runtime loop (the code of all four roles has
// to stay resident in the instruction caches): per stage wait for the ring slot, then for each of the four 32-row
// blocks pick - uniformly over the CTA - the factorised form below / above the diagonal or the per-element form.
template <class T, int NST>
__device__ __forceinline__ bool ws_build_tile(const uint8_t *smCB, uint8_t *smM, const float *tabp, int ns, int l0, int bt,
                                              int lane, float dfold, WsRing &ring, uint64_t *m_full, uint64_t *m_free,
                                              volatile int *fail) {
    const int cc = bt & 7, r0 = bt >> 3, Q = ns * 64;
    const float *f2 = tabp, *b2 = f2 + Q, *tf = b2 + Q, *tb = tf + Q, *colF = tb + Q, *colB = colF + Q;
    const uint32_t swz = (uint32_t)((cc ^ (r0 & 7)) << 4);      // r & 7 is the same for this thread's four rows
#pragma unroll 1
    for (int s = 0; s < ns; ++s) {
        const int s0 = s * 64, sc = s0 + cc * 8;
        if (ring.used >= NST &&
            !ws_wait_warp(&m_free[ring.mb], ((ring.par >> ring.mb) & 1) ^ 1, fail, 33))
            return false;
        const uint8_t *slab = smCB + s * 16384;
        uint8_t *stage = smM + ring.mb * kAStageBytes;
        // a stage has blocks below the diagonal or above it, never both (rows span 128, columns 64); the column
        // factors around the stage's reference index come from the per-tile tables
        const bool below = l0 + 127 > s0 + 63 && !(l0 < s0);
        const float ref = below ? f2[s0 + 63] : b2[s0];
        float col[8];
        {
            const float *cp = (below ? colF : colB) + sc;
            const float4 a = *reinterpret_cast<const float4 *>(cp), b = *reinterpret_cast<const float4 *>(cp + 4);
            col[0] = a.x; col[1] = a.y; col[2] = a.z; col[3] = a.w; col[4] = b.x; col[5] = b.y; col[6] = b.z; col[7] = b.w;
        }
        // rows in two halves of 64 (two 32-row blocks of the same kind each), the two blocks interleaved
#pragma unroll 1
        for (int qp = 0; qp < 2; ++qp) {
            const int lo = l0 + 64 * qp;
            const int ra = r0 + 64 * qp, rb = ra + 32, la = l0 + ra, lb = l0 + rb;
            const uint4 rawa = *reinterpret_cast<const uint4 *>(slab + ra * 128 + swz);
            const uint4 rawb = *reinterpret_cast<const uint4 *>(slab + rb * 128 + swz);
            uint4 oa, ob;
            if (lo > s0 + 63 || lo + 63 < s0) {                  // both blocks on one side of the diagonal
                const float rfa = ex2_approx((below ? f2[la] : b2[la]) - ref);
                const float rfb = ex2_approx((below ? f2[lb] : b2[lb]) - ref);
                oa = ws_scale8<T>(rawa, rfa, col);
                ob = ws_scale8<T>(rawb, rfb, col);
            } else {
                float tfv[8], tbv[8];
                {
                    const float4 a = *reinterpret_cast<const float4 *>(tf + sc), b = *reinterpret_cast<const float4 *>(tf + sc + 4);
                    tfv[0] = a.x; tfv[1] = a.y; tfv[2] = a.z; tfv[3] = a.w; tfv[4] = b.x; tfv[5] = b.y; tfv[6] = b.z; tfv[7] = b.w;
                    const float4 c = *reinterpret_cast<const float4 *>(tb + sc), e = *reinterpret_cast<const float4 *>(tb + sc + 4);
                    tbv[0] = c.x; tbv[1] = c.y; tbv[2] = c.z; tbv[3] = c.w; tbv[4] = e.x; tbv[5] = e.y; tbv[6] = e.z; tbv[7] = e.w;
                }
                float va[8], vb[8];
                unpack8<__nv_bfloat16>(rawa, va);
                unpack8<__nv_bfloat16>(rawb, vb);
                const float fa = f2[la], ba = b2[la], fb = f2[lb], bb = b2[lb];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int sj = sc + j;
                    const float wa = ex2_approx(sj <= la ? fa - tfv[j] : ba - tbv[j]);
                    const float wb = ex2_approx(sj <= lb ? fb - tfv[j] : bb - tbv[j]);
                    va[j] = (sj == la) ? fmaf(va[j], 2.f * wa, dfold) : va[j] * wa;
                    vb[j] = (sj == lb) ? fmaf(vb[j], 2.f * wb, dfold) : vb[j] * wb;
                }
                oa = pack8<T>(va);
                ob = pack8<T>(vb);
            }
            *reinterpret_cast<uint4 *>(stage + ra * 128 + swz) = oa;
            *reinterpret_cast<uint4 *>(stage + rb * 128 + swz) = ob;
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&m_full[ring.mb]);
        ring.par ^= 1u << ring.mb;
        ring.mb = (ring.mb + 1 == NST) ? 0 : ring.mb + 1;
        ++ring.used;
    }
    return true;
}

// Everything the epilogues and the table builders read or write through plain pointers.
struct WsArgs {
    View x;                  // MODE 0: x for a per-element D; MODE 1: x
    View z;                  // MODE 0: z (gate); MODE 1: g, the gated output gradient
    const float *D, *dt_out, *cs_f, *cs_b;
    MutView out, out_x;      // MODE 0: out, out_x; MODE 1: out = dx
    float *ddt_out, *nf, *nb, *dDpart;   // MODE 1
    int wide_z, wide_x, wide_o;          // 32-byte accesses allowed on z / x / the outputs
    int rows_by_tma;                     // the epilogue's z (MODE 0) / x (MODE 1) rows arrive through tmR
};

// One step of the transpose-reduce over a warp: every lane holds N values (one per column); lanes whose bit N/2 is
// clear keep the lower half of the columns and receive the partner's lower half, the others the upper half.  After
// the steps N = 8, 4, 2 lane j holds in v[0] the sum over the 8 lanes that agree with it above bit 2, for column j & 7.
template <int N>
__device__ __forceinline__ void ws_fold(float (&v)[32], int lane) {
    constexpr int H2 = N / 2;
    const bool up = (lane & H2) != 0;
#pragma unroll
    for (int k = 0; k < H2; ++k) {
        const float send = up ? v[k] : v[k + H2];
        const float keep = up ? v[k + H2] : v[k];
        v[k] = keep + __shfl_xor_sync(0xffffffffu, send, H2);
    }
}

// The epilogue's row tile ([128 rows x 64 columns] of z or x, K-major with the 128-byte swizzle) comes by TMA instead of
// 32 per-lane row pieces per load instruction.  One lane of the first epilogue warp requests the tile of the next
// step as soon as all eight epilogue warps have copied their rows of the current one into registers.
struct WsRows {
    const CUtensorMap *map;
    uint8_t *buf;
    int issued;
    __device__ __forceinline__ void request(WsShared &sh, const Dims &d, const WsIter &w, int Q) {
        mbar_expect_tx(&sh.r_full, (uint32_t)kWsRowBytes);
        tma_load4(buf, map, 0, w.h, w.c * Q + w.rt * kTileM, w.b, &sh.r_full);
        ++issued;
    }
};
// this lane's 32 columns (columns ch .. ch + 31 of row r) of the landed tile
__device__ __forceinline__ void ws_take_rows(const uint8_t *buf, int r, int ch, uint4 (&out)[4]) {
    const uint8_t *rowp = buf + r * 128;
#pragma unroll
    for (int q = 0; q < 4; ++q) out[q] = *reinterpret_cast<const uint4 *>(rowp + ((((ch >> 3) + q) ^ (r & 7)) << 4));
}
// Every epilogue warp, at the top of tile i: wait for the tile's rows, copy them, hand the buffer back; the issuing lane
// then waits for all warps and requests the rows of tile i + 1 (`next` is that tile).  False if a wait ran out.
__device__ __forceinline__ bool ws_rows_step(WsShared &sh, WsRows &rw, const Dims &d, int Q, int i, int nt, const WsIter &next,
                                             bool issuer, int r, int ch, int lane, uint4 (&out)[4], volatile int *fail) {
    if (!ws_wait_warp(&sh.r_full, i & 1, fail, 23)) return false;
    ws_take_rows(rw.buf, r, ch, out);
    __syncwarp();
    if (lane == 0) mbar_arrive(&sh.r_free);
    if (issuer && lane == 0 && i + 1 < nt) {
        if (ws_wait(&sh.r_free, i & 1, fail, 24)) {
            fence_async_smem();                                 // the warps' reads precede the next TMA write
            rw.request(sh, d, next, Q);
        }
    }
    __syncwarp();
    return true;
}

// MODE 1 epilogue (one warp: rows 32*quarter.., columns ch..ch+31 of every tile of this CTA):
//   a = wf (B.E_f^T) + wb (B.E_b^T) + Mt.g;  dx = a Delta + D g;  ddt_out = sum_p a x;  nf / nb = Delta wf|wb sum_p
//   (B.E^T) x;  dD partial = column sums of g x.  Row sums are completed across the two column halves through shared
//   memory (three tiles deep: the upper-half warp can run at most two tiles ahead of its partner).
template <class T, int NS>
__device__ __forceinline__ void ws_epilogue_dx(const Dims &d, const WsArgs &a, WsShared &sh, float (*rowred)[3][kTileM],
                                               uint32_t tl, int quarter, int ch, int lane, WsIter it, int nt, int nrt,
                                               volatile int *fail, WsRows &rw, bool issuer) {
    constexpr int P = 64, Q = NS * 64;
    const View x = a.x, g = a.z;
    const int half = ch >> 5, r = quarter * 32 + lane;
    uint4 xr[4], gr[4];
    auto load16 = [&](const T *p, bool wide, uint4 &lo, uint4 &hi) {
        if (wide) {
            ldg16(p, lo, hi);
        } else {
            lo = __ldg(reinterpret_cast<const uint4 *>(p));
            hi = __ldg(reinterpret_cast<const uint4 *>(p) + 1);
        }
    };
    auto load_rows = [&](const WsIter &w) {
        const int l = w.rt * kTileM + r;
        const bool live = l < min(Q, d.L - w.c * Q);
        const T *xp = static_cast<const T *>(x.ptr) + w.b * x.sb + (long long)(w.c * Q + l) * x.sl + w.h * x.sh + ch;
        const T *gp = static_cast<const T *>(g.ptr) + w.b * g.sb + (long long)(w.c * Q + l) * g.sl + w.h * g.sh + ch;
        if (!live) {
#pragma unroll
            for (int q = 0; q < 4; ++q) gr[q] = zero8();
            if (!a.rows_by_tma) {
#pragma unroll
                for (int q = 0; q < 4; ++q) xr[q] = zero8();
            }
        } else {
            if (!a.rows_by_tma) {
                load16(xp, a.wide_x, xr[0], xr[1]);
                load16(xp + 16, a.wide_x, xr[2], xr[3]);
            }
            load16(gp, a.wide_z, gr[0], gr[1]);
            load16(gp + 16, a.wide_z, gr[2], gr[3]);
        }
    };
    if (nt > 0) load_rows(it);
    for (int i = 0; i < nt; ++i) {
        const int buf = i & 1, slot = i % 3;
        if (a.rows_by_tma) {                                     // x rows of this tile from the TMA-fed buffer
            WsIter nx = it;
            nx.next(d, nrt);
            if (!ws_rows_step(sh, rw, d, Q, i, nt, nx, issuer, r, ch, lane, xr, fail)) break;
        }
        const int lim = min(Q, d.L - it.c * Q);
        const int l = it.rt * kTileM + r;
        const long long base = ((long long)(it.b * d.H + it.h) * d.nc + it.c) * Q;
        const bool live = l < lim;
        float dl = 0.f, e1 = 0.f, e2 = 0.f;
        if (live) {
            dl = a.dt_out[base + l];
            e1 = a.cs_f[base + Q - 1] - a.cs_f[base + l];
            e2 = a.cs_b[base] - a.cs_b[base + l];
        }
        const float Dh = (d.has_D && !d.D_hdim) ? a.D[it.h] : 0.f;
        T *pdx = static_cast<T *>(a.out.ptr) + it.b * a.out.sb + (long long)(it.c * Q + l) * a.out.sl + it.h * a.out.sh + ch;
        if (!ws_wait_warp(&sh.acc_full[buf], (i >> 1) & 1, fail, 21)) break;
        tc_fence_after();
        const float wf = live ? __expf(e1) : 0.f, wb = live ? __expf(e2) : 0.f;
        const uint32_t acc = tl + buf * 3 * P + ch;
        float rs = 0.f, rsf = 0.f, rsb = 0.f, gxs = 0.f;
        const bool d_cols = d.has_D && d.D_hdim;                 // per-(head, channel) D: column sums of g x are needed
        const long long dslot = ((long long)(it.b * d.nc + it.c) * d.H + it.h) * (nrt * 4) + it.rt * 4 + quarter;
        uint4 held = zero8();
#pragma unroll
        for (int c0 = 0; c0 < 32; c0 += 8) {
            uint32_t rf[8], rb[8], ri[8];
            tmem_ld8_nowait(acc + c0, rf);
            tmem_ld8_nowait(acc + P + c0, rb);
            tmem_ld8_nowait(acc + 2 * P + c0, ri);
            tmem_ld_wait();
            if (c0 + 8 >= 32) {                                  // the accumulator is free once the last read has landed
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh.acc_free[buf]);
            }
            float xv[8], gv[8], o[8], gx[32];
            unpack8<T>(xr[c0 >> 3], xv);
            unpack8<T>(gr[c0 >> 3], gv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float af = __uint_as_float(rf[j]), ab = __uint_as_float(rb[j]);
                const float av = fmaf(wf, af, fmaf(wb, ab, __uint_as_float(ri[j])));
                o[j] = av * dl;
                if (d.has_D) o[j] = fmaf(d.D_hdim ? a.D[it.h * P + ch + c0 + j] : Dh, gv[j], o[j]);
                rs = fmaf(av, xv[j], rs);
                rsf = fmaf(af, xv[j], rsf);
                rsb = fmaf(ab, xv[j], rsb);
                gx[j] = gv[j] * xv[j];
            }
            if (c0 & 8) {
                if (live) stg16(pdx + c0 - 8, held, pack8<T>(o), a.wide_o);
            } else {
                held = pack8<T>(o);
            }
            if (d.has_D && !d_cols) {                            // per-head D: only the total of g x matters
#pragma unroll
                for (int j = 0; j < 8; ++j) gxs += gx[j];
            }
            if (d_cols) {                                        // column sums of g x over this warp's 32 rows
                ws_fold<8>(gx, lane);
                ws_fold<4>(gx, lane);
                ws_fold<2>(gx, lane);
                float v = gx[0];                                 // sum over the 8 lanes that share lane bits 3 and 4
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                if (lane < 8) a.dDpart[dslot * P + ch + c0 + lane] = v;
            }
        }
        if (d.has_D && !d_cols) {                                // one partial per warp and tile, in a compact array
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) gxs += __shfl_xor_sync(0xffffffffu, gxs, o);
            if (lane == 0) a.dDpart[dslot * 2 + half] = gxs;
        }
        if (half == 1) {
            rowred[slot][0][r] = rs;
            rowred[slot][1][r] = rsf;
            rowred[slot][2][r] = rsb;
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.red_bar[quarter][slot]);
        } else {
            if (!ws_wait_warp(&sh.red_bar[quarter][slot], (i / 3) & 1, fail, 22)) break;
            rs += rowred[slot][0][r];
            rsf += rowred[slot][1][r];
            rsb += rowred[slot][2][r];
            a.ddt_out[base + l] = rs;
            a.nf[base + l] = dl * wf * rsf;
            a.nb[base + l] = dl * wb * rsb;
        }
        it.next(d, nrt);
        if (i + 1 < nt) load_rows(it);                           // a whole tile ahead of their use
    }
}

// NSL = dstate / 64, NS = chunk / 64
template <class T, int NSL, int NS, int MODE>
__global__ void __launch_bounds__(kWsThreads, 1)
ws_kernel(Dims d, const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmCB,
          const __grid_constant__ CUtensorMap tmSf, const __grid_constant__ CUtensorMap tmSb,
          const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmR, const WsArgs a, int *status) {
    pdl_begin();
    extern __shared__ uint8_t dyn[];
    __shared__ WsShared sh;
    __shared__ float rowred[MODE == 1 ? 3 : 1][3][kTileM];       // MODE 1: three tiles deep, (rs, rsf, rsb) per row
    const View x = a.x, z = a.z;
    const float *D = a.D, *dt_out = a.dt_out, *cs_f = a.cs_f, *cs_b = a.cs_b;
    const MutView out = a.out, out_x = a.out_x;
    const int wide_z = a.wide_z, wide_o = a.wide_o;
    constexpr int P = 64, Q = NS * 64, nrt = Q / kTileM;
    uint8_t *base_sm = smem_align1024(dyn);
    uint8_t *smC = base_sm;                                   // NSL slabs [128 x 64], K-major
    uint8_t *smCB = smC + NSL * 16384;                        // NS slabs [128 x 64] bf16, K-major
    uint8_t *smS = smCB + NS * 16384;                         // per K slab: S_f [P x 64] then S_b [P x 64]
    uint8_t *smX = smS + 2 * NSL * P * 128;                   // [Q x 64], MN-major, in NS pieces of 64 rows
    constexpr int NST = ws_m_stages(NSL);
    uint8_t *smM = smX + Q * 128;                             // NST stages [128 x 64]
    uint8_t *smR = smM + NST * kAStageBytes;           // the epilogue's row tile (tmR): z (MODE 0) or x (MODE 1)
    float *tab = reinterpret_cast<float *>(smR + kWsRowBytes);    // 2 x (f2, b2, tf, tb, colF, colB)[Q]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int *fail = &sh.fail;

    const int total = d.b * d.nc * nrt * d.H;
    const int t0 = (int)((long long)total * blockIdx.x / gridDim.x);
    const int t1 = (int)((long long)total * (blockIdx.x + 1) / gridDim.x);
    const int nt = t1 - t0;
    constexpr uint32_t ncols = 512;
    if (warp == 0) tmem_alloc(&sh.tmem_base, ncols);
    if (tid == 32) {
        mbar_init(&sh.grp_full, 1);
        mbar_init(&sh.grp_done, 1);
        mbar_init(&sh.st_full, 1);
        mbar_init(&sh.st_done, 1);
        mbar_init(&sh.tab_bar, kWsBuilderWarps);
        mbar_init(&sh.fin_bar, 1);
        for (int i = 0; i < 4; ++i) {
            for (int k = 0; k < 3; ++k) mbar_init(&sh.red_bar[i][k], 1);
            mbar_init(&sh.x_full[i], 1);
            mbar_init(&sh.x_free[i], 1);
        }
        for (int i = 0; i < NST; ++i) {
            mbar_init(&sh.m_full[i], kWsBuilderWarps);
            mbar_init(&sh.m_free[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh.acc_full[i], 1);
            mbar_init(&sh.acc_free[i], kWsEpiWarps);
        }
        mbar_init(&sh.r_full, 1);
        mbar_init(&sh.r_free, kWsEpiWarps);
        sh.fail = 0;
        fence_mbar_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0) {
        // --------------------------------------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint64_t dC = smem_desc(smem_u32(smC), 16, 1024), dS = smem_desc(smem_u32(smS), 16, 1024);
            const uint64_t dM = smem_desc(smem_u32(smM), 16, 1024), dX = smem_desc(smem_u32(smX), (uint32_t)Q * 128, 1024);
            constexpr uint32_t idesc_st = instr_desc(AbFmt<T>::v, false, false, 2 * P);
            constexpr uint32_t idesc_m = instr_desc(AbFmt<T>::v, false, true, P);
            WsIter it;
            it.init(d, nrt, t0);
            bool ok = true;
            int cur_grp = -1;
            uint32_t ngrp = 0, mb = 0, m_par = 0;
            for (int i = 0; i < nt && ok; ++i) {
                const int buf = i & 1;
                const uint32_t acc = tmem + buf * 3 * P;
                if (it.grp != cur_grp) {
                    ok = ws_wait(&sh.grp_full, ngrp & 1, fail, 1);
                    ++ngrp;
                    cur_grp = it.grp;
                }
                if (ok && i >= 2) ok = ws_wait(&sh.acc_free[buf], ((i >> 1) - 1) & 1, fail, 2);
                ok = ok && ws_wait(&sh.st_full, i & 1, fail, 3);
                if (!ok) break;
                tc_fence_after();
                // both directions in one N = 2P product: B rows 0..P-1 are S_f, rows P..2P-1 are S_b
#pragma unroll
                for (int j = 0; j < NSL; ++j)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma(acc, dC + ((j * 16384 + kk * 32) >> 4), dS + ((j * 2 * P * 128 + kk * 32) >> 4), idesc_st,
                             (j > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&sh.st_done);
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    ok = ok && ws_wait(&sh.m_full[mb], (m_par >> mb) & 1, fail, 4) && ws_wait(&sh.x_full[s], i & 1, fail, 5);
                    if (ok) {
                        tc_fence_after();
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma(acc + 2 * P, dM + ((mb * kAStageBytes + kk * 32) >> 4),
                                 dX + (((s * 64 + kk * 16) * 128) >> 4), idesc_m, (s > 0 || kk > 0) ? 1u : 0u);
                        umma_commit(&sh.m_free[mb]);
                        umma_commit(&sh.x_free[s]);
                        m_par ^= 1u << mb;
                        mb = (mb + 1 == NST) ? 0 : mb + 1;
                    }
                }
                if (!ok) break;
                umma_commit(&sh.acc_full[buf]);
                it.next(d, nrt);
                if (i + 1 < nt && it.grp != cur_grp) umma_commit(&sh.grp_done);   // C and C.B^T may be replaced
            }
            if (!ok) {
                umma_commit(&sh.fin_bar);                       // leave no MMA in flight
                mbar_wait(&sh.fin_bar, 0);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------------------------------------- TMA loads
        if (lane == 0) {
            WsIter it;
            it.init(d, nrt, t0);
            bool ok = true;
            int cur_grp = -1;
            int ngrp = 0, loads_st = 0, loads_x[4] = {0, 0, 0, 0};
            for (int j = 0; j < nt && ok; ++j) {
                if (it.grp != cur_grp) {
                    if (ngrp > 0) ok = ws_wait(&sh.grp_done, (ngrp - 1) & 1, fail, 11);
                    if (!ok) break;
                    mbar_expect_tx(&sh.grp_full, (uint32_t)((NSL + NS) * 16384));
#pragma unroll
                    for (int k = 0; k < NSL; ++k)
                        tma_load4(smC + k * 16384, &tmC, k * 64, it.g, it.c * Q + it.rt * kTileM, it.b, &sh.grp_full);
                    const int row = ((it.b * d.nc + it.c) * d.G + it.g) * Q + it.rt * kTileM;
#pragma unroll
                    for (int k = 0; k < NS; ++k) tma_load2(smCB + k * 16384, &tmCB, k * 64, row, &sh.grp_full);
                    cur_grp = it.grp;
                    ++ngrp;
                }
                if (j > 0) ok = ws_wait(&sh.st_done, (j - 1) & 1, fail, 12);
                if (!ok) break;
                const int tile = (it.b * d.nc + it.c) * d.H + it.h;
                mbar_expect_tx(&sh.st_full, (uint32_t)(2 * NSL * P * 128));
#pragma unroll
                for (int k = 0; k < NSL; ++k) {
                    tma_load2(smS + (2 * k) * P * 128, &tmSf, k * 64, tile * P, &sh.st_full);
                    tma_load2(smS + (2 * k + 1) * P * 128, &tmSb, k * 64, tile * P, &sh.st_full);
                }
                ++loads_st;
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    if (j > 0) ok = ok && ws_wait(&sh.x_free[s], (j - 1) & 1, fail, 13);
                    if (ok) {
                        mbar_expect_tx(&sh.x_full[s], 8192u);
                        tma_load4(smX + s * 8192, &tmX, 0, it.h, it.c * Q + s * 64, it.b, &sh.x_full[s]);
                        ++loads_x[s];
                    }
                }
                it.next(d, nrt);
            }
            if (!ok) {                                          // leave no load in flight
                if (loads_st) mbar_wait(&sh.st_full, (loads_st - 1) & 1);
                for (int s = 0; s < NS; ++s)
                    if (loads_x[s]) mbar_wait(&sh.x_full[s], (loads_x[s] - 1) & 1);
                if (ngrp) mbar_wait(&sh.grp_full, (ngrp - 1) & 1);
            }
        }
    } else if (warp < kWsFirstBuilder) {
        // ---------------------------------------------------------------------------------------------- epilogue
        const int quarter = warp & 3, ch = ((warp - kWsFirstEpi) >> 2) * 32;   // rows 32*quarter.., columns ch..ch+31
        const uint32_t tl = tmem + ((uint32_t)(quarter * 32) << 16);
        WsIter it;
        it.init(d, nrt, t0);
        bool ok = true;
        WsRows rw{&tmR, smR, 0};
        const bool issuer = warp == kWsFirstEpi;
        const bool rows = a.rows_by_tma != 0;
        if (rows && issuer && lane == 0 && nt > 0) rw.request(sh, d, it, Q);
        if constexpr (MODE == 1) {
            ws_epilogue_dx<T, NS>(d, a, sh, rowred, tl, quarter, ch, lane, it, nt, nrt, fail, rw, issuer);
        } else {
        uint4 zr[4];
        auto load_z = [&](const WsIter &w) {
            const int l = w.rt * kTileM + quarter * 32 + lane;
            const bool live = d.has_z && l < min(Q, d.L - w.c * Q);
            const T *zp = static_cast<const T *>(z.ptr) + w.b * z.sb + (long long)(w.c * Q + l) * z.sl + w.h * z.sh + ch;
            if (!live) {
#pragma unroll
                for (int q = 0; q < 4; ++q) zr[q] = zero8();
            } else if (wide_z) {
#pragma unroll
                for (int q = 0; q < 2; ++q) ldg16(zp + q * 16, zr[2 * q], zr[2 * q + 1]);
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) zr[q] = __ldg(reinterpret_cast<const uint4 *>(zp + q * 8));
            }
        };
        if (nt > 0 && !rows) load_z(it);
        for (int i = 0; i < nt && ok; ++i) {
            const int buf = i & 1;
            if (rows) {                                          // z rows of this tile from the TMA-fed buffer
                WsIter nx = it;
                nx.next(d, nrt);
                ok = ws_rows_step(sh, rw, d, Q, i, nt, nx, issuer, quarter * 32 + lane, ch, lane, zr, fail);
                if (!ok) break;
            }
            const int lim = min(Q, d.L - it.c * Q);
            const int l = it.rt * kTileM + quarter * 32 + lane;
            const long long base = ((long long)(it.b * d.H + it.h) * d.nc + it.c) * Q;
            const bool live = l < lim;
            float ecf = 0.f, ecb = 0.f;
            if (live) {
                ecf = cs_f[base + l];
                ecb = cs_b[base + l];
            }
            const int hh = it.h, bb = it.b, row = it.c * Q + l;
            T *po = static_cast<T *>(out.ptr) + bb * out.sb + (long long)row * out.sl + hh * out.sh + ch;
            T *px = static_cast<T *>(out_x.ptr) + bb * out_x.sb + (long long)row * out_x.sl + hh * out_x.sh + ch;
            ok = ws_wait_warp(&sh.acc_full[buf], (i >> 1) & 1, fail, 21);
            if (!ok) break;
            tc_fence_after();
            const float ef = live ? __expf(ecf) : 0.f, eb = live ? __expf(ecb) : 0.f;
            const uint32_t acc = tl + buf * 3 * P + ch;
#pragma unroll
            for (int c0 = 0; c0 < 32; c0 += 16) {
                uint32_t ry[16], rf[16], rb[16];
                tmem_ld16_nowait(acc + 2 * P + c0, ry);
                tmem_ld16_nowait(acc + c0, rf);
                tmem_ld16_nowait(acc + P + c0, rb);
                tmem_ld_wait();
                if (c0 + 16 >= 32) {                             // the accumulator is free once the last read has landed
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh.acc_free[buf]);
                }
                float y[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    y[j] = fmaf(eb, __uint_as_float(rb[j]), fmaf(ef, __uint_as_float(rf[j]), __uint_as_float(ry[j])));
                if (d.has_D && d.D_hdim && live) {               // per-element D: not folded into M
#pragma unroll
                    for (int j = 0; j < 16; j += 8) {
                        float xv[8];
                        unpack8<T>(ld8v<T>(x, bb, row, hh, ch + c0 + j), xv);
#pragma unroll
                        for (int k = 0; k < 8; ++k) y[j + k] = fmaf(D[hh * P + ch + c0 + j + k], xv[k], y[j + k]);
                    }
                }
                float o0[8], o1[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    o0[k] = y[k];
                    o1[k] = y[8 + k];
                }
                if (d.has_z) {
                    if (live) stg16(px + c0, pack8<T>(o0), pack8<T>(o1), wide_o);
                    float z0[8], z1[8];
                    unpack8<T>(zr[c0 >> 3], z0);
                    unpack8<T>(zr[(c0 >> 3) + 1], z1);
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        o0[k] *= 0.5f * z0[k] * (1.f + tanh_approx(0.5f * z0[k]));
                        o1[k] *= 0.5f * z1[k] * (1.f + tanh_approx(0.5f * z1[k]));
                    }
                }
                if (live) stg16(po + c0, pack8<T>(o0), pack8<T>(o1), wide_o);
            }
            it.next(d, nrt);
            if (i + 1 < nt && !rows) load_z(it);                 // a whole tile ahead of its use
        }
        }
        if (rows && issuer && lane == 0 && sh.fail && rw.issued)  // leave no load in flight
            mbar_wait(&sh.r_full, (rw.issued - 1) & 1);
    } else {
        // ------------------------------------------------------------------------------------------ M builders
        const int bt = tid - 32 * kWsFirstBuilder;               // 0 .. 255
        WsIter it;
        it.init(d, nrt, t0);
        bool ok = true;
        int cur_grp = -1;
        uint32_t ngrp = 0;
        WsRing ring;
        float pcf = 0.f, pcb = 0.f, pdt = 1.f, pD = 0.f;        // next tile's table inputs for entry bt, and its D
        float pr1 = 0.f, pr2 = 0.f;                              // ... and the reference values of its column factors
        const bool fold = MODE == 0 && d.has_D && !d.D_hdim;
        auto fetch_tab = [&](const WsIter &w) {
            if (bt < Q) {
                const long long base = ((long long)(w.b * d.H + w.h) * d.nc + w.c) * Q;
                pcf = cs_f[base + bt];
                pcb = cs_b[base + bt];
                pdt = dt_out[base + bt];
                pr1 = (MODE == 0 ? cs_f : cs_b)[base + (bt | 63)];      // last column of bt's stage
                pr2 = (MODE == 0 ? cs_b : cs_f)[base + (bt & ~63)];     // first column of it
            }
            if (fold) pD = D[w.h];
        };
        auto write_tab = [&](int which) {
            if (bt < Q) {
                float *t = tab + which * 6 * Q;
                const float cf = pcf * 1.4426950408889634f, cb_ = pcb * 1.4426950408889634f;
                const float r1 = pr1 * 1.4426950408889634f, r2 = pr2 * 1.4426950408889634f;
                if constexpr (MODE == 0) {
                    const float lg = __log2f(pdt);               // -inf for the zero-padded tail: those columns vanish
                    t[bt] = cf;
                    t[Q + bt] = cb_;
                    t[2 * Q + bt] = cf - lg;
                    t[3 * Q + bt] = cb_ - lg;
                    t[4 * Q + bt] = ex2_approx(r1 - (cf - lg));  // colF[s] = 2^(F[last column of the stage] - TF[s])
                    t[5 * Q + bt] = ex2_approx(r2 - (cb_ - lg)); // colB[s] = 2^(B[first column of the stage] - TB[s])
                } else {
                    // transposed tile: below the diagonal 2^(b2[s] - b2[l]), above it 2^(f2[s] - f2[l]); with the
                    // tables negated and swapped the builder's forward formulas produce exactly these
                    t[bt] = -cb_;
                    t[Q + bt] = -cf;
                    t[2 * Q + bt] = -cb_;
                    t[3 * Q + bt] = -cf;
                    t[4 * Q + bt] = ex2_approx(cb_ - r1);
                    t[5 * Q + bt] = ex2_approx(cf - r2);
                }
            }
        };
        if (nt > 0) {
            fetch_tab(it);
            write_tab(0);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.tab_bar);
            ok = ws_wait_warp(&sh.tab_bar, 0, fail, 31);
        }
        for (int i = 0; i < nt && ok; ++i) {
            const float dfold = pD;
            const int rt = it.rt;
            const int grp = it.grp;
            it.next(d, nrt);
            if (i + 1 < nt) fetch_tab(it);
            if (grp != cur_grp) {
                ok = ws_wait_warp(&sh.grp_full, ngrp & 1, fail, 32);
                ++ngrp;
                cur_grp = grp;
                if (!ok) break;
            }
            const float *tb_ = tab + (i & 1) * 6 * Q;
            ok = ws_build_tile<T, NST>(smCB, smM, tb_, NS, rt * kTileM, bt, lane, dfold, ring, sh.m_full, sh.m_free, fail);
            if (!ok) break;
            if (i + 1 < nt) {
                write_tab((i + 1) & 1);
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh.tab_bar);
                ok = ws_wait_warp(&sh.tab_bar, (i + 1) & 1, fail, 31);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (sh.fail && tid == 0) atomicExch(status, kErrWsWait + sh.fail);
    if (warp == 0) {
        __syncwarp();
        tmem_dealloc(tmem, ncols);
    }
}

}  // namespace tc
}  // namespace bissd
