// Forward chunk scan, TMA-fed variant (see simt::chunk_scan for the formula).
//
// Per CTA: one (batch, chunk, head) and 128 rows l.  C, the two entering states and x arrive by TMA and stay resident
// in shared memory; the two state products C.S_f^T and C.S_b^T go straight from those tiles into their own TMEM
// accumulators (the row factors e^{cs_f[l]}, e^{cs_b[l]} are applied in the epilogue), and only the masked-decay
// matrix M[l,s] = CB[l,s] Delta[s] (L_f + L_b)[l,s] is built by the threads, 64 columns at a time, in two stage buffers
// that reuse the C / state tiles once those products have completed.  M is evaluated in the log2 domain with
// per-column tables tf[s] = cs_f[s] log2e - log2 Delta[s] (tb likewise): M = CB * 2^(f2[l] - tf[s]) below the
// diagonal, CB * 2^(b2[l] - tb[s]) above it, twice that on it.
//
// Shapes: headdim, dstate multiples of 64, chunk 128 or 256, everything resident must fit (checked on the host).
#pragma once
#include "tc_kernels.cuh"
#include "tc_tma.cuh"

namespace bissd {
namespace tc {

struct ScanShared {
    uint64_t bar_cs, bar_x, bar_st, bar_mid, free_bar[2], done_bar;   // bar_mid: every round of the state products but the last
    uint32_t tmem_base;
    int fail;
};

// The operands of the two state products (C or B rows and both state tiles) take dstate/64 slabs each.  Where all of
// them do not fit beside x (headdim 128 with dstate 256), they come in `rounds` = 2 halves of dstate, the second
// loaded into the same buffers once the MMAs of the first have read them.
inline size_t scan_tma_smem(int P, int N, int Q, int rounds = 1) {
    const size_t nsr = (size_t)(N / 64) / rounds;
    return 1024 + nsr * 16384 + 2 * nsr * P * 128 + (size_t)(P / 64) * Q * 128 + 4 * Q * 4;
}
inline int scan_tma_rounds(int P, int N, int Q) {                // 0: shape not supported
    if (P % 64 || N % 64 || (Q != 128 && Q != 256) || P > 128 || N > 256) return 0;
    for (int rounds = 1; rounds <= 2; ++rounds) {
        if ((N / 64) % rounds) continue;
        const size_t nsr = (size_t)(N / 64) / rounds;
        if (nsr * 16384 + 2 * nsr * P * 128 < 32768) continue;       // room for the two M stages
        if (scan_tma_smem(P, N, Q, rounds) <= 200 * 1024) return rounds;
    }
    return 0;
}
inline bool scan_tma_ok(int P, int N, int Q) { return scan_tma_rounds(P, N, Q) > 0; }

template <class T>
__global__ void __launch_bounds__(kThreads, 2)
chunk_scan_tma(Dims d, const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmSf,
               const __grid_constant__ CUtensorMap tmSb, const __grid_constant__ CUtensorMap tmX, View x, View z,
               const float *D, const float *dt_out, const float *cs_f, const float *cs_b, const float *CB, MutView out,
               MutView out_x, int rounds, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ ScanShared sh;
    const int P = d.P, N = d.N, Q = d.Q;
    const int nsr = N / 64 / rounds, npb = P / 64;            // slabs of 64 dstate columns resident at a time
    uint8_t *base_sm = smem_align1024(dyn);
    uint8_t *smC = base_sm;                                   // nsr slabs [128 x 64]
    uint8_t *smSf = smC + nsr * 16384;                        // nsr slabs [P x 64]
    uint8_t *smSb = smSf + nsr * P * 128;
    uint8_t *smX = smSb + nsr * P * 128;                      // npb blocks [Q x 64]
    float *f2 = reinterpret_cast<float *>(smX + npb * Q * 128), *b2 = f2 + Q, *tf = b2 + Q, *tb = tf + Q;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % d.H, c = (blockIdx.x / d.H) % d.nc, b = blockIdx.x / (d.H * d.nc);
    const int g = h / d.R;
    const int lim = min(Q, d.L - c * Q);
    const int l0 = blockIdx.y * kTileM;
    const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
    const uint32_t ncols = tmem_cols(3 * P);
    if (warp == 0) tmem_alloc(&sh.tmem_base, ncols);
    if (tid == 32) {
        mbar_init(&sh.bar_cs, 1);
        mbar_init(&sh.bar_x, 1);
        mbar_init(&sh.bar_st, 1);
        mbar_init(&sh.bar_mid, 1);
        mbar_init(&sh.free_bar[0], 1);
        mbar_init(&sh.free_bar[1], 1);
        mbar_init(&sh.done_bar, 1);
        sh.fail = 0;
        fence_mbar_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    const int tile = (b * d.nc + c) * d.H + h;
    auto load_round = [&](int rd) {                             // thread 0: one dstate share of C and both states
        mbar_expect_tx(&sh.bar_cs, (uint32_t)(nsr * 16384 + 2 * nsr * P * 128));
        for (int j = 0; j < nsr; ++j) {
            const int n0 = (rd * nsr + j) * 64;
            tma_load4(smC + j * 16384, &tmC, n0, g, c * Q + l0, b, &sh.bar_cs);
            tma_load2(smSf + j * P * 128, &tmSf, n0, tile * P, &sh.bar_cs);
            tma_load2(smSb + j * P * 128, &tmSb, n0, tile * P, &sh.bar_cs);
        }
    };
    if (tid == 0) {
        load_round(0);
        mbar_expect_tx(&sh.bar_x, (uint32_t)(npb * Q * 128));
        for (int j = 0; j < npb; ++j) tma_load4(smX + j * Q * 128, &tmX, j * 64, h, c * Q, b, &sh.bar_x);
    }
    const float *cbt = CB + ((long long)(b * d.nc + c) * d.G + g) * Q * Q;
    // the decay tables are built while the TMA loads are in flight
    for (int i = tid; i < Q; i += kThreads) {
        const float cf = cs_f[base + i] * 1.4426950408889634f, cb_ = cs_b[base + i] * 1.4426950408889634f;
        const float lg = __log2f(dt_out[base + i]);           // -inf for the zero-padded tail: those columns vanish
        f2[i] = cf;
        b2[i] = cb_;
        tf[i] = cf - lg;
        tb[i] = cb_ - lg;
    }
    __syncthreads();
    uint4 ra[4];
    float4 raw[8];                                              // CB values of the step after next, still in flight
    auto load_raw = [&](int s0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int q = tid + i * kThreads;
            const float *src = cbt + (long long)(l0 + (q >> 3)) * Q + s0 + (q & 7) * 8;
            raw[2 * i] = __ldg(reinterpret_cast<const float4 *>(src));
            raw[2 * i + 1] = __ldg(reinterpret_cast<const float4 *>(src) + 1);
        }
    };
    auto fetch = [&](int s0) {                                  // this thread's four 8-column pieces of M[:, s0:s0+64]
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int q = tid + i * kThreads;
            const int l = l0 + (q >> 3), sc = s0 + (q & 7) * 8;
            float v[8] = {raw[2 * i].x, raw[2 * i].y, raw[2 * i].z, raw[2 * i].w,
                          raw[2 * i + 1].x, raw[2 * i + 1].y, raw[2 * i + 1].z, raw[2 * i + 1].w};
            const float fl = f2[l], bl = b2[l];
            if (sc + 7 < l) {
                const float4 t0 = *reinterpret_cast<const float4 *>(tf + sc), t1 = *reinterpret_cast<const float4 *>(tf + sc + 4);
                const float t[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= ex2_approx(fl - t[j]);
            } else if (sc > l) {
                const float4 t0 = *reinterpret_cast<const float4 *>(tb + sc), t1 = *reinterpret_cast<const float4 *>(tb + sc + 4);
                const float t[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= ex2_approx(bl - t[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int s = sc + j;
                    float w = ex2_approx(s <= l ? fl - tf[s] : bl - tb[s]);
                    if (s == l) w *= 2.f;
                    v[j] *= w;
                }
            }
            ra[i] = pack8<T>(v);
        }
    };
    load_raw(0);
    fetch(0);
    if (kStageK < Q) load_raw(kStageK);
    bool ok = true;
    if (tid == 0) {                                             // the two state products, straight from the TMA tiles
        const uint32_t idesc = instr_desc(AbFmt<T>::v, false, false, P);
        for (int rd = 0; rd < rounds; ++rd) {                   // bar_cs completes once per round, bar_st with the last one only
            if (rd > 0) {                                       // the MMAs of the round before have read the tiles
                if (!mbar_wait(&sh.bar_mid, (rd - 1) & 1)) {
                    sh.fail = 1;
                    break;
                }
                load_round(rd);
            }
            if (!mbar_wait(&sh.bar_cs, rd & 1)) {
                sh.fail = 1;
                break;
            }
            tc_fence_after();
            for (int dir = 0; dir < 2; ++dir)
                for (int j = 0; j < nsr; ++j)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma(tmem + dir * P, smem_desc(smem_u32(smC + j * 16384) + kk * 32, 16, 1024),
                             smem_desc(smem_u32((dir ? smSb : smSf) + j * P * 128) + kk * 32, 16, 1024), idesc,
                             (rd > 0 || j > 0 || kk > 0) ? 1u : 0u);
            umma_commit(rd + 1 < rounds ? &sh.bar_mid : &sh.bar_st);
        }
    }
    uint32_t it = 0;
    for (int s0 = 0; s0 < Q; s0 += kStageK, ++it) {
        const int st = it & 1;
        uint8_t *stage = base_sm + st * kAStageBytes;           // reuses the C / state tiles
        ok = (it < 2) ? mbar_wait(&sh.bar_st, 0) : mbar_wait(&sh.free_bar[st], ((it >> 1) - 1) & 1);
        if (ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int q = tid + i * kThreads;
                const int r = q >> 3, cc = q & 7;
                *reinterpret_cast<uint4 *>(stage + r * 128 + ((cc ^ (r & 7)) << 4)) = ra[i];
            }
            fence_async_smem();
            if (s0 + kStageK < Q) fetch(s0 + kStageK);
            if (s0 + 2 * kStageK < Q) load_raw(s0 + 2 * kStageK);
        }
        ok = __syncthreads_and(ok) && !sh.fail;
        if (!ok) break;
        if (tid == 0) {
            bool xok = (it > 0) || mbar_wait(&sh.bar_x, 0);
            if (xok) {
                tc_fence_after();
                const uint32_t idesc = instr_desc(AbFmt<T>::v, false, true, P);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma(tmem + 2 * P, smem_desc(smem_u32(stage) + kk * 32, 16, 1024),
                         smem_desc(smem_u32(smX) + (s0 + kk * 16) * 128, (uint32_t)Q * 128, 1024), idesc,
                         (s0 > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&sh.free_bar[st]);
            } else {
                sh.fail = 1;
            }
        }
    }
    // epilogue operands of the first strip are requested before waiting for the last MMAs
    const int el = l0 + (warp & 3) * 32 + lane, ec0 = (warp >> 2) * 32;
    uint4 xr[4], zr[4];
    float ecf = 0.f, ecb = 0.f;
    if (ok && el < lim) {
        ecf = cs_f[base + el];
        ecb = cs_b[base + el];
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        xr[q] = (ok && el < lim && d.has_D && ec0 < P) ? ld8v<T>(x, b, c * Q + el, h, ec0 + q * 8) : zero8();
        zr[q] = (ok && el < lim && d.has_z && ec0 < P) ? ld8v<T>(z, b, c * Q + el, h, ec0 + q * 8) : zero8();
    }
    if (ok) {
        if (tid == 0) umma_commit(&sh.done_bar);
        ok = mbar_wait(&sh.done_bar, 0);
        ok = __syncthreads_and(ok) && !sh.fail;
        tc_fence_after();
    }
    if (!ok && tid == 0) atomicExch(status, kErrMmaTimeout);
    if (ok) {
        const int l = l0 + (warp & 3) * 32 + lane;
        const float ef = (l < lim) ? __expf(ecf) : 0.f, eb = (l < lim) ? __expf(ecb) : 0.f;
        const uint32_t tl = tmem_lane_base(tmem);
        for (int c0 = (warp >> 2) * 32; c0 < P; c0 += 64) {
            // all global operands of this strip are requested before anything is consumed: one round trip, not eight
            if (c0 != ec0) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    xr[q] = (l < lim && d.has_D) ? ld8v<T>(x, b, c * Q + l, h, c0 + q * 8) : zero8();
                    zr[q] = (l < lim && d.has_z) ? ld8v<T>(z, b, c * Q + l, h, c0 + q * 8) : zero8();
                }
            }
            float y[32], v[32];
            tmem_ld32(tl + 2 * P + c0, y);
            tmem_ld32(tl + c0, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) y[j] = fmaf(ef, v[j], y[j]);
            tmem_ld32(tl + P + c0, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) y[j] = fmaf(eb, v[j], y[j]);
            if (l < lim) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    const int p0 = c0 + j;
                    float o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = y[j + i];
                    if (d.has_D) {
                        float xv[8];
                        unpack8<T>(xr[j >> 3], xv);
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] = fmaf(d.D_hdim ? D[h * P + p0 + i] : D[h], xv[i], o[i]);
                    }
                    const long long oo = b * out.sb + (long long)(c * Q + l) * out.sl + h * out.sh + p0;
                    if (d.has_z) {
                        const long long ox = b * out_x.sb + (long long)(c * Q + l) * out_x.sl + h * out_x.sh + p0;
                        *reinterpret_cast<uint4 *>(static_cast<T *>(out_x.ptr) + ox) = pack8<T>(o);
                        float zz[8];
                        unpack8<T>(zr[j >> 3], zz);
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] *= __fdividef(zz[i], 1.f + __expf(-zz[i]));
                    }
                    *reinterpret_cast<uint4 *>(static_cast<T *>(out.ptr) + oo) = pack8<T>(o);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, ncols);
}

}  // namespace tc
}  // namespace bissd
