// Backward, TMA-fed: the gate kernel (g = dout * silu(z), dz) and the fused dx / ddt_out / dD / "next"-term kernel.
//
// dx_tma mirrors chunk_scan_tma: B (as the A operand), the two passed state gradients E_f / E_b and g arrive by TMA
// and stay resident; B.E_f^T and B.E_b^T get their own TMEM accumulators and their row factors e^{T-cs[l]} in the
// epilogue - which also yields the "next" decay terms nf / nb for free; only the transposed masked-decay matrix
// Mt[l,s] = CB[s,l] ([s>l] 2^(f2[s]-f2[l]) + [s<l] 2^(b2[s]-b2[l]) + 2[s=l]) is built by the threads, from a
// transposed copy of CB.
#pragma once
#include "tc_scan_tma.cuh"

namespace bissd {
namespace tc {

// g = dout * z * sigmoid(z), dz = dout * out_x * sigmoid(z) * (1 + z (1 - sigmoid(z))); 8 elements per thread.
// Takes over _chunk_scan_bwd_dz_kernel (src/ssd/bi/ssd_chunk_scan.py:357-440) except its dD partials.
template <class T>
__global__ void __launch_bounds__(256) gate_bwd(Dims d, View dout, View z, View out_x, void *g_out, void *dz) {
    pdl_begin();
    const long long pc = d.P / 8;
    const long long total = (long long)d.b * d.L * d.H * pc;
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const int p0 = (int)(i % pc) * 8;
    const long long r = i / pc;
    const int h = (int)(r % d.H);
    const long long bl = r / d.H;
    const int l = (int)(bl % d.L), b = (int)(bl / d.L);
    float gv[8], zz[8], ox[8], dzv[8];
    unpack8<T>(ld8v<T>(dout, b, l, h, p0), gv);
    unpack8<T>(ld8v<T>(z, b, l, h, p0), zz);
    unpack8<T>(ld8v<T>(out_x, b, l, h, p0), ox);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float sg = __fdividef(1.f, 1.f + __expf(-zz[j]));
        dzv[j] = gv[j] * ox[j] * sg * (1.f + zz[j] * (1.f - sg));
        gv[j] *= zz[j] * sg;
    }
    const long long o = ((long long)(b * d.L + l) * d.H + h) * d.P + p0;
    *reinterpret_cast<uint4 *>(static_cast<T *>(g_out) + o) = pack8<T>(gv);
    *reinterpret_cast<uint4 *>(static_cast<T *>(dz) + o) = pack8<T>(dzv);
}

inline size_t dx_tma_smem(int P, int N, int Q, int rounds = 1) {   // rounds: see scan_tma_rounds
    const size_t nsr = (size_t)(N / 64) / rounds;
    return 1024 + nsr * 16384 + 2 * nsr * P * 128 + (size_t)(P / 64) * Q * 128 + 2 * Q * 4;
}

// grid (b*nc*H, Q/128).  g: contiguous (b,L,H,P) gated output gradient (dout itself when there is no z).
template <class T>
__global__ void __launch_bounds__(kThreads, 2)
dx_tma(Dims d, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmEf,
       const __grid_constant__ CUtensorMap tmEb, const __grid_constant__ CUtensorMap tmG, View x, View g, const float *D,
       const float *dt_out, const float *cs_f, const float *cs_b, const float *CBt, void *dx, float *ddt_out, float *nf,
       float *nb, float *dDpart, int rounds, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ ScanShared sh;
    __shared__ float rowred[3][kTileM];
    __shared__ float colred[4][128];
    const int P = d.P, N = d.N, Q = d.Q;
    const int nsr = N / 64 / rounds, npb = P / 64;            // slabs of 64 dstate columns resident at a time
    uint8_t *base_sm = smem_align1024(dyn);
    uint8_t *smB = base_sm;
    uint8_t *smEf = smB + nsr * 16384;
    uint8_t *smEb = smEf + nsr * P * 128;
    uint8_t *smG = smEb + nsr * P * 128;
    float *f2 = reinterpret_cast<float *>(smG + npb * Q * 128), *b2 = f2 + Q;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % d.H, c = (blockIdx.x / d.H) % d.nc, b = blockIdx.x / (d.H * d.nc);
    const int grp = h / d.R;
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
    auto load_round = [&](int rd) {                             // thread 0: one dstate share of B and both state gradients
        mbar_expect_tx(&sh.bar_cs, (uint32_t)(nsr * 16384 + 2 * nsr * P * 128));
        for (int j = 0; j < nsr; ++j) {
            const int n0 = (rd * nsr + j) * 64;
            tma_load4(smB + j * 16384, &tmB, n0, grp, c * Q + l0, b, &sh.bar_cs);
            tma_load2(smEf + j * P * 128, &tmEf, n0, tile * P, &sh.bar_cs);
            tma_load2(smEb + j * P * 128, &tmEb, n0, tile * P, &sh.bar_cs);
        }
    };
    if (tid == 0) {
        load_round(0);
        mbar_expect_tx(&sh.bar_x, (uint32_t)(npb * Q * 128));
        for (int j = 0; j < npb; ++j) tma_load4(smG + j * Q * 128, &tmG, j * 64, h, c * Q, b, &sh.bar_x);
    }
    const float *cbt = CBt + ((long long)(b * d.nc + c) * d.G + grp) * Q * Q;
    // the decay tables are built while the TMA loads are in flight
    for (int i = tid; i < Q; i += kThreads) {
        f2[i] = cs_f[base + i] * 1.4426950408889634f;
        b2[i] = cs_b[base + i] * 1.4426950408889634f;
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
    auto fetch = [&](int s0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int q = tid + i * kThreads;
            const int l = l0 + (q >> 3), sc = s0 + (q & 7) * 8;
            float v[8] = {raw[2 * i].x, raw[2 * i].y, raw[2 * i].z, raw[2 * i].w,
                          raw[2 * i + 1].x, raw[2 * i + 1].y, raw[2 * i + 1].z, raw[2 * i + 1].w};
            const float fl = f2[l], bl = b2[l];
            if (sc > l) {
                const float4 t0 = *reinterpret_cast<const float4 *>(f2 + sc), t1 = *reinterpret_cast<const float4 *>(f2 + sc + 4);
                const float t[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= ex2_approx(t[j] - fl);
            } else if (sc + 7 < l) {
                const float4 t0 = *reinterpret_cast<const float4 *>(b2 + sc), t1 = *reinterpret_cast<const float4 *>(b2 + sc + 4);
                const float t[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= ex2_approx(t[j] - bl);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int s = sc + j;
                    float w = ex2_approx(s >= l ? f2[s] - fl : b2[s] - bl);
                    if (s == l) w = 2.f;
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
    if (tid == 0) {
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
                        umma(tmem + dir * P, smem_desc(smem_u32(smB + j * 16384) + kk * 32, 16, 1024),
                             smem_desc(smem_u32((dir ? smEb : smEf) + j * P * 128) + kk * 32, 16, 1024), idesc,
                             (rd > 0 || j > 0 || kk > 0) ? 1u : 0u);
            umma_commit(rd + 1 < rounds ? &sh.bar_mid : &sh.bar_st);
        }
    }
    uint32_t it = 0;
    for (int s0 = 0; s0 < Q; s0 += kStageK, ++it) {
        const int st = it & 1;
        uint8_t *stage = base_sm + st * kAStageBytes;
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
                         smem_desc(smem_u32(smG) + (s0 + kk * 16) * 128, (uint32_t)Q * 128, 1024), idesc,
                         (s0 > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&sh.free_bar[st]);
            } else {
                sh.fail = 1;
            }
        }
    }
    // epilogue operands of the first strip are requested before waiting for the last MMAs
    const int el = l0 + (warp & 3) * 32 + lane, ec0 = (warp >> 2) * 32;
    uint4 xr[4], gr[4];
    float e_dl = 0.f, e_cf = 0.f, e_cb = 0.f, e_tf = 0.f, e_tb = 0.f;
    if (ok && el < lim) {
        e_dl = dt_out[base + el];
        e_cf = cs_f[base + el];
        e_cb = cs_b[base + el];
        e_tf = cs_f[base + Q - 1];
        e_tb = cs_b[base];
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        xr[q] = (ok && el < lim && ec0 < P) ? ld8v<T>(x, b, c * Q + el, h, ec0 + q * 8) : zero8();
        gr[q] = (ok && el < lim && ec0 < P) ? ld8v<T>(g, b, c * Q + el, h, ec0 + q * 8) : zero8();
    }
    if (ok) {
        if (tid == 0) umma_commit(&sh.done_bar);
        ok = mbar_wait(&sh.done_bar, 0);
        ok = __syncthreads_and(ok) && !sh.fail;
        tc_fence_after();
    }
    if (!ok && tid == 0) atomicExch(status, kErrMmaTimeout);
    const int quad = warp & 3, half = warp >> 2;
    const int r = quad * 32 + lane, l = l0 + r;
    float rs = 0.f, rsf = 0.f, rsb = 0.f;
    float wf = 0.f, wb = 0.f, dl = 0.f;
    if (ok) {
        if (l < lim) {
            dl = e_dl;
            wf = __expf(e_tf - e_cf);
            wb = __expf(e_tb - e_cb);
        }
        const uint32_t tl = tmem_lane_base(tmem);
        for (int c0 = half * 32; c0 < P; c0 += 64) {
            if (c0 != ec0) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    xr[q] = (l < lim) ? ld8v<T>(x, b, c * Q + l, h, c0 + q * 8) : zero8();
                    gr[q] = (l < lim) ? ld8v<T>(g, b, c * Q + l, h, c0 + q * 8) : zero8();
                }
            }
#pragma unroll
            for (int hs = 0; hs < 2; ++hs) {                    // two 16-column pieces keep the register footprint down
                const int cc = c0 + hs * 16;
                float af[16], ab[16], ai[16];
                tmem_ld16(tl + cc, af);
                tmem_ld16(tl + P + cc, ab);
                tmem_ld16(tl + 2 * P + cc, ai);
#pragma unroll
                for (int j = 0; j < 16; j += 8) {
                    const int p0 = cc + j;
                    float xv[8], gv[8], o[8], gx[8];
                    unpack8<T>(xr[hs * 2 + (j >> 3)], xv);
                    unpack8<T>(gr[hs * 2 + (j >> 3)], gv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float a = fmaf(wf, af[j + i], fmaf(wb, ab[j + i], ai[j + i]));
                        o[i] = a * dl;
                        if (d.has_D) o[i] = fmaf(d.D_hdim ? D[h * P + p0 + i] : D[h], gv[i], o[i]);
                        rs = fmaf(a, xv[i], rs);
                        rsf = fmaf(af[j + i], xv[i], rsf);
                        rsb = fmaf(ab[j + i], xv[i], rsb);
                        gx[i] = gv[i] * xv[i];
                    }
                    if (l < lim)
                        *reinterpret_cast<uint4 *>(static_cast<T *>(dx) + ((long long)(b * d.L + c * Q + l) * d.H + h) * P + p0) = pack8<T>(o);
                    if (d.has_D) {                              // column sums of g*x over this warp's 32 rows
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float sgx = gx[i];
#pragma unroll
                            for (int o2 = 16; o2 > 0; o2 >>= 1) sgx += __shfl_xor_sync(0xffffffffu, sgx, o2);
                            if (lane == 0) colred[quad][p0 + i] = sgx;
                        }
                    }
                }
            }
        }
    }
    if (half == 1) {
        rowred[0][r] = rs;
        rowred[1][r] = rsf;
        rowred[2][r] = rsb;
    }
    tc_fence_before();
    __syncthreads();
    if (ok) {
        if (half == 0 && l < Q) {
            const float hrs = (P > 32) ? rowred[0][r] : 0.f, hf = (P > 32) ? rowred[1][r] : 0.f, hb = (P > 32) ? rowred[2][r] : 0.f;
            ddt_out[base + l] = rs + hrs;
            nf[base + l] = dl * wf * (rsf + hf);
            nb[base + l] = dl * wb * (rsb + hb);
        }
        if (d.has_D && tid < P)
            dDpart[(((long long)(b * d.nc + c) * d.H + h) * gridDim.y + blockIdx.y) * P + tid] =
                colred[0][tid] + colred[1][tid] + colred[2][tid] + colred[3][tid];
    }
    if (warp == 0) tmem_dealloc(tmem, ncols);
}

}  // namespace tc
}  // namespace bissd
