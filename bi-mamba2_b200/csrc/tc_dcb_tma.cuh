// dCB[l,s] = sum_{h in group} (g_h[l].x_h[s]) Delta_h[s] ([s<=l] e^{cs_f[l]-cs_f[s]} + [s>=l] e^{cs_b[l]-cs_b[s]}),
// TMA-fed and software-pipelined over the heads of a group (see simt::dcb_kernel for the reference line numbers).
//
// Per CTA: one (batch, chunk, group), a 128 x 128 tile of (l, s).  For every head the g and x tiles arrive by TMA into a
// three-deep ring; G2_h = g_h x_h^T goes into one of two TMEM accumulators, so the MMA of head h+1 runs while the
// threads weight head h with its decay factors and add it to the running sum they keep in registers.  The factors:
// log2-domain tables per head (double buffered; their inputs are fetched two heads ahead, the tables written one head
// ahead).  A 16-column strip that lies wholly on one side of the diagonal of all 32 rows of a warp uses the factorised
// form  2^(f2[l] - tf[s]) = 2^(f2[l] - f2[ref]) * 2^(f2[ref] - tf[s])  with ref the strip's last column (first column
// and the b tables on the other side): one ex2 per row and strip plus a per-column table entry, both exponents <= 0.
#pragma once
#include "tc_scan_tma.cuh"

namespace bissd {
namespace tc {

struct DcbShared {
    uint64_t full[3], mma_done[2];
    uint32_t tmem_base;
};

inline size_t dcb_tma_smem(int P, int Q) { return 1024 + 3 * 2 * (size_t)(P / 64) * 16384 + 2 * 6 * (size_t)Q * 4; }

template <class T>
__global__ void __launch_bounds__(kThreads, 2)
dcb_tma(Dims d, const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmX, const float *dt_out,
        const float *cs_f, const float *cs_b, float *dCB, void *dCB16, int *status) {
    pdl_begin();
    extern __shared__ uint8_t dyn[];
    __shared__ DcbShared sh;
    const int P = d.P, Q = d.Q, R = d.R;
    const int npb = P / 64;
    const int stage_bytes = 2 * npb * 16384;
    uint8_t *base_sm = smem_align1024(dyn);
    float *tabs = reinterpret_cast<float *>(base_sm + 3 * stage_bytes);          // [2][6][Q]: f2, b2, tf, tb, colF, colB
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = blockIdx.x % d.G, c = (blockIdx.x / d.G) % d.nc, b = blockIdx.x / (d.G * d.nc);
    const int l0 = blockIdx.y * kTileM, s0 = blockIdx.z * 128;
    const int quad = warp & 3, half = warp >> 2;
    const int l = l0 + quad * 32 + lane;
    const int wl_min = l0 + quad * 32, wl_max = wl_min + 31;
    if (warp == 0) tmem_alloc(&sh.tmem_base, 256);
    if (tid == 32) {
        for (int i = 0; i < 3; ++i) mbar_init(&sh.full[i], 1);
        mbar_init(&sh.mma_done[0], 1);
        mbar_init(&sh.mma_done[1], 1);
        fence_mbar_init();
    }
    // table entry tid of head hr: inputs into registers (fetch_tab), table written later (write_tab)
    float pcf = 0.f, pcb = 0.f, pdt = 1.f, pcfr = 0.f, pcbr = 0.f;
    auto fetch_tab = [&](int hr) {
        const int h = g * R + hr;
        const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
        if (tid < Q) {
            pcf = cs_f[base + tid];
            pcb = cs_b[base + tid];
            pdt = dt_out[base + tid];
            pcfr = cs_f[base + (tid | 15)];                     // reference columns of the factorised form
            pcbr = cs_b[base + (tid & ~15)];
        }
    };
    auto write_tab = [&](int hr) {
        float *t = tabs + (hr & 1) * 6 * Q;
        if (tid < Q) {
            const float cf = pcf * 1.4426950408889634f, cb_ = pcb * 1.4426950408889634f;
            const float lg = __log2f(pdt);
            t[tid] = cf;
            t[Q + tid] = cb_;
            t[2 * Q + tid] = cf - lg;
            t[3 * Q + tid] = cb_ - lg;
            t[4 * Q + tid] = ex2_approx(pcfr * 1.4426950408889634f - (cf - lg));
            t[5 * Q + tid] = ex2_approx(pcbr * 1.4426950408889634f - (cb_ - lg));
        }
    };
    auto load_head = [&](int hr) {                              // thread 0: both tiles of head hr into ring slot hr % 3
        const int h = g * R + hr, slot = hr % 3;
        uint8_t *sg = base_sm + slot * stage_bytes, *sx = sg + npb * 16384;
        mbar_expect_tx(&sh.full[slot], (uint32_t)stage_bytes);
        for (int j = 0; j < npb; ++j) {
            tma_load4(sg + j * 16384, &tmG, j * 64, h, c * Q + l0, b, &sh.full[slot]);
            tma_load4(sx + j * 16384, &tmX, j * 64, h, c * Q + s0, b, &sh.full[slot]);
        }
    };
    auto issue_head = [&](int hr, uint32_t tmem) -> bool {      // thread 0: G2 of head hr into accumulator hr & 1
        const int slot = hr % 3;
        if (!mbar_wait(&sh.full[slot], (hr / 3) & 1)) return false;
        tc_fence_after();
        const uint8_t *sg = base_sm + slot * stage_bytes, *sx = sg + npb * 16384;
        const uint32_t idesc = instr_desc(AbFmt<T>::v, false, false, 128);
        for (int j = 0; j < npb; ++j)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma(tmem + (hr & 1) * 128, smem_desc(smem_u32(sg + j * 16384) + kk * 32, 16, 1024),
                     smem_desc(smem_u32(sx + j * 16384) + kk * 32, 16, 1024), idesc, (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&sh.mma_done[hr & 1]);
        return true;
    };
    fetch_tab(0);
    write_tab(0);
    if (R > 1) fetch_tab(1);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    bool ok = true;
    if (tid == 0) {
        for (int hr = 0; hr < 3 && hr < R; ++hr) load_head(hr);
        ok = issue_head(0, tmem);
    }
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    const uint32_t tl = tmem_lane_base(tmem);
#pragma unroll 1
    for (int hr = 0; hr < R; ++hr) {
        if (tid == 0 && ok && hr + 1 < R) ok = issue_head(hr + 1, tmem);
        if (hr + 1 < R) {
            write_tab(hr + 1);
            if (hr + 2 < R) fetch_tab(hr + 2);
        }
        if (ok) ok = mbar_wait(&sh.mma_done[hr & 1], (hr >> 1) & 1);
        if (ok) {
            tc_fence_after();
            const float *t = tabs + (hr & 1) * 6 * Q;
            const float fl = t[min(l, Q - 1)], bl = t[Q + min(l, Q - 1)];
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {                    // four 16-column strips per thread
                const int c0 = half * 32 + (ch >> 1) * 64 + (ch & 1) * 16;
                const int sb0 = s0 + c0;
                float v[16];
                tmem_ld16(tl + (hr & 1) * 128 + c0, v);
                if (sb0 + 15 < wl_min) {                        // whole strip left of the diagonal for every row here
                    const float rf = ex2_approx(fl - t[sb0 + 15]);
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[ch * 16 + j] = fmaf(v[j] * t[4 * Q + sb0 + j], rf, acc[ch * 16 + j]);
                } else if (sb0 > wl_max) {                      // whole strip right of it
                    const float rb = ex2_approx(bl - t[Q + sb0]);
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[ch * 16 + j] = fmaf(v[j] * t[5 * Q + sb0 + j], rb, acc[ch * 16 + j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int s = sb0 + j;
                        float a = (s <= l) ? fl - t[2 * Q + s] : bl - t[3 * Q + s];
                        if (s == l) a += 1.f;                   // the diagonal counts once per direction
                        acc[ch * 16 + j] = fmaf(v[j], ex2_approx(a), acc[ch * 16 + j]);
                    }
                }
            }
        }
        if (tid == 0 && ok && hr + 3 < R) load_head(hr + 3);   // slot hr % 3 is free: the MMA that read it has completed
        tc_fence_before();
        ok = __syncthreads_and(ok);
        if (!ok) break;
    }
    if (!ok && tid == 0) atomicExch(status, kErrMmaTimeout);
    if (ok && l < Q && dCB16) {                                 // the rounded copy bmm_bwd_tma multiplies with; zero outside the sequence
        const int lim = min(Q, d.L - c * Q);
        T *out = static_cast<T *>(dCB16) + ((long long)(b * d.nc + c) * d.G + g) * Q * Q + (long long)l * Q + s0;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            const int c0 = half * 32 + (ch >> 1) * 64 + (ch & 1) * 16;
#pragma unroll
            for (int j = 0; j < 16; j += 8) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = (l < lim && s0 + c0 + j + i < lim) ? acc[ch * 16 + j + i] : 0.f;
                *reinterpret_cast<uint4 *>(out + c0 + j) = pack8<T>(o);
            }
        }
    } else if (ok && l < Q) {
        float *out = dCB + ((long long)(b * d.nc + c) * d.G + g) * Q * Q + (long long)l * Q + s0;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            const int c0 = half * 32 + (ch >> 1) * 64 + (ch & 1) * 16;
#pragma unroll
            for (int j = 0; j < 16; j += 4)
                *reinterpret_cast<float4 *>(out + c0 + j) =
                    make_float4(acc[ch * 16 + j], acc[ch * 16 + j + 1], acc[ch * 16 + j + 2], acc[ch * 16 + j + 3]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------------------
// dB[s,n] = sum_l dCB[l,s] C[l,n] + dB_part[s,n];  dC[l,n] = sum_s dCB[l,s] B[s,n] + dC_part[l,n]   (see simt::bmm_bwd),
// from the 16-bit copy of dCB that dcb_tma writes (the reference's kernel rounds dCB to the input type as well).
// One shot per CTA: 128 output rows x 64 state columns; both operands by TMA - dCB once as [l x 128 s] (MN-major,
// for dB) or as [128 l x s] (K-major, for dC), B or C as [Q rows x 64 n] (MN-major) - then Q/16 MMAs and the
// epilogue that adds the per-group partial sums of dbc_accum.   grid (b*nc*G*2, Q/128, N/64); two CTAs per SM.
inline bool bmm_bwd_tma_ok(int N, int Q) { return N % 64 == 0 && (Q == 128 || Q == 256); }
inline size_t bmm_bwd_tma_smem(int Q) { return 1024 + (size_t)Q * 256 + (size_t)Q * 128; }

template <class T>
__global__ void __launch_bounds__(kThreads, 2)
bmm_bwd_tma(Dims d, const __grid_constant__ CUtensorMap tmDm, const __grid_constant__ CUtensorMap tmDk,
            const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC, const float *dB_part,
            const float *dC_part, int part_heads, void *dB, void *dC, int *status) {
    pdl_begin();
    extern __shared__ uint8_t dyn[];
    __shared__ uint64_t bar_in, bar_done;
    __shared__ uint32_t tmem_slot;
    const int N = d.N, Q = d.Q;
    uint8_t *smA = smem_align1024(dyn), *smB = smA + Q * 256;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int which = blockIdx.x & 1, bx = blockIdx.x >> 1;
    const int g = bx % d.G, c = (bx / d.G) % d.nc, b = bx / (d.G * d.nc);
    const int lim = min(Q, d.L - c * Q);
    const int r0 = blockIdx.y * kTileM, n0 = blockIdx.z * 64;
    if (warp == 0) tmem_alloc(&tmem_slot, 64);
    if (tid == 32) {                                            // barriers and loads by the same thread, before the sync
        mbar_init(&bar_in, 1);
        mbar_init(&bar_done, 1);
        fence_mbar_init();
        const int row0 = ((b * d.nc + c) * d.G + g) * Q;        // first row of this group's dCB
        mbar_expect_tx(&bar_in, (uint32_t)(Q * 256 + Q * 128));
        if (which == 0)
            for (int j = 0; j < 2; ++j) tma_load2(smA + j * Q * 128, &tmDm, r0 + j * 64, row0, &bar_in);
        else
            for (int j = 0; j < Q / 64; ++j) tma_load2(smA + j * 16384, &tmDk, j * 64, row0 + r0, &bar_in);
        for (int rb = 0; rb < Q / 128; ++rb) tma_load4(smB + rb * 16384, which ? &tmB : &tmC, n0, g, c * Q + rb * 128, b, &bar_in);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    bool ok = true;
    if (tid == 0) {
        ok = mbar_wait(&bar_in, 0);
        if (ok) {
            tc_fence_after();
            const uint32_t idesc = instr_desc(AbFmt<T>::v, which == 0, true, 64);
            for (int kk = 0; kk < Q / 16; ++kk) {
                const uint64_t da = which == 0 ? smem_desc(smem_u32(smA) + kk * 2048, (uint32_t)Q * 128, 1024)
                                               : smem_desc(smem_u32(smA) + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                umma(tmem, da, smem_desc(smem_u32(smB) + kk * 2048, (uint32_t)Q * 128, 1024), idesc, kk > 0 ? 1u : 0u);
            }
            umma_commit(&bar_done);
        }
    }
    const int row = r0 + (warp & 3) * 32 + lane, c0 = (warp >> 2) * 32;
    const int rp = part_heads / d.G;
    const float *part = (which ? dC_part : dB_part) + (((long long)b * d.nc * Q + c * Q + row) * part_heads + g * rp) * N + n0 + c0;
    float o[32];                                                // the partial sums are on their way while the MMAs run
#pragma unroll
    for (int j = 0; j < 32; ++j) o[j] = 0.f;
    if (row < lim)
        for (int q = 0; q < rp; ++q)
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 t = *reinterpret_cast<const float4 *>(part + (long long)q * N + j);
                o[j] += t.x, o[j + 1] += t.y, o[j + 2] += t.z, o[j + 3] += t.w;
            }
    if (ok) ok = mbar_wait(&bar_done, 0);
    ok = __syncthreads_and(ok);
    tc_fence_after();
    if (!ok && tid == 0) atomicExch(status, kErrMmaTimeout);
    if (ok) {
        float v[32];
        tmem_ld32(tmem_lane_base(tmem) + c0, v);
        if (row < lim) {
            T *out = static_cast<T *>(which ? dC : dB) + (((long long)b * d.L + c * Q + row) * d.G + g) * N + n0 + c0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                float t[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) t[i] = v[j + i] + o[j + i];
                *reinterpret_cast<uint4 *>(out + j) = pack8<T>(t);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 64);
}

}  // namespace tc
}  // namespace bissd
