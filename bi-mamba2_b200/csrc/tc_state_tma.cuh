// Local chunk states / local state gradients, TMA-fed (see tc::state_gemm for the thread-staged version and
// simt::chunk_state / simt::dstates for the formulae):
//   MODE 0: out[dir][p][n] = sum_l B[l,n] (x[l,p] Delta[l] e^{T-cs_dir[l]})
//   MODE 1: out[dir][p][n] = sum_l C[l,n] (g[l,p] e^{cs_dir[l]})
// Per CTA: one (batch, chunk, head), one direction, 128 state columns n.  Both operand tiles arrive by TMA with the
// sequence index as their row (= K) index, i.e. as MN-major operands; the per-row factor is applied IN PLACE to the
// smaller one (the [Q x headdim] x / g tile) by the threads, and one thread then issues the Q/16 MMAs.
// Needs dstate % 128 == 0, headdim % 64 == 0, chunk in {128, 256}.
#pragma once
#include "tc_scan_tma.cuh"

namespace bissd {
namespace tc {

// 8 packed 16-bit values times one factor.  bf16: packed multiply with the factor rounded to bf16 first (a quarter of
// the instructions of the fp32 route); f16: through fp32, where small factors do not underflow.
template <class T> __device__ __forceinline__ uint4 scale8_packed(uint4 u, float s) { return scale8<T>(u, s); }
template <> __device__ __forceinline__ uint4 scale8_packed<__nv_bfloat16>(uint4 u, float s) {
    const __nv_bfloat162 f = __float2bfloat162_rn(s);
    uint32_t in[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&in[k]), f);
        in[k] = *reinterpret_cast<const uint32_t *>(&v);
    }
    return make_uint4(in[0], in[1], in[2], in[3]);
}

inline bool state_tma_ok(int P, int N, int Q) {
    return P % 64 == 0 && P <= 128 && N % 128 == 0 && N <= 256 && (Q == 128 || Q == 256);
}
inline size_t state_tma_smem(int P, int Q) { return 1024 + 2 * (size_t)Q * 128 + (size_t)(P / 64) * Q * 128 + Q * 4; }

// grid (b*nc*H, 2, N/128)
template <class T, int MODE>
__global__ void __launch_bounds__(kThreads, 2)
state_gemm_tma(Dims d, const __grid_constant__ CUtensorMap tmRow, const __grid_constant__ CUtensorMap tmCol,
               const float *dt_out, const float *cs_f, const float *cs_b, float *out, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ uint64_t bar_a, bar_x, bar_done;
    __shared__ uint32_t tmem_slot;
    const int P = d.P, N = d.N, Q = d.Q;
    const int npb = P / 64;
    uint8_t *smA = smem_align1024(dyn);
    uint8_t *smX = smA + 2 * Q * 128;
    float *w = reinterpret_cast<float *>(smX + npb * Q * 128);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % d.H, c = (blockIdx.x / d.H) % d.nc, b = blockIdx.x / (d.H * d.nc);
    const int grp = h / d.R;
    const int dir = blockIdx.y, n0 = blockIdx.z * 128;
    const int lim = min(Q, d.L - c * Q);
    const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
    const uint32_t ncols = tmem_cols(P);
    if (warp == 0) tmem_alloc(&tmem_slot, ncols);
    if (tid == 0) {
        // the thread that initialises the barriers also issues the loads: they are in flight while the row factors are
        // computed, and everybody else meets the barriers only after the CTA-wide sync below
        mbar_init(&bar_a, 1);
        mbar_init(&bar_x, 1);
        mbar_init(&bar_done, 1);
        fence_mbar_init();
        mbar_expect_tx(&bar_x, (uint32_t)(npb * Q * 128));
        for (int j = 0; j < npb; ++j) tma_load4(smX + j * Q * 128, &tmCol, j * 64, h, c * Q, b, &bar_x);
        mbar_expect_tx(&bar_a, (uint32_t)(2 * Q * 128));
        for (int j = 0; j < 2; ++j) tma_load4(smA + j * Q * 128, &tmRow, n0 + j * 64, grp, c * Q, b, &bar_a);
    }
    {
        const float T0 = dir ? cs_b[base] : cs_f[base + Q - 1];
        for (int l = tid; l < Q; l += kThreads) {
            const float cs = dir ? cs_b[base + l] : cs_f[base + l];
            float v = 0.f;
            if (l < lim) v = (MODE == 0) ? dt_out[base + l] * __expf(T0 - cs) : __expf(cs);
            w[l] = v;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    bool ok = mbar_wait(&bar_x, 0);
    if (ok) {                                                   // scale row l of the x / g tile by w[l], in place
        const int chunks = npb * Q * 8;
        for (int q = tid; q < chunks; q += kThreads) {
            uint4 *ptr = reinterpret_cast<uint4 *>(smX) + q;
            const int l = (q >> 3) % Q;
            *ptr = scale8_packed<T>(*ptr, w[l]);
        }
        fence_async_smem();
    }
    ok = __syncthreads_and(ok);
    if (ok && tid == 0) {
        ok = mbar_wait(&bar_a, 0);
        if (ok) {
            tc_fence_after();
            const uint32_t idesc = instr_desc(AbFmt<T>::v, true, true, P);
            for (int kk = 0; kk < Q / 16; ++kk)
                umma(tmem, smem_desc(smem_u32(smA) + kk * 2048, (uint32_t)Q * 128, 1024),
                     smem_desc(smem_u32(smX) + kk * 2048, (uint32_t)Q * 128, 1024), idesc, kk > 0 ? 1u : 0u);
            umma_commit(&bar_done);
        }
    }
    if (ok) ok = mbar_wait(&bar_done, 0);
    ok = __syncthreads_and(ok);
    tc_fence_after();
    if (!ok && tid == 0) atomicExch(status, kErrMmaTimeout);
    if (ok) {
        const int n = n0 + (warp & 3) * 32 + lane;
        const long long per_dir = (long long)d.b * d.nc * d.H * P * N;
        float *o = out + dir * per_dir + ((long long)(b * d.nc + c) * d.H + h) * P * N + n;
        for (int c0 = (warp >> 2) * 32; c0 < P; c0 += 64) {
            float v[32];
            tmem_ld32(tmem_lane_base(tmem) + c0, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) o[(long long)(c0 + j) * N] = v[j];
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, ncols);
}

// ---------------------------------------------------------------------------------------------------------
// The same two products, pipelined over the heads of a group (headdim 64).  The B / C tile [Q x 128 n] - the same for
// every head of the group - is loaded once per CTA; per head the x / g tile [Q x 64] arrives twice by TMA (ring of two
// stages), is scaled in place once with the forward and once with the backward row factor, and ONE chain of Q/16 MMAs
// with N = 128 (columns 0-63 forward, 64-127 backward) forms both directions.  Accumulators are double-buffered in
// TMEM: the epilogue of head h (128 x 128 fp32 to global memory) runs while the MMAs of head h+1 execute.  Row
// factors are fetched one head ahead.
// grid (b*nc*G*ks, N/128): ks CTAs share the heads of a group (R % ks == 0).
struct StateGrpShared {
    uint64_t bar_a, full[2], scaled[2], done[2], accfree[2], wbar;
    uint32_t tmem_base;
    int fail;
};
// dstate 64 runs as half a 128-row tile: the TMA box of the second 64 state columns lies outside the tensor and reads
// as zeros, the epilogue skips those rows.
inline bool state_grp_ok(int P, int N, int Q, int R) {
    return P == 64 && (N == 64 || (N % 128 == 0 && N <= 256)) && (Q == 128 || Q == 256) && R >= 2;
}
inline size_t state_grp_smem(int Q) { return 1024 + 2 * (size_t)Q * 128 + 2 * 2 * (size_t)Q * 128 + 2 * 2 * (size_t)Q * 4; }
inline int state_grp_ksplit(int groups_total, int R, int sms) {      // CTAs per group: fill the SMs once, keep >= 2 heads per CTA
    int ks = 1;
    for (int k = 1; k <= R / 2; ++k)
        if (R % k == 0 && (long long)groups_total * k <= sms) ks = k;
    return ks;
}
constexpr int kStateGrpThreads = 2 * kThreads + 32;             // eight scaling warps, eight epilogue warps, one controller warp

// Warps 0-7 scale the tiles of head i while warps 8-15 store the accumulator of head i - 1 and lane 0 of warp 16
// issues every TMA load and every MMA, so that the three never wait behind one another.  Every blocking point is a
// bounded mbarrier wait (ids 41-47 in the status word).
template <class T, int MODE>
__global__ void __launch_bounds__(576, 1)
state_gemm_grp(Dims d, const __grid_constant__ CUtensorMap tmRow, const __grid_constant__ CUtensorMap tmCol, int ks,
               const float *dt_out, const float *cs_f, const float *cs_b, float *out, int *status) {
    pdl_begin();
    extern __shared__ uint8_t dyn[];
    __shared__ StateGrpShared sh;
    constexpr int P = 64;
    const int N = d.N, Q = d.Q, R = d.R;
    uint8_t *smA = smem_align1024(dyn);                         // 2 blocks [Q x 64 n], MN-major
    uint8_t *smX = smA + 2 * Q * 128;                           // 2 stages x (forward | backward) blocks [Q x 64 p]
    float *sc = reinterpret_cast<float *>(smX + 4 * Q * 128);   // [2 bufs][2 dirs][Q]
    const int stage_bytes = 2 * Q * 128;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x % ks, bx = blockIdx.x / ks;
    const int grp = bx % d.G, c = (bx / d.G) % d.nc, b = bx / (d.G * d.nc);
    const int n0 = blockIdx.y * 128;
    const int lim = min(Q, d.L - c * Q);
    const int nh = R / ks, h0 = grp * R + k * nh;               // this CTA's heads h0 .. h0 + nh - 1
    volatile int *fail = &sh.fail;
    auto load_head = [&](int i) {                               // the x / g tile of head i, twice, into stage i & 1
        uint8_t *dst = smX + (i & 1) * stage_bytes;
        mbar_expect_tx(&sh.full[i & 1], (uint32_t)stage_bytes);
        tma_load4(dst, &tmCol, 0, h0 + i, c * Q, b, &sh.full[i & 1]);
        tma_load4(dst + Q * 128, &tmCol, 0, h0 + i, c * Q, b, &sh.full[i & 1]);
    };
    if (warp == 0) tmem_alloc(&sh.tmem_base, 256);
    if (tid == 2 * kThreads) {                                  // the controller: barriers and the first loads
        mbar_init(&sh.bar_a, 1);
        mbar_init(&sh.wbar, 8);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh.full[i], 1);
            mbar_init(&sh.scaled[i], 8);
            mbar_init(&sh.done[i], 1);
            mbar_init(&sh.accfree[i], 8);
        }
        sh.fail = 0;
        fence_mbar_init();
        mbar_expect_tx(&sh.bar_a, (uint32_t)(2 * Q * 128));
        for (int j = 0; j < 2; ++j) tma_load4(smA + j * Q * 128, &tmRow, n0 + j * 64, grp, c * Q, b, &sh.bar_a);
        load_head(0);
        if (nh > 1) load_head(1);
    }
    // row factors: scaling thread l holds position l; inputs of head i + 1 are in flight while head i is worked on
    float pf_ = 0.f, pb_ = 0.f, pTf = 0.f, pTb = 0.f, pdt = 0.f;
    auto fetch_scale = [&](int i) {
        const long long base = ((long long)(b * d.H + h0 + i) * d.nc + c) * Q;
        if (tid < lim) {
            pf_ = cs_f[base + tid];
            pb_ = cs_b[base + tid];
            if (MODE == 0) {
                pTf = cs_f[base + Q - 1];
                pTb = cs_b[base];
                pdt = dt_out[base + tid];
            }
        }
    };
    auto write_scale = [&](int i) {
        if (tid < Q) {
            float wf = 0.f, wb = 0.f;
            if (tid < lim) {
                wf = (MODE == 0) ? pdt * __expf(pTf - pf_) : __expf(pf_);
                wb = (MODE == 0) ? pdt * __expf(pTb - pb_) : __expf(pb_);
            }
            sc[((i & 1) * 2 + 0) * Q + tid] = wf;
            sc[((i & 1) * 2 + 1) * Q + tid] = wb;
        }
    };
    if (warp < 8) {
        fetch_scale(0);
        write_scale(0);
        if (nh > 1) fetch_scale(1);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    if (warp == 16) {
        if (lane == 0) {
            bool ok = true;
            for (int i = 0; i < nh && ok; ++i) {
                uint8_t *sx = smX + (i & 1) * stage_bytes;
                if (i >= 1 && i + 1 < nh) {                     // stage (i + 1) & 1 is free once the MMAs of head i - 1 are done
                    ok = ws_wait(&sh.done[(i - 1) & 1], ((i - 1) >> 1) & 1, fail, 44);
                    if (ok) load_head(i + 1);
                }
                ok = ok && ws_wait(&sh.scaled[i & 1], (i >> 1) & 1, fail, 41);
                if (ok && i >= 2) ok = ws_wait(&sh.accfree[i & 1], ((i >> 1) - 1) & 1, fail, 42);
                if (ok && i == 0) ok = ws_wait(&sh.bar_a, 0, fail, 43);
                if (!ok) break;
                tc_fence_after();
                const uint32_t idesc = instr_desc(AbFmt<T>::v, true, true, 128);
                for (int kk = 0; kk < Q / 16; ++kk)
                    umma(tmem + (i & 1) * 128, smem_desc(smem_u32(smA) + kk * 2048, (uint32_t)Q * 128, 1024),
                         smem_desc(smem_u32(sx) + kk * 2048, (uint32_t)Q * 128, 1024), idesc, kk > 0 ? 1u : 0u);
                umma_commit(&sh.done[i & 1]);
            }
        }
    } else if (warp >= 8) {                                     // epilogue: accumulator i & 1 -> out[dir][p][n]
        const long long per_dir = (long long)d.b * d.nc * d.H * P * N;
        const int ew = warp - 8;
        const int n = n0 + (ew & 3) * 32 + lane, edir = ew >> 2;   // row n, the 64 columns of one direction
        bool ok = true;
#pragma unroll 1
        for (int i = 0; i < nh && ok; ++i) {
            ok = ws_wait_warp(&sh.done[i & 1], (i >> 1) & 1, fail, 45);
            if (!ok) break;
            tc_fence_after();
            float *o = out + edir * per_dir + ((long long)(b * d.nc + c) * d.H + h0 + i) * P * N + n;
            const uint32_t tl = tmem_lane_base(tmem) + (i & 1) * 128 + edir * 64;
            uint32_t v0[32], v1[32];                            // both halves requested before either is waited for
            tmem_ld32_nowait(tl, v0);
            tmem_ld32_nowait(tl + 32, v1);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.accfree[i & 1]);
            if (n < N) {
#pragma unroll
                for (int j = 0; j < 32; ++j) o[(long long)j * N] = __uint_as_float(v0[j]);
#pragma unroll
                for (int j = 0; j < 32; ++j) o[(long long)(32 + j) * N] = __uint_as_float(v1[j]);
            }
        }
    } else {
        bool ok = true;
#pragma unroll 1
        for (int i = 0; i < nh && ok; ++i) {
            uint8_t *sx = smX + (i & 1) * stage_bytes;
            ok = ws_wait_warp(&sh.full[i & 1], (i >> 1) & 1, fail, 46);
            if (!ok) break;
            const float *wf = sc + ((i & 1) * 2) * Q, *wb = wf + Q;
            for (int q = tid; q < Q * 8; q += kThreads) {       // rows l of both blocks times their factor, in place
                uint4 *pf4 = reinterpret_cast<uint4 *>(sx) + q, *pb4 = reinterpret_cast<uint4 *>(sx + Q * 128) + q;
                const int l = q >> 3;
                *pf4 = scale8_packed<T>(*pf4, wf[l]);
                *pb4 = scale8_packed<T>(*pb4, wb[l]);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.scaled[i & 1]);
            if (i + 1 < nh) {
                write_scale(i + 1);
                if (i + 2 < nh) fetch_scale(i + 2);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.wbar);
            // every scaling warp is done with head i and the factors of head i + 1 are written
            ok = ws_wait_warp(&sh.wbar, i & 1, fail, 47);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (sh.fail && tid == 0) atomicExch(status, kErrWsWait + sh.fail);
    if (warp == 0) {
        __syncwarp();
        tmem_dealloc(tmem, 256);
    }
}

}  // namespace tc
}  // namespace bissd
