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

}  // namespace tc
}  // namespace bissd
