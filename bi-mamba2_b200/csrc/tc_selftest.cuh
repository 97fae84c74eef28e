// A plain C = A * B^T on the tcgen05 block GEMM, for checking the engine (descriptors, swizzled staging, TMEM
// loads) against a host GEMM in all four operand-major combinations.
#pragma once
#include "tc_engine.cuh"

namespace bissd {
namespace tc {

// A: a_mn ? [K][128] : [128][K];  B: b_mn ? [K][N] : [N][K];  C: [128][N] fp32.   One CTA.
template <class T, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads) selftest_gemm(const T *A, const T *B, float *C, int N, int K, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ PipeShared sh;
    uint8_t *stage = smem_align1024(dyn);
    Pipe p;
    pipe_init(p, &sh, stage, 256 * 128, 256, status);
    auto fa = [&](int r, int k) -> uint4 {
        if (k >= K) return zero8();
        return A_MN ? ldg8(A, (long long)k * kTileM + r) : ldg8(A, (long long)r * K + k);
    };
    auto fb = [&](int r, int k) -> uint4 {
        if (k >= K || r >= N) return zero8();
        return B_MN ? ldg8(B, (long long)k * N + r) : ldg8(B, (long long)r * K + k);
    };
    bool ok = umma_gemm<T, A_MN, B_MN>(p, p.tmem, N, K, 0u, fa, fb);
    ok = ok && umma_drain(p);
    if (ok) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int row = (warp & 3) * 32 + lane;
        for (int c0 = (warp >> 2) * 32; c0 < N; c0 += 64) {
            float v[32];
            tmem_ld32(tmem_lane_base(p.tmem) + c0, v);
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (c0 + j < N) C[(long long)row * N + c0 + j] = v[j];
        }
    }
    pipe_destroy(p, 256);
}

}  // namespace tc
}  // namespace bissd
