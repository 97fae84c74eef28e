// CB[b,c,g,l,s] = C[l].B[s] with both operands by TMA (see tc::bmm_cb for the thread-staged form and the layouts).
// One shot per CTA: a 128 x 128 tile of (l, s); the C rows and the B rows arrive as K-major tiles of dstate/64 slabs,
// one MMA chain gives the tile, a second one with the operands swapped gives the same tile of the transpose, so that
// every store is a row-contiguous vector.  Outputs, each optional: CB16 (bf16), CBt16 (bf16, transposed), CBs (fp32
// in strips of 16 columns, [Q/16][Q rows][16]).  Rows past the end of the sequence read as zeros.
// grid (b*nc*G, Q/128, Q/128).
#pragma once
#include "tc_scan_tma.cuh"

namespace bissd {
namespace tc {

inline bool bmm_cb_tma_ok(int N, int Q) { return N % 64 == 0 && N <= 256 && (Q == 128 || Q == 256); }
inline size_t bmm_cb_tma_smem(int N) { return 1024 + 2 * (size_t)(N / 64) * 16384; }

template <class T>
__global__ void __launch_bounds__(kThreads)
bmm_cb_tma(Dims d, const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmB, __nv_bfloat16 *CB16,
           __nv_bfloat16 *CBt16, float *CBs, int *status) {
    pdl_begin();
    extern __shared__ uint8_t dyn[];
    __shared__ uint64_t bar_in, bar_done;
    __shared__ uint32_t tmem_slot;
    const int Q = d.Q, nsl = d.N / 64;
    uint8_t *smC = smem_align1024(dyn), *smB = smC + nsl * 16384;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = blockIdx.x % d.G, c = (blockIdx.x / d.G) % d.nc, b = blockIdx.x / (d.G * d.nc);
    const int l0 = blockIdx.y * kTileM, s0 = blockIdx.z * 128;
    const uint32_t ncols = CBt16 ? 256 : 128;
    if (warp == 0) tmem_alloc(&tmem_slot, ncols);
    if (tid == 32) {                                            // barriers and loads by the same thread, before the sync
        mbar_init(&bar_in, 1);
        mbar_init(&bar_done, 1);
        fence_mbar_init();
        mbar_expect_tx(&bar_in, (uint32_t)(2 * nsl * 16384));
        for (int j = 0; j < nsl; ++j) {
            tma_load4(smC + j * 16384, &tmC, j * 64, g, c * Q + l0, b, &bar_in);
            tma_load4(smB + j * 16384, &tmB, j * 64, g, c * Q + s0, b, &bar_in);
        }
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
            const uint32_t idesc = instr_desc(AbFmt<T>::v, false, false, 128);
            for (int t = 0; t < (CBt16 ? 2 : 1); ++t)
                for (int j = 0; j < nsl; ++j)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t dc = smem_desc(smem_u32(smC + j * 16384) + kk * 32, 16, 1024);
                        const uint64_t db = smem_desc(smem_u32(smB + j * 16384) + kk * 32, 16, 1024);
                        umma(tmem + t * 128, t ? db : dc, t ? dc : db, idesc, (j > 0 || kk > 0) ? 1u : 0u);
                    }
            umma_commit(&bar_done);
        }
    }
    if (ok) ok = mbar_wait(&bar_done, 0);
    ok = __syncthreads_and(ok);
    tc_fence_after();
    if (!ok && tid == 0) atomicExch(status, kErrMmaTimeout);
    if (ok) {
        const int r = (warp & 3) * 32 + lane, c0 = (warp >> 2) * 64;     // this thread: row r, columns c0 .. c0 + 63 of either tile
        const long long tile = ((long long)(b * d.nc + c) * d.G + g) * Q * Q;
        const uint32_t tl = tmem_lane_base(tmem) + c0;
        if (CB16 || CBs) {
            const int l = l0 + r;
#pragma unroll
            for (int hc = 0; hc < 64; hc += 32) {
                float v[32];
                tmem_ld32(tl + hc, v);
                const int sc = s0 + c0 + hc;                    // first of these 32 columns
                if (CBs) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<float4 *>(CBs + tile + (long long)((sc + j) >> 4) * Q * 16 + l * 16 + ((sc + j) & 15)) =
                            make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
                if (CB16) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        const float o[8] = {v[j], v[j + 1], v[j + 2], v[j + 3], v[j + 4], v[j + 5], v[j + 6], v[j + 7]};
                        *reinterpret_cast<uint4 *>(CB16 + tile + (long long)l * Q + sc + j) = pack8<__nv_bfloat16>(o);
                    }
                }
            }
        }
        if (CBt16) {
            const int srow = s0 + r;
#pragma unroll
            for (int hc = 0; hc < 64; hc += 32) {
                float v[32];
                tmem_ld32(tl + 128 + hc, v);
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    const float o[8] = {v[j], v[j + 1], v[j + 2], v[j + 3], v[j + 4], v[j + 5], v[j + 6], v[j + 7]};
                    *reinterpret_cast<uint4 *>(CBt16 + tile + (long long)srow * Q + l0 + c0 + hc + j) = pack8<__nv_bfloat16>(o);
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
