// Backward, TMA-fed: the "states" parts of dB / dC as one long accumulation over heads and directions, and the
// "prev" decay terms as their own small kernel (see simt::dbc_states for the formulae and reference line numbers).
//
//   dB_states[l,n] = sum_{h,dir} (x_h[l,:] Delta_h[l] e^{T-cs_dir[l]}) . E_{h,dir}[:,n]
//   dC_states[l,n] = sum_{h,dir} (g_h[l,:] e^{cs_dir[l]})              . S_{h,dir}[:,n]
// Both operands come by TMA into a three-deep ring - the left one ([128 rows x headdim], K-major) is row-scaled in
// place by the threads, the right one ([headdim x dstate], dstate contiguous -> MN-major) is used as it lands - and
// all 2*R products go into one TMEM accumulator that is read once.  The per-head row sums the reference takes from these products come from
// elsewhere: nf / nb from the dx kernel's per-direction accumulators, pf / pb from prev_terms_tma below.
#pragma once
#include "tc_scan_tma.cuh"
#include "tc_state_tma.cuh"

namespace bissd {
namespace tc {

struct DbcShared {
    uint64_t full[3], free_bar[3], done_bar;
    uint32_t tmem_base;
};

inline size_t dbc_tma_smem(int P, int nt) {
    return 1024 + 3 * ((size_t)(P / 64) * 16384 + (size_t)(nt / 64) * P * 128) + 2 * 2 * 128 * 4;
}

// grid (b*nc*G*nsplit, Q/128, 2); blockIdx.z: 0 = dB (left = x, right operand = E16), 1 = dC (left = g, right = states).
// part layout [b, nc*Q, G, N] fp32.  tmL: x or g, box [64 x 128 rows].
// Both operands of every (head, direction) stage arrive by TMA into a three-deep ring; the threads only scale the
// 128 rows of the left tile in place (packed multiply for bf16) before thread 0 issues the stage's MMAs.  The row
// factors of head h+1 are loaded while head h is being worked on.
template <class T>
__global__ void __launch_bounds__(kThreads, 2)
dbc_accum_tma(Dims d, const __grid_constant__ CUtensorMap tmEf, const __grid_constant__ CUtensorMap tmEb,
              const __grid_constant__ CUtensorMap tmSf, const __grid_constant__ CUtensorMap tmSb,
              const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmG, const float *dt_out,
              const float *cs_f, const float *cs_b, float *dB_part, float *dC_part, int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ DbcShared sh;
    const int P = d.P, N = d.N, Q = d.Q, R = d.R;
    const int npb = P / 64;
    const int nsplit = (N + 127) / 128;
    const int nt = min(N, 128), nnb = nt / 64;
    const int a_bytes = npb * 16384, b_bytes = nnb * P * 128, slot_bytes = a_bytes + b_bytes;
    uint8_t *base_sm = smem_align1024(dyn);
    float *sc = reinterpret_cast<float *>(base_sm + 3 * slot_bytes);               // [2 bufs][2 dirs][128 rows]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x % nsplit, bx = blockIdx.x / nsplit;
    const int grp = bx % d.G, c = (bx / d.G) % d.nc, b = bx / (d.G * d.nc);
    const int which = blockIdx.z;
    const int lim = min(Q, d.L - c * Q);
    const int l0 = blockIdx.y * kTileM, n0 = split * 128;
    const int total = 2 * R;
    const uint32_t ncols = tmem_cols(nt);
    auto load_stage = [&](int it) {                             // thread 0: both operands of stage it = (head, dir)
        const int hr = it >> 1, dir = it & 1, slot = it % 3;
        const int h = grp * R + hr;
        const int tile = (b * d.nc + c) * d.H + h;
        uint8_t *sa = base_sm + slot * slot_bytes, *sb = sa + a_bytes;
        const CUtensorMap *m = which ? (dir ? &tmSb : &tmSf) : (dir ? &tmEb : &tmEf);
        mbar_expect_tx(&sh.full[slot], (uint32_t)slot_bytes);
        for (int j = 0; j < npb; ++j) tma_load4(sa + j * 16384, which ? &tmG : &tmX, j * 64, h, c * Q + l0, b, &sh.full[slot]);
        for (int j = 0; j < nnb; ++j) tma_load2(sb + j * P * 128, m, n0 + j * 64, tile * P, &sh.full[slot]);
    };
    if (warp == 0) tmem_alloc(&sh.tmem_base, ncols);
    if (tid == 0) {                                             // barriers and the first loads by the same thread
        for (int i = 0; i < 3; ++i) {
            mbar_init(&sh.full[i], 1);
            mbar_init(&sh.free_bar[i], 1);
        }
        mbar_init(&sh.done_bar, 1);
        fence_mbar_init();
        load_stage(0);
        if (total > 1) load_stage(1);
        if (total > 2) load_stage(2);
    }
    // one (dir, row) per thread: the inputs of the row factor of head hr, then the factor itself
    const int sdir = tid >> 7, srow = tid & 127, sl = l0 + srow;
    float pcs = 0.f, pT = 0.f, pdt = 0.f;
    auto fetch_scale = [&](int hr) {
        const int h = grp * R + hr;
        const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
        if (sl < lim) {
            pcs = sdir ? cs_b[base + sl] : cs_f[base + sl];
            if (!which) {
                pT = sdir ? cs_b[base] : cs_f[base + Q - 1];
                pdt = dt_out[base + sl];
            }
        }
    };
    auto write_scale = [&](int hr) {
        float v = 0.f;
        if (sl < lim) v = which ? __expf(pcs) : pdt * __expf(pT - pcs);
        sc[((hr & 1) * 2 + sdir) * 128 + srow] = v;
    };
    fetch_scale(0);
    write_scale(0);
    if (R > 1) fetch_scale(1);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    bool ok = true;
#pragma unroll 1
    for (int it = 0; it < total; ++it) {
        const int slot = it % 3, hr = it >> 1, dir = it & 1;
        uint8_t *sa = base_sm + slot * slot_bytes;
        ok = mbar_wait(&sh.full[slot], (it / 3) & 1);
        if (ok) {                                               // scale row r of the left tile by its factor, in place
            const float *sf_ = sc + ((hr & 1) * 2 + dir) * 128;
            for (int q = tid; q < npb * 1024; q += kThreads) {
                uint4 *ptr = reinterpret_cast<uint4 *>(sa) + q;
                *ptr = scale8_packed<T>(*ptr, sf_[(q >> 3) & 127]);
            }
            fence_async_smem();
            if (dir == 1 && hr + 1 < R) {                       // next head's factors; then the loads for the one after
                write_scale(hr + 1);
                if (hr + 2 < R) fetch_scale(hr + 2);
            }
        }
        ok = __syncthreads_and(ok);
        if (!ok) break;
        if (tid == 0) {
            tc_fence_after();
            const uint32_t idesc = instr_desc(AbFmt<T>::v, false, true, nt);
            const uint8_t *sb = sa + a_bytes;
            for (int j = 0; j < npb; ++j)
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma(tmem, smem_desc(smem_u32(sa + j * 16384) + kk * 32, 16, 1024),
                         smem_desc(smem_u32(sb) + (j * 64 + kk * 16) * 128, (uint32_t)P * 128, 1024), idesc,
                         (it > 0 || j > 0 || kk > 0) ? 1u : 0u);
            umma_commit(&sh.free_bar[slot]);
            if (it >= 1 && it + 2 < total) {                    // refill the slot stage it-1 used, once its MMAs are done
                ok = mbar_wait(&sh.free_bar[(it + 2) % 3], ((it - 1) / 3) & 1);
                if (ok) load_stage(it + 2);
            }
        }
    }
    // a failure seen only by thread 0 in the last iteration is caught here
    if (ok) {
        if (tid == 0) umma_commit(&sh.done_bar);
        ok = mbar_wait(&sh.done_bar, 0);
    }
    ok = __syncthreads_and(ok);
    tc_fence_after();
    if (!ok && tid == 0) atomicExch(status, kErrMmaTimeout);
    if (ok) {
        const int l = l0 + (warp & 3) * 32 + lane;
        float *part = (which ? dC_part : dB_part) + (((long long)b * d.nc * Q + c * Q + l) * d.G + grp) * N + n0;
        for (int c0 = (warp >> 2) * 32; c0 < nt; c0 += 64) {
            float v[32];
            tmem_ld32(tmem_lane_base(tmem) + c0, v);
            if (l < lim) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4 *>(part + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, ncols);
}

// ---------------------------------------------------------------------------------------------------------
// The same sums with one CTA per (batch, chunk, group, 128 state columns) that walks the heads of its group: the CTA
// owns all Q rows (one 128-column accumulator per 128-row block), so the state tiles E_f / E_b (or S_f / S_b) of a head
// are fetched once instead of once per row block, and the x / g tile once.  Roles as in state_gemm_grp: warps 0-7
// turn the left tile as it landed into its two row-scaled copies (one buffer: the copies of head i + 1 are written
// once the MMAs of head i are done), lane 0 of warp 8 issues every TMA load and every MMA; two stages of (left
// tile + 2 right tiles).  All heads accumulate in tensor memory, which is read once at the end.  Bounded waits,
// ids 51-56 in the status word.
// grid (b*nc*G*nsplit, 1, 2); blockIdx.z: 0 = dB, 1 = dC.
struct DbcGrpShared {
    uint64_t full[2], scaled, done[2], wbar;
    uint32_t tmem_base;
    int fail;
};
inline bool dbc_grp_ok(int P, int N, int Q) { return P == 64 && (N == 64 || N % 128 == 0) && (Q == 128 || Q == 256); }
inline size_t dbc_grp_smem(int Q, int nt) {
    return 1024 + 2 * ((size_t)Q * 128 + 2 * (size_t)(nt / 64) * 64 * 128) + 2 * (size_t)Q * 128 + 2 * 2 * (size_t)Q * 4;
}
constexpr int kDbcGrpThreads = kThreads + 32;

template <class T>
__global__ void __launch_bounds__(kDbcGrpThreads, 1)
dbc_accum_grp(Dims d, const __grid_constant__ CUtensorMap tmEf, const __grid_constant__ CUtensorMap tmEb,
              const __grid_constant__ CUtensorMap tmSf, const __grid_constant__ CUtensorMap tmSb,
              const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmG, const float *dt_out,
              const float *cs_f, const float *cs_b, float *dB_part, float *dC_part, int *status) {
    pdl_begin();
    extern __shared__ uint8_t dyn[];
    __shared__ DbcGrpShared sh;
    constexpr int P = 64;
    const int N = d.N, Q = d.Q, R = d.R;
    const int nsplit = (N + 127) / 128, nt = min(N, 128), nnb = nt / 64, nrb = Q / 128;
    const int left_bytes = Q * 128, right_bytes = 2 * nnb * P * 128, stage_bytes = left_bytes + right_bytes;
    uint8_t *base_sm = smem_align1024(dyn);                     // per stage: left [Q rows x 128 B], right [dir][nnb][P x 128 B]
    uint8_t *smScaled = base_sm + 2 * stage_bytes;              // [dir][Q rows x 128 B]
    float *sc = reinterpret_cast<float *>(smScaled + 2 * left_bytes);   // [2 bufs][2 dirs][Q]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x % nsplit, bx = blockIdx.x / nsplit;
    const int grp = bx % d.G, c = (bx / d.G) % d.nc, b = bx / (d.G * d.nc);
    const int which = blockIdx.z;
    const int lim = min(Q, d.L - c * Q);
    const int n0 = split * 128, h0 = grp * R;
    const uint32_t ncols = tmem_cols(nrb * nt);
    volatile int *fail = &sh.fail;
    auto load_head = [&](int i) {                               // the left tile and both state tiles of head i
        uint8_t *sl = base_sm + (i & 1) * stage_bytes, *sr = sl + left_bytes;
        const int tile = (b * d.nc + c) * d.H + h0 + i;
        mbar_expect_tx(&sh.full[i & 1], (uint32_t)stage_bytes);
        for (int j = 0; j < nrb; ++j)
            tma_load4(sl + j * 16384, which ? &tmG : &tmX, 0, h0 + i, c * Q + j * 128, b, &sh.full[i & 1]);
        for (int dir = 0; dir < 2; ++dir) {
            const CUtensorMap *m = which ? (dir ? &tmSb : &tmSf) : (dir ? &tmEb : &tmEf);
            for (int j = 0; j < nnb; ++j) tma_load2(sr + (dir * nnb + j) * P * 128, m, n0 + j * 64, tile * P, &sh.full[i & 1]);
        }
    };
    if (warp == 0) tmem_alloc(&sh.tmem_base, ncols);
    if (tid == kThreads) {                                      // the controller: barriers and the first loads
        mbar_init(&sh.wbar, 8);
        mbar_init(&sh.scaled, 8);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh.full[i], 1);
            mbar_init(&sh.done[i], 1);
        }
        sh.fail = 0;
        fence_mbar_init();
        load_head(0);
        if (R > 1) load_head(1);
    }
    // row factors: scaling thread l holds row l in both directions; the inputs of head i + 2 are in flight while head i is scaled
    float pf_ = 0.f, pb_ = 0.f, pTf = 0.f, pTb = 0.f, pdt = 0.f;
    auto fetch_scale = [&](int i) {
        const long long base = ((long long)(b * d.H + h0 + i) * d.nc + c) * Q;
        if (tid < lim) {
            pf_ = cs_f[base + tid];
            pb_ = cs_b[base + tid];
            if (!which) {
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
                wf = which ? __expf(pf_) : pdt * __expf(pTf - pf_);
                wb = which ? __expf(pb_) : pdt * __expf(pTb - pb_);
            }
            sc[((i & 1) * 2 + 0) * Q + tid] = wf;
            sc[((i & 1) * 2 + 1) * Q + tid] = wb;
        }
    };
    if (warp < 8) {
        fetch_scale(0);
        write_scale(0);
        if (R > 1) fetch_scale(1);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    if (warp == 8) {
        if (lane == 0) {
            bool ok = true;
            const uint32_t idesc = instr_desc(AbFmt<T>::v, false, true, nt);
            for (int i = 0; i < R && ok; ++i) {
                if (i >= 1 && i + 1 < R) {                      // stage (i + 1) & 1 is free once the MMAs of head i - 1 are done
                    ok = ws_wait(&sh.done[(i - 1) & 1], ((i - 1) >> 1) & 1, fail, 51);
                    if (ok) load_head(i + 1);
                }
                ok = ok && ws_wait(&sh.scaled, i & 1, fail, 52);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sl = smem_u32(smScaled), sr = smem_u32(base_sm + (i & 1) * stage_bytes) + left_bytes;
                for (int rb = 0; rb < nrb; ++rb)
                    for (int dir = 0; dir < 2; ++dir)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma(tmem + rb * nt, smem_desc(sl + (dir * nrb + rb) * 16384 + kk * 32, 16, 1024),
                                 smem_desc(sr + dir * nnb * P * 128 + kk * 16 * 128, (uint32_t)P * 128, 1024), idesc,
                                 (i > 0 || dir > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&sh.done[i & 1]);
            }
        }
    } else {
        bool ok = true;
#pragma unroll 1
        for (int i = 0; i < R && ok; ++i) {
            uint8_t *sl = base_sm + (i & 1) * stage_bytes;
            ok = ws_wait_warp(&sh.full[i & 1], (i >> 1) & 1, fail, 53);
            // the scaled copies of head i - 1 have been read by its MMAs
            if (ok && i >= 1) ok = ws_wait_warp(&sh.done[(i - 1) & 1], ((i - 1) >> 1) & 1, fail, 56);
            if (!ok) break;
            const float *wf = sc + ((i & 1) * 2) * Q, *wb = wf + Q;
            for (int q = tid; q < Q * 8; q += kThreads) {
                const uint4 raw = reinterpret_cast<const uint4 *>(sl)[q];
                reinterpret_cast<uint4 *>(smScaled)[q] = scale8_packed<T>(raw, wf[q >> 3]);
                reinterpret_cast<uint4 *>(smScaled + left_bytes)[q] = scale8_packed<T>(raw, wb[q >> 3]);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.scaled);
            if (i + 1 < R) {
                write_scale(i + 1);
                if (i + 2 < R) fetch_scale(i + 2);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.wbar);
            // every scaling warp is done with head i and the factors of head i + 1 are written
            ok = ws_wait_warp(&sh.wbar, i & 1, fail, 54);
        }
        if (ok) ok = ws_wait_warp(&sh.done[(R - 1) & 1], ((R - 1) >> 1) & 1, fail, 55);
        if (ok) {
            tc_fence_after();
            for (int rb = 0; rb < nrb; ++rb) {
                const int l = rb * 128 + (warp & 3) * 32 + lane;
                float *part = (which ? dC_part : dB_part) + (((long long)b * d.nc * Q + c * Q + l) * d.G + grp) * N + n0;
                for (int c0 = (warp >> 2) * 32; c0 < nt; c0 += 64) {
                    float v[32];
                    tmem_ld32(tmem_lane_base(tmem) + rb * nt + c0, v);
                    if (l < lim) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4 *>(part + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    }
                }
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

// ---------------------------------------------------------------------------------------------------------
// "prev" decay terms:  pf[l] = e^{cs_f[l]} sum_p g[l,p] (C[l,:].S_f[p,:]),  pb[l] likewise with S_b / cs_b  - the row sums
// the reference takes inside _chunk_scan_bwd_dc_kernel (src/ssd/bi/ssd_chunk_scan.py:598-623).  C and both entering
// states arrive by TMA; nothing is staged by threads.   grid (b*nc*H, Q/128).
inline size_t prev_tma_smem(int P, int N) { return 1024 + (size_t)(N / 64) * 16384 + 2 * (size_t)(N / 64) * P * 128; }

template <class T>
__global__ void __launch_bounds__(kThreads, 2)
prev_terms_tma(Dims d, const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmSf,
               const __grid_constant__ CUtensorMap tmSb, View g, const float *cs_f, const float *cs_b, float *pf, float *pb,
               int *status) {
    extern __shared__ uint8_t dyn[];
    __shared__ uint64_t bar_in, bar_done;
    __shared__ uint32_t tmem_slot;
    __shared__ float rowred[2][kTileM];
    const int P = d.P, N = d.N, Q = d.Q;
    const int nsl = N / 64;
    uint8_t *smC = smem_align1024(dyn);
    uint8_t *smSf = smC + nsl * 16384, *smSb = smSf + nsl * P * 128;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % d.H, c = (blockIdx.x / d.H) % d.nc, b = blockIdx.x / (d.H * d.nc);
    const int grp = h / d.R;
    const int lim = min(Q, d.L - c * Q);
    const int l0 = blockIdx.y * kTileM;
    const long long base = ((long long)(b * d.H + h) * d.nc + c) * Q;
    const uint32_t ncols = tmem_cols(2 * P);
    if (warp == 0) tmem_alloc(&tmem_slot, ncols);
    if (tid == 0) {                                             // barriers and loads by the same thread, before the sync
        mbar_init(&bar_in, 1);
        mbar_init(&bar_done, 1);
        fence_mbar_init();
        const int tile = (b * d.nc + c) * d.H + h;
        mbar_expect_tx(&bar_in, (uint32_t)(nsl * 16384 + 2 * nsl * P * 128));
        for (int j = 0; j < nsl; ++j) {
            tma_load4(smC + j * 16384, &tmC, j * 64, grp, c * Q + l0, b, &bar_in);
            tma_load2(smSf + j * P * 128, &tmSf, j * 64, tile * P, &bar_in);
            tma_load2(smSb + j * P * 128, &tmSb, j * 64, tile * P, &bar_in);
        }
    }
    // this thread's g row piece and row factors are requested while the tiles are in flight
    const int quad = warp & 3, half = warp >> 2;
    const int r = quad * 32 + lane, l = l0 + r;
    uint4 gq[4];
    float ecf = 0.f, ecb = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) gq[j] = (l < lim && half * 32 < P) ? ld8v<T>(g, b, c * Q + l, h, half * 32 + j * 8) : zero8();
    if (l < lim) {
        ecf = cs_f[base + l];
        ecb = cs_b[base + l];
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
            const uint32_t idesc = instr_desc(AbFmt<T>::v, false, false, P);
            for (int dir = 0; dir < 2; ++dir)
                for (int j = 0; j < nsl; ++j)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma(tmem + dir * P, smem_desc(smem_u32(smC + j * 16384) + kk * 32, 16, 1024),
                             smem_desc(smem_u32((dir ? smSb : smSf) + j * P * 128) + kk * 32, 16, 1024), idesc,
                             (j > 0 || kk > 0) ? 1u : 0u);
            umma_commit(&bar_done);
        }
    }
    if (ok) ok = mbar_wait(&bar_done, 0);
    ok = __syncthreads_and(ok);
    tc_fence_after();
    if (!ok && tid == 0) atomicExch(status, kErrMmaTimeout);
    float sf_ = 0.f, sb_ = 0.f;
    if (ok) {
        const uint32_t tl = tmem_lane_base(tmem);
        for (int c0 = half * 32; c0 < P; c0 += 64) {
            float af[32], ab[32];
            tmem_ld32(tl + c0, af);
            tmem_ld32(tl + P + c0, ab);
            if (l < lim) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    float gv[8];
                    unpack8<T>(c0 == half * 32 ? gq[j >> 3] : ld8v<T>(g, b, c * Q + l, h, c0 + j), gv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        sf_ = fmaf(af[j + i], gv[i], sf_);
                        sb_ = fmaf(ab[j + i], gv[i], sb_);
                    }
                }
            }
        }
    }
    if (half == 1) {
        rowred[0][r] = sf_;
        rowred[1][r] = sb_;
    }
    tc_fence_before();
    __syncthreads();
    if (ok && half == 0 && l < Q) {
        const float ef = (l < lim) ? __expf(ecf) : 0.f, eb = (l < lim) ? __expf(ecb) : 0.f;
        pf[base + l] = ef * (sf_ + (P > 32 ? rowred[0][r] : 0.f));
        pb[base + l] = eb * (sb_ + (P > 32 ? rowred[1][r] : 0.f));
    }
    if (warp == 0) tmem_dealloc(tmem, ncols);
}

// ---------------------------------------------------------------------------------------------------------
// The same row sums with one CTA per (batch, chunk, group[, head range]) that keeps the C tile of all Q rows resident
// and walks its heads: per head both entering states (one [2P x dstate] K-major tile, so one N = 2P product per
// 128-row block) and the g tile arrive by TMA into two-deep rings; warps 0-7 read the products out of double-buffered
// tensor memory and dot them with their g row while lane 0 of warp 8 issues the loads and MMAs of the next head.
// Bounded waits, ids 61-66 in the status word.   grid (b*nc*G*ks).
struct PrevGrpShared {
    uint64_t bar_c, full_s[2], full_g[2], done[2], accfree[2], gfree[2];
    uint32_t tmem_base;
    int fail;
};
inline bool prev_grp_ok(int P, int N, int Q, int R) { return P == 64 && (N == 64 || N == 128) && (Q == 128 || Q == 256) && R >= 2; }
inline size_t prev_grp_smem(int N, int Q) {
    return 1024 + (size_t)(Q / 128) * (N / 64) * 16384 + 2 * 2 * (size_t)(N / 64) * 8192 + 2 * (size_t)(Q / 128) * 16384;
}
constexpr int kPrevGrpThreads = kThreads + 32;

template <class T>
__global__ void __launch_bounds__(kPrevGrpThreads, 1)
prev_terms_grp(Dims d, const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmSf,
               const __grid_constant__ CUtensorMap tmSb, const __grid_constant__ CUtensorMap tmG, int ks, const float *cs_f,
               const float *cs_b, float *pf, float *pb, int *status) {
    pdl_begin();
    extern __shared__ uint8_t dyn[];
    __shared__ PrevGrpShared sh;
    constexpr int P = 64;
    const int N = d.N, Q = d.Q, R = d.R;
    const int nsl = N / 64, nrb = Q / 128;
    const int c_bytes = nrb * nsl * 16384, s_bytes = 2 * nsl * 8192, g_bytes = nrb * 16384;
    uint8_t *smC = smem_align1024(dyn);                         // [row block][slab of 64 n][128 rows x 128 B]
    uint8_t *smS = smC + c_bytes;                               // 2 stages x [slab][f | b][64 p x 128 B]
    uint8_t *smG = smS + 2 * s_bytes;                           // 2 stages x [row block][128 rows x 128 B]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x % ks, bx = blockIdx.x / ks;
    const int grp = bx % d.G, c = (bx / d.G) % d.nc, b = bx / (d.G * d.nc);
    const int lim = min(Q, d.L - c * Q);
    const int nh = R / ks, h0 = grp * R + k * nh;
    volatile int *fail = &sh.fail;
    auto load_s = [&](int i) {
        uint8_t *dst = smS + (i & 1) * s_bytes;
        const int tile = (b * d.nc + c) * d.H + h0 + i;
        mbar_expect_tx(&sh.full_s[i & 1], (uint32_t)s_bytes);
        for (int j = 0; j < nsl; ++j) {
            tma_load2(dst + (j * 2 + 0) * 8192, &tmSf, j * 64, tile * P, &sh.full_s[i & 1]);
            tma_load2(dst + (j * 2 + 1) * 8192, &tmSb, j * 64, tile * P, &sh.full_s[i & 1]);
        }
    };
    auto load_g = [&](int i) {
        uint8_t *dst = smG + (i & 1) * g_bytes;
        mbar_expect_tx(&sh.full_g[i & 1], (uint32_t)g_bytes);
        for (int rb = 0; rb < nrb; ++rb) tma_load4(dst + rb * 16384, &tmG, 0, h0 + i, c * Q + rb * 128, b, &sh.full_g[i & 1]);
    };
    const uint32_t ncols = 2 * nrb * 128;                       // two accumulator sets of nrb x 128 columns
    if (warp == 0) tmem_alloc(&sh.tmem_base, ncols);
    if (tid == kThreads) {                                      // the controller: barriers and the first loads
        mbar_init(&sh.bar_c, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh.full_s[i], 1);
            mbar_init(&sh.full_g[i], 1);
            mbar_init(&sh.done[i], 1);
            mbar_init(&sh.accfree[i], 8);
            mbar_init(&sh.gfree[i], 8);
        }
        sh.fail = 0;
        fence_mbar_init();
        mbar_expect_tx(&sh.bar_c, (uint32_t)c_bytes);
        for (int rb = 0; rb < nrb; ++rb)
            for (int j = 0; j < nsl; ++j)
                tma_load4(smC + (rb * nsl + j) * 16384, &tmC, j * 64, grp, c * Q + rb * 128, b, &sh.bar_c);
        load_s(0);
        load_g(0);
        if (nh > 1) {
            load_s(1);
            load_g(1);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    if (warp == 8) {
        if (lane == 0) {
            bool ok = ws_wait(&sh.bar_c, 0, fail, 61);
            const uint32_t idesc = instr_desc(AbFmt<T>::v, false, false, 2 * P);
            for (int i = 0; i < nh && ok; ++i) {
                ok = ws_wait(&sh.full_s[i & 1], (i >> 1) & 1, fail, 62);
                if (ok && i >= 2) ok = ws_wait(&sh.accfree[i & 1], ((i >> 1) - 1) & 1, fail, 63);
                if (!ok) break;
                tc_fence_after();
                const uint32_t ss = smem_u32(smS + (i & 1) * s_bytes);
                for (int rb = 0; rb < nrb; ++rb)
                    for (int j = 0; j < nsl; ++j)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma(tmem + ((i & 1) * nrb + rb) * 128, smem_desc(smem_u32(smC + (rb * nsl + j) * 16384) + kk * 32, 16, 1024),
                                 smem_desc(ss + j * 16384 + kk * 32, 16, 1024), idesc, (j > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&sh.done[i & 1]);
                if (i >= 1 && i + 1 < nh) {                     // the rings of head i - 1 are refilled as they drain
                    ok = ws_wait(&sh.done[(i - 1) & 1], ((i - 1) >> 1) & 1, fail, 64);
                    if (ok) load_s(i + 1);
                    ok = ok && ws_wait(&sh.gfree[(i - 1) & 1], ((i - 1) >> 1) & 1, fail, 65);
                    if (ok) load_g(i + 1);
                }
            }
        }
    } else {
        const int quad = warp & 3, dir = warp >> 2;             // rows quad * 32 + lane of every row block, one direction
        const float *cs = dir ? cs_b : cs_f;
        float *po = dir ? pb : pf;
        bool ok = true;
        float ecs[2] = {0.f, 0.f}, ecs_next[2] = {0.f, 0.f};
        auto fetch_cs = [&](int i, float (&e)[2]) {
            const long long base = ((long long)(b * d.H + h0 + i) * d.nc + c) * Q;
#pragma unroll
            for (int rb = 0; rb < 2; ++rb) {
                const int l = rb * 128 + quad * 32 + lane;
                e[rb] = (rb < nrb && l < lim) ? cs[base + l] : 0.f;
            }
        };
        fetch_cs(0, ecs);
#pragma unroll 1
        for (int i = 0; i < nh && ok; ++i) {
            if (i + 1 < nh) fetch_cs(i + 1, ecs_next);
            ok = ws_wait_warp(&sh.done[i & 1], (i >> 1) & 1, fail, 66) && ws_wait_warp(&sh.full_g[i & 1], (i >> 1) & 1, fail, 66);
            if (!ok) break;
            tc_fence_after();
            const long long base = ((long long)(b * d.H + h0 + i) * d.nc + c) * Q;
            float sum[2] = {0.f, 0.f};
#pragma unroll
            for (int rb = 0; rb < 2; ++rb) {
                if (rb < nrb) {
                    const int r = quad * 32 + lane;
                    uint32_t v0[32], v1[32];
                    const uint32_t tl = tmem_lane_base(tmem) + ((i & 1) * nrb + rb) * 128 + dir * 64;
                    tmem_ld32_nowait(tl, v0);
                    tmem_ld32_nowait(tl + 32, v1);
                    const uint8_t *grow = smG + (i & 1) * g_bytes + rb * 16384 + r * 128;
                    uint4 gq[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) gq[q] = *reinterpret_cast<const uint4 *>(grow + ((q ^ (r & 7)) << 4));
                    tmem_ld_wait();
                    float acc = 0.f;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        float gv[8];
                        unpack8<T>(gq[q], gv);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int col = q * 8 + e;
                            acc = fmaf(__uint_as_float(col < 32 ? v0[col] : v1[col - 32]), gv[e], acc);
                        }
                    }
                    sum[rb] = acc;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&sh.accfree[i & 1]);
                mbar_arrive(&sh.gfree[i & 1]);
            }
#pragma unroll
            for (int rb = 0; rb < 2; ++rb) {
                const int l = rb * 128 + quad * 32 + lane;
                if (rb < nrb) po[base + l] = (l < lim) ? __expf(ecs[rb]) * sum[rb] : 0.f;
            }
            ecs[0] = ecs_next[0];
            ecs[1] = ecs_next[1];
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
