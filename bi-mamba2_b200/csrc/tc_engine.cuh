// tcgen05 building blocks for sm_100a: TMEM allocation, shared-memory matrix descriptors, UMMA issue, mbarrier
// waits with an iteration limit, TMEM loads - and a two-stage block GEMM whose operand tiles are written into
// shared memory by the CTA's threads (so decay factors, masks and gates are applied while staging) in the
// 128-byte-swizzled canonical layouts the tensor core reads.
//
// Tile conventions (16-bit operands):
//   * one pipeline stage holds K = 64 elements (= one 128-byte swizzle row) of A (128 rows) and of B (<= 256 rows)
//   * K-major tile:  row r, 16-byte chunk c (8 elements along K):  byte = r*128 + ((c ^ (r&7)) << 4)
//   * MN-major tile: blocks of 64 rows; inside a block K-row k holds the block's 64 row-elements contiguously:
//         byte = (r/64)*8192 + (k/8)*1024 + (k%8)*128 + ((((r%64)/8) ^ (k%8)) << 4) + (r%8)*2
//   * accumulator: UMMA M = 128, cta_group::1 -> D row m lives in TMEM lane m, column n in TMEM column n.
#pragma once
#include "common.cuh"

namespace bissd {
namespace tc {

constexpr int kThreads = 256;
constexpr int kStageK = 64;
constexpr int kTileM = 128;
constexpr uint32_t kSpinLimit = 1u << 22;      // mbarrier polls before a wait gives up and reports an error
constexpr int kAStageBytes = kTileM * kStageK * 2;

// error codes written to the status word
constexpr int kErrMmaTimeout = 1;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// First 1024-byte boundary inside the dynamic shared memory.  Plain pointer arithmetic on the array (no round trip
// through an integer) keeps the shared address space visible to the compiler, so accesses through the result are
// shared-memory instructions rather than generic ones.
__device__ __forceinline__ uint8_t *smem_align1024(uint8_t *dyn) {
    return dyn + ((1024u - (smem_u32(dyn) & 1023u)) & 1023u);
}

// ---- mbarrier ----------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Wait until the phase with the given parity has completed.  Each attempt lets the hardware suspend the thread for up
// to ~1 us (mbarrier.try_wait with a time hint) instead of spinning on test_wait - the spinning variant spent more
// issue slots polling than working.  Bounded: false after kWaitAttempts attempts (about a quarter of a second).
constexpr uint32_t kWaitAttempts = 1u << 18;
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(1000u)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    if (mbar_test(bar, parity)) return true;
    for (uint32_t i = 0; i < kWaitAttempts; ++i)
        if (mbar_try(bar, parity)) return true;
    return false;
}

// ---- waits for kernels whose warps play different roles ----------------------------------------------------------
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait that also gives up when another role has already failed.  `id` names the wait (role * 10 + barrier);
// the first wait that runs out leaves its id in the CTA-wide flag, from where it reaches the status word.
__device__ __forceinline__ bool ws_wait(uint64_t *bar, uint32_t parity, volatile int *fail, int id) {
    if (mbar_test(bar, parity)) return true;
    for (uint32_t i = 0; i < kWaitAttempts; ++i) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 7) == 7 && *fail) return false;
    }
    if (!*fail) *fail = id;
    return false;
}
// the same for a whole warp: every lane polls, the outcome is made uniform so that .aligned instructions stay legal
__device__ __forceinline__ bool ws_wait_warp(uint64_t *bar, uint32_t parity, volatile int *fail, int id) {
    return __all_sync(0xffffffffu, ws_wait(bar, parity, fail, id));
}
constexpr int kErrWsWait = 0x1000;                              // status word = kErrWsWait + id of the wait that ran out

// ---- proxies and tcgen05 fences ------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- tensor memory --------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols) {   // one full warp; ncols power of 2 >= 32
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {      // same warp that allocated
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane (lane = 32*(warp%4) + laneid); warp-collective.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 16 consecutive fp32 columns of this thread's TMEM lane; warp-collective.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// 16 fp32 columns of this thread's TMEM lane without the completion wait (tmem_ld_wait); lets several loads, or a load
// and the work on the previous one, overlap - a load takes several hundred cycles to land
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8_nowait(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t tmem_lane_base(uint32_t tmem_base) {
    return tmem_base + ((uint32_t)(((threadIdx.x >> 5) & 3) * 32) << 16);
}

// ---- descriptors ----------------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 version bit set.  lbo/sbo in bytes.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;      // descriptor version for sm_100
    d |= (uint64_t)2 << 61;      // SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::f16: fp32 accumulate, A/B both bf16 (fmt 1) or both f16 (fmt 0), M = 128.
__host__ __device__ constexpr uint32_t instr_desc(int ab_fmt, bool a_mn, bool b_mn, int n) {
    return (1u << 4) | ((uint32_t)ab_fmt << 7) | ((uint32_t)ab_fmt << 10) | ((a_mn ? 1u : 0u) << 15) |
           ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}
template <class T> struct AbFmt;
template <> struct AbFmt<__nv_bfloat16> { static constexpr int v = 1; };
template <> struct AbFmt<__half> { static constexpr int v = 0; };

// D[tmem] (+)= A[smem] * B[smem]; one thread issues.
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrives once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---- packing ----------------------------------------------------------------------------------------------------------
template <class T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
}
template <class T> __device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    return make_uint4(pack2<T>(v[0], v[1]), pack2<T>(v[2], v[3]), pack2<T>(v[4], v[5]), pack2<T>(v[6], v[7]));
}
template <class T> __device__ __forceinline__ void unpack2(uint32_t u, float &a, float &b);
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t u, float &a, float &b) {
    a = __uint_as_float(u << 16);
    b = __uint_as_float(u & 0xFFFF0000u);
}
template <> __device__ __forceinline__ void unpack2<__half>(uint32_t u, float &a, float &b) {
    __half2 h = *reinterpret_cast<__half2 *>(&u);
    float2 f = __half22float2(h);
    a = f.x;
    b = f.y;
}
template <class T> __device__ __forceinline__ void unpack8(uint4 u, float (&v)[8]) {
    unpack2<T>(u.x, v[0], v[1]);
    unpack2<T>(u.y, v[2], v[3]);
    unpack2<T>(u.z, v[4], v[5]);
    unpack2<T>(u.w, v[6], v[7]);
}
// 8 consecutive 16-bit elements (16-byte aligned) from global memory
__device__ __forceinline__ uint4 ldg8(const void *base, long long elem_index) {
    return __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(base) + elem_index));
}
__device__ __forceinline__ void ldg8f(const float *p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p));
    const float4 b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ uint4 zero8() { return make_uint4(0u, 0u, 0u, 0u); }

// ---- the pipeline --------------------------------------------------------------------------------------------------
// Lives in static shared memory of every tcgen05 kernel.
struct PipeShared {
    uint64_t free_bar[2];     // stage s may be overwritten (the MMAs that read it have completed)
    uint64_t done_bar;        // all MMAs issued so far have completed (accumulator readable)
    uint32_t tmem_base;
    uint32_t pad;
};

struct Pipe {
    PipeShared *sh;
    uint8_t *a_stage[2];      // 1024-byte aligned, kAStageBytes each
    uint8_t *b_stage[2];      // 1024-byte aligned, (rows rounded up to 64) * 128 bytes each
    uint32_t iter = 0;        // stages filled so far (uniform over the CTA)
    uint32_t done_uses = 0;   // times done_bar has been waited on
    uint32_t tmem = 0;
    int *status;              // global status word: nonzero = a wait ran out
};

// Call once at kernel start by all threads.  ncols: power of two in [32, 512].
__device__ __forceinline__ void pipe_init(Pipe &p, PipeShared *sh, uint8_t *stage_mem, int b_stage_bytes, uint32_t ncols,
                                          int *status) {
    p.sh = sh;
    p.status = status;
    p.a_stage[0] = stage_mem;
    p.a_stage[1] = stage_mem + kAStageBytes;
    p.b_stage[0] = stage_mem + 2 * kAStageBytes;
    p.b_stage[1] = stage_mem + 2 * kAStageBytes + b_stage_bytes;
    if (threadIdx.x < 32) tmem_alloc(&sh->tmem_base, ncols);
    if (threadIdx.x == 32) {
        mbar_init(&sh->free_bar[0], 1);
        mbar_init(&sh->free_bar[1], 1);
        mbar_init(&sh->done_bar, 1);
        fence_mbar_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    p.tmem = sh->tmem_base;
}
__device__ __forceinline__ void pipe_destroy(Pipe &p, uint32_t ncols) {
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(p.tmem, ncols);
}

// Accumulate  D[128 x n_tile] (+)= A[128 x K] * B[n_tile x K]^T  into TMEM columns starting at d_tmem.
//   A_MN / B_MN: operand is staged MN-major (the functor yields 8 consecutive ROWS at one k) instead of K-major
//                (8 consecutive k of one row).
//   fa(r, k): K-major: elements (r, k..k+7);  MN-major: elements (r..r+7, k).   r, k multiples of 8 where chunked.
//   fb(r, k): same for B, r in [0, n_tile).  Functors return zeros outside the problem.
//   n_tile: multiple of 16, 16..256.   first_accumulate: 0 overwrites the accumulator at the first k-step.
// Returns false (uniformly over the CTA) if a wait ran out; the status word is set.
template <class T, bool A_MN, bool B_MN, int BCH = 8, class FA, class FB>
__device__ __forceinline__ bool umma_gemm(Pipe &p, uint32_t d_tmem, int n_tile, int K, uint32_t first_accumulate, FA fa,
                                          FB fb) {
    // BCH: 16-byte pieces of the B tile each thread stages per step; needs n_tile <= 32 * BCH.
    const uint32_t idesc = instr_desc(AbFmt<T>::v, A_MN, B_MN, n_tile);
    const int tid = threadIdx.x;
    const int nb_chunks = n_tile * 8;
    const int nrc = n_tile >> 3;
    uint4 ra[4], rb[BCH];
    // The operand pieces of step k0+64 are fetched into registers while step k0 is being handed to the tensor core,
    // so the global-memory latency of one step hides behind the barrier and the MMA issue of the previous one.
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int q = tid + i * kThreads;
            if (!A_MN) ra[i] = fa(q >> 3, k0 + (q & 7) * 8);
            else ra[i] = fa((q & 15) * 8, k0 + (q >> 4));
        }
#pragma unroll
        for (int i = 0; i < BCH; ++i) {
            const int q = tid + i * kThreads;
            if (q < nb_chunks) {
                if (!B_MN) rb[i] = fb(q >> 3, k0 + (q & 7) * 8);
                else rb[i] = fb((q % nrc) * 8, k0 + q / nrc);
            }
        }
    };
    auto stash = [&](int st) {
        uint8_t *as = p.a_stage[st], *bs = p.b_stage[st];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int q = tid + i * kThreads;
            if (!A_MN) {
                const int r = q >> 3, c = q & 7;
                *reinterpret_cast<uint4 *>(as + r * 128 + ((c ^ (r & 7)) << 4)) = ra[i];
            } else {
                const int rc = q & 15, k = q >> 4;          // rc: 8-row chunk index
                *reinterpret_cast<uint4 *>(as + (rc >> 3) * 8192 + (k >> 3) * 1024 + (k & 7) * 128 +
                                           (((rc & 7) ^ (k & 7)) << 4)) = ra[i];
            }
        }
#pragma unroll
        for (int i = 0; i < BCH; ++i) {
            const int q = tid + i * kThreads;
            if (q < nb_chunks) {
                if (!B_MN) {
                    const int r = q >> 3, c = q & 7;
                    *reinterpret_cast<uint4 *>(bs + r * 128 + ((c ^ (r & 7)) << 4)) = rb[i];
                } else {
                    const int rc = q % nrc, k = q / nrc;
                    *reinterpret_cast<uint4 *>(bs + (rc >> 3) * 8192 + (k >> 3) * 1024 + (k & 7) * 128 +
                                               (((rc & 7) ^ (k & 7)) << 4)) = rb[i];
                }
            }
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += kStageK) {
        const int st = p.iter & 1;
        bool ok = true;
        if (p.iter >= 2) ok = mbar_wait(&p.sh->free_bar[st], ((p.iter >> 1) - 1) & 1);
        if (ok) {
            stash(st);
            fence_async_smem();
            if (k0 + kStageK < K) fetch(k0 + kStageK);
        }
        ok = __syncthreads_and(ok);
        if (!ok) {
            if (tid == 0) atomicExch(p.status, kErrMmaTimeout);
            return false;
        }
        if (tid == 0) {
            tc_fence_after();
            const uint32_t a0 = smem_u32(p.a_stage[st]), b0 = smem_u32(p.b_stage[st]);
#pragma unroll
            for (int kk = 0; kk < kStageK / 16; ++kk) {
                const uint64_t ad = A_MN ? smem_desc(a0 + kk * 2048, 8192, 1024) : smem_desc(a0 + kk * 32, 16, 1024);
                const uint64_t bd = B_MN ? smem_desc(b0 + kk * 2048, 8192, 1024) : smem_desc(b0 + kk * 32, 16, 1024);
                umma(d_tmem, ad, bd, idesc, (k0 > 0 || kk > 0) ? 1u : first_accumulate);
            }
            umma_commit(&p.sh->free_bar[st]);
        }
        ++p.iter;
    }
    return true;
}

// Issue the four K=16 MMAs of one K=64 stage whose tiles the caller has already written (and fenced with
// fence_async_smem + a CTA barrier).  One thread calls this.  ab_fmt: 1 = bf16, 0 = f16.
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void umma_issue_stage(uint32_t d_tmem, int n_tile, int ab_fmt, const uint8_t *a_tile,
                                                 const uint8_t *b_tile, uint32_t first_accumulate) {
    const uint32_t idesc = instr_desc(ab_fmt, A_MN, B_MN, n_tile);
    const uint32_t a0 = smem_u32(a_tile), b0 = smem_u32(b_tile);
#pragma unroll
    for (int kk = 0; kk < kStageK / 16; ++kk) {
        const uint64_t ad = A_MN ? smem_desc(a0 + kk * 2048, 8192, 1024) : smem_desc(a0 + kk * 32, 16, 1024);
        const uint64_t bd = B_MN ? smem_desc(b0 + kk * 2048, 8192, 1024) : smem_desc(b0 + kk * 32, 16, 1024);
        umma(d_tmem, ad, bd, idesc, kk > 0 ? 1u : first_accumulate);
    }
}

// CTA-wide wait on an mbarrier phase: the first warp polls, the other warps sleep in the CTA barrier that hands its
// outcome to everyone.  (Measured on the one-shot kernels: no faster than every warp polling - mbarrier.try_wait
// suspends the pollers - so those keep their own waits; kernels with sixteen warps use this form.)
// Every thread of the CTA must call it; the result is uniform.  `ok_in`: a thread that has already seen a failure
// passes false, which skips its wait and makes the common result false.
__device__ __forceinline__ bool mbar_wait_cta(uint64_t *bar, uint32_t parity, bool ok_in = true) {
    bool ok = ok_in;
    if (threadIdx.x < 32) ok = ok && mbar_wait(bar, parity);
    return __syncthreads_and(ok);
}

// Wait until every MMA issued so far has completed, so the accumulators can be read with tmem_ld32.
__device__ __forceinline__ bool umma_drain(Pipe &p) {
    if (threadIdx.x == 0) umma_commit(&p.sh->done_bar);
    bool ok = mbar_wait(&p.sh->done_bar, p.done_uses & 1);
    ++p.done_uses;
    ok = __syncthreads_and(ok);
    if (!ok && threadIdx.x == 0) atomicExch(p.status, kErrMmaTimeout);
    tc_fence_after();
    return ok;
}

// Call between reading an accumulator with tmem_ld32 and overwriting it with a new GEMM.
__device__ __forceinline__ void tmem_reads_done() {
    tc_fence_before();
    __syncthreads();
}

}  // namespace tc
}  // namespace bissd
