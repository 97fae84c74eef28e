// C ABI of libbissd (declared in include/bissd.h): argument validation, workspace layout, kernel sequencing.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"
#include "simt_kernels.cuh"
#include "conv_kernels.cuh"
#include "norm_kernels.cuh"
#include "tc_intra.cuh"
#include "tc_intra_sums.cuh"
#include "tc_intra_grp.cuh"
#include "tc_kernels.cuh"
#include "tc_dbc_tma.cuh"
#include "tc_dcb_tma.cuh"
#include "tc_bmm_tma.cuh"
#include "tc_dx_tma.cuh"
#include "tc_scan_tma.cuh"
#include "tc_scan_ws.cuh"
#include "tc_selftest.cuh"
#include "tc_state_tma.cuh"

namespace bissd {

static thread_local char g_cuda_err[256] = "";

static int note_cuda(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return BISSD_OK;
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
    return BISSD_ERR_LAUNCH;
}

// ---- tracing: optional CUDA-event brackets around every kernel launch, and a launch counter -------------
struct TraceRec {
    const char *name;
    cudaEvent_t e0, e1;
};
static std::mutex g_trace_mu;
static std::vector<TraceRec> g_trace;
static std::atomic<int> g_trace_on{0};
static std::atomic<unsigned long long> g_launches{0};

struct TraceScope {
    const char *name;
    cudaStream_t s;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    TraceScope(const char *n, cudaStream_t st) : name(n), s(st) {
        if (g_trace_on.load(std::memory_order_relaxed)) {
            if (cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess) cudaEventRecord(e0, s);
            else e0 = e1 = nullptr;
        }
    }
    void end() {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (e0 && e1) {
            cudaEventRecord(e1, s);
            std::lock_guard<std::mutex> lk(g_trace_mu);
            g_trace.push_back(TraceRec{name, e0, e1});
        }
    }
};

// Launch `...` (a full kernel<<<>>>() expression) on stream `s`, count it, bracket it with events when tracing.
// Launch with programmatic stream serialisation: the kernel may be scheduled while its predecessor drains and
// waits for it in pdl_begin().  Only kernels that open with pdl_begin() go through here.  BISSD_NO_PDL=1 turns
// the attribute off (plain stream order).
static bool no_pdl() {
    static const bool v = std::getenv("BISSD_NO_PDL") != nullptr;
    return v;
}
template <class... Exp, class... Act>
static cudaError_t launch_pdl(void (*kernel)(Exp...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Act &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = no_pdl() ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Act>(args)...);
}

#define BISSD_LAUNCH_ON(stream, name, ...)                        \
    do {                                                          \
        TraceScope ts_(name, stream);                             \
        __VA_ARGS__;                                              \
        ts_.end();                                                \
        int rc_ = note_cuda(cudaGetLastError(), name);            \
        if (rc_ != BISSD_OK) return rc_;                          \
    } while (0)
#define BISSD_LAUNCH(name, ...) BISSD_LAUNCH_ON(s, name, __VA_ARGS__)

// A second stream for the two group-walking backward kernels whose results nothing reads before the last product with
// dCB (prev_terms_grp, dbc_accum_grp): they fork from the caller's stream after the dx kernel and join it again
// before that product, so that they share the GPU with the fused dCB / decay-gradient kernel, which depends on
// neither - each of the three leaves a seventh of the SMs idle when it runs alone.  Stream order as the caller sees it is unchanged, also
// under stream capture (the side stream joins the capture through the event).  A call leases one (stream, two events)
// set of its device for its duration; sets are created on first need - in practice by the first call on a device, so
// not inside a later capture.  BISSD_NO_SIDE=1 keeps everything on the caller's stream.
struct Side {
    cudaStream_t st = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    int dev = -1;
    bool busy = false;
};
static std::mutex g_side_mu;
static std::vector<Side *> g_side;
static Side *side_acquire(cudaStream_t s) {
    static const bool off = [] { const char *e = getenv("BISSD_NO_SIDE"); return e && e[0] == '1'; }();
    if (off || g_trace_on.load(std::memory_order_relaxed)) return nullptr;   // traced runs time every kernel alone, in line
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lk(g_side_mu);
    for (Side *sd : g_side)
        if (sd->dev == dev && !sd->busy) {
            sd->busy = true;
            return sd;
        }
    // nothing free: make a set - but not while the caller's stream is being captured (creation belongs outside a capture)
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return nullptr;
    }
    cudaStream_t st = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&e0, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&e1, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;                                           // no side stream: the launch stays in line
    }
    Side *sd = new Side;
    sd->st = st; sd->fork = e0; sd->join = e1; sd->dev = dev; sd->busy = true;
    g_side.push_back(sd);
    return sd;
}
struct SideLease {                                                // gives the set back when the call returns
    Side *sd = nullptr;
    ~SideLease() {
        if (sd) {
            std::lock_guard<std::mutex> lk(g_side_mu);
            sd->busy = false;
        }
    }
};

// C and B as (dstate, group, seqlen, batch) tensors read in boxes of 64 state columns x 128 rows
template <class Args> static bool make_cb_maps(const Args &a, const Dims &d, CUtensorMap *mC, CUtensorMap *mB) {
    const unsigned long long dims[4] = {(unsigned long long)d.N, (unsigned long long)d.G, (unsigned long long)d.L, (unsigned long long)d.b};
    const unsigned long long sC[3] = {(unsigned long long)a.C.stride_head * 2, (unsigned long long)a.C.stride_seq * 2, (unsigned long long)a.C.stride_batch * 2};
    const unsigned long long sB[3] = {(unsigned long long)a.B.stride_head * 2, (unsigned long long)a.B.stride_seq * 2, (unsigned long long)a.B.stride_batch * 2};
    const unsigned box[4] = {64, 1, 128, 1};
    return tc::make_map4(mC, a.p.x_dtype, a.C.ptr, dims, sC, box) && tc::make_map4(mB, a.p.x_dtype, a.B.ptr, dims, sB, box);
}

static int make_dims(const bissd_problem &p, Dims *d) {
    if (p.batch <= 0 || p.seqlen <= 0 || p.nheads <= 0 || p.headdim <= 0 || p.ngroups <= 0 || p.dstate <= 0)
        return BISSD_ERR_SHAPE;
    if (p.nheads % p.ngroups != 0) return BISSD_ERR_SHAPE;
    // the reference requires chunk_size >= 32 (src/ssd/bi/ssd_combined.py:306); 256 is this library's ceiling
    if (p.chunk_size < 32 || p.chunk_size > 256) return BISSD_ERR_SHAPE;
    if (p.x_dtype < BISSD_F32 || p.x_dtype > BISSD_F16 || p.dt_dtype < BISSD_F32 || p.dt_dtype > BISSD_F16)
        return BISSD_ERR_DTYPE;
    d->b = p.batch; d->L = p.seqlen; d->H = p.nheads; d->P = p.headdim; d->G = p.ngroups; d->N = p.dstate;
    d->Q = p.chunk_size; d->nc = ceil_div(p.seqlen, p.chunk_size); d->R = p.nheads / p.ngroups;
    d->has_D = p.has_D; d->D_hdim = p.D_has_hdim; d->has_z = p.has_z; d->has_bias = p.has_dt_bias;
    d->softplus = p.dt_softplus; d->dt_min = p.dt_min; d->dt_max = p.dt_max;
    return BISSD_OK;
}

static inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

// Workspace carving.  The first 256 bytes hold the device status word (nonzero = a bounded device-side wait ran
// out); everything after it is fp32 scratch.
constexpr size_t kWsHeader = 256;
struct FwdWs {
    size_t loc, cb, cb16, total;
};
struct BwdWs {
    size_t cb, cbt, cbt16, cb16, cbs, gloc, E, E16, g, dTpart, ddt_out, nf, nb, pf, pb, da_f, da_b, u4, dB_part, dC_part, dCB, dDpart, dApart, dbiaspart, total;
    int nblk, nlt, nsplit;
};

static FwdWs fwd_layout(const Dims &d) {
    FwdWs w;
    size_t o = kWsHeader;
    const size_t st = (size_t)d.b * d.nc * d.H * d.P * d.N;
    w.loc = o; o = align256(o + 2 * st * 4);
    w.cb = o; o = align256(o + (size_t)d.b * d.nc * d.G * d.Q * d.Q * 4);
    w.cb16 = o; o = align256(o + (size_t)d.b * d.nc * d.G * d.Q * d.Q * 2);      // C.B^T rounded to bf16 (TMA-fed scan)
    w.total = o;
    return w;
}

// tc: sized for the tensor-core family (16-bit inputs that meet its alignment rules): the passed state gradients are
// kept in the input dtype only, and the "states" parts of dB / dC arrive summed over the heads of a group.  The
// CUDA-core family needs the fp32 copy and one partial per head.
static BwdWs bwd_layout(const Dims &d, bool tc) {
    BwdWs w;
    size_t o = kWsHeader;
    const size_t st = (size_t)d.b * d.nc * d.H * d.P * d.N;
    const size_t hq = (size_t)d.b * d.H * d.nc * d.Q;
    w.nblk = ceil_div(d.P * d.N, simt::TB);
    w.nlt = ceil_div(d.Q, simt::TILE);
    w.nsplit = ceil_div(d.N, 128);
    auto take = [&](size_t bytes) { size_t at = o; o = align256(o + bytes); return at; };
    w.cb = take((size_t)d.b * d.nc * d.G * d.Q * d.Q * 4);
    w.gloc = take(2 * st * 4);
    w.E = take(tc ? 0 : 2 * st * 4);                                 // fp32 passed state gradients (CUDA-core family)
    w.E16 = take(2 * st * 2);                                        // passed state gradients in the input dtype
    w.g = take((size_t)d.b * d.L * d.H * d.P * 2);                   // gated output gradient dout * silu(z)
    w.cbt = take((size_t)d.b * d.nc * d.G * d.Q * d.Q * 4);          // CB transposed
    w.cbs = take((size_t)d.b * d.nc * d.G * d.Q * d.Q * 4);          // CB in strips of 16 columns (tc::intra_sums)
    w.cbt16 = take((size_t)d.b * d.nc * d.G * d.Q * d.Q * 2);        // CB transposed, rounded to bf16 (TMA-fed dx)
    w.cb16 = take((size_t)d.b * d.nc * d.G * d.Q * d.Q * 2);         // CB rounded to bf16 (tc::intra_dcb_tile)
    w.dTpart = take((size_t)2 * d.b * d.H * d.nc * w.nblk * 4);
    w.ddt_out = take(hq * 4);
    w.nf = take(hq * 4 * w.nsplit); w.nb = take(hq * 4 * w.nsplit);
    w.pf = take(hq * 4 * w.nsplit); w.pb = take(hq * 4 * w.nsplit);
    w.da_f = take(hq * 4); w.da_b = take(hq * 4);
    w.u4 = take(8 * hq * 4);                                         // u_f / u_b per tile (tc::intra_sums: 2 row tiles; tc::intra_dcb_tile: 4)
    w.dB_part = take((size_t)d.b * d.nc * d.Q * (tc ? d.G : d.H) * d.N * 4);
    w.dC_part = take((size_t)d.b * d.nc * d.Q * (tc ? d.G : d.H) * d.N * 4);
    w.dCB = take((size_t)d.b * d.nc * d.G * d.Q * d.Q * 4);
    w.dDpart = take((size_t)d.b * d.nc * d.H * std::max(w.nlt, 8) * d.P * 4);   // up to 8 partial rows per (b,c,h)
    w.dApart = take((size_t)d.b * d.nc * d.H * 4);
    w.dbiaspart = take((size_t)d.b * d.nc * d.H * 4);
    w.total = o;
    return w;
}

static View view_of(const bissd_tensor &t) { return View{t.ptr, t.stride_batch, t.stride_seq, t.stride_head}; }
static MutView mview_of(const bissd_tensor &t) { return MutView{t.ptr, t.stride_batch, t.stride_seq, t.stride_head}; }

// Raise a kernel's dynamic shared-memory limit.  The attribute is per (function, device) and sticks, so it is set the
// first time a kernel needs `bytes` on a device and remembered (the driver call costs a microsecond or two per launch
// otherwise - a tenth of the host time of a whole pass).
static std::mutex g_smem_mu;
static std::map<std::pair<const void *, int>, size_t> g_smem_granted;   // (kernel, device) -> bytes already allowed
template <class K> static int allow_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return BISSD_OK;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
    const std::pair<const void *, int> key(reinterpret_cast<const void *>(kernel), dev);
    if (dev >= 0) {
        std::lock_guard<std::mutex> lk(g_smem_mu);
        auto it = g_smem_granted.find(key);
        if (it != g_smem_granted.end() && it->second >= bytes) return BISSD_OK;
    }
    int rc = note_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes),
                       "cudaFuncSetAttribute");
    if (rc == BISSD_OK && dev >= 0) {
        std::lock_guard<std::mutex> lk(g_smem_mu);
        size_t &g = g_smem_granted[key];
        g = std::max(g, bytes);
    }
    return rc;
}

// ---- which kernel family ---------------------------------------------------------------------------------
static bool tc_shape_ok(const bissd_problem &p) {
    return (p.x_dtype == BISSD_BF16 || p.x_dtype == BISSD_F16) && p.headdim % 8 == 0 && p.dstate % 8 == 0 &&
           p.chunk_size % 8 == 0 && p.headdim <= 256 && p.dstate <= 256;
}
static bool aligned16(const bissd_tensor &t) {
    if (!t.ptr) return true;
    return (reinterpret_cast<uintptr_t>(t.ptr) % 16 == 0) && t.stride_batch % 8 == 0 && t.stride_seq % 8 == 0 &&
           t.stride_head % 8 == 0;
}
static bool force_simt() {
    static const bool v = [] { const char *e = getenv("BISSD_FORCE_SIMT"); return e && e[0] == '1'; }();
    return v;
}

static bool no_ws() {    // BISSD_NO_WS=1: keep the one-tile-per-CTA TMA kernels where a persistent variant exists
    static const bool v = [] { const char *e = getenv("BISSD_NO_WS"); return e && e[0] == '1'; }();
    return v;
}
static int sm_count() {
    static int n[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!n[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n[dev] = v;
    }
    return n[dev];
}

static bool no_sums() {  // BISSD_NO_SUMS=1: keep the prefix-sweep form of the intra-chunk decay gradient
    static const bool v = [] { const char *e = getenv("BISSD_NO_SUMS"); return e && e[0] == '1'; }();
    return v;
}

static bool no_fused() {  // BISSD_NO_FUSED=1: separate dCB and intra-chunk decay-gradient kernels (for A/B comparisons)
    static const bool v = [] { const char *e = getenv("BISSD_NO_FUSED"); return e && e[0] == '1'; }();
    return v;
}

static bool no_tma() {   // BISSD_NO_TMA=1: keep the thread-staged tcgen05 kernels (for A/B comparisons)
    static const bool v = [] { const char *e = getenv("BISSD_NO_TMA"); return e && e[0] == '1'; }();
    return v;
}

// rank-4 tensor map over a (batch, seq, head, inner) 16-bit tensor; box = [64 inner, 1 head, rows seq, 1 batch]
static bool map_bshd(CUtensorMap *m, int dtype, const void *ptr, long long sb, long long sl, long long sh, int inner,
                     int heads, int seqlen, int batch, unsigned rows) {
    const unsigned long long dims[4] = {(unsigned long long)inner, (unsigned long long)heads, (unsigned long long)seqlen,
                                        (unsigned long long)batch};
    const unsigned long long str[3] = {(unsigned long long)sh * 2, (unsigned long long)sl * 2, (unsigned long long)sb * 2};
    const unsigned box[4] = {64, 1, rows, 1};
    return tc::make_map4(m, dtype, ptr, dims, str, box);
}

#define BISSD_ALLOW(kernel, bytes)                  \
    do {                                             \
        int rc_ = allow_smem(kernel, bytes);         \
        if (rc_ != BISSD_OK) return rc_;             \
    } while (0)

template <class T> struct TcKernels {   // 16-bit types only; the fp32 specialisation below never launches them
    static constexpr bool available = true;
};
template <> struct TcKernels<float> { static constexpr bool available = false; };

template <class T>
static int forward_impl(const bissd_fwd_args &a, const Dims &d, char *ws, cudaStream_t s, bool tcp) {
    const FwdWs w = fwd_layout(d);
    int *status = reinterpret_cast<int *>(ws);
    float *loc = reinterpret_cast<float *>(ws + w.loc);
    float *CB = reinterpret_cast<float *>(ws + w.cb);
    const View x = view_of(a.x), Bm = view_of(a.B), Cm = view_of(a.C), z = view_of(a.z);
    const int bch = d.b * d.nc * d.H;
    const int ntP = tc::round_up(d.P, 16), ntQ = tc::round_up(d.Q, 16);
    if (a.phases & BISSD_PHASE_LOCAL) {
        int rc = note_cuda(cudaMemsetAsync(ws, 0, kWsHeader, s), "cudaMemsetAsync");
        if (rc != BISSD_OK) return rc;
        BISSD_LAUNCH("cumsum_fwd", launch_pdl(simt::cumsum_fwd, d.b * d.nc * d.H, 256, 0, s, 
            d, a.dt.ptr, a.p.dt_dtype, a.dt.stride_batch, a.dt.stride_seq, a.dt.stride_head, a.A, a.dt_bias, a.dt_out,
            a.cs_f, a.cs_b));
        if constexpr (TcKernels<T>::available) {
            if (tcp) {
                const size_t smem = tc::smem_bytes(ntP, 2 * d.Q);
                bool st_done = false;
                if (!no_tma() && (tc::state_tma_ok(d.P, d.N, d.Q) || (!no_ws() && tc::state_grp_ok(d.P, d.N, d.Q, d.R)))) {
                    CUtensorMap mRow, mCol;
                    if (map_bshd(&mRow, a.p.x_dtype, a.B.ptr, a.B.stride_batch, a.B.stride_seq, a.B.stride_head, d.N, d.G, d.L, d.b, d.Q) &&
                        map_bshd(&mCol, a.p.x_dtype, a.x.ptr, a.x.stride_batch, a.x.stride_seq, a.x.stride_head, d.P, d.H, d.L, d.b, d.Q)) {
                        if (!no_ws() && tc::state_grp_ok(d.P, d.N, d.Q, d.R)) {
                            const size_t smem_g = tc::state_grp_smem(d.Q);
                            const int ks = tc::state_grp_ksplit(d.b * d.nc * d.G * ceil_div(d.N, 128), d.R, sm_count());
                            BISSD_ALLOW((tc::state_gemm_grp<T, 0>), smem_g);
                            BISSD_LAUNCH("tc_chunk_state_grp", launch_pdl(tc::state_gemm_grp<T, 0>, dim3(d.b * d.nc * d.G * ks, ceil_div(d.N, 128)), tc::kStateGrpThreads, smem_g, s, 
                                d, mRow, mCol, ks, a.dt_out, a.cs_f, a.cs_b, loc, status));
                        } else {
                            const size_t smem_t = tc::state_tma_smem(d.P, d.Q);
                            BISSD_ALLOW((tc::state_gemm_tma<T, 0>), smem_t);
                            BISSD_LAUNCH("tc_chunk_state_tma", tc::state_gemm_tma<T, 0><<<dim3(bch, 2, d.N / 128), tc::kThreads, smem_t, s>>>(
                                d, mRow, mCol, a.dt_out, a.cs_f, a.cs_b, loc, status));
                        }
                        st_done = true;
                    }
                }
                if (st_done) {
                } else if (ntP <= 64) {
                    BISSD_ALLOW((tc::state_gemm<T, 0, 2>), smem);
                    BISSD_LAUNCH("tc_chunk_state", tc::state_gemm<T, 0, 2><<<dim3(bch, ceil_div(2 * d.N, tc::kTileM)), tc::kThreads, smem, s>>>(
                        d, Bm, x, z, a.dt_out, a.cs_f, a.cs_b, loc, status));
                } else {
                    BISSD_ALLOW((tc::state_gemm<T, 0, 8>), smem);
                    BISSD_LAUNCH("tc_chunk_state", tc::state_gemm<T, 0, 8><<<dim3(bch, ceil_div(2 * d.N, tc::kTileM)), tc::kThreads, smem, s>>>(
                        d, Bm, x, z, a.dt_out, a.cs_f, a.cs_b, loc, status));
                }
            }
        }
        if (!tcp) {
            BISSD_LAUNCH("chunk_state", simt::chunk_state<T><<<dim3(bch, ceil_div(d.P, simt::TILE), ceil_div(2 * d.N, simt::TILE)), simt::TB, 2 * d.Q * sizeof(float), s>>>(
                d, x, Bm, a.dt_out, a.cs_f, a.cs_b, loc));
        }
    }
    // the recurrence runs in both phases: from zero (or init_*) in LOCAL, again with init_* in FINISH
    const bool need_pass = (a.phases & BISSD_PHASE_LOCAL) || (a.init_f || a.init_b);
    if (need_pass) {
        if ((d.P * d.N) % 4 == 0) {
            BISSD_LAUNCH("state_passing_fwd", launch_pdl(simt::state_passing_fwd4<T>, dim3(d.b * d.H, ceil_div(d.P * d.N, 4 * simt::TB), 2), simt::TB, 0, s, 
                d, loc, a.cs_f, a.cs_b, a.init_f, a.init_b, a.states_f, a.states_b, a.final_f, a.final_b));
        } else {
            BISSD_LAUNCH("state_passing_fwd", simt::state_passing_fwd<T><<<dim3(d.b * d.H, ceil_div(d.P * d.N, simt::TB), 2), simt::TB, 0, s>>>(
                d, loc, a.cs_f, a.cs_b, a.init_f, a.init_b, a.states_f, a.states_b, a.final_f, a.final_b));
        }
    }
    if (a.phases & BISSD_PHASE_FINISH) {
        if constexpr (TcKernels<T>::available) {
            if (tcp) {
                const size_t smem_cb = tc::smem_bytes(ntQ, 0), smem_sc = tc::smem_bytes(ntP, 3 * d.Q);
                BISSD_ALLOW(tc::bmm_cb<T>, smem_cb);
                const bool ws_path = !no_tma() && !no_ws() && tc::scan_ws_ok(d.P, d.N, d.Q);
                __nv_bfloat16 *CB16 = reinterpret_cast<__nv_bfloat16 *>(ws + w.cb16);
                CUtensorMap mCc, mBc;
                if (ws_path && tc::bmm_cb_tma_ok(d.N, d.Q) && make_cb_maps(a, d, &mCc, &mBc)) {
                    const size_t smem_ct = tc::bmm_cb_tma_smem(d.N);
                    BISSD_ALLOW(tc::bmm_cb_tma<T>, smem_ct);
                    BISSD_LAUNCH("tc_bmm_cb_tma", launch_pdl(tc::bmm_cb_tma<T>, dim3(d.b * d.nc * d.G, d.Q / 128, d.Q / 128), tc::kThreads, smem_ct, s, 
                        d, mCc, mBc, CB16, nullptr, nullptr, status));
                } else
                BISSD_LAUNCH("tc_bmm_cb", tc::bmm_cb<T><<<dim3(d.b * d.nc * d.G, ceil_div(d.Q, tc::kTileM)), tc::kThreads, smem_cb, s>>>(
                    d, Cm, Bm, ws_path ? nullptr : CB, nullptr, ws_path ? CB16 : nullptr, nullptr, nullptr, status));
                bool tma_done = false;
                if (ws_path) {
                    CUtensorMap mC, mCB, mSf, mSb, mX, mR;
                    const unsigned long long dC[4] = {(unsigned long long)d.N, (unsigned long long)d.G, (unsigned long long)d.L, (unsigned long long)d.b};
                    const unsigned long long sC[3] = {(unsigned long long)a.C.stride_head * 2, (unsigned long long)a.C.stride_seq * 2, (unsigned long long)a.C.stride_batch * 2};
                    const unsigned bC[4] = {64, 1, 128, 1};
                    const unsigned long long rows = (unsigned long long)d.b * d.nc * d.H * d.P;
                    bool maps = tc::make_map4(&mC, a.p.x_dtype, a.C.ptr, dC, sC, bC) &&
                                map_bshd(&mX, a.p.x_dtype, a.x.ptr, a.x.stride_batch, a.x.stride_seq, a.x.stride_head, d.P, d.H, d.L, d.b, 64) &&
                                tc::make_map2(&mCB, BISSD_BF16, CB16, d.Q, (unsigned long long)d.b * d.nc * d.G * d.Q, 64, 128) &&
                                tc::make_map2(&mSf, a.p.x_dtype, a.states_f, d.N, rows, 64, d.P) &&
                                tc::make_map2(&mSb, a.p.x_dtype, a.states_b, d.N, rows, 64, d.P);
                    // the epilogue's z rows by TMA (a [128 rows x 64] tile per step); without z the map is not used
                    const bool z_rows = maps && d.has_z &&
                                        map_bshd(&mR, a.p.x_dtype, a.z.ptr, a.z.stride_batch, a.z.stride_seq, a.z.stride_head, d.P, d.H, d.L, d.b, 128);
                    if (maps && !z_rows) mR = mX;
                    if (maps) {
                        const size_t smem_t = tc::scan_ws_smem(d.P, d.N, d.Q);
                        const int tiles = bch * (d.Q / tc::kTileM);
                        const int grid = std::min(sm_count(), tiles);
                        auto wide = [](const bissd_tensor &t) {   // 32-byte accesses allowed on every row piece
                            return t.ptr && reinterpret_cast<uintptr_t>(t.ptr) % 32 == 0 && t.stride_batch % 16 == 0 &&
                                   t.stride_seq % 16 == 0 && t.stride_head % 16 == 0;
                        };
                        const int wide_z = d.has_z && wide(a.z);
                        const int wide_o = wide(a.out) && (!d.has_z || wide(a.out_x));
                        tc::WsArgs wa{};
                        wa.x = x; wa.z = z; wa.D = a.D; wa.dt_out = a.dt_out; wa.cs_f = a.cs_f; wa.cs_b = a.cs_b;
                        wa.out = mview_of(a.out); wa.out_x = mview_of(a.out_x);
                        wa.wide_z = wide_z; wa.wide_o = wide_o;
                        wa.rows_by_tma = z_rows ? 1 : 0;
#define BISSD_SCAN_WS(NSL, NS)                                                                                          \
    do {                                                                                                                \
        BISSD_ALLOW((tc::ws_kernel<T, NSL, NS, 0>), smem_t);                                                            \
        BISSD_LAUNCH("tc_chunk_scan_ws", launch_pdl(tc::ws_kernel<T, NSL, NS, 0>, grid, tc::kWsThreads, smem_t, s,              \
            d, mC, mCB, mSf, mSb, mX, mR, wa, status));                                                                 \
    } while (0)
                        if (d.N == 128 && d.Q == 256) BISSD_SCAN_WS(2, 4);
                        else if (d.N == 64 && d.Q == 256) BISSD_SCAN_WS(1, 4);
                        else if (d.N == 128 && d.Q == 128) BISSD_SCAN_WS(2, 2);
                        else BISSD_SCAN_WS(1, 2);
#undef BISSD_SCAN_WS
                        tma_done = true;
                    } else {                                     // maps refused: produce the fp32 tile after all
                        BISSD_LAUNCH("tc_bmm_cb", tc::bmm_cb<T><<<dim3(d.b * d.nc * d.G, ceil_div(d.Q, tc::kTileM)), tc::kThreads, smem_cb, s>>>(
                            d, Cm, Bm, CB, nullptr, nullptr, nullptr, nullptr, status));
                    }
                }
                if (!tma_done && !no_tma() && tc::scan_tma_ok(d.P, d.N, d.Q)) {
                    CUtensorMap mC, mSf, mSb, mX;
                    const unsigned long long dC[4] = {(unsigned long long)d.N, (unsigned long long)d.G, (unsigned long long)d.L, (unsigned long long)d.b};
                    const unsigned long long sC[3] = {(unsigned long long)a.C.stride_head * 2, (unsigned long long)a.C.stride_seq * 2, (unsigned long long)a.C.stride_batch * 2};
                    const unsigned bC[4] = {64, 1, 128, 1};
                    const unsigned long long dX[4] = {(unsigned long long)d.P, (unsigned long long)d.H, (unsigned long long)d.L, (unsigned long long)d.b};
                    const unsigned long long sX[3] = {(unsigned long long)a.x.stride_head * 2, (unsigned long long)a.x.stride_seq * 2, (unsigned long long)a.x.stride_batch * 2};
                    const unsigned bX[4] = {64, 1, (unsigned)d.Q, 1};
                    const unsigned long long rows = (unsigned long long)d.b * d.nc * d.H * d.P;
                    if (tc::make_map4(&mC, a.p.x_dtype, a.C.ptr, dC, sC, bC) && tc::make_map4(&mX, a.p.x_dtype, a.x.ptr, dX, sX, bX) &&
                        tc::make_map2(&mSf, a.p.x_dtype, a.states_f, d.N, rows, 64, d.P) &&
                        tc::make_map2(&mSb, a.p.x_dtype, a.states_b, d.N, rows, 64, d.P)) {
                        const int rounds = tc::scan_tma_rounds(d.P, d.N, d.Q);
                        const size_t smem_t = tc::scan_tma_smem(d.P, d.N, d.Q, rounds);
                        BISSD_ALLOW(tc::chunk_scan_tma<T>, smem_t);
                        BISSD_LAUNCH("tc_chunk_scan_tma", tc::chunk_scan_tma<T><<<dim3(bch, ceil_div(d.Q, tc::kTileM)), tc::kThreads, smem_t, s>>>(
                            d, mC, mSf, mSb, mX, x, z, a.D, a.dt_out, a.cs_f, a.cs_b, CB, mview_of(a.out), mview_of(a.out_x), rounds, status));
                        tma_done = true;
                    }
                }
                if (tma_done) {
                } else if (ntP <= 64) {
                    BISSD_ALLOW((tc::chunk_scan<T, 2>), smem_sc);
                    BISSD_LAUNCH("tc_chunk_scan", tc::chunk_scan<T, 2><<<dim3(bch, ceil_div(d.Q, tc::kTileM)), tc::kThreads, smem_sc, s>>>(
                        d, x, Cm, z, a.D, a.dt_out, a.cs_f, a.cs_b, CB, a.states_f, a.states_b, mview_of(a.out), mview_of(a.out_x), status));
                } else {
                    BISSD_ALLOW((tc::chunk_scan<T, 8>), smem_sc);
                    BISSD_LAUNCH("tc_chunk_scan", tc::chunk_scan<T, 8><<<dim3(bch, ceil_div(d.Q, tc::kTileM)), tc::kThreads, smem_sc, s>>>(
                        d, x, Cm, z, a.D, a.dt_out, a.cs_f, a.cs_b, CB, a.states_f, a.states_b, mview_of(a.out), mview_of(a.out_x), status));
                }
            }
        }
        if (!tcp) {
            BISSD_LAUNCH("bmm_cb", simt::bmm_cb<T><<<dim3(d.b * d.nc * d.G, ceil_div(d.Q, simt::TILE), ceil_div(d.Q, simt::TILE)), simt::TB, 0, s>>>(d, Cm, Bm, CB));
            BISSD_LAUNCH("chunk_scan", simt::chunk_scan<T><<<dim3(bch, ceil_div(d.Q, simt::TILE), ceil_div(d.P, simt::TILE)), simt::TB, 3 * d.Q * sizeof(float), s>>>(
                d, x, Cm, z, a.D, a.dt_out, a.cs_f, a.cs_b, CB, a.states_f, a.states_b, mview_of(a.out), mview_of(a.out_x)));
        }
    }
    return BISSD_OK;
}

template <class T>
static int backward_impl(const bissd_bwd_args &a, const Dims &d, char *ws, cudaStream_t s, bool tcp) {
    const BwdWs w = bwd_layout(d, tcp);
    int *status = reinterpret_cast<int *>(ws);
    auto F = [&](size_t off) { return reinterpret_cast<float *>(ws + off); };
    const View x = view_of(a.x), Bm = view_of(a.B), Cm = view_of(a.C), z = view_of(a.z), dout = view_of(a.dout),
               out_x = view_of(a.out_x);
    const int bch = d.b * d.nc * d.H;
    const size_t q3 = 3 * d.Q * sizeof(float);
    const int ntP = tc::round_up(d.P, 16), ntQ = tc::round_up(d.Q, 16), ntN = std::min(tc::round_up(d.N, 16), 128);
    const int nlt_tc = ceil_div(d.Q, tc::kTileM);
    // Tensor-core family: the gate is applied once (gate_bwd writes g = dout * silu(z) and dz); every later kernel
    // then sees an ungated problem whose output gradient is g.
    Dims dg = d;
    View gv = dout;
    void *E16 = ws + w.E16;
    if (tcp && d.has_z) {
        dg.has_z = 0;
        gv = View{ws + w.g, (long long)d.L * d.H * d.P, (long long)d.H * d.P, (long long)d.P};
    }
    if (a.phases & BISSD_PHASE_LOCAL) {
        int rc = note_cuda(cudaMemsetAsync(ws, 0, kWsHeader, s), "cudaMemsetAsync");
        if (rc != BISSD_OK) return rc;
        if constexpr (TcKernels<T>::available) {
            if (tcp && d.has_z) {
                const long long chunks = (long long)d.b * d.L * d.H * (d.P / 8);
                BISSD_LAUNCH("gate_bwd", launch_pdl(tc::gate_bwd<T>, (unsigned)((chunks + 255) / 256), 256, 0, s, 
                    d, dout, z, out_x, ws + w.g, a.dz));
            }
            if (tcp) {
                const size_t smem = tc::smem_bytes(ntP, 2 * d.Q);
                bool st_done = false;
                if (!no_tma() && (tc::state_tma_ok(d.P, d.N, d.Q) || (!no_ws() && tc::state_grp_ok(d.P, d.N, d.Q, d.R)))) {
                    CUtensorMap mRow, mCol;
                    if (map_bshd(&mRow, a.p.x_dtype, a.C.ptr, a.C.stride_batch, a.C.stride_seq, a.C.stride_head, d.N, d.G, d.L, d.b, d.Q) &&
                        map_bshd(&mCol, a.p.x_dtype, gv.ptr, gv.sb, gv.sl, gv.sh, d.P, d.H, d.L, d.b, d.Q)) {
                        if (!no_ws() && tc::state_grp_ok(d.P, d.N, d.Q, d.R)) {
                            const size_t smem_g = tc::state_grp_smem(d.Q);
                            const int ks = tc::state_grp_ksplit(d.b * d.nc * d.G * ceil_div(d.N, 128), d.R, sm_count());
                            BISSD_ALLOW((tc::state_gemm_grp<T, 1>), smem_g);
                            BISSD_LAUNCH("tc_dstates_grp", launch_pdl(tc::state_gemm_grp<T, 1>, dim3(d.b * d.nc * d.G * ks, ceil_div(d.N, 128)), tc::kStateGrpThreads, smem_g, s, 
                                d, mRow, mCol, ks, a.dt_out, a.cs_f, a.cs_b, F(w.gloc), status));
                        } else {
                            const size_t smem_t = tc::state_tma_smem(d.P, d.Q);
                            BISSD_ALLOW((tc::state_gemm_tma<T, 1>), smem_t);
                            BISSD_LAUNCH("tc_dstates_tma", tc::state_gemm_tma<T, 1><<<dim3(bch, 2, d.N / 128), tc::kThreads, smem_t, s>>>(
                                d, mRow, mCol, a.dt_out, a.cs_f, a.cs_b, F(w.gloc), status));
                        }
                        st_done = true;
                    }
                }
                if (st_done) {
                } else if (ntP <= 64) {
                    BISSD_ALLOW((tc::state_gemm<T, 1, 2>), smem);
                    BISSD_LAUNCH("tc_dstates", tc::state_gemm<T, 1, 2><<<dim3(bch, ceil_div(2 * d.N, tc::kTileM)), tc::kThreads, smem, s>>>(
                        dg, Cm, gv, z, a.dt_out, a.cs_f, a.cs_b, F(w.gloc), status));
                } else {
                    BISSD_ALLOW((tc::state_gemm<T, 1, 8>), smem);
                    BISSD_LAUNCH("tc_dstates", tc::state_gemm<T, 1, 8><<<dim3(bch, ceil_div(2 * d.N, tc::kTileM)), tc::kThreads, smem, s>>>(
                        dg, Cm, gv, z, a.dt_out, a.cs_f, a.cs_b, F(w.gloc), status));
                }
            }
        }
        if (!tcp) {
            BISSD_LAUNCH("dstates", simt::dstates<T><<<dim3(bch, ceil_div(d.P, simt::TILE), ceil_div(2 * d.N, simt::TILE)), simt::TB, 2 * d.Q * sizeof(float), s>>>(
                d, dout, z, Cm, a.cs_f, a.cs_b, F(w.gloc)));
        }
    }
    const bool need_pass = (a.phases & BISSD_PHASE_LOCAL) || (a.dfinal_f || a.dfinal_b);
    int pass_nblk = ((d.P * d.N) % 4 == 0) ? ceil_div(d.P * d.N, 4 * simt::TB) : w.nblk;   // dT partial slots per chunk
    if (need_pass) {
        if ((d.P * d.N) % 4 == 0) {
            pass_nblk = ceil_div(d.P * d.N, 4 * simt::TB);
            BISSD_LAUNCH("state_passing_bwd", launch_pdl(simt::state_passing_bwd4<T>, dim3(d.b * d.H, pass_nblk, 2), simt::TB, 0, s, 
                d, F(w.gloc), a.states_f, a.states_b, a.cs_f, a.cs_b, a.dfinal_f, a.dfinal_b, tcp ? nullptr : F(w.E), tcp ? E16 : nullptr, F(w.dTpart), a.dinit_f, a.dinit_b));
        } else {
            BISSD_LAUNCH("state_passing_bwd", simt::state_passing_bwd<T><<<dim3(d.b * d.H, w.nblk, 2), simt::TB, 0, s>>>(
                d, F(w.gloc), a.states_f, a.states_b, a.cs_f, a.cs_b, a.dfinal_f, a.dfinal_b, tcp ? nullptr : F(w.E), tcp ? E16 : nullptr, F(w.dTpart), a.dinit_f, a.dinit_b));
        }
    }
    if (!(a.phases & BISSD_PHASE_FINISH)) return BISSD_OK;
    int nlt = w.nlt, nsplit = 1, part_heads = d.H;
    bool have_fp32_cb = true;                                    // fp32 CB (and its transpose) are in the workspace
    bool use_u4 = false;                                         // decay gradients arrive as u_f / u_b (tc::intra_sums)
    bool fused_cb = false;                                       // the bf16 C.B^T tile for tc::intra_dcb_tile has been written
    SideLease lease;
    cudaStream_t s_side = s;                                     // where prev_terms_grp and dbc_accum_grp are launched
    int u4_tiles = 2;                                            // (u_f, u_b) vector pairs per chunk in u4
    int dd_slots = 0;                                            // dD partial rows per (b,c,h) when not nlt
    bool dd_compact = false;                                     // per-head D from the persistent dx kernel: dd_slots scalars, no channel axis
    if constexpr (TcKernels<T>::available) {
        if (tcp) {
            nlt = nlt_tc;
            nsplit = w.nsplit;
            part_heads = d.G;
            const size_t smem_cb = tc::smem_bytes(ntQ, 0), smem_dx = tc::smem_bytes(ntP, 3 * d.Q), smem_n = tc::smem_bytes(ntN, 0);
            BISSD_ALLOW(tc::bmm_cb<T>, smem_cb);
            const bool ws_path = !no_tma() && !no_ws() && tc::scan_ws_ok(d.P, d.N, d.Q);
            const bool sums_path = !no_tma() && !no_sums() && tc::scan_tma_ok(d.P, d.N, d.Q);
            __nv_bfloat16 *CBt16 = reinterpret_cast<__nv_bfloat16 *>(ws + w.cbt16);
            __nv_bfloat16 *CB16b = reinterpret_cast<__nv_bfloat16 *>(ws + w.cb16);
            CUtensorMap mCc, mBc;
            if (ws_path && sums_path && tc::bmm_cb_tma_ok(d.N, d.Q) && make_cb_maps(a, d, &mCc, &mBc)) {
                // the fused dCB / decay-gradient kernel reads the bf16 tile by TMA; the separate intra_sums kernel
                // reads the fp32 strips
                fused_cb = !no_fused() && tc::intra_tile_ok(d.P, d.Q);
                const size_t smem_ct = tc::bmm_cb_tma_smem(d.N);
                BISSD_ALLOW(tc::bmm_cb_tma<T>, smem_ct);
                BISSD_LAUNCH("tc_bmm_cb_tma", launch_pdl(tc::bmm_cb_tma<T>, dim3(d.b * d.nc * d.G, d.Q / 128, d.Q / 128), tc::kThreads, smem_ct, s, 
                    d, mCc, mBc, fused_cb ? CB16b : nullptr, CBt16, fused_cb ? nullptr : F(w.cbs), status));
            } else
            BISSD_LAUNCH("tc_bmm_cb", tc::bmm_cb<T><<<dim3(d.b * d.nc * d.G, nlt_tc), tc::kThreads, smem_cb, s>>>(
                d, Cm, Bm, (sums_path && ws_path) ? nullptr : F(w.cb), ws_path ? nullptr : F(w.cbt), nullptr,
                ws_path ? CBt16 : nullptr, sums_path ? F(w.cbs) : nullptr, status));   // only the copies that will be read
            have_fp32_cb = !ws_path;                             // ws path: only the copies its kernels read were written
            auto ensure_fp32_cb = [&]() -> int {                 // for the kernels that read them, should a planned path fall through
                if (have_fp32_cb) return BISSD_OK;
                BISSD_LAUNCH("tc_bmm_cb", tc::bmm_cb<T><<<dim3(d.b * d.nc * d.G, nlt_tc), tc::kThreads, smem_cb, s>>>(
                    d, Cm, Bm, F(w.cb), F(w.cbt), nullptr, nullptr, nullptr, status));
                have_fp32_cb = true;
                return BISSD_OK;
            };
            bool dx_done = false;
            if (ws_path) {
                CUtensorMap mB, mCBt, mEf, mEb, mG, mR;
                const unsigned long long dB4[4] = {(unsigned long long)d.N, (unsigned long long)d.G, (unsigned long long)d.L, (unsigned long long)d.b};
                const unsigned long long sB4[3] = {(unsigned long long)a.B.stride_head * 2, (unsigned long long)a.B.stride_seq * 2, (unsigned long long)a.B.stride_batch * 2};
                const unsigned bB4[4] = {64, 1, 128, 1};
                const unsigned long long rows = (unsigned long long)d.b * d.nc * d.H * d.P;
                const char *e16 = static_cast<const char *>(E16);
                const bool maps = tc::make_map4(&mB, a.p.x_dtype, a.B.ptr, dB4, sB4, bB4) &&
                                  map_bshd(&mG, a.p.x_dtype, gv.ptr, gv.sb, gv.sl, gv.sh, d.P, d.H, d.L, d.b, 64) &&
                                  tc::make_map2(&mCBt, BISSD_BF16, CBt16, d.Q, (unsigned long long)d.b * d.nc * d.G * d.Q, 64, 128) &&
                                  tc::make_map2(&mEf, a.p.x_dtype, e16, d.N, rows, 64, d.P) &&
                                  tc::make_map2(&mEb, a.p.x_dtype, e16 + rows * d.N * 2, d.N, rows, 64, d.P);
                // the epilogue's x rows by TMA (a [128 rows x 64] tile per step)
                const bool x_rows = maps && map_bshd(&mR, a.p.x_dtype, a.x.ptr, a.x.stride_batch, a.x.stride_seq, a.x.stride_head, d.P, d.H, d.L, d.b, 128);
                if (maps && !x_rows) mR = mG;
                if (maps) {
                    auto wide = [](const void *ptr, long long sb, long long sl, long long sh) {
                        return ptr && reinterpret_cast<uintptr_t>(ptr) % 32 == 0 && sb % 16 == 0 && sl % 16 == 0 && sh % 16 == 0;
                    };
                    tc::WsArgs wa{};
                    wa.x = x; wa.z = gv; wa.D = a.D; wa.dt_out = a.dt_out; wa.cs_f = a.cs_f; wa.cs_b = a.cs_b;
                    wa.out = MutView{a.dx, (long long)d.L * d.H * d.P, (long long)d.H * d.P, (long long)d.P};
                    wa.out_x = wa.out;
                    wa.ddt_out = F(w.ddt_out); wa.nf = F(w.nf); wa.nb = F(w.nb); wa.dDpart = F(w.dDpart);
                    wa.wide_x = wide(x.ptr, x.sb, x.sl, x.sh);
                    wa.wide_z = wide(gv.ptr, gv.sb, gv.sl, gv.sh);
                    wa.wide_o = wide(a.dx, 16, 16, 16) && (d.H * d.P) % 16 == 0;
                    wa.rows_by_tma = x_rows ? 1 : 0;
                    const size_t smem_t = tc::scan_ws_smem(d.P, d.N, d.Q);
                    const int grid = std::min(sm_count(), bch * nlt_tc);
#define BISSD_DX_WS(NSL, NS)                                                                                            \
    do {                                                                                                                \
        BISSD_ALLOW((tc::ws_kernel<T, NSL, NS, 1>), smem_t);                                                            \
        BISSD_LAUNCH("tc_dx_ws", launch_pdl(tc::ws_kernel<T, NSL, NS, 1>, grid, tc::kWsThreads, smem_t, s,                      \
            d, mB, mCBt, mEf, mEb, mG, mR, wa, status));                                                                \
    } while (0)
                    if (d.N == 128 && d.Q == 256) BISSD_DX_WS(2, 4);
                    else if (d.N == 64 && d.Q == 256) BISSD_DX_WS(1, 4);
                    else if (d.N == 128 && d.Q == 128) BISSD_DX_WS(2, 2);
                    else BISSD_DX_WS(1, 2);
#undef BISSD_DX_WS
                    dx_done = true;
                    if (fused_cb && (lease.sd = side_acquire(s)) != nullptr) {      // the two group-walking kernels branch off here
                        if (cudaEventRecord(lease.sd->fork, s) == cudaSuccess && cudaStreamWaitEvent(lease.sd->st, lease.sd->fork, 0) == cudaSuccess) {
                            s_side = lease.sd->st;
                        } else {
                            cudaGetLastError();
                        }
                    }
                    dd_slots = nlt_tc * 4;
                    if (d.has_D && !d.D_hdim) {
                        dd_slots = nlt_tc * 8;                       // one scalar per epilogue warp and tile
                        dd_compact = true;
                    }
                }
            }
            if (!dx_done) {
                const int rc = ensure_fp32_cb();
                if (rc != BISSD_OK) return rc;
            }
            if (!dx_done && !no_tma() && tc::scan_tma_ok(d.P, d.N, d.Q)) {
                CUtensorMap mB, mEf, mEb, mG;
                const unsigned long long dB4[4] = {(unsigned long long)d.N, (unsigned long long)d.G, (unsigned long long)d.L, (unsigned long long)d.b};
                const unsigned long long sB4[3] = {(unsigned long long)a.B.stride_head * 2, (unsigned long long)a.B.stride_seq * 2, (unsigned long long)a.B.stride_batch * 2};
                const unsigned bB4[4] = {64, 1, 128, 1};
                const unsigned long long dG4[4] = {(unsigned long long)d.P, (unsigned long long)d.H, (unsigned long long)d.L, (unsigned long long)d.b};
                const unsigned long long sG4[3] = {(unsigned long long)gv.sh * 2, (unsigned long long)gv.sl * 2, (unsigned long long)gv.sb * 2};
                const unsigned bG4[4] = {64, 1, (unsigned)d.Q, 1};
                const unsigned long long rows = (unsigned long long)d.b * d.nc * d.H * d.P;
                const char *e16 = static_cast<const char *>(E16);
                if (tc::make_map4(&mB, a.p.x_dtype, a.B.ptr, dB4, sB4, bB4) && tc::make_map4(&mG, a.p.x_dtype, gv.ptr, dG4, sG4, bG4) &&
                    tc::make_map2(&mEf, a.p.x_dtype, e16, d.N, rows, 64, d.P) &&
                    tc::make_map2(&mEb, a.p.x_dtype, e16 + rows * d.N * 2, d.N, rows, 64, d.P)) {
                    const int rounds = tc::scan_tma_rounds(d.P, d.N, d.Q);
                    const size_t smem_t = tc::dx_tma_smem(d.P, d.N, d.Q, rounds);
                    BISSD_ALLOW(tc::dx_tma<T>, smem_t);
                    BISSD_LAUNCH("tc_dx_tma", tc::dx_tma<T><<<dim3(bch, nlt_tc), tc::kThreads, smem_t, s>>>(
                        d, mB, mEf, mEb, mG, x, gv, a.D, a.dt_out, a.cs_f, a.cs_b, F(w.cbt), a.dx, F(w.ddt_out), F(w.nf), F(w.nb),
                        F(w.dDpart), rounds, status));
                    dx_done = true;
                }
            }
            if (dx_done) {
            } else if (ntP <= 64) {
                BISSD_ALLOW((tc::dx_kernel<T, 2>), smem_dx);
                BISSD_LAUNCH("tc_dx", tc::dx_kernel<T, 2><<<dim3(bch, nlt_tc), tc::kThreads, smem_dx, s>>>(
                    dg, x, Bm, z, gv, out_x, a.D, a.dt_out, a.cs_f, a.cs_b, F(w.cb), E16, a.dx, a.dz, F(w.ddt_out), F(w.dDpart), status));
            } else {
                BISSD_ALLOW((tc::dx_kernel<T, 8>), smem_dx);
                BISSD_LAUNCH("tc_dx", tc::dx_kernel<T, 8><<<dim3(bch, nlt_tc), tc::kThreads, smem_dx, s>>>(
                    dg, x, Bm, z, gv, out_x, a.D, a.dt_out, a.cs_f, a.cs_b, F(w.cb), E16, a.dx, a.dz, F(w.ddt_out), F(w.dDpart), status));
            }
            bool dbc_done = false;
            if (dx_done) {                                           // the dx kernel has produced nf / nb
                CUtensorMap mC, mEf, mEb, mSf, mSb;
                const unsigned long long dC4[4] = {(unsigned long long)d.N, (unsigned long long)d.G, (unsigned long long)d.L, (unsigned long long)d.b};
                const unsigned long long sC4[3] = {(unsigned long long)a.C.stride_head * 2, (unsigned long long)a.C.stride_seq * 2, (unsigned long long)a.C.stride_batch * 2};
                const unsigned bC4[4] = {64, 1, 128, 1};
                const unsigned long long rows = (unsigned long long)d.b * d.nc * d.H * d.P;
                const char *e16 = static_cast<const char *>(E16);
                if (tc::make_map4(&mC, a.p.x_dtype, a.C.ptr, dC4, sC4, bC4) &&
                    tc::make_map2(&mEf, a.p.x_dtype, e16, d.N, rows, 64, d.P) &&
                    tc::make_map2(&mEb, a.p.x_dtype, e16 + rows * d.N * 2, d.N, rows, 64, d.P) &&
                    tc::make_map2(&mSf, a.p.x_dtype, a.states_f, d.N, rows, 64, d.P) &&
                    tc::make_map2(&mSb, a.p.x_dtype, a.states_b, d.N, rows, 64, d.P)) {
                    const size_t smem_p = tc::prev_tma_smem(d.P, d.N), smem_a = tc::dbc_tma_smem(d.P, std::min(d.N, 128));
                    CUtensorMap mX128, mG128;
                    if (!map_bshd(&mX128, a.p.x_dtype, a.x.ptr, a.x.stride_batch, a.x.stride_seq, a.x.stride_head, d.P, d.H, d.L, d.b, 128) ||
                        !map_bshd(&mG128, a.p.x_dtype, gv.ptr, gv.sb, gv.sl, gv.sh, d.P, d.H, d.L, d.b, 128))
                        return BISSD_ERR_ALIGN;
                    if (!no_ws() && tc::prev_grp_ok(d.P, d.N, d.Q, d.R)) {
                        const size_t smem_g = tc::prev_grp_smem(d.N, d.Q);
                        const int ks = tc::state_grp_ksplit(d.b * d.nc * d.G, d.R, sm_count());
                        BISSD_ALLOW(tc::prev_terms_grp<T>, smem_g);
                        BISSD_LAUNCH_ON(s_side, "tc_prev_terms_grp", launch_pdl(tc::prev_terms_grp<T>, dim3(d.b * d.nc * d.G * ks), tc::kPrevGrpThreads, smem_g, s_side, 
                            d, mC, mSf, mSb, mG128, ks, a.cs_f, a.cs_b, F(w.pf), F(w.pb), status));
                    } else {
                        BISSD_ALLOW(tc::prev_terms_tma<T>, smem_p);
                        BISSD_LAUNCH("tc_prev_terms_tma", tc::prev_terms_tma<T><<<dim3(bch, nlt_tc), tc::kThreads, smem_p, s>>>(
                            d, mC, mSf, mSb, gv, a.cs_f, a.cs_b, F(w.pf), F(w.pb), status));
                    }
                    BISSD_ALLOW(tc::dbc_accum_tma<T>, smem_a);
                    if (!no_ws() && tc::dbc_grp_ok(d.P, d.N, d.Q)) {
                        const size_t smem_g = tc::dbc_grp_smem(d.Q, std::min(d.N, 128));
                        BISSD_ALLOW(tc::dbc_accum_grp<T>, smem_g);
                        BISSD_LAUNCH_ON(s_side, "tc_dbc_accum_grp", launch_pdl(tc::dbc_accum_grp<T>, dim3(d.b * d.nc * d.G * w.nsplit, 1, 2), tc::kDbcGrpThreads, smem_g, s_side, 
                            d, mEf, mEb, mSf, mSb, mX128, mG128, a.dt_out, a.cs_f, a.cs_b, F(w.dB_part), F(w.dC_part), status));
                    } else
                    BISSD_LAUNCH("tc_dbc_accum_tma", tc::dbc_accum_tma<T><<<dim3(d.b * d.nc * d.G * w.nsplit, nlt_tc, 2), tc::kThreads, smem_a, s>>>(
                        d, mEf, mEb, mSf, mSb, mX128, mG128, a.dt_out, a.cs_f, a.cs_b, F(w.dB_part), F(w.dC_part), status));
                    dbc_done = true;
                    nsplit = 1;                                      // nf/nb/pf/pb now hold complete row sums
                }
            }
            if (!dbc_done) {
                BISSD_ALLOW(tc::dbc_states<T>, smem_n);
                BISSD_LAUNCH("tc_dbc_states", tc::dbc_states<T><<<dim3(d.b * d.nc * d.G * w.nsplit, nlt_tc, 2), tc::kThreads, smem_n, s>>>(
                    dg, x, Bm, Cm, z, gv, a.dt_out, a.cs_f, a.cs_b, E16, a.states_f, a.states_b, F(w.dB_part), F(w.dC_part),
                    F(w.nf), F(w.nb), F(w.pf), F(w.pb), status));
            }
        }
    }
    if (!tcp) {
        BISSD_LAUNCH("bmm_cb", simt::bmm_cb<T><<<dim3(d.b * d.nc * d.G, w.nlt, w.nlt), simt::TB, 0, s>>>(d, Cm, Bm, F(w.cb)));
        BISSD_LAUNCH("dx_kernel", simt::dx_kernel<T><<<dim3(bch, w.nlt), simt::TB, q3, s>>>(
            d, x, Bm, z, dout, out_x, a.D, a.dt_out, a.cs_f, a.cs_b, F(w.cb), F(w.E), a.dx, a.dz, F(w.ddt_out), F(w.dDpart)));
        BISSD_LAUNCH("dbc_states", simt::dbc_states<T><<<dim3(bch, w.nlt, 2), simt::TB, q3, s>>>(
            d, x, Bm, Cm, z, dout, a.dt_out, a.cs_f, a.cs_b, F(w.E), a.states_f, a.states_b, F(w.dB_part), F(w.dC_part),
            F(w.nf), F(w.nb), F(w.pf), F(w.pb)));
    }
    bool intra_tc = false;
    bool bmm_tma = false;                                        // dCB is then a 16-bit array read by TMA
    CUtensorMap mBb, mCb, mDm, mDk;
    if constexpr (TcKernels<T>::available) {
        if (tcp) {
            intra_tc = true;
            const int ntQ128 = std::min(ntQ, 128);
            const size_t smem_dcb = tc::smem_bytes(ntQ128, 3 * d.Q), smem_in = tc::smem_bytes(ntQ, 4 * d.Q + tc::kTileM * 8);
            bool dcb_done = false;
            bool fused_done = false;
            if (fused_cb) {
                // one kernel for dCB and the intra-chunk decay gradients: a CTA per (batch, chunk, group, row tile)
                CUtensorMap mG, mX128, mCB;
                const unsigned long long dBC4[4] = {(unsigned long long)d.N, (unsigned long long)d.G, (unsigned long long)d.L, (unsigned long long)d.b};
                const unsigned long long sB4[3] = {(unsigned long long)a.B.stride_head * 2, (unsigned long long)a.B.stride_seq * 2, (unsigned long long)a.B.stride_batch * 2};
                const unsigned long long sC4b[3] = {(unsigned long long)a.C.stride_head * 2, (unsigned long long)a.C.stride_seq * 2, (unsigned long long)a.C.stride_batch * 2};
                const unsigned bx4[4] = {64, 1, 128, 1};
                const unsigned long long dcb_rows = (unsigned long long)d.b * d.nc * d.G * d.Q;
                if (map_bshd(&mG, a.p.x_dtype, gv.ptr, gv.sb, gv.sl, gv.sh, d.P, d.H, d.L, d.b, 128) &&
                    map_bshd(&mX128, a.p.x_dtype, a.x.ptr, a.x.stride_batch, a.x.stride_seq, a.x.stride_head, d.P, d.H, d.L, d.b, 128) &&
                    tc::make_map2(&mCB, BISSD_BF16, ws + w.cb16, d.Q, dcb_rows, 64, 128) &&
                    tc::bmm_bwd_tma_ok(d.N, d.Q) &&
                    tc::make_map4(&mBb, a.p.x_dtype, a.B.ptr, dBC4, sB4, bx4) && tc::make_map4(&mCb, a.p.x_dtype, a.C.ptr, dBC4, sC4b, bx4) &&
                    tc::make_map2(&mDm, a.p.x_dtype, F(w.dCB), d.Q, dcb_rows, 64, d.Q) &&
                    tc::make_map2(&mDk, a.p.x_dtype, F(w.dCB), d.Q, dcb_rows, 64, 128)) {
                    const size_t smem_f = tc::intra_tile_smem(d.Q);
                    BISSD_ALLOW(tc::intra_dcb_tile<T>, smem_f);
                    BISSD_LAUNCH("tc_intra_dcb_tile", launch_pdl(tc::intra_dcb_tile<T>, dim3(d.b * d.nc * d.G, nlt_tc, nlt_tc), tc::kIntraTileThreads, smem_f, s,
                        dg, mG, mX128, mCB, a.dt_out, a.cs_f, a.cs_b, F(w.u4), (long long)d.b * d.H * d.nc * d.Q,
                        static_cast<void *>(F(w.dCB)), status));
                    u4_tiles = nlt_tc * nlt_tc;
                    fused_done = dcb_done = true;
                    bmm_tma = true;
                    use_u4 = true;
                } else {
                    return BISSD_ERR_ALIGN;                      // the bf16 tile was written for this kernel only
                }
            }
            if (!dcb_done && !no_tma() && tc::scan_tma_ok(d.P, d.N, d.Q)) {
                CUtensorMap mG, mX;
                const unsigned long long dX4[4] = {(unsigned long long)d.P, (unsigned long long)d.H, (unsigned long long)d.L, (unsigned long long)d.b};
                const unsigned long long sX4[3] = {(unsigned long long)a.x.stride_head * 2, (unsigned long long)a.x.stride_seq * 2, (unsigned long long)a.x.stride_batch * 2};
                const unsigned long long sG4[3] = {(unsigned long long)gv.sh * 2, (unsigned long long)gv.sl * 2, (unsigned long long)gv.sb * 2};
                const unsigned bx4[4] = {64, 1, 128, 1};
                if (tc::make_map4(&mX, a.p.x_dtype, a.x.ptr, dX4, sX4, bx4) && tc::make_map4(&mG, a.p.x_dtype, gv.ptr, dX4, sG4, bx4)) {
                    // the product with B / C reads dCB by TMA from a 16-bit copy when it can
                    const unsigned long long dBC4[4] = {(unsigned long long)d.N, (unsigned long long)d.G, (unsigned long long)d.L, (unsigned long long)d.b};
                    const unsigned long long sB4[3] = {(unsigned long long)a.B.stride_head * 2, (unsigned long long)a.B.stride_seq * 2, (unsigned long long)a.B.stride_batch * 2};
                    const unsigned long long sC4b[3] = {(unsigned long long)a.C.stride_head * 2, (unsigned long long)a.C.stride_seq * 2, (unsigned long long)a.C.stride_batch * 2};
                    const unsigned long long dcb_rows = (unsigned long long)d.b * d.nc * d.G * d.Q;
                    bmm_tma = !no_ws() && tc::bmm_bwd_tma_ok(d.N, d.Q) &&
                              tc::make_map4(&mBb, a.p.x_dtype, a.B.ptr, dBC4, sB4, bx4) && tc::make_map4(&mCb, a.p.x_dtype, a.C.ptr, dBC4, sC4b, bx4) &&
                              tc::make_map2(&mDm, a.p.x_dtype, F(w.dCB), d.Q, dcb_rows, 64, d.Q) &&
                              tc::make_map2(&mDk, a.p.x_dtype, F(w.dCB), d.Q, dcb_rows, 64, 128);
                    const size_t smem_t = tc::dcb_tma_smem(d.P, d.Q);
                    BISSD_ALLOW(tc::dcb_tma<T>, smem_t);
                    BISSD_LAUNCH("tc_dcb_tma", launch_pdl(tc::dcb_tma<T>, dim3(d.b * d.nc * d.G, nlt_tc, nlt_tc), tc::kThreads, smem_t, s, 
                        d, mG, mX, a.dt_out, a.cs_f, a.cs_b, bmm_tma ? nullptr : F(w.dCB), bmm_tma ? static_cast<void *>(F(w.dCB)) : nullptr, status));
                    dcb_done = true;
                }
            }
            if (!dcb_done) {
                BISSD_ALLOW(tc::dcb_kernel<T>, smem_dcb);
                BISSD_LAUNCH("tc_dcb", tc::dcb_kernel<T><<<dim3(d.b * d.nc * d.G, nlt_tc, nlt_tc), tc::kThreads, smem_dcb, s>>>(
                    dg, x, z, gv, a.dt_out, a.cs_f, a.cs_b, F(w.dCB), status));
            }
            bool intra_done = fused_done;
            const bool sums_path = !no_tma() && !no_sums() && tc::scan_tma_ok(d.P, d.N, d.Q);
            if (sums_path && !intra_done) {
                CUtensorMap mG, mX;
                if (map_bshd(&mG, a.p.x_dtype, gv.ptr, gv.sb, gv.sl, gv.sh, d.P, d.H, d.L, d.b, 128) &&
                    map_bshd(&mX, a.p.x_dtype, a.x.ptr, a.x.stride_batch, a.x.stride_seq, a.x.stride_head, d.P, d.H, d.L, d.b, d.Q)) {
                    const size_t smem_s = tc::intra_sums_smem(d.Q);
                    BISSD_ALLOW(tc::intra_sums<T>, smem_s);
                    BISSD_LAUNCH("tc_intra_sums", launch_pdl(tc::intra_sums<T>, dim3(bch, nlt_tc), tc::kThreads, smem_s, s, 
                        dg, mG, mX, a.dt_out, a.cs_f, a.cs_b, F(w.cbs), F(w.u4), (long long)d.b * d.H * d.nc * d.Q, status));
                    intra_done = true;
                    use_u4 = true;
                }
            }
            if (!intra_done && !have_fp32_cb) {                  // the prefix-sweep kernels read the fp32 matrix
                const size_t smem_cb = tc::smem_bytes(ntQ, 0);
                BISSD_LAUNCH("tc_bmm_cb", tc::bmm_cb<T><<<dim3(d.b * d.nc * d.G, nlt_tc), tc::kThreads, smem_cb, s>>>(
                    d, Cm, Bm, F(w.cb), F(w.cbt), nullptr, nullptr, nullptr, status));
                have_fp32_cb = true;
            }
            if (!intra_done && !no_tma() && tc::scan_tma_ok(d.P, d.N, d.Q)) {
                CUtensorMap mG, mX;
                if (map_bshd(&mG, a.p.x_dtype, gv.ptr, gv.sb, gv.sl, gv.sh, d.P, d.H, d.L, d.b, 128) &&
                    map_bshd(&mX, a.p.x_dtype, a.x.ptr, a.x.stride_batch, a.x.stride_seq, a.x.stride_head, d.P, d.H, d.L, d.b, d.Q)) {
                    BISSD_ALLOW((tc::intra_decay_grad<T, true>), smem_in);
                    BISSD_LAUNCH("tc_intra_decay_grad", tc::intra_decay_grad<T, true><<<dim3(bch, nlt_tc), tc::kThreads, smem_in, s>>>(
                        dg, mG, mX, x, z, gv, a.dt_out, a.cs_f, a.cs_b, F(w.cb), F(w.da_f), F(w.da_b), status));
                    intra_done = true;
                }
            }
            if (!intra_done) {
                CUtensorMap none{};
                BISSD_ALLOW((tc::intra_decay_grad<T, false>), smem_in);
                BISSD_LAUNCH("tc_intra_decay_grad", tc::intra_decay_grad<T, false><<<dim3(bch, nlt_tc), tc::kThreads, smem_in, s>>>(
                    dg, none, none, x, z, gv, a.dt_out, a.cs_f, a.cs_b, F(w.cb), F(w.da_f), F(w.da_b), status));
            }
        }
    }
    if (!intra_tc) {
        BISSD_LAUNCH("dcb_kernel", simt::dcb_kernel<T><<<dim3(d.b * d.nc * d.G, w.nlt, w.nlt), simt::TB, 0, s>>>(
            d, x, z, dout, a.dt_out, a.cs_f, a.cs_b, F(w.dCB)));
        const size_t smem = (3 * d.Q + 2 * simt::TILE * (d.Q + 1)) * sizeof(float);
        BISSD_ALLOW(simt::intra_decay_grad<T>, smem);
        BISSD_LAUNCH("intra_decay_grad", simt::intra_decay_grad<T><<<bch, simt::TB, smem, s>>>(
            d, x, z, dout, a.dt_out, a.cs_f, a.cs_b, F(w.cb), F(w.da_f), F(w.da_b)));
    }
    if (s_side != s) {                                           // the group-walking kernels rejoin before their results are read
        int rcj = note_cuda(cudaEventRecord(lease.sd->join, s_side), "cudaEventRecord");
        if (rcj == BISSD_OK) rcj = note_cuda(cudaStreamWaitEvent(s, lease.sd->join, 0), "cudaStreamWaitEvent");
        if (rcj != BISSD_OK) return rcj;
        s_side = s;
    }
    bool bmm_tc = false;
    if constexpr (TcKernels<T>::available) {
        if (tcp && bmm_tma) {
            bmm_tc = true;
            const size_t smem_b = tc::bmm_bwd_tma_smem(d.Q);
            BISSD_ALLOW(tc::bmm_bwd_tma<T>, smem_b);
            BISSD_LAUNCH("tc_bmm_bwd_tma", launch_pdl(tc::bmm_bwd_tma<T>, dim3(d.b * d.nc * d.G * 2, d.Q / 128, d.N / 64), tc::kThreads, smem_b, s, 
                d, mDm, mDk, mBb, mCb, F(w.dB_part), F(w.dC_part), part_heads, a.dB, a.dC, status));
        } else if (tcp) {
            bmm_tc = true;
            const size_t smem_n = tc::smem_bytes(ntN, 0);
            BISSD_ALLOW(tc::bmm_bwd<T>, smem_n);
            BISSD_LAUNCH("tc_bmm_bwd", tc::bmm_bwd<T><<<dim3(d.b * d.nc * d.G * 2, nlt_tc, w.nsplit), tc::kThreads, smem_n, s>>>(
                d, Bm, Cm, F(w.dCB), F(w.dB_part), F(w.dC_part), part_heads, a.dB, a.dC, status));
        }
    }
    if (!bmm_tc) {
        BISSD_LAUNCH("bmm_bwd", simt::bmm_bwd<T><<<dim3(d.b * d.nc * d.G * 2, w.nlt, ceil_div(d.N, simt::TILE)), simt::TB, 0, s>>>(
            d, Bm, Cm, F(w.dCB), F(w.dB_part), F(w.dC_part), part_heads, a.dB, a.dC));
    }
    BISSD_LAUNCH("cumsum_bwd", launch_pdl(simt::cumsum_bwd, d.b * d.nc * d.H, 256, 0, s, 
        d, a.dt.ptr, a.p.dt_dtype, a.dt.stride_batch, a.dt.stride_seq, a.dt.stride_head, a.A, a.dt_bias, a.dt_out,
        F(w.ddt_out), F(w.nf), F(w.nb), F(w.pf), F(w.pb), use_u4 ? nullptr : F(w.da_f), use_u4 ? nullptr : F(w.da_b),
        use_u4 ? F(w.u4) : nullptr, u4_tiles, F(w.dTpart), pass_nblk, nsplit, a.ddt,
        F(w.dApart), F(w.dbiaspart)));
    BISSD_LAUNCH("final_reduce", launch_pdl(simt::final_reduce<1024>, d.H, 1024, 0, s, 
        d, F(w.dApart), F(w.dbiaspart), d.has_D ? F(w.dDpart) : nullptr, dd_slots ? dd_slots : nlt, dd_compact ? 1 : 0, a.dA, d.has_bias ? a.ddt_bias : nullptr,
        d.has_D ? a.dD : nullptr));
    return BISSD_OK;
}

static int check_device() {
    static std::atomic<int> major_of[64];                        // 0 = not asked yet
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return BISSD_ERR_LAUNCH;
    int major = (dev >= 0 && dev < 64) ? major_of[dev].load(std::memory_order_relaxed) : 0;
    if (!major) {
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return BISSD_ERR_LAUNCH;
        if (dev >= 0 && dev < 64) major_of[dev].store(major, std::memory_order_relaxed);
    }
    return major == 10 ? BISSD_OK : BISSD_ERR_ARCH;
}

}  // namespace bissd

using namespace bissd;

// ---- gated RMSNorm ---------------------------------------------------------------------------------------------
static int norm_check(const bissd_norm_args *a, norm::NormDims *d, bool backward) {
    if (!a || !a->x || !a->weight || !a->rstd) return BISSD_ERR_NULL;
    if (!backward && !a->out) return BISSD_ERR_NULL;
    if (backward && (!a->dout || !a->dx || !a->dweight || (a->z && !a->dz))) return BISSD_ERR_NULL;
    if (a->rows <= 0 || a->hidden <= 0 || a->hidden % 256 != 0 || a->hidden > 4096) return BISSD_ERR_SHAPE;
    const int group = a->group_size > 0 ? a->group_size : a->hidden;
    if (group % 256 != 0 || a->hidden % group != 0) return BISSD_ERR_SHAPE;
    if (a->x_dtype < BISSD_F32 || a->x_dtype > BISSD_F16) return BISSD_ERR_DTYPE;
    if (a->w_dtype != BISSD_F32 && a->w_dtype != a->x_dtype) return BISSD_ERR_DTYPE;
    auto al = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (!al(a->x) || !al(a->z) || !al(a->weight) || !al(a->out) || !al(a->dout) || !al(a->dx) || !al(a->dz))
        return BISSD_ERR_ALIGN;
    if (a->stride_x % 8 || a->stride_z % 8 || a->stride_out % 8) return BISSD_ERR_ALIGN;
    d->rows = a->rows; d->hidden = a->hidden; d->group = group; d->ngroups = a->hidden / group;
    d->sx = a->stride_x; d->sz = a->stride_z; d->so = a->stride_out;
    d->has_z = a->z != nullptr; d->norm_before_gate = a->norm_before_gate; d->eps = a->eps;
    return BISSD_OK;
}
static int norm_grid(const norm::NormDims &d) {
    const long long want = (d.rows + norm::kWarps - 1) / norm::kWarps;
    return (int)std::min<long long>(want, (long long)sm_count() * 8);
}

template <class T, class W>
static int norm_forward_impl(const bissd_norm_args *a, const norm::NormDims &d, cudaStream_t s) {
    const int grid = norm_grid(d);
    if (d.hidden <= 2048) {
        BISSD_LAUNCH("rmsnorm_gated_fwd", norm::rmsnorm_gated_fwd<T, W, 8><<<grid, norm::kThreads, 0, s>>>(
            d, a->x, a->z, a->weight, a->out, a->rstd));
    } else {
        BISSD_LAUNCH("rmsnorm_gated_fwd", norm::rmsnorm_gated_fwd<T, W, 16><<<grid, norm::kThreads, 0, s>>>(
            d, a->x, a->z, a->weight, a->out, a->rstd));
    }
    return BISSD_OK;
}
template <class T, class W>
static int norm_backward_impl(const bissd_norm_args *a, const norm::NormDims &d, float *part, cudaStream_t s) {
    // two resident CTAs per SM and one partial weight-gradient row per CTA: a larger grid only adds rows to reduce
    const int grid = std::min(norm_grid(d), 2 * sm_count());
    const size_t smem = (size_t)norm::kWarps * d.hidden * sizeof(float);
    if (d.hidden <= 2048) {
        BISSD_ALLOW((norm::rmsnorm_gated_bwd<T, W, 8>), smem);
        BISSD_LAUNCH("rmsnorm_gated_bwd", norm::rmsnorm_gated_bwd<T, W, 8><<<grid, norm::kThreads, smem, s>>>(
            d, a->x, a->z, a->weight, a->dout, a->rstd, a->dx, a->dz, part));
    } else {
        BISSD_ALLOW((norm::rmsnorm_gated_bwd<T, W, 16>), smem);
        BISSD_LAUNCH("rmsnorm_gated_bwd", norm::rmsnorm_gated_bwd<T, W, 16><<<grid, norm::kThreads, smem, s>>>(
            d, a->x, a->z, a->weight, a->dout, a->rstd, a->dx, a->dz, part));
    }
    BISSD_LAUNCH("norm_bwd_reduce", norm::norm_bwd_reduce<W><<<(d.hidden + 255) / 256, norm::kThreads, 0, s>>>(
        part, grid, d.hidden, a->dweight));
    return BISSD_OK;
}
#define BISSD_NORM_DISPATCH(fn, ...)                                                                \
    do {                                                                                            \
        const bool wf = a->w_dtype == BISSD_F32;                                                    \
        switch (a->x_dtype) {                                                                       \
            case BISSD_F32: return fn<float, float>(__VA_ARGS__);                                   \
            case BISSD_BF16: return wf ? fn<__nv_bfloat16, float>(__VA_ARGS__) : fn<__nv_bfloat16, __nv_bfloat16>(__VA_ARGS__); \
            default: return wf ? fn<__half, float>(__VA_ARGS__) : fn<__half, __half>(__VA_ARGS__); \
        }                                                                                           \
    } while (0)


// ---- depthwise conv1d + SiLU -----------------------------------------------------------------------------------
static int conv_check(const bissd_conv_args *a, conv::ConvDims *d, bool backward) {
    if (!a || !a->x || !a->weight) return BISSD_ERR_NULL;
    if (!backward && !a->out) return BISSD_ERR_NULL;
    if (backward && (!a->dout || !a->dx || !a->dweight || (a->bias && !a->dbias))) return BISSD_ERR_NULL;
    if (a->batch <= 0 || a->seqlen <= 0 || a->channels <= 0 || a->channels % 8 != 0) return BISSD_ERR_SHAPE;
    if (a->width <= 0 || a->width > conv::kMaxK || a->width % 2 == 0) return BISSD_ERR_SHAPE;
    if (a->x_dtype < BISSD_F32 || a->x_dtype > BISSD_F16) return BISSD_ERR_DTYPE;
    if (a->w_dtype != BISSD_F32 && a->w_dtype != a->x_dtype) return BISSD_ERR_DTYPE;
    auto al = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (!al(a->x) || !al(a->out) || !al(a->dout) || !al(a->dx) || !al(a->bias)) return BISSD_ERR_ALIGN;
    if (a->x_stride_batch % 8 || a->x_stride_row % 8 || a->out_stride_batch % 8 || a->out_stride_row % 8) return BISSD_ERR_ALIGN;
    d->batch = a->batch; d->seqlen = a->seqlen; d->channels = a->channels; d->width = a->width;
    d->xsb = a->x_stride_batch; d->xsl = a->x_stride_row; d->osb = a->out_stride_batch; d->osl = a->out_stride_row;
    d->has_bias = a->bias != nullptr;
    return BISSD_OK;
}
static inline int conv_row_blocks(int seqlen) { return (seqlen + conv::kRows - 1) / conv::kRows; }
static inline size_t conv_dpre_bytes(const bissd_conv_args *a) {
    return align256((size_t)a->batch * a->seqlen * a->channels * (a->x_dtype == BISSD_F32 ? 4 : 2));
}
template <class T, class W>
static int conv_forward_impl(const bissd_conv_args *a, const conv::ConvDims &d, cudaStream_t s) {
    const dim3 grid((d.channels / 8 + 127) / 128, conv_row_blocks(d.seqlen), d.batch);
    if constexpr (sizeof(T) == 2) {
#define BISSD_CONV_FWD(K)                                                                                              \
    do {                                                                                                               \
        BISSD_LAUNCH("dwconv_win_fwd", conv::dwconv_win<T, W, 0, K><<<grid, 128, 0, s>>>(d, a->x, a->weight, a->bias,  \
                                                                                         nullptr, a->out, nullptr));   \
        return BISSD_OK;                                                                                               \
    } while (0)
        if (d.width == 7) BISSD_CONV_FWD(7);                     // rolling-window form for the odd widths
        if (d.width == 5) BISSD_CONV_FWD(5);
        if (d.width == 3) BISSD_CONV_FWD(3);
#undef BISSD_CONV_FWD
    }
    BISSD_LAUNCH("dwconv_silu_fwd", conv::dwconv_silu_fwd<T, W><<<grid, 128, 0, s>>>(d, a->x, a->weight, a->bias, a->out));
    return BISSD_OK;
}
template <class T, class W>
static int conv_backward_impl(const bissd_conv_args *a, const conv::ConvDims &d, char *ws, cudaStream_t s) {
    const dim3 grid((d.channels / 8 + 127) / 128, conv_row_blocks(d.seqlen), d.batch);
    void *dpre = ws;
    float *part = reinterpret_cast<float *>(ws + conv_dpre_bytes(a));
    // dout is required to be contiguous (checked by the caller), so dpre shares its strides
    bool win = false;
    const dim3 grid_dw(grid.x, (d.seqlen + conv::kRowsDw - 1) / conv::kRowsDw, grid.z);   // the window form's dw pass
    if constexpr (sizeof(T) == 2) {
#define BISSD_CONV_BWD(K)                                                                                              \
    do {                                                                                                               \
        win = true;                                                                                                    \
        BISSD_LAUNCH("dwconv_win_bwd_pre", conv::dwconv_win<T, W, 1, K><<<grid, 128, 0, s>>>(d, a->x, a->weight,       \
                                                                                             a->bias, a->dout, dpre, nullptr)); \
        BISSD_LAUNCH("dwconv_win_bwd_dw", conv::dwconv_win<T, W, 2, K><<<grid_dw, 128, 0, s>>>(d, a->x, nullptr, nullptr, \
                                                                                            dpre, nullptr, part));    \
        BISSD_LAUNCH("dwconv_win_bwd_dx", conv::dwconv_win<T, W, 3, K><<<grid, 128, 0, s>>>(d, dpre, a->weight,        \
                                                                                            nullptr, nullptr, a->dx, nullptr)); \
    } while (0)
        if (d.width == 7) BISSD_CONV_BWD(7);                     // rolling-window form for the odd widths
        else if (d.width == 5) BISSD_CONV_BWD(5);
        else if (d.width == 3) BISSD_CONV_BWD(3);
#undef BISSD_CONV_BWD
    }
    if (!win) {
        BISSD_LAUNCH("dwconv_silu_bwd_pre", conv::dwconv_silu_bwd_pre<T, W><<<grid, 128, 0, s>>>(
            d, a->x, a->weight, a->bias, a->dout, dpre));
        BISSD_LAUNCH("dwconv_silu_bwd_dw", conv::dwconv_silu_bwd_dw<T><<<grid, 128, 0, s>>>(d, a->x, dpre, part));
        BISSD_LAUNCH("dwconv_silu_bwd_dx", conv::dwconv_silu_bwd_dx<T, W><<<grid, 128, 0, s>>>(d, dpre, a->weight, a->dx));
    }
    const int nparts = d.batch * (win ? (int)grid_dw.y : conv_row_blocks(d.seqlen));
    const long long n = (long long)d.channels * (conv::kMaxK + 1);
    BISSD_LAUNCH("conv_bwd_reduce", conv::conv_bwd_reduce<W><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(
        part, nparts, d.channels, d.width, a->dweight, a->dbias));
    return BISSD_OK;
}

extern "C" {

int bissd_abi_version(void) { return BISSD_ABI_VERSION; }

const char *bissd_strerror(int status) {
    switch (status) {
        case BISSD_OK: return "ok";
        case BISSD_ERR_NULL: return "a required pointer is NULL";
        case BISSD_ERR_SHAPE: return "inconsistent or unsupported sizes (need nheads % ngroups == 0, 32 <= chunk_size <= 256)";
        case BISSD_ERR_DTYPE: return "unsupported dtype";
        case BISSD_ERR_ALIGN: return "pointer or stride not sufficiently aligned";
        case BISSD_ERR_WORKSPACE: return "workspace too small or misaligned";
        case BISSD_ERR_LAUNCH: return "CUDA launch or API call failed";
        case BISSD_ERR_ARCH: return "device is not compute capability 10.x (B200)";
        case BISSD_ERR_PHASE: return "invalid phase mask";
        case BISSD_ERR_TOO_LARGE: return "problem needs more scratch than the fixed array of bissd_forward_static_scratch holds";
        default: return "unknown status";
    }
}

const char *bissd_last_cuda_error(void) { return g_cuda_err; }

int bissd_workspace_bytes(const bissd_problem *p, size_t *fwd_bytes, size_t *bwd_bytes) {
    if (!p) return BISSD_ERR_NULL;
    Dims d;
    int rc = make_dims(*p, &d);
    if (rc != BISSD_OK) return rc;
    if (fwd_bytes) *fwd_bytes = fwd_layout(d).total;
    if (bwd_bytes) *bwd_bytes = bwd_layout(d, !force_simt() && tc_shape_ok(*p)).total;
    return BISSD_OK;
}

unsigned long long bissd_launch_count(void) { return g_launches.load(); }

int bissd_trace_enable(int on) {
    std::lock_guard<std::mutex> lk(g_trace_mu);
    for (auto &r : g_trace) {
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
    }
    g_trace.clear();
    g_trace_on.store(on ? 1 : 0);
    return BISSD_OK;
}

int bissd_trace_read(char *names, size_t names_cap, float *total_ms, int *launches, int cap, int *count) {
    if (!names || !total_ms || !launches || !count) return BISSD_ERR_NULL;
    std::lock_guard<std::mutex> lk(g_trace_mu);
    std::vector<const char *> keys;
    std::vector<float> ms;
    std::vector<int> cnt;
    for (auto &r : g_trace) {
        if (cudaEventSynchronize(r.e1) != cudaSuccess) return note_cuda(cudaGetLastError(), "trace sync");
        float t = 0.f;
        if (cudaEventElapsedTime(&t, r.e0, r.e1) != cudaSuccess) return note_cuda(cudaGetLastError(), "trace elapsed");
        size_t k = 0;
        for (; k < keys.size(); ++k)
            if (strcmp(keys[k], r.name) == 0) break;
        if (k == keys.size()) { keys.push_back(r.name); ms.push_back(0.f); cnt.push_back(0); }
        ms[k] += t;
        cnt[k] += 1;
    }
    size_t used = 0;
    int n = 0;
    names[0] = 0;
    for (size_t k = 0; k < keys.size() && n < cap; ++k) {
        const size_t len = strlen(keys[k]);
        if (used + len + 2 > names_cap) break;
        memcpy(names + used, keys[k], len);
        used += len;
        names[used++] = ';';
        names[used] = 0;
        total_ms[n] = ms[k];
        launches[n] = cnt[k];
        ++n;
    }
    *count = n;
    return BISSD_OK;
}

int bissd_selftest_gemm(int dtype, int a_mn_major, int b_mn_major, int n, int k, const void *A, const void *B, float *C,
                        int *status_dev, void *stream) {
    if (!A || !B || !C || !status_dev) return BISSD_ERR_NULL;
    if (dtype != BISSD_BF16 && dtype != BISSD_F16) return BISSD_ERR_DTYPE;
    if (n < 16 || n > 256 || (n % 16) || k < 8 || (k % 8)) return BISSD_ERR_SHAPE;
    int rc = check_device();
    if (rc != BISSD_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t smem = 2 * tc::kAStageBytes + 2 * 256 * 128 + 1024;
#define BISSD_SELFTEST(T, AM, BM)                                                                          \
    do {                                                                                                   \
        rc = allow_smem(tc::selftest_gemm<T, AM, BM>, smem);                                               \
        if (rc != BISSD_OK) return rc;                                                                     \
        BISSD_LAUNCH("selftest_gemm", tc::selftest_gemm<T, AM, BM><<<1, tc::kThreads, smem, s>>>(          \
                                          static_cast<const T *>(A), static_cast<const T *>(B), C, n, k, status_dev)); \
    } while (0)
#define BISSD_SELFTEST_T(T)                                        \
    do {                                                           \
        if (a_mn_major && b_mn_major) BISSD_SELFTEST(T, true, true);   \
        else if (a_mn_major) BISSD_SELFTEST(T, true, false);       \
        else if (b_mn_major) BISSD_SELFTEST(T, false, true);       \
        else BISSD_SELFTEST(T, false, false);                      \
    } while (0)
    if (dtype == BISSD_BF16) BISSD_SELFTEST_T(__nv_bfloat16);
    else BISSD_SELFTEST_T(__half);
#undef BISSD_SELFTEST_T
#undef BISSD_SELFTEST
    return BISSD_OK;
}

int bissd_rmsnorm_gated_workspace_bytes(const bissd_norm_args *a, size_t *bwd_bytes) {
    norm::NormDims d;
    if (!bwd_bytes) return BISSD_ERR_NULL;
    if (!a || a->rows <= 0 || a->hidden <= 0) return BISSD_ERR_SHAPE;
    d.rows = a->rows;
    *bwd_bytes = (size_t)norm_grid(d) * a->hidden * sizeof(float);
    return BISSD_OK;
}

int bissd_rmsnorm_gated_forward(const bissd_norm_args *a, void *stream) {
    norm::NormDims d;
    int rc = norm_check(a, &d, false);
    if (rc != BISSD_OK) return rc;
    rc = check_device();
    if (rc != BISSD_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    BISSD_NORM_DISPATCH(norm_forward_impl, a, d, s);
}

int bissd_rmsnorm_gated_backward(const bissd_norm_args *a, void *workspace, size_t workspace_bytes, void *stream) {
    norm::NormDims d;
    int rc = norm_check(a, &d, true);
    if (rc != BISSD_OK) return rc;
    if (!workspace) return BISSD_ERR_NULL;
    size_t need = 0;
    bissd_rmsnorm_gated_workspace_bytes(a, &need);
    if (workspace_bytes < need) return BISSD_ERR_WORKSPACE;
    rc = check_device();
    if (rc != BISSD_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float *part = static_cast<float *>(workspace);
    BISSD_NORM_DISPATCH(norm_backward_impl, a, d, part, s);
}

int bissd_dwconv_silu_workspace_bytes(const bissd_conv_args *a, size_t *bwd_bytes) {
    if (!a || !bwd_bytes) return BISSD_ERR_NULL;
    if (a->batch <= 0 || a->seqlen <= 0 || a->channels <= 0) return BISSD_ERR_SHAPE;
    *bwd_bytes = conv_dpre_bytes(a) +
                 (size_t)a->batch * conv_row_blocks(a->seqlen) * a->channels * (conv::kMaxK + 1) * sizeof(float);
    return BISSD_OK;
}

int bissd_dwconv_silu_forward(const bissd_conv_args *a, void *stream) {
    conv::ConvDims d;
    int rc = conv_check(a, &d, false);
    if (rc != BISSD_OK) return rc;
    rc = check_device();
    if (rc != BISSD_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    BISSD_NORM_DISPATCH(conv_forward_impl, a, d, s);
}

int bissd_dwconv_silu_backward(const bissd_conv_args *a, void *workspace, size_t workspace_bytes, void *stream) {
    conv::ConvDims d;
    int rc = conv_check(a, &d, true);
    if (rc != BISSD_OK) return rc;
    if (!workspace) return BISSD_ERR_NULL;
    size_t need = 0;
    bissd_dwconv_silu_workspace_bytes(a, &need);
    if (workspace_bytes < need) return BISSD_ERR_WORKSPACE;
    if (a->out_stride_row != a->channels || a->out_stride_batch != (int64_t)a->seqlen * a->channels)
        return BISSD_ERR_ALIGN;                                  // dout (and the dpre scratch) as contiguous rows
    rc = check_device();
    if (rc != BISSD_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    BISSD_NORM_DISPATCH(conv_backward_impl, a, d, static_cast<char *>(workspace), s);
}

const char *bissd_kernel_path(const bissd_problem *p) {
    if (!p) return "";
    return (!force_simt() && tc_shape_ok(*p)) ? "tcgen05" : "simt";
}

static int static_scratch_if_known(void **out);

int bissd_read_status(const void *workspace, void *stream, int *status_out) {
    if (!status_out) return BISSD_ERR_NULL;
    if (!workspace) {                                            // the library-owned scratch of the current device
        void *scratch = nullptr;
        int rc = static_scratch_if_known(&scratch);
        if (rc != BISSD_OK) return rc;
        workspace = scratch;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = note_cuda(cudaMemcpyAsync(status_out, workspace, sizeof(int), cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync");
    if (rc != BISSD_OK) return rc;
    return note_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize");
}

int bissd_forward(const bissd_fwd_args *a, void *workspace, size_t workspace_bytes, void *stream) {
    if (!a) return BISSD_ERR_NULL;
    Dims d;
    int rc = make_dims(a->p, &d);
    if (rc != BISSD_OK) return rc;
    if (a->phases < 1 || a->phases > BISSD_PHASE_ALL) return BISSD_ERR_PHASE;
    if (!a->x.ptr || !a->B.ptr || !a->C.ptr || !a->dt.ptr || !a->A || !a->dt_out || !a->cs_f || !a->cs_b ||
        !a->states_f || !a->states_b)
        return BISSD_ERR_NULL;
    if ((a->phases & BISSD_PHASE_FINISH) && !a->out.ptr) return BISSD_ERR_NULL;
    if (a->p.has_z && (!a->z.ptr || ((a->phases & BISSD_PHASE_FINISH) && !a->out_x.ptr))) return BISSD_ERR_NULL;
    if (a->p.has_D && !a->D) return BISSD_ERR_NULL;
    if (a->p.has_dt_bias && !a->dt_bias) return BISSD_ERR_NULL;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < fwd_layout(d).total)
        return BISSD_ERR_WORKSPACE;
    rc = check_device();
    if (rc != BISSD_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    char *ws = static_cast<char *>(workspace);
    const bool tcp = !force_simt() && tc_shape_ok(a->p) && aligned16(a->x) && aligned16(a->B) && aligned16(a->C) &&
                     aligned16(a->z) && aligned16(a->out) && aligned16(a->out_x);
    switch (a->p.x_dtype) {
        case BISSD_F32: return forward_impl<float>(*a, d, ws, s, false);
        case BISSD_BF16: return forward_impl<__nv_bfloat16>(*a, d, ws, s, tcp);
        default: return forward_impl<__half>(*a, d, ws, s, tcp);
    }
}

// ---- forward pass on library-owned scratch -------------------------------------------------------------------
// Some hosts may not allocate device memory when they reach this operator: an inference server that hands each
// plug-in a fixed set of buffers and forbids cudaMalloc after start-up, or code that runs while the allocator is
// locked.  For them the scratch of the forward pass lives in this fixed array, part of the library's device image:
// every GPU context that loads libbissd holds these 16 MiB until the process exits, whether or not it uses them.
constexpr size_t kStaticScratchBytes = BISSD_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code the name g_static_scratch is only a handle for the symbol, not a device address; the address on
// the current device comes from cudaGetSymbolAddress, asked once per device and remembered.
static std::mutex g_static_mu;
static void *g_static_addr[64] = {};

static int static_scratch_on_current_device(void **out) {
    int dev = -1;
    int rc = note_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc != BISSD_OK) return rc;
    if (dev < 0 || dev >= 64) return BISSD_ERR_LAUNCH;
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_addr[dev]) {
        void *ptr = nullptr;
        rc = note_cuda(cudaGetSymbolAddress(&ptr, g_static_scratch), "cudaGetSymbolAddress");
        if (rc != BISSD_OK) return rc;
        if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 255)) return BISSD_ERR_WORKSPACE;
        g_static_addr[dev] = ptr;
    }
    *out = g_static_addr[dev];
    return BISSD_OK;
}

// For bissd_read_status(NULL, ...): the address remembered by an earlier bissd_forward_static_scratch call on this
// device; no symbol lookup here, so a status read never triggers the set-up.
static int static_scratch_if_known(void **out) {
    int dev = -1;
    int rc = note_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc != BISSD_OK) return rc;
    if (dev < 0 || dev >= 64) return BISSD_ERR_LAUNCH;
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_addr[dev]) return BISSD_ERR_NULL;              // bissd_forward_static_scratch has not run here yet
    *out = g_static_addr[dev];
    return BISSD_OK;
}

int bissd_forward_static_scratch(const bissd_fwd_args *a, void *stream) {
    if (!a) return BISSD_ERR_NULL;
    Dims d;
    int rc = make_dims(a->p, &d);
    if (rc != BISSD_OK) return rc;
    if (a->phases != BISSD_PHASE_ALL) return BISSD_ERR_PHASE;      // a split pass needs scratch the caller keeps
    if (fwd_layout(d).total > kStaticScratchBytes) return BISSD_ERR_TOO_LARGE;
    void *scratch = nullptr;
    rc = static_scratch_on_current_device(&scratch);
    if (rc != BISSD_OK) return rc;
    // The array still holds whatever the previous call left.  Only the status word at its start is read before it
    // is written, so that is what gets cleared; every other region is fully rewritten by the kernels that use it.
    rc = note_cuda(cudaMemsetAsync(scratch, 0, kWsHeader, static_cast<cudaStream_t>(stream)), "cudaMemsetAsync");
    if (rc != BISSD_OK) return rc;
    return bissd_forward(a, scratch, kStaticScratchBytes, stream);
}

int bissd_chain_boundaries(const float *left, const float *right, const float *log_decay, int64_t rank_stride,
                           int64_t log_decay_rank_stride, int world, int rank, int64_t batch_heads, int32_t state_elems,
                           float *out_left, float *out_right, void *stream) {
    if (!left || !right || !log_decay || !out_left || !out_right) return BISSD_ERR_NULL;
    if (world < 1 || rank < 0 || rank >= world || batch_heads <= 0 || state_elems <= 0) return BISSD_ERR_SHAPE;
    int rc = check_device();
    if (rc != BISSD_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long n = (long long)batch_heads * state_elems;
    BISSD_LAUNCH("chain_boundaries", simt::chain_boundaries<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(
        left, right, log_decay, rank_stride, log_decay_rank_stride, world, rank, n, state_elems, out_left, out_right));
    return BISSD_OK;
}

int bissd_backward(const bissd_bwd_args *a, void *workspace, size_t workspace_bytes, void *stream) {
    if (!a) return BISSD_ERR_NULL;
    Dims d;
    int rc = make_dims(a->p, &d);
    if (rc != BISSD_OK) return rc;
    if (a->phases < 1 || a->phases > BISSD_PHASE_ALL) return BISSD_ERR_PHASE;
    if (!a->x.ptr || !a->B.ptr || !a->C.ptr || !a->dt.ptr || !a->dout.ptr || !a->A || !a->dt_out || !a->cs_f ||
        !a->cs_b || !a->states_f || !a->states_b)
        return BISSD_ERR_NULL;
    if (a->phases & BISSD_PHASE_FINISH) {
        if (!a->dx || !a->dB || !a->dC || !a->ddt || !a->dA) return BISSD_ERR_NULL;
        if (a->p.has_z && (!a->dz || !a->out_x.ptr)) return BISSD_ERR_NULL;
        if (a->p.has_D && !a->dD) return BISSD_ERR_NULL;
        if (a->p.has_dt_bias && !a->ddt_bias) return BISSD_ERR_NULL;
    }
    if (a->p.has_z && (!a->z.ptr || !a->dz || !a->out_x.ptr)) return BISSD_ERR_NULL;   // the gate runs in the LOCAL phase
    if (a->p.has_D && !a->D) return BISSD_ERR_NULL;
    if (a->p.has_dt_bias && !a->dt_bias) return BISSD_ERR_NULL;
    // 16-bit tensors that miss the tensor-core family's alignment rules run on the CUDA-core family, which needs the
    // larger workspace that bissd_workspace_bytes reports for the same sizes with fp32 inputs
    const bool tcp = !force_simt() && tc_shape_ok(a->p) && aligned16(a->x) && aligned16(a->B) && aligned16(a->C) &&
                     aligned16(a->z) && aligned16(a->dout) && aligned16(a->out_x);
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < bwd_layout(d, tcp).total)
        return BISSD_ERR_WORKSPACE;
    rc = check_device();
    if (rc != BISSD_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    char *ws = static_cast<char *>(workspace);
    switch (a->p.x_dtype) {
        case BISSD_F32: return backward_impl<float>(*a, d, ws, s, false);
        case BISSD_BF16: return backward_impl<__nv_bfloat16>(*a, d, ws, s, tcp);
        default: return backward_impl<__half>(*a, d, ws, s, tcp);
    }
}

}  // extern "C"
