/*
 * bissd.h - C ABI of libbissd: the bidirectional SSD chunk scan
 *     y = SS(x) + flip(SS(flip(x))) + D*x   (optionally gated by z),   forward and backward,
 * as hand-written CUDA for sm_100a (NVIDIA B200).
 *
 * The reference (Hprairie/Bi-Mamba2) is Python + Triton and has no native boundary; this header is the
 * boundary a host binding (Python ctypes, a C++ extension, ...) uses in its place.  Each entry point names the
 * reference function whose work it takes over.
 *
 * Conventions
 *   - plain C types only: raw device pointers, sizes, element strides; no torch types.
 *   - the caller owns every buffer (inputs, outputs, saved intermediates, workspace); unless an entry point
 *     says otherwise the library never allocates or frees device memory, never synchronises the device and
 *     never changes the current device.  All work is ordered on the stream passed in (a cudaStream_t cast
 *     to void*; NULL = the legacy default stream): whatever the caller enqueues on it afterwards sees the call's
 *     results.  bissd_backward may run two of its kernels on a stream of the library's own beside a third one; they
 *     leave the caller's stream after its earlier work and rejoin it through events before the call returns, also
 *     inside a stream capture (that stream and its two events are created by the first uncaptured call on a device;
 *     until then, and with BISSD_NO_SIDE=1 in the environment, every launch stays on the caller's stream).
 *   - every function returns BISSD_OK (0) or a negative bissd_status; no C++ exception crosses the boundary.
 *   - tensors named like the reference's: x (batch, seqlen, nheads, headdim), dt (batch, seqlen, nheads),
 *     A (nheads), B and C (batch, seqlen, ngroups, dstate), D (nheads) or (nheads, headdim),
 *     z like x, dt_bias (nheads).  nchunks = ceil(seqlen / chunk_size).
 */
#ifndef BISSD_H_
#define BISSD_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BISSD_ABI_VERSION 1

typedef enum bissd_status {
    BISSD_OK = 0,
    BISSD_ERR_NULL = -1,          /* a required pointer is NULL */
    BISSD_ERR_SHAPE = -2,         /* inconsistent or unsupported sizes */
    BISSD_ERR_DTYPE = -3,         /* unsupported dtype combination */
    BISSD_ERR_ALIGN = -4,         /* pointer or stride not aligned as required */
    BISSD_ERR_WORKSPACE = -5,     /* workspace smaller than bissd_workspace_bytes() reports */
    BISSD_ERR_LAUNCH = -6,        /* a CUDA launch or API call failed (see bissd_last_cuda_error) */
    BISSD_ERR_ARCH = -7,          /* the current device is not compute capability 10.x */
    BISSD_ERR_PHASE = -8,         /* invalid phase mask */
    BISSD_ERR_TOO_LARGE = -9      /* needs more scratch than bissd_forward_static_scratch's fixed array holds */
} bissd_status;

typedef enum bissd_dtype { BISSD_F32 = 0, BISSD_BF16 = 1, BISSD_F16 = 2 } bissd_dtype;

/* Phases, for callers that shard the sequence over several GPUs and must exchange boundary states between
 * the local part and the rest of a pass.  BISSD_PHASE_ALL runs a whole pass.  When a pass is split, the SAME
 * workspace (contents preserved) must be passed to both calls. */
enum {
    BISSD_PHASE_LOCAL = 1,   /* fwd: discretise, local chunk states, state passing -> final states.
                                bwd: gate, local state gradients, state-passing backward -> dinit_* */
    BISSD_PHASE_FINISH = 2,  /* fwd: state passing again with init_* , then the chunk scan.
                                bwd: state-passing backward again with dfinal_* , then all gradients */
    BISSD_PHASE_ALL = 3
};

/* Sizes and switches of one call.  Mirrors the keyword arguments of
 * bimamba_chunk_scan_combined (src/ssd/bi/ssd_combined.py:577) and the asserts of
 * _mamba_chunk_scan_combined_fwd (src/ssd/bi/ssd_combined.py:297-320). */
typedef struct bissd_problem {
    int32_t batch, seqlen, nheads, headdim, ngroups, dstate, chunk_size;
    int32_t x_dtype;        /* bissd_dtype of x, z, out, out_x, dout, dx, dz, B, C, dB, dC and the saved states */
    int32_t dt_dtype;       /* bissd_dtype of dt and ddt */
    int32_t has_D;          /* D given */
    int32_t D_has_hdim;     /* D is (nheads, headdim) instead of (nheads) */
    int32_t has_z;          /* z given: out = y * silu(z), out_x = y */
    int32_t has_dt_bias;
    int32_t dt_softplus;
    float dt_min, dt_max;   /* dt_limit; (0, +inf) by default */
} bissd_problem;

/* A (batch, seqlen, heads-or-groups, inner) tensor with a contiguous innermost dimension; strides in elements. */
typedef struct bissd_tensor {
    void *ptr;
    int64_t stride_batch, stride_seq, stride_head;
} bissd_tensor;

/* Arguments of the forward pass: replaces _mamba_chunk_scan_combined_fwd (src/ssd/bi/ssd_combined.py:297-331),
 * i.e. _chunk_cumsum_fwd (ssd_chunk_state.py:699), _chunk_state_fwd (:764), both _state_passing_fwd calls
 * (ssd_state_passing.py:190), _bmm_chunk_fwd (ssd_bmm.py:163) and _chunk_scan_fwd (ssd_chunk_scan.py:1638). */
typedef struct bissd_fwd_args {
    bissd_problem p;
    bissd_tensor x, B, C, z;              /* z.ptr NULL unless p.has_z */
    bissd_tensor dt;                      /* (batch, seqlen, nheads): stride_head is the stride of the head index */
    const float *A, *D, *dt_bias;         /* fp32; D / dt_bias NULL when absent */
    bissd_tensor out;                     /* like x */
    bissd_tensor out_x;                   /* like x; written only when p.has_z */
    /* saved for the backward pass, contiguous: */
    float *dt_out, *cs_f, *cs_b;          /* (batch, nheads, nchunks, chunk_size) fp32 */
    void *states_f, *states_b;            /* (batch, nchunks, nheads, headdim, dstate), x_dtype: state entering
                                             each chunk from the left (f) / from the right (b) */
    float *final_f, *final_b;             /* (batch, nheads, headdim, dstate) fp32; may be NULL */
    const float *init_f, *init_b;         /* optional (batch, nheads, headdim, dstate) fp32 incoming states:
                                             init_f precedes token 0, init_b follows the last token */
    int32_t phases;                       /* BISSD_PHASE_* mask */
} bissd_fwd_args;

/* Arguments of the backward pass: replaces _mamba_chunk_scan_combined_bwd (src/ssd/bi/ssd_combined.py:334-475):
 * _chunk_scan_bwd_dz, _chunk_scan_bwd_dstates, both _state_passing_bwd calls,
 * _chunk_scan_chunk_state_bwd_dx, _chunk_state_bwd_db, _chunk_scan_bwd_dC, _chunk_scan_bwd_dcb, both
 * _bmm_chunk_bwd calls, _chunk_scan_bwd_ddAcs_stable_fwd/_bwd, the host glue at :456-466 and _chunk_cumsum_bwd. */
typedef struct bissd_bwd_args {
    bissd_problem p;
    bissd_tensor x, B, C, z, dout;
    bissd_tensor out_x;                   /* the forward's pre-gate output; read only when p.has_z */
    bissd_tensor dt;
    const float *A, *D, *dt_bias;
    const float *dt_out, *cs_f, *cs_b;    /* as written by the forward */
    const void *states_f, *states_b;      /* as written by the forward */
    /* gradients, all contiguous in the layout of the tensor they belong to: */
    void *dx, *dz;                        /* x_dtype; dz NULL unless p.has_z */
    void *dB, *dC;                        /* x_dtype */
    void *ddt;                            /* dt_dtype, (batch, seqlen, nheads) */
    float *dA, *dD, *ddt_bias;            /* fp32: (nheads), (nheads[, headdim]), (nheads); dD / ddt_bias may be NULL */
    const float *dfinal_f, *dfinal_b;     /* optional gradients of final_f / final_b */
    float *dinit_f, *dinit_b;             /* optional outputs: gradients w.r.t. init_f / init_b */
    int32_t phases;
} bissd_bwd_args;

/* ABI version of the loaded library (== BISSD_ABI_VERSION of the header it was built from). */
int bissd_abi_version(void);

/* Human-readable text for a status code. */
const char *bissd_strerror(int status);

/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char *bissd_last_cuda_error(void);

/* Bytes of scratch each pass needs for `p` (either pointer may be NULL).  The reference allocates the same
 * kind of temporaries with torch.empty inside every wrapper (e.g. ssd_chunk_state.py:775-776).
 * For 16-bit problems the backward size is that of the tensor-core kernels, which take x, B, C, z, dout and out_x
 * with 16-byte aligned pointers and batch / sequence / head strides that are multiples of 8 elements.  Tensors that
 * miss this are still accepted - the CUDA-core kernels run them - but those need the (larger) backward size this
 * function reports for the same sizes with x_dtype = BISSD_F32; with less, bissd_backward returns
 * BISSD_ERR_WORKSPACE. */
int bissd_workspace_bytes(const bissd_problem *p, size_t *fwd_bytes, size_t *bwd_bytes);

/* Forward pass.  workspace must be 256-byte aligned. */
int bissd_forward(const bissd_fwd_args *args, void *workspace, size_t workspace_bytes, void *stream);

/* Forward pass for callers that cannot allocate device memory at the point where they run this operator - for
 * example a serving process that gives every plug-in its buffers up front and forbids cudaMalloc afterwards, or a
 * host whose allocator is locked while the model runs.  It has no counterpart in the reference (whose wrappers
 * call torch.empty freely).  Same arguments and results as bissd_forward with phases == BISSD_PHASE_ALL, but the
 * scratch is a fixed array of BISSD_STATIC_SCRATCH_BYTES inside the library's device image, so:
 *   - a problem whose bissd_workspace_bytes() forward size exceeds that limit is refused with BISSD_ERR_TOO_LARGE;
 *   - every GPU context that loads the library holds the array until the process exits;
 *   - the first call on each device looks the array's device address up (cudaGetSymbolAddress) and remembers it:
 *     make that first call with the intended device current, and before starting any stream capture.  With CUDA's
 *     lazy module loading that lookup (or the first kernel launch) is also the moment the driver brings the library's
 *     device image, this array included, onto the device - work a host that must not allocate later wants done at
 *     start-up, so issue one small call per device then;
 *   - the kernels' device status word (see bissd_read_status) sits at the start of the array: pass workspace == NULL
 *     to bissd_read_status to read it after a call;
 *   - all calls on a device share the one array (it keeps the previous call's contents; the status word at its
 *     start is cleared on entry, everything else is rewritten before it is read), so two calls whose GPU work can
 *     overlap - different streams, or threads - race on it: serialise them.
 * The function itself calls no cudaMalloc / cudaFree or any other allocating routine. */
#define BISSD_STATIC_SCRATCH_BYTES ((size_t)16 << 20)
int bissd_forward_static_scratch(const bissd_fwd_args *args, void *stream);

/* Backward pass. */
int bissd_backward(const bissd_bwd_args *args, void *workspace, size_t workspace_bytes, void *stream);

/* Boundary chaining between the two phases of a sequence-sharded pass (no reference counterpart: the reference is
 * single-GPU; this continues its chunk recurrence, src/ssd/bi/ssd_state_passing.py:60,81, across ranks).  Every rank
 * has gathered all ranks' boundary tensors into LOCAL memory (e.g. with one NCCL all-gather); then
 *     out_left  = sum over ranks r' < rank  of exp(sum of log_decay of the ranks strictly between) * left[r']
 *     out_right = sum over ranks r' > rank  of the same weight * right[r']
 * left / right: rank r' at offset r' * rank_stride (elements), each (batch*heads, state_elems) fp32 contiguous;
 * log_decay: rank r' at r' * log_decay_rank_stride, (batch*heads) fp32, the rank's sum of Delta*A over its tokens.
 * Forward pass: left = final_f -> init_f, right = final_b -> init_b.  Backward: left = dinit_b -> dfinal_b,
 * right = dinit_f -> dfinal_f. */
int bissd_chain_boundaries(const float *left, const float *right, const float *log_decay, int64_t rank_stride,
                           int64_t log_decay_rank_stride, int world, int rank, int64_t batch_heads, int32_t state_elems,
                           float *out_left, float *out_right, void *stream);

/* ---- gated RMSNorm (the layer that follows the scan in BiMamba2) -------------------------------------------------
 * Takes over rmsnorm_fn / _layer_norm_fwd / _layer_norm_bwd of src/ssd/bi/layernorm_gated.py:108-152, :271-340, used by
 * ssd.modules.BiMamba2 at src/ssd/modules.py:114,184:
 *     norm_before_gate:  out = x rstd w silu(z)        otherwise:  out = (x silu(z)) rstd w
 *     rstd[row, group] = rsqrt(mean over the group of the normalised quantity squared + eps)
 * x, z, out, dout, dx, dz: `rows` rows of `hidden` contiguous channels (row strides in elements, multiples of 8;
 * 16-byte aligned pointers); weight, dweight: `hidden` values of dtype w_dtype (fp32 or x's dtype); rstd: fp32
 * (rows, hidden / group_size).  hidden must be a multiple of 256 and at most 4096; group_size 0 (= hidden) or a
 * multiple of 256 dividing hidden.  No bias (the reference's RMSNorm registers none).  z may be NULL (no gate). */
typedef struct bissd_norm_args {
    int64_t rows;
    int32_t hidden, group_size;
    int32_t x_dtype, w_dtype;            /* bissd_dtype */
    int32_t norm_before_gate;
    float eps;
    int64_t stride_x, stride_z, stride_out;   /* x and dx; z and dz; out and dout */
    const void *x, *z, *weight;
    void *out;                           /* forward result */
    float *rstd;                         /* written by the forward, read by the backward */
    const void *dout;                    /* backward only, as are the next three */
    void *dx, *dz, *dweight;
} bissd_norm_args;

/* Scratch the backward needs (per-CTA partial rows of the weight gradient). */
int bissd_rmsnorm_gated_workspace_bytes(const bissd_norm_args *args, size_t *bwd_bytes);
int bissd_rmsnorm_gated_forward(const bissd_norm_args *args, void *stream);
int bissd_rmsnorm_gated_backward(const bissd_norm_args *args, void *workspace, size_t workspace_bytes, void *stream);

/* ---- depthwise conv1d + SiLU, channels-last (the front end of BiMamba2) -------------------------------------------
 * Takes over `self.act(self.conv1d(xBC.transpose(1, 2)).transpose(1, 2))` of src/ssd/modules.py:164-167 (nn.Conv1d with
 * groups = channels, padding = width / 2, then SiLU) without the two transposes:
 *     out[b,l,c] = silu(bias[c] + sum_k weight[c,k] x[b, l + k - width/2, c]),   zero outside 0 <= l < seqlen.
 * x, dx: (batch, seqlen, channels) with channel stride 1 and the given batch / row strides (elements, multiples of 8);
 * out, dout: the same shape, contiguous rows of `channels`; weight, dweight: (channels, width) contiguous, bias /
 * dbias: (channels) or NULL; w_dtype fp32 or x's dtype.  channels % 8 == 0, width odd and <= 8, 16-byte aligned
 * pointers.  The backward needs bissd_dwconv_silu_workspace_bytes() of scratch (dpre and the partial weight
 * gradients). */
typedef struct bissd_conv_args {
    int32_t batch, seqlen, channels, width;
    int32_t x_dtype, w_dtype;            /* bissd_dtype */
    int64_t x_stride_batch, x_stride_row;       /* x and dx */
    int64_t out_stride_batch, out_stride_row;   /* out and dout */
    const void *x, *weight, *bias;
    void *out;                           /* forward result */
    const void *dout;                    /* backward only, as are the next three */
    void *dx, *dweight, *dbias;
} bissd_conv_args;

int bissd_dwconv_silu_workspace_bytes(const bissd_conv_args *args, size_t *bwd_bytes);
int bissd_dwconv_silu_forward(const bissd_conv_args *args, void *stream);
int bissd_dwconv_silu_backward(const bissd_conv_args *args, void *workspace, size_t workspace_bytes, void *stream);

/* Name of the kernel family the library selects for `p` ("tcgen05" or "simt"); for reports and tests. */
const char *bissd_kernel_path(const bissd_problem *p);

/* Copies the device status word of `workspace` (written by the last pass that used it; NULL = the library-owned
 * scratch of the current device, after bissd_forward_static_scratch has run there) to *status_out and
 * WAITS for `stream` - the one call in this library that synchronises.  0 = no device-side wait ran out.  The
 * tensor-core kernels bound every wait on an mbarrier; when one gives up the kernel records it here, frees its
 * tensor memory and returns, and the results of that pass are invalid.  No reference counterpart. */
int bissd_read_status(const void *workspace, void *stream, int *status_out);

/* ---- self test -------------------------------------------------------------------------------------------- */

/* Runs C[128][n] = A * B^T (fp32 result) on the library's tcgen05 block-GEMM engine with one CTA, so a test can
 * compare the tensor-core plumbing with a host GEMM.  A is [128][k] (or [k][128] if a_mn_major), B is [n][k] (or
 * [k][n] if b_mn_major), 16-bit `dtype`; n a multiple of 16 up to 256, k a multiple of 8.  *status_dev (a device
 * int the caller zeroes) becomes nonzero if a bounded device-side wait ran out.  No reference counterpart. */
int bissd_selftest_gemm(int dtype, int a_mn_major, int b_mn_major, int n, int k, const void *A, const void *B, float *C,
                        int *status_dev, void *stream);

/* ---- tracing (the reference has none beyond triton.testing.do_bench in benchmark/*.py) ----------------------- */

/* Number of kernels this library has launched in this process so far. */
unsigned long long bissd_launch_count(void);

/* on != 0: from now on bracket every kernel launch with a pair of CUDA events on the launching stream (and drop
 * earlier records); on == 0: stop and drop the records. */
int bissd_trace_enable(int on);

/* Wait for the recorded events and sum them per kernel name.  `names` receives the names separated by ';',
 * total_ms[i] / launches[i] the summed device time and launch count of the i-th name, *count how many names. */
int bissd_trace_read(char *names, size_t names_cap, float *total_ms, int *launches, int cap, int *count);

#ifdef __cplusplus
}
#endif
#endif /* BISSD_H_ */
