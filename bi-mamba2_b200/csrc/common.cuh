// Shared device/host helpers for libbissd: element types, tensor views, problem dimensions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bissd.h"

namespace bissd {

// Derived sizes of one call, passed by value to every kernel.
struct Dims {
    int b, L, H, P, G, N, Q, nc, R;   // R = heads per group, nc = ceil(L / Q)
    int has_D, D_hdim, has_z, has_bias, softplus;
    float dt_min, dt_max;
};

// (batch, seq, head, inner) view with contiguous inner dimension; strides in elements.
struct View {
    const void *ptr;
    long long sb, sl, sh;
};
struct MutView {
    void *ptr;
    long long sb, sl, sh;
};

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

template <class T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

template <class T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

template <class T> __device__ __forceinline__ float ld(const void *p, long long i) {
    return to_f<T>(static_cast<const T *>(p)[i]);
}
template <class T> __device__ __forceinline__ void st(void *p, long long i, float v) {
    static_cast<T *>(p)[i] = from_f<T>(v);
}
template <class T> __device__ __forceinline__ float ldv(const View &t, int b, int l, int h, int i) {
    return ld<T>(t.ptr, b * t.sb + l * t.sl + h * t.sh + i);
}
template <class T> __device__ __forceinline__ void stv(const MutView &t, int b, int l, int h, int i, float v) {
    st<T>(t.ptr, b * t.sb + l * t.sl + h * t.sh + i, v);
}

// Load / store with a run-time dtype (used only for dt / ddt, which are tiny).
__device__ __forceinline__ float ld_any(const void *p, int dtype, long long i) {
    if (dtype == BISSD_F32) return static_cast<const float *>(p)[i];
    if (dtype == BISSD_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
    return __half2float(static_cast<const __half *>(p)[i]);
}
__device__ __forceinline__ void st_any(void *p, int dtype, long long i, float v) {
    if (dtype == BISSD_F32) static_cast<float *>(p)[i] = v;
    else if (dtype == BISSD_BF16) static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    else static_cast<__half *>(p)[i] = __float2half_rn(v);
}

// softplus with the reference's cut-over: identity above 20 (src/ssd/bi/softplus.py:8-11).
__device__ __forceinline__ float softplus_ref(float v) { return v <= 20.f ? log1pf(expf(v)) : v; }
__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }


// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may be scheduled while
// the kernel before it in the stream is still draining.  Every such kernel opens with pdl_begin(): it lets its own
// successor be scheduled early, then waits until the predecessor grid has completed and its writes are visible -
// before that point the kernel touches nothing but its parameters.  Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_begin() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace bissd
