// Shared helpers for the worldattention_b200 kernels: error reporting, dtype loads, strided views.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdlib>
#include <utility>
#include <cstdarg>
#include <cstdio>

#include "../../include/worldattention_b200.h"

namespace wa {

// ---- host-side error plumbing ------------------------------------------------------------------
char *last_error_buffer();  // thread-local, 512 bytes (defined in wa_api.cu)

inline int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

unsigned long long &launch_counter();  // kernels launched by this library (defined in wa_api.cu)

inline int check_launch(const char *what) {
    ++launch_counter();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
    return 0;
}

// A "done once" mark per CUDA device.  Function attributes (the dynamic shared-memory opt-in) and
// capability answers belong to a device, not to the process: a second GPU used by the same process
// needs its own set-up.  Devices beyond the 64 tracked ones simply repeat the set-up on every call.
struct PerDeviceOnce {
    std::atomic<unsigned long long> bits{0};
    static int current() {
        int dev = -1;
        return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
    }
    bool done() const {
        const int dev = current();
        return dev >= 0 && dev < 64 && ((bits.load(std::memory_order_acquire) >> dev) & 1ull);
    }
    void mark() {
        const int dev = current();
        if (dev >= 0 && dev < 64) bits.fetch_or(1ull << dev, std::memory_order_release);
    }
};

// Programmatic dependent launch: the kernel may be placed on the SMs while the kernel before it on the stream is
// still draining, runs its set-up (barriers, tensor memory, descriptor prefetch) and then blocks in
// `pdl_wait()` until that kernel has completed and its writes are visible.  A kernel launched this way must reach
// `pdl_wait()` in every thread block before it touches anything the stream's earlier work reads or writes.
// WA_B200_PDL=0 in the environment turns the attribute off (plain stream order), for timing comparisons.
inline int pdl_mode() {      // 0: plain stream order; 1: dependent launch (default); 2: and the routing kernel releases its dependents once a CTA's rows are done
    static const int mode = [] {
        const char *e = getenv("WA_B200_PDL");
        return (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
    }();
    return mode;
}
inline bool pdl_enabled() { return pdl_mode() != 0; }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

#define WA_REQUIRE(cond, code, ...)                    \
    do {                                               \
        if (!(cond)) return wa::fail(code, __VA_ARGS__); \
    } while (0)

inline bool valid_dtype(int dt) { return dt == WA_F32 || dt == WA_BF16; }
inline size_t dtype_size(int dt) { return dt == WA_BF16 ? 2 : 4; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- device-side view --------------------------------------------------------------------------
struct View4 {  // [B, L, H, D], D contiguous, strides in elements
    const void *ptr;
    int dtype;
    long long sb, sl, sh;
};

inline View4 make_view(const wa_tensor4 *t) {
    View4 v;
    v.ptr = t->ptr;
    v.dtype = t->dtype;
    v.sb = t->stride_b;
    v.sl = t->stride_l;
    v.sh = t->stride_h;
    return v;
}

__device__ __forceinline__ float bf16_round_f(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ float load_elem(const void *base, int dtype, long long off) {
    if (dtype == WA_BF16) return __bfloat162float(((const __nv_bfloat16 *)base)[off]);
    return ((const float *)base)[off];
}

__device__ __forceinline__ void store_elem(void *base, int dtype, long long off, float x) {
    if (dtype == WA_BF16)
        ((__nv_bfloat16 *)base)[off] = __float2bfloat16_rn(x);
    else
        ((float *)base)[off] = x;
}

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
__device__ __forceinline__ double warp_sum_d(double x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

}  // namespace wa
