// Shared device helpers for the sm_100a kernels of this engine.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DE_EXPORT extern "C" __attribute__((visibility("default")))

// dtype tags passed through the C interface
#define DE_F32 0
#define DE_BF16 1

template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) {
    return __bfloat162float(x);
}

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of the
// additions depends on the block's size only, never on what else runs.
__device__ __forceinline__ float block_sum(float v, float* scratch /* 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                      // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

static inline int de_check(cudaError_t e) { return e == cudaSuccess ? 0 : (int)e; }

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch: the launch of a kernel overlaps the tail of the kernel before it
// in the stream.  A kernel calls pdl_wait() before its first access to memory that another kernel
// of the step writes (or reads while this one writes); it returns once the preceding kernel has
// completed and its writes are visible.  Before that a kernel may only do index arithmetic and read
// weights and the step's arrays, which no kernel writes.  pdl_trigger() tells the scheduler that
// the next kernel may be launched; most kernels call it when their main loop is done, before they
// write their outputs (measured on B200: triggering at the start of every kernel made decode steps
// 10% slower than no overlap at all, because the waiting blocks took the place of blocks of the
// running kernel that had not started yet; triggering late made them 3% faster).  The decode
// products, whose blocks are all resident at once, trigger right after their first loads.  Every
// kernel calls pdl_wait() on all paths, so completion is transitive along the stream: once a
// kernel's wait has returned, every kernel before it has completed.  Before its wait a kernel
// knows less: only that the kernels before the last one that triggered after its own wait have
// completed (a chain of products that trigger at their start can all be resident at once).  So
// what is read before the wait must not have been written later than that.  Without the launch
// attribute both calls do nothing.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_trigger() {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// One rotated pair of features (a, b) by the angle whose cosine and sine are (c, s).  The products
// and their sum are rounded one by one (no fused multiply-add), so that every kernel that rotates
// gives the same bits and a plain float32 implementation can be matched exactly.
__device__ __forceinline__ void rope_rotate(float a, float b, float c, float s, float& ra,
                                            float& rb) {
    ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
    rb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
}

static int g_pdl = 1;          // per library; de_set_pdl switches it

// How an SM's memory is split into shared memory and L1 is a preference of each kernel, and an SM
// cannot hold blocks of two kernels that want different splits: the second kernel's blocks wait
// until the first's are gone, which takes away the overlap that programmatic dependent launch
// gives.  The kernels of a decode step therefore all ask for the same split, `g_carveout` percent
// of the memory as shared memory (-1: the driver's choice per kernel); de_set_carveout sets it
// per library.  Measured on B200, TinyLlama shape, batch 8: 0.785 ms a step at 45-55 percent
// (132 KB shared memory) against 0.815 with the driver's choices, 0.86 at 35-40, 0.96 at 75,
// 1.18 at 100 (the products' token rows no longer fit in L1).
static int g_carveout = -1;

template <typename F>
static inline void de_prefer_carveout(F kernel, int percent) {
    static const void* seen[64];
    static int value[64];
    static int count = 0;
    int at = 0;
    while (at < count && seen[at] != (const void*)kernel) ++at;
    if (at == count) {
        if (count == 64) return;
        seen[count] = (const void*)kernel;
        value[count++] = -1;
    }
    if (value[at] == percent) return;
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         percent < 0 ? (int)cudaSharedmemCarveoutDefault : percent);
    value[at] = percent;
}

template <typename... KArgs, typename... Args>
static inline int de_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, Args... args) {
    de_prefer_carveout(kernel, g_carveout);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 1 : 0;
    return de_check(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

// ---------------------------------------------------------------------------------------------
// A timeline for measurements, compiled on request only (-DDE_TRACE): thread 0 of a block appends
// (tag, block, SM, event, nanoseconds of the global timer) to a buffer of the library, which
// de_trace_dump copies to the host and empties.  Events: 0 block entered, 1 its wait for the
// kernel before it returned, 2 block done; kernels may add their own.  Without DE_TRACE the macro
// is empty and nothing of this exists.
// ---------------------------------------------------------------------------------------------
#ifdef DE_TRACE
constexpr unsigned DE_TRACE_CAP = 1u << 16;
__device__ unsigned long long de_trace_buf[DE_TRACE_CAP * 2];
__device__ unsigned de_trace_count;
__device__ __forceinline__ void de_trace_event(unsigned tag, unsigned event) {
    if (threadIdx.x != 0) return;
    unsigned long long t;
    unsigned sm;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    asm volatile("mov.u32 %0, %%smid;\n" : "=r"(sm));
    const unsigned at = atomicAdd(&de_trace_count, 1u);
    if (at >= DE_TRACE_CAP) return;
    de_trace_buf[2 * at] = ((unsigned long long)tag << 48) | ((unsigned long long)event << 40) |
                           ((unsigned long long)sm << 24) | (unsigned long long)(blockIdx.x & 0xffffff);
    de_trace_buf[2 * at + 1] = t;
}
#define DE_TRACE_EVENT(tag, event) de_trace_event(tag, event)
#define DE_DEFINE_TRACE_DUMP                                                                    \
    DE_EXPORT int de_trace_dump(unsigned long long* host_out, int max_events) {                 \
        unsigned count = 0;                                                                     \
        cudaError_t e = cudaMemcpyFromSymbol(&count, de_trace_count, sizeof(count));            \
        if (e != cudaSuccess) return -(int)e;                                                   \
        if (count > DE_TRACE_CAP) count = DE_TRACE_CAP;                                         \
        if ((int)count > max_events) count = (unsigned)max_events;                              \
        e = cudaMemcpyFromSymbol(host_out, de_trace_buf, (size_t)count * 16);                   \
        if (e != cudaSuccess) return -(int)e;                                                   \
        const unsigned zero = 0;                                                                \
        cudaMemcpyToSymbol(de_trace_count, &zero, sizeof(zero));                                \
        return (int)count;                                                                      \
    }
#else
#define DE_TRACE_EVENT(tag, event) do { } while (0)
#define DE_DEFINE_TRACE_DUMP
#endif

#define DE_DEFINE_PDL_SWITCH                                               \
    DE_DEFINE_TRACE_DUMP                                                   \
    DE_EXPORT int de_set_pdl(int on) { g_pdl = on ? 1 : 0; return 0; }     \
    DE_EXPORT int de_set_carveout(int percent) {                           \
        g_carveout = percent < 0 ? -1 : (percent > 100 ? 100 : percent);   \
        return 0;                                                          \
    }
