// Shared by every kernel file: error reporting, element types, warp and block reductions.
//
// Every launcher is `extern "C" int kb_<name>(..., void* stream)`: 0 on success, non-zero
// after storing a message that `kb_last_error()` returns. A launcher checks every size it was
// given and refuses what its kernel cannot take; it never launches a kernel on sizes it has
// not checked.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#define KB_DT_F32 0
#define KB_DT_BF16 1

namespace kb {

int fail(const char* fmt, ...);          // stores the message, returns 1
int check_launch(const char* what);      // cudaGetLastError -> fail(...)

// Programmatic dependent launch. A kernel started through `launch_dependent` may begin while the
// kernel before it on the stream still runs: it must call `dependent_wait()` before it reads what
// that kernel wrote or writes anything at all, and it lets the kernel after it begin once all its
// blocks have called `dependent_trigger()` (or ended). What does not depend on the kernel before
// (barriers, TMEM, the first tiles of weights) goes ahead of the wait. Off unless `kb_set_pdl(1)`.
//
// Only the kernels of a step of at most DEPENDENT_ROWS rows (decoding) are chained this way. The
// kernels of a prompt are launched plainly (`launch_dependent_if(false, ...)`): that is a rule of
// this library, not a tuning choice, and it holds for every prompt kernel.
constexpr int DEPENDENT_ROWS = 64;
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline void launch_dependent_if(bool dependent, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent && pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);      // the caller checks with check_launch
}
template <typename... KArgs, typename... Args>
inline void launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    launch_dependent_if(true, kernel, grid, block, smem, stream, args...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void dependent_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dependent_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

#define KB_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) return kb::fail(__VA_ARGS__); \
    } while (0)

template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// An input that may still be a stack of split-K partial sums: element i is the sum over `splits`
// slices `stride` elements apart, added in slice order. With one slice it is the element itself.
template <typename T> struct Src {
    const T* p;
    int splits;
    size_t stride;
    // Eight slices are loaded before they are added, so that their latencies overlap; the order of
    // the additions is the slices' order all the same.
    __device__ __forceinline__ float at(size_t i) const {
        float v = Elem<T>::load(p + i);
        int s = 1;
        for (; s + 8 <= splits; s += 8) {
            float t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = Elem<T>::load(p + (size_t)(s + j) * stride + i);
#pragma unroll
            for (int j = 0; j < 8; ++j) v += t[j];
        }
        if (s < splits) {                                   // the last few, asked for together as well
            float t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = s + j < splits ? Elem<T>::load(p + (size_t)(s + j) * stride + i) : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) v += t[j];          // adding zero for an absent slice changes nothing
        }
        return v;
    }
};

// The cache tables are [pages, kv_heads, page_size, head_dim]: the keys of one kv head in one page
// lie together. A "line" is page * page_size + offset; this is the row of that line's kv head.
__device__ __forceinline__ size_t kv_row(long long line, int kvh, int hkv, int page_size) {
    const long long page = line / page_size;
    const int off = (int)(line - page * page_size);
    return (size_t)(page * hkv + kvh) * page_size + off;
}

// (a, b) turned by the angle whose (cos, sin) is cs; the roundings are spelled out so that every
// kernel that rotates gives the same bits.
__device__ __forceinline__ void rope_rotate(float& a, float& b, const float2 cs) {
    const float ra = __fmaf_rn(a, cs.x, -__fmul_rn(b, cs.y));
    const float rb = __fmaf_rn(b, cs.x, __fmul_rn(a, cs.y));
    a = ra;
    b = rb;
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

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats. Every thread gets the
// total. The order of the additions depends on the block size only.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();                       // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float t = (lane < nwarps) ? scratch[lane] : 0.f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
    return warp_max(t);
}

__device__ __forceinline__ float gelu_tanh(float x) {
    // x/2 * (1 + tanh(sqrt(2/pi) * (x + 0.044715 x^3)))
    const float c = 0.7978845608028654f;
    return 0.5f * x * (1.f + tanhf(c * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

}  // namespace kb
