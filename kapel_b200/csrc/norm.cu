// RMS norms with an offset on the weight, alone and fused with the residual sum.
//
// y = x / sqrt(mean(x^2) + eps) * (offset + w), sums and products in 32-bit
// (Kapel: kernels/src/lib.rs norm_16 :2467, norm_block_any :1522; crates/kapel-ops/src/norm.rs:123-135).
// One block a row, any width. Each thread walks the same components in every pass, so a pass may
// read what the pass before wrote without a barrier beyond the reductions' own. The order of the
// additions depends on the width and the block size only, never on the number of rows.
#include <algorithm>
#include "common.cuh"
#include "timeline.cuh"

namespace kb {

KB_TIMELINE_ARRAY(norm)        // slots: kind 2 add-and-norm over split sums (slices, whether a next norm follows)


template <typename TX, typename TW, typename TY>
__global__ void rmsnorm_kernel(TY* __restrict__ y, const TX* __restrict__ x, const TW* __restrict__ w, int width,
                               float eps, float offset) {
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = Elem<TX>::load(x + base + i);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = Elem<TX>::load(x + base + i);
        Elem<TY>::store(y + base + i, v * inv * (offset + Elem<TW>::load(w + i)));
    }
}

// residual += norm_post(branch); then, if w_next, h = norm_next(residual).
// With w_post null the branch is added as it is (a block without a norm after its branches).
template <typename TB, typename TW, typename TH>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const Src<TB> branch,
                                   const TW* __restrict__ w_post, float eps_post, float off_post,
                                   const TW* __restrict__ w_next, float eps_next, float off_next,
                                   TH* __restrict__ h, int width) {
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * width;
    float inv = 1.f;
    if (w_post != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = branch.at(base + i);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        inv = 1.f / sqrtf(ss / (float)width + eps_post);
    }
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float b = branch.at(base + i);
        if (w_post != nullptr) b = b * inv * (off_post + Elem<TW>::load(w_post + i));
        const float r = residual[base + i] + b;
        residual[base + i] = r;
        ss2 += r * r;
    }
    if (w_next == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.f / sqrtf(ss2 / (float)width + eps_next);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float r = residual[base + i];       // written by this thread above
        Elem<TH>::store(h + base + i, r * inv2 * (off_next + Elem<TW>::load(w_next + i)));
    }
}

// The same with each thread's components kept in registers between the passes (at most EPT a
// thread): the branch, possibly many split-K slices, is read once, and the residual once.
template <typename TB, typename TW, typename TH, int EPT>
__global__ void add_rmsnorm_reg_kernel(float* __restrict__ residual, const Src<TB> branch,
                                       const TW* __restrict__ w_post, float eps_post, float off_post,
                                       const TW* __restrict__ w_next, float eps_next, float off_next,
                                       TH* __restrict__ h, int width) {
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * width;
    float b[EPT], r[EPT];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
        const int i = threadIdx.x + e * blockDim.x;
        b[e] = 0.f;
        r[e] = 0.f;
        if (i < width) {
            b[e] = branch.at(base + i);
            r[e] = residual[base + i];
            ss += b[e] * b[e];
        }
    }
    float inv = 1.f;
    if (w_post != nullptr) {
        ss = block_sum(ss, scratch);
        inv = 1.f / sqrtf(ss / (float)width + eps_post);
    }
    float ss2 = 0.f;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
        const int i = threadIdx.x + e * blockDim.x;
        if (i < width) {
            const float add = w_post != nullptr ? b[e] * inv * (off_post + Elem<TW>::load(w_post + i)) : b[e];
            r[e] += add;
            residual[base + i] = r[e];
            ss2 += r[e] * r[e];
        }
    }
    if (w_next == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.f / sqrtf(ss2 / (float)width + eps_next);
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
        const int i = threadIdx.x + e * blockDim.x;
        if (i < width) Elem<TH>::store(h + base + i, r[e] * inv2 * (off_next + Elem<TW>::load(w_next + i)));
    }
}

// bfloat16 branch, weights and output with a width that is a multiple of eight: a thread keeps up
// to CPT chunks of eight components in registers and moves them with 16-byte loads and stores.
template <int CPT>
__global__ void add_rmsnorm_bf16x8_kernel(float* __restrict__ residual, const __nv_bfloat16* __restrict__ branch,
                                          const __nv_bfloat16* __restrict__ w_post, float eps_post, float off_post,
                                          const __nv_bfloat16* __restrict__ w_next, float eps_next, float off_next,
                                          __nv_bfloat16* __restrict__ h, int width) {
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * width;
    const int chunks = width >> 3;
    dependent_wait();
    dependent_trigger();
    float b[CPT][8], r[CPT][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        if (ci < chunks) {
            const uint4 ub = *reinterpret_cast<const uint4*>(branch + base + ci * 8);
            const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&ub);
            const float4 r0 = *reinterpret_cast<const float4*>(residual + base + ci * 8);
            const float4 r1 = *reinterpret_cast<const float4*>(residual + base + ci * 8 + 4);
            r[c][0] = r0.x; r[c][1] = r0.y; r[c][2] = r0.z; r[c][3] = r0.w;
            r[c][4] = r1.x; r[c][5] = r1.y; r[c][6] = r1.z; r[c][7] = r1.w;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 v = __bfloat1622float2(pb[j]);
                b[c][2 * j] = v.x;
                b[c][2 * j + 1] = v.y;
                ss += v.x * v.x + v.y * v.y;
            }
        }
    }
    float inv = 1.f;
    if (w_post != nullptr) {
        ss = block_sum(ss, scratch);
        inv = 1.f / sqrtf(ss / (float)width + eps_post);
    }
    float ss2 = 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        if (ci < chunks) {
            if (w_post != nullptr) {
                const uint4 uw = *reinterpret_cast<const uint4*>(w_post + ci * 8);
                const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&uw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 w = __bfloat1622float2(pw[j]);
                    r[c][2 * j] += b[c][2 * j] * inv * (off_post + w.x);
                    r[c][2 * j + 1] += b[c][2 * j + 1] * inv * (off_post + w.y);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) r[c][j] += b[c][j];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss2 += r[c][j] * r[c][j];
            *reinterpret_cast<float4*>(residual + base + ci * 8) = make_float4(r[c][0], r[c][1], r[c][2], r[c][3]);
            *reinterpret_cast<float4*>(residual + base + ci * 8 + 4) = make_float4(r[c][4], r[c][5], r[c][6], r[c][7]);
        }
    }
    if (w_next == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.f / sqrtf(ss2 / (float)width + eps_next);
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        if (ci < chunks) {
            const uint4 uw = *reinterpret_cast<const uint4*>(w_next + ci * 8);
            const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&uw);
            uint4 uo;
            __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&uo);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 w = __bfloat1622float2(pw[j]);
                po[j] = __floats2bfloat162_rn(r[c][2 * j] * inv2 * (off_next + w.x), r[c][2 * j + 1] * inv2 * (off_next + w.y));
            }
            *reinterpret_cast<uint4*>(h + base + ci * 8) = uo;
        }
    }
}

// Float32 partial sums of a product split over K (few rows: a decode step), bfloat16 weights and
// output, a width that is a multiple of four: a thread owns up to CPT groups of four components,
// reads each slice's four with one 16-byte load, eight slices in flight, and adds them in slice
// order. The rest is the register-resident kernel's.
template <int CPT>
__global__ void add_rmsnorm_splits_kernel(float* __restrict__ residual, const float* __restrict__ parts, int splits, size_t stride,
                                          const __nv_bfloat16* __restrict__ w_post, float eps_post, float off_post,
                                          const __nv_bfloat16* __restrict__ w_next, float eps_next, float off_next,
                                          __nv_bfloat16* __restrict__ h, int width KB_TL_PARAM) {
    __shared__ float scratch[32];
    KB_TL_ENTER(norm, blockIdx.x == 0, 2, splits, w_next != nullptr);
    const size_t base = (size_t)blockIdx.x * width;
    const int chunks = width >> 2;
    // The norms' weights are constants: they are read ahead of the wait on the kernel before, so that
    // after it there is one trip to memory (the slices and the residual) and no second or third.
    uint2 wp[CPT], wn[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        wp[c] = wn[c] = make_uint2(0u, 0u);
        if (ci < chunks) {
            if (w_post != nullptr) wp[c] = *reinterpret_cast<const uint2*>(w_post + ci * 4);
            if (w_next != nullptr) wn[c] = *reinterpret_cast<const uint2*>(w_next + ci * 4);
        }
    }
    dependent_wait();
    KB_TL_MARK(norm, 2, threadIdx.x == 0 && blockIdx.x == 0);
    dependent_trigger();                                    // a few blocks with little to read: the next kernel may set up
    float4 b[CPT], r[CPT];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        b[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        r[c] = b[c];
        if (ci < chunks) {
            const float* src = parts + base + ci * 4;
            r[c] = *reinterpret_cast<const float4*>(residual + base + ci * 4);    // in flight beside the slices
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            int s = 0;
            for (; s + 8 <= splits; s += 8) {
                float4 t[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) t[j] = *reinterpret_cast<const float4*>(src + (size_t)(s + j) * stride);
#pragma unroll
                for (int j = 0; j < 8; ++j) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
            }
            if (s < splits) {                               // the last few together as well; an absent slice adds zero
                float4 t[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    t[j] = s + j < splits ? *reinterpret_cast<const float4*>(src + (size_t)(s + j) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < 8; ++j) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
            }
            b[c] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
    float inv = 1.f;
    KB_TL_MARK(norm, 3, threadIdx.x == 0 && blockIdx.x == 0);          // the slices and the residual are here
    if (w_post != nullptr) {
        ss = block_sum(ss, scratch);
        inv = 1.f / sqrtf(ss / (float)width + eps_post);
    }
    float ss2 = 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        if (ci < chunks) {
            if (w_post != nullptr) {
                const uint2 uw = wp[c];
                const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw.x));
                const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw.y));
                r[c].x += b[c].x * inv * (off_post + w0.x);
                r[c].y += b[c].y * inv * (off_post + w0.y);
                r[c].z += b[c].z * inv * (off_post + w1.x);
                r[c].w += b[c].w * inv * (off_post + w1.y);
            } else {
                r[c].x += b[c].x; r[c].y += b[c].y; r[c].z += b[c].z; r[c].w += b[c].w;
            }
            ss2 += r[c].x * r[c].x + r[c].y * r[c].y + r[c].z * r[c].z + r[c].w * r[c].w;
            *reinterpret_cast<float4*>(residual + base + ci * 4) = r[c];
        }
    }
    if (w_next == nullptr) {
        KB_TL_LEAVE(norm, blockIdx.x == 0, 0);
        return;
    }
    ss2 = block_sum(ss2, scratch);
    KB_TL_MARK(norm, 4, threadIdx.x == 0 && blockIdx.x == 0);          // both sums are known
    const float inv2 = 1.f / sqrtf(ss2 / (float)width + eps_next);
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        if (ci < chunks) {
            const uint2 uw = wn[c];
            const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw.x));
            const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw.y));
            uint2 uo;
            __nv_bfloat162 o0 = __floats2bfloat162_rn(r[c].x * inv2 * (off_next + w0.x), r[c].y * inv2 * (off_next + w0.y));
            __nv_bfloat162 o1 = __floats2bfloat162_rn(r[c].z * inv2 * (off_next + w1.x), r[c].w * inv2 * (off_next + w1.y));
            uo.x = *reinterpret_cast<uint32_t*>(&o0);
            uo.y = *reinterpret_cast<uint32_t*>(&o1);
            *reinterpret_cast<uint2*>(h + base + ci * 4) = uo;
        }
    }
    KB_TL_LEAVE(norm, blockIdx.x == 0, 0);
}

// The same with the slices brought into shared memory by bulk copies (one a slice's row, all asked
// for by one thread right after the wait) instead of loads by every thread. What the kernel before
// has just written comes much sooner that way: loads by the threads of a block that was already
// resident while that kernel ran took 2 to 3 us for sixteen slices however they were batched, the
// copy engine brings them in 1.2 us (the whole kernel: 5.5 to 2.9 us over 16 slices; a decode step
// at Gemma 2 2B sizes and batch 8: 2.38 to 2.26 ms).
__device__ int g_norm_error = 0;
__device__ __forceinline__ uint32_t nb_saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool nb_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = nb_saddr(bar);
    const long long start = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if (clock64() - start > 2000000000ll) return false;
    }
}

template <int CPT>
__global__ void add_rmsnorm_splits_bulk_kernel(float* __restrict__ residual, const float* __restrict__ parts, int splits, size_t stride,
                                               const __nv_bfloat16* __restrict__ w_post, float eps_post, float off_post,
                                               const __nv_bfloat16* __restrict__ w_next, float eps_next, float off_next,
                                               __nv_bfloat16* __restrict__ h, int width, int room KB_TL_PARAM) {
    extern __shared__ __align__(128) unsigned char nb_smem[];
    __shared__ float scratch[32];
    __shared__ __align__(8) uint64_t landed;
    float* rows = reinterpret_cast<float*>(nb_smem);        // [room][width]
    KB_TL_ENTER(norm, blockIdx.x == 0, 2, splits, w_next != nullptr);
    const size_t base = (size_t)blockIdx.x * width;
    const int chunks = width >> 2;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(nb_saddr(&landed)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    uint2 wp[CPT], wn[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        wp[c] = wn[c] = make_uint2(0u, 0u);
        if (ci < chunks) {
            if (w_post != nullptr) wp[c] = *reinterpret_cast<const uint2*>(w_post + ci * 4);
            if (w_next != nullptr) wn[c] = *reinterpret_cast<const uint2*>(w_next + ci * 4);
        }
    }
    __syncthreads();
    dependent_wait();
    KB_TL_MARK(norm, 2, threadIdx.x == 0 && blockIdx.x == 0);
    dependent_trigger();
    const uint32_t row_bytes = (uint32_t)width * 4u;
    float4 b[CPT], r[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        b[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        r[c] = b[c];
        if (ci < chunks) r[c] = *reinterpret_cast<const float4*>(residual + base + ci * 4);
    }
    // `room` slices fit the shared memory this launch has: all of them in one round as a rule, else
    // round after round into the same rows (every thread has added a round up before the next lands on it).
    bool ok = true;
    for (int s0 = 0, round = 0; s0 < splits; s0 += room, ++round) {
        const int n = min(room, splits - s0);
        if (round > 0) __syncthreads();
        if (threadIdx.x == 0) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(nb_saddr(&landed)), "r"(row_bytes * (uint32_t)n) : "memory");
            for (int s = 0; s < n; ++s)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(nb_saddr(rows + (size_t)s * width)), "l"(parts + (size_t)(s0 + s) * stride + base), "r"(row_bytes), "r"(nb_saddr(&landed)) : "memory");
        }
        ok = nb_wait(&landed, (uint32_t)round & 1u) && ok;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int ci = threadIdx.x + c * blockDim.x;
            if (ci < chunks) {
                for (int s = 0; s < n; ++s) {               // in slice order
                    const float4 t = *reinterpret_cast<const float4*>(rows + (size_t)s * width + ci * 4);
                    b[c].x += t.x; b[c].y += t.y; b[c].z += t.z; b[c].w += t.w;
                }
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) ss += b[c].x * b[c].x + b[c].y * b[c].y + b[c].z * b[c].z + b[c].w * b[c].w;
    KB_TL_MARK(norm, 3, threadIdx.x == 0 && blockIdx.x == 0);
    float inv = 1.f;
    if (w_post != nullptr) {
        ss = block_sum(ss, scratch);
        inv = 1.f / sqrtf(ss / (float)width + eps_post);
    }
    float ss2 = 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        if (ci < chunks) {
            if (w_post != nullptr) {
                const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wp[c].x));
                const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wp[c].y));
                r[c].x += b[c].x * inv * (off_post + w0.x);
                r[c].y += b[c].y * inv * (off_post + w0.y);
                r[c].z += b[c].z * inv * (off_post + w1.x);
                r[c].w += b[c].w * inv * (off_post + w1.y);
            } else {
                r[c].x += b[c].x; r[c].y += b[c].y; r[c].z += b[c].z; r[c].w += b[c].w;
            }
            ss2 += r[c].x * r[c].x + r[c].y * r[c].y + r[c].z * r[c].z + r[c].w * r[c].w;
            *reinterpret_cast<float4*>(residual + base + ci * 4) = r[c];
        }
    }
    if (!ok && threadIdx.x == 0) atomicExch(&g_norm_error, 1);
    if (w_next == nullptr) {
        KB_TL_LEAVE(norm, blockIdx.x == 0, 0);
        return;
    }
    ss2 = block_sum(ss2, scratch);
    KB_TL_MARK(norm, 4, threadIdx.x == 0 && blockIdx.x == 0);
    const float inv2 = 1.f / sqrtf(ss2 / (float)width + eps_next);
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ci = threadIdx.x + c * blockDim.x;
        if (ci < chunks) {
            const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wn[c].x));
            const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wn[c].y));
            uint2 uo;
            __nv_bfloat162 o0 = __floats2bfloat162_rn(r[c].x * inv2 * (off_next + w0.x), r[c].y * inv2 * (off_next + w0.y));
            __nv_bfloat162 o1 = __floats2bfloat162_rn(r[c].z * inv2 * (off_next + w1.x), r[c].w * inv2 * (off_next + w1.y));
            uo.x = *reinterpret_cast<uint32_t*>(&o0);
            uo.y = *reinterpret_cast<uint32_t*>(&o1);
            *reinterpret_cast<uint2*>(h + base + ci * 4) = uo;
        }
    }
    KB_TL_LEAVE(norm, blockIdx.x == 0, 0);
}

static int threads_for(int width) { return width >= 2048 ? 512 : (width >= 512 ? 256 : 128); }

}  // namespace kb

using namespace kb;
typedef __nv_bfloat16 bf16;

KB_TIMELINE_GETTER(norm)

// 1 if a wait inside a norm kernel ever ran out (and clears the flag); synchronises the device.
extern "C" int kb_norm_error() {
    int flag = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&flag, g_norm_error, sizeof(int)) != cudaSuccess) return -1;
    if (flag) cudaMemcpyToSymbol(g_norm_error, &zero, sizeof(int));
    return flag;
}

// x: f32 or bf16; w: f32 or bf16; y: f32 or bf16.
extern "C" int kb_rmsnorm(void* y, int y_dt, const void* x, int x_dt, const void* w, int w_dt, int rows, int width,
                          float eps, float offset, void* stream) {
    KB_REQUIRE(rows >= 0 && width > 0, "rmsnorm: rows %d, width %d", rows, width);
    KB_REQUIRE(eps >= 0.f, "rmsnorm: eps %g is negative", eps);
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int t = threads_for(width);
#define KB_NORM(TX, TW, TY) \
    rmsnorm_kernel<TX, TW, TY><<<rows, t, 0, s>>>((TY*)y, (const TX*)x, (const TW*)w, width, eps, offset)
    const int code = x_dt * 4 + w_dt * 2 + y_dt;
    switch (code) {
        case 0: KB_NORM(float, float, float); break;
        case 1: KB_NORM(float, float, bf16); break;
        case 2: KB_NORM(float, bf16, float); break;
        case 3: KB_NORM(float, bf16, bf16); break;
        case 4: KB_NORM(bf16, float, float); break;
        case 5: KB_NORM(bf16, float, bf16); break;
        case 6: KB_NORM(bf16, bf16, float); break;
        case 7: KB_NORM(bf16, bf16, bf16); break;
        default: return fail("rmsnorm: dtype codes x %d, w %d, y %d are not known", x_dt, w_dt, y_dt);
    }
#undef KB_NORM
    return check_launch("rmsnorm");
}

// residual: f32 in and out. branch: `branch_dt`, as `splits` slices `split_stride` elements apart
// that are added up on the way in (1 slice: the branch itself). h: `h_dt`. Both weights: `w_dt`.
extern "C" int kb_add_rmsnorm(float* residual, const void* branch, int branch_dt, int splits, long long split_stride,
                              const void* w_post, float eps_post, float off_post, const void* w_next, float eps_next,
                              float off_next, void* h, int h_dt, int w_dt, int rows, int width, void* stream) {
    KB_REQUIRE(rows >= 0 && width > 0, "add_rmsnorm: rows %d, width %d", rows, width);
    KB_REQUIRE(w_next == nullptr || h != nullptr, "add_rmsnorm: a following norm needs an output");
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= (long long)rows * width), "add_rmsnorm: %d slices %lld apart", splits, split_stride);
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int t = threads_for(width);
#define KB_ADDNORM(TB, TW, TH)                                                                                   \
    do {                                                                                                         \
        const Src<TB> src{(const TB*)branch, splits, (size_t)split_stride};                                      \
        if (width <= 8 * t && rows <= 256)              /* few rows: latency counts, not occupancy */                \
            add_rmsnorm_reg_kernel<TB, TW, TH, 8><<<rows, t, 0, s>>>(residual, src, (const TW*)w_post, eps_post, off_post, \
                                                                     (const TW*)w_next, eps_next, off_next, (TH*)h, width); \
        else                                                                                                     \
            add_rmsnorm_kernel<TB, TW, TH><<<rows, t, 0, s>>>(residual, src, (const TW*)w_post, eps_post, off_post, \
                                                              (const TW*)w_next, eps_next, off_next, (TH*)h, width); \
    } while (0)
    const int code = branch_dt * 4 + w_dt * 2 + h_dt;
    const bool aligned = (((uintptr_t)residual | (uintptr_t)branch | (uintptr_t)w_post | (uintptr_t)w_next | (uintptr_t)h) & 15) == 0;
    if (code == 7 && splits == 1 && width % 8 == 0 && width <= 4 * 8 * 1024 && aligned) {
        const int chunks = width / 8;
        const int cpt = chunks <= 1024 ? 1 : (chunks <= 2048 ? 2 : 4);
        const int tv = min(1024, ((chunks + cpt - 1) / cpt + 31) / 32 * 32);
        const bf16 *b = (const bf16*)branch, *wp = (const bf16*)w_post, *wn = (const bf16*)w_next;
        bf16* out = (bf16*)h;
        if (cpt == 1) launch_dependent_if(rows <= DEPENDENT_ROWS, add_rmsnorm_bf16x8_kernel<1>, dim3(rows), dim3(tv), 0, s, residual, b, wp, eps_post, off_post, wn, eps_next, off_next, out, width);
        else if (cpt == 2) launch_dependent_if(rows <= DEPENDENT_ROWS, add_rmsnorm_bf16x8_kernel<2>, dim3(rows), dim3(tv), 0, s, residual, b, wp, eps_post, off_post, wn, eps_next, off_next, out, width);
        else launch_dependent_if(rows <= DEPENDENT_ROWS, add_rmsnorm_bf16x8_kernel<4>, dim3(rows), dim3(tv), 0, s, residual, b, wp, eps_post, off_post, wn, eps_next, off_next, out, width);
        return check_launch("add_rmsnorm");
    }
    // float32 partial sums of a product split over K (a decode step, or a prompt portion of a few hundred rows): a block a row
    if (branch_dt == KB_DT_F32 && w_dt == KB_DT_BF16 && h_dt == KB_DT_BF16 && rows <= 65535 && width % 4 == 0 && width <= 4 * 4 * 1024 &&
        (split_stride % 4) == 0 && (((uintptr_t)residual | (uintptr_t)branch | (uintptr_t)h) & 15) == 0 &&
        (((uintptr_t)w_post | (uintptr_t)w_next) & 7) == 0) {
        const int chunks = width / 4;
        const int cpt = chunks <= 1024 ? 1 : (chunks <= 2048 ? 2 : 4);
        const int tv = min(1024, ((chunks + cpt - 1) / cpt + 31) / 32 * 32);
        const float* b = (const float*)branch;
        const bf16 *wp = (const bf16*)w_post, *wn = (const bf16*)w_next;
        const size_t stride = (size_t)split_stride;
        bf16* out = (bf16*)h;
        // A decode step's rows: the slices come into shared memory by bulk copies (see the kernel). Up to 192 KB of
        // it, so sixteen slices of 2,304 or eleven of 4,608 values land in one round.
        const int room = (int)std::min<size_t>((size_t)splits, (size_t)(192 * 1024) / ((size_t)width * 4));
        if (rows <= DEPENDENT_ROWS && splits > 1 && room >= 1) {
            static bool attr_set = false;
            if (!attr_set) {
                const cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_splits_bulk_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024);
                const cudaError_t e2 = cudaFuncSetAttribute(add_rmsnorm_splits_bulk_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024);
                const cudaError_t e4 = cudaFuncSetAttribute(add_rmsnorm_splits_bulk_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024);
                if (e != cudaSuccess || e2 != cudaSuccess || e4 != cudaSuccess) return fail("add_rmsnorm: cannot have 192 KB of shared memory");
                attr_set = true;
            }
            const size_t bytes = (size_t)room * width * 4;
            if (cpt == 1) launch_dependent_if(true, add_rmsnorm_splits_bulk_kernel<1>, dim3(rows), dim3(tv), bytes, s, residual, b, splits, stride, wp, eps_post, off_post, wn, eps_next, off_next, out, width, room KB_TL_SLOT(norm, 2, splits, wn != nullptr));
            else if (cpt == 2) launch_dependent_if(true, add_rmsnorm_splits_bulk_kernel<2>, dim3(rows), dim3(tv), bytes, s, residual, b, splits, stride, wp, eps_post, off_post, wn, eps_next, off_next, out, width, room KB_TL_SLOT(norm, 2, splits, wn != nullptr));
            else launch_dependent_if(true, add_rmsnorm_splits_bulk_kernel<4>, dim3(rows), dim3(tv), bytes, s, residual, b, splits, stride, wp, eps_post, off_post, wn, eps_next, off_next, out, width, room KB_TL_SLOT(norm, 2, splits, wn != nullptr));
            return check_launch("add_rmsnorm");
        }
        if (cpt == 1) launch_dependent_if(rows <= DEPENDENT_ROWS, add_rmsnorm_splits_kernel<1>, dim3(rows), dim3(tv), 0, s, residual, b, splits, stride, wp, eps_post, off_post, wn, eps_next, off_next, out, width KB_TL_SLOT(norm, 2, splits, wn != nullptr));
        else if (cpt == 2) launch_dependent_if(rows <= DEPENDENT_ROWS, add_rmsnorm_splits_kernel<2>, dim3(rows), dim3(tv), 0, s, residual, b, splits, stride, wp, eps_post, off_post, wn, eps_next, off_next, out, width KB_TL_SLOT(norm, 2, splits, wn != nullptr));
        else launch_dependent_if(rows <= DEPENDENT_ROWS, add_rmsnorm_splits_kernel<4>, dim3(rows), dim3(tv), 0, s, residual, b, splits, stride, wp, eps_post, off_post, wn, eps_next, off_next, out, width KB_TL_SLOT(norm, 2, splits, wn != nullptr));
        return check_launch("add_rmsnorm");
    }
    switch (code) {
        case 0: KB_ADDNORM(float, float, float); break;
        case 1: KB_ADDNORM(float, float, bf16); break;
        case 2: KB_ADDNORM(float, bf16, float); break;
        case 3: KB_ADDNORM(float, bf16, bf16); break;
        case 4: KB_ADDNORM(bf16, float, float); break;
        case 5: KB_ADDNORM(bf16, float, bf16); break;
        case 6: KB_ADDNORM(bf16, bf16, float); break;
        case 7: KB_ADDNORM(bf16, bf16, bf16); break;
        default: return fail("add_rmsnorm: dtype codes branch %d, w %d, h %d are not known", branch_dt, w_dt, h_dt);
    }
#undef KB_ADDNORM
    return check_launch("add_rmsnorm");
}
