// C[M,N] = A[M,K] . W[N,K]^T for bfloat16 inputs with 32-bit accumulation, on the warp-level
// tensor-core path (mma.sync m16n8k16). Three kernels:
//
//  * `row16_kernel` for M <= 16 (decoding a few sequences): weights straight from global memory
//    into B fragments, activations through L1, no shared memory, split over K;
//  * `stream_kernel` for M <= 64 (decode and short portions): the weight matrix is read once,
//    straight from global memory into B fragments, 16 bytes a thread; the few activation rows
//    wait in shared memory. Work is split over K when N alone gives too few blocks; partial
//    sums go to scratch memory in 32-bit and `splitk_reduce_kernel` adds them in split order.
//    The number of splits depends on N and K only, so a row's result does not depend on M.
//  * `tile_kernel` for larger M: 128x128x64 tiles, cp.async in three stages, ldmatrix.
//
// Kapel's counterpart is the cutile `batched_matmul_nt` (crates/kapel-cuda/src/tile.rs:65-87,
// tiles by m :194-203). The tcgen05 kernel for large M lives in gemm_tcgen05.cu.
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ float epilogue_apply(float v, int epi, float cap) {
    return epi == 1 ? cap * tanhf(v / cap) : v;
}

// ---------------------------------------------------------------------------------------
// M <= 64.
//
// A block has 8 warps; warp w owns columns [n0 + w*8*NT, +8*NT) as NT n8 tiles and all MT m16
// tiles. K is walked 32 at a time. Within a group of 32 the k index is permuted the same way for
// A and B so that each thread's two B registers of two MMAs are 16 contiguous bytes of one
// weight row: thread (g = lane/4, t = lane%4) reads W[n + g][k32 + 8t .. 8t+7]; elements 0..3 feed
// the first MMA (as its k = 2t, 2t+1, 2t+8, 2t+9), elements 4..7 the second. A dot product does
// not care in which order its terms are paired as long as both sides agree.
constexpr int SK_KC = 512;                       // K positions of A held in shared memory at a time
constexpr int SK_STRIDE = SK_KC + 32;            // in elements: row stride 1088 B = 64 mod 128

template <int MT, int NT>
__global__ void __launch_bounds__(256)
stream_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, float* __restrict__ partial,
              void* __restrict__ c, int c_dt, int m, int n, int k, int k_per_split, int epi, float cap) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* sa = reinterpret_cast<bf16*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n_warp = blockIdx.x * (64 * NT) + warp * (8 * NT);
    const int split = blockIdx.y;
    const int k_begin = split * k_per_split;
    const int k_end = min(k, k_begin + k_per_split);

    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

    const bf16* wrow[NT];
    bool wvalid[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int col = n_warp + j * 8 + g;
        wvalid[j] = col < n;
        wrow[j] = w + (size_t)(wvalid[j] ? col : 0) * k;
    }

    for (int kc = k_begin; kc < k_end; kc += SK_KC) {
        const int kc_len = min(SK_KC, k_end - kc);           // a multiple of 8
        __syncthreads();                                     // the chunk before is no longer read
        // Stage A[0..MT*16, kc .. kc+kc_len) with zero rows beyond m and zero tail up to a multiple of 32.
        const int chunks_per_row = (kc_len + 31) / 32 * 4;   // 16-byte chunks, padded to k32 groups
        for (int id = threadIdx.x; id < MT * 16 * chunks_per_row; id += 256) {
            const int row = id / chunks_per_row, ch = id % chunks_per_row;
            const bool valid = row < m && ch * 8 < kc_len;
            cp_async16(sa + row * SK_STRIDE + ch * 8, a + (size_t)(valid ? row : 0) * k + kc + (valid ? ch * 8 : 0), valid);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();

        const int groups = (kc_len + 31) / 32;
#pragma unroll 2
        for (int gi = 0; gi < groups; ++gi) {
            const int koff = gi * 32 + t * 8;                // within the chunk
            const bool kvalid = koff < kc_len;
            uint4 bw[NT];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                bw[j] = make_uint4(0u, 0u, 0u, 0u);
                if (wvalid[j] && kvalid) bw[j] = __ldg(reinterpret_cast<const uint4*>(wrow[j] + kc + koff));
            }
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const uint4 lo = *reinterpret_cast<const uint4*>(sa + (i * 16 + g) * SK_STRIDE + koff);
                const uint4 hi = *reinterpret_cast<const uint4*>(sa + (i * 16 + g + 8) * SK_STRIDE + koff);
                const uint32_t a1[4] = {lo.x, hi.x, lo.y, hi.y};
                const uint32_t a2[4] = {lo.z, hi.z, lo.w, hi.w};
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    mma_bf16(acc[i][j], a1, bw[j].x, bw[j].y);
                    mma_bf16(acc[i][j], a2, bw[j].z, bw[j].w);
                }
            }
        }
    }

    // c0,c1: row g, columns 2t, 2t+1; c2,c3: row g+8.
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = i * 16 + g + (e >> 1) * 8;
                const int col = n_warp + j * 8 + t * 2 + (e & 1);
                if (row >= m || col >= n) continue;
                const float v = acc[i][j][e];
                if (partial != nullptr) {
                    partial[((size_t)split * m + row) * n + col] = v;
                } else {
                    const float o = epilogue_apply(v, epi, cap);
                    if (c_dt == KB_DT_F32) static_cast<float*>(c)[(size_t)row * n + col] = o;
                    else static_cast<bf16*>(c)[(size_t)row * n + col] = __float2bfloat16_rn(o);
                }
            }
}

__global__ void splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ c, int c_dt,
                                     long long mn, int splits, int epi, float cap) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= mn) return;
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += partial[(size_t)s * mn + i];
    v = epilogue_apply(v, epi, cap);
    if (c_dt == KB_DT_F32) static_cast<float*>(c)[i] = v;
    else static_cast<bf16*>(c)[i] = __float2bfloat16_rn(v);
}

// ---------------------------------------------------------------------------------------
// M <= 16 (decoding a few sequences): nothing waits in shared memory and nothing synchronises.
// A warp owns 8 * NT columns and walks its share of K in groups of 32 with the same k permutation
// as above; the weights come straight from global memory past L1, the few activation rows come
// through L1, where every warp of the multiprocessor finds them again. Four groups of loads are
// in flight a thread before the first MMA of an iteration. HI: rows 8..15 exist (M > 8).
__device__ __forceinline__ uint4 ld_stream16(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

constexpr int R16_U = 4;                          // k32 groups a loop iteration

template <int NT, bool HI>
__global__ void __launch_bounds__(128)
row16_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, float* __restrict__ partial,
             void* __restrict__ c, int c_dt, int m, int n, int k, int k_per_split, int epi, float cap) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n_warp = blockIdx.x * (32 * NT) + warp * (8 * NT);
    const int split = blockIdx.y;
    const int k_begin = split * k_per_split;
    const int k_end = min(k, k_begin + k_per_split);

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const bf16* wrow[NT];
    bool wvalid[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int col = n_warp + j * 8 + g;
        wvalid[j] = col < n;
        wrow[j] = w + (size_t)(wvalid[j] ? col : 0) * k;
    }
    const bool lo_valid = g < m, hi_valid = HI && (g + 8) < m;
    const bf16* alo = a + (size_t)(lo_valid ? g : 0) * k;
    const bf16* ahi = a + (size_t)(hi_valid ? g + 8 : 0) * k;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    for (int k0 = k_begin; k0 < k_end; k0 += 32 * R16_U) {
        uint4 bw[R16_U][NT], al[R16_U], ah[R16_U];
#pragma unroll
        for (int u = 0; u < R16_U; ++u) {
            const int kq = k0 + u * 32 + t * 8;
            const bool ok = kq < k_end;                     // k_end is a multiple of 8: the 16 bytes are whole
#pragma unroll
            for (int j = 0; j < NT; ++j) bw[u][j] = (ok && wvalid[j]) ? ld_stream16(wrow[j] + kq) : zero;
            al[u] = (ok && lo_valid) ? __ldg(reinterpret_cast<const uint4*>(alo + kq)) : zero;
            ah[u] = (HI && ok && hi_valid) ? __ldg(reinterpret_cast<const uint4*>(ahi + kq)) : zero;
        }
#pragma unroll
        for (int u = 0; u < R16_U; ++u) {
            const uint32_t a1[4] = {al[u].x, ah[u].x, al[u].y, ah[u].y};
            const uint32_t a2[4] = {al[u].z, ah[u].z, al[u].w, ah[u].w};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                mma_bf16(acc[j], a1, bw[u][j].x, bw[u][j].y);
                mma_bf16(acc[j], a2, bw[u][j].z, bw[u][j].w);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int row = g + (e >> 1) * 8;
            const int col = n_warp + j * 8 + t * 2 + (e & 1);
            if (row >= m || col >= n) continue;
            const float v = acc[j][e];
            if (partial != nullptr) {
                partial[((size_t)split * m + row) * n + col] = v;
            } else {
                const float o = epilogue_apply(v, epi, cap);
                if (c_dt == KB_DT_F32) static_cast<float*>(c)[(size_t)row * n + col] = o;
                else static_cast<bf16*>(c)[(size_t)row * n + col] = __float2bfloat16_rn(o);
            }
        }
}

// ---------------------------------------------------------------------------------------
// Larger M: 128 x 128 x 64 tiles, 8 warps as 2 x 4, each warp 64 x 32.
constexpr int TL_BM = 128, TL_BN = 128, TL_BK = 64, TL_STAGES = 3;
constexpr int TL_STAGE_ELEMS = (TL_BM + TL_BN) * TL_BK;

__device__ __forceinline__ int swz(int row, int chunk) { return row * TL_BK + ((chunk ^ (row & 7)) << 3); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}

__global__ void __launch_bounds__(256)
tile_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, void* __restrict__ c, int c_dt, int m, int n,
            int k, int epi, float cap) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp >> 2, wn = warp & 3;
    const int m0 = blockIdx.y * TL_BM, n0 = blockIdx.x * TL_BN;
    const int k_tiles = (k + TL_BK - 1) / TL_BK;

    auto load_stage = [&](int stage, int kt) {
        bf16* sa = smem + stage * TL_STAGE_ELEMS;
        bf16* sb = sa + TL_BM * TL_BK;
        const int k0 = kt * TL_BK;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int id = threadIdx.x + i * 256;
            const int row = id >> 3, ch = id & 7;
            const int gk = k0 + ch * 8;
            const bool va = (m0 + row) < m && gk < k;
            cp_async16(sa + swz(row, ch), a + (size_t)(va ? m0 + row : 0) * k + (va ? gk : 0), va);
            const bool vb = (n0 + row) < n && gk < k;
            cp_async16(sb + swz(row, ch), w + (size_t)(vb ? n0 + row : 0) * k + (vb ? gk : 0), vb);
        }
    };

    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

#pragma unroll
    for (int s = 0; s < TL_STAGES - 1; ++s) {
        if (s < k_tiles) load_stage(s, s);
        cp_async_commit();
    }

    for (int kt = 0; kt < k_tiles; ++kt) {
        cp_async_wait<TL_STAGES - 2>();
        __syncthreads();
        {   // refill the stage that was read in the iteration before
            const int nk = kt + TL_STAGES - 1;
            if (nk < k_tiles) load_stage(nk % TL_STAGES, nk);
            cp_async_commit();
        }
        const bf16* sa = smem + (kt % TL_STAGES) * TL_STAGE_ELEMS;
        const bf16* sb = sa + TL_BM * TL_BK;
#pragma unroll
        for (int ks = 0; ks < TL_BK / 16; ++ks) {
            uint32_t af[4][4], bfr[2][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = wm * 64 + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int ch = ks * 2 + (lane >> 4);
                ldmatrix_x4(af[i], sa + swz(row, ch));
            }
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int row = wn * 32 + jj * 16 + (lane & 7) + (lane >> 4) * 8;
                const int ch = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(bfr[jj], sb + swz(row, ch));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bfr[j >> 1][(j & 1) * 2], bfr[j >> 1][(j & 1) * 2 + 1]);
        }
    }
    cp_async_wait<0>();

    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = m0 + wm * 64 + i * 16 + g + (e >> 1) * 8;
                const int col = n0 + wn * 32 + j * 8 + t * 2 + (e & 1);
                if (row >= m || col >= n) continue;
                const float o = epilogue_apply(acc[i][j][e], epi, cap);
                if (c_dt == KB_DT_F32) static_cast<float*>(c)[(size_t)row * n + col] = o;
                else static_cast<bf16*>(c)[(size_t)row * n + col] = __float2bfloat16_rn(o);
            }
}

// The number of K splits of the streaming kernel for a weight [n, k] with `bn` columns a block:
// enough blocks for two a multiprocessor, each split at least one shared-memory chunk of K.
static int stream_splits(int n, int k, int bn, int sms) {
    const int col_blocks = (n + bn - 1) / bn;
    int splits = (2 * sms + col_blocks - 1) / col_blocks;
    const int max_splits = (k + SK_KC - 1) / SK_KC;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    return splits;
}

// The same for the M <= 16 kernel (64 columns a block of 4 warps): about four blocks a
// multiprocessor, each split at least 256 long. It depends on n and k only.
constexpr int R16_NT = 2;
static void row16_plan(int n, int k, int sms, int* splits, int* k_per_split) {
    const int col_blocks = (n + 32 * R16_NT - 1) / (32 * R16_NT);
    int s = (4 * sms + col_blocks / 2) / col_blocks;
    const int max_splits = (k + 255) / 256;
    if (s > max_splits) s = max_splits;
    if (s < 1) s = 1;
    int per = (k + s - 1) / s;
    per = (per + 31) / 32 * 32;
    *k_per_split = per;
    *splits = (k + per - 1) / per;
}

static int g_sms = 0;
static int sm_count() {
    if (g_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_sms <= 0) g_sms = 148;
    }
    return g_sms;
}

}  // namespace kb

using namespace kb;

// Scratch floats the streaming kernel needs for a product of these sizes (0 when it does not split).
extern "C" long long kb_gemm_bf16_scratch_floats(int m, int n, int k) {
    if (m <= 0 || m > 64) return 0;
    int splits, per;
    if (m <= 16) row16_plan(n, k, sm_count(), &splits, &per);
    else splits = stream_splits(n, k, 64 * 2, sm_count());      // every instantiation below uses NT = 2
    return splits > 1 ? (long long)splits * m * n : 0;
}

// How many partial sums the M <= 16 kernel leaves for a weight [n, k] (1: none, it writes the result).
extern "C" int kb_gemm_bf16_row16_splits(int n, int k) {
    int splits, per;
    row16_plan(n, k, sm_count(), &splits, &per);
    return splits;
}

static int launch_row16(const bf16* a, const bf16* w, float* partial, void* c, int c_dt, int m, int n, int k, int epi,
                        float cap, cudaStream_t s) {
    int splits, per;
    row16_plan(n, k, sm_count(), &splits, &per);
    dim3 grid((n + 32 * R16_NT - 1) / (32 * R16_NT), splits);
    if (splits > 1 && partial == nullptr) return fail("gemm_bf16: %d splits over K need scratch memory", splits);
    float* out = splits > 1 ? partial : nullptr;
    if (m > 8) row16_kernel<R16_NT, true><<<grid, 128, 0, s>>>(a, w, out, c, c_dt, m, n, k, per, epi, cap);
    else row16_kernel<R16_NT, false><<<grid, 128, 0, s>>>(a, w, out, c, c_dt, m, n, k, per, epi, cap);
    return check_launch("gemm_bf16 row16");
}

template <int MT, int NT>
static int launch_stream(const bf16* a, const bf16* w, float* scratch, void* c, int c_dt, int m, int n, int k,
                         int epi, float cap, cudaStream_t s) {
    const int bn = 64 * NT;
    const int splits = stream_splits(n, k, bn, sm_count());
    int k_per_split = (k + splits - 1) / splits;
    k_per_split = (k_per_split + 31) / 32 * 32;
    const int real_splits = (k + k_per_split - 1) / k_per_split;
    const size_t smem = (size_t)MT * 16 * SK_STRIDE * sizeof(bf16);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(stream_kernel<MT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr_set = true;
    }
    dim3 grid((n + bn - 1) / bn, real_splits);
    float* partial = real_splits > 1 ? scratch : nullptr;
    if (real_splits > 1 && scratch == nullptr) return fail("gemm_bf16: %d splits over K need scratch memory", real_splits);
    stream_kernel<MT, NT><<<grid, 256, smem, s>>>(a, w, partial, c, c_dt, m, n, k, k_per_split, epi, cap);
    if (int e = check_launch("gemm_bf16 stream")) return e;
    if (real_splits > 1) {
        const long long mn = (long long)m * n;
        splitk_reduce_kernel<<<(unsigned)((mn + 255) / 256), 256, 0, s>>>(partial, c, c_dt, mn, real_splits, epi, cap);
        return check_launch("gemm_bf16 split-K reduce");
    }
    return 0;
}

// a: bf16 [m,k]; w: bf16 [n,k]; c: bf16 or f32 [m,n]; scratch: f32, kb_gemm_bf16_scratch_floats(m,n,k) long.
extern "C" int kb_gemm_bf16(void* c, int c_dt, const void* a, const void* w, int m, int n, int k, int epilogue,
                            float cap, float* scratch, void* stream) {
    KB_REQUIRE(m >= 0 && n > 0 && k > 0, "gemm_bf16: m %d, n %d, k %d", m, n, k);
    KB_REQUIRE(k % 8 == 0, "gemm_bf16: k = %d must be a multiple of 8 (16-byte rows)", k);
    KB_REQUIRE(c_dt == KB_DT_F32 || c_dt == KB_DT_BF16, "gemm_bf16: output dtype code %d is not known", c_dt);
    KB_REQUIRE(epilogue == 0 || (epilogue == 1 && cap > 0.f), "gemm_bf16: epilogue %d with cap %g", epilogue, cap);
    KB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_bf16: operands must be 16-byte aligned");
    if (m == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bf16* ap = (const bf16*)a;
    const bf16* wp = (const bf16*)w;
    if (m <= 16) {
        if (int e = launch_row16(ap, wp, scratch, c, c_dt, m, n, k, epilogue, cap, s)) return e;
        const int splits = kb_gemm_bf16_row16_splits(n, k);
        if (splits > 1) {
            const long long mn = (long long)m * n;
            splitk_reduce_kernel<<<(unsigned)((mn + 255) / 256), 256, 0, s>>>(scratch, c, c_dt, mn, splits, epilogue, cap);
            return check_launch("gemm_bf16 split-K reduce");
        }
        return 0;
    }
    if (m <= 32) return launch_stream<2, 2>(ap, wp, scratch, c, c_dt, m, n, k, epilogue, cap, s);
    if (m <= 64) return launch_stream<4, 2>(ap, wp, scratch, c, c_dt, m, n, k, epilogue, cap, s);
    const size_t smem = (size_t)TL_STAGES * TL_STAGE_ELEMS * sizeof(bf16);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr_set = true;
    }
    dim3 grid((n + TL_BN - 1) / TL_BN, (m + TL_BM - 1) / TL_BM);
    KB_REQUIRE(grid.y <= 65535, "gemm_bf16: %d rows is too many for one launch", m);
    tile_kernel<<<grid, 256, smem, s>>>(ap, wp, c, c_dt, m, n, k, epilogue, cap);
    return check_launch("gemm_bf16 tile");
}

// The M <= 16 product without its reduction: partial[s, m, n] for s < kb_gemm_bf16_row16_splits(n, k),
// to be added up by whoever reads them (a norm, a gated unit, the rotation). With one split the
// "partial" sums are the result.
extern "C" int kb_gemm_bf16_partial(float* partial, const void* a, const void* w, int m, int n, int k, void* stream) {
    KB_REQUIRE(m > 0 && m <= 16 && n > 0 && k > 0, "gemm_bf16_partial: m %d (1..16), n %d, k %d", m, n, k);
    KB_REQUIRE(k % 8 == 0, "gemm_bf16_partial: k = %d must be a multiple of 8 (16-byte rows)", k);
    KB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_bf16_partial: operands must be 16-byte aligned");
    KB_REQUIRE(partial != nullptr, "gemm_bf16_partial: no output");
    // One split writes its sums through the "direct" path as float32, which is the same memory.
    return launch_row16((const bf16*)a, (const bf16*)w, partial, partial, KB_DT_F32, m, n, k, 0, 0.f, (cudaStream_t)stream);
}

// out[i] = sum over `splits` slices of partial[s * mn + i], in slice order.
extern "C" int kb_splitk_reduce(void* out, int out_dt, const float* partial, long long mn, int splits, void* stream) {
    KB_REQUIRE(mn >= 0 && splits >= 1, "splitk_reduce: %lld elements, %d slices", mn, splits);
    KB_REQUIRE(out_dt == KB_DT_F32 || out_dt == KB_DT_BF16, "splitk_reduce: output dtype code %d is not known", out_dt);
    if (mn == 0) return 0;
    splitk_reduce_kernel<<<(unsigned)((mn + 255) / 256), 256, 0, (cudaStream_t)stream>>>(partial, out, out_dt, mn, splits, 0, 0.f);
    return check_launch("splitk_reduce");
}

// ---------------------------------------------------------------------------------------
// The product for callers that cannot allocate (declared and described in no_alloc.h; no
// counterpart in smallbard/kapel). The split-K partial sums live in this array, which is part
// of the library's image on every device that loads it.
#include "no_alloc.h"
#include <mutex>

static __device__ __align__(256) float g_no_alloc_scratch[KB_NO_ALLOC_SCRATCH_FLOATS];

namespace kb {

constexpr int NO_ALLOC_MAX_DEVICES = 64;
static float* g_no_alloc_ptr[NO_ALLOC_MAX_DEVICES] = {};
static std::mutex g_no_alloc_mutex;

// The device address of the scratch array on the current device. In host code the array's
// name is only a handle for the runtime, not an address a kernel could use; the address comes
// from cudaGetSymbolAddress, once per device, with that device current.
static int no_alloc_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail("gemm_bf16_no_alloc: no current device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= NO_ALLOC_MAX_DEVICES) return fail("gemm_bf16_no_alloc: device %d is beyond the %d this entry point keeps addresses for", dev, NO_ALLOC_MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_no_alloc_mutex);
    if (g_no_alloc_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_no_alloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail("gemm_bf16_no_alloc: cannot find the built-in scratch array on device %d: %s", dev, cudaGetErrorString(e));
        g_no_alloc_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_no_alloc_ptr[dev];
    return 0;
}

}  // namespace kb

extern "C" int kb_gemm_bf16_no_alloc(void* c, int c_dt, const void* a, const void* w, int m, int n, int k, int epilogue,
                                     float cap, void* stream) {
    KB_REQUIRE(m >= 0 && n > 0 && k > 0, "gemm_bf16_no_alloc: m %d, n %d, k %d", m, n, k);
    KB_REQUIRE(m <= 64, "gemm_bf16_no_alloc: m = %d; this entry point takes at most 64 rows", m);
    const long long need = kb_gemm_bf16_scratch_floats(m, n, k);
    KB_REQUIRE(need <= (long long)KB_NO_ALLOC_SCRATCH_FLOATS,
               "gemm_bf16_no_alloc: [%d, %d] x [%d, %d] needs %lld scratch values; the built-in array holds %d", m, k, n, k,
               need, KB_NO_ALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (int e = no_alloc_scratch(&scratch)) return e;
    // Nothing has to start at zero: each split writes all m x n of its partial sums before the
    // reduction reads them, and the reduction reads nothing else.
    return kb_gemm_bf16(c, c_dt, a, w, m, n, k, epilogue, cap, scratch, stream);
}
