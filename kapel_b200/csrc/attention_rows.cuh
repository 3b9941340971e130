// (shared by attention_f32.cu and attention_bf16.cu)
// Attention over the paged cache, one query row at a time ("rows" kernels), for any element
// type. A query row that has seen c positions (its own included) reads keys
// [max(0, c - window), c) of its sequence through the block table; score = scale * q.k, then
// cap * tanh(score / cap) if a cap is given, softmax over what it sees, weighted sum of values;
// a row that sees nothing gives zeros. Scores, soft cap, softmax and sums are 32-bit.
//
// Kapel's counterparts: kernels/src/lib.rs paged_attention :1850, paged_combine :2135; rules in
// crates/kapel-ops/src/paged.rs:16-25,65-70.
//
// One block = one row x one kv head (a slice of up to GMAX of its query heads) x one chunk of
// CHUNK key positions. Chunks are cut at absolute multiples of CHUNK, so what a row computes
// does not depend on the rest of the batch. With more than one chunk slot the blocks write
// (sum p.v, max, sum p) to scratch memory and `combine_kernel` merges them in chunk order.
#pragma once
#include "common.cuh"

namespace kb {

constexpr int ATT_CHUNK = 256;
constexpr int ATT_THREADS = 128;
constexpr int ATT_WARPS = ATT_THREADS / 32;

// exp for the softmax: the library's in the 32-bit path, the fast one otherwise.
template <typename T> __device__ __forceinline__ float soft_exp(float x) { return __expf(x); }
template <> __device__ __forceinline__ float soft_exp<float>(float x) { return expf(x); }

template <typename T> struct Vec;      // 16 bytes of T
template <> struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&out)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&out)[8]) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(u[i] << 16);
            out[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }
};

struct AttParams {
    const void* q;            // [rows, hq, d]
    const void* k_table;      // [pages, hkv, page_size, d]
    const void* v_table;
    const int* block_table;   // [entries, table_width]
    const int* row_entry;     // [rows]
    const int* row_count;     // [rows]
    void* out;                // [rows, hq, d]
    float* partial;           // [rows, hq, slots, d + 2] or null when slots == 1
    int rows, hq, hkv, d, page_size, table_width, n_pages;
    int window;               // 0: none
    int slots;                // chunk slots a row may touch
    float scale, cap;         // cap 0: none
};

// LPK: lanes that share one key (a power of two); VPL: 16-byte vectors of a key each lane holds.
template <typename T, int GMAX, int LPK, int VPL>
__global__ void __launch_bounds__(ATT_THREADS)
rows_kernel(const AttParams p) {
    constexpr int VN = Vec<T>::N;
    extern __shared__ __align__(16) float smem[];
    const int group = p.hq / p.hkv;
    const int gslices = (group + GMAX - 1) / GMAX;
    const int r = blockIdx.x;
    const int kvh = blockIdx.y / gslices;
    const int g0 = (blockIdx.y % gslices) * GMAX;
    const int gn = min(GMAX, group - g0);                 // query heads of this block
    const int d = p.d;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int count = p.row_count[r];
    const int first = (p.window > 0 && count > p.window) ? count - p.window : 0;
    const int chunk = first / ATT_CHUNK + blockIdx.z;      // absolute chunk index
    const int lo = max(first, chunk * ATT_CHUNK);
    const int hi = min(count, (chunk + 1) * ATT_CHUNK);
    const int nkeys = hi - lo;
    T* out = static_cast<T*>(p.out);

    if (nkeys <= 0) {
        // Nothing in this slot. The first slot of a row that sees nothing at all writes zeros.
        if (blockIdx.z == 0 && count <= 0)
            for (int g = 0; g < gn; ++g)
                for (int i = tid; i < d; i += ATT_THREADS)
                    Elem<T>::store(out + ((size_t)r * p.hq + kvh * group + g0 + g) * d + i, 0.f);
        return;
    }

    // shared: q [GMAX][d] | scores [GMAX][CHUNK] | lines [CHUNK] | stats [2*GMAX] | acc [groups][GMAX][d]
    float* sq = smem;
    float* ss = sq + GMAX * d;
    int* sline = reinterpret_cast<int*>(ss + GMAX * ATT_CHUNK);
    float* sstat = reinterpret_cast<float*>(sline + ATT_CHUNK);
    float* sacc = sstat + 2 * GMAX;

    const int entry = p.row_entry[r];
    const T* q = static_cast<const T*>(p.q) + ((size_t)r * p.hq + kvh * group + g0) * d;
    for (int i = tid; i < gn * d; i += ATT_THREADS) sq[i] = Elem<T>::load(q + i);
    for (int j = tid; j < nkeys; j += ATT_THREADS) {
        const int pos = lo + j;
        const int lp = pos / p.page_size;
        const int page = lp < p.table_width ? p.block_table[(size_t)entry * p.table_width + lp] : -1;
        // A page outside the table would be a fault of the cache manager; such a key is skipped
        // by giving it line -1, and its score becomes -inf below.
        sline[j] = (page >= 0 && page < p.n_pages) ? page * p.page_size + pos % p.page_size : -1;
    }
    __syncthreads();

    // ---- scores
    const T* kt = static_cast<const T*>(p.k_table);
    constexpr int KPW = 32 / LPK;                          // keys a warp handles at a time
    const int sub = lane / LPK, li = lane % LPK;
    const int nvec = d / VN;
    for (int j0 = warp * KPW; j0 < nkeys; j0 += ATT_WARPS * KPW) {
        const int j = j0 + sub;
        const bool live = j < nkeys;
        const int line = live ? sline[j] : -1;
        float kv[VPL][VN];
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int vi = li + v * LPK;
            if (line >= 0 && vi < nvec) {
                Vec<T>::load(kt + kv_row(line, kvh, p.hkv, p.page_size) * d + vi * VN, kv[v]);
            } else {
#pragma unroll
                for (int e = 0; e < VN; ++e) kv[v][e] = 0.f;
            }
        }
        for (int g = 0; g < gn; ++g) {
            float dot = 0.f;
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int vi = li + v * LPK;
                if (vi < nvec) {
#pragma unroll
                    for (int e = 0; e < VN; ++e) dot = fmaf(kv[v][e], sq[g * d + vi * VN + e], dot);
                }
            }
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (live && li == 0) {
                float s = dot * p.scale;
                if (p.cap > 0.f) s = p.cap * tanhf(s / p.cap);
                ss[g * ATT_CHUNK + j] = line >= 0 ? s : -INFINITY;
            }
        }
    }
    __syncthreads();

    // ---- softmax within the chunk: one warp a head
    for (int g = warp; g < gn; g += ATT_WARPS) {
        float m = -INFINITY;
        for (int j = lane; j < nkeys; j += 32) m = fmaxf(m, ss[g * ATT_CHUNK + j]);
        m = warp_max(m);
        float l = 0.f;
        for (int j = lane; j < nkeys; j += 32) {
            const float s = ss[g * ATT_CHUNK + j];
            const float e = (m == -INFINITY) ? 0.f : soft_exp<T>(s - m);
            ss[g * ATT_CHUNK + j] = e;
            l += e;
        }
        l = warp_sum(l);
        if (lane == 0) { sstat[2 * g] = m; sstat[2 * g + 1] = l; }
    }
    __syncthreads();

    // ---- weighted sum of values: a thread owns two neighbouring components; thread groups of
    // d/2 share the keys when d/2 < ATT_THREADS, and add up in group order afterwards.
    const T* vt = static_cast<const T*>(p.v_table);
    const int pairs = d / 2;
    const int tgroups = pairs >= ATT_THREADS ? 1 : ATT_THREADS / pairs;
    const int tg = tid / pairs;                            // this thread's group (may be >= tgroups)
    float acc[GMAX][2];
    for (int pi = (tgroups == 1 ? tid : tid % pairs); pi < pairs; pi += ATT_THREADS) {
#pragma unroll
        for (int g = 0; g < GMAX; ++g) acc[g][0] = acc[g][1] = 0.f;
        if (tgroups == 1 || tg < tgroups) {
            const int jstart = tgroups == 1 ? 0 : tg;
            for (int j = jstart; j < nkeys; j += tgroups) {
                const int line = sline[j];
                if (line < 0) continue;
                const T* vp = vt + kv_row(line, kvh, p.hkv, p.page_size) * d + 2 * pi;
                const float v0 = Elem<T>::load(vp), v1 = Elem<T>::load(vp + 1);
#pragma unroll
                for (int g = 0; g < GMAX; ++g) {
                    if (g < gn) {
                        const float w = ss[g * ATT_CHUNK + j];
                        acc[g][0] = fmaf(w, v0, acc[g][0]);
                        acc[g][1] = fmaf(w, v1, acc[g][1]);
                    }
                }
            }
        }
        if (tgroups > 1) {
            if (tg < tgroups) {
#pragma unroll
                for (int g = 0; g < GMAX; ++g)
                    if (g < gn) {
                        sacc[((size_t)tg * GMAX + g) * d + 2 * pi] = acc[g][0];
                        sacc[((size_t)tg * GMAX + g) * d + 2 * pi + 1] = acc[g][1];
                    }
            }
            __syncthreads();
            if (tg == 0) {
#pragma unroll
                for (int g = 0; g < GMAX; ++g)
                    if (g < gn)
                        for (int x = 1; x < tgroups; ++x) {
                            acc[g][0] += sacc[((size_t)x * GMAX + g) * d + 2 * pi];
                            acc[g][1] += sacc[((size_t)x * GMAX + g) * d + 2 * pi + 1];
                        }
            }
        }
        if (tgroups == 1 || tg == 0) {
#pragma unroll
            for (int g = 0; g < GMAX; ++g) {
                if (g >= gn) continue;
                const int h = kvh * group + g0 + g;
                if (p.slots == 1) {
                    const float l = sstat[2 * g + 1];
                    const float inv = l > 0.f ? 1.f / l : 0.f;
                    T* o = out + ((size_t)r * p.hq + h) * d + 2 * pi;
                    Elem<T>::store(o, acc[g][0] * inv);
                    Elem<T>::store(o + 1, acc[g][1] * inv);
                } else {
                    float* o = p.partial + (((size_t)r * p.hq + h) * p.slots + blockIdx.z) * (d + 2);
                    o[2 * pi] = acc[g][0];
                    o[2 * pi + 1] = acc[g][1];
                    if (pi == 0) { o[d] = sstat[2 * g]; o[d + 1] = sstat[2 * g + 1]; }
                }
            }
        }
    }
}

// out[r, h, :] = sum_z e^(m_z - M) acc_z / sum_z e^(m_z - M) l_z over the slots the row touched.
template <typename T>
__global__ void combine_kernel(const AttParams p) {
    const int r = blockIdx.x, h = blockIdx.y;
    const int count = p.row_count[r];
    T* o = static_cast<T*>(p.out) + ((size_t)r * p.hq + h) * p.d;
    if (count <= 0) return;                                // the rows kernel wrote zeros
    const int first = (p.window > 0 && count > p.window) ? count - p.window : 0;
    const int used = (count - 1) / ATT_CHUNK - first / ATT_CHUNK + 1;
    const float* base = p.partial + ((size_t)r * p.hq + h) * p.slots * (p.d + 2);
    float mx = -INFINITY;
    for (int z = 0; z < used; ++z) mx = fmaxf(mx, base[(size_t)z * (p.d + 2) + p.d]);
    float denom = 0.f;
    for (int z = 0; z < used; ++z) {
        const float m = base[(size_t)z * (p.d + 2) + p.d];
        denom += (m == -INFINITY ? 0.f : soft_exp<T>(m - mx)) * base[(size_t)z * (p.d + 2) + p.d + 1];
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    for (int i = threadIdx.x; i < p.d; i += blockDim.x) {
        float acc = 0.f;
        for (int z = 0; z < used; ++z) {
            const float m = base[(size_t)z * (p.d + 2) + p.d];
            const float w = m == -INFINITY ? 0.f : soft_exp<T>(m - mx);
            acc = fmaf(w, base[(size_t)z * (p.d + 2) + i], acc);
        }
        Elem<T>::store(o + i, acc * inv);
    }
}

static size_t rows_smem_bytes(int gmax, int d) {
    const int pairs = d / 2;
    const int tgroups = pairs >= ATT_THREADS ? 1 : ATT_THREADS / pairs;
    size_t floats = (size_t)gmax * d + (size_t)gmax * ATT_CHUNK + ATT_CHUNK + 2 * gmax;
    if (tgroups > 1) floats += (size_t)tgroups * gmax * d;
    return floats * sizeof(float);
}

template <typename T, int GMAX, int LPK, int VPL>
static int launch_rows(const AttParams& p, cudaStream_t s) {
    const size_t smem = rows_smem_bytes(GMAX, p.d);
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return fail("paged_attention: head_dim %d needs %zu bytes of shared memory", p.d, smem);
        cudaFuncSetAttribute(rows_kernel<T, GMAX, LPK, VPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    const int group = p.hq / p.hkv;
    dim3 grid(p.rows, p.hkv * ((group + GMAX - 1) / GMAX), p.slots);
    rows_kernel<T, GMAX, LPK, VPL><<<grid, ATT_THREADS, smem, s>>>(p);
    return check_launch("paged_attention rows");
}

template <typename T, int GMAX>
static int dispatch_lanes(const AttParams& p, cudaStream_t s) {
    const int nvec = p.d / Vec<T>::N;                     // 16-byte vectors of a key
    int lpk = 1;
    while (lpk * 2 <= nvec && lpk < 32) lpk *= 2;
    const int vpl = (nvec + lpk - 1) / lpk;
#define KB_ATT(L, V) return launch_rows<T, GMAX, L, V>(p, s)
    if (vpl == 1) {
        switch (lpk) {
            case 2: KB_ATT(2, 1);
            case 4: KB_ATT(4, 1);
            case 8: KB_ATT(8, 1);
            case 16: KB_ATT(16, 1);
            case 32: KB_ATT(32, 1);
        }
    } else if (vpl == 2) {
        switch (lpk) {
            case 4: KB_ATT(4, 2);
            case 8: KB_ATT(8, 2);
            case 16: KB_ATT(16, 2);
            case 32: KB_ATT(32, 2);
        }
    } else if (vpl <= 4 && lpk == 32) {
        KB_ATT(32, 4);
    }
#undef KB_ATT
    return fail("paged_attention: head_dim %d is not handled (at most %d)", p.d, 32 * 4 * Vec<T>::N);
}

template <typename T>
static int dispatch_group(const AttParams& p, cudaStream_t s) {
    const int group = p.hq / p.hkv;
    if (group <= 1) return dispatch_lanes<T, 1>(p, s);
    if (group <= 2) return dispatch_lanes<T, 2>(p, s);
    if (group <= 4) return dispatch_lanes<T, 4>(p, s);
    return dispatch_lanes<T, 8>(p, s);                    // larger groups run as slices of 8 heads
}


template <typename T>
static int run_rows(const AttParams& p, cudaStream_t s, bool combine) {
    if (int e = dispatch_group<T>(p, s)) return e;
    if (combine) {
        dim3 grid(p.rows, p.hq);
        combine_kernel<T><<<grid, 128, 0, s>>>(p);
        return check_launch("paged_attention combine");
    }
    return 0;
}

int rows_f32(const AttParams& p, cudaStream_t s, bool combine);
int rows_bf16(const AttParams& p, cudaStream_t s, bool combine);

}  // namespace kb
