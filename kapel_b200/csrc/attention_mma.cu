// Paged attention on tensor cores (mma.sync m16n8k16, bfloat16 inputs, 32-bit scores, softmax
// and sums), reading keys and values in place through the block table: no gather copy.
//
// Kapel's counterparts: the cutile FlashAttention forward after a gather of the pages
// (crates/kapel-cuda/src/attention.rs:107-247, crates/kapel-cuda/src/paged.rs:66-114) for prompts, and
// paged_attention_16 (kernels/src/lib.rs:2949) for decoding. Here one kernel does both:
//
//  * a tile is up to MROWS rows of one request and one kv head; a row is (token, query head of
//    the kv head's group), so the group shares every key and value it loads;
//  * keys and values arrive in shared memory 64 positions at a time by cp.async, two stages;
//  * prompt mode (DECODE = false, 64 rows): each of 4 warps owns 16 rows and walks all keys;
//  * decode mode (DECODE = true, 16 rows): the 4 warps share the 16 rows and each takes a quarter
//    of every 64 keys with a softmax state of its own, merged through shared memory at the end;
//  * score = scale * q.k, then cap * tanh(score / cap) (tanh.approx), then the mask: a row that
//    has seen c positions reads keys [max(0, c - window), c);
//  * with `split` > 0 the keys are also cut at absolute multiples of `split` across blockIdx.z;
//    each block writes (sum p.v, max, sum p) to scratch memory and a second kernel merges them.
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

constexpr int AM_THREADS = 128;
constexpr int AM_KT = 64;             // keys a tile
constexpr int AM_PAD = 8;             // elements of padding a shared-memory row (16 bytes)

struct AttMmaParams {
    const bf16* q;             // [rows, hq, d]
    const bf16* k_table;       // [lines, hkv, d]
    const bf16* v_table;
    const int* block_table;    // [entries, table_width]
    const int* row_count;      // [rows]
    const int* tile_entry;     // [tiles]
    const int* tile_row0;      // [tiles] first row (token) of the tile in the batch
    const int* tile_nq;        // [tiles] tokens in the tile
    bf16* out;                 // [rows, hq, d]
    float* partial;            // [rows, hq, slots, d + 2] when slots > 1
    int rows, hq, hkv, d, page_size, table_width, n_pages;
    int window, split, slots;
    float scale, cap;
};

__device__ __forceinline__ void am_cp_async16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void am_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void am_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void am_ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void am_ldmatrix_x4_trans(uint32_t (&r)[4], const bf16* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void am_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float am_tanh(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t am_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// HD: the largest head_dim this instantiation takes (registers are sized by it).
template <int HD, bool DECODE>
__global__ void __launch_bounds__(AM_THREADS)
attention_mma_kernel(const AttMmaParams p) {
    constexpr int MROWS = DECODE ? 16 : 64;
    constexpr int WKEYS = DECODE ? AM_KT / 4 : AM_KT;      // keys a warp handles of each tile
    constexpr int NT_S = WKEYS / 8;                         // score n-tiles a warp
    constexpr int NT_O = HD / 8;                            // output n-tiles
    extern __shared__ __align__(128) unsigned char am_smem[];

    const int d = p.d;
    const int ld = d + AM_PAD;
    bf16* sQ = reinterpret_cast<bf16*>(am_smem);
    bf16* sK = sQ + MROWS * ld;                             // [2][KT][ld]
    bf16* sV = sK + 2 * AM_KT * ld;                         // [2][KT][ld]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x, kvh = blockIdx.y, slot = blockIdx.z;
    const int group = p.hq / p.hkv;
    const int entry = p.tile_entry[tile];
    const int row0 = p.tile_row0[tile];
    const int nq = p.tile_nq[tile];
    const int rows_valid = nq * group;
    const int c_first = p.row_count[row0];
    const int c_last = c_first + nq - 1;

    // The keys this block walks.
    int klo = (p.window > 0 && c_first > p.window) ? c_first - p.window : 0;
    int khi = c_last;
    if (c_first <= 0) khi = 0;                              // a padding row sees nothing
    if (p.split > 0) {
        klo = max(klo, slot * p.split);
        khi = min(khi, (slot + 1) * p.split);
    }
    if (klo >= khi) {
        if (p.slots == 1 && c_first <= 0) {
            for (int i = tid; i < rows_valid * d; i += AM_THREADS) {
                const int r = i / d, c = i % d;
                p.out[((size_t)(row0 + r / group) * p.hq + kvh * group + r % group) * d + c] = __float2bfloat16_rn(0.f);
            }
        }
        return;
    }
    const int k_begin = klo / AM_KT * AM_KT;               // tiles are cut at multiples of KT
    const int n_tiles = (khi - k_begin + AM_KT - 1) / AM_KT;

    // ---- loads
    const int chunks = d / 8;                               // 16-byte chunks a row
    {
        for (int i = tid; i < MROWS * chunks; i += AM_THREADS) {
            const int r = i / chunks, ch = i % chunks;
            const bool valid = r < rows_valid;
            const bf16* src = p.q + ((size_t)(row0 + (valid ? r / group : 0)) * p.hq + kvh * group + (valid ? r % group : 0)) * d + ch * 8;
            am_cp_async16(sQ + r * ld + ch * 8, src, valid);
        }
    }
    // Two threads a key row: each loads half of the row's chunks, of K and of V.
    const int lrow = tid >> 1, lhalf = tid & 1;
    auto load_tile = [&](int stage, int kt) {
        const int j = k_begin + kt * AM_KT + lrow;
        bool valid = j >= klo && j < khi;
        size_t line = 0;
        if (valid) {
            const int lp = j / p.page_size;
            const int page = lp < p.table_width ? p.block_table[(size_t)entry * p.table_width + lp] : -1;
            valid = page >= 0 && page < p.n_pages;
            line = valid ? (size_t)page * p.page_size + j % p.page_size : 0;
        }
        const bf16* ksrc = p.k_table + (line * p.hkv + kvh) * d;
        const bf16* vsrc = p.v_table + (line * p.hkv + kvh) * d;
        bf16* kd = sK + ((size_t)stage * AM_KT + lrow) * ld;
        bf16* vd = sV + ((size_t)stage * AM_KT + lrow) * ld;
        const int half = (chunks + 1) / 2;
        const int c0 = lhalf * half, c1 = min(chunks, c0 + half);
        for (int ch = c0; ch < c1; ++ch) am_cp_async16(kd + ch * 8, ksrc + ch * 8, valid);
        for (int ch = c0; ch < c1; ++ch) am_cp_async16(vd + ch * 8, vsrc + ch * 8, valid);
    };
    load_tile(0, 0);
    am_commit();

    // ---- state
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    const int wrow = DECODE ? 0 : warp * 16;                // first row of this warp
    const int wkey = DECODE ? warp * WKEYS : 0;             // first key of this warp within a tile
    // rows g and g + 8 of the warp's 16: their tokens' counts and first visible keys
    int cnt[2], fst[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = wrow + g + h * 8;
        const bool valid = r < rows_valid;
        cnt[h] = valid ? c_first + r / group : 0;
        fst[h] = (p.window > 0 && cnt[h] > p.window) ? cnt[h] - p.window : 0;
    }
    const float sc = p.cap > 0.f ? p.scale / p.cap : p.scale;
    const float LOG2E = 1.4426950408889634f;

    for (int kt = 0; kt < n_tiles; ++kt) {
        am_wait<0>();
        __syncthreads();                                    // tile kt landed; the other stage is free
        if (kt + 1 < n_tiles) load_tile((kt + 1) & 1, kt + 1);
        am_commit();
        const bf16* tK = sK + (size_t)(kt & 1) * AM_KT * ld;
        const bf16* tV = sV + (size_t)(kt & 1) * AM_KT * ld;
        const int j0 = k_begin + kt * AM_KT + wkey;         // first key of this warp's part

        // scores S[16 x WKEYS] = Q K^T
        float s[NT_S][4];
#pragma unroll
        for (int i = 0; i < NT_S; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            if (ks * 16 < d) {
                uint32_t a[4];
                am_ldmatrix_x4(a, sQ + (wrow + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int nb = 0; nb < NT_S / 2; ++nb) {
                    uint32_t b[4];
                    am_ldmatrix_x4(b, tK + (wkey + nb * 16 + (lane & 7) + (lane >> 4) * 8) * ld + ks * 16 + ((lane >> 3) & 1) * 8);
                    am_mma(s[2 * nb], a, b[0], b[1]);
                    am_mma(s[2 * nb + 1], a, b[2], b[3]);
                }
            }
        }
        // scale, soft cap, mask; tile maximum
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < NT_S; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const int j = j0 + nt * 8 + t * 2 + (e & 1);
                float v = s[nt][e] * sc;
                if (p.cap > 0.f) v = p.cap * am_tanh(v);
                const bool seen = j >= fst[h] && j < cnt[h] && j >= klo && j < khi;
                v = seen ? v : -INFINITY;
                s[nt][e] = v;
                mx[h] = fmaxf(mx[h], v);
            }
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            alpha[h] = (m_new == -INFINITY) ? 1.f : exp2f((m_run[h] - m_new) * LOG2E);
            m_run[h] = m_new;
            l_run[h] *= alpha[h];
        }
        // p = exp(s - m); the row sums stay per thread until the end
        uint32_t pa[NT_S / 2][4];
#pragma unroll
        for (int nt = 0; nt < NT_S; ++nt) {
            float pv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                pv[e] = (s[nt][e] == -INFINITY) ? 0.f : exp2f((s[nt][e] - m_run[h]) * LOG2E);
                l_run[h] += pv[e];
            }
            // the C layout of two neighbouring n-tiles is the A layout of one k16 step
            pa[nt >> 1][(nt & 1) * 2] = am_pack(pv[0], pv[1]);
            pa[nt >> 1][(nt & 1) * 2 + 1] = am_pack(pv[2], pv[3]);
        }
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
        // O += P V
#pragma unroll
        for (int kb = 0; kb < NT_S / 2; ++kb) {
#pragma unroll
            for (int nd = 0; nd < HD / 16; ++nd) {
                if (nd * 16 < d) {
                    uint32_t b[4];
                    am_ldmatrix_x4_trans(b, tV + (wkey + kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + nd * 16 + (lane >> 4) * 8);
                    am_mma(o[2 * nd], pa[kb], b[0], b[1]);
                    am_mma(o[2 * nd + 1], pa[kb], b[2], b[3]);
                }
            }
        }
    }
    am_wait<0>();

    // ---- row sums across the 4 lanes of a row
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }

    if (DECODE) {
        // Merge the 4 warps' states: O, m, l per row through shared memory (the stages are free).
        __syncthreads();
        float* mO = reinterpret_cast<float*>(sK);           // [4][16][d]
        float* mM = mO + 4 * 16 * d;                        // [4][16]
        float* mL = mM + 4 * 16;
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            if (i * 8 < d) {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    mO[((size_t)warp * 16 + g + (e >> 1) * 8) * d + i * 8 + t * 2 + (e & 1)] = o[i][e];
            }
        }
        if (t == 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mM[warp * 16 + g + h * 8] = m_run[h];
                mL[warp * 16 + g + h * 8] = l_run[h];
            }
        }
        __syncthreads();
        for (int i = tid; i < rows_valid * d; i += AM_THREADS) {
            const int r = i / d, c = i % d;
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) mx = fmaxf(mx, mM[w * 16 + r]);
            float acc = 0.f, l = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float mw = mM[w * 16 + r];
                const float f = (mw == -INFINITY) ? 0.f : exp2f((mw - mx) * LOG2E);
                acc = fmaf(f, mO[((size_t)w * 16 + r) * d + c], acc);
                l = fmaf(f, mL[w * 16 + r], l);
            }
            const int row = row0 + r / group, head = kvh * group + r % group;
            if (p.slots == 1) {
                p.out[((size_t)row * p.hq + head) * d + c] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
            } else {
                float* dst = p.partial + (((size_t)row * p.hq + head) * p.slots + slot) * (d + 2);
                dst[c] = acc;
                if (c == 0) { dst[d] = mx; dst[d + 1] = l; }
            }
        }
    } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = wrow + g + h * 8;
            if (r >= rows_valid) continue;
            const int row = row0 + r / group, head = kvh * group + r % group;
            if (p.slots == 1) {
                const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
                bf16* dst = p.out + ((size_t)row * p.hq + head) * d;
#pragma unroll
                for (int i = 0; i < NT_O; ++i)
                    if (i * 8 < d)
                        *reinterpret_cast<uint32_t*>(dst + i * 8 + t * 2) = am_pack(o[i][h * 2] * inv, o[i][h * 2 + 1] * inv);
            } else {
                float* dst = p.partial + (((size_t)row * p.hq + head) * p.slots + slot) * (d + 2);
#pragma unroll
                for (int i = 0; i < NT_O; ++i)
                    if (i * 8 < d) { dst[i * 8 + t * 2] = o[i][h * 2]; dst[i * 8 + t * 2 + 1] = o[i][h * 2 + 1]; }
                if (t == 0) { dst[d] = m_run[h]; dst[d + 1] = l_run[h]; }
            }
        }
    }
}

// out[row, head, :] = sum_z e^(m_z - M) acc_z / sum_z e^(m_z - M) l_z over the absolute slots the
// row's own keys fall in; a row that sees nothing gets zeros.
__global__ void attention_mma_combine_kernel(const AttMmaParams p) {
    const int row = blockIdx.x, head = blockIdx.y;
    const int count = p.row_count[row];
    bf16* o = p.out + ((size_t)row * p.hq + head) * p.d;
    if (count <= 0) {
        for (int i = threadIdx.x; i < p.d; i += blockDim.x) o[i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int first = (p.window > 0 && count > p.window) ? count - p.window : 0;
    const int z0 = first / p.split, z1 = min(p.slots - 1, (count - 1) / p.split);
    const float* base = p.partial + ((size_t)row * p.hq + head) * p.slots * (p.d + 2);
    const int stride = p.d + 2;
    float mx = -INFINITY;
    for (int z = z0; z <= z1; ++z) mx = fmaxf(mx, base[(size_t)z * stride + p.d]);
    float denom = 0.f;
    for (int z = z0; z <= z1; ++z) {
        const float m = base[(size_t)z * stride + p.d];
        denom += (m == -INFINITY ? 0.f : __expf(m - mx)) * base[(size_t)z * stride + p.d + 1];
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    for (int i = threadIdx.x; i < p.d; i += blockDim.x) {
        float acc = 0.f;
        for (int z = z0; z <= z1; ++z) {
            const float m = base[(size_t)z * stride + p.d];
            const float w = m == -INFINITY ? 0.f : __expf(m - mx);
            acc = fmaf(w, base[(size_t)z * stride + i], acc);
        }
        o[i] = __float2bfloat16_rn(acc * inv);
    }
}

template <int HD, bool DECODE>
static int launch_mma(const AttMmaParams& p, int tiles, cudaStream_t s) {
    constexpr int MROWS = DECODE ? 16 : 64;
    const int ld = p.d + AM_PAD;
    size_t smem = ((size_t)MROWS * ld + 4 * (size_t)AM_KT * ld) * sizeof(bf16);
    if (DECODE) {
        const size_t merge = ((size_t)4 * 16 * p.d + 2 * 4 * 16) * sizeof(float);
        const size_t stages = 4 * (size_t)AM_KT * ld * sizeof(bf16);
        if (merge > stages) smem += merge - stages;
    }
    if (smem > 220 * 1024) return fail("attention_mma: head_dim %d needs %zu bytes of shared memory", p.d, smem);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(attention_mma_kernel<HD, DECODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(tiles, p.hkv, p.slots);
    attention_mma_kernel<HD, DECODE><<<grid, AM_THREADS, smem, s>>>(p);
    return check_launch("attention_mma");
}

}  // namespace kb

using namespace kb;

// Rows a tile may hold in each mode; the host cuts requests into tiles of rows / group tokens.
extern "C" int kb_attention_mma_rows(int decode) { return decode ? 16 : 64; }

extern "C" long long kb_attention_mma_scratch_floats(int rows, int hq, int d, int slots) {
    return slots > 1 ? (long long)rows * hq * slots * (d + 2) : 0;
}

extern "C" int kb_attention_mma(void* out, const void* q, const void* k_table, const void* v_table,
                                const int* block_table, const int* row_count, const int* tile_entry,
                                const int* tile_row0, const int* tile_nq, int tiles, int rows, int hq, int hkv, int d,
                                int page_size, int table_width, int n_pages, int window, int split, int slots,
                                float scale, float cap, int decode, float* scratch, void* stream) {
    KB_REQUIRE(rows >= 0 && tiles >= 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "attention_mma: rows %d, tiles %d, heads %d over %d", rows, tiles, hq, hkv);
    KB_REQUIRE(d > 0 && d % 16 == 0 && d <= 256, "attention_mma: head_dim %d must be a multiple of 16, at most 256", d);
    KB_REQUIRE(hq / hkv <= (decode ? 16 : 64), "attention_mma: %d query heads a kv head do not fit a tile of %d rows", hq / hkv, decode ? 16 : 64);
    KB_REQUIRE(page_size > 0 && table_width > 0 && n_pages > 0, "attention_mma: page_size %d, table width %d, pages %d", page_size, table_width, n_pages);
    KB_REQUIRE(window >= 0 && cap >= 0.f, "attention_mma: window %d, cap %g", window, cap);
    KB_REQUIRE((split == 0 && slots == 1) || (split > 0 && split % AM_KT == 0 && slots >= 1 && slots <= 65535),
               "attention_mma: split %d (a multiple of %d) with %d slots", split, AM_KT, slots);
    KB_REQUIRE(slots == 1 || scratch != nullptr, "attention_mma: %d slots need scratch memory", slots);
    KB_REQUIRE(hkv <= 65535, "attention_mma: %d kv heads is too many for one launch", hkv);
    if (rows == 0 || tiles == 0) return 0;
    AttMmaParams p;
    p.q = (const bf16*)q; p.k_table = (const bf16*)k_table; p.v_table = (const bf16*)v_table;
    p.block_table = block_table; p.row_count = row_count; p.tile_entry = tile_entry; p.tile_row0 = tile_row0;
    p.tile_nq = tile_nq; p.out = (bf16*)out; p.partial = slots > 1 ? scratch : nullptr;
    p.rows = rows; p.hq = hq; p.hkv = hkv; p.d = d; p.page_size = page_size; p.table_width = table_width;
    p.n_pages = n_pages; p.window = window; p.split = split; p.slots = slots; p.scale = scale; p.cap = cap;
    cudaStream_t s = (cudaStream_t)stream;
    int e;
    if (d <= 64) e = decode ? launch_mma<64, true>(p, tiles, s) : launch_mma<64, false>(p, tiles, s);
    else if (d <= 128) e = decode ? launch_mma<128, true>(p, tiles, s) : launch_mma<128, false>(p, tiles, s);
    else e = decode ? launch_mma<256, true>(p, tiles, s) : launch_mma<256, false>(p, tiles, s);
    if (e) return e;
    if (slots > 1) {
        dim3 grid(rows, hq);
        attention_mma_combine_kernel<<<grid, 128, 0, s>>>(p);
        return check_launch("attention_mma combine");
    }
    return 0;
}
