// Paged attention on tensor cores (mma.sync m16n8k16, bfloat16 inputs, 32-bit scores, softmax
// and sums), reading keys and values in place through the block table: no gather copy.
//
// Kapel's counterparts: the cutile FlashAttention forward after a gather of the pages
// (crates/kapel-cuda/src/attention.rs:107-247, crates/kapel-cuda/src/paged.rs:66-114) for prompts, and
// paged_attention_16 (kernels/src/lib.rs:2949) for decoding. Here one file does both (prompt
// portions with a soft cap and a head size of 64, 128 or 256 go to the tcgen05 kernel of
// attention_tc.cu instead; this file's prompt kernel takes the rest):
//
//  * a tile is up to MROWS rows of one request and one kv head; a row is (token, query head of
//    the kv head's group), so the group shares every key and value it loads;
//  * `attention_mma_kernel` (prompt portions, 128 rows): keys and values arrive 64 positions at a
//    time as TMA boxes in two stages; each of 8 warps owns 16 rows and walks all keys;
//  * `attention_decode_kernel` (16 rows: a few tokens of one request): the 4 warps share the rows;
//    each warp streams its own tiles of 16 keys through a three-stage pipeline of its own, filled
//    by TMA: the cache tables are [pages, kv heads, page size, head_dim], so the 16 keys of a kv
//    head lie together, and a tile arrives as head_dim / 64 boxes of 16 x 64 elements for the keys
//    and as many for the values (cp.async.bulk.tensor, 128-byte swizzle, completion on an
//    mbarrier). The loop has no block-wide barrier, a tile costs one instruction in each of 8 lanes
//    to fetch, and ~128 KB are in flight a multiprocessor. The products are taken with the
//    operands swapped (S^T = K Q^T, O^T = V^T P^T: the keys are the MMAs' M). Each warp keeps a
//    softmax state of its own and the four are merged through shared memory. Every wait on an
//    mbarrier gives up after about a second, raises a flag that `kb_attention_error` reports, and
//    the block leaves without writing;
//  * score = scale * q.k, then cap * tanh(score / cap) (tanh.approx), then the mask: a row that
//    has seen c positions reads keys [max(0, c - window), c);
//  * with `split` > 0 the keys are also cut at multiples of `split` across blocks (counted from
//    key 0 or, when every tile is one token, from the row's first visible key); each block writes
//    (sum p.v, max, sum p) to scratch memory and a second kernel merges them;
//  * the decode kernel and the merge are launched as programmatic dependents: they wait for the
//    kernel before them only where they first touch what it wrote.
#include "common.cuh"
#include "tensor_map.cuh"
#include "timeline.cuh"

namespace kb {

KB_TIMELINE_ARRAY(attention)   // slots: kind 4 decoding attention (slots, window), kind 5 its merge


typedef __nv_bfloat16 bf16;

constexpr int AM_THREADS = 128;
constexpr int AM_KT = 64;             // keys a tile
constexpr int AM_PAD = 8;             // elements of padding a shared-memory row (16 bytes)

struct AttMmaParams {
    const bf16* q;             // [rows, hq, d]
    const bf16* k_table;       // [pages, hkv, page_size, d]
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
    int decode_bar_offset;     // bytes from the start of shared memory to the decode kernel's mbarriers
    int direct;                // 1: a row whose keys all lie in one slot was written to `out` by that slot's block
    int relative;              // 1: every request brings one token (tile t = row t = request t) and slots are counted from the row's first visible key, else from key 0
    float scale, cap;
    // The decode kernel taking over the rotation and the cache's newest line (null: the queries come in `q`):
    const float* qkv_parts;    // [qkv_splits][rows][(hq + 2 hkv) d] partial sums of the stacked q|k|v product
    long long qkv_stride;      // floats from one slice to the next
    int qkv_splits;
    int stage_offset;          // bytes from the start of shared memory to where the slices land
    const float2* cos_sin;     // [rows][d / 2] (cos, sin) of each row's position
    const int* lines;          // [rows] the cache line of each row's token; negative: none
    bf16* k_new;               // the key and value tables to write the newest line to; null: the layer reads another layer's cache
    bf16* v_new;
    long long table_lines;
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
__device__ __forceinline__ float am_exp2(float x) {      // 2^x, one instruction; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t am_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---- the copy engine: bulk copies global -> shared that complete on an mbarrier
__device__ int g_attention_error = 0;       // set when a wait on an mbarrier ran out

__device__ __forceinline__ uint32_t am_saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void am_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(am_saddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void am_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(am_saddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void am_bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(am_saddr(dst)), "l"(src), "r"(bytes), "r"(am_saddr(bar)) : "memory");
}
__device__ __forceinline__ void am_tma_box(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(am_saddr(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void am_ldmatrix_x4_at(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
__device__ __forceinline__ void am_ldmatrix_x4_trans_at(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
// Waits for the phase with this parity to complete; false if it did not within ~1 s.
__device__ __forceinline__ bool am_mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = am_saddr(bar);
    const long long start = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if (clock64() - start > 2000000000ll) return false;
    }
}

// One warp's work on one tile of 16 keys with the operands swapped, for the decode kernel, where
// only a few of the 16 rows exist: S^T = K Q^T and O^T = V^T P^T. The 16 keys are the MMAs' M; the rows ("heads" here:
// (token, query head) pairs) are their N, eight a block, NB blocks. Q waits in registers as B
// fragments (`bq`), so it costs no load in the loop; O^T is 16 x NB x 4 registers instead of 128;
// and 16 keys cost 16 + 16 MMAs and ldmatrix instead of 32 + 32 and 48.
//   Lane (g, t) holds S^T[key g (+8)][head 8 nb + 2t (+1)]; cnt/fst are those heads' counts and
//   first visible keys; m_run/l_run their softmax states (every g holds a copy; the row sums stay
//   per lane until the end). `ot[nd][nb]` holds O^T[dim 16 nd + g (+8)][head 8 nb + 2t (+1)].
//   tK, tV: shared-memory addresses (1024-byte aligned) of the tile's keys and values as TMA left
//   them: boxes of 16 rows x 64 elements (2 KB), one after the other along head_dim, each under the
//   128-byte swizzle: the 16-byte piece c of row r lies at piece c ^ (r & 7).
template <int HD, int NB, bool FULL>
__device__ __forceinline__ void ad_tile(const uint32_t (&bq)[HD / 16][NB][2], uint32_t tK, uint32_t tV, int d,
                                        int j0, const int (&cnt)[NB][2], const int (&fst)[NB][2], int fst_hi, int cnt_lo,
                                        int klo, int khi, float sc, float cap, float (&ot)[HD / 16][NB][4],
                                        float (&m_run)[NB][2], float (&l_run)[NB][2], int lane) {
    const int g = lane >> 2, t = lane & 3;
    const float LOG2E = 1.4426950408889634f;
    float st[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) st[nb][0] = st[nb][1] = st[nb][2] = st[nb][3] = 0.f;
    const int krow = (lane & 7) + ((lane >> 3) & 1) * 8;       // the key row this lane addresses
    const uint32_t ka = tK + krow * 128;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        if (FULL || ks * 16 < d) {
            uint32_t a[4];
            const int piece = ((ks & 3) << 1) + (lane >> 4);   // 16-byte piece within the box's 128-byte row
            am_ldmatrix_x4_at(a, ka + (ks >> 2) * 2048 + ((piece ^ (krow & 7)) << 4));
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) am_mma(st[nb], a, bq[ks][nb][0], bq[ks][nb][1]);
        }
    }
    const bool inner = j0 >= fst_hi && j0 + 16 <= cnt_lo && j0 >= klo && j0 + 16 <= khi;
    float alpha[NB][2];
    uint32_t pb[NB][2];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int h = e & 1;                             // head 2t + h; key g + 8 (e >> 1)
            float v = st[nb][e] * sc;
            if (cap > 0.f) v = cap * am_tanh(v);
            if (!inner) {
                const int j = j0 + g + (e >> 1) * 8;
                const bool seen = j >= fst[nb][h] && j < cnt[nb][h] && j >= klo && j < khi;
                v = seen ? v : -INFINITY;
            }
            st[nb][e] = v;
            mx[h] = fmaxf(mx[h], v);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {                        // over the 16 keys: across g
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
            const float m_new = fmaxf(m_run[nb][h], mx[h]);
            alpha[nb][h] = (m_new == -INFINITY) ? 1.f : am_exp2((m_run[nb][h] - m_new) * LOG2E);
            m_run[nb][h] = m_new;
            l_run[nb][h] *= alpha[nb][h];
        }
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int h = e & 1;
            pv[e] = (st[nb][e] == -INFINITY) ? 0.f : am_exp2((st[nb][e] - m_run[nb][h]) * LOG2E);
            l_run[nb][h] += pv[e];
        }
        // P^T as a B fragment: lane (g, t) needs P[head 8 nb + g][keys 2t, 2t+1, 2t+8, 2t+9]. Key 2t
        // lives in lane (2t, g / 2), key 2t + 1 in lane (2t + 1, g / 2); the head picks the component.
        const int src_a = (2 * t) * 4 + (g >> 1), src_b = src_a + 4;
        float qa[4], qb[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            qa[e] = __shfl_sync(0xffffffffu, pv[e], src_a);
            qb[e] = __shfl_sync(0xffffffffu, pv[e], src_b);
        }
        const int odd = g & 1;
        pb[nb][0] = am_pack(odd ? qa[1] : qa[0], odd ? qb[1] : qb[0]);
        pb[nb][1] = am_pack(odd ? qa[3] : qa[2], odd ? qb[3] : qb[2]);
    }
    bool rescale = false;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) rescale = rescale || alpha[nb][0] != 1.f || alpha[nb][1] != 1.f;
    if (__any_sync(0xffffffffu, rescale)) {                  // the running maximum settles after a few tiles
#pragma unroll
        for (int nd = 0; nd < HD / 16; ++nd)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                ot[nd][nb][0] *= alpha[nb][0]; ot[nd][nb][1] *= alpha[nb][1];
                ot[nd][nb][2] *= alpha[nb][0]; ot[nd][nb][3] *= alpha[nb][1];
            }
    }
    // V^T as A fragments by transposing loads: matrix i of a load is keys 8 (i / 2).., dims 8 (i % 2)..
    const int vrow = (lane & 7) + ((lane >> 4) & 1) * 8;
    const uint32_t va = tV + vrow * 128;
#pragma unroll
    for (int nd = 0; nd < HD / 16; ++nd) {
        if (FULL || nd * 16 < d) {
            uint32_t a[4];
            const int piece = ((nd & 3) << 1) + ((lane >> 3) & 1);
            am_ldmatrix_x4_trans_at(a, va + (nd >> 2) * 2048 + ((piece ^ (vrow & 7)) << 4));
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) am_mma(ot[nd][nb], a, pb[nb][0], pb[nb][1]);
        }
    }
}

// The line of key position j of a request, or -1 if the block table has no page for it.
__device__ __forceinline__ long long am_line(const AttMmaParams& p, int entry, int j) {
    const int lp = j / p.page_size;
    const int page = lp < p.table_width ? p.block_table[(size_t)entry * p.table_width + lp] : -1;
    return (page >= 0 && page < p.n_pages) ? (long long)page * p.page_size + j % p.page_size : -1;
}

// What both kernels know of their tile.
struct AmTile {
    int entry, row0, nq, rows_valid, c_first, klo, khi, group;
};

__device__ __forceinline__ AmTile am_tile_info(const AttMmaParams& p, int tile, int slot) {
    AmTile x;
    x.group = p.hq / p.hkv;
    if (p.relative) {
        // every request brings one token: tile t is row t of request t, and the three lists need not
        // be read (one trip to memory fewer before the row's count, its pages and its first keys)
        x.entry = x.row0 = tile;
        x.nq = 1;
    } else {
        x.entry = p.tile_entry[tile];
        x.row0 = p.tile_row0[tile];
        x.nq = p.tile_nq[tile];
    }
    x.rows_valid = x.nq * x.group;
    x.c_first = p.row_count[x.row0];
    x.klo = (p.window > 0 && x.c_first > p.window) ? x.c_first - p.window : 0;
    x.khi = x.c_first > 0 ? x.c_first + x.nq - 1 : 0;       // a padding row sees nothing
    if (p.split > 0) {
        // Counted from the window's start, a windowed row's keys fill whole slots: window / split of
        // them, not one more with a sliver at each end.
        const int base = p.relative ? x.klo : 0;
        x.klo = max(x.klo, base + slot * p.split);
        x.khi = min(x.khi, base + (slot + 1) * p.split);
    }
    return x;
}

// One warp's 16 query rows against 64 keys that TMA left in shared memory as boxes of 16 keys x 64
// elements (2 KB, 128-byte swizzle): box (sub, x) of the keys holds keys 16 sub .. and elements
// 64 x .., boxes in (sub, x) order, `nbox` of them along head_dim; the values likewise.
// S = Q K^T, scale, soft cap, mask, online softmax, O += P V. HD sizes the registers; d <= HD.
//   q16: the warp's 16 query rows (rows `ld` elements apart); j0: the absolute position of the
//   first key; cnt/fst: count and first visible key of rows g and g+8 (a row beyond the tile's own
//   has count INT_MAX: what it computes is never written); fst_hi/cnt_lo: the warp's largest
//   first-visible key and smallest count, so that only tiles at an edge are masked.
//   FULL: d == HD, known when the kernel is compiled, so the loops carry no size tests.
template <int HD, bool FULL>
__device__ __forceinline__ void am_tile_boxes(const bf16* q16, uint32_t tK, uint32_t tV, int ld, int d, int nbox, int j0,
                                              const int (&cnt)[2], const int (&fst)[2], int fst_hi, int cnt_lo, int klo,
                                              int khi, float sc, float cap, float (&o)[HD / 8][4], float (&m_run)[2],
                                              float (&l_run)[2], int lane) {
    constexpr int NKEYS = 64;
    constexpr int NT_S = NKEYS / 8;
    constexpr int NT_O = HD / 8;
    const int t = lane & 3;
    const float LOG2E = 1.4426950408889634f;
    float s[NT_S][4];
#pragma unroll
    for (int i = 0; i < NT_S; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    const int kr = (lane & 7) + (lane >> 4) * 8;              // key row within a box, for the score product
    const uint32_t kbase = tK + kr * 128;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        if (FULL || ks * 16 < d) {
            uint32_t a[4];
            am_ldmatrix_x4(a, q16 + ((lane & 7) + ((lane >> 3) & 1) * 8) * ld + ks * 16 + (lane >> 4) * 8);
            const uint32_t koff = (uint32_t)(ks >> 2) * 2048u + (uint32_t)(((((ks & 3) << 1) + ((lane >> 3) & 1)) ^ (kr & 7)) << 4);
#pragma unroll
            for (int nb = 0; nb < NT_S / 2; ++nb) {             // keys 16 nb ..: box row `sub` = nb
                uint32_t b[4];
                am_ldmatrix_x4_at(b, kbase + (uint32_t)(nb * nbox) * 2048u + koff);
                am_mma(s[2 * nb], a, b[0], b[1]);
                am_mma(s[2 * nb + 1], a, b[2], b[3]);
            }
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
    const bool inner = j0 >= fst_hi && j0 + NKEYS <= cnt_lo && j0 >= klo && j0 + NKEYS <= khi;
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int h = e >> 1;
            float v = s[nt][e] * sc;
            if (cap > 0.f) v = cap * am_tanh(v);
            if (!inner) {
                const int j = j0 + nt * 8 + t * 2 + (e & 1);
                const bool seen = j >= fst[h] && j < cnt[h] && j >= klo && j < khi;
                v = seen ? v : -INFINITY;
            }
            s[nt][e] = v;
            mx[h] = fmaxf(mx[h], v);
        }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[h], mx[h]);
        alpha[h] = (m_new == -INFINITY) ? 1.f : am_exp2((m_run[h] - m_new) * LOG2E);
        m_run[h] = m_new;
        l_run[h] *= alpha[h];
    }
    uint32_t pa[NT_S / 2][4];
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int h = e >> 1;
            pv[e] = (s[nt][e] == -INFINITY) ? 0.f : am_exp2((s[nt][e] - m_run[h]) * LOG2E);
            l_run[h] += pv[e];
        }
        pa[nt >> 1][(nt & 1) * 2] = am_pack(pv[0], pv[1]);
        pa[nt >> 1][(nt & 1) * 2 + 1] = am_pack(pv[2], pv[3]);
    }
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
    }
    const int vr = (lane & 7) + ((lane >> 3) & 1) * 8;        // key row within a box, for the value product
    const uint32_t vbase = tV + vr * 128;
#pragma unroll
    for (int kb = 0; kb < NT_S / 2; ++kb) {
#pragma unroll
        for (int nd = 0; nd < HD / 16; ++nd) {
            if (FULL || nd * 16 < d) {
                uint32_t b[4];
                const uint32_t voff = (uint32_t)(kb * nbox + (nd >> 2)) * 2048u + (uint32_t)(((((nd & 3) << 1) + (lane >> 4)) ^ (vr & 7)) << 4);
                am_ldmatrix_x4_trans_at(b, vbase + voff);
                am_mma(o[2 * nd], pa[kb], b[0], b[1]);
                am_mma(o[2 * nd + 1], pa[kb], b[2], b[3]);
            }
        }
    }
}

// Prompt portions: 128 rows a block, each of 8 warps 16 of them over all the block's keys, which
// arrive 64 positions at a time as TMA boxes, two stages.
constexpr int AP_THREADS = 256;
constexpr int AP_ROWS = 128;

template <int HD, bool FULL>
__global__ void __launch_bounds__(AP_THREADS)
attention_mma_kernel(const AttMmaParams p, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v) {
    constexpr int NT_O = HD / 8;
    extern __shared__ __align__(128) unsigned char am_smem[];
    const int d = p.d;
    const int ld = d + AM_PAD;
    const int nbox = (d + 63) / 64;
    bf16* sQ = reinterpret_cast<bf16*>(am_smem);                     // [128][ld]
    const uint32_t half_bytes = 4u * nbox * 2048u;                   // a tile's keys (or values): 4 x nbox boxes
    const uint32_t stage_bytes = 2u * half_bytes;
    const uint32_t smem0 = am_saddr(am_smem);
    const uint32_t stages = (smem0 + AP_ROWS * ld * (uint32_t)sizeof(bf16) + 1023u) & ~1023u;
    unsigned char* stages_ptr = am_smem + (stages - smem0);
    uint64_t* bars = reinterpret_cast<uint64_t*>(stages_ptr + 2 * stage_bytes);    // [2] stage full
    int* sPage = reinterpret_cast<int*>(bars + 2);                   // [2][4] pages of a tile's four groups of 16 keys

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.x, slot = blockIdx.y;
    // Later tiles of a prompt see more keys: they start first, all their heads and slots together,
    // so that blocks are handed out roughly by falling length.
    const AmTile x = am_tile_info(p, gridDim.z - 1 - blockIdx.z, slot);
    const int group = x.group, row0 = x.row0, rows_valid = x.rows_valid, klo = x.klo, khi = x.khi;
    if (klo >= khi) {
        if (p.slots == 1 && x.c_first <= 0)
            for (int i = tid; i < rows_valid * d; i += AP_THREADS) {
                const int r = i / d, c = i % d;
                p.out[((size_t)(row0 + r / group) * p.hq + kvh * group + r % group) * d + c] = __float2bfloat16_rn(0.f);
            }
        return;
    }
    const int k_begin = klo / AM_KT * AM_KT;               // tiles are cut at multiples of KT
    const int n_tiles = (khi - k_begin + AM_KT - 1) / AM_KT;

    if (tid == 0) {
        am_mbar_init(bars, 1);
        am_mbar_init(bars + 1, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int chunks = d / 8;                               // 16-byte chunks a row
    for (int i = tid; i < AP_ROWS * chunks; i += AP_THREADS) {
        const int r = i / chunks, ch = i % chunks;
        const bool valid = r < rows_valid;
        const bf16* src = p.q + ((size_t)(row0 + (valid ? r / group : 0)) * p.hq + kvh * group + (valid ? r % group : 0)) * d + ch * 8;
        am_cp_async16(sQ + r * ld + ch * 8, src, valid);
    }
    am_commit();
    // The pages of tile kt's four groups of 16 keys, written one iteration ahead by four threads.
    auto find_pages = [&](int kt) {
        if (tid < 4) {
            const int j = k_begin + kt * AM_KT + tid * 16;
            int page = -1;
            if (kt < n_tiles && j < khi && j + 16 > klo) {
                const int lp = max(j, klo) / p.page_size;
                if (lp < p.table_width) page = p.block_table[(size_t)x.entry * p.table_width + lp];
                if (page >= p.n_pages) page = -1;
            }
            sPage[(kt & 1) * 4 + tid] = page;
        }
    };
    // Warp 0 asks TMA for the boxes of tile kt: operation o is group o / (2 nbox), and of that group
    // the keys' box o % (2 nbox) or, from nbox on, the values' box. Groups without a page are cleared
    // by everyone instead.
    auto load_tile = [&](int kt) {
        const int stage = kt & 1;
        const int* pages = sPage + stage * 4;
        const uint32_t dst = stages + (uint32_t)stage * stage_bytes;
        int live = 0;
#pragma unroll
        for (int sub = 0; sub < 4; ++sub) live += pages[sub] >= 0 ? 1 : 0;
        if (tid == 0) am_mbar_expect_tx(bars + stage, (uint32_t)live * 2u * nbox * 2048u);
        __syncwarp();
        if (warp == 0) {
            for (int op = lane; op < 8 * nbox; op += 32) {
                const int sub = op / (2 * nbox), bx = op % (2 * nbox);
                const int page = pages[sub];
                if (page < 0) continue;
                const int j = k_begin + kt * AM_KT + sub * 16;
                const int row = (page * p.hkv + kvh) * p.page_size + j % p.page_size;
                if (bx < nbox) am_tma_box(dst + (uint32_t)(sub * nbox + bx) * 2048u, &map_k, bx * 64, row, bars + stage);
                else am_tma_box(dst + half_bytes + (uint32_t)(sub * nbox + bx - nbox) * 2048u, &map_v, (bx - nbox) * 64, row, bars + stage);
            }
        }
        if (live < 4) {
            for (int sub = 0; sub < 4; ++sub) {
                if (pages[sub] >= 0) continue;
                uint4* zk = reinterpret_cast<uint4*>(stages_ptr + (size_t)stage * stage_bytes + (size_t)sub * nbox * 2048);
                uint4* zv = reinterpret_cast<uint4*>(stages_ptr + (size_t)stage * stage_bytes + half_bytes + (size_t)sub * nbox * 2048);
                for (int i = tid; i < nbox * 128; i += AP_THREADS) { zk[i] = make_uint4(0u, 0u, 0u, 0u); zv[i] = make_uint4(0u, 0u, 0u, 0u); }
            }
        }
    };
    find_pages(0);
    find_pages(1);
    __syncthreads();                                        // barriers initialised, pages of tiles 0 and 1 known
    load_tile(0);

    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int wrow = warp * 16;
    int cnt[2], fst[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = wrow + g + h * 8;
        const bool own = r < rows_valid;
        cnt[h] = own ? x.c_first + r / group : 0x7fffffff;
        fst[h] = (own && p.window > 0 && cnt[h] > p.window) ? cnt[h] - p.window : 0;
    }
    const int fst_hi = __reduce_max_sync(0xffffffffu, max(fst[0], fst[1]));
    const int cnt_lo = __reduce_min_sync(0xffffffffu, min(cnt[0], cnt[1]));
    const float sc = p.cap > 0.f ? p.scale / p.cap : p.scale;
    am_wait<0>();                                           // this thread's part of Q has landed

    bool failed = false;
    for (int kt = 0; kt < n_tiles; ++kt) {
        if (!am_mbar_wait(bars + (kt & 1), (uint32_t)(kt >> 1) & 1u)) failed = true;
        if (__syncthreads_or(failed)) { failed = true; break; }       // tile kt landed (and Q); the other stage is free
        if (kt + 1 < n_tiles) load_tile(kt + 1);
        find_pages(kt + 2);                                 // read after the next barrier; last read before this one
        const uint32_t tk = stages + (uint32_t)(kt & 1) * stage_bytes;
        am_tile_boxes<HD, FULL>(sQ + wrow * ld, tk, tk + half_bytes, ld, d, nbox, k_begin + kt * AM_KT, cnt, fst, fst_hi, cnt_lo,
                                klo, khi, sc, p.cap, o, m_run, l_run, lane);
    }
    if (failed) {
        if (tid == 0) atomicExch(&g_attention_error, 1);
        return;                                             // a copy never completed: nothing is written
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = wrow + g + h * 8;
        if (r >= rows_valid) continue;
        const int row = row0 + r / group, head = kvh * group + r % group;
        // With several slots, a row whose keys all lie in one slot is finished by that slot's block.
        const int z0 = p.slots > 1 ? fst[h] / p.split : 0;
        const int z1 = p.slots > 1 ? min(p.slots - 1, (cnt[h] - 1) / p.split) : 0;
        if (z0 == z1) {
            if (slot != z0) continue;
            const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
            bf16* dst = p.out + ((size_t)row * p.hq + head) * d;
#pragma unroll
            for (int i = 0; i < NT_O; ++i)
                if (FULL || i * 8 < d)
                    *reinterpret_cast<uint32_t*>(dst + i * 8 + t * 2) = am_pack(o[i][h * 2] * inv, o[i][h * 2 + 1] * inv);
        } else {
            float* dst = p.partial + (((size_t)row * p.hq + head) * p.slots + slot) * (d + 2);
#pragma unroll
            for (int i = 0; i < NT_O; ++i)
                if (FULL || i * 8 < d) { dst[i * 8 + t * 2] = o[i][h * 2]; dst[i * 8 + t * 2 + 1] = o[i][h * 2 + 1]; }
            if (t == 0) { dst[d] = m_run[h]; dst[d + 1] = l_run[h]; }
        }
    }
}

// A few tokens of one request: 16 rows a block shared by its 4 warps. Warp w walks the tiles of
// 16 keys numbered w, w + 4, w + 8, ... of the block's keys through a pipeline of its own.
constexpr int AD_WK = 16;             // keys a warp tile
constexpr int AD_STAGES = 3;

// FUSED (one token a request, the whole head rotated): the kernel takes the stacked q|k|v product's
// partial sums instead of finished queries. Every block brings its kv head's query heads of its row in
// by bulk copies (one a slice), adds the slices up in order, rotates and leaves them where the queries
// lie otherwise. The one block of a (row, kv head) whose keys end with the row's own position also
// brings the key's and the value's slices in (behind the queries, into the same place; the warp that
// owns the slot's last tile asks and waits, at the end of its walk), writes them to the cache's line
// for the steps to come, and puts them into its own copy of that tile, which TMA fetched before the
// line was written. The sums, the rotation and the roundings are rope_append's, bit for bit.
// (Asked for behind the block's first 192 KB of keys and values, the queries' slices landed 3.3 us
// after the wait, by bulk copies and by the threads' own loads alike; hence the wait first.)
template <int HD, int NB, bool FULL, bool FUSED>
__global__ void __launch_bounds__(AM_THREADS)
attention_decode_kernel(const AttMmaParams p, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v KB_TL_PARAM) {
    extern __shared__ __align__(128) unsigned char am_smem[];
    const int d = p.d;
    const int ld = d + AM_PAD;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    bf16* sQ = reinterpret_cast<bf16*>(am_smem);            // [16][ld]
    // The pipelines start at the next multiple of 1024 bytes (the swizzle's period); a stage is the
    // tile's keys then its values, each head_dim / 64 boxes of 2 KB.
    const int nbox = (d + 63) / 64;
    const uint32_t stage_bytes = 2u * nbox * 2048u;
    const uint32_t smem0 = am_saddr(am_smem);
    const uint32_t pipes = ((smem0 + 16 * ld * (uint32_t)sizeof(bf16) + 1023u) & ~1023u);
    const uint32_t my_pipe = pipes + (uint32_t)warp * AD_STAGES * stage_bytes;
    unsigned char* pipes_ptr = am_smem + (pipes - smem0);
    uint64_t* bars = reinterpret_cast<uint64_t*>(am_smem + p.decode_bar_offset) + warp * AD_STAGES;

    const int kvh = blockIdx.y, slot = blockIdx.z;
    KB_TL_ENTER(attention, blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0, 4, p.slots, p.window);
    // Counts, tiles and block tables were copied in before the step began: they may be read ahead of
    // the wait on the kernel before this one, whose work the queries and the newest keys are.
    const AmTile x = am_tile_info(p, blockIdx.x, slot);
    const int group = x.group, row0 = x.row0, rows_valid = x.rows_valid, klo = x.klo, khi = x.khi;
    if (klo >= khi) {                                       // nothing here: the merge kernel skips this slot
        dependent_wait();
        if (p.slots == 1 && x.c_first <= 0)                 // a padding row without a merge kernel: zeros
            for (int i = tid; i < rows_valid * d; i += AM_THREADS) {
                const int r = i / d, c = i % d;
                p.out[((size_t)(row0 + r / group) * p.hq + kvh * group + r % group) * d + c] = __float2bfloat16_rn(0.f);
            }
        return;
    }
    const int k_begin = klo / AD_WK * AD_WK;
    const int n_tiles = (khi - k_begin + AD_WK - 1) / AD_WK;

    uint64_t* qbar = reinterpret_cast<uint64_t*>(am_smem + p.decode_bar_offset) + 4 * AD_STAGES;     // FUSED: the queries' slices have landed
    uint64_t* kvbar = qbar + 1;                                                                       // FUSED: the key's and the value's
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < AD_STAGES; ++s) am_mbar_init(bars + s, 1);
        if (FUSED && warp == 0) { am_mbar_init(qbar, 1); am_mbar_init(kvbar, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();                                           // a warp's barriers are its own
    if (FUSED) __syncthreads();                             // but the two of the slices are everyone's
    // A tile is 16 consecutive positions from a multiple of 16: with pages of a multiple of 16
    // positions it lies in one page, where the kv head's rows are consecutive. Lane i < nbox asks
    // TMA for box i of the keys, lane nbox + i for box i of the values. A tile whose page the
    // block table does not hold is cleared instead. Positions of the tile outside the block's
    // range arrive too (they are masked): what a page holds beyond a sequence's end is what an
    // earlier sequence left there, finite values that meet a weight of exactly zero.
    const uint32_t tile_bytes = stage_bytes;
    // The pages of this warp's next 32 tiles wait in registers, one a lane, so that the loop does
    // not stall on the block table: lane l holds the page of the warp's tile number base + l.
    int pages32 = -1;
    auto fetch_pages = [&](int base) {
        const int tile = warp + 4 * (base + lane);
        pages32 = -1;
        if (tile < n_tiles) {
            const int lp = max(k_begin + tile * AD_WK, klo) / p.page_size;     // by a position the block owns
            if (lp < p.table_width) pages32 = p.block_table[(size_t)x.entry * p.table_width + lp];
            if (pages32 >= p.n_pages) pages32 = -1;
        }
    };
    auto load_tile = [&](int stage, int i) {                 // the warp's tile number i
        const int j = k_begin + (warp + 4 * i) * AD_WK;
        const int page = __shfl_sync(0xffffffffu, pages32, i & 31);
        const uint32_t dst = my_pipe + (uint32_t)stage * stage_bytes;
        if (page >= 0) {
            const int row = (page * p.hkv + kvh) * p.page_size + j % p.page_size;
            if (lane == 0) am_mbar_expect_tx(bars + stage, tile_bytes);
            __syncwarp();                                   // the expectation is set before a copy can complete
            if (lane < nbox) am_tma_box(dst + lane * 2048u, &map_k, lane * 64, row, bars + stage);
            else if (lane < 2 * nbox) am_tma_box(dst + lane * 2048u, &map_v, (lane - nbox) * 64, row, bars + stage);
        } else {
            uint4* z = reinterpret_cast<uint4*>(pipes_ptr + (size_t)(warp * AD_STAGES + stage) * stage_bytes);
            for (uint32_t k = lane; k < stage_bytes / 16; k += 32) z[k] = make_uint4(0u, 0u, 0u, 0u);
            __syncwarp();
            if (lane == 0) am_mbar_expect_tx(bars + stage, 0u);         // nothing to wait for: the phase completes
        }
    };
    const int chunks = d / 8;
    float* stg = reinterpret_cast<float*>(am_smem + p.stage_offset);       // FUSED: [slice][query heads of the kv head][d], then [slice][key, value][d]
    const int heads_all = p.hq + 2 * p.hkv;
    bool failed = false;
    float2 cs_q = make_float2(1.f, 0.f);                    // FUSED: this thread's pairs all have component tid mod d/2 (128 is a multiple of d/2)
    float2 cs_k[HD / 64];                                   // FUSED: the angles of the key's pairs lane, lane + 32, .. for the warp that owns the newest tile
    bool early[AD_STAGES];
    if (FUSED) {
        // This kernel's blocks fill a multiprocessor's shared memory: they start when the product's
        // blocks have left, so the wait is short, and it comes first. The queries' slices are then asked
        // for ahead of the 192 KB of keys and values, not behind them (behind them they landed 3.3 us
        // after the wait). A copy a thread, the copies dealt out to the four warps in turn: a request
        // keeps its thread, and with it its warp, for a while. (The barrier cannot complete before
        // thread 0 has arrived with the bytes to expect, whichever copy lands first.)
        dependent_wait();
        KB_TL_MARK(attention, 2, threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);
        dependent_trigger();
        if (tid == 0) am_mbar_expect_tx(qbar, (uint32_t)(p.qkv_splits * group * d) * 4u);
        {
            const int s = lane * 4 + warp;
            if (s < p.qkv_splits)
                am_bulk_copy(stg + (size_t)s * group * d, p.qkv_parts + (size_t)s * p.qkv_stride + ((size_t)row0 * heads_all + kvh * group) * d,
                             (uint32_t)(group * d) * 4u, qbar);
        }
        cs_q = p.cos_sin[(size_t)row0 * (d >> 1) + tid % (d >> 1)];        // on its way while the slices are
        fetch_pages(0);
#pragma unroll
        for (int s = 0; s < AD_STAGES; ++s) {
            early[s] = warp + 4 * s < n_tiles;
            if (early[s]) load_tile(s, s);
        }
    } else {
        fetch_pages(0);
        // The kernel before this one wrote the newest key of every row and nothing older: a first tile
        // that ends below the first row's last position is asked for ahead of the wait.
#pragma unroll
        for (int s = 0; s < AD_STAGES; ++s) {
            early[s] = warp + 4 * s < n_tiles && k_begin + (warp + 4 * s) * AD_WK + AD_WK < x.c_first;
            if (early[s]) load_tile(s, s);
        }
        dependent_wait();
        KB_TL_MARK(attention, 2, threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);
        dependent_trigger();
        for (int i = tid; i < 16 * chunks; i += AM_THREADS) {
            const int r = i / chunks, ch = i % chunks;
            const bool valid = r < rows_valid;
            const bf16* src = p.q + ((size_t)(row0 + (valid ? r / group : 0)) * p.hq + kvh * group + (valid ? r % group : 0)) * d + ch * 8;
            am_cp_async16(sQ + r * ld + ch * 8, src, valid);
        }
        am_commit();
    }
#pragma unroll
    for (int s = 0; s < AD_STAGES; ++s)
        if (!early[s] && warp + 4 * s < n_tiles) load_tile(s, s);
    // FUSED: which tile of this block's holds the row's own position, if any does and the layer writes its cache
    int t_new = -1, line_new = -1;
    if (FUSED) {
        const int half_d = d >> 1;
        const int newest = x.c_first - 1;
        if (p.k_new != nullptr && newest >= klo && newest < khi) {
            line_new = p.lines[row0];
            if (line_new >= 0 && line_new < p.table_lines) t_new = (newest - k_begin) / AD_WK;
        }
        for (int i = tid; i < (16 - group) * chunks; i += AM_THREADS)      // the rows no query head fills
            *reinterpret_cast<uint4*>(sQ + (group + i / chunks) * ld + (i % chunks) * 8) = make_uint4(0u, 0u, 0u, 0u);
        if (!am_mbar_wait(qbar, 0u)) failed = true;
        if (!failed)
            for (int i = tid; i < group * half_d; i += 2 * AM_THREADS) {    // two pairs at a time: four sums side by side
                const int c = i % half_d, h0 = i / half_d;
                const bool two = i + AM_THREADS < group * half_d;
                const int h1 = two ? (i + AM_THREADS) / half_d : h0;
                const float* v0 = stg + h0 * d + c;
                const float* v1 = stg + h1 * d + c;
                float a0 = v0[0], b0 = v0[half_d], a1 = v1[0], b1 = v1[half_d];
                for (int s = 1; s < p.qkv_splits; ++s) {
                    const size_t o = (size_t)s * group * d;
                    a0 += v0[o]; b0 += v0[o + half_d]; a1 += v1[o]; b1 += v1[o + half_d];
                }
                rope_rotate(a0, b0, cs_q);
                sQ[h0 * ld + c] = __float2bfloat16_rn(a0);
                sQ[h0 * ld + c + half_d] = __float2bfloat16_rn(b0);
                if (two) {
                    rope_rotate(a1, b1, cs_q);
                    sQ[h1 * ld + c] = __float2bfloat16_rn(a1);
                    sQ[h1 * ld + c + half_d] = __float2bfloat16_rn(b1);
                }
            }
    } else {
        am_wait<0>();                                       // this thread's part of Q has landed
    }
    __syncthreads();                                        // and everyone else's
    if (FUSED && t_new >= 0) {                              // everyone has read the queries' slices: the key's and the value's may land there
        if (tid == 0) am_mbar_expect_tx(kvbar, (uint32_t)(2 * p.qkv_splits * d) * 4u);
        for (int o = lane * 4 + warp; o < 2 * p.qkv_splits; o += 128) {      // dealt out to the four warps as above
            const int s = o >> 1, is_v = o & 1;
            am_bulk_copy(stg + (size_t)o * d, p.qkv_parts + (size_t)s * p.qkv_stride + ((size_t)row0 * heads_all + p.hq + (is_v ? p.hkv : 0) + kvh) * d,
                         (uint32_t)d * 4u, kvbar);
        }
        if (warp == (t_new & 3)) {                          // the warp that owns the newest tile will rotate the key
#pragma unroll
            for (int j = 0; j < HD / 64; ++j) cs_k[j] = p.cos_sin[(size_t)row0 * (d >> 1) + lane + 32 * j];
        }
    }

    // Q as B fragments: lane (g, t) holds Q[row 8 nb + g][dims 16 ks + 2t, +1 and + 8 + 2t, +1].
    uint32_t bq[HD / 16][NB][2];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            bq[ks][nb][0] = bq[ks][nb][1] = 0u;
            if (FULL || ks * 16 < d) {
                const bf16* qp = sQ + (nb * 8 + g) * ld + ks * 16 + t * 2;
                bq[ks][nb][0] = *reinterpret_cast<const uint32_t*>(qp);
                bq[ks][nb][1] = *reinterpret_cast<const uint32_t*>(qp + 8);
            }
        }
    float ot[HD / 16][NB][4];
#pragma unroll
    for (int nd = 0; nd < HD / 16; ++nd)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) ot[nd][nb][0] = ot[nd][nb][1] = ot[nd][nb][2] = ot[nd][nb][3] = 0.f;
    float m_run[NB][2], l_run[NB][2];
    int cnt[NB][2], fst[NB][2];
    int fst_max = 0, cnt_min = 0x7fffffff;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            m_run[nb][h] = -INFINITY;
            l_run[nb][h] = 0.f;
            const int r = nb * 8 + t * 2 + h;                // this lane's rows ("heads")
            const bool own = r < rows_valid;
            cnt[nb][h] = own ? x.c_first + r / group : 0x7fffffff;
            fst[nb][h] = (own && p.window > 0 && cnt[nb][h] > p.window) ? cnt[nb][h] - p.window : 0;
            fst_max = max(fst_max, fst[nb][h]);
            cnt_min = min(cnt_min, cnt[nb][h]);
        }
    const int fst_hi = __reduce_max_sync(0xffffffffu, fst_max);
    const int cnt_lo = __reduce_min_sync(0xffffffffu, cnt_min);
    const float sc = p.cap > 0.f ? p.scale / p.cap : p.scale;

    KB_TL_MARK(attention, 3, threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);          // the loop over the keys begins
    for (int i = 0; !failed && warp + 4 * i < n_tiles; ++i) {
        const int tile = warp + 4 * i, stage = i % AD_STAGES;
        if (!am_mbar_wait(bars + stage, (uint32_t)(i / AD_STAGES) & 1u)) { failed = true; break; }
        __syncwarp();                                       // zero rows written by other lanes are visible
        const uint32_t tk = my_pipe + (uint32_t)stage * stage_bytes;
        if (FUSED && tile == t_new) {
            // The row's own key and value: summed, the key rotated, rounded; to the cache's line, and over
            // what TMA brought of that line into this tile (element c of key kk: box c / 64, row kk, the
            // 16-byte piece (c % 64) / 8 exchanged by kk mod 8).
            if (!am_mbar_wait(kvbar, 0u)) { failed = true; break; }
            const int half_d = d >> 1, kk = (x.c_first - 1) & (AD_WK - 1);
            unsigned char* tile_k = pipes_ptr + (size_t)(warp * AD_STAGES + stage) * stage_bytes;
            unsigned char* tile_v = tile_k + nbox * 2048;
            auto at = [&](unsigned char* base, int c) -> bf16* {
                return reinterpret_cast<bf16*>(base + (c >> 6) * 2048 + kk * 128 + ((((c & 63) >> 3) ^ (kk & 7)) << 4)) + (c & 7);
            };
            const size_t dst_row = kv_row(line_new, kvh, p.hkv, p.page_size) * d;
            // One walk over the slices with every sum of this lane side by side (a walk a sum, each add
            // waiting for its load, took 2 to 2.8 us here, at the end of the block's longest warp).
            float ka[HD / 64], kb[HD / 64], vv[HD / 32];
#pragma unroll
            for (int j = 0; j < HD / 64; ++j) { ka[j] = stg[lane + 32 * j]; kb[j] = stg[lane + 32 * j + half_d]; }
#pragma unroll
            for (int j = 0; j < HD / 32; ++j) vv[j] = stg[d + lane + 32 * j];
            for (int s = 1; s < p.qkv_splits; ++s) {
                const float* ks = stg + (size_t)2 * s * d + lane;
#pragma unroll
                for (int j = 0; j < HD / 64; ++j) { ka[j] += ks[32 * j]; kb[j] += ks[32 * j + half_d]; }
#pragma unroll
                for (int j = 0; j < HD / 32; ++j) vv[j] += ks[d + 32 * j];
            }
#pragma unroll
            for (int j = 0; j < HD / 64; ++j) {
                const int c = lane + 32 * j;
                rope_rotate(ka[j], kb[j], cs_k[j]);
                const bf16 xa = __float2bfloat16_rn(ka[j]), xb = __float2bfloat16_rn(kb[j]);
                p.k_new[dst_row + c] = xa;
                p.k_new[dst_row + c + half_d] = xb;
                *at(tile_k, c) = xa;
                *at(tile_k, c + half_d) = xb;
            }
#pragma unroll
            for (int j = 0; j < HD / 32; ++j) {
                const int c = lane + 32 * j;
                const bf16 xv = __float2bfloat16_rn(vv[j]);
                p.v_new[dst_row + c] = xv;
                *at(tile_v, c) = xv;
            }
            __syncwarp();                                   // the tile is whole before any lane reads it
        }
        ad_tile<HD, NB, FULL>(bq, tk, tk + nbox * 2048u, d, k_begin + tile * AD_WK, cnt, fst, fst_hi, cnt_lo, klo, khi, sc, p.cap,
                              ot, m_run, l_run, lane);
        __syncwarp();                                       // every lane has read the stage
        if (tile + 4 * AD_STAGES < n_tiles) {
            if (((i + AD_STAGES) & 31) == 0) fetch_pages(i + AD_STAGES);
            load_tile(stage, i + AD_STAGES);
        }
    }
    if (failed) {
        // A copy never completed. Give the others in flight the same bounded chance to land (they
        // write into this block's shared memory), raise the flag, and leave without writing.
        for (int s = 0; s < AD_STAGES; ++s) am_mbar_wait(bars + s, 0u), am_mbar_wait(bars + s, 1u);
        if (FUSED) {
            am_mbar_wait(qbar, 0u);
            if (t_new >= 0 && warp == (t_new & 3)) am_mbar_wait(kvbar, 0u);
        }
        if (lane == 0) atomicExch(&g_attention_error, 1);
    }
    failed = __syncthreads_or(failed);
    if (failed) return;
    KB_TL_MARK(attention, 4, threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);          // and is done
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {                        // the row sums over the 16 key lanes
            l_run[nb][h] += __shfl_xor_sync(0xffffffffu, l_run[nb][h], 4);
            l_run[nb][h] += __shfl_xor_sync(0xffffffffu, l_run[nb][h], 8);
            l_run[nb][h] += __shfl_xor_sync(0xffffffffu, l_run[nb][h], 16);
        }

    // Merge the 4 warps' states through shared memory (the pipelines are drained).
    const float LOG2E = 1.4426950408889634f;
    const int md = d + 4;
    float* mO = reinterpret_cast<float*>(pipes_ptr);        // [4][16][md], over the drained pipelines
    float* mM = mO + 4 * 16 * md;                           // [4][16]
    float* mL = mM + 4 * 16;
#pragma unroll
    for (int nd = 0; nd < HD / 16; ++nd)
        if (FULL || nd * 16 < d) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = nb * 8 + t * 2 + (e & 1);
                    if (r < rows_valid) mO[((size_t)warp * 16 + r) * md + nd * 16 + g + (e >> 1) * 8] = ot[nd][nb][e];
                }
        }
    if (g == 0) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = nb * 8 + t * 2 + h;
                if (r < rows_valid) { mM[warp * 16 + r] = m_run[nb][h]; mL[warp * 16 + r] = l_run[nb][h]; }
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
            const float f = (mw == -INFINITY) ? 0.f : am_exp2((mw - mx) * LOG2E);
            acc = fmaf(f, mO[((size_t)w * 16 + r) * md + c], acc);
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
    KB_TL_LEAVE(attention, blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0, 0);
}

// out[row, head, :] = sum_z e^(m_z - M) acc_z / sum_z e^(m_z - M) l_z over the absolute slots the
// row's own keys fall in; a row that sees nothing gets zeros. One block a (row, head): its first
// warp turns the slots' maxima and sums into weights, then every thread adds up its components
// with independent loads.
__global__ void __launch_bounds__(128)
attention_mma_combine_kernel(const AttMmaParams p KB_TL_PARAM) {
    extern __shared__ float cw[];                           // [slots] weights
    const int row = blockIdx.x, head = blockIdx.y;
    KB_TL_ENTER(attention, blockIdx.x == 0 && blockIdx.y == 0, 5, p.slots, p.window);
    const int count = p.row_count[row];                     // copied in before the step began: read ahead of the wait
    dependent_wait();
    KB_TL_MARK(attention, 2, threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0);
    dependent_trigger();
    bf16* o = p.out + ((size_t)row * p.hq + head) * p.d;
    if (count <= 0) {
        for (int i = threadIdx.x; i < p.d; i += blockDim.x) o[i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int first = (p.window > 0 && count > p.window) ? count - p.window : 0;
    const int origin = p.relative ? first : 0;
    const int z0 = (first - origin) / p.split, z1 = min(p.slots - 1, (count - 1 - origin) / p.split);
    const int nz = z1 - z0 + 1;
    if (nz == 1 && p.direct) return;
    const int stride = p.d + 2;
    const float* base = p.partial + (((size_t)row * p.hq + head) * p.slots + z0) * stride;
    // The first sixteen slots' values are asked for before the weights are known: they do not depend
    // on them, and so the kernel is the count's trip to memory and one more, not four in a row. With
    // one key of history a block at batch 1 there are dozens of slots; the rest follow sixteen at a
    // time. The sums run in slot order either way.
    const int i0 = threadIdx.x * 2;                         // d and the stride are even
    const bool mine = i0 < p.d;
    float2 v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j)
        v[j] = (mine && j < nz) ? *reinterpret_cast<const float2*>(base + (size_t)j * stride + i0) : make_float2(0.f, 0.f);
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float mx = -INFINITY;
        float2 ml[4];                                       // (maximum, sum) of this lane's slots: up to 128 in registers
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int z = lane + 32 * j;
            ml[j] = z < nz ? *reinterpret_cast<const float2*>(base + (size_t)z * stride + p.d) : make_float2(-INFINITY, 0.f);
            mx = fmaxf(mx, ml[j].x);
        }
        for (int z = lane + 128; z < nz; z += 32) mx = fmaxf(mx, base[(size_t)z * stride + p.d]);
        mx = warp_max(mx);
        float denom = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int z = lane + 32 * j;
            if (z < nz) {
                const float w = (ml[j].x == -INFINITY) ? 0.f : __expf(ml[j].x - mx);
                cw[z] = w;
                denom += w * ml[j].y;
            }
        }
        for (int z = lane + 128; z < nz; z += 32) {
            const float m = base[(size_t)z * stride + p.d];
            const float w = (m == -INFINITY) ? 0.f : __expf(m - mx);
            cw[z] = w;
            denom += w * base[(size_t)z * stride + p.d + 1];
        }
        denom = warp_sum(denom);
        const float inv = denom > 0.f ? 1.f / denom : 0.f;
        for (int z = lane; z < nz; z += 32) cw[z] *= inv;
    }
    __syncthreads();
    for (int i = i0; i < p.d; i += blockDim.x * 2) {
        float a0 = 0.f, a1 = 0.f;
        int z = 0;
        if (i == i0) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (j < nz) { a0 = fmaf(cw[j], v[j].x, a0); a1 = fmaf(cw[j], v[j].y, a1); }
            z = min(nz, 16);
        }
        for (; z + 16 <= nz; z += 16) {
            float2 u[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) u[j] = *reinterpret_cast<const float2*>(base + (size_t)(z + j) * stride + i);
#pragma unroll
            for (int j = 0; j < 16; ++j) { a0 = fmaf(cw[z + j], u[j].x, a0); a1 = fmaf(cw[z + j], u[j].y, a1); }
        }
        for (; z + 4 <= nz; z += 4) {
            float2 u[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) u[j] = *reinterpret_cast<const float2*>(base + (size_t)(z + j) * stride + i);
#pragma unroll
            for (int j = 0; j < 4; ++j) { a0 = fmaf(cw[z + j], u[j].x, a0); a1 = fmaf(cw[z + j], u[j].y, a1); }
        }
        for (; z < nz; ++z) {
            const float2 u = *reinterpret_cast<const float2*>(base + (size_t)z * stride + i);
            a0 = fmaf(cw[z], u.x, a0);
            a1 = fmaf(cw[z], u.y, a1);
        }
        *reinterpret_cast<uint32_t*>(o + i) = am_pack(a0, a1);
    }
    KB_TL_LEAVE(attention, blockIdx.x == 0 && blockIdx.y == 0, 0);
}


// The same with the (row, head)'s slots brought into shared memory by one bulk copy instead of the
// threads' loads: what the attention kernel has just written arrives sooner that way (see
// add_rmsnorm_splits_bulk_kernel in norm.cu). The slots' rows are d + 2 floats, so their first byte
// is 8-byte aligned only: the copy starts at the 16-byte boundary at or before it and ends at the one
// at or after its end. The weights and the sums are computed as the kernel above computes them.
__global__ void __launch_bounds__(128)
attention_mma_combine_bulk_kernel(const AttMmaParams p KB_TL_PARAM) {
    extern __shared__ __align__(16) unsigned char cb_smem[];
    __shared__ __align__(8) uint64_t landed;
    const int row = blockIdx.x, head = blockIdx.y;
    KB_TL_ENTER(attention, blockIdx.x == 0 && blockIdx.y == 0, 5, p.slots, p.window);
    const int count = p.row_count[row];                     // copied in before the step began: read ahead of the wait
    if (threadIdx.x == 0) {
        am_mbar_init(&landed, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    dependent_wait();
    KB_TL_MARK(attention, 2, threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0);
    dependent_trigger();
    bf16* o = p.out + ((size_t)row * p.hq + head) * p.d;
    if (count <= 0) {
        for (int i = threadIdx.x; i < p.d; i += blockDim.x) o[i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int first = (p.window > 0 && count > p.window) ? count - p.window : 0;
    const int origin = p.relative ? first : 0;
    const int z0 = (first - origin) / p.split, z1 = min(p.slots - 1, (count - 1 - origin) / p.split);
    const int nz = z1 - z0 + 1;
    if (nz == 1 && p.direct) return;
    const int stride = p.d + 2;
    const size_t start = ((((size_t)row * p.hq + head) * p.slots + z0) * stride) * sizeof(float);
    const size_t from = start & ~(size_t)15;
    const uint32_t bytes = (uint32_t)((start + (size_t)nz * stride * sizeof(float) - from + 15) & ~(size_t)15);
    if (threadIdx.x == 0) {
        am_mbar_expect_tx(&landed, bytes);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(am_saddr(cb_smem)), "l"(reinterpret_cast<const unsigned char*>(p.partial) + from), "r"(bytes), "r"(am_saddr(&landed)) : "memory");
    }
    const bool ok = am_mbar_wait(&landed, 0u);
    if (!ok) {
        if (threadIdx.x == 0) atomicExch(&g_attention_error, 1);
        return;
    }
    const float* base = reinterpret_cast<const float*>(cb_smem + (start - from));
    float* cw = reinterpret_cast<float*>(cb_smem + (((size_t)p.slots * stride * sizeof(float) + 16 + 15) & ~(size_t)15));      // [slots] weights
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float mx = -INFINITY;
        for (int z = lane; z < nz; z += 32) mx = fmaxf(mx, base[(size_t)z * stride + p.d]);
        mx = warp_max(mx);
        float denom = 0.f;
        for (int z = lane; z < nz; z += 32) {
            const float m = base[(size_t)z * stride + p.d];
            const float w = (m == -INFINITY) ? 0.f : __expf(m - mx);
            cw[z] = w;
            denom += w * base[(size_t)z * stride + p.d + 1];
        }
        denom = warp_sum(denom);
        const float inv = denom > 0.f ? 1.f / denom : 0.f;
        for (int z = lane; z < nz; z += 32) cw[z] *= inv;
    }
    __syncthreads();
    for (int i = threadIdx.x * 2; i < p.d; i += blockDim.x * 2) {      // d and the stride are even
        float a0 = 0.f, a1 = 0.f;
        for (int z = 0; z < nz; ++z) {
            const float2 u = *reinterpret_cast<const float2*>(base + (size_t)z * stride + i);
            a0 = fmaf(cw[z], u.x, a0);
            a1 = fmaf(cw[z], u.y, a1);
        }
        *reinterpret_cast<uint32_t*>(o + i) = am_pack(a0, a1);
    }
    KB_TL_LEAVE(attention, blockIdx.x == 0 && blockIdx.y == 0, 0);
}

// Bytes of shared memory the kernel above takes for `slots` slots of head size d.
static size_t combine_bulk_smem(int slots, int d) {
    return (((size_t)slots * (d + 2) * sizeof(float) + 16 + 15) & ~(size_t)15) + (size_t)slots * sizeof(float);
}

// The same with one warp a (row, head), four to a block, for the tens of thousands of pairs of a
// prompt, where a block each would be bound by the rate at which blocks can be started.
constexpr int AC_WARPS = 4;
__global__ void __launch_bounds__(AC_WARPS * 32)
attention_mma_combine_warp_kernel(const AttMmaParams p) {
    extern __shared__ float cw_all[];                       // [AC_WARPS][slots] weights
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * AC_WARPS + warp;
    dependent_wait();
    dependent_trigger();
    if (pair >= (long long)p.rows * p.hq) return;
    const int row = (int)(pair / p.hq), head = (int)(pair % p.hq);
    float* cw = cw_all + warp * p.slots;
    const int count = p.row_count[row];
    bf16* o = p.out + ((size_t)row * p.hq + head) * p.d;
    if (count <= 0) {
        for (int i = lane; i < p.d; i += 32) o[i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int first = (p.window > 0 && count > p.window) ? count - p.window : 0;
    const int origin = p.relative ? first : 0;
    const int z0 = (first - origin) / p.split, z1 = min(p.slots - 1, (count - 1 - origin) / p.split);
    const int nz = z1 - z0 + 1;
    if (nz == 1 && p.direct) return;
    const int stride = p.d + 2;
    const float* base = p.partial + (((size_t)row * p.hq + head) * p.slots + z0) * stride;
    float mx = -INFINITY;
    for (int z = lane; z < nz; z += 32) mx = fmaxf(mx, base[(size_t)z * stride + p.d]);
    mx = warp_max(mx);
    float denom = 0.f;
    for (int z = lane; z < nz; z += 32) {
        const float m = base[(size_t)z * stride + p.d];
        const float w = (m == -INFINITY) ? 0.f : __expf(m - mx);
        cw[z] = w;
        denom += w * base[(size_t)z * stride + p.d + 1];
    }
    denom = warp_sum(denom);
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    __syncwarp();
    for (int i = lane * 2; i < p.d; i += 64) {              // d and the stride are even
        float a0 = 0.f, a1 = 0.f;
#pragma unroll 4
        for (int z = 0; z < nz; ++z) {
            const float2 v = *reinterpret_cast<const float2*>(base + (size_t)z * stride + i);
            a0 = fmaf(cw[z], v.x, a0);
            a1 = fmaf(cw[z], v.y, a1);
        }
        *reinterpret_cast<uint32_t*>(o + i) = am_pack(a0 * inv, a1 * inv);
    }
}

// The merge kernel's weights: beyond 48 KB of shared memory the kernel has to be told.
static int combine_smem(int slots) {
    const size_t bytes = (size_t)AC_WARPS * slots * sizeof(float);
    if (bytes <= 48 * 1024) return 0;
    const cudaError_t e = cudaFuncSetAttribute(attention_mma_combine_warp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return fail("attention merge: %d slots need %zu bytes of shared memory: %s", slots, bytes, cudaGetErrorString(e));
    return 0;
}

template <int HD>
static int launch_prompt(const AttMmaParams& p, int tiles, cudaStream_t s) {
    if (p.page_size % 16 != 0) return fail("attention_mma: pages must hold a multiple of 16 positions, got %d", p.page_size);
    const int ld = p.d + AM_PAD;
    const int nbox = (p.d + 63) / 64;
    const size_t smem = (size_t)AP_ROWS * ld * sizeof(bf16) + 2048 + 2 * (size_t)8 * nbox * 2048 + 2 * sizeof(uint64_t) + 8 * sizeof(int) + 16;
    if (smem > 225 * 1024) return fail("attention_mma: head_dim %d needs %zu bytes of shared memory", p.d, smem);
    const unsigned long long rows = (unsigned long long)p.n_pages * p.hkv * p.page_size;
    CUtensorMap map_k, map_v;
    if (int e = encode_map_bf16(&map_k, p.k_table, rows, p.d, p.d, 16)) return e;
    if (int e = encode_map_bf16(&map_v, p.v_table, rows, p.d, p.d, 16)) return e;
    if (tiles > 65535 || p.slots > 65535) return fail("attention_mma: %d tiles in %d slots is too many for one launch", tiles, p.slots);
    dim3 grid(p.hkv, p.slots, tiles);
    if (p.d == HD) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_mma_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_mma_kernel<HD, true><<<grid, AP_THREADS, smem, s>>>(p, map_k, map_v);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_mma_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_mma_kernel<HD, false><<<grid, AP_THREADS, smem, s>>>(p, map_k, map_v);
    }
    return check_launch("attention_mma");
}

// max_rows: the most rows ((token, query head) pairs) any tile holds: up to 8 take one block of
// eight "heads" in the MMAs' N, up to 16 two. The tensor maps cover the whole key and value tables
// as [pages * kv heads * page size, head_dim] matrices.
// Bytes of shared memory the decode kernel wants: Q, the four warps' pipelines (or the merge of their
// states over them), the barriers, and for the kernel that takes the q|k|v product's slices the place
// they land in (`stage_bytes`). `bars` gets the barriers' offset, `stage` the slices'.
static size_t decode_smem(int d, size_t stage_bytes, size_t* bars_at, size_t* stage_at) {
    const int ld = d + AM_PAD;
    const int nbox = (d + 63) / 64;
    const size_t stage = (size_t)2 * nbox * 2048;
    const size_t pipes = (size_t)4 * AD_STAGES * stage;
    const size_t merge = ((size_t)4 * 16 * (d + 4) + 2 * 4 * 16) * sizeof(float);
    // Q, then up to 1023 bytes to reach the swizzle's period plus whatever the base itself is off by
    size_t bars = (size_t)16 * ld * sizeof(bf16) + 2048 + (pipes > merge ? pipes : merge);
    bars = (bars + 15) / 16 * 16;
    size_t at = bars + (4 * AD_STAGES + 2) * sizeof(uint64_t);
    at = (at + 127) / 128 * 128;
    if (bars_at) *bars_at = bars;
    if (stage_at) *stage_at = at;
    return stage_bytes ? at + stage_bytes : bars + (4 * AD_STAGES + 2) * sizeof(uint64_t);
}
static size_t fused_stage_bytes(int hq, int hkv, int d, int splits) {
    const int group = hq / hkv;
    return (size_t)splits * (group > 2 ? group : 2) * d * sizeof(float);    // the queries' slices, then the key's and the value's
}

// max_rows: the most rows ((token, query head) pairs) any tile holds: up to 8 take one block of
// eight "heads" in the MMAs' N, up to 16 two. The tensor maps cover the whole key and value tables
// as [pages * kv heads * page size, head_dim] matrices.
template <int HD>
static int launch_decode(const AttMmaParams& p, int tiles, int max_rows, cudaStream_t s) {
    if (p.page_size % AD_WK != 0) return fail("attention_mma: decode mode needs pages of a multiple of %d positions, got %d", AD_WK, p.page_size);
    const bool fused = p.qkv_parts != nullptr;
    size_t bars, stage_at;
    const size_t smem = decode_smem(p.d, fused ? fused_stage_bytes(p.hq, p.hkv, p.d, p.qkv_splits) : 0, &bars, &stage_at);
    if (smem > (fused ? 227 : 220) * 1024) return fail("attention_mma: head_dim %d needs %zu bytes of shared memory", p.d, smem);
    if (fused && p.d != HD) return fail("attention_mma: the kernel that takes the q|k|v product's slices is built for head sizes 64, 128 and 256, not %d", p.d);
    AttMmaParams q = p;
    q.decode_bar_offset = (int)bars;
    q.stage_offset = (int)stage_at;
    const unsigned long long rows = (unsigned long long)p.n_pages * p.hkv * p.page_size;
    CUtensorMap map_k, map_v;
    if (int e = encode_map_bf16(&map_k, p.k_table, rows, p.d, p.d, AD_WK)) return e;
    if (int e = encode_map_bf16(&map_v, p.v_table, rows, p.d, p.d, AD_WK)) return e;
    dim3 grid(tiles, p.hkv, p.slots);
#define KB_DECODE(NB, FULL, FUSED)                                                                                             \
    do {                                                                                                                       \
        if (smem > 48 * 1024)                                                                                                  \
            cudaFuncSetAttribute(attention_decode_kernel<HD, NB, FULL, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_dependent_if(p.rows <= DEPENDENT_ROWS, attention_decode_kernel<HD, NB, FULL, FUSED>, grid, dim3(AM_THREADS), (size_t)smem, s, q, map_k, map_v KB_TL_SLOT(attention, 4, q.slots, q.window));     \
    } while (0)
    if (fused) { if (max_rows <= 8) KB_DECODE(1, true, true); else KB_DECODE(2, true, true); }
    else if (max_rows <= 8) { if (p.d == HD) KB_DECODE(1, true, false); else KB_DECODE(1, false, false); }
    else                    { if (p.d == HD) KB_DECODE(2, true, false); else KB_DECODE(2, false, false); }
#undef KB_DECODE
    return check_launch("attention_decode");
}

}  // namespace kb

using namespace kb;

KB_TIMELINE_GETTER(attention)


// Rows a tile may hold in each mode; the host cuts requests into tiles of rows / group tokens.
extern "C" int kb_attention_mma_rows(int decode) { return decode ? 16 : AP_ROWS; }

// 1 if a wait inside an attention kernel ever ran out (and clears the flag); synchronises the device.
extern "C" int kb_attention_error() {
    int flag = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&flag, g_attention_error, sizeof(int)) != cudaSuccess) return -1;
    if (flag) cudaMemcpyToSymbol(g_attention_error, &zero, sizeof(int));
    return flag;
}

extern "C" long long kb_attention_mma_scratch_floats(int rows, int hq, int d, int slots) {
    // four more than the partial sums take: the merge's bulk copy of a (row, head)'s slots starts and ends on
    // 16-byte boundaries, up to 8 bytes beyond either end of what it wants
    return slots > 1 ? (long long)rows * hq * slots * (d + 2) + 4 : 0;
}

// Merges the partial sums [rows, hq, slots, d + 2] that a prompt kernel left in `scratch`; rows whose
// keys all lie in one slot were finished by that slot's block and are left alone.
extern "C" int kb_attention_mma_combine(void* out, const int* row_count, const float* scratch, int rows, int hq, int d,
                                        int window, int split, int slots, void* stream) {
    KB_REQUIRE(rows >= 0 && hq > 0 && d > 0 && d % 2 == 0, "attention combine: rows %d, heads %d, head_dim %d", rows, hq, d);
    KB_REQUIRE(split > 0 && slots > 1 && scratch != nullptr, "attention combine: split %d, %d slots", split, slots);
    if (rows == 0) return 0;
    AttMmaParams p = {};
    p.row_count = row_count; p.out = (bf16*)out; p.partial = const_cast<float*>(scratch);
    p.rows = rows; p.hq = hq; p.d = d; p.window = window; p.split = split; p.slots = slots; p.direct = 1;
    const unsigned blocks = (unsigned)(((long long)rows * hq + AC_WARPS - 1) / AC_WARPS);
    if (int e = combine_smem(slots)) return e;
    attention_mma_combine_warp_kernel<<<blocks, AC_WARPS * 32, (size_t)AC_WARPS * slots * sizeof(float), (cudaStream_t)stream>>>(p);
    return check_launch("attention_mma combine");
}

// The launches of a filled-in AttMmaParams: the kernel of the mode, then the merge of the key slots.
static int attention_mma_run(const AttMmaParams& p, int tiles, int decode, float* scratch, void* stream) {
    const int rows = p.rows, hq = p.hq, d = p.d, slots = p.slots;
    cudaStream_t s = (cudaStream_t)stream;
    int e;
    if (d <= 64) e = decode ? launch_decode<64>(p, tiles, decode, s) : launch_prompt<64>(p, tiles, s);
    else if (d <= 128) e = decode ? launch_decode<128>(p, tiles, decode, s) : launch_prompt<128>(p, tiles, s);
    else e = decode ? launch_decode<256>(p, tiles, decode, s) : launch_prompt<256>(p, tiles, s);
    if (e) return e;
    if (slots > 1) {
        if ((long long)rows * hq >= 4096) {                 // many pairs: a warp each
            const unsigned blocks = (unsigned)(((long long)rows * hq + AC_WARPS - 1) / AC_WARPS);
            if (int e2 = combine_smem(slots)) return e2;
            launch_dependent_if(false, attention_mma_combine_warp_kernel, dim3(blocks), dim3(AC_WARPS * 32), (size_t)AC_WARPS * slots * sizeof(float), s, p);
        } else if (slots > 8 && combine_bulk_smem(slots, d) <= 40 * 1024 && ((uintptr_t)scratch & 15) == 0) {
            // few (a decode step): a block each, for the latency; many slots (a small batch): brought in by a
            // bulk copy (28 slots: 2.9 us against 3.7), a few slots by the threads' loads (4 slots: 2.2 us against 2.9)
            launch_dependent_if(rows <= DEPENDENT_ROWS, attention_mma_combine_bulk_kernel, dim3(rows, hq), dim3(128), combine_bulk_smem(slots, d), s, p KB_TL_SLOT(attention, 5, p.slots, p.window));
        } else {                                            // more slots than fit shared memory: the threads load them
            launch_dependent_if(rows <= DEPENDENT_ROWS, attention_mma_combine_kernel, dim3(rows, hq), dim3(128), (size_t)slots * sizeof(float), s, p KB_TL_SLOT(attention, 5, p.slots, p.window));
        }
        return check_launch("attention_mma combine");
    }
    return 0;
}

extern "C" int kb_attention_mma(void* out, const void* q, const void* k_table, const void* v_table,
                                const int* block_table, const int* row_count, const int* tile_entry,
                                const int* tile_row0, const int* tile_nq, int tiles, int rows, int hq, int hkv, int d,
                                int page_size, int table_width, int n_pages, int window, int split, int slots,
                                float scale, float cap, int decode, int relative, float* scratch, void* stream) {
    // decode: 0 for prompt portions; else the most rows (tokens x query heads of a kv head) any tile
    // holds, at most 16.
    KB_REQUIRE(rows >= 0 && tiles >= 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "attention_mma: rows %d, tiles %d, heads %d over %d", rows, tiles, hq, hkv);
    KB_REQUIRE(d > 0 && d % 16 == 0 && d <= 256, "attention_mma: head_dim %d must be a multiple of 16, at most 256", d);
    KB_REQUIRE(hq / hkv <= (decode ? 16 : AP_ROWS), "attention_mma: %d query heads a kv head do not fit a tile of %d rows", hq / hkv, decode ? 16 : AP_ROWS);
    KB_REQUIRE(decode >= 0 && decode <= 16 && (decode == 0 || decode >= hq / hkv), "attention_mma: decode mode with %d rows a tile (1..16, at least the group of %d)", decode, hq / hkv);
    KB_REQUIRE(page_size > 0 && table_width > 0 && n_pages > 0, "attention_mma: page_size %d, table width %d, pages %d", page_size, table_width, n_pages);
    KB_REQUIRE(window >= 0 && cap >= 0.f, "attention_mma: window %d, cap %g", window, cap);
    KB_REQUIRE((split == 0 && slots == 1) || (split > 0 && split % AM_KT == 0 && slots >= 1 && slots <= 8192),
               "attention_mma: split %d (a multiple of %d) with %d slots (at most 8192)", split, AM_KT, slots);
    KB_REQUIRE(!(decode && split == 0 && slots != 1), "attention_mma: decode mode without a split has one slot");
    KB_REQUIRE(slots == 1 || scratch != nullptr, "attention_mma: %d slots need scratch memory", slots);
    KB_REQUIRE(relative == 0 || relative == 1, "attention_mma: relative %d (0 or 1: slots counted from each tile's first visible key, for tiles of one token)", relative);
    KB_REQUIRE(!(decode && relative) || tiles == rows, "attention_mma: relative with %d tiles for %d rows (every request brings one token: tile t is row t of request t)", tiles, rows);
    KB_REQUIRE(hkv <= 65535, "attention_mma: %d kv heads is too many for one launch", hkv);
    if (rows == 0 || tiles == 0) return 0;
    AttMmaParams p;
    p.q = (const bf16*)q; p.k_table = (const bf16*)k_table; p.v_table = (const bf16*)v_table;
    p.block_table = block_table; p.row_count = row_count; p.tile_entry = tile_entry; p.tile_row0 = tile_row0;
    p.tile_nq = tile_nq; p.out = (bf16*)out; p.partial = slots > 1 ? scratch : nullptr;
    p.rows = rows; p.hq = hq; p.hkv = hkv; p.d = d; p.page_size = page_size; p.table_width = table_width;
    p.n_pages = n_pages; p.window = window; p.split = split; p.slots = slots; p.scale = scale; p.cap = cap;
    p.decode_bar_offset = 0;
    p.direct = decode ? 0 : 1;
    p.relative = (decode && relative) ? 1 : 0;
    p.qkv_parts = nullptr; p.qkv_stride = 0; p.qkv_splits = 0; p.stage_offset = 0; p.cos_sin = nullptr; p.lines = nullptr;
    p.k_new = p.v_new = nullptr; p.table_lines = 0;
    return attention_mma_run(p, tiles, decode, scratch, stream);
}

// Whether kb_attention_decode_fused takes these sizes (else: kb_rope_append, then kb_attention_mma).
extern "C" int kb_attention_decode_fused_takes(int hq, int hkv, int d, int page_size, int splits) {
    if (hq <= 0 || hkv <= 0 || hq % hkv != 0 || hq / hkv > 16 || splits < 1) return 0;
    if (d != 64 && d != 128 && d != 256) return 0;
    if (page_size <= 0 || page_size % AD_WK != 0) return 0;
    return decode_smem(d, fused_stage_bytes(hq, hkv, d, splits), nullptr, nullptr) <= 227 * 1024 ? 1 : 0;
}

// A decode step in which every request brings one token, from the stacked q|k|v product's partial sums
// (qkv_parts: f32 [splits][rows][(hq + 2 hkv) d], slices qkv_stride floats apart): rotation of the
// whole head by cos_sin ([rows][d / 2]), the newest key and value to the tables at lines[row] when
// write_kv is set, and attention over the cache as kb_attention_mma does it in decode mode with
// `relative` set. Row r is request r (block_table's row r).
extern "C" int kb_attention_decode_fused(void* out, const float* qkv_parts, int splits, long long qkv_stride, const void* cos_sin,
                                         const int* lines, void* k_table, void* v_table, int write_kv, long long table_lines,
                                         const int* block_table, const int* row_count, int rows, int hq, int hkv, int d,
                                         int page_size, int table_width, int n_pages, int window, int split, int slots,
                                         float scale, float cap, float* scratch, void* stream) {
    KB_REQUIRE(rows >= 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "attention_decode_fused: rows %d, heads %d over %d", rows, hq, hkv);
    KB_REQUIRE(kb_attention_decode_fused_takes(hq, hkv, d, page_size, splits), "attention_decode_fused: heads %d over %d of size %d, pages of %d, %d slices: not taken (head sizes 64, 128, 256; at most 16 query heads a kv head; the slices must fit shared memory)", hq, hkv, d, page_size, splits);
    KB_REQUIRE(qkv_parts != nullptr && cos_sin != nullptr && lines != nullptr, "attention_decode_fused: a null input");
    KB_REQUIRE(((uintptr_t)qkv_parts & 15) == 0 && (qkv_stride * 4) % 16 == 0, "attention_decode_fused: the slices must start at multiples of 16 bytes");
    KB_REQUIRE(table_width > 0 && n_pages > 0, "attention_decode_fused: table width %d, pages %d", table_width, n_pages);
    KB_REQUIRE(window >= 0 && cap >= 0.f, "attention_decode_fused: window %d, cap %g", window, cap);
    KB_REQUIRE((split == 0 && slots == 1) || (split > 0 && split % AM_KT == 0 && slots >= 1 && slots <= 8192),
               "attention_decode_fused: split %d (a multiple of %d) with %d slots (at most 8192)", split, AM_KT, slots);
    KB_REQUIRE(slots == 1 || scratch != nullptr, "attention_decode_fused: %d slots need scratch memory", slots);
    KB_REQUIRE(hkv <= 65535, "attention_decode_fused: %d kv heads is too many for one launch", hkv);
    if (rows == 0) return 0;
    AttMmaParams p;
    p.q = nullptr; p.k_table = (const bf16*)k_table; p.v_table = (const bf16*)v_table;
    p.block_table = block_table; p.row_count = row_count; p.tile_entry = nullptr; p.tile_row0 = nullptr;
    p.tile_nq = nullptr; p.out = (bf16*)out; p.partial = slots > 1 ? scratch : nullptr;
    p.rows = rows; p.hq = hq; p.hkv = hkv; p.d = d; p.page_size = page_size; p.table_width = table_width;
    p.n_pages = n_pages; p.window = window; p.split = split; p.slots = slots; p.scale = scale; p.cap = cap;
    p.decode_bar_offset = 0;
    p.direct = 0;
    p.relative = 1;
    p.qkv_parts = qkv_parts; p.qkv_stride = qkv_stride; p.qkv_splits = splits; p.stage_offset = 0;
    p.cos_sin = (const float2*)cos_sin; p.lines = lines;
    p.k_new = write_kv ? (bf16*)k_table : nullptr; p.v_new = write_kv ? (bf16*)v_table : nullptr;
    p.table_lines = table_lines;
    return attention_mma_run(p, rows, hq / hkv, scratch, stream);
}
