// Paged attention for prompt portions on the fifth-generation tensor cores (bfloat16, soft cap).
//
// One block takes a tile of 128 rows — (token, query head) pairs of one kv head, the same tiles as
// the mma.sync kernel — and walks its keys 64 at a time:
//   S = Q K^T      tcgen05.mma with Q [128 x d] as the A operand from tensor memory (TMEM), where
//                  it is put once (read from shared memory, Q would cost every product 4 KB), the
//                  key tile [64 x d] K-major in shared memory (128-byte swizzle), S [128 x 64]
//                  float32 in TMEM;
//   P = exp(cap tanh(S scale / cap)), masked, read from TMEM and written back over S as bfloat16
//                  by four warps, one row a thread;
//   O += P V       tcgen05.mma with P as the A operand straight from TMEM and the value tile
//                  [64 x d] as an MN-major B operand; O [128 x d] float32 stays in TMEM throughout.
// TMEM columns: O (d), two S buffers (64 each; P lies over the first 32 columns of its S), Q (d / 2).
// Issuing a tcgen05.mma keeps its thread busy for 50 to 100 cycles whatever the product's size (one
// thread issuing 128 x 64 x 16 products gets a third of the tensor cores' rate, two threads issuing
// side by side get two thirds), so the score products and the P V products have a thread each, in
// warps of their own. The scores of tile kt + 2 may land on their buffer only when the product that
// read tile kt's P from it is complete: that product's commit tells the score thread.
// Keys and values arrive by TMA in two rings of slots, one for key tiles and one for value tiles,
// each slot freed by the tcgen05.commit of the product that read it. A product costs the tensor
// cores about 50 cycles beyond its arithmetic, so the scores take all 64 keys in one product a
// 16-element step: the key tile is laid out [chunk of 64 elements][64 keys], boxes of 16 keys x 64
// elements, one a (page, chunk). The values, whose products step through the keys 16 at a time,
// come as one three-dimensional copy a page: [page][chunk][16 keys]. S and P are double-buffered so
// the exponentials of one tile run under the products of its neighbours.
//
// The soft cap bounds every score by +-cap, so exp(s) itself is safe in float32 and bfloat16 for
// cap <= 64 (e^64 times 2^17 keys < 3e38, e^-64 > 1e-38): the softmax uses the fixed reference 0
// instead of a running maximum, and O never has to be rescaled. Without a soft cap, with a larger
// cap, or with a head size other than 64, 128 or 256 the mma.sync kernel runs instead.
//
// Thirteen warps: warps 0, 12 and 11 find pages and ask TMA for the boxes of keys (half a tile each)
// and of values; warp 1 allocates TMEM and one lane issues the score products; warps 2-9 are the softmax and the epilogue, two warps to each quarter of the
// rows (a warp reads the 32 TMEM lanes of its number modulo 4), one for the first 32 keys of a tile
// and one for the last (two special-function operations an element keep a lone warp waiting); one
// lane of warp 10 issues the P V products. Every wait on an mbarrier gives up after about a second,
// raises a flag that `kb_attention_tc_error` reports, and the block still meets at its final
// barrier, frees its TMEM and returns.
#include "common.cuh"
#include "tensor_map.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

constexpr int AT_ROWS = 128, AT_KEYS = 64, AT_THREADS = 416;
constexpr int AT_WARP_PV = 10;          // the warp that issues the P V products (warp 1 issues the scores)
constexpr int AT_WARP_V = 11;           // the warp that asks for the values (warp 0 asks for the keys)
constexpr int AT_WARP_K2 = 12;          // the single-block kernel's second warp for keys: warp 0 asks for keys 0-31 of a tile, it for 32-63

__device__ int g_attention_tc_error = 0;

struct AttTcParams {
    const bf16* q;             // [rows, hq, d]
    const int* block_table;    // [entries, table_width]
    const int* row_count;      // [rows]
    const int* tile_entry;     // [tiles]
    const int* tile_row0;      // [tiles] first row (token) of the tile in the batch
    const int* tile_nq;        // [tiles] tokens in the tile
    bf16* out;                 // [rows, hq, d]
    float* partial;            // [rows, hq, slots, d + 2] when slots > 1: (sum p v, reference 0, sum p)
    int rows, hq, hkv, d, page_size, table_width, n_pages;
    int window, split, slots;
    float scale, cap;
};

__device__ __forceinline__ uint32_t at_saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(at_saddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void at_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(at_saddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(at_saddr(bar)) : "memory");
}
// false if the phase with this parity did not complete within ~1 s
__device__ __forceinline__ bool at_mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = at_saddr(bar);
    const long long start = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if (clock64() - start > 2000000000ll) return false;
    }
}
__device__ __forceinline__ void at_tma_box(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(at_saddr(bar)), "r"(x), "r"(y) : "memory");
}
// the 16 rows from `row` on, all chunks
__device__ __forceinline__ void at_tma_page(uint32_t dst, const CUtensorMap* map, int row, uint64_t* bar) {
    const int zero = 0;
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %3}], [%2];"
                 ::"r"(dst), "l"(map), "r"(at_saddr(bar)), "r"(zero), "r"(row) : "memory");
}
__device__ __forceinline__ void at_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_saddr(bar)) : "memory");
}
__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptors, 128-byte swizzle (layout type 2 at bit 61, version 1 at bit 46).
// K-major (Q, keys): rows of 128 bytes, eight-row groups `stride` bytes apart; the leading offset
// is not used. MN-major (values, [key][element]): blocks of 64 elements `lead` bytes apart along
// N, eight-key groups `stride` bytes apart along K.
__device__ __forceinline__ uint64_t at_desc(uint32_t saddr, uint32_t lead, uint32_t stride) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)((lead >> 4) & 0x3FFFu) << 16) | ((uint64_t)((stride >> 4) & 0x3FFFu) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: D float32 (bit 4), A and B bfloat16 (bits 7, 10), A K-major,
// B K-major or MN-major (bit 16), N / 8 at [17,23), M / 16 at [24,29).
__host__ __device__ constexpr uint32_t at_idesc(int m, int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void at_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void at_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void at_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void at_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ float at_tanh(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 2^x on the FMA and integer pipes, for |x| < 126: x = n + f with n the nearest integer (the magic
// constant's addition rounds it into the low bits), 2^f by a polynomial on [-1/2, 1/2] (relative error
// below 6e-5, far below bfloat16's 4e-3), 2^n added to the exponent. The special-function unit makes 16
// results a clock a multiprocessor and the softmax needs two an element (tanh and exp): half of the
// exponentials are computed this way so that both pipes work.
__device__ __forceinline__ float at_exp2_poly(float x) {
    const float t = x + 12582912.f;                              // 1.5 * 2^23: the integer part lands in the mantissa
    const float f = x - (t - 12582912.f);
    float p = fmaf(f, 0.0096181291f, 0.0555041087f);
    p = fmaf(p, f, 0.2402265070f);
    p = fmaf(p, f, 0.6931471806f);
    p = fmaf(p, f, 1.0f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
__device__ __forceinline__ uint32_t at_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Slots of the key/value ring and TMEM columns by head size.
template <int HD> struct AtCfg {
    static constexpr int NBOX = HD / 64;                        // boxes of 64 elements along the head
    static constexpr int SLOT_BYTES = AT_KEYS * HD * 2;         // a key tile or a value tile
    // Keys and values have rings of their own: a key slot is free as soon as its scores are
    // complete, two tiles before the next key tile is needed in it, and a value slot when its
    // product is, so both are loaded two tiles ahead.
    static constexpr int K_SLOTS = HD == 256 ? 3 : (HD == 128 ? 5 : 3);
    static constexpr int V_SLOTS = HD == 256 ? 4 : (HD == 128 ? 8 : 5);
    static constexpr int SLOTS = K_SLOTS + V_SLOTS;
    static constexpr int COL_O = 0, COL_S = HD, COL_Q = HD + 2 * AT_KEYS;
    static constexpr int TMEM_COLS = HD == 64 ? 256 : 512;      // 3 HD / 2 + 128 rounded up to a power of two
    static constexpr int SMEM = SLOTS * SLOT_BYTES + 1024 /* alignment */ + 320 /* barriers */ + 512 /* row sums */;
    static_assert((2 * SLOTS + 7) * 8 + 8 <= 320, "the barriers outgrew their room");
    static_assert(SMEM <= 232448, "more shared memory than a block can have");
};

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tc_kernel(const AttTcParams p, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
    using C = AtCfg<HD>;
    constexpr int NBOX = C::NBOX, NS = C::SLOTS, KS = C::K_SLOTS, VS = C::V_SLOTS;
    extern __shared__ unsigned char at_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)at_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* ring = smem;
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + NS * C::SLOT_BYTES);    // [NS] a slot's boxes have landed
    uint64_t* empty = full + NS;                                 // [NS] the product that read a slot is complete
    uint64_t* s_full = empty + NS;                               // [2] S complete (score products -> softmax)
    uint64_t* p_full = s_full + 2;                               // [2] P written (softmax -> P V products), eight warps arrive
    uint64_t* s_free = p_full + 2;                               // [2] the product that read P is complete: S may be written again
    uint64_t* o_full = s_free + 2;                               // [1] O complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
    float* l_half = reinterpret_cast<float*>(ring + NS * C::SLOT_BYTES + 320);   // [128] sum p over the last 32 keys of every tile, by row

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x, slot = blockIdx.y;
    // Later tiles of a prompt see more keys: they start first, all their heads and slots together.
    const int tile = gridDim.z - 1 - blockIdx.z;
    const int group = p.hq / p.hkv;
    const int row0 = p.tile_row0[tile], nq = p.tile_nq[tile];
    const int entry = p.tile_entry[tile];
    const int rows_valid = nq * group;
    const int c_first = p.row_count[row0];
    int klo = (p.window > 0 && c_first > p.window) ? c_first - p.window : 0;
    int khi = c_first > 0 ? c_first + nq - 1 : 0;                // a padding row sees nothing
    if (p.split > 0) {
        klo = max(klo, slot * p.split);
        khi = min(khi, (slot + 1) * p.split);
    }
    const int d = HD;
    if (klo >= khi) {                                            // nothing for this block: before anything is allocated
        dependent_wait();
        if (p.slots == 1 && c_first <= 0)
            for (int i = tid; i < rows_valid * d; i += AT_THREADS) {
                const int r = i / d, c = i % d;
                p.out[((size_t)(row0 + r / group) * p.hq + kvh * group + r % group) * d + c] = __float2bfloat16_rn(0.f);
            }
        return;
    }
    const int k_begin = klo / AT_KEYS * AT_KEYS;
    const int n_tiles = (khi - k_begin + AT_KEYS - 1) / AT_KEYS;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) { at_mbar_init(full + s, s < KS ? 2 : 1); at_mbar_init(empty + s, 1); }   // two warps bring a key tile
        for (int b = 0; b < 2; ++b) { at_mbar_init(s_full + b, 1); at_mbar_init(p_full + b, 8); at_mbar_init(s_free + b, 1); }
        at_mbar_init(o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_saddr(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    at_fence_before();
    __syncthreads();
    at_fence_after();
    const uint32_t tmem = *tmem_slot;
    dependent_wait();                                       // the queries and the newest keys are the kernel before's
    // Q into TMEM as the A operand of the score products: row r in lane r, two elements a column. The
    // two warps of a quarter of the rows take half of the head each.
    if (warp >= 2 && warp < 10) {
        const int r = (warp & 3) * 32 + lane;
        const int half = (warp - 2) >> 2;                        // 0: the head's first half, 1: its second
        const bf16* src = p.q + ((size_t)(row0 + (r < rows_valid ? r / group : 0)) * p.hq + kvh * group + (r < rows_valid ? r % group : 0)) * d;
        if (HD >= 128) {
            for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 64) {
                uint32_t w[32];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (r < rows_valid) v = *reinterpret_cast<const uint4*>(src + c0 + j * 8);
                    w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
                }
                at_st32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(C::COL_Q + c0 / 2), w);
            }
        } else if (half == 0) {                                  // 64 elements: one store, by the quarter's first warp
            uint32_t w[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (r < rows_valid) v = *reinterpret_cast<const uint4*>(src + j * 8);
                w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
            }
            at_st32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)C::COL_Q, w);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    // The score warp must see Q in place (the softmax warps and it meet here); the copying warp and
    // the P V warp need not, and go ahead.
    at_fence_before();
    if (warp >= 1 && warp < 10) asm volatile("bar.sync 1, 288;" ::: "memory");
    at_fence_after();
    bool failed = false;

    if (warp == 0 || warp == AT_WARP_V || warp == AT_WARP_K2) {
        // ---------------------------------------------------------------- pages and boxes
        // Asking TMA for a box keeps the asking warp busy for more than a hundred clocks (a tile's 16
        // boxes of keys from one warp took as long as the tile's arithmetic), so three warps ask: one
        // for the values, two for the keys, half a tile each.
        const int half = warp == AT_WARP_V ? 1 : 0;              // keys, or values
        const int key_half = warp == AT_WARP_K2 ? 1 : 0;         // keys 0-31 of a tile (pages 0, 1 of its four), or 32-63
        // The keys of tile kt go to key slot kt % KS, its values to value slot KS + kt % VS. The pages
        // of eight tiles are looked up at once, lane 4 t + sub for keys 16 sub .. of the batch's tile
        // t, and one batch ahead of their use. A group without a page (before the window, past the
        // end) is cleared instead when it holds values: 0 * garbage could be NaN.
        auto lookup = [&](int kt_first) -> int {
            const int kt = kt_first + (lane >> 2);
            const int j = k_begin + kt * AT_KEYS + (lane & 3) * 16;
            int page = -1;
            if (kt < n_tiles && j < khi && j + 16 > klo) {
                const int lp = max(j, klo) / p.page_size;
                if (lp < p.table_width) page = p.block_table[(size_t)entry * p.table_width + lp];
                if (page >= p.n_pages) page = -1;
            }
            return page;
        };
        int pages_now = 0, pages_next = lookup(0);
        constexpr uint32_t PAGE_BYTES = NBOX * 2048u;                                // a page's keys (or values) of one kv head
        for (int kt = 0; kt < n_tiles && !failed; ++kt) {
            if ((kt & 7) == 0) { pages_now = pages_next; pages_next = lookup(kt + 8); }
            const int j0 = k_begin + kt * AT_KEYS;
            const int page = __shfl_sync(0xffffffffu, pages_now, (kt & 7) * 4 + (lane & 3));
            const uint32_t have = __ballot_sync(0xffffffffu, page >= 0) & 0xFu;       // bit sub: group sub has a page
            const int live = __popc(have);
            {
                const int s = half == 0 ? kt % KS : KS + kt % VS;
                const int round = half == 0 ? kt / KS : kt / VS;
                bool ok = true;
                if (lane == 0) ok = at_mbar_wait(empty + s, ((uint32_t)round & 1u) ^ 1u);
                if (!__shfl_sync(0xffffffffu, ok ? 1 : 0, 0)) { failed = true; break; }
                unsigned char* dst = ring + s * C::SLOT_BYTES;
                if (half == 1 && live < 4) {
                    for (int sub = 0; sub < 4; ++sub) {
                        if (have & (1u << sub)) continue;
                        uint4* z = reinterpret_cast<uint4*>(dst + sub * PAGE_BYTES);
                        for (int e = lane; e < (int)(PAGE_BYTES / 16); e += 32) z[e] = make_uint4(0u, 0u, 0u, 0u);
                    }
                    at_fence_async_smem();
                    __syncwarp();
                }
                if (lane == 0) {
                    const uint32_t mine = half == 1 ? have : (have >> (2 * key_half)) & 3u;      // the page groups this warp brings
                    at_mbar_expect_tx(full + s, (uint32_t)__popc(mine) * PAGE_BYTES);
                }
                __syncwarp();
                if (half == 0) {
                    // keys: a box of 16 keys x 64 elements a lane, chunk by chunk [chunk][page][16 keys], so that
                    // the tile's eight-key groups are 1 KB apart and one product takes all 64 keys
                    const int sub = 2 * key_half + ((lane / NBOX) & 1), bx = lane % NBOX;
                    const int pg = __shfl_sync(0xffffffffu, page, sub);
                    if (lane < 2 * NBOX && pg >= 0) {
                        const int j = j0 + sub * 16;
                        const int row = (pg * p.hkv + kvh) * p.page_size + j % p.page_size;
                        at_tma_box(at_saddr(dst) + (uint32_t)(bx * 4 + sub) * 2048u, &map_k, bx * 64, row, full + s);
                    }
                } else if (lane < 4 && page >= 0) {              // values: one copy a page, [page][chunk][16 keys]
                    const int j = j0 + lane * 16;
                    const int row = (page * p.hkv + kvh) * p.page_size + j % p.page_size;
                    at_tma_page(at_saddr(dst) + (uint32_t)lane * PAGE_BYTES, &map_v, row, full + s);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- the score products, from one lane
        if (lane == 0) {
            constexpr uint32_t IDESC_S = at_idesc(AT_ROWS, AT_KEYS, false);
            const uint32_t ring_addr = at_saddr(ring);
            for (int kt = 0; kt < n_tiles; ++kt) {               // S[kt & 1] = Q K(kt)^T
                const int s = kt % KS, b = kt & 1;
                if (!at_mbar_wait(full + s, (uint32_t)(kt / KS) & 1u)) { failed = true; break; }
                // the buffer still holds tile kt - 2's P until the product that reads it is complete
                if (kt >= 2 && !at_mbar_wait(s_free + b, (uint32_t)((kt - 2) >> 1) & 1u)) { failed = true; break; }
                at_fence_after();
                const uint32_t k_addr = ring_addr + (uint32_t)s * C::SLOT_BYTES;
                const uint32_t d_tmem = tmem + (uint32_t)(C::COL_S + b * AT_KEYS);
#pragma unroll
                for (int bx = 0; bx < NBOX; ++bx) {
                    const uint32_t a_tmem = tmem + (uint32_t)(C::COL_Q + bx * 32);          // 64 elements of Q: 32 columns
                    const uint64_t bdesc = at_desc(k_addr + bx * (AT_KEYS * 128), 16, 1024);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        at_mma_ts(d_tmem, a_tmem + (uint32_t)(kk * 8), bdesc + (uint64_t)(kk * 2), IDESC_S, (bx | kk) != 0 ? 1u : 0u);
                }
                at_commit(empty + s);                            // the key slot is free when S is complete
                at_commit(s_full + b);
            }
        }
    } else if (warp == AT_WARP_PV) {
        // ---------------------------------------------------------------- the P V products, from one lane
        if (lane == 0) {
            constexpr uint32_t PAGE_BYTES = NBOX * 2048u;
            constexpr uint32_t IDESC_O = at_idesc(AT_ROWS, HD, true);
            const uint32_t ring_addr = at_saddr(ring);
            for (int kt = 0; kt < n_tiles; ++kt) {
                const int b = kt & 1;
                const int s = KS + kt % VS;
                if (!at_mbar_wait(full + s, (uint32_t)(kt / VS) & 1u)) { failed = true; break; }
                if (!at_mbar_wait(p_full + b, (uint32_t)(kt >> 1) & 1u)) { failed = true; break; }
                at_fence_after();
                const uint32_t v_addr = ring_addr + (uint32_t)s * C::SLOT_BYTES;
                const uint32_t a_tmem = tmem + (uint32_t)(C::COL_S + b * AT_KEYS);          // P lies over its S
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    // keys 16 kk ..: page kk of the tile, its two eight-key groups 1 KB apart, chunks 2 KB apart
                    const uint64_t bdesc = at_desc(v_addr + (uint32_t)kk * PAGE_BYTES, 2048, 1024);
                    at_mma_ts(tmem + C::COL_O, a_tmem + (uint32_t)(kk * 8), bdesc, IDESC_O, (kt | kk) != 0 ? 1u : 0u);
                }
                at_commit(empty + s);
                at_commit(s_free + b);                           // P has been read: the scores of tile kt + 2 may land
            }
            if (!failed) at_commit(o_full);
        }
    } else if (warp >= 2 && warp < 10) {
        // ---------------------------------------------------------------- softmax and epilogue, half a row a thread
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;                        // 0: keys 0-31 of a tile (and the head's first half), 1: the rest
        const int r = quarter * 32 + lane;                       // the row of the tile, and the TMEM lane
        const bool own = r < rows_valid;
        const int cnt = own ? c_first + r / group : 0;
        const int fst = (own && p.window > 0 && cnt > p.window) ? cnt - p.window : 0;
        const int lo = max(fst, klo), hi = min(cnt, khi);        // this row sees keys [lo, hi) of this block's
        const int lo_max = __reduce_max_sync(0xffffffffu, lo), hi_min = __reduce_min_sync(0xffffffffu, hi);
        const uint32_t lanes = tmem + ((uint32_t)(quarter * 32) << 16);
        const float c1 = p.scale / p.cap, c2 = p.cap * 1.4426950408889634f;
        float l = 0.f;
        for (int kt = 0; kt < n_tiles; ++kt) {
            const int b = kt & 1;
            const int j0 = k_begin + kt * AT_KEYS + half * 32;   // this warp's 32 keys of the tile
            if (!__all_sync(0xffffffffu, at_mbar_wait(s_full + b, (uint32_t)(kt >> 1) & 1u))) { failed = true; break; }
            at_fence_after();
            uint32_t sv[32], pr[16];
            const bool edge = j0 < lo_max || j0 + 32 > hi_min;   // the same for the whole warp
            at_ld32(lanes + (uint32_t)(C::COL_S + b * AT_KEYS + half * 32), sv);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            // P lies over the first 32 columns of its S: the second warp's scores sit in columns that
            // nobody overwrites, but the first warp's P covers columns 0-15 and the second's 16-31, which
            // hold the first warp's scores 0-31: both warps have their scores in registers before either
            // stores (the two meet on a named barrier of their own, one a quarter).
            float la = 0.f, lb = 0.f;                            // two chains of additions
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                float p0 = at_exp2(c2 * at_tanh(__uint_as_float(sv[j]) * c1));
                float p1 = at_exp2_poly(c2 * at_tanh(__uint_as_float(sv[j + 1]) * c1));
                if (edge) {
                    const int jj = j0 + j;
                    if (jj < lo || jj >= hi) p0 = 0.f;
                    if (jj + 1 < lo || jj + 1 >= hi) p1 = 0.f;
                }
                la += p0;
                lb += p1;
                pr[j >> 1] = at_pack(p0, p1);
            }
            l += la + lb;
            asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");      // the quarter's two warps have read their scores
            at_st16(lanes + (uint32_t)(C::COL_S + b * AT_KEYS + half * 16), pr);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            at_fence_before();
            __syncwarp();
            if (lane == 0) at_mbar_arrive(p_full + b);
        }
        // The row's sum: the second warp's share goes to the first through shared memory, and the
        // reciprocal of the whole comes back the same way. Both warps of a quarter pass these barriers
        // whatever happened above.
        if (half == 1) l_half[r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
        float inv = 0.f;
        if (half == 0) {
            l += l_half[r];
            inv = l > 0.f ? 1.f / l : 0.f;
        }
        asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
        if (half == 0) l_half[r] = inv;
        asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
        if (half == 1) inv = l_half[r];
        if (!failed && !__all_sync(0xffffffffu, at_mbar_wait(o_full, 0u))) failed = true;
        if (!failed) {
            at_fence_after();
            // With several slots, a row whose keys all lie in one slot is finished by that slot's block.
            const int z0 = p.slots > 1 ? fst / p.split : 0;
            const int z1 = p.slots > 1 ? min(p.slots - 1, (max(cnt, 1) - 1) / p.split) : 0;
            const bool direct = z0 == z1;
            const bool writes = own && (!direct || slot == z0);
            const int row = row0 + r / group, head = kvh * group + r % group;
            bf16* dst = p.out + ((size_t)row * p.hq + head) * d;
            float* pdst = p.partial ? p.partial + (((size_t)row * p.hq + head) * p.slots + slot) * (d + 2) : nullptr;
            // the quarter's first warp reads out the head's first half, the second its second half
            for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 32) {
                uint32_t o[32];
                __syncwarp();
                at_ld32(lanes + (uint32_t)(C::COL_O + c0), o);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (!writes) continue;
                if (direct) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 v;
                        v.x = at_pack(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv);
                        v.y = at_pack(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
                        v.z = at_pack(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
                        v.w = at_pack(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + j) = v;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 2)
                        *reinterpret_cast<float2*>(pdst + c0 + j) = make_float2(__uint_as_float(o[j]), __uint_as_float(o[j + 1]));
                }
            }
            if (writes && !direct && half == 0) { pdst[d] = 0.f; pdst[d + 1] = l; }
        }
    }
    if (failed) atomicExch(&g_attention_tc_error, 1);
    at_fence_before();
    __syncthreads();
    if (warp == 1) {
        at_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------
// The same attention by pairs of blocks (a cluster of two, on the two multiprocessors of a pair),
// for head sizes 128 and 256. A multiprocessor takes in about 35 bytes a clock from L2, and a step of
// the kernel above needs 64 KB of keys and values for 128 rows: 2,500 clocks a step whatever the
// tensor cores could do. Here tcgen05.mma.cta_group::2 works on 256 rows, the 128 of each block in
// its own TMEM, against one tile of keys and values of which each block holds half: the first block
// keys 0-31 of a step and the first half of the head's elements of the values, the second keys 32-63
// and the second half (the B operand of a cta_group::2 product is split along its N between the two
// blocks). A block takes in half as much a step and row.
//   * a tile is up to 256 rows: the first block takes rows 0-127, the second rows 128-255; each keeps its Q
//     in shared memory (the A operand of the score products) and four S buffers in TMEM;
//   * both blocks' TMA copies complete on the first block's "full" barrier (two arrivals: the first
//     block's, with the bytes expected from both, and the second block's, when it has cleared what
//     it had no page for);
//   * the first block's warps 1 and 10 issue the products for both; tcgen05.commit with a two-block
//     mask frees the key and value slots and hands over S and O in both blocks;
//   * the softmax warps of both blocks arrive on the first block's "P written" barrier;
//   * the blocks meet at a cluster barrier after their Q is in TMEM and before TMEM is freed, so
//     neither signals a block that is not there yet or has left.
constexpr uint32_t AT_PEER_MASK = 0xFEFFFFFFu;                 // clears the bit that tells the two blocks' shared windows apart

__device__ __forceinline__ void atp_tma_box(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void atp_tma_page(uint32_t dst, const CUtensorMap* map, int row, int chunk, uint32_t bar_addr) {
    const int zero = 0;
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_addr), "r"(zero), "r"(row), "r"(chunk) : "memory");
}
__device__ __forceinline__ void atp_commit_both(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(at_saddr(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void atp_commit_here(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_saddr(bar)) : "memory");
}
__device__ __forceinline__ void atp_arrive_on_first(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, 0;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(at_saddr(bar)) : "memory");
}
__device__ __forceinline__ void atp_mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same without the release: for a signal that only says "my tcgen05.st has completed" (the store was
// waited for and fenced with tcgen05.fence::before_thread_sync), which needs no ordering of ordinary
// memory. A release at cluster scope costs the arriving thread more than a thousand clocks.
__device__ __forceinline__ void atp_arrive_on_first_relaxed(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, 0;\n\t"
        "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(at_saddr(bar)) : "memory");
}
__device__ __forceinline__ void atp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void atp_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

constexpr int ATP_ROWS = 256;                                   // rows a tile of the pair kernel
// Twenty-one warps: the single-block kernel's roles in warps 0-12, and eight more softmax warps (13-20):
// the four warps of a quarter of the rows take 32 keys of a step each.
constexpr int ATP_THREADS = 672;

constexpr int ATP_KEYS = 128;                                   // keys a step of the pair kernel: one product takes them all

template <int HD> struct AtpCfg {
    static constexpr int NBOX = HD / 64;                        // chunks of 64 elements along the head
    static constexpr int SLOT_BYTES = ATP_KEYS * HD;            // a block's half of a key tile (64 keys), or of a value tile (half the head)
    static constexpr int K_SLOTS = HD == 256 ? 2 : 4;
    static constexpr int V_SLOTS = HD == 256 ? 3 : 4;          // a value slot is held until its P V product is complete, longer than a key slot
    static constexpr int SLOTS = K_SLOTS + V_SLOTS;
    // Q lies in shared memory here (the A operand of the score products), which leaves TMEM for O and
    // S buffers of 128 keys: a score product of 128 keys costs the tensor cores what one of 64 does.
    static constexpr int S_BUFS = (512 - HD) / ATP_KEYS;        // 2 at head size 256, 3 at 128
    static constexpr int Q_BYTES = AT_ROWS * HD * 2;
    static constexpr int COL_O = 0, COL_S = HD;
    static constexpr int TMEM_COLS = 512;
    static constexpr int SMEM = Q_BYTES + SLOTS * SLOT_BYTES + 1024 /* alignment */ + 384 /* barriers */;
    static_assert(HD + S_BUFS * ATP_KEYS <= TMEM_COLS, "O and the S buffers outgrew TMEM");
    static_assert((2 * SLOTS + 3 * S_BUFS + 1) * 8 + 8 <= 384, "the barriers outgrew their room");
    static_assert(SMEM <= 232448, "more shared memory than a block can have");
};

template <int HD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(ATP_THREADS, 1)
attention_tc_pair_kernel(const AttTcParams p, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
    using C = AtpCfg<HD>;
    constexpr int NBOX = C::NBOX, NS = C::SLOTS, KS = C::K_SLOTS, VS = C::V_SLOTS, SB = C::S_BUFS;
    constexpr uint32_t PAGE_FULL = NBOX * 2048u;                 // a page's keys (or values) of one kv head, both blocks' halves
    constexpr uint32_t PAGE_HALF = PAGE_FULL / 2;                // a block's half of a page of values
    extern __shared__ unsigned char at_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)at_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_smem = smem;                                // [chunk][128 rows][128 bytes], 128-byte swizzle
    unsigned char* ring = smem + C::Q_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + NS * C::SLOT_BYTES);    // [NS] the first block's: both halves of a slot have landed
    uint64_t* empty = full + NS;                                 // [NS] the product that read a slot is complete (in both blocks)
    uint64_t* s_full = empty + NS;                               // [SB] S complete (in both blocks)
    uint64_t* p_full = s_full + SB;                              // [SB] the first block's: P written by the 32 softmax warps of both
    uint64_t* s_free = p_full + SB;                              // [SB] the first block's: the product that read P is complete
    uint64_t* o_full = s_free + SB;                              // [1] O complete (in both blocks)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
    // [4][128] sum p by row, a share from each softmax warp of a quarter: over the start of Q, which nothing
    // reads any more when the softmax warps have seen the last scores complete
    float* l_part = reinterpret_cast<float*>(q_smem);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int kvh = blockIdx.x >> 1, slot = blockIdx.y;
    const int tile = gridDim.z - 1 - blockIdx.z;                 // later tiles of a prompt see more keys: they start first
    const int group = p.hq / p.hkv;
    const int row0 = p.tile_row0[tile], nq = p.tile_nq[tile];
    const int entry = p.tile_entry[tile];
    const int rows_all = nq * group;                             // rows of the tile, of which this block has 128 from rank * 128
    const int c_first = p.row_count[row0];
    int klo = (p.window > 0 && c_first > p.window) ? c_first - p.window : 0;
    int khi = c_first > 0 ? c_first + nq - 1 : 0;                // a padding row sees nothing
    if (p.split > 0) {
        klo = max(klo, slot * p.split);
        khi = min(khi, (slot + 1) * p.split);
    }
    constexpr int d = HD;
    if (klo >= khi) {                                            // nothing for this pair (the same in both blocks): before anything is allocated
        dependent_wait();
        if (p.slots == 1 && c_first <= 0)
            for (int i = tid; i < AT_ROWS * d; i += ATP_THREADS) {
                const int R = (int)rank * AT_ROWS + i / d, c = i % d;
                if (R < rows_all) p.out[((size_t)(row0 + R / group) * p.hq + kvh * group + R % group) * d + c] = __float2bfloat16_rn(0.f);
            }
        return;
    }
    const int k_begin = klo / ATP_KEYS * ATP_KEYS;
    const int n_tiles = (khi - k_begin + ATP_KEYS - 1) / ATP_KEYS;

    if (tid == 0) {
        // a key slot is filled by two warps of each block, a value slot by one of each
        for (int s = 0; s < NS; ++s) { at_mbar_init(full + s, s < KS ? 4 : 2); at_mbar_init(empty + s, 1); }
        for (int b = 0; b < SB; ++b) { at_mbar_init(s_full + b, 1); at_mbar_init(p_full + b, 32); at_mbar_init(s_free + b, 1); }
        at_mbar_init(o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_saddr(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    at_fence_before();
    __syncthreads();
    at_fence_after();
    const uint32_t tmem = *tmem_slot;
    dependent_wait();                                       // the queries and the newest keys are the kernel before's
    // Q into shared memory as the A operand of the score products, K-major under the 128-byte swizzle:
    // chunk c (64 elements) of row r at c * 16 KB + r * 128, its 16-byte pieces exchanged by r mod 8.
    // The two warps of a quarter of the rows (of the first softmax group) take half of the head each.
    if (warp >= 2 && warp < 10) {
        const int r = (warp & 3) * 32 + lane;
        const int R = (int)rank * AT_ROWS + r;
        const int half = (warp - 2) >> 2;
        const bool own = R < rows_all;
        const bf16* src = p.q + ((size_t)(row0 + (own ? R / group : 0)) * p.hq + kvh * group + (own ? R % group : 0)) * d;
        for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 64) {
            unsigned char* dst = q_smem + (size_t)(c0 / 64) * (AT_ROWS * 128) + (size_t)r * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (own) v = *reinterpret_cast<const uint4*>(src + c0 + j * 8);
                *reinterpret_cast<uint4*>(dst + ((j ^ (r & 7)) << 4)) = v;
            }
        }
        at_fence_async_smem();
    }
    // Both blocks' Q in place and both blocks' barriers made, before anything is signalled across.
    at_fence_before();
    __syncthreads();
    atp_cluster_sync();
    at_fence_after();
    bool failed = false;

    if (warp == 0 || warp == AT_WARP_V || warp == AT_WARP_K2) {
        // ---------------------------------------------------------------- pages and boxes, this block's halves
        // A step is 128 keys: eight pages of 16. Keys: the first block brings keys 0-63 of a step (pages
        // 0-3), the second keys 64-127, each with two warps (two pages a warp), laid out [chunk][64
        // keys]: eight-key groups 1 KB apart. Values: every page's 16 keys, this block's half of the
        // head's chunks, [page][chunk][16 keys], one warp. A group without a page (before the window,
        // past the end) is cleared instead when it holds values. Asking TMA for a box keeps the asking
        // warp busy for more than a hundred clocks: hence three warps.
        const int half = warp == AT_WARP_V ? 1 : 0;              // keys, or values
        const int key_half = warp == AT_WARP_K2 ? 1 : 0;         // of this block's four pages of keys: 0, 1 or 2, 3
        // The pages of four steps are looked up at once, lane 8 t + sub for keys 16 sub .. of the batch's step t.
        auto lookup = [&](int kt_first) -> int {
            const int kt = kt_first + (lane >> 3);
            const int j = k_begin + kt * ATP_KEYS + (lane & 7) * 16;
            int page = -1;
            if (kt < n_tiles && j < khi && j + 16 > klo) {
                const int lp = max(j, klo) / p.page_size;
                if (lp < p.table_width) page = p.block_table[(size_t)entry * p.table_width + lp];
                if (page >= p.n_pages) page = -1;
            }
            return page;
        };
        int pages_now = 0, pages_next = lookup(0);
        for (int kt = 0; kt < n_tiles && !failed; ++kt) {
            if ((kt & 3) == 0) { pages_now = pages_next; pages_next = lookup(kt + 4); }
            const int j0 = k_begin + kt * ATP_KEYS;
            const int page = __shfl_sync(0xffffffffu, pages_now, (kt & 3) * 8 + (lane & 7));
            const uint32_t have = __ballot_sync(0xffffffffu, page >= 0) & 0xFFu;      // bit sub: group sub has a page
            const int live = __popc(have);
            const int s = half == 0 ? kt % KS : KS + kt % VS;
            const int round = half == 0 ? kt / KS : kt / VS;
            bool ok = true;
            if (lane == 0) ok = at_mbar_wait(empty + s, ((uint32_t)round & 1u) ^ 1u);
            if (!__shfl_sync(0xffffffffu, ok ? 1 : 0, 0)) { failed = true; break; }
            unsigned char* dst = ring + s * C::SLOT_BYTES;
            const uint32_t bar = at_saddr(full + s) & AT_PEER_MASK;              // the first block's barrier
            if (half == 1 && live < 8) {
                for (int sub = 0; sub < 8; ++sub) {
                    if (have & (1u << sub)) continue;
                    uint4* z = reinterpret_cast<uint4*>(dst + sub * PAGE_HALF);
                    for (int e = lane; e < (int)(PAGE_HALF / 16); e += 32) z[e] = make_uint4(0u, 0u, 0u, 0u);
                }
                at_fence_async_smem();
                __syncwarp();
            }
            if (lane == 0) {
                // One arrival a warp. The first block's first key warp and its value warp carry the bytes that
                // all will bring; the second block's arrive with a release only when they cleared something
                // the first block's products will read.
                if (rank == 0 && key_half == 0) at_mbar_expect_tx(full + s, (uint32_t)live * PAGE_FULL);
                else if (rank == 0) at_mbar_arrive(full + s);
                else if (half == 1 && live < 8) atp_arrive_on_first(full + s);
                else atp_arrive_on_first_relaxed(full + s);
            }
            __syncwarp();
            if (half == 0) {
                // this warp's two pages of keys: a box of 16 keys x 64 elements a lane, [chunk][page][16 keys]
                const int sub_local = 2 * key_half + ((lane / NBOX) & 1), bx = lane % NBOX;
                const int sub = (int)rank * 4 + sub_local;
                const int pg = __shfl_sync(0xffffffffu, page, sub);
                if (lane < 2 * NBOX && pg >= 0) {
                    const int j = j0 + sub * 16;
                    const int row = (pg * p.hkv + kvh) * p.page_size + j % p.page_size;
                    atp_tma_box(at_saddr(dst) + (uint32_t)(bx * 4 + sub_local) * 2048u, &map_k, bx * 64, row, bar);
                }
            } else if (lane < 8 && page >= 0) {                  // values: one copy a page, this block's chunks
                const int j = j0 + lane * 16;
                const int row = (page * p.hkv + kvh) * p.page_size + j % p.page_size;
                atp_tma_page(at_saddr(dst) + (uint32_t)lane * PAGE_HALF, &map_v, row, (int)rank * (NBOX / 2), bar);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- the score products of both blocks, from one lane of the first
        if (lane == 0 && rank == 0) {
            constexpr uint32_t IDESC_S = at_idesc(ATP_ROWS, ATP_KEYS, false);
            const uint32_t ring_addr = at_saddr(ring);
            const uint32_t q_addr = at_saddr(q_smem);
            for (int kt = 0; kt < n_tiles; ++kt) {               // S[kt % SB] = Q K(kt)^T
                const int s = kt % KS, b = kt % SB;
                if (!at_mbar_wait(full + s, (uint32_t)(kt / KS) & 1u)) { failed = true; break; }
                // the buffer still holds tile kt - SB's P until the product that reads it is complete
                if (kt >= SB && !at_mbar_wait(s_free + b, (uint32_t)(kt / SB - 1) & 1u)) { failed = true; break; }
                at_fence_after();
                const uint32_t k_addr = ring_addr + (uint32_t)s * C::SLOT_BYTES;
                const uint32_t d_tmem = tmem + (uint32_t)(C::COL_S + b * ATP_KEYS);
#pragma unroll
                for (int bx = 0; bx < NBOX; ++bx) {
                    const uint64_t adesc = at_desc(q_addr + bx * (AT_ROWS * 128), 16, 1024);        // 64 elements of the 128 rows
                    const uint64_t bdesc = at_desc(k_addr + bx * (ATP_KEYS / 2 * 128), 16, 1024);  // this chunk's 64 keys a block
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        atp_mma_ss(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), IDESC_S, (bx | kk) != 0 ? 1u : 0u);
                }
                atp_commit_both(empty + s);                      // the key slot is free in both blocks when S is complete
                atp_commit_both(s_full + b);
            }
        }
    } else if (warp == AT_WARP_PV) {
        // ---------------------------------------------------------------- the P V products of both blocks
        if (lane == 0 && rank == 0) {
            constexpr uint32_t IDESC_O = at_idesc(ATP_ROWS, HD, true);
            const uint32_t ring_addr = at_saddr(ring);
            for (int kt = 0; kt < n_tiles; ++kt) {
                const int b = kt % SB;
                const int s = KS + kt % VS;
                if (!at_mbar_wait(full + s, (uint32_t)(kt / VS) & 1u)) { failed = true; break; }
                if (!at_mbar_wait(p_full + b, (uint32_t)(kt / SB) & 1u)) { failed = true; break; }
                at_fence_after();
                const uint32_t v_addr = ring_addr + (uint32_t)s * C::SLOT_BYTES;
                const uint32_t a_tmem = tmem + (uint32_t)(C::COL_S + b * ATP_KEYS);         // P lies over the first half of its S
#pragma unroll
                for (int kk = 0; kk < ATP_KEYS / 16; ++kk) {
                    // keys 16 kk ..: page kk, its two eight-key groups 1 KB apart, this block's chunks 2 KB apart
                    const uint64_t bdesc = at_desc(v_addr + (uint32_t)kk * PAGE_HALF, 2048, 1024);
                    atp_mma_ts(tmem + C::COL_O, a_tmem + (uint32_t)(kk * 8), bdesc, IDESC_O, (kt | kk) != 0 ? 1u : 0u);
                }
                atp_commit_both(empty + s);
                atp_commit_here(s_free + b);                     // P has been read: the scores of tile kt + SB may land
            }
            if (!failed) atp_commit_both(o_full);
        }
    } else if ((warp >= 2 && warp < 10) || warp >= 13) {
        // ---------------------------------------------------------------- softmax and epilogue: a row's 32 keys of a step a thread
        const int quarter = warp & 3;
        const int share = warp >= 13 ? 2 + ((warp - 13) >> 2) : (warp - 2) >> 2;    // which of the quarter's four warps: keys 32 share .. of a step
        const int r = quarter * 32 + lane;                       // the TMEM lane
        const int R = (int)rank * AT_ROWS + r;                   // the row of the tile
        const bool own = R < rows_all;
        const int cnt = own ? c_first + R / group : 0;
        const int fst = (own && p.window > 0 && cnt > p.window) ? cnt - p.window : 0;
        const int lo = max(fst, klo), hi = min(cnt, khi);
        const int lo_max = __reduce_max_sync(0xffffffffu, lo), hi_min = __reduce_min_sync(0xffffffffu, hi);
        const uint32_t lanes = tmem + ((uint32_t)(quarter * 32) << 16);
        const float c1 = p.scale / p.cap, c2 = p.cap * 1.4426950408889634f;
        float l = 0.f;
        for (int kt = 0; kt < n_tiles; ++kt) {
            const int b = kt % SB;
            const int j0 = k_begin + kt * ATP_KEYS + share * 32;
            if (!__all_sync(0xffffffffu, at_mbar_wait(s_full + b, (uint32_t)(kt / SB) & 1u))) { failed = true; break; }
            at_fence_after();
            uint32_t sv[32], pr[16];
            const bool edge = j0 < lo_max || j0 + 32 > hi_min;
            at_ld32(lanes + (uint32_t)(C::COL_S + b * ATP_KEYS + share * 32), sv);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            float la = 0.f, lb = 0.f;
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                float p0 = at_exp2(c2 * at_tanh(__uint_as_float(sv[j]) * c1));
                float p1 = at_exp2_poly(c2 * at_tanh(__uint_as_float(sv[j + 1]) * c1));
                if (edge) {
                    const int jj = j0 + j;
                    if (jj < lo || jj >= hi) p0 = 0.f;
                    if (jj + 1 < lo || jj + 1 >= hi) p1 = 0.f;
                }
                la += p0;
                lb += p1;
                pr[j >> 1] = at_pack(p0, p1);
            }
            l += la + lb;
            // P (64 columns) lies over the scores of keys 0-63: the quarter's four warps have all read
            // theirs before any of them stores
            asm volatile("bar.sync %0, 128;" ::"r"(2 + quarter) : "memory");
            at_st16(lanes + (uint32_t)(C::COL_S + b * ATP_KEYS + share * 16), pr);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            at_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) at_mbar_arrive(p_full + b);       // the first block's own barrier
                else atp_arrive_on_first_relaxed(p_full + b);
            }
        }
        // The row's sum: the quarter's four warps leave their shares in shared memory; all sixteen
        // softmax warps pass this barrier whatever happened above.
        l_part[share * AT_ROWS + r] = l;
        asm volatile("bar.sync 10, 512;" ::: "memory");
        l = l_part[r] + l_part[AT_ROWS + r] + l_part[2 * AT_ROWS + r] + l_part[3 * AT_ROWS + r];
        const float inv = l > 0.f ? 1.f / l : 0.f;
        if (!failed && !__all_sync(0xffffffffu, at_mbar_wait(o_full, 0u))) failed = true;
        if (!failed) {
            at_fence_after();
            const int z0 = p.slots > 1 ? fst / p.split : 0;
            const int z1 = p.slots > 1 ? min(p.slots - 1, (max(cnt, 1) - 1) / p.split) : 0;
            const bool direct = z0 == z1;
            const bool writes = own && (!direct || slot == z0);
            const int row = row0 + R / group, head = kvh * group + R % group;
            bf16* dst = p.out + ((size_t)row * p.hq + head) * d;
            float* pdst = p.partial ? p.partial + (((size_t)row * p.hq + head) * p.slots + slot) * (d + 2) : nullptr;
            // each of the quarter's four warps reads out a quarter of the head
            for (int c0 = share * (HD / 4); c0 < (share + 1) * (HD / 4); c0 += 32) {
                uint32_t o[32];
                __syncwarp();
                at_ld32(lanes + (uint32_t)(C::COL_O + c0), o);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (!writes) continue;
                if (direct) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 v;
                        v.x = at_pack(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv);
                        v.y = at_pack(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
                        v.z = at_pack(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
                        v.w = at_pack(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + j) = v;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 2)
                        *reinterpret_cast<float2*>(pdst + c0 + j) = make_float2(__uint_as_float(o[j]), __uint_as_float(o[j + 1]));
                }
            }
            if (writes && !direct && share == 0) { pdst[d] = 0.f; pdst[d + 1] = l; }
        }
    }
    if (failed) atomicExch(&g_attention_tc_error, 1);
    at_fence_before();
    __syncthreads();
    atp_cluster_sync();
    if (warp == 1) {
        at_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
    }
}

template <int HD>
static int launch_tc_pair(const AttTcParams& p, const void* k_table, const void* v_table, int tiles, cudaStream_t s) {
    using C = AtpCfg<HD>;
    static bool attr_set = false;
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(attention_tc_pair_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return fail("attention_tc: cannot have %d bytes of shared memory: %s", C::SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    const unsigned long long rows = (unsigned long long)p.n_pages * p.hkv * p.page_size;
    CUtensorMap map_k, map_v;
    if (int e = encode_map_bf16(&map_k, k_table, rows, p.d, p.d, 16)) return e;
    if (int e = encode_map_bf16_chunks(&map_v, v_table, rows, p.d, 16, p.d / 128)) return e;
    dim3 grid(2 * p.hkv, p.slots, tiles);
    launch_dependent_if(false, attention_tc_pair_kernel<HD>, grid, dim3(ATP_THREADS), (size_t)C::SMEM, s, p, map_k, map_v);
    return check_launch("attention_tc (pairs)");
}

template <int HD>
static int launch_tc(const AttTcParams& p, const void* k_table, const void* v_table, int tiles, cudaStream_t s) {
    using C = AtCfg<HD>;
    static bool attr_set = false;
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return fail("attention_tc: cannot have %d bytes of shared memory: %s", C::SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    const unsigned long long rows = (unsigned long long)p.n_pages * p.hkv * p.page_size;
    CUtensorMap map_k, map_v;
    if (int e = encode_map_bf16(&map_k, k_table, rows, p.d, p.d, 16)) return e;
    if (int e = encode_map_bf16_chunks(&map_v, v_table, rows, p.d, 16)) return e;
    dim3 grid(p.hkv, p.slots, tiles);
    launch_dependent_if(false, attention_tc_kernel<HD>, grid, dim3(AT_THREADS), (size_t)C::SMEM, s, p, map_k, map_v);
    return check_launch("attention_tc");
}

}  // namespace kb

using namespace kb;

// 1 if a wait inside the kernel ever ran out (and clears the flag); synchronises the device.
extern "C" int kb_attention_tc_error() {
    int flag = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&flag, g_attention_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (flag) cudaMemcpyToSymbol(g_attention_tc_error, &zero, sizeof(int));
    return flag;
}

// 1 where the kernel applies: head sizes 64, 128 and 256, a soft cap of at most 64, pages of a
// multiple of 16 positions, at most 128 query heads a kv head.
extern "C" int kb_attention_tc_takes(int hq, int hkv, int d, int page_size, float cap) {
    return (d == 64 || d == 128 || d == 256) && cap > 0.f && cap <= 64.f && page_size > 0 && page_size % 16 == 0 && hkv > 0 &&
           hq % hkv == 0 && hq / hkv <= AT_ROWS;
}

// Whether pairs of blocks run head size d. `pairs`: 0 never, 1 wherever such a kernel exists (128 and
// 256), 2 where it measured faster than single blocks (256: 42 against 47 us for a prompt of 2,048 tokens
// with 8 heads over 4; at 128 with 32 heads over 16 the pairs took 86 us, single blocks 79).
static bool tc_pairs(int d, int pairs) { return pairs == 1 ? (d == 128 || d == 256) : (pairs == 2 && d == 256); }

// Rows (token, query head of one kv head) a tile holds: 256 where pairs of blocks run it, else 128.
extern "C" int kb_attention_tc_rows(int d, int pairs) { return tc_pairs(d, pairs) ? ATP_ROWS : AT_ROWS; }

// Prompt portions; arguments as kb_attention_mma's with decode = 0, tiles of kb_attention_tc_rows(d,
// pairs) rows. With slots > 1, `scratch` holds [rows, hq, slots, d + 2] floats and the caller merges it
// (kb_attention_mma_combine). `pairs` as kb_attention_tc_rows takes it.
extern "C" int kb_attention_tc(void* out, const void* q, const void* k_table, const void* v_table, const int* block_table,
                               const int* row_count, const int* tile_entry, const int* tile_row0, const int* tile_nq, int tiles,
                               int rows, int hq, int hkv, int d, int page_size, int table_width, int n_pages, int window,
                               int split, int slots, float scale, float cap, float* scratch, int pairs, void* stream) {
    KB_REQUIRE(rows >= 0 && tiles >= 0 && hq > 0 && hkv > 0, "attention_tc: rows %d, tiles %d, heads %d over %d", rows, tiles, hq, hkv);
    KB_REQUIRE(kb_attention_tc_takes(hq, hkv, d, page_size, cap), "attention_tc: head_dim %d, %d heads over %d, pages of %d, cap %g are not taken",
               d, hq, hkv, page_size, cap);
    KB_REQUIRE(table_width > 0 && n_pages > 0 && window >= 0, "attention_tc: table width %d, pages %d, window %d", table_width, n_pages, window);
    KB_REQUIRE((split == 0 && slots == 1) || (split > 0 && split % AT_KEYS == 0 && slots >= 1 && slots <= 65535),
               "attention_tc: split %d (a multiple of %d) with %d slots", split, AT_KEYS, slots);
    KB_REQUIRE(slots == 1 || scratch != nullptr, "attention_tc: %d slots need scratch memory", slots);
    KB_REQUIRE(tiles <= 65535 && hkv <= 65535, "attention_tc: %d tiles, %d kv heads is too many for one launch", tiles, hkv);
    KB_REQUIRE((((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_table | (uintptr_t)v_table) & 15) == 0, "attention_tc: operands must be 16-byte aligned");
    if (rows == 0 || tiles == 0) return 0;
    AttTcParams p;
    p.q = (const bf16*)q; p.block_table = block_table; p.row_count = row_count; p.tile_entry = tile_entry;
    p.tile_row0 = tile_row0; p.tile_nq = tile_nq; p.out = (bf16*)out; p.partial = slots > 1 ? scratch : nullptr;
    p.rows = rows; p.hq = hq; p.hkv = hkv; p.d = d; p.page_size = page_size; p.table_width = table_width; p.n_pages = n_pages;
    p.window = window; p.split = split; p.slots = slots; p.scale = scale; p.cap = cap;
    cudaStream_t s = (cudaStream_t)stream;
    if (d == 64) return launch_tc<64>(p, k_table, v_table, tiles, s);
    if (!tc_pairs(d, pairs)) return d == 128 ? launch_tc<128>(p, k_table, v_table, tiles, s) : launch_tc<256>(p, k_table, v_table, tiles, s);
    KB_REQUIRE(2 * hkv <= 65535, "attention_tc: %d kv heads is too many for one launch of pairs", hkv);
    return d == 128 ? launch_tc_pair<128>(p, k_table, v_table, tiles, s) : launch_tc_pair<256>(p, k_table, v_table, tiles, s);
}
