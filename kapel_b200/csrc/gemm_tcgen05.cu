// C[M,N] = A[M,K] . W[N,K]^T for bfloat16 inputs on the fifth-generation tensor cores:
// tcgen05.mma issued by one thread, operands staged in shared memory by TMA (cp.async.bulk.tensor,
// 128-byte swizzle, no multicast), the 128 x 256 accumulator in tensor memory (TMEM), read back
// with tcgen05.ld for the epilogue. Kapel's counterpart is the cutile `batched_matmul_nt`
// (crates/kapel-cuda/src/tile.rs:65-87), which has no sm_100 path. Four kernels, below in this order:
// one block a 128 x 256 tile (products of about one tile a multiprocessor); persistent pairs of
// blocks with cta_group::2 and two accumulators (all other products of more than 64 rows, also with
// the gated unit in the epilogue); operands swapped for up to 64 rows, split over K; the same with
// the gated unit. The last two (decoding) are launched as programmatic dependents and wait for the
// kernel before them only before they touch the activations; the first two are launched plainly.
//
// The first: one block computes one 128 x 256 tile of C. Six warps:
//   warp 0    one lane walks K in steps of 64 and asks TMA for the A and W tiles of each step, four
//             stages deep (two, in each of two blocks a multiprocessor, for products of many
//             tiles); a stage is free again when the MMAs that read it have completed
//             (tcgen05.commit on the stage's "empty" mbarrier)
//   warp 1    allocates 256 TMEM columns; one lane waits for a stage to fill and issues four
//             128 x 256 x 16 MMAs on it (the shared-memory descriptors step 32 bytes through the
//             swizzle atom), then commits; after the last step it commits on the "accumulator full"
//             mbarrier
//   warps 2-5 wait for the accumulator, read their quarter of its 128 lanes 32 columns at a time,
//             apply the epilogue (soft cap) and store
// Rows and columns beyond M, N and K are zero-filled by TMA on the way in and skipped on the way out.
//
// Every wait on an mbarrier gives up after about a second: the waiter raises a flag that
// `kb_tcgen05_error` reports, skips its remaining work, and the block still meets at its final
// barrier, frees its TMEM and returns.
#include "common.cuh"
#include "tensor_map.cuh"
#include "timeline.cuh"

namespace kb {

KB_TIMELINE_ARRAY(gemm)        // slots: kind 0 the few-rows product [n, k], kind 1 the gated one


typedef __nv_bfloat16 bf16;

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 64;
constexpr int TC_THREADS = 192;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;                  // 16 KB
constexpr int TC_B_BYTES = TC_BN * TC_BK * 2;                  // 32 KB
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int tc_smem_bytes(int stages) { return stages * TC_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */; }
constexpr int TC_TMEM_COLS = 256;

__device__ int g_tcgen05_error = 0;

__device__ __forceinline__ uint32_t tc_saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_saddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc_saddr(bar)), "r"(bytes) : "memory");
}
// false if the phase with this parity did not complete within `limit` clocks (by default ~1 s)
__device__ __forceinline__ bool tc_mbar_wait(uint64_t* bar, uint32_t parity, long long limit = 2000000000ll) {
    const uint32_t addr = tc_saddr(bar);
    const long long start = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if (clock64() - start > limit) return false;
    }
}

// For the test of the error path only: one block whose first thread waits, with the products' own
// wait and a limit given by the caller, on a barrier at which nobody ever arrives. The wait runs
// out, the flag is raised as a product would raise it, the block meets at its barrier and returns.
__global__ void wait_probe_kernel(long long limit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        tc_mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    bool failed = false;
    if (threadIdx.x == 0) failed = !tc_mbar_wait(&bar, 0u, limit);
    if (failed) atomicExch(&g_tcgen05_error, 1);
    __syncthreads();
}
__device__ __forceinline__ void tc_tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(tc_saddr(dst)), "l"(map), "r"(tc_saddr(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_saddr(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows under the 128-byte swizzle:
// start address / 16 in bits [0,14); leading byte offset / 16 = 1 in [16,30); stride byte offset
// / 16 = 64 (eight rows of 128 bytes) in [32,46); version 1 in [46,48); layout type 2 (128-byte
// swizzle) in [61,64).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: D float32 (1 at bit 4), A and B bfloat16 (1 at bits 7 and 10),
// both K-major (0 at bits 15, 16), N / 8 at bits [17,23), M / 16 at bits [24,29).
constexpr uint32_t TC_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(TC_IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

// Epilogues, chosen at compile time so that each kernel carries only its own code:
// 0 none, 1 soft cap c * tanh(x / c), 2 and 3 the gated unit gelu_tanh(gate) * up and silu(gate) * up.
constexpr int EPI_NONE = 0, EPI_SOFTCAP = 1, EPI_GLU_GELU = 2, EPI_GLU_SILU = 3;

__device__ __forceinline__ uint4 tc_pack8(const float (&v)[8]) {
    uint4 o;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]), p3 = __floats2bfloat162_rn(v[6], v[7]);
    o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
    o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
    return o;
}

// Eight neighbouring results of one row, from column `col` on, to a row of `n` columns. Every index
// is a compile-time constant, so the values stay in registers.
__device__ __forceinline__ void tc_store8(void* __restrict__ c, int c_dt, size_t at, int col, int n, bool whole, const float (&v)[8]) {
    if (c_dt == KB_DT_BF16) {
        bf16* dst = static_cast<bf16*>(c) + at;
        if (whole) {
            *reinterpret_cast<uint4*>(dst) = tc_pack8(v);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (col + j < n) dst[j] = __float2bfloat16_rn(v[j]);
        }
    } else {
        float* dst = static_cast<float*>(c) + at;
        if (whole) {
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (col + j < n) dst[j] = v[j];
        }
    }
}

// One warp's share of a 128 x 256 accumulator: its 32 TMEM lanes start at `lanes`, this thread's
// row of C is `row`, the accumulator's first column is column `n0` of C. For the gated unit the
// accumulator's columns 0-127 are gates and 128-255 the matching ups, C is [m, n] with n the unit's
// width, and n0 counts in outputs.
template <int EPI>
__device__ __forceinline__ void tc_epilogue(uint32_t lanes, int row, int n0, void* __restrict__ c, int c_dt, int m, int n, float cap) {
    const bool vec = (c_dt == KB_DT_BF16) ? (n % 8 == 0) : (n % 4 == 0);
    if constexpr (EPI == EPI_GLU_GELU || EPI == EPI_GLU_SILU) {
        for (int c0 = 0; c0 < 128; c0 += 16) {
            if (n0 + c0 >= n) break;                            // the same for the whole warp
            uint32_t g[16], u[16];
            __syncwarp();                                       // lanes that skipped their stores rejoin here
            tc_ld16(lanes + (uint32_t)c0, g);
            tc_ld16(lanes + (uint32_t)(128 + c0), u);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row >= m) continue;
#pragma unroll
            for (int h = 0; h < 16; h += 8) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float x = __uint_as_float(g[h + j]);
                    v[j] = (EPI == EPI_GLU_GELU ? gelu_tanh(x) : silu(x)) * __uint_as_float(u[h + j]);
                }
                const int col = n0 + c0 + h;
                tc_store8(c, c_dt, (size_t)row * n + col, col, n, vec && col + 8 <= n, v);
            }
        }
    } else {
        for (int c0 = 0; c0 < 256; c0 += 32) {
            if (n0 + c0 >= n) break;
            uint32_t r[32];
            __syncwarp();
            tc_ld32(lanes + (uint32_t)c0, r);
            if (row >= m) continue;
#pragma unroll
            for (int h = 0; h < 32; h += 8) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[j] = __uint_as_float(r[h + j]);
                    if (EPI == EPI_SOFTCAP) v[j] = cap * tanhf(v[j] / cap);
                }
                const int col = n0 + c0 + h;
                tc_store8(c, c_dt, (size_t)row * n + col, col, n, vec && col + 8 <= n, v);
            }
        }
    }
}

// TC_STAGES = 4: one block a multiprocessor, for products of about one tile a multiprocessor.
// TC_STAGES = 2: two blocks a multiprocessor, for products of many tiles: while one block stores
// its tile or starts the next, the other keeps the tensor cores busy.
template <int TC_STAGES, int EPI>
__global__ void __launch_bounds__(TC_THREADS, TC_STAGES == 2 ? 2 : 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ c, int c_dt, int m, int n, int k, float cap, int k_tiles_a_split) {
    // k_tiles_a_split > 0: blockIdx.z takes that many k tiles from its multiple on and leaves its
    // sums, float32, in slice blockIdx.z of c [splits, m, n] (few tiles and a long K: see kb_gemm_tcgen05_split)
    extern __shared__ unsigned char tc_smem_raw[];
    // 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + TC_STAGES * TC_STAGE_BYTES);
    uint64_t* empty = full + TC_STAGES;
    uint64_t* accum = empty + TC_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * TC_BM, n0 = blockIdx.y * TC_BN;
    const int k_tiles_all = (k + TC_BK - 1) / TC_BK;
    const int kt0 = k_tiles_a_split > 0 ? (int)blockIdx.z * k_tiles_a_split : 0;
    const int k_tiles = k_tiles_a_split > 0 ? min(k_tiles_a_split, k_tiles_all - kt0) : k_tiles_all;
    if (k_tiles_a_split > 0) c = static_cast<float*>(c) + (size_t)blockIdx.z * m * n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { tc_mbar_init(full + s, 1); tc_mbar_init(empty + s, 1); }
        tc_mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_saddr(tmem_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool failed = false;
    dependent_wait();

    if (warp == 0) {
        if (lane == 0) {
            for (int kt = 0; kt < k_tiles; ++kt) {
                const int s = kt % TC_STAGES;
                if (kt >= TC_STAGES && !tc_mbar_wait(empty + s, (uint32_t)((kt / TC_STAGES) - 1) & 1u)) { failed = true; break; }
                unsigned char* a_dst = smem + s * TC_STAGE_BYTES;
                tc_mbar_expect_tx(full + s, TC_STAGE_BYTES);
                tc_tma_load_2d(a_dst, &map_a, (kt0 + kt) * TC_BK, m0, full + s);
                tc_tma_load_2d(a_dst + TC_A_BYTES, &map_w, (kt0 + kt) * TC_BK, n0, full + s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int kt = 0; kt < k_tiles; ++kt) {
                const int s = kt % TC_STAGES;
                if (!tc_mbar_wait(full + s, (uint32_t)(kt / TC_STAGES) & 1u)) { failed = true; break; }
                tc_fence_after();
                const uint32_t a_addr = tc_saddr(smem + s * TC_STAGE_BYTES);
                const uint64_t adesc = tc_smem_desc(a_addr), bdesc = tc_smem_desc(a_addr + TC_A_BYTES);
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk)            // 32 bytes further into the swizzle atom each step
                    tc_mma(tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), (kt | kk) != 0 ? 1u : 0u);
                tc_commit(empty + s);                               // arrives when these MMAs have read the stage
            }
            if (!failed) tc_commit(accum);                          // arrives when the accumulator is complete
        }
    } else {
        const int quarter = warp & 3;                               // the TMEM lanes this warp may read
        // the same answer in every lane: the TMEM loads below must run with the whole warp together
        if (!__all_sync(0xffffffffu, tc_mbar_wait(accum, 0u))) {
            failed = true;
        } else {
            tc_fence_after();
            tc_epilogue<EPI>(tmem + ((uint32_t)(quarter * 32) << 16), m0 + quarter * 32 + lane, n0, c, c_dt, m, n, cap);
        }
    }
    if (failed) atomicExch(&g_tcgen05_error, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------
// The same product by pairs of blocks (a cluster of two, on the two multiprocessors of a pair):
// tcgen05.mma.cta_group::2 computes a 256 x 256 tile, rows 0-127 accumulated in the first block's
// TMEM and rows 128-255 in the second's. Each block stages its own 128 rows of A and only half of
// the weight tile (128 of its 256 rows), so a k step costs a block 32 KB of shared memory instead
// of 48 KB and the weights cross from L2 half as often.
//   * both blocks' TMA copies complete on the first block's "full" barrier (the copy names that
//     barrier by its address in the cluster's shared window with the block-rank bit cleared);
//   * the first block's warp 1 issues the MMAs for both; tcgen05.commit with a two-block mask
//     arrives on the "empty" barrier of the stage, and at the end on the "accumulator" barrier, in
//     both blocks;
//   * each block's warps 2-5 read their own TMEM and store their own 128 rows;
//   * the blocks meet at a cluster barrier after the barriers are initialised and before TMEM is
//     freed, so neither signals a block that is not there yet or has left.
// With a gated-unit epilogue the weight is a stacked gate|up matrix [2 n, k]: the first block
// stages 128 gate rows and the second the 128 up rows of the same outputs, the accumulator's
// columns 0-127 and 128-255 are then gate and up of one output each, and the epilogue stores
// act(gate) * up, [m, n].
constexpr int TP_BN_HALF = 128;
constexpr int TP_B_BYTES = TP_BN_HALF * TC_BK * 2;             // 16 KB: this block's half of the weight tile
constexpr int TP_STAGE_BYTES = TC_A_BYTES + TP_B_BYTES;        // 32 KB
constexpr int tp_smem_bytes(int stages) { return stages * TP_STAGE_BYTES + 1024 + 256; }
constexpr uint32_t TP_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
constexpr uint32_t TP_PEER_MASK = 0xFEFFFFFFu;                 // clears the bit that tells the two blocks' shared windows apart

__device__ __forceinline__ void tp_tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(tc_saddr(dst)), "l"(map), "r"(bar_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tp_commit_both(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(tc_saddr(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void tp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The kernel is persistent: a cluster walks 256 x 256 tiles (cluster i takes tiles i, i + clusters,
// ...; row tiles are the fast index), each block's TMEM holds two accumulators (512 columns), and
// the epilogue of a tile runs while the MMAs of the next fill the other accumulator. Six stages of
// 32 KB in one block a multiprocessor. An accumulator is free again when the four epilogue warps
// of both blocks have arrived on the first block's "accumulator empty" barrier.
constexpr int TPP_STAGES = 6;
constexpr int TPP_TMEM_COLS = 512;

__device__ __forceinline__ void tp_arrive_on_first(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, 0;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(tc_saddr(bar)) : "memory");
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_pair_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                                    void* __restrict__ c, int c_dt, int m, int n, int k, float cap) {
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + TPP_STAGES * TP_STAGE_BYTES);
    uint64_t* empty = full + TPP_STAGES;
    uint64_t* acc_full = empty + TPP_STAGES;             // [2] accumulator complete (MMA -> both blocks' epilogues)
    uint64_t* acc_empty = acc_full + 2;                  // [2] accumulator read out (both blocks' epilogues -> MMA), first block's
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    constexpr bool glu = EPI == EPI_GLU_GELU || EPI == EPI_GLU_SILU;
    constexpr int tile_cols = glu ? TP_BN_HALF : 2 * TP_BN_HALF;
    const int m_pairs = (m + 2 * TC_BM - 1) / (2 * TC_BM), n_tiles = (n + tile_cols - 1) / tile_cols;
    const int tiles = m_pairs * n_tiles;
    const int cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    const int k_tiles = (k + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TPP_STAGES; ++s) { tc_mbar_init(full + s, 1); tc_mbar_init(empty + s, 1); }
        for (int a = 0; a < 2; ++a) { tc_mbar_init(acc_full + a, 1); tc_mbar_init(acc_empty + a, 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_saddr(tmem_slot)), "r"(TPP_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tp_cluster_sync();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool failed = false;
    dependent_wait();                                       // returns at once after a plain launch

    // A wait on a barrier nobody has arrived at yet passes with parity 1: the waiters that ask for
    // room (the producer for a stage, the MMA lane for an accumulator) start there.
    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int t = cluster; t < tiles && !failed; t += clusters) {
                const int m0 = ((t % m_pairs) * 2 + (int)rank) * TC_BM;
                const int n0 = (t / m_pairs) * tile_cols;
                const int w_row = glu ? (rank == 0 ? n0 : n + n0) : n0 + (int)rank * TP_BN_HALF;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % TPP_STAGES;
                    if (!tc_mbar_wait(empty + s, ((uint32_t)(it / TPP_STAGES) & 1u) ^ 1u)) { failed = true; break; }
                    unsigned char* a_dst = smem + s * TP_STAGE_BYTES;
                    if (rank == 0) tc_mbar_expect_tx(full + s, 2 * TP_STAGE_BYTES);
                    const uint32_t bar = tc_saddr(full + s) & TP_PEER_MASK;
                    tp_tma_load_2d(a_dst, &map_a, kt * TC_BK, m0, bar);
                    tp_tma_load_2d(a_dst + TC_A_BYTES, &map_w, kt * TC_BK, w_row, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            int it = 0, i = 0;
            for (int t = cluster; t < tiles && !failed; t += clusters, ++i) {
                const int acc = i & 1;
                if (!tc_mbar_wait(acc_empty + acc, ((uint32_t)(i >> 1) & 1u) ^ 1u)) { failed = true; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem + (uint32_t)(acc * 256);
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % TPP_STAGES;
                    if (!tc_mbar_wait(full + s, (uint32_t)(it / TPP_STAGES) & 1u)) { failed = true; break; }
                    tc_fence_after();
                    const uint32_t a_addr = tc_saddr(smem + s * TP_STAGE_BYTES);
                    const uint64_t adesc = tc_smem_desc(a_addr), bdesc = tc_smem_desc(a_addr + TC_A_BYTES);
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; ++kk) {
                        const uint32_t accumulate = (kt | kk) != 0 ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                            ::"r"(d_tmem), "l"(adesc + (uint64_t)(kk * 2)), "l"(bdesc + (uint64_t)(kk * 2)), "r"(TP_IDESC), "r"(accumulate) : "memory");
                    }
                    tp_commit_both(empty + s);
                }
                if (!failed) tp_commit_both(acc_full + acc);
            }
        }
    } else {
        const int quarter = warp & 3;
        int i = 0;
        for (int t = cluster; t < tiles; t += clusters, ++i) {
            const int acc = i & 1;
            const int m0 = ((t % m_pairs) * 2 + (int)rank) * TC_BM;
            const int n0 = (t / m_pairs) * tile_cols;
            if (!__all_sync(0xffffffffu, tc_mbar_wait(acc_full + acc, (uint32_t)(i >> 1) & 1u))) { failed = true; break; }
            tc_fence_after();
            tc_epilogue<EPI>(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 256), m0 + quarter * 32 + lane, n0, c, c_dt, m, n, cap);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tp_arrive_on_first(acc_empty + acc);
        }
    }
    if (failed) atomicExch(&g_tcgen05_error, 1);
    tc_fence_before();
    __syncthreads();
    tp_cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TPP_TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------
// Up to 64 rows (decoding): the operands change places. A block owns 128 rows of the weight
// matrix, which are the MMA's M (D^T[128 x NP] = W_tile . X^T), and the few activation rows, padded
// to NP = 16, 32 or 64, are its N. The weights stream through shared memory once, by TMA, four or
// five stages deep in each of two blocks a multiprocessor; work is split over K across blockIdx.y when the weight rows alone give too few
// blocks, and each split leaves float32 partial sums [split, m, n] for the reader to add up.
constexpr int SK2_BM = 128, SK2_BK = 64;
// Stages so that two blocks fit a multiprocessor (about 100 KB each): while one starts or stores its
// results the other streams.
template <int NP> struct Sk2 { static constexpr int STAGES = NP <= 32 ? 5 : 4; };
constexpr int SK2_A_BYTES = SK2_BM * SK2_BK * 2;                 // 16 KB of weights a stage

template <int NP>
__global__ void __launch_bounds__(TC_THREADS, 2)
gemm_skinny_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           void* __restrict__ c, int c_dt, float* __restrict__ partial, int m, int n, int k,
                           int k_tiles_per_split, int epi, float cap KB_TL_PARAM) {
    constexpr int B_BYTES = NP * SK2_BK * 2;
    constexpr int STAGE = SK2_A_BYTES + (B_BYTES < 1024 ? 1024 : B_BYTES);        // stages stay 1024-byte aligned
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NP >> 3) << 17) | ((uint32_t)(SK2_BM >> 4) << 24);
    constexpr int COLS = NP < 32 ? 32 : NP;                                        // TMEM columns: a power of two >= 32
    constexpr int SK2_STAGES = Sk2<NP>::STAGES;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + SK2_STAGES * STAGE);
    uint64_t* empty = full + SK2_STAGES;
    uint64_t* accum = empty + SK2_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * SK2_BM;
    const int split = blockIdx.y;
    const int k_tiles_all = (k + SK2_BK - 1) / SK2_BK;
    const int kt0 = split * k_tiles_per_split;
    const int k_tiles = min(k_tiles_per_split, k_tiles_all - kt0);
    KB_TL_ENTER(gemm, blockIdx.x == 0 && blockIdx.y == 0, 0, n, k);

    if (threadIdx.x == 0) {
        for (int s = 0; s < SK2_STAGES; ++s) { tc_mbar_init(full + s, 1); tc_mbar_init(empty + s, 1); }
        tc_mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();                                        // the barriers stand for every warp
    // The first stages are asked for at once, while TMEM is allocated, each by another thread (the
    // first lanes of the producer warp and of the four epilogue warps): a request keeps its thread
    // for a few hundred clocks. The weights do not depend on the kernel before this one: they are
    // asked for ahead of the wait.
    const int asker = lane != 0 ? -1 : (warp == 0 ? 0 : (warp >= 2 ? warp - 1 : -1));
    if (asker >= 0) {
        for (int kt = asker; kt < k_tiles && kt < SK2_STAGES; kt += 5) {
            tc_mbar_expect_tx(full + kt, SK2_A_BYTES + B_BYTES);
            tc_tma_load_2d(smem + kt * STAGE, &map_w, (kt0 + kt) * SK2_BK, n0, full + kt);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_saddr(tmem_slot)), "r"(COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    dependent_wait();                                       // the activations are the kernel before's to finish
    KB_TL_MARK(gemm, 2, threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0);
    if (asker >= 0) {
        for (int kt = asker; kt < k_tiles && kt < SK2_STAGES; kt += 5)
            tc_tma_load_2d(smem + kt * STAGE + SK2_A_BYTES, &map_x, (kt0 + kt) * SK2_BK, 0, full + kt);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool failed = false;

    if (warp == 0) {
        if (lane == 0) {
            for (int kt = SK2_STAGES; kt < k_tiles; ++kt) {
                const int s = kt % SK2_STAGES;
                if (!tc_mbar_wait(empty + s, (uint32_t)((kt / SK2_STAGES) - 1) & 1u)) { failed = true; break; }
                unsigned char* dst = smem + s * STAGE;
                tc_mbar_expect_tx(full + s, SK2_A_BYTES + B_BYTES);
                tc_tma_load_2d(dst, &map_w, (kt0 + kt) * SK2_BK, n0, full + s);
                tc_tma_load_2d(dst + SK2_A_BYTES, &map_x, (kt0 + kt) * SK2_BK, 0, full + s);
            }
        }
        dependent_trigger();                                // everything this block reads has been asked for
    } else if (warp == 1) {
        if (lane == 0) {
            for (int kt = 0; kt < k_tiles; ++kt) {
                const int s = kt % SK2_STAGES;
                if (!tc_mbar_wait(full + s, (uint32_t)(kt / SK2_STAGES) & 1u)) { failed = true; break; }
                KB_TL_MARK(gemm, 3, kt == 0 && blockIdx.x == 0 && blockIdx.y == 0);          // the first tile has landed
                tc_fence_after();
                const uint32_t a_addr = tc_saddr(smem + s * STAGE);
                const uint64_t adesc = tc_smem_desc(a_addr), bdesc = tc_smem_desc(a_addr + SK2_A_BYTES);
#pragma unroll
                for (int kk = 0; kk < SK2_BK / 16; ++kk) {
                    const uint32_t accumulate = (kt | kk) != 0 ? 1u : 0u;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem), "l"(adesc + (uint64_t)(kk * 2)), "l"(bdesc + (uint64_t)(kk * 2)), "r"(IDESC), "r"(accumulate) : "memory");
                }
                tc_commit(empty + s);
            }
            if (!failed) tc_commit(accum);
        }
        dependent_trigger();
    } else {
        const int quarter = warp & 3;
        const bool complete = __all_sync(0xffffffffu, tc_mbar_wait(accum, 0u));
        KB_TL_MARK(gemm, 4, warp == 2 && lane == 0 && blockIdx.x == 0 && blockIdx.y == 0);     // the sums are done
        dependent_trigger();
        if (!complete) {
            failed = true;
        } else {
            tc_fence_after();
            // lane l of this warp holds output column n0 + 32 quarter + l for every activation row
            const int col = n0 + quarter * 32 + lane;
            float* pdst = partial ? partial + (size_t)split * m * n : nullptr;
#pragma unroll
            for (int c0 = 0; c0 < NP; c0 += 16) {
                uint32_t r[16];
                __syncwarp();
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (col < n && c0 < m) {
                    if (pdst != nullptr) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < m) pdst[(size_t)(c0 + j) * n + col] = __uint_as_float(r[j]);
                    } else {
                        // The soft cap of all sixteen rows is computed whether or not a row exists (a row
                        // beyond m is sums of zeros), so that the rows' instructions interleave; only the
                        // stores ask. One row after the other, the head's epilogue took 85 us at 64 rows.
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            v[j] = __uint_as_float(r[j]);
                            if (epi == 1) v[j] = cap * tanhf(v[j] / cap);
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int row = c0 + j;
                            if (row < m) {
                                if (c_dt == KB_DT_F32) static_cast<float*>(c)[(size_t)row * n + col] = v[j];
                                else static_cast<bf16*>(c)[(size_t)row * n + col] = __float2bfloat16_rn(v[j]);
                            }
                        }
                    }
                }
            }
        }
    }
    if (failed) atomicExch(&g_tcgen05_error, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(COLS) : "memory");
    }
    KB_TL_LEAVE(gemm, blockIdx.x == 0 && blockIdx.y == 0, 64);
}

// ---------------------------------------------------------------------------------------
// Up to 64 rows with the gated unit in the epilogue: the weight is a stacked gate|up matrix
// [2 n, k]. A block owns 64 outputs: its 128 MMA rows are the 64 gate rows and the 64 up rows of
// the same outputs (two TMA boxes a stage), it walks all of K (no split: the gate and the up sums
// must meet in one block), and the epilogue's upper two warps hand their up values to the lower two
// through shared memory, which store act(gate) * up. One block a multiprocessor for Gemma-sized
// units, so the pipeline is deeper than the plain kernel's.
constexpr int SKG_ROWS = 64;                                    // outputs a block
template <int NP> struct SkGlu {
    static constexpr int B_BYTES = NP * SK2_BK * 2;
    static constexpr int STAGE = SK2_A_BYTES + (B_BYTES < 1024 ? 1024 : B_BYTES);
    static constexpr int STAGES = NP <= 16 ? 10 : (NP <= 32 ? 9 : 8);
    static constexpr int XCH_BYTES = SKG_ROWS * NP * 4;         // up values on their way to the gate warps
    static constexpr int SMEM = STAGES * STAGE + XCH_BYTES + 1024 + 256;
};

template <int NP>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_skinny_glu_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                       bf16* __restrict__ c, int m, int n, int k, int act KB_TL_PARAM) {
    using G = SkGlu<NP>;
    constexpr int STAGES = G::STAGES, STAGE = G::STAGE;
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NP >> 3) << 17) | ((uint32_t)(SK2_BM >> 4) << 24);
    constexpr int COLS = NP < 32 ? 32 : NP;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    float* xch = reinterpret_cast<float*>(smem + STAGES * STAGE);                  // [64 outputs][NP rows]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE + G::XCH_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * SKG_ROWS;
    const int k_tiles = (k + SK2_BK - 1) / SK2_BK;
    KB_TL_ENTER(gemm, blockIdx.x == 0, 1, n, k);

    auto load_weights = [&](int kt) {
        const int s = kt % STAGES;
        unsigned char* dst = smem + s * STAGE;
        tc_mbar_expect_tx(full + s, SK2_A_BYTES + G::B_BYTES);
        tc_tma_load_2d(dst, &map_w, kt * SK2_BK, n0, full + s);                           // 64 gate rows
        tc_tma_load_2d(dst + SK2_A_BYTES / 2, &map_w, kt * SK2_BK, n + n0, full + s);     // the same outputs' up rows
    };
    auto load_rows = [&](int kt) { tc_tma_load_2d(smem + (kt % STAGES) * STAGE + SK2_A_BYTES, &map_x, kt * SK2_BK, 0, full + kt % STAGES); };
    auto load_stage = [&](int kt) { load_weights(kt); load_rows(kt); };
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { tc_mbar_init(full + s, 1); tc_mbar_init(empty + s, 1); }
        tc_mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();                                        // the barriers stand for every warp
    // The first stages' tiles are asked for by five threads (the first lanes of the producer warp
    // and of the four epilogue warps), two stages each: a request keeps its thread for a few hundred
    // clocks, and twenty of them in a row by one thread made the block reach its wait 2 to 3 us
    // after the kernel before had finished.
    const int asker = lane != 0 ? -1 : (warp == 0 ? 0 : (warp >= 2 ? warp - 1 : -1));
    if (asker >= 0)
        for (int kt = asker; kt < k_tiles && kt < STAGES; kt += 5) load_weights(kt);     // on their way ahead of the wait
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_saddr(tmem_slot)), "r"(COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    dependent_wait();
    KB_TL_MARK(gemm, 2, threadIdx.x == 0 && blockIdx.x == 0);
    if (asker >= 0)
        for (int kt = asker; kt < k_tiles && kt < STAGES; kt += 5) load_rows(kt);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool failed = false;

    if (warp == 0) {
        if (lane == 0) {
            for (int kt = STAGES; kt < k_tiles; ++kt) {
                if (!tc_mbar_wait(empty + kt % STAGES, (uint32_t)((kt / STAGES) - 1) & 1u)) { failed = true; break; }
                load_stage(kt);
            }
        }
        dependent_trigger();
    } else if (warp == 1) {
        if (lane == 0) {
            for (int kt = 0; kt < k_tiles; ++kt) {
                const int s = kt % STAGES;
                if (!tc_mbar_wait(full + s, (uint32_t)(kt / STAGES) & 1u)) { failed = true; break; }
                KB_TL_MARK(gemm, 3, kt == 0 && blockIdx.x == 0);
                tc_fence_after();
                const uint32_t a_addr = tc_saddr(smem + s * STAGE);
                const uint64_t adesc = tc_smem_desc(a_addr), bdesc = tc_smem_desc(a_addr + SK2_A_BYTES);
#pragma unroll
                for (int kk = 0; kk < SK2_BK / 16; ++kk) {
                    const uint32_t accumulate = (kt | kk) != 0 ? 1u : 0u;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem), "l"(adesc + (uint64_t)(kk * 2)), "l"(bdesc + (uint64_t)(kk * 2)), "r"(IDESC), "r"(accumulate) : "memory");
                }
                tc_commit(empty + s);
            }
            if (!failed) tc_commit(accum);
        }
        dependent_trigger();
    } else {
        const int quarter = warp & 3;                       // TMEM lanes 32 quarter ..: 0, 1 gates; 2, 3 ups
        const bool ok = __all_sync(0xffffffffu, tc_mbar_wait(accum, 0u));
        KB_TL_MARK(gemm, 4, warp == 2 && lane == 0 && blockIdx.x == 0);
        dependent_trigger();
        if (!ok) failed = true;
        const int f = (quarter & 1) * 32 + lane;            // the output within the block's 64
        const bool gates = quarter < 2;
        // The gate warps finish the even rows and the up warps the odd ones: each hands the other,
        // through shared memory, its values of the rows it does not finish. (With the gate warps
        // finishing every row, one after the other, this epilogue took 17 us at 64 rows.)
        float v[NP];
        if (ok) {
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < NP; c0 += 16) {
                uint32_t r[16];
                tc_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) v[c0 + j] = __uint_as_float(r[j]);
            }
#pragma unroll
            for (int j = 0; j < NP; j += 2) {               // a row's 64 outputs side by side
                if (gates) xch[(j + 1) * SKG_ROWS + f] = v[j + 1];
                else xch[j * SKG_ROWS + f] = v[j];
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");      // the four epilogue warps; reached whether or not the wait ran out
        if (ok && n0 + f < n) {
            // Four rows at a time, computed whether or not they exist (a row beyond m is sums of
            // zeros), so that the four activations' instructions interleave; only the stores ask.
#pragma unroll
            for (int j0 = 0; j0 < NP; j0 += 8) {
                if (j0 >= m) break;
                float o[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = j0 + 2 * u;               // the even row; the up warps take the odd one after it
                    const float g = gates ? v[j] : xch[(j + 1) * SKG_ROWS + f];
                    const float up = gates ? xch[j * SKG_ROWS + f] : v[j + 1];
                    o[u] = (act == 0 ? gelu_tanh(g) : silu(g)) * up;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = j0 + 2 * u + (gates ? 0 : 1);
                    if (j < m) c[(size_t)j * n + n0 + f] = __float2bfloat16_rn(o[u]);
                }
            }
        }
    }
    if (failed) atomicExch(&g_tcgen05_error, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(COLS) : "memory");
    }
    KB_TL_LEAVE(gemm, blockIdx.x == 0, 64);
}

template <int NP>
static int launch_skinny_glu(const CUtensorMap& map_w, const CUtensorMap& map_x, bf16* c, int m, int n, int k, int act, cudaStream_t s) {
    static bool attr_set = false;
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_skinny_glu_kernel<NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SkGlu<NP>::SMEM);
        if (e != cudaSuccess) return fail("gemm_skinny_glu: cannot have %d bytes of shared memory: %s", SkGlu<NP>::SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    launch_dependent_if(m <= DEPENDENT_ROWS, gemm_skinny_glu_kernel<NP>, dim3((n + SKG_ROWS - 1) / SKG_ROWS), dim3(TC_THREADS), (size_t)SkGlu<NP>::SMEM, s, map_w, map_x, c, m, n, k, act KB_TL_SLOT(gemm, 1, n, k));
    return check_launch("gemm_skinny_glu");
}

// (splits, k tiles a split) for a weight [n, k]: about two blocks a multiprocessor (one beyond 64
// rows), a split at least four k tiles long. Depends on n, k and on whether there are more than 64 rows.
static void skinny_plan(int n, int k, int sms, int* splits, int* k_tiles_per_split, int m = 1) {
    const int n_tiles = (n + SK2_BM - 1) / SK2_BM;
    const int k_tiles = (k + SK2_BK - 1) / SK2_BK;
    // beyond 64 rows a block fills a multiprocessor's shared memory alone, and the partial sums
    // (rows x columns x splits floats) begin to weigh beside the weights: half as many splits
    int s = ((m <= 64 ? 2 : 1) * sms + n_tiles / 2) / n_tiles;
    const int max_splits = (k_tiles + 3) / 4;
    if (s > max_splits) s = max_splits;
    if (s < 1) s = 1;
    const int per = (k_tiles + s - 1) / s;
    *k_tiles_per_split = per;
    *splits = (k_tiles + per - 1) / per;
}

static int skinny_sms() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

template <int NP>
static int launch_skinny(const CUtensorMap& map_w, const CUtensorMap& map_x, void* c, int c_dt, float* partial, int m, int n,
                         int k, int splits, int per, int epi, float cap, cudaStream_t s) {
    constexpr int B_BYTES = NP * SK2_BK * 2;
    constexpr int STAGE = SK2_A_BYTES + (B_BYTES < 1024 ? 1024 : B_BYTES);
    constexpr int SMEM = Sk2<NP>::STAGES * STAGE + 1024 + 256;
    static bool attr_set = false;
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_skinny_tcgen05_kernel<NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return fail("gemm_skinny: cannot have %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    dim3 grid((n + SK2_BM - 1) / SK2_BM, splits);
    launch_dependent_if(m <= DEPENDENT_ROWS, gemm_skinny_tcgen05_kernel<NP>, grid, dim3(TC_THREADS), (size_t)SMEM, s, map_w, map_x, c, c_dt, splits > 1 ? partial : (float*)nullptr, m, n, k, per, epi, cap KB_TL_SLOT(gemm, 0, n, k));
    return check_launch("gemm_skinny_tcgen05");
}

template <int STAGES, int EPI>
static int launch_single(const CUtensorMap& map_a, const CUtensorMap& map_w, void* c, int c_dt, int m, int n, int k, float cap,
                         dim3 grid, cudaStream_t s, int k_tiles_a_split = 0) {
    static bool attr_set = false;
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes(STAGES));
        if (e != cudaSuccess) return fail("gemm_tcgen05: cannot have %d bytes of shared memory: %s", tc_smem_bytes(STAGES), cudaGetErrorString(e));
        attr_set = true;
    }
    launch_dependent_if(false, gemm_tcgen05_kernel<STAGES, EPI>, grid, dim3(TC_THREADS), (size_t)tc_smem_bytes(STAGES), s, map_a, map_w, c, c_dt, m, n, k, cap, k_tiles_a_split);
    return check_launch("gemm_tcgen05");
}

// n counts output columns (the gated unit's width with a gated epilogue).
template <int EPI>
static int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_w, void* c, int c_dt, int m, int n, int k, float cap,
                       cudaStream_t s) {
    static bool attr_set = false;
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_persistent_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, tp_smem_bytes(TPP_STAGES));
        if (e != cudaSuccess) return fail("gemm_tcgen05_pair: cannot have %d bytes of shared memory: %s", tp_smem_bytes(TPP_STAGES), cudaGetErrorString(e));
        attr_set = true;
    }
    constexpr int tile_cols = (EPI == EPI_GLU_GELU || EPI == EPI_GLU_SILU) ? TP_BN_HALF : 2 * TP_BN_HALF;
    const long long tiles = (long long)((m + 2 * TC_BM - 1) / (2 * TC_BM)) * ((n + tile_cols - 1) / tile_cols);
    const int pairs = skinny_sms() / 2;
    const int clusters = tiles < pairs ? (int)tiles : pairs;
    launch_dependent_if(false, gemm_tcgen05_pair_persistent_kernel<EPI>, dim3(2 * clusters), dim3(TC_THREADS), (size_t)tp_smem_bytes(TPP_STAGES), s, map_a, map_w, c, c_dt, m, n, k, cap);
    return check_launch("gemm_tcgen05_pair");
}

}  // namespace kb

using namespace kb;

KB_TIMELINE_GETTER(gemm)

// 1 if a wait inside the tcgen05 product ever ran out (and clears the flag); synchronises the device.
extern "C" int kb_tcgen05_error() {
    int flag = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&flag, g_tcgen05_error, sizeof(int)) != cudaSuccess) return -1;
    if (flag) cudaMemcpyToSymbol(g_tcgen05_error, &zero, sizeof(int));
    return flag;
}

// Makes a bounded wait run out on purpose, for the test of what follows it: one small block waits
// `limit_clocks` (at most four million: about two milliseconds) on a barrier nobody arrives at,
// raises the flag that kb_tcgen05_error reports and returns; the context stays usable.
extern "C" int kb_wait_probe(long long limit_clocks, void* stream) {
    KB_REQUIRE(limit_clocks > 0 && limit_clocks <= 4000000ll, "wait_probe: a limit of %lld clocks (1 to 4,000,000)", limit_clocks);
    wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit_clocks);
    return check_launch("wait_probe");
}

// a: bf16 [m,k]; w: bf16 [n,k]; c: bf16 or f32 [m,n]. Any m, n; k a multiple of 8.
// kernel: 0 chooses, 1 the one-block kernel, 2 the persistent pair kernel.
extern "C" int kb_gemm_tcgen05(void* c, int c_dt, const void* a, const void* w, int m, int n, int k, int epilogue,
                               float cap, int kernel, void* stream) {
    KB_REQUIRE(m > 0 && n > 0 && k > 0, "gemm_tcgen05: m %d, n %d, k %d", m, n, k);
    KB_REQUIRE(k % 8 == 0, "gemm_tcgen05: k = %d must be a multiple of 8 (16-byte rows)", k);
    KB_REQUIRE(c_dt == KB_DT_F32 || c_dt == KB_DT_BF16, "gemm_tcgen05: output dtype code %d is not known", c_dt);
    KB_REQUIRE(epilogue == 0 || (epilogue == 1 && cap > 0.f), "gemm_tcgen05: epilogue %d with cap %g", epilogue, cap);
    KB_REQUIRE(kernel >= 0 && kernel <= 2, "gemm_tcgen05: kernel choice %d (0 to 2)", kernel);
    KB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)c & 15) == 0, "gemm_tcgen05: operands must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    CUtensorMap map_a, map_w;
    if (int e = encode_map_bf16(&map_a, a, m, k, k, TC_BM)) return e;
    // Row tiles are the fast grid dimension: the blocks of a wave share a few weight tiles (each
    // read from memory once) and what a wave reads again is the activations, small beside L2.
    // Measured on the gate|up product of a 2,048-token prompt: 187 us against 227 us the other way.
    dim3 grid((m + TC_BM - 1) / TC_BM, (n + TC_BN - 1) / TC_BN);
    KB_REQUIRE(grid.y <= 65535, "gemm_tcgen05: %d columns is too many for one launch", n);
    const long long tiles = (long long)grid.x * grid.y;
    // About one 128 x 256 tile a multiprocessor and a short K: pairs would leave half the tiles'
    // worth of multiprocessors idle and there is no second tile whose MMAs could hide an epilogue.
    if (kernel == 0) kernel = (tiles <= 3 * (long long)skinny_sms() / 2 && k <= 4096) ? 1 : 2;
    if (kernel == 2) {
        if (int e = encode_map_bf16(&map_w, w, n, k, k, TP_BN_HALF)) return e;
        return epilogue == 0 ? launch_pair<EPI_NONE>(map_a, map_w, c, c_dt, m, n, k, cap, s)
                             : launch_pair<EPI_SOFTCAP>(map_a, map_w, c, c_dt, m, n, k, cap, s);
    }
    if (int e = encode_map_bf16(&map_w, w, n, k, k, TC_BN)) return e;
    const bool many = tiles > 3 * (long long)skinny_sms() / 2;
    if (epilogue == 0)
        return many ? launch_single<2, EPI_NONE>(map_a, map_w, c, c_dt, m, n, k, cap, grid, s)
                    : launch_single<4, EPI_NONE>(map_a, map_w, c, c_dt, m, n, k, cap, grid, s);
    return many ? launch_single<2, EPI_SOFTCAP>(map_a, map_w, c, c_dt, m, n, k, cap, grid, s)
                : launch_single<4, EPI_SOFTCAP>(map_a, map_w, c, c_dt, m, n, k, cap, grid, s);
}

// How many slices of K `kb_gemm_tcgen05_split` cuts a product of m rows into (1: it is not worth cutting).
// A prompt portion of a few hundred rows by a narrow weight has a handful of 128 x 256 tiles, each
// walking all of K on its own multiprocessor (the way down of Gemma 2 2B at 512 rows: 36 tiles, 50 us);
// cut over K the tiles fill the GPU, at the price of float32 partial sums that the reader adds up.
static void split_plan(int m, int n, int k, int* splits, int* per) {
    const long long tiles = (long long)((m + TC_BM - 1) / TC_BM) * ((n + TC_BN - 1) / TC_BN);
    const int k_tiles = (k + TC_BK - 1) / TC_BK;
    int s = (int)(skinny_sms() / (tiles > 0 ? tiles : 1));
    const int most = k_tiles / 8;                           // a slice is at least eight k tiles (512 of K) long
    if (s > most) s = most;
    if (s > 16) s = 16;
    if (s < 1) s = 1;
    *per = (k_tiles + s - 1) / s;
    *splits = (k_tiles + *per - 1) / *per;
}
extern "C" int kb_gemm_tcgen05_splits(int m, int n, int k) {
    int splits, per;
    split_plan(m, n, k, &splits, &per);
    return splits;
}
// a: bf16 [m,k]; w: bf16 [n,k]; partial: f32 [kb_gemm_tcgen05_splits(m, n, k), m, n], the slices' sums.
extern "C" int kb_gemm_tcgen05_split(float* partial, const void* a, const void* w, int m, int n, int k, void* stream) {
    KB_REQUIRE(m > 0 && n > 0 && k > 0, "gemm_tcgen05_split: m %d, n %d, k %d", m, n, k);
    KB_REQUIRE(k % 8 == 0, "gemm_tcgen05_split: k = %d must be a multiple of 8 (16-byte rows)", k);
    KB_REQUIRE(partial != nullptr && ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)partial & 15) == 0,
               "gemm_tcgen05_split: operands must be there and 16-byte aligned");
    int splits, per;
    split_plan(m, n, k, &splits, &per);
    CUtensorMap map_a, map_w;
    if (int e = encode_map_bf16(&map_a, a, m, k, k, TC_BM)) return e;
    if (int e = encode_map_bf16(&map_w, w, n, k, k, TC_BN)) return e;
    dim3 grid((m + TC_BM - 1) / TC_BM, (n + TC_BN - 1) / TC_BN, splits);
    KB_REQUIRE(grid.y <= 65535, "gemm_tcgen05_split: %d columns is too many for one launch", n);
    return launch_single<4, EPI_NONE>(map_a, map_w, partial, KB_DT_F32, m, n, k, 0.f, grid, (cudaStream_t)stream, per);
}

// The gated unit in the product's epilogue: a bf16 [m,k]; w bf16 [2 n, k], gate rows then up rows;
// c = act(a . gate^T) * (a . up^T), bf16 [m, n]; act 0 gelu_tanh, 1 silu. The gate and the up sums
// meet in 32-bit, before any rounding to bfloat16.
extern "C" int kb_gemm_tcgen05_glu(void* c, const void* a, const void* w, int m, int n, int k, int act, void* stream) {
    KB_REQUIRE(m > 0 && n > 0 && k > 0, "gemm_tcgen05_glu: m %d, n %d, k %d", m, n, k);
    KB_REQUIRE(k % 8 == 0, "gemm_tcgen05_glu: k = %d must be a multiple of 8 (16-byte rows)", k);
    KB_REQUIRE(act == 0 || act == 1, "gemm_tcgen05_glu: activation code %d is not known (0 gelu_tanh, 1 silu)", act);
    KB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)c & 15) == 0, "gemm_tcgen05_glu: operands must be 16-byte aligned");
    CUtensorMap map_a, map_w;
    if (int e = encode_map_bf16(&map_a, a, m, k, k, TC_BM)) return e;
    if (int e = encode_map_bf16(&map_w, w, 2ull * n, k, k, TP_BN_HALF)) return e;
    cudaStream_t s = (cudaStream_t)stream;
    return act == 0 ? launch_pair<EPI_GLU_GELU>(map_a, map_w, c, KB_DT_BF16, m, n, k, 0.f, s)
                    : launch_pair<EPI_GLU_SILU>(map_a, map_w, c, KB_DT_BF16, m, n, k, 0.f, s);
}

// The gated unit for up to 64 rows: a bf16 [m,k]; w bf16 [2 n, k], gate rows then up rows;
// c = act(a . gate^T) * (a . up^T), bf16 [m, n]; act 0 gelu_tanh, 1 silu.
extern "C" int kb_gemm_skinny_glu(void* c, const void* a, const void* w, int m, int n, int k, int act, void* stream) {
    KB_REQUIRE(m > 0 && m <= 64 && n > 0 && k > 0, "gemm_skinny_glu: m %d (1..64), n %d, k %d", m, n, k);
    KB_REQUIRE(k % 8 == 0, "gemm_skinny_glu: k = %d must be a multiple of 8 (16-byte rows)", k);
    KB_REQUIRE(act == 0 || act == 1, "gemm_skinny_glu: activation code %d is not known (0 gelu_tanh, 1 silu)", act);
    KB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_skinny_glu: operands must be 16-byte aligned");
    const int np = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
    CUtensorMap map_w, map_x;
    if (int e = encode_map_bf16(&map_w, w, 2ull * n, k, k, SKG_ROWS)) return e;
    if (int e = encode_map_bf16(&map_x, a, m, k, k, np)) return e;
    cudaStream_t s = (cudaStream_t)stream;
    if (np == 16) return launch_skinny_glu<16>(map_w, map_x, (bf16*)c, m, n, k, act, s);
    if (np == 32) return launch_skinny_glu<32>(map_w, map_x, (bf16*)c, m, n, k, act, s);
    return launch_skinny_glu<64>(map_w, map_x, (bf16*)c, m, n, k, act, s);
}

// Partial sums the skinny kernel leaves for a weight [n, k] and up to 64 rows (1: it writes the result itself).
extern "C" int kb_gemm_skinny_splits(int n, int k) {
    int splits, per;
    skinny_plan(n, k, skinny_sms(), &splits, &per);
    return splits;
}
// The same for m rows (up to 256).
extern "C" int kb_gemm_skinny_splits_for(int m, int n, int k) {
    int splits, per;
    skinny_plan(n, k, skinny_sms(), &splits, &per, m);
    return splits;
}

// a: bf16 [m,k], m <= 64; w: bf16 [n,k]. With one split: c (bf16 or f32 [m,n]) gets the result with
// its epilogue. With more: `partial` (f32 [splits, m, n]) gets the partial sums and c is not touched.
extern "C" int kb_gemm_skinny(void* c, int c_dt, float* partial, const void* a, const void* w, int m, int n, int k,
                              int epilogue, float cap, void* stream) {
    KB_REQUIRE(m > 0 && m <= 256 && n > 0 && k > 0, "gemm_skinny: m %d (1..256), n %d, k %d", m, n, k);
    KB_REQUIRE(k % 8 == 0, "gemm_skinny: k = %d must be a multiple of 8 (16-byte rows)", k);
    KB_REQUIRE(epilogue == 0 || (epilogue == 1 && cap > 0.f), "gemm_skinny: epilogue %d with cap %g", epilogue, cap);
    KB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_skinny: operands must be 16-byte aligned");
    int splits, per;
    skinny_plan(n, k, skinny_sms(), &splits, &per, m);
    KB_REQUIRE(splits == 1 || partial != nullptr, "gemm_skinny: %d splits over K need room for partial sums", splits);
    KB_REQUIRE(splits > 1 || (c != nullptr && (c_dt == KB_DT_F32 || c_dt == KB_DT_BF16)), "gemm_skinny: no output");
    KB_REQUIRE(splits == 1 || epilogue == 0, "gemm_skinny: an epilogue cannot be applied to partial sums");
    const int np = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256)));
    CUtensorMap map_w, map_x;
    if (int e = encode_map_bf16(&map_w, w, n, k, k, SK2_BM)) return e;
    if (int e = encode_map_bf16(&map_x, a, m, k, k, np)) return e;
    cudaStream_t s = (cudaStream_t)stream;
    if (np == 16) return launch_skinny<16>(map_w, map_x, c, c_dt, partial, m, n, k, splits, per, epilogue, cap, s);
    if (np == 32) return launch_skinny<32>(map_w, map_x, c, c_dt, partial, m, n, k, splits, per, epilogue, cap, s);
    if (np == 64) return launch_skinny<64>(map_w, map_x, c, c_dt, partial, m, n, k, splits, per, epilogue, cap, s);
    if (np == 128) return launch_skinny<128>(map_w, map_x, c, c_dt, partial, m, n, k, splits, per, epilogue, cap, s);
    return launch_skinny<256>(map_w, map_x, c, c_dt, partial, m, n, k, splits, per, epilogue, cap, s);
}
