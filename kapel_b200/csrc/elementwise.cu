// Embedding rows, rotary tables, rotation fused with the cache append, gated activations, casts.
//
// Counterparts in Kapel's thread kernels (kernels/src/lib.rs): gather_rows :1145 and affine_any
// :1328 (here one kernel), rope_table :1092, rope_any :1545 and write_rows_any :1579 (here one
// kernel), glu_any :2489, widen_16/narrow_16 :375,386.
#include "common.cuh"
#include "timeline.cuh"

namespace kb {

KB_TIMELINE_ARRAY(elementwise) // slots: kind 3 rotation and append (rows, slices)


// ---------------------------------------------------------------------------------------
// x[r, :] = table[ids[r], :] * scale, in 32-bit. An id outside the table gives a row of NaN.
template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                             int rows, int width, int vocab, float scale) {
    const int r = blockIdx.x;
    if (r >= rows) return;
    const int id = ids[r];
    float* o = out + (size_t)r * width;
    if (id < 0 || id >= vocab) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = __int_as_float(0x7fc00000);
        return;
    }
    const T* t = table + (size_t)id * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = Elem<T>::load(t + i) * scale;
}

// ---------------------------------------------------------------------------------------
// cos_sin[r, j] = (cos, sin)(positions[r] * theta^(-2j / rotary)), angle in 64-bit.
__global__ void rope_table_kernel(float2* __restrict__ cos_sin, const int* __restrict__ positions, int rows,
                                  int half, int rotary, double theta) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * half) return;
    const int r = i / half, j = i % half;
    const double w = pow(theta, -(2.0 * (double)j) / (double)rotary);
    const double a = (double)positions[r] * w;
    double s, c;
    sincos(a, &s, &c);
    cos_sin[i] = make_float2((float)c, (float)s);
}

// ---------------------------------------------------------------------------------------
// One thread a pair of components of one head vector of one row of the stacked q|k|v product.
// Heads [0, Hq) are queries (rotated, written to q_out), [Hq, Hq+Hkv) keys (rotated, written to
// the key table at the row's line), [Hq+Hkv, Hq+2Hkv) values (copied to the value table). The
// tables are [pages, Hkv, page_size, D]; a line is page * page_size + offset.
// Pairing "half": (j, j + rotary/2) for j < rotary/2; components from `rotary` on pass through.
// A row whose line is negative writes no key and no value (a padding row).
template <typename TI, typename T>
__global__ void rope_append_kernel(const Src<TI> qkv, const float2* __restrict__ cos_sin,
                                   const int* __restrict__ lines, T* __restrict__ q_out, T* __restrict__ k_table,
                                   T* __restrict__ v_table, int rows, int hq, int hkv, int d, int rotary,
                                   int write_kv, long long table_lines, int page_size KB_TL_PARAM) {
    const int half_d = d >> 1, half_r = rotary >> 1;
    const int heads = hq + 2 * hkv;
    const long long total = (long long)rows * heads * half_d;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    KB_TL_ENTER(elementwise, blockIdx.x == 0, 3, rows, qkv.splits);
    dependent_wait();
    KB_TL_MARK(elementwise, 2, threadIdx.x == 0 && blockIdx.x == 0);
    dependent_trigger();
    if (idx >= total) return;
    const int i = (int)(idx % half_d);
    const int h = (int)((idx / half_d) % heads);
    const int r = (int)(idx / ((long long)half_d * heads));
    const size_t src = ((size_t)r * heads + h) * d;
    int ia, ib;
    bool rotate;
    if (i < half_r) {
        ia = i; ib = i + half_r; rotate = true;
    } else {
        ia = rotary + 2 * (i - half_r); ib = ia + 1; rotate = false;
    }
    if (h >= hq && !write_kv) return;
    if (h >= hq + hkv) rotate = false;                      // a value
    // Everything this thread reads is asked for before anything is looked at, the line of the cache
    // included: one trip to memory, where a test of the line first made it two.
    float a = qkv.at(src + ia), b = qkv.at(src + ib);
    const float2 cs = rotate ? cos_sin[(size_t)r * half_r + i] : make_float2(1.f, 0.f);
    const int line = h >= hq ? lines[r] : 0;
    T* dst;
    if (h < hq) {
        dst = q_out + ((size_t)r * hq + h) * d;
    } else {
        if (line < 0 || line >= table_lines) return;
        const bool is_key = h < hq + hkv;
        const int kvh = is_key ? h - hq : h - hq - hkv;
        dst = (is_key ? k_table : v_table) + kv_row(line, kvh, hkv, page_size) * d;
    }
    if (rotate) rope_rotate(a, b, cs);
    Elem<T>::store(dst + ia, a);
    Elem<T>::store(dst + ib, b);
    KB_TL_LEAVE(elementwise, blockIdx.x == 0, 0);           // thread 0 of block 0 rotates a query: it never left early
}

// The same over float32 split sums for a decode step, with the slices brought into shared memory by
// bulk copies instead of the threads' loads: what the product before has just written arrives much
// sooner that way (see add_rmsnorm_splits_bulk_kernel). A block of 256 threads owns 256 pairs, which
// are 256 / (d / 2) whole heads of one row: 512 consecutive values of each slice, one copy a slice.
// The sums are added in slice order, as Src::at adds them.
__device__ int g_rope_error = 0;
template <typename T>
__global__ void __launch_bounds__(256) rope_append_bulk_kernel(const float* __restrict__ parts, int splits, size_t stride,
                                                               const float2* __restrict__ cos_sin, const int* __restrict__ lines,
                                                               T* __restrict__ q_out, T* __restrict__ k_table, T* __restrict__ v_table,
                                                               int rows, int hq, int hkv, int d, int rotary, int write_kv,
                                                               long long table_lines, int page_size KB_TL_PARAM) {
    extern __shared__ __align__(128) unsigned char rb_smem[];
    __shared__ __align__(8) uint64_t landed;
    float* vals = reinterpret_cast<float*>(rb_smem);        // [splits][512]
    const int half_d = d >> 1, half_r = rotary >> 1;
    const int heads = hq + 2 * hkv;
    const int blocks_a_row = heads * half_d / 256;
    const int r = blockIdx.x / blocks_a_row, seg = blockIdx.x % blocks_a_row;
    const int heads_a_block = 256 / half_d;
    const int h0 = seg * heads_a_block;
    KB_TL_ENTER(elementwise, blockIdx.x == 0, 3, rows, splits);
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&landed);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int h = h0 + (int)threadIdx.x / half_d, i = (int)threadIdx.x % half_d;
    int ia, ib;
    bool rotate;
    if (i < half_r) {
        ia = i; ib = i + half_r; rotate = true;
    } else {
        ia = rotary + 2 * (i - half_r); ib = ia + 1; rotate = false;
    }
    if (h >= hq + hkv) rotate = false;                      // a value
    __syncthreads();
    dependent_wait();
    KB_TL_MARK(elementwise, 2, threadIdx.x == 0 && blockIdx.x == 0);
    dependent_trigger();
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2048u * (uint32_t)splits) : "memory");
        const float* src = parts + ((size_t)r * heads + h0) * d;
        for (int s = 0; s < splits; ++s)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"((uint32_t)__cvta_generic_to_shared(vals + s * 512)), "l"(src + (size_t)s * stride), "r"(2048u), "r"(bar) : "memory");
    }
    // the angle and the cache line come by ordinary loads while the copies are on their way (in the
    // first layer the table of angles is the work of the kernel just before: not ahead of the wait)
    const float2 cs = rotate ? cos_sin[(size_t)r * half_r + i] : make_float2(1.f, 0.f);
    const int line = (h >= hq && write_kv) ? lines[r] : 0;  // a layer that writes no line is given no lines
    bool ok = false;
    {
        const long long start = clock64();
        for (;;) {
            uint32_t done;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(0u) : "memory");
            if (done) { ok = true; break; }
            if (clock64() - start > 2000000000ll) break;    // about a second: a copy never landed
        }
    }
    if (!ok) {
        if (threadIdx.x == 0) atomicExch(&g_rope_error, 1);
        return;
    }
    if (h >= hq && !write_kv) return;
    const int local = (h - h0) * d;
    float a = vals[local + ia], b = vals[local + ib];
    for (int s = 1; s < splits; ++s) {
        a += vals[s * 512 + local + ia];
        b += vals[s * 512 + local + ib];
    }
    T* dst;
    if (h < hq) {
        dst = q_out + ((size_t)r * hq + h) * d;
    } else {
        if (line < 0 || line >= table_lines) return;
        const bool is_key = h < hq + hkv;
        const int kvh = is_key ? h - hq : h - hq - hkv;
        dst = (is_key ? k_table : v_table) + kv_row(line, kvh, hkv, page_size) * d;
    }
    if (rotate) rope_rotate(a, b, cs);
    Elem<T>::store(dst + ia, a);
    Elem<T>::store(dst + ib, b);
    KB_TL_LEAVE(elementwise, blockIdx.x == 0, 0);
}

// The same for bfloat16 in and out with the whole head rotated (rotary == d, d a multiple of 16):
// one thread takes eight components of the first half and their eight partners of the second, with
// 16-byte loads and stores.
__global__ void rope_append_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, const float2* __restrict__ cos_sin,
                                          const int* __restrict__ lines, __nv_bfloat16* __restrict__ q_out,
                                          __nv_bfloat16* __restrict__ k_table, __nv_bfloat16* __restrict__ v_table, int rows,
                                          int hq, int hkv, int d, int write_kv, long long table_lines, int page_size) {
    const int half_d = d >> 1, cpr = half_d >> 3;           // chunks of eight in half a head
    const int heads = hq + 2 * hkv;
    const long long total = (long long)rows * heads * cpr;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    dependent_wait();
    dependent_trigger();
    if (idx >= total) return;
    const int c = (int)(idx % cpr);
    const int h = (int)((idx / cpr) % heads);
    const int r = (int)(idx / ((long long)cpr * heads));
    const __nv_bfloat16* src = qkv + ((size_t)r * heads + h) * d + c * 8;
    __nv_bfloat16* dst;
    bool rotate = true;
    if (h < hq) {
        dst = q_out + ((size_t)r * hq + h) * d;
    } else {
        if (!write_kv) return;
        const int line = lines[r];
        if (line < 0 || line >= table_lines) return;
        const bool is_key = h < hq + hkv;
        const int kvh = is_key ? h - hq : h - hq - hkv;
        dst = (is_key ? k_table : v_table) + kv_row(line, kvh, hkv, page_size) * d;
        rotate = is_key;
    }
    uint4 ua = *reinterpret_cast<const uint4*>(src);
    uint4 ub = *reinterpret_cast<const uint4*>(src + half_d);
    if (rotate) {
        const float4* cs4 = reinterpret_cast<const float4*>(cos_sin + (size_t)r * half_d + c * 8);
        __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&ua);
        __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&ub);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 cs = cs4[j];                       // (cos, sin) of two neighbouring components
            float2 a = __bfloat1622float2(pa[j]), b = __bfloat1622float2(pb[j]);
            rope_rotate(a.x, b.x, make_float2(cs.x, cs.y));
            rope_rotate(a.y, b.y, make_float2(cs.z, cs.w));
            pa[j] = __floats2bfloat162_rn(a.x, a.y);
            pb[j] = __floats2bfloat162_rn(b.x, b.y);
        }
    }
    *reinterpret_cast<uint4*>(dst + c * 8) = ua;
    *reinterpret_cast<uint4*>(dst + half_d + c * 8) = ub;
}

// ---------------------------------------------------------------------------------------
// out[r, i] = act(x[r, i]) * x[r, n + i]: the gated unit after a stacked gate|up product.
template <typename TI, typename T>
__global__ void glu_kernel(T* __restrict__ out, const Src<TI> x, long long rows, int n, int act) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * n) return;
    const long long r = idx / n;
    const int i = (int)(idx % n);
    const float g = x.at(r * 2 * n + i), u = x.at(r * 2 * n + n + i);
    const float a = act == 0 ? gelu_tanh(g) : silu(g);
    Elem<T>::store(out + idx, a * u);
}

// The same for bfloat16 in and out with n a multiple of 8: 16 bytes of gate, 16 of up, 16 out a thread.
__global__ void glu_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, long long rows,
                                  int n, int act) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_row = n >> 3;
    if (idx >= rows * per_row) return;
    const long long r = idx / per_row;
    const int i = (int)(idx - r * per_row) << 3;
    const uint4 gv = *reinterpret_cast<const uint4*>(x + r * 2 * n + i);
    const uint4 uv = *reinterpret_cast<const uint4*>(x + r * 2 * n + n + i);
    const uint32_t g4[4] = {gv.x, gv.y, gv.z, gv.w}, u4[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t o4[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float g0 = __uint_as_float(g4[k] << 16), g1 = __uint_as_float(g4[k] & 0xffff0000u);
        const float u0 = __uint_as_float(u4[k] << 16), u1 = __uint_as_float(u4[k] & 0xffff0000u);
        const float a0 = act == 0 ? gelu_tanh(g0) : silu(g0), a1 = act == 0 ? gelu_tanh(g1) : silu(g1);
        __nv_bfloat162 p = __floats2bfloat162_rn(a0 * u0, a1 * u1);
        o4[k] = *reinterpret_cast<uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(out + r * n + i) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
}

template <typename TO, typename TI>
__global__ void cast_kernel(TO* __restrict__ out, const TI* __restrict__ in, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) Elem<TO>::store(out + i, Elem<TI>::load(in + i));
}

// rows wanted: out[i, :] = x[rows[i], :]
__global__ void gather_rows_f32_kernel(float* __restrict__ out, const float* __restrict__ x,
                                       const int* __restrict__ rows, int n, int width, int src_rows) {
    const int i = blockIdx.x;
    if (i >= n) return;
    const int r = rows[i];
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        out[(size_t)i * width + c] = (r >= 0 && r < src_rows) ? x[(size_t)r * width + c] : __int_as_float(0x7fc00000);
}

// table[rows[i], :] = value for the rows listed; a row outside the table is skipped.
__global__ void fill_rows_f32_kernel(float* __restrict__ table, const int* __restrict__ rows, int n, long long width,
                                     int table_rows, float value) {
    const int r = rows[blockIdx.y];
    if (r < 0 || r >= table_rows) return;
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c < width) table[(size_t)r * width + c] = value;
}

// x[i] = value
__global__ void fill_u32_kernel(unsigned* __restrict__ x, long long n, unsigned value) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = value;
}
__global__ void fill_u16_kernel(unsigned short* __restrict__ x, long long n, unsigned short value) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = value;
}

}  // namespace kb

using namespace kb;
typedef __nv_bfloat16 bf16;

// table [table_rows, width] float32: the rows named in `rows` (n of them, on the device) become `value`.
extern "C" int kb_fill_rows_f32(float* table, const int* rows, int n, long long width, int table_rows, float value, void* stream) {
    KB_REQUIRE(n >= 0 && width >= 0 && table_rows >= 0, "fill_rows: n %d, width %lld, table rows %d", n, width, table_rows);
    if (n == 0 || width == 0) return 0;
    KB_REQUIRE(n <= 65535 && (width + 255) / 256 < (1ll << 31), "fill_rows: %d rows of %lld is too many for one launch", n, width);
    fill_rows_f32_kernel<<<dim3((unsigned)((width + 255) / 256), n), 256, 0, (cudaStream_t)stream>>>(table, rows, n, width, table_rows, value);
    return check_launch("fill_rows");
}

// Every element of a float32 (dt 0) or bfloat16 (dt 1) buffer becomes NaN: what a debugging run
// puts into fresh buffers so that a kernel that reads what nobody wrote shows in the result.
extern "C" int kb_poison(void* x, int dt, long long n, void* stream) {
    KB_REQUIRE(n >= 0, "poison: %lld elements", n);
    if (n == 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    KB_REQUIRE((n + 255) / 256 < (1ll << 31), "poison: %lld elements is too many for one launch", n);
    if (dt == KB_DT_F32) fill_u32_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((unsigned*)x, n, 0x7fc00000u);
    else if (dt == KB_DT_BF16) fill_u16_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((unsigned short*)x, n, (unsigned short)0x7fc0);
    else return fail("poison: dtype code %d is not known", dt);
    return check_launch("poison");
}

extern "C" int kb_embed(float* out, const void* table, int table_dt, const int* ids, int rows, int width,
                        int vocab, float scale, void* stream) {
    KB_REQUIRE(rows >= 0 && width > 0 && vocab > 0, "embed: rows %d, width %d, vocab %d", rows, width, vocab);
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dt == KB_DT_F32)
        embed_kernel<float><<<rows, threads, 0, s>>>(out, (const float*)table, ids, rows, width, vocab, scale);
    else if (table_dt == KB_DT_BF16)
        embed_kernel<bf16><<<rows, threads, 0, s>>>(out, (const bf16*)table, ids, rows, width, vocab, scale);
    else
        return fail("embed: table dtype code %d is not known", table_dt);
    return check_launch("embed");
}

extern "C" int kb_rope_table(float* cos_sin, const int* positions, int rows, int rotary, double theta,
                             void* stream) {
    KB_REQUIRE(rows >= 0 && rotary > 0 && rotary % 2 == 0, "rope_table: rows %d, rotary %d (must be even)", rows, rotary);
    KB_REQUIRE(theta > 0, "rope_table: theta %g must be positive", theta);
    if (rows == 0) return 0;
    const int half = rotary / 2;
    const long long n = (long long)rows * half;
    KB_REQUIRE(n < (1ll << 31), "rope_table: %lld entries is too many", n);
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((float2*)cos_sin, positions, rows,
                                                                                  half, rotary, theta);
    return check_launch("rope_table");
}

KB_TIMELINE_GETTER(elementwise)

// 1 if a wait inside the rotation kernel ever ran out (and clears the flag); synchronises the device.
extern "C" int kb_rope_error() {
    int flag = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&flag, g_rope_error, sizeof(int)) != cudaSuccess) return -1;
    if (flag) cudaMemcpyToSymbol(g_rope_error, &zero, sizeof(int));
    return flag;
}

// qkv: `in_dt` (float32 or bfloat16), as `splits` slices `split_stride` elements apart that are
// added up on the way in; q_out and the tables: `out_dt`.
extern "C" int kb_rope_append(const void* qkv, int in_dt, int splits, long long split_stride, const float* cos_sin,
                              const int* lines, void* q_out, void* k_table, void* v_table, int out_dt, int rows,
                              int hq, int hkv, int d, int rotary, int write_kv, long long table_lines, int page_size,
                              void* stream) {
    KB_REQUIRE(rows >= 0 && hq > 0 && hkv > 0 && d > 0 && d % 2 == 0, "rope_append: rows %d, heads %d/%d, head_dim %d", rows, hq, hkv, d);
    KB_REQUIRE(rotary >= 0 && rotary <= d && rotary % 2 == 0, "rope_append: rotary %d must be even and at most head_dim %d", rotary, d);
    KB_REQUIRE(splits >= 1, "rope_append: %d slices", splits);
    KB_REQUIRE(!write_kv || page_size > 0, "rope_append: page_size %d", page_size);
    if (rows == 0) return 0;
    const long long total = (long long)rows * (hq + 2 * hkv) * (d / 2);
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
#define KB_ROPE(TI, T)                                                                                              \
    launch_dependent_if(rows <= DEPENDENT_ROWS, rope_append_kernel<TI, T>, dim3(blocks), dim3(256), 0, s, Src<TI>{(const TI*)qkv, splits, (size_t)split_stride}, \
                     (const float2*)cos_sin, lines, (T*)q_out, (T*)k_table, (T*)v_table, rows, hq, hkv, d, rotary, write_kv,       \
                     table_lines, page_size > 0 ? page_size : 1 KB_TL_SLOT(elementwise, 3, rows, splits))
    const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_table | (uintptr_t)v_table | (uintptr_t)cos_sin) & 15) == 0;
    if (in_dt == KB_DT_BF16 && out_dt == KB_DT_BF16 && splits == 1 && rotary == d && d % 16 == 0 && aligned) {
        const long long vec = (long long)rows * (hq + 2 * hkv) * (d / 16);
        launch_dependent_if(rows <= DEPENDENT_ROWS, rope_append_bf16x8_kernel, dim3((unsigned)((vec + 255) / 256)), dim3(256), 0, s,
            (const bf16*)qkv, (const float2*)cos_sin, lines, (bf16*)q_out, (bf16*)k_table, (bf16*)v_table, rows, hq, hkv, d,
            write_kv, table_lines, page_size > 0 ? page_size : 1);
    }
    else if (in_dt == KB_DT_F32 && out_dt == KB_DT_BF16 && splits > 1 && rows <= DEPENDENT_ROWS && d % 4 == 0 && 256 % (d / 2) == 0 &&
             ((hq + 2 * hkv) * (d / 2)) % 256 == 0 && splits <= 32 && (split_stride % 4) == 0 && (((uintptr_t)qkv) & 15) == 0) {
        // a decode step's split sums: the slices come into shared memory by bulk copies (2 KB a slice and block)
        static bool attr_set = false;
        if (!attr_set) {
            if (cudaFuncSetAttribute(rope_append_bulk_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 2048) != cudaSuccess)
                return fail("rope_append: cannot have 64 KB of shared memory");
            attr_set = true;
        }
        launch_dependent_if(true, rope_append_bulk_kernel<bf16>, dim3(blocks), dim3(256), (size_t)splits * 2048, s, (const float*)qkv, splits,
                            (size_t)split_stride, (const float2*)cos_sin, lines, (bf16*)q_out, (bf16*)k_table, (bf16*)v_table, rows, hq, hkv, d,
                            rotary, write_kv, table_lines, page_size > 0 ? page_size : 1 KB_TL_SLOT(elementwise, 3, rows, splits));
    }
    else if (in_dt == KB_DT_F32 && out_dt == KB_DT_F32) KB_ROPE(float, float);
    else if (in_dt == KB_DT_F32 && out_dt == KB_DT_BF16) KB_ROPE(float, bf16);
    else if (in_dt == KB_DT_BF16 && out_dt == KB_DT_BF16) KB_ROPE(bf16, bf16);
    else return fail("rope_append: dtype codes %d -> %d are not known", in_dt, out_dt);
#undef KB_ROPE
    return check_launch("rope_append");
}

extern "C" int kb_glu(void* out, int out_dt, const void* x, int in_dt, int splits, long long split_stride,
                      long long rows, int n, int act, void* stream) {
    KB_REQUIRE(rows >= 0 && n > 0, "glu: rows %lld, width %d", rows, n);
    KB_REQUIRE(act == 0 || act == 1, "glu: activation code %d is not known (0 gelu_tanh, 1 silu)", act);
    KB_REQUIRE(splits >= 1, "glu: %d slices", splits);
    if (rows == 0) return 0;
    const long long total = rows * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
#define KB_GLU(TI, T) \
    glu_kernel<TI, T><<<blocks, 256, 0, s>>>((T*)out, Src<TI>{(const TI*)x, splits, (size_t)split_stride}, rows, n, act)
    if (in_dt == KB_DT_BF16 && out_dt == KB_DT_BF16 && splits == 1 && n % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const long long vec = rows * (n / 8);
        glu_bf16x8_kernel<<<(unsigned)((vec + 255) / 256), 256, 0, s>>>((bf16*)out, (const bf16*)x, rows, n, act);
    }
    else if (in_dt == KB_DT_F32 && out_dt == KB_DT_F32) KB_GLU(float, float);
    else if (in_dt == KB_DT_F32 && out_dt == KB_DT_BF16) KB_GLU(float, bf16);
    else if (in_dt == KB_DT_BF16 && out_dt == KB_DT_BF16) KB_GLU(bf16, bf16);
    else return fail("glu: dtype codes %d -> %d are not known", in_dt, out_dt);
#undef KB_GLU
    return check_launch("glu");
}

extern "C" int kb_cast(void* out, int out_dt, const void* in, int in_dt, long long n, void* stream) {
    KB_REQUIRE(n >= 0, "cast: %lld elements", n);
    if (n == 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dt == KB_DT_F32 && in_dt == KB_DT_BF16)
        cast_kernel<float, bf16><<<blocks, 256, 0, s>>>((float*)out, (const bf16*)in, n);
    else if (out_dt == KB_DT_BF16 && in_dt == KB_DT_F32)
        cast_kernel<bf16, float><<<blocks, 256, 0, s>>>((bf16*)out, (const float*)in, n);
    else if (out_dt == KB_DT_F32 && in_dt == KB_DT_F32)
        cast_kernel<float, float><<<blocks, 256, 0, s>>>((float*)out, (const float*)in, n);
    else if (out_dt == KB_DT_BF16 && in_dt == KB_DT_BF16)
        cast_kernel<bf16, bf16><<<blocks, 256, 0, s>>>((bf16*)out, (const bf16*)in, n);
    else
        return fail("cast: dtype codes %d -> %d are not known", in_dt, out_dt);
    return check_launch("cast");
}

extern "C" int kb_gather_rows_f32(float* out, const float* x, const int* rows, int n, int width, int src_rows,
                                  void* stream) {
    KB_REQUIRE(n >= 0 && width > 0, "gather_rows: n %d, width %d", n, width);
    if (n == 0) return 0;
    gather_rows_f32_kernel<<<n, 256, 0, (cudaStream_t)stream>>>(out, x, rows, n, width, src_rows);
    return check_launch("gather_rows");
}
