// The C entry points of paged attention; the kernels are in attention_rows.cuh.
#include "attention_rows.cuh"

using namespace kb;

extern "C" int kb_attention_chunk() { return ATT_CHUNK; }

// Scratch floats for `slots` chunk slots (0 when slots == 1).
extern "C" long long kb_paged_attention_scratch_floats(int rows, int hq, int d, int slots) {
    return slots > 1 ? (long long)rows * hq * slots * (d + 2) : 0;
}

extern "C" int kb_paged_attention_rows(void* out, const void* q, const void* k_table, const void* v_table, int dt,
                                       const int* block_table, const int* row_entry, const int* row_count, int rows,
                                       int hq, int hkv, int d, int page_size, int table_width, int n_pages, int window,
                                       int slots, float scale, float cap, float* scratch, void* stream) {
    KB_REQUIRE(rows >= 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "paged_attention: rows %d, heads %d over %d kv heads", rows, hq, hkv);
    KB_REQUIRE(d > 0 && d % 16 == 0, "paged_attention: head_dim %d must be a multiple of 16", d);
    KB_REQUIRE(page_size > 0 && table_width > 0 && n_pages > 0, "paged_attention: page_size %d, table width %d, pages %d", page_size, table_width, n_pages);
    KB_REQUIRE(window >= 0 && slots >= 1 && slots <= 65535, "paged_attention: window %d, chunk slots %d", window, slots);
    KB_REQUIRE(cap >= 0.f, "paged_attention: cap %g is negative", cap);
    KB_REQUIRE(slots == 1 || scratch != nullptr, "paged_attention: %d chunk slots need scratch memory", slots);
    KB_REQUIRE(rows <= 0x7fffffff / 1 && (long long)hkv * ((hq / hkv + 7) / 8) <= 65535, "paged_attention: too many heads for one launch");
    if (rows == 0) return 0;
    AttParams p;
    p.q = q; p.k_table = k_table; p.v_table = v_table; p.block_table = block_table; p.row_entry = row_entry;
    p.row_count = row_count; p.out = out; p.partial = slots > 1 ? scratch : nullptr;
    p.rows = rows; p.hq = hq; p.hkv = hkv; p.d = d; p.page_size = page_size; p.table_width = table_width;
    p.n_pages = n_pages; p.window = window; p.slots = slots; p.scale = scale; p.cap = cap;
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == KB_DT_F32) return rows_f32(p, s, slots > 1);
    if (dt == KB_DT_BF16) return rows_bf16(p, s, slots > 1);
    return fail("paged_attention: dtype code %d is not known", dt);
}
