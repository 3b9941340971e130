// cuTensorMapEncodeTiled, found through the runtime so that the library does not link the driver.
#include "common.cuh"
#include "tensor_map.cuh"

namespace kb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static int find_encoder() {
    if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult res;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &res);
        if (e != cudaSuccess || fn == nullptr || res != cudaDriverEntryPointSuccess)
            return fail("tensor map: the driver does not give cuTensorMapEncodeTiled (%s)", cudaGetErrorString(e));
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    return 0;
}

int encode_map_bf16_chunks(CUtensorMap* map, const void* base, unsigned long long rows, unsigned cols, unsigned box_rows,
                           unsigned box_chunks) {
    if (int e = find_encoder()) return e;
    if (((uintptr_t)base & 15) != 0 || cols % 64 != 0 || cols == 0)
        return fail("tensor map: base %p must be a multiple of 16 and %u columns a multiple of 64", base, cols);
    const cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128u};
    if (box_chunks == 0) box_chunks = cols / 64;
    if (box_chunks > cols / 64) return fail("tensor map: %u chunks a box of a matrix that has %u", box_chunks, cols / 64);
    const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)box_chunks};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("tensor map: cuTensorMapEncodeTiled failed with code %d for [%llu, %u] in chunks", (int)r, rows, cols);
    return 0;
}

int encode_map_bf16(CUtensorMap* map, const void* base, unsigned long long rows, unsigned long long cols,
                    unsigned long long pitch_elems, unsigned box_rows) {
    if (int e = find_encoder()) return e;
    if (((uintptr_t)base & 15) != 0 || (pitch_elems * 2) % 16 != 0)
        return fail("tensor map: base %p and row pitch %llu bytes must be multiples of 16", base, pitch_elems * 2);
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch_elems * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("tensor map: cuTensorMapEncodeTiled failed with code %d for [%llu, %llu]", (int)r, rows, cols);
    return 0;
}

}  // namespace kb
