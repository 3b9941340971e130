// The bfloat16 instantiations of the row-wise paged attention kernels.
#include "attention_rows.cuh"
namespace kb {
int rows_bf16(const AttParams& p, cudaStream_t s, bool combine) { return run_rows<__nv_bfloat16>(p, s, combine); }
}  // namespace kb
