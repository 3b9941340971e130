// The 32-bit instantiations of the row-wise paged attention kernels.
#include "attention_rows.cuh"
namespace kb {
int rows_f32(const AttParams& p, cudaStream_t s, bool combine) { return run_rows<float>(p, s, combine); }
}  // namespace kb
