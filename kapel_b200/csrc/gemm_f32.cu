// C[M,N] = A[M,K] . W[N,K]^T in true 32-bit: FFMA only, no tensor-core instruction, so nothing
// rounds an input (the 32-bit path of the whole model; Kapel's f32 tiles: crates/kapel-cuda/src/tile.rs:196).
//
// Each output element is one accumulator that takes its K products in ascending k, whatever M
// and N are and wherever the element lies in its tile: the result for a row does not depend on
// which other rows are in the batch.
#include "common.cuh"

namespace kb {

constexpr int F32_BM = 64, F32_BN = 64, F32_BK = 16;

// epilogue 0: none; 1: cap * tanh(acc / cap)
template <int EPI>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ c, const float* __restrict__ a, const float* __restrict__ w, int m, int n, int k,
                float cap) {
    __shared__ float sa[F32_BK][F32_BM + 4];
    __shared__ float sw[F32_BK][F32_BN + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * F32_BM, n0 = blockIdx.x * F32_BN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < k; k0 += F32_BK) {
        // 64 x 16 elements each of A and W: 1024 loads by 256 threads, k fastest.
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 256;
            const int row = e / F32_BK, kk = e % F32_BK;
            const int gm = m0 + row, gn = n0 + row, gk = k0 + kk;
            sa[kk][row] = (gm < m && gk < k) ? a[(size_t)gm * k + gk] : 0.f;
            sw[kk][row] = (gn < n && gk < k) ? w[(size_t)gn * k + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < F32_BK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = sw[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= n) continue;
            float v = acc[i][j];
            if (EPI == 1) v = cap * tanhf(v / cap);
            c[(size_t)gm * n + gn] = v;
        }
    }
}

}  // namespace kb

using namespace kb;

extern "C" int kb_gemm_f32(float* c, const float* a, const float* w, int m, int n, int k, int epilogue, float cap,
                           void* stream) {
    KB_REQUIRE(m >= 0 && n > 0 && k > 0, "gemm_f32: m %d, n %d, k %d", m, n, k);
    KB_REQUIRE(epilogue == 0 || (epilogue == 1 && cap > 0.f), "gemm_f32: epilogue %d with cap %g", epilogue, cap);
    if (m == 0) return 0;
    dim3 grid((n + F32_BN - 1) / F32_BN, (m + F32_BM - 1) / F32_BM);
    KB_REQUIRE(grid.y <= 65535, "gemm_f32: %d rows is too many for one launch", m);
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == 0)
        gemm_f32_kernel<0><<<grid, 256, 0, s>>>(c, a, w, m, n, k, cap);
    else
        gemm_f32_kernel<1><<<grid, 256, 0, s>>>(c, a, w, m, n, k, cap);
    return check_launch("gemm_f32");
}
