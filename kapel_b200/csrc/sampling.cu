// Choosing tokens where the logits are: the first largest (greedy), or a draw at a temperature.
//
// Rules as Kapel's sampler has them (crates/kapel-infer/src/sampling.rs:190-195,232-260,291-310;
// device argmax kernels/src/lib.rs argmax_rows :2528): the first index on a tie, a NaN never
// unless every value is one; a draw is the first index whose running total of probabilities
// exceeds u, and the last possible index if rounding left u above the total. Softmax in 32-bit
// here (the host sampler of the engine does it in 64-bit).
#include "common.cuh"

namespace kb {

constexpr int SMP_THREADS = 1024;

struct Best { float v; int i; };

__device__ __forceinline__ Best better(Best a, Best b) {
    // larger value wins; on a tie the smaller index; index -1 means "none yet"
    if (b.i < 0) return a;
    if (a.i < 0) return b;
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ Best block_best(Best x, Best* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    Best t;
    t.v = 0.f; t.i = -1;
    if (lane < nwarps) t = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, t.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
        t = better(t, y);
    }
    return t;
}

// One block a row. temperature[r] <= 0 (or temperature == null): argmax.
__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(int* __restrict__ tokens, const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int vocab) {
    __shared__ Best sbest[32];
    __shared__ float sred[32];
    __shared__ float sscan[SMP_THREADS];
    __shared__ int schosen;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const int tid = threadIdx.x;

    Best mine; mine.v = 0.f; mine.i = -1;
    for (int i = tid; i < vocab; i += SMP_THREADS) {
        const float v = row[i];
        if (v != v) continue;
        Best c; c.v = v; c.i = i;
        mine = better(mine, c);
    }
    const Best top = block_best(mine, sbest);
    const float temp = temperature ? temperature[r] : 0.f;
    if (!(temp > 0.f) || top.i < 0) {
        if (tid == 0) tokens[r] = top.i < 0 ? 0 : top.i;
        return;
    }
    // Contiguous ranges so that the running total follows the index order.
    const int per = (vocab + SMP_THREADS - 1) / SMP_THREADS;
    const int begin = min(vocab, tid * per), end = min(vocab, begin + per);
    const float mx = top.v / temp;
    float local = 0.f;
    for (int i = begin; i < end; ++i) {
        const float v = row[i];
        if (v == v) local += expf(v / temp - mx);
    }
    const float total = block_sum(local, sred);
    sscan[tid] = local;
    if (tid == 0) schosen = -1;
    __syncthreads();
    // Exclusive prefix of this thread's range, added in thread order.
    float before = 0.f;
    for (int t = 0; t < tid; ++t) before += sscan[t];
    const float target = uniform[r] * total;
    // The first range whose running total exceeds the target holds the draw.
    if (target >= before && target < before + local) {
        float run = before;
        int pick = -1, last = -1;
        for (int i = begin; i < end; ++i) {
            const float v = row[i];
            if (v != v) continue;
            const float e = expf(v / temp - mx);
            if (e > 0.f) {
                run += e;
                last = i;
                if (target < run) { pick = i; break; }
            }
        }
        // The range's total was added up in another order: if rounding hid the crossing, it is
        // at the range's last possible token.
        if (pick < 0) pick = last;
        if (pick >= 0) atomicCAS(&schosen, -1, pick);
    }
    __syncthreads();
    if (tid == 0) {
        int pick = schosen;
        if (pick < 0) {
            // Rounding left the target above every running total: the last possible token.
            for (int i = vocab - 1; i >= 0; --i) {
                const float v = row[i];
                if (v == v && expf(v / temp - mx) > 0.f) { pick = i; break; }
            }
            if (pick < 0) pick = top.i;
        }
        tokens[r] = pick;
    }
}

}  // namespace kb

using namespace kb;

// Greedy choice of a few rows over a large vocabulary, in two steps: SMP_PARTS blocks a row find the
// first largest value of their share of the columns, then one block a row picks among those (one
// block a row alone read a 1 MB row from one multiprocessor: 12 us at batch 8 against 4).
constexpr int SMP_PARTS = 32;
__global__ void __launch_bounds__(256) argmax_parts_kernel(int2* __restrict__ parts, const float* __restrict__ logits, int vocab) {
    __shared__ Best sbest[32];
    const int r = blockIdx.x, part = blockIdx.y;
    const float* row = logits + (size_t)r * vocab;
    const int per = (vocab + SMP_PARTS - 1) / SMP_PARTS;
    const int begin = min(vocab, part * per), end = min(vocab, begin + per);
    Best mine; mine.v = 0.f; mine.i = -1;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        if (v != v) continue;
        Best c; c.v = v; c.i = i;
        mine = better(mine, c);
    }
    const Best top = block_best(mine, sbest);
    if (threadIdx.x == 0) parts[(size_t)r * SMP_PARTS + part] = make_int2(__float_as_int(top.v), top.i);
}
__global__ void __launch_bounds__(32) argmax_pick_kernel(int* __restrict__ tokens, const int2* __restrict__ parts) {
    const int2 e = parts[(size_t)blockIdx.x * SMP_PARTS + threadIdx.x];
    Best x; x.v = __int_as_float(e.x); x.i = e.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    if (threadIdx.x == 0) tokens[blockIdx.x] = x.i < 0 ? 0 : x.i;
}

// Floats of scratch memory the greedy choice of `rows` rows wants for its two steps (0: one step).
extern "C" long long kb_sample_scratch_floats(int rows, int vocab) {
    return (rows > 0 && rows * SMP_PARTS <= 4096 && vocab >= 65536) ? (long long)rows * SMP_PARTS * 2 : 0;
}

extern "C" int kb_sample(int* tokens, const float* logits, const float* temperature, const float* uniform, int rows,
                         int vocab, float* scratch, void* stream) {
    KB_REQUIRE(rows >= 0 && vocab > 0, "sample: rows %d, vocab %d", rows, vocab);
    KB_REQUIRE(temperature == nullptr || uniform != nullptr, "sample: a temperature needs uniform numbers");
    if (rows == 0) return 0;
    if (temperature == nullptr && scratch != nullptr && kb_sample_scratch_floats(rows, vocab) > 0) {
        int2* parts = reinterpret_cast<int2*>(scratch);
        argmax_parts_kernel<<<dim3(rows, SMP_PARTS), 256, 0, (cudaStream_t)stream>>>(parts, logits, vocab);
        if (int e = check_launch("sample")) return e;
        argmax_pick_kernel<<<rows, 32, 0, (cudaStream_t)stream>>>(tokens, parts);
        return check_launch("sample");
    }
    sample_kernel<<<rows, SMP_THREADS, 0, (cudaStream_t)stream>>>(tokens, logits, temperature, uniform, vocab);
    return check_launch("sample");
}
