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

// A draw of a few rows over a large vocabulary, in two steps as well. First SMP_PARTS blocks a row
// leave, for their share of the columns, the first largest value, its index and the sum of
// exp((v - that value) / temperature). Then one block a row brings the sums to the row's largest
// value, adds them up in the order of the columns, finds the share in which the running total passes
// u x total, and walks that share alone. The rules are sample_kernel's: the first index whose running
// total exceeds the target; where rounding hid the crossing, the share's last possible token; where it
// left the target above every total, the row's last possible token.
struct DrawPart { float top; int index; float sum; int unused; };       // 16 bytes a share

__global__ void __launch_bounds__(256) draw_parts_kernel(DrawPart* __restrict__ parts, const float* __restrict__ logits,
                                                         const float* __restrict__ temperature, int vocab) {
    __shared__ Best sbest[32];
    __shared__ float sred[32];
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
    const float temp = temperature[r];
    float local = 0.f;
    if (temp > 0.f && top.i >= 0 && top.v > -INFINITY) {       // a share of nothing but -inf weighs nothing
        const float mx = top.v / temp;
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {       // the share is in the first-level cache by now
            const float v = row[i];
            if (v == v) local += expf(v / temp - mx);
        }
    }
    const float sum = block_sum(local, sred);
    if (threadIdx.x == 0) {
        DrawPart out;
        out.top = top.v; out.index = top.i; out.sum = sum; out.unused = 0;
        parts[(size_t)r * SMP_PARTS + part] = out;
    }
}

constexpr int DRAW_THREADS = 1024;
__global__ void __launch_bounds__(DRAW_THREADS) draw_pick_kernel(int* __restrict__ tokens, const DrawPart* __restrict__ parts,
                                                                 const float* __restrict__ logits, const float* __restrict__ temperature,
                                                                 const float* __restrict__ uniform, int vocab) {
    __shared__ DrawPart sparts[SMP_PARTS];
    __shared__ float swarp[DRAW_THREADS / 32];
    __shared__ int swinner, spick, slast;
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = logits + (size_t)r * vocab;
    if (tid < SMP_PARTS) sparts[tid] = parts[(size_t)r * SMP_PARTS + tid];
    if (tid == 0) { swinner = DRAW_THREADS; spick = -1; slast = -1; }
    __syncthreads();
    Best top; top.v = 0.f; top.i = -1;
    for (int p = 0; p < SMP_PARTS; ++p) {
        Best c; c.v = sparts[p].top; c.i = sparts[p].index;
        top = better(top, c);
    }
    const float temp = temperature[r];
    if (!(temp > 0.f) || top.i < 0) {
        if (tid == 0) tokens[r] = top.i < 0 ? 0 : top.i;
        return;
    }
    // Every thread adds the shares' sums in the order of the columns: the same total and the same share everywhere.
    const float mx = top.v / temp;
    float total = 0.f;
    for (int p = 0; p < SMP_PARTS; ++p)
        if (sparts[p].index >= 0) total += sparts[p].sum * expf(sparts[p].top / temp - mx);
    const float target = uniform[r] * total;
    int share = -1, last_share = -1;
    float before = 0.f, run = 0.f;
    for (int p = 0; p < SMP_PARTS; ++p) {
        if (sparts[p].index < 0) continue;
        const float w = sparts[p].sum * expf(sparts[p].top / temp - mx);
        if (w > 0.f) last_share = p;
        if (share < 0 && target < run + w) { share = p; before = run; }
        run += w;
    }
    const bool beyond = share < 0;                  // rounding left the target above every running total
    if (beyond) share = last_share;
    if (share < 0) {                                // no share holds a possible token (the row's largest value is infinite)
        if (tid == 0) tokens[r] = top.i;
        return;
    }
    const int per = (vocab + SMP_PARTS - 1) / SMP_PARTS;
    const int sbegin = min(vocab, share * per), send = min(vocab, sbegin + per);
    // Contiguous ranges a thread, so that the running total follows the index order.
    const int each = (send - sbegin + DRAW_THREADS - 1) / DRAW_THREADS;
    const int begin = min(send, sbegin + tid * each), end = min(send, begin + each);
    float local = 0.f;
    int last = -1;
    for (int i = begin; i < end; ++i) {
        const float v = row[i];
        if (v != v) continue;
        const float e = expf(v / temp - mx);
        if (e > 0.f) { local += e; last = i; }
    }
    if (last >= 0) atomicMax(&slast, last);
    // The running total after each thread's range: within a warp by five steps of shuffles, then the
    // warps before it one after the other. Thread t's range of the total is [after(t - 1), after(t)):
    // the ranges leave no gap, and where rounding lets two of them hold the target the first wins.
    float after = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, after, o);
        if (lane >= o) after += y;
    }
    if (lane == 31) swarp[warp] = after;
    __syncthreads();
    float base = before;
    for (int w = 0; w < warp; ++w) base += swarp[w];
    after += base;
    float mine_before = __shfl_up_sync(0xffffffffu, after, 1);
    if (lane == 0) mine_before = base;
    const bool holds = !beyond && target >= mine_before && target < after;
    if (holds) atomicMin(&swinner, tid);
    __syncthreads();
    if (holds && swinner == tid) {
        float walk = mine_before;
        int pick = -1, seen = -1;
        for (int i = begin; i < end; ++i) {
            const float v = row[i];
            if (v != v) continue;
            const float e = expf(v / temp - mx);
            if (e > 0.f) {
                walk += e;
                seen = i;
                if (target < walk) { pick = i; break; }
            }
        }
        if (pick < 0 && seen < 0)                   // rounding gave an empty range a width: the last possible token before it
            for (int i = begin - 1; i >= sbegin; --i) {
                const float v = row[i];
                if (v == v && expf(v / temp - mx) > 0.f) { seen = i; break; }
            }
        spick = pick < 0 ? seen : pick;             // the range's total was added up in another order: its last possible token
    }
    __syncthreads();
    if (tid == 0) {
        int pick = spick;
        if (pick < 0) pick = slast;                 // the crossing hid in rounding, or lay beyond: the share's last possible token
        tokens[r] = pick < 0 ? top.i : pick;
    }
}

// Floats of scratch memory the choice of `rows` rows wants for its two steps (0: one step).
extern "C" long long kb_sample_scratch_floats(int rows, int vocab) {
    return (rows > 0 && rows * SMP_PARTS <= 4096 && vocab >= 65536) ? (long long)rows * SMP_PARTS * 4 : 0;
}

extern "C" int kb_sample(int* tokens, const float* logits, const float* temperature, const float* uniform, int rows,
                         int vocab, float* scratch, void* stream) {
    KB_REQUIRE(rows >= 0 && vocab > 0, "sample: rows %d, vocab %d", rows, vocab);
    KB_REQUIRE(temperature == nullptr || uniform != nullptr, "sample: a temperature needs uniform numbers");
    if (rows == 0) return 0;
    if (scratch != nullptr && kb_sample_scratch_floats(rows, vocab) > 0) {
        KB_REQUIRE(((uintptr_t)scratch & 15) == 0, "sample: the scratch memory must start at a multiple of 16 bytes");
        if (temperature == nullptr) {
            int2* parts = reinterpret_cast<int2*>(scratch);
            argmax_parts_kernel<<<dim3(rows, SMP_PARTS), 256, 0, (cudaStream_t)stream>>>(parts, logits, vocab);
            if (int e = check_launch("sample")) return e;
            argmax_pick_kernel<<<rows, 32, 0, (cudaStream_t)stream>>>(tokens, parts);
            return check_launch("sample");
        }
        DrawPart* parts = reinterpret_cast<DrawPart*>(scratch);
        draw_parts_kernel<<<dim3(rows, SMP_PARTS), 256, 0, (cudaStream_t)stream>>>(parts, logits, temperature, vocab);
        if (int e = check_launch("sample")) return e;
        draw_pick_kernel<<<rows, DRAW_THREADS, 0, (cudaStream_t)stream>>>(tokens, parts, logits, temperature, uniform, vocab);
        return check_launch("sample");
    }
    sample_kernel<<<rows, SMP_THREADS, 0, (cudaStream_t)stream>>>(tokens, logits, temperature, uniform, vocab);
    return check_launch("sample");
}
