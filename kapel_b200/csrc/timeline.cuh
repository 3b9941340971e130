// Time stamps inside the kernels of a decoding step, for the question no launch list answers: where
// a step's time goes BETWEEN and INSIDE kernels that overlap one another (a kernel launched as a
// programmatic dependent sets up while the one before it still runs). Compiled in only when the
// library is built with KAPEL_B200_TIMELINE=1 (-DKB_TIMELINE); otherwise every macro here is empty
// and the kernels are what they are without it. `python -m kapel_b200.step_timeline` builds such a
// library in a folder of its own, runs a few decode steps and prints the last step's stamps in order.
//
// A translation unit that stamps declares `KB_TIMELINE_ARRAY(name)` inside namespace kb and
// `KB_TIMELINE_GETTER(name)` at file scope. A kernel's launches share a slot by what they compute
// (the host gives a product [n, k] the same slot every time: `timeline_slot`), so the stamps left at
// the end are those of the last launch of each kind: with two layers, the last layer's.
// Fields of a slot: 0 last block enters, 1 block 0 enters, 2 block 0 is past its wait on the kernel
// before, 3 and 4 two marks of the kernel's choosing, 5 last block leaves, 6 block 0 leaves,
// 7 to 9 three numbers that say what the launch was (kind, n, k).
#pragma once

#define KB_TL_SLOTS 16
#define KB_TL_FIELDS 10

namespace kb {
// The slot of (kind, a, b) among this translation unit's launches, in order of first use; -1 when full.
struct TimelineSlots {
    int n = 0;
    int kind[KB_TL_SLOTS], a[KB_TL_SLOTS], b[KB_TL_SLOTS];
    int of(int kind_, int a_, int b_) {
        for (int i = 0; i < n; ++i)
            if (kind[i] == kind_ && a[i] == a_ && b[i] == b_) return i;
        if (n == KB_TL_SLOTS) return -1;
        kind[n] = kind_; a[n] = a_; b[n] = b_;
        return n++;
    }
};
}  // namespace kb

#ifdef KB_TIMELINE
#define KB_TIMELINE_ARRAY(tu)                                                   \
    __device__ unsigned long long g_timeline_##tu[KB_TL_SLOTS][KB_TL_FIELDS];   \
    static TimelineSlots g_timeline_slots_##tu;
#define KB_TIMELINE_GETTER(tu)                                                                                      \
    extern "C" int kb_timeline_##tu(unsigned long long* out) {                                                      \
        return cudaMemcpyFromSymbol(out, kb::g_timeline_##tu, sizeof(kb::g_timeline_##tu)) == cudaSuccess ? KB_TL_SLOTS : -1; \
    }
#define KB_TL_PARAM , const int tl_slot
#define KB_TL_SLOT(tu, kind, a, b) , kb::g_timeline_slots_##tu.of(kind, a, b)
namespace kb {
__device__ __forceinline__ unsigned long long timeline_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
}  // namespace kb
#define KB_TL_ENTER(tu, first, kind, a, b)                                                          \
    do {                                                                                            \
        if (threadIdx.x == 0 && tl_slot >= 0) {                                                     \
            const unsigned long long t_ = kb::timeline_now();                                       \
            atomicMax(&kb::g_timeline_##tu[tl_slot][0], t_);                                        \
            if (first) {                                                                            \
                kb::g_timeline_##tu[tl_slot][1] = t_;                                               \
                kb::g_timeline_##tu[tl_slot][7] = (unsigned long long)(kind);                       \
                kb::g_timeline_##tu[tl_slot][8] = (unsigned long long)(a);                          \
                kb::g_timeline_##tu[tl_slot][9] = (unsigned long long)(b);                          \
            }                                                                                       \
        }                                                                                           \
    } while (0)
#define KB_TL_MARK(tu, field, cond)                                                                 \
    do {                                                                                            \
        if ((cond) && tl_slot >= 0) kb::g_timeline_##tu[tl_slot][field] = kb::timeline_now();       \
    } while (0)
#define KB_TL_LEAVE(tu, first, thread)                                                              \
    do {                                                                                            \
        if (threadIdx.x == (thread) && tl_slot >= 0) {                                              \
            const unsigned long long t_ = kb::timeline_now();                                       \
            atomicMax(&kb::g_timeline_##tu[tl_slot][5], t_);                                        \
            if (first) kb::g_timeline_##tu[tl_slot][6] = t_;                                        \
        }                                                                                           \
    } while (0)
#else
#define KB_TIMELINE_ARRAY(tu)
#define KB_TIMELINE_GETTER(tu) \
    extern "C" int kb_timeline_##tu(unsigned long long*) { return 0; }
#define KB_TL_PARAM
#define KB_TL_SLOT(tu, kind, a, b)
#define KB_TL_ENTER(tu, first, kind, a, b) do { } while (0)
#define KB_TL_MARK(tu, field, cond) do { } while (0)
#define KB_TL_LEAVE(tu, first, thread) do { } while (0)
#endif
