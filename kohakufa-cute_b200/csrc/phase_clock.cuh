// Phase timing of one CTA, compiled in only with -DKFA_PHASES (`python build.py --phases` builds such a
// library beside the ordinary one; `python phase_profile.py` runs it and prints the table).
//
// A role declares a clock (PH_DECL), marks the end of each phase of its loop (PH(i), i < 8: the cycles since
// the previous mark are added to phase i) and writes its totals to a slot of a per-translation-unit table
// when it leaves the loop (PH_FLUSH(slot)); only the CTA whose index the host selected does so.  In an
// ordinary build every macro expands to nothing.
#pragma once
#ifdef KFA_PHASES
static __device__ unsigned g_phase[32][8];
static __device__ int g_phase_cta;
struct PhaseClock {
    unsigned last, acc[8];
    __device__ __forceinline__ void start() {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0;
        last = (unsigned)clock();
    }
    __device__ __forceinline__ void mark(int i) {
        const unsigned now = (unsigned)clock();
        acc[i] += now - last;
        last = now;
    }
    __device__ __forceinline__ void flush(int slot) {
        if (blockIdx.x == g_phase_cta)
#pragma unroll
            for (int i = 0; i < 8; ++i) g_phase[slot][i] = acc[i];
    }
};
#define PH_DECL      \
    PhaseClock ph_;  \
    ph_.start()
#define PH(i) ph_.mark(i)
#define PH_FLUSH(slot) ph_.flush(slot)
// Host side of the table of one translation unit: copies it out and selects the CTA for the next launches.
#define KFA_PHASE_EXPORT(name)                                                                        \
    extern "C" __attribute__((visibility("default"))) int name(unsigned* out, int next_cta) {        \
        cudaDeviceSynchronize();                                                                      \
        if (out) cudaMemcpyFromSymbol(out, g_phase, sizeof(unsigned) * 32 * 8);                       \
        return cudaMemcpyToSymbol(g_phase_cta, &next_cta, sizeof(int)) == cudaSuccess ? 0 : 1;         \
    }
#else
#define PH_DECL \
    do {        \
    } while (0)
#define PH(i) \
    do {      \
    } while (0)
#define PH_FLUSH(slot) \
    do {               \
    } while (0)
#define KFA_PHASE_EXPORT(name)
#endif
