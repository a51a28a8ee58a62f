// PCG32 (O'Neill's pcg32: 64-bit LCG state, XSH-RR output), seeded and consumed as the reference does
// (runtime/prng.c:10-70), so that a given (seed, stream) yields the reference's draws.  Host code only.
#pragma once
#include <cstdint>

namespace tb {

struct Pcg32 {
    uint64_t state, inc;
    uint32_t next() {
        const uint64_t old = state;
        state = old * 6364136223846793005ull + inc;
        const uint32_t x = (uint32_t)(((old >> 18u) ^ old) >> 27u);
        const uint32_t rot = (uint32_t)(old >> 59u);
        return (x >> rot) | (x << ((32u - rot) & 31u));
    }
    Pcg32(uint64_t seed, uint64_t seq) : state(0), inc((seq << 1u) | 1u) {
        next();
        state += seed;
        next();
    }
    uint64_t next64() {
        const uint64_t hi = next();
        const uint64_t lo = next();
        return (hi << 32) | lo;
    }
    // [0, 1): pcg_uniform (runtime/prng.c:34-37)
    double uniform() { return (double)next() * (1.0 / 4294967296.0); }
    // unbiased draw from [lo, hi): 64-bit values below (2^64 - range) mod range are rejected
    // (runtime/prng.c:51-70)
    int64_t range(int64_t lo, int64_t hi) {
        const uint64_t r = (uint64_t)(hi - lo);
        if (r == 0) return lo;
        const uint64_t threshold = (0 - r) % r;
        uint64_t v;
        do v = next64(); while (v < threshold);
        return lo + (int64_t)(v % r);
    }
};

}  // namespace tb
