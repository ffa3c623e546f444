// rules.cuh -- device-side rules shared by every kernel of the library: the counter-based random
// streams, the epsilon-greedy choice, the TD arithmetic and the seeded start cells.  One definition,
// so the kernels cannot drift apart.
//
// Reference semantics (paths relative to the CudaRL-Arena project root):
//   TD update   src/kernels.cu:96-114 (true max as in src/gpu/kernels.cu:36-45, src/train.py:134)
//   eps-greedy  src/train.py:101-108, first-max argmax src/q_learning.cu:196-206
//   reset       src/environment.cu:6-14
#pragma once
#include "kernels.cuh"

namespace cudarl {

constexpr unsigned FULL = 0xFFFFFFFFu;

// ------------------------------------------------------------------------------------------------
// Philox4x32-10, counter-based: no generator state is stored anywhere.
struct U4 { unsigned x, y, z, w; };

__device__ __forceinline__ U4 philox4x32_10(unsigned c0, unsigned c1, unsigned c2, unsigned c3,
                                            unsigned k0, unsigned k1) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        unsigned n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return U4{c0, c1, c2, c3};
}

constexpr unsigned TAG_START = 0x53545254u, TAG_QINIT = 0x51494E49u, TAG_POLICY = 0x504F4C49u,
                   TAG_EVAL = 0x4556414Cu;

__device__ __forceinline__ float u01(unsigned w) { return (float)(w >> 8) * 5.9604644775390625e-08f; }

__device__ __forceinline__ unsigned cw_load(const unsigned short* cw, unsigned cell) { return cw[cell]; }

// Start cell of an episode.  CENTRE/FIXED: the configured cell (reference: src/environment.cu:9-10).
// RANDOM: first free non-goal cell among 64 seeded candidates, else the precomputed fallback cell.
__device__ __forceinline__ unsigned sample_start(const Params& p, unsigned gi, unsigned long long nonce, unsigned tag) {
    if (p.start_mode != 2) return p.start_cell;
#pragma unroll 1            // restarts are rare: keep the inlined copies of this loop small (the step kernel's hot loop must fit the instruction cache)
    for (unsigned k = 0; k < 16; ++k) {
        U4 w = philox4x32_10(gi, k, (unsigned)nonce, (unsigned)(nonce >> 32), p.k0, p.k1 ^ tag);
        unsigned c;
        c = __umulhi(w.x, p.S); if (!(cw_load(p.cw, c) & (CW_OBST | CW_GOAL))) return c;
        c = __umulhi(w.y, p.S); if (!(cw_load(p.cw, c) & (CW_OBST | CW_GOAL))) return c;
        c = __umulhi(w.z, p.S); if (!(cw_load(p.cw, c) & (CW_OBST | CW_GOAL))) return c;
        c = __umulhi(w.w, p.S); if (!(cw_load(p.cw, c) & (CW_OBST | CW_GOAL))) return c;
    }
    return p.fallback_start;
}

// Reward of a step that does not end on a goal, for an agent at (x, y) whose action `a` was blocked: the step cost, or -- when
// the cell it walked into is a trap -- that trap's penalty (src/kernels.cu:47,61-63 of the reference: a trap is an obstacle, the
// agent stays where it is and is charged the cell's value).  Binary search in the sparse trap table.
__device__ __forceinline__ float blocked_step_reward(const Params& p, int x, int y, int a) {
    if (!p.ntraps) return -0.01f;
    const int nx = x + (a == 1) - (a == 3), ny = y + (a == 2) - (a == 0);
    if (nx < 0 || nx >= p.W || ny < 0 || ny >= p.H) return -0.01f;
    const unsigned tgt = (unsigned)ny * (unsigned)p.W + (unsigned)nx;
    unsigned lo = 0, hi = p.ntraps;
    while (lo < hi) {
        const unsigned mid = (lo + hi) >> 1;
        const uint2 e = p.traps[mid];
        if (e.x == tgt) return __uint_as_float(e.y);
        if (e.x < tgt) lo = mid + 1u; else hi = mid;
    }
    return -0.01f;
}

__device__ __forceinline__ int argmax4(float4 r) {   // first maximum wins
    int b = 0; float bv = r.x;
    if (r.y > bv) { bv = r.y; b = 1; }
    if (r.z > bv) { bv = r.z; b = 2; }
    if (r.w > bv) { bv = r.w; b = 3; }
    return b;
}
__device__ __forceinline__ float max4(float4 r) {
    float m = r.x;
    m = r.y > m ? r.y : m; m = r.z > m ? r.z : m; m = r.w > m ? r.w : m;
    return m;
}
__device__ __forceinline__ float pick(float4 r, int a) { return a == 0 ? r.x : a == 1 ? r.y : a == 2 ? r.z : r.w; }
// One update of Q[s,a] toward `target`: q <- fma(lr, target - q, q), which is what nvcc makes of the reference's
// `q += lr * (target - q)` (src/kernels.cu:113-114).  Updates of the same (s,a) within a step are applied one
// after the other in ascending environment id, each seeing the value the previous one left (the targets come
// from Q_t), so any number of environments on one cell keeps the step a contraction.
__device__ __forceinline__ void fold(float4& r, int a, float lr, float target) {
    const float q = pick(r, a);
    const float v = __fmaf_rn(lr, __fsub_rn(target, q), q);
    r.x = a == 0 ? v : r.x; r.y = a == 1 ? v : r.y; r.z = a == 2 ? v : r.z; r.w = a == 3 ? v : r.w;
}

}  // namespace cudarl
