// kernels.cu -- hand-written sm_100a kernels of the batched grid-world + tabular Q-learning path.
//
// Data layout in HBM (per context = per GPU):
//   x[N], y[N], t[N]   int32 structure-of-arrays environment state, read/written fully coalesced;
//   Q                  one 32-byte sector per grid cell: two float4 halves.  Half `PAR(cell)` holds
//                      Q_t[cell][0..3] (one vector load = the whole action row), the other half is
//                      where Q_{t+1} of that cell is written.  Readers of step t therefore never see
//                      a write of step t, and a 16-byte row costs the same DRAM sector as 32 bytes;
//   ci                 one info byte per cell (obstacle, goal, row parity, occupancy of this and
//                      of the next step), small enough to live in L2;
//   ent / mailbox      collision entries and hashed chain heads for cells that hold several
//                      environments in one step.
//
// One batched step = two launches:
//   train_main  one thread per environment: epsilon-greedy from a Philox4x32-10 stream keyed by
//               (seed, global env, step) -> move with obstacle/goal lookup -> TD error against Q_t
//               -> if the environment is alone on its cell, write the cell's Q_{t+1} row directly;
//               otherwise append (cell, action, env, td_error) to the collision list -> auto-reset
//               -> announce its next cell in the occupancy bits of the next step.
//   train_fix   folds the collision entries of each shared cell in ascending environment index
//               (fp32 fma chain, no float atomics), flips the row parity of every occupied cell,
//               shifts next-step occupancy into place and advances the step / epsilon index.
//
// Reference semantics (paths relative to the CudaRL-Arena project root):
//   step        src/environment.cu:17-48, obstacle test src/kernels.cu:29-44, goal src/kernels.cu:56-59
//   reset       src/environment.cu:6-14
//   TD update   src/kernels.cu:96-114 (true max as in src/gpu/kernels.cu:36-45, src/train.py:134)
//   eps-greedy  src/train.py:101-108, first-max argmax src/q_learning.cu:196-206
//   episode     src/train.py:191-222
#include "kernels.cuh"
#include <cstdio>

namespace cudarl {

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

__device__ __forceinline__ unsigned ci_load(const unsigned char* ci, unsigned cell) { return ci[cell]; }

// Start cell of an episode.  CENTRE/FIXED: the configured cell (reference: src/environment.cu:9-10).
// RANDOM: first free non-goal cell among 64 seeded candidates, else the precomputed fallback cell.
__device__ __forceinline__ unsigned sample_start(const Params& p, unsigned gi, unsigned long long nonce, unsigned tag) {
    if (p.start_mode != 2) return p.start_cell;
    for (unsigned k = 0; k < 16; ++k) {
        U4 w = philox4x32_10(gi, k, (unsigned)nonce, (unsigned)(nonce >> 32), p.k0, p.k1 ^ tag);
        unsigned c;
        c = __umulhi(w.x, p.S); if (!(ci_load(p.ci, c) & (CI_OBST | CI_GOAL))) return c;
        c = __umulhi(w.y, p.S); if (!(ci_load(p.ci, c) & (CI_OBST | CI_GOAL))) return c;
        c = __umulhi(w.z, p.S); if (!(ci_load(p.ci, c) & (CI_OBST | CI_GOAL))) return c;
        c = __umulhi(w.w, p.S); if (!(ci_load(p.ci, c) & (CI_OBST | CI_GOAL))) return c;
    }
    return p.fallback_start;
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
__device__ __forceinline__ void fold(float4& r, int a, float lr, float d) {
    // Q[s,a] <- fma(lr, d, Q[s,a]): what nvcc makes of `q += lr * (target - q)` (src/kernels.cu:114)
    if (a == 0) r.x = __fmaf_rn(lr, d, r.x); else if (a == 1) r.y = __fmaf_rn(lr, d, r.y);
    else if (a == 2) r.z = __fmaf_rn(lr, d, r.z); else r.w = __fmaf_rn(lr, d, r.w);
}

// Move from (x,y) by `action`; returns the new cell and its info byte.
__device__ __forceinline__ unsigned move_cell(const Params& p, int x, int y, unsigned s, unsigned ci_s, int action,
                                              unsigned& ci_new) {
    int dx = (action == 1) - (action == 3), dy = (action == 2) - (action == 0);
    int nx = x + dx, ny = y + dy;
    bool inb = nx >= 0 && nx < p.W && ny >= 0 && ny < p.H;
    unsigned tgt = inb ? (unsigned)ny * (unsigned)p.W + (unsigned)nx : s;
    unsigned ct = (tgt != s) ? ci_load(p.ci, tgt) : ci_s;
    bool moved = (tgt != s) && !(ct & CI_OBST);
    ci_new = moved ? ct : ci_s;
    return moved ? tgt : s;
}

__device__ __forceinline__ void announce(unsigned char* ci, unsigned cell, unsigned occ_bit, unsigned multi_bit) {
    unsigned* w = reinterpret_cast<unsigned*>(ci) + (cell >> 2);
    unsigned sh = (cell & 3u) * 8u;
    unsigned old = atomicOr(w, occ_bit << sh);
    if (old & (occ_bit << sh)) atomicOr(w, multi_bit << sh);
}

__device__ __forceinline__ unsigned mb_slot(const Params& p, unsigned cell) { return (cell * 0x9E3779B1u) >> p.mb_shift; }

// ------------------------------------------------------------------------------------------------
// Occupancy rebuild (after reset / caller-driven state changes): clear the dynamic bits, then every
// environment announces its current cell in the CURRENT-step bits.
__global__ void k_occ_clear(Params p) {
    unsigned n16 = (p.S + 15u) / 16u;
    uint4* w = reinterpret_cast<uint4*>(p.ci);
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += gridDim.x * blockDim.x) {
        uint4 v = w[i];
        const unsigned keep = 0x07070707u;
        v.x &= keep; v.y &= keep; v.z &= keep; v.w &= keep;
        w[i] = v;
    }
}
__global__ void k_occ_announce(Params p) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    unsigned s = (unsigned)p.y[i] * (unsigned)p.W + (unsigned)p.x[i];
    announce(p.ci, s, CI_OCC, CI_MULTI);
}

__global__ void k_reset_all(Params p) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    unsigned c = sample_start(p, p.env_offset + i, p.ctl->step, TAG_START);
    p.x[i] = (int)(c % (unsigned)p.W); p.y[i] = (int)(c / (unsigned)p.W); p.t[i] = 0;
    if (p.reward) { p.reward[i] = 0.0f; p.done[i] = 0; }
}

// ------------------------------------------------------------------------------------------------
// The fused step: one thread per environment.
template <bool TRACE>
__global__ void __launch_bounds__(BLOCK) k_train_main(Params p) {
    __shared__ unsigned s_cnt, s_goals, s_timeouts;
    if (threadIdx.x == 0) { s_cnt = 0; s_goals = 0; s_timeouts = 0; }
    __syncthreads();
    const unsigned i = blockIdx.x * BLOCK + threadIdx.x;
    if (blockIdx.x == 0 && threadIdx.x == 0) p.ctl->scratch_cursor = 0;   // nobody reads it in this kernel
    if (i < p.N) {
        const unsigned long long g = p.ctl->step;
        const float eps = p.eps_tab[p.ctl->eps_idx];
        const int x = __ldcs(p.x + i), y = __ldcs(p.y + i), t = __ldcs(p.t + i);
        const unsigned s = (unsigned)y * (unsigned)p.W + (unsigned)x;
        const unsigned gi = p.env_offset + i;
        const unsigned cs = ci_load(p.ci, s);
        const unsigned par = (cs & CI_PAR) ? 1u : 0u;
        float4 row = __ldcg(p.Q + 2u * s + par);
        // epsilon-greedy
        U4 w = philox4x32_10(gi, 0u, (unsigned)g, (unsigned)(g >> 32), p.k0, p.k1 ^ TAG_POLICY);
        const int a = (u01(w.x) < eps) ? (int)(w.y & 3u) : argmax4(row);
        // environment transition
        unsigned c2;
        const unsigned s2 = move_cell(p, x, y, s, cs, a, c2);
        const bool done = (c2 & CI_GOAL) != 0;
        const float r = done ? 1.0f : -0.01f;
        float m = 0.0f;
        if (!done) {
            float4 row2 = (s2 == s) ? row : __ldcg(p.Q + 2u * s2 + ((c2 & CI_PAR) ? 1u : 0u));
            m = max4(row2);
            if (p.legacy_clamp && m < 0.0f) m = 0.0f;
        }
        const float target = __fmaf_rn(p.gamma, m, r);
        const float d = __fsub_rn(target, pick(row, a));
        if (!(cs & CI_MULTI)) {
            fold(row, a, p.lr, d);
            p.Q[2u * s + (par ^ 1u)] = row;          // Q_{t+1} row of a cell with a single occupant
        } else {
            unsigned rk = atomicAdd(&s_cnt, 1u);
            unsigned pos = blockIdx.x * BLOCK + rk;  // entry slot inside this block's fixed segment
            unsigned slot = mb_slot(p, s);
            unsigned prev = atomicExch(p.mailbox + slot, pos + 1u);
            p.ent[pos] = make_uint4((s << 3) | (par << 2) | (unsigned)a, i, __float_as_uint(d), prev);
        }
        if (TRACE) { p.tr_a[i] = a; p.tr_r[i] = r; p.tr_d[i] = done ? 1 : 0; }
        // episode bookkeeping + next-step occupancy
        const bool timeout = p.max_steps > 0 && t + 1 >= p.max_steps;
        int nx, ny, nt; unsigned sn;
        if (done || timeout) {
            sn = sample_start(p, gi, g + 1ull, TAG_START);
            nx = (int)(sn % (unsigned)p.W); ny = (int)(sn / (unsigned)p.W); nt = 0;
            if (done) atomicAdd(&s_goals, 1u); else atomicAdd(&s_timeouts, 1u);
        } else {
            sn = s2; nx = (int)(s2 % (unsigned)p.W); ny = (int)(s2 / (unsigned)p.W); nt = t + 1;
        }
        announce(p.ci, sn, CI_OCCN, CI_MULTIN);
        __stcs(p.x + i, nx); __stcs(p.y + i, ny); __stcs(p.t + i, nt);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_cnt) atomicAdd(&p.ctl->conflicts, (unsigned long long)s_cnt);
        if (s_goals) atomicAdd(&p.ctl->goals, (unsigned long long)s_goals);
        if (s_timeouts) atomicAdd(&p.ctl->timeouts, (unsigned long long)s_timeouts);
        if (s_goals + s_timeouts) atomicAdd(&p.ctl->episodes, (unsigned long long)(s_goals + s_timeouts));
    }
}

// ------------------------------------------------------------------------------------------------
// Collision folding.
__device__ __forceinline__ void cswap(unsigned long long& ka, float& va, unsigned long long& kb, float& vb) {
    if (ka > kb) { unsigned long long tk = ka; ka = kb; kb = tk; float tv = va; va = vb; vb = tv; }
}

// Block-wide bitonic sort of n2 (power of two) key/value pairs in shared or global memory.
__device__ void block_bitonic(unsigned long long* keys, float* vals, unsigned n2) {
    for (unsigned k = 2; k <= n2; k <<= 1) {
        for (unsigned j = k >> 1; j > 0; j >>= 1) {
            for (unsigned i = threadIdx.x; i < n2; i += blockDim.x) {
                unsigned ixj = i ^ j;
                if (ixj > i) {
                    unsigned long long a = keys[i], b = keys[ixj];
                    bool up = (i & k) == 0;
                    if ((a > b) == up) { keys[i] = b; keys[ixj] = a; float t = vals[i]; vals[i] = vals[ixj]; vals[ixj] = t; }
                }
            }
            __syncthreads();
        }
    }
}

// Fold a sorted run (same cell) starting at index j of keys/vals; returns nothing, writes Q_{t+1}.
template <bool FLIP>
__device__ void apply_run(const Params& p, const unsigned long long* keys, const float* vals, unsigned j, unsigned n) {
    unsigned w0 = (unsigned)(keys[j] >> 32);
    unsigned cellp = w0 >> 2;              // (cell << 1) | parity
    unsigned cell = w0 >> 3, par = (w0 >> 2) & 1u;
    float4 row = __ldcg(p.Q + 2u * cell + par);
    for (; j < n; ++j) {
        unsigned wj = (unsigned)(keys[j] >> 32);
        if ((wj >> 2) != cellp) break;
        fold(row, (int)(wj & 3u), p.lr, vals[j]);
    }
    p.Q[2u * cell + (par ^ 1u)] = row;
    if (FLIP) atomicXor(reinterpret_cast<unsigned*>(p.ci) + (cell >> 2), CI_PAR << ((cell & 3u) * 8u));
}

constexpr unsigned LONG_SMEM = 1024;   // chain entries sorted in shared memory; longer chains use the global scratch
constexpr int SHORT_MAX = 8;           // chain entries folded in registers by one thread

template <bool FLIP>
__device__ void process_long(const Params& p, unsigned head1, unsigned long long* s_keys, float* s_vals,
                             unsigned* s_bcast) {
    // thread 0 walks the chain (pointer chase through L2), everyone sorts, run leaders fold.
    if (threadIdx.x == 0) {
        unsigned q = head1, L = 0;
        while (q && L <= p.ent_cap) {            // a chain can never be longer than the entry array
            uint4 e = p.ent[q - 1u];
            if (L < LONG_SMEM) { s_keys[L] = ((unsigned long long)e.x << 32) | e.y; s_vals[L] = __uint_as_float(e.z); }
            ++L; q = e.w;
        }
        unsigned n2 = 1; while (n2 < L) n2 <<= 1;
        unsigned base = 0xFFFFFFFFu;
        if (q) { atomicOr(&p.ctl->error, ERR_CHAIN_CYCLE); base = 0xFFFFFFFEu; }
        else if (L > LONG_SMEM) {
            base = atomicAdd(&p.ctl->scratch_cursor, n2);
            if (base + n2 > p.sc_cap) { atomicOr(&p.ctl->error, ERR_SCRATCH_OVERFLOW); base = 0xFFFFFFFEu; }
            else {
                q = head1; unsigned k = 0;
                while (q && k < L) {
                    uint4 e = p.ent[q - 1u];
                    p.sc_key[base + k] = ((unsigned long long)e.x << 32) | e.y; p.sc_val[base + k] = __uint_as_float(e.z);
                    ++k; q = e.w;
                }
            }
        }
        s_bcast[0] = L; s_bcast[1] = n2; s_bcast[2] = base;
    }
    __syncthreads();
    const unsigned L = s_bcast[0], n2 = s_bcast[1], base = s_bcast[2];
    if (base != 0xFFFFFFFEu) {
        unsigned long long* keys = (base == 0xFFFFFFFFu) ? s_keys : p.sc_key + base;
        float* vals = (base == 0xFFFFFFFFu) ? s_vals : p.sc_val + base;
        for (unsigned i = L + threadIdx.x; i < n2; i += blockDim.x) { keys[i] = ~0ull; vals[i] = 0.0f; }
        __syncthreads();
        block_bitonic(keys, vals, n2);
        for (unsigned j = threadIdx.x; j < L; j += blockDim.x) {
            unsigned cp = (unsigned)(keys[j] >> 34);
            if (j == 0 || (unsigned)(keys[j - 1] >> 34) != cp) apply_run<FLIP>(p, keys, vals, j, L);
        }
    }
    __syncthreads();
}

constexpr unsigned MED_MAX = 32;                         // chain entries ranked by one warp with shuffles
constexpr unsigned MED_CHUNKS = LONG_SMEM / MED_MAX;     // medium chains a block can stage in shared memory

// One warp orders a staged chain of L <= 32 entries by (cell, action, index) with a shuffle ranking
// (indices are unique, so ranks are a permutation), then the first lane of every cell run folds it.
template <bool FLIP>
__device__ void process_medium(const Params& p, unsigned long long* keys, float* vals, unsigned L) {
    const unsigned lane = threadIdx.x & 31u;
    unsigned long long key = lane < L ? keys[lane] : ~0ull;
    float val = lane < L ? vals[lane] : 0.0f;
    unsigned rank = 0;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        unsigned long long other = __shfl_sync(0xFFFFFFFFu, key, k);
        rank += (other < key) ? 1u : 0u;
    }
    __syncwarp();
    if (lane < L) { keys[rank] = key; vals[rank] = val; }
    __syncwarp();
    if (lane < L) {
        unsigned cp = (unsigned)(keys[lane] >> 34);
        if (lane == 0 || (unsigned)(keys[lane - 1] >> 34) != cp) apply_run<FLIP>(p, keys, vals, lane, L);
    }
    __syncwarp();
}

// Collision folding, one thread per mailbox slot.  A slot's chain holds every entry whose cell hashes
// there; the thread that finds a non-empty slot owns the chain:
//   <= 8 entries   gathered, ordered (sorting network) and folded in registers by that thread;
//   <= 32 entries  staged in shared memory by that thread, ordered and folded by one warp;
//   longer         walked by one thread, sorted by the whole block (shared memory up to 1024 entries,
//                  the global scratch beyond that).
// TRAIN = true : part of a train step -- also sweeps the info bytes (parity ^= occupied, next-step
//                occupancy -> current) and, in the last block to finish, advances step and epsilon.
// TRAIN = false: update_batch -- flips the row parity of every folded cell instead.
template <bool TRAIN>
__global__ void __launch_bounds__(BLOCK) k_fix(Params p) {
    constexpr bool FLIP = !TRAIN;
    __shared__ unsigned long long s_keys[LONG_SMEM];
    __shared__ float s_vals[LONG_SMEM];
    __shared__ unsigned s_long[BLOCK];
    __shared__ unsigned s_medlen[MED_CHUNKS];
    __shared__ unsigned s_nlong, s_nmed, s_bcast[3];
    __shared__ bool s_last;
    if (threadIdx.x == 0) { s_nlong = 0; s_nmed = 0; }
    __syncthreads();
    const unsigned slot = blockIdx.x * BLOCK + threadIdx.x;
    const unsigned head1 = slot < p.mb_slots ? p.mailbox[slot] : 0u;
    if (head1) {
        p.mailbox[slot] = 0u;                          // leave the mailbox empty for the next step
        unsigned long long k[SHORT_MAX]; float v[SHORT_MAX];
        unsigned q = head1;
#pragma unroll
        for (int j = 0; j < SHORT_MAX; ++j) {
            if (q) {
                uint4 e = __ldcg(p.ent + (q - 1u));
                k[j] = ((unsigned long long)e.x << 32) | e.y; v[j] = __uint_as_float(e.z); q = e.w;
            } else { k[j] = ~0ull; v[j] = 0.0f; }
        }
        if (q) {
            unsigned chunk = atomicAdd(&s_nmed, 1u);
            bool staged = false;
            if (chunk < MED_CHUNKS) {
                unsigned long long* mk = s_keys + chunk * MED_MAX; float* mv = s_vals + chunk * MED_MAX;
#pragma unroll
                for (int j = 0; j < SHORT_MAX; ++j) { mk[j] = k[j]; mv[j] = v[j]; }
                unsigned L = SHORT_MAX;
                while (q && L < MED_MAX) {
                    uint4 e = __ldcg(p.ent + (q - 1u));
                    mk[L] = ((unsigned long long)e.x << 32) | e.y; mv[L] = __uint_as_float(e.z); q = e.w; ++L;
                }
                staged = (q == 0u);
                s_medlen[chunk] = staged ? L : 0u;
            }
            if (!staged) { unsigned li = atomicAdd(&s_nlong, 1u); s_long[li] = head1; }
        } else {
            // sorting network for 8 (19 comparators)
            cswap(k[0],v[0],k[1],v[1]); cswap(k[2],v[2],k[3],v[3]); cswap(k[4],v[4],k[5],v[5]); cswap(k[6],v[6],k[7],v[7]);
            cswap(k[0],v[0],k[2],v[2]); cswap(k[1],v[1],k[3],v[3]); cswap(k[4],v[4],k[6],v[6]); cswap(k[5],v[5],k[7],v[7]);
            cswap(k[1],v[1],k[2],v[2]); cswap(k[5],v[5],k[6],v[6]); cswap(k[0],v[0],k[4],v[4]); cswap(k[3],v[3],k[7],v[7]);
            cswap(k[1],v[1],k[5],v[5]); cswap(k[2],v[2],k[6],v[6]);
            cswap(k[1],v[1],k[4],v[4]); cswap(k[3],v[3],k[6],v[6]);
            cswap(k[2],v[2],k[4],v[4]); cswap(k[3],v[3],k[5],v[5]);
            cswap(k[3],v[3],k[4],v[4]);
            unsigned curcp = 0xFFFFFFFFu; float4 row = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < SHORT_MAX; ++j) {
                if (k[j] != ~0ull) {
                    unsigned w0 = (unsigned)(k[j] >> 32), cp = w0 >> 2;
                    if (cp != curcp) {
                        if (curcp != 0xFFFFFFFFu) {
                            unsigned cell = curcp >> 1, par = curcp & 1u;
                            p.Q[2u * cell + (par ^ 1u)] = row;
                            if (FLIP) atomicXor(reinterpret_cast<unsigned*>(p.ci) + (cell >> 2), CI_PAR << ((cell & 3u) * 8u));
                        }
                        curcp = cp;
                        row = __ldcg(p.Q + 2u * (cp >> 1) + (cp & 1u));
                    }
                    fold(row, (int)(w0 & 3u), p.lr, v[j]);
                }
            }
            if (curcp != 0xFFFFFFFFu) {
                unsigned cell = curcp >> 1, par = curcp & 1u;
                p.Q[2u * cell + (par ^ 1u)] = row;
                if (FLIP) atomicXor(reinterpret_cast<unsigned*>(p.ci) + (cell >> 2), CI_PAR << ((cell & 3u) * 8u));
            }
        }
    }
    __syncthreads();
    {   // medium chains: one warp each
        const unsigned nmed = s_nmed < MED_CHUNKS ? s_nmed : MED_CHUNKS;
        for (unsigned c = threadIdx.x >> 5; c < nmed; c += BLOCK / 32) {
            const unsigned L = s_medlen[c];
            if (L) process_medium<FLIP>(p, s_keys + c * MED_MAX, s_vals + c * MED_MAX, L);
        }
    }
    __syncthreads();
    const unsigned nlong = s_nlong;
    for (unsigned c = 0; c < nlong; ++c) process_long<FLIP>(p, s_long[c], s_keys, s_vals, s_bcast);
    if (threadIdx.x == 0 && nlong) atomicAdd(&p.ctl->long_chains, (unsigned long long)nlong);

    if (TRAIN) {
        // sweep: parity ^= occupied, next-step occupancy becomes current, next bits cleared
        const unsigned n16 = (p.S + 15u) / 16u;
        uint4* wv = reinterpret_cast<uint4*>(p.ci);
        for (unsigned i = blockIdx.x * BLOCK + threadIdx.x; i < n16; i += gridDim.x * BLOCK) {
            uint4 v = wv[i];
#define CUDARL_SWEEP(w) w = (w & 0x03030303u) | ((w ^ ((w & 0x08080808u) >> 1)) & 0x04040404u) | ((w >> 2) & 0x18181818u)
            CUDARL_SWEEP(v.x); CUDARL_SWEEP(v.y); CUDARL_SWEEP(v.z); CUDARL_SWEEP(v.w);
#undef CUDARL_SWEEP
            wv[i] = v;
        }
        // the last block to finish advances the step and the epsilon index
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned done_blocks = atomicAdd(&p.ctl->blocks_done, 1u);
            s_last = (done_blocks == gridDim.x - 1u);
        }
        __syncthreads();
        if (s_last && threadIdx.x == 0) {
            Ctl* c = p.ctl;
            c->blocks_done = 0;
            c->eps_used = p.eps_tab[c->eps_idx];
            c->step += 1ull;
            if (c->eps_mode == 1u) { if (c->eps_idx + 1u < c->eps_len) c->eps_idx += 1u; }
            else if (c->eps_mode == 2u) {
                unsigned long long kk = *((volatile unsigned long long*)&c->episodes) / (unsigned long long)p.N;
                unsigned long long rel = kk > c->eps_base_k ? kk - c->eps_base_k : 0ull;
                c->eps_idx = (unsigned)(rel < (unsigned long long)(c->eps_len - 1u) ? rel : (unsigned long long)(c->eps_len - 1u));
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Caller-driven step (no learning, sticky done, no auto-reset): Environment::step for all envs.
__global__ void k_step_actions(Params p, const int* actions, float* rewards, unsigned char* dones) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    int x = p.x[i], y = p.y[i];
    unsigned s = (unsigned)y * (unsigned)p.W + (unsigned)x;
    unsigned cs = ci_load(p.ci, s), c2;
    int a = actions[i];
    if (a < 0 || a > 3) a = -1;                         // any other value: no movement (src/gpu/environment.cu:31)
    unsigned s2 = move_cell(p, x, y, s, cs, a, c2);
    float r = -0.01f; unsigned char dn = p.done[i];
    if (c2 & CI_GOAL) { r = 1.0f; dn = 1; }
    p.x[i] = (int)(s2 % (unsigned)p.W); p.y[i] = (int)(s2 / (unsigned)p.W); p.t[i] += 1;
    p.reward[i] = r; p.done[i] = dn;
    if (rewards) rewards[i] = r;
    if (dones) dones[i] = dn;
}

// Greedy rollout of every environment from a fresh start cell; positions stay in registers, the
// table is read-only, so the whole rollout is one launch.
__global__ void __launch_bounds__(BLOCK) k_eval(Params p, int max_steps, unsigned long long nonce) {
    __shared__ unsigned s_reached; __shared__ unsigned long long s_steps;
    if (threadIdx.x == 0) { s_reached = 0; s_steps = 0; }
    __syncthreads();
    unsigned i = blockIdx.x * BLOCK + threadIdx.x;
    if (i < p.N) {
        unsigned s = sample_start(p, p.env_offset + i, nonce, TAG_EVAL);
        unsigned cs = ci_load(p.ci, s);
        unsigned steps = 0; bool reached = false;
        for (int k = 0; k < max_steps; ++k) {
            float4 row = __ldg(p.Q + 2u * s + ((cs & CI_PAR) ? 1u : 0u));
            int a = argmax4(row);
            int x = (int)(s % (unsigned)p.W), y = (int)(s / (unsigned)p.W);
            unsigned c2; unsigned s2 = move_cell(p, x, y, s, cs, a, c2);
            ++steps; s = s2; cs = c2;
            if (c2 & CI_GOAL) { reached = true; break; }
        }
        if (reached) atomicAdd(&s_reached, 1u);
        atomicAdd(&s_steps, (unsigned long long)steps);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_reached) atomicAdd(&p.ctl->eval_reached, (unsigned long long)s_reached);
        if (s_steps) atomicAdd(&p.ctl->eval_steps, s_steps);
    }
}

// update_batch, phase 1: TD error of every transition against the table as it is now; every
// transition becomes a collision entry (index order = fold order).
__global__ void k_update_main(Params p, unsigned n, const int* sx, const int* sy, const int* act, const float* rew,
                              const int* nxs, const int* nys, const unsigned char* dn) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0) p.ctl->scratch_cursor = 0;        // the long-chain scratch is per call; nobody reads it in this kernel
    if (i >= n) return;
    int x = sx[i], y = sy[i], a = act[i], nx = nxs[i], ny = nys[i];
    unsigned s = (unsigned)y * (unsigned)p.W + (unsigned)x;
    unsigned s2 = (unsigned)ny * (unsigned)p.W + (unsigned)nx;
    unsigned cs = ci_load(p.ci, s);
    unsigned par = (cs & CI_PAR) ? 1u : 0u;
    float4 row = __ldcg(p.Q + 2u * s + par);
    float m = 0.0f;
    if (!dn[i]) {
        unsigned c2 = ci_load(p.ci, s2);
        m = max4(__ldcg(p.Q + 2u * s2 + ((c2 & CI_PAR) ? 1u : 0u)));
        if (p.legacy_clamp && m < 0.0f) m = 0.0f;
    }
    float target = __fmaf_rn(p.gamma, m, rew[i]);
    float d = __fsub_rn(target, pick(row, a));
    unsigned prev = atomicExch(p.mailbox + mb_slot(p, s), i + 1u);
    p.ent[i] = make_uint4((s << 3) | (par << 2) | (unsigned)a, i, __float_as_uint(d), prev);
}

// ------------------------------------------------------------------------------------------------
// Table in the caller's layout: dense[(y*W+x)] = float4 of the 4 action values.
__global__ void k_q_gather(Params p, float4* dense) {
    unsigned s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= p.S) return;
    dense[s] = p.Q[2u * s + ((p.ci[s] & CI_PAR) ? 1u : 0u)];
}
__global__ void k_q_scatter(Params p, const float4* dense, float scale) {
    unsigned s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= p.S) return;
    float4 v = dense[s];
    v.x = __fmul_rn(v.x, scale); v.y = __fmul_rn(v.y, scale); v.z = __fmul_rn(v.z, scale); v.w = __fmul_rn(v.w, scale);
    p.Q[2u * s + ((p.ci[s] & CI_PAR) ? 1u : 0u)] = v;
}
__global__ void k_q_init(Params p, int kind, float scale) {
    unsigned s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= p.S) return;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (kind == 1) {
        U4 w = philox4x32_10(s, 0u, 0u, 0u, p.k0, p.k1 ^ TAG_QINIT);
        v.x = __fmul_rn(u01(w.x), scale); v.y = __fmul_rn(u01(w.y), scale);
        v.z = __fmul_rn(u01(w.z), scale); v.w = __fmul_rn(u01(w.w), scale);
    }
    p.Q[2u * s] = v; p.Q[2u * s + 1u] = v;
}
__global__ void k_cells_get(Params p, unsigned char* cells) {
    unsigned s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= p.S) return;
    unsigned c = p.ci[s];
    cells[s] = (c & CI_GOAL) ? 2 : ((c & CI_OBST) ? 1 : 0);
}
__global__ void k_cell_set(Params p, unsigned cell, unsigned cls, int clear_goals) {
    unsigned* w32 = reinterpret_cast<unsigned*>(p.ci);
    if (clear_goals) {
        unsigned n4 = (p.S + 3u) / 4u;
        for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x)
            atomicAnd(w32 + i, ~0x02020202u);
    } else if (blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned sh = (cell & 3u) * 8u;
        atomicAnd(w32 + (cell >> 2), ~(3u << sh));
        if (cls) atomicOr(w32 + (cell >> 2), cls << sh);
    }
}

// ------------------------------------------------------------------------------------------------
static inline unsigned nblk(unsigned n) { return (n + BLOCK - 1) / BLOCK; }
static inline unsigned sweep_blocks(unsigned S) { unsigned b = nblk((S + 15u) / 16u); return b < 1u ? 1u : (b > 1184u ? 1184u : b); }

void launch_rebuild_occupancy(const Params& p, cudaStream_t st) {
    k_occ_clear<<<sweep_blocks(p.S), BLOCK, 0, st>>>(p);
    if (p.N) k_occ_announce<<<nblk(p.N), BLOCK, 0, st>>>(p);
}
void launch_reset_all(const Params& p, cudaStream_t st) {
    if (p.N) k_reset_all<<<nblk(p.N), BLOCK, 0, st>>>(p);
}
void launch_train_step(const Params& p, bool trace, cudaStream_t st, cudaEvent_t ev_a, cudaEvent_t ev_b, cudaEvent_t ev_c) {
    if (ev_a) cudaEventRecord(ev_a, st);
    if (trace) k_train_main<true><<<p.nblocks_main, BLOCK, 0, st>>>(p);
    else       k_train_main<false><<<p.nblocks_main, BLOCK, 0, st>>>(p);
    if (ev_b) cudaEventRecord(ev_b, st);
    k_fix<true><<<p.mb_slots / BLOCK, BLOCK, 0, st>>>(p);
    if (ev_c) cudaEventRecord(ev_c, st);
}
void launch_step_actions(const Params& p, const int* a, float* r, unsigned char* d, cudaStream_t st) {
    if (p.N) k_step_actions<<<nblk(p.N), BLOCK, 0, st>>>(p, a, r, d);
}
void launch_eval(const Params& p, int max_steps, unsigned long long nonce, cudaStream_t st) {
    if (p.N) k_eval<<<nblk(p.N), BLOCK, 0, st>>>(p, max_steps, nonce);
}
void launch_update_batch(const Params& p, unsigned n, const int* sx, const int* sy, const int* a, const float* r,
                         const int* nx, const int* ny, const unsigned char* dn, cudaStream_t st) {
    if (!n) return;
    k_update_main<<<nblk(n), BLOCK, 0, st>>>(p, n, sx, sy, a, r, nx, ny, dn);
    k_fix<false><<<p.mb_slots / BLOCK, BLOCK, 0, st>>>(p);
}
void launch_q_gather(const Params& p, float4* dense, cudaStream_t st) { k_q_gather<<<nblk(p.S), BLOCK, 0, st>>>(p, dense); }
void launch_q_scatter(const Params& p, const float4* dense, float scale, cudaStream_t st) { k_q_scatter<<<nblk(p.S), BLOCK, 0, st>>>(p, dense, scale); }
void launch_q_init(const Params& p, int kind, float scale, cudaStream_t st) { k_q_init<<<nblk(p.S), BLOCK, 0, st>>>(p, kind, scale); }
void launch_cells_get(const Params& p, unsigned char* d_cells, cudaStream_t st) { k_cells_get<<<nblk(p.S), BLOCK, 0, st>>>(p, d_cells); }
void launch_cell_set(const Params& p, unsigned cell, unsigned cls, int clear_goals, cudaStream_t st) {
    k_cell_set<<<clear_goals ? sweep_blocks(p.S) : 1, BLOCK, 0, st>>>(p, cell, cls, clear_goals);
}

int kernel_attr_report(char* buf, int n) {
    cudaFuncAttributes a, b;
    if (cudaFuncGetAttributes(&a, k_train_main<false>) != cudaSuccess) return -1;
    if (cudaFuncGetAttributes(&b, k_fix<true>) != cudaSuccess) return -1;
    return snprintf(buf, n, "train_main: %d regs, %zu B smem; train_fix: %d regs, %zu B smem",
                    a.numRegs, a.sharedSizeBytes, b.numRegs, b.sharedSizeBytes);
}

}  // namespace cudarl
