// kernels.cu -- sm_100a kernels of the batched grid-world + tabular Q-learning path other than the fused
// train step (tile_engine.cu): environment reset and caller-driven stepping, the greedy rollout, the
// ordered TD update of caller-supplied transitions (update_batch) and table initialisation.
//
// Data layout in HBM (per context = per GPU):
//   st [N]   environment state, one int4 {x, y, t, id} per environment (record k = environment k outside
//            train steps), one aligned 16-byte vector load/store per thread;
//   Q        the table, one float4 per grid cell (index y*W + x): one vector load is the whole action row;
//   cw       one 16-bit word per cell holding the cell's class bits (obstacle, goal);
//   ent / mailbox   collision entries and chain heads of update_batch.
//
// Reference semantics (paths relative to the CudaRL-Arena project root):
//   step        src/environment.cu:17-48, obstacle test src/kernels.cu:29-44, goal src/kernels.cu:56-59
//   reset       src/environment.cu:6-14
//   TD update   src/kernels.cu:96-114 (true max as in src/gpu/kernels.cu:36-45, src/train.py:134)
//   first-max argmax src/q_learning.cu:196-206; greedy rollout src/train.py:262-311
#include "kernels.cuh"
#include "rules.cuh"
#include <cstdio>

namespace cudarl {

// Move from (x,y) by `action`; returns the new cell and its cell word.
__device__ __forceinline__ unsigned move_cell(const Params& p, int x, int y, unsigned s, unsigned cw_s, int action,
                                              unsigned& cw_new) {
    int dx = (action == 1) - (action == 3), dy = (action == 2) - (action == 0);
    int nx = x + dx, ny = y + dy;
    bool inb = nx >= 0 && nx < p.W && ny >= 0 && ny < p.H;
    unsigned tgt = inb ? (unsigned)ny * (unsigned)p.W + (unsigned)nx : s;
    unsigned ct = (tgt != s) ? cw_load(p.cw, tgt) : cw_s;
    bool moved = (tgt != s) && !(ct & CW_OBST);
    cw_new = moved ? ct : cw_s;
    return moved ? tgt : s;
}

// chain heads are indexed by the low bits of the cell: neighbouring cells -> neighbouring slots
__device__ __forceinline__ unsigned mb_slot(const Params& p, unsigned cell) { return cell & (p.mb_slots - 1u); }

__global__ void k_reset_all(Params p) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    unsigned e = (unsigned)p.st[i].w;
    unsigned c = sample_start(p, p.env_offset + e, p.step, TAG_START);
    p.st[i] = make_int4((int)(c % (unsigned)p.W), (int)(c / (unsigned)p.W), 0, (int)e);
    if (p.reward) { p.reward[e] = 0.0f; p.done[e] = 0; }
}

__global__ void k_ids_identity(Params p) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < p.N) p.st[i].w = (int)i;
}
// overwrite x / y / t of environment-ordered records from caller arrays (any of them may be null)
__global__ void k_import_state(Params p, const int* x, const int* y, const int* t) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    int4 r = p.st[i];
    if (x) r.x = x[i];
    if (y) r.y = y[i];
    if (t) r.z = t[i];
    r.w = (int)i;
    p.st[i] = r;
}
__global__ void k_export_state(Params p) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    const int4 r = p.st[i];
    int* out = reinterpret_cast<int*>(p.st2);          // the spare copy, viewed as x[N] | y[N] | t[N]
    out[r.w] = r.x; out[p.N + r.w] = r.y; out[2u * p.N + r.w] = r.z;
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
__device__ void apply_run(const Params& p, const unsigned long long* keys, const float* vals, unsigned j, unsigned n) {
    unsigned w0 = (unsigned)(keys[j] >> 32);
    unsigned cellp = w0 >> 2;              // (cell << 1) | parity
    unsigned cell = w0 >> 3;
    float4 row = __ldcg(p.Q + cell);
    for (; j < n; ++j) {
        unsigned wj = (unsigned)(keys[j] >> 32);
        if ((wj >> 2) != cellp) break;
        fold(row, (int)(wj & 3u), p.lr, vals[j]);
    }
    p.Q[cell] = row;          // in place: the targets were taken before this kernel started, and one thread owns the cell
}

constexpr unsigned LONG_SMEM = 1024;   // chain entries sorted in shared memory; longer chains use the global scratch
constexpr int SHORT_MAX = 8;           // chain entries folded in registers by one thread

// One long chain, whole block: count its entries (one hop per run), pick shared memory or a slice of the
// global scratch, copy the runs (one warp per run, batches of 256 runs), bitonic-sort by (cell, action, id)
// and let the first thread of every cell run fold it.
__device__ void process_long(const Params& p, unsigned head1, unsigned long long* s_keys, float* s_vals,
                             unsigned* s_bcast) {
    __shared__ unsigned s_run[BLOCK], s_off[BLOCK];
    if (threadIdx.x == 0) {
        unsigned q = head1, L = 0, hops = 0;
        while (q && hops <= p.ent_cap) {          // a chain can never have more runs than the entry array has slots
            L += (q >> LINK_POS_BITS) + 1u; ++hops;
            q = p.ent[(q & LINK_POS_MASK) - 1u].w;
        }
        unsigned n2 = 1; while (n2 < L) n2 <<= 1;
        unsigned base = 0xFFFFFFFFu;
        if (q || L > p.ent_cap) { atomicOr(&p.ctl->error, ERR_CHAIN_CYCLE); base = 0xFFFFFFFEu; }
        else if (L > LONG_SMEM) {
            base = atomicAdd(&p.ctl->scratch_cursor, n2);
            if (base + n2 > p.sc_cap) { atomicOr(&p.ctl->error, ERR_SCRATCH_OVERFLOW); base = 0xFFFFFFFEu; }
        }
        s_bcast[0] = L; s_bcast[1] = n2; s_bcast[2] = base;
    }
    __syncthreads();
    const unsigned L = s_bcast[0], n2 = s_bcast[1], base = s_bcast[2];
    if (base != 0xFFFFFFFEu) {
        unsigned long long* keys = (base == 0xFFFFFFFFu) ? s_keys : p.sc_key + base;
        float* vals = (base == 0xFFFFFFFFu) ? s_vals : p.sc_val + base;
        __shared__ unsigned s_q, s_nb, s_done_entries;
        if (threadIdx.x == 0) { s_q = head1; s_done_entries = 0; }
        __syncthreads();
        while (true) {                               // batches of up to 256 runs; ends when the chain is exhausted
            if (threadIdx.x == 0) {
                unsigned q = s_q, nb = 0, off = s_done_entries;
                while (q && nb < (unsigned)BLOCK) {
                    s_run[nb] = q; s_off[nb] = off; off += (q >> LINK_POS_BITS) + 1u; ++nb;
                    q = p.ent[(q & LINK_POS_MASK) - 1u].w;
                }
                s_q = q; s_nb = nb; s_done_entries = off;
            }
            __syncthreads();
            const unsigned nb = s_nb;
            if (nb == 0u) break;
            for (unsigned r = threadIdx.x >> 5; r < nb; r += BLOCK / 32) {
                const unsigned link = s_run[r], pos0 = (link & LINK_POS_MASK) - 1u, len = (link >> LINK_POS_BITS) + 1u;
                const unsigned j = threadIdx.x & 31u;
                if (j < len && s_off[r] + j < L) {
                    const uint4 e = p.ent[pos0 + j];
                    keys[s_off[r] + j] = ((unsigned long long)e.x << 32) | e.y; vals[s_off[r] + j] = __uint_as_float(e.z);
                }
            }
            __syncthreads();
        }
        for (unsigned i = L + threadIdx.x; i < n2; i += blockDim.x) { keys[i] = ~0ull; vals[i] = 0.0f; }
        __syncthreads();
        block_bitonic(keys, vals, n2);
        for (unsigned j = threadIdx.x; j < L; j += blockDim.x) {
            unsigned cp = (unsigned)(keys[j] >> 34);
            if (j == 0 || (unsigned)(keys[j - 1] >> 34) != cp) apply_run(p, keys, vals, j, L);
        }
    }
    __syncthreads();
}

constexpr unsigned MED_MAX = 32;                         // chain entries ranked by one warp with shuffles
constexpr unsigned MED_CHUNKS = LONG_SMEM / MED_MAX;     // medium chains a block can stage in shared memory

// One warp orders a staged chain of L <= 32 entries by (cell, action, index) with a shuffle ranking
// (indices are unique, so ranks are a permutation), then the first lane of every cell run folds it.
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
        if (lane == 0 || (unsigned)(keys[lane - 1] >> 34) != cp) apply_run(p, keys, vals, lane, L);
    }
    __syncwarp();
}

// Collision folding, one thread per ACTIVE mailbox slot (the producers list every slot they were the
// first to hook a chain into, so this kernel only visits slots that have work).  A slot's chain links
// RUNS of consecutive entries (one run = the lanes of one warp on one cell).  The owning thread gathers
// the chain's entries:
//   <= 8 entries   in registers, ordered by a sorting network and folded by that thread;
//   <= 32 entries  staged in shared memory by that thread, ordered and folded by one warp;
//   longer         queued for k_fix_long (one warp per chain up to 256 entries, then one block per chain).
__device__ __forceinline__ void flush_row(const Params& p, unsigned cellpar, const float4& row) { p.Q[cellpar >> 1] = row; }

__global__ void __launch_bounds__(BLOCK) k_fix(Params p) {
    __shared__ unsigned long long s_keys[LONG_SMEM];
    __shared__ float s_vals[LONG_SMEM];
    __shared__ unsigned s_medlen[MED_CHUNKS];
    __shared__ unsigned s_nmed;
    const unsigned nactive = p.ctl->active_count[p.step & 1ull];      // slots that received a chain in this step
  for (unsigned tile = blockIdx.x; tile * BLOCK < nactive; tile += gridDim.x) {
    if (threadIdx.x == 0) s_nmed = 0;
    __syncthreads();
    const unsigned ai = tile * BLOCK + threadIdx.x;
    const unsigned slot = ai < nactive ? p.active[ai] : 0u;
    const unsigned head = ai < nactive ? p.mailbox[slot] : 0u;
    if (head) {
        p.mailbox[slot] = 0u;                          // leave the mailbox empty for the next step
        unsigned long long k8[SHORT_MAX]; float v8[SHORT_MAX];
        unsigned q = head, pos = 0, rem = 0; bool fresh = false;
#pragma unroll
        for (int j = 0; j < SHORT_MAX; ++j) {
            if (rem == 0u && q) { pos = (q & LINK_POS_MASK) - 1u; rem = (q >> LINK_POS_BITS) + 1u; fresh = true; }
            if (rem) {
                const uint4 e = __ldcg(p.ent + pos);
                k8[j] = ((unsigned long long)e.x << 32) | e.y; v8[j] = __uint_as_float(e.z);
                if (fresh) { q = e.w; fresh = false; }
                ++pos; --rem;
            } else { k8[j] = ~0ull; v8[j] = 0.0f; }
        }
        if (rem == 0u && q == 0u) {
            cswap(k8[0],v8[0],k8[1],v8[1]); cswap(k8[2],v8[2],k8[3],v8[3]); cswap(k8[4],v8[4],k8[5],v8[5]); cswap(k8[6],v8[6],k8[7],v8[7]);
            cswap(k8[0],v8[0],k8[2],v8[2]); cswap(k8[1],v8[1],k8[3],v8[3]); cswap(k8[4],v8[4],k8[6],v8[6]); cswap(k8[5],v8[5],k8[7],v8[7]);
            cswap(k8[1],v8[1],k8[2],v8[2]); cswap(k8[5],v8[5],k8[6],v8[6]); cswap(k8[0],v8[0],k8[4],v8[4]); cswap(k8[3],v8[3],k8[7],v8[7]);
            cswap(k8[1],v8[1],k8[5],v8[5]); cswap(k8[2],v8[2],k8[6],v8[6]);
            cswap(k8[1],v8[1],k8[4],v8[4]); cswap(k8[3],v8[3],k8[6],v8[6]);
            cswap(k8[2],v8[2],k8[4],v8[4]); cswap(k8[3],v8[3],k8[5],v8[5]);
            cswap(k8[3],v8[3],k8[4],v8[4]);
            unsigned curcp = 0xFFFFFFFFu; float4 row = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < SHORT_MAX; ++j) {
                if (k8[j] != ~0ull) {
                    const unsigned w0 = (unsigned)(k8[j] >> 32), cp = w0 >> 2;
                    if (cp != curcp) {
                        if (curcp != 0xFFFFFFFFu) flush_row(p, curcp, row);
                        curcp = cp; row = __ldcg(p.Q + (cp >> 1));
                    }
                    fold(row, (int)(w0 & 3u), p.lr, v8[j]);
                }
            }
            if (curcp != 0xFFFFFFFFu) flush_row(p, curcp, row);
        } else {
            const unsigned chunk = atomicAdd(&s_nmed, 1u);
            bool staged = false;
            if (chunk < MED_CHUNKS) {
                unsigned long long* mk = s_keys + chunk * MED_MAX; float* mv = s_vals + chunk * MED_MAX;
#pragma unroll
                for (int j = 0; j < SHORT_MAX; ++j) { mk[j] = k8[j]; mv[j] = v8[j]; }
                unsigned L = SHORT_MAX;
                while ((rem || q) && L < MED_MAX) {
                    if (rem == 0u) { pos = (q & LINK_POS_MASK) - 1u; rem = (q >> LINK_POS_BITS) + 1u; fresh = true; }
                    const uint4 e = __ldcg(p.ent + pos);
                    mk[L] = ((unsigned long long)e.x << 32) | e.y; mv[L] = __uint_as_float(e.z);
                    if (fresh) { q = e.w; fresh = false; }
                    ++pos; --rem; ++L;
                }
                staged = (rem == 0u && q == 0u);
                s_medlen[chunk] = staged ? L : 0u;
            }
            if (!staged) {                              // hand the chain to k_fix_long
                const unsigned li = atomicAdd(&p.ctl->long_count[p.step & 1ull], 1u);
                p.longq[li] = head;
            }
        }
    }
    __syncthreads();
    {   // medium chains: one warp each
        const unsigned nmed = s_nmed < MED_CHUNKS ? s_nmed : MED_CHUNKS;
        for (unsigned c = threadIdx.x >> 5; c < nmed; c += BLOCK / 32) {
            const unsigned L = s_medlen[c];
            if (L) process_medium(p, s_keys + c * MED_MAX, s_vals + c * MED_MAX, L);
        }
    }
    __syncthreads();
  }

}

// Long chains (more than 32 entries: cells crowded with environments).  First tier: one WARP per chain for up
// to 256 entries -- lane 0 hops from run to run, all lanes copy the run's entries into the warp's slice of
// shared memory, a warp-wide bitonic sort orders them by (cell, action, id), the first lane of every cell run
// applies it.  Chains that do not fit are queued for k_fix_long2 (one block per chain).
constexpr unsigned WARP_LONG = 256;

__device__ bool process_long_warp(const Params& p, unsigned head, unsigned long long* keys, float* vals) {
    const unsigned lane = threadIdx.x & 31u;
    unsigned q = head, L = 0, hops = 0; bool fits = true;
    while (q && hops <= p.ent_cap) {                  // q is warp-uniform
        const unsigned pos0 = (q & LINK_POS_MASK) - 1u, len = (q >> LINK_POS_BITS) + 1u;
        if (L + len > WARP_LONG) { fits = false; break; }
        uint4 e = make_uint4(0u, 0u, 0u, 0u);
        if (lane < len) { e = __ldcg(p.ent + pos0 + lane); keys[L + lane] = ((unsigned long long)e.x << 32) | e.y; vals[L + lane] = __uint_as_float(e.z); }
        q = __shfl_sync(FULL, e.w, 0);                // the run's first entry carries the link to the next run
        L += len; ++hops;
    }
    if (!fits || q) return false;
    unsigned n2 = 32; while (n2 < L) n2 <<= 1;
    for (unsigned i = L + lane; i < n2; i += 32u) { keys[i] = ~0ull; vals[i] = 0.0f; }
    __syncwarp();
    for (unsigned k = 2; k <= n2; k <<= 1) {
        for (unsigned j = k >> 1; j > 0; j >>= 1) {
            for (unsigned i = lane; i < n2; i += 32u) {
                const unsigned ixj = i ^ j;
                if (ixj > i) {
                    const unsigned long long a = keys[i], b = keys[ixj];
                    const bool up = (i & k) == 0;
                    if ((a > b) == up) { keys[i] = b; keys[ixj] = a; const float t = vals[i]; vals[i] = vals[ixj]; vals[ixj] = t; }
                }
            }
            __syncwarp();
        }
    }
    for (unsigned j = lane; j < L; j += 32u) {
        const unsigned cp = (unsigned)(keys[j] >> 34);
        if (j == 0 || (unsigned)(keys[j - 1] >> 34) != cp) apply_run(p, keys, vals, j, L);
    }
    __syncwarp();
    return true;
}

__global__ void __launch_bounds__(BLOCK) k_fix_long(Params p) {
    __shared__ unsigned long long s_keys[(BLOCK / 32) * WARP_LONG];
    __shared__ float s_vals[(BLOCK / 32) * WARP_LONG];
    const unsigned n = p.ctl->long_count[p.step & 1ull];
    const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    unsigned done = 0;
    for (unsigned c = blockIdx.x * (BLOCK / 32) + warp; c < n; c += gridDim.x * (BLOCK / 32)) {
        const unsigned head = p.longq[c];
        if (!process_long_warp(p, head, s_keys + warp * WARP_LONG, s_vals + warp * WARP_LONG)) {
            if (lane == 0) p.longq2[atomicAdd(&p.ctl->long2_count[p.step & 1ull], 1u)] = head;
        }
        ++done;
    }
    if (lane == 0 && done) atomicAdd(&p.ctl->long_chains, (unsigned long long)done);
}

// Second tier: one block per chain, any length (shared memory up to 1024 entries, the global scratch beyond).
__global__ void __launch_bounds__(BLOCK) k_fix_long2(Params p) {
    __shared__ unsigned long long s_keys[LONG_SMEM];
    __shared__ float s_vals[LONG_SMEM];
    __shared__ unsigned s_bcast[3];
    const unsigned n = p.ctl->long2_count[p.step & 1ull];
    for (unsigned c = blockIdx.x; c < n; c += gridDim.x) process_long(p, p.longq2[c], s_keys, s_vals, s_bcast);
}

// ------------------------------------------------------------------------------------------------
// Caller-driven step (no learning, sticky done, no auto-reset): Environment::step for all envs.
// actions / rewards / dones are indexed by environment id.
__global__ void k_step_actions(Params p, const int* actions, float* rewards, unsigned char* dones) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    const int4 rec = p.st[i];
    unsigned e = (unsigned)rec.w;
    int x = rec.x, y = rec.y;
    unsigned s = (unsigned)y * (unsigned)p.W + (unsigned)x;
    unsigned cs = cw_load(p.cw, s), c2;
    int a = actions[e];
    if (a < 0 || a > 3) a = -1;                         // any other value: no movement (src/gpu/environment.cu:31)
    unsigned s2 = move_cell(p, x, y, s, cs, a, c2);
    float r = (s2 == s && a >= 0) ? blocked_step_reward(p, x, y, a) : -0.01f;    // a trap charges its penalty (src/kernels.cu:61-63)
    unsigned char dn = p.done[e];
    if (c2 & CW_GOAL) { r = 1.0f; dn = 1; }
    p.st[i] = make_int4((int)(s2 % (unsigned)p.W), (int)(s2 / (unsigned)p.W), rec.z + 1, rec.w);
    p.reward[e] = r; p.done[e] = dn;
    if (rewards) rewards[e] = r;
    if (dones) dones[e] = dn;
}

// Greedy rollout of every environment from a fresh start cell.  The table does not change during a rollout, so the greedy
// policy is folded into one byte per cell first (k_eval_policy: bits 0-1 the first-max action, bit 2 "that move is blocked",
// bit 3 "it ends on a goal") -- one pass over the table -- and the rollout itself walks that map: one byte per step instead
// of a 16-byte row and a move byte, and the map (one byte per cell) stays in L2.  Positions stay in registers, so the whole
// rollout is one launch; every thread walks four environments, so that four dependent chains of loads overlap.
__global__ void __launch_bounds__(BLOCK) k_eval_policy(Params p, unsigned char* __restrict__ pol) {
    const TileP& tp = p.tp;
    for (unsigned s = blockIdx.x * BLOCK + threadIdx.x; s < p.S; s += gridDim.x * BLOCK) {
        const unsigned y = s / (unsigned)p.W, x = s - y * (unsigned)p.W;
        const unsigned tile = (y >> tp.tshift) * tp.tiles_x + (x >> tp.tshift);
        const float4 row = __ldcs(p.Q + s);
        const unsigned mvb = __ldg(tp.tcls + (size_t)tile * tp.cls_stride + (((y & (tp.T - 1u)) << tp.tshift) | (x & (tp.T - 1u))));
        const int a = argmax4(row);
        pol[s] = (unsigned char)((unsigned)a | (((mvb >> a) & 1u) << 2) | (((mvb >> (4 + a)) & 1u) << 3));
    }
}
constexpr int EVAL_EPT = 4;     // environments per thread
__global__ void __launch_bounds__(BLOCK) k_eval(Params p, const unsigned char* __restrict__ pol, int max_steps, unsigned long long nonce) {
    __shared__ unsigned s_reached; __shared__ unsigned long long s_steps;
    if (threadIdx.x == 0) { s_reached = 0; s_steps = 0; }
    __syncthreads();
    const unsigned part = (p.N + (unsigned)EVAL_EPT - 1u) / (unsigned)EVAL_EPT;
    const unsigned i0 = blockIdx.x * BLOCK + threadIdx.x;
    if (i0 < part) {
        unsigned pos[EVAL_EPT]; unsigned live = 0u, reached = 0u, steps = 0u;
#pragma unroll
        for (int k = 0; k < EVAL_EPT; ++k) {
            const unsigned i = i0 + (unsigned)k * part;
            if (i < p.N) live |= 1u << k;
            pos[k] = i < p.N ? sample_start(p, p.env_offset + i, nonce, TAG_EVAL) : 0u;
        }
        for (int it = 0; it < max_steps && live; ++it) {
            unsigned b[EVAL_EPT];
#pragma unroll
            for (int k = 0; k < EVAL_EPT; ++k) b[k] = __ldg(pol + pos[k]);
#pragma unroll
            for (int k = 0; k < EVAL_EPT; ++k) {
                if (!((live >> k) & 1u)) continue;
                const unsigned a = b[k] & 3u;
                // per action the step in cells: up -W, right +1, down +W, left -1; none when the move is blocked
                if (!(b[k] & 4u)) pos[k] += a == 0u ? 0u - (unsigned)p.W : a == 1u ? 1u : a == 2u ? (unsigned)p.W : 0u - 1u;
                ++steps;
                if (b[k] & 8u) { ++reached; live &= ~(1u << k); }
            }
        }
        if (reached) atomicAdd(&s_reached, reached);
        atomicAdd(&s_steps, (unsigned long long)steps);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_reached) atomicAdd(&p.ctl->eval_reached, (unsigned long long)s_reached);
        if (s_steps) atomicAdd(&p.ctl->eval_steps, s_steps);
    }
}

__global__ void k_active_reset(Params p) { p.ctl->active_count[p.step & 1ull] = 0; p.ctl->long_count[p.step & 1ull] = 0; p.ctl->long2_count[p.step & 1ull] = 0; }

// update_batch, phase 1: TD target of every transition from the table as it is now; every
// transition becomes a collision entry (index order = fold order).
__global__ void k_update_main(Params p, unsigned n, const int* sx, const int* sy, const int* act, const float* rew,
                              const int* nxs, const int* nys, const unsigned char* dn) {
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned lane = threadIdx.x & 31u;
    if (i == 0) { p.ctl->scratch_cursor = 0; }     // the long-chain scratch is per call; nobody reads it in this kernel
    bool first = false; unsigned slot = 0;
    if (i < n) {
        int x = sx[i], y = sy[i], a = act[i], nx = nxs[i], ny = nys[i];
        unsigned s = (unsigned)y * (unsigned)p.W + (unsigned)x;
        unsigned s2 = (unsigned)ny * (unsigned)p.W + (unsigned)nx;
        float m = 0.0f;
        if (!dn[i]) {
            m = max4(__ldcg(p.Q + s2));
            if (p.legacy_clamp && m < 0.0f) m = 0.0f;
        }
        float d = __fmaf_rn(p.gamma, m, rew[i]);           // TD target
        slot = mb_slot(p, s);
        unsigned prev = atomicExch(p.mailbox + slot, i + 1u);          // a run of one entry
        p.ent[i] = make_uint4((s << 3) | (unsigned)a, i, __float_as_uint(d), prev);
        first = prev == 0u;
    }
    const unsigned fm = __ballot_sync(FULL, first);                  // list the slots that just became active
    if (fm) {
        unsigned base = 0;
        if (lane == __ffs(fm) - 1u) base = atomicAdd(&p.ctl->active_count[p.step & 1ull], __popc(fm));
        base = __shfl_sync(FULL, base, __ffs(fm) - 1);
        if (first) p.active[base + __popc(fm & ((1u << lane) - 1u))] = slot;
    }
}

// ------------------------------------------------------------------------------------------------
__global__ void k_q_init(Params p, int kind, float scale) {
    unsigned s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= p.S) return;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (kind == 1) {
        U4 w = philox4x32_10(s, 0u, 0u, 0u, p.k0, p.k1 ^ TAG_QINIT);
        v.x = __fmul_rn(u01(w.x), scale); v.y = __fmul_rn(u01(w.y), scale);
        v.z = __fmul_rn(u01(w.z), scale); v.w = __fmul_rn(u01(w.w), scale);
    }
    p.Q[s] = v;
}
__global__ void k_cell_set(Params p, unsigned cell, unsigned cls, int clear_goals) {
    unsigned* w32 = reinterpret_cast<unsigned*>(p.cw);
    if (clear_goals) {
        unsigned n2 = (p.S + 1u) / 2u;
        for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += gridDim.x * blockDim.x)
            atomicAnd(w32 + i, ~0x00020002u);
    } else if (blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned sh = (cell & 1u) * 16u;
        atomicAnd(w32 + (cell >> 1), ~(7u << sh));
        if (cls) atomicOr(w32 + (cell >> 1), cls << sh);
    }
}

// ------------------------------------------------------------------------------------------------
static inline unsigned nblk(unsigned n) { return (n + BLOCK - 1) / BLOCK; }
static inline unsigned fix_blocks(const Params& p) { unsigned b = p.mb_slots / BLOCK; return b > 1184u ? 1184u : b; }
static inline unsigned sweep_blocks(unsigned S) { unsigned b = nblk((2u * S + 15u) / 16u); return b < 1u ? 1u : (b > 1184u ? 1184u : b); }

void launch_identity_ids(const Params& p, cudaStream_t st) { if (p.N) k_ids_identity<<<nblk(p.N), BLOCK, 0, st>>>(p); }
void launch_export_state(const Params& p, cudaStream_t st) { if (p.N) k_export_state<<<nblk(p.N), BLOCK, 0, st>>>(p); }
void launch_import_state(const Params& p, const int* x, const int* y, const int* t, cudaStream_t st) { if (p.N) k_import_state<<<nblk(p.N), BLOCK, 0, st>>>(p, x, y, t); }
void launch_reset_all(const Params& p, cudaStream_t st) {
    if (p.N) k_reset_all<<<nblk(p.N), BLOCK, 0, st>>>(p);
}
void launch_step_actions(const Params& p, const int* a, float* r, unsigned char* d, cudaStream_t st) {
    if (p.N) k_step_actions<<<nblk(p.N), BLOCK, 0, st>>>(p, a, r, d);
}
void launch_eval(const Params& p, unsigned char* policy, int max_steps, unsigned long long nonce, cudaStream_t st) {
    if (!p.N) return;
    k_eval_policy<<<nblk(p.S) < 4736u ? nblk(p.S) : 4736u, BLOCK, 0, st>>>(p, policy);
    k_eval<<<nblk((p.N + (unsigned)EVAL_EPT - 1u) / (unsigned)EVAL_EPT), BLOCK, 0, st>>>(p, policy, max_steps, nonce);
}
void launch_update_batch(const Params& p, unsigned n, const int* sx, const int* sy, const int* a, const float* r,
                         const int* nx, const int* ny, const unsigned char* dn, cudaStream_t st) {
    if (!n) return;
    k_active_reset<<<1, 1, 0, st>>>(p);
    k_update_main<<<nblk(n), BLOCK, 0, st>>>(p, n, sx, sy, a, r, nx, ny, dn);
    k_fix<<<fix_blocks(p), BLOCK, 0, st>>>(p);
    k_fix_long<<<296, BLOCK, 0, st>>>(p);
    k_fix_long2<<<296, BLOCK, 0, st>>>(p);
}
void launch_q_init(const Params& p, int kind, float scale, cudaStream_t st) { k_q_init<<<nblk(p.S), BLOCK, 0, st>>>(p, kind, scale); }
void launch_cell_set(const Params& p, unsigned cell, unsigned cls, int clear_goals, cudaStream_t st) {
    k_cell_set<<<clear_goals ? sweep_blocks(p.S) : 1, BLOCK, 0, st>>>(p, cell, cls, clear_goals);
}

}  // namespace cudarl
