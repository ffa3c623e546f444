// kernels.cu -- hand-written sm_100a kernels of the batched grid-world + tabular Q-learning path.
//
// Data layout in HBM (per context = per GPU):
//   st [N]         environment state, one int4 {x, y, t, id} per SLOT (slot k holds environment id);
//                  one aligned 16-byte vector load/store per thread, fully coalesced.  Every few steps the slots are re-ordered by
//                  cell (counting sort), so neighbouring threads touch neighbouring table rows and the
//                  environments that share a cell sit in the same warp;
//   Q              one 32-byte sector per grid cell: two float4 halves.  Half PAR(cell) holds
//                  Q_t[cell][0..3] (one vector load = the whole action row), the other half is where
//                  Q_{t+1} of that cell is written, so readers of step t never see a write of step t;
//   cw             one 16-bit word per cell: obstacle, goal, row parity and two 6-bit occupant counters
//                  (this step / next step, saturating), small enough to stay in L2;
//   ent / mailbox  collision entries and chain heads for cells whose occupants are spread over
//                  several warps.
//
// One batched step = two launches:
//   train_main  one thread per slot: epsilon-greedy from a Philox4x32-10 stream keyed by
//               (seed, global env, step) -> move with obstacle/goal lookup -> TD target from Q_t.
//               The warp groups its lanes by cell (match.any).  If the cell's occupant count equals
//               the group size, every occupant is in this warp: the group applies its updates in
//               ascending environment id with shuffles and its leader writes the cell's Q_{t+1} row.
//               Otherwise the lanes append (cell, action, env, td_target) entries, linked inside the
//               group, and the leader hooks the sub-chain into the cell's mailbox chain with one
//               atomicExch.  Then auto-reset, and one saturating count per (warp, next cell) into the
//               next step's counter.
//   train_fix   folds the chained entries of each cell in ascending environment id (fp32 fma chain, no
//               float atomics), flips the row parity of every occupied cell, clears the consumed
//               counter plane and advances the step / epsilon index.
//
// Reference semantics (paths relative to the CudaRL-Arena project root):
//   step        src/environment.cu:17-48, obstacle test src/kernels.cu:29-44, goal src/kernels.cu:56-59
//   reset       src/environment.cu:6-14
//   TD update   src/kernels.cu:96-114 (true max as in src/gpu/kernels.cu:36-45, src/train.py:134)
//   eps-greedy  src/train.py:101-108, first-max argmax src/q_learning.cu:196-206
//   episode     src/train.py:191-222
#include "kernels.cuh"
#include "rules.cuh"
#include <cstdio>

namespace cudarl {

__device__ __forceinline__ unsigned cnt_shift(unsigned long long step) { return (step & 1ull) ? CW_CNT_SHIFT1 : CW_CNT_SHIFT0; }
__device__ __forceinline__ void flip_parity(const Params& p, unsigned cell) {
    atomicXor(reinterpret_cast<unsigned*>(p.cw) + (cell >> 1), CW_PAR << ((cell & 1u) * 16u));
}

// Add `g` occupants to the 6-bit counter (field at `shift`) of `cell`, saturating at 63.
__device__ __forceinline__ void count_add(const Params& p, unsigned cell, unsigned shift, unsigned g) {
    unsigned* w = reinterpret_cast<unsigned*>(p.cw) + (cell >> 1);
    const unsigned sh = shift + (cell & 1u) * 16u;
    unsigned old = *reinterpret_cast<volatile unsigned*>(w);
    for (int it = 0; it < 100000; ++it) {                 // lock-free; the bound only guards against a broken word
        unsigned f = (old >> sh) & CW_CNT_MAX;
        unsigned nf = f + g; if (nf > CW_CNT_MAX) nf = CW_CNT_MAX;
        if (nf == f) return;
        unsigned seen = atomicCAS(w, old, (old & ~(CW_CNT_MAX << sh)) | (nf << sh));
        if (seen == old) return;
        old = seen;
    }
    atomicOr(&p.ctl->error, ERR_CAS_LIMIT);
}

// Same for both cells of a 32-bit pair at once (even cell gets g0, odd cell g1).
// `old` is the caller's last view of the word (a stale view only costs one more round).
__device__ __forceinline__ void count_add2(const Params& p, unsigned pair, unsigned shift, unsigned g0, unsigned g1, unsigned old) {
    unsigned* w = reinterpret_cast<unsigned*>(p.cw) + pair;
    for (int it = 0; it < 100000; ++it) {
        unsigned f0 = (old >> shift) & CW_CNT_MAX, f1 = (old >> (shift + 16u)) & CW_CNT_MAX;
        unsigned n0 = f0 + g0; if (n0 > CW_CNT_MAX) n0 = CW_CNT_MAX;
        unsigned n1 = f1 + g1; if (n1 > CW_CNT_MAX) n1 = CW_CNT_MAX;
        if (n0 == f0 && n1 == f1) return;
        unsigned upd = (old & ~((CW_CNT_MAX << shift) | (CW_CNT_MAX << (shift + 16u)))) | (n0 << shift) | (n1 << (shift + 16u));
        unsigned seen = atomicCAS(w, old, upd);
        if (seen == old) return;
        old = seen;
    }
    atomicOr(&p.ctl->error, ERR_CAS_LIMIT);
}

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

// ------------------------------------------------------------------------------------------------
// Occupancy rebuild (after reset / caller-driven state changes): clear both counters, then every
// environment counts itself into the counter of the CURRENT step.
__global__ void k_occ_clear(Params p) {
    unsigned n16 = (2u * p.S + 15u) / 16u;
    uint4* w = reinterpret_cast<uint4*>(p.cw);
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += gridDim.x * blockDim.x) {
        uint4 v = w[i];
        const unsigned keep = 0x00070007u;
        v.x &= keep; v.y &= keep; v.z &= keep; v.w &= keep;
        w[i] = v;
    }
}
__global__ void k_occ_announce(Params p) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    const int4 r = p.st[i];
    unsigned s = (unsigned)r.y * (unsigned)p.W + (unsigned)r.x;
    count_add(p, s, cnt_shift(p.step), 1u);
}

__global__ void k_reset_all(Params p) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    unsigned e = (unsigned)p.st[i].w;
    unsigned c = sample_start(p, p.env_offset + e, p.step, TAG_START);
    p.st[i] = make_int4((int)(c % (unsigned)p.W), (int)(c / (unsigned)p.W), 0, (int)e);
    if (p.reward) { p.reward[e] = 0.0f; p.done[e] = 0; }
}

// ------------------------------------------------------------------------------------------------
// Slot order.  Counting sort of the slots by cell: count, exclusive scan over the cells, scatter.
// The order inside one cell is whatever the atomics give; nothing depends on it (folds go by id).
// sort key: the cell itself (shift 0) so that environments sharing a cell occupy consecutive slots, which
// is what the warp-level grouping below looks for; coarser keys only when cells vastly outnumber environments
__device__ __forceinline__ unsigned sort_key(const Params& p, int x, int y) { return ((unsigned)y * (unsigned)p.W + (unsigned)x) >> p.sort_shift; }

// Maximal run of consecutive lanes holding the same value `v` as mine: returns its lane mask.
__device__ __forceinline__ unsigned run_mask(unsigned v, unsigned lane) {
    const unsigned up = __shfl_up_sync(FULL, v, 1);
    const unsigned heads = __ballot_sync(FULL, lane == 0u || v != up);       // lanes that start a run
    const unsigned at_or_below = heads & ((2u << lane) - 1u);
    const unsigned start = 31u - __clz(at_or_below);
    const unsigned above = heads & ~((2u << lane) - 1u);
    const unsigned end = above ? (unsigned)__ffs(above) - 2u : 31u;           // last lane of my run
    return ((end == 31u) ? FULL : ((1u << (end + 1u)) - 1u)) & ~((1u << start) - 1u);
}

__global__ void k_ids_identity(Params p) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < p.N) p.st[i].w = (int)i;
}
// The input is nearly ordered already, so neighbouring lanes mostly share a key: one atomic per run of lanes.
__global__ void k_sort_count(Params p) {
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x, lane = threadIdx.x & 31u;
    unsigned key = 0xFFFFFFFFu - lane;
    if (i < p.N) { const int4 r = p.st[i]; key = sort_key(p, r.x, r.y); }
    const unsigned m = run_mask(key, lane);
    if (i < p.N && lane == __ffs(m) - 1u) atomicAdd(p.sort_cnt + key, __popc(m));
}
constexpr unsigned SCAN_CHUNK = 4096;      // keys per block of the scan
// phase 1: per-chunk totals; phase 2 (one block): exclusive scan of the totals; phase 3: exclusive scan inside chunks
__global__ void __launch_bounds__(BLOCK) k_scan_totals(Params p) {
    // the counter array is padded with zeros to a multiple of SCAN_CHUNK, so whole uint4 loads are safe
    __shared__ unsigned s_sum[BLOCK / 32];
    const uint4* c4 = reinterpret_cast<const uint4*>(p.sort_cnt) + blockIdx.x * (SCAN_CHUNK / 4);
    unsigned acc = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) { uint4 v = c4[j * BLOCK + threadIdx.x]; acc += v.x + v.y + v.z + v.w; }
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(FULL, acc, o);
    if ((threadIdx.x & 31) == 0) s_sum[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) { unsigned t = 0; for (int k = 0; k < BLOCK / 32; ++k) t += s_sum[k]; p.sort_blk[blockIdx.x] = t; }
}
__device__ __forceinline__ unsigned block_excl_scan(unsigned v, unsigned* s_warp) {   // exclusive prefix of v over the block
    const unsigned lane = threadIdx.x & 31u, wid = threadIdx.x >> 5;
    unsigned inc = v;
    for (int o = 1; o < 32; o <<= 1) { unsigned t = __shfl_up_sync(FULL, inc, o); if (lane >= (unsigned)o) inc += t; }
    if (lane == 31u) s_warp[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        unsigned w = lane < blockDim.x / 32u ? s_warp[lane] : 0u, winc = w;
        for (int o = 1; o < 32; o <<= 1) { unsigned t = __shfl_up_sync(FULL, winc, o); if (lane >= (unsigned)o) winc += t; }
        if (lane < blockDim.x / 32u) s_warp[lane] = winc - w;
    }
    __syncthreads();
    unsigned r = s_warp[wid] + inc - v;
    __syncthreads();
    return r;
}
__global__ void __launch_bounds__(1024) k_scan_blocks(Params p, unsigned nchunks) {
    __shared__ unsigned s_warp[32];
    __shared__ unsigned s_carry;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (unsigned base = 0; base < nchunks; base += 1024u) {
        unsigned k = base + threadIdx.x;
        unsigned v = k < nchunks ? p.sort_blk[k] : 0u;
        unsigned ex = block_excl_scan(v, s_warp);
        unsigned carry = s_carry;
        if (k < nchunks) p.sort_blk[k] = carry + ex;
        __syncthreads();
        if (threadIdx.x == 1023u) s_carry = carry + ex + v;
        __syncthreads();
    }
}
__global__ void __launch_bounds__(BLOCK) k_scan_chunks(Params p) {
    // four slabs of 256 uint4 (coalesced); each thread scans its 4 keys, the block scans the thread sums
    __shared__ unsigned s_warp[32];
    __shared__ unsigned s_tot;
    uint4* c4 = reinterpret_cast<uint4*>(p.sort_cnt) + blockIdx.x * (SCAN_CHUNK / 4);
    unsigned carry = p.sort_blk[blockIdx.x];
    for (int j = 0; j < 4; ++j) {
        const uint4 v = c4[j * BLOCK + threadIdx.x];
        const unsigned sum = v.x + v.y + v.z + v.w;
        const unsigned ex = block_excl_scan(sum, s_warp);
        if (threadIdx.x == BLOCK - 1) s_tot = ex + sum;
        const unsigned r0 = carry + ex;
        c4[j * BLOCK + threadIdx.x] = make_uint4(r0, r0 + v.x, r0 + v.x + v.y, r0 + v.x + v.y + v.z);
        __syncthreads();
        carry += s_tot;
        __syncthreads();
    }
}
__global__ void k_sort_scatter(Params p) {
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x, lane = threadIdx.x & 31u;
    unsigned key = 0xFFFFFFFFu - lane; int4 r = make_int4(0, 0, 0, 0);
    if (i < p.N) { r = p.st[i]; key = sort_key(p, r.x, r.y); }
    const unsigned m = run_mask(key, lane);
    const unsigned leader = __ffs(m) - 1u;
    unsigned base = 0;
    if (i < p.N && lane == leader) base = atomicAdd(p.sort_cnt + key, __popc(m));   // offsets become cursors
    base = __shfl_sync(FULL, base, leader);
    if (i < p.N) p.st2[base + (lane - leader)] = r;
}

// Second half of the sort: inside every key segment of st2 order the records by (cell, id) and write
// them to st.  Afterwards environments that share a cell sit in consecutive slots in ascending id, which
// is the order their updates are applied in.  Segments longer than RANK_MAX are copied as they are
// (still correct, only slower later: such cells take the sorting path of the fold kernel).
constexpr unsigned RANK_MAX = 4096;
__global__ void k_sort_rank(Params p) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    const int4 r = p.st2[i];
    const unsigned key = sort_key(p, r.x, r.y);
    const unsigned lo = key ? p.sort_cnt[key - 1u] : 0u, hi = p.sort_cnt[key];     // cursors = segment ends after the scatter
    unsigned dst = i;
    if (hi - lo > 1u && hi - lo <= RANK_MAX) {
        const unsigned long long mine = ((unsigned long long)((unsigned)r.y * (unsigned)p.W + (unsigned)r.x) << 32) | (unsigned)r.w;
        unsigned rank = 0;
        for (unsigned j = lo; j < hi; ++j) {
            const int4 o = p.st2[j];
            const unsigned long long k = ((unsigned long long)((unsigned)o.y * (unsigned)p.W + (unsigned)o.x) << 32) | (unsigned)o.w;
            rank += k < mine ? 1u : 0u;
        }
        dst = lo + rank;
    }
    p.st[dst] = r;
}

// st2[id] = st[slot]: back to environment order (slot k = environment k)
__global__ void k_normalize(Params p) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    const int4 r = p.st[i];
    p.st2[r.w] = r;
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
// The fused step: one thread per slot.
template <bool TRACE>
__global__ void __launch_bounds__(BLOCK, 8) k_train_main(Params p) {
    __shared__ unsigned s_cnt, s_goals, s_timeouts, s_shared;
    __shared__ int2 s_pair[BLOCK];
    __shared__ unsigned s_act[BLOCK], s_nact, s_done;
    if (threadIdx.x == 0) { s_cnt = 0; s_goals = 0; s_timeouts = 0; s_shared = 0; s_nact = 0; s_done = 0; }
    __syncthreads();
    const unsigned i = blockIdx.x * BLOCK + threadIdx.x;
    const unsigned lane = threadIdx.x & 31u;
    const unsigned lt = (1u << lane) - 1u;                              // lanes below mine
    if (blockIdx.x == 0 && threadIdx.x == 0) { p.ctl->scratch_cursor = 0; p.ctl->active_count[(p.step + 1ull) & 1ull] = 0; p.ctl->long_count[(p.step + 1ull) & 1ull] = 0; p.ctl->long2_count[(p.step + 1ull) & 1ull] = 0; }   // nobody reads these in this kernel
    const bool valid = i < p.N;
    const unsigned long long g = p.step;
    const unsigned shc = cnt_shift(g), shn = cnt_shift(g + 1ull);
    const float eps = p.eps_tab[p.eps_from_ctl ? p.ctl->eps_idx : p.eps_idx];
    // ---- per-lane work (lanes past the end idle through it with harmless values) ----------------------
    int x = 0, y = 0, t = 0, a = 0, nx = 0, ny = 0; unsigned e = 0, s = 0x80000000u | lane, s2 = 0, par = 0, cnt = 0, wguess = 0;
    float4 row = make_float4(0.f, 0.f, 0.f, 0.f); float d = 0.0f; bool done = false;
    if (valid) {
        const int4 rec = __ldcs(p.st + i);
        x = rec.x; y = rec.y; t = rec.z; e = (unsigned)rec.w;
        s = (unsigned)y * (unsigned)p.W + (unsigned)x;
        const unsigned* cw32 = reinterpret_cast<const unsigned*>(p.cw);
        const unsigned ws = cw32[s >> 1];                     // the 32-bit word holding this cell and its pair mate
        const unsigned cs = (ws >> ((s & 1u) * 16u)) & 0xFFFFu;
        par = (cs & CW_PAR) ? 1u : 0u;
        cnt = (cs >> shc) & CW_CNT_MAX;
        row = __ldcg(p.Q + 2u * s + par);
        // epsilon-greedy
        U4 w = philox4x32_10(p.env_offset + e, 0u, (unsigned)g, (unsigned)(g >> 32), p.k0, p.k1 ^ TAG_POLICY);
        a = (u01(w.x) < eps) ? (int)(w.y & 3u) : argmax4(row);
        // environment transition
        const int dx = (a == 1) - (a == 3), dy = (a == 2) - (a == 0);
        nx = x + dx; ny = y + dy;
        const bool inb = nx >= 0 && nx < p.W && ny >= 0 && ny < p.H;
        const unsigned tgt = inb ? (unsigned)ny * (unsigned)p.W + (unsigned)nx : s;
        const unsigned wt = inb ? cw32[tgt >> 1] : ws;
        const unsigned ct = (wt >> ((tgt & 1u) * 16u)) & 0xFFFFu;
        const bool moved = inb && !(ct & CW_OBST);
        wguess = moved ? wt : ws;                             // what the next cell's word looked like a moment ago
        const unsigned c2 = moved ? ct : cs;
        s2 = moved ? tgt : s; nx = moved ? nx : x; ny = moved ? ny : y;
        done = (c2 & CW_GOAL) != 0;
        const float r = done ? 1.0f : -0.01f;
        float m = 0.0f;
        if (!done) {
            float4 row2 = moved ? __ldcg(p.Q + 2u * s2 + ((c2 & CW_PAR) ? 1u : 0u)) : row;
            m = max4(row2);
            if (p.legacy_clamp && m < 0.0f) m = 0.0f;
        }
        d = __fmaf_rn(p.gamma, m, r);                       // the TD target; the error is taken against the running value in fold()
        if (TRACE) { p.tr_a[e] = a; p.tr_r[e] = r; p.tr_d[e] = done ? 1 : 0; }
    }
    // ---- TD update: consecutive lanes of the warp that stand on the same cell form a group -------------
    const unsigned gmask = run_mask(s, lane);      // consecutive slots on the same cell (the slot order is by cell)
    const unsigned gsize = __popc(gmask), gleader = __ffs(gmask) - 1u;
    // every occupant of the cell is in this group <=> the cell's counter equals the group size
    const bool complete = valid && cnt == gsize && gsize < CW_CNT_MAX;
    {
        // Apply the group's updates in ascending environment id.  The slot order is (cell, id) as of the
        // last re-ordering, so normally the lanes of a run already are in id order and the run's first lane
        // simply applies the (action, td_target) pairs its lanes parked in shared memory.  If some complete run
        // of the warp is out of order (environments met since), every lane first ranks its id inside its run
        // with full-warp shuffles at growing distances and parks its pair at its rank.
        const unsigned gend = gleader + gsize - 1u;
        const unsigned up_e = __shfl_up_sync(FULL, e, 1);
        const unsigned disorder = __ballot_sync(FULL, complete && lane > gleader && e < up_e);
        unsigned rank = lane - gleader;
        if (disorder) {                                     // warp-uniform
            const unsigned maxlen = __reduce_max_sync(FULL, complete ? gsize : 0u);
            rank = 0;
            for (unsigned off = 1; off < maxlen; ++off) {
                const unsigned eu = __shfl_up_sync(FULL, e, off), ed = __shfl_down_sync(FULL, e, off);
                rank += (lane >= gleader + off && eu < e) ? 1u : 0u;
                rank += (lane + off <= gend && ed < e) ? 1u : 0u;
            }
        }
        const unsigned wbase = threadIdx.x & ~31u;
        if (complete && gsize > 1u) s_pair[wbase + gleader + rank] = make_int2(a, __float_as_int(d));
        __syncwarp();
        if (complete && lane == gleader) {
            if (gsize == 1u) fold(row, a, p.lr, d);
            else for (unsigned k = 0; k < gsize; ++k) { const int2 pr = s_pair[wbase + gleader + k]; fold(row, pr.x, p.lr, __int_as_float(pr.y)); }
            p.Q[2u * s + (par ^ 1u)] = row;                                   // Q_{t+1} row of the cell
        }
    }
    {
        // occupants in other warps too: the run's lanes write consecutive entries and the run's first lane
        // hooks the whole run into the cell's chain with one exchange
        const bool gen = valid && !complete;
        const unsigned genmask = __ballot_sync(FULL, gen);
        if (genmask) {
            unsigned base = 0;
            if (lane == __ffs(genmask) - 1u) base = atomicAdd(&s_cnt, __popc(genmask));
            base = __shfl_sync(FULL, base, __ffs(genmask) - 1);
            const unsigned pos = blockIdx.x * BLOCK + base + __popc(genmask & lt);      // a run's lanes get consecutive positions
            unsigned prev = 0u;
            if (gen && lane == gleader) {
                prev = atomicExch(p.mailbox + mb_slot(p, s), ((gsize - 1u) << LINK_POS_BITS) | (pos + 1u));
                if (!prev) s_act[atomicAdd(&s_nact, 1u)] = mb_slot(p, s);    // first chain on this slot in this step
            }
            if (gen) p.ent[pos] = make_uint4((s << 3) | (par << 2) | (unsigned)a, e, __float_as_uint(d), prev);
        }
    }
    // ---- episode bookkeeping, next-step occupancy, state out ----------------------------------------------
    unsigned sn = 0x80000000u | lane;
    const bool timeout = valid && !done && p.max_steps > 0 && t + 1 >= p.max_steps;
    if (valid) {
        int nt = t + 1;
        sn = s2;
        if (done || timeout) {
            sn = sample_start(p, p.env_offset + e, g + 1ull, TAG_START);
            nx = (int)(sn % (unsigned)p.W); ny = (int)(sn / (unsigned)p.W); nt = 0;
            wguess = reinterpret_cast<const unsigned*>(p.cw)[sn >> 1];
        }
        __stcs(p.st + i, make_int4(nx, ny, nt, (int)e));
    }
    {
        // neighbours whose next cells share a 32-bit cell-word pair announce together: one CAS per pair
        const unsigned wmask = run_mask(sn >> 1, lane);
        const unsigned odd = __ballot_sync(FULL, (sn & 1u) != 0u);
        if (valid && lane == __ffs(wmask) - 1u) count_add2(p, sn >> 1, shn, __popc(wmask & ~odd), __popc(wmask & odd), wguess);
    }
    if (valid && done) atomicAdd(&s_goals, 1u);                 // rare events
    if (timeout) atomicAdd(&s_timeouts, 1u);
    {
        const unsigned ms = __ballot_sync(FULL, valid && cnt >= 2u);
        if (lane == 0 && ms) atomicAdd(&s_shared, __popc(ms));
    }
    // No block barrier at the end: the last warp of the block to get here publishes the block's
    // counters and its list of newly active slots, so finished warps free their slots right away.
    __syncwarp();
    unsigned last = 0;
    if (lane == 0) { __threadfence_block(); last = (atomicAdd(&s_done, 1u) == BLOCK / 32 - 1) ? 1u : 0u; }
    last = __shfl_sync(FULL, last, 0);
    if (last) {
        __threadfence_block();
        const unsigned nact = *(volatile unsigned*)&s_nact;
        if (nact) {
            unsigned base = 0;
            if (lane == 0) base = atomicAdd(&p.ctl->active_count[p.step & 1ull], nact);
            base = __shfl_sync(FULL, base, 0);
            for (unsigned k = lane; k < nact; k += 32u) p.active[base + k] = ((volatile unsigned*)s_act)[k];
        }
        if (lane == 0) {
            const unsigned sh = *(volatile unsigned*)&s_shared, cn = *(volatile unsigned*)&s_cnt;
            const unsigned go = *(volatile unsigned*)&s_goals, to = *(volatile unsigned*)&s_timeouts;
            if (sh) atomicAdd(&p.ctl->conflicts, (unsigned long long)sh);
            if (cn) atomicAdd(&p.ctl->general, (unsigned long long)cn);
            if (go) atomicAdd(&p.ctl->goals, (unsigned long long)go);
            if (to) atomicAdd(&p.ctl->timeouts, (unsigned long long)to);
            if (go + to) atomicAdd(&p.ctl->episodes, (unsigned long long)(go + to));
        }
    }
}

// Per-episode epsilon schedule: the table index follows the number of finished episodes, which only
// the device knows.  One thread, launched after each step in that mode only.
__global__ void k_eps_episode(Params p) {
    Ctl* c = p.ctl;
    c->eps_used = p.eps_tab[c->eps_idx];
    unsigned long long kk = c->episodes / (unsigned long long)p.N;
    unsigned long long rel = kk > c->eps_base_k ? kk - c->eps_base_k : 0ull;
    c->eps_idx = (unsigned)(rel < (unsigned long long)(c->eps_len - 1u) ? rel : (unsigned long long)(c->eps_len - 1u));
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
    if (FLIP) flip_parity(p, cell);
}

constexpr unsigned LONG_SMEM = 1024;   // chain entries sorted in shared memory; longer chains use the global scratch
constexpr int SHORT_MAX = 8;           // chain entries folded in registers by one thread

// One long chain, whole block: count its entries (one hop per run), pick shared memory or a slice of the
// global scratch, copy the runs (one warp per run, batches of 256 runs), bitonic-sort by (cell, action, id)
// and let the first thread of every cell run fold it.
template <bool FLIP>
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

// Collision folding, one thread per ACTIVE mailbox slot (the producers list every slot they were the
// first to hook a chain into, so this kernel only visits slots that have work).  A slot's chain links
// RUNS of consecutive entries (one run = the lanes of one warp on one cell).  The owning thread gathers
// the chain's entries:
//   <= 8 entries   in registers, ordered by a sorting network and folded by that thread;
//   <= 32 entries  staged in shared memory by that thread, ordered and folded by one warp;
//   longer         queued for k_fix_long (one warp per chain up to 256 entries, then one block per chain).
// TRAIN = true : part of a train step -- also sweeps the cell words (parity ^= occupied, consumed
//                counter cleared).
// TRAIN = false: update_batch -- flips the row parity of every folded cell instead.
template <bool FLIP>
__device__ __forceinline__ void flush_row(const Params& p, unsigned cellpar, const float4& row) {
    const unsigned cell = cellpar >> 1, par = cellpar & 1u;
    p.Q[2u * cell + (par ^ 1u)] = row;
    if (FLIP) flip_parity(p, cell);
}

template <bool TRAIN>
__global__ void __launch_bounds__(BLOCK) k_fix(Params p) {
    constexpr bool FLIP = !TRAIN;
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
                        if (curcp != 0xFFFFFFFFu) flush_row<FLIP>(p, curcp, row);
                        curcp = cp; row = __ldcg(p.Q + 2u * (cp >> 1) + (cp & 1u));
                    }
                    fold(row, (int)(w0 & 3u), p.lr, v8[j]);
                }
            }
            if (curcp != 0xFFFFFFFFu) flush_row<FLIP>(p, curcp, row);
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
            if (L) process_medium<FLIP>(p, s_keys + c * MED_MAX, s_vals + c * MED_MAX, L);
        }
    }
    __syncthreads();
  }

    if (TRAIN) {
        // sweep: parity ^= (counter of this step != 0), then clear that counter (it becomes the
        // "next step" counter of the following step)
        const unsigned n16 = (2u * p.S + 15u) / 16u;
        const unsigned shc = cnt_shift(p.step);
        const unsigned fmask = (CW_CNT_MAX << shc) | (CW_CNT_MAX << (shc + 16u));
        const unsigned low = (1u << shc) | (1u << (shc + 16u));
        uint4* wv = reinterpret_cast<uint4*>(p.cw);
        for (unsigned i = blockIdx.x * BLOCK + threadIdx.x; i < n16; i += gridDim.x * BLOCK) {
            uint4 v = wv[i];
#define CUDARL_SWEEP(w) { unsigned f_ = w & fmask; if (f_) { unsigned nz_ = (f_ | (f_ >> 1) | (f_ >> 2) | (f_ >> 3) | (f_ >> 4) | (f_ >> 5)) & low; \
                            w = (w ^ ((nz_ >> shc) << 2)) & ~fmask; } }
            const uint4 o = v;
            CUDARL_SWEEP(v.x); CUDARL_SWEEP(v.y); CUDARL_SWEEP(v.z); CUDARL_SWEEP(v.w);
#undef CUDARL_SWEEP
            if (o.x != v.x || o.y != v.y || o.z != v.z || o.w != v.w) wv[i] = v;
        }
    }
}

// Long chains (more than 32 entries: cells crowded with environments).  First tier: one WARP per chain for up
// to 256 entries -- lane 0 hops from run to run, all lanes copy the run's entries into the warp's slice of
// shared memory, a warp-wide bitonic sort orders them by (cell, action, id), the first lane of every cell run
// applies it.  Chains that do not fit are queued for k_fix_long2 (one block per chain).
constexpr unsigned WARP_LONG = 256;

template <bool FLIP>
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
        if (j == 0 || (unsigned)(keys[j - 1] >> 34) != cp) apply_run<FLIP>(p, keys, vals, j, L);
    }
    __syncwarp();
    return true;
}

template <bool FLIP>
__global__ void __launch_bounds__(BLOCK) k_fix_long(Params p) {
    __shared__ unsigned long long s_keys[(BLOCK / 32) * WARP_LONG];
    __shared__ float s_vals[(BLOCK / 32) * WARP_LONG];
    const unsigned n = p.ctl->long_count[p.step & 1ull];
    const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    unsigned done = 0;
    for (unsigned c = blockIdx.x * (BLOCK / 32) + warp; c < n; c += gridDim.x * (BLOCK / 32)) {
        const unsigned head = p.longq[c];
        if (!process_long_warp<FLIP>(p, head, s_keys + warp * WARP_LONG, s_vals + warp * WARP_LONG)) {
            if (lane == 0) p.longq2[atomicAdd(&p.ctl->long2_count[p.step & 1ull], 1u)] = head;
        }
        ++done;
    }
    if (lane == 0 && done) atomicAdd(&p.ctl->long_chains, (unsigned long long)done);
}

// Second tier: one block per chain, any length (shared memory up to 1024 entries, the global scratch beyond).
template <bool FLIP>
__global__ void __launch_bounds__(BLOCK) k_fix_long2(Params p) {
    __shared__ unsigned long long s_keys[LONG_SMEM];
    __shared__ float s_vals[LONG_SMEM];
    __shared__ unsigned s_bcast[3];
    const unsigned n = p.ctl->long2_count[p.step & 1ull];
    for (unsigned c = blockIdx.x; c < n; c += gridDim.x) process_long<FLIP>(p, p.longq2[c], s_keys, s_vals, s_bcast);
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
    float r = -0.01f; unsigned char dn = p.done[e];
    if (c2 & CW_GOAL) { r = 1.0f; dn = 1; }
    p.st[i] = make_int4((int)(s2 % (unsigned)p.W), (int)(s2 / (unsigned)p.W), rec.z + 1, rec.w);
    p.reward[e] = r; p.done[e] = dn;
    if (rewards) rewards[e] = r;
    if (dones) dones[e] = dn;
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
        unsigned cs = cw_load(p.cw, s);
        unsigned steps = 0; bool reached = false;
        for (int k = 0; k < max_steps; ++k) {
            float4 row = __ldg(p.Q + 2u * s + ((cs & CW_PAR) ? 1u : 0u));
            int a = argmax4(row);
            int x = (int)(s % (unsigned)p.W), y = (int)(s / (unsigned)p.W);
            unsigned c2; unsigned s2 = move_cell(p, x, y, s, cs, a, c2);
            ++steps; s = s2; cs = c2;
            if (c2 & CW_GOAL) { reached = true; break; }
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
        unsigned cs = cw_load(p.cw, s);
        unsigned par = (cs & CW_PAR) ? 1u : 0u;
        float4 row = __ldcg(p.Q + 2u * s + par);
        float m = 0.0f;
        if (!dn[i]) {
            unsigned c2 = cw_load(p.cw, s2);
            m = max4(__ldcg(p.Q + 2u * s2 + ((c2 & CW_PAR) ? 1u : 0u)));
            if (p.legacy_clamp && m < 0.0f) m = 0.0f;
        }
        float d = __fmaf_rn(p.gamma, m, rew[i]);           // TD target
        slot = mb_slot(p, s);
        unsigned prev = atomicExch(p.mailbox + slot, i + 1u);          // a run of one entry
        p.ent[i] = make_uint4((s << 3) | (par << 2) | (unsigned)a, i, __float_as_uint(d), prev);
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
// Table in the caller's layout: dense[(y*W+x)] = float4 of the 4 action values.
__global__ void k_q_gather(Params p, float4* dense) {
    unsigned s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= p.S) return;
    dense[s] = p.Q[2u * s + ((p.cw[s] & CW_PAR) ? 1u : 0u)];
}
__global__ void k_q_scatter(Params p, const float4* dense, float scale) {
    unsigned s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= p.S) return;
    float4 v = dense[s];
    v.x = __fmul_rn(v.x, scale); v.y = __fmul_rn(v.y, scale); v.z = __fmul_rn(v.z, scale); v.w = __fmul_rn(v.w, scale);
    p.Q[2u * s + ((p.cw[s] & CW_PAR) ? 1u : 0u)] = v;
}
// Replica averaging, second half: `gathered` holds the rows [cell0, cell0+n) of every rank's table, rank after
// rank.  Sum them in rank order 0..R-1 in fp32 (the order of the CPU oracle, whatever the transport did),
// scale by 1/R and store into the current half.
__global__ void k_q_average(Params p, const float4* gathered, unsigned R, unsigned cell0, unsigned n, float scale) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float4 acc = gathered[i];
    for (unsigned r = 1; r < R; ++r) {
        const float4 v = gathered[(size_t)r * n + i];
        acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
    }
    acc.x = __fmul_rn(acc.x, scale); acc.y = __fmul_rn(acc.y, scale); acc.z = __fmul_rn(acc.z, scale); acc.w = __fmul_rn(acc.w, scale);
    const unsigned s = cell0 + i;
    p.Q[2u * s + ((p.cw[s] & CW_PAR) ? 1u : 0u)] = acc;
}
__global__ void k_q_gather_range(Params p, float4* dense, unsigned cell0, unsigned n) {
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned s = cell0 + i;
    dense[i] = p.Q[2u * s + ((p.cw[s] & CW_PAR) ? 1u : 0u)];
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
__global__ void k_cell_set(Params p, unsigned cell, unsigned cls, int clear_goals) {
    unsigned* w32 = reinterpret_cast<unsigned*>(p.cw);
    if (clear_goals) {
        unsigned n2 = (p.S + 1u) / 2u;
        for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += gridDim.x * blockDim.x)
            atomicAnd(w32 + i, ~0x00020002u);
    } else if (blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned sh = (cell & 1u) * 16u;
        atomicAnd(w32 + (cell >> 1), ~(3u << sh));
        if (cls) atomicOr(w32 + (cell >> 1), cls << sh);
    }
}

// ------------------------------------------------------------------------------------------------
static inline unsigned nblk(unsigned n) { return (n + BLOCK - 1) / BLOCK; }
static inline unsigned fix_blocks(const Params& p) { unsigned b = p.mb_slots / BLOCK; return b > 1184u ? 1184u : b; }
static inline unsigned sweep_blocks(unsigned S) { unsigned b = nblk((2u * S + 15u) / 16u); return b < 1u ? 1u : (b > 1184u ? 1184u : b); }

void launch_rebuild_occupancy(const Params& p, cudaStream_t st) {
    k_occ_clear<<<sweep_blocks(p.S), BLOCK, 0, st>>>(p);
    if (p.N) k_occ_announce<<<nblk(p.N), BLOCK, 0, st>>>(p);
}
void launch_identity_ids(const Params& p, cudaStream_t st) { if (p.N) k_ids_identity<<<nblk(p.N), BLOCK, 0, st>>>(p); }
void launch_export_state(const Params& p, cudaStream_t st) { if (p.N) k_export_state<<<nblk(p.N), BLOCK, 0, st>>>(p); }
void launch_normalize(const Params& p, cudaStream_t st) { if (p.N) k_normalize<<<nblk(p.N), BLOCK, 0, st>>>(p); }
void launch_import_state(const Params& p, const int* x, const int* y, const int* t, cudaStream_t st) { if (p.N) k_import_state<<<nblk(p.N), BLOCK, 0, st>>>(p, x, y, t); }
void launch_sort_by_cell(const Params& p, cudaStream_t st) {
    if (!p.N) return;
    unsigned nchunks = (p.nkeys + SCAN_CHUNK - 1) / SCAN_CHUNK;
    cudaMemsetAsync(p.sort_cnt, 0, (size_t)nchunks * SCAN_CHUNK * sizeof(unsigned), st);
    k_sort_count<<<nblk(p.N), BLOCK, 0, st>>>(p);
    k_scan_totals<<<nchunks, BLOCK, 0, st>>>(p);
    k_scan_blocks<<<1, 1024, 0, st>>>(p, nchunks);
    k_scan_chunks<<<nchunks, BLOCK, 0, st>>>(p);
    k_sort_scatter<<<nblk(p.N), BLOCK, 0, st>>>(p);
    k_sort_rank<<<nblk(p.N), BLOCK, 0, st>>>(p);     // result is back in p.st
}
void launch_reset_all(const Params& p, cudaStream_t st) {
    if (p.N) k_reset_all<<<nblk(p.N), BLOCK, 0, st>>>(p);
}
void launch_train_step(const Params& p, bool trace, cudaStream_t st, cudaEvent_t ev_a, cudaEvent_t ev_b, cudaEvent_t ev_c) {
    if (ev_a) cudaEventRecord(ev_a, st);
    if (trace) k_train_main<true><<<p.nblocks_main, BLOCK, 0, st>>>(p);
    else       k_train_main<false><<<p.nblocks_main, BLOCK, 0, st>>>(p);
    if (ev_b) cudaEventRecord(ev_b, st);
    k_fix<true><<<fix_blocks(p), BLOCK, 0, st>>>(p);
    k_fix_long<false><<<296, BLOCK, 0, st>>>(p);
    k_fix_long2<false><<<296, BLOCK, 0, st>>>(p);
    if (p.eps_from_ctl) k_eps_episode<<<1, 1, 0, st>>>(p);
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
    k_active_reset<<<1, 1, 0, st>>>(p);
    k_update_main<<<nblk(n), BLOCK, 0, st>>>(p, n, sx, sy, a, r, nx, ny, dn);
    k_fix<false><<<fix_blocks(p), BLOCK, 0, st>>>(p);
    k_fix_long<true><<<296, BLOCK, 0, st>>>(p);
    k_fix_long2<true><<<296, BLOCK, 0, st>>>(p);
    k_active_reset<<<1, 1, 0, st>>>(p);      // a following train step starts from an empty list
}
void launch_q_gather(const Params& p, float4* dense, cudaStream_t st) { k_q_gather<<<nblk(p.S), BLOCK, 0, st>>>(p, dense); }
void launch_q_scatter(const Params& p, const float4* dense, float scale, cudaStream_t st) { k_q_scatter<<<nblk(p.S), BLOCK, 0, st>>>(p, dense, scale); }
void launch_q_gather_range(const Params& p, float4* dense, unsigned cell0, unsigned n, cudaStream_t st) { if (n) k_q_gather_range<<<nblk(n), BLOCK, 0, st>>>(p, dense, cell0, n); }
void launch_q_average(const Params& p, const float4* gathered, unsigned R, unsigned cell0, unsigned n, float scale, cudaStream_t st) {
    if (n) k_q_average<<<nblk(n), BLOCK, 0, st>>>(p, gathered, R, cell0, n, scale);
}
void launch_q_init(const Params& p, int kind, float scale, cudaStream_t st) { k_q_init<<<nblk(p.S), BLOCK, 0, st>>>(p, kind, scale); }
void launch_cell_set(const Params& p, unsigned cell, unsigned cls, int clear_goals, cudaStream_t st) {
    k_cell_set<<<clear_goals ? sweep_blocks(p.S) : 1, BLOCK, 0, st>>>(p, cell, cls, clear_goals);
}

}  // namespace cudarl
