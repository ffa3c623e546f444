// tile_engine.cu -- the fused train step as a streaming pass over the grid, one tile at a time.
//
// With a quarter as many environments as cells, nearly every 128-byte line of the table is touched in
// every step, so the step is organised around the TABLE, not around the environments:
//
//   * the grid is cut into T x T tiles; the environments are kept bucketed by tile (records {x,y,t,id});
//   * a tile of Q_t plus a one-cell halo is brought into shared memory by bulk asynchronous copies, one
//     per table row (the halo serves the max over Q_t[s'] of moves that leave the tile), together with the
//     tile's cell classes and its records;
//   * every environment of the tile is stepped against shared memory: epsilon-greedy from the Philox
//     stream keyed by (seed, global env, step), move with obstacle / goal lookup, auto-reset;
//   * the TD updates of a cell are applied from a histogram of (cell, action) counts: inside one step the
//     target of an update depends on (cell, action) only, so n environments on one (cell, action) mean the
//     same map applied n times -- the same bits as the oracle's sequential order, without sorting anything
//     and without float atomics;
//   * the tile of Q_{t+1} goes out to the OTHER dense table, one bulk copy per row (two dense tables
//     alternate, so no block ever sees a neighbour's writes of the same step);
//   * an environment that stays in the tile is appended to the front part of the tile's region of the
//     other record array; one that leaves (a walk across the edge, a restart anywhere) is appended to
//     the back part of its new tile's region with one atomic; a full back part spills to a global list
//     that every block filters.  Regions are re-sized from the actual populations every few steps.
//
// Reference semantics (paths relative to the CudaRL-Arena project root):
//   step        src/environment.cu:17-48, obstacle test src/kernels.cu:29-44, goal src/kernels.cu:56-59
//   TD update   src/kernels.cu:96-114 (true max as in src/gpu/kernels.cu:36-45, src/train.py:134)
//   eps-greedy  src/train.py:101-108, first-max argmax src/q_learning.cu:196-206
//   episode     src/train.py:191-222
#include "kernels.cuh"
#include "rules.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace cudarl {

constexpr unsigned CROWDED_CELL = 24;   // a cell with more environments than this counts as "crowded" in the run statistics

__device__ __forceinline__ unsigned tile_of(const TileP& tp, int x, int y) {
    return ((unsigned)y >> tp.tshift) * tp.tiles_x + ((unsigned)x >> tp.tshift);
}

// Exclusive prefix of v over the block (any block size up to 1024); *total receives the block sum.
__device__ __forceinline__ unsigned block_scan_excl(unsigned v, unsigned* s_warp, unsigned* total) {
    const unsigned lane = threadIdx.x & 31u, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    unsigned inc = v;
    for (int o = 1; o < 32; o <<= 1) { const unsigned t = __shfl_up_sync(FULL, inc, o); if (lane >= (unsigned)o) inc += t; }
    if (lane == 31u) s_warp[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        const unsigned w = lane < nw ? s_warp[lane] : 0u; unsigned winc = w;
        for (int o = 1; o < 32; o <<= 1) { const unsigned t = __shfl_up_sync(FULL, winc, o); if (lane >= (unsigned)o) winc += t; }
        if (lane < nw) s_warp[lane] = winc - w;
        if (lane == 31u) s_warp[32] = winc;
    }
    __syncthreads();
    const unsigned r = s_warp[wid] + inc - v;
    *total = s_warp[32];
    __syncthreads();
    return r;
}

// ---- asynchronous bulk copies (global <-> shared, no registers, no per-element instructions) -------------
// Every source / destination here is a row of float4 (or the tile's class bytes padded to 16): 16-byte
// aligned on both sides, sizes multiples of 16.
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0u;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit_wait_read() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

constexpr unsigned WAIT_LIMIT = 1u << 22;    // polls of the copy barrier before the block gives up and flags an error

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
// Wait for the phase with the given parity; false if the poll limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    for (unsigned it = 0; it < WAIT_LIMIT; ++it) if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// ------------------------------------------------------------------------------------------------
// Why no ordering is needed.  The oracle applies the updates of one (cell, action) one after the other in
// ascending environment id, each as  q <- fma(lr, target - q, q).  Inside one fused step the target of an
// update is a function of (cell, action) alone: the action fixes the next cell (the grid is static), the next
// cell fixes reward and done, and the bootstrap value is the max over Q_t of that next cell.  So all updates of
// one (cell, action) apply the SAME map, and applying it n times gives the same bits in any order; updates of
// different actions touch different components.  The step therefore only has to count, per cell and action,
// how many environments chose it -- a histogram in shared memory -- and then apply each map that many times.
// (update_batch takes arbitrary caller transitions, so it keeps its ordered fold.)
//
// The step kernel is persistent: a block walks over tiles blockIdx, blockIdx + gridDim, ...  It has eight
// CONSUMER warps, which do all the arithmetic on shared memory, and one PRODUCER warp (each lane issues the
// copies of one or two table rows), which only moves data: while the consumers work on tile k in one stage of shared memory, the producer has
// the bulk copies of tile k+1 in flight into the other stage and the rows of tile k-1 on their way out.
//
// Per stage:  s_q    HS*HS float4   Q_t of the tile and its halo; the consumers turn the interior into
//                                   Q_{t+1} in place once every read of Q_t is done
//             s_rec  RC    int4     the first records of the front part of the tile's region
//             s_recb RCB   int4     the first records of the back part
//             s_cls  HS*HS u8       cell classes of the tile and its halo
// Consumer work space, shared by both stages:
//             s_n    T*T   u64      per cell: how many environments chose action a, 16 bits per action
//             s_list T*T   u16      occupied cells
//             s_flag T*T/32 u32     one bit per cell: already listed
// A tile with more than 65,535 records counts in 32-bit counters in global scratch instead.
// full[stage] : the producer's copies have landed (transaction barrier);  done[stage] : every consumer thread
// has finished the tile in that stage.
constexpr unsigned NSTAGE = 2;           // shared-memory stages per block: tiles loaded ahead of the consumers
constexpr unsigned CONSUMERS = 256;      // consumer threads per block (+ 32 of the producer warp)
// Records staged in shared memory (front part, back part of the region); the rest is read from global memory.
__host__ __device__ constexpr unsigned rc_front(unsigned ct) { return ct + ct / 4u + 32u; }
__host__ __device__ constexpr unsigned rc_back(unsigned ct) { return ct / 4u + 32u; }
constexpr unsigned NMAX16 = 65535u;  // records of a tile the 16-bit counters can hold

struct TileHdr {                     // what the producer tells the consumers about the tile in a stage
    unsigned tile, roff, fcap, n_front, n_in, n_all, nf_s, nb_s;
    int tx0, ty0;
};

template <unsigned CT> __device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" :: "n"(CT) : "memory"); }

// Everything the per-environment step needs about the tile being processed.
struct StepCtx {
    const float4* s_q; const unsigned char* s_cls;
    int tx0, ty0; unsigned tile, roff, fcap;
    float eps; unsigned long long g;
    int4* out; int4* ovf_out; unsigned* arr_next; unsigned* ovf_cnt_next;
    unsigned* s_stay; unsigned* s_goals; unsigned* s_timeouts;
};

// One environment, one step: epsilon-greedy action, move, episode bookkeeping; writes the record of the next
// step to the region of the tile it will stand on.  Returns the cell (tile-local) and the action.
// false: the record does not lie in this tile (never seen; flagged by the caller).
template <bool TRACE, unsigned TSH>
__device__ __forceinline__ bool step_env(const Params& p, const StepCtx& c, const int4 rec, unsigned& ic, unsigned& act) {
    constexpr unsigned T = 1u << TSH, HS = T + 2u;
    const TileP& tp = p.tp;
    const int x = rec.x, y = rec.y, t = rec.z; const unsigned e = (unsigned)rec.w;
    const unsigned lx = (unsigned)(x - c.tx0), ly = (unsigned)(y - c.ty0);
    if (lx >= T || ly >= T) return false;
    ic = (ly << TSH) + lx;
    const unsigned hh = (ly + 1u) * HS + lx + 1u;
    const U4 w = philox4x32_10(p.env_offset + e, 0u, (unsigned)c.g, (unsigned)(c.g >> 32), p.k0, p.k1 ^ TAG_POLICY);
    const int a = (u01(w.x) < c.eps) ? (int)(w.y & 3u) : argmax4(c.s_q[hh]);
    act = (unsigned)a;
    const int dx = (a == 1) - (a == 3), dy = (a == 2) - (a == 0);
    int nx = x + dx, ny = y + dy;
    const bool inb = nx >= 0 && nx < p.W && ny >= 0 && ny < p.H;
    const unsigned ht = (unsigned)((int)hh + dy * (int)HS + dx);          // inside the halo whenever the move is in bounds
    const bool moved = inb && !(c.s_cls[inb ? ht : hh] & CW_OBST);
    nx = moved ? nx : x; ny = moved ? ny : y;
    const bool done = (c.s_cls[moved ? ht : hh] & CW_GOAL) != 0;
    if (TRACE) { p.tr_a[e] = a; p.tr_r[e] = done ? 1.0f : -0.01f; p.tr_d[e] = done ? 1 : 0; }
    // episode bookkeeping and the record of the next step
    const bool timeout = !done && p.max_steps > 0 && t + 1 >= p.max_steps;
    int nt = t + 1;
    if (done || timeout) {
        const unsigned sn = sample_start(p, p.env_offset + e, c.g + 1ull, TAG_START);
        nx = (int)(sn % (unsigned)p.W); ny = (int)(sn / (unsigned)p.W); nt = 0;
        atomicAdd(done ? c.s_goals : c.s_timeouts, 1u);
    }
    const int4 nrec = make_int4(nx, ny, nt, (int)e);
    const unsigned dt = ((unsigned)ny >> TSH) * tp.tiles_x + ((unsigned)nx >> TSH);
    bool placed = false;
    if (dt == c.tile) {
        cg::coalesced_group cgp = cg::coalesced_threads();
        unsigned pos = 0;
        if (cgp.thread_rank() == 0) pos = atomicAdd(c.s_stay, cgp.size());
        pos = cgp.shfl(pos, 0) + cgp.thread_rank();
        if (pos < c.fcap) { c.out[c.roff + pos] = nrec; placed = true; }
    }
    if (!placed) {
        const unsigned doff = tp.reg_off[dt], dfc = tp.front_cap[dt], dbc = tp.reg_off[dt + 1u] - doff - dfc;
        const unsigned pos = atomicAdd(&c.arr_next[dt], 1u);
        if (pos < dbc) c.out[doff + dfc + pos] = nrec;
        else {
            const unsigned q = atomicAdd(c.ovf_cnt_next, 1u);
            if (q < p.N) c.ovf_out[q] = nrec; else atomicOr(&p.ctl->error, ERR_BAD_STATE);
        }
    }
    return true;
}

// Q_{t+1} row of one cell from Q_t (still intact in s_q) and the number of environments that chose each action
// (`w`: 16 bits per action, or `n32` when the tile counts in 32 bits).  Only the actions that were chosen are visited.
template <unsigned TSH>
__device__ __forceinline__ float4 updated_row(const Params& p, const StepCtx& c, unsigned ic, unsigned long long w, const unsigned* n32) {
    constexpr unsigned T = 1u << TSH, HS = T + 2u;
    const unsigned lx = ic & (T - 1u), ly = ic >> TSH, hh = (ly + 1u) * HS + lx + 1u;
    const int x = c.tx0 + (int)lx, y = c.ty0 + (int)ly;
    float4 row = c.s_q[hh];
    unsigned mask = n32 ? ((n32[0] != 0u) | ((n32[1] != 0u) << 1) | ((n32[2] != 0u) << 2) | ((n32[3] != 0u) << 3))
                        : (((w & 0xFFFFull) != 0ull) | (((w >> 16) & 0xFFFFull) != 0ull) << 1 | (((w >> 32) & 0xFFFFull) != 0ull) << 2 | ((w >> 48) != 0ull) << 3);
    while (mask) {
        const int a = __ffs((int)mask) - 1; mask &= mask - 1u;
        const unsigned n = n32 ? n32[a] : (unsigned)(w >> (16 * a)) & 0xFFFFu;
        const int dx = (a == 1) - (a == 3), dy = (a == 2) - (a == 0);
        const int nx = x + dx, ny = y + dy;
        const bool inb = nx >= 0 && nx < p.W && ny >= 0 && ny < p.H;
        const unsigned ht = (unsigned)((int)hh + dy * (int)HS + dx);
        const bool moved = inb && !(c.s_cls[inb ? ht : hh] & CW_OBST);
        const unsigned h2 = moved ? ht : hh;
        const bool done = (c.s_cls[h2] & CW_GOAL) != 0;
        float m = 0.0f;
        if (!done) { m = max4(c.s_q[h2]); if (p.legacy_clamp && m < 0.0f) m = 0.0f; }
        const float d = __fmaf_rn(p.gamma, m, done ? 1.0f : -0.01f);     // the TD target of (cell, a), from Q_t
        float v = pick(row, a);
        for (unsigned i = 0; i < n; ++i) v = __fmaf_rn(p.lr, __fsub_rn(d, v), v);       // one application per environment
        row.x = a == 0 ? v : row.x; row.y = a == 1 ? v : row.y; row.z = a == 2 ? v : row.z; row.w = a == 3 ? v : row.w;
    }
    return row;
}

template <bool TRACE, unsigned TSH, unsigned CT>
__global__ void __launch_bounds__(CT + 32u, 3) k_tile_step(Params p) {
    constexpr unsigned T = 1u << TSH, HS = T + 2u, T2 = T * T, HS2 = HS * HS;
    constexpr unsigned RC = rc_front(CT), RCB = rc_back(CT);
    constexpr unsigned CPT = (T2 + CT - 1u) / CT;              // cells per consumer thread when every cell is occupied
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_full[NSTAGE], s_done[NSTAGE];
    __shared__ TileHdr s_hdr[NSTAGE];
    __shared__ unsigned s_stay, s_nocc, s_base, s_abort;
    __shared__ unsigned s_goals, s_timeouts, s_conf, s_nbig, s_nbigent, s_bad;     // accumulated over the block's tiles

    const TileP& tp = p.tp;
    const unsigned stage_bytes = HS2 * 16u + RC * 16u + RCB * 16u + tp.cls_stride;
    unsigned long long* s_n = reinterpret_cast<unsigned long long*>(smem + NSTAGE * stage_bytes);
    unsigned short* s_list = reinterpret_cast<unsigned short*>(s_n + T2);
    unsigned* s_flag = reinterpret_cast<unsigned*>(s_list + T2);       // one bit per cell: listed

    const unsigned tid = threadIdx.x, lane = tid & 31u;
    const unsigned long long g = p.step;
    const unsigned par = (unsigned)(g & 1ull);
    const float4* __restrict__ Qin = tp.Qd[par];
    float4* __restrict__ Qout = tp.Qd[par ^ 1u];
    const int4* __restrict__ in = tp.rec[par];
    const int4* __restrict__ ovf_in = tp.ovf[par];
    const unsigned ntl = blockIdx.x < tp.ntiles ? (tp.ntiles - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;   // tiles of this block

    if (tid == 0) {
        s_goals = 0; s_timeouts = 0; s_conf = 0; s_nbig = 0; s_nbigent = 0; s_bad = 0; s_abort = 0;
        for (unsigned q = 0; q < NSTAGE; ++q) { mbar_init(&s_full[q], 1u); mbar_init(&s_done[q], CT); }
        if (blockIdx.x == 0) { tp.tctl[(unsigned)((g + 2ull) % 3ull)] = 0u; tp.tctl[3u + (par ^ 1u)] = 0u; }   // nobody touches these in this step
    }
    __syncthreads();

    if (tid >= CT) {
        // =========================== producer warp: moves all the data ===================================
        // Lane r issues the bulk copies of rows r and r + 32, so a tile's copies are issued in a few instructions
        // per lane; the region header of the tile to load next is fetched BEFORE waiting for the consumers, so its
        // round trip to global memory is off the path.
        const unsigned n_spill = min(tp.tctl[(unsigned)(g % 3ull)], p.N);
        struct Raw { unsigned roff, fcap, rend, seg, arr; };
        auto fetch_hdr = [&](unsigned k) -> Raw {
            Raw r{0u, 0u, 0u, 0u, 0u};
            if (k < ntl) {
                const unsigned tile = blockIdx.x + k * gridDim.x;
                r.roff = tp.reg_off[tile]; r.fcap = tp.front_cap[tile]; r.rend = tp.reg_off[tile + 1u];
                r.seg = tp.seg_cnt[par][tile]; r.arr = tp.arr_cnt[par][tile];
            }
            return r;
        };
        auto load_tile = [&](unsigned k, const Raw& raw) {    // header + bulk copies of the block's k-th tile into stage k % NSTAGE
            const unsigned b = k % NSTAGE, tile = blockIdx.x + k * gridDim.x;
            unsigned char* st = smem + b * stage_bytes;
            float4* s_q = reinterpret_cast<float4*>(st);
            int4* s_rec = reinterpret_cast<int4*>(st + HS2 * 16u);
            int4* s_recb = s_rec + RC;
            unsigned char* s_cls = reinterpret_cast<unsigned char*>(s_recb + RCB);
            const int tx0 = (int)((tile % tp.tiles_x) << TSH), ty0 = (int)((tile / tp.tiles_x) << TSH);
            const unsigned roff = raw.roff, fcap = raw.fcap, bcap = raw.rend - roff - fcap;
            const unsigned n_front = min(raw.seg, fcap), n_back = min(raw.arr, bcap);
            const unsigned nf_s = min(n_front, RC), nb_s = min(n_back, RCB);
            const int xs = max(tx0 - 1, 0), xe = min(tx0 + (int)T, p.W - 1);
            const int gy_lo = max(ty0 - 1, 0), gy_hi = min(ty0 + (int)T, p.H - 1);
            const unsigned bytes_h = (unsigned)(xe - xs + 1) * 16u;
            if (lane == 0) {
                TileHdr& h = s_hdr[b];
                h.tile = tile; h.roff = roff; h.fcap = fcap; h.n_front = n_front; h.n_in = n_front + n_back; h.n_all = n_front + n_back + n_spill;
                h.nf_s = nf_s; h.nb_s = nb_s; h.tx0 = tx0; h.ty0 = ty0;
                mbar_arrive_expect_tx(&s_full[b], (unsigned)(gy_hi - gy_lo + 1) * bytes_h + tp.cls_stride + (nf_s + nb_s) * 16u);
                if (nf_s) bulk_g2s(s_rec, in + roff, nf_s * 16u, &s_full[b]);
            }
            if (lane == 1 && nb_s) bulk_g2s(s_recb, in + roff + fcap, nb_s * 16u, &s_full[b]);
            if (lane == 2) bulk_g2s(s_cls, tp.tcls + (size_t)tile * tp.cls_stride, tp.cls_stride, &s_full[b]);
            for (int gy = gy_lo + (int)lane; gy <= gy_hi; gy += 32)
                bulk_g2s(s_q + (unsigned)(gy - (ty0 - 1)) * HS + (unsigned)(xs - (tx0 - 1)), Qin + (size_t)gy * (size_t)p.W + (size_t)xs, bytes_h, &s_full[b]);
        };
        for (unsigned q = 0; q < NSTAGE; ++q) if (ntl > q) load_tile(q, fetch_hdr(q));
        for (unsigned k = 0; k < ntl; ++k) {
            const unsigned b = k % NSTAGE;
            const Raw nxt = fetch_hdr(k + NSTAGE);             // in flight while this warp waits
            // one lane polls; the others park at the warp barrier instead of spinning
            if (lane == 0 && !mbar_wait(&s_done[b], (k / NSTAGE) & 1u)) { atomicOr(&p.ctl->error, ERR_COPY_TIMEOUT); s_abort = 1u; }
            __syncwarp();
            if (*(volatile unsigned*)&s_abort) break;
            // rows of Q_{t+1} out (the consumers fenced their writes towards the async proxy before arriving)
            const unsigned tile = blockIdx.x + k * gridDim.x;
            const int tx0 = (int)((tile % tp.tiles_x) << TSH), ty0 = (int)((tile / tp.tiles_x) << TSH);
            const unsigned wi = (unsigned)min((int)T, p.W - tx0), ri = (unsigned)min((int)T, p.H - ty0);
            const float4* s_q = reinterpret_cast<const float4*>(smem + b * stage_bytes);
            for (unsigned r = lane; r < ri; r += 32u)
                bulk_s2g(Qout + (size_t)(ty0 + (int)r) * (size_t)p.W + (size_t)tx0, s_q + (r + 1u) * HS + 1u, wi * 16u);
            bulk_commit_wait_read();                            // the stage may be overwritten once its rows have been read
            __syncwarp();
            if (k + NSTAGE < ntl) load_tile(k + NSTAGE, nxt);
        }
        return;
    }

    // ================================= consumers ======================================================
    StepCtx c;
    c.eps = p.eps_tab[p.eps_from_ctl ? p.ctl->eps_idx : p.eps_idx]; c.g = g;
    c.out = tp.rec[par ^ 1u]; c.ovf_out = tp.ovf[par ^ 1u]; c.arr_next = tp.arr_cnt[par ^ 1u];
    c.ovf_cnt_next = tp.tctl + (unsigned)((g + 1ull) % 3ull);
    c.s_stay = &s_stay; c.s_goals = &s_goals; c.s_timeouts = &s_timeouts;
    unsigned conf = 0;
    for (unsigned k = 0; k < ntl; ++k) {
        const unsigned b = k % NSTAGE;
        unsigned char* st = smem + b * stage_bytes;
        float4* s_q = reinterpret_cast<float4*>(st);
        const int4* s_rec = reinterpret_cast<const int4*>(st + HS2 * 16u);
        const int4* s_recb = s_rec + RC;
        c.s_q = s_q; c.s_cls = reinterpret_cast<const unsigned char*>(s_recb + RCB);

        if (tid == 0) { s_stay = 0; s_nocc = 0; s_base = 0xFFFFFFFFu; }
        for (unsigned q = 2u * tid; q < T2; q += 2u * CT) *reinterpret_cast<uint4*>(s_n + q) = make_uint4(0u, 0u, 0u, 0u);
        for (unsigned q = tid; q < (T2 + 31u) / 32u; q += CT) s_flag[q] = 0u;
        // one thread waits for the copies; the barrier below passes the news (and the data) on to the others
        if (tid == 0 && !mbar_wait(&s_full[b], (k / NSTAGE) & 1u)) { atomicOr(&p.ctl->error, ERR_COPY_TIMEOUT); s_abort = 1u; }
        cons_sync<CT>();
        if (s_abort) break;                                    // never seen; the producer gives up at its next wait
        const TileHdr h = s_hdr[b];
        const unsigned tile = h.tile, roff = h.roff, fcap = h.fcap, n_front = h.n_front, n_in = h.n_in, n_all = h.n_all, nf_s = h.nf_s, nb_s = h.nb_s;
        c.tx0 = h.tx0; c.ty0 = h.ty0; c.tile = tile; c.roff = roff; c.fcap = fcap;
        const bool crowded = n_all > NMAX16;                        // block-uniform
        unsigned* gcnt = nullptr;
        if (crowded) {                                               // 4 x 32-bit counters per cell in global scratch
            if (tid == 0) {
                const unsigned need = T2 * 2u, q = atomicAdd(&tp.tctl[3u + par], need);
                if (q + need <= p.N) s_base = q; else { s_base = 0xFFFFFFFEu; atomicOr(&p.ctl->error, ERR_SCRATCH_OVERFLOW); }
            }
            cons_sync<CT>();
            if (s_base != 0xFFFFFFFEu) gcnt = reinterpret_cast<unsigned*>(tp.scratch + s_base);
            if (gcnt) for (unsigned q = tid; q < T2 * 4u; q += CT) gcnt[q] = 0u;
            cons_sync<CT>();
        }

        // record j of this tile's input (front part, back part, then the spill list filtered by tile)
        auto fetch = [&](unsigned j, int4& r) -> bool {
            if (j < n_front) { r = j < nf_s ? s_rec[j] : in[roff + j]; return true; }
            if (j < n_in) { const unsigned q = j - n_front; r = q < nb_s ? s_recb[q] : in[roff + fcap + q]; return true; }
            r = ovf_in[j - n_in];
            return tile_of(tp, r.x, r.y) == tile;
        };

        // ---- the step: every environment acts, moves and counts itself in its cell's histogram ----------
        for (unsigned j = tid; j < n_all; j += CT) {
            int4 rec; unsigned ic, a;
            if (!fetch(j, rec)) continue;
            if (!step_env<TRACE, TSH>(p, c, rec, ic, a)) { s_bad = 1u; continue; }
            if (!crowded) {
                // 32-bit shared-memory atomics are native; the 64-bit word of a cell is counted in its two halves
                const unsigned old = atomicAdd(reinterpret_cast<unsigned*>(s_n) + 2u * ic + (a >> 1), 1u << (16u * (a & 1u)));
                if (old == 0u) {                                                           // first on this half: maybe first on the cell
                    const unsigned bit = 1u << (ic & 31u);
                    if (!(atomicOr(&s_flag[ic >> 5], bit) & bit)) s_list[atomicAdd(&s_nocc, 1u)] = (unsigned short)ic;
                }
            } else if (gcnt) atomicAdd(&gcnt[ic * 4u + a], 1u);
        }
        cons_sync<CT>();
        if (tid == 0) {
            tp.seg_cnt[par ^ 1u][tile] = min(s_stay, fcap);
            tp.arr_cnt[par][tile] = 0u;                                   // consumed; it is the append counter again in the next step
        }

        // ---- Q_{t+1} of the occupied cells: computed from Q_t into registers, written after everybody has read ---
        float4 nrow[CPT]; unsigned nh[CPT];
        const unsigned nocc = crowded ? T2 : s_nocc;
#pragma unroll
        for (unsigned q = 0; q < CPT; ++q) {
            const unsigned idx = tid + q * CT;
            nh[q] = 0xFFFFFFFFu;
            if (idx >= nocc) continue;
            unsigned ic, tot; unsigned long long w = 0ull; unsigned n32[4];
            if (!crowded) {
                ic = s_list[idx];
                w = s_n[ic];
                tot = ((unsigned)w & 0xFFFFu) + ((unsigned)(w >> 16) & 0xFFFFu) + ((unsigned)(w >> 32) & 0xFFFFu) + (unsigned)(w >> 48);
            } else {
                ic = idx;
                if (!gcnt) continue;
                const uint4 v = *reinterpret_cast<const uint4*>(gcnt + 4u * ic);
                n32[0] = v.x; n32[1] = v.y; n32[2] = v.z; n32[3] = v.w;
                tot = v.x + v.y + v.z + v.w;
            }
            if (!tot) continue;
            if (tot > 1u) conf += tot;
            if (tot > CROWDED_CELL) { atomicAdd(&s_nbig, 1u); atomicAdd(&s_nbigent, tot); }
            nrow[q] = updated_row<TSH>(p, c, ic, w, crowded ? n32 : nullptr);
            nh[q] = ((ic >> TSH) + 1u) * HS + (ic & (T - 1u)) + 1u;
        }
        cons_sync<CT>();
#pragma unroll
        for (unsigned q = 0; q < CPT; ++q) if (nh[q] != 0xFFFFFFFFu) s_q[nh[q]] = nrow[q];
        // hand the stage to the producer: rows written through the generic proxy, read by the bulk copy
        fence_async_smem();
        mbar_arrive(&s_done[b]);
    }
    for (int o = 16; o; o >>= 1) conf += __shfl_xor_sync(FULL, conf, o);
    if (lane == 0u && conf) atomicAdd(&s_conf, conf);
    cons_sync<CT>();
    if (tid == 0) {
        if (s_conf) atomicAdd(&p.ctl->conflicts, (unsigned long long)s_conf);
        if (s_goals) atomicAdd(&p.ctl->goals, (unsigned long long)s_goals);
        if (s_timeouts) atomicAdd(&p.ctl->timeouts, (unsigned long long)s_timeouts);
        if (s_goals + s_timeouts) atomicAdd(&p.ctl->episodes, (unsigned long long)(s_goals + s_timeouts));
        if (s_nbig) { atomicAdd(&p.ctl->long_chains, (unsigned long long)s_nbig); atomicAdd(&p.ctl->general, (unsigned long long)s_nbigent); }
        if (s_bad) atomicOr(&p.ctl->error, ERR_BAD_STATE);
    }
}

// Per-episode epsilon schedule: the table index follows the number of finished episodes, which only
// the device knows.  One thread, launched after each step in that mode only.
__global__ void k_tile_eps_episode(Params p) {
    Ctl* c = p.ctl;
    c->eps_used = p.eps_tab[c->eps_idx];
    const unsigned long long kk = c->episodes / (unsigned long long)p.N;
    const unsigned long long rel = kk > c->eps_base_k ? kk - c->eps_base_k : 0ull;
    c->eps_idx = (unsigned)(rel < (unsigned long long)(c->eps_len - 1u) ? rel : (unsigned long long)(c->eps_len - 1u));
}

// ------------------------------------------------------------------------------------------------
// Bucketing: records in any order -> tile regions sized from the actual populations.
__global__ void k_te_count(Params p) {
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    const int4 r = p.st[i];
    atomicAdd(&p.tp.seg_cnt[p.step & 1ull][tile_of(p.tp, r.x, r.y)], 1u);
}
// One block: region sizes (front = population + 25 % + 32, back = 25 % + 64), their exclusive scan, counters reset.
__global__ void __launch_bounds__(1024) k_te_layout(Params p) {
    __shared__ unsigned s_warp[33];
    __shared__ unsigned s_carry;
    const TileP& tp = p.tp;
    const unsigned par = (unsigned)(p.step & 1ull);
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (unsigned base = 0; base < tp.ntiles; base += 1024u) {
        const unsigned k = base + threadIdx.x;
        const unsigned cnt = k < tp.ntiles ? tp.seg_cnt[par][k] : 0u;
        const unsigned F = cnt + cnt / 4u + 32u, B = cnt / 4u + 64u;
        unsigned total = 0;
        const unsigned ex = block_scan_excl(k < tp.ntiles ? F + B : 0u, s_warp, &total);
        const unsigned carry = s_carry;
        if (k < tp.ntiles) {
            tp.reg_off[k] = carry + ex; tp.front_cap[k] = F;
            tp.seg_cnt[par][k] = 0u; tp.seg_cnt[par ^ 1u][k] = 0u; tp.arr_cnt[0][k] = 0u; tp.arr_cnt[1][k] = 0u;
        }
        __syncthreads();
        if (threadIdx.x == 0) s_carry = carry + total;
        __syncthreads();
    }
    if (threadIdx.x == 0) { tp.reg_off[tp.ntiles] = s_carry; for (int k = 0; k < 5; ++k) tp.tctl[k] = 0u; }
}
__global__ void k_te_scatter(Params p) {
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    const TileP& tp = p.tp;
    const unsigned par = (unsigned)(p.step & 1ull);
    const int4 r = p.st[i];
    const unsigned tile = tile_of(tp, r.x, r.y);
    const unsigned pos = atomicAdd(&tp.seg_cnt[par][tile], 1u);
    tp.rec[par][tp.reg_off[tile] + pos] = r;
}
// The class bytes (obstacle / goal bits) of every tile with its halo, laid out as the step kernel copies them.
__global__ void __launch_bounds__(BLOCK) k_te_cls(Params p) {
    const TileP& tp = p.tp;
    const unsigned tile = blockIdx.x, HS = tp.T + 2u;
    const int tx0 = (int)((tile % tp.tiles_x) << tp.tshift), ty0 = (int)((tile / tp.tiles_x) << tp.tshift);
    for (unsigned k = threadIdx.x; k < tp.cls_stride; k += BLOCK) {
        const unsigned hy = k / HS, hx = k - hy * HS;
        const int gx = tx0 + (int)hx - 1, gy = ty0 + (int)hy - 1;
        unsigned cls = CW_OBST;
        if (hy < HS && gx >= 0 && gx < p.W && gy >= 0 && gy < p.H) cls = p.cw[(unsigned)gy * (unsigned)p.W + (unsigned)gx] & (CW_OBST | CW_GOAL);
        tp.tcls[(size_t)tile * tp.cls_stride + k] = (unsigned char)cls;
    }
}
// Back to environment order: st[id] = record.
__global__ void __launch_bounds__(BLOCK) k_te_export(Params p) {
    const TileP& tp = p.tp;
    const unsigned par = (unsigned)(p.step & 1ull), tile = blockIdx.x;
    const unsigned roff = tp.reg_off[tile], fcap = tp.front_cap[tile], bcap = tp.reg_off[tile + 1u] - roff - fcap;
    const unsigned n_front = min(tp.seg_cnt[par][tile], fcap), n_back = min(tp.arr_cnt[par][tile], bcap);
    const int4* in = tp.rec[par];
    for (unsigned j = threadIdx.x; j < n_front; j += BLOCK) { const int4 r = in[roff + j]; if ((unsigned)r.w < p.N) p.st[r.w] = r; }
    for (unsigned j = threadIdx.x; j < n_back; j += BLOCK) { const int4 r = in[roff + fcap + j]; if ((unsigned)r.w < p.N) p.st[r.w] = r; }
}
__global__ void k_te_export_ovf(Params p) {
    const TileP& tp = p.tp;
    const unsigned n = min(tp.tctl[(unsigned)(p.step % 3ull)], p.N);
    const int4* in = tp.ovf[p.step & 1ull];
    for (unsigned j = blockIdx.x * blockDim.x + threadIdx.x; j < n; j += gridDim.x * blockDim.x) { const int4 r = in[j]; if ((unsigned)r.w < p.N) p.st[r.w] = r; }
}

// Replica averaging on a dense table: rows [cell0, cell0+n) of every rank, rank after rank, summed in rank
// order 0..R-1 in fp32 (the order of the CPU oracle), scaled by 1/R.
__global__ void k_q_average_dense(float4* table, const float4* gathered, unsigned R, unsigned cell0, unsigned n, float scale) {
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float4 acc = gathered[i];
    for (unsigned r = 1; r < R; ++r) {
        const float4 v = gathered[(size_t)r * n + i];
        acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
    }
    acc.x = __fmul_rn(acc.x, scale); acc.y = __fmul_rn(acc.y, scale); acc.z = __fmul_rn(acc.z, scale); acc.w = __fmul_rn(acc.w, scale);
    table[cell0 + i] = acc;
}

// ------------------------------------------------------------------------------------------------
static inline unsigned nblk(unsigned n) { return (n + BLOCK - 1) / BLOCK; }

static size_t work_bytes(size_t T2) { return (T2 * 8 + T2 * 2 + (T2 + 31) / 32 * 4 + 15) / 16 * 16; }
size_t tile_step_smem(const Params& p) {
    const size_t T = p.tp.T, HS = T + 2;
    const size_t stage = HS * HS * 16 + (size_t)rc_front(CONSUMERS) * 16 + (size_t)rc_back(CONSUMERS) * 16 + p.tp.cls_stride;
    return NSTAGE * stage + work_bytes(T * T);
}
template <unsigned TSH>
static cudaError_t configure_one(int bytes, int* per_sm) {
    cudaError_t e = cudaFuncSetAttribute(k_tile_step<false, TSH, CONSUMERS>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_tile_step<true, TSH, CONSUMERS>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(per_sm, k_tile_step<false, TSH, CONSUMERS>, (int)(CONSUMERS + 32u), (size_t)bytes);
    return e;
}
int tile_engine_configure(Params& p, int device) {
    const int bytes = (int)tile_step_smem(p);
    int sms = 0, per_sm = 0;
    cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return (int)e;
    switch (p.tp.tshift) {
        case 3: e = configure_one<3>(bytes, &per_sm); break;
        case 4: e = configure_one<4>(bytes, &per_sm); break;
        case 5: e = configure_one<5>(bytes, &per_sm); break;
        default: return (int)cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) return (int)cudaErrorLaunchOutOfResources;
    p.tp.grid = (unsigned)(sms * per_sm);
    return 0;
}
void launch_tile_bucket(const Params& p, cudaStream_t st) {
    cudaMemsetAsync(p.tp.seg_cnt[p.step & 1ull], 0, (size_t)p.tp.ntiles * sizeof(unsigned), st);
    if (p.N) k_te_count<<<nblk(p.N), BLOCK, 0, st>>>(p);
    k_te_layout<<<1, 1024, 0, st>>>(p);
    if (p.N) k_te_scatter<<<nblk(p.N), BLOCK, 0, st>>>(p);
}
void launch_tile_classes(const Params& p, cudaStream_t st) { k_te_cls<<<p.tp.ntiles, BLOCK, 0, st>>>(p); }
void launch_tile_export(const Params& p, cudaStream_t st) {
    k_te_export<<<p.tp.ntiles, BLOCK, 0, st>>>(p);
    k_te_export_ovf<<<64, BLOCK, 0, st>>>(p);
}
static unsigned tile_step_grid(const Params& p) { return p.tp.ntiles < p.tp.grid ? p.tp.ntiles : p.tp.grid; }
template <unsigned TSH>
static void launch_step_one(const Params& p, bool trace, unsigned grid, size_t smem, cudaStream_t st) {
    if (trace) k_tile_step<true, TSH, CONSUMERS><<<grid, CONSUMERS + 32u, smem, st>>>(p);
    else       k_tile_step<false, TSH, CONSUMERS><<<grid, CONSUMERS + 32u, smem, st>>>(p);
}
void launch_tile_step(const Params& p, bool trace, cudaStream_t st, cudaEvent_t ev_a, cudaEvent_t ev_b, cudaEvent_t ev_c) {
    const size_t smem = tile_step_smem(p);
    const unsigned grid = tile_step_grid(p);
    if (ev_a) cudaEventRecord(ev_a, st);
    switch (p.tp.tshift) {
        case 3: launch_step_one<3>(p, trace, grid, smem, st); break;
        case 4: launch_step_one<4>(p, trace, grid, smem, st); break;
        default: launch_step_one<5>(p, trace, grid, smem, st); break;
    }
    if (ev_b) cudaEventRecord(ev_b, st);
    if (p.eps_from_ctl) k_tile_eps_episode<<<1, 1, 0, st>>>(p);
    if (ev_c) cudaEventRecord(ev_c, st);
}
void launch_q_average_dense(const Params& p, float4* table, const float4* gathered, unsigned R, unsigned cell0, unsigned n, float scale, cudaStream_t st) {
    (void)p;
    if (n) k_q_average_dense<<<nblk(n), BLOCK, 0, st>>>(table, gathered, R, cell0, n, scale);
}

}  // namespace cudarl
