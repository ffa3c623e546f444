// tile_engine.cu -- the fused train step as a streaming pass over the grid, one WARP per tile.
//
// With a quarter as many environments as cells, nearly every 128-byte line of the table is touched in
// every step, so the step is organised around the TABLE, not around the environments:
//
//   * the grid is cut into T x T tiles (16 x 16 cells, or 8 x 8 on densely populated grids); the environments
//     are kept bucketed by tile (8-byte records: environment, step count, cell inside the tile);
//   * a warp owns a tile for the whole step and needs no block-wide barrier: it fetches the tile of Q_t with
//     ONE tensor copy (cp.async.bulk.tensor, a T x T box of float4 out of the row-major table) and the tile's
//     records with two bulk copies, completion on the warp's own mbarrier; the tile's move bytes and border
//     values (16 bytes per lane) and the next tile's header are loaded while the copies are in flight;
//   * every environment of the tile is stepped against shared memory: epsilon-greedy from the Philox
//     stream keyed by (seed, global env, step), move with obstacle / goal lookup, auto-reset;
//   * the TD updates of a cell are applied from a histogram of (cell, action) counts: inside one step the
//     target of an update depends on (cell, action) only, so n environments on one (cell, action) mean the
//     same map applied n times -- the same bits as the oracle's sequential order, without sorting anything
//     and without float atomics;
//   * the table is updated IN PLACE: only the entries that were updated are stored (4 bytes each, straight from
//     registers), and no other warp reads this tile's cells in this step.  The one thing a neighbour needs
//     from a tile -- max_a Q of the cell just beyond the shared edge, for the TD target of a move across the
//     edge -- travels through a border array: at the end of its step a tile stores the max of every cell of
//     its border ring (taken from Q_{t+1}) into its four neighbours' slots of the OTHER parity;
//   * an environment that stays in the tile is appended to the tile's region of the other record array
//     (positions from a warp ballot, no atomics); one that leaves (a walk across the edge, the end of an episode:
//     the next one starts on a seeded cell anywhere) is appended to its new tile's arrival buffer with one atomic;
//     a full arrival buffer spills to a global list that every warp filters.  Regions are re-sized from the actual
//     populations every few steps.
//   * tiles are handed out from one queue per SM (one atomic per tile, drawn two tiles ahead), odd steps walk the queues
//     backwards (a step starts on what the step before touched last, still in L2), and consecutive steps are chained by
//     programmatic dependent launch (the next step's blocks are resident and initialised when this step's last tile is done).
//
// What bounds the kernel (B200, 4096 x 4096 cells, 4,194,304 environments): a tile is ~1,100 dependent instructions at ~10
// cycles each for its warp; the 451 MB a step moves are hidden behind the other resident warps (28 per SM: 72 registers,
// 7.75 KB of shared memory each).  The tile loop is rolled and reads its records from shared memory on purpose: unrolled
// over register-held records it outgrew the instruction cache.
//
// Reference semantics (paths relative to the CudaRL-Arena project root):
//   step        src/environment.cu:17-48, obstacle test src/kernels.cu:29-44, goal src/kernels.cu:56-59
//   TD update   src/kernels.cu:96-114 (true max as in src/gpu/kernels.cu:36-45, src/train.py:134)
//   eps-greedy  src/train.py:101-108, first-max argmax src/q_learning.cu:196-206
//   episode     src/train.py:191-222
#include "kernels.cuh"
#include "rules.cuh"
#include <cstring>

namespace cudarl {

constexpr unsigned CROWDED_CELL = 24;   // a cell with more environments than this counts as "crowded" in the run statistics
constexpr unsigned NMAX16 = 65535u;     // records of a tile the 16-bit counters can hold
constexpr unsigned WPB = 4;             // warps per block; every warp works on its own
constexpr unsigned FAST_MAX = 128;      // records of a tile the fast path stages in shared memory (a multiple of 32, below 256)

__device__ __forceinline__ unsigned tile_of(const TileP& tp, int x, int y) {
    return ((unsigned)y >> tp.tshift) * tp.tiles_x + ((unsigned)x >> tp.tshift);
}
// A record inside a tile's region or arrival buffer, 8 bytes: .x = environment, .y = steps of the episode << 8 | row inside the
// tile << 4 | column inside the tile (the tile is known from where the record lies).  The step counter saturates at 2^24 - 2 (step caps beyond that are refused).
constexpr unsigned T_SAT = 0xFFFFFEu;     // (T_SAT << 8 | 0xFF) stays clear of the all-ones word that marks a restart inside the step kernel
__device__ __forceinline__ uint2 pack_rec(const TileP& tp, const int4 r) {
    const unsigned m = tp.T - 1u, t = (unsigned)r.z < T_SAT ? (unsigned)r.z : T_SAT;
    return make_uint2((unsigned)r.w, (t << 8) | (((unsigned)r.y & m) << 4) | ((unsigned)r.x & m));
}
__device__ __forceinline__ int4 unpack_rec(const uint2 q, int tx0, int ty0) {
    return make_int4(tx0 + (int)(q.y & 15u), ty0 + (int)((q.y >> 4) & 15u), (int)(q.y >> 8), (int)q.x);
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

// ---- asynchronous copies into shared memory, completion on an mbarrier ----------------------------------
// Tensor copy: the box starts at float column 4 * tx0 (a multiple of 4 floats = 16 bytes) and row ty0; cells
// of the box that lie outside the table arrive as zeros.  Plain bulk copies: 16-byte aligned on both sides,
// sizes multiples of 16.  No multicast anywhere.
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    // relaxed: the barrier only tells this warp that its tensor copy has landed; no write of the arriving lane is published by it
    asm volatile("mbarrier.arrive.expect_tx.relaxed.cta.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One look at the barrier, no waiting.
__device__ __forceinline__ bool mbar_test_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0u;
}
// Sleeps in hardware until the phase completes or about `ns` nanoseconds have passed: a waiting warp issues nothing.
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity, unsigned ns) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
    return ok != 0u;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tensor_g2s_2d(void* dst, const CUtensorMap* map, int c0, int c1, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(smem_u32(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
// Shared memory through 32-bit shared-space addresses: the hot loops index a warp's arrays with plain integer arithmetic.
__device__ __forceinline__ float4 lds_f4(unsigned a) { float4 v; asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ float lds_f32(unsigned a) { float v; asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ unsigned lds_u8(unsigned a) { unsigned v; asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ unsigned lds_u32(unsigned a) { unsigned v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ unsigned lds_u16(unsigned a) { unsigned v; asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ uint2 lds_u32x2(unsigned a) { uint2 v; asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ void sts_f32(unsigned a, float v) { asm volatile("st.shared.f32 [%0], %1;" :: "r"(a), "f"(v) : "memory"); }
__device__ __forceinline__ void sts_zero8(unsigned a) { asm volatile("st.shared.v2.u32 [%0], {%1, %1};" :: "r"(a), "r"(0u) : "memory"); }
__device__ __forceinline__ unsigned atoms_add(unsigned a, unsigned v) { unsigned o; asm volatile("atom.shared.add.u32 %0, [%1], %2;" : "=r"(o) : "r"(a), "r"(v) : "memory"); return o; }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}
constexpr unsigned long long WAIT_NS = 2000000000ull;   // a copy that has not landed after two seconds never will

// Wait for the phase with the given parity.  Bounded: by `polls` tries when polls > 0 (tests make a wait run
// out that way), else by WAIT_NS of wall time.  false = gave up.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, unsigned polls) {
    if (polls) {
        for (unsigned it = 0; it < polls; ++it) if (mbar_test_wait(bar, parity)) return true;
        return false;
    }
    unsigned long long t0 = 0ull;
    for (unsigned it = 1u;; ++it) {
        if (mbar_try_wait(bar, parity, 20000u)) return true;
        if ((it & 15u) == 0u) {
            const unsigned long long now = global_ns();
            if (t0 == 0ull) t0 = now; else if (now - t0 > WAIT_NS) return false;
        }
    }
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
// Shared memory of one warp (nothing is shared between warps).  What the copies of a tile deliver:
//   s_q    T*T  float4   Q_t of the tile, row-major inside the tile
//   s_mv   T*T  u8       per cell: bit a = a move in direction a is blocked (grid edge or obstacle), bit 4+a = the
//                        cell an environment stands on after choosing a (the next cell, or its own when blocked) is a goal
//   s_halo 4T   float    max_a Q_t of the cells beyond the north / south / west / east edge (from the border array)
//   s_rec  130  8 bytes  fast path: the tile's records (bulk copies: arrivals, a pad slot when their number is odd, then the region);
//                        a record that leaves the tile is written back here
// and the work area:
//   s_n    T*T  words    per cell: how many environments chose action a; zero between tiles.  8-byte words with 16 bits per action on
//                        8 x 8 tiles; on 16 x 16 tiles 4-byte words with 8 bits per action (the fast path counts at most 128 records,
//                        the general path counts in global scratch there): the kilobyte saved pays for 128 instead of 96 staged records
//   s_kd   128  u32+f32  fast path: per record its key (cell, action, owner flag) and TD target, from the step to the owner pass
//   s_que  128  u8       fast path: the slots of the records that leave the tile
//   s_bm   4T   float    general path: max_a Q_{t+1} of the tile's own north / south / west / east border cells (shares the bytes of s_kd)
//   s_list T*T  u16      general path: the occupied cells (shares the bytes of s_rec)
// A tile with more than 65,535 records counts in 32-bit counters in global scratch instead.
template <unsigned TSH> struct WarpSmem {
    static constexpr unsigned T = 1u << TSH, T2 = T * T;
    static constexpr unsigned CLS = T2;                              // a multiple of 16 for T = 8 and 16
    static constexpr unsigned ST_MV = T2 * 16u, ST_HALO = ST_MV + CLS, ST_REC = ST_HALO + 4u * T * 4u;
    static constexpr unsigned REC_BYTES = (FAST_MAX + 2u) * 8u > T2 * 2u ? (FAST_MAX + 2u) * 8u : T2 * 2u;   // + a pad slot and the copy's round-up
    static constexpr bool NARROW = TSH >= 4u;                        // 8-bit counters in shared memory; the general path then counts in global scratch
    static constexpr unsigned CELL_BYTES = NARROW ? 4u : 8u;
    static constexpr unsigned OFF_N = ST_REC + REC_BYTES, OFF_KD = OFF_N + T2 * CELL_BYTES, OFF_QUE = OFF_KD + FAST_MAX * 8u,
                              OFF_BM = OFF_KD;
    static constexpr unsigned BYTES = (OFF_QUE + FAST_MAX + 127u) / 128u * 128u;
    static_assert(4u * T * 4u <= FAST_MAX * 8u, "s_bm must fit into the bytes of s_kd");
    static_assert(FAST_MAX < 256u && FAST_MAX % 32u == 0u, "8-bit counters and whole rounds");
    static constexpr unsigned HALO_LANES = T, MV_LANES = T2 / 16u;   // lanes that fetch 16 bytes each of the border values / move bytes
};

// Everything the per-environment step needs about the tile being processed.
struct StepCtx {
    float eps; int tmax;
    unsigned eps_thr;      // explore iff (w0 >> 8) < eps_thr: the same test as (w0 >> 8) * 2^-24 < eps, in integers
};

// TD target of (cell, action) from Q_t:  r + gamma * max_a' Q_t[s'],  0 for the max when the episode ends there.
// The next cell's max comes from the tile, or from the border values when the move crosses an edge.
template <unsigned TSH>
__device__ __forceinline__ float td_target(const Params& p, const float4* s_q, const float* s_halo, unsigned ic, int a, unsigned mvb, int tx0, int ty0) {
    constexpr unsigned T = 1u << TSH;
    const bool blocked = (mvb >> a) & 1u, done = (mvb >> (4 + a)) & 1u;
    float m = 0.0f;
    if (!done) {
        if (blocked) m = max4(s_q[ic]);
        else {
            const unsigned lx = ic & (T - 1u), ly = ic >> TSH;
            const int mx = (int)lx + (a == 1) - (a == 3), my = (int)ly + (a == 2) - (a == 0);
            if ((unsigned)mx < T && (unsigned)my < T) m = max4(s_q[((unsigned)my << TSH) + (unsigned)mx]);
            else m = s_halo[my < 0 ? lx : my >= (int)T ? T + lx : mx < 0 ? 2u * T + ly : 3u * T + ly];
        }
        if (p.legacy_clamp && m < 0.0f) m = 0.0f;
    }
    const float r = done ? 1.0f : blocked ? blocked_step_reward(p, tx0 + (int)(ic & (T - 1u)), ty0 + (int)(ic >> TSH), a) : -0.01f;
    return __fmaf_rn(p.gamma, m, r);
}

// Q_{t+1} row of one cell from Q_t and the number of environments that chose each action
// (`w`: 16 bits per action, or `n32` when the tile counts in 32 bits).  Only the actions that were chosen are visited.
template <unsigned TSH>
__device__ __forceinline__ float4 updated_row(const Params& p, const unsigned char* st, unsigned ic, unsigned long long w, const unsigned* n32, int tx0, int ty0) {
    using L = WarpSmem<TSH>;
    const float4* s_q = reinterpret_cast<const float4*>(st);
    float4 row = s_q[ic];
    const unsigned mvb = st[L::ST_MV + ic];
    unsigned mask = n32 ? ((n32[0] != 0u) | ((n32[1] != 0u) << 1) | ((n32[2] != 0u) << 2) | ((n32[3] != 0u) << 3))
                        : (((w & 0xFFFFull) != 0ull) | (((w >> 16) & 0xFFFFull) != 0ull) << 1 | (((w >> 32) & 0xFFFFull) != 0ull) << 2 | ((w >> 48) != 0ull) << 3);
    while (mask) {
        const int a = __ffs((int)mask) - 1; mask &= mask - 1u;
        const unsigned n = n32 ? n32[a] : (unsigned)(w >> (16 * a)) & 0xFFFFu;
        const float d = td_target<TSH>(p, s_q, reinterpret_cast<const float*>(st + L::ST_HALO), ic, a, mvb, tx0, ty0);
        float v = pick(row, a);
        for (unsigned i = 0; i < n; ++i) v = __fmaf_rn(p.lr, __fsub_rn(d, v), v);       // one application per environment
        row.x = a == 0 ? v : row.x; row.y = a == 1 ? v : row.y; row.z = a == 2 ? v : row.z; row.w = a == 3 ? v : row.w;
    }
    return row;
}

template <bool TRACE, unsigned TSH, unsigned MINB, bool PROBE>
__global__ void __launch_bounds__(WPB * 32u, MINB) k_tile_step(const __grid_constant__ Params p) {
    using L = WarpSmem<TSH>;
    constexpr unsigned T = L::T, T2 = L::T2;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_bar[WPB];
    __shared__ unsigned s_acc[6];            // goals, timeouts, conflicts, crowded cells, environments on them, bad records

    const TileP& tp = p.tp;
    const unsigned lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const unsigned lt = (1u << lane) - 1u;
    unsigned char* wb = smem + warp * L::BYTES;
    unsigned long long* s_n = reinterpret_cast<unsigned long long*>(wb + L::OFF_N);
    float* s_bm = reinterpret_cast<float*>(wb + L::OFF_BM);
    unsigned short* s_list = reinterpret_cast<unsigned short*>(wb + L::ST_REC);
    const unsigned sbase = smem_u32(wb), sn = sbase + L::OFF_N, srec = sbase + L::ST_REC, skd = sbase + L::OFF_KD, sque = sbase + L::OFF_QUE;

    const unsigned long long g = p.step;
    const unsigned par = (unsigned)(g & 1ull);
    const uint2* __restrict__ in = tp.rec[par];
    const uint2* __restrict__ arr_in = tp.arr[par];
    const int4* __restrict__ ovf_in = tp.ovf[par];
    uint2* __restrict__ out = tp.rec[par ^ 1u];
    uint2* __restrict__ arr_out = tp.arr[par ^ 1u];
    int4* __restrict__ ovf_out = tp.ovf[par ^ 1u];
    uint2* __restrict__ cnt_next = tp.cnt[par ^ 1u];
    unsigned* ovf_cnt_next = tp.tctl + (unsigned)((g + 1ull) % 3ull);
    const float* __restrict__ halo_in = tp.bmax[par];
    float* __restrict__ halo_out = tp.bmax[par ^ 1u];
    const unsigned gw = blockIdx.x * WPB + warp;

    if (threadIdx.x < 6u) s_acc[threadIdx.x] = 0u;
    if (lane == 0) mbar_init(&s_bar[warp], 1u);
    for (unsigned q = lane; q < T2 * L::CELL_BYTES / 4u; q += 32u) reinterpret_cast<unsigned*>(s_n)[q] = 0u;
    __syncthreads();
    // The first two tickets of this warp's tile queue (see the tile loop): this step's counters were cleared two steps ago and
    // nobody else touches them, so the tickets can be on their way before the previous kernel is known to be complete.
    const unsigned QN = min(tp.nq, gridDim.x), cq = blockIdx.x % QN;
    const unsigned qn = tp.ntiles / QN + (cq < tp.ntiles % QN ? 1u : 0u);                // tiles in this queue
    unsigned* const qctr = tp.tq + (unsigned)(g % 3ull) * tp.nq + cq;
    auto draw = [&]() -> unsigned { return lane == 0u ? atomicAdd(qctr, 1u) : 0u; };     // lane 0 holds the ticket
    unsigned tk0 = draw(), tk1 = draw();
    // The step is launched with programmatic stream serialisation: its blocks may become resident, and run everything above, while
    // the previous kernel's last blocks are still at work.  From here on that kernel is complete and its writes are visible.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Tests only (an instantiation of its own, launched when a poll bound is set): a wait bounded by a number of looks at the
    // barrier, taken before any copy has been issued, so that it must run out; the warp then does what it does when a copy never
    // arrives: it records the failure and leaves (nothing is in flight yet).
    bool gave_up = false;
    if (PROBE) {
        gave_up = !__all_sync(FULL, mbar_wait(&s_bar[threadIdx.x >> 5], 0u, p.tp.wait_polls ? p.tp.wait_polls : 1u));
        if (gave_up && (threadIdx.x & 31u) == 0u) atomicOr(&p.ctl->error, ERR_COPY_TIMEOUT);
    }
    if (gw == 0u && lane == 0u) { tp.tctl[(unsigned)((g + 2ull) % 3ull)] = 0u; tp.tctl[3u + (par ^ 1u)] = 0u; }   // nobody touches these in this step
    if (gw < tp.nq && lane == 0u) tp.tq[(unsigned)((g + 2ull) % 3ull) * tp.nq + gw] = 0u;                           // the queue counters of the step after the next

    StepCtx c;
    c.eps = p.eps_tab[p.eps_from_ctl ? p.ctl->eps_idx : p.eps_idx];
    c.tmax = p.max_steps > 0 ? p.max_steps : 0x7FFFFFFF;
    c.eps_thr = !(c.eps > 0.0f) ? 0u : c.eps >= 1.0f ? (1u << 24) : (unsigned)ceilf(c.eps * 16777216.0f);   // scaling by 2^24 is exact
    const unsigned n_spill = min(tp.tctl[(unsigned)(g % 3ull)], p.N);
    unsigned conf = 0;     // the rarer counters go straight to the block's shared-memory words

    // Border cells a lane reports at the end of a tile: entry k = lane + 32 r of the ring (north row, south row, west column,
    // east column): its cell inside the tile, and where it goes in the neighbour's block of the border array -- my north row is
    // the south halo (slot 1) of the tile above, my south row the north halo (0) of the tile below, west -> east (3), east -> west (2).
    // Per lane these never change: packed once (cell: 8 bits per entry; edge: 2 bits per entry; offsets: one int per entry).
    constexpr unsigned BR = (4u * T + 31u) / 32u;
    auto ring_cell = [&](unsigned k) -> unsigned {
        const unsigned e = k >> TSH, i = k & (T - 1u);
        return e == 0u ? i : e == 1u ? ((T - 1u) << TSH) + i : e == 2u ? (i << TSH) : (i << TSH) + T - 1u;
    };
    unsigned b_pack = 0u; int b_dst[BR];
#pragma unroll
    for (unsigned r = 0; r < BR; ++r) {
        const unsigned k = lane + 32u * r, e = k >> TSH, i = k & (T - 1u);
        const int dtile = e == 0u ? -(int)tp.tiles_x : e == 1u ? (int)tp.tiles_x : e == 2u ? -1 : 1;
        const unsigned slot = e == 0u ? 1u : e == 1u ? 0u : e == 2u ? 3u : 2u;
        b_dst[r] = (dtile * 4 + (int)slot) * (int)T + (int)i;
        b_pack |= (ring_cell(k) | (e << 8)) << (16u * r);
    }

    // Header of a tile: lane 0 loads {region start, capacity}, lane 1 {records in the region, arrivals}; the words
    // are only exchanged when the tile's copies are issued, one tile after the loads.
    const uint2* hdr_src = lane == 0u ? tp.reg : tp.cnt[par];
    auto fetch_hdr = [&](unsigned tile) -> uint2 { return (tile < tp.ntiles && lane < 2u) ? hdr_src[tile] : make_uint2(0u, 0u); };
    // One copy stage per warp.  (A second one, with the next tile's copies in flight during the work, costs more in shared
    // memory and resident warps than it hides: 134.8 us per step at 16 warps per SM against 121.6 us at 24 single-stage warps.)
    unsigned roff = 0, fcap = 0, n_front = 0, n_arr = 0, n_in = 0, n_slots = 0;
    unsigned long long* const bar = &s_bar[warp];
    uint4 side = make_uint4(0u, 0u, 0u, 0u);      // this lane's 16 bytes of the tile's border values or move bytes, on their way to shared memory
    // Issue the copies of a tile: the table box (tensor copy) and, when the tile is small enough for the fast path, its records
    // (region and arrival buffer, one bulk copy each), all completing on the warp's barrier.
    auto issue = [&](unsigned tile, unsigned txi, unsigned tyi, const uint2 hw) {
        roff = __shfl_sync(FULL, hw.x, 0); fcap = __shfl_sync(FULL, hw.y, 0);
        n_front = min(__shfl_sync(FULL, hw.x, 1), fcap); n_arr = min(__shfl_sync(FULL, hw.y, 1), ARR_CAP); n_in = n_front + n_arr;
        // Staged records: the arrivals first, then the region, each copy rounded up to 16 bytes (regions start on even records and
        // have even capacities, so the round-up stays inside them); an odd number of arrivals leaves one pad slot behind them.
        const unsigned a2 = (n_arr + 1u) & ~1u, f2 = (n_front + 1u) & ~1u;
        n_slots = a2 + n_front;
        const bool stage_records = n_slots + n_spill <= FAST_MAX;     // room even if every spilled record were this tile's
        if (lane == 0u) mbar_arrive_expect_tx(bar, T2 * 16u + (stage_records ? (a2 + f2) * 8u : 0u));
        __syncwarp();
        if (lane == 0u) tensor_g2s_2d(wb, &tp.tmq, (int)(txi << TSH) * 4, (int)(tyi << TSH), bar);
        else if (lane == 1u && stage_records && n_front) bulk_g2s(wb + L::ST_REC + a2 * 8u, in + roff, f2 * 8u, bar);
        else if (lane == 2u && stage_records && n_arr) bulk_g2s(wb + L::ST_REC, arr_in + (size_t)tile * ARR_CAP, a2 * 8u, bar);
        // the small pieces (border values 16 T bytes, move bytes T*T) come as one 16-byte load per lane, stored after the wait
        if (lane < L::HALO_LANES) side = *reinterpret_cast<const uint4*>(halo_in + (size_t)tile * (4u * T) + lane * 4u);
        else if (lane < L::HALO_LANES + L::MV_LANES) side = *reinterpret_cast<const uint4*>(tp.tcls + (size_t)tile * L::CLS + (lane - L::HALO_LANES) * 16u);
    };
    // A record that leaves its tile: one atomic on the new tile's arrival counter, then the store.  The fast path issues the
    // atomic at the end of a tile and stores a tile later, when the counter value has long arrived.
    auto store_arrival = [&](const int4 r, unsigned dt, unsigned apos) {
        if (apos < ARR_CAP) arr_out[(size_t)dt * ARR_CAP + apos] = pack_rec(tp, r);
        else {
            const unsigned qq = atomicAdd(ovf_cnt_next, 1u);
            if (qq < p.N) ovf_out[qq] = r; else s_acc[5] = 1u;
        }
    };

    // Odd steps walk the tiles in descending order: what the last step touched last (table lines, records, border values
    // of the final part of the grid) is what this step touches first, while it is still in L2.
    const bool flip = (g & 1ull) != 0ull;
    bool pend = false; int4 pend_rec = make_int4(0, 0, 0, 0); unsigned pend_dt = 0, pend_pos = 0;
    // Tiles are handed out by queue, so that a warp that got light tiles takes more of them: queue q holds the tiles q, q + nq,
    // q + 2 nq, ... and is served by the blocks q, q + nq, ... of this launch (nq = the number of SMs, or of blocks when there are
    // fewer: every queue has a block, and blocks launched nq apart normally share an SM).  A warp draws its tickets with one atomic
    // per tile, two tiles ahead of the work, so that neither the ticket nor the tile's header is waited for.
    auto ticket_tile = [&](unsigned t) -> unsigned { return t < qn ? (flip ? cq + QN * (qn - 1u - t) : cq + QN * t) : tp.ntiles; };
    unsigned phase = 0, txi = 0, tyi = 0;
    tk0 = __shfl_sync(FULL, tk0, 0);
    uint2 hw = fetch_hdr(ticket_tile(tk0));
    if (PROBE && gave_up) tk0 = qn;
    while (tk0 < qn) {
        const unsigned tile = ticket_tile(tk0);
        // tile = tyi * tiles_x + txi: the quotient from a multiplication by the precomputed reciprocal, off by at most one
        tyi = __umulhi(tile, tp.tiles_x_rcp); txi = tile - tyi * tp.tiles_x;
        if (txi >= tp.tiles_x) { txi -= tp.tiles_x; ++tyi; }
        issue(tile, txi, tyi, hw);
        tk0 = __shfl_sync(FULL, tk1, 0);                        // the ticket drawn one tile ago
        tk1 = draw();
        hw = fetch_hdr(ticket_tile(tk0));                       // in flight while this tile is worked on
        // the previous tile's leavers: their arrival counters were bumped before its border values went out; the stores go
        // out now, while this tile's copies are in flight
        if (pend) { store_arrival(pend_rec, pend_dt, pend_pos); pend = false; }
        const unsigned n_all = n_in + n_spill;
        const unsigned pad_slot = (n_arr & 1u) ? n_arr : 0xFFFFFFFFu;
        const int tx0 = (int)(txi << TSH), ty0 = (int)(tyi << TSH);
        const unsigned char* st = wb;
        const float4* s_q = reinterpret_cast<const float4*>(st);
        const unsigned sq = sbase, smv = sq + L::ST_MV, shalo = sq + L::ST_HALO;

        if (!__all_sync(FULL, mbar_wait(bar, phase, 0u))) {
            // Never seen with the time bound.  Flag it, let the copies land (they target this warp's shared memory), stop.
            if (lane == 0u) atomicOr(&p.ctl->error, ERR_COPY_TIMEOUT);
            mbar_wait(bar, phase, 0u);
            break;
        }
        phase ^= 1u;
        if (lane < L::HALO_LANES + L::MV_LANES)
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" :: "r"(lane < L::HALO_LANES ? shalo + lane * 16u : smv + (lane - L::HALO_LANES) * 16u),
                         "r"(side.x), "r"(side.y), "r"(side.z), "r"(side.w) : "memory");
        __syncwarp();

        // stays: position in the tile's own region from a ballot.  Gives back whether the record still has to go somewhere else.
        unsigned nstay = 0;
        auto put_stay = [&](bool act, bool stays, const uint2 nrec) -> bool {
            const unsigned sm = __ballot_sync(FULL, act && stays);
            const unsigned pos = nstay + __popc(sm & lt);
            nstay += __popc(sm);
            const bool placed = act && stays && pos < fcap;
            if (placed) out[roff + pos] = nrec;
            return act && !placed;
        };

        const bool fast = n_slots + n_spill <= FAST_MAX;         // warp-uniform: the tile's records are in shared memory
        if (fast) {
            // A short spill list (records that found an arrival buffer full in the last step) is filtered here: what belongs to this
            // tile joins the staged records.  Only a long list sends a tile to the general path.
            unsigned n_tot = n_slots;
            for (unsigned base = 0; base < n_spill; base += 32u) {
                int4 r = make_int4(0, 0, 0, 0); bool mine = false;
                if (base + lane < n_spill) { r = ovf_in[base + lane]; mine = tile_of(tp, r.x, r.y) == tile; }
                const unsigned mm = __ballot_sync(FULL, mine);
                if (mine) { const uint2 q = pack_rec(tp, r); asm volatile("st.shared.v2.u32 [%0], {%1, %2};" :: "r"(srec + (n_tot + __popc(mm & lt)) * 8u), "r"(q.x), "r"(q.y) : "memory"); }
                n_tot += __popc(mm);
            }
            if (n_spill) __syncwarp();
            // ---- few records: everything an update needs passes through shared memory once ------------------------
            // Each environment computes the TD target of its own (cell, action) -- it has the next cell at hand -- and
            // counts itself; the FIRST to count on a (cell, action) owns it and, once every count is in, applies the
            // map that many times to the one table entry: a 4-byte store into the table, and into the tile in shared
            // memory, which thereby becomes Q_{t+1} for the border values.  The loops are rolled on purpose: the tile
            // loop has to stay inside the instruction cache.
            const unsigned rounds = (n_tot + 31u) >> 5;
            unsigned nleave = 0;
#pragma unroll 1
            for (unsigned it = 0; it < rounds; ++it) {
                const unsigned j = it * 32u + lane;
                bool act = j < n_tot && j != pad_slot;
                unsigned id = 0u, w1 = 0u;
                if (act) asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(id), "=r"(w1) : "r"(srec + j * 8u) : "memory");
                const unsigned lx = w1 & 15u, ly = (w1 >> 4) & 15u;
                if (act && (lx | ly) >= T) { s_acc[5] = 1u; act = false; }             // never seen: the record does not lie in this tile
                uint2 nrec = make_uint2(id, 0u); bool stays = false; unsigned key = 0u; float dd = 0.0f;
                if (act) {
                    const U4 w = philox4x32_10(p.env_offset + id, 0u, (unsigned)g, (unsigned)(g >> 32), p.k0, p.k1 ^ TAG_POLICY);
                    const unsigned ic = (ly << TSH) | lx;
                    const float4 row = lds_f4(sq + ic * 16u);
                    const unsigned mvb = lds_u8(smv + ic);
                    int a = argmax4(row);
                    if ((w.x >> 8) < c.eps_thr) a = (int)(w.y & 3u);
                    const bool blocked = (mvb >> a) & 1u, done = (mvb >> (a + 4)) & 1u;
                    // per action: dx = {0, 1, 0, -1}, dy = {-1, 0, 1, 0}, one signed byte each
                    const int dx = blocked ? 0 : (int)(signed char)(0xFF000100u >> (8 * a)), dy = blocked ? 0 : (int)(signed char)(0x000100FFu >> (8 * a));
                    const unsigned mx = lx + (unsigned)dx, my = ly + (unsigned)dy;      // wraps when the move leaves the tile
                    stays = (mx | my) < T;
                    float m;
                    if (stays) m = max4(lds_f4(sq + ((my << TSH) | mx) * 16u));
                    else m = lds_f32(shalo + 4u * ((int)my < 0 ? lx : my >= T ? T + lx : (int)mx < 0 ? 2u * T + ly : 3u * T + ly));
                    if (p.legacy_clamp && m < 0.0f) m = 0.0f;
                    const float r = (blocked && p.ntraps) ? blocked_step_reward(p, tx0 + (int)lx, ty0 + (int)ly, a) : -0.01f;     // a trap charges its penalty
                    dd = done ? 1.0f : __fmaf_rn(p.gamma, m, r);                     // the TD target of (cell, a), from Q_t
                    if (TRACE) { p.tr_a[id] = a; p.tr_r[id] = done ? 1.0f : r; p.tr_d[id] = done ? 1 : 0; }
                    const unsigned idx = ic * 4u + (unsigned)a;
                    bool first;
                    if (L::NARROW) { const unsigned old = atoms_add(sn + ic * 4u, 1u << (8u * (unsigned)a)); first = ((old >> (8u * (unsigned)a)) & 0xFFu) == 0u; }
                    else { const unsigned sh = 16u * ((unsigned)a & 1u), old = atoms_add(sn + (idx >> 1) * 4u, 1u << sh); first = ((old >> sh) & 0xFFFFu) == 0u; }
                    key = (first ? 0x40000000u : 0u) | idx;
                    const unsigned t1 = min((w1 >> 8) + 1u, T_SAT);
                    // meaningful when the record stays; on 16 x 16 tiles row << 4 | column is the cell's index inside the tile
                    nrec.y = TSH == 4u ? (t1 << 8) | (((my << 4) | mx) & 0xFFu) : (t1 << 8) | ((my & 15u) << 4) | (mx & 15u);
                    if (done || t1 >= (unsigned)c.tmax) {  // the episode ends: the start cell of the next one is drawn when the record is sent (below)
                        nrec.y = 0xFFFFFFFFu; stays = false;
                        atomicAdd(&s_acc[done ? 0 : 1], 1u);
                    }
                }
                // every slot gets its key (0 = owns nothing: the pad slot, a rejected record) and target for the owner pass
                if (j < n_tot) asm volatile("st.shared.v2.u32 [%0], {%1, %2};" :: "r"(skd + j * 8u), "r"(key), "r"(__float_as_uint(dd)) : "memory");
                // a record that leaves goes back into its slot (environment and new step count, or the restart mark; where it goes
                // follows from its key) and the slot's number into the queue; it is sent when the tile is done
                const bool leaves = put_stay(act, stays, nrec);
                const unsigned lm = __ballot_sync(FULL, leaves);
                if (leaves) {
                    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" :: "r"(srec + j * 8u), "r"(nrec.x), "r"(nrec.y) : "memory");
                    asm volatile("st.shared.u8 [%0], %1;" :: "r"(sque + nleave + __popc(lm & lt)), "r"(j) : "memory");
                }
                nleave += __popc(lm);
            }
            __syncwarp();
            float* const qtile = reinterpret_cast<float*>(p.Q + ((size_t)ty0 * (size_t)p.W + (size_t)tx0));
#pragma unroll 1
            for (unsigned it = 0; it < rounds; ++it) {
                const unsigned j = it * 32u + lane;
                if (j >= n_tot) continue;
                const uint2 kd = lds_u32x2(skd + j * 8u);
                if (!(kd.x & 0x40000000u)) continue;
                const unsigned idx = kd.x & 0xFFFFu, ic = idx >> 2, a = idx & 3u;
                unsigned n, tot; bool lowest;                                          // count of (cell, a), of the cell; no lower action was chosen
                if (L::NARROW) {
                    const unsigned w = lds_u32(sn + ic * 4u);
                    n = (w >> (8u * a)) & 0xFFu; tot = __dp4a(w, 0x01010101u, 0u); lowest = (w & ((1u << (8u * a)) - 1u)) == 0u;
                } else {
                    n = lds_u16(sn + idx * 2u);
                    const uint2 w = lds_u32x2(sn + ic * 8u);
                    const unsigned s2 = w.x + w.y;                                     // at most 128 per tile: no carry between the fields
                    tot = (s2 & 0xFFFFu) + (s2 >> 16);
                    lowest = ((((unsigned long long)w.y << 32) | w.x) & ((1ull << (16u * a)) - 1ull)) == 0ull;
                }
                if (tot > 1u) conf += n;
                if (tot > CROWDED_CELL && lowest) { atomicAdd(&s_acc[3], 1u); atomicAdd(&s_acc[4], tot); }      // the lowest chosen action speaks for the cell
                const float d = __uint_as_float(kd.y);
                float v = lds_f32(sq + idx * 4u);
                for (unsigned i = 0; i < n; ++i) v = __fmaf_rn(p.lr, __fsub_rn(d, v), v);          // one application per environment
                sts_f32(sq + idx * 4u, v);
                qtile[((ic >> TSH) * (unsigned)p.W + (ic & (T - 1u))) * 4u + a] = v;    // (row inside the tile) * W + column < cells < 2^28
            }
            __syncwarp();
            // the tile's leavers, one lane each: draw the start cell of a new episode where one ended, one atomic on the new tile's
            // arrival counter; the last 32 (normally all) are stored when the next tile's copies have been issued
            for (unsigned base = 0; base < nleave; base += 32u) {
                if (pend) { store_arrival(pend_rec, pend_dt, pend_pos); pend = false; }
                pend = base + lane < nleave;
                if (pend) {
                    const unsigned slot = lds_u8(sque + base + lane);
                    unsigned id, w1;
                    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(id), "=r"(w1) : "r"(srec + slot * 8u) : "memory");
                    pend_rec.w = (int)id;
                    if (w1 == 0xFFFFFFFFu) {
                        const unsigned sn2 = sample_start(p, p.env_offset + id, g + 1ull, TAG_START);
                        pend_rec.y = (int)(sn2 / (unsigned)p.W); pend_rec.x = (int)(sn2 - (unsigned)pend_rec.y * (unsigned)p.W); pend_rec.z = 0;
                    } else {
                        // where it went: its cell and action are in its key; a blocked move (a record that stayed but found its
                        // tile's region full) keeps the cell
                        const unsigned idx = lds_u32(skd + slot * 8u) & 0xFFFFu, ic = idx >> 2, a = idx & 3u;
                        const bool blocked = (lds_u8(smv + ic) >> a) & 1u;
                        const int dx = blocked ? 0 : (int)(signed char)(0xFF000100u >> (8 * a)), dy = blocked ? 0 : (int)(signed char)(0x000100FFu >> (8 * a));
                        pend_rec.x = tx0 + (int)(ic & (T - 1u)) + dx; pend_rec.y = ty0 + (int)(ic >> TSH) + dy; pend_rec.z = (int)(w1 >> 8);
                    }
                    pend_dt = tile_of(tp, pend_rec.x, pend_rec.y);
                    pend_pos = atomicAdd(&cnt_next[pend_dt].y, 1u);
                }
            }
#pragma unroll
            for (unsigned kk = 0; kk < T2 * L::CELL_BYTES / 256u; ++kk) sts_zero8(sn + (kk * 32u + lane) * 8u);
        } else {
            // How many records are really this tile's decides the counter width.  Records of the spill list belong to any tile, so a
            // long list is counted first (one more pass over it) instead of sending every tile of the grid to the wide counters.
            unsigned n_mine = n_all;
            if (n_spill && n_all > NMAX16) {
                n_mine = n_in;
                for (unsigned base = 0; base < n_spill; base += 32u) {
                    bool mine = false;
                    if (base + lane < n_spill) { const int4 r = ovf_in[base + lane]; mine = tile_of(tp, r.x, r.y) == tile; }
                    n_mine += __popc(__ballot_sync(FULL, mine));
                }
            }
            const bool crowded = L::NARROW || n_mine > NMAX16;      // warp-uniform
            unsigned* gcnt = nullptr;
            if (crowded) {                                           // 4 x 32-bit counters per cell in global scratch
                unsigned q = 0;
                if (lane == 0u) {
                    q = atomicAdd(&tp.tctl[3u + par], T2 * 2u);
                    if (q + T2 * 2u > tp.scratch_cap) { q = 0xFFFFFFFFu; atomicOr(&p.ctl->error, ERR_SCRATCH_OVERFLOW); }
                }
                q = __shfl_sync(FULL, q, 0);
                if (q != 0xFFFFFFFFu) {
                    gcnt = reinterpret_cast<unsigned*>(tp.scratch + q);
                    for (unsigned kk = lane; kk < T2 * 4u; kk += 32u) gcnt[kk] = 0u;
                }
                __syncwarp();
            }

            // ---- the step: every environment acts, moves and counts itself in its cell's histogram ----------
            // record j of this tile's input: its region, its arrival buffer, then the spill list (filtered by tile in the loop)
            auto fetch = [&](unsigned j) -> int4 {
                if (j >= n_all) return make_int4(0, 0, 0, 0);
                return j < n_front ? unpack_rec(in[roff + j], tx0, ty0) : j < n_in ? unpack_rec(arr_in[(size_t)tile * ARR_CAP + (j - n_front)], tx0, ty0) : ovf_in[j - n_in];
            };
            int4 ahead = fetch(lane);                                 // one round ahead of the loop: its latency hides behind a round of work
            for (unsigned it = 0; it * 32u < n_all; ++it) {
                const unsigned j = it * 32u + lane;
                bool act = j < n_all;
                const int4 rec = ahead;
                ahead = fetch(j + 32u);
                if (act && j >= n_in) act = tile_of(tp, rec.x, rec.y) == tile;
                const unsigned lx = (unsigned)(rec.x - tx0), ly = (unsigned)(rec.y - ty0);
                if (act && (lx | ly) >= T) { s_acc[5] = 1u; act = false; }
                int4 nrec = rec; bool stays = false;
                if (act) {
                    const unsigned ic = (ly << TSH) | lx, e = (unsigned)rec.w;
                    const U4 w = philox4x32_10(p.env_offset + e, 0u, (unsigned)g, (unsigned)(g >> 32), p.k0, p.k1 ^ TAG_POLICY);
                    const unsigned mvb = st[L::ST_MV + ic];
                    const int a = ((w.x >> 8) < c.eps_thr) ? (int)(w.y & 3u) : argmax4(s_q[ic]);
                    const bool blocked = (mvb >> a) & 1u, done = (mvb >> (4 + a)) & 1u;
                    const int dx = blocked ? 0 : (a == 1) - (a == 3), dy = blocked ? 0 : (a == 2) - (a == 0);
                    nrec.x = rec.x + dx; nrec.y = rec.y + dy; nrec.z = (int)min((unsigned)rec.z + 1u, T_SAT);
                    if (TRACE) { p.tr_a[e] = a; p.tr_r[e] = done ? 1.0f : blocked ? blocked_step_reward(p, rec.x, rec.y, a) : -0.01f; p.tr_d[e] = done ? 1 : 0; }
                    // 32-bit shared-memory atomics are native; the 64-bit word of a cell is counted in its two halves
                    if (!crowded) atomicAdd(reinterpret_cast<unsigned*>(s_n) + 2u * ic + ((unsigned)a >> 1), 1u << (16u * ((unsigned)a & 1u)));
                    else if (gcnt) atomicAdd(&gcnt[ic * 4u + (unsigned)a], 1u);
                    if (done || nrec.z >= c.tmax) {
                        const unsigned sn2 = sample_start(p, p.env_offset + e, g + 1ull, TAG_START);
                        nrec.y = (int)(sn2 / (unsigned)p.W); nrec.x = (int)(sn2 - (unsigned)nrec.y * (unsigned)p.W); nrec.z = 0;
                        atomicAdd(&s_acc[done ? 0 : 1], 1u);
                    }
                    stays = (((unsigned)(nrec.x - tx0)) | ((unsigned)(nrec.y - ty0))) < T;
                }
                if (put_stay(act, stays, pack_rec(tp, nrec))) { const unsigned dt = tile_of(tp, nrec.x, nrec.y); store_arrival(nrec, dt, atomicAdd(&cnt_next[dt].y, 1u)); }
            }
            __syncwarp();

            // ---- the occupied cells, compacted; the border ring starts out as max Q_t ----------------------------
            unsigned nocc = 0;
            if (!crowded) {
#pragma unroll
                for (unsigned kk = 0; kk < T2 / 32u; ++kk) {
                    const unsigned ic = kk * 32u + lane;
                    const bool nz = s_n[ic] != 0ull;
                    const unsigned m = __ballot_sync(FULL, nz);
                    if (nz) s_list[nocc + __popc(m & lt)] = (unsigned short)ic;
                    nocc += __popc(m);
                }
            } else nocc = gcnt ? T2 : 0u;
#pragma unroll
            for (unsigned r = 0; r < BR; ++r) if (lane + 32u * r < 4u * T) s_bm[lane + 32u * r] = max4(s_q[(b_pack >> (16u * r)) & 0xFFu]);
            __syncwarp();

            // ---- Q_{t+1} of the occupied cells, from Q_t in shared memory straight into the table -----------------
            for (unsigned idx = lane; idx < nocc; idx += 32u) {
                unsigned ic, tot; unsigned long long w = 0ull; unsigned n32[4];
                if (!crowded) {
                    ic = s_list[idx];
                    w = s_n[ic]; s_n[ic] = 0ull;
                    tot = ((unsigned)w & 0xFFFFu) + ((unsigned)(w >> 16) & 0xFFFFu) + ((unsigned)(w >> 32) & 0xFFFFu) + (unsigned)(w >> 48);
                } else {
                    ic = idx;
                    const uint4 v = *reinterpret_cast<const uint4*>(gcnt + 4u * ic);
                    n32[0] = v.x; n32[1] = v.y; n32[2] = v.z; n32[3] = v.w;
                    tot = v.x + v.y + v.z + v.w;
                }
                if (!tot) continue;
                if (tot > 1u) conf += tot;
                if (tot > CROWDED_CELL) { atomicAdd(&s_acc[3], 1u); atomicAdd(&s_acc[4], tot); }
                const float4 row = updated_row<TSH>(p, st, ic, w, crowded ? n32 : nullptr, tx0, ty0);
                const unsigned lx = ic & (T - 1u), ly = ic >> TSH;
                p.Q[(size_t)(ty0 + (int)ly) * (size_t)p.W + (size_t)(tx0 + (int)lx)] = row;
                const float mx = max4(row);
                if (ly == 0u) s_bm[lx] = mx;
                if (ly == T - 1u) s_bm[T + lx] = mx;
                if (lx == 0u) s_bm[2u * T + ly] = mx;
                if (lx == T - 1u) s_bm[3u * T + ly] = mx;
            }
        }
        if (lane == 0u) tp.cnt[par ^ 1u][tile].x = min(nstay, fcap);
        else if (lane == 1u) tp.cnt[par][tile] = make_uint2(0u, 0u);        // consumed; .y is the append counter again in the next step
        __syncwarp();

        // ---- border values out: max_a Q_{t+1} of my border ring into the neighbours' blocks of the other parity ----------
        {
            float* const hbase = halo_out + (size_t)tile * (4u * T);
            // which of the four neighbours exist: bit e = north, south, west, east
            const unsigned have = (tyi > 0u ? 1u : 0u) | (tyi + 1u < tp.tiles_y ? 2u : 0u) | (txi > 0u ? 4u : 0u) | (txi + 1u < tp.tiles_x ? 8u : 0u);
#pragma unroll
            for (unsigned r = 0; r < BR; ++r) {
                const unsigned kk = lane + 32u * r, ent = b_pack >> (16u * r);
                if (kk < 4u * T && ((have >> ((ent >> 8) & 3u)) & 1u)) hbase[b_dst[r]] = fast ? max4(lds_f4(sq + (ent & 0xFFu) * 16u)) : s_bm[kk];
            }
        }
        fence_async_smem();                                      // this lane's reads of the stage come before the copies that will refill it
        __syncwarp();                                            // every lane is done with the tile
    }

    if (pend) store_arrival(pend_rec, pend_dt, pend_pos);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");     // the next kernel's blocks may take the slots that free up

    // ---- run statistics: warp -> block -> one atomic per counter and block ----------------------------------
    for (int o = 16; o; o >>= 1) conf += __shfl_xor_sync(FULL, conf, o);
    if (lane == 0u && conf) atomicAdd(&s_acc[2], conf);
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_acc[2]) atomicAdd(&p.ctl->conflicts, (unsigned long long)s_acc[2]);
        if (s_acc[0]) atomicAdd(&p.ctl->goals, (unsigned long long)s_acc[0]);
        if (s_acc[1]) atomicAdd(&p.ctl->timeouts, (unsigned long long)s_acc[1]);
        if (s_acc[0] + s_acc[1]) atomicAdd(&p.ctl->episodes, (unsigned long long)(s_acc[0] + s_acc[1]));
        if (s_acc[3]) { atomicAdd(&p.ctl->long_chains, (unsigned long long)s_acc[3]); atomicAdd(&p.ctl->general, (unsigned long long)s_acc[4]); }
        if (s_acc[5]) atomicOr(&p.ctl->error, ERR_BAD_STATE);
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
    atomicAdd(&p.tp.cnt[p.step & 1ull][tile_of(p.tp, r.x, r.y)].x, 1u);
}
// One block: region capacities (population + 25 % + 32), their exclusive scan, counters reset.
__global__ void __launch_bounds__(1024) k_te_layout(Params p) {
    __shared__ unsigned s_warp[33];
    __shared__ unsigned s_carry;
    const TileP& tp = p.tp;
    const unsigned par = (unsigned)(p.step & 1ull);
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (unsigned base = 0; base < tp.ntiles; base += 1024u) {
        const unsigned k = base + threadIdx.x;
        const unsigned cnt = k < tp.ntiles ? tp.cnt[par][k].x : 0u;
        const unsigned F = (cnt + cnt / 4u + 33u) & ~1u;        // even: a region starts and ends on a 16-byte boundary
        unsigned total = 0;
        const unsigned ex = block_scan_excl(k < tp.ntiles ? F : 0u, s_warp, &total);
        const unsigned carry = s_carry;
        if (k < tp.ntiles) {
            tp.reg[k] = make_uint2(carry + ex, F);
            tp.cnt[0][k] = make_uint2(0u, 0u); tp.cnt[1][k] = make_uint2(0u, 0u);
        }
        __syncthreads();
        if (threadIdx.x == 0) s_carry = carry + total;
        __syncthreads();
    }
    if (threadIdx.x == 0) { tp.reg[tp.ntiles] = make_uint2(s_carry, 0u); for (int k = 0; k < 5; ++k) tp.tctl[k] = 0u; }
}
__global__ void k_te_scatter(Params p) {
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.N) return;
    const TileP& tp = p.tp;
    const unsigned par = (unsigned)(p.step & 1ull);
    const int4 r = p.st[i];
    const unsigned tile = tile_of(tp, r.x, r.y);
    const unsigned pos = atomicAdd(&tp.cnt[par][tile].x, 1u);
    tp.rec[par][tp.reg[tile].x + pos] = pack_rec(tp, r);
}
// The move byte of every cell, tile by tile as the step kernel copies them: bit a = a move in direction a is blocked (grid
// edge or obstacle, src/kernels.cu:29-44 of the reference), bit 4+a = the cell an environment stands on after choosing a is a
// goal (src/kernels.cu:56-59, src/environment.cu:43-46).  Cells of an edge tile that lie outside the grid: all blocked.
__global__ void __launch_bounds__(BLOCK) k_te_cls(Params p) {
    const TileP& tp = p.tp;
    const unsigned T = tp.T, T2 = T * T;
    const size_t total = (size_t)tp.ntiles * T2;
    for (size_t k = (size_t)blockIdx.x * BLOCK + threadIdx.x; k < total; k += (size_t)gridDim.x * BLOCK) {
        const unsigned tile = (unsigned)(k / T2), ic = (unsigned)(k - (size_t)tile * T2);
        const int x = (int)(((tile % tp.tiles_x) << tp.tshift) + (ic & (T - 1u))), y = (int)(((tile / tp.tiles_x) << tp.tshift) + (ic >> tp.tshift));
        unsigned b = 0x0Fu;
        if (x < p.W && y < p.H) {
            const unsigned own = p.cw[(unsigned)y * (unsigned)p.W + (unsigned)x];
            b = 0u;
            for (int a = 0; a < 4; ++a) {
                const int nx = x + (a == 1) - (a == 3), ny = y + (a == 2) - (a == 0);
                unsigned cls = CW_OBST;
                if (nx >= 0 && nx < p.W && ny >= 0 && ny < p.H) cls = p.cw[(unsigned)ny * (unsigned)p.W + (unsigned)nx];
                const bool blocked = (cls & CW_OBST) != 0u;
                if (blocked) b |= 1u << a;
                if ((blocked ? own : cls) & CW_GOAL) b |= 16u << a;
            }
        }
        tp.tcls[k] = (unsigned char)b;
    }
}
// The border array of the current parity from the table: for every tile the max over actions of the cells just
// outside its four edges (0 where the grid ends).  Needed whenever the table was changed by anything but a train step.
__global__ void __launch_bounds__(BLOCK) k_te_border(Params p) {
    const TileP& tp = p.tp;
    const unsigned T = tp.T, per = 4u * T;
    const size_t total = (size_t)tp.ntiles * per;
    float* dst = tp.bmax[p.step & 1ull];
    for (size_t k = (size_t)blockIdx.x * BLOCK + threadIdx.x; k < total; k += (size_t)gridDim.x * BLOCK) {
        const unsigned tile = (unsigned)(k / per), r = (unsigned)(k - (size_t)tile * per), e = r >> tp.tshift, i = r & (T - 1u);
        const int tx0 = (int)((tile % tp.tiles_x) << tp.tshift), ty0 = (int)((tile / tp.tiles_x) << tp.tshift);
        const int x = e == 2u ? tx0 - 1 : e == 3u ? tx0 + (int)T : tx0 + (int)i;
        const int y = e == 0u ? ty0 - 1 : e == 1u ? ty0 + (int)T : ty0 + (int)i;
        float m = 0.0f;
        if (x >= 0 && x < p.W && y >= 0 && y < p.H) m = max4(p.Q[(size_t)y * (size_t)p.W + (size_t)x]);
        dst[k] = m;
    }
}
// Back to environment order: st[id] = record.
__global__ void __launch_bounds__(BLOCK) k_te_export(Params p) {
    const TileP& tp = p.tp;
    const unsigned par = (unsigned)(p.step & 1ull);
    for (unsigned tile = blockIdx.x; tile < tp.ntiles; tile += gridDim.x) {
        const uint2 rg = tp.reg[tile];
        const uint2 cn = tp.cnt[par][tile];
        const unsigned n_front = min(cn.x, rg.y), n_arr = min(cn.y, ARR_CAP);
        const uint2* in = tp.rec[par] + rg.x;
        const uint2* ain = tp.arr[par] + (size_t)tile * ARR_CAP;
        const int tx0 = (int)((tile % tp.tiles_x) << tp.tshift), ty0 = (int)((tile / tp.tiles_x) << tp.tshift);
        for (unsigned j = threadIdx.x; j < n_front; j += BLOCK) { const int4 r = unpack_rec(in[j], tx0, ty0); if ((unsigned)r.w < p.N) p.st[r.w] = r; }
        for (unsigned j = threadIdx.x; j < n_arr; j += BLOCK) { const int4 r = unpack_rec(ain[j], tx0, ty0); if ((unsigned)r.w < p.N) p.st[r.w] = r; }
    }
}
__global__ void k_te_export_ovf(Params p) {
    const TileP& tp = p.tp;
    const unsigned n = min(tp.tctl[(unsigned)(p.step % 3ull)], p.N);
    const int4* in = tp.ovf[p.step & 1ull];
    for (unsigned j = blockIdx.x * blockDim.x + threadIdx.x; j < n; j += gridDim.x * blockDim.x) { const int4 r = in[j]; if ((unsigned)r.w < p.N) p.st[r.w] = r; }
}

// Replica averaging, the slice this rank owns.  The other ranks' rows of the slice lie in `others`, R - 1 blocks of
// n rows in ascending rank order; this rank's own rows are the table's.  Summed in rank order 0..R-1 in fp32 (the
// order of the CPU oracle), scaled by 1/R, written back into the table.
__global__ void __launch_bounds__(BLOCK) k_q_average_slice(float4* table, const float4* others, unsigned R, unsigned self, size_t cell0, size_t n, float scale) {
    for (size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += (size_t)gridDim.x * BLOCK) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (unsigned r = 0; r < R; ++r) {
            const float4 v = r == self ? table[cell0 + i] : others[(size_t)(r - (r > self ? 1u : 0u)) * n + i];
            if (r == 0u) acc = v;
            else { acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w); }
        }
        acc.x = __fmul_rn(acc.x, scale); acc.y = __fmul_rn(acc.y, scale); acc.z = __fmul_rn(acc.z, scale); acc.w = __fmul_rn(acc.w, scale);
        table[cell0 + i] = acc;
    }
}

// The same over peer memory: tables[r] is rank r's whole table (this rank's own, or a peer's mapped through CUDA IPC and
// accessed over NVLink with plain loads and stores); this rank sums the slice it owns in rank order and writes the result into
// EVERY rank's table -- reduce and hand-round in one kernel, both directions of the links in use at once.  Nobody else touches
// slice `self` of any table between the two barriers that bracket the kernel (see average_now).
template <unsigned RR>        // RR = number of ranks when it is small (all loads of a cell in flight together), 0 = any number
__global__ void __launch_bounds__(BLOCK) k_q_average_peers(float4* const* __restrict__ tables, unsigned R, unsigned self, size_t cell0, size_t n, float scale) {
    float4* tb[RR ? RR : 1u];
    if constexpr (RR != 0u) {
#pragma unroll
        for (unsigned r = 0; r < RR; ++r) tb[r] = tables[r];
    }
    for (size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += (size_t)gridDim.x * BLOCK) {
        float4 acc;
        if constexpr (RR != 0u) {
            float4 v[RR ? RR : 1u];
#pragma unroll
            for (unsigned r = 0; r < RR; ++r) v[r] = tb[r][cell0 + i];
            acc = v[0];
#pragma unroll
            for (unsigned r = 1; r < RR; ++r) { acc.x = __fadd_rn(acc.x, v[r].x); acc.y = __fadd_rn(acc.y, v[r].y); acc.z = __fadd_rn(acc.z, v[r].z); acc.w = __fadd_rn(acc.w, v[r].w); }
        } else {
            acc = tables[0][cell0 + i];
            for (unsigned r = 1; r < R; ++r) {
                const float4 v = tables[r][cell0 + i];
                acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
            }
        }
        acc.x = __fmul_rn(acc.x, scale); acc.y = __fmul_rn(acc.y, scale); acc.z = __fmul_rn(acc.z, scale); acc.w = __fmul_rn(acc.w, scale);
        if constexpr (RR != 0u) {
#pragma unroll
            for (unsigned r = 0; r < RR; ++r) tb[r][cell0 + i] = acc;
        } else {
            for (unsigned r = 0; r < R; ++r) tables[(self + r) % R][cell0 + i] = acc;       // own table first, then round the ring of peers
        }
    }
    __threadfence_system();
}

// ------------------------------------------------------------------------------------------------
static inline unsigned nblk(unsigned n) { return (n + BLOCK - 1) / BLOCK; }
static inline unsigned capped_blocks(size_t n) { const size_t b = (n + BLOCK - 1) / BLOCK; return (unsigned)(b < 1 ? 1 : (b > 2368 ? 2368 : b)); }

constexpr unsigned MINB16 = 7, MINB8 = 6;     // resident blocks per SM the register budget is cut for (16 x 16 tiles: no spills at 72 registers; 8 x 8 tiles: 8 bytes at 80, faster than 5 blocks at 94)
size_t tile_step_smem(const Params& p) { return (size_t)WPB * (p.tp.tshift == 4u ? WarpSmem<4>::BYTES : WarpSmem<3>::BYTES); }
unsigned tile_cls_stride(unsigned tshift) { return tshift == 4u ? WarpSmem<4>::CLS : WarpSmem<3>::CLS; }

template <unsigned TSH, unsigned MINB>
static cudaError_t configure_one(int bytes, int* per_sm) {
    cudaError_t e = cudaSuccess;
    const void* fns[3] = {(const void*)k_tile_step<false, TSH, MINB, false>, (const void*)k_tile_step<true, TSH, MINB, false>,
                          (const void*)k_tile_step<false, TSH, MINB, true>};
    for (const void* f : fns) {
        if (e == cudaSuccess) e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    }
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(per_sm, k_tile_step<false, TSH, MINB, false>, (int)(WPB * 32u), (size_t)bytes);
    if (e == cudaSuccess && *per_sm > 0) {
        // no more shared memory than the resident blocks need (1 KB per block is the system's): the rest stays first-level cache
        int pct = (int)(((size_t)*per_sm * ((size_t)bytes + 1024u + 256u) * 100u + 228u * 1024u - 1u) / (228u * 1024u));
        pct = pct > 100 ? 100 : pct;
        for (const void* f : fns) if (e == cudaSuccess) e = cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, pct);
    }
    return e;
}
int tile_engine_configure(Params& p, int device) {
    const int bytes = (int)tile_step_smem(p);
    int sms = 0, per_sm = 0;
    cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return (int)e;
    switch (p.tp.tshift) {
        case 3: e = configure_one<3, MINB8>(bytes, &per_sm); break;
        case 4: e = configure_one<4, MINB16>(bytes, &per_sm); break;
        default: return (int)cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) return (int)cudaErrorLaunchOutOfResources;
    p.tp.grid = (unsigned)(sms * per_sm);
    return 0;
}
void launch_tile_bucket(const Params& p, cudaStream_t st) {
    cudaMemsetAsync(p.tp.cnt[p.step & 1ull], 0, (size_t)p.tp.ntiles * sizeof(uint2), st);
    if (p.N) k_te_count<<<nblk(p.N), BLOCK, 0, st>>>(p);
    k_te_layout<<<1, 1024, 0, st>>>(p);
    if (p.N) k_te_scatter<<<nblk(p.N), BLOCK, 0, st>>>(p);
}
void launch_tile_classes(const Params& p, cudaStream_t st) { k_te_cls<<<capped_blocks((size_t)p.tp.ntiles * p.tp.T * p.tp.T), BLOCK, 0, st>>>(p); }
void launch_tile_border(const Params& p, cudaStream_t st) { k_te_border<<<capped_blocks((size_t)p.tp.ntiles * 4u * p.tp.T), BLOCK, 0, st>>>(p); }
void launch_tile_export(const Params& p, cudaStream_t st) {
    k_te_export<<<p.tp.ntiles < 4736u ? p.tp.ntiles : 4736u, BLOCK, 0, st>>>(p);
    k_te_export_ovf<<<64, BLOCK, 0, st>>>(p);
}
static unsigned tile_step_grid(const Params& p) { const unsigned need = (p.tp.ntiles + WPB - 1u) / WPB; return need < p.tp.grid ? need : p.tp.grid; }
template <unsigned TSH, unsigned MINB>
static void launch_step_one(const Params& p, bool trace, unsigned grid, size_t smem, cudaStream_t st) {
    cudaLaunchConfig_t cfg; memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(WPB * 32u); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    if (trace)                cudaLaunchKernelEx(&cfg, k_tile_step<true, TSH, MINB, false>, p);
    else if (p.tp.wait_polls) cudaLaunchKernelEx(&cfg, k_tile_step<false, TSH, MINB, true>, p);     // tests only: the waits run out
    else                      cudaLaunchKernelEx(&cfg, k_tile_step<false, TSH, MINB, false>, p);
}
void launch_tile_step(const Params& p, bool trace, cudaStream_t st) {
    const size_t smem = tile_step_smem(p);
    const unsigned grid = tile_step_grid(p);
    if (p.tp.tshift == 3u) launch_step_one<3, MINB8>(p, trace, grid, smem, st);
    else                   launch_step_one<4, MINB16>(p, trace, grid, smem, st);
    if (p.eps_from_ctl) k_tile_eps_episode<<<1, 1, 0, st>>>(p);
}
void launch_q_average_peers(float4* const* tables, unsigned R, unsigned self, size_t cell0, size_t n, float scale, cudaStream_t st) {
    if (!n) return;
    const unsigned blocks = capped_blocks(n);
    switch (R) {
        case 2: k_q_average_peers<2><<<blocks, BLOCK, 0, st>>>(tables, R, self, cell0, n, scale); break;
        case 3: k_q_average_peers<3><<<blocks, BLOCK, 0, st>>>(tables, R, self, cell0, n, scale); break;
        case 4: k_q_average_peers<4><<<blocks, BLOCK, 0, st>>>(tables, R, self, cell0, n, scale); break;
        case 8: k_q_average_peers<8><<<blocks, BLOCK, 0, st>>>(tables, R, self, cell0, n, scale); break;
        default: k_q_average_peers<0><<<blocks, BLOCK, 0, st>>>(tables, R, self, cell0, n, scale); break;
    }
}
void launch_q_average_slice(float4* table, const float4* others, unsigned R, unsigned self, size_t cell0, size_t n, float scale, cudaStream_t st) {
    if (n) k_q_average_slice<<<capped_blocks(n), BLOCK, 0, st>>>(table, others, R, self, cell0, n, scale);
}

}  // namespace cudarl
