// tile_engine.cu -- the fused train step as a streaming pass over the grid, one WARP per tile.
//
// With a quarter as many environments as cells, nearly every 128-byte line of the table is touched in
// every step, so the step is organised around the TABLE, not around the environments:
//
//   * the grid is cut into T x T tiles (16 x 16 cells, or 8 x 8 on densely populated grids); the environments
//     are kept bucketed by tile (records {x,y,t,id});
//   * a warp owns a tile for the whole step and needs no block-wide barrier: it fetches the tile of Q_t with
//     ONE tensor copy (cp.async.bulk.tensor, a T x T box of float4 out of the row-major table), plus the
//     tile's class bytes and its border values, completion on the warp's own mbarrier; while the copies are
//     in flight it already holds the tile's first records in registers and the next tile's header;
//   * every environment of the tile is stepped against shared memory: epsilon-greedy from the Philox
//     stream keyed by (seed, global env, step), move with obstacle / goal lookup, auto-reset;
//   * the TD updates of a cell are applied from a histogram of (cell, action) counts: inside one step the
//     target of an update depends on (cell, action) only, so n environments on one (cell, action) mean the
//     same map applied n times -- the same bits as the oracle's sequential order, without sorting anything
//     and without float atomics;
//   * the table is updated IN PLACE: only the rows of occupied cells are stored (16 bytes each, straight from
//     registers), and no other warp reads this tile's cells in this step.  The one thing a neighbour needs
//     from a tile -- max_a Q of the cell just beyond the shared edge, for the TD target of a move across the
//     edge -- travels through a border array: at the end of its step a tile stores the max of every cell of
//     its border ring (taken from Q_{t+1}) into its four neighbours' slots of the OTHER parity;
//   * an environment that stays in the tile is appended to the tile's region of the other record array
//     (positions from a warp ballot, no atomics); one that leaves (a walk across the edge, a restart anywhere)
//     is appended to its new tile's arrival buffer with one atomic; a full arrival buffer spills to a global
//     list that every warp filters.  Regions are re-sized from the actual populations every few steps.
//
// Reference semantics (paths relative to the CudaRL-Arena project root):
//   step        src/environment.cu:17-48, obstacle test src/kernels.cu:29-44, goal src/kernels.cu:56-59
//   TD update   src/kernels.cu:96-114 (true max as in src/gpu/kernels.cu:36-45, src/train.py:134)
//   eps-greedy  src/train.py:101-108, first-max argmax src/q_learning.cu:196-206
//   episode     src/train.py:191-222
#include "kernels.cuh"
#include "rules.cuh"

namespace cudarl {

constexpr unsigned CROWDED_CELL = 24;   // a cell with more environments than this counts as "crowded" in the run statistics
constexpr unsigned NMAX16 = 65535u;     // records of a tile the 16-bit counters can hold
constexpr unsigned WPB = 4;             // warps per block; every warp works on its own
constexpr unsigned PRE = 3;             // records per lane fetched before the warp waits for its copies

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
__device__ __forceinline__ void tensor_g2s_2d(void* dst, const CUtensorMap* map, int c0, int c1, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(smem_u32(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}
constexpr unsigned long long WAIT_NS = 2000000000ull;   // a copy that has not landed after two seconds never will

// Wait for the phase with the given parity.  Bounded: by `polls` tries when polls > 0 (tests make the wait run
// out that way), else by WAIT_NS of wall time.  false = gave up.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, unsigned polls) {
    if (polls) {
        for (unsigned it = 0; it < polls; ++it) if (mbar_try_wait(bar, parity)) return true;
        return false;
    }
    unsigned long long t0 = 0ull;
    for (unsigned it = 1u;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 1023u) == 0u) {
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
// Shared memory of one warp (nothing is shared between warps):
//   s_q    T*T  float4   Q_t of the tile, row-major inside the tile; never written by the warp
//   s_n    T*T  u64      per cell: how many environments chose action a, 16 bits per action; zero between tiles
//   s_halo 4T   float    max_a Q_t of the cells beyond the north / south / west / east edge (from the border array)
//   s_bm   4T   float    max_a Q_{t+1} of the tile's own north / south / west / east border cells, on their way out
//   s_cls  (T+2)^2 u8    cell classes of the tile and a one-cell halo
//   s_list T*T  u16      occupied cells
// A tile with more than 65,535 records counts in 32-bit counters in global scratch instead.
template <unsigned TSH> struct WarpSmem {
    static constexpr unsigned T = 1u << TSH, T2 = T * T, HS = T + 2u;
    static constexpr unsigned CLS = (HS * HS + 15u) / 16u * 16u;
    static constexpr unsigned OFF_N = T2 * 16u, OFF_HALO = OFF_N + T2 * 8u, OFF_BM = OFF_HALO + 4u * T * 4u,
                              OFF_CLS = OFF_BM + 4u * T * 4u, OFF_LIST = OFF_CLS + CLS;
    static constexpr unsigned BYTES = (OFF_LIST + T2 * 2u + 127u) / 128u * 128u;
    static constexpr unsigned TX_BYTES = T2 * 16u + CLS + 4u * T * 4u;      // what the three copies of a tile deliver
};

// Everything the per-environment step needs about the tile being processed.
struct StepCtx {
    const float4* s_q; const unsigned char* s_cls; const float* s_halo;
    int tx0, ty0; unsigned tile;
    float eps; unsigned long long g;
};

// max_a Q_t of the cell reached from tile-local (lx, ly) by (dx, dy): from the tile, or from the border
// values when the move crosses an edge.
template <unsigned TSH>
__device__ __forceinline__ float next_max(const StepCtx& c, unsigned lx, unsigned ly, int dx, int dy) {
    constexpr unsigned T = 1u << TSH;
    const int mx = (int)lx + dx, my = (int)ly + dy;
    if (my < 0) return c.s_halo[lx];
    if (my >= (int)T) return c.s_halo[T + lx];
    if (mx < 0) return c.s_halo[2u * T + ly];
    if (mx >= (int)T) return c.s_halo[3u * T + ly];
    return max4(c.s_q[((unsigned)my << TSH) + (unsigned)mx]);
}

// Q_{t+1} row of one cell from Q_t and the number of environments that chose each action
// (`w`: 16 bits per action, or `n32` when the tile counts in 32 bits).  Only the actions that were chosen are visited.
template <unsigned TSH>
__device__ __forceinline__ float4 updated_row(const Params& p, const StepCtx& c, unsigned ic, unsigned long long w, const unsigned* n32) {
    constexpr unsigned T = 1u << TSH, HS = T + 2u;
    const unsigned lx = ic & (T - 1u), ly = ic >> TSH, hh = (ly + 1u) * HS + lx + 1u;
    const int x = c.tx0 + (int)lx, y = c.ty0 + (int)ly;
    float4 row = c.s_q[ic];
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
        const bool done = (c.s_cls[moved ? ht : hh] & CW_GOAL) != 0;
        float m = 0.0f;
        if (!done) { m = moved ? next_max<TSH>(c, lx, ly, dx, dy) : max4(c.s_q[ic]); if (p.legacy_clamp && m < 0.0f) m = 0.0f; }
        const float d = __fmaf_rn(p.gamma, m, done ? 1.0f : -0.01f);     // the TD target of (cell, a), from Q_t
        float v = pick(row, a);
        for (unsigned i = 0; i < n; ++i) v = __fmaf_rn(p.lr, __fsub_rn(d, v), v);       // one application per environment
        row.x = a == 0 ? v : row.x; row.y = a == 1 ? v : row.y; row.z = a == 2 ? v : row.z; row.w = a == 3 ? v : row.w;
    }
    return row;
}

template <bool TRACE, unsigned TSH, unsigned MINB>
__global__ void __launch_bounds__(WPB * 32u, MINB) k_tile_step(const __grid_constant__ Params p) {
    using L = WarpSmem<TSH>;
    constexpr unsigned T = L::T, T2 = L::T2, HS = L::HS;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_bar[WPB];
    __shared__ unsigned s_acc[6];            // goals, timeouts, conflicts, crowded cells, environments on them, bad records

    const TileP& tp = p.tp;
    const unsigned lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const unsigned lt = (1u << lane) - 1u;
    unsigned char* wb = smem + warp * L::BYTES;
    float4* s_q = reinterpret_cast<float4*>(wb);
    unsigned long long* s_n = reinterpret_cast<unsigned long long*>(wb + L::OFF_N);
    float* s_halo = reinterpret_cast<float*>(wb + L::OFF_HALO);
    float* s_bm = reinterpret_cast<float*>(wb + L::OFF_BM);
    unsigned char* s_cls = wb + L::OFF_CLS;
    unsigned short* s_list = reinterpret_cast<unsigned short*>(wb + L::OFF_LIST);
    unsigned long long* bar = &s_bar[warp];

    const unsigned long long g = p.step;
    const unsigned par = (unsigned)(g & 1ull);
    const int4* __restrict__ in = tp.rec[par];
    const int4* __restrict__ arr_in = tp.arr[par];
    const int4* __restrict__ ovf_in = tp.ovf[par];
    int4* __restrict__ out = tp.rec[par ^ 1u];
    int4* __restrict__ arr_out = tp.arr[par ^ 1u];
    int4* __restrict__ ovf_out = tp.ovf[par ^ 1u];
    unsigned* __restrict__ arr_next = tp.arr_cnt[par ^ 1u];
    unsigned* ovf_cnt_next = tp.tctl + (unsigned)((g + 1ull) % 3ull);
    const float* __restrict__ halo_in = tp.bmax[par];
    float* __restrict__ halo_out = tp.bmax[par ^ 1u];
    const unsigned gw = blockIdx.x * WPB + warp, nw = gridDim.x * WPB;

    if (threadIdx.x < 6u) s_acc[threadIdx.x] = 0u;
    if (lane == 0) mbar_init(bar, 1u);
    for (unsigned q = lane; q < T2; q += 32u) s_n[q] = 0ull;
    if (gw == 0u && lane == 0u) { tp.tctl[(unsigned)((g + 2ull) % 3ull)] = 0u; tp.tctl[3u + (par ^ 1u)] = 0u; }   // nobody touches these in this step
    __syncthreads();

    StepCtx c;
    c.s_q = s_q; c.s_cls = s_cls; c.s_halo = s_halo; c.g = g;
    c.eps = p.eps_tab[p.eps_from_ctl ? p.ctl->eps_idx : p.eps_idx];
    const unsigned n_spill = min(tp.tctl[(unsigned)(g % 3ull)], p.N);
    unsigned goals = 0, timeouts = 0, conf = 0, nbig = 0, nbigent = 0, bad = 0, phase = 0;

    // Header of a tile: lanes 0..3 each load one word {region start, capacity, records in the region, arrivals};
    // the words are only exchanged when the tile comes up, so the loads are off the path.
    auto fetch_hdr = [&](unsigned tile) -> unsigned {
        if (tile >= tp.ntiles || lane >= 4u) return 0u;
        const unsigned* src = lane == 0u ? &tp.reg[tile].x : lane == 1u ? &tp.reg[tile].y : lane == 2u ? &tp.seg_cnt[par][tile] : &tp.arr_cnt[par][tile];
        return *src;
    };
    unsigned hw = fetch_hdr(gw);

    for (unsigned tile = gw; tile < tp.ntiles; tile += nw) {
        const unsigned roff = __shfl_sync(FULL, hw, 0), fcap = __shfl_sync(FULL, hw, 1);
        const unsigned n_front = min(__shfl_sync(FULL, hw, 2), fcap), n_in = n_front + min(__shfl_sync(FULL, hw, 3), ARR_CAP);
        const unsigned n_all = n_in + n_spill;
        const unsigned tyi = tile / tp.tiles_x, txi = tile - tyi * tp.tiles_x;
        const int tx0 = (int)(txi << TSH), ty0 = (int)(tyi << TSH);
        c.tx0 = tx0; c.ty0 = ty0; c.tile = tile;

        // ---- the tile's copies: table box, class bytes, border values -------------------------------------
        if (lane == 0u) mbar_arrive_expect_tx(bar, L::TX_BYTES);
        __syncwarp();
        if (lane == 0u) tensor_g2s_2d(s_q, &tp.tmq, tx0 * 4, ty0, bar);
        else if (lane == 1u) bulk_g2s(s_cls, tp.tcls + (size_t)tile * L::CLS, L::CLS, bar);
        else if (lane == 2u) bulk_g2s(s_halo, halo_in + (size_t)tile * (4u * T), 4u * T * 4u, bar);

        // record j of this tile's input: its region, then its arrival buffer (the spill list is filtered in the loop)
        auto load_rec = [&](unsigned j) -> int4 { return j < n_front ? in[roff + j] : arr_in[(size_t)tile * ARR_CAP + (j - n_front)]; };
        int4 pre[PRE];
#pragma unroll
        for (unsigned q = 0; q < PRE; ++q) { const unsigned j = q * 32u + lane; pre[q] = j < n_in ? load_rec(j) : make_int4(0, 0, 0, 0); }
        hw = fetch_hdr(tile + nw);                              // in flight while this tile is worked on

        if (!__all_sync(FULL, mbar_wait(bar, phase, tp.wait_polls))) {
            // Never seen with the time bound.  Flag it, let the copies land (they target this warp's shared memory), stop.
            if (lane == 0u) atomicOr(&p.ctl->error, ERR_COPY_TIMEOUT);
            mbar_wait(bar, phase, 0u);
            break;
        }
        phase ^= 1u;

        const bool crowded = n_all > NMAX16;                    // warp-uniform
        unsigned* gcnt = nullptr;
        if (crowded) {                                           // 4 x 32-bit counters per cell in global scratch
            unsigned q = 0;
            if (lane == 0u) {
                q = atomicAdd(&tp.tctl[3u + par], T2 * 2u);
                if (q + T2 * 2u > p.N) { q = 0xFFFFFFFFu; atomicOr(&p.ctl->error, ERR_SCRATCH_OVERFLOW); }
            }
            q = __shfl_sync(FULL, q, 0);
            if (q != 0xFFFFFFFFu) {
                gcnt = reinterpret_cast<unsigned*>(tp.scratch + q);
                for (unsigned k = lane; k < T2 * 4u; k += 32u) gcnt[k] = 0u;
            }
            __syncwarp();
        }

        // ---- the step: every environment acts, moves and counts itself in its cell's histogram ----------
        unsigned nstay = 0;
        for (unsigned it = 0; it * 32u < n_all; ++it) {
            const unsigned j = it * 32u + lane;
            bool act = j < n_all;
            int4 rec = it == 0u ? pre[0] : it == 1u ? pre[1] : pre[2];
            if (act && j >= n_in) { rec = ovf_in[j - n_in]; act = tile_of(tp, rec.x, rec.y) == tile; }
            else if (act && it >= PRE) rec = load_rec(j);
            const unsigned e = (unsigned)rec.w;
            const unsigned lx = (unsigned)(rec.x - tx0), ly = (unsigned)(rec.y - ty0);
            if (act && (lx >= T || ly >= T)) { bad = 1u; act = false; }        // never seen: the record does not lie in this tile
            int4 nrec = make_int4(0, 0, 0, 0); unsigned dt = 0xFFFFFFFFu;
            if (act) {
                const unsigned ic = (ly << TSH) + lx, hh = (ly + 1u) * HS + lx + 1u;
                const U4 w = philox4x32_10(p.env_offset + e, 0u, (unsigned)g, (unsigned)(g >> 32), p.k0, p.k1 ^ TAG_POLICY);
                const int a = (u01(w.x) < c.eps) ? (int)(w.y & 3u) : argmax4(s_q[ic]);
                const int dx = (a == 1) - (a == 3), dy = (a == 2) - (a == 0);
                int nx = rec.x + dx, ny = rec.y + dy;
                const bool inb = nx >= 0 && nx < p.W && ny >= 0 && ny < p.H;
                const unsigned ht = (unsigned)((int)hh + dy * (int)HS + dx);      // inside the halo whenever the move is in bounds
                const bool moved = inb && !(s_cls[inb ? ht : hh] & CW_OBST);
                nx = moved ? nx : rec.x; ny = moved ? ny : rec.y;
                const bool done = (s_cls[moved ? ht : hh] & CW_GOAL) != 0;
                if (TRACE) { p.tr_a[e] = a; p.tr_r[e] = done ? 1.0f : -0.01f; p.tr_d[e] = done ? 1 : 0; }
                // the histogram: 32-bit shared-memory atomics are native; the 64-bit word of a cell is counted in its two halves
                if (!crowded) atomicAdd(reinterpret_cast<unsigned*>(s_n) + 2u * ic + ((unsigned)a >> 1), 1u << (16u * ((unsigned)a & 1u)));
                else if (gcnt) atomicAdd(&gcnt[ic * 4u + (unsigned)a], 1u);
                // episode bookkeeping and the record of the next step
                const bool timeout = !done && p.max_steps > 0 && rec.z + 1 >= p.max_steps;
                int nt = rec.z + 1;
                if (done || timeout) {
                    const unsigned sn = sample_start(p, p.env_offset + e, g + 1ull, TAG_START);
                    nx = (int)(sn % (unsigned)p.W); ny = (int)(sn / (unsigned)p.W); nt = 0;
                    if (done) ++goals; else ++timeouts;
                }
                nrec = make_int4(nx, ny, nt, (int)e);
                dt = ((unsigned)ny >> TSH) * tp.tiles_x + ((unsigned)nx >> TSH);
            }
            // stays: position in the tile's own region from a ballot; leaves (or no room): one atomic on the new tile's arrival buffer
            const bool stay = act && dt == tile;
            const unsigned sm = __ballot_sync(FULL, stay);
            const unsigned pos = nstay + __popc(sm & lt);
            nstay += __popc(sm);
            if (stay && pos < fcap) out[roff + pos] = nrec;
            else if (act) {
                const unsigned apos = atomicAdd(&arr_next[dt], 1u);
                if (apos < ARR_CAP) arr_out[(size_t)dt * ARR_CAP + apos] = nrec;
                else {
                    const unsigned q = atomicAdd(ovf_cnt_next, 1u);
                    if (q < p.N) ovf_out[q] = nrec; else bad = 1u;
                }
            }
        }
        if (lane == 0u) {
            tp.seg_cnt[par ^ 1u][tile] = min(nstay, fcap);
            tp.arr_cnt[par][tile] = 0u;                                   // consumed; it is the append counter again in the next step
        }
        __syncwarp();

        // ---- the occupied cells, compacted; the border ring starts out as max Q_t ----------------------------
        unsigned nocc = 0;
        if (!crowded) {
#pragma unroll
            for (unsigned k = 0; k < T2 / 32u; ++k) {
                const unsigned ic = k * 32u + lane;
                const bool nz = s_n[ic] != 0ull;
                const unsigned m = __ballot_sync(FULL, nz);
                if (nz) s_list[nocc + __popc(m & lt)] = (unsigned short)ic;
                nocc += __popc(m);
            }
        } else nocc = gcnt ? T2 : 0u;
        for (unsigned k = lane; k < 4u * T; k += 32u) {
            const unsigned e = k >> TSH, i = k & (T - 1u);
            const unsigned ic = e == 0u ? i : e == 1u ? ((T - 1u) << TSH) + i : e == 2u ? (i << TSH) : (i << TSH) + T - 1u;
            s_bm[k] = max4(s_q[ic]);
        }
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
            if (tot > CROWDED_CELL) { ++nbig; nbigent += tot; }
            const float4 row = updated_row<TSH>(p, c, ic, w, crowded ? n32 : nullptr);
            const unsigned lx = ic & (T - 1u), ly = ic >> TSH;
            p.Q[(size_t)(ty0 + (int)ly) * (size_t)p.W + (size_t)(tx0 + (int)lx)] = row;
            const float mx = max4(row);
            if (ly == 0u) s_bm[lx] = mx;
            if (ly == T - 1u) s_bm[T + lx] = mx;
            if (lx == 0u) s_bm[2u * T + ly] = mx;
            if (lx == T - 1u) s_bm[3u * T + ly] = mx;
        }
        __syncwarp();

        // ---- border values out: my north row is the south halo of the tile above, and so on ----------------
        for (unsigned k = lane; k < 4u * T; k += 32u) {
            const unsigned e = k >> TSH, i = k & (T - 1u);
            bool there; unsigned nt, slot;
            if (e == 0u)      { there = tyi > 0u;               nt = tile - tp.tiles_x; slot = 1u; }
            else if (e == 1u) { there = tyi + 1u < tp.tiles_y;  nt = tile + tp.tiles_x; slot = 0u; }
            else if (e == 2u) { there = txi > 0u;               nt = tile - 1u;         slot = 3u; }
            else              { there = txi + 1u < tp.tiles_x;  nt = tile + 1u;         slot = 2u; }
            if (there) halo_out[((size_t)nt * 4u + slot) * T + i] = s_bm[k];
        }
        fence_async_smem();                                      // this lane's reads of the tile come before the next copies' writes
        __syncwarp();                                            // every lane is done with the tile before the next copies are issued
    }

    // ---- run statistics: warp -> block -> one atomic per counter and block ----------------------------------
    for (int o = 16; o; o >>= 1) {
        goals += __shfl_xor_sync(FULL, goals, o); timeouts += __shfl_xor_sync(FULL, timeouts, o); conf += __shfl_xor_sync(FULL, conf, o);
        nbig += __shfl_xor_sync(FULL, nbig, o); nbigent += __shfl_xor_sync(FULL, nbigent, o); bad |= __shfl_xor_sync(FULL, bad, o);
    }
    if (lane == 0u) {
        if (goals) atomicAdd(&s_acc[0], goals);
        if (timeouts) atomicAdd(&s_acc[1], timeouts);
        if (conf) atomicAdd(&s_acc[2], conf);
        if (nbig) { atomicAdd(&s_acc[3], nbig); atomicAdd(&s_acc[4], nbigent); }
        if (bad) atomicOr(&s_acc[5], 1u);
    }
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
    atomicAdd(&p.tp.seg_cnt[p.step & 1ull][tile_of(p.tp, r.x, r.y)], 1u);
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
        const unsigned cnt = k < tp.ntiles ? tp.seg_cnt[par][k] : 0u;
        const unsigned F = cnt + cnt / 4u + 32u;
        unsigned total = 0;
        const unsigned ex = block_scan_excl(k < tp.ntiles ? F : 0u, s_warp, &total);
        const unsigned carry = s_carry;
        if (k < tp.ntiles) {
            tp.reg[k] = make_uint2(carry + ex, F);
            tp.seg_cnt[par][k] = 0u; tp.seg_cnt[par ^ 1u][k] = 0u; tp.arr_cnt[0][k] = 0u; tp.arr_cnt[1][k] = 0u;
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
    const unsigned pos = atomicAdd(&tp.seg_cnt[par][tile], 1u);
    tp.rec[par][tp.reg[tile].x + pos] = r;
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
        const unsigned n_front = min(tp.seg_cnt[par][tile], rg.y), n_arr = min(tp.arr_cnt[par][tile], ARR_CAP);
        const int4* in = tp.rec[par] + rg.x;
        const int4* ain = tp.arr[par] + (size_t)tile * ARR_CAP;
        for (unsigned j = threadIdx.x; j < n_front; j += BLOCK) { const int4 r = in[j]; if ((unsigned)r.w < p.N) p.st[r.w] = r; }
        for (unsigned j = threadIdx.x; j < n_arr; j += BLOCK) { const int4 r = ain[j]; if ((unsigned)r.w < p.N) p.st[r.w] = r; }
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

// ------------------------------------------------------------------------------------------------
static inline unsigned nblk(unsigned n) { return (n + BLOCK - 1) / BLOCK; }
static inline unsigned capped_blocks(size_t n) { const size_t b = (n + BLOCK - 1) / BLOCK; return (unsigned)(b < 1 ? 1 : (b > 2368 ? 2368 : b)); }

constexpr unsigned MINB16 = 6, MINB8 = 6;     // resident blocks per SM the register budget is cut for
size_t tile_step_smem(const Params& p) { return (size_t)WPB * (p.tp.tshift == 4u ? WarpSmem<4>::BYTES : WarpSmem<3>::BYTES); }
unsigned tile_cls_stride(unsigned tshift) { return tshift == 4u ? WarpSmem<4>::CLS : WarpSmem<3>::CLS; }

template <unsigned TSH, unsigned MINB>
static cudaError_t configure_one(int bytes, int* per_sm) {
    cudaError_t e = cudaSuccess;
    const void* fns[2] = {(const void*)k_tile_step<false, TSH, MINB>, (const void*)k_tile_step<true, TSH, MINB>};
    for (const void* f : fns) {
        if (e == cudaSuccess) e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    }
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(per_sm, k_tile_step<false, TSH, MINB>, (int)(WPB * 32u), (size_t)bytes);
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
    cudaMemsetAsync(p.tp.seg_cnt[p.step & 1ull], 0, (size_t)p.tp.ntiles * sizeof(unsigned), st);
    if (p.N) k_te_count<<<nblk(p.N), BLOCK, 0, st>>>(p);
    k_te_layout<<<1, 1024, 0, st>>>(p);
    if (p.N) k_te_scatter<<<nblk(p.N), BLOCK, 0, st>>>(p);
}
void launch_tile_classes(const Params& p, cudaStream_t st) { k_te_cls<<<p.tp.ntiles, BLOCK, 0, st>>>(p); }
void launch_tile_border(const Params& p, cudaStream_t st) { k_te_border<<<capped_blocks((size_t)p.tp.ntiles * 4u * p.tp.T), BLOCK, 0, st>>>(p); }
void launch_tile_export(const Params& p, cudaStream_t st) {
    k_te_export<<<p.tp.ntiles < 4736u ? p.tp.ntiles : 4736u, BLOCK, 0, st>>>(p);
    k_te_export_ovf<<<64, BLOCK, 0, st>>>(p);
}
static unsigned tile_step_grid(const Params& p) { const unsigned need = (p.tp.ntiles + WPB - 1u) / WPB; return need < p.tp.grid ? need : p.tp.grid; }
template <unsigned TSH, unsigned MINB>
static void launch_step_one(const Params& p, bool trace, unsigned grid, size_t smem, cudaStream_t st) {
    if (trace) k_tile_step<true, TSH, MINB><<<grid, WPB * 32u, smem, st>>>(p);
    else       k_tile_step<false, TSH, MINB><<<grid, WPB * 32u, smem, st>>>(p);
}
void launch_tile_step(const Params& p, bool trace, cudaStream_t st) {
    const size_t smem = tile_step_smem(p);
    const unsigned grid = tile_step_grid(p);
    if (p.tp.tshift == 3u) launch_step_one<3, MINB8>(p, trace, grid, smem, st);
    else                   launch_step_one<4, MINB16>(p, trace, grid, smem, st);
    if (p.eps_from_ctl) k_tile_eps_episode<<<1, 1, 0, st>>>(p);
}
void launch_q_average_slice(float4* table, const float4* others, unsigned R, unsigned self, size_t cell0, size_t n, float scale, cudaStream_t st) {
    if (n) k_q_average_slice<<<capped_blocks(n), BLOCK, 0, st>>>(table, others, R, self, cell0, n, scale);
}

}  // namespace cudarl
