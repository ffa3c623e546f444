// tile_engine.cu -- the fused train step as a streaming pass over the grid, one thread block per tile.
//
// With a quarter as many environments as cells, nearly every 128-byte line of the table is touched in
// every step, so the step is organised around the TABLE, not around the environments:
//
//   * the grid is cut into T x T tiles; the environments are kept bucketed by tile (records {x,y,t,id});
//   * one block loads its tile of Q_t plus a one-cell halo into shared memory with coalesced row loads
//     (the halo serves the max over Q_t[s'] of moves that leave the tile), and the tile's cell classes;
//   * every environment of the tile is stepped against shared memory: epsilon-greedy from the Philox
//     stream keyed by (seed, global env, step), move with obstacle / goal lookup, TD target from Q_t;
//   * a counting sort by cell (shared-memory counters) groups the (id, action, target) entries of one
//     cell; the cell's thread orders them by environment id and applies them one after the other, each
//     seeing the value the previous one left -- no float atomics, the same bits as the sequential
//     oracle however the entries arrived; cells with many occupants are sorted by the whole block;
//   * the tile of Q_{t+1} is written to the OTHER dense table with coalesced stores (two dense tables
//     alternate, so a block never sees a neighbour's writes of the same step);
//   * an environment that stays in the tile is appended to the front part of the tile's region of the
//     other record array; one that leaves (a walk across the edge, a restart anywhere) is appended to
//     the back part of its new tile's region with one atomic; a full back part spills to a global list
//     that every block filters.  Regions are re-sized from the actual populations every few steps.
//
// A tile with more environments than fit the shared sort buffer runs the same code on a slice of a
// global scratch array, so any distribution (all environments on one cell included) is handled.
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

constexpr unsigned SMALL_MAX = 24;   // occupants of one cell that the cell's own thread orders by insertion
constexpr unsigned BIG_LIST = 32;    // crowded cells a block lists; beyond that it scans all its cells

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

__device__ __forceinline__ void cswap_u2(uint2& a, uint2& b) { if (a.x > b.x) { const uint2 t = a; a = b; b = t; } }

// Block-wide ascending sort of a[0..n) by .x, any n: the bitonic network in its all-ascending form (the first
// comparator of every merge mirrors the index), so the missing tail behaves like +infinity and is never touched.
__device__ void block_sort_u2(uint2* a, unsigned n) {
    for (unsigned k = 2; (k >> 1) < n; k <<= 1) {
        for (unsigned i = threadIdx.x; i < n; i += blockDim.x) {
            const unsigned l = i ^ (k - 1u);
            if (l > i && l < n) { uint2 u = a[i], v = a[l]; if (u.x > v.x) { a[i] = v; a[l] = u; } }
        }
        __syncthreads();
        for (unsigned j = k >> 2; j > 0; j >>= 1) {
            for (unsigned i = threadIdx.x; i < n; i += blockDim.x) {
                const unsigned l = i ^ j;
                if (l > i && l < n) { uint2 u = a[i], v = a[l]; if (u.x > v.x) { a[i] = v; a[l] = u; } }
            }
            __syncthreads();
        }
    }
}

// Apply the entries e[0..n) (already in ascending environment id) to `row`.
__device__ __forceinline__ void fold_entries(float4& row, const uint2* e, unsigned n, float lr) {
    for (unsigned k = 0; k < n; ++k) { const uint2 v = e[k]; fold(row, (int)(v.x & 3u), lr, __uint_as_float(v.y)); }
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

// ------------------------------------------------------------------------------------------------
// Shared memory of one block (T = tile edge, HS = T + 2):
//   s_q    HS*HS float4   Q_t of the tile and its halo (read-only after the copy lands)
//   s_qn   T*T   float4   Q_{t+1} of the tile: starts as a copy of Q_t, updated cells are overwritten
//   s_sorted ch  uint2    fold entries {id << 2 | action, target} of the cells with several occupants
//   s_cnt  T*T   u32      occupants per cell
//   s_cur  T*T   u32      per cell: cursor into s_sorted (ends one past the cell's last entry)
//   s_list T*T   u16      cells with several occupants
//   s_ecell ch   u16      cell of each entry in s_sorted
//   s_cls  HS*HS u8       cell classes of the tile and its halo
constexpr unsigned TBLOCK = 256;
constexpr unsigned EPT = 4;          // entries a thread ranks in registers: ch = EPT * TBLOCK

template <bool TRACE>
__global__ void __launch_bounds__(TBLOCK, 4) k_tile_step(Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_bar;
    __shared__ unsigned s_stay, s_goals, s_timeouts, s_conf, s_nmulti, s_nent, s_nbig, s_nbigent, s_base, s_bad;
    __shared__ unsigned s_big[BIG_LIST];

    const TileP& tp = p.tp;
    const unsigned T = tp.T, HS = T + 2u, T2 = T * T, HS2 = HS * HS, tsh = tp.tshift;
    float4* s_q = reinterpret_cast<float4*>(smem);
    float4* s_qn = s_q + HS2;
    uint2* s_sorted = reinterpret_cast<uint2*>(s_qn + T2);
    unsigned* s_cnt = reinterpret_cast<unsigned*>(s_sorted + tp.ch);
    unsigned* s_cur = s_cnt + T2;
    unsigned short* s_list = reinterpret_cast<unsigned short*>(s_cur + T2);
    unsigned short* s_ecell = s_list + T2;
    unsigned char* s_cls = reinterpret_cast<unsigned char*>(s_ecell + tp.ch);

    const unsigned tid = threadIdx.x, lane = tid & 31u, tile = blockIdx.x;
    const unsigned long long g = p.step;
    const unsigned par = (unsigned)(g & 1ull);
    const int tx0 = (int)((tile % tp.tiles_x) << tsh), ty0 = (int)((tile / tp.tiles_x) << tsh);
    const float4* __restrict__ Qin = tp.Qd[par];
    float4* __restrict__ Qout = tp.Qd[par ^ 1u];
    const int4* __restrict__ in = tp.rec[par];
    int4* __restrict__ out = tp.rec[par ^ 1u];
    const int4* __restrict__ ovf_in = tp.ovf[par];
    int4* __restrict__ ovf_out = tp.ovf[par ^ 1u];
    unsigned* arr_next = tp.arr_cnt[par ^ 1u];
    unsigned* ovf_cnt_next = tp.tctl + (unsigned)((g + 1ull) % 3ull);

    // rows of the table this tile reads: halo rows [gy_lo, gy_hi] x columns [xs, xe], interior rows [0, ri) x [0, wi)
    const int xs = max(tx0 - 1, 0), xe = min(tx0 + (int)T, p.W - 1);
    const int gy_lo = max(ty0 - 1, 0), gy_hi = min(ty0 + (int)T, p.H - 1);
    const unsigned bytes_h = (unsigned)(xe - xs + 1) * 16u, rows_h = (unsigned)(gy_hi - gy_lo + 1);
    const unsigned wi = (unsigned)min((int)T, p.W - tx0), ri = (unsigned)min((int)T, p.H - ty0), bytes_i = wi * 16u;

    if (tid == 0) {
        s_stay = 0; s_goals = 0; s_timeouts = 0; s_conf = 0; s_nmulti = 0; s_nent = 0; s_nbig = 0; s_nbigent = 0; s_bad = 0; s_base = 0xFFFFFFFFu;
        mbar_init(&s_bar, 1u);
    }
    if (tile == 0 && tid == 0) { tp.tctl[(unsigned)((g + 2ull) % 3ull)] = 0u; tp.tctl[3u + (par ^ 1u)] = 0u; }   // nobody touches these in this step
    for (unsigned k = 4u * tid; k < T2; k += 4u * TBLOCK) *reinterpret_cast<uint4*>(s_cnt + k) = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();

    // ---- Q_t tile + halo, a second copy of the interior, the class bytes: bulk copies onto one barrier --
    if (tid == 0) mbar_arrive_expect_tx(&s_bar, rows_h * bytes_h + ri * bytes_i + tp.cls_stride);
    if (tid < HS) {
        const int gy = ty0 + (int)tid - 1;
        if (gy >= gy_lo && gy <= gy_hi)
            bulk_g2s(s_q + tid * HS + (unsigned)(xs - (tx0 - 1)), Qin + (size_t)gy * (size_t)p.W + (size_t)xs, bytes_h, &s_bar);
    } else if (tid < HS + T) {
        const unsigned r = tid - HS;
        if (r < ri) bulk_g2s(s_qn + r * T, Qin + (size_t)(ty0 + (int)r) * (size_t)p.W + (size_t)tx0, bytes_i, &s_bar);
    } else if (tid == TBLOCK - 1) {
        bulk_g2s(s_cls, tp.tcls + (size_t)tile * tp.cls_stride, tp.cls_stride, &s_bar);
    }

    const unsigned roff = tp.reg_off[tile], fcap = tp.front_cap[tile], bcap = tp.reg_off[tile + 1u] - roff - fcap;
    const unsigned n_front = min(tp.seg_cnt[par][tile], fcap);
    const unsigned n_in = n_front + min(tp.arr_cnt[par][tile], bcap);           // front part, then back part
    const unsigned n_all = n_in + min(tp.tctl[(unsigned)(g % 3ull)], p.N);      // then the global spill list, filtered by tile
    const float eps = p.eps_tab[p.eps_from_ctl ? p.ctl->eps_idx : p.eps_idx];

    // record j of this tile's input, or false if list entry j belongs to another tile
    auto fetch = [&](unsigned j, int4& r) -> bool {
        if (j < n_in) { r = in[roff + (j < n_front ? j : fcap + (j - n_front))]; return true; }
        r = ovf_in[j - n_in];
        return tile_of(tp, r.x, r.y) == tile;
    };

    // ---- pass A (while the copies fly): occupants per cell -----------------------------------------------
    for (unsigned j = tid; j < n_all; j += TBLOCK) {
        int4 r;
        if (!fetch(j, r)) continue;
        const unsigned lx = (unsigned)(r.x - tx0), ly = (unsigned)(r.y - ty0);
        if (lx >= T || ly >= T) { s_bad = 1u; continue; }
        atomicAdd(&s_cnt[(ly << tsh) + lx], 1u);
    }
    __syncthreads();

    // ---- cells with several occupants: space for their entries (one atomic per warp), and their list ----
    for (unsigned base = 0; base < T2; base += 4u * TBLOCK) {
        const unsigned c0 = base + 4u * tid;
        uint4 c = make_uint4(0u, 0u, 0u, 0u);
        if (c0 < T2) c = *reinterpret_cast<const uint4*>(s_cnt + c0);
        const unsigned m0 = c.x > 1u ? c.x : 0u, m1 = c.y > 1u ? c.y : 0u, m2 = c.z > 1u ? c.z : 0u, m3 = c.w > 1u ? c.w : 0u;
        const unsigned m = m0 + m1 + m2 + m3, nm = (m0 != 0u) + (m1 != 0u) + (m2 != 0u) + (m3 != 0u);
        unsigned im = m, il = nm;                                      // inclusive prefixes over the warp: entries, listed cells
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned t1 = __shfl_up_sync(FULL, im, o), t2 = __shfl_up_sync(FULL, il, o);
            if (lane >= (unsigned)o) { im += t1; il += t2; }
        }
        const unsigned totm = __shfl_sync(FULL, im, 31), totl = __shfl_sync(FULL, il, 31);
        unsigned wb_e = 0, wb_l = 0;
        if (lane == 0 && totl) { wb_e = atomicAdd(&s_nent, totm); wb_l = atomicAdd(&s_nmulti, totl); }
        wb_e = __shfl_sync(FULL, wb_e, 0) + im - m; wb_l = __shfl_sync(FULL, wb_l, 0) + il - nm;
        if (c0 < T2 && m) {
            const unsigned ex = wb_e;
            *reinterpret_cast<uint4*>(s_cur + c0) = make_uint4(ex, ex + m0, ex + m0 + m1, ex + m0 + m1 + m2);
            unsigned li = wb_l;
            if (m0) s_list[li++] = (unsigned short)c0;
            if (m1) s_list[li++] = (unsigned short)(c0 + 1u);
            if (m2) s_list[li++] = (unsigned short)(c0 + 2u);
            if (m3) s_list[li++] = (unsigned short)(c0 + 3u);
        }
    }
    __syncthreads();
    const unsigned nent = s_nent, nmulti = s_nmulti;
    if (nent > tp.ch) {                                           // too many for shared memory: a slice of the global scratch (block-uniform branch)
        if (tid == 0) {
            const unsigned b = atomicAdd(&tp.tctl[3u + par], nent);
            if (b + nent <= p.N) s_base = b; else { s_base = 0xFFFFFFFEu; atomicOr(&p.ctl->error, ERR_SCRATCH_OVERFLOW); }
        }
        __syncthreads();
    }
    const bool in_smem = s_base == 0xFFFFFFFFu, usable = s_base != 0xFFFFFFFEu;
    uint2* sorted = in_smem ? s_sorted : tp.scratch + (usable ? s_base : 0u);

    // the copies must have landed before this thread reads the tile
    {
        bool landed = false;
        for (unsigned it = 0; it < WAIT_LIMIT; ++it) if (mbar_try_wait(&s_bar, 0u)) { landed = true; break; }
        if (!landed) { atomicOr(&p.ctl->error, ERR_COPY_TIMEOUT); s_bad = 2u; }
    }

    // ---- pass B: the step itself ----------------------------------------------------------------------
    unsigned conf = 0;
    for (unsigned j = tid; j < n_all; j += TBLOCK) {
        int4 rec;
        if (!fetch(j, rec)) continue;
        const int x = rec.x, y = rec.y, t = rec.z; const unsigned e = (unsigned)rec.w;
        const unsigned lx = (unsigned)(x - tx0), ly = (unsigned)(y - ty0);
        if (lx >= T || ly >= T) continue;
        const unsigned ic = (ly << tsh) + lx, h = (ly + 1u) * HS + lx + 1u;
        const float4 row = s_q[h];
        const U4 w = philox4x32_10(p.env_offset + e, 0u, (unsigned)g, (unsigned)(g >> 32), p.k0, p.k1 ^ TAG_POLICY);
        const int a = (u01(w.x) < eps) ? (int)(w.y & 3u) : argmax4(row);
        const int dx = (a == 1) - (a == 3), dy = (a == 2) - (a == 0);
        int nx = x + dx, ny = y + dy;
        const bool inb = nx >= 0 && nx < p.W && ny >= 0 && ny < p.H;
        const unsigned ht = (unsigned)((int)h + dy * (int)HS + dx);       // inside the halo whenever the move is in bounds
        const bool moved = inb && !(s_cls[inb ? ht : h] & CW_OBST);
        const unsigned h2 = moved ? ht : h;
        nx = moved ? nx : x; ny = moved ? ny : y;
        const bool done = (s_cls[h2] & CW_GOAL) != 0;
        const float r = done ? 1.0f : -0.01f;
        float m = 0.0f;
        if (!done) { m = max4(s_q[h2]); if (p.legacy_clamp && m < 0.0f) m = 0.0f; }
        const float d = __fmaf_rn(p.gamma, m, r);                         // TD target from Q_t; the error is taken in fold()
        if (TRACE) { p.tr_a[e] = a; p.tr_r[e] = r; p.tr_d[e] = done ? 1 : 0; }
        if (s_cnt[ic] == 1u) {                                            // alone on the cell: its row is final right away
            float4 nr = row; fold(nr, a, p.lr, d); s_qn[ic] = nr;
        } else {
            conf += 1u;
            if (usable) {
                const unsigned pos = atomicAdd(&s_cur[ic], 1u);
                sorted[pos] = make_uint2((e << 2) | (unsigned)a, __float_as_uint(d));
                if (in_smem) s_ecell[pos] = (unsigned short)ic;
            }
        }
        // episode bookkeeping and the record of the next step
        const bool timeout = !done && p.max_steps > 0 && t + 1 >= p.max_steps;
        int nt = t + 1;
        if (done || timeout) {
            const unsigned sn = sample_start(p, p.env_offset + e, g + 1ull, TAG_START);
            nx = (int)(sn % (unsigned)p.W); ny = (int)(sn / (unsigned)p.W); nt = 0;
            atomicAdd(done ? &s_goals : &s_timeouts, 1u);
        }
        const int4 nrec = make_int4(nx, ny, nt, (int)e);
        const unsigned dt = tile_of(tp, nx, ny);
        bool placed = false;
        if (dt == tile) {
            cg::coalesced_group cgp = cg::coalesced_threads();
            unsigned pos = 0;
            if (cgp.thread_rank() == 0) pos = atomicAdd(&s_stay, cgp.size());
            pos = cgp.shfl(pos, 0) + cgp.thread_rank();
            if (pos < fcap) { out[roff + pos] = nrec; placed = true; }
        }
        if (!placed) {
            const unsigned doff = tp.reg_off[dt], dfc = tp.front_cap[dt], dbc = tp.reg_off[dt + 1u] - doff - dfc;
            const unsigned pos = atomicAdd(&arr_next[dt], 1u);
            if (pos < dbc) out[doff + dfc + pos] = nrec;
            else {
                const unsigned q = atomicAdd(ovf_cnt_next, 1u);
                if (q < p.N) ovf_out[q] = nrec; else atomicOr(&p.ctl->error, ERR_BAD_STATE);
            }
        }
    }
    __syncthreads();

    // ---- order the entries of each shared cell by environment id ------------------------------------------
    if (in_smem) {
        // every entry counts the entries of its cell with a smaller id (ids are unique): that is its place
        uint2 ent[EPT]; unsigned dst[EPT];
#pragma unroll
        for (unsigned k = 0; k < EPT; ++k) {
            const unsigned pos = tid + k * TBLOCK;
            dst[k] = 0xFFFFFFFFu; ent[k] = make_uint2(0u, 0u);
            if (pos < nent) {
                ent[k] = s_sorted[pos];
                const unsigned ic = s_ecell[pos], cnt = s_cnt[ic], start = s_cur[ic] - cnt;
                unsigned rank = 0;
                for (unsigned q = start; q < start + cnt; ++q) rank += s_sorted[q].x < ent[k].x ? 1u : 0u;
                dst[k] = start + rank;
            }
        }
        __syncthreads();
#pragma unroll
        for (unsigned k = 0; k < EPT; ++k) if (dst[k] != 0xFFFFFFFFu) s_sorted[dst[k]] = ent[k];
        __syncthreads();
        for (unsigned k = tid; k < nmulti; k += TBLOCK) {
            const unsigned ic = s_list[k], cnt = s_cnt[ic];
            float4 row = s_q[((ic >> tsh) + 1u) * HS + (ic & (T - 1u)) + 1u];
            fold_entries(row, s_sorted + (s_cur[ic] - cnt), cnt, p.lr);
            s_qn[ic] = row;
            if (cnt > SMALL_MAX) { atomicAdd(&s_nbig, 1u); atomicAdd(&s_nbigent, cnt); }
        }
    } else if (usable) {
        // a tile too crowded for shared memory: small cells are ordered by their own thread, large ones by the whole block
        for (unsigned k = tid; k < nmulti; k += TBLOCK) {
            const unsigned ic = s_list[k], cnt = s_cnt[ic];
            if (cnt <= SMALL_MAX) {
                uint2* e = sorted + (s_cur[ic] - cnt);
                for (unsigned i = 1; i < cnt; ++i) {
                    const uint2 v = e[i]; unsigned q = i;
                    while (q > 0 && e[q - 1u].x > v.x) { e[q] = e[q - 1u]; --q; }
                    e[q] = v;
                }
                float4 row = s_q[((ic >> tsh) + 1u) * HS + (ic & (T - 1u)) + 1u];
                fold_entries(row, e, cnt, p.lr);
                s_qn[ic] = row;
            } else {
                const unsigned kb = atomicAdd(&s_nbig, 1u);
                if (kb < BIG_LIST) s_big[kb] = ic;
                atomicAdd(&s_nbigent, cnt);
            }
        }
        __syncthreads();
        const unsigned nbig = s_nbig;
        if (nbig && nbig <= BIG_LIST) {
            for (unsigned k = 0; k < nbig; ++k) { const unsigned ic = s_big[k], cnt = s_cnt[ic]; block_sort_u2(sorted + (s_cur[ic] - cnt), cnt); }
            for (unsigned k = tid; k < nbig; k += TBLOCK) {
                const unsigned ic = s_big[k], cnt = s_cnt[ic];
                float4 row = s_q[((ic >> tsh) + 1u) * HS + (ic & (T - 1u)) + 1u];
                fold_entries(row, sorted + (s_cur[ic] - cnt), cnt, p.lr);
                s_qn[ic] = row;
            }
        } else if (nbig) {
            for (unsigned k = 0; k < nmulti; ++k) { const unsigned ic = s_list[k], cnt = s_cnt[ic]; if (cnt > SMALL_MAX) block_sort_u2(sorted + (s_cur[ic] - cnt), cnt); }
            for (unsigned k = tid; k < nmulti; k += TBLOCK) {
                const unsigned ic = s_list[k], cnt = s_cnt[ic];
                if (cnt <= SMALL_MAX) continue;
                float4 row = s_q[((ic >> tsh) + 1u) * HS + (ic & (T - 1u)) + 1u];
                fold_entries(row, sorted + (s_cur[ic] - cnt), cnt, p.lr);
                s_qn[ic] = row;
            }
        }
    }

    // ---- tile of Q_{t+1} out: one bulk copy per row ----------------------------------------------------
    fence_async_smem();                                                   // the rows were written through the generic proxy
    for (int o = 16; o; o >>= 1) conf += __shfl_xor_sync(FULL, conf, o);
    if (lane == 0u && conf) atomicAdd(&s_conf, conf);
    __syncthreads();
    if (tid < ri && s_bad != 2u) {
        bulk_s2g(Qout + (size_t)(ty0 + (int)tid) * (size_t)p.W + (size_t)tx0, s_qn + tid * T, bytes_i);
        bulk_commit_wait_read();
    }
    if (tid == TBLOCK - 1) {
        tp.seg_cnt[par ^ 1u][tile] = min(s_stay, fcap);
        tp.arr_cnt[par][tile] = 0u;                                       // consumed; it is the append counter again in the next step
        if (s_conf) atomicAdd(&p.ctl->conflicts, (unsigned long long)s_conf);
        if (s_goals) atomicAdd(&p.ctl->goals, (unsigned long long)s_goals);
        if (s_timeouts) atomicAdd(&p.ctl->timeouts, (unsigned long long)s_timeouts);
        if (s_goals + s_timeouts) atomicAdd(&p.ctl->episodes, (unsigned long long)(s_goals + s_timeouts));
        if (s_nbig) { atomicAdd(&p.ctl->long_chains, (unsigned long long)s_nbig); atomicAdd(&p.ctl->general, (unsigned long long)s_nbigent); }
        if (s_bad == 1u) atomicOr(&p.ctl->error, ERR_BAD_STATE);
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

size_t tile_step_smem(const Params& p) {
    const size_t T = p.tp.T, HS = T + 2;
    return HS * HS * 16 + T * T * 16 + (size_t)p.tp.ch * 8 + 2 * T * T * 4 + T * T * 2 + (size_t)p.tp.ch * 2 + ((HS * HS + 15) / 16) * 16;
}
int tile_engine_configure(const Params& p) {
    const int bytes = (int)tile_step_smem(p);
    cudaError_t e = cudaFuncSetAttribute(k_tile_step<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_tile_step<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    return (int)e;
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
void launch_tile_step(const Params& p, bool trace, cudaStream_t st, cudaEvent_t ev_a, cudaEvent_t ev_b, cudaEvent_t ev_c) {
    const size_t smem = tile_step_smem(p);
    if (ev_a) cudaEventRecord(ev_a, st);
    if (trace) k_tile_step<true><<<p.tp.ntiles, TBLOCK, smem, st>>>(p);
    else       k_tile_step<false><<<p.tp.ntiles, TBLOCK, smem, st>>>(p);
    if (ev_b) cudaEventRecord(ev_b, st);
    if (p.eps_from_ctl) k_tile_eps_episode<<<1, 1, 0, st>>>(p);
    if (ev_c) cudaEventRecord(ev_c, st);
}
void launch_q_average_dense(const Params& p, float4* table, const float4* gathered, unsigned R, unsigned cell0, unsigned n, float scale, cudaStream_t st) {
    (void)p;
    if (n) k_q_average_dense<<<nblk(n), BLOCK, 0, st>>>(table, gathered, R, cell0, n, scale);
}

}  // namespace cudarl
