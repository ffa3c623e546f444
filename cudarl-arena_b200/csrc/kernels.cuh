// kernels.cuh -- device-side data layout and launch entry points shared by kernels.cu, tile_engine.cu (the
// sm_100a kernels) and context.cu (the C ABI).  Nothing here is visible outside the library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cudarl {

// ---- per-cell word (16 bits per grid cell, array padded to 16 bytes): the cell's class ------------
enum : unsigned {
    CW_OBST = 1u,      // cell blocks movement                     (src/kernels.cu:29-36 of the reference)
    CW_GOAL = 2u,      // cell ends the episode, reward 1          (src/environment.cu:43-46)
    CW_TRAP = 4u,      // an obstacle whose penalty replaces the step cost of an agent that walks into it (src/kernels.cu:61-63)
};

// A chain link names a run of consecutive collision entries: low 26 bits = position of the first entry + 1
// (0 = end of chain), bits 26-30 = run length - 1 (a run never exceeds one warp).
constexpr unsigned LINK_POS_BITS = 26u;
constexpr unsigned LINK_POS_MASK = (1u << LINK_POS_BITS) - 1u;

// ---- control block in device memory ------------------------------------------------------------
struct Ctl {
    unsigned long long episodes, goals, timeouts, conflicts, long_chains;
    unsigned long long eval_reached, eval_steps;
    unsigned long long general;     // environment-steps that went through the entry/chain path
    unsigned int eps_idx;           // index of the current step's epsilon in the table
    unsigned int eps_mode;          // 0 fixed index, 1 advance by one per step, 2 per-episode index
    unsigned int eps_len;           // table length (clamp)
    unsigned long long eps_base_k;  // per-episode mode: table[0] belongs to episodes/N == eps_base_k
    unsigned int active_count[2];   // mailbox slots holding a chain, per step parity
    unsigned int long_count[2];     // chains queued for the warp-per-chain kernel, per step parity
    unsigned int long2_count[2];    // chains too long for a warp, queued for the block-per-chain kernel
    unsigned int scratch_cursor;    // bump allocator of the long-chain scratch, reset every step
    unsigned int error;             // sticky internal error bits
    float eps_used;                 // epsilon of the most recent step (for the stats call)
};

enum : unsigned { ERR_SCRATCH_OVERFLOW = 1u, ERR_BAD_STATE = 2u, ERR_CHAIN_CYCLE = 8u, ERR_COPY_TIMEOUT = 32u };   // = CUDARL_DEVERR_* of cudarl.h

// ---- tile engine (tile_engine.cu): the layout the train step runs on ---------------------------
// The grid is cut into T x T tiles (T = 16 or 8); one WARP steps one tile at a time.  The table is a single
// dense array updated in place: a tile's cells are read and written by the tile's own warp only, and what
// a move across a tile edge needs from the neighbour -- max_a Q_t of the cell beyond the edge -- comes from a
// small double-buffered border array that every tile refreshes at the end of its step.
// Every tile owns a REGION of the record array that only the tile's own warp writes (environments that
// stay) and a fixed arrival buffer that other warps append to with an atomic cursor (environments that
// walk or restart into the tile).  Records, counters and border values alternate by step parity, so a step
// reads one set and writes the other.
constexpr unsigned ARR_CAP = 32u;  // arrival slots per tile and step; what does not fit goes to the spill list
struct TileP {
    unsigned tshift, T;        // tile edge = 1 << tshift cells
    unsigned tiles_x, tiles_y, ntiles;
    unsigned tiles_x_rcp;      // floor(2^32 / tiles_x): umulhi(n, tiles_x_rcp) is n / tiles_x or one less, for every n < 2^32
    unsigned grid;             // blocks of the persistent step kernel (SMs x resident blocks per SM)
    unsigned wait_polls;       // 0: copy waits are bounded by time (seconds); > 0 (tests only): a wait of this many polls before the copies are issued, which must run out
    uint2* rec[2];             // 8-byte records {id, t << 8 | row in tile << 4 | column in tile} of the environments that stayed; [step & 1] is current
    uint2* reg;                // ntiles + 1: {start of the tile's region, its capacity}
    uint2* cnt[2];             // ntiles: {records in the region, records in the arrival buffer}
    uint2* arr[2];             // ntiles x ARR_CAP arrival slots, same 8-byte records
    int4* ovf[2];              // records {x, y, t, id} that found their tile's arrival buffer full, any tile, N slots
    unsigned* tctl;            // [0..2] spill counts (read step%3, append (step+1)%3, clear (step+2)%3); [3..4] scratch cursors by parity
    unsigned char* tcls;       // ntiles x cls_stride: one move byte per cell, tile by tile (which of the four moves are blocked / end on a goal)
    unsigned cls_stride;
    float* bmax[2];            // ntiles x 4T: max_a Q of the cells just outside the tile's north / south / west / east edge; [step & 1] is current
    uint2* scratch;            // scratch_cap x 8 bytes: 32-bit (cell, action) counters of the tiles the general path counts in global memory
    unsigned scratch_cap;
    unsigned nq;               // tile queues of the step kernel: one per SM
    unsigned* tq;              // 3 x nq ticket counters: [step % 3] in use, [(step + 2) % 3] cleared
    CUtensorMap tmq;           // the table as a 2-D tensor of floats (4W x H), box 4T x T: one copy instruction per tile
};

// ---- everything a kernel needs, passed by value ------------------------------------------------
struct Params {
    int W, H;
    unsigned S;            // cells
    unsigned N;            // local environments
    unsigned env_offset;   // global index of local env 0
    unsigned k0, k1;       // Philox key base = seed (k1 is xor-ed with the stream tag)
    int max_steps;
    int start_mode;
    unsigned start_cell;   // CENTRE / FIXED start
    unsigned fallback_start;
    float lr, gamma;
    int legacy_clamp;
    float4* Q;             // the table: S float4, row s = the 4 action values of cell s; every kernel updates it in place
    unsigned short* cw;    // S cell words (padded to 16 bytes)
    const uint2* traps;    // sparse trap table, ascending by cell: {cell, penalty as float bits}
    unsigned ntraps;
    // environment state outside train steps: one int4 {x, y, t, id} per environment (all int32, one
    // coalesced 16-byte vector per thread), record k = environment k
    int4* st;
    int4* st2;             // scratch of the same size (export of x[N] | y[N] | t[N])
    float* reward; unsigned char* done;        // per ENVIRONMENT (caller-driven stepping only)
    uint4* ent;            // collision entries
    unsigned ent_cap;      // slots in ent
    unsigned* mailbox;     // update_batch: chain heads (0 = empty), power-of-two size
    unsigned mb_slots;     // mailbox slots (power of two, multiple of BLOCK)
    unsigned* active;      // list of the mailbox slots that hold a chain in this step (mb_slots entries)
    unsigned* longq;       // heads of the chains left to the warp-per-chain kernel (mb_slots entries)
    unsigned* longq2;      // heads of the chains left to the block-per-chain kernel (mb_slots entries)
    Ctl* ctl;
    const float* eps_tab;
    int* tr_a; float* tr_r; unsigned char* tr_d;   // optional trace of the last step, per ENVIRONMENT
    unsigned long long* sc_key; float* sc_val; unsigned sc_cap;   // long-chain scratch (global)
    // per-launch values set by the host
    unsigned long long step;   // global batched step index g (keys the policy stream, selects the counter plane)
    unsigned eps_idx;          // index of this step's epsilon in eps_tab
    int eps_from_ctl;          // 1: take the index from ctl (per-episode schedule)
    TileP tp;
};

constexpr int BLOCK = 256;

// launch wrappers (kernels.cu); all asynchronous on `st`
void launch_identity_ids(const Params& p, cudaStream_t st);
void launch_export_state(const Params& p, cudaStream_t st);       // st2 viewed as x[N]|y[N]|t[N] in environment order
void launch_import_state(const Params& p, const int* x, const int* y, const int* t, cudaStream_t st);
void launch_reset_all(const Params& p, cudaStream_t st);
void launch_step_actions(const Params& p, const int* d_actions, float* d_rewards, unsigned char* d_dones, cudaStream_t st);
void launch_eval(const Params& p, unsigned char* policy, int max_steps, unsigned long long nonce, cudaStream_t st);   // policy: one byte per cell, scratch
void launch_update_batch(const Params& p, unsigned n, const int* sx, const int* sy, const int* a, const float* r,
                         const int* nx, const int* ny, const unsigned char* dn, cudaStream_t st);
void launch_q_init(const Params& p, int kind, float scale, cudaStream_t st);
// tile engine (tile_engine.cu)
size_t tile_step_smem(const Params& p);
int  tile_engine_configure(Params& p, int device);                  // opt in to the dynamic shared memory the step needs; sets tp.grid
void launch_tile_bucket(const Params& p, cudaStream_t st);         // p.st (any slot order) -> tile regions of parity p.step & 1
void launch_tile_classes(const Params& p, cudaStream_t st);       // cell words -> per-tile class bytes (after any change of the grid)
void launch_tile_export(const Params& p, cudaStream_t st);         // tile regions -> p.st in environment order
void launch_tile_step(const Params& p, bool trace, cudaStream_t st);
unsigned tile_cls_stride(unsigned tshift);                         // bytes of one tile's class block
void launch_tile_border(const Params& p, cudaStream_t st);         // border array of parity p.step & 1 from the table (after any change of the table outside train steps)
// Replica averaging, the slice this rank owns: table[cell0 + i] = (sum over ranks 0..R-1 in that order) / R, where rank `self`'s
// rows are the table's own and the other ranks' rows lie in `others` (R - 1 slices of n rows, ascending rank).
void launch_q_average_peers(float4* const* tables, unsigned R, unsigned self, size_t cell0, size_t n, float scale, cudaStream_t st);
void launch_q_average_slice(float4* table, const float4* others, unsigned R, unsigned self, size_t cell0, size_t n, float scale, cudaStream_t st);
void launch_cell_set(const Params& p, unsigned cell, unsigned cls, int clear_goals, cudaStream_t st);

}  // namespace cudarl
