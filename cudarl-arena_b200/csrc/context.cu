// context.cu -- the C ABI of include/cudarl.h: one context per GPU owning the shard's device
// buffers, one stream, and (optionally) an NCCL communicator for replica averaging.
// Host logic only; every hot operation is a kernel of tile_engine.cu (the fused train step and its record
// bucketing) or kernels.cu (everything else).  There is no CPU fallback: a call either runs on the device or
// returns an error code.
#include "../../include/cudarl.h"
#include "kernels.cuh"
#include <nccl.h>
#include <dlfcn.h>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <string>
#include <vector>
#include <map>
#include <new>

using namespace cudarl;

namespace {

thread_local std::string g_err;

// ---- host Philox4x32-10 for the one-time grid construction ---------------------------------------
struct HW { uint32_t w[4]; };
HW philox(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
    uint32_t c[4] = {c0, c1, c2, c3};
    for (int r = 0; r < 10; ++r) {
        uint64_t a = 0xD2511F53ull * c[0], b = 0xCD9E8D57ull * c[2];
        uint32_t t0 = (uint32_t)(b >> 32) ^ c[1] ^ k0, t2 = (uint32_t)(a >> 32) ^ c[3] ^ k1;
        c[1] = (uint32_t)b; c[3] = (uint32_t)a; c[0] = t0; c[2] = t2;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return HW{{c[0], c[1], c[2], c[3]}};
}
constexpr uint32_t TG_GRID = 0x47524944u, TG_WALL = 0x57414C4Cu, TG_GOAL = 0x474F414Cu;
inline uint32_t hi32(uint32_t a, uint32_t b) { return (uint32_t)(((uint64_t)a * b) >> 32); }

// ---- NCCL through dlopen: the library loads (and single-GPU use works) without NCCL present ------
struct NcclApi {
    void* h = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;   // optional
    bool load(std::string& err) {
        if (h) return true;
        h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) { err = std::string("dlopen libnccl.so.2: ") + dlerror(); return false; }
        GetUniqueId = (decltype(GetUniqueId))dlsym(h, "ncclGetUniqueId");
        CommInitRank = (decltype(CommInitRank))dlsym(h, "ncclCommInitRank");
        CommDestroy = (decltype(CommDestroy))dlsym(h, "ncclCommDestroy");
        AllReduce = (decltype(AllReduce))dlsym(h, "ncclAllReduce");
        AllGather = (decltype(AllGather))dlsym(h, "ncclAllGather");
        Send = (decltype(Send))dlsym(h, "ncclSend"); Recv = (decltype(Recv))dlsym(h, "ncclRecv");
        GroupStart = (decltype(GroupStart))dlsym(h, "ncclGroupStart"); GroupEnd = (decltype(GroupEnd))dlsym(h, "ncclGroupEnd");
        GetErrorString = (decltype(GetErrorString))dlsym(h, "ncclGetErrorString");
        CommGetAsyncError = (decltype(CommGetAsyncError))dlsym(h, "ncclCommGetAsyncError");
        if (!GetUniqueId || !CommInitRank || !CommDestroy || !AllReduce || !AllGather || !Send || !Recv || !GroupStart || !GroupEnd) { err = "NCCL symbols missing"; h = nullptr; return false; }
        return true;
    }
};
NcclApi g_nccl;

__global__ void k_ctl_eps(Ctl* c, unsigned mode, unsigned len, unsigned long long base_k) {
    c->eps_idx = 0; c->eps_mode = mode; c->eps_len = len; c->eps_base_k = base_k;
}
__global__ void k_ctl_eval_clear(Ctl* c) { c->eval_reached = 0; c->eval_steps = 0; }

}  // namespace

struct cudarl_ctx {
    cudarl_config cfg{};
    Params p{};
    cudaStream_t st = nullptr;
    std::string err;
    std::vector<uint8_t> cells;           // host copy of the cell classes
    std::map<uint32_t, float> traps;      // cell -> penalty; mirrored on the device as a table sorted by cell
    void* dtraps = nullptr; size_t traps_cap = 0;
    void* dtq = nullptr;                    // ticket counters of the step kernel's tile queues
    void* dpolicy = nullptr;                // greedy policy map of the evaluation rollout (one byte per cell), allocated on first use
    // device buffers
    void *dci = nullptr, *dreward = nullptr, *ddone = nullptr;
    void *dstate[2] = {nullptr, nullptr};   // int4 {x,y,t,id} per environment, and a scratch copy of the same size
    void *dimport = nullptr;              // staging for caller state arrays (3 x N int32)
    void *dactive = nullptr;
    // tile engine (the layout the train step runs on)
    void *dQ = nullptr;                    // the table (padded so that it splits into equal slices for any number of ranks)
    void *drec[2] = {nullptr, nullptr}, *darr[2] = {nullptr, nullptr}, *dovf[2] = {nullptr, nullptr}, *dbmax[2] = {nullptr, nullptr};
    void *dtmeta = nullptr, *dtscratch = nullptr, *dtcls = nullptr;   // per-tile regions / counters; 32-bit counters of crowded tiles
    bool tile_mode = false;               // true: the records live in tile regions (train steps), false: in environment order
    bool cls_dirty = true;                // the per-tile class bytes must be rebuilt from the cell words
    int64_t bucket_every = 256, since_bucket = 0;
    void *dent = nullptr, *dctl = nullptr, *deps = nullptr;
    void *dtra = nullptr, *dtrr = nullptr, *dtrd = nullptr, *dsckey = nullptr, *dscval = nullptr;
    void *dgather = nullptr;              // replica averaging: the other ranks' rows of this rank's slice
    void* dub[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr}; size_t ub_cap = 0;   // update_batch staging
    void* dact = nullptr;                 // actions staging for the host form of step_actions
    size_t ent_cap = 0, eps_cap = 0;
    float* h_eps = nullptr; size_t h_eps_cap = 0; cudaEvent_t ev_eps = nullptr; bool eps_inflight = false;
    float eps_fixed_cached = -1.0f; bool eps_fixed_valid = false;
    // host mirror of schedule state
    int64_t h_step = 0;
    int64_t epoch_step = 0;                 // the step at which every environment last started an episode together (creation, reset_all)
    int eps_mode = 0;                     // 0 one fixed value, 1 table indexed by step of the call, 2 per-episode (device index)
    float eps_used = 0.0f;
    double eps_running = 1.0;
    int64_t eval_calls = 0;
    bool trace = false;
    // communicator
    ncclComm_t comm = nullptr; int rank = 0, nranks = 1;
    // replica averaging over peer memory: every rank's table mapped into this process (CUDA IPC), pointers in rank order
    bool peer_ok = false;
    std::vector<void*> peer_tables;         // [nranks]; this rank's own entry is its table
    void* dpeer_ptrs = nullptr;             // the same pointers on the device
    void* dbarrier_word = nullptr;          // one int for the all-reduce that serves as a barrier
    // timing
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    // kernel timing: one event pair around every uninterrupted run of step-kernel launches
    bool ktiming = false, kseg_open = false; std::vector<cudaEvent_t> kev; size_t kev_used = 0;
    std::vector<int64_t> kseg_launches; int64_t kseg_count = 0;
    double main_ms = 0; int64_t klaunches = 0;
};

namespace {

int fail(cudarl_ctx* c, int code, const std::string& m) { if (c) c->err = m; g_err = m; return code; }
#define CK(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return fail(c, 1000 + (int)e_, std::string(#call) + ": " + cudaGetErrorString(e_)); } while (0)
#define NK(call) do { ncclResult_t r_ = (call); if (r_ != ncclSuccess) return fail(c, 2000 + (int)r_, std::string(#call) + ": " + (g_nccl.GetErrorString ? g_nccl.GetErrorString(r_) : "nccl error")); } while (0)

size_t pow2ceil(size_t v) { size_t r = 1; while (r < v) r <<= 1; return r; }

// Build the cell classes (0 free, 1 obstacle, 2 goal) from the config.
int build_cells(cudarl_ctx* c, std::vector<uint8_t>& cells, uint32_t& start_cell, uint32_t& fallback) {
    const cudarl_config& f = c->cfg;
    const int W = f.width, H = f.height; const uint32_t S = (uint32_t)W * (uint32_t)H;
    const uint32_t k0 = (uint32_t)f.seed, k1 = (uint32_t)(f.seed >> 32);
    cells.assign(S, 0);
    if (f.obstacle_kind == CUDARL_OBST_BERNOULLI) {
        double t = (double)f.obstacle_p * 4294967296.0;
        uint32_t thr = t <= 0.0 ? 0u : (t >= 4294967295.0 ? 0xFFFFFFFFu : (uint32_t)t);
        for (uint32_t q = 0; q * 4u < S; ++q) {
            HW r = philox(q, 0, 0, 0, k0, k1 ^ TG_GRID);
            for (uint32_t j = 0; j < 4 && q * 4u + j < S; ++j) cells[q * 4u + j] = r.w[j] < thr ? 1 : 0;
        }
    } else if (f.obstacle_kind == CUDARL_OBST_WALLS) {
        const int64_t want = (int64_t)std::floor((double)f.obstacle_p * (double)S);
        int64_t have = 0;
        for (uint32_t k = 0; have < want && k < 0x7fffffffu; ++k) {
            HW r = philox(k, 0, 0, 0, k0, k1 ^ TG_WALL);
            uint32_t o = hi32(r.w[0], S);
            int ox = (int)(o % (uint32_t)W), oy = (int)(o / (uint32_t)W);
            const bool horizontal = r.w[1] & 1u; const int len = 1 + (int)(r.w[2] & 31u);
            for (int j = 0; j < len; ++j) {
                int px = ox + (horizontal ? j : 0), py = oy + (horizontal ? 0 : j);
                if (px >= W || py >= H) break;
                uint8_t& cell = cells[(size_t)py * W + px];
                if (!cell) { cell = 1; ++have; }
            }
        }
    } else if (f.obstacle_kind != CUDARL_OBST_NONE) return fail(c, -1, "bad obstacle_kind");

    int64_t fixed = -1;
    if (f.start_mode == CUDARL_START_CENTRE) fixed = (int64_t)(H / 2) * W + W / 2;
    else if (f.start_mode == CUDARL_START_FIXED) {
        if (f.start_x < 0 || f.start_x >= W || f.start_y < 0 || f.start_y >= H) return fail(c, -1, "start cell out of range");
        fixed = (int64_t)f.start_y * W + f.start_x;
    } else if (f.start_mode != CUDARL_START_RANDOM) return fail(c, -1, "bad start_mode");
    if (fixed >= 0) cells[fixed] = 0;
    start_cell = fixed >= 0 ? (uint32_t)fixed : 0u;

    if (f.goal_mode == CUDARL_GOAL_TOP_RIGHT) cells[W - 1] = 2;
    else if (f.goal_mode == CUDARL_GOAL_LIST || f.goal_mode == CUDARL_GOAL_SEEDED) {
        if (f.num_goals < 1 || f.num_goals > CUDARL_MAX_GOALS) return fail(c, -1, "num_goals out of range");
        for (int g = 0; g < f.num_goals; ++g) {
            if (f.goal_mode == CUDARL_GOAL_LIST) {
                int gx = f.goal_xy[2 * g], gy = f.goal_xy[2 * g + 1];
                if (gx < 0 || gx >= W || gy < 0 || gy >= H) return fail(c, -1, "goal cell out of range");
                cells[(size_t)gy * W + gx] = 2;
            } else {
                uint32_t attempt = 0; bool ok = false;
                for (; attempt < (1u << 20); ++attempt) {
                    uint32_t cand = hi32(philox((uint32_t)g, attempt, 0, 0, k0, k1 ^ TG_GOAL).w[0], S);
                    if (cells[cand] == 0 && (int64_t)cand != fixed) { cells[cand] = 2; ok = true; break; }
                }
                if (!ok) return fail(c, -1, "could not place a seeded goal");
            }
        }
    } else return fail(c, -1, "bad goal_mode");

    fallback = 0xFFFFFFFFu;
    for (uint32_t s = 0; s < S; ++s) if (cells[s] == 0) { fallback = s; break; }
    if (f.start_mode == CUDARL_START_RANDOM && fallback == 0xFFFFFFFFu) return fail(c, -1, "no free cell");
    if (fallback == 0xFFFFFFFFu) fallback = start_cell;
    return 0;
}

int upload_cells(cudarl_ctx* c) {
    const size_t S = c->p.S, pad = (S + 7) / 8 * 8;
    std::vector<uint16_t> b(pad, 0);
    for (size_t s = 0; s < S; ++s) b[s] = c->cells[s] == 1 ? CW_OBST : (c->cells[s] == 2 ? CW_GOAL : 0);
    CK(cudaMemcpyAsync(c->dci, b.data(), pad * 2, cudaMemcpyHostToDevice, c->st));
    CK(cudaStreamSynchronize(c->st));
    return 0;
}

// (Re)allocate the collision entry array and the long-chain scratch for `cap` entries.
int ensure_entry_capacity(cudarl_ctx* c, size_t cap) {
    if (cap <= c->ent_cap) return 0;
    CK(cudaStreamSynchronize(c->st));
    cudaFree(c->dent); cudaFree(c->dsckey); cudaFree(c->dscval);
    c->dent = c->dsckey = c->dscval = nullptr; c->ent_cap = 0;
    size_t sc = 2 * pow2ceil(cap); if (sc < 4096) sc = 4096;
    CK(cudaMalloc(&c->dent, cap * sizeof(uint4)));
    CK(cudaMalloc(&c->dsckey, sc * sizeof(unsigned long long)));
    CK(cudaMalloc(&c->dscval, sc * sizeof(float)));
    c->p.ent = (uint4*)c->dent;
    c->p.sc_key = (unsigned long long*)c->dsckey; c->p.sc_val = (float*)c->dscval; c->p.sc_cap = (unsigned)sc;
    c->ent_cap = cap; c->p.ent_cap = (unsigned)cap;
    return 0;
}

// The per-cell class words, and the chain heads / work lists of update_batch.
int alloc_hot(cudarl_ctx* c) {
    const size_t S = c->p.S, N = c->p.N ? c->p.N : 1;
    const size_t ci_bytes = (2 * S + 255) / 256 * 256;      // one 16-bit word per cell
    size_t slots = pow2ceil(N) / 2; if (slots < (1u << 16)) slots = 1u << 16; if (slots > (1u << 24)) slots = 1u << 24;
    const size_t total = ci_bytes + slots * sizeof(unsigned);
    CK(cudaMalloc(&c->dci, total));
    CK(cudaMemsetAsync(c->dci, 0, total, c->st));
    c->p.cw = (unsigned short*)c->dci;
    c->p.mailbox = (unsigned*)((char*)c->dci + ci_bytes); c->p.mb_slots = (unsigned)slots;
    CK(cudaMalloc(&c->dactive, 3 * slots * sizeof(unsigned)));
    c->p.active = (unsigned*)c->dactive; c->p.longq = (unsigned*)c->dactive + slots; c->p.longq2 = (unsigned*)c->dactive + 2 * slots;
    return 0;
}

int ensure_step_buffers(cudarl_ctx* c) {
    if (c->dreward) return 0;
    size_t N = c->p.N ? c->p.N : 1;
    CK(cudaMalloc(&c->dreward, N * sizeof(float)));
    CK(cudaMalloc(&c->ddone, N));
    CK(cudaMalloc(&c->dact, N * sizeof(int)));
    CK(cudaMemsetAsync(c->dreward, 0, N * sizeof(float), c->st));
    CK(cudaMemsetAsync(c->ddone, 0, N, c->st));
    c->p.reward = (float*)c->dreward; c->p.done = (unsigned char*)c->ddone;
    return 0;
}

// Stage `n` epsilons (host array) into the device table.
int upload_eps(cudarl_ctx* c, const float* eps, size_t n) {
    if (c->eps_inflight) { CK(cudaEventSynchronize(c->ev_eps)); c->eps_inflight = false; }
    if (n > c->h_eps_cap) {
        if (c->h_eps) cudaFreeHost(c->h_eps);
        c->h_eps = nullptr; c->h_eps_cap = 0;
        size_t cap = pow2ceil(n < 256 ? 256 : n);
        CK(cudaMallocHost((void**)&c->h_eps, cap * sizeof(float)));
        c->h_eps_cap = cap;
    }
    if (n > c->eps_cap) {
        CK(cudaStreamSynchronize(c->st));
        cudaFree(c->deps); c->deps = nullptr; c->eps_cap = 0;
        size_t cap = pow2ceil(n < 256 ? 256 : n);
        CK(cudaMalloc(&c->deps, cap * sizeof(float)));
        c->eps_cap = cap; c->p.eps_tab = (const float*)c->deps;
    }
    std::memcpy(c->h_eps, eps, n * sizeof(float));
    CK(cudaMemcpyAsync(c->deps, c->h_eps, n * sizeof(float), cudaMemcpyHostToDevice, c->st));
    CK(cudaEventRecord(c->ev_eps, c->st));
    c->eps_inflight = true; c->eps_fixed_valid = false;
    return 0;
}

// Close the open run of step-kernel launches (an event after its last launch).
int close_kernel_segment(cudarl_ctx* c) {
    if (!c->kseg_open) return 0;
    CK(cudaEventRecord(c->kev[c->kev_used + 1], c->st));
    c->kev_used += 2; c->kseg_launches.push_back(c->kseg_count);
    c->kseg_open = false; c->kseg_count = 0;
    return 0;
}
int drain_kernel_events(cudarl_ctx* c) {
    { int rc = close_kernel_segment(c); if (rc) return rc; }
    if (!c->kev_used) return 0;
    CK(cudaStreamSynchronize(c->st));
    for (size_t k = 0; k + 1 < c->kev_used; k += 2) {
        float a = 0;
        CK(cudaEventElapsedTime(&a, c->kev[k], c->kev[k + 1]));
        c->main_ms += a; c->klaunches += c->kseg_launches[k / 2];
    }
    c->kev_used = 0; c->kseg_launches.clear();
    return 0;
}

// After a synchronisation: has any kernel recorded an internal failure (a copy that never landed, a full
// scratch area, a record outside its tile)?  The word is sticky; the results of the context are not to be trusted.
int check_device_error(cudarl_ctx* c) {
    unsigned err = 0;
    CK(cudaMemcpyAsync(&err, (const char*)c->dctl + offsetof(Ctl, error), sizeof(err), cudaMemcpyDeviceToHost, c->st));
    CK(cudaStreamSynchronize(c->st));
    if (err) return fail(c, CUDARL_ERR_DEVICE + (int)err, "device error bits " + std::to_string(err) +
                         ((err & ERR_COPY_TIMEOUT) ? " (a tile copy did not land within its wait bound)" : "") +
                         ((err & ERR_SCRATCH_OVERFLOW) ? " (scratch area full)" : "") + ((err & ERR_BAD_STATE) ? " (a record outside its tile or the grid)" : "") +
                         ((err & ERR_CHAIN_CYCLE) ? " (update_batch chain longer than the batch)" : ""));
    if (c->comm && g_nccl.CommGetAsyncError) {               // a collective that failed after it was enqueued (a peer that went away)
        ncclResult_t ar = ncclSuccess;
        const ncclResult_t qr = g_nccl.CommGetAsyncError(c->comm, &ar);
        if (qr == ncclSuccess && ar != ncclSuccess && ar != ncclInProgress)
            return fail(c, 2000 + (int)ar, std::string("replica averaging failed asynchronously: ") + (g_nccl.GetErrorString ? g_nccl.GetErrorString(ar) : "nccl error"));
    }
    return 0;
}

// ---- tile engine: buffers, entering and leaving the tile layout ------------------------------------
// The table as a 2-D tensor of floats, 4W wide and H high, fetched in boxes of one tile (4T x T floats).
int make_table_map(cudarl_ctx* c) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* f = nullptr; cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !f) return fail(c, -5, "cuTensorMapEncodeTiled is not available in this driver");
        encode = (EncodeFn)f;
    }
    const Params& p = c->p;
    const cuuint64_t dims[2] = {(cuuint64_t)p.W * 4u, (cuuint64_t)p.H};
    const cuuint64_t strides[1] = {(cuuint64_t)p.W * 16u};                 // bytes between table rows: a multiple of 16
    const cuuint32_t box[2] = {4u * p.tp.T, p.tp.T}, estr[2] = {1u, 1u};
    const CUresult r = encode(&c->p.tp.tmq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, p.Q, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, p.tp.T >= 16u ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(c, -5, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return 0;
}

// Tile edge: 16 cells while a 16 x 16 tile holds few enough environments for most tiles to stay on the step kernel's fast
// path (at most 128 staged records), else 8.  Measured on B200, 4096 x 4096 cells, us per step with edge 16 / edge 8:
// 64 per tile 124 / 250, 96 per tile 182 / 271, 128 per tile 731 / 323 -- the crossover lies near 110.
int alloc_tiles(cudarl_ctx* c) {
    Params& p = c->p; TileP& tp = p.tp;
    const size_t S = p.S, N = p.N ? p.N : 1;
    CK(cudaMalloc(&c->dQ, (S + 64) * sizeof(float4)));
    CK(cudaMemsetAsync(c->dQ, 0, (S + 64) * sizeof(float4), c->st));
    p.Q = (float4*)c->dQ;
    const size_t nt16 = (((size_t)p.W + 15) >> 4) * (((size_t)p.H + 15) >> 4);
    unsigned tsh = (N / nt16 <= 104) ? 4u : 3u;
    if (c->cfg.tile_edge == 8) tsh = 3u; else if (c->cfg.tile_edge == 16) tsh = 4u;
    tp.tshift = tsh; tp.T = 1u << tsh;
    tp.tiles_x = (unsigned)((p.W + (int)tp.T - 1) >> tsh); tp.tiles_y = (unsigned)((p.H + (int)tp.T - 1) >> tsh);
    tp.ntiles = tp.tiles_x * tp.tiles_y;
    tp.tiles_x_rcp = tp.tiles_x > 1u ? (unsigned)((1ull << 32) / tp.tiles_x) : 0xFFFFFFFFu;
    const size_t nt = tp.ntiles;
    for (int k = 0; k < 2; ++k) {
        CK(cudaMalloc(&c->drec[k], (N + N / 4 + 34 * nt + 64) * sizeof(uint2)));
        CK(cudaMalloc(&c->darr[k], nt * ARR_CAP * sizeof(uint2)));
        CK(cudaMalloc(&c->dovf[k], N * sizeof(int4)));
        CK(cudaMalloc(&c->dbmax[k], nt * 4 * tp.T * sizeof(float)));
        CK(cudaMemsetAsync(c->dbmax[k], 0, nt * 4 * tp.T * sizeof(float), c->st));
        tp.rec[k] = (uint2*)c->drec[k]; tp.arr[k] = (uint2*)c->darr[k]; tp.ovf[k] = (int4*)c->dovf[k]; tp.bmax[k] = (float*)c->dbmax[k];
    }
    const size_t meta = 2 * (nt + 1) + 4 * nt + 8;          // reg (uint2 x (nt+1)), cnt[2] (uint2 x nt each), tctl
    CK(cudaMalloc(&c->dtmeta, meta * sizeof(unsigned)));
    CK(cudaMemsetAsync(c->dtmeta, 0, meta * sizeof(unsigned), c->st));
    unsigned* m = (unsigned*)c->dtmeta;
    tp.reg = (uint2*)m; m += 2 * (nt + 1);
    tp.cnt[0] = (uint2*)m; m += 2 * nt; tp.cnt[1] = (uint2*)m; m += 2 * nt;
    tp.tctl = m;
    tp.cls_stride = tile_cls_stride(tsh);
    CK(cudaMalloc(&c->dtcls, nt * tp.cls_stride));
    tp.tcls = (unsigned char*)c->dtcls;
    // 16 bytes per cell of every tile that counts in global memory: on 16 x 16 tiles that is every tile the general path takes
    // (in the worst case -- a step with a spill list -- all of them), on 8 x 8 tiles only tiles with more than 65,535 records
    size_t scratch_cap = N > 65536 ? N : 65536;
    if (tsh >= 4 && nt * tp.T * tp.T * 2 > scratch_cap) scratch_cap = nt * tp.T * tp.T * 2;
    CK(cudaMalloc(&c->dtscratch, scratch_cap * sizeof(uint2)));
    tp.scratch = (uint2*)c->dtscratch; tp.scratch_cap = (unsigned)scratch_cap;
    tp.wait_polls = 0;
    { int sms = 0; CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->cfg.device)); tp.nq = (unsigned)(sms > 0 ? sms : 1); }
    CK(cudaMalloc(&c->dtq, 3 * (size_t)tp.nq * sizeof(unsigned)));
    CK(cudaMemsetAsync(c->dtq, 0, 3 * (size_t)tp.nq * sizeof(unsigned), c->st));
    tp.tq = (unsigned*)c->dtq;
    { int rm = make_table_map(c); if (rm) return rm; }
    if (tile_engine_configure(p, c->cfg.device) != 0) { cudaGetLastError(); return fail(c, -5, "tile step: shared memory request refused"); }
    return 0;
}

// records in environment order -> tile regions; border values from the table as it is now
int enter_tiles(cudarl_ctx* c) {
    if (c->tile_mode) return 0;
    c->p.step = (unsigned long long)c->h_step;
    if (c->cls_dirty) { launch_tile_classes(c->p, c->st); c->cls_dirty = false; }
    launch_tile_bucket(c->p, c->st);
    launch_tile_border(c->p, c->st);
    CK(cudaGetLastError());
    c->tile_mode = true; c->since_bucket = 0;
    return 0;
}
// tile regions -> records back in environment order
int leave_tiles(cudarl_ctx* c) {
    if (!c->tile_mode) return 0;
    { int rc = close_kernel_segment(c); if (rc) return rc; }
    c->p.step = (unsigned long long)c->h_step;
    launch_tile_export(c->p, c->st);
    CK(cudaGetLastError());
    c->tile_mode = false;
    return 0;
}
// re-size the tile regions from the current populations
int rebucket_tiles(cudarl_ctx* c) {
    { int rc = close_kernel_segment(c); if (rc) return rc; }
    c->p.step = (unsigned long long)c->h_step;
    launch_tile_export(c->p, c->st);
    launch_tile_bucket(c->p, c->st);
    CK(cudaGetLastError());
    c->since_bucket = 0;
    return 0;
}

// Map every rank's table into this process: the CUDA IPC handles travel by an NCCL all-gather, each peer's handle is opened
// (one process per GPU: a handle cannot be opened by the process that made it), and the ranks agree by an all-reduce whether
// ALL of them succeeded -- only then is the peer-memory averaging used; otherwise every rank keeps the NCCL send / receive path.
int map_peer_tables(cudarl_ctx* c) {
    const int R = c->nranks, self = c->rank;
    c->peer_ok = false;
    std::vector<cudaIpcMemHandle_t> hs((size_t)R);
    int ok = cudaIpcGetMemHandle(&hs[(size_t)self], c->dQ) == cudaSuccess ? 1 : 0;
    cudaGetLastError();
    void* dh = nullptr; int* dflag = nullptr;
    CK(cudaMalloc(&dh, (size_t)R * sizeof(cudaIpcMemHandle_t)));
    CK(cudaMalloc(&c->dbarrier_word, sizeof(int)));
    dflag = (int*)c->dbarrier_word;
    CK(cudaMemcpyAsync((char*)dh + (size_t)self * sizeof(cudaIpcMemHandle_t), &hs[(size_t)self], sizeof(cudaIpcMemHandle_t), cudaMemcpyHostToDevice, c->st));
    NK(g_nccl.AllGather((char*)dh + (size_t)self * sizeof(cudaIpcMemHandle_t), dh, sizeof(cudaIpcMemHandle_t), ncclChar, c->comm, c->st));
    CK(cudaMemcpyAsync(hs.data(), dh, (size_t)R * sizeof(cudaIpcMemHandle_t), cudaMemcpyDeviceToHost, c->st));
    CK(cudaStreamSynchronize(c->st));
    CK(cudaFree(dh));
    c->peer_tables.assign((size_t)R, nullptr);
    c->peer_tables[(size_t)self] = c->dQ;
    for (int r = 0; r < R && ok; ++r) {
        if (r == self) continue;
        if (cudaIpcOpenMemHandle(&c->peer_tables[(size_t)r], hs[(size_t)r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { ok = 0; c->peer_tables[(size_t)r] = nullptr; }
    }
    cudaGetLastError();
    // all or none
    CK(cudaMemcpyAsync(dflag, &ok, sizeof(int), cudaMemcpyHostToDevice, c->st));
    NK(g_nccl.AllReduce(dflag, dflag, 1, ncclInt, ncclMin, c->comm, c->st));
    int all_ok = 0;
    CK(cudaMemcpyAsync(&all_ok, dflag, sizeof(int), cudaMemcpyDeviceToHost, c->st));
    CK(cudaStreamSynchronize(c->st));
    CK(cudaMemsetAsync(dflag, 0, sizeof(int), c->st));          // from here on the word only carries the barrier all-reduce
    if (all_ok) {
        CK(cudaMalloc(&c->dpeer_ptrs, (size_t)R * sizeof(void*)));
        CK(cudaMemcpyAsync(c->dpeer_ptrs, c->peer_tables.data(), (size_t)R * sizeof(void*), cudaMemcpyHostToDevice, c->st));
        CK(cudaStreamSynchronize(c->st));
        c->peer_ok = true;
    } else {
        for (int r = 0; r < R; ++r) if (r != self && c->peer_tables[(size_t)r]) { cudaIpcCloseMemHandle(c->peer_tables[(size_t)r]); c->peer_tables[(size_t)r] = nullptr; }
    }
    return 0;
}

// Q <- (Q_0 + Q_1 + ... + Q_{R-1}) * (1/R), summed in rank order on every GPU, shaped like an all-reduce: the table
// is cut into R equal slices, rank j owns slice j.  (1) every rank sends its rows of slice j to rank j (grouped NCCL
// send / receive over NVLink / NVSwitch); (2) rank j sums the R versions of its slice in rank order 0..R-1 in our own
// kernel, scale fused, into its table; (3) an in-place all-gather hands the averaged slices round.  Each GPU receives
// 2 (R-1)/R of the table per averaging, and because the summation order is ours, not the library's, every rank ends
// up with the same bits as the CPU oracle for any R.
int average_now(cudarl_ctx* c) {
    if (!c->comm || c->nranks <= 1) return 0;
    { int rc = close_kernel_segment(c); if (rc) return rc; }
    const size_t S = c->p.S, R = (size_t)c->nranks, self = (size_t)c->rank;
    const size_t slice = (S + R - 1) / R;                      // cells; R * slice <= S + 64 = the padded table
    if (R > 64) return fail(c, -1, "replica averaging supports at most 64 ranks");
    if (c->peer_ok) {
        // Exchange, ordered sum and hand-round fused in one kernel over NVLink: when every rank has finished its steps (the
        // one-word all-reduce is the barrier), rank j reads slice j of every replica straight out of its peers' memory (plain
        // loads, no staging copy), sums in rank order, scales, and writes the result into slice j of EVERY rank's table (plain
        // stores).  Slice j of any table is read and written by rank j alone, so the kernels of different ranks never meet; the
        // second barrier tells a rank that all the others have delivered their slices into its table.
        NK(g_nccl.AllReduce(c->dbarrier_word, c->dbarrier_word, 1, ncclInt, ncclSum, c->comm, c->st));
        launch_q_average_peers((float4* const*)c->dpeer_ptrs, (unsigned)R, (unsigned)self, self * slice, slice, 1.0f / (float)R, c->st);
        NK(g_nccl.AllReduce(c->dbarrier_word, c->dbarrier_word, 1, ncclInt, ncclSum, c->comm, c->st));
        if (c->tile_mode) { c->p.step = (unsigned long long)c->h_step; launch_tile_border(c->p, c->st); }
        CK(cudaGetLastError());
        return 0;
    }
    if (!c->dgather) CK(cudaMalloc(&c->dgather, (R - 1) * slice * sizeof(float4)));
    float4* table = c->p.Q; float4* others = (float4*)c->dgather;
    NK(g_nccl.GroupStart());
    for (size_t r = 0; r < R; ++r) {
        if (r == self) continue;
        NK(g_nccl.Send(table + r * slice, slice * 4, ncclFloat, (int)r, c->comm, c->st));
        NK(g_nccl.Recv(others + (r - (r > self ? 1 : 0)) * slice, slice * 4, ncclFloat, (int)r, c->comm, c->st));
    }
    NK(g_nccl.GroupEnd());
    launch_q_average_slice(table, others, (unsigned)R, (unsigned)self, self * slice, slice, 1.0f / (float)R, c->st);
    NK(g_nccl.AllGather(table + self * slice, table, slice * 4, ncclFloat, c->comm, c->st));
    if (c->tile_mode) { c->p.step = (unsigned long long)c->h_step; launch_tile_border(c->p, c->st); }
    CK(cudaGetLastError());
    return 0;
}

int run_steps(cudarl_ctx* c, int64_t n) {
    { int re = enter_tiles(c); if (re) return re; }
    for (int64_t k = 0; k < n; ++k) {
        if (c->bucket_every > 0 && c->since_bucket >= c->bucket_every) { int rs = rebucket_tiles(c); if (rs) return rs; }
        // Environments that started together and never reached a goal hit the step cap together: the step before this one sent
        // them all to fresh start cells, far more arrivals than the tiles' arrival buffers hold, and the rest sits in the spill
        // list that every tile would have to filter.  Re-bucketing now puts them into regions instead (same results either way).
        if (c->bucket_every > 0 && c->cfg.max_steps > 0 && c->since_bucket > 0 && c->h_step > c->epoch_step &&
            (c->h_step - c->epoch_step) % c->cfg.max_steps == 0) { int rs = rebucket_tiles(c); if (rs) return rs; }
        if (c->ktiming && !c->kseg_open) {
            if (c->kev_used + 2 > c->kev.size()) { int rc = drain_kernel_events(c); if (rc) return rc; }
            CK(cudaEventRecord(c->kev[c->kev_used], c->st));
            c->kseg_open = true; c->kseg_count = 0;
        }
        c->p.step = (unsigned long long)c->h_step;
        c->p.eps_idx = c->eps_mode == 1 ? (unsigned)k : 0u;
        c->p.eps_from_ctl = c->eps_mode == 2 ? 1 : 0;
        if (c->eps_mode != 2 && c->h_eps) c->eps_used = c->h_eps[c->p.eps_idx];
        launch_tile_step(c->p, c->trace, c->st);
        c->h_step += 1; c->since_bucket += 1; c->kseg_count += 1;
        if (c->cfg.sync_every > 0 && c->comm && (c->h_step % c->cfg.sync_every) == 0) { int rc = average_now(c); if (rc) return rc; }
    }
    { int rc = close_kernel_segment(c); if (rc) return rc; }
    CK(cudaGetLastError());
    return 0;
}

void free_all(cudarl_ctx* c) {
    if (c->st) cudaStreamSynchronize(c->st);
    for (size_t r = 0; r < c->peer_tables.size(); ++r) if ((int)r != c->rank && c->peer_tables[r]) cudaIpcCloseMemHandle(c->peer_tables[r]);
    if (c->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(c->comm);
    void* bufs[] = {c->dci, c->dstate[0], c->dstate[1], c->dimport, c->dactive, c->dreward, c->ddone, c->dent, c->dctl, c->deps,
                    c->dtra, c->dtrr, c->dtrd, c->dsckey, c->dscval, c->dgather, c->dact,
                    c->dub[0], c->dub[1], c->dub[2], c->dub[3], c->dub[4], c->dub[5], c->dub[6],
                    c->dQ, c->drec[0], c->drec[1], c->darr[0], c->darr[1], c->dovf[0], c->dovf[1], c->dbmax[0], c->dbmax[1],
                    c->dtmeta, c->dtscratch, c->dtcls, c->dtraps, c->dpolicy, c->dtq, c->dpeer_ptrs, c->dbarrier_word};
    for (void* b : bufs) if (b) cudaFree(b);
    if (c->h_eps) cudaFreeHost(c->h_eps);
    for (auto e : c->kev) cudaEventDestroy(e);
    if (c->ev_eps) cudaEventDestroy(c->ev_eps);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    if (c->st) cudaStreamDestroy(c->st);
}

}  // namespace

// =================================================================================================
extern "C" {

const char* cudarl_version(void) { return "0.1.0"; }
const char* cudarl_last_global_error(void) { return g_err.c_str(); }
const char* cudarl_last_error(const cudarl_ctx* c) { return c ? c->err.c_str() : g_err.c_str(); }

void cudarl_default_config(cudarl_config* f) {
    std::memset(f, 0, sizeof(*f));
    f->struct_size = (uint32_t)sizeof(*f);
    f->width = 10; f->height = 10; f->num_envs = 1;
    f->goal_mode = CUDARL_GOAL_TOP_RIGHT; f->start_mode = CUDARL_START_CENTRE;
    f->lr = 0.1f; f->gamma = 0.99f;
    f->eps_kind = CUDARL_EPS_MULT_PER_STEP; f->eps0 = 1.0; f->eps_decay = 0.995; f->eps_end = 0.0;
    f->q_init_kind = CUDARL_QINIT_ZERO; f->q_init_scale = 0.01f;
}

int cudarl_create(const cudarl_config* f, cudarl_ctx** out) {
    if (!f || !out) return fail(nullptr, -1, "null argument");
    *out = nullptr;
    if (f->struct_size != sizeof(cudarl_config)) return fail(nullptr, -1, "cudarl_config.struct_size mismatch");
    if (f->width < 1 || f->height < 1) return fail(nullptr, -1, "grid must be at least 1x1");
    if ((uint64_t)f->width * (uint64_t)f->height >= (1ull << 28)) return fail(nullptr, -1, "grid larger than 2^28 cells");
    if (f->num_envs < 0 || f->num_envs >= (1ll << 26)) return fail(nullptr, -1, "num_envs out of range (at most 2^26 - 1 per context)");
    if (f->env_offset < 0 || f->env_offset + f->num_envs >= (1ll << 32)) return fail(nullptr, -1, "env_offset out of range");
    if (f->max_steps < 0) return fail(nullptr, -1, "max_steps negative");
    if (f->max_steps > 0xFFFFFE) return fail(nullptr, -1, "max_steps above 16,777,214 (the records keep 24 bits of an episode's step count; 0 = no cap)");
    if (f->eps_kind < 0 || f->eps_kind > 3) return fail(nullptr, -1, "bad eps_kind");
    if (f->tile_edge != 0 && f->tile_edge != 8 && f->tile_edge != 16) return fail(nullptr, -1, "tile_edge must be 0 (automatic), 8 or 16");
    cudarl_ctx* c = new (std::nothrow) cudarl_ctx();
    if (!c) return fail(nullptr, -1, "out of host memory");
    c->cfg = *f;
    int rc = 0;
    do {
        cudaError_t e = cudaSetDevice(f->device);
        if (e != cudaSuccess) { rc = fail(c, 1000 + (int)e, std::string("cudaSetDevice: ") + cudaGetErrorString(e)); break; }
        Params& p = c->p;
        p.W = f->width; p.H = f->height; p.S = (unsigned)(f->width * f->height); p.N = (unsigned)f->num_envs;
        p.env_offset = (unsigned)f->env_offset; p.k0 = (uint32_t)f->seed; p.k1 = (uint32_t)(f->seed >> 32);
        p.max_steps = f->max_steps; p.start_mode = f->start_mode; p.lr = f->lr; p.gamma = f->gamma; p.legacy_clamp = f->legacy_clamp;
        uint32_t sc = 0, fb = 0;
        rc = build_cells(c, c->cells, sc, fb); if (rc) break;
        p.start_cell = sc; p.fallback_start = fb;
        auto body = [&]() -> int {
            CK(cudaStreamCreateWithFlags(&c->st, cudaStreamNonBlocking));
            CK(cudaEventCreateWithFlags(&c->ev_eps, cudaEventDisableTiming));
            CK(cudaEventCreate(&c->ev0)); CK(cudaEventCreate(&c->ev1));
            const size_t N = p.N ? p.N : 1;
            { int r0 = alloc_hot(c); if (r0) return r0; }
            for (int cp = 0; cp < 2; ++cp) { CK(cudaMalloc(&c->dstate[cp], N * 16)); CK(cudaMemsetAsync(c->dstate[cp], 0, N * 16, c->st)); }
            CK(cudaMalloc(&c->dctl, sizeof(Ctl)));
            CK(cudaMemsetAsync(c->dctl, 0, sizeof(Ctl), c->st));
            p.st = (int4*)c->dstate[0]; p.st2 = (int4*)c->dstate[1];
            p.ctl = (Ctl*)c->dctl;
            int r2 = ensure_entry_capacity(c, N); if (r2) return r2;
            r2 = alloc_tiles(c); if (r2) return r2;
            r2 = upload_cells(c); if (r2) return r2;
            launch_q_init(p, f->q_init_kind, f->q_init_scale, c->st);
            float e0 = (float)f->eps0; r2 = upload_eps(c, &e0, 1); if (r2) return r2;
            k_ctl_eps<<<1, 1, 0, c->st>>>(p.ctl, 0u, 1u, 0ull);
            launch_identity_ids(p, c->st);
            launch_reset_all(p, c->st);
            CK(cudaGetLastError());
            CK(cudaStreamSynchronize(c->st));
            return 0;
        };
        c->bucket_every = f->rebucket_every > 0 ? f->rebucket_every : (f->rebucket_every < 0 ? 0 : 256);
        rc = body();
    } while (0);
    if (rc) { g_err = c->err; free_all(c); delete c; return rc; }
    c->eps_running = (double)f->eps0;
    *out = c;
    return 0;
}

void cudarl_destroy(cudarl_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->cfg.device);
    free_all(c);
    delete c;
}

int cudarl_get_config(const cudarl_ctx* c, cudarl_config* out) { if (!c || !out) return -1; *out = c->cfg; return 0; }

int cudarl_synchronize(cudarl_ctx* c) {
    if (!c) return -1;
    CK(cudaSetDevice(c->cfg.device));
    CK(cudaStreamSynchronize(c->st));
    return check_device_error(c);
}
int cudarl_debug_set_copy_wait_polls(cudarl_ctx* c, int32_t polls) {
    if (!c || polls < 0) return fail(c, -1, "bad argument");
    c->p.tp.wait_polls = (unsigned)polls;
    return 0;
}

int cudarl_reset_all(cudarl_ctx* c) {
    if (!c) return -1;
    CK(cudaSetDevice(c->cfg.device));
    { int rl = leave_tiles(c); if (rl) return rl; }
    c->p.step = (unsigned long long)c->h_step;
    launch_reset_all(c->p, c->st);
    CK(cudaGetLastError());
    c->epoch_step = c->h_step;
    return 0;
}

int cudarl_step_actions_device(cudarl_ctx* c, const int32_t* d_actions, float* d_rewards, uint8_t* d_dones) {
    if (!c || !d_actions) return fail(c, -1, "null argument");
    CK(cudaSetDevice(c->cfg.device));
    { int rl = leave_tiles(c); if (rl) return rl; }
    int rc = ensure_step_buffers(c); if (rc) return rc;
    launch_step_actions(c->p, d_actions, d_rewards, d_dones, c->st);
    CK(cudaGetLastError());
    return 0;
}

int cudarl_step_actions(cudarl_ctx* c, const int32_t* actions, float* rewards, uint8_t* dones) {
    if (!c || !actions) return fail(c, -1, "null argument");
    CK(cudaSetDevice(c->cfg.device));
    { int rl = leave_tiles(c); if (rl) return rl; }
    int rc = ensure_step_buffers(c); if (rc) return rc;
    const size_t N = c->p.N;
    CK(cudaMemcpyAsync(c->dact, actions, N * sizeof(int), cudaMemcpyHostToDevice, c->st));
    launch_step_actions(c->p, (const int*)c->dact, nullptr, nullptr, c->st);
    CK(cudaGetLastError());
    if (rewards) CK(cudaMemcpyAsync(rewards, c->dreward, N * sizeof(float), cudaMemcpyDeviceToHost, c->st));
    if (dones) CK(cudaMemcpyAsync(dones, c->ddone, N, cudaMemcpyDeviceToHost, c->st));
    CK(cudaStreamSynchronize(c->st));
    return 0;
}

int cudarl_get_reward_done(cudarl_ctx* c, float* rewards, uint8_t* dones) {
    if (!c) return -1;
    CK(cudaSetDevice(c->cfg.device));
    int rc = ensure_step_buffers(c); if (rc) return rc;
    if (rewards) CK(cudaMemcpyAsync(rewards, c->dreward, (size_t)c->p.N * sizeof(float), cudaMemcpyDeviceToHost, c->st));
    if (dones) CK(cudaMemcpyAsync(dones, c->ddone, (size_t)c->p.N, cudaMemcpyDeviceToHost, c->st));
    CK(cudaStreamSynchronize(c->st));
    return 0;
}

int cudarl_train_steps(cudarl_ctx* c, int64_t n) {
    if (!c || n < 0) return fail(c, -1, "bad argument");
    if (n == 0 || c->p.N == 0) return 0;
    CK(cudaSetDevice(c->cfg.device));
    int rc = 0;
    const cudarl_config& f = c->cfg;
    if (f.eps_kind == CUDARL_EPS_FIXED) {
        if (!c->eps_fixed_valid) {
            float e = (float)f.eps0; rc = upload_eps(c, &e, 1); if (rc) return rc;
            k_ctl_eps<<<1, 1, 0, c->st>>>(c->p.ctl, 0u, 1u, 0ull);
            c->eps_fixed_valid = true;
        }
        c->eps_mode = 0;
    } else if (f.eps_kind == CUDARL_EPS_MULT_PER_STEP || f.eps_kind == CUDARL_EPS_LINEAR) {
        std::vector<float> tab((size_t)n);
        for (int64_t k = 0; k < n; ++k) {
            if (f.eps_kind == CUDARL_EPS_MULT_PER_STEP) { tab[k] = (float)c->eps_running; c->eps_running *= (double)f.eps_decay; }
            else {
                int64_t g = c->h_step + k;
                tab[k] = (f.eps_steps <= 0 || g >= f.eps_steps) ? (float)f.eps_end
                       : (float)((double)f.eps0 + ((double)f.eps_end - (double)f.eps0) * (double)g / (double)f.eps_steps);
            }
        }
        rc = upload_eps(c, tab.data(), (size_t)n); if (rc) return rc;
        k_ctl_eps<<<1, 1, 0, c->st>>>(c->p.ctl, 1u, (unsigned)n, 0ull);
        c->eps_mode = 1;
    } else {  // per episode: index = episodes finished / environments, resolved on the device every step
        Ctl h; CK(cudaMemcpyAsync(&h, c->dctl, sizeof(Ctl), cudaMemcpyDeviceToHost, c->st));
        CK(cudaStreamSynchronize(c->st));
        unsigned long long k0 = h.episodes / (unsigned long long)c->p.N;
        std::vector<float> tab((size_t)n + 1);
        double e = (double)f.eps0;
        for (unsigned long long j = 0; j < k0; ++j) e *= (double)f.eps_decay;
        for (int64_t k = 0; k <= n; ++k) { tab[k] = (float)e; e *= (double)f.eps_decay; }
        rc = upload_eps(c, tab.data(), (size_t)n + 1); if (rc) return rc;
        k_ctl_eps<<<1, 1, 0, c->st>>>(c->p.ctl, 2u, (unsigned)(n + 1), k0);
        c->eps_mode = 2;
    }
    return run_steps(c, n);
}

int cudarl_train_steps_eps(cudarl_ctx* c, int64_t n, const float* eps_host) {
    if (!c || n < 0 || (n > 0 && !eps_host)) return fail(c, -1, "bad argument");
    if (n == 0 || c->p.N == 0) return 0;
    CK(cudaSetDevice(c->cfg.device));
    int rc = upload_eps(c, eps_host, (size_t)n); if (rc) return rc;
    k_ctl_eps<<<1, 1, 0, c->st>>>(c->p.ctl, 1u, (unsigned)n, 0ull);
    c->eps_mode = 1;
    return run_steps(c, n);
}

int cudarl_set_trace(cudarl_ctx* c, int on) {
    if (!c) return -1;
    CK(cudaSetDevice(c->cfg.device));
    if (on && !c->dtra) {
        size_t N = c->p.N ? c->p.N : 1;
        CK(cudaMalloc(&c->dtra, N * 4)); CK(cudaMalloc(&c->dtrr, N * 4)); CK(cudaMalloc(&c->dtrd, N));
        c->p.tr_a = (int*)c->dtra; c->p.tr_r = (float*)c->dtrr; c->p.tr_d = (unsigned char*)c->dtrd;
    }
    c->trace = on != 0;
    return 0;
}
int cudarl_get_trace(cudarl_ctx* c, int32_t* a, float* r, uint8_t* d) {
    if (!c || !c->dtra) return fail(c, -2, "trace is off");
    CK(cudaSetDevice(c->cfg.device));
    const size_t N = c->p.N;
    if (a) CK(cudaMemcpyAsync(a, c->dtra, N * 4, cudaMemcpyDeviceToHost, c->st));
    if (r) CK(cudaMemcpyAsync(r, c->dtrr, N * 4, cudaMemcpyDeviceToHost, c->st));
    if (d) CK(cudaMemcpyAsync(d, c->dtrd, N, cudaMemcpyDeviceToHost, c->st));
    CK(cudaStreamSynchronize(c->st));
    return 0;
}

int cudarl_eval_rollout(cudarl_ctx* c, int32_t max_steps, cudarl_eval_stats* out) {
    if (!c || !out || max_steps < 0) return fail(c, -1, "bad argument");
    CK(cudaSetDevice(c->cfg.device));
    { int rl = leave_tiles(c); if (rl) return rl; }
    if (c->cls_dirty) { launch_tile_classes(c->p, c->st); c->cls_dirty = false; }       // the rollout reads the per-tile move bytes
    k_ctl_eval_clear<<<1, 1, 0, c->st>>>(c->p.ctl);
    if (!c->dpolicy) CK(cudaMalloc(&c->dpolicy, c->p.S));                                // one byte per cell, kept until the context goes
    launch_eval(c->p, (unsigned char*)c->dpolicy, max_steps, (unsigned long long)c->eval_calls, c->st);
    CK(cudaGetLastError());
    Ctl h; CK(cudaMemcpyAsync(&h, c->dctl, sizeof(Ctl), cudaMemcpyDeviceToHost, c->st));
    CK(cudaStreamSynchronize(c->st));
    c->eval_calls += 1;
    out->envs = c->p.N; out->reached = (int64_t)h.eval_reached; out->total_steps = (int64_t)h.eval_steps;
    out->reward_sum = (double)out->reached * 1.0 - 0.01 * (double)(out->total_steps - out->reached);
    return 0;
}

int cudarl_update_batch(cudarl_ctx* c, int64_t n, const int32_t* sx, const int32_t* sy, const int32_t* a,
                        const float* r, const int32_t* nx, const int32_t* ny, const uint8_t* dn) {
    if (!c || n < 0) return fail(c, -1, "bad argument");
    if (n == 0) return 0;
    if (!sx || !sy || !a || !r || !nx || !ny || !dn) return fail(c, -1, "null argument");
    if (n >= (1ll << 26)) return fail(c, -1, "batch too large (at most 2^26 - 1 transitions per call)");
    const int W = c->p.W, H = c->p.H;
    for (int64_t i = 0; i < n; ++i)   // src/q_learning.cu:192-194,212-214 reject these; the reference kernel would read out of bounds
        if (sx[i] < 0 || sx[i] >= W || sy[i] < 0 || sy[i] >= H || a[i] < 0 || a[i] >= CUDARL_ACTIONS ||
            nx[i] < 0 || nx[i] >= W || ny[i] < 0 || ny[i] >= H) return fail(c, -3, "Invalid state or action");
    CK(cudaSetDevice(c->cfg.device));
    { int rl = leave_tiles(c); if (rl) return rl; }
    int rc = ensure_entry_capacity(c, (size_t)n); if (rc) return rc;
    if ((size_t)n > c->ub_cap) {
        CK(cudaStreamSynchronize(c->st));
        for (auto& b : c->dub) { if (b) cudaFree(b); b = nullptr; }
        c->ub_cap = 0;
        size_t cap = pow2ceil((size_t)n);
        for (int k = 0; k < 7; ++k) CK(cudaMalloc(&c->dub[k], cap * 4));
        c->ub_cap = cap;
    }
    const void* src[7] = {sx, sy, a, r, nx, ny, dn};
    for (int k = 0; k < 7; ++k) CK(cudaMemcpyAsync(c->dub[k], src[k], (size_t)n * (k == 6 ? 1 : 4), cudaMemcpyHostToDevice, c->st));
    c->p.step = (unsigned long long)c->h_step;
    launch_update_batch(c->p, (unsigned)n, (const int*)c->dub[0], (const int*)c->dub[1], (const int*)c->dub[2], (const float*)c->dub[3],
                        (const int*)c->dub[4], (const int*)c->dub[5], (const unsigned char*)c->dub[6], c->st);
    CK(cudaGetLastError());
    CK(cudaStreamSynchronize(c->st));
    return 0;
}

int cudarl_get_state(cudarl_ctx* c, int32_t* x, int32_t* y, int32_t* t) {
    if (!c) return -1;
    CK(cudaSetDevice(c->cfg.device));
    { int rl = leave_tiles(c); if (rl) return rl; }
    const size_t b = (size_t)c->p.N * 4;
    // state lives in slot order as int4 records; the export kernel writes x[N] | y[N] | t[N] in
    // environment order into the spare copy
    launch_export_state(c->p, c->st); CK(cudaGetLastError());
    const char* base = (const char*)c->p.st2;
    if (x) CK(cudaMemcpyAsync(x, base, b, cudaMemcpyDeviceToHost, c->st));
    if (y) CK(cudaMemcpyAsync(y, base + b, b, cudaMemcpyDeviceToHost, c->st));
    if (t) CK(cudaMemcpyAsync(t, base + 2 * b, b, cudaMemcpyDeviceToHost, c->st));
    return check_device_error(c);
}

int cudarl_set_state(cudarl_ctx* c, const int32_t* x, const int32_t* y, const int32_t* t) {
    if (!c) return -1;
    const size_t N = c->p.N;
    if (x) for (size_t i = 0; i < N; ++i) if (x[i] < 0 || x[i] >= c->p.W) return fail(c, -3, "Invalid state");
    if (y) for (size_t i = 0; i < N; ++i) if (y[i] < 0 || y[i] >= c->p.H) return fail(c, -3, "Invalid state");
    if (t) for (size_t i = 0; i < N; ++i) if (t[i] < 0 || t[i] > 0xFFFFFE) return fail(c, -3, "Invalid state (an episode's step count lies in 0 .. 16,777,214)");
    CK(cudaSetDevice(c->cfg.device));
    { int rl = leave_tiles(c); if (rl) return rl; }
    if (!c->dimport) CK(cudaMalloc(&c->dimport, (N ? N : 1) * 12));
    int* dx = (int*)c->dimport; int* dy = dx + N; int* dt = dy + N;
    if (x) CK(cudaMemcpyAsync(dx, x, N * 4, cudaMemcpyHostToDevice, c->st));
    if (y) CK(cudaMemcpyAsync(dy, y, N * 4, cudaMemcpyHostToDevice, c->st));
    if (t) CK(cudaMemcpyAsync(dt, t, N * 4, cudaMemcpyHostToDevice, c->st));
    launch_import_state(c->p, x ? dx : nullptr, y ? dy : nullptr, t ? dt : nullptr, c->st);
    CK(cudaGetLastError());
    CK(cudaStreamSynchronize(c->st));
    return 0;
}

int cudarl_get_q(cudarl_ctx* c, float* q) {
    if (!c || !q) return fail(c, -1, "null argument");
    CK(cudaSetDevice(c->cfg.device));
    { int rl = leave_tiles(c); if (rl) return rl; }
    CK(cudaMemcpyAsync(q, c->p.Q, (size_t)c->p.S * sizeof(float4), cudaMemcpyDeviceToHost, c->st));   // the table already is in the caller's layout
    return check_device_error(c);
}
int cudarl_set_q(cudarl_ctx* c, const float* q) {
    if (!c || !q) return fail(c, -1, "null argument");
    CK(cudaSetDevice(c->cfg.device));
    { int rl = leave_tiles(c); if (rl) return rl; }
    CK(cudaMemcpyAsync(c->p.Q, q, (size_t)c->p.S * sizeof(float4), cudaMemcpyHostToDevice, c->st));
    CK(cudaStreamSynchronize(c->st));
    return 0;
}

int cudarl_get_cells(cudarl_ctx* c, uint8_t* cells) {
    if (!c || !cells) return fail(c, -1, "null argument");
    std::memcpy(cells, c->cells.data(), c->cells.size());
    return 0;
}

// The device copy of the trap table: {cell, penalty bits}, ascending by cell (std::map iterates in that order).
static int upload_traps(cudarl_ctx* c) {
    const size_t n = c->traps.size();
    if (n > c->traps_cap) {
        CK(cudaStreamSynchronize(c->st));
        if (c->dtraps) cudaFree(c->dtraps);
        c->dtraps = nullptr; c->traps_cap = 0;
        const size_t cap = pow2ceil(n < 64 ? 64 : n);
        CK(cudaMalloc(&c->dtraps, cap * sizeof(uint2)));
        c->traps_cap = cap;
    }
    std::vector<uint2> h; h.reserve(n);
    for (auto& t : c->traps) { uint2 e; e.x = t.first; std::memcpy(&e.y, &t.second, 4); h.push_back(e); }
    if (n) CK(cudaMemcpyAsync(c->dtraps, h.data(), n * sizeof(uint2), cudaMemcpyHostToDevice, c->st));
    CK(cudaStreamSynchronize(c->st));           // `h` is pageable and dies here
    c->p.traps = (const uint2*)c->dtraps; c->p.ntraps = (unsigned)n;
    return 0;
}

static int set_cell(cudarl_ctx* c, int32_t x, int32_t y, unsigned cls, bool single_goal, const float* trap_penalty = nullptr) {
    if (!c) return -1;
    if (x < 0 || x >= c->p.W || y < 0 || y >= c->p.H) return fail(c, -3, "Invalid state");
    CK(cudaSetDevice(c->cfg.device));
    { int rl = leave_tiles(c); if (rl) return rl; }
    const unsigned cell = (unsigned)y * (unsigned)c->p.W + (unsigned)x;
    const bool is_trap = trap_penalty && *trap_penalty < 0.0f && *trap_penalty > -1.0f;      // src/kernels.cu:61 of the reference
    const bool had_trap = c->traps.erase(cell) != 0;
    if (is_trap) c->traps[cell] = *trap_penalty;
    if (is_trap || had_trap) { int rt = upload_traps(c); if (rt) return rt; }
    if (single_goal) {
        for (auto& v : c->cells) if (v == 2) v = 0;
        launch_cell_set(c->p, 0, 0, 1, c->st);
    }
    c->cells[cell] = (uint8_t)cls; c->cls_dirty = true;
    launch_cell_set(c->p, cell, cls == 1 ? (is_trap ? (CW_OBST | CW_TRAP) : CW_OBST) : (cls == 2 ? CW_GOAL : 0u), 0, c->st);
    CK(cudaGetLastError());
    uint32_t fb = 0xFFFFFFFFu;
    for (uint32_t s = 0; s < c->p.S; ++s) if (c->cells[s] == 0) { fb = s; break; }
    c->p.fallback_start = fb == 0xFFFFFFFFu ? c->p.start_cell : fb;
    CK(cudaStreamSynchronize(c->st));
    return 0;
}
int cudarl_add_obstacle(cudarl_ctx* c, int32_t x, int32_t y) { return set_cell(c, x, y, 1, false); }
int cudarl_set_goal(cudarl_ctx* c, int32_t x, int32_t y) { return set_cell(c, x, y, 2, true); }
int cudarl_add_trap(cudarl_ctx* c, int32_t x, int32_t y, float penalty) { return set_cell(c, x, y, 1, false, &penalty); }
int cudarl_get_traps(cudarl_ctx* c, int32_t capacity, int32_t* cells, float* penalties, int32_t* count) {
    if (!c || !count || capacity < 0) return fail(c, -1, "bad argument");
    *count = (int32_t)c->traps.size();
    int32_t k = 0;
    for (auto& t : c->traps) { if (k >= capacity) break; if (cells) cells[k] = (int32_t)t.first; if (penalties) penalties[k] = t.second; ++k; }
    return 0;
}

int cudarl_set_legacy_clamp(cudarl_ctx* c, int on) {
    if (!c) return -1;
    c->cfg.legacy_clamp = on ? 1 : 0; c->p.legacy_clamp = on ? 1 : 0;
    return 0;
}

int cudarl_get_stats(cudarl_ctx* c, cudarl_stats* out) {
    if (!c || !out) return -1;
    CK(cudaSetDevice(c->cfg.device));
    Ctl h; CK(cudaMemcpyAsync(&h, c->dctl, sizeof(Ctl), cudaMemcpyDeviceToHost, c->st));
    CK(cudaStreamSynchronize(c->st));
    std::memset(out, 0, sizeof(*out));
    out->steps = c->h_step; out->env_steps = c->h_step * (int64_t)c->p.N;
    out->episodes = (int64_t)h.episodes; out->goals = (int64_t)h.goals; out->timeouts = (int64_t)h.timeouts;
    out->conflicts = (int64_t)h.conflicts; out->long_chains = (int64_t)h.long_chains; out->chained = (int64_t)h.general;
    out->reward_sum = (double)out->goals * 1.0 - 0.01 * (double)(out->env_steps - out->goals);
    out->epsilon = c->eps_mode == 2 ? h.eps_used : c->eps_used; out->device_error = (int32_t)h.error;
    if (h.error) return fail(c, CUDARL_ERR_DEVICE + (int)h.error, "device error bits " + std::to_string(h.error) + " (statistics filled in; the results of this context are not to be trusted)");
    return 0;
}

int cudarl_comm_unique_id(void* id128) {
    cudarl_ctx* c = nullptr;
    if (!id128) return fail(c, -1, "null argument");
    std::string e; if (!g_nccl.load(e)) return fail(c, -4, e);
    static_assert(sizeof(ncclUniqueId) == CUDARL_COMM_ID_BYTES, "ncclUniqueId size");
    ncclUniqueId id; NK(g_nccl.GetUniqueId(&id));
    std::memcpy(id128, &id, sizeof(id));
    return 0;
}
int cudarl_comm_init(cudarl_ctx* c, const void* id128, int32_t rank, int32_t nranks) {
    if (!c || !id128 || nranks < 1 || rank < 0 || rank >= nranks) return fail(c, -1, "bad argument");
    std::string e; if (!g_nccl.load(e)) return fail(c, -4, e);
    CK(cudaSetDevice(c->cfg.device));
    ncclUniqueId id; std::memcpy(&id, id128, sizeof(id));
    NK(g_nccl.CommInitRank(&c->comm, nranks, id, rank));
    c->rank = rank; c->nranks = nranks;
    if (nranks > 1 && !c->cfg.avg_over_nccl) { int rp = map_peer_tables(c); if (rp) return rp; }
    return 0;
}
int cudarl_comm_peer_memory(const cudarl_ctx* c) { return (c && c->peer_ok) ? 1 : 0; }
int cudarl_average_replicas(cudarl_ctx* c) {
    if (!c) return -1;
    CK(cudaSetDevice(c->cfg.device));
    return average_now(c);
}

int cudarl_timer_start(cudarl_ctx* c) { if (!c) return -1; CK(cudaSetDevice(c->cfg.device)); CK(cudaEventRecord(c->ev0, c->st)); return 0; }
int cudarl_timer_stop_ms(cudarl_ctx* c, float* ms) {
    if (!c || !ms) return -1;
    CK(cudaSetDevice(c->cfg.device));
    CK(cudaEventRecord(c->ev1, c->st));
    CK(cudaEventSynchronize(c->ev1));
    CK(cudaEventElapsedTime(ms, c->ev0, c->ev1));
    return 0;
}
int cudarl_kernel_timing(cudarl_ctx* c, int on) {
    if (!c) return -1;
    CK(cudaSetDevice(c->cfg.device));
    if (on && c->kev.empty()) {
        c->kev.resize(2 * 2048);
        for (auto& e : c->kev) CK(cudaEventCreate(&e));
    }
    if (!on) { int rc = drain_kernel_events(c); if (rc) return rc; }
    else { c->main_ms = 0; c->klaunches = 0; c->kev_used = 0; c->kseg_open = false; c->kseg_launches.clear(); }
    c->ktiming = on != 0;
    return 0;
}
int cudarl_kernel_time_ms(cudarl_ctx* c, float* step_ms, int64_t* launches) {
    if (!c) return -1;
    CK(cudaSetDevice(c->cfg.device));
    int rc = drain_kernel_events(c); if (rc) return rc;
    if (step_ms) *step_ms = (float)c->main_ms;
    if (launches) *launches = c->klaunches;
    return 0;
}

}  // extern "C"
