// oracle.cpp -- TEST INFRASTRUCTURE, not product code.
//
// Sequential CPU restatement of the batched grid-world step + epsilon-greedy + tabular TD update
// path of life423/CudaRL-Arena, with the batched semantics of the GPU library (N environments per
// step, all TD targets see the table as it was at the start of the step, updates of one (state, action)
// are applied one after the other in ascending environment index).  Only tests, the smoke check and the CPU-baseline
// leg of the benchmark may load this file's shared object; the product never does.
//
// It is written independently of the CUDA sources (own Philox, own grid generator, own step) so
// that an error in one is not silently shared by the other.  Each function cites the reference
// lines (paths relative to the reference project's root) it restates.
//
// Pinning: the environment step/reset are pinned by the known-answer cases of the reference's
// tests/test_environment.cpp and by fixtures generated from the reference's own Python CPU code
// (src/gui.py MockEnvironment, src/train.py QTableAgent) -- see tests/golden/.  Philox4x32-10 is
// pinned by the published Random123 known-answer vectors.  The batched extensions (collision
// order, seeded starts, replica averaging) have no counterpart in the reference.
#include <cstdint>
#include <cstring>
#include <cmath>
#include <vector>
#include <thread>
#include <mutex>
#include <condition_variable>
#include <functional>
#include <unordered_map>
#include <algorithm>
#include <string>
#include "../include/cudarl.h"

namespace {

// ---------------------------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11).
struct U4 { uint32_t v[4]; };

inline U4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
    for (int r = 0; r < 10; ++r) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return U4{{c0, c1, c2, c3}};
}

const uint32_t TAG_GRID = 0x47524944u, TAG_WALL = 0x57414C4Cu, TAG_GOAL = 0x474F414Cu,
               TAG_START = 0x53545254u, TAG_QINIT = 0x51494E49u, TAG_POLICY = 0x504F4C49u,
               TAG_EVAL = 0x4556414Cu;

inline uint32_t mulhi32(uint32_t a, uint32_t b) { return (uint32_t)(((uint64_t)a * b) >> 32); }
inline float u01(uint32_t w) { return (float)(w >> 8) * 5.9604644775390625e-08f; }  // * 2^-24

// Worker threads that live as long as the oracle: run(f) calls f(k) on thread k for k = 0..T-1 (the caller is thread 0)
// and returns when all are done.  Timing runs use it; results never depend on the number of threads.
struct Pool {
    int T = 1; std::vector<std::thread> th;
    std::mutex mu; std::condition_variable cv_go, cv_done;
    std::function<void(int)> job; uint64_t gen = 0; int left = 0; bool stop = false;
    void start(int threads) {
        shutdown(); T = threads < 1 ? 1 : threads; stop = false;
        for (int k = 1; k < T; ++k) th.emplace_back([this, k] {
            uint64_t seen = 0;
            for (;;) {
                std::function<void(int)> f;
                { std::unique_lock<std::mutex> l(mu); cv_go.wait(l, [&] { return stop || gen != seen; }); if (stop) return; seen = gen; f = job; }
                f(k);
                { std::lock_guard<std::mutex> l(mu); if (--left == 0) cv_done.notify_one(); }
            }
        });
    }
    void run(const std::function<void(int)>& f) {
        if (T <= 1) { f(0); return; }
        { std::lock_guard<std::mutex> l(mu); job = f; left = T - 1; ++gen; }
        cv_go.notify_all();
        f(0);
        std::unique_lock<std::mutex> l(mu); cv_done.wait(l, [&] { return left == 0; });
    }
    void shutdown() {
        { std::lock_guard<std::mutex> l(mu); stop = true; }
        cv_go.notify_all();
        for (auto& t : th) t.join();
        th.clear();
    }
    ~Pool() { shutdown(); }
};

struct Oracle {
    cudarl_config cfg;
    int W, H; int64_t S, N;
    uint32_t k0; uint32_t k1base;
    std::vector<uint8_t> cells;      // 0 free, 1 obstacle, 2 goal
    std::vector<float> q;            // (y*W+x)*4 + a
    std::vector<int32_t> x, y, t;
    std::vector<float> reward; std::vector<uint8_t> done;   // facade step
    std::vector<int32_t> tr_a; std::vector<float> tr_r; std::vector<uint8_t> tr_d;  // trace of last train step
    int64_t fallback_start = -1;
    int64_t step = 0, episodes = 0, goals = 0, timeouts = 0, conflicts = 0;
    int64_t eval_calls = 0;
    double eps_running;              // MULT_PER_STEP: eps for the next step, in double
    float eps_last = 0.f;
    int threads = 1;
    std::string err;
    // scratch of a train step
    std::vector<int32_t> ps; std::vector<uint8_t> pa; std::vector<float> pd;
    std::vector<uint32_t> occ; bool count_conflicts = true;
    std::unordered_map<int64_t, float> traps;      // cell -> penalty in (-1, 0); the cell is an obstacle as well (src/kernels.cu:29-36,61-63)
    Pool pool;
    std::vector<std::vector<int32_t>> bins;        // [thread * T + stripe]: transitions of that thread's environments whose cell lies in the stripe

    // Reward of a step that did not end on a goal, given the cell the action pointed at: the step cost, or the penalty of a
    // trap the agent walked into (it does not move: a trap is an obstacle) -- src/kernels.cu:47,61-63.
    float step_reward(int x, int y, int action) const {
        if (traps.empty()) return -0.01f;
        int dx = 0, dy = 0;
        switch (action) { case 0: dy = -1; break; case 1: dx = 1; break; case 2: dy = 1; break; case 3: dx = -1; break; default: break; }
        const int nx = x + dx, ny = y + dy;
        if (nx < 0 || nx >= W || ny < 0 || ny >= H) return -0.01f;
        auto it = traps.find((int64_t)ny * W + nx);
        return it == traps.end() ? -0.01f : it->second;
    }

    uint32_t key1(uint32_t tag) const { return k1base ^ tag; }
    bool is_obst(int64_t c) const { return cells[c] == 1; }
    bool is_goal(int64_t c) const { return cells[c] == 2; }
};

// ---------------------------------------------------------------------------------------------
// Grid from the seed.  The reference only ever builds an obstacle-free grid with the goal in the
// top-right corner (src/environment.cu:138-147); obstacle cells follow the rule of
// src/kernels.cu:29-36 (a cell blocks iff its class is "obstacle").
bool build_grid(Oracle& o) {
    const cudarl_config& c = o.cfg;
    o.cells.assign(o.S, 0);
    if (c.obstacle_kind == CUDARL_OBST_BERNOULLI) {
        double t = (double)c.obstacle_p * 4294967296.0;
        uint32_t thr = t >= 4294967295.0 ? 4294967295u : (t <= 0.0 ? 0u : (uint32_t)t);
        for (int64_t base = 0; base < o.S; base += 4) {
            U4 w = philox4x32_10((uint32_t)(base >> 2), 0, 0, 0, o.k0, o.key1(TAG_GRID));
            for (int j = 0; j < 4 && base + j < o.S; ++j) if (w.v[j] < thr) o.cells[base + j] = 1;
        }
    } else if (c.obstacle_kind == CUDARL_OBST_WALLS) {
        int64_t target = (int64_t)std::floor((double)c.obstacle_p * (double)o.S);
        int64_t count = 0;
        for (uint32_t k = 0; count < target && k < 0x7fffffffu; ++k) {
            U4 w = philox4x32_10(k, 0, 0, 0, o.k0, o.key1(TAG_WALL));
            int64_t origin = mulhi32(w.v[0], (uint32_t)o.S);
            int ox = (int)(origin % o.W), oy = (int)(origin / o.W);
            bool horiz = (w.v[1] & 1u) != 0; int len = 1 + (int)(w.v[2] & 31u);
            for (int j = 0; j < len; ++j) {
                int px = horiz ? ox + j : ox, py = horiz ? oy : oy + j;
                if (px >= o.W || py >= o.H) break;
                int64_t cc = (int64_t)py * o.W + px;
                if (o.cells[cc] == 0) { o.cells[cc] = 1; ++count; }
            }
        }
    }
    int64_t fixed_start = -1;
    if (c.start_mode == CUDARL_START_CENTRE) fixed_start = (int64_t)(o.H / 2) * o.W + o.W / 2;
    if (c.start_mode == CUDARL_START_FIXED) {
        if (c.start_x < 0 || c.start_x >= o.W || c.start_y < 0 || c.start_y >= o.H) { o.err = "start cell out of range"; return false; }
        fixed_start = (int64_t)c.start_y * o.W + c.start_x;
    }
    if (fixed_start >= 0) o.cells[fixed_start] = 0;
    if (c.goal_mode == CUDARL_GOAL_TOP_RIGHT) {
        o.cells[o.W - 1] = 2;                       // src/environment.cu:43, :146
    } else if (c.goal_mode == CUDARL_GOAL_LIST) {
        if (c.num_goals < 1 || c.num_goals > CUDARL_MAX_GOALS) { o.err = "num_goals out of range"; return false; }
        for (int g = 0; g < c.num_goals; ++g) {
            int gx = c.goal_xy[2 * g], gy = c.goal_xy[2 * g + 1];
            if (gx < 0 || gx >= o.W || gy < 0 || gy >= o.H) { o.err = "goal cell out of range"; return false; }
            o.cells[(int64_t)gy * o.W + gx] = 2;
        }
    } else if (c.goal_mode == CUDARL_GOAL_SEEDED) {
        if (c.num_goals < 1 || c.num_goals > CUDARL_MAX_GOALS) { o.err = "num_goals out of range"; return false; }
        for (int g = 0; g < c.num_goals; ++g) {
            bool placed = false;
            for (uint32_t a = 0; a < (1u << 20) && !placed; ++a) {
                U4 w = philox4x32_10((uint32_t)g, a, 0, 0, o.k0, o.key1(TAG_GOAL));
                int64_t cand = mulhi32(w.v[0], (uint32_t)o.S);
                if (o.cells[cand] == 0 && cand != fixed_start) { o.cells[cand] = 2; placed = true; }
            }
            if (!placed) { o.err = "could not place a seeded goal"; return false; }
        }
    } else { o.err = "bad goal_mode"; return false; }
    o.fallback_start = -1;
    for (int64_t cc = 0; cc < o.S; ++cc) if (o.cells[cc] == 0) { o.fallback_start = cc; break; }
    if (c.start_mode == CUDARL_START_RANDOM && o.fallback_start < 0) { o.err = "no free cell"; return false; }
    return true;
}

// Start cell of global environment gi for the episode identified by `nonce`.
// Reference: centre of the grid (src/environment.cu:9-10).  RANDOM is the batched extension.
int64_t start_cell(const Oracle& o, uint32_t gi, uint64_t nonce, uint32_t tag) {
    const cudarl_config& c = o.cfg;
    if (c.start_mode == CUDARL_START_CENTRE) return (int64_t)(o.H / 2) * o.W + o.W / 2;
    if (c.start_mode == CUDARL_START_FIXED) return (int64_t)c.start_y * o.W + c.start_x;
    for (uint32_t k = 0; k < 16; ++k) {
        U4 w = philox4x32_10(gi, k, (uint32_t)nonce, (uint32_t)(nonce >> 32), o.k0, o.key1(tag));
        for (int j = 0; j < 4; ++j) {
            int64_t cand = mulhi32(w.v[j], (uint32_t)o.S);
            if (o.cells[cand] == 0) return cand;
        }
    }
    return o.fallback_start;
}

void refresh_fallback(Oracle& o) {
    o.fallback_start = -1;
    for (int64_t cc = 0; cc < o.S; ++cc) if (o.cells[cc] == 0) { o.fallback_start = cc; break; }
}

void init_q(Oracle& o) {
    o.q.assign(o.S * 4, 0.0f);                                  // src/q_learning.cu:13
    if (o.cfg.q_init_kind == CUDARL_QINIT_UNIFORM) {
        for (int64_t s = 0; s < o.S; ++s) {
            U4 w = philox4x32_10((uint32_t)s, 0, 0, 0, o.k0, o.key1(TAG_QINIT));
            for (int a = 0; a < 4; ++a) o.q[s * 4 + a] = u01(w.v[a]) * o.cfg.q_init_scale;
        }
    }
}

void reset_all(Oracle& o) {
    for (int64_t i = 0; i < o.N; ++i) {
        int64_t c = start_cell(o, (uint32_t)(o.cfg.env_offset + i), (uint64_t)o.step, TAG_START);
        o.x[i] = (int32_t)(c % o.W); o.y[i] = (int32_t)(c / o.W); o.t[i] = 0;   // src/environment.cu:9-12
        o.reward[i] = 0.0f; o.done[i] = 0;
    }
}

// One environment transition: src/environment.cu:17-48 with the obstacle test of
// src/kernels.cu:29-44.  Returns the new cell; `moved` is informational.
inline int64_t move_cell(const Oracle& o, int x, int y, int action) {
    int dx = 0, dy = 0;
    switch (action) { case 0: dy = -1; break; case 1: dx = 1; break; case 2: dy = 1; break; case 3: dx = -1; break; default: break; }
    int nx = x + dx, ny = y + dy;
    bool inb = nx >= 0 && nx < o.W && ny >= 0 && ny < o.H;
    if (inb && !o.is_obst((int64_t)ny * o.W + nx)) return (int64_t)ny * o.W + nx;
    return (int64_t)y * o.W + x;
}

// First-maximum argmax: np.argmax at src/train.py:108, strict '>' at src/q_learning.cu:200-206.
inline int argmax4(const float* r) {
    int b = 0; float bv = r[0];
    for (int a = 1; a < 4; ++a) if (r[a] > bv) { bv = r[a]; b = a; }
    return b;
}
inline float max4(const float* r) {           // true max: src/gpu/kernels.cu:36-45, src/train.py:134
    float m = r[0];
    for (int a = 1; a < 4; ++a) m = r[a] > m ? r[a] : m;
    return m;
}

float epsilon_for_step(Oracle& o) {
    const cudarl_config& c = o.cfg;
    switch (c.eps_kind) {
        case CUDARL_EPS_FIXED: return (float)c.eps0;
        case CUDARL_EPS_MULT_PER_STEP: return (float)o.eps_running;     // src/train.py:141 (float64 product)
        case CUDARL_EPS_MULT_PER_EPISODE: {
            int64_t k = o.episodes / o.N; double e = (double)c.eps0;
            for (int64_t j = 0; j < k; ++j) e *= (double)c.eps_decay;
            return (float)e;
        }
        case CUDARL_EPS_LINEAR: {
            if (c.eps_steps <= 0 || o.step >= c.eps_steps) return (float)c.eps_end;
            return (float)((double)c.eps0 + ((double)c.eps_end - (double)c.eps0) * (double)o.step / (double)c.eps_steps);
        }
    }
    return (float)c.eps0;
}

// One batched train step.  Phase 1 reads only Q_t (so it may run on several threads); phase 2
// folds the TD errors into the table in ascending environment index.
void train_step(Oracle& o, float eps) {
    const cudarl_config& c = o.cfg;
    const uint64_t g = (uint64_t)o.step;
    o.eps_last = eps;
    const int T = (o.threads > 1 && o.N >= 4096) ? o.threads : 1;
    if (T > 1 && o.pool.T != T) o.pool.start(T);
    std::vector<int64_t> ep(T, 0), go(T, 0), to(T, 0);
    std::vector<int32_t> nxs(o.N), nys(o.N), nts(o.N);
    const int64_t chunk = (o.N + T - 1) / T, stripe = (o.S + T - 1) / T;
    if (T > 1) { o.bins.resize((size_t)T * T); for (auto& b : o.bins) b.clear(); }
    auto phase1 = [&](int tid) {
        const int64_t lo = tid * chunk, hi = std::min(o.N, lo + chunk);
        for (int64_t i = lo; i < hi; ++i) {
            uint32_t gi = (uint32_t)(c.env_offset + i);
            int x = o.x[i], y = o.y[i];
            int64_t s = (int64_t)y * o.W + x;
            const float* row = &o.q[s * 4];
            // epsilon-greedy: src/train.py:101-108
            U4 w = philox4x32_10(gi, 0, (uint32_t)g, (uint32_t)(g >> 32), o.k0, o.key1(TAG_POLICY));
            int a = (u01(w.v[0]) < eps) ? (int)(w.v[1] & 3u) : argmax4(row);
            int64_t s2 = move_cell(o, x, y, a);
            bool done = o.is_goal(s2);                       // src/environment.cu:43-46
            float r = done ? 1.0f : o.step_reward(x, y, a);  // src/environment.cu:40,44; trap: src/kernels.cu:61-63
            float m = 0.0f;                                  // src/kernels.cu:100-110
            if (!done) { m = max4(&o.q[s2 * 4]); if (c.legacy_clamp && m < 0.0f) m = 0.0f; }
            float target = std::fmaf(c.gamma, m, r);         // src/kernels.cu:113 as nvcc contracts it
            o.ps[i] = (int32_t)s; o.pa[i] = (uint8_t)a; o.pd[i] = target;
            o.tr_a[i] = a; o.tr_r[i] = r; o.tr_d[i] = done ? 1 : 0;
            if (T > 1) o.bins[(size_t)tid * T + (size_t)(s / stripe)].push_back((int32_t)i);
            // episode bookkeeping: src/train.py:191-222 (reset on done or after max_steps)
            bool timeout = c.max_steps > 0 && o.t[i] + 1 >= c.max_steps;
            if (done || timeout) {
                int64_t sc = start_cell(o, gi, g + 1, TAG_START);
                nxs[i] = (int32_t)(sc % o.W); nys[i] = (int32_t)(sc / o.W); nts[i] = 0;
                ++ep[tid]; if (done) ++go[tid]; else ++to[tid];
            } else {
                nxs[i] = (int32_t)(s2 % o.W); nys[i] = (int32_t)(s2 / o.W); nts[i] = o.t[i] + 1;
            }
        }
    };
    // Phase 2: the reference update Q[s,a] = fma(lr, target - Q[s,a], Q[s,a]) (src/kernels.cu:113-114 as compiled)
    // applied one transition after the other in environment order: an update of the same (s,a) sees the value
    // the previous one left; the targets were taken from Q_t in phase 1.  (The reference kernel leaves
    // same-(s,a) collisions to a data race.)
    if (T <= 1) {
        phase1(0);
        for (int64_t i = 0; i < o.N; ++i) {
            float* p = &o.q[(int64_t)o.ps[i] * 4 + o.pa[i]];
            *p = std::fmaf(c.lr, o.pd[i] - *p, *p);
        }
    } else {
        // Same fold, split by cell stripe: thread k applies the updates whose cell falls in stripe k.  Phase 1 has sorted every
        // thread's transitions into stripes already; visiting the source threads in order 0..T-1 (their environments are
        // ascending ranges) keeps every (s,a) in ascending environment index.
        o.pool.run(phase1);
        o.pool.run([&](int k) {
            for (int j = 0; j < T; ++j)
                for (int32_t i : o.bins[(size_t)j * T + k]) { float* p = &o.q[(int64_t)o.ps[i] * 4 + o.pa[i]]; *p = std::fmaf(c.lr, o.pd[i] - *p, *p); }
        });
    }
    if (o.count_conflicts) {
        if ((int64_t)o.occ.size() != o.S) o.occ.assign(o.S, 0);
        for (int64_t i = 0; i < o.N; ++i) o.occ[o.ps[i]] += 1;
        for (int64_t i = 0; i < o.N; ++i) if (o.occ[o.ps[i]] > 1) o.conflicts += 1;
        for (int64_t i = 0; i < o.N; ++i) o.occ[o.ps[i]] = 0;
    }
    o.x.swap(nxs); o.y.swap(nys); o.t.swap(nts);
    for (int k = 0; k < T; ++k) { o.episodes += ep[k]; o.goals += go[k]; o.timeouts += to[k]; }
    o.step += 1;
    if (c.eps_kind == CUDARL_EPS_MULT_PER_STEP) o.eps_running *= (double)c.eps_decay;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
extern "C" {

void orc_philox(const uint32_t* ctr, const uint32_t* key, uint32_t* out) {
    U4 w = philox4x32_10(ctr[0], ctr[1], ctr[2], ctr[3], key[0], key[1]);
    std::memcpy(out, w.v, 16);
}

void* orc_create(const cudarl_config* cfg) {
    Oracle* o = new Oracle();
    o->cfg = *cfg; o->W = cfg->width; o->H = cfg->height; o->S = (int64_t)cfg->width * cfg->height; o->N = cfg->num_envs;
    o->k0 = (uint32_t)cfg->seed; o->k1base = (uint32_t)(cfg->seed >> 32);
    o->eps_running = (double)cfg->eps0;
    if (o->W < 1 || o->H < 1 || o->N < 0 || !build_grid(*o)) return o;   // err set or bad size; caller checks orc_error
    init_q(*o);
    o->x.assign(o->N, 0); o->y.assign(o->N, 0); o->t.assign(o->N, 0);
    o->reward.assign(o->N, 0.f); o->done.assign(o->N, 0);
    o->tr_a.assign(o->N, 0); o->tr_r.assign(o->N, 0.f); o->tr_d.assign(o->N, 0);
    o->ps.assign(o->N, 0); o->pa.assign(o->N, 0); o->pd.assign(o->N, 0.f);
    reset_all(*o);
    return o;
}
void orc_destroy(void* h) { delete (Oracle*)h; }
const char* orc_error(void* h) { return ((Oracle*)h)->err.c_str(); }
void orc_set_threads(void* h, int t) { ((Oracle*)h)->threads = t < 1 ? 1 : t; }
void orc_count_conflicts(void* h, int on) { ((Oracle*)h)->count_conflicts = on != 0; }

void orc_reset_all(void* h) { reset_all(*(Oracle*)h); }

// Environment::step for every environment with caller actions; done is sticky
// (src/environment.cu:45; only reset clears it, :12).
void orc_step_actions(void* h, const int32_t* actions, float* rewards, uint8_t* dones) {
    Oracle& o = *(Oracle*)h;
    for (int64_t i = 0; i < o.N; ++i) {
        const float r0 = o.step_reward(o.x[i], o.y[i], actions[i]);
        int64_t s2 = move_cell(o, o.x[i], o.y[i], actions[i]);
        o.x[i] = (int32_t)(s2 % o.W); o.y[i] = (int32_t)(s2 / o.W); o.t[i] += 1;
        o.reward[i] = r0;
        if (o.is_goal(s2)) { o.reward[i] = 1.0f; o.done[i] = 1; }
        if (rewards) rewards[i] = o.reward[i];
        if (dones) dones[i] = o.done[i];
    }
}

void orc_train_steps(void* h, int64_t n) {
    Oracle& o = *(Oracle*)h;
    for (int64_t k = 0; k < n; ++k) train_step(o, epsilon_for_step(o));
}
void orc_train_steps_eps(void* h, int64_t n, const float* eps) {
    Oracle& o = *(Oracle*)h;
    for (int64_t k = 0; k < n; ++k) train_step(o, eps[k]);
}
void orc_get_trace(void* h, int32_t* a, float* r, uint8_t* d) {
    Oracle& o = *(Oracle*)h;
    if (a) std::memcpy(a, o.tr_a.data(), o.N * 4);
    if (r) std::memcpy(r, o.tr_r.data(), o.N * 4);
    if (d) std::memcpy(d, o.tr_d.data(), o.N);
}

// evaluate(): src/train.py:262-311 -- reset, greedy (training=False, :284), stop on done or cap.
void orc_eval_rollout(void* h, int32_t max_steps, cudarl_eval_stats* out) {
    Oracle& o = *(Oracle*)h;
    int64_t reached = 0, total = 0;
    for (int64_t i = 0; i < o.N; ++i) {
        int64_t s = start_cell(o, (uint32_t)(o.cfg.env_offset + i), (uint64_t)o.eval_calls, TAG_EVAL);
        for (int k = 0; k < max_steps; ++k) {
            int a = argmax4(&o.q[s * 4]);
            s = move_cell(o, (int)(s % o.W), (int)(s / o.W), a);
            ++total;
            if (o.is_goal(s)) { ++reached; break; }
        }
    }
    o.eval_calls += 1;
    out->envs = o.N; out->reached = reached; out->total_steps = total;
    out->reward_sum = (double)reached * 1.0 - 0.01 * (double)(total - reached);
}

// CudaQLearning::update_batch: src/q_learning.cu:108-174 + src/kernels.cu:68-116.
int orc_update_batch(void* h, int64_t n, const int32_t* sx, const int32_t* sy, const int32_t* a,
                     const float* r, const int32_t* nx, const int32_t* ny, const uint8_t* dn) {
    Oracle& o = *(Oracle*)h; const cudarl_config& c = o.cfg;
    std::vector<float> d(n);
    for (int64_t i = 0; i < n; ++i) {
        if (sx[i] < 0 || sx[i] >= o.W || sy[i] < 0 || sy[i] >= o.H || a[i] < 0 || a[i] >= 4 ||
            nx[i] < 0 || nx[i] >= o.W || ny[i] < 0 || ny[i] >= o.H) return -1;
    }
    for (int64_t i = 0; i < n; ++i) {
        int64_t s = (int64_t)sy[i] * o.W + sx[i], s2 = (int64_t)ny[i] * o.W + nx[i];
        float m = 0.0f;
        if (!dn[i]) { m = max4(&o.q[s2 * 4]); if (c.legacy_clamp && m < 0.0f) m = 0.0f; }
        (void)s;
        d[i] = std::fmaf(c.gamma, m, r[i]);                 // TD target from the table before the call
    }
    for (int64_t i = 0; i < n; ++i) {
        float* p = &o.q[((int64_t)sy[i] * o.W + sx[i]) * 4 + a[i]];
        *p = std::fmaf(c.lr, d[i] - *p, *p);
    }
    return 0;
}

void orc_get_state(void* h, int32_t* x, int32_t* y, int32_t* t) {
    Oracle& o = *(Oracle*)h;
    if (x) std::memcpy(x, o.x.data(), o.N * 4);
    if (y) std::memcpy(y, o.y.data(), o.N * 4);
    if (t) std::memcpy(t, o.t.data(), o.N * 4);
}
void orc_set_state(void* h, const int32_t* x, const int32_t* y, const int32_t* t) {
    Oracle& o = *(Oracle*)h;
    if (x) std::memcpy(o.x.data(), x, o.N * 4);
    if (y) std::memcpy(o.y.data(), y, o.N * 4);
    if (t) std::memcpy(o.t.data(), t, o.N * 4);
}
void orc_get_q(void* h, float* q) { Oracle& o = *(Oracle*)h; std::memcpy(q, o.q.data(), o.q.size() * 4); }
void orc_set_q(void* h, const float* q) { Oracle& o = *(Oracle*)h; std::memcpy(o.q.data(), q, o.q.size() * 4); }
void orc_get_cells(void* h, uint8_t* c) { Oracle& o = *(Oracle*)h; std::memcpy(c, o.cells.data(), o.S); }
int orc_add_obstacle(void* h, int x, int y) {
    Oracle& o = *(Oracle*)h; if (x < 0 || x >= o.W || y < 0 || y >= o.H) return -1;
    o.cells[(int64_t)y * o.W + x] = 1; o.traps.erase((int64_t)y * o.W + x); refresh_fallback(o); return 0;
}
// A trap: an obstacle whose penalty (in (-1, 0)) replaces the step cost of an agent that walks into it (src/kernels.cu:61-63;
// stub at src/environment_bridge.cu:72-78).  Any other penalty leaves a plain obstacle.
int orc_add_trap(void* h, int x, int y, float penalty) {
    Oracle& o = *(Oracle*)h; if (x < 0 || x >= o.W || y < 0 || y >= o.H) return -1;
    const int64_t cell = (int64_t)y * o.W + x;
    o.cells[cell] = 1; o.traps.erase(cell);
    if (penalty < 0.0f && penalty > -1.0f) o.traps[cell] = penalty;
    refresh_fallback(o); return 0;
}
int orc_set_goal(void* h, int x, int y) {
    Oracle& o = *(Oracle*)h; if (x < 0 || x >= o.W || y < 0 || y >= o.H) return -1;
    for (auto& c : o.cells) if (c == 2) c = 0;
    o.cells[(int64_t)y * o.W + x] = 2; o.traps.erase((int64_t)y * o.W + x); refresh_fallback(o); return 0;
}
void orc_get_stats(void* h, cudarl_stats* s) {
    Oracle& o = *(Oracle*)h; std::memset(s, 0, sizeof(*s));
    s->steps = o.step; s->env_steps = o.step * o.N; s->episodes = o.episodes; s->goals = o.goals;
    s->timeouts = o.timeouts; s->conflicts = o.conflicts; s->epsilon = o.eps_last;
    s->reward_sum = (double)o.goals * 1.0 - 0.01 * (double)(s->env_steps - o.goals);
}

// Replica averaging: Q <- (1/R) * (Q_0 + Q_1 + ... + Q_{R-1}), summed in rank order in fp32.
void orc_average_replicas(void** hs, int R) {
    Oracle& o0 = *(Oracle*)hs[0];
    size_t n = o0.q.size(); float inv = 1.0f / (float)R;
    for (size_t k = 0; k < n; ++k) {
        float s = o0.q[k];
        for (int r = 1; r < R; ++r) s += ((Oracle*)hs[r])->q[k];
        s *= inv;
        for (int r = 0; r < R; ++r) ((Oracle*)hs[r])->q[k] = s;
    }
}

}  // extern "C"
