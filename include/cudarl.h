/*
 * cudarl.h -- C ABI of the B200 (sm_100a) batched grid-world + tabular Q-learning path.
 *
 * One context = one GPU = one shard of environments + one Q-table replica.
 * Every entry point takes plain pointers and sizes; nothing here throws, and
 * nothing here knows about Python, PyTorch or C++ containers.  The C++ facade
 * classes (Environment, EnvironmentBridge, CudaQLearning) and the pybind11
 * module `cudarl_core` are thin layers over exactly these calls.
 *
 * Each declaration cites the interface of life423/CudaRL-Arena it stands in for
 * (paths relative to that project's root).
 *
 * Return value of every `int` function: 0 = ok, <0 = bad argument / bad state,
 * >0 = CUDA (1000+cudaError) or NCCL (2000+ncclResult) failure, or CUDARL_ERR_DEVICE + bits when a
 * kernel of this library recorded an internal failure (see CUDARL_DEVERR_*; reported by the next call
 * that waits for the device: cudarl_synchronize, cudarl_get_stats, cudarl_get_q, cudarl_get_state).
 * A text for the last failure is kept per context (cudarl_last_error) and per thread for
 * failures of cudarl_create (cudarl_last_global_error).
 *
 * Threading: one context is single-threaded; different contexts may be used
 * from different threads.  All work of a context is ordered on its own stream.
 */
#ifndef CUDARL_H
#define CUDARL_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library itself is built with -fvisibility=hidden */
#endif

#define CUDARL_ACTIONS 4 /* 0=up(y-1) 1=right(x+1) 2=down(y+1) 3=left(x-1): src/environment.cu:19-27 */

enum { CUDARL_OBST_NONE = 0, CUDARL_OBST_BERNOULLI = 1, CUDARL_OBST_WALLS = 2 };
enum { CUDARL_GOAL_TOP_RIGHT = 0, /* (W-1,0): src/environment.cu:43 */
       CUDARL_GOAL_LIST = 1,      /* explicit cells in goal_xy */
       CUDARL_GOAL_SEEDED = 2 };  /* num_goals cells drawn from the seed among free cells */
enum { CUDARL_START_CENTRE = 0,   /* (W/2,H/2): src/environment.cu:9-10 */
       CUDARL_START_FIXED = 1,    /* (start_x,start_y) */
       CUDARL_START_RANDOM = 2 }; /* uniform free non-goal cell per (env, episode) */
enum { CUDARL_EPS_FIXED = 0,
       CUDARL_EPS_MULT_PER_STEP = 1,    /* eps *= eps_decay after every update: src/train.py:141 */
       CUDARL_EPS_MULT_PER_EPISODE = 2, /* eps0 * eps_decay^(episodes finished / envs) */
       CUDARL_EPS_LINEAR = 3 };         /* eps0 -> eps_end linearly over eps_steps steps, then eps_end */
enum { CUDARL_QINIT_ZERO = 0,           /* src/q_learning.cu:13 */
       CUDARL_QINIT_UNIFORM = 1 };      /* U[0, q_init_scale) from the seed */

#define CUDARL_MAX_GOALS 64

/* Failures recorded by kernels (sticky bits, also in cudarl_stats.device_error). */
#define CUDARL_ERR_DEVICE 3000
enum { CUDARL_DEVERR_SCRATCH_OVERFLOW = 1, /* a work area was too small for the step */
       CUDARL_DEVERR_BAD_STATE = 2,        /* a record outside its tile or outside the grid */
       CUDARL_DEVERR_CHAIN_CYCLE = 8,      /* update_batch: a collision chain longer than the batch */
       CUDARL_DEVERR_COPY_TIMEOUT = 32 };  /* train step: a tile copy did not land within its wait bound */

typedef struct cudarl_config {
    uint32_t struct_size;   /* = sizeof(cudarl_config); checked */
    int32_t  device;        /* CUDA device ordinal */
    int32_t  width, height; /* grid; cell index = y*width + x (src/kernels.cu:30) */
    int64_t  num_envs;      /* environments held by THIS context */
    int64_t  env_offset;    /* global index of local env 0 (rank * num_envs); keys the random streams */
    uint64_t seed;
    int32_t  obstacle_kind;
    float    obstacle_p;    /* Bernoulli probability, or target obstacle fraction for walls */
    int32_t  goal_mode;
    int32_t  num_goals;     /* for LIST and SEEDED, 1..CUDARL_MAX_GOALS */
    int32_t  goal_xy[2 * CUDARL_MAX_GOALS]; /* LIST: x0,y0,x1,y1,... */
    int32_t  start_mode;
    int32_t  start_x, start_y;
    int32_t  max_steps;     /* episode cap (auto-reset after this many steps); 0 = none; at most 16,777,214 -- an episode's step count is kept in 24 bits and saturates there when there is no cap */
    float    lr, gamma;
    int32_t  eps_kind;
    int32_t  reserved0;
    double   eps0, eps_decay, eps_end; /* schedule in double as in src/train.py:45,141; cast to float per step */
    int64_t  eps_steps;
    int32_t  q_init_kind;
    float    q_init_scale;
    int32_t  legacy_clamp;  /* 1: max_next = max(0, max_a' Q) as in src/kernels.cu:102-110 */
    int32_t  sync_every;    /* average the replicas every this many train steps; 0 = never */
    int32_t  rebucket_every;/* re-size the per-tile record regions every this many train steps (0 = default 256, <0 = only when
                               training starts); results never depend on it */
    int32_t  tile_edge;     /* tile edge of the train step in cells: 0 = chosen from the population density, or 8 / 16;
                               results never depend on it */
    int32_t  avg_over_nccl; /* 1: the replica averaging always moves its slices by NCCL send / receive, never over IPC-mapped
                               peer memory (same results; must be the same on every rank) */
    int32_t  reserved[1];
} cudarl_config;

typedef struct cudarl_stats {
    int64_t steps;       /* batched steps taken by cudarl_train_steps since creation */
    int64_t env_steps;   /* steps * num_envs */
    int64_t episodes;    /* episodes finished (goal or cap) */
    int64_t goals;       /* episodes that ended on a goal cell */
    int64_t timeouts;    /* episodes that ended on the step cap */
    int64_t conflicts;   /* environment-steps that shared their cell with another environment */
    int64_t long_chains; /* (cell, step) pairs with more than 24 environments on the cell */
    int64_t chained;     /* environment-steps spent on such crowded cells */
    double  reward_sum;  /* goals * 1.0 - 0.01 * (env_steps - goals), derived from the counters */
    float   epsilon;     /* epsilon used by the most recent train step */
    int32_t device_error;/* nonzero if a kernel recorded an internal limit or bounds violation */
} cudarl_stats;

typedef struct cudarl_eval_stats {
    int64_t envs;        /* environments rolled out */
    int64_t reached;     /* reached a goal within max_steps */
    int64_t total_steps; /* sum of episode lengths */
    double  reward_sum;  /* sum of episode returns */
} cudarl_eval_stats;

typedef struct cudarl_ctx cudarl_ctx;

/* Fill a config with the reference defaults: 10x10, one env, goal top-right, start centre,
 * lr 0.1, gamma 0.99, eps 1.0 * 0.995 per step (src/environment.h:19, src/train.py:43-45). */
void cudarl_default_config(cudarl_config* cfg);

/* Environment::Environment (src/environment.cu:50-77) + CudaQLearning::CudaQLearning
 * (src/q_learning.cu:6-94): allocates every device buffer of the shard, builds the grid from the
 * seed, zero/seed-initialises Q and places the environments (same as cudarl_reset_all). */
int  cudarl_create(const cudarl_config* cfg, cudarl_ctx** out);
/* Environment::~Environment (src/environment.cu:79-100), CudaQLearning::~CudaQLearning (:96-106). */
void cudarl_destroy(cudarl_ctx* ctx);
const char* cudarl_last_error(const cudarl_ctx* ctx);
const char* cudarl_last_global_error(void);

/* Environment::reset (src/environment.cu:102-111) for every environment of the shard; with
 * CUDARL_START_RANDOM each environment gets a fresh seeded free cell.  Episode step counters -> 0. */
int cudarl_reset_all(cudarl_ctx* ctx);

/* Environment::step (src/environment.cu:113-125) with the obstacle/goal lookup of
 * step_environment_kernel (src/kernels.cu:13-66), for all environments at once, actions given
 * by the caller.  Done is sticky and there is no auto-reset, as in the reference class.
 * Host-buffer form: actions[num_envs] in, rewards[num_envs] / dones[num_envs] out (may be NULL). */
int cudarl_step_actions(cudarl_ctx* ctx, const int32_t* actions, float* rewards, uint8_t* dones);
/* Same with device pointers (no copies, returns after enqueueing on the context's stream). */
int cudarl_step_actions_device(cudarl_ctx* ctx, const int32_t* d_actions, float* d_rewards, uint8_t* d_dones);

/* The fused hot path: n batched steps of
 *   epsilon-greedy (src/train.py:86-108) -> step (src/environment.cu:17-48 + src/kernels.cu:29-44,56-59)
 *   -> TD update (src/kernels.cu:96-114 with the true max of src/gpu/kernels.cu:36-45)
 *   -> auto-reset (src/train.py:191-222) -> epsilon decay (src/train.py:141),
 * i.e. the body of the loop at src/train.py:198-222 for all environments, n times, on the device.
 * Replicas are averaged every cfg.sync_every steps when a communicator is attached. */
int cudarl_train_steps(cudarl_ctx* ctx, int64_t n);
/* Same, epsilon for each of the n steps read from a caller array in host memory (pinned or not);
 * this is the form whose inputs arrive from the host every call. */
int cudarl_train_steps_eps(cudarl_ctx* ctx, int64_t n, const float* eps_host);
/* Wait for everything enqueued on the context's stream; reports a failure recorded by a kernel. */
int cudarl_synchronize(cudarl_ctx* ctx);
/* Test hook, no counterpart in the reference: with polls > 0 every warp of the train step first waits for its
 * tile barrier for `polls` tries BEFORE any copy has been issued -- a wait nothing can complete, so it runs
 * out: the warp records CUDARL_DEVERR_COPY_TIMEOUT and leaves, which is what it does when a copy never
 * arrives within the normal bound (two seconds of wall time), exercised without any fault.  0 = normal operation. */
int cudarl_debug_set_copy_wait_polls(cudarl_ctx* ctx, int32_t polls);

/* When on, cudarl_train_steps records the action, reward and done flag of the LAST step of each
 * call for every environment (the per-step data the reference loop sees at src/train.py:200-201). */
int cudarl_set_trace(cudarl_ctx* ctx, int on);
int cudarl_get_trace(cudarl_ctx* ctx, int32_t* actions, float* rewards, uint8_t* dones);

/* evaluate() of src/train.py:262-311 for every environment: reset, then greedy steps (no
 * exploration, no update) until a goal or max_steps.  Training state is left untouched. */
int cudarl_eval_rollout(cudarl_ctx* ctx, int32_t max_steps, cudarl_eval_stats* out);

/* CudaQLearning::update_batch (src/q_learning.cu:108-174): n transitions in structure-of-arrays
 * host buffers.  All targets are computed from the table as it was before the call; updates of
 * one (state, action) are applied in ascending transition index.  No batch-size cap. */
int cudarl_update_batch(cudarl_ctx* ctx, int64_t n,
                        const int32_t* state_x, const int32_t* state_y, const int32_t* actions,
                        const float* rewards, const int32_t* next_x, const int32_t* next_y,
                        const uint8_t* dones);

/* No counterpart in the reference.  The same batched TD update for callers that cannot allocate
 * device memory at call time (a real-time loop that must not block in the allocator, a plug-in whose
 * host framework owns the device heap, a process at its memory cap): nothing in this call allocates
 * or frees.  All arrays are DEVICE pointers owned by the caller -- d_q is the table in the layout
 * (y*width + x)*4 + a (16-byte aligned), updated in place; the transition arrays hold n elements.
 * The kernels' working memory is one fixed static device array inside the library, which limits n to
 * CUDARL_STATIC_MAX_BATCH (larger n returns -5 and launches nothing).  Every call on a GPU shares
 * that array: calls that could overlap on the GPU must be serialised by the caller.  The first call
 * on each device looks up the array's device address; make that call outside stream capture.
 * Asynchronous on `stream` (a cudaStream_t, NULL = default stream).  A transition whose state, next state or action is
 * out of range is skipped without a report; a table pointer that is not 16-byte aligned, or an int32 / float array that
 * is not 4-byte aligned, returns -1 and launches nothing. */
#define CUDARL_STATIC_MAX_BATCH 65536
int cudarl_update_batch_static(float* d_q, int32_t width, int32_t height, int64_t n,
                               const int32_t* d_state_x, const int32_t* d_state_y, const int32_t* d_actions,
                               const float* d_rewards, const int32_t* d_next_x, const int32_t* d_next_y,
                               const uint8_t* d_dones, float lr, float gamma, int32_t legacy_clamp, void* stream);

/* Environment::getAgentX/getAgentY (src/environment.h:27-28) for all environments, plus the
 * per-episode step counters.  Any pointer may be NULL.  cudarl_set_state refuses positions outside the grid and
 * step counters outside 0 .. 16,777,214 ("Invalid state"). */
int cudarl_get_state(cudarl_ctx* ctx, int32_t* x, int32_t* y, int32_t* t);
int cudarl_set_state(cudarl_ctx* ctx, const int32_t* x, const int32_t* y, const int32_t* t);
/* Environment::getReward / isDone (src/environment.h:29-30) after cudarl_step_actions. */
int cudarl_get_reward_done(cudarl_ctx* ctx, float* rewards, uint8_t* dones);

/* CudaQLearning::get_q_table / set_q_table (src/q_learning.cu:176-189):
 * width*height*4 floats, index (y*width + x)*4 + a. */
int cudarl_get_q(cudarl_ctx* ctx, float* q);
int cudarl_set_q(cudarl_ctx* ctx, const float* q);

/* Environment::getGrid (src/environment.cu:134-136) as cell classes: cells[y*width+x] =
 * 0 free, 1 obstacle, 2 goal.  The float grid of the reference is derived from it by the facade. */
int cudarl_get_cells(cudarl_ctx* ctx, uint8_t* cells);
/* EnvironmentBridge::addObstacle / setGoal (src/environment_bridge.cu:53-70; print-only there). */
int cudarl_add_obstacle(cudarl_ctx* ctx, int32_t x, int32_t y);
int cudarl_set_goal(cudarl_ctx* ctx, int32_t x, int32_t y);
/* EnvironmentBridge::addTrap (src/environment_bridge.cu:72-78; print-only there) with the rule of
 * step_environment_kernel (src/kernels.cu:29-36,61-63): the cell becomes an obstacle, and an agent that
 * walks into it stays where it is and receives `penalty` instead of the step cost -- in cudarl_step_actions
 * and in the fused train step alike (the TD target of that (state, action) uses the penalty as its reward).
 * Only penalties in (-1, 0) make a trap, as in the reference; any other value leaves a plain obstacle.
 * Kept on the device as a sparse table {cell, penalty} sorted by cell beside the cell classes.
 * cudarl_stats.reward_sum is derived from the goal and step counters and does not include trap penalties. */
int cudarl_add_trap(cudarl_ctx* ctx, int32_t x, int32_t y, float penalty);
/* The traps set so far, ascending by cell (y*width + x): at most `capacity` entries are written, *count
 * receives how many there are.  cells / penalties may be NULL. */
int cudarl_get_traps(cudarl_ctx* ctx, int32_t capacity, int32_t* cells, float* penalties, int32_t* count);

/* Switch the max(0, .) clamp of the flat reference kernel (src/kernels.cu:102-110) on or off. */
int cudarl_set_legacy_clamp(cudarl_ctx* ctx, int on);

int cudarl_get_stats(cudarl_ctx* ctx, cudarl_stats* out);
int cudarl_get_config(const cudarl_ctx* ctx, cudarl_config* out);

/* Replica averaging across GPUs, one process per GPU (no counterpart in the reference, which is
 * single-GPU).  The 128-byte id is made on one rank and handed to the others by the caller. */
#define CUDARL_COMM_ID_BYTES 128
int cudarl_comm_unique_id(void* id128);
int cudarl_comm_init(cudarl_ctx* ctx, const void* id128, int32_t rank, int32_t nranks);
int cudarl_average_replicas(cudarl_ctx* ctx);
/* 1 when the averaging works straight on the peers' memory (every rank a process of its own on one NVLink domain: the
 * tables are mapped through CUDA IPC at cudarl_comm_init; one kernel per rank reads its slice of every replica with peer
 * loads, sums in rank order and stores the result into every rank's table; NCCL only carries two one-word barriers);
 * 0 when the slices travel by NCCL send / receive and all-gather instead (chosen by all ranks together when any mapping
 * fails, or with avg_over_nccl); the results are the same bits either way. */
int cudarl_comm_peer_memory(const cudarl_ctx* ctx);

/* Timing helpers for benchmarks: record events on the context's stream. */
int cudarl_timer_start(cudarl_ctx* ctx);
int cudarl_timer_stop_ms(cudarl_ctx* ctx, float* ms); /* synchronises */
/* When enabled, every uninterrupted run of step-kernel launches (k_tile_step, back to back; a run ends where the
 * record regions are re-sized, the replicas are averaged or the call returns) is bracketed by ONE pair of events:
 * step_ms = summed time of those runs, launches = step kernels inside them.  Used for the roofline figure. */
int cudarl_kernel_timing(cudarl_ctx* ctx, int on);
int cudarl_kernel_time_ms(cudarl_ctx* ctx, float* step_ms, int64_t* launches);

const char* cudarl_version(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* CUDARL_H */
