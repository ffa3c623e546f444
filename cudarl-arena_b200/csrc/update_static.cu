// update_static.cu -- cudarl_update_batch_static: the batched TD update for callers that must not
// allocate device memory.
//
// Who needs it: code that runs inside a region where cudaMalloc / cudaFree are off limits -- a
// real-time control loop that may not block on the allocator, a plug-in running under a host
// framework that owns the device heap and forbids outside allocations, a process that is already
// at its memory cap.  cudarl_update_batch (context form) grows staging, entry and scratch buffers
// on demand; this form never does.  The caller hands in device pointers for the table and the
// transitions; the only other memory the kernels need -- collision entries, chain heads and a sort
// area -- lives in ONE file-scope `static __device__` array of fixed size below, which every GPU
// that loads this library carries until the process exits (CUDARL_STATIC_MAX_BATCH transitions,
// about 2 MiB).
//
// Rules that follow from the shared array:
//   * batches larger than CUDARL_STATIC_MAX_BATCH are rejected (-5), nothing is launched;
//   * all calls on one GPU use the same array and it keeps whatever the previous call left, so
//     the parts that must start at zero (chain heads, sort cursor) are cleared by every call,
//     and two calls that overlap on the GPU (different streams, different host threads) race:
//     run them one after the other;
//   * the first call on each device resolves the array's device address with
//     cudaGetSymbolAddress (in host code the array's name is only a handle, not an address the
//     GPU can use).  That first call per device should therefore be made outside any stream
//     capture.
//
// Semantics are those of cudarl_update_batch: every TD target is computed from the table as it was
// before the call, and updates of one (state, action) are applied one after the other in ascending
// transition index, q <- fma(lr, target - q, q).  The table is the caller's dense layout, (y*width + x)*4 + a, 16-byte aligned.
// Transitions whose state, next state or action is out of range are skipped.
#include "../../include/cudarl.h"
#include <cuda_runtime.h>
#include <cstdint>
#include <mutex>

namespace {

constexpr unsigned MAXB = CUDARL_STATIC_MAX_BATCH;       // transitions per call
constexpr unsigned SLOTS = MAXB;                         // chain heads (power of two)
constexpr unsigned SLOT_SHIFT = 16;                      // 32 - log2(SLOTS)
static_assert((1u << (32 - SLOT_SHIFT)) == SLOTS, "SLOTS must be 2^(32-SLOT_SHIFT)");

// layout of the static scratch (bytes):  [entries uint4 x MAXB][sort keys u64 x MAXB][sort vals f32 x MAXB]
//                                         [heads u32 x SLOTS][cursor u32, error u32, pad]
constexpr size_t OFF_ENT = 0;
constexpr size_t OFF_KEY = OFF_ENT + sizeof(uint4) * MAXB;
constexpr size_t OFF_VAL = OFF_KEY + sizeof(unsigned long long) * MAXB;
constexpr size_t OFF_HEAD = OFF_VAL + sizeof(float) * MAXB;
constexpr size_t OFF_CTL = OFF_HEAD + sizeof(unsigned) * SLOTS;
constexpr size_t SCRATCH_BYTES = OFF_CTL + 256;

static __device__ __align__(256) unsigned char g_static_scratch[SCRATCH_BYTES];

struct Scratch {
    uint4* ent; unsigned long long* key; float* val; unsigned* head; unsigned* ctl;
};
__host__ __device__ inline Scratch carve(unsigned char* base) {
    Scratch s;
    s.ent = reinterpret_cast<uint4*>(base + OFF_ENT);
    s.key = reinterpret_cast<unsigned long long*>(base + OFF_KEY);
    s.val = reinterpret_cast<float*>(base + OFF_VAL);
    s.head = reinterpret_cast<unsigned*>(base + OFF_HEAD);
    s.ctl = reinterpret_cast<unsigned*>(base + OFF_CTL);
    return s;
}

__device__ __forceinline__ unsigned slot_of(unsigned cell) { return (cell * 0x9E3779B1u) >> SLOT_SHIFT; }

__global__ void ks_clear(unsigned char* base) {
    Scratch s = carve(base);
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < SLOTS) s.head[i] = 0u;
    if (i == 0) { s.ctl[0] = 0u; s.ctl[1] = 0u; }
}

// TD error of transition i against the untouched table; link it into its cell's chain.
__global__ void ks_main(unsigned char* base, const float4* q, int W, int H, unsigned n, const int* sx, const int* sy, const int* act,
                        const float* rew, const int* nx, const int* ny, const unsigned char* dn, float gamma, int clamp) {
    Scratch s = carve(base);
    unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    // a transition outside the grid or the action set is skipped (and flagged) instead of read
    if ((unsigned)sx[i] >= (unsigned)W || (unsigned)sy[i] >= (unsigned)H || (unsigned)act[i] >= 4u ||
        (unsigned)nx[i] >= (unsigned)W || (unsigned)ny[i] >= (unsigned)H) { atomicOr(s.ctl + 1, 4u); return; }
    unsigned cell = (unsigned)sy[i] * (unsigned)W + (unsigned)sx[i];
    unsigned a = (unsigned)act[i];
    float m = 0.0f;
    if (!dn[i]) {
        float4 r2 = q[(unsigned)ny[i] * (unsigned)W + (unsigned)nx[i]];
        m = r2.x; m = r2.y > m ? r2.y : m; m = r2.z > m ? r2.z : m; m = r2.w > m ? r2.w : m;
        if (clamp && m < 0.0f) m = 0.0f;
    }
    float d = __fmaf_rn(gamma, m, rew[i]);               // TD target from the untouched table
    unsigned prev = atomicExch(s.head + slot_of(cell), i + 1u);
    s.ent[i] = make_uint4((cell << 2) | a, i, __float_as_uint(d), prev);
}

__device__ void sift_down(unsigned long long* k, float* v, unsigned start, unsigned end) {
    unsigned root = start;
    while (2u * root + 1u < end) {
        unsigned child = 2u * root + 1u;
        if (child + 1u < end && k[child] < k[child + 1u]) ++child;
        if (k[root] >= k[child]) return;
        unsigned long long tk = k[root]; k[root] = k[child]; k[child] = tk;
        float tv = v[root]; v[root] = v[child]; v[child] = tv;
        root = child;
    }
}

// One thread per chain: copy it into a private segment of the sort area, order it by
// (cell, action, transition index), then fold each (cell, action) run into the table.
__global__ void ks_fix(unsigned char* base, float* q, float lr, unsigned n) {
    Scratch s = carve(base);
    unsigned slot = blockIdx.x * blockDim.x + threadIdx.x;
    if (slot >= SLOTS) return;
    unsigned p = s.head[slot];
    if (!p) return;
    unsigned L = 0;
    for (unsigned w = p; w && L <= n; w = s.ent[w - 1u].w) ++L;      // bounded: a chain has at most n links
    if (L > n) { atomicOr(s.ctl + 1, 1u); return; }
    unsigned off = atomicAdd(s.ctl, L);
    if (off + L > MAXB) { atomicOr(s.ctl + 1, 2u); return; }
    unsigned long long* k = s.key + off; float* v = s.val + off;
    unsigned j = 0;
    for (unsigned w = p; w && j < L; ++j) {
        uint4 e = s.ent[w - 1u];
        k[j] = ((unsigned long long)e.x << 32) | e.y; v[j] = __uint_as_float(e.z); w = e.w;
    }
    if (L <= 24) {                                                   // insertion sort
        for (unsigned a = 1; a < L; ++a) {
            unsigned long long kk = k[a]; float vv = v[a]; unsigned b = a;
            while (b > 0 && k[b - 1u] > kk) { k[b] = k[b - 1u]; v[b] = v[b - 1u]; --b; }
            k[b] = kk; v[b] = vv;
        }
    } else {                                                         // heapsort, O(L log L) in place
        for (unsigned st = L / 2u; st-- > 0u;) sift_down(k, v, st, L);
        for (unsigned end = L - 1u; end > 0u; --end) {
            unsigned long long tk = k[0]; k[0] = k[end]; k[end] = tk;
            float tv = v[0]; v[0] = v[end]; v[end] = tv;
            sift_down(k, v, 0u, end);
        }
    }
    unsigned cur = 0xFFFFFFFFu; float acc = 0.0f;
    for (j = 0; j < L; ++j) {
        unsigned qi = (unsigned)(k[j] >> 32);                        // (cell << 2) | action == index into the dense table
        if (qi != cur) { if (cur != 0xFFFFFFFFu) q[cur] = acc; cur = qi; acc = q[qi]; }
        acc = __fmaf_rn(lr, __fsub_rn(v[j], acc), acc);     // each update sees the value the previous one left
    }
    if (cur != 0xFFFFFFFFu) q[cur] = acc;
}

// device address of the static array, resolved once per device
constexpr int MAX_DEVICES = 64;
unsigned char* g_addr[MAX_DEVICES];
bool g_ready[MAX_DEVICES];
std::mutex g_mu;

}  // namespace

extern "C" int cudarl_update_batch_static(float* d_q, int32_t width, int32_t height, int64_t n,
                                          const int32_t* d_sx, const int32_t* d_sy, const int32_t* d_actions,
                                          const float* d_rewards, const int32_t* d_nx, const int32_t* d_ny,
                                          const uint8_t* d_dones, float lr, float gamma, int32_t legacy_clamp,
                                          void* stream) {
    if (n < 0 || width < 1 || height < 1 || (int64_t)width * height >= (1ll << 30)) return -1;
    if (n > (int64_t)MAXB) return -5;                   // larger than the static scratch: refuse, launch nothing
    if (n == 0) return 0;
    if (!d_q || !d_sx || !d_sy || !d_actions || !d_rewards || !d_nx || !d_ny || !d_dones) return -1;
    // the kernels read the table as 16-byte rows and the other arrays as 4-byte words: a misaligned pointer would be a device fault
    if ((reinterpret_cast<uintptr_t>(d_q) & 15u) || ((reinterpret_cast<uintptr_t>(d_sx) | reinterpret_cast<uintptr_t>(d_sy) |
         reinterpret_cast<uintptr_t>(d_actions) | reinterpret_cast<uintptr_t>(d_rewards) | reinterpret_cast<uintptr_t>(d_nx) |
         reinterpret_cast<uintptr_t>(d_ny)) & 3u)) return -1;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return 1000 + (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return -1;
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_ready[dev]) {
            // In host code `g_static_scratch` is a stand-in for the symbol; its device address on the
            // CURRENT device has to be asked for.
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess) return 1000 + (int)e;
            g_addr[dev] = static_cast<unsigned char*>(ptr);
            g_ready[dev] = true;
        }
        base = g_addr[dev];
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned un = (unsigned)n;
    ks_clear<<<SLOTS / 256, 256, 0, st>>>(base);
    ks_main<<<(un + 255u) / 256u, 256, 0, st>>>(base, reinterpret_cast<const float4*>(d_q), width, height, un, d_sx, d_sy, d_actions,
                                                 d_rewards, d_nx, d_ny, d_dones, gamma, legacy_clamp);
    ks_fix<<<SLOTS / 256, 256, 0, st>>>(base, d_q, lr, un);
    e = cudaGetLastError();
    return e == cudaSuccess ? 0 : 1000 + (int)e;
}
