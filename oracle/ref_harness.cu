// ref_harness.cu -- TEST INFRASTRUCTURE.  Launches the reference's OWN kernels on raw buffers so that
// the GPU tests can cross-check this library against the real thing:
//   step_environment          src/environment.cu:17-48      (the step the reference actually runs)
//   step_environment_kernel   src/kernels.cu:13-66          (obstacle / goal / trap aware, never launched upstream)
//   update_q_values_kernel    src/kernels.cu:68-116         (flat tree TD update, max clamped at 0)
//   cudarl::updateQValuesKernel  src/gpu/kernels.cu:7-54    (refactored tree TD update, true max)
// The reference sources are compiled from where they lie (include path given on the command line by
// cudarl-arena_b200/build.py: -I<reference>/src); nothing of them is copied into this repository.
// CudaQLearning::update_batch itself does not compile with libstdc++ (src/q_learning.cu:146 calls
// std::vector<bool>::data()), so the kernels are driven directly with device buffers.
#include <cuda_runtime.h>
#include <cstdint>
#include <vector>
#include "kernels.cu"        // reference: reset_environment_kernel, step_environment_kernel, update_q_values_kernel
#include "environment.cu"    // reference: reset_environment, step_environment, class Environment
#include "gpu/kernels.cu"    // reference: cudarl::updateQValuesKernel

#define RCK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) return 1000 + (int)e_; } while (0)

extern "C" __attribute__((visibility("default")))
int ref_walk(int which, int W, int H, const float* grid, int x0, int y0, int n, const int* actions,
             int* xs, int* ys, float* rewards, uint8_t* dones) {
    float* d_grid = nullptr; EnvironmentState* d_state = nullptr;
    RCK(cudaMalloc(&d_grid, sizeof(float) * W * H));
    RCK(cudaMemcpy(d_grid, grid, sizeof(float) * W * H, cudaMemcpyHostToDevice));
    EnvironmentState h; h.width = W; h.height = H; h.grid = d_grid; h.agent_x = x0; h.agent_y = y0; h.reward = 0.0f; h.done = false;
    RCK(cudaMalloc(&d_state, sizeof(h)));
    RCK(cudaMemcpy(d_state, &h, sizeof(h), cudaMemcpyHostToDevice));
    for (int i = 0; i < n; ++i) {
        if (which == 0) step_environment<<<1, 1>>>(d_state, actions[i]);
        else step_environment_kernel<<<1, 1>>>(d_state, actions[i]);
        RCK(cudaDeviceSynchronize());
        RCK(cudaMemcpy(&h, d_state, sizeof(h), cudaMemcpyDeviceToHost));
        xs[i] = h.agent_x; ys[i] = h.agent_y; rewards[i] = h.reward; dones[i] = h.done ? 1 : 0;
    }
    cudaFree(d_state); cudaFree(d_grid);
    return 0;
}

extern "C" __attribute__((visibility("default")))
int ref_update(int which, float* q, int W, int H, int n, const int* sx, const int* sy, const int* a, const float* r,
               const int* nx, const int* ny, const uint8_t* dn, float lr, float gamma) {
    float* d_q; int *d_sx, *d_sy, *d_a, *d_nx, *d_ny; float* d_r; bool* d_dn;
    size_t qb = sizeof(float) * W * H * 4;
    RCK(cudaMalloc(&d_q, qb)); RCK(cudaMemcpy(d_q, q, qb, cudaMemcpyHostToDevice));
    std::vector<int> s1(n), s2(n); std::vector<uint8_t> b(n);
    for (int i = 0; i < n; ++i) { s1[i] = sy[i] * W + sx[i]; s2[i] = ny[i] * W + nx[i]; b[i] = dn[i] ? 1 : 0; }
    RCK(cudaMalloc(&d_sx, 4 * n)); RCK(cudaMalloc(&d_sy, 4 * n)); RCK(cudaMalloc(&d_a, 4 * n)); RCK(cudaMalloc(&d_r, 4 * n));
    RCK(cudaMalloc(&d_nx, 4 * n)); RCK(cudaMalloc(&d_ny, 4 * n)); RCK(cudaMalloc(&d_dn, n));
    RCK(cudaMemcpy(d_a, a, 4 * n, cudaMemcpyHostToDevice)); RCK(cudaMemcpy(d_r, r, 4 * n, cudaMemcpyHostToDevice));
    RCK(cudaMemcpy(d_dn, b.data(), n, cudaMemcpyHostToDevice));
    int blocks = (n + 255) / 256;
    if (which == 0) {
        RCK(cudaMemcpy(d_sx, sx, 4 * n, cudaMemcpyHostToDevice)); RCK(cudaMemcpy(d_sy, sy, 4 * n, cudaMemcpyHostToDevice));
        RCK(cudaMemcpy(d_nx, nx, 4 * n, cudaMemcpyHostToDevice)); RCK(cudaMemcpy(d_ny, ny, 4 * n, cudaMemcpyHostToDevice));
        update_q_values_kernel<<<blocks, 256>>>(d_q, d_sx, d_sy, d_a, d_r, d_nx, d_ny, d_dn, n, W, H, 4, lr, gamma);
    } else {
        RCK(cudaMemcpy(d_sx, s1.data(), 4 * n, cudaMemcpyHostToDevice)); RCK(cudaMemcpy(d_nx, s2.data(), 4 * n, cudaMemcpyHostToDevice));
        cudarl::updateQValuesKernel<<<blocks, 256>>>(d_q, d_sx, d_a, d_r, d_nx, d_dn, W * H, 4, lr, gamma, n);
    }
    RCK(cudaDeviceSynchronize());
    RCK(cudaMemcpy(q, d_q, qb, cudaMemcpyDeviceToHost));
    cudaFree(d_q); cudaFree(d_sx); cudaFree(d_sy); cudaFree(d_a); cudaFree(d_r); cudaFree(d_nx); cudaFree(d_ny); cudaFree(d_dn);
    return 0;
}
