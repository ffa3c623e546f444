// facade.h -- the reference's C++ classes, same names / signatures / error behaviour, as thin
// wrappers over the C ABI of include/cudarl.h.  A program written against the reference's
// src/environment.h, src/environment_bridge.h and src/q_learning.cuh compiles against this header
// unchanged and links libcudarl.so instead of the reference's static library.
//
//   Environment        src/environment.h:17-47       (ctor args: id, width, height)
//   EnvironmentBridge  src/environment_bridge.h:10-80
//   CudaQLearning      src/q_learning.cuh:8-95
//
// Differences on purpose: no per-call printing to stdout (src/environment.cu:76,99,110,121-124 print
// a line per call, which dominates the reference's step time); update_batch has no 1024 cap;
// addObstacle / setGoal / addTrap really edit the grid (print-only stubs at
// src/environment_bridge.cu:53-78); CUDA failures throw std::runtime_error as in the refactored
// tree (src/core/cuda_utils.h:11-19).
#pragma once
#include <memory>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

#if defined(__GNUC__)
#define CUDARL_CXX_API __attribute__((visibility("default")))
#else
#define CUDARL_CXX_API
#endif

struct cudarl_ctx;

class CUDARL_CXX_API Environment {
public:
    Environment(int id = 0, int width = 10, int height = 10);
    ~Environment();
    Environment(const Environment&) = delete;
    Environment& operator=(const Environment&) = delete;
    Environment(Environment&&) noexcept;
    Environment& operator=(Environment&&) noexcept;

    void reset();
    void step(int action);

    int getWidth() const { return width_; }
    int getHeight() const { return height_; }
    int getAgentX() const { return x_; }
    int getAgentY() const { return y_; }
    float getReward() const { return reward_; }
    bool isDone() const { return done_; }
    float getCellValue(int x, int y) const;     // 0.0 outside the grid (src/environment.cu:127-132)
    std::vector<float> getGrid() const;         // free 0.0, goal 1.0, obstacle -1.0, trap = its penalty

    // grid edits used by EnvironmentBridge
    void addObstacle(int x, int y);
    void setGoal(int x, int y);
    void addTrap(int x, int y, float penalty);
    int getId() const { return env_id_; }

private:
    void refresh_grid();
    int env_id_, width_, height_;
    int x_ = 0, y_ = 0;
    float reward_ = 0.0f;
    bool done_ = false;
    cudarl_ctx* ctx_ = nullptr;
    std::vector<float> grid_;                   // host copy of the float view of the cell classes and traps
};

class CUDARL_CXX_API EnvironmentBridge {
public:
    EnvironmentBridge(int width = 10, int height = 10, int env_id = 0);   // env_id: third argument of the reference's second binding (src/bindings/python_bindings.cpp:55-81)
    std::vector<float> reset();
    std::tuple<std::vector<float>, float, bool, std::string> step(int action);
    std::vector<float> getObservation() const;
    int getWidth() const;
    int getHeight() const;
    std::pair<int, int> getAgentPosition() const;
    void addObstacle(int x, int y);
    void setGoal(int x, int y);
    void addTrap(int x, int y, float penalty = -1.0f);
    // the duck type python/cudarl/environment.py:62-69,89 of the reference expects from its backend
    int getEnvId() const { return env->getId(); }
    float getReward() const { return env->getReward(); }
    bool isDone() const { return env->isDone(); }
private:
    std::unique_ptr<Environment> env;
    int width;
    int height;
};

class CUDARL_CXX_API CudaQLearning {
public:
    CudaQLearning(int width, int height, int action_space_size, float learning_rate = 0.1f, float discount_factor = 0.99f);
    ~CudaQLearning();
    CudaQLearning(const CudaQLearning&) = delete;
    CudaQLearning& operator=(const CudaQLearning&) = delete;

    void update_batch(const std::vector<std::pair<int, int>>& states, const std::vector<int>& actions,
                      const std::vector<float>& rewards, const std::vector<std::pair<int, int>>& next_states,
                      const std::vector<bool>& dones);
    std::vector<float> get_q_table() const;
    void set_q_table(const std::vector<float>& q_table);
    int get_best_action(int x, int y) const;
    float get_q_value(int x, int y, int action) const;
    // opt-in: max_next = max(0, max Q) exactly as the flat reference kernel (src/kernels.cu:102-110)
    void set_legacy_clamp(bool on);

private:
    void refresh() const;
    int width, height, action_space_size;
    float learning_rate, discount_factor;
    cudarl_ctx* ctx_ = nullptr;
    mutable std::vector<float> h_q_table;
    mutable bool dirty_ = true;
};
