// facade.cpp -- Environment / EnvironmentBridge / CudaQLearning of the reference over the C ABI.
#include "facade.h"
#include "../../include/cudarl.h"
#include <sstream>
#include <stdexcept>

namespace {
void check(int rc, cudarl_ctx* ctx, const char* what) {
    if (rc == 0) return;
    std::string m = ctx ? cudarl_last_error(ctx) : cudarl_last_global_error();
    throw std::runtime_error(m.empty() ? std::string(what) : m);
}
}

// ---- Environment -------------------------------------------------------------------------------
Environment::Environment(int id, int width, int height) : env_id_(id), width_(width), height_(height) {
    cudarl_config cfg;
    cudarl_default_config(&cfg);
    cfg.width = width; cfg.height = height; cfg.num_envs = 1; cfg.env_offset = id >= 0 ? id : 0;
    check(cudarl_create(&cfg, &ctx_), nullptr, "cudarl_create failed");
    x_ = width / 2; y_ = height / 2;          // src/environment.cu:54-55
    refresh_grid();
}
Environment::~Environment() { if (ctx_) cudarl_destroy(ctx_); }
Environment::Environment(Environment&& o) noexcept { *this = std::move(o); }
Environment& Environment::operator=(Environment&& o) noexcept {
    if (this != &o) {
        if (ctx_) cudarl_destroy(ctx_);
        env_id_ = o.env_id_; width_ = o.width_; height_ = o.height_; x_ = o.x_; y_ = o.y_;
        reward_ = o.reward_; done_ = o.done_; ctx_ = o.ctx_; grid_ = std::move(o.grid_);
        o.ctx_ = nullptr;
    }
    return *this;
}

void Environment::refresh_grid() {
    std::vector<uint8_t> cells((size_t)width_ * height_);
    check(cudarl_get_cells(ctx_, cells.data()), ctx_, "get_cells");
    grid_.assign(cells.size(), 0.0f);
    for (size_t i = 0; i < cells.size(); ++i) grid_[i] = cells[i] == 2 ? 1.0f : (cells[i] == 1 ? -1.0f : 0.0f);
    int32_t nt = 0;
    check(cudarl_get_traps(ctx_, 0, nullptr, nullptr, &nt), ctx_, "get_traps");
    std::vector<int32_t> tc((size_t)nt); std::vector<float> tpn((size_t)nt);
    if (nt) check(cudarl_get_traps(ctx_, nt, tc.data(), tpn.data(), &nt), ctx_, "get_traps");
    for (int32_t k = 0; k < nt; ++k) grid_[(size_t)tc[k]] = tpn[k];      // a trap shows its penalty, as src/kernels.cu:61 reads it
}

void Environment::reset() {
    check(cudarl_reset_all(ctx_), ctx_, "reset");
    int32_t x, y;
    check(cudarl_get_state(ctx_, &x, &y, nullptr), ctx_, "get_state");
    x_ = x; y_ = y; reward_ = 0.0f; done_ = false;
}

void Environment::step(int action) {
    int32_t a = action, x, y; float r; uint8_t d;
    check(cudarl_step_actions(ctx_, &a, &r, &d), ctx_, "step");       // obstacles, goals and traps are looked up on the device
    check(cudarl_get_state(ctx_, &x, &y, nullptr), ctx_, "get_state");
    x_ = x; y_ = y; reward_ = r; done_ = d != 0;
}

float Environment::getCellValue(int x, int y) const {
    if (x >= 0 && x < width_ && y >= 0 && y < height_) return grid_[(size_t)y * width_ + x];
    return 0.0f;
}
std::vector<float> Environment::getGrid() const { return grid_; }

void Environment::addObstacle(int x, int y) { check(cudarl_add_obstacle(ctx_, x, y), ctx_, "add_obstacle"); refresh_grid(); }
void Environment::setGoal(int x, int y) { check(cudarl_set_goal(ctx_, x, y), ctx_, "set_goal"); refresh_grid(); }
void Environment::addTrap(int x, int y, float penalty) { check(cudarl_add_trap(ctx_, x, y, penalty), ctx_, "add_trap"); refresh_grid(); }

// ---- EnvironmentBridge -------------------------------------------------------------------------
EnvironmentBridge::EnvironmentBridge(int width, int height, int env_id) : width(width), height(height) {
    env = std::make_unique<Environment>(env_id, width, height);
}
std::vector<float> EnvironmentBridge::reset() { env->reset(); return getObservation(); }
std::tuple<std::vector<float>, float, bool, std::string> EnvironmentBridge::step(int action) {
    env->step(action);
    std::stringstream info;
    info << "agent_pos: (" << env->getAgentX() << "," << env->getAgentY() << ")";   // src/environment_bridge.cu:30-31
    return std::make_tuple(getObservation(), env->getReward(), env->isDone(), info.str());
}
std::vector<float> EnvironmentBridge::getObservation() const { return env->getGrid(); }
int EnvironmentBridge::getWidth() const { return width; }
int EnvironmentBridge::getHeight() const { return height; }
std::pair<int, int> EnvironmentBridge::getAgentPosition() const { return std::make_pair(env->getAgentX(), env->getAgentY()); }
void EnvironmentBridge::addObstacle(int x, int y) { env->addObstacle(x, y); }
void EnvironmentBridge::setGoal(int x, int y) { env->setGoal(x, y); }
void EnvironmentBridge::addTrap(int x, int y, float penalty) { env->addTrap(x, y, penalty); }

// ---- CudaQLearning -----------------------------------------------------------------------------
CudaQLearning::CudaQLearning(int width, int height, int action_space_size, float learning_rate, float discount_factor)
    : width(width), height(height), action_space_size(action_space_size), learning_rate(learning_rate), discount_factor(discount_factor) {
    if (action_space_size != CUDARL_ACTIONS) throw std::runtime_error("CudaQLearning: action_space_size must be 4 (one float4 row per state)");
    cudarl_config cfg;
    cudarl_default_config(&cfg);
    cfg.width = width; cfg.height = height; cfg.num_envs = 0; cfg.lr = learning_rate; cfg.gamma = discount_factor;
    check(cudarl_create(&cfg, &ctx_), nullptr, "Failed to allocate device memory for Q-table");
    h_q_table.assign((size_t)width * height * action_space_size, 0.0f);    // src/q_learning.cu:13
    dirty_ = false;
}
CudaQLearning::~CudaQLearning() { if (ctx_) cudarl_destroy(ctx_); }

void CudaQLearning::set_legacy_clamp(bool on) { check(cudarl_set_legacy_clamp(ctx_, on ? 1 : 0), ctx_, "set_legacy_clamp"); }

void CudaQLearning::update_batch(const std::vector<std::pair<int, int>>& states, const std::vector<int>& actions,
                                 const std::vector<float>& rewards, const std::vector<std::pair<int, int>>& next_states,
                                 const std::vector<bool>& dones) {
    const size_t n = states.size();
    if (n != actions.size() || n != rewards.size() || n != next_states.size() || n != dones.size())
        throw std::runtime_error("Inconsistent batch sizes");               // src/q_learning.cu:121-124
    std::vector<int32_t> sx(n), sy(n), nx(n), ny(n); std::vector<uint8_t> dn(n);
    for (size_t i = 0; i < n; ++i) {
        sx[i] = states[i].first; sy[i] = states[i].second; nx[i] = next_states[i].first; ny[i] = next_states[i].second; dn[i] = dones[i] ? 1 : 0;
    }
    check(cudarl_update_batch(ctx_, (int64_t)n, sx.data(), sy.data(), actions.data(), rewards.data(), nx.data(), ny.data(), dn.data()),
          ctx_, "update_batch");
    dirty_ = true;
}

void CudaQLearning::refresh() const {
    if (!dirty_) return;
    check(cudarl_get_q(ctx_, h_q_table.data()), ctx_, "get_q");
    dirty_ = false;
}
std::vector<float> CudaQLearning::get_q_table() const { refresh(); return h_q_table; }
void CudaQLearning::set_q_table(const std::vector<float>& q_table) {
    if (q_table.size() != (size_t)width * height * action_space_size) throw std::runtime_error("Invalid Q-table size");   // :181-183
    check(cudarl_set_q(ctx_, q_table.data()), ctx_, "set_q");
    h_q_table = q_table; dirty_ = false;
}
int CudaQLearning::get_best_action(int x, int y) const {
    if (x < 0 || x >= width || y < 0 || y >= height) throw std::runtime_error("Invalid state");                          // :192-194
    refresh();
    size_t base = ((size_t)y * width + x) * action_space_size;
    int best = 0; float bv = h_q_table[base];
    for (int a = 1; a < action_space_size; ++a) if (h_q_table[base + a] > bv) { bv = h_q_table[base + a]; best = a; }
    return best;
}
float CudaQLearning::get_q_value(int x, int y, int action) const {
    if (x < 0 || x >= width || y < 0 || y >= height || action < 0 || action >= action_space_size)
        throw std::runtime_error("Invalid state or action");                                                            // :212-214
    refresh();
    return h_q_table[((size_t)y * width + x) * action_space_size + action];
}
