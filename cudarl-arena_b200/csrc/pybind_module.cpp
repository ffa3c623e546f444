// pybind_module.cpp -- Python module `cudarl_core` with the reference's surface
// (src/python_bindings.cpp:8-26): class Environment = EnvironmentBridge with reset / step /
// get_observation / get_width / get_height / get_agent_position / add_obstacle / set_goal / add_trap
// and __version__ == "0.1.0".  Additions that do not change that surface:
//   * the property / method aliases of the reference's second binding (src/bindings/python_bindings.cpp:67-81)
//     and of the backend duck type of python/cudarl/environment.py:62-69,89;
//   * CudaQLearning (never bound by the reference);
//   * VecEnvironment: the batched fused path (train_steps, eval_rollout, ...) with NumPy arrays.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <cstring>
#include <stdexcept>
#include "../../include/cudarl.h"
#include "facade.h"

namespace py = pybind11;

namespace {

class VecEnvironment {
public:
    explicit VecEnvironment(const py::dict& kw) {
        cudarl_default_config(&cfg_);
        for (auto item : kw) {
            std::string k = py::cast<std::string>(item.first);
            py::handle v = item.second;
#define F(name, type) if (k == #name) { cfg_.name = py::cast<type>(v); continue; }
            F(device, int) F(width, int) F(height, int) F(num_envs, long long) F(env_offset, long long) F(seed, unsigned long long)
            F(obstacle_kind, int) F(obstacle_p, float) F(goal_mode, int) F(num_goals, int) F(start_mode, int) F(start_x, int) F(start_y, int)
            F(max_steps, int) F(lr, float) F(gamma, float) F(eps_kind, int) F(eps0, double) F(eps_decay, double) F(eps_end, double)
            F(eps_steps, long long) F(q_init_kind, int) F(q_init_scale, float) F(legacy_clamp, int) F(sync_every, int)
            F(rebucket_every, int) F(tile_edge, int) F(avg_over_nccl, int)
#undef F
            if (k == "goals") {
                auto lst = py::cast<std::vector<std::pair<int, int>>>(v);
                if (lst.size() > CUDARL_MAX_GOALS) throw std::runtime_error("too many goals");
                cfg_.goal_mode = CUDARL_GOAL_LIST; cfg_.num_goals = (int)lst.size();
                for (size_t i = 0; i < lst.size(); ++i) { cfg_.goal_xy[2 * i] = lst[i].first; cfg_.goal_xy[2 * i + 1] = lst[i].second; }
                continue;
            }
            throw std::runtime_error("unknown configuration key: " + k);
        }
        if (cudarl_create(&cfg_, &ctx_) != 0) throw std::runtime_error(cudarl_last_global_error());
    }
    ~VecEnvironment() { if (ctx_) cudarl_destroy(ctx_); }
    VecEnvironment(const VecEnvironment&) = delete;

    void ck(int rc) const { if (rc) throw std::runtime_error(cudarl_last_error(ctx_)); }
    size_t n() const { return (size_t)cfg_.num_envs; }
    void reset() { ck(cudarl_reset_all(ctx_)); }
    py::tuple step(py::array_t<int32_t, py::array::c_style | py::array::forcecast> actions) {
        if ((size_t)actions.size() != n()) throw std::runtime_error("actions must have num_envs entries");
        py::array_t<float> r(n()); py::array_t<uint8_t> d(n());
        { py::gil_scoped_release rel; ck(cudarl_step_actions(ctx_, actions.data(), r.mutable_data(), d.mutable_data())); }
        return py::make_tuple(r, d);
    }
    void train_steps(long long k) { py::gil_scoped_release rel; ck(cudarl_train_steps(ctx_, k)); ck(cudarl_synchronize(ctx_)); }
    py::dict eval_rollout(int max_steps) {
        cudarl_eval_stats s; { py::gil_scoped_release rel; ck(cudarl_eval_rollout(ctx_, max_steps, &s)); }
        py::dict o; o["envs"] = s.envs; o["reached"] = s.reached; o["total_steps"] = s.total_steps; o["reward_sum"] = s.reward_sum;
        return o;
    }
    py::tuple positions() {
        py::array_t<int32_t> x(n()), y(n()), t(n());
        ck(cudarl_get_state(ctx_, x.mutable_data(), y.mutable_data(), t.mutable_data()));
        return py::make_tuple(x, y, t);
    }
    py::array_t<float> q_table() {
        py::array_t<float> q({(py::ssize_t)cfg_.height, (py::ssize_t)cfg_.width, (py::ssize_t)CUDARL_ACTIONS});
        ck(cudarl_get_q(ctx_, q.mutable_data()));
        return q;
    }
    void set_q_table(py::array_t<float, py::array::c_style | py::array::forcecast> q) {
        if ((size_t)q.size() != (size_t)cfg_.width * cfg_.height * CUDARL_ACTIONS) throw std::runtime_error("Invalid Q-table size");
        ck(cudarl_set_q(ctx_, q.data()));
    }
    void add_obstacle(int x, int y) { ck(cudarl_add_obstacle(ctx_, x, y)); }
    void set_goal(int x, int y) { ck(cudarl_set_goal(ctx_, x, y)); }
    void add_trap(int x, int y, float penalty) { ck(cudarl_add_trap(ctx_, x, y, penalty)); }
    py::array_t<uint8_t> cells() {
        py::array_t<uint8_t> c({(py::ssize_t)cfg_.height, (py::ssize_t)cfg_.width});
        ck(cudarl_get_cells(ctx_, c.mutable_data()));
        return c;
    }
    py::dict stats() {
        cudarl_stats s; ck(cudarl_get_stats(ctx_, &s));
        py::dict o; o["steps"] = s.steps; o["env_steps"] = s.env_steps; o["episodes"] = s.episodes; o["goals"] = s.goals;
        o["timeouts"] = s.timeouts; o["conflicts"] = s.conflicts; o["reward_sum"] = s.reward_sum; o["epsilon"] = s.epsilon;
        o["device_error"] = s.device_error;      // always 0 here: a recorded failure makes the call above throw
        return o;
    }
private:
    cudarl_config cfg_;
    cudarl_ctx* ctx_ = nullptr;
};

}  // namespace

PYBIND11_MODULE(cudarl_core, m) {
    m.doc() = "CudaRL-Arena Python bindings (B200-native batched implementation)";

    py::class_<EnvironmentBridge>(m, "Environment")
        .def(py::init<int, int>(), py::arg("width") = 10, py::arg("height") = 10)
        .def(py::init<int, int, int>(), py::arg("width"), py::arg("height"), py::arg("env_id"))
        .def("reset", &EnvironmentBridge::reset)
        .def("step", &EnvironmentBridge::step)
        .def("get_observation", &EnvironmentBridge::getObservation)
        .def("get_width", &EnvironmentBridge::getWidth)
        .def("get_height", &EnvironmentBridge::getHeight)
        .def("get_agent_position", &EnvironmentBridge::getAgentPosition)
        .def("add_obstacle", &EnvironmentBridge::addObstacle)
        .def("set_goal", &EnvironmentBridge::setGoal)
        .def("add_trap", &EnvironmentBridge::addTrap)
        // aliases (second binding / backend duck type of the reference)
        .def_property_readonly("width", &EnvironmentBridge::getWidth)
        .def_property_readonly("height", &EnvironmentBridge::getHeight)
        .def_property_readonly("env_id", &EnvironmentBridge::getEnvId)
        .def("get_reward", &EnvironmentBridge::getReward)
        .def("is_done", &EnvironmentBridge::isDone)
        .def("get_agent_x", [](const EnvironmentBridge& e) { return e.getAgentPosition().first; })
        .def("get_agent_y", [](const EnvironmentBridge& e) { return e.getAgentPosition().second; })
        .def("get_grid_data", &EnvironmentBridge::getObservation);

    py::class_<CudaQLearning>(m, "CudaQLearning")
        .def(py::init<int, int, int, float, float>(), py::arg("width"), py::arg("height"), py::arg("action_space_size") = 4,
             py::arg("learning_rate") = 0.1f, py::arg("discount_factor") = 0.99f)
        .def("update_batch", &CudaQLearning::update_batch, py::call_guard<py::gil_scoped_release>())
        .def("get_q_table", &CudaQLearning::get_q_table)
        .def("set_q_table", &CudaQLearning::set_q_table)
        .def("get_best_action", &CudaQLearning::get_best_action)
        .def("get_q_value", &CudaQLearning::get_q_value)
        .def("set_legacy_clamp", &CudaQLearning::set_legacy_clamp);

    py::class_<VecEnvironment>(m, "VecEnvironment")
        .def(py::init([](py::kwargs kw) { return new VecEnvironment(kw); }))
        .def("reset", &VecEnvironment::reset)
        .def("step", &VecEnvironment::step)
        .def("train_steps", &VecEnvironment::train_steps)
        .def("eval_rollout", &VecEnvironment::eval_rollout)
        .def("positions", &VecEnvironment::positions)
        .def("q_table", &VecEnvironment::q_table)
        .def("set_q_table", &VecEnvironment::set_q_table)
        .def("cells", &VecEnvironment::cells)
        .def("add_obstacle", &VecEnvironment::add_obstacle)
        .def("set_goal", &VecEnvironment::set_goal)
        .def("add_trap", &VecEnvironment::add_trap, py::arg("x"), py::arg("y"), py::arg("penalty") = -0.5f)
        .def("stats", &VecEnvironment::stats);

    m.attr("__version__") = "0.1.0";
}
