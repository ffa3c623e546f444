// facade_consumer.cpp -- TEST PROGRAM.  A plain C++ consumer of the reference's class surface, compiled against the
// compatibility headers (same include names as the reference: "core/environment.h", "environment_bridge.h",
// "q_learning.cuh") and linked with libcudarl.so.  It restates, case by case, the reference's Catch2 file
// tests/test_environment.cpp:6-140 (Catch2 is not installed here, so a small REQUIRE stands in), then the flow of the
// demo src/main.cu:21-99, then what the reference never tests: move semantics, getCellValue, the bridge and grid edits.
// Exit code 0 = every check held; each failure prints its line.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>
#include "core/environment.h"
#include "environment_bridge.h"
#include "q_learning.cuh"

using namespace cudarl;

static int g_failed = 0, g_checked = 0;
#define REQUIRE(cond) do { ++g_checked; if (!(cond)) { ++g_failed; std::printf("FAILED %s:%d  %s\n", __FILE__, __LINE__, #cond); } } while (0)
static bool approx(float a, float b) { return std::fabs(a - b) <= 1e-6f * (1.0f + std::fabs(b)); }

static void environment_initialization() {          // tests/test_environment.cpp:6-26
    Environment env(0);
    REQUIRE(env.getWidth() == 10); REQUIRE(env.getHeight() == 10);
    REQUIRE(env.getAgentX() == 5); REQUIRE(env.getAgentY() == 5);
    REQUIRE(env.getReward() == 0.0f);
    REQUIRE(env.isDone() == false);
}
static void environment_reset() {                   // :28-50
    Environment env(0);
    env.step(1); env.step(1);
    env.reset();
    REQUIRE(env.getAgentX() == 5); REQUIRE(env.getAgentY() == 5);
    REQUIRE(env.getReward() == 0.0f);
    REQUIRE(env.isDone() == false);
}
static void environment_step() {                    // :52-100
    { Environment env(0); env.step(1); REQUIRE(env.getAgentX() == 6); REQUIRE(env.getAgentY() == 5); }
    { Environment env(0); env.step(2); REQUIRE(env.getAgentX() == 5); REQUIRE(env.getAgentY() == 6); }
    { Environment env(0); env.step(3); REQUIRE(env.getAgentX() == 4); REQUIRE(env.getAgentY() == 5); }
    { Environment env(0); env.step(0); REQUIRE(env.getAgentX() == 5); REQUIRE(env.getAgentY() == 4); }
    { Environment small_env(1, 3, 3); small_env.step(1); REQUIRE(small_env.getAgentX() == 2); small_env.step(1); REQUIRE(small_env.getAgentX() == 2); }
    { Environment env(0); env.step(1); REQUIRE(approx(env.getReward(), -0.01f)); }
}
static void environment_goal_detection() {          // :102-120
    Environment env(0, 5, 5);
    env.reset();
    env.step(1); env.step(1); env.step(0); env.step(0);
    REQUIRE(env.isDone() == true);
    REQUIRE(approx(env.getReward(), 1.0f));
}
static void environment_grid_access() {             // :122-140
    Environment env(0, 5, 5);
    std::vector<float> grid = env.getGrid();
    REQUIRE(grid.size() == 25);
    REQUIRE(approx(env.getCellValue(4, 0), 1.0f));
    REQUIRE(env.getCellValue(10, 10) == 0.0f);
}

static void demo_flow() {                           // src/main.cu:21-99 without the printing and the half-second naps
    Environment env(0);
    CudaQLearning q_learning(env.getWidth(), env.getHeight(), 4, 0.1f, 0.99f);
    env.reset();
    std::vector<std::pair<int, int>> states, next_states; std::vector<int> actions; std::vector<float> rewards; std::vector<bool> dones;
    std::srand(1);
    for (int step = 0; step < 10; step++) {
        const int x = env.getAgentX(), y = env.getAgentY(), action = std::rand() % 4;
        states.push_back({x, y}); actions.push_back(action);
        env.step(action);
        rewards.push_back(env.getReward()); next_states.push_back({env.getAgentX(), env.getAgentY()}); dones.push_back(env.isDone());
        if (env.isDone()) break;
    }
    q_learning.update_batch(states, actions, rewards, next_states, dones);
    float touched = 0.0f;
    for (size_t i = 0; i < states.size(); ++i) touched += std::fabs(q_learning.get_q_value(states[i].first, states[i].second, actions[i]));
    REQUIRE(touched > 0.0f);                         // every visited (state, action) moved away from the zero table
    for (int a = 0; a < 4; a++) REQUIRE(q_learning.get_q_value(0, 0, a) == 0.0f);      // (0,0) was never visited in 10 steps from the centre
    REQUIRE(q_learning.get_q_table().size() == 400);
}

static void beyond_the_reference_tests() {
    Environment a(7, 6, 4);                          // move-only, as src/core/environment.h:29-35
    a.step(1);
    Environment b(std::move(a));
    REQUIRE(b.getAgentX() == 4 && b.getAgentY() == 2 && b.getWidth() == 6 && b.getHeight() == 4);
    Environment c(0, 3, 3);
    c = std::move(b);
    c.step(3);
    REQUIRE(c.getAgentX() == 3 && c.getId() == 7);
    REQUIRE(c.getCellValue(-1, 0) == 0.0f && c.getCellValue(0, 4) == 0.0f && approx(c.getCellValue(5, 0), 1.0f));

    EnvironmentBridge br(5, 5);                      // src/environment_bridge.h:10-80
    std::vector<float> obs = br.reset();
    REQUIRE(obs.size() == 25 && obs[4] == 1.0f);
    auto r = br.step(1);
    REQUIRE(std::get<3>(r) == "agent_pos: (3,2)" && approx(std::get<1>(r), -0.01f) && !std::get<2>(r));
    br.addObstacle(4, 2);
    r = br.step(1);
    REQUIRE(br.getAgentPosition() == std::make_pair(3, 2));                 // blocked: src/kernels.cu:39-44
    br.addTrap(3, 1, -0.25f);
    r = br.step(0);
    REQUIRE(br.getAgentPosition() == std::make_pair(3, 2) && std::get<1>(r) == -0.25f);      // trap penalty: src/kernels.cu:61-63
    br.setGoal(3, 3);
    r = br.step(2);
    REQUIRE(std::get<2>(r) && std::get<1>(r) == 1.0f);
    obs = br.getObservation();
    REQUIRE(obs[3 * 5 + 3] == 1.0f && obs[4] == 0.0f && obs[2 * 5 + 4] == -1.0f && obs[1 * 5 + 3] == -0.25f);

    CudaQLearning q(4, 4, 4);
    bool threw = false;
    try { q.update_batch({{0, 0}}, {0, 1}, {0.0f}, {{0, 0}}, {false}); } catch (const std::runtime_error& e) { threw = std::string(e.what()) == "Inconsistent batch sizes"; }
    REQUIRE(threw);
    threw = false;
    try { q.get_best_action(4, 0); } catch (const std::runtime_error& e) { threw = std::string(e.what()) == "Invalid state"; }
    REQUIRE(threw);
}

int main() {
    try {
        environment_initialization(); environment_reset(); environment_step(); environment_goal_detection(); environment_grid_access();
        demo_flow(); beyond_the_reference_tests();
    } catch (const std::exception& e) { std::printf("FAILED with exception: %s\n", e.what()); return 2; }
    std::printf("%d checks, %d failed\n", g_checked, g_failed);
    return g_failed ? 1 : 0;
}
