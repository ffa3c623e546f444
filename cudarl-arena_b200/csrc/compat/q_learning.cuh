// q_learning.cuh -- same file name as the reference's src/q_learning.cuh (class CudaQLearning, :8-95).
#pragma once
#include "../facade.h"
