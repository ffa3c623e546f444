// environment_bridge.h -- same file name as the reference's src/environment_bridge.h (class EnvironmentBridge, :10-80).
#pragma once
#include "../facade.h"
