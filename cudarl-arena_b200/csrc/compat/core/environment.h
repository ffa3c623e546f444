// core/environment.h -- same file name as the reference's refactored header src/core/environment.h:29-35, whose class lives
// in namespace cudarl and is move-only; the class of this library is both.
#pragma once
#include "../../facade.h"
namespace cudarl { using ::Environment; }
