// environment.h -- same file name as the reference's src/environment.h: a program that includes it gets
// class Environment (src/environment.h:17-47) from this library.  Put this directory on the include path instead of
// the reference's src/.
#pragma once
#include "../facade.h"
