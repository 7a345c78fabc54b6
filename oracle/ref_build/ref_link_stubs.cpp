// Definitions the reference's Memoria host sources expect from translation units that are not
// part of this path.  Test infrastructure only.
#include "machina/model.h"
#include <cstdio>
#include <cstdlib>

namespace deusridet {
// The pool sizes itself from this process-wide static (block_pool.cpp:27).
int ModelConfig::NUM_FA_LAYERS = 1;

}  // namespace deusridet
