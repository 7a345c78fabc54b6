// Definitions the reference's Memoria host sources expect from translation units that are not
// part of this path.  Test infrastructure only.
#include "machina/model.h"
#include "memoria/importance_scorer.h"
#include <cstdio>
#include <cstdlib>

namespace deusridet {
// The pool sizes itself from this process-wide static (block_pool.cpp:27).
int ModelConfig::NUM_FA_LAYERS = 1;

// importance_scorer.cu is CUDA; only the host arg-min is reachable from cache_manager.cpp and
// only when a scorer is attached, which these checkers never do.
ImportanceScorer::~ImportanceScorer() {}
int ImportanceScorer::least_important(const int*, int) const {
    std::fprintf(stderr, "reference checker: ImportanceScorer is not linked\n");
    std::abort();
}
}  // namespace deusridet
