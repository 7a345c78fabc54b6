// One allocate / evict scenario written against the reference's class interface
// (BlockPool, CacheManager).  It is compiled twice by the tests: against the shim header and
// libdrkv.so, and — where the reference tree is mounted — against the reference's own headers
// and sources; both builds must print the same text.
#ifdef SCENARIO_USE_REFERENCE
#include "memoria/block_pool.h"
#include "memoria/cache_manager.h"
#include "memoria/importance_scorer.h"
#include "communis/log.h"
#define PER_PAGE_BYTES ((size_t)2 * 2 * 4 * 16 * 256 * 2)   // layers * K,V * 4 heads * 16 slots * 256 dims * 2 B
#else
#include "deusridet_shim.hpp"
#define PER_PAGE_BYTES ((size_t)2 * 2 * 4 * 16 * 256 * 2)
#endif
#include <cstdio>
#include <vector>

using namespace deusridet;

static void dump(const char* tag, CacheManager& cm, int n_logical) {
    std::vector<int> t(n_logical, -7);
#ifdef SCENARIO_USE_REFERENCE
    cm.sync_block_table(0);
    for (int i = 0; i < n_logical; i++) t[i] = cm.d_block_table()[i];   // host memory under the CUDA stub
#else
    cm.host_table(t.data(), n_logical);
#endif
    std::printf("%s free=%d used=%d nlog=%d table=", tag, cm.free_blocks(), cm.gpu_blocks_used(),
                cm.num_logical_blocks());
    for (int v : t) std::printf("%d,", v);
    std::printf("\n");
}

int main() {
#ifdef SCENARIO_USE_REFERENCE
    deusridet::log::set_level(deusridet::log::Level::ERROR);
    ModelConfig::NUM_FA_LAYERS = 2;
#else
    shim_geometry() = drkv_geometry{2, 24, 4, 256, 16, DRKV_DTYPE_F16, 64, 1e7f};
#endif
    {
        BlockPool small;
        const bool ok = small.init(3 * PER_PAGE_BYTES, 16);
        std::printf("small pool init=%d\n", (int)ok);
    }
    BlockPool bp;
    const bool ok = bp.init(6 * PER_PAGE_BYTES + 100, 16);
    std::printf("pool init=%d max=%d bs=%d total=%zu\n", (int)ok, bp.max_blocks(), bp.block_size(), bp.total_bytes());
    const int a = bp.alloc_block();
    const int b = bp.alloc_block();
    const int c = bp.alloc_block();
    std::printf("alloc %d %d %d free=%d koff=%zu voff=%zu\n", a, b, c, bp.free_count(), bp.k_offset(1, 2),
                bp.v_offset(1, 2));
    bp.free_block(a);
    bp.free_block(c);
    const int r0 = bp.alloc_block();
    const int r1 = bp.alloc_block();
    std::printf("realloc %d %d free=%d\n", r0, r1, bp.free_count());

    CacheManager cm;
    const bool cm_ok = cm.init(8 * PER_PAGE_BYTES, "", 16);
    std::printf("cm init=%d\n", (int)cm_ok);
    const int NL = 16;
    for (int pos = 0; pos < 12 * 16; pos += 16) {
        bool ok = cm.ensure_blocks_for(pos);
        cm.set_seq_len(pos + 16);
        char tag[32];
        std::snprintf(tag, sizeof tag, "ensure(%d)=%d", pos, (int)ok);
        dump(tag, cm, NL);
    }
    const int ev3 = cm.evict_blocks(3);
    std::printf("evict3=%d\n", ev3);
    dump("after evict", cm, NL);
    const bool rg = cm.ensure_blocks_for_range(12 * 16 + 5, 40);
    std::printf("range=%d\n", (int)rg);
    dump("after range", cm, NL);
    const bool ef = cm.ensure_free_blocks(5);
    std::printf("ensure_free(5)=%d\n", (int)ef);
    dump("after ensure_free", cm, NL);
    const bool beyond = cm.ensure_blocks_for(16 * 16);
    std::printf("beyond=%d\n", (int)beyond);
    const int eva = cm.evict_blocks(100);
    std::printf("evict_all=%d\n", eva);
    dump("end", cm, NL);

    // The same manager with an importance scorer attached: victims follow the scores, ties the
    // allocation order.  The values live in host memory, which is what "device" memory is in both
    // builds of this scenario (CUDA stub / engine without a device).
    ImportanceScorer scorer;
    const bool sc_ok = scorer.init(NL, 0.5f);
    CacheManager scored;
    const bool scm_ok = scored.init(8 * PER_PAGE_BYTES, "", 16, nullptr, &scorer);
    std::printf("scored init=%d %d\n", (int)sc_ok, (int)scm_ok);
    for (int pos = 0; pos < 7 * 16; pos += 16) scored.ensure_blocks_for(pos);
    scored.set_seq_len(7 * 16);
    const float first[7] = {4.f, 1.f, 3.f, 1.f, 0.5f, 2.f, 0.5f};
    scorer.update(first, 7);
    scorer.sync_to_host();
    std::printf("scores");
    for (int i = 0; i < 8; i++) std::printf(" %.4f", scorer.score(i));
    std::printf("\n");
    std::printf("scored evict2=%d\n", scored.evict_blocks(2));
    dump("scored after evict", scored, NL);
    const float second[7] = {0.f, 0.f, 0.f, 8.f, 0.f, 0.f, 0.f};
    scorer.update(second, 7);
    scorer.sync_to_host();
    std::printf("scores");
    for (int i = 0; i < 8; i++) std::printf(" %.4f", scorer.score(i));
    std::printf("\n");
    for (int pos = 7 * 16; pos < 12 * 16; pos += 16) {      // the pool runs dry: allocation evicts by score
        const bool more = scored.ensure_blocks_for(pos);
        char tag[32];
        std::snprintf(tag, sizeof tag, "scored ensure(%d)=%d", pos, (int)more);
        dump(tag, scored, NL);
    }
    scored.destroy();
    scorer.destroy();
    return 0;
}
