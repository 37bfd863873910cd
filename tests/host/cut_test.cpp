// The work cut of the split-K attention kernels and the record ranges of the merge kernel (csrc/work_cut.h), checked
// on the host over many shapes: the shares of the CTAs partition the tile order; the pieces a CTA walks through (as
// the kernels do, with locate()) cover every (sequence, kv head, tile) exactly once; record slots cta + item are
// unique and inside the workspace; the merge's CTA range of an item is exactly the set of CTAs that wrote a piece of
// it; with the per-head cut of a single sequence no CTA has more than one piece.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <random>
#include <set>
#include <vector>

#include "../../bruce-engine_b200/csrc/work_cut.h"

using namespace battn::fd;

#define CHECK(c)                                                                   \
    do {                                                                           \
        if (!(c)) {                                                                \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #c);             \
            std::exit(1);                                                          \
        }                                                                          \
    } while (0)

static void check_shape(const std::vector<int>& tiles, int Hkv, int grid, bool per_head) {
    const int n_seq = (int)tiles.size();
    std::vector<int> cum(n_seq + 1, 0);
    for (int i = 0; i < n_seq; ++i) cum[i + 1] = cum[i] + tiles[i];
    const int total = Hkv * cum[n_seq];
    const int cph = per_head ? grid / Hkv : 0;
    std::map<int, std::set<int>> ctas_of_item;                  // item -> CTAs with a piece of it
    std::set<int> slots;
    std::vector<std::vector<char>> seen(n_seq * Hkv);
    for (int i = 0; i < n_seq; ++i)
        for (int h = 0; h < Hkv; ++h) seen[i * Hkv + h].assign(tiles[i], 0);
    int per = 0, covered = 0;
    for (int cta = 0; cta < grid; ++cta) {
        const Share sh = cut_share(cum.data(), n_seq, Hkv, cph, cta, grid);
        CHECK(cta == 0 || sh.per == per);
        per = sh.per;
        CHECK(sh.g0 <= sh.g1 && sh.g1 <= total && sh.g1 - sh.g0 <= per);
        int pieces = 0;
        for (int g = sh.g0; g < sh.g1;) {
            const Piece pc = locate(g, sh.g1, cum.data(), n_seq, Hkv);
            CHECK(pc.i >= 0 && pc.i < n_seq && pc.kvh >= 0 && pc.kvh < Hkv && pc.n >= 1);
            CHECK(pc.tl >= 0 && pc.tl + pc.n <= tiles[pc.i]);
            const int item = pc.i * Hkv + pc.kvh;
            for (int t = pc.tl; t < pc.tl + pc.n; ++t) {
                CHECK(!seen[item][t]);
                seen[item][t] = 1;
                ++covered;
            }
            CHECK(ctas_of_item[item].insert(cta).second);        // one piece per (CTA, item)
            const int slot = cta + item;
            CHECK(slots.insert(slot).second);                    // record slots never collide
            CHECK(slot < grid + n_seq * Hkv);                    // ... and stay inside the workspace
            g += pc.n;
            ++pieces;
        }
        if (per_head) CHECK(pieces <= 1);
    }
    CHECK(covered == total);
    for (int i = 0; i < n_seq; ++i)
        for (int h = 0; h < Hkv; ++h) {
            if (tiles[i] == 0) continue;
            int clo, chi;
            item_ctas(cph, per, Hkv, cum[i], tiles[i], h, clo, chi);
            const std::set<int>& want = ctas_of_item[i * Hkv + h];
            CHECK(!want.empty() && *want.begin() == clo && *want.rbegin() == chi);
            CHECK((int)want.size() == chi - clo + 1);            // a contiguous CTA range, as the merge assumes
        }
}

int main() {
    std::mt19937 rng(12345);
    // one sequence, both cuts, the grids of the library (3 or 2 CTAs per SM on 148 SMs, one per SM) and odd ones
    for (int Hkv : {1, 2, 4, 8})
        for (int grid : {8, 37, 148, 296, 444, 445})
            for (int nt : {1, 2, 3, 7, 54, 55, 56, 64, 65, 128, 129, 512, 1000, 4096, 16385}) {
                check_shape({nt}, Hkv, grid, false);
                if (grid >= Hkv) check_shape({nt}, Hkv, grid, true);
            }
    // ragged batches, idle sequences included (linear cut only)
    for (int rep = 0; rep < 300; ++rep) {
        const int n_seq = 1 + (int)(rng() % 70), Hkv = 1 << (rng() % 4), grid = 1 + (int)(rng() % 600);
        std::vector<int> tiles(n_seq);
        for (int& t : tiles) t = (rng() % 5 == 0) ? 0 : 1 + (int)(rng() % (rep % 3 == 0 ? 3000 : 40));
        check_shape(tiles, Hkv, grid, false);
    }
    std::printf("OK\n");
    return 0;
}
