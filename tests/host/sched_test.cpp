// CPU test driver of include/battn_sched.h with a fake engine (compiled and run by tests/test_sched_host.py).
#include <cassert>
#include <cstdio>
#include <cstdlib>
#include <string>

#include "battn_sched.h"

using namespace battn_sched;

#define CHECK(c) do { if (!(c)) { std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #c); std::exit(1); } } while (0)

// The fake model: the next token after token t at position p of slot s is a fixed function of (t, p, s).
static int fake_next(int tok, int pos, int slot) { return (tok * 31 + pos * 7 + slot * 13 + 1) % 1000; }

struct FakeEngine : StepEngine {
    std::mutex mu;
    std::vector<std::string> log;            // "D<rows>", "P<slot>:<rows>", "V<rows>"
    std::vector<int> step_rows;
    int max_rows_seen = 0;
    void decode_step(int rows, const int* toks, const int* pos, const int* slots, int* amax) override {
        std::this_thread::sleep_for(std::chrono::microseconds(300));           // a step takes a while
        for (int i = 0; i < rows; ++i) {
            for (int k = 0; k < i; ++k) CHECK(slots[k] != slots[i]);             // one row per slot per step
            amax[i] = fake_next(toks[i], pos[i], slots[i]);
        }
        std::lock_guard<std::mutex> lk(mu);
        log.push_back("D" + std::to_string(rows));
        step_rows.push_back(rows);
        max_rows_seen = std::max(max_rows_seen, rows);
    }
    void prefill_chunk(int slot, const int*, int rows, int, bool) override {
        std::this_thread::sleep_for(std::chrono::microseconds(1500));
        std::lock_guard<std::mutex> lk(mu);
        log.push_back("P" + std::to_string(slot) + ":" + std::to_string(rows));
    }
    void verify_round(int slot, const int* toks, int rows, int pos, int* amax) override {
        for (int i = 0; i < rows; ++i) amax[i] = fake_next(toks[i], pos + i, slot);
        std::lock_guard<std::mutex> lk(mu);
        log.push_back("V" + std::to_string(rows));
    }
};

// brute-force statement of the drafter's rule
static std::vector<int> brute_draft(const std::vector<int>& h, int dmax, int nmax, int nmin) {
    const int n = (int)h.size();
    for (int g = nmax; g >= nmin; --g) {
        if (n < g) continue;
        for (int j = n - 2; j >= g - 1; --j) {                 // j = last token of an EARLIER occurrence, most recent first
            bool eq = true;
            for (int i = 0; i < g; ++i) eq = eq && h[(size_t)(j - g + 1 + i)] == h[(size_t)(n - g + i)];
            if (!eq) continue;
            const int span = n - 1 - j;
            std::vector<int> d;
            for (int i = 0; i < dmax; ++i) d.push_back(h[(size_t)(j + 1 + (j + 1 + i <= n - 1 ? i : i % span))]);
            return d;
        }
    }
    return {};
}

static void test_drafter() {
    NgramDrafter d(7, 4, 1);
    const int seq[] = {5, 6, 7, 8, 5, 6};
    for (int t : seq) d.push(t);
    const std::vector<int> want = {7, 8, 5, 6, 7, 8, 5};      // continuation of the earlier "5 6", repeated periodically
    CHECK(d.draft() == want);
    CHECK(d.matched_ngram() == 2);
    d.push(99);                                              // a token never seen: no draft
    CHECK(d.draft().empty());
    // random token streams over a small alphabet against the brute-force rule
    uint64_t s = 12345;
    for (int trial = 0; trial < 50; ++trial) {
        NgramDrafter x(5 + trial % 3, 1 + trial % 4, 1);
        std::vector<int> h;
        for (int i = 0; i < 200; ++i) {
            s = s * 6364136223846793005ull + 1442695040888963407ull;
            const int t = (int)((s >> 33) % (3 + trial % 5));
            h.push_back(t);
            x.push(t);
            CHECK(x.draft() == brute_draft(h, 5 + trial % 3, 1 + trial % 4, 1));
        }
        x.clear();
        CHECK(x.draft().empty());
    }
}

static void test_spec_round() {
    SpecRound r(7);
    std::vector<int> drafts = {1, 2, 3, 4, 5, 6, 7};
    CHECK(r.plan(7, 100) == 7 && r.plan(3, 100) == 3 && r.plan(7, 4) == 3 && r.plan(7, 1) == 0);
    const std::vector<int> rows = SpecRound::rows(42, drafts, 3);
    CHECK((rows == std::vector<int>{42, 1, 2, 3}));
    int amax_all[8] = {1, 2, 3, 4, 5, 6, 7, 70};             // every draft confirmed: next token is row k's argmax
    SpecOutcome o = r.judge(drafts, 7, amax_all);
    CHECK(o.accepted == 7 && o.next_token == 70 && o.rows == 8 && r.kmax() == 7);
    int amax_none[8] = {9, 0, 0, 0, 0, 0, 0, 0};             // first draft wrong: nothing accepted, shorter drafts next
    o = r.judge(drafts, 7, amax_none);
    CHECK(o.accepted == 0 && o.next_token == 9 && r.kmax() == 6);
    int amax_some[8] = {1, 2, 8, 0, 0, 0, 0, 0};             // two accepted: length unchanged
    o = r.judge(drafts, 6, amax_some);
    CHECK(o.accepted == 2 && o.next_token == 8 && r.kmax() == 6);
    for (int i = 0; i < 10; ++i) r.judge(drafts, 1, amax_none);
    CHECK(r.kmax() == 1);                                    // never below one
    int amax_one[2] = {1, 5};
    r.judge(drafts, 1, amax_one);
    CHECK(r.kmax() == 2);                                    // grows again after a fully accepted round
}

static void test_slot_pool() {
    SlotPool pool(3);
    int hit = -1;
    CHECK(pool.acquire({1, 2, 3}, &hit) == 0 && hit == 0);
    CHECK(pool.acquire({1, 2, 3}) == 1);
    pool.release(0, {1, 2, 3, 4, 5});
    pool.release(1, {1, 2, 9});
    CHECK(pool.free_slots() == 3);
    CHECK(pool.acquire({1, 2, 3, 4, 7}, &hit) == 0 && hit == 4);     // the returning conversation finds its prefix
    CHECK(pool.acquire({1, 2, 9, 9}, &hit) == 1 && hit == 3);
    CHECK(pool.acquire({7}, &hit) == 2 && hit == 0);
    std::atomic<int> got{-2};
    std::thread waiter([&] { got = pool.acquire({1}); });                // blocks: all busy
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
    CHECK(got == -2);
    pool.release(2, {});
    waiter.join();
    CHECK(got == 2);
    std::thread stopper([&] { got = pool.acquire({1}); });
    std::this_thread::sleep_for(std::chrono::milliseconds(10));
    pool.stop();
    stopper.join();
    CHECK(got == -1);
}

static void test_page_pool() {
    PagePool pool(/*n_pages*/ 10, /*page_len*/ 256, /*rows*/ 3, /*max_pages*/ 6);
    CHECK(pool.free_pages() == 10);
    CHECK(pool.reserve(0, 700) && pool.pages_of(0) == 3 && pool.capacity_of(0) == 768 && pool.free_pages() == 7);
    CHECK(pool.reserve(0, 700) && pool.pages_of(0) == 3);                    // already there
    CHECK(!pool.reserve(0, 6 * 256 + 1));                                    // beyond the row's table
    CHECK(pool.take_dirty(0) && !pool.take_dirty(0));
    // a second request shares the first 600 positions: two whole pages
    CHECK(pool.share_prefix(0, 1, 600) == 512 && pool.pages_of(1) == 2);
    CHECK(pool.row(1)[0] == pool.row(0)[0] && pool.row(1)[1] == pool.row(0)[1]);
    CHECK(pool.refcount(pool.row(0)[0]) == 2 && pool.free_pages() == 7);
    CHECK(pool.share_prefix(0, 1, 600) == 0);                                // only an empty row may adopt a prefix
    CHECK(pool.reserve(1, 900) && pool.pages_of(1) == 4 && pool.free_pages() == 5);
    int from, to;
    CHECK(pool.make_writable(1, 800, &from, &to) && from == -1 && to == -1); // its own page
    // row 1 rewrites position 300, which lives in a shared page: copy on write
    const int shared = pool.row(0)[1];
    CHECK(pool.make_writable(1, 300, &from, &to) && from == shared && to >= 0 && to != shared);
    CHECK(pool.row(1)[1] == to && pool.row(0)[1] == shared && pool.refcount(shared) == 1 && pool.refcount(to) == 1);
    CHECK(pool.free_pages() == 4);
    // releasing the first row keeps the page the second still uses
    const int kept = pool.row(0)[0];
    pool.release(0);
    CHECK(pool.pages_of(0) == 0 && pool.refcount(kept) == 1 && pool.free_pages() == 6 && pool.row(0)[0] == -1);
    CHECK(!pool.reserve(2, 7 * 256));                                        // more than the pool holds (and the table)
    CHECK(pool.reserve(2, 6 * 256) && pool.free_pages() == 0);
    CHECK(!pool.reserve(0, 1));                                              // exhausted: nothing changes
    CHECK(pool.share_prefix(1, 0, 256) == 256);                              // sharing needs no free page
    CHECK(!pool.make_writable(0, 10, &from, &to));                           // but un-sharing does
    pool.release(2);
    CHECK(pool.make_writable(0, 10, &from, &to) && from == kept);
    pool.release(0); pool.release(1);
    CHECK(pool.free_pages() == 10);
    for (int p = 0; p < 10; ++p) CHECK(pool.refcount(p) == 0);
}

static void test_chunk_policy() {
    SchedConfig c;
    CHECK(StepScheduler::next_chunk(c, 1, 0, 5000) == 512);          // one request, ingesting: nobody else -> solo... (pending 1)
    CHECK(StepScheduler::next_chunk(c, 3, 2, 5000) == 384);          // one prompt behind live decoders: narrow chunk
    CHECK(StepScheduler::next_chunk(c, 5, 1, 5000) == 512);          // a burst of prompts: wide chunk
    CHECK(StepScheduler::next_chunk(c, 2, 2, 5000) == 512);          // nothing pending
    CHECK(StepScheduler::next_chunk(c, 3, 2, 100) == 100);           // the last, shorter chunk
}

static void test_scheduler() {
    FakeEngine eng;
    SchedConfig cfg;
    cfg.max_rows = 16;
    StepScheduler sch(&eng, cfg);
    sch.start();
    const int n_req = 24, n_tok = 12;                                // more requests than rows per step
    std::vector<std::thread> th;
    std::atomic<int> bad{0};
    for (int r = 0; r < n_req; ++r)
        th.emplace_back([&, r] {
            sch.enter();
            sch.enter_decode();
            int tok = r, pos = 100 + r;
            for (int i = 0; i < n_tok; ++i) {
                const int got = sch.decode(r, tok, pos);
                if (got != fake_next(tok, pos, r)) ++bad;
                tok = got; ++pos;
            }
            sch.leave_decode();
            sch.leave();
        });
    for (auto& t : th) t.join();
    CHECK(bad == 0);
    SchedStats st = sch.stats();
    CHECK(st.rows == n_req * n_tok);
    CHECK(eng.max_rows_seen <= 16 && eng.max_rows_seen >= 8);        // concurrent submits were fused
    CHECK(st.steps * 4 <= st.rows);                                  // on average at least four rows per step
    // a long prompt behind two live decoders: 384-row chunks, and the decoders get steps between them
    std::atomic<bool> go{true};
    std::vector<std::thread> dec;
    for (int r = 0; r < 2; ++r)
        dec.emplace_back([&, r] {
            sch.enter(); sch.enter_decode();
            int tok = 1, pos = 0;
            while (go) { tok = sch.decode(r, tok, pos); ++pos; }
            sch.leave_decode(); sch.leave();
        });
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
    { std::lock_guard<std::mutex> lk(eng.mu); eng.log.clear(); }
    sch.enter();
    std::vector<int> prompt(1000, 3);
    sch.prefill(7, prompt, 0, true);
    std::vector<std::string> log;
    { std::lock_guard<std::mutex> lk(eng.mu); log = eng.log; }
    go = false;
    for (auto& t : dec) t.join();
    sch.leave();
    std::vector<std::string> chunks;
    int first = -1, last = -1, decodes_between = 0;
    for (int i = 0; i < (int)log.size(); ++i)
        if (log[(size_t)i][0] == 'P') { chunks.push_back(log[(size_t)i]); if (first < 0) first = i; last = i; }
    for (int i = first; i < last; ++i) decodes_between += log[(size_t)i][0] == 'D';
    CHECK((chunks == std::vector<std::string>{"P7:384", "P7:384", "P7:232"}));
    CHECK(decodes_between >= 2);                                     // a decode step after each of the first two chunks
    // a verify round goes through as one call
    const std::vector<int> am = sch.verify(3, {10, 11, 12}, 50);
    CHECK(am.size() == 3 && am[0] == fake_next(10, 50, 3) && am[2] == fake_next(12, 52, 3));
    CHECK(sch.stats().verify_rounds == 1);
    sch.shutdown();
}

static void test_row_graphs() {
    int built = 0;
    RowGraphs<int> g(2, 8, [&](int rows) { ++built; return rows * 100; });
    CHECK(g.get(5) == 500 && g.get(5) == 500 && built == 1);
    g.warm();
    CHECK(built == 7 && g.captures() == 7 && g.get(8) == 800 && g.get(2) == 200);
}

// a whole greedy generation with speculation against the fake model: must produce exactly the tokens of plain decoding
static void test_spec_generation_matches_plain_decoding() {
    FakeEngine eng;
    auto next = [](int tok, int pos) { return (tok + 1) % 5; };        // a periodic "model": easy to draft for
    struct Periodic : StepEngine {
        void decode_step(int rows, const int* t, const int*, const int*, int* a) override { for (int i = 0; i < rows; ++i) a[i] = (t[i] + 1) % 5; }
        void prefill_chunk(int, const int*, int, int, bool) override {}
        void verify_round(int, const int* t, int rows, int, int* a) override { for (int i = 0; i < rows; ++i) a[i] = (t[i] + 1) % 5; ++rounds; total_rows += rows; }
        int rounds = 0, total_rows = 0;
    } model;
    (void)next; (void)eng;
    std::vector<int> plain, spec;
    int t = 0;
    for (int i = 0; i < 60; ++i) { plain.push_back(t); t = (t + 1) % 5; }
    NgramDrafter drafter;
    SpecRound round;
    t = 0;
    int pos = 0, launches = 0;
    while ((int)spec.size() < 60) {
        spec.push_back(t);
        drafter.push(t);
        const std::vector<int> drafts = drafter.draft();
        const int k = round.plan((int)drafts.size(), 60 - (int)spec.size());
        if (k <= 0) {
            int a = -1, s = 0;
            model.decode_step(1, &t, &pos, &s, &a);
            ++launches; ++pos; t = a;
            continue;
        }
        const std::vector<int> rows = SpecRound::rows(t, drafts, k);
        std::vector<int> amax(rows.size());
        model.verify_round(0, rows.data(), (int)rows.size(), pos, amax.data());
        ++launches;
        const SpecOutcome o = round.judge(drafts, k, amax.data());
        for (int i = 0; i < o.accepted && (int)spec.size() < 60; ++i) { spec.push_back(drafts[(size_t)i]); drafter.push(drafts[(size_t)i]); }
        pos += o.accepted + 1;
        t = o.next_token;
    }
    CHECK(spec == plain);
    CHECK(launches < 25);                                              // most tokens came from accepted drafts
}

int main() {
    test_drafter();
    test_spec_round();
    test_slot_pool();
    test_page_pool();
    test_chunk_policy();
    test_row_graphs();
    test_spec_generation_matches_plain_decoding();
    test_scheduler();
    std::printf("OK\n");
    return 0;
}
