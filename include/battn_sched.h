/*
 * battn_sched.h -- host-side control around the attention step: which rows run in which launch.
 *
 * The kernels behind battn.h take whatever (rows, slots, chunk) shape the host hands them.  In the reference engine
 * that shape is decided by three pieces of host code, restated here as a small header-only C++17 library (no CUDA
 * in this file: the GPU work is behind the StepEngine interface, so everything is testable with a fake engine):
 *
 *   SlotPool        the server's slot pool with prefix affinity: a request takes the free slot whose cached token
 *                   ids share the longest prefix with its prompt        (engine/src/server.h:376-396,
 *                   Session::cache_hit / common_prefix, engine/src/session.h:337-346)
 *   StepScheduler   the batch coordinator: request threads submit decode tokens, prompts and verify rounds and block;
 *                   one worker thread owns the device, fuses every decode that is queued (plus those that arrive
 *                   within a grace window) into one multi-slot step, and cuts prompts into chunks between which
 *                   waiting decodes get a step                          (BatchCoordinator, session.h:34-222;
 *                   run_decodes, session.h:733-765).  Generalised from the reference's 8 rows to any row count.
 *   NgramDrafter    prompt-lookup drafting: the continuation of the most recent earlier occurrence of the current
 *                   suffix                                              (engine/src/bruce.cu:8499-8537)
 *   SpecRound       one speculative round: accepted token + drafts in, per-row argmax out, accepted prefix and the
 *                   adaptive draft length                               (session.h:648-703)
 *   RowGraphs       one captured launch sequence per row count, built once and replayed
 *                                                                       (capture_verify_graphs, bruce.cu:7877-7900)
 */
#ifndef BATTN_SCHED_H
#define BATTN_SCHED_H

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

namespace battn_sched {

/* What the scheduler drives.  One call = one pass of the model over the given rows; attention inside it is
 * battn_decode (decode_step: one row per slot), battn_prefill (prefill_chunk) or battn_verify (verify_round). */
struct StepEngine {
    virtual ~StepEngine() = default;
    /* rows independent sequences: token toks[i] at position pos[i] of slot slots[i]; argmax_out[i] (if non-null)
     * receives the greedy next token of row i                                  (bruce_decode_step, bruce.cu:8246) */
    virtual void decode_step(int rows, const int* toks, const int* pos, const int* slots, int* argmax_out) = 0;
    /* `rows` prompt tokens of one slot at positions pos .. pos+rows-1          (bruce_prefill_chunk) */
    virtual void prefill_chunk(int slot, const int* toks, int rows, int pos, bool need_logits) = 0;
    /* rows = 1 accepted token + drafts at pos .. pos+rows-1; argmax per row    (bruce_verify_round) */
    virtual void verify_round(int slot, const int* toks, int rows, int pos, int* argmax_out) = 0;
};

/* ---- slot pool with prefix affinity ------------------------------------------------------------------------- */
class SlotPool {
public:
    explicit SlotPool(int n_slots) : busy_(n_slots, 0), cached_(n_slots) {}

    static int common_prefix(const std::vector<int>& a, const std::vector<int>& b) {
        const size_t n = std::min(a.size(), b.size());
        size_t i = 0;
        while (i < n && a[i] == b[i]) ++i;
        return (int)i;
    }
    /* Blocks until a slot is free (or stop() was called: returns -1).  Among the free slots the one whose cached ids
     * share the longest prefix with `prompt` wins; ties go to the lowest index.  *hit receives that prefix length. */
    int acquire(const std::vector<int>& prompt, int* hit = nullptr) {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return stop_ || std::find(busy_.begin(), busy_.end(), 0) != busy_.end(); });
        if (stop_) return -1;
        int best = -1, best_hit = -1;
        for (int i = 0; i < (int)busy_.size(); ++i) {
            if (busy_[(size_t)i]) continue;
            const int h = common_prefix(prompt, cached_[(size_t)i]);
            if (h > best_hit) { best_hit = h; best = i; }
        }
        busy_[(size_t)best] = 1;
        if (hit) *hit = best_hit;
        return best;
    }
    /* The slot's cache now holds exactly these token ids (what a later request can reuse). */
    void release(int slot, std::vector<int> cached_ids) {
        {
            std::lock_guard<std::mutex> lk(mu_);
            cached_[(size_t)slot] = std::move(cached_ids);
            busy_[(size_t)slot] = 0;
        }
        cv_.notify_one();
    }
    void stop() {
        { std::lock_guard<std::mutex> lk(mu_); stop_ = true; }
        cv_.notify_all();
    }
    int free_slots() {
        std::lock_guard<std::mutex> lk(mu_);
        return (int)std::count(busy_.begin(), busy_.end(), 0);
    }

private:
    std::mutex mu_;
    std::condition_variable cv_;
    std::vector<char> busy_;
    std::vector<std::vector<int>> cached_;
    bool stop_ = false;
};

/* ---- page allocator of a paged cache, with prefix sharing between table rows ---------------------------------------
 * Host-side owner of the page table that battn_*_paged calls read (include/battn.h): hands out pages on demand
 * instead of the reference's fixed ctx/N partition per slot (bruce.cu:5471-5503), lets a new request start from the
 * pages that already hold another row's prefix (the reference reuses a prefix inside one slot only,
 * session.h:337-346), and tells the caller which page to copy before a row appends into a page it shares.
 * Not thread-safe: the scheduler thread owns it.  The caller uploads table() (or the rows marked dirty) to the
 * device before the next launch. */
class PagePool {
public:
    PagePool(int n_pages, int page_len, int n_rows, int max_pages)
        : page_len_(page_len), max_pages_(max_pages), table_((size_t)n_rows * max_pages, -1), used_(n_rows, 0),
          ref_(n_pages, 0), dirty_(n_rows, 0) {
        for (int p = n_pages - 1; p >= 0; --p) free_.push_back(p);
    }
    /* Row `row` can hold positions [0, n_pos) afterwards.  False (and nothing changed) when the pool or the row's
     * table is too small. */
    bool reserve(int row, int n_pos) {
        const int need = (n_pos + page_len_ - 1) / page_len_;
        int& have = used_[(size_t)row];
        if (need > max_pages_ || need - have > (int)free_.size()) return false;
        for (; have < need; ++have) {
            const int p = free_.back();
            free_.pop_back();
            ref_[(size_t)p] = 1;
            at(row, have) = p;
            dirty_[(size_t)row] = 1;
        }
        return true;
    }
    /* The empty row `dst` starts with the pages that hold the first n_pos positions of `src`; only whole pages are
     * shared.  Returns the number of positions dst now holds (a multiple of the page length). */
    int share_prefix(int src, int dst, int n_pos) {
        if (used_[(size_t)dst] != 0) return 0;
        const int n = std::min(n_pos / page_len_, used_[(size_t)src]);
        for (int i = 0; i < n; ++i) {
            at(dst, i) = at(src, i);
            ++ref_[(size_t)at(src, i)];
        }
        used_[(size_t)dst] = n;
        if (n) dirty_[(size_t)dst] = 1;
        return n * page_len_;
    }
    /* Call before appending at `pos` of `row` (the page must be reserved).  If the page is shared with another row,
     * the row gets a private page and *from / *to name the physical pages whose records the caller must copy
     * (battn_pages_copy) before the append; otherwise both are -1.  False when no page is free. */
    bool make_writable(int row, int pos, int* from, int* to) {
        *from = *to = -1;
        int& p = at(row, pos / page_len_);
        if (ref_[(size_t)p] <= 1) return true;
        if (free_.empty()) return false;
        const int q = free_.back();
        free_.pop_back();
        --ref_[(size_t)p];
        ref_[(size_t)q] = 1;
        *from = p; *to = q;
        p = q;
        dirty_[(size_t)row] = 1;
        return true;
    }
    /* Drops the row's pages; a page returns to the pool when its last row lets go of it. */
    void release(int row) {
        for (int i = 0; i < used_[(size_t)row]; ++i) {
            int& p = at(row, i);
            if (--ref_[(size_t)p] == 0) free_.push_back(p);
            p = -1;
        }
        used_[(size_t)row] = 0;
        dirty_[(size_t)row] = 1;
    }
    const int* table() const { return table_.data(); }                  /* [n_rows][max_pages], -1 = unmapped */
    const int* row(int r) const { return table_.data() + (size_t)r * max_pages_; }
    int pages_of(int r) const { return used_[(size_t)r]; }
    int capacity_of(int r) const { return used_[(size_t)r] * page_len_; }
    int free_pages() const { return (int)free_.size(); }
    int refcount(int page) const { return ref_[(size_t)page]; }
    bool take_dirty(int r) { const bool d = dirty_[(size_t)r] != 0; dirty_[(size_t)r] = 0; return d; }

private:
    int& at(int r, int i) { return table_[(size_t)r * max_pages_ + i]; }
    int page_len_, max_pages_;
    std::vector<int> table_, used_, ref_;
    std::vector<char> dirty_;
    std::vector<int> free_;
};

/* ---- the step scheduler ----------------------------------------------------------------------------------------- */
struct SchedConfig {
    int max_rows = 64;          /* decode rows fused into one step (the reference stops at 8, bruce.cu:94)          */
    int chunk_solo = 512;       /* prompt rows per chunk when nothing else runs              (MBUF)                */
    int chunk_shared = 384;     /* ... while other slots decode and this is the only prompt  (session.h:48)        */
    int chunk_burst = 512;      /* ... while several prompts are queued                       (session.h:49)        */
    int batch_wait_us = 2000;   /* grace period to fuse decode submits still in flight        (session.h:50)        */
};

struct SchedStats {
    long long steps = 0, rows = 0, prefill_chunks = 0, verify_rounds = 0, wait_us = 0;
};

class StepScheduler {
public:
    StepScheduler(StepEngine* eng, SchedConfig cfg = SchedConfig()) : eng_(eng), cfg_(cfg) {}
    ~StepScheduler() { shutdown(); }

    void start() { th_ = std::thread([this] { run(); }); }
    void shutdown() {
        { std::lock_guard<std::mutex> lk(mu_); stop_ = true; }
        cv_work_.notify_all();
        if (th_.joinable()) th_.join();
    }

    /* a request holds a slot between enter() and leave(), and is between enter_decode() and leave_decode() while it
     * generates: the scheduler waits for that many decode submits before it launches a step (session.h:64-68) */
    void enter() { std::lock_guard<std::mutex> lk(mu_); ++active_; }
    void leave() { std::lock_guard<std::mutex> lk(mu_); --active_; }
    void enter_decode() { std::lock_guard<std::mutex> lk(mu_); ++decoders_; }
    void leave_decode() { std::lock_guard<std::mutex> lk(mu_); --decoders_; }
    bool solo() { std::lock_guard<std::mutex> lk(mu_); return active_ <= 1; }

    /* Blocking submits, called from request threads.  decode() returns the row's greedy next token. */
    int decode(int slot, int tok, int pos) {
        auto j = std::make_shared<Job>();
        j->kind = Job::DECODE; j->slot = slot; j->toks.assign(1, tok); j->pos = pos;
        submit(j);
        return j->argmax.empty() ? -1 : j->argmax[0];
    }
    void prefill(int slot, const std::vector<int>& toks, int pos, bool need_logits) {
        auto j = std::make_shared<Job>();
        j->kind = Job::PREFILL; j->slot = slot; j->toks = toks; j->pos = pos; j->need_logits = need_logits;
        submit(j);
    }
    std::vector<int> verify(int slot, const std::vector<int>& toks, int pos) {
        auto j = std::make_shared<Job>();
        j->kind = Job::VERIFY; j->slot = slot; j->toks = toks; j->pos = pos;
        submit(j);
        return j->argmax;
    }
    SchedStats stats() { std::lock_guard<std::mutex> lk(mu_); return stats_; }

    /* The chunk policy on its own (session.h:196-207): rows of the next chunk of a prompt with `remaining` rows,
     * given how many requests hold a slot and how many of them are generating. */
    static int next_chunk(const SchedConfig& c, int active, int decoders, int remaining) {
        const int pending = active - decoders;                   /* requests still ingesting their prompt */
        int chunk = (decoders > 0 && pending <= 1) ? c.chunk_shared : c.chunk_burst;
        if (pending <= 0) chunk = c.chunk_solo;
        return std::max(1, std::min(chunk, remaining));
    }

private:
    struct Job {
        enum Kind { DECODE, PREFILL, VERIFY } kind = DECODE;
        int slot = 0, pos = 0;
        std::vector<int> toks, argmax;
        bool need_logits = true, done = false;
    };
    using JobP = std::shared_ptr<Job>;

    void submit(const JobP& j) {
        std::unique_lock<std::mutex> lk(mu_);
        q_.push_back(j);
        cv_work_.notify_one();
        cv_done_.wait(lk, [&] { return j->done; });
    }
    void finish(const JobP& j) {
        { std::lock_guard<std::mutex> lk(mu_); j->done = true; }
        cv_done_.notify_all();
    }
    /* moves every queued decode job (up to max_rows in total) into `batch`; caller holds the lock.  Two rows of one
     * slot never share a step: the second waits for the next one. */
    void steal_decodes(std::vector<JobP>& batch) {
        for (auto it = q_.begin(); it != q_.end() && (int)batch.size() < cfg_.max_rows;) {
            bool dup = false;
            if ((*it)->kind == Job::DECODE)
                for (const auto& b : batch) dup = dup || b->slot == (*it)->slot;
            if ((*it)->kind == Job::DECODE && !dup) { batch.push_back(*it); it = q_.erase(it); }
            else ++it;
        }
    }
    /* everything already queued plus, for up to batch_wait_us, the submits still in flight from the other generating
     * requests: without the grace period every request would arrive just after the previous step ended and every
     * step would run with one row (session.h:141-165) */
    std::vector<JobP> gather(std::vector<JobP> batch) {
        const auto t0 = std::chrono::steady_clock::now();
        std::unique_lock<std::mutex> lk(mu_);
        const auto deadline = t0 + std::chrono::microseconds(std::max(0, cfg_.batch_wait_us));
        for (;;) {
            steal_decodes(batch);
            if ((int)batch.size() >= cfg_.max_rows || (int)batch.size() >= decoders_) break;
            if (cfg_.batch_wait_us <= 0 || stop_) break;
            if (cv_work_.wait_until(lk, deadline) == std::cv_status::timeout) { steal_decodes(batch); break; }
        }
        stats_.wait_us += std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
        return batch;
    }
    void run_decodes(std::vector<JobP> batch) {
        if (batch.empty()) return;
        const int rows = (int)batch.size();
        std::vector<int> toks(rows), pos(rows), slots(rows), amax(rows, -1);
        for (int i = 0; i < rows; ++i) { toks[i] = batch[i]->toks[0]; pos[i] = batch[i]->pos; slots[i] = batch[i]->slot; }
        eng_->decode_step(rows, toks.data(), pos.data(), slots.data(), amax.data());
        { std::lock_guard<std::mutex> lk(mu_); stats_.steps += 1; stats_.rows += rows; }
        for (int i = 0; i < rows; ++i) { batch[i]->argmax.assign(1, amax[i]); finish(batch[i]); }
    }
    void run_prefill(const JobP& j) {
        const int n = (int)j->toks.size();
        int done = 0;
        while (done < n) {
            int chunk;
            { std::lock_guard<std::mutex> lk(mu_); chunk = next_chunk(cfg_, active_, decoders_, n - done); }
            const bool last = done + chunk == n;
            eng_->prefill_chunk(j->slot, j->toks.data() + done, chunk, j->pos + done, last && j->need_logits);
            done += chunk;
            std::vector<JobP> dec;
            { std::lock_guard<std::mutex> lk(mu_); stats_.prefill_chunks += 1; steal_decodes(dec); }
            if (!dec.empty()) run_decodes(gather(std::move(dec)));       /* waiting decodes get a step between chunks */
        }
    }
    void run() {
        for (;;) {
            JobP j;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_work_.wait(lk, [&] { return stop_ || !q_.empty(); });
                if (q_.empty()) { if (stop_) return; continue; }
                j = q_.front();
                q_.pop_front();
            }
            if (j->kind == Job::DECODE) {
                std::vector<JobP> b; b.push_back(j);
                run_decodes(gather(std::move(b)));
            } else if (j->kind == Job::PREFILL) {
                run_prefill(j);
                finish(j);
            } else {
                j->argmax.assign(j->toks.size(), -1);
                eng_->verify_round(j->slot, j->toks.data(), (int)j->toks.size(), j->pos, j->argmax.data());
                { std::lock_guard<std::mutex> lk(mu_); stats_.verify_rounds += 1; }
                finish(j);
            }
        }
    }

    StepEngine* eng_;
    SchedConfig cfg_;
    std::mutex mu_;
    std::condition_variable cv_work_, cv_done_;
    std::deque<JobP> q_;
    std::thread th_;
    bool stop_ = false;
    int active_ = 0, decoders_ = 0;
    SchedStats stats_;
};

/* ---- prompt-lookup drafter ------------------------------------------------------------------------------------------ */
class NgramDrafter {
public:
    explicit NgramDrafter(int draft_max = 7, int ngram_max = 4, int ngram_min = 1)
        : dmax_(draft_max), nmax_(std::min(ngram_max, 11)), nmin_(std::max(1, ngram_min)) {}

    void clear() { for (auto& t : tab_) t.clear(); hist_.clear(); last_.clear(); }
    int draft_max() const { return dmax_; }
    int matched_ngram() const { return last_.empty() ? 0 : lastg_; }

    /* Append a token; afterwards draft() is the continuation of the most recent EARLIER occurrence of the longest
     * suffix (ngram_max down to ngram_min tokens) that has one.  A continuation shorter than draft_max repeats
     * periodically.  Drafts are always verified by the model: a hash collision costs speed, never correctness. */
    void push(int t) {
        hist_.push_back(t);
        const int n = (int)hist_.size();
        last_.clear();
        for (int g = nmax_; g >= nmin_ && last_.empty(); --g) {
            if (n < g) continue;
            auto it = tab_[g].find(hash(&hist_[(size_t)(n - g)], g));      /* looked up before this position is entered */
            if (it == tab_[g].end()) continue;
            const int j = it->second;                                     /* last token of the earlier occurrence */
            if (j + 1 >= n) continue;
            lastg_ = g;
            const int span = n - 1 - j;                                   /* tokens known to follow it */
            for (int i = 0; i < dmax_; ++i)
                last_.push_back(hist_[(size_t)(j + 1 + (j + 1 + i <= n - 1 ? i : i % span))]);
        }
        for (int g = nmin_; g <= nmax_; ++g)
            if (n >= g) tab_[g][hash(&hist_[(size_t)(n - g)], g)] = n - 1;
    }
    std::vector<int> draft() const {
        return std::vector<int>(last_.begin(), last_.begin() + std::min((int)last_.size(), dmax_));
    }

private:
    static uint64_t hash(const int* p, int n) {                           /* FNV-1a over the token ids */
        uint64_t k = 1469598103934665603ull;
        for (int i = 0; i < n; ++i) { k ^= (uint64_t)(uint32_t)p[i]; k *= 1099511628211ull; }
        return k;
    }
    std::unordered_map<uint64_t, int> tab_[12];
    std::vector<int> hist_, last_;
    int dmax_, nmax_, nmin_, lastg_ = 0;
};

/* ---- one speculative round -------------------------------------------------------------------------------------------- */
struct SpecOutcome {
    int accepted = 0;            /* drafts the model agreed with (0 .. k)                                      */
    int next_token = -1;         /* the model's token after the accepted prefix (argmax of row `accepted`)     */
    int rows = 0;                /* rows verified in this round (k + 1), 0 if no draft was available           */
};

class SpecRound {
public:
    explicit SpecRound(int draft_max = 7) : kmax_(draft_max), dmax_(draft_max) {}
    int kmax() const { return kmax_; }

    /* How many of `drafts` to verify this round: the adaptive length, capped by the tokens the request may still
     * produce (max_tokens - produced - 1, session.h:653-655). */
    int plan(int n_drafts, int tokens_left) const { return std::max(0, std::min({n_drafts, kmax_, tokens_left - 1})); }

    /* Rows of the round: the accepted token t followed by k drafts, at positions pos .. pos+k. */
    static std::vector<int> rows(int t, const std::vector<int>& drafts, int k) {
        std::vector<int> r;
        r.reserve((size_t)k + 1);
        r.push_back(t);
        for (int i = 0; i < k; ++i) r.push_back(drafts[(size_t)i]);
        return r;
    }
    /* argmax[i] = the model's next token after row i.  Draft i is accepted while argmax[i] == drafts[i]; the first
     * disagreement ends the prefix.  The draft length adapts: +1 after a fully accepted round, -1 (not below 1)
     * after a round that accepted nothing (session.h:676-682).  The cache then holds pos .. pos+accepted, so the
     * request's position advances by accepted + 1. */
    SpecOutcome judge(const std::vector<int>& drafts, int k, const int* argmax) {
        SpecOutcome o;
        o.rows = k + 1;
        int j = k;
        for (int i = 0; i < k; ++i)
            if (argmax[i] != drafts[(size_t)i]) { j = i; break; }
        if (j == k) kmax_ = std::min(dmax_, kmax_ + 1);
        else if (j == 0) kmax_ = std::max(1, kmax_ - 1);
        o.accepted = j;
        o.next_token = argmax[j];
        return o;
    }

private:
    int kmax_, dmax_;
};

/* ---- one captured launch sequence per row count ------------------------------------------------------------------------- */
/* `Graph` is whatever the host replays (a cudaGraphExec_t wrapper); `capture(rows)` records the launches of a verify
 * round of that many rows and returns it.  Graphs are built on first use (or all at once with warm()) and replayed
 * afterwards: positions are device-resident, so one graph per row count serves every round. */
template <typename Graph>
class RowGraphs {
public:
    RowGraphs(int min_rows, int max_rows, std::function<Graph(int)> capture)
        : lo_(min_rows), graphs_((size_t)(max_rows - min_rows + 1)), built_((size_t)(max_rows - min_rows + 1), 0),
          capture_(std::move(capture)) {}
    void warm() { for (int r = lo_; r < lo_ + (int)graphs_.size(); ++r) get(r); }
    Graph& get(int rows) {
        const size_t i = (size_t)(rows - lo_);
        if (!built_.at(i)) { graphs_[i] = capture_(rows); built_[i] = 1; ++captures_; }
        return graphs_[i];
    }
    int captures() const { return captures_; }

private:
    int lo_;
    std::vector<Graph> graphs_;
    std::vector<char> built_;
    std::function<Graph(int)> capture_;
    int captures_ = 0;
};

}  /* namespace battn_sched */
#endif /* BATTN_SCHED_H */
