// The scheduler above step(): admits requests, cuts prompts into portions under a token budget,
// decodes, finishes and frees.
//
// It is the reference's server loop without sockets (src/kipp_server.c): FIFO admission with
// head-of-line blocking (:2514-2531), a prompt portion for each request still prefilling beside
// one token for each decoding request (step_eval, :2044-2125), sample-then-eval (:2533-2535),
// "stop" on a stop token (the token is not kept, :1937-1940) and "length" when max_tokens are
// made (:1970-1971).  Where the reference gives every prefilling request a fixed 32-token
// portion and has no budget (:62, docs/ROADMAP.md:19-20), this one fills a per-step token
// budget: decoded tokens first, then prompt portions in arrival order.
//
// What happens when pages run out is decided by the `preempt` option:
//   0 (the reference's rule, src/kipp_server.c:1736-1777): a request is admitted only if every
//     group's free pages cover its own peak need plus what the running requests may still take;
//     so a step can never fail for pages, and requests wait in the queue instead.
//   1: a request is admitted as soon as its first portion fits.  If a later step does not fit,
//     the youngest running request is put back at the head of the queue, its pages are freed,
//     and it is recomputed from its prompt plus the tokens it had generated; the oldest request
//     always proceeds.
//
// The scheduler talks to the cache manager only (host bookkeeping) and never to the device, so
// its decisions are tested without a GPU.
#pragma once
#include <deque>

#include "engine.hpp"

namespace kipp {

constexpr int RECENT_WINDOW = 64;   // tokens the penalties look back over (src/kipp_server.c:869-887)

struct SchedulerHost {
    void* cm = nullptr;                      // the cache manager (cache_core.h)
    int page_size = 16;
    std::vector<int> group_pages;
    std::vector<int> group_windows;          // 0: every key is kept
    int max_requests = 1;
    int max_batch_tokens = 1;
    long long max_positions = 0;             // 0: no limit
    std::function<void(int64_t)> admit;      // take a slot (an engine also clears the request's state)
    std::function<void(int64_t)> release;    // give back pages and slot
};

struct GenRequest {
    int64_t id = 0;
    std::vector<int32_t> prompt, output, stop;
    int max_new_tokens = 0;
    kipp_sample_params sampling{};
    std::vector<int32_t> bias_tokens;
    std::vector<float> bias_values;
    std::vector<int32_t> recent;             // the window handed to the sampler
    uint64_t rng_state = 1;
    int state = 0;                           // 0 waiting, 1 running, 2 finished
    int reason = 0;                          // 1 stop, 2 length, 3 abort
    int fed = 0;                             // tokens of prompt + output already in the cache
    long long arrival = 0;
    int preemptions = 0;

    int known() const { return (int)(prompt.size() + output.size()); }
    int pending() const { return known() - fed; }
    int total_budget() const { return (int)prompt.size() + max_new_tokens; }
    int32_t token_at(int i) const {
        return i < (int)prompt.size() ? prompt[(size_t)i] : output[(size_t)i - prompt.size()];
    }
    bool decoding() const { return pending() == 1 && fed >= (int)prompt.size(); }
};

struct PlanEntry {
    GenRequest* request = nullptr;
    int first = 0, n_tokens = 0;
    bool want_last = false;                  // the logits of its last token are sampled
};

struct StepPlan {
    std::vector<PlanEntry> entries;
    int tokens() const {
        int n = 0;
        for (auto& e : entries) n += e.n_tokens;
        return n;
    }
    int sampled() const {
        int n = 0;
        for (auto& e : entries) n += e.want_last;
        return n;
    }
};

class Scheduler {
public:
    Scheduler(SchedulerHost host, const kipp_scheduler_options& o) : host_(std::move(host)) {
        budget_ = o.max_batch_tokens > 0 ? o.max_batch_tokens : host_.max_batch_tokens;
        if (budget_ <= 0) fail(KIPP_E_ARGUMENT, "max_batch_tokens must be positive");
        chunk_ = o.chunk > 0 ? o.chunk : budget_;
        max_running_ = o.max_running > 0 ? std::min(o.max_running, host_.max_requests) : host_.max_requests;
        max_positions_ = o.max_positions > 0 ? o.max_positions : host_.max_positions;
        if (host_.max_positions > 0 && max_positions_ > host_.max_positions) max_positions_ = host_.max_positions;
        preempt_ = o.preempt != 0;
    }

    long long stat_preemptions = 0, stat_steps = 0, stat_admitted = 0, stat_tokens_fed = 0, stat_tokens_sampled = 0;

    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    const std::deque<GenRequest*>& waiting() const { return waiting_; }
    const std::vector<GenRequest*>& running() const { return running_; }
    const std::vector<GenRequest*>& finished() const { return finished_; }
    int budget() const { return budget_; }

    void submit(const kipp_generation_request& r) {
        if (all_.count(r.id)) fail(KIPP_E_ARGUMENT, format("request %lld is already known", (long long)r.id));
        if (r.n_prompt <= 0 || !r.prompt) fail(KIPP_E_ARGUMENT, "a request needs at least one prompt token");
        if (r.max_new_tokens < 0) fail(KIPP_E_ARGUMENT, "max_new_tokens must not be negative");
        const kipp_sample_params& p = r.sampling;
        if (!(p.top_p > 0.f && p.top_p <= 1.f)) fail(KIPP_E_ARGUMENT, "top_p must be greater than 0 and at most 1");
        if (!(p.min_p >= 0.f && p.min_p <= 1.f)) fail(KIPP_E_ARGUMENT, "min_p must be between 0 and 1");
        if (p.top_k < 0) fail(KIPP_E_ARGUMENT, "top_k must not be negative");
        if (p.temperature > 0.f && r.seed == 0) fail(KIPP_E_ARGUMENT, "sampling requires a nonzero seed");
        auto q = std::make_unique<GenRequest>();
        q->id = r.id;
        q->prompt.assign(r.prompt, r.prompt + r.n_prompt);
        q->max_new_tokens = r.max_new_tokens;
        if (max_positions_ > 0 && q->total_budget() > max_positions_)
            // the reference rejects prompt + max_tokens > context (src/kipp_server.c:1676-1684)
            fail(KIPP_E_ARGUMENT, format("request %lld: prompt + max_new_tokens (%d) exceeds the context of %lld",
                                         (long long)r.id, q->total_budget(), max_positions_));
        for (size_t g = 0; g < host_.group_pages.size(); ++g)
            if (peak_pages((int)g, q->total_budget()) > host_.group_pages[g])
                fail(KIPP_E_ARGUMENT, format("request %lld can never fit: it needs more pages than group %zu has (%d)",
                                             (long long)r.id, g, host_.group_pages[g]));
        q->sampling = p;
        if (p.logit_bias_count > 0) {
            q->bias_tokens.assign(p.logit_bias_tokens, p.logit_bias_tokens + p.logit_bias_count);
            q->bias_values.assign(p.logit_bias_values, p.logit_bias_values + p.logit_bias_count);
        }
        q->sampling.recent_tokens = nullptr;
        q->sampling.recent_count = 0;
        if (r.n_stop_tokens > 0) q->stop.assign(r.stop_tokens, r.stop_tokens + r.n_stop_tokens);
        q->rng_state = r.seed ? r.seed : 1;          // never 0 (src/kipp_server.c:1852-1862)
        q->arrival = arrivals_++;
        waiting_.push_back(q.get());
        all_[r.id] = std::move(q);
    }

    // The next step's batch; empty when nothing can run.
    StepPlan schedule() {
        admit_waiting();
        while (true) {
            if (running_.empty()) return {};
            StepPlan plan = make_plan();
            if (plan.entries.empty()) return {};
            if (fits(plan)) {
                ++stat_steps;
                return plan;
            }
            if (!preempt_) fail(KIPP_E_STATE, "reservation failed to keep a step within the pool");
            if (preempt_youngest()) continue;
            // one request alone does not fit: shrink its portion to what does
            PlanEntry e = plan.entries[0];
            GenRequest* r = e.request;
            long long room = -1;
            for (size_t g = 0; g < host_.group_pages.size(); ++g) {
                const long long free_tokens = (long long)free_pages((int)g) * host_.page_size;
                room = room < 0 ? free_tokens : std::min(room, free_tokens);
            }
            room = std::max<long long>(room, 0) + (host_.page_size - r->fed % host_.page_size) % host_.page_size;
            if (room <= 0) fail(KIPP_E_OUT_OF_PAGES, format("request %lld cannot grow: the pool is exhausted", (long long)r->id));
            const int n = (int)std::min<long long>(e.n_tokens, room);
            const bool last = r->fed + n == r->known();
            StepPlan small;
            small.entries.push_back({r, r->fed, n, last && e.want_last});
            if (!fits(small))
                fail(KIPP_E_OUT_OF_PAGES, format("request %lld cannot grow: the pool is exhausted", (long long)r->id));
            ++stat_steps;
            return small;
        }
    }

    // Records a finished step: tokens[i] is the token sampled for the i-th entry with want_last.
    // The cache manager's lengths must already have advanced (the step does that).
    void complete(const StepPlan& plan, const int32_t* tokens, int n_tokens) {
        if (n_tokens != plan.sampled()) fail(KIPP_E_ARGUMENT, "one sampled token per sampled entry");
        for (auto& e : plan.entries) e.request->fed += e.n_tokens;
        stat_tokens_fed += plan.tokens();
        stat_tokens_sampled += n_tokens;
        std::vector<GenRequest*> done;
        int k = 0;
        for (auto& e : plan.entries) {
            if (!e.want_last) continue;
            GenRequest* r = e.request;
            const int32_t tok = tokens[k++];
            if (std::find(r->stop.begin(), r->stop.end(), tok) != r->stop.end()) {
                r->reason = 1;                                   // the stop token is not kept
            } else {
                r->output.push_back(tok);
                if ((int)r->output.size() >= r->max_new_tokens) r->reason = 2;
                else if (max_positions_ > 0 && r->known() >= max_positions_) r->reason = 2;
            }
            if (r->reason) done.push_back(r);
        }
        for (GenRequest* r : running_)
            if (!r->reason && r->max_new_tokens == 0 && r->pending() == 0) {
                r->reason = 2;
                done.push_back(r);
            }
        for (GenRequest* r : done) finish(r);
    }

    void abort(int64_t id) {
        GenRequest* r = find(id);
        if (r->state == 2) return;
        r->reason = 3;
        if (r->state == 1) {
            finish(r);
        } else {
            waiting_.erase(std::find(waiting_.begin(), waiting_.end(), r));
            r->state = 2;
            finished_.push_back(r);
        }
    }
    void poll(int64_t id, kipp_generation_state* out) {
        GenRequest* r = find(id);
        out->id = id;
        out->finished = r->state == 2;
        out->reason = r->reason;
        out->n_tokens = (int)r->output.size();
        out->preemptions = r->preemptions;
    }
    void output(int64_t id, int32_t* tokens, int capacity, int* n) {
        GenRequest* r = find(id);
        const int count = (int)r->output.size();
        if (n) *n = count;
        for (int i = 0; i < count && i < capacity; ++i) tokens[i] = r->output[(size_t)i];
    }
    void forget(int64_t id) {
        GenRequest* r = find(id);
        if (r->state != 2) fail(KIPP_E_STATE, format("request %lld has not finished", (long long)id));
        finished_.erase(std::find(finished_.begin(), finished_.end(), r));
        all_.erase(id);
    }
    GenRequest* find(int64_t id) {
        auto it = all_.find(id);
        if (it == all_.end()) fail(KIPP_E_ARGUMENT, format("request %lld is not known", (long long)id));
        return it->second.get();
    }

    // Most pages a request of total_tokens holds at any time when no step brings more than the
    // step cap of it.
    int peak_pages(int group, int total_tokens) const {
        const int page = host_.page_size;
        const int full = (total_tokens + page - 1) / page;
        const int window = host_.group_windows[(size_t)group];
        if (window <= 0) return full;
        const int span = window - 1 + step_cap();
        return std::min(full, (span + page - 1) / page + 1);
    }

private:
    SchedulerHost host_;
    int budget_ = 0, chunk_ = 0, max_running_ = 0;
    long long max_positions_ = 0;
    bool preempt_ = false;
    long long arrivals_ = 0;
    std::map<int64_t, std::unique_ptr<GenRequest>> all_;
    std::deque<GenRequest*> waiting_;
    std::vector<GenRequest*> running_, finished_;

    int step_cap() const { return std::min(chunk_, budget_); }
    int free_pages(int g) const { return kipp_pool_free_pages(kipp_cm_pool(host_.cm, g)); }
    int free_slots() const { return kipp_slots_free_count(kipp_cm_slots(host_.cm)); }

    // pages the running requests may still take in a group
    int outstanding(int g) const {
        int total = 0;
        std::vector<int> held(host_.group_pages.size() + 1);
        for (GenRequest* r : running_) {
            kipp_cm_pages_held(host_.cm, r->id, held.data());
            total += std::max(0, peak_pages(g, r->total_budget()) - held[(size_t)g]);
        }
        return total;
    }
    bool can_admit(const GenRequest& r) const {
        if ((int)running_.size() >= max_running_ || free_slots() == 0) return false;
        for (int g = 0; g < (int)host_.group_pages.size(); ++g) {
            if (!preempt_) {
                if (free_pages(g) < peak_pages(g, r.total_budget()) + outstanding(g)) return false;
            } else {
                const int first = std::min(r.pending(), step_cap());
                if (free_pages(g) < (first + host_.page_size - 1) / host_.page_size) return false;
            }
        }
        return true;
    }
    void admit_waiting() {
        while (!waiting_.empty() && can_admit(*waiting_.front())) {     // head-of-line blocking
            GenRequest* r = waiting_.front();
            waiting_.pop_front();
            host_.admit(r->id);
            r->state = 1;
            r->fed = 0;
            running_.push_back(r);
            ++stat_admitted;
        }
    }
    StepPlan make_plan() const {
        StepPlan plan;
        int budget = budget_;
        // decoding requests first: one token each
        for (GenRequest* r : running_)
            if (r->decoding() && budget > 0) {
                plan.entries.push_back({r, r->fed, 1, true});
                --budget;
            }
        // then prompt portions (and recomputation after a preemption) in arrival order
        for (GenRequest* r : running_) {
            if (budget <= 0) break;
            if (r->decoding()) continue;
            const int n = std::min({r->pending(), chunk_, budget});
            if (n <= 0) continue;
            const bool last = r->fed + n == r->known();
            plan.entries.push_back({r, r->fed, n, last && (int)r->output.size() < r->max_new_tokens});
            budget -= n;
        }
        return plan;
    }
    bool fits(const StepPlan& plan) const {
        std::vector<int> need(host_.group_pages.size(), 0), missing(host_.group_pages.size() + 1);
        for (auto& e : plan.entries) {
            kipp_cm_missing_pages(host_.cm, e.request->id, e.request->fed + e.n_tokens, missing.data());
            for (size_t g = 0; g < need.size(); ++g) need[g] += missing[g];
        }
        for (size_t g = 0; g < need.size(); ++g)
            if (need[g] > free_pages((int)g)) return false;
        return true;
    }
    bool preempt_youngest() {
        if (running_.size() <= 1) return false;
        auto it = std::max_element(running_.begin(), running_.end(),
                                   [](GenRequest* a, GenRequest* b) { return a->arrival < b->arrival; });
        GenRequest* victim = *it;
        running_.erase(it);
        host_.release(victim->id);
        victim->state = 0;
        victim->fed = 0;
        ++victim->preemptions;
        ++stat_preemptions;
        waiting_.push_front(victim);
        return true;
    }
    void finish(GenRequest* r) {
        r->state = 2;
        running_.erase(std::find(running_.begin(), running_.end(), r));
        host_.release(r->id);                          // pages and slot go back at once
        finished_.push_back(r);
    }
};

inline SchedulerHost engine_scheduler_host(Engine& e) {
    SchedulerHost h;
    h.cm = e.cache_manager();
    h.page_size = e.options().page_size;
    for (int g = 0; g < e.groups(); ++g) {
        h.group_pages.push_back(e.group_pages(g));
        h.group_windows.push_back(e.group_window(g));
    }
    h.max_requests = e.options().max_requests;
    h.max_batch_tokens = e.options().max_batch_tokens;
    h.max_positions = e.max_positions();
    h.admit = [&e](int64_t rid) { e.add_request(rid); };
    h.release = [&e](int64_t rid) { e.finish(rid); };
    return h;
}

// Whether the planned step can be the first of a burst (Engine::decode_burst: greedy steps whose
// tokens are fed back on the device): every running request is in the plan with one decoded
// token, is greedy without penalties, bias or stop tokens (nothing the host would have to look at
// between steps).  Returns the number of steps until the first request ends (0: no burst).
inline int burst_length(const Scheduler& sched, const StepPlan& plan, long long max_positions) {
    if (plan.entries.size() != sched.running().size()) return 0;
    int steps = 1 << 30;
    for (auto& e : plan.entries) {
        const GenRequest& r = *e.request;
        const kipp_sample_params& p = r.sampling;
        if (e.n_tokens != 1 || !e.want_last || !r.decoding()) return 0;
        if (p.temperature > 0.f || p.frequency_penalty != 0.f || p.presence_penalty != 0.f ||
            (p.repetition_penalty != 0.f && p.repetition_penalty != 1.f) || !r.bias_tokens.empty() || !r.stop.empty())
            return 0;
        steps = std::min(steps, r.max_new_tokens - (int)r.output.size());
        if (max_positions > 0) steps = std::min<long long>(steps, max_positions - r.known());
    }
    return steps;
}

// Drives the scheduler until no request is left (or max_steps steps ran): plan, step, sample,
// record.  Token ids go to the device with each step's metadata and the sampled ids come back to
// the host after each step; where nothing has to be looked at between steps (burst_length) a run
// of decode steps goes as one burst and its tokens come back together.  Returns the steps run.
inline int run_scheduler(Engine& engine, Scheduler& sched, int max_steps, bool bursts = true) {
    int steps = 0;
    std::vector<StepEntryView> views;
    std::vector<std::vector<int32_t>> tokens;
    std::vector<int32_t> want;
    std::vector<kipp_sample_params> params;
    std::vector<uint64_t> states;
    std::vector<int32_t> sampled;
    while (sched.has_work() && (max_steps <= 0 || steps < max_steps)) {
        StepPlan plan = sched.schedule();
        if (plan.entries.empty()) fail(KIPP_E_STATE, "requests are waiting but none can be admitted");
        const size_t n = plan.entries.size();
        int burst = bursts ? burst_length(sched, plan, engine.max_positions()) : 0;
        if (max_steps > 0) burst = std::min(burst, max_steps - steps);
        if (burst >= 2) {
            std::vector<int64_t> rids(n);
            std::vector<int32_t> first(n), ring((size_t)burst * n);
            for (size_t i = 0; i < n; ++i) {
                rids[i] = plan.entries[i].request->id;
                first[i] = plan.entries[i].request->token_at(plan.entries[i].first);
            }
            bool ran = true;
            try {
                engine.decode_burst(rids.data(), first.data(), (int)n, burst, ring.data());
            } catch (const Error& e) {
                if (e.code != KIPP_E_OUT_OF_PAGES) throw;
                ran = false;                 // the pages of all steps cannot be had at once: step by step
            }
            if (ran) {
                for (int k = 0; k < burst; ++k) {
                    if (k > 0) {
                        plan = sched.schedule();
                        if (plan.entries.size() != n) fail(KIPP_E_STATE, "the batch changed inside a burst");
                    }
                    // the ring's columns follow the order of the burst's requests
                    sampled.resize(n);
                    for (size_t i = 0; i < n; ++i) {
                        size_t col = 0;
                        while (rids[col] != plan.entries[i].request->id) ++col;
                        sampled[i] = ring[(size_t)k * n + col];
                    }
                    sched.complete(plan, sampled.data(), (int)n);
                }
                steps += burst;
                continue;
            }
        }
        views.resize(n);
        tokens.resize(n);
        want.resize(n);
        for (size_t i = 0; i < n; ++i) {
            const PlanEntry& e = plan.entries[i];
            tokens[i].resize((size_t)e.n_tokens);
            for (int t = 0; t < e.n_tokens; ++t) tokens[i][(size_t)t] = e.request->token_at(e.first + t);
            want[i] = e.n_tokens - 1;
            views[i] = {e.request->id, tokens[i].data(), e.n_tokens, &want[i], e.want_last ? 1 : 0};
        }
        int rows = 0;
        engine.step(views.data(), (int)n, &rows);
        params.clear();
        states.clear();
        std::vector<GenRequest*> rs;
        for (auto& e : plan.entries) {
            if (!e.want_last) continue;
            GenRequest* r = e.request;
            // the window penalties look back over: the last generated tokens
            // (choice_remember_token, src/kipp_server.c:1019-1027)
            const size_t keep = std::min<size_t>(r->output.size(), RECENT_WINDOW);
            r->recent.assign(r->output.end() - (long)keep, r->output.end());
            kipp_sample_params p = r->sampling;
            p.recent_tokens = r->recent.data();
            p.recent_count = (int)r->recent.size();
            p.logit_bias_tokens = r->bias_tokens.data();
            p.logit_bias_values = r->bias_values.data();
            p.logit_bias_count = (int)r->bias_tokens.size();
            params.push_back(p);
            states.push_back(r->rng_state);
            rs.push_back(r);
        }
        sampled.resize(rs.size());
        if (!rs.empty()) {
            engine.sample(params.data(), states.data(), (int)rs.size(), sampled.data());
            for (size_t i = 0; i < rs.size(); ++i) rs[i]->rng_state = states[i];
        }
        sched.complete(plan, sampled.data(), (int)sampled.size());
        ++steps;
    }
    if (!sched.has_work()) engine.check_status();
    return steps;
}

}  // namespace kipp
