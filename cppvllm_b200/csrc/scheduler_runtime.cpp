// The scheduler in C++: requests with their tokens and counters, admission, prompts cut into portions under a token
// budget, decoding, preemption by recomputation when pages run out, finishing and freeing; with the steps in flight that
// the engine's pipeline keeps (a token sampled by the step in flight is a placeholder on the host and travels on the
// device).  The decisions are those of engine/scheduler.py, which stays as the plain twin that the tests compare this
// with step by step (and which is compared with the reference's own scheduler, engine/scheduler.cpp:36-151, through the
// golden batches).  The cache manager is called directly (runtime.hpp).  Plain C entry points, called through ctypes.
#include <algorithm>
#include <deque>
#include <unordered_set>

#include "runtime.hpp"

using namespace cvb_rt;

namespace {

constexpr int kPending = -1;          // a token that was sampled on the device and has not been read back yet
enum Status : int { kWaiting = 0, kRunning = 1, kFinished = 2 };

struct Seq {
    int id = 0;
    std::vector<int> tokens;          // prompt, then generated (placeholders included)
    int prompt_len = 0, cached = 0, scheduled = 0, max_tokens = 0, inflight = 0, preemptions = 0;
    int slot = -1, capacity = 0, status = kWaiting, sampler_index = -1;
    bool ignore_eos = false, stopped_on_eos = false;
    float temperature = 0.f;
    unsigned long long seed = 0;
    int len() const { return static_cast<int>(tokens.size()); }
};

struct Launched {                      // a step that was handed to the device
    std::vector<int> ids, sample_pos;  // per sequence: index of its placeholder in its tokens, or -1
};

struct Sched {
    void* cm = nullptr;                // the cache manager (not owned)
    int budget = 0, max_seqs = 0, chunk_cap = 0, max_model_len = 0, page_size = 0, smallest_pool = 0;
    std::unordered_set<int> eos;
    std::unordered_map<int, Seq> seqs;
    std::deque<int> waiting;
    std::vector<int> running;
    long long num_preemptions = 0;
    // the batch that schedule() made last, until on_launched() takes it
    std::vector<int> batch, batch_preempted, batch_admitted;
    std::deque<Launched> inflight;

    Seq& at(int id) { return seqs.find(id)->second; }
    void preempt(Seq& s) {
        cvb_cm_release(cm, s.slot);
        s.slot = -1; s.status = kWaiting; s.cached = 0; s.scheduled = 0; s.capacity = 0;
        ++s.preemptions; ++num_preemptions;
        waiting.push_front(s.id);
    }
};

inline Sched* S(void* h) { return static_cast<Sched*>(h); }

}  // namespace

extern "C" {

void* cvb_sched_create(void* cache_manager, int budget, int max_seqs, int chunk_cap, int max_model_len, int page_size,
                       int smallest_pool, const int* eos, int n_eos) {
    if (cache_manager == nullptr || budget <= 0 || max_seqs <= 0 || max_model_len <= 0 || page_size <= 0) return nullptr;
    Sched* s = new Sched();
    s->cm = cache_manager; s->budget = budget; s->max_seqs = max_seqs; s->chunk_cap = chunk_cap;
    s->max_model_len = max_model_len; s->page_size = page_size; s->smallest_pool = smallest_pool;
    for (int i = 0; i < n_eos; ++i) s->eos.insert(eos[i]);
    return s;
}

void cvb_sched_destroy(void* h) { delete S(h); }

// A new request.  -1: it has no prompt; -2: prompt + max_tokens exceed max_model_len; -3: it needs more pages than
// the smallest pool has; -4: the id is in use.
int cvb_sched_add(void* h, int id, const int* prompt, int n, int max_tokens, int ignore_eos, float temperature,
                  unsigned long long seed) {
    Sched* s = S(h);
    if (n <= 0) return -1;
    const int max_len = n + (max_tokens > 0 ? max_tokens : 0);
    if (max_len > s->max_model_len) return -2;
    if ((max_len + s->page_size - 1) / s->page_size > s->smallest_pool) return -3;
    if (s->seqs.count(id)) return -4;
    Seq& q = s->seqs[id];
    q.id = id; q.tokens.assign(prompt, prompt + n); q.prompt_len = n; q.max_tokens = max_tokens;
    q.ignore_eos = ignore_eos != 0; q.temperature = temperature; q.seed = seed;
    s->waiting.push_back(id);
    return 0;
}

int cvb_sched_is_finished(void* h) { return S(h)->waiting.empty() && S(h)->running.empty() ? 1 : 0; }
int cvb_sched_num_waiting(void* h) { return static_cast<int>(S(h)->waiting.size()); }
int cvb_sched_num_running(void* h) { return static_cast<int>(S(h)->running.size()); }
long long cvb_sched_num_preemptions(void* h) { return S(h)->num_preemptions; }
int cvb_sched_queue(void* h, int which, int* out, int max_out) {       // 0: waiting, 1: running (ids, in order)
    Sched* s = S(h);
    int n = 0;
    if (which == 0) { for (int id : s->waiting) if (n < max_out) out[n++] = id; }
    else { for (int id : s->running) if (n < max_out) out[n++] = id; }
    return n;
}

// ---- one step's decisions ---------------------------------------------------------------------------------------------
// The step is planned in two passes over the queues.
//   Pass 1, the running requests: the list is seen through a window [i, live).  Request i is served from the front; when
//   its pages cannot grow, the request at the window's far end (live - 1) gives up everything it holds and waits again,
//   which shrinks the window from behind; if the window has shrunk onto request i itself, it is the one that goes.  With a
//   step in flight nobody may be taken out (allow_preempt 0): the request is left as it is and the plan is marked blocked.
//   What is left of the window afterwards is the new running list.
//   Pass 2, the waiting requests: admitted first come first served while rows, tokens and pages last; not at all in a step
//   that took somebody out or was blocked.
// The policy is the reference's (engine/scheduler.cpp:36-106); the golden batches under tests/golden hold it to that.
struct StepPlan {
    Sched* s;
    int tokens_left;              // of the step's token budget
    int portion_cap;              // longest portion of a prompt in one step
    int total = 0;
    bool blocked = false, took_out = false;

    bool rows_full() const { return static_cast<int>(s->batch.size()) >= s->max_seqs; }
    // how many of its tokens request q would run now: what it has not computed, cut to the cap and to the budget
    int portion(const Seq& q) const { return std::min(std::min(q.len() - q.cached, portion_cap), tokens_left); }
    void take(Seq& q, int n) {
        q.scheduled = n;
        s->batch.push_back(q.id);
        total += n;
        tokens_left -= n;
    }
};

enum class Room { kHasIt, kBlocked, kGaveWay };

// Pages for all of q's tokens (q is running[i]).  May take requests out from the far end of the window.
static Room make_room(StepPlan& plan, Seq& q, size_t i, size_t& live, bool allow_preempt) {
    Sched* s = plan.s;
    const int n_tok = q.len();
    if (n_tok <= q.capacity) return Room::kHasIt;                       // most decode steps need no new page
    while (cvb_cm_can_reserve(s->cm, q.slot, n_tok) <= 0) {
        if (!allow_preempt) return Room::kBlocked;
        Seq& last = s->at(s->running[--live]);                         // live - 1 >= i: at worst q itself
        s->preempt(last);
        s->batch_preempted.push_back(last.id);
        plan.took_out = true;
        if (live == i) return Room::kGaveWay;
    }
    q.capacity = cvb_cm_reserve(s->cm, q.slot, n_tok);
    return Room::kHasIt;
}

static void serve_running(StepPlan& plan, bool allow_preempt) {
    Sched* s = plan.s;
    size_t live = s->running.size();
    for (size_t i = 0; i < live; ++i) {
        Seq& q = s->at(s->running[i]);
        const int generated = q.len() - q.prompt_len;
        if (generated > 0 && generated >= q.max_tokens) continue;      // complete but for the token still in flight
        const int n = plan.portion(q);
        if (n <= 0 || plan.rows_full()) continue;
        const Room room = make_room(plan, q, i, live, allow_preempt);
        if (room == Room::kBlocked) plan.blocked = true;
        else if (room == Room::kHasIt) plan.take(q, n);
    }
    s->running.resize(live);
}

static void admit_waiting(StepPlan& plan) {
    Sched* s = plan.s;
    if (plan.took_out || plan.blocked) return;
    while (!s->waiting.empty() && plan.tokens_left > 0 && static_cast<int>(s->running.size()) < s->max_seqs && !plan.rows_full()) {
        Seq& q = s->at(s->waiting.front());
        if (!cvb_cm_can_admit(s->cm, q.tokens.data(), q.len(), q.len())) return;    // first come first served: nobody overtakes
        s->waiting.pop_front();
        q.slot = cvb_cm_admit(s->cm, q.tokens.data(), q.len());     // with the prefix cache: shared pages count as computed
        q.cached = cvb_rt::manager_computed(s->cm, q.slot);
        q.capacity = cvb_cm_reserve(s->cm, q.slot, q.len());
        q.status = kRunning;
        s->running.push_back(q.id);
        s->batch_admitted.push_back(q.id);
        plan.take(q, plan.portion(q));
    }
}

// info: [sequences, tokens, blocked, preempted, admitted].
int cvb_sched_schedule(void* h, int allow_preempt, int* info) {
    Sched* s = S(h);
    s->batch.clear(); s->batch_preempted.clear(); s->batch_admitted.clear();
    StepPlan plan{s, s->budget, s->chunk_cap > 0 ? s->chunk_cap : 0x7fffffff};
    serve_running(plan, allow_preempt != 0);
    admit_waiting(plan);
    info[0] = static_cast<int>(s->batch.size()); info[1] = plan.total; info[2] = plan.blocked ? 1 : 0;
    info[3] = static_cast<int>(s->batch_preempted.size()); info[4] = static_cast<int>(s->batch_admitted.size());
    return info[0];
}

// What the last schedule() decided, for the step function and the sampler.  Per sequence of the batch: its id, state
// slot, where its tokens start, how many run, whether the step samples for it; the tokens themselves, flat, with 0 in
// place of a placeholder and in feed_src the row of the step in flight whose sample replaces it (-1: keep); for the
// sequences that sample: temperature, seed and the number of tokens generated so far.  `lists`: the ids that were
// preempted, then those that were admitted (with their state slots after them).  Returns the number of sampling rows;
// *need_feed says whether any token comes from the device.
int cvb_sched_batch(void* h, int* ids, int* slots, int* starts, int* counts, int* samples, int* tokens, int* feed_src,
                    float* temps, unsigned long long* seeds, int* generated, int* lists, int* need_feed) {
    Sched* s = S(h);
    int t = 0, r = 0, k = 0;
    *need_feed = 0;
    for (size_t i = 0; i < s->batch.size(); ++i) {
        Seq& q = s->at(s->batch[i]);
        ids[i] = q.id; slots[i] = q.slot; starts[i] = q.cached; counts[i] = q.scheduled;
        const bool samp = q.cached + q.scheduled == q.len();
        samples[i] = samp ? 1 : 0;
        for (int j = 0; j < q.scheduled; ++j) {
            const int tok = q.tokens[q.cached + j];
            tokens[t] = tok == kPending ? 0 : tok;
            feed_src[t] = -1;
            if (tok == kPending) { feed_src[t] = q.sampler_index; *need_feed = 1; }
            ++t;
        }
        if (samp) {
            temps[r] = q.temperature; seeds[r] = q.seed; generated[r] = q.len() - q.prompt_len;
            ++r;
        }
    }
    for (int id : s->batch_preempted) lists[k++] = id;
    for (int id : s->batch_admitted) { lists[k++] = id; lists[k++] = s->at(id).slot; }
    return r;
}

// The step was handed to the device: its tokens count as cached, and every sequence that samples in it gets a
// placeholder for the token that is not known on the host yet.  Returns the number of sampling rows.
int cvb_sched_on_launched(void* h) {
    Sched* s = S(h);
    Launched rec;
    int r = 0;
    for (int id : s->batch) {
        Seq& q = s->at(id);
        const bool samp = q.cached + q.scheduled == q.len();
        q.cached += q.scheduled;
        q.scheduled = 0;
        ++q.inflight;
        rec.ids.push_back(id);
        if (samp) {
            rec.sample_pos.push_back(q.len());
            q.tokens.push_back(kPending);
            q.sampler_index = r++;
        } else {
            rec.sample_pos.push_back(-1);
        }
    }
    s->inflight.push_back(std::move(rec));
    s->batch.clear();
    return r;
}

int cvb_sched_num_inflight(void* h) { return static_cast<int>(S(h)->inflight.size()); }

// The samples of the oldest step in flight arrived (one per sampling sequence, in batch order): they replace the
// placeholders; requests finish (end-of-sequence token unless ignored, or max_tokens) and give back what they hold.
// Results for a request that finished in an earlier step while this one was in flight are dropped.  Returns the number
// of requests that finished (their ids in `finished`), or -1 if no step is in flight or the samples do not match.
int cvb_sched_postprocess(void* h, const int* sampled, int n_sampled, int* finished, int max_finished) {
    Sched* s = S(h);
    if (s->inflight.empty()) return -1;
    Launched rec = std::move(s->inflight.front());
    s->inflight.pop_front();
    int used = 0, n_fin = 0;
    for (size_t i = 0; i < rec.ids.size(); ++i) {
        Seq& q = s->at(rec.ids[i]);
        const int pos = rec.sample_pos[i];
        --q.inflight;
        if (pos < 0) {
            if (q.status != kFinished) cvb_cm_commit(s->cm, q.slot, q.tokens.data(), q.len());   // full pages become shareable
            continue;
        }
        if (used >= n_sampled) return -1;
        const int tok = sampled[used++];
        if (q.status == kFinished) continue;
        q.tokens[pos] = tok;
        const bool hit_eos = !q.ignore_eos && s->eos.count(tok) > 0;
        const bool hit_len = pos + 1 - q.prompt_len >= q.max_tokens;
        if (hit_eos || hit_len) {
            q.tokens.resize(pos + 1);                       // drops the placeholder of a later step that is still in flight
            if (q.cached > q.len()) q.cached = q.len();
            q.stopped_on_eos = hit_eos;
            q.status = kFinished;
            cvb_cm_commit(s->cm, q.slot, q.tokens.data(), q.len());
            cvb_cm_release(s->cm, q.slot);
            q.slot = -1;
            if (n_fin < max_finished) finished[n_fin] = q.id;
            ++n_fin;
        } else {
            cvb_cm_commit(s->cm, q.slot, q.tokens.data(), q.len());
        }
    }
    if (n_fin > 0) {
        std::vector<int> still;
        for (int id : s->running)
            if (s->at(id).status != kFinished) still.push_back(id);
        s->running.swap(still);
    }
    return n_fin;
}

// A request's state: [status, prompt tokens, tokens, cached, scheduled, preemptions, in flight, stopped on eos, slot].
int cvb_sched_seq_info(void* h, int id, int* out) {
    Sched* s = S(h);
    auto it = s->seqs.find(id);
    if (it == s->seqs.end()) return -1;
    const Seq& q = it->second;
    out[0] = q.status; out[1] = q.prompt_len; out[2] = q.len(); out[3] = q.cached; out[4] = q.scheduled;
    out[5] = q.preemptions; out[6] = q.inflight; out[7] = q.stopped_on_eos ? 1 : 0; out[8] = q.slot;
    return 0;
}

int cvb_sched_seq_tokens(void* h, int id, int* out, int max_out) {
    Sched* s = S(h);
    auto it = s->seqs.find(id);
    if (it == s->seqs.end()) return -1;
    const int n = it->second.len() < max_out ? it->second.len() : max_out;
    std::memcpy(out, it->second.tokens.data(), sizeof(int) * n);
    return it->second.len();
}

// Forget a finished request whose result has been taken (it may still be named by a step in flight: then it stays
// until that step has been read back).
int cvb_sched_forget(void* h, int id) {
    Sched* s = S(h);
    auto it = s->seqs.find(id);
    if (it == s->seqs.end() || it->second.status != kFinished) return -1;
    if (it->second.inflight > 0) return 1;
    s->seqs.erase(it);
    return 0;
}

}  // extern "C"
