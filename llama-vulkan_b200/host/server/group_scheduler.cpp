#include "group_scheduler.h"

#include <algorithm>

#include "../llava_context.h"
#include "../llava_session.h"
#include "../llava_session_group.h"

using namespace std;
using namespace lsrv;

namespace {
constexpr auto kWindow = chrono::microseconds(500);      // how long the first caller of a round waits for the other runners
constexpr size_t kCachedGroups = 8;
}  // namespace

group_scheduler::group_scheduler(llava_context* _ctx) : ctx(_ctx) {}

group_scheduler::~group_scheduler() {
    for (auto& [key, g] : groups) delete g;
}

void group_scheduler::runner_enters() {
    lock_guard<mutex> lock(m);
    ++runners;
}

void group_scheduler::runner_leaves() {
    {
        lock_guard<mutex> lock(m);
        if (runners) --runners;
    }
    cv_leader.notify_one();     // a leader may be waiting for a runner that will not come
}

void group_scheduler::settle_locked(llava_session* session) {
    if (ahead_group == nullptr) return;
    const auto& mem = ahead_group->get_members();
    if (find(mem.begin(), mem.end(), session) == mem.end()) return;
    ahead_group->discard_ahead();
    ahead_group = nullptr;
    given.clear();
}

void group_scheduler::settle(llava_session* session) {
    lock_guard<mutex> lock(m);
    settle_locked(session);
}

void group_scheduler::forget(llava_session* session) {
    lock_guard<mutex> lock(m);
    settle_locked(session);
    for (auto it = groups.begin(); it != groups.end();) {
        if (find(it->first.begin(), it->first.end(), session) != it->first.end()) {
            delete it->second;
            it = groups.erase(it);
        } else {
            ++it;
        }
    }
}

u32 group_scheduler::evaluate(llava_session* session) {
    // what a group step cannot serve goes through the session's own step
    const bool groupable = session->get_token_count() - session->get_tokens_in_gpu() == 1 && !session->samples_on_host() &&
                           !session->is_tracing_enabled() && ctx->tp_size() == 1;
    if (!groupable) {
        settle(session);
        return session->predict_next_token();
    }
    unique_lock<mutex> lock(m);
    waiting.push_back(session);
    cv_leader.notify_one();                   // a leader that collects a round counts the callers
    while (results.count(session) == 0) {
        if (!leader_present) {
            // whoever finds no leader leads the next round (it is one of the waiting callers itself)
            leader_present = true;
            lead(lock);                       // collects the round, runs it, publishes the results
            leader_present = false;
            cv_results.notify_all();          // once per round: the callers pick up their tokens, one of the others may lead
        } else {
            cv_results.wait(lock);
        }
    }
    const u32 token = results[session];
    results.erase(session);
    return token;
}

// Called with the lock held by the first caller of a round.
void group_scheduler::lead(unique_lock<mutex>& lock) {
    const auto t_begin = chrono::steady_clock::now();
    const auto deadline = t_begin + kWindow;
    cv_leader.wait_until(lock, deadline, [&]() { return waiting.size() >= max<u32>(runners, 1u) || waiting.size() >= llava_session::max_batch_limit; });
    const auto t_collected = chrono::steady_clock::now();
    us_collect += u64(chrono::duration_cast<chrono::microseconds>(t_collected - t_begin).count());
    struct device_timer {
        std::atomic<u64>& sum;
        chrono::steady_clock::time_point t0;
        ~device_timer() { sum += u64(chrono::duration_cast<chrono::microseconds>(chrono::steady_clock::now() - t0).count()); }
    } timer{us_device, t_collected};
    vector<llava_session*> round;
    round.swap(waiting);
    if (round.size() > llava_session::max_batch_limit) {          // the rest forms the next round
        waiting.assign(round.begin() + llava_session::max_batch_limit, round.end());
        round.resize(llava_session::max_batch_limit);
    }
    vector<u32> tokens(round.size(), ~0U);
    vector<llava_session*> key = round;
    sort(key.begin(), key.end());
    // a step queued ahead: booked if exactly its members came back, each having pushed the token it was handed
    if (ahead_group != nullptr) {
        bool same = key == ahead_group->get_members();
        for (size_t i = 0; same && i < key.size(); ++i) {
            const auto it = given.find(key[i]);
            same = it != given.end() && key[i]->get_token_buffer().back() == it->second;
        }
        llava_session_group* g = ahead_group;
        if (same) {
            ahead_group = nullptr;                          // ours while the lock is released
            lock.unlock();
            vector<u32> by_key;
            const bool ok = g->finish_ahead(&by_key);
            if (ok) {
                for (size_t i = 0; i < round.size(); ++i)
                    tokens[i] = by_key[size_t(lower_bound(key.begin(), key.end(), round[i]) - key.begin())];
                n_grouped_steps += 1;
                n_grouped_tokens += round.size();
                n_steps_ahead += 1;
            }
            const bool again = ok && g->launch_ahead();
            lock.lock();
            given.clear();
            if (again) {
                ahead_group = g;
                for (size_t i = 0; i < key.size(); ++i) given[key[i]] = by_key[i];
            }
            if (ok) {
                for (size_t i = 0; i < round.size(); ++i) results[round[i]] = tokens[i];
                return;
            }
            // the queued step failed: the callers go through their own steps below
        } else {
            for (llava_session* s : round) settle_locked(s);
            if (ahead_group != nullptr) {                  // another group's step: it would be stale by the time its callers return
                ahead_group->discard_ahead();
                ahead_group = nullptr;
                given.clear();
            }
        }
    }
    if (round.size() == 1) {
        lock.unlock();
        tokens[0] = round[0]->predict_next_token();
        lock.lock();
    } else {
        llava_session_group* g = nullptr;
        const auto it = groups.find(key);
        if (it != groups.end()) {
            g = it->second;
        } else {
            if (groups.size() >= kCachedGroups) {             // membership changes rarely; keep the table small
                if (groups.begin()->second == ahead_group) {  // (its destructor drops the step it has queued)
                    ahead_group = nullptr;
                    given.clear();
                }
                delete groups.begin()->second;
                groups.erase(groups.begin());
            }
            g = new llava_session_group(ctx, key);
            groups.emplace(key, g);
        }
        lock.unlock();
        vector<u32> by_key;
        const bool ok = g->is_valid() && g->step(&by_key);
        bool queued = false;
        if (ok) {
            for (size_t i = 0; i < round.size(); ++i)
                tokens[i] = by_key[size_t(lower_bound(key.begin(), key.end(), round[i]) - key.begin())];
            n_grouped_steps += 1;
            n_grouped_tokens += round.size();
            queued = g->launch_ahead();                       // the next step needs nothing from the host
        } else {
            // e.g. a model the batched products do not take: every caller falls back to its own step
            for (size_t i = 0; i < round.size(); ++i) tokens[i] = round[i]->predict_next_token();
        }
        lock.lock();
        if (queued) {
            ahead_group = g;
            given.clear();
            for (size_t i = 0; i < key.size(); ++i) given[key[i]] = by_key[i];
        }
    }
    for (size_t i = 0; i < round.size(); ++i) results[round[i]] = tokens[i];
}
