// Steps the running sessions of a server together.
//
// Every lsrv::session_wrapper thread that wants its next token calls evaluate(); the calls that arrive while a step is
// in flight (or within a short window) are served by ONE llava_session_group step: one pass over the weights for all
// of them.  The reference's sessions each submit their own work (server/session_wrapper.cpp:55-105), so k running
// sessions stream the weights k times per round.
//
// A caller is grouped when its session holds exactly one token that is not evaluated yet and does not sample on the
// host; any other call (a prompt to ingest, a lone session) is evaluated by the session itself.
#ifndef LLAVA_B200_GROUP_SCHEDULER_H
#define LLAVA_B200_GROUP_SCHEDULER_H

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <map>
#include <mutex>
#include <vector>

#include "../types.h"

namespace lsrv {

class group_scheduler {
public:
    explicit group_scheduler(llava_context* ctx);
    ~group_scheduler();
    group_scheduler(const group_scheduler&) = delete;
    group_scheduler& operator=(const group_scheduler&) = delete;

    // A session enters / leaves the state in which it asks for token after token: the scheduler waits for that many
    // callers (or for the window to pass) before it runs a step.
    void runner_enters();
    void runner_leaves();
    // Evaluates the session's pending token(s) and returns its next token (~0U on failure).  Blocks.
    u32 evaluate(llava_session* session);
    // The session is about to be used directly (a tick, an order that evaluates, the end of its running state): a step
    // that the scheduler queued ahead for its group is dropped first, so that the device is where the session thinks it is.
    void settle(llava_session* session);
    // The session is about to be destroyed: groups that contain it are dropped.
    void forget(llava_session* session);

    u64 grouped_steps() const { return n_grouped_steps; }        // steps that served two or more sessions
    u64 grouped_tokens() const { return n_grouped_tokens; }      // tokens those steps produced
    u64 steps_ahead() const { return n_steps_ahead; }
    // where the rounds' time went, in microseconds since the scheduler was made: waiting for the callers of a round to
    // arrive, and waiting for the device (the step itself, or the rest of a step that was queued ahead)
    u64 collect_us() const { return us_collect; }
    u64 device_us() const { return us_device; }            // grouped steps that were already queued when their callers arrived

private:
    void lead(std::unique_lock<std::mutex>& lock);
    void settle_locked(llava_session* session);

    llava_context* const ctx;
    std::mutex m;
    std::condition_variable cv_leader;                    // an arrival, or a runner that left: only the collecting leader waits here
    std::condition_variable cv_results;                   // a round's results are out (or the leadership is free)
    std::vector<llava_session*> waiting;                  // callers of the round being collected
    std::map<llava_session*, u32> results;                // tokens of finished rounds, picked up by their callers
    bool leader_present = false;
    u32 runners = 0;
    std::map<std::vector<llava_session*>, llava_session_group*> groups;     // by member list (sorted)
    // After a grouped step the next step of the same group is queued at once (the device fed every member its token,
    // greedy or drawn); it is booked when the same callers come back having pushed exactly those tokens, else dropped.
    llava_session_group* ahead_group = nullptr;
    std::map<llava_session*, u32> given;                  // the token each member of ahead_group was handed last
    std::atomic<u64> n_grouped_steps{0}, n_grouped_tokens{0}, n_steps_ahead{0}, us_collect{0}, us_device{0};
};

}  // namespace lsrv

#endif
