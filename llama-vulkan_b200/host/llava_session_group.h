// One decoding step for several sessions at once.
//
// The reference's server gives every session a thread that evaluates its own tokens
// (server/session_wrapper.cpp:55-105): k running sessions stream the weights k times per round.
// A group evaluates one token of each member with ONE pass over the weights: the rows of all
// members go through the batched (tcgen05) products that prompts use, and only the operations
// that touch per-session state -- embedding row, cache append, attention, argmax and position --
// work member by member inside their launch (lv_*_group in lv_b200.h).  The members stay ordinary
// llava_session objects: their caches, token buffers and positions are the ones a group step
// reads and advances, so a session can leave a group and go on by itself (and the other way round).
//
// A member decodes greedily or draws its token with the device sampler, whichever its session is set to
// (set_deterministic); members that sample on the host are refused.
#ifndef LLAVA_B200_SESSION_GROUP_H
#define LLAVA_B200_SESSION_GROUP_H

#include <vector>

#include "../../include/lv_b200.h"
#include "types.h"

class llava_session_group {
public:
    // 2..64 sessions of the same (single-GPU) context, model of ggjt version 3
    llava_session_group(llava_context* ctx, std::vector<llava_session*> members);
    ~llava_session_group();
    llava_session_group(const llava_session_group&) = delete;
    llava_session_group& operator=(const llava_session_group&) = delete;

    bool is_valid() const { return valid; }
    u32 size() const { return u32(members.size()); }
    // Every member must hold exactly one token that is not evaluated yet (the one pushed last).  Evaluates it for all
    // members and returns, per member, the greedy next token (not pushed: the caller decides, as with
    // llava_session::predict_next_token).  False on a failed precondition or a device error.
    bool step(std::vector<u32>* next_tokens);
    // n steps in a row with no host round trip: every member's greedy token is fed back on the device
    // (out[i] receives member i's n tokens; they are appended to the members' token buffers).
    bool generate_greedy_on_device(u32 n, std::vector<std::vector<u32>>* out);
    // Stepping ahead: the step after a successful step() needs nothing from the host when every member is going to push
    // exactly the token it was given (the device fed it into the member's token log already).  launch_ahead() queues
    // that step at once; finish_ahead() waits for it and books it to the members (call it once every member HAS pushed
    // its token and holds it as the one pending token: the caller checks); discard_ahead() drops it when a member did
    // something else: the members' device positions are marked unknown, so that their next evaluation uploads them again
    // (the cache rows and log entries the dropped step wrote lie beyond the evaluated tokens and are overwritten later).
    // The sampler state of members that sample is saved before the step and put back when it is dropped.
    bool can_step_ahead() const;
    bool launch_ahead();
    bool finish_ahead(std::vector<u32>* next_tokens);
    void discard_ahead();
    bool ahead_in_flight() const { return ahead; }
    const std::vector<llava_session*>& get_members() const { return members; }
    // logits of member i from the last step (vocab floats)
    bool get_logits(u32 member, std::vector<float>* out);
    u32 kernel_launches() const { return launches; }

private:
    bool record(u32 backlog);
    bool prepare_members(u32* backlog);
    void drop_graph();

    llava_context* const ctx;
    std::vector<llava_session*> members;
    bool valid = false;
    llava_device_memory* memory = nullptr;
    llava_buffer *x = nullptr, *q = nullptr, *vout = nullptr, *ff = nullptr, *split = nullptr, *logits = nullptr, *scratch = nullptr,
                 *tables = nullptr, *tokens_dev = nullptr, *sampler_backup = nullptr;
    std::vector<bool> sampled;               // per member: the recorded step ends with its sampler launch
    std::vector<u8> uploaded_table;          // the member tables as the device holds them
    u32* pinned_tokens = nullptr;
    lv_graph* graph = nullptr;
    u32 graph_backlog = 0;
    u32 launches = 0;
    bool ahead = false;                      // a step queued by launch_ahead() has not been booked or dropped yet
};

#endif
