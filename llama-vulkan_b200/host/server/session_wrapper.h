// One thread + one llava_session per served session: an order queue fed by the front end, a
// run/tick loop that overlaps order processing with token evaluation, and outbound packets
// handed back to the owner.  Counterpart of the reference's lsrv::session_wrapper
// (server/session_wrapper.h:17-23, server/session_wrapper.cpp:19-229); the owner is an
// interface here so that the TCP front end (lsrv::tlv_server) and an in-process collector can both drive it.
#ifndef LLAVA_B200_SESSION_WRAPPER_H
#define LLAVA_B200_SESSION_WRAPPER_H

#include <condition_variable>
#include <list>
#include <mutex>
#include <string>
#include <thread>
#include <tuple>
#include <vector>

#include "types.h"

namespace lsrv {

class group_scheduler;

// (client id, reply opcode, request id, payload) and (session id, opcode, payload)
using outbound_packet = std::tuple<u32, OutCommands, u32, std::vector<u8>>;
using outbound_broadcast = std::tuple<u32, OutCommands, std::vector<u8>>;

// What the reference's llava_server offers a session (server/server.cpp:319-331 and the `ctx` member).
class session_owner {
public:
    virtual ~session_owner() = default;
    virtual llava_context* context() = 0;
    virtual void receive_session_outbound_packets(std::list<outbound_packet>& packets, std::list<outbound_broadcast>& broadcasts) = 0;
    virtual void notify_session_death(u32 session_id) = 0;
    // non-null: sessions in the running state ask it for their tokens, so that it can step them together
    virtual group_scheduler* scheduler() { return nullptr; }
};

class session_wrapper {
public:
    explicit session_wrapper(session_owner* owner);
    ~session_wrapper();
    u32 const session_id;
    session_owner* const owner;
    void start();
    void push_order(u32 client_id, u32 request_id, u32 opcode, u32 arg1 = 0, std::string s = {});
    void join();
    // greedy decoding for every session started afterwards (the reference always samples)
    static void set_deterministic_sessions(bool on) { deterministic = on; }
    // tokens per recorded step while a session ingests a prompt (llava_session::set_max_batch; 1 = token by token)
    static void set_prompt_batch(u32 n) { prompt_batch = n; }

private:
    void run();
    void process_orders(llava_session& session, bool blocking);
    void flush_outbound_packets();
    void add_outbound_ack(u32 client_id, u32 request_id, ReturnCode return_code);

    std::mutex session_mutex;
    std::condition_variable cv;
    std::thread* loop_thread = nullptr;
    std::list<session_order> orders;
    std::list<outbound_packet> outbound_packets;
    std::list<outbound_broadcast> outbound_broadcasts;
    bool should_run = false;
    u32 should_tick = 0;
    u32 tick_client = 0;
    bool should_die = false;
    static u32 ticker;
    static bool deterministic;
    static u32 prompt_batch;
};

}  // namespace lsrv

#endif
