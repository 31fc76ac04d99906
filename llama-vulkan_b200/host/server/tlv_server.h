// TCP front end of the session protocol: framed requests from any number of clients, dispatched to
// lsrv::session_wrapper threads; their replies and the tokens they generate travel back as framed packets.
// Counterpart of the reference's lsrv::llava_server and lsrv::client (server/server.cpp:44-331,
// server/client.cpp:43-313), with the wire format of server/types.h:111-115 and server/client.cpp:302-313:
//
//   request  {u32 command; u32 request_id; u32 length; u8 payload[length]}      length <= 0x10000
//   reply    {u32 out_command; u32 request_id (0 for broadcasts); u32 size; u8 payload[size]}
//
// One thread runs the event loop (epoll); session threads hand their packets over through a locked queue and
// an eventfd.  Differences from the reference, none visible in replies: the port and the bind address are
// parameters (default 0.0.0.0:1337), standard input is watched only when asked to, a frame above the size limit
// closes the connection, a path or text argument with an embedded NUL is refused with bad_arguments instead of
// an assert, and a departing client's subscriptions are removed from the sessions it had subscribed to.
#ifndef LLAVA_B200_TLV_SERVER_H
#define LLAVA_B200_TLV_SERVER_H

#include <atomic>
#include <deque>
#include <list>
#include <map>
#include <mutex>
#include <set>
#include <vector>

#include "session_wrapper.h"

namespace lsrv {

class tlv_server : public session_owner {
public:
    explicit tlv_server(llava_context* ctx, u16 port = 1337, const char* bind_address = "0.0.0.0", bool watch_stdin = false);
    ~tlv_server() override;
    tlv_server(const tlv_server&) = delete;
    tlv_server& operator=(const tlv_server&) = delete;

    void set_announce(bool on) { announce = on; }     // print "[*] Started server on ..." on standard output (default: yes)
    bool open();                     // socket, bind, listen; false (with a message on stderr) on failure
    u16 port() const { return bound_port; }      // the port actually bound (useful with port 0)
    void serve_forever();            // returns after stop(), a signal on the context's signal fd, or input on stdin
    void stop();                     // from any thread: kills the sessions and ends serve_forever once they are gone

    // session_owner
    llava_context* context() override { return ctx; }
    group_scheduler* scheduler() override { return sched; }
    // steps that served two or more sessions at once, and the tokens they produced
    u64 grouped_steps() const;
    u64 grouped_tokens() const;
    u64 steps_ahead() const;
    u64 scheduler_collect_us() const;   // time the scheduler's rounds waited for their callers / for the device
    u64 scheduler_device_us() const;         // of those steps, the ones that were already queued when their sessions asked
    void receive_session_outbound_packets(std::list<outbound_packet>& packets, std::list<outbound_broadcast>& broadcasts) override;
    void notify_session_death(u32 session_id) override;

private:
    struct connection {
        int fd = -1;
        u32 id = 0;
        std::vector<u8> in;
        std::deque<std::vector<u8>> out;
        size_t out_offset = 0;           // bytes of out.front() already sent
        bool want_write = false;
        std::set<u32> subscriptions;     // session ids
    };

    void wake() const;
    void accept_clients();
    bool read_from(connection& c);       // false: drop the connection
    bool write_to(connection& c);
    void handle_frame(connection& c, u32 command, u32 request_id, const u8* payload, u32 length);
    void send_packet(connection& c, OutCommands op, u32 request_id, const void* payload, size_t size);
    void acknowledge(connection& c, u32 request_id, ReturnCode rc);
    void update_interest(connection& c);
    void drop_connection(u32 id);
    void deliver_session_traffic();
    void reap_sessions();
    void begin_shutdown();
    session_wrapper* find_session(u32 id) const;

    llava_context* const ctx;
    group_scheduler* sched = nullptr;        // null on a context without a device
    const u16 requested_port;
    const std::string address;
    const bool stdin_watched;
    u16 bound_port = 0;
    int listen_fd = -1, epoll_fd = -1, wake_fd = -1;
    u32 next_client_id = 1;
    bool shutting_down = false;
    bool announce = true;
    std::atomic<bool> stop_requested{false};
    std::vector<u8> token_map;                        // payload of the tokenMap reply
    std::map<u32, connection> clients;                // by client id
    std::map<int, u32> client_of_fd;
    std::map<u32, session_wrapper*> sessions;
    std::map<u32, std::set<u32>> subscribers;         // session id -> client ids

    std::mutex traffic_mutex;                         // the three lists below are filled by session threads
    std::list<outbound_packet> pending_packets;
    std::list<outbound_broadcast> pending_broadcasts;
    std::list<u32> dead_sessions;
};

}  // namespace lsrv

#endif
