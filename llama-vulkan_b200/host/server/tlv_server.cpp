#include "tlv_server.h"

#include <arpa/inet.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <iostream>

#include "../ggml_file.h"
#include "../llava_context.h"
#include "group_scheduler.h"

using namespace std;
using namespace lsrv;

namespace {
constexpr u32 kMaxFrame = 0x10000;        // server/client.cpp:128
constexpr size_t kHeader = 12;

u32 word(const u8* p) {
    u32 v;
    memcpy(&v, p, 4);
    return v;
}

// epoll user data: the fd itself (every fd of the loop is distinct)
bool watch(int epoll_fd, int fd, u32 events, bool modify = false) {
    epoll_event ev{};
    ev.events = events;
    ev.data.fd = fd;
    return epoll_ctl(epoll_fd, modify ? EPOLL_CTL_MOD : EPOLL_CTL_ADD, fd, &ev) == 0;
}
}  // namespace

tlv_server::tlv_server(llava_context* _ctx, u16 port, const char* bind_address, bool watch_stdin)
    : ctx(_ctx), requested_port(port), address(bind_address ? bind_address : "0.0.0.0"), stdin_watched(watch_stdin) {
    if (ctx->has_device()) sched = new group_scheduler(ctx);
    // tokenMap reply: for every token {u32 length; bytes} (server/server.cpp:28-42)
    for (const ggml_token& t : ctx->get_model()->get_tokens()) {
        const u32 n = u32(t.text.size());
        const size_t at = token_map.size();
        token_map.resize(at + 4 + n);
        memcpy(token_map.data() + at, &n, 4);
        memcpy(token_map.data() + at + 4, t.text.data(), n);
    }
}

tlv_server::~tlv_server() {
    for (auto& [id, s] : sessions) {
        s->push_order(0, 0, cmdKillSession);
        s->join();
        delete s;
    }
    for (auto& [id, c] : clients) ::close(c.fd);
    for (int fd : {listen_fd, epoll_fd, wake_fd})
        if (fd >= 0) ::close(fd);
    delete sched;
}

u64 tlv_server::grouped_steps() const { return sched ? sched->grouped_steps() : 0; }
u64 tlv_server::grouped_tokens() const { return sched ? sched->grouped_tokens() : 0; }
u64 tlv_server::scheduler_collect_us() const { return sched ? sched->collect_us() : 0; }
u64 tlv_server::scheduler_device_us() const { return sched ? sched->device_us() : 0; }
u64 tlv_server::steps_ahead() const { return sched ? sched->steps_ahead() : 0; }

bool tlv_server::open() {
    listen_fd = ::socket(AF_INET, SOCK_STREAM | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
    if (listen_fd < 0) { perror("socket"); return false; }
    const int on = 1;
    ::setsockopt(listen_fd, SOL_SOCKET, SO_REUSEADDR, &on, sizeof on);
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons(requested_port);
    if (inet_pton(AF_INET, address.c_str(), &addr.sin_addr) != 1) { cerr << "[!] bad bind address " << address << endl; return false; }
    if (::bind(listen_fd, reinterpret_cast<sockaddr*>(&addr), sizeof addr) < 0) { perror("bind"); return false; }
    if (::listen(listen_fd, 16) < 0) { perror("listen"); return false; }
    socklen_t len = sizeof addr;
    if (::getsockname(listen_fd, reinterpret_cast<sockaddr*>(&addr), &len) == 0) bound_port = ntohs(addr.sin_port);
    epoll_fd = ::epoll_create1(EPOLL_CLOEXEC);
    wake_fd = ::eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
    if (epoll_fd < 0 || wake_fd < 0) { perror("epoll/eventfd"); return false; }
    bool ok = watch(epoll_fd, listen_fd, EPOLLIN) && watch(epoll_fd, wake_fd, EPOLLIN);
    if (ctx->get_signal_fd() >= 0) ok = ok && watch(epoll_fd, ctx->get_signal_fd(), EPOLLIN);
    if (stdin_watched) ok = ok && watch(epoll_fd, STDIN_FILENO, EPOLLIN);
    if (!ok) perror("epoll_ctl");
    return ok;
}

void tlv_server::wake() const {
    const uint64_t one = 1;
    if (::write(wake_fd, &one, 8) != 8 && errno != EAGAIN) perror("eventfd");
}

void tlv_server::stop() {
    stop_requested = true;
    if (wake_fd >= 0) wake();
}

// session threads
void tlv_server::receive_session_outbound_packets(list<outbound_packet>& packets, list<outbound_broadcast>& broadcasts) {
    {
        lock_guard<mutex> lock(traffic_mutex);
        pending_packets.splice(pending_packets.end(), packets);
        pending_broadcasts.splice(pending_broadcasts.end(), broadcasts);
    }
    wake();
}

void tlv_server::notify_session_death(u32 session_id) {
    {
        lock_guard<mutex> lock(traffic_mutex);
        dead_sessions.push_back(session_id);
    }
    wake();
}

session_wrapper* tlv_server::find_session(u32 id) const {
    const auto it = sessions.find(id);
    return it == sessions.end() ? nullptr : it->second;
}

void tlv_server::send_packet(connection& c, OutCommands op, u32 request_id, const void* payload, size_t size) {
    vector<u8> frame(kHeader + size);
    const u32 words[3] = {u32(op), request_id, u32(size)};
    memcpy(frame.data(), words, kHeader);
    if (size) memcpy(frame.data() + kHeader, payload, size);
    c.out.push_back(std::move(frame));
    if (!c.want_write) write_to(c);                 // usually goes out at once; the rest waits for EPOLLOUT
}

void tlv_server::acknowledge(connection& c, u32 request_id, ReturnCode rc) {
    send_packet(c, outCmdAck, request_id, &rc, 4);
}

void tlv_server::update_interest(connection& c) {
    const bool need = !c.out.empty();
    if (need == c.want_write) return;
    c.want_write = need;
    watch(epoll_fd, c.fd, EPOLLIN | (need ? EPOLLOUT : 0), true);
}

bool tlv_server::write_to(connection& c) {
    while (!c.out.empty()) {
        const vector<u8>& f = c.out.front();
        const ssize_t r = ::send(c.fd, f.data() + c.out_offset, f.size() - c.out_offset, MSG_DONTWAIT | MSG_NOSIGNAL);
        if (r < 0) {
            if (errno == EAGAIN || errno == EWOULDBLOCK) break;
            if (errno == EINTR) continue;
            return false;
        }
        c.out_offset += size_t(r);
        if (c.out_offset == f.size()) {
            c.out.pop_front();
            c.out_offset = 0;
        }
    }
    update_interest(c);
    return true;
}

bool tlv_server::read_from(connection& c) {
    u8 buf[4096];
    for (;;) {
        const ssize_t r = ::recv(c.fd, buf, sizeof buf, MSG_DONTWAIT);
        if (r < 0) {
            if (errno == EAGAIN || errno == EWOULDBLOCK) break;
            if (errno == EINTR) continue;
            return false;
        }
        if (r == 0) return false;                    // the peer closed
        c.in.insert(c.in.end(), buf, buf + r);
        if (c.in.size() > 2 * size_t(kMaxFrame)) break;       // enough to work on; the rest next time round
    }
    size_t at = 0;
    while (c.in.size() - at >= kHeader) {
        const u32 command = word(c.in.data() + at), request_id = word(c.in.data() + at + 4), length = word(c.in.data() + at + 8);
        if (length > kMaxFrame) {
            cerr << "[!] Packet too large" << endl;
            return false;
        }
        if (c.in.size() - at < kHeader + length) break;
        handle_frame(c, command, request_id, c.in.data() + at + kHeader, length);
        at += kHeader + length;
    }
    c.in.erase(c.in.begin(), c.in.begin() + long(at));
    return true;
}

// server/client.cpp:146-300
void tlv_server::handle_frame(connection& c, u32 command, u32 request_id, const u8* payload, u32 length) {
    if (command < 16) {
        if (command == cmdGetTokenMap) {
            send_packet(c, outCmdTokenMap, request_id, token_map.data(), token_map.size());
        } else if (command == cmdNewSession) {
            if (shutting_down || !ctx->has_device()) { acknowledge(c, request_id, ReturnCode::nok); return; }
            auto* s = new session_wrapper(this);
            sessions.emplace(s->session_id, s);
            const u32 id = s->session_id;
            for (auto& [cid, other] : clients) send_packet(other, outCmdNewSession, cid == c.id ? request_id : 0u, &id, 4);    // everyone learns of it
            s->start();
        } else if (command == cmdListSessions) {
            vector<u32> ids;
            for (const auto& [id, s] : sessions) ids.push_back(id);
            send_packet(c, outCmdSessionList, request_id, ids.data(), ids.size() * 4);
        } else {
            acknowledge(c, request_id, ReturnCode::unknown_command);
        }
        return;
    }
    if (length < 4) { acknowledge(c, request_id, ReturnCode::bad_arguments); return; }
    const u32 session_id = word(payload);
    // expected payload: session only (16..31), session + one word (rewind, addToken, setSessionOptions), session + characters
    const bool one_word = command == cmdRewind || command == cmdAddToken || command == cmdSetSessionOptions;
    const bool characters = command == cmdAddText || command == cmdSaveFrame || command == cmdSnapshot || command == cmdRestore;
    if (command >= 32 && !one_word && !characters) { acknowledge(c, request_id, ReturnCode::unknown_command); return; }
    if ((command < 32 && length != 4) || (one_word && length != 8) || (characters && length <= 4)) {
        acknowledge(c, request_id, ReturnCode::bad_arguments);
        return;
    }
    session_wrapper* s = find_session(session_id);
    if (s == nullptr) { acknowledge(c, request_id, ReturnCode::no_such_session); return; }
    switch (command) {
        case cmdSubscribe:
            c.subscriptions.insert(session_id);
            subscribers[session_id].insert(c.id);
            acknowledge(c, request_id, ReturnCode::ok);
            return;
        case cmdUnsubscribe:
            c.subscriptions.erase(session_id);
            subscribers[session_id].erase(c.id);
            acknowledge(c, request_id, ReturnCode::ok);
            return;
        case cmdGetSessionTokens: case cmdKillSession: case cmdStartSessionGeneration: case cmdStopSessionGeneration:
        case cmdTick: case cmdGetSessionStatus:
            s->push_order(c.id, request_id, command);
            return;
        case cmdRewind: case cmdAddToken: case cmdSetSessionOptions:
            s->push_order(c.id, request_id, command, word(payload + 4));
            return;
        case cmdAddText: case cmdSaveFrame: case cmdSnapshot: case cmdRestore: {
            string text(reinterpret_cast<const char*>(payload + 4), length - 4);
            if (text.find('\0') != string::npos) {
                if (command != cmdAddText) { acknowledge(c, request_id, ReturnCode::bad_arguments); return; }
                cerr << "[?] Null byte in added string" << endl;          // the reference keeps the part before it
                text.resize(text.find('\0'));
            }
            s->push_order(c.id, request_id, command, 0, std::move(text));
            return;
        }
        default:
            acknowledge(c, request_id, ReturnCode::unknown_command);
    }
}

void tlv_server::accept_clients() {
    for (;;) {
        sockaddr_in peer{};
        socklen_t len = sizeof peer;
        const int fd = ::accept4(listen_fd, reinterpret_cast<sockaddr*>(&peer), &len, SOCK_NONBLOCK | SOCK_CLOEXEC);
        if (fd < 0) {
            if (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) perror("accept");
            return;
        }
        const int on = 1;
        ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &on, sizeof on);
        char text[INET_ADDRSTRLEN + 1] = {0};
        inet_ntop(AF_INET, &peer.sin_addr, text, sizeof text);
        if (ctx->verbosity) cout << "[*] New client from " << text << ":" << ntohs(peer.sin_port) << endl;
        connection c;
        c.fd = fd;
        c.id = next_client_id++;
        if (!watch(epoll_fd, fd, EPOLLIN)) { ::close(fd); continue; }
        client_of_fd[fd] = c.id;
        clients.emplace(c.id, std::move(c));
    }
}

void tlv_server::drop_connection(u32 id) {
    const auto it = clients.find(id);
    if (it == clients.end()) return;
    for (u32 session_id : it->second.subscriptions) subscribers[session_id].erase(id);
    epoll_ctl(epoll_fd, EPOLL_CTL_DEL, it->second.fd, nullptr);
    client_of_fd.erase(it->second.fd);
    ::close(it->second.fd);
    clients.erase(it);
}

// packets from the session threads: replies to one client, broadcasts to the subscribers of a session
void tlv_server::deliver_session_traffic() {
    list<outbound_packet> packets;
    list<outbound_broadcast> broadcasts;
    {
        lock_guard<mutex> lock(traffic_mutex);
        packets.swap(pending_packets);
        broadcasts.swap(pending_broadcasts);
    }
    for (auto& [session_id, op, payload] : broadcasts) {
        const auto subs = subscribers.find(session_id);
        if (subs == subscribers.end()) continue;
        for (u32 client_id : subs->second) {
            const auto it = clients.find(client_id);
            if (it != clients.end()) send_packet(it->second, op, 0, payload.data(), payload.size());
        }
    }
    for (auto& [client_id, op, request_id, payload] : packets) {
        const auto it = clients.find(client_id);
        if (it != clients.end()) send_packet(it->second, op, request_id, payload.data(), payload.size());
    }
}

void tlv_server::reap_sessions() {
    list<u32> dead;
    {
        lock_guard<mutex> lock(traffic_mutex);
        dead.swap(dead_sessions);
    }
    for (u32 id : dead) {
        const auto it = sessions.find(id);
        if (it == sessions.end()) continue;
        it->second->join();
        delete it->second;
        sessions.erase(it);
        for (u32 client_id : subscribers[id]) {
            const auto c = clients.find(client_id);
            if (c != clients.end()) c->second.subscriptions.erase(id);
        }
        subscribers.erase(id);
    }
}

void tlv_server::begin_shutdown() {
    if (shutting_down) return;
    shutting_down = true;
    for (auto& [id, s] : sessions) s->push_order(0, 0, cmdKillSession);
}

void tlv_server::serve_forever() {
    if (listen_fd < 0 && !open()) return;
    if (announce) cout << "[*] Started server on " << address << ":" << bound_port << endl;
    const int sigfd = ctx->get_signal_fd();
    epoll_event events[32];
    while (!shutting_down || !sessions.empty()) {
        const int n = ::epoll_wait(epoll_fd, events, 32, 1000);
        if (n < 0) {
            if (errno == EINTR) continue;
            cerr << "[?] Error while polling " << strerror(errno) << endl;
            break;
        }
        if (stop_requested) begin_shutdown();
        vector<u32> to_drop;
        for (int i = 0; i < n; ++i) {
            const int fd = events[i].data.fd;
            const u32 ev = events[i].events;
            if (fd == listen_fd) {
                accept_clients();
            } else if (fd == wake_fd) {
                uint64_t count;
                while (::read(wake_fd, &count, 8) == 8) {}
                deliver_session_traffic();
                reap_sessions();
            } else if (fd == sigfd && sigfd >= 0) {
                ctx->pop_signal(false);
                begin_shutdown();
            } else if (fd == STDIN_FILENO && stdin_watched) {
                begin_shutdown();                  // any input ends the server (server/server.cpp:178-184)
                epoll_ctl(epoll_fd, EPOLL_CTL_DEL, STDIN_FILENO, nullptr);
            } else {
                const auto who = client_of_fd.find(fd);
                if (who == client_of_fd.end()) continue;
                connection& c = clients.at(who->second);
                bool alive = !(ev & (EPOLLERR | EPOLLHUP));
                if (alive && (ev & EPOLLOUT)) alive = write_to(c);
                if (alive && (ev & EPOLLIN)) alive = read_from(c);
                if (!alive) to_drop.push_back(c.id);
            }
        }
        for (u32 id : to_drop) drop_connection(id);
    }
    deliver_session_traffic();
    while (!clients.empty()) drop_connection(clients.begin()->first);
}
