#include "session_wrapper.h"

#include <csignal>
#include <cstring>
#include <iostream>

#include "../llava_context.h"
#include "../llava_session.h"
#include "group_scheduler.h"

using namespace std;
using namespace lsrv;

u32 session_wrapper::ticker = 1U;
bool session_wrapper::deterministic = false;
u32 session_wrapper::prompt_batch = 1;

session_wrapper::session_wrapper(session_owner* _owner) : session_id(ticker++), owner(_owner) {}

session_wrapper::~session_wrapper() {
    if (loop_thread != nullptr && loop_thread->joinable()) loop_thread->join();
    delete loop_thread;
}

void session_wrapper::start() {
    if (loop_thread == nullptr) loop_thread = new thread([this]() { run(); });
}

void session_wrapper::join() {
    if (loop_thread != nullptr && loop_thread->joinable()) loop_thread->join();
}

// front-end thread
void session_wrapper::push_order(u32 client_id, u32 request_id, u32 opcode, u32 arg1, string s) {
    {
        lock_guard<mutex> lock(session_mutex);
        orders.push_back({client_id, request_id, opcode, arg1, std::move(s)});
    }
    cv.notify_one();
}

// session thread (server/session_wrapper.cpp:55-105)
void session_wrapper::run() {
    if (!owner->context()->signal_debug_on()) {
        sigset_t mask;                       // signals belong to the front-end thread
        sigemptyset(&mask);
        for (int s : {SIGINT, SIGQUIT, SIGHUP, SIGTERM}) sigaddset(&mask, s);
        pthread_sigmask(SIG_BLOCK, &mask, nullptr);
    }
    llava_session session(owner->context());
    session.set_deterministic(deterministic);
    if (prompt_batch > 1 && !session.set_max_batch(prompt_batch)) cerr << "[?] prompt batches of " << prompt_batch << " refused; token by token" << endl;

    group_scheduler* sched = owner->scheduler();
    bool registered = false;                 // counted by the scheduler among the sessions that ask for token after token
    auto sync_registration = [&]() {
        if (sched == nullptr || registered == should_run) return;
        if (should_run) {
            sched->runner_enters();
        } else {
            sched->runner_leaves();
            sched->settle(&session);         // a step queued ahead for this session's group is dropped
        }
        registered = should_run;
    };

    while (!should_die) {
        process_orders(session, !(should_run || should_tick));
        sync_registration();
        if (!(should_run || should_tick)) continue;
        if (sched != nullptr && should_run) {
            // running: the scheduler evaluates this session's token together with the other running sessions'
            const u32 token = sched->evaluate(&session);
            process_orders(session, false);
            if (token == ~0U) {
                cerr << "Error starting token generation" << endl;
                should_run = false;
                sync_registration();
                continue;
            }
            vector<u8> payload(12);
            const u32 pos = session.get_token_count();
            memcpy(payload.data(), &session_id, 4);
            memcpy(payload.data() + 4, &token, 4);
            memcpy(payload.data() + 8, &pos, 4);
            if (!session.push_token(token)) {
                cerr << "Out of buffer ?" << endl;
                should_run = false;
            }
            outbound_broadcasts.emplace_back(session_id, outCmdNewToken, payload);
            flush_outbound_packets();
            continue;
        }
        if (!session.start_next_token_prediction()) {
            should_run = false;
            cerr << "Error starting token generation" << endl;
            if (should_tick) {
                add_outbound_ack(tick_client, should_tick, ReturnCode::nok);
                flush_outbound_packets();
            }
            should_tick = 0;
            tick_client = 0;
            continue;
        }
        process_orders(session, false);      // handled while the device evaluates the token
        const u32 new_token_id = session.finish_next_token_prediction();

        vector<u8> payload(12);
        const u32 pos = session.get_token_count();
        memcpy(payload.data(), &session_id, 4);
        memcpy(payload.data() + 4, &new_token_id, 4);
        memcpy(payload.data() + 8, &pos, 4);
        if (new_token_id == ~0U || !session.push_token(new_token_id)) {
            cerr << "Out of buffer ?" << endl;
            should_run = false;
        }
        outbound_broadcasts.emplace_back(session_id, outCmdNewToken, payload);
        if (should_tick) outbound_packets.emplace_back(tick_client, outCmdNewToken, should_tick, payload);
        flush_outbound_packets();
        should_tick = 0;
        tick_client = 0;
    }
    process_orders(session, false);
    should_run = false;
    sync_registration();
    if (sched != nullptr) sched->forget(&session);
    owner->notify_session_death(session_id);
}

// session thread (server/session_wrapper.cpp:120-210)
void session_wrapper::process_orders(llava_session& session, bool blocking) {
    unique_lock<mutex> lock(session_mutex);
    if (orders.empty() && blocking) cv.wait(lock, [this]() { return !orders.empty(); });
    while (!orders.empty()) {
        const session_order order = orders.front();
        orders.pop_front();
        ReturnCode rc = ReturnCode::ok;
        bool acknowledge = true;
        // orders that change or read the session's device state: no step queued ahead for its group may be in flight
        if (group_scheduler* sched = owner->scheduler()) {
            switch (order.opcode) {
                case cmdRewind: case cmdSetSessionOptions: case cmdAddToken: case cmdAddText: case cmdSaveFrame: case cmdSnapshot:
                case cmdRestore: case cmdTick:
                    sched->settle(&session);
                    break;
                default: break;
            }
        }
        switch (order.opcode) {
            case cmdStartSessionGeneration:
                if (should_tick) rc = ReturnCode::tick_already_requested;
                else should_run = true;
                break;
            case cmdTick:
                if (should_run) rc = ReturnCode::already_running;
                else if (should_tick != 0) rc = ReturnCode::tick_already_requested;
                else {
                    should_tick = order.request_id;
                    tick_client = order.client_id;
                    acknowledge = false;          // answered by the newToken packet
                }
                break;
            case cmdStopSessionGeneration: should_run = false; break;
            case cmdRewind: session.rewind(order.arg1); break;
            case cmdSetSessionOptions: rc = session.set_options(order.arg1); break;
            case cmdKillSession: should_die = true; break;
            case cmdAddToken:
                if (!session.push_token(order.arg1)) rc = ReturnCode::nok;
                break;
            case cmdAddText:
                if (!session.add_text(order.s)) rc = ReturnCode::nok;
                break;
            case cmdGetSessionTokens: {
                acknowledge = false;
                const auto& toks = session.get_token_buffer();
                vector<u8> bytes(4 * toks.size());
                memcpy(bytes.data(), toks.data(), bytes.size());
                outbound_packets.emplace_back(order.client_id, outCmdBuffer, order.request_id, std::move(bytes));
                break;
            }
            case cmdSaveFrame: rc = session.save_frame(order.s); break;
            case cmdSnapshot: rc = session.snapshot(order.s); break;
            case cmdRestore:
                if (should_run) rc = ReturnCode::already_running;
                else if (should_tick) rc = ReturnCode::tick_already_requested;
                else rc = session.restore(order.s);
                break;
            default: break;                       // e.g. cmdGetSessionStatus: acknowledged, no handler
        }
        if (order.client_id && order.request_id && acknowledge) add_outbound_ack(order.client_id, order.request_id, rc);
    }
    lock.unlock();
    flush_outbound_packets();
}

void session_wrapper::flush_outbound_packets() {
    if (!(outbound_packets.empty() && outbound_broadcasts.empty())) owner->receive_session_outbound_packets(outbound_packets, outbound_broadcasts);
}

void session_wrapper::add_outbound_ack(u32 client_id, u32 request_id, ReturnCode return_code) {
    vector<u8> packet(4);
    memcpy(packet.data(), &return_code, 4);
    outbound_packets.emplace_back(client_id, outCmdAck, request_id, std::move(packet));
}
