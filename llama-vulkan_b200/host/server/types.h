// Opcodes and reply codes of the reference's session protocol (server/types.h:50-84), shared by
// lsrv::session_wrapper (one thread per session) and lsrv::tlv_server (the TCP front end).
#ifndef LLAVA_B200_SERVER_TYPES_H
#define LLAVA_B200_SERVER_TYPES_H

#include <string>

#include "../types.h"

namespace lsrv {

enum Commands : u32 {
    cmdGetTokenMap = 0, cmdNewSession = 1, cmdListSessions = 2,
    cmdGetSessionTokens = 16, cmdSubscribe = 17, cmdUnsubscribe = 18, cmdKillSession = 19,
    cmdStartSessionGeneration = 20, cmdStopSessionGeneration = 21, cmdTick = 22, cmdGetSessionStatus = 23,
    cmdRewind = 32, cmdAddToken = 33, cmdAddText = 34, cmdSetSessionOptions = 35, cmdSaveFrame = 36,
    cmdSnapshot = 37, cmdRestore = 38,
};

enum OutCommands : u32 {
    outCmdNewToken = 0, outCmdBuffer = 1, outCmdTokenMap = 2, outCmdNewSession = 3, outCmdSessionList = 4,
    outCmdDroppedSession = 5, outCmdAck = 6, outCmdSessionStatus = 7,
};

struct session_order {
    u32 client_id;
    u32 request_id;
    u32 opcode;
    u32 arg1;
    std::string s;
};

}  // namespace lsrv

#endif
