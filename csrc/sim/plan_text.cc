// A small text form of the schedule IR, so that a schedule can be written down by hand and put through the offline checker:
// regression cases for the checker itself (a dropped notify, a shifted offset) and experiments with new algorithms.
//
//   op=<HcclCMDType> n=<ranks> es=<element bytes> count=<elements> ccl=<scratch bytes> [root=<r>] [peer=<r>] [mbx=<slot bytes>]
//   r<k>[.q<j>]: <task>; <task>; ...
// tasks:  COPY dst src bytes | REDUCE dst src bytes | WRITE peer dst src bytes | WRITER peer dst src bytes (write-reduce)
//         READ peer dst src bytes | READR peer dst src bytes (read-reduce) | POST peer slot | WAIT peer slot
//         LPOST queue | LWAIT queue (notify another queue of the same rank / wait for its next notify)
// buffers: in@<off> out@<off> ccl@<off> mbx@<off>. Lines starting with '#' are comments. All ranks share one chunk.
#include <cstdlib>
#include <sstream>
#include "../common/log.h"
#include "checker.h"
#include "hccl/hccl_dfx.h"

namespace hccl {
namespace {

bool ParseBuf(const std::string &tok, BufRef *b)
{
    size_t at = tok.find('@');
    if (at == std::string::npos) return false;
    const std::string kind = tok.substr(0, at);
    if (kind == "in") b->kind = BufKind::INPUT;
    else if (kind == "out") b->kind = BufKind::OUTPUT;
    else if (kind == "ccl") b->kind = BufKind::CCL;
    else if (kind == "mbx") b->kind = BufKind::MAILBOX;
    else return false;
    char *end = nullptr;
    b->off = strtoull(tok.c_str() + at + 1, &end, 0);
    return end && *end == 0;
}

bool ParseTask(const std::string &text, Task *t, std::string *err)
{
    std::istringstream is(text);
    std::string name;
    is >> name;
    std::vector<std::string> a;
    for (std::string s; is >> s;) a.push_back(s);
    auto num = [](const std::string &s) { return strtoull(s.c_str(), nullptr, 0); };
    *t = Task{};
    if ((name == "COPY" || name == "REDUCE") && a.size() == 3) {
        t->type = name == "COPY" ? TaskType::LOCAL_COPY : TaskType::LOCAL_REDUCE;
        if (!ParseBuf(a[0], &t->dst) || !ParseBuf(a[1], &t->src)) { *err = "bad buffer in '" + text + "'"; return false; }
        t->bytes = num(a[2]);
        return true;
    }
    if ((name == "WRITE" || name == "WRITER" || name == "READ" || name == "READR") && a.size() == 4) {
        t->type = name == "WRITE" ? TaskType::WRITE : name == "WRITER" ? TaskType::WRITE_REDUCE : name == "READ" ? TaskType::READ : TaskType::READ_REDUCE;
        t->rank = (uint32_t)num(a[0]);
        if (!ParseBuf(a[1], &t->dst) || !ParseBuf(a[2], &t->src)) { *err = "bad buffer in '" + text + "'"; return false; }
        t->bytes = num(a[3]);
        return true;
    }
    if ((name == "POST" || name == "WAIT") && a.size() == 2) {
        t->type = name == "POST" ? TaskType::POST : TaskType::WAIT;
        t->rank = (uint32_t)num(a[0]);
        t->slot = (uint32_t)num(a[1]);
        return true;
    }
    if ((name == "LPOST" || name == "LWAIT") && a.size() == 1) {
        t->type = name == "LPOST" ? TaskType::LOCAL_POST : TaskType::LOCAL_WAIT;
        t->rank = (uint32_t)num(a[0]);
        return true;
    }
    *err = "cannot parse task '" + text + "'";
    return false;
}

}  // namespace
}  // namespace hccl

using namespace hccl;

extern "C" HcclResult HcclCheckPlanText(const char *text, char *msg, uint32_t msgLen)
{
    if (!text) return HCCL_E_PTR;
    auto say = [&](const std::string &s, HcclResult r) { if (msg && msgLen) snprintf(msg, msgLen, "%s", s.c_str()); return r; };
    CheckSpec spec{HCCL_CMD_INVALID, 0, 4, 0, 0, 0, {}};
    std::vector<Plan> plans;
    std::istringstream lines(text);
    bool haveHeader = false;
    for (std::string line; std::getline(lines, line);) {
        size_t first = line.find_first_not_of(" \t");
        if (first == std::string::npos || line[first] == '#') continue;
        if (!haveHeader) {
            std::istringstream is(line);
            for (std::string kv; is >> kv;) {
                size_t eq = kv.find('=');
                if (eq == std::string::npos) return say("bad header field '" + kv + "'", HCCL_E_PARA);
                const std::string k = kv.substr(0, eq);
                const uint64_t v = strtoull(kv.c_str() + eq + 1, nullptr, 0);
                if (k == "op") spec.op = (HcclCMDType)v;
                else if (k == "n") spec.nranks = (uint32_t)v;
                else if (k == "es") spec.elemSize = (uint32_t)v;
                else if (k == "count") spec.count = v;
                else if (k == "ccl") spec.cclBytes = v;
                else if (k == "root") spec.root = (uint32_t)v;
                else if (k == "peer") spec.peer = (uint32_t)v;
                else if (k == "mbx") spec.mailboxBytes = v;
                else return say("unknown header field '" + k + "'", HCCL_E_PARA);
            }
            if (spec.nranks < 2 || spec.nranks > 64 || spec.elemSize == 0) return say("header needs n=2..64 and es>0", HCCL_E_PARA);
            plans.assign(spec.nranks, Plan{});
            for (auto &p : plans) p.EnsureQueues(1);
            haveHeader = true;
            continue;
        }
        size_t colon = line.find(':');
        if (colon == std::string::npos || line[first] != 'r') return say("expected 'r<k>[.q<j>]: tasks' in '" + line + "'", HCCL_E_PARA);
        const std::string who = line.substr(first + 1, colon - first - 1);
        uint32_t rank = (uint32_t)strtoul(who.c_str(), nullptr, 10), queue = 0;
        size_t dot = who.find(".q");
        if (dot != std::string::npos) queue = (uint32_t)strtoul(who.c_str() + dot + 2, nullptr, 10);
        if (rank >= spec.nranks || queue > 63) return say("rank or queue out of range in '" + line + "'", HCCL_E_PARA);
        plans[rank].EnsureQueues(queue + 1);
        std::istringstream tasks(line.substr(colon + 1));
        for (std::string t; std::getline(tasks, t, ';');) {
            if (t.find_first_not_of(" \t") == std::string::npos) continue;
            Task task;
            std::string err;
            if (!ParseTask(t, &task, &err)) return say(err, HCCL_E_PARA);
            plans[rank].queues[queue].push_back(task);
        }
    }
    if (!haveHeader) return say("no header line", HCCL_E_PARA);
    std::string why;
    HcclResult r = CheckPlans(spec, {plans}, &why);
    return say(r == HCCL_SUCCESS ? "ok" : why, r);
}
