#include "log.h"
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <sstream>
#include <sys/syscall.h>
#include <unistd.h>

namespace hccl {
namespace {
std::atomic<int> g_level{LOG_WARNING};
std::atomic<uint32_t> g_mask{0};
std::atomic<uint64_t> g_count[6];
LogSink g_sink = nullptr;
void *g_sinkUser = nullptr;
std::mutex g_mu;
thread_local int t_errToWarn = 0;
thread_local int t_mute = 0;
const char *kNames[] = {"DEBUG", "INFO", "WARNING", "ERROR", "RUN", "OFF"};
std::once_flag g_envOnce;
}  // namespace

bool LogParseDebugConfig(const std::string &value, uint32_t *maskOut)
{
    std::string v = value;
    bool invert = false;
    if (!v.empty() && v[0] == '^') { invert = true; v = v.substr(1); }
    uint32_t m = 0;
    std::stringstream ss(v);
    std::string tok;
    while (std::getline(ss, tok, ',')) {
        while (!tok.empty() && tok.back() == ' ') tok.pop_back();
        while (!tok.empty() && tok.front() == ' ') tok.erase(tok.begin());
        if (tok.empty()) continue;
        if (tok == "ALG") m |= MOD_ALG;
        else if (tok == "TASK") m |= MOD_TASK;
        else if (tok == "RESOURCE") m |= MOD_RESOURCE;
        else if (tok == "KERNEL" || tok == "AIV_OPS_EXC") m |= MOD_KERNEL;
        else if (tok == "BOOT") m |= MOD_BOOT;
        else return false;
    }
    const uint32_t all = MOD_ALG | MOD_TASK | MOD_RESOURCE | MOD_KERNEL | MOD_BOOT;
    *maskOut = invert ? (all & ~m) : m;
    return true;
}

void LogInitFromEnv()
{
    std::call_once(g_envOnce, [] {
        if (const char *e = getenv("HCCL_LOG_LEVEL")) {
            std::string s(e);
            if (s == "DEBUG" || s == "0") g_level = LOG_DEBUG;
            else if (s == "INFO" || s == "1") g_level = LOG_INFO;
            else if (s == "WARNING" || s == "2") g_level = LOG_WARNING;
            else if (s == "ERROR" || s == "3") g_level = LOG_ERROR;
            else if (s == "OFF") g_level = LOG_OFF;
        }
        if (const char *e = getenv("HCCL_DEBUG_CONFIG")) {
            uint32_t m = 0;
            if (LogParseDebugConfig(e, &m)) g_mask = m;
            else fprintf(stderr, "[hccl][WARNING] HCCL_DEBUG_CONFIG=%s has an unknown module; ignored\n", e);
        }
    });
}

void LogSetLevel(int level) { g_level = level; }
int LogGetLevel() { return g_level.load(std::memory_order_relaxed); }
void LogSetSink(LogSink sink, void *user)
{
    std::lock_guard<std::mutex> lk(g_mu);
    g_sink = sink;
    g_sinkUser = user;
}
void LogSetModuleMask(uint32_t mask) { g_mask = mask; }
uint32_t LogGetModuleMask() { return g_mask; }
void LogPushErrorToWarn() { ++t_errToWarn; }
void LogPopErrorToWarn() { if (t_errToWarn > 0) --t_errToWarn; }
void LogPushMute() { ++t_mute; }
void LogPopMute() { if (t_mute > 0) --t_mute; }
bool LogModuleEnabled(uint32_t module) { return (g_mask.load(std::memory_order_relaxed) & module) != 0; }
uint64_t LogRecordCount(int level) { return (level >= 0 && level < 6) ? g_count[level].load() : 0; }

void LogWrite(int level, const char *file, int line, const char *func, const char *fmt, ...)
{
    if (t_mute > 0 && level <= LOG_ERROR) return;
    if (level == LOG_ERROR && t_errToWarn > 0) level = LOG_WARNING;
    if (level < 0 || level > LOG_RUN_INFO) return;
    g_count[level]++;
    char body[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(body, sizeof(body), fmt, ap);
    va_end(ap);
    const char *base = strrchr(file, '/');
    base = base ? base + 1 : file;
    using namespace std::chrono;
    auto us = duration_cast<microseconds>(system_clock::now().time_since_epoch()).count();
    char lineBuf[1300];
    snprintf(lineBuf, sizeof(lineBuf), "[hccl][%s][%lld.%06lld][%d:%ld][%s:%d %s] %s", kNames[level],
             (long long)(us / 1000000), (long long)(us % 1000000), (int)getpid(), (long)syscall(SYS_gettid), base,
             line, func, body);
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_sink) g_sink(level, lineBuf, g_sinkUser);
    else fprintf(stderr, "%s\n", lineBuf);
}

}  // namespace hccl
