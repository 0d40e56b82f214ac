// Logging: five severities, per-subsystem masks, optional sink callback.
// Mirrors the behaviours of HCCL's log layer (reference: src/common/log.h:51-115 for the macro set and the
// error->warning downgrade switch; src/common/config_log.cc:31-48 for HCCL_DEBUG_CONFIG module masks with
// '^' inversion) on top of a plain stderr / callback sink instead of dlog.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <string>

namespace hccl {

enum LogLevel : int { LOG_DEBUG = 0, LOG_INFO = 1, LOG_WARNING = 2, LOG_ERROR = 3, LOG_RUN_INFO = 4, LOG_OFF = 5 };

// Sub-module bits selected by HCCL_DEBUG_CONFIG (comma list; a leading '^' selects everything but the list).
enum LogModule : uint32_t {
    MOD_ALG = 1u << 0,
    MOD_TASK = 1u << 1,
    MOD_RESOURCE = 1u << 2,
    MOD_KERNEL = 1u << 3,   // device-kernel launches and their exceptions (HCCL's AIV_OPS_EXC)
    MOD_BOOT = 1u << 4,
    MOD_ALL = 0xffffffffu
};

using LogSink = void (*)(int level, const char *line, void *user);

void LogInitFromEnv();                       // HCCL_LOG_LEVEL, HCCL_DEBUG_CONFIG, HCCL_ENTRY_LOG_ENABLE
void LogSetLevel(int level);
int LogGetLevel();
void LogSetSink(LogSink sink, void *user);   // nullptr restores stderr
void LogSetModuleMask(uint32_t mask);
uint32_t LogGetModuleMask();
bool LogParseDebugConfig(const std::string &value, uint32_t *maskOut);  // returns false on unknown token
// While > 0 on this thread, ERROR records are emitted as WARNING (used around fallbacks that are expected
// to fail, e.g. probing NVLS and falling back to peer loads).
void LogPushErrorToWarn();
void LogPopErrorToWarn();
// Nothing below RUN_INFO is written by this thread between the two calls (trial runs whose failure is an expected answer).
void LogPushMute();
void LogPopMute();
bool LogModuleEnabled(uint32_t module);
void LogWrite(int level, const char *file, int line, const char *func, const char *fmt, ...)
    __attribute__((format(printf, 5, 6)));
uint64_t LogRecordCount(int level);          // counters for tests / observability

}  // namespace hccl

#define HCCL_LOG_(lvl, ...)                                                        \
    do {                                                                           \
        if ((lvl) >= ::hccl::LogGetLevel())                                        \
            ::hccl::LogWrite((lvl), __FILE__, __LINE__, __func__, __VA_ARGS__);    \
    } while (0)
#define HCCL_DEBUG(...) HCCL_LOG_(::hccl::LOG_DEBUG, __VA_ARGS__)
#define HCCL_INFO(...) HCCL_LOG_(::hccl::LOG_INFO, __VA_ARGS__)
#define HCCL_WARNING(...) HCCL_LOG_(::hccl::LOG_WARNING, __VA_ARGS__)
#define HCCL_ERROR(...) HCCL_LOG_(::hccl::LOG_ERROR, __VA_ARGS__)
#define HCCL_RUN_INFO(...) HCCL_LOG_(::hccl::LOG_RUN_INFO, __VA_ARGS__)
#define HCCL_MOD_DEBUG(mod, ...)                                                   \
    do {                                                                           \
        if (::hccl::LogModuleEnabled(mod)) HCCL_LOG_(::hccl::LOG_DEBUG, __VA_ARGS__); \
    } while (0)

// Return-on-error helpers used all over the host code.
#define CHK_RET(expr)                                                              \
    do {                                                                           \
        HcclResult _r = (expr);                                                    \
        if (_r != HCCL_SUCCESS) {                                                  \
            HCCL_ERROR("call failed: %s -> %d", #expr, (int)_r);                   \
            return _r;                                                             \
        }                                                                          \
    } while (0)
#define CHK_PTR_NULL(p)                                                            \
    do {                                                                           \
        if ((p) == nullptr) {                                                      \
            HCCL_ERROR("[EI0003] pointer %s is null", #p);                         \
            return HCCL_E_PTR;                                                     \
        }                                                                          \
    } while (0)
#define CHK_PRT_RET(cond, logstmt, ret)                                            \
    do {                                                                           \
        if (cond) {                                                                \
            logstmt;                                                               \
            return (ret);                                                          \
        }                                                                          \
    } while (0)
