// One-shot environment configuration.
//
// Same variable names and value grammar as HCCL where the concept carries over to an NVSwitch box
// (reference: src/common/alg_env_config.cc:169-316 InitEnvConfig; :762-830 HCCL_OP_EXPANSION_MODE; :318 HCCL_ALGO;
// :948 HCCL_DETERMINISTIC; :69 HCCL_EXEC_TIMEOUT; :914 HCCL_OP_RETRY_ENABLE; :996 HCCL_DFS_CONFIG; :119
// HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO; struct AlgEnvConfig alg_env_config.h:35-83).
// Engine names: SM | NVLS | COPY_ENGINE | HOST; the Ascend names are accepted as aliases
// (AIV -> SM, CCU_MS / CCU_SCHED -> NVLS, AI_CPU / AICPU_TS -> COPY_ENGINE).
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include "hccl/hccl_types.h"

namespace hccl {

enum class AlgoType : uint8_t {  // HCCL_ALGO vocabulary (reference: src/common/alg_type.h:19-33)
    DEFAULT = 0, RING, PIPELINE, FULLMESH, HDR, PAIRWISE, NHR, NHR_V1, NB, AHC, NA
};
enum class Deterministic : uint8_t { OFF = 0, ON = 1, STRICT = 2 };
enum class InconsistentCheck : uint8_t { OFF = 0, FIRST = 1, EVERY = 2 };

struct AlgoLevels {
    AlgoType level[3] = {AlgoType::DEFAULT, AlgoType::DEFAULT, AlgoType::DEFAULT};
};

struct AlgEnvConfig {
    // engine selection: global default and per-op overrides ("allreduce:NVLS;allgather:SM")
    HcclCommEngine expansionMode = HCCL_ENGINE_DEFAULT;
    std::map<HcclCMDType, HcclCommEngine> expansionModePerOp;
    // HCCL_ALGO: global and per-op level configuration
    AlgoLevels algo;
    std::map<HcclCMDType, AlgoLevels> algoPerOp;
    bool algoSet = false;
    // explicit algorithm-name override, e.g. HCCL_ALGO_NAME="allreduce=SmAllReduceMesh1DTwoShot"
    std::map<HcclCMDType, std::string> algoNamePerOp;
    Deterministic deterministic = Deterministic::OFF;
    uint32_t execTimeoutSec = 1836;      // host-visible op timeout (HCCL default)
    bool execTimeoutSet = false;
    uint32_t deviceWaitTimeoutMs = 20000;  // bound of every in-kernel spin; HCCL_DEVICE_WAIT_TIMEOUT_MS
    uint32_t connectTimeoutSec = 120;
    uint64_t bufferSizeBytes = 200ull << 20;  // per CCL buffer, two per communicator
    bool entryLogEnable = false;
    // op retry (parsed and reported; retries re-run the op from unpolluted input on the host engines)
    bool opRetryIntraServer = false, opRetryInterServer = false, opRetryInterSuperPod = false;
    uint32_t opRetryMaxCnt = 1, opRetryHoldTimeMs = 5000, opRetryIntervalMs = 1000;
    // DFS (fault detection) switches
    bool clusterHeartbeat = true, stuckDetection = true, taskException = true;
    uint32_t connectionFaultDetectionSec = 20;
    uint32_t taskMonitorIntervalMs = 0;
    InconsistentCheck inconsistentCheck = InconsistentCheck::FIRST;
    // split ratio of the concurrent algorithms (one payload shared by two algorithms in one launch): first : second part
    uint32_t multiDimSplitRatio[2] = {1, 1};
    bool multiDimSplitSet = false;
    // link-type switches accepted for compatibility
    bool intraRoceEnable = false, intraPcieEnable = false, interHccsDisable = false;
    // bootstrap
    std::string ifIp = "127.0.0.1";
    uint32_t ifBasePort = 0;             // 0 = ephemeral
    std::string socketIfName;
    // B200-specific
    bool nvlsEnable = true;              // HCCL_NVLS_ENABLE=0 keeps every kernel on plain peer loads/stores
    uint32_t maxCtas = 0;                // HCCL_MAX_CTAS caps the grid of collective kernels (0 = selector decides)
    std::string tuningFile;              // HCCL_TUNING_FILE: text crossover table (rows as in hccl_b200/tuning/b200.txt) laid over the built-in one
};

HcclResult InitEnvConfig();                     // idempotent; parses once
const AlgEnvConfig &GetEnvConfig();
void ResetAlgEnvConfigInitState();              // tests: force re-parse on the next InitEnvConfig
// Address of the interface HCCL_SOCKET_IFNAME selects (false: none matches).
bool ResolveSocketIfName(const std::string &spec, std::string *ip, std::string *ifName);
// Individual parsers (exposed for unit tests)
HcclResult ParseExpansionMode(const std::string &v, AlgEnvConfig *cfg);
HcclResult ParseHcclAlgo(const std::string &v, AlgEnvConfig *cfg);
HcclResult ParseDeterministic(const std::string &v, AlgEnvConfig *cfg);
HcclResult ParseExecTimeout(const std::string &v, AlgEnvConfig *cfg);
HcclResult ParseDfsConfig(const std::string &v, AlgEnvConfig *cfg);
HcclResult ParseOpRetryEnable(const std::string &v, AlgEnvConfig *cfg);
HcclResult ParseOpRetryParams(const std::string &v, AlgEnvConfig *cfg);
HcclResult ParseBufferSize(const std::string &v, AlgEnvConfig *cfg);
HcclResult ParseSplitRatio(const std::string &v, AlgEnvConfig *cfg);
HcclResult ParseAlgoName(const std::string &v, AlgEnvConfig *cfg);
bool ParseEngineName(const std::string &name, HcclCommEngine *out);
bool ParseOpName(const std::string &name, HcclCMDType *out);
const char *EngineName(HcclCommEngine e);
const char *AlgoTypeName(AlgoType a);

}  // namespace hccl
