#include "plan.h"
#include <sstream>

namespace hccl {

const char *TaskTypeName(TaskType t)
{
    switch (t) {
        case TaskType::LOCAL_COPY: return "LOCAL_COPY";
        case TaskType::LOCAL_REDUCE: return "LOCAL_REDUCE";
        case TaskType::WRITE: return "WRITE";
        case TaskType::WRITE_REDUCE: return "WRITE_REDUCE";
        case TaskType::READ: return "READ";
        case TaskType::READ_REDUCE: return "READ_REDUCE";
        case TaskType::POST: return "POST";
        case TaskType::WAIT: return "WAIT";
        case TaskType::LOCAL_POST: return "LOCAL_POST";
        case TaskType::LOCAL_WAIT: return "LOCAL_WAIT";
    }
    return "?";
}

std::string DumpPlan(const Plan &p, uint32_t rank)
{
    static const char *kBuf[] = {"IN", "OUT", "CCL", "MBOX", "ABS"};
    std::ostringstream os;
    for (size_t q = 0; q < p.queues.size(); ++q) {
        for (const Task &t : p.queues[q]) {
            os << "r" << rank << " q" << q << " " << TaskTypeName(t.type) << " peer=" << t.rank << " slot=" << t.slot
               << " dst=" << kBuf[(int)t.dst.kind] << "+" << t.dst.off << " src=" << kBuf[(int)t.src.kind] << "+"
               << t.src.off << " bytes=" << t.bytes << "\n";
        }
    }
    return os.str();
}

}  // namespace hccl
