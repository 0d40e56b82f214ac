#include "bootstrap.h"
#include <arpa/inet.h>
#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <random>
#include <set>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>
#include "../common/env_config.h"
#include "../common/log.h"

namespace hccl {
namespace {

enum : uint32_t { OP_HELLO = 1, OP_ALLGATHER, OP_PUT, OP_GET, OP_HEARTBEAT, OP_BYE };
constexpr uint32_t kMsgMagic = 0x48434d53u;

struct MsgHdr {
    uint32_t magic, op, rank, chan;
    uint64_t seq, len;
};
struct ReplyHdr {
    uint32_t status;
    uint32_t pad;
    uint64_t len;
};

int64_t NowMs()
{
    using namespace std::chrono;
    return duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count();
}

bool WriteAll(int fd, const void *buf, size_t n)
{
    const char *p = (const char *)buf;
    while (n > 0) {
        ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
        if (w < 0) { if (errno == EINTR) continue; return false; }
        p += w;
        n -= (size_t)w;
    }
    return true;
}
// 0 ok, 1 timeout, 2 closed / error
int ReadAll(int fd, void *buf, size_t n)
{
    char *p = (char *)buf;
    while (n > 0) {
        ssize_t r = ::recv(fd, p, n, 0);
        if (r == 0) return 2;
        if (r < 0) {
            if (errno == EINTR) continue;
            if (errno == EAGAIN || errno == EWOULDBLOCK) return 1;
            return 2;
        }
        p += r;
        n -= (size_t)r;
    }
    return 0;
}
void SetRecvTimeout(int fd, uint32_t sec)
{
    struct timeval tv;
    tv.tv_sec = sec;
    tv.tv_usec = 0;
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
}

std::mutex g_listenMu;
std::map<uint64_t, int> g_listeners;  // nonce -> listening fd created by CreateRootInfo

}  // namespace

// ------------------------------------------------------------------------------------------- service (rank 0)
class BootstrapRoot {
public:
    BootstrapRoot(int listenFd, uint32_t nranks) : listenFd_(listenFd), n_(nranks)
    {
        stopFd_ = eventfd(0, EFD_NONBLOCK);
        // HCCL_DFS_CONFIG connection_fault_detection_time (seconds; default 20, 0 = a silent peer is never declared lost, only a closed
        // connection is); HCCL_HEARTBEAT_LOST_MS overrides it in milliseconds
        const uint32_t detectSec = GetEnvConfig().connectionFaultDetectionSec;
        lostMs_ = detectSec ? (int64_t)detectSec * 1000 : INT64_MAX / 4;
        if (const char *e = getenv("HCCL_HEARTBEAT_LOST_MS")) lostMs_ = atoi(e) > 0 ? atoi(e) : lostMs_;
        lastSeen_.assign(n_, 0);
        hbOpen_.assign(n_, false);
        opsIssued_.assign(n_, 0);
        opsDone_.assign(n_, 0);
        reported_.assign(n_, false);
        th_ = std::thread([this] { Run(); });
    }
    ~BootstrapRoot()
    {
        uint64_t one = 1;
        (void)!write(stopFd_, &one, 8);
        if (th_.joinable()) th_.join();
        for (auto &c : conns_) if (c.fd >= 0) close(c.fd);
        close(listenFd_);
        close(stopFd_);
    }

private:
    struct Conn { int fd; int rank; int chan; };
    struct Round { std::vector<std::vector<uint8_t>> parts; uint32_t have = 0; };

    void Reply(int fd, uint32_t status, const void *p, size_t len)
    {
        ReplyHdr h{status, 0, (uint64_t)len};
        if (WriteAll(fd, &h, sizeof(h)) && len) WriteAll(fd, p, len);
    }
    int MainFd(int rank)
    {
        for (auto &c : conns_) if (c.rank == rank && c.chan == 0 && c.fd >= 0) return c.fd;
        return -1;
    }
    void Handle(Conn &c)
    {
        MsgHdr h;
        if (ReadAll(c.fd, &h, sizeof(h)) != 0 || h.magic != kMsgMagic || h.len > (1ull << 30)) { Drop(c, false); return; }
        std::vector<uint8_t> payload(h.len);
        if (h.len && ReadAll(c.fd, payload.data(), h.len) != 0) { Drop(c, false); return; }
        switch (h.op) {
            case OP_HELLO:
                c.rank = (int)h.rank;
                c.chan = (int)h.chan;
                if (c.chan == 1 && c.rank >= 0 && c.rank < (int)n_) { hbOpen_[c.rank] = true; lastSeen_[c.rank] = NowMs(); }
                Reply(c.fd, 0, nullptr, 0);
                break;
            case OP_ALLGATHER: {
                Round &r = rounds_[h.seq];
                if (r.parts.empty()) r.parts.resize(n_);
                if (h.rank < n_ && r.parts[h.rank].empty()) { r.parts[h.rank] = payload; r.parts[h.rank].push_back(0); r.have++; }
                if (r.have == n_) {
                    std::vector<uint8_t> all;
                    for (auto &p : r.parts) all.insert(all.end(), p.begin(), p.end() - 1);
                    for (uint32_t k = 0; k < n_; ++k) { int fd = MainFd((int)k); if (fd >= 0) Reply(fd, 0, all.data(), all.size()); }
                    rounds_.erase(h.seq);
                }
                break;
            }
            case OP_PUT: {
                size_t klen = h.seq;  // key length rides in seq
                if (klen > payload.size()) { Reply(c.fd, 1, nullptr, 0); break; }
                std::string key((char *)payload.data(), klen);
                kv_[key].assign(payload.begin() + klen, payload.end());
                Reply(c.fd, 0, nullptr, 0);
                auto it = pendingGets_.find(key);
                if (it != pendingGets_.end()) {
                    for (int fd : it->second) Reply(fd, 0, kv_[key].data(), kv_[key].size());
                    pendingGets_.erase(it);
                }
                break;
            }
            case OP_GET: {
                std::string key((char *)payload.data(), payload.size());
                auto it = kv_.find(key);
                if (it != kv_.end()) Reply(c.fd, 0, it->second.data(), it->second.size());
                else pendingGets_[key].push_back(c.fd);
                break;
            }
            case OP_HEARTBEAT: {
                HeartbeatMsg m{0, 0, 0, 0};
                memcpy(&m, payload.data(), std::min(payload.size(), sizeof(m)));
                const int32_t err = m.error;
                if (h.rank < n_) {
                    lastSeen_[h.rank] = NowMs();
                    if (payload.size() >= sizeof(m)) { opsIssued_[h.rank] = m.opsIssued; opsDone_[h.rank] = m.opsDone; reported_[h.rank] = true; }
                }
                if (m.clearError) { errorRank_ = -1; errorCode_ = 0; }
                if (err != 0 && errorRank_ < 0) { errorRank_ = (int)h.rank; errorCode_ = err; }
                HeartbeatReply rep{-1, errorRank_, errorCode_, 0, -1, 0, 0, 0};
                bool allReported = true;
                for (uint32_t k = 0; k < n_; ++k) allReported = allReported && reported_[k];
                if (allReported) {
                    rep.lagRank = 0;
                    for (uint32_t k = 0; k < n_; ++k) {
                        if (opsDone_[k] < opsDone_[rep.lagRank]) rep.lagRank = (int32_t)k;
                        rep.maxIssued = std::max(rep.maxIssued, opsIssued_[k]);
                    }
                    rep.lagDone = opsDone_[rep.lagRank];
                }
                int64_t now = NowMs();
                for (uint32_t k = 0; k < n_; ++k) {
                    if (hbOpen_[k]) rep.aliveMask |= 1u << (k & 31);
                    bool lost = (lastSeen_[k] != 0 && now - lastSeen_[k] > lostMs_) || (everOpen_.count((int)k) && !hbOpen_[k] && !saidBye_.count((int)k));
                    if (lost && rep.deadRank < 0) rep.deadRank = (int)k;
                }
                Reply(c.fd, 0, &rep, sizeof(rep));
                break;
            }
            case OP_BYE:
                saidBye_.insert(c.rank);
                Reply(c.fd, 0, nullptr, 0);
                break;
            default: Reply(c.fd, 1, nullptr, 0);
        }
        if (c.chan == 1 && c.rank >= 0) everOpen_.insert(c.rank);
    }
    void Drop(Conn &c, bool)
    {
        if (c.chan == 1 && c.rank >= 0 && c.rank < (int)n_) hbOpen_[c.rank] = false;
        for (auto &kv : pendingGets_) {
            auto &v = kv.second;
            for (size_t i = 0; i < v.size();) { if (v[i] == c.fd) v.erase(v.begin() + i); else ++i; }
        }
        close(c.fd);
        c.fd = -1;
    }
    void Run()
    {
        while (true) {
            std::vector<pollfd> pf;
            pf.push_back({stopFd_, POLLIN, 0});
            pf.push_back({listenFd_, POLLIN, 0});
            for (auto &c : conns_) if (c.fd >= 0) pf.push_back({c.fd, POLLIN, 0});
            int rc = poll(pf.data(), pf.size(), 1000);
            if (rc < 0) { if (errno == EINTR) continue; break; }
            if (pf[0].revents) break;
            if (pf[1].revents & POLLIN) {
                int fd = accept(listenFd_, nullptr, nullptr);
                if (fd >= 0) {
                    int one = 1;
                    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
                    SetRecvTimeout(fd, 10);
                    conns_.push_back({fd, -1, -1});
                }
            }
            for (size_t i = 2; i < pf.size(); ++i) {
                if (!(pf[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
                for (auto &c : conns_) if (c.fd == pf[i].fd) { Handle(c); break; }
            }
        }
    }

    int listenFd_, stopFd_;
    uint32_t n_;
    std::thread th_;
    std::vector<Conn> conns_;
    std::map<uint64_t, Round> rounds_;
    std::map<std::string, std::vector<uint8_t>> kv_;
    std::map<std::string, std::vector<int>> pendingGets_;
    std::vector<int64_t> lastSeen_;
    std::vector<bool> hbOpen_;
    std::set<int> everOpen_, saidBye_;
    int errorRank_ = -1, errorCode_ = 0;
    std::vector<uint64_t> opsIssued_, opsDone_;
    std::vector<bool> reported_;
    int64_t lostMs_;
};

// ------------------------------------------------------------------------------------------- client
Bootstrap::~Bootstrap() { Close(); }

void Bootstrap::Close()
{
    if (fd_ >= 0) {
        std::vector<uint8_t> rep;
        if (hbFd_ >= 0) { Request(hbFd_, OP_BYE, 0, nullptr, 0, &rep, 2); close(hbFd_); hbFd_ = -1; }
        close(fd_);
        fd_ = -1;
    }
    root_.reset();
}

HcclResult Bootstrap::CreateRootInfo(HcclRootInfo *out)
{
    if (out == nullptr) return HCCL_E_PTR;
    InitEnvConfig();
    const AlgEnvConfig &env = GetEnvConfig();
    int fd = socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return HCCL_E_SYSCALL;
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)env.ifBasePort);
    if (inet_pton(AF_INET, env.ifIp.c_str(), &addr.sin_addr) != 1) { close(fd); HCCL_ERROR("HCCL_IF_IP=%s is not an IPv4 address", env.ifIp.c_str()); return HCCL_E_PARA; }
    if (bind(fd, (sockaddr *)&addr, sizeof(addr)) != 0 || listen(fd, 256) != 0) {
        HCCL_ERROR("bootstrap: cannot listen on %s:%u (%s)", env.ifIp.c_str(), env.ifBasePort, strerror(errno));
        close(fd);
        return HCCL_E_TCP_CONNECT;
    }
    socklen_t len = sizeof(addr);
    getsockname(fd, (sockaddr *)&addr, &len);
    memset(out, 0, sizeof(*out));
    RootInfoBlob *b = reinterpret_cast<RootInfoBlob *>(out->internal);
    b->magic = kRootMagic;
    b->port = ntohs(addr.sin_port);
    std::random_device rd;
    b->nonce = ((uint64_t)rd() << 32) ^ rd() ^ ((uint64_t)getpid() << 16);
    b->pid = getpid();
    snprintf(b->ip, sizeof(b->ip), "%s", env.ifIp.c_str());
    std::lock_guard<std::mutex> lk(g_listenMu);
    g_listeners[b->nonce] = fd;
    return HCCL_SUCCESS;
}

// Root info for rank-table initialisation: every rank derives the same (ip, port, nonce); only rank 0 listens.
HcclResult BootstrapFixedRootInfo(const std::string &ip, uint32_t port, uint64_t nonce, bool doListen, HcclRootInfo *out)
{
    memset(out, 0, sizeof(*out));
    RootInfoBlob *b = reinterpret_cast<RootInfoBlob *>(out->internal);
    b->magic = kRootMagic;
    b->port = port;
    b->nonce = nonce;
    b->pid = 0;
    snprintf(b->ip, sizeof(b->ip), "%s", ip.c_str());
    if (!doListen) return HCCL_SUCCESS;
    int fd = socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return HCCL_E_SYSCALL;
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)port);
    addr.sin_addr.s_addr = htonl(INADDR_ANY);
    if (bind(fd, (sockaddr *)&addr, sizeof(addr)) != 0 || listen(fd, 256) != 0) {
        HCCL_ERROR("bootstrap: cannot listen on port %u (%s)", port, strerror(errno));
        close(fd);
        return HCCL_E_TCP_CONNECT;
    }
    std::lock_guard<std::mutex> lk(g_listenMu);
    g_listeners[nonce] = fd;
    return HCCL_SUCCESS;
}

static int ConnectTo(const char *ip, uint32_t port, uint32_t timeoutSec)
{
    int64_t deadline = NowMs() + (int64_t)timeoutSec * 1000;
    while (true) {
        int fd = socket(AF_INET, SOCK_STREAM, 0);
        if (fd < 0) return -1;
        sockaddr_in addr{};
        addr.sin_family = AF_INET;
        addr.sin_port = htons((uint16_t)port);
        inet_pton(AF_INET, ip, &addr.sin_addr);
        if (connect(fd, (sockaddr *)&addr, sizeof(addr)) == 0) {
            int one = 1;
            setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
            return fd;
        }
        close(fd);
        if (NowMs() > deadline) return -1;
        usleep(20000);
    }
}

HcclResult Bootstrap::Init(const HcclRootInfo &info, uint32_t rank, uint32_t nranks, uint32_t timeoutSec, bool heartbeat)
{
    const RootInfoBlob *b = reinterpret_cast<const RootInfoBlob *>(info.internal);
    if (b->magic != kRootMagic) { HCCL_ERROR("bootstrap: root info blob is not initialised"); return HCCL_E_PARA; }
    rank_ = rank;
    nranks_ = nranks;
    nonce_ = b->nonce;
    timeoutSec_ = timeoutSec;
    if (rank == 0) {
        int lfd = -1;
        {
            std::lock_guard<std::mutex> lk(g_listenMu);
            auto it = g_listeners.find(b->nonce);
            if (it != g_listeners.end()) { lfd = it->second; g_listeners.erase(it); }
        }
        if (lfd < 0) { HCCL_ERROR("bootstrap: rank 0 must run in the process that called HcclGetRootInfo"); return HCCL_E_PARA; }
        root_ = std::make_shared<BootstrapRoot>(lfd, nranks);
    }
    fd_ = ConnectTo(b->ip, b->port, timeoutSec);
    if (fd_ < 0) { HCCL_ERROR("bootstrap: rank %u cannot reach root %s:%u within %u s", rank, b->ip, b->port, timeoutSec); return HCCL_E_TCP_CONNECT; }
    std::vector<uint8_t> rep;
    {
        MsgHdr h{kMsgMagic, OP_HELLO, rank_, 0, 0, 0};
        SetRecvTimeout(fd_, timeoutSec);
        if (!WriteAll(fd_, &h, sizeof(h))) return HCCL_E_TCP_TRANSFER;
        ReplyHdr rh;
        if (ReadAll(fd_, &rh, sizeof(rh)) != 0) return HCCL_E_TCP_TRANSFER;
    }
    if (heartbeat) {
        hbFd_ = ConnectTo(b->ip, b->port, timeoutSec);
        if (hbFd_ >= 0) {
            MsgHdr h{kMsgMagic, OP_HELLO, rank_, 1, 0, 0};
            SetRecvTimeout(hbFd_, 5);
            ReplyHdr rh;
            if (!WriteAll(hbFd_, &h, sizeof(h)) || ReadAll(hbFd_, &rh, sizeof(rh)) != 0) { close(hbFd_); hbFd_ = -1; }
        }
    }
    return Barrier();
}

HcclResult Bootstrap::Request(int fd, uint32_t op, uint64_t seq, const void *payload, size_t len,
                              std::vector<uint8_t> *reply, uint32_t timeoutSec)
{
    if (fd < 0) return HCCL_E_INTERNAL;
    MsgHdr h{kMsgMagic, op, rank_, 0, seq, (uint64_t)len};
    SetRecvTimeout(fd, timeoutSec);
    if (!WriteAll(fd, &h, sizeof(h)) || (len && !WriteAll(fd, payload, len))) return HCCL_E_TCP_TRANSFER;
    ReplyHdr rh;
    int rc = ReadAll(fd, &rh, sizeof(rh));
    if (rc == 1) return HCCL_E_TIMEOUT;
    if (rc != 0) return HCCL_E_TCP_TRANSFER;
    reply->resize(rh.len);
    if (rh.len) { rc = ReadAll(fd, reply->data(), rh.len); if (rc != 0) return rc == 1 ? HCCL_E_TIMEOUT : HCCL_E_TCP_TRANSFER; }
    return rh.status == 0 ? HCCL_SUCCESS : HCCL_E_INTERNAL;
}

HcclResult Bootstrap::AllGather(const void *in, size_t bytesEach, void *out)
{
    std::lock_guard<std::mutex> lk(mu_);
    uint64_t seq = ++seq_;
    if (dropNext_ > 0) {   // injected fault: this rank's contribution never leaves
        --dropNext_;
        std::vector<uint8_t> rep;
        ReplyHdr rh;
        SetRecvTimeout(fd_, timeoutSec_);
        int rc = ReadAll(fd_, &rh, sizeof(rh));
        return rc == 1 ? HCCL_E_TIMEOUT : HCCL_E_TCP_TRANSFER;
    }
    std::vector<uint8_t> rep;
    HcclResult r = Request(fd_, OP_ALLGATHER, seq, in, bytesEach, &rep, timeoutSec_);
    if (r != HCCL_SUCCESS) {
        HCCL_ERROR("bootstrap: allgather #%llu failed on rank %u (%d): a peer did not join within %u s",
                   (unsigned long long)seq, rank_, (int)r, timeoutSec_);
        return r;
    }
    if (rep.size() != bytesEach * nranks_) { HCCL_ERROR("bootstrap: allgather size mismatch: got %zu, want %zu (ranks disagree on the payload size)", rep.size(), bytesEach * nranks_); return HCCL_E_INTERNAL; }
    if (bytesEach) memcpy(out, rep.data(), rep.size());
    return HCCL_SUCCESS;
}

HcclResult Bootstrap::Barrier() { return AllGather(nullptr, 0, nullptr); }

HcclResult Bootstrap::Broadcast(void *buf, size_t bytes, uint32_t root)
{
    std::vector<uint8_t> all(bytes * nranks_);
    HcclResult r = AllGather(buf, bytes, all.data());
    if (r != HCCL_SUCCESS) return r;
    memcpy(buf, all.data() + bytes * root, bytes);
    return HCCL_SUCCESS;
}

HcclResult Bootstrap::Put(const std::string &key, const void *val, size_t bytes)
{
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<uint8_t> payload(key.begin(), key.end());
    payload.insert(payload.end(), (const uint8_t *)val, (const uint8_t *)val + bytes);
    std::vector<uint8_t> rep;
    return Request(fd_, OP_PUT, key.size(), payload.data(), payload.size(), &rep, timeoutSec_);
}

HcclResult Bootstrap::Get(const std::string &key, std::vector<uint8_t> *val, uint32_t timeoutSec)
{
    std::lock_guard<std::mutex> lk(mu_);
    return Request(fd_, OP_GET, 0, key.data(), key.size(), val, timeoutSec);
}

HcclResult Bootstrap::Heartbeat(const HeartbeatMsg &msg, HeartbeatReply *reply)
{
    std::lock_guard<std::mutex> lk(hbMu_);
    if (hbFd_ < 0) return HCCL_E_UNAVAIL;
    std::vector<uint8_t> rep;
    HcclResult r = Request(hbFd_, OP_HEARTBEAT, 0, &msg, sizeof(msg), &rep, 5);
    if (r != HCCL_SUCCESS) return r;
    if (rep.size() != sizeof(HeartbeatReply)) return HCCL_E_INTERNAL;
    memcpy(reply, rep.data(), sizeof(HeartbeatReply));
    return HCCL_SUCCESS;
}

// ------------------------------------------------------------------------------------------- fd passing
namespace {
socklen_t AbstractAddr(sockaddr_un *sa, uint64_t nonce, const std::string &tag, uint32_t rank)
{
    memset(sa, 0, sizeof(*sa));
    sa->sun_family = AF_UNIX;
    int n = snprintf(sa->sun_path + 1, sizeof(sa->sun_path) - 1, "hcclb200-%016llx-%s-%u", (unsigned long long)nonce, tag.c_str(), rank);
    return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}
bool SendFdList(int sock, const std::vector<int> &fds)
{
    uint32_t n = (uint32_t)fds.size();
    char cbuf[CMSG_SPACE(sizeof(int) * 16)];
    memset(cbuf, 0, sizeof(cbuf));
    iovec iov{&n, sizeof(n)};
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    if (n > 0) {
        msg.msg_control = cbuf;
        msg.msg_controllen = CMSG_SPACE(sizeof(int) * n);
        cmsghdr *c = CMSG_FIRSTHDR(&msg);
        c->cmsg_level = SOL_SOCKET;
        c->cmsg_type = SCM_RIGHTS;
        c->cmsg_len = CMSG_LEN(sizeof(int) * n);
        memcpy(CMSG_DATA(c), fds.data(), sizeof(int) * n);
    }
    return sendmsg(sock, &msg, MSG_NOSIGNAL) == (ssize_t)sizeof(n);
}
bool RecvFdList(int sock, std::vector<int> *fds)
{
    uint32_t n = 0;
    char cbuf[CMSG_SPACE(sizeof(int) * 16)];
    iovec iov{&n, sizeof(n)};
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = cbuf;
    msg.msg_controllen = sizeof(cbuf);
    if (recvmsg(sock, &msg, 0) != (ssize_t)sizeof(n)) return false;
    fds->clear();
    if (n == 0) return true;
    cmsghdr *c = CMSG_FIRSTHDR(&msg);
    if (c == nullptr || c->cmsg_type != SCM_RIGHTS) return false;
    fds->resize(n);
    memcpy(fds->data(), CMSG_DATA(c), sizeof(int) * n);
    return true;
}
}  // namespace

HcclResult FdExchange::AllGatherFds(uint64_t nonce, const std::string &tag, uint32_t rank, uint32_t nranks,
                                    const std::vector<int> &fds, std::vector<std::vector<int>> *out, Bootstrap *boot,
                                    uint32_t timeoutSec)
{
    if (fds.size() > 16) return HCCL_E_PARA;
    out->assign(nranks, {});
    (*out)[rank] = fds;
    if (nranks == 1) return HCCL_SUCCESS;
    int lfd = socket(AF_UNIX, SOCK_STREAM, 0);
    if (lfd < 0) return HCCL_E_SYSCALL;
    sockaddr_un sa;
    socklen_t sl = AbstractAddr(&sa, nonce, tag, rank);
    if (bind(lfd, (sockaddr *)&sa, sl) != 0 || listen(lfd, 64) != 0) {
        HCCL_ERROR("fd exchange: bind/listen failed: %s", strerror(errno));
        close(lfd);
        return HCCL_E_SYSCALL;
    }
    std::atomic<bool> serveOk{true};
    std::thread server([&] {
        for (uint32_t k = 0; k + 1 < nranks; ++k) {
            pollfd p{lfd, POLLIN, 0};
            if (poll(&p, 1, (int)timeoutSec * 1000) <= 0) { serveOk = false; return; }
            int c = accept(lfd, nullptr, nullptr);
            if (c < 0) { serveOk = false; return; }
            if (!SendFdList(c, fds)) serveOk = false;
            char ack;
            SetRecvTimeout(c, timeoutSec);
            (void)!recv(c, &ack, 1, 0);
            close(c);
        }
    });
    HcclResult res = boot->Barrier();  // every listener is up
    if (res == HCCL_SUCCESS) {
        for (uint32_t k = 1; k < nranks && res == HCCL_SUCCESS; ++k) {
            uint32_t peer = (rank + k) % nranks;
            int c = socket(AF_UNIX, SOCK_STREAM, 0);
            sockaddr_un pa;
            socklen_t pl = AbstractAddr(&pa, nonce, tag, peer);
            if (connect(c, (sockaddr *)&pa, pl) != 0) { HCCL_ERROR("fd exchange: connect to rank %u failed: %s", peer, strerror(errno)); res = HCCL_E_SYSCALL; close(c); break; }
            SetRecvTimeout(c, timeoutSec);
            if (!RecvFdList(c, &(*out)[peer])) { HCCL_ERROR("fd exchange: no descriptors from rank %u", peer); res = HCCL_E_SYSCALL; }
            char ack = 1;
            (void)!send(c, &ack, 1, MSG_NOSIGNAL);
            close(c);
        }
    }
    server.join();
    close(lfd);
    if (res == HCCL_SUCCESS && !serveOk) res = HCCL_E_TIMEOUT;
    HcclResult b2 = boot->Barrier();
    return res != HCCL_SUCCESS ? res : b2;
}

}  // namespace hccl
