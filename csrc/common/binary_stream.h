// Minimal binary (de)serialiser for PODs, strings, vectors and maps.
// Used to ship resource contexts / op parameters through the bootstrap network and into the engine-context
// store, as HCCL does for its host->device resource context (reference: src/common/binary_stream.h,
// src/ops/op_common/inc/alg_param.h:445-511).
#pragma once
#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

namespace hccl {

class BinaryStream {
public:
    BinaryStream() = default;
    explicit BinaryStream(std::vector<uint8_t> data) : buf_(std::move(data)) {}
    const std::vector<uint8_t> &Data() const { return buf_; }
    size_t Remaining() const { return buf_.size() - rd_; }

    template <typename T, typename std::enable_if<std::is_trivially_copyable<T>::value, int>::type = 0>
    BinaryStream &operator<<(const T &v)
    {
        const uint8_t *p = reinterpret_cast<const uint8_t *>(&v);
        buf_.insert(buf_.end(), p, p + sizeof(T));
        return *this;
    }
    template <typename T, typename std::enable_if<std::is_trivially_copyable<T>::value, int>::type = 0>
    BinaryStream &operator>>(T &v)
    {
        Need(sizeof(T));
        memcpy(&v, buf_.data() + rd_, sizeof(T));
        rd_ += sizeof(T);
        return *this;
    }
    BinaryStream &operator<<(const std::string &s)
    {
        *this << (uint64_t)s.size();
        buf_.insert(buf_.end(), s.begin(), s.end());
        return *this;
    }
    BinaryStream &operator>>(std::string &s)
    {
        uint64_t n;
        *this >> n;
        Need(n);
        s.assign(reinterpret_cast<const char *>(buf_.data() + rd_), n);
        rd_ += n;
        return *this;
    }
    template <typename T> BinaryStream &operator<<(const std::vector<T> &v)
    {
        *this << (uint64_t)v.size();
        for (const T &e : v) *this << e;
        return *this;
    }
    template <typename T> BinaryStream &operator>>(std::vector<T> &v)
    {
        uint64_t n;
        *this >> n;
        if (n > Remaining()) throw std::runtime_error("BinaryStream: vector length exceeds payload");
        v.resize(n);
        for (T &e : v) *this >> e;
        return *this;
    }
    template <typename K, typename V> BinaryStream &operator<<(const std::map<K, V> &m)
    {
        *this << (uint64_t)m.size();
        for (const auto &kv : m) { *this << kv.first; *this << kv.second; }
        return *this;
    }
    template <typename K, typename V> BinaryStream &operator>>(std::map<K, V> &m)
    {
        uint64_t n;
        *this >> n;
        m.clear();
        for (uint64_t i = 0; i < n; ++i) { K k; V v; *this >> k; *this >> v; m.emplace(std::move(k), std::move(v)); }
        return *this;
    }

private:
    void Need(size_t n) const
    {
        if (n > buf_.size() - rd_) throw std::runtime_error("BinaryStream: read past end");
    }
    std::vector<uint8_t> buf_;
    size_t rd_ = 0;
};

}  // namespace hccl
