// Minimal JSON reader (objects, arrays, strings, numbers, true/false/null) for rank tables and tuning files.
#pragma once
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace hccl {

struct JsonValue {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<JsonValue> arr;
    std::map<std::string, JsonValue> obj;
    const JsonValue *Get(const std::string &k) const
    {
        auto it = obj.find(k);
        return it == obj.end() ? nullptr : &it->second;
    }
    // numbers in rank tables are often quoted
    bool AsInt(long long *out) const
    {
        if (kind == NUM) { *out = (long long)num; return true; }
        if (kind == STR && !str.empty()) { char *e; long long v = strtoll(str.c_str(), &e, 10); if (*e == 0) { *out = v; return true; } }
        return false;
    }
};

class JsonParser {
public:
    explicit JsonParser(const std::string &s) : s_(s) {}
    JsonValue Parse()
    {
        JsonValue v = Value();
        Ws();
        if (i_ != s_.size()) Fail("trailing characters");
        return v;
    }
private:
    [[noreturn]] void Fail(const char *m) { throw std::runtime_error(std::string("json: ") + m + " at offset " + std::to_string(i_)); }
    void Ws() { while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_; }
    JsonValue Value()
    {
        Ws();
        if (i_ >= s_.size()) Fail("unexpected end");
        char c = s_[i_];
        JsonValue v;
        if (c == '{') {
            v.kind = JsonValue::OBJ;
            ++i_;
            Ws();
            if (i_ < s_.size() && s_[i_] == '}') { ++i_; return v; }
            while (true) {
                Ws();
                std::string k = Str();
                Ws();
                if (i_ >= s_.size() || s_[i_] != ':') Fail("expected ':'");
                ++i_;
                v.obj[k] = Value();
                Ws();
                if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
                if (i_ < s_.size() && s_[i_] == '}') { ++i_; break; }
                Fail("expected ',' or '}'");
            }
        } else if (c == '[') {
            v.kind = JsonValue::ARR;
            ++i_;
            Ws();
            if (i_ < s_.size() && s_[i_] == ']') { ++i_; return v; }
            while (true) {
                v.arr.push_back(Value());
                Ws();
                if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
                if (i_ < s_.size() && s_[i_] == ']') { ++i_; break; }
                Fail("expected ',' or ']'");
            }
        } else if (c == '"') {
            v.kind = JsonValue::STR;
            v.str = Str();
        } else if (s_.compare(i_, 4, "true") == 0) { v.kind = JsonValue::BOOL; v.b = true; i_ += 4; }
        else if (s_.compare(i_, 5, "false") == 0) { v.kind = JsonValue::BOOL; v.b = false; i_ += 5; }
        else if (s_.compare(i_, 4, "null") == 0) { i_ += 4; }
        else {
            char *e;
            v.num = strtod(s_.c_str() + i_, &e);
            if (e == s_.c_str() + i_) Fail("bad value");
            v.kind = JsonValue::NUM;
            i_ = (size_t)(e - s_.c_str());
        }
        return v;
    }
    std::string Str()
    {
        if (i_ >= s_.size() || s_[i_] != '"') Fail("expected string");
        ++i_;
        std::string out;
        while (i_ < s_.size() && s_[i_] != '"') {
            if (s_[i_] == '\\' && i_ + 1 < s_.size()) {
                char e = s_[++i_];
                out.push_back(e == 'n' ? '\n' : e == 't' ? '\t' : e);
            } else out.push_back(s_[i_]);
            ++i_;
        }
        if (i_ >= s_.size()) Fail("unterminated string");
        ++i_;
        return out;
    }
    const std::string &s_;
    size_t i_ = 0;
};

}  // namespace hccl
