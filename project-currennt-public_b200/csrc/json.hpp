// Minimal JSON reader for the network file (objects, arrays, strings, numbers, true/false/null).
// Enough for the reference toolkit's network.jsn: {"layers":[{...}], "weights":{name:{"input":[..],..}}}
#pragma once
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace b2 {
namespace json {

struct Value {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<Value> arr;
    std::vector<std::pair<std::string, Value> > obj;

    const Value *find(const std::string &key) const {
        for (size_t i = 0; i < obj.size(); ++i)
            if (obj[i].first == key) return &obj[i].second;
        return nullptr;
    }
    bool has(const std::string &key) const { return find(key) != nullptr; }
    const Value &at(const std::string &key) const {
        const Value *v = find(key);
        if (!v) throw std::runtime_error("json: missing key '" + key + "'");
        return *v;
    }
};

class Parser {
public:
    explicit Parser(const char *text) : p_(text) {}
    Value parse() {
        Value v = value();
        ws();
        if (*p_) fail("trailing characters");
        return v;
    }

private:
    const char *p_;
    void fail(const char *what) { throw std::runtime_error(std::string("json: ") + what); }
    void ws() {
        while (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r') ++p_;
    }
    Value value() {
        ws();
        Value v;
        if (*p_ == '{') {
            v.kind = Value::Object;
            ++p_;
            ws();
            if (*p_ == '}') { ++p_; return v; }
            for (;;) {
                ws();
                if (*p_ != '"') fail("expected string key");
                std::string k = string();
                ws();
                if (*p_ != ':') fail("expected ':'");
                ++p_;
                v.obj.push_back(std::make_pair(k, value()));
                ws();
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == '}') { ++p_; break; }
                fail("expected ',' or '}'");
            }
        } else if (*p_ == '[') {
            v.kind = Value::Array;
            ++p_;
            ws();
            if (*p_ == ']') { ++p_; return v; }
            for (;;) {
                v.arr.push_back(value());
                ws();
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == ']') { ++p_; break; }
                fail("expected ',' or ']'");
            }
        } else if (*p_ == '"') {
            v.kind = Value::String;
            v.str = string();
        } else if (!strncmp(p_, "true", 4)) { v.kind = Value::Bool; v.b = true; p_ += 4; }
        else if (!strncmp(p_, "false", 5)) { v.kind = Value::Bool; v.b = false; p_ += 5; }
        else if (!strncmp(p_, "null", 4)) { v.kind = Value::Null; p_ += 4; }
        else {
            char *end = nullptr;
            v.num = strtod(p_, &end);
            if (end == p_) fail("unexpected character");
            v.kind = Value::Number;
            p_ = end;
        }
        return v;
    }
    std::string string() {
        std::string s;
        ++p_;  // opening quote
        while (*p_ && *p_ != '"') {
            if (*p_ == '\\') {
                ++p_;
                switch (*p_) {
                    case 'n': s.push_back('\n'); break;
                    case 't': s.push_back('\t'); break;
                    case 'r': s.push_back('\r'); break;
                    case 'b': s.push_back('\b'); break;
                    case 'f': s.push_back('\f'); break;
                    case 'u': p_ += 4; s.push_back('?'); break;
                    default: s.push_back(*p_);
                }
                if (*p_) ++p_;
            } else s.push_back(*p_++);
        }
        if (*p_ != '"') fail("unterminated string");
        ++p_;
        return s;
    }
};

}  // namespace json
}  // namespace b2
