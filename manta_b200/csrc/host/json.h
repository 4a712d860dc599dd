// Minimal JSON value, parser and writer for the plan (Module) documents the host executor reads.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace mjson {

struct Value;
using Array = std::vector<Value>;
using Object = std::vector<std::pair<std::string, Value>>;  // insertion order kept

struct Value {
    enum Kind { Null, Bool, Number, String, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::shared_ptr<Array> arr;
    std::shared_ptr<Object> obj;

    static Value make_string(const std::string& s) { Value v; v.kind = String; v.str = s; return v; }
    static Value make_number(double d) { Value v; v.kind = Number; v.num = d; return v; }
    static Value make_bool(bool x) { Value v; v.kind = Bool; v.b = x; return v; }
    static Value make_array() { Value v; v.kind = Arr; v.arr = std::make_shared<Array>(); return v; }
    static Value make_object() { Value v; v.kind = Obj; v.obj = std::make_shared<Object>(); return v; }

    bool is_object() const { return kind == Obj; }
    bool is_array() const { return kind == Arr; }
    bool is_string() const { return kind == String; }
    const Value* get(const std::string& key) const {
        if (kind != Obj) return nullptr;
        for (const auto& kv : *obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    std::string get_string(const std::string& key, const std::string& dflt = "") const {
        const Value* v = get(key);
        return (v && v->kind == String) ? v->str : dflt;
    }
    const Array& items() const {
        static const Array empty;
        return kind == Arr ? *arr : empty;
    }
    void set(const std::string& key, Value v) {
        for (auto& kv : *obj)
            if (kv.first == key) { kv.second = std::move(v); return; }
        obj->emplace_back(key, std::move(v));
    }
    void push(Value v) { arr->push_back(std::move(v)); }
};

class Parser {
  public:
    explicit Parser(const std::string& text) : s_(text) {}
    bool parse(Value* out, std::string* err) {
        skip();
        if (!value(out, err)) return false;
        skip();
        if (i_ != s_.size()) return fail(err, "trailing characters");
        return true;
    }

  private:
    const std::string& s_;
    size_t i_ = 0;
    bool fail(std::string* err, const char* what) {
        if (err) *err = std::string("json: ") + what + " at offset " + std::to_string(i_);
        return false;
    }
    void skip() {
        while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_;
    }
    bool literal(const char* lit) {
        size_t n = 0;
        while (lit[n]) ++n;
        if (s_.compare(i_, n, lit) != 0) return false;
        i_ += n;
        return true;
    }
    bool string(std::string* out, std::string* err) {
        if (s_[i_] != '"') return fail(err, "expected string");
        ++i_;
        out->clear();
        while (i_ < s_.size() && s_[i_] != '"') {
            char c = s_[i_++];
            if (c != '\\') { out->push_back(c); continue; }
            if (i_ >= s_.size()) return fail(err, "bad escape");
            char e = s_[i_++];
            switch (e) {
                case '"': out->push_back('"'); break;
                case '\\': out->push_back('\\'); break;
                case '/': out->push_back('/'); break;
                case 'b': out->push_back('\b'); break;
                case 'f': out->push_back('\f'); break;
                case 'n': out->push_back('\n'); break;
                case 'r': out->push_back('\r'); break;
                case 't': out->push_back('\t'); break;
                case 'u': {
                    if (i_ + 4 > s_.size()) return fail(err, "bad \\u escape");
                    unsigned cp = (unsigned)strtoul(s_.substr(i_, 4).c_str(), nullptr, 16);
                    i_ += 4;
                    if (cp < 0x80) out->push_back((char)cp);
                    else if (cp < 0x800) { out->push_back((char)(0xC0 | (cp >> 6))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                    else { out->push_back((char)(0xE0 | (cp >> 12))); out->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                    break;
                }
                default: return fail(err, "bad escape");
            }
        }
        if (i_ >= s_.size()) return fail(err, "unterminated string");
        ++i_;
        return true;
    }
    bool value(Value* out, std::string* err) {
        if (i_ >= s_.size()) return fail(err, "unexpected end");
        char c = s_[i_];
        if (c == '{') {
            ++i_;
            *out = Value::make_object();
            skip();
            if (i_ < s_.size() && s_[i_] == '}') { ++i_; return true; }
            for (;;) {
                skip();
                std::string key;
                if (i_ >= s_.size() || !string(&key, err)) return fail(err, "expected object key");
                skip();
                if (i_ >= s_.size() || s_[i_] != ':') return fail(err, "expected ':'");
                ++i_;
                skip();
                Value v;
                if (!value(&v, err)) return false;
                out->obj->emplace_back(std::move(key), std::move(v));
                skip();
                if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
                if (i_ < s_.size() && s_[i_] == '}') { ++i_; return true; }
                return fail(err, "expected ',' or '}'");
            }
        }
        if (c == '[') {
            ++i_;
            *out = Value::make_array();
            skip();
            if (i_ < s_.size() && s_[i_] == ']') { ++i_; return true; }
            for (;;) {
                skip();
                Value v;
                if (!value(&v, err)) return false;
                out->arr->push_back(std::move(v));
                skip();
                if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
                if (i_ < s_.size() && s_[i_] == ']') { ++i_; return true; }
                return fail(err, "expected ',' or ']'");
            }
        }
        if (c == '"') {
            out->kind = Value::String;
            return string(&out->str, err);
        }
        if (literal("true")) { *out = Value::make_bool(true); return true; }
        if (literal("false")) { *out = Value::make_bool(false); return true; }
        if (literal("null")) { *out = Value(); return true; }
        char* end = nullptr;
        double d = strtod(s_.c_str() + i_, &end);
        if (end == s_.c_str() + i_) return fail(err, "unexpected character");
        i_ = (size_t)(end - s_.c_str());
        *out = Value::make_number(d);
        return true;
    }
};

inline void write_string(const std::string& s, std::string* out) {
    out->push_back('"');
    for (char c : s) {
        switch (c) {
            case '"': *out += "\\\""; break;
            case '\\': *out += "\\\\"; break;
            case '\n': *out += "\\n"; break;
            case '\r': *out += "\\r"; break;
            case '\t': *out += "\\t"; break;
            default:
                if ((unsigned char)c < 0x20) { char buf[8]; snprintf(buf, sizeof buf, "\\u%04x", c); *out += buf; }
                else out->push_back(c);
        }
    }
    out->push_back('"');
}

inline void write(const Value& v, std::string* out) {
    switch (v.kind) {
        case Value::Null: *out += "null"; break;
        case Value::Bool: *out += v.b ? "true" : "false"; break;
        case Value::Number: {
            char buf[40];
            if (v.num == std::floor(v.num) && std::fabs(v.num) < 1e15) snprintf(buf, sizeof buf, "%lld", (long long)v.num);
            else snprintf(buf, sizeof buf, "%.17g", v.num);
            *out += buf;
            break;
        }
        case Value::String: write_string(v.str, out); break;
        case Value::Arr: {
            out->push_back('[');
            bool first = true;
            for (const auto& e : *v.arr) { if (!first) out->push_back(','); first = false; write(e, out); }
            out->push_back(']');
            break;
        }
        case Value::Obj: {
            out->push_back('{');
            bool first = true;
            for (const auto& kv : *v.obj) { if (!first) out->push_back(','); first = false; write_string(kv.first, out); out->push_back(':'); write(kv.second, out); }
            out->push_back('}');
            break;
        }
    }
}

}  // namespace mjson
