// Minimal JSON reader for config.json and the safetensors header: objects, arrays, strings
// (with \uXXXX kept as raw bytes for the BMP), numbers, true/false/null.  No dependencies.
#pragma once
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace lumi {

struct JsonValue {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<JsonValue> arr;
    std::vector<std::pair<std::string, JsonValue>> obj;   // insertion order kept

    const JsonValue* find(const std::string& key) const {
        for (auto& kv : obj) if (kv.first == key) return &kv.second;
        return nullptr;
    }
};

class JsonParser {
public:
    JsonParser(const char* p, size_t n) : p_(p), end_(p + n) {}
    bool parse(JsonValue& out, std::string& err) {
        skip();
        if (!value(out, err, 0)) return false;
        skip();
        if (p_ != end_) { err = "trailing characters after JSON value"; return false; }
        return true;
    }

private:
    const char* p_;
    const char* end_;
    void skip() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_; }
    bool lit(const char* s) {
        const char* q = p_;
        while (*s) { if (q >= end_ || *q != *s) return false; ++q; ++s; }
        p_ = q;
        return true;
    }
    bool string(std::string& out, std::string& err) {
        if (p_ >= end_ || *p_ != '"') { err = "expected string"; return false; }
        ++p_;
        while (p_ < end_ && *p_ != '"') {
            char c = *p_++;
            if (c == '\\') {
                if (p_ >= end_) break;
                char e = *p_++;
                switch (e) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (end_ - p_ < 4) { err = "bad \\u escape"; return false; }
                        unsigned v = (unsigned)strtoul(std::string(p_, 4).c_str(), nullptr, 16);
                        p_ += 4;
                        if (v < 0x80) out += (char)v;
                        else if (v < 0x800) { out += (char)(0xC0 | (v >> 6)); out += (char)(0x80 | (v & 0x3F)); }
                        else { out += (char)(0xE0 | (v >> 12)); out += (char)(0x80 | ((v >> 6) & 0x3F)); out += (char)(0x80 | (v & 0x3F)); }
                        break;
                    }
                    default: out += e;
                }
            } else out += c;
        }
        if (p_ >= end_) { err = "unterminated string"; return false; }
        ++p_;
        return true;
    }
    bool value(JsonValue& v, std::string& err, int depth) {
        if (depth > 64) { err = "JSON nested too deeply"; return false; }
        skip();
        if (p_ >= end_) { err = "unexpected end of JSON"; return false; }
        char c = *p_;
        if (c == '{') {
            v.kind = JsonValue::Object;
            ++p_; skip();
            if (p_ < end_ && *p_ == '}') { ++p_; return true; }
            for (;;) {
                skip();
                std::string k;
                if (!string(k, err)) return false;
                skip();
                if (p_ >= end_ || *p_ != ':') { err = "expected ':'"; return false; }
                ++p_;
                JsonValue child;
                if (!value(child, err, depth + 1)) return false;
                v.obj.emplace_back(std::move(k), std::move(child));
                skip();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return true; }
                err = "expected ',' or '}'";
                return false;
            }
        }
        if (c == '[') {
            v.kind = JsonValue::Array;
            ++p_; skip();
            if (p_ < end_ && *p_ == ']') { ++p_; return true; }
            for (;;) {
                JsonValue child;
                if (!value(child, err, depth + 1)) return false;
                v.arr.push_back(std::move(child));
                skip();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return true; }
                err = "expected ',' or ']'";
                return false;
            }
        }
        if (c == '"') { v.kind = JsonValue::String; return string(v.str, err); }
        if (lit("true")) { v.kind = JsonValue::Bool; v.b = true; return true; }
        if (lit("false")) { v.kind = JsonValue::Bool; v.b = false; return true; }
        if (lit("null")) { v.kind = JsonValue::Null; return true; }
        {
            std::string tmp;
            const char* q = p_;
            while (q < end_ && (*q == '-' || *q == '+' || *q == '.' || *q == 'e' || *q == 'E' || (*q >= '0' && *q <= '9'))) ++q;
            if (q == p_) { err = "unexpected character in JSON"; return false; }
            tmp.assign(p_, q);
            char* endp = nullptr;
            v.num = strtod(tmp.c_str(), &endp);
            if (endp == tmp.c_str()) { err = "bad number"; return false; }
            v.kind = JsonValue::Number;
            p_ = q;
            return true;
        }
    }
};

}  // namespace lumi
