// Minimal JSON reader for Hugging Face tokenizer.json files.
//
// Builds a small DOM (objects keep their members in file order), decodes
// string escapes including \uXXXX surrogate pairs into UTF-8, and reports
// errors by returning false rather than throwing.  Numbers are kept as double
// plus an exact int64 when the literal is an integer.  Nothing here is specific
// to tokenizers; the loader in vocab.cc interprets the tree.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace gtok {
namespace json {

struct Value;
using Member = std::pair<std::string, Value>;

struct Value {
    enum Kind : uint8_t { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    bool is_int = false;
    double num = 0.0;
    int64_t inum = 0;
    std::string str;
    std::vector<Value> arr;
    std::vector<Member> obj;

    bool is_null() const { return kind == Null; }
    bool is_bool() const { return kind == Bool; }
    bool is_string() const { return kind == String; }
    bool is_array() const { return kind == Array; }
    bool is_object() const { return kind == Object; }
    bool is_number() const { return kind == Number; }

    // Member lookup; nullptr when this is not an object or the key is absent.
    // The last occurrence wins, as in most JSON readers.
    const Value* find(const char* key) const {
        if (kind != Object) return nullptr;
        const Value* hit = nullptr;
        for (const Member& m : obj)
            if (m.first == key) hit = &m.second;
        return hit;
    }
};

class Parser {
public:
    Parser(const char* data, size_t len) : p_(data), end_(data + len) {}

    bool parse(Value& out, std::string& err) {
        skip_ws();
        if (!value(out, 0)) { err = err_; return false; }
        skip_ws();
        if (p_ != end_) { err = "trailing characters after JSON value"; return false; }
        return true;
    }

private:
    const char* p_;
    const char* end_;
    std::string err_;
    static constexpr int kMaxDepth = 64;

    bool fail(const char* msg) { if (err_.empty()) err_ = msg; return false; }

    void skip_ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
    }

    bool literal(const char* word) {
        size_t n = std::strlen(word);
        if (static_cast<size_t>(end_ - p_) < n || std::memcmp(p_, word, n) != 0)
            return fail("bad literal");
        p_ += n;
        return true;
    }

    static void put_utf8(std::string& s, uint32_t cp) {
        if (cp < 0x80) {
            s.push_back(static_cast<char>(cp));
        } else if (cp < 0x800) {
            s.push_back(static_cast<char>(0xC0 | (cp >> 6)));
            s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else if (cp < 0x10000) {
            s.push_back(static_cast<char>(0xE0 | (cp >> 12)));
            s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else {
            s.push_back(static_cast<char>(0xF0 | (cp >> 18)));
            s.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
            s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        }
    }

    bool hex4(uint32_t& v) {
        if (end_ - p_ < 4) return fail("short \\u escape");
        v = 0;
        for (int i = 0; i < 4; ++i) {
            char c = *p_++;
            uint32_t d;
            if (c >= '0' && c <= '9') d = c - '0';
            else if (c >= 'a' && c <= 'f') d = 10 + c - 'a';
            else if (c >= 'A' && c <= 'F') d = 10 + c - 'A';
            else return fail("bad hex digit in \\u escape");
            v = (v << 4) | d;
        }
        return true;
    }

    bool string(std::string& out) {
        if (p_ >= end_ || *p_ != '"') return fail("expected string");
        ++p_;
        out.clear();
        for (;;) {
            // Copy the run of plain bytes in one go.
            const char* q = p_;
            while (q < end_ && *q != '"' && *q != '\\' && static_cast<unsigned char>(*q) >= 0x20) ++q;
            out.append(p_, q);
            p_ = q;
            if (p_ >= end_) return fail("unterminated string");
            char c = *p_++;
            if (c == '"') return true;
            if (c != '\\') return fail("control character in string");
            if (p_ >= end_) return fail("unterminated escape");
            char e = *p_++;
            switch (e) {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'n': out.push_back('\n'); break;
                case 'r': out.push_back('\r'); break;
                case 't': out.push_back('\t'); break;
                case 'u': {
                    uint32_t cp;
                    if (!hex4(cp)) return false;
                    if (cp >= 0xD800 && cp <= 0xDBFF && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        const char* save = p_;
                        p_ += 2;
                        uint32_t lo;
                        if (!hex4(lo)) return false;
                        if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        else p_ = save;
                    }
                    put_utf8(out, cp);
                    break;
                }
                default: return fail("unknown escape");
            }
        }
    }

    bool number(Value& out) {
        const char* s = p_;
        bool integral = true;
        if (p_ < end_ && *p_ == '-') ++p_;
        while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        if (p_ < end_ && *p_ == '.') { integral = false; ++p_; while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_; }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false; ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ == s || (p_ == s + 1 && *s == '-')) return fail("bad number");
        std::string tmp(s, p_);
        out.kind = Value::Number;
        out.num = std::strtod(tmp.c_str(), nullptr);
        out.is_int = integral && tmp.size() < 19;
        out.inum = out.is_int ? std::strtoll(tmp.c_str(), nullptr, 10) : static_cast<int64_t>(out.num);
        return true;
    }

    bool value(Value& out, int depth) {
        if (depth > kMaxDepth) return fail("nesting too deep");
        if (p_ >= end_) return fail("unexpected end of input");
        switch (*p_) {
            case 'n': out.kind = Value::Null; return literal("null");
            case 't': out.kind = Value::Bool; out.b = true; return literal("true");
            case 'f': out.kind = Value::Bool; out.b = false; return literal("false");
            case '"': out.kind = Value::String; return string(out.str);
            case '[': {
                ++p_;
                out.kind = Value::Array;
                skip_ws();
                if (p_ < end_ && *p_ == ']') { ++p_; return true; }
                for (;;) {
                    out.arr.emplace_back();
                    skip_ws();
                    if (!value(out.arr.back(), depth + 1)) return false;
                    skip_ws();
                    if (p_ >= end_) return fail("unterminated array");
                    if (*p_ == ',') { ++p_; continue; }
                    if (*p_ == ']') { ++p_; return true; }
                    return fail("expected , or ] in array");
                }
            }
            case '{': {
                ++p_;
                out.kind = Value::Object;
                skip_ws();
                if (p_ < end_ && *p_ == '}') { ++p_; return true; }
                for (;;) {
                    skip_ws();
                    out.obj.emplace_back();
                    if (!string(out.obj.back().first)) return false;
                    skip_ws();
                    if (p_ >= end_ || *p_ != ':') return fail("expected : in object");
                    ++p_;
                    skip_ws();
                    if (!value(out.obj.back().second, depth + 1)) return false;
                    skip_ws();
                    if (p_ >= end_) return fail("unterminated object");
                    if (*p_ == ',') { ++p_; continue; }
                    if (*p_ == '}') { ++p_; return true; }
                    return fail("expected , or } in object");
                }
            }
            default: return number(out);
        }
    }
};

}  // namespace json
}  // namespace gtok
