// A small JSON value with a parser and a writer: what config.json, the safetensors
// header and the model plans need (objects keep the order of their keys; numbers keep
// whether they were written as integers).  The reference carries its own JSON reader
// for the same reason (src/kipp_json.c): no dependency for a few hundred lines.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace kipp {

struct JsonError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class Json {
public:
    enum Kind { Null, Bool, Int, Real, String, Array, Object };

    Json() = default;
    Json(std::nullptr_t) {}
    Json(bool v) : kind_(Bool), b_(v) {}
    Json(int v) : kind_(Int), i_(v) {}
    Json(long v) : kind_(Int), i_(v) {}
    Json(long long v) : kind_(Int), i_(v) {}
    Json(unsigned long v) : kind_(Int), i_((long long)v) {}
    Json(double v) : kind_(Real), d_(v) {}
    Json(const char* s) : kind_(String), s_(s) {}
    Json(std::string s) : kind_(String), s_(std::move(s)) {}
    static Json array() { Json j; j.kind_ = Array; return j; }
    static Json object() { Json j; j.kind_ = Object; return j; }

    Kind kind() const { return kind_; }
    bool is_null() const { return kind_ == Null; }
    bool is_bool() const { return kind_ == Bool; }
    bool is_int() const { return kind_ == Int; }
    bool is_number() const { return kind_ == Int || kind_ == Real; }
    bool is_string() const { return kind_ == String; }
    bool is_array() const { return kind_ == Array; }
    bool is_object() const { return kind_ == Object; }

    bool as_bool() const { need(Bool, "a boolean"); return b_; }
    long long as_int() const {
        if (kind_ == Real && std::floor(d_) == d_ && std::fabs(d_) < 9e15) return (long long)d_;
        need(Int, "an integer");
        return i_;
    }
    double as_double() const {
        if (kind_ == Int) return (double)i_;
        need(Real, "a number");
        return d_;
    }
    const std::string& as_string() const { need(String, "a string"); return s_; }

    // arrays
    size_t size() const { return kind_ == Array ? a_.size() : kind_ == Object ? o_.size() : 0; }
    const Json& at(size_t i) const { need(Array, "an array"); return a_.at(i); }
    Json& push(Json v) { need(Array, "an array"); a_.push_back(std::move(v)); return a_.back(); }
    const std::vector<Json>& items() const { need(Array, "an array"); return a_; }

    // objects
    const std::vector<std::pair<std::string, Json>>& members() const { need(Object, "an object"); return o_; }
    const Json* find(const std::string& key) const {
        if (kind_ != Object) return nullptr;
        for (auto& kv : o_) if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool has(const std::string& key) const { return find(key) != nullptr; }
    const Json& get(const std::string& key) const {
        const Json* v = find(key);
        if (!v) throw JsonError("key '" + key + "' is missing");
        return *v;
    }
    Json& set(const std::string& key, Json v) {
        need(Object, "an object");
        for (auto& kv : o_) if (kv.first == key) { kv.second = std::move(v); return kv.second; }
        o_.emplace_back(key, std::move(v));
        return o_.back().second;
    }
    long long get_int(const std::string& key, long long fallback) const {
        const Json* v = find(key);
        return v && !v->is_null() ? v->as_int() : fallback;
    }
    double get_double(const std::string& key, double fallback) const {
        const Json* v = find(key);
        return v && !v->is_null() ? v->as_double() : fallback;
    }
    bool get_bool(const std::string& key, bool fallback) const {
        const Json* v = find(key);
        return v && !v->is_null() ? v->as_bool() : fallback;
    }
    std::string get_string(const std::string& key, const std::string& fallback) const {
        const Json* v = find(key);
        return v && !v->is_null() ? v->as_string() : fallback;
    }

    static Json parse(const char* text, size_t n) {
        Parser p{text, text + n};
        p.skip();
        Json v = p.value(0);
        p.skip();
        if (p.at != p.end) p.fail("text after the value");
        return v;
    }
    static Json parse(const std::string& text) { return parse(text.data(), text.size()); }

    std::string dump() const {
        std::string out;
        write(out);
        return out;
    }

private:
    Kind kind_ = Null;
    bool b_ = false;
    long long i_ = 0;
    double d_ = 0.0;
    std::string s_;
    std::vector<Json> a_;
    std::vector<std::pair<std::string, Json>> o_;

    void need(Kind k, const char* what) const {
        if (kind_ != k) throw JsonError(std::string("JSON value is not ") + what);
    }

    static void write_string(std::string& out, const std::string& s) {
        out.push_back('"');
        for (unsigned char c : s) {
            switch (c) {
                case '"': out += "\\\""; break;
                case '\\': out += "\\\\"; break;
                case '\n': out += "\\n"; break;
                case '\r': out += "\\r"; break;
                case '\t': out += "\\t"; break;
                default:
                    if (c < 0x20) {
                        char buf[8];
                        snprintf(buf, sizeof buf, "\\u%04x", c);
                        out += buf;
                    } else {
                        out.push_back((char)c);
                    }
            }
        }
        out.push_back('"');
    }

    void write(std::string& out) const {
        char buf[40];
        switch (kind_) {
            case Null: out += "null"; break;
            case Bool: out += b_ ? "true" : "false"; break;
            case Int: snprintf(buf, sizeof buf, "%lld", i_); out += buf; break;
            case Real:
                if (!std::isfinite(d_)) { out += "null"; break; }
                snprintf(buf, sizeof buf, "%.17g", d_);
                out += buf;
                if (!strpbrk(buf, ".eEn")) out += ".0";
                break;
            case String: write_string(out, s_); break;
            case Array:
                out.push_back('[');
                for (size_t i = 0; i < a_.size(); ++i) {
                    if (i) out += ", ";
                    a_[i].write(out);
                }
                out.push_back(']');
                break;
            case Object:
                out.push_back('{');
                for (size_t i = 0; i < o_.size(); ++i) {
                    if (i) out += ", ";
                    write_string(out, o_[i].first);
                    out += ": ";
                    o_[i].second.write(out);
                }
                out.push_back('}');
                break;
        }
    }

    struct Parser {
        const char* at;
        const char* end;
        const char* begin = at;

        [[noreturn]] void fail(const std::string& what) const {
            throw JsonError("not valid JSON at byte " + std::to_string(at - begin) + ": " + what);
        }
        void skip() {
            while (at != end && (*at == ' ' || *at == '\n' || *at == '\r' || *at == '\t')) ++at;
        }
        bool word(const char* w) {
            size_t n = strlen(w);
            if ((size_t)(end - at) >= n && memcmp(at, w, n) == 0) { at += n; return true; }
            return false;
        }
        static void utf8(std::string& out, unsigned cp) {
            if (cp < 0x80) out.push_back((char)cp);
            else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
            else if (cp < 0x10000) {
                out.push_back((char)(0xE0 | (cp >> 12)));
                out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
                out.push_back((char)(0x80 | (cp & 0x3F)));
            } else {
                out.push_back((char)(0xF0 | (cp >> 18)));
                out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
                out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
                out.push_back((char)(0x80 | (cp & 0x3F)));
            }
        }
        unsigned hex4() {
            if (end - at < 4) fail("short \\u escape");
            unsigned v = 0;
            for (int i = 0; i < 4; ++i) {
                char c = *at++;
                v <<= 4;
                if (c >= '0' && c <= '9') v |= (unsigned)(c - '0');
                else if (c >= 'a' && c <= 'f') v |= (unsigned)(c - 'a' + 10);
                else if (c >= 'A' && c <= 'F') v |= (unsigned)(c - 'A' + 10);
                else fail("bad \\u escape");
            }
            return v;
        }
        std::string string() {
            if (at == end || *at != '"') fail("a string was expected");
            ++at;
            std::string out;
            while (true) {
                if (at == end) fail("unterminated string");
                char c = *at++;
                if (c == '"') break;
                if (c != '\\') { out.push_back(c); continue; }
                if (at == end) fail("unterminated escape");
                char e = *at++;
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
                        unsigned cp = hex4();
                        if (cp >= 0xD800 && cp < 0xDC00 && end - at >= 6 && at[0] == '\\' && at[1] == 'u') {
                            at += 2;
                            unsigned lo = hex4();
                            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        }
                        utf8(out, cp);
                        break;
                    }
                    default: fail("unknown escape");
                }
            }
            return out;
        }
        Json number() {
            const char* start = at;
            bool real = false;
            if (at != end && (*at == '-' || *at == '+')) ++at;
            while (at != end && ((*at >= '0' && *at <= '9') || *at == '.' || *at == 'e' || *at == 'E' || *at == '-' ||
                                 *at == '+')) {
                if (*at == '.' || *at == 'e' || *at == 'E') real = true;
                ++at;
            }
            std::string text(start, at);
            if (text.empty() || text == "-") fail("a number was expected");
            char* stop = nullptr;
            if (!real) {
                errno = 0;
                long long v = strtoll(text.c_str(), &stop, 10);
                if (*stop == 0 && errno == 0) return Json(v);
            }
            double d = strtod(text.c_str(), &stop);
            if (*stop != 0) fail("bad number '" + text + "'");
            return Json(d);
        }
        Json value(int depth) {
            if (depth > 200) fail("nested too deeply");
            skip();
            if (at == end) fail("unexpected end");
            char c = *at;
            if (c == '{') {
                ++at;
                Json obj = Json::object();
                skip();
                if (at != end && *at == '}') { ++at; return obj; }
                while (true) {
                    skip();
                    std::string key = string();
                    skip();
                    if (at == end || *at != ':') fail("':' was expected");
                    ++at;
                    obj.set(key, value(depth + 1));
                    skip();
                    if (at != end && *at == ',') { ++at; continue; }
                    if (at != end && *at == '}') { ++at; return obj; }
                    fail("',' or '}' was expected");
                }
            }
            if (c == '[') {
                ++at;
                Json arr = Json::array();
                skip();
                if (at != end && *at == ']') { ++at; return arr; }
                while (true) {
                    arr.push(value(depth + 1));
                    skip();
                    if (at != end && *at == ',') { ++at; continue; }
                    if (at != end && *at == ']') { ++at; return arr; }
                    fail("',' or ']' was expected");
                }
            }
            if (c == '"') return Json(string());
            if (word("true")) return Json(true);
            if (word("false")) return Json(false);
            if (word("null")) return Json(nullptr);
            if (word("NaN")) return Json(std::nan(""));
            if (word("Infinity")) return Json(HUGE_VAL);
            if (word("-Infinity")) return Json(-HUGE_VAL);
            return number();
        }
    };
};

}  // namespace kipp
