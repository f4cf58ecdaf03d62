// A small JSON value: parse, look up, write.  Objects keep the order of their keys (a dump of
// config.json prints them as the file has them).  Numbers remember whether they were written as
// integers, because configuration keys are typed (an integer key must not silently take 2.5).
//
// Role in the reference: the typed metadata values of a GGUF file (kv_t, fastgguf.c:262-270) and
// their readers kv_find / kv_num (fastgguf.c:442-454); a model folder carries the same numbers as
// JSON text, so the host needs a JSON reader of its own.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace fg {

struct JsonError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class Json {
public:
    enum Type { Null, Bool, Int, Float, String, Array, Object };
    using Member = std::pair<std::string, Json>;

    Json() : type_(Null) {}
    Json(std::nullptr_t) : type_(Null) {}
    Json(bool b) : type_(Bool), b_(b) {}
    Json(int v) : type_(Int), i_(v), d_((double)v) {}
    Json(long v) : type_(Int), i_(v), d_((double)v) {}
    Json(long long v) : type_(Int), i_(v), d_((double)v) {}
    Json(unsigned long long v) : type_(Int), i_((long long)v), d_((double)v) {}
    Json(double v) : type_(Float), i_((long long)v), d_(v) {}
    Json(const char *s) : type_(String), s_(s) {}
    Json(std::string s) : type_(String), s_(std::move(s)) {}

    static Json array() { Json j; j.type_ = Array; return j; }
    static Json object() { Json j; j.type_ = Object; return j; }

    Type type() const { return type_; }
    bool is_null() const { return type_ == Null; }
    bool is_bool() const { return type_ == Bool; }
    bool is_int() const { return type_ == Int; }
    bool is_number() const { return type_ == Int || type_ == Float; }
    bool is_string() const { return type_ == String; }
    bool is_array() const { return type_ == Array; }
    bool is_object() const { return type_ == Object; }
    const char *type_name() const {
        static const char *n[] = {"null", "bool", "int", "float", "str", "list", "dict"};
        return n[type_];
    }

    bool as_bool() const { return b_; }
    long long as_int() const { return i_; }
    double as_double() const { return d_; }
    const std::string &as_string() const { return s_; }
    const std::vector<Json> &items() const { return a_; }
    std::vector<Json> &items() { return a_; }
    const std::vector<Member> &members() const { return o_; }

    size_t size() const { return type_ == Array ? a_.size() : type_ == Object ? o_.size() : 0; }
    const Json &operator[](size_t i) const { return a_[i]; }

    // object access: a missing key reads as null
    const Json *find(const std::string &key) const {
        if (type_ != Object) return nullptr;
        for (auto &m : o_)
            if (m.first == key) return &m.second;
        return nullptr;
    }
    bool has(const std::string &key) const { return find(key) != nullptr; }
    const Json &get(const std::string &key) const {
        static const Json null_value;
        const Json *j = find(key);
        return j ? *j : null_value;
    }
    void set(const std::string &key, Json v) {
        if (type_ != Object) { *this = object(); }
        for (auto &m : o_)
            if (m.first == key) { m.second = std::move(v); return; }
        o_.emplace_back(key, std::move(v));
    }
    void push(Json v) {
        if (type_ != Array) { *this = array(); }
        a_.push_back(std::move(v));
    }

    bool operator==(const Json &o) const {
        if (is_number() && o.is_number()) return d_ == o.d_;
        if (type_ != o.type_) return false;
        switch (type_) {
        case Null: return true;
        case Bool: return b_ == o.b_;
        case String: return s_ == o.s_;
        case Array: return a_ == o.a_;
        case Object: return o_ == o.o_;
        default: return false;
        }
    }
    bool operator!=(const Json &o) const { return !(*this == o); }

    // ---------------------------------------------------------------- text
    static Json parse(const std::string &text) {
        Parser p{text.data(), text.data() + text.size(), text.data()};
        Json v = p.value(0);
        p.skip();
        if (p.cur != p.end) p.fail("text after the document's end");
        return v;
    }

    std::string dump(int indent = -1) const {
        std::string out;
        write(out, indent, 0);
        return out;
    }

private:
    Type type_;
    bool b_ = false;
    long long i_ = 0;
    double d_ = 0.0;
    std::string s_;
    std::vector<Json> a_;
    std::vector<Member> o_;

    struct Parser {
        const char *begin, *end, *cur;
        [[noreturn]] void fail(const char *what) const {
            int line = 1, col = 1;
            for (const char *p = begin; p < cur; p++) {
                if (*p == '\n') { line++; col = 1; } else col++;
            }
            char buf[200];
            snprintf(buf, sizeof buf, "%s: line %d column %d (char %ld)", what, line, col, (long)(cur - begin));
            throw JsonError(buf);
        }
        void skip() {
            while (cur < end && (*cur == ' ' || *cur == '\t' || *cur == '\n' || *cur == '\r')) cur++;
        }
        bool lit(const char *w) {
            size_t n = strlen(w);
            if ((size_t)(end - cur) >= n && memcmp(cur, w, n) == 0) { cur += n; return true; }
            return false;
        }
        Json value(int depth) {
            if (depth > 200) fail("nesting too deep");
            skip();
            if (cur == end) fail("expecting a value");
            char c = *cur;
            if (c == '{') return object_(depth);
            if (c == '[') return array_(depth);
            if (c == '"') return Json(string_());
            if (lit("true")) return Json(true);
            if (lit("false")) return Json(false);
            if (lit("null")) return Json();
            if (lit("NaN")) return Json(std::nan(""));
            if (lit("Infinity")) return Json(INFINITY);
            if (lit("-Infinity")) return Json(-INFINITY);
            if (c == '-' || (c >= '0' && c <= '9')) return number_();
            fail("expecting a value");
        }
        Json number_() {
            const char *s = cur;
            bool is_float = false;
            if (cur < end && *cur == '-') cur++;
            if (cur == end || *cur < '0' || *cur > '9') fail("bad number");
            while (cur < end && *cur >= '0' && *cur <= '9') cur++;
            if (cur < end && *cur == '.') {
                is_float = true;
                cur++;
                if (cur == end || *cur < '0' || *cur > '9') fail("bad number");
                while (cur < end && *cur >= '0' && *cur <= '9') cur++;
            }
            if (cur < end && (*cur == 'e' || *cur == 'E')) {
                is_float = true;
                cur++;
                if (cur < end && (*cur == '+' || *cur == '-')) cur++;
                if (cur == end || *cur < '0' || *cur > '9') fail("bad number");
                while (cur < end && *cur >= '0' && *cur <= '9') cur++;
            }
            std::string t(s, cur);
            if (!is_float) {
                errno = 0;
                long long v = strtoll(t.c_str(), nullptr, 10);
                if (errno == 0) return Json(v);
            }
            return Json(strtod(t.c_str(), nullptr));
        }
        static void utf8(std::string &out, unsigned cp) {
            if (cp < 0x80) out += (char)cp;
            else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
            else if (cp < 0x10000) {
                out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F));
            } else {
                out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F));
                out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F));
            }
        }
        unsigned hex4() {
            if (end - cur < 4) fail("bad \\u escape");
            unsigned v = 0;
            for (int i = 0; i < 4; i++) {
                char c = *cur++;
                v <<= 4;
                if (c >= '0' && c <= '9') v |= c - '0';
                else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
                else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
                else fail("bad \\u escape");
            }
            return v;
        }
        std::string string_() {
            cur++;                         // the opening quote
            std::string out;
            while (true) {
                if (cur == end) fail("unterminated string");
                unsigned char c = (unsigned char)*cur++;
                if (c == '"') return out;
                if (c < 0x20) { cur--; fail("control character in a string"); }
                if (c != '\\') { out += (char)c; continue; }
                if (cur == end) fail("unterminated string");
                char e = *cur++;
                switch (e) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    unsigned cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && end - cur >= 6 && cur[0] == '\\' && cur[1] == 'u') {
                        cur += 2;
                        unsigned lo = hex4();
                        if (lo >= 0xDC00 && lo < 0xE000) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: cur--; fail("bad escape in a string");
                }
            }
        }
        Json array_(int depth) {
            cur++;
            Json a = Json::array();
            skip();
            if (cur < end && *cur == ']') { cur++; return a; }
            while (true) {
                a.a_.push_back(value(depth + 1));
                skip();
                if (cur == end) fail("unterminated list");
                if (*cur == ',') { cur++; continue; }
                if (*cur == ']') { cur++; return a; }
                fail("expecting ',' or ']'");
            }
        }
        Json object_(int depth) {
            cur++;
            Json o = Json::object();
            skip();
            if (cur < end && *cur == '}') { cur++; return o; }
            while (true) {
                skip();
                if (cur == end || *cur != '"') fail("expecting a key in double quotes");
                std::string k = string_();
                skip();
                if (cur == end || *cur != ':') fail("expecting ':'");
                cur++;
                Json v = value(depth + 1);
                o.set(k, std::move(v));
                skip();
                if (cur == end) fail("unterminated object");
                if (*cur == ',') { cur++; continue; }
                if (*cur == '}') { cur++; return o; }
                fail("expecting ',' or '}'");
            }
        }
    };

    static void write_string(std::string &out, const std::string &s) {
        out += '"';
        for (unsigned char c : s) {
            switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
                else out += (char)c;
            }
        }
        out += '"';
    }
    static void newline(std::string &out, int indent, int level) {
        if (indent < 0) return;
        out += '\n';
        out.append((size_t)indent * level, ' ');
    }
    void write(std::string &out, int indent, int level) const {
        char buf[64];
        switch (type_) {
        case Null: out += "null"; break;
        case Bool: out += b_ ? "true" : "false"; break;
        case Int: snprintf(buf, sizeof buf, "%lld", i_); out += buf; break;
        case Float:
            if (std::isnan(d_)) out += "NaN";
            else if (std::isinf(d_)) out += d_ > 0 ? "Infinity" : "-Infinity";
            else {
                // the shortest text that reads back as the same double; always marked as a float
                for (int prec = 1; prec <= 17; prec++) {
                    snprintf(buf, sizeof buf, "%.*g", prec, d_);
                    if (strtod(buf, nullptr) == d_) break;
                }
                out += buf;
                if (!strpbrk(buf, ".eEn")) out += ".0";
            }
            break;
        case String: write_string(out, s_); break;
        case Array:
            out += '[';
            for (size_t i = 0; i < a_.size(); i++) {
                if (i) out += indent < 0 ? ", " : ",";
                newline(out, indent, level + 1);
                a_[i].write(out, indent, level + 1);
            }
            if (!a_.empty()) newline(out, indent, level);
            out += ']';
            break;
        case Object:
            out += '{';
            for (size_t i = 0; i < o_.size(); i++) {
                if (i) out += indent < 0 ? ", " : ",";
                newline(out, indent, level + 1);
                write_string(out, o_[i].first);
                out += ": ";
                o_[i].second.write(out, indent, level + 1);
            }
            if (!o_.empty()) newline(out, indent, level);
            out += '}';
            break;
        }
    }
};

}  // namespace fg
