#include "json.h"

#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace jb {

static const Json kNull;

bool Json::has(const std::string &k) const {
    for (auto &m : o_) if (m.first == k) return true;
    return false;
}

const Json &Json::get(const std::string &k) const {
    for (auto &m : o_) if (m.first == k) return m.second;
    return kNull;
}

Json &Json::set(const std::string &k, Json v) {
    if (type_ != Object) { *this = Json::object(); }
    for (auto &m : o_) if (m.first == k) { m.second = std::move(v); return m.second; }
    o_.emplace_back(k, std::move(v));
    return o_.back().second;
}

class JsonParser {
public:
    explicit JsonParser(const std::string &t) : s(t) {}

    Json run() {
        ws();
        Json v = value(0);
        ws();
        if (p != s.size()) fail("text after the value");
        return v;
    }

private:
    const std::string &s;
    size_t p = 0;

    [[noreturn]] void fail(const char *what) {
        throw JsonError(std::string(what) + " at byte " + std::to_string(p));
    }
    void ws() { while (p < s.size() && (s[p] == ' ' || s[p] == '\n' || s[p] == '\t' || s[p] == '\r')) p++; }
    bool lit(const char *w) {
        size_t n = strlen(w);
        if (s.compare(p, n, w) == 0) { p += n; return true; }
        return false;
    }

    Json value(int depth) {
        if (depth > 64) fail("nested too deep");
        if (p >= s.size()) fail("the text ends early");
        char c = s[p];
        if (c == '{') return object(depth);
        if (c == '[') return array(depth);
        if (c == '"') return Json(string());
        if (lit("true")) return Json(true);
        if (lit("false")) return Json(false);
        if (lit("null")) return Json();
        // Python's json writes these for floats that JSON has no word for
        if (lit("NaN")) return Json(std::nan(""));
        if (lit("Infinity")) return Json(HUGE_VAL);
        if (lit("-Infinity")) return Json(-HUGE_VAL);
        return number();
    }

    Json number() {
        size_t a = p;
        if (p < s.size() && (s[p] == '-' || s[p] == '+')) p++;
        bool digits = false, real = false;
        while (p < s.size()) {
            char c = s[p];
            if (c >= '0' && c <= '9') { digits = true; p++; }
            else if (c == '.' || c == 'e' || c == 'E' || ((c == '-' || c == '+') && p > a &&
                     (s[p - 1] == 'e' || s[p - 1] == 'E'))) { real = true; p++; }
            else break;
        }
        if (!digits) fail("a value is expected");
        std::string t = s.substr(a, p - a);
        if (!real) {
            errno = 0;
            char *end = nullptr;
            if (t[0] == '-') {
                long long v = strtoll(t.c_str(), &end, 10);
                if (errno == 0 && *end == 0) return Json(v);
            } else {
                unsigned long long v = strtoull(t.c_str(), &end, 10);
                if (errno == 0 && *end == 0) return Json(v);
            }
        }
        char *end = nullptr;
        double d = strtod(t.c_str(), &end);
        if (*end != 0) fail("a malformed number");
        return Json(d);
    }

    static void utf8(std::string &out, unsigned cp) {
        if (cp < 0x80) out += (char)cp;
        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) {
            out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F));
            out += (char)(0x80 | (cp & 0x3F));
        } else {
            out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F));
            out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F));
        }
    }

    unsigned hex4() {
        if (p + 4 > s.size()) fail("a short \\u escape");
        unsigned v = 0;
        for (int i = 0; i < 4; i++) {
            char c = s[p++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else fail("a malformed \\u escape");
        }
        return v;
    }

    std::string string() {
        p++;  // the quote
        std::string out;
        while (true) {
            if (p >= s.size()) fail("a string does not end");
            char c = s[p++];
            if (c == '"') return out;
            if (c != '\\') { out += c; continue; }
            if (p >= s.size()) fail("a string does not end");
            char e = s[p++];
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
                    if (cp >= 0xD800 && cp < 0xDC00 && p + 1 < s.size() && s[p] == '\\' && s[p + 1] == 'u') {
                        p += 2;
                        unsigned lo = hex4();
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: fail("an unknown escape");
            }
        }
    }

    Json array(int depth) {
        p++;
        Json a = Json::array();
        ws();
        if (p < s.size() && s[p] == ']') { p++; return a; }
        while (true) {
            ws();
            a.push(value(depth + 1));
            ws();
            if (p >= s.size()) fail("an array does not end");
            if (s[p] == ',') { p++; continue; }
            if (s[p] == ']') { p++; return a; }
            fail("',' or ']' is expected");
        }
    }

    Json object(int depth) {
        p++;
        Json o = Json::object();
        ws();
        if (p < s.size() && s[p] == '}') { p++; return o; }
        while (true) {
            ws();
            if (p >= s.size() || s[p] != '"') fail("a key is expected");
            std::string k = string();
            ws();
            if (p >= s.size() || s[p] != ':') fail("':' is expected");
            p++;
            ws();
            o.set(k, value(depth + 1));
            ws();
            if (p >= s.size()) fail("an object does not end");
            if (s[p] == ',') { p++; continue; }
            if (s[p] == '}') { p++; return o; }
            fail("',' or '}' is expected");
        }
    }
};

Json Json::parse(const std::string &text) { return JsonParser(text).run(); }

static void dump_string(std::string &out, const std::string &s) {
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

static void dump_value(std::string &out, const Json &j) {
    switch (j.type()) {
        case Json::Null: out += "null"; break;
        case Json::Bool: out += j.as_bool() ? "true" : "false"; break;
        case Json::Int: {
            char b[32];
            if (j.big())
                snprintf(b, sizeof b, "%llu", j.as_uint());
            else
                snprintf(b, sizeof b, "%lld", j.as_int());
            out += b;
            break;
        }
        case Json::Real: {
            double d = j.as_double();
            if (std::isnan(d)) out += "NaN";
            else if (std::isinf(d)) out += d > 0 ? "Infinity" : "-Infinity";
            else { char b[40]; snprintf(b, sizeof b, "%.17g", d); out += b;
                   if (!strpbrk(b, ".eE")) out += ".0"; }
            break;
        }
        case Json::String: dump_string(out, j.as_string()); break;
        case Json::Array: {
            out += '[';
            bool first = true;
            for (auto &v : j.items()) { if (!first) out += ','; first = false; dump_value(out, v); }
            out += ']';
            break;
        }
        case Json::Object: {
            out += '{';
            bool first = true;
            for (auto &m : j.members()) {
                if (!first) out += ',';
                first = false;
                dump_string(out, m.first);
                out += ':';
                dump_value(out, m.second);
            }
            out += '}';
            break;
        }
    }
}

std::string Json::dump() const {
    std::string out;
    dump_value(out, *this);
    return out;
}

}  // namespace jb
