// A small JSON reader for the records the training data and checkpoint files carry
// (packed.json, binding.json, a checkpoint's manifest): objects keep their members in file order,
// numbers keep their text so that a u64 is read without passing through a double.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace msx {
namespace json {

struct Value {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool boolean = false;
    std::string text;  // a string's characters, or a number as written
    std::vector<Value> items;
    std::vector<std::pair<std::string, Value>> members;

    const Value* get(const std::string& key) const {
        if (kind != Object) return nullptr;
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
    const Value& at(const std::string& key) const {
        const Value* v = get(key);
        if (!v) throw std::runtime_error("missing field `" + key + "`");
        return *v;
    }
    const std::string& str() const {
        if (kind != String) throw std::runtime_error("expected a string");
        return text;
    }
    uint64_t u64() const {
        if (kind != Number || text.empty() || text.find_first_not_of("0123456789") != std::string::npos || text.size() > 20)
            throw std::runtime_error("expected an unsigned integer");
        unsigned long long value = 0;
        for (char c : text) {
            unsigned long long next = value * 10 + static_cast<unsigned>(c - '0');
            if (next / 10 != value) throw std::runtime_error("integer out of range");
            value = next;
        }
        return value;
    }
    double f64() const {
        if (kind != Number) throw std::runtime_error("expected a number");
        return std::strtod(text.c_str(), nullptr);
    }
};

class Reader {
  public:
    explicit Reader(const std::string& text) : s(text) {}
    Value document() {
        Value v = value(0);
        skip();
        if (i != s.size()) fail("trailing characters");
        return v;
    }

  private:
    const std::string& s;
    size_t i = 0;

    [[noreturn]] void fail(const std::string& why) const {
        throw std::runtime_error(why + " at byte " + std::to_string(i));
    }
    void skip() {
        while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
    }
    bool take(char c) {
        skip();
        if (i < s.size() && s[i] == c) {
            ++i;
            return true;
        }
        return false;
    }
    void expect(const char* word) {
        for (const char* p = word; *p; ++p, ++i)
            if (i >= s.size() || s[i] != *p) fail(std::string("expected `") + word + "`");
    }
    static void utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) out += static_cast<char>(cp);
        else if (cp < 0x800) {
            out += static_cast<char>(0xC0 | (cp >> 6));
            out += static_cast<char>(0x80 | (cp & 0x3F));
        } else if (cp < 0x10000) {
            out += static_cast<char>(0xE0 | (cp >> 12));
            out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
            out += static_cast<char>(0x80 | (cp & 0x3F));
        } else {
            out += static_cast<char>(0xF0 | (cp >> 18));
            out += static_cast<char>(0x80 | ((cp >> 12) & 0x3F));
            out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
            out += static_cast<char>(0x80 | (cp & 0x3F));
        }
    }
    uint32_t hex4() {
        if (i + 4 > s.size()) fail("short \\u escape");
        uint32_t v = 0;
        for (int k = 0; k < 4; ++k, ++i) {
            char c = s[i];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= static_cast<uint32_t>(c - '0');
            else if (c >= 'a' && c <= 'f') v |= static_cast<uint32_t>(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= static_cast<uint32_t>(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        std::string out;
        for (;;) {
            if (i >= s.size()) fail("unterminated string");
            char c = s[i++];
            if (c == '"') return out;
            if (static_cast<unsigned char>(c) < 0x20) fail("control character in a string");
            if (c != '\\') {
                out += c;
                continue;
            }
            if (i >= s.size()) fail("unterminated escape");
            char e = s[i++];
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
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && i + 1 < s.size() && s[i] == '\\' && s[i + 1] == 'u') {
                        i += 2;
                        uint32_t low = hex4();
                        if (low < 0xDC00 || low > 0xDFFF) fail("bad surrogate pair");
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (low - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: fail("bad escape");
            }
        }
    }
    Value value(int depth) {
        if (depth > 64) fail("nested too deeply");
        skip();
        if (i >= s.size()) fail("unexpected end");
        Value v;
        char c = s[i];
        if (c == '{') {
            ++i;
            v.kind = Value::Object;
            if (take('}')) return v;
            do {
                skip();
                if (i >= s.size() || s[i] != '"') fail("expected a member name");
                ++i;
                std::string key = string();
                if (!take(':')) fail("expected `:`");
                v.members.emplace_back(std::move(key), value(depth + 1));
            } while (take(','));
            if (!take('}')) fail("expected `}`");
        } else if (c == '[') {
            ++i;
            v.kind = Value::Array;
            if (take(']')) return v;
            do v.items.push_back(value(depth + 1));
            while (take(','));
            if (!take(']')) fail("expected `]`");
        } else if (c == '"') {
            ++i;
            v.kind = Value::String;
            v.text = string();
        } else if (c == 't') {
            expect("true");
            v.kind = Value::Bool;
            v.boolean = true;
        } else if (c == 'f') {
            expect("false");
            v.kind = Value::Bool;
        } else if (c == 'n') {
            expect("null");
        } else {
            size_t start = i;
            if (s[i] == '-') ++i;
            while (i < s.size() && ((s[i] >= '0' && s[i] <= '9') || s[i] == '.' || s[i] == 'e' || s[i] == 'E' || s[i] == '+' || s[i] == '-')) ++i;
            if (i == start) fail("unexpected character");
            v.kind = Value::Number;
            v.text = s.substr(start, i - start);
        }
        return v;
    }
};

inline Value parse(const std::string& text) { return Reader(text).document(); }

// A string as JSON writes it (serde_json's escapes: the two-character forms, \u00XX for the other
// control characters, everything else as it is).
inline std::string quoted(const std::string& text) {
    std::string out = "\"";
    for (char ch : text) {
        unsigned char c = static_cast<unsigned char>(ch);
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\b': out += "\\b"; break;
            case '\f': out += "\\f"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (c < 0x20) {
                    const char* hex = "0123456789abcdef";
                    out += "\\u00";
                    out += hex[c >> 4];
                    out += hex[c & 15];
                } else {
                    out += ch;
                }
        }
    }
    return out + "\"";
}

// A finite f64 as serde_json writes it (the ryu crate's layout of the shortest digits that read
// back to the same f64): plain decimals while the decimal point stays within 16 digits of the
// first one or at most five zeros follow "0.", exponent form otherwise; an integer keeps ".0".
inline std::string f64_text(double v) {
    if (v == 0.0) return std::signbit(v) ? "-0.0" : "0.0";
    std::string sign = v < 0 ? "-" : "";
    double a = std::fabs(v);
    char buf[64];
    for (int prec = 0; prec < 17; ++prec) {
        std::snprintf(buf, sizeof buf, "%.*e", prec, a);
        if (std::strtod(buf, nullptr) == a) break;
    }
    std::string s(buf);
    size_t e = s.find('e');
    int kk = std::atoi(s.c_str() + e + 1) + 1;  // a = 0.d1d2...dn x 10^kk
    std::string digits;
    for (char c : s.substr(0, e))
        if (c >= '0' && c <= '9') digits.push_back(c);
    while (digits.size() > 1 && digits.back() == '0') digits.pop_back();
    int n = static_cast<int>(digits.size()), k = kk - n;
    if (k >= 0 && kk <= 16) return sign + digits + std::string(static_cast<size_t>(k), '0') + ".0";
    if (kk > 0 && kk <= 16) return sign + digits.substr(0, static_cast<size_t>(kk)) + "." + digits.substr(static_cast<size_t>(kk));
    if (kk > -5 && kk <= 0) return sign + "0." + std::string(static_cast<size_t>(-kk), '0') + digits;
    std::string out = sign + digits.substr(0, 1);
    if (n > 1) out += "." + digits.substr(1);
    return out + "e" + std::to_string(kk - 1);
}

}  // namespace json
}  // namespace msx
