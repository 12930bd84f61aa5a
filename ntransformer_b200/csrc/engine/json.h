// json.h — a small JSON reader (objects, arrays, strings, numbers, true/false/null) for model folders' config.json,
// safetensors headers and the trace replayer's step lines.  Header only; values are immutable trees.
#pragma once
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace nt { namespace b200 {

class Json {
public:
    enum Kind { Null, Bool, Number, String, Array, Object };
    Kind kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;     // insertion order kept

    bool is_null() const { return kind == Null; }
    bool is_object() const { return kind == Object; }
    bool is_array() const { return kind == Array; }
    bool is_number() const { return kind == Number; }
    bool is_string() const { return kind == String; }
    const Json* find(const std::string& key) const {
        if (kind != Object) return nullptr;
        for (const auto& kv : obj) if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool has(const std::string& key) const { const Json* j = find(key); return j && !j->is_null(); }
    const Json& at(const std::string& key) const { static const Json none; const Json* j = find(key); return j ? *j : none; }
    double number_or(double d) const { return kind == Number ? num : d; }
    long long int_or(long long d) const { return kind == Number ? (long long)num : d; }
    const std::string& string_or(const std::string& d) const { return kind == String ? str : d; }

    // Parses one value from text[0..n); false on malformed input (err says where).
    static bool parse(const char* text, size_t n, Json& out, std::string* err = nullptr) {
        P p{text, text + n};
        if (!p.value(out, 0)) { if (err) *err = "JSON: malformed input near byte " + std::to_string(p.s - text); return false; }
        p.ws();
        if (p.s != p.e) { if (err) *err = "JSON: trailing bytes after the value"; return false; }
        return true;
    }
    static bool parse(const std::string& text, Json& out, std::string* err = nullptr) { return parse(text.data(), text.size(), out, err); }

private:
    struct P {
        const char* s; const char* e;
        void ws() { while (s < e && (*s == ' ' || *s == '\n' || *s == '\t' || *s == '\r')) s++; }
        bool lit(const char* w) { size_t n = strlen(w); if ((size_t)(e - s) < n || memcmp(s, w, n) != 0) return false; s += n; return true; }
        static void utf8(std::string& o, unsigned cp) {
            if (cp < 0x80) o += (char)cp;
            else if (cp < 0x800) { o += (char)(0xC0 | (cp >> 6)); o += (char)(0x80 | (cp & 63)); }
            else if (cp < 0x10000) { o += (char)(0xE0 | (cp >> 12)); o += (char)(0x80 | ((cp >> 6) & 63)); o += (char)(0x80 | (cp & 63)); }
            else { o += (char)(0xF0 | (cp >> 18)); o += (char)(0x80 | ((cp >> 12) & 63)); o += (char)(0x80 | ((cp >> 6) & 63)); o += (char)(0x80 | (cp & 63)); }
        }
        bool hex4(unsigned& v) {
            if (e - s < 4) return false;
            v = 0;
            for (int i = 0; i < 4; i++) {
                char c = *s++; v <<= 4;
                if (c >= '0' && c <= '9') v |= (unsigned)(c - '0'); else if (c >= 'a' && c <= 'f') v |= (unsigned)(c - 'a' + 10);
                else if (c >= 'A' && c <= 'F') v |= (unsigned)(c - 'A' + 10); else return false;
            }
            return true;
        }
        bool string(std::string& o) {
            if (s >= e || *s != '"') return false;
            s++;
            while (s < e && *s != '"') {
                if (*s == '\\') {
                    if (++s >= e) return false;
                    char c = *s++;
                    switch (c) {
                        case 'n': o += '\n'; break; case 't': o += '\t'; break; case 'r': o += '\r'; break;
                        case 'b': o += '\b'; break; case 'f': o += '\f'; break;
                        case 'u': {
                            unsigned cp; if (!hex4(cp)) return false;
                            if (cp >= 0xD800 && cp < 0xDC00 && e - s >= 6 && s[0] == '\\' && s[1] == 'u') {
                                s += 2; unsigned lo; if (!hex4(lo)) return false;
                                cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                            }
                            utf8(o, cp); break;
                        }
                        default: o += c;
                    }
                } else o += *s++;
            }
            if (s >= e) return false;
            s++;
            return true;
        }
        bool value(Json& o, int depth) {
            if (depth > 64) return false;
            ws();
            if (s >= e) return false;
            if (*s == '{') {
                s++; o.kind = Object; ws();
                if (s < e && *s == '}') { s++; return true; }
                for (;;) {
                    ws();
                    std::string k;
                    if (!string(k)) return false;
                    ws();
                    if (s >= e || *s++ != ':') return false;
                    o.obj.emplace_back(std::move(k), Json());
                    if (!value(o.obj.back().second, depth + 1)) return false;
                    ws();
                    if (s < e && *s == ',') { s++; continue; }
                    if (s < e && *s == '}') { s++; return true; }
                    return false;
                }
            }
            if (*s == '[') {
                s++; o.kind = Array; ws();
                if (s < e && *s == ']') { s++; return true; }
                for (;;) {
                    o.arr.emplace_back();
                    if (!value(o.arr.back(), depth + 1)) return false;
                    ws();
                    if (s < e && *s == ',') { s++; continue; }
                    if (s < e && *s == ']') { s++; return true; }
                    return false;
                }
            }
            if (*s == '"') { o.kind = String; return string(o.str); }
            if (lit("true")) { o.kind = Bool; o.b = true; return true; }
            if (lit("false")) { o.kind = Bool; o.b = false; return true; }
            if (lit("null")) { o.kind = Null; return true; }
            std::string t;
            while (s < e && (strchr("+-.eE", *s) || (*s >= '0' && *s <= '9'))) t += *s++;
            if (t.empty()) return false;
            char* end = nullptr;
            o.num = strtod(t.c_str(), &end);
            if (!end || *end) return false;
            o.kind = Number;
            return true;
        }
    };
};

}}  // namespace nt::b200
