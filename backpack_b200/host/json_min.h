// Minimal JSON reader for the harness's manifest files: objects, arrays, strings, numbers,
// true/false/null.  Stands in for the reference's runtime/json_parser.{h,cpp}.
#pragma once
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

namespace jsonmin {

struct Value {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    double num = 0;
    bool b = false;
    std::string str;
    std::vector<Value> arr;
    std::map<std::string, Value> obj;
    size_t size() const { return kind == Arr ? arr.size() : 0; }
    const Value& operator[](size_t i) const { return arr[i]; }
    const Value& operator[](const std::string& k) const {
        static const Value none;
        auto it = obj.find(k);
        return it == obj.end() ? none : it->second;
    }
};

struct Parser {
    const std::string& s;
    size_t i = 0;
    bool ok = true;
    void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) i++; }
    bool lit(const char* w) {
        size_t n = 0;
        while (w[n]) n++;
        if (s.compare(i, n, w) == 0) { i += n; return true; }
        return false;
    }
    std::string string() {
        std::string out;
        i++;  // opening quote
        while (i < s.size() && s[i] != '"') {
            if (s[i] == '\\' && i + 1 < s.size()) {
                const char c = s[++i];
                out += c == 'n' ? '\n' : c == 't' ? '\t' : c;
            } else out += s[i];
            i++;
        }
        if (i >= s.size()) ok = false;
        i++;
        return out;
    }
    Value value() {
        Value v;
        ws();
        if (i >= s.size()) { ok = false; return v; }
        const char c = s[i];
        if (c == '{') {
            v.kind = Value::Obj;
            i++;
            ws();
            if (i < s.size() && s[i] == '}') { i++; return v; }
            while (ok) {
                ws();
                if (i >= s.size() || s[i] != '"') { ok = false; break; }
                std::string k = string();
                ws();
                if (i >= s.size() || s[i] != ':') { ok = false; break; }
                i++;
                v.obj[k] = value();
                ws();
                if (i < s.size() && s[i] == ',') { i++; continue; }
                if (i < s.size() && s[i] == '}') { i++; break; }
                ok = false;
            }
        } else if (c == '[') {
            v.kind = Value::Arr;
            i++;
            ws();
            if (i < s.size() && s[i] == ']') { i++; return v; }
            while (ok) {
                v.arr.push_back(value());
                ws();
                if (i < s.size() && s[i] == ',') { i++; continue; }
                if (i < s.size() && s[i] == ']') { i++; break; }
                ok = false;
            }
        } else if (c == '"') {
            v.kind = Value::Str;
            v.str = string();
        } else if (lit("true")) { v.kind = Value::Bool; v.b = true; }
        else if (lit("false")) { v.kind = Value::Bool; }
        else if (lit("null")) {}
        else {
            char* end = nullptr;
            v.num = std::strtod(s.c_str() + i, &end);
            if (end == s.c_str() + i) ok = false;
            else { v.kind = Value::Num; i = (size_t)(end - s.c_str()); }
        }
        return v;
    }
};

inline bool parse(const std::string& text, Value& out) {
    Parser p{text};
    out = p.value();
    return p.ok;
}

}  // namespace jsonmin
