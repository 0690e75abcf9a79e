// Minimal TOML reader for the generator -> runner contract: one flat table of integers, booleans,
// basic strings and (possibly multi-line, possibly trailing-comma) arrays of integers.  The reference
// reads the same file with a vendored general-purpose TOML library (runner/generator_runner.cpp:14,101);
// the runner only ever needs these four value kinds, so this reader accepts exactly them, skips
// comments, [table] headers and keys it does not know, and reports the line of anything it cannot parse.
#pragma once
#include <cctype>
#include <cstdint>
#include <cstdlib>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

namespace sgemm_toml {

struct Value {
    enum Kind { Int, Bool, String, IntArray } kind = Int;
    int64_t i = 0;
    bool b = false;
    std::string s;
    std::vector<int64_t> a;
};

struct Table {
    std::map<std::string, Value> values;
    bool get_int(const char *key, int64_t *out) const {
        auto it = values.find(key);
        if (it == values.end() || it->second.kind != Value::Int) return false;
        *out = it->second.i;
        return true;
    }
    bool get_bool(const char *key, bool *out) const {
        auto it = values.find(key);
        if (it == values.end() || it->second.kind != Value::Bool) return false;
        *out = it->second.b;
        return true;
    }
    bool get_string(const char *key, std::string *out) const {
        auto it = values.find(key);
        if (it == values.end() || it->second.kind != Value::String) return false;
        *out = it->second.s;
        return true;
    }
    bool get_int_array(const char *key, std::vector<int64_t> *out) const {
        auto it = values.find(key);
        if (it == values.end() || it->second.kind != Value::IntArray) return false;
        *out = it->second.a;
        return true;
    }
};

namespace detail {

struct Cursor {
    const std::string &text;
    size_t pos = 0;
    int line = 1;
    explicit Cursor(const std::string &t) : text(t) {}
    bool done() const { return pos >= text.size(); }
    char peek() const { return done() ? '\0' : text[pos]; }
    char take() {
        const char c = text[pos++];
        if (c == '\n') ++line;
        return c;
    }
    // skip blanks; with `newlines` also line breaks and comments (inside arrays, between statements)
    void skip(bool newlines) {
        while (!done()) {
            const char c = peek();
            if (c == ' ' || c == '\t' || c == '\r') take();
            else if (newlines && c == '\n') take();
            else if (c == '#') { while (!done() && peek() != '\n') take(); if (!newlines) return; }
            else return;
        }
    }
};

inline bool parse_int(Cursor &c, int64_t *out) {
    std::string digits;
    if (c.peek() == '+' || c.peek() == '-') digits += c.take();
    while (std::isdigit((unsigned char)c.peek()) || c.peek() == '_') {
        const char ch = c.take();
        if (ch != '_') digits += ch;
    }
    if (digits.empty() || digits == "+" || digits == "-") return false;
    *out = std::strtoll(digits.c_str(), nullptr, 10);
    return true;
}

inline bool parse_string(Cursor &c, std::string *out) {
    const char quote = c.take();  // " or '
    out->clear();
    while (!c.done() && c.peek() != quote) {
        char ch = c.take();
        if (ch == '\n') return false;
        if (ch == '\\' && quote == '"' && !c.done()) {
            const char e = c.take();
            ch = e == 'n' ? '\n' : e == 't' ? '\t' : e;
        }
        out->push_back(ch);
    }
    if (c.done()) return false;
    c.take();
    return true;
}

}  // namespace detail

inline bool parse_text(const std::string &text, Table *table, std::string *error) {
    detail::Cursor c(text);
    auto bad = [&](const std::string &what) {
        *error = "TOML line " + std::to_string(c.line) + ": " + what;
        return false;
    };
    for (;;) {
        c.skip(true);
        if (c.done()) return true;
        if (c.peek() == '[') {  // table header: the contract is flat, keys of sub-tables are ignored by name
            while (!c.done() && c.peek() != '\n') c.take();
            continue;
        }
        std::string key;
        if (c.peek() == '"' || c.peek() == '\'') {
            if (!detail::parse_string(c, &key)) return bad("unterminated quoted key");
        } else {
            while (std::isalnum((unsigned char)c.peek()) || c.peek() == '_' || c.peek() == '-' || c.peek() == '.') key += c.take();
        }
        if (key.empty()) return bad("expected a key");
        c.skip(false);
        if (c.peek() != '=') return bad("expected '=' after key '" + key + "'");
        c.take();
        c.skip(false);
        Value v;
        const char p = c.peek();
        if (p == '"' || p == '\'') {
            v.kind = Value::String;
            if (!detail::parse_string(c, &v.s)) return bad("unterminated string for key '" + key + "'");
        } else if (p == '[') {
            v.kind = Value::IntArray;
            c.take();
            for (;;) {
                c.skip(true);
                if (c.peek() == ']') { c.take(); break; }
                int64_t x;
                if (!detail::parse_int(c, &x)) return bad("array '" + key + "' may hold integers only");
                v.a.push_back(x);
                c.skip(true);
                if (c.peek() == ',') { c.take(); continue; }
                if (c.peek() == ']') { c.take(); break; }
                return bad("expected ',' or ']' in array '" + key + "'");
            }
        } else if (text.compare(c.pos, 4, "true") == 0) {
            v.kind = Value::Bool; v.b = true; c.pos += 4;
        } else if (text.compare(c.pos, 5, "false") == 0) {
            v.kind = Value::Bool; v.b = false; c.pos += 5;
        } else {
            v.kind = Value::Int;
            if (!detail::parse_int(c, &v.i)) return bad("unsupported value for key '" + key + "'");
            if (c.peek() == '.' || c.peek() == 'e' || c.peek() == 'E') return bad("floating-point value for key '" + key + "' is not part of the contract");
        }
        c.skip(false);
        if (!c.done() && c.peek() != '\n') return bad("trailing characters after the value of '" + key + "'");
        table->values[key] = v;
    }
}

inline bool parse_file(const char *path, Table *table, std::string *error) {
    std::ifstream f(path, std::ios::binary);
    if (!f) {
        *error = std::string("cannot open '") + path + "'";
        return false;
    }
    std::stringstream ss;
    ss << f.rdbuf();
    return parse_text(ss.str(), table, error);
}

}  // namespace sgemm_toml
