// Minimal JSON reader for task_graph.json (objects, arrays, strings, numbers, true / false / null), enough to walk the
// document the reference writes (src/codegen/task_graph_json.rs:33-226) without a third-party dependency.
#pragma once
#include <stdlib.h>
#include <string.h>
#include <map>
#include <string>
#include <vector>

struct JVal {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false; double num = 0.0; std::string str;
    std::vector<JVal> arr; std::vector<std::pair<std::string, JVal>> obj;
    const JVal *get(const char *key) const {
        if (kind != OBJ) return nullptr;
        for (const auto &kv : obj) if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool is_int() const { return kind == NUM && num == (double)(long long)num; }
};
struct JParser {
    const char *p, *end; std::string err; int depth = 0;
    explicit JParser(const char *text) : p(text), end(text + strlen(text)) {}
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool fail(const char *what) { if (err.empty()) { err = what; err += " at offset "; err += std::to_string((long long)(p - (end - strlen(end)))); } return false; }
    bool parse(JVal &v) {
        if (++depth > 64) return fail("nesting too deep");
        ws();
        if (p >= end) return fail("unexpected end");
        bool ok;
        if (*p == '{') ok = object(v);
        else if (*p == '[') ok = array(v);
        else if (*p == '"') { v.kind = JVal::STR; ok = string(v.str); }
        else if (!strncmp(p, "true", 4)) { v.kind = JVal::BOOL; v.b = true; p += 4; ok = true; }
        else if (!strncmp(p, "false", 5)) { v.kind = JVal::BOOL; v.b = false; p += 5; ok = true; }
        else if (!strncmp(p, "null", 4)) { v.kind = JVal::NUL; p += 4; ok = true; }
        else {
            char *e = nullptr; v.num = strtod(p, &e);
            if (e == p) return fail("unexpected character");
            v.kind = JVal::NUM; p = e; ok = true;
        }
        --depth;
        return ok;
    }
    bool string(std::string &out) {
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("bad escape");
                switch (*p) {
                case 'n': out += '\n'; break; case 't': out += '\t'; break; case 'r': out += '\r'; break;
                case 'b': out += '\b'; break; case 'f': out += '\f'; break;
                case 'u': { if (end - p < 5) return fail("bad \\u escape"); out += '?'; p += 4; break; }      // role strings are ASCII
                default: out += *p;
                }
                ++p;
            } else out += *p++;
        }
        if (p >= end) return fail("unterminated string");
        ++p; return true;
    }
    bool array(JVal &v) {
        v.kind = JVal::ARR; ++p; ws();
        if (p < end && *p == ']') { ++p; return true; }
        for (;;) {
            v.arr.emplace_back();
            if (!parse(v.arr.back())) return false;
            ws();
            if (p < end && *p == ',') { ++p; continue; }
            if (p < end && *p == ']') { ++p; return true; }
            return fail("expected , or ]");
        }
    }
    bool object(JVal &v) {
        v.kind = JVal::OBJ; ++p; ws();
        if (p < end && *p == '}') { ++p; return true; }
        for (;;) {
            ws();
            if (p >= end || *p != '"') return fail("expected a key");
            std::string key; if (!string(key)) return false;
            ws();
            if (p >= end || *p != ':') return fail("expected :");
            ++p;
            v.obj.emplace_back(key, JVal());
            if (!parse(v.obj.back().second)) return false;
            ws();
            if (p < end && *p == ',') { ++p; continue; }
            if (p < end && *p == '}') { ++p; return true; }
            return fail("expected , or }");
        }
    }
};
