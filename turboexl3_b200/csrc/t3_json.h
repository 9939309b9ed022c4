// A small JSON reader (objects, arrays, strings, numbers, literals) for the pack's config blocks: the quant-plugin table's
// `trunk_quant` / `expert_quant` blocks (table/config.zig:31-44) and spec.parseExpertQuant (src/core/spec.zig:38-50). Host only.
#pragma once

#include <cctype>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace t3json {

struct Json {
    enum Kind { kNull, kBool, kInt, kFloat, kString, kArray, kObject } kind = kNull;
    bool b = false;
    long long i = 0;
    double f = 0;
    std::string s;
    std::vector<Json> items;
    std::map<std::string, Json> fields;
    const Json* get(const char* key) const {
        if (kind != kObject) return nullptr;
        auto it = fields.find(key);
        return it == fields.end() ? nullptr : &it->second;
    }
};

struct JsonReader {
    const char* p;
    const char* end;
    bool ok = true;
    void skip() {
        while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p;
    }
    bool eat(char c) {
        skip();
        if (p < end && *p == c) {
            ++p;
            return true;
        }
        return false;
    }
    std::string str() {
        std::string out;
        if (!eat('"')) {
            ok = false;
            return out;
        }
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                ++p;
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u':
                        out += '?';
                        p += (end - p > 4) ? 4 : 0;
                        break;
                    default: out += *p;
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= end) ok = false;
        else ++p;
        return out;
    }
    Json value(int depth = 0) {
        Json v;
        skip();
        if (p >= end || depth > 64) {
            ok = false;
            return v;
        }
        if (*p == '{') {
            ++p;
            v.kind = Json::kObject;
            if (eat('}')) return v;
            do {
                std::string key = str();
                if (!ok || !eat(':')) {
                    ok = false;
                    return v;
                }
                v.fields[key] = value(depth + 1);
                if (!ok) return v;
            } while (eat(','));
            if (!eat('}')) ok = false;
        } else if (*p == '[') {
            ++p;
            v.kind = Json::kArray;
            if (eat(']')) return v;
            do {
                v.items.push_back(value(depth + 1));
                if (!ok) return v;
            } while (eat(','));
            if (!eat(']')) ok = false;
        } else if (*p == '"') {
            v.kind = Json::kString;
            v.s = str();
        } else if (end - p >= 4 && !strncmp(p, "true", 4)) {
            v.kind = Json::kBool, v.b = true, p += 4;
        } else if (end - p >= 5 && !strncmp(p, "false", 5)) {
            v.kind = Json::kBool, p += 5;
        } else if (end - p >= 4 && !strncmp(p, "null", 4)) {
            p += 4;
        } else {
            const char* q = p;
            bool is_float = false;
            while (q < end && (isdigit((unsigned char)*q) || *q == '-' || *q == '+' || *q == '.' || *q == 'e' || *q == 'E')) {
                if (*q == '.' || *q == 'e' || *q == 'E') is_float = true;
                ++q;
            }
            if (q == p) {
                ok = false;
                return v;
            }
            const std::string tok(p, q);
            char* tail = nullptr;
            if (is_float) {
                v.kind = Json::kFloat;
                v.f = strtod(tok.c_str(), &tail);
            } else {
                v.kind = Json::kInt;
                v.i = strtoll(tok.c_str(), &tail, 10);
                v.f = (double)v.i;
            }
            if (!tail || *tail != '\0') ok = false;
            p = q;
        }
        return v;
    }
};


}  // namespace t3json
