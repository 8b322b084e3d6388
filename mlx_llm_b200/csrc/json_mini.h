// Minimal JSON reader (objects, arrays, strings, numbers, bools, null) for config.json and the
// safetensors header.  Value-parsed like the reference does with serde_json (src/config.rs:315-502).
#pragma once
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace b2json {

struct Value;
using ValuePtr = std::shared_ptr<Value>;

struct Value {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0;
    bool is_int = false;
    std::string str;
    std::vector<ValuePtr> arr;
    std::vector<std::pair<std::string, ValuePtr>> obj;  // insertion order kept

    const Value* get(const std::string& key) const {
        if (kind != Object) return nullptr;
        for (auto& kv : obj)
            if (kv.first == key) return kv.second.get();
        return nullptr;
    }
    bool as_i64(long long& out) const {
        if (kind != Number || !is_int) return false;
        out = (long long)num;
        return true;
    }
    bool as_f64(double& out) const {
        if (kind != Number) return false;
        out = num;
        return true;
    }
};

class Parser {
   public:
    explicit Parser(const std::string& s) : s_(s) {}
    ValuePtr parse(std::string& err) {
        ValuePtr v = value(err);
        if (!v) return nullptr;
        ws();
        if (i_ != s_.size()) {
            err = "trailing characters in JSON";
            return nullptr;
        }
        return v;
    }

   private:
    const std::string& s_;
    size_t i_ = 0;
    void ws() {
        while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) i_++;
    }
    ValuePtr value(std::string& err) {
        ws();
        if (i_ >= s_.size()) {
            err = "unexpected end of JSON";
            return nullptr;
        }
        char c = s_[i_];
        auto v = std::make_shared<Value>();
        if (c == '{') {
            v->kind = Value::Object;
            i_++;
            ws();
            if (i_ < s_.size() && s_[i_] == '}') {
                i_++;
                return v;
            }
            while (true) {
                ws();
                std::string key;
                if (!string(key, err)) return nullptr;
                ws();
                if (i_ >= s_.size() || s_[i_] != ':') {
                    err = "expected ':' in JSON object";
                    return nullptr;
                }
                i_++;
                ValuePtr child = value(err);
                if (!child) return nullptr;
                v->obj.emplace_back(key, child);
                ws();
                if (i_ < s_.size() && s_[i_] == ',') {
                    i_++;
                    continue;
                }
                if (i_ < s_.size() && s_[i_] == '}') {
                    i_++;
                    return v;
                }
                err = "expected ',' or '}' in JSON object";
                return nullptr;
            }
        }
        if (c == '[') {
            v->kind = Value::Array;
            i_++;
            ws();
            if (i_ < s_.size() && s_[i_] == ']') {
                i_++;
                return v;
            }
            while (true) {
                ValuePtr child = value(err);
                if (!child) return nullptr;
                v->arr.push_back(child);
                ws();
                if (i_ < s_.size() && s_[i_] == ',') {
                    i_++;
                    continue;
                }
                if (i_ < s_.size() && s_[i_] == ']') {
                    i_++;
                    return v;
                }
                err = "expected ',' or ']' in JSON array";
                return nullptr;
            }
        }
        if (c == '"') {
            v->kind = Value::String;
            if (!string(v->str, err)) return nullptr;
            return v;
        }
        if (s_.compare(i_, 4, "true") == 0) {
            v->kind = Value::Bool;
            v->b = true;
            i_ += 4;
            return v;
        }
        if (s_.compare(i_, 5, "false") == 0) {
            v->kind = Value::Bool;
            i_ += 5;
            return v;
        }
        if (s_.compare(i_, 4, "null") == 0) {
            i_ += 4;
            return v;
        }
        // number
        size_t st = i_;
        bool is_int = true;
        if (i_ < s_.size() && (s_[i_] == '-' || s_[i_] == '+')) i_++;
        while (i_ < s_.size() && ((s_[i_] >= '0' && s_[i_] <= '9') || s_[i_] == '.' || s_[i_] == 'e' || s_[i_] == 'E' || s_[i_] == '-' || s_[i_] == '+')) {
            if (s_[i_] == '.' || s_[i_] == 'e' || s_[i_] == 'E') is_int = false;
            i_++;
        }
        if (i_ == st) {
            err = "unexpected character in JSON";
            return nullptr;
        }
        v->kind = Value::Number;
        v->num = std::strtod(s_.substr(st, i_ - st).c_str(), nullptr);
        v->is_int = is_int;
        return v;
    }
    bool string(std::string& out, std::string& err) {
        if (i_ >= s_.size() || s_[i_] != '"') {
            err = "expected string in JSON";
            return false;
        }
        i_++;
        while (i_ < s_.size() && s_[i_] != '"') {
            if (s_[i_] == '\\' && i_ + 1 < s_.size()) {
                char e = s_[i_ + 1];
                switch (e) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u':
                        // keep the escape verbatim; keys of interest are ASCII
                        out += "\\u";
                        break;
                    default: out += e;
                }
                i_ += 2;
            } else {
                out += s_[i_++];
            }
        }
        if (i_ >= s_.size()) {
            err = "unterminated JSON string";
            return false;
        }
        i_++;
        return true;
    }
};

inline ValuePtr parse(const std::string& s, std::string& err) {
    Parser p(s);
    return p.parse(err);
}

}  // namespace b2json
