// Minimal JSON reader for model files: objects, arrays, numbers, strings, booleans, null.
// Arrays whose elements are all numbers are stored flat (`nums`), which is what makes
// multi-hundred-megabyte model files (tens of millions of spline nodes) load in seconds.
// Plays the part nlohmann::json plays in the reference loader (libsymmetrix/source/mace.cpp:908-909);
// a malformed file raises JsonError, the analogue of nlohmann's parse_error that callers treat
// as "not a symmetrix JSON file" (symmetrix/source/symmetrix/symmetrix_calc.py:54-68).
#pragma once

#include <charconv>
#include <limits>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace smx {

struct JsonError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

struct JsonValue {
    enum Type { Null, Bool, Number, String, Array, NumArray, Object } type = Null;
    double num = 0.0;
    bool boolean = false;
    std::string str;
    std::vector<JsonValue> arr;                 // Array
    std::vector<double> nums;                   // NumArray
    std::vector<std::pair<std::string, JsonValue>> obj;  // Object, insertion order kept

    const JsonValue* find(const std::string& key) const {
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    const JsonValue& at(const std::string& key) const {
        const JsonValue* v = find(key);
        if (!v) throw JsonError("model file: missing key '" + key + "'");
        return *v;
    }
    bool is_array() const { return type == Array || type == NumArray; }
    size_t size() const { return type == NumArray ? nums.size() : (type == Array ? arr.size() : obj.size()); }
    double as_double() const {
        if (type != Number) throw JsonError("model file: expected a number");
        return num;
    }
    int as_int() const { return static_cast<int>(as_double()); }
    bool as_bool() const {
        if (type == Bool) return boolean;
        if (type == Number) return num != 0.0;
        throw JsonError("model file: expected a boolean");
    }
    // Flatten nested numeric arrays (row-major) into `out`; returns nothing, appends.
    void flatten(std::vector<double>& out) const {
        if (type == NumArray) {
            out.insert(out.end(), nums.begin(), nums.end());
        } else if (type == Array) {
            for (const auto& v : arr) v.flatten(out);
        } else if (type == Number) {
            out.push_back(num);
        } else {
            throw JsonError("model file: expected a (nested) numeric array");
        }
    }
    std::vector<double> flat() const {
        std::vector<double> out;
        flatten(out);
        return out;
    }
    std::vector<int> flat_int() const {
        std::vector<double> d = flat();
        std::vector<int> out(d.size());
        for (size_t i = 0; i < d.size(); ++i) out[i] = static_cast<int>(d[i]);
        return out;
    }
};

class JsonParser {
public:
    JsonParser(const char* begin, const char* end) : p_(begin), end_(end), begin_(begin) {}

    JsonValue parse() {
        JsonValue v = value();
        ws();
        if (p_ != end_) fail("trailing characters");
        return v;
    }

private:
    const char* p_;
    const char* end_;
    const char* begin_;

    [[noreturn]] void fail(const char* what) const {
        throw JsonError(std::string("[json] parse error at byte ") + std::to_string(p_ - begin_) + ": " + what);
    }
    void ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
    }
    JsonValue value() {
        ws();
        if (p_ >= end_) fail("unexpected end of input");
        const char c = *p_;
        if (c == '{') return object();
        if (c == '[') return array();
        if (c == '"') {
            JsonValue v;
            v.type = JsonValue::String;
            v.str = string();
            return v;
        }
        if (c == 't' || c == 'f' || c == 'n') return literal();
        return number();
    }
    JsonValue literal() {
        JsonValue v;
        auto match = [&](const char* w) {
            const size_t n = std::strlen(w);
            if (static_cast<size_t>(end_ - p_) >= n && std::memcmp(p_, w, n) == 0) {
                p_ += n;
                return true;
            }
            return false;
        };
        if (match("true")) { v.type = JsonValue::Bool; v.boolean = true; }
        else if (match("false")) { v.type = JsonValue::Bool; v.boolean = false; }
        else if (match("null")) { v.type = JsonValue::Null; }
        else if (match("NaN")) { v.type = JsonValue::Number; v.num = std::numeric_limits<double>::quiet_NaN(); }
        else fail("invalid literal");
        return v;
    }
    double raw_number() {
        double d = 0.0;
        const char* start = p_;
        if (p_ < end_ && *p_ == '+') ++p_;
        auto res = std::from_chars(p_, end_, d);
        if (res.ec != std::errc() || res.ptr == start) fail("invalid number");
        p_ = res.ptr;
        return d;
    }
    JsonValue number() {
        JsonValue v;
        v.type = JsonValue::Number;
        v.num = raw_number();
        return v;
    }
    std::string string() {
        if (*p_ != '"') fail("expected string");
        ++p_;
        std::string s;
        while (p_ < end_ && *p_ != '"') {
            if (*p_ == '\\') {
                ++p_;
                if (p_ >= end_) fail("bad escape");
                switch (*p_) {
                    case 'n': s.push_back('\n'); break;
                    case 't': s.push_back('\t'); break;
                    case 'r': s.push_back('\r'); break;
                    case 'b': s.push_back('\b'); break;
                    case 'f': s.push_back('\f'); break;
                    case 'u': s.push_back('?'); p_ += 4; break;
                    default: s.push_back(*p_);
                }
                ++p_;
            } else {
                s.push_back(*p_++);
            }
        }
        if (p_ >= end_) fail("unterminated string");
        ++p_;
        return s;
    }
    JsonValue array() {
        ++p_;  // [
        JsonValue v;
        ws();
        if (p_ < end_ && *p_ == ']') {
            ++p_;
            v.type = JsonValue::NumArray;
            return v;
        }
        // Fast path: try to read a flat numeric array.
        const char c = *p_;
        if (c == '-' || c == '+' || (c >= '0' && c <= '9')) {
            v.type = JsonValue::NumArray;
            while (true) {
                ws();
                v.nums.push_back(raw_number());
                ws();
                if (p_ >= end_) fail("unterminated array");
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == ']') { ++p_; break; }
                fail("expected ',' or ']' in numeric array");
            }
            return v;
        }
        v.type = JsonValue::Array;
        while (true) {
            v.arr.push_back(value());
            ws();
            if (p_ >= end_) fail("unterminated array");
            if (*p_ == ',') { ++p_; continue; }
            if (*p_ == ']') { ++p_; break; }
            fail("expected ',' or ']'");
        }
        return v;
    }
    JsonValue object() {
        ++p_;  // {
        JsonValue v;
        v.type = JsonValue::Object;
        ws();
        if (p_ < end_ && *p_ == '}') { ++p_; return v; }
        while (true) {
            ws();
            std::string key = string();
            ws();
            if (p_ >= end_ || *p_ != ':') fail("expected ':'");
            ++p_;
            v.obj.emplace_back(std::move(key), value());
            ws();
            if (p_ >= end_) fail("unterminated object");
            if (*p_ == ',') { ++p_; continue; }
            if (*p_ == '}') { ++p_; break; }
            fail("expected ',' or '}'");
        }
        return v;
    }
};

}  // namespace smx
