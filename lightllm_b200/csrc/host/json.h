// A small JSON reader for config.json and the header of a safetensors file: objects, arrays, strings (with the
// standard escapes), numbers, true, false and null.  Errors are exceptions that say where in the text they arose.
#pragma once
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace llb {

struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool boolean = false;
    double number = 0.0;
    bool integral = false;           // the number was written without fraction or exponent
    std::string text;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;      // in the order of the file

    const Json* find(const std::string& key) const {
        if (kind != Object) return nullptr;
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
};

class JsonParser {
public:
    JsonParser(const char* begin, size_t size, std::string where) : p_(begin), end_(begin + size), begin_(begin), where_(std::move(where)) {}

    Json parse() {
        Json v = value(0);
        skip();
        if (p_ != end_) fail("text after the value");
        return v;
    }

private:
    const char *p_, *end_, *begin_;
    std::string where_;

    [[noreturn]] void fail(const std::string& what) const {
        throw std::runtime_error(where_ + ": not valid JSON at byte " + std::to_string(p_ - begin_) + ": " + what);
    }
    void skip() {
        while (p_ != end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
    }
    bool word(const char* w) {
        const char* q = p_;
        for (; *w; ++w, ++q)
            if (q == end_ || *q != *w) return false;
        p_ = q;
        return true;
    }
    static void utf8(std::string& out, unsigned cp) {
        if (cp < 0x80) out += (char)cp;
        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
        else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    }
    unsigned hex4() {
        unsigned v = 0;
        for (int i = 0; i < 4; ++i) {
            if (p_ == end_) fail("unfinished \\u escape");
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        std::string out;
        ++p_;                                       // the opening quote
        for (;;) {
            if (p_ == end_) fail("unfinished string");
            const char c = *p_++;
            if (c == '"') return out;
            if (c != '\\') { out += c; continue; }
            if (p_ == end_) fail("unfinished escape");
            const char e = *p_++;
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
                    if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        const unsigned lo = hex4();
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: fail("unknown escape");
            }
        }
    }
    Json value(int depth) {
        if (depth > 64) fail("nested too deeply");
        skip();
        if (p_ == end_) fail("unexpected end");
        Json v;
        const char c = *p_;
        if (c == '{') {
            v.kind = Json::Object;
            ++p_;
            skip();
            if (p_ != end_ && *p_ == '}') { ++p_; return v; }
            for (;;) {
                skip();
                if (p_ == end_ || *p_ != '"') fail("a member name was expected");
                std::string key = string();
                skip();
                if (p_ == end_ || *p_ != ':') fail("':' was expected");
                ++p_;
                v.members.emplace_back(std::move(key), value(depth + 1));
                skip();
                if (p_ != end_ && *p_ == ',') { ++p_; continue; }
                if (p_ != end_ && *p_ == '}') { ++p_; return v; }
                fail("',' or '}' was expected");
            }
        }
        if (c == '[') {
            v.kind = Json::Array;
            ++p_;
            skip();
            if (p_ != end_ && *p_ == ']') { ++p_; return v; }
            for (;;) {
                v.items.push_back(value(depth + 1));
                skip();
                if (p_ != end_ && *p_ == ',') { ++p_; continue; }
                if (p_ != end_ && *p_ == ']') { ++p_; return v; }
                fail("',' or ']' was expected");
            }
        }
        if (c == '"') { v.kind = Json::String; v.text = string(); return v; }
        if (word("true")) { v.kind = Json::Bool; v.boolean = true; return v; }
        if (word("false")) { v.kind = Json::Bool; return v; }
        if (word("null")) return v;
        if (c == '-' || (c >= '0' && c <= '9')) {
            const char* q = p_;
            bool integral = true;
            if (*q == '-') ++q;
            while (q != end_ && ((*q >= '0' && *q <= '9') || *q == '.' || *q == 'e' || *q == 'E' || *q == '+' || *q == '-')) {
                if (*q == '.' || *q == 'e' || *q == 'E') integral = false;
                ++q;
            }
            const std::string num(p_, q);
            char* stop = nullptr;
            v.number = std::strtod(num.c_str(), &stop);
            if (stop == num.c_str() || *stop) fail("bad number '" + num + "'");
            v.kind = Json::Number;
            v.integral = integral;
            p_ = q;
            return v;
        }
        fail(std::string("unexpected character '") + c + "'");
    }
};

}  // namespace llb
