// A small JSON reader: enough for safetensors headers, checkpoint indexes and configuration
// files. Numbers keep whether they were written as integers. Objects keep their order.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <string>
#include <utility>
#include <vector>

#include "host.hpp"

namespace llmh {

struct Json {
    enum Kind { Null, Bool, Integer, Real, String, Array, Object } kind = Null;
    bool boolean = false;
    long long integer = 0;
    double real = 0.0;
    std::string string;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;

    const Json* find(const std::string& key) const {
        for (const auto& member : members)
            if (member.first == key) return &member.second;
        return nullptr;
    }
};

class JsonReader {
public:
    JsonReader(const char* text, size_t size, std::string where) : p_(text), end_(text + size), begin_(text), where_(std::move(where)) {}

    Json read() {
        Json value = value_(0);
        space_();
        if (p_ != end_) bad_("text after the value");
        return value;
    }

private:
    const char *p_, *end_, *begin_;
    std::string where_;

    [[noreturn]] void bad_(const std::string& what) const {
        throw Failure{LLMH_FORMAT, where_ + ": not JSON (" + what + " at byte " + std::to_string(p_ - begin_) + ")"};
    }
    void space_() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
    }
    bool word_(const char* word) {
        size_t n = 0;
        while (word[n]) ++n;
        if ((size_t)(end_ - p_) < n) return false;
        for (size_t i = 0; i < n; ++i)
            if (p_[i] != word[i]) return false;
        p_ += n;
        return true;
    }
    static void utf8_(std::string& out, uint32_t code) {
        if (code < 0x80) out += (char)code;
        else if (code < 0x800) { out += (char)(0xC0 | (code >> 6)); out += (char)(0x80 | (code & 0x3F)); }
        else if (code < 0x10000) { out += (char)(0xE0 | (code >> 12)); out += (char)(0x80 | ((code >> 6) & 0x3F)); out += (char)(0x80 | (code & 0x3F)); }
        else { out += (char)(0xF0 | (code >> 18)); out += (char)(0x80 | ((code >> 12) & 0x3F)); out += (char)(0x80 | ((code >> 6) & 0x3F)); out += (char)(0x80 | (code & 0x3F)); }
    }
    uint32_t hex4_() {
        if (end_ - p_ < 4) bad_("short \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else bad_("bad \\u escape");
        }
        return v;
    }
    std::string string_() {
        ++p_;                                          // the opening quote
        std::string out;
        while (true) {
            if (p_ >= end_) bad_("unterminated string");
            unsigned char c = (unsigned char)*p_++;
            if (c == '"') return out;
            if (c < 0x20) bad_("control character in a string");
            if (c != '\\') { out += (char)c; continue; }
            if (p_ >= end_) bad_("unterminated escape");
            char e = *p_++;
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
                    uint32_t code = hex4_();
                    if (code >= 0xD800 && code < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        uint32_t low = hex4_();
                        if (low >= 0xDC00 && low < 0xE000) code = 0x10000 + ((code - 0xD800) << 10) + (low - 0xDC00);
                        else bad_("unpaired surrogate");
                    }
                    utf8_(out, code);
                    break;
                }
                default: bad_("unknown escape");
            }
        }
    }
    Json number_() {
        const char* start = p_;
        bool integral = true;
        if (p_ < end_ && *p_ == '-') ++p_;
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') bad_("a number needs digits");
        while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        if (p_ < end_ && *p_ == '.') {
            integral = false;
            ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') bad_("digits must follow the point");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false;
            ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') bad_("digits must follow the exponent");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        std::string text(start, p_);
        Json value;
        if (integral && text.size() <= 18) {
            value.kind = Json::Integer;
            value.integer = std::strtoll(text.c_str(), nullptr, 10);
            value.real = (double)value.integer;
        } else {
            value.kind = Json::Real;
            value.real = std::strtod(text.c_str(), nullptr);
        }
        return value;
    }
    Json value_(int depth) {
        if (depth > 64) bad_("nested too deeply");
        space_();
        if (p_ >= end_) bad_("the text ends where a value should be");
        Json value;
        char c = *p_;
        if (c == '{') {
            ++p_;
            value.kind = Json::Object;
            space_();
            if (p_ < end_ && *p_ == '}') { ++p_; return value; }
            while (true) {
                space_();
                if (p_ >= end_ || *p_ != '"') bad_("a member needs a name in quotes");
                std::string key = string_();
                space_();
                if (p_ >= end_ || *p_ != ':') bad_("':' missing after a member's name");
                ++p_;
                value.members.emplace_back(std::move(key), value_(depth + 1));
                space_();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return value; }
                bad_("',' or '}' missing in an object");
            }
        }
        if (c == '[') {
            ++p_;
            value.kind = Json::Array;
            space_();
            if (p_ < end_ && *p_ == ']') { ++p_; return value; }
            while (true) {
                value.items.push_back(value_(depth + 1));
                space_();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return value; }
                bad_("',' or ']' missing in an array");
            }
        }
        if (c == '"') { value.kind = Json::String; value.string = string_(); return value; }
        if (word_("true")) { value.kind = Json::Bool; value.boolean = true; return value; }
        if (word_("false")) { value.kind = Json::Bool; return value; }
        if (word_("null")) return value;
        if (c == '-' || (c >= '0' && c <= '9')) return number_();
        bad_("unexpected character");
    }
};

}  // namespace llmh
