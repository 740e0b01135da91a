#include "json.h"

#include <charconv>
#include <cmath>
#include <cstdio>
#include <cstdlib>

namespace liyab {
namespace {

class Parser {
public:
    Parser(std::string_view text, const std::string& what) : s_(text), what_(what) {}

    Json document() {
        skip();
        Json v = value(0);
        skip();
        if (i_ != s_.size()) fail("unexpected characters after the document");
        return v;
    }

private:
    [[noreturn]] void fail(const std::string& why) const {
        throw invalid_argument("{} is not valid JSON: {} at byte {}", what_, why, i_);
    }
    void skip() {
        while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\t' || s_[i_] == '\n' || s_[i_] == '\r')) ++i_;
    }
    bool take(char c) {
        if (i_ < s_.size() && s_[i_] == c) { ++i_; return true; }
        return false;
    }
    void literal(std::string_view word) {
        if (s_.substr(i_, word.size()) != word) fail("unknown literal");
        i_ += word.size();
    }

    Json value(int depth) {
        if (depth > 64) fail("nesting too deep");
        if (i_ >= s_.size()) fail("unexpected end");
        const char c = s_[i_];
        if (c == '{') return object(depth);
        if (c == '[') return array(depth);
        if (c == '"') return Json(string());
        if (c == 't') { literal("true"); return Json(true); }
        if (c == 'f') { literal("false"); return Json(false); }
        if (c == 'n') { literal("null"); return Json(nullptr); }
        if (c == 'N') { literal("NaN"); return Json(std::nan("")); }
        if (c == 'I') { literal("Infinity"); return Json(HUGE_VAL); }
        return number();
    }

    Json object(int depth) {
        ++i_;
        Json out = Json::object();
        skip();
        if (take('}')) return out;
        while (true) {
            skip();
            if (i_ >= s_.size() || s_[i_] != '"') fail("expected a member name");
            std::string key = string();
            if (out.contains(key)) throw invalid_argument("{}: '{}' appears twice", what_, key);
            skip();
            if (!take(':')) fail("expected ':'");
            skip();
            out.set(std::move(key), value(depth + 1));
            skip();
            if (take(',')) continue;
            if (take('}')) return out;
            fail("expected ',' or '}'");
        }
    }

    Json array(int depth) {
        ++i_;
        Json out = Json::array();
        skip();
        if (take(']')) return out;
        while (true) {
            skip();
            out.push(value(depth + 1));
            skip();
            if (take(',')) continue;
            if (take(']')) return out;
            fail("expected ',' or ']'");
        }
    }

    static void append_utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) out.push_back(static_cast<char>(cp));
        else if (cp < 0x800) { out.push_back(static_cast<char>(0xC0 | (cp >> 6))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
        else if (cp < 0x10000) {
            out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else {
            out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        }
    }

    uint32_t hex4() {
        if (i_ + 4 > s_.size()) fail("short \\u escape");
        uint32_t v = 0;
        for (int k = 0; k < 4; ++k) {
            const char c = s_[i_++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else fail("bad \\u escape");
        }
        return v;
    }

    std::string string() {
        ++i_;
        std::string out;
        while (true) {
            if (i_ >= s_.size()) fail("unterminated string");
            const char c = s_[i_++];
            if (c == '"') return out;
            if (static_cast<unsigned char>(c) < 0x20) fail("control character in a string");
            if (c != '\\') { out.push_back(c); continue; }
            if (i_ >= s_.size()) fail("unterminated escape");
            const char e = s_[i_++];
            switch (e) {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'n': out.push_back('\n'); break;
                case 'r': out.push_back('\r'); break;
                case 't': out.push_back('\t'); break;
                case 'u': {
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && s_.substr(i_, 2) == "\\u") {
                        i_ += 2;
                        const uint32_t lo = hex4();
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    append_utf8(out, cp);
                    break;
                }
                default: fail("unknown escape");
            }
        }
    }

    Json number() {
        const size_t start = i_;
        if (take('-') && s_.substr(i_, 8) == "Infinity") { i_ += 8; return Json(-HUGE_VAL); }
        bool integral = true;
        while (i_ < s_.size()) {
            const char c = s_[i_];
            if (c >= '0' && c <= '9') { ++i_; continue; }
            if (c == '.' || c == 'e' || c == 'E' || c == '+' || c == '-') { integral = false; ++i_; continue; }
            break;
        }
        const std::string_view tok = s_.substr(start, i_ - start);
        if (tok.empty() || tok == "-") { i_ = start; fail("expected a value"); }
        if (integral) {
            int64_t v = 0;
            auto [p, ec] = std::from_chars(tok.data(), tok.data() + tok.size(), v);
            if (ec == std::errc() && p == tok.data() + tok.size()) return Json(v);
        }
        const std::string copy(tok);
        char* end = nullptr;
        const double d = std::strtod(copy.c_str(), &end);
        if (end != copy.c_str() + copy.size()) { i_ = start; fail("malformed number"); }
        return Json(d);
    }

    std::string_view s_;
    const std::string& what_;
    size_t i_ = 0;
};

void write_string(std::string& out, const std::string& s) {
    out.push_back('"');
    for (const char ch : s) {
        const unsigned char c = static_cast<unsigned char>(ch);
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (c < 0x20) {
                    char buf[8];
                    std::snprintf(buf, sizeof buf, "\\u%04x", c);
                    out += buf;
                } else {
                    out.push_back(ch);
                }
        }
    }
    out.push_back('"');
}

}  // namespace

Json Json::parse(std::string_view text, const std::string& what) { return Parser(text, what).document(); }

void Json::expect(Type t, const char* what) const {
    if (type_ != t) throw invalid_argument("JSON value is not {}", what);
}

const Json* Json::find(std::string_view key) const {
    if (type_ != Type::Object) return nullptr;
    for (const auto& m : members_)
        if (m.first == key) return &m.second;
    return nullptr;
}

const Json& Json::at(std::string_view key) const {
    const Json* v = find(key);
    if (v == nullptr) throw invalid_argument("JSON object has no member '{}'", key);
    return *v;
}

Json& Json::set(std::string key, Json value) {
    if (type_ == Type::Null) type_ = Type::Object;
    expect(Type::Object, "an object");
    for (auto& m : members_)
        if (m.first == key) { m.second = std::move(value); return *this; }
    members_.emplace_back(std::move(key), std::move(value));
    return *this;
}

Json& Json::push(Json value) {
    if (type_ == Type::Null) type_ = Type::Array;
    expect(Type::Array, "an array");
    items_.push_back(std::move(value));
    return *this;
}

int64_t Json::get_int(std::string_view key, int64_t fallback) const {
    const Json* v = find(key);
    if (v == nullptr || v->is_null()) return fallback;
    if (!v->is_int()) throw invalid_argument("'{}' must be an integer", key);
    return v->int_;
}

double Json::get_number(std::string_view key, double fallback) const {
    const Json* v = find(key);
    if (v == nullptr || v->is_null()) return fallback;
    if (!v->is_number()) throw invalid_argument("'{}' must be a number", key);
    return v->as_number();
}

bool Json::get_bool(std::string_view key, bool fallback) const {
    const Json* v = find(key);
    if (v == nullptr || v->is_null()) return fallback;
    if (!v->is_bool()) throw invalid_argument("'{}' must be true or false", key);
    return v->int_ != 0;
}

std::string Json::get_string(std::string_view key, const std::string& fallback) const {
    const Json* v = find(key);
    if (v == nullptr || v->is_null()) return fallback;
    if (!v->is_string()) throw invalid_argument("'{}' must be a string", key);
    return v->string_;
}

std::vector<int64_t> Json::int_list() const {
    std::vector<int64_t> out;
    for (const auto& v : items()) out.push_back(v.as_int());
    return out;
}

bool Json::operator==(const Json& o) const {
    if (is_number() && o.is_number()) return as_number() == o.as_number();
    if (type_ != o.type_) return false;
    switch (type_) {
        case Type::Null: return true;
        case Type::Bool: return int_ == o.int_;
        case Type::String: return string_ == o.string_;
        case Type::Array: return items_ == o.items_;
        case Type::Object: return members_ == o.members_;
        default: return false;
    }
}

void Json::write(std::string& out, int indent, int depth) const {
    auto newline = [&](int d) {
        if (indent < 0) return;
        out.push_back('\n');
        out.append(static_cast<size_t>(indent * d), ' ');
    };
    switch (type_) {
        case Type::Null: out += "null"; break;
        case Type::Bool: out += int_ ? "true" : "false"; break;
        case Type::Int: out += std::to_string(int_); break;
        case Type::Double: {
            if (std::isnan(double_)) { out += "NaN"; break; }
            if (std::isinf(double_)) { out += double_ > 0 ? "Infinity" : "-Infinity"; break; }
            char buf[40];
            std::snprintf(buf, sizeof buf, "%.17g", double_);
            std::string s(buf);
            // the shortest form that reads back to the same double
            for (int prec = 1; prec < 17; ++prec) {
                char t[40];
                std::snprintf(t, sizeof t, "%.*g", prec, double_);
                if (std::strtod(t, nullptr) == double_) { s = t; break; }
            }
            if (s.find_first_of(".eEn") == std::string::npos) s += ".0";
            out += s;
            break;
        }
        case Type::String: write_string(out, string_); break;
        case Type::Array:
            out.push_back('[');
            for (size_t i = 0; i < items_.size(); ++i) {
                if (i) out += indent < 0 ? ", " : ",";
                if (items_[i].is_array() || items_[i].is_object()) newline(depth + 1);
                items_[i].write(out, indent, depth + 1);
            }
            out.push_back(']');
            break;
        case Type::Object:
            out.push_back('{');
            for (size_t i = 0; i < members_.size(); ++i) {
                if (i) out += indent < 0 ? ", " : ",";
                newline(depth + 1);
                write_string(out, members_[i].first);
                out += ": ";
                members_[i].second.write(out, indent, depth + 1);
            }
            if (!members_.empty()) newline(depth);
            out.push_back('}');
            break;
    }
}

std::string Json::dump(int indent) const {
    std::string out;
    write(out, indent, 0);
    return out;
}

}  // namespace liyab
