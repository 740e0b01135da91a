// A small JSON value, parser and writer: config.json, the safetensors header,
// model descriptions, replay steps and the command line's --json lines all go
// through it.  Objects keep their members in file order; a key that appears
// twice is an error (a safetensors header with a duplicate tensor must be
// refused, not silently resolved).
#pragma once

#include <cstdint>
#include <string>
#include <string_view>
#include <utility>
#include <vector>

#include "status.h"

namespace liyab {

class Json {
public:
    enum class Type { Null, Bool, Int, Double, String, Array, Object };
    using Member = std::pair<std::string, Json>;

    Json() = default;
    Json(std::nullptr_t) {}
    Json(bool v) : type_(Type::Bool), int_(v) {}
    Json(int v) : type_(Type::Int), int_(v) {}
    Json(int64_t v) : type_(Type::Int), int_(v) {}
    Json(uint64_t v) : type_(Type::Int), int_(static_cast<int64_t>(v)) {}
    Json(double v) : type_(Type::Double), double_(v) {}
    Json(const char* v) : type_(Type::String), string_(v) {}
    Json(std::string v) : type_(Type::String), string_(std::move(v)) {}
    Json(std::string_view v) : type_(Type::String), string_(v) {}

    static Json array() { Json j; j.type_ = Type::Array; return j; }
    static Json object() { Json j; j.type_ = Type::Object; return j; }
    template <class T>
    static Json array_of(const std::vector<T>& values) {
        Json j = array();
        for (const auto& v : values) j.push(Json(v));
        return j;
    }

    // Parses one JSON document; `what` names the source in error messages.
    static Json parse(std::string_view text, const std::string& what = "JSON");
    std::string dump(int indent = -1) const;

    Type type() const { return type_; }
    bool is_null() const { return type_ == Type::Null; }
    bool is_bool() const { return type_ == Type::Bool; }
    bool is_int() const { return type_ == Type::Int; }
    bool is_number() const { return type_ == Type::Int || type_ == Type::Double; }
    bool is_string() const { return type_ == Type::String; }
    bool is_array() const { return type_ == Type::Array; }
    bool is_object() const { return type_ == Type::Object; }

    bool as_bool() const { expect(Type::Bool, "a boolean"); return int_ != 0; }
    int64_t as_int() const { expect(Type::Int, "an integer"); return int_; }
    double as_number() const {
        if (type_ == Type::Int) return static_cast<double>(int_);
        expect(Type::Double, "a number");
        return double_;
    }
    const std::string& as_string() const { expect(Type::String, "a string"); return string_; }
    const std::vector<Json>& items() const { expect(Type::Array, "an array"); return items_; }
    const std::vector<Member>& members() const { expect(Type::Object, "an object"); return members_; }
    size_t size() const { return type_ == Type::Array ? items_.size() : type_ == Type::Object ? members_.size() : 0; }

    // Object access: find returns null when the key is absent.
    const Json* find(std::string_view key) const;
    const Json& at(std::string_view key) const;
    bool contains(std::string_view key) const { return find(key) != nullptr; }
    Json& set(std::string key, Json value);      // replaces an existing member
    Json& push(Json value);
    const Json& operator[](size_t i) const { return items()[i]; }

    // Typed reads with defaults, for part options (`what` names the owner in errors).
    int64_t get_int(std::string_view key, int64_t fallback) const;
    double get_number(std::string_view key, double fallback) const;
    bool get_bool(std::string_view key, bool fallback) const;
    std::string get_string(std::string_view key, const std::string& fallback) const;
    std::vector<int64_t> int_list() const;

    bool operator==(const Json& o) const;

private:
    void expect(Type t, const char* what) const;
    void write(std::string& out, int indent, int depth) const;

    Type type_ = Type::Null;
    int64_t int_ = 0;
    double double_ = 0.0;
    std::string string_;
    std::vector<Json> items_;
    std::vector<Member> members_;
};

}  // namespace liyab
