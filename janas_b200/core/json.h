// A small JSON value: parse, build, write.  config.json, the safetensors
// header, model specs and the argument lists of the library's generic calls
// are all JSON; nothing here knows what any of them means.
//
// Numbers keep whether they were written as whole numbers (so that "a whole
// number is needed" can be said of 2.5 and of 1e400, and 64-bit seeds survive).
// Objects keep the order of their keys.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace jb {

struct JsonError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class Json {
public:
    enum Type { Null, Bool, Int, Real, String, Array, Object };

    Json() : type_(Null) {}
    Json(std::nullptr_t) : type_(Null) {}
    Json(bool b) : type_(Bool), b_(b) {}
    Json(int v) : type_(Int), i_(v) {}
    Json(unsigned v) : type_(Int), i_(v) {}
    Json(long v) : type_(Int), i_(v) {}
    Json(long long v) : type_(Int), i_(v) {}
    Json(unsigned long v) : type_(Int), i_((long long)v), u_(v), big_(v > (1ull << 63) - 1) {}
    Json(unsigned long long v) : type_(Int), i_((long long)v), u_(v), big_(v > (1ull << 63) - 1) {}
    Json(double v) : type_(Real), d_(v) {}
    Json(const char *s) : type_(String), s_(s) {}
    Json(std::string s) : type_(String), s_(std::move(s)) {}

    static Json array() { Json j; j.type_ = Array; return j; }
    static Json object() { Json j; j.type_ = Object; return j; }
    static Json parse(const std::string &text);      // throws JsonError

    Type type() const { return type_; }
    bool is_null() const { return type_ == Null; }
    bool is_bool() const { return type_ == Bool; }
    bool is_int() const { return type_ == Int; }
    bool big() const { return big_; }   // a whole number above 2^63 - 1
    bool is_number() const { return type_ == Int || type_ == Real; }
    bool is_string() const { return type_ == String; }
    bool is_array() const { return type_ == Array; }
    bool is_object() const { return type_ == Object; }

    bool as_bool() const { return type_ == Bool ? b_ : type_ == Int ? i_ != 0 : false; }
    long long as_int() const { return type_ == Int ? i_ : type_ == Real ? (long long)d_ : 0; }
    unsigned long long as_uint() const { return type_ == Int ? (big_ ? u_ : (unsigned long long)i_) : 0; }
    double as_double() const { return type_ == Real ? d_ : type_ == Int ? (big_ ? (double)u_ : (double)i_) : 0.0; }
    const std::string &as_string() const { return s_; }
    // true when the number is a whole one that a 64-bit integer holds
    bool whole() const { return type_ == Int || (type_ == Real && d_ == (double)(long long)d_ &&
                                                  d_ > -9.2e18 && d_ < 9.2e18); }

    // arrays
    size_t size() const { return type_ == Array ? a_.size() : type_ == Object ? o_.size() : 0; }
    const Json &operator[](size_t i) const { return a_.at(i); }
    Json &operator[](size_t i) { return a_.at(i); }
    void push(Json v) { a_.push_back(std::move(v)); }
    const std::vector<Json> &items() const { return a_; }

    // objects
    bool has(const std::string &k) const;
    const Json &get(const std::string &k) const;            // Null value when absent
    Json &set(const std::string &k, Json v);
    const std::vector<std::pair<std::string, Json>> &members() const { return o_; }

    std::string dump() const;

private:
    Type type_;
    bool b_ = false;
    long long i_ = 0;
    unsigned long long u_ = 0;
    bool big_ = false;
    double d_ = 0.0;
    std::string s_;
    std::vector<Json> a_;
    std::vector<std::pair<std::string, Json>> o_;
    friend class JsonParser;
};

}  // namespace jb
