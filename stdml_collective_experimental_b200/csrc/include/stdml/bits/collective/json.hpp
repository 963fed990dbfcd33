// A small JSON value with a reader and a writer.  The reference ships writer
// helpers only (include/stdml/bits/collective/json.hpp:14-36; its parser
// classes are empty) and therefore needs a Go shim to read cluster
// configurations; here the elastic controller reads them natively.
#pragma once
#include <cstdint>
#include <map>
#include <optional>
#include <string>
#include <utility>
#include <vector>

namespace stdml::collective::json
{
class value
{
  public:
    enum kind { null_k, bool_k, number_k, string_k, array_k, object_k };

    value() = default;
    static value boolean(bool b);
    static value number(double d);
    static value integer(int64_t i);
    static value string(std::string s);
    static value array(std::vector<value> xs = {});
    static value object(std::vector<std::pair<std::string, value>> kv = {});

    kind type() const { return kind_; }
    bool is_null() const { return kind_ == null_k; }

    bool as_bool() const { return bool_; }
    double as_double() const { return num_; }
    int64_t as_int() const { return is_int_ ? int_ : static_cast<int64_t>(num_); }
    const std::string &as_string() const { return str_; }
    const std::vector<value> &items() const { return arr_; }
    const std::vector<std::pair<std::string, value>> &members() const { return obj_; }

    // member lookup; nullptr when absent or when *this is not an object
    const value *get(const std::string &key) const;
    void set(const std::string &key, value v);
    void push(value v) { arr_.push_back(std::move(v)); }

    std::string dump() const;

  private:
    kind kind_ = null_k;
    bool bool_ = false;
    bool is_int_ = false;
    double num_ = 0;
    int64_t int_ = 0;
    std::string str_;
    std::vector<value> arr_;
    std::vector<std::pair<std::string, value>> obj_;  // insertion order kept
};

// nullopt on any syntax error or trailing garbage
std::optional<value> parse(const std::string &text);

std::string quote(const std::string &s);

// writer helpers with the reference's names
std::string to_json(const std::string &s);
std::string to_json(int64_t i);
template <typename V>
std::string to_json(const std::pair<std::string, V> &kv)
{
    return quote(kv.first) + ":" + to_json(kv.second);
}
}  // namespace stdml::collective::json
