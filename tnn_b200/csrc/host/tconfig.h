// Typed key/value configuration with a JSON round trip that keeps an explicit
// type tag per value: {"name":..,"type":..,"parameters":{key:{"type":tag,"value":v}}}.
// Layer configs inside checkpoints use exactly this text form (reference:
// include/common/config.hpp:34-121, src/common/config.cpp:86-253), so the tags
// ("int", "unsigned long", "float", "json", "vector<size_t>", ...) and the
// key-sorted compact dump are part of the file format.
#pragma once
#include <map>
#include <nlohmann/json.hpp>
#include <string>
#include <variant>
#include <vector>

namespace tnnb {

using Json = nlohmann::json;

struct TValue {
  std::string tag;  // type tag as written to JSON
  Json value;
};

class TConfig {
 public:
  std::string name;
  std::string type;

  void set_int(const std::string& k, int v) { params_[k] = {"int", v}; }
  void set_size(const std::string& k, unsigned long v) { params_[k] = {"unsigned long", v}; }
  void set_float(const std::string& k, float v) { params_[k] = {"float", v}; }
  void set_double(const std::string& k, double v) { params_[k] = {"double", v}; }
  void set_bool(const std::string& k, bool v) { params_[k] = {"bool", v}; }
  void set_string(const std::string& k, const std::string& v) { params_[k] = {"string", v}; }
  void set_json(const std::string& k, const Json& v) { params_[k] = {"json", v}; }
  void set_tagged(const std::string& k, const std::string& tag, const Json& v);

  bool has(const std::string& k) const { return params_.count(k) != 0; }
  bool remove(const std::string& k) { return params_.erase(k) > 0; }
  const TValue& at(const std::string& k) const;
  template <typename T>
  T get(const std::string& k, const T& dflt) const {
    auto it = params_.find(k);
    if (it == params_.end()) return dflt;
    return it->second.value.get<T>();
  }
  const std::map<std::string, TValue>& parameters() const { return params_; }

  Json to_json() const;
  static TConfig from_json(const Json& j);
  std::string dump() const { return to_json().dump(); }
  static TConfig parse(const std::string& text) { return from_json(Json::parse(text)); }

  static bool valid_tag(const std::string& tag);

 private:
  std::map<std::string, TValue> params_;
};

}  // namespace tnnb
