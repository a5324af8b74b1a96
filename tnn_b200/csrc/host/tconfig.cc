#include "tconfig.h"

#include <stdexcept>

namespace tnnb {

static const char* kTags[] = {"int", "long", "long long", "unsigned int", "unsigned long", "unsigned long long",
                              "size_t", "float", "double", "bool", "string", "json", "vector<size_t>",
                              "vector<int>", "vector<float>", "vector<double>", "vector<string>"};

bool TConfig::valid_tag(const std::string& tag) {
  for (const char* t : kTags)
    if (tag == t) return true;
  return false;
}

// Normalise a JSON value to what the tagged C++ type would hold (a "float" is
// rounded to binary32 so that it prints like a widened float, integers are
// range-checked by the conversion).
static Json coerce(const std::string& tag, const Json& v) {
  if (tag == "int") return v.get<int>();
  if (tag == "long") return v.get<long>();
  if (tag == "long long") return v.get<long long>();
  if (tag == "unsigned int") return v.get<unsigned int>();
  if (tag == "unsigned long" || tag == "size_t") return v.get<unsigned long>();
  if (tag == "unsigned long long") return v.get<unsigned long long>();
  if (tag == "float") return v.get<float>();
  if (tag == "double") return v.get<double>();
  if (tag == "bool") return v.get<bool>();
  if (tag == "string") return v.get<std::string>();
  if (tag == "json") return v;
  if (tag == "vector<size_t>") return v.get<std::vector<unsigned long>>();
  if (tag == "vector<int>") return v.get<std::vector<int>>();
  if (tag == "vector<float>") return v.get<std::vector<float>>();
  if (tag == "vector<double>") return v.get<std::vector<double>>();
  if (tag == "vector<string>") return v.get<std::vector<std::string>>();
  throw std::runtime_error("Unknown type in JSON: " + tag);
}

void TConfig::set_tagged(const std::string& k, const std::string& tag, const Json& v) {
  params_[k] = {tag, coerce(tag, v)};
}

const TValue& TConfig::at(const std::string& k) const {
  auto it = params_.find(k);
  if (it == params_.end()) throw std::out_of_range("TConfig: no parameter '" + k + "'");
  return it->second;
}

Json TConfig::to_json() const {
  Json j;
  j["name"] = name;
  j["type"] = type;
  Json p = Json::object();
  for (const auto& kv : params_) {
    Json e;
    e["type"] = kv.second.tag;
    e["value"] = kv.second.value;
    p[kv.first] = e;
  }
  j["parameters"] = p;
  return j;
}

TConfig TConfig::from_json(const Json& j) {
  TConfig c;
  c.name = j.value("name", "");
  c.type = j.value("type", "");
  if (j.contains("parameters") && j["parameters"].is_object()) {
    for (auto it = j["parameters"].begin(); it != j["parameters"].end(); ++it) {
      const Json& tv = it.value();
      if (!tv.is_object() || !tv.contains("type") || !tv.contains("value")) continue;  // skipped, like the reference's warning path
      const std::string tag = tv["type"].get<std::string>();
      try {
        c.params_[it.key()] = {tag, coerce(tag, tv["value"])};
      } catch (const std::exception&) {
      }
    }
  }
  return c;
}

}  // namespace tnnb
