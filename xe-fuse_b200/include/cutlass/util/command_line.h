// cutlass::CommandLine: `--key=value` (and bare `--flag`) parsing for the harness mains.
#pragma once
#include <cstdlib>
#include <map>
#include <sstream>
#include <string>
#include <vector>

namespace cutlass {

class CommandLine {
 public:
  CommandLine(int argc, const char** argv) {
    for (int i = 1; i < argc; ++i) {
      std::string a = argv[i];
      if (a.size() < 2 || a[0] != '-') { positional_.push_back(a); continue; }
      a = a.substr(a[1] == '-' ? 2 : 1);
      const size_t eq = a.find('=');
      if (eq == std::string::npos) kv_[a] = "";
      else kv_[a.substr(0, eq)] = a.substr(eq + 1);
    }
  }
  bool check_cmd_line_flag(const char* name) const { return kv_.count(name) != 0; }

  template <class T>
  void get_cmd_line_argument(const char* name, T& value, T const& default_value = T()) const {
    auto it = kv_.find(name);
    if (it == kv_.end() || it->second.empty()) { value = default_value; return; }
    std::istringstream ss(it->second);
    T v{};
    if (ss >> v) value = v; else value = default_value;
  }
  void get_cmd_line_argument(const char* name, bool& value, bool default_value = false) const {
    auto it = kv_.find(name);
    if (it == kv_.end()) { value = default_value; return; }
    value = it->second.empty() || it->second == "1" || it->second == "true";
  }
  void get_cmd_line_argument(const char* name, std::string& value, std::string const& d = "") const {
    auto it = kv_.find(name);
    value = it == kv_.end() ? d : it->second;
  }
  size_t num_naked_args() const { return positional_.size(); }

 private:
  std::map<std::string, std::string> kv_;
  std::vector<std::string> positional_;
};

}  // namespace cutlass
