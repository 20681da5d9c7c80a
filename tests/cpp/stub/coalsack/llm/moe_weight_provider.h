// TEST DOUBLE of coalsack's moe_weight_provider (include/coalsack/llm/moe_weight_provider.h:18-70):
// same class name and the same get(tensor_name, expert_id) as the reference's provider, but the expert
// slices come from memory instead of GGUF shards, so the graph check needs no model file.  It sits ahead
// of the reference's header on the include path of tests/cpp/graph_check.cpp only.
#pragma once

#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <variant>

#include "coalsack/tensor/dynamic_mx_tensor.h"
#include "coalsack/tensor/dynamic_tensor.h"

namespace coalsack {

class moe_weight_provider {
 public:
  using value = std::variant<dynamic_tensor, dynamic_mx_tensor>;
  void put(const std::string& tensor_name, int expert_id, value v) { map_[{tensor_name, expert_id}] = std::move(v); }
  value get(const std::string& tensor_name, int expert_id) {
    ++gets_;
    auto it = map_.find({tensor_name, expert_id});
    if (it == map_.end()) throw std::runtime_error("moe_weight_provider: no tensor " + tensor_name + " for expert " + std::to_string(expert_id));
    return it->second;
  }
  bool has_tensor(const std::string& tensor_name) const { return map_.lower_bound({tensor_name, 0}) != map_.end(); }
  size_t gets() const { return gets_; }

 private:
  std::map<std::pair<std::string, int>, value> map_;
  size_t gets_ = 0;
};

}  // namespace coalsack
