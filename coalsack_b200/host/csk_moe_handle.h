// RAII helpers shared by the coalsack-side operator bindings: a device layer
// handle that is (re)created when its shape changes, and the translation of a
// C-ABI status into the exception the operators' own envelope expects.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>

#include "csk_moe.h"

namespace coalsack {
namespace csk_host {

inline void check(int rc, csk_moe_layer* h) {
  if (rc != CSK_OK) throw std::runtime_error(csk_moe_last_error(h));
}

class layer_handle {
 public:
  layer_handle() = default;
  layer_handle(const layer_handle&) = delete;
  layer_handle& operator=(const layer_handle&) = delete;
  ~layer_handle() { reset(); }

  // Returns a handle for this configuration, creating a new one if anything changed
  // (max_tokens only ever grows).
  csk_moe_layer* get(const csk_moe_config& want) {
    const bool same = h_ && want.num_experts == cfg_.num_experts && want.top_k == cfg_.top_k &&
                      want.hidden == cfg_.hidden && want.ffn == cfg_.ffn && want.activation == cfg_.activation &&
                      want.has_bias == cfg_.has_bias && want.sigmoid_gating == cfg_.sigmoid_gating &&
                      want.weight_before_ffn == cfg_.weight_before_ffn && want.expert_begin == cfg_.expert_begin &&
                      want.expert_count == cfg_.expert_count && want.max_tokens <= cfg_.max_tokens;
    if (!same) {
      reset();
      cfg_ = want;
      if (int rc = csk_moe_create(&cfg_, &h_)) {
        h_ = nullptr;
        throw std::runtime_error(csk_moe_last_error(nullptr));
      }
      created_ = true;
    } else {
      created_ = false;
    }
    return h_;
  }
  bool just_created() const { return created_; }
  void reset() {
    if (h_) csk_moe_destroy(h_);
    h_ = nullptr;
  }

 private:
  csk_moe_layer* h_ = nullptr;
  csk_moe_config cfg_{};
  bool created_ = false;
};

}  // namespace csk_host
}  // namespace coalsack
