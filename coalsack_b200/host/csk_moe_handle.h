// RAII helpers shared by the coalsack-side operator bindings: a device layer
// handle that is (re)created when its shape changes, and the translation of a
// C-ABI status into the exception the operators' own envelope expects.
#pragma once

#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "coalsack/tensor/dynamic_tensor.h"
#include "csk_moe.h"

namespace coalsack {
namespace csk_host {

inline void check(int rc, csk_moe_layer* h) {
  if (rc != CSK_OK) throw std::runtime_error(csk_moe_last_error(h));
}

// 64-bit mix over every 16th eight-byte word of a buffer (a 1.5 MB gate matrix costs about 20 us):
// enough to notice that a weight buffer was reloaded in place (a reload rewrites nearly every word);
// an edit confined to words the sample skips goes unnoticed -- call the node's invalidate hook then.
inline uint64_t content_hash(const void* p, size_t bytes) {
  const unsigned char* c = static_cast<const unsigned char*>(p);
  uint64_t h = 0xCBF29CE484222325ull ^ bytes;
  for (size_t i = 0; i + 8 <= bytes; i += 128) {
    uint64_t w;
    std::memcpy(&w, c + i, 8);
    h = (h ^ w) * 0x100000001B3ull;
    h ^= h >> 29;
  }
  if (bytes >= 8) {
    uint64_t w;
    std::memcpy(&w, c + bytes - 8, 8);
    h = (h ^ w) * 0x100000001B3ull;
  }
  return h;
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
                      want.expert_count == cfg_.expert_count && want.weight_format == cfg_.weight_format &&
                      want.max_tokens <= cfg_.max_tokens;
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

// ---------------------------------------------------------------------------
// Fused mode: the graph keeps coalsack's topology (router -> weight fetch -> E expert
// nodes -> merge), but the heavy work of a layer is ONE csk_moe_forward call issued by
// the merge node.  The nodes of a layer meet in a per-layer context found by the
// layer's name prefix ("blk.7"): the fetch node uploads the experts a frame selects
// that are not resident yet, the expert nodes pass the hidden states along and answer
// with the {0}-shaped placeholder, the merge node (which coalsack's sync node fires
// once per frame, when all E expert messages have arrived) runs the layer.
//
// Off by default: the strict mode (one csk_moe_expert_forward per expert node, dense
// outputs with zero rows exactly like the reference) is what the parity tests use.
// set_fused_moe(true), or CSK_MOE_FUSED=1 in the environment, switches it on.
// ---------------------------------------------------------------------------
inline std::atomic<int>& fused_flag() {
  static std::atomic<int> f{-1};
  return f;
}
inline void set_fused_moe(bool on) { fused_flag().store(on ? 1 : 0); }
inline bool fused_moe() {
  int v = fused_flag().load();
  if (v < 0) {
    const char* e = std::getenv("CSK_MOE_FUSED");
    v = (e && e[0] == '1') ? 1 : 0;
    fused_flag().store(v);
  }
  return v == 1;
}

struct moe_layer_context {
  std::mutex mu;
  layer_handle handle;
  csk_moe_config cfg{};
  bool usable = false;          // a handle exists and every expert this frame needs is resident
  std::vector<uint64_t> resident_gen;  // per expert: generation it was uploaded at (0 = not resident)
  uint64_t generation = 1;      // bumped by invalidate(): experts are uploaded again on next use
  dynamic_tensor hidden;        // the frame's hidden states, left by the first expert node to see them
  bool have_hidden = false;
  int activation = CSK_ACT_MODIFIED_SWIGLU;
  bool weight_before_ffn = false;
};

class layer_registry {
 public:
  static std::shared_ptr<moe_layer_context> get(const std::string& prefix) {
    static std::mutex mu;
    static std::unordered_map<std::string, std::shared_ptr<moe_layer_context>> map;
    std::lock_guard<std::mutex> lk(mu);
    auto& slot = map[prefix];
    if (!slot) slot = std::make_shared<moe_layer_context>();
    return slot;
  }
  // Weights of this layer changed in place (another checkpoint at the same addresses): upload again.
  static void invalidate(const std::string& prefix) {
    auto c = get(prefix);
    std::lock_guard<std::mutex> lk(c->mu);
    ++c->generation;
  }
};

// "blk.7.expert_12.w_up" / "blk.7.expert_12_out" -> "blk.7"; empty when the name has no ".expert_" part.
inline std::string layer_prefix_of(const std::string& name) {
  const size_t p = name.rfind(".expert_");
  return p == std::string::npos ? std::string() : name.substr(0, p);
}

}  // namespace csk_host
}  // namespace coalsack
