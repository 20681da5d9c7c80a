// GPU binding of coalsack's MoE router operator.  Placed ahead of the reference's
// include directory it takes the place of include/coalsack/nn/nn_ops/moe_router_node.h:
// same class name, setters, inputs (hidden_states [B,S,H], gate_weights [E,H],
// optional gate_bias [E]) and output ([B,S,k,2] = expert id as float, weight);
// the arithmetic runs in libcsk_moe.so (csk_moe_route).
#pragma once

#include <string>
#include <vector>

#include "coalsack/nn/nn_op_node.h"
#include "csk_moe_handle.h"

namespace coalsack {

class moe_router_node : public variadic_op_node {
 public:
  moe_router_node() : variadic_op_node("moe_router", 3) {}

  void set_config(int64_t num_experts, int64_t top_k) {
    num_experts_ = num_experts;
    top_k_ = top_k;
  }
  void set_sigmoid_gating(bool v) { use_sigmoid_gating_ = v; }

  dynamic_tensor compute_test(const dynamic_tensor& hidden_states, const dynamic_tensor& gate_weights,
                              const dynamic_tensor& gate_bias) {
    return compute({hidden_states, gate_weights, gate_bias});
  }
  dynamic_tensor compute_test(const dynamic_tensor& hidden_states, const dynamic_tensor& gate_weights) {
    return compute({hidden_states, gate_weights});
  }

 protected:
  dynamic_tensor compute(const std::vector<dynamic_tensor>& in) override {
    if (in.size() != 2 && in.size() != 3)
      throw std::runtime_error(
          "moe_router: expected 2 or 3 inputs (hidden_states, gate_weights[, gate_bias]), got " +
          std::to_string(in.size()));
    const dynamic_tensor& hidden = in[0];
    const dynamic_tensor& gate = in[1];
    const bool biased = in.size() == 3;
    if (hidden.ndim() != 3)
      throw std::runtime_error("moe_router: hidden_states must be 3D [batch, seq_len, hidden_dim], got " +
                               std::to_string(hidden.ndim()) + "D");
    if (gate.ndim() != 2)
      throw std::runtime_error("moe_router: gate_weights must be 2D [num_experts, hidden_dim], got " +
                               std::to_string(gate.ndim()) + "D");
    if (biased && in[2].ndim() != 1)
      throw std::runtime_error("moe_router: gate_bias must be 1D [num_experts], got " +
                               std::to_string(in[2].ndim()) + "D");
    const int64_t B = hidden.dim(0), S = hidden.dim(1), H = hidden.dim(2);
    if (gate.dim(0) != num_experts_ || gate.dim(1) != H)
      throw std::runtime_error("moe_router: gate_weights shape mismatch, expected [" + std::to_string(num_experts_) +
                               ", " + std::to_string(H) + "], got [" + std::to_string(gate.dim(0)) + ", " +
                               std::to_string(gate.dim(1)) + "]");
    if (biased && in[2].dim(0) != num_experts_)
      throw std::runtime_error("moe_router: gate_bias must have num_experts=" + std::to_string(num_experts_) +
                               " elements, got " + std::to_string(in[2].dim(0)));
    if (hidden.get_dtype() != dtype::float32)
      throw std::runtime_error("moe_router: only float32 is supported on the GPU");
    if (H % 32) throw std::runtime_error("moe_router: hidden_dim must be a multiple of 32 on the GPU");

    csk_moe_config c{};
    c.num_experts = (int32_t)num_experts_;
    c.top_k = (int32_t)top_k_;
    c.hidden = (int32_t)H;
    c.ffn = 32;  // the router-only handle carries no experts
    c.sigmoid_gating = use_sigmoid_gating_;
    c.max_tokens = B * S;
    csk_moe_layer* h = handle_.get(c);
    // router weights are constants of the model: upload when the buffer OR its contents change (a
    // checkpoint reloaded into the same allocation keeps the address; the reference reads the tensors
    // on every call, so a stale copy on the GPU would be a silent difference)
    const float* w = gate.data_ptr<float>();
    const float* b = biased ? in[2].data_ptr<float>() : nullptr;
    const uint64_t sum = csk_host::content_hash(w, sizeof(float) * num_experts_ * H) ^
                         (biased ? csk_host::content_hash(b, sizeof(float) * num_experts_) * 0x9E3779B97F4A7C15ull : 0);
    if (handle_.just_created() || w != last_w_ || b != last_b_ || sum != last_sum_) {
      csk_host::check(csk_moe_set_router(h, w, b), h);
      last_w_ = w;
      last_b_ = b;
      last_sum_ = sum;
    }
    dynamic_tensor out(dtype::float32, {B, S, top_k_, 2});
    csk_host::check(csk_moe_route(h, hidden.data_ptr<float>(), B * S, out.data_ptr<float>()), h);
    return out;
  }

 private:
  int64_t num_experts_ = 0, top_k_ = 0;
  bool use_sigmoid_gating_ = false;
  csk_host::layer_handle handle_;
 public:
  // Forget the uploaded router weights (after an in-place edit the sampled content check could miss).
  void invalidate_weights() { last_w_ = nullptr; }

 private:
  const float* last_w_ = nullptr;
  const float* last_b_ = nullptr;
  uint64_t last_sum_ = 0;
};

}  // namespace coalsack

COALSACK_REGISTER_NODE(coalsack::moe_router_node, coalsack::graph_node)
