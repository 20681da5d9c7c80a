// GPU binding of coalsack's expert merge operator; takes the place of
// include/coalsack/nn/nn_ops/expert_merge_node.h.  Inputs: router output
// [B,S,k,2] then one tensor per expert ([B,S,H], or {0}-shaped for an expert no
// token selected); output [B,S,H] = sum over the k slots, in router order, of
// weight * expert row (csk_moe_merge).
#pragma once

#include <string>
#include <vector>

#include "coalsack/nn/nn_op_node.h"
#include "csk_moe_handle.h"

namespace coalsack {

class expert_merge_node : public variadic_op_node {
 public:
  expert_merge_node() : variadic_op_node("expert_merge", 33) {}

  void set_config(int64_t num_experts, int64_t top_k) {
    num_experts_ = num_experts;
    top_k_ = top_k;
  }
  void set_weight_before_ffn(bool v) { weight_before_ffn_ = v; }
  dynamic_tensor compute_test(const std::vector<dynamic_tensor>& inputs) { return compute(inputs); }

 protected:
  dynamic_tensor compute(const std::vector<dynamic_tensor>& in) override {
    if (in.size() != static_cast<size_t>(num_experts_ + 1))
      throw std::runtime_error("expert_merge: expected " + std::to_string(num_experts_ + 1) + " inputs, got " +
                               std::to_string(in.size()));
    const dynamic_tensor& router = in[0];
    if (router.ndim() != 4 || router.dim(2) != top_k_ || router.dim(3) != 2)
      throw std::runtime_error("expert_merge: router output must have shape [batch, seq_len, " +
                               std::to_string(top_k_) + ", 2]");
    if (router.get_dtype() != dtype::float32) throw std::runtime_error("expert_merge: only float32 supported");
    const int64_t B = router.dim(0), S = router.dim(1);
    {
      dynamic_tensor fused;
      if (run_fused(router, fused)) return fused;
    }
    int64_t H = 0;
    std::vector<const float*> rows(num_experts_, nullptr);
    for (int64_t e = 0; e < num_experts_; ++e) {
      const dynamic_tensor& t = in[1 + e];
      if (t.ndim() != 3 || t.dim(0) == 0) continue;  // the empty tensor of an unselected expert
      if (H == 0) H = t.dim(2);
      if (t.dim(0) != B || t.dim(1) != S || t.dim(2) != H)
        throw std::runtime_error("expert_merge: all non-empty expert outputs must have same shape");
      rows[e] = t.data_ptr<float>();
    }
    if (H == 0) throw std::runtime_error("expert_merge: no non-empty expert outputs found");
    if (H % 32) throw std::runtime_error("expert_merge: hidden_dim must be a multiple of 32 on the GPU");

    csk_moe_config c{};
    c.num_experts = (int32_t)num_experts_;
    c.top_k = (int32_t)top_k_;
    c.hidden = (int32_t)H;
    c.ffn = 32;
    c.weight_before_ffn = weight_before_ffn_;
    c.max_tokens = B * S;
    csk_moe_layer* h = handle_.get(c);
    dynamic_tensor out(dtype::float32, {B, S, H});
    csk_host::check(csk_moe_merge(h, router.data_ptr<float>(), B * S, rows.data(), out.data_ptr<float>()), h);
    return out;
  }

 private:
  // Fused mode: the layer's context holds the frame's hidden states and every selected expert's weights
  // on the GPU: the whole layer (dispatch, grouped MXFP4 MLP, weighted combine in router order) is one
  // csk_moe_forward with the routing this node was given.
  bool run_fused(const dynamic_tensor& router, dynamic_tensor& out) {
    if (!csk_host::fused_moe() || input_names_.size() < 2) return false;
    const std::string prefix = csk_host::layer_prefix_of(input_names_[1]);
    if (prefix.empty()) return false;
    auto ctx = csk_host::layer_registry::get(prefix);
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (!ctx->usable || !ctx->have_hidden) return false;
    const dynamic_tensor& hidden = ctx->hidden;
    const int64_t B = router.dim(0), S = router.dim(1);
    if (hidden.ndim() != 3 || hidden.dim(0) != B || hidden.dim(1) != S || hidden.dim(2) != ctx->cfg.hidden)
      throw std::runtime_error("expert_merge: hidden states and router output disagree in shape");
    csk_moe_layer* h = ctx->handle.get(ctx->cfg);
    csk_host::check(csk_moe_set_activation(h, ctx->activation, ctx->weight_before_ffn), h);
    out = dynamic_tensor(dtype::float32, {B, S, hidden.dim(2)});
    const int rc = csk_moe_forward(h, hidden.data_ptr<float>(), B * S, router.data_ptr<float>(), nullptr, out.data_ptr<float>());
    ctx->have_hidden = false;
    ctx->hidden = dynamic_tensor();
    csk_host::check(rc, h);
    return true;
  }

  int64_t num_experts_ = 0, top_k_ = 0;
  bool weight_before_ffn_ = false;
  csk_host::layer_handle handle_;
};

}  // namespace coalsack

COALSACK_REGISTER_NODE(coalsack::expert_merge_node, coalsack::graph_node)
