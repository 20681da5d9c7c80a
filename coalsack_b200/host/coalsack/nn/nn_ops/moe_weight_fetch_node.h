// GPU binding of coalsack's expert weight fetch operator; takes the place of
// include/coalsack/nn/nn_ops/moe_weight_fetch_node.h (same constructor, set_has_bias,
// add_expert_output and field names).
//
// Strict mode (default): what the reference does -- for every expert a frame selected, the
// three weight matrices (MXFP4 blocks, or the FLOAT16 tensors the provider makes of Q4_K / Q6_K /
// F16 slices) and biases from the moe_weight_provider travel to that expert's
// node; unselected experts get {0}-shaped tensors (moe_weight_fetch_node.h:162-218).
//
// Fused mode (csk_host::set_fused_moe): the layer's weights live on the GPU.  Only the
// selected experts that are NOT resident yet are pulled from the provider and uploaded
// (csk_moe_load_expert_mxfp4 or csk_moe_load_expert_f16, one repack each); every expert node gets {0}-shaped
// placeholders plus the router output, i.e. a few bytes instead of 13 MB of host tensors.
#pragma once

#include <spdlog/spdlog.h>

#include <memory>
#include <set>
#include <string>
#include <unordered_map>

#include "coalsack/core/graph_edge.h"
#include "coalsack/core/graph_node.h"
#include "coalsack/llm/moe_weight_provider.h"
#include "coalsack/nn/nn_op_node.h"
#include "coalsack/nn/result_message.h"
#include "coalsack/tensor/dynamic_mx_tensor_message.h"
#include "coalsack/tensor/dynamic_tensor.h"
#include "coalsack/tensor/dynamic_tensor_message.h"
#include "csk_moe_handle.h"

namespace coalsack {

class moe_weight_fetch_node : public graph_node {
 public:
  moe_weight_fetch_node(std::shared_ptr<moe_weight_provider> provider, const std::string& layer_prefix)
      : graph_node(), weight_provider_(std::move(provider)), layer_prefix_(layer_prefix) {
    if (!weight_provider_) throw std::invalid_argument("weight_provider cannot be null");
  }

  void set_has_bias(bool has_bias) { has_bias_ = has_bias; }
  bool get_has_bias() const { return has_bias_; }
  std::string get_proc_name() const override { return "moe_weight_fetch_node"; }

  graph_edge_ptr add_expert_output(int expert_id) {
    auto it = expert_outputs_.find(expert_id);
    if (it != expert_outputs_.end()) return it->second;
    auto edge = std::make_shared<graph_edge>(this);
    edge->set_name("expert_" + std::to_string(expert_id));
    expert_outputs_[expert_id] = edge;
    set_output(edge, "expert_" + std::to_string(expert_id));
    return edge;
  }

  void process(std::string, graph_message_ptr message) override {
    auto in = std::dynamic_pointer_cast<result_message>(message);
    if (!in) return;
    const uint64_t frame = in->get_frame_number();
    const double stamp = in->get_timestamp();
    auto send = [&](const graph_edge_ptr& edge, std::shared_ptr<result_message> m) {
      m->set_frame_number(frame);
      m->set_timestamp(stamp);
      edge->send(m);
    };
    auto fields_of = [&](int expert_id, const graph_message_ptr& weights, const graph_message_ptr& router) {
      std::unordered_map<std::string, graph_message_ptr> f;
      const std::string ep = layer_prefix_ + ".expert_" + std::to_string(expert_id);
      for (const char* n : {".w_up", ".w_gate", ".w_down"}) f[ep + n] = weights;
      if (has_bias_)
        for (const char* n : {".b_up", ".b_gate", ".b_down"}) f[ep + n] = weights;
      f[ep + ".router_out"] = router;
      return f;
    };
    auto fail_all = [&](const std::string& what) {
      for (const auto& [id, edge] : expert_outputs_) send(edge, result_message::error(fields_of(id, nullptr, nullptr), what));
    };
    if (!in->is_ok()) return fail_all("Input error");

    dynamic_tensor router;
    std::shared_ptr<dynamic_tensor_message> router_msg;
    std::set<int> selected;
    try {
      router = get_tensor_from_result_message(in, layer_prefix_ + ".router_out");
      router_msg = std::make_shared<dynamic_tensor_message>(router);
      if (router.ndim() == 4 && router.dim(3) == 2) {
        const float* r = router.data_ptr<float>();
        const int64_t n = router.dim(0) * router.dim(1) * router.dim(2);
        for (int64_t i = 0; i < n; ++i) selected.insert(static_cast<int>(r[2 * i]));
      }
    } catch (const std::exception& e) {
      spdlog::error("moe_weight_fetch_node [{}]: {}", layer_prefix_, e.what());
      return fail_all(e.what());
    }
    auto empty = std::make_shared<dynamic_tensor_message>(dynamic_tensor(dtype::float32, {0}));

    if (csk_host::fused_moe()) {
      std::string err;
      if (make_resident(router, selected, err)) {
        for (const auto& [id, edge] : expert_outputs_) send(edge, result_message::ok(fields_of(id, empty, router_msg)));
        return;
      }
      if (!err.empty()) {
        spdlog::error("moe_weight_fetch_node [{}]: {}", layer_prefix_, err);
        return fail_all(err);
      }
      // weights the fused path does not take (fp32, odd sizes): this layer goes the strict way below
    }

    auto to_message = [](const auto& v) -> graph_message_ptr {
      if (std::holds_alternative<dynamic_tensor>(v)) {
        auto m = std::make_shared<dynamic_tensor_message>();
        m->set_tensor(std::get<dynamic_tensor>(v));
        return m;
      }
      auto m = std::make_shared<dynamic_mx_tensor_message>();
      m->set_mx_tensor(std::get<dynamic_mx_tensor>(v));
      return m;
    };
    for (const auto& [id, edge] : expert_outputs_) {
      if (!selected.count(id)) {
        send(edge, result_message::ok(fields_of(id, empty, router_msg)));
        continue;
      }
      std::shared_ptr<result_message> out;
      try {
        const std::string ep = layer_prefix_ + ".expert_" + std::to_string(id);
        std::unordered_map<std::string, graph_message_ptr> f;
        f[ep + ".w_up"] = to_message(weight_provider_->get(layer_prefix_ + ".ffn_up_exps.weight", id));
        f[ep + ".w_gate"] = to_message(weight_provider_->get(layer_prefix_ + ".ffn_gate_exps.weight", id));
        f[ep + ".w_down"] = to_message(weight_provider_->get(layer_prefix_ + ".ffn_down_exps.weight", id));
        if (has_bias_) {
          f[ep + ".b_up"] = to_message(weight_provider_->get(layer_prefix_ + ".ffn_up_exps.bias", id));
          f[ep + ".b_gate"] = to_message(weight_provider_->get(layer_prefix_ + ".ffn_gate_exps.bias", id));
          f[ep + ".b_down"] = to_message(weight_provider_->get(layer_prefix_ + ".ffn_down_exps.bias", id));
        }
        f[ep + ".router_out"] = router_msg;
        out = result_message::ok(f);
      } catch (const std::exception& e) {
        spdlog::error("moe_weight_fetch_node [{}] expert {}: {}", layer_prefix_, id, e.what());
        out = result_message::error(fields_of(id, nullptr, nullptr), e.what());
      }
      send(edge, out);
    }
  }

 private:
  // Fused mode: the layer's device handle exists and holds every selected expert.  Returns false with an
  // empty `err` when the provider's tensors are neither MXFP4 nor FLOAT16 (the caller then goes the strict way).
  bool make_resident(const dynamic_tensor& router, const std::set<int>& selected, std::string& err) {
    auto ctx = csk_host::layer_registry::get(layer_prefix_);
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->usable = false;
    ctx->have_hidden = false;
    try {
      if (router.ndim() != 4 || router.dim(3) != 2) throw std::runtime_error("router output must be [batch, seq_len, top_k, 2]");
      const int E = static_cast<int>(expert_outputs_.size());
      const int64_t tokens = router.dim(0) * router.dim(1);
      for (int id : selected) {
        if (id < 0 || id >= E) throw std::runtime_error("expert_idx out of range: " + std::to_string(id));
      }
      if (selected.empty()) throw std::runtime_error("router output selects no expert");
      // shapes come from the first selected expert's up projection [F, H]
      auto up0 = weight_provider_->get(layer_prefix_ + ".ffn_up_exps.weight", *selected.begin());
      // MXFP4 blocks, or the FLOAT16 matrices the provider makes of Q4_K / Q6_K / F16 slices
      const bool is_mx = std::holds_alternative<dynamic_mx_tensor>(up0);
      int64_t dim_f = 0, dim_h = 0;
      if (is_mx) {
        const dynamic_mx_tensor& u = std::get<dynamic_mx_tensor>(up0);
        if (u.ndim() != 2) throw std::runtime_error("expert weights must be 2D");
        dim_f = u.dim(0);
        dim_h = u.dim(1);
      } else {
        const dynamic_tensor& u = std::get<dynamic_tensor>(up0);
        // anything else (fp32 weights, sizes the tensor-core tiles do not take) goes the strict way,
        // where the expert node answers with the reference's own message
        if (u.get_dtype() != dtype::float16 || u.ndim() != 2 || u.dim(0) % 32 || u.dim(1) % 32) return false;
        dim_f = u.dim(0);
        dim_h = u.dim(1);
      }
      csk_moe_config c{};
      c.num_experts = E;
      c.top_k = static_cast<int32_t>(router.dim(2));
      c.hidden = static_cast<int32_t>(dim_h);
      c.ffn = static_cast<int32_t>(dim_f);
      c.weight_format = is_mx ? CSK_WEIGHTS_MXFP4 : CSK_WEIGHTS_F16;
      c.activation = CSK_ACT_MODIFIED_SWIGLU;  // the merge node sets what the expert nodes were configured with
      c.has_bias = has_bias_;
      c.weight_before_ffn = 0;
      c.max_tokens = std::max<int64_t>(tokens, ctx->cfg.max_tokens ? ctx->cfg.max_tokens : 64);
      csk_moe_layer* h = ctx->handle.get(c);
      if (ctx->handle.just_created()) ctx->resident_gen.assign(E, 0);
      ctx->cfg = c;
      for (int id : selected) {
        if (ctx->resident_gen[id] == ctx->generation) continue;
        auto mx = [&](const char* name) -> dynamic_mx_tensor {
          auto v = weight_provider_->get(layer_prefix_ + name, id);
          if (!std::holds_alternative<dynamic_mx_tensor>(v)) throw std::runtime_error(std::string(name) + " is not MXFP4");
          return std::get<dynamic_mx_tensor>(v);
        };
        auto plain = [&](const char* name) -> dynamic_tensor {
          auto v = weight_provider_->get(layer_prefix_ + name, id);
          if (!std::holds_alternative<dynamic_tensor>(v)) throw std::runtime_error(std::string(name) + " is not a plain tensor");
          return std::get<dynamic_tensor>(v);
        };
        dynamic_tensor bu, bg, bd;
        if (has_bias_) {
          bu = plain(".ffn_up_exps.bias");
          bg = plain(".ffn_gate_exps.bias");
          bd = plain(".ffn_down_exps.bias");
        }
        const float* pbu = has_bias_ ? bu.data_ptr<float>() : nullptr;
        const float* pbg = has_bias_ ? bg.data_ptr<float>() : nullptr;
        const float* pbd = has_bias_ ? bd.data_ptr<float>() : nullptr;
        auto dims_ok = [&](const auto& up, const auto& gate, const auto& down) {
          return up.ndim() == 2 && gate.ndim() == 2 && down.ndim() == 2 && up.dim(0) == c.ffn && up.dim(1) == c.hidden &&
                 gate.dim(0) == c.ffn && gate.dim(1) == c.hidden && down.dim(0) == c.hidden && down.dim(1) == c.ffn;
        };
        if (is_mx) {
          const dynamic_mx_tensor up = mx(".ffn_up_exps.weight"), gate = mx(".ffn_gate_exps.weight"), down = mx(".ffn_down_exps.weight");
          if (!dims_ok(up, gate, down)) throw std::runtime_error("expert_mlp: weight dimension mismatch");
          csk_host::check(csk_moe_load_expert_mxfp4(h, id, up.data_ptr(), gate.data_ptr(), down.data_ptr(), pbu, pbg, pbd), h);
        } else {
          const dynamic_tensor up = plain(".ffn_up_exps.weight"), gate = plain(".ffn_gate_exps.weight"), down = plain(".ffn_down_exps.weight");
          if (!dims_ok(up, gate, down)) throw std::runtime_error("expert_mlp: weight dimension mismatch");
          if (up.get_dtype() != dtype::float16 || gate.get_dtype() != dtype::float16 || down.get_dtype() != dtype::float16)
            throw std::runtime_error("expert_mlp: all weights must be FLOAT16");
          csk_host::check(csk_moe_load_expert_f16(h, id, up.data_ptr<uint16_t>(), gate.data_ptr<uint16_t>(),
                                                  down.data_ptr<uint16_t>(), pbu, pbg, pbd),
                          h);
        }
        ctx->resident_gen[id] = ctx->generation;
      }
      ctx->usable = true;
      return true;
    } catch (const std::exception& e) {
      err = e.what();
      return false;
    }
  }

  std::shared_ptr<moe_weight_provider> weight_provider_;
  std::string layer_prefix_;
  std::unordered_map<int, graph_edge_ptr> expert_outputs_;
  bool has_bias_{true};
};

}  // namespace coalsack
