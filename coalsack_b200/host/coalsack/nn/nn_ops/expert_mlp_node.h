// GPU binding of coalsack's expert MLP operator; takes the place of
// include/coalsack/nn/nn_ops/expert_mlp_node.h.  One node = one expert: from a
// result_message carrying hidden_states [B,S,H], w_up/w_gate [F,H] and w_down
// [H,F] -- MXFP4 blocks as dynamic_mx_tensor messages, or FLOAT16 matrices as
// dynamic_tensor messages (what the weight provider makes of Q4_K / Q6_K / F16
// expert slices) -- optional fp32 biases and the router output [B,S,k,2] it
// emits the dense [B,S,H] output of this expert (zero rows for tokens that did
// not select it), or a {0}-shaped tensor when no token selected it.  Weights are
// repacked and uploaded once per weight buffer (csk_moe_load_expert_mxfp4 /
// csk_moe_load_expert_f16); the forward is csk_moe_expert_forward.
// In fused mode (csk_moe_handle.h) the node only passes the hidden states along and
// answers with the {0}-shaped placeholder; the merge node runs the whole layer.
#pragma once

#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "coalsack/nn/nn_op_node.h"
#include "coalsack/tensor/dynamic_mx_tensor_message.h"
#include "csk_moe_handle.h"

namespace coalsack {

class expert_mlp_node : public graph_node {
 public:
  enum class activation_type { MODIFIED_SWIGLU, STANDARD_SWIGLU };

  explicit expert_mlp_node(int expert_id = 0)
      : graph_node(), expert_id_(expert_id), output_(std::make_shared<graph_edge>(this)) {
    set_output(output_);
  }

  int get_expert_id() const { return expert_id_; }
  std::string get_proc_name() const override { return "expert_mlp"; }
  void set_input_names(const std::vector<std::string>& names) { input_names_ = names; }
  void set_output_name(const std::string& name) { output_name_ = name; }
  void set_node_name(const std::string& name) { node_name_ = name; }
  void set_activation_type(activation_type t) { activation_type_ = t; }
  activation_type get_activation_type() const { return activation_type_; }
  void set_weight_before_ffn(bool v) { weight_before_ffn_ = v; }
  std::vector<std::string> get_input_names() const { return input_names_; }
  std::string get_output_name() const { return output_name_; }

  // The FLOAT16-weight operator on plain tensors (the reference's test wrapper of the same name):
  // hidden, w_up, w_gate, w_down[, b_up, b_gate, b_down], router_output.
  dynamic_tensor compute_test(const std::vector<dynamic_tensor>& inputs) { return run_f16(inputs); }

  // One token through this expert with raw 17-byte-block weights.
  void compute_test_mxfp4(const float* hidden_vec, const uint8_t* w_up, const uint8_t* w_gate, const uint8_t* w_down,
                          const float* b_up, const float* b_gate, const float* b_down, float* output_vec,
                          int64_t hidden_dim, int64_t expert_ffn_dim) {
    const float router[2] = {static_cast<float>(expert_id_), 1.0f};
    int32_t selected = 0;
    csk_moe_layer* h = layer_for(hidden_dim, expert_ffn_dim, b_up != nullptr, 1, expert_id_ + 1, 1);
    upload(h, w_up, w_gate, w_down, b_up, b_gate, b_down);
    csk_host::check(csk_moe_expert_forward(h, expert_id_, hidden_vec, 1, router, output_vec, &selected), h);
  }

  void process(std::string, graph_message_ptr message) override {
    auto in = std::dynamic_pointer_cast<result_message>(message);
    const uint64_t frame = in ? in->get_frame_number() : 0;
    const double stamp = in ? in->get_timestamp() : 0.0;
    std::shared_ptr<result_message> out;
    if (in && !in->is_ok()) {
      out = result_message::error({{output_name_, nullptr}}, "Input error");
    } else {
      try {
        if (!in || input_names_.empty()) throw std::runtime_error("expert_mlp: invalid input");
        std::vector<graph_message_ptr> fields;
        for (const auto& name : input_names_) {
          auto f = in->get_field(name);
          if (!f) throw std::runtime_error("expert_mlp: missing field " + name);
          fields.push_back(f);
        }
        if (pass_along(fields)) {
          // fused mode: the layer runs once, in the merge node; this node answers with the placeholder
          out = result_message::ok({{output_name_, std::make_shared<dynamic_tensor_message>(dynamic_tensor(dtype::float32, {0}))}});
          out->set_frame_number(frame);
          out->set_timestamp(stamp);
          output_->send(out);
          return;
        }
        dynamic_tensor result;
        if (std::dynamic_pointer_cast<dynamic_mx_tensor_message>(fields[1])) {
          result = run_mxfp4(fields);
        } else {
          // plain tensors: FLOAT16 weights, or what the fetch node sends to an expert no token selected
          // ({0}-shaped); the reference answers the latter with the {0}-shaped tensor before it looks at
          // any weight (expert_mlp_node.h:296-302), and so does run_f16
          std::vector<dynamic_tensor> inputs;
          for (const auto& m : fields) {
            auto t = std::dynamic_pointer_cast<dynamic_tensor_message>(m);
            if (!t) throw std::runtime_error("expert_mlp: expected dynamic_tensor_message");
            inputs.push_back(t->get_tensor());
          }
          result = run_f16(inputs);
        }
        auto tensor = std::make_shared<dynamic_tensor_message>(result);
        out = result_message::ok({{output_name_, tensor}});
      } catch (const std::exception& e) {
        spdlog::error("{} [{}]: {}", "expert_mlp", node_name_, e.what());
        out = result_message::error({{output_name_, nullptr}}, e.what());
      }
    }
    out->set_frame_number(frame);
    out->set_timestamp(stamp);
    output_->send(out);
  }

 private:
  template <class T>
  static std::shared_ptr<T> as(const graph_message_ptr& m, const char* what) {
    auto p = std::dynamic_pointer_cast<T>(m);
    if (!p) throw std::runtime_error(std::string("expert_mlp: invalid ") + what + " message type for MXFP4");
    return p;
  }

  // FLOAT16 weights: the checks, their order and texts are compute_fp16's (expert_mlp_node.h:269-389).
  dynamic_tensor run_f16(const std::vector<dynamic_tensor>& in) {
    if (in.size() != 5 && in.size() != 8)
      throw std::runtime_error(
          "expert_mlp: expected 5 or 8 inputs (hidden, w_up, w_gate, w_down[, b_up, b_gate, "
          "b_down], router_output), got " +
          std::to_string(in.size()));
    const bool biased = in.size() == 8;
    const dynamic_tensor &hidden = in[0], &up = in[1], &gate = in[2], &down = in[3], &router = in[biased ? 7 : 4];
    if (router.ndim() != 4 || router.dim(3) != 2)
      throw std::runtime_error("expert_mlp: router_output must be 4D [batch, seq_len, top_k, 2], got " +
                               std::to_string(router.ndim()) + "D");
    if (router.get_dtype() != dtype::float32) throw std::runtime_error("expert_mlp: router_output must be float32");
    const float* r = router.data_ptr<float>();
    const int64_t pairs = router.dim(0) * router.dim(1) * router.dim(2), k = router.dim(2);
    bool any = false;
    int max_id = expert_id_;
    for (int64_t i = 0; i < pairs; ++i) {
      const int id = static_cast<int>(r[2 * i]);
      any = any || id == expert_id_;
      if (id > max_id) max_id = id;
    }
    if (!any) return dynamic_tensor(dtype::float32, {0});
    if (hidden.ndim() != 3)
      throw std::runtime_error("expert_mlp: hidden_states must be 3D [batch, seq_len, hidden_dim], got " +
                               std::to_string(hidden.ndim()) + "D");
    const int64_t B = hidden.dim(0), S = hidden.dim(1), H = hidden.dim(2);
    if (up.ndim() != 2 || gate.ndim() != 2 || down.ndim() != 2)
      throw std::runtime_error(
          "expert_mlp: all weights must be 2D [expert_ffn_dim, hidden_dim] or [hidden_dim, "
          "expert_ffn_dim]");
    const int64_t F = up.dim(0);
    auto dims = [](const dynamic_tensor& t) { return "[" + std::to_string(t.dim(0)) + ", " + std::to_string(t.dim(1)) + "]"; };
    const std::string fh = "[" + std::to_string(F) + ", " + std::to_string(H) + "]";
    if (up.dim(1) != H) throw std::runtime_error("expert_mlp: w_up must be " + fh + ", got " + dims(up));
    if (gate.dim(0) != F || gate.dim(1) != H)
      throw std::runtime_error("expert_mlp: w_gate must be " + fh + ", got " + dims(gate));
    if (down.dim(0) != H || down.dim(1) != F)
      throw std::runtime_error("expert_mlp: w_down must be [" + std::to_string(H) + ", " + std::to_string(F) +
                               "], got " + dims(down));
    if (biased) {
      const dynamic_tensor &bu = in[4], &bg = in[5], &bd = in[6];
      if (bu.ndim() != 1 || bu.dim(0) != F)
        throw std::runtime_error("expert_mlp: b_up must be [expert_ffn_dim=" + std::to_string(F) + "], got [" +
                                 std::to_string(bu.dim(0)) + "]");
      if (bg.ndim() != 1 || bg.dim(0) != F)
        throw std::runtime_error("expert_mlp: b_gate must be [expert_ffn_dim=" + std::to_string(F) + "], got [" +
                                 std::to_string(bg.dim(0)) + "]");
      if (bd.ndim() != 1 || bd.dim(0) != H)
        throw std::runtime_error("expert_mlp: b_down must be [hidden_dim=" + std::to_string(H) + "], got [" +
                                 std::to_string(bd.dim(0)) + "]");
    }
    if (up.get_dtype() != dtype::float16 || gate.get_dtype() != dtype::float16 || down.get_dtype() != dtype::float16)
      throw std::runtime_error("expert_mlp: all weights must be FLOAT16");
    if (hidden.get_dtype() != dtype::float32) throw std::runtime_error("expert_mlp: hidden_states must be FLOAT32");
    // the tensor-core kernel's tiles: a limit of this binding, not of the reference
    if (H % 32 || F % 32)
      throw std::runtime_error("expert_mlp: this GPU binding needs hidden_dim and expert_ffn_dim to be multiples of 32, got " +
                               std::to_string(H) + " and " + std::to_string(F));

    csk_moe_layer* h = layer_for(H, F, biased, k, max_id + 1, B * S, CSK_WEIGHTS_F16);
    const void *pu = up.data_ptr<uint16_t>(), *pg = gate.data_ptr<uint16_t>(), *pd = down.data_ptr<uint16_t>();
    if (pu != last_up_ || pg != last_gate_ || pd != last_down_) {
      csk_host::check(csk_moe_load_expert_f16(h, expert_id_, up.data_ptr<uint16_t>(), gate.data_ptr<uint16_t>(),
                                              down.data_ptr<uint16_t>(), biased ? in[4].data_ptr<float>() : nullptr,
                                              biased ? in[5].data_ptr<float>() : nullptr,
                                              biased ? in[6].data_ptr<float>() : nullptr),
                      h);
      last_up_ = pu;
      last_gate_ = pg;
      last_down_ = pd;
    }
    dynamic_tensor out(dtype::float32, hidden.shape());
    int32_t selected = 0;
    csk_host::check(csk_moe_expert_forward(h, expert_id_, hidden.data_ptr<float>(), B * S, r, out.data_ptr<float>(),
                                           &selected),
                    h);
    return out;
  }

  // Fused mode: true when this layer's context took over the frame (the fetch node made the selected
  // experts resident).  The first expert node of a frame leaves the hidden states there for the merge node.
  bool pass_along(const std::vector<graph_message_ptr>& f) {
    if (!csk_host::fused_moe() || input_names_.size() < 2) return false;
    const std::string prefix = csk_host::layer_prefix_of(input_names_[1]);
    if (prefix.empty()) return false;
    auto ctx = csk_host::layer_registry::get(prefix);
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (!ctx->usable) return false;
    ctx->activation = activation_type_ == activation_type::MODIFIED_SWIGLU ? CSK_ACT_MODIFIED_SWIGLU : CSK_ACT_STANDARD_SWIGLU;
    ctx->weight_before_ffn = weight_before_ffn_;
    if (!ctx->have_hidden) {
      ctx->hidden = as<dynamic_tensor_message>(f[0], "input")->get_tensor();
      ctx->have_hidden = true;
    }
    return true;
  }

  dynamic_tensor run_mxfp4(const std::vector<graph_message_ptr>& f) {
    if (f.size() != 5 && f.size() != 8)
      throw std::runtime_error("expert_mlp: expected 5 or 8 inputs for MXFP4, got " + std::to_string(f.size()));
    const bool biased = f.size() == 8;
    const dynamic_tensor& hidden = as<dynamic_tensor_message>(f[0], "input")->get_tensor();
    const dynamic_mx_tensor& up = as<dynamic_mx_tensor_message>(f[1], "weight")->get_mx_tensor();
    const dynamic_mx_tensor& gate = as<dynamic_mx_tensor_message>(f[2], "weight")->get_mx_tensor();
    const dynamic_mx_tensor& down = as<dynamic_mx_tensor_message>(f[3], "weight")->get_mx_tensor();
    const dynamic_tensor& router = as<dynamic_tensor_message>(f[biased ? 7 : 4], "input")->get_tensor();
    const float *b_up = nullptr, *b_gate = nullptr, *b_down = nullptr;
    if (biased) {
      b_up = as<dynamic_tensor_message>(f[4], "bias")->get_tensor().data_ptr<float>();
      b_gate = as<dynamic_tensor_message>(f[5], "bias")->get_tensor().data_ptr<float>();
      b_down = as<dynamic_tensor_message>(f[6], "bias")->get_tensor().data_ptr<float>();
    }
    if (hidden.ndim() != 3) throw std::runtime_error("expert_mlp: hidden_states must be 3D");
    if (router.ndim() != 4 || router.dim(3) != 2)
      throw std::runtime_error("expert_mlp: router_output must be 4D [batch, seq_len, top_k, 2]");
    const int64_t B = hidden.dim(0), S = hidden.dim(1), H = hidden.dim(2), k = router.dim(2);

    // an expert nobody selected answers with the {0}-shaped tensor
    const float* r = router.data_ptr<float>();
    bool any = false;
    int max_id = expert_id_;
    for (int64_t i = 0; i < B * S * k; ++i) {
      const int id = static_cast<int>(r[2 * i]);
      any = any || id == expert_id_;
      if (id > max_id) max_id = id;
    }
    if (!any) return dynamic_tensor(dtype::float32, {0});

    if (up.ndim() != 2 || gate.ndim() != 2 || down.ndim() != 2)
      throw std::runtime_error("expert_mlp: all weights must be 2D");
    const int64_t F = up.dim(0);
    if (up.dim(1) != H || gate.dim(0) != F || gate.dim(1) != H || down.dim(0) != H || down.dim(1) != F)
      throw std::runtime_error("expert_mlp: weight dimension mismatch");
    if (H % 32)
      throw std::runtime_error("expert_mlp: hidden_dim must be a multiple of 32 for MXFP4, got " + std::to_string(H));
    if (F % 32)
      throw std::runtime_error("expert_mlp: expert_ffn_dim must be a multiple of 32 for MXFP4, got " +
                               std::to_string(F));

    csk_moe_layer* h = layer_for(H, F, biased, k, max_id + 1, B * S);
    upload(h, up.data_ptr(), gate.data_ptr(), down.data_ptr(), b_up, b_gate, b_down);
    dynamic_tensor out(dtype::float32, hidden.shape());
    int32_t selected = 0;
    csk_host::check(csk_moe_expert_forward(h, expert_id_, hidden.data_ptr<float>(), B * S, r, out.data_ptr<float>(),
                                           &selected),
                    h);
    return out;
  }

  // A layer handle on which this node's expert is the only resident one.
  csk_moe_layer* layer_for(int64_t H, int64_t F, bool biased, int64_t k, int64_t id_space, int64_t tokens,
                          int32_t weight_format = CSK_WEIGHTS_MXFP4) {
    csk_moe_config c{};
    c.num_experts = static_cast<int32_t>(id_space > k ? id_space : k);
    c.top_k = static_cast<int32_t>(k);
    c.hidden = static_cast<int32_t>(H);
    c.ffn = static_cast<int32_t>(F);
    c.activation = activation_type_ == activation_type::MODIFIED_SWIGLU ? CSK_ACT_MODIFIED_SWIGLU : CSK_ACT_STANDARD_SWIGLU;
    c.has_bias = biased;
    c.weight_before_ffn = weight_before_ffn_;
    c.expert_begin = expert_id_;
    c.expert_count = 1;
    c.max_tokens = tokens;
    c.weight_format = weight_format;
    csk_moe_layer* h = handle_.get(c);
    if (handle_.just_created()) last_up_ = nullptr;
    return h;
  }

  // Expert weights are constants of the model: repack and upload when the buffer changes.  A buffer that
  // is REWRITTEN in place keeps its address: call invalidate_weights() after such a reload (hashing
  // 13 MB per expert and frame to notice it would cost more than the expert itself).
 public:
  void invalidate_weights() { last_up_ = last_gate_ = last_down_ = nullptr; }

 private:
  void upload(csk_moe_layer* h, const uint8_t* up, const uint8_t* gate, const uint8_t* down, const float* b_up,
              const float* b_gate, const float* b_down) {
    if (up == last_up_ && gate == last_gate_ && down == last_down_) return;
    csk_host::check(csk_moe_load_expert_mxfp4(h, expert_id_, up, gate, down, b_up, b_gate, b_down), h);
    last_up_ = up;
    last_gate_ = gate;
    last_down_ = down;
  }

  int expert_id_;
  graph_edge_ptr output_;
  std::vector<std::string> input_names_;
  std::string output_name_, node_name_;
  activation_type activation_type_ = activation_type::MODIFIED_SWIGLU;
  bool weight_before_ffn_ = false;
  csk_host::layer_handle handle_;
  const void *last_up_ = nullptr, *last_gate_ = nullptr, *last_down_ = nullptr;
};

}  // namespace coalsack

COALSACK_REGISTER_NODE(coalsack::expert_mlp_node, coalsack::graph_node)
