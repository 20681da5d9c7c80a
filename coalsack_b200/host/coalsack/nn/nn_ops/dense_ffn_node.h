// GPU binding of coalsack's dense FFN operator (the shared expert of MoE transformer blocks); takes the
// place of include/coalsack/nn/nn_ops/dense_ffn_node.h.  Inputs: hidden [B,S,D] fp32, gate_w [F,D],
// up_w [F,D], down_w [D,F] all FLOAT16 or all FLOAT32 [, gate_b [F], up_b [F], down_b [D] fp32]; output
// [B,S,D] fp32 = down(silu(gate(x)) * up(x)), every token through the one weight set.  On the device this is
// a layer with one expert and top-1 in the fp16 weight format (csk_moe_load_expert_f16, csk_moe_dense_forward).
// FLOAT32 weights (the reference's scalar path) are rounded to fp16 on the device, the tensor-core kernel's
// operand type (csk_moe_load_expert_f32; refused when a weight exceeds the fp16 range).
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "coalsack/nn/nn_op_node.h"
#include "csk_moe_handle.h"

namespace coalsack {

class dense_ffn_node : public variadic_op_node {
 public:
  dense_ffn_node() : variadic_op_node("dense_ffn", 4) {}

  std::string get_proc_name() const override { return "dense_ffn"; }
  dynamic_tensor compute_test(const std::vector<dynamic_tensor>& inputs) { return compute(inputs); }
  // Weights that changed in place at the same address (another checkpoint): upload again on the next call.
  void invalidate_weights() { key_ = 0; }

 protected:
  dynamic_tensor compute(const std::vector<dynamic_tensor>& inputs) override {
    if (inputs.size() != 4 && inputs.size() != 7) {
      throw std::runtime_error(
          "dense_ffn: expected 4 or 7 inputs (hidden, gate_w, up_w, down_w[, gate_b, up_b, "
          "down_b]), got " +
          std::to_string(inputs.size()));
    }
    const auto& hidden = inputs[0];
    const auto& gate_w = inputs[1];
    const auto& up_w = inputs[2];
    const auto& down_w = inputs[3];
    const bool has_bias = (inputs.size() == 7);
    if (hidden.ndim() != 3)
      throw std::runtime_error("dense_ffn: hidden_states must be 3D [B, S, D], got " + std::to_string(hidden.ndim()) + "D");
    if (gate_w.ndim() != 2 || up_w.ndim() != 2 || down_w.ndim() != 2)
      throw std::runtime_error("dense_ffn: weight tensors must be 2D");
    const dtype weight_dtype = gate_w.get_dtype();
    if ((weight_dtype != dtype::float16 && weight_dtype != dtype::float32) || up_w.get_dtype() != weight_dtype ||
        down_w.get_dtype() != weight_dtype)
      throw std::runtime_error("dense_ffn: weight tensors must all be FLOAT16 or all FLOAT32");
    if (hidden.get_dtype() != dtype::float32) throw std::runtime_error("dense_ffn: hidden_states must be FLOAT32");
    const int64_t batch = hidden.dim(0), seq_len = hidden.dim(1), hidden_dim = hidden.dim(2);
    const int64_t ffn_dim = gate_w.dim(0);
    if (gate_w.dim(1) != hidden_dim || up_w.dim(0) != ffn_dim || up_w.dim(1) != hidden_dim)
      throw std::runtime_error("dense_ffn: gate_w/up_w shape mismatch");
    if (down_w.dim(0) != hidden_dim || down_w.dim(1) != ffn_dim)
      throw std::runtime_error("dense_ffn: down_w shape mismatch, expected [" + std::to_string(hidden_dim) + ", " +
                               std::to_string(ffn_dim) + "], got [" + std::to_string(down_w.dim(0)) + ", " +
                               std::to_string(down_w.dim(1)) + "]");
    if (hidden_dim % 32 || ffn_dim % 32)
      throw std::runtime_error("dense_ffn: hidden and ffn sizes must be multiples of 32 on the GPU");

    csk_moe_config c{};
    c.num_experts = 1;
    c.top_k = 1;
    c.hidden = (int32_t)hidden_dim;
    c.ffn = (int32_t)ffn_dim;
    c.activation = CSK_ACT_STANDARD_SWIGLU;
    c.has_bias = has_bias ? 1 : 0;
    c.weight_format = CSK_WEIGHTS_F16;
    c.max_tokens = batch * seq_len;
    csk_moe_layer* h = handle_.get(c);
    const bool f16 = weight_dtype == dtype::float16;
    const size_t wbytes = (f16 ? sizeof(uint16_t) : sizeof(float)) * (size_t)hidden_dim * ffn_dim;
    const void* pg = f16 ? static_cast<const void*>(gate_w.data_ptr<uint16_t>()) : gate_w.data_ptr<float>();
    const void* pu = f16 ? static_cast<const void*>(up_w.data_ptr<uint16_t>()) : up_w.data_ptr<float>();
    const void* pd = f16 ? static_cast<const void*>(down_w.data_ptr<uint16_t>()) : down_w.data_ptr<float>();
    const uint64_t key = csk_host::content_hash(pg, wbytes) ^ (csk_host::content_hash(pu, wbytes) * 3) ^
                         (csk_host::content_hash(pd, wbytes) * 5) ^ (uint64_t)reinterpret_cast<uintptr_t>(pg) ^
                         (f16 ? 0 : 0x9E3779B97F4A7C15ull);
    if (handle_.just_created() || key != key_ || key_ == 0) {
      const float* bu = has_bias ? inputs[5].data_ptr<float>() : nullptr;
      const float* bg = has_bias ? inputs[4].data_ptr<float>() : nullptr;
      const float* bd = has_bias ? inputs[6].data_ptr<float>() : nullptr;
      if (f16)
        csk_host::check(csk_moe_load_expert_f16(h, 0, static_cast<const uint16_t*>(pu), static_cast<const uint16_t*>(pg),
                                                static_cast<const uint16_t*>(pd), bu, bg, bd),
                        h);
      else
        csk_host::check(csk_moe_load_expert_f32(h, 0, static_cast<const float*>(pu), static_cast<const float*>(pg),
                                                static_cast<const float*>(pd), bu, bg, bd),
                        h);
      key_ = key ? key : 1;
    }
    dynamic_tensor output(dtype::float32, {batch, seq_len, hidden_dim});
    csk_host::check(csk_moe_dense_forward(h, hidden.data_ptr<float>(), batch * seq_len, output.data_ptr<float>()), h);
    return output;
  }

 private:
  csk_host::layer_handle handle_;
  uint64_t key_ = 0;
};

}  // namespace coalsack

COALSACK_REGISTER_NODE(coalsack::dense_ffn_node, coalsack::graph_node)
