// TEST INFRASTRUCTURE ONLY -- never part of the product path.
//
// C-callable wrapper around the UNMODIFIED reference implementation of the MoE
// hot path.  This translation unit includes the reference's own headers from
// where they lie in the reference checkout (no reference source is copied into
// this repository) and exposes plain-C entry points so the Python tests and the
// benchmark's CPU arm can run the reference on the same seeded buffers as the
// CUDA path.
//
// Reference entry points driven here (paths within the reference project):
//   include/coalsack/nn/nn_ops/moe_router_node.h:37-48   moe_router_node::compute_test
//   include/coalsack/nn/nn_ops/expert_mlp_node.h:63-70   expert_mlp_node::compute_test_mxfp4
//   include/coalsack/nn/nn_ops/expert_mlp_node.h:73-148  expert_mlp_node::process (MXFP4 branch)
//   include/coalsack/nn/nn_ops/expert_merge_node.h:27    expert_merge_node::compute_test
//   include/coalsack/gguf/gguf_dequant.h:419-455         e8m0_to_fp32_half, dequantize_block_mxfp4
//
// Built by oracle/Makefile into oracle/_ref/libcsk_ref.so.
#include <atomic>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "coalsack/gguf/gguf_dequant.h"
#include "coalsack/nn/nn_ops/dense_ffn_node.h"
#include "coalsack/nn/nn_ops/expert_merge_node.h"
#include "coalsack/nn/nn_ops/expert_mlp_node.h"
#include "coalsack/nn/nn_ops/rmsnorm_node.h"
#include "coalsack/nn/nn_ops/moe_router_node.h"
#include "coalsack/tensor/dynamic_mx_tensor_message.h"
#include "coalsack/tensor/dynamic_tensor_message.h"

using namespace coalsack;

namespace {

thread_local std::string g_last_error;

// Collects whatever an upstream node sends on its output edge.
class capture_node : public graph_node {
 public:
  std::string get_proc_name() const override { return "capture"; }
  void process(std::string, graph_message_ptr message) override { last = message; }
  graph_message_ptr last;
};

dynamic_tensor make_f32(const std::vector<int64_t>& shape, const float* data) {
  return dynamic_tensor(dtype::float32, shape, data);
}

dynamic_mx_tensor make_mx(int64_t rows, int64_t cols, const uint8_t* blocks) {
  dynamic_mx_tensor t({rows, cols});
  std::memcpy(t.data_ptr(), blocks, t.size_bytes());
  return t;
}

expert_mlp_node::activation_type act_of(int act) {
  return act == 0 ? expert_mlp_node::activation_type::MODIFIED_SWIGLU
                  : expert_mlp_node::activation_type::STANDARD_SWIGLU;
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_last_error.c_str(); }

float ref_e8m0_to_fp32_half(uint8_t x) { return e8m0_to_fp32_half(x); }

void ref_dequantize_block_mxfp4(const uint8_t* src, float* dst, int64_t k) {
  dequantize_block_mxfp4(src, dst, k);
}

// Router over T tokens.  out is [T, k, 2] fp32 = (expert id as float, weight).
int ref_router(const float* hidden, int64_t T, int64_t H, const float* Wg, const float* bias,
               int64_t E, int64_t k, int sigmoid, float* out) {
  try {
    moe_router_node node;
    node.set_config(E, k);
    node.set_sigmoid_gating(sigmoid != 0);
    auto h = make_f32({1, T, H}, hidden);
    auto w = make_f32({E, H}, Wg);
    dynamic_tensor r = bias ? node.compute_test(h, w, make_f32({E}, bias)) : node.compute_test(h, w);
    std::memcpy(out, r.data_ptr<float>(), sizeof(float) * T * k * 2);
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -1;
  }
}

// One token through one expert with raw 17-byte-block MXFP4 weights.
int ref_expert_token_mxfp4(const float* hidden_vec, const uint8_t* w_up, const uint8_t* w_gate,
                           const uint8_t* w_down, const float* b_up, const float* b_gate,
                           const float* b_down, float* out, int64_t H, int64_t F, int act) {
  try {
    expert_mlp_node node(0);
    node.set_activation_type(act_of(act));
    node.compute_test_mxfp4(hidden_vec, w_up, w_gate, w_down, b_up, b_gate, b_down, out, H, F);
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -1;
  }
}

// The full expert node, driven through process() with a result_message as the
// graph would deliver it.  Returns 1 and fills out[T*H] when the node produced
// a dense [1,T,H] tensor, 0 when it produced the {0}-shaped "not selected"
// tensor, -1 on an error message (text in ref_last_error()).
int ref_expert_node_mxfp4(int expert_id, const float* hidden, int64_t T, int64_t H, int64_t F,
                          const uint8_t* w_up, const uint8_t* w_gate, const uint8_t* w_down,
                          const float* b_up, const float* b_gate, const float* b_down,
                          const float* router_out, int64_t k, int act, int weight_before_ffn,
                          float* out) {
  try {
    auto node = std::make_shared<expert_mlp_node>(expert_id);
    node->set_activation_type(act_of(act));
    node->set_weight_before_ffn(weight_before_ffn != 0);
    const bool has_bias = b_up != nullptr;
    std::vector<std::string> names = {"h", "w_up", "w_gate", "w_down"};
    if (has_bias) {
      names.insert(names.end(), {"b_up", "b_gate", "b_down"});
    }
    names.push_back("router");
    node->set_input_names(names);
    node->set_output_name("y");
    node->set_node_name("oracle_expert");

    auto sink = std::make_shared<capture_node>();
    sink->set_input(node->get_output());

    std::unordered_map<std::string, graph_message_ptr> fields;
    fields["h"] = std::make_shared<dynamic_tensor_message>(make_f32({1, T, H}, hidden));
    fields["w_up"] = std::make_shared<dynamic_mx_tensor_message>(make_mx(F, H, w_up));
    fields["w_gate"] = std::make_shared<dynamic_mx_tensor_message>(make_mx(F, H, w_gate));
    fields["w_down"] = std::make_shared<dynamic_mx_tensor_message>(make_mx(H, F, w_down));
    if (has_bias) {
      fields["b_up"] = std::make_shared<dynamic_tensor_message>(make_f32({F}, b_up));
      fields["b_gate"] = std::make_shared<dynamic_tensor_message>(make_f32({F}, b_gate));
      fields["b_down"] = std::make_shared<dynamic_tensor_message>(make_f32({H}, b_down));
    }
    fields["router"] = std::make_shared<dynamic_tensor_message>(make_f32({1, T, k, 2}, router_out));
    auto msg = result_message::ok(fields);
    msg->set_frame_number(7);
    node->process("default", msg);

    auto res = std::dynamic_pointer_cast<result_message>(sink->last);
    if (!res) {
      g_last_error = "no result message";
      return -1;
    }
    if (!res->is_ok()) {
      g_last_error = res->get_error_message();
      return -1;
    }
    auto tm = std::dynamic_pointer_cast<dynamic_tensor_message>(res->get_field("y"));
    if (!tm) {
      g_last_error = "no output tensor";
      return -1;
    }
    const auto& t = tm->get_tensor();
    if (t.ndim() == 1 && t.dim(0) == 0) {
      return 0;
    }
    std::memcpy(out, t.data_ptr<float>(), sizeof(float) * T * H);
    return 1;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -1;
  }
}

// expert_merge_node over router_out plus E per-expert tensors; expert_outs[e]
// is a dense [T,H] buffer or NULL for the {0}-shaped empty tensor.
int ref_merge(const float* router_out, int64_t T, int64_t k, int64_t E, int64_t H,
              const float* const* expert_outs, int weight_before_ffn, float* out) {
  try {
    expert_merge_node node;
    node.set_config(E, k);
    node.set_weight_before_ffn(weight_before_ffn != 0);
    std::vector<dynamic_tensor> inputs;
    inputs.push_back(make_f32({1, T, k, 2}, router_out));
    for (int64_t e = 0; e < E; ++e) {
      if (expert_outs[e]) {
        inputs.push_back(make_f32({1, T, H}, expert_outs[e]));
      } else {
        inputs.push_back(dynamic_tensor(dtype::float32, {0}));
      }
    }
    dynamic_tensor r = node.compute_test(inputs);
    std::memcpy(out, r.data_ptr<float>(), sizeof(float) * T * H);
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -1;
  }
}

// Whole MoE layer on the reference's code: router compute_test, then for every
// (token, selected expert) one compute_test_mxfp4 call, then the weighted sum
// in router order exactly as expert_merge_node evaluates it (zero, then
// out += w * y for k = 0..top_k-1).  The per-expert dense [T,H] intermediates
// the graph would build are not materialised (128 x 8192 x 2880 floats would
// not fit); each (token, expert) result is consumed immediately, which yields
// the same floating-point values.  Tokens are spread over nthreads host
// threads; nthreads = 1 is the reference's own execution model.
//
// w_up/w_gate/w_down: [E] pointers to 17-byte-block matrices; b_*: [E] pointers
// or NULL when the layer has no biases.  router_out_io: [T,k,2]; computed here
// when compute_router != 0, else taken as input.
int ref_moe_layer(const float* hidden, int64_t T, int64_t H, int64_t F, int64_t E, int64_t k,
                  const float* Wg, const float* router_bias, int sigmoid,
                  const uint8_t* const* w_up, const uint8_t* const* w_gate,
                  const uint8_t* const* w_down, const float* const* b_up,
                  const float* const* b_gate, const float* const* b_down, int act,
                  int weight_before_ffn, int nthreads, int compute_router, float* router_out_io,
                  float* out) {
  try {
    if (compute_router) {
      int rc = ref_router(hidden, T, H, Wg, router_bias, E, k, sigmoid, router_out_io);
      if (rc) return rc;
    }
    if (nthreads < 1) nthreads = 1;
    std::atomic<int64_t> next{0};
    std::atomic<int> failed{0};
    std::string err;
    auto work = [&]() {
      try {
        expert_mlp_node node(0);
        node.set_activation_type(act_of(act));
        std::vector<float> y(H), scaled(H);
        for (;;) {
          int64_t t = next.fetch_add(1);
          if (t >= T) break;
          float* o = out + t * H;
          std::memset(o, 0, sizeof(float) * H);
          for (int64_t j = 0; j < k; ++j) {
            int e = static_cast<int>(router_out_io[(t * k + j) * 2]);
            float w = router_out_io[(t * k + j) * 2 + 1];
            if (e < 0 || e >= E) throw std::runtime_error("expert id out of range");
            const float* x = hidden + t * H;
            if (weight_before_ffn) {
              for (int64_t d = 0; d < H; ++d) scaled[d] = x[d] * w;
              x = scaled.data();
            }
            node.compute_test_mxfp4(x, w_up[e], w_gate[e], w_down[e], b_up ? b_up[e] : nullptr,
                                    b_gate ? b_gate[e] : nullptr, b_down ? b_down[e] : nullptr,
                                    y.data(), H, F);
            if (weight_before_ffn) {
              for (int64_t d = 0; d < H; ++d) o[d] += y[d];
            } else {
              for (int64_t d = 0; d < H; ++d) o[d] += w * y[d];
            }
          }
        }
      } catch (const std::exception& e) {
        if (!failed.exchange(1)) err = e.what();
      }
    };
    std::vector<std::thread> pool;
    for (int i = 1; i < nthreads; ++i) pool.emplace_back(work);
    work();
    for (auto& th : pool) th.join();
    if (failed) {
      g_last_error = err;
      return -1;
    }
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -1;
  }
}

// FFN RMSNorm (rmsnorm_node::compute_test) over [T, H] with weight [H].
int ref_rmsnorm(const float* x, const float* w, float eps, float* out, int64_t T, int64_t H) {
  try {
    rmsnorm_node node;
    node.set_epsilon(eps);
    dynamic_tensor r = node.compute_test(make_f32({1, T, H}, x), make_f32({H}, w));
    std::memcpy(out, r.data_ptr<float>(), sizeof(float) * T * H);
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -1;
  }
}

// The shared expert's dense FFN (dense_ffn_node::compute, protected: reached through a subclass).
struct dense_ffn_probe : public dense_ffn_node {
  using dense_ffn_node::compute;
};
int ref_dense_ffn_f16(const float* hidden, int64_t T, int64_t H, int64_t F, const uint16_t* gate_w,
                      const uint16_t* up_w, const uint16_t* down_w, const float* gate_b, const float* up_b,
                      const float* down_b, float* out) {
  try {
    dense_ffn_probe node;
    std::vector<dynamic_tensor> in;
    in.push_back(make_f32({1, T, H}, hidden));
    in.push_back(dynamic_tensor(dtype::float16, {F, H}, gate_w));
    in.push_back(dynamic_tensor(dtype::float16, {F, H}, up_w));
    in.push_back(dynamic_tensor(dtype::float16, {H, F}, down_w));
    if (gate_b) {
      in.push_back(make_f32({F}, gate_b));
      in.push_back(make_f32({F}, up_b));
      in.push_back(make_f32({H}, down_b));
    }
    dynamic_tensor r = node.compute(in);
    std::memcpy(out, r.data_ptr<float>(), sizeof(float) * T * H);
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -1;
  }
}

int ref_dense_ffn_f32(const float* hidden, int64_t T, int64_t H, int64_t F, const float* gate_w, const float* up_w,
                      const float* down_w, const float* gate_b, const float* up_b, const float* down_b, float* out) {
  try {
    dense_ffn_probe node;
    std::vector<dynamic_tensor> in;
    in.push_back(make_f32({1, T, H}, hidden));
    in.push_back(make_f32({F, H}, gate_w));
    in.push_back(make_f32({F, H}, up_w));
    in.push_back(make_f32({H, F}, down_w));
    if (gate_b) {
      in.push_back(make_f32({F}, gate_b));
      in.push_back(make_f32({F}, up_b));
      in.push_back(make_f32({H}, down_b));
    }
    dynamic_tensor r = node.compute(in);
    std::memcpy(out, r.data_ptr<float>(), sizeof(float) * T * H);
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -1;
  }
}

// src/llm/moe_weight_provider.cpp:17-33 keeps these two helpers in an unnamed namespace of a file that
// needs the GGUF loader; they are two calls into the reference's header, made here in the same order:
// the block decoder to fp32, then fp32_to_fp16 on every value.
int ref_dequant_kquant_f16(int ggml_type_id, const uint8_t* src, int64_t n, uint16_t* dst) {
  try {
    std::vector<float> temp(n);
    if (ggml_type_id == static_cast<int>(ggml_type::Q4_K)) {
      dequantize_block_q4_K(src, temp.data(), n);
    } else if (ggml_type_id == static_cast<int>(ggml_type::Q6_K)) {
      dequantize_block_q6_K(src, temp.data(), n);
    } else {
      g_last_error = "ref_dequant_kquant_f16: type not handled";
      return -1;
    }
    for (int64_t i = 0; i < n; ++i) dst[i] = fp32_to_fp16(temp[i]);
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -1;
  }
}

}  // extern "C"
