// Drives coalsack's expert node with FLOAT16 weight tensors (what the weight provider makes of Q4_K / Q6_K /
// F16 expert slices) through process() with result_messages, with the GPU operator binding in place of the
// reference's CPU operator, merges the experts' outputs with the merge node and writes the result back.
// The router output comes from the test (file), so that only the expert path is under test here.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <vector>

#include "coalsack/nn/nn_nodes.h"

using namespace coalsack;

class sink_node : public graph_node {
 public:
  std::string get_proc_name() const override { return "sink"; }
  void process(std::string, graph_message_ptr m) override { last = m; }
  graph_message_ptr last;
};

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  // file: int32 E,k,H,F,T,act,has_bias ; hidden[T,H] f32 ; router[T,k,2] f32 ;
  //       per expert: up[F,H], gate[F,H], down[H,F] f16, (b_up[F], b_gate[F], b_down[H] f32)
  std::ifstream fi(argv[1], std::ios::binary);
  std::vector<char> buf((std::istreambuf_iterator<char>(fi)), std::istreambuf_iterator<char>());
  const char* p = buf.data();
  auto take = [&](size_t n) { const char* q = p; p += n; return q; };
  const int32_t* hd = reinterpret_cast<const int32_t*>(take(7 * 4));
  const int E = hd[0], k = hd[1], H = hd[2], F = hd[3], T = hd[4], act = hd[5], has_bias = hd[6];
  dynamic_tensor hidden(dtype::float32, {1, T, H}, take(sizeof(float) * T * H));
  dynamic_tensor ro(dtype::float32, {1, T, k, 2}, take(sizeof(float) * T * k * 2));

  std::vector<dynamic_tensor> merge_in = {ro};
  int placeholders = 0;
  for (int e = 0; e < E; ++e) {
    auto node = std::make_shared<expert_mlp_node>(e);
    node->set_activation_type(act == 0 ? expert_mlp_node::activation_type::MODIFIED_SWIGLU
                                       : expert_mlp_node::activation_type::STANDARD_SWIGLU);
    std::vector<std::string> names = {"h", "w_up", "w_gate", "w_down"};
    if (has_bias) names.insert(names.end(), {"b_up", "b_gate", "b_down"});
    names.push_back("router");
    node->set_input_names(names);
    node->set_output_name("y");
    auto sink = std::make_shared<sink_node>();
    sink->set_input(node->get_output());
    std::unordered_map<std::string, graph_message_ptr> f;
    f["h"] = std::make_shared<dynamic_tensor_message>(hidden);
    dynamic_tensor up(dtype::float16, {F, H}, take(2u * F * H));
    dynamic_tensor gate(dtype::float16, {F, H}, take(2u * F * H));
    dynamic_tensor down(dtype::float16, {H, F}, take(2u * F * H));
    f["w_up"] = std::make_shared<dynamic_tensor_message>(up);
    f["w_gate"] = std::make_shared<dynamic_tensor_message>(gate);
    f["w_down"] = std::make_shared<dynamic_tensor_message>(down);
    if (has_bias) {
      f["b_up"] = std::make_shared<dynamic_tensor_message>(dynamic_tensor(dtype::float32, {F}, take(sizeof(float) * F)));
      f["b_gate"] = std::make_shared<dynamic_tensor_message>(dynamic_tensor(dtype::float32, {F}, take(sizeof(float) * F)));
      f["b_down"] = std::make_shared<dynamic_tensor_message>(dynamic_tensor(dtype::float32, {H}, take(sizeof(float) * H)));
    }
    f["router"] = std::make_shared<dynamic_tensor_message>(ro);
    auto msg = result_message::ok(f);
    msg->set_frame_number(5);
    dynamic_tensor first;
    for (int rep = 0; rep < 2; ++rep) {  // the second frame reuses the uploaded weights
      node->process("default", msg);
      auto res = std::dynamic_pointer_cast<result_message>(sink->last);
      if (!res || !res->is_ok()) {
        std::cerr << "expert " << e << ": " << (res ? res->get_error_message() : "no message") << "\n";
        return 1;
      }
      if (res->get_frame_number() != 5) return 1;
      dynamic_tensor y = std::dynamic_pointer_cast<dynamic_tensor_message>(res->get_field("y"))->get_tensor();
      if (rep == 0) {
        first = y;
      } else if (y.numel() != first.numel() ||
                 std::memcmp(y.data_ptr<float>(), first.data_ptr<float>(), sizeof(float) * y.numel()) != 0) {
        std::cerr << "expert " << e << ": second frame differs\n";
        return 1;
      }
    }
    if (first.numel() == 0) ++placeholders;
    merge_in.push_back(first);
    if (e == 0) {
      // error envelope: the reference's texts
      try {
        node->compute_test({hidden, up, gate});
        return 1;
      } catch (const std::exception& ex) {
        if (std::string(ex.what()).find("expected 5 or 8 inputs") == std::string::npos) return 1;
      }
      try {
        dynamic_tensor f32w(dtype::float32, {F, H});
        std::vector<dynamic_tensor> in = {hidden, f32w, gate, down};
        if (has_bias) {
          in.push_back(dynamic_tensor(dtype::float32, {F}));
          in.push_back(dynamic_tensor(dtype::float32, {F}));
          in.push_back(dynamic_tensor(dtype::float32, {H}));
        }
        // a router tensor that selects expert 0 for sure
        dynamic_tensor sel(dtype::float32, {1, 1, 1, 2});
        sel.data_ptr<float>()[0] = 0.0f;
        sel.data_ptr<float>()[1] = 1.0f;
        in.push_back(sel);
        in[0] = dynamic_tensor(dtype::float32, {1, 1, H});
        node->compute_test(in);
        return 1;
      } catch (const std::exception& ex) {
        if (std::string(ex.what()).find("all weights must be FLOAT16") == std::string::npos) {
          std::cerr << "unexpected text: " << ex.what() << "\n";
          return 1;
        }
      }
    }
  }
  expert_merge_node merge;
  merge.set_config(E, k);
  dynamic_tensor out = merge.compute_test(merge_in);
  std::ofstream o(argv[2], std::ios::binary);
  o.write(reinterpret_cast<const char*>(out.data_ptr<float>()), sizeof(float) * T * H);
  std::printf("expert_f16_check ok: E=%d k=%d H=%d F=%d T=%d placeholders=%d\n", E, k, H, F, T, placeholders);
  return 0;
}
