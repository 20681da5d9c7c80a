// Drives coalsack's own graph_builder (make_moe_router / make_expert_mlp /
// make_expert_merge) with the GPU operator bindings in place of the reference's
// CPU operators, on a small seeded layer read from a file written by the test,
// and writes the merged output back.  Built against the reference checkout; the
// binary runs wherever libcsk_moe.so and a B200 are.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <vector>

#include "coalsack/nn/nn_nodes.h"

using namespace coalsack;

static std::vector<char> slurp(const char* path) {
  std::ifstream f(path, std::ios::binary);
  return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

class sink_node : public graph_node {
 public:
  std::string get_proc_name() const override { return "sink"; }
  void process(std::string, graph_message_ptr m) override { last = m; }
  graph_message_ptr last;
};

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  // file: int32 E,k,H,F,T,act,has_bias ; hidden[T,H] ; Wg[E,H] ; rb[E] ; per expert: up,gate,down bytes, b_up,b_gate,b_down
  std::vector<char> buf = slurp(argv[1]);
  const char* p = buf.data();
  auto take = [&](size_t n) { const char* q = p; p += n; return q; };
  const int32_t* hd = reinterpret_cast<const int32_t*>(take(7 * 4));
  const int E = hd[0], k = hd[1], H = hd[2], F = hd[3], T = hd[4], act = hd[5], has_bias = hd[6];
  dynamic_tensor hidden(dtype::float32, {1, T, H}, take(sizeof(float) * T * H));
  dynamic_tensor Wg(dtype::float32, {E, H}, take(sizeof(float) * E * H));
  dynamic_tensor rb(dtype::float32, {E}, take(sizeof(float) * E));
  const size_t wbytes = (size_t)H * F / 32 * 17;

  const bool verbose = argc > 3;
  moe_router_node router;
  router.set_config(E, k);
  if (verbose) std::fprintf(stderr, "router ...\n");
  dynamic_tensor ro = router.compute_test(hidden, Wg, rb);
  if (verbose) std::fprintf(stderr, "router done\n");

  // gate weights refilled IN PLACE (same address, same size) must reach the GPU: the node keys its upload on content
  {
    float* w = Wg.data_ptr<float>();
    const size_t n = (size_t)E * H;
    for (size_t i = 0; i < n; ++i) w[i] = -w[i];
    dynamic_tensor cached = router.compute_test(hidden, Wg, rb);
    moe_router_node fresh;
    fresh.set_config(E, k);
    dynamic_tensor want = fresh.compute_test(hidden, Wg, rb);
    for (size_t i = 0; i < n; ++i) w[i] = -w[i];
    if (std::memcmp(cached.data_ptr<float>(), want.data_ptr<float>(), sizeof(float) * T * k * 2) != 0) {
      std::cerr << "router kept stale weights after an in-place refill\n";
      return 1;
    }
    dynamic_tensor back = router.compute_test(hidden, Wg, rb);
    if (std::memcmp(back.data_ptr<float>(), ro.data_ptr<float>(), sizeof(float) * T * k * 2) != 0) {
      std::cerr << "router did not return to the first weights\n";
      return 1;
    }
  }

  std::vector<dynamic_tensor> merge_in = {ro};
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
    for (const char* w : {"w_up", "w_gate", "w_down"}) {
      dynamic_mx_tensor t(std::string(w) == "w_down" ? std::vector<int64_t>{H, F} : std::vector<int64_t>{F, H});
      std::memcpy(t.data_ptr(), take(wbytes), wbytes);
      f[w] = std::make_shared<dynamic_mx_tensor_message>(t);
    }
    if (has_bias) {
      f["b_up"] = std::make_shared<dynamic_tensor_message>(dynamic_tensor(dtype::float32, {F}, take(sizeof(float) * F)));
      f["b_gate"] = std::make_shared<dynamic_tensor_message>(dynamic_tensor(dtype::float32, {F}, take(sizeof(float) * F)));
      f["b_down"] = std::make_shared<dynamic_tensor_message>(dynamic_tensor(dtype::float32, {H}, take(sizeof(float) * H)));
    }
    f["router"] = std::make_shared<dynamic_tensor_message>(ro);
    auto msg = result_message::ok(f);
    msg->set_frame_number(3);
    if (verbose) std::fprintf(stderr, "expert %d ...\n", e);
    node->process("default", msg);
    auto res = std::dynamic_pointer_cast<result_message>(sink->last);
    if (!res || !res->is_ok()) {
      std::cerr << "expert " << e << ": " << (res ? res->get_error_message() : "no message") << "\n";
      return 1;
    }
    merge_in.push_back(std::dynamic_pointer_cast<dynamic_tensor_message>(res->get_field("y"))->get_tensor());
  }
  if (verbose) std::fprintf(stderr, "merge ...\n");
  expert_merge_node merge;
  merge.set_config(E, k);
  dynamic_tensor out = merge.compute_test(merge_in);

  std::ofstream o(argv[2], std::ios::binary);
  o.write(reinterpret_cast<const char*>(ro.data_ptr<float>()), sizeof(float) * T * k * 2);
  o.write(reinterpret_cast<const char*>(out.data_ptr<float>()), sizeof(float) * T * H);
  std::printf("shim_check ok: E=%d k=%d H=%d F=%d T=%d\n", E, k, H, F, T);
  return 0;
}
