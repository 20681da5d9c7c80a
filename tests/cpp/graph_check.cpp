// Drives coalsack's own graph_builder -- make_moe_router, make_moe_weight_fetch, make_expert_mlp (E of
// them) and make_expert_merge, with their result_message_sync_nodes, initialised by graph_proc -- with
// the GPU operator bindings in place of the reference's CPU operators and an in-memory weight provider.
// Reads a small seeded layer from a file written by the test, sends `frames` frames through the graph
// and writes the last frame's routing and merged output back.
//   graph_check <in> <out> strict|fused [frames]
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <vector>

#include "coalsack/core/graph_proc.h"
#include "coalsack/llm/graph_builder.h"

using namespace coalsack;

static std::vector<char> slurp(const char* path) {
  std::ifstream f(path, std::ios::binary);
  return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

class source_node : public graph_node {
 public:
  source_node() : out_(std::make_shared<graph_edge>(this)) { set_output(out_); }
  std::string get_proc_name() const override { return "source"; }
  void emit(const std::string& field, const dynamic_tensor& t, uint64_t frame) {
    auto m = result_message::ok({{field, std::make_shared<dynamic_tensor_message>(t)}});
    m->set_frame_number(frame);
    out_->send(m);
  }
  graph_edge_ptr edge() const { return out_; }

 private:
  graph_edge_ptr out_;
};

class sink_node : public graph_node {
 public:
  std::string get_proc_name() const override { return "sink"; }
  void process(std::string, graph_message_ptr m) override { last = m; }
  graph_message_ptr last;
};

int main(int argc, char** argv) {
  if (argc < 4) return 2;
  const bool fused = std::string(argv[3]) == "fused";
  const int frames = argc > 4 ? std::atoi(argv[4]) : 2;
  const bool f16 = argc > 5 && std::string(argv[5]) == "f16";  // expert weights in the file are FLOAT16 matrices
  csk_host::set_fused_moe(fused);
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
  const std::string L = "blk.0";
  auto provider = std::make_shared<moe_weight_provider>();
  for (int e = 0; e < E; ++e) {
    for (const char* w : {"up", "gate", "down"}) {
      const std::vector<int64_t> shape = std::string(w) == "down" ? std::vector<int64_t>{H, F} : std::vector<int64_t>{F, H};
      if (f16) {
        provider->put(L + ".ffn_" + w + "_exps.weight", e, dynamic_tensor(dtype::float16, shape, take(2u * H * F)));
        continue;
      }
      dynamic_mx_tensor t(shape);
      std::memcpy(t.data_ptr(), take(wbytes), wbytes);
      provider->put(L + ".ffn_" + w + "_exps.weight", e, t);
    }
    if (has_bias) {
      provider->put(L + ".ffn_up_exps.bias", e, dynamic_tensor(dtype::float32, {F}, take(sizeof(float) * F)));
      provider->put(L + ".ffn_gate_exps.bias", e, dynamic_tensor(dtype::float32, {F}, take(sizeof(float) * F)));
      provider->put(L + ".ffn_down_exps.bias", e, dynamic_tensor(dtype::float32, {H}, take(sizeof(float) * H)));
    }
  }

  graph_proc proc;
  auto g = proc.get_graph();
  graph_builder::config cfg;
  cfg.num_experts = E;
  cfg.expert_top_k = k;
  graph_builder gb(g, cfg);
  auto src_h = std::make_shared<source_node>(), src_w = std::make_shared<source_node>(), src_b = std::make_shared<source_node>();
  g->add_node(src_h);
  g->add_node(src_w);
  g->add_node(src_b);
  const std::string in_name = L + ".ffn_norm_out", w_name = L + ".ffn_gate_inp.weight", b_name = L + ".ffn_gate_inp.bias";
  auto router_out = gb.make_moe_router(src_h->edge(), in_name, src_w->edge(), w_name, src_b->edge(), b_name,
                                       L + ".router_out", L + ".router");
  auto fetch = gb.make_moe_weight_fetch(provider, L, router_out, has_bias != 0);
  std::vector<graph_edge_ptr> outs;
  for (int e = 0; e < E; ++e)
    outs.push_back(gb.make_expert_mlp(e, src_h->edge(), in_name, fetch[e], L + ".expert_" + std::to_string(e), has_bias != 0,
                                      act == 0 ? expert_mlp_node::activation_type::MODIFIED_SWIGLU
                                               : expert_mlp_node::activation_type::STANDARD_SWIGLU));
  auto merged = gb.make_expert_merge(router_out, L + ".router_out", outs, L, L + ".expert_merge_out");
  auto sink = std::make_shared<sink_node>(), sink_r = std::make_shared<sink_node>();
  sink->set_input(merged);
  sink_r->set_input(router_out);
  g->add_node(sink);
  g->add_node(sink_r);
  proc.initialize();
  proc.run();

  double last_ms = 0;
  size_t gets_before_last = 0;
  for (int f = 1; f <= frames; ++f) {
    gets_before_last = provider->gets();
    const auto t0 = std::chrono::steady_clock::now();
    src_w->emit(w_name, Wg, f);
    src_b->emit(b_name, rb, f);
    src_h->emit(in_name, hidden, f);
    last_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    auto res = std::dynamic_pointer_cast<result_message>(sink->last);
    if (!res || !res->is_ok() || res->get_frame_number() != (uint64_t)f) {
      std::cerr << "frame " << f << ": " << (res ? res->get_error_message() : "no message reached the sink") << "\n";
      return 1;
    }
  }
  auto res = std::dynamic_pointer_cast<result_message>(sink->last);
  auto rres = std::dynamic_pointer_cast<result_message>(sink_r->last);
  const dynamic_tensor out = std::dynamic_pointer_cast<dynamic_tensor_message>(res->get_field(L + ".expert_merge_out"))->get_tensor();
  const dynamic_tensor ro = std::dynamic_pointer_cast<dynamic_tensor_message>(rres->get_field(L + ".router_out"))->get_tensor();
  std::ofstream o(argv[2], std::ios::binary);
  o.write(reinterpret_cast<const char*>(ro.data_ptr<float>()), sizeof(float) * T * k * 2);
  o.write(reinterpret_cast<const char*>(out.data_ptr<float>()), sizeof(float) * T * H);
  std::printf("graph_check ok: mode=%s E=%d k=%d H=%d F=%d T=%d frames=%d last_frame_ms=%.3f provider_gets_last_frame=%zu\n",
              fused ? "fused" : "strict", E, k, H, F, T, frames, last_ms, provider->gets() - gets_before_last);
  proc.stop();
  proc.finalize();
  return 0;
}
