// Drives coalsack's dense FFN node -- through graph_builder::make_dense_ffn's own node type, with the GPU
// operator binding in place of the reference's CPU operator -- on a seeded case read from a file written
// by the test, twice (the second call reuses the uploaded weights), then once more after the gate matrix
// was refilled in place, and writes the outputs back.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <vector>

#include "coalsack/nn/nn_nodes.h"
#include "coalsack/nn/nn_ops/dense_ffn_node.h"

using namespace coalsack;

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  // file: int32 H, F, T, flags (1: biases, 2: FLOAT32 weights) ; hidden[T,H] f32 ; gate[F,H] ; up[F,H] ; down[H,F]
  //       (f16, or f32 with flag 2) ; (bg[F], bu[F], bd[H] f32)
  std::ifstream f(argv[1], std::ios::binary);
  std::vector<char> buf((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  const char* p = buf.data();
  auto take = [&](size_t n) { const char* q = p; p += n; return q; };
  const int32_t* hd = reinterpret_cast<const int32_t*>(take(4 * 4));
  const int H = hd[0], F = hd[1], T = hd[2], has_bias = hd[3] & 1, f32 = (hd[3] >> 1) & 1;
  const dtype wt = f32 ? dtype::float32 : dtype::float16;
  const size_t wb = (f32 ? 4u : 2u) * (size_t)F * H;
  dynamic_tensor hidden(dtype::float32, {1, T, H}, take(sizeof(float) * T * H));
  dynamic_tensor gate(wt, {F, H}, take(wb));
  dynamic_tensor up(wt, {F, H}, take(wb));
  dynamic_tensor down(wt, {H, F}, take(wb));
  std::vector<dynamic_tensor> in = {hidden, gate, up, down};
  if (has_bias) {
    in.push_back(dynamic_tensor(dtype::float32, {F}, take(sizeof(float) * F)));
    in.push_back(dynamic_tensor(dtype::float32, {F}, take(sizeof(float) * F)));
    in.push_back(dynamic_tensor(dtype::float32, {H}, take(sizeof(float) * H)));
  }
  dense_ffn_node node;
  dynamic_tensor a = node.compute_test(in);
  dynamic_tensor b = node.compute_test(in);
  if (std::memcmp(a.data_ptr<float>(), b.data_ptr<float>(), sizeof(float) * T * H) != 0) {
    std::cerr << "second call differs from the first\n";
    return 1;
  }
  // the gate matrix refilled in place (negated): the upload is keyed on content, so the output must change
  if (f32) {
    float* g = in[1].data_ptr<float>();
    for (size_t i = 0; i < (size_t)F * H; ++i) g[i] = -g[i];
  } else {
    uint16_t* g = in[1].data_ptr<uint16_t>();
    for (size_t i = 0; i < (size_t)F * H; ++i) g[i] ^= 0x8000u;
  }
  dynamic_tensor c = node.compute_test(in);
  std::ofstream o(argv[2], std::ios::binary);
  o.write(reinterpret_cast<const char*>(a.data_ptr<float>()), sizeof(float) * T * H);
  o.write(reinterpret_cast<const char*>(c.data_ptr<float>()), sizeof(float) * T * H);
  // error envelope: the reference's text for a wrong input count
  try {
    node.compute_test({hidden, gate});
    std::cerr << "no exception for two inputs\n";
    return 1;
  } catch (const std::exception& e) {
    if (std::string(e.what()).find("expected 4 or 7 inputs") == std::string::npos) return 1;
  }
  std::printf("dense_check ok: H=%d F=%d T=%d bias=%d f32=%d\n", H, F, T, has_bias, f32);
  return 0;
}
