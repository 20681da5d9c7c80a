/* TEST INFRASTRUCTURE ONLY -- never part of the product path.
 *
 * CPU restatement, in plain C, of the reference's mixture-of-experts hot path:
 * router, MXFP4 codec, per-token gated expert MLP and the weighted merge.  It
 * exists to check the CUDA kernels; only tests, the smoke check and the
 * benchmark's CPU arm may load it.
 *
 * Parity pin: every function here is compared against the reference's own
 * code (oracle/_ref/libcsk_ref.so, built from the reference checkout by
 * oracle/Makefile) and against the committed golden vectors that library
 * produced (tests/golden/), including the reference's own known-answer tests
 * (E8M0 127/128/129 -> 0.5/1/2, all-zero nibbles -> zeros, TopKSelection
 * -> experts 5,4,3, routing weights summing to 1).
 *
 * Each function cites the reference file:line it follows (paths within the
 * reference project).  Build: see oracle/Makefile (-O2 -ffp-contract=off so
 * that a*b+c is never fused unless written as fmaf()).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* include/coalsack/gguf/gguf_dequant.h:413-415 -- E2M1 code -> doubled value. */
static const int8_t k_e2m1_x2[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

/* include/coalsack/gguf/gguf_dequant.h:419-433 -- E8M0 byte -> 2^(x-128);
 * x = 0 and x = 1 give the fp32 subnormals 2^-128 and 2^-127. */
float orc_e8m0_half(uint8_t x) {
  uint32_t bits = (x < 2) ? (0x00200000u << x) : ((uint32_t)(x - 1) << 23);
  float f;
  memcpy(&f, &bits, sizeof f);
  return f;
}

/* include/coalsack/gguf/gguf_dequant.h:437-455 -- k elements (k % 32 == 0) of
 * 17-byte blocks: byte 0 the scale, byte 1+j holds element j in its low nibble
 * and element j+16 in its high nibble. */
void orc_dequant_mxfp4(const uint8_t* src, float* dst, int64_t k) {
  for (int64_t b = 0; b < k / 32; ++b) {
    const uint8_t* blk = src + 17 * b;
    const float s = orc_e8m0_half(blk[0]);
    for (int j = 0; j < 16; ++j) {
      dst[32 * b + j] = (float)k_e2m1_x2[blk[1 + j] & 0x0F] * s;
      dst[32 * b + j + 16] = (float)k_e2m1_x2[blk[1 + j] >> 4] * s;
    }
  }
}

/* include/coalsack/nn/nn_ops/moe_router_node.h:140-214.
 * logit[e] = (((0 + h0*w0) + h1*w1) + ...) + bias[e], all fp32, no fusing;
 * top-k by descending logit (order among exactly equal logits is unspecified
 * in the reference, here the lower expert id wins); weights = softmax over the
 * k selected logits (max-subtracted, expf, sum in k order, times 1/sum) or a
 * per-expert sigmoid.  out is [T,k,2] = (expert id as float, weight). */
int orc_router(const float* hidden, int64_t T, int64_t H, const float* Wg, const float* bias,
               int64_t E, int64_t k, int sigmoid, float* out, float* logits_out) {
  if (k > E || k <= 0) return -1;
  float* logit = (float*)malloc(sizeof(float) * (size_t)E);
  int* order = (int*)malloc(sizeof(int) * (size_t)E);
  float* w = (float*)malloc(sizeof(float) * (size_t)k);
  if (!logit || !order || !w) return -2;
  for (int64_t t = 0; t < T; ++t) {
    const float* h = hidden + t * H;
    for (int64_t e = 0; e < E; ++e) {
      float sum = 0.0f;
      const float* g = Wg + e * H;
      for (int64_t d = 0; d < H; ++d) {
        float p = h[d] * g[d];
        sum = sum + p;
      }
      logit[e] = sum + (bias ? bias[e] : 0.0f);
      if (logits_out) logits_out[t * E + e] = logit[e];
    }
    /* selection sort of the k largest: same result as partial_sort wherever
     * the logits are distinct */
    for (int64_t e = 0; e < E; ++e) order[e] = (int)e;
    for (int64_t j = 0; j < k; ++j) {
      int64_t best = j;
      for (int64_t i = j + 1; i < E; ++i) {
        float a = logit[order[i]], b = logit[order[best]];
        if (a > b || (a == b && order[i] < order[best])) best = i;
      }
      int tmp = order[j];
      order[j] = order[best];
      order[best] = tmp;
    }
    if (sigmoid) {
      for (int64_t j = 0; j < k; ++j) w[j] = 1.0f / (1.0f + expf(-logit[order[j]]));
    } else {
      float mx = logit[order[0]];
      for (int64_t j = 1; j < k; ++j)
        if (logit[order[j]] > mx) mx = logit[order[j]];
      float se = 0.0f;
      for (int64_t j = 0; j < k; ++j) {
        w[j] = expf(logit[order[j]] - mx);
        se += w[j];
      }
      const float inv = (se > 0.0f) ? (1.0f / se) : 0.0f;
      for (int64_t j = 0; j < k; ++j) w[j] *= inv;
    }
    for (int64_t j = 0; j < k; ++j) {
      out[(t * k + j) * 2 + 0] = (float)order[j];
      out[(t * k + j) * 2 + 1] = w[j];
    }
  }
  free(logit);
  free(order);
  free(w);
  return 0;
}

/* One output row of an MXFP4 GEMV, in the reference's summation order
 * (include/coalsack/nn/nn_ops/expert_mlp_node.h:194-206, 211-245, 259-266,
 * 684-692): eight running lanes; within a 32-element block the four groups of
 * eight consecutive elements are fused-multiply-added into the lanes in turn;
 * the lanes are folded as (l0+l4)+(l1+l5) then (l2+l6)+(l3+l7), then added. */
static float row_dot_mxfp4(const float* x, const uint8_t* row_blocks, int64_t nblk) {
  float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float wv[32];
  for (int64_t b = 0; b < nblk; ++b) {
    orc_dequant_mxfp4(row_blocks + 17 * b, wv, 32);
    const float* xb = x + 32 * b;
    for (int g = 0; g < 4; ++g)
      for (int l = 0; l < 8; ++l) lane[l] = fmaf(xb[8 * g + l], wv[8 * g + l], lane[l]);
  }
  float s0 = lane[0] + lane[4], s1 = lane[1] + lane[5];
  float s2 = lane[2] + lane[6], s3 = lane[3] + lane[7];
  return (s0 + s1) + (s2 + s3);
}

/* include/coalsack/nn/nn_ops/expert_mlp_node.h:651-732 -- one token through
 * one expert.  act: 0 = clamped gpt-oss gate (alpha 1.702, limit 7, gate
 * clamped above only, up clamped both sides, then +1), 1 = silu(gate)*up.
 * Biases (may be NULL) are added before the activation and after the down
 * projection. */
int orc_expert_token_mxfp4(const float* x, const uint8_t* w_up, const uint8_t* w_gate,
                           const uint8_t* w_down, const float* b_up, const float* b_gate,
                           const float* b_down, float* out, int64_t H, int64_t F, int act) {
  if (H % 32 || F % 32) return -1;
  float* a = (float*)malloc(sizeof(float) * (size_t)F);
  if (!a) return -2;
  const int64_t nbh = H / 32, nbf = F / 32;
  for (int64_t o = 0; o < F; ++o) {
    float up = row_dot_mxfp4(x, w_up + o * nbh * 17, nbh) + (b_up ? b_up[o] : 0.0f);
    float gate = row_dot_mxfp4(x, w_gate + o * nbh * 17, nbh) + (b_gate ? b_gate[o] : 0.0f);
    if (act == 0) {
      const float lim = 7.0f, alpha = 1.702f;
      float g = gate < lim ? gate : lim;
      float u = up < -lim ? -lim : (up > lim ? lim : up);
      float glu = g / (1.0f + expf(alpha * (-g)));
      a[o] = glu * (u + 1.0f);
    } else {
      float silu = gate / (1.0f + expf(-gate));
      a[o] = silu * up;
    }
  }
  for (int64_t o = 0; o < H; ++o)
    out[o] = row_dot_mxfp4(a, w_down + o * nbf * 17, nbf) + (b_down ? b_down[o] : 0.0f);
  free(a);
  return 0;
}

/* include/coalsack/nn/nn_ops/expert_mlp_node.h:488-530 -- the expert node's
 * dense output: [T,H] with zero rows for tokens that did not select it.
 * Returns 0 when no token selected the expert (the reference then emits a
 * {0}-shaped tensor, :441-443), 1 otherwise. */
int orc_expert_node_mxfp4(int expert_id, const float* hidden, int64_t T, int64_t H, int64_t F,
                          const uint8_t* w_up, const uint8_t* w_gate, const uint8_t* w_down,
                          const float* b_up, const float* b_gate, const float* b_down,
                          const float* router_out, int64_t k, int act, int weight_before_ffn,
                          float* out) {
  int any = 0;
  for (int64_t i = 0; i < T * k; ++i)
    if ((int)router_out[2 * i] == expert_id) any = 1;
  if (!any) return 0;
  float* scaled = (float*)malloc(sizeof(float) * (size_t)H);
  for (int64_t t = 0; t < T; ++t) {
    int sel = 0;
    float w = 0.0f;
    for (int64_t j = 0; j < k; ++j)
      if ((int)router_out[(t * k + j) * 2] == expert_id) {
        sel = 1;
        w = router_out[(t * k + j) * 2 + 1];
        break;
      }
    if (!sel) {
      memset(out + t * H, 0, sizeof(float) * (size_t)H);
      continue;
    }
    const float* x = hidden + t * H;
    if (weight_before_ffn) {
      for (int64_t d = 0; d < H; ++d) scaled[d] = x[d] * w;
      x = scaled;
    }
    orc_expert_token_mxfp4(x, w_up, w_gate, w_down, b_up, b_gate, b_down, out + t * H, H, F, act);
  }
  free(scaled);
  return 1;
}

/* include/coalsack/nn/nn_ops/expert_merge_node.h:88-131 -- out[t] = sum over
 * k in router order of w[t,k] * expert_out[e(t,k)][t]; NULL entries of
 * expert_outs stand for the {0}-shaped empty tensors and are skipped; with
 * weight_before_ffn the rows are summed unweighted.  Returns -1 for an expert
 * id out of range, -2 when every expert output is empty. */
int orc_merge(const float* router_out, int64_t T, int64_t k, int64_t E, int64_t H,
              const float* const* expert_outs, int weight_before_ffn, float* out) {
  int any = 0;
  for (int64_t e = 0; e < E; ++e)
    if (expert_outs[e]) any = 1;
  if (!any) return -2;
  memset(out, 0, sizeof(float) * (size_t)(T * H));
  for (int64_t t = 0; t < T; ++t)
    for (int64_t j = 0; j < k; ++j) {
      int e = (int)router_out[(t * k + j) * 2];
      float w = router_out[(t * k + j) * 2 + 1];
      if (e < 0 || e >= E) return -1;
      const float* y = expert_outs[e];
      if (!y) continue;
      for (int64_t d = 0; d < H; ++d) {
        if (weight_before_ffn) {
          out[t * H + d] += y[t * H + d];
        } else {
          float p = w * y[t * H + d];
          out[t * H + d] += p;
        }
      }
    }
  return 0;
}

/* The whole layer for tokens [t0, t1): router (unless router_out is given),
 * one expert call per (token, selected expert), weighted sum in router order.
 * Same value flow as orc_expert_node_mxfp4 + orc_merge without building the E
 * dense intermediates. */
int orc_moe_layer(const float* hidden, int64_t t0, int64_t t1, int64_t H, int64_t F, int64_t E,
                  int64_t k, const float* Wg, const float* router_bias, int sigmoid,
                  const uint8_t* const* w_up, const uint8_t* const* w_gate,
                  const uint8_t* const* w_down, const float* const* b_up,
                  const float* const* b_gate, const float* const* b_down, int act,
                  int weight_before_ffn, int compute_router, float* router_out_io, float* out) {
  float* y = (float*)malloc(sizeof(float) * (size_t)H);
  float* scaled = (float*)malloc(sizeof(float) * (size_t)H);
  if (!y || !scaled) return -2;
  for (int64_t t = t0; t < t1; ++t) {
    float* r = router_out_io + t * k * 2;
    if (compute_router) {
      int rc = orc_router(hidden + t * H, 1, H, Wg, router_bias, E, k, sigmoid, r, NULL);
      if (rc) return rc;
    }
    float* o = out + t * H;
    memset(o, 0, sizeof(float) * (size_t)H);
    for (int64_t j = 0; j < k; ++j) {
      int e = (int)r[2 * j];
      float w = r[2 * j + 1];
      if (e < 0 || e >= E) return -1;
      const float* x = hidden + t * H;
      if (weight_before_ffn) {
        for (int64_t d = 0; d < H; ++d) scaled[d] = x[d] * w;
        x = scaled;
      }
      orc_expert_token_mxfp4(x, w_up[e], w_gate[e], w_down[e], b_up ? b_up[e] : NULL,
                             b_gate ? b_gate[e] : NULL, b_down ? b_down[e] : NULL, y, H, F, act);
      for (int64_t d = 0; d < H; ++d) {
        if (weight_before_ffn) {
          o[d] += y[d];
        } else {
          float p = w * y[d];
          o[d] += p;
        }
      }
    }
  }
  free(y);
  free(scaled);
  return 0;
}

/* include/coalsack/nn/nn_ops/rmsnorm_node.h:60-82 -- RMSNorm over the last dimension (the FFN norm in
 * front of the router, src/llm/llm_engine.cpp:714-719): the sum of squares is a sequential fp32 chain of
 * separate multiplies and adds, rms = sqrt(sum / H + eps), out = (x / rms) * w. */
int orc_rmsnorm(const float* x, const float* w, float eps, float* out, int64_t T, int64_t H) {
  for (int64_t i = 0; i < T; ++i) {
    float sum_sq = 0;
    for (int64_t j = 0; j < H; ++j) {
      float val = x[i * H + j];
      sum_sq += val * val;
    }
    float rms = sqrtf(sum_sq / (float)H + eps);
    for (int64_t j = 0; j < H; ++j) out[i * H + j] = (x[i * H + j] / rms) * w[j];
  }
  return 0;
}

/* fp16 bit pattern -> fp32 (what _mm256_cvtph_ps / _cvtsh_ss compute: exact). */
static float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  /* subnormal: normalise */
      int e = -1;
      uint32_t m = man;
      do {
        ++e;
        m <<= 1;
      } while ((m & 0x400u) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* include/coalsack/nn/nn_ops/dense_ffn_node.h:164-216 -- one row of fp16 weights against an fp32
 * vector: eight running lanes, one fused multiply-add per lane and group of eight columns, the lanes
 * folded by horizontal_sum_avx2 (:151-161: lo + hi halves, then (s0 + s1) + (s2 + s3) with s_i =
 * lane_i + lane_{i+4}).  n must be a multiple of eight: the reference's scalar loop for the columns past
 * the last full group is left to its compiler (partly vectorised, partly fused at -O2), and no layer this
 * library accepts has such columns (hidden and ffn sizes are multiples of 32). */
static float row_dot_f16(const float* x, const uint16_t* w, int64_t n) {
  float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int64_t i = 0;
  for (; i + 7 < n; i += 8)
    for (int l = 0; l < 8; ++l) lane[l] = fmaf(x[i + l], half_to_float(w[i + l]), lane[l]);
  /* sum128 = lo + hi; sums = sum128 + movehdup(sum128): element 0 = s0 + s1, element 2 = s2 + s3;
   * movehl brings element 2 down; add_ss: (s0 + s1) + (s2 + s3) */
  const float s0 = lane[0] + lane[4], s1 = lane[1] + lane[5], s2 = lane[2] + lane[6], s3 = lane[3] + lane[7];
  float sum = (s0 + s1) + (s2 + s3);
  return sum;
}

/* include/coalsack/nn/nn_ops/dense_ffn_node.h:28-118, 164-216 -- the dense gated FFN of the shared
 * expert, fp16 weights: gate = x.Wg + bg, up = x.Wu + bu, act = gate / (1 + exp(-gate)) * up,
 * out = act.Wd + bd; weights [F,H], [F,H], [H,F] as fp16 bit patterns, biases fp32 or NULL. */
int orc_dense_ffn_f16(const float* hidden, int64_t T, int64_t H, int64_t F, const uint16_t* gate_w,
                      const uint16_t* up_w, const uint16_t* down_w, const float* gate_b, const float* up_b,
                      const float* down_b, float* out) {
  if (H % 8 || F % 8) return -3;  /* see row_dot_f16 */
  float* act = (float*)malloc(sizeof(float) * (size_t)F);
  if (!act) return -2;
  for (int64_t t = 0; t < T; ++t) {
    const float* x = hidden + t * H;
    for (int64_t o = 0; o < F; ++o) {
      float g = row_dot_f16(x, gate_w + o * H, H), u = row_dot_f16(x, up_w + o * H, H);
      if (gate_b) g += gate_b[o];
      if (up_b) u += up_b[o];
      const float silu = g / (1.0f + expf(-g));
      act[o] = silu * u;
    }
    for (int64_t o = 0; o < H; ++o) {
      float s = row_dot_f16(act, down_w + o * F, F);
      if (down_b) s += down_b[o];
      out[t * H + o] = s;
    }
  }
  free(act);
  return 0;
}

/* include/coalsack/nn/nn_ops/dense_ffn_node.h:121-149 -- the same FFN with FLOAT32 weights: plain scalar loops,
 * one running sum per output taken in index order, product and sum rounded separately (the reference's build has
 * no fused multiply-add and a sequential float sum is not reassociated). */
int orc_dense_ffn_f32(const float* hidden, int64_t T, int64_t H, int64_t F, const float* gate_w,
                      const float* up_w, const float* down_w, const float* gate_b, const float* up_b,
                      const float* down_b, float* out) {
  float* act = (float*)malloc(sizeof(float) * (size_t)F);
  if (!act) return -2;
  for (int64_t t = 0; t < T; ++t) {
    const float* x = hidden + t * H;
    for (int64_t o = 0; o < F; ++o) {
      float g = 0.0f, u = 0.0f;
      for (int64_t i = 0; i < H; ++i) {
        g += x[i] * gate_w[o * H + i];
        u += x[i] * up_w[o * H + i];
      }
      if (gate_b) g += gate_b[o];
      if (up_b) u += up_b[o];
      const float silu = g / (1.0f + expf(-g));
      act[o] = silu * u;
    }
    for (int64_t o = 0; o < H; ++o) {
      float s = 0.0f;
      for (int64_t i = 0; i < F; ++i) s += act[i] * down_w[o * F + i];
      if (down_b) s += down_b[o];
      out[t * H + o] = s;
    }
  }
  free(act);
  return 0;
}

/* ---- Q4_K / Q6_K expert slices to fp16 --------------------------------------------------------
 * src/llm/moe_weight_provider.cpp:17-33: the slice is decoded to fp32 by dequantize_block_q4_K /
 * dequantize_block_q6_K and each value then passes fp32_to_fp16. */

/* include/coalsack/gguf/gguf_dequant.h:458-489.  nearest = 0: the branch the reference's own build
 * flags select (no F16C): the mantissa is cut, not rounded; values below 2^-25 become zero, fp16
 * subnormals are cut as well, everything from 2^16 up (NaN included) becomes infinity.
 * nearest = 1: the F16C branch, round to nearest even (NaN payloads are not modelled: quiet NaN). */
static uint16_t float_to_half_ref(float f, int nearest) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  const uint32_t sign = (bits >> 16) & 0x8000u;
  const int32_t exponent = (int32_t)((bits >> 23) & 0xFFu) - 127 + 15;
  uint32_t mantissa = (bits >> 13) & 0x3FFu;
  if (!nearest) {
    if (exponent <= 0) {
      if (exponent < -10) return (uint16_t)sign;
      mantissa |= 0x400u;
      mantissa >>= (1 - exponent);
      return (uint16_t)(sign | mantissa);
    }
    if (exponent >= 31) return (uint16_t)(sign | 0x7C00u);
    return (uint16_t)(sign | ((uint32_t)exponent << 10) | mantissa);
  }
  if (((bits >> 23) & 0xFFu) == 0xFFu) return (uint16_t)(sign | ((bits & 0x7FFFFFu) ? 0x7E00u : 0x7C00u));
  if (exponent >= 31) return (uint16_t)(sign | 0x7C00u);
  if (exponent <= 0) {
    if (exponent < -10) return (uint16_t)sign;  /* below half of the smallest subnormal */
    /* subnormal result: shift the 24-bit significand right by (14 - exponent), round to nearest even */
    const uint32_t sig = (bits & 0x7FFFFFu) | 0x800000u;
    const int sh = 14 - exponent;            /* 14 .. 24 */
    uint32_t q = sig >> sh;
    const uint32_t rem = sig & ((1u << sh) - 1u), halfway = 1u << (sh - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    return (uint16_t)(sign | q);
  }
  {
    uint32_t h = ((uint32_t)exponent << 10) | mantissa;   /* a carry out of the mantissa raises the exponent */
    const uint32_t rem = bits & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return (uint16_t)(sign | h);
  }
}

/* include/coalsack/gguf/gguf_dequant.h:147-207 -- 144-byte super-blocks: fp16 d, fp16 dmin, 12 bytes
 * holding eight 6-bit scales and eight 6-bit minima, 128 bytes of nibbles; 32 bytes give 64 values:
 * value l of sub-block 2p from the low nibbles, of sub-block 2p+1 from the high ones;
 * y = (d * scale) * q - (dmin * min), each product and the difference rounded to fp32. */
int orc_dequant_q4k_f16(const uint8_t* src, int64_t n, uint16_t* dst, int nearest) {
  if (n % 256) return -3;
  for (int64_t b = 0; b < n / 256; ++b, src += 144) {
    uint16_t dh, mh;
    memcpy(&dh, src, 2);
    memcpy(&mh, src + 2, 2);
    const float d = half_to_float(dh), dmin = half_to_float(mh);
    const uint8_t* sc = src + 4;
    const uint8_t* q = src + 16;
    for (int j = 0; j < 8; ++j) {
      uint8_t s, m;
      if (j < 4) {
        s = sc[j] & 0x3F;
        m = sc[j + 4] & 0x3F;
      } else {
        s = (uint8_t)((sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4));
        m = (uint8_t)((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
      }
      const float ds = d * (float)s, ms = dmin * (float)m;
      for (int l = 0; l < 32; ++l) {
        const uint8_t byte = q[(j / 2) * 32 + l];
        const int v = (j & 1) ? (byte >> 4) : (byte & 0x0F);
        const float prod = ds * (float)v;
        dst[b * 256 + j * 32 + l] = float_to_half_ref(prod - ms, nearest);
      }
    }
  }
  return 0;
}

/* include/coalsack/gguf/gguf_dequant.h:220-261 -- 210-byte super-blocks: 128 bytes of low nibbles,
 * 64 bytes of high bit pairs, 16 int8 scales (one per 16 values), fp16 d; per half of 128 values, value
 * l + 32 i (i = 0..3) takes its low nibble from ql[l + 32 (i & 1)] (low half for i < 2, high half
 * otherwise), its two high bits from qh[l] >> 2 i, its scale from sc[l / 16 + 2 i];
 * y = (d * scale) * (q - 32), the products taken in that order. */
int orc_dequant_q6k_f16(const uint8_t* src, int64_t n, uint16_t* dst, int nearest) {
  if (n % 256) return -3;
  for (int64_t b = 0; b < n / 256; ++b, src += 210) {
    uint16_t dh;
    memcpy(&dh, src + 208, 2);
    const float d = half_to_float(dh);
    for (int half = 0; half < 2; ++half) {
      const uint8_t* ql = src + half * 64;
      const uint8_t* qh = src + 128 + half * 32;
      const int8_t* sc = (const int8_t*)(src + 192) + half * 8;
      for (int l = 0; l < 32; ++l)
        for (int i = 0; i < 4; ++i) {
          const uint8_t lo = ql[l + 32 * (i & 1)];
          const int nib = (i < 2) ? (lo & 0x0F) : (lo >> 4);
          const int q = (nib | (((qh[l] >> (2 * i)) & 3) << 4)) - 32;
          const float ds = d * (float)sc[l / 16 + 2 * i];
          dst[b * 256 + half * 128 + l + 32 * i] = float_to_half_ref(ds * (float)q, nearest);
        }
    }
  }
  return 0;
}
