// Streaming grouped contraction over repacked MXFP4 weights (the decode-side
// kernel).  Memory-bound by design: every weight byte of every expert that
// received rows is read once per row tile with 128-bit loads, dequantised in
// registers (cvt.e2m1x2 -> half2) and multiplied against up to 8*NT8 token
// rows on the tensor cores (mma.sync m16n8k16, fp16 in, fp32 out).  The E8M0
// block scale is applied in fp32 to each 32-column partial sum, so dequant is
// exact for every scale exponent.
//
// Follows the arithmetic of expert_mlp_node::compute_token_mxfp4
// (include/coalsack/nn/nn_ops/expert_mlp_node.h:651-732): up/gate projections
// + bias, gated activation, down projection + bias.
#pragma once

#include "csk_common.cuh"

namespace csk {

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void* p) {
  uint32_t r;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}

struct StreamArgs {
  const uint8_t* weights;     // base of the resident experts
  size_t expert_stride;       // bytes between experts
  size_t mat_offset;          // offset of this matrix inside an expert
  size_t bias_offset;         // offset of the expert's bias block
  MatLayout L;
  const __half* x;            // grouped input rows [rows, ldx] fp16
  int ldx;
  __half* a_out;              // GATED: activated rows [rows, lda] fp16
  int lda;
  float* y_out;               // !GATED: output rows [rows, ldy] fp32
  int ldy;
  const RowTile* tiles;       // row tiles of height 8*NT8
  const int* n_tiles_ptr;     // number of row tiles (device)
  int has_bias;
  int act;
  int F;                      // ffn dim (bias block: b_up[F], b_gate[F], b_down[H])
  float out_scale;            // unused (1.0)
};

// One CTA = 4 warps = one (row tile, group of 16 output rows); the warps split
// the contraction dimension and meet in shared memory.
template <int NT8, bool GATED>
__global__ void __launch_bounds__(128) k_stream(const StreamArgs A) {
  constexpr int NACC = GATED ? 2 : 1;
  __shared__ float red[3][NACC * NT8 * 4][32];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const MatLayout& L = A.L;
  const int groups = (GATED ? L.n_pad() : L.n_pad()) / 16;  // 16-row groups (feature pairs when gated)
  const int subs_half = GATED ? L.subs / 2 : L.subs;
  const int n_row_tiles = *A.n_tiles_ptr;
  const long n_tasks = (long)n_row_tiles * groups;

  for (long task = blockIdx.x; task < n_tasks; task += gridDim.x) {
    const int tile_i = (int)(task / groups);
    const int grp = (int)(task % groups);
    const RowTile rt = A.tiles[tile_i];
    const int n_tile = grp / subs_half, s = grp % subs_half;
    const uint8_t* wbase = A.weights + (size_t)rt.expert * A.expert_stride + A.mat_offset +
                           (size_t)n_tile * L.k_tiles * L.tile_bytes();
    const size_t kt_stride = L.tile_bytes();
    const uint8_t* p0 = wbase + (size_t)s * kSubBytes;                   // gate (or the only) record
    const uint8_t* p1 = wbase + (size_t)(s + subs_half) * kSubBytes;     // up record

    float acc[NACC][NT8][4];
#pragma unroll
    for (int m = 0; m < NACC; ++m)
#pragma unroll
      for (int j = 0; j < NT8; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[m][j][c] = 0.f;

    // this warp's share of the k tiles
    const int kt_begin = (int)((long)L.k_tiles * warp / 4);
    const int kt_end = (int)((long)L.k_tiles * (warp + 1) / 4);

    constexpr int PF = 4;
    for (int kb = kt_begin; kb < kt_end; kb += PF) {
      uint4 cw[NACC][PF];
      uint32_t sw[NACC][PF];
#pragma unroll
      for (int p = 0; p < PF; ++p) {
        if (kb + p < kt_end) {
          const size_t o = (size_t)(kb + p) * kt_stride;
          cw[0][p] = ldg_stream_v4(p0 + o + lane * 16);
          sw[0][p] = ldg_stream_u32(p0 + o + kSubCodeBytes + g * 4);
          if (GATED) {
            cw[NACC - 1][p] = ldg_stream_v4(p1 + o + lane * 16);
            sw[NACC - 1][p] = ldg_stream_u32(p1 + o + kSubCodeBytes + g * 4);
          }
        }
      }
#pragma unroll
      for (int p = 0; p < PF; ++p) {
        if (kb + p < kt_end) {
          const int kt = kb + p;
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            uint32_t af[NACC][2][4];  // [matrix][k16 step][a0..a3]
            float sc[NACC][2];        // scale of row g, row g+8
#pragma unroll
            for (int m = 0; m < NACC; ++m) {
              const uint32_t wlo = b ? cw[m][p].y : cw[m][p].x;  // row g
              const uint32_t whi = b ? cw[m][p].w : cw[m][p].z;  // row g+8
              uint32_t hlo[4], hhi[4];
              dequant_word(wlo, hlo);
              dequant_word(whi, hhi);
              af[m][0][0] = hlo[0]; af[m][0][1] = hhi[0]; af[m][0][2] = hlo[1]; af[m][0][3] = hhi[1];
              af[m][1][0] = hlo[2]; af[m][1][1] = hhi[2]; af[m][1][2] = hlo[3]; af[m][1][3] = hhi[3];
              sc[m][0] = e8m0_scale_f32((sw[m][p] >> (8 * b)) & 0xFF);
              sc[m][1] = e8m0_scale_f32((sw[m][p] >> (16 + 8 * b)) & 0xFF);
            }
#pragma unroll
            for (int j = 0; j < NT8; ++j) {
              uint4 xb = make_uint4(0, 0, 0, 0);
              if (j * 8 + g < rt.rows) {
                xb = *reinterpret_cast<const uint4*>(A.x + (size_t)(rt.row0 + j * 8 + g) * A.ldx +
                                                     kt * kTileK + b * 32 + q * 8);
              }
#pragma unroll
              for (int m = 0; m < NACC; ++m) {
                float t[4] = {0.f, 0.f, 0.f, 0.f};
                mma16816(t, af[m][0], xb.x, xb.y);
                mma16816(t, af[m][1], xb.z, xb.w);
                acc[m][j][0] = fmaf(t[0], sc[m][0], acc[m][j][0]);
                acc[m][j][1] = fmaf(t[1], sc[m][0], acc[m][j][1]);
                acc[m][j][2] = fmaf(t[2], sc[m][1], acc[m][j][2]);
                acc[m][j][3] = fmaf(t[3], sc[m][1], acc[m][j][3]);
              }
            }
          }
        }
      }
    }

    // combine the four k-splits
    __syncthreads();  // previous task's readers are done with `red`
    if (warp > 0) {
#pragma unroll
      for (int m = 0; m < NACC; ++m)
#pragma unroll
        for (int j = 0; j < NT8; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) red[warp - 1][(m * NT8 + j) * 4 + c][lane] = acc[m][j][c];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int m = 0; m < NACC; ++m)
#pragma unroll
        for (int j = 0; j < NT8; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int r = (m * NT8 + j) * 4 + c;
            acc[m][j][c] = ((acc[m][j][c] + red[0][r][lane]) + red[1][r][lane]) + red[2][r][lane];
          }
      const float* bias =
          reinterpret_cast<const float*>(A.weights + (size_t)rt.expert * A.expert_stride + A.bias_offset);
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const int n = n_tile * L.rows_per_tile() + s * 16 + g + hrow * 8;  // feature / output index
        if (n >= L.N) continue;
        float bu = 0.f, bg = 0.f, bd = 0.f;
        if (A.has_bias) {
          if (GATED) {
            bu = bias[n];
            bg = bias[A.F + n];
          } else {
            bd = bias[2 * A.F + n];
          }
        }
#pragma unroll
        for (int j = 0; j < NT8; ++j)
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int r = j * 8 + q * 2 + cc;
            if (r >= rt.rows) continue;
            const size_t row = (size_t)(rt.row0 + r);
            if (GATED) {
              const float gate = acc[0][j][hrow * 2 + cc] + bg;
              const float up = acc[NACC - 1][j][hrow * 2 + cc] + bu;
              A.a_out[row * A.lda + n] = __float2half_rn(gated_act(gate, up, A.act));
            } else {
              A.y_out[row * A.ldy + n] = acc[0][j][hrow * 2 + cc] + bd;
            }
          }
      }
    }
  }
}

}  // namespace csk
