// Streaming grouped contraction over repacked MXFP4 weights (the decode-side
// kernel).  Memory-bound by design: every weight byte of every expert that
// received rows is read once per row tile.
//
//   * weights: the records of one 16-row group lie one after the other along
//     the contraction dimension, so a warp's work is ONE contiguous byte stream.
//     Each warp owns a ring of 2176-byte shared-memory stages; lane 0 keeps it
//     full with one bulk copy per stage (cp.async.bulk, an mbarrier per stage),
//     so the bytes in flight cost no registers, and the copies are large because
//     an SM starts only about one bulk copy per 70-100 cycles.  A stage holds
//     four records: gate and up of two k-tiles, or (plain matrix) the records of
//     four consecutive k-tiles.  A record is consumed with one
//     conflict-free 128-bit shared load per lane, dequantised in registers
//     (cvt.e2m1x2 -> half2) and multiplied against the tile's 8*NT8 token rows
//     on the tensor cores (mma.sync m16n8k16, fp16 in, fp32 out).  The E8M0
//     block scale is applied in fp32 to each 32-column partial sum, so
//     dequantisation is exact for every scale exponent (a block with scale
//     byte 0, i.e. 2^-127, contributes zero);
//   * token rows: the current row tile sits in shared memory (fp16, copied once
//     per tile with cp.async; only as many rows as the batch can put in a tile);
//     a CTA works through a contiguous range of work units, so it changes tile
//     rarely and its weight reads are long streams;
//   * KSPLIT = 1: a unit is W neighbouring 16-row groups of a weight matrix,
//     one per warp, each warp walking the whole contraction dimension;
//     KSPLIT = W: a unit is one group whose contraction dimension is split over
//     the warps (a handful of rows in the batch: more units, more loads in
//     flight), partial sums meet in shared memory.
//
// Every wait on a stage's mbarrier is bounded; when one runs out the warp
// records kDevErrWaitTimeout in the status word and stops waiting (its results
// are then meaningless, which the status word tells the host).
//
// Follows the arithmetic of expert_mlp_node::compute_token_mxfp4
// (include/coalsack/nn/nn_ops/expert_mlp_node.h:651-732): up/gate projections
// + bias, gated activation, down projection + bias.
#pragma once

#include "csk_common.cuh"

namespace csk {

// d = a * b (+ 0): the zero accumulator comes from constants, not from registers
__device__ __forceinline__ void mma16816_first(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Scale byte `slot` (0..3) of a packed word -> fp32 2^(e-127): the byte moved to
// the exponent field by one shift and one mask.  The codes are read as E2M1
// VALUES (0, 0.5 .. 6) where the reference multiplies doubled values (0, 1 .. 12)
// by 2^(e-128) (gguf_dequant.h:413-433): the same number for 1 <= e <= 254.
// e = 0 (2^-128 in the reference, an fp32 subnormal) gives 0 here: the block
// contributes nothing.  e = 255 (2^127 in the reference, where every code but
// +-1 overflows fp32; NaN in the OCP MX specification) is read as e = 254, so
// a block of zero codes stays zero under any scale byte: the repack stores 254
// for it (k_repack), which keeps the clamp out of this kernel's inner loop
// (there it cost 7 % of the decode step).
template <int SLOT>
__device__ __forceinline__ float scale_of(uint32_t sw) {
  const uint32_t bits = SLOT < 3 ? (sw << (23 - 8 * SLOT)) : (sw >> 1);
  return __uint_as_float(bits & 0x7F800000u);
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
  int* meta;                  // meta[3] = device status word
  int has_bias;
  int act;
  int F;                      // ffn dim (bias block: b_up[F], b_gate[F], b_down[H])
  int x_rows;                 // token rows staged per tile: >= the rows of every tile, <= 8*NT8
  // GATED, optional: gather the tile's token rows straight from the layer's input instead of from x
  // (row r of the grouped order is pair pair_of_row[r] = token * top_k + slot; fp32 -> fp16 on the way,
  // times the pair's routing weight when that is applied before the expert)
  const float* gather_hidden; // [T,H] fp32 or null
  const int* pair_of_row;     // [rows]
  const float* router;        // [T,k,2]
  int top_k, H, weight_before_ffn;
};

constexpr int kStreamXPad = 32;      // halves: staggers consecutive token rows by 64 bytes in shared memory
constexpr int kStreamRecsPerStage = 4;  // records per ring stage = per bulk copy
constexpr int kStreamStageBytes = kStreamRecsPerStage * kSubBytes;

__host__ __device__ inline size_t stream_x_bytes(int x_rows, int k_pad) {
  return ((size_t)x_rows * (k_pad + kStreamXPad) * sizeof(__half) + 127) / 128 * 128;
}
inline size_t stream_smem_bytes(int x_rows, int nt8, int k_pad, int ksplit, bool gated, int warps, int stages) {
  const size_t ring = (size_t)warps * stages * kStreamStageBytes;
  const size_t bars = (size_t)warps * stages * 8;
  const size_t red = ksplit > 1 ? (size_t)(warps - 1) * (gated ? 2 : 1) * nt8 * 4 * 32 * sizeof(float) : 0;
  return stream_x_bytes(x_rows, k_pad) + ring + bars + red + 128;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// W warps per CTA.  KSPLIT = 1: a unit is W neighbouring 16-row groups, one per warp;
// KSPLIT = W: a unit is one group, its k-tiles split over the warps.
// NSTG = ring stages per warp.
template <int NT8, bool GATED, int KSPLIT, int W, int NSTG>
__global__ void __launch_bounds__(W * 32, W > 8 ? 2 : 3) k_stream(const StreamArgs A) {
  constexpr int NACC = GATED ? 2 : 1;
  constexpr int KPS = kStreamRecsPerStage / NACC;  // k-tiles per stage
  constexpr int SB = kStreamStageBytes;
  static_assert(KSPLIT == 1 || KSPLIT == W, "split over all warps or not at all");
  extern __shared__ __align__(128) uint8_t stream_smem[];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const MatLayout L = A.L;
  const int k_tiles = L.k_tiles;
  const int ldxs = L.k_pad() + kStreamXPad;
  const int x_rows = A.x_rows;
  const size_t x_bytes = stream_x_bytes(x_rows, L.k_pad());
  __half* xs = reinterpret_cast<__half*>(stream_smem);
  const uint32_t xs_u32 = smem_u32(xs);
  const uint32_t ring_u32 = smem_u32(stream_smem + x_bytes) + (uint32_t)warp * (NSTG * SB);
  const uint32_t bar_u32 = smem_u32(stream_smem + x_bytes + (size_t)W * NSTG * SB) + (uint32_t)warp * (NSTG * 8);
  float(*red)[NACC * NT8 * 4][32] = reinterpret_cast<float(*)[NACC * NT8 * 4][32]>(
      stream_smem + x_bytes + (size_t)W * (NSTG * SB + NSTG * 8));

  if (lane == 0)
    for (int i = 0; i < NSTG; ++i) mbar_init(bar_u32 + 8u * i, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();
  griddep_wait();
  griddep_launch();

  const int groups = L.groups;  // 16-row groups (16 features, gate and up, when GATED)
  const int units_per_tile = KSPLIT == 1 ? (groups + W - 1) / W : groups;
  const long n_units = (long)(*A.n_tiles_ptr) * units_per_tile;
  // balanced contiguous ranges
  const long u_begin = n_units * blockIdx.x / gridDim.x;
  const long u_end = n_units * (blockIdx.x + 1) / gridDim.x;
  const size_t group_bytes = L.group_bytes();
  const int n_stages = (k_tiles + KPS - 1) / KPS;  // stages of a whole group
  const int sb = KSPLIT == 1 ? 0 : (int)((long)n_stages * warp / KSPLIT);
  const int se = KSPLIT == 1 ? n_stages : (int)((long)n_stages * (warp + 1) / KSPLIT);

  // per-lane shared-memory addresses: code words, scale word, token fragments
  const uint32_t rec_lane = ring_u32 + (uint32_t)lane * 16;
  const uint32_t scl_lane = ring_u32 + kSubCodeBytes + (uint32_t)g * 4;
  uint32_t x_lane[NT8];
#pragma unroll
  for (int j = 0; j < NT8; ++j) {
    // lanes whose token row does not exist read the last staged row: their result columns are never stored
    const int r = min(j * 8 + g, x_rows - 1);
    x_lane[j] = xs_u32 + (uint32_t)(r * ldxs + q * 8) * 2;
  }

  uint32_t stage_phase = 0;  // bit i = parity to wait for on stage i
  bool waits_ok = true;
  int cur_tile = -1;
  RowTile rt{};
  for (long u = u_begin; u < u_end; ++u) {
    const int tile_i = (int)(u / units_per_tile);
    const int uq = (int)(u % units_per_tile);
    const bool new_tile = tile_i != cur_tile;
    if (new_tile) rt = A.tiles[tile_i];
    const int grp = KSPLIT == 1 ? uq * W + warp : uq;
    const bool active = grp < groups;
    const uint8_t* wsrc =
        A.weights + (size_t)rt.expert * A.expert_stride + A.mat_offset + (size_t)grp * group_bytes;
    // lane 0 is this warp's producer: ring stage st <- stage i of the group's stream (requested once the
    // tile's token rows are staged: asking earlier measured 1 % slower)
    auto fill = [&](int st, int i) {
      const uint32_t bar = bar_u32 + 8u * st;
      const size_t off = (size_t)i * SB;
      const uint32_t bytes = (uint32_t)min((size_t)SB, group_bytes - off);
      mbar_expect_tx(bar, bytes);
      bulk_load(ring_u32 + (uint32_t)st * SB, wsrc + off, bytes, bar);
    };
    if (new_tile) {
      // bring the tile's token rows into shared memory
      __syncthreads();
      cur_tile = tile_i;
      const int n_rows = min(rt.rows, x_rows);
      if (GATED && A.gather_hidden) {
        const int w4 = L.k_pad() / 4;
        for (int i = threadIdx.x; i < n_rows * w4; i += W * 32) {
          const int r = i / w4, c = (i % w4) * 4;
          const int pair = A.pair_of_row[rt.row0 + r];
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (c < A.H) v = __ldg(reinterpret_cast<const float4*>(A.gather_hidden + (size_t)(pair / A.top_k) * A.H + c));
          const float mul = A.weight_before_ffn ? A.router[2 * (size_t)pair + 1] : 1.0f;
          const __half2 lo = __floats2half2_rn(v.x * mul, v.y * mul), hi = __floats2half2_rn(v.z * mul, v.w * mul);
          uint2 o;
          o.x = *reinterpret_cast<const uint32_t*>(&lo);
          o.y = *reinterpret_cast<const uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(xs) + (size_t)(r * ldxs + c) * 2) = o;
        }
      } else {
        const int w16 = L.k_pad() / 8;
        for (int i = threadIdx.x; i < n_rows * w16; i += W * 32) {
          const int r = i / w16, c = (i % w16) * 8;
          const __half* src = A.x + (size_t)(rt.row0 + r) * A.ldx + c;
          const uint32_t dst = xs_u32 + (uint32_t)(r * ldxs + c) * 2;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
      }
      __syncthreads();
    }

    float acc[NACC][NT8][4];
#pragma unroll
    for (int m = 0; m < NACC; ++m)
#pragma unroll
      for (int j = 0; j < NT8; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[m][j][c] = 0.f;

    if (active && sb < se) {
      if (lane == 0)
        for (int i = 0; i < NSTG && sb + i < se; ++i) fill(i, sb + i);
      __syncwarp();

      for (int i0 = sb; i0 < se; i0 += NSTG) {
#pragma unroll
        for (int st = 0; st < NSTG; ++st) {
          const int i = i0 + st;
          if (i >= se) break;
          if (waits_ok) {
            const uint32_t bar = bar_u32 + 8u * st, par = (stage_phase >> st) & 1u;
            if (!mbar_try(bar, par)) {
              const long long t0 = clock64();
              while (!mbar_try(bar, par)) {
                if (clock64() - t0 > wait_budget()) {
                  waits_ok = false;
                  if (lane == 0) atomicOr(&A.meta[3], kDevErrWaitTimeout);
                  break;
                }
              }
            }
          }
          stage_phase ^= 1u << st;
#pragma unroll
          for (int kk = 0; kk < KPS; ++kk) {
            const int kt = i * KPS + kk;
            if (kt >= k_tiles) break;  // the last stage of a group may hold fewer k-tiles
            const uint32_t xk = (uint32_t)kt * (kTileK * 2);  // byte offset of the k-tile in a token row
            uint4 c[NACC];
            uint32_t sc[NACC];
#pragma unroll
            for (int m = 0; m < NACC; ++m) {
              c[m] = lds128(rec_lane + st * SB + (kk * NACC + m) * kSubBytes);
              sc[m] = lds32(scl_lane + st * SB + (kk * NACC + m) * kSubBytes);
            }
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              // the gate and the up record of a k-tile share the token fragments
              uint4 xb[NT8];
#pragma unroll
              for (int j = 0; j < NT8; ++j)
                if (j == 0 || j * 8 < rt.rows) xb[j] = lds128(x_lane[j] + xk + b * 64);
#pragma unroll
              for (int m = 0; m < NACC; ++m) {
                uint32_t lo[4], hi[4];
                dequant_word(b ? c[m].y : c[m].x, lo);  // row g
                dequant_word(b ? c[m].w : c[m].z, hi);  // row g+8
                const uint32_t a0[4] = {lo[0], hi[0], lo[1], hi[1]}, a1[4] = {lo[2], hi[2], lo[3], hi[3]};
                const float s_lo = b ? scale_of<1>(sc[m]) : scale_of<0>(sc[m]);
                const float s_hi = b ? scale_of<3>(sc[m]) : scale_of<2>(sc[m]);
#pragma unroll
                for (int j = 0; j < NT8; ++j) {
                  if (j == 0 || j * 8 < rt.rows) {  // warp-uniform: skip row groups the tile does not have
                    float t[4];
                    mma16816_first(t, a0, xb[j].x, xb[j].y);
                    mma16816(t, a1, xb[j].z, xb[j].w);
                    acc[m][j][0] = fmaf(t[0], s_lo, acc[m][j][0]);
                    acc[m][j][1] = fmaf(t[1], s_lo, acc[m][j][1]);
                    acc[m][j][2] = fmaf(t[2], s_hi, acc[m][j][2]);
                    acc[m][j][3] = fmaf(t[3], s_hi, acc[m][j][3]);
                  }
                }
              }
            }
          }
          // the stage's bytes are in registers: refill it (every lane has read before lane 0 goes on)
          __syncwarp();
          if (lane == 0 && i + NSTG < se) fill(st, i + NSTG);
        }
      }
    }

    if (KSPLIT > 1) {
      // combine the k-splits
      __syncthreads();  // the previous unit's readers are done with `red`
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
              float v = acc[m][j][c];
#pragma unroll
              for (int w = 0; w < W - 1; ++w) v += red[w][r][lane];
              acc[m][j][c] = v;
            }
      }
    }
    if (active && (KSPLIT == 1 || warp == 0)) {
      const float* bias =
          reinterpret_cast<const float*>(A.weights + (size_t)rt.expert * A.expert_stride + A.bias_offset);
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const int n = grp * 16 + g + hrow * 8;  // feature / output index
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
