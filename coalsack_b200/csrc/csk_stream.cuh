// Streaming grouped contraction over repacked MXFP4 weights (the decode-side
// kernel).  Memory-bound by design: every weight byte of every expert that
// received rows is read once per row tile.
//
//   * weights: each warp owns a ring of shared-memory stages; lane 0 keeps it
//     full with bulk copies (cp.async.bulk, one 544-byte record per copy, an
//     mbarrier per stage), so the bytes in flight cost no registers.  A stage is
//     consumed with one conflict-free 128-bit shared load per lane, dequantised
//     in registers (cvt.e2m1x2 -> half2) and multiplied against the tile's
//     8*NT8 token rows on the tensor cores (mma.sync m16n8k16, fp16 in, fp32
//     out).  The E8M0 block scale is applied in fp32 to each 32-column partial
//     sum, so dequantisation is exact for every scale exponent (a block with
//     scale byte 0, i.e. 2^-127, contributes zero);
//   * token rows: the current row tile sits in shared memory (fp16, copied once
//     per tile with cp.async); a CTA works through a contiguous range of work
//     units, so it changes tile rarely and its weight reads are one long stream;
//   * KSPLIT = 1: a unit is eight neighbouring 16-row groups of a weight matrix,
//     one per warp, each warp walking the whole contraction dimension;
//     KSPLIT = 8: a unit is one group whose contraction dimension is split over
//     the eight warps (a handful of rows in the batch: more units, more loads in
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
// the exponent field by one shift and one mask.
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
};

constexpr int kStreamWarps = 8;
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kStreamXPad = 32;  // halves: staggers consecutive token rows by 64 bytes in shared memory
constexpr int kStreamRingBytes = 3 * 2 * kSubBytes;  // per warp: 3 stages of a gate+up record pair, or 6 of one record

__host__ __device__ inline size_t stream_x_bytes(int nt8, int k_pad) {
  return ((size_t)8 * nt8 * (k_pad + kStreamXPad) * sizeof(__half) + 127) / 128 * 128;
}
inline size_t stream_smem_bytes(int nt8, int k_pad, int ksplit, bool gated) {
  const size_t ring = (size_t)kStreamWarps * kStreamRingBytes;
  const size_t bars = (size_t)kStreamWarps * 12 * 8;
  const size_t red = ksplit > 1 ? (size_t)(kStreamWarps - 1) * (gated ? 2 : 1) * nt8 * 4 * 32 * sizeof(float) : 0;
  return stream_x_bytes(nt8, k_pad) + ring + bars + red + 128;
}

template <int NT8, bool GATED, int KSPLIT>
__global__ void __launch_bounds__(kStreamThreads) k_stream(const StreamArgs A) {
  constexpr int NACC = GATED ? 2 : 1;
  constexpr int REC = NACC * kSubBytes;          // bytes of one stage
  constexpr int NSTG = kStreamRingBytes / REC;   // 3 (gated) or 6 stages per warp
  extern __shared__ __align__(128) uint8_t stream_smem[];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const MatLayout& L = A.L;
  const int ldxs = L.k_pad() + kStreamXPad;
  __half* xs = reinterpret_cast<__half*>(stream_smem);
  uint8_t* ring = stream_smem + stream_x_bytes(NT8, L.k_pad()) + (size_t)warp * kStreamRingBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stream_smem + stream_x_bytes(NT8, L.k_pad()) +
                                               (size_t)kStreamWarps * kStreamRingBytes) + warp * 12;
  float(*red)[NACC * NT8 * 4][32] = reinterpret_cast<float(*)[NACC * NT8 * 4][32]>(
      stream_smem + stream_x_bytes(NT8, L.k_pad()) + (size_t)kStreamWarps * (kStreamRingBytes + 12 * 8));
  const uint32_t ring_u32 = smem_u32(ring), bar_u32 = smem_u32(bars);

  if (lane == 0)
    for (int i = 0; i < NSTG; ++i) mbar_init(bar_u32 + 8u * i, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();

  const int groups = L.n_pad() / 16;  // 16-row groups (feature pairs when gated)
  const int subs_half = GATED ? L.subs / 2 : L.subs;
  const int units_per_tile = KSPLIT == 1 ? (groups + kStreamWarps - 1) / kStreamWarps : groups;
  const long n_units = (long)(*A.n_tiles_ptr) * units_per_tile;
  // balanced contiguous ranges
  const long u_begin = n_units * blockIdx.x / gridDim.x;
  const long u_end = n_units * (blockIdx.x + 1) / gridDim.x;
  const size_t kt_stride = L.tile_bytes();

  uint32_t stage_phase = 0;  // bit i = parity to wait for on stage i
  bool waits_ok = true;
  int cur_tile = -1;
  RowTile rt{};
  for (long u = u_begin; u < u_end; ++u) {
    const int tile_i = (int)(u / units_per_tile);
    const int uq = (int)(u % units_per_tile);
    if (tile_i != cur_tile) {
      // bring the tile's token rows into shared memory (rows beyond the tile's count read as zero)
      __syncthreads();
      rt = A.tiles[tile_i];
      cur_tile = tile_i;
      const int w16 = L.k_pad() / 8;
      for (int i = threadIdx.x; i < 8 * NT8 * w16; i += kStreamThreads) {
        const int r = i / w16, c = (i % w16) * 8;
        const bool ok = r < rt.rows;
        const __half* src = ok ? A.x + (size_t)(rt.row0 + r) * A.ldx + c : A.x;
        const uint32_t dst = smem_u32(xs + (size_t)r * ldxs + c);
        const int nbytes = ok ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(nbytes) : "memory");
      }
      asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
      __syncthreads();
    }
    const int grp = KSPLIT == 1 ? uq * kStreamWarps + warp : uq;
    const bool active = grp < groups;
    const int n_tile = grp / subs_half, s = grp % subs_half;
    const uint8_t* wbase = A.weights + (size_t)rt.expert * A.expert_stride + A.mat_offset +
                           (size_t)n_tile * L.k_tiles * L.tile_bytes();
    const uint8_t* p0 = wbase + (size_t)s * kSubBytes;                  // gate (or the only) record
    const uint8_t* p1 = wbase + (size_t)(s + subs_half) * kSubBytes;    // up record

    float acc[NACC][NT8][4];
#pragma unroll
    for (int m = 0; m < NACC; ++m)
#pragma unroll
      for (int j = 0; j < NT8; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[m][j][c] = 0.f;

    const int kt_begin = KSPLIT == 1 ? 0 : (int)((long)L.k_tiles * warp / KSPLIT);
    const int kt_end = KSPLIT == 1 ? L.k_tiles : (int)((long)L.k_tiles * (warp + 1) / KSPLIT);

    if (active && kt_begin < kt_end) {
      // lane 0 is this warp's producer: stage st <- k-tile kt
      auto fill = [&](int st, int kt) {
        const uint32_t bar = bar_u32 + 8u * st, dst = ring_u32 + (uint32_t)st * REC;
        const size_t o = (size_t)kt * kt_stride;
        mbar_expect_tx(bar, REC);
        bulk_load(dst, p0 + o, kSubBytes, bar);
        if (GATED) bulk_load(dst + kSubBytes, p1 + o, kSubBytes, bar);
      };
      if (lane == 0)
        for (int i = 0; i < NSTG && kt_begin + i < kt_end; ++i) fill(i, kt_begin + i);
      __syncwarp();

      int st = 0;
      for (int kt = kt_begin; kt < kt_end; ++kt) {
        if (waits_ok) {
          const uint32_t bar = bar_u32 + 8u * st, par = (stage_phase >> st) & 1u;
          if (!mbar_try(bar, par)) {
            const long long t0 = clock64();
            while (!mbar_try(bar, par)) {
              if (clock64() - t0 > kWaitBudget) {
                waits_ok = false;
                if (lane == 0) atomicOr(&A.meta[3], kDevErrWaitTimeout);
                break;
              }
            }
          }
        }
        stage_phase ^= 1u << st;
        const uint8_t* rec = ring + (size_t)st * REC;
        uint4 c[NACC];
        uint32_t sc[NACC];
#pragma unroll
        for (int m = 0; m < NACC; ++m) {
          c[m] = *reinterpret_cast<const uint4*>(rec + m * kSubBytes + lane * 16);
          sc[m] = *reinterpret_cast<const uint32_t*>(rec + m * kSubBytes + kSubCodeBytes + g * 4);
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          uint32_t af[NACC][2][4];  // [matrix][k16 step][a0..a3]
          float s_lo[NACC], s_hi[NACC];
#pragma unroll
          for (int m = 0; m < NACC; ++m) {
            uint32_t hlo[4], hhi[4];
            dequant_word(b ? c[m].y : c[m].x, hlo);  // row g
            dequant_word(b ? c[m].w : c[m].z, hhi);  // row g+8
            af[m][0][0] = hlo[0]; af[m][0][1] = hhi[0]; af[m][0][2] = hlo[1]; af[m][0][3] = hhi[1];
            af[m][1][0] = hlo[2]; af[m][1][1] = hhi[2]; af[m][1][2] = hlo[3]; af[m][1][3] = hhi[3];
            s_lo[m] = b ? scale_of<1>(sc[m]) : scale_of<0>(sc[m]);
            s_hi[m] = b ? scale_of<3>(sc[m]) : scale_of<2>(sc[m]);
          }
#pragma unroll
          for (int j = 0; j < NT8; ++j) {
            if (j * 8 < rt.rows) {  // warp-uniform: skip row groups the tile does not have
              const uint4 xb =
                  *reinterpret_cast<const uint4*>(xs + (size_t)(j * 8 + g) * ldxs + kt * kTileK + b * 32 + q * 8);
#pragma unroll
              for (int m = 0; m < NACC; ++m) {
                float t[4];
                mma16816_first(t, af[m][0], xb.x, xb.y);
                mma16816(t, af[m][1], xb.z, xb.w);
                acc[m][j][0] = fmaf(t[0], s_lo[m], acc[m][j][0]);
                acc[m][j][1] = fmaf(t[1], s_lo[m], acc[m][j][1]);
                acc[m][j][2] = fmaf(t[2], s_hi[m], acc[m][j][2]);
                acc[m][j][3] = fmaf(t[3], s_hi[m], acc[m][j][3]);
              }
            }
          }
        }
        // the stage's bytes are in registers: refill it (every lane has read before lane 0 goes on)
        __syncwarp();
        if (lane == 0 && kt + NSTG < kt_end) fill(st, kt + NSTG);
        if (++st == NSTG) st = 0;
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
              for (int w = 0; w < kStreamWarps - 1; ++w) v += red[w][r][lane];
              acc[m][j][c] = v;
            }
      }
    }
    if (active && (KSPLIT == 1 || warp == 0)) {
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
