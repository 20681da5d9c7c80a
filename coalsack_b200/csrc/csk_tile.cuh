// Tensor-core grouped contraction over repacked MXFP4 weights (the prefill-side
// kernel), written for sm_100a: TMA-staged operands, MXFP4 tiles dequantised in
// shared memory to fp16, tcgen05.mma (kind::f16) with fp32 accumulators in
// tensor memory, and a fused epilogue (bias + gated activation -> fp16 rows, or
// bias -> fp32 rows).
//
// One persistent CTA per SM walks work items (row tile of 128 grouped rows x
// weight tile of BN rows).  Warp roles:
//   warp 0      producer: per k-tile one TMA tensor load of the 128 x 64 fp16
//               activation tile (128-byte swizzle) and one bulk copy of the
//               packed weight tile (codes + E8M0 scales, one contiguous span)
//   warp 1      issues the MMAs (one lane), owns the tensor-memory allocation
//   warps 2-9   dequantise the packed tile into the K-major, 128-byte-swizzled
//               fp16 operand tile (cvt.e2m1x2 -> half2, times 2^(e - e_max + 13))
//   warps 10-13 epilogue: tcgen05.ld of the accumulator, scale by the matrix's
//               power of two, bias, activation, store
// Two accumulators of BN columns alternate, so the epilogue of one work item
// overlaps the contraction of the next.
//
// fp16 operands: every MXFP4 value is value(E2M1) * 2^(e-127).  Within a matrix
// the tile is held as value * 2^(e - e_max + 13) (at most 6 * 2^13, exact in
// fp16 while e_max - e <= 36; smaller blocks lose low bits below 2^-24 of that
// range), and the accumulator is multiplied by 2^(e_max - 140) afterwards.
//
// Every wait on an mbarrier is bounded: past a clock budget the CTA records
// kDevErrWaitTimeout in the status word, all roles leave their loops, copies in
// flight are waited for (bounded again), tensor memory is freed and the kernel
// returns.
#pragma once

#include <cuda.h>

#include <functional>
#include <string>

#include "csk_common.cuh"

namespace csk {

constexpr int kTileM = 128;          // rows of a tensor-core row tile
constexpr int kDequantWarps = 8;
constexpr int kTileThreads = (2 + kDequantWarps + 4) * 32;  // producer, MMA, dequantisers, epilogue
constexpr long long kWaitBudget = 2000000000LL;  // clock cycles (~1 s) before a wait gives up

struct TileState {
  bool available = false;
  std::string err;
  CUtensorMap tmap_x{};   // grouped input rows  [rows, ldx] fp16
  CUtensorMap tmap_a{};   // activated rows      [rows, lda] fp16
  bool maps_ready = false;
  void* encode_fn = nullptr;
};

// ---- small PTX wrappers -----------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the CTA's abort flag) when the clock
// budget ran out or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitBudget) {
      *abort_flag = 1;
      return false;
    }
  }
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, groups of 8
// rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);  // start address
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset: next 8-row group
  d |= (uint64_t)1 << 46;                        // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}
// kind::f16, fp16 x fp16 -> fp32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_f16(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
      "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// fp16 bit pattern (in both halves) of 2^s for s in [-24, 15]; 0 below, 2^15 above.
__device__ __forceinline__ uint32_t h2_pow2(int s) {
  s = s > 15 ? 15 : s;
  uint32_t b = s >= -14 ? (uint32_t)(s + 15) << 10 : (s >= -24 ? 1u << (s + 24) : 0u);
  return b | (b << 16);
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

struct TileArgs {
  const uint8_t* weights;
  size_t expert_stride, mat_offset, bias_offset, meta_offset;
  MatLayout L;
  __half* a_out;          // GATED: activated rows [rows, lda]
  int lda;
  float* y_out;           // !GATED: output rows [rows, ldy]
  int ldy;
  const int* out_row_map; // optional indirection of output rows (!GATED)
  const RowTile* tiles;
  const int* n_tiles_ptr;
  int* meta;              // meta[3] = device status word
  int has_bias, act, F, meta_slot, stages;
};

inline size_t tile_stage_bytes(const MatLayout& L) {
  const size_t packed = ((size_t)L.subs * kSubBytes + 1023) / 1024 * 1024;  // keeps every stage 1024-byte aligned
  return (size_t)kTileM * 128 + (size_t)L.BN * 128 + packed;
}
inline int tile_stages(const MatLayout& L) {
  const size_t budget = 227 * 1024 - 2048;
  int s = (int)(budget / tile_stage_bytes(L));
  return s > 6 ? 6 : s;
}

template <bool GATED>
__global__ void __launch_bounds__(kTileThreads, 1)
k_tile(const __grid_constant__ CUtensorMap tmap, const TileArgs A) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const MatLayout& L = A.L;
  const int BN = L.BN, KT = L.k_tiles, NS = A.stages;
  const uint32_t tile_bytes = (uint32_t)L.tile_bytes();
  const uint32_t a_bytes = kTileM * 128, b_bytes = (uint32_t)BN * 128;
  const uint32_t packed_bytes = (tile_bytes + 1023) / 1024 * 1024;
  const uint32_t stage_bytes = a_bytes + b_bytes + packed_bytes;

  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  uint8_t* ctrl = smem + (size_t)NS * stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);  // full_raw[6], full_b[6], empty[6], tmem_full[2], tmem_empty[2], drain
  const uint32_t bar_base = smem_u32(bars);
  auto bar_full_raw = [&](int s) { return bar_base + 8u * s; };
  auto bar_full_b = [&](int s) { return bar_base + 8u * (6 + s); };
  auto bar_empty = [&](int s) { return bar_base + 8u * (12 + s); };
  auto bar_tmem_full = [&](int b) { return bar_base + 8u * (18 + b); };
  auto bar_tmem_empty = [&](int b) { return bar_base + 8u * (20 + b); };
  const uint32_t bar_drain = bar_base + 8u * 22;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 8 * 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 8 * 24 + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tmem_cols = BN * 2 <= 256 ? 256u : 512u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 6; ++s) {
      mbar_init(bar_full_raw(s), 1);
      mbar_init(bar_full_b(s), kDequantWarps);
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tmem_full(b), 1);
      mbar_init(bar_tmem_empty(b), 4);
    }
    mbar_init(bar_drain, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_row_tiles = *A.n_tiles_ptr;
  const long n_items = (long)n_row_tiles * L.n_tiles;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      int issued = 0;
      bool ok = true;
      for (long item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        const RowTile rt = A.tiles[item / L.n_tiles];
        const int nt = (int)(item % L.n_tiles);
        const uint8_t* wsrc = A.weights + (size_t)rt.expert * A.expert_stride + A.mat_offset + (size_t)nt * KT * tile_bytes;
        for (int kt = 0; kt < KT; ++kt) {
          if (!mbar_wait(bar_empty(s), ph ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t st = smem_base + (uint32_t)s * stage_bytes;
          mbar_expect_tx(bar_full_raw(s), a_bytes + tile_bytes);
          tma_load_2d(st, &tmap, kt * kTileK, rt.row0, bar_full_raw(s));
          bulk_load(st + a_bytes + b_bytes, wsrc + (size_t)kt * tile_bytes, tile_bytes, bar_full_raw(s));
          ++issued;
          if (++s == NS) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      if (!ok) {
        // let the copies still in flight land before the CTA goes away
        int s2 = s;
        uint32_t ph2 = ph;
        for (int i = 0; i < NS && i < issued; ++i) {
          if (--s2 < 0) {
            s2 = NS - 1;
            ph2 ^= 1;
          }
          const long long t0 = clock64();
          while (!mbar_try(bar_full_raw(s2), ph2) && clock64() - t0 < kWaitBudget) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(BN);
      int s = 0;
      uint32_t ph = 0;
      long it = 0;
      bool ok = true;
      for (long item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++it) {
        const int buf = (int)(it & 1);
        const uint32_t use_ph = (uint32_t)((it >> 1) & 1);
        if (!mbar_wait(bar_tmem_empty(buf), use_ph ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
        for (int kt = 0; kt < KT; ++kt) {
          if (!mbar_wait(bar_full_raw(s), ph, abort_flag) || !mbar_wait(bar_full_b(s), ph, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t st = smem_base + (uint32_t)s * stage_bytes;
          const uint64_t da = umma_desc_sw128(st), db = umma_desc_sw128(st + a_bytes);
#pragma unroll
          for (int k4 = 0; k4 < kTileK / 16; ++k4)
            umma_f16(d_tmem, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kt | k4) ? 1u : 0u);
          umma_commit(bar_empty(s));
          if (++s == NS) {
            s = 0;
            ph ^= 1;
          }
        }
        if (ok) umma_commit(bar_tmem_full(buf));
      }
      // everything issued has to retire before tensor memory is freed
      umma_commit(bar_drain);
      const long long t0 = clock64();
      while (!mbar_try(bar_drain, 0) && clock64() - t0 < kWaitBudget) {
      }
    }
  } else if (warp < 2 + kDequantWarps) {
    // ------------------------------ dequantisers ------------------------------
    const int dw = warp - 2;
    const int g = lane >> 2, q = lane & 3;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (long item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
      const RowTile rt = A.tiles[item / L.n_tiles];
      const int* emeta = reinterpret_cast<const int*>(A.weights + (size_t)rt.expert * A.expert_stride + A.meta_offset);
      const int emax = emeta[A.meta_slot];
      for (int kt = 0; kt < KT; ++kt) {
        if (!mbar_wait(bar_full_raw(s), ph, abort_flag)) {
          ok = false;
          break;
        }
        uint8_t* st = smem + (size_t)s * stage_bytes;
        uint8_t* btile = st + a_bytes;
        const uint8_t* packed = st + a_bytes + b_bytes;
        for (int sub = dw; sub < L.subs; sub += kDequantWarps) {
          const uint4 c = *reinterpret_cast<const uint4*>(packed + sub * kSubBytes + lane * 16);
          const uint32_t sc = *reinterpret_cast<const uint32_t*>(packed + sub * kSubBytes + kSubCodeBytes + g * 4);
          // odd rows start with the other 32-column block: a quarter-warp's eight
          // 16-byte stores then hit eight different bank groups
          const int b_first = g & 1;
#pragma unroll
          for (int hi = 0; hi < 2; ++hi) {
            const uint32_t w_b0 = hi ? c.z : c.x, w_b1 = hi ? c.w : c.y;  // row g + 8*hi, column blocks 0 / 1
            const int row = sub * 16 + g + hi * 8;
            uint8_t* rowp = btile + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
            for (int ord = 0; ord < 2; ++ord) {
              const int b = b_first ^ ord;
              const uint32_t w = b ? w_b1 : w_b0;
              const int e = (int)((sc >> (8 * (hi * 2 + b))) & 0xFF);
              const uint32_t sh2 = h2_pow2(e - emax + 13);
              uint32_t h[4];
              dequant_word(w, h);
              uint4 o;
              o.x = hmul2_u32(h[0], sh2);
              o.y = hmul2_u32(h[1], sh2);
              o.z = hmul2_u32(h[2], sh2);
              o.w = hmul2_u32(h[3], sh2);
              const int chunk = (b * 4 + q) ^ (row & 7);
              *reinterpret_cast<uint4*>(rowp + chunk * 16) = o;
            }
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full_b(s));
        if (++s == NS) {
          s = 0;
          ph ^= 1;
        }
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quarter = warp & 3;  // tensor-memory lanes 32*quarter .. +31 belong to this warp
    const int m = quarter * 32 + lane;
    long it = 0;
    bool ok = true;
    for (long item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++it) {
      const RowTile rt = A.tiles[item / L.n_tiles];
      const int nt = (int)(item % L.n_tiles);
      const int buf = (int)(it & 1);
      const uint32_t use_ph = (uint32_t)((it >> 1) & 1);
      const uint8_t* ebase = A.weights + (size_t)rt.expert * A.expert_stride;
      const float* bias = reinterpret_cast<const float*>(ebase + A.bias_offset);
      const int emax = reinterpret_cast<const int*>(ebase + A.meta_offset)[A.meta_slot];
      const float oscale = ldexpf(1.0f, emax - 140);
      if (!mbar_wait(bar_tmem_full(buf), use_ph, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * BN;
      const bool row_ok = m < rt.rows;
      if (GATED) {
        const int half = BN / 2;
        __half* orow = A.a_out + (size_t)(rt.row0 + m) * A.lda;
        for (int c0 = 0; c0 < half; c0 += 32) {
          uint32_t rg[32], ru[32];
          tmem_ld32(t_acc + c0, rg);
          tmem_ld32(t_acc + half + c0, ru);
          tmem_ld_wait();
          const int n0 = nt * half + c0;
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t packed[4];
#pragma unroll
              for (int p = 0; p < 4; ++p) {
                float a2[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                  const int i = v * 8 + p * 2 + u, n = n0 + i;
                  float gate = __uint_as_float(rg[i]) * oscale, up = __uint_as_float(ru[i]) * oscale;
                  if (A.has_bias && n < L.N) {
                    up += bias[n];
                    gate += bias[A.F + n];
                  }
                  a2[u] = gated_act(gate, up, A.act);
                }
                __half2 h2 = __floats2half2_rn(a2[0], a2[1]);
                packed[p] = *reinterpret_cast<uint32_t*>(&h2);
              }
              const int n = n0 + v * 8;
              if (n + 8 <= L.N) {
                *reinterpret_cast<uint4*>(orow + n) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              } else {
                for (int i = 0; i < 8 && n + i < L.N; ++i)
                  orow[n + i] = reinterpret_cast<const __half*>(packed)[i];
              }
            }
          }
        }
      } else {
        const int orow_i = A.out_row_map ? (row_ok ? A.out_row_map[rt.row0 + m] : 0) : rt.row0 + m;
        float* orow = A.y_out + (size_t)orow_i * A.ldy;
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(t_acc + c0, r);
          tmem_ld_wait();
          const int n0 = nt * BN + c0;
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              float o[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int n = n0 + v * 4 + u;
                o[u] = __uint_as_float(r[v * 4 + u]) * oscale + ((A.has_bias && n < L.N) ? bias[2 * A.F + n] : 0.f);
              }
              const int n = n0 + v * 4;
              if (n + 4 <= L.N) {
                *reinterpret_cast<float4*>(orow + n) = make_float4(o[0], o[1], o[2], o[3]);
              } else {
                for (int i = 0; i < 4 && n + i < L.N; ++i) orow[n + i] = o[i];
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tmem_empty(buf));
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicOr(&A.meta[3], kDevErrWaitTimeout);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline int tile_init(TileState& st, int device) {
  (void)device;
  st.available = false;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
    cudaGetLastError();
    st.err = "cuTensorMapEncodeTiled not found in the driver";
    return CSK_ERR_CUDA;
  }
  st.encode_fn = fn;
  for (auto* f : {(const void*)k_tile<true>, (const void*)k_tile<false>}) {
    if (cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      st.err = std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(cudaGetLastError());
      return CSK_ERR_CUDA;
    }
  }
  st.available = true;
  return CSK_OK;
}
inline void tile_destroy(TileState&) {}

// [rows, ld] fp16 row-major, boxes of 128 rows x 64 columns, 128-byte swizzle.
inline int tile_make_map(TileState& st, CUtensorMap* map, const __half* base, size_t rows, int ld) {
  const cuuint64_t dims[2] = {(cuuint64_t)ld, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(__half)};
  const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)kTileM};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = ((EncodeTiledFn)st.encode_fn)(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)base, dims, strides, box,
                                             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    st.err = "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r);
    return CSK_ERR_CUDA;
  }
  return CSK_OK;
}

inline int tile_set_buffers(TileState& st, const __half* x16, int ldx, const __half* a16, int lda, size_t rows_alloc) {
  if (!st.available) return CSK_OK;
  int rc = tile_make_map(st, &st.tmap_x, x16, rows_alloc, ldx);
  if (rc) return rc;
  rc = tile_make_map(st, &st.tmap_a, a16, rows_alloc, lda);
  if (rc) return rc;
  st.maps_ready = true;
  return CSK_OK;
}

inline int tile_launch(TileState& st, const uint8_t* weights, size_t expert_stride, size_t off_gu, size_t off_d,
                       size_t off_bias, size_t off_meta, const MatLayout& Lgu, const MatLayout& Ld, __half* a16, int lda,
                       float* y, int ldy, const int* out_row_map, const RowTile* tiles, int* meta, int has_bias,
                       int act, int F, int sm_count, cudaStream_t s, const std::function<void()>& mark) {
  if (!st.available || !st.maps_ready) {
    st.err = "tensor-core path is not initialised";
    return CSK_ERR_INVALID;
  }
  TileArgs a{};
  a.weights = weights;
  a.expert_stride = expert_stride;
  a.bias_offset = off_bias;
  a.meta_offset = off_meta;
  a.tiles = tiles;
  a.n_tiles_ptr = meta;
  a.meta = meta;
  a.has_bias = has_bias;
  a.act = act;
  a.F = F;
  // gate/up + activation
  a.mat_offset = off_gu;
  a.L = Lgu;
  a.a_out = a16;
  a.lda = lda;
  a.meta_slot = 0;
  a.stages = tile_stages(Lgu);
  size_t smem = (size_t)a.stages * tile_stage_bytes(Lgu) + 1024 + 256;
  k_tile<true><<<sm_count, kTileThreads, smem, s>>>(st.tmap_x, a);
  mark();
  // down
  a.mat_offset = off_d;
  a.L = Ld;
  a.y_out = y;
  a.ldy = ldy;
  a.out_row_map = out_row_map;
  a.meta_slot = 1;
  a.stages = tile_stages(Ld);
  smem = (size_t)a.stages * tile_stage_bytes(Ld) + 1024 + 256;
  k_tile<false><<<sm_count, kTileThreads, smem, s>>>(st.tmap_a, a);
  mark();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    st.err = std::string("launch failed: ") + cudaGetErrorString(e);
    return CSK_ERR_CUDA;
  }
  return CSK_OK;
}

}  // namespace csk
