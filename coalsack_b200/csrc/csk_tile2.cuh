// Tensor-core grouped contraction over repacked MXFP4 weights on PAIRS of CTAs
// (thread-block clusters of two, tcgen05 cta_group::2), for sm_100a.
//
// Why pairs.  The contraction is computed transposed, D[weight row, token] = W · Xᵀ, with the
// dequantised weights as the tensor-memory operand (see csk_tile.cuh).  Every weight that is
// dequantised feeds 2 N flops, N = token rows of the work item, and N is bounded by tensor
// memory: a CTA that holds BOTH 128-row halves of a weight tile has 2 N accumulator columns
// and no room beyond N = 192.  An expert with 256 rows is then two items (192 + 64) that both
// pay the full dequantisation of the weight tile, and the small one cannot keep the tensor
// pipe busy.  A pair of CTAs issues ONE MMA of M = 256 (128 weight rows in each CTA's tensor
// memory) against a token tile that is split between the two CTAs' shared memory:
//   * each CTA dequantises only ITS 128 weight rows per k-step (half the work per item),
//   * each CTA loads only ITS half of the token tile (half the L2 -> SM traffic per item),
//   * one accumulator of N <= 192 columns per CTA (instead of two) leaves room for a SECOND
//     accumulator buffer: the epilogue of an item runs while the MMAs of the next item fill
//     the other buffer -- and for a ring of FOUR dequantised weight tiles (32 columns each)
//     filled by four dequantiser groups.
//
// A work item is (row tile of up to 192 grouped token rows of one expert) x (weight tile of the
// tile layout: 256 weight rows).  For the fused gate/up matrix CTA c takes features
// 64c .. 64c+63 of the tile, gate and up rows INTERLEAVED on neighbouring tensor-memory lanes
// (lane 2f = gate, lane 2f+1 = up of feature f; the epilogue pairs them with one shuffle); it
// reads them out of the tile layout's two halves, so the same repacked weights serve both
// tensor-core kernels.  For a plain matrix CTA c takes half c of the tile.
//
// Per k-step (64 columns) and CTA: the producer warp issues one TMA load of its 96 x 64 fp16
// token half tile (no multicast, this CTA's own barrier) and one bulk copy of the packed weight
// tile; a dequantiser group converts the CTA's 128 rows and stores them to tensor memory
// (tcgen05.st), then arrives -- across the cluster -- on the LEADER CTA's barrier of that ring
// slot.  Because a group waits for its own CTA's loads before it converts, eight arrivals (four
// warps in each CTA) tell the leader's MMA warp that both weight halves are in tensor memory and
// both token halves in shared memory.  It issues four tcgen05.mma.cta_group::2 (K = 16 each)
// and commits to the "retired" barrier of that k-step (one of eight, by k-step number mod 8) in BOTH
// CTAs (tcgen05.commit with cluster multicast): the producers wait on it before they reuse the
// shared-memory stage (eight k-steps later), the dequantisers before they reuse the tensor-memory
// slot (four k-steps later).  After the item's last k-step it commits "accumulator complete" for
// the item's buffer to both CTAs; eight epilogue warps per CTA read their CTA's accumulator and
// arrive on the leader's "accumulator free" barrier of that buffer.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises the abort flag of BOTH
// CTAs, every role leaves its loop, copies in flight and outstanding MMAs are drained, the two
// CTAs meet at a cluster barrier, tensor memory is freed, and kDevErrWaitTimeout reaches the
// host.  No load here uses cluster multicast and no tensor map covers another GPU's memory.
//
// Status: selected by name only (CSK_PATH_TILE_PAIR).  A shared-memory stage is held from its copies'
// request until its MMAs retire (about 1.5 us of load latency plus conversion plus the MMA queue), and
// eight 21.5 KB stages cover 0.43 us per k-step where the tensor pipe needs 0.2: on the measured
// prefill workloads the one-CTA kernel is the faster of the two (0.96 against 1.7 ms for gate/up on the
// 128-expert layer).  Copying only the CTA's half of the packed gate/up tile (a layout change) would
// make room for thirteen stages.
#pragma once

#include "csk_tile.cuh"

namespace csk {

constexpr int kPairN = 192;                         // token rows of a row tile (MMA N <= 192, a multiple of 32)
constexpr int kPairGroups = 4;                      // dequantiser groups (four warps each)
constexpr int kPairSlots = 4;                       // dequantised weight tiles resident in tensor memory
constexpr int kPairStages = 8;                      // shared-memory stages = "retired" barriers (k-step number mod 8)
constexpr int kPairEpilogueWarps = 8;
constexpr int kPairThreads = (2 + 4 * kPairGroups + kPairEpilogueWarps) * 32;
constexpr int kPairHalfRows = kPairN / 2;           // token rows of a CTA's half tile (TMA box height)
constexpr int kPairABytes = kPairHalfRows * 128;    // token half tile in shared memory (96 rows x 64 fp16)
constexpr int kPairRawBytes = kPairABytes + 9216;   // one stage: token half tile + packed weight tile
constexpr uint32_t kPairRingBase = 2 * kPairN;      // first tensor-memory column of the weight ring (after two accumulators)
static_assert(kPairRawBytes % 1024 == 0, "stage alignment");
static_assert(2 * kPairN + 32 * kPairSlots <= 512, "tensor memory");
static_assert(kPairStages == 8 && kPairSlots == 4 && kPairGroups == 4, "the barrier arithmetic below assumes these");

inline size_t pair_smem_bytes() { return (size_t)kPairStages * kPairRawBytes + 1024 + 512; }

// ---- cluster helpers ------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local_addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]^T over the CTA pair: M = 256 (128 rows in each CTA), B's N rows split between the CTAs
__device__ __forceinline__ void umma2_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far have retired
__device__ __forceinline__ void umma2_commit_both(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ uint32_t umma2_idesc_f16(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <bool GATED>
__global__ void __launch_bounds__(kPairThreads, 1)
k_tile2(const __grid_constant__ CUtensorMap tmap, const TileArgs A) {
  extern __shared__ __align__(1024) uint8_t tile2_smem[];
  const TileLayout& L = A.L;
  const int KT = L.k_tiles;
  constexpr int NR = kPairStages, NA = kPairSlots, NG = kPairGroups;

  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)tile2_smem + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);  // ring of [token half tile | packed weight tile]
  uint8_t* ctrl = smem + (size_t)NR * kPairRawBytes;
  const uint32_t bar_base = smem_u32(ctrl);
  // k-step c uses shared-memory stage c % 8 and tensor-memory slot c % 4; its MMAs' retirement is signalled on
  // "retired" barrier c % 8, whose phase number is c / 8
  auto bar_full_raw = [&](int s) { return bar_base + 8u * s; };          // this CTA's loads of the stage landed
  auto bar_retired = [&](int j) { return bar_base + 8u * (8 + j); };     // MMAs of a k-step with number = j mod 8 retired (both CTAs)
  auto bar_full_a = [&](int s) { return bar_base + 8u * (16 + s); };     // leader: both CTAs' rows of the slot are in tensor memory
  auto bar_tmem_full = [&](int b) { return bar_base + 8u * (32 + b); };  // accumulator buffer b complete (both CTAs)
  auto bar_tmem_empty = [&](int b) { return bar_base + 8u * (34 + b); }; // leader: both CTAs' epilogues are done with buffer b
  const uint32_t bar_drain = bar_base + 8u * 36;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 8 * 40);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 8 * 40 + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const uint32_t peer_abort = map_to_cta(smem_u32((const void*)abort_flag), rank ^ 1u);
  // a wait ran out here: the peer's roles must leave their loops too
  auto tell_peer = [&]() { st_cluster_u32(peer_abort, 1u); };
  auto wait_or_abort = [&](uint32_t bar, uint32_t parity) {
    if (mbar_wait(bar, parity, abort_flag)) return true;
    tell_peer();
    return false;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < NR; ++s) {
      mbar_init(bar_full_raw(s), 1);
      mbar_init(bar_retired(s), 1);
    }
    for (int s = 0; s < NA; ++s) mbar_init(bar_full_a(s), 8);  // four warps of a dequantiser group in each CTA
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tmem_full(b), 1);
      mbar_init(bar_tmem_empty(b), 2 * kPairEpilogueWarps);
    }
    mbar_init(bar_drain, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone arrives on the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_row_tiles = *A.n_tiles_ptr;
  const long n_items = (long)n_row_tiles * L.n_tiles;
  const long pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  // bytes of packed weights this CTA copies per k-step, and where they start inside a tile
  const uint32_t w_bytes = GATED ? kTilePacked : kHalfPacked;
  const uint32_t w_skip = GATED ? 0u : rank * kHalfPacked;

  if (warp == 0) {
    // ------------------------------ producer (each CTA) ------------------------------
    if (lane == 0) {
      long c = 0;
      int issued = 0;
      bool ok = true;
      for (long item = pair; ok && !A.stall && item < n_items; item += n_pairs) {
        const RowTile rt = A.tiles[item / L.n_tiles];
        const int nt = (int)(item % L.n_tiles);
        const int n_mma = max(32, (rt.rows + 31) & ~31);
        const int my_row0 = rt.row0 + (int)rank * (n_mma / 2);  // this CTA's half of the item's token rows
        const uint8_t* wsrc = A.weights + (size_t)rt.expert * A.expert_stride + A.mat_offset +
                              (size_t)nt * KT * kTilePacked + w_skip;
        for (int kt = 0; kt < KT; ++kt, ++c) {
          const int s = (int)(c % NR);
          // the stage was last read by k-step c - 8
          if (c >= NR && !wait_or_abort(bar_retired(s), (uint32_t)((c / NR - 1) & 1))) {
            ok = false;
            break;
          }
          const uint32_t st = smem_base + (uint32_t)s * kPairRawBytes;
          mbar_expect_tx(bar_full_raw(s), kPairABytes + w_bytes);
          tma_load_2d(st, &tmap, kt * kTileK, my_row0, bar_full_raw(s));
          bulk_load(st + kPairABytes, wsrc + (size_t)kt * kTilePacked, w_bytes, bar_full_raw(s));
          ++issued;
        }
      }
      if (!ok) {
        // let the copies still in flight land before the CTA goes away
        for (int i = 0; i < NR && i < issued; ++i) {
          const long cc = c - 1 - i;
          const long long t0 = clock64();
          while (!mbar_try(bar_full_raw((int)(cc % NR)), (uint32_t)((cc / NR) & 1)) && clock64() - t0 < drain_budget()) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (rank == 0) {
      // The WHOLE warp runs this loop and one elected lane issues.  tcgen05.mma and tcgen05.commit take
      // their operands from the warp-uniform register file: in a loop that only one lane runs (a divergent
      // branch) the compiler has to move every descriptor and address across for every instruction, and a
      // K=16 MMA then issues every ~185 clocks whatever its shape (measured; the pipe needs 96 for
      // 256 x 192 x 16), which halves the kernel.  Run warp-wide, the same loop keeps the pipe full.
      uint32_t c = 0, it = 0;
      bool ok = true;
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint64_t db0 = umma_desc_sw128(smem_base);
      const uint32_t a_tmem0 = tb + kPairRingBase;
      for (long item = pair; ok && item < n_items; item += n_pairs, ++it) {
        const RowTile rt = A.tiles[item / L.n_tiles];
        const int n_mma = max(32, (rt.rows + 31) & ~31);
        const uint32_t idesc = umma2_idesc_f16(n_mma);
        const uint32_t buf = it & 1u;  // the item's accumulator buffer
        ok = __all_sync(0xffffffffu, wait_or_abort(bar_tmem_empty(buf), ((it >> 1) & 1u) ^ 1u));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tb + buf * (uint32_t)kPairN;
        for (int kt = 0; kt < KT; ++kt, ++c) {
          const uint32_t s = c % NR, sa = c % NA;
          ok = __all_sync(0xffffffffu, wait_or_abort(bar_full_a(sa), (c / NA) & 1u));
          if (!ok) break;
          tc_fence_after();
          const uint64_t db = db0 + (uint64_t)((s * (uint32_t)kPairRawBytes) >> 4);  // start-address field, 16-byte units
          const uint32_t a_tmem = a_tmem0 + sa * 32;
          if (elect_one()) {
#pragma unroll
            for (int k4 = 0; k4 < kTileK / 16; ++k4)
              umma2_f16_ts(d_tmem, a_tmem + (uint32_t)k4 * 8, db + (uint64_t)(k4 * 2), idesc, (kt | k4) ? 1u : 0u);
            umma2_commit_both(bar_retired(s));
            if (kt == KT - 1) umma2_commit_both(bar_tmem_full(buf));
          }
          __syncwarp();
        }
      }
      // everything issued has to retire before tensor memory is freed
      if (lane == 0) {
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_drain) : "memory");
        const long long t0 = clock64();
        while (!mbar_try(bar_drain, 0) && clock64() - t0 < drain_budget()) {
        }
      }
      __syncwarp();
    }
  } else if (warp < 2 + 4 * NG) {
    // ------------------------------ dequantisers (each CTA) ------------------------------
    // NG groups of four warps; group g converts the k-steps whose running number is g mod NG and
    // fills the ring slots that go with them.  thread = one of this CTA's 128 weight rows
    // (tensor-memory lane) x the 64 columns of the k-step.
    const int quarter = warp & 3;            // lanes 32*quarter .. +31 are this warp's
    const int grp = (warp - 2) >> 2;
    const int trow = quarter * 32 + lane;
    // where this lane's weight row sits in the packed tile of the stage
    const int pk_half = GATED ? (trow & 1) : 0;                       // gate/up: even lanes gate (half 0), odd lanes up (half 1)
    const int pk_row = GATED ? (int)rank * 64 + (trow >> 1) : trow;   // plain: the CTA copied only its own half
    const uint32_t leader_full_a0 = map_to_cta(bar_full_a(0), 0);
    long c = 0;
    bool ok = true;
    for (long item = pair; ok && item < n_items; item += n_pairs) {
      const RowTile rt = A.tiles[item / L.n_tiles];
      const int* emeta = reinterpret_cast<const int*>(A.weights + (size_t)rt.expert * A.expert_stride + A.meta_offset);
      const int emax = emeta[A.meta_slot];
      for (int kt = 0; kt < KT; ++kt, ++c) {
        if ((int)(c % NG) != grp) continue;
        const int s = (int)(c % NR), sa = (int)(c % NA);
        if (!wait_or_abort(bar_full_raw(s), (uint32_t)((c / NR) & 1))) {
          ok = false;
          break;
        }
        const uint8_t* packed = smem + (size_t)s * kPairRawBytes + kPairABytes + (size_t)pk_half * kHalfPacked;
        uint32_t h[2][16];
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          const uint4 cw = *reinterpret_cast<const uint4*>(packed + (blk * 128 + pk_row) * 16);
          const int e = min((int)packed[4096 + blk * 128 + pk_row], 254);  // scale byte 255 is read as 254
          const uint32_t sh2 = h2_pow2(e - emax + 13);
          uint32_t t[4];
          dequant_word(cw.x, t);
          h[blk][0] = t[0]; h[blk][1] = t[1]; h[blk][2] = t[2]; h[blk][3] = t[3];
          dequant_word(cw.y, t);
          h[blk][4] = t[0]; h[blk][5] = t[1]; h[blk][6] = t[2]; h[blk][7] = t[3];
          dequant_word(cw.z, t);
          h[blk][8] = t[0]; h[blk][9] = t[1]; h[blk][10] = t[2]; h[blk][11] = t[3];
          dequant_word(cw.w, t);
          h[blk][12] = t[0]; h[blk][13] = t[1]; h[blk][14] = t[2]; h[blk][15] = t[3];
#pragma unroll
          for (int i = 0; i < 16; ++i) h[blk][i] = hmul2_u32(h[blk][i], sh2);
        }
        // the slot was last read by k-step c - 4, whose retirement is phase (c - 4) / 8 of barrier (c - 4) % 8
        if (c >= NA && !wait_or_abort(bar_retired((int)((c - NA) % NR)), (uint32_t)(((c - NA) / NR) & 1))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t_slot = tmem_base + ((uint32_t)(quarter * 32) << 16) + kPairRingBase + (uint32_t)sa * 32;
        tmem_st16(t_slot, h[0]);
        tmem_st16(t_slot + 16, h[1]);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_full_a0 + 8u * (uint32_t)sa);
      }
    }
  } else {
    // ------------------------------ epilogue (each CTA) ------------------------------
    const int quarter = warp & 3;  // tensor-memory lanes 32*quarter .. +31 belong to this warp
    const int ew = warp - 2 - 4 * NG;
    const int c_begin = (ew >> 2) * (kPairN / 2), c_end = c_begin + kPairN / 2;  // two warps per lane quarter: 96 columns each
    const int trow = quarter * 32 + lane;
    const uint32_t leader_tmem_empty0 = map_to_cta(bar_tmem_empty(0), 0);
    long it = 0;
    bool ok = true;
    for (long item = pair; ok && item < n_items; item += n_pairs, ++it) {
      const RowTile rt = A.tiles[item / L.n_tiles];
      const int nt = (int)(item % L.n_tiles);
      const uint8_t* ebase = A.weights + (size_t)rt.expert * A.expert_stride;
      const float* bias = reinterpret_cast<const float*>(ebase + A.bias_offset);
      const int emax = reinterpret_cast<const int*>(ebase + A.meta_offset)[A.meta_slot];
      const float oscale = ldexpf(1.0f, emax - 140);
      const int buf = (int)(it & 1);
      if (!wait_or_abort(bar_tmem_full(buf), (uint32_t)((it >> 1) & 1))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * kPairN;
      if (GATED) {
        // even lane = gate, odd lane = up of feature nt*128 + 64*rank + lane/2
        const int feat = nt * kTileW + (int)rank * 64 + (trow >> 1);
        const bool feat_ok = feat < L.N;
        float my_bias = 0.f;
        if (A.has_bias && feat_ok) my_bias = (trow & 1) ? bias[feat] : bias[A.F + feat];
        __half* out = A.a_out + (size_t)rt.row0 * A.lda + feat;
        // Both lanes of a feature's pair work: the even (gate) lane finishes the even token columns, the odd
        // (up) lane the odd ones; each gets the other's accumulator by one shuffle.  The next 16 columns are
        // on their way out of tensor memory while these are finished.
        const int odd = trow & 1;
        const int c_stop = min(rt.rows, c_end);
        auto finish16 = [&](const uint32_t (&r)[16], int c0) {
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const float m0 = fmaf(__uint_as_float(r[2 * jj]), oscale, my_bias);
            const float m1 = fmaf(__uint_as_float(r[2 * jj + 1]), oscale, my_bias);
            const float o0 = __shfl_xor_sync(0xffffffffu, m0, 1), o1 = __shfl_xor_sync(0xffffffffu, m1, 1);
            const float gate = odd ? o1 : m0;  // even lane: column 2jj, its own gate; odd lane: column 2jj+1, the partner's
            const float up = odd ? m1 : o0;
            const int col = c0 + 2 * jj + odd;
            if (feat_ok && col < rt.rows) out[(size_t)col * A.lda] = __float2half_rn(gated_act_fast(gate, up, A.act));
          }
        };
        uint32_t ra[16], rb[16];
        if (c_begin < c_stop) tmem_ld16(t_acc + c_begin, ra);
        for (int c0 = c_begin; c0 < c_stop; c0 += 32) {
          tmem_ld_wait();
          if (c0 + 16 < c_stop) tmem_ld16(t_acc + c0 + 16, rb);
          finish16(ra, c0);
          if (c0 + 16 < c_stop) {
            tmem_ld_wait();
            if (c0 + 32 < c_stop) tmem_ld16(t_acc + c0 + 32, ra);
            finish16(rb, c0 + 16);
          }
        }
      } else {
        const int n = nt * 2 * kTileW + (int)rank * kTileW + trow;
        const bool n_ok = n < L.N;
        const float my_bias = (A.has_bias && n_ok) ? bias[2 * A.F + n] : 0.f;
        const int c_stop = min(rt.rows, c_end);
        auto finish16 = [&](const uint32_t (&r)[16], int c0) {
          // lane j < 16 fetches the address of token c0 + j's output row once; every lane then reads it by shuffle
          float* my_row = nullptr;
          if (lane < 16 && c0 + lane < rt.rows) {
            const int gr = rt.row0 + c0 + lane;
            my_row = A.out_row_ptr ? A.out_row_ptr[gr]
                                   : A.y_out + (size_t)(A.out_row_map ? A.out_row_map[gr] : gr) * A.ldy;
          }
          const unsigned long long my_bits = reinterpret_cast<unsigned long long>(my_row);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float* row = reinterpret_cast<float*>(__shfl_sync(0xffffffffu, my_bits, j));
            if (n_ok && row && c0 + j < rt.rows) row[n] = __uint_as_float(r[j]) * oscale + my_bias;
          }
        };
        uint32_t ra[16], rb[16];
        if (c_begin < c_stop) tmem_ld16(t_acc + c_begin, ra);
        for (int c0 = c_begin; c0 < c_stop; c0 += 32) {
          tmem_ld_wait();
          if (c0 + 16 < c_stop) tmem_ld16(t_acc + c0 + 16, rb);
          finish16(ra, c0);
          if (c0 + 16 < c_stop) {
            tmem_ld_wait();
            if (c0 + 32 < c_stop) tmem_ld16(t_acc + c0 + 32, ra);
            finish16(rb, c0 + 16);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tmem_empty0 + 8u * (uint32_t)buf);
    }
    if (!GATED && A.out_row_ptr) __threadfence_system();  // rows written to other GPUs before the kernel is seen as done
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicOr(&A.meta[3], kDevErrWaitTimeout);
  cluster_sync_all();  // neither CTA leaves, or frees tensor memory, while the other may still use its barriers or memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------
struct PairState {
  bool available = false;
  int pairs = 0;  // CTA pairs that can be resident at once
  std::string err = "the one-CTA tensor kernel is unavailable too";
};

inline int pair_init(PairState& ps, TileState& st, int sm_count) {
  ps.available = false;
  if (!st.available) return CSK_OK;
  for (auto* f : {(const void*)k_tile2<true>, (const void*)k_tile2<false>}) {
    if (cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pair_smem_bytes()) != cudaSuccess) {
      cudaGetLastError();
      ps.err = "the kernel's shared memory cannot be reserved";
      return CSK_OK;  // the one-CTA kernel serves the tensor-core path
    }
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(sm_count & ~1));
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = pair_smem_bytes();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, k_tile2<true>, &cfg) != cudaSuccess || clusters < 1) {
    cudaGetLastError();
    ps.err = "no cluster of two CTAs can be resident";
    return CSK_OK;
  }
  ps.pairs = std::min(clusters, sm_count / 2);
  ps.available = ps.pairs >= 1;
  return CSK_OK;
}

template <bool GATED>
inline cudaError_t pair_launch_one(const PairState& ps, const CUtensorMap& map, const TileArgs& a, cudaStream_t s) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(2 * ps.pairs));
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = pair_smem_bytes();
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, k_tile2<GATED>, map, a);
}

// Both contractions on CTA pairs; same arguments as tile_launch (the token tiles are read through
// tensor maps with boxes of kPairHalfRows rows).
inline int pair_launch(const PairState& ps, TileState& st, const CUtensorMap& map_x, const CUtensorMap& map_a,
                       const uint8_t* weights, size_t expert_stride, size_t off_gu, size_t off_d, size_t off_bias,
                       size_t off_meta, const TileLayout& Lgu, const TileLayout& Ld, __half* a16, int lda, float* y, int ldy,
                       const int* out_row_map, float* const* out_row_ptr, const RowTile* tiles, int* meta, int has_bias,
                       int act, int F, cudaStream_t s, const std::function<void()>& mark, bool stall) {
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
  a.stall = stall ? 1 : 0;
  a.mat_offset = off_gu;
  a.L = Lgu;
  a.a_out = a16;
  a.lda = lda;
  a.meta_slot = 0;
  cudaError_t e = pair_launch_one<true>(ps, map_x, a, s);
  mark();
  a.mat_offset = off_d;
  a.L = Ld;
  a.y_out = y;
  a.ldy = ldy;
  a.out_row_map = out_row_map;
  a.out_row_ptr = out_row_ptr;
  a.meta_slot = 1;
  if (e == cudaSuccess) e = pair_launch_one<false>(ps, map_a, a, s);
  mark();
  if (e != cudaSuccess) {
    st.err = std::string("launch failed: ") + cudaGetErrorString(e);
    return CSK_ERR_CUDA;
  }
  return CSK_OK;
}

}  // namespace csk
