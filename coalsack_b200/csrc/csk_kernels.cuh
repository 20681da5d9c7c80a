// The small kernels around the expert contractions: MXFP4 repack, router,
// permutation by expert, gather to fp16 rows, weighted combine.
#pragma once

#include "csk_common.cuh"

namespace csk {

// ---------------------------------------------------------------------------
// Repack: 17-byte MXFP4 blocks (row-major, [rows][K/32]) -> device tile layout.
// src0 is the matrix itself, or the gate matrix of a fused gate/up pair whose
// up matrix is src1.  One thread per destination word; the last 8 "words" of a
// sub-tile record are its scale bytes.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t raw_code(const uint8_t* src, int K, int row, int col) {
  const uint8_t* blk = src + ((size_t)row * (K / 32) + col / 32) * 17;
  const int j = col & 31;
  const uint8_t byte = blk[1 + (j & 15)];
  return j < 16 ? (byte & 0xF) : (byte >> 4);
}

__global__ void k_repack(const uint8_t* __restrict__ src0, const uint8_t* __restrict__ src1,
                         uint8_t* __restrict__ dst, MatLayout L, int* __restrict__ emax_out) {
  const size_t n_words = L.bytes() / 4;
  for (size_t w = (size_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_words;
       w += (size_t)gridDim.x * blockDim.x) {
    const size_t rec = w / (kSubBytes / 4);
    const int wi = (int)(w % (kSubBytes / 4));
    const int m = (int)(rec % L.recs());  // 0 = the matrix itself / gate, 1 = up
    const int kt = (int)((rec / L.recs()) % L.k_tiles);
    const int grp = (int)(rec / ((size_t)L.recs() * L.k_tiles));
    const uint8_t* src = m ? src1 : src0;
    uint32_t out = 0;
    if (wi < kSubCodeBytes / 4) {
      const int lane = wi >> 2, word = wi & 3;
      const int g = lane >> 2, q = lane & 3;
      const int row = grp * 16 + g + ((word & 2) ? 8 : 0);
      const int col = kt * kTileK + (word & 1) * 32 + q * 8;
      if (row < L.N && col < L.K) {
#pragma unroll
        for (int i = 0; i < 8; ++i) out |= raw_code(src, L.K, row, col + i) << (4 * i);
      }
    } else {
      const int g = wi - kSubCodeBytes / 4;
      int emax = -1;
#pragma unroll
      for (int slot = 0; slot < 4; ++slot) {
        const int row = grp * 16 + g + ((slot & 2) ? 8 : 0);
        const int col = kt * kTileK + (slot & 1) * 32;
        uint32_t e = 0;  // padding: zero codes under the smallest scale
        if (row < L.N && col < L.K) {
          const uint8_t* blk = src + ((size_t)row * (L.K / 32) + col / 32) * 17;
          e = min((uint32_t)blk[0], 254u);  // scale byte 255 is read as 254: stored that way, so the kernel need not clamp
          // a block of zero codes is zero under any scale: it does not widen the matrix's exponent range
          bool any = false;
          for (int j = 1; j < 17; ++j) any = any || blk[j] != 0;
          if (any) emax = max(emax, (int)e);
        }
        out |= e << (8 * slot);
      }
      if (emax >= 0) atomicMax(emax_out, emax);  // largest scale exponent among the matrix's non-zero blocks
    }
    reinterpret_cast<uint32_t*>(dst)[w] = out;
  }
}

// Inverse of k_repack for one source matrix (which_half: 0 = the matrix itself
// or the gate half, 1 = the up half).  One thread per 17-byte block.
__global__ void k_unpack(const uint8_t* __restrict__ packed, uint8_t* __restrict__ out, MatLayout L,
                         int which_half) {
  const int kb = L.K / 32;
  const size_t n_blocks = (size_t)L.N * kb;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_blocks;
       i += (size_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / kb), blk = (int)(i % kb);
    const int grp = row / 16, r16 = row % 16;
    const int g = r16 & 7, hi = r16 >> 3;
    const int kt = blk / 2, b = blk & 1;
    const uint8_t* rec = packed + (((size_t)grp * L.k_tiles + kt) * L.recs() + which_half) * kSubBytes;
    uint8_t* o = out + i * 17;
    o[0] = rec[kSubCodeBytes + g * 4 + hi * 2 + b];
    uint32_t codes[32];
    for (int q = 0; q < 4; ++q) {
      const uint32_t w = reinterpret_cast<const uint32_t*>(rec)[(g * 4 + q) * 4 + hi * 2 + b];
      for (int t = 0; t < 8; ++t) codes[q * 8 + t] = (w >> (4 * t)) & 0xF;
    }
    for (int j = 0; j < 16; ++j) o[1 + j] = (uint8_t)(codes[j] | (codes[j + 16] << 4));
  }
}

// ---------------------------------------------------------------------------
// Router (moe_router_node::compute_impl, moe_router_node.h:140-214).
//
// The selected expert indices must equal the reference's bit for bit, and the
// reference accumulates each logit sequentially in fp32 with separate multiply
// and add.  So each (token, expert) logit is ONE thread's in-order chain of
// __fmul_rn / __fadd_rn over the hidden dimension (never contracted into an
// FMA, never reassociated).  Parallelism comes from the T*E independent chains.
// k_router_topk then selects per token: one warp, k rounds of arg-max by
// shuffles (ties -> lower expert id; the reference leaves ties unspecified),
// softmax over the selected logits (or sigmoid) exactly as the reference.
// ---------------------------------------------------------------------------
constexpr int kRouterPad = 4;       // row stride 4 mod 32 words: a quarter-warp's 128-bit loads hit distinct banks
// ring depth: four stages, three for the widest blocks (shared memory for two blocks per SM)
__host__ __device__ constexpr int router_stages(int tokens_per_block) { return tokens_per_block >= 32 ? 3 : 4; }
constexpr int kMaxTopK = 16;
constexpr int kMaxExperts = 1024;

// ch = columns of the hidden dimension per pipeline stage
inline size_t router_smem_bytes(int tokens_per_block, int ch) {
  return (size_t)router_stages(tokens_per_block) * (32 + tokens_per_block) * (ch + kRouterPad) * sizeof(float) + 128;
}

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Router weights repacked for the logits kernel: [group of 32 experts][chunk of
// CH columns][32 rows][CH + pad] floats, so that a stage of the kernel's ring
// is ONE contiguous span (one bulk copy).  Rows past E and columns past H are 0.
inline size_t router_packed_floats(int E, int H, int ch) {
  return (size_t)((E + 31) / 32) * ((H + ch - 1) / ch) * 32 * (ch + kRouterPad);
}
__global__ void k_pack_router(const float* __restrict__ wg, float* __restrict__ packed, int E, int H, int ch) {
  const int ld = ch + kRouterPad, n_chunks = (H + ch - 1) / ch;
  const size_t n = (size_t)((E + 31) / 32) * n_chunks * 32 * ld;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % ld);
    const int r = (int)((i / ld) % 32);
    const int ci = (int)((i / ((size_t)ld * 32)) % n_chunks);
    const int g = (int)(i / ((size_t)ld * 32 * n_chunks));
    const int e = g * 32 + r, d = ci * ch + c;
    packed[i] = (c < ch && e < E && d < H) ? wg[(size_t)e * H + d] : 0.f;
  }
}

// Top-k of one token's logits by one warp, then softmax over the selected
// logits (or sigmoid) exactly as the reference (moe_router_node.h:165-214).
// The logits sit in registers (lane l holds experts l, l+32, ...); each of the
// k rounds is an arg-max by shuffles (ties -> lower expert id; the reference
// leaves ties unspecified).
//
// With `bounds` (the logits then come from the fast kernel, see k_router_logits)
// one more round finds the runner-up, and the selection is CERTIFIED only if every
// gap between neighbours of the k+1 best logits exceeds the sum of their error
// bounds: the reference's own logits, which lie within those bounds, then order
// the same experts the same way.  Returns false (warp-uniform) when a gap is too
// small; the caller then sends the token through the order-faithful chain.
// CG: logits and bounds are global memory written by other blocks (read through L2); else
// they are the block's own shared memory.
// NV: logits per lane (E <= 32 * NV); the selection loops are unrolled over it.
template <bool CG, int NV>
__device__ __forceinline__ bool warp_topk_nv(const float* __restrict__ l, int E, int k, int sigmoid,
                                             float* __restrict__ out /* [k][2] */,
                                             const float* __restrict__ bounds) {
  const int lane = threadIdx.x & 31;
  float v[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i)
    v[i] = (i * 32 < E && i * 32 + lane < E) ? (CG ? __ldcg(l + i * 32 + lane) : l[i * 32 + lane]) : -INFINITY;
  float sel_v[kMaxTopK + 1];
  int sel_i[kMaxTopK + 1];
  const int rounds = bounds ? min(k + 1, E) : k;
  for (int j = 0; j < rounds; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (i * 32 < E) {  // warp-uniform
        const float x = v[i];
        if (x > bv) {  // ascending expert id within the lane: '>' keeps the lowest on ties
          bv = x;
          bi = i * 32 + lane;
        }
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    sel_v[j] = bv;
    sel_i[j] = bi;
    // the winner leaves the pool: NaN never wins a '>' test again
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (i * 32 < E && bi == i * 32 + lane) v[i] = __int_as_float(0xffc00000);
  }
  int certified = 1;
  if (bounds && lane == 0) {
    float b[kMaxTopK + 1];
    for (int j = 0; j < rounds; ++j)
      b[j] = (sel_i[j] >= 0 && sel_i[j] < E) ? (CG ? __ldcg(bounds + sel_i[j]) : bounds[sel_i[j]]) : INFINITY;
    for (int j = 0; j + 1 < rounds; ++j)
      if (!(sel_v[j] - sel_v[j + 1] > b[j] + b[j + 1])) certified = 0;  // also false for NaN
  }
  certified = __shfl_sync(0xffffffffu, certified, 0);
  if (lane == 0) {
    float w[kMaxTopK];
    if (sigmoid) {
      for (int j = 0; j < k; ++j) w[j] = 1.0f / (1.0f + expf(-sel_v[j]));
    } else {
      float mx = sel_v[0];
      for (int j = 1; j < k; ++j) mx = fmaxf(mx, sel_v[j]);
      float se = 0.f;
      for (int j = 0; j < k; ++j) {
        w[j] = expf(sel_v[j] - mx);
        se += w[j];
      }
      const float inv = se > 0.f ? 1.0f / se : 0.f;
      for (int j = 0; j < k; ++j) w[j] *= inv;
    }
    for (int j = 0; j < k; ++j) {
      out[j * 2 + 0] = (float)sel_i[j];
      out[j * 2 + 1] = w[j];
    }
  }
  return certified != 0;
}

template <bool CG = true>
__device__ __forceinline__ bool warp_topk(const float* __restrict__ l, int E, int k, int sigmoid,
                                          float* __restrict__ out /* [k][2] */,
                                          const float* __restrict__ bounds = nullptr) {
  if (E <= 32) return warp_topk_nv<CG, 1>(l, E, k, sigmoid, out, bounds);
  if (E <= 64) return warp_topk_nv<CG, 2>(l, E, k, sigmoid, out, bounds);
  if (E <= 128) return warp_topk_nv<CG, 4>(l, E, k, sigmoid, out, bounds);
  if (E <= 256) return warp_topk_nv<CG, 8>(l, E, k, sigmoid, out, bounds);
  return warp_topk_nv<CG, kMaxExperts / 32>(l, E, k, sigmoid, out, bounds);
}

struct RouterArgs {
  const float* hidden;   // [T,H], 16-byte aligned
  const float* wg;       // PACKED: router_packed layout for this CH; else [E,H], 16-byte aligned
  const float* bias;     // [E] or null
  float* logits;         // [T,E] scratch
  float* router_out;     // [T,k,2]; written when `counters` is given
  int* counters;         // one per token block, all zero between launches; null = logits only
  int* status;           // device status word or null
  int T, H, E, k, sigmoid;
  // order-faithful kernel over a token list (the fall-back pass): token_list[0 .. *n_list)
  const int* token_list;
  int* n_list;           // read at start; reset to zero, with fb_done, by the last block to finish
  int* fb_done;          // ticket of that reset
  unsigned long long* fb_total;  // running number of tokens that took the fall-back pass (statistics)
};

// A block is one producer warp (four with plain weights) plus TW consumer warps.  A
// consumer warp owns TT tokens, its lanes 32 neighbouring experts: a thread runs TT chains.
//   * expert rows: a four-stage ring of CH-column chunks filled by bulk copies
//     (cp.async.bulk, completion counted on the stage's mbarrier).  An SM starts
//     only about one bulk copy per 70-100 cycles, so with PACKED weights a stage
//     is one copy issued by one thread; with plain [E,H] weights the producers'
//     lanes issue one copy per row;
//   * token rows: each consumer warp keeps its own TT rows in a ring of the same
//     depth, filled with cp.async by the warp itself (nobody else reads them);
//   * a lane reads its own expert row with 128-bit loads (conflict-free by the
//     row padding) and the token rows by broadcast.  A chain costs one dependent
//     add per column, so a logit takes about H x (add latency) cycles however
//     many run at once: TT = 1 keeps two 32-column register blocks in flight to
//     run one chain at that speed (few tokens), larger TT trades latency for
//     fewer shared-memory reads per chain (many tokens);
//   * with `counters`, the last block to finish a token block's logits (an
//     atomic ticket after a fence) also selects the top-k for those tokens.
// Waits are bounded; a wait that runs out sets kDevErrWaitTimeout in *status
// (when given) and the block leaves.
// Bounded wait that naps between polls, for a warp that shares its scheduler with a
// warp doing the real work.
__device__ __forceinline__ bool mbar_wait_nap(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    __nanosleep(64);
    if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > wait_budget()) {
      *abort_flag = 1;
      return false;
    }
  }
}

__host__ __device__ constexpr int router_producer_warps(bool packed) { return packed ? 1 : 4; }

template <int TW, int TT, int CH, bool PACKED>
__global__ void __launch_bounds__((TW + router_producer_warps(PACKED)) * 32)
k_router_logits(const RouterArgs A) {
  extern __shared__ __align__(128) uint8_t router_smem_raw[];
  constexpr int LD = CH + kRouterPad;
  constexpr int NS = router_stages(TW * TT), NP = router_producer_warps(PACKED);
  constexpr int BT = TW * TT;                   // tokens of the block
  constexpr int stage_floats = (32 + BT) * LD;  // ws[32][LD] then hs[BT][LD]
  float* stages = reinterpret_cast<float*>(router_smem_raw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(router_smem_raw + (size_t)NS * stage_floats * sizeof(float));
  const uint32_t bar_base = smem_u32(bars);
  auto bar_full = [&](int s) { return bar_base + 8u * s; };
  auto bar_empty = [&](int s) { return bar_base + 8u * (NS + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * NS);
  volatile int* ticket = abort_flag + 1;

  const int T = A.T, H = A.H, E = A.E;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int e0 = blockIdx.y * 32;
  const int n_chunks = (H + CH - 1) / CH;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar_full(s), PACKED ? 1 : NP);
      mbar_init(bar_empty(s), TW);
    }
    *abort_flag = 0;
    *ticket = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  griddep_wait();
  griddep_launch();
  // tokens of this launch: all T, or the entries of a list built by an earlier kernel
  const int* const list = A.token_list;
  const int n_tok = list ? min(*reinterpret_cast<volatile int*>(A.n_list), T) : T;
  auto token_at = [&](int ti) { return ti < n_tok ? (list ? list[ti] : ti) : -1; };

  // A block takes the token blocks blockIdx.x, blockIdx.x + gridDim.x, ...  (one each unless the launch
  // is list-driven and the list turned out longer than the grid).  The ring's barriers carry on from
  // one token block to the next: cg0 = chunks this block has moved so far.
  for (int tb = blockIdx.x, iter = 0; tb * BT < n_tok; tb += gridDim.x, ++iter) {
  const int t0 = tb * BT;
  const int cg0 = iter * n_chunks;
  if (warp < NP) {
    // ------------------------------ producers ------------------------------
    const int n_e = min(32, E - e0);
    const bool mine = PACKED ? (warp == 0 && lane == 0) : (warp + NP * lane < n_e);
    const int row = warp + NP * lane;  // !PACKED: producer p moves expert rows p, p+NP, ...
    const int n_mine = __popc(__ballot_sync(0xffffffffu, mine));  // !PACKED: may be 0, the warp still posts its arrival
    const float* src = PACKED ? A.wg + (size_t)blockIdx.y * n_chunks * 32 * LD : A.wg + (size_t)(e0 + row) * H;
    int issued = 0;
    bool ok = true;
    if (!PACKED || n_mine) {
      for (int ci = 0; ci < n_chunks; ++ci) {
        const int cg = cg0 + ci, st = cg % NS;
        if (cg >= NS && !mbar_wait_nap(bar_empty(st), (uint32_t)((cg / NS - 1) & 1), abort_flag)) {
          ok = false;
          break;
        }
        const uint32_t dst = smem_u32(stages + (size_t)st * stage_floats);
        if (PACKED) {
          if (mine) {
            mbar_expect_tx(bar_full(st), 32 * LD * 4);
            bulk_load(dst, src + (size_t)ci * 32 * LD, 32 * LD * 4, bar_full(st));
          }
        } else {
          const int d0 = ci * CH;
          const uint32_t row_bytes = (uint32_t)min(CH, H - d0) * sizeof(float);  // H % 32 == 0: a multiple of 128
          if (lane == 0) mbar_expect_tx(bar_full(st), (uint32_t)n_mine * row_bytes);
          __syncwarp();
          if (mine) bulk_load(dst + (uint32_t)row * LD * 4, src + d0, row_bytes, bar_full(st));
        }
        ++issued;
      }
    }
    if (!ok) {
      // let the copies still in flight land before the block goes away
      for (int i = 0; i < NS && i < issued; ++i) {
        const int cg = cg0 + issued - 1 - i;
        const long long tc = clock64();
        while (!mbar_try(bar_full(cg % NS), (uint32_t)((cg / NS) & 1)) && clock64() - tc < drain_budget()) {
        }
      }
    }
  } else {
    // ------------------------------ consumers ------------------------------
    const int w = warp - NP;
    float acc[TT];
    int tok[TT];
#pragma unroll
    for (int i = 0; i < TT; ++i) {
      acc[i] = 0.f;
      tok[i] = token_at(t0 + w * TT + i);
    }
    // this warp's token rows of chunk ci -> its rows of stage ci % NS
    auto load_tokens = [&](int ci) {
      const int d0 = ci * CH;
      const int dc = min(CH, H - d0);
      const uint32_t dst = smem_u32(stages + (size_t)((cg0 + ci) % NS) * stage_floats + (32 + w * TT) * LD);
#pragma unroll
      for (int i = 0; i < TT; ++i) {
        const int t = tok[i];
        if (t >= 0)
          for (int c = lane * 4; c < dc; c += 128)
            cp_async16(dst + (uint32_t)(i * LD + c) * 4, A.hidden + (size_t)t * H + d0 + c);
      }
    };
    for (int i = 0; i < NS - 1; ++i) {
      if (i < n_chunks) load_tokens(i);
      cp_async_commit();
    }
    bool ok = true;
    for (int ci = 0; ci < n_chunks; ++ci) {
      const int cg = cg0 + ci, st = cg % NS;
      cp_async_wait<NS - 2>();  // this lane's part of the token rows of chunk ci has landed ...
      __syncwarp();             // ... and the other lanes'; the rows used in the last iteration are free
      if (ci + NS - 1 < n_chunks) load_tokens(ci + NS - 1);
      cp_async_commit();
      if (!__all_sync(0xffffffffu, mbar_wait(bar_full(st), (uint32_t)((cg / NS) & 1), abort_flag))) {  // warp-uniform
        ok = false;
        break;
      }
      const float* wp = stages + (size_t)st * stage_floats + lane * LD;
      const float* hp = stages + (size_t)st * stage_floats + (32 + w * TT) * LD;
      const int dc = min(CH, H - ci * CH);
      if (dc < CH) {
        // last, partial chunk: the code below always walks CH columns, so the missing ones must
        // multiply to zero.  Every lane clears the tail of its own expert row (stale but written
        // only with zeros by anyone) and of the warp's token rows.
        float* wrow = stages + (size_t)st * stage_floats + lane * LD;
        for (int c = dc; c < CH; ++c) wrow[c] = 0.f;
        float* hrow = stages + (size_t)st * stage_floats + (32 + w * TT) * LD;
        for (int i = 0; i < TT; ++i)
          for (int c = dc + lane; c < CH; c += 32) hrow[i * LD + c] = 0.f;
        __syncwarp();
      }
      if (TT == 1) {
        // 32-column blocks, straight-line code for the whole chunk.  The add chain issues one
        // instruction per four cycles; the loads and the (independent) products of the NEXT block
        // are written between its adds so they go into those idle issue slots.
        constexpr int NBLK = CH / 32;
        float p[2][32];
        float a = acc[0];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 wv = *reinterpret_cast<const float4*>(wp + i * 4);
          const float4 hv = *reinterpret_cast<const float4*>(hp + i * 4);
          p[0][4 * i] = __fmul_rn(hv.x, wv.x);
          p[0][4 * i + 1] = __fmul_rn(hv.y, wv.y);
          p[0][4 * i + 2] = __fmul_rn(hv.z, wv.z);
          p[0][4 * i + 3] = __fmul_rn(hv.w, wv.w);
        }
#pragma unroll
        for (int blk = 0; blk < NBLK; ++blk) {
          const int cur = blk & 1, nxt = cur ^ 1;
          float4 wv[8], hv[8];
          if (blk + 1 < NBLK) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              wv[i] = *reinterpret_cast<const float4*>(wp + (blk + 1) * 32 + i * 4);
              hv[i] = *reinterpret_cast<const float4*>(hp + (blk + 1) * 32 + i * 4);
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            a = __fadd_rn(a, p[cur][4 * i]);
            if (blk + 1 < NBLK) p[nxt][4 * i] = __fmul_rn(hv[i].x, wv[i].x);
            a = __fadd_rn(a, p[cur][4 * i + 1]);
            if (blk + 1 < NBLK) p[nxt][4 * i + 1] = __fmul_rn(hv[i].y, wv[i].y);
            a = __fadd_rn(a, p[cur][4 * i + 2]);
            if (blk + 1 < NBLK) p[nxt][4 * i + 2] = __fmul_rn(hv[i].z, wv[i].z);
            a = __fadd_rn(a, p[cur][4 * i + 3]);
            if (blk + 1 < NBLK) p[nxt][4 * i + 3] = __fmul_rn(hv[i].w, wv[i].w);
          }
        }
        acc[0] = a;
      } else {
#pragma unroll 4
        for (int d = 0; d < CH; d += 4) {
          const float4 wv = *reinterpret_cast<const float4*>(wp + d);
          float4 hv[TT];
#pragma unroll
          for (int i = 0; i < TT; ++i) hv[i] = *reinterpret_cast<const float4*>(hp + i * LD + d);
#pragma unroll
          for (int i = 0; i < TT; ++i) {
            float a = acc[i];
            a = __fadd_rn(a, __fmul_rn(hv[i].x, wv.x));
            a = __fadd_rn(a, __fmul_rn(hv[i].y, wv.y));
            a = __fadd_rn(a, __fmul_rn(hv[i].z, wv.z));
            a = __fadd_rn(a, __fmul_rn(hv[i].w, wv.w));
            acc[i] = a;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty(st));
    }
    cp_async_wait<0>();
    if (ok) {
      const int e = e0 + lane;
      const float b = (A.bias && e < E) ? A.bias[e] : 0.f;
#pragma unroll
      for (int i = 0; i < TT; ++i) {
        const int t = tok[i];
        if (t >= 0 && e < E) A.logits[(size_t)t * E + e] = __fadd_rn(acc[i], b);
      }
      __threadfence();  // the logits before the block's ticket below
    }
  }
  __syncthreads();
  if (*abort_flag) break;  // a wait ran out: the ring's state is unknown, the block stops here

  // ---- the last block of this token block selects the top-k ----
  if (A.counters != nullptr) {
    if (tid == 0) {
      int last = 1;
      if (gridDim.y > 1) {
        __threadfence();  // this block's logits before its ticket
        last = atomicAdd(&A.counters[tb], 1) == (int)gridDim.y - 1;
        if (last) {
          A.counters[tb] = 0;  // ready for the next launch
          __threadfence();     // the other blocks' logits after their tickets
        }
      }
      *ticket = last;
    }
    __syncthreads();
    if (*ticket) {
      for (int i = warp; i < BT; i += TW + NP) {
        const int t = token_at(t0 + i);
        if (t < 0) continue;
        warp_topk(A.logits + (size_t)t * E, E, A.k, A.sigmoid, A.router_out + (size_t)t * A.k * 2);
      }
    }
    __syncthreads();  // `ticket` is rewritten by the next token block
  }
  }  // token blocks of this block

  if (tid == 0 && *abort_flag && A.status) atomicOr(A.status, kDevErrWaitTimeout);
  if (list && tid == 0) {
    // every block of a list-driven launch, busy or idle, has read the list's length by now: the last
    // one to get here clears it for the next step
    __threadfence();
    if (atomicAdd(A.fb_done, 1) == (int)(gridDim.x * gridDim.y) - 1) {
      if (A.fb_total) atomicAdd(A.fb_total, (unsigned long long)n_tok);
      *A.n_list = 0;
      *A.fb_done = 0;
      __threadfence();
    }
  }
}

template <int TW, int TT, int CH, bool PACKED>
cudaError_t router_prepare_one() {
  return cudaFuncSetAttribute(k_router_logits<TW, TT, CH, PACKED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)router_smem_bytes(TW * TT, CH));
}
constexpr int kRouterChunkFew = 256, kRouterChunkMany = 128;  // columns per stage: few / many tokens
template <bool PACKED>
cudaError_t router_prepare_set() {
  cudaError_t e = router_prepare_one<1, 1, kRouterChunkFew, PACKED>();
  if (e == cudaSuccess) e = router_prepare_one<2, 1, kRouterChunkFew, PACKED>();
  if (e == cudaSuccess) e = router_prepare_one<4, 1, kRouterChunkFew, PACKED>();
  if (e == cudaSuccess) e = router_prepare_one<4, 2, kRouterChunkMany, PACKED>();
  if (e == cudaSuccess) e = router_prepare_one<4, 4, kRouterChunkMany, PACKED>();
  if (e == cudaSuccess) e = router_prepare_one<8, 4, kRouterChunkMany, PACKED>();
  return e;
}
// Lets the router kernels use more than the default 48 KB of dynamic shared
// memory.  Once per device.
inline cudaError_t router_prepare_device();

template <int TW, int TT, int CH, bool PACKED>
void launch_router_one(const RouterArgs& a, int token_slots, cudaStream_t s, bool pdl) {
  const dim3 grid((unsigned)((token_slots + TW * TT - 1) / (TW * TT)), (unsigned)((a.E + 31) / 32));
  launch_k(k_router_logits<TW, TT, CH, PACKED>, grid, dim3((TW + router_producer_warps(PACKED)) * 32),
           router_smem_bytes(TW * TT, CH), s, pdl, a);
}

// Few tokens per block while that still leaves SMs idle (a block's speed is bounded by its
// shared-memory reads: one 16-byte word per lane per four columns and chain), more chains per
// thread once the machine is full.  wg_few / wg_many: the weights packed for the two chunk
// widths (PACKED) or both the plain [E,H] matrix.  token_slots: tokens the grid is sized for
// (a.T, or for a list-driven launch the most entries the list can have).
template <bool PACKED>
inline void launch_router_logits(RouterArgs a, const float* wg_few, const float* wg_many, int sm_count,
                                 cudaStream_t s, bool pdl = false, int token_slots = -1) {
  if (token_slots < 0) token_slots = a.T;
  const int64_t token_blocks = (int64_t)token_slots * ((a.E + 31) / 32);  // blocks if every block held one token
  if (token_blocks <= 4 * (int64_t)sm_count) {
    a.wg = wg_few;
    if (token_blocks <= sm_count) launch_router_one<1, 1, kRouterChunkFew, PACKED>(a, token_slots, s, pdl);
    else if (token_blocks <= 2 * (int64_t)sm_count) launch_router_one<2, 1, kRouterChunkFew, PACKED>(a, token_slots, s, pdl);
    else launch_router_one<4, 1, kRouterChunkFew, PACKED>(a, token_slots, s, pdl);
  } else {
    a.wg = wg_many;
    if (token_blocks <= 8 * (int64_t)sm_count) launch_router_one<4, 2, kRouterChunkMany, PACKED>(a, token_slots, s, pdl);
    else if (token_blocks <= 64 * (int64_t)sm_count) launch_router_one<4, 4, kRouterChunkMany, PACKED>(a, token_slots, s, pdl);
    else launch_router_one<8, 4, kRouterChunkMany, PACKED>(a, token_slots, s, pdl);
  }
}

// ---------------------------------------------------------------------------
// Fast router with certified selection.
//
// The reference's logit is a sequential fp32 chain, which runs at the add latency and, for a
// handful of tokens, on a handful of SMs.  Here the logits are computed with fused
// multiply-adds, split over the hidden dimension across many CTAs, and every logit carries a
// rigorous bound on its distance from the reference's chain value C:
//   |C - S| <= u (sum_i |S_i| + A),  S_i the exact partial sums in column order, A = sum |h w|
//   (one rounding per product, one per addition; u = 2^-24), and for column i of 32-column
//   block j:  |S_i| <= |R_j| + A_j  (R_j the prefix at the block's start), so
//   sum_i |S_i| <= 32 sum_j |R_j| + 32 A;
//   the block-wise FMA sum itself is within u (17 A + sum_j |R_j|) of S;
//   A <= |h|_2 |w_e|_2 (Cauchy-Schwarz; |w_e|_2 precomputed, |h|_2 summed on the way).
// bound = 1.05 u (33 sum_j |R_j| + 50 |h| |w_e|) + 4 u |logit| covers both, the two roundings
// of the bias addition and the rounding of the bound's own arithmetic.  The top-k step accepts
// a selection only when the gaps between neighbours of the k+1 best logits exceed the sum of
// their bounds; every other token goes through the order-faithful chain (k_router_logits over
// the list of those tokens).  Expert indices are therefore the reference's in every case.
//
// k_router_fast: CTA = (block of 4*TPW tokens, group of 32 experts, part m of the hidden
// dimension).  A part is a run of 96-column slices; per slice the CTA stages the 32 x 96
// weight block and its tokens' 96 columns in shared memory, every lane takes ITS expert's 96
// weights into registers and runs its warp's TPW tokens against them (token values by
// broadcast loads: one shared-memory wavefront per four FMAs).  Per (token, expert, part) it
// leaves c = the part's sum and a = sum over the part's blocks of |prefix inside the part|.
// k_router_finish: one warp per token adds the parts in order (prefix P_m before part m:
// sum_j |R_j| <= sum_m (blocks_m |P_m| + a_m)), forms logits and bounds, selects and certifies.
// ---------------------------------------------------------------------------
constexpr int kFastSliceBlocks = 3;                     // 32-column blocks per slice
constexpr int kFastSliceCols = 32 * kFastSliceBlocks;   // 96
constexpr int kFastLdw = kFastSliceCols + 4;            // weight row stride in shared memory (16-byte multiple;
                                                        // a quarter-warp's 128-bit reads of one column group
                                                        // of eight neighbouring rows hit distinct banks)

struct FastRouterArgs {
  const float* hidden;  // [T,H], 16-byte aligned
  const float* wg;      // [E,H] plain, 16-byte aligned
  float2* part;         // [T][parts][E]: (c, a)
  float* hn2;           // [T][parts]: the part's share of the token row's sum of squares
  int T, H, E;
};

inline int fast_router_slices(int H) { return (H / 32 + kFastSliceBlocks - 1) / kFastSliceBlocks; }
inline size_t fast_router_smem(int tpw) { return 2 * (size_t)(32 * kFastLdw + 4 * tpw * kFastSliceCols) * sizeof(float); }

template <int TPW>
__global__ void __launch_bounds__(128) k_router_fast(const FastRouterArgs A) {
  constexpr int TB = 4 * TPW;
  constexpr int kStage = 32 * kFastLdw + TB * kFastSliceCols;  // floats: weight block, then token block
  extern __shared__ __align__(16) float fast_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int T = A.T, H = A.H, E = A.E;
  const int t_base = blockIdx.x * TB, e0 = blockIdx.y * 32;
  const int parts = gridDim.z, m = blockIdx.z;
  const int n_slices = (H / 32 + kFastSliceBlocks - 1) / kFastSliceBlocks;
  const int s_begin = n_slices * m / parts, s_end = n_slices * (m + 1) / parts;
  float R[TPW], aR[TPW], h2[TPW];
#pragma unroll
  for (int i = 0; i < TPW; ++i) R[i] = aR[i] = h2[i] = 0.f;
  griddep_wait();
  griddep_launch();
  // all 16-byte pieces of a slice are requested at once (cp.async); what lies outside the matrices is zero
  auto stage_slice = [&](int sl, int buf) {
    float* Ws = fast_smem + buf * kStage;
    float* Hs = Ws + 32 * kFastLdw;
    const int col0 = sl * kFastSliceCols;
    for (int idx = tid; idx < 32 * (kFastSliceCols / 4); idx += 128) {
      const int r = idx / (kFastSliceCols / 4), q = idx % (kFastSliceCols / 4);
      const int e = e0 + r, col = col0 + q * 4;  // H is a multiple of 32: col < H means the whole piece is inside
      float* d = Ws + r * kFastLdw + q * 4;
      if (e < E && col < H) cp_async16(smem_u32(d), A.wg + (size_t)e * H + col);
      else *reinterpret_cast<float4*>(d) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int idx = tid; idx < TB * (kFastSliceCols / 4); idx += 128) {
      const int r = idx / (kFastSliceCols / 4), q = idx % (kFastSliceCols / 4);
      const int t = t_base + r, col = col0 + q * 4;
      float* d = Hs + r * kFastSliceCols + q * 4;
      if (t < T && col < H) cp_async16(smem_u32(d), A.hidden + (size_t)t * H + col);
      else *reinterpret_cast<float4*>(d) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    cp_async_commit();
  };
  if (s_begin < s_end) stage_slice(s_begin, 0);
  for (int sl = s_begin; sl < s_end; ++sl) {
    const int buf = (sl - s_begin) & 1;
    if (sl + 1 < s_end) {
      stage_slice(sl + 1, buf ^ 1);  // the other buffer's readers finished before the barrier that ended slice sl - 1
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* Ws = fast_smem + buf * kStage;
    const float* Hs = Ws + 32 * kFastLdw;
    float w[kFastSliceCols];
#pragma unroll
    for (int q = 0; q < kFastSliceCols / 4; ++q) {
      const float4 v = *reinterpret_cast<const float4*>(Ws + lane * kFastLdw + q * 4);
      w[q * 4 + 0] = v.x;
      w[q * 4 + 1] = v.y;
      w[q * 4 + 2] = v.z;
      w[q * 4 + 3] = v.w;
    }
    // TG tokens at a time: 2 * TG independent FMA chains and TG broadcast loads in flight per lane
    constexpr int TG = TPW < 4 ? TPW : 4;
#pragma unroll
    for (int i0 = 0; i0 < TPW; i0 += TG) {
      const float* hp = Hs + (warp * TPW + i0) * kFastSliceCols;
#pragma unroll
      for (int blk = 0; blk < kFastSliceBlocks; ++blk) {
        float b0[TG], b1[TG];
#pragma unroll
        for (int j = 0; j < TG; ++j) b0[j] = b1[j] = 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float4 hv[TG];
#pragma unroll
          for (int j = 0; j < TG; ++j)
            hv[j] = *reinterpret_cast<const float4*>(hp + j * kFastSliceCols + blk * 32 + q * 4);
#pragma unroll
          for (int j = 0; j < TG; ++j) {
            b0[j] = fmaf(hv[j].x, w[blk * 32 + q * 4 + 0], b0[j]);
            b1[j] = fmaf(hv[j].y, w[blk * 32 + q * 4 + 1], b1[j]);
          }
#pragma unroll
          for (int j = 0; j < TG; ++j) {
            b0[j] = fmaf(hv[j].z, w[blk * 32 + q * 4 + 2], b0[j]);
            b1[j] = fmaf(hv[j].w, w[blk * 32 + q * 4 + 3], b1[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < TG; ++j) {
          const float hx = hp[j * kFastSliceCols + blk * 32 + lane];  // the warp's lanes share the row's squares
          h2[i0 + j] = fmaf(hx, hx, h2[i0 + j]);
          R[i0 + j] += b0[j] + b1[j];
          aR[i0 + j] += fabsf(R[i0 + j]);
        }
      }
    }
    __syncthreads();  // this buffer is refilled during the next slice
  }
  const int e = e0 + lane;
#pragma unroll
  for (int i = 0; i < TPW; ++i) {
    const int t = t_base + warp * TPW + i;
    float q = h2[i];
    if (blockIdx.y == 0) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    }
    if (t < T) {
      if (e < E) A.part[((size_t)t * parts + m) * E + e] = make_float2(R[i], aR[i]);
      if (blockIdx.y == 0 && lane == 0) A.hn2[(size_t)t * parts + m] = q;
    }
  }
}

struct FinishRouterArgs {
  const float2* part;   // [T][parts][E]
  const float* hn2;     // [T][parts]
  const float* bias;    // [E] or null
  const float* wnorm;   // [E] upper bounds of the gate rows' 2-norms
  float* router_out;    // [T,k,2]
  int* fb_list;         // tokens whose selection is not certified ...
  int* fb_count;        // ... and how many (zero between steps)
  int T, H, E, k, sigmoid, parts;
};

constexpr int kFastMaxParts = 32;

// One block per token, one thread per expert (at most 256 threads; more experts take turns): a
// thread's loads of its expert's parts are all in flight at once; logits and bounds meet in
// shared memory, where warp 0 selects.
__global__ void __launch_bounds__(256) k_router_finish(const FinishRouterArgs A) {
  __shared__ float s_logit[kMaxExperts], s_bound[kMaxExperts];
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int parts = A.parts, E = A.E;
  const int n_slices = (A.H / 32 + kFastSliceBlocks - 1) / kFastSliceBlocks;
  griddep_wait();
  griddep_launch();
  float h2 = lane < parts ? __ldcg(A.hn2 + (size_t)t * parts + lane) : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) h2 += __shfl_xor_sync(0xffffffffu, h2, o);  // every warp, all lanes
  const float hn = sqrtf(h2) * 1.001f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float2 v[kFastMaxParts];
#pragma unroll
    for (int m = 0; m < kFastMaxParts; ++m)
      v[m] = m < parts ? __ldcg(A.part + ((size_t)t * parts + m) * E + e) : make_float2(0.f, 0.f);
    const float bias = A.bias ? A.bias[e] : 0.f;
    const float wn = A.wnorm[e];
    float P = 0.f, sr = 0.f;
#pragma unroll
    for (int m = 0; m < kFastMaxParts; ++m) {
      if (m < parts) {
        const int blocks = kFastSliceBlocks * (n_slices * (m + 1) / parts - n_slices * m / parts);
        sr += (float)blocks * fabsf(P) + v[m].y;
        P += v[m].x;
      }
    }
    const float logit = __fadd_rn(P, bias);
    s_logit[e] = logit;
    s_bound[e] = 6.3e-8f * (33.f * sr + 50.f * hn * wn) + 2.4e-7f * fabsf(logit) + 1e-30f;
  }
  __syncthreads();
  if (threadIdx.x >= 32) return;
  const bool sure = warp_topk<false>(s_logit, E, A.k, A.sigmoid, A.router_out + (size_t)t * A.k * 2, s_bound);
  if (!sure && lane == 0) A.fb_list[atomicAdd(A.fb_count, 1)] = t;  // at most one entry per token
}

inline cudaError_t router_prepare_device() {
  cudaError_t e = router_prepare_set<true>();
  if (e == cudaSuccess) e = router_prepare_set<false>();
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k_router_fast<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fast_router_smem(8));
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k_router_fast<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fast_router_smem(16));
  return e;
}

// 2-norm of every expert's gate row, rounded up (the fast router's Cauchy-Schwarz term).
__global__ void k_router_wnorm(const float* __restrict__ wg, float* __restrict__ wnorm, int E, int H) {
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= E) return;
  float acc = 0.f;
  for (int d = lane; d < H; d += 32) acc = fmaf(wg[(size_t)e * H + d], wg[(size_t)e * H + d], acc);
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) wnorm[e] = sqrtf(acc) * 1.001f;
}

__global__ void __launch_bounds__(128)
k_router_topk(const float* __restrict__ logits, float* __restrict__ router_out, int T, int E, int k, int sigmoid) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  warp_topk(logits + (size_t)t * E, E, k, sigmoid, router_out + (size_t)t * k * 2);
}

// ---------------------------------------------------------------------------
// Permutation by expert ("dispatch").  The reference's dispatch
// (moe_weight_fetch_node::extract_selected_experts, moe_weight_fetch_node.h:31-60,
// and the per-expert membership scans of expert_mlp_node.h:784-822) only finds
// WHICH experts were selected; grouping the (token, expert) rows by expert is
// what lets every expert's weights be read once.
//
// meta layout (int32): [0] row tiles, [1] total rows, [2] distinct experts,
//                      [3] device status word (or-ed kDevErr*), [4..7] spare.
// ---------------------------------------------------------------------------
__global__ void k_hist(const float* __restrict__ router_out, int n_pairs, int E, int only_expert,
                       int* __restrict__ counts, int* __restrict__ meta) {
  extern __shared__ int sc[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) sc[e] = 0;
  __syncthreads();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += gridDim.x * blockDim.x) {
    const int e = (int)router_out[2 * (size_t)i];
    if (e < 0 || e >= E) {
      atomicOr(&meta[3], kDevErrExpertRange);
      continue;
    }
    if (only_expert >= 0 && e != only_expert) continue;
    atomicAdd(&sc[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    if (sc[e]) atomicAdd(&counts[e], sc[e]);
}

// Exclusive scan of the per-expert row counts, row-tile list for tiles of
// `tile_rows` rows, cursor reset.  One block of 1024 threads, E <= 1024.
// counts are indexed by GLOBAL expert id; tiles carry the id local to this
// device (e - e_begin); rows of experts outside [e_begin, e_begin+e_count) get
// offsets but no tiles (under expert parallelism they belong to other devices).
//
// With router_out given (small batches) the block first builds the histogram
// itself -- counts and the status word then need no clearing beforehand and the
// whole plan is one launch.
//
// With row_of_pair / pair_of_row given as well (the streaming kernel then gathers its token
// rows itself) the block also places every pair: row_of_pair[i] = its row in the grouped
// order (-1: not placed), pair_of_row[row] = i.  Which row of its expert's segment a pair
// gets depends on the order of the block's atomics; a row's value does not depend on it.
__global__ void __launch_bounds__(1024)
k_scan(int* __restrict__ counts, int E, int e_begin, int e_count, int tile_rows, int max_rows,
       int max_tiles, const uint8_t* __restrict__ resident, int* __restrict__ offsets,
       int* __restrict__ cursor, RowTile* __restrict__ tiles, int* __restrict__ meta,
       const float* __restrict__ router_out, int n_pairs, int only_expert,
       int* __restrict__ row_of_pair = nullptr, int* __restrict__ pair_of_row = nullptr) {
  __shared__ int s_row_off[1025];
  __shared__ int s_tile_off[1025];
  __shared__ int s_warp[2][32];
  __shared__ int s_distinct;
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  if (e == 0) s_distinct = 0;
  griddep_wait();
  griddep_launch();
  if (router_out) {
    s_tile_off[e] = 0;  // serves as the histogram until the scan below overwrites it
    if (e == 0) meta[3] = 0;
    __syncthreads();
    for (int i = e; i < n_pairs; i += 1024) {
      const int x = (int)router_out[2 * (size_t)i];
      if (x < 0 || x >= E) {
        atomicOr(&meta[3], kDevErrExpertRange);
      } else if (only_expert < 0 || x == only_expert) {
        atomicAdd(&s_tile_off[x], 1);
      }
    }
  }
  __syncthreads();
  const int c = router_out ? s_tile_off[e] : (e < E ? counts[e] : 0);
  if (router_out && e < E) counts[e] = c;
  __syncthreads();  // every thread holds its count before s_tile_off is reused
  const bool local = e >= e_begin && e < e_begin + e_count;
  const int nt = local ? (c + tile_rows - 1) / tile_rows : 0;
  if (c > 0) {
    atomicAdd(&s_distinct, 1);
    if (local && resident && !resident[e - e_begin]) atomicOr(&meta[3], kDevErrNotResident);
  }
  // block-wide inclusive scans of (c, nt)
  int rc = c, rt = nt;
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, rc, o), b = __shfl_up_sync(0xffffffffu, rt, o);
    if (lane >= o) {
      rc += a;
      rt += b;
    }
  }
  if (lane == 31) {
    s_warp[0][warp] = rc;
    s_warp[1][warp] = rt;
  }
  __syncthreads();
  if (warp == 0) {
    int a = s_warp[0][lane], b = s_warp[1][lane];
    for (int o = 1; o < 32; o <<= 1) {
      const int ua = __shfl_up_sync(0xffffffffu, a, o), ub = __shfl_up_sync(0xffffffffu, b, o);
      if (lane >= o) {
        a += ua;
        b += ub;
      }
    }
    s_warp[0][lane] = a;
    s_warp[1][lane] = b;
  }
  __syncthreads();
  const int base_c = warp ? s_warp[0][warp - 1] : 0, base_t = warp ? s_warp[1][warp - 1] : 0;
  const int row_off = base_c + rc - c, tile_off = base_t + rt - nt;
  s_row_off[e] = row_off;
  s_tile_off[e] = tile_off;
  if (e < E) {
    offsets[e] = row_off;
    cursor[e] = 0;
  }
  const int total_rows = s_warp[0][31], total_tiles = s_warp[1][31];
  if (e == 0) {
    s_row_off[1024] = total_rows;
    s_tile_off[1024] = total_tiles;
    offsets[E] = total_rows;
    const bool over = total_rows > max_rows || total_tiles > max_tiles;
    if (over) atomicOr(&meta[3], kDevErrCapacity);
    meta[0] = over ? 0 : total_tiles;
    meta[1] = total_rows;
  }
  __syncthreads();
  if (e == 0) meta[2] = s_distinct;
  if (router_out && row_of_pair) {
    // s_warp is free now: reuse nothing of it; the cursors live in s_cur
    __shared__ int s_cur[1024];
    s_cur[e] = 0;
    __syncthreads();
    const bool over = total_rows > max_rows || total_tiles > max_tiles;
    for (int i = e; i < n_pairs; i += 1024) {
      const int x = (int)router_out[2 * (size_t)i];
      int pos = -1;
      if (!over && x >= 0 && x < E && (only_expert < 0 || x == only_expert)) {
        pos = s_row_off[x] + atomicAdd(&s_cur[x], 1);
        if (pos >= max_rows) pos = -1;
      }
      row_of_pair[i] = pos;
      if (pos >= 0) pair_of_row[pos] = i;
    }
  }
  if (total_rows > max_rows || total_tiles > max_tiles) return;
  for (int i = threadIdx.x; i < total_tiles; i += blockDim.x) {
    // largest expert x with s_tile_off[x] <= i (experts without tiles repeat an offset)
    int lo = 0, hi = 1023;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_tile_off[mid] <= i) lo = mid; else hi = mid - 1;
    }
    // step back over empty experts that share the offset: the owner is the last
    // expert with that offset that actually has tiles, i.e. the largest index.
    const int cnt = (lo < 1023 ? s_row_off[lo + 1] : s_row_off[1024]) - s_row_off[lo];
    // An expert with two to four tensor-core tiles gets them equally tall (rounded up to the MMA's 16-row
    // step) instead of full tiles and a short rest: a tile's cost is nearly flat below ~175 rows, so
    // 128 + 128 rows are cheaper than 192 + 64.  (More tiles: only the last one would change.)
    const int ntl = (cnt + tile_rows - 1) / tile_rows;
    int per = tile_rows;
    if (tile_rows >= 64 && ntl >= 2 && ntl <= 4) per = min(tile_rows, (((cnt + ntl - 1) / ntl) + 15) & ~15);
    const int r = (i - s_tile_off[lo]) * per;
    RowTile t;
    t.expert = lo - e_begin;
    t.row0 = s_row_off[lo] + r;
    t.rows = min(per, cnt - r);
    t.pad = 0;
    tiles[i] = t;
  }
}

// One warp per (token, slot) pair: claim a row in the expert's segment, record
// the maps, and write the token's hidden row there as fp16 (times the routing
// weight when it is applied before the expert).
__global__ void k_scatter(const float* __restrict__ router_out, const float* __restrict__ hidden,
                          int n_pairs, int k, int H, int E, int only_expert,
                          const int* __restrict__ offsets, int* __restrict__ cursor,
                          int* __restrict__ row_of_pair, __half* __restrict__ x16, int ldx,
                          int max_rows, int weight_before_ffn) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  griddep_wait();
  griddep_launch();
  for (int i = blockIdx.x * warps_per_block + (threadIdx.x >> 5); i < n_pairs;
       i += gridDim.x * warps_per_block) {
    const int e = (int)router_out[2 * (size_t)i];
    const float w = router_out[2 * (size_t)i + 1];
    int pos = -1;
    if (e >= 0 && e < E && (only_expert < 0 || e == only_expert)) {
      if (lane == 0) pos = offsets[e] + atomicAdd(&cursor[e], 1);
      pos = __shfl_sync(0xffffffffu, pos, 0);
      if (pos >= max_rows) pos = -1;
    }
    if (lane == 0) row_of_pair[i] = pos;
    if (pos < 0) continue;
    const float* src = hidden + (size_t)(i / k) * H;
    __half* dst = x16 + (size_t)pos * ldx;
    const float mul = weight_before_ffn ? w : 1.0f;
    for (int d = lane * 4; d < H; d += 128) {
      const float4 v = *reinterpret_cast<const float4*>(src + d);
      __half2 a = __floats2half2_rn(v.x * mul, v.y * mul);
      __half2 b = __floats2half2_rn(v.z * mul, v.w * mul);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&a);
      o.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(dst + d) = o;
    }
  }
}

// ---------------------------------------------------------------------------
// Weighted combine (expert_merge_node::compute, expert_merge_node.h:88-131):
// out[t] = sum over slots j = 0..k-1, in that order, of w[t,j] * y[row(t,j)],
// a separate multiply and add per term as the reference does.  mode 1 is the
// dense single-expert output of expert_mlp_node (expert_mlp_node.h:503-529):
// the token's row unweighted, or zeros.
// ---------------------------------------------------------------------------
//
// carry (optional; the host entry point that runs a batch in several passes): block 0 folds this
// pass's status word into a sticky one and adds its per-expert row counts to running totals --
// layout: carry[0] = sticky status, carry[1 .. E] = rows per expert.
__global__ void k_combine(const float* __restrict__ router_out, const int* __restrict__ row_of_pair,
                          const float* __restrict__ y, int ldy, float* __restrict__ out, int T,
                          int k, int H, int unweighted, int dense_single,
                          const int* __restrict__ meta = nullptr, const int* __restrict__ counts = nullptr,
                          int* __restrict__ carry = nullptr, int E = 0, const float* __restrict__ residual = nullptr,
                          const float* __restrict__ shared_out = nullptr) {
  const int t = blockIdx.x;
  griddep_wait();
  griddep_launch();
  if (carry && t == 0) {
    if (threadIdx.x == 0 && meta[3]) atomicOr(&carry[0], meta[3]);
    for (int e = threadIdx.x; e < E; e += blockDim.x) carry[1 + e] += counts[e];
  }
  if (t >= T) return;
  for (int d = threadIdx.x * 4; d < H; d += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; ++j) {
      const int row = row_of_pair[(size_t)t * k + j];
      if (row < 0) continue;
      const float4 v = *reinterpret_cast<const float4*>(y + (size_t)row * ldy + d);
      if (dense_single) {
        acc = v;
        break;
      }
      if (unweighted) {
        acc.x = __fadd_rn(acc.x, v.x);
        acc.y = __fadd_rn(acc.y, v.y);
        acc.z = __fadd_rn(acc.z, v.z);
        acc.w = __fadd_rn(acc.w, v.w);
      } else {
        const float w = router_out[((size_t)t * k + j) * 2 + 1];
        acc.x = __fadd_rn(acc.x, __fmul_rn(w, v.x));
        acc.y = __fadd_rn(acc.y, __fmul_rn(w, v.y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(w, v.z));
        acc.w = __fadd_rn(acc.w, __fmul_rn(w, v.w));
      }
    }
    if (shared_out) {
      // the shared expert's dense FFN on the same rows: add(merge output, shared output), llm_engine.cpp:766-769
      const float4 sh = *reinterpret_cast<const float4*>(shared_out + (size_t)t * H + d);
      acc.x = __fadd_rn(acc.x, sh.x);
      acc.y = __fadd_rn(acc.y, sh.y);
      acc.z = __fadd_rn(acc.z, sh.z);
      acc.w = __fadd_rn(acc.w, sh.w);
    }
    if (residual) {
      // the residual connection around the layer: add(residual, merge output), llm_engine.cpp:773-777
      const float4 r = *reinterpret_cast<const float4*>(residual + (size_t)t * H + d);
      acc.x = __fadd_rn(r.x, acc.x);
      acc.y = __fadd_rn(r.y, acc.y);
      acc.z = __fadd_rn(r.z, acc.z);
      acc.w = __fadd_rn(r.w, acc.w);
    }
    *reinterpret_cast<float4*>(out + (size_t)t * H + d) = acc;
  }
}

// ---------------------------------------------------------------------------
// RMSNorm in front of the router (rmsnorm_node::compute_impl, rmsnorm_node.h:60-82):
// out = (x / sqrt(sum(x^2) / H + eps)) * w.  The router's expert indices must equal the
// reference's bit for bit, so its INPUT must too: the sum of squares is the reference's
// sequential fp32 chain of separate multiplies and adds (one lane walks the row, staged in
// shared memory by the whole warp), division, square root and products are the IEEE
// round-to-nearest operations the reference's scalar code performs.  One warp per token.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) k_rmsnorm(const float* __restrict__ x, const float* __restrict__ w, float eps,
                                                 float* __restrict__ out, int T, int H) {
  extern __shared__ __align__(16) float rms_rows[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  float* row = rms_rows + (size_t)warp * H;
  griddep_wait();
  griddep_launch();
  for (int t = blockIdx.x * wpb + warp; t < T; t += gridDim.x * wpb) {
    const float* src = x + (size_t)t * H;
    for (int d = lane * 4; d < H; d += 128) *reinterpret_cast<float4*>(row + d) = __ldg(reinterpret_cast<const float4*>(src + d));
    __syncwarp();
    float rms = 0.f;
    if (lane == 0) {
      float s = 0.f;
#pragma unroll 8
      for (int d = 0; d < H; ++d) s = __fadd_rn(s, __fmul_rn(row[d], row[d]));
      rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(s, (float)H), eps));
    }
    rms = __shfl_sync(0xffffffffu, rms, 0);
    for (int d = lane * 4; d < H; d += 128) {
      const float4 v = *reinterpret_cast<const float4*>(row + d);
      const float4 g = __ldg(reinterpret_cast<const float4*>(w + d));
      float4 o;
      o.x = __fmul_rn(__fdiv_rn(v.x, rms), g.x);
      o.y = __fmul_rn(__fdiv_rn(v.y, rms), g.y);
      o.z = __fmul_rn(__fdiv_rn(v.z, rms), g.z);
      o.w = __fmul_rn(__fdiv_rn(v.w, rms), g.w);
      *reinterpret_cast<float4*>(out + (size_t)t * H + d) = o;
    }
    __syncwarp();  // the row buffer is rewritten for the warp's next token
  }
}

// Router output with logical expert ids replaced by the slots their rows are grouped
// under: the primary slot, or for odd-numbered tokens the slot of the expert's second copy.
__global__ void k_ep_slots(const float* __restrict__ router, float* __restrict__ out, int n_pairs, int k, int E_logical,
                           const int* __restrict__ primary, const int* __restrict__ replica) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += gridDim.x * blockDim.x) {
    const float ef = router[2 * i];
    const int e = (int)ef;
    const int t = i / k;
    float o = -1.f;  // an id the permutation reports as out of range
    if (e >= 0 && e < E_logical) {
      const int r = replica[e];
      o = (float)((r >= 0 && (t & 1)) ? r : primary[e]);
    }
    out[2 * i] = o;
    out[2 * i + 1] = router[2 * i + 1];
  }
}

// ---------------------------------------------------------------------------
// Expert-parallel receive side.  Rows arrive as n_src segments (one per source
// device), each ordered by local expert; the contractions want them grouped by
// expert.  seg layout (int32): [0..1024] exclusive offsets of the (src, expert)
// segments in arrival order, [1025..2048] rows of the same expert that arrive
// from lower-numbered sources.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
k_ep_plan(const int* __restrict__ recv_counts, int n_src, int e_count, int e_begin,
          int* __restrict__ counts, int* __restrict__ seg) {
  __shared__ int s_warp[32];
  const int i = threadIdx.x, lane = i & 31, warp = i >> 5;
  const int n_seg = n_src * e_count;
  const int c = i < n_seg ? recv_counts[i] : 0;
  int r = c;
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, r, o);
    if (lane >= o) r += a;
  }
  if (lane == 31) s_warp[warp] = r;
  __syncthreads();
  if (warp == 0) {
    int a = s_warp[lane];
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, a, o);
      if (lane >= o) a += u;
    }
    s_warp[lane] = a;
  }
  __syncthreads();
  const int base = warp ? s_warp[warp - 1] : 0;
  seg[i] = base + r - c;
  if (i == 0) seg[1024] = s_warp[31];
  if (i < n_seg) {
    const int src = i / e_count, e = i % e_count;
    int before = 0;
    for (int s2 = 0; s2 < src; ++s2) before += recv_counts[s2 * e_count + e];
    seg[1025 + i] = before;
    if (src == 0) {
      int tot = 0;
      for (int s2 = 0; s2 < n_src; ++s2) tot += recv_counts[s2 * e_count + e];
      counts[e_begin + e] = tot;
    }
  }
}

// Blocks (x = segment, y = row slice): copy the segment's rows to their
// expert-major place and remember where each came from.  A row is ldx/8 16-byte
// words, so every thread has only a couple of independent loads per row and
// many rows are in flight across the y dimension.
__global__ void k_ep_regroup(const __half* __restrict__ recv, __half* __restrict__ x16, int ldx,
                             const int* __restrict__ seg, const int* __restrict__ offsets, int n_src,
                             int e_count, int e_begin, int* __restrict__ out_row_map) {
  const int b = blockIdx.x;
  const int e = b % e_count;
  const int src_row0 = seg[b], n = seg[b + 1] - seg[b];
  const int dst_row0 = offsets[e_begin + e] + seg[1025 + b];
  const int w16 = ldx / 8;
  for (int r = blockIdx.y; r < n; r += gridDim.y) {
    const uint4* s = reinterpret_cast<const uint4*>(recv + (size_t)(src_row0 + r) * ldx);
    uint4* d = reinterpret_cast<uint4*>(x16 + (size_t)(dst_row0 + r) * ldx);
    for (int i = threadIdx.x; i < w16; i += blockDim.x) d[i] = s[i];
    if (threadIdx.x == 0) out_row_map[dst_row0 + r] = src_row0 + r;
  }
}

// Stream path only: rows computed in expert-major order go back to arrival order.
__global__ void k_ep_ungroup(const float* __restrict__ y, float* __restrict__ ret, int H,
                             const int* __restrict__ out_row_map, int rows) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
    const float4* s = reinterpret_cast<const float4*>(y + (size_t)r * H);
    float4* d = reinterpret_cast<float4*>(ret + (size_t)out_row_map[r] * H);
    for (int i = lane; i < H / 4; i += 32) d[i] = s[i];
  }
}

// ---------------------------------------------------------------------------
// Expert parallelism over peer memory (NVLink): the dispatch writes every row
// straight into the row buffer of the rank that owns its expert slot, at its
// final expert-grouped position, and the down projection's epilogue writes
// every output row straight into the return buffer of the rank that owns the
// token.  The only collectives left are the (tiny) exchange of row counts and
// two barriers.  All cross-GPU traffic is plain stores to peer pointers.
//
// Layout of a destination's row buffer: slot-major, within a slot the rows of
// source rank 0, then 1, ...  Every rank derives all positions from the full
// count table all_counts[source][slot].
// ---------------------------------------------------------------------------
struct RowOrigin {
  int src;   // rank that sent the row
  int pair;  // index of the (token, k) pair there = row of its return buffer
};

// One block of 1024 threads, E <= 1024.  base[e] = first row, in the buffer of the
// rank owning slot e, of the rows THIS rank sends to e; cursor[e] = 0.
__global__ void __launch_bounds__(1024)
k_ep_p2p_base(const int* __restrict__ all_counts, int world, int me, int E, int e_per_rank, int max_rows,
              int* __restrict__ base, int* __restrict__ cursor, int* __restrict__ meta) {
  __shared__ int s_scan[1024];
  __shared__ int s_warp[32];
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  int tot = 0, before = 0;
  if (e < E)
    for (int s = 0; s < world; ++s) {
      const int c = all_counts[s * E + e];
      tot += c;
      if (s < me) before += c;
    }
  int r = tot;
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, r, o);
    if (lane >= o) r += a;
  }
  if (lane == 31) s_warp[warp] = r;
  __syncthreads();
  if (warp == 0) {
    int a = s_warp[lane];
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, a, o);
      if (lane >= o) a += u;
    }
    s_warp[lane] = a;
  }
  __syncthreads();
  s_scan[e] = (warp ? s_warp[warp - 1] : 0) + r - tot;  // exclusive prefix over all slots
  __syncthreads();
  if (e < E) {
    const int first = (e / e_per_rank) * e_per_rank;  // first slot of the owning rank
    const int in_rank = s_scan[e] - s_scan[first];    // rows of that rank's earlier slots
    base[e] = in_rank + before;
    cursor[e] = 0;
    if (in_rank + tot > max_rows) atomicOr(&meta[3], kDevErrCapacity);
  }
}

// One warp per (token, slot) pair: claim the next row of this rank's share of the slot on
// the owning rank, write the token's hidden row there as fp16 (peer store) with its origin.
__global__ void k_ep_p2p_scatter(const float* __restrict__ router_out, const float* __restrict__ hidden,
                                 int n_pairs, int k, int H, int E, int e_per_rank, int me,
                                 const int* __restrict__ base, int* __restrict__ cursor,
                                 __half* const* __restrict__ peer_x16, RowOrigin* const* __restrict__ peer_info,
                                 int ldx, int max_rows, int weight_before_ffn, int* __restrict__ row_of_pair,
                                 int* __restrict__ meta) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  for (int i = blockIdx.x * warps_per_block + (threadIdx.x >> 5); i < n_pairs; i += gridDim.x * warps_per_block) {
    const int e = (int)router_out[2 * (size_t)i];
    const float w = router_out[2 * (size_t)i + 1];
    int pos = -1;
    if (e >= 0 && e < E) {
      if (lane == 0) pos = base[e] + atomicAdd(&cursor[e], 1);
      pos = __shfl_sync(0xffffffffu, pos, 0);
      if (pos >= max_rows) pos = -1;
    } else if (lane == 0) {
      atomicOr(&meta[3], kDevErrExpertRange);
    }
    if (lane == 0) row_of_pair[i] = pos < 0 ? -1 : i;  // the return buffer is indexed by pair
    if (pos < 0) continue;
    const int dst_rank = e / e_per_rank;
    const float* src = hidden + (size_t)(i / k) * H;
    __half* dst = peer_x16[dst_rank] + (size_t)pos * ldx;
    if (lane == 0) peer_info[dst_rank][pos] = RowOrigin{me, i};
    const float mul = weight_before_ffn ? w : 1.0f;
    for (int d = lane * 8; d < H; d += 256) {
      const float4 v0 = *reinterpret_cast<const float4*>(src + d);
      const float4 v1 = *reinterpret_cast<const float4*>(src + d + 4);
      __half2 a = __floats2half2_rn(v0.x * mul, v0.y * mul), b = __floats2half2_rn(v0.z * mul, v0.w * mul);
      __half2 c = __floats2half2_rn(v1.x * mul, v1.y * mul), f = __floats2half2_rn(v1.z * mul, v1.w * mul);
      uint4 o;
      o.x = *reinterpret_cast<uint32_t*>(&a);
      o.y = *reinterpret_cast<uint32_t*>(&b);
      o.z = *reinterpret_cast<uint32_t*>(&c);
      o.w = *reinterpret_cast<uint32_t*>(&f);
      *reinterpret_cast<uint4*>(dst + d) = o;
    }
  }
  __threadfence_system();  // the peer stores before whatever signals their arrival
}

// counts[e] of the slots this rank owns = rows it received (all sources); zero elsewhere.
__global__ void k_ep_p2p_local_counts(const int* __restrict__ all_counts, int world, int E, int e_begin, int e_count,
                                      int* __restrict__ counts) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  int tot = 0;
  if (e >= e_begin && e < e_begin + e_count)
    for (int s = 0; s < world; ++s) tot += all_counts[s * E + e];
  counts[e] = tot;
}

// Where each received row's output goes: the pair's row of the sender's return buffer.
// Nothing is derived when the row plan overran the buffers (the expert kernels then have no
// tiles either), and a row whose origin record is not a valid (rank, pair) gets a null
// pointer, which every consumer skips, plus kDevErrPeerRow in the status word.
__global__ void k_ep_p2p_rowptr(const RowOrigin* __restrict__ info, int* __restrict__ meta,
                                float* const* __restrict__ peer_back, int H, float** __restrict__ row_ptr, int max_rows,
                                int world, int max_pairs) {
  if (meta[3] & kDevErrCapacity) return;
  const int rows = min(meta[1], max_rows);
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
    const RowOrigin o = info[r];
    const bool ok = o.src >= 0 && o.src < world && o.pair >= 0 && o.pair < max_pairs;
    row_ptr[r] = ok ? peer_back[o.src] + (size_t)o.pair * H : nullptr;
    if (!ok) atomicOr(&meta[3], kDevErrPeerRow);
  }
}

// Output rows computed into a local buffer (streaming path) -> their owners' return buffers.
__global__ void k_ep_p2p_return(const float* __restrict__ y, int H, float* const* __restrict__ row_ptr,
                                const int* __restrict__ meta, int max_rows) {
  if (meta[3] & kDevErrCapacity) return;
  const int rows = min(meta[1], max_rows);
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
    const float4* s = reinterpret_cast<const float4*>(y + (size_t)r * H);
    float4* d = reinterpret_cast<float4*>(row_ptr[r]);
    if (!d) continue;
    for (int i = lane; i < H / 4; i += 32) d[i] = s[i];
  }
  __threadfence_system();
}

// ---------------------------------------------------------------------------
// Barrier (and, with a payload, the exchange of the per-slot row counts) between the ranks of
// the peer-memory step, without a collective library: every rank owns a small sync area at
// the tail of its return buffer, which all peers can write --
//   flags[3][64]         flags[b][r] = last epoch of barrier b that rank r has reached
//   all_counts[64][E]    all_counts[r][.] = rank r's row counts of this step
// A rank stores its payload into every peer's area, fences (system scope), stores the epoch
// into its flag on every peer, then waits until all of its own flags show the epoch.  Flags only
// grow, nothing is reset.  The wait is bounded (clock budget); when it runs out the kernel sets
// kDevErrWaitTimeout and returns.  One block; ranks run on different GPUs, so no rank's wait
// depends on a kernel queued behind it on the same device.
// ---------------------------------------------------------------------------
constexpr int kEpMaxWorld = 64;
__host__ __device__ inline size_t ep_sync_ints(int E) { return (size_t)3 * kEpMaxWorld + (size_t)kEpMaxWorld * E; }

__global__ void __launch_bounds__(1024)
k_ep_p2p_sync(float* const* __restrict__ peer_back, size_t tail_floats, int me, int world, int which,
              int* __restrict__ epochs, const int* __restrict__ my_counts, int E, int* __restrict__ all_counts_out,
              int* __restrict__ meta) {
  __shared__ int s_timeout, s_epoch;
  const int tid = threadIdx.x;
  // The barrier's generation lives on the device and every launch advances its own rank's copy: all
  // ranks launch the same sequence, so their copies agree, and a captured launch sequence can be
  // replayed (a generation passed from the host would be frozen into the graph).
  if (tid == 0) {
    s_timeout = 0;
    s_epoch = ++epochs[which];
  }
  __syncthreads();
  const int epoch = s_epoch;
  if (my_counts) {
    for (int idx = tid; idx < world * E; idx += blockDim.x) {
      const int r = idx / E, e = idx % E;
      int* tail = reinterpret_cast<int*>(peer_back[r] + tail_floats);
      tail[3 * kEpMaxWorld + (size_t)me * E + e] = my_counts[e];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < world) {
    volatile int* theirs = reinterpret_cast<volatile int*>(peer_back[tid] + tail_floats);
    theirs[which * kEpMaxWorld + me] = epoch;
    volatile int* mine = reinterpret_cast<volatile int*>(peer_back[me] + tail_floats);
    const long long t0 = clock64();
    while (mine[which * kEpMaxWorld + tid] < epoch) {
      if (clock64() - t0 > 4 * wait_budget()) {
        s_timeout = 1;
        break;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (s_timeout) {
    if (tid == 0) atomicOr(&meta[8], kDevErrWaitTimeout);  // the sticky word: later stages do not clear it
    return;
  }
  if (all_counts_out) {
    const volatile int* mine = reinterpret_cast<const volatile int*>(peer_back[me] + tail_floats);
    for (int idx = tid; idx < world * E; idx += blockDim.x) all_counts_out[idx] = mine[3 * kEpMaxWorld + idx];
  }
}

}  // namespace csk
