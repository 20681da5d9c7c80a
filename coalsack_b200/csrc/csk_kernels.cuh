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
    const int sub = (int)(rec % L.subs);
    const int kt = (int)((rec / L.subs) % L.k_tiles);
    const int n_tile = (int)(rec / ((size_t)L.subs * L.k_tiles));
    uint32_t out = 0;
    if (wi < kSubCodeBytes / 4) {
      const int lane = wi >> 2, word = wi & 3;
      const int g = lane >> 2, q = lane & 3;
      int r_in_tile = sub * 16 + g + ((word & 2) ? 8 : 0);
      const int col = kt * kTileK + (word & 1) * 32 + q * 8;
      const uint8_t* src = src0;
      if (L.paired && r_in_tile >= L.BN / 2) {
        src = src1;
        r_in_tile -= L.BN / 2;
      }
      const int row = n_tile * L.rows_per_tile() + r_in_tile;
      if (row < L.N && col < L.K) {
#pragma unroll
        for (int i = 0; i < 8; ++i) out |= raw_code(src, L.K, row, col + i) << (4 * i);
      }
    } else {
      const int g = wi - kSubCodeBytes / 4;
      int emax = -1;
#pragma unroll
      for (int slot = 0; slot < 4; ++slot) {
        int r_in_tile = sub * 16 + g + ((slot & 2) ? 8 : 0);
        const int col = kt * kTileK + (slot & 1) * 32;
        const uint8_t* src = src0;
        if (L.paired && r_in_tile >= L.BN / 2) {
          src = src1;
          r_in_tile -= L.BN / 2;
        }
        const int row = n_tile * L.rows_per_tile() + r_in_tile;
        uint32_t e = 0;  // padding: zero codes under the smallest scale
        if (row < L.N && col < L.K) {
          e = src[((size_t)row * (L.K / 32) + col / 32) * 17];
          emax = max(emax, (int)e);
        }
        out |= e << (8 * slot);
      }
      if (emax >= 0) atomicMax(emax_out, emax);  // largest scale exponent of the matrix
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
    const int n_tile = row / L.rows_per_tile();
    int r_in_tile = row % L.rows_per_tile() + (which_half ? L.BN / 2 : 0);
    const int sub = r_in_tile / 16, r16 = r_in_tile % 16;
    const int g = r16 & 7, hi = r16 >> 3;
    const int kt = blk / 2, b = blk & 1;
    const uint8_t* rec = packed + (((size_t)n_tile * L.k_tiles + kt) * L.subs + sub) * kSubBytes;
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
// FMA, never reassociated).  Parallelism comes from the T*E independent chains:
// a block owns a BT x BE tile of (tokens x experts), a thread a TT x EE
// sub-tile, and both operand tiles are staged through shared memory in chunks
// of the hidden dimension so every global load is coalesced along it.
//   k_router_logits<4,4>: prefill (many tokens), 16 chains per thread, 64-column chunks
//   k_router_logits<1,1>: decode (a few tokens), one chain per thread, 4 experts per block,
//                         the block's rows staged whole where they fit
// k_router_topk then selects per token: one warp, k rounds of arg-max by
// shuffles (ties -> lower expert id; the reference leaves ties unspecified),
// softmax over the selected logits (or sigmoid) exactly as the reference.
// ---------------------------------------------------------------------------
constexpr int kRouterChunk = 64;
constexpr int kRouterPad = 4;
constexpr int kRouterThreads = 128;
constexpr int kMaxTopK = 16;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;  // src-size 0 -> the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int TT, int EE>
__global__ void __launch_bounds__(kRouterThreads)
k_router_logits(const float* __restrict__ hidden, const float* __restrict__ wg,
                const float* __restrict__ bias, float* __restrict__ logits, int T, int H, int E,
                int ntx /* threads along tokens; 128/ntx along experts */,
                int nty_used /* thread rows along experts that hold chains (<= 128/ntx) */,
                int ch /* columns of the hidden dimension staged per step */) {
  extern __shared__ __align__(16) float smem[];
  const int LD = ch + kRouterPad;
  const int BT = ntx * TT, BE = nty_used * EE;
  const int tile_floats = (BT + BE) * LD;  // one stage: hs[BT][LD] then ws[BE][LD]
  const int tid = threadIdx.x;
  const int tx = tid % ntx, ty = tid / ntx;
  const bool has_chains = ty < nty_used;
  const int nty = nty_used;
  const int t0 = blockIdx.x * BT, e0 = blockIdx.y * BE;

  float acc[TT][EE];
#pragma unroll
  for (int i = 0; i < TT; ++i)
#pragma unroll
    for (int j = 0; j < EE; ++j) acc[i][j] = 0.f;

  // asynchronous, coalesced 16-byte copies along the hidden dimension into stage `st`
  auto load_chunk = [&](int st, int d0) {
    float* base = smem + st * tile_floats;
    const int dc = min(ch, H - d0);  // H % 32 == 0 and ch % 32 == 0, so dc is a multiple of 32
    const int w = ch / 4;
    for (int i = tid; i < (BT + BE) * w; i += kRouterThreads) {
      const int r = i / w, c = (i % w) * 4;
      if (r < BT) {
        const bool ok = t0 + r < T && c < dc;
        cp_async16(base + r * LD + c, ok ? hidden + (size_t)(t0 + r) * H + d0 + c : hidden, ok);
      } else {
        const int e = e0 + r - BT;
        const bool ok = e < E && c < dc;
        cp_async16(base + r * LD + c, ok ? wg + (size_t)e * H + d0 + c : wg, ok);
      }
    }
    cp_async_commit();
  };

  const int n_chunks = (H + ch - 1) / ch;  // one chunk: everything is requested at once, one stage
  load_chunk(0, 0);
  for (int c_i = 0; c_i < n_chunks; ++c_i) {
    const int st = c_i & 1;
    if (c_i + 1 < n_chunks) {
      load_chunk(st ^ 1, (c_i + 1) * ch);  // stage st^1 was released by the barrier ending chunk c_i-1
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // thread (tx, ty) owns tokens tx + i*ntx and experts ty + j*nty: neighbouring
    // threads read neighbouring rows (stride LD = 4 mod 32 words), so the 128-bit
    // shared loads of a quarter-warp fall in distinct banks
    const float* hp = smem + st * tile_floats + tx * LD;
    const float* wp = smem + st * tile_floats + BT * LD + ty * LD;
    const int dc = min(ch, H - c_i * ch);
    if (has_chains) {
      // unrolled so the shared-memory loads of later steps are in flight while the
      // (serial) add chain of the current one retires
#pragma unroll 8
      for (int d = 0; d < dc; d += 4) {
        float4 hv[TT], wv[EE];
#pragma unroll
        for (int i = 0; i < TT; ++i) hv[i] = *reinterpret_cast<const float4*>(hp + i * ntx * LD + d);
#pragma unroll
        for (int j = 0; j < EE; ++j) wv[j] = *reinterpret_cast<const float4*>(wp + j * nty * LD + d);
#pragma unroll
        for (int i = 0; i < TT; ++i)
#pragma unroll
          for (int j = 0; j < EE; ++j) {
            float a = acc[i][j];
            a = __fadd_rn(a, __fmul_rn(hv[i].x, wv[j].x));
            a = __fadd_rn(a, __fmul_rn(hv[i].y, wv[j].y));
            a = __fadd_rn(a, __fmul_rn(hv[i].z, wv[j].z));
            a = __fadd_rn(a, __fmul_rn(hv[i].w, wv[j].w));
            acc[i][j] = a;
          }
      }
    }
    __syncthreads();
  }
  if (has_chains) {
#pragma unroll
    for (int i = 0; i < TT; ++i)
#pragma unroll
      for (int j = 0; j < EE; ++j) {
        const int t = t0 + tx + i * ntx, e = e0 + ty + j * nty;
        if (t < T && e < E) logits[(size_t)t * E + e] = __fadd_rn(acc[i][j], bias ? bias[e] : 0.f);
      }
  }
}

constexpr int kRouterSmemMax = 200 * 1024;

// Lets the router kernels use more than the default 48 KB of dynamic shared
// memory.  Once per device.
inline cudaError_t router_prepare_device() {
  cudaError_t e = cudaFuncSetAttribute(k_router_logits<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRouterSmemMax);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k_router_logits<2, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRouterSmemMax);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k_router_logits<1, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRouterSmemMax);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k_router_logits<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRouterSmemMax);
  return e;
}

// Picks the chain tile per thread so that the grid fills the machine, and launches.
inline void launch_router_logits(const float* d_hidden, const float* d_wg, const float* d_bias, float* d_logits,
                                 int64_t T, int H, int E, int sm_count, cudaStream_t s) {
  auto smem_of = [&](int BT, int BE, int ch, int stages) {
    return (size_t)stages * (BT + BE) * (ch + kRouterPad) * sizeof(float);
  };
  if (T <= 256) {
    // few tokens: one chain per thread and only 4 experts per block, so even a single
    // token spreads its E chains (and the loads of the router weights) over E/4 SMs;
    // threads without a chain still help with the copies.  When the block's rows fit
    // in shared memory whole, everything is requested at once (one round trip to L2
    // instead of one per chunk); else long double-buffered chunks.
    int ntx = 1;
    while (ntx < T && ntx < 32) ntx <<= 1;
    const int BT = ntx, BE = 4;
    int ch = (H + 31) / 32 * 32, stages = 1;
    if (smem_of(BT, BE, ch, 1) > (size_t)kRouterSmemMax) {
      stages = 2;
      ch = 480;
      while (smem_of(BT, BE, ch, 2) > (size_t)kRouterSmemMax) ch -= 32;
    }
    dim3 grid((unsigned)((T + BT - 1) / BT), (unsigned)((E + BE - 1) / BE));
    k_router_logits<1, 1><<<grid, kRouterThreads, smem_of(BT, BE, ch, stages), s>>>(
        d_hidden, d_wg, d_bias, d_logits, (int)T, H, E, ntx, BE, ch);
    return;
  }
  // threads along experts: as many as E fills with EE = 4 (E <= 16 -> 4)
  int nty = 16;
  while (nty > 4 && (nty / 2) * 4 >= E) nty >>= 1;
  const int ntx = kRouterThreads / nty;
  const long chains = (long)T * E;
  const long want_blocks = 3L * sm_count;
  const int CH = kRouterChunk;
  if (chains / (16 * kRouterThreads) >= want_blocks) {
    const int BT = ntx * 4, BE = nty * 4;
    dim3 grid((unsigned)((T + BT - 1) / BT), (unsigned)((E + BE - 1) / BE));
    k_router_logits<4, 4><<<grid, kRouterThreads, smem_of(BT, BE, CH, 2), s>>>(d_hidden, d_wg, d_bias, d_logits, (int)T, H, E, ntx, nty, CH);
  } else if (chains / (8 * kRouterThreads) >= want_blocks) {
    const int BT = ntx * 2, BE = nty * 4;
    dim3 grid((unsigned)((T + BT - 1) / BT), (unsigned)((E + BE - 1) / BE));
    k_router_logits<2, 4><<<grid, kRouterThreads, smem_of(BT, BE, CH, 2), s>>>(d_hidden, d_wg, d_bias, d_logits, (int)T, H, E, ntx, nty, CH);
  } else {
    const int BT = ntx, BE = nty * 4;
    dim3 grid((unsigned)((T + BT - 1) / BT), (unsigned)((E + BE - 1) / BE));
    k_router_logits<1, 4><<<grid, kRouterThreads, smem_of(BT, BE, CH, 2), s>>>(d_hidden, d_wg, d_bias, d_logits, (int)T, H, E, ntx, nty, CH);
  }
}

__global__ void __launch_bounds__(128)
k_router_topk(float* __restrict__ logits, float* __restrict__ router_out, int T, int E, int k,
              int sigmoid) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  float* l = logits + (size_t)t * E;
  float sel_v[kMaxTopK];
  int sel_i[kMaxTopK];
  for (int j = 0; j < k; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = l[e];
      if (v > bv || (v == bv && e < bi)) {
        bv = v;
        bi = e;
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
    __syncwarp();
    if (lane == 0 && bi < E) l[bi] = __int_as_float(0xffc00000);  // NaN: never wins a '>' test again
    __syncwarp();
  }
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
      router_out[((size_t)t * k + j) * 2 + 0] = (float)sel_i[j];
      router_out[((size_t)t * k + j) * 2 + 1] = w[j];
    }
  }
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
__global__ void __launch_bounds__(1024)
k_scan(int* __restrict__ counts, int E, int e_begin, int e_count, int tile_rows, int max_rows,
       int max_tiles, const uint8_t* __restrict__ resident, int* __restrict__ offsets,
       int* __restrict__ cursor, RowTile* __restrict__ tiles, int* __restrict__ meta,
       const float* __restrict__ router_out, int n_pairs, int only_expert) {
  __shared__ int s_row_off[1025];
  __shared__ int s_tile_off[1025];
  __shared__ int s_warp[2][32];
  __shared__ int s_distinct;
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  if (e == 0) s_distinct = 0;
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
    const int r = (i - s_tile_off[lo]) * tile_rows;
    const int cnt = (lo < 1023 ? s_row_off[lo + 1] : s_row_off[1024]) - s_row_off[lo];
    RowTile t;
    t.expert = lo - e_begin;
    t.row0 = s_row_off[lo] + r;
    t.rows = min(tile_rows, cnt - r);
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
__global__ void k_combine(const float* __restrict__ router_out, const int* __restrict__ row_of_pair,
                          const float* __restrict__ y, int ldy, float* __restrict__ out, int T,
                          int k, int H, int unweighted, int dense_single) {
  const int t = blockIdx.x;
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
    *reinterpret_cast<float4*>(out + (size_t)t * H + d) = acc;
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

}  // namespace csk
