// Tensor-core grouped contraction over repacked MXFP4 weights (the prefill-side
// kernel), written for sm_100a.
//
// The contraction is computed transposed, D[weight row, token] = W · Xᵀ, so that
// the WEIGHTS are the tensor-memory operand of tcgen05.mma and only the token
// rows go through shared memory:
//
//   * a work item is (row tile of up to 192 grouped token rows of one expert) x
//     (weight tile of 256 rows, as two halves of 128); the MMA's N is the item's
//     own row count rounded up to 16, so ragged expert sizes cost no padded
//     tensor work, and every token tile fetched from L2 feeds 256 weight rows;
//   * per 64-column k-step the producer warp issues one TMA tensor load of the
//     192 x 64 fp16 token tile (128-byte swizzle) and one bulk copy of the packed
//     weight tile (2 x 4352 bytes: codes + E8M0 scales, one contiguous span);
//   * eight dequantiser warps in two groups of four turn the packed tile into fp16
//     (cvt.e2m1x2 -> half2, times 2^(e - e_max + 13)) and write it straight into
//     tensor memory with tcgen05.st: thread = one weight row x the 64 columns of
//     the k-step, one half of the tile after the other.  The groups alternate
//     k-steps and each owns one slot of the two-slot weight ring; the first half
//     is converted before the slot is awaited.  The dequantised weights never
//     touch shared memory.  (fp16 weights -- the dense FFN, fp16 expert slices --
//     take the same route with a copy in place of the conversion.);
//   * the MMA warp runs its loop warp-wide with one elected lane issuing: per
//     k-step ONE barrier test (the slot is full), then eight tcgen05.mma (kind::f16,
//     A from tensor memory, B = the token tile via a shared-memory descriptor),
//     four per half, into two fp32 accumulators in tensor memory, then one commit
//     that releases both the shared-memory stage and the slot;
//   * twelve epilogue warps (three per lane quarter) read the accumulators (lane =
//     weight row, column = token), scale by the matrix's power of two, add the bias
//     and either apply the gated activation (the gate and the up accumulator of a
//     feature sit in the same lane, 192 columns apart; a warp finishes 64 token
//     columns) and store fp16 rows, or (plain matrix: a warp finishes 128 of the
//     two halves' 2 x 192 columns) store fp32 output rows.
//
// Tensor memory (512 columns): [0,384) the accumulators of the two halves, 192
// columns each; [384,512) a ring of two dequantised weight tiles, 2 x 32 columns
// (2 x 64 fp16 per row) each.
//
// fp16 operands: every MXFP4 value is value(E2M1) * 2^(e-127).  Within a matrix
// the tile holds value * 2^(e - e_max + 13) (at most 6 * 2^13; exact in fp16
// while e_max - e <= 36, smaller blocks lose bits below 2^-24 of that range) and
// the accumulator is multiplied by 2^(e_max - 140) afterwards.
//
// Every wait on an mbarrier is bounded: past a clock budget the CTA records
// kDevErrWaitTimeout in the status word, all roles leave their loops, copies in
// flight are waited for (bounded again), outstanding MMAs are drained, tensor
// memory is freed and the kernel returns.
#pragma once

#include <cuda.h>

#include <functional>
#include <string>

#include "csk_common.cuh"

namespace csk {

constexpr int kTileM = 192;          // token rows of a row tile (TMA box height, MMA N <= 192)
constexpr int kTileW = 128;          // weight rows of half a weight tile (tensor-memory lanes, MMA M)
constexpr int kDequantWarps = 8;
constexpr int kEpilogueWarps = 12;    // four lane quarters x three column ranges (sixteen measured no faster)
constexpr int kTileThreads = (2 + kDequantWarps + kEpilogueWarps) * 32;  // producer, MMA, dequantisers, epilogue
constexpr int kTileABytes = kTileM * 128;                   // token tile in shared memory
constexpr int kTileBoxes = kTileM / 32;                     // TMA boxes of 32, 64, ... kTileM rows: a row tile is fetched
                                                            // with the smallest that holds it (a 128-row tile costs 16 KB
                                                            // of L2 -> SM traffic per k-step instead of 24 KB)
struct TileMaps {
  CUtensorMap m[kTileBoxes];
};
constexpr int kHalfPacked = 4352;                           // packed half tile: 4096 codes + 256 scales
constexpr int kTilePacked = 2 * kHalfPacked;                // packed weight tile (two halves)
constexpr int kTileRawBytes = kTileABytes + 9216;           // one shared-memory stage (1024-byte multiple)
constexpr int kTileStages = 6;
// fp16 weights (dense FFN, fp16 expert slices): a half tile is 128 rows x 64 fp16 = 16 KB, rows of 128 bytes
// whose eight 16-byte pieces are stored at piece ^ (row & 7) (a quarter-warp reading one piece of eight
// neighbouring rows then hits eight different bank groups)
constexpr int kHalf16 = 128 * 128;
constexpr int kTile16 = 2 * kHalf16;
constexpr int kTileRawBytes16 = kTileABytes + kTile16;      // 57344, a 1024-byte multiple
constexpr int kTileStages16 = 3;
constexpr int kTileAStages = 2;                             // weight tiles resident in tensor memory
constexpr int kPairBoxRows = 96;                            // TMA box height of the CTA-pair kernel's half tiles
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemABase = 2 * kTileM;                 // first column of the weight ring

// Device layout of a matrix for this kernel: tiles of 256 rows x 64 columns,
// stored [n_tile][k_tile]; a tile is two halves of 128 rows, 4352 bytes each:
//   bytes    0..4095  codes: [column block 0/1][row 0..127][16 bytes = 32 codes, nibble i of
//                     word w = column 8w + i]
//   bytes 4096..4351  E8M0 scales: [column block][row]
// For the fused gate/up matrix half 0 holds the gate rows and half 1 the up rows of the
// SAME 128 features (128*n_tile ..), so a feature's two accumulators sit in one
// tensor-memory lane, 192 columns apart.
struct TileLayout {
  int N, K, paired, n_tiles, k_tiles, w16;
  __host__ __device__ int half_bytes() const { return w16 ? kHalf16 : kHalfPacked; }
  __host__ __device__ int tile_bytes() const { return 2 * half_bytes(); }
  __host__ __device__ int feats_per_tile() const { return paired ? kTileW : 2 * kTileW; }
  // halves of tile nt that hold any real row (the last tile of a plain matrix may need only one)
  __host__ __device__ int halves(int nt) const { return paired || nt * 2 * kTileW + kTileW < N ? 2 : 1; }
  __host__ __device__ size_t bytes() const { return (size_t)n_tiles * k_tiles * tile_bytes(); }
  __host__ __device__ int k_pad() const { return k_tiles * kTileK; }
};
inline TileLayout make_tile_layout(int N, int K, bool paired, bool w16 = false) {
  TileLayout L{};
  L.w16 = w16 ? 1 : 0;
  L.N = N;
  L.K = K;
  L.paired = paired ? 1 : 0;
  L.n_tiles = ceil_div(N, L.feats_per_tile());
  L.k_tiles = ceil_div(K, kTileK);
  return L;
}

// Repack of 17-byte blocks into the layout above (src1 = up matrix when paired).
__global__ void k_repack_tile(const uint8_t* __restrict__ src0, const uint8_t* __restrict__ src1,
                              uint8_t* __restrict__ dst, TileLayout L) {
  const size_t n_words = L.bytes() / 4;
  constexpr int WPT = kHalfPacked / 4;  // 1088 words per half tile
  for (size_t w = (size_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_words; w += (size_t)gridDim.x * blockDim.x) {
    const size_t half_idx = w / WPT;
    const int wi = (int)(w % WPT);
    const int half = (int)(half_idx & 1);
    const size_t tile = half_idx >> 1;
    const int kt = (int)(tile % L.k_tiles), nt = (int)(tile / L.k_tiles);
    uint32_t out = 0;
    auto source = [&](int trow, const uint8_t*& src, int& feat) {
      if (L.paired) {
        src = half ? src1 : src0;
        feat = nt * kTileW + trow;
      } else {
        src = src0;
        feat = nt * 2 * kTileW + half * kTileW + trow;
      }
    };
    if (wi < 1024) {
      const int blk = wi >> 9, trow = (wi & 511) >> 2, q = wi & 3;
      const int col = kt * kTileK + blk * 32 + q * 8;
      const uint8_t* src;
      int feat;
      source(trow, src, feat);
      if (feat < L.N && col < L.K) {
        const uint8_t* b = src + ((size_t)feat * (L.K / 32) + col / 32) * 17;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int j = q * 8 + i;
          const uint32_t code = j < 16 ? (b[1 + j] & 0xF) : (b[1 + j - 16] >> 4);
          out |= code << (4 * i);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int bi = (wi - 1024) * 4 + t;
        const int blk = bi >> 7, trow = bi & 127;
        const int col = kt * kTileK + blk * 32;
        const uint8_t* src;
        int feat;
        source(trow, src, feat);
        uint32_t e = 0;  // padding: zero codes under the smallest scale
        if (feat < L.N && col < L.K) e = src[((size_t)feat * (L.K / 32) + col / 32) * 17];
        out |= e << (8 * t);
      }
    }
    reinterpret_cast<uint32_t*>(dst)[w] = out;
  }
}

// fp16 weights, row-major [N,K] (src1 = up matrix when paired), into the fp16 tile layout.  One thread
// per 16-byte piece (eight columns of one row).
__global__ void k_repack_tile_f16(const __half* __restrict__ src0, const __half* __restrict__ src1,
                                  uint8_t* __restrict__ dst, TileLayout L) {
  const size_t n_pieces = L.bytes() / 16;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_pieces; i += (size_t)gridDim.x * blockDim.x) {
    const size_t half_idx = i >> 10;  // 1024 pieces per half tile
    const int pi = (int)(i & 1023);
    const int trow = pi >> 3, piece = (pi & 7) ^ (trow & 7);  // the piece stored here
    const int half = (int)(half_idx & 1);
    const size_t tile = half_idx >> 1;
    const int kt = (int)(tile % L.k_tiles), nt = (int)(tile / L.k_tiles);
    const __half* src = L.paired ? (half ? src1 : src0) : src0;
    const int feat = L.paired ? nt * kTileW + trow : nt * 2 * kTileW + half * kTileW + trow;
    const int col = kt * kTileK + piece * 8;
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (feat < L.N && col < L.K) {  // K is a multiple of 32: a piece is inside or outside as a whole
      const __half* p = src + (size_t)feat * L.K + col;
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        w[e] = (uint32_t)__half_as_ushort(p[2 * e]) | ((uint32_t)__half_as_ushort(p[2 * e + 1]) << 16);
      out = make_uint4(w[0], w[1], w[2], w[3]);
    }
    reinterpret_cast<uint4*>(dst)[i] = out;
  }
}

// Inverse of k_repack_tile for one source matrix (which_half: 0 = the matrix
// itself or the gate rows, 1 = the up rows).  One thread per 17-byte block.
__global__ void k_unpack_tile(const uint8_t* __restrict__ packed, uint8_t* __restrict__ out, TileLayout L,
                              int which_half) {
  const int kb = L.K / 32;
  const size_t n_blocks = (size_t)L.N * kb;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_blocks; i += (size_t)gridDim.x * blockDim.x) {
    const int feat = (int)(i / kb), blk_g = (int)(i % kb);
    const int nt = feat / L.feats_per_tile();
    const int half = L.paired ? which_half : (feat % (2 * kTileW)) / kTileW;
    const int trow = feat % kTileW;
    const int kt = blk_g / 2, blk = blk_g & 1;
    const uint8_t* tile = packed + ((size_t)nt * L.k_tiles + kt) * kTilePacked + (size_t)half * kHalfPacked;
    uint8_t* o = out + i * 17;
    o[0] = tile[4096 + blk * 128 + trow];
    const uint32_t* words = reinterpret_cast<const uint32_t*>(tile + ((size_t)blk * 128 + trow) * 16);
    uint32_t codes[32];
    for (int q = 0; q < 4; ++q)
      for (int t = 0; t < 8; ++t) codes[q * 8 + t] = (words[q] >> (4 * t)) & 0xF;
    for (int j = 0; j < 16; ++j) o[1 + j] = (uint8_t)(codes[j] | (codes[j + 16] << 4));
  }
}

struct TileState {
  bool available = false;
  std::string err;
  TileMaps maps_x{};      // grouped input rows  [rows, ldx] fp16, one map per box height
  TileMaps maps_a{};      // activated rows      [rows, lda] fp16
  CUtensorMap tmap_xh{};  // the same with boxes of half a row tile (the CTA-pair kernel's half tiles)
  CUtensorMap tmap_ah{};
  bool maps_ready = false;
  void* encode_fn = nullptr;
};

// ---- tensor-core PTX wrappers (mbarrier / bulk-copy helpers live in csk_common.cuh) ----
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\telect.sync rx|px, 0xffffffff;\n\tselp.b32 %0, 1, 0, px;\n\t}" : "=r"(pred));
  return pred != 0;
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
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileW >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem]^T
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

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
  TileLayout L;
  __half* a_out;          // GATED: activated rows [rows, lda]
  int lda;
  float* y_out;           // !GATED: output rows [rows, ldy]
  int ldy;
  const int* out_row_map; // optional indirection of output rows (!GATED)
  float* const* out_row_ptr;  // or: where each output row goes (possibly another GPU's memory); wins over the map
  const RowTile* tiles;
  const int* n_tiles_ptr;
  int* meta;              // meta[3] = device status word
  int has_bias, act, F, meta_slot;
  int stall;              // test hook: the copy role issues nothing, so every other role's wait runs out
};

inline size_t tile_smem_bytes(bool w16 = false) {
  return (w16 ? (size_t)kTileStages16 * kTileRawBytes16 : (size_t)kTileStages * kTileRawBytes) + 1024 + 512;
}

template <bool GATED, bool W16>
__global__ void __launch_bounds__(kTileThreads, 1)
k_tile(const __grid_constant__ TileMaps maps, const TileArgs A) {
  extern __shared__ __align__(1024) uint8_t tile_smem[];
  const TileLayout& L = A.L;
  const int KT = L.k_tiles;
  constexpr int NR = W16 ? kTileStages16 : kTileStages, NA = kTileAStages;
  constexpr int RAW = W16 ? kTileRawBytes16 : kTileRawBytes;  // bytes of a shared-memory stage
  constexpr int HALF_B = W16 ? kHalf16 : kHalfPacked, TILE_B = 2 * HALF_B;

  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)tile_smem + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);  // ring of [token tile | packed weight tile]
  uint8_t* ctrl = smem + (size_t)NR * RAW;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);
  const uint32_t bar_base = smem_u32(bars);
  // k-step c uses shared-memory stage c % NR and tensor-memory slot c % NA; one barrier per stage tells both the
  // copy role (stage free) and the dequantisers (slot of k-step c - NA free) that its MMAs have retired
  auto bar_full_raw = [&](int s) { return bar_base + 8u * s; };               // TMA landed
  auto bar_retired = [&](int s) { return bar_base + 8u * (8 + s); };          // MMAs of the k-step in that stage retired
  auto bar_full_a = [&](int s) { return bar_base + 8u * (16 + s); };          // both halves of the slot are in tensor memory
  const uint32_t bar_tmem_full = bar_base + 8u * 24;    // both accumulators complete
  const uint32_t bar_tmem_empty = bar_base + 8u * 26;   // all epilogue warps done reading them
  const uint32_t bar_drain = bar_base + 8u * 28;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 8 * 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 8 * 32 + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 8; ++s) {
      mbar_init(bar_full_raw(s), 1);
      mbar_init(bar_retired(s), 1);
    }
    for (int s = 0; s < NA; ++s) mbar_init(bar_full_a(s), kDequantWarps / 2);
    mbar_init(bar_tmem_full, 1);
    mbar_init(bar_tmem_empty, kEpilogueWarps);
    mbar_init(bar_drain, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                 "r"(kTmemCols)
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
      for (long item = blockIdx.x; ok && !A.stall && item < n_items; item += gridDim.x) {
        const RowTile rt = A.tiles[item / L.n_tiles];
        const int nt = (int)(item % L.n_tiles);
        const uint8_t* wsrc =
            A.weights + (size_t)rt.expert * A.expert_stride + A.mat_offset + (size_t)nt * KT * TILE_B;
        const uint32_t w_bytes = (uint32_t)L.halves(nt) * HALF_B;
        const int box = min(kTileBoxes - 1, max(0, (rt.rows + 31) / 32 - 1));
        const CUtensorMap* tmap = &maps.m[box];
        const uint32_t box_bytes = (uint32_t)(box + 1) * 32u * 128u;
        for (int kt = 0; kt < KT; ++kt) {
          if (!mbar_wait(bar_retired(s), ph ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t st = smem_base + (uint32_t)s * RAW;
          mbar_expect_tx(bar_full_raw(s), box_bytes + w_bytes);
          tma_load_2d(st, tmap, kt * kTileK, rt.row0, bar_full_raw(s));
          bulk_load(st + kTileABytes, wsrc + (size_t)kt * TILE_B, w_bytes, bar_full_raw(s));
          ++issued;
          if (++s == NR) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      if (!ok) {
        // let the copies still in flight land before the CTA goes away
        int s2 = s;
        uint32_t ph2 = ph;
        for (int i = 0; i < NR && i < issued; ++i) {
          if (--s2 < 0) {
            s2 = NR - 1;
            ph2 ^= 1;
          }
          const long long t0 = clock64();
          while (!mbar_try(bar_full_raw(s2), ph2) && clock64() - t0 < drain_budget()) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // The WHOLE warp runs this loop and one elected lane issues.  tcgen05.mma and tcgen05.commit take
    // their operands from the warp-uniform register file: in a loop that only one lane runs (a divergent
    // branch) every descriptor and address has to be moved across for every instruction, and a K=16 MMA
    // then issues once per ~185 clocks whatever its shape (measured; the pipe needs 96 for 128 x 192 x 16).
    // The loop is also kept to ONE barrier test per k-step (a satisfied test still costs ~110 clocks): the
    // token tile of a stage needs no test of its own, because the dequantisers waited for the same stage's
    // copies before they wrote the slot this warp waits for.  Both halves' MMAs are always issued; a half
    // that is padding (the last weight tile of a plain matrix) accumulates into columns nobody reads.
    {
      uint32_t c = 0, it = 0;
      bool ok = true;
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint64_t db0 = umma_desc_sw128(smem_base);
      const uint32_t a_tmem0 = tb + kTmemABase;
      for (long item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++it) {
        const RowTile rt = A.tiles[item / L.n_tiles];
        const int n_mma = max(16, (rt.rows + 15) & ~15);
        const uint32_t idesc = umma_idesc_f16(n_mma);
        ok = __all_sync(0xffffffffu, mbar_wait(bar_tmem_empty, (it & 1u) ^ 1u, abort_flag));
        if (!ok) break;
        tc_fence_after();
        for (int kt = 0; kt < KT; ++kt, ++c) {
          const uint32_t s = c % NR, sa = c % NA;
          ok = __all_sync(0xffffffffu, mbar_wait(bar_full_a(sa), (c / NA) & 1u, abort_flag));
          if (!ok) break;
          tc_fence_after();
          const uint64_t db = db0 + (uint64_t)((s * (uint32_t)RAW) >> 4);  // start-address field, 16-byte units
          const uint32_t a_tmem = a_tmem0 + sa * 64;
          if (elect_one()) {
#pragma unroll
            for (int k4 = 0; k4 < kTileK / 16; ++k4)
              umma_f16_ts(tb, a_tmem + (uint32_t)k4 * 8, db + (uint64_t)(k4 * 2), idesc, (kt | k4) ? 1u : 0u);
#pragma unroll
            for (int k4 = 0; k4 < kTileK / 16; ++k4)
              umma_f16_ts(tb + kTileM, a_tmem + 32 + (uint32_t)k4 * 8, db + (uint64_t)(k4 * 2), idesc, (kt | k4) ? 1u : 0u);
            umma_commit(bar_retired(s));
            if (kt == KT - 1) umma_commit(bar_tmem_full);
          }
          __syncwarp();
        }
      }
      // everything issued has to retire before tensor memory is freed
      if (lane == 0) {
        umma_commit(bar_drain);
        const long long t0 = clock64();
        while (!mbar_try(bar_drain, 0) && clock64() - t0 < drain_budget()) {
        }
      }
      __syncwarp();
    }
  } else if (warp < 2 + kDequantWarps) {
    // ------------------------------ dequantisers ------------------------------
    // Two groups of four warps; group g converts the k-steps whose running number is g mod 2
    // and owns slot g of the tensor-memory weight ring.  thread = weight row (tensor-memory
    // lane) x the 64 columns of the k-step, one half after the other: the first half is
    // converted BEFORE the slot is awaited (so only the store is on the slot's critical path),
    // the second while the MMAs of the first run.
    const int quarter = warp & 3;            // lanes 32*quarter .. +31 are this warp's
    const int grp = (warp - 2) >> 2;         // which k-steps / which slot
    const int trow = quarter * 32 + lane;
    long c = 0;                              // running k-step number of this CTA
    bool ok = true;
    auto convert = [&](const uint8_t* packed, int emax, uint32_t (&h)[2][16]) {
      if (W16) {  // the row's 64 fp16 values as they are: eight 16-byte pieces, stored at piece ^ (row & 7)
        const uint8_t* row = packed + trow * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 v = *reinterpret_cast<const uint4*>(row + ((j ^ (trow & 7)) << 4));
          h[j >> 2][(j & 3) * 4 + 0] = v.x;
          h[j >> 2][(j & 3) * 4 + 1] = v.y;
          h[j >> 2][(j & 3) * 4 + 2] = v.z;
          h[j >> 2][(j & 3) * 4 + 3] = v.w;
        }
        return;
      }
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        const uint4 cw = *reinterpret_cast<const uint4*>(packed + (blk * 128 + trow) * 16);
        const int e = min((int)packed[4096 + blk * 128 + trow], 254);  // scale byte 255 is read as 254
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
    };
    for (long item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
      const RowTile rt = A.tiles[item / L.n_tiles];
      const int halves = L.halves((int)(item % L.n_tiles));
      const int* emeta = reinterpret_cast<const int*>(A.weights + (size_t)rt.expert * A.expert_stride + A.meta_offset);
      const int emax = emeta[A.meta_slot];
      for (int kt = 0; kt < KT; ++kt, ++c) {
        if ((int)(c & 1) != grp) continue;
        const int s = (int)(c % NR);
        const uint32_t ph = (uint32_t)((c / NR) & 1);
        if (NR % 2 != 0 && c >= NR) {
          // An odd ring hands a stage to the two groups in turn, so this group never saw the stage's previous
          // fill complete: were that fill still in flight (copies may complete out of order), the parity test
          // below would take the fill before it for the one awaited, and the conversion would read the
          // wrong k-step.  The stage's previous MMAs having retired implies its previous fill has landed.
          if (!mbar_wait(bar_retired(s), (uint32_t)(((c - NR) / NR) & 1), abort_flag)) {
            ok = false;
            break;
          }
        }
        if (!mbar_wait(bar_full_raw(s), ph, abort_flag)) {
          ok = false;
          break;
        }
        const uint8_t* packed = smem + (size_t)s * RAW + kTileABytes;
        const int sa = (int)(c % NA);
        const uint32_t t_slot = tmem_base + ((uint32_t)(quarter * 32) << 16) + kTmemABase + (uint32_t)sa * 64;
        uint32_t h[2][16];
        convert(packed, emax, h);
        // the slot was last read by k-step c - NA
        if (c >= NA && !mbar_wait(bar_retired((int)((c - NA) % NR)), (uint32_t)(((c - NA) / NR) & 1), abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        tmem_st16(t_slot, h[0]);
        tmem_st16(t_slot + 16, h[1]);
        if (halves > 1) {
          // h is reused: the stores above read their registers asynchronously, so they have to be waited for
          // before the registers change (with fp16 weights the second conversion is only eight loads, and
          // without this wait rows of the first half were occasionally stored with the second half's values).
          // Converting both halves ahead of the slot wait (64 registers), or giving each thread half a row
          // of both halves (sixteen dequantiser warps), both measured slower than this.
          tmem_st_wait();
          convert(packed + HALF_B, emax, h);
          tmem_st16(t_slot + 32, h[0]);
          tmem_st16(t_slot + 48, h[1]);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full_a(sa));
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quarter = warp & 3;  // tensor-memory lanes 32*quarter .. +31 belong to this warp
    const int ew = warp - 2 - kDequantWarps;
    // three warps per lane quarter.  gate/up: both halves (gate and up of its lane's feature) x one of three
    // 64-column ranges.  Plain matrix: the two halves' columns laid end to end (2 x 192) x one of three
    // 128-column ranges, walked in steps of 32 that never straddle the halves.
    constexpr int kRange = GATED ? kTileM / 3 : 2 * kTileM / 3;
    static_assert(kTileM % 96 == 0, "three equal column ranges of whole 32-column steps");
    const int c_begin = (ew >> 2) * kRange;
    const int c_end = c_begin + kRange;
    const int trow = quarter * 32 + lane;
    long it = 0;
    bool ok = true;
    for (long item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++it) {
      const RowTile rt = A.tiles[item / L.n_tiles];
      const int nt = (int)(item % L.n_tiles);
      const int halves = L.halves(nt);
      const uint8_t* ebase = A.weights + (size_t)rt.expert * A.expert_stride;
      const float* bias = reinterpret_cast<const float*>(ebase + A.bias_offset);
      const int emax = reinterpret_cast<const int*>(ebase + A.meta_offset)[A.meta_slot];
      const float oscale = W16 ? 1.0f : ldexpf(1.0f, emax - 140);
      if (!mbar_wait(bar_tmem_full, (uint32_t)(it & 1), abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16);
      if (GATED) {
        // lane = feature; its gate accumulator is in half 0, its up accumulator in half 1
        const int feat = nt * kTileW + trow;
        const bool feat_ok = feat < L.N;
        float bu = 0.f, bg = 0.f;
        if (A.has_bias && feat_ok) {
          bu = bias[feat];
          bg = bias[A.F + feat];
        }
        __half* out = A.a_out + (size_t)rt.row0 * A.lda + feat;
        for (int c0 = c_begin; c0 < min(rt.rows, c_end); c0 += 16) {
          uint32_t rg[16], ru[16];
          tmem_ld16(t_acc + c0, rg);
          tmem_ld16(t_acc + kTileM + c0, ru);
          tmem_ld_wait();
          // two columns at a time: one packed conversion (an ALU instruction) instead of two single ones
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const float g0 = fmaf(__uint_as_float(rg[j]), oscale, bg), u0 = fmaf(__uint_as_float(ru[j]), oscale, bu);
            const float g1 = fmaf(__uint_as_float(rg[j + 1]), oscale, bg), u1 = fmaf(__uint_as_float(ru[j + 1]), oscale, bu);
            const __half2 a = __floats2half2_rn(gated_act_fast(g0, u0, A.act), gated_act_fast(g1, u1, A.act));
            if (feat_ok && c0 + j < rt.rows) out[(size_t)(c0 + j) * A.lda] = __low2half(a);
            if (feat_ok && c0 + j + 1 < rt.rows) out[(size_t)(c0 + j + 1) * A.lda] = __high2half(a);
          }
        }
      } else {
        for (int v0 = c_begin; v0 < c_end; v0 += 32) {
          const int half = v0 >= kTileM ? 1 : 0, c0 = v0 - half * kTileM;
          if (half >= halves || c0 >= rt.rows) continue;
          const int n = nt * 2 * kTileW + half * kTileW + trow;
          const bool n_ok = n < L.N;
          const float my_bias = (A.has_bias && n_ok) ? bias[2 * A.F + n] : 0.f;
          uint32_t r[32];
          tmem_ld32(t_acc + (uint32_t)v0, r);
          tmem_ld_wait();
          // lane j fetches the address of token c0 + j's output row once; every lane then reads it by shuffle
          float* my_row = nullptr;
          if (c0 + lane < rt.rows) {
            const int gr = rt.row0 + c0 + lane;
            my_row = A.out_row_ptr ? A.out_row_ptr[gr]
                                   : A.y_out + (size_t)(A.out_row_map ? A.out_row_map[gr] : gr) * A.ldy;
          }
          const unsigned long long my_bits = reinterpret_cast<unsigned long long>(my_row);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float* row = reinterpret_cast<float*>(__shfl_sync(0xffffffffu, my_bits, j));
            if (n_ok && row && c0 + j < rt.rows) row[n] = __uint_as_float(r[j]) * oscale + my_bias;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tmem_empty);
    }
    if (!GATED && A.out_row_ptr) __threadfence_system();  // rows written to other GPUs before the kernel is seen as done
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicOr(&A.meta[3], kDevErrWaitTimeout);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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
  for (int w16 = 0; w16 < 2; ++w16) {
    const void* fs[2] = {w16 ? (const void*)k_tile<true, true> : (const void*)k_tile<true, false>,
                         w16 ? (const void*)k_tile<false, true> : (const void*)k_tile<false, false>};
    for (const void* f : fs) {
      if (cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_smem_bytes(w16 != 0)) != cudaSuccess) {
        st.err = std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(cudaGetLastError());
        return CSK_ERR_CUDA;
      }
    }
  }
  st.available = true;
  return CSK_OK;
}
inline void tile_destroy(TileState&) {}

// [rows, ld] fp16 row-major, boxes of box_rows rows x 64 columns, 128-byte swizzle.
inline int tile_make_map(TileState& st, CUtensorMap* map, const __half* base, size_t rows, int ld, int box_rows = kTileM) {
  const cuuint64_t dims[2] = {(cuuint64_t)ld, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(__half)};
  const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
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
  int rc = CSK_OK;
  for (int b = 0; b < kTileBoxes && !rc; ++b) {
    rc = tile_make_map(st, &st.maps_x.m[b], x16, rows_alloc, ldx, 32 * (b + 1));
    if (!rc) rc = tile_make_map(st, &st.maps_a.m[b], a16, rows_alloc, lda, 32 * (b + 1));
  }
  if (!rc) rc = tile_make_map(st, &st.tmap_xh, x16, rows_alloc, ldx, kPairBoxRows);
  if (!rc) rc = tile_make_map(st, &st.tmap_ah, a16, rows_alloc, lda, kPairBoxRows);
  if (rc) return rc;
  st.maps_ready = true;
  return CSK_OK;
}

inline int tile_launch(TileState& st, const uint8_t* weights, size_t expert_stride, size_t off_gu, size_t off_d,
                       size_t off_bias, size_t off_meta, const TileLayout& Lgu, const TileLayout& Ld, __half* a16,
                       int lda, float* y, int ldy, const int* out_row_map, float* const* out_row_ptr,
                       const RowTile* tiles, int* meta,
                       int has_bias, int act, int F, int sm_count, cudaStream_t s, const std::function<void()>& mark,
                       bool stall = false) {
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
  a.stall = stall ? 1 : 0;
  const bool w16 = Lgu.w16 != 0;
  const size_t smem = tile_smem_bytes(w16);
  // gate/up + activation
  a.mat_offset = off_gu;
  a.L = Lgu;
  a.a_out = a16;
  a.lda = lda;
  a.meta_slot = 0;
  if (w16) k_tile<true, true><<<sm_count, kTileThreads, smem, s>>>(st.maps_x, a);
  else k_tile<true, false><<<sm_count, kTileThreads, smem, s>>>(st.maps_x, a);
  mark();
  // down
  a.mat_offset = off_d;
  a.L = Ld;
  a.y_out = y;
  a.ldy = ldy;
  a.out_row_map = out_row_map;
  a.out_row_ptr = out_row_ptr;
  a.meta_slot = 1;
  if (w16) k_tile<false, true><<<sm_count, kTileThreads, smem, s>>>(st.maps_a, a);
  else k_tile<false, false><<<sm_count, kTileThreads, smem, s>>>(st.maps_a, a);
  mark();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    st.err = std::string("launch failed: ") + cudaGetErrorString(e);
    return CSK_ERR_CUDA;
  }
  return CSK_OK;
}

}  // namespace csk
