// C ABI of the MoE layer (see include/csk_moe.h): handle, weight repack,
// host- and device-buffer entry points, expert-parallel stages.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "csk_common.cuh"
#include "csk_kernels.cuh"
#include "csk_kquant.cuh"
#include "csk_stream.cuh"
#include "csk_tile.cuh"
#include "csk_tile2.cuh"

using namespace csk;

namespace {
std::mutex g_err_mu;
std::string g_create_error;
}  // namespace

struct csk_moe_layer {
  csk_moe_config cfg{};
  int E = 0, k = 0, H = 0, F = 0, e0 = 0, Eloc = 0;
  MatLayout Lgu{}, Ld{};    // streaming kernel's layout
  TileLayout Tgu{}, Td{};   // tensor-core kernel's layout (a second copy of the codes)
  size_t off_gu = 0, off_d = 0, off_tgu = 0, off_td = 0, off_bias = 0, off_meta = 0, expert_stride = 0;
  uint8_t* d_weights = nullptr;
  uint8_t* d_resident = nullptr;  // [Eloc] flags on the device
  std::vector<uint8_t> resident;
  uint8_t* d_stage = nullptr;     // raw 17-byte blocks during load / unpack
  uint8_t* d_stage2 = nullptr;    // second staging area (bulk load)
  size_t stage_bytes = 0;
  bool w16 = false;            // fp16 weights: tensor-core kernel only, no streaming layout
  float* d_unit_router = nullptr;  // dense FFN (E = k = 1): (expert 0, weight 1) for every token

  float* d_wg = nullptr;   // [E,H]
  float* d_wg_few = nullptr;   // the same repacked for the router kernel's two chunk widths
  float* d_wg_many = nullptr;
  int* d_route_cnt = nullptr;  // [max_T] tickets of the router's token blocks (zero between launches)
  float2* d_part = nullptr;    // [part_rows,E] partial sums of the fast router, one row per (token, part of H)
  float* d_hn2 = nullptr;      // [part_rows] the parts' shares of the token rows' sums of squares
  int64_t part_rows = 0;
  float* d_wnorm = nullptr;    // [E] 2-norms of the gate rows
  int* d_fb_list = nullptr;    // [max_T] tokens the fast router could not certify
  int* d_fb = nullptr;         // [0] entries of d_fb_list, [1] ticket of its reset, [2..3] 64-bit running total
  int router_mode = CSK_ROUTER_AUTO;
  int64_t routed_tokens = 0;   // tokens routed in certified mode since creation
  float* d_logits = nullptr;  // [max_T,E] router scratch
  float* d_rbias = nullptr;
  bool router_set = false, has_rbias = false;
  // expert parallelism over peer memory
  int p2p_rank = -1, p2p_world = 0;
  size_t back_tail = 0;               // floats of d_back in front of its sync area
  int* d_p2p_epoch = nullptr;         // device: generations of the three flag barriers of a step
  RowOrigin* d_info = nullptr;        // [max_rows] origin of every received row
  float* d_back = nullptr;            // [max_T*k, H] output rows returned for this rank's pairs
  float** d_row_ptr = nullptr;        // [max_rows] where each received row's output goes
  int* d_p2p_base = nullptr;          // [E]
  __half** d_peer_x16 = nullptr;      // [world] every rank's row buffer (own entry: d_x16)
  RowOrigin** d_peer_info = nullptr;  // [world]
  float** d_peer_back = nullptr;      // [world]
  std::vector<void*> ipc_opened;      // peer mappings to close
  bool pdl = false;  // launch the layer's kernels with programmatic dependent launch (small batches)
  bool debug_stall = false;  // test hook: the next tensor-core launch's copy role issues nothing (one shot)

  float* d_norm_w = nullptr;   // [H] weight of the RMSNorm in front of the router (csk_moe_set_ffn_norm)
  float* d_normed = nullptr;   // [max_T,H] its output
  float* d_shared_out = nullptr;  // [max_T,H] the shared expert's rows of a block forward
  cudaEvent_t ev_shared_fork = nullptr, ev_shared_join = nullptr;
  float norm_eps = 1e-5f;
  int64_t max_T = 0, max_rows = 0;
  int max_tiles = 0;
  float* d_hidden = nullptr;  // [max_T,H] staging for the host entry points
  float* d_router = nullptr;  // [max_T,k,2]
  float* d_router_phys = nullptr;  // the same with logical expert ids replaced by slots (expert-parallel dispatch)
  int* d_slot_map = nullptr;       // [2][E]: primary slot, replica slot (or -1) of each logical expert
  bool has_slot_map = false;
  int E_router = 0;                // experts the router scores (= E without a slot map)
  float* d_out = nullptr;     // [max_T,H]
  __half* d_x16 = nullptr;    // [max_rows+pad, ldx]
  __half* d_a16 = nullptr;    // [max_rows+pad, lda]
  float* d_y = nullptr;       // [max_rows, H]
  int ldx = 0, lda = 0;
  int* d_counts = nullptr;       // [E]
  int* d_offsets = nullptr;      // [E+1]
  int* d_cursor = nullptr;       // [E]
  int* d_row_of_pair = nullptr;  // [max_rows]
  int* d_pair_of_row = nullptr;  // [max_rows] inverse map (small batches on the streaming kernel)
  const float* gather_hidden = nullptr;  // transient: the streaming kernel's gate/up launch gathers rows from here
  const float* gather_router = nullptr;
  int* d_out_row_map = nullptr;  // [max_rows] (expert-parallel receive side)
  int* d_seg = nullptr;          // [2*1024+2] segment plan (expert-parallel receive side)
  RowTile* d_tiles = nullptr;
  int* d_meta = nullptr;  // 16 ints: [0..7] rewritten by every permutation, [8] the router's status word
  int* h_meta = nullptr;  // pinned mirror
  int64_t* h_counts64 = nullptr;

  cudaStream_t stream = nullptr;
  // the host entry point's pipeline: copy-in and copy-out streams beside `stream`, one event pair per pass
  cudaStream_t stream_in = nullptr, stream_out = nullptr;
  static constexpr int kMaxPasses = 8;
  cudaEvent_t ev_in[kMaxPasses]{}, ev_done[kMaxPasses]{}, ev_free = nullptr;
  int* d_carry = nullptr;      // [1 + E]: sticky status and per-expert row totals over the passes of one call
  bool carry_active = false;   // the combine kernel folds each pass into d_carry
  bool counts_in_carry = false;  // the last call's counters are the totals in d_carry
  cudaEvent_t ev[8]{};
  bool timing = false;
  csk_moe_timings last{};
  int path = CSK_PATH_AUTO;
  int sm_count = 148;
  TileState tile;  // tensor maps and launch state of the tensor-core path
  PairState pair;  // the CTA-pair kernel, where clusters of two can be launched

  // Small batches are launch-bound: their kernel sequence is captured once per
  // (T, buffers, stream) into a CUDA graph and replayed.
  struct GraphEntry {
    int64_t T;
    const void *hidden, *router_in;
    void *router_out, *out;
    cudaStream_t stream;
    cudaGraphExec_t exec;
  };
  std::vector<GraphEntry> graphs;
  bool use_graphs = true;

  std::string err;
  int64_t last_T = 0;
  int n_marks = 0;
  bool last_routed = false;
  cudaStream_t last_stream = nullptr;
};

namespace {

int fail(csk_moe_layer* L, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (L) {
    L->err = buf;
  } else {
    std::lock_guard<std::mutex> lk(g_err_mu);
    g_create_error = buf;
  }
  return code;
}

#define CSK_CUDA(L, call)                                                                    \
  do {                                                                                       \
    cudaError_t _e = (call);                                                                 \
    if (_e != cudaSuccess)                                                                   \
      return fail(L, CSK_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e),   \
                  __FILE__, __LINE__);                                                       \
  } while (0)

int grid_for(size_t work_items, int threads, int cap) {
  size_t b = (work_items + threads - 1) / threads;
  return (int)std::max<size_t>(1, std::min<size_t>(b, (size_t)cap));
}

cudaStream_t pick(csk_moe_layer* L, void* s) { return s ? (cudaStream_t)s : L->stream; }

struct StageTimer {
  csk_moe_layer* L;
  cudaStream_t s;
  int n = 0;
  StageTimer(csk_moe_layer* l, cudaStream_t st) : L(l), s(st) {}
  void mark() {
    if (L->timing && n < 8) cudaEventRecord(L->ev[n++], s);
  }
};

// ---- the stages ----------------------------------------------------------

int launch_router(csk_moe_layer* L, const float* d_hidden, int64_t T, float* d_router,
                  cudaStream_t s) {
  if (!L->router_set) return fail(L, CSK_ERR_INVALID, "router weights were never set");
  if (reinterpret_cast<uintptr_t>(d_hidden) % 16)
    return fail(L, CSK_ERR_INVALID, "hidden states must be 16-byte aligned");
  RouterArgs a{};
  a.hidden = d_hidden;
  a.bias = L->has_rbias ? L->d_rbias : nullptr;
  a.logits = L->d_logits;
  a.router_out = d_router;
  a.counters = L->d_route_cnt;
  a.status = L->d_meta + 8;
  a.T = (int)T;
  a.H = L->H;
  a.E = L->E_router;
  a.k = L->k;
  a.sigmoid = L->cfg.sigmoid_gating;
  // The certified pass (three launches: sliced FMA logits, certification, chain over the few tokens it
  // could not separate) beats the one-launch chain only for a handful of tokens, where the chain is a
  // single 2880-step dependency on a few SMs: measured in graph replay on the 128-expert layer it is
  // 51 vs 53 us per step at T=1, level at T=4, and behind from T=16 on (361 vs 342 us at T=64).
  constexpr int64_t kCertifiedMaxTokens = 4;
  if (L->router_mode == CSK_ROUTER_CHAIN || (L->router_mode == CSK_ROUTER_AUTO && T > kCertifiedMaxTokens)) {
    launch_router_logits<true>(a, L->d_wg_few, L->d_wg_many, L->sm_count, s, L->pdl);
    CSK_CUDA(L, cudaGetLastError());
    L->last.launches += 1;
    return CSK_OK;
  }
  // fast logits with error bounds; tokens whose selection the bounds do not certify are listed ...
  const int groups = (L->E_router + 31) / 32;
  {
    FastRouterArgs f{};
    f.hidden = d_hidden;
    f.wg = L->d_wg;
    f.part = L->d_part;
    f.hn2 = L->d_hn2;
    f.T = (int)T;
    f.H = L->H;
    f.E = L->E_router;
    const int tpw = T <= 4 ? 1 : T <= 8 ? 2 : T <= 16 ? 4 : T <= 32 ? 8 : 16;
    const int token_blocks = (int)((T + 4 * tpw - 1) / (4 * tpw));
    // enough parts of the hidden dimension to put a CTA on every SM (few tokens); one part once
    // the token blocks alone fill the machine
    int parts = std::min(std::min(fast_router_slices(L->H), kFastMaxParts),
                         std::max(1, (L->sm_count + token_blocks * groups - 1) / (token_blocks * groups)));
    while (parts > 1 && T * parts > L->part_rows) --parts;
    const dim3 grid((unsigned)token_blocks, (unsigned)groups, (unsigned)parts);
    const size_t smem = fast_router_smem(tpw);
    switch (tpw) {
      case 1: launch_k(k_router_fast<1>, grid, dim3(128), smem, s, L->pdl, f); break;
      case 2: launch_k(k_router_fast<2>, grid, dim3(128), smem, s, L->pdl, f); break;
      case 4: launch_k(k_router_fast<4>, grid, dim3(128), smem, s, L->pdl, f); break;
      case 8: launch_k(k_router_fast<8>, grid, dim3(128), smem, s, L->pdl, f); break;
      default: launch_k(k_router_fast<16>, grid, dim3(128), smem, s, L->pdl, f); break;
    }
    FinishRouterArgs g{};
    g.part = L->d_part;
    g.hn2 = L->d_hn2;
    g.bias = a.bias;
    g.wnorm = L->d_wnorm;
    g.router_out = d_router;
    g.fb_list = L->d_fb_list;
    g.fb_count = L->d_fb;
    g.T = (int)T;
    g.H = L->H;
    g.E = L->E_router;
    g.k = L->k;
    g.sigmoid = L->cfg.sigmoid_gating;
    g.parts = parts;
    launch_k(k_router_finish, dim3((unsigned)T), dim3((unsigned)std::min(32 * groups, 256)), 0, s, L->pdl, g);
  }
  // ... and go through the order-faithful chain (a grid for a few percent of the tokens; its blocks
  // walk the list however long it turned out, and leave at once when it is empty)
  RouterArgs b = a;
  b.token_list = L->d_fb_list;
  b.n_list = L->d_fb;
  b.fb_done = L->d_fb + 1;
  b.fb_total = reinterpret_cast<unsigned long long*>(L->d_fb + 2);
  const int slots = (int)std::min<int64_t>(T, std::max(1, 4 * L->sm_count / groups));
  launch_router_logits<true>(b, L->d_wg_few, L->d_wg_many, L->sm_count, s, L->pdl, slots);
  CSK_CUDA(L, cudaGetLastError());
  L->last.launches += 3;
  L->routed_tokens += T;
  return CSK_OK;
}

// histogram -> scan (+ row tiles of `tile_rows`) -> scatter rows as fp16 into x16
constexpr int kOneBlockPairs = 8192;  // up to here histogram, scan and tile list are one single-block launch

// place_only: no fp16 row buffer is written; the block that scans also places every pair
// (row_of_pair, pair_of_row) and the streaming kernel gathers its token rows itself.
int launch_permute(csk_moe_layer* L, const float* d_hidden, const float* d_router, int64_t T,
                   int only_expert, int tile_rows, int e_begin, int e_count, __half* x16, int ldx,
                   int64_t max_rows, cudaStream_t s, bool place_only = false) {
  const int n_pairs = (int)(T * L->k);
  const uint8_t* res = e_count ? L->d_resident : nullptr;
  if (place_only) {
    if (n_pairs > kOneBlockPairs) return fail(L, CSK_ERR_INVALID, "internal: too many pairs for the one-block plan");
    launch_k(k_scan, dim3(1), dim3(1024), 0, s, L->pdl, L->d_counts, L->E, e_begin, e_count, tile_rows, (int)max_rows,
             L->max_tiles, res, L->d_offsets, L->d_cursor, L->d_tiles, L->d_meta, d_router, n_pairs, only_expert,
             L->d_row_of_pair, L->d_pair_of_row);
    CSK_CUDA(L, cudaGetLastError());
    L->last.launches += 1;
    return CSK_OK;
  }
  if (n_pairs <= kOneBlockPairs) {
    // small batch: histogram, scan and tile list in one single-block launch
    launch_k(k_scan, dim3(1), dim3(1024), 0, s, L->pdl, L->d_counts, L->E, e_begin, e_count, tile_rows, (int)max_rows,
             L->max_tiles, res, L->d_offsets, L->d_cursor, L->d_tiles, L->d_meta, d_router, n_pairs, only_expert,
             (int*)nullptr, (int*)nullptr);
    L->last.launches += 1;
  } else {
    CSK_CUDA(L, cudaMemsetAsync(L->d_counts, 0, sizeof(int) * L->E, s));
    CSK_CUDA(L, cudaMemsetAsync(L->d_meta, 0, sizeof(int) * 8, s));
    k_hist<<<grid_for(n_pairs, 256, 2 * L->sm_count), 256, sizeof(int) * L->E, s>>>(
        d_router, n_pairs, L->E, only_expert, L->d_counts, L->d_meta);
    k_scan<<<1, 1024, 0, s>>>(L->d_counts, L->E, e_begin, e_count, tile_rows, (int)max_rows, L->max_tiles, res,
                              L->d_offsets, L->d_cursor, L->d_tiles, L->d_meta, nullptr, 0, -1, nullptr, nullptr);
    L->last.launches += 2;
  }
  launch_k(k_scatter, dim3(grid_for(n_pairs, 8, 8 * L->sm_count)), dim3(256), 0, s, L->pdl, d_router, d_hidden,
           n_pairs, L->k, L->H, L->E, only_expert, L->d_offsets, L->d_cursor, L->d_row_of_pair, x16, ldx, (int)max_rows,
           L->cfg.weight_before_ffn);
  CSK_CUDA(L, cudaGetLastError());
  L->last.launches += 1;
  return CSK_OK;
}

// Warps per CTA and ring stages of the streaming kernel (measured on B200): ten warps with
// three-stage rings when every warp walks a whole contraction, eight warps with three stages
// when the contraction is split over the warps.
constexpr int kStreamWarps = 10, kStreamStages = 3, kStreamSplitStages = 3;
template <int NT8, int KSPLIT, int W, int NSTG>
void launch_stream_pair(csk_moe_layer* L, const __half* x16, float* y, int ldy, int x_rows, cudaStream_t s,
                        StageTimer& tm) {
  StreamArgs a{};
  a.weights = L->d_weights;
  a.expert_stride = L->expert_stride;
  a.bias_offset = L->off_bias;
  a.tiles = L->d_tiles;
  a.n_tiles_ptr = L->d_meta;
  a.has_bias = L->cfg.has_bias;
  a.act = L->cfg.activation;
  a.F = L->F;
  a.meta = L->d_meta;
  a.x_rows = x_rows;
  a.gather_hidden = L->gather_hidden;  // set by the caller for this launch only (null: rows come from x16)
  a.pair_of_row = L->d_pair_of_row;
  a.router = L->gather_router;
  a.top_k = L->k;
  a.H = L->H;
  a.weight_before_ffn = L->cfg.weight_before_ffn;
  // every CTA takes one contiguous range of work units; as many CTAs as fit at once
  const size_t per_sm_limit = W > 8 ? 2 : 3;
  auto grid_for_smem = [&](size_t smem) {
    return L->sm_count * (int)std::max<size_t>(1, std::min<size_t>(per_sm_limit, (227 * 1024) / (smem + 1024)));
  };
  // gate/up + activation
  a.mat_offset = L->off_gu;
  a.L = L->Lgu;
  a.x = x16;
  a.ldx = L->ldx;
  a.a_out = L->d_a16;
  a.lda = L->lda;
  size_t smem = stream_smem_bytes(x_rows, NT8, L->Lgu.k_pad(), KSPLIT, true, W, NSTG);
  launch_k(k_stream<NT8, true, KSPLIT, W, NSTG>, dim3(grid_for_smem(smem)), dim3(W * 32), smem, s, L->pdl, a);
  tm.mark();
  // down
  a.gather_hidden = nullptr;
  a.mat_offset = L->off_d;
  a.L = L->Ld;
  a.x = L->d_a16;
  a.ldx = L->lda;
  a.y_out = y;
  a.ldy = ldy;
  smem = stream_smem_bytes(x_rows, NT8, L->Ld.k_pad(), KSPLIT, false, W, NSTG);
  launch_k(k_stream<NT8, false, KSPLIT, W, NSTG>, dim3(grid_for_smem(smem)), dim3(W * 32), smem, s, L->pdl, a);
  tm.mark();
  L->last.launches += 2;
}

template <int NT8, int KSPLIT, int W, int NSTG>
cudaError_t stream_prepare_one() {
  cudaError_t e = cudaFuncSetAttribute(k_stream<NT8, true, KSPLIT, W, NSTG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(k_stream<NT8, false, KSPLIT, W, NSTG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  return e;
}
cudaError_t stream_prepare_device() {
  cudaError_t e = stream_prepare_one<1, 1, kStreamWarps, kStreamStages>();
  if (e == cudaSuccess) e = stream_prepare_one<1, 8, 8, kStreamSplitStages>();
  if (e == cudaSuccess) e = stream_prepare_one<2, 1, 8, 3>();
  return e;
}

int stream_tile_rows(const csk_moe_layer* L, int64_t rows) {
  // 8-row tiles up to an average of twelve rows per expert: the 16-row variant of the streaming kernel is
  // 1.8x slower per weight byte (558 vs 314 us per step at 64 tokens on the 128-expert layer), so it pays
  // only when nearly every expert would otherwise stream its weights twice.  (Under CSK_PATH_AUTO the
  // tensor-core kernel has taken over before that point.)
  return rows <= 12 * (int64_t)std::max(1, L->Eloc) ? 8 : 16;
}

int choose_path(const csk_moe_layer* L, int64_t rows) {
  if (L->w16) return CSK_PATH_TILE;  // fp16 weights exist in the tensor-core layout only
  if (L->path == CSK_PATH_STREAM) return CSK_PATH_STREAM;
  if (L->path == CSK_PATH_TILE || L->path == CSK_PATH_TILE_PAIR) return CSK_PATH_TILE;
  // The tensor-core kernel's time is nearly flat in the rows per expert (600 us per step at 256 tokens,
  // 700 at 1024 on the 128-expert layer), the streaming kernel's grows with the number of 8-row tiles
  // (494 us at 256 tokens, 816 at 512): they cross at about ten rows per expert.
  return (L->tile.available && rows >= 10 * (int64_t)std::max(1, L->Eloc)) ? CSK_PATH_TILE : CSK_PATH_STREAM;
}

// the CTA-pair kernel runs only when asked for by name (and clusters of two can be launched)
bool use_pairs(const csk_moe_layer* L) { return L->pair.available && L->path == CSK_PATH_TILE_PAIR; }

int tile_rows_for(const csk_moe_layer* L, int path, int64_t rows) {
  return path == CSK_PATH_TILE ? (use_pairs(L) ? kPairN : kTileM) : stream_tile_rows(L, rows);
}

// grouped gate/up + activation + down over the row tiles listed in d_tiles;
// x16 holds the grouped rows; output rows go to y (through out_row_map if set)
int launch_experts(csk_moe_layer* L, int path, int tile_rows, int64_t n_rows_hint, int64_t rows_per_expert_max,
                   const __half* x16, float* y, int ldy, const int* out_row_map, cudaStream_t s, StageTimer& tm,
                   float* const* out_row_ptr = nullptr) {
  if (path == CSK_PATH_TILE) {
    if (x16 != L->d_x16) return fail(L, CSK_ERR_INVALID, "the tile path reads the handle's own row buffer");
    int rc;
    if (use_pairs(L))
      rc = pair_launch(L->pair, L->tile, L->tile.tmap_xh, L->tile.tmap_ah, L->d_weights, L->expert_stride, L->off_tgu,
                       L->off_td, L->off_bias, L->off_meta, L->Tgu, L->Td, L->d_a16, L->lda, y, ldy, out_row_map,
                       out_row_ptr, L->d_tiles, L->d_meta, L->cfg.has_bias, L->cfg.activation, L->F, s,
                       [&]() { tm.mark(); }, L->debug_stall);
    else
      rc = tile_launch(L->tile, L->d_weights, L->expert_stride, L->off_tgu, L->off_td, L->off_bias,
                       L->off_meta, L->Tgu, L->Td, L->d_a16, L->lda, y, ldy, out_row_map, out_row_ptr, L->d_tiles,
                       L->d_meta, L->cfg.has_bias, L->cfg.activation, L->F, L->sm_count, s,
                       [&]() { tm.mark(); }, L->debug_stall);
    L->debug_stall = false;
    if (rc) return fail(L, rc, "tensor-core path: %s", L->tile.err.c_str());
    L->last.launches += 2;
  } else {
    if (out_row_map || out_row_ptr) return fail(L, CSK_ERR_INVALID, "row maps need the tile path");
    // no tile holds more rows than its expert received
    const int x_rows = (int)std::max<int64_t>(1, std::min<int64_t>(tile_rows, rows_per_expert_max));
    const int kp = std::max(L->Lgu.k_pad(), L->Ld.k_pad());
    const size_t need = tile_rows == 8 ? std::max(stream_smem_bytes(x_rows, 1, kp, 8, true, 8, kStreamSplitStages),
                                                  stream_smem_bytes(x_rows, 1, kp, 1, true, kStreamWarps, kStreamStages))
                                       : stream_smem_bytes(x_rows, 2, kp, 1, true, 8, 3);
    if (need > 200 * 1024)
      return fail(L, CSK_ERR_NOMEM, "hidden/ffn dimension too large for the streaming kernel's row buffer");
    if (tile_rows == 8) {
      constexpr int64_t kSplitRows = 8;
      if (n_rows_hint <= kSplitRows) {  // measured: the split pays only while the whole batch is a handful of rows
        launch_stream_pair<1, 8, 8, kStreamSplitStages>(L, x16, y, ldy, x_rows, s, tm);  // a handful of rows: split the contraction over the warps
      } else {
        launch_stream_pair<1, 1, kStreamWarps, kStreamStages>(L, x16, y, ldy, x_rows, s, tm);
      }
    } else {
      launch_stream_pair<2, 1, 8, 3>(L, x16, y, ldy, x_rows, s, tm);
    }
  }
  CSK_CUDA(L, cudaGetLastError());
  L->last.path = path;
  return CSK_OK;
}

int report_status(csk_moe_layer* L, int st, cudaStream_t s);

int check_device_status(csk_moe_layer* L, cudaStream_t s) {
  CSK_CUDA(L, cudaMemcpyAsync(L->h_meta, L->d_meta, sizeof(int) * 16, cudaMemcpyDeviceToHost, s));
  CSK_CUDA(L, cudaStreamSynchronize(s));
  return report_status(L, L->h_meta[3] | L->h_meta[8], s);
}

// The host's view of a status word (h_meta holds the copy it came from).
int report_status(csk_moe_layer* L, int st, cudaStream_t s) {
  if (L->h_meta[8]) cudaMemsetAsync(L->d_meta + 8, 0, sizeof(int), s);
  if (st & kDevErrExpertRange)
    return fail(L, CSK_ERR_INVALID, "expert_idx out of range in router output");
  if (st & kDevErrCapacity)
    return fail(L, CSK_ERR_NOMEM, "more rows than max_tokens allows (%d rows)", L->h_meta[1]);
  if (st & kDevErrNotResident)
    return fail(L, CSK_ERR_MISSING, "tokens were routed to an expert whose weights are not loaded");
  if (st & kDevErrPeerRow)
    return fail(L, CSK_ERR_DEVICE, "a row received from a peer carries no valid origin (rank, pair)");
  if (st & kDevErrWaitTimeout)
    return fail(L, CSK_ERR_DEVICE, "a bounded device-side wait ran out");
  return CSK_OK;
}

void finish_timings(csk_moe_layer* L, int n_marks, bool routed) {
  if (!L->timing) return;
  float ms[8] = {0};
  for (int i = 0; i + 1 < n_marks; ++i) cudaEventElapsedTime(&ms[i], L->ev[i], L->ev[i + 1]);
  int i = 0;
  L->last.route_ms = routed ? ms[i++] : 0.f;
  L->last.permute_ms = ms[i++];
  L->last.gate_up_ms = ms[i++];
  L->last.down_ms = ms[i++];
  L->last.combine_ms = ms[i++];
  cudaEventElapsedTime(&L->last.total_ms, L->ev[0], L->ev[n_marks - 1]);
}

// The whole layer on device buffers.  only_expert >= 0 gives the dense output
// of that single expert node.
int forward_dev(csk_moe_layer* L, const float* d_hidden, int64_t T, const float* d_router_in,
                float* d_router_out, float* d_out, int only_expert, cudaStream_t s, bool sync_check,
                const float* d_residual = nullptr, const float* d_shared = nullptr, cudaEvent_t shared_ready = nullptr) {
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens=%lld]",
                                          (long long)T, (long long)L->max_T);
  if (L->has_slot_map)
    return fail(L, CSK_ERR_INVALID, "the layer has an expert-parallel slot map: use the csk_moe_ep_* stages");
  L->last = csk_moe_timings{};
  L->last_T = T;
  if (!L->carry_active) L->counts_in_carry = false;
  // small batches are launch-bound: let each kernel become resident while its predecessor drains
  struct PdlScope {
    csk_moe_layer* l;
    ~PdlScope() { l->pdl = false; }
  } pdl_scope{L};
  L->pdl = T <= 512 && !L->timing;
  StageTimer tm(L, s);
  tm.mark();
  const float* router = d_router_in;
  const bool routed = d_router_in == nullptr;
  if (routed) {
    // the routing is written where the caller wants it (else into the handle's buffer) and read from there
    float* route_to = d_router_out ? d_router_out : L->d_router;
    int rc = launch_router(L, d_hidden, T, route_to, s);
    if (rc) return rc;
    router = route_to;
    tm.mark();
  } else if (d_router_out && d_router_out != router) {
    CSK_CUDA(L, cudaMemcpyAsync(d_router_out, router, sizeof(float) * T * L->k * 2,
                                cudaMemcpyDeviceToDevice, s));
  }
  const int64_t rows = only_expert >= 0 ? T : T * L->k;
  const int path = choose_path(L, only_expert >= 0 ? rows * std::max(1, L->Eloc) : rows);
  const int tile_rows = tile_rows_for(L, path, only_expert >= 0 ? rows * std::max(1, L->Eloc) : rows);
  if (reinterpret_cast<uintptr_t>(d_hidden) % 16) return fail(L, CSK_ERR_INVALID, "hidden states must be 16-byte aligned");
  // small batches on the streaming kernel: no fp16 row buffer in between, the kernel gathers its rows
  // (up to 64 pairs: measured, the launch it saves is worth 2-3 us of a 50-190 us step there; with more rows per
  // tile every work unit's copy of the gather costs more than the launch -- 7 % of the step at 32 tokens on 32 experts)
  constexpr int64_t kGatherMaxPairs = 64;
  const bool gather = path == CSK_PATH_STREAM && T * L->k <= kGatherMaxPairs;
  int rc = launch_permute(L, d_hidden, router, T, only_expert, tile_rows, L->e0, L->Eloc, L->d_x16,
                          L->ldx, L->max_rows, s, gather);
  if (rc) return rc;
  tm.mark();
  L->gather_hidden = gather ? d_hidden : nullptr;
  L->gather_router = router;
  rc = launch_experts(L, path, tile_rows, rows, T, L->d_x16, L->d_y, L->H, nullptr, s, tm);
  L->gather_hidden = nullptr;
  if (rc) return rc;
  // the shared expert's rows come from another stream: the combine is the first kernel that reads them
  if (shared_ready) CSK_CUDA(L, cudaStreamWaitEvent(s, shared_ready, 0));
  launch_k(k_combine, dim3((unsigned)T), dim3(256), 0, s, L->pdl && !shared_ready, router, L->d_row_of_pair,
           (const float*)L->d_y, L->H, d_out, (int)T, L->k, L->H, (int)L->cfg.weight_before_ffn, (int)(only_expert >= 0),
           (const int*)L->d_meta, (const int*)L->d_counts, L->carry_active ? L->d_carry : (int*)nullptr, L->E, d_residual,
           d_shared);
  CSK_CUDA(L, cudaGetLastError());
  L->last.launches++;
  tm.mark();
  L->n_marks = tm.n;
  L->last_routed = routed;
  L->last_stream = s;
  if (!sync_check) return CSK_OK;
  rc = check_device_status(L, s);
  if (rc) return rc;
  finish_timings(L, tm.n, routed);
  return CSK_OK;
}

int check_layer(csk_moe_layer* L) { return L ? CSK_OK : CSK_ERR_INVALID; }

// Captured launch sequences embed kernel arguments (which router bias, which path, which
// slot map): whatever changes one of those drops them.
void drop_graphs(csk_moe_layer* L) {
  for (auto& g : L->graphs)
    if (g.exec) cudaGraphExecDestroy(g.exec);
  L->graphs.clear();
}

}  // namespace

// ===========================================================================
extern "C" {

int csk_moe_device_ok(int device) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) {
    cudaGetLastError();
    return 0;
  }
  cudaDeviceProp p{};
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) return 0;
  return p.major == 10 ? 1 : 0;
}

const char* csk_moe_last_error(const csk_moe_layer* layer) {
  if (layer) return layer->err.c_str();
  std::lock_guard<std::mutex> lk(g_err_mu);
  return g_create_error.c_str();
}

int csk_moe_create(const csk_moe_config* cfg, csk_moe_layer** out) {
  if (!cfg || !out) return fail(nullptr, CSK_ERR_INVALID, "null argument");
  *out = nullptr;
  if (cfg->num_experts <= 0 || cfg->num_experts > 1024)
    return fail(nullptr, CSK_ERR_INVALID, "num_experts must be in [1,1024], got %d", cfg->num_experts);
  if (cfg->top_k <= 0 || cfg->top_k > kMaxTopK || cfg->top_k > cfg->num_experts)
    return fail(nullptr, CSK_ERR_INVALID, "top_k must be in [1,%d] and <= num_experts, got %d",
                kMaxTopK, cfg->top_k);
  if (cfg->hidden <= 0 || cfg->hidden % 32)
    return fail(nullptr, CSK_ERR_INVALID,
                "expert_mlp: hidden_dim must be a multiple of 32 for MXFP4, got %d", cfg->hidden);
  if (cfg->ffn <= 0 || cfg->ffn % 32)
    return fail(nullptr, CSK_ERR_INVALID,
                "expert_mlp: expert_ffn_dim must be a multiple of 32 for MXFP4, got %d", cfg->ffn);
  if (cfg->weight_format != CSK_WEIGHTS_MXFP4 && cfg->weight_format != CSK_WEIGHTS_F16)
    return fail(nullptr, CSK_ERR_INVALID, "unknown weight format %d", cfg->weight_format);
  if (cfg->activation != CSK_ACT_MODIFIED_SWIGLU && cfg->activation != CSK_ACT_STANDARD_SWIGLU)
    return fail(nullptr, CSK_ERR_INVALID, "unknown activation %d", cfg->activation);
  if (cfg->max_tokens <= 0 || cfg->max_tokens * cfg->top_k > (1 << 28))
    return fail(nullptr, CSK_ERR_INVALID, "max_tokens out of range");
  const int eloc = cfg->expert_count ? cfg->expert_count : cfg->num_experts;
  const int e0 = cfg->expert_count ? cfg->expert_begin : 0;
  if (e0 < 0 || eloc <= 0 || e0 + eloc > cfg->num_experts)
    return fail(nullptr, CSK_ERR_INVALID, "expert range [%d,%d) outside [0,%d)", e0, e0 + eloc,
                cfg->num_experts);
  if (!csk_moe_device_ok(cfg->device))
    return fail(nullptr, CSK_ERR_CUDA, "device %d is not a usable sm_100 GPU (no CPU fallback exists)",
                cfg->device);

  csk_moe_layer* L = new (std::nothrow) csk_moe_layer();
  if (!L) return fail(nullptr, CSK_ERR_NOMEM, "out of host memory");
  L->cfg = *cfg;
  L->E = cfg->num_experts;
  L->k = cfg->top_k;
  L->H = cfg->hidden;
  L->F = cfg->ffn;
  L->e0 = e0;
  L->Eloc = eloc;
  L->w16 = cfg->weight_format == CSK_WEIGHTS_F16;
  L->Lgu = make_layout(L->F, L->H, true);
  L->Ld = make_layout(L->H, L->F, false);
  L->Tgu = make_tile_layout(L->F, L->H, true, L->w16);
  L->Td = make_tile_layout(L->H, L->F, false, L->w16);
  auto up256 = [](size_t v) { return (v + 255) / 256 * 256; };
  L->off_gu = 0;
  L->off_d = L->w16 ? 0 : up256(L->Lgu.bytes());                  // fp16 weights have no streaming layout
  L->off_tgu = L->w16 ? 0 : L->off_d + up256(L->Ld.bytes());
  L->off_td = L->off_tgu + up256(L->Tgu.bytes());
  L->off_bias = L->off_td + up256(L->Td.bytes());
  L->off_meta = L->off_bias + sizeof(float) * (2 * (size_t)L->F + L->H);  // int[4]: e_max of gate/up, of down
  L->expert_stride = (L->off_meta + 16 + 255) / 256 * 256;
  L->resident.assign(eloc, 0);
  L->max_T = cfg->max_tokens;
  L->max_rows = cfg->max_tokens * cfg->top_k;
  L->ldx = L->Lgu.k_pad();
  L->lda = L->Ld.k_pad();
  L->max_tiles = (int)(L->max_rows / 8 + eloc + 8);

#define CK(call)                                                                              \
  do {                                                                                        \
    cudaError_t _e = (call);                                                                  \
    if (_e != cudaSuccess) {                                                                  \
      int rc = fail(nullptr, _e == cudaErrorMemoryAllocation ? CSK_ERR_NOMEM : CSK_ERR_CUDA,  \
                    "%s failed: %s", #call, cudaGetErrorString(_e));                          \
      csk_moe_destroy(L);                                                                     \
      return rc;                                                                              \
    }                                                                                         \
  } while (0)

  CK(cudaSetDevice(cfg->device));
  cudaDeviceProp prop{};
  CK(cudaGetDeviceProperties(&prop, cfg->device));
  L->sm_count = prop.multiProcessorCount;
  CK(cudaStreamCreateWithFlags(&L->stream, cudaStreamNonBlocking));
  CK(cudaStreamCreateWithFlags(&L->stream_in, cudaStreamNonBlocking));
  CK(cudaStreamCreateWithFlags(&L->stream_out, cudaStreamNonBlocking));
  for (auto& e : L->ev) CK(cudaEventCreate(&e));
  for (auto& e : L->ev_in) CK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  for (auto& e : L->ev_done) CK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  CK(cudaEventCreateWithFlags(&L->ev_free, cudaEventDisableTiming));
  CK(cudaMalloc(&L->d_carry, sizeof(int) * (1 + L->E)));
  CK(cudaMemset(L->d_carry, 0, sizeof(int) * (1 + L->E)));
  CK(cudaMalloc(&L->d_weights, L->expert_stride * eloc));
  CK(cudaMemset(L->d_weights, 0, L->expert_stride * eloc));
  CK(cudaMalloc(&L->d_resident, eloc));
  CK(cudaMemset(L->d_resident, 0, eloc));
  L->stage_bytes = L->w16 ? (size_t)L->H * L->F * 2 : (size_t)L->H * L->F / 32 * 17;
  CK(cudaMalloc(&L->d_stage, 3 * L->stage_bytes));
  CK(cudaMalloc(&L->d_wg, sizeof(float) * L->E * L->H));
  CK(cudaMalloc(&L->d_wg_few, sizeof(float) * router_packed_floats(L->E, L->H, kRouterChunkFew)));
  CK(cudaMalloc(&L->d_wg_many, sizeof(float) * router_packed_floats(L->E, L->H, kRouterChunkMany)));
  CK(cudaMalloc(&L->d_route_cnt, sizeof(int) * L->max_T));
  CK(cudaMemset(L->d_route_cnt, 0, sizeof(int) * L->max_T));
  CK(cudaMalloc(&L->d_logits, sizeof(float) * L->max_T * L->E));
  CK(cudaMalloc(&L->d_wnorm, sizeof(float) * L->E));
  L->part_rows = L->max_T + 64 * (int64_t)(L->sm_count + fast_router_slices(L->H));
  CK(cudaMalloc(&L->d_part, sizeof(float2) * L->part_rows * L->E));
  CK(cudaMalloc(&L->d_hn2, sizeof(float) * L->part_rows));
  CK(cudaMalloc(&L->d_fb_list, sizeof(int) * L->max_T));
  CK(cudaMalloc(&L->d_fb, sizeof(int) * 4));
  CK(cudaMemset(L->d_fb, 0, sizeof(int) * 4));
  CK(cudaMalloc(&L->d_rbias, sizeof(float) * L->E));
  CK(cudaMalloc(&L->d_hidden, sizeof(float) * L->max_T * L->H));
  CK(cudaMalloc(&L->d_router, sizeof(float) * L->max_T * L->k * 2));
  CK(cudaMalloc(&L->d_router_phys, sizeof(float) * L->max_T * L->k * 2));
  CK(cudaMalloc(&L->d_p2p_epoch, sizeof(int) * 4));
  CK(cudaMemset(L->d_p2p_epoch, 0, sizeof(int) * 4));
  if (L->E == 1 && L->k == 1) {  // a dense FFN: every token goes to expert 0 with weight 1
    std::vector<float> unit(2 * (size_t)L->max_T);
    for (int64_t t = 0; t < L->max_T; ++t) {
      unit[2 * t] = 0.0f;
      unit[2 * t + 1] = 1.0f;
    }
    CK(cudaMalloc(&L->d_unit_router, sizeof(float) * unit.size()));
    CK(cudaMemcpy(L->d_unit_router, unit.data(), sizeof(float) * unit.size(), cudaMemcpyHostToDevice));
  }
  CK(cudaMalloc(&L->d_slot_map, sizeof(int) * 2 * L->E));
  CK(cudaMalloc(&L->d_p2p_base, sizeof(int) * L->E));
  L->E_router = L->E;
  CK(cudaMalloc(&L->d_out, sizeof(float) * L->max_T * L->H));
  const size_t pad_rows = std::max(kTileM, kPairN);  // a row tile's loads may reach this far past the last row
  CK(cudaMalloc(&L->d_x16, sizeof(__half) * (L->max_rows + pad_rows) * L->ldx));
  CK(cudaMemset(L->d_x16, 0, sizeof(__half) * (L->max_rows + pad_rows) * L->ldx));
  CK(cudaMalloc(&L->d_a16, sizeof(__half) * (L->max_rows + pad_rows) * L->lda));
  CK(cudaMemset(L->d_a16, 0, sizeof(__half) * (L->max_rows + pad_rows) * L->lda));
  CK(cudaMalloc(&L->d_y, sizeof(float) * L->max_rows * L->H));
  CK(cudaMalloc(&L->d_counts, sizeof(int) * L->E));
  CK(cudaMalloc(&L->d_offsets, sizeof(int) * (L->E + 1)));
  CK(cudaMalloc(&L->d_cursor, sizeof(int) * L->E));
  CK(cudaMalloc(&L->d_row_of_pair, sizeof(int) * L->max_rows));
  CK(cudaMalloc(&L->d_pair_of_row, sizeof(int) * L->max_rows));
  CK(cudaMemset(L->d_pair_of_row, 0, sizeof(int) * L->max_rows));
  CK(cudaMalloc(&L->d_out_row_map, sizeof(int) * L->max_rows));
  CK(cudaMalloc(&L->d_seg, sizeof(int) * (3 * 1024 + 8)));
  CK(cudaMalloc(&L->d_tiles, sizeof(RowTile) * L->max_tiles));
  CK(cudaMalloc(&L->d_meta, sizeof(int) * 16));
  CK(cudaMemset(L->d_meta, 0, sizeof(int) * 16));
  CK(cudaMallocHost(&L->h_meta, sizeof(int) * 16));
  CK(cudaMallocHost(&L->h_counts64, sizeof(int64_t) * L->E));
  CK(router_prepare_device());
  CK(stream_prepare_device());
  {
    int rc = tile_init(L->tile, cfg->device);
    if (!rc) rc = tile_set_buffers(L->tile, L->d_x16, L->ldx, L->d_a16, L->lda, (size_t)L->max_rows + pad_rows);
    if (!rc) rc = pair_init(L->pair, L->tile, L->sm_count);
    if (rc) {
      rc = fail(nullptr, rc, "tensor-core path setup: %s", L->tile.err.c_str());
      csk_moe_destroy(L);
      return rc;
    }
  }
  CK(cudaDeviceSynchronize());
#undef CK
  *out = L;
  return CSK_OK;
}

int csk_moe_destroy(csk_moe_layer* L) {
  if (!L) return CSK_OK;
  cudaSetDevice(L->cfg.device);
  if (L->stream) cudaStreamSynchronize(L->stream);
  for (auto& g : L->graphs)
    if (g.exec) cudaGraphExecDestroy(g.exec);
  tile_destroy(L->tile);
  for (void* p : L->ipc_opened) cudaIpcCloseMemHandle(p);
  void* dev[] = {L->d_shared_out, L->d_p2p_epoch, L->d_unit_router, L->d_stage2, L->d_norm_w, L->d_normed, L->d_part, L->d_hn2, L->d_wnorm, L->d_fb_list, L->d_fb, L->d_info, L->d_back, L->d_row_ptr, L->d_p2p_base, L->d_peer_x16, L->d_peer_info, L->d_peer_back,
                 L->d_router_phys, L->d_slot_map, L->d_weights, L->d_resident, L->d_stage, L->d_wg, L->d_wg_few, L->d_wg_many, L->d_route_cnt, L->d_logits, L->d_rbias, L->d_hidden,
                 L->d_router, L->d_out, L->d_x16, L->d_a16, L->d_y, L->d_counts, L->d_offsets,
                 L->d_cursor, L->d_row_of_pair, L->d_pair_of_row, L->d_out_row_map, L->d_seg, L->d_tiles, L->d_meta};
  for (void* p : dev)
    if (p) cudaFree(p);
  if (L->h_meta) cudaFreeHost(L->h_meta);
  if (L->h_counts64) cudaFreeHost(L->h_counts64);
  for (auto& e : L->ev)
    if (e) cudaEventDestroy(e);
  for (auto& e : L->ev_in)
    if (e) cudaEventDestroy(e);
  for (auto& e : L->ev_done)
    if (e) cudaEventDestroy(e);
  if (L->ev_free) cudaEventDestroy(L->ev_free);
  if (L->ev_shared_fork) cudaEventDestroy(L->ev_shared_fork);
  if (L->ev_shared_join) cudaEventDestroy(L->ev_shared_join);
  if (L->d_carry) cudaFree(L->d_carry);
  if (L->stream_in) cudaStreamDestroy(L->stream_in);
  if (L->stream_out) cudaStreamDestroy(L->stream_out);
  if (L->stream) cudaStreamDestroy(L->stream);
  delete L;
  return CSK_OK;
}

int csk_moe_set_router(csk_moe_layer* L, const float* gate_w, const float* gate_bias) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!gate_w) return fail(L, CSK_ERR_INVALID, "gate_weights is null");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  CSK_CUDA(L, cudaMemcpyAsync(L->d_wg, gate_w, sizeof(float) * L->E_router * L->H, cudaMemcpyHostToDevice,
                              L->stream));
  k_pack_router<<<grid_for(router_packed_floats(L->E_router, L->H, kRouterChunkFew), 256, 1024), 256, 0, L->stream>>>(
      L->d_wg, L->d_wg_few, L->E_router, L->H, kRouterChunkFew);
  k_pack_router<<<grid_for(router_packed_floats(L->E_router, L->H, kRouterChunkMany), 256, 1024), 256, 0, L->stream>>>(
      L->d_wg, L->d_wg_many, L->E_router, L->H, kRouterChunkMany);
  k_router_wnorm<<<(L->E_router + 7) / 8, 256, 0, L->stream>>>(L->d_wg, L->d_wnorm, L->E_router, L->H);
  CSK_CUDA(L, cudaGetLastError());
  L->has_rbias = gate_bias != nullptr;
  if (gate_bias)
    CSK_CUDA(L, cudaMemcpyAsync(L->d_rbias, gate_bias, sizeof(float) * L->E_router, cudaMemcpyHostToDevice,
                                L->stream));
  CSK_CUDA(L, cudaStreamSynchronize(L->stream));
  L->router_set = true;
  drop_graphs(L);
  return CSK_OK;
}

namespace {
// One expert: raw blocks to a staging area, the four repacks, biases.  Enqueue only; `stage` is one
// of the handle's two staging areas (3 * stage_bytes each).  With null weight pointers the staging
// area already holds the three matrices (decoded there by the caller).
int load_expert_enqueue(csk_moe_layer* L, int le, const uint8_t* w_up, const uint8_t* w_gate, const uint8_t* w_down,
                        const float* b_up, const float* b_gate, const float* b_down, uint8_t* stage, cudaStream_t s) {
  uint8_t* base = L->d_weights + (size_t)le * L->expert_stride;
  uint8_t *s_up = stage, *s_gate = stage + L->stage_bytes, *s_down = stage + 2 * L->stage_bytes;
  if (w_up) {
    CSK_CUDA(L, cudaMemcpyAsync(s_up, w_up, L->stage_bytes, cudaMemcpyHostToDevice, s));
    CSK_CUDA(L, cudaMemcpyAsync(s_gate, w_gate, L->stage_bytes, cudaMemcpyHostToDevice, s));
    CSK_CUDA(L, cudaMemcpyAsync(s_down, w_down, L->stage_bytes, cudaMemcpyHostToDevice, s));
  }
  int* emeta = reinterpret_cast<int*>(base + L->off_meta);
  CSK_CUDA(L, cudaMemsetAsync(emeta, 0, 16, s));
  if (L->w16) {
    const __half *h_up = reinterpret_cast<const __half*>(s_up), *h_gate = reinterpret_cast<const __half*>(s_gate),
                 *h_down = reinterpret_cast<const __half*>(s_down);
    k_repack_tile_f16<<<grid_for(L->Tgu.bytes() / 16, 256, 4096), 256, 0, s>>>(h_gate, h_up, base + L->off_tgu, L->Tgu);
    k_repack_tile_f16<<<grid_for(L->Td.bytes() / 16, 256, 4096), 256, 0, s>>>(h_down, nullptr, base + L->off_td, L->Td);
  } else {
  k_repack<<<grid_for(L->Lgu.bytes() / 4, 256, 4096), 256, 0, s>>>(s_gate, s_up, base + L->off_gu, L->Lgu, emeta);
  k_repack<<<grid_for(L->Ld.bytes() / 4, 256, 4096), 256, 0, s>>>(s_down, nullptr, base + L->off_d, L->Ld, emeta + 1);
  k_repack_tile<<<grid_for(L->Tgu.bytes() / 4, 256, 4096), 256, 0, s>>>(s_gate, s_up, base + L->off_tgu, L->Tgu);
  k_repack_tile<<<grid_for(L->Td.bytes() / 4, 256, 4096), 256, 0, s>>>(s_down, nullptr, base + L->off_td, L->Td);
  }
  CSK_CUDA(L, cudaGetLastError());
  if (L->cfg.has_bias) {
    float* b = reinterpret_cast<float*>(base + L->off_bias);
    CSK_CUDA(L, cudaMemcpyAsync(b, b_up, sizeof(float) * L->F, cudaMemcpyHostToDevice, s));
    CSK_CUDA(L, cudaMemcpyAsync(b + L->F, b_gate, sizeof(float) * L->F, cudaMemcpyHostToDevice, s));
    CSK_CUDA(L, cudaMemcpyAsync(b + 2 * L->F, b_down, sizeof(float) * L->H, cudaMemcpyHostToDevice, s));
  }
  CSK_CUDA(L, cudaMemsetAsync(L->d_resident + le, 1, 1, s));
  return CSK_OK;
}
}  // namespace

int csk_moe_load_expert_mxfp4(csk_moe_layer* L, int32_t expert_id, const uint8_t* w_up,
                              const uint8_t* w_gate, const uint8_t* w_down, const float* b_up,
                              const float* b_gate, const float* b_down) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (expert_id < L->e0 || expert_id >= L->e0 + L->Eloc)
    return fail(L, CSK_ERR_INVALID, "expert %d is not resident on this device (range [%d,%d))",
                expert_id, L->e0, L->e0 + L->Eloc);
  if (!w_up || !w_gate || !w_down) return fail(L, CSK_ERR_INVALID, "null weight pointer");
  if (L->cfg.has_bias && (!b_up || !b_gate || !b_down))
    return fail(L, CSK_ERR_INVALID, "layer has biases but a bias pointer is null");
  if (L->w16) return fail(L, CSK_ERR_INVALID, "this layer holds fp16 weights: use csk_moe_load_expert_f16");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  const int le = expert_id - L->e0;
  int rc = load_expert_enqueue(L, le, w_up, w_gate, w_down, b_up, b_gate, b_down, L->d_stage, L->stream);
  if (rc) return rc;
  CSK_CUDA(L, cudaStreamSynchronize(L->stream));
  L->resident[le] = 1;
  return CSK_OK;
}

int csk_moe_load_expert_f16(csk_moe_layer* L, int32_t expert_id, const uint16_t* w_up, const uint16_t* w_gate,
                            const uint16_t* w_down, const float* b_up, const float* b_gate, const float* b_down) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!L->w16) return fail(L, CSK_ERR_INVALID, "this layer holds MXFP4 weights: use csk_moe_load_expert_mxfp4");
  if (expert_id < L->e0 || expert_id >= L->e0 + L->Eloc)
    return fail(L, CSK_ERR_INVALID, "expert %d is not resident on this device (range [%d,%d))",
                expert_id, L->e0, L->e0 + L->Eloc);
  if (!w_up || !w_gate || !w_down) return fail(L, CSK_ERR_INVALID, "null weight pointer");
  if (L->cfg.has_bias && (!b_up || !b_gate || !b_down))
    return fail(L, CSK_ERR_INVALID, "layer has biases but a bias pointer is null");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  const int le = expert_id - L->e0;
  int rc = load_expert_enqueue(L, le, reinterpret_cast<const uint8_t*>(w_up), reinterpret_cast<const uint8_t*>(w_gate),
                               reinterpret_cast<const uint8_t*>(w_down), b_up, b_gate, b_down, L->d_stage, L->stream);
  if (rc) return rc;
  CSK_CUDA(L, cudaStreamSynchronize(L->stream));
  L->resident[le] = 1;
  return CSK_OK;
}

namespace {
size_t ggml_bytes(int32_t type, int64_t n) {
  switch (type) {
    case CSK_GGML_F16: return (size_t)n * 2;
    case CSK_GGML_Q4_K: return (size_t)(n / kQkK) * kQ4kBytes;
    case CSK_GGML_Q6_K: return (size_t)(n / kQkK) * kQ6kBytes;
  }
  return 0;
}
// Raw blocks of one matrix (device) to fp16 (device).  Enqueue only.
void ggml_decode_enqueue(int32_t type, const uint8_t* d_raw, unsigned short* d_f16, int64_t n, bool nearest,
                         cudaStream_t s) {
  const int64_t nb = n / kQkK;
  if (type == CSK_GGML_Q4_K) {
    const int grid = grid_for((size_t)nb * 4 * 32, 256, 8192);
    if (nearest) k_dequant_q4k<true><<<grid, 256, 0, s>>>(d_raw, d_f16, nb);
    else k_dequant_q4k<false><<<grid, 256, 0, s>>>(d_raw, d_f16, nb);
  } else {
    const int grid = grid_for((size_t)nb * 2 * 32, 256, 8192);
    if (nearest) k_dequant_q6k<true><<<grid, 256, 0, s>>>(d_raw, d_f16, nb);
    else k_dequant_q6k<false><<<grid, 256, 0, s>>>(d_raw, d_f16, nb);
  }
}
}  // namespace

int csk_moe_load_expert_ggml(csk_moe_layer* L, int32_t expert_id, int32_t type_up, const void* w_up,
                             int32_t type_gate, const void* w_gate, int32_t type_down, const void* w_down,
                             const float* b_up, const float* b_gate, const float* b_down, int32_t f16_rounding) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!L->w16)
    return fail(L, CSK_ERR_INVALID, "this layer holds MXFP4 weights: Q4_K / Q6_K / F16 slices need a layer created "
                                    "with CSK_WEIGHTS_F16");
  if (expert_id < L->e0 || expert_id >= L->e0 + L->Eloc)
    return fail(L, CSK_ERR_INVALID, "expert %d is not resident on this device (range [%d,%d))",
                expert_id, L->e0, L->e0 + L->Eloc);
  if (!w_up || !w_gate || !w_down) return fail(L, CSK_ERR_INVALID, "null weight pointer");
  if (L->cfg.has_bias && (!b_up || !b_gate || !b_down))
    return fail(L, CSK_ERR_INVALID, "layer has biases but a bias pointer is null");
  if (f16_rounding != CSK_F16_TRUNCATE && f16_rounding != CSK_F16_NEAREST)
    return fail(L, CSK_ERR_INVALID, "f16_rounding must be CSK_F16_TRUNCATE or CSK_F16_NEAREST, got %d", f16_rounding);
  const int32_t types[3] = {type_up, type_gate, type_down};
  const void* src[3] = {w_up, w_gate, w_down};
  const int64_t n = (int64_t)L->H * L->F;  // a multiple of 1024: whole super-blocks
  for (int i = 0; i < 3; ++i)
    if (types[i] != CSK_GGML_F16 && types[i] != CSK_GGML_Q4_K && types[i] != CSK_GGML_Q6_K)
      return fail(L, CSK_ERR_INVALID, "ggml type %d is not handled (F16 = %d, Q4_K = %d, Q6_K = %d)", types[i],
                  CSK_GGML_F16, CSK_GGML_Q4_K, CSK_GGML_Q6_K);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  if (!L->d_stage2) {
    cudaError_t e = cudaMalloc(&L->d_stage2, 3 * L->stage_bytes);
    if (e != cudaSuccess) return fail(L, CSK_ERR_NOMEM, "cudaMalloc failed: %s", cudaGetErrorString(e));
  }
  cudaStream_t s = L->stream;
  for (int i = 0; i < 3; ++i) {
    uint8_t* f16 = L->d_stage + (size_t)i * L->stage_bytes;
    if (types[i] == CSK_GGML_F16) {
      CSK_CUDA(L, cudaMemcpyAsync(f16, src[i], L->stage_bytes, cudaMemcpyHostToDevice, s));
    } else {
      // the blocks are smaller than the fp16 matrix: they fit the second staging area's slot
      uint8_t* raw = L->d_stage2 + (size_t)i * L->stage_bytes;
      CSK_CUDA(L, cudaMemcpyAsync(raw, src[i], ggml_bytes(types[i], n), cudaMemcpyHostToDevice, s));
      ggml_decode_enqueue(types[i], raw, reinterpret_cast<unsigned short*>(f16), n, f16_rounding == CSK_F16_NEAREST, s);
    }
  }
  CSK_CUDA(L, cudaGetLastError());
  const int le = expert_id - L->e0;
  int rc = load_expert_enqueue(L, le, nullptr, nullptr, nullptr, b_up, b_gate, b_down, L->d_stage, s);
  if (rc) return rc;
  CSK_CUDA(L, cudaStreamSynchronize(s));
  L->resident[le] = 1;
  return CSK_OK;
}

int csk_moe_load_expert_f32(csk_moe_layer* L, int32_t expert_id, const float* w_up, const float* w_gate,
                            const float* w_down, const float* b_up, const float* b_gate, const float* b_down) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!L->w16)
    return fail(L, CSK_ERR_INVALID, "this layer holds MXFP4 weights: fp32 matrices need a layer created with CSK_WEIGHTS_F16");
  if (expert_id < L->e0 || expert_id >= L->e0 + L->Eloc)
    return fail(L, CSK_ERR_INVALID, "expert %d is not resident on this device (range [%d,%d))",
                expert_id, L->e0, L->e0 + L->Eloc);
  if (!w_up || !w_gate || !w_down) return fail(L, CSK_ERR_INVALID, "null weight pointer");
  if (L->cfg.has_bias && (!b_up || !b_gate || !b_down))
    return fail(L, CSK_ERR_INVALID, "layer has biases but a bias pointer is null");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  const int64_t n = (int64_t)L->H * L->F;
  // one fp32 matrix at a time through a temporary of its size (load time only), plus the overflow counter
  uint8_t* tmp = nullptr;
  cudaError_t e = cudaMalloc(&tmp, (size_t)n * 4 + 16);
  if (e != cudaSuccess) return fail(L, CSK_ERR_NOMEM, "cudaMalloc failed: %s", cudaGetErrorString(e));
  int* d_over = reinterpret_cast<int*>(tmp + (size_t)n * 4);
  cudaStream_t s = L->stream;
  const float* src[3] = {w_up, w_gate, w_down};
  int over = 0;
  e = cudaMemsetAsync(d_over, 0, 4, s);
  for (int i = 0; i < 3 && e == cudaSuccess; ++i) {
    e = cudaMemcpyAsync(tmp, src[i], (size_t)n * 4, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) break;
    k_f32_to_f16<<<grid_for((size_t)n, 256, 4096), 256, 0, s>>>(
        reinterpret_cast<const float*>(tmp), reinterpret_cast<unsigned short*>(L->d_stage + (size_t)i * L->stage_bytes), n, d_over);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpyAsync(&over, d_over, 4, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaFree(tmp);
  if (e != cudaSuccess) return fail(L, CSK_ERR_CUDA, "load_expert_f32: %s", cudaGetErrorString(e));
  if (over)
    return fail(L, CSK_ERR_INVALID, "load_expert_f32: a weight lies beyond the fp16 range (|w| > 65504); the tensor-core "
                                    "kernel's operands are fp16");
  const int le = expert_id - L->e0;
  int rc = load_expert_enqueue(L, le, nullptr, nullptr, nullptr, b_up, b_gate, b_down, L->d_stage, s);
  if (rc) return rc;
  CSK_CUDA(L, cudaStreamSynchronize(s));
  L->resident[le] = 1;
  return CSK_OK;
}

int csk_moe_dequant_ggml_f16(int32_t device, int32_t ggml_type, const void* blocks, int64_t n_elements, uint16_t* out_f16,
                         int32_t f16_rounding) {
  if (!blocks || !out_f16) return fail(nullptr, CSK_ERR_INVALID, "dequant_ggml: null argument");
  if (ggml_type != CSK_GGML_Q4_K && ggml_type != CSK_GGML_Q6_K)
    return fail(nullptr, CSK_ERR_INVALID, "dequant_ggml: ggml type %d is not handled (Q4_K = %d, Q6_K = %d)", ggml_type,
                CSK_GGML_Q4_K, CSK_GGML_Q6_K);
  if (n_elements <= 0 || n_elements % kQkK)
    return fail(nullptr, CSK_ERR_INVALID, "dequant_ggml: the element count must be a positive multiple of %d, got %lld",
                kQkK, (long long)n_elements);
  if (f16_rounding != CSK_F16_TRUNCATE && f16_rounding != CSK_F16_NEAREST)
    return fail(nullptr, CSK_ERR_INVALID, "dequant_ggml: f16_rounding must be CSK_F16_TRUNCATE or CSK_F16_NEAREST");
  if (!csk_moe_device_ok(device)) return fail(nullptr, CSK_ERR_CUDA, "dequant_ggml: device %d is not an sm_100 GPU; no CPU fallback exists", device);
  CSK_CUDA(nullptr, cudaSetDevice(device));
  const size_t qb = ggml_bytes(ggml_type, n_elements);
  uint8_t* d_raw = nullptr;
  unsigned short* d_out = nullptr;
  cudaError_t e = cudaMalloc(&d_raw, qb);
  if (e == cudaSuccess) e = cudaMalloc(&d_out, (size_t)n_elements * 2);
  if (e != cudaSuccess) {
    cudaFree(d_raw);
    return fail(nullptr, CSK_ERR_NOMEM, "dequant_ggml: cudaMalloc failed: %s", cudaGetErrorString(e));
  }
  e = cudaMemcpy(d_raw, blocks, qb, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) {
    ggml_decode_enqueue(ggml_type, d_raw, d_out, n_elements, f16_rounding == CSK_F16_NEAREST, 0);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpy(out_f16, d_out, (size_t)n_elements * 2, cudaMemcpyDeviceToHost);
  cudaFree(d_raw);
  cudaFree(d_out);
  if (e != cudaSuccess) return fail(nullptr, CSK_ERR_CUDA, "dequant_ggml: %s", cudaGetErrorString(e));
  return CSK_OK;
}

int csk_moe_load_experts_mxfp4(csk_moe_layer* L, int32_t first_expert, int32_t count, const uint8_t* w_up,
                               const uint8_t* w_gate, const uint8_t* w_down, const float* b_up, const float* b_gate,
                               const float* b_down) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (L->w16) return fail(L, CSK_ERR_INVALID, "this layer holds fp16 weights: use csk_moe_load_expert_f16");
  if (count <= 0 || first_expert < L->e0 || first_expert + count > L->e0 + L->Eloc)
    return fail(L, CSK_ERR_INVALID, "experts [%d,%d) are not all resident on this device (range [%d,%d))", first_expert,
                first_expert + count, L->e0, L->e0 + L->Eloc);
  if (!w_up || !w_gate || !w_down) return fail(L, CSK_ERR_INVALID, "null weight pointer");
  if (L->cfg.has_bias && (!b_up || !b_gate || !b_down))
    return fail(L, CSK_ERR_INVALID, "layer has biases but a bias pointer is null");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  if (!L->d_stage2) {
    cudaError_t e = cudaMalloc(&L->d_stage2, 3 * L->stage_bytes);
    if (e != cudaSuccess) return fail(L, CSK_ERR_NOMEM, "cudaMalloc failed: %s", cudaGetErrorString(e));
  }
  // two staging areas: the copies of expert i+1 run while expert i is repacked
  cudaStream_t s = L->stream, s2 = L->stream_in;
  for (int i = 0; i < count; ++i) {
    const int le = first_expert - L->e0 + i;
    cudaStream_t st = (i & 1) ? s2 : s;
    uint8_t* stage = (i & 1) ? L->d_stage2 : L->d_stage;
    const size_t wb = L->stage_bytes;
    int rc = load_expert_enqueue(L, le, w_up + (size_t)i * wb, w_gate + (size_t)i * wb, w_down + (size_t)i * wb,
                                 b_up ? b_up + (size_t)i * L->F : nullptr, b_gate ? b_gate + (size_t)i * L->F : nullptr,
                                 b_down ? b_down + (size_t)i * L->H : nullptr, stage, st);
    if (rc) return rc;
  }
  CSK_CUDA(L, cudaStreamSynchronize(s));
  CSK_CUDA(L, cudaStreamSynchronize(s2));
  for (int i = 0; i < count; ++i) L->resident[first_expert - L->e0 + i] = 1;
  return CSK_OK;
}

namespace {
struct ImageHeader {
  char magic[8];
  int32_t E, k, H, F, has_bias, e0, eloc, reserved;
  uint64_t expert_stride, off_gu, off_d, off_tgu, off_td, off_bias, off_meta;
};
ImageHeader image_header_of(const csk_moe_layer* L) {
  ImageHeader h{};
  memcpy(h.magic, "CSKMOE02", 8);  // 02: the streaming layout stores scale byte 255 as 254
  h.E = L->E; h.k = L->k; h.H = L->H; h.F = L->F; h.has_bias = L->cfg.has_bias; h.e0 = L->e0; h.eloc = L->Eloc;
  h.expert_stride = L->expert_stride; h.off_gu = L->off_gu; h.off_d = L->off_d; h.off_tgu = L->off_tgu;
  h.off_td = L->off_td; h.off_bias = L->off_bias; h.off_meta = L->off_meta;
  return h;
}
}  // namespace

int csk_moe_save_image(csk_moe_layer* L, const char* path) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!path) return fail(L, CSK_ERR_INVALID, "null path");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  FILE* f = fopen(path, "wb");
  if (!f) return fail(L, CSK_ERR_INVALID, "cannot open %s for writing", path);
  const ImageHeader h = image_header_of(L);
  bool ok = fwrite(&h, sizeof h, 1, f) == 1 && fwrite(L->resident.data(), 1, L->Eloc, f) == (size_t)L->Eloc;
  std::vector<uint8_t> buf(L->expert_stride);
  for (int e = 0; ok && e < L->Eloc; ++e) {
    if (cudaMemcpy(buf.data(), L->d_weights + (size_t)e * L->expert_stride, L->expert_stride, cudaMemcpyDeviceToHost) != cudaSuccess) ok = false;
    ok = ok && fwrite(buf.data(), 1, buf.size(), f) == buf.size();
  }
  ok = fclose(f) == 0 && ok;
  if (!ok) return fail(L, CSK_ERR_CUDA, "writing the weight image to %s failed", path);
  return CSK_OK;
}

int csk_moe_load_image(csk_moe_layer* L, const char* path) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!path) return fail(L, CSK_ERR_INVALID, "null path");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  FILE* f = fopen(path, "rb");
  if (!f) return fail(L, CSK_ERR_INVALID, "cannot open %s", path);
  ImageHeader h{};
  const ImageHeader want = image_header_of(L);
  std::vector<uint8_t> res(L->Eloc);
  bool ok = fread(&h, sizeof h, 1, f) == 1;
  if (ok && memcmp(&h, &want, sizeof h) != 0) {
    fclose(f);
    return fail(L, CSK_ERR_INVALID, "%s was written for another layer shape, expert range or library layout", path);
  }
  ok = ok && fread(res.data(), 1, L->Eloc, f) == (size_t)L->Eloc;
  std::vector<uint8_t> buf(L->expert_stride);
  for (int e = 0; ok && e < L->Eloc; ++e) {
    ok = fread(buf.data(), 1, buf.size(), f) == buf.size();
    if (ok && cudaMemcpy(L->d_weights + (size_t)e * L->expert_stride, buf.data(), L->expert_stride, cudaMemcpyHostToDevice) != cudaSuccess) ok = false;
  }
  fclose(f);
  if (!ok) return fail(L, CSK_ERR_CUDA, "reading the weight image from %s failed", path);
  CSK_CUDA(L, cudaMemcpy(L->d_resident, res.data(), L->Eloc, cudaMemcpyHostToDevice));
  L->resident = res;
  return CSK_OK;
}

int csk_moe_unpack_expert_mxfp4(csk_moe_layer* L, int32_t expert_id, int32_t which, uint8_t* out) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (expert_id < L->e0 || expert_id >= L->e0 + L->Eloc || !L->resident[expert_id - L->e0])
    return fail(L, CSK_ERR_MISSING, "expert %d is not loaded", expert_id);
  if (which < 0 || which > 5 || !out) return fail(L, CSK_ERR_INVALID, "bad argument");
  if (L->w16) return fail(L, CSK_ERR_INVALID, "this layer holds fp16 weights, not MXFP4 blocks");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  const uint8_t* base = L->d_weights + (size_t)(expert_id - L->e0) * L->expert_stride;
  if (which < 3) {
    const MatLayout& lay = which == 2 ? L->Ld : L->Lgu;
    const uint8_t* packed = base + (which == 2 ? L->off_d : L->off_gu);
    k_unpack<<<grid_for((size_t)lay.N * (lay.K / 32), 128, 4096), 128, 0, L->stream>>>(
        packed, L->d_stage, lay, which == 0 ? 1 : 0);
  } else {
    const int w = which - 3;
    const TileLayout& lay = w == 2 ? L->Td : L->Tgu;
    const uint8_t* packed = base + (w == 2 ? L->off_td : L->off_tgu);
    k_unpack_tile<<<grid_for((size_t)lay.N * (lay.K / 32), 128, 4096), 128, 0, L->stream>>>(
        packed, L->d_stage, lay, w == 0 ? 1 : 0);
  }
  CSK_CUDA(L, cudaGetLastError());
  CSK_CUDA(L, cudaMemcpyAsync(out, L->d_stage, L->stage_bytes, cudaMemcpyDeviceToHost, L->stream));
  CSK_CUDA(L, cudaStreamSynchronize(L->stream));
  return CSK_OK;
}

int csk_moe_expert_resident(const csk_moe_layer* L, int32_t expert_id) {
  if (!L || expert_id < L->e0 || expert_id >= L->e0 + L->Eloc) return 0;
  return L->resident[expert_id - L->e0];
}

int csk_moe_set_path(csk_moe_layer* L, int32_t path) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (path < CSK_PATH_AUTO || path > CSK_PATH_TILE_PAIR) return fail(L, CSK_ERR_INVALID, "unknown path %d", path);
  if (L->w16 && (path == CSK_PATH_STREAM || path == CSK_PATH_TILE_PAIR))
    return fail(L, CSK_ERR_INVALID, "fp16 weights run on the one-CTA tensor-core kernel only");
  if (path == CSK_PATH_TILE_PAIR && !L->pair.available)
    return fail(L, CSK_ERR_INVALID, "the CTA-pair kernel is not available on this device: %s", L->pair.err.c_str());
  L->path = path;
  drop_graphs(L);
  return CSK_OK;
}

int csk_moe_set_activation(csk_moe_layer* L, int32_t activation, int32_t weight_before_ffn) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (activation != CSK_ACT_MODIFIED_SWIGLU && activation != CSK_ACT_STANDARD_SWIGLU)
    return fail(L, CSK_ERR_INVALID, "unknown activation %d", activation);
  if (L->cfg.activation == activation && (L->cfg.weight_before_ffn != 0) == (weight_before_ffn != 0)) return CSK_OK;
  L->cfg.activation = activation;
  L->cfg.weight_before_ffn = weight_before_ffn != 0;
  drop_graphs(L);
  return CSK_OK;
}

int csk_moe_set_router_mode(csk_moe_layer* L, int32_t mode) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (mode < CSK_ROUTER_AUTO || mode > CSK_ROUTER_CERTIFIED) return fail(L, CSK_ERR_INVALID, "unknown router mode %d", mode);
  L->router_mode = mode;
  drop_graphs(L);
  return CSK_OK;
}

int csk_moe_get_router_stats(csk_moe_layer* L, int64_t* routed_tokens, int64_t* chain_tokens) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  unsigned long long fb = 0;
  CSK_CUDA(L, cudaMemcpy(&fb, L->d_fb + 2, sizeof(fb), cudaMemcpyDeviceToHost));
  if (routed_tokens) *routed_tokens = L->routed_tokens;
  if (chain_tokens) *chain_tokens = (int64_t)fb;
  return CSK_OK;
}

int csk_moe_enable_timing(csk_moe_layer* L, int32_t on) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  L->timing = on != 0;
  return CSK_OK;
}

int csk_moe_sync(csk_moe_layer* L) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  int rc = check_device_status(L, L->last_stream ? L->last_stream : L->stream);
  if (rc) return rc;
  if (L->timing && L->n_marks > 1) finish_timings(L, L->n_marks, L->last_routed);
  return CSK_OK;
}

int csk_moe_get_timings(csk_moe_layer* L, csk_moe_timings* out) {
  if (check_layer(L) || !out) return CSK_ERR_INVALID;
  *out = L->last;
  return CSK_OK;
}

int csk_moe_get_counters(csk_moe_layer* L, int64_t* rows_per_expert, int64_t* distinct,
                         int64_t* weight_bytes) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  std::vector<int> c(L->E);
  CSK_CUDA(L, cudaMemcpy(c.data(), L->counts_in_carry ? L->d_carry + 1 : L->d_counts, sizeof(int) * L->E,
                         cudaMemcpyDeviceToHost));
  int64_t d = 0;
  for (int e = 0; e < L->E; ++e) {
    if (rows_per_expert) rows_per_expert[e] = c[e];
    if (c[e] > 0) ++d;
  }
  if (distinct) *distinct = d;
  if (weight_bytes) {
    const int64_t per = (int64_t)3 * L->H * L->F / 32 * 17 +
                        (L->cfg.has_bias ? (int64_t)sizeof(float) * (2 * L->F + L->H) : 0);
    *weight_bytes = d * per;
  }
  return CSK_OK;
}

// ---- device-buffer entry points -------------------------------------------
int csk_moe_route_dev(csk_moe_layer* L, const float* d_hidden, int64_t T, float* d_router_out, void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!d_hidden || !d_router_out) return fail(L, CSK_ERR_INVALID, "null argument");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  L->last = csk_moe_timings{};
  return launch_router(L, d_hidden, T, d_router_out, pick(L, stream));
}

int csk_moe_forward_dev(csk_moe_layer* L, const float* d_hidden, int64_t T, const float* d_router_in,
                        float* d_router_out, float* d_out, void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!d_hidden || !d_out) return fail(L, CSK_ERR_INVALID, "null argument");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = pick(L, stream);
  constexpr int64_t kGraphMaxTokens = 512;
  if (!L->use_graphs || L->timing || L->debug_stall || T > kGraphMaxTokens || T <= 0 || T > L->max_T)
    return forward_dev(L, d_hidden, T, d_router_in, d_router_out, d_out, -1, s, false);
  for (auto& g : L->graphs)
    if (g.T == T && g.hidden == d_hidden && g.router_in == d_router_in && g.router_out == d_router_out &&
        g.out == d_out && g.stream == s) {
      CSK_CUDA(L, cudaGraphLaunch(g.exec, s));
      L->last_T = T;
      L->last_stream = s;
      L->n_marks = 0;
      return CSK_OK;
    }
  // first call with these arguments: capture the sequence, then replay it
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) {
    cudaGetLastError();  // the caller is capturing this stream itself: just enqueue
    return forward_dev(L, d_hidden, T, d_router_in, d_router_out, d_out, -1, s, false);
  }
  if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    cudaGetLastError();
    return forward_dev(L, d_hidden, T, d_router_in, d_router_out, d_out, -1, s, false);
  }
  int rc = forward_dev(L, d_hidden, T, d_router_in, d_router_out, d_out, -1, s, false);
  cudaGraph_t graph = nullptr;
  cudaError_t ce = cudaStreamEndCapture(s, &graph);
  if (rc || ce != cudaSuccess || !graph) {
    cudaGetLastError();
    if (graph) cudaGraphDestroy(graph);
    if (rc) return rc;
    L->use_graphs = false;  // capture is not possible here: fall back to plain launches for good
    return forward_dev(L, d_hidden, T, d_router_in, d_router_out, d_out, -1, s, false);
  }
  cudaGraphExec_t exec = nullptr;
  ce = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (ce != cudaSuccess || !exec) {
    cudaGetLastError();
    L->use_graphs = false;
    return forward_dev(L, d_hidden, T, d_router_in, d_router_out, d_out, -1, s, false);
  }
  if (L->graphs.size() >= 32) {
    cudaGraphExecDestroy(L->graphs.front().exec);
    L->graphs.erase(L->graphs.begin());
  }
  L->graphs.push_back({T, d_hidden, d_router_in, d_router_out, d_out, s, exec});
  CSK_CUDA(L, cudaGraphLaunch(exec, s));
  return CSK_OK;
}

// ---- the layer with the steps either side of it ------------------------------
int csk_moe_set_ffn_norm(csk_moe_layer* L, const float* weight, float eps) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!weight) return fail(L, CSK_ERR_INVALID, "norm weight is null");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  if (!L->d_norm_w) {
    cudaError_t e = cudaMalloc(&L->d_norm_w, sizeof(float) * L->H);
    if (e == cudaSuccess) e = cudaMalloc(&L->d_normed, sizeof(float) * L->max_T * L->H);
    if (e != cudaSuccess) return fail(L, CSK_ERR_NOMEM, "cudaMalloc failed: %s", cudaGetErrorString(e));
    CSK_CUDA(L, cudaFuncSetAttribute(k_rmsnorm, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * (int)sizeof(float) * L->H));
  }
  CSK_CUDA(L, cudaMemcpyAsync(L->d_norm_w, weight, sizeof(float) * L->H, cudaMemcpyHostToDevice, L->stream));
  CSK_CUDA(L, cudaStreamSynchronize(L->stream));
  L->norm_eps = eps;
  return CSK_OK;
}

int csk_moe_block_forward_dev(csk_moe_layer* L, const float* d_x, int64_t T, float* d_router_out, float* d_out,
                              void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!d_x || !d_out) return fail(L, CSK_ERR_INVALID, "null argument");
  if (!L->d_norm_w) return fail(L, CSK_ERR_INVALID, "the norm weight was never set (csk_moe_set_ffn_norm)");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  if (reinterpret_cast<uintptr_t>(d_x) % 16 || reinterpret_cast<uintptr_t>(d_out) % 16)
    return fail(L, CSK_ERR_INVALID, "activations must be 16-byte aligned");
  if ((size_t)L->H * sizeof(float) * 4 > 200 * 1024) return fail(L, CSK_ERR_NOMEM, "hidden dimension too large for the norm kernel's row buffer");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = pick(L, stream);
  const int blocks = (int)std::min<int64_t>((T + 3) / 4, 4 * (int64_t)L->sm_count);
  k_rmsnorm<<<blocks, 128, 4 * sizeof(float) * L->H, s>>>(d_x, L->d_norm_w, L->norm_eps, L->d_normed, (int)T, L->H);
  CSK_CUDA(L, cudaGetLastError());
  return forward_dev(L, L->d_normed, T, nullptr, d_router_out, d_out, -1, s, false, d_x);
}

int csk_moe_block_forward_shared_dev(csk_moe_layer* L, csk_moe_layer* S, const float* d_x, int64_t T,
                                     float* d_router_out, float* d_out, void* stream) {
  if (!S) return csk_moe_block_forward_dev(L, d_x, T, d_router_out, d_out, stream);
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!d_x || !d_out) return fail(L, CSK_ERR_INVALID, "null argument");
  if (!L->d_norm_w) return fail(L, CSK_ERR_INVALID, "the norm weight was never set (csk_moe_set_ffn_norm)");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  if (S == L || !S->d_unit_router || S->H != L->H || S->cfg.device != L->cfg.device)
    return fail(L, CSK_ERR_INVALID, "the shared expert must be another layer on the same device with num_experts = top_k = 1 "
                                    "and the same hidden size");
  if (T > S->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld exceeds the shared expert's max_tokens", (long long)T);
  if (!S->resident[0]) return fail(L, CSK_ERR_MISSING, "the shared expert's weights are not loaded");
  if (reinterpret_cast<uintptr_t>(d_x) % 16 || reinterpret_cast<uintptr_t>(d_out) % 16)
    return fail(L, CSK_ERR_INVALID, "activations must be 16-byte aligned");
  if ((size_t)L->H * sizeof(float) * 4 > 200 * 1024) return fail(L, CSK_ERR_NOMEM, "hidden dimension too large for the norm kernel's row buffer");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  if (!L->d_shared_out) {
    cudaError_t e = cudaMalloc(&L->d_shared_out, sizeof(float) * L->max_T * L->H);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&L->ev_shared_fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&L->ev_shared_join, cudaEventDisableTiming);
    if (e != cudaSuccess) return fail(L, CSK_ERR_NOMEM, "shared-expert buffers: %s", cudaGetErrorString(e));
  }
  cudaStream_t s = pick(L, stream);
  const int blocks = (int)std::min<int64_t>((T + 3) / 4, 4 * (int64_t)L->sm_count);
  k_rmsnorm<<<blocks, 128, 4 * sizeof(float) * L->H, s>>>(d_x, L->d_norm_w, L->norm_eps, L->d_normed, (int)T, L->H);
  CSK_CUDA(L, cudaGetLastError());
  // the shared expert reads the normed rows on its own stream, next to the routed experts; the combine joins them
  CSK_CUDA(L, cudaEventRecord(L->ev_shared_fork, s));
  CSK_CUDA(L, cudaStreamWaitEvent(S->stream, L->ev_shared_fork, 0));
  int rc = csk_moe_dense_forward_dev(S, L->d_normed, T, L->d_shared_out, S->stream);
  if (rc) return fail(L, rc, "shared expert: %s", S->err.c_str());
  CSK_CUDA(L, cudaEventRecord(L->ev_shared_join, S->stream));
  return forward_dev(L, L->d_normed, T, nullptr, d_router_out, d_out, -1, s, false, d_x, L->d_shared_out, L->ev_shared_join);
}

int csk_moe_block_forward_shared(csk_moe_layer* L, csk_moe_layer* S, const float* x, int64_t T, float* router_out,
                                 float* out) {
  if (!S) return csk_moe_block_forward(L, x, T, router_out, out);
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!x || !out) return fail(L, CSK_ERR_INVALID, "null argument");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = L->stream;
  CSK_CUDA(L, cudaMemcpyAsync(L->d_hidden, x, sizeof(float) * T * L->H, cudaMemcpyHostToDevice, s));
  int rc = csk_moe_block_forward_shared_dev(L, S, L->d_hidden, T, L->d_router, L->d_out, s);
  if (rc) return rc;
  rc = check_device_status(L, s);
  if (rc) return rc;
  rc = check_device_status(S, S->stream);
  if (rc) return fail(L, rc, "shared expert: %s", S->err.c_str());
  CSK_CUDA(L, cudaMemcpyAsync(out, L->d_out, sizeof(float) * T * L->H, cudaMemcpyDeviceToHost, s));
  if (router_out)
    CSK_CUDA(L, cudaMemcpyAsync(router_out, L->d_router, sizeof(float) * T * L->k * 2, cudaMemcpyDeviceToHost, s));
  CSK_CUDA(L, cudaStreamSynchronize(s));
  return CSK_OK;
}

int csk_moe_block_forward(csk_moe_layer* L, const float* x, int64_t T, float* router_out, float* out) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!x || !out) return fail(L, CSK_ERR_INVALID, "null argument");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = L->stream;
  CSK_CUDA(L, cudaMemcpyAsync(L->d_hidden, x, sizeof(float) * T * L->H, cudaMemcpyHostToDevice, s));
  int rc = csk_moe_block_forward_dev(L, L->d_hidden, T, L->d_router, L->d_out, s);
  if (rc) return rc;
  rc = check_device_status(L, s);
  if (rc) return rc;
  CSK_CUDA(L, cudaMemcpyAsync(out, L->d_out, sizeof(float) * T * L->H, cudaMemcpyDeviceToHost, s));
  if (router_out)
    CSK_CUDA(L, cudaMemcpyAsync(router_out, L->d_router, sizeof(float) * T * L->k * 2, cudaMemcpyDeviceToHost, s));
  CSK_CUDA(L, cudaStreamSynchronize(s));
  return CSK_OK;
}

// ---- host-buffer entry points ----------------------------------------------
int csk_moe_route(csk_moe_layer* L, const float* hidden, int64_t T, float* router_out) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!hidden || !router_out) return fail(L, CSK_ERR_INVALID, "null argument");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = L->stream;
  L->last = csk_moe_timings{};
  CSK_CUDA(L, cudaMemcpyAsync(L->d_hidden, hidden, sizeof(float) * T * L->H, cudaMemcpyHostToDevice, s));
  int rc = launch_router(L, L->d_hidden, T, L->d_router, s);
  if (rc) return rc;
  CSK_CUDA(L, cudaMemcpyAsync(router_out, L->d_router, sizeof(float) * T * L->k * 2, cudaMemcpyDeviceToHost, s));
  CSK_CUDA(L, cudaStreamSynchronize(s));
  return CSK_OK;
}

namespace {
// How many passes the host entry point cuts a batch into so that the copies of one pass overlap
// the kernels of another: as many as leave every expert about 128 rows per pass (the tensor-core
// kernel's cost per row tile is nearly flat below that), at most two (measured: four passes cost more
// in kernel time than they hide in copies); small batches take one.
int host_passes(const csk_moe_layer* L, int64_t T) {
  if (L->timing || L->path == CSK_PATH_STREAM) return 1;
  const int64_t rows_per_expert = T * L->k / std::max(1, L->Eloc);
  return (int)std::max<int64_t>(1, std::min<int64_t>(2, rows_per_expert / 128));
}
}  // namespace

int csk_moe_forward(csk_moe_layer* L, const float* hidden, int64_t T, const float* router_in,
                    float* router_out, float* out) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!hidden || !out) return fail(L, CSK_ERR_INVALID, "null argument");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = L->stream;
  const int passes = host_passes(L, T);
  if (passes == 1) {
    CSK_CUDA(L, cudaMemcpyAsync(L->d_hidden, hidden, sizeof(float) * T * L->H, cudaMemcpyHostToDevice, s));
    if (router_in)
      CSK_CUDA(L, cudaMemcpyAsync(L->d_router, router_in, sizeof(float) * T * L->k * 2, cudaMemcpyHostToDevice, s));
    int rc = csk_moe_forward_dev(L, L->d_hidden, T, router_in ? L->d_router : nullptr, nullptr, L->d_out, s);
    if (rc) return rc;
    rc = check_device_status(L, s);
    if (rc) return rc;
    if (L->timing && L->n_marks > 1) finish_timings(L, L->n_marks, L->last_routed);
    CSK_CUDA(L, cudaMemcpyAsync(out, L->d_out, sizeof(float) * T * L->H, cudaMemcpyDeviceToHost, s));
    if (router_out)
      CSK_CUDA(L, cudaMemcpyAsync(router_out, L->d_router, sizeof(float) * T * L->k * 2, cudaMemcpyDeviceToHost, s));
    CSK_CUDA(L, cudaStreamSynchronize(s));
    return CSK_OK;
  }
  // Several passes over token ranges, three streams: the rows of pass i+1 arrive and the results of
  // pass i-1 leave while the kernels of pass i run (tokens are independent, so the passes give the
  // same rows as one pass would).  One cudaMemcpyAsync per range and direction.  The status word of
  // every pass is folded into a sticky one that is read once, at the end.
  CSK_CUDA(L, cudaMemsetAsync(L->d_carry, 0, sizeof(int) * (1 + L->E), s));
  CSK_CUDA(L, cudaEventRecord(L->ev_free, s));  // earlier work on this handle is done before the copies overwrite d_hidden
  CSK_CUDA(L, cudaStreamWaitEvent(L->stream_in, L->ev_free, 0));
  struct CarryScope {
    csk_moe_layer* l;
    ~CarryScope() { l->carry_active = false; }
  } carry_scope{L};
  L->carry_active = true;
  const int k2 = L->k * 2;
  int rc = CSK_OK;
  for (int p = 0; p < passes && !rc; ++p) {
    const int64_t t0 = T * p / passes, t1 = T * (p + 1) / passes, n = t1 - t0;

    CSK_CUDA(L, cudaMemcpyAsync(L->d_hidden + t0 * L->H, hidden + t0 * L->H, sizeof(float) * n * L->H,
                                cudaMemcpyHostToDevice, L->stream_in));
    if (router_in)
      CSK_CUDA(L, cudaMemcpyAsync(L->d_router + t0 * k2, router_in + t0 * k2, sizeof(float) * n * k2,
                                  cudaMemcpyHostToDevice, L->stream_in));
    CSK_CUDA(L, cudaEventRecord(L->ev_in[p], L->stream_in));
    CSK_CUDA(L, cudaStreamWaitEvent(s, L->ev_in[p], 0));
    // the router writes the pass's routing to its place in d_router (kept for router_out and for the counters)
    rc = forward_dev(L, L->d_hidden + t0 * L->H, n, router_in ? L->d_router + t0 * k2 : nullptr,
                     router_in ? nullptr : L->d_router + t0 * k2, L->d_out + t0 * L->H, -1, s, false);
    if (rc) break;
    CSK_CUDA(L, cudaEventRecord(L->ev_done[p], s));
    CSK_CUDA(L, cudaStreamWaitEvent(L->stream_out, L->ev_done[p], 0));
    CSK_CUDA(L, cudaMemcpyAsync(out + t0 * L->H, L->d_out + t0 * L->H, sizeof(float) * n * L->H,
                                cudaMemcpyDeviceToHost, L->stream_out));
    if (router_out)
      CSK_CUDA(L, cudaMemcpyAsync(router_out + t0 * k2, L->d_router + t0 * k2, sizeof(float) * n * k2,
                                  cudaMemcpyDeviceToHost, L->stream_out));
  }
  L->counts_in_carry = true;
  L->last_T = T;
  // the sticky status word travels with the last results
  cudaMemcpyAsync(L->h_meta, L->d_meta, sizeof(int) * 16, cudaMemcpyDeviceToHost, L->stream_out);
  cudaMemcpyAsync(L->h_meta + 3, L->d_carry, sizeof(int), cudaMemcpyDeviceToHost, L->stream_out);
  cudaError_t e1 = cudaStreamSynchronize(L->stream_in), e2 = cudaStreamSynchronize(s), e3 = cudaStreamSynchronize(L->stream_out);
  if (rc) return rc;
  if (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess)
    return fail(L, CSK_ERR_CUDA, "pipelined forward: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2 != cudaSuccess ? e2 : e3));
  return report_status(L, L->h_meta[3] | L->h_meta[8], s);
}

int csk_moe_dense_forward_dev(csk_moe_layer* L, const float* d_hidden, int64_t T, float* d_out, void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!L->d_unit_router) return fail(L, CSK_ERR_INVALID, "dense forward needs a layer with num_experts = top_k = 1");
  return csk_moe_forward_dev(L, d_hidden, T, L->d_unit_router, nullptr, d_out, stream);
}

int csk_moe_dense_forward(csk_moe_layer* L, const float* hidden, int64_t T, float* out) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!L->d_unit_router) return fail(L, CSK_ERR_INVALID, "dense forward needs a layer with num_experts = top_k = 1");
  if (!hidden || !out) return fail(L, CSK_ERR_INVALID, "null argument");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = L->stream;
  CSK_CUDA(L, cudaMemcpyAsync(L->d_hidden, hidden, sizeof(float) * T * L->H, cudaMemcpyHostToDevice, s));
  int rc = forward_dev(L, L->d_hidden, T, L->d_unit_router, nullptr, L->d_out, -1, s, true);
  if (rc) return rc;
  CSK_CUDA(L, cudaMemcpyAsync(out, L->d_out, sizeof(float) * T * L->H, cudaMemcpyDeviceToHost, s));
  CSK_CUDA(L, cudaStreamSynchronize(s));
  return CSK_OK;
}

int csk_moe_expert_forward(csk_moe_layer* L, int32_t expert_id, const float* hidden, int64_t T,
                           const float* router_out, float* out, int32_t* selected) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!hidden || !router_out || !out || !selected) return fail(L, CSK_ERR_INVALID, "null argument");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  if (expert_id < L->e0 || expert_id >= L->e0 + L->Eloc || !L->resident[expert_id - L->e0])
    return fail(L, CSK_ERR_MISSING, "expert %d is not loaded", expert_id);
  // the reference's early return: no token selected this expert (expert_mlp_node.h:441-443)
  bool any = false;
  for (int64_t i = 0; i < T * L->k && !any; ++i) any = (int)router_out[2 * i] == expert_id;
  *selected = any ? 1 : 0;
  if (!any) return CSK_OK;
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = L->stream;
  CSK_CUDA(L, cudaMemcpyAsync(L->d_hidden, hidden, sizeof(float) * T * L->H, cudaMemcpyHostToDevice, s));
  CSK_CUDA(L, cudaMemcpyAsync(L->d_router, router_out, sizeof(float) * T * L->k * 2, cudaMemcpyHostToDevice, s));
  int rc = forward_dev(L, L->d_hidden, T, L->d_router, nullptr, L->d_out, expert_id, s, true);
  if (rc) return rc;
  CSK_CUDA(L, cudaMemcpyAsync(out, L->d_out, sizeof(float) * T * L->H, cudaMemcpyDeviceToHost, s));
  CSK_CUDA(L, cudaStreamSynchronize(s));
  return CSK_OK;
}

int csk_moe_merge(csk_moe_layer* L, const float* router_out, int64_t T, const float* const* expert_outs,
                  float* out) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!router_out || !expert_outs || !out) return fail(L, CSK_ERR_INVALID, "null argument");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  bool any = false;
  for (int e = 0; e < L->E; ++e) any = any || expert_outs[e];
  if (!any) return fail(L, CSK_ERR_INVALID, "expert_merge: no non-empty expert outputs found");
  // Only the k rows each token actually uses travel to the device: row (t,j)
  // of expert e(t,j), or nothing when that expert's output is the empty tensor.
  std::vector<int> rows((size_t)T * L->k, -1);
  std::vector<float> packed;
  packed.reserve((size_t)T * L->k * L->H);
  int n = 0;
  for (int64_t t = 0; t < T; ++t)
    for (int j = 0; j < L->k; ++j) {
      const int e = (int)router_out[(t * L->k + j) * 2];
      if (e < 0 || e >= L->E)
        return fail(L, CSK_ERR_INVALID, "expert_merge: expert_idx out of range: %d", e);
      if (!expert_outs[e]) continue;
      rows[t * L->k + j] = n++;
      const float* src = expert_outs[e] + t * L->H;
      packed.insert(packed.end(), src, src + L->H);
    }
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = L->stream;
  CSK_CUDA(L, cudaMemcpyAsync(L->d_y, packed.data(), sizeof(float) * packed.size(), cudaMemcpyHostToDevice, s));
  CSK_CUDA(L, cudaMemcpyAsync(L->d_row_of_pair, rows.data(), sizeof(int) * rows.size(), cudaMemcpyHostToDevice, s));
  CSK_CUDA(L, cudaMemcpyAsync(L->d_router, router_out, sizeof(float) * T * L->k * 2, cudaMemcpyHostToDevice, s));
  k_combine<<<(unsigned)T, 256, 0, s>>>(L->d_router, L->d_row_of_pair, L->d_y, L->H, L->d_out, (int)T,
                                        L->k, L->H, L->cfg.weight_before_ffn, 0, nullptr, nullptr, nullptr, 0);
  CSK_CUDA(L, cudaGetLastError());
  CSK_CUDA(L, cudaMemcpyAsync(out, L->d_out, sizeof(float) * T * L->H, cudaMemcpyDeviceToHost, s));
  CSK_CUDA(L, cudaStreamSynchronize(s));
  return CSK_OK;
}

// ---- expert parallelism -------------------------------------------------------
int csk_moe_ep_row_pitch(const csk_moe_layer* L) { return L ? L->ldx : CSK_ERR_INVALID; }

int csk_moe_ep_dispatch_dev(csk_moe_layer* L, const float* d_hidden, int64_t T, const float* d_router_in,
                            void* d_send_f16, int32_t* d_counts, void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!d_hidden || !d_send_f16 || !d_counts) return fail(L, CSK_ERR_INVALID, "null argument");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = pick(L, stream);
  L->last = csk_moe_timings{};
  L->last_T = T;
  if (!d_router_in) {
    int rc = launch_router(L, d_hidden, T, L->d_router, s);
    if (rc) return rc;
  } else if (d_router_in != L->d_router) {
    CSK_CUDA(L, cudaMemcpyAsync(L->d_router, d_router_in, sizeof(float) * T * L->k * 2,
                                cudaMemcpyDeviceToDevice, s));
  }
  const float* router = L->d_router;
  if (L->has_slot_map) {
    k_ep_slots<<<grid_for((size_t)T * L->k, 256, 4 * L->sm_count), 256, 0, s>>>(
        L->d_router, L->d_router_phys, (int)(T * L->k), L->k, L->E_router, L->d_slot_map, L->d_slot_map + L->E);
    CSK_CUDA(L, cudaGetLastError());
    router = L->d_router_phys;
  }
  // group by global expert id; no tiles are built here (e_count = 0)
  int rc = launch_permute(L, d_hidden, router, T, -1, 8, 0, 0, (__half*)d_send_f16, L->ldx,
                          T * L->k, s);
  if (rc) return rc;
  CSK_CUDA(L, cudaMemcpyAsync(d_counts, L->d_counts, sizeof(int) * L->E, cudaMemcpyDeviceToDevice, s));
  return CSK_OK;
}

int csk_moe_ep_set_slot_map(csk_moe_layer* L, int32_t n_logical, const int32_t* primary_slot,
                            const int32_t* replica_slot) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  drop_graphs(L);
  if (n_logical == 0) {
    if (L->has_slot_map) L->router_set = false;
    L->has_slot_map = false;
    L->E_router = L->E;
    return CSK_OK;
  }
  if (n_logical < L->k || n_logical > L->E || !primary_slot)
    return fail(L, CSK_ERR_INVALID, "slot map: need top_k <= n_logical <= num_experts (%d) and a primary_slot array, got %d",
                L->E, n_logical);
  std::vector<int> map(2 * (size_t)L->E, -1);
  std::vector<char> used(L->E, 0);
  for (int e = 0; e < n_logical; ++e) {
    for (int c = 0; c < 2; ++c) {
      const int s = c == 0 ? primary_slot[e] : (replica_slot ? replica_slot[e] : -1);
      if (c == 1 && s == -1) continue;
      if (s < 0 || s >= L->E) return fail(L, CSK_ERR_INVALID, "slot map: slot %d of expert %d is outside [0,%d)", s, e, L->E);
      if (used[s]) return fail(L, CSK_ERR_INVALID, "slot map: slot %d is used twice", s);
      used[s] = 1;
      map[(size_t)c * L->E + e] = s;
    }
  }
  CSK_CUDA(L, cudaMemcpyAsync(L->d_slot_map, map.data(), sizeof(int) * map.size(), cudaMemcpyHostToDevice, L->stream));
  CSK_CUDA(L, cudaStreamSynchronize(L->stream));
  L->has_slot_map = true;
  L->E_router = n_logical;
  L->router_set = false;  // the router's weights are per logical expert from here on
  return CSK_OK;
}

// ---- expert parallelism over peer memory ----------------------------------------
namespace {
// End of an experts stage: enqueue only, unless timing is on (then wait, check the status word, read the events).
int ep_finish(csk_moe_layer* L, cudaStream_t s, int n_marks) {
  L->last_stream = s;
  if (!L->timing) return CSK_OK;  // csk_moe_sync reports what the kernels found
  int rc = check_device_status(L, s);
  if (rc) return rc;
  if (n_marks == 3) {  // the status check above already waited for the stream
    cudaEventElapsedTime(&L->last.gate_up_ms, L->ev[0], L->ev[1]);
    cudaEventElapsedTime(&L->last.down_ms, L->ev[1], L->ev[2]);
    L->last.total_ms = L->last.gate_up_ms + L->last.down_ms;
  }
  return CSK_OK;
}
int p2p_alloc_local(csk_moe_layer* L) {
  if (L->d_info) return CSK_OK;
  CSK_CUDA(L, cudaMalloc(&L->d_info, sizeof(RowOrigin) * (size_t)L->max_rows));
  // 0xFF bytes: (-1, -1), which no reader accepts as an origin (rows a sender had to skip stay that way)
  CSK_CUDA(L, cudaMemset(L->d_info, 0xFF, sizeof(RowOrigin) * (size_t)L->max_rows));
  // the return buffer carries the sync area of the flag barriers at its tail (peers can write both)
  L->back_tail = (size_t)L->max_T * L->k * L->H;
  const size_t back_bytes = sizeof(float) * L->back_tail + sizeof(int) * ep_sync_ints(L->E);
  CSK_CUDA(L, cudaMalloc(&L->d_back, back_bytes));
  CSK_CUDA(L, cudaMemset(reinterpret_cast<uint8_t*>(L->d_back) + sizeof(float) * L->back_tail, 0, sizeof(int) * ep_sync_ints(L->E)));
  CSK_CUDA(L, cudaMalloc(&L->d_row_ptr, sizeof(float*) * (size_t)L->max_rows));
  return CSK_OK;
}
int p2p_set_peers(csk_moe_layer* L, int rank, int world, void* const* x16, void* const* info, void* const* back) {
  if (world < 1 || world > 64 || rank < 0 || rank >= world) return fail(L, CSK_ERR_INVALID, "p2p: bad rank/world %d/%d", rank, world);
  if (L->E % world || L->Eloc != L->E / world || L->e0 != rank * L->Eloc)
    return fail(L, CSK_ERR_INVALID, "p2p: rank %d of %d must own expert slots [%d, %d)", rank, world,
                rank * (L->E / std::max(1, world)), (rank + 1) * (L->E / std::max(1, world)));
  for (void** p : {(void**)&L->d_peer_x16, (void**)&L->d_peer_info, (void**)&L->d_peer_back}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  CSK_CUDA(L, cudaMalloc(&L->d_peer_x16, sizeof(void*) * world));
  CSK_CUDA(L, cudaMalloc(&L->d_peer_info, sizeof(void*) * world));
  CSK_CUDA(L, cudaMalloc(&L->d_peer_back, sizeof(void*) * world));
  CSK_CUDA(L, cudaMemcpy(L->d_peer_x16, x16, sizeof(void*) * world, cudaMemcpyHostToDevice));
  CSK_CUDA(L, cudaMemcpy(L->d_peer_info, info, sizeof(void*) * world, cudaMemcpyHostToDevice));
  CSK_CUDA(L, cudaMemcpy(L->d_peer_back, back, sizeof(void*) * world, cudaMemcpyHostToDevice));
  L->p2p_rank = rank;
  L->p2p_world = world;
  return CSK_OK;
}
}  // namespace

int csk_moe_ep_p2p_local_ptrs(csk_moe_layer* L, void** x16, void** info, void** back) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  int rc = p2p_alloc_local(L);
  if (rc) return rc;
  if (x16) *x16 = L->d_x16;
  if (info) *info = L->d_info;
  if (back) *back = L->d_back;
  return CSK_OK;
}

int csk_moe_ep_p2p_export(csk_moe_layer* L, uint8_t* handles) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!handles) return fail(L, CSK_ERR_INVALID, "null argument");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  int rc = p2p_alloc_local(L);
  if (rc) return rc;
  static_assert(sizeof(cudaIpcMemHandle_t) + sizeof(uint64_t) == CSK_IPC_HANDLE_BYTES, "handle size");
  // the driver entry point is looked up at run time: the library has no link-time dependency on libcuda
  typedef CUresult (*GetRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
    cudaGetLastError();
    return fail(L, CSK_ERR_CUDA, "p2p: cuMemGetAddressRange not found in the driver");
  }
  const GetRangeFn get_range = (GetRangeFn)fn;
  void* bufs[3] = {L->d_x16, L->d_info, L->d_back};
  for (int i = 0; i < 3; ++i) {
    // a handle names the whole allocation a pointer lies in (small buffers share one): ship the offset too
    cudaIpcMemHandle_t h;
    CSK_CUDA(L, cudaIpcGetMemHandle(&h, bufs[i]));
    CUdeviceptr base = 0;
    size_t size = 0;
    if (get_range(&base, &size, (CUdeviceptr)bufs[i]) != CUDA_SUCCESS)
      return fail(L, CSK_ERR_CUDA, "p2p: cuMemGetAddressRange failed");
    const uint64_t off = (uint64_t)((CUdeviceptr)bufs[i] - base);
    memcpy(handles + (size_t)i * CSK_IPC_HANDLE_BYTES, &h, sizeof(h));
    memcpy(handles + (size_t)i * CSK_IPC_HANDLE_BYTES + sizeof(h), &off, sizeof(off));
  }
  return CSK_OK;
}

int csk_moe_ep_p2p_import(csk_moe_layer* L, int32_t rank, int32_t world, const uint8_t* all_handles) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!all_handles) return fail(L, CSK_ERR_INVALID, "null argument");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  int rc = p2p_alloc_local(L);
  if (rc) return rc;
  if (world < 1 || world > 64 || rank < 0 || rank >= world) return fail(L, CSK_ERR_INVALID, "p2p: bad rank/world %d/%d", rank, world);
  std::vector<void*> ptr(3 * (size_t)world, nullptr);
  std::vector<cudaIpcMemHandle_t> opened_handles;
  std::vector<void*> opened_ptrs;
  void* own[3] = {L->d_x16, L->d_info, L->d_back};
  for (int r = 0; r < world; ++r)
    for (int i = 0; i < 3; ++i) {
      if (r == rank) {
        ptr[(size_t)i * world + r] = own[i];
        continue;
      }
      cudaIpcMemHandle_t h;
      uint64_t off = 0;
      const uint8_t* rec = all_handles + ((size_t)r * 3 + i) * CSK_IPC_HANDLE_BYTES;
      memcpy(&h, rec, sizeof(h));
      memcpy(&off, rec + sizeof(h), sizeof(off));
      // two of a peer's buffers may lie in one allocation: open each allocation once
      void* p = nullptr;
      for (size_t j = 0; j < opened_handles.size(); ++j)
        if (!memcmp(&opened_handles[j], &h, sizeof(h))) p = opened_ptrs[j];
      if (!p) {
        CSK_CUDA(L, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        L->ipc_opened.push_back(p);
        opened_handles.push_back(h);
        opened_ptrs.push_back(p);
      }
      ptr[(size_t)i * world + r] = static_cast<uint8_t*>(p) + off;
    }
  return p2p_set_peers(L, rank, world, ptr.data(), ptr.data() + world, ptr.data() + 2 * (size_t)world);
}

int csk_moe_ep_p2p_import_ptrs(csk_moe_layer* L, int32_t rank, int32_t world, void* const* x16, void* const* info,
                               void* const* back) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!x16 || !info || !back) return fail(L, CSK_ERR_INVALID, "null argument");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  int rc = p2p_alloc_local(L);
  if (rc) return rc;
  return p2p_set_peers(L, rank, world, x16, info, back);
}

// Stage 1: route, map to slots, count this rank's rows per slot.
int csk_moe_ep_p2p_counts_dev(csk_moe_layer* L, const float* d_hidden, int64_t T, const float* d_router_in,
                              int32_t* d_counts, void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!d_hidden || !d_counts) return fail(L, CSK_ERR_INVALID, "null argument");
  if (L->p2p_world <= 0) return fail(L, CSK_ERR_INVALID, "p2p: peers were never imported");
  if (T <= 0 || T > L->max_T) return fail(L, CSK_ERR_NOMEM, "T=%lld outside (0, max_tokens]", (long long)T);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = pick(L, stream);
  L->last = csk_moe_timings{};
  L->last_T = T;
  if (!d_router_in) {
    int rc = launch_router(L, d_hidden, T, L->d_router, s);
    if (rc) return rc;
  } else if (d_router_in != L->d_router) {
    CSK_CUDA(L, cudaMemcpyAsync(L->d_router, d_router_in, sizeof(float) * T * L->k * 2, cudaMemcpyDeviceToDevice, s));
  }
  const int n_pairs = (int)(T * L->k);
  const float* router = L->d_router;
  if (L->has_slot_map) {
    k_ep_slots<<<grid_for((size_t)n_pairs, 256, 4 * L->sm_count), 256, 0, s>>>(
        L->d_router, L->d_router_phys, n_pairs, L->k, L->E_router, L->d_slot_map, L->d_slot_map + L->E);
    router = L->d_router_phys;
  }
  CSK_CUDA(L, cudaMemsetAsync(L->d_counts, 0, sizeof(int) * L->E, s));
  CSK_CUDA(L, cudaMemsetAsync(L->d_meta, 0, sizeof(int) * 8, s));
  k_hist<<<grid_for(n_pairs, 256, 2 * L->sm_count), 256, sizeof(int) * L->E, s>>>(router, n_pairs, L->E, -1, L->d_counts,
                                                                                 L->d_meta);
  CSK_CUDA(L, cudaGetLastError());
  CSK_CUDA(L, cudaMemcpyAsync(d_counts, L->d_counts, sizeof(int) * L->E, cudaMemcpyDeviceToDevice, s));
  return CSK_OK;
}

// Barrier `which` (0: counts, 1: rows landed, 2: outputs landed) between the ranks, by flags in peer
// memory; with d_counts / d_all_counts it also exchanges the per-slot row counts (the all-gather).
int csk_moe_ep_p2p_sync_dev(csk_moe_layer* L, int32_t which, const int32_t* d_counts, int32_t* d_all_counts, void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (L->p2p_world <= 0) return fail(L, CSK_ERR_INVALID, "p2p: peers were never imported");
  if (which < 0 || which > 2 || (d_counts == nullptr) != (d_all_counts == nullptr))
    return fail(L, CSK_ERR_INVALID, "p2p sync: which must be 0..2, counts and all_counts go together");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = pick(L, stream);
  k_ep_p2p_sync<<<1, 1024, 0, s>>>(L->d_peer_back, L->back_tail, L->p2p_rank, L->p2p_world, which, L->d_p2p_epoch,
                                   d_counts, L->E, d_all_counts, L->d_meta);
  CSK_CUDA(L, cudaGetLastError());
  L->last_stream = s;
  return CSK_OK;
}

// Stage 2 (after the all-gather of the counts): rows to the ranks that own their slots.
int csk_moe_ep_p2p_scatter_dev(csk_moe_layer* L, const float* d_hidden, int64_t T, const int32_t* d_all_counts,
                               void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!d_hidden || !d_all_counts) return fail(L, CSK_ERR_INVALID, "null argument");
  if (L->p2p_world <= 0) return fail(L, CSK_ERR_INVALID, "p2p: peers were never imported");
  if (T != L->last_T) return fail(L, CSK_ERR_INVALID, "p2p: scatter must follow counts of the same batch");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = pick(L, stream);
  const int n_pairs = (int)(T * L->k);
  const float* router = L->has_slot_map ? L->d_router_phys : L->d_router;
  k_ep_p2p_base<<<1, 1024, 0, s>>>(d_all_counts, L->p2p_world, L->p2p_rank, L->E, L->Eloc, (int)L->max_rows,
                                   L->d_p2p_base, L->d_cursor, L->d_meta);
  k_ep_p2p_scatter<<<grid_for(n_pairs, 8, 8 * L->sm_count), 256, 0, s>>>(
      router, d_hidden, n_pairs, L->k, L->H, L->E, L->Eloc, L->p2p_rank, L->d_p2p_base, L->d_cursor, L->d_peer_x16,
      L->d_peer_info, L->ldx, (int)L->max_rows, L->cfg.weight_before_ffn, L->d_row_of_pair, L->d_meta);
  CSK_CUDA(L, cudaGetLastError());
  return CSK_OK;
}

// Stage 3 (after a barrier: every rank's rows have landed): the resident experts over the
// received rows; output rows go straight to their owners' return buffers.
int csk_moe_ep_p2p_experts_dev(csk_moe_layer* L, const int32_t* d_all_counts, int64_t rows_hint, void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!d_all_counts) return fail(L, CSK_ERR_INVALID, "null argument");
  if (L->p2p_world <= 0) return fail(L, CSK_ERR_INVALID, "p2p: peers were never imported");
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = pick(L, stream);
  rows_hint = std::max<int64_t>(1, std::min<int64_t>(rows_hint, L->max_rows));
  const int path = choose_path(L, rows_hint);
  const int tile_rows = tile_rows_for(L, path, rows_hint);
  // the status word of the dispatch stays; the tile list is rebuilt from the received counts
  k_ep_p2p_local_counts<<<(L->E + 255) / 256, 256, 0, s>>>(d_all_counts, L->p2p_world, L->E, L->e0, L->Eloc, L->d_counts);
  k_scan<<<1, 1024, 0, s>>>(L->d_counts, L->E, L->e0, L->Eloc, tile_rows, (int)L->max_rows, L->max_tiles,
                            L->d_resident, L->d_offsets, L->d_cursor, L->d_tiles, L->d_meta, nullptr, 0, -1, nullptr, nullptr);
  k_ep_p2p_rowptr<<<4 * L->sm_count, 256, 0, s>>>(L->d_info, L->d_meta, L->d_peer_back, L->H, L->d_row_ptr,
                                                  (int)L->max_rows, L->p2p_world, (int)L->max_rows);
  CSK_CUDA(L, cudaGetLastError());
  StageTimer tm(L, s);
  tm.mark();
  int rc;
  if (path == CSK_PATH_TILE) {
    rc = launch_experts(L, path, tile_rows, rows_hint, rows_hint, L->d_x16, nullptr, L->H, nullptr, s, tm, L->d_row_ptr);
  } else {
    rc = launch_experts(L, path, tile_rows, rows_hint, rows_hint, L->d_x16, L->d_y, L->H, nullptr, s, tm);
    if (!rc) {
      k_ep_p2p_return<<<8 * L->sm_count, 256, 0, s>>>(L->d_y, L->H, L->d_row_ptr, L->d_meta, (int)L->max_rows);
      CSK_CUDA(L, cudaGetLastError());
    }
  }
  if (rc) return rc;
  return ep_finish(L, s, tm.n);
}

// Stage 4 (after a second barrier: every output row of this rank's pairs has landed).
int csk_moe_ep_p2p_combine_dev(csk_moe_layer* L, int64_t T, float* d_out, float* d_router_out, void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (L->p2p_world <= 0) return fail(L, CSK_ERR_INVALID, "p2p: peers were never imported");
  return csk_moe_ep_combine_dev(L, L->d_back, T, d_out, d_router_out, stream);
}

int csk_moe_ep_experts_dev(csk_moe_layer* L, const void* d_recv_f16, const int32_t* d_recv_counts,
                           int32_t n_src, int64_t total_rows, float* d_ret, void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!d_recv_f16 || !d_recv_counts || !d_ret) return fail(L, CSK_ERR_INVALID, "null argument");
  if (n_src <= 0 || (int64_t)n_src * L->Eloc > 1024)
    return fail(L, CSK_ERR_INVALID, "n_src * local experts must be in [1,1024]");
  if (total_rows < 0 || total_rows > L->max_rows)
    return fail(L, CSK_ERR_NOMEM, "%lld received rows exceed max_tokens*top_k = %lld",
                (long long)total_rows, (long long)L->max_rows);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = pick(L, stream);
  if (total_rows == 0) return CSK_OK;
  const int path = choose_path(L, total_rows);
  const int tile_rows = tile_rows_for(L, path, total_rows);
  CSK_CUDA(L, cudaMemsetAsync(L->d_meta, 0, sizeof(int) * 8, s));
  CSK_CUDA(L, cudaMemsetAsync(L->d_counts, 0, sizeof(int) * L->E, s));
  k_ep_plan<<<1, 1024, 0, s>>>(d_recv_counts, n_src, L->Eloc, L->e0, L->d_counts, L->d_seg);
  k_scan<<<1, 1024, 0, s>>>(L->d_counts, L->E, L->e0, L->Eloc, tile_rows, (int)L->max_rows, L->max_tiles,
                            L->d_resident, L->d_offsets, L->d_cursor, L->d_tiles, L->d_meta, nullptr, 0, -1, nullptr, nullptr);
  k_ep_regroup<<<dim3((unsigned)(n_src * L->Eloc), (unsigned)std::max(1, 16 * L->sm_count / (n_src * L->Eloc))), 128, 0, s>>>((const __half*)d_recv_f16, L->d_x16, L->ldx, L->d_seg,
                                               L->d_offsets, n_src, L->Eloc, L->e0, L->d_out_row_map);
  CSK_CUDA(L, cudaGetLastError());
  StageTimer tm(L, s);
  tm.mark();
  int rc;
  if (path == CSK_PATH_TILE) {
    rc = launch_experts(L, path, tile_rows, total_rows, total_rows, L->d_x16, d_ret, L->H, L->d_out_row_map, s, tm);
  } else {
    rc = launch_experts(L, path, tile_rows, total_rows, total_rows, L->d_x16, L->d_y, L->H, nullptr, s, tm);
    if (!rc) {
      k_ep_ungroup<<<grid_for((size_t)total_rows, 8, 8 * L->sm_count), 256, 0, s>>>(
          L->d_y, d_ret, L->H, L->d_out_row_map, (int)total_rows);
      CSK_CUDA(L, cudaGetLastError());
    }
  }
  if (rc) return rc;
  return ep_finish(L, s, tm.n);
}

int csk_moe_ep_combine_dev(csk_moe_layer* L, const float* d_back, int64_t T, float* d_out,
                           float* d_router_out, void* stream) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  if (!d_back || !d_out) return fail(L, CSK_ERR_INVALID, "null argument");
  if (T != L->last_T) return fail(L, CSK_ERR_INVALID, "combine T=%lld does not match dispatch T=%lld",
                                  (long long)T, (long long)L->last_T);
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  cudaStream_t s = pick(L, stream);
  k_combine<<<(unsigned)T, 256, 0, s>>>(L->d_router, L->d_row_of_pair, d_back, L->H, d_out, (int)T, L->k,
                                        L->H, L->cfg.weight_before_ffn, 0, nullptr, nullptr, nullptr, 0);
  CSK_CUDA(L, cudaGetLastError());
  if (d_router_out)
    CSK_CUDA(L, cudaMemcpyAsync(d_router_out, L->d_router, sizeof(float) * T * L->k * 2,
                                cudaMemcpyDeviceToDevice, s));
  return CSK_OK;
}

// ---- routing without any allocation ---------------------------------------------
// Scratch for csk_moe_route_static: the [T,E] logits between its two kernels.
// File-scope device memory, so every GPU that loads this library carries these
// 1 MiB until the process exits.  In host code `g_static_logits` is only a
// stand-in for the symbol; the device address comes from cudaGetSymbolAddress.
constexpr int64_t kStaticLogitsMax = 256 * 1024;  // floats: T * E may not exceed this
static __device__ __align__(256) float g_static_logits[kStaticLogitsMax];
// Status word of the same entry point (kDevErr* bits or-ed by its kernels), read and cleared by
// csk_moe_route_static_status.
static __device__ int g_static_status;

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
float* g_static_logits_addr[kMaxDevices] = {nullptr};
int* g_static_status_addr[kMaxDevices] = {nullptr};
}  // namespace

int csk_moe_route_static(const float* d_hidden, int64_t T, int32_t H, const float* d_gate_w,
                         const float* d_gate_bias, int32_t E, int32_t k, int32_t sigmoid_gating,
                         float* d_router_out, void* stream) {
  if (!d_hidden || !d_gate_w || !d_router_out) return fail(nullptr, CSK_ERR_INVALID, "route_static: null argument");
  if (T <= 0 || H <= 0 || H % 32 || E <= 0 || E > 1024 || k <= 0 || k > kMaxTopK || k > E)
    return fail(nullptr, CSK_ERR_INVALID,
                "route_static: need T > 0, H a positive multiple of 32, 1 <= E <= 1024, 1 <= k <= min(E, %d); "
                "got T=%lld H=%d E=%d k=%d", kMaxTopK, (long long)T, H, E, k);
  if (T * (int64_t)E > kStaticLogitsMax)
    return fail(nullptr, CSK_ERR_NOMEM,
                "route_static: T*E = %lld exceeds the built-in scratch of %lld logits; split the batch or use "
                "csk_moe_route_dev on a handle", (long long)(T * (int64_t)E), (long long)kStaticLogitsMax);
  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return fail(nullptr, CSK_ERR_CUDA, "route_static: cudaGetDevice: %s", cudaGetErrorString(ce));
  if (dev < 0 || dev >= kMaxDevices) return fail(nullptr, CSK_ERR_INVALID, "route_static: device ordinal %d not supported", dev);
  float* logits = nullptr;
  {
    // once per device, with that device current: resolve the symbol to its address there
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_logits_addr[dev]) {
      void* p = nullptr;
      ce = cudaGetSymbolAddress(&p, g_static_logits);
      if (ce != cudaSuccess || !p)
        return fail(nullptr, CSK_ERR_CUDA, "route_static: cudaGetSymbolAddress: %s", cudaGetErrorString(ce));
      void* ps = nullptr;
      ce = cudaGetSymbolAddress(&ps, g_static_status);
      if (ce != cudaSuccess || !ps)
        return fail(nullptr, CSK_ERR_CUDA, "route_static: cudaGetSymbolAddress: %s", cudaGetErrorString(ce));
      ce = router_prepare_device();
      if (ce != cudaSuccess)
        return fail(nullptr, CSK_ERR_CUDA, "route_static: cudaFuncSetAttribute: %s", cudaGetErrorString(ce));
      g_static_status_addr[dev] = static_cast<int*>(ps);
      g_static_logits_addr[dev] = static_cast<float*>(p);
    }
    logits = g_static_logits_addr[dev];
  }
  cudaStream_t s = (cudaStream_t)stream;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (reinterpret_cast<uintptr_t>(d_hidden) % 16 || reinterpret_cast<uintptr_t>(d_gate_w) % 16)
    return fail(nullptr, CSK_ERR_INVALID, "route_static: hidden states and gate weights must be 16-byte aligned");
  RouterArgs a{};
  a.hidden = d_hidden;
  a.bias = d_gate_bias;
  a.logits = logits;
  a.status = g_static_status_addr[dev];
  a.T = (int)T;
  a.H = H;
  a.E = E;
  launch_router_logits<false>(a, d_gate_w, d_gate_w, sms, s);
  k_router_topk<<<(unsigned)((T + 3) / 4), 128, 0, s>>>(logits, d_router_out, (int)T, E, k, sigmoid_gating);
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(nullptr, CSK_ERR_CUDA, "route_static: launch failed: %s", cudaGetErrorString(ce));
  return CSK_OK;
}

int csk_moe_route_static_status(void) {
  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return fail(nullptr, CSK_ERR_CUDA, "route_static_status: cudaGetDevice: %s", cudaGetErrorString(ce));
  int* addr = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (dev >= 0 && dev < kMaxDevices) addr = g_static_status_addr[dev];
  }
  if (!addr) return CSK_OK;  // csk_moe_route_static never ran on this device
  int st = 0;
  ce = cudaMemcpy(&st, addr, sizeof(int), cudaMemcpyDeviceToHost);
  if (ce != cudaSuccess) return fail(nullptr, CSK_ERR_CUDA, "route_static_status: %s", cudaGetErrorString(ce));
  if (!st) return CSK_OK;
  ce = cudaMemset(addr, 0, sizeof(int));
  if (ce != cudaSuccess) return fail(nullptr, CSK_ERR_CUDA, "route_static_status: %s", cudaGetErrorString(ce));
  return fail(nullptr, CSK_ERR_DEVICE, "route_static: a bounded device-side wait ran out; the routing output of that call is not valid");
}

// ---- test hooks ---------------------------------------------------------------------
int csk_moe_debug_set(csk_moe_layer* L, int32_t key, int64_t value) {
  if (check_layer(L)) return CSK_ERR_INVALID;
  CSK_CUDA(L, cudaSetDevice(L->cfg.device));
  if (key == CSK_DEBUG_WAIT_BUDGET) {
    if (value < 1000) return fail(L, CSK_ERR_INVALID, "debug: the wait budget must be at least 1000 cycles");
    const long long v = value;
    CSK_CUDA(L, cudaStreamSynchronize(L->stream));
    CSK_CUDA(L, cudaMemcpyToSymbol(g_wait_budget, &v, sizeof(v)));
    return CSK_OK;
  }
  if (key == CSK_DEBUG_STALL_TILE_PRODUCER) {
    L->debug_stall = value != 0;
    return CSK_OK;
  }
  return fail(L, CSK_ERR_INVALID, "debug: unknown key %d", key);
}

}  // extern "C"
