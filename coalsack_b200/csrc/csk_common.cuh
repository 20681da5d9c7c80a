// Shared definitions of the MoE library: the repacked MXFP4 device layout, the
// dequantisation helpers and the handle.  sm_100a only.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "csk_moe.h"

namespace csk {

// ---------------------------------------------------------------------------
// Device layout of one repacked MXFP4 matrix W[N, K] (K = contraction dim) for
// the streaming kernel.
//
// The rows are cut into groups of 16; a group is stored as one contiguous run
// of records along K: [group][k_tile][record], a record being 16 rows x 64
// columns in 544 bytes:
//
//   bytes   0..511  codes, lane-major for a warp: lane l = 4*g + q owns 16 bytes
//                   = four 32-bit words
//                     word 0: row g,   columns 32*0 + 8q .. +7
//                     word 1: row g,   columns 32*1 + 8q .. +7
//                     word 2: row g+8, columns 32*0 + 8q .. +7
//                     word 3: row g+8, columns 32*1 + 8q .. +7
//                   nibble i of a word (bits 4i..4i+3) is the E2M1 code of
//                   column 8q + i, i.e. the codes are in natural column order.
//   bytes 512..543  E8M0 scales: for g = 0..7 four bytes
//                     (row g blk 0, row g blk 1, row g+8 blk 0, row g+8 blk 1)
//
// One warp reads a record with a single 128-bit load per lane (plus one 32-bit
// scale load).  For the fused gate/up matrix a group is 16 FEATURES and every
// k-tile has two records, gate then up, so one warp sees both operands of the
// gated activation.  Rows >= N and columns >= K are padded with zero codes.
// ---------------------------------------------------------------------------
constexpr int kSubBytes = 544;
constexpr int kSubCodeBytes = 512;
constexpr int kTileK = 64;

struct MatLayout {
  int N;        // logical rows (for gate/up: F features, stored as 2 x F rows)
  int K;        // logical columns
  int paired;   // 1 = fused gate/up
  int groups;   // 16-row groups
  int k_tiles;  // 64-column tiles along K
  __host__ __device__ int recs() const { return paired ? 2 : 1; }
  __host__ __device__ size_t group_bytes() const { return (size_t)k_tiles * recs() * kSubBytes; }
  __host__ __device__ size_t bytes() const { return (size_t)groups * group_bytes(); }
  __host__ __device__ int k_pad() const { return k_tiles * kTileK; }
};

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

inline MatLayout make_layout(int N, int K, bool paired) {
  MatLayout L{};
  L.N = N;
  L.K = K;
  L.paired = paired ? 1 : 0;
  L.groups = ceil_div(N, 16);
  L.k_tiles = ceil_div(K, kTileK);
  return L;
}

// Two packed E2M1 codes (one byte) -> half2, low nibble in the low half.
__device__ __forceinline__ uint32_t e2m1x2_to_h2(uint32_t byte) {
  uint32_t r;
  asm("{\n\t.reg .b8 b;\n\tcvt.u8.u32 b, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}" : "=r"(r) : "r"(byte));
  return r;
}

// A word of eight codes -> four half2 (columns 0-1, 2-3, 4-5, 6-7).
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}

// The same activations with the hardware's approximate exp2 and reciprocal (one MUFU
// operation each, relative error around 2^-22, far below the fp16 rounding of the stored
// result).  Used in the tensor-core kernel's epilogue, which sits on the critical path.
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float gated_act_fast(float gate, float up, int act) {
  constexpr float kLog2e = 1.4426950408889634f;
  if (act == CSK_ACT_MODIFIED_SWIGLU) {
    const float lim = 7.0f, alpha = 1.702f;
    const float g = fminf(gate, lim);
    const float u = fminf(fmaxf(up, -lim), lim);
    return g * rcp_approx(1.0f + ex2_approx(-alpha * kLog2e * g)) * (u + 1.0f);
  }
  return gate * rcp_approx(1.0f + ex2_approx(-kLog2e * gate)) * up;
}

// Gated activations of the reference (expert_mlp_node.h:657-658, 699-707).
__device__ __forceinline__ float gated_act(float gate, float up, int act) {
  if (act == CSK_ACT_MODIFIED_SWIGLU) {
    const float lim = 7.0f, alpha = 1.702f;
    float g = fminf(gate, lim);
    float u = fminf(fmaxf(up, -lim), lim);
    float glu = g / (1.0f + expf(alpha * (-g)));
    return glu * (u + 1.0f);
  }
  float silu = gate / (1.0f + expf(-gate));
  return silu * up;
}

// ---- mbarrier and bulk-copy helpers shared by the two expert kernels -----------
// Clock cycles before a bounded wait gives up (about one second at full clock).  A device
// variable rather than a constant so that a test can shorten it and watch a wait run out
// without hanging anything (csk_moe_debug_set, key 0).  Read only on the slow path of a wait.
__device__ long long g_wait_budget = 2000000000LL;
__device__ __forceinline__ long long wait_budget() { return *(volatile long long*)&g_wait_budget; }
// Waits for copies or MMAs that are already in flight (teardown after a wait ran out) keep a
// floor of a few milliseconds however short the budget was made: what is in flight must land.
__device__ __forceinline__ long long drain_budget() { return wait_budget() + 8000000LL; }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
    for (int i = 0; i < 32; ++i)
      if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > wait_budget()) {
      *abort_flag = 1;
      return false;
    }
  }
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}


// Programmatic dependent launch: a kernel launched with `pdl` may become resident while
// the kernel before it in the stream is still running.  Every kernel of the layer therefore
// calls griddep_wait() before it touches global memory that an earlier kernel may still be
// writing or reading (a no-op for an ordinary launch), and griddep_launch() to let its own
// successor start early.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... P, typename... A>
inline cudaError_t launch_k(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl,
                            A&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, P(std::forward<A>(args))...);
}

// Work item lists built on the device by the permutation step.
struct RowTile {
  int expert;  // expert index local to this device
  int row0;    // first row of the tile in the grouped activation buffer
  int rows;    // rows in the tile (1 .. tile height)
  int pad;
};

// Device-side status word values (or-ed).
enum : int {
  kDevErrExpertRange = 1,   // router output names an expert outside [0, E)
  kDevErrCapacity = 2,      // more rows than the scratch buffers hold
  kDevErrWaitTimeout = 4,   // a bounded wait in a kernel ran out
  kDevErrNotResident = 8,   // rows were routed to an expert that is not loaded
  kDevErrPeerRow = 16,      // a row received from a peer carries no valid origin record
};

}  // namespace csk
