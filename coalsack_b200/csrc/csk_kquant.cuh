// Q4_K and Q6_K super-blocks (256 values; 144 and 210 bytes) to fp16, the conversion the reference's weight
// provider does on the host for every expert slice it fetches (src/llm/moe_weight_provider.cpp:17-33, 134-159,
// decoders include/coalsack/gguf/gguf_dequant.h:147-207, 220-261, fp32 -> fp16 :458-489).  Here the raw blocks
// are copied to the device and decoded there, bit for bit: the same fp32 products and differences, each
// rounded once (no fused multiply-add), then the reference's fp32 -> fp16 step.
//
// That step has two builds in the reference: the portable one (its CMake flags: no -march) TRUNCATES the
// mantissa, sends NaN to infinity and values under 2^-25 to zero; an F16C build rounds to nearest even.
// `NEAREST` selects the second.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace csk {

constexpr int kQkK = 256;        // values per super-block
constexpr int kQ4kBytes = 144;   // fp16 d, fp16 dmin, 12 scale bytes, 128 nibble bytes
constexpr int kQ6kBytes = 210;   // 128 low-nibble bytes, 64 high-bit bytes, 16 int8 scales, fp16 d

// Headers may hold any bit pattern.  The host code the result is compared with keeps the SIGN of a NaN
// through its arithmetic (an operand that is a NaN comes back with its sign; a NaN made by inf * 0 or
// inf - inf is the negative default NaN), and the truncating fp32 -> fp16 step turns a NaN into the
// infinity of that sign.  The GPU's arithmetic returns one canonical NaN, so the sign is carried here.
__device__ __forceinline__ float kq_nan_like(float a) {
  return __uint_as_float((__float_as_uint(a) & 0x80000000u) | 0x7FC00000u);
}
__device__ __forceinline__ float kq_half_bits_to_float(const uint8_t* p) {
  const uint32_t h = p[0] | (static_cast<uint32_t>(p[1]) << 8);
  if ((h & 0x7C00u) == 0x7C00u && (h & 0x3FFu)) return __uint_as_float(((h & 0x8000u) << 16) | 0x7FC00000u);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}
__device__ __forceinline__ float kq_mul(float a, float b) {
  const float r = __fmul_rn(a, b);
  if (r == r) return r;
  if (a != a) return kq_nan_like(a);
  if (b != b) return kq_nan_like(b);
  return __uint_as_float(0xFFC00000u);
}
__device__ __forceinline__ float kq_sub(float a, float b) {
  const float r = __fsub_rn(a, b);
  if (r == r) return r;
  if (a != a) return kq_nan_like(a);
  if (b != b) return kq_nan_like(b);
  return __uint_as_float(0xFFC00000u);
}

// gguf_dequant.h:458-489, the branch without F16C
__device__ __forceinline__ unsigned short kq_f32_to_f16_truncating(float f) {
  const uint32_t bits = __float_as_uint(f);
  const uint32_t sign = (bits >> 16) & 0x8000u;
  const int32_t exponent = static_cast<int32_t>((bits >> 23) & 0xFF) - 127 + 15;
  uint32_t mantissa = (bits >> 13) & 0x3FFu;
  if (exponent <= 0) {
    if (exponent < -10) return static_cast<unsigned short>(sign);
    mantissa |= 0x400u;
    mantissa >>= (1 - exponent);
    return static_cast<unsigned short>(sign | mantissa);
  }
  if (exponent >= 31) return static_cast<unsigned short>(sign | 0x7C00u);
  return static_cast<unsigned short>(sign | (static_cast<uint32_t>(exponent) << 10) | mantissa);
}

template <bool NEAREST>
__device__ __forceinline__ unsigned short kq_to_f16(float f) {
  if (NEAREST) return __half_as_ushort(__float2half_rn(f));
  return kq_f32_to_f16_truncating(f);
}

// One warp per (super-block, pair of 32-value sub-blocks): lane l decodes byte l of the pair's 32 nibble
// bytes into value l of the first sub-block (low nibble) and of the second (high nibble).
template <bool NEAREST>
__global__ void __launch_bounds__(256) k_dequant_q4k(const uint8_t* __restrict__ src, unsigned short* __restrict__ dst,
                                                     int64_t nblocks) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < nblocks * 4; w += warps) {
    const int64_t b = w >> 2;
    const int pair = static_cast<int>(w & 3);
    const uint8_t* blk = src + b * kQ4kBytes;
    const float d = kq_half_bits_to_float(blk), dmin = kq_half_bits_to_float(blk + 2);
    const uint8_t* sc = blk + 4;
    uint32_t s1, m1, s2, m2;
    if (pair < 2) {  // sub-blocks 0..3: six bits of the first eight bytes
      s1 = sc[2 * pair] & 0x3F;
      m1 = sc[2 * pair + 4] & 0x3F;
      s2 = sc[2 * pair + 1] & 0x3F;
      m2 = sc[2 * pair + 5] & 0x3F;
    } else {         // sub-blocks 4..7: four bits of bytes 8..11 and the top two bits of bytes 0..7
      const int i1 = 2 * pair, i2 = 2 * pair + 1;
      s1 = (sc[i1 + 4] & 0x0F) | ((sc[i1 - 4] >> 6) << 4);
      m1 = (sc[i1 + 4] >> 4) | ((sc[i1] >> 6) << 4);
      s2 = (sc[i2 + 4] & 0x0F) | ((sc[i2 - 4] >> 6) << 4);
      m2 = (sc[i2 + 4] >> 4) | ((sc[i2] >> 6) << 4);
    }
    const float d1 = kq_mul(d, static_cast<float>(s1)), mm1 = kq_mul(dmin, static_cast<float>(m1));
    const float d2 = kq_mul(d, static_cast<float>(s2)), mm2 = kq_mul(dmin, static_cast<float>(m2));
    const uint32_t q = blk[16 + pair * 32 + lane];
    unsigned short* out = dst + b * kQkK + pair * 64;
    out[lane] = kq_to_f16<NEAREST>(kq_sub(kq_mul(d1, static_cast<float>(q & 0x0F)), mm1));
    out[32 + lane] = kq_to_f16<NEAREST>(kq_sub(kq_mul(d2, static_cast<float>(q >> 4)), mm2));
  }
}

// One warp per (super-block, half of 128 values): lane l decodes values l, l+32, l+64, l+96 of the half from
// two low-nibble bytes and one high-bit byte; value = (d * scale) * q, the products taken in that order.
template <bool NEAREST>
__global__ void __launch_bounds__(256) k_dequant_q6k(const uint8_t* __restrict__ src, unsigned short* __restrict__ dst,
                                                     int64_t nblocks) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < nblocks * 2; w += warps) {
    const int64_t b = w >> 1;
    const int half = static_cast<int>(w & 1);
    const uint8_t* blk = src + b * kQ6kBytes;
    const uint8_t* ql = blk + half * 64;
    const uint8_t* qh = blk + 128 + half * 32;
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192) + half * 8;
    const float d = kq_half_bits_to_float(blk + 208);
    const int is = lane >> 4;
    const uint32_t lo0 = ql[lane], lo1 = ql[lane + 32], hi = qh[lane];
    const int q1 = static_cast<int>((lo0 & 0xF) | (((hi >> 0) & 3) << 4)) - 32;
    const int q2 = static_cast<int>((lo1 & 0xF) | (((hi >> 2) & 3) << 4)) - 32;
    const int q3 = static_cast<int>((lo0 >> 4) | (((hi >> 4) & 3) << 4)) - 32;
    const int q4 = static_cast<int>((lo1 >> 4) | (((hi >> 6) & 3) << 4)) - 32;
    unsigned short* out = dst + b * kQkK + half * 128;
    out[lane] = kq_to_f16<NEAREST>(kq_mul(kq_mul(d, static_cast<float>(sc[is + 0])), static_cast<float>(q1)));
    out[lane + 32] = kq_to_f16<NEAREST>(kq_mul(kq_mul(d, static_cast<float>(sc[is + 2])), static_cast<float>(q2)));
    out[lane + 64] = kq_to_f16<NEAREST>(kq_mul(kq_mul(d, static_cast<float>(sc[is + 4])), static_cast<float>(q3)));
    out[lane + 96] = kq_to_f16<NEAREST>(kq_mul(kq_mul(d, static_cast<float>(sc[is + 6])), static_cast<float>(q4)));
  }
}

// fp32 weight matrices (the reference's dense FFN also takes FLOAT32 weights, dense_ffn_node.h:58-62, 121-149) to the
// fp16 operands of the tensor-core kernel, round to nearest even.  A finite weight beyond the fp16 range would
// become an infinity: counted in *overflow, and the load is refused.
__global__ void __launch_bounds__(256) k_f32_to_f16(const float* __restrict__ src, unsigned short* __restrict__ dst,
                                                    int64_t n, int* __restrict__ overflow) {
  int bad = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float f = src[i];
    const unsigned short h = __half_as_ushort(__float2half_rn(f));
    if ((h & 0x7FFFu) == 0x7C00u && fabsf(f) <= 3.0e38f) bad = 1;   // finite in, infinite out
    dst[i] = h;
  }
  if (bad) atomicAdd(overflow, 1);
}

}  // namespace csk
