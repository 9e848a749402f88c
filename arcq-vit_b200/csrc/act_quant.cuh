// Activation quantizer kernel (group size 64): packed codes + per-group mean / scale / code sum,
// and optionally the reconstruction.  HBM-bound: every input element is read once, every output
// byte written once.
//
// Bit-exactness contract.  Codes must equal the reference CPU quantizer's, which computes in fp32
// with torch's reduction order: the 64 values of a group are seen as 8 chunks of 8 lanes; chunk c
// is added lane-wise to accumulator c % 4, the four accumulators are then added 0+1, +2, +3, and
// the 8 lanes of the result are added one after the other.  The mapping below gives lane l of an
// 8-lane "octet" exactly the elements {8c + l}, so the lane-wise part is local arithmetic in the
// same order and the final 8-term sum is a sequential shuffle chain.  All arithmetic uses the
// round-to-nearest intrinsics so that nothing is contracted into fused multiply-adds, and division
// and square root are the IEEE ones.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include "ptx.cuh"

namespace arcq {

template <typename T> __device__ __forceinline__ float load_f32(const T* p);
template <> __device__ __forceinline__ float load_f32<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float load_f32<__half>(const __half* p) {
  return __half2float(__ldg(p));
}
template <> __device__ __forceinline__ float load_f32<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(__ldg(p));
}
template <typename T> __device__ __forceinline__ void store_from_f32(T* p, float v);
template <> __device__ __forceinline__ void store_from_f32<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_from_f32<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <> __device__ __forceinline__ void store_from_f32<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

// Optional element-wise op applied to the input before it is quantised (fused from the preceding layer).
// PRE = 1: exact GELU, 0.5*x*(1+erf(x/sqrt 2)) in fp32, then rounded to the input's element type -- the
// value a separate GELU kernel would have stored -- so the quantizer sees the same numbers as unfused.
template <typename T> __device__ __forceinline__ float round_to(float v);
template <> __device__ __forceinline__ float round_to<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <> __device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <typename T, int PRE> __device__ __forceinline__ float pre_op(float x) {
  if (PRE == 1) return round_to<T>(x * 0.5f * (1.0f + erff(x * 0.70710678118654752440f)));
  return x;
}

// Exact GELU, 0.5*x*(1+erf(x/sqrt 2)) in fp32, for code that all 32 lanes of a warp run together.
// erf(z) for |z| < 0.9277 is z*P(z*z) with a degree-7 least-squares fit on Chebyshev nodes (max error 1e-11
// before rounding); over every fp16 input in that range the GELU rounded to fp16 differs from the exactly
// rounded one for 3 inputs of 31 360 -- the library erff gives 2.  Larger arguments call erff, but only when
// some lane of the warp needs it: the branch is warp-uniform, so the common case (pre-activations of a few
// units at most) never executes the long path.  Each element's result depends on its own value only.
__device__ __forceinline__ float gelu_warp(float x) {
  const float z = x * 0.70710678118654752440f;
  const float s = z * z;
  float r = -1.0267135621688794e-05f;
  r = fmaf(r, s, 0.00011447568977018818f);
  r = fmaf(r, s, -0.0008505592122673988f);
  r = fmaf(r, s, 0.005222289357334375f);
  r = fmaf(r, s, -0.026865806430578232f);
  r = fmaf(r, s, 0.11283788084983826f);
  r = fmaf(r, s, -0.37612637877464294f);
  r = fmaf(r, s, 1.128379225730896f);
  float e = z * r;
  const bool big = !(fabsf(z) < 0.9277f);
  if (__any_sync(0xffffffffu, big)) {
    const float el = erff(z);
    e = big ? el : e;
  }
  return x * 0.5f * (1.0f + e);
}
// The same, rounded to the element type T: the value a separate GELU kernel would have stored.
template <typename T> __device__ __forceinline__ float gelu_rounded_warp(float x) { return round_to<T>(gelu_warp(x)); }

// Sum of the value held by the 8 lanes of an octet, lane 0 first, as a chain of fp32 additions.
__device__ __forceinline__ float octet_chain_sum(float p, int octet_base) {
  float s = __shfl_sync(0xffffffffu, p, octet_base);
#pragma unroll
  for (int i = 1; i < 8; ++i) s = __fadd_rn(s, __shfl_sync(0xffffffffu, p, octet_base + i));
  return s;
}

// In: lane l of an octet holds, in nibble c, the code of element 8c + l.
// Out: lane l holds, in nibble j, the code of element 8l + j (an 8x8 nibble transpose over lanes).
__device__ __forceinline__ uint32_t octet_transpose_nibbles(uint32_t w, int l) {
  uint32_t p = __shfl_xor_sync(0xffffffffu, w, 4);
  w = (l & 4) ? ((w & 0xFFFF0000u) | (p >> 16)) : ((w & 0x0000FFFFu) | (p << 16));
  p = __shfl_xor_sync(0xffffffffu, w, 2);
  w = (l & 2) ? ((w & 0xFF00FF00u) | ((p >> 8) & 0x00FF00FFu)) : ((w & 0x00FF00FFu) | ((p << 8) & 0xFF00FF00u));
  p = __shfl_xor_sync(0xffffffffu, w, 1);
  w = (l & 1) ? ((w & 0xF0F0F0F0u) | ((p >> 4) & 0x0F0F0F0Fu)) : ((w & 0x0F0F0F0Fu) | ((p << 4) & 0xF0F0F0F0u));
  return w;
}

// 8 nibbles (each holding a 3-bit code) -> 24 contiguous bits; (2-bit codes) -> 16 contiguous bits.
__device__ __forceinline__ uint32_t squeeze_nibbles_3(uint32_t w) {
  uint32_t t = (w & 0x07070707u) | ((w & 0x70707070u) >> 1);
  uint32_t u = (t & 0x003F003Fu) | ((t & 0x3F003F00u) >> 2);
  return (u & 0xFFFu) | ((u >> 4) & 0xFFF000u);
}
__device__ __forceinline__ uint32_t squeeze_nibbles_2(uint32_t w) {
  uint32_t t = (w & 0x03030303u) | ((w & 0x30303030u) >> 2);
  uint32_t u = (t & 0x000F000Fu) | ((t & 0x0F000F00u) >> 4);
  return (u & 0xFFu) | ((u >> 8) & 0xFF00u);
}

// One warp handles 4 consecutive groups per step (8 lanes per group).  Groups are numbered
// row-major over [M, K/64]; with K a multiple of 64 the input, the packed output and the statistics
// are all contiguous in that numbering.
template <typename T, int BITS, typename XH, bool WRITE_XHAT, int PRE = 0>
__global__ void __launch_bounds__(256) act_quant_kernel(const T* __restrict__ x, long long total_groups,
                                                        const float* __restrict__ thresholds,
                                                        const float* __restrict__ codebook,
                                                        uint8_t* __restrict__ packed, float* __restrict__ mu_out,
                                                        float* __restrict__ sigma_out,
                                                        float* __restrict__ codesum_out, XH* __restrict__ xhat) {
  pdl_launch_dependents();   // the next kernel of the stream may start its set-up

  constexpr int L = 1 << BITS;
  __shared__ float s_th[16];
  __shared__ float s_cb[16];
  if (threadIdx.x < 16) {
    const int t = threadIdx.x;
    s_th[t] = (t < L - 1) ? thresholds[t] : __int_as_float(0x7f800000);
    s_cb[t] = (t < L) ? codebook[t] : 0.0f;
  }
  __syncthreads();
  pdl_wait();                // the tables above are the layer's constants; x may be the previous kernel's output

  const int lane = threadIdx.x & 31;
  const int l = lane & 7;
  const int octet_base = lane & ~7;
  const long long warps_total = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long tasks = (total_groups + 3) >> 2;

  for (long long task = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); task < tasks;
       task += warps_total) {
    const long long gi = task * 4 + (lane >> 3);
    const bool valid = gi < total_groups;
    const long long gs = valid ? gi : total_groups - 1;  // idle octets shadow the last group, store nothing
    const T* xg = x + gs * 64 + l;

    float v[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = pre_op<T, PRE>(load_f32<T>(xg + 8 * c));

    // mean
    float a0 = __fadd_rn(v[0], v[4]), a1 = __fadd_rn(v[1], v[5]);
    float a2 = __fadd_rn(v[2], v[6]), a3 = __fadd_rn(v[3], v[7]);
    float part = __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3);
    const float mean = __fdiv_rn(octet_chain_sum(part, octet_base), 64.0f);

    // scale = sqrt(mean(r^2) + 1e-6)
    float r[8], q[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      r[c] = __fsub_rn(v[c], mean);
      q[c] = __fmul_rn(r[c], r[c]);
    }
    a0 = __fadd_rn(q[0], q[4]); a1 = __fadd_rn(q[1], q[5]);
    a2 = __fadd_rn(q[2], q[6]); a3 = __fadd_rn(q[3], q[7]);
    part = __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3);
    const float var = __fdiv_rn(octet_chain_sum(part, octet_base), 64.0f);
    const float scale = __fsqrt_rn(__fadd_rn(var, 1.0e-6f));

    // codes: number of thresholds strictly below t (binary search in the sorted table)
    uint32_t w = 0;
    float cv[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float t = __fdiv_rn(r[c], scale);
      int code = 0;
      if (BITS >= 4) code = (t > s_th[7]) ? 8 : 0;
      if (BITS >= 3) code += (t > s_th[code + 3]) ? 4 : 0;
      code += (t > s_th[code + 1]) ? 2 : 0;
      code += (t > s_th[code]) ? 1 : 0;
      w |= static_cast<uint32_t>(code) << (4 * c);
      cv[c] = s_cb[code];
    }
    a0 = __fadd_rn(cv[0], cv[4]); a1 = __fadd_rn(cv[1], cv[5]);
    a2 = __fadd_rn(cv[2], cv[6]); a3 = __fadd_rn(cv[3], cv[7]);
    part = __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3);
    const float code_sum = octet_chain_sum(part, octet_base);

    if (WRITE_XHAT) {
      // mean + scale * (cb[c] - code_sum/64), each step rounded as the reference's fp32 tensor ops
      const float vm = __fdiv_rn(code_sum, 64.0f);
      if (valid) {
        XH* og = xhat + gi * 64 + l;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          store_from_f32<XH>(og + 8 * c, __fadd_rn(mean, __fmul_rn(scale, __fsub_rn(cv[c], vm))));
      }
    }

    if (packed != nullptr) {
      w = octet_transpose_nibbles(w, l);  // lane l now holds codes of elements 8l .. 8l+7
      if (BITS == 4) {
        if (valid) reinterpret_cast<uint32_t*>(packed)[gi * 8 + l] = w;
      } else if (BITS == 3) {
        const uint32_t v24 = squeeze_nibbles_3(w);
        // 8 lanes x 3 bytes -> 6 words; word j starts at byte 4j = chunk q, byte r of it
        const int q = (4 * l) / 3, rr = (4 * l) % 3;
        const uint32_t lo = __shfl_sync(0xffffffffu, v24, octet_base + (q & 7));
        const uint32_t hi = __shfl_sync(0xffffffffu, v24, octet_base + ((q + 1) & 7));
        const uint32_t word = (lo >> (8 * rr)) | (hi << (24 - 8 * rr));
        if (valid && l < 6) reinterpret_cast<uint32_t*>(packed)[gi * 6 + l] = word;
      } else {
        const uint32_t v16 = squeeze_nibbles_2(w);
        const uint32_t lo = __shfl_sync(0xffffffffu, v16, octet_base + ((2 * l) & 7));
        const uint32_t hi = __shfl_sync(0xffffffffu, v16, octet_base + ((2 * l + 1) & 7));
        if (valid && l < 4) reinterpret_cast<uint32_t*>(packed)[gi * 4 + l] = lo | (hi << 16);
      }
    }
    if (valid && mu_out != nullptr) {
      if (l == 0) mu_out[gi] = mean;
      if (l == 1) sigma_out[gi] = scale;
      if (l == 2 && codesum_out != nullptr) codesum_out[gi] = code_sum;
    }
  }
}

}  // namespace arcq
