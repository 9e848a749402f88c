// Residual add + LayerNorm in one pass over fp16 rows (the glue between the packed linears of a block):
//   s = fp16(x + y)   (written out when y is given: the updated residual stream)
//   h = fp16((s - mean(s)) * rsqrt(var(s) + eps) * gamma + beta)
// One warp per row, 16-byte loads/stores, statistics in fp32 with a two-pass (mean, then centred sum of
// squares) over values held in registers.  HBM-bound: reads x (and y), writes h (and s) once.
#pragma once
#include <cuda_fp16.h>
#include "ptx.cuh"

namespace arcq {

constexpr int kLnMaxChunks = 8;  // 16-byte chunks per lane: rows up to 32 * 8 * 8 = 2048 values

__global__ void __launch_bounds__(256) add_layernorm_kernel(const __half* __restrict__ x, const __half* __restrict__ y,
                                                            const float* __restrict__ gamma,
                                                            const float* __restrict__ beta, float eps, long long M, int K,
                                                            __half* __restrict__ sum_out, __half* __restrict__ h_out) {
  pdl_launch_dependents();   // the next kernel of the stream may start its set-up
  pdl_wait();                // the input may be the previous kernel's output

  const int lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const int chunks = K >> 3;
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < M; row += warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * K);
    const uint4* yr = (y != nullptr) ? reinterpret_cast<const uint4*>(y + row * K) : nullptr;
    float v[kLnMaxChunks][8];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kLnMaxChunks; ++i) {
      const int c = lane + 32 * i;
      if (c < chunks) {
        const uint4 a = __ldg(xr + c);
        const __half2* ah = reinterpret_cast<const __half2*>(&a);
        if (yr != nullptr) {
          const uint4 b = __ldg(yr + c);
          const __half2* bh = reinterpret_cast<const __half2*>(&b);
          uint4 so;
          __half2* sh = reinterpret_cast<__half2*>(&so);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 fa = __half22float2(ah[j]), fb = __half22float2(bh[j]);
            sh[j] = __floats2half2_rn(fa.x + fb.x, fa.y + fb.y);   // the fp16 sum a separate add would store
            const float2 fs = __half22float2(sh[j]);
            v[i][2 * j] = fs.x;
            v[i][2 * j + 1] = fs.y;
          }
          if (sum_out != nullptr) reinterpret_cast<uint4*>(sum_out + row * K)[c] = so;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 fa = __half22float2(ah[j]);
            v[i][2 * j] = fa.x;
            v[i][2 * j + 1] = fa.y;
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += v[i][j];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / static_cast<float>(K);
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < kLnMaxChunks; ++i) {
      if (lane + 32 * i < chunks) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[i][j] - mean;
          sq += d * d;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq / static_cast<float>(K) + eps);
#pragma unroll
    for (int i = 0; i < kLnMaxChunks; ++i) {
      const int c = lane + 32 * i;
      if (c < chunks) {
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c);
        const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c + 1);
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta) + 2 * c);
        const float4 b1 = __ldg(reinterpret_cast<const float4*>(beta) + 2 * c + 1);
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          oh[j] = __floats2half2_rn((v[i][2 * j] - mean) * rstd * gg[2 * j] + bb[2 * j],
                                    (v[i][2 * j + 1] - mean) * rstd * gg[2 * j + 1] + bb[2 * j + 1]);
        reinterpret_cast<uint4*>(h_out + row * K)[c] = o;
      }
    }
  }
}

// One row of LANES * 24 values (192 / 384 / 768: the DeiT widths) on LANES lanes, three 16-byte chunks per lane:
// s = fp16(x + y) (stored when asked), statistics in two passes, h = fp16((s - mean) * rstd * gamma + beta) returned
// as the lane's three packed chunks.  `rs` is the row to read (idle sub-warps shadow the last row), `row` the row
// to store (only if `valid`).  Shared by the LayerNorm kernel below and by the small-batch LayerNorm + quantizer
// kernel (ln_act_quant.cuh), so that the two produce the same bits.
// The lane's three chunks of row `rs` of x (and of y, if given).
template <int LANES>
__device__ __forceinline__ void layernorm_row_load(const __half* __restrict__ x, const __half* __restrict__ y,
                                                   long long rs, int l, uint4 (&a)[3], uint4 (&b)[3]) {
  constexpr int K = LANES * 24;
  const uint4* xr = reinterpret_cast<const uint4*>(x + rs * K);
#pragma unroll
  for (int i = 0; i < 3; ++i) a[i] = __ldg(xr + l + LANES * i);
  if (y != nullptr) {
    const uint4* yr = reinterpret_cast<const uint4*>(y + rs * K);
#pragma unroll
    for (int i = 0; i < 3; ++i) b[i] = __ldg(yr + l + LANES * i);
  }
}

// The arithmetic of one row on chunks already loaded (`has_y`: b holds the residual branch).
template <int LANES>
__device__ __forceinline__ void layernorm_row_compute(const uint4 (&a)[3], const uint4 (&b)[3], bool has_y,
                                                      long long row, bool valid, int l, const float (&gg)[3][8],
                                                      const float (&bb)[3][8], float eps,
                                                      __half* __restrict__ sum_out, uint4 (&h)[3]) {
  constexpr int K = LANES * 24;
  const bool yr = has_y;
  float v[3][8];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const __half2* ah = reinterpret_cast<const __half2*>(&a[i]);
    if (yr) {
      const __half2* bh = reinterpret_cast<const __half2*>(&b[i]);
      uint4 so;
      __half2* sh = reinterpret_cast<__half2*>(&so);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = __half22float2(ah[j]), fb = __half22float2(bh[j]);
        sh[j] = __floats2half2_rn(fa.x + fb.x, fa.y + fb.y);   // the fp16 sum a separate add would store
        const float2 fs = __half22float2(sh[j]);
        v[i][2 * j] = fs.x;
        v[i][2 * j + 1] = fs.y;
      }
      if (valid && sum_out != nullptr) reinterpret_cast<uint4*>(sum_out + row * K)[l + LANES * i] = so;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = __half22float2(ah[j]);
        v[i][2 * j] = fa.x;
        v[i][2 * j + 1] = fa.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += v[i][j];
  }
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float mean = sum * (1.0f / static_cast<float>(K));
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float d = v[i][j] - mean;
      sq += d * d;
    }
  }
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  const float rstd = rsqrtf(sq * (1.0f / static_cast<float>(K)) + eps);
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    __half2* oh = reinterpret_cast<__half2*>(&h[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      oh[j] = __floats2half2_rn((v[i][2 * j] - mean) * rstd * gg[i][2 * j] + bb[i][2 * j],
                                (v[i][2 * j + 1] - mean) * rstd * gg[i][2 * j + 1] + bb[i][2 * j + 1]);
  }
}

template <int LANES>
__device__ __forceinline__ void layernorm_row(const __half* __restrict__ x, const __half* __restrict__ y, long long rs,
                                              long long row, bool valid, int l, const float (&gg)[3][8],
                                              const float (&bb)[3][8], float eps, __half* __restrict__ sum_out,
                                              uint4 (&h)[3]) {
  uint4 a[3], b[3];
  layernorm_row_load<LANES>(x, y, rs, l, a, b);
  layernorm_row_compute<LANES>(a, b, y != nullptr, row, valid, l, gg, bb, eps, sum_out, h);
}

// gamma and beta of the lane's three chunks
template <int LANES>
__device__ __forceinline__ void layernorm_lane_params(const float* __restrict__ gamma, const float* __restrict__ beta,
                                                      int l, float (&gg)[3][8], float (&bb)[3][8]) {
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const int c = l + LANES * i;
    const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c);
    const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c + 1);
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta) + 2 * c);
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(beta) + 2 * c + 1);
    gg[i][0] = g0.x; gg[i][1] = g0.y; gg[i][2] = g0.z; gg[i][3] = g0.w;
    gg[i][4] = g1.x; gg[i][5] = g1.y; gg[i][6] = g1.z; gg[i][7] = g1.w;
    bb[i][0] = b0.x; bb[i][1] = b0.y; bb[i][2] = b0.z; bb[i][3] = b0.w;
    bb[i][4] = b1.x; bb[i][5] = b1.y; bb[i][6] = b1.z; bb[i][7] = b1.w;
  }
}

// Residual add + LayerNorm for rows of LANES * 24 values: LANES lanes per row, so every lane carries the same load
// and a warp works on 32 / LANES rows at once; gamma and beta stay in registers for all the rows a lane visits.
template <int LANES>
__global__ void __launch_bounds__(256) add_layernorm_rows_kernel(const __half* __restrict__ x,
                                                                 const __half* __restrict__ y,
                                                                 const float* __restrict__ gamma,
                                                                 const float* __restrict__ beta, float eps,
                                                                 long long M, __half* __restrict__ sum_out,
                                                                 __half* __restrict__ h_out) {
  pdl_launch_dependents();   // the next kernel of the stream may start its set-up

  constexpr int K = LANES * 24, kRowsPerWarp = 32 / LANES;
  const int lane = threadIdx.x & 31, l = lane % LANES, sub = lane / LANES;
  float gg[3][8], bb[3][8];
  layernorm_lane_params<LANES>(gamma, beta, l, gg, bb);
  pdl_wait();                // gamma and beta are the layer's constants; x and y may be the previous kernel's output
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long first = (static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kRowsPerWarp;
  for (long long row0 = first; row0 < M; row0 += warps * kRowsPerWarp) {
    const long long row = row0 + sub;
    const bool valid = row < M;
    const long long rs = valid ? row : M - 1;          // idle sub-warps shadow the last row, store nothing
    uint4 h[3];
    layernorm_row<LANES>(x, y, rs, row, valid, l, gg, bb, eps, sum_out, h);
    if (valid) {
#pragma unroll
      for (int i = 0; i < 3; ++i) reinterpret_cast<uint4*>(h_out + row * K)[l + LANES * i] = h[i];
    }
  }
}

}  // namespace arcq
