// Bit-stream helpers and the small format kernels (unpack, pack, reconstruct).
// Layout: code j of a row occupies bits [j*bits, (j+1)*bits) of the row's little-endian bit stream.
#pragma once
#include <cuda_fp16.h>
#include "ptx.cuh"
#include "act_quant.cuh"

namespace arcq {

// Inverse of squeeze_nibbles_3/2: spread 8 packed codes into one nibble each.
__device__ __forceinline__ uint32_t spread_3_to_nibbles(uint32_t v24) {
  uint32_t u = (v24 & 0xFFFu) | ((v24 & 0xFFF000u) << 4);
  uint32_t t = (u & 0x003F003Fu) | ((u & 0x0FC00FC0u) << 2);
  return (t & 0x07070707u) | ((t & 0x38383838u) << 1);
}
__device__ __forceinline__ uint32_t spread_2_to_nibbles(uint32_t v16) {
  uint32_t u = (v16 & 0xFFu) | ((v16 & 0xFF00u) << 8);
  uint32_t t = (u & 0x000F000Fu) | ((u & 0x00F000F0u) << 4);
  return (t & 0x03030303u) | ((t & 0x0C0C0C0Cu) << 2);
}

// The 8 codes of chunk `chunk` (elements 8*chunk .. 8*chunk+7) of a packed row, one per nibble.
// Reads exactly the bytes that hold those codes, never past the row.
template <int BITS>
__device__ __forceinline__ uint32_t load_codes8(const uint8_t* __restrict__ row, int chunk) {
  if (BITS == 4) {
    return __ldg(reinterpret_cast<const uint32_t*>(row) + chunk);
  } else if (BITS == 3) {
    const uint8_t* p = row + 3 * chunk;
    const uint32_t v = static_cast<uint32_t>(__ldg(p)) | (static_cast<uint32_t>(__ldg(p + 1)) << 8) |
                       (static_cast<uint32_t>(__ldg(p + 2)) << 16);
    return spread_3_to_nibbles(v);
  } else {
    return spread_2_to_nibbles(__ldg(reinterpret_cast<const uint16_t*>(row) + chunk));
  }
}

__global__ void unpack_codes_kernel(const uint8_t* __restrict__ packed, long long rows, long long length,
                                    long long packed_cols, int bits, uint8_t* __restrict__ out) {
  const long long total = rows * length;
  const unsigned mask = (1u << bits) - 1u;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / length, j = i - r * length;
    const long long bit = j * bits;
    const uint8_t* p = packed + r * packed_cols + (bit >> 3);
    const int sh = static_cast<int>(bit & 7);
    unsigned v = static_cast<unsigned>(p[0]) >> sh;
    if (sh + bits > 8) v |= static_cast<unsigned>(p[1]) << (8 - sh);
    out[i] = static_cast<uint8_t>(v & mask);
  }
}

// One thread per output byte: gathers the (at most 5) codes that overlap it.
__global__ void pack_codes_kernel(const uint8_t* __restrict__ codes, long long rows, long long length,
                                  long long packed_cols, int bits, uint8_t* __restrict__ out) {
  const long long total = rows * packed_cols;
  const unsigned mask = (1u << bits) - 1u;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / packed_cols, b = i - r * packed_cols;
    const long long bit0 = b * 8;
    long long j = bit0 / bits;
    unsigned acc = 0;
    for (; j < length && j * bits < bit0 + 8; ++j) {
      const long long cb = j * bits;  // first bit of code j
      const unsigned c = static_cast<unsigned>(codes[r * length + j]) & mask;
      acc |= (cb >= bit0) ? (c << (cb - bit0)) : (c >> (bit0 - cb));
    }
    out[i] = static_cast<uint8_t>(acc & 0xffu);
  }
}

// out[r, k] = mu + sigma * (cb[c] - codesum/gs); one thread per chunk of 8 codes.
template <int BITS, typename OUT>
__global__ void dequant_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ mu,
                               const float* __restrict__ sigma, const float* __restrict__ codesum,
                               const float* __restrict__ codebook, long long rows, int K, int gs,
                               OUT* __restrict__ out) {
  __shared__ float s_cb[16];
  if (threadIdx.x < 16) s_cb[threadIdx.x] = (threadIdx.x < (1 << BITS)) ? codebook[threadIdx.x] : 0.0f;
  __syncthreads();
  const int chunks = K / 8;
  const int G = K / gs;
  const long long pc = static_cast<long long>(K) * BITS / 8;
  const long long total = rows * chunks;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / chunks;
    const int ch = static_cast<int>(i - r * chunks);
    const int g = (ch * 8) / gs;
    const uint32_t w = load_codes8<BITS>(packed + r * pc, ch);
    const float m = mu[r * G + g], s = sigma[r * G + g];
    const float vm = __fdiv_rn(codesum[r * G + g], static_cast<float>(gs));
    OUT* o = out + r * K + ch * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float v = __fadd_rn(m, __fmul_rn(s, __fsub_rn(s_cb[(w >> (4 * j)) & 15u], vm)));
      store_from_f32<OUT>(o + j, v);
    }
  }
}

// out[r, k] = fp16(mu' + sigma16 * cb16[c]) with mu' = fp16(mu - sigma*codesum/64), sigma16 = fp16(sigma),
// cb16 = fp16(cb[c]) and one half-precision fused multiply-add: bit for bit the weight the packed-weight
// GEMM kernels rebuild in shared memory, written out so that a dense GEMM can read it by TMA.
// One thread per chunk of 8 codes (16 bytes of output); groups of 64.
struct UnpackWeightJob {
  const uint8_t* packed;     // null: nothing to do
  const float* mu;
  const float* sigma;
  const float* codesum;
  const float* codebook;
  __half* out;
  long long rows;
  int K;
  int bits;
};

// Chunks first, first + stride, ... of the job; `s_cb` holds the 16 codebook values in fp16.  Four chunks per
// round, all their loads issued before the first result is used: a caller with few warps (the spare warps of a
// GEMM kernel) has nothing else to hide the load latency with.
template <int BITS>
__device__ __forceinline__ void unpack_weight_f16_chunks(const UnpackWeightJob& j, const __half* s_cb, long long first,
                                                         long long stride) {
  const int chunks = j.K / 8;
  const int G = j.K / 64;
  const long long pc = static_cast<long long>(j.K) * BITS / 8;
  const long long total = j.rows * chunks;
  constexpr int U = 4;
  for (long long i0 = first; i0 < total; i0 += U * stride) {
    uint32_t w[U];
    float sg[U], cs[U], mu[U];
    long long off[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      const bool in = i < total;
      const long long ii = in ? i : first;
      const long long r = ii / chunks;
      const int ch = static_cast<int>(ii - r * chunks);
      const long long sgi = r * G + (ch >> 3);
      w[u] = load_codes8<BITS>(j.packed + r * pc, ch);
      sg[u] = __ldg(j.sigma + sgi);
      cs[u] = __ldg(j.codesum + sgi);
      mu[u] = __ldg(j.mu + sgi);
      off[u] = in ? r * j.K + ch * 8 : -1;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (off[u] < 0) continue;
      const __half2 f2 = __floats2half2_rn(sg[u], fmaf(-sg[u], cs[u] * (1.0f / 64.0f), mu[u]));
      const __half2 s2 = __low2half2(f2), m2 = __high2half2(f2);
      uint32_t h[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const __half2 v2 = __halves2half2(s_cb[(w[u] >> (8 * q)) & 15u], s_cb[(w[u] >> (8 * q + 4)) & 15u]);
        const __half2 r2 = __hfma2(s2, v2, m2);
        h[q] = *reinterpret_cast<const uint32_t*>(&r2);
      }
      *reinterpret_cast<uint4*>(j.out + off[u]) = make_uint4(h[0], h[1], h[2], h[3]);
    }
  }
}

template <int BITS>
__global__ void unpack_weight_f16_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ mu,
                                         const float* __restrict__ sigma, const float* __restrict__ codesum,
                                         const float* __restrict__ codebook, long long rows, int K,
                                         __half* __restrict__ out) {
  __shared__ __half s_cb[16];
  if (threadIdx.x < 16) s_cb[threadIdx.x] = __float2half_rn((threadIdx.x < (1 << BITS)) ? codebook[threadIdx.x] : 0.0f);
  __syncthreads();
  const UnpackWeightJob j = {packed, mu, sigma, codesum, codebook, out, rows, K, BITS};
  unpack_weight_f16_chunks<BITS>(j, s_cb, blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x,
                                 static_cast<long long>(gridDim.x) * blockDim.x);
}

}  // namespace arcq
