// Activation quantizer, two lanes per 64-element group (16-bit element types).  Same staging, same exact
// arithmetic and the same first-guess classification as the one-thread-per-group kernel (act_quant_v2.cuh,
// which documents them); the difference is occupancy.  That kernel holds a whole group in one thread's
// registers (128 registers, 16 warps per SM) and is bound by the latency of its dependent chains.  Here a
// thread holds half a group -- the reference's summation lanes l = 4h .. 4h+3 of every 8-element chunk, i.e.
// 8 contiguous bytes per chunk -- so twice as many warps share an SM and every chain is half as long.
//   v[l] = ((x[l]+x[32+l]) + (x[8+l]+x[40+l])) + (x[16+l]+x[48+l])) + (x[24+l]+x[56+l])   stays in one thread;
//   sum  = ((((((v0+v1)+v2)+v3)+v4)+v5)+v6)+v7                                            crosses to the partner once.
// The two lanes of a group build its 15 limits together (8 + 7) in one column of the shared-memory table.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include "ptx.cuh"
#include "act_quant.cuh"
#include "act_quant_v2.cuh"

namespace arcq {

constexpr int kAq4Threads = 256;
constexpr int kAq4Groups = kAq4Threads / 2;   // groups per tile

template <typename T> __host__ __device__ constexpr size_t aq4_smem_bytes() {
  return 2 * kAq4Groups * Aq2Row<T>::kPitch + 2 * 16 * kAq4Groups * 4 + 4 * 16 * 4 + kAq2Cells * 4 + 16;
}

// four consecutive 16-bit values (8 bytes) -> floats
template <typename T> __device__ __forceinline__ void aq4_load4(const uint8_t* p, float* x);
template <> __device__ __forceinline__ void aq4_load4<__half>(const uint8_t* p, float* x) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}
template <> __device__ __forceinline__ void aq4_load4<__nv_bfloat16>(const uint8_t* p, float* x) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  x[0] = __uint_as_float(u.x << 16); x[1] = __uint_as_float(u.x & 0xFFFF0000u);
  x[2] = __uint_as_float(u.y << 16); x[3] = __uint_as_float(u.y & 0xFFFF0000u);
}

// Lane sums of this thread's 32 values, held as v[4c + e] = element 8c + 4h + e.
__device__ __forceinline__ void aq4_lane_sums(const float (&v)[32], float (&p)[4]) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float a0 = __fadd_rn(v[0 + e], v[16 + e]), a1 = __fadd_rn(v[4 + e], v[20 + e]);
    const float a2 = __fadd_rn(v[8 + e], v[24 + e]), a3 = __fadd_rn(v[12 + e], v[28 + e]);
    p[e] = __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3);
  }
}
// The 8-term chain over the two lanes of a group (h = 0 holds v0..v3, h = 1 holds v4..v7); both get the result.
__device__ __forceinline__ float aq4_group_chain(const float (&p)[4], int lane) {
  const float s0 = __fadd_rn(__fadd_rn(__fadd_rn(p[0], p[1]), p[2]), p[3]);        // meaningful in the h = 0 lane
  const float t = __shfl_sync(0xffffffffu, s0, lane & ~1);
  const float s1 = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(t, p[0]), p[1]), p[2]), p[3]);   // ... in the h = 1 lane
  return __shfl_sync(0xffffffffu, s1, lane | 1);
}

template <typename T, int BITS, bool WRITE_XHAT, int PRE = 0, bool WRITE_PACKED = true>
__global__ void __launch_bounds__(kAq4Threads, 4) act_quant_v4_kernel(const T* __restrict__ x, long long total_groups,
                                                                   const float* __restrict__ thresholds,
                                                                   const float* __restrict__ codebook,
                                                                   uint8_t* __restrict__ packed,
                                                                   float* __restrict__ mu_out,
                                                                   float* __restrict__ sigma_out,
                                                                   float* __restrict__ codesum_out,
                                                                   T* __restrict__ xhat) {
  pdl_launch_dependents();   // the next kernel of the stream may start its set-up

  static_assert(sizeof(T) == 2, "two-lane kernel is written for 16-bit element types");
  constexpr int L = 1 << BITS;
  constexpr int kPitch = Aq2Row<T>::kPitch, kRowBytes = Aq2Row<T>::kBytes;   // 144, 128
  constexpr int kChunksPerRow = kRowBytes / 16;                               // 8
  constexpr int kStride = kAq4Groups;                                         // floats between table entries of a group
  constexpr int kStep = kStride * 4;                                          // 512 bytes
  static_assert(kStep == 512, "code extraction below assumes a 512-byte table step");
  extern __shared__ __align__(16) uint8_t aq4_smem[];
  uint8_t* const s_stage = aq4_smem;                                                        // 2 x 128 rows
  float* const s_table = reinterpret_cast<float*>(aq4_smem + 2 * kAq4Groups * kPitch);      // [16][128] limits
  float* const s_cbt = s_table + 16 * kStride;                                              // [16][128] codebook
  float* const s_th = s_cbt + 16 * kStride;
  float* const s_h = s_th + 16;
  float* const s_cb = s_h + 16;
  float* const s_pos = s_cb + 16;
  int* const s_guess = reinterpret_cast<int*>(s_pos + 16);                                  // [kAq2Cells]
  const int tid = threadIdx.x, lane = tid & 31;
  const int gl = tid >> 1, h = tid & 1;

  int my_exact = 1;
  if (tid < 16) {
    float th = __int_as_float(0x7f800000), hg = 0.0f;
    if (tid < L - 1) {
      th = thresholds[tid];
      if (th == 0.0f) {
        hg = 0x1p-100f;
      } else {
        const int b = __float_as_int(th);
        const float up = __int_as_float(th > 0.0f ? b + 1 : b - 1);
        hg = __fmul_rn(__fsub_rn(up, th), 0.5f);
      }
      my_exact = (th == 0.0f || fabsf(th) > 1.0e-15f) ? 1 : 0;
    }
    s_th[tid] = th;
    s_h[tid] = hg;
    s_cb[tid] = tid < L ? codebook[tid] : 0.0f;
  }
  const bool exact_r = __syncthreads_and(my_exact) != 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) s_cbt[(8 * h + i) * kStride + gl] = s_cb[8 * h + i];

  float grid_scale = 0.0f, grid_off = 0.0f;
  bool use_guess = false;
  if (L >= 4) {
    const float th_first = s_th[0], th_last = s_th[L - 2];
    grid_scale = static_cast<float>(kAq2Cells - 2) / (th_last - th_first);
    grid_off = 1.0f - th_first * grid_scale;
    int gap_ok = 1;
    if (tid < 16) {
      const float pos = tid < L - 1 ? fmaf(s_th[tid], grid_scale, grid_off) : __int_as_float(0x7f800000);
      s_pos[tid] = pos;
      if (tid < L - 2) gap_ok = (fmaf(s_th[tid + 1], grid_scale, grid_off) - pos > 1.1f) ? 1 : 0;
    }
    use_guess = __syncthreads_and(gap_ok) != 0 && exact_r && isfinite(grid_scale);
    for (int k = tid; k < kAq2Cells; k += kAq4Threads) {
      const float lim = static_cast<float>(k) - 0.05f;
      int c = (s_pos[7] < lim) ? 8 : 0;
      c += (s_pos[c + 3] < lim) ? 4 : 0;
      c += (s_pos[c + 1] < lim) ? 2 : 0;
      c += (s_pos[c] < lim) ? 1 : 0;
      s_guess[k] = c * kStep;
    }
  }

  const long long tiles = (total_groups + kAq4Groups - 1) / kAq4Groups;
  auto issue_tile = [&](long long tile, int buf) {
    const long long g0 = tile * kAq4Groups;
    const long long ng = min(static_cast<long long>(kAq4Groups), total_groups - g0);
    const int nchunks = static_cast<int>(ng) * kChunksPerRow;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(x) + g0 * kRowBytes;
    const uint32_t dst = smem_u32(s_stage) + buf * kAq4Groups * kPitch;
#pragma unroll
    for (int i = 0; i < kAq4Groups * kChunksPerRow / kAq4Threads; ++i) {
      const int q = tid + kAq4Threads * i;
      if (q < nchunks) cp_async16(dst + (q / kChunksPerRow) * kPitch + (q % kChunksPerRow) * 16, src + q * 16);
    }
    cp_async_commit();
  };

  const char* const col = reinterpret_cast<const char*>(s_table + gl);
  const char* const cbcol = reinterpret_cast<const char*>(s_cbt + gl);
  // Everything above reads only the layer's thresholds and codebook, which no kernel of this library writes: when
  // launched as a programmatic dependent, the block builds its tables while the previous kernel is still running
  // and waits for it here, before the first read of x.
  pdl_wait();
  long long tile = blockIdx.x;
  int buf = 0;
  if (tile < tiles) issue_tile(tile, 0);
  for (; tile < tiles; tile += gridDim.x, buf ^= 1) {
    const long long next = tile + gridDim.x;
    if (next < tiles) {
      issue_tile(next, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    const long long gi = tile * kAq4Groups + gl;
    const bool valid = gi < total_groups;
    uint8_t* const row = s_stage + buf * kAq4Groups * kPitch + gl * kPitch + 8 * h;
    float v[32];
    if (valid) {
#pragma unroll
      for (int c = 0; c < 8; ++c) aq4_load4<T>(row + 16 * c, &v[4 * c]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = 0.0f;
    }
    if (PRE == 1) {   // every lane takes part (idle ones on zeros): the GELU votes across the warp
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = gelu_rounded_warp<T>(v[j]);
    }

    float p[4];
    aq4_lane_sums(v, p);
    const float mean = __fmul_rn(aq4_group_chain(p, lane), 0.015625f);   // /64: exact scaling
    {
      float q[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        v[j] = __fsub_rn(v[j], mean);
        q[j] = __fmul_rn(v[j], v[j]);
      }
      aq4_lane_sums(q, p);
    }
    const float var = __fmul_rn(aq4_group_chain(p, lane), 0.015625f);
    const float scale = __fsqrt_rn(__fadd_rn(var, 1.0e-6f));

    // the group's limits in r-space (or the thresholds themselves when dividing): entries 8h .. 8h+7 by lane h
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = 8 * h + i;
      float t = __int_as_float(0x7f800000);
      if (e < L - 1) {
        const float th = s_th[e];
        const float hs = __fmul_rd(__fmul_rn(s_h[e], scale), th == 0.0f ? 0x1p-50f : 1.0f);
        t = exact_r ? __fmaf_rd(th, scale, hs) : th;
      }
      s_table[e * kStride + gl] = t;
    }
    __syncwarp();

    // code of every residual -> codebook value (kept in v); nibbles of the codes in `half_words`
    uint32_t half_words[8];
    if (use_guess) {
      const float inv = grid_scale * __frcp_rn(scale);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t w = 0;
#pragma unroll
        for (int e = 3; e >= 0; --e) {
          const float r = v[4 * c + e];
          const unsigned cell = min(__float2uint_rz(fmaf(r, inv, grid_off)), static_cast<unsigned>(kAq2Cells - 1));
          int off = s_guess[cell];
          off += (r > *reinterpret_cast<const float*>(col + off)) ? kStep : 0;
          if (WRITE_PACKED) w = (w << 4) | static_cast<uint32_t>(off >> 9);
          v[4 * c + e] = *reinterpret_cast<const float*>(cbcol + off);
        }
        half_words[c] = w;
      }
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t w = 0;
#pragma unroll
        for (int e = 3; e >= 0; --e) {
          const float key = exact_r ? v[4 * c + e] : __fdiv_rn(v[4 * c + e], scale);
          int off = 0;
          if (BITS >= 4) off += (key > *reinterpret_cast<const float*>(col + off + 7 * kStep)) ? 8 * kStep : 0;
          if (BITS >= 3) off += (key > *reinterpret_cast<const float*>(col + off + 3 * kStep)) ? 4 * kStep : 0;
          off += (key > *reinterpret_cast<const float*>(col + off + 1 * kStep)) ? 2 * kStep : 0;
          off += (key > *reinterpret_cast<const float*>(col + off)) ? kStep : 0;
          if (WRITE_PACKED) w = (w << 4) | static_cast<uint32_t>(off >> 9);
          v[4 * c + e] = *reinterpret_cast<const float*>(cbcol + off);
        }
        half_words[c] = w;
      }
    }
    aq4_lane_sums(v, p);
    const float code_sum = aq4_group_chain(p, lane);

    if (WRITE_PACKED) {
      // Lane h holds nibbles 4h .. 4h+3 of each of the group's 8 words.  Swap halves with the partner so that
      // lane 0 ends up with words 0..3 and lane 1 with words 4..7, each complete.
      const uint32_t keep0 = h ? half_words[4] : half_words[0], keep1 = h ? half_words[5] : half_words[1];
      const uint32_t keep2 = h ? half_words[6] : half_words[2], keep3 = h ? half_words[7] : half_words[3];
      const uint32_t give0 = h ? half_words[0] : half_words[4], give1 = h ? half_words[1] : half_words[5];
      const uint32_t give2 = h ? half_words[2] : half_words[6], give3 = h ? half_words[3] : half_words[7];
      const uint32_t got01 = __shfl_xor_sync(0xffffffffu, give0 | (give1 << 16), 1);
      const uint32_t got23 = __shfl_xor_sync(0xffffffffu, give2 | (give3 << 16), 1);
      const uint32_t got[4] = {got01 & 0xFFFFu, got01 >> 16, got23 & 0xFFFFu, got23 >> 16};
      const uint32_t keep[4] = {keep0, keep1, keep2, keep3};
      uint32_t words[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) words[k] = h ? (got[k] | (keep[k] << 16)) : (keep[k] | (got[k] << 16));
      if (valid && packed != nullptr) {
        if (BITS == 4) {
          *reinterpret_cast<uint4*>(packed + gi * 32 + 16 * h) = make_uint4(words[0], words[1], words[2], words[3]);
        } else if (BITS == 3) {
          const uint32_t a = squeeze_nibbles_3(words[0]), b = squeeze_nibbles_3(words[1]);
          const uint32_t c2 = squeeze_nibbles_3(words[2]), d = squeeze_nibbles_3(words[3]);
          uint32_t* o = reinterpret_cast<uint32_t*>(packed + gi * 24 + 12 * h);    // 4-byte aligned
          o[0] = a | (b << 24);
          o[1] = (b >> 8) | (c2 << 16);
          o[2] = (c2 >> 16) | (d << 8);
        } else {
          *reinterpret_cast<uint2*>(packed + gi * 16 + 8 * h) =
              make_uint2(squeeze_nibbles_2(words[0]) | (squeeze_nibbles_2(words[1]) << 16),
                         squeeze_nibbles_2(words[2]) | (squeeze_nibbles_2(words[3]) << 16));
        }
      }
    }
    if (valid && h == 0 && mu_out != nullptr) {
      mu_out[gi] = mean;
      sigma_out[gi] = scale;
      if (codesum_out != nullptr) codesum_out[gi] = code_sum;
    }

    if (WRITE_XHAT) {
      // mean + scale*(cb - code_sum/64) as one fused multiply-add around mean - scale*code_sum/64 (the same
      // expression as the one-thread-per-group kernel), written over this lane's staged values and copied
      // out coalesced by the block
      const float vm = __fmul_rn(code_sum, 1.0f / 64.0f);   // exact: a power of two
      auto rec = [&](float cbv) { return __fadd_rn(mean, __fmul_rn(scale, __fsub_rn(cbv, vm))); };   // the reference's three rounded steps
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t lo = aq2_pack2<T>(rec(v[4 * c]), rec(v[4 * c + 1]));
        const uint32_t hi = aq2_pack2<T>(rec(v[4 * c + 2]), rec(v[4 * c + 3]));
        *reinterpret_cast<uint2*>(row + 16 * c) = make_uint2(lo, hi);
      }
      __syncthreads();
      const long long g0 = tile * kAq4Groups;
      const int ng = static_cast<int>(min(static_cast<long long>(kAq4Groups), total_groups - g0));
      uint8_t* dst = reinterpret_cast<uint8_t*>(xhat) + g0 * kRowBytes;
      const uint8_t* sbuf = s_stage + buf * kAq4Groups * kPitch;
#pragma unroll
      for (int i = 0; i < kAq4Groups * kChunksPerRow / kAq4Threads; ++i) {
        const int q = tid + kAq4Threads * i;
        if (q < ng * kChunksPerRow)
          *reinterpret_cast<uint4*>(dst + q * 16) =
              *reinterpret_cast<const uint4*>(sbuf + (q / kChunksPerRow) * kPitch + (q % kChunksPerRow) * 16);
      }
    }
    __syncthreads();  // everybody is done with this buffer (and this tile's table columns) before the next tile
  }
}

}  // namespace arcq
