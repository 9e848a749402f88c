// Fused packed GEMM: y = A^ . W^T + bias with both operands rebuilt from packed codes on the fly.
//
// One CTA computes a 128 x BN tile of y.  The K loop advances one quantisation group (64 values)
// per stage: all threads rebuild the 128x64 slice of A^ and the BNx64 slice of W^ as fp16
//   v = mu' + sigma * cb[code],   mu' = mu - sigma * code_sum / 64
// straight into shared memory in the layout tcgen05.mma reads (K-major rows of 128 bytes, 128-byte
// swizzle), one thread then issues four 128xBNx16 MMAs that accumulate in fp32 in tensor memory,
// and a commit on an mbarrier tells everybody when that stage's buffers may be overwritten.  Two
// stages are in flight so the rebuild of group g+1 overlaps the MMAs of group g.  The epilogue
// reads the accumulator from tensor memory, adds the bias and stores fp16 or fp32.
//
// Every result element is the fp32 sum over k in a fixed order that does not depend on how rows
// are tiled, so a row's output is the same whatever M it is computed with.
#pragma once
#include <cuda_fp16.h>
#include "ptx.cuh"
#include "codes.cuh"

namespace arcq {

struct GemmParams {
  const uint8_t* pa;
  const float* mu_a;
  const float* sg_a;
  const float* cs_a;
  const uint8_t* pw;
  const float* mu_w;
  const float* sg_w;
  const float* cs_w;
  const float* cb_a;
  const float* cb_w;
  const float* bias;  // may be null
  void* y;
  int M, N, K, G;
  int pc;      // packed bytes per row
  int bn;      // tile width, multiple of 16, <= 256
  int y_f32;   // 1: fp32 output, 0: fp16
  int* status; // device status word
};

constexpr int kGemmThreads = 256;
constexpr int kTileM = 128;
constexpr int kStageA = kTileM * 128;  // bytes of one A stage (128 rows x 64 fp16)

// Status codes left in the device status word when a bounded wait runs out.
constexpr int kStatusGemmStageTimeout = 0x101;
constexpr int kStatusGemmAccTimeout = 0x102;

// Byte offset of 16-byte chunk `chunk` (0..7) of row `r` inside a swizzled K-major tile.
__device__ __forceinline__ uint32_t sw128_offset(int r, int chunk) {
  return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4));
}

// Rebuild 8 values from 8 codes (one per nibble of w) and store them as one 16-byte chunk.
__device__ __forceinline__ void rebuild_store8(uint32_t w, float sigma, float mu_f, const float* lut,
                                               uint8_t* dst) {
  uint32_t h[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float v0 = fmaf(sigma, lut[(w >> (8 * j)) & 15u], mu_f);
    const float v1 = fmaf(sigma, lut[(w >> (8 * j + 4)) & 15u], mu_f);
    __half2 p = __floats2half2_rn(v0, v1);
    h[j] = *reinterpret_cast<uint32_t*>(&p);
  }
  *reinterpret_cast<uint4*>(dst) = make_uint4(h[0], h[1], h[2], h[3]);
}

// Fill one K-major swizzled tile [rows_tile x 64] for group g from packed rows row0.. of a matrix
// with `rows_total` rows; rows beyond the matrix are zero.
template <int BITS>
__device__ __forceinline__ void rebuild_tile(uint8_t* tile, int rows_tile, long long row0, int rows_total, int g,
                                             const uint8_t* __restrict__ packed, int pc, int G,
                                             const float* __restrict__ mu, const float* __restrict__ sg,
                                             const float* __restrict__ cs, const float* lut) {
  for (int u = threadIdx.x; u < rows_tile * 8; u += kGemmThreads) {
    const int r = u >> 3, chunk = u & 7;
    uint8_t* dst = tile + sw128_offset(r, chunk);
    const long long row = row0 + r;
    if (row < rows_total) {
      const long long si = row * G + g;
      const float sigma = __ldg(sg + si);
      const float mu_f = fmaf(-sigma, __ldg(cs + si) * (1.0f / 64.0f), __ldg(mu + si));
      const uint32_t w = load_codes8<BITS>(packed + row * pc, g * 8 + chunk);
      rebuild_store8(w, sigma, mu_f, lut, dst);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

template <int BITS>
__global__ void __launch_bounds__(kGemmThreads, 1) packed_gemm_kernel(const GemmParams p) {
  pdl_launch_dependents();   // the next kernel of the stream may start its set-up
  pdl_wait();                // the input may be the previous kernel's output

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is what the 128-byte swizzle pattern is anchored to
  uint8_t* const smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int bn = p.bn;
  const int stage_b = bn * 128;
  uint8_t* const sA0 = smem;                 // two A stages, then two B stages
  uint8_t* const sB0 = smem + 2 * kStageA;
  float* s_lut_a = reinterpret_cast<float*>(smem + 2 * kStageA + 2 * stage_b);
  float* s_lut_w = s_lut_a + 16;
  float* s_bias = s_lut_w + 16;                                    // [bn]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + 256);      // [2] stage free
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 2);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const long long m0 = static_cast<long long>(blockIdx.x) * kTileM;
  const int n0 = blockIdx.y * bn;

  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(bn)) tmem_cols <<= 1;

  if (tid < 16) {
    s_lut_a[tid] = (tid < (1 << BITS)) ? p.cb_a[tid] : 0.0f;
    s_lut_w[tid] = (tid < (1 << BITS)) ? p.cb_w[tid] : 0.0f;
  }
  for (int i = tid; i < bn; i += kGemmThreads)
    s_bias[i] = (p.bias != nullptr && n0 + i < p.N) ? p.bias[n0 + i] : 0.0f;
  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(s_tmem, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem;
  const uint32_t idesc = umma_idesc_f16(kTileM, bn);

  bool ok = true;
  for (int g = 0; g < p.G; ++g) {
    const int s = g & 1;
    if (g >= 2) {
      // the MMAs of group g-2 read this stage; their commit is completion number (g>>1) of bars[s]
      if (!mbar_wait(&bars[s], ((g >> 1) - 1) & 1)) ok = false;
    }
    uint8_t* const sA = sA0 + s * kStageA;
    uint8_t* const sB = sB0 + s * stage_b;
    rebuild_tile<BITS>(sA, kTileM, m0, p.M, g, p.pa, p.pc, p.G, p.mu_a, p.sg_a, p.cs_a, s_lut_a);
    rebuild_tile<BITS>(sB, bn, n0, p.N, g, p.pw, p.pc, p.G, p.mu_w, p.sg_w, p.cs_w, s_lut_w);
    fence_proxy_async_smem();  // make the generic-proxy stores visible to the tensor core's reads
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      const uint64_t da = umma_desc_sw128(smem_u32(sA));
      const uint64_t db = umma_desc_sw128(smem_u32(sB));
#pragma unroll
      for (int k = 0; k < 4; ++k)  // 16 fp16 = 32 bytes = 2 descriptor units per K step
        umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, (g > 0 || k > 0) ? 1u : 0u);
      umma_commit(&bars[s]);
    }
  }
  // the last commit covers every MMA issued before it
  {
    const int gl = p.G - 1;
    if (!mbar_wait(&bars[gl & 1], (gl >> 1) & 1)) ok = false;
  }
  tc_fence_after_sync();
  if (!ok && lane == 0) atomicExch(p.status, kStatusGemmStageTimeout);

  // Epilogue: warp w reads tensor-memory lanes 32*(w%4)..+31 (one output row per thread); the two
  // warps that share a lane quarter take alternate 16-column chunks.
  {
    const int lq = warp & 3;
    const long long m = m0 + lq * 32 + lane;
    const bool row_ok = m < p.M;
    for (int ci = (warp >> 2); ci < bn / 16; ci += 2) {
      uint32_t acc[16];
      tmem_ld_32x16(tmem_base + (static_cast<uint32_t>(lq * 32) << 16) + ci * 16, acc);
      tmem_ld_wait();
      const int n = n0 + ci * 16;
      if (row_ok && n < p.N) {
        float f[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(acc[j]) + s_bias[ci * 16 + j];
        if (p.y_f32) {
          float* o = reinterpret_cast<float*>(p.y) + m * p.N + n;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (n + 4 * j < p.N)
              *reinterpret_cast<float4*>(o + 4 * j) = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
        } else {
          __half* o = reinterpret_cast<__half*>(p.y) + m * p.N + n;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            if (n + 8 * j < p.N) {
              uint32_t h[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                __half2 t = __floats2half2_rn(f[8 * j + 2 * q], f[8 * j + 2 * q + 1]);
                h[q] = *reinterpret_cast<uint32_t*>(&t);
              }
              *reinterpret_cast<uint4*>(o + 8 * j) = make_uint4(h[0], h[1], h[2], h[3]);
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, tmem_cols);
}

inline size_t packed_gemm_smem_bytes(int bn) {
  return 1024 /*alignment slack*/ + 2 * kStageA + 2 * static_cast<size_t>(bn) * 128 + (32 + 256) * 4 + 2 * 8 + 16;
}

}  // namespace arcq
