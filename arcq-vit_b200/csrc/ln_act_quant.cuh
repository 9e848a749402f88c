// Residual add + LayerNorm + activation quantizer in one kernel over fp16 rows: the glue in front of the first
// packed linear of a sub-block (norm1 -> qkv, norm2 -> fc1) merged with that linear's input quantizer.
//   s    = fp16(x + y)                                    (written out when y is given: the residual stream)
//   h    = fp16((s - mean(s)) * rsqrt(var(s) + eps) * gamma + beta)     (never written, unless asked for)
//   xhat = fp16(reconstruction of the ARCQ quantization of h in groups of 64)
// The separate kernels write h and read it back; here it goes through shared memory.
//
// Two phases per tile, each in the thread layout that suits it, and each with the arithmetic of the kernel it
// replaces, so that the results are bit-identical to arcq_add_layernorm followed by arcq_act_quant:
//   1. LayerNorm with the lane layout of add_layernorm_rows_kernel (LANES lanes per row, 16-byte accesses, the same
//      device function), writing h into padded group rows of shared memory;
//   2. the quantizer of act_quant_v2_kernel: one thread per 64-group reads its row, classifies with the exact
//      division-free test and the first-guess grid (that file documents both), writes the reconstruction back over
//      the row, and the block copies the rows out coalesced.
// A tile is 128 consecutive groups (the quantizer's unit), whatever the row length: the LayerNorm phase computes
// every row the tile touches (a row shared with the neighbouring tile is normalised by both; 1 row in 22 at
// K = 384) and keeps the groups that are the tile's.  Rows are owned (s and h written) by the tile that holds
// their first group.
#pragma once
#include <cuda_fp16.h>
#include "ptx.cuh"
#include "act_quant.cuh"
#include "act_quant_v2.cuh"
#include "add_layernorm.cuh"

namespace arcq {

constexpr int kLnqThreads = 128;
constexpr int kLnqPitch = 144;      // bytes between staged group rows (128 data bytes, conflict-free pitch)

__host__ __device__ constexpr size_t lnq_smem_bytes() {
  return kLnqThreads * kLnqPitch                // h, then reconstruction rows
         + 16 * kLnqThreads * 4                 // per-thread limit columns
         + 4 * 16 * 4 + kAq2Cells * 4 + 16;     // thresholds, half-gaps, codebook, grid positions, first guesses
}

template <int LANES, int BITS, bool HAS_Y>
__global__ void __launch_bounds__(kLnqThreads, 4)
    add_layernorm_act_quant_kernel(const __half* __restrict__ x, const __half* __restrict__ y,
                                   const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                                   long long M, const float* __restrict__ thresholds,
                                   const float* __restrict__ codebook, __half* __restrict__ sum_out,
                                   __half* __restrict__ h_out, __half* __restrict__ xhat) {
  pdl_launch_dependents();   // the next kernel of the stream may start its set-up

  constexpr int L = 1 << BITS;
  constexpr int K = LANES * 24, G = K / 64, kRowsPerWarp = 32 / LANES, kRowsPerPass = 4 * kRowsPerWarp;
  constexpr int kMaxRows = kLnqThreads / G + 2;                       // rows a tile of 128 groups can touch
  constexpr int kPasses = (kMaxRows + kRowsPerPass - 1) / kRowsPerPass;
  constexpr int kTableStride = kLnqThreads;
  extern __shared__ __align__(16) uint8_t lnq_smem[];
  uint8_t* const s_rows = lnq_smem;                                                   // [128] group rows
  float* const s_table = reinterpret_cast<float*>(s_rows + kLnqThreads * kLnqPitch);  // [16][128]
  float* const s_th = s_table + 16 * kTableStride;                                    // [16]
  float* const s_h = s_th + 16;
  float* const s_cb = s_h + 16;
  float* const s_pos = s_cb + 16;
  int* const s_guess = reinterpret_cast<int*>(s_pos + 16);                            // [kAq2Cells]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, l = lane % LANES, sub = lane / LANES;

  // ---- per-block set-up (reads only this layer's constants, so it runs before the wait below)
  int my_exact = 1;
  if (tid < 16) {
    float th = __int_as_float(0x7f800000), h = 0.0f;
    if (tid < L - 1) {
      th = thresholds[tid];
      if (th == 0.0f) {
        h = 0x1p-100f;
      } else {
        const int b = __float_as_int(th);
        const float up = __int_as_float(th > 0.0f ? b + 1 : b - 1);
        h = __fmul_rn(__fsub_rn(up, th), 0.5f);
      }
      my_exact = (th == 0.0f || fabsf(th) > 1.0e-15f) ? 1 : 0;
    }
    s_th[tid] = th;
    s_h[tid] = h;
    s_cb[tid] = tid < L ? codebook[tid] : 0.0f;
  }
  const bool exact_r = __syncthreads_and(my_exact) != 0;
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
    for (int k = tid; k < kAq2Cells; k += kLnqThreads) {
      const float lim = static_cast<float>(k) - 0.05f;
      int c = (s_pos[7] < lim) ? 8 : 0;
      c += (s_pos[c + 3] < lim) ? 4 : 0;
      c += (s_pos[c + 1] < lim) ? 2 : 0;
      c += (s_pos[c] < lim) ? 1 : 0;
      s_guess[k] = c * (kLnqThreads * 4);
    }
  }
  float* const my_table = s_table + tid;
  const char* const col = reinterpret_cast<const char*>(my_table);
  constexpr int kStep = kTableStride * 4;
  static_assert(kStep == 512, "the code extraction below assumes a 512-byte table step");
  uint8_t* const my_row = s_rows + tid * kLnqPitch;

  pdl_wait();                // x and y may be the previous kernels' outputs

  const long long total_groups = M * G;
  const long long tiles = (total_groups + kLnqThreads - 1) / kLnqThreads;
  for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const long long gi0 = tile * kLnqThreads;
    const int ngroups = static_cast<int>(min(static_cast<long long>(kLnqThreads), total_groups - gi0));
    const long long r_first = gi0 / G;
    // ---- phase 1: LayerNorm of every row the tile touches, LANES lanes per row
    {
      float gg[3][8], bb[3][8];
      layernorm_lane_params<LANES>(gamma, beta, l, gg, bb);
      // (issuing the loads of all passes before the first pass computes was tried: 72 more live registers, spills,
      // 13.5 us instead of 11.3 us; one pass ahead, with gamma and beta re-read per pass to make room: 11.4 us, no gain)
#pragma unroll 1
      for (int pass = 0; pass < kPasses; ++pass) {
        const long long row = r_first + pass * kRowsPerPass + warp * kRowsPerWarp + sub;
        const long long lg0 = row * G - gi0;                       // tile-local index of the row's first group
        const bool in_tile = row < M && lg0 < ngroups;             // the row has groups in this tile
        const bool owned = in_tile && lg0 >= 0;                    // ... and its first group is one of them
        const long long rs = row < M ? row : M - 1;                // idle sub-warps shadow the last row
        uint4 h[3];
        layernorm_row<LANES>(x, HAS_Y ? y : nullptr, rs, row, owned, l, gg, bb, eps, sum_out, h);
        if (in_tile) {
#pragma unroll
          for (int i = 0; i < 3; ++i) {
            const int ch = l + LANES * i;                          // 16-byte chunk of the row: group ch / 8, part ch % 8
            const long long lg = lg0 + (ch >> 3);
            if (lg >= 0 && lg < ngroups)
              *reinterpret_cast<uint4*>(s_rows + lg * kLnqPitch + (ch & 7) * 16) = h[i];
            if (owned && h_out != nullptr) reinterpret_cast<uint4*>(h_out + row * K)[ch] = h[i];
          }
        }
      }
    }
    __syncthreads();

    // ---- phase 2: the activation quantizer on h, one thread per group (same steps as act_quant_v2_kernel)
    const bool valid = tid < ngroups;
    float v[64];
    if (valid) {
      aq2_load_row<__half>(my_row, v);
    } else {
#pragma unroll
      for (int j = 0; j < 64; ++j) v[j] = 0.0f;
    }
    const float mean = __fdiv_rn(sum64_ref_order(v), 64.0f);
    float var;
    {
      float q[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        v[j] = __fsub_rn(v[j], mean);
        q[j] = __fmul_rn(v[j], v[j]);
      }
      var = __fdiv_rn(sum64_ref_order(q), 64.0f);
    }
    const float scale = __fsqrt_rn(__fadd_rn(var, 1.0e-6f));
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float t = __int_as_float(0x7f800000);
      if (i < L - 1) {
        const float th = s_th[i];
        const float hs = __fmul_rd(__fmul_rn(s_h[i], scale), th == 0.0f ? 0x1p-50f : 1.0f);
        t = exact_r ? __fmaf_rd(th, scale, hs) : th;
      }
      if (i < L) my_table[i * kTableStride] = t;
    }
    const char* const cbp = reinterpret_cast<const char*>(s_cb);
    if (use_guess) {
      const float inv = grid_scale * __frcp_rn(scale);
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        const float r = v[j];
        const unsigned cell = min(__float2uint_rz(fmaf(r, inv, grid_off)), static_cast<unsigned>(kAq2Cells - 1));
        int off = s_guess[cell];
        off += (r > *reinterpret_cast<const float*>(col + off)) ? kStep : 0;
        v[j] = *reinterpret_cast<const float*>(cbp + (off >> 7));          // code = off / 512, four bytes per entry
      }
    } else {
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        const float key = exact_r ? v[j] : __fdiv_rn(v[j], scale);
        int off = 0;
        if (BITS >= 4) off += (key > *reinterpret_cast<const float*>(col + off + 7 * kStep)) ? 8 * kStep : 0;
        if (BITS >= 3) off += (key > *reinterpret_cast<const float*>(col + off + 3 * kStep)) ? 4 * kStep : 0;
        off += (key > *reinterpret_cast<const float*>(col + off + 1 * kStep)) ? 2 * kStep : 0;
        off += (key > *reinterpret_cast<const float*>(col + off)) ? kStep : 0;
        v[j] = *reinterpret_cast<const float*>(cbp + (off >> 7));
      }
    }
    const float code_sum = sum64_ref_order(v);
    if (valid) {
      // reconstruction mean + scale*(cb[c] - code_sum/64) in the reference's three rounded steps
      const float vm = __fmul_rn(code_sum, 1.0f / 64.0f);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int e = 8 * c + 2 * j;
          o[j] = aq2_pack2<__half>(__fadd_rn(mean, __fmul_rn(scale, __fsub_rn(v[e], vm))),
                                   __fadd_rn(mean, __fmul_rn(scale, __fsub_rn(v[e + 1], vm))));
        }
        *reinterpret_cast<uint4*>(my_row + 16 * c) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    __syncthreads();
    // ---- coalesced copy-out of the reconstruction (groups are contiguous in memory)
    {
      const int nchunks = ngroups * 8;
      uint8_t* xo = reinterpret_cast<uint8_t*>(xhat) + gi0 * 128;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int q = tid + kLnqThreads * i;
        if (q < nchunks)
          *reinterpret_cast<uint4*>(xo + q * 16) = *reinterpret_cast<const uint4*>(s_rows + (q >> 3) * kLnqPitch + (q & 7) * 16);
      }
    }
    __syncthreads();   // the rows are free for the next tile
  }
}

// ---------------------------------------------------------------------------------------------------------
// The same operation for small inputs (a few hundred rows: batch 1-16 of a ViT), where the forward is a chain of
// short launches and one launch fewer counts for more than instruction counts.  Blocks of twelve warps, two phases per
// tile of 128 / LANES rows, through 6 KB of shared memory (the quantizer phase has three times as many lanes as the
// LayerNorm phase has, so that it is a single pass and the block's latency is one LayerNorm plus one quantizer step):
//   1. warps 0-3: residual add + LayerNorm with the lane layout and the arithmetic of add_layernorm_rows_kernel
//      (the same device function), so s and h are bit-identical to that kernel's;
//   2. all warps: the quantizer with the lane layout and the arithmetic of act_quant_kernel (eight lanes per group, IEEE
//      division, chain sums in the reference's order), reading h from shared memory.
// Its reconstruction therefore equals, bit for bit, what the two separate kernels produce, and a model may switch
// between the merged and the separate form by batch size without changing a single output bit.
constexpr int kLnqRowsThreads = 384;

template <int LANES, int BITS, bool HAS_Y>
__global__ void __launch_bounds__(kLnqRowsThreads) add_layernorm_act_quant_rows_kernel(const __half* __restrict__ x,
                                                                          const __half* __restrict__ y,
                                                                          const float* __restrict__ gamma,
                                                                          const float* __restrict__ beta, float eps,
                                                                          long long M,
                                                                          const float* __restrict__ thresholds,
                                                                          const float* __restrict__ codebook,
                                                                          __half* __restrict__ sum_out,
                                                                          __half* __restrict__ h_out,
                                                                          __half* __restrict__ xhat) {
  pdl_launch_dependents();
  constexpr int L = 1 << BITS;
  constexpr int K = LANES * 24, G = K / 64, kRowsPerWarp = 32 / LANES, kRows = 4 * kRowsPerWarp;   // rows per tile
  constexpr int kSlots = kRows * G * 8;            // (group, lane-of-eight) pairs per tile: 384 for every width
  static_assert(kSlots == kLnqRowsThreads, "the quantizer phase is one pass of the block");
  __shared__ __align__(16) __half s_hid[kRows * K];
  __shared__ float s_th[16];
  __shared__ float s_cb[16];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, l = lane % LANES, sub = lane / LANES;
  if (tid < 16) {
    s_th[tid] = (tid < L - 1) ? thresholds[tid] : __int_as_float(0x7f800000);
    s_cb[tid] = (tid < L) ? codebook[tid] : 0.0f;
  }
  float gg[3][8] = {}, bb[3][8] = {};
  if (warp < 4) layernorm_lane_params<LANES>(gamma, beta, l, gg, bb);
  __syncthreads();
  pdl_wait();                // everything above is the layer's constants; x and y may be the previous kernel's output

  const int l8 = lane & 7, octet_base = lane & ~7;
  for (long long row0 = static_cast<long long>(blockIdx.x) * kRows; row0 < M; row0 += static_cast<long long>(gridDim.x) * kRows) {
    // ---- phase 1 (warps 0-3): one row per LANES lanes
    if (warp < 4) {
      const int local = warp * kRowsPerWarp + sub;
      const long long row = row0 + local;
      const bool valid = row < M;
      const long long rs = valid ? row : M - 1;
      uint4 h[3];
      layernorm_row<LANES>(x, HAS_Y ? y : nullptr, rs, row, valid, l, gg, bb, eps, sum_out, h);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        reinterpret_cast<uint4*>(s_hid + local * K)[l + LANES * i] = h[i];
        if (valid && h_out != nullptr) reinterpret_cast<uint4*>(h_out + row * K)[l + LANES * i] = h[i];
      }
    }
    __syncthreads();
    // ---- phase 2 (all warps): eight lanes per 64-group, lane l8 holds elements 8c + l8
    {
      const int grp = tid >> 3;                              // group of the tile
      const int local = grp / G, g = grp - local * G;
      const long long row = row0 + local;
      const bool valid = row < M;
      const __half* hg = s_hid + local * K + g * 64 + l8;
      float v[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) v[c] = __half2float(hg[8 * c]);
      float a0 = __fadd_rn(v[0], v[4]), a1 = __fadd_rn(v[1], v[5]);
      float a2 = __fadd_rn(v[2], v[6]), a3 = __fadd_rn(v[3], v[7]);
      float part = __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3);
      const float mean = __fdiv_rn(octet_chain_sum(part, octet_base), 64.0f);
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
      float cv[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float t = __fdiv_rn(r[c], scale);
        int code = 0;
        if (BITS >= 4) code = (t > s_th[7]) ? 8 : 0;
        if (BITS >= 3) code += (t > s_th[code + 3]) ? 4 : 0;
        code += (t > s_th[code + 1]) ? 2 : 0;
        code += (t > s_th[code]) ? 1 : 0;
        cv[c] = s_cb[code];
      }
      a0 = __fadd_rn(cv[0], cv[4]); a1 = __fadd_rn(cv[1], cv[5]);
      a2 = __fadd_rn(cv[2], cv[6]); a3 = __fadd_rn(cv[3], cv[7]);
      part = __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3);
      const float code_sum = octet_chain_sum(part, octet_base);
      const float vm = __fdiv_rn(code_sum, 64.0f);
      if (valid) {
        __half* og = xhat + row * K + g * 64 + l8;
#pragma unroll
        for (int c = 0; c < 8; ++c) og[8 * c] = __float2half_rn(__fadd_rn(mean, __fmul_rn(scale, __fsub_rn(cv[c], vm))));
      }
    }
    __syncthreads();   // the tile's rows in shared memory are free for the next tile
  }
}

}  // namespace arcq
