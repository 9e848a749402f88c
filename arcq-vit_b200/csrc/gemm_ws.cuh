// Persistent, warp-specialised packed-weight GEMM for sm_100a:
//     y[M,N] = A[M,K] . W^[N,K]^T + bias,   A fp16 (already reconstructed activations),
//     W^ rebuilt on the fly from packed 2/3/4-bit codes + per-group statistics.
//
// One CTA per SM, each owning one slab of `bn` output columns and a strided set of 128-row tiles.
//   warp 0      TMA issuer: A tiles (128 x 64 fp16, 128-byte swizzle) and packed W codes (bn rows x two
//               groups of codes) into shared memory, each load completing on an mbarrier.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x bn x 16, fp16 in, fp32 accumulate in
//               tensor memory) and commits mbarriers that free the operand stages.
//   warps 2-5   epilogue: tensor memory -> registers -> + bias -> fp16/fp32 -> global.
//   warps 6-13  W producers: packed codes (shared memory) -> LUT -> mu' + sigma * v -> fp16 sub-tile
//               [bn x 64] in the layout tcgen05.mma reads.
// W sub-tiles live in a ring of `ws` slots.  When all K/64 sub-tiles of the slab fit (K = 384 with
// bn = 192) the ring is filled once and stays put for every tile of the CTA ("W-stationary"), so
// the rebuild cost is paid once per CTA and the steady state is TMA + MMA only.  Otherwise the ring
// streams, and each rebuilt sub-tile is used for the `nbb` tiles of a batch (one accumulator each).
// Two accumulators of up to 256 columns sit in tensor memory, so the epilogue of one tile overlaps
// the MMAs of the next.  Every wait is bounded; a wait that runs out sets the status word and the
// role stops issuing work, the CTA then drains and frees its tensor memory.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include "ptx.cuh"
#include "codes.cuh"
#include "packed_gemm.cuh"

namespace arcq {

struct WsParams {
  const float* mu_w;
  const float* sg_w;
  const float* cs_w;
  const float* cb_w;
  const float* bias;  // may be null
  void* y;
  int M, N, K, G;
  int bn;         // slab width: multiple of 16, <= 256, divides N
  int ws;         // W^ ring slots
  int sa;         // A stages
  int nbb;        // tiles per batch (1 or 2)
  int stationary; // 1: ring holds all G sub-tiles, filled once
  int y_f32;
  int* status;
};

constexpr int kWsThreads = 14 * 32;
constexpr int kWsProducerWarps = 8;
constexpr int kWsProducerThreads = kWsProducerWarps * 32;
constexpr int kRawSlots = 2;
constexpr int kStatusWsTimeout = 0x201;

// bytes of packed codes per row for the two groups one raw load brings in
__host__ __device__ constexpr int raw_row_bytes(int bits) { return 2 * 8 * bits; }

struct WsSmem {
  // offsets from the 1024-aligned base
  uint32_t a, w, raw, misc;
  uint32_t total;
};
__host__ __device__ inline WsSmem ws_smem_layout(int bn, int ws, int sa, int bits) {
  WsSmem s;
  s.a = 0;
  s.w = s.a + static_cast<uint32_t>(sa) * kStageA;
  s.raw = s.w + static_cast<uint32_t>(ws) * bn * 128;
  const uint32_t raw_slot = static_cast<uint32_t>(bn) * raw_row_bytes(bits) + 16;  // +16: 3-bit reads may look 3 bytes ahead
  s.misc = s.raw + kRawSlots * ((raw_slot + 127) & ~127u);
  s.total = s.misc + 16 * 4 /*lut*/ + 256 * 4 /*bias*/ + 64 * 8 /*barriers*/ + 16;
  return s;
}

template <int BITS>
__global__ void __launch_bounds__(kWsThreads, 1)
packed_weight_gemm_ws_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                             const WsParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const WsSmem L = ws_smem_layout(p.bn, p.ws, p.sa, BITS);
  uint8_t* const sA = smem + L.a;
  uint8_t* const sW = smem + L.w;
  uint8_t* const sRaw = smem + L.raw;
  const uint32_t raw_slot_bytes = (static_cast<uint32_t>(p.bn) * raw_row_bytes(BITS) + 16 + 127) & ~127u;
  float* const s_lut = reinterpret_cast<float*>(smem + L.misc);
  float* const s_bias = s_lut + 16;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(s_bias + 256);
  uint64_t* const a_full = bars;             // [sa]   <= 8
  uint64_t* const a_empty = bars + 8;        // [sa]
  uint64_t* const w_full = bars + 16;        // [ws]   <= 16
  uint64_t* const w_empty = bars + 32;       // [ws]
  uint64_t* const raw_full = bars + 48;      // [2]
  uint64_t* const raw_empty = bars + 50;     // [2]
  uint64_t* const acc_full = bars + 52;      // [2]
  uint64_t* const acc_empty = bars + 54;     // [2]
  uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(bars + 64);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bn = p.bn, G = p.G;
  const int n_slabs = p.N / bn;
  const int slab = blockIdx.x % n_slabs;
  const int rank = blockIdx.x / n_slabs;
  const int ctas_in_slab = (static_cast<int>(gridDim.x) - slab + n_slabs - 1) / n_slabs;
  const int tiles_m = (p.M + kTileM - 1) / kTileM;
  const int my_tiles = (rank < tiles_m) ? (tiles_m - rank + ctas_in_slab - 1) / ctas_in_slab : 0;
  const int n0 = slab * bn;
  const int nbb = p.nbb;
  const bool stationary = p.stationary != 0;

  if (tid < 16) s_lut[tid] = (tid < (1 << BITS)) ? p.cb_w[tid] : 0.0f;
  for (int i = tid; i < bn; i += kWsThreads) s_bias[i] = (p.bias != nullptr) ? p.bias[n0 + i] : 0.0f;
  if (tid == 0) {
    for (int i = 0; i < p.sa; ++i) { mbar_init(&a_full[i], 1); mbar_init(&a_empty[i], 1); }
    for (int i = 0; i < p.ws; ++i) { mbar_init(&w_full[i], kWsProducerWarps); mbar_init(&w_empty[i], 1); }
    for (int i = 0; i < kRawSlots; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], kWsProducerWarps); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
  }
  if (warp == 0) {
    tmem_alloc(s_tmem, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem;
  bool ok = true;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA issuer
    if (lane == 0) {
      uint32_t seq_a = 0, seq_r = 0;
      for (int b0 = 0; b0 < my_tiles && ok; b0 += nbb) {
        const int nb = min(nbb, my_tiles - b0);
        for (int g = 0; g < G && ok; ++g) {
          if ((!stationary || b0 == 0) && (g & 1) == 0) {
            const uint32_t slot = seq_r % kRawSlots;
            ok = mbar_wait(&raw_empty[slot], ((seq_r / kRawSlots) & 1) ^ 1);
            if (!ok) break;
            mbar_arrive_expect_tx(&raw_full[slot], static_cast<uint32_t>(bn) * raw_row_bytes(BITS));
            tma_load_2d(sRaw + slot * raw_slot_bytes, &tm_w, &raw_full[slot], (g >> 1) * raw_row_bytes(BITS), n0);
            ++seq_r;
          }
          for (int j = 0; j < nb; ++j) {
            const int tile = rank + (b0 + j) * ctas_in_slab;
            const uint32_t slot = seq_a % p.sa;
            ok = mbar_wait(&a_empty[slot], ((seq_a / p.sa) & 1) ^ 1);
            if (!ok) break;
            mbar_arrive_expect_tx(&a_full[slot], kStageA);
            tma_load_2d(sA + slot * kStageA, &tm_a, &a_full[slot], g * 64, tile * kTileM);
            ++seq_a;
          }
        }
      }
      if (!ok) atomicExch(p.status, kStatusWsTimeout);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(kTileM, bn);
      uint32_t seq_a = 0, seq_w = 0, tile_seq = 0;
      for (int b0 = 0; b0 < my_tiles && ok; b0 += nbb) {
        const int nb = min(nbb, my_tiles - b0);
        for (int j = 0; j < nb && ok; ++j) {
          const uint32_t ts = tile_seq + j;
          ok = mbar_wait(&acc_empty[ts & 1], ((ts >> 1) & 1) ^ 1);
        }
        tc_fence_after_sync();
        for (int g = 0; g < G && ok; ++g) {
          const uint32_t wslot = stationary ? static_cast<uint32_t>(g) : seq_w % p.ws;
          ok = mbar_wait(&w_full[wslot], stationary ? 0u : ((seq_w / p.ws) & 1));
          if (!ok) break;
          const uint64_t db = umma_desc_sw128(smem_u32(sW + wslot * bn * 128));
          for (int j = 0; j < nb; ++j) {
            const uint32_t slot = seq_a % p.sa;
            ok = mbar_wait(&a_full[slot], (seq_a / p.sa) & 1);
            if (!ok) break;
            tc_fence_after_sync();
            const uint64_t da = umma_desc_sw128(smem_u32(sA + slot * kStageA));
            const uint32_t d = tmem_base + ((tile_seq + j) & 1) * 256;
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_f16(d, da + 2 * k, db + 2 * k, idesc, (g > 0 || k > 0) ? 1u : 0u);
            umma_commit(&a_empty[slot]);
            ++seq_a;
          }
          if (!stationary) umma_commit(&w_empty[wslot]);
          ++seq_w;
        }
        if (ok)
          for (int j = 0; j < nb; ++j) umma_commit(&acc_full[(tile_seq + j) & 1]);
        tile_seq += nb;
      }
      if (!ok) atomicExch(p.status, kStatusWsTimeout);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue
    const int lq = warp & 3;  // tensor-memory lane quarter this warp may read
    uint32_t tile_seq = 0;
    for (int t = 0; t < my_tiles && ok; ++t, ++tile_seq) {
      const int tile = rank + t * ctas_in_slab;
      const uint32_t buf = tile_seq & 1;
      ok = mbar_wait(&acc_full[buf], (tile_seq >> 1) & 1);
      if (!ok) break;
      tc_fence_after_sync();
      const long long m = static_cast<long long>(tile) * kTileM + lq * 32 + lane;
      const bool row_ok = m < p.M;
      const uint32_t t_row = tmem_base + buf * 256 + (static_cast<uint32_t>(lq * 32) << 16);
      for (int c0 = 0; c0 < bn; c0 += 32) {
        uint32_t acc[32];
        if (c0 + 32 <= bn) {
          tmem_ld_32x32(t_row + c0, acc);
        } else {
          uint32_t lo[16];
          tmem_ld_32x16(t_row + c0, lo);
#pragma unroll
          for (int j = 0; j < 16; ++j) { acc[j] = lo[j]; acc[16 + j] = 0u; }
        }
        tmem_ld_wait();
        const int ncols = min(32, bn - c0);
        if (row_ok) {
          if (p.y_f32) {
            float* o = reinterpret_cast<float*>(p.y) + m * p.N + n0 + c0;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (4 * j < ncols)
                *reinterpret_cast<float4*>(o + 4 * j) =
                    make_float4(__uint_as_float(acc[4 * j]) + s_bias[c0 + 4 * j],
                                __uint_as_float(acc[4 * j + 1]) + s_bias[c0 + 4 * j + 1],
                                __uint_as_float(acc[4 * j + 2]) + s_bias[c0 + 4 * j + 2],
                                __uint_as_float(acc[4 * j + 3]) + s_bias[c0 + 4 * j + 3]);
          } else {
            __half* o = reinterpret_cast<__half*>(p.y) + m * p.N + n0 + c0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (8 * j < ncols) {
                uint32_t h[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const int c = 8 * j + 2 * q;
                  __half2 v = __floats2half2_rn(__uint_as_float(acc[c]) + s_bias[c0 + c],
                                                __uint_as_float(acc[c + 1]) + s_bias[c0 + c + 1]);
                  h[q] = *reinterpret_cast<uint32_t*>(&v);
                }
                *reinterpret_cast<uint4*>(o + 8 * j) = make_uint4(h[0], h[1], h[2], h[3]);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (!ok && lane == 0) atomicExch(p.status, kStatusWsTimeout);
  } else {
    // ------------------------------------------------------------------ W producers
    const int ptid = tid - 6 * 32;
    uint32_t seq_r = 0, seq_w = 0;
    const int fills = stationary ? 1 : (my_tiles + nbb - 1) / nbb;  // how many times the slab is walked
    for (int f = 0; f < fills && ok; ++f) {
      if (my_tiles == 0) break;
      for (int g = 0; g < G && ok; ++g) {
        const uint32_t rslot = seq_r % kRawSlots;
        if ((g & 1) == 0) ok = mbar_wait(&raw_full[rslot], (seq_r / kRawSlots) & 1);
        const uint32_t wslot = stationary ? static_cast<uint32_t>(g) : seq_w % p.ws;
        if (ok && !stationary) ok = mbar_wait(&w_empty[wslot], ((seq_w / p.ws) & 1) ^ 1);
        if (!ok) break;
        const uint8_t* raw = sRaw + rslot * raw_slot_bytes + (g & 1) * (8 * BITS);
        uint8_t* dstw = sW + wslot * bn * 128;
        for (int u = ptid; u < bn * 8; u += kWsProducerThreads) {
          const int r = u >> 3, chunk = u & 7;
          const uint8_t* rp = raw + r * raw_row_bytes(BITS);
          uint32_t w;
          if (BITS == 4) {
            w = *reinterpret_cast<const uint32_t*>(rp + 4 * chunk);
          } else if (BITS == 3) {
            const int off = 3 * chunk, al = off & ~3, sh = (off & 3) * 8;  // rp is 8-byte aligned
            const uint32_t lo = *reinterpret_cast<const uint32_t*>(rp + al);
            const uint32_t hi = *reinterpret_cast<const uint32_t*>(rp + al + 4);
            w = spread_3_to_nibbles(__funnelshift_r(lo, hi, sh) & 0xFFFFFFu);
          } else {
            w = spread_2_to_nibbles(*reinterpret_cast<const uint16_t*>(rp + 2 * chunk));
          }
          const long long si = static_cast<long long>(n0 + r) * G + g;
          const float sigma = __ldg(p.sg_w + si);
          const float mu_f = fmaf(-sigma, __ldg(p.cs_w + si) * (1.0f / 64.0f), __ldg(p.mu_w + si));
          rebuild_store8(w, sigma, mu_f, s_lut, dstw + sw128_offset(r, chunk));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&w_full[wslot]);
          if ((g & 1) == 1 || g == G - 1) mbar_arrive(&raw_empty[rslot]);
        }
        if ((g & 1) == 1 || g == G - 1) ++seq_r;
        ++seq_w;
      }
    }
    if (!ok && lane == 0) atomicExch(p.status, kStatusWsTimeout);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace arcq
