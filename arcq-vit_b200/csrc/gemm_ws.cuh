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
  int dense;      // 1: the weight operand is an fp16 matrix [N,K] in global memory (its sub-tiles arrive by TMA, nothing is rebuilt)
  int y_f32;
  int rotate;     // 1: slabs walk their tile list from different starting points
  int tma_store;  // 1: epilogue stages 32-row x 128-byte blocks in shared memory and stores them with TMA
  int* status;
  long long* trace;  // debugging: per-CTA timestamps (64 slots each), or null
};

constexpr int kWsThreads = 14 * 32;
constexpr int kWsProducerWarps = 8;
constexpr int kWsProducerThreads = kWsProducerWarps * 32;
constexpr int kRawSlots = 2;
constexpr int kStatusWsTimeout = 0x201;

// One raw load brings in the packed codes of `raw_groups` 64-column groups for every row of the slab: the
// fewest groups whose bytes per row (8 * bits each) are a multiple of the 16 bytes a TMA box row must be.
__host__ __device__ constexpr int raw_groups(int bits) { return bits == 3 ? 2 : 1; }
__host__ __device__ constexpr int raw_row_bytes(int bits) { return raw_groups(bits) * 8 * bits; }
__host__ __device__ constexpr uint32_t raw_slot_size(int bn, int bits) {
  return (static_cast<uint32_t>(bn) * raw_row_bytes(bits) + 16 + 127) & ~127u;   // +16: 3-bit reads may look 3 bytes ahead
}
// Narrow stationary slabs (few rows: small batches, where one CTA's latency chain is the whole kernel) take
// all their packed codes in one burst -- every raw load issued at once on one barrier -- and rebuild all the
// sub-tiles in one pass with one hand-over, instead of one load / rebuild / hand-over round per sub-tile.
__host__ __device__ constexpr int raw_loads(int G, int bits) { return (G + raw_groups(bits) - 1) / raw_groups(bits); }
__host__ __device__ constexpr bool ws_burst(int bn, int bits, int G, bool stationary, bool dense) {
  return stationary && !dense && raw_loads(G, bits) * raw_slot_size(bn, bits) <= 16384u;
}

struct WsSmem {
  // offsets from the 1024-aligned base
  uint32_t a, w, stage, raw, fold, misc;
  uint32_t total;
};
constexpr uint32_t kEpiStageBytes = 4 * 4096;  // 4 epilogue warps x (32 rows x 128 bytes)
constexpr int kLutCopies = 8;   // copies of the pair table, one per (lane & 7): fewer bank conflicts on the look-ups
// A | W^ ring | build + epilogue area | tables and barriers.  The build area holds the raw-code slots and the
// slab's folded statistics (bn * G words), the epilogue area the output staging blocks.  A W-stationary slab
// is built once, before the first accumulator is complete, so there the two areas share their bytes; a
// streaming ring keeps rebuilding while the epilogue runs and gets both.
__host__ __device__ inline WsSmem ws_smem_layout(int bn, int ws, int sa, int bits, int G, bool stationary,
                                                 bool dense = false) {
  WsSmem s;
  s.a = 0;
  s.w = s.a + static_cast<uint32_t>(sa) * kStageA;
  const uint32_t area = s.w + static_cast<uint32_t>(ws) * bn * 128;
  const uint32_t raw_bytes = dense ? 0u
                             : (ws_burst(bn, bits, G, stationary, dense) ? raw_loads(G, bits) : kRawSlots) *
                                   raw_slot_size(bn, bits);
  const uint32_t fold_bytes = dense ? 0u : (static_cast<uint32_t>(bn) * G * 4u + 127) & ~127u;
  uint32_t area_bytes;
  if (stationary) {
    s.stage = area;
    s.raw = area;
    s.fold = s.raw + raw_bytes;
    area_bytes = raw_bytes + fold_bytes > kEpiStageBytes ? raw_bytes + fold_bytes : kEpiStageBytes;
  } else {
    s.stage = area;
    s.raw = s.stage + kEpiStageBytes;
    s.fold = s.raw + raw_bytes;
    area_bytes = kEpiStageBytes + raw_bytes + fold_bytes;
  }
  s.misc = area + area_bytes;
  s.total = s.misc + 16 * 4 /*lut*/ + 256 * 4 /*bias*/ + 64 * 8 /*barriers*/ + 16 + 256 * 4 * kLutCopies /*pair lut*/;
  return s;
}

template <int BITS, bool TRACE = false>
__global__ void __launch_bounds__(kWsThreads, 1)
packed_weight_gemm_ws_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                             const __grid_constant__ CUtensorMap tm_y, const WsParams p) {
  extern __shared__ uint8_t smem_raw[];
  // round up to 1024 bytes by pointer arithmetic, so the compiler still knows this is shared memory
  uint8_t* const smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const WsSmem L = ws_smem_layout(p.bn, p.ws, p.sa, BITS, p.G, p.stationary != 0, p.dense != 0);
  uint8_t* const sA = smem + L.a;
  uint8_t* const sW = smem + L.w;
  uint8_t* const sRaw = smem + L.raw;
  uint8_t* const sStage = smem + L.stage;
  const uint32_t raw_slot_bytes = raw_slot_size(p.bn, BITS);
  constexpr int RG = raw_groups(BITS);
  float* const s_lut = reinterpret_cast<float*>(smem + L.misc);
  float* const s_bias = s_lut + 16;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(s_bias + 256);
  uint64_t* const a_full = bars;             // [sa]   <= 8
  uint64_t* const a_empty = bars + 8;        // [sa]
  uint64_t* const w_full = bars + 16;        // [ws]   <= 16 (ring) or <= 32 (stationary)
  uint64_t* const w_empty = bars + 32;       // [ws]
  uint64_t* const raw_full = bars + 48;      // [2]
  uint64_t* const raw_empty = bars + 50;     // [2]
  uint64_t* const acc_full = bars + 52;      // [2]
  uint64_t* const acc_empty = bars + 54;     // [2]
  uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(bars + 64);
  uint32_t* const s_lut2 = s_tmem + 4;          // [256][8] half2: codebook values of (low nibble, high nibble)
  // folded statistics of the slab: half2 (sigma, mu - sigma*code_sum/64) per (row, group)
  uint32_t* const s_fold = reinterpret_cast<uint32_t*>(smem + L.fold);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bn = p.bn, G = p.G;
  const int n_slabs = p.N / bn;
  const int slab = blockIdx.x % n_slabs;
  const int rank = blockIdx.x / n_slabs;
  const int ctas_in_slab = (static_cast<int>(gridDim.x) - slab + n_slabs - 1) / n_slabs;
  const int tiles_m = (p.M + kTileM - 1) / kTileM;
  const int my_tiles = (rank < tiles_m) ? (tiles_m - rank + ctas_in_slab - 1) / ctas_in_slab : 0;
  const int n0 = slab * bn;
  // The CTAs of different slabs that share a rank walk the same tiles; each slab starts at a different
  // point of that list so that they do not all ask L2 for the same lines at the same moment.
  const int rot = (my_tiles > 0 && p.rotate) ? (slab * my_tiles) / n_slabs : 0;
  auto tile_of = [&](int t) { int q = t + rot; if (q >= my_tiles) q -= my_tiles; return rank + q * ctas_in_slab; };
  const int nbb = p.nbb;
  const bool stationary = p.stationary != 0;

  const bool dense = p.dense != 0;
  const bool burst = ws_burst(p.bn, BITS, p.G, p.stationary != 0, dense);
  // Only the barriers and the tensor-memory allocation are set up before the roles part: the pair table and
  // the bias are filled by the roles that read them (builders, epilogue), so their global-memory latency does
  // not hold back the first TMA loads.
  pdl_launch_dependents();
  if (tid == 0) {
    for (int i = 0; i < p.sa; ++i) { mbar_init(&a_full[i], 1); mbar_init(&a_empty[i], 1); }
    // a stationary slab never recycles a slot: its (up to 32) full barriers may run into the empty ones' space
    for (int i = 0; i < p.ws; ++i) mbar_init(&w_full[i], dense ? 1 : kWsProducerWarps);
    if (p.stationary == 0)
      for (int i = 0; i < p.ws; ++i) mbar_init(&w_empty[i], 1);
    for (int i = 0; i < kRawSlots; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], kWsProducerWarps); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_y);
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
  // Timestamps for the debugging entry point only: in the production instantiation (TRACE = false) `tr` is a
  // compile-time null and every stamp below folds away.
  long long* const tr = (TRACE && p.trace != nullptr) ? p.trace + static_cast<long long>(blockIdx.x) * 128 : nullptr;
  auto stamp = [&](int slot) {
    if (TRACE && tr != nullptr && slot < 128) {
      long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      tr[slot] = t;
    }
  };
  if (tid == 0) stamp(0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA issuer
    // The whole warp walks the loop and waits (converged code is far cheaper to run than a lone lane in a
    // divergent branch); lane 0 arms the barriers and issues the copies.
    uint32_t a_slot = 0, a_ph = 1, r_slot = 0, r_ph = 1;     // "empty" barriers: first pass is free
    uint32_t w_slot = 0, w_ph = 1;                            // dense operand only
    const uint32_t sa = p.sa, wsn = p.ws;
    const int raw_x_step = raw_row_bytes(BITS);
    // The activation (and, in the dense form, the weight matrix) may be the previous kernel's output.  The packed
    // weight, its statistics and the bias are constants of the layer: the other roles read them without waiting.
    pdl_wait();
    for (int b0 = 0; b0 < my_tiles; b0 += nbb) {
      const int nb = min(nbb, my_tiles - b0);
      for (int g = 0; g < G; ++g) {
        if (dense) {
          if (!stationary || b0 == 0) {
            const uint32_t wi = stationary ? static_cast<uint32_t>(g) : w_slot;
            if (!stationary) ok = ok && mbar_wait_relaxed(&w_empty[wi], w_ph, 32);
            if (lane == 0 && ok) {
              mbar_arrive_expect_tx(&w_full[wi], static_cast<uint32_t>(bn) * 128u);
              tma_load_2d(sW + wi * bn * 128, &tm_w, &w_full[wi], g * 64, n0);
            }
            __syncwarp();
            if (!stationary) {
              const bool wrap = w_slot + 1 == wsn;
              w_slot = wrap ? 0u : w_slot + 1;
              w_ph ^= wrap ? 1u : 0u;
            }
          }
        } else if (burst) {
          if (b0 == 0 && g == 0) {
            if (lane == 0) {
              const int n_loads = raw_loads(G, BITS);
              mbar_arrive_expect_tx(&raw_full[0], static_cast<uint32_t>(n_loads) * bn * raw_row_bytes(BITS));
              for (int q = 0; q < n_loads; ++q)
                tma_load_2d(sRaw + q * raw_slot_bytes, &tm_w, &raw_full[0], q * raw_x_step, n0);
            }
            __syncwarp();
          }
        } else if ((!stationary || b0 == 0) && (g % RG) == 0) {
          ok = ok && mbar_wait_relaxed(&raw_empty[r_slot], r_ph);
          if (lane == 0 && ok) {
            mbar_arrive_expect_tx(&raw_full[r_slot], static_cast<uint32_t>(bn) * raw_row_bytes(BITS));
            tma_load_2d(sRaw + r_slot * raw_slot_bytes, &tm_w, &raw_full[r_slot], (g / RG) * raw_x_step, n0);
          }
          __syncwarp();
          const bool wrap = r_slot + 1 == kRawSlots;
          r_slot = wrap ? 0u : r_slot + 1;
          r_ph ^= wrap ? 1u : 0u;
        }
        for (int j = 0; j < nb; ++j) {
          ok = ok && mbar_wait_relaxed(&a_empty[a_slot], a_ph, 32);
          if (lane == 0 && ok) {
            mbar_arrive_expect_tx(&a_full[a_slot], kStageA);
            tma_load_2d(sA + a_slot * kStageA, &tm_a, &a_full[a_slot], g * 64, tile_of(b0 + j) * kTileM);
          }
          __syncwarp();
          const bool wrap = a_slot + 1 == sa;
          a_slot = wrap ? 0u : a_slot + 1;
          a_ph ^= wrap ? 1u : 0u;
        }
      }
    }
    if (lane == 0) {
      stamp(1);
      if (!ok) atomicExch(p.status, kStatusWsTimeout);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Same shape: all lanes wait and keep the ring positions, lane 0 issues the MMAs and the commits.
    const uint32_t idesc = umma_idesc_f16(kTileM, bn);
    const uint64_t desc_hi = umma_desc_sw128(0);     // descriptors: a constant high part plus (address >> 4)
    const uint32_t sa = p.sa, wsn = p.ws;
    const uint32_t a_base = smem_u32(sA) >> 4, w_base = smem_u32(sW) >> 4;
    const uint32_t a_step = kStageA >> 4, w_step = static_cast<uint32_t>(bn) * 128 >> 4;
    uint32_t a_slot = 0, a_ph = 0, w_slot = 0, w_ph = 0;
    uint32_t acc_ph0 = 1, acc_ph1 = 1;   // acc_empty phases: first use of each buffer is free
    uint32_t buf = 0;                    // accumulator buffer of the next tile
    int batch = 0;
    for (int b0 = 0; b0 < my_tiles; b0 += nbb, ++batch) {
      const int nb = min(nbb, my_tiles - b0);
      const uint32_t buf0 = buf;
      for (int j = 0; j < nb; ++j) {
        const uint32_t bj = (buf0 + j) & 1;
        ok = ok && mbar_wait_relaxed(&acc_empty[bj], bj ? acc_ph1 : acc_ph0, 32);
        acc_ph0 ^= bj ? 0u : 1u;
        acc_ph1 ^= bj ? 1u : 0u;
      }
      tc_fence_after_sync();
      if (lane == 0) stamp(8 + 2 * batch);
      bool w_waits = !stationary || b0 == 0;   // a stationary slab is built once
      if (burst && b0 == 0) {
        // a slab built in one burst hands all its sub-tiles over together: take them all now (nothing the
        // builders wait for depends on the MMAs), so that even the first tile runs the lean loop below
        for (int g = 0; g < G; ++g) ok = ok && mbar_wait_relaxed(&w_full[g], 0u, 32);
        w_waits = false;
      }
      const bool st = TRACE && tr != nullptr && batch == 2 && lane == 0;
      const uint32_t leader = lane == 0 ? 1u : 0u;
      if (!w_waits && nb == 1) {
        // steady state of a stationary slab: nothing but "A stage landed -> four MMAs -> free the stage"
        const uint32_t d = tmem_base + (buf0 & 1) * 256;
        for (int g = 0; g < G; ++g) {
          ok = ok && mbar_wait_spin(&a_full[a_slot], a_ph);
          const uint64_t da = desc_hi | (a_base + a_slot * a_step);
          const uint64_t db = desc_hi | (w_base + g * w_step);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_f16_if(leader, d, da + 2 * k, db + 2 * k, idesc, (g > 0 || k > 0) ? 1u : 0u);
            if (st && g < 8) tr[64 + g * 8 + k] = clock64();
          }
          umma_commit_if(leader, &a_empty[a_slot]);
          const bool wrap = a_slot + 1 == sa;
          a_slot = wrap ? 0u : a_slot + 1;
          a_ph ^= wrap ? 1u : 0u;
        }
      } else
      for (int g = 0; g < G; ++g) {
        const uint32_t wi = stationary ? static_cast<uint32_t>(g) : w_slot;
        if (w_waits) ok = ok && mbar_wait_spin(&w_full[wi], stationary ? 0u : w_ph);
        if (st && g < 8) tr[64 + g * 8 + 6] = clock64();
        const uint64_t db = desc_hi | (w_base + wi * w_step);
        for (int j = 0; j < nb; ++j) {
          ok = ok && mbar_wait_spin(&a_full[a_slot], a_ph);
          if (st && g < 8) tr[64 + g * 8 + 7] = clock64();
          const uint64_t da = desc_hi | (a_base + a_slot * a_step);
          const uint32_t d = tmem_base + ((buf0 + j) & 1) * 256;
          if (lane == 0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              umma_f16(d, da + 2 * k, db + 2 * k, idesc, (g > 0 || k > 0) ? 1u : 0u);
              if (st && g < 8) tr[64 + g * 8 + k] = clock64();
            }
            umma_commit(&a_empty[a_slot]);
            if (st && g < 8) tr[64 + g * 8 + 4] = clock64();
          }
          __syncwarp();
          const bool wrap = a_slot + 1 == sa;
          a_slot = wrap ? 0u : a_slot + 1;
          a_ph ^= wrap ? 1u : 0u;
          if (st && g < 8) tr[64 + g * 8 + 5] = clock64();
        }
        if (!stationary) {
          if (lane == 0) umma_commit(&w_empty[w_slot]);
          __syncwarp();
          const bool wrap = w_slot + 1 == wsn;
          w_slot = wrap ? 0u : w_slot + 1;
          w_ph ^= wrap ? 1u : 0u;
        }
      }
      if (lane == 0) {
        if (ok)
          for (int j = 0; j < nb; ++j) umma_commit(&acc_full[(buf0 + j) & 1]);
        stamp(9 + 2 * batch);
      }
      __syncwarp();
      buf = (buf0 + nb) & 1;
    }
    if (!ok && lane == 0) atomicExch(p.status, kStatusWsTimeout);
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue
    for (int i = tid - 2 * 32; i < bn; i += 4 * 32) s_bias[i] = (p.bias != nullptr) ? __ldg(p.bias + n0 + i) : 0.0f;
    asm volatile("bar.sync 2, 128;" ::: "memory");   // the four epilogue warps
    const int lq = warp & 3;  // tensor-memory lane quarter this warp may read
    uint32_t tile_seq = 0;
    uint32_t half = 0;   // staging block of the next TMA store; alternates across tiles as well as within one
    for (int t = 0; t < my_tiles && ok; ++t, ++tile_seq) {
      const int tile = tile_of(t);
      const uint32_t buf = tile_seq & 1;
      ok = mbar_wait_relaxed(&acc_full[buf], (tile_seq >> 1) & 1, 128);
      if (!ok) break;
      tc_fence_after_sync();
      if (warp == 2 && lane == 0) stamp(32 + 2 * t);
      const long long m = static_cast<long long>(tile) * kTileM + lq * 32 + lane;
      const bool row_ok = m < p.M;
      const uint32_t t_row = tmem_base + buf * 256 + (static_cast<uint32_t>(lq * 32) << 16);
      if (p.tma_store) {
        // 32 rows x 64 bytes per step (32 fp16 or 16 fp32 columns): registers -> staging block with the
        // 64-byte swizzle (conflict-free 16-byte stores) -> one TMA store.  Two blocks per warp alternate (from
        // tile to tile too, so a tile with an odd number of steps does not reuse the block its last store
        // is still reading), so a step only waits for the store issued two steps earlier to have read its block.
        uint8_t* const stg = sStage + lq * 4096;
        const int cw = p.y_f32 ? 16 : 32;
        for (int c0 = 0; c0 < bn; c0 += cw, half ^= 1) {
          uint32_t acc[32];
          if (p.y_f32) {
            tmem_ld_32x16(t_row + c0, *reinterpret_cast<uint32_t(*)[16]>(&acc[0]));
          } else {
            tmem_ld_32x32(t_row + c0, acc);
          }
          tmem_ld_wait();
          if (lane == 0) tma_store_wait_read_1();
          __syncwarp();
          uint8_t* const rowp = stg + half * 2048 + lane * 64;
          const int sw = (lane >> 1) & 3;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 v;
            if (p.y_f32) {
              const float4 b4 = *reinterpret_cast<const float4*>(s_bias + c0 + 4 * ch);
              v.x = __float_as_uint(__uint_as_float(acc[4 * ch]) + b4.x);
              v.y = __float_as_uint(__uint_as_float(acc[4 * ch + 1]) + b4.y);
              v.z = __float_as_uint(__uint_as_float(acc[4 * ch + 2]) + b4.z);
              v.w = __float_as_uint(__uint_as_float(acc[4 * ch + 3]) + b4.w);
            } else {
              const float4 b0 = *reinterpret_cast<const float4*>(s_bias + c0 + 8 * ch);
              const float4 b1 = *reinterpret_cast<const float4*>(s_bias + c0 + 8 * ch + 4);
              __half2 h0 = __floats2half2_rn(__uint_as_float(acc[8 * ch]) + b0.x, __uint_as_float(acc[8 * ch + 1]) + b0.y);
              __half2 h1 = __floats2half2_rn(__uint_as_float(acc[8 * ch + 2]) + b0.z, __uint_as_float(acc[8 * ch + 3]) + b0.w);
              __half2 h2 = __floats2half2_rn(__uint_as_float(acc[8 * ch + 4]) + b1.x, __uint_as_float(acc[8 * ch + 5]) + b1.y);
              __half2 h3 = __floats2half2_rn(__uint_as_float(acc[8 * ch + 6]) + b1.z, __uint_as_float(acc[8 * ch + 7]) + b1.w);
              v.x = *reinterpret_cast<uint32_t*>(&h0);
              v.y = *reinterpret_cast<uint32_t*>(&h1);
              v.z = *reinterpret_cast<uint32_t*>(&h2);
              v.w = *reinterpret_cast<uint32_t*>(&h3);
            }
            *reinterpret_cast<uint4*>(rowp + ((ch ^ sw) << 4)) = v;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tm_y, stg + half * 2048, n0 + c0, tile * kTileM + lq * 32);
            tma_store_commit();
          }
        }
      } else
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
      if (warp == 2 && lane == 0) stamp(33 + 2 * t);
    }
    if (lane == 0) tma_store_wait_all();
    if (!ok && lane == 0) atomicExch(p.status, kStatusWsTimeout);
  } else {
    // ------------------------------------------------------------------ W producers
    const int ptid = tid - 6 * 32;
    uint32_t r_slot = 0, r_ph = 0, w_slot = 0, w_ph = 1;
    const int fills = stationary ? 1 : (my_tiles + nbb - 1) / nbb;  // how many times the slab is walked
    // Each thread owns the (row, 16-byte chunk) units u = ptid + 256*i of a sub-tile: row (ptid>>3) + 32*i,
    // chunk ptid&7.  Statistics come from shared memory when the slab's arrays were staged there
    // (W-stationary), else from global memory (L2 after the first walk of the slab).
    const int chunk = ptid & 7;
    const int units = (bn * 8 + kWsProducerThreads - 1 - ptid) / kWsProducerThreads;
    // pair table: codebook values of (low nibble, high nibble) of a byte, kLutCopies copies side by side
    if (my_tiles > 0 && !dense) {
      const int lo = ptid & 15, hi = ptid >> 4;
      __half2 v = __floats2half2_rn(lo < (1 << BITS) ? __ldg(p.cb_w + lo) : 0.0f, hi < (1 << BITS) ? __ldg(p.cb_w + hi) : 0.0f);
#pragma unroll
      for (int c = 0; c < kLutCopies; ++c) s_lut2[ptid * kLutCopies + c] = *reinterpret_cast<uint32_t*>(&v);
    }
    // fold the slab's statistics once: (sigma, mu') as one half2 word per (row, group)
    if (my_tiles > 0 && !dense) {
      for (int i = ptid; i < bn * G; i += kWsProducerThreads) {
        const long long si = static_cast<long long>(n0) * G + i;
        const float sigma = __ldg(p.sg_w + si);
        const __half2 f2 = __floats2half2_rn(sigma, fmaf(-sigma, __ldg(p.cs_w + si) * (1.0f / 64.0f), __ldg(p.mu_w + si)));
        s_fold[i] = *reinterpret_cast<const uint32_t*>(&f2);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kWsProducerThreads) : "memory");   // producer warps only
    }
    if (burst && my_tiles > 0) {
      // every (sub-tile, row, chunk) unit of the slab in one strided pass, then one hand-over per sub-tile
      ok = mbar_wait_relaxed(&raw_full[0], 0u);
      const int per_g = bn * 8;
      int g = 0, idx = ptid;
      while (ok) {
        while (idx >= per_g) { idx -= per_g; ++g; }
        if (g >= G) break;
        const int r = idx >> 3, ch = idx & 7;
        const uint8_t* rp = sRaw + (g / RG) * raw_slot_bytes + (g % RG) * (8 * BITS) + r * raw_row_bytes(BITS);
        uint32_t w;
        if (BITS == 4) {
          w = *reinterpret_cast<const uint32_t*>(rp + 4 * ch);
        } else if (BITS == 3) {
          const int off = 3 * ch, al = off & ~3, sh = (off & 3) * 8;
          w = spread_3_to_nibbles(__funnelshift_r(*reinterpret_cast<const uint32_t*>(rp + al),
                                                  *reinterpret_cast<const uint32_t*>(rp + al + 4), sh) & 0xFFFFFFu);
        } else {
          w = spread_2_to_nibbles(*reinterpret_cast<const uint16_t*>(rp + 2 * ch));
        }
        const uint32_t fw = s_fold[r * G + g];
        const __half2 f2 = *reinterpret_cast<const __half2*>(&fw);
        const __half2 s2 = __low2half2(f2);
        const __half2 m2 = __high2half2(f2);
        uint32_t hv[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t pv = s_lut2[((w >> (8 * q)) & 0xFFu) * kLutCopies + (lane & (kLutCopies - 1))];
          const __half2 r2 = __hfma2(s2, *reinterpret_cast<const __half2*>(&pv), m2);
          hv[q] = *reinterpret_cast<const uint32_t*>(&r2);
        }
        *reinterpret_cast<uint4*>(sW + g * bn * 128 + sw128_offset(r, ch)) = make_uint4(hv[0], hv[1], hv[2], hv[3]);
        idx += kWsProducerThreads;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0)
        for (int gg = 0; gg < G; ++gg) mbar_arrive(&w_full[gg]);
      if (ptid == 0) stamp(7);
    }
    for (int f = 0; f < fills && ok; ++f) {
      if (my_tiles == 0 || dense || burst) break;
      for (int g = 0; g < G && ok; ++g) {
        const uint32_t rslot = r_slot;
        if ((g % RG) == 0) ok = mbar_wait_relaxed(&raw_full[rslot], r_ph);
        const uint32_t wslot = stationary ? static_cast<uint32_t>(g) : w_slot;
        if (ok && !stationary) ok = mbar_wait_relaxed(&w_empty[wslot], w_ph);
        if (!ok) break;
        const uint8_t* const raw = sRaw + rslot * raw_slot_bytes + (g % RG) * (8 * BITS);
        uint8_t* const dstw = sW + wslot * bn * 128;
#pragma unroll 3
        for (int i = 0; i < units; ++i) {
          const int r = (ptid >> 3) + 32 * i;
          const uint8_t* rp = raw + r * raw_row_bytes(BITS);
          uint32_t w;
          if (BITS == 4) {
            w = *reinterpret_cast<const uint32_t*>(rp + 4 * chunk);
          } else if (BITS == 3) {
            const int off = 3 * chunk, al = off & ~3, sh = (off & 3) * 8;  // rp is 8-byte aligned
            w = spread_3_to_nibbles(__funnelshift_r(*reinterpret_cast<const uint32_t*>(rp + al),
                                                    *reinterpret_cast<const uint32_t*>(rp + al + 4), sh) & 0xFFFFFFu);
          } else {
            w = spread_2_to_nibbles(*reinterpret_cast<const uint16_t*>(rp + 2 * chunk));
          }
          // mu' + sigma * cb[code] for two codes at a time: one look-up in the pair table per byte of nibbles,
          // one half2 fused multiply-add.  (The rebuild is bound by shared-memory accesses, not arithmetic:
          // one word of codes, one word of folded statistics, four table look-ups and a 16-byte store per
          // eight values.)
          const uint32_t fw = s_fold[r * G + g];
          const __half2 f2 = *reinterpret_cast<const __half2*>(&fw);
          const __half2 s2 = __low2half2(f2);
          const __half2 m2 = __high2half2(f2);
          uint32_t h[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t pv = s_lut2[((w >> (8 * q)) & 0xFFu) * kLutCopies + (lane & (kLutCopies - 1))];
            const __half2 r2 = __hfma2(s2, *reinterpret_cast<const __half2*>(&pv), m2);
            h[q] = *reinterpret_cast<const uint32_t*>(&r2);
          }
          *reinterpret_cast<uint4*>(dstw + sw128_offset(r, chunk)) = make_uint4(h[0], h[1], h[2], h[3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&w_full[wslot]);
          if ((g % RG) == RG - 1 || g == G - 1) mbar_arrive(&raw_empty[rslot]);
        }
        if ((g % RG) == RG - 1 || g == G - 1) {
          if (++r_slot == kRawSlots) { r_slot = 0; r_ph ^= 1; }
        }
        if (!stationary && ++w_slot == static_cast<uint32_t>(p.ws)) { w_slot = 0; w_ph ^= 1; }
        if (f == 0 && ptid == 0) stamp(2 + (g < 5 ? g : 5));
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
