// Dense-weight GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a:
//     y[M,N] = A[M,K] . W16[N,K]^T + bias,   A fp16 (reconstructed activations), W16 the fp16 weight a
//     separate unpack kernel wrote into a scratch matrix (the reference's own data flow,
//     fair_qat/arcq_packed_on_the_fly.py:147-160).
//
// Same pair geometry, barriers, epilogue and bounded waits as the packed-weight pair kernel (gemm_pair.cuh);
// the difference is where the B operand comes from.  Both operands arrive by TMA: a stage holds this CTA's
// 128 rows of A and its bn/2 rows of W16 for `ks` 64-wide K sub-tiles, and one barrier in the leader counts
// the bytes of both CTAs.  There are no weight-building warps; a CTA is ten warps:
//   warp 0      TMA: A and W16 sub-tiles of every stage
//   warp 1      MMA issue (leader CTA only)
//   warps 2-9   epilogue: tensor memory -> registers -> + bias -> fp16/fp32 -> staging -> TMA store
//               In the PREFETCH form (arcq_dense_weight_gemm_prefetch) they first unpack the NEXT layer's weight into
//               the other scratch matrix, at a time when no accumulator is ready yet: no launch, no second stream,
//               no events for the unpack.  They wait for the previous kernel first, so the matrix they overwrite is
//               no longer read by anybody (its last reader is two GEMMs back).
// and the kernel starts issuing as soon as its first stage has landed (no table or statistics set-up).
//
// STATIONARY: the pair's whole W16 slab (bn/2 rows x K per CTA) is loaded once and stays in shared memory for
// all the row tiles the pair works on; only A streams through the stages.  With K = 384 the operands of a
// 256 x 192 tile are used for so few flops that the L2 -> shared-memory traffic (about 8 TB/s over all SMs)
// bounds the kernel, and the slab is 43 % of that traffic.
//
// Each output element is the fp32 sum over k in ascending order of 16-wide steps, as in every other GEMM
// kernel of this library.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include "ptx.cuh"
#include "gemm_pair.cuh"
#include "codes.cuh"

namespace arcq {

struct PairDenseParams {
  const float* bias;  // may be null
  int M, N, K, G;
  int bn;          // slab width per pair: multiple of 32, <= 256, divides N
  int sa;          // stages
  int ks;          // 64-wide K sub-tiles per stage; divides G
  int y_f32;
  uint32_t poll_limit;  // sleeping waits give up after this many polls
  uint32_t spin_limit;  // the issuing thread's busy waits give up after this many probes
  int* status;
  UnpackWeightJob next;  // the weight of the layer that runs after this one, unpacked by two spare warps (or none)
};

constexpr int kPairDenseThreads = (2 + kPairEpiWarps) * 32;
// Staging blocks (2 KB: 32 rows x 64 bytes) per epilogue warp; a block can be rewritten once the TMA store that
// reads it has done so.  Four blocks instead of two measured slower on every DeiT-S shape (qkv 13.6 -> 15.5 us,
// fc2 17.5 -> 22.3 us): the 32 KB they take away from the operand stages cost more than deeper stores gain.  One
// block (16 KB more for the stages) helped only the layer with few stores per flop (fc2 17.5 -> 17.0 us) and cost
// the store-heavy ones (qkv 13.8 -> 14.5 us, fc1 16.5 -> 16.9 us).
#ifndef ARCQ_DENSE_STAGE_BLOCKS
#define ARCQ_DENSE_STAGE_BLOCKS 2
#endif
constexpr int kDenseStageBlocks = ARCQ_DENSE_STAGE_BLOCKS;
constexpr uint32_t kPairDenseEpiStageBytes = kPairEpiWarps * kDenseStageBlocks * 2048;

struct PairDenseSmem {
  uint32_t stages, slab, stage, misc, total;
};
constexpr int kPairDenseBarriers = 72;
__host__ __device__ inline PairDenseSmem pair_dense_smem_layout(int bn, int sa, int ks, int G, bool stationary) {
  PairDenseSmem s;
  const uint32_t wtile = static_cast<uint32_t>(bn / 2) * 128u;
  const uint32_t stage_bytes = static_cast<uint32_t>(ks) * (kStageA + (stationary ? 0u : wtile));
  s.stages = 0;
  s.slab = static_cast<uint32_t>(sa) * stage_bytes;
  s.stage = s.slab + (stationary ? static_cast<uint32_t>(G) * wtile : 0u);
  s.misc = s.stage + kPairDenseEpiStageBytes;
  s.total = s.misc + 256 * 4 /*bias*/ + kPairDenseBarriers * 8 + 16 /*tensor-memory address*/ + 32 /*next codebook*/;
  return s;
}

template <bool STATIONARY, bool PREFETCH = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairDenseThreads, 1)
    dense_weight_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                                  const __grid_constant__ CUtensorMap tm_y, const PairDenseParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* const smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const PairDenseSmem L = pair_dense_smem_layout(p.bn, p.sa, p.ks, p.G, STATIONARY);
  uint8_t* const sStages = smem + L.stages;
  uint8_t* const sSlab = smem + L.slab;
  uint8_t* const sStage = smem + L.stage;
  float* const s_bias = reinterpret_cast<float*>(smem + L.misc);
  uint64_t* const bars = reinterpret_cast<uint64_t*>(s_bias + 256);
  // barriers: full [sa] <= 16 at 0 (leader: both CTAs' bytes of the stage landed);  empty [sa] at 16 (both: the
  // MMAs that read the stage are done);  acc_full [2] at 32 (both);  acc_empty [2] at 34 (leader);
  // slab_full [G] <= 32 at 40 (leader, stationary slab only: sub-tile g of both CTAs landed)
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t full = bar0, empty = bar0 + 16 * 8, acc_full = bar0 + 32 * 8, acc_empty = bar0 + 34 * 8;
  const uint32_t slab_full = bar0 + 40 * 8;
  uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(bars + kPairDenseBarriers);
  __half* const s_next_cb = reinterpret_cast<__half*>(s_tmem + 4);     // [16], unpack warps only

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t crank = cluster_ctarank();     // 0: leader
  const int bn = p.bn, hb = bn >> 1, G = p.G, ks = p.ks;
  const int n_pairs = static_cast<int>(gridDim.x) >> 1;
  const int pair = static_cast<int>(blockIdx.x) >> 1;
  const int n_slabs = p.N / bn;
  const int slab = pair % n_slabs;
  const int rank = pair / n_slabs;
  const int pairs_in_slab = (n_pairs - slab + n_slabs - 1) / n_slabs;
  const int tiles_m = (p.M + kPairTileM - 1) / kPairTileM;
  const int my_tiles = (rank < tiles_m) ? (tiles_m - rank + pairs_in_slab - 1) / pairs_in_slab : 0;
  const int n0 = slab * bn;            // first column of the slab
  const int nh0 = n0 + crank * hb;     // first W16 row this CTA loads
  // pairs of different slabs that share a rank walk the same row tiles; stagger their starting points
  const int rot = (my_tiles > 0) ? (slab * my_tiles) / n_slabs : 0;
  auto row_of = [&](int t) {
    int q = t + rot;
    if (q >= my_tiles) q -= my_tiles;
    return (rank + q * pairs_in_slab) * kPairTileM + static_cast<int>(crank) * kTileM;
  };
  const uint32_t poll_limit = p.poll_limit, spin_limit = p.spin_limit;
  const uint32_t wtile_bytes = static_cast<uint32_t>(hb) * 128u;
  const uint32_t stage_bytes = static_cast<uint32_t>(ks) * (kStageA + (STATIONARY ? 0u : wtile_bytes));

  pdl_launch_dependents();
  if (tid == 0) {
    for (int i = 0; i < p.sa; ++i) { mbar_init(&bars[i], 1); mbar_init(&bars[16 + i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[32 + i], 1); mbar_init(&bars[34 + i], 2 * kPairEpiWarps); }
    if (STATIONARY)
      for (int i = 0; i < p.G; ++i) mbar_init(&bars[40 + i], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_y);
  }
  if (warp == 0) {
    tmem_alloc_pair(s_tmem, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();          // barriers of both CTAs initialised, tensor memory allocated in both
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem;
  bool ok = true;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA: this CTA's half of every stage
    const uint32_t sa = p.sa;
    const uint32_t full_leader = mapa_shared(full, 0);
    const uint32_t st0 = smem_u32(sStages);
    uint32_t slot = 0, ph = 1;     // "empty" barriers: the first pass is free
    uint32_t good = 1;
    // Both operands are other kernels' outputs (the activation quantizer's and the weight unpack's).
    pdl_wait();
    if (STATIONARY && my_tiles > 0) {
      // the whole slab, once; its sub-tiles land while the first A stages do
      if (elect_one()) {
        const uint32_t slab_leader = mapa_shared(slab_full, 0);
        const uint32_t sl0 = smem_u32(sSlab);
        for (int g = 0; g < G; ++g) {
          if (crank == 0) mbar_expect_tx(slab_full + g * 8, 2u * wtile_bytes);
          tma_load_2d_pair(sl0 + g * wtile_bytes, &tm_w, slab_leader + g * 8, g * 64, nh0);
        }
      }
      __syncwarp();
    }
    for (int t = 0; t < my_tiles; ++t) {
      const int row0 = row_of(t);
      for (int g0 = 0; g0 < G; g0 += ks) {
        good &= mbar_park_flag(empty + slot * 8, ph, good ? poll_limit : 0u);
        if (elect_one()) {
          if (good) {
            if (crank == 0) mbar_expect_tx(full + slot * 8, 2u * stage_bytes);
            const uint32_t dst = st0 + slot * stage_bytes;
            for (int q = 0; q < ks; ++q)
              tma_load_2d_pair(dst + q * kStageA, &tm_a, full_leader + slot * 8, (g0 + q) * 64, row0);
            if (!STATIONARY)
              for (int q = 0; q < ks; ++q)
                tma_load_2d_pair(dst + ks * kStageA + q * wtile_bytes, &tm_w, full_leader + slot * 8, (g0 + q) * 64, nh0);
          }
        }
        __syncwarp();
        if (++slot == sa) { slot = 0; ph ^= 1; }
      }
      if (__any_sync(0xffffffffu, good == 0)) break;
    }
    ok = __all_sync(0xffffffffu, good != 0);
    if (!ok) {
      // give copies that are still in flight time to land before this CTA's shared memory goes away
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
      if (lane == 0) atomicExch(p.status, kStatusPairTimeout);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue (leader CTA only)
    if (crank == 0 && my_tiles > 0) {
      const uint32_t idesc = umma_idesc_f16(kPairTileM, bn);
      const uint32_t sa = p.sa;
      const uint32_t lo0 = ((smem_u32(sStages) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t s_step = stage_bytes >> 4, w_off = (static_cast<uint32_t>(ks) * kStageA) >> 4, w_step = wtile_bytes >> 4;
      const uint32_t slab_lo0 = ((smem_u32(sSlab) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t empty_r = mapa_shared(empty, 1), acc_full_r = mapa_shared(acc_full, 1);
      uint32_t slot = 0, ph = 0, lo = lo0;
      uint32_t acc_ph0 = 1, acc_ph1 = 1;   // acc_empty phases: the first use of each buffer is free
      uint32_t buf = 0;
      uint32_t good = 1;
      for (int t = 0; t < my_tiles; ++t) {
        good &= mbar_park_flag(acc_empty + buf * 8, buf ? acc_ph1 : acc_ph0, good ? poll_limit : 0u);
        acc_ph0 ^= buf ? 0u : 1u;
        acc_ph1 ^= buf ? 1u : 0u;
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * 256;
        uint32_t acc = 0;
        for (int g0 = 0; g0 < G; g0 += ks) {
          if (STATIONARY && t == 0) {   // the slab lands while the first tile runs
            for (int q = 0; q < ks; ++q) good &= mbar_spin_flag(slab_full + (g0 + q) * 8, 0u, good ? spin_limit : 0u);
          }
          good &= mbar_spin_flag(full + slot * 8, ph, good ? spin_limit : 0u);
          tc_fence_after_sync();
          if (elect_one()) {
            if (good) {
              uint32_t al = lo, wl = STATIONARY ? slab_lo0 + static_cast<uint32_t>(g0) * w_step : lo + w_off;
              for (int q = 0; q < ks; ++q) {
                umma_pair_f16_x4(d, al, wl, idesc, (q == 0) ? acc : 1u);
                al += kStageA >> 4;
                wl += w_step;
              }
              umma_pair_commit(empty + slot * 8);
              umma_pair_commit(empty_r + slot * 8);
              if (g0 + ks >= G) {
                umma_pair_commit(acc_full + buf * 8);
                umma_pair_commit(acc_full_r + buf * 8);
              }
            }
          }
          __syncwarp();
          acc = 1u;
          lo += s_step;
          if (++slot == sa) { slot = 0; ph ^= 1; lo = lo0; }
        }
        buf ^= 1;
        if (__any_sync(0xffffffffu, good == 0)) break;
      }
      ok = __all_sync(0xffffffffu, good != 0);
      __syncwarp();
      if (!ok && lane == 0) atomicExch(p.status, kStatusPairTimeout);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (own 128 rows of each tile)
    // Eight warps: two per tensor-memory lane quarter, taking alternate column steps of 64 bytes per row.
    // A step goes registers -> + bias -> fp16/fp32 -> one of this warp's two 2 KB staging blocks (64-byte
    // swizzle, conflict-free 16-byte stores) -> one TMA store.
    const int ew = warp - 2;
    for (int i = tid - 64; i < bn; i += kPairEpiWarps * 32) s_bias[i] = (p.bias != nullptr) ? __ldg(p.bias + n0 + i) : 0.0f;
    if (PREFETCH && tid - 64 < 16)
      s_next_cb[tid - 64] = __float2half_rn(tid - 64 < (1 << p.next.bits) ? __ldg(p.next.codebook + (tid - 64)) : 0.0f);
    asm volatile("bar.sync 2, %0;" ::"n"(kPairEpiWarps * 32) : "memory");   // bias table (and codebook) complete
    if (PREFETCH) {
      // The next layer's weight, while these warps have no accumulator to drain yet.  Wait for the previous kernel
      // first: the scratch matrix being overwritten was last read two GEMMs back and is then free for certain.
      pdl_wait();
      const long long first = static_cast<long long>(blockIdx.x) * (kPairEpiWarps * 32) + (tid - 64);
      const long long stride = static_cast<long long>(gridDim.x) * (kPairEpiWarps * 32);
      if (p.next.bits == 4) unpack_weight_f16_chunks<4>(p.next, s_next_cb, first, stride);
      else if (p.next.bits == 3) unpack_weight_f16_chunks<3>(p.next, s_next_cb, first, stride);
      else unpack_weight_f16_chunks<2>(p.next, s_next_cb, first, stride);
    }
    const int lq = warp & 3;                          // tensor-memory lane quarter this warp may read
    const int half_id = ew >> 2;                      // which of the two warps of the quarter
    const uint32_t acc_empty_leader = mapa_shared(acc_empty, 0);
    uint8_t* const stg = sStage + ew * (kDenseStageBlocks * 2048);
    const int cw = p.y_f32 ? 16 : 32;
    const bool f32 = p.y_f32 != 0;
    uint32_t blk = 0;      // staging block of the next store; the blocks are used in turn
    auto emit = [&](const uint32_t (&acc)[32], int c0, int row0) {
      if (lane == 0) tma_store_wait_read_n<kDenseStageBlocks - 1>();   // the store that last used this block has read it
      __syncwarp();
      uint8_t* const rowp = stg + blk * 2048 + lane * 64;
      const int sw = (lane >> 1) & 3;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint4 v;
        if (f32) {
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
        tma_store_2d(&tm_y, stg + blk * 2048, n0 + c0, row0);     // rows beyond M are clipped
        tma_store_commit();
      }
      blk = (blk + 1 == kDenseStageBlocks) ? 0 : blk + 1;
    };
    auto load = [&](uint32_t (&acc)[32], uint32_t taddr) {
      if (f32) tmem_ld_32x16(taddr, *reinterpret_cast<uint32_t(*)[16]>(&acc[0]));
      else tmem_ld_32x32(taddr, acc);
    };
    const int step = 2 * cw;
    for (int t = 0; t < my_tiles && ok; ++t) {
      const uint32_t buf = static_cast<uint32_t>(t) & 1;
      if (!mbar_wait_sleep_a(acc_full + buf * 8, (static_cast<uint32_t>(t) >> 1) & 1, poll_limit, 32)) { ok = false; break; }
      tc_fence_after_sync();
      const int row0 = row_of(t) + lq * 32;
      const uint32_t t_row = tmem_base + buf * 256 + (static_cast<uint32_t>(lq * 32) << 16);
      const bool live = row0 < p.M;     // some of these 32 rows are inside the matrix
      // The tensor-memory reads run one step ahead of the conversion, and the accumulator is handed back as
      // soon as the last read has landed, before its values are converted.
      uint32_t ra[32], rb[32];
      int c0 = half_id * cw;
      bool released = false;
      auto release = [&]() {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader + buf * 8);
        released = true;
      };
      if (live && c0 < bn) {
        load(ra, t_row + c0);
        while (true) {
          tmem_ld_wait();
          bool more = c0 + step < bn;
          if (more) load(rb, t_row + c0 + step); else release();
          emit(ra, c0, row0);
          if (!more) break;
          c0 += step;
          tmem_ld_wait();
          more = c0 + step < bn;
          if (more) load(ra, t_row + c0 + step); else release();
          emit(rb, c0, row0);
          if (!more) break;
          c0 += step;
        }
      }
      if (!released) release();
    }
    if (lane == 0) tma_store_wait_all();
    if (!ok && lane == 0) atomicExch(p.status, kStatusPairTimeout);
  }

  // Both CTAs stay until the other is done: the leader's MMAs read the peer's shared memory and signal its
  // barriers, the peer's warps arrive on the leader's barriers.
  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 0) tmem_dealloc_pair(tmem_base, 512);
}

}  // namespace arcq
