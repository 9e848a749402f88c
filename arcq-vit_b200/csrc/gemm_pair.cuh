// Packed-weight GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a:
//     y[M,N] = A[M,K] . W^[N,K]^T + bias,   A fp16 (reconstructed activations),
//     W^ rebuilt on the fly from packed 2/3/4-bit codes + per-group statistics.
//
// The grid is a list of two-CTA clusters, one per pair of SMs.  A pair owns one slab of `bn` output columns
// and a strided set of 256-row tiles.  One thread of the pair's first CTA (the leader) issues
// tcgen05.mma.cta_group::2 instructions of shape 256 x bn x 16: each CTA supplies the 128 rows of A it
// loaded and the bn/2 rows of W^ it rebuilt, from the same shared-memory offsets, and receives the
// 128 x bn accumulator of its own rows in its own tensor memory.  Compared with one CTA per tile this
// halves the W^ slab each SM has to rebuild and hold (so K = 384 leaves room for eight A stages instead
// of three), halves the shared-memory operand traffic per flop, and issues one instruction for two SMs.
//
// Roles, the same in both CTAs unless noted:
//   warp 0      TMA: its half of every A tile (128 x 64 fp16 per load, 128-byte swizzle) and the packed
//               codes of its half slab.  A loads of both CTAs complete on the leader's barrier.
//   warp 1      MMA issue (leader only): waits for operands, issues, commits barriers in both CTAs.
//   warps 2-5   epilogue: own tensor memory -> registers -> + bias -> fp16/fp32 -> staging -> TMA store.
//   warps 6-13  W^ producers: packed codes -> pair table -> mu' + sigma * v -> fp16 sub-tile [bn/2 x 64].
// Barriers that count MMA completions (A stage free, W^ slot free, accumulator full) exist in both CTAs
// and the leader commits to both; barriers the issuing thread waits on (A stage landed, W^ sub-tile
// built, accumulator drained) live in the leader and take arrivals from both CTAs.  No load uses
// cluster multicast.  Every wait is bounded by a poll limit passed in; a wait that runs out sets the
// status word, the role stops issuing work, and both CTAs still meet at the closing cluster barrier
// and free their tensor memory.
//
// Each output element is the fp32 sum over k in ascending order of 16-wide steps, whatever the tiling,
// so a row's result does not depend on M, on the slab width or on which kernel variant computed it.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include "ptx.cuh"
#include "codes.cuh"
#include "packed_gemm.cuh"
#include "gemm_ws.cuh"

namespace arcq {

struct PairParams {
  const uint8_t* pw;  // packed weight codes [N, pc]
  const float* mu_w;
  const float* sg_w;
  const float* cs_w;
  const float* cb_w;
  const float* bias;  // may be null
  void* y;            // [M, N] fp16 or fp32
  int M, N, K, G;
  int pc;          // packed bytes per weight row (K * bits / 8)
  int bn;          // slab width per pair: multiple of 32, <= 256, divides N
  int ws;          // W^ sub-tile slots per CTA (= G when stationary)
  int sa;          // A stages
  int ks;          // 64-wide K sub-tiles per A stage; divides G
  int nbb;         // 256-row tiles per batch (1, or 2 when the W^ ring streams)
  int stationary;  // 1: all G sub-tiles stay in shared memory for the CTA's lifetime
  int lut_shift;   // log2 of the number of side-by-side copies of the pair table (3..5)
  int y_f32;
  uint32_t poll_limit;  // sleeping waits give up after this many polls
  uint32_t spin_limit;  // the issuing thread's busy waits give up after this many probes
  int* status;
};

constexpr int kPairEpiWarps = 8;
constexpr int kPairProducerWarps = 8;
constexpr int kPairThreads = (2 + kPairEpiWarps + kPairProducerWarps) * 32;
constexpr int kPairProducerThreads = kPairProducerWarps * 32;
constexpr int kPairTileM = 256;
constexpr int kStatusPairTimeout = 0x301;
constexpr uint32_t kPairEpiStageBytes = kPairEpiWarps * 4096;   // two 2 KB blocks per epilogue warp

// ---------------------------------------------------------------- cluster helpers
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on an mbarrier anywhere in the cluster (address from mapa_shared)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Bounded waits on a barrier given by its 32-bit shared address; the limit is an argument.
__device__ __forceinline__ bool mbar_try_wait_a(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait_a(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_sleep_a(uint32_t bar, uint32_t parity, uint32_t limit, uint32_t ns) {
  if (mbar_try_wait_a(bar, parity)) return true;
  for (uint32_t i = 0; i < limit; ++i) {
    __nanosleep(ns);
    if (mbar_try_wait_a(bar, parity)) return true;
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait_spin_a(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_test_wait_a(bar, parity)) return true;
  }
  return false;
}

// Bounded waits that return a flag instead of steering control flow: the loop lives inside the asm block,
// the result (1 = phase completed, 0 = gave up after `limit` further probes) is data.  The issuing loops
// accumulate it and test it once per tile with a warp vote, so that their ring positions and descriptor
// words stay provably the same in every lane (the tensor-core and TMA instructions take them from the
// uniform datapath).
__device__ __forceinline__ uint32_t mbar_spin_flag(uint32_t bar, uint32_t parity, uint32_t limit) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .u32 i;\n\t"
      "mov.u32 i, 0;\n\t"
      "WAIT_%=:\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra DONE_%=;\n\t"
      "add.u32 i, i, 1;\n\t"
      "setp.lt.u32 q, i, %3;\n\t"
      "@q bra WAIT_%=;\n\t"
      "DONE_%=:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(limit)
      : "memory");
  return ok;
}
// Same with the suspending probe (try_wait parks the thread for a hardware-defined slice), for waits that
// are expected to last.
__device__ __forceinline__ uint32_t mbar_park_flag(uint32_t bar, uint32_t parity, uint32_t limit) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .u32 i;\n\t"
      "mov.u32 i, 0;\n\t"
      "WAIT_%=:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra DONE_%=;\n\t"
      "add.u32 i, i, 1;\n\t"
      "setp.lt.u32 q, i, %3;\n\t"
      "@q bra WAIT_%=;\n\t"
      "DONE_%=:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(limit)
      : "memory");
  return ok;
}

// ---------------------------------------------------------------- pair-wide tcgen05 / TMA
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 2-D tile load into this CTA's shared memory (32-bit shared address) whose completion bytes are counted on
// an mbarrier that may live in the other CTA of the pair (`bar_cluster_addr` from mapa_shared).  Not a
// multicast: one destination, one barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const void* tmap, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_if(uint32_t go, uint32_t smem_dst, const void* tmap,
                                                    uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];\n\t}" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(go)
      : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// High word of the shared-memory operand descriptor (128-byte swizzle, 8-row groups 1024 bytes apart,
// descriptor version 1); the low word is (address >> 4) | 1 << 16.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
// D[tmem of both CTAs] (+)= A . B^T over the pair, issued by one lane (`leader` != 0) of a converged warp.
// Operands are the low words of the two descriptors; `kstep` (0..3) selects the 16-wide K slice.
template <int KSTEP>
__device__ __forceinline__ void umma_pair_f16_lo(uint32_t leader, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b32 al, bl;\n\t.reg .b64 da, db;\n\t"
      "add.u32 al, %1, %7;\n\t"
      "add.u32 bl, %2, %7;\n\t"
      "mov.b64 da, {al, %6};\n\t"
      "mov.b64 db, {bl, %6};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(leader), "r"(kDescHi), "n"(2 * KSTEP)
      : "memory");
}
// One lane of the (converged) warp, chosen by the hardware; the compiler knows the guarded code runs in a
// single thread.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}
// The four 16-wide K steps of one 64-wide sub-tile, unpredicated (for code already running in one thread).
__device__ __forceinline__ void umma_pair_f16_x4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b32 al, bl;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n\t"
      "add.u32 al, %1, 2;\n\tadd.u32 bl, %2, 2;\n\tmov.b64 da, {al, %5};\n\tmov.b64 db, {bl, %5};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, 1;\n\t"
      "add.u32 al, %1, 4;\n\tadd.u32 bl, %2, 4;\n\tmov.b64 da, {al, %5};\n\tmov.b64 db, {bl, %5};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, 1;\n\t"
      "add.u32 al, %1, 6;\n\tadd.u32 bl, %2, 6;\n\tmov.b64 da, {al, %5};\n\tmov.b64 db, {bl, %5};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, 1;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi)
      : "memory");
}
__device__ __forceinline__ void umma_pair_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}
// One arrival on the barrier at `bar_cluster_addr` (this CTA's or the peer's) once every MMA issued so far
// by this thread has completed.
__device__ __forceinline__ void umma_pair_commit_if(uint32_t leader, uint32_t bar_cluster_addr) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar_cluster_addr),
      "r"(leader)
      : "memory");
}

// ---------------------------------------------------------------- shared-memory plan (per CTA)
struct PairSmem {
  uint32_t a, w, stage, fold, misc, lut2;
  uint32_t total;
};
constexpr int kPairBarriers = 80;
__host__ __device__ inline PairSmem pair_smem_layout(int bn, int ws, int sa, int ks, int G, bool stationary,
                                                     int lut_shift) {
  const int hb = bn / 2;
  PairSmem s;
  s.a = 0;
  s.w = s.a + static_cast<uint32_t>(sa) * ks * kStageA;
  const uint32_t area = s.w + static_cast<uint32_t>(ws) * hb * 128;
  const uint32_t fold_bytes = (static_cast<uint32_t>(hb) * G * 4u + 127) & ~127u;
  uint32_t area_bytes;
  s.stage = area;
  if (stationary) {
    // the slab is built once, before the first accumulator is complete: the folded statistics share their
    // bytes with the epilogue's staging blocks
    s.fold = area;
    area_bytes = fold_bytes > kPairEpiStageBytes ? fold_bytes : kPairEpiStageBytes;
  } else {
    s.fold = s.stage + kPairEpiStageBytes;
    area_bytes = kPairEpiStageBytes + fold_bytes;
  }
  s.misc = area + area_bytes;
  s.lut2 = s.misc + 256 * 4 /*bias*/ + kPairBarriers * 8 + 16 /*tensor-memory address*/;
  s.total = s.lut2 + ((256u * 4u) << lut_shift);
  return s;
}

constexpr int kPairJobBlock = 3;   // weight sub-tiles whose packed codes a producer thread holds in registers at once
constexpr int kPairMaxUnits = 3;   // (row, 16-byte chunk) units of one sub-tile per producer thread: bn/2 <= 96 rows
constexpr int kPairMaxBn = 64 * kPairMaxUnits;   // widest slab

// What a weight-building thread needs to know (all values are the same for every thread of the CTA).
struct PairBuildCtx {
  const uint8_t* wrow;     // packed codes of the first weight row of this CTA's half slab
  long long pc;            // packed bytes per weight row
  uint8_t* sW;             // sub-tile slots
  const uint32_t* s_fold;  // half2 (sigma, mu') per (row, group)
  const uint32_t* s_lut2;  // pair table
  uint32_t wtile_bytes, lut_shift, w_full_leader, w_empty, poll_limit;
  int G, hb, ws, n_builders;
  bool stationary;
};

// Rebuild the sub-tiles of jobs first, first + stride, ... (< n_jobs; job j is group j % G) with the 256 threads
// of one builder group (`bt` = thread index in the group).  Packed codes come straight from global memory
// (a few KB per CTA, resident in L2): each thread loads the code words of its units for a block of jobs ahead
// of time into registers, two blocks in flight, so the rebuild never waits for a load it has just issued.
// `sync_first`: meet the CTA's other builder threads first (pair table and statistics complete).
// Returns false if a bounded wait ran out.
template <int BITS>
__device__ __forceinline__ bool pair_build_jobs(const PairBuildCtx& c, int bt, int lane, int first, int stride,
                                                int n_jobs, bool sync_first) {
  const int chunk = bt & 7, r_base = bt >> 3;   // unit i of a sub-tile: row r_base + 32*i, 16-byte chunk `chunk`
  const uint32_t lut_mask = (1u << c.lut_shift) - 1u;
  const uint8_t* const wrow0 = c.wrow + r_base * c.pc;
  const long long row_step = 32LL * c.pc;
  // code words of one block of jobs: c0 (and c1 for 3-bit codes, whose 24 bits may straddle two words)
  uint32_t ca0[kPairJobBlock][kPairMaxUnits], ca1[kPairJobBlock][kPairMaxUnits];
  uint32_t cb0[kPairJobBlock][kPairMaxUnits], cb1[kPairJobBlock][kPairMaxUnits];
  bool ok = true;
  auto load_block = [&](int j0, uint32_t (&c0)[kPairJobBlock][kPairMaxUnits], uint32_t (&c1)[kPairJobBlock][kPairMaxUnits]) {
#pragma unroll
    for (int jj = 0; jj < kPairJobBlock; ++jj) {
      const int j = j0 + jj * stride;
      if (j < n_jobs) {
        const int g = j % c.G;
#pragma unroll
        for (int i = 0; i < kPairMaxUnits; ++i) {
          c0[jj][i] = 0u;
          c1[jj][i] = 0u;
          if (r_base + 32 * i < c.hb) {
            const uint8_t* rp = wrow0 + i * row_step + g * (8 * BITS);
            if (BITS == 4) {
              c0[jj][i] = __ldg(reinterpret_cast<const uint32_t*>(rp) + chunk);
            } else if (BITS == 3) {
              const int off = 3 * chunk, al = off & ~3;
              c0[jj][i] = __ldg(reinterpret_cast<const uint32_t*>(rp + al));
              if ((off & 3) >= 2) c1[jj][i] = __ldg(reinterpret_cast<const uint32_t*>(rp + al + 4));   // inside the group
            } else {
              c0[jj][i] = __ldg(reinterpret_cast<const uint16_t*>(rp) + chunk);
            }
          }
        }
      }
    }
  };
  auto build_block = [&](int j0, uint32_t (&c0)[kPairJobBlock][kPairMaxUnits], uint32_t (&c1)[kPairJobBlock][kPairMaxUnits]) {
#pragma unroll
    for (int jj = 0; jj < kPairJobBlock; ++jj) {
      const int j = j0 + jj * stride;
      if (j >= n_jobs || !ok) break;
      const int g = j % c.G;
      // ring: job j uses slot j % ws for the (j / ws)-th time; its first use needs no wait
      const uint32_t wslot = c.stationary ? static_cast<uint32_t>(g) : static_cast<uint32_t>(j % c.ws);
      if (!c.stationary && !mbar_wait_sleep_a(c.w_empty + wslot * 8, ((static_cast<uint32_t>(j / c.ws) & 1u) ^ 1u), c.poll_limit, 64)) {
        ok = false;
        break;
      }
      uint8_t* const dstw = c.sW + wslot * c.wtile_bytes;
#pragma unroll
      for (int i = 0; i < kPairMaxUnits; ++i) {
        const int r = r_base + 32 * i;
        if (r < c.hb) {
          uint32_t w;
          if (BITS == 4) {
            w = c0[jj][i];
          } else if (BITS == 3) {
            w = spread_3_to_nibbles(__funnelshift_r(c0[jj][i], c1[jj][i], ((3 * chunk) & 3) * 8) & 0xFFFFFFu);
          } else {
            w = spread_2_to_nibbles(c0[jj][i]);
          }
          // mu' + sigma * cb[code] for two codes at a time: one pair-table look-up per byte of nibbles and one
          // half2 fused multiply-add
          const uint32_t fw = c.s_fold[r * c.G + g];
          const __half2 f2 = *reinterpret_cast<const __half2*>(&fw);
          const __half2 s2 = __low2half2(f2);
          const __half2 m2 = __high2half2(f2);
          uint32_t h[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t pv = c.s_lut2[(((w >> (8 * q)) & 0xFFu) << c.lut_shift) + (static_cast<uint32_t>(lane) & lut_mask)];
            const __half2 r2 = __hfma2(s2, *reinterpret_cast<const __half2*>(&pv), m2);
            h[q] = *reinterpret_cast<const uint32_t*>(&r2);
          }
          *reinterpret_cast<uint4*>(dstw + sw128_offset(r, chunk)) = make_uint4(h[0], h[1], h[2], h[3]);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(c.w_full_leader + wslot * 8);
    }
  };
  const int blk = kPairJobBlock * stride;
  load_block(first, ca0, ca1);
  load_block(first + blk, cb0, cb1);
  // the pair table and the folded statistics are complete (all builder threads of the CTA)
  if (sync_first) asm volatile("bar.sync 1, %0;" ::"r"(c.n_builders) : "memory");
  for (int j0 = first; j0 < n_jobs && ok; j0 += 2 * blk) {
    build_block(j0, ca0, ca1);
    load_block(j0 + 2 * blk, ca0, ca1);
    build_block(j0 + blk, cb0, cb1);
    load_block(j0 + 3 * blk, cb0, cb1);
  }
  return ok;
}

template <int BITS, bool STATIONARY>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
packed_weight_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_y,
                               const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* const smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const PairSmem L = pair_smem_layout(p.bn, p.ws, p.sa, p.ks, p.G, STATIONARY, p.lut_shift);
  uint8_t* const sA = smem + L.a;
  uint8_t* const sW = smem + L.w;
  uint8_t* const sStage = smem + L.stage;
  float* const s_bias = reinterpret_cast<float*>(smem + L.misc);
  uint64_t* const bars = reinterpret_cast<uint64_t*>(s_bias + 256);
  // barrier groups (index into `bars`):  a_full [sa] <= 8 at 0 (leader: A stage landed, bytes of both CTAs);
  // a_empty [sa] at 8 (both: the MMAs that read the stage are done);  w_full [ws] <= 32 at 16 (leader: sub-tile
  // built in both CTAs);  w_empty [ws] <= 16 at 48 (both: ring slot may be rebuilt);  acc_full [2] at 64 (both:
  // accumulator complete);  acc_empty [2] at 66 (leader: accumulator drained by both CTAs)
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t a_full = bar0, a_empty = bar0 + 8 * 8, w_full = bar0 + 16 * 8, w_empty = bar0 + 48 * 8;
  const uint32_t acc_full = bar0 + 64 * 8, acc_empty = bar0 + 66 * 8;
  uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(bars + kPairBarriers);
  uint32_t* const s_lut2 = reinterpret_cast<uint32_t*>(smem + L.lut2);
  uint32_t* const s_fold = reinterpret_cast<uint32_t*>(smem + L.fold);

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
  const int nh0 = n0 + crank * hb;     // first W^ row this CTA rebuilds
  // pairs of different slabs that share a rank walk the same row tiles; stagger their starting points
  const int rot = (my_tiles > 0) ? (slab * my_tiles) / n_slabs : 0;
  // first row of this CTA's half of the t-th tile the pair works on
  auto row_of = [&](int t) {
    int q = t + rot;
    if (q >= my_tiles) q -= my_tiles;
    return (rank + q * pairs_in_slab) * kPairTileM + static_cast<int>(crank) * kTileM;
  };
  const int nbb = p.nbb;
  constexpr bool stationary = STATIONARY;
  const uint32_t poll_limit = p.poll_limit, spin_limit = p.spin_limit;
  const uint32_t stage_bytes = static_cast<uint32_t>(ks) * kStageA;
  const uint32_t wtile_bytes = static_cast<uint32_t>(hb) * 128u;

  // Let the next kernel of the stream start its own set-up while this one runs (no effect unless that kernel
  // was launched as a programmatic dependent).
  pdl_launch_dependents();
  if (tid == 0) {
    for (int i = 0; i < p.sa; ++i) { mbar_init(&bars[i], 1); mbar_init(&bars[8 + i], 1); }
    for (int i = 0; i < p.ws; ++i) mbar_init(&bars[16 + i], 2 * kPairProducerWarps);
    if (!stationary)
      for (int i = 0; i < p.ws; ++i) mbar_init(&bars[48 + i], 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[64 + i], 1); mbar_init(&bars[66 + i], 2 * kPairEpiWarps); }
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
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
    // ------------------------------------------------------------------ TMA: this CTA's half of every A tile
    // The whole warp walks the loop and waits; lane 0 arms the barrier and issues the copies.
    const uint32_t sa = p.sa;
    const uint32_t a_full_leader = mapa_shared(a_full, 0);
    const uint32_t sa0 = smem_u32(sA);
    uint32_t slot = 0, ph = 1;     // "empty" barriers: the first pass is free
    uint32_t good = 1;             // 0 once a wait has run out (later waits then give up at once)
    // Everything above (and the whole weight rebuild) reads only this layer's constants.  The activation is
    // the previous kernel's output: when launched as a programmatic dependent, wait for that kernel here.
    pdl_wait();
    for (int b0 = 0; b0 < my_tiles; b0 += nbb) {
      const int nb = min(nbb, my_tiles - b0);
      const int row0 = row_of(b0), row1 = (nb > 1) ? row_of(b0 + 1) : 0;
      for (int g0 = 0; g0 < G; g0 += ks) {
        for (int j = 0; j < nb; ++j) {
          good &= mbar_park_flag(a_empty + slot * 8, ph, good ? poll_limit : 0u);
          if (elect_one()) {
            if (good) {
              if (crank == 0) mbar_expect_tx(a_full + slot * 8, 2u * stage_bytes);
              const uint32_t dst = sa0 + slot * stage_bytes;
              for (int q = 0; q < ks; ++q)
                tma_load_2d_pair(dst + q * kStageA, &tm_a, a_full_leader + slot * 8, (g0 + q) * 64, j ? row1 : row0);
            }
          }
          __syncwarp();
          if (++slot == sa) { slot = 0; ph ^= 1; }
        }
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
    // All lanes wait and keep the ring positions, lane 0 issues.  The per-stage code is kept as short as it
    // can be: a lone warp executes its instructions one dependent step at a time, and every instruction
    // here is on the critical path of two SMs' tensor pipes.
    if (crank == 0 && my_tiles > 0) {
      const uint32_t idesc = umma_idesc_f16(kPairTileM, bn);
      const uint32_t sa = p.sa, wsn = p.ws;
      const uint32_t a_lo0 = ((smem_u32(sA) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t w_lo0 = ((smem_u32(sW) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t a_step = stage_bytes >> 4, w_step = wtile_bytes >> 4;
      const uint32_t a_empty_r = mapa_shared(a_empty, 1), w_empty_r = mapa_shared(w_empty, 1);
      const uint32_t acc_full_r = mapa_shared(acc_full, 1);
      uint32_t slot = 0, ph = 0, a_lo = a_lo0;
      uint32_t acc_ph0 = 1, acc_ph1 = 1;   // acc_empty phases: the first use of each buffer is free
      uint32_t buf = 0;
      uint32_t good = 1;   // 0 once a wait has run out: later waits give up at once, nothing more is issued
      if (stationary) {
        for (int t = 0; t < my_tiles; ++t) {
          good &= mbar_park_flag(acc_empty + buf * 8, buf ? acc_ph1 : acc_ph0, good ? poll_limit : 0u);
          acc_ph0 ^= buf ? 0u : 1u;
          acc_ph1 ^= buf ? 1u : 0u;
          tc_fence_after_sync();
          const uint32_t d = tmem_base + buf * 256;
          uint32_t w_lo = w_lo0, acc = 0;
          for (int g0 = 0; g0 < G; g0 += ks) {
            if (t == 0) {   // the slab is being built while the first tile runs
              for (int q = 0; q < ks; ++q) good &= mbar_spin_flag(w_full + (g0 + q) * 8, 0u, good ? spin_limit : 0u);
            }
            good &= mbar_spin_flag(a_full + slot * 8, ph, good ? spin_limit : 0u);
            if (elect_one()) {
              if (good) {
                uint32_t al = a_lo, wl = w_lo;
                for (int q = 0; q < ks; ++q) {
                  umma_pair_f16_x4(d, al, wl, idesc, (q == 0) ? acc : 1u);
                  al += kStageA >> 4;
                  wl += w_step;
                }
                umma_pair_commit(a_empty + slot * 8);
                umma_pair_commit(a_empty_r + slot * 8);
                if (g0 + ks >= G) {
                  umma_pair_commit(acc_full + buf * 8);
                  umma_pair_commit(acc_full_r + buf * 8);
                }
              }
            }
            __syncwarp();
            acc = 1u;
            w_lo += ks * w_step;
            a_lo += a_step;
            if (++slot == sa) { slot = 0; ph ^= 1; a_lo = a_lo0; }
          }
          buf ^= 1;
          if (__any_sync(0xffffffffu, good == 0)) break;
        }
      } else {
        uint32_t w_slot = 0, w_ph = 0;
        for (int b0 = 0; b0 < my_tiles; b0 += nbb) {
          const int nb = min(nbb, my_tiles - b0);
          const uint32_t buf0 = buf;
          for (int j = 0; j < nb; ++j) {
            const uint32_t bj = (buf0 + j) & 1;
            good &= mbar_park_flag(acc_empty + bj * 8, bj ? acc_ph1 : acc_ph0, good ? poll_limit : 0u);
            acc_ph0 ^= bj ? 0u : 1u;
            acc_ph1 ^= bj ? 1u : 0u;
          }
          tc_fence_after_sync();
          uint32_t acc = 0;
          for (int g0 = 0; g0 < G; g0 += ks) {
            // ks consecutive ring slots (ks divides the ring size, so they do not wrap inside a stage)
            for (int q = 0; q < ks; ++q) good &= mbar_spin_flag(w_full + (w_slot + q) * 8, w_ph, good ? spin_limit : 0u);
            for (int j = 0; j < nb; ++j) {
              good &= mbar_spin_flag(a_full + slot * 8, ph, good ? spin_limit : 0u);
              const uint32_t d = tmem_base + ((buf0 + j) & 1) * 256;
              if (elect_one()) {
                if (good) {
                  uint32_t al = a_lo, wl = w_lo0 + w_slot * w_step;
                  for (int q = 0; q < ks; ++q) {
                    umma_pair_f16_x4(d, al, wl, idesc, (q == 0) ? acc : 1u);
                    al += kStageA >> 4;
                    wl += w_step;
                  }
                  umma_pair_commit(a_empty + slot * 8);
                  umma_pair_commit(a_empty_r + slot * 8);
                  if (j == nb - 1) {
                    for (int q = 0; q < ks; ++q) {
                      umma_pair_commit(w_empty + (w_slot + q) * 8);
                      umma_pair_commit(w_empty_r + (w_slot + q) * 8);
                    }
                  }
                  if (g0 + ks >= G) {
                    umma_pair_commit(acc_full + ((buf0 + j) & 1) * 8);
                    umma_pair_commit(acc_full_r + ((buf0 + j) & 1) * 8);
                  }
                }
              }
              __syncwarp();
              a_lo += a_step;
              if (++slot == sa) { slot = 0; ph ^= 1; a_lo = a_lo0; }
            }
            acc = 1u;
            w_slot += ks;
            if (w_slot == wsn) { w_slot = 0; w_ph ^= 1; }
          }
          buf = (buf0 + nb) & 1;
          if (__any_sync(0xffffffffu, good == 0)) break;
        }
      }
      ok = __all_sync(0xffffffffu, good != 0);
      __syncwarp();
      if (!ok && lane == 0) atomicExch(p.status, kStatusPairTimeout);
    }
  } else {
    // ------------------------------------------------------------------ builders / epilogue
    // Warps 2-9 drain the accumulators, warps 10-17 rebuild the weight.  A stationary slab is built once, at a
    // time when the epilogue warps have nothing to do yet, so there both groups build (alternate sub-tiles).
    const bool is_epi = warp < 2 + kPairEpiWarps;
    const int bt = is_epi ? tid - 2 * 32 : tid - (2 + kPairEpiWarps) * 32;   // thread index within its group
    const int n_builders = 2 * kPairProducerThreads;
    if (is_epi)
      for (int i = bt; i < bn; i += kPairEpiWarps * 32) s_bias[i] = (p.bias != nullptr) ? __ldg(p.bias + n0 + i) : 0.0f;
    PairBuildCtx c = {};
    const int fills = stationary ? 1 : (my_tiles + nbb - 1) / nbb;   // how many times the slab is walked
    if (my_tiles > 0) {
      const int bid = is_epi ? kPairProducerThreads + bt : bt;    // thread index among all builders
      // Pair table (codebook values of the low and high nibble of a byte, several copies side by side) and folded
      // statistics of the half slab (half2 (sigma, mu - sigma*code_sum/64) per (row, group)).  All global loads
      // of a thread are issued before any of their results is used, so their latencies overlap.
      const int lo = bid & 15, hi = (bid >> 4) & 15;
      const float cb_lo = (bid < 256 && lo < (1 << BITS)) ? __ldg(p.cb_w + lo) : 0.0f;
      const float cb_hi = (bid < 256 && hi < (1 << BITS)) ? __ldg(p.cb_w + hi) : 0.0f;
      const long long base = static_cast<long long>(nh0) * G;
      const int n_fold = hb * G;
      float sg[4], cs[4], mu[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = bid + u * n_builders;
        const bool in = i < n_fold;
        sg[u] = in ? __ldg(p.sg_w + base + i) : 0.0f;
        cs[u] = in ? __ldg(p.cs_w + base + i) : 0.0f;
        mu[u] = in ? __ldg(p.mu_w + base + i) : 0.0f;
      }
      if (bid < 256) {
        const __half2 v = __floats2half2_rn(cb_lo, cb_hi);
        for (uint32_t cp = 0; cp < (1u << p.lut_shift); ++cp)
          s_lut2[(static_cast<uint32_t>(bid) << p.lut_shift) + cp] = *reinterpret_cast<const uint32_t*>(&v);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = bid + u * n_builders;
        if (i < n_fold) {
          const __half2 f2 = __floats2half2_rn(sg[u], fmaf(-sg[u], cs[u] * (1.0f / 64.0f), mu[u]));
          s_fold[i] = *reinterpret_cast<const uint32_t*>(&f2);
        }
      }
      for (int i = bid + 4 * n_builders; i < n_fold; i += n_builders) {      // long slabs: the rest, one at a time
        const float sgi = __ldg(p.sg_w + base + i);
        const __half2 f2 = __floats2half2_rn(sgi, fmaf(-sgi, __ldg(p.cs_w + base + i) * (1.0f / 64.0f), __ldg(p.mu_w + base + i)));
        s_fold[i] = *reinterpret_cast<const uint32_t*>(&f2);
      }
      c.wrow = p.pw + static_cast<long long>(nh0) * p.pc;
      c.pc = p.pc;
      c.sW = sW;
      c.s_fold = s_fold;
      c.s_lut2 = s_lut2;
      c.wtile_bytes = wtile_bytes;
      c.lut_shift = static_cast<uint32_t>(p.lut_shift);
      c.w_full_leader = mapa_shared(w_full, 0);
      c.w_empty = w_empty;
      c.poll_limit = poll_limit;
      c.G = G; c.hb = hb; c.ws = p.ws; c.n_builders = n_builders;
      c.stationary = stationary;
      // A slab that is walked once (stationary, or a streaming ring with a single batch of tiles) is built while
      // the epilogue warps have nothing to drain yet: the two groups alternate on its sub-tiles (each sub-tile is
      // still the work of eight warps).  A ring that is walked several times is rebuilt by the weight warps alone.
      if (stationary || fills == 1) ok = pair_build_jobs<BITS>(c, bt, lane, is_epi ? 1 : 0, 2, fills * G, true);
      else if (!is_epi) ok = pair_build_jobs<BITS>(c, bt, lane, 0, 1, fills * G, true);
      else asm volatile("bar.sync 1, %0;" ::"r"(n_builders) : "memory");   // only orders the table fill above
    }
    if (is_epi) {
      // ---------------------------------------------------------------- epilogue (own 128 rows of each tile)
      // Eight warps: two per tensor-memory lane quarter, taking alternate column steps of 64 bytes per row.
      // A step goes registers -> + bias -> fp16/fp32 -> one of this warp's two 2 KB staging blocks (64-byte
      // swizzle, conflict-free 16-byte stores) -> one TMA store.
      const int ew = warp - 2;
      asm volatile("bar.sync 2, %0;" ::"n"(kPairEpiWarps * 32) : "memory");   // bias table complete
      const int lq = warp & 3;                          // tensor-memory lane quarter this warp may read
      const int half_id = ew >> 2;                      // which of the two warps of the quarter
      const uint32_t acc_empty_leader = mapa_shared(acc_empty, 0);
      uint8_t* const stg = sStage + ew * 4096;
      const int cw = p.y_f32 ? 16 : 32;
      const bool f32 = p.y_f32 != 0;
      uint32_t blk = 0;      // staging block of the next store; the two blocks alternate from store to store
      auto emit = [&](const uint32_t (&acc)[32], int c0, int row0) {
        if (lane == 0) tma_store_wait_read_1();      // the store issued two stores ago has read this block
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
        blk ^= 1;
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
        // The tensor-memory reads of this warp's column steps run one step ahead of the conversion, and the
        // accumulator is handed back as soon as the last read has landed, before its values are converted.
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
    }
    if (!ok && lane == 0) atomicExch(p.status, kStatusPairTimeout);
  }

  // Both CTAs stay until the other is done: the leader's MMAs read the peer's shared memory and signal its
  // barriers, the peer's warps arrive on the leader's barriers.
  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 0) tmem_dealloc_pair(tmem_base, 512);
}

}  // namespace arcq
