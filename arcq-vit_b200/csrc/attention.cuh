// Multi-head self-attention for short sequences (ViT: 197 tokens, head width 64), optionally fused with the
// activation quantizer of the projection that consumes its output.
//   qkv  [B*T, 3*H*64] fp16: the output of the packed qkv linear (q | k | v, each H heads of 64)
//   out  [B*T, H*64] fp16:   softmax(q k^T / 8) v, heads side by side (the layout timm's Attention feeds to proj)
//   or   xhat [B*T, H*64] fp16: the ARCQ reconstruction of that matrix in groups of 64.  A head's 64 outputs of a
//        token are exactly one quantizer group, so the quantizer needs nothing beyond the registers that hold them.
//
// One CTA per (image, head), seven warps.  K and V of the head (T x 64 each) are staged once in shared memory
// (16-byte cp.async, XOR-swizzled rows so that ldmatrix is conflict-free); each warp owns 16-row blocks of queries
// and walks the keys in blocks of 64 with an online softmax: S = Q K^T on mma.sync.m16n8k16 (fp32 accumulate), row
// maxima and sums in fp32, P rounded to fp16 and fed straight from the accumulator registers into the second
// product O += P V -- the sequence never leaves registers.  The whole problem is 2 x 197 x 197 x 64 flops per head:
// too small for a 128-row tensor-memory tile to pay (two thirds of a second tile would be padding), and the kernel is
// bound by its latency chain, not by the tensor pipe.
//
// Quantizer epilogue: same arithmetic as the quantizer kernels (act_quant_v2.cuh), on the fp16-rounded outputs, so
// the result is bit-identical to quantising the matrix the plain form of this kernel writes.  A row's 64 values
// sit in four lanes (lane%4 = q holds columns 8n+2q, 8n+2q+1, n = 0..7): the reference's lane sums
//   v[l] = ((x[l]+x[32+l]) + (x[8+l]+x[40+l])) + (x[16+l]+x[48+l])) + (x[24+l]+x[56+l])   for l = 2q, 2q+1
// are thread-local, and the closing chain ((((((v0+v1)+v2)+v3)+v4)+v5)+v6)+v7 is evaluated by every lane on the
// eight values gathered with shuffles.
#pragma once
#include <cuda_fp16.h>
#include "ptx.cuh"
#include "act_quant_v2.cuh"

namespace arcq {

constexpr int kAttnWarps = 7;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kAttnMaxT = 256;

struct AttnParams {
  const __half* qkv;
  __half* out;
  int B, T, H;
  int tp;                      // T rounded up to 16: rows of K / V held in shared memory
  const float* thresholds;     // quantizer form only
  const float* codebook;
};

__host__ __device__ constexpr size_t attn_smem_bytes(int tp) {
  return static_cast<size_t>(2) * tp * 128 + kAttnWarps * 2048 + 3 * 16 * 4;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D (16x8, fp32) += A (16x16, fp16, row) . B (16x8, fp16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// The reference's closing chain over the eight lane sums of a row; lane q of the row's four lanes holds
// (v_even, v_odd) = (v[2q], v[2q+1]).  Every lane returns the same value.
__device__ __forceinline__ float row_chain_sum(float v_even, float v_odd, int lane) {
  const int base = lane & ~3;
  float s = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float e = __shfl_sync(0xffffffffu, v_even, base + j);
    const float o = __shfl_sync(0xffffffffu, v_odd, base + j);
    s = (j == 0) ? __fadd_rn(e, o) : __fadd_rn(__fadd_rn(s, e), o);
  }
  return s;
}
// lane sums v[2q], v[2q+1] of one row from its 16 thread-local values x[2n], x[2n+1] = columns 8n+2q, 8n+2q+1
__device__ __forceinline__ void lane_sums(const float (&x)[16], float& v_even, float& v_odd) {
  // l = 2q:   a0 = x[l] + x[32+l] -> n = 0, 4;  a1 -> n = 1, 5;  a2 -> n = 2, 6;  a3 -> n = 3, 7
  v_even = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(x[0], x[8]), __fadd_rn(x[2], x[10])), __fadd_rn(x[4], x[12])), __fadd_rn(x[6], x[14]));
  v_odd = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(x[1], x[9]), __fadd_rn(x[3], x[11])), __fadd_rn(x[5], x[13])), __fadd_rn(x[7], x[15]));
}

template <bool QUANT, int BITS>
__global__ void __launch_bounds__(kAttnThreads, 2) attention_kernel(const AttnParams p) {
  pdl_launch_dependents();
  constexpr int L = 1 << BITS;
  extern __shared__ __align__(128) uint8_t attn_smem[];
  const int tp = p.tp, T = p.T, C = p.H * 64;
  uint8_t* const sK = attn_smem;
  uint8_t* const sV = sK + tp * 128;
  uint8_t* const sStage = sV + tp * 128;
  float* const s_th = reinterpret_cast<float*>(sStage + kAttnWarps * 2048);   // [16] thresholds, +inf padded
  float* const s_h = s_th + 16;                                               // [16] half-gaps to the next float
  float* const s_cb = s_h + 16;                                               // [16] codebook
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x / p.H, h = blockIdx.x - b * p.H;
  const __half* const base = p.qkv + static_cast<long long>(b) * T * (3 * C) + h * 64;

  int my_exact = 1;
  if (QUANT) {
    if (tid < 16) {
      float th = __int_as_float(0x7f800000), hg = 0.0f;
      if (tid < L - 1) {
        th = p.thresholds[tid];
        if (th == 0.0f) {
          hg = 0x1p-100f;
        } else {
          const int bi = __float_as_int(th);
          const float up = __int_as_float(th > 0.0f ? bi + 1 : bi - 1);
          hg = __fmul_rn(__fsub_rn(up, th), 0.5f);
        }
        my_exact = (th == 0.0f || fabsf(th) > 1.0e-15f) ? 1 : 0;
      }
      s_th[tid] = th;
      s_h[tid] = hg;
      s_cb[tid] = tid < L ? p.codebook[tid] : 0.0f;
    }
  }

  pdl_wait();                // qkv is the previous kernel's output
  // ---- K and V of this head into shared memory: row r at r*128, 16-byte chunk c at ((c ^ (r & 7)) * 16)
  {
    const uint32_t k0 = smem_u32(sK), v0 = smem_u32(sV);
    for (int i = tid; i < tp * 8; i += kAttnThreads) {
      const int r = i >> 3, c = i & 7;
      const uint32_t off = r * 128 + ((c ^ (r & 7)) << 4);
      if (r < T) {
        const __half* src = base + static_cast<long long>(r) * (3 * C) + c * 8;
        cp_async16(k0 + off, src + C);
        cp_async16(v0 + off, src + 2 * C);
      } else {
        *reinterpret_cast<uint4*>(sK + off) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(sV + off) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  }
  const bool exact_r = QUANT ? (__syncthreads_and(my_exact) != 0) : true;
  cp_async_wait<0>();
  __syncthreads();

  const int q4 = lane & 3, r8 = lane >> 2;
  const float c_exp = 0.125f * 1.4426950408889634f;      // 1/sqrt(64) * log2(e)
  const uint32_t sK0 = smem_u32(sK), sV0 = smem_u32(sV);
  const int n_row_blocks = tp >> 4;
  const int key_blocks = (tp + 63) >> 6;

  for (int rb = warp; rb < n_row_blocks; rb += kAttnWarps) {
    // ---- Q fragments of this warp's 16 rows (rows beyond T shadow the last row; they are not stored)
    uint32_t qa[4][4];
    {
      const int row_lo = min(rb * 16 + r8, T - 1), row_hi = min(rb * 16 + r8 + 8, T - 1);
      const uint32_t* q_lo = reinterpret_cast<const uint32_t*>(base + static_cast<long long>(row_lo) * (3 * C));
      const uint32_t* q_hi = reinterpret_cast<const uint32_t*>(base + static_cast<long long>(row_hi) * (3 * C));
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        qa[ks][0] = __ldg(q_lo + ks * 8 + q4);
        qa[ks][1] = __ldg(q_hi + ks * 8 + q4);
        qa[ks][2] = __ldg(q_lo + ks * 8 + 4 + q4);
        qa[ks][3] = __ldg(q_hi + ks * 8 + 4 + q4);
      }
    }
    float o[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

    for (int kb = 0; kb < key_blocks; ++kb) {
      const int key0 = kb * 64;
      const int nb16 = min(4, (tp - key0) >> 4);          // 16-key steps in this block
      float s[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
      // S = Q K^T: B fragments by ldmatrix from K rows (keys), 16 keys x 16 d per instruction
      // (d step outermost: the eight products of a step go to eight different accumulators)
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          if (jj < nb16) {
            const int mi = lane >> 3, rr = lane & 7;
            const int key = key0 + jj * 16 + (mi >> 1) * 8 + rr;
            const int chunk = ks * 2 + (mi & 1);
            uint32_t kf[4];
            ldmatrix_x4(sK0 + key * 128 + ((chunk ^ (key & 7)) << 4), kf);
            mma_16816(s[2 * jj], qa[ks], kf[0], kf[1]);
            mma_16816(s[2 * jj + 1], qa[ks], kf[2], kf[3]);
          }
        }
      }
      // mask keys beyond T (only the last block can have them), row maxima
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = key0 + j * 8 + 2 * q4;
        if (j >= 2 * nb16 || col >= T) { s[j][0] = -INFINITY; s[j][2] = -INFINITY; }
        if (j >= 2 * nb16 || col + 1 >= T) { s[j][1] = -INFINITY; s[j][3] = -INFINITY; }
        mx_lo = fmaxf(mx_lo, fmaxf(s[j][0], s[j][1]));
        mx_hi = fmaxf(mx_hi, fmaxf(s[j][2], s[j][3]));
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);     // finite: key 0 is never masked
      const float al_lo = exp2f((m_lo - mn_lo) * c_exp), al_hi = exp2f((m_hi - mn_hi) * c_exp);
      m_lo = mn_lo;
      m_hi = mn_hi;
      l_lo *= al_lo;
      l_hi *= al_hi;
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j][0] *= al_lo; o[j][1] *= al_lo; o[j][2] *= al_hi; o[j][3] *= al_hi; }
      const float ms_lo = m_lo * c_exp, ms_hi = m_hi * c_exp;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[j][0] = exp2f(fmaf(s[j][0], c_exp, -ms_lo));
        s[j][1] = exp2f(fmaf(s[j][1], c_exp, -ms_lo));
        s[j][2] = exp2f(fmaf(s[j][2], c_exp, -ms_hi));
        s[j][3] = exp2f(fmaf(s[j][3], c_exp, -ms_hi));
        l_lo += s[j][0] + s[j][1];
        l_hi += s[j][2] + s[j][3];
      }
      // O += P V: P from the accumulator registers, V fragments by transposing ldmatrix (16 keys x 16 d)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        if (jj < nb16) {
          uint32_t pa[4];
          pa[0] = pack_half2(s[2 * jj][0], s[2 * jj][1]);
          pa[1] = pack_half2(s[2 * jj][2], s[2 * jj][3]);
          pa[2] = pack_half2(s[2 * jj + 1][0], s[2 * jj + 1][1]);
          pa[3] = pack_half2(s[2 * jj + 1][2], s[2 * jj + 1][3]);
#pragma unroll
          for (int nn = 0; nn < 4; ++nn) {
            const int mi = lane >> 3, rr = lane & 7;
            const int key = key0 + jj * 16 + (mi & 1) * 8 + rr;
            const int chunk = nn * 2 + (mi >> 1);
            uint32_t vf[4];
            ldmatrix_x4_trans(sV0 + key * 128 + ((chunk ^ (key & 7)) << 4), vf);
            mma_16816(o[2 * nn], pa, vf[0], vf[1]);
            mma_16816(o[2 * nn + 1], pa, vf[2], vf[3]);
          }
        }
      }
    }
    // ---- normalise
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
    // the fp16 outputs: x_lo[2n], x_lo[2n+1] = columns 8n+2q, 8n+2q+1 of row r8; x_hi the same of row r8 + 8
    uint32_t w_lo[8], w_hi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      w_lo[j] = pack_half2(o[j][0] * inv_lo, o[j][1] * inv_lo);
      w_hi[j] = pack_half2(o[j][2] * inv_hi, o[j][3] * inv_hi);
    }
    if (QUANT) {
#pragma unroll
      for (int half_id = 0; half_id < 2; ++half_id) {
        uint32_t (&w)[8] = half_id ? w_hi : w_lo;
        float x[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
          x[2 * j] = f.x;
          x[2 * j + 1] = f.y;
        }
        float ve, vo;
        lane_sums(x, ve, vo);
        const float mean = __fdiv_rn(row_chain_sum(ve, vo, lane), 64.0f);
        float sq[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          x[i] = __fsub_rn(x[i], mean);
          sq[i] = __fmul_rn(x[i], x[i]);
        }
        lane_sums(sq, ve, vo);
        const float var = __fdiv_rn(row_chain_sum(ve, vo, lane), 64.0f);
        const float scale = __fsqrt_rn(__fadd_rn(var, 1.0e-6f));
        // codes: number of thresholds below r / scale, by the exact division-free test (or the IEEE quotient
        // for thresholds too close to zero), then the codebook value
        int code[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) code[i] = 0;
        if (!exact_r) {
#pragma unroll
          for (int i = 0; i < 16; ++i) x[i] = __fdiv_rn(x[i], scale);       // compared against the thresholds themselves
        }
#pragma unroll
        for (int t = 0; t < L - 1; ++t) {
          const float th = s_th[t];
          const float hs = __fmul_rd(__fmul_rn(s_h[t], scale), th == 0.0f ? 0x1p-50f : 1.0f);
          const float lim = exact_r ? __fmaf_rd(th, scale, hs) : th;
#pragma unroll
          for (int i = 0; i < 16; ++i) code[i] += (x[i] > lim) ? 1 : 0;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = s_cb[code[i]];
        lane_sums(x, ve, vo);
        const float code_sum = row_chain_sum(ve, vo, lane);
        const float vm = __fmul_rn(code_sum, 1.0f / 64.0f);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          w[j] = pack_half2(__fadd_rn(mean, __fmul_rn(scale, __fsub_rn(x[2 * j], vm))),
                            __fadd_rn(mean, __fmul_rn(scale, __fsub_rn(x[2 * j + 1], vm))));
      }
    }
    // ---- through this warp's staging block (16 rows x 128 bytes, XOR-swizzled) to 16-byte row stores
    uint8_t* const stg = sStage + warp * 2048;
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      *reinterpret_cast<uint32_t*>(stg + r8 * 128 + ((j ^ (r8 & 7)) << 4) + q4 * 4) = w_lo[j];
      *reinterpret_cast<uint32_t*>(stg + (r8 + 8) * 128 + ((j ^ (r8 & 7)) << 4) + q4 * 4) = w_hi[j];
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = lane + 32 * i, r = idx >> 3, c = idx & 7;
      const int row = rb * 16 + r;
      if (row < T) {
        const uint4 v = *reinterpret_cast<const uint4*>(stg + r * 128 + ((c ^ (r & 7)) << 4));
        *reinterpret_cast<uint4*>(p.out + (static_cast<long long>(b) * T + row) * C + h * 64 + c * 8) = v;
      }
    }
  }
}

}  // namespace arcq
