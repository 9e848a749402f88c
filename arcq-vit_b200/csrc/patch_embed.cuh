// The two data-movement steps around the patch-embedding GEMM of a ViT (timm PatchEmbed + _pos_embed), which the
// generic strided-copy and concatenation kernels of the framework do at a fraction of copy speed:
//   patchify:  images [B, C, H, W] fp16 -> rows [B * (H/P) * (W/P), C*P*P] fp16, row (b, gy, gx), column (c, py, px):
//              the matrix whose product with the flattened convolution weight is the PxP / stride-P convolution;
//   assemble:  tokens [B, 1 + T, D] = concat(class token, embedded patches [B*T, D]) + position embedding [1 + T, D],
//              the sum rounded to fp16 like the framework's elementwise add.
// 16-byte accesses on both sides; P is a multiple of 8, so a run of eight pixels never crosses a patch row.
#pragma once
#include <cuda_fp16.h>
#include "ptx.cuh"

namespace arcq {

__global__ void __launch_bounds__(256) patchify_kernel(const __half* __restrict__ img, int B, int C, int H, int W, int P,
                                                       __half* __restrict__ rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int gw = W / P, gh = H / P, cpr = P / 8;                 // chunks of eight pixels per patch row
  const long long row_chunks = static_cast<long long>(C) * P * cpr;         // chunks per output row
  const long long total = static_cast<long long>(B) * gh * gw * row_chunks;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / row_chunks;                          // output row: (b, gy, gx)
    const int q = static_cast<int>(i - r * row_chunks);           // chunk of the row: (c, py, px / 8)
    const int b = static_cast<int>(r / (gh * gw)), g = static_cast<int>(r - static_cast<long long>(b) * gh * gw);
    const int gy = g / gw, gx = g - gy * gw;
    const int c = q / (P * cpr), rem = q - c * (P * cpr), py = rem / cpr, pc = rem - py * cpr;
    const __half* src = img + ((static_cast<long long>(b) * C + c) * H + gy * P + py) * W + gx * P + pc * 8;
    reinterpret_cast<uint4*>(rows)[i] = __ldg(reinterpret_cast<const uint4*>(src));
  }
}

__global__ void __launch_bounds__(256) assemble_tokens_kernel(const __half* __restrict__ patches,
                                                              const __half* __restrict__ cls,
                                                              const __half* __restrict__ pos, int B, int T, int D,
                                                              __half* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int dc = D / 8;
  const long long total = static_cast<long long>(B) * (T + 1) * dc;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long tok = i / dc;
    const int ch = static_cast<int>(i - tok * dc);
    const int b = static_cast<int>(tok / (T + 1)), t = static_cast<int>(tok - static_cast<long long>(b) * (T + 1));
    const uint4 a = (t == 0) ? __ldg(reinterpret_cast<const uint4*>(cls) + ch)
                             : __ldg(reinterpret_cast<const uint4*>(patches) + (static_cast<long long>(b) * T + t - 1) * dc + ch);
    const uint4 p = __ldg(reinterpret_cast<const uint4*>(pos) + static_cast<long long>(t) * dc + ch);
    uint4 o;
    const __half2* ah = reinterpret_cast<const __half2*>(&a);
    const __half2* ph = reinterpret_cast<const __half2*>(&p);
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = __half22float2(ah[j]), fp = __half22float2(ph[j]);
      oh[j] = __floats2half2_rn(fa.x + fp.x, fa.y + fp.y);
    }
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

}  // namespace arcq
