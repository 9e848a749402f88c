// C ABI of the B200 back end: argument checks, launch configuration, error reporting.
// The kernels live in the .cuh files included below; this is the only translation unit.
#include <cuda_runtime.h>
#include <mutex>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <stdlib.h>

#include "../../include/arcq_b200.h"
#include "ptx.cuh"
#include "act_quant.cuh"
#include "act_quant_v2.cuh"
#include "act_quant_v4.cuh"
#include "codes.cuh"
#include "packed_gemm.cuh"
#include "gemm_ws.cuh"
#include "add_layernorm.cuh"
#include <cudaTypedefs.h>

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(ARCQ_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

__device__ int g_status_word = 0;
long long* g_trace_buf = nullptr;   // set by arcq_debug_trace; 64 timestamps per CTA

int* status_ptr() {
  // one address per device; looked up once per device and cached
  static thread_local int cached_dev = -1;
  static thread_local int* cached = nullptr;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != cached_dev) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    cached = static_cast<int*>(p);
    cached_dev = dev;
  }
  return cached;
}

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int sms = 148;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != cached_dev) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cached_dev = dev;
  }
  return sms;
}

// Tuning overrides for experiments (unset in normal use): ARCQ_WS_BN, ARCQ_WS_SA, ARCQ_WS_WS,
// ARCQ_WS_STATIONARY, ARCQ_WS_NBB, ARCQ_WS_GRID,
// ARCQ_WS_TMA_STORE, ARCQ_WS_ROTATE, ARCQ_ACT_QUANT_V1, ARCQ_ACT_QUANT_V2, ARCQ_LN_PLAIN.
int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v != nullptr && *v != 0) ? atoi(v) : dflt;
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

int grid_for(long long work_items, int per_block, int blocks_per_sm) {
  long long need = (work_items + per_block - 1) / per_block;
  long long cap = static_cast<long long>(sm_count()) * blocks_per_sm;
  if (need < 1) need = 1;
  return static_cast<int>(need < cap ? need : cap);
}

template <typename T, int BITS, int PRE = 0>
cudaError_t launch_act_quant(const void* x, long long groups, const float* th, const float* cb, uint8_t* packed,
                             float* mu, float* sg, float* cs, void* xhat, int xhat_dtype, cudaStream_t st) {
  const int grid = grid_for((groups + 3) / 4, 8, 8);
  const T* xt = static_cast<const T*>(x);
  if (xhat == nullptr) {
    arcq::act_quant_kernel<T, BITS, float, false, PRE><<<grid, 256, 0, st>>>(xt, groups, th, cb, packed, mu, sg, cs, nullptr);
  } else if (xhat_dtype == ARCQ_DT_F32) {
    arcq::act_quant_kernel<T, BITS, float, true, PRE>
        <<<grid, 256, 0, st>>>(xt, groups, th, cb, packed, mu, sg, cs, static_cast<float*>(xhat));
  } else if (xhat_dtype == ARCQ_DT_F16) {
    arcq::act_quant_kernel<T, BITS, __half, true, PRE>
        <<<grid, 256, 0, st>>>(xt, groups, th, cb, packed, mu, sg, cs, static_cast<__half*>(xhat));
  } else {
    arcq::act_quant_kernel<T, BITS, __nv_bfloat16, true, PRE>
        <<<grid, 256, 0, st>>>(xt, groups, th, cb, packed, mu, sg, cs, static_cast<__nv_bfloat16*>(xhat));
  }
  return cudaGetLastError();
}

// Second-design quantizer (one thread per group, staged loads): taken when the buffers are aligned for its
// 16-byte accesses and the reconstruction, if asked for, has the input's element type.
template <typename T, int BITS, int PRE = 0>
cudaError_t launch_act_quant_v2(const void* x, long long groups, const float* th, const float* cb, uint8_t* packed,
                                float* mu, float* sg, float* cs, void* xhat, cudaStream_t st) {
  const size_t smem = arcq::aq2_smem_bytes<T>();
  const long long tiles = (groups + arcq::kAq2Threads - 1) / arcq::kAq2Threads;
  const long long cap = static_cast<long long>(sm_count()) * 4;
  const int grid = static_cast<int>(tiles < cap ? tiles : cap);
  const T* xt = static_cast<const T*>(x);
  cudaError_t e;
  if (xhat == nullptr) {
    auto k = arcq::act_quant_v2_kernel<T, BITS, T, false, PRE>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    k<<<grid, arcq::kAq2Threads, smem, st>>>(xt, groups, th, cb, packed, mu, sg, cs, nullptr);
  } else if (packed == nullptr) {
    auto k = arcq::act_quant_v2_kernel<T, BITS, T, true, PRE, false>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    k<<<grid, arcq::kAq2Threads, smem, st>>>(xt, groups, th, cb, nullptr, mu, sg, cs, static_cast<T*>(xhat));
  } else {
    auto k = arcq::act_quant_v2_kernel<T, BITS, T, true, PRE>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    k<<<grid, arcq::kAq2Threads, smem, st>>>(xt, groups, th, cb, packed, mu, sg, cs, static_cast<T*>(xhat));
  }
  return cudaGetLastError();
}

// Two-lanes-per-group form of the staged quantizer (16-bit element types): same results, twice the warps.
template <typename T, int BITS, int PRE = 0>
cudaError_t launch_act_quant_v4(const void* x, long long groups, const float* th, const float* cb, uint8_t* packed,
                                float* mu, float* sg, float* cs, void* xhat, cudaStream_t st) {
  const size_t smem = arcq::aq4_smem_bytes<T>();
  const long long tiles = (groups + arcq::kAq4Groups - 1) / arcq::kAq4Groups;
  const long long cap = static_cast<long long>(sm_count()) * 4;
  const int grid = static_cast<int>(tiles < cap ? tiles : cap);
  const T* xt = static_cast<const T*>(x);
  T* xo = static_cast<T*>(xhat);
  cudaError_t e;
#define ARCQ_AQ4(WX, WP)                                                                                          \
  do {                                                                                                           \
    auto k = arcq::act_quant_v4_kernel<T, BITS, WX, PRE, WP>;                                                    \
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));            \
    if (e != cudaSuccess) return e;                                                                              \
    k<<<grid, arcq::kAq4Threads, smem, st>>>(xt, groups, th, cb, packed, mu, sg, cs, xo);                        \
  } while (0)
  if (xhat == nullptr) ARCQ_AQ4(false, true);
  else if (packed == nullptr) ARCQ_AQ4(true, false);
  else ARCQ_AQ4(true, true);
#undef ARCQ_AQ4
  return cudaGetLastError();
}

template <typename T> struct IsSixteenBit { static constexpr bool value = sizeof(T) == 2; };

template <typename T, int BITS, int PRE>
cudaError_t launch_staged(bool two_lane, const void* x, long long groups, const float* th, const float* cb,
                          uint8_t* packed, float* mu, float* sg, float* cs, void* xhat, cudaStream_t st) {
  if constexpr (IsSixteenBit<T>::value) {
    if (two_lane) return launch_act_quant_v4<T, BITS, PRE>(x, groups, th, cb, packed, mu, sg, cs, xhat, st);
  }
  return launch_act_quant_v2<T, BITS, PRE>(x, groups, th, cb, packed, mu, sg, cs, xhat, st);
}

template <typename T, int PRE>
cudaError_t dispatch_act_quant_bits(int bits, const void* x, int x_dtype, long long groups, const float* th,
                                    const float* cb, uint8_t* packed, float* mu, float* sg, float* cs, void* xhat,
                                    int xhat_dtype, cudaStream_t st) {
  // The one-thread-per-group kernel needs enough groups to fill the machine (148 SMs x 4 blocks x 128
  // threads); below that the 8-lanes-per-group kernel has 8 times the parallelism and lower latency.
  const bool enough = groups >= static_cast<long long>(sm_count()) * 4 * arcq::kAq2Threads / 2;
  const bool v2 = enough && env_int("ARCQ_ACT_QUANT_V1", 0) == 0 && aligned(x, 16) &&
                  (packed == nullptr || aligned(packed, 16)) &&
                  (xhat == nullptr || (xhat_dtype == x_dtype && aligned(xhat, 16)));
  if (v2) {
    // The two-lanes-per-group form (16-bit inputs) measured faster only where the per-element arithmetic is
    // long, i.e. with the fused GELU (42 vs 48 us on [12608,1536]); the plain quantizer stays one thread per
    // group (9.3 vs 10.8 us on [12608,384]).  ARCQ_ACT_QUANT_V2 = 1 / 2 forces the one-lane / two-lane form.
    const int force = env_int("ARCQ_ACT_QUANT_V2", 0);
    const bool two_lane = force == 2 || (force == 0 && PRE == 1);
    switch (bits) {
      case 4: return launch_staged<T, 4, PRE>(two_lane, x, groups, th, cb, packed, mu, sg, cs, xhat, st);
      case 3: return launch_staged<T, 3, PRE>(two_lane, x, groups, th, cb, packed, mu, sg, cs, xhat, st);
      default: return launch_staged<T, 2, PRE>(two_lane, x, groups, th, cb, packed, mu, sg, cs, xhat, st);
    }
  }
  switch (bits) {
    case 4: return launch_act_quant<T, 4, PRE>(x, groups, th, cb, packed, mu, sg, cs, xhat, xhat_dtype, st);
    case 3: return launch_act_quant<T, 3, PRE>(x, groups, th, cb, packed, mu, sg, cs, xhat, xhat_dtype, st);
    default: return launch_act_quant<T, 2, PRE>(x, groups, th, cb, packed, mu, sg, cs, xhat, xhat_dtype, st);
  }
}

// Tile width for the packed GEMM: the widest multiple of 16 (<= 256) that divides N, narrowed while
// the grid would leave most of the SMs idle.
int choose_bn(long long M, long long N) {
  static const int cand[] = {256, 192, 128, 96, 64, 48, 32, 16};
  const long long tiles_m = (M + arcq::kTileM - 1) / arcq::kTileM;
  int widest = 0, narrowest = 0;
  for (int c : cand) {
    if (N % c != 0) continue;
    if (widest == 0) widest = c;
    if (tiles_m * (N / c) >= sm_count()) return c;  // widest tile that still fills the machine
    if (c >= 32 || narrowest == 0) narrowest = c;
  }
  if (widest != 0) return narrowest;
  const long long r = (N + 15) / 16 * 16;  // N not a multiple of 16: pad the last tile column
  return static_cast<int>(r < 256 ? r : 256);
}


// ---- tensor maps (driver entry point fetched through the runtime, so libcuda is not linked) ----
PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-byte elements, box [box_cols x box_rows].
bool make_tensor_map_2d(CUtensorMap* tm, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                        uint64_t cols, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swz) {
  PFN_cuTensorMapEncodeTiled_v12000 enc = tensor_map_encoder();
  if (enc == nullptr) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct WsConfig {
  int bn, ws, sa, nbb, stationary, grid;
  size_t smem;
};

// Shared memory one CTA may ask for on B200 (227 KB) minus the 1 KB alignment slack.
constexpr size_t kSmemBudget = 232448 - 1024;

// Pick slab width, ring depths and grid for the warp-specialised GEMM; false if the shape is not
// one it handles (the caller then reports ARCQ_E_UNSUPPORTED).
bool choose_ws_config(long long M, long long N, long long K, int bits, bool dense, WsConfig* c) {
  const int G = static_cast<int>(K / 64);
  const long long tiles_m = (M + arcq::kTileM - 1) / arcq::kTileM;
  const int sms = sm_count();
  static const int cand[] = {192, 256, 128, 96, 64, 48, 32, 16};
  int best_bn = 0;
  long long best_ctas = -1;
  for (int bn : cand) {
    if (N % bn != 0) continue;
    const long long slabs = N / bn;
    if (slabs > sms) continue;
    const long long per = sms / slabs;
    const long long ctas = slabs * (tiles_m < per ? tiles_m : per);
    if (ctas * 4 >= 3LL * sms) { best_bn = bn; best_ctas = ctas; break; }  // first (widest) that fills 3/4 of the SMs
    if (ctas > best_ctas) { best_ctas = ctas; best_bn = bn; }
  }
  const int force_bn = env_int("ARCQ_WS_BN", 0);
  if (force_bn > 0 && force_bn % 16 == 0 && force_bn <= 256 && N % force_bn == 0) best_bn = force_bn;
  if (best_bn == 0) return false;
  c->bn = best_bn;
  const long long slabs = N / best_bn;
  const long long per = sms / slabs;
  c->grid = static_cast<int>(slabs * (tiles_m < per ? tiles_m : per));
  const int force_grid = env_int("ARCQ_WS_GRID", 0);
  if (force_grid > 0 && force_grid <= sms) c->grid = force_grid;
  const int force_stat = env_int("ARCQ_WS_STATIONARY", -1), force_sa = env_int("ARCQ_WS_SA", 0);
  const int force_ws = env_int("ARCQ_WS_WS", 0), force_nbb = env_int("ARCQ_WS_NBB", 0);
  // stationary if all G sub-tiles plus two A stages fit
  for (int stationary = 1; stationary >= 0; --stationary) {
    if (force_stat >= 0 && stationary != force_stat) continue;
    const int stream_slots = dense ? 4 : 3;
    int ws = stationary ? G : (G < stream_slots ? G : stream_slots);
    if (!stationary && force_ws > 0 && force_ws <= 16) ws = force_ws;
    if (ws > (stationary ? 32 : 16)) continue;   // barrier slots: 16 full/empty pairs for a ring, 32 full for a stationary slab
    for (int sa = 8; sa >= 2; --sa) {
      if (force_sa > 0 && sa != force_sa) continue;
      const size_t need = arcq::ws_smem_layout(best_bn, ws, sa, bits, G, stationary != 0, dense).total;
      if (need <= kSmemBudget) {
        c->ws = ws; c->sa = sa; c->stationary = stationary;
        c->nbb = stationary ? 1 : 2;
        if (force_nbb == 1 || force_nbb == 2) c->nbb = force_nbb;
        c->smem = need + 1024;
        return true;
      }
    }
  }
  return false;
}

}  // namespace

extern "C" {

int arcq_version(void) { return ARCQ_B200_VERSION; }

const char* arcq_last_error_string(void) { return g_err; }

int arcq_debug_trace(void* device_buffer) {
  g_trace_buf = static_cast<long long*>(device_buffer);
  return ARCQ_OK;
}

int arcq_device_status(void) {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return fail(ARCQ_E_CUDA, "device synchronize failed: %s",
                                                          cudaGetErrorString(cudaGetLastError()));
  if (cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int)) != cudaSuccess) return fail(ARCQ_E_CUDA, "status read failed");
  if (v != 0) cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int));
  return v;
}

static int act_quant_impl(int pre, const void* x, int x_dtype, int64_t M, int64_t K, const float* thresholds,
                          const float* codebook, int bits, int group_size, uint8_t* packed_out, float* mu_out,
                          float* sigma_out, float* codesum_out, void* xhat_out, int xhat_dtype, void* stream) {
  if (x == nullptr || thresholds == nullptr || codebook == nullptr) return fail(ARCQ_E_BAD_ARG, "null input pointer");
  if (packed_out == nullptr && xhat_out == nullptr) return fail(ARCQ_E_BAD_ARG, "no output requested");
  if ((mu_out != nullptr) != (sigma_out != nullptr)) return fail(ARCQ_E_BAD_ARG, "mu_out and sigma_out go together");
  if (packed_out != nullptr && mu_out == nullptr) return fail(ARCQ_E_BAD_ARG, "packed_out needs mu_out and sigma_out");
  if (codesum_out != nullptr && mu_out == nullptr) return fail(ARCQ_E_BAD_ARG, "codesum_out needs mu_out");
  if (bits < 2 || bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", bits);
  if (x_dtype < ARCQ_DT_F32 || x_dtype > ARCQ_DT_BF16) return fail(ARCQ_E_BAD_ARG, "bad x_dtype %d", x_dtype);
  if (xhat_out != nullptr && (xhat_dtype < ARCQ_DT_F32 || xhat_dtype > ARCQ_DT_BF16))
    return fail(ARCQ_E_BAD_ARG, "bad xhat_dtype %d", xhat_dtype);
  if (M < 0 || K <= 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape M=%lld K=%lld", (long long)M, (long long)K);
  if (group_size <= 0 || K % group_size != 0)
    return fail(ARCQ_E_BAD_SHAPE, "K=%lld is not a multiple of group_size=%d", (long long)K, group_size);
  if (group_size != 64) return fail(ARCQ_E_UNSUPPORTED, "group_size %d: only 64 is built", group_size);
  if (packed_out != nullptr && !aligned(packed_out, 4)) return fail(ARCQ_E_ALIGN, "packed_out must be 4-byte aligned");
  if (M == 0) return ARCQ_OK;
  const long long groups = static_cast<long long>(M) * (K / 64);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (pre == 1) {
    if (x_dtype != ARCQ_DT_F16) return fail(ARCQ_E_UNSUPPORTED, "the fused GELU is built for fp16 input only");
    e = dispatch_act_quant_bits<__half, 1>(bits, x, x_dtype, groups, thresholds, codebook, packed_out, mu_out,
                                           sigma_out, codesum_out, xhat_out, xhat_dtype, st);
  } else if (x_dtype == ARCQ_DT_F32)
    e = dispatch_act_quant_bits<float, 0>(bits, x, x_dtype, groups, thresholds, codebook, packed_out, mu_out, sigma_out,
                                          codesum_out, xhat_out, xhat_dtype, st);
  else if (x_dtype == ARCQ_DT_F16)
    e = dispatch_act_quant_bits<__half, 0>(bits, x, x_dtype, groups, thresholds, codebook, packed_out, mu_out, sigma_out,
                                           codesum_out, xhat_out, xhat_dtype, st);
  else
    e = dispatch_act_quant_bits<__nv_bfloat16, 0>(bits, x, x_dtype, groups, thresholds, codebook, packed_out, mu_out,
                                                  sigma_out, codesum_out, xhat_out, xhat_dtype, st);
  if (e != cudaSuccess) return cuda_fail(e, "act_quant launch");
  return ARCQ_OK;
}

int arcq_act_quant(const void* x, int x_dtype, int64_t M, int64_t K, const float* thresholds, const float* codebook,
                   int bits, int group_size, uint8_t* packed_out, float* mu_out, float* sigma_out, float* codesum_out,
                   void* xhat_out, int xhat_dtype, void* stream) {
  return act_quant_impl(0, x, x_dtype, M, K, thresholds, codebook, bits, group_size, packed_out, mu_out, sigma_out,
                        codesum_out, xhat_out, xhat_dtype, stream);
}

int arcq_gelu_act_quant(const void* x, int x_dtype, int64_t M, int64_t K, const float* thresholds,
                        const float* codebook, int bits, int group_size, uint8_t* packed_out, float* mu_out,
                        float* sigma_out, float* codesum_out, void* xhat_out, int xhat_dtype, void* stream) {
  return act_quant_impl(1, x, x_dtype, M, K, thresholds, codebook, bits, group_size, packed_out, mu_out, sigma_out,
                        codesum_out, xhat_out, xhat_dtype, stream);
}

int arcq_packed_gemm(const uint8_t* packed_x, const float* mu_a, const float* sigma_a, const float* codesum_a,
                     const uint8_t* packed_w, const float* mu_w, const float* sigma_w, const float* codesum_w,
                     const float* act_codebook, const float* w_codebook, const float* bias, int bits, int group_size,
                     int64_t M, int64_t N, int64_t K, void* y, int y_dtype, void* stream) {
  if (!packed_x || !mu_a || !sigma_a || !codesum_a || !packed_w || !mu_w || !sigma_w || !codesum_w ||
      !act_codebook || !w_codebook || !y)
    return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (bits < 2 || bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", bits);
  if (y_dtype != ARCQ_DT_F16 && y_dtype != ARCQ_DT_F32) return fail(ARCQ_E_BAD_ARG, "y_dtype must be f16 or f32");
  if (M < 0 || N <= 0 || K <= 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape M=%lld N=%lld K=%lld", (long long)M,
                                              (long long)N, (long long)K);
  if (group_size <= 0 || K % group_size != 0)
    return fail(ARCQ_E_BAD_SHAPE, "K=%lld is not a multiple of group_size=%d", (long long)K, group_size);
  if (group_size != 64) return fail(ARCQ_E_UNSUPPORTED, "group_size %d: only 64 is built", group_size);
  if (N % 8 != 0) return fail(ARCQ_E_BAD_SHAPE, "N=%lld must be a multiple of 8", (long long)N);
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > (1 << 20)) return fail(ARCQ_E_TOO_LARGE, "shape too large");
  if (!aligned(packed_x, 4) || !aligned(packed_w, 4)) return fail(ARCQ_E_ALIGN, "packed codes must be 4-byte aligned");
  if (!aligned(y, 16)) return fail(ARCQ_E_ALIGN, "y must be 16-byte aligned");
  if (M == 0) return ARCQ_OK;

  arcq::GemmParams p;
  p.pa = packed_x; p.mu_a = mu_a; p.sg_a = sigma_a; p.cs_a = codesum_a;
  p.pw = packed_w; p.mu_w = mu_w; p.sg_w = sigma_w; p.cs_w = codesum_w;
  p.cb_a = act_codebook; p.cb_w = w_codebook; p.bias = bias; p.y = y;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K); p.G = static_cast<int>(K / 64);
  p.pc = static_cast<int>(K * bits / 8);
  p.bn = choose_bn(M, N);
  p.y_f32 = (y_dtype == ARCQ_DT_F32) ? 1 : 0;
  p.status = status_ptr();
  if (p.status == nullptr) return fail(ARCQ_E_CUDA, "device status word not reachable");

  const size_t smem = arcq::packed_gemm_smem_bytes(p.bn);
  dim3 grid(static_cast<unsigned>((M + arcq::kTileM - 1) / arcq::kTileM), static_cast<unsigned>((N + p.bn - 1) / p.bn));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSuccess;
#define ARCQ_LAUNCH_GEMM(B)                                                                                  \
  do {                                                                                                       \
    e = cudaFuncSetAttribute(arcq::packed_gemm_kernel<B>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                             static_cast<int>(smem));                                                        \
    if (e == cudaSuccess) {                                                                                  \
      arcq::packed_gemm_kernel<B><<<grid, arcq::kGemmThreads, smem, st>>>(p);                                \
      e = cudaGetLastError();                                                                                \
    }                                                                                                        \
  } while (0)
  if (bits == 4) ARCQ_LAUNCH_GEMM(4);
  else if (bits == 3) ARCQ_LAUNCH_GEMM(3);
  else ARCQ_LAUNCH_GEMM(2);
#undef ARCQ_LAUNCH_GEMM
  if (e != cudaSuccess) return cuda_fail(e, "packed_gemm launch");
  return ARCQ_OK;
}


// Launch of the persistent GEMM for either weight form: packed codes + statistics (rebuilt in shared
// memory) or an fp16 matrix (`dense`; mu_w .. w_codebook unused).  Arguments are already validated.
static int launch_ws_gemm(bool dense, const void* xhat, const void* w, const float* mu_w, const float* sigma_w,
                          const float* codesum_w, const float* w_codebook, const float* bias, int bits, int64_t M,
                          int64_t N, int64_t K, void* y, int y_dtype, void* stream) {
  WsConfig cfg;
  if (!choose_ws_config(M, N, K, bits, dense, &cfg)) return fail(ARCQ_E_UNSUPPORTED, "no tile configuration for this shape");

  CUtensorMap tm_a, tm_w;
  if (!make_tensor_map_2d(&tm_a, xhat, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, static_cast<uint64_t>(M),
                          static_cast<uint64_t>(K), 64, arcq::kTileM, CU_TENSOR_MAP_SWIZZLE_128B))
    return fail(ARCQ_E_CUDA, "cuTensorMapEncodeTiled failed for the activation matrix");
  if (dense) {
    if (!make_tensor_map_2d(&tm_w, w, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, static_cast<uint64_t>(N),
                            static_cast<uint64_t>(K), 64, cfg.bn, CU_TENSOR_MAP_SWIZZLE_128B))
      return fail(ARCQ_E_CUDA, "cuTensorMapEncodeTiled failed for the weight matrix");
  } else if (!make_tensor_map_2d(&tm_w, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, static_cast<uint64_t>(N),
                                 static_cast<uint64_t>(K * bits / 8), arcq::raw_row_bytes(bits), cfg.bn,
                                 CU_TENSOR_MAP_SWIZZLE_NONE)) {
    return fail(ARCQ_E_CUDA, "cuTensorMapEncodeTiled failed for the packed weight");
  }

  // output tensor map for the TMA-store epilogue: 32-row blocks of 64 bytes (32 fp16 / 16 fp32 columns)
  const int out_cw = (y_dtype == ARCQ_DT_F32) ? 16 : 32;
  const bool use_tma_store = (cfg.bn % out_cw == 0) && env_int("ARCQ_WS_TMA_STORE", 1) != 0;
  CUtensorMap tm_y;
  if (!make_tensor_map_2d(&tm_y, y, (y_dtype == ARCQ_DT_F32) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                          (y_dtype == ARCQ_DT_F32) ? 4 : 2, static_cast<uint64_t>(M), static_cast<uint64_t>(N),
                          out_cw, 32, CU_TENSOR_MAP_SWIZZLE_64B))
    return fail(ARCQ_E_CUDA, "cuTensorMapEncodeTiled failed for the output matrix");

  arcq::WsParams p;
  p.tma_store = use_tma_store ? 1 : 0;
  p.rotate = env_int("ARCQ_WS_ROTATE", 1);
  p.mu_w = mu_w; p.sg_w = sigma_w; p.cs_w = codesum_w; p.cb_w = w_codebook; p.bias = bias; p.y = y;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K); p.G = static_cast<int>(K / 64);
  p.bn = cfg.bn; p.ws = cfg.ws; p.sa = cfg.sa; p.nbb = cfg.nbb; p.stationary = cfg.stationary;
  p.dense = dense ? 1 : 0;
  p.y_f32 = (y_dtype == ARCQ_DT_F32) ? 1 : 0;
  p.status = status_ptr();
  p.trace = g_trace_buf;
  if (p.status == nullptr) return fail(ARCQ_E_CUDA, "device status word not reachable");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSuccess;
#define ARCQ_LAUNCH_WS(B)                                                                                          \
  do {                                                                                                             \
    e = cudaFuncSetAttribute(arcq::packed_weight_gemm_ws_kernel<B>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                             static_cast<int>(cfg.smem));                                                          \
    if (e == cudaSuccess) {                                                                                        \
      arcq::packed_weight_gemm_ws_kernel<B><<<cfg.grid, arcq::kWsThreads, cfg.smem, st>>>(tm_a, tm_w, tm_y, p);          \
      e = cudaGetLastError();                                                                                      \
    }                                                                                                              \
  } while (0)
  if (bits == 4) ARCQ_LAUNCH_WS(4);
  else if (bits == 3) ARCQ_LAUNCH_WS(3);
  else ARCQ_LAUNCH_WS(2);
#undef ARCQ_LAUNCH_WS
  if (e != cudaSuccess) return cuda_fail(e, "packed_weight_gemm launch");
  return ARCQ_OK;
}

int arcq_packed_weight_gemm(const void* xhat, const uint8_t* packed_w, const float* mu_w, const float* sigma_w,
                            const float* codesum_w, const float* w_codebook, const float* bias, int bits,
                            int group_size, int64_t M, int64_t N, int64_t K, void* y, int y_dtype, void* stream) {
  if (!xhat || !packed_w || !mu_w || !sigma_w || !codesum_w || !w_codebook || !y)
    return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (bits < 2 || bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", bits);
  if (y_dtype != ARCQ_DT_F16 && y_dtype != ARCQ_DT_F32) return fail(ARCQ_E_BAD_ARG, "y_dtype must be f16 or f32");
  if (M < 0 || N <= 0 || K <= 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape M=%lld N=%lld K=%lld", (long long)M,
                                              (long long)N, (long long)K);
  if (group_size <= 0 || K % group_size != 0)
    return fail(ARCQ_E_BAD_SHAPE, "K=%lld is not a multiple of group_size=%d", (long long)K, group_size);
  if (group_size != 64) return fail(ARCQ_E_UNSUPPORTED, "group_size %d: only 64 is built", group_size);
  if (N % 16 != 0) return fail(ARCQ_E_UNSUPPORTED, "N=%lld: this entry point needs N %% 16 == 0", (long long)N);
  if ((K * bits / 8) % 16 != 0)
    return fail(ARCQ_E_UNSUPPORTED, "packed row of %lld bytes is not a multiple of 16 (TMA stride rule)",
                (long long)(K * bits / 8));
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > (1 << 20)) return fail(ARCQ_E_TOO_LARGE, "shape too large");
  if (!aligned(xhat, 16) || !aligned(packed_w, 16) || !aligned(y, 16))
    return fail(ARCQ_E_ALIGN, "xhat, packed_w and y must be 16-byte aligned");
  if (M == 0) return ARCQ_OK;
  return launch_ws_gemm(false, xhat, packed_w, mu_w, sigma_w, codesum_w, w_codebook, bias, bits, M, N, K, y, y_dtype,
                        stream);
}

int arcq_dense_weight_gemm(const void* xhat, const void* w16, const float* bias, int64_t M, int64_t N, int64_t K,
                           void* y, int y_dtype, void* stream) {
  if (!xhat || !w16 || !y) return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (y_dtype != ARCQ_DT_F16 && y_dtype != ARCQ_DT_F32) return fail(ARCQ_E_BAD_ARG, "y_dtype must be f16 or f32");
  if (M < 0 || N <= 0 || K <= 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape M=%lld N=%lld K=%lld", (long long)M,
                                              (long long)N, (long long)K);
  if (K % 64 != 0) return fail(ARCQ_E_UNSUPPORTED, "K=%lld: this entry point needs K %% 64 == 0", (long long)K);
  if (N % 16 != 0) return fail(ARCQ_E_UNSUPPORTED, "N=%lld: this entry point needs N %% 16 == 0", (long long)N);
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > (1 << 20)) return fail(ARCQ_E_TOO_LARGE, "shape too large");
  if (!aligned(xhat, 16) || !aligned(w16, 16) || !aligned(y, 16))
    return fail(ARCQ_E_ALIGN, "xhat, w16 and y must be 16-byte aligned");
  if (M == 0) return ARCQ_OK;
  return launch_ws_gemm(true, xhat, w16, nullptr, nullptr, nullptr, nullptr, bias, 4, M, N, K, y, y_dtype, stream);
}

int arcq_add_layernorm(const void* x, const void* y, const float* gamma, const float* beta, float eps, int64_t M,
                       int64_t K, void* sum_out, void* h_out, void* stream) {
  if (x == nullptr || gamma == nullptr || beta == nullptr || h_out == nullptr)
    return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (M < 0 || K <= 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape M=%lld K=%lld", (long long)M, (long long)K);
  if (K % 8 != 0) return fail(ARCQ_E_BAD_SHAPE, "K=%lld must be a multiple of 8", (long long)K);
  if (K > 32 * 8 * arcq::kLnMaxChunks) return fail(ARCQ_E_TOO_LARGE, "rows longer than %d values are not built", 32 * 8 * arcq::kLnMaxChunks);
  if (!aligned(x, 16) || !aligned(h_out, 16) || (y != nullptr && !aligned(y, 16)) ||
      (sum_out != nullptr && !aligned(sum_out, 16)) || !aligned(gamma, 16) || !aligned(beta, 16))
    return fail(ARCQ_E_ALIGN, "all buffers must be 16-byte aligned");
  if (M == 0) return ARCQ_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __half *xh = static_cast<const __half*>(x), *yh = static_cast<const __half*>(y);
  __half *so = static_cast<__half*>(sum_out), *ho = static_cast<__half*>(h_out);
  const bool plain = env_int("ARCQ_LN_PLAIN", 0) != 0;
  if (K == 384 && !plain) {          // 16 lanes per row, 2 rows per warp
    arcq::add_layernorm_rows_kernel<16><<<grid_for(M, 16, 6), 256, 0, st>>>(xh, yh, gamma, beta, eps, M, so, ho);
  } else if (K == 192 && !plain) {
    arcq::add_layernorm_rows_kernel<8><<<grid_for(M, 32, 6), 256, 0, st>>>(xh, yh, gamma, beta, eps, M, so, ho);
  } else if (K == 768 && !plain) {
    arcq::add_layernorm_rows_kernel<32><<<grid_for(M, 8, 6), 256, 0, st>>>(xh, yh, gamma, beta, eps, M, so, ho);
  } else {
    arcq::add_layernorm_kernel<<<grid_for(M, 8, 8), 256, 0, st>>>(xh, yh, gamma, beta, eps, M, static_cast<int>(K), so, ho);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "add_layernorm launch");
  return ARCQ_OK;
}

int arcq_unpack_codes(const uint8_t* packed, int64_t rows, int64_t length, int bits, uint8_t* codes_out, void* stream) {
  if (!packed || !codes_out) return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (bits < 2 || bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", bits);
  if (rows < 0 || length < 0) return fail(ARCQ_E_BAD_SHAPE, "negative shape");
  if (rows == 0 || length == 0) return ARCQ_OK;
  const long long pc = (length * bits + 7) / 8;
  arcq::unpack_codes_kernel<<<grid_for(rows * length, 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      packed, rows, length, pc, bits, codes_out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "unpack launch");
  return ARCQ_OK;
}

int arcq_pack_codes(const uint8_t* codes, int64_t rows, int64_t length, int bits, uint8_t* packed_out, void* stream) {
  if (!codes || !packed_out) return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (bits < 2 || bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", bits);
  if (rows < 0 || length < 0) return fail(ARCQ_E_BAD_SHAPE, "negative shape");
  if (rows == 0 || length == 0) return ARCQ_OK;
  const long long pc = (length * bits + 7) / 8;
  arcq::pack_codes_kernel<<<grid_for(rows * pc, 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      codes, rows, length, pc, bits, packed_out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "pack launch");
  return ARCQ_OK;
}

int arcq_dequant(const uint8_t* packed, const float* mu, const float* sigma, const float* codesum, const float* codebook,
                 int bits, int group_size, int64_t rows, int64_t K, void* out, int out_dtype, void* stream) {
  if (!packed || !mu || !sigma || !codesum || !codebook || !out) return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (bits < 2 || bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", bits);
  if (out_dtype != ARCQ_DT_F16 && out_dtype != ARCQ_DT_F32) return fail(ARCQ_E_BAD_ARG, "out_dtype must be f16 or f32");
  if (rows < 0 || K <= 0 || group_size <= 0 || K % group_size != 0 || group_size % 8 != 0)
    return fail(ARCQ_E_BAD_SHAPE, "bad shape rows=%lld K=%lld group_size=%d", (long long)rows, (long long)K, group_size);
  if (!aligned(packed, 4)) return fail(ARCQ_E_ALIGN, "packed codes must be 4-byte aligned");
  if (rows == 0) return ARCQ_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(rows * (K / 8), 256, 8);
  const int k = static_cast<int>(K);
#define ARCQ_LAUNCH_DQ(B)                                                                                          \
  do {                                                                                                             \
    if (out_dtype == ARCQ_DT_F32)                                                                                  \
      arcq::dequant_kernel<B, float><<<grid, 256, 0, st>>>(packed, mu, sigma, codesum, codebook, rows, k,          \
                                                           group_size, static_cast<float*>(out));                 \
    else                                                                                                           \
      arcq::dequant_kernel<B, __half><<<grid, 256, 0, st>>>(packed, mu, sigma, codesum, codebook, rows, k,         \
                                                            group_size, static_cast<__half*>(out));               \
  } while (0)
  if (bits == 4) ARCQ_LAUNCH_DQ(4);
  else if (bits == 3) ARCQ_LAUNCH_DQ(3);
  else ARCQ_LAUNCH_DQ(2);
#undef ARCQ_LAUNCH_DQ
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "dequant launch");
  return ARCQ_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Linear with the library's own weight scratch.
//
// The dense route above needs room for the unpacked fp16 weight, and so far the caller brings it.  Some
// callers have no way to: a C host that binds this ABI from a runtime whose device memory was handed out in
// full at start-up, or a serving loop in which a device allocation (and the device-wide wait it may imply) is
// not acceptable once requests are flowing.  For them the scratch lives in the library image itself: a
// file-scope device array, sized for the largest DeiT-B linear (768 x 3072 fp16 values, 4.5 MB per device).
// Nothing here allocates or frees memory.
//  * Set-up: the array's device address is looked up once per device, on the first call made with that
//    device current.  That look-up is host-side work of the CUDA runtime; make the first call outside any
//    stream capture, later calls only launch kernels.
//  * Nothing has to start at zero: every element the contraction reads was written by the unpack kernel of
//    the same call, which is ordered before it on `stream`.
//  * One array per device: two calls in flight at once on the same device (different streams or host
//    threads) would overwrite each other's weight.  Calls must be ordered one after the other.
constexpr long long kStaticWeightElems = ARCQ_STATIC_WEIGHT_ELEMS;
static __device__ __align__(256) __half g_static_w16[kStaticWeightElems];

static __half* static_weight_scratch() {
  constexpr int kMaxDevices = 64;
  static __half* cached[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fail(ARCQ_E_CUDA, "no current CUDA device (or device index above %d)", kMaxDevices - 1);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_w16);
    if (e != cudaSuccess || p == nullptr) {
      cuda_fail(e, "address of the static weight scratch");
      return nullptr;
    }
    cached[dev] = static_cast<__half*>(p);
  }
  return cached[dev];
}

int arcq_packed_linear_static_scratch(const void* xhat, const uint8_t* packed_w, const float* mu_w,
                                      const float* sigma_w, const float* codesum_w, const float* w_codebook,
                                      const float* bias, int bits, int group_size, int64_t M, int64_t N, int64_t K,
                                      void* y, int y_dtype, void* stream) {
  if (!xhat || !packed_w || !mu_w || !sigma_w || !codesum_w || !w_codebook || !y)
    return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (M < 0 || N <= 0 || K <= 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape M=%lld N=%lld K=%lld", (long long)M,
                                              (long long)N, (long long)K);
  if (group_size != 64) return fail(ARCQ_E_UNSUPPORTED, "group_size %d: only 64 is built", group_size);
  if (N > kStaticWeightElems || K > kStaticWeightElems || N * K > kStaticWeightElems)
    return fail(ARCQ_E_TOO_LARGE, "weight of %lld x %lld values exceeds the static scratch of %lld values; "
                                  "use arcq_dequant + arcq_dense_weight_gemm with a buffer of your own",
                (long long)N, (long long)K, (long long)kStaticWeightElems);
  __half* const w16 = static_weight_scratch();
  if (w16 == nullptr) return ARCQ_E_CUDA;
  if (M == 0) return ARCQ_OK;
  const int rc = arcq_dequant(packed_w, mu_w, sigma_w, codesum_w, w_codebook, bits, group_size, N, K, w16,
                              ARCQ_DT_F16, stream);
  if (rc != ARCQ_OK) return rc;
  return arcq_dense_weight_gemm(xhat, w16, bias, M, N, K, y, y_dtype, stream);
}

}  // extern "C"
