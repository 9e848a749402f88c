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
#include <string.h>

#include "../../include/arcq_b200.h"
#include "ptx.cuh"
#include "act_quant.cuh"
#include "act_quant_v2.cuh"
#include "act_quant_v4.cuh"
#include "codes.cuh"
#include "packed_gemm.cuh"
#include "gemm_ws.cuh"
#include "gemm_pair.cuh"
#include "gemm_pair_dense.cuh"
#include "add_layernorm.cuh"
#include "ln_act_quant.cuh"
#include "attention.cuh"
#include "patch_embed.cuh"
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
// which GEMM kernel the last GEMM entry point of this host thread launched (arcq_debug_last_gemm_kernel)
thread_local int g_last_gemm_kernel = 0;
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

// Tuning options.  Each has a built-in default; an environment variable of the same name, read once when the
// library is first used, or arcq_debug_set_option() at any time, overrides it.  Normal use sets none of them.
enum Opt {
  O_WS_BN, O_WS_SA, O_WS_WS, O_WS_STATIONARY, O_WS_NBB, O_WS_GRID, O_WS_TMA_STORE, O_WS_ROTATE,
  O_ACT_QUANT_V1, O_ACT_QUANT_V2, O_LN_PLAIN,
  O_PAIR, O_PAIR_MIN_M, O_PAIR_BN, O_PAIR_SA, O_PAIR_KS, O_PAIR_NBB, O_PAIR_LUT, O_PAIR_PAIRS, O_PAIR_STATIONARY,
  O_PAIR_WS, O_LNQ_SMALL, O_AQ2_MIN_GROUPS, O_PDL, O_POLL_LIMIT, O_SPIN_LIMIT, O_COUNT
};
struct OptDef { const char* name; int dflt; };
const OptDef kOptDefs[O_COUNT] = {
    {"ARCQ_WS_BN", 0},        {"ARCQ_WS_SA", 0},          {"ARCQ_WS_WS", 0},       {"ARCQ_WS_STATIONARY", -1},
    {"ARCQ_WS_NBB", 0},       {"ARCQ_WS_GRID", 0},        {"ARCQ_WS_TMA_STORE", 1}, {"ARCQ_WS_ROTATE", 1},
    {"ARCQ_ACT_QUANT_V1", 0}, {"ARCQ_ACT_QUANT_V2", 0},   {"ARCQ_LN_PLAIN", 0},
    {"ARCQ_PAIR", 1},         {"ARCQ_PAIR_MIN_M", 1024},  {"ARCQ_PAIR_BN", 0},     {"ARCQ_PAIR_SA", 0},
    {"ARCQ_PAIR_KS", 0},      {"ARCQ_PAIR_NBB", 0},       {"ARCQ_PAIR_LUT", 0},    {"ARCQ_PAIR_PAIRS", 0},
    {"ARCQ_PAIR_STATIONARY", -1}, {"ARCQ_PAIR_WS", 0}, {"ARCQ_LNQ_SMALL", 1}, {"ARCQ_AQ2_MIN_GROUPS", 0}, {"ARCQ_PDL", 1},
    {"ARCQ_POLL_LIMIT", 1 << 21}, {"ARCQ_SPIN_LIMIT", 1 << 25},
};
int g_opt[O_COUNT];
void load_options() {
  static const bool once = [] {
    for (int i = 0; i < O_COUNT; ++i) {
      const char* v = getenv(kOptDefs[i].name);
      g_opt[i] = (v != nullptr && *v != 0) ? atoi(v) : kOptDefs[i].dflt;
    }
    return true;
  }();
  (void)once;
}
int opt(Opt o) {
  load_options();
  return g_opt[o];
}

// Launch as a programmatic dependent of the kernel before it in the stream (unless ARCQ_PDL is 0): the grid may
// become resident while that kernel drains; every kernel launched this way calls pdl_wait() before it reads
// anything a predecessor writes.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t lc = {};
  lc.gridDim = grid;
  lc.blockDim = block;
  lc.dynamicSmemBytes = smem;
  lc.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attr;
  lc.numAttrs = opt(O_PDL) != 0 ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kernel, static_cast<KArgs>(args)...);
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
    launch_pdl(arcq::act_quant_kernel<T, BITS, float, false, PRE>, grid, 256, 0, st, xt, groups, th, cb, packed, mu, sg, cs, static_cast<float*>(nullptr));
  } else if (xhat_dtype == ARCQ_DT_F32) {
    launch_pdl(arcq::act_quant_kernel<T, BITS, float, true, PRE>, grid, 256, 0, st, xt, groups, th, cb, packed, mu, sg, cs, static_cast<float*>(xhat));
  } else if (xhat_dtype == ARCQ_DT_F16) {
    launch_pdl(arcq::act_quant_kernel<T, BITS, __half, true, PRE>, grid, 256, 0, st, xt, groups, th, cb, packed, mu, sg, cs, static_cast<__half*>(xhat));
  } else {
    launch_pdl(arcq::act_quant_kernel<T, BITS, __nv_bfloat16, true, PRE>, grid, 256, 0, st, xt, groups, th, cb, packed, mu, sg, cs, static_cast<__nv_bfloat16*>(xhat));
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
    launch_pdl(k, grid, arcq::kAq2Threads, smem, st, xt, groups, th, cb, packed, mu, sg, cs, static_cast<T*>(nullptr));
  } else if (packed == nullptr) {
    auto k = arcq::act_quant_v2_kernel<T, BITS, T, true, PRE, false>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    launch_pdl(k, grid, arcq::kAq2Threads, smem, st, xt, groups, th, cb, static_cast<uint8_t*>(nullptr), mu, sg, cs, static_cast<T*>(xhat));
  } else {
    auto k = arcq::act_quant_v2_kernel<T, BITS, T, true, PRE>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    launch_pdl(k, grid, arcq::kAq2Threads, smem, st, xt, groups, th, cb, packed, mu, sg, cs, static_cast<T*>(xhat));
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
    launch_pdl(k, grid, arcq::kAq4Threads, smem, st, xt, groups, th, cb, packed, mu, sg, cs, xo);                  \
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
  const long long min_groups = opt(O_AQ2_MIN_GROUPS) > 0 ? opt(O_AQ2_MIN_GROUPS) : static_cast<long long>(sm_count()) * 4 * arcq::kAq2Threads / 2;
  const bool enough = groups >= min_groups;
  const bool v2 = enough && opt(O_ACT_QUANT_V1) == 0 && aligned(x, 16) &&
                  (packed == nullptr || aligned(packed, 16)) &&
                  (xhat == nullptr || (xhat_dtype == x_dtype && aligned(xhat, 16)));
  if (v2) {
    // The two-lanes-per-group form (16-bit inputs) measured faster only where the per-element arithmetic is
    // long, i.e. with the fused GELU (42 vs 48 us on [12608,1536]); the plain quantizer stays one thread per
    // group (9.3 vs 10.8 us on [12608,384]).  ARCQ_ACT_QUANT_V2 = 1 / 2 forces the one-lane / two-lane form.
    const int force = opt(O_ACT_QUANT_V2);
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
  static const PFN_cuTensorMapEncodeTiled_v12000 fn = [] {   // resolved once; the initialisation is thread-safe
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    return static_cast<PFN_cuTensorMapEncodeTiled_v12000>(nullptr);
  }();
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-byte elements, box [box_cols x box_rows].  A descriptor
// depends only on these values (not on what the memory holds), so the last few are kept per host thread:
// a model's layers present the same (pointer, shape) again on every forward.
struct TensorMapKey {
  const void* base;
  uint64_t rows, cols;
  uint32_t box_cols, box_rows;
  int dt, swz;
  bool operator==(const TensorMapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && box_cols == o.box_cols && box_rows == o.box_rows &&
           dt == o.dt && swz == o.swz;
  }
};
bool make_tensor_map_2d(CUtensorMap* tm, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                        uint64_t cols, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swz) {
  constexpr int kSlots = 256;
  struct Slot { TensorMapKey key; CUtensorMap map; bool used; };
  static thread_local Slot cache[kSlots] = {};
  const TensorMapKey key{base, rows, cols, box_cols, box_rows, static_cast<int>(dt), static_cast<int>(swz)};
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
  h = (h ^ (rows * 0x9E3779B97F4A7C15ull) ^ (cols << 7) ^ (static_cast<uint64_t>(box_rows) << 29) ^ (static_cast<uint64_t>(box_cols) << 41)) * 0xD6E8FEB86659FD93ull;
  Slot& slot = cache[(h >> 40) % kSlots];
  if (slot.used && slot.key == key) {
    *tm = slot.map;
    return true;
  }
  PFN_cuTensorMapEncodeTiled_v12000 enc = tensor_map_encoder();
  if (enc == nullptr) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  if (enc(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  slot.key = key;
  slot.map = *tm;
  slot.used = true;
  return true;
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
  const int force_bn = opt(O_WS_BN);
  if (force_bn > 0 && force_bn % 16 == 0 && force_bn <= 256 && N % force_bn == 0) best_bn = force_bn;
  if (best_bn == 0) return false;
  c->bn = best_bn;
  const long long slabs = N / best_bn;
  const long long per = sms / slabs;
  c->grid = static_cast<int>(slabs * (tiles_m < per ? tiles_m : per));
  const int force_grid = opt(O_WS_GRID);
  if (force_grid > 0 && force_grid <= sms) c->grid = force_grid;
  const int force_stat = opt(O_WS_STATIONARY), force_sa = opt(O_WS_SA);
  const int force_ws = opt(O_WS_WS), force_nbb = opt(O_WS_NBB);
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


// A one-CTA kernel whose only job is to let a bounded wait run out: it initialises an mbarrier that nothing
// ever arrives on, waits for it with the given poll limit, and leaves kStatusDebugTimeout in the status word.
// Exercises the error path of the kernels' waits (status set, kernel returns) without hanging anything.
constexpr int kStatusDebugTimeout = 0x7E57;
__global__ void debug_wait_timeout_kernel(uint32_t poll_limit, int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    arcq::mbar_init(&bar, 1);
    arcq::mbar_fence_init();
  }
  __syncthreads();
  const bool ok = arcq::mbar_wait_sleep_a(arcq::smem_u32(&bar), 0u, poll_limit, 32);
  if (!ok && threadIdx.x == 0) atomicExch(status, kStatusDebugTimeout);
}

// ---- CTA-pair kernel: configuration ----
struct PairConfig {
  int bn, ws, sa, ks, nbb, stationary, lut_shift, pairs;
  size_t smem;
};

// How many two-CTA clusters of the pair kernel can be resident at once (each takes two whole SMs).
int max_resident_pairs(int bits, size_t smem) {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev == cached_dev && cached > 0) return cached;
  int n = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sm_count() / 2 * 2));
  cfg.blockDim = dim3(arcq::kPairThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaErrorUnknown;
  if (bits == 4) e = cudaOccupancyMaxActiveClusters(&n, arcq::packed_weight_gemm_pair_kernel<4, true>, &cfg);
  else if (bits == 3) e = cudaOccupancyMaxActiveClusters(&n, arcq::packed_weight_gemm_pair_kernel<3, true>, &cfg);
  else e = cudaOccupancyMaxActiveClusters(&n, arcq::packed_weight_gemm_pair_kernel<2, true>, &cfg);
  if (e != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = sm_count() / 2;
  }
  if (n > sm_count() / 2) n = sm_count() / 2;
  cached = n;
  cached_dev = dev;
  return n;
}

template <int B>
cudaError_t pair_set_smem(size_t smem) {
  cudaError_t e = cudaFuncSetAttribute(arcq::packed_weight_gemm_pair_kernel<B, true>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(arcq::packed_weight_gemm_pair_kernel<B, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(smem));
}

// Slab width, stages and grid for the CTA-pair kernel; false when the shape is left to the one-CTA kernel
// (small M, N without a slab width that is a multiple of 32, ...).  The cost model counts tensor-pipe
// cycles per SM: a 256 x bn x 64 stage is four instructions of bn/2 cycles each; rebuilding one
// [bn/2 x 64] sub-tile costs about 300 + 6.5 * bn/2 cycles on the eight producer warps.
bool choose_pair_config(long long M, long long N, long long K, int bits, bool y_f32, PairConfig* c) {
  if (opt(O_PAIR) == 0 || M < opt(O_PAIR_MIN_M)) return false;
  const int G = static_cast<int>(K / 64);
  if (G < 1 || G > 64) return false;
  const long long tiles_m = (M + arcq::kPairTileM - 1) / arcq::kPairTileM;
  const size_t full_smem = kSmemBudget + 1024;
  {
    // raise the kernel's dynamic shared-memory ceiling once per (host thread, device, code width)
    static thread_local int done_dev[5] = {-1, -1, -1, -1, -1};
    int dev = 0;
    cudaGetDevice(&dev);
    if (done_dev[bits] != dev) {
      if (bits == 4 ? pair_set_smem<4>(full_smem) != cudaSuccess
                    : bits == 3 ? pair_set_smem<3>(full_smem) != cudaSuccess : pair_set_smem<2>(full_smem) != cudaSuccess) {
        cudaGetLastError();
        return false;
      }
      done_dev[bits] = dev;
    }
  }
  int max_pairs = max_resident_pairs(bits, full_smem);
  if (opt(O_PAIR_PAIRS) > 0 && opt(O_PAIR_PAIRS) < max_pairs) max_pairs = opt(O_PAIR_PAIRS);
  static const int cand[] = {192, 160, 128, 96, 64, 32};     // at most arcq::kPairMaxBn
  double best_cost = 0;
  bool found = false;
  PairConfig best = {};
  for (int bn : cand) {
    if (N % bn != 0) continue;
    if (opt(O_PAIR_BN) > 0 && bn != opt(O_PAIR_BN)) continue;
    const long long slabs = N / bn;
    if (slabs > max_pairs) continue;
    const int hb = bn / 2;
    long long per = max_pairs / slabs;
    if (per > tiles_m) per = tiles_m;
    const long long tiles_pp = (tiles_m + per - 1) / per;
    // Cost model in microseconds, constants from time stamps taken inside the kernel on the DeiT shapes: a tile is
    // bound by its output stores (about 22 GB/s per SM) or by the issuing thread (about 110 cycles per
    // instruction plus 0.15 us per stage); a sub-tile rebuild takes 0.12 + 0.0026 * rows us when both warp
    // groups build (stationary slab) and about twice that when only the weight warps do (streaming ring).
    const int esize = y_f32 ? 4 : 2;
    const double t_write = 128.0 * bn * esize / 22.0e3;
    const double t_l2 = static_cast<double>(slabs) * M * K * 2.0 / 5.0e6;    // every slab streams the whole activation
    for (int stationary = 1; stationary >= 0; --stationary) {
      if (opt(O_PAIR_STATIONARY) >= 0 && stationary != opt(O_PAIR_STATIONARY)) continue;
      PairConfig k = {};
      k.bn = bn; k.stationary = stationary; k.pairs = static_cast<int>(slabs * per);
      k.nbb = stationary ? 1 : 2;
      if (opt(O_PAIR_NBB) == 1 || opt(O_PAIR_NBB) == 2) k.nbb = opt(O_PAIR_NBB);
      // two 64-wide sub-tiles per stage: one wait and one pair of commits per eight instructions keeps the
      // issuing thread ahead of the tensor pipe
      k.ks = (G % 2 == 0) ? 2 : (G % 3 == 0) ? 3 : 1;
      if (opt(O_PAIR_KS) > 0 && G % opt(O_PAIR_KS) == 0) k.ks = opt(O_PAIR_KS);
      k.ws = stationary ? G : (opt(O_PAIR_WS) > 0 ? opt(O_PAIR_WS) : (k.ks == 2 || k.ks == 3 ? 6 : 4));
      if (!stationary && k.ws > G) k.ws = G;
      if (k.ws > (stationary ? 32 : 16) || k.ws < k.ks || (!stationary && k.ws % k.ks != 0)) continue;
      // eight copies of the pair table (more did not measure faster); as many A stages as fit, eight sub-stages at most
      bool fits = false;
      for (int lut = (opt(O_PAIR_LUT) > 0 ? opt(O_PAIR_LUT) : 3); lut >= 3 && !fits; --lut) {
        for (int sa = 8; sa >= 2 && !fits; --sa) {
          if (opt(O_PAIR_SA) > 0 && sa != opt(O_PAIR_SA)) continue;
          if (sa * k.ks > 8 && opt(O_PAIR_SA) == 0) continue;            // eight 16 KB sub-stages are plenty
          const size_t need = arcq::pair_smem_layout(bn, k.ws, sa, k.ks, G, stationary != 0, lut).total;
          if (need <= kSmemBudget) {
            k.sa = sa; k.lut_shift = lut; k.smem = need + 1024; fits = true;
          }
        }
        if (opt(O_PAIR_LUT) > 0) break;
      }
      if (!fits) continue;
      const double t_issue = (G / k.ks) * (k.ks * 4 * 0.056 + 0.15);
      double cost;
      if (stationary) {
        const double t_tile = (t_write > t_issue ? t_write : t_issue) + 0.15;
        const double path = G * (0.12 + 0.0026 * hb) + tiles_pp * t_tile;
        cost = 2.2 + (path > t_l2 ? path : t_l2);
      } else {
        double path = 0;
        for (long long t = 0; t < tiles_pp; t += k.nbb) {
          const long long nb = (tiles_pp - t) < k.nbb ? (tiles_pp - t) : k.nbb;
          const double build = G * (0.25 + 0.0055 * hb), issue = nb * t_issue;
          path += (build > issue ? build : issue) * 1.2 + nb * (t_write + 0.15);
        }
        cost = 2.2 + (path > t_l2 ? path : t_l2);
      }
      if (!found || cost < best_cost) { best = k; best_cost = cost; found = true; }
    }
  }
  if (!found) return false;
  *c = best;
  return true;
}


// ---- dense-weight CTA-pair kernel: configuration ----
struct PairDenseConfig {
  int bn, sa, ks, pairs, stationary;
  size_t smem;
};

int max_resident_dense_pairs(size_t smem) {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev == cached_dev && cached > 0) return cached;
  int n = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sm_count() / 2 * 2));
  cfg.blockDim = dim3(arcq::kPairDenseThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, arcq::dense_weight_gemm_pair_kernel<true>, &cfg);
  if (e != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = sm_count() / 2;
  }
  if (n > sm_count() / 2) n = sm_count() / 2;
  cached = n;
  cached_dev = dev;
  return n;
}

// Slab width, stages and grid for the dense-weight pair kernel; false leaves the shape to the one-CTA kernel.
// Cost model in microseconds, same constants as the packed-weight pair kernel's: a tile is bound by its output
// stores (about 22 GB/s per SM) or by the issuing thread, and every slab streams the whole activation from L2.
bool choose_pair_dense_config(long long M, long long N, long long K, bool y_f32, PairDenseConfig* c) {
  // No row threshold (ARCQ_PAIR_MIN_M gates the packed-weight pair kernel only): with nothing to rebuild, the pair
  // form measured faster than the one-CTA form from one row tile on (DeiT-S batch 1: 0.55 against 0.68 ms).
  if (opt(O_PAIR) == 0) return false;
  const int G = static_cast<int>(K / 64);
  if (G < 1) return false;
  const long long tiles_m = (M + arcq::kPairTileM - 1) / arcq::kPairTileM;
  const size_t full_smem = kSmemBudget + 1024;
  {
    static thread_local int done_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (done_dev != dev) {
      if (cudaFuncSetAttribute(arcq::dense_weight_gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(full_smem)) != cudaSuccess ||
          cudaFuncSetAttribute(arcq::dense_weight_gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(full_smem)) != cudaSuccess) {
        cudaGetLastError();
        return false;
      }
      done_dev = dev;
    }
  }
  int max_pairs = max_resident_dense_pairs(full_smem);
  if (opt(O_PAIR_PAIRS) > 0 && opt(O_PAIR_PAIRS) < max_pairs) max_pairs = opt(O_PAIR_PAIRS);
  static const int cand[] = {256, 192, 160, 128, 96, 64, 32};
  double best_cost = 0;
  bool found = false;
  PairDenseConfig best = {};
  // One or two row tiles (batch 1-2 of a ViT): the launch is a latency chain, not a throughput problem.  The
  // narrowest slab that still gives every (tile, slab) its own pair spreads the epilogue over the most SMs
  // (DeiT-S batch 1: 0.528 ms with 32-column slabs against 0.555 ms with the throughput model's choice).
  int narrow_bn = 0;
  if (tiles_m <= 2 && opt(O_PAIR_BN) == 0)
    for (int bn : cand)
      if (N % bn == 0 && (N / bn) * tiles_m <= max_pairs) narrow_bn = bn;      // candidates descend: keeps the narrowest
  for (int bn : cand) {
    if (N % bn != 0) continue;
    if (opt(O_PAIR_BN) > 0 && bn != opt(O_PAIR_BN)) continue;
    if (narrow_bn != 0 && bn != narrow_bn) continue;
    const long long slabs = N / bn;
    if (slabs > max_pairs) continue;
    long long per = max_pairs / slabs;
    if (per > tiles_m) per = tiles_m;
    const long long tiles_pp = (tiles_m + per - 1) / per;
    const int esize = y_f32 ? 4 : 2;
    const double t_write = 128.0 * bn * esize / 22.0e3;
    for (int stationary = 1; stationary >= 0; --stationary) {
      if (opt(O_PAIR_STATIONARY) >= 0 && stationary != opt(O_PAIR_STATIONARY)) continue;
      if (stationary && G > 32) continue;
      PairDenseConfig k = {};
      k.bn = bn; k.pairs = static_cast<int>(slabs * per); k.stationary = stationary;
      k.ks = (G % 2 == 0) ? 2 : (G % 3 == 0) ? 3 : 1;
      if (opt(O_PAIR_KS) > 0 && G % opt(O_PAIR_KS) == 0) k.ks = opt(O_PAIR_KS);
      bool fits = false;
      for (int sa = 16; sa >= 2 && !fits; --sa) {
        if (opt(O_PAIR_SA) > 0 && sa != opt(O_PAIR_SA)) continue;
        if (sa * k.ks > 8 && opt(O_PAIR_SA) == 0) continue;             // eight sub-stages in flight are plenty
        const size_t need = arcq::pair_dense_smem_layout(bn, sa, k.ks, G, stationary != 0).total;
        if (need <= kSmemBudget) { k.sa = sa; k.smem = need + 1024; fits = true; }
      }
      if (!fits) continue;
      if (stationary && opt(O_PAIR_STATIONARY) < 0 && (k.sa * k.ks < 4 || tiles_pp < 3))
        continue;   // too little room left for A, or too few tiles to pay for loading the whole slab first
      const double t_issue = (G / k.ks) * (k.ks * 4 * (bn > 128 ? 0.056 * bn / 192.0 : 0.04) + 0.1);
      // shared-memory fill through L2, about 8 TB/s over the machine: every tile streams its A rows, and its
      // W16 rows too unless the slab is stationary
      const double fill_mb = (static_cast<double>(slabs) * M * K * 2.0 +
                              (stationary ? static_cast<double>(k.pairs) : static_cast<double>(slabs * tiles_m)) * bn * K * 2.0) / 1.0e6;
      const double t_fill = fill_mb / 8.0;
      // 0.45 us per tile that neither the stores nor the issue account for (measured: at equal store volume, 192-wide
      // slabs beat 128-wide ones on N = 1152 by 1 us over 5 against 7 tiles per pair)
      const double path = tiles_pp * ((t_write > t_issue ? t_write : t_issue) + 0.45) * (stationary ? 0.95 : 1.0);
      const double cost = 1.5 + (path > t_fill ? path : t_fill);
      if (!found || cost < best_cost) { best = k; best_cost = cost; found = true; }
    }
  }
  if (!found) return false;
  *c = best;
  return true;
}

}  // namespace

extern "C" {

int arcq_version(void) { return ARCQ_B200_VERSION; }

const char* arcq_last_error_string(void) { return g_err; }

int arcq_debug_trace(void* device_buffer) {
  g_trace_buf = static_cast<long long*>(device_buffer);
  return ARCQ_OK;
}

int arcq_debug_set_option(const char* name, int value) {
  if (name == nullptr) return fail(ARCQ_E_BAD_ARG, "null option name");
  load_options();
  for (int i = 0; i < O_COUNT; ++i) {
    if (strcmp(name, kOptDefs[i].name) == 0) {
      g_opt[i] = value;
      return ARCQ_OK;
    }
  }
  return fail(ARCQ_E_BAD_ARG, "unknown option %s", name);
}

int arcq_debug_last_gemm_kernel(void) { return g_last_gemm_kernel; }

int arcq_debug_get_option(const char* name, int* value_out) {
  if (name == nullptr || value_out == nullptr) return fail(ARCQ_E_BAD_ARG, "null argument");
  load_options();
  for (int i = 0; i < O_COUNT; ++i) {
    if (strcmp(name, kOptDefs[i].name) == 0) {
      *value_out = g_opt[i];
      return ARCQ_OK;
    }
  }
  return fail(ARCQ_E_BAD_ARG, "unknown option %s", name);
}

int arcq_debug_wait_timeout(unsigned poll_limit, void* stream) {
  if (poll_limit > (1u << 16)) return fail(ARCQ_E_BAD_ARG, "poll_limit above 65536: this entry point is for short waits");
  int* st = status_ptr();
  if (st == nullptr) return fail(ARCQ_E_CUDA, "device status word not reachable");
  debug_wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(poll_limit, st);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "debug_wait_timeout launch");
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
      launch_pdl(arcq::packed_gemm_kernel<B>, grid, arcq::kGemmThreads, smem, st, p);                         \
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
  g_last_gemm_kernel = dense ? ARCQ_GEMM_ONE_CTA_DENSE : ARCQ_GEMM_ONE_CTA_PACKED;
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
  const bool use_tma_store = (cfg.bn % out_cw == 0) && opt(O_WS_TMA_STORE) != 0;
  CUtensorMap tm_y;
  if (!make_tensor_map_2d(&tm_y, y, (y_dtype == ARCQ_DT_F32) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                          (y_dtype == ARCQ_DT_F32) ? 4 : 2, static_cast<uint64_t>(M), static_cast<uint64_t>(N),
                          out_cw, 32, CU_TENSOR_MAP_SWIZZLE_64B))
    return fail(ARCQ_E_CUDA, "cuTensorMapEncodeTiled failed for the output matrix");

  arcq::WsParams p;
  p.tma_store = use_tma_store ? 1 : 0;
  p.rotate = opt(O_WS_ROTATE);
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
#define ARCQ_LAUNCH_WS_T(B, T)                                                                                     \
  do {                                                                                                             \
    e = cudaFuncSetAttribute(arcq::packed_weight_gemm_ws_kernel<B, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                             static_cast<int>(cfg.smem));                                                          \
    if (e == cudaSuccess) {                                                                                        \
      launch_pdl(arcq::packed_weight_gemm_ws_kernel<B, T>, cfg.grid, arcq::kWsThreads, cfg.smem, st, tm_a, tm_w, tm_y, p); \
      e = cudaGetLastError();                                                                                      \
    }                                                                                                              \
  } while (0)
  // the instantiation with time stamps runs only while arcq_debug_trace() has a buffer registered
#define ARCQ_LAUNCH_WS(B)                                                                                          \
  do {                                                                                                             \
    if (p.trace != nullptr) ARCQ_LAUNCH_WS_T(B, true);                                                             \
    else ARCQ_LAUNCH_WS_T(B, false);                                                                               \
  } while (0)
  if (bits == 4) ARCQ_LAUNCH_WS(4);
  else if (bits == 3) ARCQ_LAUNCH_WS(3);
  else ARCQ_LAUNCH_WS(2);
#undef ARCQ_LAUNCH_WS_T
#undef ARCQ_LAUNCH_WS
  if (e != cudaSuccess) return cuda_fail(e, "packed_weight_gemm launch");
  return ARCQ_OK;
}

// Launch of the CTA-pair kernel (packed weight form only).  Arguments are already validated.
static int launch_pair_gemm(const PairConfig& cfg, const void* xhat, const void* w, const float* mu_w,
                            const float* sigma_w, const float* codesum_w, const float* w_codebook, const float* bias,
                            int bits, int64_t M, int64_t N, int64_t K, void* y, int y_dtype, void* stream) {
  CUtensorMap tm_a, tm_y;
  if (!make_tensor_map_2d(&tm_a, xhat, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, static_cast<uint64_t>(M),
                          static_cast<uint64_t>(K), 64, arcq::kTileM, CU_TENSOR_MAP_SWIZZLE_128B))
    return fail(ARCQ_E_CUDA, "cuTensorMapEncodeTiled failed for the activation matrix");
  const int out_cw = (y_dtype == ARCQ_DT_F32) ? 16 : 32;
  if (!make_tensor_map_2d(&tm_y, y, (y_dtype == ARCQ_DT_F32) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                          (y_dtype == ARCQ_DT_F32) ? 4 : 2, static_cast<uint64_t>(M), static_cast<uint64_t>(N),
                          out_cw, 32, CU_TENSOR_MAP_SWIZZLE_64B))
    return fail(ARCQ_E_CUDA, "cuTensorMapEncodeTiled failed for the output matrix");
  arcq::PairParams p;
  p.pw = static_cast<const uint8_t*>(w); p.pc = static_cast<int>(K * bits / 8);
  p.mu_w = mu_w; p.sg_w = sigma_w; p.cs_w = codesum_w; p.cb_w = w_codebook; p.bias = bias; p.y = y;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K); p.G = static_cast<int>(K / 64);
  p.bn = cfg.bn; p.ws = cfg.ws; p.sa = cfg.sa; p.ks = cfg.ks; p.nbb = cfg.nbb; p.stationary = cfg.stationary;
  p.lut_shift = cfg.lut_shift;
  p.y_f32 = (y_dtype == ARCQ_DT_F32) ? 1 : 0;
  p.poll_limit = static_cast<uint32_t>(opt(O_POLL_LIMIT));
  p.spin_limit = static_cast<uint32_t>(opt(O_SPIN_LIMIT));
  p.status = status_ptr();
  if (p.status == nullptr) return fail(ARCQ_E_CUDA, "device status word not reachable");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(2 * cfg.pairs);
  // the dynamic shared-memory ceiling of the kernel was raised when the configuration was chosen
#define ARCQ_LAUNCH_PAIR(B)                                                                                              \
  do {                                                                                                                  \
    if (cfg.stationary)                                                                                                 \
      launch_pdl(arcq::packed_weight_gemm_pair_kernel<B, true>, grid, arcq::kPairThreads, cfg.smem, st, tm_a, tm_y, p);  \
    else                                                                                                                \
      launch_pdl(arcq::packed_weight_gemm_pair_kernel<B, false>, grid, arcq::kPairThreads, cfg.smem, st, tm_a, tm_y, p); \
  } while (0)
  if (bits == 4) ARCQ_LAUNCH_PAIR(4);
  else if (bits == 3) ARCQ_LAUNCH_PAIR(3);
  else ARCQ_LAUNCH_PAIR(2);
#undef ARCQ_LAUNCH_PAIR
  g_last_gemm_kernel = ARCQ_GEMM_PAIR_PACKED;
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "packed_weight_gemm (pair) launch");
  return ARCQ_OK;
}

static int launch_pair_dense_gemm(const PairDenseConfig& cfg, const void* xhat, const void* w16, const float* bias,
                                  int64_t M, int64_t N, int64_t K, void* y, int y_dtype, void* stream,
                                  const arcq::UnpackWeightJob* next = nullptr) {
  CUtensorMap tm_a, tm_w, tm_y;
  if (!make_tensor_map_2d(&tm_a, xhat, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, static_cast<uint64_t>(M),
                          static_cast<uint64_t>(K), 64, arcq::kTileM, CU_TENSOR_MAP_SWIZZLE_128B))
    return fail(ARCQ_E_CUDA, "cuTensorMapEncodeTiled failed for the activation matrix");
  if (!make_tensor_map_2d(&tm_w, w16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, static_cast<uint64_t>(N),
                          static_cast<uint64_t>(K), 64, cfg.bn / 2, CU_TENSOR_MAP_SWIZZLE_128B))
    return fail(ARCQ_E_CUDA, "cuTensorMapEncodeTiled failed for the weight matrix");
  const int out_cw = (y_dtype == ARCQ_DT_F32) ? 16 : 32;
  if (!make_tensor_map_2d(&tm_y, y, (y_dtype == ARCQ_DT_F32) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                          (y_dtype == ARCQ_DT_F32) ? 4 : 2, static_cast<uint64_t>(M), static_cast<uint64_t>(N),
                          out_cw, 32, CU_TENSOR_MAP_SWIZZLE_64B))
    return fail(ARCQ_E_CUDA, "cuTensorMapEncodeTiled failed for the output matrix");
  arcq::PairDenseParams p;
  p.bias = bias;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K); p.G = static_cast<int>(K / 64);
  p.bn = cfg.bn; p.sa = cfg.sa; p.ks = cfg.ks;
  p.y_f32 = (y_dtype == ARCQ_DT_F32) ? 1 : 0;
  p.poll_limit = static_cast<uint32_t>(opt(O_POLL_LIMIT));
  p.spin_limit = static_cast<uint32_t>(opt(O_SPIN_LIMIT));
  p.status = status_ptr();
  if (p.status == nullptr) return fail(ARCQ_E_CUDA, "device status word not reachable");
  p.next = arcq::UnpackWeightJob{};
  if (next != nullptr) p.next = *next;
  const unsigned grid = static_cast<unsigned>(2 * cfg.pairs);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (next != nullptr) {
    static thread_local int done_dev = -1;      // the prefetch form's shared-memory ceiling, once per (thread, device)
    int dev = 0;
    cudaGetDevice(&dev);
    if (done_dev != dev) {
      cudaFuncSetAttribute(arcq::dense_weight_gemm_pair_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kSmemBudget + 1024));
      cudaFuncSetAttribute(arcq::dense_weight_gemm_pair_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kSmemBudget + 1024));
      done_dev = dev;
    }
    if (cfg.stationary)
      launch_pdl(arcq::dense_weight_gemm_pair_kernel<true, true>, grid, arcq::kPairDenseThreads, cfg.smem, st, tm_a, tm_w, tm_y, p);
    else
      launch_pdl(arcq::dense_weight_gemm_pair_kernel<false, true>, grid, arcq::kPairDenseThreads, cfg.smem, st, tm_a, tm_w, tm_y, p);
  } else if (cfg.stationary) {
    launch_pdl(arcq::dense_weight_gemm_pair_kernel<true>, grid, arcq::kPairDenseThreads, cfg.smem, st, tm_a, tm_w, tm_y, p);
  } else {
    launch_pdl(arcq::dense_weight_gemm_pair_kernel<false>, grid, arcq::kPairDenseThreads, cfg.smem, st, tm_a, tm_w, tm_y, p);
  }
  g_last_gemm_kernel = next != nullptr ? ARCQ_GEMM_PAIR_DENSE_PREFETCH : ARCQ_GEMM_PAIR_DENSE;
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "dense_weight_gemm (pair) launch");
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
  PairConfig pc;
  if (choose_pair_config(M, N, K, bits, y_dtype == ARCQ_DT_F32, &pc))
    return launch_pair_gemm(pc, xhat, packed_w, mu_w, sigma_w, codesum_w, w_codebook, bias, bits, M, N, K, y, y_dtype,
                            stream);
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
  PairDenseConfig pc;
  if (choose_pair_dense_config(M, N, K, y_dtype == ARCQ_DT_F32, &pc))
    return launch_pair_dense_gemm(pc, xhat, w16, bias, M, N, K, y, y_dtype, stream);
  return launch_ws_gemm(true, xhat, w16, nullptr, nullptr, nullptr, nullptr, bias, 4, M, N, K, y, y_dtype, stream);
}

int arcq_dense_weight_gemm_prefetch(const void* xhat, const void* w16, const float* bias, int64_t M, int64_t N,
                                    int64_t K, void* y, int y_dtype, const uint8_t* next_packed, const float* next_mu,
                                    const float* next_sigma, const float* next_codesum, const float* next_codebook,
                                    int next_bits, int next_group_size, int64_t next_rows, int64_t next_K,
                                    void* next_out, void* stream) {
  if (!next_packed || !next_mu || !next_sigma || !next_codesum || !next_codebook || !next_out)
    return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (next_bits < 2 || next_bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", next_bits);
  if (next_group_size != 64) return fail(ARCQ_E_UNSUPPORTED, "group_size %d: only 64 is built", next_group_size);
  if (next_rows <= 0 || next_K <= 0 || next_K % 64 != 0)
    return fail(ARCQ_E_BAD_SHAPE, "bad shape of the next weight: rows=%lld K=%lld", (long long)next_rows, (long long)next_K);
  if (!aligned(next_packed, 4) || !aligned(next_out, 16))
    return fail(ARCQ_E_ALIGN, "next packed codes must be 4-byte, next_out 16-byte aligned");
  if (!xhat || !w16 || !y) return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (y_dtype != ARCQ_DT_F16 && y_dtype != ARCQ_DT_F32) return fail(ARCQ_E_BAD_ARG, "y_dtype must be f16 or f32");
  if (M < 0 || N <= 0 || K <= 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape M=%lld N=%lld K=%lld", (long long)M,
                                              (long long)N, (long long)K);
  if (K % 64 != 0) return fail(ARCQ_E_UNSUPPORTED, "K=%lld: this entry point needs K %% 64 == 0", (long long)K);
  if (N % 16 != 0) return fail(ARCQ_E_UNSUPPORTED, "N=%lld: this entry point needs N %% 16 == 0", (long long)N);
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > (1 << 20)) return fail(ARCQ_E_TOO_LARGE, "shape too large");
  if (!aligned(xhat, 16) || !aligned(w16, 16) || !aligned(y, 16))
    return fail(ARCQ_E_ALIGN, "xhat, w16 and y must be 16-byte aligned");
  const arcq::UnpackWeightJob job = {next_packed, next_mu, next_sigma, next_codesum, next_codebook,
                                     static_cast<__half*>(next_out), static_cast<long long>(next_rows),
                                     static_cast<int>(next_K), next_bits};
  PairDenseConfig pc;
  if (M > 0 && choose_pair_dense_config(M, N, K, y_dtype == ARCQ_DT_F32, &pc))
    return launch_pair_dense_gemm(pc, xhat, w16, bias, M, N, K, y, y_dtype, stream, &job);
  // no pair configuration (or nothing to multiply): the GEMM by the one-CTA kernel, the unpack by its own kernel
  if (M > 0) {
    const int rc = launch_ws_gemm(true, xhat, w16, nullptr, nullptr, nullptr, nullptr, bias, 4, M, N, K, y, y_dtype, stream);
    if (rc != ARCQ_OK) return rc;
  }
  return arcq_unpack_weight_f16(next_packed, next_mu, next_sigma, next_codesum, next_codebook, next_bits, next_group_size,
                                next_rows, next_K, next_out, stream);
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
  const bool plain = opt(O_LN_PLAIN) != 0;
  if (K == 384 && !plain) {          // 16 lanes per row, 2 rows per warp
    launch_pdl(arcq::add_layernorm_rows_kernel<16>, grid_for(M, 16, 6), 256, 0, st, xh, yh, gamma, beta, eps, M, so, ho);
  } else if (K == 192 && !plain) {
    launch_pdl(arcq::add_layernorm_rows_kernel<8>, grid_for(M, 32, 6), 256, 0, st, xh, yh, gamma, beta, eps, M, so, ho);
  } else if (K == 768 && !plain) {
    launch_pdl(arcq::add_layernorm_rows_kernel<32>, grid_for(M, 8, 6), 256, 0, st, xh, yh, gamma, beta, eps, M, so, ho);
  } else {
    launch_pdl(arcq::add_layernorm_kernel, grid_for(M, 8, 8), 256, 0, st, xh, yh, gamma, beta, eps, M, static_cast<int>(K), so, ho);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "add_layernorm launch");
  return ARCQ_OK;
}

int arcq_add_layernorm_act_quant(const void* x, const void* y, const float* gamma, const float* beta, float eps,
                                 int64_t M, int64_t K, const float* thresholds, const float* codebook, int bits,
                                 int group_size, void* sum_out, void* h_out, void* xhat, void* stream) {
  if (x == nullptr || gamma == nullptr || beta == nullptr || thresholds == nullptr || codebook == nullptr || xhat == nullptr)
    return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (bits < 2 || bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", bits);
  if (group_size != 64) return fail(ARCQ_E_UNSUPPORTED, "group_size %d: only 64 is built", group_size);
  if (M < 0 || K <= 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape M=%lld K=%lld", (long long)M, (long long)K);
  if (K % 64 != 0) return fail(ARCQ_E_BAD_SHAPE, "K=%lld is not a multiple of the group size 64", (long long)K);
  if (K != 192 && K != 384 && K != 768)
    return fail(ARCQ_E_UNSUPPORTED, "K=%lld: the merged kernel is built for rows of 192, 384 and 768 values", (long long)K);
  if (y == nullptr && sum_out != nullptr) return fail(ARCQ_E_BAD_ARG, "sum_out without y");
  if (!aligned(x, 16) || !aligned(xhat, 16) || (y != nullptr && !aligned(y, 16)) ||
      (sum_out != nullptr && !aligned(sum_out, 16)) || (h_out != nullptr && !aligned(h_out, 16)))
    return fail(ARCQ_E_ALIGN, "all matrices must be 16-byte aligned");
  if (M == 0) return ARCQ_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int G = static_cast<int>(K / 64);
  {
    // Small inputs, where the tiled kernel's 128-group tiles would not give every SM a block: the twelve-warp
    // form (48 groups per block, lower latency).  Both forms give the same bits.  (DeiT-T at batch 64, 37 824
    // groups, measured 8 % slower through the small form than through the tiled one.)
    const bool small = M * G < static_cast<long long>(sm_count()) * arcq::kLnqThreads && opt(O_LNQ_SMALL) != 0;
    if (small) {
      const __half *xs = static_cast<const __half*>(x), *ys = static_cast<const __half*>(y);
      __half *so2 = static_cast<__half*>(sum_out), *ho2 = static_cast<__half*>(h_out), *xo2 = static_cast<__half*>(xhat);
      const int lanes = static_cast<int>(K / 24), rows_tile = 4 * (32 / lanes);
      const long long tiles2 = (M + rows_tile - 1) / rows_tile;
      const long long cap2 = static_cast<long long>(sm_count()) * 8;
      const unsigned grid2 = static_cast<unsigned>(tiles2 < cap2 ? tiles2 : cap2);
#define ARCQ_LAUNCH_LNQ_ROWS(LN, B, HASY)                                                                            \
  launch_pdl(arcq::add_layernorm_act_quant_rows_kernel<LN, B, HASY>, grid2, arcq::kLnqRowsThreads, 0, st, xs, ys, gamma, beta, eps,     \
             static_cast<long long>(M), thresholds, codebook, so2, ho2, xo2)
#define ARCQ_LNQ_ROWS_BITS(LN, HASY)                                                                                  \
  do {                                                                                                                \
    if (bits == 4) ARCQ_LAUNCH_LNQ_ROWS(LN, 4, HASY);                                                                  \
    else if (bits == 3) ARCQ_LAUNCH_LNQ_ROWS(LN, 3, HASY);                                                             \
    else ARCQ_LAUNCH_LNQ_ROWS(LN, 2, HASY);                                                                            \
  } while (0)
      if (y != nullptr) {
        if (lanes == 8) ARCQ_LNQ_ROWS_BITS(8, true); else if (lanes == 16) ARCQ_LNQ_ROWS_BITS(16, true); else ARCQ_LNQ_ROWS_BITS(32, true);
      } else {
        if (lanes == 8) ARCQ_LNQ_ROWS_BITS(8, false); else if (lanes == 16) ARCQ_LNQ_ROWS_BITS(16, false); else ARCQ_LNQ_ROWS_BITS(32, false);
      }
#undef ARCQ_LNQ_ROWS_BITS
#undef ARCQ_LAUNCH_LNQ_ROWS
      cudaError_t e2 = cudaGetLastError();
      if (e2 != cudaSuccess) return cuda_fail(e2, "add_layernorm_act_quant (rows) launch");
      return ARCQ_OK;
    }
  }
  const long long tiles = (M * G + arcq::kLnqThreads - 1) / arcq::kLnqThreads;
  const long long cap = static_cast<long long>(sm_count()) * 4;
  const unsigned grid = static_cast<unsigned>(tiles < cap ? tiles : cap);
  const size_t smem = arcq::lnq_smem_bytes();
  const __half *xh = static_cast<const __half*>(x), *yh = static_cast<const __half*>(y);
  __half *so = static_cast<__half*>(sum_out), *ho = static_cast<__half*>(h_out), *xo = static_cast<__half*>(xhat);
#define ARCQ_LAUNCH_LNQ(LN, B, HASY)                                                                                   \
  launch_pdl(arcq::add_layernorm_act_quant_kernel<LN, B, HASY>, grid, arcq::kLnqThreads, smem, st, xh, yh, gamma, beta, \
             eps, static_cast<long long>(M), thresholds, codebook, so, ho, xo)
#define ARCQ_LNQ_BITS(LN, HASY)                                                                                         \
  do {                                                                                                                  \
    if (bits == 4) ARCQ_LAUNCH_LNQ(LN, 4, HASY);                                                                         \
    else if (bits == 3) ARCQ_LAUNCH_LNQ(LN, 3, HASY);                                                                    \
    else ARCQ_LAUNCH_LNQ(LN, 2, HASY);                                                                                   \
  } while (0)
  {
    const int lanes = static_cast<int>(K / 24);
    if (y != nullptr) {
      if (lanes == 8) ARCQ_LNQ_BITS(8, true); else if (lanes == 16) ARCQ_LNQ_BITS(16, true); else ARCQ_LNQ_BITS(32, true);
    } else {
      if (lanes == 8) ARCQ_LNQ_BITS(8, false); else if (lanes == 16) ARCQ_LNQ_BITS(16, false); else ARCQ_LNQ_BITS(32, false);
    }
  }
#undef ARCQ_LNQ_BITS
#undef ARCQ_LAUNCH_LNQ
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "add_layernorm_act_quant launch");
  return ARCQ_OK;
}

static int launch_attention(const void* qkv, int64_t B, int64_t T, int64_t H, int head_dim, const float* thresholds,
                            const float* codebook, int bits, void* out, void* stream) {
  if (qkv == nullptr || out == nullptr) return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (head_dim != 64) return fail(ARCQ_E_UNSUPPORTED, "head_dim %d: only 64 is built", head_dim);
  if (B < 0 || T <= 0 || H <= 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape B=%lld T=%lld H=%lld", (long long)B, (long long)T, (long long)H);
  if (T > arcq::kAttnMaxT) return fail(ARCQ_E_TOO_LARGE, "sequences longer than %d tokens are not built", arcq::kAttnMaxT);
  if (B * H > 0x7fffffffLL) return fail(ARCQ_E_TOO_LARGE, "too many (image, head) pairs");
  if (!aligned(qkv, 16) || !aligned(out, 16)) return fail(ARCQ_E_ALIGN, "qkv and out must be 16-byte aligned");
  if (B == 0) return ARCQ_OK;
  arcq::AttnParams p;
  p.qkv = static_cast<const __half*>(qkv);
  p.out = static_cast<__half*>(out);
  p.B = static_cast<int>(B); p.T = static_cast<int>(T); p.H = static_cast<int>(H);
  p.tp = static_cast<int>((T + 15) / 16 * 16);
  p.thresholds = thresholds;
  p.codebook = codebook;
  const size_t smem = arcq::attn_smem_bytes(p.tp);
  const unsigned grid = static_cast<unsigned>(B * H);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define ARCQ_LAUNCH_ATTN(Q, BT)                                                                                      \
  do {                                                                                                                \
    static thread_local int done_dev = -1;                                                                            \
    int dev = 0;                                                                                                      \
    cudaGetDevice(&dev);                                                                                              \
    if (done_dev != dev) {                                                                                            \
      cudaFuncSetAttribute(arcq::attention_kernel<Q, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize,                \
                           static_cast<int>(arcq::attn_smem_bytes(arcq::kAttnMaxT)));                                 \
      done_dev = dev;                                                                                                 \
    }                                                                                                                 \
    launch_pdl(arcq::attention_kernel<Q, BT>, grid, arcq::kAttnThreads, smem, st, p);                                 \
  } while (0)
  if (thresholds == nullptr) ARCQ_LAUNCH_ATTN(false, 4);
  else if (bits == 4) ARCQ_LAUNCH_ATTN(true, 4);
  else if (bits == 3) ARCQ_LAUNCH_ATTN(true, 3);
  else ARCQ_LAUNCH_ATTN(true, 2);
#undef ARCQ_LAUNCH_ATTN
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "attention launch");
  return ARCQ_OK;
}

int arcq_attention(const void* qkv, int64_t B, int64_t T, int64_t H, int head_dim, void* out, void* stream) {
  return launch_attention(qkv, B, T, H, head_dim, nullptr, nullptr, 4, out, stream);
}

int arcq_attention_act_quant(const void* qkv, int64_t B, int64_t T, int64_t H, int head_dim, const float* thresholds,
                             const float* codebook, int bits, int group_size, void* xhat, void* stream) {
  if (thresholds == nullptr || codebook == nullptr) return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (bits < 2 || bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", bits);
  if (group_size != 64) return fail(ARCQ_E_UNSUPPORTED, "group_size %d: only 64 is built", group_size);
  return launch_attention(qkv, B, T, H, head_dim, thresholds, codebook, bits, xhat, stream);
}

int arcq_patchify(const void* images, int64_t B, int64_t C, int64_t H, int64_t W, int patch, void* rows, void* stream) {
  if (images == nullptr || rows == nullptr) return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (B < 0 || C <= 0 || H <= 0 || W <= 0 || patch <= 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape");
  if (patch % 8 != 0 || H % patch != 0 || W % patch != 0)
    return fail(ARCQ_E_UNSUPPORTED, "patch %d: must be a multiple of 8 that divides H=%lld and W=%lld", patch, (long long)H, (long long)W);
  if (B * C * H * W > 0x7fffffffffLL) return fail(ARCQ_E_TOO_LARGE, "image batch too large");
  if (!aligned(images, 16) || !aligned(rows, 16)) return fail(ARCQ_E_ALIGN, "images and rows must be 16-byte aligned");
  if (B == 0) return ARCQ_OK;
  const long long chunks = B * C * H * W / 8;
  launch_pdl(arcq::patchify_kernel, grid_for(chunks, 256, 8), 256, 0, static_cast<cudaStream_t>(stream),
             static_cast<const __half*>(images), static_cast<int>(B), static_cast<int>(C), static_cast<int>(H),
             static_cast<int>(W), patch, static_cast<__half*>(rows));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "patchify launch");
  return ARCQ_OK;
}

int arcq_assemble_tokens(const void* patches, const void* cls_token, const void* pos_embed, int64_t B, int64_t T, int64_t D,
                         void* tokens, void* stream) {
  if (patches == nullptr || cls_token == nullptr || pos_embed == nullptr || tokens == nullptr)
    return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (B < 0 || T <= 0 || D <= 0 || D % 8 != 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape B=%lld T=%lld D=%lld", (long long)B, (long long)T, (long long)D);
  if (!aligned(patches, 16) || !aligned(cls_token, 16) || !aligned(pos_embed, 16) || !aligned(tokens, 16))
    return fail(ARCQ_E_ALIGN, "all buffers must be 16-byte aligned");
  if (B == 0) return ARCQ_OK;
  const long long chunks = B * (T + 1) * (D / 8);
  launch_pdl(arcq::assemble_tokens_kernel, grid_for(chunks, 256, 8), 256, 0, static_cast<cudaStream_t>(stream),
             static_cast<const __half*>(patches), static_cast<const __half*>(cls_token),
             static_cast<const __half*>(pos_embed), static_cast<int>(B), static_cast<int>(T), static_cast<int>(D),
             static_cast<__half*>(tokens));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "assemble_tokens launch");
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

int arcq_unpack_weight_f16(const uint8_t* packed, const float* mu, const float* sigma, const float* codesum,
                           const float* codebook, int bits, int group_size, int64_t rows, int64_t K, void* out,
                           void* stream) {
  if (!packed || !mu || !sigma || !codesum || !codebook || !out) return fail(ARCQ_E_BAD_ARG, "null pointer argument");
  if (bits < 2 || bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", bits);
  if (group_size != 64) return fail(ARCQ_E_UNSUPPORTED, "group_size %d: only 64 is built", group_size);
  if (rows < 0 || K <= 0 || K % 64 != 0) return fail(ARCQ_E_BAD_SHAPE, "bad shape rows=%lld K=%lld", (long long)rows, (long long)K);
  if (!aligned(packed, 4) || !aligned(out, 16)) return fail(ARCQ_E_ALIGN, "packed codes must be 4-byte, out 16-byte aligned");
  if (rows == 0) return ARCQ_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(rows * (K / 8), 256, 8);
  const int k = static_cast<int>(K);
  __half* o = static_cast<__half*>(out);
  if (bits == 4) arcq::unpack_weight_f16_kernel<4><<<grid, 256, 0, st>>>(packed, mu, sigma, codesum, codebook, rows, k, o);
  else if (bits == 3) arcq::unpack_weight_f16_kernel<3><<<grid, 256, 0, st>>>(packed, mu, sigma, codesum, codebook, rows, k, o);
  else arcq::unpack_weight_f16_kernel<2><<<grid, 256, 0, st>>>(packed, mu, sigma, codesum, codebook, rows, k, o);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "unpack_weight_f16 launch");
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
  // everything the two launches below would reject is rejected here, before the first of them runs and
  // overwrites the shared scratch
  if (bits < 2 || bits > 4) return fail(ARCQ_E_BAD_ARG, "bits must be 2, 3 or 4, got %d", bits);
  if (y_dtype != ARCQ_DT_F16 && y_dtype != ARCQ_DT_F32) return fail(ARCQ_E_BAD_ARG, "y_dtype must be f16 or f32");
  if (K % 64 != 0) return fail(ARCQ_E_UNSUPPORTED, "K=%lld: this entry point needs K %% 64 == 0", (long long)K);
  if (N % 16 != 0) return fail(ARCQ_E_UNSUPPORTED, "N=%lld: this entry point needs N %% 16 == 0", (long long)N);
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > (1 << 20)) return fail(ARCQ_E_TOO_LARGE, "shape too large");
  if (!aligned(xhat, 16) || !aligned(y, 16)) return fail(ARCQ_E_ALIGN, "xhat and y must be 16-byte aligned");
  if (!aligned(packed_w, 4)) return fail(ARCQ_E_ALIGN, "packed codes must be 4-byte aligned");
  if (M > 0) {
    WsConfig probe;
    if (!choose_ws_config(M, N, K, 4, true, &probe)) return fail(ARCQ_E_UNSUPPORTED, "no tile configuration for this shape");
  }
  __half* const w16 = static_weight_scratch();
  if (w16 == nullptr) return ARCQ_E_CUDA;
  if (M == 0) return ARCQ_OK;
  const int rc = arcq_dequant(packed_w, mu_w, sigma_w, codesum_w, w_codebook, bits, group_size, N, K, w16,
                              ARCQ_DT_F16, stream);
  if (rc != ARCQ_OK) return rc;
  return arcq_dense_weight_gemm(xhat, w16, bias, M, N, K, y, y_dtype, stream);
}

}  // extern "C"
