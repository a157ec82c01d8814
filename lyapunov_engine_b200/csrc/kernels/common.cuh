// Shared by every kernel file: the C interface's conventions, element types,
// reductions and the device status word.
//
// Every launcher is `extern "C" int le_*(...)`: raw device pointers, sizes,
// a dtype code and the CUDA stream; it returns 0 or a cudaError_t, or
// LE_INVALID for arguments it refuses (le_last_error() then says why).  No
// launcher allocates or synchronises.
//
// The reference's helpers of the same kind are csrc/include/utils/cuda_utils.cuh
// (CUDA_CHECK, to_float/from_float, warp and block reductions).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#define LE_API extern "C" __attribute__((visibility("default")))

enum : int { LE_F32 = 0, LE_BF16 = 1 };
enum : int { LE_INVALID = -1 };

// Bits of the device status word that kernels set instead of faulting.
enum : int {
  LE_STATUS_BAD_TOKEN = 1,     // a token id outside the vocabulary
  LE_STATUS_BAD_PAGE = 2,      // a block table entry outside the pool
  LE_STATUS_BAD_POSITION = 4,  // a position outside the rotary table
  LE_STATUS_WAIT_TIMEOUT = 8,  // a bounded wait inside a kernel ran out
};

namespace le {

inline char *error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

inline int invalid(const char *fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(error_buffer(), 512, fmt, args);
  va_end(args);
  return LE_INVALID;
}

inline int launched() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) snprintf(error_buffer(), 512, "CUDA: %s", cudaGetErrorString(e));
  return static_cast<int>(e);
}

// Programmatic dependent launch: a kernel launched with launch_chained() may
// start while its predecessor in the stream still runs.  It must call
// wait_for_predecessor() before it reads anything the predecessor wrote and
// before it writes anything the predecessor may still read; what it does
// before that (address arithmetic, fetching weights) overlaps the predecessor's
// tail.  let_successor_start() lets the next kernel in the stream begin its own
// preamble.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_successor_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool chaining_enabled() {
  static const bool on = [] {
    const char *env = getenv("LYAPUNOV_PDL");
    return env == nullptr || env[0] != '0';
  }();
  return on;
}

template <typename... KernelArgs, typename... Args>
inline int launch_chained(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = chaining_enabled() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
  if (e != cudaSuccess) {
    snprintf(error_buffer(), 512, "CUDA: %s", cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  return launched();
}

// The same for a kernel whose blocks form thread-block clusters of `cluster_x`
// blocks along x (they are scheduled together and can read one another's shared
// memory); more than 8 to a cluster needs the kernel's non-portable attribute.
template <typename... KernelArgs, typename... Args>
inline int launch_chained_cluster(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  int cluster_x, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(cluster_x);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = chaining_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
  if (e != cudaSuccess) {
    snprintf(error_buffer(), 512, "CUDA: %s", cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  return launched();
}

// Every thread of every block of the cluster arrives; returns when all have.
// What a block wrote to its shared memory before is visible to the others after.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// A float at the same shared-memory address in block `rank` of the cluster.
__device__ __forceinline__ float cluster_peer_f32(const float *mine, unsigned rank) {
  const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(mine));
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Which keys a query at position p sees besides "none after itself", as one
// integer `reach`: 0: every key; r > 0: the last r keys (p - r + 1 .. p, a
// sliding window); r < 0: the keys of its own chunk of -r positions
// (floor(p / -r) * -r .. p; chunks are counted from position 0 of the request).
// The first visible key never decreases as p grows.
__host__ __device__ __forceinline__ int first_visible_key(int p, int reach) {
  if (reach > 0) return p - reach + 1 > 0 ? p - reach + 1 : 0;
  if (reach < 0) return p / (-reach) * (-reach);
  return 0;
}

// With `keep_first` n > 0 the keys at positions below n stay visible to every later query, whatever the window or
// chunk: a query at p sees key j <= p when j >= first_visible_key(p, reach) or j < n.
__host__ __device__ __forceinline__ bool key_visible(int j, int p, int lo, int keep_first) {
  return j <= p && (j >= lo || j < keep_first);
}

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// The 16 bytes at p (16-byte aligned) as floats: 8 bfloat16 or 4 float32 values.
template <typename T> struct Piece16 { static constexpr int COUNT = 16 / sizeof(T); };
template <typename T>
__device__ __forceinline__ void load_piece16(float (&dst)[Piece16<T>::COUNT], const T *p) {
  const uint4 raw = *reinterpret_cast<const uint4 *>(p);
  const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
  for (int v = 0; v < Piece16<T>::COUNT; ++v) dst[v] = to_f32(e[v]);
}

// 2^x in one instruction (ex2.approx, relative error about 2^-22, results
// below the normal range flush to zero); exp2f() spends several more on them.
// For softmax numerators in the bfloat16 kernels; the 32-bit path uses expf.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// e^x for factors that are multiplied up over many steps (the decays of a recurrence).  expf() is accurate to
// two units in the last place but leans to one side (its results average about 1.5e-8 too large, relatively, for
// small negative x on this device), and a thousand factors that lean the same way move a long memory by 1.5e-5,
// several times what unbiased rounding does.  Here: x = k ln 2 + r with ln 2 in two parts, a degree-7 polynomial
// for e^r on |r| <= ln 2 / 2 (coefficients of the Cephes library's expf), the result times 2^k.  Error below one
// unit in the last place, mean error below 2e-9 of the value.  Results below 2^-126 flush to about 1e-38.
__device__ __forceinline__ float exp_unbiased(float x) {
  x = fminf(fmaxf(x, -87.0f), 88.0f);
  const float k = rintf(x * 1.44269504f);
  float r = fmaf(k, -0.693145752f, x);
  r = fmaf(k, -1.42860677e-06f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  const float e = fmaf(r * r, p, r) + 1.0f;
  return e * __int_as_float((static_cast<int>(k) + 127) << 23);
}

// cap * tanh(x) with x = score / cap already: capped attention scores for the bfloat16 kernels.  tanh(x) = 1 -
// 2 / (2^(2 x log2 e) + 1) with ex2.approx and a fast division: absolute error about 1e-7 over the whole range
// (the exponential overflows to +inf, which gives 1, and underflows to 0, which gives -1).
__device__ __forceinline__ float capped_score(float x, float cap) {
  const float e = fast_exp2(x * 2.8853900817779268f);
  return cap * (1.0f - __fdividef(2.0f, e + 1.0f));
}

// Gated activations of a fused gate/up product, act(g, u), in 32 bits:
//   kind 0: silu(g) * u
//   kind 1: g' = min(g, limit), u' = clamp(u, -limit, limit); g' * sigmoid(slope * g') * (u' + 1)
//   kind 2: max(g, 0) * u
// `bias` (float32 [2 * inter], the gate's entries first, or null): what a
// product's epilogue adds to column n of g (bias[n]) and of u (bias[inter + n])
// before the activation (gated_bias()).
struct GatedActivation {
  int kind = 0;
  float slope = 1.0f;
  float limit = 0.0f;
  const float *bias = nullptr;
  int inter = 0;
};
__device__ __forceinline__ void gated_bias(float &g, float &u, int n, const GatedActivation &a) {
  if (a.bias != nullptr) g += a.bias[n], u += a.bias[a.inter + n];
}
template <bool FAST_EXP = false>
__device__ __forceinline__ float gated_activation(float g, float u, const GatedActivation &a) {
  if (a.kind == 1) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit) + 1.0f;
    if constexpr (FAST_EXP) return __fdividef(g, 1.0f + __expf(-a.slope * g)) * u;
    return g / (1.0f + expf(-a.slope * g)) * u;
  }
  if (a.kind == 2) return fmaxf(g, 0.0f) * u;
  if constexpr (FAST_EXP) return __fdividef(g, 1.0f + __expf(-g)) * u;
  return g / (1.0f + expf(-g)) * u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block; every thread gets it.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float s = lane < warps ? scratch[lane] : 0.0f;
    s = warp_sum(s);
    if (lane == 0) scratch[32] = s;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float s = lane < warps ? scratch[lane] : -INFINITY;
    s = warp_max(s);
    if (lane == 0) scratch[32] = s;
  }
  __syncthreads();
  return scratch[32];
}

}  // namespace le

#define LE_DISPATCH_DTYPE(code, T, ...)                                  \
  do {                                                                   \
    if ((code) == LE_F32) { using T = float; __VA_ARGS__; }              \
    else if ((code) == LE_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else return le::invalid("unknown dtype code %d", (code));            \
  } while (0)
