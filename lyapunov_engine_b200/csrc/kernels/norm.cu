// RMSNorm over the 32-bit residual stream, with the residual addition fused.
//
//   resid[r] += delta[0][r] + delta[1][r] + ...   (when delta is given)
//   out[r]    = resid[r] * rsqrt(mean(resid[r]^2) + eps) * weight
//
// With `delta_scale` (one number per column) the sum of the deltas is multiplied by it, in 32 bits, before it
// enters the stream: resid[r] += delta_scale * (delta[0][r] + ...).
//
// With `groups` > 1 a row is cut into that many equal consecutive parts and
// each part is divided by its own root mean square (one block per row and part).
//
// delta is the output of the sub-layer before the norm: one tensor in the
// activations' type, or the float32 partial sums of a split-K product, which
// are added here in their fixed order.
//
// Sum, mean, rsqrt and the product are 32-bit; the output is rounded once.
// Rows of up to 8192 values are read once and kept in registers between the
// sum of squares and the scaling.
// With `rows` given, only those rows are normed, into consecutive rows of
// `out`, and the residual stream is left as it is (the final norm before the
// output head runs on the wanted rows alone).
//
// With taps (decode steps, one token per request, row b = request b): the
// normed row then passes through a short causal convolution over time before it
// is stored, out = h + sum_j w[j] * h(j steps back), whose earlier inputs are the
// request's state row [taps - 1, channels] (oldest first), shifted here by the
// new input.  Same arithmetic, order and roundings as the norm followed by the
// convolution's own kernel (the normed value is rounded to the output type
// before it enters the convolution and the state, as that path stores it).
//
// Reference: rmsnorm_kernel, csrc/kernels/fused_rmsnorm_swiglu.cu:15-113 (same
// arithmetic; its residual stream has the activations' type, ours is 32-bit).
#include "common.cuh"

namespace {

// VEC values at p (aligned to VEC elements) as floats, in one memory access where VEC is 4.
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(float (&dst)[VEC], const T *p) {
  if constexpr (VEC == 4 && sizeof(T) == 4) {
    const float4 v = *reinterpret_cast<const float4 *>(p);
    dst[0] = v.x, dst[1] = v.y, dst[2] = v.z, dst[3] = v.w;
  } else if constexpr (VEC == 4 && sizeof(T) == 2) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
    dst[0] = a.x, dst[1] = a.y, dst[2] = b.x, dst[3] = b.y;
  } else {
#pragma unroll
    for (int v = 0; v < VEC; ++v) dst[v] = le::to_f32(p[v]);
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T *p, const float (&src)[VEC]) {
  if constexpr (VEC == 4 && sizeof(T) == 4) {
    *reinterpret_cast<float4 *>(p) = make_float4(src[0], src[1], src[2], src[3]);
  } else if constexpr (VEC == 4 && sizeof(T) == 2) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162 *>(&raw.x) = __floats2bfloat162_rn(src[0], src[1]);
    *reinterpret_cast<__nv_bfloat162 *>(&raw.y) = __floats2bfloat162_rn(src[2], src[3]);
    *reinterpret_cast<uint2 *>(p) = raw;
  } else {
#pragma unroll
    for (int v = 0; v < VEC; ++v) p[v] = le::from_f32<T>(src[v]);
  }
}

struct TapsArgs {
  const float *delta_scale = nullptr;   // [row width]: a factor per column on what enters the stream (rides here: every form gets it)
  const float *w = nullptr;        // [taps, channels]
  float *state = nullptr;          // [num_state_rows, taps - 1, channels]
  const int32_t *slots = nullptr;  // state row of each request (< 0: none; zeros before it, nothing kept)
  int taps = 0, channels = 0, num_state_rows = 0;
};

// h: VEC normed values of channels channel .. channel + VEC of request `request`; replaced by the convolution's output.
template <typename TO, int VEC>
__device__ __forceinline__ void taps_step(float (&h)[VEC], const TapsArgs &t, int64_t channel, int request) {
#pragma unroll
  for (int v = 0; v < VEC; ++v) h[v] = le::to_f32(le::from_f32<TO>(h[v]));
  const int keep = t.taps - 1;
  const int slot = t.slots[request];
  float *mine = (slot >= 0 && slot < t.num_state_rows && keep > 0) ? t.state + (static_cast<int64_t>(slot) * keep) * t.channels + channel : nullptr;
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = h[v];
  for (int s = 0; s < keep; ++s) {
    float prev[VEC], wt[VEC];
    load_vec<float, VEC>(wt, t.w + static_cast<int64_t>(s) * t.channels + channel);
    if (mine) {
      load_vec<float, VEC>(prev, mine + static_cast<int64_t>(s) * t.channels);
      if (s > 0) store_vec<float, VEC>(mine + static_cast<int64_t>(s - 1) * t.channels, prev);
    } else {
#pragma unroll
      for (int v = 0; v < VEC; ++v) prev[v] = 0.0f;
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = fmaf(wt[v], prev[v], acc[v]);
  }
  float wt[VEC];
  load_vec<float, VEC>(wt, t.w + static_cast<int64_t>(keep) * t.channels + channel);
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = fmaf(wt[v], h[v], acc[v]);
  if (mine) store_vec<float, VEC>(mine + static_cast<int64_t>(keep - 1) * t.channels, h);
#pragma unroll
  for (int v = 0; v < VEC; ++v) h[v] = acc[v];
}

// The same in two halves for up to TAPS_AHEAD taps: what does not depend on the normed values (weights, old state)
// is asked for before the row's sum of squares is known, so that those loads run beside the reduction.
constexpr int TAPS_AHEAD = 4;
template <int VEC>
struct TapsFetched {
  float w[TAPS_AHEAD][VEC];
  float prev[TAPS_AHEAD - 1][VEC];
  float *mine;
};
template <int VEC>
__device__ __forceinline__ void taps_fetch(TapsFetched<VEC> &f, const TapsArgs &t, int64_t channel, int request) {
  const int keep = t.taps - 1;
  const int slot = t.slots[request];
  f.mine = (slot >= 0 && slot < t.num_state_rows && keep > 0) ? t.state + (static_cast<int64_t>(slot) * keep) * t.channels + channel : nullptr;
#pragma unroll
  for (int s = 0; s < TAPS_AHEAD; ++s)
    if (s < t.taps) load_vec<float, VEC>(f.w[s], t.w + static_cast<int64_t>(s) * t.channels + channel);
#pragma unroll
  for (int s = 0; s < TAPS_AHEAD - 1; ++s) {
    if (s < keep && f.mine) {
      load_vec<float, VEC>(f.prev[s], f.mine + static_cast<int64_t>(s) * t.channels);
    } else {
#pragma unroll
      for (int v = 0; v < VEC; ++v) f.prev[s][v] = 0.0f;
    }
  }
}
template <typename TO, int VEC>
__device__ __forceinline__ void taps_apply(float (&h)[VEC], const TapsFetched<VEC> &f, const TapsArgs &t) {
#pragma unroll
  for (int v = 0; v < VEC; ++v) h[v] = le::to_f32(le::from_f32<TO>(h[v]));
  const int keep = t.taps - 1;
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = h[v];
#pragma unroll
  for (int s = 0; s < TAPS_AHEAD - 1; ++s) {
    if (s < keep) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] = fmaf(f.w[s][v], f.prev[s][v], acc[v]);
      if (f.mine && s > 0) store_vec<float, VEC>(f.mine + static_cast<int64_t>(s - 1) * t.channels, f.prev[s]);
    }
  }
#pragma unroll
  for (int s = 0; s < TAPS_AHEAD; ++s) {
    if (s == keep) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] = fmaf(f.w[s][v], h[v], acc[v]);
    }
  }
  if (f.mine) store_vec<float, VEC>(f.mine + static_cast<int64_t>(keep - 1) * t.channels, h);
#pragma unroll
  for (int v = 0; v < VEC; ++v) h[v] = acc[v];
}

// PER_THREAD > 0: the row fits in PER_THREAD vectors of VEC values per thread, which stay in registers
// between the sum of squares and the scaling (one pass over memory).  0: any width, two passes.
// PARTIALS > 0: `num_partials` is this number, known when compiling, so that every load of a thread is asked
// for before the first is used (a decode step's norm is one round trip to memory, not one per partial sum).
// TAPS: the short convolution follows in the same kernel (PER_THREAD > 0 only).
template <typename TO, typename TD, int VEC, int PER_THREAD, int PARTIALS, bool TAPS>
__global__ void rmsnorm_kernel(TO *__restrict__ out, float *__restrict__ resid, const TD *__restrict__ delta,
                               int num_partials, int64_t partial_stride, const float *__restrict__ weight,
                               const int32_t *__restrict__ rows, float eps, int hidden, int row_width, TapsArgs taps) {
  // `hidden`: the values that share one root mean square (the row, or one of its equal parts: blockIdx.y);
  // `row_width`: the values of a whole row
  __shared__ float scratch[33];
  le::let_successor_start();
  le::wait_for_predecessor();
  const int64_t src_row = rows ? rows[blockIdx.x] : blockIdx.x;
  const int64_t part = static_cast<int64_t>(blockIdx.y) * hidden;
  float *x = resid + src_row * row_width + part;
  const TD *d = delta ? delta + src_row * row_width + part : nullptr;
  TO *o = out + static_cast<int64_t>(blockIdx.x) * row_width + part;
  weight += part;
  const bool write_back = (d != nullptr) && (rows == nullptr);
  const float *dscale = taps.delta_scale ? taps.delta_scale + part : nullptr;

  if constexpr (PER_THREAD > 0 && PARTIALS > 0) {
    float val[PER_THREAD][VEC], add[PER_THREAD][PARTIALS][VEC], w[PER_THREAD][VEC];
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int i = (it * blockDim.x + threadIdx.x) * VEC;
      if (i < hidden) {
        load_vec<float, VEC>(val[it], x + i);
        if (d) {
#pragma unroll
          for (int p = 0; p < PARTIALS; ++p) load_vec<TD, VEC>(add[it][p], d + p * partial_stride + i);
        }
        load_vec<float, VEC>(w[it], weight + i);
      }
    }
    TapsFetched<VEC> ahead[TAPS ? PER_THREAD : 1];
    const bool fetch_ahead = TAPS && taps.taps <= TAPS_AHEAD;
    if constexpr (TAPS) {
      if (fetch_ahead) {
#pragma unroll
        for (int it = 0; it < PER_THREAD; ++it) {
          const int i = (it * blockDim.x + threadIdx.x) * VEC;
          if (i < hidden) taps_fetch<VEC>(ahead[it], taps, part + i, static_cast<int>(src_row));
        }
      }
    }
    float ss = 0.0f;
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int i = (it * blockDim.x + threadIdx.x) * VEC;
      if (i < hidden) {
        if (d && dscale == nullptr) {
#pragma unroll
          for (int p = 0; p < PARTIALS; ++p)       // in the partial sums' order, as the general form adds them
#pragma unroll
            for (int v = 0; v < VEC; ++v) val[it][v] += add[it][p][v];
        } else if (d) {
          float sc[VEC];
          load_vec<float, VEC>(sc, dscale + i);
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            float sum = add[it][0][v];
#pragma unroll
            for (int p = 1; p < PARTIALS; ++p) sum += add[it][p][v];
            val[it][v] = fmaf(sc[v], sum, val[it][v]);
          }
        }
        if (write_back) store_vec<float, VEC>(x + i, val[it]);
#pragma unroll
        for (int v = 0; v < VEC; ++v) ss += val[it][v] * val[it][v];
      }
    }
    ss = le::block_sum(ss, scratch);
    const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int i = (it * blockDim.x + threadIdx.x) * VEC;
      if (i < hidden) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) w[it][v] = val[it][v] * inv * w[it][v];
        if constexpr (TAPS) {
          if (fetch_ahead) taps_apply<TO, VEC>(w[it], ahead[it], taps);
          else taps_step<TO, VEC>(w[it], taps, part + i, static_cast<int>(src_row));
        }
        store_vec<TO, VEC>(o + i, w[it]);
      }
    }
    return;
  }
  if constexpr (PER_THREAD > 0) {
    float val[PER_THREAD][VEC];
    float ss = 0.0f;
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int i = (it * blockDim.x + threadIdx.x) * VEC;
      if (i < hidden) {
        load_vec<float, VEC>(val[it], x + i);
        if (d && dscale == nullptr) {
          for (int p = 0; p < num_partials; ++p) {
            float add[VEC];
            load_vec<TD, VEC>(add, d + p * partial_stride + i);
#pragma unroll
            for (int v = 0; v < VEC; ++v) val[it][v] += add[v];
          }
        } else if (d) {
          float sum[VEC], sc[VEC];
          load_vec<TD, VEC>(sum, d + i);
          for (int p = 1; p < num_partials; ++p) {
            float add[VEC];
            load_vec<TD, VEC>(add, d + p * partial_stride + i);
#pragma unroll
            for (int v = 0; v < VEC; ++v) sum[v] += add[v];
          }
          load_vec<float, VEC>(sc, dscale + i);
#pragma unroll
          for (int v = 0; v < VEC; ++v) val[it][v] = fmaf(sc[v], sum[v], val[it][v]);
        }
        if (write_back) store_vec<float, VEC>(x + i, val[it]);
#pragma unroll
        for (int v = 0; v < VEC; ++v) ss += val[it][v] * val[it][v];
      }
    }
    ss = le::block_sum(ss, scratch);
    const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int i = (it * blockDim.x + threadIdx.x) * VEC;
      if (i < hidden) {
        float w[VEC];
        load_vec<float, VEC>(w, weight + i);
#pragma unroll
        for (int v = 0; v < VEC; ++v) w[v] = val[it][v] * inv * w[v];
        if constexpr (TAPS) taps_step<TO, VEC>(w, taps, part + i, static_cast<int>(src_row));
        store_vec<TO, VEC>(o + i, w);
      }
    }
    return;
  }

  float ss = 0.0f;
  for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float val = x[i + v];
      if (d && dscale == nullptr) {
        for (int p = 0; p < num_partials; ++p) val += le::to_f32(d[p * partial_stride + i + v]);
      } else if (d) {
        float sum = le::to_f32(d[i + v]);
        for (int p = 1; p < num_partials; ++p) sum += le::to_f32(d[p * partial_stride + i + v]);
        val = fmaf(dscale[i + v], sum, val);
      }
      if (write_back) x[i + v] = val;
      ss += val * val;
    }
  }
  ss = le::block_sum(ss, scratch);
  const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
  for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float val = x[i + v];
      if (d && !write_back && dscale == nullptr) {
        for (int p = 0; p < num_partials; ++p) val += le::to_f32(d[p * partial_stride + i + v]);
      } else if (d && !write_back) {
        float sum = le::to_f32(d[i + v]);
        for (int p = 1; p < num_partials; ++p) sum += le::to_f32(d[p * partial_stride + i + v]);
        val = fmaf(dscale[i + v], sum, val);
      }
      o[i + v] = le::from_f32<TO>(val * inv * weight[i + v]);
    }
  }
}

template <typename TO, typename TD>
int launch(void *out, float *resid, const void *delta, int num_partials, int64_t partial_stride, const float *weight,
           const int32_t *rows, float eps, int num_rows, int row_width, int groups, const TapsArgs &taps, cudaStream_t stream) {
  const int hidden = row_width / groups;
  int threads = 32;
  while (threads < 512 && threads * 8 < hidden) threads *= 2;
#define LE_NORM_T(VEC, PER, PARTIALS, TAPS)                                                                             \
  return le::launch_chained(rmsnorm_kernel<TO, TD, VEC, PER, PARTIALS, TAPS>, dim3(num_rows, groups), dim3(threads), 0, stream, \
                            static_cast<TO *>(out), resid, static_cast<const TD *>(delta), num_partials, partial_stride, \
                            weight, rows, eps, hidden, row_width, taps)
#define LE_NORM_P(VEC, PER, PARTIALS)                                                                                  \
  do {                                                                                                                 \
    if constexpr (VEC == 4 && PER == 2) {                                                                              \
      if (taps.w != nullptr) LE_NORM_T(VEC, PER, PARTIALS, true);                                                      \
    }                                                                                                                  \
    if (taps.w != nullptr) return le::invalid("le_rmsnorm_taps: rows of this width have no form with taps");           \
    LE_NORM_T(VEC, PER, PARTIALS, false);                                                                              \
  } while (0)
#define LE_NORM(VEC, PER)                                                                                               \
  do {                                                                                                                  \
    if (PER > 0 && PER <= 2) {                                                                                          \
      if (delta == nullptr || num_partials == 1) LE_NORM_P(VEC, PER, 1);                                                \
      if (num_partials == 2) LE_NORM_P(VEC, PER, 2);                                                                    \
      if (num_partials == 3) LE_NORM_P(VEC, PER, 3);                                                                    \
      if (num_partials == 4) LE_NORM_P(VEC, PER, 4);                                                                    \
    }                                                                                                                   \
    LE_NORM_P(VEC, PER, 0);                                                                                             \
  } while (0)
  const bool aligned = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(delta) |
                         reinterpret_cast<uintptr_t>(weight)) & 15) == 0 && partial_stride % 4 == 0;
  if (hidden % 4 == 0 && aligned) {
    const int per_thread = (hidden / 4 + threads - 1) / threads;   // vectors of 4 a thread holds
    if (per_thread <= 2) LE_NORM(4, 2);
    if (per_thread <= 4) LE_NORM(4, 4);
    LE_NORM(4, 0);
  }
  LE_NORM(1, 0);
#undef LE_NORM
#undef LE_NORM_P
#undef LE_NORM_T
}

}  // namespace

// `groups`: equal consecutive parts of a row, each with its own root mean square (1: the whole row).
// `out_dtype` is the type of `out`; `delta_dtype` that of `delta`, which holds
// `num_partials` tensors of the residual stream's shape, `partial_stride`
// elements apart.  `delta_scale`: float32 [hidden] or null, the factor per column on the deltas' sum.
LE_API int le_rmsnorm(void *out, int out_dtype, float *resid, const void *delta, int delta_dtype, int num_partials,
                      int64_t partial_stride, const float *weight, const int32_t *rows, float eps, int num_rows, int hidden,
                      int groups, const float *delta_scale, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (hidden <= 0) return le::invalid("le_rmsnorm: hidden must be positive");
  if (groups < 1 || groups > 65535 || hidden % groups)
    return le::invalid("le_rmsnorm: a row of %d values does not divide into %d equal parts", hidden, groups);
  if (delta != nullptr && num_partials < 1) return le::invalid("le_rmsnorm: num_partials must be at least 1");
  if (delta_scale != nullptr && (reinterpret_cast<uintptr_t>(delta_scale) & 15)) return le::invalid("le_rmsnorm: delta_scale must be 16-byte aligned");
  TapsArgs taps{};
  taps.delta_scale = delta != nullptr ? delta_scale : nullptr;
#define LE_GO(TO, TD) return launch<TO, TD>(out, resid, delta, num_partials, partial_stride, weight, rows, eps, num_rows, hidden, groups, taps, stream)
  if (out_dtype == LE_F32 && (delta == nullptr || delta_dtype == LE_F32)) LE_GO(float, float);
  if (out_dtype == LE_BF16 && (delta == nullptr || delta_dtype == LE_BF16)) LE_GO(__nv_bfloat16, __nv_bfloat16);
  if (out_dtype == LE_BF16 && delta_dtype == LE_F32) LE_GO(__nv_bfloat16, float);
#undef LE_GO
  return le::invalid("le_rmsnorm: unsupported types: out %d, delta %d", out_dtype, delta_dtype);
}

// 1 when le_rmsnorm_taps has a form for rows of `hidden` values in `groups` parts.
LE_API int le_rmsnorm_taps_applies(int hidden, int groups) {
  if (groups < 1 || hidden % groups) return 0;
  const int part = hidden / groups;
  int threads = 32;
  while (threads < 512 && threads * 8 < part) threads *= 2;
  return part % 4 == 0 && (part / 4 + threads - 1) / threads <= 2 ? 1 : 0;
}

// le_rmsnorm over every row of a step whose requests bring one token each (row b is request b), followed in the same
// kernel by a short causal convolution over time with per-request state: taps_w [taps, hidden] float32, state
// [num_state_rows, taps - 1, hidden] float32, state_slots[b] the state row of request b (< 0: none).  All buffers
// 16-byte aligned.
LE_API int le_rmsnorm_taps(void *out, int out_dtype, float *resid, const void *delta, int delta_dtype, int num_partials,
                           int64_t partial_stride, const float *weight, float eps, int num_rows, int hidden, int groups,
                           const float *taps_w, float *state, int num_state_rows, const int32_t *state_slots, int num_taps,
                           cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (!le_rmsnorm_taps_applies(hidden, groups)) return le::invalid("le_rmsnorm_taps: rows of %d values in %d parts have no form with taps", hidden, groups);
  if (delta != nullptr && num_partials < 1) return le::invalid("le_rmsnorm_taps: num_partials must be at least 1");
  if (num_taps < 1 || taps_w == nullptr || (num_taps > 1 && state == nullptr)) return le::invalid("le_rmsnorm_taps: %d taps need weights and state", num_taps);
  if ((reinterpret_cast<uintptr_t>(taps_w) | reinterpret_cast<uintptr_t>(state)) & 15) return le::invalid("le_rmsnorm_taps: weights and state must be 16-byte aligned");
  TapsArgs taps;
  taps.w = taps_w, taps.state = state, taps.slots = state_slots, taps.taps = num_taps, taps.channels = hidden, taps.num_state_rows = num_state_rows;
#define LE_GO(TO, TD) return launch<TO, TD>(out, resid, delta, num_partials, partial_stride, weight, nullptr, eps, num_rows, hidden, groups, taps, stream)
  if (out_dtype == LE_F32 && (delta == nullptr || delta_dtype == LE_F32)) LE_GO(float, float);
  if (out_dtype == LE_BF16 && (delta == nullptr || delta_dtype == LE_BF16)) LE_GO(__nv_bfloat16, __nv_bfloat16);
  if (out_dtype == LE_BF16 && delta_dtype == LE_F32) LE_GO(__nv_bfloat16, float);
#undef LE_GO
  return le::invalid("le_rmsnorm_taps: unsupported types: out %d, delta %d", out_dtype, delta_dtype);
}
