// Embedding gather (optionally with a sinusoidal position vector added),
// gated activations, the per-head output gate and small helpers.
//
// Reference counterparts: nn.Embedding (python/lyapunov_engine/models/llama.py:172,205)
// and swiglu_kernel (csrc/kernels/fused_rmsnorm_swiglu.cu:152-179).
#include "common.cuh"

LE_API const char *le_last_error() { return le::error_buffer(); }

namespace {

// One block per token: row `ids[t]` of the table goes to row t of the
// 32-bit residual stream.  An id outside the table sets the status word and
// writes zeros instead of reading out of bounds.
template <typename T>
__global__ void embed_kernel(float *__restrict__ out, const T *__restrict__ table, const int32_t *__restrict__ ids,
                             int hidden, int vocab, float scale, int *__restrict__ status) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const int id = ids[t];
  float *dst = out + static_cast<int64_t>(t) * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_TOKEN);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.0f;
    return;
  }
  const T *src = table + static_cast<int64_t>(id) * hidden;
  if (scale == 1.0f) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = le::to_f32(src[i]);
  } else {       // (one factor on the whole table, applied in 32 bits)
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = le::to_f32(src[i]) * scale;
  }
}

// The same with a sinusoidal position vector added in 32 bits: for the token at
// position p, entry 2i gets sin(p * rate[i]) and entry 2i + 1 the cosine of the
// same angle.  `rates` holds ceil(hidden / 2) floats; angle, sine and cosine
// are 32-bit (sinf / cosf, not the fast approximations).
template <typename T>
__global__ void embed_sinusoid_kernel(float *__restrict__ out, const T *__restrict__ table, const int32_t *__restrict__ ids,
                                      const int32_t *__restrict__ positions, const float *__restrict__ rates, int hidden,
                                      int vocab, int *__restrict__ status) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const int id = ids[t];
  const float p = static_cast<float>(positions[t]);
  float *dst = out + static_cast<int64_t>(t) * hidden;
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_TOKEN);
  const T *src = table + static_cast<int64_t>(bad ? 0 : id) * hidden;
  // a thread takes the two entries that share an angle: one sincosf for both
  for (int pair = threadIdx.x; 2 * pair < hidden; pair += blockDim.x) {
    float s, c;
    sincosf(p * rates[pair], &s, &c);
    const int i = 2 * pair;
    dst[i] = bad ? 0.0f : le::to_f32(src[i]) + s;
    if (i + 1 < hidden) dst[i + 1] = bad ? 0.0f : le::to_f32(src[i + 1]) + c;
  }
}

// out[t, i] = act(gu[t, i] + bias[i], gu[t, I + i] + bias[I + i]) (le::gated_activation; bias null: none), in 32-bit,
// rounded once.
template <typename T>
__global__ void glu_kernel(T *__restrict__ out, const T *__restrict__ gu, int64_t total, int inter, le::GatedActivation act,
                           const float *__restrict__ bias) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t t = idx / inter;
  const int i = static_cast<int>(idx - t * inter);
  float g = le::to_f32(gu[t * 2 * inter + i]);
  float u = le::to_f32(gu[t * 2 * inter + inter + i]);
  if (bias != nullptr) g += bias[i], u += bias[inter + i];
  out[idx] = le::from_f32<T>(le::gated_activation(g, u, act));
}

// x[t, h, :] *= sigmoid(gate[t, h]): one number per token and head scales that
// head's `head_width` values.  Sigmoid and product are 32-bit, rounded once.
// VEC values per thread and access (16 bytes where VEC > 1; head_width, the
// row strides and the base address then are multiples of VEC values).
template <typename T, int VEC>
__global__ void head_gate_kernel(T *__restrict__ x, int64_t x_stride, const T *__restrict__ gate, int64_t gate_stride,
                                 int num_tokens, int num_heads, int head_width) {
  const int per_row = num_heads * head_width / VEC;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(num_tokens) * per_row) return;
  const int64_t t = idx / per_row;
  const int i = static_cast<int>(idx - t * per_row) * VEC;
  const float g = le::to_f32(gate[t * gate_stride + i / head_width]);
  const float s = 1.0f / (1.0f + expf(-g));
  T *p = x + t * x_stride + i;
  if constexpr (VEC == 1) {
    *p = le::from_f32<T>(le::to_f32(*p) * s);
  } else {
    uint4 raw = *reinterpret_cast<const uint4 *>(p);
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int v = 0; v < VEC; ++v) e[v] = le::from_f32<T>(le::to_f32(e[v]) * s);
    *reinterpret_cast<uint4 *>(p) = raw;
  }
}

// out[t, i] = x[t, i] * sigmoid(gate[t, i]) * scale: a gate of its own for every entry; 32-bit, rounded once.
template <typename T, int VEC>
__global__ void sigmoid_gate_kernel(T *__restrict__ out, int64_t out_stride, const T *__restrict__ x, int64_t x_stride,
                                    const T *__restrict__ gate, int64_t gate_stride, int num_tokens, int width, float scale) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int per_row = width / VEC;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(num_tokens) * per_row) return;
  const int64_t t = idx / per_row;
  const int i = static_cast<int>(idx - t * per_row) * VEC;
  if constexpr (VEC == 1) {
    const float g = le::to_f32(gate[t * gate_stride + i]);
    out[t * out_stride + i] = le::from_f32<T>(le::to_f32(x[t * x_stride + i]) * (scale / (1.0f + expf(-g))));
  } else {
    uint4 xr = *reinterpret_cast<const uint4 *>(x + t * x_stride + i);
    const uint4 gr = *reinterpret_cast<const uint4 *>(gate + t * gate_stride + i);
    T *xe = reinterpret_cast<T *>(&xr);
    const T *ge = reinterpret_cast<const T *>(&gr);
#pragma unroll
    for (int v = 0; v < VEC; ++v) xe[v] = le::from_f32<T>(le::to_f32(xe[v]) * (scale / (1.0f + expf(-le::to_f32(ge[v])))));
    *reinterpret_cast<uint4 *>(out + t * out_stride + i) = xr;
  }
}

// out[t, i] = silu(gu[t, i]) * gu[t, I + i], in 32-bit, rounded once.
template <typename T>
__global__ void swiglu_kernel(T *__restrict__ out, const T *__restrict__ gu, int64_t total, int inter) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t t = idx / inter;
  const int i = static_cast<int>(idx - t * inter);
  const float g = le::to_f32(gu[t * 2 * inter + i]);
  const float u = le::to_f32(gu[t * 2 * inter + inter + i]);
  out[idx] = le::from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// The same with 16-byte accesses; `inter` is a multiple of 8.
__global__ void swiglu_bf16x8_kernel(__nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *__restrict__ gu, int64_t total8,
                                     int inter8) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int64_t t = idx / inter8;
  const int i = static_cast<int>(idx - t * inter8);
  const uint4 g4 = *reinterpret_cast<const uint4 *>(gu + (t * 2 * inter8 + i) * 8);
  const uint4 u4 = *reinterpret_cast<const uint4 *>(gu + (t * 2 * inter8 + inter8 + i) * 8);
  const __nv_bfloat162 *g2 = reinterpret_cast<const __nv_bfloat162 *>(&g4);
  const __nv_bfloat162 *u2 = reinterpret_cast<const __nv_bfloat162 *>(&u4);
  uint4 o4;
  __nv_bfloat162 *o2 = reinterpret_cast<__nv_bfloat162 *>(&o4);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
    o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
  }
  *reinterpret_cast<uint4 *>(out + idx * 8) = o4;
}

template <typename TO, typename TI>
__global__ void convert_kernel(TO *__restrict__ out, const TI *__restrict__ in, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = le::from_f32<TO>(le::to_f32(in[i]));
}

// One block per request of the step: a request none of whose tokens are in the
// cache yet (ctx_before == 0) gets its row of a per-request state buffer
// zeroed.  Rows that stand for no request (slot < 0) are skipped.
__global__ void zero_fresh_state_kernel(uint32_t *__restrict__ state, int64_t row_words, int num_rows,
                                        const int32_t *__restrict__ slots, const int32_t *__restrict__ ctx_before) {
  const int b = blockIdx.x;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_rows || ctx_before[b] != 0) return;
  uint32_t *row = state + static_cast<int64_t>(slot) * row_words;
  for (int64_t i = threadIdx.x; i < row_words; i += blockDim.x) row[i] = 0u;
}

// The same for several state buffers in one launch (blockIdx.y: the buffer).  `table` holds, per buffer, its
// address and the bytes of one of its rows.
struct StateBuffer {
  uint32_t *base;
  int64_t row_words;
};
__global__ void zero_fresh_states_kernel(const StateBuffer *__restrict__ table, int num_rows,
                                         const int32_t *__restrict__ slots, const int32_t *__restrict__ ctx_before) {
  const int b = blockIdx.x;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_rows || ctx_before[b] != 0) return;
  const StateBuffer buffer = table[blockIdx.y];
  uint32_t *row = buffer.base + static_cast<int64_t>(slot) * buffer.row_words;
  for (int64_t i = threadIdx.x; i < buffer.row_words; i += blockDim.x) row[i] = 0u;
}

}  // namespace

// How many multiprocessors the current device has (grids are sized by it).
LE_API int le_sm_count() {
  int device = 0, count = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
  return count;
}

// state: [num_rows, row_bytes] bytes, row_bytes a multiple of 4.
LE_API int le_zero_fresh_state(void *state, int64_t row_bytes, int num_rows, const int32_t *slots,
                               const int32_t *ctx_before, int num_requests, cudaStream_t stream) {
  if (num_requests <= 0 || row_bytes <= 0) return 0;
  if (row_bytes % 4) return le::invalid("le_zero_fresh_state: rows of %lld bytes are not a multiple of 4", (long long)row_bytes);
  zero_fresh_state_kernel<<<num_requests, 256, 0, stream>>>(static_cast<uint32_t *>(state), row_bytes / 4, num_rows, slots,
                                                            ctx_before);
  return le::launched();
}

// table: `num_buffers` pairs of 64-bit integers on the device (address of a buffer of [num_rows, row] bytes; the
// row's size in 4-byte words).  One launch zeroes the fresh requests' rows of all of them.
LE_API int le_zero_fresh_states(const void *table, int num_buffers, int num_rows, const int32_t *slots,
                                const int32_t *ctx_before, int num_requests, cudaStream_t stream) {
  if (num_requests <= 0 || num_buffers <= 0) return 0;
  if (num_buffers > 65535) return le::invalid("le_zero_fresh_states: %d buffers are too many for one launch", num_buffers);
  static_assert(sizeof(StateBuffer) == 16, "two 64-bit words per buffer");
  zero_fresh_states_kernel<<<dim3(num_requests, num_buffers), 256, 0, stream>>>(static_cast<const StateBuffer *>(table), num_rows,
                                                                                slots, ctx_before);
  return le::launched();
}

LE_API int le_embed(float *out, const void *table, int table_dtype, const int32_t *ids, int num_tokens, int hidden,
                    int vocab, float scale, int *status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  LE_DISPATCH_DTYPE(table_dtype, T,
                    return le::launch_chained(embed_kernel<T>, dim3(num_tokens), dim3(threads), 0, stream, out,
                                              static_cast<const T *>(table), ids, hidden, vocab, scale, status));
}

// The embedding with the sinusoidal position vector (see embed_sinusoid_kernel).
LE_API int le_embed_sinusoid(float *out, const void *table, int table_dtype, const int32_t *ids, const int32_t *positions,
                             const float *rates, int num_tokens, int hidden, int vocab, int *status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  LE_DISPATCH_DTYPE(table_dtype, T,
                    return le::launch_chained(embed_sinusoid_kernel<T>, dim3(num_tokens), dim3(threads), 0, stream, out,
                                              static_cast<const T *>(table), ids, positions, rates, hidden, vocab, status));
}

// out[T, I] from gate_up[T, 2 I] (gate columns first) by the activation `kind` (see le::GatedActivation).
LE_API int le_glu_bias(void *out, const void *gate_up, int dtype, int num_tokens, int inter, int kind, float alpha,
                       float limit, const float *bias, cudaStream_t stream);
LE_API int le_glu(void *out, const void *gate_up, int dtype, int num_tokens, int inter, int kind, float alpha, float limit,
                  cudaStream_t stream) {
  return le_glu_bias(out, gate_up, dtype, num_tokens, inter, kind, alpha, limit, nullptr, stream);
}

// The same with a bias [2 I] (float32; gate's entries first) added to the product's columns before the activation.
LE_API int le_glu_bias(void *out, const void *gate_up, int dtype, int num_tokens, int inter, int kind, float alpha,
                       float limit, const float *bias, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (kind < 0 || kind > 2) return le::invalid("le_glu: unknown activation %d", kind);
  const int64_t total = static_cast<int64_t>(num_tokens) * inter;
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 2147483647LL) return le::invalid("le_glu: %lld elements are too many for one launch", (long long)total);
  LE_DISPATCH_DTYPE(dtype, T,
                    glu_kernel<T><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
                        static_cast<T *>(out), static_cast<const T *>(gate_up), total, inter, le::GatedActivation{kind, alpha, limit}, bias));
  return le::launched();
}

// x: [T, num_heads * head_width] with row stride x_stride; gate: rows of stride gate_stride holding num_heads values.
LE_API int le_head_gate(void *x, int64_t x_stride, const void *gate, int64_t gate_stride, int dtype, int num_tokens,
                        int num_heads, int head_width, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int vec = dtype == LE_BF16 ? 8 : 4;
  const bool wide = head_width % vec == 0 && x_stride % vec == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const int64_t items = static_cast<int64_t>(num_tokens) * num_heads * head_width / (wide ? vec : 1);
  const int64_t blocks = (items + 255) / 256;
  if (blocks > 2147483647LL) return le::invalid("le_head_gate: too many elements for one launch");
#define LE_GO(T, V)                                                                                                  \
  head_gate_kernel<T, V><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<T *>(x), x_stride,           \
                                                                            static_cast<const T *>(gate), gate_stride, \
                                                                            num_tokens, num_heads, head_width)
  if (dtype == LE_BF16) { if (wide) LE_GO(__nv_bfloat16, 8); else LE_GO(__nv_bfloat16, 1); }
  else if (dtype == LE_F32) { if (wide) LE_GO(float, 4); else LE_GO(float, 1); }
  else return le::invalid("le_head_gate: unknown dtype code %d", dtype);
#undef LE_GO
  return le::launched();
}

// out, x, gate: [T, width] with row strides of their own (column ranges of wider rows are fine; out may be x).
LE_API int le_sigmoid_gate(void *out, int64_t out_stride, const void *x, int64_t x_stride, const void *gate,
                           int64_t gate_stride, int dtype, int num_tokens, int width, float scale, cudaStream_t stream) {
  if (num_tokens <= 0 || width <= 0) return 0;
  const int vec = dtype == LE_BF16 ? 8 : 4;
  const bool wide = width % vec == 0 && out_stride % vec == 0 && x_stride % vec == 0 && gate_stride % vec == 0 &&
                    ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gate)) & 15) == 0;
  const int64_t items = static_cast<int64_t>(num_tokens) * width / (wide ? vec : 1);
  const int64_t blocks = (items + 255) / 256;
  if (blocks > 2147483647LL) return le::invalid("le_sigmoid_gate: too many elements for one launch");
#define LE_GO(T, V)                                                                                                       \
  return le::launch_chained(sigmoid_gate_kernel<T, V>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream,         \
                            static_cast<T *>(out), out_stride, static_cast<const T *>(x), x_stride,                       \
                            static_cast<const T *>(gate), gate_stride, num_tokens, width, scale)
  if (dtype == LE_BF16) { if (wide) LE_GO(__nv_bfloat16, 8); LE_GO(__nv_bfloat16, 1); }
  if (dtype == LE_F32) { if (wide) LE_GO(float, 4); LE_GO(float, 1); }
#undef LE_GO
  return le::invalid("le_sigmoid_gate: unknown dtype code %d", dtype);
}

LE_API int le_swiglu(void *out, const void *gate_up, int dtype, int num_tokens, int inter, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int64_t total = static_cast<int64_t>(num_tokens) * inter;
  const int threads = 256;
  if (dtype == LE_BF16 && inter % 8 == 0) {
    const int64_t total8 = total / 8;
    const int64_t blocks8 = (total8 + threads - 1) / threads;
    if (blocks8 > 2147483647LL) return le::invalid("le_swiglu: %lld elements are too many for one launch", (long long)total);
    swiglu_bf16x8_kernel<<<static_cast<unsigned>(blocks8), threads, 0, stream>>>(
        static_cast<__nv_bfloat16 *>(out), static_cast<const __nv_bfloat16 *>(gate_up), total8, inter / 8);
    return le::launched();
  }
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 2147483647LL) return le::invalid("le_swiglu: %lld elements are too many for one launch", (long long)total);
  LE_DISPATCH_DTYPE(dtype, T,
                    swiglu_kernel<T><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
                        static_cast<T *>(out), static_cast<const T *>(gate_up), total, inter));
  return le::launched();
}

// out (f32) = in (bf16) or out (bf16) = in (f32).
LE_API int le_convert(void *out, int out_dtype, const void *in, int in_dtype, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n + threads - 1) / threads);
  if (out_dtype == LE_F32 && in_dtype == LE_BF16)
    convert_kernel<float, __nv_bfloat16><<<blocks, threads, 0, stream>>>(static_cast<float *>(out), static_cast<const __nv_bfloat16 *>(in), n);
  else if (out_dtype == LE_BF16 && in_dtype == LE_F32)
    convert_kernel<__nv_bfloat16, float><<<blocks, threads, 0, stream>>>(static_cast<__nv_bfloat16 *>(out), static_cast<const float *>(in), n);
  else
    return le::invalid("le_convert: unsupported pair of dtypes %d -> %d", in_dtype, out_dtype);
  return le::launched();
}
