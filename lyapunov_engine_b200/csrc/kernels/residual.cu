// Kernels of block arrangements whose sub-layers read the same residual
// stream side by side, and of inputs that enter the stream token by token.
//
// An "addend" below is a sub-layer's output on its way into the 32-bit
// stream: [rows, W] in the activations' type, or float32 partial sums
// [parts, rows, W] of a split-K product, which are added in order.
//
// rmsnorm_pair_kernel: one row of the stream, an optional addend y that
// enters first, either plainly (x += y) or normed, x += y / sqrt(mean(y^2) +
// eps_y) * wy, then up to two norms of the same x with weights of their own,
// out_i = x / sqrt(mean(x^2) + eps) * w_i.  With a row list only those rows
// are normed and the stream is left as it is.
//
// residual_add_kernel: x += a + f + bias (every addend optional), and a copy
// of the new x in the activations' type for a product that reads the stream
// itself.
//
// gate_rows_kernel: g[t, j] = gelu_tanh(z[t, j]) * table[id[t], col + j]: a
// gate over an embedding looked up per token (tanh form of gelu, 32-bit).
//
// stream_entry_kernel: x[t] += table[id[t]] + vec: what a pass over a stretch of
// layers adds before its first layer (either part optional).
#include "common.cuh"

namespace {

struct Addend {
  const void *data;     // null: none
  int dtype;
  int parts;
  int64_t part_stride;  // elements between partial sums
};

__device__ __forceinline__ float addend_at(const Addend &a, int64_t at) {
  if (a.dtype == LE_BF16) return le::to_f32(static_cast<const __nv_bfloat16 *>(a.data)[at]);
  const float *p = static_cast<const float *>(a.data);
  float v = p[at];
  for (int s = 1; s < a.parts; ++s) v += p[at + s * a.part_stride];
  return v;
}

// Four consecutive values at once (the address a multiple of 16 bytes for floats, of 8 for bfloat16).
__device__ __forceinline__ float4 load4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16 *p) {
  const uint2 r = *reinterpret_cast<const uint2 *>(p);
  return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u), __uint_as_float(r.y << 16),
                     __uint_as_float(r.y & 0xffff0000u));
}
__device__ __forceinline__ void store4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16 *p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 r;
  r.x = *reinterpret_cast<const uint32_t *>(&lo), r.y = *reinterpret_cast<const uint32_t *>(&hi);
  *reinterpret_cast<uint2 *>(p) = r;
}
__device__ __forceinline__ float4 addend4(const Addend &a, int64_t at) {
  if (a.dtype == LE_BF16) return load4(static_cast<const __nv_bfloat16 *>(a.data) + at);
  const float *p = static_cast<const float *>(a.data);
  float4 v = load4(p + at);
  for (int s = 1; s < a.parts; ++s) {
    const float4 w = load4(p + at + s * a.part_stride);
    v.x += w.x, v.y += w.y, v.z += w.z, v.w += w.w;
  }
  return v;
}

// rmsnorm_pair_kernel for rows of up to 1024 * V values, a multiple of four, everything on 16-byte addresses: a thread
// keeps V pieces of four values in registers, and the row is read once.
template <typename T, int V>
__global__ void __launch_bounds__(256)
rmsnorm_pair_wide_kernel(T *__restrict__ out1, T *__restrict__ out2, float *__restrict__ resid, Addend y,
                         const float *__restrict__ wy, float eps_y, const float *__restrict__ w1,
                         const float *__restrict__ w2, float eps, const int32_t *__restrict__ rows, int width) {
  __shared__ float scratch[33];
  le::let_successor_start();
  le::wait_for_predecessor();
  const int64_t r = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  const int n4 = width >> 2;
  float *x = resid + r * width;
  float4 xv[V], yv[V];
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int i = threadIdx.x + v * 256;
    xv[v] = yv[v] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (i < n4) {
      xv[v] = load4(x + 4 * i);
      if (y.data != nullptr) yv[v] = addend4(y, r * width + 4 * i);
    }
  }
  if (y.data != nullptr) {
    float scale = 1.0f;
    if (wy != nullptr) {
      float yy = 0.0f;
#pragma unroll
      for (int v = 0; v < V; ++v) yy = fmaf(yv[v].x, yv[v].x, fmaf(yv[v].y, yv[v].y, fmaf(yv[v].z, yv[v].z, fmaf(yv[v].w, yv[v].w, yy))));
      scale = rsqrtf(le::block_sum(yy, scratch) / static_cast<float>(width) + eps_y);
    }
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int i = threadIdx.x + v * 256;
      if (i < n4) {
        if (wy != nullptr) {
          const float4 w = load4(wy + 4 * i);
          xv[v].x += yv[v].x * scale * w.x, xv[v].y += yv[v].y * scale * w.y;
          xv[v].z += yv[v].z * scale * w.z, xv[v].w += yv[v].w * scale * w.w;
        } else {
          xv[v].x += yv[v].x, xv[v].y += yv[v].y, xv[v].z += yv[v].z, xv[v].w += yv[v].w;
        }
        if (rows == nullptr) store4(x + 4 * i, xv[v]);
      }
    }
  }
  if (out1 == nullptr) return;
  float ss = 0.0f;
#pragma unroll
  for (int v = 0; v < V; ++v) ss = fmaf(xv[v].x, xv[v].x, fmaf(xv[v].y, xv[v].y, fmaf(xv[v].z, xv[v].z, fmaf(xv[v].w, xv[v].w, ss))));
  const float inv = rsqrtf(le::block_sum(ss, scratch) / static_cast<float>(width) + eps);
  T *o1 = out1 + static_cast<int64_t>(blockIdx.x) * width;
  T *o2 = out2 != nullptr ? out2 + static_cast<int64_t>(blockIdx.x) * width : nullptr;
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int i = threadIdx.x + v * 256;
    if (i < n4) {
      const float4 a = make_float4(xv[v].x * inv, xv[v].y * inv, xv[v].z * inv, xv[v].w * inv);
      const float4 p = load4(w1 + 4 * i);
      store4(o1 + 4 * i, make_float4(a.x * p.x, a.y * p.y, a.z * p.z, a.w * p.w));
      if (o2 != nullptr) {
        const float4 q = load4(w2 + 4 * i);
        store4(o2 + 4 * i, make_float4(a.x * q.x, a.y * q.y, a.z * q.z, a.w * q.w));
      }
    }
  }
}

// residual_add_kernel, four values a thread (everything on 16-byte addresses, width a multiple of four).
template <typename T>
__global__ void __launch_bounds__(256)
residual_add_wide_kernel(float *__restrict__ resid, T *__restrict__ copy, Addend a, Addend f, const float *__restrict__ bias,
                         int64_t total4, int width) {
  le::let_successor_start();
  le::wait_for_predecessor();
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total4;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float4 v = load4(resid + 4 * i);
    float4 add = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (a.data != nullptr) add = addend4(a, 4 * i);
    if (f.data != nullptr) {
      const float4 w = addend4(f, 4 * i);
      add.x += w.x, add.y += w.y, add.z += w.z, add.w += w.w;
    }
    if (bias != nullptr) {
      const float4 w = load4(bias + (4 * i) % width);
      add.x += w.x, add.y += w.y, add.z += w.z, add.w += w.w;
    }
    v.x += add.x, v.y += add.y, v.z += add.z, v.w += add.w;
    store4(resid + 4 * i, v);
    if (copy != nullptr) store4(copy + 4 * i, v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_pair_kernel(T *__restrict__ out1, T *__restrict__ out2, float *__restrict__ resid, Addend y,
                    const float *__restrict__ wy, float eps_y, const float *__restrict__ w1,
                    const float *__restrict__ w2, float eps, const int32_t *__restrict__ rows, int width) {
  extern __shared__ float xs[];          // the row
  __shared__ float scratch[33];
  le::let_successor_start();
  le::wait_for_predecessor();
  const int64_t r = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  float *x = resid + r * width;
  float ss = 0.0f;
  if (y.data != nullptr) {
    float yy = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      const float v = addend_at(y, r * width + i);
      xs[i] = v;
      yy = fmaf(v, v, yy);
    }
    float scale = 1.0f;
    if (wy != nullptr) scale = rsqrtf(le::block_sum(yy, scratch) / static_cast<float>(width) + eps_y);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      const float v = x[i] + (wy != nullptr ? xs[i] * scale * wy[i] : xs[i]);
      xs[i] = v;
      if (rows == nullptr) x[i] = v;
      ss = fmaf(v, v, ss);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      const float v = x[i];
      xs[i] = v;
      ss = fmaf(v, v, ss);
    }
  }
  if (out1 == nullptr) return;
  const float inv = rsqrtf(le::block_sum(ss, scratch) / static_cast<float>(width) + eps);
  T *o1 = out1 + static_cast<int64_t>(blockIdx.x) * width;
  T *o2 = out2 != nullptr ? out2 + static_cast<int64_t>(blockIdx.x) * width : nullptr;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = xs[i] * inv;
    o1[i] = le::from_f32<T>(v * w1[i]);
    if (o2 != nullptr) o2[i] = le::from_f32<T>(v * w2[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
residual_add_kernel(float *__restrict__ resid, T *__restrict__ copy, Addend a, Addend f, const float *__restrict__ bias,
                    int64_t total, int width) {
  le::let_successor_start();
  le::wait_for_predecessor();
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float v = resid[i];
    float add = 0.0f;
    if (a.data != nullptr) add = addend_at(a, i);
    if (f.data != nullptr) add += addend_at(f, i);
    if (bias != nullptr) add += bias[i % width];
    v += add;
    resid[i] = v;
    if (copy != nullptr) copy[i] = le::from_f32<T>(v);
  }
}

template <typename T, typename E>
__global__ void __launch_bounds__(256)
gate_rows_kernel(T *__restrict__ out, const T *__restrict__ z, const E *__restrict__ table, int64_t table_stride, int col,
                 const int32_t *__restrict__ ids, int vocab, int64_t total, int dim, int *__restrict__ status) {
  le::let_successor_start();
  le::wait_for_predecessor();
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / dim;
    const int j = static_cast<int>(i - t * dim);
    const int id = ids[t];
    if (id < 0 || id >= vocab) {
      atomicOr(status, LE_STATUS_BAD_TOKEN);
      out[i] = le::from_f32<T>(0.0f);
      continue;
    }
    const float v = le::to_f32(z[i]);
    const float g = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    out[i] = le::from_f32<T>(g * le::to_f32(table[static_cast<int64_t>(id) * table_stride + col + j]));
  }
}

template <typename E>
__global__ void __launch_bounds__(256)
stream_entry_kernel(float *__restrict__ resid, const E *__restrict__ table, const int32_t *__restrict__ ids, int vocab,
                    const float *__restrict__ vec, int64_t total, int width, int *__restrict__ status) {
  le::let_successor_start();
  le::wait_for_predecessor();
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / width;
    const int j = static_cast<int>(i - t * width);
    float add = vec != nullptr ? vec[j] : 0.0f;
    if (table != nullptr) {
      const int id = ids[t];
      if (id < 0 || id >= vocab) {
        atomicOr(status, LE_STATUS_BAD_TOKEN);
      } else {
        add += le::to_f32(table[static_cast<int64_t>(id) * width + j]);
      }
    }
    resid[i] += add;
  }
}

bool on16(const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

int blocks_for(int64_t total) {
  const int64_t b = (total + 255) / 256;
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

// out1 / out2: [n, width] (out2 null: one norm; out1 null too: the addend enters and nothing is normed); resid
// [rows, width] float32; y: an addend or null, y_parts partial sums y_stride elements apart; wy null: y enters plainly.
LE_API int le_rmsnorm_pair(void *out1, void *out2, int out_dtype, float *resid, const void *y, int y_dtype, int y_parts,
                           int64_t y_stride, const float *wy, float eps_y, const float *w1, const float *w2, float eps,
                           const int32_t *rows, int n, int width, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width < 1 || width > 32 * 1024) return le::invalid("le_rmsnorm_pair: rows of %d values (at most 32768)", width);
  if (out1 == nullptr && (out2 != nullptr || rows != nullptr)) return le::invalid("le_rmsnorm_pair: nothing to write");
  const Addend add{y, y_dtype, y_parts < 1 ? 1 : y_parts, y_stride};
  if (width % 4 == 0 && width <= 8192 && y_stride % 4 == 0 && on16(out1) && on16(out2) && on16(resid) && on16(y) &&
      on16(wy) && on16(w1) && on16(w2)) {
#define LE_GO(V)                                                                                                        \
  LE_DISPATCH_DTYPE(out_dtype, T,                                                                                       \
                    return le::launch_chained(rmsnorm_pair_wide_kernel<T, V>, dim3(n), dim3(256), 0, stream,            \
                                              static_cast<T *>(out1), static_cast<T *>(out2), resid, add, wy, eps_y, w1, \
                                              w2, eps, rows, width))
    if (width <= 1024) LE_GO(1);
    if (width <= 2048) LE_GO(2);
    if (width <= 4096) LE_GO(4);
    LE_GO(8);
#undef LE_GO
  }
  const size_t smem = sizeof(float) * width;
  LE_DISPATCH_DTYPE(out_dtype, T,
                    if (smem > 40 * 1024) cudaFuncSetAttribute(rmsnorm_pair_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
                    return le::launch_chained(rmsnorm_pair_kernel<T>, dim3(n), dim3(256), smem, stream,
                                              static_cast<T *>(out1), static_cast<T *>(out2), resid, add, wy, eps_y, w1, w2,
                                              eps, rows, width));
}

// resid [rows, width] float32 += a + f + bias (bias [width] float32); copy: the new rows in the type `copy_dtype`, or null.
LE_API int le_residual_add(float *resid, void *copy, int copy_dtype, const void *a, int a_dtype, int a_parts,
                           int64_t a_stride, const void *f, int f_dtype, int f_parts, int64_t f_stride, const float *bias,
                           int rows, int width, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int64_t total = static_cast<int64_t>(rows) * width;
  const Addend aa{a, a_dtype, a_parts < 1 ? 1 : a_parts, a_stride}, ff{f, f_dtype, f_parts < 1 ? 1 : f_parts, f_stride};
  if (width % 4 == 0 && a_stride % 4 == 0 && f_stride % 4 == 0 && on16(resid) && on16(copy) && on16(a) && on16(f) &&
      on16(bias)) {
    LE_DISPATCH_DTYPE(copy_dtype, T,
                      return le::launch_chained(residual_add_wide_kernel<T>, dim3(blocks_for(total / 4)), dim3(256), 0,
                                                stream, resid, static_cast<T *>(copy), aa, ff, bias, total / 4, width));
  }
  LE_DISPATCH_DTYPE(copy_dtype, T,
                    return le::launch_chained(residual_add_kernel<T>, dim3(blocks_for(total)), dim3(256), 0, stream, resid,
                                              static_cast<T *>(copy), aa, ff, bias, total, width));
}

// out, z: [tokens, dim] contiguous in the type `dtype`; table: [vocab, table_stride] in the type `table_dtype`.
LE_API int le_gate_rows(void *out, const void *z, int dtype, const void *table, int table_dtype, int64_t table_stride,
                        int col, const int32_t *ids, int vocab, int tokens, int dim, int *status, cudaStream_t stream) {
  if (tokens <= 0 || dim <= 0) return 0;
  const int64_t total = static_cast<int64_t>(tokens) * dim;
#define LE_GO(T, E)                                                                                                   \
  return le::launch_chained(gate_rows_kernel<T, E>, dim3(blocks_for(total)), dim3(256), 0, stream, static_cast<T *>(out), \
                            static_cast<const T *>(z), static_cast<const E *>(table), table_stride, col, ids, vocab, total, \
                            dim, status)
  if (dtype == LE_BF16 && table_dtype == LE_BF16) LE_GO(__nv_bfloat16, __nv_bfloat16);
  if (dtype == LE_F32 && table_dtype == LE_F32) LE_GO(float, float);
  if (dtype == LE_F32 && table_dtype == LE_BF16) LE_GO(float, __nv_bfloat16);
  if (dtype == LE_BF16 && table_dtype == LE_F32) LE_GO(__nv_bfloat16, float);
#undef LE_GO
  return le::invalid("le_gate_rows: unknown dtype codes %d, %d", dtype, table_dtype);
}

// resid[t] += table[ids[t]] + vec; table ([vocab, width], type `table_dtype`) or vec ([width] float32) may be null.
LE_API int le_stream_entry(float *resid, const void *table, int table_dtype, const int32_t *ids, int vocab, const float *vec,
                           int tokens, int width, int *status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int64_t total = static_cast<int64_t>(tokens) * width;
  if (table_dtype == LE_BF16)
    return le::launch_chained(stream_entry_kernel<__nv_bfloat16>, dim3(blocks_for(total)), dim3(256), 0, stream, resid,
                              static_cast<const __nv_bfloat16 *>(table), ids, vocab, vec, total, width, status);
  if (table_dtype == LE_F32)
    return le::launch_chained(stream_entry_kernel<float>, dim3(blocks_for(total)), dim3(256), 0, stream, resid,
                              static_cast<const float *>(table), ids, vocab, vec, total, width, status);
  return le::invalid("le_stream_entry: unknown dtype code %d", table_dtype);
}
