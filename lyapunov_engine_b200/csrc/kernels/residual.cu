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
