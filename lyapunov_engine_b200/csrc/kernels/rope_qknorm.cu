// Queries and keys of a fused projection's rows: bias, a norm over the whole
// of q (and of k) at once, rotary positions in the rotate-half layout, and the
// cache write, in one kernel.
//
// Per token, rows hold q [heads, head_dim] | k [kv_heads, head_dim] | v
// [kv_heads, head_dim] (heads may be padded with zero columns behind their
// real entries):
//
//   q += b_q, k += b_k, v += b_v                                  (where biases are given)
//   q <- q / sqrt(sum(q^2) / q_count + eps) * w_q                 (one root mean square over all heads; same for k)
//   in every head of q and k, for i < rot / 2:  (x_i, x_{i + rot/2}) turns by the angle p * rates[i]:
//       (u, v) -> ((u cos - v sin) * m, (v cos + u sin) * m)      m: one factor on cosines and sines
//   q is rewritten in place, k and v go to the pages of the token's position.
//
// The rates come as 64-bit numbers and the angle, position times rate, is
// taken in 64 bits (and brought into [-pi, pi] there) before its cosine and sine are made
// here in 32: at position p a 32-bit product would be off by up to p * 2^-24
// radians, which at a thousand tokens is more than all other rounding of a
// 32-bit run together.  So there is no table and no longest position.  Sums,
// norms and the rotation are 32-bit; every output is rounded once.  `q_count` and
// `k_count` are the real entries the means run over (padding columns are zero
// and do not count).  One block per token.
#include "common.cuh"

namespace {

constexpr int QKN_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(QKN_THREADS)
rope_qknorm_store_kernel(T *__restrict__ rows, int64_t row_stride, const float *__restrict__ bias,
                         const float *__restrict__ w_q, const float *__restrict__ w_k, float eps, int q_count, int k_count,
                         const double *__restrict__ rates, int rot, float magnitude, T *__restrict__ k_cache,
                         T *__restrict__ v_cache, const int32_t *__restrict__ positions,
                         const int32_t *__restrict__ request_of_token, const int32_t *__restrict__ block_table,
                         int max_blocks, int heads, int kv_heads, int head_dim, int page_size, int num_pages, int write_kv,
                         int *__restrict__ status) {
  extern __shared__ __align__(16) float qkn_smem[];
  __shared__ float2 scratch2[QKN_THREADS / 32];
  const int q_width = heads * head_dim, k_width = kv_heads * head_dim;
  float *s_x = qkn_smem;                        // q then k, as floats
  float *s_cos = s_x + q_width + k_width;       // [rot / 2]
  float *s_sin = s_cos + rot / 2;
  le::let_successor_start();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int b = request_of_token[t];
  for (int i = threadIdx.x; i < rot / 2; i += QKN_THREADS) {
    // the angle in 64 bits, brought into [-pi, pi] there; its cosine and sine in 32
    double a = static_cast<double>(pos) * rates[i];
    a -= 6.283185307179586 * rint(a * 0.15915494309189535);
    float s, c;
    sincosf(static_cast<float>(a), &s, &c);
    s_cos[i] = c * magnitude;
    s_sin[i] = s * magnitude;
  }
  int page = -1;
  if (write_kv) {
    page = pos >= 0 ? block_table[static_cast<int64_t>(b) * max_blocks + pos / page_size] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_PAGE);
      page = -1;
    }
  }
  le::wait_for_predecessor();
  T *row = rows + static_cast<int64_t>(t) * row_stride;
  float ss_q = 0.0f, ss_k = 0.0f;
  // rows, pages and the rotated halves in 16-byte pieces where the sizes allow it
  constexpr int PIECE = le::Piece16<T>::COUNT;
  const bool pieces = head_dim % PIECE == 0 && (rot / 2) % PIECE == 0 && row_stride % PIECE == 0 &&
                      ((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(k_cache) |
                        reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
  if (pieces) {
    for (int i = threadIdx.x * PIECE; i < q_width + k_width; i += QKN_THREADS * PIECE) {
      float v[PIECE];
      le::load_piece16<T>(v, row + i);
#pragma unroll
      for (int e = 0; e < PIECE; ++e) {
        if (bias != nullptr) v[e] += bias[i + e];
        s_x[i + e] = v[e];
        if (i < q_width) ss_q = fmaf(v[e], v[e], ss_q);
        else ss_k = fmaf(v[e], v[e], ss_k);
      }
    }
  } else {
    for (int i = threadIdx.x; i < q_width + k_width; i += QKN_THREADS) {
      float v = le::to_f32(row[i]);
      if (bias != nullptr) v += bias[i];
      s_x[i] = v;
      if (i < q_width) ss_q = fmaf(v, v, ss_q);
      else ss_k = fmaf(v, v, ss_k);
    }
  }
  if (w_q != nullptr) {
    // both sums of squares in one meeting of the block
    ss_q = le::warp_sum(ss_q);
    ss_k = le::warp_sum(ss_k);
    if ((threadIdx.x & 31) == 0) scratch2[threadIdx.x >> 5] = make_float2(ss_q, ss_k);
    __syncthreads();
    ss_q = ss_k = 0.0f;
#pragma unroll
    for (int wi = 0; wi < QKN_THREADS / 32; ++wi) ss_q += scratch2[wi].x, ss_k += scratch2[wi].y;
    const float inv_q = rsqrtf(ss_q / static_cast<float>(q_count) + eps);
    const float inv_k = rsqrtf(ss_k / static_cast<float>(k_count) + eps);
    for (int i = threadIdx.x; i < q_width + k_width; i += QKN_THREADS)
      s_x[i] = i < q_width ? s_x[i] * inv_q * w_q[i] : s_x[i] * inv_k * w_k[i - q_width];
  }
  __syncthreads();
  const int half = rot / 2;
  const int64_t page_at = page >= 0 ? (static_cast<int64_t>(page) * kv_heads * page_size + pos % page_size) * head_dim : 0;
  if (pieces) {
    for (int i = threadIdx.x * PIECE; i < q_width + k_width; i += QKN_THREADS * PIECE) {
      const int h = i / head_dim, d = i - h * head_dim;       // (a piece lies within one head and on one side of the halves)
      uint4 raw;
      T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
      for (int u = 0; u < PIECE; ++u) {
        float v = s_x[i + u];
        if (d < half) v = v * s_cos[d + u] - s_x[i + u + half] * s_sin[d + u];
        else if (d < rot) v = v * s_cos[d + u - half] + s_x[i + u - half] * s_sin[d + u - half];
        e[u] = le::from_f32<T>(v);
      }
      if (i < q_width) *reinterpret_cast<uint4 *>(row + i) = raw;
      else if (page >= 0) *reinterpret_cast<uint4 *>(k_cache + page_at + static_cast<int64_t>(h - heads) * page_size * head_dim + d) = raw;
    }
    if (page >= 0) {
      for (int i = threadIdx.x * PIECE; i < k_width; i += QKN_THREADS * PIECE) {
        const int kvh = i / head_dim, d = i - kvh * head_dim;
        float v[PIECE];
        le::load_piece16<T>(v, row + q_width + k_width + i);
        uint4 raw;
        T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
        for (int u = 0; u < PIECE; ++u) e[u] = le::from_f32<T>(bias != nullptr ? v[u] + bias[q_width + k_width + i + u] : v[u]);
        *reinterpret_cast<uint4 *>(v_cache + page_at + static_cast<int64_t>(kvh) * page_size * head_dim + d) = raw;
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < q_width + k_width; i += QKN_THREADS) {
    const int h = i / head_dim, d = i - h * head_dim;
    float v = s_x[i];
    if (d < half) v = v * s_cos[d] - s_x[i + half] * s_sin[d];
    else if (d < rot) v = v * s_cos[d - half] + s_x[i - half] * s_sin[d - half];
    if (i < q_width) {
      row[i] = le::from_f32<T>(v);
    } else if (page >= 0) {
      const int kvh = h - heads;
      k_cache[page_at + static_cast<int64_t>(kvh) * page_size * head_dim + d] = le::from_f32<T>(v);
    }
  }
  if (page >= 0) {
    for (int i = threadIdx.x; i < k_width; i += QKN_THREADS) {
      const int kvh = i / head_dim, d = i - kvh * head_dim;
      float v = le::to_f32(row[q_width + k_width + i]);
      if (bias != nullptr) v += bias[q_width + k_width + i];
      v_cache[page_at + static_cast<int64_t>(kvh) * page_size * head_dim + d] = le::from_f32<T>(v);
    }
  }
}

}  // namespace

// rows: [T, >= (heads + 2 kv_heads) * head_dim] of type `dtype`, row stride row_stride; bias: float32 [(heads + 2
// kv_heads) * head_dim] or null; w_q [heads * head_dim], w_k [kv_heads * head_dim] float32 or both null (no norm);
// rates: float64 [rot / 2]; caches [num_pages, kv_heads, page_size, head_dim].  write_kv 0: queries only.
LE_API int le_rope_qknorm_store(void *rows, int64_t row_stride, int dtype, const float *bias, const float *w_q,
                                const float *w_k, float eps, int q_count, int k_count, const double *rates, int rot,
                                float magnitude, void *k_cache, void *v_cache, const int32_t *positions,
                                const int32_t *request_of_token, const int32_t *block_table, int max_blocks, int num_tokens,
                                int heads, int kv_heads, int head_dim, int page_size, int num_pages, int write_kv, int *status,
                                cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rot < 0 || rot % 2 || rot > head_dim) return le::invalid("le_rope_qknorm_store: %d rotated entries in heads of %d", rot, head_dim);
  if ((w_q == nullptr) != (w_k == nullptr)) return le::invalid("le_rope_qknorm_store: norm weights for both q and k, or neither");
  if (w_q != nullptr && (q_count < 1 || k_count < 1)) return le::invalid("le_rope_qknorm_store: the norms need the entries they run over");
  const size_t smem = sizeof(float) * (static_cast<size_t>(heads + kv_heads) * head_dim + rot);
  if (smem > 200 * 1024) return le::invalid("le_rope_qknorm_store: rows of %d values do not fit", (heads + kv_heads) * head_dim);
#define LE_GO(T)                                                                                                            \
  do {                                                                                                                      \
    auto kernel = rope_qknorm_store_kernel<T>;                                                                              \
    if (smem > 48 * 1024) {                                                                                                 \
      static size_t raised = 0;                                                                                             \
      if (smem > raised) {                                                                                                  \
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));  \
        if (e != cudaSuccess) return le::invalid("le_rope_qknorm_store: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
        raised = smem;                                                                                                      \
      }                                                                                                                     \
    }                                                                                                                       \
    return le::launch_chained(kernel, dim3(num_tokens), dim3(QKN_THREADS), smem, stream, static_cast<T *>(rows), row_stride, \
                              bias, w_q, w_k, eps, q_count, k_count, rates, rot, magnitude, static_cast<T *>(k_cache),      \
                              static_cast<T *>(v_cache), positions, request_of_token, block_table, max_blocks, heads,       \
                              kv_heads, head_dim, page_size, num_pages, write_kv, status);                                  \
  } while (0)
  if (dtype == LE_F32) LE_GO(float);
  if (dtype == LE_BF16) LE_GO(__nv_bfloat16);
#undef LE_GO
  return le::invalid("le_rope_qknorm_store: unknown dtype code %d", dtype);
}
