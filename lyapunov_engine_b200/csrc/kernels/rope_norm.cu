// Rotary positions on neighbouring pairs, a weightless norm per head after
// the turn, and the paged cache write, for projections whose values are the
// keys themselves; and the same turn for the shared rotated part of a latent
// attention's keys, fused with the latent's norm and cache write.
//
// rope_norm_store_kernel.  The projection's row of a token holds query heads
// [heads][head_dim] and, behind them, key heads [kv_heads][head_dim].  In every
// head the entries (rot_col + 2i, rot_col + 2i + 1), 2i + 1 < rot, turn by the
// angle position * rates[i]: (a, b) -> (a cos - b sin, b cos + a sin).  With
// `unit` set the turned head is then divided by sqrt(mean(head^2) + eps) over
// its first norm_dim entries (the entries behind them are padding and zero).
// Queries are rewritten in place; keys go to the key pool; the value pool
// receives the keys as projected (before turn and norm) when
// `values_are_keys`, else nothing.  A warp takes a head, a lane up to eight
// pairs of it; a token's sines and cosines are made once per block.  Angle,
// sine, cosine, turn and norm are 32-bit; the result is rounded once.
//
// latent_rope_store_kernel.  Columns [col, col + rank) of a token's row are a
// latent: normed with a weight over `rank`; the `rot` columns behind it are one
// rotated key part shared by all heads: turned as above, not normed.  Both go
// to the one pool of the layer, [pages, 1, page, padded] with the latent at
// columns [0, rank), the rotated part at [rank, rank + rot) and zeros behind.
// Optionally a second latent at columns [col2, col2 + rank2) (the queries'
// own) is normed with its weight into `out2`.
#include "common.cuh"

namespace {

constexpr int RN_MAX_PAIRS = 8;      // pairs a lane holds: heads of up to 512 entries

// Two neighbouring entries at once where the address allows it.
template <typename T>
__device__ __forceinline__ void load_pair(const T *p, bool together, float &u, float &v) {
  if (together) {
    if constexpr (sizeof(T) == 2) {
      const uint32_t r = *reinterpret_cast<const uint32_t *>(p);
      u = __uint_as_float(r << 16), v = __uint_as_float(r & 0xffff0000u);
    } else {
      const float2 r = *reinterpret_cast<const float2 *>(p);
      u = r.x, v = r.y;
    }
  } else {
    u = le::to_f32(p[0]), v = le::to_f32(p[1]);
  }
}
template <typename T>
__device__ __forceinline__ void store_pair(T *p, bool together, float u, float v) {
  if (together) {
    if constexpr (sizeof(T) == 2) {
      *reinterpret_cast<__nv_bfloat162 *>(p) = __floats2bfloat162_rn(u, v);
    } else {
      *reinterpret_cast<float2 *>(p) = make_float2(u, v);
    }
  } else {
    p[0] = le::from_f32<T>(u), p[1] = le::from_f32<T>(v);
  }
}

// A block takes a token and `heads_per_block` of its heads (queries first, then keys), a warp one head at a time.  The
// token's sines and cosines are made once per block, in shared memory.
template <typename T>
__global__ void __launch_bounds__(128)
rope_norm_store_kernel(T *__restrict__ rows, int64_t row_stride, T *__restrict__ k_cache, T *__restrict__ v_cache,
                       const float *__restrict__ rates, const int32_t *__restrict__ positions,
                       const int32_t *__restrict__ request_of_token, const int32_t *__restrict__ block_table,
                       int max_blocks, int heads, int kv_heads, int head_dim, int rot_col, int rot, int unit, float eps,
                       int norm_dim, int page_size, int num_pages, int write_kv, int values_are_keys, int heads_per_block,
                       int together, int *__restrict__ status) {
  extern __shared__ float turn[];            // [rot / 2][2]: sine, cosine
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const float fpos = static_cast<float>(pos);
  for (int i = threadIdx.x; i < (rot >> 1); i += blockDim.x) sincosf(fpos * rates[i], &turn[2 * i], &turn[2 * i + 1]);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  T *row = rows + static_cast<int64_t>(t) * row_stride;
  int page = 0;
  bool bad = false;
  if (write_kv) {
    const int b = request_of_token[t];
    page = pos >= 0 ? block_table[static_cast<int64_t>(b) * max_blocks + pos / page_size] : -1;
    bad = page < 0 || page >= num_pages;
    if (bad && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, LE_STATUS_BAD_PAGE);
  }
  __syncthreads();
  const int pairs = head_dim >> 1;
  const int all = heads + (write_kv ? kv_heads : 0);
  const int h_end = min(all, (static_cast<int>(blockIdx.y) + 1) * heads_per_block);
  for (int h = blockIdx.y * heads_per_block + warp; h < h_end; h += warps) {
    T *x = row + static_cast<int64_t>(h) * head_dim;
    const bool is_key = h >= heads;
    if (is_key && bad) continue;
    float a[RN_MAX_PAIRS], b[RN_MAX_PAIRS];
    float ss = 0.0f;
    T *k_dst = nullptr, *v_dst = nullptr;
    if (is_key) {
      const int64_t at = ((static_cast<int64_t>(page) * kv_heads + (h - heads)) * page_size + pos % page_size) * head_dim;
      k_dst = k_cache + at;
      v_dst = values_are_keys ? v_cache + at : nullptr;
    }
#pragma unroll
    for (int i = 0; i < RN_MAX_PAIRS; ++i) {
      const int p = lane + 32 * i;
      if (p < pairs) {
        float u, v;
        load_pair(x + 2 * p, together, u, v);
        if (v_dst != nullptr) store_pair(v_dst + 2 * p, together, u, v);     // (as projected: the same bits)
        const int j = 2 * p - rot_col;
        if (j >= 0 && j + 1 < rot) {
          const float s = turn[j], c = turn[j + 1];
          const float nu = u * c - v * s, nv = v * c + u * s;
          u = nu, v = nv;
        }
        a[i] = u, b[i] = v;
        ss = fmaf(u, u, fmaf(v, v, ss));
      }
    }
    float inv = 1.0f;
    if (unit) inv = rsqrtf(le::warp_sum(ss) / static_cast<float>(norm_dim) + eps);
    T *dst = is_key ? k_dst : x;
#pragma unroll
    for (int i = 0; i < RN_MAX_PAIRS; ++i) {
      const int p = lane + 32 * i;
      if (p < pairs) store_pair(dst + 2 * p, together, a[i] * inv, b[i] * inv);
    }
  }
}

// 16 bytes of a head at once, as floats and back.
template <typename T>
struct Piece;
template <>
struct Piece<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void open(const uint4 &r, float *d) {
    d[0] = __uint_as_float(r.x << 16), d[1] = __uint_as_float(r.x & 0xffff0000u);
    d[2] = __uint_as_float(r.y << 16), d[3] = __uint_as_float(r.y & 0xffff0000u);
    d[4] = __uint_as_float(r.z << 16), d[5] = __uint_as_float(r.z & 0xffff0000u);
    d[6] = __uint_as_float(r.w << 16), d[7] = __uint_as_float(r.w & 0xffff0000u);
  }
  static __device__ __forceinline__ uint4 close(const float *d, float f) {
    uint4 r;
    __nv_bfloat162 *o = reinterpret_cast<__nv_bfloat162 *>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(d[2 * i] * f, d[2 * i + 1] * f);
    return r;
  }
};
template <>
struct Piece<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void open(const uint4 &r, float *d) {
    d[0] = __uint_as_float(r.x), d[1] = __uint_as_float(r.y), d[2] = __uint_as_float(r.z), d[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ uint4 close(const float *d, float f) {
    return make_uint4(__float_as_uint(d[0] * f), __float_as_uint(d[1] * f), __float_as_uint(d[2] * f), __float_as_uint(d[3] * f));
  }
};

// The same in 16-byte pieces (heads that are whole pieces, rows and pools that start on 16 bytes): a head belongs to
// `lph` neighbouring lanes (a power of two), a lane holds every lph-th piece of it, so a warp takes 32 / lph heads at
// once and the sum of squares meets over lph lanes.
template <typename T>
__global__ void __launch_bounds__(128)
rope_norm_store_pieces_kernel(T *__restrict__ rows, int64_t row_stride, T *__restrict__ k_cache, T *__restrict__ v_cache,
                              const float *__restrict__ rates, const int32_t *__restrict__ positions,
                              const int32_t *__restrict__ request_of_token, const int32_t *__restrict__ block_table,
                              int max_blocks, int heads, int kv_heads, int head_dim, int rot_col, int rot, int unit, float eps,
                              int norm_dim, int page_size, int num_pages, int write_kv, int values_are_keys,
                              int heads_per_block, int lph, int *__restrict__ status) {
  constexpr int N = Piece<T>::N;
  constexpr int HELD = 2 * RN_MAX_PAIRS / N;          // pieces a lane holds at most
  extern __shared__ float turn[];                     // [rot / 2][2]: sine, cosine
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const float fpos = static_cast<float>(pos);
  for (int i = threadIdx.x; i < (rot >> 1); i += blockDim.x) sincosf(fpos * rates[i], &turn[2 * i], &turn[2 * i + 1]);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  T *row = rows + static_cast<int64_t>(t) * row_stride;
  int page = 0;
  bool bad = false;
  if (write_kv) {
    const int b = request_of_token[t];
    page = pos >= 0 ? block_table[static_cast<int64_t>(b) * max_blocks + pos / page_size] : -1;
    bad = page < 0 || page >= num_pages;
    if (bad && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, LE_STATUS_BAD_PAGE);
  }
  __syncthreads();
  const int at_once = 32 / lph, sub = lane % lph, mine = lane / lph;
  const int pieces = head_dim / N;
  const int all = heads + (write_kv ? kv_heads : 0);
  const int h_end = min(all, (static_cast<int>(blockIdx.y) + 1) * heads_per_block);
  for (int h0 = blockIdx.y * heads_per_block + warp * at_once; h0 < h_end; h0 += warps * at_once) {
    const int h = h0 + mine;
    const bool is_key = h >= heads;
    const bool live = h < h_end && !(is_key && bad);
    T *x = row + static_cast<int64_t>(h) * head_dim;
    T *k_dst = nullptr, *v_dst = nullptr;
    if (live && is_key) {
      const int64_t at = ((static_cast<int64_t>(page) * kv_heads + (h - heads)) * page_size + pos % page_size) * head_dim;
      k_dst = k_cache + at;
      v_dst = values_are_keys ? v_cache + at : nullptr;
    }
    float val[HELD][N];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < HELD; ++i) {
      const int c = sub + i * lph;
      if (live && c < pieces) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(x + c * N);
        if (v_dst != nullptr) *reinterpret_cast<uint4 *>(v_dst + c * N) = raw;     // (as projected: the same bits)
        Piece<T>::open(raw, val[i]);
#pragma unroll
        for (int e = 0; e < N; e += 2) {
          const int j = c * N + e - rot_col;
          float u = val[i][e], v = val[i][e + 1];
          if (j >= 0 && j + 1 < rot) {
            const float sn = turn[j], cs = turn[j + 1];
            const float nu = u * cs - v * sn, nv = v * cs + u * sn;
            u = nu, v = nv;
          }
          val[i][e] = u, val[i][e + 1] = v;
          ss = fmaf(u, u, fmaf(v, v, ss));
        }
      }
    }
    float inv = 1.0f;
    if (unit) {
      for (int o = 1; o < lph; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      inv = rsqrtf(ss / static_cast<float>(norm_dim) + eps);
    }
    T *dst = is_key ? k_dst : x;
#pragma unroll
    for (int i = 0; i < HELD; ++i) {
      const int c = sub + i * lph;
      if (live && c < pieces) *reinterpret_cast<uint4 *>(dst + c * N) = Piece<T>::close(val[i], inv);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_rope_store_kernel(const T *__restrict__ src, int64_t src_stride, int col, int rank, int rot, int padded,
                         const float *__restrict__ weight, float eps, const float *__restrict__ rates, T *__restrict__ cache,
                         int col2, int rank2, const float *__restrict__ weight2, T *__restrict__ out2, int64_t out2_stride,
                         const int32_t *__restrict__ positions, const int32_t *__restrict__ request_of_token,
                         const int32_t *__restrict__ block_table, int max_blocks, int page_size, int num_pages,
                         int *__restrict__ status) {
  __shared__ float scratch[33];
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const T *row = src + static_cast<int64_t>(t) * src_stride;
  // Everything is asked for before anything is waited for: the page, both latents' sums of squares.
  int pos = 0, page = -1;
  if (cache != nullptr) {
    pos = positions[t];
    const int b = request_of_token[t];
    page = pos >= 0 ? block_table[static_cast<int64_t>(b) * max_blocks + pos / page_size] : -1;
  }
  const T *x = row + col;
  float ss2 = 0.0f, ss = 0.0f;
  if (out2 != nullptr) {
    for (int i = threadIdx.x; i < rank2; i += blockDim.x) {
      const float v = le::to_f32(row[col2 + i]);
      ss2 = fmaf(v, v, ss2);
    }
  }
  if (cache != nullptr) {
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
      const float v = le::to_f32(x[i]);
      ss = fmaf(v, v, ss);
    }
  }
  if (out2 != nullptr) {
    ss2 = le::block_sum(ss2, scratch);
    const float inv = rsqrtf(ss2 / static_cast<float>(rank2) + eps);
    T *dst = out2 + static_cast<int64_t>(t) * out2_stride;
    for (int i = threadIdx.x; i < rank2; i += blockDim.x) dst[i] = le::from_f32<T>(le::to_f32(row[col2 + i]) * inv * weight2[i]);
  }
  if (cache == nullptr) return;
  const bool bad = page < 0 || page >= num_pages;
  if (bad && threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_PAGE);
  ss = le::block_sum(ss, scratch);
  if (bad) return;
  const float inv = rsqrtf(ss / static_cast<float>(rank) + eps);
  const float fpos = static_cast<float>(pos);
  T *dst = cache + (static_cast<int64_t>(page) * page_size + pos % page_size) * padded;
  for (int i = threadIdx.x; i < padded; i += blockDim.x) {
    float v = 0.0f;
    if (i < rank) {
      v = le::to_f32(x[i]) * inv * weight[i];
    } else if (i < rank + rot) {
      const int j = i - rank;
      v = le::to_f32(x[i]);
      if ((j | 1) < rot) {
        const float other = le::to_f32(x[rank + (j ^ 1)]);
        float s, c;
        sincosf(fpos * rates[j >> 1], &s, &c);
        v = (j & 1) ? v * c + other * s : v * c - other * s;
      }
    }
    dst[i] = le::from_f32<T>(v);
  }
}

}  // namespace

// rows: [tokens] rows of row_stride elements, queries then keys, heads of head_dim entries (even, at most 512).
// k_cache / v_cache: [pages, kv_heads, page, head_dim].  write_kv 0: queries only (the keys' columns are not read).
LE_API int le_rope_norm_store(void *rows, int64_t row_stride, int dtype, void *k_cache, void *v_cache, const float *rates,
                              const int32_t *positions, const int32_t *request_of_token, const int32_t *block_table,
                              int max_blocks, int num_tokens, int heads, int kv_heads, int head_dim, int rot_col, int rot,
                              int unit, float eps, int norm_dim, int page_size, int num_pages, int write_kv,
                              int values_are_keys, int *status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (head_dim < 2 || head_dim % 2 || head_dim > 64 * RN_MAX_PAIRS)
    return le::invalid("le_rope_norm_store: heads of %d entries (even, at most %d)", head_dim, 64 * RN_MAX_PAIRS);
  if (rot < 0 || rot % 2 || rot_col < 0 || rot_col % 2 || rot_col + rot > head_dim)
    return le::invalid("le_rope_norm_store: %d turned entries from column %d of a head of %d", rot, rot_col, head_dim);
  const int all = heads + (write_kv ? kv_heads : 0);
  const int per_block = num_tokens >= 512 ? 16 : 4;       // few tokens: more blocks; many: the sines serve more heads
  const dim3 grid(num_tokens, (all + per_block - 1) / per_block);
  if (grid.y > 65535) return le::invalid("le_rope_norm_store: %d heads are too many for one launch", all);
  const size_t elem = dtype == LE_BF16 ? 2 : 4;
  const auto pairs_aligned = [&](const void *p) { return reinterpret_cast<uintptr_t>(p) % (2 * elem) == 0; };
  const int together = pairs_aligned(rows) && row_stride % 2 == 0 && pairs_aligned(k_cache) && pairs_aligned(v_cache);
  const size_t smem = sizeof(float) * (rot > 0 ? rot : 2);
  const int per_piece = static_cast<int>(16 / elem);
  const auto on16 = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (head_dim % per_piece == 0 && row_stride % per_piece == 0 && on16(rows) && on16(k_cache) && on16(v_cache)) {
    int lph = 1;
    while (lph < 32 && lph * per_piece < head_dim) lph <<= 1;
    LE_DISPATCH_DTYPE(dtype, T,
                      return le::launch_chained(rope_norm_store_pieces_kernel<T>, grid, dim3(128), smem, stream,
                                                static_cast<T *>(rows), row_stride, static_cast<T *>(k_cache),
                                                static_cast<T *>(v_cache), rates, positions, request_of_token, block_table,
                                                max_blocks, heads, kv_heads, head_dim, rot_col, rot, unit, eps, norm_dim,
                                                page_size, num_pages, write_kv, values_are_keys, per_block, lph, status));
  }
  LE_DISPATCH_DTYPE(dtype, T,
                    return le::launch_chained(rope_norm_store_kernel<T>, grid, dim3(128), smem, stream,
                                              static_cast<T *>(rows), row_stride, static_cast<T *>(k_cache),
                                              static_cast<T *>(v_cache), rates, positions, request_of_token, block_table,
                                              max_blocks, heads, kv_heads, head_dim, rot_col, rot, unit, eps, norm_dim,
                                              page_size, num_pages, write_kv, values_are_keys, per_block, together, status));
}

// cache: [pages, 1, page, padded] or null (nothing is stored); out2 null: no second latent.
LE_API int le_latent_rope_store(const void *src, int64_t src_stride, int dtype, int col, int rank, int rot, int padded,
                                const float *weight, float eps, const float *rates, void *cache, int col2, int rank2,
                                const float *weight2, void *out2, int64_t out2_stride, const int32_t *positions,
                                const int32_t *request_of_token, const int32_t *block_table, int max_blocks, int num_tokens,
                                int page_size, int num_pages, int *status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rank < 1 || rot < 0 || rot % 2 || padded < rank + rot)
    return le::invalid("le_latent_rope_store: rank %d, %d turned entries, padded %d", rank, rot, padded);
  LE_DISPATCH_DTYPE(dtype, T,
                    return le::launch_chained(latent_rope_store_kernel<T>, dim3(num_tokens), dim3(128), 0, stream,
                                              static_cast<const T *>(src), src_stride, col, rank, rot, padded, weight, eps,
                                              rates, static_cast<T *>(cache), col2, rank2, weight2, static_cast<T *>(out2),
                                              out2_stride, positions, request_of_token, block_table, max_blocks, page_size,
                                              num_pages, status));
}
