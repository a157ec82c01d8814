// The gated delta rule: a linear recurrence over a matrix of state per head.
//
// Per head, with S the state [dim, vdim] (32-bit, carried from token to token
// for each request), k and q unit vectors of the head's key group (q also
// times dim^-1/2), v the head's values, and two numbers per token,
//   g    = exp(-exp(A_log) * softplus(a + dt_bias))     the decay, in (0, 1)
//   beta = sigmoid(b)                                   the step size,
// a token does, in this order,
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.
// Every column of S (one entry of v, u and o) goes its own way: column j needs
// k, q, g, beta and v_j only.  With S0 the state before the token,
//   u_j = beta (v_j - g (S0[:, j] . k)),   o_j = g (S0[:, j] . q) + (k . q) u_j,
// so both dot products run over the old column, and the column is then
// brought up to date with one multiply-add per entry.
//
// gated_delta_prepare_kernel: what a token brings to the recurrence besides
// its vectors, made once for all columns: per key group the inverse lengths of
// k and q (q's times the query scale) and the unit vectors' product k . q, per
// head the decay and the step size; five 32-bit numbers a (token, head) in a
// row of 4 * groups + 2 * heads floats per token.
//
// gated_delta_scan_kernel: a block takes one request, one head and a slice of
// columns; a column belongs to `lanes` neighbouring lanes, each holding ROWS of
// its entries in registers (lanes * ROWS >= dim; partial dot products meet by
// shuffles).  The request's tokens of the step are walked in order, in tiles
// of up to SCAN_MAX_TILE tokens held twice in shared memory: while the
// threads that hold the state run one tile, two more warps fetch the next one
// (k and q as projected, in their own type; the column slice of v; the
// token's five numbers).  The unit vectors are never written out: with a and
// c the inverse lengths,
//   S0 . k_unit = a (S0 . k),   S += k_unit u^T = k (a u)^T,   S . q_unit = c (S . q).
// The state is kept transposed, [vdim, dim] per head, so that a thread's
// entries are consecutive; it is read before the first token and written
// after the last.  Rows that stand for no request (slot < 0) give zeros and
// keep nothing.
//
// head_norm_gate_kernel: o of every (token, head) is divided by its root mean
// square over vdim, times a weight [vdim], times silu(gate).
//
// Everything here is 32-bit except the inputs (projections and convolution
// outputs in the activations' type) and the gated result, which is rounded once.
#include "common.cuh"

namespace {

constexpr int SCAN_HOLDERS = 128;     // threads that hold state
constexpr int SCAN_FETCHERS = 64;     // threads that fetch the next tile
constexpr int SCAN_THREADS = SCAN_HOLDERS + SCAN_FETCHERS;
constexpr int SCAN_MAX_TILE = 16;
constexpr int SCAN_NUMBERS = 8;       // floats a token has in shared memory: 1/|k|, scale/|q|, k.q, decay, step, -, -, -
constexpr int PREP_THREADS = 128;

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS)
gated_delta_prepare_kernel(float *__restrict__ prep, int prep_stride, const T *__restrict__ qkv, int64_t qkv_stride, int q_col,
                           int k_col, const T *__restrict__ proj, int64_t proj_stride, int b_col, int a_col,
                           const float *__restrict__ a_log, const float *__restrict__ dt_bias, int heads, int kv_heads,
                           int dim, float unit_eps, float q_scale) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = PREP_THREADS / 32;
  float *dst = prep + t * prep_stride;
  for (int g = blockIdx.y * warps + warp; g < kv_heads; g += gridDim.y * warps) {
    const T *kr = qkv + t * qkv_stride + k_col + g * dim;
    const T *qr = qkv + t * qkv_stride + q_col + g * dim;
    float kk = 0.0f, qq = 0.0f, kq = 0.0f;
    for (int i = lane; i < dim; i += 32) {
      const float a = le::to_f32(kr[i]), c = le::to_f32(qr[i]);
      kk = fmaf(a, a, kk);
      qq = fmaf(c, c, qq);
      kq = fmaf(a, c, kq);
    }
    kk = le::warp_sum(kk);
    qq = le::warp_sum(qq);
    kq = le::warp_sum(kq);
    if (lane == 0) {
      const float k_inv = rsqrtf(kk + unit_eps), q_inv = rsqrtf(qq + unit_eps) * q_scale;
      dst[4 * g + 0] = k_inv;
      dst[4 * g + 1] = q_inv;
      dst[4 * g + 2] = kq * k_inv * q_inv;
      dst[4 * g + 3] = 0.0f;
    }
  }
  for (int h = blockIdx.y * PREP_THREADS + threadIdx.x; h < heads; h += gridDim.y * PREP_THREADS) {
    const float av = le::to_f32(proj[t * proj_stride + a_col + h]), bv = le::to_f32(proj[t * proj_stride + b_col + h]);
    dst[4 * kv_heads + 2 * h + 0] = expf(-expf(a_log[h]) * softplus_f32(av + dt_bias[h]));
    dst[4 * kv_heads + 2 * h + 1] = sigmoid_f32(bv);
  }
}

// ROWS consecutive entries of a tile's row, as floats.
template <int ROWS>
__device__ __forceinline__ void load_rows(const __nv_bfloat16 *p, float *d) {
#pragma unroll
  for (int i = 0; i < ROWS / 8; ++i) {
    const uint4 r = reinterpret_cast<const uint4 *>(p)[i];
    d[8 * i + 0] = __uint_as_float(r.x << 16), d[8 * i + 1] = __uint_as_float(r.x & 0xffff0000u);
    d[8 * i + 2] = __uint_as_float(r.y << 16), d[8 * i + 3] = __uint_as_float(r.y & 0xffff0000u);
    d[8 * i + 4] = __uint_as_float(r.z << 16), d[8 * i + 5] = __uint_as_float(r.z & 0xffff0000u);
    d[8 * i + 6] = __uint_as_float(r.w << 16), d[8 * i + 7] = __uint_as_float(r.w & 0xffff0000u);
  }
}
template <int ROWS>
__device__ __forceinline__ void load_rows(const float *p, float *d) {
#pragma unroll
  for (int i = 0; i < ROWS / 4; ++i) {
    const float4 r = reinterpret_cast<const float4 *>(p)[i];
    d[4 * i + 0] = r.x, d[4 * i + 1] = r.y, d[4 * i + 2] = r.z, d[4 * i + 3] = r.w;
  }
}

template <typename T, int ROWS>
__global__ void __launch_bounds__(SCAN_THREADS)
gated_delta_scan_kernel(float *__restrict__ out, int64_t out_stride, const T *__restrict__ qkv, int64_t qkv_stride, int q_col,
                        int k_col, int v_col, const float *__restrict__ prep, int prep_stride, float *__restrict__ state,
                        int num_state_rows, const int32_t *__restrict__ state_slots, const int32_t *__restrict__ cu_q,
                        int heads, int kv_heads, int dim, int vdim, int lanes, int tile, int wide) {
  extern __shared__ __align__(16) unsigned char scan_smem[];
  constexpr int VEC = 16 / sizeof(T);               // entries of a 16-byte piece
  const int dpad = lanes * ROWS;
  const int cols = SCAN_HOLDERS / lanes;            // columns of this block
  // One of the two buffers: k [tile][dpad] T | q [tile][dpad] T | v [tile][cols] float | numbers [tile][SCAN_NUMBERS] float.
  const size_t vec_bytes = static_cast<size_t>(tile) * dpad * sizeof(T);
  const size_t buf_bytes = 2 * vec_bytes + sizeof(float) * tile * (cols + SCAN_NUMBERS);
  le::let_successor_start();
  const int b = blockIdx.z, h = blockIdx.y;
  const int group = h / (heads / kv_heads);
  const int first = cu_q[b], q_len = cu_q[b + 1] - first;
  const int slot = state_slots[b];
  const bool kept = slot >= 0 && slot < num_state_rows;
  const bool holder = threadIdx.x < SCAN_HOLDERS;
  const int col = (threadIdx.x % SCAN_HOLDERS) / lanes, part = threadIdx.x % lanes;
  const int j = blockIdx.x * cols + col;            // this thread's column of the state
  const bool col_ok = j < vdim;
  float S[ROWS];
  float *mine = nullptr;
  if (holder && kept && col_ok)
    mine = state + ((static_cast<int64_t>(slot) * heads + h) * vdim + j) * dim + part * ROWS;
  if (mine != nullptr && dim % 4 == 0) {            // (every thread's entries then start on 16 bytes)
#pragma unroll
    for (int i = 0; i < ROWS; i += 4) {
      float4 r = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (part * ROWS + i < dim) r = *reinterpret_cast<const float4 *>(mine + i);
      S[i] = r.x, S[i + 1] = r.y, S[i + 2] = r.z, S[i + 3] = r.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) S[i] = (mine != nullptr && part * ROWS + i < dim) ? mine[i] : 0.0f;
  }

  auto fetch = [&](int buf, int t0, int n, int tid, int nthreads) {
    unsigned char *base = scan_smem + buf * buf_bytes;
    T *kt = reinterpret_cast<T *>(base), *qt = reinterpret_cast<T *>(base + vec_bytes);
    float *vt = reinterpret_cast<float *>(base + 2 * vec_bytes), *nt = vt + tile * cols;
    const T *src0 = qkv + static_cast<int64_t>(first + t0) * qkv_stride + group * dim;
    if (wide) {
      const int pieces = dpad / VEC, per = n * pieces;
      for (int idx = tid; idx < 2 * per; idx += nthreads) {
        const int which = idx >= per, r = idx - which * per, t = r / pieces, c = (r - t * pieces) * VEC;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (c < dim) val = *reinterpret_cast<const uint4 *>(src0 + t * qkv_stride + (which ? q_col : k_col) + c);
        *reinterpret_cast<uint4 *>((which ? qt : kt) + t * dpad + c) = val;
      }
    } else {
      const int per = n * dpad;
      for (int idx = tid; idx < 2 * per; idx += nthreads) {
        const int which = idx >= per, r = idx - which * per, t = r / dpad, c = r - t * dpad;
        T val = le::from_f32<T>(0.0f);
        if (c < dim) val = src0[t * qkv_stride + (which ? q_col : k_col) + c];
        (which ? qt : kt)[t * dpad + c] = val;
      }
    }
    for (int idx = tid; idx < n * cols; idx += nthreads) {
      const int t = idx / cols, c = idx - t * cols;
      const int jj = blockIdx.x * cols + c;
      vt[idx] = jj < vdim ? le::to_f32(qkv[static_cast<int64_t>(first + t0 + t) * qkv_stride + v_col + h * vdim + jj]) : 0.0f;
    }
    for (int idx = tid; idx < n * 5; idx += nthreads) {
      const int t = idx / 5, s = idx - t * 5;
      const float *row = prep + static_cast<int64_t>(first + t0 + t) * prep_stride;
      nt[t * SCAN_NUMBERS + s] = s < 3 ? row[4 * group + s] : row[4 * kv_heads + 2 * h + (s - 3)];
    }
  };

  le::wait_for_predecessor();
  if (q_len > 0) fetch(0, 0, min(tile, q_len), threadIdx.x, SCAN_THREADS);
  __syncthreads();
  int buf = 0;
  for (int t0 = 0; t0 < q_len; t0 += tile, buf ^= 1) {
    const int n = min(tile, q_len - t0);
    if (!holder) {
      if (t0 + tile < q_len) fetch(buf ^ 1, t0 + tile, min(tile, q_len - t0 - tile), threadIdx.x - SCAN_HOLDERS, SCAN_FETCHERS);
    } else {
      const unsigned char *base = scan_smem + buf * buf_bytes;
      const T *kt = reinterpret_cast<const T *>(base) + part * ROWS;
      const T *qt = reinterpret_cast<const T *>(base + vec_bytes) + part * ROWS;
      const float *vt = reinterpret_cast<const float *>(base + 2 * vec_bytes), *nt = vt + tile * cols;
      for (int t = 0; t < n; ++t) {
        float kreg[ROWS], qreg[ROWS];
        load_rows<ROWS>(kt + t * dpad, kreg);
        load_rows<ROWS>(qt + t * dpad, qreg);
        const float4 num = *reinterpret_cast<const float4 *>(nt + t * SCAN_NUMBERS);   // 1/|k|, scale/|q|, k.q, decay
        const float beta = nt[t * SCAN_NUMBERS + 4];
        const float v = vt[t * cols + col];
        float dk[4] = {0.0f, 0.0f, 0.0f, 0.0f}, dq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < ROWS; ++i) dk[i & 3] = fmaf(S[i], kreg[i], dk[i & 3]), dq[i & 3] = fmaf(S[i], qreg[i], dq[i & 3]);
        float sk = (dk[0] + dk[1]) + (dk[2] + dk[3]), sq = (dq[0] + dq[1]) + (dq[2] + dq[3]);
        for (int o = 1; o < lanes; o <<= 1) {
          sk += __shfl_xor_sync(0xffffffffu, sk, o);
          sq += __shfl_xor_sync(0xffffffffu, sq, o);
        }
        const float g = num.w;
        const float u = beta * (v - g * (sk * num.x));       // beta (v - (g S0)^T k_unit)
        const float uk = u * num.x;
#pragma unroll
        for (int i = 0; i < ROWS; ++i) S[i] = fmaf(kreg[i], uk, g * S[i]);
        // o = (g S0 + k_unit u^T)^T q_unit = g (S0 . q_unit) + (k_unit . q_unit) u
        if (part == 0 && col_ok)
          out[static_cast<int64_t>(first + t0 + t) * out_stride + h * vdim + j] = kept ? fmaf(g * num.y, sq, num.z * u) : 0.0f;
      }
    }
    __syncthreads();            // the next tile is there, and this one is done with
  }
  if (mine != nullptr) {
    if (dim % 4 == 0) {
#pragma unroll
      for (int i = 0; i < ROWS; i += 4)
        if (part * ROWS + i < dim) *reinterpret_cast<float4 *>(mine + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < ROWS; ++i)
        if (part * ROWS + i < dim) mine[i] = S[i];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(T *__restrict__ out, int64_t out_stride, const float *__restrict__ o, int64_t o_stride,
                      const T *__restrict__ gate, int64_t gate_stride, const float *__restrict__ weight, float eps,
                      int num_tokens, int heads, int vdim) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<int64_t>(num_tokens) * heads) return;
  const int64_t t = item / heads;
  const int h = static_cast<int>(item - t * heads);
  const float *x = o + t * o_stride + h * vdim;
  float ss = 0.0f;
  for (int i = lane; i < vdim; i += 32) ss = fmaf(x[i], x[i], ss);
  ss = le::warp_sum(ss);
  const float inv = rsqrtf(ss / static_cast<float>(vdim) + eps);
  const T *gr = gate + t * gate_stride + h * vdim;
  T *dst = out + t * out_stride + h * vdim;
  for (int i = lane; i < vdim; i += 32) {
    const float z = le::to_f32(gr[i]);
    dst[i] = le::from_f32<T>(x[i] * inv * weight[i] * (z / (1.0f + expf(-z))));
  }
}

}  // namespace

// The lanes that share a column of the state for heads of `dim` entries (a power of two; 0: dim is too large).
LE_API int le_gated_delta_lanes(int dim) {
  for (int lanes = 1; lanes <= 32; lanes <<= 1)
    if (lanes * (dim <= 256 ? 8 : 32) >= dim) return lanes;
  return 0;
}

// Floats per token of the scratch rows that le_gated_delta_scan needs.
LE_API int le_gated_delta_scratch(int heads, int kv_heads) { return 4 * kv_heads + 2 * heads; }

// out [tokens, heads * vdim] float32.  qkv: rows holding the convolved, activated queries and keys [kv_heads, dim]
// at columns q_col and k_col and values [heads, vdim] at v_col.  proj: rows holding one number per head at b_col
// (step size before its sigmoid) and at a_col (decay before its softplus).  state: [rows, heads, vdim, dim] float32.
// scratch: [tokens, le_gated_delta_scratch()] float32, rewritten here.
LE_API int le_gated_delta_scan(float *out, int64_t out_stride, const void *qkv, int64_t qkv_stride, int q_col, int k_col,
                               int v_col, const void *proj, int64_t proj_stride, int b_col, int a_col, int dtype,
                               const float *a_log, const float *dt_bias, float *state, int num_state_rows,
                               const int32_t *state_slots, const int32_t *cu_q, int num_requests, int num_tokens, int heads,
                               int kv_heads, int dim, int vdim, float unit_eps, float q_scale, float *scratch,
                               cudaStream_t stream) {
  if (num_requests <= 0 || num_tokens <= 0) return 0;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads) return le::invalid("le_gated_delta_scan: %d heads, %d groups", heads, kv_heads);
  const int lanes = le_gated_delta_lanes(dim);
  if (dim < 1 || lanes == 0) return le::invalid("le_gated_delta_scan: heads of %d entries (at most 1024)", dim);
  if (dtype != LE_BF16 && dtype != LE_F32) return le::invalid("le_gated_delta_scan: unknown dtype code %d", dtype);
  const int rows = dim <= 256 ? 8 : 32;
  const int cols = SCAN_HOLDERS / lanes;
  const int prep_stride = le_gated_delta_scratch(heads, kv_heads);
  const size_t elem = dtype == LE_BF16 ? 2 : 4;
  const int vec = static_cast<int>(16 / elem);
  const int wide = dim % vec == 0 && qkv_stride % vec == 0 && q_col % vec == 0 && k_col % vec == 0 &&
                   reinterpret_cast<uintptr_t>(qkv) % 16 == 0;
  const size_t per_token = 2 * static_cast<size_t>(lanes) * rows * elem + sizeof(float) * (cols + SCAN_NUMBERS);
  int tile = static_cast<int>((40 * 1024) / per_token);
  tile = tile < 1 ? 1 : (tile > SCAN_MAX_TILE ? SCAN_MAX_TILE : tile);
  const size_t smem = 2 * tile * per_token;
  const dim3 prep_grid(num_tokens, (kv_heads + PREP_THREADS / 32 - 1) / (PREP_THREADS / 32));
  const dim3 grid((vdim + cols - 1) / cols, heads, num_requests);
  if (grid.y > 65535 || grid.z > 65535 || prep_grid.y > 65535)
    return le::invalid("le_gated_delta_scan: too many heads or requests for one launch");
#define LE_GO(T, R)                                                                                                     \
  do {                                                                                                                  \
    int rc = le::launch_chained(gated_delta_prepare_kernel<T>, prep_grid, dim3(PREP_THREADS), 0, stream, scratch,       \
                                prep_stride, static_cast<const T *>(qkv), qkv_stride, q_col, k_col,                     \
                                static_cast<const T *>(proj), proj_stride, b_col, a_col, a_log, dt_bias, heads, kv_heads, \
                                dim, unit_eps, q_scale);                                                                \
    if (rc != 0) return rc;                                                                                             \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(gated_delta_scan_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    return le::launch_chained(gated_delta_scan_kernel<T, R>, grid, dim3(SCAN_THREADS), smem, stream, out, out_stride,   \
                              static_cast<const T *>(qkv), qkv_stride, q_col, k_col, v_col,                             \
                              static_cast<const float *>(scratch), prep_stride, state, num_state_rows, state_slots, cu_q, \
                              heads, kv_heads, dim, vdim, lanes, tile, wide);                                           \
  } while (0)
  if (dtype == LE_BF16) { if (rows == 8) LE_GO(__nv_bfloat16, 8); LE_GO(__nv_bfloat16, 32); }
  if (rows == 8) LE_GO(float, 8);
  LE_GO(float, 32);
#undef LE_GO
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * silu(gate[t, h, :]).
LE_API int le_head_norm_gate(void *out, int64_t out_stride, const float *o, int64_t o_stride, const void *gate,
                             int64_t gate_stride, int dtype, const float *weight, float eps, int num_tokens, int heads,
                             int vdim, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int64_t items = static_cast<int64_t>(num_tokens) * heads;
  const dim3 grid(static_cast<unsigned>((items + 3) / 4));
  LE_DISPATCH_DTYPE(dtype, T,
                    return le::launch_chained(head_norm_gate_kernel<T>, grid, dim3(128), 0, stream, static_cast<T *>(out),
                                              out_stride, o, o_stride, static_cast<const T *>(gate), gate_stride, weight,
                                              eps, num_tokens, heads, vdim));
}
