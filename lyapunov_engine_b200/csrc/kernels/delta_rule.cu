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
// gated_delta_scan_kernel: a block takes one request, one head and a slice of
// columns; a column belongs to R neighbouring lanes, each holding ROWS of its
// entries in registers (R * ROWS >= dim; partial dot products meet by
// shuffles).  The request's tokens of the step are walked in order, in tiles
// of SCAN_TILE tokens: the block first makes the tile's unit vectors, k . q,
// decays and step sizes in shared memory (a warp per token), then every
// thread runs the tile's tokens over its part of the column.  The state is
// kept transposed, [vdim, dim] per head, so that a thread's entries are
// consecutive; it is read before the first token and written after the last.
// Rows that stand for no request (slot < 0) give zeros and keep nothing.
//
// head_norm_gate_kernel: o of every (token, head) is divided by its root mean
// square over vdim, times a weight [vdim], times silu(gate).
//
// Everything here is 32-bit except the inputs (projections and convolution
// outputs in the activations' type) and the gated result, which is rounded once.
#include "common.cuh"

namespace {

constexpr int SCAN_THREADS = 128;
constexpr int SCAN_TILE = 16;

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename T, int ROWS>
__global__ void __launch_bounds__(SCAN_THREADS)
gated_delta_scan_kernel(float *__restrict__ out, int64_t out_stride, const T *__restrict__ qkv, int64_t qkv_stride, int q_col,
                        int k_col, int v_col, const T *__restrict__ proj, int64_t proj_stride, int b_col, int a_col,
                        const float *__restrict__ a_log, const float *__restrict__ dt_bias, float *__restrict__ state,
                        int num_state_rows, const int32_t *__restrict__ state_slots, const int32_t *__restrict__ cu_q,
                        int heads, int kv_heads, int dim, int vdim, int lanes, float unit_eps, float q_scale) {
  extern __shared__ float smem[];
  const int dpad = lanes * ROWS;
  const int cols = SCAN_THREADS / lanes;           // columns of this block
  float *k_tile = smem;                            // [SCAN_TILE][dpad]
  float *q_tile = k_tile + SCAN_TILE * dpad;       // [SCAN_TILE][dpad]
  float *v_tile = q_tile + SCAN_TILE * dpad;       // [SCAN_TILE][cols]
  float *scalars = v_tile + SCAN_TILE * cols;      // [SCAN_TILE][4]: g, beta, k . q
  le::let_successor_start();
  const int b = blockIdx.z, h = blockIdx.y;
  const int group = h / (heads / kv_heads);
  const int col = threadIdx.x / lanes, part = threadIdx.x % lanes;
  const int j = blockIdx.x * cols + col;           // this thread's column of the state
  const bool col_ok = j < vdim;
  const int first = cu_q[b], q_len = cu_q[b + 1] - first;
  const int slot = state_slots[b];
  const bool kept = slot >= 0 && slot < num_state_rows;
  float S[ROWS];
  float *mine = nullptr;
  if (kept && col_ok)
    mine = state + ((static_cast<int64_t>(slot) * heads + h) * vdim + j) * dim + part * ROWS;
#pragma unroll
  for (int i = 0; i < ROWS; ++i) S[i] = (mine != nullptr && part * ROWS + i < dim) ? mine[i] : 0.0f;
  const float decay_rate = -expf(a_log[h]), bias = dt_bias[h];

  le::wait_for_predecessor();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t0 = 0; t0 < q_len; t0 += SCAN_TILE) {
    const int n = min(SCAN_TILE, q_len - t0);
    __syncthreads();            // the tile before is done with
    for (int t = warp; t < n; t += SCAN_THREADS / 32) {
      const int64_t row = first + t0 + t;
      const T *kr = qkv + row * qkv_stride + k_col + group * dim;
      const T *qr = qkv + row * qkv_stride + q_col + group * dim;
      float kk = 0.0f, qq = 0.0f;
      for (int i = lane; i < dim; i += 32) {
        const float a = le::to_f32(kr[i]), c = le::to_f32(qr[i]);
        kk += a * a;
        qq += c * c;
      }
      kk = le::warp_sum(kk);
      qq = le::warp_sum(qq);
      const float k_inv = rsqrtf(kk + unit_eps), q_inv = rsqrtf(qq + unit_eps) * q_scale;
      float kq = 0.0f;
      for (int i = lane; i < dpad; i += 32) {
        const float a = i < dim ? le::to_f32(kr[i]) * k_inv : 0.0f, c = i < dim ? le::to_f32(qr[i]) * q_inv : 0.0f;
        k_tile[t * dpad + i] = a;
        q_tile[t * dpad + i] = c;
        kq += a * c;
      }
      kq = le::warp_sum(kq);
      if (lane == 0) {
        const float av = le::to_f32(proj[row * proj_stride + a_col + h]), bv = le::to_f32(proj[row * proj_stride + b_col + h]);
        scalars[t * 4 + 0] = expf(decay_rate * softplus_f32(av + bias));
        scalars[t * 4 + 1] = sigmoid_f32(bv);
        scalars[t * 4 + 2] = kq;
      }
    }
    for (int i = threadIdx.x; i < n * cols; i += SCAN_THREADS) {
      const int t = i / cols, c = i - t * cols;
      const int jj = blockIdx.x * cols + c;
      v_tile[i] = jj < vdim ? le::to_f32(qkv[(first + t0 + t) * qkv_stride + v_col + h * vdim + jj]) : 0.0f;
    }
    __syncthreads();
    for (int t = 0; t < n; ++t) {
      const float *kt = k_tile + t * dpad + part * ROWS, *qt = q_tile + t * dpad + part * ROWS;
      float dk = 0.0f, dq = 0.0f;
      float kreg[ROWS];
#pragma unroll
      for (int i = 0; i < ROWS; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4 *>(kt + i), q4 = *reinterpret_cast<const float4 *>(qt + i);
        kreg[i] = k4.x, kreg[i + 1] = k4.y, kreg[i + 2] = k4.z, kreg[i + 3] = k4.w;
        dk = fmaf(S[i], k4.x, dk), dq = fmaf(S[i], q4.x, dq);
        dk = fmaf(S[i + 1], k4.y, dk), dq = fmaf(S[i + 1], q4.y, dq);
        dk = fmaf(S[i + 2], k4.z, dk), dq = fmaf(S[i + 2], q4.z, dq);
        dk = fmaf(S[i + 3], k4.w, dk), dq = fmaf(S[i + 3], q4.w, dq);
      }
      for (int o = 1; o < lanes; o <<= 1) {
        dk += __shfl_xor_sync(0xffffffffu, dk, o);
        dq += __shfl_xor_sync(0xffffffffu, dq, o);
      }
      const float g = scalars[t * 4 + 0], beta = scalars[t * 4 + 1], kq = scalars[t * 4 + 2];
      const float u = beta * (v_tile[t * cols + col] - g * dk);
#pragma unroll
      for (int i = 0; i < ROWS; ++i) S[i] = fmaf(kreg[i], u, g * S[i]);
      if (part == 0 && col_ok) out[(first + t0 + t) * out_stride + h * vdim + j] = kept ? fmaf(g, dq, kq * u) : 0.0f;
    }
  }
  if (mine != nullptr) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
      if (part * ROWS + i < dim) mine[i] = S[i];
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
    if (lanes * (dim <= 64 ? 16 : 32) >= dim) return lanes;
  return 0;
}

// out [tokens, heads * vdim] float32.  qkv: rows holding the convolved, activated queries and keys [kv_heads, dim]
// at columns q_col and k_col and values [heads, vdim] at v_col.  proj: rows holding one number per head at b_col
// (step size before its sigmoid) and at a_col (decay before its softplus).  state: [rows, heads, vdim, dim] float32.
LE_API int le_gated_delta_scan(float *out, int64_t out_stride, const void *qkv, int64_t qkv_stride, int q_col, int k_col,
                               int v_col, const void *proj, int64_t proj_stride, int b_col, int a_col, int dtype,
                               const float *a_log, const float *dt_bias, float *state, int num_state_rows,
                               const int32_t *state_slots, const int32_t *cu_q, int num_requests, int heads, int kv_heads,
                               int dim, int vdim, float unit_eps, float q_scale, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads) return le::invalid("le_gated_delta_scan: %d heads, %d groups", heads, kv_heads);
  const int lanes = le_gated_delta_lanes(dim);
  if (dim < 1 || lanes == 0) return le::invalid("le_gated_delta_scan: heads of %d entries (at most 1024)", dim);
  const int rows = dim <= 64 ? 16 : 32;
  const int cols = SCAN_THREADS / lanes;
  const dim3 grid((vdim + cols - 1) / cols, heads, num_requests);
  if (grid.y > 65535 || grid.z > 65535) return le::invalid("le_gated_delta_scan: too many heads or requests for one launch");
  const size_t smem = sizeof(float) * (2 * SCAN_TILE * lanes * rows + SCAN_TILE * cols + SCAN_TILE * 4);
#define LE_GO(T, R)                                                                                                     \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(gated_delta_scan_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    return le::launch_chained(gated_delta_scan_kernel<T, R>, grid, dim3(SCAN_THREADS), smem, stream, out, out_stride,   \
                              static_cast<const T *>(qkv), qkv_stride, q_col, k_col, v_col, static_cast<const T *>(proj), \
                              proj_stride, b_col, a_col, a_log, dt_bias, state, num_state_rows, state_slots, cu_q, heads, \
                              kv_heads, dim, vdim, lanes, unit_eps, q_scale);                                           \
  } while (0)
  if (dtype == LE_BF16) { if (rows == 16) LE_GO(__nv_bfloat16, 16); LE_GO(__nv_bfloat16, 32); }
  if (dtype == LE_F32) { if (rows == 16) LE_GO(float, 16); LE_GO(float, 32); }
#undef LE_GO
  return le::invalid("le_gated_delta_scan: unknown dtype code %d", dtype);
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
