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
// columns; a column belongs to LANES neighbouring lanes, each holding ROWS of
// its entries in registers, four at a time with LANES groups of four between
// them (LANES * ROWS >= dim; partial dot products meet by shuffles).  The
// request's tokens of the step are walked in order, in tiles of up to
// SCAN_MAX_TILE tokens held twice in shared memory: while the threads that
// hold the state run one tile, four more warps fetch the next one and make of
// it what the recurrence reads: k and q as 32-bit unit vectors (the projected
// entries times the token's inverse lengths), the column slice of v, and k . q,
// decay and step size.  So a token costs a holder two dot products over its
// rows, the shuffles, and one multiply-add and one multiply per entry.  The
// state is kept transposed, [vdim, dim] per head, so that a column is
// consecutive; it is read before the first token and written after the last.
// Rows that stand for no request (slot < 0) give zeros and keep nothing.  In a
// step of single tokens the block has no fetching warps.
//
// head_norm_gate_kernel: o of every (token, head) is divided by its root mean
// square over vdim, times a weight ([vdim], the same for every head, or [heads,
// vdim]), times silu(gate) or sigmoid(gate), times one number.
//
// Everything here is 32-bit except the inputs (projections and convolution
// outputs in the activations' type) and the gated result, which is rounded once.
#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int SCAN_HOLDERS = 128;     // threads that hold state
constexpr int SCAN_FETCHERS = 128;    // threads that fetch the next tile
constexpr int SCAN_THREADS = SCAN_HOLDERS + SCAN_FETCHERS;
constexpr int SCAN_MAX_TILE = 32;
constexpr int SCAN_BATCH = 4;         // pieces a fetching thread has in flight
constexpr int SCAN_NUMBERS = 4;       // floats a token has in shared memory: k . q, decay, step size, -
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

// A piece of a row as it is fetched: 16 bytes where the addresses allow it, else one entry.
template <typename T, int P>
struct RowPiece {
  using Raw = uint4;
  static __device__ __forceinline__ Raw zero() { return make_uint4(0u, 0u, 0u, 0u); }
  static __device__ __forceinline__ Raw load(const T *p) { return *reinterpret_cast<const uint4 *>(p); }
  // The piece as floats times `f`, to shared memory (16-byte aligned).
  static __device__ __forceinline__ void store(float *dst, const Raw &r, float f) {
    if constexpr (sizeof(T) == 2) {
      *reinterpret_cast<float4 *>(dst) = make_float4(__uint_as_float(r.x << 16) * f, __uint_as_float(r.x & 0xffff0000u) * f,
                                                     __uint_as_float(r.y << 16) * f, __uint_as_float(r.y & 0xffff0000u) * f);
      *reinterpret_cast<float4 *>(dst + 4) = make_float4(__uint_as_float(r.z << 16) * f, __uint_as_float(r.z & 0xffff0000u) * f,
                                                         __uint_as_float(r.w << 16) * f, __uint_as_float(r.w & 0xffff0000u) * f);
    } else {
      *reinterpret_cast<float4 *>(dst) = make_float4(__uint_as_float(r.x) * f, __uint_as_float(r.y) * f,
                                                     __uint_as_float(r.z) * f, __uint_as_float(r.w) * f);
    }
  }
};
template <typename T>
struct RowPiece<T, 1> {
  using Raw = float;
  static __device__ __forceinline__ Raw zero() { return 0.0f; }
  static __device__ __forceinline__ Raw load(const T *p) { return le::to_f32(*p); }
  static __device__ __forceinline__ void store(float *dst, const Raw &r, float f) { *dst = r * f; }
};

// n tokens' keys and queries of one group as 32-bit unit vectors (the query's times its scale) into kt and qt
// [n][dpad], zeros behind dim.  Every thread asks for SCAN_BATCH pieces before it waits for one.
template <typename T, int P>
__device__ __forceinline__ void fetch_unit_vectors(float *kt, float *qt, const T *src0, int64_t stride, int q_col, int k_col,
                                                   const float *prep0, int prep_stride, int group, int n, int dim, int dpad,
                                                   int tid, int nthreads) {
  using Piece = RowPiece<T, P>;
  const int pieces = dpad / P, per = n * pieces;
  for (int i0 = tid; i0 < 2 * per; i0 += SCAN_BATCH * nthreads) {
    typename Piece::Raw raw[SCAN_BATCH];
    float scale[SCAN_BATCH];
#pragma unroll
    for (int u = 0; u < SCAN_BATCH; ++u) {
      const int idx = i0 + u * nthreads;
      raw[u] = Piece::zero();
      scale[u] = 0.0f;
      if (idx < 2 * per) {
        const int which = idx >= per, r = idx - which * per, t = r / pieces, c = (r - t * pieces) * P;
        if (c < dim) {
          raw[u] = Piece::load(src0 + t * stride + (which ? q_col : k_col) + c);
          scale[u] = prep0[static_cast<int64_t>(t) * prep_stride + 4 * group + which];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < SCAN_BATCH; ++u) {
      const int idx = i0 + u * nthreads;
      if (idx < 2 * per) {
        const int which = idx >= per, r = idx - which * per;
        Piece::store((which ? qt : kt) + static_cast<int64_t>(r) * P, raw[u], scale[u]);
      }
    }
  }
}

template <typename T, int ROWS, int LANES>
__global__ void __launch_bounds__(SCAN_THREADS)
gated_delta_scan_kernel(float *__restrict__ out, int64_t out_stride, const T *__restrict__ qkv, int64_t qkv_stride, int q_col,
                        int k_col, int v_col, const float *__restrict__ prep, int prep_stride, float *__restrict__ state,
                        int num_state_rows, const int32_t *__restrict__ state_slots, const int32_t *__restrict__ cu_q,
                        int heads, int kv_heads, int dim, int vdim, int tile, int wide) {
  extern __shared__ __align__(16) unsigned char scan_smem[];
  constexpr int QUADS = ROWS / 4;                   // groups of four rows a thread holds
  constexpr int DPAD = ROWS * LANES;
  constexpr int COLS = SCAN_HOLDERS / LANES;        // columns of this block
  // One of the two buffers: k [tile][DPAD] | q [tile][DPAD] | v [tile][COLS] | numbers [tile][SCAN_NUMBERS], all float.
  const int vec_floats = tile * DPAD;
  const int buf_floats = 2 * vec_floats + tile * (COLS + SCAN_NUMBERS);
  float *smem = reinterpret_cast<float *>(scan_smem);
  le::let_successor_start();
  const int b = blockIdx.z, h = blockIdx.y;
  const int group = h / (heads / kv_heads);
  const int first = cu_q[b], q_len = cu_q[b + 1] - first;
  const int slot = state_slots[b];
  const bool kept = slot >= 0 && slot < num_state_rows;
  const bool holder = threadIdx.x < SCAN_HOLDERS;
  const int col = (threadIdx.x % SCAN_HOLDERS) / LANES, part = threadIdx.x % LANES;
  const int j = blockIdx.x * COLS + col;            // this thread's column of the state
  const bool col_ok = j < vdim;
  // Of its column a thread holds the rows 4 (i LANES + part) .. + 3, i < QUADS: neighbouring threads hold
  // neighbouring 16 bytes, of the state as of the tiles in shared memory.
  float S[ROWS];
  float *mine = nullptr;
  if (holder && kept && col_ok) mine = state + ((static_cast<int64_t>(slot) * heads + h) * vdim + j) * dim;
  const bool quads_whole = dim % 4 == 0;            // (every group of four then starts on 16 bytes and ends inside dim)
#pragma unroll
  for (int i = 0; i < QUADS; ++i) {
    const int r0 = 4 * (i * LANES + part);
    float4 r = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (mine != nullptr) {
      if (quads_whole) {
        if (r0 < dim) r = *reinterpret_cast<const float4 *>(mine + r0);
      } else {
        if (r0 < dim) r.x = mine[r0];
        if (r0 + 1 < dim) r.y = mine[r0 + 1];
        if (r0 + 2 < dim) r.z = mine[r0 + 2];
        if (r0 + 3 < dim) r.w = mine[r0 + 3];
      }
    }
    S[4 * i] = r.x, S[4 * i + 1] = r.y, S[4 * i + 2] = r.z, S[4 * i + 3] = r.w;
  }

  auto fetch = [&](int buf, int t0, int n, int tid, int nthreads) {
    float *kt = smem + buf * buf_floats, *qt = kt + vec_floats, *vt = qt + vec_floats, *nt = vt + tile * COLS;
    const T *src0 = qkv + static_cast<int64_t>(first + t0) * qkv_stride + group * dim;
    const float *prep0 = prep + static_cast<int64_t>(first + t0) * prep_stride;
    if (wide)
      fetch_unit_vectors<T, 16 / sizeof(T)>(kt, qt, src0, qkv_stride, q_col, k_col, prep0, prep_stride, group, n, dim, DPAD, tid, nthreads);
    else
      fetch_unit_vectors<T, 1>(kt, qt, src0, qkv_stride, q_col, k_col, prep0, prep_stride, group, n, dim, DPAD, tid, nthreads);
    // v's columns and three numbers a token: k . q, decay, step size
    constexpr int EACH = COLS + 3, SMALL = 4;
    const int small = n * EACH;
    for (int i0 = tid; i0 < small; i0 += SMALL * nthreads) {
      float val[SMALL];
#pragma unroll
      for (int u = 0; u < SMALL; ++u) {
        const int idx = i0 + u * nthreads;
        val[u] = 0.0f;
        if (idx < small) {
          const int t = idx / EACH, c = idx - t * EACH;
          if (c < COLS) {
            const int jj = blockIdx.x * COLS + c;
            if (jj < vdim) val[u] = le::to_f32(qkv[static_cast<int64_t>(first + t0 + t) * qkv_stride + v_col + h * vdim + jj]);
          } else {
            const float *row = prep0 + static_cast<int64_t>(t) * prep_stride;
            val[u] = c == COLS ? row[4 * group + 2] : row[4 * kv_heads + 2 * h + (c - COLS - 1)];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < SMALL; ++u) {
        const int idx = i0 + u * nthreads;
        if (idx < small) {
          const int t = idx / EACH, c = idx - t * EACH;
          if (c < COLS) vt[t * COLS + c] = val[u];
          else nt[t * SCAN_NUMBERS + (c - COLS)] = val[u];
        }
      }
    }
  };

  le::wait_for_predecessor();
  const int fetchers = static_cast<int>(blockDim.x) - SCAN_HOLDERS;    // (none in a step of single tokens)
  if (q_len > 0) fetch(0, 0, min(tile, q_len), threadIdx.x, blockDim.x);
  __syncthreads();
  const bool writer = holder && part == 0 && col_ok;
  int buf = 0;
  for (int t0 = 0; t0 < q_len; t0 += tile, buf ^= 1) {
    const int n = min(tile, q_len - t0);
    const bool more = t0 + tile < q_len;
    if (!holder) {
      if (more) fetch(buf ^ 1, t0 + tile, min(tile, q_len - t0 - tile), threadIdx.x - SCAN_HOLDERS, fetchers);
    } else {
      const float *kt = smem + buf * buf_floats + 4 * part, *qt = kt + vec_floats;
      const float *vt = smem + buf * buf_floats + 2 * vec_floats + col;
      const float *nt = smem + buf * buf_floats + 2 * vec_floats + tile * COLS;
      float *dst = out + static_cast<int64_t>(first + t0) * out_stride + h * vdim + j;
      for (int t = 0; t < n; ++t, kt += DPAD, qt += DPAD, vt += COLS, nt += SCAN_NUMBERS, dst += out_stride) {
        float kreg[ROWS], qreg[ROWS];
#pragma unroll
        for (int i = 0; i < QUADS; ++i) {
          const float4 k4 = *reinterpret_cast<const float4 *>(kt + 4 * i * LANES);
          const float4 q4 = *reinterpret_cast<const float4 *>(qt + 4 * i * LANES);
          kreg[4 * i] = k4.x, kreg[4 * i + 1] = k4.y, kreg[4 * i + 2] = k4.z, kreg[4 * i + 3] = k4.w;
          qreg[4 * i] = q4.x, qreg[4 * i + 1] = q4.y, qreg[4 * i + 2] = q4.z, qreg[4 * i + 3] = q4.w;
        }
        const float4 num = *reinterpret_cast<const float4 *>(nt);       // k . q, decay, step size
        const float v = *vt;
        float dk[4] = {0.0f, 0.0f, 0.0f, 0.0f}, dq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < ROWS; ++i) dk[i & 3] = fmaf(S[i], kreg[i], dk[i & 3]), dq[i & 3] = fmaf(S[i], qreg[i], dq[i & 3]);
        float sk = (dk[0] + dk[1]) + (dk[2] + dk[3]), sq = (dq[0] + dq[1]) + (dq[2] + dq[3]);
#pragma unroll
        for (int o = 1; o < LANES; o <<= 1) {
          sk += __shfl_xor_sync(0xffffffffu, sk, o);
          sq += __shfl_xor_sync(0xffffffffu, sq, o);
        }
        const float g = num.y;
        const float u = num.z * (v - g * sk);               // beta (v - (g S0)^T k)
#pragma unroll
        for (int i = 0; i < ROWS; ++i) S[i] = fmaf(kreg[i], u, g * S[i]);
        // o = (g S0 + k u^T)^T q = g (S0 . q) + (k . q) u
        if (writer) *dst = kept ? fmaf(g, sq, num.x * u) : 0.0f;
      }
    }
    __syncthreads();            // the next tile is there, and this one is done with
    if (fetchers <= 0 && more) {
      fetch(buf ^ 1, t0 + tile, min(tile, q_len - t0 - tile), threadIdx.x, blockDim.x);
      __syncthreads();
    }
  }
  if (mine != nullptr) {
#pragma unroll
    for (int i = 0; i < QUADS; ++i) {
      const int r0 = 4 * (i * LANES + part);
      if (quads_whole) {
        if (r0 < dim) *reinterpret_cast<float4 *>(mine + r0) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (r0 + e < dim) mine[r0 + e] = S[4 * i + e];
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(T *__restrict__ out, int64_t out_stride, const float *__restrict__ o, int64_t o_stride,
                      const T *__restrict__ gate, int64_t gate_stride, const float *__restrict__ weight, float eps,
                      int num_tokens, int heads, int vdim, int weight_per_head, int gate_kind, float out_scale) {
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
  if (weight_per_head) weight += h * vdim;
  if (gate_kind == 0 && out_scale == 1.0f) {
    for (int i = lane; i < vdim; i += 32) {
      const float z = le::to_f32(gr[i]);
      dst[i] = le::from_f32<T>(x[i] * inv * weight[i] * (z / (1.0f + expf(-z))));
    }
    return;
  }
  for (int i = lane; i < vdim; i += 32) {
    const float z = le::to_f32(gr[i]);
    const float g = gate_kind == 0 ? z / (1.0f + expf(-z)) : 1.0f / (1.0f + expf(-z));
    dst[i] = le::from_f32<T>(x[i] * inv * weight[i] * g * out_scale);
  }
}

}  // namespace

namespace {

// How a column of the state is shared out for heads of `dim` entries: `rows` entries a thread, `lanes` threads a
// column (a power of two, rows * lanes >= dim); false: dim is too large.  Heads of 128 to 256 entries may be held 8 or
// 16 rows a thread (LYAPUNOV_DELTA_ROWS=8|16; the default is the one measured faster).
bool scan_shape(int dim, int &rows, int &lanes) {
  static const int preferred = [] {
    const char *v = std::getenv("LYAPUNOV_DELTA_ROWS");
    return v != nullptr && std::atoi(v) == 8 ? 8 : 16;
  }();
  if (dim < 1 || dim > 1024) return false;
  rows = dim <= 256 ? (dim >= 128 ? preferred : 8) : (dim <= 512 ? 16 : 32);
  lanes = 1;
  while (lanes * rows < dim) lanes <<= 1;
  return true;
}

}  // namespace

// The lanes that share a column of the state for heads of `dim` entries (a power of two; 0: dim is too large).
LE_API int le_gated_delta_lanes(int dim) {
  int rows = 0, lanes = 0;
  return scan_shape(dim, rows, lanes) ? lanes : 0;
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
  int rows = 0, lanes = 0;
  if (!scan_shape(dim, rows, lanes)) return le::invalid("le_gated_delta_scan: heads of %d entries (at most 1024)", dim);
  if (dtype != LE_BF16 && dtype != LE_F32) return le::invalid("le_gated_delta_scan: unknown dtype code %d", dtype);
  const int cols = SCAN_HOLDERS / lanes;
  const int prep_stride = le_gated_delta_scratch(heads, kv_heads);
  const size_t elem = dtype == LE_BF16 ? 2 : 4;
  const int vec = static_cast<int>(16 / elem);
  const int wide = dim % vec == 0 && qkv_stride % vec == 0 && q_col % vec == 0 && k_col % vec == 0 &&
                   reinterpret_cast<uintptr_t>(qkv) % 16 == 0;
  const size_t per_token = sizeof(float) * (2 * static_cast<size_t>(lanes) * rows + cols + SCAN_NUMBERS);
  int tile = static_cast<int>((36 * 1024) / per_token);
  tile = tile < 1 ? 1 : (tile > SCAN_MAX_TILE ? SCAN_MAX_TILE : tile);
  const bool single = num_tokens == num_requests;      // a step of single tokens: one tile of one token, nobody fetches ahead
  if (single) tile = 1;
  const int threads = single ? SCAN_HOLDERS : SCAN_THREADS;
  const size_t smem = 2 * tile * per_token;
  const dim3 prep_grid(num_tokens, (kv_heads + PREP_THREADS / 32 - 1) / (PREP_THREADS / 32));
  const dim3 grid((vdim + cols - 1) / cols, heads, num_requests);
  if (grid.y > 65535 || grid.z > 65535 || prep_grid.y > 65535)
    return le::invalid("le_gated_delta_scan: too many heads or requests for one launch");
#define LE_GO(T, R, L)                                                                                                  \
  do {                                                                                                                  \
    int rc = le::launch_chained(gated_delta_prepare_kernel<T>, prep_grid, dim3(PREP_THREADS), 0, stream, scratch,       \
                                prep_stride, static_cast<const T *>(qkv), qkv_stride, q_col, k_col,                     \
                                static_cast<const T *>(proj), proj_stride, b_col, a_col, a_log, dt_bias, heads, kv_heads, \
                                dim, unit_eps, q_scale);                                                                \
    if (rc != 0) return rc;                                                                                             \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(gated_delta_scan_kernel<T, R, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    return le::launch_chained(gated_delta_scan_kernel<T, R, L>, grid, dim3(threads), smem, stream, out, out_stride,     \
                              static_cast<const T *>(qkv), qkv_stride, q_col, k_col, v_col,                             \
                              static_cast<const float *>(scratch), prep_stride, state, num_state_rows, state_slots, cu_q, \
                              heads, kv_heads, dim, vdim, tile, wide);                                                  \
  } while (0)
#define LE_SHAPE(T, R, L) \
  if (rows == R && lanes == L) LE_GO(T, R, L)
#define LE_SHAPES(T)                                                                                                    \
  LE_SHAPE(T, 8, 1); LE_SHAPE(T, 8, 2); LE_SHAPE(T, 8, 4); LE_SHAPE(T, 8, 8); LE_SHAPE(T, 8, 16); LE_SHAPE(T, 8, 32);   \
  LE_SHAPE(T, 16, 8); LE_SHAPE(T, 16, 16); LE_SHAPE(T, 16, 32); LE_SHAPE(T, 32, 32)
  if (dtype == LE_BF16) { LE_SHAPES(__nv_bfloat16); }
  else { LE_SHAPES(float); }
#undef LE_SHAPES
#undef LE_SHAPE
#undef LE_GO
  return le::invalid("le_gated_delta_scan: no kernel for %d rows a thread and %d threads a column", rows, lanes);
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * act(gate[t, h, :]) * out_scale; weight is
// [vdim], or [heads, vdim] with weight_per_head; act is silu (gate_kind 0) or the sigmoid (1).
LE_API int le_head_norm_gate(void *out, int64_t out_stride, const float *o, int64_t o_stride, const void *gate,
                             int64_t gate_stride, int dtype, const float *weight, float eps, int num_tokens, int heads,
                             int vdim, int weight_per_head, int gate_kind, float out_scale, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int64_t items = static_cast<int64_t>(num_tokens) * heads;
  const dim3 grid(static_cast<unsigned>((items + 3) / 4));
  LE_DISPATCH_DTYPE(dtype, T,
                    return le::launch_chained(head_norm_gate_kernel<T>, grid, dim3(128), 0, stream, static_cast<T *>(out),
                                              out_stride, o, o_stride, static_cast<const T *>(gate), gate_stride, weight,
                                              eps, num_tokens, heads, vdim, weight_per_head, gate_kind, out_scale));
}
